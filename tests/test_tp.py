"""Tensor-parallel decode.

CPU (gloo, world_size 2): the sharding plan and the gather points reproduce the single-rank oracle bit for bit.
GPU (needs 2 devices): the library's push-style exchange gives the single-GPU token stream on every rank."""
import os
import socket
import subprocess
import sys

import numpy as np
import pytest

from oracle import oracle as orc

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import tp_worker  # noqa: E402


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close()
    return p


def _run_ranks(mode, world, tmp_path, timeout):
    port = _free_port()
    outs = [str(tmp_path / f"{mode}_r{r}.npz") for r in range(world)]
    procs = [subprocess.Popen([sys.executable, os.path.join(HERE, "tp_worker.py"), mode, str(r), str(world), str(port), outs[r]],
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT) for r in range(world)]
    logs = []
    for p in procs:
        try:
            o, _ = p.communicate(timeout=timeout)
        except subprocess.TimeoutExpired:
            p.kill(); o, _ = p.communicate()
        logs.append(o.decode(errors="replace")[-3000:])
    assert all(p.returncode == 0 for p in procs), "\n---\n".join(logs)
    return [np.load(o) for o in outs]


def _single_rank_reference():
    model = orc.gen_model(tp_worker.SEED, **tp_worker.SMALL)
    d = orc.Decoder(model, 64)
    toks = d.generate(tp_worker.PROMPT, tp_worker.N_NEW)
    return model, np.array(toks, np.int32), d.logits.copy()


def test_row_ranges_cover_every_matrix_once():
    from __graft_entry__ import load_package
    import importlib
    tp = importlib.import_module(load_package().__name__ + ".tp")
    cfg = dict(n_layers=36, hidden=2560, n_heads=32, n_kv_heads=8, head_dim=128, ffn=9728, vocab=151936)
    for world in (2, 4, 8):
        seen = {}
        for r in range(world):
            for k, (a, b) in tp.row_ranges(cfg, world, r).items():
                seen.setdefault(k, []).append((a, b))
        for k, spans in seen.items():
            assert spans[0][0] == 0 and all(spans[i][1] == spans[i + 1][0] for i in range(world - 1)), (k, spans)
        assert seen["wq"][-1][1] == 4096 and seen["wk"][-1][1] == 1024 and seen["output"][-1][1] == 151936
        # a rank's query heads attend to its own KV heads only
        for r in range(world):
            q0, q1 = seen["wq"][r]; k0, k1 = seen["wk"][r]
            assert q0 // 128 // 4 == k0 // 128 and (q1 // 128 - 1) // 4 == k1 // 128 - 1
    with pytest.raises(ValueError):
        tp.row_ranges(dict(cfg, n_kv_heads=6), 4, 0)


def test_slices_are_views_of_contiguous_byte_ranges():
    from __graft_entry__ import load_package
    import importlib
    tp = importlib.import_module(load_package().__name__ + ".tp")
    rng = np.random.Generator(np.random.PCG64(5))
    W = orc.gen_weight(rng, 14, 12, 512)
    s = tp.slice_rows(W, 14, 512, 3, 9)
    assert s.base is not None and s.size == 6 * 2 * 210 and np.array_equal(s, W.reshape(-1)[3 * 420:9 * 420])


@pytest.mark.parametrize("world", [2, 4])
def test_gloo_ranks_match_single_rank_oracle(tmp_path, world):
    model, want_tokens, want_logits = _single_rank_reference()
    res = _run_ranks("cpu", world, tmp_path, 600)
    V_l = tp_worker.SMALL["vocab"] // world
    for r, z in enumerate(res):
        assert np.array_equal(z["tokens"], want_tokens), (r, z["tokens"], want_tokens)
        assert np.array_equal(z["logits"], want_logits[r * V_l:(r + 1) * V_l])


@pytest.mark.gpu
@pytest.mark.parametrize("world", [2, 4])
def test_gpu_ranks_match_single_gpu(tmp_path, world):
    import torch
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    from gpu_util import pkg
    import importlib
    jb = pkg()
    decmod = importlib.import_module(jb.__name__ + ".decoder")
    model = orc.gen_model(tp_worker.SEED, **tp_worker.SMALL)
    d = decmod.Decoder(model["cfg"], decmod.upload(model), 64)
    want = d.generate(tp_worker.PROMPT, tp_worker.N_NEW, torch.cuda.Stream())
    d.close()
    res = _run_ranks("gpu", world, tmp_path, 600)
    for r, z in enumerate(res):
        assert int(z["status"]) == 0
        for name in ("graph", "nograph", "chain"):
            assert np.array_equal(z[name], want), (r, name, z[name], want)
            assert np.array_equal(z[name + "2"], want), (r, name)
        # every exchange but the attention output rides in a GEMV epilogue; the chained variant also folds the four
        # GEMVs between two attentions into one launch
        assert int(z["chain_kernels"]) < int(z["graph_kernels"])


@pytest.mark.gpu
@pytest.mark.parametrize("n_layers", [1, 3])
def test_rank_that_never_arrives_is_reported_not_waited_for_forever(n_layers):
    """Failure detection without a fault: rank 0 of a two-rank group whose peer region is a buffer that nothing ever writes.
    The first wait for the peer's packets runs out after its bound (in polls and in time) and records
    JLLM_B200_ERR_TIMEOUT; every later wait of the step sees the recorded timeout and gives up at once, so the step
    ends after about one bound whatever the number of layers, and the context stays usable."""
    import ctypes as C
    import importlib
    import time
    import torch
    from gpu_util import pkg
    jb = pkg()
    decmod = importlib.import_module(jb.__name__ + ".decoder")
    tp = importlib.import_module(jb.__name__ + ".tp")
    small = dict(tp_worker.SMALL, n_layers=n_layers)
    model = orc.gen_model(7, **small)
    cfg = model["cfg"]
    local = decmod.upload(tp.shard_model(model, 2, 0))
    lib = jb.lib
    lib.jllm_b200_tp_alloc.restype = C.c_void_p
    lib.jllm_b200_tp_region_bytes.restype = C.c_size_t
    lib.jllm_b200_decoder_create_tp.restype = C.c_void_p
    nbytes = lib.jllm_b200_tp_region_bytes(cfg["hidden"], cfg["n_heads"] * cfg["head_dim"], cfg["ffn"])
    mine, silent = lib.jllm_b200_tp_alloc(C.c_size_t(nbytes)), lib.jllm_b200_tp_alloc(C.c_size_t(nbytes))
    assert mine and silent
    regions = (C.c_void_p * 2)(mine, silent)
    layers = (decmod.LayerDesc * n_layers)()
    names = dict(wq="wq", wk="wk", wv="wv", wo="wo", w_gate="gate", w_up="up", w_down="down")
    for i in range(n_layers):
        for f, k in names.items():
            setattr(layers[i], f, local["layers"][i][k][0].data_ptr())
            setattr(layers[i], "type_" + f, local["layers"][i][k][1])
        for k in ("rms_attn", "rms_ffn", "q_norm", "k_norm"):
            setattr(layers[i], k, local["layers"][i][k].data_ptr())
    m = decmod.ModelDesc()
    m.n_layers, m.hidden_dim, m.n_heads, m.n_kv_heads = n_layers, cfg["hidden"], cfg["n_heads"], cfg["n_kv_heads"]
    m.head_dim, m.intermediate_dim, m.vocab_size, m.max_context = cfg["head_dim"], cfg["ffn"], cfg["vocab"], 16
    m.rope_theta, m.rms_eps, m.rope_neox = cfg["rope_theta"], cfg["eps"], 1
    m.tok_embd, m.embd_type = local["tok_embd"][0].data_ptr(), local["tok_embd"][1]
    m.output, m.output_type = local["output"][0].data_ptr(), local["output"][1]
    m.output_norm = local["out_norm"].data_ptr()
    m.layers = layers
    h = lib.jllm_b200_decoder_create_tp(C.byref(m), C.c_int(1), C.c_int(0), C.c_int(2), regions)
    assert h, jb.last_error()
    st = torch.cuda.Stream()
    t0 = time.time()
    rc = lib.jllm_b200_decoder_step(C.c_void_p(h), 5, 0, C.c_void_p(st.cuda_stream))
    assert rc == 0                                       # the step was enqueued; the failure shows on the device
    status = jb.device_status(st)
    took = time.time() - t0
    assert status == 7, status                           # JLLM_B200_ERR_TIMEOUT
    assert took < 10, took                               # one bound (half a second), not one per wait, kernel or layer
    assert jb.device_status(st) == 0                     # reading the status clears it
    # the context is still usable: an ordinary GEMV gives the oracle's result
    rng = np.random.Generator(np.random.PCG64(3))
    W = orc.gen_weight(rng, 12, 64, 512); x = orc.gen_act(rng, 512)
    y = torch.zeros(64, dtype=torch.float16, device="cuda")
    from gpu_util import dev, close
    jb.gemv_quant(y, dev(W), 12, dev(x), 64, 512)
    ok, md = close(y.float().cpu().numpy(), orc.entry_gemv_quant(W, 12, x, 64, 512).astype(np.float32))
    assert ok, md
    lib.jllm_b200_decoder_destroy(C.c_void_p(h))
    lib.jllm_b200_tp_free(C.c_void_p(mine)); lib.jllm_b200_tp_free(C.c_void_p(silent))
