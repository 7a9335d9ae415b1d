"""Child process of the tensor-parallel tests: one rank of a 127.0.0.1 rendezvous.

    python tests/tp_worker.py cpu <rank> <world> <port> <out.npz>    oracle pieces + gloo all_gather (no GPU)
    python tests/tp_worker.py gpu <rank> <world> <port> <out.npz>    library TPDecoder on cuda:<rank>

Both decode the same seeded small model with the same prompt and write the token stream (and rank-local logits of
the last step) for the parent test to compare with the single-rank result.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

SMALL = dict(n_layers=2, hidden=512, n_heads=8, n_kv=4, hd=64, ffn=1024, vocab=4096)
PROMPT = [11, 4000, 7, 123, 2047]
N_NEW = 6
SEED = 4242


def oracle_tp_generate(model, rank, world, all_gather, prompt, n_new, max_ctx=64):
    """Greedy decode of one rank's shard through the oracle's kernel-level entry points, mirroring the order of
    orc_decode_step (oracle/oracle.c) with a gather after each sharded product."""
    from oracle import oracle as orc
    from __graft_entry__ import load_package
    import importlib
    tp = importlib.import_module(load_package().__name__ + ".tp")
    c = model["cfg"]
    loc = tp.shard_model(model, world, rank)
    H, hd, I = c["hidden"], c["head_dim"], c["ffn"]
    nh_l, nkv_l = c["n_heads"] // world, c["n_kv_heads"] // world
    QD, QD_l, KVD_l, I_l, H_l, V_l = c["n_heads"] * hd, nh_l * hd, nkv_l * hd, I // world, H // world, c["vocab"] // world
    L = c["n_layers"]
    kc = np.zeros((L, 2, max_ctx, nkv_l, hd), np.int8)
    ks = np.zeros((L, 2, max_ctx, nkv_l), np.float32)
    scale = np.float32(1.0 / np.sqrt(np.float32(hd)))

    def step(token, pos):
        x = orc.dequant_embedding_row(model["tok_embd"][0], model["tok_embd"][1], token, H)
        for l, w in enumerate(loc["layers"]):
            normed = orc.rmsnorm(x, None, w["rms_attn"], 1, H, c["eps"])
            q, k, v = orc.entry_gemv_multi([w["wq"][0], w["wk"][0], w["wv"][0]], [w["wq"][1], w["wk"][1], w["wv"][1]], [QD_l, KVD_l, KVD_l], normed, H)
            q = orc.rmsnorm(q, None, w["q_norm"], nh_l, hd, c["eps"])
            k = orc.rmsnorm(k, None, w["k_norm"], nkv_l, hd, c["eps"])
            q, k = orc.rope(q, k, nh_l, nkv_l, hd, pos, c["rope_theta"], True)
            kc[l, 0, pos], ks[l, 0, pos] = orc.fp16_to_int8(k, nkv_l, hd)
            kc[l, 1, pos], ks[l, 1, pos] = orc.fp16_to_int8(v, nkv_l, hd)
            att_l = orc.attention_decode(q, kc[l, 0, :pos + 1], kc[l, 1, :pos + 1], nh_l, nkv_l, hd, pos + 1, scale, True,
                                         ks[l, 0, :pos + 1], ks[l, 1, :pos + 1]).reshape(-1)
            att = all_gather(att_l)
            x2_l = orc.entry_gemv_quant_add(w["wo"][0], w["wo"][1], att, x[rank * H_l:(rank + 1) * H_l], H_l, QD)
            x2 = all_gather(x2_l)
            normed = orc.rmsnorm(x2, None, w["rms_ffn"], 1, H, c["eps"])
            g, u = orc.entry_gemv_multi([w["gate"][0], w["up"][0]], [w["gate"][1], w["up"][1]], [I_l, I_l], normed, H)
            sw = all_gather(orc.swiglu(g, u))
            x_l = orc.entry_gemv_quant_add(w["down"][0], w["down"][1], sw, x2[rank * H_l:(rank + 1) * H_l], H_l, I)
            x = all_gather(x_l)
        normed = orc.rmsnorm(x, None, model["out_norm"], 1, H, c["eps"])
        logits = orc.entry_gemv_quant_f32(loc["output"][0], loc["output"][1], normed, V_l, H)
        return all_gather(logits), logits

    tok, out, last = None, [], None
    for pos, t in enumerate(prompt):
        full, last = step(t, pos)
        tok = int(np.argmax(full))
    pos = len(prompt)
    for i in range(n_new):
        out.append(tok)
        if i + 1 < n_new:
            full, last = step(tok, pos)
            tok = int(np.argmax(full))
            pos += 1
    return np.array(out, np.int32), last


def main():
    mode, rank, world, port, out_path = sys.argv[1], int(sys.argv[2]), int(sys.argv[3]), int(sys.argv[4]), sys.argv[5]
    import torch
    import torch.distributed as dist
    from oracle import oracle as orc
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    model = orc.gen_model(SEED, **SMALL)
    if mode == "cpu":
        def all_gather(a):
            t = torch.from_numpy(np.ascontiguousarray(a).view(np.uint8).copy())
            parts = [torch.empty_like(t) for _ in range(world)]
            dist.all_gather(parts, t)
            return np.concatenate([p.numpy() for p in parts]).view(a.dtype)
        toks, logits = oracle_tp_generate(model, rank, world, all_gather, PROMPT, N_NEW)
        np.savez(out_path, tokens=toks, logits=logits)
    else:
        import importlib
        from __graft_entry__ import load_package
        pk = load_package()
        tp = importlib.import_module(pk.__name__ + ".tp")
        decmod = importlib.import_module(pk.__name__ + ".decoder")
        torch.cuda.set_device(rank)
        local = decmod.upload(tp.shard_model(model, world, rank))
        st = torch.cuda.Stream()
        res = {}
        for name, flags in (("graph", 3), ("nograph", 1), ("chain", 11)):
            d = tp.TPDecoder(model["cfg"], local, 64, rank, world, flags=flags)
            res[name] = d.generate(PROMPT, N_NEW, st)
            res[name + "2"] = d.generate(PROMPT, N_NEW, st)          # a second run through the same exchange regions
            res[name + "_kernels"] = np.int32(d.kernels_per_step())
            d.close()
        np.savez(out_path, status=np.int32(pk.device_status(st)), **res)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
