"""Lock-step batch decoder (jllm_b200_batch_decoder_*) against the oracle's batched arithmetic: every stream must follow the
stream the oracle decodes for it through the reference's batched (prefill-arithmetic) GEMM."""
import numpy as np
import pytest

from oracle import oracle as orc
from gpu_util import pkg

pytestmark = pytest.mark.gpu

SMALL = dict(n_layers=2, hidden=512, n_heads=4, n_kv=2, hd=128, ffn=1024, vocab=2048)
# Bounds, in units of the logit RMS.  The activation quantiser between the layers amplifies any one-ULP difference (a changed
# group maximum re-rounds 32 codes), so even the CUDA-core GEMM, whose products match the oracle to 1e-5, ends at an error
# RMS of 0.024 and a maximum of 0.15 on this model; the tensor-core GEMM (operand products rounded to fp16, 3.6e-4 per
# product) ends at 0.05 and 0.43.
ERR_RMS, ERR_MAX = 0.08, 0.6


def oracle_batch(model, prompts, n_new, ctx):
    c = model["cfg"]
    B, P = prompts.shape
    H, hd, I, V = c["hidden"], c["head_dim"], c["ffn"], c["vocab"]
    nh, nkv = c["n_heads"], c["n_kv_heads"]
    QD, KVD, L = nh * hd, nkv * hd, c["n_layers"]
    kc = np.zeros((B, L, 2, ctx, nkv, hd), np.int8)
    ks = np.zeros((B, L, 2, ctx, nkv), np.float32)
    scale = np.float32(1.0 / np.sqrt(np.float32(hd)))
    add = lambda a, b: (a.astype(np.float32) + b.astype(np.float32)).astype(np.float16)
    gemm = lambda Wt, X, M, K: np.asarray(orc.entry_gemm_quant_batched(Wt[0], Wt[1], X.reshape(-1), M, B, K)).reshape(B, M)

    def step(tokens, pos):
        X = np.stack([orc.dequant_embedding_row(model["tok_embd"][0], model["tok_embd"][1], int(t), H) for t in tokens])
        for l, w in enumerate(model["layers"]):
            normed = orc.rmsnorm(X.reshape(-1), None, w["rms_attn"], B, H, c["eps"])
            q, k, v = gemm(w["wq"], normed, QD, H), gemm(w["wk"], normed, KVD, H), gemm(w["wv"], normed, KVD, H)
            att = np.zeros((B, QD), np.float16)
            for b in range(B):
                qb = orc.rmsnorm(q[b], None, w["q_norm"], nh, hd, c["eps"])
                kb = orc.rmsnorm(k[b], None, w["k_norm"], nkv, hd, c["eps"])
                qb, kb = orc.rope(qb, kb, nh, nkv, hd, pos, c["rope_theta"], True)
                kc[b, l, 0, pos], ks[b, l, 0, pos] = orc.fp16_to_int8(kb, nkv, hd)
                kc[b, l, 1, pos], ks[b, l, 1, pos] = orc.fp16_to_int8(v[b], nkv, hd)
                att[b] = orc.attention_decode(qb, kc[b, l, 0, :pos + 1], kc[b, l, 1, :pos + 1], nh, nkv, hd, pos + 1, scale, True,
                                              ks[b, l, 0, :pos + 1], ks[b, l, 1, :pos + 1]).reshape(-1)
            x2 = add(X, gemm(w["wo"], att, H, QD))
            normed = orc.rmsnorm(x2.reshape(-1), None, w["rms_ffn"], B, H, c["eps"])
            g, u = gemm(w["gate"], normed, I, H), gemm(w["up"], normed, I, H)
            sw = orc.swiglu(g.reshape(-1), u.reshape(-1)).reshape(B, I)
            X = add(x2, gemm(w["down"], sw, H, I))
        normed = orc.rmsnorm(X.reshape(-1), None, model["out_norm"], B, H, c["eps"])
        return gemm(model["output"], normed, V, H).astype(np.float32)

    out, logits, toks, all_logits = [], None, None, []
    for pos in range(P + n_new - 1):
        cur = prompts[:, pos] if pos < P else toks
        logits = step(cur, pos)
        toks = np.argmax(logits, axis=1).astype(np.int32)
        if pos >= P - 1:
            out.append(toks.copy())
            all_logits.append(logits.copy())
    return np.stack(out), logits, all_logits


def test_batch_streams_follow_the_oracle():
    import torch
    jb = pkg()
    m = orc.gen_model(77, **SMALL)
    w = jb.decoder.upload(m)
    rng = np.random.Generator(np.random.PCG64(1010))
    B, P, n_new, ctx = 3, 4, 4, 32
    prompts = rng.integers(0, SMALL["vocab"], (B, P)).astype(np.int32)
    want, want_logits, step_logits = oracle_batch(m, prompts, n_new, ctx)
    d = jb.decoder.BatchDecoder(m["cfg"], w, ctx, B)
    st = torch.cuda.Stream()
    got = d.generate(prompts, n_new, st)
    got2 = d.generate(prompts, n_new, st)
    assert jb.device_status(st) == 0
    assert np.array_equal(got, got2)                       # a session can be reused
    lg = d.logits().float().cpu().numpy()
    rms = float(np.sqrt(np.mean(want_logits.astype(np.float64) ** 2)))
    same = np.array_equal(got, want)
    if same:                                               # identical streams: the last step's logits are comparable row by row
        err = np.abs(lg - want_logits)
        print("logit error: max %.4f, rms %.4f, logit rms %.4f" % (float(err.max()), float(np.sqrt(np.mean(err ** 2))), rms))
        assert float(np.sqrt(np.mean(err ** 2))) <= ERR_RMS * rms and float(err.max()) <= ERR_MAX * rms
    else:                                                  # a stream may part from the oracle only at a near tie of its two top logits
        # up to the first parting step every stream fed both decoders the same tokens, so the oracle's logits of that step are
        # the ones to judge the margin by: the oracle's own choice must lead the GPU's by no more than the logit error bound
        s0 = int(np.argwhere(got != want)[0][0])
        for b in np.argwhere(got[s0] != want[s0]).reshape(-1):
            lg0 = step_logits[s0][b]
            margin = float(lg0[want[s0][b]] - lg0[got[s0][b]])
            print("stream %d parts at step %d: oracle margin %.4f (logit RMS %.3f)" % (b, s0, margin, rms))
            assert 0 <= margin <= ERR_MAX * rms, (int(b), s0, margin, rms)
    d.close()


def test_batch_decoder_argument_errors():
    jb = pkg()
    m = orc.gen_model(78, **SMALL)
    w = jb.decoder.upload(m)
    with pytest.raises(jb.JllmError):
        jb.decoder.BatchDecoder(m["cfg"], w, 32, 1)        # a batch of one is the single-stream decoder's job
    d = jb.decoder.BatchDecoder(m["cfg"], w, 16, 2)
    with pytest.raises(jb.JllmError):
        d.generate(np.zeros((2, 10), np.int32), 10)        # 20 tokens do not fit a context of 16
    with pytest.raises(jb.JllmError):
        d.generate(np.full((2, 3), 5000, np.int32), 2)     # token outside the vocabulary
    d.close()


def test_batch_decoder_step_device_is_bounded_by_the_context():
    """step_device keeps a host mirror of the device-side position: before generate it is an error (code 8), and a step that
    would write K/V rows past the per-stream pools returns code 6 without launching anything."""
    import torch
    jb = pkg()
    m = orc.gen_model(79, **SMALL)
    w = jb.decoder.upload(m)
    d = jb.decoder.BatchDecoder(m["cfg"], w, 8, 2)
    st = torch.cuda.Stream()
    with pytest.raises(jb.JllmError) as e:
        d.step_device(st)
    assert e.value.code == 8
    d.generate(np.zeros((2, 3), np.int32), 2, st)          # positions 0..3 used: the session stands at position 4
    for _ in range(4):
        d.step_device(st)                                   # positions 4..7
    n0 = jb.launch_count()
    with pytest.raises(jb.JllmError) as e:
        d.step_device(st)                                   # position 8 does not exist
    assert e.value.code == 6 and jb.launch_count() == n0
    assert jb.device_status(st) == 0
    d.close()
