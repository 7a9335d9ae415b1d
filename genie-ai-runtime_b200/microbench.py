"""Kernel-level micro-benchmarks of the hot path (configurations 0-3 of the baseline), timed with CUDA events.

    python genie-ai-runtime_b200/microbench.py gemv  --type 12 --M 9728 --K 2560            # config 0
    python genie-ai-runtime_b200/microbench.py gemv  --type 14 --M 2560 --K 9728            # config 1
    python genie-ai-runtime_b200/microbench.py pair  --M 9728 --K 2560 [--swiglu]           # gate/up
    python genie-ai-runtime_b200/microbench.py add   --type 14 --M 2560 --K 9728            # W_down + residual
    python genie-ai-runtime_b200/microbench.py f32   --type 14 --M 151936 --K 2560          # logits
    python genie-ai-runtime_b200/microbench.py attn  --L 8192 [--batch 64]                  # config 2
    python genie-ai-runtime_b200/microbench.py mmq   --type 12 --M 9728 --K 2560 --N 512    # config 3
    python genie-ai-runtime_b200/microbench.py layer [--trace]                              # the four GEMVs of a decoder layer, chained

Weights are random block images; `--copies` distinct copies (default: enough for 3x the 126 MB L2) are used in
rotation so that every launch streams from HBM.  Prints one JSON line with the average launch time and the
algorithmic GB/s (bytes every launch must move at least once: weights + activations in + results out).
"""
import argparse
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
L2_BYTES = 126 << 20


def blocks(ggml_type, rows, K, dev, gen):
    import torch
    bb = 144 if ggml_type == 12 else 210
    B = rows * (K // 256)
    img = torch.randint(0, 256, (B, bb), dtype=torch.uint8, device=dev, generator=gen)
    d = (torch.randn(B, device=dev, generator=gen).abs() * 0.01).to(torch.float16).view(torch.uint8).reshape(B, 2)
    if ggml_type == 12:
        img[:, 0:2] = d
        img[:, 2:4] = (torch.randn(B, device=dev, generator=gen).abs() * 0.01).to(torch.float16).view(torch.uint8).reshape(B, 2)
    else:
        img[:, 208:210] = d
    return img.reshape(rows, -1).contiguous()


def parser():
    ap = argparse.ArgumentParser()
    ap.add_argument("kind", choices=["gemv", "pair", "triple", "add", "f32", "attn", "pattn", "mmq", "layer"])
    ap.add_argument("--type", type=int, default=12)
    ap.add_argument("--M", type=int, default=9728)
    ap.add_argument("--K", type=int, default=2560)
    ap.add_argument("--N", type=int, default=512)
    ap.add_argument("--L", type=int, default=8192)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--nh", type=int, default=32, help="attn: query heads")
    ap.add_argument("--nkv", type=int, default=8, help="attn: KV heads")
    ap.add_argument("--copies", type=int, default=0)
    ap.add_argument("--iters", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--swiglu", action="store_true", help="pair: SwiGLU applied in the epilogue")
    ap.add_argument("--norm", action="store_true", help="pair/triple: RMSNorm fused in front of the activation quantiser")
    ap.add_argument("--no-pdl", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="launch from Python every iteration instead of replaying a CUDA graph")
    ap.add_argument("--interleave", type=int, default=0, help="layer: this many launches of a tiny unrelated kernel between the GEMVs "
                    "(how much a change of kernel costs the next GEMV)")
    ap.add_argument("--trace", action="store_true", help="GEMV kinds: record per-CTA time stamps of every launch (diagnostic kernel "
                    "instantiation) and print where the time of a launch goes")
    return ap


def measure(jb, argv):
    """One measurement; `argv` as on the command line (e.g. ["gemv", "--type", "12"]).  Returns the result record."""
    import torch
    a = parser().parse_args([str(v) for v in argv])
    dev = torch.device("cuda", torch.cuda.current_device())
    gen = torch.Generator(device=dev)
    gen.manual_seed(1000)
    if a.no_pdl:
        jb.lib.jllm_b200_set_pdl(0)
    st = torch.cuda.Stream()
    bb = lambda t: 144 if t == 12 else 210
    M, K, t = a.M, a.K, a.type
    calls, nbytes = [], 0
    if a.kind in ("gemv", "add", "f32", "pair", "triple", "mmq"):
        nmat = {"pair": 2, "triple": 3}.get(a.kind, 1)
        Ms = [M] * nmat if a.kind != "triple" else [4096, 1024, 1024]
        ts = [t] * nmat if a.kind != "triple" else [12, 12, 14]
        wbytes = sum(m * (K // 256) * bb(tt) for m, tt in zip(Ms, ts))
        copies = a.copies or max(2, int(np.ceil(3 * L2_BYTES / wbytes)))
        Ws = [[blocks(tt, m, K, dev, gen) for m, tt in zip(Ms, ts)] for _ in range(copies)]
        N = a.N if a.kind == "mmq" else 1
        x = torch.randn(N * K, device=dev, generator=gen).to(torch.float16)
        res = torch.randn(M, device=dev, generator=gen).to(torch.float16)
        ys = [torch.zeros(N * m, dtype=torch.float32 if a.kind == "f32" else torch.float16, device=dev) for m in Ms]
        nw = torch.ones(K, dtype=torch.float32, device=dev)
        for W in Ws:
            if a.kind == "gemv":
                calls.append(lambda W=W: jb.gemv_quant(ys[0], W[0], t, x, M, K, st))
            elif a.kind == "add":
                calls.append(lambda W=W: jb.gemv_quant_add(ys[0], W[0], t, x, res, M, K, st))
            elif a.kind == "f32":
                calls.append(lambda W=W: jb.gemv_quant_f32(ys[0], W[0], t, x, M, K, st))
            elif a.kind == "pair" and a.swiglu:
                calls.append(lambda W=W: jb.norm_gemv_pair_swiglu(ys[0], W[0], W[1], t, M, x, nw if a.norm else None, True, 1e-6, K, st))
            elif a.kind == "pair" and a.norm:
                calls.append(lambda W=W: jb.norm_gemv_quant_pair(ys[0], W[0], t, M, ys[1], W[1], t, M, x, nw, True, 1e-6, K, st))
            elif a.kind == "triple" and a.norm:
                calls.append(lambda W=W: jb.norm_gemv_quant_triple(ys[0], W[0], 12, Ms[0], ys[1], W[1], 12, Ms[1], ys[2], W[2], 14, Ms[2], x, nw, True, 1e-6, K, st))
            elif a.kind == "pair":
                calls.append(lambda W=W: jb.gemv_quant_pair(ys[0], W[0], t, M, ys[1], W[1], t, M, x, K, st))
            elif a.kind == "triple":
                calls.append(lambda W=W: jb.gemv_quant_triple(ys[0], W[0], 12, Ms[0], ys[1], W[1], 12, Ms[1], ys[2], W[2], 14, Ms[2], x, K, st))
            else:
                calls.append(lambda W=W: jb.gemm_quant_batched(ys[0], W[0], t, x, M, a.N, K, st))
        nbytes = wbytes + N * K * 2 + sum(N * m * ys[0].element_size() for m in Ms)
        shape = dict(M=Ms, K=K, types=ts, N=N, copies=copies)
    elif a.kind == "layer":
        # The four weight products of one decoder layer of the 4B shape, each reading what the one before wrote (Q/K/V with the
        # RMSNorm in front -> Wo + residual -> gate/up with RMSNorm and SwiGLU -> W_down + residual), without the attention
        # between them: how the GEMV launches behave next to one another, which a single kernel repeated does not show.
        H, QD, KVD, FF = 2560, 4096, 1024, 9728
        per = (QD + 2 * KVD) * 10 * 144 + KVD * 10 * (210 - 144) + H * 16 * 144 + 2 * FF * 10 * 144 + H * 38 * 210
        copies = a.copies or max(2, int(np.ceil(3 * L2_BYTES / per)))
        h = torch.randn(H, device=dev, generator=gen).to(torch.float16)
        h2 = torch.zeros(H, dtype=torch.float16, device=dev)
        q = torch.zeros(QD, dtype=torch.float16, device=dev); kk = torch.zeros(KVD, dtype=torch.float16, device=dev); vv = torch.zeros(KVD, dtype=torch.float16, device=dev)
        act = torch.zeros(FF, dtype=torch.float16, device=dev)
        nw = torch.ones(H, dtype=torch.float32, device=dev)
        layer_launches = []
        for _ in range(copies):
            Wq, Wk, Wv = blocks(12, QD, H, dev, gen), blocks(12, KVD, H, dev, gen), blocks(14, KVD, H, dev, gen)
            Wo, Wg, Wu, Wd = blocks(12, H, QD, dev, gen), blocks(12, FF, H, dev, gen), blocks(12, FF, H, dev, gen), blocks(14, H, FF, dev, gen)
            layer_launches.append([
                lambda Wq=Wq, Wk=Wk, Wv=Wv: jb.norm_gemv_quant_triple(q, Wq, 12, QD, kk, Wk, 12, KVD, vv, Wv, 14, KVD, h, nw, True, 1e-6, H, st),
                lambda Wo=Wo: jb.gemv_quant_add(h2, Wo, 12, q, h, H, QD, st),
                lambda Wg=Wg, Wu=Wu: jb.norm_gemv_pair_swiglu(act, Wg, Wu, 12, FF, h2, nw, True, 1e-6, H, st),
                lambda Wd=Wd: jb.gemv_quant_add(h, Wd, 14, act, h2, H, FF, st)])
        tiny_buf = torch.ones(256, dtype=torch.float16, device=dev)
        tiny = lambda: [jb.vec_scale(tiny_buf, 256, 1.0, st) for _ in range(a.interleave)]
        for L in layer_launches:
            calls.append(lambda L=L: [(f(), tiny()) for f in L])
        nbytes = per
        shape = dict(layer="qkv(norm) -> wo+res -> gate/up(norm, swiglu) -> down+res", copies=copies)
    elif a.kind == "pattn":
        # causal prefill attention of N query tokens from position 0 over an INT8 cache (the cache fits the L2: a prompt's K/V
        # were written just before); algorithmic bytes = K/V/scales of the N positions once + q in + out
        nh, nkv, hd, N = 32, 8, 128, a.N
        scale = float(1 / np.sqrt(hd))
        k = torch.randint(-127, 128, (N, nkv, hd), dtype=torch.int8, device=dev, generator=gen)
        v = torch.randint(-127, 128, (N, nkv, hd), dtype=torch.int8, device=dev, generator=gen)
        ksc = (torch.randn((N, nkv), device=dev, generator=gen).abs() * 0.02).to(torch.float16).float()
        vsc = (torch.randn((N, nkv), device=dev, generator=gen).abs() * 0.02).to(torch.float16).float()
        q = torch.randn(N * nh * hd, device=dev, generator=gen).to(torch.float16)
        out = torch.zeros(N * nh * hd, dtype=torch.float16, device=dev)
        calls.append(lambda: jb.flash_attention_prefill_batched(out, q, k, v, nh, nkv, hd, hd, N, 0, scale, True, ksc, vsc, 0, st))
        nbytes = 2112 * N + 2 * N * nh * hd * 2
        shape = dict(N=N, flops=4.0 * nh * hd * N * (N + 1) / 2)
    else:
        nh, nkv, hd, L, B = a.nh, a.nkv, 128, a.L, a.batch
        lens = [L] if B == 1 else [int(v) for v in np.random.Generator(np.random.PCG64(1002)).integers(256, 8193, B)]
        per = sum((2 * nkv * hd + 8 * nkv) * l + 4 * nh * hd for l in lens)      # K + V + scales of every position once, q in, out
        copies = a.copies or max(2, int(np.ceil(3 * L2_BYTES / per)))
        if B > 1:
            copies = min(copies, 2)          # 64 caches of 8192 positions are 1 GB per copy
        scale = float(1 / np.sqrt(hd))
        Lmax = max(lens)
        keep = []
        for _ in range(copies):
            # every cache holds Lmax positions (a plan's tensor maps cover whole caches); a sequence uses its first L
            ks = [torch.randint(-127, 128, (Lmax if B > 1 else l, nkv, hd), dtype=torch.int8, device=dev, generator=gen) for l in lens]
            vs = [torch.randint(-127, 128, (Lmax if B > 1 else l, nkv, hd), dtype=torch.int8, device=dev, generator=gen) for l in lens]
            kss = [(torch.randn((Lmax if B > 1 else l, nkv), device=dev, generator=gen).abs() * 0.02).to(torch.float16).float() for l in lens]
            vss = [(torch.randn((Lmax if B > 1 else l, nkv), device=dev, generator=gen).abs() * 0.02).to(torch.float16).float() for l in lens]
            q = torch.randn(B * nh * hd, device=dev, generator=gen).to(torch.float16)
            out = torch.zeros(B * nh * hd, dtype=torch.float16, device=dev)
            if B == 1:
                calls.append(lambda q=q, out=out, k=ks[0], v=vs[0], s1=kss[0], s2=vss[0]:
                             jb.flash_attention_decode(out, q, k, v, nh, nkv, hd, hd, L, scale, True, s1, s2, 0, st))
            else:
                plan = jb.AttnPlan(ks, vs, kss, vss, Lmax, nkv)
                lens_d = torch.tensor(lens, dtype=torch.int32, device=dev)
                keep.append((plan, ks, vs, kss, vss))
                calls.append(lambda q=q, out=out, plan=plan, lens_d=lens_d: plan.decode(out, q, lens_d, nh, scale, st))
        nbytes = per
        shape = dict(L=L, batch=B, copies=copies)
    trace = None
    if a.trace:
        import ctypes as C
        jb.lib.jllm_b200_init(C.c_int(-1))                     # the per-device context must exist before the capture starts
        calls[0]()
        torch.cuda.synchronize()
        NCTA, NST = 2 * 148, 16
        per_call = 4 if a.kind == "layer" else 1
        trace = torch.zeros((a.iters * per_call, NCTA, NST), dtype=torch.int64, device=dev)
        plain = calls
        def traced(i):
            if a.kind == "layer":
                for k, f in enumerate(layer_launches[i % len(layer_launches)]):
                    jb.lib.jllm_b200_debug_gemv_trace(C.c_void_p(trace[4 * i + k].data_ptr()))
                    f()
                return
            jb.lib.jllm_b200_debug_gemv_trace(C.c_void_p(trace[i].data_ptr()))
            plain[i % len(plain)]()
        calls = [lambda i=i: traced(i) for i in range(a.iters)]
    with torch.cuda.stream(st):
        for i in range(max(a.warmup, len(calls)) if not a.trace else 0):
            calls[i % len(calls)]()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        if a.no_graph:
            e0.record(st)
            for i in range(a.iters):
                calls[i % len(calls)]()
            e1.record(st)
        else:
            # one graph holding `iters` launches over the rotating copies: the host's per-call cost (several
            # microseconds through ctypes) stays out of the measurement
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=st):
                for i in range(a.iters):
                    calls[i % len(calls)]()
            g.replay()
            torch.cuda.synchronize()
            e0.record(st)
            g.replay()
            e1.record(st)
        torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / a.iters
    if a.trace:
        t = trace.cpu().numpy().astype(np.int64)              # [launch][cta][stamp], ns
        names = ["entry_first", "entry_last", "copies_issued_last", "producer_done_first", "producer_done_last", "staged_last",
                 "first_rows_landed_first", "first_rows_landed_last", "warp0_done_last", "all_done",
                 "t0_landed", "t0_done", "t1_landed", "t1_done", "x_loaded", "norm_known", "quantised", "barriers_ready",
                 "range_known", "entry_median"]
        rows = []
        per_call = 4 if a.kind == "layer" else 1
        by_kind = [[] for _ in range(per_call)]
        for i in range(2 * per_call, a.iters * per_call):
            live = t[i][:, 0] > 0
            cur, prev = t[i][live], t[i - 1][t[i - 1][:, 0] > 0]
            base = prev[:, 6].max()                             # the previous launch's last warp finishes
            rows.append([cur[:, 0].min() - base, cur[:, 0].max() - base, cur[:, 1].max() - base, cur[:, 2].min() - base, cur[:, 2].max() - base,
                         cur[:, 3].max() - base, cur[:, 4].min() - base, cur[:, 4].max() - base, cur[:, 5].max() - base, cur[:, 6].max() - base])
            for k in list(range(8, 16)) + [7]:                  # warp 0's tasks and staging phases: median over CTAs
                ok = cur[:, k] > 0
                rows[-1].append(np.median(cur[ok, k]) - base if ok.any() else 0)
            rows[-1].append(np.median(cur[:, 0]) - base)       # median CTA entry
            by_kind[i % per_call].append(rows[-1])
        for k, rk in enumerate(by_kind):
            r = np.median(np.array(rk, np.float64), axis=0) / 1e3
            print(json.dumps({"launch": ["qkv", "wo", "gate_up", "down"][k] if per_call == 4 else a.kind,
                              "trace_us_after_previous_launch_finished(median)": {n: round(float(v), 2) for n, v in zip(names, r)},
                              "ctas": int((t[2 * per_call + k][:, 0] > 0).sum())}))
    extra = {"TFLOPs": 2.0 * a.M * a.N * a.K / us / 1e6} if a.kind == "mmq" else ({"TFLOPs": shape["flops"] / us / 1e6} if a.kind == "pattn" else {})
    if a.no_pdl:
        jb.lib.jllm_b200_set_pdl(1)
    return {"kind": a.kind, "shape": shape, "us_per_launch": us, "algorithmic_bytes": nbytes, **extra,
            "GBps": nbytes / us / 1e3, "pdl": not a.no_pdl, "graph": not a.no_graph, "device_status": jb.device_status(st)}


def main():
    import torch
    from __graft_entry__ import load_package
    jb = load_package()
    torch.cuda.set_device(0)
    print(json.dumps(measure(jb, sys.argv[1:])))


if __name__ == "__main__":
    main()
