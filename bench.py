#!/usr/bin/env python
"""Benchmark of the quantized decode hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (configuration 4 of the baseline): a Qwen3-4B-shaped decoder — 36 layers, hidden 2560, 32 query /
8 KV heads of 128, SwiGLU FFN 9728, vocabulary 151936, RoPE theta 1e6 — with random-init GGUF K-quant
weights (Q4_K everywhere, Q6_K for attn_v, ffn_down and output), INT8 KV cache, batch 1.  A 33-token
random-id prompt is decoded first (untimed), then W warm-up steps, then K timed greedy decode steps; one
step = one token through all 36 layers, the logits GEMV and the device-side argmax.

One JSON line is printed (rank 0).  `value` times the steps on the device with every input resident
(CUDA-graph replay, no host synchronisation inside the timed region); `e2e` times the user-facing per-token
call, which copies {position, token} host->device and the sampled token device->host and waits for it.
`roofline` times the dominant kernel (fused norm + gate/up GEMV + SwiGLU, 28 MB of Q4_K weights per launch)
over the 36 layers' distinct weights with CUDA events on its own stream.  `cpu_baseline` runs the CPU oracle
(oracle/, the reference's golden arithmetic restated in C with OpenMP) on a bounded sample of the same steps.

N > 1 (torchrun): the same single request is decoded tensor-parallel — weight rows and KV heads sharded over the N
GPUs, slices gathered after each sharded product by the library's own NVLink push kernels — so `value` is the
tok/s of that one stream (strong scaling).  --parallelism replicas runs N independent copies of the 1-GPU
engine instead (weak scaling, no data-path collective).  Times are reduced with MAX over ranks.

--impl reference: times the CPU oracle port of the reference's arithmetic on the host cores (the reference has
no CPU implementation of INT8-KV attention, src/kernels/attention.cu:1078-1082, and its CPU GEMV golden is
single-threaded and reachable only behind a CUDA copy), same metric and configuration.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CFG = dict(n_layers=36, hidden=2560, n_heads=32, n_kv_heads=8, head_dim=128, ffn=9728, vocab=151936, rope_theta=1e6, eps=1e-6)
N_PROMPT, MAX_CTX, SEED = 33, 512, 1004
Q4_K, Q6_K = 12, 14
W_RMS = {Q4_K: 327.0, Q6_K: 683.0}      # RMS of a dequantised weight per unit sigma (see oracle.model_sigma)


# ── synthetic weights, drawn on the GPU ────────────────────────────────────
def gen_blocks_gpu(gen, ggml_type, rows, K, dev):
    """Random GGUF block image [rows, K/256*bytes] (uint8) with the whole-model value distributions: every quant and
    packed 6-bit scale/min uniform, Q6_K int8 scales U{-64..63}, d = |N(0,1)| * sigma with sigma chosen for unit-RMS
    outputs, Q4_K dmin = 7.5 * |N(0,1)| * sigma (zero-mean weights)."""
    import torch
    B = rows * (K // 256)
    bb = 144 if ggml_type == Q4_K else 210
    sigma = 1.0 / (W_RMS[ggml_type] * np.sqrt(K))
    img = torch.randint(0, 256, (B, bb), dtype=torch.uint8, device=dev, generator=gen)
    d = (torch.randn(B, device=dev, generator=gen).abs() * sigma).to(torch.float16)
    if ggml_type == Q4_K:
        dm = (torch.randn(B, device=dev, generator=gen).abs() * sigma * 7.5).to(torch.float16)
        img[:, 0:2] = d.view(torch.uint8).reshape(B, 2)
        img[:, 2:4] = dm.view(torch.uint8).reshape(B, 2)
    else:
        sc = (img[:, 192:208].to(torch.int16) % 128 - 64).to(torch.int8)
        img[:, 192:208] = sc.view(torch.uint8)
        img[:, 208:210] = d.view(torch.uint8).reshape(B, 2)
    return img.reshape(rows, -1).contiguous()


def gen_model_gpu(dev, cfg=CFG, seed=SEED, shard=None):
    """Whole model, or with shard=(rank, world) the row slices of one tensor-parallel rank: sharded matrices hold
    rows/world rows drawn from a per-rank generator, replicated tensors (embedding, norms) come from the shared one."""
    import torch
    g = torch.Generator(device=dev)
    g.manual_seed(seed)
    gl, div = g, 1
    if shard is not None:
        gl = torch.Generator(device=dev)
        gl.manual_seed(seed * 1000 + shard[0])
        div = shard[1]
    H, QD, KVD, I, V = cfg["hidden"], cfg["n_heads"] * cfg["head_dim"], cfg["n_kv_heads"] * cfg["head_dim"], cfg["ffn"], cfg["vocab"]
    nrm = lambda n: (1.0 + 0.02 * torch.randn(n, device=dev, generator=g)).float()
    w = dict(layers=[])
    for _ in range(cfg["n_layers"]):
        w["layers"].append(dict(
            wq=(gen_blocks_gpu(gl, Q4_K, QD // div, H, dev), Q4_K), wk=(gen_blocks_gpu(gl, Q4_K, KVD // div, H, dev), Q4_K),
            wv=(gen_blocks_gpu(gl, Q6_K, KVD // div, H, dev), Q6_K), wo=(gen_blocks_gpu(gl, Q4_K, H // div, QD, dev), Q4_K),
            gate=(gen_blocks_gpu(gl, Q4_K, I // div, H, dev), Q4_K), up=(gen_blocks_gpu(gl, Q4_K, I // div, H, dev), Q4_K),
            down=(gen_blocks_gpu(gl, Q6_K, H // div, I, dev), Q6_K),
            rms_attn=nrm(H), rms_ffn=nrm(H), q_norm=nrm(cfg["head_dim"]), k_norm=nrm(cfg["head_dim"])))
    w["tok_embd"] = (gen_blocks_gpu(g, Q4_K, V, H, dev), Q4_K)
    w["output"] = (gen_blocks_gpu(gl, Q6_K, V // div, H, dev), Q6_K)
    w["out_norm"] = nrm(H)
    return w


def model_to_host(w):
    """torch CUDA weights -> the numpy structure the CPU oracle takes."""
    h = lambda t: t.cpu().numpy()
    m = dict(cfg=dict(CFG), layers=[], tok_embd=(h(w["tok_embd"][0]), w["tok_embd"][1]), output=(h(w["output"][0]), w["output"][1]),
             out_norm=h(w["out_norm"]))
    for lw in w["layers"]:
        m["layers"].append({k: ((h(v[0]), v[1]) if isinstance(v, tuple) else h(v)) for k, v in lw.items()})
    return m


def weight_bytes_per_token(cfg=CFG):
    H, QD, KVD, I, V = cfg["hidden"], cfg["n_heads"] * cfg["head_dim"], cfg["n_kv_heads"] * cfg["head_dim"], cfg["ffn"], cfg["vocab"]
    q4 = lambda r, k: r * (k // 256) * 144
    q6 = lambda r, k: r * (k // 256) * 210
    layer = q4(QD, H) + q4(KVD, H) + q6(KVD, H) + q4(H, QD) + 2 * q4(I, H) + q6(H, I)
    return cfg["n_layers"] * layer + q6(V, H)


# ── clocks during the timed region ─────────────────────────────────────────
class ClockSampler:
    Q = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
        "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index):
        self.index, self.samples, self._stop, self._t = index, [], threading.Event(), None

    def _run(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-i", str(self.index)],
                                     capture_output=True, text=True, timeout=5).stdout.strip()
                if out:
                    self.samples.append([p.strip() for p in out.split(",")])
            except Exception:
                pass
            self._stop.wait(0.05)

    def __enter__(self):
        self._t = threading.Thread(target=self._run, daemon=True)
        self._t.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        self._t.join(timeout=6)

    def summary(self):
        mhz = [int(s[0]) for s in self.samples if s[0].isdigit()]
        mx = [int(s[1]) for s in self.samples if len(s) > 1 and s[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for s in self.samples for n, v in zip(names, s[2:6]) if v.lower().startswith("active")})
        return {"sm_mhz": int(np.median(mhz)) if mhz else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(self.samples)}


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
        except Exception:
            pass
    return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


# ── CPU baseline (oracle port) ──────────────────────────────────────────────
def cpu_decode_sample(host_model, prompt, n_steps, threads=None):
    """Times n_steps decode steps of the CPU oracle at positions following a short prefix (the KV prefix is
    built by the same oracle steps and is not timed separately: every step is a full pass over the weights)."""
    from oracle import oracle as orc
    if threads:
        orc.lib().orc_set_threads(int(threads))
    dec = orc.Decoder(host_model, MAX_CTX)
    tok = int(prompt[0])
    t0 = time.perf_counter()
    for pos in range(n_steps):
        tok = dec.step(tok if pos >= len(prompt) else int(prompt[pos]), pos)
    dt = time.perf_counter() - t0
    return n_steps / dt, int(orc.lib().orc_num_threads())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--cpu-steps", type=int, default=3)
    ap.add_argument("--streams", type=int, default=64, help="N = 1: also time this many concurrent streams (0/1: skip)")
    ap.add_argument("--parallelism", default="tp", choices=["tp", "replicas"],
                    help="N > 1: one request decoded tensor-parallel over the N GPUs (default), or N independent replicas")
    a = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    W = max(a.warmup, 3)
    K = a.steps
    config = {"workload": "qwen3-4b-shape decoder, Q4_K_M mix (Q6_K attn_v/ffn_down/output), INT8 KV, greedy decode after a "
                          f"{N_PROMPT}-token random-id prompt, batch 1",
              "n_prompt": N_PROMPT,
              "parallelism": "single" if int(os.environ.get("WORLD_SIZE", "1")) == 1 else
                             (f"tp{os.environ.get('WORLD_SIZE')} (weight rows and KV heads sharded, push gathers over NVLink)" if a.parallelism == "tp"
                              else f"{os.environ.get('WORLD_SIZE')} independent replicas"),
              "l2": "2.6 GB of weights are streamed per step (>> 126 MB L2); no explicit flush"}

    import torch

    if a.impl == "reference":
        if rank != 0:
            return
        if not torch.cuda.is_available():
            print(json.dumps({"impl": "reference", "unavailable": "needs the GPU box to draw the synthetic weights"}))
            return
        dev = torch.device("cuda", local_rank)
        torch.cuda.set_device(dev)
        host = model_to_host(gen_model_gpu(dev))
        prompt = np.random.Generator(np.random.PCG64(SEED)).integers(0, CFG["vocab"], N_PROMPT)
        n = max(1, min(K, 4))
        for _ in range(min(W, 1)):
            cpu_decode_sample(host, prompt, 1)
        v, cores = cpu_decode_sample(host, prompt, n)
        line = {"metric": "decode_tok_s", "value": v, "unit": "tok/s", "n_gpus": 0, "steps": n, "warmup": min(W, 1), "ms_per_step": 1e3 / v,
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8xq4/q6 dots, fp32 accumulate, fp16 activations",
                "data": "synthetic", "config": config, "impl": "reference",
                "cpu_baseline": {"value": v, "unit": "tok/s", "cores": cores, "kind": "port",
                                 "sample": f"{n} decode steps of the full model at positions 0..{n - 1}"},
                "e2e": {"value": v, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
        return

    from __graft_entry__ import load_package
    jb = load_package()
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    tp_mode = world > 1 and a.parallelism == "tp"
    prompt = np.random.Generator(np.random.PCG64(SEED)).integers(0, CFG["vocab"], N_PROMPT).astype(np.int32)
    if tp_mode:
        import importlib
        tpm = importlib.import_module(jb.__name__ + ".tp")
        weights = gen_model_gpu(dev, shard=(rank, world))
        dec = tpm.TPDecoder(CFG, weights, MAX_CTX, rank, world)
    else:
        weights = gen_model_gpu(dev)
        dec = jb.decoder.Decoder(CFG, weights, MAX_CTX, jb.decoder.FUSED | jb.decoder.GRAPH)
    streams = 1 if (tp_mode or world == 1) else world        # requests decoded at the same time
    stream = torch.cuda.Stream(device=dev)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    # ── e2e: per-token user call, host boundary inside ──
    pos_tok = torch.zeros(2, dtype=torch.int32).pin_memory()
    nxt = torch.zeros(1, dtype=torch.int32).pin_memory()

    def run_prompt():
        tok = None
        for p in range(N_PROMPT):
            pos_tok[0], pos_tok[1] = p, int(prompt[p])
            dec.step_sync(pos_tok, nxt, stream)
            tok = int(nxt[0])
        return tok

    with torch.cuda.stream(stream):
        tok = run_prompt()
        for i in range(W):
            pos_tok[0], pos_tok[1] = N_PROMPT + i, tok
            dec.step_sync(pos_tok, nxt, stream)
            tok = int(nxt[0])
        barrier()
        t0 = time.perf_counter()
        e2e_tokens = []
        for i in range(K):
            pos_tok[0], pos_tok[1] = N_PROMPT + W + i, tok
            dec.step_sync(pos_tok, nxt, stream)
            tok = int(nxt[0])
            e2e_tokens.append(tok)
        barrier()
        e2e_s = time.perf_counter() - t0

    # ── device-resident timing: prompt + warm-up + K steps enqueued without host synchronisation ──
    import ctypes as C
    lib = jb.lib
    h = C.c_void_p(dec._h)
    sp = C.c_void_p(stream.cuda_stream)
    out_host = np.zeros(N_PROMPT + W + K + 1, np.int32)
    # generate() = prompt steps + new tokens in one enqueue; to time only the K decode steps we enqueue the first part,
    # record an event, enqueue K more graph replays, record again.
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        tok = run_prompt()
        pos_tok[0], pos_tok[1] = N_PROMPT, tok
        dec.step_sync(pos_tok, nxt, stream)                  # leaves position/token on the device; later steps self-feed
        for _ in range(W - 1):
            jb.check(lib.jllm_b200_decoder_step_device(h, sp))
        barrier()
        l0 = jb.launch_count()
        with ClockSampler(local_rank) as clk:
            ev0.record(stream)
            for _ in range(K):
                jb.check(lib.jllm_b200_decoder_step_device(h, sp))
            ev1.record(stream)
            barrier()
        launches = jb.launch_count() - l0
    dev_ms = ev0.elapsed_time(ev1)
    status = jb.device_status(stream)

    # ── roofline of the dominant kernel: fused norm + gate/up GEMV + SwiGLU over the 36 layers' weights ──
    H, I = CFG["hidden"], CFG["ffn"] // (world if tp_mode else 1)
    x = (torch.randn(H, device=dev) * 1.0).to(torch.float16)
    sw = torch.zeros(I, dtype=torch.float16, device=dev)
    reps = 5
    with torch.cuda.stream(stream):
        for lw in weights["layers"][:4]:
            jb.norm_gemv_pair_swiglu(sw, lw["gate"][0], lw["up"][0], Q4_K, I, x, lw["rms_ffn"], True, 1e-6, H, stream)
        k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        k0.record(stream)
        for _ in range(reps):
            for lw in weights["layers"]:
                jb.norm_gemv_pair_swiglu(sw, lw["gate"][0], lw["up"][0], Q4_K, I, x, lw["rms_ffn"], True, 1e-6, H, stream)
        k1.record(stream)
        torch.cuda.synchronize()
    kern_ms = k0.elapsed_time(k1) / (reps * CFG["n_layers"])
    kern_bytes = 2 * I * (H // 256) * 144 + H * 2 + H * 4 + I * 2      # both matrices + x + norm weights + output
    peak, peak_src = measured_peaks()
    achieved = kern_bytes / (kern_ms * 1e-3) / 1e9

    # MAX over ranks
    times = torch.tensor([dev_ms, e2e_s * 1e3], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    dev_ms, e2e_ms = float(times[0]), float(times[1])

    if rank == 0:
        wbytes = weight_bytes_per_token()
        line = {
            "metric": "decode_tok_s", "value": streams * K / (dev_ms * 1e-3), "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": dev_ms / K, "higher_is_better": True, "scaling": "strong" if tp_mode else "weak", "vs_baseline": None,
            "dtype": "int8xq4/q6 dots, fp32 accumulate, fp16 activations", "data": "synthetic", "config": config,
            "e2e": {"value": streams * K / (e2e_ms * 1e-3), "unit": "tok/s", "h2d_bytes_per_step": 8, "d2h_bytes_per_step": 4},
            "gpu_launches": int(launches),
            "kernels_per_step": dec.kernels_per_step(),
            "clocks": clk.summary(),
            "roofline": {"bound": "hbm", "kernel": "gemv_stream_kernel<q8_1> (fused RMSNorm + gate/up Q4_K GEMV + SwiGLU)",
                         "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         # dram__bytes_read.sum + dram__bytes_write.sum of one launch of this kernel at this shape, from the ncu
                         # capture summarised in profiles/gemv_pair_swiglu_q4k_9728x2560.md (scaled by rows when sharded)
                         "traffic": 28077824 // (world if tp_mode else 1),
                         "bytes_per_launch": kern_bytes, "us_per_launch": kern_ms * 1e3, "peak_source": peak_src},
            "step_hbm": {"weight_bytes_per_step": wbytes, "achieved_gbs": wbytes / (dev_ms / K * 1e-3) / 1e9,
                         "frac_of_peak": wbytes / (dev_ms / K * 1e-3) / 1e9 / (peak * (world if tp_mode else 1))},
            "device_status": status,
        }
        # second workload of the same configuration: 64 concurrent streams decoded in lock step (N = 1 only)
        if world == 1 and a.streams > 1:
            try:
                bd = jb.decoder.BatchDecoder(CFG, weights, MAX_CTX, a.streams)
                bp = np.random.Generator(np.random.PCG64(SEED + 1)).integers(0, CFG["vocab"], (a.streams, N_PROMPT)).astype(np.int32)
                with torch.cuda.stream(stream):
                    bd.generate(bp, 4, stream)
                    for _ in range(3):
                        bd.step_device(stream)
                    b0, b1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    torch.cuda.synchronize()
                    b0.record(stream)
                    for _ in range(8):
                        bd.step_device(stream)
                    b1.record(stream)
                    torch.cuda.synchronize()
                bms = b0.elapsed_time(b1) / 8
                line["batch_streams"] = {"streams": a.streams, "value": a.streams / (bms * 1e-3), "unit": "tok/s", "ms_per_step": bms,
                                         "kernels_per_step": bd.kernels_per_step(), "steps": 8}
                bd.close()
            except Exception as e:          # the headline line must not depend on the side measurement
                line["batch_streams"] = {"error": str(e)[:200]}
        # CPU baseline on a bounded sample (rank 0, N = 1 only)
        if world == 1 and a.cpu_steps > 0:
            host = model_to_host(weights)
            v, cores = cpu_decode_sample(host, prompt, a.cpu_steps)
            line["cpu_baseline"] = {"value": v, "unit": "tok/s", "cores": cores, "kind": "port",
                                    "sample": f"{a.cpu_steps} decode steps of the full model at positions 0..{a.cpu_steps - 1}"}
        print(json.dumps(line))
    dec.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
