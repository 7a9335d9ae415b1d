"""Throughput of the lock-step batch decoder on the Qwen3-4B-shaped model (configuration 4, "64 concurrent streams").

    python genie-ai-runtime_b200/batchbench.py [--streams 64] [--steps 32] [--prompt 33]

Same synthetic weights as bench.py.  Every stream gets its own random-id prompt of the same length; after the prompt
and three warm-up steps, `steps` decode steps are timed with CUDA events (all inputs resident, no host copies inside).
Prints one JSON line: tokens per second over all streams and the time of one step.
"""
import argparse
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    import torch
    import bench
    from __graft_entry__ import load_package
    jb = load_package()
    ap = argparse.ArgumentParser()
    ap.add_argument("--streams", type=int, default=64)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--prompt", type=int, default=33)
    a = ap.parse_args()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    weights = bench.gen_model_gpu(dev)
    d = jb.decoder.BatchDecoder(bench.CFG, weights, bench.MAX_CTX, a.streams)
    rng = np.random.Generator(np.random.PCG64(bench.SEED))
    prompts = rng.integers(0, bench.CFG["vocab"], (a.streams, a.prompt)).astype(np.int32)
    st = torch.cuda.Stream(device=dev)
    with torch.cuda.stream(st):
        d.generate(prompts, 4, st)                      # prompt + 3 decode steps (warm-up); state stays on the device
        for _ in range(3):
            d.step_device(st)                           # the first call records the step as a CUDA graph
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        l0 = jb.launch_count()
        e0.record(st)
        for _ in range(a.steps):
            d.step_device(st)
        e1.record(st)
        torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / a.steps
    print(json.dumps({"metric": "batch_decode_tok_s", "streams": a.streams, "value": a.streams / (ms * 1e-3), "unit": "tok/s", "ms_per_step": ms,
                      "steps": a.steps, "kernels_per_step": d.kernels_per_step(), "gpu_launches": int(jb.launch_count() - l0),
                      "device_status": jb.device_status(st)}))
    d.close()


if __name__ == "__main__":
    main()
