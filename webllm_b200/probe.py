"""Small fixed workloads of the hot path, one per sub-command, for profilers and quick timing.

    python -m webllm_b200.probe gemv   K N [--m 1] [--copies 8] [--act f32|f16] [--reps 2]
    python -m webllm_b200.probe gemm   K N M [--reps 2]
    python -m webllm_b200.probe decode [--steps 3] [--prompt 64] [--mode auto|graph|single] [--layers 24]
    python -m webllm_b200.probe sweep  [--which batch|big|all]

``gemv`` / ``gemm`` run one GPTQ-int4 linear (wb_linear) over ``copies`` separately registered copies of
the same synthetic weight, so that consecutive launches read different memory (no L2 reuse between
them); ``decode`` builds the Qwen2.5-0.5B-shaped synthetic GPTQ model, prefills a short random prompt and
decodes ``steps`` tokens greedily. Every run prints the launch plan and a wall-clock figure; the figure is
only a sanity check (a profiler serialises kernels), the numbers that count come from ``bench.py``.
``sweep`` is the timing table behind the batch-size sweep (M = 1 .. 64 over the seven 0.5B projection shapes)
and the 7B-class shapes (M = 1 and M = 4096): each case is a command batch over weight copies larger than L2,
replayed and timed with CUDA events (needs torch for the events).
"""
from __future__ import annotations

import argparse
import dataclasses
import time

import numpy as np

from . import Gpu, QwenGpt, synthetic


def _linear(args, M: int, act: str) -> None:
    K, N = args.K, args.N
    t = synthetic.random_gptq(K, N, 128, seed=1)
    copies = args.copies
    gpu = Gpu(0, weight_bytes=copies * (t.nbytes + (1 << 16)) + (64 << 20), act_bytes=max(64 << 20, 8 * M * (K + N)))
    hs = [gpu.gptq_register(f"w{i}", t.qweight, t.qzeros, t.scales, K, N, 128) for i in range(copies)]
    A = gpu.arena.alloc(M * K, dtype=act)
    Cc = gpu.arena.alloc(M * N, dtype=act)
    gpu.write(A, np.random.default_rng(0).standard_normal(M * K).astype(np.float32 if act == "f32" else np.float16))
    print("plan", gpu.plan(hs[0], M, act))
    gpu.synchronize()
    t0 = time.perf_counter()
    for _ in range(args.reps):
        for h in hs:
            gpu.linear(h, A, Cc, None, M)
    gpu.synchronize()
    dt = (time.perf_counter() - t0) / (args.reps * copies)
    print(f"{args.reps * copies} launches, {dt * 1e6:.1f} us each by wall clock, weight {t.nbytes} bytes per launch")


def _decode(args) -> None:
    cfg = synthetic.QWEN25_05B
    if args.layers != cfg.n_layer:
        cfg = dataclasses.replace(cfg, n_layer=args.layers)
    weights = synthetic.random_qwen_gptq(cfg, seed=0)
    gpu = Gpu(0, weight_bytes=(1 << 30) + (512 << 20), act_bytes=256 << 20)
    model = QwenGpt(gpu, cfg, max_t=1024, kv_dtype="f16")
    model.upload_gptq_model(weights, fuse=True)
    prompt = np.random.default_rng(100).integers(0, cfg.vocab_size, args.prompt).astype(np.uint32)
    tok = int(np.argmax(model.read_tensor(model.prefill(prompt, last_only=True))))
    model.set_decode_mode(args.mode)
    toks = model.decode_greedy(tok, 1)  # builds the graph / the kernel's buffers
    gpu.synchronize()
    t0 = time.perf_counter()
    toks = model.decode_greedy(int(toks[-1]), args.steps)
    dt = (time.perf_counter() - t0) / args.steps
    print(f"{args.steps} steps, {dt * 1e3:.3f} ms per step by wall clock, tokens {toks[:4].tolist()}")


def _sweep(args) -> None:
    import torch
    gpu = Gpu(0, weight_bytes=6 << 30, act_bytes=3 << 30)
    stream = torch.cuda.Stream()
    gpu.set_stream(stream.cuda_stream)

    def timed(batch, launches, reps=10):
        for _ in range(3):
            batch.submit()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(reps):
            batch.submit()
        e1.record(stream)
        e1.synchronize()
        return e0.elapsed_time(e1) * 1e3 / reps / launches  # us per launch

    def case(name, K, N, Ms, act="f16"):
        t = synthetic.random_gptq(K, N, 128, seed=1)
        copies = max(2, min(64, int(300e6 // t.nbytes)))  # > 126 MB of distinct weights per pass
        hs = [gpu.gptq_register(f"{name}_{K}x{N}_{i}", t.qweight, t.qzeros, t.scales, K, N, 128) for i in range(copies)]
        for M in Ms:
            gpu.arena.reset()
            A = gpu.arena.alloc(M * K, dtype=act)
            Cc = gpu.arena.alloc(M * N, dtype=act)
            plan = gpu.plan(hs[0], M, act)
            with gpu.batch() as b:
                for h in hs:
                    gpu.linear(h, A, Cc, None, M)
            us = timed(b, copies)
            b.destroy()
            esz = 2 if act == "f16" else 4
            nbytes = t.nbytes + esz * M * (K + N)
            print(f"{name:7s} K={K:5d} N={N:5d} M={M:4d} {plan['kernel_name']:8s} split={plan['split_k']:2d} "
                  f"{us:9.2f} us {nbytes / us / 1e3:8.1f} GB/s {2.0 * M * N * K / us / 1e6:8.2f} TFLOP/s", flush=True)
        for i in range(copies):  # weights are a stack: hand the copies back
            gpu.weight_pop()

    if args.which in ("batch", "all"):
        for name, (K, N) in synthetic.QWEN05B_SHAPES.items():
            case(name, K, N, (1, 2, 4, 8, 16, 32, 64))
    if args.which in ("big", "all"):
        for name, (K, N) in synthetic.QWEN7B_SHAPES.items():
            if name in ("q", "k", "gate", "down"):
                case(name + "7b", K, N, (1, 4096))


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(prog="python -m webllm_b200.probe", description=__doc__.split("\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    g = sub.add_parser("gemv")
    g.add_argument("K", type=int), g.add_argument("N", type=int)
    g.add_argument("--m", type=int, default=1), g.add_argument("--copies", type=int, default=8)
    g.add_argument("--act", choices=("f32", "f16"), default="f32"), g.add_argument("--reps", type=int, default=2)
    m = sub.add_parser("gemm")
    m.add_argument("K", type=int), m.add_argument("N", type=int), m.add_argument("M", type=int)
    m.add_argument("--copies", type=int, default=2), m.add_argument("--reps", type=int, default=2)
    d = sub.add_parser("decode")
    d.add_argument("--steps", type=int, default=3), d.add_argument("--prompt", type=int, default=64)
    d.add_argument("--mode", choices=("auto", "graph", "single"), default="auto")
    d.add_argument("--layers", type=int, default=synthetic.QWEN25_05B.n_layer)
    w = sub.add_parser("sweep")
    w.add_argument("--which", choices=("batch", "big", "all"), default="all")
    args = ap.parse_args(argv)
    if args.cmd == "sweep":
        _sweep(args)
    elif args.cmd == "gemv":
        _linear(args, args.m, args.act)
    elif args.cmd == "gemm":
        _linear(args, args.M, "f16")
    else:
        _decode(args)


if __name__ == "__main__":
    main()
