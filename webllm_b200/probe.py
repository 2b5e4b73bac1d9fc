"""Small fixed workloads of the hot path, one per sub-command, for profilers and quick timing.

    python -m webllm_b200.probe gemv   K N [--m 1] [--copies 8] [--act f32|f16] [--reps 2]
    python -m webllm_b200.probe gemm   K N M [--reps 2]
    python -m webllm_b200.probe decode [--steps 3] [--prompt 64] [--mode auto|graph|single] [--layers 24]

``gemv`` / ``gemm`` run one GPTQ-int4 linear (wb_linear) over ``copies`` separately registered copies of
the same synthetic weight, so that consecutive launches read different memory (no L2 reuse between
them); ``decode`` builds the Qwen2.5-0.5B-shaped synthetic GPTQ model, prefills a short random prompt and
decodes ``steps`` tokens greedily. Every run prints the launch plan and a wall-clock figure; the figure is
only a sanity check (a profiler serialises kernels), the numbers that count come from ``bench.py``.
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
    args = ap.parse_args(argv)
    if args.cmd == "gemv":
        _linear(args, args.m, args.act)
    elif args.cmd == "gemm":
        _linear(args, args.M, "f16")
    else:
        _decode(args)


if __name__ == "__main__":
    main()
