"""Small fixed workloads of the hot path, one per sub-command, for profilers and quick timing.

    python -m webllm_b200.probe gemv   K N [--m 1] [--copies 8] [--act f32|f16] [--reps 2]
    python -m webllm_b200.probe gemm   K N M [--reps 2]
    python -m webllm_b200.probe decode [--steps 3] [--prompt 64] [--mode auto|graph|single] [--layers 24]
    python -m webllm_b200.probe sweep  [--which batch|big|all]
    python -m webllm_b200.probe read   [--mb 35.3]         (plain read of that many bytes, the GEMV's yardstick)
    python -m webllm_b200.probe shard      [--m 4096]      (one process per GPU: run under torch.distributed.run)
    python -m webllm_b200.probe dp-prefill [--seqs 256]    (one process per GPU: run under torch.distributed.run)

``gemv`` / ``gemm`` run one GPTQ-int4 linear (wb_linear) over ``copies`` separately registered copies of
the same synthetic weight, so that consecutive launches read different memory (no L2 reuse between
them); ``decode`` builds the Qwen2.5-0.5B-shaped synthetic GPTQ model, prefills a short random prompt and
decodes ``steps`` tokens greedily. Every run prints the launch plan and a wall-clock figure; the figure is
only a sanity check (a profiler serialises kernels), the numbers that count come from ``bench.py``.
``sweep`` is the timing table behind the batch-size sweep (M = 1 .. 64 over the seven 0.5B projection shapes)
and the 7B-class shapes (M = 1 and M = 4096): each case is a command batch over weight copies larger than L2,
replayed and timed with CUDA events (needs torch for the events).
``shard`` times the 7B-class projections split by output columns over the ranks (decode M = 1 and prefill M = --m):
the local product alone, the local product followed by the NCCL all-gather of the ``[M, N/G]`` pieces (rank-major,
and copied to row-major), and the variant whose kernel stores its tiles into every rank's slab itself
(``wb_linear_gather``) followed by a one-element all-reduce as the barrier.
``dp-prefill`` runs independent 2048-token sequences through the 96 projections of the 0.5B-shaped model
(q|k|v, o, gate|up, down per layer, fp16 activations), the sequences dealt round-robin to the ranks, weights
replicated, no collective on the data path. Both time with CUDA events and report the slowest rank.
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


def _read(args) -> None:
    """A kernel that only reads: `copies` ranges of --mb megabytes in rotation (more than L2 in all), replayed as a
    command batch like the GEMV timings, for several grid sizes."""
    import torch
    nbytes = int(args.mb * 1e6) // 256 * 256
    copies = max(2, int(300e6 // nbytes) + 1)
    gpu = Gpu(0, weight_bytes=copies * nbytes + (1 << 20), act_bytes=1 << 20)
    stream = torch.cuda.Stream()
    gpu.set_stream(stream.cuda_stream)
    for ctas in (148, 296, 592, 1184):
        with gpu.batch() as b:
            for i in range(copies):
                gpu.read_sweep(i * nbytes, nbytes, ctas)
        for _ in range(3):
            b.submit()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(10):
            b.submit()
        e1.record(stream)
        e1.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / 10 / copies
        b.destroy()
        print(f"read {nbytes} bytes, {ctas:4d} CTAs x 256: {us:7.2f} us per launch, {nbytes / us / 1e3:7.1f} GB/s", flush=True)


def _dist_init():
    """Process group over the GPUs of one node: NCCL, one rank per GPU; a plain ``python -m`` run is world size 1."""
    import os

    import torch
    import torch.distributed as dist
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device(f"cuda:{local}"))
    return torch, dist, rank, world, local


def _timed_ranks(torch, dist, fn, reps: int) -> float:
    """Device time of one call of ``fn`` in us: warm-up, barrier, CUDA events on the current stream, max over ranks."""
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    e1.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) * 1e3 / reps], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def _shard(args) -> None:
    from . import parallel
    torch, dist, rank, world, local = _dist_init()
    stream = torch.cuda.Stream()  # kernels, collectives and events all go to this stream
    torch.cuda.set_stream(stream)
    host = parallel.TorchSlabGpu(local, weight_bytes=3 << 30, act_bytes=2 << 30)
    peer = parallel.PeerSlabGpu(local, weight_bytes=3 << 30, act_bytes=2 << 30)  # for the store-to-peers variant
    gpu = host.gpu
    try:
        for name in ("q", "k", "gate", "down"):
            K, N = synthetic.QWEN7B_SHAPES[name]
            t = synthetic.random_gptq(K, N, 128, seed=1)
            for M in (1, args.m):
                # decode: rotate over copies so that a launch reads weights that are not in L2
                copies = 1 if M > 1 else max(2, min(16, int(300e6 // (t.nbytes // world))))
                lins = [parallel.ColumnShardedLinear(host, f"{name}7b_{M}_{i}", t) for i in range(copies)]
                n_loc = lins[0].shard.count
                gpu.arena.reset()
                A = gpu.arena.alloc(M * K, [M, K], "f16")
                Cl = gpu.arena.alloc(M * n_loc, [M, n_loc], "f16")
                piece = host.view(Cl).view(M, n_loc)
                out = torch.empty((world, M, n_loc), dtype=torch.float16, device=host.device)  # rank-major pieces

                def local_only():
                    for lin in lins:
                        lin.local(A, Cl, M)

                def with_gather():
                    for lin in lins:
                        lin.local(A, Cl, M)
                        dist.all_gather_into_tensor(out, piece)

                def with_gather_rowmajor():
                    for lin in lins:
                        lin.local(A, Cl, M)
                        dist.all_gather_into_tensor(out, piece)
                        out.permute(1, 0, 2).reshape(M, -1).contiguous()

                plins = [parallel.ColumnShardedLinear(peer, f"{name}7b_{M}_{i}", t) for i in range(copies)]
                peer.gpu.arena.reset()
                A2 = peer.gpu.arena.alloc(M * K, [M, K], "f16")
                Cfull = peer.gpu.arena.alloc(M * N, [M, N], "f16")
                tmp2 = peer.gpu.arena.alloc(M * n_loc, [M, n_loc], "f16")

                def fused():
                    for lin in plins:
                        lin.forward_fused(A2, Cfull, tmp2, M)

                reps = 5 if M > 1 else 3
                us_f = _timed_ranks(torch, dist, fused, reps) / copies
                for _ in plins:
                    peer.gpu.weight_pop()
                us_l = _timed_ranks(torch, dist, local_only, reps) / copies
                us_g = _timed_ranks(torch, dist, with_gather, reps) / copies
                us_r = _timed_ranks(torch, dist, with_gather_rowmajor, reps) / copies if M > 1 else us_g
                if rank == 0:
                    tf = 2.0 * M * N * K / 1e6
                    print(f"{name}7b K={K:5d} N={N:5d} M={M:4d} G={world}: local {us_l:8.2f} us, + all-gather {us_g:8.2f} us"
                          f" ({tf / us_g:7.1f} TFLOP/s, {t.nbytes / us_g / 1e3:7.1f} GB/s of int4 weights over all ranks),"
                          f" + row-major copy {us_r:8.2f} us; stores to peers + barrier {us_f:8.2f} us"
                          f" ({tf / us_f:7.1f} TFLOP/s); gathered {M * N * 2} bytes", flush=True)
                for _ in lins:
                    gpu.weight_pop()
    finally:
        peer.close()
        host.close()
        dist.destroy_process_group()


def _dp_prefill(args) -> None:
    from . import parallel
    torch, dist, rank, world, local = _dist_init()
    stream = torch.cuda.Stream()  # a command batch cannot be recorded on the default stream
    torch.cuda.set_stream(stream)
    host = parallel.TorchSlabGpu(local, weight_bytes=1 << 30, act_bytes=1 << 30)
    gpu = host.gpu
    try:
        cfg = synthetic.QWEN25_05B
        C, KV, I, M = cfg.n_embd, cfg.kv_dim, cfg.intermediate, 2048
        shapes = (("qkv", C, C + 2 * KV), ("o", C, C), ("gateup", C, 2 * I), ("down", I, C))
        tensors = {n: synthetic.random_gptq(K, N, 128, seed=3 + i) for i, (n, K, N) in enumerate(shapes)}
        handles = []
        for layer in range(cfg.n_layer):  # replicated weights, one registration per layer (186 MB > L2)
            for n, K, N in shapes:
                t = tensors[n]
                handles.append((gpu.gptq_register(f"L{layer}.{n}", t.qweight, t.qzeros, t.scales, K, N, 128), K, N))
        A = gpu.arena.alloc(M * max(C, I), dtype="f16")
        Y = gpu.arena.alloc(M * 2 * I, dtype="f16")
        mine = len(parallel.replica_share(args.seqs, rank, world))
        with gpu.batch() as one_sequence:
            for h, K, N in handles:
                gpu.linear(h, A, Y, None, M)

        def my_share():
            for _ in range(mine):
                one_sequence.submit()

        us = _timed_ranks(torch, dist, my_share, 2)
        if rank == 0:
            flops = args.seqs * cfg.n_layer * 2.0 * M * (C * (C + 2 * KV) + C * C + C * 2 * I + I * C)
            print(f"dp-prefill G={world}: {args.seqs} sequences x {M} tokens, {len(handles)} projections each: {us / 1e3:9.2f} ms,"
                  f" {args.seqs * M / us * 1e6:12.0f} tokens/s, {flops / us / 1e6:8.1f} TFLOP/s over all ranks", flush=True)
        one_sequence.destroy()
    finally:
        host.close()
        dist.destroy_process_group()


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
    rd = sub.add_parser("read")
    rd.add_argument("--mb", type=float, default=35.273728)
    sh = sub.add_parser("shard")
    sh.add_argument("--m", type=int, default=4096)
    dp = sub.add_parser("dp-prefill")
    dp.add_argument("--seqs", type=int, default=256)
    args = ap.parse_args(argv)
    if args.cmd == "read":
        _read(args)
    elif args.cmd == "shard":
        _shard(args)
    elif args.cmd == "dp-prefill":
        _dp_prefill(args)
    elif args.cmd == "sweep":
        _sweep(args)
    elif args.cmd == "gemv":
        _linear(args, args.m, args.act)
    elif args.cmd == "gemm":
        _linear(args, args.M, "f16")
    else:
        _decode(args)


if __name__ == "__main__":
    main()
