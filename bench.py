"""Benchmark of the quantized-linear hot path: greedy decode of a Qwen2.5-0.5B-shaped GPTQ-int4 model.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

A step is one decode step (one token) of the 24-layer model: 96 fused int4 linears (q|k|v, o, gate|up,
down per layer), the fp16 tied lm_head, the steps between them and the on-device argmax, replayed as one
CUDA graph. Weights are N(0, 0.02) quantised by round-to-nearest into the GPTQ checkpoint layout, the
prompt is 512 random ids (synthetic: no checkpoint or dataset is available offline). Every token streams
458 MB of weights, more than the 126 MB L2, so no explicit L2 flush is needed between steps.

With N > 1 (torchrun, one rank per GPU) every rank decodes its own sequence with replicated weights and
no collective; the value is the sum over ranks divided by the slowest rank's time.

`--impl reference` times the reference's CPU path for the same step (the C restatement of
dequantizeGptqInt4 + gemmNTRef + qwenForwardRef, all host threads): the reference is TypeScript and no
JavaScript engine exists on these machines.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

PROMPT_LEN = 512
METRIC = "decode_tokens_per_s"
WORKLOAD = ("Qwen2.5-0.5B-shaped GPTQ-int4 greedy decode: 24 layers, hidden 896, 14q/2kv heads x 64, MLP 4864, g=128, "
            "tied fp16 lm_head 151936x896, fp16 KV cache, 512-token random prompt, batch 1")


def int4_bytes_per_token(cfg) -> int:
    """Packed weights + fp16 scales + packed zeros of the 7 projections of every layer (algorithmic bytes)."""
    from webllm_b200 import synthetic
    total = 0
    for K, N in synthetic.QWEN05B_SHAPES.values():
        total += (K // 8) * N * 4 + (K // 128) * N * 2 + (K // 128) * (N // 8) * 4
    return total * cfg.n_layer


def measured_peak_gbs() -> tuple[float, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons every 200 ms while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self._stop, self._thread = index, [], threading.Event(), None

    def _run_nvml(self) -> bool:
        """Reads clocks and throttle reasons through NVML every 5 ms (read-only calls). False if NVML is unusable."""
        try:
            import pynvml as nv
            nv.nvmlInit()
            h = nv.nvmlDeviceGetHandleByIndex(self.index)
            mx = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
            nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)
        except Exception:
            return False
        bits = ((nv.nvmlClocksThrottleReasonHwSlowdown, 2), (nv.nvmlClocksThrottleReasonHwThermalSlowdown, 3),
                (nv.nvmlClocksThrottleReasonSwThermalSlowdown, 4), (nv.nvmlClocksThrottleReasonSwPowerCap, 5))
        while not self._stop.is_set():
            try:
                row = [str(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)), str(mx), "", "", "", ""]
                reasons = nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                for bit, col in bits:
                    row[col] = "Active" if reasons & bit else "Not Active"
                self.rows.append(row)
            except Exception:
                pass
            self._stop.wait(0.005)
        return True

    def _run(self):
        if self._run_nvml():
            return
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                      "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5).stdout
                parts = [p.strip() for p in out.strip().split(",")]
                if len(parts) >= 6:
                    self.rows.append(parts)
            except Exception:
                pass
            self._stop.wait(0.2)

    def __enter__(self):
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._thread.join(timeout=6)

    def summary(self) -> dict:
        sm = [float(r[0]) for r in self.rows if r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if r[1].replace(".", "").isdigit()]
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        reasons = sorted({n for r in self.rows for n, v in zip(names, r[2:6]) if v.lower().startswith("active")})
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(self.rows)}


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


def dense_weights_for_cpu(G):
    """Host f32 [out, in] weights of the synthetic checkpoint: what loadQwenWeights produces on the CPU
    (dequantGptqLinear per projection, src/weights/qwen-loader.ts:144-165), via the oracle's dequantiser."""
    from oracle import oracle

    def w(t):
        return oracle.dequantize_gptq_int4(t.qweight, t.qzeros, oracle.f16_bits_to_f32(t.scales.view(np.uint16)),
                                           t.in_features, t.out_features, t.group_size)
    layers = [{"input_norm": L["input_norm"], "post_norm": L["post_norm"], "qW": w(L["q"]), "qB": L["q_bias"],
               "kW": w(L["k"]), "kB": L["k_bias"], "vW": w(L["v"]), "vB": L["v_bias"], "oW": w(L["o"]),
               "gateW": w(L["gate"]), "upW": w(L["up"]), "downW": w(L["down"])} for L in G["layers"]]
    return {"embed": G["embed"].astype(np.float32), "final_norm": G["final_norm"], "layers": layers}


def cpu_decode_tokens_per_s(G, cfg, steps: int, warmup: int = 1) -> dict:
    """Times `steps` decode steps of the CPU reference path at context 512 with all host threads. The cache is
    filled with random values instead of running a 512-token CPU prefill: the arithmetic per step is the same."""
    from oracle import oracle
    threads = oracle.max_threads()
    W = dense_weights_for_cpu(G)
    ocfg = oracle.QwenConfig(cfg.vocab_size, cfg.n_layer, cfg.n_head, cfg.n_kv_head, cfg.n_embd, cfg.intermediate,
                             cfg.rms_eps, cfg.rope_theta)
    fwd = oracle.CachedForward(ocfg, W, max_t=PROMPT_LEN + steps + warmup + 1, kv_f16=True, threads=threads)
    rng = np.random.default_rng(1)
    fwd.k_cache[:, :PROMPT_LEN] = rng.standard_normal(fwd.k_cache[:, :PROMPT_LEN].shape).astype(np.float32) * 0.1
    fwd.v_cache[:, :PROMPT_LEN] = rng.standard_normal(fwd.v_cache[:, :PROMPT_LEN].shape).astype(np.float32) * 0.1
    fwd.cache_len = PROMPT_LEN
    tok = 1
    for _ in range(warmup):
        tok = oracle.sample_greedy(fwd.decode_step(tok))
    t0 = time.perf_counter()
    for _ in range(steps):
        tok = oracle.sample_greedy(fwd.decode_step(tok))
    dt = time.perf_counter() - t0
    return {"value": steps / dt, "unit": "tokens/s", "cores": threads, "kind": "port",
            "sample": f"{steps} decode steps at context {PROMPT_LEN} (cache pre-filled with random values), "
                      f"C restatement of the reference's CPU path, f32 [out,in] weights, double accumulation",
            "ms_per_step": dt / steps * 1e3}


def run_reference(args) -> None:
    """The reference arm: the CPU path of the same decode step, on rank 0 only."""
    rank, world, _ = dist_env()
    if rank != 0:
        return
    from webllm_b200 import synthetic
    cfg = synthetic.QWEN25_05B
    G = synthetic.random_qwen_gptq(cfg, seed=0)
    steps = max(1, min(args.steps, 32))  # bounded sample: a CPU step takes ~0.1 s
    base = cpu_decode_tokens_per_s(G, cfg, steps, warmup=1)
    line = {"impl": "reference", "metric": METRIC, "value": base["value"], "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": base["ms_per_step"], "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f64 accumulate over f32 weights", "data": "synthetic",
            "config": {"workload": WORKLOAD, "timed_steps": steps},
            "cpu_baseline": {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": base["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def time_batch(gpu, torch, stream, batch, reps: int) -> float:
    """Average device time of one replay of a command batch, in ms (CUDA events on the context's stream)."""
    for _ in range(3):
        batch.submit()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(reps):
        batch.submit()
    e1.record(stream)
    e1.synchronize()
    return e0.elapsed_time(e1) / reps


def kernel_sections(gpu, torch, stream, cfg, G, args) -> dict:
    """Per-kernel numbers measured live (CUDA events on the launching stream, command batches so that the
    CPU launch cost is not what is timed):
      roofline  the int4 streaming kernel (gptq_gemv_mma_kernel) over the 96 fused linears of one token;
                algorithmic bytes = packed weights + scales + zeros + f32 x + f32 y of every launch.
      extras    the other two parts of the headline metric: the single-linear GEMV case and the 7B-class
                gate shape over rotating weight copies larger than L2, and the prefill GEMM at M = 2048.
    """
    from webllm_b200 import synthetic
    peak, peak_kind = measured_peak_gbs()
    out = {}
    gpu.arena.reset()
    C, KV, I = cfg.n_embd, cfg.kv_dim, cfg.intermediate
    xin = gpu.arena.alloc(max(C, I))
    yout = gpu.arena.alloc(max(C + 2 * KV, 2 * I))
    names = []
    for i in range(cfg.n_layer):
        names += [f"L{i}.qkvW", f"L{i}.oW", f"L{i}.gateUpW", f"L{i}.downW"]
    handles = [gpu.weight(n) for n in names]
    shapes = [(C, C + 2 * KV), (C, C), (C, 2 * I), (I, C)] * cfg.n_layer
    act_bytes = sum(4 * k + 4 * n for k, n in shapes)
    algo = int4_bytes_per_token(cfg) + act_bytes
    with gpu.batch() as b:
        for h in handles:
            gpu.linear(h, xin, yout, None, 1)
    ms = time_batch(gpu, torch, stream, b, reps=20)
    b.destroy()
    per_launch_us = ms * 1e3 / len(handles)
    achieved = algo / (ms * 1e-3) / 1e9
    out["roofline"] = {"bound": "hbm", "kernel": "gptq_gemv_mma_kernel", "achieved": achieved, "peak": peak,
                       "unit": "GB/s", "frac": achieved / peak, "peak_source": f"of {peak_kind}",
                       "launches_timed": len(handles), "avg_launch_us": per_launch_us,
                       "algorithmic_bytes_per_launch": algo / len(handles), "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH}

    extras = {}
    # single-linear case: K=896 -> N=4864, batch 1, rotating over 64 distinct copies (143 MB > L2)
    def rotating_gemv(tag, K, N, copies, M=1):
        t = synthetic.random_gptq(K, N, 128, seed=0)
        hs = [gpu.gptq_register(f"bench_{tag}_{i}", t.qweight, t.qzeros, t.scales, K, N, 128) for i in range(copies)]
        gpu.arena.reset()
        A = gpu.arena.alloc(M * K, dtype="f16")
        Cc = gpu.arena.alloc(M * N, dtype="f16")
        with gpu.batch() as bb:
            for h in hs:
                gpu.linear(h, A, Cc, None, M)
        ms_ = time_batch(gpu, torch, stream, bb, reps=10)
        bb.destroy()
        nbytes = t.nbytes + 2 * M * K + 2 * M * N
        gbs = nbytes * copies / (ms_ * 1e-3) / 1e9
        return {"us_per_launch": ms_ * 1e3 / copies, "GB/s": gbs, "frac_of_hbm_peak": gbs / peak, "copies": copies,
                "bytes_per_launch": nbytes}
    extras["int4_gemv_896x4864_m1"] = rotating_gemv("c1", 896, 4864, 64)
    extras["int4_gemv_3584x18944_m1"] = rotating_gemv("g7", 3584, 18944, 8)
    # the same projection as the decode path runs it, gate|up as one matrix (70 MB per launch)
    extras["int4_gemv_3584x37888_m1"] = rotating_gemv("gu7", 3584, 37888, 4)

    # prefill GEMM, M = 2048 tokens x the four distinct 0.5B projection shapes, fp16 activations
    tf = {}
    total_flops, total_ms = 0.0, 0.0
    for tag, (K, N), count in (("q_o", (896, 896), 2), ("k_v", (896, 128), 2), ("gate_up", (896, 4864), 2), ("down", (4864, 896), 1)):
        t = synthetic.random_gptq(K, N, 128, seed=1)
        h = gpu.gptq_register(f"bench_pf_{tag}", t.qweight, t.qzeros, t.scales, K, N, 128)
        gpu.arena.reset()
        M = 2048
        A = gpu.arena.alloc(M * K, dtype="f16")
        Cc = gpu.arena.alloc(M * N, dtype="f16")
        with gpu.batch() as bb:
            for _ in range(8):
                gpu.linear(h, A, Cc, None, M)
        ms_ = time_batch(gpu, torch, stream, bb, reps=5) / 8
        bb.destroy()
        flops = 2.0 * M * N * K
        tf[tag] = {"us": ms_ * 1e3, "TFLOP/s": flops / (ms_ * 1e-3) / 1e12}
        total_flops += flops * count
        total_ms += ms_ * count
    tf["layer_aggregate_TFLOP/s"] = total_flops / (total_ms * 1e-3) / 1e12
    extras["prefill_gemm_m2048"] = tf
    # the same layer as the model launches it: q|k|v and gate|up as one projection each (4 launches per layer)
    C_, KV_, I_ = cfg.n_embd, cfg.kv_dim, cfg.intermediate
    fused_flops, fused_ms = 0.0, 0.0
    for tag, (K, N) in (("qkv", (C_, C_ + 2 * KV_)), ("o", (C_, C_)), ("gateup", (C_, 2 * I_)), ("down", (I_, C_))):
        t = synthetic.random_gptq(K, N, 128, seed=2)
        h = gpu.gptq_register(f"bench_pff_{tag}", t.qweight, t.qzeros, t.scales, K, N, 128)
        gpu.arena.reset()
        A = gpu.arena.alloc(2048 * K, dtype="f16")
        Cc = gpu.arena.alloc(2048 * N, dtype="f16")
        with gpu.batch() as bb:
            for _ in range(8):
                gpu.linear(h, A, Cc, None, 2048)
        ms_ = time_batch(gpu, torch, stream, bb, reps=5) / 8
        bb.destroy()
        fused_flops += 2.0 * 2048 * N * K
        fused_ms += ms_
    extras["prefill_gemm_m2048_fused_projections"] = {"us_per_layer": fused_ms * 1e3,
                                                      "layer_aggregate_TFLOP/s": fused_flops / (fused_ms * 1e-3) / 1e12}
    out["extras"] = extras
    return out


# dram__bytes_read.sum + dram__bytes_write.sum per launch of gptq_gemv_mma_kernel, mean over the four projections
# of a layer, from an ncu capture of a 2-layer model of the same shapes (one pass per launch, caches flushed between
# launches, the L2 prefetch of the next weight switched off); traffic is proportional to the number of layers, so the
# mean carries over to the 24-layer step. Algorithmic bytes of the same four launches: 1 956 704 on average.
NCU_TRAFFIC_BYTES_PER_LAUNCH = 2019392


def run_ours(args) -> None:
    rank, world, local = dist_env()
    import torch
    import torch.distributed as dist
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    from webllm_b200 import Gpu, QwenGpt, synthetic

    cfg = synthetic.QWEN25_05B
    G = synthetic.random_qwen_gptq(cfg, seed=0)
    K, W = args.steps, max(args.warmup, 3)
    e2e_steps = min(K, 64)
    max_t = PROMPT_LEN + W + K + e2e_steps + 8
    gpu = Gpu(local, weight_bytes=2 << 30, act_bytes=256 << 20)
    stream = torch.cuda.ExternalStream(gpu.stream, device=torch.device(f"cuda:{local}"))
    model = QwenGpt(gpu, cfg, max_t=max_t, kv_dtype="f16")
    model.upload_gptq_model(G, fuse=True)
    prompt = np.random.default_rng(100 + rank).integers(0, cfg.vocab_size, PROMPT_LEN).astype(np.uint32)
    row = model.read_tensor(model.prefill(prompt, last_only=True))
    tok = int(np.argmax(row))

    def barrier():
        gpu.synchronize()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], device=f"cuda:{local}", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- device-timed decode: W warm-up steps (captures the graph), then exactly K steps
    toks = model.decode_greedy(tok, W)
    tok = int(toks[-1])
    barrier()
    launches0 = gpu.launch_count
    with ClockSampler(local) as clocks:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        toks = model.decode_greedy(tok, K)
        e1.record(stream)
        e1.synchronize()
        barrier()
    ms_total = max_over_ranks(e0.elapsed_time(e1))
    launches = gpu.launch_count - launches0
    tok = int(toks[-1])

    # ---- end to end: one public-API call per token, token id up and sampled id down every step
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        tok = int(model.decode_greedy(tok, 1)[0])
    gpu.synchronize()
    e2e_ms = max_over_ranks((time.perf_counter() - t0) * 1e3)

    line = {"metric": METRIC, "value": world * K / (ms_total / 1e3), "unit": "tokens/s", "n_gpus": world, "steps": K,
            "warmup": W, "ms_per_step": ms_total / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "int4 weights x f32 activations (fp16 hi+lo operands), f32 accumulate", "data": "synthetic",
            "config": {"workload": WORKLOAD, "parallelism": f"replicas x{world}, no collective",
                       "l2": "each step streams 458 MB of weights (> 126 MB L2); no flush needed"},
            "e2e": {"value": world * e2e_steps / (e2e_ms / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": 12,
                    "d2h_bytes_per_step": 4, "steps": e2e_steps},
            "gpu_launches": int(launches), "clocks": clocks.summary()}

    if rank == 0:
        line.update(kernel_sections(gpu, torch, stream, cfg, G, args))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        if world == 1 and not args.no_cpu:
            base = cpu_decode_tokens_per_s(G, cfg, steps=4, warmup=1)
            line["cpu_baseline"] = {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")}
        print(json.dumps(line), flush=True)
    model.close()
    gpu.close()


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg of the default arm")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
