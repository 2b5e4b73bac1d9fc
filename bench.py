"""Benchmark of the quantized-linear hot path: greedy decode of a Qwen2.5-0.5B-shaped GPTQ-int4 model.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--no-cpu] [--no-extras]
    python bench.py --case gemv|gemm|decode|read ...          (small fixed workloads for a profiler, see below)

Headline. A step is one decode step (one token) of the 24-layer model: 96 fused int4 linears (q|k|v, o, gate|up,
down per layer), the fp16 tied lm_head, the steps between them and the on-device argmax, replayed as one CUDA graph.
Weights are N(0, 0.02) quantised by round-to-nearest into the GPTQ checkpoint layout, the prompt is 512 random ids
(synthetic: no checkpoint or dataset is available offline). Every token streams 458 MB of weights, more than the
126 MB L2, so no explicit L2 flush is needed between steps. The timed region is exactly K steps after the 512-token
prompt; it is repeated (prompt re-filled, untimed, in between) until at least 0.5 s has been timed, and the median
region is reported, so that the clock sampler sees the GPU under load at every N.

With N > 1 (torchrun, one rank per GPU) every rank decodes its own sequence with replicated weights and no collective;
the value is the sum over ranks divided by the slowest rank's time. Rank 0's line also carries, under `extras`, the
other parts of the metric and the configurations that shard: the single-linear GEMV and the 7B-class shapes (GB/s, % of
the measured HBM peak), the prefill GEMM at M = 2048 (0.5B shapes) and M = 4096 (7B-class shapes) in TFLOP/s and % of
the measured bf16 peak, the batch sweep M = 1..64, a prefill measured end to end, 256 independent 2048-token sequences
dealt over the ranks (replicas, no collective), and with N > 1 the 7B-class projections split by output columns over
the ranks: local product, + NCCL all-gather, + the variant whose kernels store into the peers' slabs, each with a
check of the gathered result against the unsharded product.

`--impl reference` times the reference's CPU path for the same step (the C restatement of dequantizeGptqInt4 +
gemmNTRef + qwenForwardRef, all host threads): the reference is TypeScript and no JavaScript engine exists on these
machines.

`--case` runs one small workload and prints its launch plan and a wall-clock figure (a sanity check only: profilers
serialise kernels); these are the commands the summaries under profiles/ were captured from:
    --case gemv   --K 3584 --N 18944 [--M 1] [--copies 6] [--act f16|f32] [--reps 2]   one int4 linear over `copies`
                  separately registered copies of a synthetic weight, so consecutive launches read different memory
    --case gemm   --K 896 --N 9728 --M 2048 [--copies 2] [--reps 2]                     the same with fp16 activations
    --case decode [--layers 24] [--steps 3] [--prompt 64]                                the decode step of this bench
    --case prefill [--layers 4] [--prompt 2048]                                          one prefill of that many tokens
    --case read   [--mb 35.27]                                                           a kernel that only reads (yardstick)
"""
from __future__ import annotations

import argparse
import dataclasses
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
MIN_TIMED_S = 0.5
METRIC = "decode_tokens_per_s"
WORKLOAD = ("Qwen2.5-0.5B-shaped GPTQ-int4 greedy decode: 24 layers, hidden 896, 14q/2kv heads x 64, MLP 4864, g=128, "
            "tied fp16 lm_head 151936x896, fp16 KV cache, 512-token random prompt, batch 1")
# Both arms print this same dictionary.
CONFIG = {"workload": WORKLOAD,
          "timed_region": "exactly --steps decode steps after the 512-token prompt; repeated until >= 0.5 s is timed, median region",
          "l2": "each step streams 458 MB of weights (> 126 MB L2); no flush needed"}

# dram__bytes_read.sum + dram__bytes_write.sum per launch of gptq_gemv_mma_kernel, mean over the four projections
# of a layer, from an ncu capture of a 2-layer model of the same shapes (one pass per launch, caches flushed between
# launches, the L2 prefetch of the next weight switched off); traffic is proportional to the number of layers, so the
# mean carries over to the 24-layer step. Algorithmic bytes of the same four launches: 1 956 704 on average.
NCU_TRAFFIC_BYTES_PER_LAUNCH = 2019392


def int4_bytes_per_token(cfg) -> int:
    """Packed weights + fp16 scales + packed zeros of the 7 projections of every layer (algorithmic bytes)."""
    from webllm_b200 import synthetic
    total = 0
    for K, N in synthetic.QWEN05B_SHAPES.values():
        total += (K // 8) * N * 4 + (K // 128) * N * 2 + (K // 128) * (N // 8) * 4
    return total * cfg.n_layer


def measured_peaks() -> dict:
    """HBM GB/s and bf16 TFLOP/s (burst, sustained) measured on this pool, else the documented fallback."""
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return {"hbm_gbs": float(d["hbm_gbs"]), "tflops": float(d["bf16_tflops"]),
                    "tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
        except Exception:
            pass
    return {"hbm_gbs": 6650.0, "tflops": 1590.0, "tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons while `active` is set (the timed regions): every 5 ms through NVML's
    read-only queries, nvidia-smi polling as the fallback."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self._stop, self._thread = index, [], threading.Event(), None
        self.active = threading.Event()

    def _run_nvml(self) -> bool:
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
            if self.active.is_set():
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
            if self.active.is_set():
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
    return int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))


# ---------------------------------------------------------------------------------------------------- CPU side
def oracle_weight(t):
    from oracle import oracle
    return oracle.dequantize_gptq_int4(t.qweight, t.qzeros, oracle.f16_bits_to_f32(t.scales.view(np.uint16)),
                                       t.in_features, t.out_features, t.group_size)


def dense_weights_for_cpu(G):
    """Host f32 [out, in] weights of the synthetic checkpoint: what loadQwenWeights produces on the CPU
    (dequantGptqLinear per projection, src/weights/qwen-loader.ts:144-165), via the oracle's dequantiser."""
    w = oracle_weight
    layers = [{"input_norm": L["input_norm"], "post_norm": L["post_norm"], "qW": w(L["q"]), "qB": L["q_bias"],
               "kW": w(L["k"]), "kB": L["k_bias"], "vW": w(L["v"]), "vB": L["v_bias"], "oW": w(L["o"]),
               "gateW": w(L["gate"]), "upW": w(L["up"]), "downW": w(L["down"])} for L in G["layers"]]
    return {"embed": G["embed"].astype(np.float32), "final_norm": G["final_norm"], "layers": layers}


def cpu_decode_tokens_per_s(G, cfg, steps: int, warmup: int = 1, threads: int | None = None, dense=None) -> dict:
    """Times `steps` decode steps of the CPU reference path at context 512. The cache is filled with random values
    instead of running a 512-token CPU prefill: the arithmetic per step is the same."""
    from oracle import oracle
    threads = threads or oracle.max_threads()
    W = dense if dense is not None else dense_weights_for_cpu(G)
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


def cpu_per_op(threads_all: int) -> dict:
    """The reference's CPU functions on the single-linear case (K = 896 -> N = 4864, g = 128, seed 0), one thread as in
    the reference's single-threaded JavaScript and all host threads: dequantizeGptqInt4 (ms), gemmNTRef at M = 1 (ms and
    GB/s by the GPU's algorithmic-bytes formula: int4 weights + scales + zeros + x + y), gemmNTRef at M = 64 (GFLOP/s)."""
    from oracle import oracle
    from webllm_b200 import synthetic
    rng = np.random.default_rng(0)
    K, N = 896, 4864
    t = synthetic.random_gptq(K, N, 128, rng=rng)
    x = rng.standard_normal((1, K)).astype(np.float32)
    scales = oracle.f16_bits_to_f32(t.scales.view(np.uint16))

    def best(fn, reps=3):
        ts = []
        for _ in range(reps):
            t0 = time.perf_counter()
            fn()
            ts.append(time.perf_counter() - t0)
        return min(ts)

    out = {"shape": "K=896 -> N=4864, g=128 (the single-linear case)"}
    out["dequant_ms_1_thread"] = best(lambda: oracle.dequantize_gptq_int4(t.qweight, t.qzeros, scales, K, N, 128)) * 1e3
    W = oracle.dequantize_gptq_int4(t.qweight, t.qzeros, scales, K, N, 128)
    algo = t.nbytes + 4 * K + 4 * N
    for label, th in (("1_thread", 1), (f"{threads_all}_threads", threads_all)):
        s = best(lambda: oracle.gemm_nt_ref(x, W, 1, N, K, threads=th))
        out[f"gemv_ms_{label}"] = s * 1e3
        out[f"gemv_GB/s_{label}"] = algo / s / 1e9
        xm = np.random.default_rng(1).standard_normal((64, K)).astype(np.float32)
        s = best(lambda: oracle.gemm_nt_ref(xm, W, 64, N, K, threads=th), reps=2)
        out[f"gemm_m64_GFLOP/s_{label}"] = 2.0 * 64 * N * K / s / 1e9
    return out


def run_reference(args) -> None:
    """The reference arm: the CPU path of the same decode step, on rank 0 only."""
    rank, world, _ = dist_env()
    if rank != 0:
        return
    from webllm_b200 import synthetic
    cfg = synthetic.QWEN25_05B
    G = synthetic.random_qwen_gptq(cfg, seed=0)
    steps = max(1, min(args.steps, 32))  # bounded sample: a CPU step takes ~30-100 ms
    base = cpu_decode_tokens_per_s(G, cfg, steps, warmup=1)
    line = {"impl": "reference", "metric": METRIC, "value": base["value"], "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": base["ms_per_step"], "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f64 accumulate over f32 weights", "data": "synthetic",
            "config": CONFIG, "timed_steps": steps,
            "cpu_baseline": {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": base["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------- GPU timing helpers
class Clock:
    """CUDA-event timing on the context's stream, max over ranks."""

    def __init__(self, torch, dist, stream, world: int, device):
        self.torch, self.dist, self.stream, self.world, self.device = torch, dist, stream, world, device

    def barrier(self):
        self.torch.cuda.synchronize()
        if self.world > 1:
            self.dist.barrier()

    def max_over_ranks(self, v: float) -> float:
        if self.world == 1:
            return v
        t = self.torch.tensor([v], device=self.device, dtype=self.torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def all_true(self, ok: bool) -> bool:
        if self.world == 1:
            return bool(ok)
        t = self.torch.tensor([1 if ok else 0], device=self.device, dtype=self.torch.int32)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MIN)
        return bool(int(t.item()))

    def timed_ms(self, fn, reps: int, warm: int = 3, ranks: bool = False) -> float:
        """Average device time of one call of fn() in ms."""
        for _ in range(warm):
            fn()
        if ranks:
            self.barrier()
        e0, e1 = self.torch.cuda.Event(enable_timing=True), self.torch.cuda.Event(enable_timing=True)
        e0.record(self.stream)
        for _ in range(reps):
            fn()
        e1.record(self.stream)
        e1.synchronize()
        ms = e0.elapsed_time(e1) / reps
        return self.max_over_ranks(ms) if ranks else ms


def rotating_linear(gpu, clock, tag, t, M, act="f16", copies=None, reps=10):
    """us per launch of one GPTQ linear at M rows, replayed as a command batch over separately registered copies of
    the weight (more than L2 in all), so that every launch streams its weight from HBM. Returns (us, plan)."""
    K, N = t.in_features, t.out_features
    copies = copies or max(2, min(64, int(300e6 // t.nbytes)))
    hs = [gpu.gptq_register(f"{tag}_{i}", t.qweight, t.qzeros, t.scales, K, N, t.group_size) for i in range(copies)]
    try:
        out = {}
        for m in (M if isinstance(M, (list, tuple)) else [M]):
            gpu.arena.reset()
            A = gpu.arena.alloc(m * K, dtype=act)
            Cc = gpu.arena.alloc(m * N, dtype=act)
            plan = gpu.plan(hs[0], m, act)
            with gpu.batch() as b:
                for h in hs:
                    gpu.linear(h, A, Cc, None, m)
            ms = clock.timed_ms(b.submit, reps)
            b.destroy()
            out[m] = (ms * 1e3 / copies, plan)
        return out if isinstance(M, (list, tuple)) else out[M]
    finally:
        for _ in hs:
            gpu.weight_pop()


# ---------------------------------------------------------------------------------------------------- sections of the line
def kernel_sections(gpu, clock, cfg, peaks) -> dict:
    """roofline: the int4 GEMV over the 96 fused linears of one token (command batch, CUDA events on the launching
    stream); algorithmic bytes = packed weights + scales + zeros + f32 x + f32 y of every launch."""
    peak = peaks["hbm_gbs"]
    gpu.arena.reset()
    C, KV, I = cfg.n_embd, cfg.kv_dim, cfg.intermediate
    xin = gpu.arena.alloc(max(C, I))
    yout = gpu.arena.alloc(max(C + 2 * KV, 2 * I))
    names = []
    for i in range(cfg.n_layer):
        names += [f"L{i}.qkvW", f"L{i}.oW", f"L{i}.gateUpW", f"L{i}.downW"]
    handles = [gpu.weight(n) for n in names]
    shapes = [(C, C + 2 * KV), (C, C), (C, 2 * I), (I, C)] * cfg.n_layer
    algo = int4_bytes_per_token(cfg) + sum(4 * k + 4 * n for k, n in shapes)
    with gpu.batch() as b:
        for h in handles:
            gpu.linear(h, xin, yout, None, 1)
    ms = clock.timed_ms(b.submit, reps=20)
    b.destroy()
    achieved = algo / (ms * 1e-3) / 1e9
    return {"bound": "hbm", "kernel": "gptq_gemv_mma_kernel", "achieved": achieved, "peak": peak, "unit": "GB/s",
            "frac": achieved / peak, "peak_source": f"of {peaks['source']}", "launches_timed": len(handles),
            "avg_launch_us": ms * 1e3 / len(handles), "algorithmic_bytes_per_launch": algo / len(handles),
            "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH}


def gemv_extras(gpu, clock, peaks) -> dict:
    """The decode GEMV part of the metric: the single-linear case and the 7B-class shapes at M = 1, fp16 activations."""
    from webllm_b200 import synthetic
    out = {}
    for tag, K, N, copies in (("int4_gemv_896x4864_m1", 896, 4864, 64), ("int4_gemv_3584x18944_m1", 3584, 18944, 8),
                              ("int4_gemv_3584x37888_m1", 3584, 37888, 4), ("int4_gemv_18944x3584_m1", 18944, 3584, 8),
                              ("int4_gemv_3584x3584_m1", 3584, 3584, 40)):
        t = synthetic.random_gptq(K, N, 128, seed=0)
        us, plan = rotating_linear(gpu, clock, "bx_" + tag, t, 1, "f16", copies)
        nbytes = t.nbytes + 2 * K + 2 * N
        gbs = nbytes / us / 1e3
        out[tag] = {"us_per_launch": us, "GB/s": gbs, "frac_of_hbm_peak": gbs / peaks["hbm_gbs"], "copies": copies,
                    "bytes_per_launch": nbytes, "kernel": plan["kernel_name"], "split_k": plan["split_k"]}
    return out


def gemm_extras(gpu, clock, cfg, peaks) -> dict:
    """The prefill GEMM part of the metric, fp16 activations and outputs: M = 2048 on the 0.5B shapes (separately and
    as the model launches them, q|k|v and gate|up fused) and M = 4096 on the 7B-class shapes."""
    from webllm_b200 import synthetic
    out = {}

    def one(tag, K, N, M, seed):
        t = synthetic.random_gptq(K, N, 128, seed=seed)
        h = gpu.gptq_register(tag, t.qweight, t.qzeros, t.scales, K, N, 128)
        try:
            gpu.arena.reset()
            A = gpu.arena.alloc(M * K, dtype="f16")
            Cc = gpu.arena.alloc(M * N, dtype="f16")
            plan = gpu.plan(h, M, "f16")
            with gpu.batch() as bb:
                for _ in range(8):
                    gpu.linear(h, A, Cc, None, M)
            ms = clock.timed_ms(bb.submit, reps=5) / 8
            bb.destroy()
        finally:
            gpu.weight_pop()
        return ms, plan

    tf, total_flops, total_ms = {}, 0.0, 0.0
    for tag, (K, N), count in (("q_o", (896, 896), 2), ("k_v", (896, 128), 2), ("gate_up", (896, 4864), 2), ("down", (4864, 896), 1)):
        ms, plan = one(f"bench_pf_{tag}", K, N, 2048, 1)
        flops = 2.0 * 2048 * N * K
        tf[tag] = {"us": ms * 1e3, "TFLOP/s": flops / (ms * 1e-3) / 1e12, "tile": [plan["tile_m"], plan["tile_n"]], "split_k": plan["split_k"]}
        total_flops += flops * count
        total_ms += ms * count
    tf["layer_aggregate_TFLOP/s"] = total_flops / (total_ms * 1e-3) / 1e12
    tf["frac_of_bf16_peak"] = tf["layer_aggregate_TFLOP/s"] / peaks["tflops"]
    out["prefill_gemm_m2048"] = tf
    C_, KV_, I_ = cfg.n_embd, cfg.kv_dim, cfg.intermediate
    fused_flops, fused_ms, per = 0.0, 0.0, {}
    for tag, (K, N) in (("qkv", (C_, C_ + 2 * KV_)), ("o", (C_, C_)), ("gateup", (C_, 2 * I_)), ("down", (I_, C_))):
        ms, _ = one(f"bench_pff_{tag}", K, N, 2048, 2)
        per[tag] = {"us": ms * 1e3, "TFLOP/s": 2.0 * 2048 * N * K / (ms * 1e-3) / 1e12}
        fused_flops += 2.0 * 2048 * N * K
        fused_ms += ms
    agg = fused_flops / (fused_ms * 1e-3) / 1e12
    out["prefill_gemm_m2048_fused_projections"] = {"us_per_layer": fused_ms * 1e3, "layer_aggregate_TFLOP/s": agg,
                                                   "frac_of_bf16_peak": agg / peaks["tflops"], **per}
    big = {}
    for tag, name in (("q", "q"), ("k", "k"), ("gate", "gate"), ("down", "down")):
        K, N = synthetic.QWEN7B_SHAPES[name]
        ms, plan = one(f"bench_7b_{tag}", K, N, 4096, 3)
        tfl = 2.0 * 4096 * N * K / (ms * 1e-3) / 1e12
        big[tag] = {"K": K, "N": N, "us": ms * 1e3, "TFLOP/s": tfl, "frac_of_bf16_peak": tfl / peaks["tflops"],
                    "frac_of_bf16_sustained": tfl / peaks["tflops_sustained"], "tile": [plan["tile_m"], plan["tile_n"]],
                    "split_k": plan["split_k"]}
    out["prefill_gemm_7b_m4096"] = big
    return out


def batch_sweep(gpu, clock) -> dict:
    """Batched decode, M in {1, 2, 4, 8, 16, 32, 64} over the four distinct 0.5B projection shapes, fp16 activations:
    us per launch and the kernel the planner picks (the switch from the GEMV to the tcgen05 GEMM)."""
    from webllm_b200 import synthetic
    out = {}
    for name in ("q", "k", "gate", "down"):
        K, N = synthetic.QWEN05B_SHAPES[name]
        t = synthetic.random_gptq(K, N, 128, seed=1)
        res = rotating_linear(gpu, clock, f"sweep_{name}", t, [1, 2, 4, 8, 16, 32, 64], "f16", reps=5)
        out[f"{name}_{K}x{N}"] = {f"M={m}": {"us": round(us, 3), "kernel": plan["kernel_name"], "split_k": plan["split_k"],
                                              "GB/s": round((t.nbytes + 2 * m * (K + N)) / us / 1e3, 1),
                                              "TFLOP/s": round(2.0 * m * N * K / us / 1e6, 2)} for m, (us, plan) in res.items()}
    return out


def prefill_e2e(gpu, cfg, tokens_n: int = 2048) -> dict:
    """Prefill through the public host API: 2048 token ids from host memory -> wb_qwen_prefill(last_only) -> the logits
    row back in host memory, wall clock around the whole call chain (a second model object on the same weights)."""
    from webllm_b200 import QwenGpt
    model = QwenGpt(gpu, cfg, max_t=tokens_n, kv_dtype="f16")
    try:
        toks = np.random.default_rng(7).integers(0, cfg.vocab_size, tokens_n).astype(np.uint32)
        ts = []
        for i in range(4):
            model.reset_cache()
            gpu.synchronize()
            t0 = time.perf_counter()
            row = model.read_tensor(model.prefill(toks, last_only=True))
            ts.append(time.perf_counter() - t0)
        assert np.isfinite(row).all()
        dt = statistics.median(ts[1:])
        return {"tokens": tokens_n, "ms": dt * 1e3, "tokens/s": tokens_n / dt, "h2d_bytes": int(toks.nbytes), "d2h_bytes": int(row.nbytes)}
    finally:
        model.close()


def replicated_prefill(gpu, clock, cfg, peaks, rank: int, world: int, seqs: int = 256, M: int = 2048) -> dict:
    """256 independent 2048-token sequences through the 96 projections of the model (q|k|v, o, gate|up, down per layer,
    fp16 activations), dealt round-robin to the ranks, weights replicated, no collective on the data path."""
    from webllm_b200 import parallel
    C, KV, I = cfg.n_embd, cfg.kv_dim, cfg.intermediate
    shapes = (("qkvW", C, C + 2 * KV), ("oW", C, C), ("gateUpW", C, 2 * I), ("downW", I, C))
    gpu.arena.reset()
    A = gpu.arena.alloc(M * max(C, I), dtype="f16")
    Y = gpu.arena.alloc(M * 2 * I, dtype="f16")
    mine = len(parallel.replica_share(seqs, rank, world))
    with gpu.batch() as one_sequence:
        for layer in range(cfg.n_layer):
            for n, K, N in shapes:
                gpu.linear(gpu.weight(f"L{layer}.{n}"), A, Y, None, M)

    def my_share():
        for _ in range(mine):
            one_sequence.submit()

    ms = clock.timed_ms(my_share, reps=2, warm=1, ranks=True)
    one_sequence.destroy()
    flops = seqs * cfg.n_layer * 2.0 * M * sum(K * N for _, K, N in shapes)
    tfl = flops / (ms * 1e-3) / 1e12
    return {"sequences": seqs, "tokens_per_sequence": M, "ranks": world, "ms": ms, "tokens/s": seqs * M / (ms * 1e-3),
            "TFLOP/s": tfl, "frac_of_bf16_peak_per_gpu": tfl / world / peaks["tflops"], "scaling": "strong", "collective": "none"}


def column_shards(torch, dist, clock, rank: int, world: int, local: int, m_prefill: int = 4096) -> dict:
    """7B-class projections split by output columns over the ranks: decode (M = 1) and prefill (M = 4096), fp16 in and
    out. Per case: the unsharded product on one GPU, the local product of a shard, + the NCCL all-gather enqueued by the
    library (rank-major pieces, and rearranged to row-major), and the variant whose kernels store into every rank's slab
    followed by the library's barrier kernel. `ok_*`: every rank compared sampled rows of the gathered [M, N] with its
    own unsharded product."""
    from webllm_b200 import parallel, synthetic
    stream = torch.cuda.Stream()
    out = {}
    with torch.cuda.stream(stream):
        host = parallel.ShardGroup(local, weight_bytes=(2 << 30) + (512 << 20), act_bytes=1 << 30)
        gpu = host.gpu
        sclock = Clock(torch, dist, stream, world, clock.device)
        try:
            for name in ("gate", "down", "q"):
                K, N = synthetic.QWEN7B_SHAPES[name]
                t = synthetic.random_gptq(K, N, 128, seed=1)
                for M in (1, m_prefill):
                    progress(f"column shards: {name} M={M} (rank {rank})")
                    copies = 1 if M > 1 else max(2, min(16, int(300e6 // (t.nbytes // world))))
                    full_copies = 1 if M > 1 else max(2, min(8, int(300e6 // t.nbytes)))
                    lins = [parallel.ColumnShardedLinear(host, f"{name}7b_{M}_{i}", t) for i in range(copies)]
                    fulls = [gpu.gptq_register(f"{name}7b_full_{M}_{i}", t.qweight, t.qzeros, t.scales, K, N, 128) for i in range(full_copies)]
                    n_loc = lins[0].shard.count
                    gpu.arena.reset()
                    A = gpu.arena.alloc(M * K, [M, K], "f16")
                    Cf = gpu.arena.alloc(M * N, [M, N], "f16")
                    Cref = gpu.arena.alloc(M * N, [M, N], "f16")
                    Cl = gpu.arena.alloc(M * n_loc, [M, n_loc], "f16")
                    scratch = gpu.arena.alloc(lins[0].scratch_elems(M), dtype="f16")
                    gpu.write(A, np.random.default_rng(3).standard_normal(M * K).astype(np.float16))
                    rows = sorted({0, M - 1} | set(np.random.default_rng(4).integers(0, M, 6).tolist()))

                    def sample(tn):
                        return np.stack([gpu.read(tn, r * N, N).astype(np.float32) for r in rows])

                    def agrees(tn, ref):
                        got = sample(tn)
                        rms = float(np.sqrt(np.mean(ref.astype(np.float64) ** 2))) + 1e-30
                        return bool(np.all(np.abs(got - ref) <= 2e-3 * rms + 2e-3 * np.abs(ref)))

                    gpu.linear(fulls[0], A, Cref, None, M)
                    ref = sample(Cref)
                    lins[0].forward(A, Cf, scratch, M, row_major=True)
                    ok_nccl = agrees(Cf, ref)
                    gpu.write(Cf, np.zeros(M * N, np.float16))  # the second check must not pass on the first one's result
                    gpu.synchronize()
                    dist.barrier()
                    lins[0].forward_fused(A, Cf, Cl, M)
                    ok_stores = agrees(Cf, ref)
                    gpu.synchronize()
                    dist.barrier()

                    # kernels of this library are timed as replayed command batches (the host's launch rate is not what
                    # is measured); the NCCL variant is enqueued call by call
                    def batched(calls):
                        with gpu.batch() as b:
                            for c in calls:
                                c()
                        return b

                    reps = 5 if M > 1 else 10
                    b_full = batched([lambda h=h: gpu.linear(h, A, Cref, None, M) for h in fulls])
                    b_local = batched([lambda lin=lin: lin.local(A, Cl, M) for lin in lins])
                    b_st = batched([lambda lin=lin: lin.forward_fused(A, Cf, Cl, M) for lin in lins])
                    us_full = sclock.timed_ms(b_full.submit, reps, ranks=True) * 1e3 / full_copies
                    us_local = sclock.timed_ms(b_local.submit, reps, ranks=True) * 1e3 / copies
                    us_st = sclock.timed_ms(b_st.submit, reps, ranks=True) * 1e3 / copies
                    for b in (b_full, b_local, b_st):
                        b.destroy()
                    nreps = 5 if M > 1 else 3
                    us_rank = sclock.timed_ms(lambda: [lin.forward(A, Cf, scratch, M, row_major=False) for lin in lins], nreps, ranks=True) * 1e3 / copies
                    us_row = (sclock.timed_ms(lambda: [lin.forward(A, Cf, scratch, M, row_major=True) for lin in lins], nreps, ranks=True) * 1e3 / copies
                              if M > 1 else us_rank)
                    gpu.synchronize()
                    dist.barrier()
                    for _ in range(full_copies + copies):
                        gpu.weight_pop()
                    out[f"{name}_{K}x{N}_m{M}"] = {
                        "ranks": world, "unsharded_us": us_full, "local_us": us_local, "nccl_allgather_rank_major_us": us_rank,
                        "nccl_allgather_row_major_us": us_row, "peer_stores_barrier_us": us_st,
                        "speedup_nccl": us_full / us_row, "speedup_peer_stores": us_full / us_st,
                        "ok_nccl": sclock.all_true(ok_nccl), "ok_peer_stores": sclock.all_true(ok_stores),
                        "gathered_bytes": M * N * 2}
        finally:
            host.close()
    return out


# ---------------------------------------------------------------------------------------------------- our arm
def run_ours(args) -> None:
    rank, world, local = dist_env()
    # libraries (NCCL's version banner) may write to stdout: everything but the JSON line goes to stderr
    json_out = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    import torch
    import torch.distributed as dist
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    from webllm_b200 import Gpu, QwenGpt, synthetic

    peaks = measured_peaks()
    cfg = synthetic.QWEN25_05B
    G = synthetic.random_qwen_gptq(cfg, seed=0)
    K, W = args.steps, max(args.warmup, 3)
    e2e_steps = min(K, 64)
    max_t = PROMPT_LEN + max(W, K, e2e_steps) + 8
    gpu = Gpu(local, weight_bytes=(2 << 30) + (512 << 20), act_bytes=1 << 30)
    device = torch.device(f"cuda:{local}")
    stream = torch.cuda.ExternalStream(gpu.stream, device=device)
    clock = Clock(torch, dist, stream, world, device)
    model = QwenGpt(gpu, cfg, max_t=max_t, kv_dtype="f16")
    model.upload_gptq_model(G, fuse=True)
    prompt = np.random.default_rng(100 + rank).integers(0, cfg.vocab_size, PROMPT_LEN).astype(np.uint32)

    def refill() -> int:
        """Back to the state right after the prompt (untimed); returns the first sampled token."""
        model.reset_cache()
        return int(np.argmax(model.read_tensor(model.prefill(prompt, last_only=True))))

    def barrier():
        gpu.synchronize()
        clock.barrier()

    # ---- device-timed decode: W warm-up steps (captures the graph), then regions of exactly K steps
    tok = refill()
    model.decode_greedy(tok, W)
    launches_per_region, regions = 0, []
    with ClockSampler(local) as clocks:
        timed_s = 0.0
        while timed_s < MIN_TIMED_S and len(regions) < 200:
            tok = refill()
            barrier()
            launches0 = gpu.launch_count
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            clocks.active.set()
            e0.record(stream)
            toks = model.decode_greedy(tok, K)
            e1.record(stream)
            e1.synchronize()
            clocks.active.clear()
            barrier()
            launches_per_region = gpu.launch_count - launches0
            ms = clock.max_over_ranks(e0.elapsed_time(e1))
            regions.append(ms)
            timed_s += ms / 1e3
    ms_total = statistics.median(regions)
    tok = int(toks[-1])

    # ---- end to end: one public-API call per token, token id up and sampled id down every step
    tok = refill()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        tok = int(model.decode_greedy(tok, 1)[0])
    gpu.synchronize()
    e2e_ms = clock.max_over_ranks((time.perf_counter() - t0) * 1e3)

    line = {"metric": METRIC, "value": world * K / (ms_total / 1e3), "unit": "tokens/s", "n_gpus": world, "steps": K,
            "warmup": W, "ms_per_step": ms_total / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "int4 weights x f32 activations (fp16 hi+lo operands), f32 accumulate", "data": "synthetic",
            "config": CONFIG, "parallelism": f"replicas x{world}, no collective on the data path",
            "timed_regions": len(regions), "region_ms_min_max": [min(regions), max(regions)],
            "e2e": {"value": world * e2e_steps / (e2e_ms / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": 12,
                    "d2h_bytes_per_step": 4, "steps": e2e_steps},
            "gpu_launches": int(launches_per_region), "clocks": clocks.summary()}

    extras = {}
    if rank == 0:
        line["roofline"] = kernel_sections(gpu, clock, cfg, peaks)
        # the same question for the whole step (all 125 launches, lm_head included), from the headline's own timing:
        # weight bytes that one token has to stream / the measured step time
        step_bytes = int4_bytes_per_token(cfg) + cfg.vocab_size * cfg.n_embd * 2
        step_gbs = step_bytes / (line["ms_per_step"] * 1e-3) / 1e9
        line["roofline"]["whole_step"] = {"algorithmic_bytes": step_bytes, "achieved": step_gbs, "unit": "GB/s",
                                          "frac": step_gbs / peaks["hbm_gbs"], "hbm_floor_ms": step_bytes / peaks["hbm_gbs"] / 1e6}
    if not args.no_extras:
        if rank == 0:
            progress("extras: gemv")
            extras.update(gemv_extras(gpu, clock, peaks))
            progress("extras: gemm")
            extras.update(gemm_extras(gpu, clock, cfg, peaks))
            progress("extras: batch sweep")
            extras["batch_sweep_05b"] = batch_sweep(gpu, clock)
            progress("extras: prefill end to end")
            extras["prefill_e2e_2048"] = prefill_e2e(gpu, cfg)
        barrier()
        progress(f"extras: replicated prefill (rank {rank})")
        rp = replicated_prefill(gpu, clock, cfg, peaks, rank, world)  # every rank takes part
        if rank == 0:
            extras["replicated_prefill_256x2048"] = rp
    model.close()
    gpu.close()
    if world > 1 and not args.no_extras:
        progress(f"extras: column shards (rank {rank})")
        cs = column_shards(torch, dist, clock, rank, world, local)
        if rank == 0:
            extras["column_shards_7b"] = cs
    if rank == 0:
        line["extras"] = extras
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        if world == 1 and not args.no_cpu:
            from oracle import oracle
            dense = dense_weights_for_cpu(G)
            base = cpu_decode_tokens_per_s(G, cfg, steps=4, warmup=1, dense=dense)
            one = cpu_decode_tokens_per_s(G, cfg, steps=2, warmup=0, threads=1, dense=dense)
            line["cpu_baseline"] = {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")}
            line["cpu_baseline"]["decode_tokens_per_s_1_thread"] = one["value"]
            line["cpu_baseline"]["per_op"] = cpu_per_op(oracle.max_threads())
        json_out.write(json.dumps(line) + "\n")
        json_out.flush()


# ---------------------------------------------------------------------------------------------------- profiler cases
def progress(msg: str) -> None:
    """One line on stderr per section: a run that dies half-way says where."""
    print(f"[bench] {msg}", file=sys.stderr, flush=True)


def run_case(args) -> None:
    from webllm_b200 import Gpu, QwenGpt, synthetic
    if args.case in ("gemv", "gemm"):
        K, N = args.K, args.N
        M = args.M if args.case == "gemm" or args.M else 1
        act = "f16" if args.case == "gemm" else args.act
        t = synthetic.random_gptq(K, N, 128, seed=1)
        gpu = Gpu(0, weight_bytes=args.copies * (t.nbytes + (1 << 16)) + (64 << 20), act_bytes=max(64 << 20, 8 * M * (K + N)))
        hs = [gpu.gptq_register(f"w{i}", t.qweight, t.qzeros, t.scales, K, N, 128) for i in range(args.copies)]
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
        dt = (time.perf_counter() - t0) / (args.reps * args.copies)
        print(f"{args.reps * args.copies} launches, {dt * 1e6:.1f} us each by wall clock, weight {t.nbytes} bytes per launch")
        gpu.close()
    elif args.case == "decode":
        cfg = synthetic.QWEN25_05B
        if args.layers != cfg.n_layer:
            cfg = dataclasses.replace(cfg, n_layer=args.layers)
        weights = synthetic.random_qwen_gptq(cfg, seed=0)
        gpu = Gpu(0, weight_bytes=(1 << 30) + (512 << 20), act_bytes=256 << 20)
        model = QwenGpt(gpu, cfg, max_t=1024, kv_dtype="f16")
        model.upload_gptq_model(weights, fuse=True)
        prompt = np.random.default_rng(100).integers(0, cfg.vocab_size, args.prompt).astype(np.uint32)
        tok = int(np.argmax(model.read_tensor(model.prefill(prompt, last_only=True))))
        toks = model.decode_greedy(tok, 1)  # builds the graph
        gpu.synchronize()
        t0 = time.perf_counter()
        toks = model.decode_greedy(int(toks[-1]), args.steps)
        dt = (time.perf_counter() - t0) / args.steps
        print(f"{args.steps} steps, {dt * 1e3:.3f} ms per step by wall clock, tokens {toks[:4].tolist()}")
        model.close()
        gpu.close()
    elif args.case == "prefill":
        cfg = dataclasses.replace(synthetic.QWEN25_05B, n_layer=args.layers)
        weights = synthetic.random_qwen_gptq(cfg, seed=0)
        gpu = Gpu(0, weight_bytes=(1 << 30) + (512 << 20), act_bytes=1 << 30)
        model = QwenGpt(gpu, cfg, max_t=args.prompt, kv_dtype="f16")
        model.upload_gptq_model(weights, fuse=True)
        prompt = np.random.default_rng(100).integers(0, cfg.vocab_size, args.prompt).astype(np.uint32)
        for _ in range(2):
            model.reset_cache()
            gpu.synchronize()
            t0 = time.perf_counter()
            row = model.read_tensor(model.prefill(prompt, last_only=True))
            dt = time.perf_counter() - t0
        print(f"prefill of {args.prompt} tokens through {cfg.n_layer} layers: {dt * 1e3:.3f} ms by wall clock, argmax {int(row.argmax())}")
        model.close()
        gpu.close()
    elif args.case == "read":
        import torch
        nbytes = int(args.mb * 1e6) // 256 * 256
        copies = max(2, int(300e6 // nbytes) + 1)
        gpu = Gpu(0, weight_bytes=copies * nbytes + (1 << 20), act_bytes=1 << 20)
        stream = torch.cuda.Stream()
        gpu.set_stream(stream.cuda_stream)
        clock = Clock(torch, None, stream, 1, torch.device("cuda:0"))
        for ctas in (148, 296, 592, 1184):
            with gpu.batch() as b:
                for i in range(copies):
                    gpu.read_sweep(i * nbytes, nbytes, ctas)
            us = clock.timed_ms(b.submit, 10) * 1e3 / copies
            b.destroy()
            print(f"read {nbytes} bytes, {ctas:4d} CTAs x 256: {us:7.2f} us per launch, {nbytes / us / 1e3:7.1f} GB/s", flush=True)
        gpu.close()


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg of the default arm")
    ap.add_argument("--no-extras", action="store_true", help="headline and roofline only")
    ap.add_argument("--case", choices=("gemv", "gemm", "decode", "prefill", "read"), help="run one small profiler workload instead")
    ap.add_argument("--K", type=int, default=3584), ap.add_argument("--N", type=int, default=18944)
    ap.add_argument("--M", type=int, default=0), ap.add_argument("--copies", type=int, default=8)
    ap.add_argument("--act", choices=("f32", "f16"), default="f32"), ap.add_argument("--reps", type=int, default=2)
    ap.add_argument("--layers", type=int, default=24), ap.add_argument("--prompt", type=int, default=64)
    ap.add_argument("--mb", type=float, default=35.273728)
    args = ap.parse_args()
    if args.case:
        if args.case == "decode" and args.steps == 128:
            args.steps = 3
        if args.case == "prefill" and args.layers == 24:
            args.layers = 4
        if args.case == "prefill" and args.prompt == 64:
            args.prompt = 2048
        run_case(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
