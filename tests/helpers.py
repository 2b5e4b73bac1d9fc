"""Shared helpers of the GPU parity tests."""
import numpy as np

from webllm_b200 import synthetic


def assert_close(oracle, got, ref, rtol, what=""):
    """|got - ref| <= atol + rtol*|ref| (checkTolerance, src/reference/cpu-ref.ts:27-47) with
    atol = rtol * rms(ref): a pure relative bound is unbounded where the reference output is ~0."""
    ref = np.asarray(ref, np.float32)
    atol = rtol * float(np.sqrt(np.mean(ref.astype(np.float64) ** 2)) + 1e-30)
    r = oracle.check_tolerance(np.asarray(got, np.float32), ref, atol, rtol)
    assert r.ok, f"{what}: max_abs={r.max_abs:.3e} max_rel={r.max_rel:.3e} atol={atol:.3e} rtol={rtol:g}"
    return r


def register(gpu, name, t: synthetic.GptqTensors, cols=None):
    return gpu.gptq_register(name, t.qweight, t.qzeros, t.scales, t.in_features, t.out_features, t.group_size, 4, cols)


def oracle_weight(oracle, t: synthetic.GptqTensors) -> np.ndarray:
    """The reference's dense f32 weight [N, K] for a GPTQ triple (scales decoded to f32 as readTensorF32 does)."""
    return oracle.dequantize_gptq_int4(t.qweight, t.qzeros, oracle.f16_bits_to_f32(t.scales.view(np.uint16)),
                                       t.in_features, t.out_features, t.group_size)


def run_linear(gpu, h, x, M, N, bias=None, act="f32", out="f32", exact=False):
    gpu.arena.reset()
    K = x.size // M
    A = gpu.arena.alloc(M * K, [M, K], act)
    Cc = gpu.arena.alloc(M * N, [M, N], out)
    gpu.write(A, x)
    gpu.linear(h, A, Cc, bias, M, exact=exact)
    return gpu.read(Cc).astype(np.float32).reshape(M, N)
