"""GPU parity: the fused int4 linear (GEMV / split-K / small batch / ragged) and the fp16 dense GEMV
against gemmNTRef on the oracle's dequantised weights, through the C ABI."""
import numpy as np
import pytest

from helpers import assert_close, oracle_weight, register, run_linear
from webllm_b200 import WebllmError, _lib, synthetic

pytestmark = pytest.mark.gpu

F32_RTOL = 1e-5   # fp32-activation mode
F16_RTOL = 1e-3   # fp16 activations


def _x(M, K, seed, f16=False):
    x = np.random.default_rng(seed).standard_normal((M, K)).astype(np.float32)
    return x.astype(np.float16) if f16 else x


def test_single_linear_benchmark_case(gpu, oracle):
    """K=896 -> N=4864, batch 1, group 128, stored zeros in {7,8}, scales |N(0.01,0.003)|, x ~ N(0,1), seed 0
    (draw order: qweight, qzeros, scales, x)."""
    rng = np.random.default_rng(0)
    t = synthetic.random_gptq(896, 4864, 128, rng=rng)
    x = rng.standard_normal((1, 896)).astype(np.float32)
    h = register(gpu, "up_proj", t)
    ref = oracle.gemm_nt_ref(x, oracle_weight(oracle, t), 1, 4864, 896)
    p = gpu.plan(h, 1)
    assert p["kernel_name"] == "gemv_mma"
    assert_close(oracle, run_linear(gpu, h, x, 1, 4864), ref, F32_RTOL, "f32 activations")
    x16 = x.astype(np.float16)
    ref16 = oracle.gemm_nt_ref(x16.astype(np.float32), oracle_weight(oracle, t), 1, 4864, 896)
    assert_close(oracle, run_linear(gpu, h, x16, 1, 4864, act="f16"), ref16, F16_RTOL, "f16 activations")
    # the reference's own GEMV bar (atol 1e-5 + rtol 1e-4, src/tests/kernels.ts:61-74,1267)
    assert oracle.check_tolerance(run_linear(gpu, h, x, 1, 4864), ref, 1e-5, 1e-4).ok


@pytest.mark.parametrize("name,K,N", [(n, k, nn) for n, (k, nn) in synthetic.QWEN05B_SHAPES.items() if n in ("q", "k", "gate", "down")]
                         + [("q7b", 3584, 3584), ("kv7b", 3584, 512), ("down7b", 18944, 3584)])
@pytest.mark.parametrize("M", [1, 2, 3, 4, 6, 8, 9, 16, 32])
def test_small_batch_all_shapes(gpu, oracle, name, K, N, M):
    if K == 18944 and M not in (1, 8):
        pytest.skip("one small and one larger batch are enough at the largest K")
    key = f"sb_{name}"
    try:
        h = gpu.weight(key)
        t = test_small_batch_all_shapes.cache[key]
    except WebllmError:
        t = synthetic.random_gptq(K, N, 128, seed=K + N, zeros="any")
        h = register(gpu, key, t)
        test_small_batch_all_shapes.cache[key] = t
    W = test_small_batch_all_shapes.wcache.setdefault(key, oracle_weight(oracle, t))
    bias_key = f"sbb_{name}"
    try:
        hb = gpu.weight(bias_key)
    except WebllmError:
        hb = gpu.f32_upload(bias_key, np.random.default_rng(N).standard_normal(N).astype(np.float32))
    bias = np.random.default_rng(N).standard_normal(N).astype(np.float32)
    gpu.plan_override(_lib.WB_KERNEL_GEMV_MMA, 0)
    try:
        x = _x(M, K, M * 31 + K)
        ref = oracle.gemm_nt_ref(x, W, M, N, K, bias, threads=oracle.max_threads())
        assert_close(oracle, run_linear(gpu, h, x, M, N, hb), ref, F32_RTOL, f"{name} M={M} f32")
        x16 = _x(M, K, M * 31 + K + 1, f16=True)
        ref = oracle.gemm_nt_ref(x16.astype(np.float32), W, M, N, K, None, threads=oracle.max_threads())
        got = run_linear(gpu, h, x16, M, N, None, act="f16", out="f16")
        assert_close(oracle, got, ref, F16_RTOL, f"{name} M={M} f16 in/out")
    finally:
        gpu.plan_override(0, 0)


test_small_batch_all_shapes.cache = {}
test_small_batch_all_shapes.wcache = {}


@pytest.mark.parametrize("K,N,S", [(896, 128, 2), (896, 128, 7), (896, 896, 4), (4864, 896, 8), (4864, 896, 38), (896, 4864, 3)])
def test_split_k_is_deterministic_and_adds_bias_once(gpu, oracle, K, N, S):
    """Forced split counts (the reference tests S in {3, 4, 8}, src/tests/kernels.ts:1378-1400): the sum of the
    slices plus the bias, added once at the reduce (gemm_gemv_split_reduce.wgsl:36-38), bitwise repeatable."""
    t = synthetic.random_gptq(K, N, 128, seed=S, zeros="any")
    h = register(gpu, f"split{K}x{N}s{S}", t)
    hb = gpu.f32_upload(f"splitb{K}x{N}s{S}", np.full(N, 1000.0, np.float32))
    W = oracle_weight(oracle, t)
    x = _x(1, K, S)
    gpu.plan_override(_lib.WB_KERNEL_GEMV_MMA, S)
    try:
        assert gpu.plan(h, 1)["split_k"] == min(S, -(-K // 128))
        ref = oracle.gemm_nt_ref(x, W, 1, N, K, np.full(N, 1000.0, np.float32))
        a = run_linear(gpu, h, x, 1, N, hb)
        assert_close(oracle, a - 1000.0, ref - 1000.0, 2e-4, "split with bias")  # 1000 costs f32 ulps
        outs = [run_linear(gpu, h, x, 1, N, None) for _ in range(3)]
        assert all(np.array_equal(o.view(np.uint32), outs[0].view(np.uint32)) for o in outs)
        assert_close(oracle, outs[0], oracle.gemm_nt_ref(x, W, 1, N, K), F32_RTOL, "split no bias")
        x3 = _x(3, K, S + 1)
        assert_close(oracle, run_linear(gpu, h, x3, 3, N, None), oracle.gemm_nt_ref(x3, W, 3, N, K), F32_RTOL, "split M=3")
    finally:
        gpu.plan_override(0, 0)


def test_planner_never_splits_when_columns_fill_the_gpu(gpu):
    t = synthetic.random_gptq(896, 151936 // 8, 128, seed=9)
    h = register(gpu, "wide", t)
    p = gpu.plan(h, 1)
    assert p["split_k"] == 1 and p["launches"] == 1 and p["scratch_bytes"] == 0


@pytest.mark.parametrize("M,N,K,group", [(1, 53, 42, 8), (1, 5, 16, 8), (3, 53, 40, 8), (37, 53, 41, 8), (2, 12, 136, 32)])
def test_ragged_shapes_take_the_generic_kernel(gpu, oracle, M, N, K, group):
    """Odd sizes as in the reference's tests (N=53,K=42; M=37,N=53,K=41): K % 8, N % 4, small groups."""
    t = synthetic.random_gptq(K, N, group, seed=M + N + K, zeros="any")
    h = register(gpu, f"rag{M}_{N}_{K}", t)
    assert gpu.plan(h, M)["kernel_name"] == "generic"
    bias = np.random.default_rng(1).standard_normal(N).astype(np.float32)
    hb = gpu.f32_upload(f"ragb{M}_{N}_{K}", bias)
    W = oracle_weight(oracle, t)
    x = _x(M, K, 3)
    got = run_linear(gpu, h, x, M, N, hb, exact=True)
    assert_close(oracle, got, oracle.gemm_nt_ref(x, W, M, N, K, bias), 1e-6, "generic exact")
    if M > 1:
        # default mode rounds f32 activations to fp16 for M > 1, like gemm_nt_f16_from_f32.wgsl:58-62
        got = run_linear(gpu, h, x, M, N, hb)
        assert_close(oracle, got, oracle.gemm_nt_ref(oracle.round_f16(x), W, M, N, K, bias), 1e-6, "generic rounded A")


def test_reference_seeded_gemv_cases_with_dense_f16_weights(gpu, oracle, golden):
    """testGemmGemvF16 / testGemmGemvSplitF16 / testGemmNtF16 (src/tests/kernels.ts:1261-1269, 1378-1400,
    545-585): the reference's seeds and its own tolerance (atol 1e-5, rtol 1e-4; 5e-3 for the f16 GEMM),
    with the dense fp16 weight the reference uploads."""
    for i, c in enumerate(golden["gemv_cases"]):
        M, N, K = c["M"], c["N"], c["K"]
        rng = oracle.Rng(c["seed"])
        A = rng.random_f32(M * K)
        B = oracle.round_f16(rng.random_f32(N * K))
        bias = rng.random_f32(N)
        if c["round_a"]:
            A = oracle.round_f16(A)
        h = gpu.f16_alloc(f"ref_dense_{i}", N, K)
        gpu.f16_write_chunk(h, 0, B)
        hb = gpu.f32_upload(f"ref_bias_{i}", bias)
        rtol = 5e-3 if c["kind"] == "gemm_nt_f16" else 1e-4
        for b, key in ((hb, "want_bias_bits"), (None, "want_nobias_bits")):
            got = run_linear(gpu, h, A, M, N, b, exact=True)
            want = np.array(c[key], np.uint32).view(np.float32).reshape(M, N)
            r = oracle.check_tolerance(got, want, 1e-5, rtol)
            assert r.ok, (c["kind"], N, K, r)


@pytest.mark.parametrize("M", [1, 2, 5, 8])
def test_dense_f16_gemv_lm_head_shape(gpu, oracle, M):
    """Tied lm_head: fp16 [V, 896]; V trimmed to keep the CPU side quick, with a ragged tail of rows."""
    V, K = 151936 // 16 + 3, 896
    try:
        h = gpu.weight("lm_head_small")
    except WebllmError:
        rng = np.random.default_rng(4)
        test_dense_f16_gemv_lm_head_shape.W = rng.normal(0, 0.02, size=(V, K)).astype(np.float16)
        h = gpu.f16_alloc("lm_head_small", V, K)
        gpu.f16_write_bits(h, 0, test_dense_f16_gemv_lm_head_shape.W)
    W = test_dense_f16_gemv_lm_head_shape.W.astype(np.float32)
    assert gpu.plan(h, M)["kernel_name"] == "dense_gemv"
    x = _x(M, K, M)
    ref = oracle.gemm_nt_ref(x, W, M, V, K, threads=oracle.max_threads())
    assert_close(oracle, run_linear(gpu, h, x, M, V), ref, F32_RTOL, "dense f32")
    x16 = _x(M, K, M + 9, f16=True)
    ref = oracle.gemm_nt_ref(x16.astype(np.float32), W, M, V, K, threads=oracle.max_threads())
    assert_close(oracle, run_linear(gpu, h, x16, M, V, act="f16"), ref, F32_RTOL, "dense f16 in")


def test_argument_errors(gpu):
    t = synthetic.random_gptq(128, 8, 128, seed=1)
    h = register(gpu, "argerr", t)
    gpu.arena.reset()
    A = gpu.arena.alloc(128)
    Cc = gpu.arena.alloc(8)
    with pytest.raises(WebllmError, match="M must be positive"):
        gpu.linear(h, A, Cc, None, 0)
    hb = gpu.f32_upload("argerr_bias", np.zeros(9, np.float32))
    with pytest.raises(WebllmError, match="bias"):
        gpu.linear(h, A, Cc, hb, 1)
    from webllm_b200 import Tensor
    with pytest.raises(WebllmError, match="outside arena"):
        gpu.linear(h, Tensor(gpu.arena.capacity - 256, 128), Cc, None, 1)
    with pytest.raises(WebllmError, match="缺少 f16 权重"):
        gpu.linear(hb, A, Cc, None, 1)


def test_hint_next_prefetches_without_changing_results(gpu, oracle):
    """wb_linear_hint_next only asks the L2 for a later call's weight: results are bitwise the same with it, the
    hint is consumed by one call, and a bad handle is refused."""
    from webllm_b200 import _lib
    a = synthetic.random_gptq(896, 1152, 128, seed=41, zeros="any")
    b = synthetic.random_gptq(896, 4864, 128, seed=42, zeros="any")
    ha, hb = register(gpu, "hint_a", a), register(gpu, "hint_b", b)
    x = np.random.default_rng(9).standard_normal((1, 896)).astype(np.float32)
    plain = [run_linear(gpu, ha, x, 1, 1152), run_linear(gpu, hb, x, 1, 4864)]
    gpu.hint_next(hb)
    hinted_a = run_linear(gpu, ha, x, 1, 1152)
    hinted_b = run_linear(gpu, hb, x, 1, 4864)  # no hint pending any more
    assert np.array_equal(hinted_a.view(np.uint32), plain[0].view(np.uint32))
    assert np.array_equal(hinted_b.view(np.uint32), plain[1].view(np.uint32))
    gpu.hint_next(None)
    with pytest.raises(_lib.WebllmError) as e:
        gpu.hint_next(10 ** 6)
    assert e.value.status == _lib.WB_ERR_NOT_FOUND


@pytest.mark.parametrize("K,N,S", [(2560, 640, 1), (3584, 2048, 1), (5120, 256, 2), (7680, 96, 3)])
@pytest.mark.parametrize("M", [1, 2, 3, 4])
@pytest.mark.parametrize("zeros", ["any", "none"])
def test_streaming_kernel_matches_oracle(gpu, oracle, K, N, S, M, zeros):
    """The streaming variant of the int4 GEMV (M <= 4, >= 20 whole chunks per K slice, N % 32 == 0), forced so that
    nothing else can take the call: both activation types against the oracle, bias once, split-K through the
    workspace, and bitwise agreement between repeated launches. The general kernel on the same shapes agrees."""
    t = synthetic.random_gptq(K, N, 128, seed=K + N + M, zeros=zeros)
    W = oracle_weight(oracle, t)
    h = register(gpu, f"stream_{K}x{N}_{M}_{zeros}", t)
    bias = np.random.default_rng(N + M).standard_normal(N).astype(np.float32)
    hb = gpu.f32_upload(f"streamb_{K}x{N}_{M}_{zeros}", bias)
    x = _x(M, K, 7 * M + K)
    gpu.plan_override(_lib.WB_KERNEL_GEMV_STREAM, S)
    try:
        p = gpu.plan(h, M, "f32")
        assert p["kernel_name"] == "gemv_stream" and p["split_k"] == S and p["block"] == 256
        ref = oracle.gemm_nt_ref(x, W, M, N, K, bias, threads=oracle.max_threads())
        got = run_linear(gpu, h, x, M, N, hb)
        assert_close(oracle, got, ref, F32_RTOL, f"stream K={K} N={N} M={M} S={S} f32")
        again = run_linear(gpu, h, x, M, N, hb)
        assert np.array_equal(got.view(np.uint32), again.view(np.uint32))
        x16 = x.astype(np.float16)
        ref16 = oracle.gemm_nt_ref(x16.astype(np.float32), W, M, N, K, bias, threads=oracle.max_threads())
        assert_close(oracle, run_linear(gpu, h, x16, M, N, hb, act="f16"), ref16, F16_RTOL, f"stream K={K} N={N} M={M} S={S} f16")
        # a forced kind means that kernel and no other: the general kernel on the same shape and split
        gpu.plan_override(_lib.WB_KERNEL_GEMV_MMA, S)
        assert gpu.plan(h, M, "f32")["kernel_name"] == "gemv_mma"
        assert_close(oracle, run_linear(gpu, h, x, M, N, hb), ref, F32_RTOL, f"general kernel K={K} N={N} M={M} S={S}")
    finally:
        gpu.plan_override(0, 0)


@pytest.mark.parametrize("K,N", [(3584, 18944), (3584, 37888)])
def test_7b_gate_up_decode_takes_the_streaming_kernel(gpu, oracle, K, N):
    """The 7B-class gate / up projection (3584 -> 18944) and gate|up as one matrix (3584 -> 37888), the shapes behind
    the GEMV bandwidth figures: the planner's own choice is the streaming kernel; M = 1 and M = 4, f32 activations
    (1e-5) and fp16 activations (1e-3), against the oracle on every output."""
    t = synthetic.random_gptq(K, N, 128, seed=N, zeros="any")
    W = oracle_weight(oracle, t)
    h = register(gpu, f"gate7b_{N}", t)
    try:
        for M in ((1, 4) if N == 18944 else (1,)):
            for act in ("f32", "f16"):
                p = gpu.plan(h, M, act)
                assert p["kernel_name"] == "gemv_stream", p
                x = _x(M, K, 11 * M + N, f16=(act == "f16"))
                ref = oracle.gemm_nt_ref(x.astype(np.float32), W, M, N, K, threads=oracle.max_threads())
                got = run_linear(gpu, h, x, M, N, None, act=act)
                assert_close(oracle, got, ref, F32_RTOL if act == "f32" else F16_RTOL, f"7B gate N={N} M={M} {act}")
    finally:
        gpu.weight_pop()  # 35 / 70 MB: hand the space back to the module's arena


def test_streaming_kernel_refuses_a_last_slice_without_a_chunk_per_warp(gpu, oracle):
    """K = 34176 is 267 chunks of 128: 14 slices of 20 leave a last slice of 7 chunks, fewer than the kernel's 8 warps.
    The streaming kernel refuses that split (the general kernel takes it); 13 slices (21 + ... + 15) run and match."""
    K, N = 34176, 64
    t = synthetic.random_gptq(K, N, 128, seed=77, zeros="any")
    W = oracle_weight(oracle, t)
    h = register(gpu, "stream_longk", t)
    x = _x(1, K, 3)
    ref = oracle.gemm_nt_ref(x, W, 1, N, K, threads=oracle.max_threads())
    try:
        gpu.plan_override(_lib.WB_KERNEL_GEMV_STREAM, 14)
        with pytest.raises(WebllmError) as e:
            gpu.plan(h, 1, "f32")
        assert e.value.status == _lib.WB_ERR_UNSUPPORTED
        gpu.plan_override(_lib.WB_KERNEL_GEMV_MMA, 14)
        assert_close(oracle, run_linear(gpu, h, x, 1, N), ref, F32_RTOL, "general kernel, 14 slices")
        gpu.plan_override(_lib.WB_KERNEL_GEMV_STREAM, 13)
        assert gpu.plan(h, 1, "f32")["kernel_name"] == "gemv_stream"
        assert_close(oracle, run_linear(gpu, h, x, 1, N), ref, F32_RTOL, "streaming kernel, 13 slices")
    finally:
        gpu.plan_override(0, 0)


_MERGE_TIMEOUT_CHILD = r"""
import numpy as np
from webllm_b200 import Gpu, _lib, synthetic
from webllm_b200._lib import WebllmError
g = Gpu(0, weight_bytes=256 << 20, act_bytes=64 << 20)
t = synthetic.random_gptq(4864, 896, 128, seed=5, zeros="any")
h = g.gptq_register("down", t.qweight, t.qzeros, t.scales, 4864, 896, 128, 4, None)
p = g.plan(h, 1)
assert p["kernel_name"] == "gemv_mma" and p["split_k"] > 1, p
def run(M):
    g.arena.reset()
    A = g.arena.alloc(M * 4864, [M, 4864], "f32")
    C = g.arena.alloc(M * 896, [M, 896], "f32")
    g.write(A, np.random.default_rng(M).standard_normal((M, 4864)).astype(np.float32))
    g.linear(h, A, C, None, M)
    return C
run(1)                      # K slices as a cluster; the first CTA waits for 4 bytes that nobody sends
try:
    g.synchronize()
    raise SystemExit("the wait did not run out")
except WebllmError as e:
    assert e.status == _lib.WB_ERR_TIMEOUT, e
g.synchronize()             # the status word was consumed
y = g.read(run(64)).astype(np.float32)   # another kernel on the same context still works
assert np.isfinite(y).all() and float(np.abs(y).max()) > 0
g.close()
print("merge-timeout-ok")
"""


def test_cluster_merge_wait_gives_up_instead_of_hanging(built_lib):
    """The first CTA of a split-K cluster waits on an mbarrier for the other slices' partial sums. With the test setting
    that arms the barrier for 4 bytes more than are sent the wait runs out after its poll limit, the kernel returns, the
    next synchronize reports WB_ERR_TIMEOUT and the context keeps working. (The setting is read once per process, so
    the case runs in a child process.)"""
    import os, subprocess, sys
    from pathlib import Path
    env = dict(os.environ, WEBLLM_B200_CLUSTER_ASYNC="2")
    r = subprocess.run([sys.executable, "-c", _MERGE_TIMEOUT_CHILD], env=env, cwd=str(Path(__file__).resolve().parent.parent),
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "merge-timeout-ok" in r.stdout, r.stdout + r.stderr
