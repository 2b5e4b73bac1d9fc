"""GPU parity: the tcgen05 / TMEM GEMM (int4 unpack in shared memory, and dense fp16 weights) against
gemmNTRef on the fp16 weights the reference keeps on the device, through the C ABI."""
import os
import subprocess
import sys

import numpy as np
import pytest

from helpers import assert_close, oracle_weight, register, run_linear
from webllm_b200 import WebllmError, _lib, synthetic

pytestmark = pytest.mark.gpu

F16_RTOL = 1e-3

_cache = {}


def _weight(gpu, oracle, name, K, N, zeros="any"):
    key = f"tc_{name}"
    if key not in _cache:
        t = synthetic.random_gptq(K, N, 128, seed=K * 3 + N, zeros=zeros)
        h = register(gpu, key, t)
        # the tensor-core path multiplies fp16 weights: f32ToF16Bits of the dequantised value
        _cache[key] = (h, oracle.round_f16(oracle_weight(oracle, t)).reshape(N, K))
    return _cache[key]


def _ref_rows(oracle, x16, W16, rows, bias=None):
    xs = x16[rows].astype(np.float32)
    return oracle.gemm_nt_ref(xs, W16, len(rows), W16.shape[0], W16.shape[1], bias, threads=oracle.max_threads())


@pytest.mark.parametrize("name,K,N", [("q", 896, 896), ("k", 896, 128), ("gate", 896, 4864), ("down", 4864, 896)])
@pytest.mark.parametrize("M", [9, 12, 16, 17, 32, 64, 100, 128, 300])
def test_gemm_tc_small_and_ragged_m(gpu, oracle, name, K, N, M):
    """Every tile height (16, 32, 64, 128, 256) incl. token counts that do not fill the tile."""
    h, W16 = _weight(gpu, oracle, name, K, N)
    bias = np.random.default_rng(N).standard_normal(N).astype(np.float32)
    try:
        hb = gpu.weight(f"tcb_{name}")
    except WebllmError:
        hb = gpu.f32_upload(f"tcb_{name}", bias)
    x16 = np.random.default_rng(M + K).standard_normal((M, K)).astype(np.float16)
    gpu.plan_override(_lib.WB_KERNEL_GEMM_TC, 0)
    try:
        p = gpu.plan(h, M, "f16")
        assert p["kernel_name"] == "gemm_tc" and p["tile_m"] >= min(M, 256) // 2
        got = run_linear(gpu, h, x16, M, N, hb, act="f16")
        ref = _ref_rows(oracle, x16, W16, list(range(M)), bias)
        assert_close(oracle, got, ref, F16_RTOL, f"{name} M={M}")
        gpu.synchronize()  # surfaces a device-side wait that gave up
    finally:
        gpu.plan_override(0, 0)


@pytest.mark.parametrize("name,K,N", [(n, k, nn) for n, (k, nn) in synthetic.QWEN05B_SHAPES.items() if n in ("q", "k", "gate", "down")])
def test_prefill_m2048(gpu, oracle, name, K, N):
    """Prefill size, M = 2048: the planner picks the tensor-core kernel; 96 sampled rows are checked
    against the oracle (a full 2048-row double-precision reference would take minutes on the host)."""
    h, W16 = _weight(gpu, oracle, name, K, N)
    M = 2048
    x16 = np.random.default_rng(7).standard_normal((M, K)).astype(np.float16)
    assert gpu.plan(h, M, "f16")["kernel_name"] in ("gemm_tc", "gemm_tc_pair")
    got = run_linear(gpu, h, x16, M, N, None, act="f16")
    rows = sorted(set(np.random.default_rng(1).integers(0, M, 94).tolist()) | {0, M - 1})
    assert_close(oracle, got[rows], _ref_rows(oracle, x16, W16, rows), F16_RTOL, f"{name} M=2048")
    # fp16 output: the f32 result rounded once
    got16 = run_linear(gpu, h, x16, M, N, None, act="f16", out="f16")
    assert np.array_equal(got16.astype(np.float16).view(np.uint16), got.astype(np.float16).view(np.uint16))
    # f32 activations are rounded to fp16 first, like gemm_nt_f16_from_f32.wgsl:58-62
    got32 = run_linear(gpu, h, x16.astype(np.float32) * np.float32(1.0002), M, N, None)
    x_r = (x16.astype(np.float32) * np.float32(1.0002)).astype(np.float16)
    assert_close(oracle, got32[rows], _ref_rows(oracle, x_r, W16, rows), F16_RTOL, f"{name} f32 activations")


@pytest.mark.parametrize("name,K,N", [("q", 896, 896), ("qkv", 896, 1152), ("gate", 896, 4864), ("down", 4864, 896)])
@pytest.mark.parametrize("M,split", [(128, 0), (300, 0), (1000, 0), (2048, 0), (520, 3)])
def test_gemm_pair_kernel(gpu, oracle, name, K, N, M, split):
    """The CTA-pair kernel (cta_group::2) forced: every token tile (128, 192, 256), token counts that leave the second
    CTA's half of the activation tile partly or wholly empty, column counts that leave the second CTA's weight half empty
    (896 = 3.5 x 256, 1152 = 4.5 x 256), work-item counts below and above the number of pairs, and K slices."""
    h, W16 = _weight(gpu, oracle, name, K, N)
    bias = np.random.default_rng(N).standard_normal(N).astype(np.float32)
    try:
        hb = gpu.weight(f"tcb_{name}")
    except WebllmError:
        hb = gpu.f32_upload(f"tcb_{name}", bias)
    x16 = np.random.default_rng(M + K).standard_normal((M, K)).astype(np.float16)
    gpu.plan_override(_lib.WB_KERNEL_GEMM_TC_PAIR, split)
    try:
        p = gpu.plan(h, M, "f16")
        assert p["kernel_name"] == "gemm_tc_pair" and p["tile_n"] == 256 and (split == 0 or p["split_k"] == split)
        got = run_linear(gpu, h, x16, M, N, hb, act="f16")
        gpu.synchronize()  # surfaces a device-side wait that gave up
        rows = sorted(set(np.random.default_rng(2).integers(0, M, 60).tolist()) | {0, M // 2 - 1, M // 2, M - 1})
        assert_close(oracle, got[rows], _ref_rows(oracle, x16, W16, rows, bias), F16_RTOL, f"pair {name} M={M}")
        got16 = run_linear(gpu, h, x16, M, N, hb, act="f16", out="f16")
        assert np.array_equal(got16.astype(np.float16).view(np.uint16), got.astype(np.float16).view(np.uint16))
    finally:
        gpu.plan_override(0, 0)


@pytest.mark.parametrize("M", [4096, 4000])
def test_gemm_pair_last_round_cut_along_k(gpu, oracle, M):
    """3584 -> 3584 at M ~ 4096 is 224 work items of 256 x 256 for 74 CTA pairs: three whole rounds and 2 items left over.
    The launch cuts those 2 along K (28 slices of 2 k-blocks, one per otherwise idle pair) and a second small launch adds
    the slices; the plan shows the extra launch and its scratch, and every column (the leftover items are the last 256
    columns of the last two token tiles) matches the oracle, with a bias, for f32 and fp16 results and with a ragged
    last token tile."""
    K = N = 3584
    h, W16 = _weight(gpu, oracle, "q7", K, N, zeros="7or8")
    bias = np.random.default_rng(N).standard_normal(N).astype(np.float32)
    try:
        hb = gpu.weight("tcb_q7")
    except WebllmError:
        hb = gpu.f32_upload("tcb_q7", bias)
    x16 = np.random.default_rng(M).standard_normal((M, K)).astype(np.float16)
    gpu.plan_override(_lib.WB_KERNEL_GEMM_TC_PAIR, 0)
    try:
        p = gpu.plan(h, M, "f16")
        assert p["kernel_name"] == "gemm_tc_pair" and p["split_k"] == 1
        if p["tile_m"] == 256:  # 148 SMs: 74 pairs, one partial tile each
            assert p["launches"] == 2 and p["scratch_bytes"] == 74 * 256 * 256 * 4
        got = run_linear(gpu, h, x16, M, N, hb, act="f16")
        gpu.synchronize()
        rows = sorted(set(np.random.default_rng(3).integers(0, M, 24).tolist()) | {0, 3583, 3584, 3839, 3840, M - 1})
        assert_close(oracle, got[rows], _ref_rows(oracle, x16, W16, rows, bias), F16_RTOL, f"pair tail M={M}")
        got16 = run_linear(gpu, h, x16, M, N, hb, act="f16", out="f16")
        assert np.array_equal(got16.astype(np.float16).view(np.uint16), got.astype(np.float16).view(np.uint16))
        again = run_linear(gpu, h, x16, M, N, hb, act="f16")
        assert np.array_equal(got.view(np.uint32), again.view(np.uint32))
    finally:
        gpu.plan_override(0, 0)


@pytest.mark.parametrize("group,zeros", [(64, "any"), (256, "any"), (128, "none"), (64, "sym")])
@pytest.mark.parametrize("kind", ["gemm_tc", "gemm_tc_pair"])
def test_gemm_group_sizes_and_zero_modes(gpu, oracle, kind, group, zeros):
    """Both tensor-core kernels with one and with four k-blocks per group, arbitrary zero points, and a checkpoint
    without a qzeros tensor (the symmetric default, stored 7); K = 1024, N = 640 (2.5 column tiles of the pair kernel),
    M = 300."""
    K, N, M = 1024, 640, 300
    t = synthetic.random_gptq(K, N, group, seed=group + len(zeros), zeros=zeros)
    name = f"tc_g{group}_{zeros}"
    try:
        h = gpu.weight(name)
    except WebllmError:
        h = register(gpu, name, t)
    W16 = oracle.round_f16(oracle_weight(oracle, t)).reshape(N, K)
    x16 = np.random.default_rng(group).standard_normal((M, K)).astype(np.float16)
    gpu.plan_override(_lib.WB_KERNEL_GEMM_TC if kind == "gemm_tc" else _lib.WB_KERNEL_GEMM_TC_PAIR, 0)
    try:
        assert gpu.plan(h, M, "f16")["kernel_name"] == kind
        got = run_linear(gpu, h, x16, M, N, None, act="f16")
        gpu.synchronize()
        assert_close(oracle, got, _ref_rows(oracle, x16, W16, list(range(M))), F16_RTOL, f"{kind} g={group} zeros={zeros}")
    finally:
        gpu.plan_override(0, 0)


def test_gemm_pair_kernel_refuses_what_it_cannot_do(gpu, oracle):
    h, _ = _weight(gpu, oracle, "k", 896, 128)
    gpu.plan_override(_lib.WB_KERNEL_GEMM_TC_PAIR, 0)
    try:
        with pytest.raises(WebllmError, match="GEMM_TC_PAIR"):
            gpu.plan(h, 512, "f16")  # N < 256
        hq, _ = _weight(gpu, oracle, "q", 896, 896)
        with pytest.raises(WebllmError, match="GEMM_TC_PAIR"):
            gpu.plan(hq, 64, "f16")  # M < 128
    finally:
        gpu.plan_override(0, 0)


def test_linearity_at_full_size(gpu, oracle):
    """Size-independent property at M = 2048 x (896 -> 4864): f(a) + f(b) == f(a + b) up to fp16/f32
    rounding, with a and b chosen so that a + b is exact in fp16."""
    h, _ = _weight(gpu, oracle, "gate", 896, 4864)
    rng = np.random.default_rng(3)
    a = (rng.integers(-64, 64, size=(2048, 896)) / 32).astype(np.float16)
    b = (rng.integers(-64, 64, size=(2048, 896)) / 32).astype(np.float16)
    fa = run_linear(gpu, h, a, 2048, 4864, None, act="f16")
    fb = run_linear(gpu, h, b, 2048, 4864, None, act="f16")
    fab = run_linear(gpu, h, (a + b).astype(np.float16), 2048, 4864, None, act="f16")
    assert_close(oracle, fa + fb, fab, 1e-4, "linearity")


def test_gemv_and_gemm_paths_agree(gpu, oracle):
    """The switch between the GEMV and the tensor-core kernel (forced both ways at M = 32) must not be visible beyond
    fp16-weight rounding."""
    h, _ = _weight(gpu, oracle, "gate", 896, 4864)
    x16 = np.random.default_rng(5).standard_normal((32, 896)).astype(np.float16)
    outs = {}
    for kind in (_lib.WB_KERNEL_GEMV_MMA, _lib.WB_KERNEL_GEMM_TC):
        gpu.plan_override(kind, 0)
        try:
            outs[kind] = run_linear(gpu, h, x16, 32, 4864, None, act="f16")
        finally:
            gpu.plan_override(0, 0)
    # the tensor-core path multiplies weights rounded to fp16 (2^-11), the streaming path exact ones
    assert_close(oracle, outs[_lib.WB_KERNEL_GEMM_TC], outs[_lib.WB_KERNEL_GEMV_MMA], 4e-3, "paths")
    # where the planner switches: after M = 8, except on short-K wide-N shapes like this one (12 with fp16, 16 with f32)
    assert gpu.plan(h, 12, "f16")["kernel_name"] == "gemv_mma" and gpu.plan(h, 13, "f16")["kernel_name"] == "gemm_tc"
    assert gpu.plan(h, 16, "f32")["kernel_name"] == "gemv_mma" and gpu.plan(h, 17, "f32")["kernel_name"] == "gemm_tc"
    assert gpu.plan(h, 33, "f16")["kernel_name"] == "gemm_tc"
    hq, _ = _weight(gpu, oracle, "q", 896, 896)
    for act in ("f16", "f32"):
        assert gpu.plan(hq, 8, act)["kernel_name"] == "gemv_mma" and gpu.plan(hq, 9, act)["kernel_name"] == "gemm_tc"
    assert gpu.plan(hq, 16, "f32", exact=True)["kernel_name"] == "gemv_mma"  # exact mode keeps f32 activations off the fp16 path


@pytest.mark.parametrize("name,K,N", [("q", 896, 896), ("down", 4864, 896), ("kv7", 3584, 512)])
@pytest.mark.parametrize("M", [9, 12, 16])
def test_small_batch_default_goes_to_the_tensor_cores(gpu, oracle, name, K, N, M):
    """9 <= M <= 16 with the planner's own choice (the tensor-core kernel on these shapes), fp16 and f32 activations
    (the latter rounded to fp16 first, as the reference's tiled GEMM stages them: gemm_nt_f16_from_f32.wgsl:58-62)."""
    h, W16 = _weight(gpu, oracle, name, K, N)
    x = np.random.default_rng(M * 7 + K).standard_normal((M, K)).astype(np.float32)
    x16 = x.astype(np.float16)
    ref = _ref_rows(oracle, x16, W16, list(range(M)))
    for act, xin in (("f16", x16), ("f32", x)):
        assert gpu.plan(h, M, act)["kernel_name"] == "gemm_tc"
        got = run_linear(gpu, h, xin, M, N, None, act=act, out=act)
        assert_close(oracle, got, ref, F16_RTOL, f"{name} M={M} {act}")
    gpu.synchronize()


@pytest.mark.parametrize("M", [9, 64, 200])
def test_dense_f16_gemm(gpu, oracle, M):
    """Dense fp16 weight (the tied lm_head at prefill): both operands arrive by TMA."""
    V, K = 1000, 896
    if "dense" not in _cache:
        W = np.random.default_rng(8).normal(0, 0.02, size=(V, K)).astype(np.float16)
        h = gpu.f16_alloc("tc_dense", V, K)
        gpu.f16_write_bits(h, 0, W)
        _cache["dense"] = (h, W.astype(np.float32))
    h, W = _cache["dense"]
    x16 = np.random.default_rng(M).standard_normal((M, K)).astype(np.float16)
    assert gpu.plan(h, M, "f16")["kernel_name"] == "gemm_tc"
    got = run_linear(gpu, h, x16, M, V, None, act="f16")
    assert_close(oracle, got, _ref_rows(oracle, x16, W, list(range(M))), F16_RTOL, f"dense M={M}")


def test_7b_shapes(gpu, oracle):
    """7B-class projections at prefill size, sampled rows against the oracle: q and k/v, the gate / up shape
    3584 -> 18944 at M = 4096 (the 256 x 256 tile) and down 18944 -> 3584 at M = 512 and M = 4096 (the long-K GEMM)."""
    for name, K, N, M in (("q7", 3584, 3584, 4096), ("kv7", 3584, 512, 4096), ("down7", 18944, 3584, 512),
                          ("gate7", 3584, 18944, 4096), ("down7", 18944, 3584, 4096)):
        h, W16 = _weight(gpu, oracle, name, K, N, zeros="7or8")
        x16 = np.random.default_rng(K).standard_normal((M, K)).astype(np.float16)
        got = run_linear(gpu, h, x16, M, N, None, act="f16")
        rows = sorted(set(np.random.default_rng(2).integers(0, M, 30).tolist()) | {0, M - 1})
        assert_close(oracle, got[rows], _ref_rows(oracle, x16, W16, rows), F16_RTOL, f"{name} M={M}")
    gpu.synchronize()


@pytest.mark.parametrize("M,act", [(48, "f16"), (128, "f32")])
def test_split_k_gemm_when_few_tiles(gpu, oracle, M, act):
    """K = 4864 -> N = 896 at a mid-size batch gives 7 tiles for 148 SMs: the planner cuts K into slices (f32 partial
    sums in the workspace, one reduce launch, bias added once), the result is the same as the reference's and
    repeats bit for bit; a forced single slice agrees with it to rounding."""
    h, W16 = _weight(gpu, oracle, "down", 4864, 896)
    bias = np.random.default_rng(896).standard_normal(896).astype(np.float32)
    try:
        hb = gpu.weight("tcb_down")
    except WebllmError:
        hb = gpu.f32_upload("tcb_down", bias)
    x16 = np.random.default_rng(M).standard_normal((M, 4864)).astype(np.float16)
    x = x16 if act == "f16" else x16.astype(np.float32)
    ref = _ref_rows(oracle, x16, W16, list(range(M)), bias)
    gpu.plan_override(_lib.WB_KERNEL_GEMM_TC, 0)
    try:
        p = gpu.plan(h, M, act)
        assert p["kernel_name"] == "gemm_tc" and p["split_k"] > 1 and p["grid_z"] == p["split_k"]
        assert p["launches"] == (2 if act == "f16" else 3)
        got = run_linear(gpu, h, x, M, 896, hb, act=act)
        assert_close(oracle, got, ref, F16_RTOL, f"split-K gemm M={M}")
        again = run_linear(gpu, h, x, M, 896, hb, act=act)
        assert np.array_equal(got.view(np.uint32), again.view(np.uint32))
        gpu.plan_override(_lib.WB_KERNEL_GEMM_TC, 1)
        assert gpu.plan(h, M, act)["split_k"] == 1
        one = run_linear(gpu, h, x, M, 896, hb, act=act)
        assert_close(oracle, one, got, F16_RTOL, "one slice vs split")  # both are rounded to the output type
        gpu.synchronize()
    finally:
        gpu.plan_override(0, 0)


def test_planner_picks_tile_and_slices_together(gpu, oracle):
    """The plan is self-consistent for either tile width, K is cut into slices where the tiles alone would leave
    SMs idle (down at M = 2048: 56 or 32 tiles for 148 SMs), and a long-K, many-tile shape takes 256 output columns
    per CTA (two accumulators sharing one activation tile)."""
    for name, K, N in (("gate", 896, 4864), ("down", 4864, 896)):
        h, _ = _weight(gpu, oracle, name, K, N)
        p = gpu.plan(h, 2048, "f16")
        assert p["tile_n"] in (128, 256) and p["tile_m"] in (128, 192, 256)
        assert p["grid_y"] == -(-N // p["tile_n"]) and p["grid_x"] == -(-2048 // p["tile_m"])
        assert (p["split_k"] > 1) == (name == "down") and p["grid_z"] == p["split_k"]
    if os.environ.get("WEBLLM_B200_GEMM_NH") is None and os.environ.get("WEBLLM_B200_GEMM_MT") is None:
        h, _ = _weight(gpu, oracle, "q7", 3584, 3584, zeros="7or8")
        p = gpu.plan(h, 4096, "f16")
        assert (p["tile_m"], p["tile_n"], p["split_k"]) == (256, 256, 1)


_FORCED = any(os.environ.get(v) is not None for v in ("WEBLLM_B200_GEMM_NH", "WEBLLM_B200_GEMM_MT", "WEBLLM_B200_GEMM_PERSIST"))


@pytest.mark.skipif(_FORCED, reason="already the forced run")
@pytest.mark.parametrize("var,value", [("WEBLLM_B200_GEMM_NH", "2"), ("WEBLLM_B200_GEMM_MT", "192"),
                                       ("WEBLLM_B200_GEMM_PERSIST", "0")])
def test_every_tile_shape_forced(var, value):
    """The tile switches are read once per process, so the ragged-M, dense and split-K cases above run again in child
    processes: once with the 256-column tile forced for every token count from 100 up (128 x 256 and 256 x 256), and
    once with the 192-token tile (the one the planner picks to fit the waves, 256 or 512 TMEM columns) forced for
    every token count, and once with the persistent tile loop switched off, so that the prefill sizes (more tiles than
    SMs), which otherwise take the persistent kernel, also go through the one-tile-per-CTA kernel."""
    env = dict(os.environ)
    env[var] = value
    r = subprocess.run([sys.executable, "-m", "pytest", __file__, "-q", "-x", "-k", "ragged or dense or split_k_gemm or 7b or m2048"],
                       env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
