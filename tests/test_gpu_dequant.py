"""GPU parity: GPTQ dequant export, bit-exact against the oracle, through the C ABI."""
import numpy as np
import pytest

from conftest import bits_to_f32
from helpers import oracle_weight, register
from webllm_b200 import GptqInt4Params, WebllmError, dequantize_gptq_int4, synthetic

pytestmark = pytest.mark.gpu


def _export(gpu, h, N, K, dtype):
    gpu.arena.reset()
    t = gpu.arena.alloc(N * K, [N, K], dtype)
    gpu.gptq_dequant(h, t)
    return gpu.read(t).reshape(N, K)


def test_known_answer_through_host_api(gpu, oracle, golden):
    """The reference's closed-form case (src/tests/qwen/weights.ts:62-137). Its scales are arbitrary f32;
    the checkpoint stores fp16, so they are rounded to fp16 first, on both sides."""
    kat = golden["weights_kat"]
    qw, qz = np.array(kat["qweight_u32"], np.uint32), np.array(kat["qzeros_u32"], np.uint32)
    sc = oracle.round_f16(bits_to_f32(kat["scales_f32_bits"]))
    for zeros in (qz, None):
        got = dequantize_gptq_int4(gpu, GptqInt4Params(qw, sc, kat["in"], kat["out"], zeros, kat["group"]))
        want = oracle.dequantize_gptq_int4(qw, zeros, sc, kat["in"], kat["out"], kat["group"])
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    assert gpu.arena.used_bytes == 0  # the call leaves no allocation behind


@pytest.mark.parametrize("K,N,group,zeros", [
    (896, 4864, 128, "7or8"),   # the single-linear benchmark case
    (896, 896, 128, "any"), (896, 128, 128, "any"), (4864, 896, 128, "any"),
    (3584, 512, 128, "sym"), (896, 128, 128, "none"),
    (21, 11, 8, "any"), (42, 53, 8, "any"), (100, 5, 32, "any"), (136, 24, 8, "none"),
])
def test_bit_exact_f32_and_f16(gpu, oracle, K, N, group, zeros):
    t = synthetic.random_gptq(K, N, group, seed=K * 7 + N, zeros=zeros)
    h = register(gpu, f"w{K}x{N}g{group}{zeros}", t)
    want = oracle_weight(oracle, t)
    got = _export(gpu, h, N, K, "f32")
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    got16 = _export(gpu, h, N, K, "f16")
    # the reference's device copy: f32ToF16Bits of the f32 weight (src/tests/infer/qwen-infer.ts:45-52)
    assert np.array_equal(got16.view(np.uint16), oracle.f32_to_f16_bits(want))


def test_real_file_invariants_on_synthetic_weights(gpu, oracle):
    """The structural checks the reference runs on the real checkpoint (src/tests/qwen/qwen-format.ts:82-167),
    restated on a synthetic symmetric layer: |w| <= 8 * max scale."""
    t = synthetic.random_gptq(896, 896, 128, seed=11, zeros="sym")
    got = _export(gpu, register(gpu, "sym896", t), 896, 896, "f32")
    assert np.max(np.abs(got)) <= 8 * float(t.scales.astype(np.float32).max())


def test_extreme_scales_keep_reference_rounding(gpu, oracle):
    """fp16 subnormal / huge scales: products that overflow fp16 become inf, tiny ones keep RNE."""
    K, N = 128, 8
    t = synthetic.random_gptq(K, N, 128, seed=2, zeros="any")
    t.scales = np.array([[6e-8, 1e-7, 3e-5, 6.1e-5, 1.0, 4096.0, 8192.0, 65504.0]], np.float16)
    h = register(gpu, "extreme", t)
    want = oracle_weight(oracle, t)
    assert np.array_equal(_export(gpu, h, N, K, "f32").view(np.uint32), want.view(np.uint32))
    assert np.array_equal(_export(gpu, h, N, K, "f16").view(np.uint16), oracle.f32_to_f16_bits(want))


@pytest.mark.parametrize("kw,msg", [
    (dict(bits=8), "当前仅支持 4bit"), (dict(group_size=0), "groupSize 必须为正"),
    (dict(in_features=0), "in/out 必须为正"), (dict(group_size=12), "必须是 packFactor=8 的整数倍"),
    (dict(short="qweight"), "qweight 字节不足"), (dict(short="scales"), "scales 数量不足"),
    (dict(short="qzeros"), "qzeros 字节不足"),
])
def test_validation_messages_match_reference(gpu, kw, msg):
    K, N, g = 16, 8, 8
    qw, qz, sc = np.zeros((2, N), np.uint32), np.zeros((2, 1), np.uint32), np.ones((2, N), np.float16)
    short = kw.pop("short", None)
    qw = qw[:1] if short == "qweight" else qw
    sc = sc[:1] if short == "scales" else sc
    qz = qz[:1] if short == "qzeros" else qz
    args = dict(in_features=K, out_features=N, group_size=g, bits=4)
    args.update(kw)
    with pytest.raises(WebllmError, match=msg):
        dequantize_gptq_int4(gpu, GptqInt4Params(qw, sc, qzeros=qz, **args))


def test_duplicate_and_missing_names(gpu):
    """"权重已存在" / "缺少 ... 权重" (src/model/qwen.ts:247-276, 620-646)."""
    t = synthetic.random_gptq(128, 8, 128, seed=1)
    register(gpu, "dup", t)
    with pytest.raises(WebllmError, match="权重已存在: dup"):
        register(gpu, "dup", t)
    with pytest.raises(WebllmError, match="缺少权重: nope"):
        gpu.weight("nope")


def test_f16_upload_matches_reference_conversion(gpu, oracle, golden):
    """writeF16 (src/gpu/buffer.ts:103-120): every vector of the hand-written table plus a random sweep."""
    table = np.array([b for b, _ in golden["f16_table"]], np.uint32).view(np.float32)
    rng = np.random.default_rng(5)
    rnd = rng.integers(0, 2**32, size=70000, dtype=np.uint64).astype(np.uint32).view(np.float32)
    small = (rng.standard_normal(30000) * 1e-6).astype(np.float32)
    data = np.concatenate([table, rnd, small])
    h = gpu.f16_alloc("f16conv", 1, data.size)
    gpu.f16_write_chunk(h, 0, data)
    got = gpu.read_weight_f16(h, 0, data.size)
    assert np.array_equal(got, oracle.f32_to_f16_bits(data))
    assert got[: len(table)].tolist() == [hh for _, hh in golden["f16_table"]]
    # chunked writes (writeF16Chunk) land at their element offset
    gpu.f16_write_chunk(h, 10, np.array([1.0, -0.5], np.float32))
    assert gpu.read_weight_f16(h, 10, 2).tolist() == [0x3C00, 0xB800]


def test_read_sweep_diagnostic_runs_and_checks_its_range(gpu):
    """wb_read_sweep (the bandwidth yardstick of `bench.py --case read`) launches one kernel over a slab range and refuses
    ranges outside the slab or not in 16-byte units; it never writes, so the slab is unchanged afterwards."""
    from webllm_b200 import _lib
    data = np.arange(1 << 16, dtype=np.float32)
    t = gpu.arena.alloc(data.size)
    gpu.write(t, data)
    before = gpu.launch_count
    gpu.read_sweep(t.offset, data.nbytes, 148, arena=_lib.WB_ARENA_ACT)
    gpu.synchronize()
    assert np.array_equal(gpu.read(t), data)
    assert gpu.launch_count == before + 1
    with pytest.raises(WebllmError):
        gpu.read_sweep(t.offset + 8, 1024, 148, arena=_lib.WB_ARENA_ACT)
    with pytest.raises(WebllmError, match="outside the slab"):
        gpu.read_sweep(0, 1 << 40, 148, arena=_lib.WB_ARENA_ACT)
