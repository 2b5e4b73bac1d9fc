"""CPU tests: the C oracle against the reference's formula-defined vectors (tests/golden) and against
independent numpy float64 evaluations of the defining formulas. No GPU needed."""
import numpy as np
import pytest

from conftest import bits_to_f32


def test_dequant_known_answer(oracle, golden):
    """src/tests/qwen/weights.ts:62-137: closed-form GPTQ known-answer test, with and without qzeros."""
    kat = golden["weights_kat"]
    qw = np.array(kat["qweight_u32"], np.uint32)
    qz = np.array(kat["qzeros_u32"], np.uint32)
    sc = bits_to_f32(kat["scales_f32_bits"])
    want = bits_to_f32(kat["want_f32_bits"]).reshape(kat["out"], kat["in"])
    got = oracle.dequantize_gptq_int4(qw, qz, sc, kat["in"], kat["out"], kat["group"])
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    r = oracle.check_tolerance(got, want, 1e-6, 1e-6)  # the reference's own criterion
    assert r.ok and r.max_abs == 0
    sym = oracle.dequantize_gptq_int4(qw, None, sc, kat["in"], kat["out"], kat["group"])
    assert np.array_equal(sym.view(np.uint32), want.view(np.uint32))


def test_dequant_zero_plus_one_does_not_wrap(oracle):
    """Stored nibble 15 means zero point 16 (src/weights/quant.ts:99), not 0."""
    qw = np.array([[0x76543210]], np.uint32)
    qz = np.array([[0x0000000F]], np.uint32)
    sc = np.array([[0.5]], np.float32)
    got = oracle.dequantize_gptq_int4(qw, qz, sc, 8, 1, 8)
    assert got.ravel().tolist() == [(q - 16) * 0.5 for q in range(8)]


def test_dequant_ragged(oracle):
    """in/out that are not multiples of 8 (src/weights/quant.ts:54-55,110)."""
    rng = np.random.default_rng(3)
    K, N, g = 21, 11, 8
    rows, zc, G = 3, 2, 3
    qw = rng.integers(0, 2**32, size=(rows, N), dtype=np.uint64).astype(np.uint32)
    qz = rng.integers(0, 2**32, size=(G, zc), dtype=np.uint64).astype(np.uint32)
    sc = rng.random((G, N)).astype(np.float32)
    got = oracle.dequantize_gptq_int4(qw, qz, sc, K, N, g)
    for n in range(N):
        for k in range(K):
            q = (int(qw[k // 8, n]) >> (4 * (k % 8))) & 15
            z = ((int(qz[k // g, n // 8]) >> (4 * (n % 8))) & 15) + 1
            assert got[n, k] == np.float32((q - z) * float(sc[k // g, n]))


@pytest.mark.parametrize("kw,msg", [
    (dict(bits=8), "当前仅支持 4bit"),
    (dict(group_size=0), "groupSize 必须为正"),
    (dict(in_features=0), "in/out 必须为正"),
    (dict(group_size=12), "必须是 packFactor=8 的整数倍"),
    (dict(short="qweight"), "qweight 字节不足"),
    (dict(short="scales"), "scales 数量不足"),
    (dict(short="qzeros"), "qzeros 字节不足"),
])
def test_dequant_validation(oracle, kw, msg):
    """The validation list of src/weights/quant.ts:46-79, with the reference's message texts."""
    K, N, g = 16, 8, 8
    qw, qz, sc = np.zeros((2, N), np.uint32), np.zeros((2, 1), np.uint32), np.ones((2, N), np.float32)
    short = kw.pop("short", None)
    if short == "qweight":
        qw = qw[:1]
    if short == "scales":
        sc = sc[:1]
    if short == "qzeros":
        qz = qz[:1]
    args = dict(in_features=K, out_features=N, group_size=g, bits=4)
    args.update(kw)
    with pytest.raises(oracle.OracleError, match=msg):
        oracle.dequantize_gptq_int4(qw, qz, sc, **args)


def test_f16_table(oracle, golden):
    """Hand-written f32 -> fp16 vectors for f32ToF16Bits (src/gpu/buffer.ts:57-100)."""
    f32 = np.array([b for b, _ in golden["f16_table"]], np.uint32).view(np.float32)
    want = np.array([h for _, h in golden["f16_table"]], np.uint16)
    assert oracle.f32_to_f16_bits(f32).tolist() == want.tolist()


def test_f16_decode_exhaustive(oracle):
    """f16BitsToF32 (src/weights/safetensors.ts:144-152) over all 65536 patterns vs IEEE binary16."""
    bits = np.arange(65536, dtype=np.uint32).astype(np.uint16)
    got = oracle.f16_bits_to_f32(bits)
    want = bits.view(np.float16).astype(np.float32)
    nan = np.isnan(want)
    assert np.array_equal(np.isnan(got), nan)
    assert np.array_equal(got[~nan].view(np.uint32), want[~nan].view(np.uint32))


def test_f16_encode_sweep(oracle):
    """f32ToF16Bits equals IEEE round-to-nearest-even (numpy) except where the reference deviates:
    NaN -> 0x7e00 and |x| in [2^-25, 2^-24) -> signed zero."""
    rng = np.random.default_rng(7)
    bits = rng.integers(0, 2**32, size=400000, dtype=np.uint64).astype(np.uint32)
    # dense coverage of the fp16 range, where random exponents rarely land
    near = (rng.integers(0, 2**23, size=400000, dtype=np.uint64).astype(np.uint32)
            | (rng.integers(127 - 27, 127 + 17, size=400000, dtype=np.uint64).astype(np.uint32) << 23)
            | (rng.integers(0, 2, size=400000, dtype=np.uint64).astype(np.uint32) << 31))
    f = np.concatenate([bits, near]).view(np.float32)
    got = oracle.f32_to_f16_bits(f)
    with np.errstate(over="ignore"):
        want = f.astype(np.float16).view(np.uint16)
    nan = np.isnan(f)
    tiny = (np.abs(f) < 2.0**-24) & ~nan
    plain = ~nan & ~tiny
    assert np.array_equal(got[plain], want[plain])
    assert np.all(got[nan] == 0x7E00)
    assert np.array_equal(got[tiny], (f[tiny].view(np.uint32) >> 16).astype(np.uint16) & 0x8000)
    # round trip of every finite fp16 value is the identity
    allh = np.arange(65536, dtype=np.uint32).astype(np.uint16)
    fin = ~np.isnan(allh.view(np.float16))
    assert np.array_equal(oracle.f32_to_f16_bits(oracle.f16_bits_to_f32(allh[fin])), allh[fin])


def test_rng(oracle, golden):
    """makeRng (src/reference/cpu-ref.ts:57-67) against an independent pure-Python xorshift32."""
    for seed, vals in golden["rng"].items():
        r = oracle.Rng(int(seed))
        assert [repr(r()) for _ in range(len(vals))] == vals
    # seed 0 is replaced by 1
    assert oracle.Rng(0)() == oracle.Rng(1)()


def _case_inputs(oracle, c):
    rng = oracle.Rng(c["seed"])
    A = rng.random_f32(c["M"] * c["K"])
    B = oracle.round_f16(rng.random_f32(c["N"] * c["K"]))
    bias = rng.random_f32(c["N"])
    if c["round_a"]:
        A = oracle.round_f16(A)
    return A, B, bias


def test_gemm_nt_ref_seeded_cases(oracle, golden):
    """gemmNTRef on the inputs of the reference's GEMV / split-K / f16 GEMM tests
    (src/tests/kernels.ts:1261-1269, 1378-1400, 545-585) against float64 numpy results."""
    for c in golden["gemv_cases"]:
        A, B, bias = _case_inputs(oracle, c)
        assert A[:4].view(np.uint32).tolist() == c["a_head_bits"]
        assert B[:4].view(np.uint32).tolist() == c["b_head_bits"]
        got = oracle.gemm_nt_ref(A, B, c["M"], c["N"], c["K"], bias)
        want = bits_to_f32(c["want_bias_bits"]).reshape(c["M"], c["N"])
        # float64 BLAS may sum in another order than the k-ascending loop: allow 1 ulp of f32
        assert np.max(np.abs(got.view(np.int32).astype(np.int64) - want.view(np.int32).astype(np.int64))) <= 1
        got = oracle.gemm_nt_ref(A, B, c["M"], c["N"], c["K"], None)
        want = bits_to_f32(c["want_nobias_bits"]).reshape(c["M"], c["N"])
        assert np.max(np.abs(got.view(np.int32).astype(np.int64) - want.view(np.int32).astype(np.int64))) <= 1


def test_gemm_threads_do_not_change_results(oracle):
    rng = np.random.default_rng(0)
    A, W = rng.standard_normal((5, 64)).astype(np.float32), rng.standard_normal((33, 64)).astype(np.float32)
    a = oracle.gemm_nt_ref(A, W, 5, 33, 64, None, threads=1)
    b = oracle.gemm_nt_ref(A, W, 5, 33, 64, None, threads=4)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


def test_check_tolerance_and_greedy(oracle):
    r = oracle.check_tolerance(np.array([1.0, 2.0], np.float32), np.array([1.0, 2.1], np.float32), 1e-5, 1e-4)
    assert not r.ok and abs(r.max_abs - 0.1) < 1e-6
    assert oracle.check_tolerance(np.array([1.00001], np.float32), np.array([1.0], np.float32), 1e-5, 1e-4).ok
    # sampler.ts:30-36: first strict maximum wins
    assert oracle.sample_greedy(np.array([0.0, 3.0, 3.0, 1.0], np.float32)) == 1
    assert oracle.sample_greedy(np.array([9, 0, 5, 5, 7, 7], np.float32), offset=2, vocab=4) == 2


# ---- forward pieces against independent numpy float64 restatements of the formulas ------------------

def _np_rmsnorm(x, w, eps):
    x64 = x.astype(np.float64)
    return (x64 / np.sqrt((x64 * x64).mean(axis=1, keepdims=True) + eps) * w.astype(np.float64)).astype(np.float32)


def _np_rope(x, rows, H, D, T, base, off):
    x64 = x.reshape(rows, H, D).astype(np.float64)
    pos = (np.arange(rows) % T + off).astype(np.float64)
    inv = base ** (-(2.0 * np.arange(D // 2)) / D)
    ang = pos[:, None] * inv[None, :]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    x0, x1 = x64[..., : D // 2], x64[..., D // 2:]
    return np.concatenate([x0 * c - x1 * s, x0 * s + x1 * c], axis=-1).astype(np.float32).ravel()


def _np_attention(q, k, v, B, T, H, KV, D):
    q64 = q.reshape(B, T, H, D).astype(np.float64)
    k64 = k.reshape(B, T, KV, D).astype(np.float64)
    v64 = v.reshape(B, T, KV, D).astype(np.float64)
    out = np.zeros((B, T, H, D))
    for b in range(B):
        for h in range(H):
            kvh = h // (H // KV)
            sc = q64[b, :, h] @ k64[b, :, kvh].T / np.sqrt(D)
            sc = np.where(np.tril(np.ones((T, T), bool)), sc, -np.inf)
            p = np.exp(sc - sc.max(axis=1, keepdims=True))
            p /= p.sum(axis=1, keepdims=True)
            out[b, :, h] = p @ v64[b, :, kvh]
    return out.astype(np.float32).ravel()


def test_rmsnorm_rope_attention_silu(oracle):
    """Shapes and seeds of the reference's adjacent-op tests (src/tests/kernels.ts:195-233, 1012-1157);
    tolerance is the reference's assertClose (atol 1e-5 + rtol 1e-4)."""
    rng = oracle.Rng(33)
    x, w = rng.random_f32(5 * 64), rng.random_f32(64)
    assert oracle.check_tolerance(oracle.rmsnorm_ref(x, w, 5, 64, 1e-5), _np_rmsnorm(x.reshape(5, 64), w, 1e-5), 1e-6, 1e-6).ok
    rng = oracle.Rng(0xA1)
    x = rng.random_f32(2 * 5 * 3 * 8)
    for off in (0, 7):
        got = oracle.rope_half_ref(x, 10, 3, 8, 5, 1e6, off)
        assert oracle.check_tolerance(got, _np_rope(x, 10, 3, 8, 5, 1e6, off), 1e-6, 1e-6).ok
    rng = oracle.Rng(0xA2)
    q, k, v = rng.random_f32(2 * 5 * 4 * 8), rng.random_f32(2 * 5 * 2 * 8), rng.random_f32(2 * 5 * 2 * 8)
    got = oracle.attention_gqa_ref(q, k, v, 2, 5, 4, 2, 8)
    assert oracle.check_tolerance(got, _np_attention(q, k, v, 2, 5, 4, 2, 8), 1e-6, 1e-5).ok
    rng = oracle.Rng(0xA3)
    g, u = rng.random_f32(4096), rng.random_f32(4096)
    want = (g.astype(np.float64) / (1 + np.exp(-g.astype(np.float64))) * u.astype(np.float64)).astype(np.float32)
    assert oracle.check_tolerance(oracle.silu_mul_ref(g, u), want, 1e-7, 1e-6).ok


def _tiny_weights(oracle, cfg, seed):
    """randomQwenWeights of src/tests/qwen/qwen-arch.ts:36-77 (same RNG, same draw order)."""
    rng = oracle.Rng(seed)
    C, KV, I, V = cfg.n_embd, cfg.kv_dim, cfg.intermediate, cfg.vocab_size
    s = 0.12

    def mat(n):
        return oracle.round_f16(np.array([np.float32((rng() * 2 - 1) * s) for _ in range(n)], np.float32))

    def norm(n):
        return oracle.round_f16(np.array([np.float32(1 + (rng() - 0.5) * 0.2) for _ in range(n)], np.float32))

    layers = []
    for _ in range(cfg.n_layer):
        L = {}
        L["input_norm"] = norm(C)
        L["qW"], L["qB"] = mat(C * C), mat(C)
        L["kW"], L["kB"] = mat(KV * C), mat(KV)
        L["vW"], L["vB"] = mat(KV * C), mat(KV)
        L["oW"] = mat(C * C)
        L["post_norm"] = norm(C)
        L["gateW"], L["upW"], L["downW"] = mat(I * C), mat(I * C), mat(C * I)
        layers.append(L)
    return {"embed": mat(V * C), "final_norm": norm(C), "layers": layers}


def _np_forward(cfg, W, tokens, B, T):
    C, H, KVH, D, KV, I = cfg.n_embd, cfg.n_head, cfg.n_kv_head, cfg.head_dim, cfg.kv_dim, cfg.intermediate
    M = B * T
    f32 = np.float32

    def lin(x, w, n, k, b=None):
        y = x.astype(np.float64) @ w.reshape(n, k).astype(np.float64).T
        return (y + (0 if b is None else b.astype(np.float64))).astype(f32)

    x = W["embed"].reshape(-1, C)[tokens].astype(f32)
    for L in W["layers"]:
        n1 = _np_rmsnorm(x, L["input_norm"], cfg.rms_eps)
        q, k, v = lin(n1, L["qW"], C, C, L["qB"]), lin(n1, L["kW"], KV, C, L["kB"]), lin(n1, L["vW"], KV, C, L["vB"])
        qr = _np_rope(q.ravel(), M, H, D, T, cfg.rope_theta, 0)
        kr = _np_rope(k.ravel(), M, KVH, D, T, cfg.rope_theta, 0)
        att = _np_attention(qr, kr, v.ravel(), B, T, H, KVH, D).reshape(M, C)
        xa = (x + lin(att, L["oW"], C, C)).astype(f32)
        n2 = _np_rmsnorm(xa, L["post_norm"], cfg.rms_eps)
        g, u = lin(n2, L["gateW"], I, C), lin(n2, L["upW"], I, C)
        act = (g.astype(np.float64) / (1 + np.exp(-g.astype(np.float64))) * u).astype(f32)
        x = (xa + lin(act, L["downW"], C, I)).astype(f32)
    return lin(_np_rmsnorm(x, W["final_norm"], cfg.rms_eps), W["embed"], cfg.vocab_size, C)


def test_forward_ref_and_cache_equivalence(oracle):
    """qwenForwardRef on the reference's tiny config (src/tests/qwen/qwen-arch.ts:8-19: vocab 97, 2 layers,
    4/2 heads, C=32, odd intermediate 53; weights seed 20241006, tokens seed 0xbeef, B=2, T=6) against a
    numpy float64 forward; and prefill + decode with a KV cache equals the uncached forward
    (src/tests/qwen/qwen-arch.ts:139-210)."""
    cfg = oracle.QwenConfig(97, 2, 4, 2, 32, 53)
    W = _tiny_weights(oracle, cfg, 20241006)
    rng = oracle.Rng(0xBEEF)
    B, T = 2, 6
    tokens = np.array([int(rng() * cfg.vocab_size) for _ in range(B * T)], np.uint32)
    logits, layers = oracle.qwen_forward_ref(cfg, W, tokens, B, T, want_layers=True)
    want = _np_forward(cfg, W, tokens, B, T)
    assert oracle.check_tolerance(logits, want, 1e-5, 1e-4).ok
    assert np.array_equal(logits.argmax(axis=1), want.argmax(axis=1))
    assert len(layers) == 2 and layers[0].shape == (B * T, 32)

    seq = tokens[:T]
    full = oracle.qwen_forward_ref(cfg, W, seq, 1, T)
    cached = oracle.CachedForward(cfg, W, max_t=16)
    row = cached.prefill(seq[:4])
    assert np.array_equal(row.view(np.uint32), full[3].view(np.uint32))
    for t in (4, 5):
        row = cached.decode_step(int(seq[t]))
        assert np.array_equal(row.view(np.uint32), full[t].view(np.uint32))
    assert cached.cache_len == T
    # an fp16 cache only perturbs the result slightly
    c16 = oracle.CachedForward(cfg, W, max_t=16, kv_f16=True)
    c16.prefill(seq[:5])
    assert oracle.check_tolerance(c16.decode_step(int(seq[5])), full[5], 2e-3, 2e-2).ok
