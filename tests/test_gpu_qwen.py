"""GPU parity: the Qwen2 forward / prefill / decode path against qwenForwardRef (oracle), through the C ABI.
Mirrors testQwenArch and testQwenKvCache (src/tests/qwen/qwen-arch.ts:78-210) and adds the GPTQ model."""
import numpy as np
import pytest

from webllm_b200 import Gpu, QwenGpt, SamplerOptions, WebllmError, generate_qwen, sample_token, synthetic

pytestmark = pytest.mark.gpu

TINY = synthetic.QwenShape(97, 2, 4, 2, 32, 53)  # TEST_CONFIG, src/tests/qwen/qwen-arch.ts:8-19


def _tiny_weights(oracle, cfg, seed):
    """randomQwenWeights (src/tests/qwen/qwen-arch.ts:36-77): same RNG, same draw order."""
    rng = oracle.Rng(seed)
    C, KV, I, V = cfg.n_embd, cfg.kv_dim, cfg.intermediate, cfg.vocab_size

    def mat(n):
        return oracle.round_f16(np.array([np.float32((rng() * 2 - 1) * 0.12) for _ in range(n)], np.float32))

    def norm(n):
        return oracle.round_f16(np.array([np.float32(1 + (rng() - 0.5) * 0.2) for _ in range(n)], np.float32))

    layers = []
    for _ in range(cfg.n_layer):
        L = {"inputNorm": norm(C)}
        L["qW"], L["qB"] = mat(C * C), mat(C)
        L["kW"], L["kB"] = mat(KV * C), mat(KV)
        L["vW"], L["vB"] = mat(KV * C), mat(KV)
        L["oW"] = mat(C * C)
        L["postNorm"] = norm(C)
        L["gateW"], L["upW"], L["downW"] = mat(I * C), mat(I * C), mat(C * I)
        layers.append(L)
    return {"embed": mat(V * C), "finalNorm": norm(C), "layers": layers}


def _oracle_weights(W):
    ren = {"inputNorm": "input_norm", "postNorm": "post_norm"}
    return {"embed": W["embed"], "final_norm": W["finalNorm"],
            "layers": [{ren.get(k, k): v for k, v in L.items()} for L in W["layers"]]}


def _ocfg(oracle, cfg):
    return oracle.QwenConfig(cfg.vocab_size, cfg.n_layer, cfg.n_head, cfg.n_kv_head, cfg.n_embd, cfg.intermediate,
                             cfg.rms_eps, cfg.rope_theta)


@pytest.fixture(scope="module")
def tiny(built_lib, oracle):
    gpu = Gpu(0, weight_bytes=64 << 20, act_bytes=64 << 20)
    W = _tiny_weights(oracle, TINY, 20241006)
    model = QwenGpt(gpu, TINY, max_t=16)
    model.upload_weights(W)
    yield gpu, model, W
    model.close()
    gpu.close()


def test_qwen_arch_forward_matches_reference(tiny, oracle):
    """testQwenArch: B=2, T=6, tokens from makeRng(0xbeef); atol 2e-3, rtol 2e-2 and identical per-row argmax."""
    gpu, model, W = tiny
    rng = oracle.Rng(0xBEEF)
    B, T = 2, 6
    tokens = np.array([int(rng() * TINY.vocab_size) for _ in range(B * T)], np.uint32)
    ref = oracle.qwen_forward_ref(_ocfg(oracle, TINY), _oracle_weights(W), tokens, B, T)
    for exact, atol, rtol in ((False, 2e-3, 2e-2), (True, 2e-5, 2e-4)):
        model.set_exact(exact)
        got = model.read_tensor(model.forward(tokens, B, T)).reshape(B * T, -1)
        r = oracle.check_tolerance(got, ref, atol, rtol)
        assert r.ok, (exact, r)
        assert np.array_equal(got.argmax(axis=1), ref.argmax(axis=1))
    model.set_exact(False)
    with pytest.raises(WebllmError, match="tokens 长度"):
        model.forward(tokens[:5], B, T)


def test_qwen_kv_cache_matches_uncached_forward(tiny, oracle):
    """testQwenKvCache: prefill(4) + 2 decode steps reproduce rows 3, 4, 5 of the uncached forward; decode
    before prefill, a second prefill and an over-long context are rejected."""
    gpu, model, W = tiny
    rng = oracle.Rng(0xBEEF)
    T = 6
    seq = np.array([int(rng() * TINY.vocab_size) for _ in range(T)], np.uint32)
    full = model.read_tensor(model.forward(seq, 1, T)).reshape(T, -1)
    ref = oracle.qwen_forward_ref(_ocfg(oracle, TINY), _oracle_weights(W), seq, 1, T)
    model.reset_cache()
    with pytest.raises(WebllmError, match="decodeStep 前请先调用 prefill"):
        model.decode_step(1)
    pre = model.read_tensor(model.prefill(seq[:4])).reshape(4, -1)
    assert oracle.check_tolerance(pre, full[:4], 1e-4, 1e-3).ok          # the reference's prefill bar
    assert model.cache_len == 4
    with pytest.raises(WebllmError, match="prefill 前请先 resetCache"):
        model.prefill(seq[:2])
    for t in (4, 5):
        row = model.read_tensor(model.decode_step(int(seq[t])))
        assert oracle.check_tolerance(row, full[t], 2e-3, 2e-2).ok       # the reference's decode bar
        assert oracle.check_tolerance(row, ref[t], 2e-3, 2e-2).ok
        assert int(row.argmax()) == int(ref[t].argmax())
    assert model.cache_len == 6
    model.reset_cache()
    model.prefill(np.zeros(16, np.uint32), last_only=True)
    with pytest.raises(WebllmError, match="超过 blockSize=16"):
        model.decode_step(0)
    model.reset_cache()
    with pytest.raises(WebllmError, match="超过 blockSize=16"):
        model.prefill(np.zeros(17, np.uint32))
    with pytest.raises(WebllmError, match="outside the vocabulary"):
        model.prefill(np.array([97], np.uint32))


SMALL = synthetic.QwenShape(512, 3, 4, 2, 256, 384)  # head_dim 64, two groups of 128 along C, three along I


def _dense_from_gptq(oracle, G):
    def w(t):
        return oracle.dequantize_gptq_int4(t.qweight, t.qzeros, oracle.f16_bits_to_f32(t.scales.view(np.uint16)),
                                           t.in_features, t.out_features, t.group_size)
    layers = [{"input_norm": L["input_norm"], "post_norm": L["post_norm"], "qW": w(L["q"]), "qB": L["q_bias"],
               "kW": w(L["k"]), "kB": L["k_bias"], "vW": w(L["v"]), "vB": L["v_bias"], "oW": w(L["o"]),
               "gateW": w(L["gate"]), "upW": w(L["up"]), "downW": w(L["down"])} for L in G["layers"]]
    return {"embed": G["embed"].astype(np.float32), "final_norm": G["final_norm"], "layers": layers}


@pytest.mark.parametrize("fuse", [True, False])
@pytest.mark.parametrize("kv", ["f32", "f16"])
def test_gptq_model_prefill_decode_and_greedy(built_lib, oracle, fuse, kv):
    """A small GPTQ model: prefill logits, eager decode steps and the on-device greedy loop against the
    oracle on the dequantised weights (fp32-activation mode), with fused and separate projections and
    both cache types (the oracle rounds its cache to fp16 too)."""
    G = synthetic.random_qwen_gptq(SMALL, seed=3, std=0.05)
    Wd = _dense_from_gptq(oracle, G)
    prompt = np.random.default_rng(1).integers(0, SMALL.vocab_size, 40).astype(np.uint32)
    steps = 24
    with Gpu(0, weight_bytes=64 << 20, act_bytes=128 << 20) as gpu:
        model = QwenGpt(gpu, SMALL, max_t=80, kv_dtype=kv)
        model.upload_gptq_model(G, fuse=fuse)
        model.set_exact(True)
        ref = oracle.CachedForward(_ocfg(oracle, SMALL), Wd, max_t=80, kv_f16=(kv == "f16"), threads=oracle.max_threads())
        ref_row = ref.prefill(prompt)
        row = model.read_tensor(model.prefill(prompt, last_only=True))
        rms = float(np.sqrt(np.mean(ref_row.astype(np.float64) ** 2)))
        assert oracle.check_tolerance(row, ref_row, 2e-4 * rms, 2e-4).ok
        tok = oracle.sample_greedy(ref_row)
        assert int(row.argmax()) == tok
        # reference greedy trajectory
        want, t = [], tok
        for _ in range(steps):
            lr = ref.decode_step(t)
            t = oracle.sample_greedy(lr)
            want.append(t)
        got = model.decode_greedy(tok, steps - 5).tolist()
        got += model.decode_greedy(got[-1], 5).tolist()  # a second call continues from the device-resident state
        assert got == want
        assert model.cache_len == 40 + steps
        assert oracle.check_tolerance(model.last_logits(), lr, 5e-4 * rms, 5e-4).ok
        # the reference's host loop (generateQwen) gives the same ids as the device loop
        res_dev = generate_qwen(model, SMALL, prompt.tolist(), steps + 1, SamplerOptions(temperature=0))
        res_host = generate_qwen(model, SMALL, prompt.tolist(), steps + 1, SamplerOptions(temperature=0), on_device=False)
        assert res_dev.ids == res_host.ids == prompt.tolist() + [tok] + want
        assert res_dev.generated == steps + 1 and res_dev.prompt_length == 40
        # default mode (prefill rounds activations to fp16 like the reference's tiled GEMM) stays within its bar
        model.set_exact(False)
        model.reset_cache()
        row = model.read_tensor(model.prefill(prompt, last_only=True))
        assert oracle.check_tolerance(row, ref_row, 2e-2 * rms, 2e-2).ok
        model.close()


def test_sampler_matches_reference_rules():
    logits = np.array([0.1, 2.0, 2.0, -1.0], np.float32)
    assert sample_token(logits, 0, 4, SamplerOptions(temperature=0)) == 1        # first strict maximum
    assert sample_token(logits, 1, 3, SamplerOptions(temperature=0)) == 0
    picks = [sample_token(logits, 0, 4, SamplerOptions(temperature=1.0, top_k=2, rng=lambda v=v: v)) for v in (0.0, 0.49, 0.51, 0.99)]
    assert picks == [1, 1, 2, 2]
    assert sample_token(logits, 0, 4, SamplerOptions(temperature=1.0, top_p=0.3, rng=lambda: 0.9)) == 1
    with pytest.raises(ValueError, match="logits 越界"):
        sample_token(logits, 2, 4)


def test_full_size_decode_token_identical(built_lib, oracle):
    """One Qwen2.5-0.5B-shaped model with RTN-quantised N(0, 0.02) weights: 512-token random prompt, then
    128 greedy tokens with an fp16 KV cache, compared token by token with the oracle (fp32-activation mode
    on the GPU; the oracle rounds its cache to fp16 as well)."""
    cfg = synthetic.QWEN25_05B
    G = synthetic.random_qwen_gptq(cfg, seed=0)
    Wd = _dense_from_gptq(oracle, G)
    prompt = np.random.default_rng(0).integers(0, cfg.vocab_size, 512).astype(np.uint32)
    steps = 128
    ref = oracle.CachedForward(_ocfg(oracle, cfg), Wd, max_t=640, kv_f16=True, threads=oracle.max_threads())
    ref_row = ref.prefill(prompt)
    tok = oracle.sample_greedy(ref_row)
    want, margins, t = [], [], tok
    for _ in range(steps - 1):
        lr = ref.decode_step(t)
        t = oracle.sample_greedy(lr)
        top2 = np.partition(lr, -2)[-2:]
        margins.append(float(top2[1] - top2[0]))
        want.append(t)
    with Gpu(0, weight_bytes=1 << 30, act_bytes=256 << 20) as gpu:
        model = QwenGpt(gpu, cfg, max_t=640, kv_dtype="f16")
        model.upload_gptq_model(G, fuse=True)
        model.set_exact(True)
        row = model.read_tensor(model.prefill(prompt, last_only=True))
        rms = float(np.sqrt(np.mean(ref_row.astype(np.float64) ** 2)))
        r = oracle.check_tolerance(row, ref_row, 1e-3 * rms, 1e-3)
        assert r.ok, r
        assert int(row.argmax()) == tok
        got = model.decode_greedy(tok, steps - 1).tolist()
        first_diff = next((i for i, (a, b) in enumerate(zip(got, want)) if a != b), None)
        assert first_diff is None, (f"diverged at step {first_diff}: top-2 margin there {margins[first_diff]:.3e} "
                                    f"(logit rms {rms:.3e})")
        model.close()


@pytest.mark.parametrize("kv", ["f16", "f32"])
@pytest.mark.parametrize("n_prompt", [16, 150, 257])
def test_tensor_core_prefill_attention_every_row(built_lib, oracle, kv, n_prompt):
    """Prefill in the default mode runs the causal attention on the tensor cores (head size 64): the logits of EVERY
    row against qwenForwardRef, so that a wrong mask or a key block skipped too early shows up on the row it hits;
    token counts that end inside a 64-row block and cross several 64-key blocks; both cache types. The bar is that of
    the default mode (fp16 operands in every linear and in the attention: 1e-2 of the logits' rms, rtol 2e-2, and no
    row's rms error above 1e-2); the fp32-activation mode on the same prompt keeps the scalar kernel and its tighter bar."""
    G = synthetic.random_qwen_gptq(SMALL, seed=7, std=0.05)
    Wd = _dense_from_gptq(oracle, G)
    prompt = np.random.default_rng(n_prompt).integers(0, SMALL.vocab_size, n_prompt).astype(np.uint32)
    ref = oracle.qwen_forward_ref(_ocfg(oracle, SMALL), Wd, prompt, 1, n_prompt, threads=oracle.max_threads())
    rms = float(np.sqrt(np.mean(ref.astype(np.float64) ** 2)))
    with Gpu(0, weight_bytes=64 << 20, act_bytes=128 << 20) as gpu:
        model = QwenGpt(gpu, SMALL, max_t=n_prompt, kv_dtype=kv)
        model.upload_gptq_model(G, fuse=True)
        got = model.read_tensor(model.prefill(prompt)).reshape(n_prompt, -1)
        row_err = np.sqrt(np.mean((got - ref).astype(np.float64) ** 2, axis=1)) / rms
        r = oracle.check_tolerance(got, ref, 1e-2 * rms, 2e-2)
        assert r.ok, (kv, n_prompt, r, rms, float(row_err.max()), int(row_err.argmax()))
        assert row_err.max() < 1e-2, (float(row_err.max()), int(row_err.argmax()))  # no single row stands out: the mask is per row
        if kv == "f32":  # (an fp16 cache rounds k and v, which the uncached reference forward does not)
            model.set_exact(True)
            model.reset_cache()
            got = model.read_tensor(model.prefill(prompt)).reshape(n_prompt, -1)
            assert oracle.check_tolerance(got, ref, 2e-4 * rms, 2e-4).ok
        model.close()
