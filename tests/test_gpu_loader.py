"""``load_qwen_weights``: a safetensors checkpoint image → device, compared with the same tensors uploaded
directly, and with the reference's checks on what it loads (src/tests/infer/qwen-infer.ts:35-57: dequantised
layer and embedding rows read back from the GPU must equal the CPU values bit for bit)."""
import numpy as np
import pytest

from webllm_b200 import Gpu, QwenGpt, load_qwen_weights, qwen_loader, synthetic
from webllm_b200 import safetensors as st

pytestmark = pytest.mark.gpu

CFG = synthetic.QwenShape(512, 3, 4, 2, 256, 384)


def _f16_round(a):
    return np.asarray(a, np.float32).astype(np.float16).astype(np.float32)


@pytest.fixture(scope="module")
def checkpoint():
    W = synthetic.random_qwen_gptq(CFG, seed=77)
    # the file stores norms and biases as F16: the direct upload must use the same rounded values
    W["final_norm"] = _f16_round(W["final_norm"])
    for L in W["layers"]:
        for k in ("input_norm", "post_norm", "q_bias", "k_bias", "v_bias"):
            L[k] = _f16_round(L[k])
    return W, st.build_safetensors(qwen_loader.qwen_checkpoint_tensors(W), metadata={"format": "pt"})


def _model(kv="f32"):
    gpu = Gpu(0, weight_bytes=64 << 20, act_bytes=64 << 20)
    return gpu, QwenGpt(gpu, CFG, max_t=64, kv_dtype=kv)


def test_loaded_model_equals_direct_upload(built_lib, oracle, checkpoint, tmp_path):
    W, image = checkpoint
    path = tmp_path / "model.safetensors"
    path.write_bytes(image)
    progress = []
    gpu_a, a = _model()
    res = load_qwen_weights(a, str(path), on_progress=lambda d, t, s: progress.append((d, t, s)), keep_layer=1,
                            keep_embed_rows=(5, 3))
    gpu_b, b = _model()
    b.upload_gptq_model(W, fuse=True)

    assert res.tensor_count == 2 + 12 * CFG.n_layer and res.file_bytes == len(image)
    assert res.gpu_bytes == a.weight_bytes == b.weight_bytes
    assert progress == [(i + 1, CFG.n_layer, f"layer {i + 1}/{CFG.n_layer}") for i in range(CFG.n_layer)]

    # what the reference checks after loading: kept layer and embedding rows, bit for bit
    L1 = W["layers"][1]
    for key, name in (("q", "qW"), ("k", "kW"), ("v", "vW"), ("o", "oW"), ("gate", "gateW"), ("up", "upW"), ("down", "downW")):
        t = L1[key]
        ref = oracle.dequantize_gptq_int4(t.qweight, t.qzeros, t.scales, t.in_features, t.out_features, t.group_size)
        assert np.array_equal(res.layer[name].view(np.uint32), ref.view(np.uint32)), name
    assert np.array_equal(res.layer["inputNorm"], L1["input_norm"]) and np.array_equal(res.layer["kB"], L1["k_bias"])
    assert np.array_equal(res.embed_rows, W["embed"][5:8].astype(np.float32))
    got = a.read_weight_f16_bytes("embed", 5 * CFG.n_embd, 3 * CFG.n_embd)
    assert np.array_equal(got.view(np.uint16).ravel(), W["embed"][5:8].view(np.uint16).ravel())

    # and the two models compute the same thing
    prompt = np.random.default_rng(3).integers(0, CFG.vocab_size, 20).astype(np.uint32)
    la = a.read_tensor(a.prefill(prompt, last_only=True))
    lb = b.read_tensor(b.prefill(prompt, last_only=True))
    assert np.array_equal(la.view(np.uint32), lb.view(np.uint32))
    ta = a.decode_greedy(int(np.argmax(la)), 8)
    tb = b.decode_greedy(int(np.argmax(lb)), 8)
    assert np.array_equal(ta, tb)
    a.close(), b.close(), gpu_a.close(), gpu_b.close()


def test_loader_refuses_a_checkpoint_of_another_shape(built_lib, checkpoint):
    _, image = checkpoint
    other = synthetic.QwenShape(512, 3, 4, 2, 256, 512)
    gpu = Gpu(0, weight_bytes=64 << 20, act_bytes=16 << 20)
    with pytest.raises(st.SafetensorsError, match=r"gate_proj.qweight shape=\[32,384\]，期望 \[32,512\]"):
        load_qwen_weights(QwenGpt(gpu, other, max_t=16), image)
    gpu.close()
    small_vocab = synthetic.QwenShape(256, 3, 4, 2, 256, 384)
    gpu = Gpu(0, weight_bytes=64 << 20, act_bytes=16 << 20)
    with pytest.raises(qwen_loader.QwenLoaderError, match=r"embed_tokens 形状 \[512,256\]，期望 \[256,256\]"):
        load_qwen_weights(QwenGpt(gpu, small_vocab, max_t=16), image)
    gpu.close()
