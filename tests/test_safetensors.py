"""The safetensors reader and the checkpoint loader's file handling (CPU; the upload half is in
test_gpu_loader.py). Known answers are the reference's own (src/tests/qwen/weights.ts:7-60)."""
import json

import numpy as np
import pytest

from webllm_b200 import qwen_loader, synthetic
from webllm_b200 import safetensors as st


def reference_test_file() -> bytes:
    """The file the reference's test builds by hand: F32 [1, -2, 0.5], F16 bits 0x3c00 0xb800, BF16 bits 0x3f80 0xc000."""
    tensors = [("bias", "F32", [3], np.array([1, -2, 0.5], np.float32).tobytes()),
               ("half", "F16", [2], bytes([0x00, 0x3C, 0x00, 0xB8])),
               ("bfloat", "BF16", [2], bytes([0x80, 0x3F, 0x00, 0xC0]))]
    header, off = {"__metadata__": {"format": "test"}}, 0
    for name, dtype, shape, data in tensors:
        header[name] = {"dtype": dtype, "shape": shape, "data_offsets": [off, off + len(data)]}
        off += len(data)
    hb = json.dumps(header).encode()
    return len(hb).to_bytes(4, "little") + bytes(4) + hb + b"".join(t[3] for t in tensors)


def test_reference_known_answers():
    f = st.parse_safetensors(reference_test_file())
    st.expect_tensor(f, "bias", "F32", [3])
    st.expect_tensor(f, "half", "F16", [2])
    st.expect_tensor(f, "bfloat", "BF16", [2])
    assert st.read_tensor_f32(f, "bias").tolist() == [1.0, -2.0, 0.5]
    assert st.read_tensor_f32(f, "half").tolist() == [1.0, -0.5]
    assert st.read_tensor_f32(f, "bfloat").tolist() == [1.0, -2.0]
    assert "__metadata__" not in f.header
    assert st.tensor_count(f.header["bias"]) == 3 and st.tensor_count(st.SafetensorEntry("F32", [], (0, 4))) == 1
    assert bytes(st.read_tensor_bytes(f, "half")) == bytes([0x00, 0x3C, 0x00, 0xB8])


def test_f16_bits_match_the_oracle_for_every_pattern(oracle):
    bits = np.arange(65536, dtype=np.uint16)
    got, ref = st.f16_bits_to_f32(bits), oracle.f16_bits_to_f32(bits)
    nan = np.isnan(ref)
    assert np.array_equal(np.isnan(got), nan)
    assert np.array_equal(got[~nan].view(np.uint32), ref[~nan].view(np.uint32))


def _image(header: dict, data: bytes = b"") -> bytes:
    hb = json.dumps(header).encode()
    return len(hb).to_bytes(8, "little") + hb + data


@pytest.mark.parametrize("image,text", [
    (b"\x01\x02\x03", "buffer 过短"),
    ((5).to_bytes(4, "little") + (1).to_bytes(4, "little") + b"{}   ", "超过 4GiB"),
    ((0).to_bytes(8, "little") + b"{}", "header 长度非法"),
    ((100).to_bytes(8, "little") + b"{}", "header 长度非法"),
    ((3).to_bytes(8, "little") + b"{x}", "JSON 解析失败"),
    ((2).to_bytes(8, "little") + b"[]", "不是 JSON object"),
    (_image({"a": 3}), "a 条目非法"),
    (_image({"a": {"shape": [1], "data_offsets": [0, 4]}}), "a 缺少 dtype"),
    (_image({"a": {"dtype": "F32", "data_offsets": [0, 4]}}), "a 缺少 shape"),
    (_image({"a": {"dtype": "F32", "shape": [1], "data_offsets": [0]}}), "a data_offsets 非法"),
    (_image({"a": {"dtype": "F32", "shape": [1], "data_offsets": [4, 0]}}), "a data_offsets 数值非法"),
    (_image({"a": {"dtype": "F32", "shape": [1], "data_offsets": [-4, 0]}}), "a data_offsets 数值非法"),
    (_image({"a": {"dtype": "F32", "shape": [1], "data_offsets": ["x", 4]}}), "a data_offsets 数值非法"),
    (_image({"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}}, bytes(4)), "a 数据越界 end=8"),
])
def test_validation_failures_carry_the_reference_messages(image, text):
    with pytest.raises(st.SafetensorsError, match=text):
        st.parse_safetensors(image)


def test_require_expect_and_unsupported_dtype():
    f = st.parse_safetensors(st.build_safetensors({"w": ("I32", (2, 2), np.arange(4, dtype=np.int32)),
                                                   "d": ("F64", (1,), np.zeros(1))}))
    with pytest.raises(st.SafetensorsError, match="缺少 tensor nope"):
        st.require_tensor(f, "nope")
    with pytest.raises(st.SafetensorsError, match=r"w dtype=I32，期望 F16"):
        st.expect_tensor(f, "w", "F16", [2, 2])
    with pytest.raises(st.SafetensorsError, match=r"w shape=\[2,2\]，期望 \[4\]"):
        st.expect_tensor(f, "w", "I32", [4])
    with pytest.raises(st.SafetensorsError, match="不支持的 dtype F64"):
        st.read_tensor_f32(f, "d")
    assert st.read_tensor_bytes(f, "w").view("<i4").tolist() == [0, 1, 2, 3]
    assert [st.dtype_byte_size(d) for d in ("F64", "I64", "F32", "I32", "F16", "BF16", "I16", "I8", "U8", "BOOL")] == \
        [8, 8, 4, 4, 2, 2, 2, 1, 1, 1]


def test_header_only_parse_does_not_need_the_data():
    img = st.build_safetensors({"w": ("F16", (4, 8), np.zeros((4, 8), np.float16))}, metadata={"format": "pt"})
    n = int.from_bytes(img[:8], "little")
    h = st.parse_safetensors_header(img[8:8 + n])
    assert h["w"].dtype == "F16" and h["w"].shape == [4, 8] and h["w"].data_offsets == (0, 64)
    assert (8 + n) % 8 == 0


def test_checkpoint_image_round_trip_and_projection_views(oracle):
    cfg = synthetic.QwenShape(64, 2, 4, 2, 256, 384)
    W = synthetic.random_qwen_gptq(cfg, seed=5)
    img = st.build_safetensors(qwen_loader.qwen_checkpoint_tensors(W))
    f = qwen_loader.open_safetensors(img)
    assert len(f.header) == 2 + cfg.n_layer * (2 + 7 * 4 + 3)
    t = qwen_loader.read_gptq_linear(f, "model.layers.1.mlp.down_proj", cfg.intermediate, cfg.n_embd)
    src = W["layers"][1]["down"]
    assert np.array_equal(t.qweight, src.qweight) and np.array_equal(t.qzeros, src.qzeros)
    assert np.array_equal(t.scales.view(np.uint16), src.scales.view(np.uint16))
    # the views feed the oracle's dequantiser unchanged: same weights as from the in-memory tensors
    a = oracle.dequantize_gptq_int4(t.qweight, t.qzeros, t.scales, t.in_features, t.out_features, t.group_size)
    b = oracle.dequantize_gptq_int4(src.qweight, src.qzeros, src.scales, src.in_features, src.out_features, src.group_size)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    rows = qwen_loader.read_f16_rows(f, "model.embed_tokens.weight", 3, 2, cfg.n_embd)
    assert np.array_equal(rows, W["embed"][3:5].view(np.uint16))
    with pytest.raises(qwen_loader.QwenLoaderError, match="rowLength=100 不符"):
        qwen_loader.read_f16_rows(f, "model.embed_tokens.weight", 0, 1, 100)
    with pytest.raises(qwen_loader.QwenLoaderError, match="期望 F16，实际 I32"):
        qwen_loader.read_f16_rows(f, "model.layers.0.mlp.down_proj.qweight", 0, 1, cfg.n_embd)
    with pytest.raises(st.SafetensorsError, match=r"期望 \[48,128\]"):
        qwen_loader.read_gptq_linear(f, "model.layers.0.mlp.down_proj", cfg.intermediate, 128)
