"""Loads a Qwen2.5 GPTQ-int4 safetensors checkpoint into a ``QwenGpt`` — ``loadQwenWeights``
(src/weights/qwen-loader.ts:102-177) without its CPU dequantisation.

Same file format as the reference documents (:4-8): per layer seven GPTQ projections
(``qweight`` I32 / ``qzeros`` I32, stored zero - 1 / ``scales`` F16 / ``g_idx`` I32, the identity, ignored),
F16 biases on q/k/v only, F16 layer norms, ``model.embed_tokens.weight`` F16 [vocab, C] doubling as the tied
lm_head. Where the reference dequantises every projection to f32 on the CPU (``dequantGptqLinear`` :55-67)
and uploads fp16, the three tensors of a projection go to the device as the file stores them: they are numpy
views of the (memory-mapped) file handed to ``wb_gptq_register``. The embedding's fp16 bits are uploaded in
row chunks (``EMBED_CHUNK_ROWS``, :98-100) without a float round trip.
"""
from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path

import numpy as np

from . import safetensors as st
from .qwen import QwenGpt
from .quant import GptqInt4Params, dequantize_gptq_int4
from .synthetic import GptqTensors

EMBED_CHUNK_ROWS = 8192
GROUP_SIZE = 128

# projection -> (input width, output width) as attribute names of the shape
_PROJECTIONS = (("self_attn.q_proj", "q", "n_embd", "n_embd"), ("self_attn.k_proj", "k", "n_embd", "kv_dim"),
                ("self_attn.v_proj", "v", "n_embd", "kv_dim"), ("self_attn.o_proj", "o", "n_embd", "n_embd"),
                ("mlp.gate_proj", "gate", "n_embd", "intermediate"), ("mlp.up_proj", "up", "n_embd", "intermediate"),
                ("mlp.down_proj", "down", "intermediate", "n_embd"))


class QwenLoaderError(ValueError):
    """What the reference signals with ``throw new Error('qwen-loader: …')``."""


@dataclass
class QwenLoadResult:
    """``QwenLoadResult`` (src/weights/qwen-loader.ts:38-50)."""
    gpu_bytes: int
    tensor_count: int
    file_bytes: int
    layer: dict | None = None        # keep_layer: that layer's projections dequantised to f32 [out, in] + norms, biases
    embed_rows: np.ndarray | None = None


def read_gptq_linear(file: st.SafetensorFile, prefix: str, in_features: int, out_features: int,
                     group_size: int = GROUP_SIZE) -> GptqTensors:
    """The three tensors of one projection as views of the file (no copy, no dequantisation), shape-checked the
    way ``dequantizeGptqInt4`` will check their byte lengths (src/weights/quant.ts:54-79)."""
    rows, groups, zcols = -(-in_features // 8), -(-in_features // group_size), -(-out_features // 8)
    st.expect_tensor(file, f"{prefix}.qweight", "I32", [rows, out_features])
    st.expect_tensor(file, f"{prefix}.qzeros", "I32", [groups, zcols])
    st.expect_tensor(file, f"{prefix}.scales", "F16", [groups, out_features])
    qw = st.read_tensor_bytes(file, f"{prefix}.qweight").view("<i4").reshape(rows, out_features)
    qz = st.read_tensor_bytes(file, f"{prefix}.qzeros").view("<i4").reshape(groups, zcols)
    sc = st.read_tensor_bytes(file, f"{prefix}.scales").view("<f2").reshape(groups, out_features)
    return GptqTensors(qw, qz, sc, in_features, out_features, group_size)


def read_f16_rows(file: st.SafetensorFile, name: str, row_start: int, row_count: int, row_length: int) -> np.ndarray:
    """Rows [row_start, row_start + row_count) of an F16 matrix as raw fp16 bits (``readF16Rows`` :70-95 returns
    them converted to f32; ``st.f16_bits_to_f32`` does that)."""
    entry = st.require_tensor(file, name)
    if entry.dtype != "F16":
        raise QwenLoaderError(f"qwen-loader: {name} 期望 F16，实际 {entry.dtype}")
    if len(entry.shape) != 2 or entry.shape[1] != row_length:
        raise QwenLoaderError(f"qwen-loader: {name} 形状 {','.join(map(str, entry.shape))} 与 rowLength={row_length} 不符")
    bits = st.read_tensor_bytes(file, name).view("<u2").reshape(entry.shape[0], row_length)
    return bits[row_start:row_start + row_count]


def open_safetensors(source) -> st.SafetensorFile:
    """A path (memory-mapped, so a 450 MB checkpoint is never read twice) or a bytes-like file image."""
    if isinstance(source, (str, Path)):
        return st.parse_safetensors(np.memmap(source, dtype=np.uint8, mode="r"))
    return st.parse_safetensors(source)


def load_qwen_weights(model: QwenGpt, source, on_progress=None, keep_layer: int | None = None,
                      keep_embed_rows: tuple[int, int] | None = None, fuse: bool = True) -> QwenLoadResult:
    """``loadQwenWeights(gpu, model, options)``: embed (chunked) → final norm → layer by layer. ``fuse`` registers
    q|k|v and gate|up as single projections (what the fast decode step needs)."""
    cfg = model.config
    C, V = cfg.n_embd, cfg.vocab_size
    file = open_safetensors(source)
    count = 0

    embed = st.require_tensor(file, "model.embed_tokens.weight")
    if list(embed.shape) != [V, C]:
        raise QwenLoaderError(f"qwen-loader: embed_tokens 形状 [{','.join(map(str, embed.shape))}]，期望 [{V},{C}]")
    handle = model.gpu.f16_alloc("embed", V, C)
    for start in range(0, V, EMBED_CHUNK_ROWS):
        rows = min(EMBED_CHUNK_ROWS, V - start)
        model.gpu.f16_write_bits(handle, start * C, read_f16_rows(file, "model.embed_tokens.weight", start, rows, C))
    count += 1
    embed_rows = None
    if keep_embed_rows is not None:
        embed_rows = st.f16_bits_to_f32(read_f16_rows(file, "model.embed_tokens.weight", keep_embed_rows[0], keep_embed_rows[1], C))

    model.upload_f32("finalNorm", st.read_tensor_f32(file, "model.norm.weight"))
    count += 1

    kept = None
    for i in range(cfg.n_layer):
        p = f"model.layers.{i}"
        layer = {"input_norm": st.read_tensor_f32(file, f"{p}.input_layernorm.weight"),
                 "post_norm": st.read_tensor_f32(file, f"{p}.post_attention_layernorm.weight")}
        for proj, key, kin, kout in _PROJECTIONS:
            layer[key] = read_gptq_linear(file, f"{p}.{proj}", getattr(cfg, kin), getattr(cfg, kout))
        for key in ("q", "k", "v"):
            layer[f"{key}_bias"] = st.read_tensor_f32(file, f"{p}.self_attn.{key}_proj.bias")
        count += 12
        model.upload_gptq_layer(i, layer, fuse)
        if keep_layer == i:
            kept = _dequantised_layer(model, layer)
        if on_progress is not None:
            on_progress(i + 1, cfg.n_layer, f"layer {i + 1}/{cfg.n_layer}")

    return QwenLoadResult(model.weight_bytes, count, int(file.buffer.size), kept, embed_rows)


def _dequantised_layer(model: QwenGpt, layer: dict) -> dict:
    """``QwenLayerWeights`` of one layer for checking: the projections dequantised on the device to f32 [out, in]."""
    names = {"q": "qW", "k": "kW", "v": "vW", "o": "oW", "gate": "gateW", "up": "upW", "down": "downW"}
    out = {"inputNorm": layer["input_norm"], "postNorm": layer["post_norm"],
           "qB": layer["q_bias"], "kB": layer["k_bias"], "vB": layer["v_bias"]}
    for key, ref_name in names.items():
        t = layer[key]
        params = GptqInt4Params(qweight=t.qweight, scales=t.scales, in_features=t.in_features, out_features=t.out_features,
                                qzeros=t.qzeros, group_size=t.group_size)
        out[ref_name] = dequantize_gptq_int4(model.gpu, params, "f32")
    return out


def qwen_checkpoint_tensors(weights: dict) -> dict:
    """A synthetic checkpoint (``synthetic.random_qwen_gptq``) as ``{name: (dtype, shape, data)}`` with the
    tensor names and dtypes of the real file, for ``safetensors.build_safetensors``."""
    def f16(a):
        return np.asarray(a, np.float32).astype(np.float16)

    embed = np.asarray(weights["embed"])
    out = {"model.embed_tokens.weight": ("F16", embed.shape, embed.view(np.uint16) if embed.dtype == np.float16 else embed),
           "model.norm.weight": ("F16", weights["final_norm"].shape, f16(weights["final_norm"]))}
    for i, L in enumerate(weights["layers"]):
        p = f"model.layers.{i}"
        out[f"{p}.input_layernorm.weight"] = ("F16", L["input_norm"].shape, f16(L["input_norm"]))
        out[f"{p}.post_attention_layernorm.weight"] = ("F16", L["post_norm"].shape, f16(L["post_norm"]))
        for proj, key, _, _ in _PROJECTIONS:
            t = L[key]
            out[f"{p}.{proj}.qweight"] = ("I32", t.qweight.shape, t.qweight)
            out[f"{p}.{proj}.qzeros"] = ("I32", t.qzeros.shape, t.qzeros)
            out[f"{p}.{proj}.scales"] = ("F16", t.scales.shape, np.asarray(t.scales).view(np.uint16))
            out[f"{p}.{proj}.g_idx"] = ("I32", (t.in_features,), (np.arange(t.in_features) // t.group_size).astype(np.int32))
        for key in ("q", "k", "v"):
            out[f"{p}.self_attn.{key}_proj.bias"] = ("F16", L[f"{key}_bias"].shape, f16(L[f"{key}_bias"]))
    return out
