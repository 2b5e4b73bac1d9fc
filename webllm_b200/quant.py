"""GPTQ int4 dequantisation with the reference's call shape (src/weights/quant.ts:16-118), run on the GPU."""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from . import _lib as L
from .device import Gpu


@dataclass
class GptqInt4Params:
    """``GptqInt4Params`` (src/weights/quant.ts:16-30). ``scales`` may be fp16 (as in the checkpoint) or
    f32 values that are exactly representable in fp16 (what ``readTensorF32`` yields for an F16 tensor)."""
    qweight: np.ndarray
    scales: np.ndarray
    in_features: int
    out_features: int
    qzeros: np.ndarray | None = None
    group_size: int = 128
    bits: int = 4


def scales_to_f16(scales: np.ndarray) -> np.ndarray:
    s = np.asarray(scales)
    if s.dtype == np.float16:
        return np.ascontiguousarray(s)
    h = s.astype(np.float16)
    if not np.array_equal(h.astype(np.float32), s.astype(np.float32), equal_nan=True):
        raise L.WebllmError(L.WB_ERR_BAD_ARG, "GPTQ: scales must be fp16 values (the checkpoint stores F16)")
    return np.ascontiguousarray(h)


def dequantize_gptq_int4(gpu: Gpu, params: GptqInt4Params, dtype: str = "f32") -> np.ndarray:
    """``dequantizeGptqInt4(params)``: returns ``[out_features, in_features]`` — f32 equal to the
    reference's result bit for bit, or (``dtype="f16"``) the fp16 copy the reference uploads. Raises
    ``WebllmError`` with the reference's message on the reference's validation failures."""
    h = gpu.gptq_register("__dequant_tmp__", params.qweight, params.qzeros, scales_to_f16(params.scales),
                          params.in_features, params.out_features, params.group_size, params.bits)
    mark = gpu.arena.used_bytes
    try:
        t = gpu.arena.alloc(params.in_features * params.out_features, [params.out_features, params.in_features], dtype)
        gpu.gptq_dequant(h, t)
        out = gpu.read(t)
    finally:
        gpu.arena.rewind(mark)
        gpu.weight_pop()
    return out.reshape(params.out_features, params.in_features)
