"""``QwenGpt`` — the host-side model object of the reference (src/model/qwen.ts:124-646), over the C ABI.

Same surface: ``alloc_f16 / write_f16_chunk / upload_f16 / upload_f32 / upload_layer / upload_weights``,
``forward / prefill / decode_step / reset_cache``, ``gemm`` and the read-back helpers. New here: GPTQ
tensors are uploaded packed (``upload_gptq`` / ``upload_gptq_layer``) instead of being dequantised on the
host, and ``decode_greedy`` keeps the whole sampling loop on the device.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib as L
from .buffer import Tensor
from .device import Gpu
from .synthetic import GptqTensors, QwenShape


def concat_gptq(parts: list[GptqTensors]) -> GptqTensors:
    """Concatenates GPTQ linears that share their input along the output dimension (q|k|v, gate|up).
    Every part must have a multiple of 8 output columns, so no qzeros word is split."""
    K, g = parts[0].in_features, parts[0].group_size
    for p in parts:
        if p.in_features != K or p.group_size != g or p.out_features % 8 or (p.qzeros is None) != (parts[0].qzeros is None):
            raise L.WebllmError(L.WB_ERR_BAD_ARG, "concat_gptq: parts must share K, group and qzeros presence; N % 8 == 0")
    qz = None if parts[0].qzeros is None else np.concatenate([p.qzeros for p in parts], axis=1)
    return GptqTensors(np.concatenate([p.qweight for p in parts], axis=1), qz,
                       np.concatenate([p.scales for p in parts], axis=1), K, sum(p.out_features for p in parts), g)


class QwenGpt:
    def __init__(self, gpu: Gpu, config: QwenShape, max_t: int = 128, kv_dtype: str = "f32"):
        self.gpu, self.config, self.max_t, self.kv_dtype = gpu, config, max_t, kv_dtype
        self._model = C.c_void_p()
        self._lib = gpu._lib
        self._exact = False

    # ------------------------------------------------------------------ weight upload (qwen.ts:247-301)
    def alloc_f16(self, name: str, length: int, rows: int | None = None) -> None:
        rows = 1 if rows is None else rows
        self.gpu.f16_alloc(name, rows, length // rows)

    def write_f16_chunk(self, name: str, offset_elements: int, data) -> None:
        self.gpu.f16_write_chunk(self.gpu.weight(name), offset_elements, data)

    def upload_f16(self, name: str, data, rows: int | None = None) -> None:
        """``uploadF16``: f32 data rounded to fp16 on the device with the reference's rules. ``rows`` gives
        the matrix its [rows, cols] shape (the reference keeps only the length and passes N, K to gemm)."""
        data = np.asarray(data, np.float32)
        if rows is None:
            rows = data.shape[0] if data.ndim == 2 else 1
        self.alloc_f16(name, data.size, rows)
        self.write_f16_chunk(name, 0, data)

    def upload_f16_bits(self, name: str, bits, rows: int) -> None:
        bits = np.ascontiguousarray(bits)
        h = self.gpu.f16_alloc(name, rows, bits.size // rows)
        self.gpu.f16_write_bits(h, 0, bits)

    def upload_f32(self, name: str, data) -> None:
        self.gpu.f32_upload(name, data)

    def upload_layer(self, index: int, Lw: dict) -> None:
        """``uploadLayer`` with the reference's ``QwenLayerWeights`` (dense f32 [out, in] matrices)."""
        p, cfg = f"L{index}", self.config
        C_, KV, I = cfg.n_embd, cfg.kv_dim, cfg.intermediate
        self.upload_f32(f"{p}.inNorm", Lw["inputNorm"])
        self.upload_f16(f"{p}.qW", Lw["qW"], C_)
        self.upload_f32(f"{p}.qB", Lw["qB"])
        self.upload_f16(f"{p}.kW", Lw["kW"], KV)
        self.upload_f32(f"{p}.kB", Lw["kB"])
        self.upload_f16(f"{p}.vW", Lw["vW"], KV)
        self.upload_f32(f"{p}.vB", Lw["vB"])
        self.upload_f16(f"{p}.oW", Lw["oW"], C_)
        self.upload_f32(f"{p}.postNorm", Lw["postNorm"])
        self.upload_f16(f"{p}.gateW", Lw["gateW"], I)
        self.upload_f16(f"{p}.upW", Lw["upW"], I)
        self.upload_f16(f"{p}.downW", Lw["downW"], C_)

    def upload_weights(self, weights: dict) -> None:
        """``uploadWeights``: {"embed", "finalNorm", "layers": [QwenLayerWeights]} as f32 arrays."""
        self.upload_f16("embed", weights["embed"], self.config.vocab_size)
        self.upload_f32("finalNorm", weights["finalNorm"])
        for i, Lw in enumerate(weights["layers"]):
            self.upload_layer(i, Lw)

    def upload_gptq(self, name: str, t: GptqTensors) -> int:
        return self.gpu.gptq_register(name, t.qweight, t.qzeros, t.scales, t.in_features, t.out_features, t.group_size)

    def upload_gptq_layer(self, index: int, Lw: dict, fuse: bool = True) -> None:
        """One layer of a GPTQ checkpoint ({"q".."down": GptqTensors, "q_bias", "k_bias", "v_bias", "input_norm",
        "post_norm"}), what dequantGptqLinear + uploadLayer do in the reference (src/weights/qwen-loader.ts:144-165)
        minus the dequantisation. ``fuse`` registers q|k|v and gate|up as single projections."""
        p = f"L{index}"
        self.upload_f32(f"{p}.inNorm", Lw["input_norm"])
        self.upload_f32(f"{p}.postNorm", Lw["post_norm"])
        if fuse:
            self.upload_gptq(f"{p}.qkvW", concat_gptq([Lw["q"], Lw["k"], Lw["v"]]))
            self.upload_f32(f"{p}.qkvB", np.concatenate([Lw["q_bias"], Lw["k_bias"], Lw["v_bias"]]))
            self.upload_gptq(f"{p}.gateUpW", concat_gptq([Lw["gate"], Lw["up"]]))
        else:
            for k, b in (("q", "q_bias"), ("k", "k_bias"), ("v", "v_bias")):
                self.upload_gptq(f"{p}.{k}W", Lw[k])
                self.upload_f32(f"{p}.{k}B", Lw[b])
            self.upload_gptq(f"{p}.gateW", Lw["gate"])
            self.upload_gptq(f"{p}.upW", Lw["up"])
        self.upload_gptq(f"{p}.oW", Lw["o"])
        self.upload_gptq(f"{p}.downW", Lw["down"])

    def upload_gptq_model(self, weights: dict, fuse: bool = True) -> None:
        """A whole synthetic / loaded GPTQ checkpoint: fp16 embedding bits, f32 final norm, GPTQ layers."""
        self.upload_f16_bits("embed", weights["embed"], self.config.vocab_size)
        self.upload_f32("finalNorm", weights["final_norm"])
        for i, Lw in enumerate(weights["layers"]):
            self.upload_gptq_layer(i, Lw, fuse)

    @property
    def weight_bytes(self) -> int:
        return self.gpu.weight_bytes

    # ------------------------------------------------------------------ model object
    def _ensure(self):
        if not self._model:
            cfg = self.config
            c = L.QwenConfigC(cfg.vocab_size, cfg.n_layer, cfg.n_head, cfg.n_kv_head, cfg.n_embd, cfg.intermediate,
                              self.max_t, L.WB_F16 if self.kv_dtype == "f16" else L.WB_F32, cfg.rms_eps, cfg.rope_theta)
            L.check(self._lib.wb_qwen_create(self.gpu.ctx, C.byref(c), C.byref(self._model)))
            L.check(self._lib.wb_qwen_set_exact(self._model, 1 if self._exact else 0))
        return self._model

    def close(self) -> None:
        if self._model:
            self._lib.wb_qwen_destroy(self._model)
            self._model = C.c_void_p()

    def set_exact(self, exact: bool) -> None:
        """fp32-activation mode for every linear of the forward pass."""
        self._exact = exact
        if self._model:
            L.check(self._lib.wb_qwen_set_exact(self._model, 1 if exact else 0))

    # ------------------------------------------------------------------ forward (qwen.ts:305-331)
    def reset_cache(self) -> None:
        L.check(self._lib.wb_qwen_reset_cache(self._ensure()))

    @property
    def cache_len(self) -> int:
        n = C.c_int64()
        L.check(self._lib.wb_qwen_cache_len(self._ensure(), C.byref(n)))
        return n.value

    def _tokens(self, tokens):
        t = np.ascontiguousarray(tokens, dtype=np.uint32).ravel()
        return t, t.ctypes.data_as(C.c_void_p)

    def forward(self, tokens, B: int, T: int) -> Tensor:
        t, p = self._tokens(tokens)
        if t.size != B * T:
            raise L.WebllmError(L.WB_ERR_BAD_ARG, f"tokens 长度 {t.size} != M={B * T}")
        off = C.c_uint64()
        L.check(self._lib.wb_qwen_forward(self._ensure(), p, B, T, C.byref(off)))
        return Tensor(off.value, B * T * self.config.vocab_size, [B * T, self.config.vocab_size])

    def prefill(self, tokens, last_only: bool = False) -> Tensor:
        t, p = self._tokens(tokens)
        off = C.c_uint64()
        L.check(self._lib.wb_qwen_prefill(self._ensure(), p, t.size, 1 if last_only else 0, C.byref(off)))
        rows = 1 if last_only else t.size
        return Tensor(off.value, rows * self.config.vocab_size, [rows, self.config.vocab_size])

    def decode_step(self, token: int) -> Tensor:
        off = C.c_uint64()
        L.check(self._lib.wb_qwen_decode_step(self._ensure(), int(token), C.byref(off)))
        return Tensor(off.value, self.config.vocab_size, [1, self.config.vocab_size])

    def decode_greedy(self, first_token: int, n_steps: int) -> np.ndarray:
        """Feeds ``first_token`` and samples ``n_steps`` tokens greedily without leaving the device."""
        out = np.empty(n_steps, np.uint32)
        L.check(self._lib.wb_qwen_decode_greedy(self._ensure(), int(first_token), n_steps, out.ctypes.data_as(C.c_void_p)))
        return out

    def last_logits(self) -> np.ndarray:
        out = np.empty(self.config.vocab_size, np.float32)
        L.check(self._lib.wb_qwen_last_logits(self._ensure(), out.ctypes.data_as(C.c_void_p)))
        return out

    # ------------------------------------------------------------------ linear (qwen.ts:568-618)
    def gemm(self, A: Tensor, weight: str, Cout: Tensor, bias: str | None, M: int, N: int, K: int,
             exact: bool | None = None) -> None:
        """``gemm(A, weight, C, bias, M, N, K)``: C = A . W^T (+ bias). N and K are checked against the
        registered weight (the reference trusts the caller)."""
        h = self.gpu.weight(weight)
        p = self.gpu.plan(h, M, A.dtype)  # raises for a non-matrix weight
        del p
        hb = None if bias is None else self.gpu.weight(bias)
        if A.length < M * K or Cout.length < M * N:
            raise L.WebllmError(L.WB_ERR_BAD_ARG, f"gemm: tensors too small for M={M} N={N} K={K}")
        self.gpu.linear(h, A, Cout, hb, M, exact=self._exact if exact is None else exact)

    # ------------------------------------------------------------------ read-back (qwen.ts:514-531)
    def read_tensor(self, t: Tensor) -> np.ndarray:
        return self.gpu.read(t)

    def read_tensor_slice(self, t: Tensor, element_offset: int, element_count: int) -> np.ndarray:
        return self.gpu.read(t, element_offset, element_count)

    def read_weight_f16_bytes(self, name: str, element_offset: int, element_count: int) -> np.ndarray:
        return self.gpu.read_weight_f16(self.gpu.weight(name), element_offset, element_count)
