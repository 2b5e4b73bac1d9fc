"""ctypes front end of the CPU oracle (``webllm_oracle.c``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by the smoke check and by the CPU-baseline legs
of ``bench.py``. The product package never imports this module.

Every function mirrors one function of the reference (cited in ``webllm_oracle.c``) and takes /
returns numpy arrays with the reference's layouts.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from dataclasses import dataclass
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "_build" / "libwebllm_oracle.so"
_lib = None


def build(force: bool = False) -> Path:
    """Compile the oracle with the Makefile beside this file (gcc only, a second or two)."""
    src = _HERE / "webllm_oracle.c"
    if force or not _LIB_PATH.exists() or _LIB_PATH.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(_HERE)], check=True, capture_output=True)
    return _LIB_PATH


class _Layer(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in (
        "input_norm", "qW", "qB", "kW", "kB", "vW", "vB", "oW", "post_norm", "gateW", "upW", "downW")]


class _Config(C.Structure):
    _fields_ = [("vocab", C.c_int64), ("n_layer", C.c_int64), ("n_head", C.c_int64), ("n_kv_head", C.c_int64),
                ("n_embd", C.c_int64), ("intermediate", C.c_int64), ("rms_eps", C.c_double),
                ("rope_theta", C.c_double)]


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(str(_LIB_PATH))
        L.wo_f16_bits_to_f32.restype = C.c_float
        L.wo_f16_bits_to_f32.argtypes = [C.c_uint16]
        L.wo_f32_to_f16_bits.restype = C.c_uint16
        L.wo_f32_to_f16_bits.argtypes = [C.c_float]
        L.wo_rng_next.restype = C.c_double
        L.wo_rng_next.argtypes = [C.POINTER(C.c_uint32)]
        L.wo_rng_seed.restype = C.c_uint32
        L.wo_rng_seed.argtypes = [C.c_uint32]
        L.wo_sample_greedy.restype = C.c_int64
        L.wo_max_threads.restype = C.c_int
        _lib = L
    return _lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def max_threads() -> int:
    return int(os.cpu_count() or lib().wo_max_threads())


# ------------------------------------------------------------------ fp16

def f16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    bits = np.ascontiguousarray(bits, dtype=np.uint16)
    out = np.empty(bits.shape, np.float32)
    lib().wo_f16_to_f32_array(_p(bits), _p(out), C.c_int64(bits.size))
    return out


def f32_to_f16_bits(x: np.ndarray) -> np.ndarray:
    x = _f32(x)
    out = np.empty(x.shape, np.uint16)
    lib().wo_f32_to_f16_array(_p(x), _p(out), C.c_int64(x.size))
    return out


def round_f16(x: np.ndarray) -> np.ndarray:
    return f16_bits_to_f32(f32_to_f16_bits(x))


# ------------------------------------------------------------------- RNG

class Rng:
    """``makeRng(seed)`` of the reference: xorshift32, ``state / 2**32``."""

    def __init__(self, seed: int):
        self._state = C.c_uint32(lib().wo_rng_seed(C.c_uint32(seed & 0xFFFFFFFF)))

    def __call__(self) -> float:
        return float(lib().wo_rng_next(C.byref(self._state)))

    def random_f32(self, n: int) -> np.ndarray:
        """``randomF32(n, rng)``: ``rng()*2-1`` stored to f32."""
        out = np.empty(n, np.float32)
        lib().wo_random_f32(_p(out), C.c_int64(n), C.byref(self._state))
        return out


# ------------------------------------------------------------- tolerance

@dataclass
class Tolerance:
    ok: bool
    max_abs: float
    max_rel: float


def check_tolerance(got, ref, atol: float, rtol: float) -> Tolerance:
    got, ref = _f32(got).ravel(), _f32(ref).ravel()
    if got.size != ref.size:
        raise ValueError(f"checkTolerance: 长度不一致 got={got.size} ref={ref.size}")
    ma, mr = C.c_double(), C.c_double()
    ok = lib().wo_check_tolerance(_p(got), _p(ref), C.c_int64(ref.size), C.c_double(atol), C.c_double(rtol),
                                  C.byref(ma), C.byref(mr))
    return Tolerance(bool(ok), ma.value, mr.value)


# --------------------------------------------------------------- dequant

class OracleError(Exception):
    pass


def dequantize_gptq_int4(qweight: np.ndarray, qzeros, scales: np.ndarray, in_features: int, out_features: int,
                         group_size: int = 128, bits: int = 4) -> np.ndarray:
    """``dequantizeGptqInt4``: qweight / qzeros are the raw little-endian bytes (any integer dtype is viewed
    as bytes), scales is f32 ``[groups, out]``; returns f32 ``[out, in]``."""
    qw = np.ascontiguousarray(qweight).view(np.uint8).ravel()
    qz = None if qzeros is None else np.ascontiguousarray(qzeros).view(np.uint8).ravel()
    sc = _f32(scales).ravel()
    n_out = max(in_features, 0) * max(out_features, 0)
    out = np.zeros(n_out, np.float32)
    err = C.create_string_buffer(256)
    rc = lib().wo_dequantize_gptq_int4(_p(qw), C.c_int64(qw.size), _p(qz), C.c_int64(0 if qz is None else qz.size),
                                       _p(sc), C.c_int64(sc.size), C.c_int64(in_features), C.c_int64(out_features),
                                       C.c_int64(group_size), C.c_int(bits), _p(out), err, C.c_int(256))
    if rc != 0:
        raise OracleError(err.value.decode("utf-8"))
    return out.reshape(out_features, in_features)


# ------------------------------------------------------------------ GEMM

def gemm_nt_ref(A, W, M: int, N: int, K: int, bias=None, threads: int = 1) -> np.ndarray:
    A, W = _f32(A).ravel(), _f32(W).ravel()
    assert A.size >= M * K and W.size >= N * K
    b = None if bias is None else _f32(bias).ravel()
    out = np.empty(M * N, np.float32)
    lib().wo_gemm_nt_ref(_p(A), _p(W), C.c_int64(M), C.c_int64(N), C.c_int64(K), _p(b), _p(out), C.c_int(threads))
    return out.reshape(M, N)


def rmsnorm_ref(x, w, rows: int, D: int, eps: float) -> np.ndarray:
    x, w = _f32(x).ravel(), _f32(w).ravel()
    out = np.empty(rows * D, np.float32)
    lib().wo_rmsnorm_ref(_p(x), _p(w), C.c_int64(rows), C.c_int64(D), C.c_double(eps), _p(out))
    return out.reshape(rows, D)


def rope_half_ref(x, rows: int, n_head: int, D: int, T: int, base: float, pos_offset: int = 0) -> np.ndarray:
    x = _f32(x).ravel()
    out = np.empty_like(x)
    lib().wo_rope_half_ref(_p(x), C.c_int64(rows), C.c_int64(n_head), C.c_int64(D), C.c_int64(T), C.c_double(base),
                           C.c_int64(pos_offset), _p(out))
    return out


def attention_gqa_ref(q, k, v, B: int, T: int, n_head: int, n_kv: int, D: int) -> np.ndarray:
    q, k, v = _f32(q).ravel(), _f32(k).ravel(), _f32(v).ravel()
    out = np.empty(B * T * n_head * D, np.float32)
    lib().wo_attention_gqa_ref(_p(q), _p(k), _p(v), C.c_int64(B), C.c_int64(T), C.c_int64(n_head), C.c_int64(n_kv),
                               C.c_int64(D), _p(out))
    return out


def silu_mul_ref(gate, up) -> np.ndarray:
    gate, up = _f32(gate).ravel(), _f32(up).ravel()
    out = np.empty_like(gate)
    lib().wo_silu_mul_ref(_p(gate), _p(up), C.c_int64(gate.size), _p(out))
    return out


def sample_greedy(logits, offset: int = 0, vocab: int | None = None) -> int:
    logits = _f32(logits).ravel()
    vocab = logits.size - offset if vocab is None else vocab
    return int(lib().wo_sample_greedy(_p(logits), C.c_int64(offset), C.c_int64(vocab)))


# ------------------------------------------------------------ forward

@dataclass
class QwenConfig:
    """``QwenConfig`` of src/model/qwen-config.ts:12-28 (blockSize is a limit of the GPU path, not of the
    reference forward, and is not needed here)."""
    vocab_size: int
    n_layer: int
    n_head: int
    n_kv_head: int
    n_embd: int
    intermediate: int
    rms_eps: float = 1e-6
    rope_theta: float = 1000000.0

    @property
    def head_dim(self) -> int:
        return self.n_embd // self.n_head

    @property
    def kv_dim(self) -> int:
        return self.head_dim * self.n_kv_head


_LAYER_KEYS = ("input_norm", "qW", "qB", "kW", "kB", "vW", "vB", "oW", "post_norm", "gateW", "upW", "downW")


def _pack_weights(cfg: QwenConfig, weights: dict):
    """weights: {"embed": [V,C], "final_norm": [C], "layers": [ {key: array} ... ]} as f32."""
    keep = []
    layers = (_Layer * cfg.n_layer)()
    for i, L in enumerate(weights["layers"]):
        for key in _LAYER_KEYS:
            a = _f32(L[key]).ravel()
            keep.append(a)
            setattr(layers[i], key, a.ctypes.data)
    embed = _f32(weights["embed"]).ravel()
    fnorm = _f32(weights["final_norm"]).ravel()
    keep += [embed, fnorm]
    c = _Config(cfg.vocab_size, cfg.n_layer, cfg.n_head, cfg.n_kv_head, cfg.n_embd, cfg.intermediate, cfg.rms_eps,
                cfg.rope_theta)
    return c, embed, fnorm, layers, keep


def qwen_forward_ref(cfg: QwenConfig, weights: dict, tokens, B: int, T: int, threads: int = 1,
                     want_layers: bool = False):
    """``qwenForwardRef``: returns logits ``[B*T, V]`` (and the per-layer hidden states if asked)."""
    c, embed, fnorm, layers, keep = _pack_weights(cfg, weights)
    tok = np.ascontiguousarray(tokens, dtype=np.uint32).ravel()
    assert tok.size == B * T
    logits = np.empty((B * T, cfg.vocab_size), np.float32)
    louts = [np.empty((B * T, cfg.n_embd), np.float32) for _ in range(cfg.n_layer)] if want_layers else None
    lptr = None
    if louts is not None:
        lptr = (C.c_void_p * cfg.n_layer)(*[a.ctypes.data for a in louts])
    lib().wo_qwen_forward_ref(C.byref(c), _p(embed), _p(fnorm), layers, _p(tok), C.c_int64(B), C.c_int64(T),
                              _p(logits), lptr, C.c_int(threads))
    return (logits, louts) if want_layers else logits


class CachedForward:
    """The reference forward with a KV cache (one sequence): ``prefill`` then ``decode_step``, each
    returning the logits row of the last processed token."""

    def __init__(self, cfg: QwenConfig, weights: dict, max_t: int, kv_f16: bool = False, threads: int = 1):
        self.cfg, self.max_t, self.kv_f16, self.threads = cfg, max_t, kv_f16, threads
        self._c, self._embed, self._fnorm, self._layers, self._keep = _pack_weights(cfg, weights)
        self.k_cache = np.zeros((cfg.n_layer, max_t, cfg.kv_dim), np.float32)
        self.v_cache = np.zeros((cfg.n_layer, max_t, cfg.kv_dim), np.float32)
        self.cache_len = 0

    def _run(self, tokens) -> np.ndarray:
        tok = np.ascontiguousarray(tokens, dtype=np.uint32).ravel()
        if self.cache_len + tok.size > self.max_t:
            raise ValueError("context exceeds max_t")
        logits = np.empty(self.cfg.vocab_size, np.float32)
        lib().wo_qwen_forward_cached(C.byref(self._c), _p(self._embed), _p(self._fnorm), self._layers, _p(tok),
                                     C.c_int64(tok.size), C.c_int64(self.cache_len), C.c_int64(self.max_t),
                                     _p(self.k_cache), _p(self.v_cache), C.c_int(1 if self.kv_f16 else 0),
                                     _p(logits), C.c_int(self.threads))
        self.cache_len += tok.size
        return logits

    def prefill(self, tokens) -> np.ndarray:
        assert self.cache_len == 0
        return self._run(tokens)

    def decode_step(self, token: int) -> np.ndarray:
        assert self.cache_len > 0
        return self._run([token])
