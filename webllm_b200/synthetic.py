"""Seeded synthetic GPTQ tensors and Qwen2-shaped models.

No checkpoint is available offline, so tests and benchmarks use random tensors with the shapes, packing
and value distributions of Qwen2.5-0.5B-Instruct-GPTQ-Int4 (src/weights/qwen-loader.ts:1-12;
src/weights/quant.ts:1-14). The reference ships no quantiser; ``rtn_quantize`` is a plain
round-to-nearest one that emits the checkpoint format.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

# (in_features K, out_features N) of the seven projections, src/weights/qwen-loader.ts:152-163
QWEN05B_SHAPES = {
    "q": (896, 896), "k": (896, 128), "v": (896, 128), "o": (896, 896),
    "gate": (896, 4864), "up": (896, 4864), "down": (4864, 896),
}
QWEN7B_SHAPES = {
    "q": (3584, 3584), "k": (3584, 512), "v": (3584, 512), "o": (3584, 3584),
    "gate": (3584, 18944), "up": (3584, 18944), "down": (18944, 3584),
}


@dataclass
class GptqTensors:
    """One GPTQ linear in checkpoint layout: qweight int32 [ceil(K/8), N], qzeros int32 [ceil(K/g), ceil(N/8)]
    (stored value = zero point - 1), scales fp16 [ceil(K/g), N]."""
    qweight: np.ndarray
    qzeros: np.ndarray | None
    scales: np.ndarray
    in_features: int
    out_features: int
    group_size: int = 128

    @property
    def nbytes(self) -> int:
        return self.qweight.nbytes + self.scales.nbytes + (0 if self.qzeros is None else self.qzeros.nbytes)


def pack_nibbles_along_k(q: np.ndarray) -> np.ndarray:
    """q: uint8 [K, N] of values 0..15 -> int32 [ceil(K/8), N], nibble j of word [r, n] = q[8r+j, n]."""
    K, N = q.shape
    rows = -(-K // 8)
    pad = np.zeros((rows * 8, N), np.uint32)
    pad[:K] = q
    pad = pad.reshape(rows, 8, N)
    word = np.zeros((rows, N), np.uint32)
    for j in range(8):
        word |= pad[:, j, :] << np.uint32(4 * j)
    return word.view(np.int32)


def pack_nibbles_along_n(z: np.ndarray) -> np.ndarray:
    """z: uint8 [G, N] of values 0..15 -> int32 [G, ceil(N/8)], nibble n%8 of word [g, n//8] = z[g, n]."""
    G, N = z.shape
    cols = -(-N // 8)
    pad = np.zeros((G, cols * 8), np.uint32)
    pad[:, :N] = z
    pad = pad.reshape(G, cols, 8)
    word = np.zeros((G, cols), np.uint32)
    for j in range(8):
        word |= pad[:, :, j] << np.uint32(4 * j)
    return word.view(np.int32)


def random_gptq(K: int, N: int, group: int = 128, seed: int = 0, zeros: str = "7or8",
                rng: np.random.Generator | None = None) -> GptqTensors:
    """Random nibbles with the distributions of the single-linear benchmark case: qweight nibbles uniform
    on 0..15; stored zeros uniform on {7, 8} ("7or8"), all 7 ("sym"), uniform 0..15 ("any") or absent
    ("none"); scales |N(0.01, 0.003)| in fp16. Draw order: qweight, qzeros, scales."""
    rng = np.random.default_rng(seed) if rng is None else rng
    G = -(-K // group)
    q = rng.integers(0, 16, size=(K, N), dtype=np.uint8)
    if zeros == "7or8":
        z = rng.integers(7, 9, size=(G, N), dtype=np.uint8)
    elif zeros == "sym":
        z = np.full((G, N), 7, np.uint8)
    elif zeros == "any":
        z = rng.integers(0, 16, size=(G, N), dtype=np.uint8)
    elif zeros == "none":
        z = None
    else:
        raise ValueError(zeros)
    scales = np.abs(rng.normal(0.01, 0.003, size=(G, N))).astype(np.float16)
    return GptqTensors(pack_nibbles_along_k(q), None if z is None else pack_nibbles_along_n(z), scales, K, N, group)


def rtn_quantize(W: np.ndarray, group: int = 128) -> GptqTensors:
    """Round-to-nearest asymmetric int4 quantisation of W [N, K] (Linear layout [out, in]) into the GPTQ
    checkpoint format: per output column and per group of `group` input channels, scale = (max-min)/15
    (stored as fp16, and the fp16 value is what both sides use), zero = round(-min/scale) clipped so that
    the stored zero-1 fits a nibble, q = clip(round(w/scale) + zero, 0, 15)."""
    N, K = W.shape
    G = -(-K // group)
    Wt = np.zeros((G * group, N), np.float32)
    Wt[:K] = W.T
    Wg = Wt.reshape(G, group, N)
    if K % group:
        # padded channels must not widen the range of the last group
        valid = (np.arange(G * group) < K).reshape(G, group, 1)
        lo = np.where(valid, Wg, np.inf).min(axis=1)
        hi = np.where(valid, Wg, -np.inf).max(axis=1)
    else:
        lo, hi = Wg.min(axis=1), Wg.max(axis=1)
    lo, hi = np.minimum(lo, 0), np.maximum(hi, 0)
    scale = ((hi - lo) / 15.0).astype(np.float16)
    scale = np.where(scale == 0, np.float16(1e-4), scale).astype(np.float16)
    s32 = scale.astype(np.float32)
    zero = np.clip(np.rint(-lo / s32), 1, 16)
    q = np.clip(np.rint(Wg / s32[:, None, :]) + zero[:, None, :], 0, 15).astype(np.uint8)
    q = q.reshape(G * group, N)[:K]
    return GptqTensors(pack_nibbles_along_k(q), pack_nibbles_along_n((zero - 1).astype(np.uint8)), scale, K, N, group)


def dequant_numpy(t: GptqTensors) -> np.ndarray:
    """Plain numpy evaluation of w[n,k] = (q - (z+1)) * scale, f32 [N, K]: a vectorised way to expand
    large synthetic models on the host (for CPU baselines and test inputs)."""
    K, N, g = t.in_features, t.out_features, t.group_size
    qw = t.qweight.view(np.uint32)
    q = np.stack([(qw >> np.uint32(4 * j)) & np.uint32(15) for j in range(8)], axis=1).reshape(-1, N)[:K].astype(np.int32)
    grp = np.arange(K) // g
    if t.qzeros is None:
        z = np.full((qw.shape[0] * 8 // g + 1, N), 8, np.int32)
    else:
        zw = t.qzeros.view(np.uint32)
        z = np.stack([(zw >> np.uint32(4 * j)) & np.uint32(15) for j in range(8)], axis=2).reshape(zw.shape[0], -1)[:, :N].astype(np.int32) + 1
    s = t.scales.astype(np.float32)
    return ((q - z[grp]).astype(np.float32) * s[grp]).T.copy()


@dataclass
class QwenShape:
    """``QwenConfig`` (src/model/qwen-config.ts:12-28)."""
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


# QWEN25_05B (src/model/qwen-config.ts:44-54)
QWEN25_05B = QwenShape(151936, 24, 14, 2, 896, 4864)

_PROJ = (("q", "n_embd", "n_embd"), ("k", "n_embd", "kv_dim"), ("v", "n_embd", "kv_dim"), ("o", "n_embd", "n_embd"),
         ("gate", "n_embd", "intermediate"), ("up", "n_embd", "intermediate"), ("down", "intermediate", "n_embd"))


def random_qwen_gptq(cfg: QwenShape, seed: int = 0, group: int = 128, std: float = 0.02) -> dict:
    """A random Qwen2-shaped GPTQ checkpoint: every projection N(0, std) quantised by RTN; fp16 embedding
    (tied lm_head) N(0, std); q/k/v biases N(0, std); norm weights 1 + N(0, 0.02), as f32.

    Returns {"embed": fp16 [V, C], "final_norm": f32 [C], "layers": [{"q": GptqTensors, ..., "q_bias": f32,
    "k_bias", "v_bias", "input_norm", "post_norm"}]}.
    """
    rng = np.random.default_rng(seed)
    out = {"embed": rng.normal(0, std, size=(cfg.vocab_size, cfg.n_embd)).astype(np.float16),
           "final_norm": (1 + rng.normal(0, 0.02, size=cfg.n_embd)).astype(np.float32), "layers": []}
    for _ in range(cfg.n_layer):
        L = {}
        for name, kin, kout in _PROJ:
            K, N = getattr(cfg, kin), getattr(cfg, kout)
            L[name] = rtn_quantize(rng.normal(0, std, size=(N, K)).astype(np.float32), group)
        for name, dim in (("q_bias", cfg.n_embd), ("k_bias", cfg.kv_dim), ("v_bias", cfg.kv_dim)):
            L[name] = rng.normal(0, std, size=dim).astype(np.float32)
        L["input_norm"] = (1 + rng.normal(0, 0.02, size=cfg.n_embd)).astype(np.float32)
        L["post_norm"] = (1 + rng.normal(0, 0.02, size=cfg.n_embd)).astype(np.float32)
        out["layers"].append(L)
    return out
