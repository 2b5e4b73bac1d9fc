"""``generateQwen`` and ``sampleToken`` (src/infer/qwen-generate.ts:29-84, src/infer/sampler.ts:18-79)."""
from __future__ import annotations

import math
import random
import time
from dataclasses import dataclass, field

import numpy as np

from .qwen import QwenGpt


@dataclass
class SamplerOptions:
    """``SamplerOptions`` (src/infer/sampler.ts:3-12) plus ``stop_tokens`` of ``QwenGenerateOptions``."""
    temperature: float = 1.0
    top_k: int = 0
    top_p: float = 1.0
    rng: object = None
    stop_tokens: list = field(default_factory=list)


def sample_token(logits: np.ndarray, offset: int, vocab_size: int, options: SamplerOptions | None = None) -> int:
    """``sampleToken``: greedy (first strict maximum) when temperature <= 0, else temperature / top-k /
    top-p sampling with the reference's order of operations."""
    options = options or SamplerOptions()
    if vocab_size <= 0:
        raise ValueError("sampleToken: vocabSize 必须为正")
    if offset < 0 or offset + vocab_size > logits.size:
        raise ValueError(f"sampleToken: logits 越界 offset={offset} vocab={vocab_size}")
    row = np.asarray(logits, np.float32).ravel()[offset:offset + vocab_size]
    if not (options.temperature > 0):
        best = 0
        # np.argmax returns the first maximum; NaNs never win in the reference's strict comparison
        clean = np.where(np.isnan(row), -np.inf, row)
        best = int(np.argmax(clean)) if not np.isnan(row[0]) else 0
        return best
    scaled = (row / np.float32(options.temperature)).astype(np.float32)
    weights = np.exp((scaled - scaled.max()).astype(np.float64)).astype(np.float32)
    total = float(weights.astype(np.float64).sum())
    order = sorted(range(vocab_size), key=lambda i: -float(weights[i]))  # stable, like Array.prototype.sort
    limit = min(vocab_size, max(1, int(math.floor(options.top_k)))) if options.top_k > 0 else vocab_size
    kept = order[:limit]
    if options.top_p < 1:
        cum, cut = 0.0, kept
        for i, idx in enumerate(kept):
            cum += float(weights[idx]) / total
            if cum >= options.top_p:
                cut = kept[:i + 1]
                break
        kept = cut
    kept_sum = sum(float(weights[i]) for i in kept)
    r = (options.rng or random.random)() * kept_sum
    acc = 0.0
    for idx in kept:
        acc += float(weights[idx])
        if acc >= r:
            return idx
    return kept[-1]


@dataclass
class QwenGenerateResult:
    ids: list
    prompt_length: int
    generated: int
    tokens_per_second: float
    prefill_ms: float


def generate_qwen(model: QwenGpt, config, prompt: list, max_new_tokens: int, options: SamplerOptions | None = None,
                  on_device: bool | None = None) -> QwenGenerateResult:
    """``generateQwen``: one prefill, then one decode step per token.

    Greedy decoding without stop tokens runs entirely on the device (``decode_greedy``: argmax and token
    feedback inside a replayed CUDA graph) unless ``on_device=False``; every other option takes the
    reference's loop: read the logits row back, sample on the host, feed the token."""
    options = options or SamplerOptions()
    if len(prompt) == 0:
        raise ValueError("generateQwen: prompt 不能为空")
    if max_new_tokens <= 0:
        raise ValueError("generateQwen: maxNewTokens 必须为正")
    if len(prompt) > model.max_t:
        raise ValueError(f"generateQwen: prompt 长度 {len(prompt)} 超过 blockSize={model.max_t}")
    stop = set(options.stop_tokens or [])
    context = list(prompt)
    vocab = config.vocab_size
    model.reset_cache()

    t0 = time.perf_counter()
    logits = model.prefill(np.asarray(prompt, np.uint32), last_only=True)
    row = model.read_tensor_slice(logits, 0, vocab)
    prefill_ms = (time.perf_counter() - t0) * 1e3

    t1 = time.perf_counter()
    generated = 0
    nxt = sample_token(row, 0, vocab, options)
    greedy = not (options.temperature > 0)
    if on_device is None:
        on_device = greedy and not stop
    if on_device and greedy and not stop and max_new_tokens > 1 and nxt not in stop:
        # token 1 is `nxt`; tokens 2..max_new come from max_new-1 device steps
        rest = model.decode_greedy(nxt, max_new_tokens - 1)
        context.append(nxt)
        context.extend(int(t) for t in rest)
        generated = max_new_tokens
    else:
        while generated < max_new_tokens and nxt not in stop:
            context.append(nxt)
            generated += 1
            if generated >= max_new_tokens:
                break
            logits = model.decode_step(nxt)
            row = model.read_tensor_slice(logits, 0, vocab)
            nxt = sample_token(row, 0, vocab, options)
    seconds = max(1e-6, time.perf_counter() - t1)
    return QwenGenerateResult(context, len(prompt), generated, generated / seconds, prefill_ms)
