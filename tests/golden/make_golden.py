"""Regenerates ``tests/golden/*.json``: run ``python tests/golden/make_golden.py``.

The reference is TypeScript and no JavaScript engine is available, so these vectors are NOT outputs of
the reference run here. They are the reference's own formula-defined test vectors, evaluated by this
script in pure Python / numpy float64, independently of the C oracle:

  weights_kat      the closed-form GPTQ known-answer test of src/tests/qwen/weights.ts:62-137
                   (in=16, out=5, group=8, q[o][i] = (o*7+i*3)&15, scale[g][o] = 0.01(g+1)(o+1),
                   stored zero 7; want = (q-8)*scale), plus the same with qzeros omitted.
  rng              first outputs of makeRng(seed) (xorshift32 13/17/5, src/reference/cpu-ref.ts:57-67)
                   for the seeds the reference's GEMV tests use.
  gemv_cases       inputs of testGemmGemvF16 / testGemmGemvSplitF16 / testGemmNtF16
                   (src/tests/kernels.ts:1261-1269, 1378-1400, 545-585) regenerated from that RNG in
                   the reference's draw order, with expected outputs by float64 dot products
                   (gemmNTRef's arithmetic: double accumulate, bias added in double, one f32 rounding).
  f16              a table of f32 -> fp16 bit patterns covering ties, subnormals, overflow, NaN and the
                   reference's flush of |x| < 2^-24 (src/gpu/buffer.ts:57-100), written out by hand.
"""
import json
import struct
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent


def make_rng(seed):
    state = (seed & 0xFFFFFFFF) or 1

    def nxt():
        nonlocal state
        state ^= (state << 13) & 0xFFFFFFFF
        state ^= state >> 17
        state ^= (state << 5) & 0xFFFFFFFF
        return state / 4294967296.0
    return nxt


def random_f32(n, rng):
    return np.array([np.float32(rng() * 2 - 1) for _ in range(n)], np.float32)


def f32_bits(x):
    return struct.unpack("<I", struct.pack("<f", float(x)))[0]


def gemm_f64(A, W, M, N, K, bias):
    C = A.reshape(M, K).astype(np.float64) @ W.reshape(N, K).astype(np.float64).T
    if bias is not None:
        C = C + bias.astype(np.float64)[None, :]
    return C.astype(np.float32)


def weights_kat():
    inF, outF, g, pack = 16, 5, 8, 8
    q = [[(o * 7 + i * 3) & 15 for i in range(inF)] for o in range(outF)]
    scales = np.zeros((inF // g, outF), np.float32)
    for gi in range(inF // g):
        for o in range(outF):
            scales[gi, o] = np.float32(0.01 * (gi + 1) * (o + 1))
    qweight = []
    for p in range(inF // pack):
        for o in range(outF):
            word = 0
            for k in range(pack):
                word |= (q[o][p * pack + k] & 15) << (4 * k)
            qweight.append(word)
    zero_cols = -(-outF // pack)
    qzeros = [0x77777777] * ((inF // g) * zero_cols)
    want = np.zeros((outF, inF), np.float32)
    for o in range(outF):
        for i in range(inF):
            want[o, i] = np.float32((q[o][i] - 8) * float(scales[i // g, o]))
    return {"in": inF, "out": outF, "group": g, "qweight_u32": qweight, "qzeros_u32": qzeros,
            "scales_f32_bits": [f32_bits(v) for v in scales.ravel()], "want_f32_bits": [f32_bits(v) for v in want.ravel()]}


def gemv_cases():
    from numpy import float16
    cases = []

    def add(kind, M, N, K, seed, S=None, round_a=False):
        rng = make_rng(seed)
        A = random_f32(M * K, rng)
        B = random_f32(N * K, rng)
        bias = random_f32(N, rng)
        if round_a:
            A = A.astype(float16).astype(np.float32)
        B = B.astype(float16).astype(np.float32)  # roundF16
        cases.append({"kind": kind, "M": M, "N": N, "K": K, "seed": seed, "S": S, "round_a": round_a,
                      "a_head_bits": [f32_bits(v) for v in A[:4]], "b_head_bits": [f32_bits(v) for v in B[:4]],
                      "want_bias_bits": [f32_bits(v) for v in gemm_f64(A, B, M, N, K, bias).ravel()],
                      "want_nobias_bits": [f32_bits(v) for v in gemm_f64(A, B, M, N, K, None).ravel()]})

    for N, K in ((53, 42), (64, 896)):
        add("gemv", 1, N, K, 0x9E00 + N)
    for N, K, S in ((53, 42, 3), (128, 896, 8), (64, 896, 4)):
        add("split", 1, N, K, 0x5E10 + N * 31 + S, S)
    add("gemm_nt_f16", 37, 53, 41, 333, round_a=True)
    return cases


F16_TABLE = [  # (f32 bits, fp16 bits) under the reference's f32ToF16Bits
    (0x00000000, 0x0000), (0x80000000, 0x8000), (0x3F800000, 0x3C00), (0xBF000000, 0xB800),
    (0x477FE000, 0x7BFF), (0x477FF000, 0x7C00), (0x47800000, 0x7C00), (0x7F800000, 0x7C00), (0xFF800000, 0xFC00),
    (0x7FC00000, 0x7E00), (0xFFC12345, 0x7E00),
    (0x3F801000, 0x3C00), (0x3F801001, 0x3C01), (0x3F803000, 0x3C02),  # ties to even / just above
    (0x38800000, 0x0400), (0x387FE000, 0x0400), (0x387FA000, 0x03FE),  # min normal, subnormal ties to even (0x3FF.5 -> 0x400, 0x3FE.5 -> 0x3FE)
    (0x33800000, 0x0001), (0x33C00000, 0x0002), (0x34000000, 0x0002),  # 2^-24, 1.5*2^-24 ties up to even 2, 2^-23
    (0x33000000, 0x0000), (0x337FFFFF, 0x0000), (0xB3400000, 0x8000),  # [2^-25, 2^-24) flushes to signed zero in the reference
    (0x00000001, 0x0000),
]


def main():
    out = {"weights_kat": weights_kat(), "gemv_cases": gemv_cases(), "f16_table": F16_TABLE}
    rng_out = {}
    for seed in (0x9E00 + 53, 0x9E00 + 64, 0x5E10 + 53 * 31 + 3, 333, 0, 1, 20241006, 0xBEEF):
        r = make_rng(seed)
        rng_out[str(seed)] = [repr(r()) for _ in range(6)]
    out["rng"] = rng_out
    (HERE / "reference_vectors.json").write_text(json.dumps(out))
    print("wrote", HERE / "reference_vectors.json", (HERE / "reference_vectors.json").stat().st_size, "bytes")


if __name__ == "__main__":
    main()
