// GPTQ int4 -> dense [N, K] export (f32 and fp16). Replaces the CPU triple loop of dequantizeGptqInt4
// (src/weights/quant.ts:82-115) and the f32 -> fp16 conversion of writeF16 (src/gpu/buffer.ts:103-120).
//
// w[n, k] = (q - zero) * scale[g, n], zero = stored nibble + 1 (no wrap: 15 -> 16), or 8 when the
// checkpoint has no qzeros. q - zero is an integer in [-16, 14] and scale an fp16 value, so the product
// has at most 16 significant bits: the single f32 multiply below is exact and therefore equal to the
// reference's double-precision product rounded to f32.
//
// HBM-bound transpose: a block reads a 32 (packed rows) x 32 (columns) tile of words with 128-byte
// coalesced rows, passes it through shared memory, and each warp then writes one output row segment of
// 256 consecutive k (1 KB f32 / 512 B fp16).
#include "common.cuh"

namespace wb {

template <bool F16>
__global__ void __launch_bounds__(256) gptq_dequant_kernel(const uint32_t *__restrict__ qw,
                                                           const uint32_t *__restrict__ qz,
                                                           const __half *__restrict__ sc, void *__restrict__ out,
                                                           int64_t K, int64_t N, int64_t pack_rows, int64_t group,
                                                           int64_t zcols)
{
    __shared__ uint32_t tile[32][33];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t n0 = (int64_t)blockIdx.x * 32, r0 = (int64_t)blockIdx.y * 32;

    for (int i = warp; i < 32; i += 8) {
        const int64_t r = r0 + i, n = n0 + lane;
        tile[i][lane] = (r < pack_rows && n < N) ? qw[r * N + n] : 0u;
    }
    __syncthreads();

    for (int c = warp; c < 32; c += 8) {
        const int64_t n = n0 + c, r = r0 + lane;
        if (n >= N || r >= pack_rows) continue;
        const uint32_t word = tile[lane][c];
        const int64_t g = (r * 8) / group;
        const float scale = __half2float(sc[g * N + n]);
        int zero = 8;
        if (qz) zero = (int)((qz[g * zcols + (n >> 3)] >> (4 * (n & 7))) & 15u) + 1;
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; j++) v[j] = (float)((int)((word >> (4 * j)) & 15u) - zero) * scale;
        const int64_t k0 = r * 8;
        if constexpr (F16) {
            unsigned short *o = (unsigned short *)out + n * K + k0;
            if ((K & 7) == 0) {
                uint4 p;
                p.x = f32_to_f16_bits_ref(v[0]) | ((uint32_t)f32_to_f16_bits_ref(v[1]) << 16);
                p.y = f32_to_f16_bits_ref(v[2]) | ((uint32_t)f32_to_f16_bits_ref(v[3]) << 16);
                p.z = f32_to_f16_bits_ref(v[4]) | ((uint32_t)f32_to_f16_bits_ref(v[5]) << 16);
                p.w = f32_to_f16_bits_ref(v[6]) | ((uint32_t)f32_to_f16_bits_ref(v[7]) << 16);
                *(uint4 *)o = p;
            } else {
#pragma unroll
                for (int j = 0; j < 8; j++)
                    if (k0 + j < K) o[j] = f32_to_f16_bits_ref(v[j]);
            }
        } else {
            float *o = (float *)out + n * K + k0;
            if ((K & 7) == 0) {
                *(float4 *)o = make_float4(v[0], v[1], v[2], v[3]);
                *(float4 *)(o + 4) = make_float4(v[4], v[5], v[6], v[7]);
            } else {
#pragma unroll
                for (int j = 0; j < 8; j++)
                    if (k0 + j < K) o[j] = v[j];
            }
        }
    }
}

int launch_dequant(wb_context *ctx, const Weight &w, void *out, bool f16)
{
    const char *base = ctx->arena[WB_ARENA_WEIGHTS].base;
    const uint32_t *qw = (const uint32_t *)(base + w.off_main);
    const uint32_t *qz = w.has_zeros ? (const uint32_t *)(base + w.off_zeros) : nullptr;
    const __half *sc = (const __half *)(base + w.off_scales);
    dim3 grid((unsigned)((w.N + 31) / 32), (unsigned)((w.pack_rows + 31) / 32));
    if (f16)
        gptq_dequant_kernel<true><<<grid, 256, 0, ctx->stream>>>(qw, qz, sc, out, w.K, w.N, w.pack_rows, w.group, w.zcols);
    else
        gptq_dequant_kernel<false><<<grid, 256, 0, ctx->stream>>>(qw, qz, sc, out, w.K, w.N, w.pack_rows, w.group, w.zcols);
    ctx->launches++;
    WB_CUDA(cudaGetLastError());
    return WB_OK;
}

}  // namespace wb
