// Prefill attention on the tensor cores: causal GQA attention of many query rows against the KV cache,
// attention_gqa_cache.wgsl (attentionGqaRef, src/reference/qwen-ref.ts:67-116) for M >= 16 rows in the default
// (fp16-operand) mode. The scalar kernel in qwen_ops.cu stays the path for the fp32-activation mode, for head sizes
// other than 64 / 128 and for the uncached forward.
//
// One CTA = 4 warps = 64 query rows of one head; a warp owns 16 rows. Keys are walked in blocks of 64: the K and V
// rows of a block are staged in shared memory as fp16 (cp.async straight from an fp16 cache, double-buffered; an f32
// cache is converted on the way), S = Q K^T and O += P V run on the warp-level MMA (m16n8k16, fp16 operands, f32
// accumulate), and the softmax is the online form in f32 registers: per row a running maximum and sum, the
// accumulator rescaled when the maximum moves. The accumulator fragments of S are, element for element, the A
// fragments of the P V product, so P never leaves the registers; V is read transposed with ldmatrix.
// A query row r sees keys [0, past + r]; blocks past a warp's last row are skipped by that warp, and only the blocks
// that straddle the diagonal pay for the mask. Heavy row blocks (late rows, many keys) are scheduled first.
#include "qwen_ops.cuh"
#include "gemv_core.cuh"

namespace wb {

namespace {

constexpr int kQRows = 64;   // query rows per CTA
constexpr int kKeys = 64;    // keys per block

__device__ __forceinline__ void cp16(void *dst_smem, const void *src)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst_smem)), "l"(src) : "memory");
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void *smem_row)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"((uint32_t)__cvta_generic_to_shared(smem_row)));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void *smem_row)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"((uint32_t)__cvta_generic_to_shared(smem_row)));
}

__device__ __forceinline__ uint32_t pack_h2(float a, float b) { return h2_as_u32(__floats2half2_rn(a, b)); }

// 2^x by the special-function unit (the softmax only needs a few ulp: its weights are rounded to fp16 next)
__device__ __forceinline__ float ex2(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Stages keys [key0, key0 + 64) of one KV head into `dst` ([64][D + 8] halves); rows at or past n_keys become zeros.
// A thread copies the same pieces of every block (piece u: row (tid + 128 u) / (D / 8), 16 bytes), so the offsets are
// computed once by the caller: dst_off[u] in halves, src_off[u] in elements of the cache row.
template <typename KV, int D>
__device__ __forceinline__ void stage_block(__half *dst, const KV *src, int key0, int n_keys, int kv_ld, const int (&dst_off)[D / 16],
                                            const int (&src_off)[D / 16], const int (&row)[D / 16])
{
    const KV *base = src + (int64_t)key0 * kv_ld;
    const bool whole = key0 + kKeys <= n_keys;
#pragma unroll
    for (int u = 0; u < D / 16; u++) {
        __half *d = dst + dst_off[u];
        if (whole || key0 + row[u] < n_keys) {
            const KV *sp = base + src_off[u];
            if constexpr (sizeof(KV) == 2) {
                cp16(d, sp);
            } else {
                const float4 a = *reinterpret_cast<const float4 *>(sp), b = *reinterpret_cast<const float4 *>(sp + 4);
                uint4 o;
                o.x = pack_h2(a.x, a.y), o.y = pack_h2(a.z, a.w), o.z = pack_h2(b.x, b.y), o.w = pack_h2(b.z, b.w);
                *reinterpret_cast<uint4 *>(d) = o;
            }
        } else {
            *reinterpret_cast<uint4 *>(d) = make_uint4(0, 0, 0, 0);
        }
    }
}

template <typename KV, int D>
__global__ void __launch_bounds__(128, D == 64 ? 4 : 2) attention_prefill_mma_kernel(const float *__restrict__ q, const KV *__restrict__ kmem,
                                                                    const KV *__restrict__ vmem, float *__restrict__ out,
                                                                    __half *__restrict__ out16, int M, int H, int KVH,
                                                                    const int *__restrict__ past_ptr, int past_imm, int ldq,
                                                                    int kv_ld, float scale)
{
    pdl_sync();
    constexpr int LD = D + 8;     // padded row of a staged block, in halves: rows 16 bytes apart modulo 128
    constexpr int KS = D / 16;    // k-steps of Q K^T
    constexpr int DT = D / 8;     // 8-wide tiles of the head dimension
    extern __shared__ uint4 smem_u4[];
    __half *Ks = reinterpret_cast<__half *>(smem_u4);       // [2][64][LD]
    __half *Vs = Ks + 2 * kKeys * LD;                        // [2][64][LD]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    const int rb = (int)gridDim.x - 1 - (int)blockIdx.x;     // late (long) row blocks first
    const int h = blockIdx.y, kvh = h / (H / KVH);
    const int past = past_ptr ? *past_ptr : past_imm;
    const int r0 = rb * kQRows;
    const int n_keys = past + M;                             // rows of the cache that exist
    const int last_row = min(r0 + kQRows, M) - 1;
    const int n_blocks = (past + last_row) / kKeys + 1;
    const KV *kbase = kmem + kvh * D, *vbase = vmem + kvh * D;

    // this thread's pieces of a staged block: 64 rows x D / 8 pieces of 16 bytes over 128 threads
    int st_dst[D / 16], st_src[D / 16], st_row[D / 16];
#pragma unroll
    for (int u = 0; u < D / 16; u++) {
        const int i = tid + 128 * u, r = i / (D / 8), c = (i - r * (D / 8)) * 8;
        st_row[u] = r, st_dst[u] = r * LD + c, st_src[u] = r * kv_ld + c;
    }
    // first block on its way while the Q fragments are loaded
    stage_block<KV, D>(Ks, kbase, 0, n_keys, kv_ld, st_dst, st_src, st_row);
    stage_block<KV, D>(Vs, vbase, 0, n_keys, kv_ld, st_dst, st_src, st_row);
    cp_async_commit();

    // Q fragments of this warp's 16 rows (rows g and g + 8 of the tile), fp16, kept for the whole kernel
    const int row_a = r0 + warp * 16 + g, row_b = row_a + 8;
    uint32_t qa[KS][4];
    {
        const float *qa_p = q + (int64_t)row_a * ldq + h * D, *qb_p = q + (int64_t)row_b * ldq + h * D;
#pragma unroll
        for (int ks = 0; ks < KS; ks++) {
            const int d = ks * 16 + 2 * t;
            float2 a0 = make_float2(0.f, 0.f), a1 = a0, a2 = a0, a3 = a0;
            if (row_a < M) a0 = *reinterpret_cast<const float2 *>(qa_p + d), a2 = *reinterpret_cast<const float2 *>(qa_p + d + 8);
            if (row_b < M) a1 = *reinterpret_cast<const float2 *>(qb_p + d), a3 = *reinterpret_cast<const float2 *>(qb_p + d + 8);
            qa[ks][0] = pack_h2(a0.x, a0.y), qa[ks][1] = pack_h2(a1.x, a1.y);
            qa[ks][2] = pack_h2(a2.x, a2.y), qa[ks][3] = pack_h2(a3.x, a3.y);
        }
    }
    float o[DT][4];
#pragma unroll
    for (int j = 0; j < DT; j++) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const int warp_last_key = past + min(r0 + warp * 16 + 15, M - 1);  // the last key any row of this warp sees
    const float sl2 = scale * 1.4426950408889634f;                     // scores are kept in units of log2(e)

    for (int kb = 0; kb < n_blocks; kb++) {
        const int buf = kb & 1;
        if (kb + 1 < n_blocks) {  // next block into the other buffer (its last readers passed the barrier below)
            stage_block<KV, D>(Ks + (buf ^ 1) * kKeys * LD, kbase, (kb + 1) * kKeys, n_keys, kv_ld, st_dst, st_src, st_row);
            stage_block<KV, D>(Vs + (buf ^ 1) * kKeys * LD, vbase, (kb + 1) * kKeys, n_keys, kv_ld, st_dst, st_src, st_row);
        }
        cp_async_commit();
        cp_async_wait(1);  // everything but the newest group: block kb has landed
        __syncthreads();
        const int key0 = kb * kKeys;
        if (key0 <= warp_last_key && r0 + warp * 16 < M) {
            const __half *Kb = Ks + buf * kKeys * LD, *Vb = Vs + buf * kKeys * LD;
            // ---- S = Q K^T for 16 rows x 64 keys: 8 key tiles x KS k-steps; one ldmatrix.x4 brings the K fragments of
            // two k-steps of a key tile (lanes 0-7 / 8-15 address d 0..7 / 8..15 of k-step ks, lanes 16-31 of ks + 1)
            float s[8][4];
            const __half *klane = Kb + (lane & 7) * LD + (lane >> 3) * 8;
#pragma unroll
            for (int j = 0; j < 8; j++) {
                s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
                for (int ks = 0; ks < KS; ks += 2) {
                    uint32_t kf[4];
                    ldmatrix_x4(kf, klane + j * 8 * LD + ks * 16);
                    mma_16816(s[j], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], kf[0], kf[1]);
                    mma_16816(s[j], qa[ks + 1][0], qa[ks + 1][1], qa[ks + 1][2], qa[ks + 1][3], kf[2], kf[3]);
                }
            }
            // ---- mask (only blocks that reach past the first row's diagonal), running maximum of the raw scores (the
            // scale is positive, so it commutes with the maximum and is folded into the exponent's multiply-add)
            const bool need_mask = key0 + kKeys - 1 > past + r0 + warp * 16;
            if (need_mask) {
                const int lim_a = past + row_a, lim_b = past + row_b;  // last visible key of rows g / g + 8
#pragma unroll
                for (int j = 0; j < 8; j++) {
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const int key = key0 + j * 8 + 2 * t + (i & 1);
                        if (key > ((i & 2) ? lim_b : lim_a)) s[j][i] = -INFINITY;
                    }
                }
            }
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int j = 0; j < 8; j++) {
                mx[0] = fmaxf(mx[0], fmaxf(s[j][0], s[j][1]));
                mx[1] = fmaxf(mx[1], fmaxf(s[j][2], s[j][3]));
            }
            float alpha[2], neg_m[2];  // neg_m: minus the running maximum, in units of log2(e) / sqrt(D)
#pragma unroll
            for (int r = 0; r < 2; r++) {
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
                const float m_new = fmaxf(m_run[r], mx[r]);
                const float m_use = m_new == -INFINITY ? 0.f : m_new;  // a row with no visible key yet (rows past M): keep zeros, no NaN
                alpha[r] = ex2((m_run[r] - m_use) * sl2);
                neg_m[r] = -m_use * sl2;
                m_run[r] = m_new;
                l_run[r] *= alpha[r];
            }
#pragma unroll
            for (int j = 0; j < DT; j++) o[j][0] *= alpha[0], o[j][1] *= alpha[0], o[j][2] *= alpha[1], o[j][3] *= alpha[1];
            // ---- P = 2^(S sl2 - m), packed as the A fragments of P V; row sums stay per thread until the end
            uint32_t pa[4][4];
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const float p0 = ex2(fmaf(s[j][0], sl2, neg_m[0])), p1 = ex2(fmaf(s[j][1], sl2, neg_m[0]));
                const float p2 = ex2(fmaf(s[j][2], sl2, neg_m[1])), p3 = ex2(fmaf(s[j][3], sl2, neg_m[1]));
                l_run[0] += p0 + p1, l_run[1] += p2 + p3;
                pa[j >> 1][(j & 1) * 2] = pack_h2(p0, p1);       // a0 / a2: row g, keys 16 kk + 2t (+8)
                pa[j >> 1][(j & 1) * 2 + 1] = pack_h2(p2, p3);   // a1 / a3: row g + 8
            }
            // ---- O += P V: 4 key steps of 16 x DT head-dimension tiles; V transposed by ldmatrix
#pragma unroll
            for (int kk = 0; kk < 4; kk++) {
                // lanes 0-7 / 8-15 address keys 16 kk + 0..7 / + 8..15 of tile jd, lanes 16-31 the same keys of tile jd + 1
                const __half *vrow = Vb + (kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * LD + (lane >> 4) * 8;
#pragma unroll
                for (int jd = 0; jd < DT; jd += 2) {
                    uint32_t vb[4];
                    ldmatrix_x4_trans(vb, vrow + jd * 8);
                    mma_16816(o[jd], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], vb[0], vb[1]);
                    mma_16816(o[jd + 1], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], vb[2], vb[3]);
                }
            }
        }
        __syncthreads();  // block kb's buffer is refilled by the next iteration's staging
    }
    cp_async_wait(0);
    // ---- normalise and store (f32)
#pragma unroll
    for (int r = 0; r < 2; r++) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
    const float inv_a = l_run[0] > 0.f ? 1.f / l_run[0] : 0.f, inv_b = l_run[1] > 0.f ? 1.f / l_run[1] : 0.f;
    const int64_t ia = (int64_t)row_a * (H * D) + h * D + 2 * t, ib = (int64_t)row_b * (H * D) + h * D + 2 * t;
#pragma unroll
    for (int j = 0; j < DT; j++) {
        if (out16) {  // the o projection is a tensor-core GEMM: it takes the fp16 value it would round to itself
            if (row_a < M) *reinterpret_cast<uint32_t *>(out16 + ia + j * 8) = pack_h2(o[j][0] * inv_a, o[j][1] * inv_a);
            if (row_b < M) *reinterpret_cast<uint32_t *>(out16 + ib + j * 8) = pack_h2(o[j][2] * inv_b, o[j][3] * inv_b);
        } else {
            if (row_a < M) *reinterpret_cast<float2 *>(out + ia + j * 8) = make_float2(o[j][0] * inv_a, o[j][1] * inv_a);
            if (row_b < M) *reinterpret_cast<float2 *>(out + ib + j * 8) = make_float2(o[j][2] * inv_b, o[j][3] * inv_b);
        }
    }
}

template <typename KV, int D>
cudaError_t launch_prefill(cudaStream_t st, const float *q, const void *kmem, const void *vmem, float *out, __half *out16, int M, int H,
                           int KVH, const int *past_ptr, int past_imm, int ldq, int kv_ld)
{
    const size_t smem = (size_t)4 * kKeys * (D + 8) * sizeof(__half);
    auto kern = attention_prefill_mma_kernel<KV, D>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    const dim3 grid((unsigned)((M + kQRows - 1) / kQRows), (unsigned)H);
    return launch_pdl(kern, grid, dim3(128), smem, st, q, (const KV *)kmem, (const KV *)vmem, out, out16, M, H, KVH, past_ptr, past_imm,
                      ldq, kv_ld, 1.0f / sqrtf((float)D));
}

}  // namespace

bool op_attention_prefill_supported(int M, int H, int KVH, int D, int ldq, int kv_ld)
{
    return M >= 16 && (D == 64 || D == 128) && KVH > 0 && H % KVH == 0 && ldq % 2 == 0 && kv_ld % 8 == 0;
}

int op_attention_prefill(wb_context *ctx, const float *q, const void *kmem, const void *vmem, int kv_f16, float *out, int M, int H,
                         int KVH, int D, const int *past_ptr, int past_imm, int ldq, int kv_ld, __half *out16)
{
    if (!op_attention_prefill_supported(M, H, KVH, D, ldq, kv_ld))
        return fail(WB_ERR_UNSUPPORTED, "tensor-core prefill attention needs M >= 16 and a head size of 64 or 128");
    cudaError_t e;
    if (D == 64)
        e = kv_f16 ? launch_prefill<__half, 64>(ctx->stream, q, kmem, vmem, out, out16, M, H, KVH, past_ptr, past_imm, ldq, kv_ld)
                   : launch_prefill<float, 64>(ctx->stream, q, kmem, vmem, out, out16, M, H, KVH, past_ptr, past_imm, ldq, kv_ld);
    else
        e = kv_f16 ? launch_prefill<__half, 128>(ctx->stream, q, kmem, vmem, out, out16, M, H, KVH, past_ptr, past_imm, ldq, kv_ld)
                   : launch_prefill<float, 128>(ctx->stream, q, kmem, vmem, out, out16, M, H, KVH, past_ptr, past_imm, ldq, kv_ld);
    ctx->launches++;
    WB_CUDA(e);
    return WB_OK;
}

}  // namespace wb
