// The non-linear steps either side of each projection in the Qwen2 forward pass. They replace the WGSL
// kernels embedding_f16, rmsnorm, rope_half, kv_store, attention_gqa(_cache), silu_mul and vec_add that
// QwenGpt.runForward dispatches between its gemm() calls (src/model/qwen.ts:391-489). All activations
// are f32, as in the reference; the KV cache is fp16 or f32.
#include "qwen_ops.cuh"

namespace wb {

// embedding_f16.wgsl: x[m, :] = f32(embed[token[m], :])
__global__ void embed_f16_kernel(const __half *__restrict__ table, const uint32_t *__restrict__ tokens,
                                 float *__restrict__ x, int M, int C, int vocab)
{
    pdl_sync();
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (int64_t)M * C) return;
    const int m = (int)(idx / C), c = (int)(idx - (int64_t)m * C);
    uint32_t tok = tokens[m];
    if (tok >= (uint32_t)vocab) tok = 0;  // ids are validated on the host; never read out of bounds
    x[idx] = __half2float(table[(int64_t)tok * C + c]);
}

__device__ __forceinline__ float block_sum(float v, float *red)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = 0.f;
    for (int i = 0; i < nw; i++) t += red[i];  // same order in every thread: deterministic
    __syncthreads();
    return t;
}

// rmsnorm.wgsl / rmsNormRef (src/reference/qwen-ref.ts:12-29): y = x / sqrt(mean(x^2) + eps) * w,
// optionally fused with the residual add that precedes it: x_out = x + delta (vec_add.wgsl).
// y16 != nullptr: the result is stored as fp16 instead (the next step is a tensor-core GEMM, which would round its
// f32 input to fp16 anyway: same values, one pass over the activations fewer).
__global__ void __launch_bounds__(256) rmsnorm_kernel(const float *__restrict__ x, const float *__restrict__ delta,
                                                      float *__restrict__ x_out, const float *__restrict__ w,
                                                      float *__restrict__ y, __half *__restrict__ y16, int D, float eps)
{
    pdl_sync();
    __shared__ float red[8];
    const int64_t base = (int64_t)blockIdx.x * D;
    float ss = 0.f;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float v = x[base + d];
        if (delta) {
            v += delta[base + d];
            x_out[base + d] = v;
        }
        ss = fmaf(v, v, ss);
    }
    const float rstd = rsqrtf(block_sum(ss, red) / (float)D + eps);
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        const float v = delta ? x_out[base + d] : x[base + d];
        const float r = v * rstd * w[d];
        if (y16) y16[base + d] = __float2half_rn(r);
        else y[base + d] = r;
    }
}

// The same for D % 4 == 0, D <= 4096: one pass, the row stays in registers (up to four float4 per thread).
__global__ void __launch_bounds__(256) rmsnorm_vec4_kernel(const float *__restrict__ x, const float *__restrict__ delta,
                                                           float *__restrict__ x_out, const float *__restrict__ w,
                                                           float *__restrict__ y, __half *__restrict__ y16, int D, float eps)
{
    pdl_sync();
    __shared__ float red[8];
    const int64_t base = (int64_t)blockIdx.x * D;
    const int q = D >> 2;
    float4 v[4];
    float ss = 0.f;
#pragma unroll
    for (int u = 0; u < 4; u++) {
        const int i = threadIdx.x + 256 * u;
        v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < q) {
            v[u] = *reinterpret_cast<const float4 *>(x + base + 4 * i);
            if (delta) {
                const float4 d = *reinterpret_cast<const float4 *>(delta + base + 4 * i);
                v[u].x += d.x, v[u].y += d.y, v[u].z += d.z, v[u].w += d.w;
                *reinterpret_cast<float4 *>(x_out + base + 4 * i) = v[u];
            }
            ss = fmaf(v[u].x, v[u].x, ss), ss = fmaf(v[u].y, v[u].y, ss), ss = fmaf(v[u].z, v[u].z, ss), ss = fmaf(v[u].w, v[u].w, ss);
        }
    }
    const float rstd = rsqrtf(block_sum(ss, red) / (float)D + eps);
#pragma unroll
    for (int u = 0; u < 4; u++) {
        const int i = threadIdx.x + 256 * u;
        if (i < q) {
            const float4 ww = *reinterpret_cast<const float4 *>(w + 4 * i);
            const float4 r = make_float4(v[u].x * rstd * ww.x, v[u].y * rstd * ww.y, v[u].z * rstd * ww.z, v[u].w * rstd * ww.w);
            if (y16) {
                const __half2 a = __floats2half2_rn(r.x, r.y), b = __floats2half2_rn(r.z, r.w);
                uint2 o;
                o.x = *reinterpret_cast<const uint32_t *>(&a), o.y = *reinterpret_cast<const uint32_t *>(&b);
                *reinterpret_cast<uint2 *>(y16 + base + 4 * i) = o;
            } else {
                *reinterpret_cast<float4 *>(y + base + 4 * i) = r;
            }
        }
    }
}

// vec_add.wgsl
__global__ void add_kernel(const float *__restrict__ a, const float *__restrict__ b, float *__restrict__ out, int64_t n)
{
    pdl_sync();
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = a[i] + b[i];
}

// silu_mul.wgsl / siluMulRef (src/reference/qwen-ref.ts:119-123): out = gate / (1 + exp(-gate)) * up.
// gate and up may be two column halves of one [M, 2I] tensor (fused gate_up projection): ld = row pitch.
__global__ void silu_mul_kernel(const float *__restrict__ gate, const float *__restrict__ up, float *__restrict__ out,
                                int M, int I, int ld)
{
    pdl_sync();
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (int64_t)M * I) return;
    const int m = (int)(idx / I), i = (int)(idx - (int64_t)m * I);
    const float g = gate[(int64_t)m * ld + i], u = up[(int64_t)m * ld + i];
    out[idx] = g / (1.f + expf(-g)) * u;
}

// The same, four values per thread (I and ld multiples of 4), result in f32 or, with out16, in fp16 for the tensor-core
// GEMM that follows (which would round the f32 value to fp16 itself: same values).
__global__ void __launch_bounds__(256) silu_mul_vec4_kernel(const float *__restrict__ gate, const float *__restrict__ up,
                                                            float *__restrict__ out, __half *__restrict__ out16, int M, int I, int ld)
{
    pdl_sync();
    const int q = I >> 2;
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (int64_t)M * q) return;
    const int m = (int)(idx / q), i = (int)(idx - (int64_t)m * q) * 4;
    const float4 g = *reinterpret_cast<const float4 *>(gate + (int64_t)m * ld + i);
    const float4 u = *reinterpret_cast<const float4 *>(up + (int64_t)m * ld + i);
    float4 r;
    r.x = g.x / (1.f + expf(-g.x)) * u.x, r.y = g.y / (1.f + expf(-g.y)) * u.y;
    r.z = g.z / (1.f + expf(-g.z)) * u.z, r.w = g.w / (1.f + expf(-g.w)) * u.w;
    if (out16) {
        const __half2 a = __floats2half2_rn(r.x, r.y), b = __floats2half2_rn(r.z, r.w);
        uint2 o;
        o.x = *reinterpret_cast<const uint32_t *>(&a), o.y = *reinterpret_cast<const uint32_t *>(&b);
        *reinterpret_cast<uint2 *>(out16 + (int64_t)m * I + i) = o;
    } else {
        *reinterpret_cast<float4 *>(out + (int64_t)m * I + i) = r;
    }
}

// rope_half.wgsl + kv_store.wgsl (ropeHalfRef, src/reference/qwen-ref.ts:35-64): HF rotate-half with
// pos = row % T + pos_offset; cos/sin come from a table computed in double on the host. q is rotated in
// place; k is rotated and, with v, appended to the cache rows [cache_row0 + row] (or written back in
// place when there is no cache).
template <typename KV>
__global__ void rope_kv_kernel(float *__restrict__ q, float *__restrict__ k, const float *__restrict__ v,
                               KV *__restrict__ k_cache, KV *__restrict__ v_cache, const float *__restrict__ cs_table,
                               int M, int H, int KVH, int D, int T, const int *__restrict__ pos_offset_ptr,
                               int pos_offset_imm, int ldq, int ldk, int ldv)
{
    pdl_sync();
    const int half = D >> 1;
    const int per_row = (H + 2 * KVH) * half;
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (int64_t)M * per_row) return;
    const int row = (int)(idx / per_row);
    int rem = (int)(idx - (int64_t)row * per_row);
    const int pos_offset = pos_offset_ptr ? *pos_offset_ptr : pos_offset_imm;
    const int pos = row % T + pos_offset;
    const int hh = rem / half, i = rem - hh * half;
    const float c = cs_table[((int64_t)pos * half + i) * 2], s = cs_table[((int64_t)pos * half + i) * 2 + 1];
    if (hh < H) {
        float *p = q + (int64_t)row * ldq + hh * D;
        const float x0 = p[i], x1 = p[i + half];
        p[i] = x0 * c - x1 * s;
        p[i + half] = x0 * s + x1 * c;
    } else if (hh < H + KVH) {
        const int kh = hh - H;
        float *p = k + (int64_t)row * ldk + kh * D;
        const float x0 = p[i], x1 = p[i + half];
        const float r0 = x0 * c - x1 * s, r1 = x0 * s + x1 * c;
        if (k_cache) {
            KV *dst = k_cache + ((int64_t)(pos_offset + row) * KVH + kh) * D;
            dst[i] = (KV)r0;
            dst[i + half] = (KV)r1;
        } else {
            p[i] = r0;
            p[i + half] = r1;
        }
    } else if (v_cache) {
        const int vh = hh - H - KVH;
        const float *p = v + (int64_t)row * ldv + vh * D;
        KV *dst = v_cache + ((int64_t)(pos_offset + row) * KVH + vh) * D;
        dst[i] = (KV)p[i];
        dst[i + half] = (KV)p[i + half];
    }
}

__device__ __forceinline__ float kv_load(const float *p) { return *p; }
__device__ __forceinline__ float kv_load(const __half *p) { return __half2float(*p); }

// attention_gqa_cache.wgsl / attention_gqa.wgsl (attentionGqaRef, src/reference/qwen-ref.ts:67-116): one
// block per (query row, head). Keys/values are rows of `kmem`/`vmem` with pitch kv_ld: the KV cache, or
// the current k/v tensors when there is no cache. Row r sees keys [key_row0(r), key_row0(r) + n_keys(r)):
//   cache:    key_row0 = 0,           n_keys = past + r + 1
//   no cache: key_row0 = (r / T) * T, n_keys = r % T + 1
// Unlike the reference kernel there is no 512-key cap: scores live in dynamic shared memory.
template <typename KV>
__global__ void __launch_bounds__(128) attention_kernel(const float *__restrict__ q, const KV *__restrict__ kmem,
                                                        const KV *__restrict__ vmem, float *__restrict__ out, int H,
                                                        int KVH, int D, int T, const int *__restrict__ past_ptr,
                                                        int past_imm, int use_cache, int ldq, int kv_ld, float scale)
{
    pdl_sync();
    extern __shared__ float sm[];  // [D] query, [n_keys] scores
    __shared__ float red[4];
    const int row = blockIdx.x, h = blockIdx.y, kvh = h / (H / KVH);
    const int past = past_ptr ? *past_ptr : past_imm;
    const int key_row0 = use_cache ? 0 : (row / T) * T;
    const int n_keys = use_cache ? past + row + 1 : row % T + 1;
    float *qs = sm, *sc = sm + D;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    for (int d = threadIdx.x; d < D; d += blockDim.x) qs[d] = q[(int64_t)row * ldq + h * D + d];
    __syncthreads();

    // scores: one warp per key, lanes stride the head dimension
    float lmax = -INFINITY;
    for (int s = warp; s < n_keys; s += nw) {
        const KV *kp = kmem + (int64_t)(key_row0 + s) * kv_ld + kvh * D;
        float dot = 0.f;
        for (int d = lane; d < D; d += 32) dot = fmaf(qs[d], kv_load(kp + d), dot);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
        dot *= scale;
        if (lane == 0) sc[s] = dot;
        lmax = fmaxf(lmax, dot);
    }
    if (lane == 0) red[warp] = lmax;
    __syncthreads();
    float mx = red[0];
    for (int i = 1; i < nw; i++) mx = fmaxf(mx, red[i]);
    __syncthreads();
    float lsum = 0.f;
    for (int s = threadIdx.x; s < n_keys; s += blockDim.x) {
        const float e = expf(sc[s] - mx);
        sc[s] = e;
        lsum += e;
    }
    const float total = block_sum(lsum, red);
    const float inv = 1.f / total;
    // out[d] = sum_s p[s] v[s, d]: threads own d (coalesced across the value row), keys in order
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float acc = 0.f;
        const KV *vp = vmem + (int64_t)key_row0 * kv_ld + kvh * D + d;
        for (int s = 0; s < n_keys; s++) acc = fmaf(sc[s] * inv, kv_load(vp + (int64_t)s * kv_ld), acc);
        out[(int64_t)row * (H * D) + h * D + d] = acc;
    }
}

// Decode-time attention (one query row against the whole cache), attention_gqa_cache.wgsl for M = 1. The
// reference gives one workgroup per head the whole key range; here the keys are also split over
// ATT_SPLITS CTAs per head so that 14 heads x 8 slices fill the GPU, each slice keeps an online-softmax
// triple (max, sum, weighted values), and the last slice to arrive for a head (arrival counter, no
// waiting) merges the triples in slice order.
constexpr int ATT_SPLITS = 8;

template <typename KV>
__device__ __forceinline__ float dot_row(const float *qs, const KV *kp, int D);

template <>
__device__ __forceinline__ float dot_row<__half>(const float *qs, const __half *kp, int D)
{
    float dot = 0.f;
    for (int d = 0; d < D; d += 8) {
        const uint4 raw = *reinterpret_cast<const uint4 *>(kp + d);
        const __half2 *h = reinterpret_cast<const __half2 *>(&raw);
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float2 f = __half22float2(h[j]);
            dot = fmaf(qs[d + 2 * j], f.x, dot);
            dot = fmaf(qs[d + 2 * j + 1], f.y, dot);
        }
    }
    return dot;
}

template <>
__device__ __forceinline__ float dot_row<float>(const float *qs, const float *kp, int D)
{
    float dot = 0.f;
    for (int d = 0; d < D; d += 4) {
        const float4 f = *reinterpret_cast<const float4 *>(kp + d);
        dot = fmaf(qs[d], f.x, dot), dot = fmaf(qs[d + 1], f.y, dot);
        dot = fmaf(qs[d + 2], f.z, dot), dot = fmaf(qs[d + 3], f.w, dot);
    }
    return dot;
}

// Decode attention: one query row against the KV cache, the keys of each head split over ATT_SPLITS CTAs (online
// softmax per split, the last split to arrive merges). The kernel is a chain of dependent memory round trips, so the
// order of its loads is the design: q (and the raw k, v) are requested before the position is known; as soon as it
// is, the split's V rows start moving into shared memory (cp.async) and its K rows into registers, and they arrive
// while the scores and the softmax are computed; the merge issues all of its loads before it uses any. In a decode
// step (early_kv) the position, the rotary entry and the cache rows are even requested before the kernel waits for its
// predecessor, and only q and the raw k, v after it.
//
// With k_raw != nullptr the kernel also does the work of rope_half.wgsl + kv_store.wgsl for the new position
// (ropeHalfRef, src/reference/qwen-ref.ts:35-64): q, k_raw, v_raw are the projection outputs; q is rotated while it is
// staged; the split that owns the newest key rotates k itself (rounded to the cache type, as a later step will read
// it) instead of reading the cache row, and the first head of each KV group stores k and v to the cache.
__device__ __forceinline__ void att_cp_async_16(void *dst_smem, const void *src)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst_smem)), "l"(src)
                 : "memory");
}

template <typename KV>
__global__ void __launch_bounds__(128) attention_decode_kernel(const float *__restrict__ q, KV *__restrict__ kmem,
                                                               KV *__restrict__ vmem, float *__restrict__ out,
                                                               float *__restrict__ scratch, unsigned *__restrict__ counters,
                                                               int H, int KVH, int D, const int *__restrict__ past_ptr,
                                                               int past_imm, int kv_ld, float scale,
                                                               const float *__restrict__ k_raw, const float *__restrict__ v_raw,
                                                               const float *__restrict__ cs_table, int chunk_max, int early_kv,
                                                               int cl_async, int *status)
{
    // cl_async: the splits send their partial results to an mbarrier of the head's first CTA (cluster_merge_init)
    __shared__ uint64_t merge_bar;
    if (cl_async) cluster_merge_init(&merge_bar, (uint32_t)((ATT_SPLITS - 1) * (D + 2) * 4), blockIdx.y == 0);
    // early_kv: the cache rows of the earlier positions, the position itself and the rotary table entry are requested
    // BEFORE the wait on the previous kernel; only q and the new k, v (what that kernel wrote) come after it. The caller
    // sets it where every kernel in front of this one releases its successor after its own wait (pdl_sync), so that this
    // kernel cannot start before the kernel two places ahead, and everything older (the cache, the position), is complete.
    if (!early_kv) pdl_sync();
    // [D] query (pre-scaled), [2][D] new k, v, [chunk] scores, [4][D] per-warp value sums, [ATT_SPLITS][D + 2] merge slots
    // (written by the other CTAs of the cluster), then (16-byte aligned) the split's V rows [chunk_max][D] in the cache type
    extern __shared__ float sm[];
    __shared__ float red[4];
    const int h = blockIdx.x, s = blockIdx.y, kvh = h / (H / KVH);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int half = D >> 1;  // D <= 128: one (i, i + half) pair per thread
    const bool fused = k_raw != nullptr;
    float q0 = 0.f, q1 = 0.f, x0 = 0.f, x1 = 0.f, v0f = 0.f, v1f = 0.f;
    auto load_new = [&]() {
        if (tid < half) {
            q0 = q[h * D + tid], q1 = q[h * D + tid + half];
            if (fused) {
                x0 = k_raw[kvh * D + tid], x1 = k_raw[kvh * D + tid + half];
                v0f = v_raw[kvh * D + tid], v1f = v_raw[kvh * D + tid + half];
            }
        }
    };
    if (!early_kv) load_new();
    const int pos = past_ptr ? *past_ptr : past_imm;
    const int n_keys = pos + 1;
    const int chunk = (n_keys + ATT_SPLITS - 1) / ATT_SPLITS;
    const int k0 = s * chunk, k1 = min(n_keys, k0 + chunk), nk = max(0, k1 - k0);
    float *qs = sm, *knew = sm + D, *vnew = sm + 2 * D, *sc = sm + 3 * D, *wacc = sc + chunk_max, *merge = wacc + 4 * D;
    KV *vt = reinterpret_cast<KV *>(sm + ((7 * D + chunk_max + ATT_SPLITS * (D + 2) + 3) & ~3));
    const bool own_new = fused && k1 == n_keys && nk > 0;  // this split holds the newest key
    const int nk_mem = own_new ? nk - 1 : nk;               // keys of this split that are read from memory

    // rotary table entry of this position first: it is the shortest wait and gates the staging of q
    float rc = 1.f, rs = 0.f;
    if (fused && tid < half) rc = cs_table[((int64_t)pos * half + tid) * 2], rs = cs_table[((int64_t)pos * half + tid) * 2 + 1];
    // V rows of this split -> shared memory, in flight from here on
    {
        const int per_row = D * (int)sizeof(KV) / 16;  // 16-byte pieces per row
        for (int i = tid; i < nk_mem * per_row; i += blockDim.x) {
            const int j = i / per_row, c = i - j * per_row;
            att_cp_async_16(reinterpret_cast<char *>(vt + (size_t)j * D) + c * 16,
                            reinterpret_cast<const char *>(vmem + (int64_t)(k0 + j) * kv_ld + kvh * D) + c * 16);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    // Warps are specialised for the staging phase: the first warp(s) (tid < half) rotate q and the new k, the others
    // own the keys. A key thread requests the K row of its first key (rows of up to 128 bytes) into registers right
    // away, so the row's HBM latency overlaps the staging of q; the rotating warps issue no K loads, so their wait on
    // the rotary table is not held up by them (loads that share a scoreboard complete together).
    constexpr int KREGS = 8;
    const int k_pieces = D * (int)sizeof(KV) / 16;
    const int kbase = ((half + 31) >> 5) << 5, kthreads = (int)blockDim.x - kbase, kt = tid - kbase;
    const bool k_pre = k_pieces <= KREGS && kt >= 0 && kt < nk_mem;
    uint4 kreg[KREGS];
    if (k_pre) {
        const uint4 *kp = reinterpret_cast<const uint4 *>(kmem + (int64_t)(k0 + kt) * kv_ld + kvh * D);
#pragma unroll
        for (int c = 0; c < KREGS; c++)
            if (c < k_pieces) kreg[c] = kp[c];
    }
    if (early_kv) {
        pdl_sync();
        load_new();
    }
    if (tid < half) {
        if (!fused) {
            qs[tid] = q0 * scale, qs[tid + half] = q1 * scale;
        } else {
            const int i = tid;
            const float c = rc, sn = rs;
            qs[i] = (q0 * c - q1 * sn) * scale;
            qs[i + half] = (q0 * sn + q1 * c) * scale;
            if (own_new) {
                const KV r0 = (KV)(x0 * c - x1 * sn), r1 = (KV)(x0 * sn + x1 * c);
                const KV v0 = (KV)v0f, v1 = (KV)v1f;
                knew[i] = (float)r0, knew[i + half] = (float)r1, vnew[i] = (float)v0, vnew[i + half] = (float)v1;
                if (h == kvh * (H / KVH)) {
                    KV *kd = kmem + (int64_t)pos * kv_ld + kvh * D, *vd = vmem + (int64_t)pos * kv_ld + kvh * D;
                    kd[i] = r0, kd[i + half] = r1, vd[i] = v0, vd[i + half] = v1;
                }
            }
        }
    }
    __syncthreads();

    float lmax = -INFINITY;
    if (k_pre) {  // same order of operations as dot_row
        float dot = 0.f;
#pragma unroll
        for (int c = 0; c < KREGS; c++) {
            if (c < k_pieces) {
                if constexpr (sizeof(KV) == 2) {
                    const __half2 *hh = reinterpret_cast<const __half2 *>(&kreg[c]);
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        const float2 f = __half22float2(hh[j]);
                        dot = fmaf(qs[c * 8 + 2 * j], f.x, dot);
                        dot = fmaf(qs[c * 8 + 2 * j + 1], f.y, dot);
                    }
                } else {
                    const float4 f = *reinterpret_cast<const float4 *>(&kreg[c]);
                    dot = fmaf(qs[c * 4], f.x, dot), dot = fmaf(qs[c * 4 + 1], f.y, dot);
                    dot = fmaf(qs[c * 4 + 2], f.z, dot), dot = fmaf(qs[c * 4 + 3], f.w, dot);
                }
            }
        }
        sc[kt] = dot;
        lmax = dot;
    }
    for (int j = kt >= 0 ? kt + (k_pre ? kthreads : 0) : nk_mem; j < nk_mem; j += kthreads) {
        const float dot = dot_row<KV>(qs, kmem + (int64_t)(k0 + j) * kv_ld + kvh * D, D);
        sc[j] = dot;
        lmax = fmaxf(lmax, dot);
    }
    if (own_new && tid == (nk_mem & 127)) {  // the thread whose turn index nk - 1 would have been
        const float dot = dot_row<float>(qs, knew, D);
        sc[nk_mem] = dot;
        lmax = fmaxf(lmax, dot);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) lmax = fmaxf(lmax, __shfl_xor_sync(0xffffffffu, lmax, o));
    if (lane == 0) red[warp] = lmax;
    __syncthreads();
    const float mx = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
    __syncthreads();
    float lsum = 0.f;
    for (int j = tid; j < nk; j += blockDim.x) {
        const float e = expf(sc[j] - mx);
        sc[j] = e;
        lsum += e;
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");  // this thread's V pieces; the barrier below covers the others'
    const float total = block_sum(lsum, red);  // also orders the sc[] and V-tile writes before the reads below
    // weighted values: warp w takes keys w, w+4, ...; lane owns dims 2*lane, 2*lane+1 (and +64 for D = 128)
    for (int d0 = 0; d0 < D; d0 += 64) {
        float a0 = 0.f, a1 = 0.f;
        const int d = d0 + 2 * lane;
        if (d < D) {
            for (int j = warp; j < nk_mem; j += 4) {
                const KV *vp = vt + (size_t)j * D + d;
                a0 = fmaf(sc[j], kv_load(vp), a0);
                a1 = fmaf(sc[j], kv_load(vp + 1), a1);
            }
            if (own_new && warp == (nk_mem & 3)) a0 = fmaf(sc[nk_mem], vnew[d], a0), a1 = fmaf(sc[nk_mem], vnew[d + 1], a1);
        }
        if (d < D) wacc[warp * D + d] = a0, wacc[warp * D + d + 1] = a1;
    }
    __syncthreads();
    // The ATT_SPLITS CTAs of a head form one cluster: each stores its (max, sum, weighted values) into the shared memory
    // of the cluster's first CTA, and after the cluster barrier (with cl_async: once its mbarrier has counted the other
    // splits' bytes) that CTA merges them in split order. No global scratch, no atomic, and nothing depends on which CTA
    // finishes last.
    if (cl_async) {
        if (s != 0) {
            const uint32_t dst = cluster_map_shared(merge + (size_t)s * (D + 2), 0), bar = cluster_map_shared(&merge_bar, 0);
            for (int d = tid; d < D; d += blockDim.x)
                cluster_send_f32(dst + (2 + d) * 4, wacc[d] + wacc[D + d] + wacc[2 * D + d] + wacc[3 * D + d], bar);
            if (tid == 0) cluster_send_f32(dst, mx, bar), cluster_send_f32(dst + 4, total, bar);
            return;
        }
        for (int d = tid; d < D; d += blockDim.x) merge[2 + d] = wacc[d] + wacc[D + d] + wacc[2 * D + d] + wacc[3 * D + d];
        if (tid == 0) merge[0] = mx, merge[1] = total;
        __syncthreads();
        if (tid < D) cluster_merge_wait(&merge_bar, status);
    } else {
        const uint32_t dst = cluster_map_shared(merge + (size_t)s * (D + 2), 0);
        for (int d = tid; d < D; d += blockDim.x)
            cluster_store_f32(dst + (2 + d) * 4, wacc[d] + wacc[D + d] + wacc[2 * D + d] + wacc[3 * D + d]);
        if (tid == 0) cluster_store_f32(dst, mx), cluster_store_f32(dst + 4, total);
        cluster_barrier();
    }
    if (s != 0) return;
    for (int d = tid; d < D; d += blockDim.x) {
        float M = -INFINITY;
#pragma unroll
        for (int i = 0; i < ATT_SPLITS; i++) M = fmaxf(M, merge[i * (D + 2)]);
        float Lsum = 0.f, acc = 0.f;
#pragma unroll
        for (int i = 0; i < ATT_SPLITS; i++) {
            const float li = merge[i * (D + 2) + 1];
            if (li > 0.f) {
                const float e = expf(merge[i * (D + 2)] - M);
                Lsum += li * e;
                acc = fmaf(merge[i * (D + 2) + 2 + d], e, acc);
            }
        }
        out[h * D + d] = acc / Lsum;
    }
}

// Greedy sampling (sampleToken with temperature <= 0, src/infer/sampler.ts:30-36): index of the first
// strict maximum. Stage 1: per-block (value, index) candidates; stage 2: one block reduces them.
__global__ void __launch_bounds__(256) argmax_stage1(const float *__restrict__ logits, int V, float *__restrict__ bval,
                                                     int *__restrict__ bidx)
{
    pdl_sync();
    __shared__ float sv[256];
    __shared__ int si[256];
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < V; i += gridDim.x * blockDim.x) {
        const float v = logits[i];
        if (v > best || (v == best && i < bi)) best = v, bi = i;
    }
    sv[threadIdx.x] = best, si[threadIdx.x] = bi;
    __syncthreads();
    for (int o = 128; o > 0; o >>= 1) {
        if (threadIdx.x < o) {
            const float v = sv[threadIdx.x + o];
            const int i = si[threadIdx.x + o];
            if (v > sv[threadIdx.x] || (v == sv[threadIdx.x] && i < si[threadIdx.x])) sv[threadIdx.x] = v, si[threadIdx.x] = i;
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) bval[blockIdx.x] = sv[0], bidx[blockIdx.x] = si[0];
}

// Stage 2 also advances the decode state on the device: next token -> token buffer and output ring,
// cache length += 1, so that a captured graph can be replayed step after step with no host round trip.
__global__ void __launch_bounds__(256) argmax_stage2(const float *__restrict__ bval, const int *__restrict__ bidx, int nb,
                                                     uint32_t *__restrict__ token_out, uint32_t *__restrict__ history,
                                                     int *__restrict__ step_counter, int *__restrict__ cache_len)
{
    pdl_sync();
    __shared__ float sv[256];
    __shared__ int si[256];
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < nb; i += blockDim.x) {
        const float v = bval[i];
        const int ix = bidx[i];
        if (v > best || (v == best && ix < bi)) best = v, bi = ix;
    }
    sv[threadIdx.x] = best, si[threadIdx.x] = bi;
    __syncthreads();
    for (int o = 128; o > 0; o >>= 1) {
        if (threadIdx.x < o) {
            const float v = sv[threadIdx.x + o];
            const int i = si[threadIdx.x + o];
            if (v > sv[threadIdx.x] || (v == sv[threadIdx.x] && i < si[threadIdx.x])) sv[threadIdx.x] = v, si[threadIdx.x] = i;
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        const uint32_t tok = si[0] == 0x7fffffff ? 0u : (uint32_t)si[0];  // all-NaN logits: JS returns index 0
        *token_out = tok;
        if (history) {
            history[*step_counter] = tok;
            *step_counter += 1;
        }
        if (cache_len) *cache_len += 1;
    }
}

// ---------------------------------------------------------------------------------------------------

#define LAUNCH_OK(ctx)                \
    do {                              \
        (ctx)->launches++;            \
        WB_CUDA(cudaGetLastError());  \
        return WB_OK;                 \
    } while (0)

int op_embed(wb_context *ctx, const __half *table, const uint32_t *tokens, float *x, int M, int C, int vocab)
{
    const int64_t n = (int64_t)M * C;
    WB_CUDA(launch_pdl(embed_f16_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, ctx->stream, table, tokens, x, M, C, vocab));
    LAUNCH_OK(ctx);
}

int op_rmsnorm(wb_context *ctx, const float *x, const float *delta, float *x_out, const float *w, float *y, int M, int D, float eps,
               __half *y16)
{
    // rows kept in registers where they fit; the summation order inside a thread differs from the scalar kernel's
    // (both are f32 sums of D squares: the difference is rounding noise of the statistic)
    if (M > 1 && D % 4 == 0 && D <= 4096)
        WB_CUDA(launch_pdl(rmsnorm_vec4_kernel, dim3(M), dim3(256), 0, ctx->stream, x, delta, x_out, w, y, y16, D, eps));
    else
        WB_CUDA(launch_pdl(rmsnorm_kernel, dim3(M), dim3(256), 0, ctx->stream, x, delta, x_out, w, y, y16, D, eps));
    LAUNCH_OK(ctx);
}

int op_add(wb_context *ctx, const float *a, const float *b, float *out, int64_t n)
{
    WB_CUDA(launch_pdl(add_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, ctx->stream, a, b, out, n));
    LAUNCH_OK(ctx);
}

int op_silu_mul(wb_context *ctx, const float *gate, const float *up, float *out, int M, int I, int ld, __half *out16)
{
    const int64_t n = (int64_t)M * I;
    if (I % 4 == 0 && ld % 4 == 0 && ((uintptr_t)gate % 16) == 0 && ((uintptr_t)up % 16) == 0) {
        WB_CUDA(launch_pdl(silu_mul_vec4_kernel, dim3((unsigned)((n / 4 + 255) / 256)), dim3(256), 0, ctx->stream, gate, up, out, out16, M, I, ld));
    } else {
        if (out16) return fail(WB_ERR_UNSUPPORTED, "fp16 silu output needs I %% 4 == 0");
        WB_CUDA(launch_pdl(silu_mul_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, ctx->stream, gate, up, out, M, I, ld));
    }
    LAUNCH_OK(ctx);
}

int op_rope_kv(wb_context *ctx, float *q, float *k, const float *v, void *k_cache, void *v_cache, int kv_f16,
               const float *cs_table, int M, int H, int KVH, int D, int T, const int *pos_ptr, int pos_imm, int ldq,
               int ldk, int ldv)
{
    const int64_t n = (int64_t)M * (H + 2 * KVH) * (D / 2);
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (kv_f16)
        WB_CUDA(launch_pdl(rope_kv_kernel<__half>, dim3(blocks), dim3(256), 0, ctx->stream, q, k, v, (__half *)k_cache, (__half *)v_cache, cs_table, M, H,
                                                                 KVH, D, T, pos_ptr, pos_imm, ldq, ldk, ldv));
    else
        WB_CUDA(launch_pdl(rope_kv_kernel<float>, dim3(blocks), dim3(256), 0, ctx->stream, q, k, v, (float *)k_cache, (float *)v_cache, cs_table, M, H, KVH,
                                                                D, T, pos_ptr, pos_imm, ldq, ldk, ldv));
    LAUNCH_OK(ctx);
}

int op_attention(wb_context *ctx, const float *q, const void *kmem, const void *vmem, int kv_f16, float *out, int M, int H,
                 int KVH, int D, int T, const int *past_ptr, int past_imm, int use_cache, int max_keys, int ldq, int kv_ld)
{
    const size_t smem = (size_t)(D + max_keys) * sizeof(float);
    const float scale = 1.0f / sqrtf((float)D);
    dim3 grid(M, H);
    if (kv_f16) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(attention_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        WB_CUDA(launch_pdl(attention_kernel<__half>, dim3(grid), dim3(128), smem, ctx->stream, q, (const __half *)kmem, (const __half *)vmem, out, H, KVH, D, T,
                                                                    past_ptr, past_imm, use_cache, ldq, kv_ld, scale));
    } else {
        if (smem > 48 * 1024) cudaFuncSetAttribute(attention_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        WB_CUDA(launch_pdl(attention_kernel<float>, dim3(grid), dim3(128), smem, ctx->stream, q, (const float *)kmem, (const float *)vmem, out, H, KVH, D, T,
                                                                   past_ptr, past_imm, use_cache, ldq, kv_ld, scale));
    }
    LAUNCH_OK(ctx);
}

size_t op_attention_decode_smem(int D, int max_keys, int kv_f16)
{
    const int chunk = (max_keys + ATT_SPLITS - 1) / ATT_SPLITS;
    return (size_t)((7 * D + chunk + ATT_SPLITS * (D + 2) + 3) & ~3) * sizeof(float) + (size_t)chunk * D * (kv_f16 ? 2 : 4);
}

int op_attention_decode(wb_context *ctx, const float *q, void *kmem, void *vmem, int kv_f16, float *out, float *scratch,
                        unsigned *counters, int H, int KVH, int D, const int *past_ptr, int past_imm, int max_keys, int kv_ld,
                        const float *k_raw, const float *v_raw, const float *cs_table, int early_kv)
{
    const int chunk = (max_keys + ATT_SPLITS - 1) / ATT_SPLITS;
    const size_t smem = op_attention_decode_smem(D, max_keys, kv_f16);
    const float scale = 1.0f / sqrtf((float)D);
    static const int cl_async = [] { const char *e = getenv("WEBLLM_B200_CLUSTER_ASYNC"); return (e && e[0] == '0') ? 0 : 1; }();  // see gemv.cu
    dim3 grid(H, ATT_SPLITS);
    if (kv_f16) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(attention_decode_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        WB_CUDA(launch_pdl_cluster(attention_decode_kernel<__half>, grid, dim3(128), smem, ctx->stream, ATT_SPLITS, q, (__half *)kmem, (__half *)vmem, out,
                           scratch, counters, H, KVH, D, past_ptr, past_imm, kv_ld, scale, k_raw, v_raw, cs_table, chunk, early_kv, cl_async, ctx->status_word));
    } else {
        if (smem > 48 * 1024) cudaFuncSetAttribute(attention_decode_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        WB_CUDA(launch_pdl_cluster(attention_decode_kernel<float>, grid, dim3(128), smem, ctx->stream, ATT_SPLITS, q, (float *)kmem, (float *)vmem, out,
                           scratch, counters, H, KVH, D, past_ptr, past_imm, kv_ld, scale, k_raw, v_raw, cs_table, chunk, early_kv, cl_async, ctx->status_word));
    }
    LAUNCH_OK(ctx);
}

int op_attention_decode_scratch_floats(int H, int D) { return H * ATT_SPLITS * (D + 2); }

int op_argmax(wb_context *ctx, const float *logits, int V, float *bval, int *bidx, uint32_t *token_out, uint32_t *history,
              int *step_counter, int *cache_len)
{
    const int nb = 128;
    WB_CUDA(launch_pdl(argmax_stage1, dim3(nb), dim3(256), 0, ctx->stream, logits, V, bval, bidx));
    ctx->launches++;
    WB_CUDA(launch_pdl(argmax_stage2, dim3(1), dim3(256), 0, ctx->stream, bval, bidx, nb, token_out, history, step_counter, cache_len));
    LAUNCH_OK(ctx);
}

}  // namespace wb
