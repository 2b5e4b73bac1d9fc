// One decode step of the Qwen2 model as a single persistent kernel.
//
// At batch 1 a 0.5B-class model is launch-latency bound: the 24 layers are ~220 small kernels of 2-5 us each,
// although all their weights together stream in ~70 us. Here one cooperative kernel (one CTA per SM, all
// co-resident) walks the whole step, QwenGpt.runForward with M = 1 (src/model/qwen.ts:391-489), and the
// kernel boundaries become grid-wide barriers:
//
//   per layer   P1  x = residual (+ down partials); n = rmsnorm(x);  q|k|v = n W^T        -> partial sums
//               P2  rope(q, k), append k, v to the cache, attention over 8 key slices/head  -> (max, sum, acc)
//               P3  merge slices -> att;                          o = att W^T              -> partial sums
//               P4  xa = x + o;  n = rmsnorm(xa);                 gate|up = n W^T          -> partial sums
//               P5  act = silu(gate) * up;                        down = act W^T           -> partial sums
//   finally         x = xa + down; rmsnorm; fp16 lm_head; per-CTA argmax candidates; barrier; CTA 0 picks the token
//                   (first strict maximum, src/infer/sampler.ts:30-36), appends it and bumps the cache length.
//
// A projection is cut into units of (32-column tile) x (range of 128-k chunks), at most one unit per CTA at
// a time, one chunk per warp; the unit's warps are reduced in shared memory in warp order and the unit writes
// one row of partial sums. The consumer of a projection adds the partial rows in row order while it stages
// its input, so results do not depend on scheduling, no atomics touch the data, and every CTA recomputes the
// cheap vector steps (norms, rope, activation) for itself instead of waiting for another barrier.
// The chunk arithmetic is that of the streaming GEMV (gemv_core.cuh, f32 activations as hi + lo fp16).
//
// Everything one CTA writes for another is read back with ld.global.cg (L1 is not coherent across SMs).
// The grid barrier is an atomic counter with a bounded spin: a wait that gives up sets an abort flag and a
// status code, every CTA leaves, and wb_qwen_decode_greedy reports WB_ERR_TIMEOUT.
#include <algorithm>
#include <memory>

#include "qwen_internal.cuh"

#include "gemv_core.cuh"

namespace wbq {

using namespace wb;

constexpr int MEGA_THREADS = 512;
constexpr int MEGA_WARPS = MEGA_THREADS / 32;
constexpr int MEGA_ATT_SPLITS = 8;
constexpr unsigned MEGA_SPIN_LIMIT = 1u << 22;

struct MLinear {
    const uint32_t *qw;
    const uint32_t *qz;
    const __half *sc;
    const float *bias;
    int K, N, chunks, tiles, R, cpr, zcols, group_chunks;
};

struct MLayer {
    MLinear qkv, o, gu, down;
    const float *in_norm, *post_norm;
    void *kc, *vc;
};

struct MParams {
    const MLayer *layers;
    int n_layer, C, H, KVH, D, KV, I, V, max_t, kv_f16;
    float eps;
    const __half *embed;
    const float *final_norm, *cs_table;
    int *cache_len, *step;
    uint32_t *token, *history;
    float *xa;         // [2][C] residual stream after the attention sub-layer, by layer parity
    float *part_qkv, *part_o, *part_gu, *part_down;  // [R][N] partial sums of the four projections
    float *att_part;   // [H][MEGA_ATT_SPLITS][D + 2]
    float *logits;     // [V]
    float *cand_val;   // [grid]
    int *cand_idx;
    unsigned long long *barrier;
    unsigned long long bar_base;
    int *abort_flag, *status;
};

struct Mega {
    MLayer *d_layers = nullptr;
    MParams p{};
    unsigned long long launches = 0;
    int grid = 0;
    size_t smem = 0;
    int barriers_per_launch = 0;
};

// ---------------------------------------------------------------------------------------------- device

__device__ __forceinline__ unsigned long long ld_acquire_u64(const unsigned long long *p)
{
    unsigned long long v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

struct MegaSmem {
    float *xin;      // [max(C, I)] input vector of the current projection (f32)
    uint4 *xs_hi;    // [2][stride] staged operand rows (row 1 = zeros)
    uint4 *xs_lo;
    float *xsum;     // [chunks]
    float *red;      // [MEGA_WARPS][64]
    float *misc;     // attention: q[D], k_new[D], v_new[D], scores
    int *flag;
    int stride;
};

// Grid-wide barrier number `epoch` of this launch. Returns false when it gave up (or another CTA did).
__device__ bool grid_barrier(const MParams &p, int &epoch, const MegaSmem &sm)
{
    epoch++;
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        atomicAdd(p.barrier, 1ULL);
        const unsigned long long target = p.bar_base + (unsigned long long)epoch * gridDim.x;
        int ok = 0;
        for (unsigned it = 0; it < MEGA_SPIN_LIMIT; it++) {
            if (ld_acquire_u64(p.barrier) >= target) {
                ok = 1;
                break;
            }
            if ((it & 255u) == 255u && *(volatile int *)p.abort_flag) break;
        }
        if (!ok) {
            *(volatile int *)p.abort_flag = 1;
            *(volatile int *)p.status = 100 + epoch;
        }
        *sm.flag = ok;
    }
    __syncthreads();
    return *sm.flag != 0;
}

__device__ __forceinline__ float block_sum_512(float v, float *red)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = 0.f;
    for (int i = 0; i < MEGA_WARPS; i++) t += red[i];
    __syncthreads();
    return t;
}

// Sum of R partial rows written by other CTAs (row 0 carries the bias), added in row order. An L2 round trip
// costs ~0.8 us here and a plain loop pays one per row, so up to 8 loads are issued before the first add;
// part_sum2 does the same for two projections at once (plus an optional residual value).
__device__ __forceinline__ float part_sum(const float *part, int R, int N, int n)
{
    float v = 0.f;
    for (int r0 = 0; r0 < R; r0 += 8) {
        float a[8];
#pragma unroll
        for (int j = 0; j < 8; j++) a[j] = r0 + j < R ? __ldcg(part + (size_t)(r0 + j) * N + n) : 0.f;
#pragma unroll
        for (int j = 0; j < 8; j++) v += a[j];
    }
    return v;
}

__device__ __forceinline__ float part_sum2(const float *base, const float *pa, int Ra, const float *pb, int Rb, int N, int n)
{
    float a[8], b[8];
    const float x0 = base ? __ldcg(base + n) : 0.f;
#pragma unroll
    for (int j = 0; j < 8; j++) a[j] = j < Ra ? __ldcg(pa + (size_t)j * N + n) : 0.f;
#pragma unroll
    for (int j = 0; j < 8; j++) b[j] = j < Rb ? __ldcg(pb + (size_t)j * N + n) : 0.f;
    float va = 0.f, vb = 0.f;
#pragma unroll
    for (int j = 0; j < 8; j++) va += a[j];
    for (int r = 8; r < Ra; r++) va += __ldcg(pa + (size_t)r * N + n);
#pragma unroll
    for (int j = 0; j < 8; j++) vb += b[j];
    for (int r = 8; r < Rb; r++) vb += __ldcg(pb + (size_t)r * N + n);
    return (x0 + va) + vb;
}

// Every CTA reads the same vectors from L2 at the same moment; starting each CTA's sweep at a different
// offset keeps them from queueing on the same L2 slice in lockstep (measured: 11 us -> ~2 us for 39 KB).
__device__ __forceinline__ int rotated(int idx, int n)
{
    const int d = idx + (int)((blockIdx.x * 1031u) % (unsigned)n);
    return d >= n ? d - n : d;
}

// xin[0..D) *= rsqrt(mean(xin^2) + eps) * w   (rmsNormRef, src/reference/qwen-ref.ts:12-29)
__device__ void rmsnorm_inplace(float *xin, const float *w, int D, float eps, float *red)
{
    float ss = 0.f;
    for (int d = threadIdx.x; d < D; d += MEGA_THREADS) ss = fmaf(xin[d], xin[d], ss);
    const float rstd = rsqrtf(block_sum_512(ss, red) / (float)D + eps);
    for (int d = threadIdx.x; d < D; d += MEGA_THREADS) xin[d] = xin[d] * rstd * w[d];
    __syncthreads();
}

// One projection: y = xin W^T as partial rows part[r][n] (r = chunk range of the unit; row 0 also gets the bias).
// xin holds the K input values in shared memory; every CTA stages all of them (hi + lo fp16, MMA k-slot order).
// The first chunk of a CTA's first unit does not depend on the input vector: it is requested ahead (before the
// grid barrier that precedes the phase) so that its HBM latency overlaps the barrier and the staging.
__device__ __forceinline__ GemvParams linear_params(const MLinear &L, int stride)
{
    GemvParams gp{};
    gp.qw = L.qw, gp.qz = L.qz, gp.sc = L.sc;
    gp.M = 1, gp.N = L.N, gp.K = L.K, gp.pack_rows = L.K >> 3, gp.zcols = L.zcols, gp.group_chunks = L.group_chunks;
    gp.xs_stride = stride;
    return gp;
}

__device__ __forceinline__ bool gemv_prefetch(const MLinear &L, const MegaSmem &sm, ChunkRegs &regs)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const int u = blockIdx.x;
    if (u >= L.tiles * L.R) return false;
    const int tile = u / L.R, r = u - tile * L.R;
    const int ch = r * L.cpr + warp;
    if (ch >= min(L.chunks, r * L.cpr + L.cpr)) return false;
    const int c = tile * 32 + 4 * g;
    const GemvParams gp = linear_params(L, sm.stride);
    fetch_chunk(gp, ch, t, c, c < L.N, regs);
    return true;
}

__device__ void gemv_phase(const MLinear &L, const MegaSmem &sm, float *part, ChunkRegs &ra, bool has_pre)
{
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    const int rows = L.K >> 3;
    // ---- stage the input vector: row 0 = data, row 1 = zeros (lanes without a batch row read it) ----
    for (int rl = tid; rl < rows; rl += MEGA_THREADS) {
        float v[8];
        const float4 a = *reinterpret_cast<const float4 *>(sm.xin + rl * 8);
        const float4 b = *reinterpret_cast<const float4 *>(sm.xin + rl * 8 + 4);
        v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
        __half hi[8], lo[8];
#pragma unroll
        for (int j = 0; j < 8; j++) {
            hi[j] = __float2half_rn(v[j]);
            lo[j] = __float2half_rn(v[j] - __half2float(hi[j]));
        }
        uint4 o;
        o.x = h2_as_u32(__halves2half2(hi[0], hi[4])), o.y = h2_as_u32(__halves2half2(hi[2], hi[6]));
        o.z = h2_as_u32(__halves2half2(hi[1], hi[5])), o.w = h2_as_u32(__halves2half2(hi[3], hi[7]));
        sm.xs_hi[rl] = o;
        o.x = h2_as_u32(__halves2half2(lo[0], lo[4])), o.y = h2_as_u32(__halves2half2(lo[2], lo[6]));
        o.z = h2_as_u32(__halves2half2(lo[1], lo[5])), o.w = h2_as_u32(__halves2half2(lo[3], lo[7]));
        sm.xs_lo[rl] = o;
        sm.xs_hi[sm.stride + rl] = make_uint4(0, 0, 0, 0);
        sm.xs_lo[sm.stride + rl] = make_uint4(0, 0, 0, 0);
    }
    __syncthreads();
    for (int idx = tid; idx < L.chunks * 16; idx += MEGA_THREADS) {  // per-chunk sums of the staged values
        const int cl = idx >> 4, rr = idx & 15;
        auto sum8 = [](const uint4 &o) {
            const float2 a = __half22float2(u32_as_h2(o.x)), b = __half22float2(u32_as_h2(o.y));
            const float2 c = __half22float2(u32_as_h2(o.z)), d = __half22float2(u32_as_h2(o.w));
            return ((a.x + a.y) + (b.x + b.y)) + ((c.x + c.y) + (d.x + d.y));
        };
        float sx = sum8(sm.xs_hi[cl * 16 + rr]) + sum8(sm.xs_lo[cl * 16 + rr]);
        const unsigned half_mask = (lane & 16) ? 0xffff0000u : 0x0000ffffu;
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) sx += __shfl_xor_sync(half_mask, sx, o);
        if (rr == 0) sm.xsum[cl] = sx;
    }
    __syncthreads();

    const GemvParams gp = linear_params(L, sm.stride);
    const int units = L.tiles * L.R;
    // This CTA's units u = blockIdx.x + j * gridDim.x, j < nu, flattened with their chunks into items
    // (j, chunk index within the unit); warp w takes items w, w + 16, ... Up to two items per warp are loaded
    // before anything is computed, so that their HBM latencies overlap (the first one was requested before the
    // grid barrier). Each item leaves 32 column sums in red[item]; a unit's items are then added in chunk order.
    const int nu = (int)blockIdx.x < units ? (units - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
    const int cpu_ = L.cpr;                    // items per unit (<= 16; the last range of a tile may hold fewer chunks)
    const int upr = (2 * MEGA_WARPS) / cpu_;   // whole units per round of 32 items (>= 2)
    for (int j0 = 0; j0 < nu; j0 += upr) {
        const int ru = min(upr, nu - j0), ri = ru * cpu_;
        ChunkRegs rb;  // `ra` is the caller's register set: it may already hold the chunk requested ahead
        int tl[2], rr[2], ch[2];
        bool valid[2];
#pragma unroll
        for (int half = 0; half < 2; half++) {
            const int li = warp + half * MEGA_WARPS;
            const int j = j0 + li / cpu_, k = li % cpu_;
            const int u = (int)blockIdx.x + j * (int)gridDim.x;
            tl[half] = u / L.R, rr[half] = u - tl[half] * L.R;
            ch[half] = rr[half] * L.cpr + k;
            valid[half] = li < ri && ch[half] < L.chunks;
        }
        if (valid[0]) {
            // (unit blockIdx.x, chunk `warp`) may have been requested ahead
            if (!(has_pre && j0 == 0 && warp < cpu_)) fetch_chunk(gp, ch[0], t, tl[0] * 32 + 4 * g, tl[0] * 32 + 4 * g < L.N, ra);
        }
        if (valid[1]) fetch_chunk(gp, ch[1], t, tl[1] * 32 + 4 * g, tl[1] * 32 + 4 * g < L.N, rb);
#pragma unroll
        for (int half = 0; half < 2; half++) {
            const int li = warp + half * MEGA_WARPS;
            if (li < ri) {
                float tot[1][2][4] = {};
                if (valid[half]) {
                    if (half == 0) compute_chunk<1, true>(gp, ra, ch[0] * 16 + t, g, t, sm.xs_hi, sm.xs_lo, sm.xsum, ch[0], L.chunks, tot);
                    else compute_chunk<1, true>(gp, rb, ch[1] * 16 + t, g, t, sm.xs_hi, sm.xs_lo, sm.xsum, ch[1], L.chunks, tot);
                }
                if (t == 0) {  // activation row 0 sits in accumulator column 0 of the lanes with t == 0
                    float *dst = sm.red + li * 32 + 4 * g;
                    dst[0] = tot[0][0][0], dst[1] = tot[0][0][2], dst[2] = tot[0][1][0], dst[3] = tot[0][1][2];
                }
            }
        }
        __syncthreads();
        for (int o = tid; o < ru * 32; o += MEGA_THREADS) {  // one thread per (unit of the round, column)
            const int ju = o >> 5, col = o & 31;
            const int u = (int)blockIdx.x + (j0 + ju) * (int)gridDim.x;
            const int tile = u / L.R, r = u - tile * L.R;
            const int n = tile * 32 + col;
            float v = 0.f;
            for (int k = 0; k < cpu_; k++) v += sm.red[(ju * cpu_ + k) * 32 + col];  // chunk order: deterministic
            if (n < L.N) {
                if (r == 0 && L.bias) v += L.bias[n];
                part[(size_t)r * L.N + n] = v;
            }
        }
        __syncthreads();
    }
}

__device__ __forceinline__ float kv_get(const void *base, size_t idx, int f16)
{
    return f16 ? __half2float(((const __half *)base)[idx]) : ((const float *)base)[idx];
}

// P2: rope, cache append and one (head, key slice) of the attention; attentionGqaRef for a single query row.
__device__ void attention_phase(const MParams &p, const MLayer &L, const MegaSmem &sm, int pos)
{
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int D = p.D, half = D >> 1, Nq = p.C + 2 * p.KV;
    const int u = blockIdx.x;
    if (u >= p.H * MEGA_ATT_SPLITS) return;
    const int h = u / MEGA_ATT_SPLITS, s = u - h * MEGA_ATT_SPLITS, kvh = h / (p.H / p.KVH);
    float *q = sm.misc, *kn = sm.misc + D, *vn = sm.misc + 2 * D, *sc = sm.misc + 3 * D;
    float *wacc = sm.xin;  // [MEGA_WARPS][D], xin is free during this phase
    const float scale = rsqrtf((float)D);
    // q, k, v of this head from the partial rows, one element per thread (6 * D/2 threads, one L2 round trip),
    // then rotate q and k (ropeHalfRef, src/reference/qwen-ref.ts:35-64)
    float *raw = sc;  // [3][D] scratch before the scores use it
    for (int e = tid; e < 3 * D; e += MEGA_THREADS) {
        const int which = e / D, d = e - which * D;
        const int col = which == 0 ? h * D + d : (which == 1 ? p.C + kvh * D + d : p.C + p.KV + kvh * D + d);
        raw[e] = part_sum(p.part_qkv, L.qkv.R, Nq, col);
    }
    __syncthreads();
    for (int i = tid; i < half; i += MEGA_THREADS) {
        const float c = p.cs_table[((size_t)pos * half + i) * 2], sn = p.cs_table[((size_t)pos * half + i) * 2 + 1];
        const float q0 = raw[i], q1 = raw[i + half];
        q[i] = (q0 * c - q1 * sn) * scale;
        q[i + half] = (q0 * sn + q1 * c) * scale;
        const float k0 = raw[D + i], k1 = raw[D + i + half];
        float r0 = k0 * c - k1 * sn, r1 = k0 * sn + k1 * c;
        float v0 = raw[2 * D + i], v1 = raw[2 * D + i + half];
        if (p.kv_f16) {  // what later steps will read back from the cache
            r0 = __half2float(__float2half_rn(r0)), r1 = __half2float(__float2half_rn(r1));
            v0 = __half2float(__float2half_rn(v0)), v1 = __half2float(__float2half_rn(v1));
        }
        kn[i] = r0, kn[i + half] = r1, vn[i] = v0, vn[i + half] = v1;
    }
    __syncthreads();
    const int n_keys = pos + 1;
    const int chunk = (n_keys + MEGA_ATT_SPLITS - 1) / MEGA_ATT_SPLITS;
    const int k0 = s * chunk, k1 = min(n_keys, k0 + chunk), nk = max(0, k1 - k0);
    // the slice that holds position `pos` of the first query head of the group appends the new row
    if (h % (p.H / p.KVH) == 0 && pos >= k0 && pos < k1) {
        for (int d = tid; d < D; d += MEGA_THREADS) {
            const size_t idx = ((size_t)pos * p.KVH + kvh) * D + d;
            if (p.kv_f16) ((__half *)L.kc)[idx] = __float2half_rn(kn[d]), ((__half *)L.vc)[idx] = __float2half_rn(vn[d]);
            else ((float *)L.kc)[idx] = kn[d], ((float *)L.vc)[idx] = vn[d];
        }
    }
    float lmax = -INFINITY;
    for (int j = tid; j < nk; j += MEGA_THREADS) {
        const int key = k0 + j;
        float dot = 0.f;
        if (key == pos) {
            for (int d = 0; d < D; d++) dot = fmaf(q[d], kn[d], dot);
        } else if (p.kv_f16) {  // the whole key row in 16-byte loads, all issued before the arithmetic
            const __half *kp = (const __half *)L.kc + ((size_t)key * p.KVH + kvh) * D;
            for (int d0 = 0; d0 < D; d0 += 64) {
                uint4 raw[8];
#pragma unroll
                for (int c8 = 0; c8 < 8; c8++) raw[c8] = d0 + c8 * 8 < D ? *reinterpret_cast<const uint4 *>(kp + d0 + c8 * 8) : make_uint4(0, 0, 0, 0);
#pragma unroll
                for (int c8 = 0; c8 < 8; c8++) {
                    if (d0 + c8 * 8 >= D) break;
                    const __half2 *hh = reinterpret_cast<const __half2 *>(&raw[c8]);
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        const float2 f = __half22float2(hh[e]);
                        dot = fmaf(q[d0 + c8 * 8 + 2 * e], f.x, dot);
                        dot = fmaf(q[d0 + c8 * 8 + 2 * e + 1], f.y, dot);
                    }
                }
            }
        } else {
            const float *kp = (const float *)L.kc + ((size_t)key * p.KVH + kvh) * D;
#pragma unroll 4
            for (int d = 0; d < D; d += 4) {
                const float4 f = *reinterpret_cast<const float4 *>(kp + d);
                dot = fmaf(q[d], f.x, dot), dot = fmaf(q[d + 1], f.y, dot), dot = fmaf(q[d + 2], f.z, dot), dot = fmaf(q[d + 3], f.w, dot);
            }
        }
        sc[j] = dot;
        lmax = fmaxf(lmax, dot);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) lmax = fmaxf(lmax, __shfl_xor_sync(0xffffffffu, lmax, o));
    if (lane == 0) sm.red[warp] = lmax;
    __syncthreads();
    float mx = -INFINITY;
    for (int i = 0; i < MEGA_WARPS; i++) mx = fmaxf(mx, sm.red[i]);
    __syncthreads();
    float lsum = 0.f;
    for (int j = tid; j < nk; j += MEGA_THREADS) {
        const float e = expf(sc[j] - mx);
        sc[j] = e;
        lsum += e;
    }
    const float total = block_sum_512(lsum, sm.red);
    for (int d0 = 0; d0 < D; d0 += 64) {  // warp w takes keys w, w+16, ...; lane owns dims 2*lane, 2*lane+1
        const int d = d0 + 2 * lane;
        float a0 = 0.f, a1 = 0.f;
        if (d < D)
#pragma unroll 4
            for (int j = warp; j < nk; j += MEGA_WARPS) {
                const int key = k0 + j;
                float v0, v1;
                if (key == pos) v0 = vn[d], v1 = vn[d + 1];
                else {
                    const size_t base = ((size_t)key * p.KVH + kvh) * D + d;
                    v0 = kv_get(L.vc, base, p.kv_f16), v1 = kv_get(L.vc, base + 1, p.kv_f16);
                }
                a0 = fmaf(sc[j], v0, a0), a1 = fmaf(sc[j], v1, a1);
            }
        if (d < D) wacc[warp * D + d] = a0, wacc[warp * D + d + 1] = a1;
    }
    __syncthreads();
    float *slot = p.att_part + ((size_t)h * MEGA_ATT_SPLITS + s) * (D + 2);
    for (int d = tid; d < D; d += MEGA_THREADS) {
        float a = 0.f;
        for (int w = 0; w < MEGA_WARPS; w++) a += wacc[w * D + d];
        slot[2 + d] = a;
    }
    if (tid == 0) slot[0] = mx, slot[1] = total;
}

// P3 input: merge the key slices of every head (online-softmax merge in slice order) into xin[0..C)
__device__ void merge_attention(const MParams &p, const MegaSmem &sm)
{
    const int D = p.D;
    for (int i = threadIdx.x; i < p.H * D; i += MEGA_THREADS) {
        const int idx = rotated(i, p.H * D);
        const int h = idx / D, d = idx - h * D;
        const float *base = p.att_part + (size_t)h * MEGA_ATT_SPLITS * (D + 2);
        float M = -INFINITY;
        for (int i = 0; i < MEGA_ATT_SPLITS; i++) M = fmaxf(M, __ldcg(base + i * (D + 2)));
        float Ls = 0.f, acc = 0.f;
        for (int i = 0; i < MEGA_ATT_SPLITS; i++) {
            const float mi = __ldcg(base + i * (D + 2)), li = __ldcg(base + i * (D + 2) + 1);
            if (li > 0.f) {
                const float w = expf(mi - M);
                Ls += li * w;
                acc = fmaf(__ldcg(base + i * (D + 2) + 2 + d), w, acc);
            }
        }
        sm.xin[idx] = acc / Ls;
    }
    __syncthreads();
}

// Tied lm_head: logits[n] = xin . embed[n, :] for this CTA's contiguous block of rows, plus its argmax candidate.
__device__ void lm_head_phase(const MParams &p, const MegaSmem &sm)
{
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int K = p.C, chunks = K >> 3;
    const int rows_cta = (p.V + gridDim.x - 1) / gridDim.x;
    const int n_begin = blockIdx.x * rows_cta, n_end = min(p.V, n_begin + rows_cta);
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    for (int n0 = n_begin + warp * 4; n0 < n_end; n0 += MEGA_WARPS * 4) {
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        for (int ck = lane; ck < chunks; ck += 32) {
            uint4 wv[4];
#pragma unroll
            for (int r = 0; r < 4; r++)
                wv[r] = n0 + r < n_end ? ldg_stream_v4(p.embed + (size_t)(n0 + r) * K + ck * 8) : make_uint4(0, 0, 0, 0);
            const float4 xa = *reinterpret_cast<const float4 *>(sm.xin + ck * 8);
            const float4 xb = *reinterpret_cast<const float4 *>(sm.xin + ck * 8 + 4);
#pragma unroll
            for (int r = 0; r < 4; r++) {
                const float2 w0 = __half22float2(u32_as_h2(wv[r].x)), w1 = __half22float2(u32_as_h2(wv[r].y));
                const float2 w2 = __half22float2(u32_as_h2(wv[r].z)), w3 = __half22float2(u32_as_h2(wv[r].w));
                float a = acc[r];
                a = fmaf(w0.x, xa.x, a), a = fmaf(w0.y, xa.y, a), a = fmaf(w1.x, xa.z, a), a = fmaf(w1.y, xa.w, a);
                a = fmaf(w2.x, xb.x, a), a = fmaf(w2.y, xb.y, a), a = fmaf(w3.x, xb.z, a), a = fmaf(w3.y, xb.w, a);
                acc[r] = a;
            }
        }
#pragma unroll
        for (int r = 0; r < 4; r++) {
            float v = acc[r];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0 && n0 + r < n_end) {
                p.logits[n0 + r] = v;
                if (v > best || (v == best && n0 + r < best_i)) best = v, best_i = n0 + r;
            }
        }
    }
    float *cv = sm.red;
    int *ci = reinterpret_cast<int *>(sm.red + MEGA_WARPS);
    if (lane == 0) cv[warp] = best, ci[warp] = best_i;
    __syncthreads();
    if (tid == 0) {
        for (int w = 1; w < MEGA_WARPS; w++)
            if (cv[w] > best || (cv[w] == best && ci[w] < best_i)) best = cv[w], best_i = ci[w];
        p.cand_val[blockIdx.x] = best;
        p.cand_idx[blockIdx.x] = best_i;
    }
}


__global__ void __launch_bounds__(MEGA_THREADS, 1) qwen_decode_mega_kernel(const MParams p)
{
    extern __shared__ uint4 mega_smem[];
    MegaSmem sm;
    const int kmax = max(p.C, p.I);
    sm.stride = (kmax >> 3) + 4;
    sm.xs_hi = mega_smem;
    sm.xs_lo = sm.xs_hi + 2 * sm.stride;
    sm.xin = reinterpret_cast<float *>(sm.xs_lo + 2 * sm.stride);
    sm.xsum = sm.xin + kmax;
    sm.red = sm.xsum + ((kmax >> 7) + 4);
    sm.misc = sm.red + 2 * MEGA_WARPS * 32 + 64;
    sm.flag = reinterpret_cast<int *>(sm.misc + 3 * p.D + max(3 * p.D, (p.max_t + MEGA_ATT_SPLITS - 1) / MEGA_ATT_SPLITS) + 4);

    const int tid = threadIdx.x;
    const int C = p.C, I = p.I;
    const int pos = *p.cache_len;  // nothing changes these two before the last barrier of the launch
    const uint32_t tok = min(*p.token, (uint32_t)(p.V - 1));
    int epoch = 0;
    ChunkRegs pre;
    bool has_pre = gemv_prefetch(p.layers[0].qkv, sm, pre);

    for (int l = 0; l < p.n_layer; l++) {
        const MLayer &L = p.layers[l];
        const float *xa_prev = p.xa + (size_t)((l + 1) & 1) * C;  // written by layer l - 1
        float *xa_cur = p.xa + (size_t)(l & 1) * C;
        const MLinear &prev_down = p.layers[l > 0 ? l - 1 : 0].down;
        // layer input x: the embedding row, or the previous layer's xa plus its down projection
        auto layer_input = [&](int d) {
            return l == 0 ? __half2float(p.embed[(size_t)tok * C + d])
                          : part_sum2(xa_prev, p.part_down, prev_down.R, nullptr, 0, C, d);
        };
        // ---- P1
#pragma unroll 2
        for (int i = tid; i < C; i += MEGA_THREADS) {
            const int d = rotated(i, C);
            sm.xin[d] = layer_input(d);
        }
        __syncthreads();
        rmsnorm_inplace(sm.xin, L.in_norm, C, p.eps, sm.red);
        gemv_phase(L.qkv, sm, p.part_qkv, pre, has_pre);
        if (!grid_barrier(p, epoch, sm)) return;
        // ---- P2
        attention_phase(p, L, sm, pos);
        has_pre = gemv_prefetch(L.o, sm, pre);
        if (!grid_barrier(p, epoch, sm)) return;
        // ---- P3
        merge_attention(p, sm);
        gemv_phase(L.o, sm, p.part_o, pre, has_pre);
        has_pre = gemv_prefetch(L.gu, sm, pre);
        if (!grid_barrier(p, epoch, sm)) return;
        // ---- P4: xa = x + o; CTA 0 keeps it for the next phases (ping-pong by layer parity)
#pragma unroll 2
        for (int i = tid; i < C; i += MEGA_THREADS) {
            const int d = rotated(i, C);
            const float v = l == 0 ? __half2float(p.embed[(size_t)tok * C + d]) + part_sum(p.part_o, L.o.R, C, d)
                                   : part_sum2(xa_prev, p.part_down, prev_down.R, p.part_o, L.o.R, C, d);
            sm.xin[d] = v;
            if (blockIdx.x == 0) xa_cur[d] = v;
        }
        __syncthreads();
        rmsnorm_inplace(sm.xin, L.post_norm, C, p.eps, sm.red);
        gemv_phase(L.gu, sm, p.part_gu, pre, has_pre);
        has_pre = gemv_prefetch(L.down, sm, pre);
        if (!grid_barrier(p, epoch, sm)) return;
        // ---- P5: act = silu(gate) * up (siluMulRef, src/reference/qwen-ref.ts:119-123)
        {
            // only the k-range of this CTA's unit is needed (a CTA with several units, or none, takes all / nothing)
            const MLinear &Ld = L.down;
            const int units = Ld.tiles * Ld.R;
            int k_lo = 0, k_hi = I;
            if ((int)blockIdx.x >= units) k_hi = 0;
            else if ((int)blockIdx.x + (int)gridDim.x >= units) {
                const int r = (int)blockIdx.x % Ld.R;
                k_lo = r * Ld.cpr * 128, k_hi = min(I, (r + 1) * Ld.cpr * 128);
            }
            const int span = k_hi - k_lo;
            for (int i0 = tid; i0 < span; i0 += 4 * MEGA_THREADS) {  // 8 loads in flight per thread, then the arithmetic
                float gt[4], up[4];
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const int i = k_lo + i0 + j * MEGA_THREADS;
                    gt[j] = i < k_hi ? part_sum(p.part_gu, L.gu.R, 2 * I, i) : 0.f;
                    up[j] = i < k_hi ? part_sum(p.part_gu, L.gu.R, 2 * I, I + i) : 0.f;
                }
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const int i = k_lo + i0 + j * MEGA_THREADS;
                    if (i < k_hi) sm.xin[i] = gt[j] / (1.f + expf(-gt[j])) * up[j];
                }
            }
        }
        __syncthreads();
        gemv_phase(L.down, sm, p.part_down, pre, has_pre);
        has_pre = l + 1 < p.n_layer ? gemv_prefetch(p.layers[l + 1].qkv, sm, pre) : false;
        if (!grid_barrier(p, epoch, sm)) return;
    }
    // ---- final norm, lm_head, argmax
    {
        const int l = p.n_layer - 1;
        const float *xa_last = p.xa + (size_t)(l & 1) * C;
        const MLinear &dn = p.layers[l].down;
        for (int d = tid; d < C; d += MEGA_THREADS) sm.xin[d] = __ldcg(xa_last + d) + part_sum(p.part_down, dn.R, C, d);
        __syncthreads();
        rmsnorm_inplace(sm.xin, p.final_norm, C, p.eps, sm.red);
        lm_head_phase(p, sm);
        if (!grid_barrier(p, epoch, sm)) return;
        if (blockIdx.x == 0 && tid < 32) {
            float best = -INFINITY;
            int best_i = 0x7fffffff;
            for (int i = tid; i < (int)gridDim.x; i += 32) {
                const float v = __ldcg(p.cand_val + i);
                const int ix = __ldcg(p.cand_idx + i);
                if (v > best || (v == best && ix < best_i)) best = v, best_i = ix;
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float v = __shfl_xor_sync(0xffffffffu, best, o);
                const int ix = __shfl_xor_sync(0xffffffffu, best_i, o);
                if (v > best || (v == best && ix < best_i)) best = v, best_i = ix;
            }
            if (tid == 0) {
                const uint32_t next = best_i == 0x7fffffff ? 0u : (uint32_t)best_i;
                *p.token = next;
                p.history[*p.step] = next;
                *p.step += 1;
                *p.cache_len = pos + 1;
            }
        }
    }
}

// ------------------------------------------------------------------------------------------------ host

static int carve_bytes(wb_context *ctx, uint64_t bytes, void **out)
{
    uint64_t off = 0;
    WB_CHECK(wb_arena_alloc(ctx, WB_ARENA_WEIGHTS, bytes, &off));
    *out = ctx->arena[WB_ARENA_WEIGHTS].base + off;
    return WB_OK;
}

static bool linear_ok(const wb_context *ctx, int h)
{
    if (h < 0) return false;
    const Weight &w = ctx->weights[h];
    return w.kind == WeightKind::Gptq && w.K % 128 == 0 && w.N % 4 == 0 && w.group % 128 == 0;
}

bool mega_supported(const wb_qwen *m)
{
    if (m->layers.empty() || m->layers[0].qkv < 0 || m->layers[0].gate_up < 0) return false;
    if (m->D % 2 || m->D > 128 || m->C % 8 || m->I % 8) return false;
    for (const LayerW &L : m->layers)
        if (!linear_ok(m->ctx, L.qkv) || !linear_ok(m->ctx, L.o) || !linear_ok(m->ctx, L.gate_up) || !linear_ok(m->ctx, L.down))
            return false;
    return m->ctx->weights[m->embed].kind == WeightKind::DenseF16;
}

static MLinear make_linear(const wb_context *ctx, int h, int bias, int grid)
{
    const Weight &w = ctx->weights[h];
    const char *base = ctx->arena[WB_ARENA_WEIGHTS].base;
    MLinear L{};
    L.qw = (const uint32_t *)(base + w.off_main);
    L.qz = w.has_zeros ? (const uint32_t *)(base + w.off_zeros) : nullptr;
    L.sc = (const __half *)(base + w.off_scales);
    L.bias = bias >= 0 ? (const float *)(base + ctx->weights[bias].off_main) : nullptr;
    L.K = (int)w.K, L.N = (int)w.N;
    L.chunks = (int)(w.K / 128);
    L.tiles = (int)((w.N + 31) / 32);
    L.zcols = (int)w.zcols;
    L.group_chunks = (int)(w.group / 128);
    // ranges of chunks per column tile: enough units to occupy the grid, at most one chunk per warp and unit
    int R = L.tiles >= grid ? 1 : grid / L.tiles;
    const int min_r = (L.chunks + MEGA_WARPS - 1) / MEGA_WARPS;  // a unit has 16 warps
    if (R < min_r) R = min_r;
    if (R > L.chunks) R = L.chunks;
    L.cpr = (L.chunks + R - 1) / R;
    L.R = (L.chunks + L.cpr - 1) / L.cpr;
    return L;
}

static int mega_prepare(wb_qwen *m)
{
    wb_context *ctx = m->ctx;
    std::unique_ptr<Mega> mg(new Mega());
    int coop = 0;
    WB_CUDA(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, ctx->device));
    if (!coop) return fail(WB_ERR_UNSUPPORTED, "device does not support cooperative launches");
    const int kmax = std::max(m->C, m->I), stride = (kmax >> 3) + 4;
    mg->smem = (size_t)4 * stride * 16 + (size_t)kmax * 4 + ((kmax >> 7) + 4) * 4 + (2 * MEGA_WARPS * 32 + 64) * 4 +
               (3 * m->D + std::max(3 * m->D, (m->cfg.max_t + MEGA_ATT_SPLITS - 1) / MEGA_ATT_SPLITS) + 4) * 4 + 64;
    WB_CUDA(cudaFuncSetAttribute(qwen_decode_mega_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)mg->smem));
    int per_sm = 0;
    WB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, qwen_decode_mega_kernel, MEGA_THREADS, mg->smem));
    if (per_sm < 1) return fail(WB_ERR_UNSUPPORTED, "the decode kernel does not fit on an SM");
    mg->grid = ctx->sm_count;  // one CTA per SM; all of them are resident, which the grid barrier relies on
    if (mg->grid < m->H * MEGA_ATT_SPLITS)
        return fail(WB_ERR_UNSUPPORTED, "%d heads x %d key slices need more CTAs than the %d SMs", m->H, MEGA_ATT_SPLITS, mg->grid);

    std::vector<MLayer> layers(m->cfg.n_layer);
    const size_t layer_stride = (size_t)m->cfg.max_t * m->KV * (m->cfg.kv_dtype == WB_F16 ? 2 : 4);
    int rq = 0, ro = 0, rg = 0, rd = 0;
    for (int i = 0; i < m->cfg.n_layer; i++) {
        const LayerW &L = m->layers[i];
        MLayer &d = layers[i];
        d.qkv = make_linear(ctx, L.qkv, L.qkvb, mg->grid);
        d.o = make_linear(ctx, L.o, -1, mg->grid);
        d.gu = make_linear(ctx, L.gate_up, -1, mg->grid);
        d.down = make_linear(ctx, L.down, -1, mg->grid);
        const char *base = ctx->arena[WB_ARENA_WEIGHTS].base;
        d.in_norm = (const float *)(base + ctx->weights[L.in_norm].off_main);
        d.post_norm = (const float *)(base + ctx->weights[L.post_norm].off_main);
        d.kc = m->k_cache + i * layer_stride;
        d.vc = m->v_cache + i * layer_stride;
        rq = std::max(rq, d.qkv.R), ro = std::max(ro, d.o.R), rg = std::max(rg, d.gu.R), rd = std::max(rd, d.down.R);
    }
    MParams &p = mg->p;
    WB_CHECK(carve_bytes(ctx, layers.size() * sizeof(MLayer), (void **)&mg->d_layers));
    WB_CUDA(cudaMemcpyAsync(mg->d_layers, layers.data(), layers.size() * sizeof(MLayer), cudaMemcpyHostToDevice, ctx->stream));
    p.layers = mg->d_layers;
    p.n_layer = m->cfg.n_layer, p.C = m->C, p.H = m->H, p.KVH = m->KVH, p.D = m->D, p.KV = m->KV, p.I = m->I, p.V = m->V;
    p.max_t = m->cfg.max_t, p.kv_f16 = m->cfg.kv_dtype == WB_F16, p.eps = m->cfg.rms_eps;
    const char *base = ctx->arena[WB_ARENA_WEIGHTS].base;
    p.embed = (const __half *)(base + ctx->weights[m->embed].off_main);
    p.final_norm = (const float *)(base + ctx->weights[m->final_norm].off_main);
    p.cs_table = m->cs_table;
    p.cache_len = m->d_cache_len, p.step = m->d_step, p.token = m->dec.tokens, p.history = m->d_history;
    p.logits = m->dec.logits;
    const int Nq = m->C + 2 * m->KV;
    WB_CHECK(carve_bytes(ctx, (uint64_t)2 * m->C * 4, (void **)&p.xa));
    WB_CHECK(carve_bytes(ctx, (uint64_t)rq * Nq * 4, (void **)&p.part_qkv));
    WB_CHECK(carve_bytes(ctx, (uint64_t)ro * m->C * 4, (void **)&p.part_o));
    WB_CHECK(carve_bytes(ctx, (uint64_t)rg * 2 * m->I * 4, (void **)&p.part_gu));
    WB_CHECK(carve_bytes(ctx, (uint64_t)rd * m->C * 4, (void **)&p.part_down));
    WB_CHECK(carve_bytes(ctx, (uint64_t)m->H * MEGA_ATT_SPLITS * (m->D + 2) * 4, (void **)&p.att_part));
    WB_CHECK(carve_bytes(ctx, (uint64_t)mg->grid * 4, (void **)&p.cand_val));
    WB_CHECK(carve_bytes(ctx, (uint64_t)mg->grid * 4, (void **)&p.cand_idx));
    void *sync_words = nullptr;
    WB_CHECK(carve_bytes(ctx, 512, &sync_words));
    WB_CUDA(cudaMemsetAsync(sync_words, 0, 512, ctx->stream));
    p.barrier = (unsigned long long *)sync_words;
    p.abort_flag = (int *)sync_words + 4;
    p.status = ctx->status_word;
    mg->barriers_per_launch = 5 * m->cfg.n_layer + 1;
    WB_CUDA(cudaStreamSynchronize(ctx->stream));
    m->mega = mg.release();
    return WB_OK;
}

int mega_decode(wb_qwen *m, int64_t n_steps)
{
    wb_context *ctx = m->ctx;
    if (!m->mega) WB_CHECK(mega_prepare(m));
    Mega *mg = m->mega;
    for (int64_t s = 0; s < n_steps; s++) {
        mg->p.bar_base = mg->launches * (unsigned long long)mg->barriers_per_launch * (unsigned long long)mg->grid;
        void *args[] = {(void *)&mg->p};
        WB_CUDA(cudaLaunchCooperativeKernel((const void *)qwen_decode_mega_kernel, dim3(mg->grid), dim3(MEGA_THREADS), args,
                                            mg->smem, ctx->stream));
        mg->launches++;
        ctx->launches++;
    }
    return WB_OK;
}

void mega_destroy(wb_qwen *m)
{
    delete m->mega;
    m->mega = nullptr;
}

}  // namespace wbq
