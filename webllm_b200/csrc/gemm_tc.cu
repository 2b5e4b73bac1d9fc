// Prefill / batched linear on the 5th-generation tensor cores: C[M,N] = A[M,K] . W[N,K]^T (+bias) with
// W either GPTQ int4 (unpacked inside the kernel) or dense fp16. Replaces gemm_nt_f16_from_f32.wgsl
// (src/gpu/kernels/gemm/gemm_nt_f16_from_f32.wgsl:39-95), the tiled GEMM behind QwenGpt.gemm for M > 1
// (src/model/qwen.ts:613-617).
//
// One CTA computes a (128 * NH output columns n) x (MT tokens m) tile of C^T, NH = 1 or 2: each 128-column half of
// the weight tile is the 128-row operand of a tcgen05.mma, the activation tile the MT-column operand both halves
// share, and each half has its f32 accumulator in TMEM (128 lanes x MT columns). With NH = 2 an activation tile
// fetched from L2 feeds twice the arithmetic. Roles, 21 warps (which warp id has which role, and why, is at MMA_WARP in
// gemm_tc.cuh: the issuing warp shares its warp scheduler with no unpack warp):
//   TMA warp    producer: per 64-k block one box of activations [MT x 64] fp16 (128-byte swizzle) and one box of
//               packed weights [8 packed rows x 128 * NH columns] int32, into a ring of up to 8 stages (as many as
//               fit the shared memory). The weight boxes of the first stages are requested before the wait on the
//               previous kernel (the weights are constants), the activation boxes after it.
//   MMA warp    allocates TMEM, then one elected lane issues 4 x NH tcgen05.mma (K = 16 each) per block, after ONE
//               wait (the unpack sets' barrier, which covers the boxes), and commits the stage back to the producer.
//   16 unpack   warps, in 4 / NH sets of one thread per column that take the k-blocks in turn: a thread turns
//               the 8 words of its column into 64 fp16 values w = (q - zero) * scale (exact integer in fp16, one
//               rounding in the multiply: the fp16 weight the reference uploads, src/gpu/buffer.ts:103-120) and
//               stores them as the K-major, 128-byte-swizzled operand tile; the scale and zero point of the
//               set's next k-block are requested while the current one is unpacked.
//   epilogue    all 21 warps drain TMEM (tcgen05.ld, the lane quarter id % 4), add the bias and store, after the wait
//               on the previous kernel.
// With the unpack's work left out the rest of the kernel runs at 0.84 of the cuBLAS fp16 rate; with it, at 0.82.
// Every wait on an mbarrier is bounded: when a wait gives up it raises a CTA-wide abort flag, records a
// code in the context's status word, and all roles fall through to the common exit where TMEM is freed.
#include "gemm_tc.cuh"

namespace wb {

namespace tc {

template <int MT, bool DENSE, int NH, int EXTRA = 0>
struct Smem {
    static constexpr int COLS = BN * NH;  // output columns per CTA
    static constexpr int X_BYTES = MT * BK * 2;
    static constexpr int WD_BYTES = COLS * BK * 2;
    static constexpr int WP_BYTES = DENSE ? 0 : 8 * COLS * 4;
    static constexpr int STAGE_BYTES = X_BYTES + WD_BYTES + WP_BYTES;  // every piece is a multiple of 1024
    static constexpr int FIT = (227 * 1024 - 1280 - EXTRA) / STAGE_BYTES;
    static constexpr int STAGES = FIT > 8 ? 8 : FIT;  // small tiles are latency-bound: as deep as the barrier area allows
    static constexpr int TOTAL = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/ + EXTRA;
    static_assert(TOTAL <= 227 * 1024, "tile does not fit the shared memory of one CTA");
    
};

// GATHER: the epilogue stores to the placement in Params (several destinations, row pitch ld_out) instead of to the
// dense local result; a template parameter so that the plain kernel's code is untouched by it.
template <int MT, bool DENSE, bool SPLIT, int NH, bool GATHER = false>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, const Params p)
{
    using S = Smem<MT, DENSE, NH>;
    constexpr int STAGES = S::STAGES;
    constexpr int COLS = S::COLS;
    constexpr uint32_t ACC_COLS = MT < 32 ? 32 : MT;  // TMEM columns of one accumulator
    // TMEM is allocated in powers of two (the 192-token tile takes 256 or 512 columns)
    constexpr uint32_t TMEM_COLS = ACC_COLS * NH <= 32 ? 32 : ACC_COLS * NH <= 64 ? 64 : ACC_COLS * NH <= 128 ? 128
                                   : ACC_COLS * NH <= 256 ? 256 : 512;
    static_assert(ACC_COLS * NH <= 512, "accumulators exceed the tensor memory");
    // The unpack warps form KG sets of one thread per column; set g unpacks k-blocks g, g + KG, ... so that KG
    // k-blocks are in the works at once and a warp pays the waits and the fence of a block once per 8 packed rows.
    constexpr int KG = 32 * UNPACK_WARPS / COLS;
    static_assert(KG <= STAGES && UNPACK_WARPS % KG == 0 && (32 * UNPACK_WARPS / KG) % COLS == 0, "unpack sets");
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t *bars = (uint64_t *)(smem + STAGES * S::STAGE_BYTES);
    uint64_t *full = bars, *deq = bars + STAGES, *empty = bars + 2 * STAGES, *acc_full = bars + 3 * STAGES;
    uint32_t *tmem_slot = (uint32_t *)(bars + 3 * STAGES + 1);
    volatile int *abort_flag = (volatile int *)(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.x * MT, n0 = blockIdx.y * COLS;
    // split-K: slice blockIdx.z covers k-blocks [kb0, KB); the ring's stage and phase count from the slice start
    // (SPLIT is a template parameter so that the unsplit kernel keeps compile-time zero here)
    const int kb0 = SPLIT ? blockIdx.z * p.kb_per_slice : 0;
    const int KB = SPLIT ? min(p.K / BK, kb0 + p.kb_per_slice) : p.K / BK;

    auto xs = [&](int s) { return smem + s * S::STAGE_BYTES; };
    auto wd = [&](int s) { return smem + s * S::STAGE_BYTES + S::X_BYTES; };
    auto wp = [&](int s) { return (uint32_t *)(smem + s * S::STAGE_BYTES + S::X_BYTES + S::WD_BYTES); };

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&deq[s], UNPACK_WARPS / KG);
            mbar_init(&empty[s], 1);
        }
        mbar_init(acc_full, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == MMA_WARP) tmem_alloc(tmem_slot, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // Everything above (barriers, TMEM) ran under the tail of the previous kernel when this one was launched with
    // programmatic stream serialization. The weights are constants: their first boxes are requested before the wait
    // on that kernel; the activation loads and the result stores come after it.
    pdl_trigger();

    bool ok = true;
    if (warp == TMA_WARP) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            auto load_w = [&](int s, int kb) {
                if constexpr (DENSE) tma_load_2d(wd(s), &map_w, kb * BK, n0, &full[s]);
                else tma_load_2d(wp(s), &map_w, n0, kb * 8, &full[s]);
            };
            int pre = 0;
            for (int kb = kb0; kb < KB && pre < STAGES; kb++, pre++) {  // fresh stages: nothing to wait for
                mbar_expect_tx(&full[pre], S::X_BYTES + (DENSE ? S::WD_BYTES : S::WP_BYTES));
                load_w(pre, kb);
            }
            pdl_wait();
            int s = 0;
            uint32_t ph = 0;
            for (int kb = kb0; kb < KB; kb++) {
                if (!mbar_wait(&empty[s], ph ^ 1, abort_flag, p.status, 1)) break;
                if (kb - kb0 >= pre) {
                    mbar_expect_tx(&full[s], S::X_BYTES + (DENSE ? S::WD_BYTES : S::WP_BYTES));
                    load_w(s, kb);
                }
                tma_load_2d(xs(s), &map_x, kb * BK, m0, &full[s]);
                if (++s == STAGES) s = 0, ph ^= 1;
            }
        }
        __syncwarp();
    } else if (warp == MMA_WARP) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = idesc_f16(BN, MT);
            int s = 0;
            uint32_t ph = 0;
            for (int kb = kb0; kb < KB && ok; kb++) {
                // the unpack sets waited for the stage's boxes themselves: their barrier covers both
                ok = DENSE ? mbar_wait(&full[s], ph, abort_flag, p.status, 2) : mbar_wait(&deq[s], ph, abort_flag, p.status, 3);
                if (!ok) break;
                tc_fence_after();
                const uint64_t a0 = smem_desc_sw128(smem_u32(wd(s)));
                const uint64_t b0 = smem_desc_sw128(smem_u32(xs(s)));
#pragma unroll
                for (int k = 0; k < BK / 16; k++) {  // 16 fp16 = 32 bytes = 2 descriptor units along K
#pragma unroll
                    for (int h = 0; h < NH; h++)  // the halves of the weight tile are 128 rows = 16 KB = 1024 units apart
                        umma_f16(tmem_base + h * ACC_COLS, a0 + 1024 * h + 2 * k, b0 + 2 * k, idesc, ((kb - kb0) | k) != 0);
                }
                umma_commit(&empty[s]);
                if (++s == STAGES) s = 0, ph ^= 1;
            }
            if (ok) umma_commit(acc_full);
        }
        __syncwarp();
    } else if (is_unpack_warp(warp)) {
        // ------------------------------------------------------------------ unpack
        constexpr int SET_THREADS = 32 * UNPACK_WARPS / KG;
        constexpr int RPT = 8 * COLS / SET_THREADS;    // packed rows of a k-block per thread: 8 rows x COLS words in all
        const int ut = unpack_index(warp) * 32 + lane;
        const int kg = ut / SET_THREADS;          // which set
        const int tn = ut % SET_THREADS % COLS;   // column of the tile
        const int rhalf = ut % SET_THREADS / COLS;  // which RPT of the 8 packed rows
        if constexpr (!DENSE) {
            const int n = n0 + tn;
            const bool n_ok = n < p.N;
            __half2 scale2 = __float2half2_rn(0.f), zsub = scale2, zfma = scale2;
            const __half2 sixteenth = __float2half2_rn(0.0625f);
            // scale and zero point of a group are requested one group ahead, so that the trip to L2 overlaps the
            // unpack of the current group instead of standing in front of it
            const int n_groups = p.K / (p.group_blocks * BK);
            __half next_scale = __float2half_rn(0.f);
            uint32_t next_zeros = 0x77777777u;  // stored zero - 1 = 7: the symmetric default
            auto request_group = [&](int g) {
                if (n_ok && g < n_groups) {
                    next_scale = p.sc[(int64_t)g * p.N + n];
                    if (p.qz) next_zeros = p.qz[(int64_t)g * p.zcols + (n >> 3)];
                }
            };
            // the set's first k-block, its group and position in the group; both advance without a division
            int group = (kb0 + kg) / p.group_blocks, in_group = (kb0 + kg) % p.group_blocks;
            bool fresh = true;  // next_scale / next_zeros hold a group that is not applied yet
            if (kb0 + kg < KB) request_group(group);
            // loop-invariant addressing: the thread's first word in a stage and the swizzled 16-byte slots it fills
            const int src_off = S::X_BYTES + S::WD_BYTES + (tn + rhalf * RPT * COLS) * 4;
            int dst_off[RPT];
#pragma unroll
            for (int rr = 0; rr < RPT; rr++)  // 16-byte chunk r of row tn, at its 128-byte-swizzle position
                dst_off[rr] = S::X_BYTES + tn * 128 + (((rhalf * RPT + rr) ^ (tn & 7)) << 4);
            int s = kg;
            uint32_t ph = 0;
            for (int kb = kb0 + kg; kb < KB; kb += KG) {
                if (fresh) {
                    const float z = (float)(((next_zeros >> ((n & 7) * 4)) & 15u) + 1u);
                    scale2 = __half2half2(next_scale);
                    zsub = __float2half2_rn(1024.f + z);
                    zfma = __float2half2_rn(-(64.f + z));
                    fresh = false;
                }
                // the group of the set's next k-block is requested now and lands while this one is unpacked
                in_group += KG;
                if (in_group >= p.group_blocks) {
                    do in_group -= p.group_blocks, group++;
                    while (in_group >= p.group_blocks);
                    request_group(group);
                    fresh = true;
                }
                ok = mbar_wait(&full[s], ph, abort_flag, p.status, 4);
                if (!ok) break;
                uint8_t *stage = smem + s * S::STAGE_BYTES;
                const uint32_t *src = (const uint32_t *)(stage + src_off);
#pragma unroll
                for (int rr = 0; rr < RPT; rr++) {
                    uint32_t w = src[rr * COLS];
                    const uint32_t lo0 = (w & 0x000f000fu) | 0x64006400u;
                    const uint32_t hi0 = (w & 0x00f000f0u) | 0x64006400u;
                    w >>= 8;
                    const uint32_t lo1 = (w & 0x000f000fu) | 0x64006400u;
                    const uint32_t hi1 = (w & 0x00f000f0u) | 0x64006400u;
                    const __half2 a = __hmul2(__hsub2(*(const __half2 *)&lo0, zsub), scale2);          // k0, k4
                    const __half2 b = __hmul2(__hfma2(*(const __half2 *)&hi0, sixteenth, zfma), scale2);  // k1, k5
                    const __half2 c = __hmul2(__hsub2(*(const __half2 *)&lo1, zsub), scale2);          // k2, k6
                    const __half2 d = __hmul2(__hfma2(*(const __half2 *)&hi1, sixteenth, zfma), scale2);  // k3, k7
                    const uint32_t ua = *(const uint32_t *)&a, ub = *(const uint32_t *)&b;
                    const uint32_t uc = *(const uint32_t *)&c, ud = *(const uint32_t *)&d;
                    uint4 o;
                    o.x = __byte_perm(ua, ub, 0x5410);
                    o.y = __byte_perm(uc, ud, 0x5410);
                    o.z = __byte_perm(ua, ub, 0x7632);
                    o.w = __byte_perm(uc, ud, 0x7632);
                    *(uint4 *)(stage + dst_off[rr]) = o;
                }
                fence_async_smem();  // make the generic-proxy stores visible to the tensor core's reads
                __syncwarp();
                if (lane == 0) mbar_arrive(&deq[s]);
                s += KG;
                if (s >= STAGES) s -= STAGES, ph ^= 1;
            }
        }
    }
    // ---------------------------------------------------------------------- epilogue, all 21 warps: warp w may touch
    // TMEM lanes 32 * (w % 4) .. + 31; the warps of a lane quarter (six for quarter 0, five for the others) take the
    // 16-token blocks of the accumulator in turn
    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;  // the single-thread roles report for their warp
    pdl_wait();  // nothing is stored before the kernel before this one is done
    {
        if (ok) ok = mbar_wait(acc_full, 0, abort_flag, p.status, 5);
        if (ok) {
            tc_fence_after();
            const int q = warp & 3;
            // split-K: slices write f32 partial sums, splitk_reduce_kernel adds them and the bias
            constexpr bool split = SPLIT;
            float *part = SPLIT ? p.partial + (int64_t)blockIdx.z * p.M * p.N : nullptr;
            const int share = q == 0 ? 6 : 5;  // warps of this lane quarter
            const int c_begin = (warp >> 2) * 16, c_step = share * 16;
            // where the block goes: this slice's f32 partial sums, the dense local result, or the placement of a
            // column-sharded call
            StoreDst d;
            bool out16;
            if (split) {
                d.dst[0] = part, d.n_dst = 1, d.ld = p.N, d.col0 = 0, out16 = false;
            } else if constexpr (GATHER) {
#pragma unroll
                for (int g = 0; g < kMaxGatherDst; g++) d.dst[g] = p.dst[g];
                d.n_dst = p.n_dst, d.ld = p.ld_out, d.col0 = p.col0, out16 = p.out_f16 != 0;
            } else {
                d.dst[0] = p.out, d.n_dst = 1, d.ld = p.N, d.col0 = 0, out16 = p.out_f16 != 0;
            }
            const bool vec = (p.N & 7) == 0 && (d.ld & 7) == 0 && (d.col0 & 7) == 0;
#pragma unroll 1
            for (int h = 0; h < NH; h++) {
                const int n_warp = n0 + h * BN + q * 32;
                const int n = n_warp + lane;
                const float bias = (!split && p.bias && n < p.N) ? p.bias[n] : 0.f;
#pragma unroll 1
                for (int c = c_begin; c < MT; c += c_step) {
                    uint32_t r[16];
                    tmem_ld_32x32b_x16(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(h * ACC_COLS + c), r);
                    tmem_ld_wait();
                    store_block16<GATHER>(d, out16, vec, r, bias, m0 + c, p.M, n_warp, p.N, lane);
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == MMA_WARP) tmem_dealloc(tmem_base, TMEM_COLS);
}

// ----------------------------------------------------------------------------------------------------
// Persistent variant, for launches with more tiles than SMs and no K split: one CTA per SM walks the tiles
// t = blockIdx.x, + gridDim.x, ... (tile t covers token tile t % tiles_m of weight-column tile t / tiles_m, so the
// CTAs that run at the same time share weight columns in L2). The TMA ring and the unpack run on across tile
// boundaries, the accumulators are double-buffered in TMEM wherever two sets fit its 512 columns, and four warps of
// their own drain a finished accumulator while the MMAs of the next tile are issued: pipeline fill, TMEM drain and
// the stores (to peers too, in a column-sharded call) leave the critical path of every tile but the last.
// Roles as above plus four epilogue warps (ids 21 .. 24, TMEM lane quarter id % 4): 25 warps.
constexpr int EPI_WARPS = 4;         // warps 21 .. 24, after the roles listed at MMA_WARP
constexpr int kGatherStageBytes = 16384;  // staging tile of a column-sharded call's epilogue: [64][128] fp16 or [32][128] f32
constexpr int THREADS_P = 32 * (WARPS + EPI_WARPS);

template <int MT, bool DENSE, int NH, bool GATHER>
__global__ void __launch_bounds__(THREADS_P, 1)
gemm_tc_persist_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, const Params p,
                       const int tiles_m, const int n_tiles)
{
    using S = Smem<MT, DENSE, NH, GATHER ? kGatherStageBytes : 0>;
    constexpr int STAGES = S::STAGES;
    constexpr int COLS = S::COLS;
    constexpr uint32_t ACC_COLS = MT < 32 ? 32 : MT;
    constexpr uint32_t ACC_ALL = ACC_COLS * NH;             // TMEM columns of one tile's accumulators
    constexpr int NBUF = 2 * ACC_ALL <= 512 ? 2 : 1;        // accumulator sets
    constexpr uint32_t USED = ACC_ALL * NBUF;
    constexpr uint32_t TMEM_COLS = USED <= 32 ? 32 : USED <= 64 ? 64 : USED <= 128 ? 128 : USED <= 256 ? 256 : 512;
    static_assert(USED <= 512, "accumulators exceed the tensor memory");
    constexpr int KG = 32 * UNPACK_WARPS / COLS;
    static_assert(KG <= STAGES && UNPACK_WARPS % KG == 0 && (32 * UNPACK_WARPS / KG) % COLS == 0, "unpack sets");
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t *bars = (uint64_t *)(smem + STAGES * S::STAGE_BYTES);
    uint64_t *full = bars, *deq = bars + STAGES, *empty = bars + 2 * STAGES;
    uint64_t *acc_full = bars + 3 * STAGES, *acc_empty = bars + 3 * STAGES + 2;
    uint32_t *tmem_slot = (uint32_t *)(bars + 3 * STAGES + 4);
    volatile int *abort_flag = (volatile int *)(tmem_slot + 1);
    static_assert((3 * STAGES + 4) * 8 + 8 <= 256, "barrier area");

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int KBt = p.K / BK;  // k-blocks per tile
    const int tiles_cta = (int)blockIdx.x < n_tiles ? (n_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
    auto tile_m0 = [&](int ti) { return (((int)blockIdx.x + ti * (int)gridDim.x) % tiles_m) * MT; };
    auto tile_n0 = [&](int ti) { return (((int)blockIdx.x + ti * (int)gridDim.x) / tiles_m) * COLS; };

    auto xs = [&](int s) { return smem + s * S::STAGE_BYTES; };
    auto wd = [&](int s) { return smem + s * S::STAGE_BYTES + S::X_BYTES; };
    auto wp = [&](int s) { return (uint32_t *)(smem + s * S::STAGE_BYTES + S::X_BYTES + S::WD_BYTES); };

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&deq[s], UNPACK_WARPS / KG);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], EPI_WARPS);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == MMA_WARP) tmem_alloc(tmem_slot, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // Everything above (barriers, TMEM) ran under the tail of the previous kernel when this one was launched with
    // programmatic stream serialization; the first weight boxes are requested before the wait on that kernel, the
    // activation loads and the result stores come after it.
    pdl_trigger();

    if (warp == TMA_WARP) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            auto load_w = [&](int s, int kb, int n0) {
                if constexpr (DENSE) tma_load_2d(wd(s), &map_w, kb * BK, n0, &full[s]);
                else tma_load_2d(wp(s), &map_w, n0, kb * 8, &full[s]);
            };
            int pre = 0;
            for (int ti = 0; ti < tiles_cta && pre < STAGES; ti++)
                for (int kb = 0; kb < KBt && pre < STAGES; kb++, pre++) {  // fresh stages: nothing to wait for
                    mbar_expect_tx(&full[pre], S::X_BYTES + (DENSE ? S::WD_BYTES : S::WP_BYTES));
                    load_w(pre, kb, tile_n0(ti));
                }
            pdl_wait();
            int s = 0, seq = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int ti = 0; ti < tiles_cta && ok; ti++) {
                const int m0 = tile_m0(ti), n0 = tile_n0(ti);
                for (int kb = 0; kb < KBt; kb++, seq++) {
                    ok = mbar_wait(&empty[s], ph ^ 1, abort_flag, p.status, 1);
                    if (!ok) break;
                    if (seq >= pre) {
                        mbar_expect_tx(&full[s], S::X_BYTES + (DENSE ? S::WD_BYTES : S::WP_BYTES));
                        load_w(s, kb, n0);
                    }
                    tma_load_2d(xs(s), &map_x, kb * BK, m0, &full[s]);
                    if (++s == STAGES) s = 0, ph ^= 1;
                }
            }
        }
    } else if (warp == MMA_WARP) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = idesc_f16(BN, MT);
            bool ok = true;
            int s = 0;
            uint32_t ph = 0;
            for (int ti = 0; ti < tiles_cta && ok; ti++) {
                const int buf = ti % NBUF, use = ti / NBUF;  // `use` earlier tiles went through this accumulator set
                if (use > 0) ok = mbar_wait(&acc_empty[buf], (uint32_t)(use - 1) & 1u, abort_flag, p.status, 6);
                if (!ok) break;
                tc_fence_after();
                const uint32_t acc = tmem_base + (uint32_t)buf * ACC_ALL;
                for (int kb = 0; kb < KBt; kb++) {
                    ok = DENSE ? mbar_wait(&full[s], ph, abort_flag, p.status, 2) : mbar_wait(&deq[s], ph, abort_flag, p.status, 3);
                    if (!ok) break;
                    tc_fence_after();
                    const uint64_t a0 = smem_desc_sw128(smem_u32(wd(s)));
                    const uint64_t b0 = smem_desc_sw128(smem_u32(xs(s)));
#pragma unroll
                    for (int k = 0; k < BK / 16; k++) {
#pragma unroll
                        for (int h = 0; h < NH; h++)
                            umma_f16(acc + h * ACC_COLS, a0 + 1024 * h + 2 * k, b0 + 2 * k, idesc, (kb | k) != 0);
                    }
                    umma_commit(&empty[s]);
                    if (++s == STAGES) s = 0, ph ^= 1;
                }
                if (ok) umma_commit(&acc_full[buf]);
            }
        }
        __syncwarp();
    } else if (is_unpack_warp(warp)) {
        // ------------------------------------------------------------------ unpack: the sets take the k-blocks of the
        // CTA's whole sequence (tile after tile) in turn
        if constexpr (!DENSE) {
            constexpr int SET_THREADS = 32 * UNPACK_WARPS / KG;
            constexpr int RPT = 8 * COLS / SET_THREADS;
            const int ut = unpack_index(warp) * 32 + lane;
            const int kg = ut / SET_THREADS;
            const int tn = ut % SET_THREADS % COLS;
            const int rhalf = ut % SET_THREADS / COLS;
            const __half2 sixteenth = __float2half2_rn(0.0625f);
            const int src_off = S::X_BYTES + S::WD_BYTES + (tn + rhalf * RPT * COLS) * 4;
            int dst_off[RPT];
#pragma unroll
            for (int rr = 0; rr < RPT; rr++) dst_off[rr] = S::X_BYTES + tn * 128 + (((rhalf * RPT + rr) ^ (tn & 7)) << 4);
            // position of the set's current item: tile index in the CTA's sequence, k-block in the tile, its group
            int ti = 0, kb = kg;
            while (kb >= KBt) kb -= KBt, ti++;
            int group = kb / p.group_blocks, in_group = kb % p.group_blocks;
            // scale and zero point are requested one item ahead, and only when the item's tile or group differs
            __half next_scale = __float2half_rn(0.f);
            uint32_t next_zeros = 0x77777777u;
            int n = tile_n0(ti) + tn;  // this thread's column in the current tile
            auto request = [&]() {
                next_scale = __float2half_rn(0.f), next_zeros = 0x77777777u;
                if (ti < tiles_cta && n < p.N) {
                    next_scale = p.sc[(int64_t)group * p.N + n];
                    if (p.qz) next_zeros = p.qz[(int64_t)group * p.zcols + (n >> 3)] >> ((n & 7) * 4);
                }
            };
            request();
            bool fresh = true;
            __half2 scale2 = __float2half2_rn(0.f), zsub = scale2, zfma = scale2;
            int s = kg;
            uint32_t ph = 0;
            bool ok = true;
            while (ti < tiles_cta && ok) {
                if (fresh) {
                    const float z = (float)((next_zeros & 15u) + 1u);
                    scale2 = __half2half2(next_scale);
                    zsub = __float2half2_rn(1024.f + z);
                    zfma = __float2half2_rn(-(64.f + z));
                    fresh = false;
                }
                // advance to the set's next item; a new tile or group is requested now and lands during this unpack
                kb += KG, in_group += KG;
                if (kb >= KBt) {
                    do kb -= KBt, ti++;
                    while (kb >= KBt);
                    n = tile_n0(ti) + tn;
                    group = kb / p.group_blocks, in_group = kb % p.group_blocks;
                    request();
                    fresh = true;
                } else if (in_group >= p.group_blocks) {
                    do in_group -= p.group_blocks, group++;
                    while (in_group >= p.group_blocks);
                    request();
                    fresh = true;
                }
                ok = mbar_wait(&full[s], ph, abort_flag, p.status, 4);
                if (!ok) break;
                uint8_t *stage = smem + s * S::STAGE_BYTES;
                const uint32_t *src = (const uint32_t *)(stage + src_off);
#pragma unroll
                for (int rr = 0; rr < RPT; rr++) {
                    uint32_t w = src[rr * COLS];
                    const uint32_t lo0 = (w & 0x000f000fu) | 0x64006400u;
                    const uint32_t hi0 = (w & 0x00f000f0u) | 0x64006400u;
                    w >>= 8;
                    const uint32_t lo1 = (w & 0x000f000fu) | 0x64006400u;
                    const uint32_t hi1 = (w & 0x00f000f0u) | 0x64006400u;
                    const __half2 a = __hmul2(__hsub2(*(const __half2 *)&lo0, zsub), scale2);
                    const __half2 b = __hmul2(__hfma2(*(const __half2 *)&hi0, sixteenth, zfma), scale2);
                    const __half2 c = __hmul2(__hsub2(*(const __half2 *)&lo1, zsub), scale2);
                    const __half2 d = __hmul2(__hfma2(*(const __half2 *)&hi1, sixteenth, zfma), scale2);
                    const uint32_t ua = *(const uint32_t *)&a, ub = *(const uint32_t *)&b;
                    const uint32_t uc = *(const uint32_t *)&c, ud = *(const uint32_t *)&d;
                    uint4 o;
                    o.x = __byte_perm(ua, ub, 0x5410);
                    o.y = __byte_perm(uc, ud, 0x5410);
                    o.z = __byte_perm(ua, ub, 0x7632);
                    o.w = __byte_perm(uc, ud, 0x7632);
                    *(uint4 *)(stage + dst_off[rr]) = o;
                }
                fence_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(&deq[s]);
                s += KG;
                if (s >= STAGES) s -= STAGES, ph ^= 1;
            }
        }
    } else if (warp >= WARPS) {
        // ------------------------------------------------------------------ epilogue: warp w drains TMEM lanes 32 * (w % 4) ..
        const int q = warp & 3;
        bool ok = true;
        pdl_wait();  // nothing is stored before the kernel before this one is done
        for (int ti = 0; ti < tiles_cta && ok; ti++) {
            const int buf = ti % NBUF, use = ti / NBUF;
            ok = mbar_wait_idle(&acc_full[buf], (uint32_t)use & 1u, abort_flag, p.status, 5);
            if (!GATHER && !ok) break;  // (the GATHER epilogue's warps meet at barriers: they agree below)
            tc_fence_after();
            const int m0 = tile_m0(ti), n0 = tile_n0(ti);
            const uint32_t acc = tmem_base + (uint32_t)buf * ACC_ALL + ((uint32_t)(q * 32) << 16);
            StoreDst d;
            if constexpr (GATHER) {
#pragma unroll
                for (int g = 0; g < kMaxGatherDst; g++) d.dst[g] = p.dst[g];
                d.n_dst = p.n_dst, d.ld = p.ld_out, d.col0 = p.col0;
            } else {
                d.dst[0] = p.out, d.n_dst = 1, d.ld = p.N, d.col0 = 0;
            }
            const bool out16 = p.out_f16 != 0;
            const bool vec = (p.N & 7) == 0 && (d.ld & 7) == 0 && (d.col0 & 7) == 0;
            if constexpr (GATHER) {
                // A column-sharded call: the four warps first put 64 (fp16) or 32 (f32) token rows of the tile side by side
                // in a 16 KB staging tile, then copy whole rows of it (256 or 512 contiguous bytes) to every destination,
                // this GPU's slab and the peers'. A warp's own columns are only 64 bytes of a row, and stores of that
                // size are what held the peer stores back.
                bool staged = vec;
                {
                    uint32_t all;
                    asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.u32 p, %1, 0;\n\tbar.red.and.pred q, 1, 128, p;\n\tselp.u32 %0, 1, 0, q;\n\t}"
                                 : "=r"(all) : "r"((uint32_t)(ok ? 1 : 0)) : "memory");
                    if (!all) break;  // the four warps go on together or not at all
                }
                if (staged) {
                    uint8_t *stg = reinterpret_cast<uint8_t *>(bars) + 256;
                    const int epi_tid = (warp - WARPS) * 32 + lane;
                    const int esz = out16 ? 2 : 4, rows = out16 ? 64 : 32, cpr = BN * esz / 16;  // 16-byte chunks per row
#pragma unroll 1
                    for (int h = 0; h < NH; h++) {
                        const int n_base = n0 + h * BN;
                        const int n = n_base + q * 32 + lane;
                        const float bias = (p.bias && n < p.N) ? p.bias[n] : 0.f;
#pragma unroll 1
                        for (int c = 0; c < MT; c += rows) {
                            asm volatile("bar.sync 1, 128;" ::: "memory");  // the copy-out of the previous chunk is done
#pragma unroll 1
                            for (int cc = 0; cc < rows; cc += 16) {
                                uint32_t r[16];
                                tmem_ld_32x32b_x16(acc + (uint32_t)(h * ACC_COLS + c + cc), r);
                                tmem_ld_wait();
                                if (out16) {
                                    __half *tile = reinterpret_cast<__half *>(stg) + q * 32 + lane;
#pragma unroll
                                    for (int j = 0; j < 16; j++) tile[(cc + j) * BN] = __float2half_rn(__uint_as_float(r[j]) + bias);
                                } else {
                                    float *tile = reinterpret_cast<float *>(stg) + q * 32 + lane;
#pragma unroll
                                    for (int j = 0; j < 16; j++) tile[(cc + j) * BN] = __uint_as_float(r[j]) + bias;
                                }
                            }
                            asm volatile("bar.sync 1, 128;" ::: "memory");
                            for (int idx = epi_tid; idx < rows * cpr; idx += 128) {
                                const int row = idx / cpr, seg = idx - row * cpr;
                                const int m = m0 + c + row, ncol = n_base + seg * (16 / esz);
                                if (m < p.M && ncol < p.N) {
                                    const uint4 v = reinterpret_cast<const uint4 *>(stg)[idx];
                                    const int64_t off = ((int64_t)m * d.ld + d.col0 + ncol) * esz;
#pragma unroll
                                    for (int g = 0; g < kMaxGatherDst; g++)
                                        if (g < d.n_dst) *reinterpret_cast<uint4 *>(reinterpret_cast<char *>(d.dst[g]) + off) = v;
                                }
                            }
                        }
                    }
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&acc_empty[buf]);
                    continue;
                }
            }
#pragma unroll 1
            for (int h = 0; h < NH; h++) {
                const int n_warp = n0 + h * BN + q * 32;
                const int n = n_warp + lane;
                const float bias = (p.bias && n < p.N) ? p.bias[n] : 0.f;
#pragma unroll 1
                for (int c = 0; c < MT; c += 16) {
                    uint32_t r[16];
                    tmem_ld_32x32b_x16(acc + (uint32_t)(h * ACC_COLS + c), r);
                    tmem_ld_wait();
                    store_block16<GATHER>(d, out16, vec, r, bias, m0 + c, p.M, n_warp, p.N, lane);
                }
            }
            // the accumulator set may be overwritten once all four warps have read it
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == MMA_WARP) tmem_dealloc(tmem_base, TMEM_COLS);
}

__global__ void cast_f32_to_f16_kernel(const float *__restrict__ in, __half *__restrict__ out, int64_t n)
{
    int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x * 4;
    for (; i + 3 < n; i += stride) {
        const float4 v = *reinterpret_cast<const float4 *>(in + i);
        __half2 a = __floats2half2_rn(v.x, v.y), b = __floats2half2_rn(v.z, v.w);
        uint2 o;
        o.x = *reinterpret_cast<uint32_t *>(&a);
        o.y = *reinterpret_cast<uint32_t *>(&b);
        *reinterpret_cast<uint2 *>(out + i) = o;
    }
}

// out[m, n] = bias[n] + sum over slices (in slice order) of partial[s][m][n], stored at every destination of `pl`
__global__ void splitk_reduce_kernel(const float *__restrict__ partial, const float *__restrict__ bias, const OutPlace pl,
                                     int64_t MN, int N, int S, int out_f16)
{
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= MN) return;
    float v = 0.f;
    for (int s = 0; s < S; s++) v += partial[(int64_t)s * MN + i];
    const int64_t m = i / N;
    const int n = (int)(i - m * N);
    if (bias) v += bias[n];
    const int64_t o = m * pl.ld + pl.col0 + n;
#pragma unroll
    for (int g = 0; g < kMaxGatherDst; g++) {  // static indices into the parameter
        if (g < pl.n_dst) {
            if (out_f16) ((__half *)pl.dst[g])[o] = __float2half_rn(v);
            else ((float *)pl.dst[g])[o] = v;
        }
    }
}

// The same, four consecutive columns per thread (N, the pitch and the column offset multiples of 4; 16-byte stores for
// f32, 8-byte for fp16).
__global__ void __launch_bounds__(256) splitk_reduce_vec4_kernel(const float *__restrict__ partial, const float *__restrict__ bias,
                                                                 const OutPlace pl, int64_t MN4, int N4, int S, int out_f16)
{
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    pdl_sync();  // launched under the tail of the GEMM whose partial sums it reads
    if (i >= MN4) return;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s < S; s++) {
        const float4 a = *reinterpret_cast<const float4 *>(partial + ((int64_t)s * MN4 + i) * 4);
        v.x += a.x, v.y += a.y, v.z += a.z, v.w += a.w;
    }
    const int64_t m = i / N4;
    const int n = (int)(i - m * N4) * 4;
    if (bias) {
        const float4 b = *reinterpret_cast<const float4 *>(bias + n);
        v.x += b.x, v.y += b.y, v.z += b.z, v.w += b.w;
    }
    const int64_t o = m * pl.ld + pl.col0 + n;
#pragma unroll
    for (int g = 0; g < kMaxGatherDst; g++) {  // static indices into the parameter
        if (g < pl.n_dst) {
            if (out_f16) {
                const __half2 a = __floats2half2_rn(v.x, v.y), b = __floats2half2_rn(v.z, v.w);
                uint2 w;
                w.x = *reinterpret_cast<const uint32_t *>(&a), w.y = *reinterpret_cast<const uint32_t *>(&b);
                *reinterpret_cast<uint2 *>((__half *)pl.dst[g] + o) = w;
            } else {
                *reinterpret_cast<float4 *>((float *)pl.dst[g] + o) = v;
            }
        }
    }
}

// Copies a dense local [M, N] result to its columns of every destination (the decode-size kernels write a dense
// result; at those sizes the pieces are a few KB and a second small launch costs less than a collective).
__global__ void scatter_cols_kernel(const void *__restrict__ src, const OutPlace pl, int64_t MN, int N, int f16)
{
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= MN) return;
    const int64_t m = i / N;
    const int64_t o = m * pl.ld + pl.col0 + (i - m * N);
#pragma unroll
    for (int g = 0; g < kMaxGatherDst; g++) {  // static indices into the parameter
        if (g < pl.n_dst) {
            if (f16) ((__half *)pl.dst[g])[o] = ((const __half *)src)[i];
            else ((float *)pl.dst[g])[o] = ((const float *)src)[i];
        }
    }
}

}  // namespace tc

// ----------------------------------------------------------------------------------------------------
// host side
// ----------------------------------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static int make_map_2d(wb_context *ctx, CUtensorMap *map, CUtensorMapDataType dt, int elem_bytes, const void *base,
                       uint64_t inner, uint64_t outer, uint32_t box_inner, uint32_t box_outer, bool swizzle128)
{
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {inner * (uint64_t)elem_bytes};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = ((EncodeTiledFn)ctx->tmap_encode)(map, dt, 2, const_cast<void *>(base), dims, strides, box, estr,
                                                   CU_TENSOR_MAP_INTERLEAVE_NONE,
                                                   swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                                                   CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(WB_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
    return WB_OK;
}

// gemm_pair.cu
bool gemm_pair_supports(const Weight &w, int64_t M);
cudaError_t launch_gemm_pair(int mt, const CUtensorMap &mx, const CUtensorMap &mw, const CUtensorMap *mc, const tc::Params &p, int tiles_m,
                             int tiles_n, int S, cudaStream_t st, int sms, float *tail_partial, int *extra_launches);
bool pair_tail_plan(int64_t n_items, int pairs, int kblocks, int *rounds, int *rem, int *St, int *per);

bool gemm_tc_supports(const Weight &w, int64_t M)
{
    if (M < 1 || w.K % 64 != 0) return false;
    if (w.kind == WeightKind::Gptq) return w.N % 4 == 0 && w.group % 64 == 0;
    return w.kind == WeightKind::DenseF16;
}

// microseconds per 64-k block of a pair's work item (measured)
constexpr double kPairKb256 = 0.37, kPairKb192 = 0.35, kPairKb128 = 0.34, kPairItem = 0.4;
constexpr int kPairStageKb = 32;  // up to this many k-blocks per work item the 256-token tile stages its fp16 result

static int env_int(const char *name)
{
    const char *v = getenv(name);
    return v ? atoi(v) : 0;
}

// WEBLLM_B200_GEMM_PERSIST=0 keeps every launch on the one-tile-per-CTA kernel (for comparisons). Otherwise launches
// with more tiles than SMs whose accumulators fit TMEM twice take the persistent tile loop.
static bool persist_enabled()
{
    static const bool on = [] { const char *e = getenv("WEBLLM_B200_GEMM_PERSIST"); return !(e && e[0] == '0'); }();
    return on;
}

// Tile (mt tokens x 128 * nh output columns) and number of K slices, by a small cost model in microseconds whose
// constants are measurements: the time of one 64-k block of a tile (the unpack of the weight tile bounds it, so it
// depends on the columns far more than on the tokens), a fixed time per tile (pipeline fill, TMEM drain and stores),
// and for split-K the reduce launch, which moves slices + 1 copies of the output.
// WEBLLM_B200_GEMM_MT / _NH / _SPLIT pin one of the three for experiments.
static double pick_plan(int64_t M, int64_t N, int kblocks, int sms, int force_split, double t_remote, int *mt_out, int *nh_out, int *s_out)
{
    static const int force_mt = env_int("WEBLLM_B200_GEMM_MT"), force_nh = env_int("WEBLLM_B200_GEMM_NH"),
                     env_split = env_int("WEBLLM_B200_GEMM_SPLIT");
    if (force_split <= 0) force_split = env_split;
    static const int mts[6] = {16, 32, 64, 128, 192, 256};  // 192 exists to fit the waves (e.g. 11 x 38 tiles on 148 SMs)
    double best = -1.;
    *mt_out = 128, *nh_out = 1, *s_out = 1;
    for (int mt : mts) {
        // up to 128 tokens the smallest tile that holds them, above that 128 or 256
        const bool fits = M > 128 ? mt >= 128 : (mt >= M && (mt == 16 || mt < 2 * M));
        if (force_mt ? mt != force_mt : !fits) continue;
        for (int nh = 1; nh <= 2; nh++) {
            if (force_nh && nh != force_nh && mt >= 128 && N >= 256) continue;  // pinned wherever it exists
            if (nh == 2 && (mt < 128 || N < 256)) continue;
            const double t_kb = nh == 2 ? (mt == 256 ? 0.89 : mt == 192 ? 0.84 : 0.80) : (mt == 256 ? 0.54 : mt == 192 ? 0.48 : mt == 128 ? 0.33 : 0.25);
            const double t_tile = 1.5 + 2.7 * nh * mt / 256.;
            const int64_t tiles = ((M + mt - 1) / mt) * ((N + 128 * nh - 1) / (128 * nh));
            for (int S = 1; S <= 16; S++) {
                // a slice keeps at least 8 k-blocks, except where so few tiles exist (a quarter of the SMs or fewer) that
                // a launch is all start-up and hand-over: there slices down to 2 k-blocks measured 25 % faster
                const int min_per = tiles * 4 <= sms ? 2 : 8;
                if (force_split > 0 ? S != (force_split < kblocks ? force_split : kblocks) : (S > 1 && kblocks / S < min_per)) continue;
                const int per = (kblocks + S - 1) / S;
                if ((kblocks + per - 1) / per != S) continue;  // would leave an empty slice
                if (S > 1 && (double)S * M * N * 4. > 64e6) continue;  // partial sums must fit the workspace
                const int64_t waves = (tiles * S + sms - 1) / sms;
                double t = 2.0 + waves * (per * t_kb + t_tile);
                // persistent CTAs (where TMEM holds two accumulator sets): fill, drain and stores are paid once
                const bool persist = S == 1 && tiles > sms && persist_enabled() && 2 * (mt < 32 ? 32 : mt) * nh <= 512;
                if (persist) t = 2.0 + t_tile + waves * per * t_kb;
                // a column-sharded call also stores the result into the peers: under the next tile's MMAs in the
                // persistent loop, at the end of every CTA (on top of the arithmetic) otherwise
                if (t_remote > 0.) t = persist ? (t > t_remote ? t : t_remote) : t + t_remote;
                if (S > 1) t += 1.5 + (S + 1) * (double)M * N * 4. / 5e6;
                if (best < 0. || t < best) best = t, *mt_out = mt, *nh_out = nh, *s_out = S;
            }
        }
    }
    return best;
}

// The same model for the CTA-pair kernel (gemm_pair.cu): work items of mt tokens x 256 columns x one K slice, walked by
// sms / 2 persistent pairs; fill, drain and stores are paid once per pair.
static double pick_plan_pair(int64_t M, int64_t N, int kblocks, int sms, int force_split, bool tail_ok, int *mt_out, int *s_out)
{
    static const int force_mt = env_int("WEBLLM_B200_GEMM_MT"), env_split = env_int("WEBLLM_B200_GEMM_SPLIT");
    if (force_split <= 0) force_split = env_split;
    static const int mts[3] = {128, 192, 256};
    const int pairs = sms / 2;
    double best = -1.;
    *mt_out = 256, *s_out = 1;
    for (int mt : mts) {
        if (force_mt ? mt != force_mt : (M <= 128 && mt != 128)) continue;
        const double t_kb = mt == 256 ? kPairKb256 : mt == 192 ? kPairKb192 : kPairKb128;
        const double t_tile = 1.5 + 2.7 * mt / 256.;
        const int64_t tiles = ((M + mt - 1) / mt) * ((N + 255) / 256);
        for (int S = 1; S <= 16; S++) {
            const int min_per = tiles * 4 <= pairs ? 2 : 8;
            if (force_split > 0 ? S != (force_split < kblocks ? force_split : kblocks) : (S > 1 && kblocks / S < min_per)) continue;
            const int per = (kblocks + S - 1) / S;
            if ((kblocks + per - 1) / per != S) continue;
            if (S > 1 && (double)S * M * N * 4. > 64e6) continue;
            const int64_t rounds = (tiles * S + pairs - 1) / pairs;
            double t = 3.3 + t_tile + rounds * (per * t_kb + kPairItem);
            int tr, trem, tst, tper;
            if (S == 1 && tail_ok && pair_tail_plan(tiles, pairs, kblocks, &tr, &trem, &tst, &tper))  // the last round cut along K
                t = 3.3 + t_tile + tr * (per * t_kb + kPairItem) + (tper * t_kb + kPairItem) + 3.0;
            if (S > 1) t += 1.5 + (S + 1) * (double)M * N * 4. / 5e6;
            if (best < 0. || t < best) best = t, *mt_out = mt, *s_out = S;
        }
    }
    return best;
}

// pair_mode: 0 = one-CTA kernels only, 1 = whichever the cost model prefers, 2 = the CTA-pair kernel or nothing
// (plan->kernel stays 0 when the shape does not qualify).
int plan_gemm_tc(wb_context *ctx, const Weight &w, int64_t M, int act_dtype, int exact, int pair_mode, wb_plan *plan)
{
    (void)exact;
    const int kblocks = (int)(w.K / 64);
    int mt, nh, S;
    // microseconds that the stores to the peers of a column-sharded call take at ~700 GB/s per direction
    const double t_remote = ctx->place.n_dst > 1 ? (double)(ctx->place.n_dst - 1) * M * w.N * ctx->place.elem_bytes / 700e3 : 0.;
    const double t_one = pick_plan(M, w.N, kblocks, ctx->sm_count, ctx->force_split, t_remote, &mt, &nh, &S);
    // Stores into peers' slabs stay with the one-CTA kernels: a two-GPU run of the pair kernel with peer destinations
    // (7B-class shards at M = 4096) ended in a launch failure whose cause reading has not shown, so it is not launched so.
    const bool pair_ok = pair_mode > 0 && ctx->place.n_dst <= 1 && gemm_pair_supports(w, M) && ctx->sm_count >= 2;
    if (pair_mode == 2 && !pair_ok) return WB_OK;
    if (pair_ok) {
        int pmt, pS;
        double t_pair = pick_plan_pair(M, w.N, kblocks, ctx->sm_count, ctx->force_split, ctx->place.n_dst == 0, &pmt, &pS);
        if (t_remote > 0. && pS == 1 && t_pair < t_remote) t_pair = t_remote;  // the stores to the peers run under the MMAs
        if (pair_mode == 2 || (t_pair > 0. && t_pair < t_one)) {
            plan->kernel = WB_KERNEL_GEMM_TC_PAIR;
            plan->grid_x = (int)((M + pmt - 1) / pmt);
            plan->grid_y = (int)((w.N + 255) / 256);
            plan->split_k = plan->grid_z = pS;
            plan->block = 800;
            plan->tile_m = pmt;
            plan->tile_n = 256;
            mt = pmt, nh = 2, S = pS;
        }
    }
    if (plan->kernel == 0) {
        plan->kernel = WB_KERNEL_GEMM_TC;
        plan->grid_x = (int)((M + mt - 1) / mt);
        plan->grid_y = (int)((w.N + 128 * nh - 1) / (128 * nh));
        plan->split_k = S;
        plan->grid_z = S;
        plan->block = tc::THREADS;
        plan->tile_m = mt;
        plan->tile_n = 128 * nh;
    }
    const uint64_t stage_bytes = act_dtype == WB_F32 ? align_up((uint64_t)M * w.K * 2) : 0;
    // a pair launch that cuts its last round along K (PairTail, gemm_pair.cu) parks one partial tile per pair and adds a launch
    int tr, trem, tst, tper;
    const bool pair_tail = plan->kernel == WB_KERNEL_GEMM_TC_PAIR && S == 1 && ctx->place.n_dst == 0 &&
                           pair_tail_plan((int64_t)plan->grid_x * plan->grid_y, ctx->sm_count / 2, kblocks, &tr, &trem, &tst, &tper);
    plan->launches = (act_dtype == WB_F32 ? 2 : 1) + (S > 1 || pair_tail ? 1 : 0);
    plan->scratch_bytes = stage_bytes + (S > 1 ? (uint64_t)S * M * w.N * 4 : 0) +
                          (pair_tail ? (uint64_t)(ctx->sm_count / 2) * mt * 256 * 4 : 0);
    if (plan->scratch_bytes > kWorkspaceBytes)
        return fail(WB_ERR_OOM, "fp16 staging of %lld x %lld activations exceeds the workspace; pass fp16 activations or split M",
                    (long long)M, (long long)w.K);
    return WB_OK;
}

template <int MT, bool DENSE, int NH>
static cudaError_t launch_tc(const CUtensorMap &mx, const CUtensorMap &mw, const tc::Params &p, dim3 grid, cudaStream_t st, int sms)
{
    constexpr int smem = tc::Smem<MT, DENSE, NH>::TOTAL;
    // the shared-memory attribute of a kernel instance is set once per device, not on every call (variant: 0 = one
    // tile per CTA, 1 = split-K, 2 = gather, 3 = persistent, 4 = persistent gather)
    static bool attr_set[5][16] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    auto ensure_attr = [&](auto kernel, int variant) -> cudaError_t {
        if (dev >= 0 && dev < 16 && attr_set[variant][dev]) return cudaSuccess;
        const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e == cudaSuccess && dev >= 0 && dev < 16) attr_set[variant][dev] = true;
        return e;
    };
    auto go = [&](auto kernel, int variant) {
        cudaError_t e = ensure_attr(kernel, variant);
        if (e != cudaSuccess) return e;
        return launch_pdl(kernel, grid, dim3(tc::THREADS), (size_t)smem, st, mx, mw, p);
    };
    // more tiles than SMs and no K split: one persistent CTA per SM walks the tiles
    const bool persist_on = persist_enabled();
    const int n_tiles = (int)(grid.x * grid.y);
    auto go_persist = [&](auto kernel, int variant) {
        // the column-sharded instantiation carries a staging tile (and sizes its ring around it)
        const int smem_p = variant == 4 ? tc::Smem<MT, DENSE, NH, tc::kGatherStageBytes>::TOTAL : smem;
        if (!(dev >= 0 && dev < 16 && attr_set[variant][dev])) {
            const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_p);
            if (e != cudaSuccess) return e;
            if (dev >= 0 && dev < 16) attr_set[variant][dev] = true;
        }
        return launch_pdl(kernel, dim3((unsigned)sms), dim3(tc::THREADS_P), (size_t)smem_p, st, mx, mw, p, (int)grid.x, n_tiles);
    };
    if (grid.z > 1) return go(tc::gemm_tc_kernel<MT, DENSE, true, NH, false>, 1);  // slices write partial sums: no placement
    // only where TMEM holds two accumulator sets: with one set the MMAs would wait for four warps to drain it
    constexpr bool two_sets = 2 * (MT < 32 ? 32 : MT) * NH <= 512;
    const bool persist = persist_on && two_sets && n_tiles > sms;
    if constexpr (!DENSE) {
        if (p.n_dst > 0)
            return persist ? go_persist(tc::gemm_tc_persist_kernel<MT, DENSE, NH, true>, 4)
                           : go(tc::gemm_tc_kernel<MT, DENSE, false, NH, true>, 2);
    }
    return persist ? go_persist(tc::gemm_tc_persist_kernel<MT, DENSE, NH, false>, 3)
                   : go(tc::gemm_tc_kernel<MT, DENSE, false, NH, false>, 0);
}

// tile_n = 256 (two accumulators per CTA) exists for the 128-, 192- and 256-token tiles only
template <bool DENSE>
static cudaError_t launch_tc_mt(int mt, int nh, const CUtensorMap &mx, const CUtensorMap &mw, const tc::Params &p, dim3 grid,
                                cudaStream_t st, int sms)
{
    switch (mt) {
    case 16: return launch_tc<16, DENSE, 1>(mx, mw, p, grid, st, sms);
    case 32: return launch_tc<32, DENSE, 1>(mx, mw, p, grid, st, sms);
    case 64: return launch_tc<64, DENSE, 1>(mx, mw, p, grid, st, sms);
    case 128: return nh == 2 ? launch_tc<128, DENSE, 2>(mx, mw, p, grid, st, sms) : launch_tc<128, DENSE, 1>(mx, mw, p, grid, st, sms);
    case 192: return nh == 2 ? launch_tc<192, DENSE, 2>(mx, mw, p, grid, st, sms) : launch_tc<192, DENSE, 1>(mx, mw, p, grid, st, sms);
    default: return nh == 2 ? launch_tc<256, DENSE, 2>(mx, mw, p, grid, st, sms) : launch_tc<256, DENSE, 1>(mx, mw, p, grid, st, sms);
    }
}

int launch_gemm_tc(wb_context *ctx, const Weight &w, const void *A, void *C, const float *bias, int64_t M, int act_dtype,
                   int out_dtype, int exact, const wb_plan &plan)
{
    (void)exact;
    const char *base = ctx->arena[WB_ARENA_WEIGHTS].base;
    const void *a16 = A;
    if (act_dtype == WB_F32) {
        // The reference rounds f32 activations to fp16 when it stages a tile (gemm_nt_f16_from_f32.wgsl:58-62).
        const int64_t n = M * w.K;  // K % 64 == 0, so n % 4 == 0
        int blocks = (int)((n / 4 + 255) / 256);
        if (blocks > ctx->sm_count * 8) blocks = ctx->sm_count * 8;
        tc::cast_f32_to_f16_kernel<<<blocks, 256, 0, ctx->stream>>>((const float *)A, (__half *)ctx->workspace, n);
        ctx->launches++;
        WB_CUDA(cudaGetLastError());
        a16 = ctx->workspace;
    }
    const int mt = plan.tile_m;
    const bool pair = plan.kernel == WB_KERNEL_GEMM_TC_PAIR;
    const int nh = pair ? 1 : plan.tile_n == 2 * tc::BN ? 2 : 1;  // a CTA of a pair takes 128-column boxes
    // the activation map depends on the call (pointer, M, tile); the weight map only on the weight and the tile width:
    // it is encoded once and kept with the weight
    CUtensorMap mx;
    TmapSlot &wslot = w.tmap_tc[nh - 1];
    CUtensorMap &mw = *reinterpret_cast<CUtensorMap *>(wslot.bytes);
    WB_CHECK(make_map_2d(ctx, &mx, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, a16, (uint64_t)w.K, (uint64_t)M, tc::BK,
                         (uint32_t)(pair ? mt / 2 : mt), true));
    tc::Params p;
    p.out = C, p.bias = bias, p.status = ctx->status_word;
    p.M = (int)M, p.N = (int)w.N, p.K = (int)w.K;
    p.out_f16 = out_dtype == WB_F16;
    const int S = plan.split_k > 0 ? plan.split_k : 1;
    const int kblocks = (int)(w.K / tc::BK);
    p.kb_per_slice = (kblocks + S - 1) / S;
    p.partial = (float *)(ctx->workspace + (act_dtype == WB_F32 ? align_up((uint64_t)M * w.K * 2) : 0));
    OutPlace place = ctx->place;  // n_dst > 0: a column-sharded call (wb_linear_gather)
    if (place.n_dst > 0 && w.kind != WeightKind::Gptq)
        return fail(WB_ERR_UNSUPPORTED, "wb_linear_gather takes GPTQ weights only");
    if (pair && w.kind != WeightKind::Gptq) return fail(WB_ERR_UNSUPPORTED, "the CTA-pair GEMM takes GPTQ weights");
    p.ld_out = place.ld, p.col0 = place.col0, p.n_dst = place.n_dst;
    for (int g = 0; g < kMaxGatherDst; g++) p.dst[g] = place.dst[g];
    if (place.n_dst == 0) place.ld = w.N, place.col0 = 0, place.n_dst = 1, place.dst[0] = C;  // for the split-K reduce
    dim3 grid(plan.grid_x, plan.grid_y, S);
    cudaError_t e;
    if (w.kind == WeightKind::Gptq) {
        if (!wslot.ok)
            WB_CHECK(make_map_2d(ctx, &mw, CU_TENSOR_MAP_DATA_TYPE_INT32, 4, base + w.off_main, (uint64_t)w.N,
                                 (uint64_t)w.pack_rows, tc::BN * nh, 8, false));
        wslot.ok = true;
        p.qz = w.has_zeros ? (const uint32_t *)(base + w.off_zeros) : nullptr;
        p.sc = (const __half *)(base + w.off_scales);
        p.zcols = (int)w.zcols;
        p.group_blocks = (int)(w.group / 64);
        if (pair) {
            // the result (or the K slices' f32 partial sums) leaves the epilogue through shared memory and TMA stores
            // where a work item has few k-blocks: with many, the drain hides under the next item's MMAs anyway and the
            // shared memory serves the 256-token tile better as a sixth pipeline stage
            CUtensorMap mc;
            const bool c16 = S == 1 && out_dtype == WB_F16;
            void *cbase = S > 1 ? (void *)p.partial : C;
            const bool tma_store = (S > 1 || p.n_dst == 0) && w.N % (c16 ? 8 : 4) == 0 && ((uintptr_t)cbase & 15) == 0 && (mt < 256 || p.kb_per_slice <= kPairStageKb);
            if (tma_store) {
                cuuint64_t dims[3] = {(cuuint64_t)w.N, (cuuint64_t)M, (cuuint64_t)S};
                cuuint64_t strides[2] = {(cuuint64_t)w.N * (c16 ? 2 : 4), (cuuint64_t)w.N * M * (c16 ? 2 : 4)};
                cuuint32_t box[3] = {(cuuint32_t)tc::BN, c16 ? 64u : 32u, 1u};
                cuuint32_t estr[3] = {1, 1, 1};
                CUresult r = ((EncodeTiledFn)ctx->tmap_encode)(&mc, c16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3,
                                                               cbase, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                                               CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
                if (r != CUDA_SUCCESS) return fail(WB_ERR_CUDA, "cuTensorMapEncodeTiled (result) failed with code %d", (int)r);
            }
            int extra = 0;
            e = launch_gemm_pair(mt, mx, mw, tma_store ? &mc : nullptr, p, plan.grid_x, plan.grid_y, S, ctx->stream, ctx->sm_count,
                                 S == 1 ? p.partial : nullptr, &extra);
            ctx->launches += (uint64_t)extra;
        } else {
            e = launch_tc_mt<false>(mt, nh, mx, mw, p, grid, ctx->stream, ctx->sm_count);
        }
    } else {
        if (!wslot.ok)
            WB_CHECK(make_map_2d(ctx, &mw, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, base + w.off_main, (uint64_t)w.K, (uint64_t)w.N,
                                 tc::BK, tc::BN * nh, true));
        wslot.ok = true;
        p.qz = nullptr, p.sc = nullptr, p.zcols = 0, p.group_blocks = 1;
        e = launch_tc_mt<true>(mt, nh, mx, mw, p, grid, ctx->stream, ctx->sm_count);
    }
    ctx->launches++;
    WB_CUDA(e);
    if (S > 1) {
        const int64_t MN = M * w.N;
        if (w.N % 4 == 0 && place.ld % 4 == 0 && place.col0 % 4 == 0)
            WB_CUDA(launch_pdl(tc::splitk_reduce_vec4_kernel, dim3((unsigned)((MN / 4 + 255) / 256)), dim3(256), 0, ctx->stream,
                               (const float *)p.partial, bias, place, MN / 4, (int)(w.N / 4), S, (int)(out_dtype == WB_F16)));
        else
            tc::splitk_reduce_kernel<<<(unsigned)((MN + 255) / 256), 256, 0, ctx->stream>>>(p.partial, bias, place, MN, (int)w.N, S,
                                                                                             out_dtype == WB_F16);
        ctx->launches++;
        WB_CUDA(cudaGetLastError());
    }
    return WB_OK;
}

int launch_scatter_cols(wb_context *ctx, const void *src, int64_t M, int64_t N, bool f16)
{
    const int64_t MN = M * N;
    tc::scatter_cols_kernel<<<(unsigned)((MN + 255) / 256), 256, 0, ctx->stream>>>(src, ctx->place, MN, (int)N, f16 ? 1 : 0);
    ctx->launches++;
    WB_CUDA(cudaGetLastError());
    return WB_OK;
}

}  // namespace wb
