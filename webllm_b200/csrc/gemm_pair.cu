// The prefill GEMM on CTA pairs: C[M,N] = A[M,K] . W[N,K]^T (+bias) for GPTQ int4 weights, with every tcgen05.mma
// issued for two SMs at once (cta_group::2). Same contract as gemm_tc.cu (replaces gemm_nt_f16_from_f32.wgsl,
// src/gpu/kernels/gemm/gemm_nt_f16_from_f32.wgsl:39-95, behind QwenGpt.gemm, src/model/qwen.ts:613-617).
//
// A pair (a cluster of two CTAs on the two SMs of one TPC) computes 256 output columns x MT tokens of C^T per work
// item. Each CTA unpacks ITS 128 weight columns (the 128-row half of the M = 256 operand, accumulated in the 128 lanes
// of its own tensor memory) and loads only HALF of the activation tile (MT/2 tokens); the tensor cores of the pair
// read both halves. Per SM and 64-k block that is half the activation bytes from L2, half the shared-memory fill and
// half the operand reads of the one-CTA kernel, for the same arithmetic and the same unpack work.
//
// Roles per CTA: a TMA producer warp (own packed-weight box, own half of the activation box), an MMA issuer warp
// (rank 0 of the pair only; both ranks allocate and free tensor memory), sixteen unpack warps (four sets of one thread
// per column that take the k-blocks in turn) and four epilogue warps (drain one of the two accumulator sets while the
// MMAs of the next item run); which warp id has which role is listed at WARPS_PAIR. The pair walks the work items pair,
// pair + pairs, ...; an item is (K slice, column tile, token tile); with more than one K slice the items write f32
// partial sums that the split-K reduce launch adds.
//   * The weights are constants: the producer requests the packed boxes of the first stages, and the unpack sets unpack
//     them, before the wait on the previous kernel (programmatic dependent launch); the activation loads and the
//     epilogue's stores come after it.
//   * Where a work item is short (K = 896: 14 k-blocks) the result leaves through two 16 KB staging tiles and TMA stores
//     (fp16, f32, or the f32 partial sums of a K slice; STG instantiations); where it is long, from registers, and the
//     shared memory holds a sixth pipeline stage instead.
//   * A launch whose last round of work items would leave most pairs idle for a long item cuts those items along K over
//     the idle pairs (PairTail) and adds the slices in a small second launch.
//
// Barriers (mbarriers in shared memory, all waits bounded):
//   full_w[s]   local    the packed-weight box of stage s has landed (own TMA)
//   ready[s]    rank 0   both halves of the activation tile have landed (each CTA's TMA signals rank 0's barrier) and
//                        both CTAs' unpack sets have written their operand half (remote arrive from rank 1): one wait
//                        per k-block for the thread that issues the MMAs, whose own instruction latency is the pace
//   empty[s]    local    the MMAs that read stage s have completed (tcgen05.commit to both CTAs)
//   acc_full[b] local    accumulator set b is complete (tcgen05.commit to both CTAs)
//   acc_empty[b] rank 0  both CTAs' epilogue warps have drained set b (remote arrive from rank 1)
// No load in this file is a cluster-multicast load: every CTA fetches its own boxes.
#include "gemm_tc.cuh"

namespace wb {

namespace tcp {

using namespace tc;

constexpr int EPI_WARPS = 4;
// Warp roles as listed at MMA_WARP (gemm_tc.cuh), plus the four epilogue warps 21 .. 24 (a warp reads the tensor-memory
// lane quarter id % 4).
constexpr int WARPS_PAIR = WARPS + EPI_WARPS;
constexpr int THREADS_PAIR = 32 * WARPS_PAIR;
constexpr int KG = 4;  // unpack sets: 128 threads each, one thread per weight column
constexpr int STG_ROWS = 64;                 // token rows of an fp16 epilogue staging tile (half as many of f32)
constexpr int STG_BYTES = STG_ROWS * BN * 2;  // [64 tokens][128 columns] fp16 or [32][128] f32

// STG: two epilogue staging tiles are carved out of the shared memory (one pipeline stage fewer for the 256-token tile)
template <int MT, bool STG>
struct SmemPair {
    static constexpr int X_BYTES = (MT / 2) * BK * 2;   // this CTA's half of the activation tile
    static constexpr int WD_BYTES = BN * BK * 2;        // unpacked fp16 operand, 128 columns x 64 k
    static constexpr int WP_BYTES = 8 * BN * 4;         // packed box, 8 rows x 128 columns
    static constexpr int STAGE_BYTES = X_BYTES + WD_BYTES + WP_BYTES;  // every piece is a multiple of 1024
    static constexpr int STG_TOTAL = STG ? 2 * STG_BYTES : 0;
    static constexpr int MAX_STAGES = (227 * 1024 - 1280 - STG_TOTAL) / STAGE_BYTES;
    static constexpr int STAGES = MAX_STAGES > 6 ? 6 : MAX_STAGES;
    static constexpr int TOTAL = STAGES * STAGE_BYTES + STG_TOTAL + 1024 /*alignment slack*/ + 256 /*barriers*/;
    static_assert(STAGES >= KG, "every unpack set needs a stage of its own");
    static_assert(X_BYTES % 1024 == 0, "operand tiles start on a swizzle atom");
};

__device__ __forceinline__ void cluster_sync_all()
{
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t *dst_smem, uint32_t cols)
{
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols)
{
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrives on the barrier at this shared-memory offset in BOTH CTAs of the pair once the MMAs issued so far are complete.
__device__ __forceinline__ void umma_commit_pair(uint64_t *bar)
{
    const uint16_t both = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"(both)
                 : "memory");
}
// Tiled load into this CTA's shared memory whose completion bytes go to a barrier of the pair (a shared::cluster address).
__device__ __forceinline__ void tma_load_2d_pairbar(void *dst, const CUtensorMap *map, int x, int y, uint32_t bar_cluster_addr)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(bar_cluster_addr)
        : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_addr)
{
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}
// The last, partly filled round of work items (items % pairs of them) would leave most pairs idle for a whole item. With
// `slots` > 0 those items are cut along K instead: every pair runs `rounds` whole items and then at most one K slice
// (`per` k-blocks, `St` slices per item) of a leftover item, whose f32 partial tile it writes to partial[pair]; a
// small launch adds the slices. Whole items are unaffected.
struct PairTail {
    int rounds = 0, slots = 0, St = 1, per = 0;
    float *partial = nullptr;  // [slots][MT][256]
};

// GATHER: the result goes to the placement in Params (this GPU's slab and its peers', row pitch ld_out) from registers.
template <int MT, bool SPLIT, bool STG, bool GATHER = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS_PAIR, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                 const __grid_constant__ CUtensorMap map_c, const Params p, const int tiles_m, const int tiles_n, const int n_items,
                 const int use_tma_store, const PairTail tail)
{
    using S = SmemPair<MT, STG>;
    constexpr int STAGES = S::STAGES;
    constexpr uint32_t ACC_COLS = MT;                       // TMEM columns of one accumulator set
    constexpr uint32_t USED = 2 * ACC_COLS;
    constexpr uint32_t TMEM_COLS = USED <= 256 ? 256 : 512;
    static_assert(USED <= 512 && MT % STG_ROWS == 0 && MT >= 128, "token tile");
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t *stg = smem + STAGES * S::STAGE_BYTES;  // two epilogue staging tiles
    uint64_t *bars = (uint64_t *)(stg + S::STG_TOTAL);
    uint64_t *full_w = bars, *ready = bars + STAGES, *empty = bars + 2 * STAGES;
    uint64_t *acc_full = bars + 3 * STAGES, *acc_empty = bars + 3 * STAGES + 2;
    uint32_t *tmem_slot = (uint32_t *)(bars + 3 * STAGES + 4);
    volatile int *abort_flag = (volatile int *)(tmem_slot + 1);
    static_assert((3 * STAGES + 4) * 8 + 8 <= 256, "barrier area");

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_cta_rank();           // 0 issues the MMAs
    const int pair = (int)blockIdx.x >> 1, n_pairs = (int)gridDim.x >> 1;
    const int KB = p.K / BK;
    const bool tail_on = !SPLIT && tail.slots > 0;
    const int items_cta = tail_on ? tail.rounds + (pair < tail.slots ? 1 : 0)
                                  : pair < n_items ? (n_items - pair + n_pairs - 1) / n_pairs : 0;
    const int tiles_mn = tiles_m * tiles_n;
    // work item ti of this pair: K slice, first token, this CTA's first column, k-blocks
    auto is_tail = [&](int ti) { return tail_on && ti == tail.rounds; };
    auto item_index = [&](int ti) { return is_tail(ti) ? tail.rounds * n_pairs + pair / tail.St : pair + ti * n_pairs; };
    auto item_slice = [&](int ti) { return item_index(ti) / tiles_mn; };
    auto item_m0 = [&](int ti) { return (item_index(ti) % tiles_mn % tiles_m) * MT; };
    auto item_n0 = [&](int ti) { return (item_index(ti) % tiles_mn / tiles_m) * (2 * BN) + (int)rank * BN; };
    auto item_kb0 = [&](int ti) { return SPLIT ? item_slice(ti) * p.kb_per_slice : is_tail(ti) ? (pair % tail.St) * tail.per : 0; };
    auto item_kbn = [&](int ti) {
        if (!SPLIT && !is_tail(ti)) return KB;
        const int per = SPLIT ? p.kb_per_slice : tail.per;
        const int left = KB - item_kb0(ti);
        return left < per ? left : per;
    };

    auto xs = [&](int s) { return smem + s * S::STAGE_BYTES; };
    auto wd = [&](int s) { return smem + s * S::STAGE_BYTES + S::X_BYTES; };
    auto wp = [&](int s) { return (uint32_t *)(smem + s * S::STAGE_BYTES + S::X_BYTES + S::WD_BYTES); };

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&full_w[s], 1);
            mbar_init(&ready[s], 1 + 2 * (UNPACK_WARPS / KG));
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 2 * EPI_WARPS);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == MMA_WARP) tmem_alloc_pair(tmem_slot, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // the other CTA's barriers are initialised before anything arrives on them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // Programmatic dependent launch: the packed weights are constants, so their first boxes are requested (and unpacked)
    // while the kernel before this one still runs; only the activation loads and the result stores wait for it.
    pdl_trigger();

    const int unpack_idx = unpack_index(warp);
    if (warp == TMA_WARP) {
        // ------------------------------------------------------------------ TMA producer (both CTAs)
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            // weight boxes of the first STAGES k-blocks (fresh stages, nothing to wait for), then the dependence
            int pre = 0;
            for (int ti = 0; ti < items_cta && pre < STAGES; ti++) {
                const int n0 = item_n0(ti), kb0 = item_kb0(ti), kbn = item_kbn(ti);
                for (int kb = 0; kb < kbn && pre < STAGES; kb++, pre++) {
                    mbar_expect_tx(&full_w[pre], S::WP_BYTES);
                    tma_load_2d(wp(pre), &map_w, n0, (kb0 + kb) * 8, &full_w[pre]);
                }
            }
            pdl_wait();
            int seq = 0;
            for (int ti = 0; ti < items_cta && ok; ti++) {
                const int m0 = item_m0(ti) + (int)rank * (MT / 2), n0 = item_n0(ti), kb0 = item_kb0(ti), kbn = item_kbn(ti);
                for (int kb = 0; kb < kbn; kb++, seq++) {
                    ok = mbar_wait(&empty[s], ph ^ 1, abort_flag, p.status, 1);
                    if (!ok) break;
                    if (seq >= pre) {
                        mbar_expect_tx(&full_w[s], S::WP_BYTES);
                        tma_load_2d(wp(s), &map_w, n0, (kb0 + kb) * 8, &full_w[s]);
                    }
                    if (rank == 0) mbar_expect_tx(&ready[s], 2 * S::X_BYTES);
                    tma_load_2d_pairbar(xs(s), &map_x, (kb0 + kb) * BK, m0, cluster_map_shared(&ready[s], 0));
                    if (++s == STAGES) s = 0, ph ^= 1;
                }
            }
            // drain: the last arrivals on this CTA's `empty` barriers come from the other SM's commits; they must have
            // landed before this CTA may leave
            for (int i = 0; i < STAGES && ok; i++) {
                ok = mbar_wait(&empty[s], ph ^ 1, abort_flag, p.status, 1);
                if (++s == STAGES) s = 0, ph ^= 1;
            }
        }
    } else if (warp == MMA_WARP) {
        // ------------------------------------------------------------------ MMA issuer (rank 0 for both SMs)
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc = idesc_f16(2 * BN, MT);
            bool ok = true;
            int s = 0;
            uint32_t ph = 0;
            for (int ti = 0; ti < items_cta && ok; ti++) {
                const int buf = ti & 1, use = ti >> 1;
                if (use > 0) ok = mbar_wait(&acc_empty[buf], (uint32_t)(use - 1) & 1u, abort_flag, p.status, 6);
                if (!ok) break;
                tc_fence_after();
                const uint32_t acc = tmem_base + (uint32_t)buf * ACC_COLS;
                const int kbn = item_kbn(ti);
                for (int kb = 0; kb < kbn; kb++) {
                    ok = mbar_wait(&ready[s], ph, abort_flag, p.status, 2);
                    if (!ok) break;
                    tc_fence_after();
                    const uint64_t a0 = smem_desc_sw128(smem_u32(wd(s)));
                    const uint64_t b0 = smem_desc_sw128(smem_u32(xs(s)));
#pragma unroll
                    for (int k = 0; k < BK / 16; k++) umma_f16_pair(acc, a0 + 2 * k, b0 + 2 * k, idesc, (kb | k) != 0);
                    umma_commit_pair(&empty[s]);
                    if (++s == STAGES) s = 0, ph ^= 1;
                }
                if (ok) umma_commit_pair(&acc_full[buf]);
            }
        }
        __syncwarp();
    } else if (is_unpack_warp(warp)) {
        // ------------------------------------------------------------------ unpack: the sets take the k-blocks of the
        // CTA's whole sequence (item after item) in turn
        constexpr int SET_THREADS = 32 * UNPACK_WARPS / KG;
        static_assert(SET_THREADS == BN, "one thread per weight column");
        const int kg = (unpack_idx * 32 + lane) / SET_THREADS;
        const int tn = (unpack_idx * 32 + lane) % SET_THREADS;
        const __half2 sixteenth = __float2half2_rn(0.0625f);
        const int src_off = S::X_BYTES + S::WD_BYTES + tn * 4;
        int dst_off[8];
#pragma unroll
        for (int rr = 0; rr < 8; rr++) dst_off[rr] = S::X_BYTES + tn * 128 + ((rr ^ (tn & 7)) << 4);
        const uint32_t ready0 = cluster_map_shared(&ready[0], 0);
        int ti = 0, kb = kg;
        int kbn = items_cta > 0 ? item_kbn(0) : 1;
        while (ti < items_cta && kb >= kbn) {
            kb -= kbn, ti++;
            if (ti < items_cta) kbn = item_kbn(ti);
        }
        const int gshift = (p.group_blocks & (p.group_blocks - 1)) == 0 ? 31 - __clz(p.group_blocks) : -1;
        int kb0_item = ti < items_cta ? item_kb0(ti) : 0;
        int kabs = kb0_item + kb;  // k-block index in the whole K
        int group = kabs / p.group_blocks;
        int n = (ti < items_cta ? item_n0(ti) : 0) + tn;
        __half next_scale = __float2half_rn(0.f);
        uint32_t next_zeros = 0x77777777u;
        auto request = [&]() {
            next_scale = __float2half_rn(0.f), next_zeros = 0x77777777u;
            if (ti < items_cta && n < p.N) {
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
        while (ti < items_cta && ok) {
            if (fresh) {
                const float z = (float)((next_zeros & 15u) + 1u);
                scale2 = __half2half2(next_scale);
                zsub = __float2half2_rn(1024.f + z);
                zfma = __float2half2_rn(-(64.f + z));
                fresh = false;
            }
            // advance to the set's next k-block; a new item or group is requested now and lands during this unpack
            {
                kb += KG;
                const int old_group = group, old_ti = ti;
                while (ti < items_cta && kb >= kbn) {
                    kb -= kbn, ti++;
                    if (ti < items_cta) kbn = item_kbn(ti);
                }
                if (ti < items_cta) {
                    if (ti != old_ti) n = item_n0(ti) + tn, kb0_item = item_kb0(ti);
                    kabs = kb0_item + kb;
                    group = gshift >= 0 ? kabs >> gshift : kabs / p.group_blocks;
                    if (ti != old_ti || group != old_group) request(), fresh = true;
                }
            }
            ok = mbar_wait(&full_w[s], ph, abort_flag, p.status, 4);
            if (!ok) break;
            uint8_t *stage = smem + s * S::STAGE_BYTES;
            const uint32_t *src = (const uint32_t *)(stage + src_off);
#pragma unroll
            for (int rr = 0; rr < 8; rr++) {
                uint32_t w = src[rr * BN];
                const uint32_t lo0 = (w & 0x000f000fu) | 0x64006400u;
                const uint32_t hi0 = (w & 0x00f000f0u) | 0x64006400u;
                w >>= 8;
                const uint32_t lo1 = (w & 0x000f000fu) | 0x64006400u;
                const uint32_t hi1 = (w & 0x00f000f0u) | 0x64006400u;
                const __half2 a = __hmul2(__hsub2(*(const __half2 *)&lo0, zsub), scale2);              // k0, k4
                const __half2 b = __hmul2(__hfma2(*(const __half2 *)&hi0, sixteenth, zfma), scale2);  // k1, k5
                const __half2 c = __hmul2(__hsub2(*(const __half2 *)&lo1, zsub), scale2);              // k2, k6
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
            fence_async_smem();  // make the generic-proxy stores visible to the tensor cores' reads
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(ready0 + (uint32_t)s * 8u);
            s += KG;
            if (s >= STAGES) s -= STAGES, ph ^= 1;
        }
    } else if (warp >= WARPS) {
        // ------------------------------------------------------------------ epilogue: warp w drains TMEM lanes 32 * (w % 4) ..
        const int q = warp & 3;
        const uint32_t acc_empty0 = cluster_map_shared(&acc_empty[0], 0);
        bool ok = true;
        int stg_sel = 0;
        pdl_wait();  // nothing is stored before the kernel before this one is done with its reads and writes
        for (int ti = 0; ti < items_cta && ok; ti++) {
            const int buf = ti & 1, use = ti >> 1;
            ok = mbar_wait_idle(&acc_full[buf], (uint32_t)use & 1u, abort_flag, p.status, 5);
            // the four warps meet at barriers below: they go on together or not at all
            {
                uint32_t all;
                asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.u32 p, %1, 0;\n\tbar.red.and.pred q, 1, 128, p;\n\tselp.u32 %0, 1, 0, q;\n\t}"
                             : "=r"(all) : "r"((uint32_t)ok) : "memory");
                ok = all != 0;
            }
            if (!ok) break;
            tc_fence_after();
            const int m0 = item_m0(ti), n0 = item_n0(ti);
            const uint32_t acc = tmem_base + (uint32_t)buf * ACC_COLS + ((uint32_t)(q * 32) << 16);
            StoreDst d;
            d.n_dst = 1, d.ld = p.N, d.col0 = 0;
            bool out16;
            if (SPLIT) {
                d.dst[0] = p.partial + (int64_t)item_slice(ti) * p.M * p.N, out16 = false;
            } else if constexpr (GATHER) {
#pragma unroll
                for (int g = 0; g < kMaxGatherDst; g++) d.dst[g] = p.dst[g];
                d.n_dst = p.n_dst, d.ld = p.ld_out, d.col0 = p.col0, out16 = p.out_f16 != 0;
            } else {
                d.dst[0] = p.out, out16 = p.out_f16 != 0;
            }
            const bool vec = (p.N & 7) == 0 && (d.ld & 7) == 0 && (d.col0 & 7) == 0;
            const int n_warp = n0 + q * 32;
            const int n = n_warp + lane;
            const float bias = (!SPLIT && p.bias && n < p.N) ? p.bias[n] : 0.f;
            if (is_tail(ti)) {
                // a K slice of a leftover item: the f32 partial tile [MT][256] of this pair, no bias
                StoreDst dt;
                dt.dst[0] = tail.partial + (size_t)pair * MT * (2 * BN), dt.n_dst = 1, dt.ld = 2 * BN, dt.col0 = 0;
#pragma unroll 1
                for (int c = 0; c < MT; c += 16) {
                    uint32_t r[16];
                    tmem_ld_32x32b_x16(acc + (uint32_t)c, r);
                    tmem_ld_wait();
                    store_block16<false>(dt, false, true, r, 0.f, c, MT, (int)rank * BN + q * 32, 2 * BN, lane);
                }
            } else if (!STG || !use_tma_store) {
#pragma unroll 1
                for (int c = 0; c < MT; c += 16) {
                    uint32_t r[16];
                    tmem_ld_32x32b_x16(acc + (uint32_t)c, r);
                    tmem_ld_wait();
                    store_block16<GATHER>(d, out16, vec, r, bias, m0 + c, p.M, n_warp, p.N, lane);
                }
            } else {
                // The result leaves through shared memory: a lane holds one output column of 16 token rows, so it writes
                // 16 words into a [tokens][128 columns] staging tile (no exchange between lanes, no dependent chain), and
                // one thread hands each finished tile to a TMA store, which also clips the ragged edges. A tile is 16 KB:
                // 64 token rows of fp16 or 32 of f32 (also the partial sums of a K slice, third map coordinate). Two tiles
                // alternate; a tile is rewritten once the store that read it has finished reading.
                const int epi_tid = (warp - WARPS) * 32 + lane;  // 0 .. 127, thread 0 issues the stores
                const bool o16 = !SPLIT && out16;
                const int rows = o16 ? STG_ROWS : STG_ROWS / 2;
                const int slice = SPLIT ? item_slice(ti) : 0;
#pragma unroll 1
                for (int c = 0; c < MT; c += rows) {
                    if (epi_tid == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    uint8_t *tile_base = stg + stg_sel * STG_BYTES;
#pragma unroll 1
                    for (int cc = 0; cc < rows; cc += 16) {
                        uint32_t r[16];
                        tmem_ld_32x32b_x16(acc + (uint32_t)(c + cc), r);
                        tmem_ld_wait();
                        if (o16) {
                            __half *tile = (__half *)tile_base + q * 32 + lane;
#pragma unroll
                            for (int j = 0; j < 16; j++) tile[(cc + j) * BN] = __float2half_rn(__uint_as_float(r[j]) + bias);
                        } else {
                            float *tile = (float *)tile_base + q * 32 + lane;
#pragma unroll
                            for (int j = 0; j < 16; j++) tile[(cc + j) * BN] = __uint_as_float(r[j]) + bias;
                        }
                    }
                    fence_async_smem();
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    if (epi_tid == 0) {
                        if (m0 + c < p.M && n0 < p.N)
                            asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%1, %2, %3}], [%4];"
                                         ::"l"(&map_c), "r"(n0), "r"(m0 + c), "r"(slice), "r"(smem_u32(tile_base))
                                         : "memory");
                        asm volatile("cp.async.bulk.commit_group;" ::: "memory");  // also when empty: the waits count groups
                    }
                    stg_sel ^= 1;
                }
            }
            // the accumulator set may be overwritten once the four warps of both CTAs have read it
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(acc_empty0 + (uint32_t)buf * 8u);
        }
        // the staging tiles must outlive the stores that read them
        if (warp == WARPS && lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // neither CTA leaves (or frees tensor memory) while the other may still reach into it
    if (warp == MMA_WARP) tmem_dealloc_pair(tmem_base, TMEM_COLS);
}

// Adds the K slices of the leftover items (PairTail) and stores the tiles: grid (MT rows, leftover items) x 64 threads
// of four columns each.
__global__ void __launch_bounds__(64) pair_tail_reduce_kernel(const float *__restrict__ partial, const int St, const int first_item,
                                                              const int tiles_m, const int MT, const float *__restrict__ bias,
                                                              void *__restrict__ out, const int out_f16, const int M, const int N)
{
    const int r = blockIdx.x, t = blockIdx.y, item = first_item + t;
    const int m = (item % tiles_m) * MT + r, n = (item / tiles_m) * (2 * BN) + (int)threadIdx.x * 4;
    pdl_sync();
    if (m >= M || n >= N) return;  // N % 4 == 0
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s < St; s++) {
        const float4 a = *reinterpret_cast<const float4 *>(partial + (((size_t)(t * St + s) * MT + r) * (2 * BN) + threadIdx.x * 4));
        v.x += a.x, v.y += a.y, v.z += a.z, v.w += a.w;
    }
    if (bias) {
        const float4 b = *reinterpret_cast<const float4 *>(bias + n);
        v.x += b.x, v.y += b.y, v.z += b.z, v.w += b.w;
    }
    const size_t o = (size_t)m * N + n;
    if (out_f16) {
        const __half2 a = __floats2half2_rn(v.x, v.y), b = __floats2half2_rn(v.z, v.w);
        uint2 w;
        w.x = *reinterpret_cast<const uint32_t *>(&a), w.y = *reinterpret_cast<const uint32_t *>(&b);
        *reinterpret_cast<uint2 *>((__half *)out + o) = w;
    } else {
        *reinterpret_cast<float4 *>((float *)out + o) = v;
    }
}

}  // namespace tcp

// How a launch of n_items whole items on `pairs` pairs cuts its last round (see PairTail). False: no cut (the items
// fill the rounds, or the leftover is more than half a round, or K is too short to slice).
bool pair_tail_plan(int64_t n_items, int pairs, int kblocks, int *rounds, int *rem, int *St, int *per)
{
    static const bool on = [] { const char *e = getenv("WEBLLM_B200_GEMM_TAIL"); return !(e && e[0] == '0'); }();
    if (!on || pairs < 2 || n_items <= pairs || kblocks < 8) return false;
    *rounds = (int)(n_items / pairs), *rem = (int)(n_items % pairs);
    if (*rem == 0 || 2 * *rem > pairs) return false;
    int st = pairs / *rem;
    int pr = (kblocks + st - 1) / st;
    if (pr < 2) pr = 2;
    st = (kblocks + pr - 1) / pr;
    if (st < 2) return false;
    // the cut costs a register epilogue of partial tiles and a second launch (~10 us measured): it pays where the k-blocks
    // it takes off the critical path are worth more (K = 3584: 20 us; K = 896: 4 us, where it measured 4.5 us slower)
    if ((kblocks - pr) * 0.37 < 12.) return false;
    *St = st, *per = pr;
    return true;
}

// WEBLLM_B200_GEMM_PAIR=0 keeps every launch on the one-CTA kernels (for comparisons).
static bool pair_enabled()
{
    static const bool on = [] { const char *e = getenv("WEBLLM_B200_GEMM_PAIR"); return !(e && e[0] == '0'); }();
    return on;
}

bool gemm_pair_supports(const Weight &w, int64_t M)
{
    return pair_enabled() && w.kind == WeightKind::Gptq && M >= 128 && w.N >= 256 && w.K % 64 == 0 && w.N % 4 == 0 && w.group % 64 == 0;
}

template <int MT>
static cudaError_t launch_pair_mt(const CUtensorMap &mx, const CUtensorMap &mw, const CUtensorMap *mc, const tc::Params &p, int tiles_m,
                                  int tiles_n, int S, cudaStream_t st, int sms, const tcp::PairTail &tail)
{
    static bool attr_set[5][16] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    const int n_items = tiles_m * tiles_n * S;
    int pairs = sms / 2;
    if (pairs > n_items) pairs = n_items;
    auto go = [&](auto kernel, int variant, int smem) -> cudaError_t {
        if (!(dev >= 0 && dev < 16 && attr_set[variant][dev])) {
            cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
            if (e != cudaSuccess) return e;
            if (dev >= 0 && dev < 16) attr_set[variant][dev] = true;
        }
        return launch_pdl(kernel, dim3((unsigned)(2 * pairs)), dim3(tcp::THREADS_PAIR), (size_t)smem, st, mx, mw, mc ? *mc : mx, p, tiles_m,
                          tiles_n, n_items, mc ? 1 : 0, tail);
    };
    if (S > 1)
        return mc ? go(tcp::gemm_pair_kernel<MT, true, true>, 3, tcp::SmemPair<MT, true>::TOTAL)
                  : go(tcp::gemm_pair_kernel<MT, true, false>, 1, tcp::SmemPair<MT, false>::TOTAL);
    if (p.n_dst > 0) return go(tcp::gemm_pair_kernel<MT, false, false, true>, 4, tcp::SmemPair<MT, false>::TOTAL);
    if (mc) return go(tcp::gemm_pair_kernel<MT, false, true>, 2, tcp::SmemPair<MT, true>::TOTAL);
    return go(tcp::gemm_pair_kernel<MT, false, false>, 0, tcp::SmemPair<MT, false>::TOTAL);
}

// mc: tensor map of the result or of the K slices' partial sums ([slices, M, N], boxes of 128 columns x 64 fp16 or 32 f32
// rows) for the epilogue's TMA stores, or nullptr (a row pitch that is not a multiple of 16 bytes; a long-K launch that
// would rather have the shared memory as a pipeline stage): then the epilogue stores from registers.
// tail_partial: room for sms / 2 partial tiles [mt][256] f32 (the launch cuts its last round along K where that pays, and
// then also launches the small kernel that adds the slices; *extra_launches says so), or nullptr to never cut.
cudaError_t launch_gemm_pair(int mt, const CUtensorMap &mx, const CUtensorMap &mw, const CUtensorMap *mc, const tc::Params &p, int tiles_m,
                             int tiles_n, int S, cudaStream_t st, int sms, float *tail_partial, int *extra_launches)
{
    tcp::PairTail tail;
    int rem = 0;
    *extra_launches = 0;
    if (S == 1 && p.n_dst == 0 && tail_partial &&
        pair_tail_plan((int64_t)tiles_m * tiles_n, sms / 2, p.K / tc::BK, &tail.rounds, &rem, &tail.St, &tail.per)) {
        tail.slots = rem * tail.St;
        tail.partial = tail_partial;
    }
    cudaError_t e;
    switch (mt) {
    case 128: e = launch_pair_mt<128>(mx, mw, mc, p, tiles_m, tiles_n, S, st, sms, tail); break;
    case 192: e = launch_pair_mt<192>(mx, mw, mc, p, tiles_m, tiles_n, S, st, sms, tail); break;
    default: e = launch_pair_mt<256>(mx, mw, mc, p, tiles_m, tiles_n, S, st, sms, tail); break;
    }
    if (e != cudaSuccess || tail.slots == 0) return e;
    *extra_launches = 1;
    return launch_pdl(tcp::pair_tail_reduce_kernel, dim3((unsigned)mt, (unsigned)rem), dim3(64), 0, st, (const float *)tail.partial, tail.St,
                      tail.rounds * (sms / 2), tiles_m, mt, p.bias, p.out, p.out_f16, p.M, p.N);
}

}  // namespace wb
