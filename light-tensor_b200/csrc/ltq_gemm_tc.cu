// uint8 x uint8 -> int32 GEMM on the 5th-generation tensor cores (tcgen05, kind::i8) for sm_100a, with the fused
// zero-point / bias / ReLU / dequantise / requantise epilogue of l-ten's quantized_matmul
// (l-ten/math_fns.cpp:1433-1474).  FullyConnected_q's layout only: A = activations [M,K], B = weights [N,K], both
// K-contiguous (transpose_A = false, transpose_B = true in l-ten/fully_connected.cpp:389-393).
//
// One persistent CTA per SM, 192 threads, three roles:
//   warp 0      TMA producer  : cp.async.bulk.tensor.2d (no multicast) -> 128B-swizzled smem ring, mbarrier tx counts
//   warp 1      MMA issuer    : one thread issues tcgen05.mma.cta_group::1.kind::i8 (128 x BN x 32), u8 x u8 -> s32,
//                               accumulators in TMEM, double buffered (2 x BN columns) so the epilogue of tile t overlaps
//                               the main loop of tile t+1; tcgen05.commit releases smem stages / publishes accumulators
//   warps 2..5  epilogue      : tcgen05.ld 32 lanes x 32 columns at a time, correction terms, conversion, 16-byte stores
//
// Every wait on an mbarrier is bounded (wall-clock limit read from %globaltimer): on expiry the kernel records a code
// in a device status word, stops issuing work, drains and frees its TMEM, and returns.
#include <cuda.h>
#include <stdio.h>
#include <stdlib.h>

#include <type_traits>

#include "ltq_common.cuh"
#include "ltq_gemm_tc.cuh"
#include "ltq_tcgen05.cuh"

namespace ltq {

namespace {

constexpr int BM = 128;          // UMMA M (TMEM lanes)
constexpr int BK = 128;          // bytes (= elements) of K per smem stage: one 128-byte swizzle atom wide
constexpr int UMMA_K = 32;       // kind::i8
constexpr int NUM_THREADS = 192;

template <int BN>
struct Cfg {
    static constexpr int STAGES = (BN == 256) ? 4 : (BN == 128 ? 6 : 8);
    static constexpr int A_BYTES = BM * BK;
    static constexpr int B_BYTES = BN * BK;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int TMEM_COLS = (2 * BN < 32) ? 32 : 2 * BN;  // power of two >= 32
    // ring + 1024 B alignment slack + column terms (2 x BN x 4) + barriers
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 2 * BN * 4 + 256;
};

}  // namespace

// OUT: 0 = uint8, 1 = float, 2 = int32 (ltq_out_mode).
template <int BN, int OUT>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, uint32_t M,
               uint32_t N, uint32_t K, Epilogue epi, void *__restrict__ out, uint32_t *status)
{
    griddep_launch_dependents();
    using C = Cfg<BN>;
    extern __shared__ uint8_t smem_raw[];
    // 128B-swizzled tiles need a 1024-byte aligned base.
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t ring = (raw + 1023u) & ~1023u;
    uint8_t *after = smem_raw + (ring - raw) + C::STAGES * C::STAGE_BYTES;
    uint32_t *s_col = reinterpret_cast<uint32_t *>(after);                 // [2][BN] column terms
    uint64_t *bars = reinterpret_cast<uint64_t *>(after + 2 * BN * 4);     // full[S] empty[S] tfull[2] tempty[2]
    uint32_t *s_misc = reinterpret_cast<uint32_t *>(bars + 2 * C::STAGES + 4);  // [0] tmem base, [1] abort flag
    volatile uint32_t *abort_flag = s_misc + 1;

    const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8 * C::STAGES;
    const uint32_t tfull0 = empty0 + 8 * C::STAGES, tempty0 = tfull0 + 16;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN;
    const uint32_t num_tiles = tiles_m * tiles_n;
    const uint32_t num_kb = (K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; s++) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        for (int s = 0; s < 2; s++) {
            mbar_init(tfull0 + 8 * s, 1);
            mbar_init(tempty0 + 8 * s, 4);  // one arrival per epilogue warp
        }
        s_misc[1] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(s_misc), C::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    // Programmatic dependent launch: everything above ran while the kernel in front may still have been finishing;
    // from here on its results (activations, row sums, device-side qparams) are read.
    griddep_wait();
    epilogue_housekeeping(epi);
    const uint32_t tmem_base = s_misc[0];

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
            uint32_t st = 0, ph = 0;
            bool ok = true;
            for (uint32_t t = blockIdx.x; ok && t < num_tiles; t += gridDim.x) {
                const int32_t m0 = (int32_t)((t / tiles_n) * BM), n0 = (int32_t)((t % tiles_n) * BN);
                for (uint32_t kb = 0; kb < num_kb; kb++) {
                    ok = mbar_wait(empty0 + 8 * st, ph ^ 1, abort_flag, status, 0x100u | st);
                    if (!ok) break;
                    const uint32_t a_dst = ring + st * C::STAGE_BYTES, b_dst = a_dst + C::A_BYTES;
                    mbar_expect_tx(full0 + 8 * st, C::STAGE_BYTES);
                    tma_load_2d(a_dst, &map_a, full0 + 8 * st, (int32_t)(kb * BK), m0);
                    tma_load_2d(b_dst, &map_b, full0 + 8 * st, (int32_t)(kb * BK), n0);
                    if (++st == C::STAGES) { st = 0; ph ^= 1; }
                }
            }
        }
        __syncwarp();  // the warp arrives at the CTA-wide barriers below as a whole
    } else if (warp == 1) {
        // ---------------- MMA issuer: the whole warp runs the loop, one elected lane issues ----------------
        constexpr uint32_t idesc = make_idesc_i8(BM, BN);
        uint32_t st = 0, ph = 0, as = 0, aph = 0;
        bool ok = true;
        for (uint32_t t = blockIdx.x; ok && t < num_tiles; t += gridDim.x) {
            ok = __all_sync(0xFFFFFFFFu, mbar_wait(tempty0 + 8 * as, aph ^ 1, abort_flag, status, 0x200u | as));
            if (!ok) break;
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + as * BN;
            for (uint32_t kb = 0; kb < num_kb; kb++) {
                ok = __all_sync(0xFFFFFFFFu, mbar_wait(full0 + 8 * st, ph, abort_flag, status, 0x300u | st));
                if (!ok) break;
                tc_fence_after();
                const uint32_t a_src = ring + st * C::STAGE_BYTES, b_src = a_src + C::A_BYTES;
                const uint64_t a_desc = make_smem_desc(a_src), b_desc = make_smem_desc(b_src);
                if (elect_one()) {
                    // +32 bytes of K per step: +2 in the descriptor's 16-byte address units
                    umma_i8(d_tmem, a_desc, b_desc, idesc, kb != 0u);
#pragma unroll
                    for (int k = 1; k < BK / UMMA_K; k++) umma_i8(d_tmem, a_desc + 2u * k, b_desc + 2u * k, idesc, 1u);
                    umma_commit(empty0 + 8 * st);  // frees the smem stage once these MMAs have read it
                }
                __syncwarp();
                if (++st == C::STAGES) { st = 0; ph ^= 1; }
            }
            if (!ok) break;
            if (elect_one()) umma_commit(tfull0 + 8 * as);  // accumulator complete
            __syncwarp();
            if (++as == 2) { as = 0; aph ^= 1; }
        }
    } else {
        // ---------------- epilogue (warps 2..5 = 128 threads) ----------------
        const uint32_t q = (uint32_t)warp & 3u;       // TMEM lane quarter this warp may read
        const uint32_t et = threadIdx.x - 64;         // 0..127
        const EpilogueConsts c = epilogue_consts(epi);
        const bool relu = epi.flags & LTQ_FLAG_RELU, sat = epi.flags & LTQ_FLAG_SATURATE;
        using OutT = typename std::conditional<OUT == 0, uint8_t, typename std::conditional<OUT == 1, float, int32_t>::type>::type;
        const uint64_t ldc = epilogue_pitch(epi, N);
        const bool vec_ok = epilogue_vec_ok(epi, out, N, sizeof(OutT));
        uint32_t as = 0, aph = 0;
        bool ok = true;
        for (uint32_t t = blockIdx.x; t < num_tiles; t += gridDim.x) {
            const uint32_t m0 = (t / tiles_n) * BM, n0 = (t % tiles_n) * BN;
            // column terms of this tile -> smem (shared by all 128 rows)
            uint32_t *col = s_col + as * BN;
            for (uint32_t j = et; j < (uint32_t)BN; j += 128) {
                const uint32_t gj = n0 + j;
                col[j] = gj < N ? epilogue_col_term(epi, c, gj) : 0u;
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            const uint32_t row = m0 + q * 32 + lane;
            const uint32_t rt = row < M ? epilogue_row_term(epi, c, row) : 0u;

            if (ok) ok = mbar_wait(tfull0 + 8 * as, aph, abort_flag, status, 0x400u | as);
            if (ok) {
                tc_fence_after();
                const uint32_t taddr = tmem_base + ((q * 32u) << 16) + as * BN;
                uint32_t rsum = 0;  // sum of this row's uint8 outputs in this tile
#pragma unroll 1
                for (int ch = 0; ch < BN / 32; ch++) {
                    uint32_t v[32];
                    tmem_ld32(taddr + ch * 32, v);
                    tmem_ld_wait();
                    const uint32_t c0 = n0 + ch * 32;
                    if (row < M && c0 < N)
                        rsum += epilogue_chunk<OUT, 32>(v, rt, col + ch * 32, c, relu, sat, epi, out, epilogue_offset(epi, row, c0, ldc),
                                                        vec_ok, (N - c0) < 32u ? (int)(N - c0) : 32);
                }
                if (OUT == 0 && epi.out_rowsum && row < M) atomicAdd(&epi.out_rowsum[row], (int32_t)rsum);
                // all of this warp's reads of the accumulator are done -> hand the buffer back to the MMA warp
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(tempty0 + 8 * as);
            }
            if (++as == 2) { as = 0; aph ^= 1; }
        }
    }

    // Teardown: nobody leaves before every role is done with TMEM and shared memory.
    tc_fence_before();
    __syncthreads();
    if (warp == 0 && lane == 0 && *abort_flag) {
        // After a timeout bulk copies issued by this thread may still be in flight towards this CTA's shared memory.
        // They complete within microseconds of being issued; hold the CTA for a bounded 2 ms before it exits.
        const uint64_t t0 = global_ns();
        while (global_ns() - t0 < 2000000ull) __nanosleep(1000);
    }
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
}

// ---- CTA-pair variant ---------------------------------------------------------------------------------------------------
// Large problems: two CTAs of a 2-CTA cluster work on one 256-row output tile with tcgen05.mma.cta_group::2.  Each CTA
// loads its own 128 rows of A and only HALF of the tile's B rows, so a CTA moves at most 32 KB per 128-deep K block
// instead of 48 KB: one third less L2 -> SM traffic, and six stages instead of four fit in shared memory, which is what
// it takes to cover the L2 round trip at the tensor pipe's rate.  The leader CTA (cluster rank 0) issues the MMAs for
// both; every barrier that both CTAs must observe is signalled through tcgen05.commit with a two-CTA mask.
// Eight epilogue warps per CTA (two per TMEM lane quarter, splitting the columns) keep the exposed epilogue of a CTA's
// last tile short.
//
// Tile widths are chosen per problem (PairTiling): an MMA of 256 x W x 32 costs W / 2 cycles for any W that is a multiple
// of 16 from ~128 up, so tiles need not be equally wide.  The host cuts every 256-row band of the output into tiles
// whose count over all bands is a whole number of rounds of the device's CTA pairs and whose widths differ by 16 within
// a band; tiles are numbered widest first, so each round of the round-robin hands every pair (almost) the same
// amount of work and the narrowest tiles - with the shortest epilogue - come last.  4096^3 on 74 pairs: 296 tiles of
// 240 / 224 / 208 columns = exactly 4 rounds costing 240 + 224 + 224 + 208 = 896 columns, against 4 x 256 for uniform
// 256-wide tiles (256 tiles, last round a third full) or 4 x 240 for uniform 240-wide ones (288 tiles, 224 wasted columns).
// Two alternatives for the remainder behind the last whole round were built and measured: half-width tiles (an MMA
// with N = 128 needs 24 KB stages at twice the rate, more bytes in flight than the ring holds: 9.1 us per half tile
// against 9.6 us for a whole one) and splitting K over two pairs with an exchange of partial sums through L2 (the
// exchange's three dependent L2 round trips cost 6 us).
namespace {

constexpr int P_MAX_STAGES = 6;
constexpr int P_THREADS = 64 + 8 * 32;  // producer warp, MMA warp, 8 epilogue warps
constexpr int P_BN = 256;               // widest tile
constexpr int P_A_BYTES = BM * BK;
constexpr int P_B_BYTES = (P_BN / 2) * BK;  // room for this CTA's half of the widest tile's B rows
constexpr int P_STAGE_BYTES = P_A_BYTES + P_B_BYTES;
constexpr int P_TAIL_BYTES = 1024 + 2 * P_BN * 4 + 256;  // alignment slack + column terms + barriers
constexpr int P_PEER_STAGE_BYTES = 8 * PeerStage::BYTES_PER_WARP;
inline size_t pair_smem_bytes(int stages, bool peer_stage)
{
    return (size_t)stages * P_STAGE_BYTES + P_TAIL_BYTES + (peer_stage ? P_PEER_STAGE_BYTES : 0);
}

struct PairTile {
    uint32_t m0, n0, width, cls;
};
// (selects instead of indexing: a kernel parameter indexed with a run-time value would be copied to local memory)
__device__ __forceinline__ uint32_t pick4(const uint32_t (&a)[4], uint32_t k)
{
    return k == 0 ? a[0] : (k == 1 ? a[1] : (k == 2 ? a[2] : a[3]));
}
__device__ __forceinline__ PairTile pair_tile(const PairTiling &tl, uint32_t t)
{
    uint32_t k = 0;
    if (t >= tl.start[1]) k = 1;
    if (t >= tl.start[2]) k = 2;
    if (t >= tl.start[3]) k = 3;
    const uint32_t local = t - pick4(tl.start, k), per_row = pick4(tl.per_row, k);
    const uint32_t r = local / per_row, j = local - r * per_row;
    PairTile pt;
    pt.m0 = (pick4(tl.row0, k) + r) * (2 * BM);
    pt.width = pick4(tl.width, k);
    pt.n0 = pick4(tl.col0, k) + j * pt.width;
    pt.cls = k;
    return pt;
}

}  // namespace

template <int OUT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(P_THREADS, 2)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b0,
                    const __grid_constant__ CUtensorMap map_b1, const __grid_constant__ CUtensorMap map_b2,
                    const __grid_constant__ CUtensorMap map_b3, const PairTiling tl, uint32_t M, uint32_t N, uint32_t K,
                    uint32_t stages, Epilogue epi, void *__restrict__ out, uint32_t *status)
{
    griddep_launch_dependents();
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t ring = (raw + 1023u) & ~1023u;
    uint8_t *after = smem_raw + (ring - raw) + stages * P_STAGE_BYTES;
    uint32_t *s_col = reinterpret_cast<uint32_t *>(after);                  // [2][P_BN] column terms
    uint64_t *bars = reinterpret_cast<uint64_t *>(after + 2 * P_BN * 4);    // full[S] empty[S] tfull[2] tempty[2]
    uint32_t *s_misc = reinterpret_cast<uint32_t *>(bars + 2 * P_MAX_STAGES + 4);  // [0] tmem base, [1] abort flag
    volatile uint32_t *abort_flag = s_misc + 1;
    uint8_t *s_stage = after + 2 * P_BN * 4 + 256;    // [8 warps][32 rows][128 B], only allocated when epi.staged

    const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8 * P_MAX_STAGES;
    const uint32_t tfull0 = empty0 + 8 * P_MAX_STAGES, tempty0 = tfull0 + 16;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();          // 0 = leader
    const uint32_t pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
    const uint32_t num_tiles = tl.num_tiles;
    const uint32_t num_kb = (K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < stages; s++) {
            mbar_init(full0 + 8 * s, 1);    // leader's own arrive.expect_tx; bytes come from both CTAs
            mbar_init(empty0 + 8 * s, 1);   // the leader's commit, delivered to both CTAs
        }
        for (int s = 0; s < 2; s++) {
            mbar_init(tfull0 + 8 * s, 1);    // the leader's commit, delivered to both CTAs
            mbar_init(tempty0 + 8 * s, 16);  // eight epilogue warps in each of the two CTAs (used in the leader only)
        }
        s_misc[1] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 0 && lane == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b0) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b1) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b2) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b3) : "memory");
    }
    if (warp == 1) {
        tmem_alloc_pair(smem_u32(s_misc), 512);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync();  // the peer's barriers exist before anything is signalled across
    griddep_wait();  // programmatic dependent launch: the set-up above overlapped the previous kernel's tail
    epilogue_housekeeping(epi);
    tc_fence_after();
    const uint32_t tmem_base = s_misc[0];

    if (warp == 0) {
        // ---------------- TMA producer (both CTAs): own A rows, own half of the tile's B rows ----------------
        // (Asking the boxes a few K blocks ahead into L2 with cp.async.bulk.prefetch.tensor was measured: 58 us instead of
        // 46 us at 4096^3 - the prefetches take the TMA unit's time away from the loads.)
        if (lane == 0) {
            uint32_t st = 0, ph = 0;
            bool ok = true;
            for (uint32_t t = pair; ok && t < num_tiles; t += num_pairs) {
                const PairTile pt = pair_tile(tl, t);
                const uint32_t b_rows = pt.width / 2;
                const CUtensorMap *mb = pt.cls == 0 ? &map_b0 : (pt.cls == 1 ? &map_b1 : (pt.cls == 2 ? &map_b2 : &map_b3));
                const int32_t m0 = (int32_t)(pt.m0 + rank * BM);
                const int32_t n0 = (int32_t)(pt.n0 + rank * b_rows);
                const uint32_t tx = 2u * (uint32_t)(P_A_BYTES + b_rows * BK);
                for (uint32_t kb = 0; kb < num_kb; kb++) {
                    ok = mbar_wait(empty0 + 8 * st, ph ^ 1, abort_flag, status, 0x100u | st);
                    if (!ok) break;
                    const uint32_t a_dst = ring + st * P_STAGE_BYTES, b_dst = a_dst + P_A_BYTES;
                    const uint32_t lbar = in_leader_cta(full0 + 8 * st);
                    if (rank == 0) mbar_expect_tx(full0 + 8 * st, tx);
                    tma_load_2d_pair(a_dst, &map_a, lbar, (int32_t)(kb * BK), m0);
                    tma_load_2d_pair(b_dst, mb, lbar, (int32_t)(kb * BK), n0);
                    if (++st == stages) { st = 0; ph ^= 1; }
                }
            }
        }
        __syncwarp();  // the warp arrives at the CTA-wide barriers below as a whole
    } else if (warp == 1) {
        // ---------------- MMA issuer (leader CTA only): warp-uniform loop, one elected lane issues ----------------
        if (rank == 0) {
            uint32_t st = 0, ph = 0, as = 0, aph = 0;
            bool ok = true;
            for (uint32_t t = pair; ok && t < num_tiles; t += num_pairs) {
                const uint32_t idesc = make_idesc_i8(2 * BM, (int)pair_tile(tl, t).width);
                ok = __all_sync(0xFFFFFFFFu, mbar_wait(tempty0 + 8 * as, aph ^ 1, abort_flag, status, 0x200u | as));
                if (!ok) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + as * P_BN;
                for (uint32_t kb = 0; kb < num_kb; kb++) {
                    ok = __all_sync(0xFFFFFFFFu, mbar_wait(full0 + 8 * st, ph, abort_flag, status, 0x300u | st));
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t a_src = ring + st * P_STAGE_BYTES, b_src = a_src + P_A_BYTES;
                    const uint64_t a_desc = make_smem_desc(a_src), b_desc = make_smem_desc(b_src);
                    if (elect_one()) {
                        umma_i8_pair(d_tmem, a_desc, b_desc, idesc, kb != 0u);
#pragma unroll
                        for (int k = 1; k < BK / UMMA_K; k++)
                            umma_i8_pair(d_tmem, a_desc + 2u * k, b_desc + 2u * k, idesc, 1u);
                        umma_commit_pair(empty0 + 8 * st, 3);  // both CTAs may refill the stage
                    }
                    __syncwarp();
                    if (++st == stages) { st = 0; ph ^= 1; }
                }
                if (!ok) break;
                if (elect_one()) umma_commit_pair(tfull0 + 8 * as, 3);  // accumulators complete in both CTAs
                __syncwarp();
                if (++as == 2) { as = 0; aph ^= 1; }
            }
        }
    } else {
        // ---------------- epilogue (warps 2..9 of both CTAs): own 128 rows; two warps share a lane quarter ------------
        const uint32_t q = (uint32_t)warp & 3u;            // TMEM lane quarter this warp may read
        const uint32_t h = (uint32_t)(warp - 2) >> 2;      // 0: lower column range of the tile, 1: upper
        const uint32_t et = threadIdx.x - 64;              // 0..255
        const EpilogueConsts c = epilogue_consts(epi);
        const bool relu = epi.flags & LTQ_FLAG_RELU, sat = epi.flags & LTQ_FLAG_SATURATE;
        using OutT = typename std::conditional<OUT == 0, uint8_t, typename std::conditional<OUT == 1, float, int32_t>::type>::type;
        const uint64_t ldc = epilogue_pitch(epi, N);
        const bool vec_ok = epilogue_vec_ok(epi, out, N, sizeof(OutT));
        const bool staged = epi.staged && vec_ok && epi.col_block == 0;
        constexpr int ESZ = (int)sizeof(OutT), BLOCK_COLS = 128 / ESZ;   // a staged block: 128 bytes per row
        uint8_t *stage = s_stage + (warp - 2) * PeerStage::BYTES_PER_WARP;
        uint32_t as = 0, aph = 0;
        bool ok = true;
        for (uint32_t t = pair; t < num_tiles; t += num_pairs) {
            const PairTile pt = pair_tile(tl, t);
            const uint32_t m0 = pt.m0 + rank * BM, n0 = pt.n0;
            const int width = (int)pt.width;
            const int split = ((width / 2 + 15) / 16) * 16;   // columns [0, split) go to the h = 0 warps, the rest to h = 1
            uint32_t *col = s_col + as * P_BN;
            for (uint32_t j = et; j < (uint32_t)width; j += 256) {
                const uint32_t gj = n0 + j;
                col[j] = gj < N ? epilogue_col_term(epi, c, gj) : 0u;
            }
            asm volatile("bar.sync 1, 256;" ::: "memory");
            const uint32_t row = m0 + q * 32 + lane;
            const uint32_t rt = row < M ? epilogue_row_term(epi, c, row) : 0u;

            if (ok) ok = mbar_wait(tfull0 + 8 * as, aph, abort_flag, status, 0x400u | as);
            if (ok) {
                tc_fence_after();
                const uint32_t taddr = tmem_base + ((q * 32u) << 16) + as * P_BN;
                const int cb = h ? split : 0, ce = h ? width : split;
                const bool rows_full = m0 + q * 32 + 32 <= M;
                uint32_t rsum = 0;  // sum of this row's uint8 outputs in this warp's part of the tile
                // One chunk of CW (32, or 16 for a remainder) accumulator columns.  Blocks of 128 output bytes per row go
                // through the row-coalescing stage when results leave the GPU and the warp's 32 rows and the block's columns
                // are all inside the matrix; everything else is stored directly.  (32-column chunks with two adjacent
                // 16-byte stores per row measured 20 % faster than 16-column chunks with one, software-pipelined TMEM
                // loads included: the stores, one 32-byte sector per row, are what the chunk waits for.)
                auto chunk = [&](auto &v, int cc) {
                    constexpr int CW = (int)(sizeof(v) / sizeof(uint32_t));
                    const uint32_t c0 = n0 + cc;
                    const int bc0 = cb + ((cc - cb) / BLOCK_COLS) * BLOCK_COLS;          // first column of cc's block
                    const int bcols = (ce - bc0) < BLOCK_COLS ? (ce - bc0) : BLOCK_COLS;  // its width
                    const bool via_stage = staged && rows_full && n0 + bc0 + bcols <= N;
                    if (via_stage) {
                        uint32_t res[CW];
                        epilogue_convert<OUT, CW>(v, rt, col + cc, c, relu, sat, res);
                        PeerStage::put<CW>(stage, lane, (cc - bc0) * ESZ / 16, res, CW * ESZ / 16);
                        if (OUT == 0) rsum += packed_byte_sum<CW>(res, CW);
                        const int next = cc + CW;
                        if (next == ce || (next - cb) % BLOCK_COLS == 0)   // the block is complete
                            PeerStage::flush(stage, lane, bcols * ESZ / 16, epi, out,
                                             ((uint64_t)(m0 + q * 32) * ldc + n0 + bc0) * ESZ, ldc * ESZ);
                    } else if (row < M && c0 < N) {
                        rsum += epilogue_chunk<OUT, CW>(v, rt, col + cc, c, relu, sat, epi, out, epilogue_offset(epi, row, c0, ldc),
                                                        vec_ok, (N - c0) < (uint32_t)CW ? (int)(N - c0) : CW);
                    }
                };
                int cc = cb;
#pragma unroll 1
                for (; cc + 32 <= ce; cc += 32) {
                    uint32_t v[32];
                    tmem_ld32(taddr + cc, v);
                    tmem_ld_wait();
                    chunk(v, cc);
                }
                if (cc < ce) {  // widths are multiples of 16
                    uint32_t v[16];
                    tmem_ld16(taddr + cc, v);
                    tmem_ld_wait();
                    chunk(v, cc);
                }
                if (OUT == 0 && epi.out_rowsum && row < M) atomicAdd(&epi.out_rowsum[row], (int32_t)rsum);
                // this warp has read its part of the accumulator: tell the leader's MMA warp (in this or the other CTA)
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_remote(in_leader_cta(tempty0 + 8 * as));
            }
            if (++as == 2) { as = 0; aph ^= 1; }
        }
    }

    // Teardown.  The leader's MMAs read the peer's shared memory and both CTAs' barriers receive remote arrivals, so
    // neither CTA may exit before both are completely done.
    tc_fence_before();
    __syncthreads();
    if (warp == 0 && lane == 0 && *abort_flag) {
        const uint64_t t0 = global_ns();
        while (global_ns() - t0 < 2000000ull) __nanosleep(1000);
    }
    __syncthreads();
    cluster_sync();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, 512);
    }
}

// ---- host side ------------------------------------------------------------------------------------------------------
namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn()
{
    // resolved once; a function-local static is initialised under the language's own lock, so two host threads that
    // arrive together both see the finished pointer
    static const EncodeTiledFn fn = [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            return reinterpret_cast<EncodeTiledFn>(p);
        return static_cast<EncodeTiledFn>(nullptr);
    }();
    return fn;
}

template <int BN, int OUT>
cudaError_t launch_cfg(const CUtensorMap &ma, const CUtensorMap &mb, uint64_t M, uint64_t N, uint64_t K,
                       const Epilogue &epi, void *out, uint32_t *status, int sms, cudaStream_t stream)
{
    using C = Cfg<BN>;
    static bool attr_done[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_done[dev]) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<BN, OUT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             C::SMEM_BYTES);
        if (e != cudaSuccess) return e;
        attr_done[dev] = true;
    }
    const uint64_t tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
    const unsigned grid = (unsigned)(tiles < (uint64_t)sms ? tiles : (uint64_t)sms);
    cudaError_t e = launch_chained(gemm_tc_kernel<BN, OUT>, dim3(grid), dim3(NUM_THREADS), (size_t)C::SMEM_BYTES, stream, ma, mb,
                                   (uint32_t)M, (uint32_t)N, (uint32_t)K, epi, out, status);
    count_launch();
    note_kernel("gemm_tc_kernel<%d,%s>", BN, out_mode_name(OUT));
    return e;
}

template <int BN>
cudaError_t launch_out(const CUtensorMap &ma, const CUtensorMap &mb, uint64_t M, uint64_t N, uint64_t K,
                       const Epilogue &epi, void *out, uint32_t *status, int sms, cudaStream_t stream)
{
    switch (epi.out_mode) {
        case LTQ_OUT_U8: return launch_cfg<BN, 0>(ma, mb, M, N, K, epi, out, status, sms, stream);
        case LTQ_OUT_F32: return launch_cfg<BN, 1>(ma, mb, M, N, K, epi, out, status, sms, stream);
        default: return launch_cfg<BN, 2>(ma, mb, M, N, K, epi, out, status, sms, stream);
    }
}

}  // namespace

namespace {

template <int OUT>
cudaError_t launch_pair(const CUtensorMap &ma, const CUtensorMap *const mb[4], const PairTiling &tl, uint64_t M, uint64_t N,
                        uint64_t K, const Epilogue &epi, void *out, uint32_t *status, int sms, cudaStream_t stream)
{
    static bool attr_done[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_done[dev]) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_pair_kernel<OUT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)pair_smem_bytes(P_MAX_STAGES, false));
        if (e != cudaSuccess) return e;
        attr_done[dev] = true;
    }
    const uint64_t all_pairs = (uint64_t)(sms / 2);
    const uint64_t pairs = tl.num_tiles < all_pairs ? tl.num_tiles : all_pairs;
    // With further destinations (peer GPUs) the epilogue warps get a row-coalescing stage in place of one ring stage
    // (such launches are bound by the links, not by the tensor pipe).  Local-only stores gain nothing from it: measured.
    Epilogue epi_l = epi;
    epi_l.staged = (epi.n_more > 0 || epi.mc) ? 1 : 0;
    uint32_t stages = epi_l.staged ? P_MAX_STAGES - 1 : P_MAX_STAGES;
    const size_t smem = pair_smem_bytes((int)stages, epi_l.staged != 0);
    cudaError_t e = launch_chained(gemm_tc_pair_kernel<OUT>, dim3((unsigned)(2 * pairs)), dim3(P_THREADS), smem, stream, ma,
                                   *mb[0], *mb[1], *mb[2], *mb[3], tl, (uint32_t)M, (uint32_t)N, (uint32_t)K, stages,
                                   epi_l, out, status);
    count_launch();
    char widths[48];
    int n = 0;
    for (int k = 0; k < 4 && tl.start[k] < tl.num_tiles; k++)
        n += snprintf(widths + n, sizeof widths - n, "%s%u", k ? "/" : "", tl.width[k]);
    note_kernel("gemm_tc_pair_kernel<%s> (%u tiles of %s columns)", out_mode_name(OUT), tl.num_tiles, widths);
    return e;
}

}  // namespace

bool tc_pair_preferred(uint64_t M, uint64_t N, int sms)
{
    // Worth pairing once 256 x 256 tiles can occupy most CTA pairs of the device.
    // (with at most 128 rows the second CTA of a pair would have nothing to do)
    const uint64_t tiles = ((M + 2 * BM - 1) / (2 * BM)) * ((N + 255) / 256);
    return M > (uint64_t)BM && tiles * 4 >= (uint64_t)(sms / 2) * 3;
}

PairTiling tc_pair_tiling(uint64_t M, uint64_t N, int sms, bool unit32)
{
    // Every 256-row band is cut into tiles whose widths are multiples of `unit` columns and differ by at most one unit
    // within the band.  The number of tiles over all bands is the smallest whole number of rounds of the CTA pairs that
    // keeps every tile at most 256 columns wide (uniform 256-wide tiles when that would make tiles narrower than 128
    // columns: a narrow MMA no longer costs in proportion to its width).
    const uint64_t unit = unit32 ? 32 : 16, wmax = P_BN / unit;
    const uint64_t TM = (M + 2 * BM - 1) / (2 * BM), U = (N + unit - 1) / unit, P = (uint64_t)(sms / 2);
    const uint64_t c_min = (U + wmax - 1) / wmax;             // tiles per band at full width
    uint64_t T = ((TM * c_min + P - 1) / P) * P;               // whole rounds that hold at least that many tiles
    if (T / TM > U) T = TM * U;                                // (never narrower than one unit)
    if ((U / ((T + TM - 1) / TM)) * unit < 128) T = TM * c_min;
    const uint64_t c_lo = T / TM, n_hi = T % TM, n_lo = TM - n_hi;
    struct Cls {
        uint64_t row0, rows, per_row, col0, w;
    } cls[4];
    int nc = 0;
    auto band = [&](uint64_t row0, uint64_t rows, uint64_t c) {
        if (rows == 0 || c == 0) return;
        const uint64_t base = U / c, extra = U % c;
        if (extra) cls[nc++] = Cls{row0, rows, extra, 0, (base + 1) * unit};
        if (c - extra) cls[nc++] = Cls{row0, rows, c - extra, extra * (base + 1) * unit, base * unit};
    };
    band(0, n_lo, c_lo);
    band(n_lo, n_hi, c_lo + 1);
    for (int a = 1; a < nc; a++)  // widest first (insertion sort, stable)
        for (int b = a; b > 0 && cls[b].w > cls[b - 1].w; b--) {
            const Cls tmp = cls[b];
            cls[b] = cls[b - 1];
            cls[b - 1] = tmp;
        }
    PairTiling tl;
    uint64_t start = 0;
    for (int k = 0; k < 4; k++) {
        if (k < nc) {
            tl.start[k] = (uint32_t)start;
            tl.per_row[k] = (uint32_t)cls[k].per_row;
            tl.row0[k] = (uint32_t)cls[k].row0;
            tl.col0[k] = (uint32_t)cls[k].col0;
            tl.width[k] = (uint32_t)cls[k].w;
            start += cls[k].rows * cls[k].per_row;
        } else {
            tl.start[k] = 0xFFFFFFFFu;
            tl.per_row[k] = 1;
            tl.row0[k] = tl.col0[k] = 0;
            tl.width[k] = nc ? tl.width[nc - 1] : 256;
        }
    }
    tl.num_tiles = (uint32_t)start;
    return tl;
}

cudaError_t launch_gemm_tc_pair(const TcOperandMap &map_a, const TcOperandMap *const map_b[4], const PairTiling &tl, uint64_t M,
                                uint64_t N, uint64_t K, const Epilogue &epi, void *out, uint32_t *status, int sms,
                                cudaStream_t stream)
{
    const CUtensorMap &ma = *reinterpret_cast<const CUtensorMap *>(map_a.opaque);
    const CUtensorMap *mb[4];
    for (int k = 0; k < 4; k++) mb[k] = reinterpret_cast<const CUtensorMap *>(map_b[k]->opaque);
    switch (epi.out_mode) {
        case LTQ_OUT_U8: return launch_pair<0>(ma, mb, tl, M, N, K, epi, out, status, sms, stream);
        case LTQ_OUT_F32: return launch_pair<1>(ma, mb, tl, M, N, K, epi, out, status, sms, stream);
        default: return launch_pair<2>(ma, mb, tl, M, N, K, epi, out, status, sms, stream);
    }
}

bool tc_shape_ok(uint64_t M, uint64_t N, uint64_t K, const void *A, const void *B)
{
    return M >= 1 && N >= 1 && K >= 16 && (K % 16 == 0) && M < (1ull << 31) && N < (1ull << 31) &&
           K < (1ull << 31) && (((uintptr_t)A & 15) == 0) && (((uintptr_t)B & 15) == 0) && encode_fn() != nullptr;
}

int tc_pick_bn(uint64_t M, uint64_t N, int sms)
{
    // Widest tile that still gives every SM a tile; problems too small for that get narrower tiles (more CTAs).
    const uint64_t tm = (M + BM - 1) / BM, s = (uint64_t)sms;
    if (tm * ((N + 255) / 256) >= s) return 256;
    if (tm * ((N + 127) / 128) >= s) return 128;
    if (N <= 64) return 64;
    return tm * ((N + 127) / 128) >= s / 2 ? 128 : 64;
}

int tc_make_map(TcOperandMap *m, const uint8_t *base, uint64_t rows, uint64_t K, int box_rows)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn) return -1;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)K};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(reinterpret_cast<CUtensorMap *>(m->opaque), CU_TENSOR_MAP_DATA_TYPE_UINT8, 2,
                    const_cast<uint8_t *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return (int)r;
    m->base = base;
    m->rows = rows;
    m->K = K;
    m->box_rows = box_rows;
    m->box_lines = 0;
    return 0;
}

int tc_make_map_lines(TcOperandMap *m, const uint8_t *base, uint64_t rows, uint64_t K, int box_rows, int box_lines)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn) return -1;
    if (K % 128 != 0) return -2;
    // dim0: the 128 bytes of a line; dim1: matrix rows (pitch K); dim2: lines along K (pitch 128).
    cuuint64_t dims[3] = {128, (cuuint64_t)rows, (cuuint64_t)(K / 128)};
    cuuint64_t strides[2] = {(cuuint64_t)K, 128};
    cuuint32_t box[3] = {128, (cuuint32_t)box_rows, (cuuint32_t)box_lines};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(reinterpret_cast<CUtensorMap *>(m->opaque), CU_TENSOR_MAP_DATA_TYPE_UINT8, 3,
                    const_cast<uint8_t *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return (int)r;
    m->base = base;
    m->rows = rows;
    m->K = K;
    m->box_rows = box_rows;
    m->box_lines = box_lines;
    return 0;
}

cudaError_t launch_gemm_tc(const TcOperandMap &map_a, const TcOperandMap &map_b, int bn, uint64_t M, uint64_t N,
                           uint64_t K, const Epilogue &epi, void *out, uint32_t *status, int sms, cudaStream_t stream)
{
    const CUtensorMap &ma = *reinterpret_cast<const CUtensorMap *>(map_a.opaque);
    const CUtensorMap &mb = *reinterpret_cast<const CUtensorMap *>(map_b.opaque);
    switch (bn) {
        case 256: return launch_out<256>(ma, mb, M, N, K, epi, out, status, sms, stream);
        case 128: return launch_out<128>(ma, mb, M, N, K, epi, out, status, sms, stream);
        case 64: return launch_out<64>(ma, mb, M, N, K, epi, out, status, sms, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace ltq
