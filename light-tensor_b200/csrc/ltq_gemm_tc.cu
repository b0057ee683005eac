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
// Large problems: two CTAs of a 2-CTA cluster work on one 256 x PBN output tile with tcgen05.mma.cta_group::2.  Each CTA
// loads its own 128 rows of A and only HALF of the tile's B rows, so a CTA moves at most 32 KB per 128-deep K block
// instead of 48 KB: one third less L2 -> SM traffic, and six stages instead of four fit in shared memory, which is what
// it takes to cover the L2 round trip at the tensor pipe's rate.  The leader CTA (cluster rank 0) issues the MMAs for
// both; every barrier that both CTAs must observe is signalled through tcgen05.commit with a two-CTA mask.
// Eight epilogue warps per CTA (two per TMEM lane quarter, splitting the columns) keep the exposed epilogue of a CTA's
// last tile short.  PBN (256, 240, 224 or 192) is picked per problem so that the last wave of tiles is as full as
// possible: integer tiles x CTA pairs rarely divide evenly, and a narrower tile can save a whole wave.
//
// Tail wave: work is a list of items handed out round-robin to the CTA pairs.  The first n_full tiles are one item
// each; every tile behind them is TWO items of half the width (256 x PBN/2: an MMA with N = PBN/2, a B box of PBN/4
// rows per CTA, same ring, same accumulator buffers).  The host chooses n_full so that the full tiles fill whole rounds
// and the remainder runs as one round of half tiles: 4096^3 on 74 pairs is 3 rounds of 256 x 256 plus 68 half tiles
// instead of 4 rounds, and the epilogue left exposed at the very end is that of a half tile.  Integer sums make every
// tiling of the output bit-identical.
namespace {

constexpr int P_STAGES = 6;
constexpr int P_THREADS = 64 + 8 * 32;  // producer warp, MMA warp, 8 epilogue warps

template <int PBN>
struct PCfg {
    static constexpr int A_BYTES = BM * BK;
    static constexpr int B_BYTES = (PBN / 2) * BK;  // this CTA's half of the tile's B rows
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int SMEM_BYTES = P_STAGES * STAGE_BYTES + 1024 + 2 * PBN * 4 + 256;
    static constexpr bool HALVES = PBN == 256;      // half-width items exist for this tile width
    static_assert(B_BYTES % 1024 == 0, "swizzled tiles must stay 1024-byte aligned");
    static_assert(PBN % 16 == 0 && PBN >= 144 && PBN <= 256, "tile width");
};

// Work item `i` of a launch: tile row block, first column, and whether it is a half-width item.
struct PairItem {
    uint32_t tm, n0;
    bool half;
};
template <int PBN>
__device__ __forceinline__ PairItem pair_item(uint32_t i, uint32_t n_full, uint32_t tiles_n)
{
    PairItem it;
    it.half = i >= n_full;
    uint32_t t = i, sel = 0;
    if (it.half) {
        const uint32_t j = i - n_full;
        t = n_full + (j >> 1);
        sel = j & 1u;
    }
    it.tm = t / tiles_n;
    it.n0 = (t % tiles_n) * PBN + sel * (PBN / 2);
    return it;
}

}  // namespace

template <int PBN, int OUT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(P_THREADS, 2)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const __grid_constant__ CUtensorMap map_b_half, uint32_t M, uint32_t N, uint32_t K, uint32_t n_full,
                    Epilogue epi, void *__restrict__ out, uint32_t *status)
{
    griddep_launch_dependents();
    using C = PCfg<PBN>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t ring = (raw + 1023u) & ~1023u;
    uint8_t *after = smem_raw + (ring - raw) + P_STAGES * C::STAGE_BYTES;
    uint32_t *s_col = reinterpret_cast<uint32_t *>(after);                  // [2][PBN] column terms
    uint64_t *bars = reinterpret_cast<uint64_t *>(after + 2 * PBN * 4);     // full[S] empty[S] tfull[2] tempty[2]
    uint32_t *s_misc = reinterpret_cast<uint32_t *>(bars + 2 * P_STAGES + 4);  // [0] tmem base, [1] abort flag
    volatile uint32_t *abort_flag = s_misc + 1;
    uint8_t *s_stage = after + 2 * PBN * 4 + 256;     // [8 warps][32 rows][128 B], only allocated when epi.staged

    const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8 * P_STAGES;
    const uint32_t tfull0 = empty0 + 8 * P_STAGES, tempty0 = tfull0 + 16;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();          // 0 = leader
    const uint32_t pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
    const uint32_t tiles_m = (M + 2 * BM - 1) / (2 * BM), tiles_n = (N + PBN - 1) / PBN;
    const uint32_t num_tiles = tiles_m * tiles_n;
    if (!C::HALVES || n_full > num_tiles) n_full = num_tiles;
    const uint32_t num_items = n_full + 2 * (num_tiles - n_full);
    const uint32_t num_kb = (K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < P_STAGES; s++) {
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
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
        if (C::HALVES) asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b_half) : "memory");
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
        // ---------------- TMA producer (both CTAs): own A rows, own half of the item's B rows ----------------
        if (lane == 0) {
            uint32_t st = 0, ph = 0;
            bool ok = true;
            for (uint32_t i = pair; ok && i < num_items; i += num_pairs) {
                const PairItem it = pair_item<PBN>(i, n_full, tiles_n);
                const uint32_t b_rows = it.half ? PBN / 4 : PBN / 2;
                const CUtensorMap *mb = it.half ? &map_b_half : &map_b;
                const int32_t m0 = (int32_t)(it.tm * (2 * BM) + rank * BM);
                const int32_t n0 = (int32_t)(it.n0 + rank * b_rows);
                const uint32_t tx = 2u * (uint32_t)(C::A_BYTES + b_rows * BK);
                for (uint32_t kb = 0; kb < num_kb; kb++) {
                    ok = mbar_wait(empty0 + 8 * st, ph ^ 1, abort_flag, status, 0x100u | st);
                    if (!ok) break;
                    const uint32_t a_dst = ring + st * C::STAGE_BYTES, b_dst = a_dst + C::A_BYTES;
                    const uint32_t lbar = in_leader_cta(full0 + 8 * st);
                    if (rank == 0) mbar_expect_tx(full0 + 8 * st, tx);
                    tma_load_2d_pair(a_dst, &map_a, lbar, (int32_t)(kb * BK), m0);
                    tma_load_2d_pair(b_dst, mb, lbar, (int32_t)(kb * BK), n0);
                    if (++st == P_STAGES) { st = 0; ph ^= 1; }
                }
            }
        }
        __syncwarp();  // the warp arrives at the CTA-wide barriers below as a whole
    } else if (warp == 1) {
        // ---------------- MMA issuer (leader CTA only): warp-uniform loop, one elected lane issues ----------------
        if (rank == 0) {
            constexpr uint32_t idesc_full = make_idesc_i8(2 * BM, PBN), idesc_half = make_idesc_i8(2 * BM, PBN / 2);
            uint32_t st = 0, ph = 0, as = 0, aph = 0;
            bool ok = true;
            for (uint32_t i = pair; ok && i < num_items; i += num_pairs) {
                const uint32_t idesc = (C::HALVES && i >= n_full) ? idesc_half : idesc_full;
                ok = __all_sync(0xFFFFFFFFu, mbar_wait(tempty0 + 8 * as, aph ^ 1, abort_flag, status, 0x200u | as));
                if (!ok) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + as * 256;
                for (uint32_t kb = 0; kb < num_kb; kb++) {
                    ok = __all_sync(0xFFFFFFFFu, mbar_wait(full0 + 8 * st, ph, abort_flag, status, 0x300u | st));
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t a_src = ring + st * C::STAGE_BYTES, b_src = a_src + C::A_BYTES;
                    const uint64_t a_desc = make_smem_desc(a_src), b_desc = make_smem_desc(b_src);
                    if (elect_one()) {
                        umma_i8_pair(d_tmem, a_desc, b_desc, idesc, kb != 0u);
#pragma unroll
                        for (int k = 1; k < BK / UMMA_K; k++)
                            umma_i8_pair(d_tmem, a_desc + 2u * k, b_desc + 2u * k, idesc, 1u);
                        umma_commit_pair(empty0 + 8 * st, 3);  // both CTAs may refill the stage
                    }
                    __syncwarp();
                    if (++st == P_STAGES) { st = 0; ph ^= 1; }
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
        const uint32_t h = (uint32_t)(warp - 2) >> 2;      // 0: lower column range of the item, 1: upper
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
        for (uint32_t i = pair; i < num_items; i += num_pairs) {
            const PairItem it = pair_item<PBN>(i, n_full, tiles_n);
            const uint32_t m0 = it.tm * (2 * BM) + rank * BM, n0 = it.n0;
            const int width = it.half ? PBN / 2 : PBN;
            const int split = it.half ? PBN / 4 : 128;     // columns [0, split) go to the h = 0 warps, the rest to h = 1
            uint32_t *col = s_col + as * PBN;
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
                const uint32_t taddr = tmem_base + ((q * 32u) << 16) + as * 256;
                const int cb = h ? split : 0, ce = h ? width : split;
                const bool rows_full = m0 + q * 32 + 32 <= M;
                uint32_t rsum = 0;  // sum of this row's uint8 outputs in this warp's part of the item
                // One chunk of 16 accumulator columns.  Blocks of 128 output bytes per row go through the row-coalescing
                // stage when results leave the GPU and the warp's 32 rows and the block's columns are all inside the
                // matrix; everything else is stored directly.
                auto chunk = [&](uint32_t (&v)[16], int cc) {
                    const uint32_t c0 = n0 + cc;
                    const int bc0 = cb + ((cc - cb) / BLOCK_COLS) * BLOCK_COLS;          // first column of cc's block
                    const int bcols = (ce - bc0) < BLOCK_COLS ? (ce - bc0) : BLOCK_COLS;  // its width
                    const bool via_stage = staged && rows_full && n0 + bc0 + bcols <= N;
                    if (via_stage) {
                        uint32_t res[16];
                        epilogue_convert<OUT, 16>(v, rt, col + cc, c, relu, sat, res);
                        PeerStage::put<16>(stage, lane, (cc - bc0) * ESZ / 16, res, 16 * ESZ / 16);
                        if (OUT == 0) rsum += packed_byte_sum<16>(res, 16);
                        const int next = cc + 16;
                        if (next == ce || (next - cb) % BLOCK_COLS == 0)   // the block is complete
                            PeerStage::flush(stage, lane, bcols * ESZ / 16, epi, out,
                                             ((uint64_t)(m0 + q * 32) * ldc + n0 + bc0) * ESZ, ldc * ESZ);
                    } else if (row < M && c0 < N) {
                        rsum += epilogue_chunk<OUT, 16>(v, rt, col + cc, c, relu, sat, epi, out, epilogue_offset(epi, row, c0, ldc),
                                                        vec_ok, (N - c0) < 16u ? (int)(N - c0) : 16);
                    }
                };
                // Two register buffers: the TMEM load of the next chunk is in flight while this one is converted.
                uint32_t va[16], vb[16];
                tmem_ld16(taddr + cb, va);
#pragma unroll 1
                for (int cc = cb; cc < ce; cc += 32) {
                    tmem_ld_wait();
                    if (cc + 16 < ce) tmem_ld16(taddr + cc + 16, vb);
                    chunk(va, cc);
                    if (cc + 16 < ce) {
                        tmem_ld_wait();
                        if (cc + 32 < ce) tmem_ld16(taddr + cc + 32, va);
                        chunk(vb, cc + 16);
                    }
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
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void *p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
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

template <int PBN, int OUT>
cudaError_t launch_pair(const CUtensorMap &ma, const CUtensorMap &mb, const CUtensorMap &mbh, uint32_t n_full, uint64_t M,
                        uint64_t N, uint64_t K, const Epilogue &epi, void *out, uint32_t *status, int sms,
                        cudaStream_t stream)
{
    using C = PCfg<PBN>;
    static bool attr_done[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    // With further destinations (peer GPUs) the epilogue warps get a row-coalescing stage, where it fits beside the ring.
    constexpr int STAGE_BYTES = 8 * PeerStage::BYTES_PER_WARP;
    constexpr bool STAGE_FITS = C::SMEM_BYTES + STAGE_BYTES <= 227 * 1024;
    if (dev >= 0 && dev < 64 && !attr_done[dev]) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_pair_kernel<PBN, OUT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             C::SMEM_BYTES + (STAGE_FITS ? STAGE_BYTES : 0));
        if (e != cudaSuccess) return e;
        attr_done[dev] = true;
    }
    const uint64_t tiles = ((M + 2 * BM - 1) / (2 * BM)) * ((N + PBN - 1) / PBN);
    if (!C::HALVES || n_full > tiles) n_full = (uint32_t)tiles;
    const uint64_t items = n_full + 2 * (tiles - n_full);
    const uint64_t pairs = items < (uint64_t)(sms / 2) ? items : (uint64_t)(sms / 2);
    Epilogue epi_l = epi;
    epi_l.staged = (epi.n_more > 0 && STAGE_FITS) ? 1 : 0;  // (local-only stores gain nothing from the stage: measured)
    const size_t smem = C::SMEM_BYTES + (epi_l.staged ? STAGE_BYTES : 0);
    cudaError_t e = launch_chained(gemm_tc_pair_kernel<PBN, OUT>, dim3((unsigned)(2 * pairs)), dim3(P_THREADS), smem, stream,
                                   ma, mb, mbh, (uint32_t)M, (uint32_t)N, (uint32_t)K, n_full, epi_l, out, status);
    count_launch();
    if (items != tiles)
        note_kernel("gemm_tc_pair_kernel<%d,%s> (%llu tiles + %llu half-width items)", PBN, out_mode_name(OUT),
                    (unsigned long long)n_full, (unsigned long long)(items - n_full));
    else
        note_kernel("gemm_tc_pair_kernel<%d,%s>", PBN, out_mode_name(OUT));
    return e;
}

template <int PBN>
cudaError_t launch_pair_out(const CUtensorMap &ma, const CUtensorMap &mb, const CUtensorMap &mbh, uint32_t n_full,
                            uint64_t M, uint64_t N, uint64_t K, const Epilogue &epi, void *out, uint32_t *status, int sms,
                            cudaStream_t stream)
{
    switch (epi.out_mode) {
        case LTQ_OUT_U8: return launch_pair<PBN, 0>(ma, mb, mbh, n_full, M, N, K, epi, out, status, sms, stream);
        case LTQ_OUT_F32: return launch_pair<PBN, 1>(ma, mb, mbh, n_full, M, N, K, epi, out, status, sms, stream);
        default: return launch_pair<PBN, 2>(ma, mb, mbh, n_full, M, N, K, epi, out, status, sms, stream);
    }
}

}  // namespace

bool tc_pair_preferred(uint64_t M, uint64_t N, int sms)
{
    // Worth pairing once 256 x 256 tiles can occupy most CTA pairs of the device.
    // (with at most 128 rows the second CTA of a pair would have nothing to do)
    const uint64_t tiles = ((M + 2 * BM - 1) / (2 * BM)) * ((N + 255) / 256);
    return M > (uint64_t)BM && tiles * 4 >= (uint64_t)(sms / 2) * 3;
}

bool tail_split_enabled()
{
    static const bool on = getenv("LTQ_NO_TAIL_SPLIT") == nullptr;  // debugging / A-B switch
    return on;
}

PairPlan tc_pair_plan(uint64_t M, uint64_t N, int sms, bool peer_stores, bool chunks_aligned_32)
{
    // Time ~ sum over the rounds of items handed to the CTA pairs of the round's item width.  Wider tiles reuse operands
    // better, so a narrower one must win by a clear margin (3 %).  With 256-wide tiles the remainder behind the last
    // whole round may run as half-width items.
    const uint64_t tm = (M + 2 * BM - 1) / (2 * BM), pairs = (uint64_t)(sms / 2);
    PairPlan best{peer_stores ? 224 : 256, 0xFFFFFFFFu};
    double best_cost = 1e30;
    for (int bn : {256, 240, 224, 192}) {
        if (peer_stores && bn == 256) continue;  // no room for the row-coalescing stage beside a 6 x 32 KB ring
        if (chunks_aligned_32 && bn % 32 != 0) continue;  // column-blocked outputs: chunks must not straddle a block
        const uint64_t tiles = tm * ((N + bn - 1) / bn);
        double cost = (double)((tiles + pairs - 1) / pairs) * bn;
        uint32_t n_full = 0xFFFFFFFFu;
        if (bn == 256 && tail_split_enabled() && tiles > pairs) {
            const uint64_t whole = tiles / pairs, rem = tiles - whole * pairs;
            if (rem != 0 && 2 * rem <= pairs) {  // the remainder fits one round of half tiles
                cost = (double)whole * bn + bn / 2;
                n_full = (uint32_t)(whole * pairs);
            }
        }
        if (cost < best_cost * 0.97) {
            best_cost = cost;
            best = PairPlan{bn, n_full};
        }
    }
    return best;
}

cudaError_t launch_gemm_tc_pair(const TcOperandMap &map_a, const TcOperandMap &map_b, const TcOperandMap *map_b_half,
                                const PairPlan &plan, uint64_t M, uint64_t N, uint64_t K, const Epilogue &epi, void *out,
                                uint32_t *status, int sms, cudaStream_t stream)
{
    const CUtensorMap &ma = *reinterpret_cast<const CUtensorMap *>(map_a.opaque);
    const CUtensorMap &mb = *reinterpret_cast<const CUtensorMap *>(map_b.opaque);
    // without half-width items the third map is never dereferenced; pass the full-width one
    const CUtensorMap &mbh = *reinterpret_cast<const CUtensorMap *>(map_b_half ? map_b_half->opaque : map_b.opaque);
    const uint32_t n_full = map_b_half ? plan.n_full : 0xFFFFFFFFu;
    switch (plan.bn) {
        case 256: return launch_pair_out<256>(ma, mb, mbh, n_full, M, N, K, epi, out, status, sms, stream);
        case 240: return launch_pair_out<240>(ma, mb, mbh, n_full, M, N, K, epi, out, status, sms, stream);
        case 224: return launch_pair_out<224>(ma, mb, mbh, n_full, M, N, K, epi, out, status, sms, stream);
        case 192: return launch_pair_out<192>(ma, mb, mbh, n_full, M, N, K, epi, out, status, sms, stream);
        default: return cudaErrorInvalidValue;
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
