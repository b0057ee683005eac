// Skinny (M <= 16) quantized linear: out[M,N] = epilogue(x[M,K] . W[N,K]^T).  Decode-like shapes are bound by reading
// the weight matrix once from HBM (N*K bytes against M*N*K MACs), so the kernel is a weight-streaming pipeline that
// keeps the SM's instruction issue out of the data path altogether:
//
//  * operands are swapped for the tensor core: the WEIGHT rows are the 128-row (M) operand of tcgen05.mma and the
//    <= 16 activation rows are its 16-column (N) operand, D[weight row, token] accumulating in TMEM.  Such a narrow MMA
//    still costs its issuing thread ~70 cycles, so four warps issue: warp k owns the k-th 32-byte K step of every line
//    and its own 16-column accumulator (the epilogue adds the four up), which keeps a stage's hold time short;
//  * one persistent CTA per SM owns a contiguous band of weight rows (N split evenly in units of 8 rows; a band is one
//    MMA tile of up to 128 rows, of which only the band's rows are loaded - the tile's remaining rows compute on stale
//    shared memory and are never stored);
//  * the producer thread issues TMA tensor copies (cp.async.bulk.tensor.3d, no multicast) into a shared-memory ring.
//    The matrices are described to TMA as {128-byte line, row, line index along K}: a box of R rows x L lines lands as
//    L consecutive K-major tiles [R rows][128 B] under the 128-byte swizzle, exactly the layout the MMA's shared-memory
//    descriptors read, while each row contributes L x 128 contiguous bytes of DRAM per box.  Every ring stage holds a
//    weight box and the matching box of the activation block (rows beyond M are zero-filled by TMA; the activations
//    come out of L2, every CTA reads the same ones).  Nothing but the ring lives in shared memory: one CTA per SM with
//    4-6 stages of 30-45 KB.  (A ring of half an SM, so that the next launch's CTA fits beside this one, was measured
//    too: its hand-over is smoother but its stream is slower, 10.5 against 9.3 us on 45 MB of weights);
//  * four epilogue warps read the accumulators with tcgen05.ld (thread = weight row, register = token), apply the fused
//    epilogue (l-ten/math_fns.cpp:1469-1474) and store; for every token the 32 lanes of a warp write 32 consecutive
//    outputs.  Accumulators are double buffered in TMEM.
//
//  * with `early_weights` the kernel is launched as a programmatic dependent of the kernel before it in the stream.
//    Every CTA releases its dependents at once, so the next launch's CTAs are scheduled the moment an SM's shared
//    memory frees up, and fill their rings with WEIGHTS straight away (the caller guarantees that nothing in flight
//    writes them) and ask the boxes behind the ring into L2.  Everything that can depend on the previous kernel - the
//    activation boxes, the activation row sums, every store - comes after griddepcontrol.wait.  In a chain of such
//    launches the start-up (barrier set-up, first DRAM round trip) of one launch overlaps the tail (last MMAs,
//    epilogue, stragglers) of the one before.
//
// Every mbarrier wait is bounded (2 s by %globaltimer); on expiry a code is left in the device status word.
#include <cuda.h>

#include <type_traits>

#include "ltq_common.cuh"
#include "ltq_gemv.cuh"
#include "ltq_tcgen05.cuh"

namespace ltq {

namespace {

constexpr int THREADS = 288;               // warp 0 producer, warps 1,6,7,8 MMA issuers, warps 2..5 epilogue
constexpr int LINE = 128;                  // bytes of K per line (one swizzle atom wide)
constexpr int XROWS = 16;                  // activation rows as seen by the MMA (N = 16), TMEM columns per accumulator
constexpr int TILE_M = 128;                // MMA M: weight rows per tile (upper bound)
constexpr int MAX_STAGES = 16;
constexpr int SMEM_FULL = 220 * 1024;      // one CTA per SM with as deep a ring as fits
constexpr int OVERREAD = TILE_M * LINE;    // an MMA reads 128 rows from a tile's start whatever the band holds
constexpr int NACC = 4;                    // independent partial accumulators per tile (summed in the epilogue)
constexpr uint32_t TMEM_COLS = 2 * NACC * XROWS;  // two buffers of NACC accumulators of 16 columns = 128
constexpr uint32_t PREFETCH_AHEAD = 6;     // boxes requested into L2 beyond the ring (~170-240 KB per CTA, 25-35 MB per
                                           // GPU; 2-3 times as much already costs 10-20 % of the streaming rate)
constexpr uint64_t BIG_WEIGHTS = 128ull << 20;  // weight bytes from which a launch is mostly steady-state streaming
constexpr uint32_t BOX_SMALL_W = 40 * 1024;     // target bytes of a weight box below / from BIG_WEIGHTS
constexpr uint32_t BOX_BIG_W = 32 * 1024;

struct Plan {
    uint32_t grid, tiles_per_cta, tiles;   // tiles = grid * tiles_per_cta
    uint32_t oct_lo, oct_hi;               // a tile holds oct_lo or oct_hi groups of 8 rows (oct_hi <= 16)
    uint32_t lines;                        // lines per stage (per TMA box)
    uint32_t stages;
    uint32_t prefetch;                     // boxes requested into L2 beyond the ring
    uint32_t w_stage, x_stage;             // bytes per stage: lines * oct_hi * 8 * 128 and lines * (8 or 16) * 128
    uint32_t slack;                        // bytes kept free behind the activation boxes for the MMA's over-reads
    size_t smem;
    bool ok;
};

Plan make_plan(uint64_t M, uint64_t N, uint64_t K, int sms, size_t smem_limit)
{
    Plan p{};
    const uint64_t octs = (N + 7) / 8;
    p.grid = (uint32_t)(octs < (uint64_t)sms ? octs : (uint64_t)sms);
    p.tiles_per_cta = (uint32_t)((octs + (uint64_t)p.grid * 16 - 1) / ((uint64_t)p.grid * 16));
    p.tiles = p.grid * p.tiles_per_cta;
    p.oct_lo = (uint32_t)(octs / p.tiles);
    p.oct_hi = (uint32_t)((octs + p.tiles - 1) / p.tiles);
    const uint32_t klines = (uint32_t)(K / LINE);
    const uint32_t line_bytes = p.oct_hi * 8 * LINE;
    // Box size, measured on B200 (M = 16, fp32 out, chained launches over distinct weights): every row should give
    // DRAM at least 256 contiguous bytes per box (128-byte pieces at a pitch of K stream at ~5 TB/s, 256 and more at
    // ~6 TB/s), and a weight matrix of a few tens of MB, whose launch is mostly start-up and hand-over, does best with
    // boxes of ~40 KB, while a large one prefers ~30 KB and the deeper ring that leaves room for.
    const uint32_t box_target = N * K < BIG_WEIGHTS ? BOX_SMALL_W : BOX_BIG_W;
    uint32_t L = box_target / line_bytes;
    L = L < 1 ? 1 : (L > 4 ? 4 : L);
    if (L > klines) L = klines;
    p.lines = L;
    p.w_stage = L * line_bytes;
    p.prefetch = PREFETCH_AHEAD;
    // Activation boxes hold 8 rows per line when M <= 8 (the MMA still reads 16 rows per line tile; rows 8..15 are then
    // the next line's rows, whose products land in TMEM columns that are never stored).
    p.x_stage = L * (uint32_t)(M > 8 ? 16 : 8) * LINE;
    p.ok = p.oct_hi <= 16 && p.oct_lo >= 1;
    if (!p.ok) return p;
    // Layout: [W boxes of all stages][x boxes of all stages][slack][barriers].  The MMA reads 128 rows from the start of
    // every weight line tile, so up to OVERREAD bytes behind the last weight box are read (never used), and 1 KB behind
    // the last activation box when those hold 8 rows.
    for (uint32_t st = MAX_STAGES; st >= 2; st--) {
        const size_t after = (size_t)st * p.x_stage;
        const size_t slack = (after >= (size_t)OVERREAD ? 0 : (size_t)OVERREAD - after) + 1024;
        const size_t total = 1024 + (size_t)st * (p.w_stage + p.x_stage) + slack + 512;
        if (total <= smem_limit) {
            p.stages = st;
            p.slack = (uint32_t)slack;
            p.smem = total;
            return p;
        }
    }
    p.ok = false;
    return p;
}

// Band geometry of the launch that follows (GemvNext), as the kernel needs it to name that launch's first boxes.
struct NextBand {
    uint32_t boxes;  // 0: no hint
    uint32_t tiles_per_cta, tiles, octs, oct_lo, lines, chunks;
};

}  // namespace

// OUT: 0 = uint8, 1 = float, 2 = int32 (ltq_out_mode).
template <int OUT>
__global__ void __launch_bounds__(THREADS, 2)
gemv_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w_lo,
            const __grid_constant__ CUtensorMap map_w_hi, uint32_t M, uint32_t N, uint32_t K, uint32_t tiles_per_cta,
            uint32_t tiles, uint32_t oct_lo, uint32_t lines, uint32_t stages, uint32_t prefetch, uint32_t w_stage,
            uint32_t x_stage, uint32_t slack, Epilogue epi, void *__restrict__ out, uint32_t *status,
            const __grid_constant__ CUtensorMap map_n_lo, const __grid_constant__ CUtensorMap map_n_hi, NextBand nx)
{
    // By every thread, first thing: the CTA counts as released once all of them have said so, and the next launch's CTAs
    // should move in (and start fetching their weights) as early as they can.
    griddep_launch_dependents();
    if (threadIdx.x == 0) {  // the first tensor copy waits for its descriptor: have all three on their way at once
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w_hi) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w_lo) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
    }
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw0 = smem_u32(smem_raw);
    const uint32_t ring = (raw0 + 1023u) & ~1023u;                       // [stages][lines][rows][128 B]
    const uint32_t xs = ring + stages * w_stage;                         // [stages][lines][8 or 16][128 B]
    const uint32_t xrows = x_stage / (lines * LINE);                             // rows per line tile of an activation box
    uint8_t *after = smem_raw + (xs - raw0) + stages * x_stage + slack;
    uint64_t *bars = reinterpret_cast<uint64_t *>(after);                // full[S] empty[S] tfull[2] tempty[2]
    uint32_t *misc = reinterpret_cast<uint32_t *>(bars + 2 * MAX_STAGES + 4);  // [0] tmem base, [1] abort flag
    volatile uint32_t *abort_flag = misc + 1;

    const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8 * MAX_STAGES;
    const uint32_t tfull0 = empty0 + 8 * MAX_STAGES, tempty0 = tfull0 + 16;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t octs = (N + 7) / 8;
    const uint32_t klines = K / LINE, chunks = (klines + lines - 1) / lines;
    const uint32_t t_begin = blockIdx.x * tiles_per_cta, t_end = t_begin + tiles_per_cta;
    const uint32_t x_bytes = lines * xrows * LINE;

    const uint64_t w_policy = l2_policy_evict_first();  // weights are read once per launch
    // Producer state lives in thread 0.  A cursor names a box: (tile, K chunk), the tile's first row, row count and
    // tensor map, and the ring slot with its phase.
    struct Cursor {
        uint32_t t, kc, st, ph, row0, rows;
        const CUtensorMap *map;
    };
    auto enter_tile = [&](Cursor &c) {
        const uint32_t o0 = (uint32_t)(((uint64_t)c.t * octs) / tiles), o1 = (uint32_t)(((uint64_t)(c.t + 1) * octs) / tiles);
        c.row0 = o0 * 8;
        c.rows = (o1 - o0) * 8;
        c.map = (o1 - o0) == oct_lo ? &map_w_lo : &map_w_hi;
    };
    auto advance = [&](Cursor &c) {
        if (++c.st == stages) { c.st = 0; c.ph ^= 1; }
        if (++c.kc == chunks) {
            c.kc = 0;
            if (++c.t < t_end) enter_tile(c);
        }
    };
    // Weight box of cursor c.  A box always transfers its full size: lines or rows outside the matrix arrive as zeros.
    // `with_x`: the activation box goes out with it and the pair makes the stage's one arrival; otherwise only the byte
    // count is announced and the arrival comes later with the activation box.
    auto issue_w = [&](const Cursor &c, bool with_x) {
        const uint32_t w_bytes = lines * c.rows * LINE;
        if (with_x) mbar_expect_tx(full0 + 8 * c.st, w_bytes + x_bytes);
        else mbar_expect_tx_only(full0 + 8 * c.st, w_bytes);
        tma_load_3d_hint(ring + c.st * w_stage, c.map, full0 + 8 * c.st, 0, (int32_t)c.row0, (int32_t)(c.kc * lines), w_policy);
    };
    auto issue_x = [&](const Cursor &c, bool arrive) {
        if (arrive) mbar_expect_tx(full0 + 8 * c.st, x_bytes);
        tma_load_3d(xs + c.st * x_stage, &map_x, full0 + 8 * c.st, 0, 0, (int32_t)(c.kc * lines));
    };
    Cursor cur{t_begin, 0, 0, 0, 0, 0, nullptr};  // next box to load into the ring
    Cursor pf = cur;                              // next box to ask into L2; runs up to PREFETCH_AHEAD boxes in front

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < stages; s++) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, NACC);  // one commit per MMA-issuing warp
        }
        for (int s = 0; s < 2; s++) {
            mbar_init(tfull0 + 8 * s, NACC);  // one commit per MMA-issuing warp
            mbar_init(tempty0 + 8 * s, 4);    // one arrival per epilogue warp
        }
        misc[1] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        // Fill the ring with weights before anything else happens in the CTA: the first bytes from HBM are more than a
        // microsecond away.  Weights do not depend on the previous kernel, so this runs ahead of the grid dependency.
        enter_tile(cur);
        pf = cur;
        uint32_t primed = 0;
        for (; primed < stages && pf.t < t_end; primed++) {
            issue_w(pf, false);
            advance(pf);
        }
        // The ring is all this CTA can hold while it waits for its turn, a fraction of its weights.  The boxes behind it
        // are requested into L2, so that HBM keeps streaming through the hand-over between two launches (the wait for
        // the previous kernel, the first activation fetch, the previous kernel's last MMAs and epilogue) and the ring
        // later refills from L2.
        for (uint32_t i = 0; i < prefetch && pf.t < t_end; i++) {
            tma_prefetch_3d(pf.map, 0, (int32_t)pf.row0, (int32_t)(pf.kc * lines));
            advance(pf);
        }
        // The activations may have been written by the previous kernel.
        griddep_wait();
        for (uint32_t i = 0; i < primed; i++) {
            issue_x(cur, true);
            advance(cur);
        }
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(misc), TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = misc[0];

    if (warp == 0) {
        // ---------------- TMA producer (continues where the pre-fill stopped) ----------------
        if (lane == 0) {
            while (cur.t < t_end) {
                if (!mbar_wait(empty0 + 8 * cur.st, cur.ph ^ 1, abort_flag, status, 0x500u | cur.st)) break;
                issue_w(cur, true);
                issue_x(cur, false);
                advance(cur);
                if (pf.t < t_end) {
                    tma_prefetch_3d(pf.map, 0, (int32_t)pf.row0, (int32_t)(pf.kc * lines));
                    advance(pf);
                }
            }
            // Everything this launch reads is on its way.  The CTA that takes this CTA's place in the next launch will
            // want the first boxes of the same band of the next weight matrix: ask them into L2 now, behind this
            // launch's own requests, so that they arrive while this CTA is busy with its last MMAs and its epilogue.
            if (nx.boxes && !*abort_flag) {
                uint32_t t = blockIdx.x * nx.tiles_per_cta, kc = 0;
                const uint32_t t_last = t + nx.tiles_per_cta;
                for (uint32_t i = 0; i < nx.boxes && t < t_last; i++) {
                    const uint32_t o0 = (uint32_t)(((uint64_t)t * nx.octs) / nx.tiles);
                    const uint32_t o1 = (uint32_t)(((uint64_t)(t + 1) * nx.octs) / nx.tiles);
                    tma_prefetch_3d((o1 - o0) == nx.oct_lo ? &map_n_lo : &map_n_hi, 0, (int32_t)(o0 * 8), (int32_t)(kc * nx.lines));
                    if (++kc == nx.chunks) { kc = 0; t++; }
                }
            }
        }
        __syncwarp();  // the warp arrives at the CTA-wide barriers below as a whole
    } else if (warp == 1 || warp >= 6) {
        // ---------------- MMA issuers (warps 1, 6, 7, 8): warp-uniform loops, one elected lane issues ----------------
        // Issuer k handles K step k (bytes [32k, 32k + 32) of every 128-byte line) into accumulator k.
        constexpr uint32_t idesc = make_idesc_i8(TILE_M, XROWS);
        const uint32_t kstep = warp == 1 ? 0u : (uint32_t)(warp - 5);
        uint32_t st = 0, ph = 0, as = 0, aph = 0;
        bool ok = true;
        for (uint32_t t = t_begin; ok && t < t_end; t++) {
            const uint32_t o0 = (uint32_t)(((uint64_t)t * octs) / tiles), o1 = (uint32_t)(((uint64_t)(t + 1) * octs) / tiles);
            const uint32_t line_stride = (o1 - o0) * 8 * LINE;  // bytes between the K-major tiles of one box
            ok = __all_sync(0xFFFFFFFFu, mbar_wait(tempty0 + 8 * as, aph ^ 1, abort_flag, status, 0x200u | as));
            if (!ok) break;
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + as * (NACC * XROWS) + kstep * XROWS;
            for (uint32_t kc = 0; kc < chunks; kc++) {
                ok = __all_sync(0xFFFFFFFFu, mbar_wait(full0 + 8 * st, ph, abort_flag, status, 0x300u | st));
                if (!ok) break;
                tc_fence_after();
                const uint32_t l0 = kc * lines, nl = (klines - l0) < lines ? (klines - l0) : lines;
                const uint64_t a_desc = make_smem_desc(ring + st * w_stage) + 2u * kstep;
                const uint64_t b_desc = make_smem_desc(xs + st * x_stage) + 2u * kstep;
                if (elect_one()) {
                    for (uint32_t l = 0; l < nl; l++)  // the first line of a tile overwrites, later lines accumulate
                        umma_i8(d_tmem, a_desc + (uint64_t)((l * line_stride) >> 4), b_desc + (uint64_t)((l * xrows * LINE) >> 4),
                                idesc, (l0 + l) >= 1u);
                    umma_commit(empty0 + 8 * st);
                }
                __syncwarp();
                if (++st == stages) { st = 0; ph ^= 1; }
            }
            if (!ok) break;
            if (elect_one()) umma_commit(tfull0 + 8 * as);
            __syncwarp();
            if (++as == 2) { as = 0; aph ^= 1; }
        }
    } else {
        // ---------------- epilogue (warps 2..5): thread = weight row, register = token ----------------
        const uint32_t q = (uint32_t)warp & 3u;
        griddep_wait();  // the activation row sums (and device-side qparams) come from the previous kernel
        if (blockIdx.x == 0 && epi.clear_ptr)  // chain housekeeping, see Epilogue::clear_ptr (128 epilogue threads)
            for (uint32_t i = threadIdx.x - 64; i < epi.clear_count; i += 128) epi.clear_ptr[i] = 0;
        const EpilogueConsts c = epilogue_consts(epi);
        const bool relu = epi.flags & LTQ_FLAG_RELU, sat = epi.flags & LTQ_FLAG_SATURATE;
        using OutT = typename std::conditional<OUT == 0, uint8_t, typename std::conditional<OUT == 1, float, int32_t>::type>::type;
        OutT *o = static_cast<OutT *>(out);
        const uint64_t ldc = epilogue_pitch(epi, N);
        uint32_t rt[XROWS];  // per-token part of the correction; identical for every weight row
#pragma unroll
        for (int m = 0; m < XROWS; m++) rt[m] = (uint32_t)m < M ? epilogue_row_term(epi, c, (uint32_t)m) : 0u;
        uint32_t as = 0, aph = 0;
        bool ok = true;
        for (uint32_t t = t_begin; t < t_end; t++) {
            const uint32_t o0 = (uint32_t)(((uint64_t)t * octs) / tiles), o1 = (uint32_t)(((uint64_t)(t + 1) * octs) / tiles);
            const uint32_t n = o0 * 8 + q * 32 + lane;
            const bool valid = (q * 32 + lane) < (o1 - o0) * 8 && n < N;
            // fetched before waiting, so the global-memory latency passes under the stream
            const uint32_t ct = valid ? epilogue_col_term(epi, c, n) : 0u;
            if (ok) ok = mbar_wait(tfull0 + 8 * as, aph, abort_flag, status, 0x400u | as);
            if (ok) {
                tc_fence_after();
                uint32_t v[XROWS];
                const uint32_t tacc = tmem_base + ((q * 32u) << 16) + as * (NACC * XROWS);
                uint32_t w1[XROWS], w2[XROWS], w3[XROWS];
                static_assert(NACC == 4, "the epilogue adds four accumulators");
                tmem_ld16(tacc, v);
                tmem_ld16(tacc + XROWS, w1);
                tmem_ld16(tacc + 2 * XROWS, w2);
                tmem_ld16(tacc + 3 * XROWS, w3);
                tmem_ld_wait();
#pragma unroll
                for (int m = 0; m < XROWS; m++) v[m] += w1[m] + w2[m] + w3[m];
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(tempty0 + 8 * as);  // accumulator buffer may be overwritten
                const bool plain = epi.n_more == 0 && epi.col_block == 0 && !(OUT == 0 && epi.out_rowsum);
                if (plain) {
                    // one dense destination: the common case, kept free of the general path's loops
                    if (valid) {
#pragma unroll
                        for (int m = 0; m < XROWS; m++) {
                            if ((uint32_t)m < M) {
                                const int32_t a = epilogue_acc(v[m], rt[m], ct, relu);
                                OutT r;
                                if (OUT == 0) r = (OutT)epilogue_u8(a, c, sat);
                                else if (OUT == 1) r = (OutT)epilogue_f32(a, c);
                                else r = (OutT)a;
                                o[(size_t)m * ldc + n] = r;
                            }
                        }
                    }
                } else {
                    // several destinations, column-blocked output, row sums (warp-wide reductions: all lanes run the loop)
#pragma unroll
                    for (int m = 0; m < XROWS; m++) {
                        if ((uint32_t)m < M) {
                            const int32_t a = epilogue_acc(v[m], rt[m], ct, relu);
                            OutT r;
                            if (OUT == 0) r = (OutT)epilogue_u8(a, c, sat);
                            else if (OUT == 1) r = (OutT)epilogue_f32(a, c);
                            else r = (OutT)a;
                            if (valid)
                                for (int d = -1; d < epi.n_more; d++)
                                    (d < 0 ? o : static_cast<OutT *>(epi.more_out[d]))[epilogue_offset(epi, (uint64_t)m, n, ldc)] = r;
                            if (OUT == 0 && epi.out_rowsum) {  // token m: this warp's 32 outputs add up first
                                const uint32_t t32 = __reduce_add_sync(0xFFFFFFFFu, valid ? (uint32_t)r : 0u);
                                if (lane == 0 && t32) atomicAdd(&epi.out_rowsum[m], (int32_t)t32);
                            }
                        }
                    }
                }
            }
            if (++as == 2) { as = 0; aph ^= 1; }
        }
    }

    // Teardown: nobody leaves before every role is done with TMEM and shared memory.
    tc_fence_before();
    __syncthreads();
    if (warp == 0 && lane == 0 && *abort_flag) {
        // After a timeout, copies issued by the producer may still be landing in this CTA's shared memory; they
        // complete within microseconds, so hold the CTA for a bounded 2 ms before it exits.
        const uint64_t t0 = global_ns();
        while (global_ns() - t0 < 2000000ull) __nanosleep(1000);
    }
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

namespace {

template <int OUT>
cudaError_t launch_t(const TcOperandMap &mx, const TcOperandMap &lo, const TcOperandMap &hi, const Plan &p, uint64_t M,
                     uint64_t N, uint64_t K, const Epilogue &epi, void *out, uint32_t *status, cudaStream_t stream,
                     bool early_weights, const TcOperandMap &nlo, const TcOperandMap &nhi, const NextBand &nx)
{
    // The opt-in shared-memory size is set once per device: the kernel runs for a few microseconds and a runtime
    // attribute call per launch would cost as much as the launch.
    static bool attr_done[64] = {false};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (!attr_done[dev]) {
        e = cudaFuncSetAttribute(gemv_kernel<OUT>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_FULL);
        if (e != cudaSuccess) return e;
        // Ask for the largest shared-memory configuration of the SM whatever this launch needs (see below).
        e = cudaFuncSetAttribute(gemv_kernel<OUT>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        if (e != cudaSuccess) return e;
        attr_done[dev] = true;
    }
    // An SM is configured with the smallest shared-memory size (... 164, 196, 228 KB) that holds the CTAs running on it,
    // and CTAs of other kernels only fit into what that size leaves.  A ring of 4 x 48 KB (M > 8) ends 0.5 KB under the
    // 196 KB step: small kernels launched beside this one (the activation quantise of the next batch, which would
    // otherwise run early next to this kernel's CTAs) then find no SM to go to, pile up on the first SMs that become
    // free and keep this kernel's next launch off them (measured: 14.7 us per step instead of 9.3 at M = 16).  A request
    // just over the step selects the 228 KB configuration, which leaves room beside the ring.
    constexpr size_t STEP_196K = 196 * 1024 - 1024;   // largest request that still fits the 196 KB configuration
    size_t smem = p.smem;
    if (smem > STEP_196K - 8 * 1024 && smem <= STEP_196K) smem = STEP_196K + 16;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.grid);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = early_weights ? 1 : 0;
    e = cudaLaunchKernelEx(&cfg, gemv_kernel<OUT>, *reinterpret_cast<const CUtensorMap *>(mx.opaque),
                           *reinterpret_cast<const CUtensorMap *>(lo.opaque), *reinterpret_cast<const CUtensorMap *>(hi.opaque),
                           (uint32_t)M, (uint32_t)N, (uint32_t)K, p.tiles_per_cta, p.tiles, p.oct_lo, p.lines, p.stages,
                           p.prefetch, p.w_stage, p.x_stage, p.slack, epi, out, status,
                           *reinterpret_cast<const CUtensorMap *>(nlo.opaque), *reinterpret_cast<const CUtensorMap *>(nhi.opaque), nx);
    count_launch();
    note_kernel("gemv_kernel<%s>", out_mode_name(OUT));
    return e;
}

}  // namespace

bool gemv_shape_ok(uint64_t M, uint64_t N, uint64_t K, const void *x, const void *W, int sms)
{
    return M >= 1 && M <= 16 && N >= 1 && N < (1ull << 31) && K >= 128 && K % 128 == 0 && K < (1ull << 31) &&
           (((uintptr_t)x & 15) == 0) && (((uintptr_t)W & 15) == 0) && make_plan(M, N, K, sms, SMEM_FULL).ok;
}

cudaError_t launch_gemv(const uint8_t *x, const uint8_t *W, uint64_t M, uint64_t N, uint64_t K, const Epilogue &epi,
                        void *out, uint32_t *status, int sms, cudaStream_t stream, GemvWeightMaps *cache, bool early_weights,
                        const GemvNext *next)
{
    const Plan p = make_plan(M, N, K, sms, SMEM_FULL);
    if (!p.ok) return cudaErrorInvalidConfiguration;
    TcOperandMap mx;
    GemvWeightMaps local;
    // activations: a box is [lines][8 or 16 rows][128 B]; rows >= M are out of bounds -> zeros
    if (tc_make_map_lines(&mx, x, M, K, (int)(p.x_stage / (p.lines * LINE)), (int)p.lines) != 0) return cudaErrorInvalidValue;
    GemvWeightMaps *wm = cache ? cache : &local;
    if (!wm->lo.matches(W, N, K, (int)p.oct_lo * 8, (int)p.lines)) {
        if (tc_make_map_lines(&wm->lo, W, N, K, (int)p.oct_lo * 8, (int)p.lines) != 0) return cudaErrorInvalidValue;
    }
    if (!wm->hi.matches(W, N, K, (int)p.oct_hi * 8, (int)p.lines)) {
        if (tc_make_map_lines(&wm->hi, W, N, K, (int)p.oct_hi * 8, (int)p.lines) != 0) return cudaErrorInvalidValue;
    }
    // The launch behind this one (a hint): its plan must put the same band on the same CTA index for the boxes asked into
    // L2 to be the ones that CTA's successor reads first.  Without a usable hint the kernel gets this launch's own maps
    // (never dereferenced: boxes = 0).
    NextBand nx{};
    const TcOperandMap *nlo = &wm->lo, *nhi = &wm->hi;
    GemvWeightMaps next_local;
    if (next && next->W && next->boxes && (((uintptr_t)next->W & 15) == 0) && next->K >= 128 && next->K % 128 == 0 &&
        next->N >= 1 && next->N < (1ull << 31) && next->K < (1ull << 31)) {
        const Plan q = make_plan(M, next->N, next->K, sms, SMEM_FULL);
        if (q.ok && q.grid == p.grid) {
            GemvWeightMaps *nm = next->cache ? next->cache : &next_local;
            bool ok = true;
            if (!nm->lo.matches(next->W, next->N, next->K, (int)q.oct_lo * 8, (int)q.lines))
                ok = tc_make_map_lines(&nm->lo, next->W, next->N, next->K, (int)q.oct_lo * 8, (int)q.lines) == 0;
            if (ok && !nm->hi.matches(next->W, next->N, next->K, (int)q.oct_hi * 8, (int)q.lines))
                ok = tc_make_map_lines(&nm->hi, next->W, next->N, next->K, (int)q.oct_hi * 8, (int)q.lines) == 0;
            if (ok) {
                const uint32_t klines = (uint32_t)(next->K / LINE);
                nx = NextBand{next->boxes, q.tiles_per_cta, q.tiles, (uint32_t)((next->N + 7) / 8), q.oct_lo, q.lines,
                              (klines + q.lines - 1) / q.lines};
                nlo = &nm->lo;
                nhi = &nm->hi;
            }
        }
    }
    switch (epi.out_mode) {
        case LTQ_OUT_U8: return launch_t<0>(mx, wm->lo, wm->hi, p, M, N, K, epi, out, status, stream, early_weights, *nlo, *nhi, nx);
        case LTQ_OUT_F32: return launch_t<1>(mx, wm->lo, wm->hi, p, M, N, K, epi, out, status, stream, early_weights, *nlo, *nhi, nx);
        default: return launch_t<2>(mx, wm->lo, wm->hi, p, M, N, K, epi, out, status, stream, early_weights, *nlo, *nhi, nx);
    }
}

}  // namespace ltq
