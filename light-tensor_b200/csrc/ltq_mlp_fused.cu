// A short chain of quantized linear layers in ONE launch per batch: the launch-latency-bound case of the path, a small
// MLP run batch after batch (the reference's QNet loop, tests/nn_tests.cpp:630-640 and 930-963: quantise the input, then
// FullyConnected_q after FullyConnected_q, each a kernel launch and a round trip of the activations through memory).
//
// One cluster of 8 CTAs handles 16, 32 or 64 rows of the batch (few rows per cluster while the batch is small: every
// hand-over moves rows x features bytes into every CTA) and keeps everything on chip between the layers:
//
//  * every CTA holds, for every layer, a slice of n weight rows (output features; N / 8 rounded up to 16), loaded once
//    at the start by TMA into 128-byte-swizzled K-major tiles - the weights are a layer's static data and are fetched
//    before the programmatic-launch dependency on the previous kernel is waited for;
//  * the CTAs quantise the fp32 input together: CTA c takes the 128-column slab c of all rows (the reference's Quantize
//    arithmetic, every load issued before the arithmetic starts) into its own copy of the input tile;
//  * per layer, one warp issues tcgen05.mma (128 x n x 32, uint8 x uint8 -> int32 in TMEM; rows beyond the cluster's own
//    are whatever lies behind the tile and their results are never read), four warps run the fused epilogue of l-ten's
//    quantized_matmul (l-ten/math_fns.cpp:1433-1474) and write the uint8 result slice into their own copy of the next
//    layer's activation tile; the last layer's result goes to global memory;
//  * hand-over: what a CTA produced for the next tile is one contiguous piece (a K slab of the input tile; n / 16 chunks
//    of a tile between layers, which are unswizzled - core matrices of 8 rows x 16 bytes - so that any slice of features
//    is contiguous).  The CTA sends that piece, and the partial row sums of its bytes that the next layer's zero-point
//    correction needs, to each of the other seven with bulk copies through distributed shared memory (cp.async.bulk
//    shared::cta -> shared::cluster), which count their bytes on the receiver's mbarrier: data and "it is there" arrive
//    together, no cluster-scope fence, no remote arrival.  Nothing waits on anything outside its own cluster, every
//    wait is bounded, and no CTA leaves before every CTA has received what was sent to it.
//
// Integer sums are exact whatever the order, so the result equals the layer-by-layer path bit for bit.
//
// Measured on the 784-512-512-10 network, batch 64 (B200, a CUDA graph of back-to-back launches), per batch, against
// 15.1-16.7 us layer by layer (4 launches):
//   13.5 us  first form: 64 rows per cluster, rows of the input split over the CTAs, results written into all 8 CTAs with
//            16-byte remote stores, then fence.acq_rel.cluster (~1 us per hand-over) and one remote arrival per warp
//            (one per thread: 4-5 us per hand-over);
//   11.3 us  bulk copies instead (no fence, no arrivals), input loads issued ahead of the arithmetic, the cluster barrier
//            at the end split around the last layer;
//    9.3-9.5 us  16 rows per cluster (4 clusters), input split by K slab instead of by row (one piece per CTA: with a piece
//            per slab and row group the 56 copies queued for 1.4 us on the SM's copy unit, ~40 ns per copy).
// What is left is a chain of latencies (after the grid dependency resolves: ~2.2 us until the first MMA, per hidden
// layer 0.6-0.9 us of MMAs + ~0.9 us epilogue + ~0.5 us to issue the copies + ~0.3 us until they have landed, ~1 us from the
// last store to the next launch's start).  Two further steps were built, measured on the same box and left out, because
// neither changed the time: bytes and sums of a hand-over in ONE copy (7 copies instead of 14 per hand-over), and a
// conversion-free uint8 epilogue (integer / float bit tricks in place of the two conversion instructions per element).
// A variant with clusters of 4, the weights streamed through a ring, was built and measured at 18.3 us: with both
// operands 128 rows tall in one SM's shared memory its MMAs take 140 cycles instead of 70.  Dealing the four 32-byte K
// steps of every slab over four accumulators (added up in the epilogue) to break the chain of dependent MMAs was also
// built and measured, bit-exact and slower (10.2 us against 9.3 us on the same box): MMAs issued by one thread do not
// overlap better for having different accumulators, and the epilogue reads four times the TMEM columns.
#include <cuda.h>

#include <new>
#include <type_traits>

#include "ltq_common.cuh"
#include "ltq_gemm_tc.cuh"
#include "ltq_layer.cuh"
#include "ltq_quant.cuh"
#include "ltq_tcgen05.cuh"

namespace ltq {
namespace {

constexpr int CL = 8;               // CTAs per cluster
constexpr int ROWS = 64;            // batch rows per cluster, at most (the layout is planned for this many)
constexpr int MAX_LAYERS = 4;
constexpr int THREADS = 256;        // warps 0,1,4,5: epilogue (TMEM lanes 0..63); 2: MMA issuer; 3: weight loads; all: input quantise
constexpr int SLAB = ROWS * 128;    // one 128-byte-wide K slab of an activation tile
constexpr int SMEM_LIMIT = 224 * 1024;

struct MlpLayer {
    uint32_t K, N, n;               // input features, output features, columns per CTA (multiple of 16)
    uint32_t slabs;                 // ceil(K / 128)
    uint32_t w_off, col_off;        // byte offsets of this CTA's weight slice / column terms in shared memory
    const int32_t *wsum, *bias;
    float sA, sB, sC;
    int32_t zA, zB, zC;
    unsigned flags;                 // LTQ_FLAG_RELU | LTQ_FLAG_SATURATE
};

struct MlpParams {
    int n_layers;
    MlpLayer L[MAX_LAYERS];
    uint32_t act_off[2];            // the two activation tiles (layer l reads act[l % 2], writes act[(l + 1) % 2])
    uint32_t asum_off;              // int32 [2][CL * 2][ROWS]: partial row sums per source CTA and column half
    uint32_t bar_off;               // mbarriers: w_full[4], act_ready[4], acc_full[4]
    uint32_t tmem_cols;
    uint32_t smem_bytes;
    int out_mode;                   // of the last layer
    uint32_t rows;                  // batch rows per cluster (16, 32 or ROWS), chosen per call
};

__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t cta)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(cta));
    return r;
}
// Bulk copy from this CTA's shared memory into another CTA's (both 16-byte aligned, a multiple of 16 bytes); the bytes
// are counted on that CTA's mbarrier, so data and "it has arrived" travel together: no fence, no separate arrival.
__device__ __forceinline__ void bulk_copy_to_cta(uint32_t dst_cluster, uint32_t src_local, uint32_t bytes, uint32_t bar_cluster)
{
    asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst_cluster), "r"(src_local), "r"(bytes), "r"(bar_cluster)
                 : "memory");
}
// The two halves of the cluster-wide barrier (every thread of every CTA arrives once, then waits once).
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire;" ::: "memory"); }
// Barrier among the four epilogue warps only (the MMA and weight warps do not take part).
__device__ __forceinline__ void epilogue_warps_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
__device__ __forceinline__ bool try_wait_cluster(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded like mbar_wait, acquiring at cluster scope (the arrivals come from other CTAs).
__device__ __forceinline__ bool wait_cluster(uint32_t bar, volatile uint32_t *abort_flag, uint32_t *status, uint32_t code)
{
    uint64_t t0 = 0;
    for (uint32_t spin = 1;; spin++) {
        if (try_wait_cluster(bar, 0)) return true;
        if ((spin & 1023u) == 0) {
            if (*abort_flag) return false;
            const uint64_t now = global_ns();
            if (t0 == 0) {
                t0 = now;
            } else if (now - t0 > WAIT_LIMIT_NS) {
                *abort_flag = 1;
                atomicCAS(status, 0u, code);
                return false;
            }
        }
    }
}

// Byte offset of element (row, k) inside the FIRST activation tile (the quantised input): 128-byte-wide K slabs of R
// rows, 16-byte pieces XORed with the row's low three bits (the 128-byte swizzle of the MMA descriptor).  A slab is one
// contiguous piece of R x 128 bytes: CTA c quantises slab c (c + 8, ...) of all rows and sends it as one bulk copy.
// (Rows per CTA, a piece per slab, was measured first: 49 + 7 copies queue for 1.4 us on the SM's one copy unit.)
__device__ __forceinline__ uint32_t act_offset(uint32_t row, uint32_t k, uint32_t R)
{
    return (k >> 7) * (R * 128) + row * 128 + ((((k >> 4) & 7u) ^ (row & 7u)) << 4) + (k & 15u);
}
// ... and inside the tiles BETWEEN layers: no swizzle, [K / 16][R rows][16 bytes] (core matrices of 8 rows x 16 bytes,
// 128 bytes apart along the rows, R * 16 bytes apart along K).  The n output features a CTA produces are n / 16
// consecutive chunks: one contiguous piece, whatever n is, and a warp's 32 rows of a chunk are 512 consecutive bytes.
__device__ __forceinline__ uint32_t mid_offset(uint32_t row, uint32_t k, uint32_t R) { return (k >> 4) * (R * 16) + row * 16 + (k & 15u); }

}  // namespace

template <int OUT>
__global__ void __cluster_dims__(CL, 1, 1) __launch_bounds__(THREADS, 1)
mlp_fused_kernel(const __grid_constant__ CUtensorMap map0, const __grid_constant__ CUtensorMap map1,
                 const __grid_constant__ CUtensorMap map2, const __grid_constant__ CUtensorMap map3, const MlpParams P,
                 const float *__restrict__ x, uint32_t M, float in_scale, float in_zpf, void *__restrict__ out, uint32_t *status)
{
    griddep_launch_dependents();
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *base_ptr = smem_raw + (base - raw);
    const uint32_t bar0 = base + P.bar_off;  // w_full[l] = +8l, act_ready[l] = +32+8l, acc_full[l] = +64+8l
    uint32_t *misc = reinterpret_cast<uint32_t *>(base_ptr + P.bar_off + 96);  // [0] tmem base, [1] abort flag
    volatile uint32_t *abort_flag = misc + 1;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t cta = cluster_ctarank();
    const uint32_t R = P.rows;                              // batch rows per cluster: 16, 32 or 64
    const uint32_t chunk = R * 16;                          // one 16-byte step along K of a tile between layers
    const uint32_t row_base = (blockIdx.x / CL) * R;        // first batch row of this cluster
    const uint32_t rows_here = M - row_base < R ? M - row_base : R;

    if (threadIdx.x == 0) {
        for (int l = 0; l < MAX_LAYERS; l++) {
            mbar_init(bar0 + 8 * l, 1);
            // Hand-over barriers: ONE local arrival (this CTA's own part of the tile is written) plus the bytes the other
            // CTAs send with bulk copies.  (Remote stores + a cluster-scope fence + one remote arrival per warp were
            // measured first: the fence alone cost ~1 us per hand-over; one arrival per thread, 4-5 us.)
            mbar_init(bar0 + 32 + 8 * l, 1);
            mbar_init(bar0 + 64 + 8 * l, 1);
        }
        // Every hand-over brings 512 bytes of partial row sums from each other CTA, plus: for the input tile the slabs the
        // others quantise; for the tile behind layer l, n / 16 chunks from every other CTA that has columns of layer l.
        const uint32_t slabs0 = P.L[0].slabs, mine0 = cta < slabs0 ? (slabs0 - cta + CL - 1) / CL : 0u;
        mbar_expect_tx_only(bar0 + 32, (CL - 1) * 512 + (slabs0 - mine0) * R * 128);
        for (int l = 0; l + 1 < P.n_layers; l++) {
            const uint32_t senders = (P.L[l].N + P.L[l].n - 1) / P.L[l].n;
            const uint32_t others = senders - (cta < senders ? 1u : 0u);
            mbar_expect_tx_only(bar0 + 32 + 8 * (l + 1), (CL - 1) * 512 + others * (P.L[l].n / 16) * chunk);
        }
        misc[1] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    // both partial-row-sum tables start at zero (16 slots of ROWS sums each; whoever has nothing to add leaves zeros)
    for (uint32_t i = threadIdx.x; i < 2u * CL * 2 * ROWS; i += THREADS) reinterpret_cast<uint32_t *>(base_ptr + P.asum_off)[i] = 0;
    if (warp == 2) {
        tmem_alloc(smem_u32(misc), P.tmem_cols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    // ---- weights: this CTA's slice of every layer, fetched before anything that depends on the previous kernel ----
    if (warp == 3 && lane == 0) {
        for (int l = 0; l < P.n_layers; l++) {
            const MlpLayer &ly = P.L[l];
            if (cta * ly.n >= ly.N) continue;   // no columns of this layer here
            const CUtensorMap *mp = l == 0 ? &map0 : (l == 1 ? &map1 : (l == 2 ? &map2 : &map3));
            mbar_expect_tx(bar0 + 8 * l, ly.slabs * ly.n * 128);
            for (uint32_t s = 0; s < ly.slabs; s++)
                tma_load_2d(base + ly.w_off + s * ly.n * 128, mp, bar0 + 8 * l, (int32_t)(s * 128), (int32_t)(cta * ly.n));
        }
    }
    // ---- column terms of every layer's slice (-zA * wsum[j] + bias[j]) into shared memory: layer data, like the weights ----
    for (int l = 0; l < P.n_layers; l++) {
        const MlpLayer &ly = P.L[l];
        uint32_t *col = reinterpret_cast<uint32_t *>(base_ptr + ly.col_off);
        for (uint32_t j = threadIdx.x; j < ly.n; j += THREADS) {
            const uint32_t gj = cta * ly.n + j;
            uint32_t t = 0;
            if (gj < ly.N) {
                t = (uint32_t)(-ly.zA) * (uint32_t)ly.wsum[gj];
                if (ly.bias) t += (uint32_t)ly.bias[gj];
            }
            col[j] = t;
        }
    }

    cluster_sync();  // every CTA's barriers exist before anybody writes or arrives across (and the column terms are in place)
    tc_fence_after();
    const uint32_t tmem_base = misc[0];
    griddep_wait();  // from here on: the input, the row-sum / bias vectors and the output may depend on the previous kernel

    // ---- input quantise: CTA c takes the 128-column slab c (c + 8, ...) of all R rows into its own tile - warp w rows
    //      w, w + 8, ..., a lane four columns, every load of a slab issued before the arithmetic - and sends each slab and
    //      its partial row sums (slot 2c of the table) to the other CTAs as bulk copies ----
    {
        const MlpLayer &l0 = P.L[0];
        const float inv = quant_screen_inv(in_scale);
        uint8_t *tile = base_ptr + P.act_off[0];
        uint32_t *sums = reinterpret_cast<uint32_t *>(base_ptr + P.asum_off) + (cta * 2) * ROWS;
        const bool vec = ((l0.K & 3u) == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0);
        uint32_t acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};          // row sums of rows warp, warp + 8, ... over this CTA's slabs
        for (uint32_t sl = cta; sl < l0.slabs; sl += CL) {
            const uint32_t k = sl * 128 + 4 * lane;          // this lane's four columns
            float4 v[8];
#pragma unroll
            for (uint32_t u = 0; u < 8; u++) {
                const uint32_t r = (uint32_t)warp + 8 * u;
                v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (r < rows_here && k < l0.K) {
                    const float *xr = x + (size_t)(row_base + r) * l0.K + k;
                    if (vec) {
                        v[u] = __ldcs(reinterpret_cast<const float4 *>(xr));
                    } else {
                        v[u].x = xr[0];
                        if (k + 1 < l0.K) v[u].y = xr[1];
                        if (k + 2 < l0.K) v[u].z = xr[2];
                        if (k + 3 < l0.K) v[u].w = xr[3];
                    }
                }
            }
#pragma unroll
            for (uint32_t u = 0; u < 8; u++) {
                const uint32_t r = (uint32_t)warp + 8 * u;
                if (r < rows_here && k < l0.K) {
                    uint32_t p = quant4_u8(v[u], in_scale, in_zpf, inv);
                    if (k + 4 > l0.K) p &= 0xFFFFFFFFu >> (8 * (k + 4 - l0.K));   // columns beyond K: bytes that count for nothing
                    acc[u] = __dp4a(p, 0x01010101u, acc[u]);
                    *reinterpret_cast<uint32_t *>(tile + act_offset(r, k, R)) = p;
                }
            }
        }
        if (cta < l0.slabs) {
#pragma unroll
            for (uint32_t u = 0; u < 8; u++) {
                uint32_t t = acc[u];
                for (int o = 16; o; o >>= 1) t += __shfl_xor_sync(0xFFFFFFFFu, t, o);
                if (lane == 0 && (uint32_t)warp + 8 * u < R) sums[warp + 8 * u] = t;
            }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // plain stores -> the copy engine's reads
        __syncthreads();
        if (warp == 0 && lane < CL) {
            if ((uint32_t)lane == cta) {
                mbar_arrive(bar0 + 32);
            } else {
                const uint32_t bar_there = map_to_cta(bar0 + 32, (uint32_t)lane);
                for (uint32_t sl = cta; sl < l0.slabs; sl += CL) {
                    const uint32_t t = base + P.act_off[0] + sl * R * 128;
                    bulk_copy_to_cta(map_to_cta(t, (uint32_t)lane), t, R * 128, bar_there);
                }
                const uint32_t a = base + P.asum_off + (cta * 2) * ROWS * 4;
                bulk_copy_to_cta(map_to_cta(a, (uint32_t)lane), a, 512, bar_there);
            }
        }
    }

    // ---- layers ----
    bool ok = true;
    for (int l = 0; l < P.n_layers; l++) {
        const MlpLayer &ly = P.L[l];
        const bool last = l == P.n_layers - 1;
        const bool have_cols = cta * ly.n < ly.N;
        const uint32_t a_tile = base + P.act_off[l & 1];
        // The last hand-over has been issued by everybody once the last layer starts.  A CTA may leave when every CTA of the
        // cluster has RECEIVED everything sent to it (copies still landing in a CTA that has exited would hit whoever got
        // its shared memory next): each CTA's MMA warp says so after its wait below, all other threads right away, and
        // the matching wait is at the very end - the barrier's round trip passes under the last layer.
        if (last && warp != 2) cluster_arrive();
        if (warp == 2) {
            // MMA issuer: needs this layer's activations (from all CTAs) and this CTA's weight slice.  It waits for the
            // activations even when this CTA has no columns of the layer, so that every byte sent here has landed.
            ok = ok && __all_sync(0xFFFFFFFFu, wait_cluster(bar0 + 32 + 8 * l, abort_flag, status, 0xA00u | l));
            if (last) cluster_arrive();
            if (have_cols) {
                ok = ok && __all_sync(0xFFFFFFFFu, mbar_wait(bar0 + 8 * l, 0, abort_flag, status, 0xB00u | l));
                if (ok) {
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // peers' plain stores -> tensor-core reads
                    tc_fence_after();
                    const uint32_t idesc = make_idesc_i8(128, (int)ly.n);
                    if (elect_one()) {
                        for (uint32_t s = 0; s < ly.slabs; s++) {
                            const uint64_t b_desc = make_smem_desc(base + ly.w_off + s * ly.n * 128);
                            if (l == 0) {
                                const uint64_t a_desc = make_smem_desc(a_tile + s * R * 128);
#pragma unroll
                                for (int k = 0; k < 4; k++) umma_i8(tmem_base, a_desc + 2u * k, b_desc + 2u * k, idesc, (s | k) != 0u);
                            } else {
                                // 32 bytes of K = two chunks of the unswizzled tile
                                const uint64_t a_desc = make_smem_desc_plain(a_tile + s * 8 * chunk, chunk, 128);
#pragma unroll
                                for (int k = 0; k < 4; k++)
                                    umma_i8(tmem_base, a_desc + (uint64_t)((2u * k * chunk) >> 4), b_desc + 2u * k, idesc, (s | k) != 0u);
                            }
                        }
                        umma_commit(bar0 + 64 + 8 * l);
                    }
                    __syncwarp();
                }
            }
        } else if ((warp & 3) < 2) {
            // epilogue warps 0, 1, 4, 5: TMEM lanes (= batch rows) 32 * (warp & 3) ..., columns split in two halves
            const uint32_t q = (uint32_t)warp & 3u, h = (uint32_t)warp >> 2;
            const uint32_t r = q * 32 + lane;
            const uint32_t half = ((ly.n / 2 + 15) / 16) * 16;
            const uint32_t cb = h ? half : 0, ce = h ? ly.n : half;
            uint32_t rsum = 0;
            if (have_cols) {
                // activation row sum of this layer's input: 16 partial sums per row, written by the producers
                ok = ok && wait_cluster(bar0 + 32 + 8 * l, abort_flag, status, 0xC00u | l);
                uint32_t asum = 0;
                if (ok) {
                    const uint32_t *part = reinterpret_cast<const uint32_t *>(base_ptr + P.asum_off) + (l & 1) * CL * 2 * ROWS;
#pragma unroll
                    for (int p = 0; p < CL * 2; p++) asum += part[p * ROWS + r];
                }
                Epilogue e = make_epilogue(nullptr, nullptr, nullptr, ltq_qparams{ly.sA, (uint8_t)ly.zA}, ltq_qparams{ly.sB, (uint8_t)ly.zB},
                                           ltq_qparams{ly.sC, (uint8_t)ly.zC}, ly.K, last ? P.out_mode : LTQ_OUT_U8, ly.flags);
                const EpilogueConsts c = epilogue_consts(e);
                const uint32_t rt = c.neg_zB * asum + c.bc;
                const bool relu = ly.flags & LTQ_FLAG_RELU, sat = ly.flags & LTQ_FLAG_SATURATE;
                const uint32_t *col = reinterpret_cast<const uint32_t *>(base_ptr + ly.col_off);
                ok = ok && mbar_wait(bar0 + 64 + 8 * l, 0, abort_flag, status, 0xD00u | l);
                if (ok) {
                    tc_fence_after();
                    const uint32_t taddr = tmem_base + ((q * 32u) << 16);
                    uint32_t vn[16];
                    if (cb < ce) tmem_ld16(taddr + cb, vn);
#pragma unroll 1
                    for (uint32_t cc = cb; cc < ce; cc += 16) {
                        uint32_t v[16];
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 16; j++) v[j] = vn[j];
                        if (cc + 16 < ce) tmem_ld16(taddr + cc + 16, vn);   // the next chunk travels while this one is converted
                        const uint32_t gcol = cta * ly.n + cc;          // first output feature of the chunk
                        if (gcol >= ly.N) continue;
                        const int valid = ly.N - gcol < 16u ? (int)(ly.N - gcol) : 16;
                        if (!last) {
                            uint32_t res[16];
                            epilogue_convert<0, 16>(v, rt, col + cc, c, relu, sat, res);
                            rsum += packed_byte_sum<16>(res, valid);
                            // columns beyond N meet zero weights in the next layer; whatever is written there is harmless
                            if (r < R)   // (TMEM lanes beyond the cluster's rows hold products of whatever lay behind the tile)
                                *reinterpret_cast<uint4 *>(base_ptr + P.act_off[(l + 1) & 1] + mid_offset(r, gcol, R)) =
                                    make_uint4(res[0], res[1], res[2], res[3]);
                        } else if (r < rows_here) {
                            const uint64_t o = (uint64_t)(row_base + r) * ly.N + gcol;
                            epilogue_chunk<OUT, 16>(v, rt, col + cc, c, relu, sat, e, out, o, false, valid);
                        }
                    }
                    tc_fence_before();
                }
            }
            if (!last) {
                // partial row sum of this CTA's columns (this warp's half) for the next layer (zero without columns), then
                // the hand-over: this CTA's chunks of the next tile and its 2 x 64 partial sums go to the other CTAs
                reinterpret_cast<uint32_t *>(base_ptr + P.asum_off)[(((l + 1) & 1) * CL * 2 + cta * 2 + h) * ROWS + r] = rsum;
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                epilogue_warps_sync();
                if (warp == 0 && lane < CL) {
                    const uint32_t bar_next = bar0 + 32 + 8 * (l + 1);
                    if ((uint32_t)lane == cta) {
                        mbar_arrive(bar_next);
                    } else {
                        const uint32_t bar_there = map_to_cta(bar_next, (uint32_t)lane);
                        if (have_cols) {
                            const uint32_t a = base + P.act_off[(l + 1) & 1] + cta * (ly.n / 16) * chunk;
                            bulk_copy_to_cta(map_to_cta(a, (uint32_t)lane), a, (ly.n / 16) * chunk, bar_there);
                        }
                        const uint32_t a = base + P.asum_off + ((((l + 1) & 1) * CL * 2 + cta * 2) * ROWS) * 4;
                        bulk_copy_to_cta(map_to_cta(a, (uint32_t)lane), a, 512, bar_there);
                    }
                }
            }
        }
        // The accumulator columns are reused by the next layer: the MMA warp may only go on once the epilogue warps have
        // read them (and a timed-out role takes everybody with it).
        __syncthreads();
        ok = ok && !*abort_flag;
    }

    // Teardown: nobody leaves before every CTA of the cluster has everything that was sent to it (the arrivals were
    // made at the start of the last layer).
    tc_fence_before();
    __syncthreads();
    cluster_wait();
    if (warp == 2) {
        tc_fence_after();
        tmem_dealloc(tmem_base, P.tmem_cols);
    }
}

}  // namespace ltq

// ---- host side ------------------------------------------------------------------------------------------------------
using namespace ltq;

struct ltq_mlp {
    int device = 0;
    int n_layers = 0;
    ltq_layer *layers[MAX_LAYERS] = {nullptr};
    TcOperandMap maps[MAX_LAYERS];
    MlpParams P;
};

namespace {

template <int OUT>
cudaError_t launch_mlp(const ltq_mlp *m, const float *x, uint64_t M, float scale, float zpf, void *out, uint32_t *status,
                       cudaStream_t stream)
{
    static bool attr_done[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_done[dev]) {
        cudaError_t e = cudaFuncSetAttribute(mlp_fused_kernel<OUT>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT);
        if (e != cudaSuccess) return e;
        attr_done[dev] = true;
    }
    const unsigned clusters = (unsigned)((M + m->P.rows - 1) / m->P.rows);
    auto mp = [&](int l) -> const CUtensorMap & {
        return *reinterpret_cast<const CUtensorMap *>(m->maps[l < m->n_layers ? l : 0].opaque);
    };
    cudaError_t e = launch_chained(mlp_fused_kernel<OUT>, dim3(clusters * CL), dim3(THREADS), (size_t)m->P.smem_bytes, stream, mp(0),
                                   mp(1), mp(2), mp(3), m->P, x, (uint32_t)M, scale, zpf, out, status);
    count_launch();
    note_kernel("mlp_fused_kernel<%s> (%d layers, %u clusters of %d)", out_mode_name(OUT), m->n_layers, clusters, CL);
    return e;
}

}  // namespace

extern "C" {

int ltq_mlp_create(ltq_mlp **mlp, ltq_layer *const *layers, int n_layers)
{
    LTQ_REQUIRE(mlp, LTQ_ERR_INVALID_ARG, "Invalid argument");
    *mlp = nullptr;
    LTQ_REQUIRE(layers && n_layers >= 2 && n_layers <= MAX_LAYERS, LTQ_ERR_INVALID_ARG, "a fused chain has 2 to %d layers", MAX_LAYERS);
    for (int l = 0; l < n_layers; l++) {
        LTQ_REQUIRE(layers[l] && layers[l]->w, LTQ_ERR_INVALID_ARG, "layer %d has no weights bound (ltq_layer_set_weights)", l);
        LTQ_REQUIRE(layers[l]->device == layers[0]->device, LTQ_ERR_INVALID_ARG, "the layers live on different devices");
        LTQ_REQUIRE(l == 0 || layers[l]->K == layers[l - 1]->N, LTQ_ERR_INVALID_ARG,
                    "layer %d takes %llu features, layer %d produces %llu", l, (unsigned long long)layers[l]->K, l - 1,
                    (unsigned long long)layers[l - 1]->N);
    }
    ltq_mlp *m = new (std::nothrow) ltq_mlp;
    LTQ_REQUIRE(m, LTQ_ERR_NO_MEMORY, "out of host memory");
    m->device = layers[0]->device;
    m->n_layers = n_layers;
    MlpParams &P = m->P;
    memset(&P, 0, sizeof P);
    P.n_layers = n_layers;
    // shared-memory plan: [act 0][act 1][weights of all layers][8 KB the last MMA may read beyond its slab][column terms]
    // [partial row sums][barriers]
    uint32_t act_bytes[2] = {0, 0}, max_n = 0;
    const char *why = nullptr;
    for (int l = 0; l < n_layers; l++) {
        MlpLayer &ly = P.L[l];
        m->layers[l] = layers[l];
        ly.K = (uint32_t)layers[l]->K;
        ly.N = (uint32_t)layers[l]->N;
        ly.n = (uint32_t)((layers[l]->N + CL * 16 - 1) / (CL * 16)) * 16;
        ly.slabs = (ly.K + 127) / 128;
        if (ly.K % 16 != 0 || (reinterpret_cast<uintptr_t>(layers[l]->w) & 15)) why = "K must be a multiple of 16 and the weights 16-byte aligned";
        if (ly.n > 256) why = "more than 2048 output features in a layer";
        // the input tile is ly.slabs swizzled slabs; a tile between layers holds 8 chunks per slab of the consumer's K and
        // must also take n / 16 chunks from each of the producer's CTAs
        uint32_t tile = ly.slabs * SLAB;
        if (l > 0 && CL * (P.L[l - 1].n / 16) * (ROWS * 16u) > tile) tile = CL * (P.L[l - 1].n / 16) * (ROWS * 16u);
        if (tile > act_bytes[l & 1]) act_bytes[l & 1] = tile;
        if (ly.n > max_n) max_n = ly.n;
    }
    uint32_t off = 0;
    P.act_off[0] = off;
    off += act_bytes[0];
    P.act_off[1] = off;
    off += act_bytes[1];
    for (int l = 0; l < n_layers; l++) {
        P.L[l].w_off = off;
        off += P.L[l].slabs * P.L[l].n * 128;   // n is a multiple of 16, so every slab tile stays 1024-byte aligned ... for n % 8 == 0
    }
    off += SLAB;                                 // rows 64..127 of the last activation slab / weight rows up to 128 are read, never used
    for (int l = 0; l < n_layers; l++) {
        P.L[l].col_off = off;
        off += P.L[l].n * 4;
    }
    off = (off + 15) & ~15u;
    P.asum_off = off;
    off += 2 * CL * 2 * ROWS * 4;
    off = (off + 15) & ~15u;
    P.bar_off = off;
    off += 96 + 16;
    P.smem_bytes = off + 1024;                   // alignment slack
    // an MMA reads 128 rows from the start of a slab or chunk, whatever the cluster's row count: 16 KB from the input tile's
    // last slab, 2 KB from a later tile's last chunk - all inside the allocation
    if (P.smem_bytes < P.act_off[1] + act_bytes[1] + 16 * 1024 + 2048) P.smem_bytes = P.act_off[1] + act_bytes[1] + 16 * 1024 + 2048;
    P.tmem_cols = 32;
    while (P.tmem_cols < max_n) P.tmem_cols *= 2;
    // a weight slab tile of n rows x 128 B must start on a 1024-byte boundary for the swizzled descriptor: n % 8 == 0 holds
    if (!why && P.smem_bytes > (uint32_t)SMEM_LIMIT) why = "the chain's weights and activations do not fit one cluster's shared memory";
    if (why) {
        set_error("this chain cannot run fused: %s", why);
        delete m;
        return LTQ_ERR_UNSUPPORTED;
    }
    for (int l = 0; l < n_layers; l++) {
        const int er = tc_make_map(&m->maps[l], layers[l]->w, layers[l]->N, layers[l]->K, (int)P.L[l].n);
        if (er != 0) {
            set_error("cuTensorMapEncodeTiled failed for layer %d (CUresult %d)", l, er);
            delete m;
            return LTQ_ERR_CUDA;
        }
    }
    *mlp = m;
    return LTQ_OK;
}

int ltq_mlp_destroy(ltq_mlp *mlp)
{
    delete mlp;
    return LTQ_OK;
}

int ltq_mlp_forward(ltq_mlp *mlp, const float *x_dev, uint64_t M, const unsigned *layer_flags, int out_mode, void *out_dev,
                    void *stream)
{
    LTQ_REQUIRE(mlp && x_dev && out_dev, LTQ_ERR_INVALID_ARG, "Invalid argument");
    LTQ_REQUIRE(out_mode == LTQ_OUT_U8 || out_mode == LTQ_OUT_F32 || out_mode == LTQ_OUT_I32, LTQ_ERR_INVALID_ARG,
                "unknown out_mode %d", out_mode);
    LTQ_REQUIRE(M < (1ull << 31), LTQ_ERR_TOO_LARGE, "M must be below 2^31");
    if (M == 0) return LTQ_OK;
    LTQ_ENTER_DEVICE(mlp->device);
    MlpParams &P = mlp->P;
    for (int l = 0; l < mlp->n_layers; l++) {
        const ltq_layer *ly = mlp->layers[l];
        MlpLayer &d = P.L[l];
        LTQ_REQUIRE(static_cast<const void *>(ly->w) == mlp->maps[l].base, LTQ_ERR_INVALID_ARG,
                    "layer %d's weights were rebound after ltq_mlp_create; create the chain again", l);
        d.wsum = ly->wsum;
        d.bias = ly->bias;
        d.sA = ly->qp_in.scale;
        d.zA = ly->qp_in.zero_point;
        d.sB = ly->qp_wt.scale;
        d.zB = ly->qp_wt.zero_point;
        d.sC = ly->qp_out.scale;
        d.zC = ly->qp_out.zero_point;
        d.flags = (layer_flags ? layer_flags[l] : 0u) & (LTQ_FLAG_RELU | LTQ_FLAG_SATURATE);
        const uint64_t bc = (uint64_t)d.K * (uint64_t)d.zA * (uint64_t)d.zB;
        LTQ_REQUIRE(bc <= 0x7FFFFFFFull, LTQ_ERR_UNSUPPORTED, "K*zA*zB = %llu does not fit an int", (unsigned long long)bc);
    }
    P.out_mode = out_mode;
    // Rows per cluster: a small batch is spread over more clusters (every hand-over moves rows x features bytes into
    // every CTA, and the SM-to-SM copies are what a layer waits for); a large one gets the full 64 rows per cluster.
    const uint64_t sms = (uint64_t)mlp->layers[0]->dev->sms;
    P.rows = ((M + 15) / 16) * CL <= sms ? 16u : (((M + 31) / 32) * CL <= sms ? 32u : (uint32_t)ROWS);
    const ltq_layer *l0 = mlp->layers[0];
    const float scale = l0->qp_in.scale, zpf = (float)(int)l0->qp_in.zero_point;
    cudaStream_t st = (cudaStream_t)stream;
    uint32_t *status = l0->dev->status;
    switch (out_mode) {
        case LTQ_OUT_U8: LTQ_CUDA_TRY(launch_mlp<0>(mlp, x_dev, M, scale, zpf, out_dev, status, st)); break;
        case LTQ_OUT_F32: LTQ_CUDA_TRY(launch_mlp<1>(mlp, x_dev, M, scale, zpf, out_dev, status, st)); break;
        default: LTQ_CUDA_TRY(launch_mlp<2>(mlp, x_dev, M, scale, zpf, out_dev, status, st));
    }
    return LTQ_OK;
}

}  // extern "C"
