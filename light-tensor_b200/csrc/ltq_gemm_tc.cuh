// Host-visible interface of the tcgen05 GEMM (ltq_gemm_tc.cu), kept free of <cuda.h> so the API layer can hold tensor
// maps inside its layer handle without seeing driver types.
#pragma once
#include "ltq_common.cuh"

namespace ltq {

// A TMA tensor map (CUtensorMap is 128 bytes, 64-byte aligned) over a K-contiguous uint8 matrix [rows, K], tiled in
// boxes of box_rows x 128 bytes with the 128-byte swizzle, plus the facts it was built from so a cached map can be
// checked against the next call.
struct TcOperandMap {
    alignas(64) unsigned char opaque[128];
    const void *base = nullptr;
    uint64_t rows = 0, K = 0;
    int box_rows = 0;
    int box_lines = 0;  // 0 for the 2-D form; lines of 128 bytes along K per box for the 3-D form
    bool matches(const void *b, uint64_t r, uint64_t k, int br, int bl = 0) const
    {
        return base == b && rows == r && K == k && box_rows == br && box_lines == bl;
    }
};

// True when the tensor-core kernel can take the problem: K a multiple of 16 (TMA row pitch), 16-byte aligned bases,
// extents below 2^31, and the driver exports cuTensorMapEncodeTiled.
bool tc_shape_ok(uint64_t M, uint64_t N, uint64_t K, const void *A, const void *B);
// Output-tile width (64, 128 or 256 columns) for a problem on a device with `sms` SMs.
int tc_pick_bn(uint64_t M, uint64_t N, int sms);
// Encodes a map; box_rows is 128 for the A operand and the tile width for the B operand. 0 on success.
int tc_make_map(TcOperandMap *m, const uint8_t *base, uint64_t rows, uint64_t K, int box_rows);
// CTA-pair variant (256-row tiles, tcgen05.mma.cta_group::2).  tc_pair_preferred says when the problem is large enough.
// tc_pair_tiling cuts the output into tiles of up to four widths (multiples of 16 columns, or of 32 with `unit32`, at
// most 256), numbered widest first in up to four classes: tiles [start[k], start[k+1]) belong to class k, which covers
// tile rows row0[k] ... with per_row[k] tiles each, the first at column col0[k], all width[k] wide.  Unused classes
// have start = 0xFFFFFFFF.  map_a uses 128-row boxes; map_b[k] boxes of width[k] / 2 rows (each CTA of a pair loads half
// of a tile's B rows); entries of unused classes may repeat a used one.
struct PairTiling {
    uint32_t num_tiles;
    uint32_t start[4], per_row[4], row0[4], col0[4], width[4];
};
bool tc_pair_preferred(uint64_t M, uint64_t N, int sms);
PairTiling tc_pair_tiling(uint64_t M, uint64_t N, int sms, bool unit32);
cudaError_t launch_gemm_tc_pair(const TcOperandMap &map_a, const TcOperandMap *const map_b[4], const PairTiling &tl, uint64_t M,
                                uint64_t N, uint64_t K, const Epilogue &epi, void *out, uint32_t *status, int sms,
                                cudaStream_t stream);
// 3-D view of the same kind of matrix for the weight-streaming kernel (K % 128 == 0): dims {128 B line, rows, K/128
// lines}, box {128 B, box_rows, box_lines}.  One box lands in shared memory as [line][row][128 B]; with the 128-byte
// swizzle the 16-byte chunk index is XORed with the low three bits of (line * box_rows + row), so the rows of a box
// read at the same K offset fall in different banks.  0 on success.
int tc_make_map_lines(TcOperandMap *m, const uint8_t *base, uint64_t rows, uint64_t K, int box_rows, int box_lines);
cudaError_t launch_gemm_tc(const TcOperandMap &map_a, const TcOperandMap &map_b, int bn, uint64_t M, uint64_t N,
                           uint64_t K, const Epilogue &epi, void *out, uint32_t *status, int sms, cudaStream_t stream);

}  // namespace ltq
