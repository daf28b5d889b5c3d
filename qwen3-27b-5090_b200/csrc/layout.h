// Host/device index arithmetic shared by the kernels, the launchers and the CPU tests: the swizzled scale-factor
// layout, the gate | up interleave, and the M-independent work split of the weight-streaming GEMM.
#pragma once

#include <cstdint>

#if defined(__CUDACC__)
#define Q27B_HD __host__ __device__ inline
#else
#define Q27B_HD inline
#endif

namespace q27b {

// Byte offset of scale (row, k-block) of a [rows][kblocks] scale matrix in the swizzled layout: 512-byte atoms
// of 128 rows x 4 k-blocks, atom (row / 128, kb / 4) stored row-of-atoms major; inside an atom row r sits at
// line r % 32 (16 bytes per line), word r / 32, byte kb % 4. (Replaces sf_offset, engine/src/kernels.h:192-195.)
Q27B_HD int64_t sf_offset(int64_t row, int64_t kb, int64_t kblocks) {
  const int64_t katoms = (kblocks + 3) / 4;
  return ((row / 128) * katoms + kb / 4) * 512 + (row % 32) * 16 + ((row % 128) / 32) * 4 + (kb % 4);
}
// Bytes of a swizzled scale buffer (rows padded to 128, k-blocks to 4). (engine/src/kernels.h:197-199)
Q27B_HD int64_t sf_bytes(int64_t rows, int64_t kblocks) {
  return ((rows + 127) / 128) * 128 * ((kblocks + 3) / 4) * 4;
}
// Row of gate (half 0) / up (half 1) row r in the interleaved gate | up matrix. (engine/src/kernels.h:186)
Q27B_HD int64_t glu_row(int64_t r, int half) { return (r / 64) * 128 + half * 64 + r % 64; }

// ---------------------------------------------------------------------------------------------------------------
// Work split of the weight-streaming GEMM. The weight matrix is cut into units of 128 rows x 256 K-elements
// (one pipeline stage); unit u = tile * chunks + chunk. Range g of `grid` (one or two per CTA) is the contiguous unit range
// [unit_begin(g), unit_begin(g + 1)), so every SM streams the same number of bytes (+-1 unit). A tile whose
// units all fall into one CTA is finished by that CTA; a tile cut by a range boundary is summed from per-CTA
// partial tiles, in ascending K order, by the last of its CTAs to arrive. Nothing here depends on the token
// count, so a token's result is the same whatever M it is computed with.
struct SkinnyPlan {
  int tiles;       // N / 128
  int chunks;      // ceil(K / 256)
  int grid;        // unit ranges
  int64_t units;   // tiles * chunks
};

// First unit of range g. (32-bit arithmetic when it cannot overflow: a 64-bit division costs the GPU hundreds of
// cycles and this runs on the kernels' critical path.)
Q27B_HD int64_t unit_begin(const SkinnyPlan& p, int g) {
  if (p.units <= 0x7fffffff / (p.grid > 0 ? p.grid : 1)) return int64_t(uint32_t(p.units) * uint32_t(g) / uint32_t(p.grid));
  return p.units * g / p.grid;
}

// The CTA that owns unit u.
Q27B_HD int unit_owner(const SkinnyPlan& p, int64_t u) {
  int g = p.units <= 0x7fffffff / (p.grid > 0 ? p.grid : 1) ? int(uint32_t(u) * uint32_t(p.grid) / uint32_t(p.units))
                                                             : int(u * p.grid / p.units);
  if (g >= p.grid) g = p.grid - 1;
  while (g + 1 < p.grid && unit_begin(p, g + 1) <= u) g++;
  while (g > 0 && unit_begin(p, g) > u) g--;
  return g;
}

// One contiguous piece of a CTA's range inside a single tile.
struct Segment {
  int tile;
  int c0, c1;      // chunk range [c0, c1)
  int slot;        // partial-tile slot in the workspace (2 * cta + {0: piece at the range start, 1: at its end}), or -1
                   // when the piece covers the whole tile and is finished in place
};

// Pieces of CTA g, in the order the CTA works through them; returns false when all have been handed out. Start
// with u = -1. A cut tile at the END of the range comes first: its other part is the first piece of the next CTA,
// so both parts are ready early and the tile is summed while the uncut tiles are still streaming, instead of
// after everything else.
Q27B_HD bool next_segment(const SkinnyPlan& p, int g, int64_t& u, Segment& s) {
  const int64_t u0 = unit_begin(p, g), u1 = unit_begin(p, g + 1);
  const int64_t tail = p.units <= 0x7fffffff ? int64_t(uint32_t(u1 - 1) / uint32_t(p.chunks) * uint32_t(p.chunks))
                                             : (u1 - 1) / p.chunks * p.chunks;  // first unit of the last tile touched
  const bool tail_first = u1 != tail + p.chunks && tail > u0;
  const int64_t end = tail_first ? tail : u1;
  if (u < 0) {
    u = u0;
    if (tail_first) {
      s.tile = p.units <= 0x7fffffff ? int(uint32_t(tail) / uint32_t(p.chunks)) : int(tail / p.chunks);
      s.c0 = 0, s.c1 = int(u1 - tail), s.slot = 2 * g + 1;
      return true;
    }
  }
  if (u >= end) return false;
  s.tile = p.units <= 0x7fffffff ? int(uint32_t(u) / uint32_t(p.chunks)) : int(u / p.chunks);
  s.c0 = int(u - int64_t(s.tile) * p.chunks);
  const int64_t left = end - u;
  s.c1 = left < int64_t(p.chunks - s.c0) ? s.c0 + int(left) : p.chunks;
  const bool whole = s.c0 == 0 && s.c1 == p.chunks;
  s.slot = whole ? -1 : 2 * g + (u == u0 ? 0 : 1);
  u += s.c1 - s.c0;
  return true;
}

// The split of a shape into `ranges` unit ranges (the launchers use two per multiprocessor).
Q27B_HD SkinnyPlan make_skinny_plan(int N, int K, int ranges) {
  SkinnyPlan p;
  p.tiles = N / 128;
  p.chunks = (K + 255) / 256;
  p.units = int64_t(p.tiles) * p.chunks;
  p.grid = p.units < ranges ? int(p.units) : ranges;
  return p;
}

// Bytes of partial tiles the weight-streaming GEMM may write: two tiles [M][128] fp32 per CTA.
Q27B_HD int64_t skinny_workspace_bytes(int M, int grid) { return int64_t(2) * grid * M * 128 * 4; }

}  // namespace q27b
