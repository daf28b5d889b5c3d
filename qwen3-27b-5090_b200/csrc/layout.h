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
// (one pipeline stage); unit u = tile * chunks + chunk. Two ways of dealing the units to `grid` CTAs:
//
//  * ranges (split == 0): CTA g owns the contiguous unit range [unit_begin(g), unit_begin(g + 1)), so every CTA
//    streams the same number of bytes (+-1 unit); a range boundary may cut a tile;
//  * aligned (split == s >= 1): every tile is cut into s K-parts of (almost) equal length and the items
//    (tile, part) are dealt round-robin; with s == 1 no tile is cut at all.
//
// A tile that is not cut is finished by its CTA; a cut tile is summed from partial tiles, in ascending K order.
// choose_skinny_plan picks the cheaper way from a small cost model. Nothing here depends on the token count, so a
// token's result is the same whatever M it is computed with.
struct SkinnyPlan {
  int tiles;       // N / 128
  int chunks;      // ceil(K / 256)
  int grid;        // CTAs
  int64_t units;   // tiles * chunks
  int split;       // 0: contiguous unit ranges; s >= 1: s aligned K-parts per tile
};

// First unit of range g. (32-bit arithmetic when it cannot overflow: a 64-bit division costs the GPU hundreds of
// cycles and this runs on the kernels' critical path.)
Q27B_HD int64_t unit_begin(const SkinnyPlan& p, int g) {
  if (p.units <= 0x7fffffff / (p.grid > 0 ? p.grid : 1)) return int64_t(uint32_t(p.units) * uint32_t(g) / uint32_t(p.grid));
  return p.units * g / p.grid;
}

// The range that owns unit u.
Q27B_HD int unit_owner(const SkinnyPlan& p, int64_t u) {
  int g = p.units <= 0x7fffffff / (p.grid > 0 ? p.grid : 1) ? int(uint32_t(u) * uint32_t(p.grid) / uint32_t(p.units))
                                                             : int(u * p.grid / p.units);
  if (g >= p.grid) g = p.grid - 1;
  while (g + 1 < p.grid && unit_begin(p, g + 1) <= u) g++;
  while (g > 0 && unit_begin(p, g) > u) g--;
  return g;
}

// One contiguous piece of work inside a single tile.
struct Segment {
  int tile;
  int c0, c1;      // chunk range [c0, c1)
  int slot;        // partial-tile slot in the workspace, or -1 when the piece covers the whole tile (finished in place)
};

// Pieces of CTA g, in the order the CTA works through them; returns false when all have been handed out. Start
// with u = -1. With ranges, a cut tile at the END of the range comes first: its other part is the first piece of
// the next CTA, so both parts are ready early and the tile is summed while the uncut tiles are still streaming.
Q27B_HD bool next_segment(const SkinnyPlan& p, int g, int64_t& u, Segment& s) {
  if (p.split > 0) {
    u = u < 0 ? g : u + p.grid;  // item index
    if (u >= int64_t(p.tiles) * p.split) return false;
    s.tile = int(uint32_t(u) / uint32_t(p.split));
    const int part = int(u) - s.tile * p.split;
    s.c0 = part * p.chunks / p.split, s.c1 = (part + 1) * p.chunks / p.split;
    s.slot = p.split == 1 ? -1 : int(u);
    return true;
  }
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
  s.slot = whole ? -1 : 2 * g + (u == u0 ? 0 : 1);  // 2 g: the piece at the range start, 2 g + 1: at its end
  u += s.c1 - s.c0;
  return true;
}

// The partial tiles a cut tile is summed from, in ascending K order: their number (1: the tile is not cut) and,
// through part_slot, the workspace slot of the i-th.
struct TileParts {
  int n, g0;
  int64_t ubeg;
};
Q27B_HD TileParts tile_parts(const SkinnyPlan& p, int tile) {
  TileParts t;
  t.ubeg = int64_t(tile) * p.chunks;
  if (p.split > 0) {
    t.n = p.split, t.g0 = tile * p.split;
  } else {
    t.g0 = unit_owner(p, t.ubeg);
    t.n = unit_owner(p, t.ubeg + p.chunks - 1) - t.g0 + 1;
  }
  return t;
}
Q27B_HD int part_slot(const SkinnyPlan& p, const TileParts& t, int i) {
  if (p.split > 0) return t.g0 + i;
  return 2 * (t.g0 + i) + (unit_begin(p, t.g0 + i) >= t.ubeg ? 0 : 1);
}

// Number of partial-tile slots the workspace must hold, and whether any tile is cut.
Q27B_HD int64_t plan_slots(const SkinnyPlan& p) {
  return p.split > 0 ? (p.split == 1 ? 0 : int64_t(p.tiles) * p.split) : int64_t(2) * p.grid;
}
Q27B_HD bool plan_cuts_tiles(const SkinnyPlan& p) {
  if (p.split > 0) return p.split > 1;
  for (int g = 1; g < p.grid; g++)
    if (unit_begin(p, g) % p.chunks != 0) return true;
  return false;
}

// The split of a shape for `slots` CTAs that can run at once (the launchers use two per multiprocessor). Cost model, in hundredths of a microsecond as measured on B200: 0.76 us per unit a CTA
// streams while the GPU is full, ~3.3 us to publish and sum a cut tile at the end of a CTA, ~1 us for an epilogue
// in place.
Q27B_HD SkinnyPlan choose_skinny_plan(int N, int K, int slots) {
  SkinnyPlan p;
  p.tiles = N / 128;
  p.chunks = (K + 255) / 256;
  p.units = int64_t(p.tiles) * p.chunks;
  p.grid = p.units < slots ? int(p.units) : slots;
  p.split = 0;
  if (p.units <= slots) return p;  // one unit per CTA either way
  const int64_t per_range = (p.units + slots - 1) / slots;
  const int64_t cost_ranges = per_range * 76 + 330;
  int s = slots / p.tiles;
  s = s < 1 ? 1 : (s > p.chunks ? p.chunks : s);
  const int64_t items = int64_t(p.tiles) * s;
  const int grid = items < slots ? int(items) : slots;
  const int64_t waves = (items + grid - 1) / grid;
  const int64_t cost_aligned = ((p.chunks + s - 1) / s) * waves * 76 + (s == 1 ? 100 : 330);
  if (cost_aligned <= cost_ranges) p.split = s, p.grid = grid;
  return p;
}

// Bytes of partial tiles the weight-streaming GEMM may write: [M][128] fp32 per slot.
Q27B_HD int64_t skinny_workspace_bytes(int M, const SkinnyPlan& p) { return plan_slots(p) * M * 128 * 4; }

}  // namespace q27b
