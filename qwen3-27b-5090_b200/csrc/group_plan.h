// Work schedule of the grouped weight-streaming GEMM: one persistent launch walks a list of problems (the
// projections of one or several layers), and every CTA streams its share of ALL their weight tiles back to back,
// so the fixed costs of a launch (ring fill, tail, hand-over) are paid once per group instead of once per GEMM.
//
// Each problem keeps exactly the K split its stand-alone launch would use (choose_skinny_plan, layout.h): the
// pieces {tile, chunk range} and the order in which the pieces of a cut tile are summed are the same, which makes
// the grouped results bit-identical to per-GEMM calls. What changes is only WHO streams a piece: the pieces of
// all problems are dealt to the CTAs longest first onto the least loaded CTA, and every CTA walks first its pieces
// of cut tiles, then its whole tiles, each in problem order: the pieces of one tile are then streamed at about the
// same time by their CTAs, and early, so the CTA that sums the tile (fixed by the plan: piece tile % pieces) finds
// the other pieces there soon after its own and sums while whole tiles are still streaming.
// (`rotate`: every CTA starts at a different point of its list instead; kept for experiments only - it spreads the
// pieces of a tile over the whole run of the kernel.)
//
// Whole-tile mode. A group with many tiles (several layers) does not need the K split at all: uncut tiles of all
// problems fill the CTAs evenly by themselves (one layer: 408 tiles of 20 or 68 stages on 296 CTAs does not; eight
// layers do). No partial tiles are written, nothing is summed. Every output is then one accumulation chain over all
// of K, which is what the many-row GEMM computes: the results are bit-identical to q27b_gemm_fp4 / _bf16 / _glu_bf16
// instead of to the weight-streaming launch (whose three K-split shapes add their parts in another order). Both
// modes are deterministic and independent of M.
//
// Host-only code (no CUDA): shared by the launcher and the CPU tests.
#pragma once

#include <algorithm>
#include <cstdint>
#include <queue>
#include <utility>
#include <vector>

#include "layout.h"

namespace q27b {

// One piece of work: a contiguous chunk range of one 128-row weight tile of one problem. 64 bytes, read by the
// kernel as four 16-byte words.
struct GroupItem {
  int prob, tile, c0, c1;    // problem index, tile (128 weight rows), chunk range [c0, c1) of 256 K-elements each
  int slot;                  // partial-tile slot of this piece in the group's workspace; -1: the piece is the whole tile
  int nparts;                // pieces the tile is cut into (1: not cut)
  int slot0;                 // the tile's pieces occupy slots slot0 .. slot0 + nparts - 1 in ascending K order
  int ksteps;                // K / 64 of the problem
  const uint8_t* w_sf_tile;  // scale atoms of this tile's 128 weight rows (device pointer)
  const uint8_t* a_sf;       // scale atoms of the problem's activation (device pointer)
  int counter;               // index of the tile's arrival counter in the workspace
  int sums;                  // 1: the CTA that streams this piece also sums the tile (one piece per cut tile)
  int pad[2];
};
static_assert(sizeof(GroupItem) == 64, "GroupItem is read as four 16-byte words");

struct GroupShape {
  int N, K;
};

struct GroupSchedule {
  std::vector<GroupItem> items;    // grouped by CTA, each CTA's pieces in problem order (pointers not set)
  std::vector<int> cta_first;      // items of CTA g: [cta_first[g], cta_first[g + 1])
  std::vector<int64_t> cta_units;  // units (stages) CTA g streams
  int64_t slots = 0;               // partial-tile slots the workspace must hold
  int counters = 0;                // arrival counters (one per cut tile)
  // stages of the busiest CTA over the mean: 1 = perfectly even (whole tiles of few problems can be far from it)
  double imbalance() const {
    int64_t most = 0, total = 0;
    for (int64_t u : cta_units) most = u > most ? u : most, total += u;
    return total ? double(most) * double(cta_units.size()) / double(total) : 1.0;
  }
};

// The pieces of one problem exactly as its stand-alone launch cuts them, in (tile, K) order.
inline void problem_pieces(int prob, const GroupShape& s, int cta_slots, bool whole_tiles, int tile_rows, int64_t& next_slot,
                           int& next_counter, std::vector<GroupItem>& out) {
  SkinnyPlan plan = choose_skinny_plan(s.N, s.K, cta_slots);
  if (whole_tiles) {  // every tile in one piece (tiles of tile_rows weight rows: 128, or 256 for the many-row roles)
    plan.tiles = s.N / tile_rows, plan.units = int64_t(plan.tiles) * plan.chunks;
    plan.split = 1, plan.grid = plan.tiles < cta_slots ? plan.tiles : cta_slots;
  }
  std::vector<GroupItem> pieces;
  for (int g = 0; g < plan.grid; g++) {
    int64_t u = -1;
    Segment seg;
    while (next_segment(plan, g, u, seg)) {
      GroupItem it = {};
      it.prob = prob, it.tile = seg.tile, it.c0 = seg.c0, it.c1 = seg.c1;
      it.slot = seg.slot >= 0 ? 0 : -1;  // (renumbered below)
      it.ksteps = s.K / 64;
      pieces.push_back(it);
    }
  }
  std::stable_sort(pieces.begin(), pieces.end(), [](const GroupItem& a, const GroupItem& b) {
    return a.tile != b.tile ? a.tile < b.tile : a.c0 < b.c0;
  });
  for (size_t i = 0; i < pieces.size();) {
    size_t j = i;
    while (j < pieces.size() && pieces[j].tile == pieces[i].tile) j++;
    const int n = int(j - i);
    for (size_t k = i; k < j; k++) {
      pieces[k].nparts = n;
      pieces[k].slot0 = n > 1 ? int(next_slot) : -1;
      pieces[k].slot = n > 1 ? int(next_slot + int64_t(k - i)) : -1;
      pieces[k].counter = n > 1 ? next_counter : -1;
      // which piece's CTA sums the tile: dealt round the pieces so that the sums spread over the CTAs
      pieces[k].sums = n > 1 && int(k - i) == pieces[i].tile % n;
    }
    if (n > 1) next_slot += n, next_counter++;
    i = j;
  }
  out.insert(out.end(), pieces.begin(), pieces.end());
}

// Deals the pieces of all problems to at most `cta_slots` CTAs (the CTAs that can be resident at once).
inline GroupSchedule schedule_group(const GroupShape* shapes, int n, int cta_slots, bool whole_tiles = false, bool rotate = false,
                                    int tile_rows = 128) {
  GroupSchedule sch;
  std::vector<GroupItem> all;
  int64_t next_slot = 0;
  int next_counter = 0;
  for (int p = 0; p < n; p++) problem_pieces(p, shapes[p], cta_slots, whole_tiles, tile_rows, next_slot, next_counter, all);
  sch.slots = next_slot, sch.counters = next_counter;
  const int ctas = int(std::min<size_t>(size_t(cta_slots), all.size()));
  // longest piece first onto the CTA with the least to stream (ties: the lower index)
  std::vector<int> order(all.size());
  for (size_t i = 0; i < all.size(); i++) order[i] = int(i);
  std::stable_sort(order.begin(), order.end(),
                   [&](int a, int b) { return all[a].c1 - all[a].c0 > all[b].c1 - all[b].c0; });
  using Load = std::pair<int64_t, int>;  // (units, cta)
  std::priority_queue<Load, std::vector<Load>, std::greater<Load>> heap;
  for (int g = 0; g < ctas; g++) heap.push({0, g});
  std::vector<std::vector<int>> mine(ctas);
  sch.cta_units.assign(ctas, 0);
  for (int i : order) {
    Load l = heap.top();
    heap.pop();
    mine[l.second].push_back(i);
    l.first += all[i].c1 - all[i].c0;
    sch.cta_units[l.second] = l.first;
    heap.push(l);
  }
  sch.cta_first.assign(ctas + 1, 0);
  for (int g = 0; g < ctas; g++) {
    // Pieces of cut tiles first, whole tiles last, each in problem order (then tile, then K): a cut tile can be summed
    // only when all its pieces have been streamed, so they are streamed early by every CTA and summed while the whole
    // tiles (each finished by its own CTA alone) are still streaming. With the plain problem order the pieces of the last
    // problem's cut tiles end every CTA's list and all their sums pile up behind the stream: 13 of 46 us for one layer.
    std::stable_sort(mine[g].begin(), mine[g].end(), [&](int a, int b) {
      const bool wa = all[a].nparts == 1, wb = all[b].nparts == 1;
      return wa != wb ? wb : a < b;
    });
    if (rotate && !mine[g].empty()) std::rotate(mine[g].begin(), mine[g].begin() + g % int(mine[g].size()), mine[g].end());
    for (int i : mine[g]) sch.items.push_back(all[i]);
    sch.cta_first[g + 1] = int(sch.items.size());
  }
  return sch;
}

}  // namespace q27b
