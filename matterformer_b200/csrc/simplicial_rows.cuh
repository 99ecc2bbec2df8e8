// Row packing shared by the forward and backward row-packed tensor-core simplicial kernels.
//
// A tcgen05 tile has 128 rows.  A molecule with n queries rarely fills a multiple of 128, and a walk over the
// first key index j with one query per row wastes every row beyond n.  These kernels therefore give each row of
// the tile its own (query i, first key j) pair: the queries of a molecule are split into `tiles` ranges of
// `rows_per_tile` queries, and `groups` = floor(128 / rows_per_tile) consecutive first keys are processed per
// step, group g on rows [g * rows_per_tile, (g + 1) * rows_per_tile).  A step then covers `groups` values of j
// and the walk takes ceil(valid_keys / groups) steps.  The plan minimises tiles * steps.
#pragma once

#include <stdint.h>

namespace mf {

constexpr int kMaxGroups = 8;     // first keys per step (bounded by the per-step staging of k1 / v1 rows)
constexpr int kMaxRowTiles = 8;   // query ranges per molecule

struct RowPlan {
  int tiles;          // query ranges actually used
  int rows_per_tile;  // queries per range (last range may hold fewer)
  int groups;         // first keys per step
  int steps;          // steps per tile
};

__host__ __device__ inline RowPlan plan_rows(int n_queries, int valid_keys) {
  RowPlan best{0, 0, 0, 0};
  long long best_cost = -1;
  if (n_queries <= 0 || valid_keys <= 0) return best;
  for (int t = 1; t <= kMaxRowTiles; ++t) {
    const int rt = (n_queries + t - 1) / t;
    if (rt > 128) continue;
    int g = 128 / rt;
    if (g > kMaxGroups) g = kMaxGroups;
    const int tiles = (n_queries + rt - 1) / rt;
    const int steps = (valid_keys + g - 1) / g;
    const long long cost = (long long)tiles * steps;
    if (best_cost < 0 || cost < best_cost) {
      best_cost = cost;
      best = RowPlan{tiles, rt, g, steps};
    }
  }
  return best;
}

// Largest `tiles` any molecule with at most `tokens` queries and keys can get (sizes the grid).
inline int max_row_tiles(int tokens) {
  int m = 1;
  for (int nq = 1; nq <= tokens; ++nq)
    for (int nk = 1; nk <= tokens; ++nk) {
      const int t = plan_rows(nq, nk).tiles;
      if (t > m) m = t;
    }
  return m;
}

}  // namespace mf
