// Work list of a CTA pair in the persistent pair kernels (FP8 and FP16), and the host-side decision
// that goes with it.
#pragma once

#include "host_common.h"

namespace llmmm {

// A split tile is published as one fp32 256x256 partial tile per pair ("slot").
constexpr size_t SPLIT_SLOT_FLOATS = 256 * 256;
constexpr int    SPLIT_MAX_PAIRS   = 80;  // slots covered by the scratch size llmmm_fp8_workspace_bytes() reports
constexpr int    SPLIT_MAX_WAYS    = 8;   // chunks per tile: the warp that sums them reads them one after another

// Work of one pair: whole tiles round-robin (tile = pair + i * n_pairs below dp_tiles).  With fewer tiles
// left for the last wave than there are pairs, that wave would keep only some pairs busy; when scratch is
// registered, each of those tiles is instead cut along K into `split_s` chunks of `split_chunk` K-steps,
// one chunk per pair: pair q ends with chunk q % split_s of tile dp_tiles + q / split_s.  All roles of a
// CTA walk the same list.
struct PairWalk {
  int i, pair, n_pairs, k_blocks, dp_tiles, split_s, split_chunk;
  bool split_pending;

  __device__ PairWalk(int pair_, int n_pairs_, int k_blocks_, int dp_tiles_, int split_pairs, int split_s_, int split_chunk_):
    i(0), pair(pair_), n_pairs(n_pairs_), k_blocks(k_blocks_), dp_tiles(dp_tiles_), split_s(split_s_),
    split_chunk(split_chunk_), split_pending(pair_ < split_pairs)
  {
  }

  __device__ int chunk_begin() const
  {
    return (pair % split_s) * split_chunk;
  }

  __device__ int chunk_end() const
  {
    const int e = chunk_begin() + split_chunk;
    return e < k_blocks ? e : k_blocks;
  }

  __device__ uint32_t total_k_blocks() const
  {
    const int whole = pair < dp_tiles ? (dp_tiles - pair + n_pairs - 1) / n_pairs : 0;
    return (uint32_t)(whole * k_blocks + (split_pending ? chunk_end() - chunk_begin() : 0));
  }

  // next piece of work: K-blocks [kb0, kb1) of `tile`
  __device__ bool next(int& tile, int& kb0, int& kb1)
  {
    const int t = pair + i * n_pairs;
    if (t < dp_tiles) {
      tile = t;
      kb0  = 0;
      kb1  = k_blocks;
      ++i;
      return true;
    }
    if (!split_pending) {
      return false;
    }
    split_pending = false;
    tile          = dp_tiles + pair / split_s;
    kb0           = chunk_begin();
    kb1           = chunk_end();
    return true;
  }
};

// What the launcher decides (plan_split in common.cu): how many tiles run whole, how the rest is cut, the
// grid, and where the partial tiles and their arrival counters live in the registered scratch.
struct SplitPlan {
  int       dp_tiles;
  int       split_pairs;
  int       split_s;
  int       split_chunk;
  int       pairs;  // clusters to launch
  float*    partials;
  uint32_t* counters;
};

// `k_steps` per tile; the cost of a split is estimated as fixed + per_way_x2 * ways / 2 K-steps, and a
// split is planned only if it is expected to save at least `min_gain` K-steps over running the last wave
// with idle pairs.  Without registered scratch (or with nothing to gain) the plan is whole tiles only.
// `count` = false leaves llmmm_split_launch_count() alone (a query, not a launch).
SplitPlan plan_split(const DeviceInfo* info, int tiles, int k_steps, int fixed, int per_way_x2, int min_gain, bool count = true);

}  // namespace llmmm
