// What the kernels of the grouped softmax attention share: the argument block, the visibility rule
// and the walk over the key tiles that a window and kept first tokens leave.
#pragma once

#include "common.cuh"

struct GroupedArgs {
  void* out;                 // [T, QH * DV] of the cache's dtype (written when partial_o is null)
  float* partial_o;          // [parts, T, QH, DV] unnormalized sums, or null
  float* partial_ml;         // [parts, T, QH, 2] running maximum and denominator
  const void* q;             // [T, QH * DK]
  const void* kcache;        // [pages, page_size, KH, DK]
  const void* vcache;        // [pages, page_size, VH, DV]
  const int* table;
  const int* req_q_start;
  const int* req_pos0;
  const float* slopes;       // [QH] or null
  const float* gate;         // float32 rows whose first QH * DV numbers gate the output, or null
  long long gate_stride;
  int table_stride, num_req, total_rows;
  int QH, KH, VH, DK, DV, page_size;
  int window, keep_first;    // window <= 0: every earlier key
  int chunk;                 // > 0: only keys of the query's own run of ``chunk`` positions (runs counted from position 0)
  int parts, part_keys;      // part_keys 0: the context is not cut
  float scale;
};

// Does the query at position i see the key at position j?
__host__ __device__ __forceinline__ bool grouped_visible(int i, int j, int window, int keep_first, int chunk = 0) {
  return j <= i && (window <= 0 || i - j < window || j < keep_first) && (chunk <= 0 || j >= i / chunk * chunk);
}

// Tiles of ``step`` keys from k_first on that hold a key some row of the block may see: those below
// keep_first, then those from the window's start (or the start of the chunk) of the block's first row (pos0) on.
struct GroupedTiles {
  int k_first, step, keep_first, win_tile;
  __device__ GroupedTiles(int k_first_, int k_last, int pos0, int window, int keep_first_, int step_, int chunk = 0)
      : k_first(k_first_), step(step_), keep_first(keep_first_) {
    (void)k_last;
    int win0 = window > 0 ? max(0, pos0 - window + 1) : 0;
    if (chunk > 0) win0 = max(win0, pos0 / chunk * chunk);
    win_tile = win0 > k_first ? k_first + (win0 - k_first) / step * step : k_first;
  }
  __device__ int next(int k0) const {
    int k = k0 + step;
    if (k >= keep_first && k < win_tile) k = win_tile;
    return k;
  }
  __device__ int first() const { return next(k_first - step); }
};
