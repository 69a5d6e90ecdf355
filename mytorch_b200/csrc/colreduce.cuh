// Per-channel (column) reductions over a row-major [rows, C] matrix — the shape every
// channels-last activation takes when viewed as pixels x channels.
//
// A CTA of 256 threads owns L column groups (L a power of two <= 256, each group VEC
// channels wide) and R = 256 / L rows per iteration, so consecutive threads read
// consecutive addresses.  Each CTA reduces a contiguous row range and writes one partial
// row per quantity into scratch; a small second kernel combines the partials in a fixed
// order, so results are bit-reproducible (no float atomics).
#pragma once
#include "common.cuh"

struct ColCfg {
  int vec;              // 4 (float4) or 1
  int cv;               // column groups = C / vec
  int lanes;            // L
  int rows_per_iter;    // R
  int col_blocks;
  int row_blocks;       // P: number of partial rows per quantity
  long long rows_per_block;
};

static inline ColCfg mtb_col_cfg(long long rows, int C, bool aligned, int max_row_blocks = 0, int ctas_per_sm = 4) {
  ColCfg c;
  c.vec = (aligned && C % 4 == 0) ? 4 : 1;
  c.cv = C / c.vec;
  int lanes = 1;
  while (lanes < c.cv && lanes < 256) lanes <<= 1;
  c.lanes = lanes;
  c.rows_per_iter = 256 / lanes;
  c.col_blocks = (c.cv + lanes - 1) / lanes;
  long long target = (long long)mtb_sm_count() * ctas_per_sm / c.col_blocks;
  if (target < 1) target = 1;
  if (max_row_blocks > 0 && target > max_row_blocks) target = max_row_blocks;
  long long min_rows = (long long)c.rows_per_iter * 8;  // at least 8 loop trips per thread
  long long want = (rows + min_rows - 1) / min_rows;
  if (want < 1) want = 1;
  c.row_blocks = (int)(want < target ? want : target);
  long long rpb = (rows + c.row_blocks - 1) / c.row_blocks;
  rpb = (rpb + c.rows_per_iter - 1) / c.rows_per_iter * c.rows_per_iter;
  if (rpb < c.rows_per_iter) rpb = c.rows_per_iter;
  c.rows_per_block = rpb;
  c.row_blocks = (int)((rows + rpb - 1) / rpb);
  if (c.row_blocks < 1) c.row_blocks = 1;
  return c;
}

// Upper bound on row_blocks for any shape (used to size scratch).
static inline int mtb_col_max_partials() { return mtb_sm_count() * 4; }

template <int V> struct VecF { float v[V]; };

template <int V>
__device__ __forceinline__ VecF<V> vload(const float* p) {
  VecF<V> r;
  if (V == 4) {
    float4 t = *reinterpret_cast<const float4*>(p);
    r.v[0] = t.x; r.v[1 % V] = t.y; r.v[2 % V] = t.z; r.v[3 % V] = t.w;
  } else {
    r.v[0] = *p;
  }
  return r;
}

template <int V>
__device__ __forceinline__ void vstore(float* p, const VecF<V>& r) {
  if (V == 4) *reinterpret_cast<float4*>(p) = make_float4(r.v[0], r.v[1 % V], r.v[2 % V], r.v[3 % V]);
  else *p = r.v[0];
}
