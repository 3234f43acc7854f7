// The cache write fused into the [q | k | v] projection: where a key or value element of the projection's
// output goes in the pages.  Shared by the linear kernels that have such an epilogue.
#pragma once

#include "common.cuh"

struct KvScatter {
  const int* positions;     // [M]
  const int* token_req;     // [M] row of the block table, < 0 for padding rows
  const int* block_table;   // [*, max_pages]
  __nv_bfloat16* k_pool;    // [n_pages, Hkv, page, Dh]
  __nv_bfloat16* v_pool;
  int* status;
  int max_pages, n_pages, page, Hkv, Dh, q_width;
};

// Where the key or value element of output column n (>= q_width) of token m lives in the pages; null for a
// padding row or an index out of range (which sets the status bit).
__device__ __forceinline__ __nv_bfloat16* kv_slot(const KvScatter& kv, int m, int n) {
  const int r = kv.token_req[m];
  if (r < 0) return nullptr;
  const int pos = kv.positions[m];
  const int lp = pos / kv.page;
  const int pg = (pos >= 0 && lp < kv.max_pages) ? kv.block_table[(size_t)r * kv.max_pages + lp] : -2;
  if (pg == -2) {
    atomicOr(kv.status, MLXB_ST_POSITION_RANGE);
    return nullptr;
  }
  if (pg >= kv.n_pages) {
    atomicOr(kv.status, MLXB_ST_PAGE_RANGE);
    return nullptr;
  }
  if (pg < 0) return nullptr;
  const int kvw = kv.Hkv * kv.Dh;
  int c2 = n - kv.q_width;
  __nv_bfloat16* pool = kv.k_pool;
  if (c2 >= kvw) { c2 -= kvw; pool = kv.v_pool; }
  const int hh = c2 / kv.Dh, d = c2 - hh * kv.Dh;
  return pool + (((size_t)pg * kv.Hkv + hh) * kv.page + (pos % kv.page)) * kv.Dh + d;
}


// The same in two steps, for kernels that write many elements of a row: the row's part of the address once
// (element offset of head 0, dim 0 of the token's slot; -1 for a padding row or an index out of range, which
// sets the status bit) ...
__device__ __forceinline__ long long kv_row_base(const KvScatter& kv, int m) {
  const int r = kv.token_req[m];
  if (r < 0) return -1;
  const int pos = kv.positions[m];
  const int lp = pos / kv.page;
  const int pg = (pos >= 0 && lp < kv.max_pages) ? kv.block_table[(size_t)r * kv.max_pages + lp] : -2;
  if (pg == -2) {
    atomicOr(kv.status, MLXB_ST_POSITION_RANGE);
    return -1;
  }
  if (pg >= kv.n_pages) {
    atomicOr(kv.status, MLXB_ST_PAGE_RANGE);
    return -1;
  }
  if (pg < 0) return -1;
  return ((long long)pg * kv.Hkv * kv.page + (pos % kv.page)) * kv.Dh;
}

// ... and the column's part: where output column n (>= q_width) of that row goes.
__device__ __forceinline__ __nv_bfloat16* kv_slot_at(const KvScatter& kv, long long row_base, int n) {
  if (row_base < 0) return nullptr;
  const int kvw = kv.Hkv * kv.Dh;
  int c2 = n - kv.q_width;
  __nv_bfloat16* pool = kv.k_pool;
  if (c2 >= kvw) { c2 -= kvw; pool = kv.v_pool; }
  const int hh = c2 / kv.Dh, d = c2 - hh * kv.Dh;
  return pool + row_base + (long long)hh * kv.page * kv.Dh + d;
}
