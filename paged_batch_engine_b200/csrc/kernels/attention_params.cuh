// Arguments shared by the paged attention kernels (plain and tensor-core) and by the
// merge of split partial results.
#pragma once
#include <stdint.h>

struct AttnParams {
  const void* q;            // [T, H * hd]
  const void* k_cache;      // this layer's pages: [page][kv_head][page_tokens][hd]
  const void* v_cache;
  void* out;                // [T, H * hd]
  float* part_o;            // [split_rows, H, max_splits, hd] unnormalised partial sums
  float* part_ml;           // [split_rows, H, max_splits, 2] running maximum and sum
  const int32_t* q_start;   // [R] first batch row of the request
  const int32_t* q_len;     // [R] its rows in this step
  const int32_t* seq_len;   // [R] its context after this step
  const int32_t* block_table;  // [R, bt_stride] page of logical block i, -1: given back
  const int32_t* work;      // [num_work, 4]: request (-1: idle), row tile, split, number of splits
  const int32_t* tok_split_row;  // [T] row of the token in the partial buffers, or -1
  int bt_stride, num_heads, num_kv_heads, page_tokens;
  int window;               // 0: all keys; W: keys p-W+1..p
  int split_keys;           // keys per split, a multiple of the key tile
  int max_splits;
  int tile_rows;            // packed rows (query row x head of the group) per row tile
  float scale;
  int kinds;                // tensor-core kernel: bit 0 small row tiles present, bit 1 large ones (0: unknown);
                            // bit 2: few requests, small tiles go to the block-cooperative instance;
                            // bit 4 (set by the launcher): key tiles arrive as one tensor-map box a page
  int num_pages;            // pages of the cache tensors (0: unknown; key tiles then come row by row)
};

// What the fused decode kernel needs beyond AttnParams: it applies the bias and the rotary
// position encoding to the new token's query, key and value itself, writes the key and value
// into the cache, and merges its key splits inside a thread-block cluster.
struct AttnFusedParams {
  const void* qkv;            // [T, (H + 2*KV) * hd] the fused projection's output
  const float* bias;          // [(H + 2*KV) * hd] or null
  const int32_t* positions;   // [T]
  const int32_t* slots;       // [T]: page * page_tokens + offset of the new token
  const float* inv_freq;      // [hd / 2], pairs (i, i + hd/2)
  int num_requests;           // rows of the grid (requests beyond the live ones have q_len 0)
};

struct AttnMergeParams {
  const float* part_o;
  const float* part_ml;
  void* out;
  const int32_t* split_tokens;   // [split_rows] batch row of each split row
  const int32_t* split_counts;   // [split_rows] number of splits (<= 1: nothing to merge)
  int num_heads, head_dim, max_splits;
};
