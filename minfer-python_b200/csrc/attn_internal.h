// Internal declarations shared by the C-ABI layer and the kernels.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace minfer_attn {

// values a kernel writes to status[0] (MINFER_ATTN_STATUS_* of the public header)
constexpr int32_t kStatusWaitTimeout = 100;  // a bounded wait ran out
constexpr int32_t kStatusBadPage = 101;      // a block-table entry outside [0, n_pages)
constexpr int32_t kStatusBadPosition = 102;  // a cache row outside [0, max_len)

// Records `e` as the calling thread's latest CUDA result (what minfer_attn_last_cuda_error() reports)
// and maps it to MINFER_ATTN_OK / MINFER_ATTN_ECUDA.
int cuda_result(cudaError_t e);

// Kernel-side view of a prefill call (tensor maps travel separately).
struct PrefillArgs {
  void* out;
  const uint8_t* mask;
  const uint8_t* cls;     // per (batch, query tile, key tile) mask class, or null: see mask_classify.cu
  int32_t* status;
  int* counter;           // persistent kernel: work-item counter in the caller's workspace, or null (static order)
  int64_t out_stride[3];  // elements: batch, head, row
  int32_t batch, n_heads, n_kv_heads, seq_q, seq_k;
  int32_t group;          // query heads per kv head
  int32_t causal;
  int32_t mask_vec;       // mask rows may be read with 16-byte loads
  int32_t pair_heads;     // slots are two heads of one kv head (else two row tiles of one head)
  int32_t max_ctas;       // upper bound on the grid (0: one CTA per SM)
  int32_t n_peers;        // output replicas on other GPUs: every output tile is also stored through PeerMaps::m[0 .. n_peers)
  int32_t items_x, items_y;  // persistent kernel: work-item grid (query tile [pairs], head [pairs]); set by its launcher
  int32_t order_by_kv_set;   // persistent kernel, dynamic claiming: item order (see its launcher)
  float scale_log2;       // softmax scale * log2(e)
  // position (1..3) of the batch / head / row coordinate inside each tensor
  // map; coordinate 0 is always head_dim
  int32_t q_pos[3];
  int32_t kv_pos[3];
  int32_t out_pos[3];  // coordinate slots of the output tensor map (persistent kernel only)
};

// Output tensor maps of the replicas of `out` on other GPUs (PrefillArgs::n_peers of them are valid).
constexpr int kMaxPeerOut = 7;
struct PeerMaps {
  CUtensorMap m[kMaxPeerOut];
};

cudaError_t launch_prefill_persist(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                                   const CUtensorMap& to, const PeerMaps& peers, const PrefillArgs& a, int head_dim,
                                   bool bf16, cudaStream_t stream);

// Classifies every 128 x 128 tile of a dense [batch, 1, seq_q, seq_k] byte mask: 0 = no byte set,
// 1 = every in-range byte set, 2 = mixed.  cls is [batch, ceil(seq_q/128), ceil(seq_k/128)].
cudaError_t launch_mask_classify(const uint8_t* mask, uint8_t* cls, int batch, int seq_q, int seq_k,
                                 cudaStream_t stream);

// Kernel-side view of a RoPE + KV-append call.  Strides in elements.
struct RopeArgs {
  void* q;              // [batch, seq, n_heads, head_dim], rotated in place; may be null
  const void* k;        // [batch, seq, n_kv_heads, head_dim]; may be null
  const void* v;        // same shape as k; may be null
  void* k_cache;        // [batch, n_kv_heads, max_len, head_dim]; null: rotate k in place
  void* v_cache;
  const int32_t* start; // device [batch] first position per sequence, or null: start_pos
  int64_t q_stride[3];      // batch, token, head
  int64_t kv_stride[3];     // batch, token, head
  int64_t cache_stride[3];  // batch, head, row
  int32_t batch, seq, n_heads, n_kv_heads, head_dim, rotary_dim, start_pos;
  int32_t max_len;          // rows per (batch, head) of the caches: positions outside [0, max_len) are not written
  int32_t n_pages;          // paged cache: valid table entries are [0, n_pages)
  int32_t* status;          // optional device int32[4] for kStatusBadPage / kStatusBadPosition
  int32_t cache_q8;         // caches hold GGML Q8_0 blocks; cache_stride then in bytes (batch, head), rows contiguous
  float freq_base;
  const int32_t* block_table;  // paged cache: [batch, table_stride] page indices; cache_stride[0] is then per page
  int32_t page_size, table_stride;
  float freq[64];           // freq_base ^ (-2 i / rotary_dim) for i < rotary_dim / 2, filled by the launcher
};
cudaError_t launch_rope_append(const RopeArgs& a, bool bf16, bool neox, cudaStream_t stream);

// Kernel-side view of a decode call.
struct DecodeArgs {
  const void* q;
  const void* k;
  const void* v;
  const int32_t* lens;
  void* out;
  float* part_o;   // [batch, n_heads, n_split, head_dim] fp32, unnormalised
  float* part_ml;  // [batch, n_heads, n_split, 2] running max (log2 domain) and sum
  int64_t q_stride[2];
  int64_t kv_stride[3];   // elements; for a Q8_0 cache: bytes (batch, head), rows contiguous
  int64_t out_stride[2];
  int32_t batch, n_heads, n_kv_heads, max_len;
  int32_t group;
  int32_t chunk;    // keys per thread block
  int32_t n_split;  // ceil(max_len / chunk)
  float scale_log2;
  const int32_t* block_table;  // paged cache: [batch, table_stride] page indices; kv_stride[0] is then per page
  int32_t page_size, table_stride;
  int32_t n_pages;             // paged cache: valid table entries are [0, n_pages)
  int32_t* status;             // optional device int32[4] for kStatusBadPage
};

cudaError_t launch_decode(const DecodeArgs& a, int head_dim, bool bf16, bool q8, cudaStream_t stream);

}  // namespace minfer_attn
