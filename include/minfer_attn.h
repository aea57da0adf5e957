/*
 * minfer_attn.h — C ABI of the sm_100a attention library (libminfer_attn.so).
 *
 * Plain pointers and sizes only: no torch types cross this boundary.  Every
 * pointer named "device" must be a CUDA device pointer valid on the current
 * device; `stream` is a cudaStream_t passed as void*.  All entry points are
 * asynchronous with respect to the host (they enqueue work on `stream` and
 * return) and allocate no device memory: the caller owns inputs, outputs and
 * the optional workspace.
 *
 * Return value: 0 on success, otherwise one of the MINFER_ATTN_E* codes;
 * minfer_attn_strerror() gives a one-line description.  The library never
 * falls back to a CPU path; without a usable sm_100 device calls fail.
 *
 * Reference interface this replaces (dsuarez01/minfer-python):
 *   src/minfer/kernels/torch_ext/csrc/cuda/flash_attn/op.cuh:21-106
 *     (flash_attn_cuda: argument validation, stride capture, stream fetch,
 *      then an unimplemented launch)
 *   src/minfer/kernels/torch_ext/csrc/cuda/flash_attn/kernels/kernel.cuh:11-27
 *     (QKVStrides, HALF_MIN, the empty flash_attn_cuda_impl kernel)
 */
#ifndef MINFER_ATTN_H_
#define MINFER_ATTN_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MINFER_ATTN_ABI_VERSION 5

#define MINFER_ATTN_MAX_PEER_OUT 7   /* output replicas on other GPUs a prefill call can write (8-GPU node) */

/* element types of q/k/v/out */
#define MINFER_ATTN_F16  0
#define MINFER_ATTN_BF16 1

/* KV-cache formats (kv_format / cache_format fields) */
#define MINFER_ATTN_KV_16BIT 0  /* the same 16-bit type as q                                    */
#define MINFER_ATTN_KV_Q8_0  1  /* GGML Q8_0 blocks: 32 int8 + one fp16 scale = 34 bytes        */

/* status[0] values a kernel may leave in a caller-provided status word (device int32[4]) */
#define MINFER_ATTN_STATUS_WAIT_TIMEOUT 100  /* {code, blockIdx.x, blockIdx.y, wait site}                       */
#define MINFER_ATTN_STATUS_BAD_PAGE     101  /* {code, sequence, table index, entry}: entry outside [0, n_pages) */
#define MINFER_ATTN_STATUS_BAD_POSITION 102  /* {code, sequence, position, max_len}: row outside the cache       */

/* error codes */
#define MINFER_ATTN_OK            0
#define MINFER_ATTN_EINVAL        1  /* bad shape / stride / pointer / dtype        */
#define MINFER_ATTN_EUNSUPPORTED  2  /* valid request this build has no kernel for  */
#define MINFER_ATTN_ECUDA         3  /* a CUDA runtime / driver call failed          */
#define MINFER_ATTN_ENODEVICE     4  /* current device is not compute capability 10 */
#define MINFER_ATTN_EWORKSPACE    5  /* workspace missing or too small              */
#define MINFER_ATTN_ETOOLARGE     6  /* needs more scratch than the built-in buffer  */

/*
 * Prefill attention:  out = softmax(q k^T * scale + mask) v  with grouped-query
 * heads (kv head of query head h is h / (n_heads / n_kv_heads), i.e. the
 * repeat_interleave expansion the reference's callers apply before SDPA,
 * test/kernels.py:253-255).
 *
 * Layout: q,out are [batch, n_heads, seq_q, head_dim]; k,v are
 * [batch, n_kv_heads, seq_k, head_dim].  The innermost stride is 1; the three
 * outer strides are given in ELEMENTS, exactly the QKVStrides fields of
 * kernel.cuh:12-15 (the reference passes transposed views, so the strides are
 * arbitrary; each must be a multiple of 8 elements and the base pointers must
 * be 16-byte aligned).  k and v share one stride triple as op.cuh:46-48 demands.
 *
 * mask: NULL, or a contiguous [batch, 1, seq_q, seq_k] array of bytes where a
 * non-zero byte means "attend" (the reference's bool mask, op.cuh:28,50).
 * causal != 0 applies j <= i + (seq_k - seq_q) instead and ignores `mask`.
 * A row with no visible key yields zeros.
 *
 * softmax_scale == 0 selects 1/sqrt(head_dim) (the SDPA default used by
 * refs.py:55).  head_dim is 64 or 128.
 *
 * status: optional device int32[4].  A kernel that gives up a bounded wait
 * writes {MINFER_ATTN_STATUS_WAIT_TIMEOUT, blockIdx.x, blockIdx.y, site} there;
 * it is never written on success.  The caller zeroes it and reads it after
 * synchronising.  (The decode and RoPE structs carry the same kind of word for
 * bad block-table entries and out-of-range positions, see there.)
 */
typedef struct MinferAttnPrefillParams {
  const void*    q;
  const void*    k;
  const void*    v;
  void*          out;
  const uint8_t* mask;
  int32_t*       status;
  int64_t q_stride[3];    /* elements: batch, head, row */
  int64_t kv_stride[3];
  int64_t out_stride[3];
  int32_t batch;
  int32_t n_heads;
  int32_t n_kv_heads;
  int32_t seq_q;
  int32_t seq_k;
  int32_t head_dim;
  int32_t dtype;          /* MINFER_ATTN_F16 / MINFER_ATTN_BF16 */
  int32_t causal;
  float   softmax_scale;
  int32_t flags;          /* reserved, must be 0 */
  void*   workspace;      /* optional device scratch for dense masks, see below */
  size_t  workspace_bytes;
  int32_t max_ctas;       /* 0: one thread block per SM; n > 0: at most n thread blocks (leaves SMs free for
                             kernels of other streams, e.g. a collective that overlaps this call) */
  int32_t reserved;       /* must be 0 */
  /* Output replicas on other GPUs (multi-GPU prefill, the all-gather fused into the kernel): every output tile
   * is stored to `out` AND to each peer_out[i], a device pointer this process can write - the same tensor as
   * `out` (same shape and strides) in the memory of another GPU, mapped by CUDA IPC or peer access.  The
   * stores are plain (non-multicast) TMA tensor stores; they are complete when the kernel is, and the caller
   * orders the readers on the other GPUs after that (a barrier across the ranks).  Causal / unmasked calls
   * only.  n_peer_out = 0: none. */
  int32_t n_peer_out;
  int32_t reserved2;      /* must be 0 */
  void*   peer_out[MINFER_ATTN_MAX_PEER_OUT];
} MinferAttnPrefillParams;

int minfer_attn_prefill(const MinferAttnPrefillParams* params, void* stream);

/*
 * Optional scratch of a prefill call (device memory, 16-byte aligned).
 * The first 4 bytes serve as a counter from which the persistent thread blocks
 * claim work items (zeroed by the call on `stream`); 16 bytes are enough for a
 * causal / unmasked call, and without them the items are dealt out in a fixed
 * order.  Dense mask: when `workspace` holds at least the number of bytes returned
 * here, one pass over the mask classifies its 128 x 128 tiles (nothing visible /
 * everything visible / mixed) into the bytes after the counter; the attention
 * kernel then skips tiles nobody can see and reads mask bytes only for mixed
 * ones, so a dense causal or sliding-window mask costs about what the structure
 * it encodes costs.  Without it every tile is visited and masked byte by byte.
 * The result is the same with or without a workspace, only the time differs.
 * Calls that may overlap on the GPU need separate workspaces.  Returns 0 for
 * invalid sizes, else 16 + one byte per mask tile.
 */
size_t minfer_attn_prefill_workspace_bytes(int32_t batch, int32_t seq_q, int32_t seq_k);

/*
 * Decode attention over a padded KV cache (one query token per sequence).
 * No counterpart exists in the reference: its op insists on seq_q == seq_k
 * (op.cuh:76).  The cache layout is the one the reference's model skeleton
 * allocates, [batch, n_kv_heads, max_seq_len, head_dim] (src/minfer/core.py:105-127).
 *
 * q,out: [batch, n_heads, 1, head_dim] with element strides for batch and head.
 * k_cache,v_cache: [batch, n_kv_heads, max_len, head_dim], element strides for
 * batch, head, row; innermost stride 1.  lens: device int32[batch], sequence b
 * attends keys [0, lens[b]); entries beyond lens[b] are never read.  A
 * sequence with lens[b] == 0 yields zeros.
 *
 * The KV range of a sequence is cut into chunks of `chunk` keys, each handled
 * by its own thread block (split-KV); partial results go through `workspace`,
 * a device buffer of at least minfer_attn_decode_workspace_bytes() bytes that
 * the caller owns (any content); a second, small kernel merges the splits of
 * every sequence and writes `out`.  chunk == 0 lets the library choose; otherwise it must be a
 * positive multiple of 64.
 *
 * kv_format == MINFER_ATTN_KV_Q8_0: the caches hold GGML Q8_0 blocks (the
 * reference's block_q8_0, csrc/common/types.hpp:141-146): a cache row is
 * head_dim/32 blocks of 34 bytes, rows of one (batch, head) are contiguous,
 * kv_stride[0] and kv_stride[1] are then in BYTES (multiples of 16) and
 * kv_stride[2] is ignored; max_len must be even (a multiple of 4 for head_dim 64),
 * so that the rows of one (batch, head) end on a 16-byte boundary.  Every cached value is used as
 * (16-bit type)(q * d), the reference's dequant_row_q8_0 (csrc/quants/impl.cpp:
 * 1153-1166), so the result equals the 16-bit path run on the dequantised cache.
 *
 * Paged cache (block_table != NULL): the caches are pools of pages,
 * [n_pages, n_kv_heads, page_size, head_dim]; key j of sequence b lives in page
 * block_table[b * table_stride + j / page_size] at row j % page_size.
 * kv_stride[0] is then the stride between PAGES (elements, or bytes for Q8_0),
 * kv_stride[1] / [2] those of a head / row inside a page, page_size a positive
 * multiple of 16, max_len <= table_stride * page_size.  Only the table entries
 * below ceil(lens[b] / page_size) are read.  The reference's cache
 * (src/minfer/core.py:105-127) is the contiguous special case.
 */
typedef struct MinferAttnDecodeParams {
  const void*    q;
  const void*    k_cache;
  const void*    v_cache;
  const int32_t* lens;
  void*          out;
  void*          workspace;
  size_t         workspace_bytes;
  int64_t q_stride[2];    /* elements: batch, head */
  int64_t kv_stride[3];   /* elements: batch, head, row */
  int64_t out_stride[2];
  int32_t batch;
  int32_t n_heads;
  int32_t n_kv_heads;
  int32_t max_len;
  int32_t head_dim;
  int32_t dtype;
  int32_t chunk;
  float   softmax_scale;
  int32_t kv_format;      /* MINFER_ATTN_KV_16BIT (0) or MINFER_ATTN_KV_Q8_0 */
  const int32_t* block_table;  /* NULL: contiguous cache; else device int32[batch, table_stride] of page indices */
  int32_t page_size;      /* keys per page (multiple of 16); ignored without a block table */
  int32_t table_stride;   /* entries per sequence in block_table */
  int32_t n_pages;        /* pages in the pools (required with a block table): an entry outside [0, n_pages) is
                             never dereferenced - the kernel reads page 0 instead and reports it through status */
  int32_t flags;          /* reserved, must be 0 */
  int32_t* status;        /* optional device int32[4], see MINFER_ATTN_STATUS_BAD_PAGE; written only on error */
} MinferAttnDecodeParams;

int minfer_attn_decode(const MinferAttnDecodeParams* params, void* stream);

/* Bytes of workspace minfer_attn_decode() needs for this shape and chunk
 * (chunk == 0: the library's own choice).  Returns 0 for invalid arguments. */
size_t minfer_attn_decode_workspace_bytes(int32_t batch, int32_t n_heads,
                                          int32_t max_len, int32_t head_dim,
                                          int32_t chunk);

/* The chunk minfer_attn_decode() uses when params->chunk == 0. */
int32_t minfer_attn_decode_default_chunk(int32_t batch, int32_t n_kv_heads,
                                         int32_t max_len);

/*
 * Decode attention without any device allocation, for callers that cannot
 * allocate: a process that gave all device memory to its own pool at start-up,
 * or a decode loop that must never reach the allocator.  Same arguments and
 * results as minfer_attn_decode(), except that params->workspace and
 * params->workspace_bytes are ignored: the split-KV partials live in a fixed
 * MINFER_ATTN_STATIC_SCRATCH_BYTES array inside the library (each device that
 * loads the library holds that much memory until the process exits).
 *   - A shape whose partials need more than that is refused with
 *     MINFER_ATTN_ETOOLARGE and nothing is launched (the need is
 *     minfer_attn_decode_workspace_bytes() for the same arguments).
 *   - The first call on a device looks up the array's device address, and with
 *     the CUDA runtime's lazy module loading that first call (not loading the
 *     library) is also when the device reserves the array's bytes.  Make that
 *     first call - a small warm-up shape will do - before any stream capture
 *     begins on that device and BEFORE the process hands the rest of the
 *     device's memory to its own pool; a pool filled first leaves no room for
 *     the array and the call then fails with MINFER_ATTN_ECUDA
 *     (minfer_attn_last_cuda_error() names the cause).
 *   - All calls on a device share the one array, which keeps the last call's
 *     contents.  Nothing in it has to start at zero (every partial that is read
 *     was written earlier in the same call), but two calls whose kernels overlap
 *     on the GPU race on it: issue them on one stream, or order them with events.
 *   - The function calls neither cudaMalloc/cudaFree nor any allocating
 *     library routine.
 * This entry point has no counterpart in the reference.
 */
#define MINFER_ATTN_STATIC_SCRATCH_BYTES (32u << 20)
int minfer_attn_decode_static(const MinferAttnDecodeParams* params, void* stream);

/*
 * Rotary position embedding of q and k fused with the KV-cache append (the step
 * right before attention).  Reference semantics: il_rope / neox_rope,
 *   src/minfer/kernels/torch_ext/csrc/cuda/il_rope/op.cuh:21-59, kernel.cuh:9-39
 *   src/minfer/kernels/torch_ext/csrc/cuda/neox_rope/kernel.cuh:9-38
 * (one [B, L, H, D] tensor rotated in place per call); the cache layout
 * [batch, n_kv_heads, max_len, head_dim] is the one src/minfer/core.py:105-127
 * allocates.  The reference has no fused append.
 *
 * q [batch, seq, n_heads, head_dim] is rotated in place.  k, v
 * [batch, seq, n_kv_heads, head_dim]: with caches given, rotated k and plain v of
 * token l of sequence b are written to cache row start[b] + l (start: device
 * int32[batch], or NULL for the scalar start_pos); without caches k is rotated
 * in place and v is not touched.  Any of q / k / v may be NULL.  Strides are in
 * elements (batch, token, head for q/k/v; batch, head, row for the caches),
 * innermost stride 1, multiples of 8; pointers 16-byte aligned.  rotary_dim is
 * a multiple of 8 (16 for the neox style) and at most head_dim; head_dim is a
 * multiple of 8.  style: 0 = interleaved pairs, 1 = neox (two halves).
 * A position start[b] + l outside [0, max_len) is not written to the caches
 * (q is still rotated) and is reported through `status`; the scalar start_pos is
 * checked on the host.  The reference's kernels accept any even rotary_dim; this
 * one moves 16-byte chunks and therefore wants the granularity stated above.
 *
 * cache_format == MINFER_ATTN_KV_Q8_0: the caches hold Q8_0 blocks (layout as for
 * minfer_attn_decode; cache_stride[0..1] in bytes, [2] ignored): the row the
 * 16-bit cache would receive is quantised as the reference's quant_row_q8_0 does
 * (csrc/quants/impl.cpp:1169-1193).  Needs head_dim % 32 == 0, and for the neox
 * style rotary_dim % 64 == 0.
 */
typedef struct MinferRopeParams {
  void*          q;
  const void*    k;
  const void*    v;
  void*          k_cache;
  void*          v_cache;
  const int32_t* start;
  int64_t q_stride[3];
  int64_t kv_stride[3];
  int64_t cache_stride[3];
  int32_t batch;          /* batch * seq * head_dim / 8 must stay below 2^31 - 64 (EINVAL otherwise) */
  int32_t seq;
  int32_t n_heads;
  int32_t n_kv_heads;
  int32_t head_dim;
  int32_t rotary_dim;     /* <= 128 (MINFER_ATTN_EUNSUPPORTED beyond) */
  int32_t start_pos;
  int32_t max_len;
  int32_t dtype;
  int32_t style;
  float   freq_base;
  int32_t cache_format;   /* MINFER_ATTN_KV_16BIT (0) or MINFER_ATTN_KV_Q8_0 */
  const int32_t* block_table;  /* NULL, or the paged cache's int32[batch, table_stride] (see MinferAttnDecodeParams): */
  int32_t page_size;      /*   row start[b] + l goes to page block_table[b][pos / page_size], row pos % page_size; */
  int32_t table_stride;   /*   cache_stride[0] is then the stride between pages and page_size may be any value > 0 */
  int32_t n_pages;        /* pages in the pools (required with a block table); a table entry outside [0, n_pages)
                             is not followed: that row is not written and status reports it */
  int32_t flags;          /* reserved, must be 0 */
  int32_t* status;        /* optional device int32[4]: MINFER_ATTN_STATUS_BAD_PAGE / _BAD_POSITION; written only
                             on error */
} MinferRopeParams;

int minfer_attn_rope_append(const MinferRopeParams* params, void* stream);

const char* minfer_attn_strerror(int code);
/* Text of the CUDA error behind the calling thread's latest MINFER_ATTN_ECUDA
 * from a launch ("no error" if none). */
const char* minfer_attn_last_cuda_error(void);
int minfer_attn_abi_version(void);

#ifdef __cplusplus
}
#endif
#endif /* MINFER_ATTN_H_ */
