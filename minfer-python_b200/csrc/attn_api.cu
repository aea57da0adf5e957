// C-ABI layer of libminfer_attn.so: argument validation, TMA tensor-map
// construction and kernel launches.  Mirrors the checks of the reference's
// launcher (src/minfer/kernels/torch_ext/csrc/cuda/flash_attn/op.cuh:32-103)
// on plain pointers and sizes.
#include "../../include/minfer_attn.h"
#include "attn_internal.h"

#include <atomic>

#include <algorithm>
#include <cmath>
#include <cstring>
#include <mutex>

namespace minfer_attn {
namespace {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// Is the current device compute capability 10.x?  Cached per device.
int check_device() {
  // 0 unknown, 1 ok, 2 wrong arch; atomics: several host threads may drive different devices
  static std::atomic<int> cached[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return MINFER_ATTN_ECUDA;
  if (dev < 64) {
    const int c = cached[dev].load(std::memory_order_acquire);
    if (c != 0) return c == 1 ? MINFER_ATTN_OK : MINFER_ATTN_ENODEVICE;
  }
  int major = 0;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return MINFER_ATTN_ECUDA;
  if (dev < 64) cached[dev].store((major == 10) ? 1 : 2, std::memory_order_release);
  return major == 10 ? MINFER_ATTN_OK : MINFER_ATTN_ENODEVICE;
}

// Tensor map over a [batch, heads, rows, head_dim] 16-bit tensor with element
// strides (s_b, s_h, s_r, 1).  The three outer dimensions are ordered by
// ascending stride; pos[] receives the coordinate slot (1..3) of batch, head
// and row.  Box = 64 elements x box_rows rows, 128-byte swizzle, zero fill.
int encode_tensor_map(CUtensorMap* tm, const void* base, bool bf16, int head_dim, int64_t batch, int64_t heads,
                      int64_t rows, const int64_t stride[3], int32_t pos[3], int box_rows) {
  EncodeTiledFn enc = get_encode_fn();
  if (enc == nullptr) return MINFER_ATTN_ECUDA;
  struct Dim {
    int64_t size, stride;
    int which;
  } dims[3] = {{batch, stride[0], 0}, {heads, stride[1], 1}, {rows, stride[2], 2}};
  // a dimension of extent 1 may carry any stride; give it one that encodes
  int64_t span = head_dim;
  for (auto& d : dims)
    if (d.size > 1) span = std::max<int64_t>(span, d.size * d.stride);
  for (auto& d : dims)
    if (d.size == 1) d.stride = span;
  std::stable_sort(dims, dims + 3, [](const Dim& x, const Dim& y) { return x.stride < y.stride; });
  cuuint64_t gdim[4] = {static_cast<cuuint64_t>(head_dim), 0, 0, 0};
  cuuint64_t gstr[3];
  cuuint32_t box[4] = {64, 1, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  for (int i = 0; i < 3; ++i) {
    gdim[i + 1] = static_cast<cuuint64_t>(dims[i].size);
    gstr[i] = static_cast<cuuint64_t>(dims[i].stride) * 2;
    pos[dims[i].which] = i + 1;
    if (dims[i].which == 2) box[i + 1] = static_cast<cuuint32_t>(box_rows);
  }
  CUresult r = enc(tm, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
                   const_cast<void*>(base), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? MINFER_ATTN_OK : MINFER_ATTN_EINVAL;
}

// A tensor map is a pure function of (base, type, extents, strides, box), and a decode loop or a
// benchmark calls with the same tensors over and over: keep the encoded maps in a small per-thread,
// direct-mapped table so that a repeated call costs a hash and a compare instead of four driver calls.
struct MapKey {
  int64_t base, batch, heads, rows, stride[3], misc;  // misc: head_dim | box_rows << 16 | bf16 << 32
};
struct MapEntry {
  MapKey key;
  CUtensorMap map;
  int32_t pos[3];
  bool valid;
};
constexpr int kMapCacheSize = 64;

int make_tensor_map(CUtensorMap* tm, const void* base, bool bf16, int head_dim, int64_t batch, int64_t heads,
                    int64_t rows, const int64_t stride[3], int32_t pos[3], int box_rows = 128) {
  alignas(64) static thread_local MapEntry cache[kMapCacheSize] = {};
  MapKey key;
  std::memset(&key, 0, sizeof(key));
  key.base = static_cast<int64_t>(reinterpret_cast<uintptr_t>(base));
  key.batch = batch;
  key.heads = heads;
  key.rows = rows;
  for (int i = 0; i < 3; ++i) key.stride[i] = stride[i];
  key.misc = static_cast<int64_t>(head_dim) | (static_cast<int64_t>(box_rows) << 16) | (static_cast<int64_t>(bf16) << 32);
  uint64_t h = 1469598103934665603ull;
  const uint64_t* w = reinterpret_cast<const uint64_t*>(&key);
  for (size_t i = 0; i < sizeof(key) / 8; ++i) h = (h ^ w[i]) * 1099511628211ull;
  MapEntry& e = cache[(h >> 20) % kMapCacheSize];
  if (e.valid && std::memcmp(&e.key, &key, sizeof(key)) == 0) {
    *tm = e.map;
    for (int i = 0; i < 3; ++i) pos[i] = e.pos[i];
    return MINFER_ATTN_OK;
  }
  const int rc = encode_tensor_map(tm, base, bf16, head_dim, batch, heads, rows, stride, pos, box_rows);
  if (rc != MINFER_ATTN_OK) return rc;
  e.key = key;
  e.map = *tm;
  for (int i = 0; i < 3; ++i) e.pos[i] = pos[i];
  e.valid = true;
  return MINFER_ATTN_OK;
}

thread_local cudaError_t g_last_cuda_error = cudaSuccess;

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

bool strides_ok(const int64_t* s, int n) {
  for (int i = 0; i < n; ++i)
    if (s[i] < 0 || (s[i] % 8) != 0) return false;
  return true;
}

int32_t default_chunk(int32_t batch, int32_t n_kv_heads, int32_t max_len) {
  int32_t c = 512;
  while (c > 64 && c >= 2 * max_len) c >>= 1;
  // few sequences and heads: shorter chunks, so that the grid still offers every SM two thread blocks (a decode
  // step of a small batch is a latency problem: each block then walks fewer key tiles in sequence)
  while (c > 128 && static_cast<int64_t>(batch) * n_kv_heads * ((max_len + c - 1) / c) < 2 * 148) c >>= 1;
  return c;
}

}  // namespace

int cuda_result(cudaError_t e) {
  g_last_cuda_error = e;
  if (e != cudaSuccess) (void)cudaGetLastError();  // clear the runtime's (non-sticky) error state
  return e == cudaSuccess ? MINFER_ATTN_OK : MINFER_ATTN_ECUDA;
}

}  // namespace minfer_attn

using namespace minfer_attn;

extern "C" {

int minfer_attn_abi_version(void) { return MINFER_ATTN_ABI_VERSION; }

const char* minfer_attn_last_cuda_error(void) { return cudaGetErrorString(g_last_cuda_error); }

const char* minfer_attn_strerror(int code) {
  switch (code) {
    case MINFER_ATTN_OK: return "ok";
    case MINFER_ATTN_EINVAL: return "invalid argument (shape, stride, alignment, dtype or null pointer)";
    case MINFER_ATTN_EUNSUPPORTED: return "unsupported configuration (head_dim must be 64 or 128, group <= 16)";
    case MINFER_ATTN_ECUDA: return "a CUDA runtime or driver call failed";
    case MINFER_ATTN_ENODEVICE: return "current CUDA device is not compute capability 10.x (sm_100)";
    case MINFER_ATTN_EWORKSPACE: return "decode workspace missing or too small";
    case MINFER_ATTN_ETOOLARGE: return "shape needs more scratch than the library's built-in static buffer holds";
    default: return "unknown error code";
  }
}

int minfer_attn_prefill(const MinferAttnPrefillParams* p, void* stream) {
  if (p == nullptr || p->q == nullptr || p->k == nullptr || p->v == nullptr || p->out == nullptr)
    return MINFER_ATTN_EINVAL;
  if (p->batch <= 0 || p->n_heads <= 0 || p->n_kv_heads <= 0 || p->seq_q <= 0 || p->seq_k <= 0)
    return MINFER_ATTN_EINVAL;
  if (p->n_heads % p->n_kv_heads != 0) return MINFER_ATTN_EINVAL;
  if (p->dtype != MINFER_ATTN_F16 && p->dtype != MINFER_ATTN_BF16) return MINFER_ATTN_EINVAL;
  if (p->head_dim != 64 && p->head_dim != 128) return MINFER_ATTN_EUNSUPPORTED;
  if (p->causal && p->seq_k < p->seq_q) return MINFER_ATTN_EINVAL;
  if (!aligned16(p->q) || !aligned16(p->k) || !aligned16(p->v) || !aligned16(p->out)) return MINFER_ATTN_EINVAL;
  if (!strides_ok(p->q_stride, 3) || !strides_ok(p->kv_stride, 3) || !strides_ok(p->out_stride, 3))
    return MINFER_ATTN_EINVAL;
  if (!(p->softmax_scale >= 0.f)) return MINFER_ATTN_EINVAL;
  if (p->batch > 65535 || p->n_heads > 65535) return MINFER_ATTN_EUNSUPPORTED;
  if (p->flags != 0 || p->reserved != 0 || p->reserved2 != 0) return MINFER_ATTN_EUNSUPPORTED;
  if (p->max_ctas < 0) return MINFER_ATTN_EINVAL;
  if (p->n_peer_out < 0 || p->n_peer_out > MINFER_ATTN_MAX_PEER_OUT) return MINFER_ATTN_EINVAL;
  for (int i = 0; i < p->n_peer_out; ++i)
    if (p->peer_out[i] == nullptr || !aligned16(p->peer_out[i])) return MINFER_ATTN_EINVAL;
  // the fused output exchange exists for the causal / unmasked form (a dense-mask call may write rows directly)
  if (p->n_peer_out > 0 && !p->causal && p->mask != nullptr) return MINFER_ATTN_EUNSUPPORTED;
  // the masked kernel's tile list holds 1024 key tiles
  if (!p->causal && p->mask != nullptr && p->seq_k > 128 * 1024) return MINFER_ATTN_EUNSUPPORTED;
  int rc = check_device();
  if (rc != MINFER_ATTN_OK) return rc;

  const bool bf16 = p->dtype == MINFER_ATTN_BF16;
  PrefillArgs a{};
  alignas(64) CUtensorMap tq, tk, tv;
  rc = make_tensor_map(&tq, p->q, bf16, p->head_dim, p->batch, p->n_heads, p->seq_q, p->q_stride, a.q_pos);
  if (rc != MINFER_ATTN_OK) return rc;
  rc = make_tensor_map(&tk, p->k, bf16, p->head_dim, p->batch, p->n_kv_heads, p->seq_k, p->kv_stride, a.kv_pos);
  if (rc != MINFER_ATTN_OK) return rc;
  int32_t vpos[3];
  rc = make_tensor_map(&tv, p->v, bf16, p->head_dim, p->batch, p->n_kv_heads, p->seq_k, p->kv_stride, vpos);
  if (rc != MINFER_ATTN_OK) return rc;

  // output map of the persistent kernel's epilogue: one softmax warp stores 32 rows x 64 columns at a time
  alignas(64) CUtensorMap to;
  rc = make_tensor_map(&to, p->out, bf16, p->head_dim, p->batch, p->n_heads, p->seq_q, p->out_stride, a.out_pos, 32);
  if (rc != MINFER_ATTN_OK) return rc;

  static_assert(MINFER_ATTN_MAX_PEER_OUT == kMaxPeerOut, "peer output count");
  alignas(64) PeerMaps peers;
  for (int i = 0; i < kMaxPeerOut; ++i) {
    // unused entries repeat the local map, so that the kernel's parameter block never holds garbage
    int32_t pos_unused[3];
    void* base = i < p->n_peer_out ? p->peer_out[i] : p->out;
    rc = make_tensor_map(&peers.m[i], base, bf16, p->head_dim, p->batch, p->n_heads, p->seq_q, p->out_stride, pos_unused, 32);
    if (rc != MINFER_ATTN_OK) return rc;
  }
  a.n_peers = p->n_peer_out;

  a.out = p->out;
  a.mask = p->causal ? nullptr : p->mask;
  a.cls = nullptr;
  a.counter = nullptr;
  // the first word of a (16-byte aligned) workspace is the work-item counter of the persistent kernel;
  // the tile classes of a dense mask follow at byte 16
  if (p->workspace != nullptr && p->workspace_bytes >= 16 && aligned16(p->workspace))
    a.counter = static_cast<int*>(p->workspace);
  if (a.mask != nullptr) {
    const size_t need = minfer_attn_prefill_workspace_bytes(p->batch, p->seq_q, p->seq_k);
    if (a.counter != nullptr && p->workspace_bytes >= need) {
      uint8_t* cls = static_cast<uint8_t*>(p->workspace) + 16;
      cudaError_t ce = launch_mask_classify(a.mask, cls, p->batch, p->seq_q, p->seq_k, static_cast<cudaStream_t>(stream));
      if (ce != cudaSuccess) return cuda_result(ce);
      a.cls = cls;
    }
  }
  a.status = p->status;
  for (int i = 0; i < 3; ++i) a.out_stride[i] = p->out_stride[i];
  a.batch = p->batch;
  a.n_heads = p->n_heads;
  a.n_kv_heads = p->n_kv_heads;
  a.seq_q = p->seq_q;
  a.seq_k = p->seq_k;
  a.group = p->n_heads / p->n_kv_heads;
  a.causal = p->causal ? 1 : 0;
  a.mask_vec = (a.mask != nullptr && aligned16(a.mask) && (p->seq_k % 16) == 0) ? 1 : 0;
  const float scale = p->softmax_scale > 0.f ? p->softmax_scale : 1.0f / std::sqrt(static_cast<float>(p->head_dim));
  a.scale_log2 = scale * 1.4426950408889634f;

  a.pair_heads = (a.group % 2 == 0) ? 1 : 0;
  a.max_ctas = p->max_ctas;
  return cuda_result(launch_prefill_persist(tq, tk, tv, to, peers, a, p->head_dim, bf16, static_cast<cudaStream_t>(stream)));
}

size_t minfer_attn_prefill_workspace_bytes(int32_t batch, int32_t seq_q, int32_t seq_k) {
  if (batch <= 0 || seq_q <= 0 || seq_k <= 0) return 0;
  const size_t cls = static_cast<size_t>(batch) * ((seq_q + 127) / 128) * ((seq_k + 127) / 128);
  return 16 + cls;  // the work-item counter, then the tile classes of a dense mask
}

int minfer_attn_rope_append(const MinferRopeParams* p, void* stream) {
  if (p == nullptr) return MINFER_ATTN_EINVAL;
  if (p->q == nullptr && p->k == nullptr && p->v == nullptr) return MINFER_ATTN_EINVAL;
  if (p->batch <= 0 || p->seq <= 0 || p->head_dim <= 0 || p->head_dim % 8 != 0) return MINFER_ATTN_EINVAL;
  // the kernel indexes (token, 16-byte chunk) pairs in 32 bits
  if (static_cast<long long>(p->batch) * p->seq * (p->head_dim / 8) >= (1ll << 31) - 64) return MINFER_ATTN_EINVAL;
  if (p->dtype != MINFER_ATTN_F16 && p->dtype != MINFER_ATTN_BF16) return MINFER_ATTN_EINVAL;
  if (p->style != 0 && p->style != 1) return MINFER_ATTN_EINVAL;
  if (p->rotary_dim < 0 || p->rotary_dim > p->head_dim || p->rotary_dim % (p->style == 1 ? 16 : 8) != 0)
    return MINFER_ATTN_EINVAL;
  if (!(p->freq_base > 0.f)) return MINFER_ATTN_EINVAL;
  if (p->rotary_dim > 128) return MINFER_ATTN_EUNSUPPORTED;  // the launcher's frequency table holds 64 entries
  if (p->q != nullptr && (p->n_heads <= 0 || !aligned16(p->q) || !strides_ok(p->q_stride, 3))) return MINFER_ATTN_EINVAL;
  if ((p->k != nullptr || p->v != nullptr) && (p->n_kv_heads <= 0 || !strides_ok(p->kv_stride, 3)))
    return MINFER_ATTN_EINVAL;
  if ((p->k != nullptr && !aligned16(p->k)) || (p->v != nullptr && !aligned16(p->v))) return MINFER_ATTN_EINVAL;
  if ((p->k_cache == nullptr) != (p->v_cache == nullptr)) return MINFER_ATTN_EINVAL;
  const bool cq8 = p->cache_format == MINFER_ATTN_KV_Q8_0;
  if (p->cache_format != MINFER_ATTN_KV_16BIT && !cq8) return MINFER_ATTN_EINVAL;
  if (cq8 && (p->k_cache == nullptr || p->head_dim % 32 != 0 || (p->style == 1 && p->rotary_dim % 64 != 0)))
    return MINFER_ATTN_EINVAL;
  if (p->k_cache != nullptr) {
    if (p->k == nullptr || p->v == nullptr) return MINFER_ATTN_EINVAL;
    if (!aligned16(p->k_cache) || !aligned16(p->v_cache)) return MINFER_ATTN_EINVAL;
    if (cq8 ? (p->cache_stride[0] < 0 || p->cache_stride[1] < 0 || p->cache_stride[0] % 2 != 0 || p->cache_stride[1] % 2 != 0)
            : !strides_ok(p->cache_stride, 3))
      return MINFER_ATTN_EINVAL;
    if (p->max_len <= 0) return MINFER_ATTN_EINVAL;
    if (p->start == nullptr && (p->start_pos < 0 || p->start_pos + p->seq > p->max_len)) return MINFER_ATTN_EINVAL;
    if (p->block_table != nullptr) {
      if (p->page_size <= 0 || p->table_stride <= 0 || p->n_pages <= 0 ||
          (reinterpret_cast<uintptr_t>(p->block_table) & 3) != 0)
        return MINFER_ATTN_EINVAL;
      if (static_cast<int64_t>(p->page_size) * p->table_stride < p->max_len) return MINFER_ATTN_EINVAL;
    }
  } else if (p->block_table != nullptr) {
    return MINFER_ATTN_EINVAL;
  }
  if (p->start == nullptr && p->start_pos < 0) return MINFER_ATTN_EINVAL;
  if (p->flags != 0) return MINFER_ATTN_EUNSUPPORTED;
  if (p->status != nullptr && (reinterpret_cast<uintptr_t>(p->status) & 3) != 0) return MINFER_ATTN_EINVAL;
  int rc = check_device();
  if (rc != MINFER_ATTN_OK) return rc;
  RopeArgs a{};
  a.q = p->q;
  a.k = p->k;
  a.v = p->v;
  a.k_cache = p->k_cache;
  a.v_cache = p->v_cache;
  a.start = p->start;
  for (int i = 0; i < 3; ++i) {
    a.q_stride[i] = p->q_stride[i];
    a.kv_stride[i] = p->kv_stride[i];
    a.cache_stride[i] = p->cache_stride[i];
  }
  a.batch = p->batch;
  a.seq = p->seq;
  a.n_heads = p->n_heads;
  a.n_kv_heads = p->n_kv_heads;
  a.head_dim = p->head_dim;
  a.rotary_dim = p->rotary_dim;
  a.start_pos = p->start_pos;
  a.max_len = p->max_len;
  a.n_pages = p->block_table != nullptr ? p->n_pages : 0;
  a.status = p->status;
  a.freq_base = p->freq_base;
  a.cache_q8 = cq8 ? 1 : 0;
  a.block_table = p->block_table;
  a.page_size = p->block_table != nullptr ? p->page_size : 0;
  a.table_stride = p->block_table != nullptr ? p->table_stride : 0;
  return cuda_result(launch_rope_append(a, p->dtype == MINFER_ATTN_BF16, p->style == 1, static_cast<cudaStream_t>(stream)));
}

int32_t minfer_attn_decode_default_chunk(int32_t batch, int32_t n_kv_heads, int32_t max_len) {
  if (batch <= 0 || n_kv_heads <= 0 || max_len <= 0) return 0;
  return default_chunk(batch, n_kv_heads, max_len);
}

size_t minfer_attn_decode_workspace_bytes(int32_t batch, int32_t n_heads, int32_t max_len, int32_t head_dim,
                                          int32_t chunk) {
  if (batch <= 0 || n_heads <= 0 || max_len <= 0 || (head_dim != 64 && head_dim != 128)) return 0;
  if (chunk == 0) chunk = default_chunk(batch, 1, max_len);
  if (chunk < 64 || chunk % 64 != 0) return 0;
  const size_t n_split = (static_cast<size_t>(max_len) + chunk - 1) / chunk;
  return static_cast<size_t>(batch) * n_heads * n_split * (static_cast<size_t>(head_dim) + 2) * sizeof(float);
}

int minfer_attn_decode(const MinferAttnDecodeParams* p, void* stream) {
  if (p == nullptr || p->q == nullptr || p->k_cache == nullptr || p->v_cache == nullptr || p->lens == nullptr ||
      p->out == nullptr)
    return MINFER_ATTN_EINVAL;
  if (p->batch <= 0 || p->n_heads <= 0 || p->n_kv_heads <= 0 || p->max_len <= 0) return MINFER_ATTN_EINVAL;
  if (p->n_heads % p->n_kv_heads != 0) return MINFER_ATTN_EINVAL;
  if (p->dtype != MINFER_ATTN_F16 && p->dtype != MINFER_ATTN_BF16) return MINFER_ATTN_EINVAL;
  if (p->head_dim != 64 && p->head_dim != 128) return MINFER_ATTN_EUNSUPPORTED;
  const int group = p->n_heads / p->n_kv_heads;
  if (group > 16) return MINFER_ATTN_EUNSUPPORTED;
  if (!aligned16(p->q) || !aligned16(p->k_cache) || !aligned16(p->v_cache) || !aligned16(p->out))
    return MINFER_ATTN_EINVAL;
  const bool q8 = p->kv_format == MINFER_ATTN_KV_Q8_0;
  if (p->kv_format != MINFER_ATTN_KV_16BIT && !q8) return MINFER_ATTN_EINVAL;
  if (!strides_ok(p->q_stride, 2) || !strides_ok(p->out_stride, 2)) return MINFER_ATTN_EINVAL;
  if (q8) {
    if (p->kv_stride[0] < 0 || p->kv_stride[1] < 0 || p->kv_stride[0] % 16 != 0 || p->kv_stride[1] % 16 != 0)
      return MINFER_ATTN_EINVAL;
    // the rows of one (batch, head) must end on a 16-byte boundary (rows are 136 / 68 bytes)
    if (p->max_len % (p->head_dim == 64 ? 4 : 2) != 0) return MINFER_ATTN_EINVAL;
  } else if (!strides_ok(p->kv_stride, 3)) {
    return MINFER_ATTN_EINVAL;
  }
  if (!(p->softmax_scale >= 0.f)) return MINFER_ATTN_EINVAL;
  if (p->batch > 65535 || p->n_kv_heads > 65535) return MINFER_ATTN_EUNSUPPORTED;
  if (p->block_table != nullptr) {
    if (p->page_size <= 0 || p->page_size % 16 != 0 || p->table_stride <= 0 || p->n_pages <= 0)
      return MINFER_ATTN_EINVAL;
    if (static_cast<int64_t>(p->table_stride) * p->page_size < p->max_len) return MINFER_ATTN_EINVAL;
    if ((reinterpret_cast<uintptr_t>(p->block_table) & 3) != 0) return MINFER_ATTN_EINVAL;
  }
  if (p->flags != 0) return MINFER_ATTN_EUNSUPPORTED;
  if (p->status != nullptr && (reinterpret_cast<uintptr_t>(p->status) & 3) != 0) return MINFER_ATTN_EINVAL;
  int32_t chunk = p->chunk;
  if (chunk == 0) chunk = default_chunk(p->batch, p->n_kv_heads, p->max_len);
  if (chunk < 64 || chunk % 64 != 0) return MINFER_ATTN_EINVAL;
  const size_t need = minfer_attn_decode_workspace_bytes(p->batch, p->n_heads, p->max_len, p->head_dim, chunk);
  if (p->workspace == nullptr || p->workspace_bytes < need || !aligned16(p->workspace)) return MINFER_ATTN_EWORKSPACE;
  int rc = check_device();
  if (rc != MINFER_ATTN_OK) return rc;

  DecodeArgs a{};
  a.q = p->q;
  a.k = p->k_cache;
  a.v = p->v_cache;
  a.lens = p->lens;
  a.out = p->out;
  a.batch = p->batch;
  a.n_heads = p->n_heads;
  a.n_kv_heads = p->n_kv_heads;
  a.max_len = p->max_len;
  a.group = group;
  a.chunk = chunk;
  a.n_split = (p->max_len + chunk - 1) / chunk;
  a.part_o = static_cast<float*>(p->workspace);
  a.part_ml = a.part_o + static_cast<size_t>(p->batch) * p->n_heads * a.n_split * p->head_dim;
  for (int i = 0; i < 2; ++i) {
    a.q_stride[i] = p->q_stride[i];
    a.out_stride[i] = p->out_stride[i];
  }
  for (int i = 0; i < 3; ++i) a.kv_stride[i] = p->kv_stride[i];
  const float scale = p->softmax_scale > 0.f ? p->softmax_scale : 1.0f / std::sqrt(static_cast<float>(p->head_dim));
  a.scale_log2 = scale * 1.4426950408889634f;
  a.block_table = p->block_table;
  a.page_size = p->block_table != nullptr ? p->page_size : 0;
  a.table_stride = p->block_table != nullptr ? p->table_stride : 0;
  a.n_pages = p->block_table != nullptr ? p->n_pages : 0;
  a.status = p->status;

  cudaError_t e = launch_decode(a, p->head_dim, p->dtype == MINFER_ATTN_BF16, q8, static_cast<cudaStream_t>(stream));
  return cuda_result(e);
}

}  // extern "C"
