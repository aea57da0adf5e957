// Decode attention for callers that must not allocate device memory.
//
// minfer_attn_decode() needs a caller-provided workspace for its split-KV
// partials.  Some callers cannot provide one: a serving process that handed
// all of its device memory to a KV-cache pool at start-up (any later
// allocation fails; such a process makes its first call here BEFORE it fills
// the pool, see scratch_on_current_device), or a latency-critical decode loop that cannot afford the
// device-wide synchronisation an allocation may imply.  For them this file
// offers the same kernels with the partials kept in a fixed array that is part
// of the library image.  It has no counterpart in the reference.
#include "../../include/minfer_attn.h"
#include "attn_internal.h"

#include <cuda_runtime.h>

#include <mutex>

namespace {

// The scratch itself.  Every device that loads the library holds these bytes
// until the process exits.
static __device__ __align__(256) unsigned char g_decode_scratch[MINFER_ATTN_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
void* g_scratch_addr[kMaxDevices] = {};
std::mutex g_scratch_mu;

// In host code `g_decode_scratch` is only a handle for the runtime, not a
// device address; the address on the current device has to be looked up.  With
// lazy module loading this lookup is also the moment the device reserves the
// array, so it can fail for lack of memory: the result goes through the same
// last-error record as every other entry point.
int scratch_on_current_device(void** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return minfer_attn::cuda_result(e);
  if (dev < 0 || dev >= kMaxDevices) return MINFER_ATTN_EUNSUPPORTED;
  std::lock_guard<std::mutex> lock(g_scratch_mu);
  if (g_scratch_addr[dev] == nullptr) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_decode_scratch);
    if (e != cudaSuccess) return minfer_attn::cuda_result(e);
    if (ptr == nullptr) return minfer_attn::cuda_result(cudaErrorInvalidSymbol);
    g_scratch_addr[dev] = ptr;
  }
  *out = g_scratch_addr[dev];
  return MINFER_ATTN_OK;
}

}  // namespace

extern "C" int minfer_attn_decode_static(const MinferAttnDecodeParams* p, void* stream) {
  if (p == nullptr) return MINFER_ATTN_EINVAL;
  int32_t chunk = p->chunk;
  if (chunk == 0) chunk = minfer_attn_decode_default_chunk(p->batch, p->n_kv_heads, p->max_len);
  const size_t need = minfer_attn_decode_workspace_bytes(p->batch, p->n_heads, p->max_len, p->head_dim, chunk);
  if (need == 0) return p->head_dim != 64 && p->head_dim != 128 && p->batch > 0 && p->n_heads > 0 && p->max_len > 0
                            ? MINFER_ATTN_EUNSUPPORTED
                            : MINFER_ATTN_EINVAL;
  if (need > MINFER_ATTN_STATIC_SCRATCH_BYTES) return MINFER_ATTN_ETOOLARGE;
  void* scratch = nullptr;
  const int rc = scratch_on_current_device(&scratch);
  if (rc != MINFER_ATTN_OK) return rc;
  MinferAttnDecodeParams c = *p;
  c.workspace = scratch;
  c.workspace_bytes = MINFER_ATTN_STATIC_SCRATCH_BYTES;
  return minfer_attn_decode(&c, stream);
}
