// One pass over a dense attention mask that lets the prefill kernel skip key
// tiles nobody can see and read mask bytes only where a tile is mixed.
//
// The reference's op takes a dense bool mask [B, 1, L, L] for every call
// (src/minfer/kernels/torch_ext/csrc/cuda/flash_attn/op.cuh:28; its callers
// build a causal or a sliding-window one, test/kernels.py:242,276-278), so a
// drop-in cannot assume causality; classifying 128 x 128 tiles recovers the
// structure at the cost of reading the mask once (HBM-bound, ~1 byte per
// score instead of the B*H re-reads a per-head kernel would do).
#include "attn_internal.h"

namespace minfer_attn {

namespace {

constexpr int kTile = 128;

// grid (key tiles, query tiles, batch), 256 threads: thread t handles row t/2,
// 64 columns (half a tile row)
__global__ void __launch_bounds__(256) mask_classify_kernel(const uint8_t* __restrict__ mask, uint8_t* __restrict__ cls,
                                                            int seq_q, int seq_k) {
  const int kt = blockIdx.x, qt = blockIdx.y, b = blockIdx.z;
  const int row = qt * kTile + (threadIdx.x >> 1);
  const int col0 = kt * kTile + (threadIdx.x & 1) * 64;
  bool any = false, all = true;
  if (row < seq_q) {
    const uint8_t* p = mask + (static_cast<size_t>(b) * seq_q + row) * seq_k + col0;
    const int n = min(64, seq_k - col0);
    if (n == 64 && (reinterpret_cast<uintptr_t>(p) & 15) == 0) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(p) + i);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          // per byte: non-zero?  (b | (b >> 1) | ... folded into bit 0 of each byte)
          uint32_t x = w[k];
          x |= x >> 4;
          x |= x >> 2;
          x |= x >> 1;
          x &= 0x01010101u;
          any |= x != 0u;
          all &= x == 0x01010101u;
        }
      }
    } else {
      for (int i = 0; i < n; ++i) {
        const bool s = p[i] != 0;
        any |= s;
        all &= s;
      }
    }
  }
  const int any_cta = __syncthreads_or(any ? 1 : 0);
  const int all_cta = __syncthreads_and(all ? 1 : 0);
  if (threadIdx.x == 0)
    cls[(static_cast<size_t>(b) * gridDim.y + qt) * gridDim.x + kt] = any_cta ? (all_cta ? 1 : 2) : 0;
}

}  // namespace

cudaError_t launch_mask_classify(const uint8_t* mask, uint8_t* cls, int batch, int seq_q, int seq_k,
                                 cudaStream_t stream) {
  dim3 grid((seq_k + kTile - 1) / kTile, (seq_q + kTile - 1) / kTile, batch);
  mask_classify_kernel<<<grid, 256, 0, stream>>>(mask, cls, seq_q, seq_k);
  return cudaGetLastError();
}

}  // namespace minfer_attn
