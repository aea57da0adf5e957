// Rotary position embedding of q and k fused with the KV-cache append: the step
// immediately before attention.  HBM-bound and elementwise.
//
// Semantics follow the reference's RoPE ops
// (src/minfer/kernels/torch_ext/csrc/cuda/il_rope/kernel.cuh:9-39 and
// .../neox_rope/kernel.cuh:9-38; oracles src/minfer/kernels/refs.py:12-47):
//   freq_i  = freq_base ^ (-2 i / rotary_dim)            (fp32)
//   angle   = (position) * freq_i                        (fp32)
//   interleaved: (x[2i], x[2i+1])            rotated by angle_i
//   neox:        (x[i],  x[i + rotary_dim/2]) rotated by angle_i
// for i < rotary_dim/2, elements beyond rotary_dim untouched, math in fp32,
// result rounded to the 16-bit type.  The reference rotates one [B, L, H, D]
// tensor in place per call; here one launch rotates q in place, rotates k into
// the cache [B, Hkv, Lmax, D] at row position and copies v into its cache, so
// q, k and v are each read once and the [B, L, H, D] -> [B, H, L, D] transposition
// of k/v costs nothing extra (the cache layout is the reference's,
// src/minfer/core.py:105-127).
//
// With cache_q8 the caches hold GGML Q8_0 blocks instead (the reference's block_q8_0,
// csrc/common/types.hpp:141-146): the row that the 16-bit cache would receive (rotated k,
// plain v, rounded to the 16-bit type) is quantised as the reference's quant_row_q8_0 does
// (csrc/quants/impl.cpp:1169-1193): d = max|x| / 127, q = roundf(x / d), 32 values per block.
// The four threads that own one block's four chunks agree on the maximum with two shuffles.
//
// Thread mapping: a thread owns one token and one 16-byte chunk of head_dim
// (neox: the chunk and its partner chunk) and walks a slice of the token's rows
// (query heads, k heads, v heads), four rows at a time with all loads issued
// first; the sin/cos of its 4 (8) angles are computed once per thread.
#include "../../include/minfer_attn.h"
#include "attn_internal.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace minfer_attn {

namespace {

template <bool BF16>
__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if constexpr (BF16) {
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    } else {
      const __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
      const float2 t = __half22float2(h);
      f[2 * i] = t.x;
      f[2 * i + 1] = t.y;
    }
  }
}

template <bool BF16>
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if constexpr (BF16) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
      w[i] = *reinterpret_cast<const uint32_t*>(&h);
    } else {
      const __half2 h = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
      w[i] = *reinterpret_cast<const uint32_t*>(&h);
    }
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

// Quantise 8 values (this thread's quarter of a 32-value block) and store them into the Q8_0
// block at `blk`; `part` = which quarter.  All four threads of the block call this together.
__device__ __forceinline__ void store_q8_quarter(const float (&x)[8], uint8_t* blk, int part) {
  float amax = 0.f;
#pragma unroll
  for (int t = 0; t < 8; ++t) amax = fmaxf(amax, fabsf(x[t]));
  const unsigned mask = __activemask();
  amax = fmaxf(amax, __shfl_xor_sync(mask, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(mask, amax, 2));
  const float d = amax / 127.f;
  const float id = d ? 1.0f / d : 0.0f;
  if (part == 0) *reinterpret_cast<__half*>(blk) = __float2half_rn(d);
  uint16_t* q16 = reinterpret_cast<uint16_t*>(blk + 2 + part * 8);  // 2-byte aligned
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    const int q0 = static_cast<int>(roundf(x[2 * t] * id));
    const int q1 = static_cast<int>(roundf(x[2 * t + 1] * id));
    q16[t] = static_cast<uint16_t>((q0 & 0xFF) | ((q1 & 0xFF) << 8));
  }
}

// values as the 16-bit cache would hold them (rounded to the 16-bit type), back in fp32
template <bool BF16>
__device__ __forceinline__ void round16(float (&x)[8]) {
#pragma unroll
  for (int t = 0; t < 8; ++t) {
    if constexpr (BF16) x[t] = __bfloat162float(__float2bfloat16_rn(x[t]));
    else x[t] = __half2float(__float2half_rn(x[t]));
  }
}

// kNeox = false: interleaved pairs; true: two halves.
template <bool BF16, bool kNeox>
__global__ void __launch_bounds__(256) rope_append_kernel(const RopeArgs a) {
  const int chunks = a.head_dim / 8;                 // 16-byte chunks per head row
  const int rot_chunks = a.rotary_dim / 8;
  const int work_chunks = kNeox ? chunks - rot_chunks / 2 : chunks;  // neox: a thread takes a chunk and its partner
  const long long gid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long token = gid / work_chunks;
  if (token >= static_cast<long long>(a.batch) * a.seq) return;
  int c = static_cast<int>(gid % work_chunks);
  // neox work item c: c < rot_chunks/2 -> rotated pair (c, c + rot_chunks/2); else passthrough chunk c + rot_chunks/2
  int c2 = -1;
  bool rotate;
  if (kNeox) {
    if (c < rot_chunks / 2) {
      c2 = c + rot_chunks / 2;
      rotate = true;
    } else {
      c += rot_chunks / 2;
      rotate = false;
    }
  } else {
    rotate = c < rot_chunks;
  }
  const int b = static_cast<int>(token / a.seq);
  const int l = static_cast<int>(token % a.seq);
  const int pos = (a.start ? a.start[b] : a.start_pos) + l;
  // where the row of position `pos` starts inside a cache, in units of the cache strides, head offset excluded:
  // contiguous [batch][head][row] caches, or a pool of pages reached through the block table
  size_t cb = static_cast<size_t>(b);
  int crow = pos;
  // A position outside the cache, or a table entry outside the pools, is never written: the row is
  // dropped (q is still rotated) and the first such event is reported through the status word.  The
  // threads of one token decide alike, so the shuffles of the Q8_0 path stay among live threads.
  bool cache_ok = a.k_cache != nullptr;
  if (cache_ok && (pos < 0 || pos >= a.max_len)) {
    cache_ok = false;
    if (a.status != nullptr && atomicCAS(a.status, 0, kStatusBadPosition) == 0) {
      a.status[1] = b;
      a.status[2] = pos;
      a.status[3] = a.max_len;
    }
  }
  if (cache_ok && a.block_table != nullptr) {
    const int slot = pos / a.page_size;
    const int page = a.block_table[static_cast<size_t>(b) * a.table_stride + slot];
    if (static_cast<unsigned>(page) >= static_cast<unsigned>(a.n_pages)) {
      cache_ok = false;
      if (a.status != nullptr && atomicCAS(a.status, 0, kStatusBadPage) == 0) {
        a.status[1] = b;
        a.status[2] = slot;
        a.status[3] = page;
      }
    }
    cb = static_cast<size_t>(page);
    crow = pos % a.page_size;
  }
  const bool to_cache = a.k_cache != nullptr;  // the call appends (as opposed to rotating k in place)

  float cs[8], sn[8];
  if (rotate) {
    const int n_ang = kNeox ? 8 : 4;
    const int i0 = kNeox ? 8 * c : 4 * c;
#pragma unroll
    for (int t = 0; t < 8; ++t) {
      if (t < n_ang) {
        const float freq = powf(a.freq_base, -2.0f * static_cast<float>(i0 + t) / static_cast<float>(a.rotary_dim));
        const float ang = static_cast<float>(pos) * freq;
        sincosf(ang, &sn[t], &cs[t]);
      }
    }
  }

  const int q_row_bytes = (a.head_dim / 32) * 34;  // a Q8_0 cache row

  const size_t co = static_cast<size_t>(c) * 16, co2 = static_cast<size_t>(c2 < 0 ? 0 : c2) * 16;
  // The rows of this token - its query heads, then its k heads, then its v heads - are dealt out over
  // gridDim.y slices, and a thread takes its rows four at a time, all loads first: a thread that walked
  // every head alone, one dependent load at a time, left the memory system idle (decode-sized calls took
  // tens of microseconds, prefill-sized ones reached 0.64 of the copy bandwidth).
  // The row list is the same for every thread of the launch (the threads that share a Q8_0 block must
  // meet in the same row at the same step); what differs per thread is which kinds of row it has work for.
  const bool do_q = rotate;
  const bool do_k = to_cache ? cache_ok : rotate;
  const bool do_v = cache_ok;
  const int n_q = a.q != nullptr ? a.n_heads : 0;
  const int n_k = a.k != nullptr ? a.n_kv_heads : 0;
  const int n_rows = n_q + n_k + ((a.v != nullptr && a.v_cache != nullptr) ? a.n_kv_heads : 0);
  const uint8_t* q_base = reinterpret_cast<const uint8_t*>(a.q) + 2 * (static_cast<size_t>(b) * a.q_stride[0] + static_cast<size_t>(l) * a.q_stride[1]);
  const uint8_t* k_base = reinterpret_cast<const uint8_t*>(a.k) + 2 * (static_cast<size_t>(b) * a.kv_stride[0] + static_cast<size_t>(l) * a.kv_stride[1]);
  const uint8_t* v_base = reinterpret_cast<const uint8_t*>(a.v) + 2 * (static_cast<size_t>(b) * a.kv_stride[0] + static_cast<size_t>(l) * a.kv_stride[1]);
  // source row of combined row index r (kind 0 = q, 1 = k, 2 = v) and its head
  auto row_of = [&](int r, int& kind, int& h) -> const uint8_t* {
    if (r < n_q) {
      kind = 0;
      h = r;
      return q_base + 2 * static_cast<size_t>(h) * a.q_stride[2];
    }
    if (r < n_q + n_k) {
      kind = 1;
      h = r - n_q;
      return k_base + 2 * static_cast<size_t>(h) * a.kv_stride[2];
    }
    kind = 2;
    h = r - n_q - n_k;
    return v_base + 2 * static_cast<size_t>(h) * a.kv_stride[2];
  };
  const int n_slices = static_cast<int>(gridDim.y);
  for (int r0 = static_cast<int>(blockIdx.y); r0 < n_rows; r0 += 4 * n_slices) {
    const uint8_t* src[4];
    int kind[4], hh[4];
    uint4 xa[4], xb[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int r = r0 + j * n_slices;
      kind[j] = -1;
      if (r < n_rows) {
        src[j] = row_of(r, kind[j], hh[j]);
        if (!(kind[j] == 0 ? do_q : (kind[j] == 1 ? do_k : do_v))) kind[j] = -1;  // nothing to do for this row
      }
      if (kind[j] >= 0) {
        xa[j] = *reinterpret_cast<const uint4*>(src[j] + co);
        if (c2 >= 0) xb[j] = *reinterpret_cast<const uint4*>(src[j] + co2);
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (kind[j] < 0) continue;
      const int h = hh[j];
      if (kind[j] == 2) {  // v: copied into the cache
        if (a.cache_q8) {
          uint8_t* qrow = reinterpret_cast<uint8_t*>(a.v_cache) + cb * a.cache_stride[0] +
                          static_cast<size_t>(h) * a.cache_stride[1] + static_cast<size_t>(crow) * q_row_bytes;
          float x[8];
          unpack8<BF16>(xa[j], x);
          store_q8_quarter(x, qrow + (c >> 2) * 34, c & 3);
          if (c2 >= 0) {
            unpack8<BF16>(xb[j], x);
            store_q8_quarter(x, qrow + (c2 >> 2) * 34, c2 & 3);
          }
        } else {
          uint8_t* drow = reinterpret_cast<uint8_t*>(a.v_cache) + 2 * (cb * a.cache_stride[0] + static_cast<size_t>(h) * a.cache_stride[1] + static_cast<size_t>(crow) * a.cache_stride[2]);
          *reinterpret_cast<uint4*>(drow + co) = xa[j];
          if (c2 >= 0) *reinterpret_cast<uint4*>(drow + co2) = xb[j];
        }
        continue;
      }
      // q and k: rotate
      float ox[8], oy[8];
      {
        float x[8];
        unpack8<BF16>(xa[j], x);
        if (!rotate) {
#pragma unroll
          for (int t = 0; t < 8; ++t) ox[t] = x[t];
        } else if (kNeox) {
          float y[8];
          unpack8<BF16>(xb[j], y);
#pragma unroll
          for (int t = 0; t < 8; ++t) {
            ox[t] = x[t] * cs[t] - y[t] * sn[t];
            oy[t] = x[t] * sn[t] + y[t] * cs[t];
          }
        } else {
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            ox[2 * t] = x[2 * t] * cs[t] - x[2 * t + 1] * sn[t];
            ox[2 * t + 1] = x[2 * t] * sn[t] + x[2 * t + 1] * cs[t];
          }
        }
      }
      if (kind[j] == 1 && a.cache_q8) {  // k into a Q8_0 cache (strides in bytes, rows contiguous)
        uint8_t* qrow = reinterpret_cast<uint8_t*>(a.k_cache) + cb * a.cache_stride[0] +
                        static_cast<size_t>(h) * a.cache_stride[1] + static_cast<size_t>(crow) * q_row_bytes;
        round16<BF16>(ox);
        store_q8_quarter(ox, qrow + (c >> 2) * 34, c & 3);
        if (c2 >= 0) {
          round16<BF16>(oy);
          store_q8_quarter(oy, qrow + (c2 >> 2) * 34, c2 & 3);
        }
        continue;
      }
      // q in place; k into the 16-bit cache, or in place when the call has no cache
      uint8_t* drow = (kind[j] == 1 && a.k_cache != nullptr)
                          ? reinterpret_cast<uint8_t*>(a.k_cache) + 2 * (cb * a.cache_stride[0] + static_cast<size_t>(h) * a.cache_stride[1] + static_cast<size_t>(crow) * a.cache_stride[2])
                          : const_cast<uint8_t*>(src[j]);
      if (rotate || drow != src[j]) *reinterpret_cast<uint4*>(drow + co) = pack8<BF16>(ox);
      if (rotate && kNeox) *reinterpret_cast<uint4*>(drow + co2) = pack8<BF16>(oy);
    }
  }
}

}  // namespace

cudaError_t launch_rope_append(const RopeArgs& a, bool bf16, bool neox, cudaStream_t stream) {
  const int chunks = a.head_dim / 8;
  const int work_chunks = neox ? chunks - a.rotary_dim / 16 : chunks;
  const long long threads = static_cast<long long>(a.batch) * a.seq * work_chunks;
  // Slices over the token's rows (query heads + k heads + v heads): enough of them that the grid is about eight
  // waves of the three 256-thread blocks an SM holds (with one slice a prefill-sized call is 2.3 waves and a
  // quarter of the GPU idles through the last one), but no fewer than four rows per thread where there is that much
  // work (every thread computes the sines and cosines of its chunk's angles once, whatever its number of rows)
  const int n_rows = (a.q != nullptr ? a.n_heads : 0) + (a.k != nullptr ? a.n_kv_heads : 0) +
                     (a.v != nullptr && a.v_cache != nullptr ? a.n_kv_heads : 0);
  const long long blocks_x = (threads + 255) / 256;
  long long slices = (8 * 3 * 148 + blocks_x - 1) / blocks_x;
  const long long max_slices = threads >= 65536 ? (n_rows + 3) / 4 : n_rows;
  if (slices > max_slices) slices = max_slices;
  if (slices < 1) slices = 1;
  const dim3 grid(static_cast<unsigned>((threads + 255) / 256), static_cast<unsigned>(slices));
  if (bf16) {
    if (neox) rope_append_kernel<true, true><<<grid, 256, 0, stream>>>(a);
    else rope_append_kernel<true, false><<<grid, 256, 0, stream>>>(a);
  } else {
    if (neox) rope_append_kernel<false, true><<<grid, 256, 0, stream>>>(a);
    else rope_append_kernel<false, false><<<grid, 256, 0, stream>>>(a);
  }
  return cudaGetLastError();
}

}  // namespace minfer_attn
