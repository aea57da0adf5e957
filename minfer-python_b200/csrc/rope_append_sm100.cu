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
// Thread mapping: a (token, 16-byte chunk of head_dim) pair (neox: the chunk and its
// partner chunk) is served by four threads of a block, one per slice of the token's
// rows (query heads, k heads, v heads; more slices over gridDim.y for small calls).
// The frequencies freq_base^(-2i/rotary_dim) come from a 64-entry table that the
// launcher computes on the host (they depend on two scalars of the call); the four
// threads compute one (two) of the pair's 4 (8) sincosf each - about a hundred
// instructions apiece, which with a powf per angle on top made the kernel
// instruction-bound when every thread computed all of them - and share them through
// shared memory; then each walks its rows in batches whose 16-byte chunks it first
// brings into shared memory with asynchronous copies, so that no registers are held
// while the loads are in flight (interleaved form: the next batch flies while this one
// is worked on).
#include "../../include/minfer_attn.h"
#include "attn_internal.h"
#include "ptx.cuh"

#include <cmath>
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
// The kernel waits on its loads more than on anything else, so residency decides: four 256-thread blocks per SM
// (64 registers) with four rows in flight per thread take 77 us on a prefill-sized call (B=4, L=4096, 32/8 heads,
// D=128) where three blocks (80 registers, no spills) take 82 and two blocks with six rows 93; the two-halves form
// holds twice the data per row and keeps its registers with two rows per step (83 us; four rows spill: 125).
#ifndef MINFER_ATTN_ROPE_MINBLOCKS
#define MINFER_ATTN_ROPE_MINBLOCKS 4
#endif
// Loads staged in shared memory by asynchronous copies before the thread works through them (0: plain loads into
// registers, four rows at a time).  Measured on the prefill-sized call (B=4, L=4096, 32/8 heads, D=128; interleaved /
// two-halves / D=64 interleaved, us): registers 77.7 / 84.1 / 47.4; one buffer of 6 chunks 72.0 / 70.9 / 43.0 (8
// chunks 74.1 / 70.4 / 43.2, 10 chunks 79.2 / 72.2 / 44.7); two buffers of 4 chunks, the next batch in flight while
// this one is worked on, 67.4 / 78.0 / 41.4 (of 2 chunks 70.0 / 76.0 / 43.2).  The interleaved form therefore uses two
// buffers of four rows, the two-halves form (two chunks per row, more registers) one buffer of three rows.
#ifndef MINFER_ATTN_ROPE_STAGED
#define MINFER_ATTN_ROPE_STAGED 1
#endif
#ifndef MINFER_ATTN_ROPE_SLICES
#define MINFER_ATTN_ROPE_SLICES 4
#endif
constexpr int kRopeSlices = MINFER_ATTN_ROPE_SLICES;  // threads per pair = row slices inside a block (warp-uniform)
constexpr int kRopePairs = 256 / kRopeSlices;         // (token, chunk) pairs per 256-thread block

template <bool BF16, bool kNeox>
__global__ void __launch_bounds__(kRopePairs * kRopeSlices, MINFER_ATTN_ROPE_MINBLOCKS) rope_append_kernel(const RopeArgs a) {
  constexpr int kRopeRows = kNeox ? 2 : 4;           // rows a thread loads before it computes
  __shared__ __align__(16) float s_cs[kRopePairs][8];
  __shared__ __align__(16) float s_sn[kRopePairs][8];
  const int chunks = a.head_dim / 8;                 // 16-byte chunks per head row
  const int rot_chunks = a.rotary_dim / 8;
  const int work_chunks = kNeox ? chunks - rot_chunks / 2 : chunks;  // neox: a thread takes a chunk and its partner
  const int pair = static_cast<int>(threadIdx.x) % kRopePairs;
  const int slice_in = static_cast<int>(threadIdx.x) / kRopePairs;
  // 32-bit index arithmetic (the launcher refuses calls with 2^31 pairs or more): a 64-bit division is some
  // hundred instructions, and there were four of them per thread
  const unsigned gid = blockIdx.x * static_cast<unsigned>(kRopePairs) + static_cast<unsigned>(pair);
  const unsigned n_tokens = static_cast<unsigned>(a.batch) * static_cast<unsigned>(a.seq);
  const unsigned tok_raw = gid / static_cast<unsigned>(work_chunks);
  const bool valid = tok_raw < n_tokens;              // the last block may hold pairs beyond the last token
  const unsigned token = valid ? tok_raw : n_tokens - 1;
  int c = static_cast<int>(gid - tok_raw * static_cast<unsigned>(work_chunks));
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
  const int b = static_cast<int>(token / static_cast<unsigned>(a.seq));
  const int l = static_cast<int>(token - static_cast<unsigned>(b) * static_cast<unsigned>(a.seq));
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
  {
    constexpr int kAng = kNeox ? 8 : 4;               // angles of a pair
    static_assert(kAng % kRopeSlices == 0, "the angles of a pair are dealt out evenly");
    constexpr int kPer = kAng / kRopeSlices;          // angles this thread computes
    if (rotate) {
      const int i0 = kNeox ? 8 * c : 4 * c;
#pragma unroll
      for (int u = 0; u < kPer; ++u) {
        const int t = slice_in * kPer + u;
        const float ang = static_cast<float>(pos) * a.freq[i0 + t];  // the launcher's table: no powf per thread
        float sv, cv;
        sincosf(ang, &sv, &cv);
        s_sn[pair][t] = sv;
        s_cs[pair][t] = cv;
      }
    }
    __syncthreads();
    if (!valid) return;                               // after the only barrier
    if (rotate) {
#pragma unroll
      for (int t4 = 0; t4 < kAng / 4; ++t4) {
        const float4 cq = *reinterpret_cast<const float4*>(&s_cs[pair][4 * t4]);
        const float4 sq = *reinterpret_cast<const float4*>(&s_sn[pair][4 * t4]);
        cs[4 * t4] = cq.x; cs[4 * t4 + 1] = cq.y; cs[4 * t4 + 2] = cq.z; cs[4 * t4 + 3] = cq.w;
        sn[4 * t4] = sq.x; sn[4 * t4 + 1] = sq.y; sn[4 * t4 + 2] = sq.z; sn[4 * t4 + 3] = sq.w;
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
  // one row of the token: rotate (q, k) or copy (v) this thread's chunk(s) and store them
  auto process = [&](int kd, int h, const uint8_t* srcp, const uint4& xa_, const uint4& xb_) {
      if (kd == 2) {  // v: copied into the cache
        if (a.cache_q8) {
          uint8_t* qrow = reinterpret_cast<uint8_t*>(a.v_cache) + cb * a.cache_stride[0] +
                          static_cast<size_t>(h) * a.cache_stride[1] + static_cast<size_t>(crow) * q_row_bytes;
          float x[8];
          unpack8<BF16>(xa_, x);
          store_q8_quarter(x, qrow + (c >> 2) * 34, c & 3);
          if (c2 >= 0) {
            unpack8<BF16>(xb_, x);
            store_q8_quarter(x, qrow + (c2 >> 2) * 34, c2 & 3);
          }
        } else {
          uint8_t* drow = reinterpret_cast<uint8_t*>(a.v_cache) + 2 * (cb * a.cache_stride[0] + static_cast<size_t>(h) * a.cache_stride[1] + static_cast<size_t>(crow) * a.cache_stride[2]);
          *reinterpret_cast<uint4*>(drow + co) = xa_;
          if (c2 >= 0) *reinterpret_cast<uint4*>(drow + co2) = xb_;
        }
        return;
      }
      // q and k: rotate
      float ox[8], oy[8];
      {
        float x[8];
        unpack8<BF16>(xa_, x);
        if (!rotate) {
#pragma unroll
          for (int t = 0; t < 8; ++t) ox[t] = x[t];
        } else if (kNeox) {
          float y[8];
          unpack8<BF16>(xb_, y);
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
      if (kd == 1 && a.cache_q8) {  // k into a Q8_0 cache (strides in bytes, rows contiguous)
        uint8_t* qrow = reinterpret_cast<uint8_t*>(a.k_cache) + cb * a.cache_stride[0] +
                        static_cast<size_t>(h) * a.cache_stride[1] + static_cast<size_t>(crow) * q_row_bytes;
        round16<BF16>(ox);
        store_q8_quarter(ox, qrow + (c >> 2) * 34, c & 3);
        if (c2 >= 0) {
          round16<BF16>(oy);
          store_q8_quarter(oy, qrow + (c2 >> 2) * 34, c2 & 3);
        }
        return;
      }
      // q in place; k into the 16-bit cache, or in place when the call has no cache
      uint8_t* drow = (kd == 1 && a.k_cache != nullptr)
                          ? reinterpret_cast<uint8_t*>(a.k_cache) + 2 * (cb * a.cache_stride[0] + static_cast<size_t>(h) * a.cache_stride[1] + static_cast<size_t>(crow) * a.cache_stride[2])
                          : const_cast<uint8_t*>(srcp);
      if (rotate || drow != srcp) *reinterpret_cast<uint4*>(drow + co) = pack8<BF16>(ox);
      if (rotate && kNeox) *reinterpret_cast<uint4*>(drow + co2) = pack8<BF16>(oy);
  };
  const int n_slices = static_cast<int>(gridDim.y) * kRopeSlices;
  auto wanted = [&](int kd) { return kd == 0 ? do_q : (kd == 1 ? do_k : do_v); };
#if MINFER_ATTN_ROPE_STAGED
  // Loads through shared memory: a thread issues the 16-byte asynchronous copies of up to kStageRows of its rows
  // (cp.async, no registers held while they fly), waits for its own copies and then works through the rows.
  constexpr int kNC = kNeox ? 2 : 1;                                    // chunks per row and thread
  constexpr int kStageRows = kNeox ? 3 : 4;                             // rows per batch
  constexpr int kBufs = kNeox ? 1 : 2;                                  // 2: the next batch flies while this one is worked on
  constexpr int kBatch = kStageRows * kNC * kRopePairs * kRopeSlices;   // uint4 per buffer
  __shared__ __align__(16) uint4 s_rows[kBufs * kBatch];
  const int tid = static_cast<int>(threadIdx.x);
  const int step = kStageRows * n_slices;
  auto issue = [&](int r0, int buf) {
#pragma unroll
    for (int j = 0; j < kStageRows; ++j) {
      const int r = r0 + j * n_slices;
      if (r < n_rows) {
        int kd, h;
        const uint8_t* srcp = row_of(r, kd, h);
        if (wanted(kd)) {
          cp_async_16(&s_rows[buf * kBatch + (j * kNC) * 256 + tid], srcp + co, true);
          if (kNeox && c2 >= 0) cp_async_16(&s_rows[buf * kBatch + (j * kNC + kNC - 1) * 256 + tid], srcp + co2, true);
        }
      }
    }
    cp_async_commit();
  };
  const int first = static_cast<int>(blockIdx.y) * kRopeSlices + slice_in;
  if (kBufs == 2 && first < n_rows) issue(first, 0);
  int buf = 0;
  for (int r0 = first; r0 < n_rows; r0 += step, buf ^= (kBufs - 1)) {
    if constexpr (kBufs == 2) {
      issue(r0 + step, buf ^ 1);     // (an empty group when there is no next batch)
      cp_async_wait<1>();
    } else {
      issue(r0, 0);
      cp_async_wait<0>();
    }
#pragma unroll
    for (int j = 0; j < kStageRows; ++j) {
      const int r = r0 + j * n_slices;
      if (r >= n_rows) break;
      int kd, h;
      const uint8_t* srcp = row_of(r, kd, h);
      if (!wanted(kd)) continue;
      const uint4 xa_ = s_rows[buf * kBatch + (j * kNC) * 256 + tid];
      const uint4 xb_ = (kNeox && c2 >= 0) ? s_rows[buf * kBatch + (j * kNC + kNC - 1) * 256 + tid] : make_uint4(0u, 0u, 0u, 0u);
      process(kd, h, srcp, xa_, xb_);
    }
  }
#else
  for (int r0 = static_cast<int>(blockIdx.y) * kRopeSlices + slice_in; r0 < n_rows; r0 += kRopeRows * n_slices) {
    const uint8_t* src[kRopeRows];
    int kind[kRopeRows], hh[kRopeRows];
    uint4 xa[kRopeRows], xb[kRopeRows];
#pragma unroll
    for (int j = 0; j < kRopeRows; ++j) {
      const int r = r0 + j * n_slices;
      kind[j] = -1;
      if (r < n_rows) {
        src[j] = row_of(r, kind[j], hh[j]);
        if (!wanted(kind[j])) kind[j] = -1;  // nothing to do for this row
      }
      if (kind[j] >= 0) {
        xa[j] = *reinterpret_cast<const uint4*>(src[j] + co);
        if (c2 >= 0) xb[j] = *reinterpret_cast<const uint4*>(src[j] + co2);
      }
    }
#pragma unroll
    for (int j = 0; j < kRopeRows; ++j) {
      if (kind[j] < 0) continue;
      process(kind[j], hh[j], src[j], xa[j], xb[j]);
    }
  }
#endif
}

}  // namespace

cudaError_t launch_rope_append(const RopeArgs& a_in, bool bf16, bool neox, cudaStream_t stream) {
  RopeArgs a = a_in;
  // The frequencies depend on (freq_base, rotary_dim) only: computed here, once per change of the two, as the
  // reference's kernels compute them - the exponent -2 i / rotary_dim rounded to fp32, the power taken of it
  // (csrc/cuda/il_rope/kernel.cuh:9-39) - with the power itself in double, so the table is within half an ulp.
  {
    thread_local float cached_base = 0.f;
    thread_local int cached_rot = -1;
    thread_local float table[64];
    if (a.rotary_dim / 2 > 64) return cudaErrorInvalidValue;
    if (cached_base != a.freq_base || cached_rot != a.rotary_dim) {
      for (int i = 0; i < a.rotary_dim / 2; ++i) {
        const float x = -2.0f * static_cast<float>(i) / static_cast<float>(a.rotary_dim);
        table[i] = static_cast<float>(std::pow(static_cast<double>(a.freq_base), static_cast<double>(x)));
      }
      for (int i = a.rotary_dim / 2; i < 64; ++i) table[i] = 0.f;
      cached_base = a.freq_base;
      cached_rot = a.rotary_dim;
    }
    for (int i = 0; i < 64; ++i) a.freq[i] = table[i];
  }
  const int chunks = a.head_dim / 8;
  const int work_chunks = neox ? chunks - a.rotary_dim / 16 : chunks;
  const long long pairs = static_cast<long long>(a.batch) * a.seq * work_chunks;
  // A block serves 64 (token, chunk) pairs with four threads each, one per slice of the token's rows (query heads +
  // k heads + v heads).  Small calls get further slices over gridDim.y, down to one row per thread, so that the
  // grid still covers the GPU; large ones keep at least four rows per thread (all loads of a step in flight).
  const int n_rows = (a.q != nullptr ? a.n_heads : 0) + (a.k != nullptr ? a.n_kv_heads : 0) +
                     (a.v != nullptr && a.v_cache != nullptr ? a.n_kv_heads : 0);
  if (pairs > 0x7FFFFFFFll - kRopePairs) return cudaErrorInvalidValue;  // the kernel indexes pairs in 32 bits
  const long long blocks_x = (pairs + kRopePairs - 1) / kRopePairs;
  long long slices_y = (8 * 3 * 148 + blocks_x - 1) / blocks_x;
  const long long max_slices = (pairs >= 65536 ? (n_rows + 3) / 4 : n_rows) / kRopeSlices;
  if (slices_y > max_slices) slices_y = max_slices;
  if (slices_y < 1) slices_y = 1;
  const dim3 grid(static_cast<unsigned>(blocks_x), static_cast<unsigned>(slices_y));
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
