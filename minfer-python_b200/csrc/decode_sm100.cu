// Split-KV decode attention over a padded KV cache, HBM-bound.
//
// The reference has no decode op (its attention op requires seq_q == seq_k,
// src/minfer/kernels/torch_ext/csrc/cuda/flash_attn/op.cuh:76); the cache
// layout [batch, n_kv_heads, max_len, head_dim] is the one its model skeleton
// allocates (src/minfer/core.py:105-127).
//
// Kernel 1 (decode_split_kernel): grid (n_split, n_kv_heads, batch).  A thread
// block streams `chunk` keys of one (sequence, kv head) and serves all `group`
// query heads of that kv head at once, so every cache byte is read once.  Each
// warp runs a private cp.async ring of 16-key tiles (128-bit loads, rows of the
// cache are contiguous, so a warp instruction covers whole 256/128-byte rows)
// and keeps its own online-softmax state; the grouped query heads occupy the
// 16 rows of m16n8k16 tensor-core tiles so the arithmetic stays far below the
// memory time.  The warps' states are merged through shared memory and written
// as one fp32 partial (max, sum, unnormalised output) per (query head, split).
//
// Q8 = true: the caches hold GGML Q8_0 blocks (32 int8 + one fp16 scale, 34 bytes;
// the reference's block_q8_0, src/minfer/kernels/torch_ext/csrc/common/types.hpp:141-146).
// The raw bytes of a 16-key tile are contiguous in the cache and ride the same
// cp.async ring; every lane then builds its tensor-core B fragments straight from
// the raw rows in shared memory - two int8 dropped into the mantissas of a pair of
// halves, the bias subtracted, one multiply by the block's scale - so each value
// is (16-bit type)(q * d), rounded once, exactly as the reference's
// dequant_row_q8_0<half> produces it (csrc/quants/impl.cpp:1153-1166), and no
// 16-bit copy of the tile is ever written.  K keeps the key and dimension order of
// the 16-bit path, so the scores are the same bits; for V a lane takes four
// consecutive dimensions of each block (the output columns come out permuted
// inside a block and are put back in the merge), which leaves every sum over the
// keys as it was.  Cache bytes per key drop from 4 D to 2.125 D.
//
// Kernel 2 (decode_combine_kernel): grid (n_heads, batch) merges the partials
// of the ceil(len / chunk) splits of a sequence and writes the 16-bit output.
// (A one-launch form - every thread block takes a ticket from a counter after
// writing its partial and the last one of a (sequence, kv head) merges - was
// built and measured: the fence and the atomic add about 2 us to every 12 us
// thread block, which costs more than this second launch does.)
#include "attn_internal.h"
#include "ptx.cuh"

#include <atomic>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace minfer_attn {

namespace {

constexpr int kWarps = 4;
constexpr int kStages = 3;
// Q8_0: thread blocks per SM and ring depth (raw tiles are about half the bytes of 16-bit ones)
#ifndef MINFER_ATTN_Q8_CTAS
#define MINFER_ATTN_Q8_CTAS 3
#endif
#ifndef MINFER_ATTN_Q8_STAGES
#define MINFER_ATTN_Q8_STAGES 4
#endif
constexpr int kTileKeys = 16;

// kept out of line: the error path must not cost the streaming loop registers
__device__ __noinline__ void report_bad_page(int32_t* status, int b, int slot, int page) {
  if (status != nullptr && atomicCAS(status, 0, kStatusBadPage) == 0) {
    status[1] = b;
    status[2] = slot;
    status[3] = page;
  }
}

template <int D>
__device__ __forceinline__ uint32_t swz(int row, int chunk) {
  // 16-byte chunk index -> swizzled byte offset inside a [16 x D] 16-bit tile
  if constexpr (D == 128) return row * 256 + (((chunk & 8) | ((chunk ^ row) & 7)) << 4);
  else return row * 128 + (((chunk ^ row) & 7) << 4);
}

// Two int8 of a Q8_0 block -> a pair of 16-bit values (q * d), rounded once.  `src` holds the bytes already
// XORed with 0x80 (q + 128 as an unsigned byte); I0 / I1 pick the bytes of the low / high value.
//   float16: the byte dropped into the mantissa of the half 1024.0 reads 1024 + 128 + q; subtracting 1152 leaves q
//   exactly and one half multiply by d rounds once, as (half)(q * d) does.  No conversion instruction.
//   bfloat16: the same in fp32 (2^23 + 128 + q), where q * d is exact, then one rounding to bfloat16.
template <bool BF16>
struct Q8Scale { uint32_t h2; };          // two fp16 scales (low value's, high value's)
template <>
struct Q8Scale<true> { float2 f2; };
template <bool BF16>
__device__ __forceinline__ Q8Scale<BF16> q8_scale(uint32_t d_lo, uint32_t d_hi) {  // fp16 bit patterns
  Q8Scale<BF16> r;
  if constexpr (BF16) {
    r.f2 = make_float2(__half2float(__ushort_as_half(static_cast<unsigned short>(d_lo))),
                       __half2float(__ushort_as_half(static_cast<unsigned short>(d_hi))));
  } else {
    r.h2 = d_lo | (d_hi << 16);
  }
  return r;
}
template <bool BF16, int I0, int I1>
__device__ __forceinline__ uint32_t q8_pair(uint32_t src, const Q8Scale<BF16>& d) {
  if constexpr (BF16) {
    const float lo = __uint_as_float(__byte_perm(src, 0x4B000000u, 0x7650 | I0));
    const float hi = __uint_as_float(__byte_perm(src, 0x4B000000u, 0x7650 | I1));
    const float2 q = __fadd2_rn(make_float2(lo, hi), make_float2(-8388736.f, -8388736.f));
    const float2 v = __fmul2_rn(q, d.f2);
    return pack2<true>(v.x, v.y);
  } else {
    const uint32_t x = __byte_perm(src, 0x64646464u, 0x5040 | I0 | (I1 << 8));
    const uint32_t bias = 0x64806480u;  // 1152.0 twice
    const __half2 q = __hsub2(*reinterpret_cast<const __half2*>(&x), *reinterpret_cast<const __half2*>(&bias));
    const __half2 v = __hmul2(q, *reinterpret_cast<const __half2*>(&d.h2));
    return *reinterpret_cast<const uint32_t*>(&v);
  }
}

// Paged: the caches are pools of pages reached through a.block_table (a separate instantiation, so that the
// contiguous form keeps its registers).
template <int D, bool BF16, bool Q8, bool Paged>
__global__ void __launch_bounds__(kWarps * 32, Q8 ? MINFER_ATTN_Q8_CTAS : 2) decode_split_kernel(const DecodeArgs a) {
  constexpr int kSt = Q8 ? MINFER_ATTN_Q8_STAGES : kStages;
  constexpr int kRowBytes = D * 2;
  constexpr int kTileBytes = kTileKeys * kRowBytes;        // one of K or V, 16-bit
  constexpr int kChunksPerRow = D / 8;                     // 16-byte chunks
  constexpr int kLoadsPerLane = kTileKeys * kChunksPerRow / 32;
  // Q8_0: raw rows of D/32 blocks of 34 bytes; a 16-row tile is one contiguous, 16-byte aligned span
  constexpr int kQRowBytes = (D / 32) * 34;
  constexpr int kQTileBytes = kTileKeys * kQRowBytes;      // 2176 (D=128) / 1088 (D=64): multiples of 16
  constexpr int kQChunks = kQTileBytes / 16;
  constexpr int kQLoadsPerLane = (kQChunks + 31) / 32;
  // per warp: the ring of raw tiles
  constexpr int kWarpBytes = kSt * 2 * (Q8 ? kQTileBytes : kTileBytes);

  extern __shared__ __align__(128) uint8_t smem[];

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int split = blockIdx.x;
  const int kvh = blockIdx.y;
  const int b = blockIdx.z;

  const int len = min(a.lens[b], a.max_len);
  const int c0 = split * a.chunk;
  if (c0 >= len) return;
  const int c1 = min(len, c0 + a.chunk);
  const int nt = (c1 - c0 + kTileKeys - 1) / kTileKeys;
  const int nt_w = (nt > warp) ? (nt - warp + kWarps - 1) / kWarps : 0;

  uint8_t* wsm = smem + warp * kWarpBytes;
  const uint32_t wsm_u32 = smem_u32(wsm);
  // Byte offset of the first row of a 16-key tile inside either cache.  Paged caches: the tile lies inside one
  // page (page_size is a multiple of 16), found through the block table; strides are then those of the pool.
  // (Everything is recomputed per tile from kernel parameters, which costs no registers between tiles.)
  auto tile_offset = [&](int key0) -> size_t {
    constexpr size_t kUnit = Q8 ? 1 : 2;  // Q8_0 strides are in bytes
    const size_t row_bytes = Q8 ? static_cast<size_t>((D / 32) * 34) : 2 * static_cast<size_t>(a.kv_stride[2]);
    const size_t head_off = kUnit * static_cast<size_t>(kvh) * a.kv_stride[1];
    if constexpr (Paged) {
      const int slot = key0 / a.page_size;
      int page = __ldg(a.block_table + static_cast<size_t>(b) * a.table_stride + slot);
      if (static_cast<unsigned>(page) >= static_cast<unsigned>(a.n_pages)) {
        // never follow an entry that points outside the pools: report it and read page 0 instead
        if (lane == 0) report_bad_page(a.status, b, slot, page);
        page = 0;
      }
      return kUnit * static_cast<size_t>(page) * a.kv_stride[0] + head_off + static_cast<size_t>(key0 % a.page_size) * row_bytes;
    }
    return kUnit * static_cast<size_t>(b) * a.kv_stride[0] + head_off + static_cast<size_t>(key0) * row_bytes;
  };
  const size_t row_stride_bytes = 2 * static_cast<size_t>(a.kv_stride[2]);  // 16-bit caches

  auto issue_tile = [&](int i) {  // i-th tile of this warp -> stage i % kSt
    if (i < nt_w) {
      const int key0 = c0 + (warp + i * kWarps) * kTileKeys;
      const size_t toff = tile_offset(key0);
      if constexpr (Q8) {
        // strides of a Q8_0 cache are in bytes; rows are contiguous
        const uint8_t* kq = reinterpret_cast<const uint8_t*>(a.k) + toff;
        const uint8_t* vq = reinterpret_cast<const uint8_t*>(a.v) + toff;
        uint8_t* dst_k = wsm + (i % kSt) * 2 * kQTileBytes;
        uint8_t* dst_v = dst_k + kQTileBytes;
        // bytes of live rows in this tile (rows beyond the sequence are neither read nor used)
        const int live = min(kTileKeys, c1 - key0) * kQRowBytes;
#pragma unroll
        for (int t = 0; t < kQLoadsPerLane; ++t) {
          const int ch = t * 32 + lane;
          if (ch < kQChunks) {
            const bool pred = ch * 16 < live;  // a chunk that starts inside a live row stays inside the cache
            cp_async_16(dst_k + ch * 16, kq + (pred ? ch * 16 : 0), pred);
            cp_async_16(dst_v + ch * 16, vq + (pred ? ch * 16 : 0), pred);
          }
        }
        cp_async_commit();
        return;
      }
      uint8_t* dst_k = wsm + (i % kSt) * 2 * kTileBytes;
      uint8_t* dst_v = dst_k + kTileBytes;
#pragma unroll
      for (int t = 0; t < kLoadsPerLane; ++t) {
        const int idx = t * 32 + lane;
        const int row = idx / kChunksPerRow;
        const int chunk = idx % kChunksPerRow;
        const bool pred = key0 + row < c1;
        const size_t goff = toff + static_cast<size_t>(pred ? row : 0) * row_stride_bytes + chunk * 16;
        cp_async_16(dst_k + swz<D>(row, chunk), reinterpret_cast<const uint8_t*>(a.k) + goff, pred);
        cp_async_16(dst_v + swz<D>(row, chunk), reinterpret_cast<const uint8_t*>(a.v) + goff, pred);
      }
    }
    cp_async_commit();
  };

#pragma unroll
  for (int s = 0; s < kSt - 1; ++s) issue_tile(s);

  // ---- Q fragments: rows = query heads of this kv head (zero beyond group) ----
  const int g0 = lane >> 2;
  const int tq = lane & 3;
  uint32_t qf[D / 16][4];
  {
    const uint8_t* qb = reinterpret_cast<const uint8_t*>(a.q) + 2 * static_cast<size_t>(b) * a.q_stride[0];
    const int h0 = kvh * a.group + g0;
    const int h1 = h0 + 8;
    const uint8_t* q0p = qb + 2 * static_cast<size_t>(h0) * a.q_stride[1];
    const uint8_t* q1p = qb + 2 * static_cast<size_t>(h1) * a.q_stride[1];
    const bool v0 = g0 < a.group;
    const bool v1 = g0 + 8 < a.group;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      const int d = ks * 16 + tq * 2;
      qf[ks][0] = v0 ? *reinterpret_cast<const uint32_t*>(q0p + 2 * d) : 0u;
      qf[ks][1] = v1 ? *reinterpret_cast<const uint32_t*>(q1p + 2 * d) : 0u;
      qf[ks][2] = v0 ? *reinterpret_cast<const uint32_t*>(q0p + 2 * (d + 8)) : 0u;
      qf[ks][3] = v1 ? *reinterpret_cast<const uint32_t*>(q1p + 2 * (d + 8)) : 0u;
    }
  }

  float oacc[D / 8][4];
#pragma unroll
  for (int n = 0; n < D / 8; ++n) oacc[n][0] = oacc[n][1] = oacc[n][2] = oacc[n][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY};  // log2 domain (already scaled)
  float l_run[2] = {0.f, 0.f};              // this thread's share of the row sums
  const float sl2 = a.scale_log2;

  // ldmatrix lane roles
  const int lm_mi = lane >> 3;
  const int lm_r = lane & 7;

  for (int i = 0; i < nt_w; ++i) {
    cp_async_wait<kSt - 2>();
    __syncwarp();
    issue_tile(i + kSt - 1);

    const int key0 = c0 + (warp + i * kWarps) * kTileKeys;
    // ---- S[16 heads x 16 keys] = Q K^T ----
    float sacc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    [[maybe_unused]] const uint8_t* raw_k = wsm + (i % kSt) * 2 * kQTileBytes;  // Q8: this tile's raw K rows, then V
    [[maybe_unused]] uint32_t sv = 0;
    if constexpr (Q8) {
      // B fragments from the raw rows: lane (g0, tq) holds keys g0 / g0 + 8 and, per 16-dimension step, the pairs
      // at 2 tq and 2 tq + 8 - two-byte loads (the blocks' 34 bytes leave nothing better aligned), the four lanes
      // of a key reading 8 consecutive bytes.  Rows beyond the chunk were zero-filled by the copy (scale 0).
#pragma unroll
      for (int blk = 0; blk < D / 32; ++blk) {
#pragma unroll
        for (int nb = 0; nb < 2; ++nb) {
          const uint8_t* bp = raw_k + (g0 + 8 * nb) * kQRowBytes + blk * 34;
          const uint32_t db = *reinterpret_cast<const uint16_t*>(bp);
          const Q8Scale<BF16> d = q8_scale<BF16>(db, db);
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const uint32_t u0 = *reinterpret_cast<const uint16_t*>(bp + 2 + 16 * h + 2 * tq);
            const uint32_t u1 = *reinterpret_cast<const uint16_t*>(bp + 2 + 16 * h + 8 + 2 * tq);
            mma_16816<BF16>(sacc[nb], qf[2 * blk + h], q8_pair<BF16, 0, 1>(u0 ^ 0x8080u, d),
                            q8_pair<BF16, 0, 1>(u1 ^ 0x8080u, d));
          }
        }
      }
    } else {
      const uint32_t sk = wsm_u32 + (i % kSt) * 2 * kTileBytes;
      sv = sk + kTileBytes;
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        uint32_t r0, r1, r2, r3;
        const int key = (lm_mi >> 1) * 8 + lm_r;
        const int chunk = 2 * ks + (lm_mi & 1);
        ldmatrix_x4(sk + swz<D>(key, chunk), r0, r1, r2, r3);
        mma_16816<BF16>(sacc[0], qf[ks], r0, r1);
        mma_16816<BF16>(sacc[1], qf[ks], r2, r3);
      }
    }

    // ---- scale, mask the ragged end, online softmax ----
    const bool partial = key0 + kTileKeys > c1;
#pragma unroll
    for (int nb = 0; nb < 2; ++nb) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float s = sacc[nb][e] * sl2;
        if (partial && (key0 + nb * 8 + tq * 2 + (e & 1) >= c1)) s = -INFINITY;
        sacc[nb][e] = s;
      }
    }
    float alpha[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      float mx = fmaxf(fmaxf(sacc[0][2 * r], sacc[0][2 * r + 1]), fmaxf(sacc[1][2 * r], sacc[1][2 * r + 1]));
      mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 2));
      const float m_new = fmaxf(m_run[r], mx);  // finite: every tile holds at least one live key
      alpha[r] = ex2_approx(m_run[r] - m_new);  // first tile: exp2(-inf) = 0
      m_run[r] = m_new;
      float sum = 0.f;
#pragma unroll
      for (int nb = 0; nb < 2; ++nb) {
        const float p0 = ex2_approx(sacc[nb][2 * r] - m_new);
        const float p1 = ex2_approx(sacc[nb][2 * r + 1] - m_new);
        sacc[nb][2 * r] = p0;
        sacc[nb][2 * r + 1] = p1;
        sum += p0 + p1;
      }
      l_run[r] = l_run[r] * alpha[r] + sum;
    }
    if (__any_sync(0xFFFFFFFFu, alpha[0] != 1.f || alpha[1] != 1.f)) {
#pragma unroll
      for (int n = 0; n < D / 8; ++n) {
        oacc[n][0] *= alpha[0];
        oacc[n][1] *= alpha[0];
        oacc[n][2] *= alpha[1];
        oacc[n][3] *= alpha[1];
      }
    }
    uint32_t pa[4];
    pa[0] = pack2<BF16>(sacc[0][0], sacc[0][1]);
    pa[1] = pack2<BF16>(sacc[0][2], sacc[0][3]);
    pa[2] = pack2<BF16>(sacc[1][0], sacc[1][1]);
    pa[3] = pack2<BF16>(sacc[1][2], sacc[1][3]);

    // ---- O[16 heads x D] += P V ----
    if constexpr (Q8) {
      // B fragments pair two keys per register: lane (g0, tq) reads, for keys 2 tq, 2 tq + 1, 2 tq + 8, 2 tq + 9, the
      // four bytes at dimensions 4 g0 .. 4 g0 + 3 of every block, interleaves the rows pairwise and converts.
      // Output tile 4 blk + j then holds, in column c, dimension 32 blk + 4 c + j (see q8_dim below).
      const uint8_t* rv = raw_k + kQTileBytes + (2 * tq) * kQRowBytes + 4 * g0;
      // The copy zero-fills whole 16-byte pieces beyond the chunk, so the first row past the end can hold a few
      // real cache bytes, a scale among them: rows past the end get scale 0 (their weights are 0, and 0 * 0 = 0
      // whatever the cache holds there).
      uint32_t row_ok[4];
#pragma unroll
      for (int r = 0; r < 4; ++r) row_ok[r] = (key0 + 2 * tq + (r & 1) + 8 * (r >> 1) < c1) ? 0xFFFFu : 0u;
#pragma unroll
      for (int blk = 0; blk < D / 32; ++blk) {
        uint32_t x[4], dsc[4];
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const uint8_t* bp = rv + ((r & 1) + 8 * (r >> 1)) * kQRowBytes + blk * 34;
          dsc[r] = *reinterpret_cast<const uint16_t*>(bp - 4 * g0) & row_ok[r];
          uint32_t w;
          if (blk & 1) {  // 34 blk + 2 is a multiple of 4 for odd blocks
            w = *reinterpret_cast<const uint32_t*>(bp + 2);
          } else {
            w = static_cast<uint32_t>(*reinterpret_cast<const uint16_t*>(bp + 2)) |
                (static_cast<uint32_t>(*reinterpret_cast<const uint16_t*>(bp + 4)) << 16);
          }
          x[r] = w ^ 0x80808080u;
        }
        const Q8Scale<BF16> d01 = q8_scale<BF16>(dsc[0], dsc[1]);
        const Q8Scale<BF16> d23 = q8_scale<BF16>(dsc[2], dsc[3]);
        const uint32_t lo01 = __byte_perm(x[0], x[1], 0x5140), hi01 = __byte_perm(x[0], x[1], 0x7362);
        const uint32_t lo23 = __byte_perm(x[2], x[3], 0x5140), hi23 = __byte_perm(x[2], x[3], 0x7362);
        mma_16816<BF16>(oacc[4 * blk + 0], pa, q8_pair<BF16, 0, 1>(lo01, d01), q8_pair<BF16, 0, 1>(lo23, d23));
        mma_16816<BF16>(oacc[4 * blk + 1], pa, q8_pair<BF16, 2, 3>(lo01, d01), q8_pair<BF16, 2, 3>(lo23, d23));
        mma_16816<BF16>(oacc[4 * blk + 2], pa, q8_pair<BF16, 0, 1>(hi01, d01), q8_pair<BF16, 0, 1>(hi23, d23));
        mma_16816<BF16>(oacc[4 * blk + 3], pa, q8_pair<BF16, 2, 3>(hi01, d01), q8_pair<BF16, 2, 3>(hi23, d23));
      }
    } else {
#pragma unroll
      for (int dn = 0; dn < D / 16; ++dn) {
        uint32_t r0, r1, r2, r3;
        const int key = (lm_mi & 1) * 8 + lm_r;
        const int chunk = 2 * dn + (lm_mi >> 1);
        ldmatrix_x4_trans(sv + swz<D>(key, chunk), r0, r1, r2, r3);
        mma_16816<BF16>(oacc[2 * dn], pa, r0, r1);
        mma_16816<BF16>(oacc[2 * dn + 1], pa, r2, r3);
      }
    }
  }
  cp_async_wait<0>();

  // ---- row sums across the 4 lanes of a row ----
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xFFFFFFFFu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xFFFFFFFFu, l_run[r], 2);
  }

  // ---- merge the warps through shared memory (reusing the ring buffers) ----
  __syncthreads();
  float* mo = reinterpret_cast<float*>(wsm);             // [16][D]
  float* mml = reinterpret_cast<float*>(wsm) + 16 * D;   // [16][2]
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int g = g0 + 8 * r;
    if (g < a.group) {
#pragma unroll
      for (int n = 0; n < D / 8; ++n) {
        if constexpr (Q8) {
          // column c of output tile 4 blk + j is dimension 32 blk + 4 c + j; this lane holds columns 2 tq, 2 tq + 1
          const int d0 = 32 * (n >> 2) + 8 * tq + (n & 3);
          mo[g * D + d0] = oacc[n][2 * r];
          mo[g * D + d0 + 4] = oacc[n][2 * r + 1];
        } else {
          *reinterpret_cast<float2*>(&mo[g * D + n * 8 + tq * 2]) = make_float2(oacc[n][2 * r], oacc[n][2 * r + 1]);
        }
      }
      if (tq == 0) {
        mml[g * 2] = m_run[r];
        mml[g * 2 + 1] = l_run[r];
      }
    }
  }
  __syncthreads();
  for (int idx = tid; idx < a.group * D; idx += kWarps * 32) {
    const int g = idx / D;
    const int d = idx % D;
    float mw[kWarps];
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      mw[w] = reinterpret_cast<const float*>(smem + w * kWarpBytes)[16 * D + g * 2];
      M = fmaxf(M, mw[w]);
    }
    float o = 0.f, l = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      const float* wf = reinterpret_cast<const float*>(smem + w * kWarpBytes);
      const float sc = (mw[w] == -INFINITY) ? 0.f : ex2_approx(mw[w] - M);
      o += sc * wf[g * D + d];
      l += sc * wf[16 * D + g * 2 + 1];
    }
    const int h = kvh * a.group + g;
    const size_t pidx = (static_cast<size_t>(b) * a.n_heads + h) * a.n_split + split;
    a.part_o[pidx * D + d] = o;
    if (d == 0) {
      a.part_ml[pidx * 2] = M;
      a.part_ml[pidx * 2 + 1] = l;
    }
  }
}

// The merge is a latency problem (a few hundred bytes per thread, every load a trip to L2 or HBM), so the loads are
// issued eight at a time: the (max, sum) pairs of eight splits, then the eight partial outputs they weight.
template <int D, bool BF16>
__global__ void __launch_bounds__(D) decode_combine_kernel(const DecodeArgs a) {
  const int h = blockIdx.x;
  const int b = blockIdx.y;
  const int d = threadIdx.x;
  const int len = min(a.lens[b], a.max_len);
  const int ns = (len + a.chunk - 1) / a.chunk;
  const size_t p0 = (static_cast<size_t>(b) * a.n_heads + h) * a.n_split;
  const float2* ml = reinterpret_cast<const float2*>(a.part_ml) + p0;
  const float* po = a.part_o + p0 * D + d;
  constexpr int kBatch = 8;
  float M = -INFINITY;
  for (int s0 = 0; s0 < ns; s0 += kBatch) {
    float m[kBatch];
#pragma unroll
    for (int j = 0; j < kBatch; ++j) m[j] = (s0 + j < ns) ? ml[s0 + j].x : -INFINITY;
#pragma unroll
    for (int j = 0; j < kBatch; ++j) M = fmaxf(M, m[j]);
  }
  float o = 0.f, l = 0.f;
  for (int s0 = 0; s0 < ns; s0 += kBatch) {
    float2 w[kBatch];
    float x[kBatch];
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      const bool live = s0 + j < ns;
      w[j] = live ? ml[s0 + j] : make_float2(-INFINITY, 0.f);
      x[j] = live ? po[static_cast<size_t>(s0 + j) * D] : 0.f;
    }
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      const float sc = (w[j].x == -INFINITY) ? 0.f : ex2_approx(w[j].x - M);
      l += sc * w[j].y;
      o += sc * x[j];
    }
  }
  const float r = (l > 0.f) ? o / l : 0.f;
  uint8_t* op = reinterpret_cast<uint8_t*>(a.out) +
                2 * (static_cast<size_t>(b) * a.out_stride[0] + static_cast<size_t>(h) * a.out_stride[1] + d);
  if constexpr (BF16) *reinterpret_cast<__nv_bfloat16*>(op) = __float2bfloat16_rn(r);
  else *reinterpret_cast<__half*>(op) = __float2half_rn(r);
}

template <int D, bool BF16, bool Q8, bool Paged>
cudaError_t launch_paged(const DecodeArgs& a, cudaStream_t stream) {
  constexpr int kRaw = Q8 ? kTileKeys * (D / 32) * 34 : kTileKeys * D * 2;
  constexpr int smem = kWarps * (Q8 ? MINFER_ATTN_Q8_STAGES : kStages) * 2 * kRaw;
  static_assert(smem / kWarps >= 16 * D * 4 + 128, "the per-warp region also holds the fp32 merge buffer");
  static std::atomic<bool> attr_done[64] = {};  // set-once flags; the attribute call itself is idempotent
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 64 && !attr_done[dev].load(std::memory_order_acquire)) {
    e = cudaFuncSetAttribute(decode_split_kernel<D, BF16, Q8, Paged>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    attr_done[dev].store(true, std::memory_order_release);
  }
  dim3 grid(a.n_split, a.n_kv_heads, a.batch);
  decode_split_kernel<D, BF16, Q8, Paged><<<grid, kWarps * 32, smem, stream>>>(a);
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  decode_combine_kernel<D, BF16><<<dim3(a.n_heads, a.batch), D, 0, stream>>>(a);
  return cudaGetLastError();
}

template <int D, bool BF16, bool Q8>
cudaError_t launch_one(const DecodeArgs& a, cudaStream_t stream) {
  return a.block_table != nullptr ? launch_paged<D, BF16, Q8, true>(a, stream) : launch_paged<D, BF16, Q8, false>(a, stream);
}

}  // namespace

cudaError_t launch_decode(const DecodeArgs& a, int head_dim, bool bf16, bool q8, cudaStream_t stream) {
  if (q8) {
    if (head_dim == 128) return bf16 ? launch_one<128, true, true>(a, stream) : launch_one<128, false, true>(a, stream);
    return bf16 ? launch_one<64, true, true>(a, stream) : launch_one<64, false, true>(a, stream);
  }
  if (head_dim == 128) return bf16 ? launch_one<128, true, false>(a, stream) : launch_one<128, false, false>(a, stream);
  return bf16 ? launch_one<64, true, false>(a, stream) : launch_one<64, false, false>(a, stream);
}

}  // namespace minfer_attn
