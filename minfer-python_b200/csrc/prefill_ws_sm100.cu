// Warp-specialised prefill attention for sm_100a: two 128-row query tiles per
// CTA ping-pong on the tensor core so that the softmax of one tile overlaps the
// MMAs of the other.
//
// Fills the launch the reference leaves unimplemented
// (src/minfer/kernels/torch_ext/csrc/cuda/flash_attn/op.cuh:105; empty kernel at
// .../flash_attn/kernels/kernel.cuh:16-27).
//
// Work of one CTA: two "slots".  With an even GQA group the slots are two query
// heads of one kv head at the same 128 rows (identical key ranges); otherwise
// they are two consecutive 128-row tiles of one head.  Both slots share every
// K/V tile the CTA loads.
//
// Roles (384 threads = 3 warpgroups; the third gives registers to the first two
// with setmaxnreg):
//   warps 0-3  softmax of slot 0 (thread t owns score row t = TMEM lane t)
//   warps 4-7  softmax of slot 1
//   warp  8    lane 0 issues every tcgen05.mma / tcgen05.commit
//   warp  9    lane 0 issues every TMA load (no multicast)
//   warps 10-11 idle
// Tensor memory (512 columns): S0 [0,128)  S1 [128,256)  O0 [256,256+D)  O1 [384,384+D).
// P (16-bit) overwrites the first 64 columns of its S region and is read by the
// PV MMA straight from tensor memory (A operand in TMEM), V is the B operand as
// an MN-major shared-memory descriptor.
// Shared memory: Q 2 x D/64 blocks, then a ring of kStages K/V tiles; every
// block is [128 rows x 128 bytes] with the 128-byte swizzle TMA writes.
//
// Issue order of the MMA thread:  S0(0) S1(0) | PV0(0) S0(1) | PV1(0) S1(1) | ...
// so softmax of slot s for key tile j+1 runs while the tensor core works for
// the other slot.  O is rescaled lazily: a row's reference maximum only moves
// when the new maximum exceeds it by more than 2^8, so P stays below 256 and
// most key tiles need no pass over O at all.
#include "attn_internal.h"
#include "ptx.cuh"

namespace minfer_attn {

namespace {

constexpr int kTileM = 128;
constexpr int kTileN = 128;
constexpr int kBlockBytes = 128 * 128;
constexpr int kThreads = 384;  // three warpgroups: softmax 0, softmax 1, MMA + TMA (+ 2 idle warps)
// register budget per thread after the role split (the launch budget is 65536 / 384 = 168)
constexpr int kRegsSoftmax = 216;
constexpr int kRegsOther = 72;
constexpr float kRescaleThreshold = 8.0f;  // log2 units
#ifndef MINFER_ATTN_POLY_OF_8
#define MINFER_ATTN_POLY_OF_8 0
#endif
// Share (of 8) of the exp2 evaluations done with a cubic on the FMA pipes instead of the special-function
// unit.  2 gains ~3 % in a short burst at full clock, but the extra instructions cost ~1.5 % once the
// 1 kW power cap holds the clock down, which is where a sustained run lives: off by default.
constexpr int kPolyOf8 = MINFER_ATTN_POLY_OF_8;

// barrier indices
constexpr int kQFull = 0;                 // [2]
constexpr int kSFull = 2;                 // [2]
constexpr int kPFull = 4;                 // [2]
constexpr int kODone = 6;                 // [2]
constexpr int kKvFull = 8;                // [kStages], then kKvEmpty [kStages]
constexpr int kMaxList = 1024;            // key tiles a masked call may have (seq_k <= 131072)
// per-tile flag bits: slot s visits the tile (1 << 2s), and must read mask bytes for it (2 << 2s)

// Optional timeline for tuning (compiled in only with -DMINFER_ATTN_TRACE): the
// roles of one CTA write clock64() stamps behind the 16 status words.
#ifdef MINFER_ATTN_TRACE
#define WS_TRACE(role, idx, ev)                                                                        \
  do {                                                                                                 \
    if (trace_on && (idx) < 64) trace_buf[((role) * 64 + (idx)) * 8 + (ev)] = clock64();              \
  } while (0)
#else
#define WS_TRACE(role, idx, ev) \
  do {                          \
  } while (0)
#endif

__device__ __forceinline__ void report_ws(int32_t* status, int site) {
  if (status != nullptr && atomicCAS(status, 0, kStatusWaitTimeout) == 0) {
    status[1] = static_cast<int32_t>(blockIdx.x);
    status[2] = static_cast<int32_t>(blockIdx.y + gridDim.y * blockIdx.z);
    status[3] = site;
  }
}

// kMasked = false: causal (or unmasked) attention, the key tiles of a slot are the
// prefix [0, n_tiles).  kMasked = true: a dense mask; the CTA first compacts the
// per-tile classes written by mask_classify_kernel (0 = nothing visible, 1 = all
// visible, 2 = mixed) into a list of the key tiles at least one slot must visit,
// skips the others entirely and reads mask bytes only for mixed tiles.
template <int D, bool BF16, bool kMasked>
__global__ void __launch_bounds__(kThreads, 1)
prefill_ws_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                  const __grid_constant__ CUtensorMap tm_v, const PrefillArgs a) {
  constexpr int kDB = D / 64;
  constexpr int kTileBytes = kDB * kBlockBytes;  // one Q, K or V tile
  // ring depth: 4 tiles at D=128; 8 at D=64, which also keeps the CTA above half
  // of the shared memory so that two CTAs never compete for the 512 TMEM columns
  constexpr int kStages = (D == 128) ? 4 : 8;
  constexpr int kKvEmpty = kKvFull + kStages;
  constexpr int kNumBars = kKvFull + 2 * kStages;
  constexpr uint32_t kTmemCols = 512;
  constexpr uint32_t kIdescS = umma_idesc(kTileM, kTileN, BF16, false, false);
  constexpr uint32_t kIdescO = umma_idesc(kTileM, D, BF16, false, true);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* s_q = smem;                       // [2][kTileBytes]
  uint8_t* s_kv = s_q + 2 * kTileBytes;      // [kStages][kTileBytes]
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_kv + kStages * kTileBytes);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + kNumBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* n_list = reinterpret_cast<int*>(tmem_slot + 2);
  uint16_t* u_tile = reinterpret_cast<uint16_t*>(tmem_slot + 4);         // [kMaxList] key tile index
  uint8_t* u_flag = reinterpret_cast<uint8_t*>(u_tile + kMaxList);      // [kMaxList] visit / needs-mask bits

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int b = blockIdx.z;
  const int off = a.seq_k - a.seq_q;

  // ---- slot geometry ----
  int head[2], q0[2], n_tiles[2];
  {
    const int xr = static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x);  // long tiles first
    if (a.pair_heads) {
      head[0] = 2 * blockIdx.y;
      head[1] = head[0] + 1;
      q0[0] = q0[1] = xr * kTileM;
    } else {
      head[0] = head[1] = blockIdx.y;
      q0[0] = 2 * xr * kTileM;
      q0[1] = q0[0] + kTileM;
    }
    const int n_all = (a.seq_k + kTileN - 1) / kTileN;
#pragma unroll
    for (int s = 0; s < 2; ++s) {
      if (q0[s] >= a.seq_q) {
        n_tiles[s] = 0;
      } else if (a.causal) {
        const int last_row = min(q0[s] + kTileM - 1, a.seq_q - 1);
        n_tiles[s] = min(n_all, (last_row + off) / kTileN + 1);
      } else {
        n_tiles[s] = n_all;
      }
    }
  }
  const int kvh = head[0] / a.group;
  const int n_max = max(n_tiles[0], n_tiles[1]);
#ifdef MINFER_ATTN_TRACE
  const bool trace_on = a.status != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (tid & 127) == 0;  // thread 256 = lane 0 of the MMA warp
  long long* trace_buf = reinterpret_cast<long long*>(a.status + 16);
#endif

  if (tid == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars[kQFull + i], 1);
      mbar_init(&bars[kSFull + i], 1);
      mbar_init(&bars[kPFull + i], 128);
      mbar_init(&bars[kODone + i], 1);
    }
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&bars[kKvFull + i], 1);
      mbar_init(&bars[kKvEmpty + i], 1);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 8) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  if constexpr (kMasked) {
    if (warp == 0) {
      // compact the tile classes of the two slots into the visit list
      const int n_kt = (a.seq_k + kTileN - 1) / kTileN;
      const int n_qt = (a.seq_q + kTileM - 1) / kTileM;
      const bool act0 = q0[0] < a.seq_q, act1 = q0[1] < a.seq_q;
      const uint8_t* c0 = (a.cls && act0) ? a.cls + (static_cast<size_t>(b) * n_qt + q0[0] / kTileM) * n_kt : nullptr;
      const uint8_t* c1 = (a.cls && act1) ? a.cls + (static_cast<size_t>(b) * n_qt + q0[1] / kTileM) * n_kt : nullptr;
      int count = 0;
      for (int base = 0; base < n_kt; base += 32) {
        const int t = base + lane;
        uint32_t f = 0;
        if (t < n_kt) {
          // without a class table every tile counts as mixed
          const uint32_t k0 = act0 ? (c0 ? c0[t] : 2u) : 0u;
          const uint32_t k1 = act1 ? (c1 ? c1[t] : 2u) : 0u;
          if (k0) f |= 1u | (k0 == 2u ? 2u : 0u);
          if (k1) f |= 4u | (k1 == 2u ? 8u : 0u);
        }
        const uint32_t m = __ballot_sync(0xFFFFFFFFu, f != 0);
        if (f) {
          const int pos = count + __popc(m & ((1u << lane) - 1u));
          if (pos < kMaxList) {
            u_tile[pos] = static_cast<uint16_t>(t);
            u_flag[pos] = static_cast<uint8_t>(f);
          }
        }
        count += __popc(m);
      }
      if (lane == 0) *n_list = min(count, kMaxList);
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // the key tiles this CTA walks, and who visits each
  const int n_u = kMasked ? *n_list : n_max;
  auto tile_at = [&](int i) -> int {
    if constexpr (kMasked) return u_tile[i];
    else return i;
  };
  auto flag_at = [&](int i) -> uint32_t {
    if constexpr (kMasked) return u_flag[i];
    else return (i < n_tiles[0] ? 1u : 0u) | (i < n_tiles[1] ? 4u : 0u);
  };
  const bool act[2] = {q0[0] < a.seq_q, q0[1] < a.seq_q};

  if (warp >= 8) {
    // third warpgroup: hand registers to the softmax warpgroups
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsOther));
  if (warp == 9) {
    // ====================================================================
    // TMA producer
    // ====================================================================
    // The whole warp runs the loops (so addresses and coordinates stay in the
    // uniform datapath); one elected lane issues the copies.
    const bool leader = elect_one() != 0;
    {
      if (leader) {
        tma_prefetch_desc(&tm_q);
        tma_prefetch_desc(&tm_k);
        tma_prefetch_desc(&tm_v);
      }
      // coordinate slot i (1..3) of a tensor map holds batch, head or row
      auto pick = [](int i, const int32_t* pos, int vb, int vh, int vr) {
        return pos[0] == i ? vb : (pos[1] == i ? vh : vr);
      };
      auto load_tile = [&](const CUtensorMap* tm, uint32_t dst, uint64_t* bar, const int32_t* pos, int hh, int row) {
        const int c1 = pick(1, pos, b, hh, row), c2 = pick(2, pos, b, hh, row), c3 = pick(3, pos, b, hh, row);
        if (leader) {
          mbar_arrive_expect_tx(bar, kTileBytes);
#pragma unroll
          for (int db = 0; db < kDB; ++db) tma_load_4d_addr(dst + db * kBlockBytes, tm, bar, db * 64, c1, c2, c3);
        }
      };
      const uint32_t q_addr = smem_u32(s_q), kv_addr = smem_u32(s_kv);
      if (act[0] && n_u > 0) load_tile(&tm_q, q_addr, &bars[kQFull + 0], a.q_pos, head[0], q0[0]);
      if (act[1] && n_u > 0) load_tile(&tm_q, q_addr + kTileBytes, &bars[kQFull + 1], a.q_pos, head[1], q0[1]);
      bool ok = true;
      int r_done = 0;
      const int n_loads = 2 * n_u;  // K V K V ... of the listed tiles
      for (int r = 0; r < n_loads; ++r) {
        const int st = r % kStages;
        if (r >= kStages) {
          if (!(ok = mbar_wait(&bars[kKvEmpty + st], ((r / kStages) - 1) & 1, abort_flag))) {
            report_ws(a.status, 20);
            break;
          }
        }
        load_tile((r & 1) ? &tm_v : &tm_k, kv_addr + st * kTileBytes, &bars[kKvFull + st], a.kv_pos, kvh,
                  tile_at(r >> 1) * kTileN);
        r_done = r + 1;
      }
      if (!ok || *abort_flag) {
        // the CTA is giving up: let the copies already issued land before the
        // shared memory is handed back (bounded polls)
        for (int i = 0; i < 4000000; ++i) {
          bool pending = false;
          if (act[0] && n_u > 0) pending |= !mbar_try_wait(&bars[kQFull + 0], 0);
          if (act[1] && n_u > 0) pending |= !mbar_try_wait(&bars[kQFull + 1], 0);
          for (int r = max(0, r_done - kStages); r < r_done; ++r)
            pending |= !mbar_try_wait(&bars[kKvFull + r % kStages], (r / kStages) & 1);
          if (!pending) break;
        }
      }
    }
    __syncwarp();
  } else if (warp == 8) {
    // ====================================================================
    // MMA issuer.  Descriptors are (hi, lo) pairs; only the 14-bit start
    // address in `lo` changes between instructions.
    // ====================================================================
    // Converged warp; one elected lane issues.  Keeping the control flow and the
    // descriptor arithmetic warp-uniform lets them live in uniform registers,
    // which is what tcgen05.mma takes its descriptors from.
    const bool leader = elect_one() != 0;
    {
      bool ok = true;
      constexpr uint32_t kHi = (1024u >> 4) | (1u << 14) | (2u << 29);  // SBO 1024, version 1, 128-byte swizzle
      constexpr uint32_t kLoK = (16u >> 4) << 16;                        // LBO field of the K-major operands
      constexpr uint32_t kLoV = (static_cast<uint32_t>(kBlockBytes) >> 4) << 16;  // LBO = one block for MN-major V
      const uint32_t q_lo = (smem_u32(s_q) >> 4) | kLoK;
      const uint32_t k_lo = (smem_u32(s_kv) >> 4) | kLoK;
      const uint32_t v_lo = (smem_u32(s_kv) >> 4) | kLoV;
      auto desc = [](uint32_t lo, uint32_t hi) { return (static_cast<uint64_t>(hi) << 32) | lo; };

      // Fully unrolled on purpose: the issuing thread must feed one MMA per ~64
      // tensor-core cycles, so each issue may only cost a handful of instructions
      // (one add per descriptor; everything else is an immediate).
      auto issue_s = [&](int s, int st) {
        const uint32_t qa = q_lo + s * (kTileBytes >> 4);
        const uint32_t ka = k_lo + st * (kTileBytes >> 4);
        const uint32_t ts = tmem_base + s * kTileN;
#pragma unroll
        for (int i = 0; i < kDB * 4; ++i) {
          const uint32_t o = (i >> 2) * (kBlockBytes >> 4) + (i & 3) * 2;  // 32 bytes per 16-element k step
          if (leader) {
            if (i == 0) umma_ss_first(ts, desc(qa + o, kHi), desc(ka + o, kHi), kIdescS);
            else umma_ss_acc(ts, desc(qa + o, kHi), desc(ka + o, kHi), kIdescS);
          }
        }
        if (leader) umma_commit(&bars[kSFull + s]);
      };
      auto issue_pv = [&](int s, int st, bool accumulate) {
        const uint32_t va = v_lo + st * (kTileBytes >> 4);
        const uint32_t tp = tmem_base + s * kTileN;  // P: packed 16-bit pairs, 8 columns per 16 keys
        const uint32_t to = tmem_base + 256 + s * 128;
        if (leader) umma_ts(to, tp, desc(va, kHi), kIdescO, accumulate ? 1u : 0u);
#pragma unroll
        for (int kk = 1; kk < kTileN / 16; ++kk)
          if (leader) umma_ts_acc(to, tp + kk * 8, desc(va + kk * (2048 >> 4), kHi), kIdescO);
        if (leader) umma_commit(&bars[kODone + s]);
      };

      do {
        if (n_u == 0) break;
        if (act[0] && !(ok = mbar_wait(&bars[kQFull + 0], 0, abort_flag))) { report_ws(a.status, 30); break; }
        if (act[1] && !(ok = mbar_wait(&bars[kQFull + 1], 0, abort_flag))) { report_ws(a.status, 30); break; }
        // first listed K tile
        if (!(ok = mbar_wait(&bars[kKvFull + 0], 0, abort_flag))) { report_ws(a.status, 31); break; }
        tc_fence_after();
        {
          const uint32_t f0 = flag_at(0);
          if (f0 & 1u) issue_s(0, 0);
          if (f0 & 4u) issue_s(1, 0);
        }
        if (leader) umma_commit(&bars[kKvEmpty + 0]);

        // Per listed tile i and slot s:  PV_s(i) if s visits i, then S_s(i+1) if s
        // visits i+1.  Only K of the next listed tile is ever needed ahead, so the
        // ring cannot deadlock however sparse a slot's visits are.
        uint32_t done[2] = {0u, 0u};  // tiles finished per slot: parity of p_full / first-PV flag
        for (int i = 0; i < n_u && ok; ++i) {
          const int rv = 2 * i + 1;  // ring index of V of tile i
          const int rk = 2 * i + 2;  // ring index of K of tile i+1
          const int stv = rv % kStages, stk = rk % kStages;
          const uint32_t f = flag_at(i);
          const uint32_t fn = (i + 1 < n_u) ? flag_at(i + 1) : 0u;
          if (!(ok = mbar_wait(&bars[kKvFull + stv], (rv / kStages) & 1, abort_flag))) { report_ws(a.status, 32); break; }
          bool k_waited = false;
#pragma unroll
          for (int s = 0; s < 2; ++s) {
            if (!ok) break;
            if (f & (1u << (2 * s))) {
              WS_TRACE(2, i, s * 3 + 0);
              if (!(ok = mbar_wait(&bars[kPFull + s], done[s] & 1u, abort_flag))) { report_ws(a.status, 33); break; }
              WS_TRACE(2, i, s * 3 + 1);
              tc_fence_after();
              issue_pv(s, stv, done[s] > 0);
              ++done[s];
            }
            if (fn & (1u << (2 * s))) {
              if (!k_waited) {
                if (!(ok = mbar_wait(&bars[kKvFull + stk], (rk / kStages) & 1, abort_flag))) { report_ws(a.status, 34); break; }
                k_waited = true;
                tc_fence_after();
              }
              issue_s(s, stk);
            }
            WS_TRACE(2, i, s * 3 + 2);
          }
          if (!ok) break;
          if (leader) {
            umma_commit(&bars[kKvEmpty + stv]);
            if (i + 1 < n_u) umma_commit(&bars[kKvEmpty + stk]);
          }
        }
      } while (false);
    }
    __syncwarp();
  }
  } else {
    // ====================================================================
    // softmax (+ lazy correction + epilogue) of slot s
    // ====================================================================
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsSoftmax));
    const int s = warp >> 2;
    const int row = tid & 127;
    const int q0s = s ? q0[1] : q0[0];
    const int heads = s ? head[1] : head[0];
    const int r_glob = q0s + row;
    const uint32_t t_lane = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tmem_s = tmem_base + s * kTileN + t_lane;
    const uint32_t tmem_o = tmem_base + 256 + s * 128 + t_lane;
    const float sl2 = a.scale_log2;
    const bool active = s ? act[1] : act[0];
    const uint32_t visit_bit = 1u << (2 * s), mixed_bit = 2u << (2 * s);
    float m_ref = -INFINITY;  // reference maximum the stored P and O are relative to
    float l_run = 0.f;
    bool ok = true;
    const uint8_t* mrow = (kMasked && active)
                              ? a.mask + (static_cast<size_t>(b) * a.seq_q + min(r_glob, a.seq_q - 1)) * a.seq_k
                              : nullptr;
    int j = 0;  // key tiles this slot has processed so far

    for (int i = 0; i < n_u; ++i) {
      const uint32_t fl = flag_at(i);
      if (!(fl & visit_bit)) continue;
      const int kv0 = tile_at(i) * kTileN;
      WS_TRACE(s, j, 0);
      if (!(ok = mbar_wait(&bars[kSFull + s], j & 1, abort_flag))) { report_ws(a.status, 40); break; }
      WS_TRACE(s, j, 1);
      tc_fence_after();

      uint32_t sr[kTileN];
#pragma unroll
      for (int c = 0; c < kTileN / 32; ++c)
        tmem_ld32(tmem_s + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&sr[c * 32]));
      tc_wait_ld();
      WS_TRACE(s, j, 2);

      // ---- masking (tile-uniform decision) ----
      const bool tail = kv0 + kTileN > a.seq_k;
      const bool diag = !kMasked && a.causal && (kv0 + kTileN - 1 > q0s + off);
      if (kMasked && (fl & mixed_bit)) {
        if (!tail && a.mask_vec) {
          const uint4* mp = reinterpret_cast<const uint4*>(mrow + kv0);
#pragma unroll
          for (int c = 0; c < kTileN / 16; ++c) {
            const uint4 mv = __ldg(mp + c);
            const uint32_t w[4] = {mv.x, mv.y, mv.z, mv.w};
#pragma unroll
            for (int e = 0; e < 16; ++e)
              if (((w[e >> 2] >> ((e & 3) * 8)) & 0xFFu) == 0) sr[c * 16 + e] = 0xFF800000u;
          }
        } else {
#pragma unroll
          for (int c = 0; c < kTileN; ++c) {
            const int col = kv0 + c;
            const bool vis = col < a.seq_k && mrow[col] != 0;
            if (!vis) sr[c] = 0xFF800000u;
          }
        }
      } else if (tail || diag) {
        const int lim = (!kMasked && a.causal) ? min(a.seq_k - 1, r_glob + off) : a.seq_k - 1;
#pragma unroll
        for (int c = 0; c < kTileN; ++c)
          if (kv0 + c > lim) sr[c] = 0xFF800000u;
      }

      // ---- row maximum; move the reference only when it lags by > 2^8 ----
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
      for (int c = 0; c < kTileN; c += 8) {
        mx0 = fmax3(mx0, __uint_as_float(sr[c]), __uint_as_float(sr[c + 1]));
        mx1 = fmax3(mx1, __uint_as_float(sr[c + 2]), __uint_as_float(sr[c + 3]));
        mx2 = fmax3(mx2, __uint_as_float(sr[c + 4]), __uint_as_float(sr[c + 5]));
        mx3 = fmax3(mx3, __uint_as_float(sr[c + 6]), __uint_as_float(sr[c + 7]));
      }
      const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
      const bool move = (mx != -INFINITY) && (m_ref == -INFINITY || (mx - m_ref) * sl2 > kRescaleThreshold);
      if (__any_sync(0xFFFFFFFFu, move)) {
        const float alpha = (move && m_ref != -INFINITY) ? ex2_approx((m_ref - mx) * sl2) : 1.f;
        if (move) m_ref = mx;
        l_run *= alpha;
        if (j > 0) {
          // PV(j-1) of this slot must have landed before O is touched
          if (!(ok = mbar_wait(&bars[kODone + s], (j - 1) & 1, abort_flag))) { report_ws(a.status, 41); break; }
          tc_fence_after();
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            uint32_t o[32];
            tmem_ld32(tmem_o + c * 32, o);
            tc_wait_ld();
#pragma unroll
            for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
            tmem_st32(tmem_o + c * 32, o);
          }
        }
      }

      WS_TRACE(s, j, 3);
      // ---- P = exp2(S*c - m*c) -> 16-bit pairs -> tensor memory (over S) ----
      const float mb = (m_ref == -INFINITY) ? 0.f : m_ref * sl2;
      const float2 sl2_2 = make_float2(sl2, sl2);
      const float2 nmb_2 = make_float2(-mb, -mb);
      float2 sum2 = make_float2(0.f, 0.f);
#pragma unroll
      for (int c = 0; c < kTileN / 32; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          const float2 sp = make_float2(__uint_as_float(sr[c * 32 + 2 * e]), __uint_as_float(sr[c * 32 + 2 * e + 1]));
          const float2 x = __ffma2_rn(sp, sl2_2, nmb_2);
          float2 p;
          // kPolyOf8 of every 8 pairs go through the FMA-pipe polynomial, the rest
          // through the special-function unit, so both units stay busy
          if ((e & 7) < kPolyOf8) {
            p = ex2_poly2(x);
          } else {
            p.x = ex2_approx(x.x);
            p.y = ex2_approx(x.y);
          }
          sum2 = __fadd2_rn(sum2, p);
          pk[e] = pack2<BF16>(p.x, p.y);
        }
        tmem_st16(tmem_s + c * 16, pk);
      }
      l_run += sum2.x + sum2.y;
      WS_TRACE(s, j, 4);
      tc_wait_st();
      tc_fence_before();
      mbar_arrive(&bars[kPFull + s]);
      WS_TRACE(s, j, 5);
      ++j;
    }
    const int nt = j;

    // ---- epilogue: O / l -> out ----
    if (ok && nt > 0) {
      if (!(ok = mbar_wait(&bars[kODone + s], (nt - 1) & 1, abort_flag))) report_ws(a.status, 42);
    }
    if (ok && nt == 0 && active && r_glob < a.seq_q) {
      // no key tile holds a visible key for this slot: the rows are zeros
      uint8_t* orow = reinterpret_cast<uint8_t*>(a.out) +
                      2 * (static_cast<size_t>(b) * a.out_stride[0] + static_cast<size_t>(heads) * a.out_stride[1] +
                           static_cast<size_t>(r_glob) * a.out_stride[2]);
#pragma unroll
      for (int c = 0; c < D / 8; ++c) *reinterpret_cast<uint4*>(orow + c * 16) = make_uint4(0u, 0u, 0u, 0u);
    }
    if (ok && nt > 0) {
      tc_fence_after();
      const float inv = (l_run > 0.f) ? 1.f / l_run : 0.f;
      const bool row_valid = r_glob < a.seq_q;
      uint8_t* orow = reinterpret_cast<uint8_t*>(a.out) +
                      2 * (static_cast<size_t>(b) * a.out_stride[0] + static_cast<size_t>(heads) * a.out_stride[1] +
                           static_cast<size_t>(min(r_glob, a.seq_q - 1)) * a.out_stride[2]);
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t o[32];
        tmem_ld32(tmem_o + c * 32, o);
        tc_wait_ld();
        if (row_valid) {
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            uint4 w;
            w.x = pack2<BF16>(__uint_as_float(o[q4 * 8 + 0]) * inv, __uint_as_float(o[q4 * 8 + 1]) * inv);
            w.y = pack2<BF16>(__uint_as_float(o[q4 * 8 + 2]) * inv, __uint_as_float(o[q4 * 8 + 3]) * inv);
            w.z = pack2<BF16>(__uint_as_float(o[q4 * 8 + 4]) * inv, __uint_as_float(o[q4 * 8 + 5]) * inv);
            w.w = pack2<BF16>(__uint_as_float(o[q4 * 8 + 6]) * inv, __uint_as_float(o[q4 * 8 + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + (c * 32 + q4 * 8) * 2) = w;
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 8) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

template <int D, bool BF16, bool kMasked>
cudaError_t launch_ws_one(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const PrefillArgs& a,
                          cudaStream_t stream) {
  constexpr int kStages = (D == 128) ? 4 : 8;
  constexpr size_t smem = static_cast<size_t>(2 + kStages) * (D / 64) * kBlockBytes + 512 + 3 * kMaxList + 1024;
  static bool attr_done[64] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 64 && !attr_done[dev]) {
    e = cudaFuncSetAttribute(prefill_ws_kernel<D, BF16, kMasked>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem));
    if (e != cudaSuccess) return e;
    attr_done[dev] = true;
  }
  const int n_qt = (a.seq_q + kTileM - 1) / kTileM;
  dim3 grid = a.pair_heads ? dim3(n_qt, a.n_heads / 2, a.batch) : dim3((n_qt + 1) / 2, a.n_heads, a.batch);
  prefill_ws_kernel<D, BF16, kMasked><<<grid, kThreads, smem, stream>>>(tq, tk, tv, a);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_prefill_ws(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                              const PrefillArgs& a, int head_dim, bool bf16, cudaStream_t stream) {
  const bool masked = a.mask != nullptr;
  if (head_dim == 128) {
    if (masked) return bf16 ? launch_ws_one<128, true, true>(tq, tk, tv, a, stream) : launch_ws_one<128, false, true>(tq, tk, tv, a, stream);
    return bf16 ? launch_ws_one<128, true, false>(tq, tk, tv, a, stream) : launch_ws_one<128, false, false>(tq, tk, tv, a, stream);
  }
  if (masked) return bf16 ? launch_ws_one<64, true, true>(tq, tk, tv, a, stream) : launch_ws_one<64, false, true>(tq, tk, tv, a, stream);
  return bf16 ? launch_ws_one<64, true, false>(tq, tk, tv, a, stream) : launch_ws_one<64, false, false>(tq, tk, tv, a, stream);
}

}  // namespace minfer_attn
