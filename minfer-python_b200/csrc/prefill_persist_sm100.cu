// Persistent two-tile prefill kernel: causal, unmasked and dense-mask calls.
//
// A work item is two 128-row query tiles ("slots") that share every K/V tile.  One CTA
// per SM walks a list of work items instead of exiting after one.  What that buys: tensor
// memory and the barriers are set up once; the TMA warp already streams the next item's Q/K/V
// while the softmax warps write the previous item's output; and the MMA warp
// starts the next item's first score tiles as soon as its operands have landed,
// so the ~3k-cycle prologue and most of the epilogue of an item disappear from
// the critical path.
//
// Fills the launch the reference leaves unimplemented
// (src/minfer/kernels/torch_ext/csrc/cuda/flash_attn/op.cuh:105; empty kernel at
// .../flash_attn/kernels/kernel.cuh:16-27).
//
// Work items are (query tile or tile pair, head pair or head, batch) ordered by
// decreasing number of key tiles.  With a counter in the caller's workspace the
// CTAs claim items dynamically (longest first, whoever is free takes the next):
// the TMA warp does the atomicAdd and publishes the item through a small
// shared-memory ring to the other roles.  Without a workspace CTA c takes items
// c, 2G-1-c, 2G+c, ... (a snake over rounds of G = gridDim.x items), which gives
// every CTA the same mix of long and short items without any global state.
//
// Dense masks (kMasked): the scheduler warp also compacts the item's tile classes into a
// visit list that travels with the item through the ring, so every role skips the key
// tiles nobody can see; sched_free[entry] (all consumer roles have left the item) guards
// the reuse of a ring entry.
//
// Hand-offs between items, per slot s (all counted over the CTA's lifetime, so
// mbarrier parities keep alternating):
//   q_empty[s]  MMA -> TMA      last S MMA of the item has read Q_s
//   o_free[s]   softmax -> MMA  the epilogue has copied O_s out of tensor memory
// The K/V ring simply continues across items.
//
// Roles and tensor memory.  (1) One S region for both slots
// (tensor memory: S [0,128), P0 [128,192), P1 [192,256), O0, O1): warp 8 issues every
// score MMA, the two slots taking the region in turn, and the next one is issued as
// soon as the softmax warps of the previous one hold their scores in registers
// (s_free) - i.e. while that softmax runs; P has its own columns (p_free tells the
// softmax when the PV MMAs have read them) and warp 10 issues every PV MMA.  No MMA
// is left on a slot's critical path; what bounds the kernel is the softmax itself
// (special-function unit + issue slots of the two warps per SM sub-partition).
// (2) P is handed to the PV issuer in two pieces (p_full[s][piece], one barrier per
// piece), so the PV MMAs of a tile's first half run under the second half's
// exponentials.  (3) The output leaves through the TMA unit: each softmax warp packs
// its 32 rows, 64 columns at a time, into 4 KB of swizzled shared memory and one lane
// issues a tensor store, instead of every thread storing its own row.
#include "attn_internal.h"
#include "ptx.cuh"

#include <atomic>

namespace minfer_attn {

namespace {

constexpr int kTileM = 128;
constexpr int kTileN = 128;
constexpr int kBlockBytes = 128 * 128;
constexpr int kEpiBytes = 32 * 128;  // 32 rows x 64 columns of 16-bit output per softmax warp
// Staging buffers per softmax warp.  With two, the two 64-column passes of a head_dim-128 epilogue do not wait for
// each other's TMA read; the 32 KB have to come out of the K/V ring (MINFER_ATTN_STAGES128=3).  Measured, interleaved
// in one process (burst TFLOP/s at B=4 L=4096 / L=16384 bf16 shard / B=8 L=1024): four stages, one buffer 1194 / 1418 /
// 750; three stages, one buffer 1113 / 1310 / 721; three stages, two buffers 1107 / 1312 / 722.  The fourth ring stage
// is worth 7 %, the second buffer nothing: the wait between the passes is not what the epilogue spends its time on.
#ifndef MINFER_ATTN_EPI_BUFS
#define MINFER_ATTN_EPI_BUFS 1
#endif
constexpr int kEpiBufs = MINFER_ATTN_EPI_BUFS;
constexpr int kThreads = 384;  // softmax 0 (warps 0-3), softmax 1 (4-7), score MMAs (8), scheduler + TMA (9), PV MMAs (10), idle (11)
// setmaxnreg split of the 384 x 168 launch allocation: 8 x 208 + 4 x 88 = 12 x 168
#ifndef MINFER_ATTN_REGS_SOFTMAX
#define MINFER_ATTN_REGS_SOFTMAX 208
#define MINFER_ATTN_REGS_OTHER 88
#endif
constexpr int kRegsSoftmax = MINFER_ATTN_REGS_SOFTMAX;
constexpr int kRegsOther = MINFER_ATTN_REGS_OTHER;
constexpr float kRescaleThreshold = 8.0f;  // log2 units
#ifndef MINFER_ATTN_POLY_OF_8
#define MINFER_ATTN_POLY_OF_8 0
#endif
// Share (of 8) of the exp2 evaluations done with a cubic on the FMA pipes instead of the special-function
// unit.  Measured in this kernel: 1 of 8 is neutral, 2 or more cost 5 % and up (the extra instructions
// outweigh the relieved unit): off by default.
constexpr int kPolyOf8 = MINFER_ATTN_POLY_OF_8;
#ifndef MINFER_ATTN_P_SPLIT
#define MINFER_ATTN_P_SPLIT 2
#endif
// P is written as four 32-key chunks and published to the PV issuer in two pieces: chunks [0, kPSplit)
// and [kPSplit, 4).  The PV MMAs of the first piece run under the second piece's exponentials, which
// shortens the waits for o_done and p_free.  0 publishes P in one piece.
constexpr int kPSplit = MINFER_ATTN_P_SPLIT;
#ifndef MINFER_ATTN_DEFER_P_ARRIVE
#define MINFER_ATTN_DEFER_P_ARRIVE 0
#endif
// Publish the first piece of P after the NEXT chunk's exponentials instead of right after its own stores (the wait
// for the tensor-memory stores then costs nothing).  Measured: 1236 vs 1235 TFLOP/s at the bench shape, 1457 vs 1454
// at L = 16384 - inside the noise; off.  The same goes for a 216 / 72 register split (no spills in the softmax warps).
constexpr bool kDeferPArrive = MINFER_ATTN_DEFER_P_ARRIVE != 0;
#ifndef MINFER_ATTN_BF16_ROUNDED_SUM
#define MINFER_ATTN_BF16_ROUNDED_SUM 0
#endif
// bfloat16 calls: sum the weights after their rounding to bfloat16 (8 significand bits) instead of before it.
// Measured on the long-context shard (one kv head, 8 query heads, L = 32768): 4.5 % slower, and of the elements
// outside the plain tolerance in rows 0-127 it recovers 6 of 23 - the rounding of the weights themselves is what
// moves those short rows, not the mismatch between numerator and denominator.  Off.
constexpr bool kRoundedSum = MINFER_ATTN_BF16_ROUNDED_SUM != 0;
static_assert(kPSplit >= 0 && kPSplit <= 3, "P is written as four 32-key chunks");
constexpr int kPPieces = kPSplit == 0 ? 1 : 2;
// Tensor-memory plan: S [0,128) used by the two slots in turn, P0 [128,192), P1 [192,256), O0 [256,384),
// O1 [384,512); the next score tile is computed while the current softmax runs.

// barrier indices ([2] = one per slot)
constexpr int kQFull = 0;
constexpr int kQEmpty = 2;
constexpr int kSFull = 4;
constexpr int kPFull = 16;   // [2 slots][4]: one barrier per piece (two used), so a fast thread's next piece cannot complete a phase early
constexpr int kODone = 8;
constexpr int kOFree = 10;
constexpr int kSched = 12;   // [kSchedRing] item published by the TMA warp
constexpr int kSchedRing = 4; // the TMA warp is never more than two items ahead of the slowest role
constexpr int kSchedFree = 24;  // [kSchedRing] every consumer role has finished the item of this ring entry
constexpr int kSFree = 6;       // the scores issued last are in registers, the S columns may be overwritten
constexpr int kPFree = 28;      // [2] the PV MMAs reading the slot's P columns have finished
constexpr int kKvFull = 30;  // [kStages], then kKvEmpty [kStages]
constexpr int kMaxTiles = 1024;  // key tiles a masked call may have (seq_k <= 131072)
constexpr int kMaskRing = 3;     // ring entries used by dense-mask calls (their bit planes must fit beside four K/V stages)

// Optional accounting for tuning (compiled in only with -DMINFER_ATTN_TRACE): one thread per slot of every
// CTA sums where its clocks went, and CTA 0 records a timeline of its first item, into a buffer of the
// library's own (g_trace) that minfer_attn_debug_read_trace() copies to the host.  The product build
// has neither.
#ifdef MINFER_ATTN_TRACE
constexpr int kTraceCtas = 160;
constexpr int kTraceWords = kTraceCtas * 2 * 12 + 7 * 64 * 12;
__device__ long long g_trace[kTraceWords];
#define P_ACC(stmt) do { if (acc_on) { stmt; } } while (0)
// timeline of CTA 0's first item: role r (0/1 softmax slot, 2 S issuer, 3 PV issuer), tile jj, event e
#define P_TL(r, jj, e) do { if (tl_on && k == 0 && (jj) < 64) tl_buf[((r) * 64 + (jj)) * 12 + (e)] = clock64(); } while (0)
#else
#define P_ACC(stmt) do { } while (0)
#define P_TL(r, jj, e) do { } while (0)
#endif
#if defined(MINFER_ATTN_TRACE) && defined(MINFER_ATTN_TRACE_EPI)
// tuning builds: the epilogue's phases replace the softmax phases in the accounting words 7..10
#define P_EPI(stmt) do { if (acc_on) { stmt; } } while (0)
#define P_SMX(stmt) do { if (acc_on) { acc_c = acc_c2 = clock64(); } } while (0)
#else
#define P_EPI(stmt) do { } while (0)
#define P_SMX(stmt) P_ACC(stmt)
#endif

__device__ __forceinline__ void report_p(int32_t* status, int site) {
  if (status != nullptr && atomicCAS(status, 0, kStatusWaitTimeout) == 0) {
    status[1] = static_cast<int32_t>(blockIdx.x);
    status[2] = 0;
    status[3] = site;
  }
}

// One work item: the two slots' heads, first query rows and key-tile counts.
struct Item {
  int b, kvh;
  int head[2], q0[2], n[2];  // n: key tiles of the slot when they are a prefix (causal / unmasked calls)
};

__device__ __forceinline__ Item decode_item(const PrefillArgs& a, int id, bool by_kv_set) {
  Item it;
  int xr, y;
  if (by_kv_set) {
    // dynamic claiming: all items of one (batch, kv head) are adjacent, long query tiles first, so the
    // CTAs running at any moment share a few K/V sets in L2; the list ends with short items
    const int per_kv = a.items_y / a.n_kv_heads;  // head pairs (or heads) per kv head
    const int per_set = a.items_x * per_kv;
    const int set = id / per_set, w = id % per_set;
    xr = a.items_x - 1 - w / per_kv;
    y = (set % a.n_kv_heads) * per_kv + w % per_kv;
    it.b = set / a.n_kv_heads;
  } else {
    // static dealing: globally longest first, so that a snake over rounds balances the CTAs
    const int per_x = a.items_y * a.batch;
    xr = a.items_x - 1 - id / per_x;
    const int rem = id % per_x;
    y = rem % a.items_y;
    it.b = rem / a.items_y;
  }
  if (a.pair_heads) {
    it.head[0] = 2 * y;
    it.head[1] = 2 * y + 1;
    it.q0[0] = it.q0[1] = xr * kTileM;
  } else {
    it.head[0] = it.head[1] = y;
    it.q0[0] = 2 * xr * kTileM;
    it.q0[1] = it.q0[0] + kTileM;
  }
  it.kvh = it.head[0] / a.group;
  const int n_all = (a.seq_k + kTileN - 1) / kTileN;
  const int off = a.seq_k - a.seq_q;
#pragma unroll
  for (int s = 0; s < 2; ++s) {
    if (it.q0[s] >= a.seq_q) {
      it.n[s] = 0;
    } else if (a.causal) {
      const int last_row = min(it.q0[s] + kTileM - 1, a.seq_q - 1);
      it.n[s] = min(n_all, (last_row + off) / kTileN + 1);
    } else {
      it.n[s] = n_all;
    }
  }
  return it;
}

// k-th item of this CTA (snake over rounds), or -1 past the end
__device__ __forceinline__ int item_id(int k, int n_items) {
  const int g = gridDim.x;
  const int c = (k & 1) ? (g - 1 - static_cast<int>(blockIdx.x)) : static_cast<int>(blockIdx.x);
  const int id = k * g + c;
  return id < n_items ? id : -1;
}

// What a role needs to walk one item's key tiles.  Causal / unmasked calls: the tiles of slot s are the
// prefix [0, n[s]).  Dense-mask calls (kMasked): the scheduler warp turns the per-tile classes written by
// mask_classify_kernel (0 = nothing visible, 1 = all visible, 2 = mixed) into four bit planes over the key
// tiles, published with the item through the shared-memory ring; a tile with no bit set is neither loaded
// nor computed, and mask bytes are read only for mixed tiles.
// flag bits per tile: slot s visits it (1 << 2s), and must read mask bytes for it (2 << 2s).
struct TileList {
  int n_t;                        // key tiles to scan: [0, n_t)
  int n_u;                        // of which at least one slot visits ("listed": these take K/V ring positions)
  int nvis[2];                    // of which slot s visits
  const volatile uint32_t* planes;  // kMasked only: [n_t / 32][4] bit planes of the flags
  int n0, n1;                     // prefix lengths otherwise
  // Flags of tile t.  `pw` caches the four plane words of t's group of 32 tiles (the caller scans t upwards
  // from 0); a group nobody visits is skipped as a whole by advancing t to its last tile.
  template <bool kMasked>
  __device__ __forceinline__ uint32_t flag_at(int& t, uint32_t (&pw)[4]) const {
    if constexpr (kMasked) {
      if ((t & 31) == 0) {
        const volatile uint32_t* g = planes + (t >> 5) * 4;
        pw[0] = g[0];
        pw[1] = g[1];
        pw[2] = g[2];
        pw[3] = g[3];
        if ((pw[0] | pw[2]) == 0u) {
          t += 31;
          return 0u;
        }
      }
      const int sh = t & 31;
      return ((pw[0] >> sh) & 1u) | (((pw[1] >> sh) & 1u) << 1) | (((pw[2] >> sh) & 1u) << 2) |
             (((pw[3] >> sh) & 1u) << 3);
    } else {
      return (t < n0 ? 1u : 0u) | (t < n1 ? 4u : 0u);
    }
  }
  // Dense masks, one slot's view: bit 0 = slot s visits tile t, bit 1 = it must read mask bytes.  `pv`, `pm`
  // cache the slot's two plane words of t's group; a group the slot does not visit is skipped as a whole.
  __device__ __forceinline__ uint32_t slot_flag_at(int s, int& t, uint32_t& pv, uint32_t& pm) const {
    if ((t & 31) == 0) {
      const volatile uint32_t* g = planes + (t >> 5) * 4 + 2 * s;
      pv = g[0];
      pm = g[1];
      if (pv == 0u) {
        t += 31;
        return 0u;
      }
    }
    const int sh = t & 31;
    return ((pv >> sh) & 1u) | (((pm >> sh) & 1u) << 1);
  }
};

template <int D, bool BF16, bool kMasked>
__global__ void __launch_bounds__(kThreads, 1)
prefill_persist_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                       const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
                       const __grid_constant__ PeerMaps tm_peers, const PrefillArgs a) {
  constexpr int kDB = D / 64;
  constexpr int kTileBytes = kDB * kBlockBytes;
  // K/V ring depth.  head_dim 64 (16 KB tiles): 4 / 6 / 8 / 10 stages measure 794 / 798 / 810 / 804 TFLOP/s at B=2
  // L=8192 - flat beyond two tile pairs; head_dim 128 (32 KB tiles) has room for exactly two pairs, and three stages
  // cost 7 %.
#ifndef MINFER_ATTN_STAGES64
#define MINFER_ATTN_STAGES64 8
#endif
#ifndef MINFER_ATTN_STAGES128
#define MINFER_ATTN_STAGES128 4
#endif
  constexpr int kStages = (D == 128) ? MINFER_ATTN_STAGES128 : MINFER_ATTN_STAGES64;
  constexpr int kRing = kMasked ? kMaskRing : kSchedRing;  // ring entries in use
  // Bit c set: the exponentials of a tile's c-th 32-key chunk use the cubic on the FMA pipes.  At D = 64 the
  // kernel is bound by the special-function unit alone (half the MMA work per exponential) and one chunk of four
  // gains 6 %; a second chunk, or any at D = 128, loses.
#ifndef MINFER_ATTN_POLY_CHUNKS_D128
#define MINFER_ATTN_POLY_CHUNKS_D128 0
#endif
  constexpr int kPolyChunks = (D == 64) ? 2 : MINFER_ATTN_POLY_CHUNKS_D128;
  constexpr int kKvEmpty = kKvFull + kStages;
  constexpr int kNumBars = kKvFull + 2 * kStages;
  constexpr uint32_t kTmemCols = 512;
  // head_dim 64 leaves tensor memory to spare, so each slot could have an S region of its own (S0 [0,128),
  // P0 [128,192), P1 [192,256), O0 [256,320), O1 [320,384), S1 [384,512)) and its next score tile issued as soon as
  // that slot has read its previous one, whatever the other slot is doing (MINFER_ATTN_D64_TWO_S=1).  Measured
  // against the shared region, interleaved in one process: 767 vs 806 TFLOP/s at B=2 L=8192, 234 vs 237 at B=8
  // L=512 (bursts), 728 vs 778 and 247 vs 256 sustained: the alternation that the shared region forces keeps the
  // two slots' softmax half a period apart, which is what lets them share the special-function unit.  Off.
#ifndef MINFER_ATTN_D64_TWO_S
#define MINFER_ATTN_D64_TWO_S 0
#endif
  constexpr bool kTwoS = (D == 64) && MINFER_ATTN_D64_TWO_S != 0;
  constexpr uint32_t kOStride = kTwoS ? 64u : 128u;   // columns between O0 and O1
  constexpr uint32_t kS1 = kTwoS ? 384u : 0u;         // first column of slot 1's scores
  constexpr uint32_t kIdescS = umma_idesc(kTileM, kTileN, BF16, BF16, false, false);
  // A and B of one MMA share their 16-bit format: a float16 P beside a bfloat16 V (formats 0 and 1 in the two
  // fields) is refused by the hardware as an illegal instruction.
  constexpr uint32_t kIdescO = umma_idesc(kTileM, D, BF16, BF16, false, true);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* s_q = smem;                   // [2][kTileBytes]
  uint8_t* s_kv = s_q + 2 * kTileBytes;  // [kStages][kTileBytes]
  uint8_t* s_epi = s_kv + kStages * kTileBytes;  // [8 softmax warps][kEpiBytes] transposing buffers of the epilogue
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_epi + 8 * kEpiBufs * kEpiBytes);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + kNumBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* sched_id = reinterpret_cast<volatile int*>(tmem_slot + 4);  // [kSchedRing]
  // ring entries of the masked form: {n_u, nvis0, nvis1, -} and the flags' bit planes
  volatile int* list_hdr = reinterpret_cast<volatile int*>(tmem_slot + 8);                           // [kSchedRing][4]
  volatile uint32_t* planes = reinterpret_cast<volatile uint32_t*>(tmem_slot + 8 + 4 * kSchedRing);  // [kMaskRing][kMaxTiles / 8]

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int n_items = a.items_x * a.items_y * a.batch;
  const bool dynamic = a.counter != nullptr;
  // items (and, for dense masks, their tile lists) reach the consumer roles through the ring
  const bool use_ring = dynamic || kMasked;
#ifdef MINFER_ATTN_TRACE
  const bool tl_on = blockIdx.x == 0 && (tid & 127) == 0;  // threads 0, 128, 256 (S issuer); PV issuer: 320
  const bool tl_on2 = blockIdx.x == 0 && tid == 320;
  long long* tl_buf = g_trace + kTraceCtas * 2 * 12;
#endif
  // k-th item of this CTA as seen by a consumer role (MMA, softmax): from the ring, else by the static
  // rule; -1 = no more
  auto next_item = [&](int k, bool& ok) -> int {
    if (!use_ring) return item_id(k, n_items);
    if (!(ok = mbar_wait(&bars[kSched + k % kRing], (k / kRing) & 1, abort_flag))) return -1;
    return sched_id[k % kRing];
  };
  // a consumer role is done with the k-th item: its ring entry may be reused
  auto release_item = [&](int k) {
    if (use_ring) mbar_arrive(&bars[kSchedFree + k % kRing]);
  };
  auto list_of = [&](const Item& it, int k) -> TileList {
    TileList v;
    v.n0 = it.n[0];
    v.n1 = it.n[1];
    if constexpr (kMasked) {
      const int e = k % kRing;
      v.n_t = (a.seq_k + kTileN - 1) / kTileN;
      v.n_u = list_hdr[e * 4 + 0];
      v.nvis[0] = list_hdr[e * 4 + 1];
      v.nvis[1] = list_hdr[e * 4 + 2];
      v.planes = planes + e * (kMaxTiles / 8);
    } else {
      v.n_u = max(it.n[0], it.n[1]);
      v.n_t = v.n_u;
      v.nvis[0] = it.n[0];
      v.nvis[1] = it.n[1];
      v.planes = nullptr;
    }
    return v;
  };

  if (tid == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars[kQFull + i], 1);
      mbar_init(&bars[kQEmpty + i], 1);
      mbar_init(&bars[kSFull + i], 1);
      for (int c = 0; c < 4; ++c) mbar_init(&bars[kPFull + 4 * i + c], 128);
      mbar_init(&bars[kODone + i], 1);
      mbar_init(&bars[kOFree + i], 128);
      mbar_init(&bars[kPFree + i], 1);
    }
    mbar_init(&bars[kSFree], 128);
    mbar_init(&bars[kSFree + 1], 128);  // slot 1's own, with two S regions
    for (int i = 0; i < kSchedRing; ++i) {
      mbar_init(&bars[kSched + i], 1);
      mbar_init(&bars[kSchedFree + i], 258);  // the two MMA warps' leaders and the 256 softmax threads
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
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp >= 8) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsOther));
    if (warp == 9) {
      // ==================================================================
      // Scheduler + TMA producer (converged warp, one elected lane issues)
      // ==================================================================
      const bool leader = elect_one() != 0;
      const int lane = tid & 31;
      if (leader) {
        tma_prefetch_desc(&tm_q);
        tma_prefetch_desc(&tm_k);
        tma_prefetch_desc(&tm_v);
      }
      auto pick = [](int i, const int32_t* pos, int vb, int vh, int vr) {
        return pos[0] == i ? vb : (pos[1] == i ? vh : vr);
      };
      auto load_tile = [&](const CUtensorMap* tm, uint32_t dst, uint64_t* bar, const int32_t* pos, int bb, int hh,
                           int row) {
        const int c1 = pick(1, pos, bb, hh, row), c2 = pick(2, pos, bb, hh, row), c3 = pick(3, pos, bb, hh, row);
        if (leader) {
          mbar_arrive_expect_tx(bar, kTileBytes);
#pragma unroll
          for (int db = 0; db < kDB; ++db) tma_load_4d_addr(dst + db * kBlockBytes, tm, bar, db * 64, c1, c2, c3);
        }
      };
      const uint32_t q_addr = smem_u32(s_q), kv_addr = smem_u32(s_kv);
      bool ok = true;
      uint32_t q_loads[2] = {0u, 0u};  // Q tiles loaded so far per slot
      uint32_t r = 0;                  // K/V ring position over the CTA's lifetime
      const int leader_lane = __ffs(__ballot_sync(0xFFFFFFFFu, leader)) - 1;
      for (int k = 0; ok; ++k) {
        int id;
        if (dynamic) {
          // first item: the CTA's own index; later ones from the global counter
          id = static_cast<int>(blockIdx.x);
          if (k > 0) {
            if (leader) id = static_cast<int>(gridDim.x) + atomicAdd(a.counter, 1);
            id = __shfl_sync(0xFFFFFFFFu, id, leader_lane);
          }
          if (id >= n_items) id = -1;
        } else {
          id = item_id(k, n_items);
        }
        Item it{};
        if (id >= 0) it = decode_item(a, id, dynamic && a.order_by_kv_set);
        if (use_ring) {
          const int e = k % kRing;
          // the entry's previous item (k - kSchedRing) must have been left by every consumer role
          if (k >= kRing &&
              !(ok = mbar_wait(&bars[kSchedFree + e], ((k / kRing) - 1) & 1u, abort_flag))) {
            report_p(a.status, 22);
            break;
          }
          if constexpr (kMasked) {
            if (id >= 0) {
              // the tile classes of the two slots -> the entry's four bit planes
              const int n_kt = (a.seq_k + kTileN - 1) / kTileN;
              const int n_qt = (a.seq_q + kTileM - 1) / kTileM;
              const bool act0 = it.q0[0] < a.seq_q, act1 = it.q0[1] < a.seq_q;
              const uint8_t* c0 =
                  (a.cls && act0) ? a.cls + (static_cast<size_t>(it.b) * n_qt + it.q0[0] / kTileM) * n_kt : nullptr;
              const uint8_t* c1 =
                  (a.cls && act1) ? a.cls + (static_cast<size_t>(it.b) * n_qt + it.q0[1] / kTileM) * n_kt : nullptr;
              volatile uint32_t* pl = planes + e * (kMaxTiles / 8);
              int count = 0, v0 = 0, v1 = 0;
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
                const uint32_t b0 = __ballot_sync(0xFFFFFFFFu, (f & 1u) != 0), b1 = __ballot_sync(0xFFFFFFFFu, (f & 2u) != 0);
                const uint32_t b2 = __ballot_sync(0xFFFFFFFFu, (f & 4u) != 0), b3 = __ballot_sync(0xFFFFFFFFu, (f & 8u) != 0);
                if (lane == 0) {
                  pl[(base >> 5) * 4 + 0] = b0;
                  pl[(base >> 5) * 4 + 1] = b1;
                  pl[(base >> 5) * 4 + 2] = b2;
                  pl[(base >> 5) * 4 + 3] = b3;
                }
                count += __popc(b0 | b2);
                v0 += __popc(b0);
                v1 += __popc(b2);
              }
              if (lane == 0) {
                list_hdr[e * 4 + 0] = count;
                list_hdr[e * 4 + 1] = v0;
                list_hdr[e * 4 + 2] = v1;
              }
              __syncwarp();
            }
          }
          if (leader) sched_id[e] = id;
          __threadfence_block();
          __syncwarp();
          if (leader) mbar_arrive(&bars[kSched + e]);
        }
        if (id < 0) break;
        const TileList tl = list_of(it, k);
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          if (tl.nvis[s] == 0 || !ok) continue;
          if (q_loads[s] > 0 &&
              !(ok = mbar_wait(&bars[kQEmpty + s], (q_loads[s] - 1) & 1u, abort_flag))) {
            report_p(a.status, 21);
            continue;
          }
          load_tile(&tm_q, q_addr + s * kTileBytes, &bars[kQFull + s], a.q_pos, it.b, it.head[s], it.q0[s]);
          ++q_loads[s];
        }
        // K V K V ... of the listed tiles
        uint32_t pw[4] = {0u, 0u, 0u, 0u};
        for (int t = 0; t < tl.n_t && ok; ++t) {
          if (tl.template flag_at<kMasked>(t, pw) == 0u) continue;
#pragma unroll
          for (int h = 0; h < 2 && ok; ++h, ++r) {
            const uint32_t st = r % kStages;
            if (r >= kStages && !(ok = mbar_wait(&bars[kKvEmpty + st], ((r / kStages) - 1) & 1u, abort_flag))) {
              report_p(a.status, 20);
              break;
            }
            load_tile(h ? &tm_v : &tm_k, kv_addr + st * kTileBytes, &bars[kKvFull + st], a.kv_pos, it.b, it.kvh,
                      t * kTileN);
          }
        }
      }
      if (!ok || *abort_flag) {
        // the CTA is giving up: let the copies already issued land before the
        // shared memory is handed back (bounded polls)
        for (int i = 0; i < 4000000; ++i) {
          bool pending = false;
#pragma unroll
          for (int s = 0; s < 2; ++s)
            if (q_loads[s] > 0) pending |= !mbar_try_wait(&bars[kQFull + s], (q_loads[s] - 1) & 1u);
          const uint32_t lo = r > static_cast<uint32_t>(kStages) ? r - kStages : 0u;
          for (uint32_t x = lo; x < r; ++x) pending |= !mbar_try_wait(&bars[kKvFull + x % kStages], (x / kStages) & 1u);
          if (!pending) break;
        }
      }
      __syncwarp();
    } else if (warp == 8 || warp == 10) {
      // ==================================================================
      // MMA issuers (converged warps, one elected lane issues):
      // warp 8 issues every score MMA, warp 10 every PV MMA.  The single S region is used by
      // the two slots in turn: the next S (whichever slot's) is issued as soon as the softmax
      // warps of the previous one hold their scores in registers (s_free), i.e. WHILE that
      // softmax runs, and P has its own columns, so no MMA is left on a slot's critical path.
      // ==================================================================
      const bool leader = elect_one() != 0;
      bool ok = true;
      constexpr uint32_t kHi = (1024u >> 4) | (1u << 14) | (2u << 29);  // SBO 1024, version 1, 128-byte swizzle
      constexpr uint32_t kLoK = (16u >> 4) << 16;
      constexpr uint32_t kLoV = (static_cast<uint32_t>(kBlockBytes) >> 4) << 16;  // LBO = one block for MN-major V
      const uint32_t q_lo = (smem_u32(s_q) >> 4) | kLoK;
      const uint32_t k_lo = (smem_u32(s_kv) >> 4) | kLoK;
      const uint32_t v_lo = (smem_u32(s_kv) >> 4) | kLoV;
      auto desc = [](uint32_t lo, uint32_t hi) { return (static_cast<uint64_t>(hi) << 32) | lo; };
      uint32_t items[2] = {0u, 0u};  // items in which the slot had work (parity of q_full / o_free)
      uint32_t r = 0;                // K/V ring position, in step with the TMA warp

      if (warp == 8) {
        // ---- scores: S = Q_s K^T into the shared S columns ----
        auto issue_s = [&](int s, uint32_t st) {
          const uint32_t qa = q_lo + s * (kTileBytes >> 4);
          const uint32_t ka = k_lo + st * (kTileBytes >> 4);
#pragma unroll
          for (int i = 0; i < kDB * 4; ++i) {
            const uint32_t o = (i >> 2) * (kBlockBytes >> 4) + (i & 3) * 2;  // 32 bytes per 16-element k step
            if (leader) {
              if (i == 0) umma_ss_first(tmem_base + (s ? kS1 : 0u), desc(qa + o, kHi), desc(ka + o, kHi), kIdescS);
              else umma_ss_acc(tmem_base + (s ? kS1 : 0u), desc(qa + o, kHi), desc(ka + o, kHi), kIdescS);
            }
          }
          if (leader) umma_commit(&bars[kSFull + s]);
        };
        uint32_t s_count = 0;  // score tiles issued over the CTA's lifetime (parity of s_free)
        [[maybe_unused]] uint32_t s_slot[2] = {0u, 0u};  // the same per slot (two S regions)
        for (int k = 0; ok; ++k) {
          const int id = next_item(k, ok);
          if (!ok) { report_p(a.status, 37); break; }
          if (id < 0) break;
          const Item it = decode_item(a, id, dynamic && a.order_by_kv_set);
          const TileList tl = list_of(it, k);
          if (tl.n_u == 0) {
            if (leader) release_item(k);
            continue;
          }
#pragma unroll
          for (int s = 0; s < 2; ++s) {
            if (tl.nvis[s] > 0 && ok && !(ok = mbar_wait(&bars[kQFull + s], items[s] & 1u, abort_flag)))
              report_p(a.status, 30);
          }
          if (!ok) break;
          [[maybe_unused]] int s_issued[2] = {0, 0};
          uint32_t pw[4] = {0u, 0u, 0u, 0u};
          for (int t = 0, li = 0; t < tl.n_t && ok; ++t) {
            const uint32_t f = tl.template flag_at<kMasked>(t, pw);
            if (f == 0u) continue;
            const uint32_t rk = r + 2 * li;  // ring position of K of this (the li-th listed) tile
            const uint32_t stk = rk % kStages;
            ++li;
            if (!(ok = mbar_wait(&bars[kKvFull + stk], (rk / kStages) & 1u, abort_flag))) { report_p(a.status, 31); break; }
#pragma unroll
            for (int s = 0; s < 2; ++s) {
              if (!ok || !(f & (1u << (2 * s)))) continue;
              // the scores issued last (either slot's) must have been copied out of the S columns
              P_TL(2, t, s * 3 + 0);
              if constexpr (kTwoS) {
                // the slot's own previous scores must have been copied out of its S columns
                if (s_slot[s] > 0 && !(ok = mbar_wait(&bars[kSFree + s], (s_slot[s] - 1) & 1u, abort_flag))) { report_p(a.status, 38); continue; }
              } else {
                if (s_count > 0 && !(ok = mbar_wait(&bars[kSFree], (s_count - 1) & 1u, abort_flag))) { report_p(a.status, 38); continue; }
              }
              tc_fence_after();
              P_TL(2, t, s * 3 + 1);
              issue_s(s, stk);
              P_TL(2, t, s * 3 + 2);
              ++s_count;
              ++s_slot[s];
              bool last;
              if constexpr (kMasked) last = ++s_issued[s] == tl.nvis[s];
              else last = t + 1 == tl.nvis[s];
              if (last && leader) umma_commit(&bars[kQEmpty + s]);  // the slot's last S of the item
            }
            if (!ok) break;
            if (leader) umma_commit(&bars[kKvEmpty + stk]);
          }
          r += 2 * tl.n_u;
#pragma unroll
          for (int s = 0; s < 2; ++s)
            if (tl.nvis[s] > 0) ++items[s];
          if (leader) release_item(k);
        }
      } else {
        // ---- O_s (+)= P_s V, P from its own tensor-memory columns ----
        auto issue_pv = [&](int s, uint32_t st, int c, bool accumulate) {
          const int kk0 = (c == 0) ? 0 : 2 * kPSplit;  // 16-key steps [kk0, kk1)
          const int kk1 = (c == kPPieces - 1) ? kTileN / 16 : 2 * kPSplit;
          const uint32_t va = v_lo + st * (kTileBytes >> 4);
          const uint32_t tp = tmem_base + 128 + s * 64;  // P: packed 16-bit pairs, 8 columns per 16 keys
          const uint32_t to = tmem_base + 256 + s * kOStride;
#pragma unroll
          for (int kk = 0; kk < kTileN / 16; ++kk) {
            if (kk < kk0 || kk >= kk1) continue;
            if (leader) {
              if (kk == kk0) umma_ts(to, tp + kk * 8, desc(va + kk * (2048 >> 4), kHi), kIdescO, accumulate ? 1u : 0u);
              else umma_ts_acc(to, tp + kk * 8, desc(va + kk * (2048 >> 4), kHi), kIdescO);
            }
          }
          if (c == kPPieces - 1 && leader) {
            umma_commit(&bars[kODone + s]);
            umma_commit(&bars[kPFree + s]);
          }
        };
        uint32_t tiles[2] = {0u, 0u};  // key tiles finished per slot over the CTA's lifetime (parity of p_full)
        for (int k = 0; ok; ++k) {
          const int id = next_item(k, ok);
          if (!ok) { report_p(a.status, 37); break; }
          if (id < 0) break;
          const Item it = decode_item(a, id, dynamic && a.order_by_kv_set);
          const TileList tl = list_of(it, k);
          if (tl.n_u == 0) {
            if (leader) release_item(k);
            continue;
          }
          [[maybe_unused]] int pv_done[2] = {0, 0};
          uint32_t pw[4] = {0u, 0u, 0u, 0u};
          for (int t = 0, li = 0; t < tl.n_t && ok; ++t) {
            const uint32_t f = tl.template flag_at<kMasked>(t, pw);
            if (f == 0u) continue;
            const uint32_t rv = r + 2 * li + 1;  // ring position of V of this (the li-th listed) tile
            const uint32_t stv = rv % kStages;
            ++li;
            if (!(ok = mbar_wait(&bars[kKvFull + stv], (rv / kStages) & 1u, abort_flag))) { report_p(a.status, 32); break; }
#pragma unroll
            for (int s = 0; s < 2; ++s) {
              if (!ok || !(f & (1u << (2 * s)))) continue;
              const bool first_pv = kMasked ? pv_done[s] == 0 : t == 0;
              if (first_pv && items[s] > 0) {
                // O_s still holds the previous item's result until its epilogue has read it
                if (!(ok = mbar_wait(&bars[kOFree + s], (items[s] - 1) & 1u, abort_flag))) { report_p(a.status, 35); continue; }
              }
#pragma unroll
              for (int c = 0; c < kPPieces; ++c) {
                if (!ok) continue;
                if (!(ok = mbar_wait(&bars[kPFull + 4 * s + c], tiles[s] & 1u, abort_flag))) { report_p(a.status, 33); continue; }
                tc_fence_after();
#ifdef MINFER_ATTN_TRACE
                if (tl_on2 && k == 0 && t < 64) tl_buf[(3 * 64 + t) * 12 + s * 4 + 2 * c] = clock64();
#endif
                issue_pv(s, stv, c, !first_pv || c > 0);
#ifdef MINFER_ATTN_TRACE
                if (tl_on2 && k == 0 && t < 64) tl_buf[(3 * 64 + t) * 12 + s * 4 + 2 * c + 1] = clock64();
#endif
              }
              if (!ok) continue;
              ++tiles[s];
              if constexpr (kMasked) ++pv_done[s];
            }
            if (!ok) break;
            if (leader) umma_commit(&bars[kKvEmpty + stv]);
          }
          r += 2 * tl.n_u;
#pragma unroll
          for (int s = 0; s < 2; ++s)
            if (tl.nvis[s] > 0) ++items[s];
          if (leader) release_item(k);
        }
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
    const int lane = tid & 31;
    const uint32_t t_lane = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tmem_s = tmem_base + (s ? kS1 : 0u) + t_lane;  // scores (one region shared by the slots, or the slot's own)
    const uint32_t tmem_p = tmem_base + 128 + s * 64 + t_lane;  // packed P
    const uint32_t tmem_o = tmem_base + 256 + s * kOStride + t_lane;
    const float sl2 = a.scale_log2;
    const int off = a.seq_k - a.seq_q;
    bool ok = true;
    uint32_t jt = 0;  // key tiles this slot has processed over the CTA's lifetime
#ifdef MINFER_ATTN_TRACE
    const bool acc_on = (tid & 127) == 0 && blockIdx.x < kTraceCtas;
    long long acc_t0 = clock64(), acc_c = 0, acc_first = 0, acc_wait = 0, acc_epi = 0, acc_sched = 0, acc_items = 0, acc_ld = 0, acc_max = 0, acc_exp = 0, acc_resc = 0, acc_c2 = 0, acc_ew = 0, acc_el = 0; [[maybe_unused]] long long acc_e0 = 0, acc_e1 = 0;
#endif

    for (int k = 0; ok; ++k) {
      P_ACC(acc_c = clock64());
      const int id = next_item(k, ok);
      P_ACC(acc_sched += clock64() - acc_c);
      if (!ok) { report_p(a.status, 43); break; }
      if (id < 0) break;
      const Item it = decode_item(a, id, dynamic && a.order_by_kv_set);
      const TileList tl = list_of(it, k);
      const int q0s = s ? it.q0[1] : it.q0[0];
      const int nvis = s ? tl.nvis[1] : tl.nvis[0];
      const int heads = s ? it.head[1] : it.head[0];
      const int r_glob = q0s + row;
      if (nvis == 0) {
        if (kMasked && q0s < a.seq_q && r_glob < a.seq_q) {
          // no key tile holds a visible key for this slot: the rows are zeros
          uint8_t* orow = reinterpret_cast<uint8_t*>(a.out) +
                          2 * (static_cast<size_t>(it.b) * a.out_stride[0] + static_cast<size_t>(heads) * a.out_stride[1] +
                               static_cast<size_t>(r_glob) * a.out_stride[2]);
#pragma unroll
          for (int c = 0; c < D / 8; ++c) *reinterpret_cast<uint4*>(orow + c * 16) = make_uint4(0u, 0u, 0u, 0u);
        }
        release_item(k);
        continue;
      }
      const uint8_t* mrow =
          kMasked ? a.mask + (static_cast<size_t>(it.b) * a.seq_q + min(r_glob, a.seq_q - 1)) * a.seq_k : nullptr;
      float m_ref = -INFINITY;  // reference maximum the stored P and O are relative to
      float l_run = 0.f;
      int jm = 0;  // key tiles this slot has processed in this item (dense masks; else the loop index)

      const int n_iter = kMasked ? tl.n_t : nvis;
      [[maybe_unused]] uint32_t pv = 0u, pm = 0u;
      for (int i = 0; i < n_iter; ++i) {
        bool mixed = false;  // dense masks: the tile needs its mask bytes
        if constexpr (kMasked) {
          const uint32_t fl = tl.slot_flag_at(s, i, pv, pm);
          if (!(fl & 1u)) continue;
          mixed = (fl & 2u) != 0u;
        }
        const int kv0 = i * kTileN;
        const int j = kMasked ? jm : i;
        P_ACC(acc_c = clock64());
        P_TL(s, j, 0);
        if (!(ok = mbar_wait(&bars[kSFull + s], jt & 1u, abort_flag))) { report_p(a.status, 40); break; }
        P_TL(s, j, 1);
        P_ACC(acc_c2 = clock64(); if (j == 0) acc_first += acc_c2 - acc_c; else acc_wait += acc_c2 - acc_c);
        tc_fence_after();

        uint32_t sr[kTileN];
#pragma unroll
        for (int c = 0; c < kTileN / 32; ++c)
          tmem_ld32(tmem_s + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&sr[c * 32]));
        tc_wait_ld();
        // the scores are in registers: the S columns may take the next score tile (either slot's)
        tc_fence_before();
        mbar_arrive(&bars[kSFree + (kTwoS ? s : 0)]);
        P_TL(s, j, 2);
        P_SMX(acc_c = clock64(); acc_ld += acc_c - acc_c2);

        // ---- masking (tile-uniform decision): mask bytes only for mixed tiles of a dense mask; else only
        // the diagonal and the ragged last tile need it ----
        const bool tail = kv0 + kTileN > a.seq_k;
        const bool diag = !kMasked && a.causal && (kv0 + kTileN - 1 > q0s + off);
        if (kMasked && mixed) {
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
            P_SMX(++acc_resc);
            // PV(j-1) of this slot must have landed before O is touched
            if (!(ok = mbar_wait(&bars[kODone + s], (jt - 1) & 1u, abort_flag))) { report_p(a.status, 41); break; }
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

        P_TL(s, j, 3);
        P_SMX(acc_c2 = clock64(); acc_max += acc_c2 - acc_c);
        // ---- P = exp2(S*c - m*c) -> 16-bit pairs -> tensor memory ----
        // the PV MMAs of this slot's previous tile must have finished reading the P columns
        if (jt > 0 && !(ok = mbar_wait(&bars[kPFree + s], (jt - 1) & 1u, abort_flag))) { report_p(a.status, 44); break; }
        tc_fence_after();
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
            // the chunks in kPolyChunks (and kPolyOf8 of every 8 pairs elsewhere) go through the FMA-pipe
            // polynomial, the rest through the special-function unit
            if (((kPolyChunks >> c) & 1) || (e & 7) < kPolyOf8) {
              p = ex2_poly2(x);
            } else {
              p.x = ex2_approx(x.x);
              p.y = ex2_approx(x.y);
            }
            pk[e] = pack2<BF16>(p.x, p.y);
            if constexpr (BF16 && kRoundedSum) {
              // the row sum of the weights as the PV MMA will see them (rounded to bfloat16): numerator and
              // denominator then carry the same rounding, which matters for rows that average only a few keys
              sum2 = __fadd2_rn(sum2, make_float2(__uint_as_float(pk[e] << 16), __uint_as_float(pk[e] & 0xFFFF0000u)));
            } else {
              sum2 = __fadd2_rn(sum2, p);
            }
          }
          if constexpr (kDeferPArrive) {
            // the first piece is published one chunk late: its tensor-memory stores have long landed by the time
            // the next chunk's exponentials are done, so the wait for them costs nothing
            if (kPPieces == 2 && c == kPSplit) {
              tc_wait_st();
              tc_fence_before();
              mbar_arrive(&bars[kPFull + 4 * s]);
              P_TL(s, j, 4);
            }
          }
          tmem_st16(tmem_p + c * 16, pk);
          if (c == 3 || (!kDeferPArrive && c + 1 == kPSplit)) {
            tc_wait_st();
            tc_fence_before();
            mbar_arrive(&bars[kPFull + 4 * s + (c == 3 ? kPPieces - 1 : 0)]);
            P_TL(s, j, c == 3 ? 5 : 4);
          }
        }
        l_run += sum2.x + sum2.y;
        P_SMX(acc_exp += clock64() - acc_c2);
        if constexpr (kMasked) ++jm;
        ++jt;
      }
      if (!ok) break;

      // ---- epilogue: copy O out of tensor memory, release it, then write O / l ----
      P_ACC(acc_c = clock64(); ++acc_items);
      if (!(ok = mbar_wait(&bars[kODone + s], (jt - 1) & 1u, abort_flag))) { report_p(a.status, 42); break; }
      P_ACC(acc_c2 = clock64(); acc_ew += acc_c2 - acc_c);
      tc_fence_after();
      // a row that never saw a visible key (m_ref still -inf) is zeros, whatever the exponentials of
      // its masked scores summed to (the FMA-pipe cubic returns a tiny positive value for -inf)
      const float inv = (m_ref != -INFINITY && l_run > 0.f) ? 1.f / l_run : 0.f;
      // A thread owns one row of O, but a row-per-thread store would touch 32 cache lines per
      // instruction and hold the warp behind the SM's store path.  Instead each warp packs 64 columns of
      // its 32 rows into its own 4 KB of shared memory (16-byte chunks XOR-swizzled by row, the layout of
      // a 128-byte-swizzled tensor map) and one lane hands the box to the TMA unit; rows past seq_q are
      // clipped by the tensor map.
      {
        const uint32_t stage0 = smem_u32(s_epi + warp * kEpiBufs * kEpiBytes);
        const int row0 = q0s + (warp & 3) * 32;  // first row of this warp
        auto pick = [&](int i) { return a.out_pos[0] == i ? it.b : (a.out_pos[1] == i ? heads : row0); };
        const int c1 = pick(1), c2 = pick(2), c3 = pick(3);
        // 64 columns at a time: load, pack, hand to the TMA unit; the next 64 columns are loaded while the
        // unit reads the staging buffer
#pragma unroll
        for (int h = 0; h < D / 64; ++h) {
          uint32_t o[64];
          P_EPI(acc_e0 = clock64());
          tmem_ld32(tmem_o + h * 64, *reinterpret_cast<uint32_t(*)[32]>(&o[0]));
          tmem_ld32(tmem_o + h * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&o[32]));
          tc_wait_ld();
          P_EPI(acc_e1 = clock64(); acc_ld += acc_e1 - acc_e0);
          if (h == D / 64 - 1) {
            tc_fence_before();
            mbar_arrive(&bars[kOFree + s]);  // the MMA warp may overwrite O_s for the next item
            P_ACC(acc_el += clock64() - acc_c2);
          }
          uint32_t v[32];
#pragma unroll
          for (int e = 0; e < 32; ++e)
            v[e] = pack2<BF16>(__uint_as_float(o[2 * e]) * inv, __uint_as_float(o[2 * e + 1]) * inv);
          // the staging buffer is free once the previous box (this pass's predecessor, or the last
          // one of the previous item) has been read by the TMA unit
          P_EPI(acc_e0 = clock64(); acc_max += acc_e0 - acc_e1);
          // (two buffers: pass h owns buffer h, and only that buffer's previous box - two groups back - must have
          // been read; head_dim 64 has one pass per item and keeps the single-buffer rule)
          constexpr bool kTwoBufs = kEpiBufs == 2 && D == 128;
          const uint32_t stage = stage0 + (kTwoBufs ? (h & 1) * kEpiBytes : 0);
          if (lane == 0) {
            if constexpr (kTwoBufs) bulk_wait_read_but<1>();
            else bulk_wait_read();
          }
          __syncwarp();
          P_EPI(acc_e1 = clock64(); acc_exp += acc_e1 - acc_e0);
#pragma unroll
          for (int c = 0; c < 8; ++c)
            st_shared_v4(stage + lane * 128 + ((c ^ (lane & 7)) << 4), v[c * 4], v[c * 4 + 1], v[c * 4 + 2], v[c * 4 + 3]);
          fence_proxy_async_smem();  // generic-proxy writes -> visible to the TMA unit
          __syncwarp();
          if (lane == 0 && row0 < a.seq_q) {
            tma_store_4d(&tm_o, stage, h * 64, c1, c2, c3);
            // multi-GPU prefill: the same box goes to the replicas of `out` on the other GPUs (plain tensor
            // stores over NVLink, no multicast), so the output exchange rides along tile by tile
            for (int pr = 0; pr < a.n_peers; ++pr) tma_store_4d(&tm_peers.m[pr], stage, h * 64, c1, c2, c3);
            bulk_commit();
          }
          P_EPI(acc_resc += clock64() - acc_e1);
        }
      }
      P_ACC(acc_epi += clock64() - acc_c);
      release_item(k);
    }
    if (lane == 0) bulk_wait_all();  // the staging buffers stay allocated until the last box has left
#ifdef MINFER_ATTN_TRACE
    if (acc_on) {
      long long* w = g_trace + (blockIdx.x * 2 + s) * 12;
      w[0] = clock64() - acc_t0; w[1] = acc_first; w[2] = acc_wait; w[3] = acc_epi;
      w[4] = acc_sched; w[5] = acc_items; w[6] = jt; w[7] = acc_ld; w[8] = acc_max; w[9] = acc_exp; w[10] = acc_resc; w[11] = (acc_ew << 32) | acc_el;
    }
#endif
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 8) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

template <int D, bool BF16, bool kMasked>
cudaError_t launch_persist_one(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                               const CUtensorMap& to, const PeerMaps& peers, PrefillArgs a,
                               cudaStream_t stream) {
  constexpr int kStages = (D == 128) ? MINFER_ATTN_STAGES128 : MINFER_ATTN_STAGES64;
  // tiles, epilogue staging, barriers and ring heads, (dense masks) the ring's bit planes, alignment slack:
  // exactly the 227 KB an SM offers for the masked D = 128 form
  constexpr size_t smem = static_cast<size_t>(2 + kStages) * (D / 64) * kBlockBytes + 8 * kEpiBufs * kEpiBytes + 512 +
                          (kMasked ? kMaskRing * (kMaxTiles / 8) * 4 : 0) + 1024;
  static_assert(smem <= 232448, "shared memory per CTA");
  // set once per device (0 = not yet); atomic because several host threads may drive different devices
  static std::atomic<int> sm_count[64] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev >= 64) return cudaErrorInvalidDevice;
  int sms = sm_count[dev].load(std::memory_order_acquire);
  if (sms == 0) {
    e = cudaFuncSetAttribute(prefill_persist_kernel<D, BF16, kMasked>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem));
    if (e != cudaSuccess) return e;
    e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return e;
    sm_count[dev].store(sms, std::memory_order_release);
  }
  const int n_qt = (a.seq_q + kTileM - 1) / kTileM;
  a.items_x = a.pair_heads ? n_qt : (n_qt + 1) / 2;
  a.items_y = a.pair_heads ? a.n_heads / 2 : a.n_heads;
  const long long n_items = static_cast<long long>(a.items_x) * a.items_y * a.batch;
  if (n_items > 0x7FFFFFFF) return cudaErrorInvalidValue;
  int ctas = sms;
  if (a.max_ctas > 0 && a.max_ctas < ctas) ctas = a.max_ctas;
  const int grid = static_cast<int>(n_items < ctas ? n_items : ctas);
  // Order of the dynamically claimed items: globally longest-first while all K/V of the call fit
  // comfortably in the 126 MB L2; grouped by (batch, kv head) beyond that, so that the CTAs running
  // at one time share a few K/V sets instead of sweeping all of them.
  const double kv_bytes = 4.0 * a.batch * a.n_kv_heads * static_cast<double>(a.seq_k) * D;
  a.order_by_kv_set = kv_bytes > 96.0 * 1024 * 1024 ? 1 : 0;
  if (a.counter != nullptr) {
    e = cudaMemsetAsync(a.counter, 0, sizeof(int), stream);
    if (e != cudaSuccess) return e;
  }
  prefill_persist_kernel<D, BF16, kMasked><<<grid, kThreads, smem, stream>>>(tq, tk, tv, to, peers, a);
  return cudaGetLastError();
}

}  // namespace

#ifdef MINFER_ATTN_TRACE
// tuning builds only: copies the accounting buffer of the latest launches to the host
extern "C" int minfer_attn_debug_read_trace(void* dst, size_t bytes) {
  if (bytes > sizeof(long long) * kTraceWords) bytes = sizeof(long long) * kTraceWords;
  return cudaMemcpyFromSymbol(dst, g_trace, bytes) == cudaSuccess ? 0 : 3;
}
#endif

cudaError_t launch_prefill_persist(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                                   const CUtensorMap& to, const PeerMaps& peers, const PrefillArgs& a, int head_dim,
                                   bool bf16, cudaStream_t stream) {
  if (a.mask != nullptr) {
    if (head_dim == 128)
      return bf16 ? launch_persist_one<128, true, true>(tq, tk, tv, to, peers, a, stream)
                  : launch_persist_one<128, false, true>(tq, tk, tv, to, peers, a, stream);
    return bf16 ? launch_persist_one<64, true, true>(tq, tk, tv, to, peers, a, stream)
                : launch_persist_one<64, false, true>(tq, tk, tv, to, peers, a, stream);
  }
  if (head_dim == 128)
    return bf16 ? launch_persist_one<128, true, false>(tq, tk, tv, to, peers, a, stream)
                : launch_persist_one<128, false, false>(tq, tk, tv, to, peers, a, stream);
  return bf16 ? launch_persist_one<64, true, false>(tq, tk, tv, to, peers, a, stream)
              : launch_persist_one<64, false, false>(tq, tk, tv, to, peers, a, stream);
}

}  // namespace minfer_attn
