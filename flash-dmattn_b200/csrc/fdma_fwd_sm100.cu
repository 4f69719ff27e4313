// Forward dynamic-mask attention for sm_100a: TMA loads, tcgen05.mma with TMEM accumulators, warp-specialised.
//
// What it computes is the reference's compute_attn_1rowblock
// (csrc/flash_sparse_attn/src/flash_fwd_kernel.h:53-804): S = scale*Q K^T + bias, -inf where the bool mask is
// false / causal / k >= Sk, online softmax, O = P V, LSE. How it computes it is new:
//
//   CTA = 2 query tiles of 128 rows (same batch, same head) x all KV tiles of 128 keys.
//   warp 0      TMA producer: Q once, then K_j, V_j of every KEPT tile into a 4-slot ring (tiles whose mask-OR
//               is zero are never loaded and never multiplied -- the reference's any_active test,
//               flash_fwd_kernel.h:388-404, moved in front of the copy engine)
//   warp 1      MMA issuer (one thread): S_t = Q_t K_j^T (SS), O_t += P_t V_j (A = P from TMEM, B = V MN-major)
//   warp 2      row-broadcast mode: turns bias+mask of a key tile into one fp32 addend per key
//               (bias*log2e, or -inf when masked) in a small shared-memory ring
//   warps 4-7   softmax warpgroup of query tile 0: one thread per query row (TMEM lane = row)
//   warps 8-11  softmax warpgroup of query tile 1
//   TMEM (512 columns): S_0 | S_1 | O_0 | O_1, 128 columns each; P_t (16-bit) overwrites the first 64 columns
//   of S_t. The running max is only raised when it grows by more than 8 (log2 units), so O in TMEM is rescaled
//   rarely and by the softmax threads themselves.
//
// Two bias/mask modes: kBcast (both are broadcast over the query dimension, or absent) and per-query (each
// softmax thread reads its own bias/mask row; kept tiles come from a per-tile activity map that a small
// pre-kernel writes into the workspace).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math_constants.h>

#include <algorithm>
#include <mutex>

#include <type_traits>

#include "fdma_internal.h"
#include "fdma_ptx.cuh"

namespace fdma {
namespace {

constexpr int kBM = 128;          // query rows per tile
constexpr int kBN = 128;          // keys per tile
constexpr int kBmSlots = 4;       // bias+mask addend ring slots
constexpr int kMaxTiles = 8192;   // key tiles per row the tile-flag table can hold (Sk <= 1M)
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kRescaleThreshold = 8.0f;
#ifndef FDMA_POLY_PAIRS
#define FDMA_POLY_PAIRS 0x0000u
#endif
constexpr unsigned kPolyPairs = FDMA_POLY_PAIRS;  // bit i: pair i of every 16 pairs uses exp2_poly2

// Codes stored in the status word when a wait gives up.
enum WaitCode {
  kWaitQ = 101, kWaitKvEmpty = 102, kWaitKvFullK = 103, kWaitKvFullV = 104, kWaitP = 105, kWaitS = 106,
  kWaitO = 107, kWaitBmEmpty = 108, kWaitBmFull = 109, kWaitQEmpty = 110, kWaitOFree = 111, kWaitFlagsFull = 112,
  kWaitFlagsEmpty = 113
};

struct FwdKernelParams {
  CUtensorMap tm_q, tm_k, tm_v;
  const uint8_t* mask;
  const void* bias;
  void* out;
  float* lse;
  const uint8_t* act;  // per-query mode: activity bytes [B][h_mask][ceil(Sq/128)][ceil(Sk/128)], or null
  const int32_t* key_pos;  // broadcast mode only: ascending key positions of compacted keys, or null
  int64_t pos_batch_stride, pos_head_stride;
  int h_pos, causal_shift;
  int* status;
  int64_t o_batch_stride, o_row_stride, o_head_stride;
  int64_t mask_batch_stride, mask_head_stride, mask_row_stride;
  int64_t bias_batch_stride, bias_head_stride, bias_row_stride;
  int b, seqlen_q, seqlen_k, h, h_k, h_mask, h_bias;
  int is_causal;
  int n_mblk;        // query blocks (of kNQ tiles) per (batch, head)
  int n_items;       // work items = n_mblk * h * b
  unsigned* sched;   // zeroed by the launcher: index of the next item nobody has taken yet
  float scale_log2;  // softmax_scale * log2(e)
};

// Head dims 64 and 128: two query tiles (softmax warpgroups) per CTA share every K / V tile; TMEM S0|S1|O0|O1.
// Head dim 256: the O accumulator alone takes 256 TMEM columns and a K or V tile 64 KiB of shared memory, so a CTA
// owns ONE query tile (TMEM S|O = 128 + 256 columns) and the K/V ring has two slots.
template <int D>
struct Smem {
  static constexpr int kNQ = D == 256 ? 1 : 2;          // query tiles per CTA
  static constexpr int kThreads = 128 + 128 * kNQ;
  static constexpr int kStages = D == 256 ? 2 : 4;      // K/V ring slots
  static constexpr int kQBytes = kBM * D * 2;
  static constexpr int kKvBytes = kBN * D * 2;
  static constexpr int kQOff = 0;
  static constexpr int kKvOff = kQOff + kNQ * kQBytes;
  static constexpr int kBmOff = kKvOff + kStages * kKvBytes;
  static constexpr int kPosOff = kBmOff + kBmSlots * kBN * 4;
  static constexpr int kFlagsOff = kPosOff + kBmSlots * kBN * 4;   // two tables: this work item's and the next one's
  static constexpr int kBarOff = kFlagsOff + 2 * kMaxTiles;
  static constexpr int kNumBars = 2 + 2 * kStages + 2 + 2 + 1 + 2 + 2 * kBmSlots + 1 + 4;
  static constexpr int kMiscOff = kBarOff + kNumBars * 8;
  static constexpr int kTotal = kMiscOff + 16;
  static constexpr int kAlloc = kTotal + 1024;  // slack to align the base to 1024 B
};

// Key-tile OR of the bool mask for query-tile rows, with the causal and length limits applied:
// act[b][hm][mt][nt] != 0 iff some (q, k) of the 128x128 tile has mask set, k <= q + Sk - Sq (if causal).
__global__ void tile_activity_kernel(const uint8_t* __restrict__ mask, int64_t sb, int64_t sh, int64_t sr, int B,
                                     int Hm, int Sq, int Sk, int is_causal, uint8_t* __restrict__ act) {
  const int MT = (Sq + kBM - 1) / kBM, NT = (Sk + kBN - 1) / kBN;
  const int lane = threadIdx.x & 31;
  const int64_t total = static_cast<int64_t>(B) * Hm * MT * NT;
  const int64_t w = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5;
  if (w >= total) return;
  const int nt = static_cast<int>(w % NT);
  const int mt = static_cast<int>((w / NT) % MT);
  const int hm = static_cast<int>((w / (static_cast<int64_t>(NT) * MT)) % Hm);
  const int b = static_cast<int>(w / (static_cast<int64_t>(NT) * MT * Hm));
  const uint8_t* base = mask + b * sb + hm * sh;
  const int off = Sk - Sq;
  const int kcol = nt * kBN + (lane & 7) * 16;  // this lane's 16 keys
  const int rows = sr == 0 ? 1 : kBM;           // a row-broadcast mask has one distinct row
  bool any = false;
  for (int r0 = 0; r0 < rows && !any; r0 += 4) {
    const int q = mt * kBM + r0 + (lane >> 3);
    if (q < Sq && (r0 + (lane >> 3)) < rows) {
      const uint4 v = *reinterpret_cast<const uint4*>(base + static_cast<int64_t>(q) * sr + kcol);
      const uint32_t words[4] = {v.x, v.y, v.z, v.w};
      // with a broadcast row the causal limit of the LAST row of the tile decides
      const int qlim = sr == 0 ? min(Sq - 1, mt * kBM + kBM - 1) : q;
      int kmax = Sk - 1;
      if (is_causal) kmax = min(kmax, qlim + off);
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const bool set = (words[i >> 2] >> ((i & 3) * 8)) & 0xFFu;
        if (set && kcol + i <= kmax) any = true;
      }
    }
    any = __any_sync(0xffffffffu, any);
  }
  if (lane == 0) act[w] = any ? 1 : 0;
}

// Work item = one query block (kNQ query tiles of 128 rows) of one (batch, head). CTAs are persistent: the list is
// ordered by decreasing causal extent (last query blocks first) and a CTA takes the next item nobody has taken yet
// (one atomicAdd per item on a counter the launcher zeroes), which balances the SMs to within one short item. Barrier phases, ring positions and tensor memory carry over
// from one item to the next; nothing is re-initialised, and the pieces of an item that no role of the PREVIOUS
// item needs any more start early: the tile flags of the next item are built by warp 3 during the current item,
// its Q and first K / V tiles are loaded as soon as the tensor core has finished with the current Q, its first
// S = Q K^T products are issued while the softmax warps still write out the current O.
struct FwdItem {
  int mblk, h, b, hk, hm, hb;
};

__device__ __forceinline__ FwdItem fwd_item(const FwdKernelParams& p, int item) {
  FwdItem w;
  const int per_block = p.h * p.b;
  const int rem = item % per_block;
  w.mblk = p.n_mblk - 1 - item / per_block;
  w.h = rem % p.h;  // heads of one kv group are neighbours in the list: they meet their shared tiles in L2
  w.b = rem / p.h;
  w.hk = w.h / (p.h / p.h_k);
  w.hm = w.h / (p.h / p.h_mask);
  w.hb = w.h / (p.h / p.h_bias);
  return w;
}

// kBits (per-query kernel only): the mask holds one bit per key instead of one byte.
template <int D, bool kBf16, bool kBcast, bool kBits = false>
__global__ void __launch_bounds__(Smem<D>::kThreads, 1) fwd_kernel(const __grid_constant__ FwdKernelParams p) {
  using L = Smem<D>;
  constexpr int kNQ = L::kNQ, kStages = L::kStages;
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) &
                                                         ~static_cast<uintptr_t>(1023));
  unsigned char* s_q = smem + L::kQOff;
  unsigned char* s_kv = smem + L::kKvOff;
  float* s_bm = reinterpret_cast<float*>(smem + L::kBmOff);
  int* s_pos = reinterpret_cast<int*>(smem + L::kPosOff);
  uint8_t* s_flags_all = smem + L::kFlagsOff;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* bar_q = bars;                           // Q of the item has landed
  uint64_t* bar_q_empty = bars + 1;                 // the tensor core is done with the item's Q
  uint64_t* bar_kv_full = bars + 2;
  uint64_t* bar_kv_empty = bar_kv_full + kStages;
  uint64_t* bar_s_full = bar_kv_empty + kStages;    // [2]
  uint64_t* bar_p_full = bar_s_full + 2;            // [2]
  uint64_t* bar_o_done = bar_p_full + 2;            // every product of the item has completed
  uint64_t* bar_o_free = bar_o_done + 1;            // [2] the softmax warps have read O_t out of tensor memory
  uint64_t* bar_bm_full = bar_o_free + 2;
  uint64_t* bar_bm_empty = bar_bm_full + kBmSlots;
  uint64_t* bar_stagger = bar_bm_empty + kBmSlots;  // warpgroup 0 -> warpgroup 1, once
  uint64_t* bar_flags_full = bar_stagger + 1;       // [2]
  uint64_t* bar_flags_empty = bar_flags_full + 2;   // [2]
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(smem + L::kMiscOff);
  volatile int* s_abort = reinterpret_cast<volatile int*>(smem + L::kMiscOff + 4);
  volatile int* s_item = reinterpret_cast<volatile int*>(smem + L::kMiscOff + 8);  // [2]: item of the flag table
  constexpr int kFlagReaders = 3 + 4 * kNQ;  // producer, MMA issuer, addend warp, one arrival per softmax warp

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int Sq = p.seqlen_q, Sk = p.seqlen_k;
  const int off = Sk - Sq;
  const int nt_all = (Sk + kBN - 1) / kBN;
  const bool causal = p.is_causal != 0;
  const WaitCtl ctl{s_abort, p.status};
  // Per item: number of key tiles each query tile can see at most (causal / length limit), and their maximum.
  auto tile_limits = [&](const FwdItem& w, int (&n_end)[kNQ], const int32_t*& pos_row) {
    pos_row = nullptr;
    if (kBcast && causal && p.key_pos)  // compacted keys: the causal limit is tested on the keys' positions
      pos_row = p.key_pos + w.b * p.pos_batch_stride +
                (p.h_pos == p.h ? w.h : (p.h_pos == p.h_k ? w.hk : 0)) * p.pos_head_stride;
    int nT = 0;
#pragma unroll
    for (int t = 0; t < kNQ; ++t) {
      const int m0 = (w.mblk * kNQ + t) * kBM;
      int ne = nt_all;
      if (causal && !pos_row) ne = min(ne, max(0, (m0 + kBM + off + kBN - 1) / kBN));
      if (m0 >= Sq) ne = 0;
      n_end[t] = ne;
      nT = max(nT, ne);
    }
    return nT;
  };

  // ---------------- set-up: barriers, TMEM ----------------
  if (tid == 0) {
    *s_abort = 0;
    mbar_init(bar_q, 1);
    mbar_init(bar_q_empty, 1);
    for (int i = 0; i < kStages; ++i) {
      mbar_init(bar_kv_full + i, 1);
      mbar_init(bar_kv_empty + i, 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(bar_s_full + t, 1);
      mbar_init(bar_p_full + t, kBM);
      mbar_init(bar_o_free + t, 4);  // one arrival per softmax warp of the query tile
      mbar_init(bar_flags_full + t, 1);
      mbar_init(bar_flags_empty + t, kFlagReaders);
    }
    mbar_init(bar_o_done, 1);
    mbar_init(bar_stagger, kBM);
    for (int i = 0; i < kBmSlots; ++i) {
      mbar_init(bar_bm_full + i, 1);
      mbar_init(bar_bm_empty + i, 4 * kNQ);  // one arrival per softmax warp
    }
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(s_tmem, 512);
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    prefetch_tmap(&p.tm_q);
    prefetch_tmap(&p.tm_k);
    prefetch_tmap(&p.tm_v);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *s_tmem;

  // ---------------- roles ----------------
  if (warp < 4) {
  // (one query tile per CTA: 256 threads have 256 registers each available, nothing to re-partition)
  if (kNQ == 2) asm volatile("setmaxnreg.dec.sync.aligned.u32 64;");
  if (warp == 0) {
    if (lane == 0) {
      FDMA_PROF_BEGIN();
      int it = 0;
      bool ok = true;
      for (int ic = 0; ok; ++ic) {
        ok = mbar_wait(bar_flags_full + (ic & 1), (ic >> 1) & 1, ctl, kWaitFlagsFull);
        if (!ok) break;
        const int item = s_item[ic & 1];
        if (item >= p.n_items) break;
        const FwdItem w = fwd_item(p, item);
        int n_end[kNQ];
        const int32_t* pos_row;
        const int nT = tile_limits(w, n_end, pos_row);
        const uint8_t* s_flags = s_flags_all + (ic & 1) * kMaxTiles;
        ok = mbar_wait(bar_q_empty, (ic & 1) ^ 1, ctl, kWaitQEmpty);
        if (!ok) break;
        // Q tiles (rows beyond Sq are zero-filled by TMA)
        mbar_arrive_expect_tx(bar_q, kNQ * L::kQBytes);
#pragma unroll
        for (int t = 0; t < kNQ; ++t)
#pragma unroll
          for (int kb = 0; kb < D / 64; ++kb)
            tma_load_4d(s_q + t * L::kQBytes + kb * (kBM * 128), &p.tm_q, bar_q, kb * 64, w.h,
                        (w.mblk * kNQ + t) * kBM, w.b);
        for (int j = 0; j < nT && ok; ++j) {
          if (s_flags[j] == 0) continue;
#pragma unroll
          for (int kv = 0; kv < 2; ++kv) {
            const int slot = it % kStages;
            ok = FDMA_PROF_WAIT(0, mbar_wait(bar_kv_empty + slot, ((it / kStages) & 1) ^ 1, ctl, kWaitKvEmpty));
            if (!ok) break;
            mbar_arrive_expect_tx(bar_kv_full + slot, L::kKvBytes);
            const CUtensorMap* tm = kv == 0 ? &p.tm_k : &p.tm_v;
#pragma unroll
            for (int kb = 0; kb < D / 64; ++kb)
              tma_load_4d(s_kv + slot * L::kKvBytes + kb * (kBN * 128), tm, bar_kv_full + slot, kb * 64, w.hk, j * kBN,
                          w.b);
            ++it;
          }
        }
        mbar_arrive(bar_flags_empty + (ic & 1));
      }
      FDMA_PROF_END(0, true);
    }
  } else if (warp == 1) {
    // whole warp, uniform control flow; the issue wrappers elect one lane
    constexpr uint32_t idesc_qk = umma_idesc(kBM, kBN, kBf16, false, false);
    constexpr uint32_t idesc_pv = umma_idesc(kBM, D, kBf16, false, true);
    const uint32_t q_addr = smem_u32(s_q), kv_addr = smem_u32(s_kv);
    FDMA_PROF_BEGIN();
    int a = 0;                    // ring position: K of the a-th kept tile (over all items) is ring item 2a, V 2a+1
    uint32_t pcnt[2] = {0, 0};    // P hand-overs received per query tile, over all items (barrier parity)
    bool ok = true;
    for (int ic = 0; ok; ++ic) {
      ok = __all_sync(0xffffffffu, mbar_wait(bar_flags_full + (ic & 1), (ic >> 1) & 1, ctl, kWaitFlagsFull));
      if (!ok) break;
      const int item = s_item[ic & 1];
      if (item >= p.n_items) break;
      const FwdItem w = fwd_item(p, item);
      int n_end[kNQ];
      const int32_t* pos_row;
      const int nT = tile_limits(w, n_end, pos_row);
      const uint8_t* s_flags = s_flags_all + (ic & 1) * kMaxTiles;
      ok = __all_sync(0xffffffffu, FDMA_PROF_WAIT(0, mbar_wait(bar_q, ic & 1, ctl, kWaitQ)));
      if (!ok) break;
      tc_fence_after_sync();
      int prev_j = -1;            // previous kept tile of this item (its PV is still to be issued)
      uint32_t pv_done[2] = {0, 0};  // PV products issued for this item per query tile (0: the first one overwrites O)
      for (int j = 0; j <= nT && ok; ++j) {
        const bool last = (j == nT);
        const uint8_t fl = last ? 0 : s_flags[j];
        if (!last && fl == 0) continue;
        if (last && prev_j < 0) break;  // the item has no kept tile at all
        if (last) umma_commit(bar_q_empty);  // every S = Q K^T of the item has been issued: Q may be replaced as soon
                                             // as they complete, while the last P V products are still to come
        const uint8_t pfl = prev_j >= 0 ? s_flags[prev_j] : 0;
        const int k_it = 2 * a, v_it = 2 * (a - 1) + 1;
        if (!last) {
          ok = __all_sync(0xffffffffu, FDMA_PROF_WAIT(1, mbar_wait(bar_kv_full + (k_it % kStages), (k_it / kStages) & 1,
                                                                     ctl, kWaitKvFullK)));
          if (!ok) break;
        }
        if (prev_j >= 0) {
          ok = __all_sync(0xffffffffu, FDMA_PROF_WAIT(2, mbar_wait(bar_kv_full + (v_it % kStages), (v_it / kStages) & 1,
                                                                     ctl, kWaitKvFullV)));
          if (!ok) break;
        }
        tc_fence_after_sync();
#pragma unroll
        for (int t = 0; t < kNQ; ++t) {
          const uint32_t s_col = tmem_base + t * kBN;
          if (pfl & (1 << t)) {
            ok = __all_sync(0xffffffffu, FDMA_PROF_WAIT(3 + t, mbar_wait(bar_p_full + t, pcnt[t] & 1, ctl, kWaitP)));
            if (!ok) break;
            if (pv_done[t] == 0 && ic > 0) {  // the previous item's O_t must have left tensor memory
              ok = __all_sync(0xffffffffu, mbar_wait(bar_o_free + t, (ic - 1) & 1, ctl, kWaitOFree));
              if (!ok) break;
            }
            tc_fence_after_sync();
            const uint32_t o_col = tmem_base + kNQ * kBN + t * 128;
            const uint32_t v_base = kv_addr + (v_it % kStages) * L::kKvBytes;
#pragma unroll
            for (int kk = 0; kk < kBN / 16; ++kk) {
              const uint64_t bd = umma_desc_sw128(v_base + kk * 2048, kBN * 128, 1024);
              umma_ts(o_col, s_col + kk * 8, bd, idesc_pv, (pv_done[t] > 0 || kk > 0) ? 1u : 0u);
            }
            ++pcnt[t];
            ++pv_done[t];
          }
          if (fl & (1 << t)) {
            const uint32_t qa = q_addr + t * L::kQBytes;
            const uint32_t ka = kv_addr + (k_it % kStages) * L::kKvBytes;
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
              const uint32_t o2 = (kk >> 2) * (kBM * 128) + (kk & 3) * 32;
              umma_ss(s_col, umma_desc_sw128(qa + o2, 16, 1024), umma_desc_sw128(ka + o2, 16, 1024), idesc_qk,
                      kk > 0 ? 1u : 0u);
            }
            umma_commit(bar_s_full + t);
          }
        }
        if (!ok) break;
        if (prev_j >= 0) umma_commit(bar_kv_empty + (v_it % kStages));
        if (!last) umma_commit(bar_kv_empty + (k_it % kStages));
        if (!last) {
          prev_j = j;
          ++a;
        }
      }
      if (!ok) break;
      if (prev_j < 0) umma_commit(bar_q_empty);  // (an item without kept tiles never read its Q)
      umma_commit(bar_o_done);
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_flags_empty + (ic & 1));
    }
    FDMA_PROF_END(8, lane == 0);
  } else if (warp == 2) {
    // bias + mask of a key tile -> one fp32 addend per key (row-broadcast mode); other modes only release the flags
    int bi = 0;
    bool ok = true;
    for (int ic = 0; ok; ++ic) {
      ok = __all_sync(0xffffffffu, mbar_wait(bar_flags_full + (ic & 1), (ic >> 1) & 1, ctl, kWaitFlagsFull));
      if (!ok) break;
      const int item = s_item[ic & 1];
      if (item >= p.n_items) break;
      const FwdItem w = fwd_item(p, item);
      int n_end[kNQ];
      const int32_t* pos_row;
      const int nT = tile_limits(w, n_end, pos_row);
      const uint8_t* s_flags = s_flags_all + (ic & 1) * kMaxTiles;
      if (kBcast) {
        const uint8_t* mrow = p.mask ? p.mask + w.b * p.mask_batch_stride + w.hm * p.mask_head_stride : nullptr;
        const uint16_t* brow = p.bias ? reinterpret_cast<const uint16_t*>(p.bias) + w.b * p.bias_batch_stride +
                                            w.hb * p.bias_head_stride
                                      : nullptr;
        for (int j = 0; j < nT && ok; ++j) {
          if (s_flags[j] == 0) continue;
          const int slot = bi % kBmSlots;
          ok = __all_sync(0xffffffffu, mbar_wait(bar_bm_empty + slot, ((bi / kBmSlots) & 1) ^ 1, ctl, kWaitBmEmpty));
          if (!ok) break;
          const int k0 = j * kBN + lane * 4;
          float v[4];
          uint32_t mbits = 0x01010101u;
          if (mrow) mbits = *reinterpret_cast<const uint32_t*>(mrow + k0);
          uint2 braw = make_uint2(0u, 0u);
          if (brow) braw = *reinterpret_cast<const uint2*>(brow + k0);
          const uint16_t bh[4] = {static_cast<uint16_t>(braw.x & 0xFFFFu), static_cast<uint16_t>(braw.x >> 16),
                                  static_cast<uint16_t>(braw.y & 0xFFFFu), static_cast<uint16_t>(braw.y >> 16)};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            float bf;
            if (kBf16) bf = __uint_as_float(static_cast<uint32_t>(bh[i]) << 16);
            else bf = __half2float(__ushort_as_half(bh[i]));
            const bool keep = ((mbits >> (8 * i)) & 0xFFu) != 0 && (k0 + i) < Sk;
            v[i] = keep ? bf * kLog2e : -CUDART_INF_F;
          }
          *reinterpret_cast<float4*>(s_bm + slot * kBN + lane * 4) = make_float4(v[0], v[1], v[2], v[3]);
          if (pos_row) {
            int4 pv = make_int4(0x7FFFFFFF, 0x7FFFFFFF, 0x7FFFFFFF, 0x7FFFFFFF);
            if (k0 + 3 < Sk) {
              pv = *reinterpret_cast<const int4*>(pos_row + k0);
            } else {
              if (k0 < Sk) pv.x = pos_row[k0];
              if (k0 + 1 < Sk) pv.y = pos_row[k0 + 1];
              if (k0 + 2 < Sk) pv.z = pos_row[k0 + 2];
            }
            *reinterpret_cast<int4*>(s_pos + slot * kBN + lane * 4) = pv;
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_bm_full + slot);
          ++bi;
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_flags_empty + (ic & 1));
    }
  } else {
    // warp 3: tile flags of every item, one item ahead of the other roles. Bit t of flags[j] = key tile j is
    // processed for query tile t.
    bool ok = true;
    for (int ic = 0; ok; ++ic) {
      ok = __all_sync(0xffffffffu, mbar_wait(bar_flags_empty + (ic & 1), ((ic >> 1) & 1) ^ 1, ctl, kWaitFlagsEmpty));
      if (!ok) break;
      int item = 0;
      if (lane == 0) item = static_cast<int>(min(atomicAdd(p.sched, 1u), static_cast<unsigned>(p.n_items)));
      item = __shfl_sync(0xffffffffu, item, 0);
      if (lane == 0) s_item[ic & 1] = item;  // n_items = no item left: the other roles leave their loops on it
      if (item >= p.n_items) {
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_flags_full + (ic & 1));
        break;
      }
      const FwdItem w = fwd_item(p, item);
      int n_end[kNQ];
      const int32_t* pos_row;
      const int nT = tile_limits(w, n_end, pos_row);
      uint8_t* s_flags = s_flags_all + (ic & 1) * kMaxTiles;
      for (int j = lane; j < nT; j += 32) {
        uint8_t f = 0;
        if (kBcast) {
          bool any = true;
          if (p.mask) {
            const uint8_t* mrow = p.mask + w.b * p.mask_batch_stride + w.hm * p.mask_head_stride + j * kBN;
            uint32_t acc = 0;
#pragma unroll
            for (int i = 0; i < kBN / 16; ++i) {
              const uint4 v = *reinterpret_cast<const uint4*>(mrow + i * 16);
              uint32_t wd[4] = {v.x, v.y, v.z, v.w};
              if (j * kBN + i * 16 + 16 > Sk) {  // ragged last tile: drop keys >= Sk
#pragma unroll
                for (int e = 0; e < 16; ++e)
                  if (j * kBN + i * 16 + e >= Sk) wd[e >> 2] &= ~(0xFFu << ((e & 3) * 8));
              }
              acc |= wd[0] | wd[1] | wd[2] | wd[3];
            }
            any = acc != 0;
          }
          if (any) {
#pragma unroll
            for (int t = 0; t < kNQ; ++t)
              if (j < n_end[t]) f |= (1 << t);
            if (pos_row) {  // the tile's smallest position against the last row of each query tile
              const int64_t pmin = pos_row[j * kBN];
#pragma unroll
              for (int t = 0; t < kNQ; ++t) {
                const int qlast = min((w.mblk * kNQ + t) * kBM + kBM - 1, Sq - 1);
                if (pmin > static_cast<int64_t>(qlast) + p.causal_shift) f &= ~(1 << t);
              }
            }
          }
        } else {
#pragma unroll
          for (int t = 0; t < kNQ; ++t) {
            if (j < n_end[t]) {
              bool act = true;
              if (p.act) {
                const int MT = (Sq + kBM - 1) / kBM;
                act = p.act[((static_cast<int64_t>(w.b) * p.h_mask + w.hm) * MT + (w.mblk * kNQ + t)) * nt_all + j] != 0;
              }
              if (act) f |= (1 << t);
            }
          }
        }
        s_flags[j] = f;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_flags_full + (ic & 1));
    }
  }
  } else {
    if (kNQ == 2) asm volatile("setmaxnreg.inc.sync.aligned.u32 208;");
    // ---------------- softmax warpgroup for query tile t ----------------
    const int t = (warp - 4) >> 2;
    const int row = (warp & 3) * 32 + lane;          // row inside the tile == TMEM lane
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t s_taddr = tmem_base + lane_addr + t * kBN;
    const uint32_t o_taddr = tmem_base + lane_addr + kNQ * kBN + t * 128;
    FDMA_PROF_BEGIN();
    uint32_t scnt = 0;   // S tiles received over all items (barrier parity)
    int bi = 0;          // addend-ring position over all items
    bool ok = true;
    bool stagger_sent = false;
    for (int ic = 0; ok; ++ic) {
    ok = __all_sync(0xffffffffu, mbar_wait(bar_flags_full + (ic & 1), (ic >> 1) & 1, ctl, kWaitFlagsFull));
    if (!ok) break;
    const int item = s_item[ic & 1];
    if (item >= p.n_items) break;
    const FwdItem w = fwd_item(p, item);
    const int h = w.h, b = w.b;
    int n_end[kNQ];
    const int32_t* pos_row;
    const int nT = tile_limits(w, n_end, pos_row);
    const uint8_t* s_flags = s_flags_all + (ic & 1) * kMaxTiles;
    const int m0 = (w.mblk * kNQ + t) * kBM;
    const int qrow = m0 + row;
    const int qclamp = min(qrow, Sq - 1);
    const uint8_t* mrow = nullptr;
    const uint16_t* brow = nullptr;
    if (!kBcast) {
      if (p.mask)  // bit-packed: 4-byte units, i.e. the same expression on a word pointer
        mrow = p.mask + (b * p.mask_batch_stride + w.hm * p.mask_head_stride + qclamp * p.mask_row_stride) *
                            (kBits ? 4 : 1);
      if (p.bias)
        brow = reinterpret_cast<const uint16_t*>(p.bias) + b * p.bias_batch_stride + w.hb * p.bias_head_stride +
               qclamp * p.bias_row_stride;
    }
    // 32-byte loads of the row pieces where the tensors' alignment allows them
    const bool wide_m = ((reinterpret_cast<uintptr_t>(p.mask) | static_cast<uintptr_t>(p.mask_batch_stride) |
                          static_cast<uintptr_t>(p.mask_head_stride) | static_cast<uintptr_t>(p.mask_row_stride)) & 31) == 0;
    const bool wide_b = (reinterpret_cast<uintptr_t>(p.bias) & 31) == 0 &&
                        ((p.bias_batch_stride | p.bias_head_stride | p.bias_row_stride) & 15) == 0;
    float m_ref = -CUDART_INF_F, l = 0.f;
    uint32_t sitem = 0;  // S tiles of this item processed by this warpgroup
    // The two warpgroups share the transcendental unit; running their exp2 phases at the same time doubles the
    // length of both. Warpgroup 1 therefore starts only when warpgroup 0 reaches the exp2 phase of its first
    // tile, which keeps the two loops roughly half a period apart.
    if (kNQ == 2 && t == 1 && ic == 0) ok = __all_sync(0xffffffffu, mbar_wait(bar_stagger, 0, ctl, kWaitS));
    for (int j = 0; j < nT && ok; ++j) {
      const uint8_t fl = s_flags[j];
      if (fl == 0) continue;
      const int slot = bi % kBmSlots;
      if (kBcast) {
        ok = __all_sync(0xffffffffu, FDMA_PROF_WAIT(0, mbar_wait(bar_bm_full + slot, (bi / kBmSlots) & 1, ctl, kWaitBmFull)));
        if (!ok) break;
      }
      if (fl & (1 << t)) {
        const int kbase = j * kBN;
        const float2 sc2 = make_float2(p.scale_log2, p.scale_log2);
        // Per-query bias / mask: this row's 128 + 256 bytes of the tile are requested BEFORE the wait for the score
        // tile, so the load latency overlaps the wait; the scores then leave TMEM 32 columns at a time and take the
        // place of the addend registers they consume.
        uint32_t bw[kBcast ? 1 : 8][8], mw[(kBcast || kBits) ? 1 : 4][8];
        if (!kBcast) {
          // ... and of the next tile this row will process: into L2 while this tile is worked on
          int jn = j + 1;
          while (jn < nT && !(s_flags[jn] & (1 << t))) ++jn;
          if (jn < nT) {
            if (mrow) prefetch_l2(mrow + (kBits ? jn * (kBN / 8) : jn * kBN));
            if (brow) {
              prefetch_l2(brow + jn * kBN);
              prefetch_l2(brow + jn * kBN + 64);
            }
          }
#pragma unroll
          if (kBits) {  // 128 bits of this row: one 16-byte load, kept in mw[0][0..3]
            const uint4 mb = mrow ? ld_nc_v4(mrow + (kbase >> 3)) : make_uint4(~0u, ~0u, ~0u, ~0u);
            mw[0][0] = mb.x; mw[0][1] = mb.y; mw[0][2] = mb.z; mw[0][3] = mb.w;
          }
#pragma unroll
          for (int c2 = 0; c2 < 4; ++c2) {
            if (kBits) {
            } else if (!mrow) {
#pragma unroll
              for (int i = 0; i < 8; ++i) mw[c2][i] = 0x01010101u;
            } else if (wide_m) {
              ld_nc_v8(mrow + kbase + c2 * 32, mw[c2]);
            } else {
              const uint4 m0 = *reinterpret_cast<const uint4*>(mrow + kbase + c2 * 32);
              const uint4 m1 = *reinterpret_cast<const uint4*>(mrow + kbase + c2 * 32 + 16);
              mw[c2][0] = m0.x; mw[c2][1] = m0.y; mw[c2][2] = m0.z; mw[c2][3] = m0.w;
              mw[c2][4] = m1.x; mw[c2][5] = m1.y; mw[c2][6] = m1.z; mw[c2][7] = m1.w;
            }
          }
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            if (!brow) {
#pragma unroll
              for (int i = 0; i < 8; ++i) bw[c][i] = 0u;
            } else if (wide_b) {
              ld_nc_v8(brow + kbase + c * 16, bw[c]);
            } else {
              const uint4 b0 = *reinterpret_cast<const uint4*>(brow + kbase + c * 16);
              const uint4 b1 = *reinterpret_cast<const uint4*>(brow + kbase + c * 16 + 8);
              bw[c][0] = b0.x; bw[c][1] = b0.y; bw[c][2] = b0.z; bw[c][3] = b0.w;
              bw[c][4] = b1.x; bw[c][5] = b1.y; bw[c][6] = b1.z; bw[c][7] = b1.w;
            }
          }
        }
        ok = __all_sync(0xffffffffu, FDMA_PROF_WAIT(1, mbar_wait(bar_s_full + t, scnt & 1, ctl, kWaitS)));
        if (!ok) break;
        tc_fence_after_sync();
        // Scores are kept as 64 register pairs so that the scale/bias FMA, the max-subtraction and the row sum run
        // as packed fp32x2 instructions (half the issue slots of scalar code). Scores in log2 units with bias and
        // mask folded in.
        float2 s2[kBN / 2];
        if (kBcast) {
          uint32_t su[kBN];
#pragma unroll
          for (int c = 0; c < 4; ++c) tmem_ld_x32(s_taddr + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&su[c * 32]));
          tmem_wait_ld();
          const float4* bm4 = reinterpret_cast<const float4*>(s_bm + slot * kBN);
#pragma unroll
          for (int i = 0; i < kBN / 4; ++i) {
            const float4 a4 = bm4[i];
            s2[2 * i] = __ffma2_rn(make_float2(__uint_as_float(su[4 * i]), __uint_as_float(su[4 * i + 1])), sc2,
                                   make_float2(a4.x, a4.y));
            s2[2 * i + 1] = __ffma2_rn(make_float2(__uint_as_float(su[4 * i + 2]), __uint_as_float(su[4 * i + 3])), sc2,
                                       make_float2(a4.z, a4.w));
          }
        } else {
          const float2 l2e2 = make_float2(kLog2e, kLog2e);
#pragma unroll
          for (int c2 = 0; c2 < kBN / 32; ++c2) {
            uint32_t su[32];
            tmem_ld_x32(s_taddr + c2 * 32, su);
            tmem_wait_ld();
#pragma unroll
            for (int cc = 0; cc < 2; ++cc) {
              const int c = c2 * 2 + cc;  // 16-key chunk
#pragma unroll
              for (int i = 0; i < 8; ++i) {  // pair i of this 16-key chunk
                float2 bf;
                if (kBf16) {
                  bf = make_float2(__uint_as_float(bw[c][i] << 16), __uint_as_float(bw[c][i] & 0xFFFF0000u));
                } else {
                  const __half2 hh = *reinterpret_cast<const __half2*>(&bw[c][i]);
                  bf = make_float2(__low2float(hh), __high2float(hh));
                }
                float2 add = __fmul2_rn(bf, l2e2);
                if (kBits) {
                  const uint32_t mpair = mw[0][c2] >> (cc * 16 + 2 * i);
                  if ((mpair & 1u) == 0) add.x = -CUDART_INF_F;
                  if ((mpair & 2u) == 0) add.y = -CUDART_INF_F;
                } else {
                  const uint32_t mpair = mw[c2][cc * 4 + (i >> 1)] >> ((i & 1) * 16);
                  if ((mpair & 0xFFu) == 0) add.x = -CUDART_INF_F;
                  if ((mpair & 0xFF00u) == 0) add.y = -CUDART_INF_F;
                }
                s2[c * 8 + i] = __ffma2_rn(make_float2(__uint_as_float(su[cc * 16 + 2 * i]),
                                                       __uint_as_float(su[cc * 16 + 2 * i + 1])), sc2, add);
              }
            }
          }
        }
        // causal / length limit, only on tiles that cross it
        {
          int klim = Sk;  // keys < klim are visible to this row
          const int warp_q0 = m0 + (warp & 3) * 32;  // smallest query row of this warp
          int wlim = Sk;
          if (pos_row) {
            const int* tp = s_pos + slot * kBN;
            if (static_cast<int64_t>(tp[kBN - 1]) > static_cast<int64_t>(warp_q0) + p.causal_shift) {
              // positions ascend: the visible keys of this row are a prefix of the tile, found by bisection
              const int64_t lim = static_cast<int64_t>(qrow) + p.causal_shift;
              int cnt = 0;
#pragma unroll
              for (int step = kBN / 2; step > 0; step >>= 1)
                if (tp[cnt + step - 1] <= lim) cnt += step;
              if (cnt == kBN - 1 && tp[kBN - 1] <= lim) cnt = kBN;
              klim = min(klim, kbase + cnt);
              wlim = kbase;  // take the per-element path
            }
          } else if (causal) {
            klim = min(klim, qrow + off + 1);
            wlim = min(wlim, warp_q0 + off + 1);
          }
          if (kbase + kBN > wlim) {
#pragma unroll
            for (int i = 0; i < kBN / 2; ++i) {
              if (kbase + 2 * i >= klim) s2[i].x = -CUDART_INF_F;
              if (kbase + 2 * i + 1 >= klim) s2[i].y = -CUDART_INF_F;
            }
          }
        }
        float m_tile;
        {  // four independent chains of three-input max
          float mx[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
          for (int i = 0; i < kBN / 2; i += 4) {
            mx[0] = fmax3(mx[0], s2[i].x, s2[i].y);
            mx[1] = fmax3(mx[1], s2[i + 1].x, s2[i + 1].y);
            mx[2] = fmax3(mx[2], s2[i + 2].x, s2[i + 2].y);
            mx[3] = fmax3(mx[3], s2[i + 3].x, s2[i + 3].y);
          }
          m_tile = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
        }
        const bool need = m_tile > m_ref + kRescaleThreshold || (m_ref == -CUDART_INF_F && m_tile > m_ref);
        if (__any_sync(0xffffffffu, need)) {
          const float m_new = need ? fmaxf(m_ref, m_tile) : m_ref;
          const float alpha = (m_new == -CUDART_INF_F) ? 1.f : fast_exp2(m_ref - m_new);
          if (sitem > 0) {  // O_t holds earlier tiles: rescale it (their MMAs finished before this S arrived)
            uint32_t r[32];
#pragma unroll
            for (int c = 0; c < D / 32; ++c) {
              tmem_ld_x32(o_taddr + c * 32, r);
              tmem_wait_ld();
#pragma unroll
              for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
              tmem_st_x32(o_taddr + c * 32, r);
            }
            tmem_wait_st();
          }
          l *= alpha;
          m_ref = m_new;
        }
        if (t == 0 && !stagger_sent) {
          mbar_arrive(bar_stagger);
          stagger_sent = true;
        }
        const float m_use = (m_ref == -CUDART_INF_F) ? 0.f : m_ref;
        float2 ls[4] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
        const float2 nm2 = make_float2(-m_use, -m_use);
#pragma unroll
        for (int c = 0; c < kBN / 32; ++c) {
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float2 x = __fadd2_rn(s2[c * 16 + i], nm2);
            // a fixed subset of the pairs is exponentiated on the FMA pipe to unload the transcendental unit
            const float2 pp = ((kPolyPairs >> i) & 1) ? exp2_poly2(x) : make_float2(fast_exp2(x.x), fast_exp2(x.y));
            ls[i & 3] = __fadd2_rn(ls[i & 3], pp);
            pk[i] = pack_16x2<kBf16>(pp.x, pp.y);
          }
          tmem_st_x16(s_taddr + c * 16, pk);
        }
        {
          const float2 t01 = __fadd2_rn(ls[0], ls[1]), t23 = __fadd2_rn(ls[2], ls[3]);
          const float2 tt = __fadd2_rn(t01, t23);
          l += tt.x + tt.y;
        }
        tmem_wait_st();
        tc_fence_before_sync();
        mbar_arrive(bar_p_full + t);
        ++scnt;
        ++sitem;
      }
      if (kBcast) {
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_bm_empty + slot);
      }
      ++bi;
    }
    if (!ok) break;
    if (t == 0 && !stagger_sent) {  // no tile processed: release warpgroup 1 anyway
      mbar_arrive(bar_stagger);
      stagger_sent = true;
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(bar_flags_empty + (ic & 1));
    // ---------------- epilogue of the item ----------------
    ok = __all_sync(0xffffffffu, FDMA_PROF_WAIT(2, mbar_wait(bar_o_done, ic & 1, ctl, kWaitO)));
    if (!ok) break;
    tc_fence_after_sync();
    {
      const bool in_range = qrow < Sq;  // TMEM loads below are warp-collective: every lane runs them
      const bool wide_o = (reinterpret_cast<uintptr_t>(p.out) & 31) == 0 &&
                          ((p.o_batch_stride | p.o_row_stride | p.o_head_stride) & 15) == 0;
      // m_ref stays -inf iff every score of the row was masked (l can then hold 2^-125 terms of exp2_poly2)
      const bool alive = sitem > 0 && l > 0.f && m_ref != -CUDART_INF_F;
      const float inv = alive ? 1.f / l : 0.f;
      unsigned char* orow = reinterpret_cast<unsigned char*>(p.out) +
                            (b * p.o_batch_stride + static_cast<int64_t>(qclamp) * p.o_row_stride +
                             h * p.o_head_stride) * 2;
      if (in_range)
        p.lse[(static_cast<int64_t>(b) * p.h + h) * Sq + qrow] = alive ? (m_ref + fast_log2(l)) * kLn2 : CUDART_INF_F;
      if (sitem > 0) {
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t r[32];
          tmem_ld_x32(o_taddr + c * 32, r);
          tmem_wait_ld();
          if (c == D / 32 - 1) {  // O_t is in registers: the next item's first P V product may overwrite it
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_o_free + t);
          }
          if (in_range) {
#pragma unroll
            for (int v8 = 0; v8 < 2; ++v8) {   // 16 outputs = 32 bytes per store where the alignment allows
              uint32_t o[8];
#pragma unroll
              for (int e = 0; e < 8; ++e)
                o[e] = pack_16x2<kBf16>(__uint_as_float(r[v8 * 16 + 2 * e]) * inv,
                                        __uint_as_float(r[v8 * 16 + 2 * e + 1]) * inv);
              if (wide_o) {
                st_v8(orow + c * 64 + v8 * 32, o);
              } else {
                *reinterpret_cast<uint4*>(orow + c * 64 + v8 * 32) = make_uint4(o[0], o[1], o[2], o[3]);
                *reinterpret_cast<uint4*>(orow + c * 64 + v8 * 32 + 16) = make_uint4(o[4], o[5], o[6], o[7]);
              }
            }
          }
        }
      } else {
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_o_free + t);
        if (in_range) {
#pragma unroll
          for (int c = 0; c < D / 8; ++c) *reinterpret_cast<uint4*>(orow + c * 16) = make_uint4(0, 0, 0, 0);
        }
      }
    }
    }  // item loop
    FDMA_PROF_END(16, tid == 128);
    FDMA_PROF_END(24, tid == 256);
  }

  // ---------------- tear-down ----------------
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

// Item counters of the persistent forward: a ring of words in device memory that is part of the library image, one
// word per launch (zeroed on the launch's stream just before it). Launches only share a word when more than
// kSchedSlots of them are in flight on one device at the same time.
constexpr int kSchedSlots = 256;
__device__ unsigned g_fwd_sched[kSchedSlots];

unsigned* next_sched_slot() {
  static std::mutex mu;
  static unsigned* base[64] = {nullptr};
  static unsigned next[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (!base[dev]) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_fwd_sched) != cudaSuccess) return nullptr;
    base[dev] = static_cast<unsigned*>(ptr);
  }
  return base[dev] + (next[dev]++ % kSchedSlots);
}

struct FwdPlan {
  bool bcast;
  bool needs_act;
  size_t act_bytes;
};

FwdPlan plan(const fdma_fwd_params& p) {
  FwdPlan pl;
  const bool mask_b = !p.mask || p.mask_row_stride == 0 || p.seqlen_q == 1;
  const bool bias_b = !p.bias || p.bias_row_stride == 0 || p.seqlen_q == 1;
  pl.bcast = mask_b && bias_b;
  pl.needs_act = !pl.bcast && p.mask != nullptr;
  const size_t mt = (p.seqlen_q + kBM - 1) / kBM, nt = (p.seqlen_k + kBN - 1) / kBN;
  pl.act_bytes = pl.needs_act && !p.tile_activity ? align256(static_cast<size_t>(p.b) * p.h_mask * mt * nt) : 0;
  return pl;
}

bool aligned16(const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15u) == 0; }

template <int D, bool kBf16, bool kBcast, bool kBits = false>
int launch(const fdma_fwd_params& p, const FwdPlan& pl, cudaStream_t stream) {
  using L = Smem<D>;
  constexpr int kNQ = L::kNQ;
  FwdKernelParams kp;
  const uint32_t box[4] = {64, 1, static_cast<uint32_t>(kBM), 1};
  // Tensor maps over (d, heads, rows, batch). A dimension of extent 1 is never stepped over, so whatever stride
  // the caller reports for it is replaced by a dense one (the encoder wants non-zero multiples of 16 bytes).
  auto encode = [&](CUtensorMap* tm, const void* base, int heads, int rows, int64_t sb, int64_t sr, int64_t sh) {
    if (heads == 1) sh = p.d;
    if (rows == 1) sr = static_cast<int64_t>(heads) * p.d;
    if (p.b == 1) sb = static_cast<int64_t>(rows) * heads * p.d;
    const uint64_t dims[4] = {static_cast<uint64_t>(p.d), static_cast<uint64_t>(heads), static_cast<uint64_t>(rows),
                              static_cast<uint64_t>(p.b)};
    const uint64_t str[3] = {static_cast<uint64_t>(sh) * 2, static_cast<uint64_t>(sr) * 2,
                             static_cast<uint64_t>(sb) * 2};
    return encode_tmap_4d(tm, base, 2, dims, str, box);
  };
  int st = encode(&kp.tm_q, p.q, p.h, p.seqlen_q, p.q_batch_stride, p.q_row_stride, p.q_head_stride);
  if (st) return st;
  st = encode(&kp.tm_k, p.k, p.h_k, p.seqlen_k, p.k_batch_stride, p.k_row_stride, p.k_head_stride);
  if (st) return st;
  st = encode(&kp.tm_v, p.v, p.h_k, p.seqlen_k, p.v_batch_stride, p.v_row_stride, p.v_head_stride);
  if (st) return st;
  kp.mask = static_cast<const uint8_t*>(p.mask);
  kp.bias = p.bias;
  kp.out = p.out;
  kp.lse = p.lse;
  kp.act = nullptr;
  kp.status = kernel_status_ptr();
  if (!kp.status) return FDMA_ERR_DRIVER;
  kp.o_batch_stride = p.o_batch_stride; kp.o_row_stride = p.o_row_stride; kp.o_head_stride = p.o_head_stride;
  kp.mask_batch_stride = p.mask_batch_stride; kp.mask_head_stride = p.mask_head_stride;
  kp.mask_row_stride = p.mask_row_stride;
  kp.bias_batch_stride = p.bias_batch_stride; kp.bias_head_stride = p.bias_head_stride;
  kp.bias_row_stride = p.bias_row_stride;
  kp.b = p.b; kp.seqlen_q = p.seqlen_q; kp.seqlen_k = p.seqlen_k; kp.h = p.h; kp.h_k = p.h_k;
  kp.h_mask = p.h_mask; kp.h_bias = p.h_bias;
  kp.is_causal = p.is_causal;
  kp.key_pos = p.key_pos;
  kp.pos_batch_stride = p.key_pos_batch_stride; kp.pos_head_stride = p.key_pos_head_stride;
  kp.h_pos = p.h_pos; kp.causal_shift = p.causal_shift;
  kp.scale_log2 = p.softmax_scale * kLog2e;

  if (pl.needs_act && p.tile_activity) {
    kp.act = p.tile_activity;
  } else if (pl.needs_act) {
    if (!p.workspace || p.workspace_bytes < pl.act_bytes) return FDMA_ERR_WORKSPACE;
    uint8_t* act = static_cast<uint8_t*>(p.workspace);
    st = launch_tile_activity(p, act, stream);
    if (st) return st;
    kp.act = act;
  }

  auto kern = fwd_kernel<D, kBf16, kBcast, kBits>;
  // The attribute belongs to the (function, device) pair: set it on every call, whichever device is current.
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kAlloc);
  if (e != cudaSuccess) return static_cast<int>(e);
  kp.n_mblk = (p.seqlen_q + kNQ * kBM - 1) / (kNQ * kBM);
  const int64_t n_items = static_cast<int64_t>(kp.n_mblk) * p.h * p.b;
  if (n_items > 0x7FFFFFFF) return FDMA_ERR_TOO_LARGE;
  kp.n_items = static_cast<int>(n_items);
  dim3 grid(static_cast<unsigned>(std::min<int64_t>(n_items, sm_count())));  // persistent CTAs, one per SM
  kp.sched = next_sched_slot();
  if (!kp.sched) return FDMA_ERR_DRIVER;
  e = cudaMemsetAsync(kp.sched, 0, sizeof(unsigned), stream);
  if (e != cudaSuccess) return static_cast<int>(e);
  cudaEvent_t ev0, ev1;
  take_timing_events(&ev0, &ev1);
  if (ev0) cudaEventRecord(ev0, stream);
  kern<<<grid, L::kThreads, L::kAlloc, stream>>>(kp);
  if (ev1) cudaEventRecord(ev1, stream);
  return static_cast<int>(cudaGetLastError());
}

template <int D>
int launch_d(const fdma_fwd_params& p, const FwdPlan& pl, cudaStream_t stream) {
  if (p.dtype == FDMA_BF16) {
    if (pl.bcast) return launch<D, true, true>(p, pl, stream);
    return (p.mask && p.mask_bits) ? launch<D, true, false, true>(p, pl, stream) : launch<D, true, false>(p, pl, stream);
  }
  if (pl.bcast) return launch<D, false, true>(p, pl, stream);
  return (p.mask && p.mask_bits) ? launch<D, false, false, true>(p, pl, stream) : launch<D, false, false>(p, pl, stream);
}

}  // namespace

int launch_tile_activity(const fdma_fwd_params& p, uint8_t* act, cudaStream_t stream) {
  const int64_t tiles = static_cast<int64_t>(p.b) * p.h_mask * ((p.seqlen_q + kBM - 1) / kBM) *
                        ((p.seqlen_k + kBN - 1) / kBN);
  const int64_t blocks = (tiles * 32 + 255) / 256;
  tile_activity_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
      static_cast<const uint8_t*>(p.mask), p.mask_batch_stride, p.mask_head_stride,
      p.seqlen_q == 1 ? 0 : p.mask_row_stride, p.b, p.h_mask, p.seqlen_q, p.seqlen_k, p.is_causal, act);
  return static_cast<int>(cudaGetLastError());
}

bool tc_fwd_supported(const fdma_fwd_params& p) {
  if (p.d != 64 && p.d != 128 && p.d != 256) return false;
  if (p.seqlen_k <= 0 || p.seqlen_k > kMaxTiles * kBN) return false;
  if (p.h > 65535 || p.b > 65535) return false;
  // TMA: 16-byte aligned bases and strides
  const void* ptrs[4] = {p.q, p.k, p.v, p.out};
  for (const void* x : ptrs)
    if (!aligned16(x)) return false;
  auto ok_strides = [&](int heads, int rows, int64_t sb, int64_t sr, int64_t sh) {
    if (heads > 1 && (sh <= 0 || sh % 8)) return false;
    if (rows > 1 && (sr <= 0 || sr % 8)) return false;
    if (p.b > 1 && (sb <= 0 || sb % 8)) return false;
    return true;
  };
  if (!ok_strides(p.h, p.seqlen_q, p.q_batch_stride, p.q_row_stride, p.q_head_stride)) return false;
  if (!ok_strides(p.h_k, p.seqlen_k, p.k_batch_stride, p.k_row_stride, p.k_head_stride)) return false;
  if (!ok_strides(p.h_k, p.seqlen_k, p.v_batch_stride, p.v_row_stride, p.v_head_stride)) return false;
  if (p.o_batch_stride % 8 || p.o_row_stride % 8 || p.o_head_stride % 8) return false;
  // 16-byte vector loads of bias (2-byte elements) and mask (bytes)
  if (p.bias) {
    if (!aligned16(p.bias)) return false;
    if (p.bias_batch_stride % 8 || p.bias_head_stride % 8 || p.bias_row_stride % 8) return false;
  }
  if (p.mask && p.mask_bits) {  // bit-packed: per-query rows of 16-byte multiples, tile activity supplied
    if (!aligned16(p.mask) || !p.tile_activity) return false;
    if (p.mask_batch_stride % 4 || p.mask_head_stride % 4 || p.mask_row_stride % 4) return false;
    if (p.mask_row_stride == 0 || p.seqlen_q == 1) return false;
  } else if (p.mask) {
    if (!aligned16(p.mask)) return false;
    if (p.mask_batch_stride % 16 || p.mask_head_stride % 16 || p.mask_row_stride % 16) return false;
  }
  if (p.key_pos && p.is_causal) {  // key positions: broadcast mode only, 16-byte vector loads of int32
    if (!plan(p).bcast) return false;
    if (!aligned16(p.key_pos) || p.key_pos_batch_stride % 4 || p.key_pos_head_stride % 4) return false;
  }
  return true;
}

size_t tc_fwd_workspace_bytes(const fdma_fwd_params& p) { return plan(p).act_bytes; }

int tc_fwd(const fdma_fwd_params& p, cudaStream_t stream) {
  const FwdPlan pl = plan(p);
  if (p.d == 64) return launch_d<64>(p, pl, stream);
  if (p.d == 256) return launch_d<256>(p, pl, stream);
  return launch_d<128>(p, pl, stream);
}

}  // namespace fdma

#ifdef FDMA_PROF
// Tracing build only: forward kernel's wait-cycle counters. Slots: [0,8) producer, [8,16) MMA issuer,
// [16,24) one softmax thread of query tile 0, [24,32) one of query tile 1; slot 7 of each group is the lifetime.
extern "C" int fdma_prof_read_fwd(unsigned long long* out) {
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return static_cast<int>(e);
  e = cudaMemcpyFromSymbol(out, fdma::g_prof, sizeof(unsigned long long) * 64);
  if (e != cudaSuccess) return static_cast<int>(e);
  static const unsigned long long zeros[64] = {};
  return static_cast<int>(cudaMemcpyToSymbol(fdma::g_prof, zeros, sizeof(zeros)));
}
#endif
