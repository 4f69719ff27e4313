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
  kWaitO = 107, kWaitBmEmpty = 108, kWaitBmFull = 109
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
  static constexpr int kFlagsOff = kPosOff + kBmSlots * kBN * 4;
  static constexpr int kBarOff = kFlagsOff + kMaxTiles;
  static constexpr int kNumBars = 1 + 2 * kStages + 2 + 2 + 1 + 2 * kBmSlots + 1;
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

template <int D, bool kBf16, bool kBcast>
__global__ void __launch_bounds__(Smem<D>::kThreads, 1) fwd_kernel(const __grid_constant__ FwdKernelParams p) {
  using L = Smem<D>;
  constexpr int kNQ = L::kNQ, kStages = L::kStages, kThreads = L::kThreads;
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) &
                                                         ~static_cast<uintptr_t>(1023));
  unsigned char* s_q = smem + L::kQOff;
  unsigned char* s_kv = smem + L::kKvOff;
  float* s_bm = reinterpret_cast<float*>(smem + L::kBmOff);
  int* s_pos = reinterpret_cast<int*>(smem + L::kPosOff);
  uint8_t* s_flags = smem + L::kFlagsOff;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* bar_q = bars;
  uint64_t* bar_kv_full = bars + 1;
  uint64_t* bar_kv_empty = bar_kv_full + kStages;
  uint64_t* bar_s_full = bar_kv_empty + kStages;  // [2]
  uint64_t* bar_p_full = bar_s_full + 2;          // [2]
  uint64_t* bar_o_done = bar_p_full + 2;
  uint64_t* bar_bm_full = bar_o_done + 1;
  uint64_t* bar_bm_empty = bar_bm_full + kBmSlots;
  uint64_t* bar_stagger = bar_bm_empty + kBmSlots;  // warpgroup 0 -> warpgroup 1, once
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(smem + L::kMiscOff);
  volatile int* s_abort = reinterpret_cast<volatile int*>(smem + L::kMiscOff + 4);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // Query block and head of this CTA. Heaviest (latest) query blocks first under causal masking. Per-query masks
  // and biases are read from global memory by every head that shares them, so in that mode the heads of one kv
  // group take consecutive CTA indices for the same query block and meet their shared tiles in L2.
  int mblk = gridDim.x - 1 - blockIdx.x;
  int h = blockIdx.y;
  if (!kBcast) {
    const int G = p.h / p.h_k;
    const int lin = blockIdx.x + gridDim.x * blockIdx.y;
    h = (lin / (G * static_cast<int>(gridDim.x))) * G + lin % G;
    mblk = gridDim.x - 1 - (lin / G) % gridDim.x;
  }
  const int b = blockIdx.z;
  const int hk = h / (p.h / p.h_k);
  const int hm = h / (p.h / p.h_mask);
  const int hb = h / (p.h / p.h_bias);
  const int Sq = p.seqlen_q, Sk = p.seqlen_k;
  const int off = Sk - Sq;
  const int nt_all = (Sk + kBN - 1) / kBN;
  const bool causal = p.is_causal != 0;
  // Compacted keys: the causal limit is tested on the keys' original positions (ascending along the tile index).
  const int32_t* pos_row = nullptr;
  if (kBcast && causal && p.key_pos)
    pos_row = p.key_pos + b * p.pos_batch_stride +
              (p.h_pos == p.h ? h : (p.h_pos == p.h_k ? hk : 0)) * p.pos_head_stride;

  int n_end[kNQ];
#pragma unroll
  for (int t = 0; t < kNQ; ++t) {
    const int m0 = (mblk * kNQ + t) * kBM;
    int ne = nt_all;
    if (causal && !pos_row) ne = min(ne, max(0, (m0 + kBM + off + kBN - 1) / kBN));
    if (m0 >= Sq) ne = 0;
    n_end[t] = ne;
  }
  const int nT = max(n_end[0], n_end[kNQ - 1]);
  const WaitCtl ctl{s_abort, p.status};

  // ---------------- set-up: barriers, TMEM, tile flags ----------------
  if (tid == 0) {
    *s_abort = 0;
    mbar_init(bar_q, 1);
    for (int i = 0; i < kStages; ++i) {
      mbar_init(bar_kv_full + i, 1);
      mbar_init(bar_kv_empty + i, 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(bar_s_full + t, 1);
      mbar_init(bar_p_full + t, kBM);
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
  // Tile flags: bit t of s_flags[j] = key tile j is processed for query tile t.
  for (int j = tid; j < nT; j += kThreads) {
    uint8_t f = 0;
    if (kBcast) {
      bool any = true;
      if (p.mask) {
        const uint8_t* mrow = p.mask + b * p.mask_batch_stride + hm * p.mask_head_stride + j * kBN;
        uint32_t acc = 0;
#pragma unroll
        for (int i = 0; i < kBN / 16; ++i) {
          const uint4 v = *reinterpret_cast<const uint4*>(mrow + i * 16);
          uint32_t w[4] = {v.x, v.y, v.z, v.w};
          if (j * kBN + i * 16 + 16 > Sk) {  // ragged last tile: drop keys >= Sk
#pragma unroll
            for (int e = 0; e < 16; ++e)
              if (j * kBN + i * 16 + e >= Sk) w[e >> 2] &= ~(0xFFu << ((e & 3) * 8));
          }
          acc |= w[0] | w[1] | w[2] | w[3];
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
            const int qlast = min((mblk * kNQ + t) * kBM + kBM - 1, Sq - 1);
            if (pmin > static_cast<int64_t>(qlast) + p.causal_shift) f &= ~(1 << t);
          }
        }
      }
    } else {
#pragma unroll
      for (int t = 0; t < kNQ; ++t) {
        if (j < n_end[t]) {
          bool a = true;
          if (p.act) {
            const int MT = (Sq + kBM - 1) / kBM;
            a = p.act[((static_cast<int64_t>(b) * p.h_mask + hm) * MT + (mblk * kNQ + t)) * nt_all + j] != 0;
          }
          if (a) f |= (1 << t);
        }
      }
    }
    s_flags[j] = f;
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
    if (lane == 0 && nT > 0) {
      FDMA_PROF_BEGIN();
      // Q tiles (rows beyond Sq are zero-filled by TMA)
      mbar_arrive_expect_tx(bar_q, kNQ * L::kQBytes);
#pragma unroll
      for (int t = 0; t < kNQ; ++t)
#pragma unroll
        for (int kb = 0; kb < D / 64; ++kb)
          tma_load_4d(s_q + t * L::kQBytes + kb * (kBM * 128), &p.tm_q, bar_q, kb * 64, h, (mblk * kNQ + t) * kBM, b);
      int it = 0;
      bool ok = true;
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
            tma_load_4d(s_kv + slot * L::kKvBytes + kb * (kBN * 128), tm, bar_kv_full + slot, kb * 64, hk, j * kBN, b);
          ++it;
        }
      }
      FDMA_PROF_END(0, true);
    }
  } else if (warp == 1) {
    if (nT > 0) {  // whole warp, uniform control flow; the issue wrappers elect one lane
      constexpr uint32_t idesc_qk = umma_idesc(kBM, kBN, kBf16, false, false);
      constexpr uint32_t idesc_pv = umma_idesc(kBM, D, kBf16, false, true);
      const uint32_t q_addr = smem_u32(s_q), kv_addr = smem_u32(s_kv);
      FDMA_PROF_BEGIN();
      bool ok = __all_sync(0xffffffffu, FDMA_PROF_WAIT(0, mbar_wait(bar_q, 0, ctl, kWaitQ)));
      tc_fence_after_sync();
      int a = 0;            // index of the current kept tile; its K is ring item 2a, its V item 2a+1
      int prev_j = -1;      // previous kept tile (its PV is still to be issued)
      uint32_t pcnt[2] = {0, 0};
      for (int j = 0; j <= nT && ok; ++j) {
        const bool last = (j == nT);
        const uint8_t fl = last ? 0 : s_flags[j];
        if (!last && fl == 0) continue;
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
            tc_fence_after_sync();
            const uint32_t o_col = tmem_base + kNQ * kBN + t * 128;
            const uint32_t v_base = kv_addr + (v_it % kStages) * L::kKvBytes;
#pragma unroll
            for (int kk = 0; kk < kBN / 16; ++kk) {
              const uint64_t bd = umma_desc_sw128(v_base + kk * 2048, kBN * 128, 1024);
              umma_ts(o_col, s_col + kk * 8, bd, idesc_pv, (pcnt[t] > 0 || kk > 0) ? 1u : 0u);
            }
            ++pcnt[t];
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
      umma_commit(bar_o_done);
      FDMA_PROF_END(8, lane == 0);
    }
  } else if (warp == 2) {
    if (kBcast) {
      const uint8_t* mrow = p.mask ? p.mask + b * p.mask_batch_stride + hm * p.mask_head_stride : nullptr;
      const uint16_t* brow = p.bias ? reinterpret_cast<const uint16_t*>(p.bias) + b * p.bias_batch_stride +
                                          hb * p.bias_head_stride
                                    : nullptr;
      int bi = 0;
      bool ok = true;
      for (int j = 0; j < nT && ok; ++j) {
        if (s_flags[j] == 0) continue;
        const int slot = bi % kBmSlots;
        ok = mbar_wait(bar_bm_empty + slot, ((bi / kBmSlots) & 1) ^ 1, ctl, kWaitBmEmpty);
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
  }
  } else {
    if (kNQ == 2) asm volatile("setmaxnreg.inc.sync.aligned.u32 208;");
    // ---------------- softmax warpgroup for query tile t ----------------
    const int t = (warp - 4) >> 2;
    const int row = (warp & 3) * 32 + lane;          // row inside the tile == TMEM lane
    const int m0 = (mblk * kNQ + t) * kBM;
    const int qrow = m0 + row;
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t s_taddr = tmem_base + lane_addr + t * kBN;
    const uint32_t o_taddr = tmem_base + lane_addr + kNQ * kBN + t * 128;
    const int qclamp = min(qrow, Sq - 1);
    const uint8_t* mrow = nullptr;
    const uint16_t* brow = nullptr;
    if (!kBcast) {
      if (p.mask) mrow = p.mask + b * p.mask_batch_stride + hm * p.mask_head_stride + qclamp * p.mask_row_stride;
      if (p.bias)
        brow = reinterpret_cast<const uint16_t*>(p.bias) + b * p.bias_batch_stride + hb * p.bias_head_stride +
               qclamp * p.bias_row_stride;
    }
    float m_ref = -CUDART_INF_F, l = 0.f;
    FDMA_PROF_BEGIN();
    uint32_t scnt = 0;
    int bi = 0;
    bool ok = true;
    // The two warpgroups share the transcendental unit; running their exp2 phases at the same time doubles the
    // length of both. Warpgroup 1 therefore starts only when warpgroup 0 reaches the exp2 phase of its first
    // tile, which keeps the two loops roughly half a period apart.
    bool stagger_sent = false;
    if (kNQ == 2 && t == 1) ok = __all_sync(0xffffffffu, mbar_wait(bar_stagger, 0, ctl, kWaitS));
    for (int j = 0; j < nT && ok; ++j) {
      const uint8_t fl = s_flags[j];
      if (fl == 0) continue;
      const int slot = bi % kBmSlots;
      if (kBcast) {
        ok = __all_sync(0xffffffffu, FDMA_PROF_WAIT(0, mbar_wait(bar_bm_full + slot, (bi / kBmSlots) & 1, ctl, kWaitBmFull)));
        if (!ok) break;
      }
      if (fl & (1 << t)) {
        ok = __all_sync(0xffffffffu, FDMA_PROF_WAIT(1, mbar_wait(bar_s_full + t, scnt & 1, ctl, kWaitS)));
        if (!ok) break;
        tc_fence_after_sync();
        // Scores are kept as 64 register pairs so that the scale/bias FMA, the max-subtraction and the row sum run
        // as packed fp32x2 instructions (half the issue slots of scalar code).
        float2 s2[kBN / 2];
        {
          uint32_t su[kBN];
#pragma unroll
          for (int c = 0; c < 4; ++c) tmem_ld_x32(s_taddr + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&su[c * 32]));
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < kBN / 2; ++i) s2[i] = make_float2(__uint_as_float(su[2 * i]), __uint_as_float(su[2 * i + 1]));
        }
        const int kbase = j * kBN;
        const float2 sc2 = make_float2(p.scale_log2, p.scale_log2);
        if (!kBcast) {
          // this row's mask and bias bytes of the next tile it will process: into L2 while this tile is worked on
          int jn = j + 1;
          while (jn < nT && !(s_flags[jn] & (1 << t))) ++jn;
          if (jn < nT) {
            if (mrow) prefetch_l2(mrow + jn * kBN);
            if (brow) {
              prefetch_l2(brow + jn * kBN);
              prefetch_l2(brow + jn * kBN + 64);
            }
          }
        }
        // scores in log2 units with bias and mask folded in
        if (kBcast) {
          const float4* bm4 = reinterpret_cast<const float4*>(s_bm + slot * kBN);
#pragma unroll
          for (int i = 0; i < kBN / 4; ++i) {
            const float4 a4 = bm4[i];
            s2[2 * i] = __ffma2_rn(s2[2 * i], sc2, make_float2(a4.x, a4.y));
            s2[2 * i + 1] = __ffma2_rn(s2[2 * i + 1], sc2, make_float2(a4.z, a4.w));
          }
        } else {
          const float2 l2e2 = make_float2(kLog2e, kLog2e);
#pragma unroll
          for (int c = 0; c < kBN / 16; ++c) {
            uint4 mb = make_uint4(0x01010101u, 0x01010101u, 0x01010101u, 0x01010101u);
            if (mrow) mb = *reinterpret_cast<const uint4*>(mrow + kbase + c * 16);
            uint4 b0 = make_uint4(0, 0, 0, 0), b1 = make_uint4(0, 0, 0, 0);
            if (brow) {
              b0 = *reinterpret_cast<const uint4*>(brow + kbase + c * 16);
              b1 = *reinterpret_cast<const uint4*>(brow + kbase + c * 16 + 8);
            }
            const uint32_t mw[4] = {mb.x, mb.y, mb.z, mb.w};
            const uint32_t bw[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i) {  // pair i of this 16-key chunk
              float2 bf;
              if (kBf16) {
                bf = make_float2(__uint_as_float(bw[i] << 16), __uint_as_float(bw[i] & 0xFFFF0000u));
              } else {
                const __half2 hh = *reinterpret_cast<const __half2*>(&bw[i]);
                bf = make_float2(__low2float(hh), __high2float(hh));
              }
              float2 add = __fmul2_rn(bf, l2e2);
              const uint32_t mpair = mw[i >> 1] >> ((i & 1) * 16);
              if ((mpair & 0xFFu) == 0) add.x = -CUDART_INF_F;
              if ((mpair & 0xFF00u) == 0) add.y = -CUDART_INF_F;
              s2[c * 8 + i] = __ffma2_rn(s2[c * 8 + i], sc2, add);
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
          if (scnt > 0) {  // O_t holds earlier tiles: rescale it (their MMAs finished before this S arrived)
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
      }
      if (kBcast) {
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_bm_empty + slot);
      }
      ++bi;
    }
    if (t == 0 && !stagger_sent) mbar_arrive(bar_stagger);  // no tile processed: release warpgroup 1 anyway
    // ---------------- epilogue ----------------
    if (ok && nT > 0) ok = __all_sync(0xffffffffu, FDMA_PROF_WAIT(2, mbar_wait(bar_o_done, 0, ctl, kWaitO)));
    FDMA_PROF_END(16, tid == 128);
    FDMA_PROF_END(24, tid == 256);
    tc_fence_after_sync();
    if (ok) {
      const bool in_range = qrow < Sq;  // TMEM loads below are warp-collective: every lane runs them
      // m_ref stays -inf iff every score of the row was masked (l can then hold 2^-125 terms of exp2_poly2)
      const bool alive = scnt > 0 && l > 0.f && m_ref != -CUDART_INF_F;
      const float inv = alive ? 1.f / l : 0.f;
      unsigned char* orow = reinterpret_cast<unsigned char*>(p.out) +
                            (b * p.o_batch_stride + static_cast<int64_t>(qclamp) * p.o_row_stride +
                             h * p.o_head_stride) * 2;
      if (in_range)
        p.lse[(static_cast<int64_t>(b) * p.h + h) * Sq + qrow] = alive ? (m_ref + fast_log2(l)) * kLn2 : CUDART_INF_F;
      if (scnt > 0) {
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t r[32];
          tmem_ld_x32(o_taddr + c * 32, r);
          tmem_wait_ld();
          if (in_range) {
#pragma unroll
            for (int v4 = 0; v4 < 4; ++v4) {
              uint4 o;
              o.x = pack_16x2<kBf16>(__uint_as_float(r[v4 * 8 + 0]) * inv, __uint_as_float(r[v4 * 8 + 1]) * inv);
              o.y = pack_16x2<kBf16>(__uint_as_float(r[v4 * 8 + 2]) * inv, __uint_as_float(r[v4 * 8 + 3]) * inv);
              o.z = pack_16x2<kBf16>(__uint_as_float(r[v4 * 8 + 4]) * inv, __uint_as_float(r[v4 * 8 + 5]) * inv);
              o.w = pack_16x2<kBf16>(__uint_as_float(r[v4 * 8 + 6]) * inv, __uint_as_float(r[v4 * 8 + 7]) * inv);
              *reinterpret_cast<uint4*>(orow + c * 64 + v4 * 16) = o;
            }
          }
        }
      } else if (in_range) {
#pragma unroll
        for (int c = 0; c < D / 8; ++c) *reinterpret_cast<uint4*>(orow + c * 16) = make_uint4(0, 0, 0, 0);
      }
    }
  }

  // ---------------- tear-down ----------------
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
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
  pl.act_bytes = pl.needs_act ? align256(static_cast<size_t>(p.b) * p.h_mask * mt * nt) : 0;
  return pl;
}

bool aligned16(const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15u) == 0; }

template <int D, bool kBf16, bool kBcast>
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

  if (pl.needs_act) {
    if (!p.workspace || p.workspace_bytes < pl.act_bytes) return FDMA_ERR_WORKSPACE;
    uint8_t* act = static_cast<uint8_t*>(p.workspace);
    st = launch_tile_activity(p, act, stream);
    if (st) return st;
    kp.act = act;
  }

  auto kern = fwd_kernel<D, kBf16, kBcast>;
  // The attribute belongs to the (function, device) pair: set it on every call, whichever device is current.
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kAlloc);
  if (e != cudaSuccess) return static_cast<int>(e);
  dim3 grid((p.seqlen_q + kNQ * kBM - 1) / (kNQ * kBM), p.h, p.b);
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
    return pl.bcast ? launch<D, true, true>(p, pl, stream) : launch<D, true, false>(p, pl, stream);
  }
  return pl.bcast ? launch<D, false, true>(p, pl, stream) : launch<D, false, false>(p, pl, stream);
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
  if (p.mask) {
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
