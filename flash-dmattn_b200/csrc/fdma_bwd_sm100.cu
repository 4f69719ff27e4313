// Backward dynamic-mask attention for sm_100a (head dim 128): dQ, dK, dV and dBias from dO, O, LSE.
//
// Math of the reference's compute_dq_dk_dv_1colblock (csrc/flash_sparse_attn/src/flash_bwd_kernel.h:79-1142):
//   P = exp(S - LSE), dP = dO V^T, dS = P o (dP - D), D = rowsum(dO o O),
//   dV = P^T dO, dK = scale dS^T Q, dQ = scale dS K, dBias = dS,
// laid out for tcgen05 instead of mma.sync. One CTA owns one tile of 128 keys of one (batch, kv head) and walks
// over every 64-row query tile of every query head that shares the kv head, so dK, dV and dBias leave the CTA
// already summed over the head group (the reference writes per-query-head temporaries and reduces them on the
// host with at::sum_out, flash_api.cpp:970-983, :1027-1047). Everything is computed TRANSPOSED so that the
// softmax threads own one KEY each (TMEM lane = key):
//   St  = K Q^T        (128 keys x 64 queries, SS MMA)        dPt = V dO^T        (SS MMA)
//   P^T, dS^T          written back into the St / dPt columns as 16-bit, used as the A operand (from TMEM) of
//   dV += P^T dO,  dK += dS^T Q   (B = dO / Q tiles read MN-major from the same shared-memory copy)
//   dQ^T = K^T dS^T    (A = K MN-major, B = dS^T staged in shared memory), added to an fp32 dQ buffer by a
//                      dedicated warpgroup: transpose through shared memory, one bulk reduce-add per 32 queries
// Query-broadcast bias gives dBias = column sums of dS: one fp32 register per softmax thread for the whole CTA.
//
// Warps: 0 TMA producer | 1 MMA issuer | 4-7, 8-11 softmax (query columns 0-31 / 32-63) | 12-15 dQ writer.
// TMEM: St[2] 2x64 | dPt 64 | dQ^T 64 | dV 128 | dK 128 = 512 columns.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math_constants.h>

#include <algorithm>

#include "fdma_internal.h"
#include "fdma_ptx.cuh"

namespace fdma {
namespace {

constexpr int kD = 128;
constexpr int kBN = 128;  // keys per CTA
constexpr int kBM = 64;   // query rows per step
constexpr int kQStages = 3;
constexpr int kThreads = 512;
constexpr int kMaxAct = 4096;  // bytes of the per-CTA tile-activity table
constexpr int kDetFracBits = 40;  // deterministic dQ: |dQ / scale| < 2^23, resolution 2^-40
constexpr float kLog2e = 1.4426950408889634f;

enum DbiasMode { kDbNone = 0, kDbColsum = 1, kDbDirect = 2, kDbAtomic = 3 };


enum WaitCode {
  kWaitKv = 201, kWaitQdoEmpty = 202, kWaitQdoFull = 203, kWaitSFull = 204, kWaitDpFull = 205, kWaitPds = 206,
  kWaitDqFull = 207, kWaitDqEmpty = 208, kWaitDpFree = 209, kWaitFinal = 210
};

struct BwdKernelParams {
  CUtensorMap tm_q, tm_do, tm_k, tm_v;  // q/do: 64-row boxes, k/v: 128-row boxes
  const uint8_t* mask;
  const void* bias;
  const float* lse2;   // (B,H,Sq_r) LSE * log2(e); +inf for empty and padded rows
  const float* dsum;   // (B,H,Sq_r) D = rowsum(dO o O)
  float* dq_acc;       // (B,H,Sq,128) fp32, zeroed by the launcher; deterministic kernels: the same shape in 64-bit
                       // fixed point (kDetFracBits fractional bits), whose sums do not depend on the order of addition
  void* dk;
  void* dv;
  void* dbias;         // direct / column-sum modes: the output tensor
  float* dbias_acc;    // atomic mode: fp32 buffer (dbias_b, dbias_h, dbias_rows, dbias_keys), zeroed
  float* dkv_part;     // nsplit > 1: fp32 partials [2: dV, dK][nsplit][B][h_k][NT*128][128]
  float* dbias_part;   // nsplit > 1, column-sum mode: fp32 partials [nsplit][B][h_k][NT*128]
  int nsplit;          // query-range splits per key tile
  const uint8_t* act;  // per-query mask: activity bytes [B][h_mask][ceil(Sq/128)][ceil(Sk/128)], else null
  int mask_bits;       // per-query mask given as one bit per key (uint32 words, strides in words)
  int* status;
  int64_t mask_batch_stride, mask_head_stride, mask_row_stride;
  int64_t bias_batch_stride, bias_head_stride, bias_row_stride;
  int64_t dk_batch_stride, dk_row_stride, dk_head_stride;
  int64_t dv_batch_stride, dv_row_stride, dv_head_stride;
  int64_t dbias_batch_stride, dbias_head_stride, dbias_row_stride;
  int b, seqlen_q, seqlen_k, sq_r, h, h_k, h_mask, h_bias;
  int dbias_b, dbias_h, dbias_rows, dbias_keys, dbias_mode;
  int is_causal;
  const int32_t* key_pos;  // ascending positions of compacted keys, or null
  int64_t pos_batch_stride, pos_head_stride;
  int h_pos, causal_shift;
  float scale_log2, scale;
};

struct SmemB {
  static constexpr int kKOff = 0;
  static constexpr int kVOff = kBN * kD * 2;                       // 32 KB
  static constexpr int kQdoOff = 2 * kBN * kD * 2;                 // 64 KB
  static constexpr int kQBytes = kBM * kD * 2;                     // 16 KB
  static constexpr int kStageBytes = 2 * kQBytes;                  // Q then dO
  static constexpr int kDsOff = kQdoOff + kQStages * kStageBytes;  // 160 KB
  static constexpr int kDsBytes = kBN * kBM * 2;                   // 16 KB
  static constexpr int kActOff = kDsOff + 2 * kDsBytes;            // 192 KB
  static constexpr int kLdOff = kActOff + kMaxAct;                 // per stage: 64 x LSE*log2e, 64 x D (fp32)
  static constexpr int kLdBytes = 2 * kBM * 4;
  static constexpr int kDqOff = kLdOff + kQStages * kLdBytes;      // [32 q][128 d] fp32 staging tile of the dQ writer
  static constexpr int kTrOff = kDqOff + 32 * kD * 4;              // per softmax warp: 1 KB transposition scratch
  static constexpr int kTrBytes = 8 * 1024;
  static constexpr int kRedOff = kTrOff + kTrBytes;
  static constexpr int kBarOff = kRedOff + kBN * 4;
  static constexpr int kNumBars = 1 + 2 * kQStages + 2 + 2 + 1 + 1 + 1 + 1;
  static constexpr int kMiscOff = kBarOff + kNumBars * 8;
  static constexpr int kTotal = kMiscOff + 32;
  static constexpr int kAlloc = kTotal + 1024;
};

// D = rowsum(dO o O), LSE in log2 units; rows [Sq, Sq_r) are padding (+inf / 0). Head dim 128: sixteen lanes hold
// one row (16 B each), a warp covers eight consecutive query rows of one (b, h) with all loads issued up front.
template <bool kBf16>
__global__ void __launch_bounds__(256) bwd_prep_kernel(const void* __restrict__ out, const void* __restrict__ dout,
                                                        const float* __restrict__ lse, float* __restrict__ lse2,
                                                        float* __restrict__ dsum, int B, int H, int Sq, int Sq_r,
                                                        int64_t ob, int64_t orow, int64_t oh, int64_t gb, int64_t grow,
                                                        int64_t gh) {
  const int lane = threadIdx.x & 31, sub = lane >> 4, l16 = lane & 15;
  const int64_t w = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5;
  const int groups = Sq_r / 8;
  const int64_t total = static_cast<int64_t>(B) * H * groups;
  if (w >= total) return;
  const int q0 = static_cast<int>(w % groups) * 8;
  const int h = static_cast<int>((w / groups) % H);
  const int b = static_cast<int>(w / (static_cast<int64_t>(groups) * H));
  const uint16_t* o = reinterpret_cast<const uint16_t*>(out) + b * ob + h * oh + l16 * 8;
  const uint16_t* g = reinterpret_cast<const uint16_t*>(dout) + b * gb + h * gh + l16 * 8;
  uint4 a[4], c[4];
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const int q = q0 + u * 2 + sub;
    a[u] = c[u] = make_uint4(0, 0, 0, 0);
    if (q < Sq) {
      a[u] = *reinterpret_cast<const uint4*>(o + static_cast<int64_t>(q) * orow);
      c[u] = *reinterpret_cast<const uint4*>(g + static_cast<int64_t>(q) * grow);
    }
  }
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    const uint32_t aw[4] = {a[u].x, a[u].y, a[u].z, a[u].w}, cw[4] = {c[u].x, c[u].y, c[u].z, c[u].w};
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float a0, a1, c0, c1;
      if (kBf16) {
        a0 = __uint_as_float(aw[j] << 16); a1 = __uint_as_float(aw[j] & 0xFFFF0000u);
        c0 = __uint_as_float(cw[j] << 16); c1 = __uint_as_float(cw[j] & 0xFFFF0000u);
      } else {
        const __half2 ah = *reinterpret_cast<const __half2*>(&aw[j]);
        const __half2 ch = *reinterpret_cast<const __half2*>(&cw[j]);
        a0 = __low2float(ah); a1 = __high2float(ah); c0 = __low2float(ch); c1 = __high2float(ch);
      }
      acc = fmaf(a0, c0, acc);
      acc = fmaf(a1, c1, acc);
    }
#pragma unroll
    for (int sft = 8; sft > 0; sft >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, sft);
    const int q = q0 + u * 2 + sub;
    if (l16 == 0) {
      const int64_t idx = (static_cast<int64_t>(b) * H + h) * Sq_r + q;
      if (q < Sq) {
        lse2[idx] = lse[(static_cast<int64_t>(b) * H + h) * Sq + q] * kLog2e;
        dsum[idx] = acc;
      } else {
        lse2[idx] = CUDART_INF_F;
        dsum[idx] = 0.f;
      }
    }
  }
}

// fp32 dQ accumulator (B,H,Sq,128) * scale -> dq (B,Sq,H,128 strided, 16-bit)
template <bool kBf16>
__global__ void bwd_convert_dq_kernel(const float* __restrict__ acc, void* __restrict__ dq, int64_t n_vec, int Sq,
                                      int H, int64_t sb, int64_t sr, int64_t sh, float scale) {
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n_vec;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t e = i * 8;
    const int dd = static_cast<int>(e % kD);
    const int q = static_cast<int>((e / kD) % Sq);
    const int h = static_cast<int>((e / (static_cast<int64_t>(kD) * Sq)) % H);
    const int b = static_cast<int>(e / (static_cast<int64_t>(kD) * Sq * H));
    const float4 x = *reinterpret_cast<const float4*>(acc + e);
    const float4 y = *reinterpret_cast<const float4*>(acc + e + 4);
    uint4 o;
    o.x = pack_16x2<kBf16>(x.x * scale, x.y * scale);
    o.y = pack_16x2<kBf16>(x.z * scale, x.w * scale);
    o.z = pack_16x2<kBf16>(y.x * scale, y.y * scale);
    o.w = pack_16x2<kBf16>(y.z * scale, y.w * scale);
    *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(dq) + b * sb + q * sr + h * sh + dd) = o;
  }
}

// Deterministic mode: 64-bit fixed-point accumulator -> 16-bit dQ.
template <bool kBf16>
__global__ void bwd_convert_dq_fixed_kernel(const long long* __restrict__ acc, void* __restrict__ dq, int64_t n_vec,
                                            int Sq, int H, int64_t sb, int64_t sr, int64_t sh, float scale,
                                            const float* __restrict__ dsum, int sq_r) {
  const float unit = scale * (1.0f / static_cast<float>(1ll << kDetFracBits));
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n_vec;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t e = i * 8;
    const int dd = static_cast<int>(e % kD);
    const int q = static_cast<int>((e / kD) % Sq);
    const int h = static_cast<int>((e / (static_cast<int64_t>(kD) * Sq)) % H);
    const int b = static_cast<int>(e / (static_cast<int64_t>(kD) * Sq * H));
    float x[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const longlong2 v = *reinterpret_cast<const longlong2*>(acc + e + 2 * j);
      x[2 * j] = __ll2float_rn(v.x) * unit;
      x[2 * j + 1] = __ll2float_rn(v.y) * unit;
    }
    // Fixed point cannot carry NaN / Inf. A non-finite dO or O element makes D = rowsum(dO o O) of its row
    // non-finite, and with it every dS of the row: such rows come out as NaN, as the fp32 path would give.
    if (!isfinite(dsum[(static_cast<int64_t>(b) * H + h) * sq_r + q])) {
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] = __int_as_float(0x7FC00000);
    }
    uint4 o;
    o.x = pack_16x2<kBf16>(x[0], x[1]);
    o.y = pack_16x2<kBf16>(x[2], x[3]);
    o.z = pack_16x2<kBf16>(x[4], x[5]);
    o.w = pack_16x2<kBf16>(x[6], x[7]);
    *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(dq) + b * sb + q * sr + h * sh + dd) = o;
  }
}

// fp32 (nb,nh,nr,nk) contiguous -> strided 16-bit dbias
template <bool kBf16>
__global__ void bwd_convert_dbias_kernel(const float* __restrict__ acc, void* __restrict__ out, int nb, int nh,
                                         int nr, int nk, int64_t sb, int64_t sh, int64_t sr) {
  const int64_t n = static_cast<int64_t>(nb) * nh * nr * nk;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int kk = static_cast<int>(i % nk);
    const int rr = static_cast<int>((i / nk) % nr);
    const int hh = static_cast<int>((i / (static_cast<int64_t>(nk) * nr)) % nh);
    const int bb = static_cast<int>(i / (static_cast<int64_t>(nk) * nr * nh));
    const uint32_t pk = pack_16x2<kBf16>(acc[i], 0.f);
    reinterpret_cast<uint16_t*>(out)[bb * sb + hh * sh + rr * sr + kk] = static_cast<uint16_t>(pk & 0xFFFFu);
  }
}

template <bool kBf16>
__device__ __forceinline__ float raw16_to_float(uint16_t u) {
  if (kBf16) return __uint_as_float(static_cast<uint32_t>(u) << 16);
  return __half2float(__ushort_as_half(u));
}
template <bool kBf16>
__device__ __forceinline__ uint16_t float_to_raw16(float x) {
  return static_cast<uint16_t>(pack_16x2<kBf16>(x, 0.f) & 0xFFFFu);
}

template <bool kBf16, bool kBcast, bool kDet>
__global__ void __launch_bounds__(kThreads, 1) bwd_kernel(const __grid_constant__ BwdKernelParams p) {
  using L = SmemB;
  // Row-broadcast kernel: the two softmax warpgroups are two teams that take alternate steps (all 64 queries of
  // a step, in two passes of 32), so the fixed latencies of one team's step -- barrier round trips, TMEM loads and
  // stores, the hand-over to the MMA warp -- overlap the other team's arithmetic. Per-query kernel: both warpgroups
  // work on every step, 32 queries each.
  constexpr bool kTeams = kBcast;
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) &
                                                         ~static_cast<uintptr_t>(1023));
  unsigned char* s_k = smem + L::kKOff;
  unsigned char* s_v = smem + L::kVOff;
  unsigned char* s_qdo = smem + L::kQdoOff;
  unsigned char* s_ds = smem + L::kDsOff;
  uint8_t* s_act = smem + L::kActOff;
  float* s_ld = reinterpret_cast<float*>(smem + L::kLdOff);
  float* s_red = reinterpret_cast<float*>(smem + L::kRedOff);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* bar_kv = bars;
  uint64_t* bar_qdo_full = bars + 1;
  uint64_t* bar_qdo_empty = bar_qdo_full + kQStages;
  uint64_t* bar_dp_full = bar_qdo_empty + kQStages;
  uint64_t* bar_pds = bar_dp_full + 2;              // bar_dp_full: [2], by step parity
  uint64_t* bar_dq_full = bar_pds + 2;              // bar_pds: [2], one per softmax team (broadcast kernel)
  uint64_t* bar_dq_empty = bar_dq_full + 1;
  uint64_t* bar_dp_free = bar_dq_empty + 1;
  uint64_t* bar_final = bar_dp_free + 1;
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(smem + L::kMiscOff);
  volatile int* s_abort = reinterpret_cast<volatile int*>(smem + L::kMiscOff + 4);
  int* s_nsteps = reinterpret_cast<int*>(smem + L::kMiscOff + 8);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int hk = blockIdx.y, b = blockIdx.z;
  const int G = p.h / p.h_k;
  const int Sq = p.seqlen_q, Sk = p.seqlen_k;
  const int off = Sk - Sq;
  const int MT = (Sq + 127) / 128;
  const int NT = (Sk + kBN - 1) / kBN;
  // blockIdx.x = (query-range split, key tile). With more than one split a CTA covers the 64-row query tiles
  // [m_lo, M64) of its key tile and leaves fp32 partial dK / dV / column sums for a reduction kernel. The last
  // query ranges, which causal masking never empties, are scheduled first.
  const int n = blockIdx.x % NT;  // key tile
  const int split = p.nsplit - 1 - blockIdx.x / NT;
  const int M64_all = (Sq + kBM - 1) / kBM;
  const int m_chunk = (M64_all + p.nsplit - 1) / p.nsplit;
  const int m_lo = split * m_chunk;
  const int M64 = min(M64_all, m_lo + m_chunk);  // end of this CTA's query range
  const bool causal = p.is_causal != 0;
  const int act_g = (p.h_mask == p.h && G > 1) ? G : 1;  // activity differs per query head only for per-head masks
  // Compacted keys carry their original positions (ascending); the causal test then runs on positions.
  const int32_t* pos_row = nullptr;
  if (causal && p.key_pos)
    pos_row = p.key_pos + b * p.pos_batch_stride + (p.h_pos == p.h_k ? hk : 0) * p.pos_head_stride;
  const int coff = pos_row ? p.causal_shift : off;
  int m_start = 0;
  if (pos_row) {
    const int64_t first = (static_cast<int64_t>(pos_row[n * kBN]) - coff) / kBM;
    m_start = static_cast<int>(max(static_cast<int64_t>(0), min(first, static_cast<int64_t>(M64))));
  } else if (causal) {
    m_start = max(0, (n * kBN - off) / kBM);  // first query tile with a row that sees key n*128
  }
  m_start = max(m_start, m_lo);
  const WaitCtl ctl{s_abort, p.status};

  // ---------------- set-up ----------------
  if (tid == 0) {
    *s_abort = 0;
    mbar_init(bar_kv, 1);
    for (int i = 0; i < kQStages; ++i) {
      mbar_init(bar_qdo_full + i, 1);
      mbar_init(bar_qdo_empty + i, 1);
    }
    mbar_init(bar_dp_full + 0, 1);
    mbar_init(bar_dp_full + 1, 1);
    mbar_init(bar_pds + 0, kTeams ? 4 : 8);  // one arrival per softmax warp that works on the step
    mbar_init(bar_pds + 1, kTeams ? 4 : 8);
    mbar_init(bar_dq_full, 1);
    mbar_init(bar_dq_empty, 4);   // one arrival per dQ-writer warp
    mbar_init(bar_dp_free, kTeams ? 4 : 8);
    mbar_init(bar_final, 1);
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(s_tmem, 512);
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    prefetch_tmap(&p.tm_q);
    prefetch_tmap(&p.tm_do);
    prefetch_tmap(&p.tm_k);
    prefetch_tmap(&p.tm_v);
  }
  // activity table: s_act[ga * MT + mt] != 0 iff (128-row query tile mt, this key tile) holds a kept element
  for (int idx = tid; idx < act_g * MT; idx += kThreads) {
    const int ga = idx / MT, mt = idx % MT;
    const int hq = hk * G + (act_g > 1 ? ga : 0);
    const int hm = hq / (p.h / p.h_mask);
    uint8_t a = 1;
    if (p.mask) {
      if (kBcast || p.mask_row_stride == 0) {
        const uint8_t* mrow = p.mask + b * p.mask_batch_stride + hm * p.mask_head_stride + n * kBN;
        uint32_t accw = 0;
#pragma unroll
        for (int i = 0; i < kBN / 16; ++i) {
          const uint4 v = *reinterpret_cast<const uint4*>(mrow + i * 16);
          uint32_t w[4] = {v.x, v.y, v.z, v.w};
          if (n * kBN + i * 16 + 16 > Sk) {
#pragma unroll
            for (int e = 0; e < 16; ++e)
              if (n * kBN + i * 16 + e >= Sk) w[e >> 2] &= ~(0xFFu << ((e & 3) * 8));
          }
          accw |= w[0] | w[1] | w[2] | w[3];
        }
        a = accw != 0;
      } else if (p.act) {
        a = p.act[((static_cast<int64_t>(b) * p.h_mask + hm) * MT + mt) * NT + n];
      }
    }
    s_act[idx] = a;
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == 1) {
    int cnt = 0;
    for (int m = m_start + lane; m < M64; m += 32)
      for (int g = 0; g < G; ++g) cnt += s_act[(act_g > 1 ? g : 0) * MT + (m >> 1)] ? 1 : 0;
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, s);
    if (lane == 0) *s_nsteps = cnt;
  }
  __syncthreads();
  const uint32_t tmem_base = *s_tmem;
  const int n_steps = *s_nsteps;
  constexpr uint32_t kColSt = 0, kColDp = 128, kColDq = 192, kColDv = 256, kColDk = 384;

  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
    if (warp == 0) {
      // ---------------- TMA producer ----------------
      if (lane == 0 && n_steps > 0) {
        FDMA_PROF_BEGIN();
        mbar_arrive_expect_tx(bar_kv, 2 * kBN * kD * 2);
#pragma unroll
        for (int kb = 0; kb < 2; ++kb) {
          tma_load_4d(s_k + kb * (kBN * 128), &p.tm_k, bar_kv, kb * 64, hk, n * kBN, b);
          tma_load_4d(s_v + kb * (kBN * 128), &p.tm_v, bar_kv, kb * 64, hk, n * kBN, b);
        }
        int i = 0;
        bool ok = true;
        for (int m = m_start; m < M64 && ok; ++m) {
          for (int g = 0; g < G; ++g) {
            if (!s_act[(act_g > 1 ? g : 0) * MT + (m >> 1)]) continue;
            const int stage = i % kQStages;
            ok = FDMA_PROF_WAIT(0, mbar_wait(bar_qdo_empty + stage, ((i / kQStages) & 1) ^ 1, ctl, kWaitQdoEmpty));
            if (!ok) break;
            mbar_arrive_expect_tx(bar_qdo_full + stage, L::kStageBytes + L::kLdBytes);
            unsigned char* dst = s_qdo + stage * L::kStageBytes;
            const int h = hk * G + g;
            const int64_t row0 = (static_cast<int64_t>(b) * p.h + h) * p.sq_r + m * kBM;
            bulk_load_1d(s_ld + stage * (2 * kBM), p.lse2 + row0, kBM * 4, bar_qdo_full + stage);
            bulk_load_1d(s_ld + stage * (2 * kBM) + kBM, p.dsum + row0, kBM * 4, bar_qdo_full + stage);
#pragma unroll
            for (int kb = 0; kb < 2; ++kb) {
              tma_load_4d(dst + kb * (kBM * 128), &p.tm_q, bar_qdo_full + stage, kb * 64, h, m * kBM, b);
              tma_load_4d(dst + L::kQBytes + kb * (kBM * 128), &p.tm_do, bar_qdo_full + stage, kb * 64, h, m * kBM, b);
            }
            ++i;
          }
        }
        FDMA_PROF_END(0, true);
      }
    } else if (warp == 1) {
      // ---------------- MMA issuer (whole warp, uniform control flow; the issue wrappers elect one lane) -------
      if (n_steps > 0) {
        constexpr uint32_t idesc_s = umma_idesc(kBN, kBM, kBf16, false, false);  // St/dPt: 128 x 64, K-major
        constexpr uint32_t idesc_g = umma_idesc(kBN, kD, kBf16, false, true);    // dV/dK: A from TMEM, B MN-major
        constexpr uint32_t idesc_q = umma_idesc(kD, kBM, kBf16, true, true);     // dQ^T: both MN-major
        const uint32_t k_addr = smem_u32(s_k), v_addr = smem_u32(s_v), qdo_addr = smem_u32(s_qdo),
                       ds_addr = smem_u32(s_ds);
        auto issue_st = [&](int step) {  // St[step & 1] = K Q^T
          const uint32_t qa = qdo_addr + (step % kQStages) * L::kStageBytes;
#pragma unroll
          for (int kk = 0; kk < kD / 16; ++kk) {
            const uint32_t ko = (kk >> 2) * (kBN * 128) + (kk & 3) * 32;
            const uint32_t qo = (kk >> 2) * (kBM * 128) + (kk & 3) * 32;
            umma_ss(tmem_base + kColSt + (step & 1) * kBM, umma_desc_sw128(k_addr + ko, 16, 1024),
                    umma_desc_sw128(qa + qo, 16, 1024), idesc_s, kk > 0 ? 1u : 0u);
          }
        };
        auto issue_dp = [&](int step) {  // dPt = V dO^T; the commit covers S of the same step, issued just before
          const uint32_t ga = qdo_addr + (step % kQStages) * L::kStageBytes + L::kQBytes;
#pragma unroll
          for (int kk = 0; kk < kD / 16; ++kk) {
            const uint32_t ko = (kk >> 2) * (kBN * 128) + (kk & 3) * 32;
            const uint32_t qo = (kk >> 2) * (kBM * 128) + (kk & 3) * 32;
            umma_ss(tmem_base + kColDp, umma_desc_sw128(v_addr + ko, 16, 1024), umma_desc_sw128(ga + qo, 16, 1024),
                    idesc_s, kk > 0 ? 1u : 0u);
          }
          umma_commit(bar_dp_full + (step & 1));
        };
        FDMA_PROF_BEGIN();
        bool ok = __all_sync(0xffffffffu, FDMA_PROF_WAIT(0, mbar_wait(bar_kv, 0, ctl, kWaitKv)));
        if (ok) ok = __all_sync(0xffffffffu, FDMA_PROF_WAIT(1, mbar_wait(bar_qdo_full + 0, 0, ctl, kWaitQdoFull)));
        if (ok) {
          tc_fence_after_sync();
          issue_st(0);
          issue_dp(0);
        }
        if (ok && n_steps > 1) {
          ok = __all_sync(0xffffffffu, FDMA_PROF_WAIT(1, mbar_wait(bar_qdo_full + 1, 0, ctl, kWaitQdoFull)));
          if (ok) {
            tc_fence_after_sync();
            issue_st(1);
          }
          if (ok) ok = __all_sync(0xffffffffu, FDMA_PROF_WAIT(3, mbar_wait(bar_dp_free, 0, ctl, kWaitDpFree)));
          if (ok) {
            tc_fence_after_sync();
            issue_dp(1);
          }
        }
        for (int i = 0; i < n_steps && ok; ++i) {
          ok = __all_sync(0xffffffffu, FDMA_PROF_WAIT(2, mbar_wait(bar_pds + (i & 1), (i >> 1) & 1, ctl, kWaitPds)));
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t stage_addr = qdo_addr + (i % kQStages) * L::kStageBytes;
          const uint32_t acc = i > 0 ? 1u : 0u;
          // A operands from TMEM, 16-bit pairs: each softmax pass writes back into the 32 columns of the St block it
          // read -- P^T of queries 0-31 in columns [0,16), their dS^T in [16,32); queries 32-63 in [32,48) and
          // [48,64). dS^T does not go back into the dPt block, so dP of a later step never waits for the dK product.
#pragma unroll
          for (int s = 0; s < 4; ++s) {
            const uint32_t a_col = 16 + (s < 2 ? s * 8 : 32 + (s - 2) * 8);
            umma_ts(tmem_base + kColDk, tmem_base + kColSt + (i & 1) * kBM + a_col,
                    umma_desc_sw128(stage_addr + s * 2048, kBM * 128, 1024), idesc_g, (acc || s > 0) ? 1u : 0u);
          }
#pragma unroll
          for (int s = 0; s < 4; ++s) {
            const uint32_t a_col = (s < 2 ? s * 8 : 32 + (s - 2) * 8);
            umma_ts(tmem_base + kColDv, tmem_base + kColSt + (i & 1) * kBM + a_col,
                    umma_desc_sw128(stage_addr + L::kQBytes + s * 2048, kBM * 128, 1024), idesc_g,
                    (acc || s > 0) ? 1u : 0u);
          }
          if (i > 0) {
            ok = __all_sync(0xffffffffu, FDMA_PROF_WAIT(3, mbar_wait(bar_dq_empty, (i - 1) & 1, ctl, kWaitDqEmpty)));
            if (!ok) break;
            tc_fence_after_sync();
          }
          // dQ^T = K^T dS^T : 8 k-steps of 16 keys
#pragma unroll
          for (int s = 0; s < kBN / 16; ++s) {
            umma_ss(tmem_base + kColDq, umma_desc_sw128(k_addr + s * 2048, kBN * 128, 1024),
                    umma_desc_sw128(ds_addr + (i & 1) * L::kDsBytes + s * 2048, 16, 1024), idesc_q, s > 0 ? 1u : 0u);
          }
          umma_commit(bar_dq_full);
          umma_commit(bar_qdo_empty + (i % kQStages));
          if (i + 2 < n_steps) {
            ok = __all_sync(0xffffffffu, FDMA_PROF_WAIT(1, mbar_wait(bar_qdo_full + ((i + 2) % kQStages),
                                                                     ((i + 2) / kQStages) & 1, ctl, kWaitQdoFull)));
            if (!ok) break;
            tc_fence_after_sync();
            issue_st(i + 2);
            // dP of step i+2 goes out two steps ahead as well, as soon as the softmax threads have read dP of step
            // i+1 out of the (single) dPt block -- which they do at the start of their step, long before this point.
            ok = __all_sync(0xffffffffu, FDMA_PROF_WAIT(3, mbar_wait(bar_dp_free, (i + 1) & 1, ctl, kWaitDpFree)));
            if (!ok) break;
            tc_fence_after_sync();
            issue_dp(i + 2);
          }
        }
        umma_commit(bar_final);
        FDMA_PROF_END(8, lane == 0);
      }
    }
  } else if (warp < 12) {
    // 65536 registers = 128 x 56 (warps 0-3) + 256 x 184 (softmax) + 128 x 88 (dQ writer); the deterministic writer
    // converts to 64-bit fixed point and keeps 104, leaving the softmax warps 176. (184 / 88 against 176 / 104:
    // 2-3 % on the backward kernel of the 32k benchmark; 192 and more for the softmax warps make the others spill.)
    if constexpr (kDet) asm volatile("setmaxnreg.inc.sync.aligned.u32 176;");
    else asm volatile("setmaxnreg.inc.sync.aligned.u32 184;");
    // ---------------- softmax warpgroups: thread = key, half = which 32 query columns ----------------
    const int half = (warp - 4) >> 2;
    const int krow = (warp & 3) * 32 + lane;  // key inside the tile == TMEM lane
    const int key = n * kBN + krow;
    unsigned char* s_tr = smem + L::kTrOff + (warp - 4) * 1024;
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const bool key_ok = key < Sk;
    // value compared with q + coff in the causal test: the key's position
    // (clamped so that ckey - coff cannot overflow; padding slots hold INT_MAX and are masked out anyway)
    const int ckey = pos_row ? (key_ok ? min(pos_row[key], 0x3FFFFFFF) : 0x3FFFFFFF) : key;
    const int ckey_wmax = pos_row ? __shfl_sync(0xffffffffu, ckey, 31) : n * kBN + (warp & 3) * 32 + 31;
    const int mode = p.dbias_mode;
    float colsum = 0.f;       // column-sum mode
    float dacc[32];           // direct mode with dbias_h == h_k: sum over the head group
#pragma unroll
    for (int j = 0; j < 32; ++j) dacc[j] = 0.f;
    const bool direct_group = mode == kDbDirect && p.dbias_h != p.h;  // one dbias head per kv head
    uint16_t* dbias16 = reinterpret_cast<uint16_t*>(p.dbias);
    // Direct mode: a warp's 32 queries x 32 keys of dBias leave through its transposition scratch as 16-byte row
    // pieces (64 bytes per row) when the tensor allows it; `vals` null stores zeros.
    const bool db_vec = mode == kDbDirect && (reinterpret_cast<uintptr_t>(p.dbias) & 15u) == 0 &&
                        ((p.dbias_batch_stride | p.dbias_head_stride | p.dbias_row_stride) & 7) == 0 &&
                        n * kBN + (warp & 3) * 32 + 32 <= p.dbias_keys;
    auto store_dbias = [&](uint16_t* dst_key, int q_first, const float* vals) {  // dst_key: (query 0, this key)
      if (db_vec) {
        uint16_t* tr16 = reinterpret_cast<uint16_t*>(s_tr);
        const uint4* tr4 = reinterpret_cast<const uint4*>(s_tr);
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          if (vals) {
#pragma unroll
            for (int j = 0; j < 16; ++j) tr16[j * 32 + lane] = float_to_raw16<kBf16>(vals[r * 16 + j]);
            __syncwarp();
          }
#pragma unroll
          for (int t = 0; t < 2; ++t) {
            const int row = q_first + r * 16 + t * 8 + (lane >> 2);
            if (row < Sq)
              *reinterpret_cast<uint4*>(dst_key - lane + static_cast<int64_t>(row) * p.dbias_row_stride + (lane & 3) * 8) =
                  vals ? tr4[lane + 32 * t] : make_uint4(0, 0, 0, 0);
          }
          if (vals) __syncwarp();
        }
      } else if (key < p.dbias_keys) {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (q_first + j < Sq)
            dst_key[static_cast<int64_t>(q_first + j) * p.dbias_row_stride] = vals ? float_to_raw16<kBf16>(vals[j]) : 0;
      }
    };
    // Row-broadcast bias / mask that do not depend on the query head: one value per thread for the whole CTA.
    const bool group_inv = G == 1 || ((!p.bias || p.h_bias != p.h) && (!p.mask || p.h_mask != p.h));
    const bool hoist = kBcast && group_inv;
    // mask / bias head of query head h, without integer division (extents are 1, h_k or h)
    auto hm_of = [&](int h) { return p.h_mask == p.h ? h : (p.h_mask == p.h_k ? hk : 0); };
    auto hb_of = [&](int h) { return p.h_bias == p.h ? h : (p.h_bias == p.h_k ? hk : 0); };
    float bv_h = -CUDART_INF_F;  // bias*log2e of this key, or -inf when the key is masked out
    if (hoist) {
      const int hm0 = hm_of(hk * G), hb0 = hb_of(hk * G);
      bool kp = key_ok;
      if (p.mask && kp) kp = p.mask[b * p.mask_batch_stride + hm0 * p.mask_head_stride + key] != 0;
      if (kp)
        bv_h = p.bias ? raw16_to_float<kBf16>(reinterpret_cast<const uint16_t*>(
                            p.bias)[b * p.bias_batch_stride + hb0 * p.bias_head_stride + key]) * kLog2e
                      : 0.f;
    }
    int i = 0;
    bool ok = true;
    FDMA_PROF_BEGIN();
    const int m_first = (mode == kDbDirect) ? m_lo : m_start;  // direct mode also zero-fills tiles it skips
    for (int m = m_first; m < M64 && ok; ++m) {
      const int q0 = m * kBM + half * 32;
      bool group_touched = false;
      // Per-query bias / mask shared by the query heads of the group: the 32 (query, key) addends of this thread are
      // fetched for the first active head of the query tile and reused by the others.
      float2 bias2[16];
      bool bias2_loaded = false;
      for (int g = 0; g < G && ok; ++g) {
        const int h = hk * G + g;
        const bool active = m >= m_start && s_act[(act_g > 1 ? g : 0) * MT + (m >> 1)] != 0;
        if (!active) {
          if (mode == kDbDirect && !direct_group)
            store_dbias(dbias16 + b * p.dbias_batch_stride + h * p.dbias_head_stride + key, q0, nullptr);
          continue;
        }
        if (kTeams && (i & 1) != half) {  // the other team's step
          ++i;
          continue;
        }
        group_touched = true;
        // ---- bias (log2 units) for this thread's key; masked elements get -inf, which turns into
        //      P = exp2(-inf) = 0 without any per-element select. Row-broadcast bias: one scalar per thread; the
        //      per-element array is only filled for per-query bias/mask and on tiles that cross the causal limit ----
        float bv = bv_h;
        if (kBcast) {
          if (!hoist) {
            const int hm = hm_of(h), hb = hb_of(h);
            bool kp = key_ok;
            if (p.mask && kp) kp = p.mask[b * p.mask_batch_stride + hm * p.mask_head_stride + key] != 0;
            bv = -CUDART_INF_F;
            if (kp)
              bv = p.bias ? raw16_to_float<kBf16>(reinterpret_cast<const uint16_t*>(
                                p.bias)[b * p.bias_batch_stride + hb * p.bias_head_stride + key]) * kLog2e
                          : 0.f;
          }
        } else {
          if (!(group_inv && bias2_loaded)) {
          bias2_loaded = true;
          {
            const int hm = hm_of(h), hb = hb_of(h);
            const uint16_t* bcol = p.bias ? reinterpret_cast<const uint16_t*>(p.bias) + b * p.bias_batch_stride +
                                                hb * p.bias_head_stride + key
                                          : nullptr;
            const bool mbits = p.mask && p.mask_bits;
            const uint8_t* mcol = (p.mask && !mbits) ? p.mask + b * p.mask_batch_stride + hm * p.mask_head_stride + key
                                                     : nullptr;
            const int wkey = -lane;  // the warp's first key, relative to this lane's
            // Bit-packed mask: the warp's 32 x 32 block is one word per query row. Lane j fetches row j's word and a
            // five-step exchange transposes the bit matrix across the lanes: lane k ends up with column k (its key).
            uint32_t colbits = 0xFFFFFFFFu;
            if (mbits) {
              const uint32_t* mw32 = reinterpret_cast<const uint32_t*>(p.mask) + b * p.mask_batch_stride +
                                     hm * p.mask_head_stride + ((n * kBN + (warp & 3) * 32) >> 5);
              if (g == 0 && m + 1 < M64)
                prefetch_l2(mw32 + static_cast<int64_t>(min((m + 1) * kBM + half * 32 + lane, Sq - 1)) * p.mask_row_stride);
              uint32_t a = __ldg(mw32 + static_cast<int64_t>(min(q0 + lane, Sq - 1)) * p.mask_row_stride);
              uint32_t msk = 0x0000FFFFu;
#pragma unroll
              for (int j = 16; j > 0; j >>= 1) {
                const uint32_t other = __shfl_xor_sync(0xffffffffu, a, j);
                // blocks of j x j bits: the upper-right one (rows without bit j, columns with it) changes places
                // with the lower-left one
                if ((lane & j) == 0) a ^= (((a >> j) ^ other) & msk) << j;
                else a ^= (a ^ (other >> j)) & msk;
                msk ^= msk << (j >> 1);
              }
              colbits = a;
            }
            if (g == 0 && m + 1 < M64) {
              // next query tile's bias / mask sectors of this warp's 32 keys: lane j asks L2 for row j
              const int64_t qn = min((m + 1) * kBM + half * 32 + lane, Sq - 1);
              if (bcol) {
                prefetch_l2(bcol + wkey + qn * p.bias_row_stride);
                prefetch_l2(bcol + wkey + qn * p.bias_row_stride + 16);
              }
              if (mcol) prefetch_l2(mcol + wkey + qn * p.mask_row_stride);
            }
            // The thread wants one column (its key) of 32 query rows, the tensors are contiguous along keys: the
            // warp fetches its 32 x 32 block with 16-byte loads along keys (6 per lane) and turns it through its
            // 1 KB of shared memory -- 16 bias rows, 16 bias rows, 32 mask rows -- instead of 64 scalar loads per
            // thread.
            uint4 vb[4], vm[2];
#pragma unroll
            for (int t = 0; t < 4; ++t) {
              const int qq = min(q0 + (t >> 1) * 16 + (t & 1) * 8 + (lane >> 2), Sq - 1);
              vb[t] = bcol ? ld_nc_v4(bcol + wkey + static_cast<int64_t>(qq) * p.bias_row_stride + (lane & 3) * 8)
                           : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int t = 0; t < 2; ++t) {
              const int qq = min(q0 + t * 16 + (lane >> 1), Sq - 1);
              vm[t] = mcol ? ld_nc_v4(mcol + wkey + static_cast<int64_t>(qq) * p.mask_row_stride + (lane & 1) * 16)
                           : make_uint4(0x01010101u, 0x01010101u, 0x01010101u, 0x01010101u);
            }
            uint4* tr4 = reinterpret_cast<uint4*>(s_tr);
            const uint16_t* tr16 = reinterpret_cast<const uint16_t*>(s_tr);
            float braw[32];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
              tr4[lane] = vb[2 * r];
              tr4[lane + 32] = vb[2 * r + 1];
              __syncwarp();
#pragma unroll
              for (int j = 0; j < 16; ++j) braw[r * 16 + j] = raw16_to_float<kBf16>(tr16[j * 32 + lane]) * kLog2e;
              __syncwarp();
            }
            if (mbits) {
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                const bool k0 = key_ok && ((colbits >> (2 * j)) & 1u);
                const bool k1 = key_ok && ((colbits >> (2 * j + 1)) & 1u);
                bias2[j] = make_float2(k0 ? braw[2 * j] : -CUDART_INF_F, k1 ? braw[2 * j + 1] : -CUDART_INF_F);
              }
            } else {
              tr4[lane] = vm[0];
              tr4[lane + 32] = vm[1];
              __syncwarp();
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                const bool k0 = key_ok && s_tr[(2 * j) * 32 + lane] != 0;
                const bool k1 = key_ok && s_tr[(2 * j + 1) * 32 + lane] != 0;
                bias2[j] = make_float2(k0 ? braw[2 * j] : -CUDART_INF_F, k1 ? braw[2 * j + 1] : -CUDART_INF_F);
              }
              __syncwarp();
            }
          }
          if (causal && static_cast<int64_t>(ckey_wmax) > static_cast<int64_t>(q0) + coff) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              if (ckey - coff > q0 + 2 * j) bias2[j].x = -CUDART_INF_F;
              if (ckey - coff > q0 + 2 * j + 1) bias2[j].y = -CUDART_INF_F;
            }
          }
          }
        }

        // ---- P^T and dS^T in one pass: both accumulators are loaded together ----
        // Barriers that alternate between the teams come in pairs indexed by step parity, so that a team only ever
        // waits on consecutive phases of a barrier. dP of step i is committed after S of step i was issued, so
        // dp_full covers both accumulators. The dS^T buffer (i & 1) was last read by the dQ product of step i-2,
        // issued before dP of step i: the tcgen05.commit behind dP covers every earlier MMA of the issuing thread, so
        // dp_full(i) also says that buffer is free. The LSE / D values of the stage were bulk-copied under the
        // stage barrier, which the MMA warp observed before it issued S and dP of this step; the per-query kernel
        // waits on that barrier itself as well.
        if (!kTeams) {
          ok = __all_sync(0xffffffffu, FDMA_PROF_WAIT(0, mbar_wait(bar_qdo_full + (i % kQStages),
                                                                     (i / kQStages) & 1, ctl, kWaitQdoFull)));
          if (!ok) break;
        }
        ok = __all_sync(0xffffffffu, FDMA_PROF_WAIT(2, mbar_wait(bar_dp_full + (i & 1), (i >> 1) & 1, ctl, kWaitDpFull)));
        if (!ok) break;
        tc_fence_after_sync();
        float step_sum = 0.f;
#pragma unroll 1
        for (int sub = 0; sub < (kTeams ? 2 : 1); ++sub) {
          const int qh = kTeams ? sub : half;  // which 32 of the step's 64 queries
          const int q0s = m * kBM + qh * 32;
          // LSE*log2e and D of the step's 64 queries arrive in shared memory with the Q/dO stage
          const float* lrow = s_ld + (i % kQStages) * (2 * kBM) + qh * 32;
          const float* drow = lrow + kBM;
          const bool diag = causal && static_cast<int64_t>(ckey_wmax) > static_cast<int64_t>(q0s) + coff;  // warp-uniform
          const bool per_elem = !kBcast || diag;
          if (kBcast && diag) {
#pragma unroll
            for (int j = 0; j < 16; ++j)
              bias2[j] = make_float2(ckey - coff > q0s + 2 * j ? -CUDART_INF_F : bv,
                                     ckey - coff > q0s + 2 * j + 1 ? -CUDART_INF_F : bv);
          }
          uint32_t dsk[16];
          uint32_t rs[32], rp[32];
          tmem_ld_x32(tmem_base + lane_addr + kColSt + (i & 1) * kBM + qh * 32, rs);
          tmem_ld_x32(tmem_base + lane_addr + kColDp + qh * 32, rp);
          tmem_wait_ld();
          if (!kTeams || sub == 1) {
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_dp_free);  // the dPt block may be overwritten from here on
          }
          // packed fp32x2 arithmetic: two queries per instruction
          float2 pp[16], dd[16];
          float2 part[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
          const float2 sc2 = make_float2(p.scale_log2, p.scale_log2);
          const float2 bv2 = make_float2(bv, bv);
          const float2 neg1 = make_float2(-1.f, -1.f);
#pragma unroll
          for (int j4 = 0; j4 < 8; ++j4) {
            const float4 l4 = reinterpret_cast<const float4*>(lrow)[j4];
            const float4 d4 = reinterpret_cast<const float4*>(drow)[j4];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const int j = j4 * 2 + e;  // pair index
              const float2 lv = e == 0 ? make_float2(l4.x, l4.y) : make_float2(l4.z, l4.w);
              const float2 dv = e == 0 ? make_float2(d4.x, d4.y) : make_float2(d4.z, d4.w);
              const float2 addend = __ffma2_rn(lv, neg1, per_elem ? bias2[j] : bv2);       // bias - LSE
              const float2 x = __ffma2_rn(make_float2(__uint_as_float(rs[2 * j]), __uint_as_float(rs[2 * j + 1])), sc2,
                                          addend);
              const float2 pj = make_float2(fast_exp2(x.x), fast_exp2(x.y));
              const float2 dpd = __ffma2_rn(dv, neg1, make_float2(__uint_as_float(rp[2 * j]), __uint_as_float(rp[2 * j + 1])));
              const float2 ds = __fmul2_rn(pj, dpd);
              pp[j] = pj;
              dd[j] = ds;
              part[e] = __fadd2_rn(part[e], ds);
            }
          }
          float pv[32];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            pv[2 * j] = dd[j].x;
            pv[2 * j + 1] = dd[j].y;
          }
          step_sum += (part[0].x + part[0].y) + (part[1].x + part[1].y);
          uint32_t pk[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            pk[j] = pack_16x2<kBf16>(pp[j].x, pp[j].y);
            dsk[j] = pack_16x2<kBf16>(pv[2 * j], pv[2 * j + 1]);
          }
          // back into the 32 columns just read: P^T pairs in the first 16, dS^T pairs in the last 16
          tmem_st_x16(tmem_base + lane_addr + kColSt + (i & 1) * kBM + qh * 32, pk);
          tmem_st_x16(tmem_base + lane_addr + kColSt + (i & 1) * kBM + qh * 32 + 16, dsk);
          if (mode == kDbDirect) {  // only reached by the per-query kernel (one pass: q0s == q0)
            if (direct_group) {
#pragma unroll
              for (int j = 0; j < 32; ++j) dacc[j] += pv[j];
            } else {
              store_dbias(dbias16 + b * p.dbias_batch_stride + h * p.dbias_head_stride + key, q0s, pv);
            }
          } else if (mode == kDbAtomic && key_ok && p.dbias_rows != 1) {
            const int b2 = p.dbias_b == 1 ? 0 : b;
            const int h2 = h / (p.h / p.dbias_h);
            float* base = p.dbias_acc + (static_cast<int64_t>(b2) * p.dbias_h + h2) * p.dbias_rows * p.dbias_keys + key;
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (q0s + j < Sq && pv[j] != 0.f) atomicAdd(base + static_cast<int64_t>(q0s + j) * p.dbias_keys, pv[j]);
          }
          // ---- dS^T tile to shared memory for the dQ MMA: row = key, 64 queries x 2 B = 128 B, 128-byte swizzle ----
          {
            unsigned char* rowp = s_ds + (i & 1) * L::kDsBytes + krow * 128;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              const int chunk = (qh * 4 + c) ^ (krow & 7);
              *reinterpret_cast<uint4*>(rowp + chunk * 16) = make_uint4(dsk[c * 4], dsk[c * 4 + 1], dsk[c * 4 + 2], dsk[c * 4 + 3]);
            }
          }
        }
        if (mode == kDbColsum) {
          colsum += step_sum;
        } else if (mode == kDbAtomic && key_ok && p.dbias_rows == 1) {
          const int b2 = p.dbias_b == 1 ? 0 : b;
          const int h2 = h / (p.h / p.dbias_h);
          atomicAdd(p.dbias_acc + (static_cast<int64_t>(b2) * p.dbias_h + h2) * p.dbias_keys + key, step_sum);
        }
        tmem_wait_st();
        fence_proxy_async_smem();
        tc_fence_before_sync();
        // One arrival per warp: single-thread arrivals of a whole warpgroup on one barrier word serialise in the
        // shared-memory pipe.
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_pds + (i & 1));
        ++i;
      }
      if (direct_group && ok) {  // one store per (query, key) after the whole head group
        store_dbias(dbias16 + b * p.dbias_batch_stride + hk * p.dbias_head_stride + key, q0,
                    group_touched ? dacc : nullptr);
#pragma unroll
        for (int j = 0; j < 32; ++j) dacc[j] = 0.f;
      }
    }
    FDMA_PROF_END(16, tid == 128);
    // ---------------- epilogue: dV (half 0) and dK (half 1), column-sum dBias ----------------
    if (mode == kDbColsum) {
      if (half == 1) s_red[krow] = colsum;
      named_bar_sync(1, 256);
      if (half == 0 && key < p.dbias_keys) {
        // dbias_h == h_k: this CTA saw every query head of the group. dbias_h == h with a group of one: same.
        const float tot = colsum + s_red[krow];
        if (p.nsplit > 1)
          p.dbias_part[((static_cast<int64_t>(split) * p.b + b) * p.h_k + hk) * (NT * kBN) + key] = key_ok ? tot : 0.f;
        else
          dbias16[b * p.dbias_batch_stride + hk * p.dbias_head_stride + key] = float_to_raw16<kBf16>(key_ok ? tot : 0.f);
      }
    }
    if (ok && n_steps > 0) ok = __all_sync(0xffffffffu, mbar_wait(bar_final, 0, ctl, kWaitFinal));
    tc_fence_after_sync();
    if (ok) {
      const uint32_t col = half == 0 ? kColDv : kColDk;
      const float mul = half == 0 ? 1.f : p.scale;
      uint16_t* dst = half == 0
                          ? reinterpret_cast<uint16_t*>(p.dv) + b * p.dv_batch_stride + hk * p.dv_head_stride +
                                static_cast<int64_t>(min(key, Sk - 1)) * p.dv_row_stride
                          : reinterpret_cast<uint16_t*>(p.dk) + b * p.dk_batch_stride + hk * p.dk_head_stride +
                                static_cast<int64_t>(min(key, Sk - 1)) * p.dk_row_stride;
#pragma unroll
      for (int c = 0; c < kD / 32; ++c) {
        uint32_t r[32];
        if (n_steps > 0) {
          tmem_ld_x32(tmem_base + lane_addr + col + c * 32, r);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = 0u;
        }
        if (p.nsplit > 1) {
          // fp32 partial: part[dv|dk][split][b][hk][key][d]
          float* part = p.dkv_part + ((((static_cast<int64_t>(half) * p.nsplit + split) * p.b + b) * p.h_k + hk) *
                                          (NT * kBN) + key) * kD + c * 32;
#pragma unroll
          for (int v4 = 0; v4 < 8; ++v4)
            *reinterpret_cast<float4*>(part + v4 * 4) =
                make_float4(__uint_as_float(r[v4 * 4 + 0]) * mul, __uint_as_float(r[v4 * 4 + 1]) * mul,
                            __uint_as_float(r[v4 * 4 + 2]) * mul, __uint_as_float(r[v4 * 4 + 3]) * mul);
        } else if (key_ok) {
#pragma unroll
          for (int v4 = 0; v4 < 4; ++v4) {
            uint4 o;
            o.x = pack_16x2<kBf16>(__uint_as_float(r[v4 * 8 + 0]) * mul, __uint_as_float(r[v4 * 8 + 1]) * mul);
            o.y = pack_16x2<kBf16>(__uint_as_float(r[v4 * 8 + 2]) * mul, __uint_as_float(r[v4 * 8 + 3]) * mul);
            o.z = pack_16x2<kBf16>(__uint_as_float(r[v4 * 8 + 4]) * mul, __uint_as_float(r[v4 * 8 + 5]) * mul);
            o.w = pack_16x2<kBf16>(__uint_as_float(r[v4 * 8 + 6]) * mul, __uint_as_float(r[v4 * 8 + 7]) * mul);
            *reinterpret_cast<uint4*>(dst + c * 32 + v4 * 8) = o;
          }
        }
      }
    }
  } else {
    if constexpr (kDet) asm volatile("setmaxnreg.dec.sync.aligned.u32 104;");
    else asm volatile("setmaxnreg.dec.sync.aligned.u32 88;");
    // ---------------- dQ writer: thread = head-dim index (row of dQ^T) ----------------
    // dQ^T (128 d x 64 q, fp32) leaves TMEM in two halves of 32 queries: transposed into a [32 q][128 d] fp32
    // staging tile in shared memory, then ONE bulk reduce-add (cp.reduce.async.bulk ... add.f32) per half into
    // the fp32 dQ buffer, whose (B,H,Sq,128) layout makes the 32 rows contiguous.
    const int dl = (warp & 3) * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
    float* s_dq = reinterpret_cast<float*>(smem + L::kDqOff);
    int i = 0;
    bool ok = true;
    FDMA_PROF_BEGIN();
    for (int m = m_start; m < M64 && ok; ++m) {
      for (int g = 0; g < G && ok; ++g) {
        if (!s_act[(act_g > 1 ? g : 0) * MT + (m >> 1)]) continue;
        const int h = hk * G + g;
        ok = __all_sync(0xffffffffu, FDMA_PROF_WAIT(0, mbar_wait(bar_dq_full, i & 1, ctl, kWaitDqFull)));
        if (!ok) break;
        tc_fence_after_sync();
        uint32_t r0[32], r1[32];
        tmem_ld_x32(tmem_base + lane_addr + kColDq, r0);
        tmem_ld_x32(tmem_base + lane_addr + kColDq + 32, r1);
        tmem_wait_ld();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_dq_empty);  // dQ^T columns may be overwritten by the next step from here on
        float* gdst = p.dq_acc + ((static_cast<int64_t>(b) * p.h + h) * Sq + m * kBM) * kD;
        if constexpr (kDet) {
          // 64-bit fixed point: integer sums are the same in any order. 16 queries fill the staging tile.
          long long* s_dq64 = reinterpret_cast<long long*>(s_dq);
          long long* gdst64 = reinterpret_cast<long long*>(p.dq_acc) +
                              ((static_cast<int64_t>(b) * p.h + h) * Sq + m * kBM) * kD;
          constexpr float kFix = static_cast<float>(1ll << kDetFracBits);
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            if (tid == 384) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
            named_bar_sync(2, 128);
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const uint32_t raw = c < 2 ? r0[(c & 1) * 16 + j] : r1[(c & 1) * 16 + j];
              s_dq64[j * kD + dl] = __float2ll_rn(__uint_as_float(raw) * kFix);
            }
            fence_proxy_async_smem();
            named_bar_sync(3, 128);
            if (tid == 384) {
              const int rows = min(16, Sq - (m * kBM + c * 16));
              if (rows > 0) {
                asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.u64 [%0], [%1], %2;"
                             :
                             : "l"(reinterpret_cast<uint64_t>(gdst64 + c * 16 * kD)), "r"(smem_u32(s_dq)),
                               "r"(static_cast<uint32_t>(rows * kD * 8))
                             : "memory");
              }
              asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
          }
          ++i;
          continue;
        }
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          if (tid == 384) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");  // staging tile free again
          named_bar_sync(2, 128);
#pragma unroll
          for (int j = 0; j < 32; ++j) s_dq[j * kD + dl] = __uint_as_float(c == 0 ? r0[j] : r1[j]);
          fence_proxy_async_smem();
          named_bar_sync(3, 128);
          if (tid == 384) {
            const int rows = min(32, Sq - (m * kBM + c * 32));
            if (rows > 0) {
              asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;"
                           :
                           : "l"(reinterpret_cast<uint64_t>(gdst + c * 32 * kD)), "r"(smem_u32(s_dq)),
                             "r"(static_cast<uint32_t>(rows * kD * 4))
                           : "memory");
            }
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          }
        }
        ++i;
      }
    }
    if (tid == 384) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    FDMA_PROF_END(24, tid == 384);
  }

  // ---------------- tear-down ----------------
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

// Sum of the query-range partials of dK or dV: part [nsplit][B][h_k][keys_r][128] fp32 -> 16-bit (B, Sk, h_k, 128).
template <bool kBf16>
__global__ void __launch_bounds__(256) bwd_reduce_dkv_kernel(const float* __restrict__ part, void* __restrict__ dst,
                                                              int nsplit, int B, int Hk, int Sk, int keys_r,
                                                              int64_t sb, int64_t sr, int64_t sh) {
  const int64_t n_vec = static_cast<int64_t>(B) * Hk * Sk * (kD / 8);
  const int64_t split_stride = static_cast<int64_t>(B) * Hk * keys_r * kD;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n_vec;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(i % (kD / 8));
    const int key = static_cast<int>((i / (kD / 8)) % Sk);
    const int hk = static_cast<int>((i / (static_cast<int64_t>(kD / 8) * Sk)) % Hk);
    const int b = static_cast<int>(i / (static_cast<int64_t>(kD / 8) * Sk * Hk));
    const float* src = part + ((static_cast<int64_t>(b) * Hk + hk) * keys_r + key) * kD + c * 8;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < nsplit; ++s) {
      const float4 a = *reinterpret_cast<const float4*>(src + s * split_stride);
      const float4 d = *reinterpret_cast<const float4*>(src + s * split_stride + 4);
      acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
      acc[4] += d.x; acc[5] += d.y; acc[6] += d.z; acc[7] += d.w;
    }
    uint4 o;
    o.x = pack_16x2<kBf16>(acc[0], acc[1]);
    o.y = pack_16x2<kBf16>(acc[2], acc[3]);
    o.z = pack_16x2<kBf16>(acc[4], acc[5]);
    o.w = pack_16x2<kBf16>(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(dst) + b * sb + static_cast<int64_t>(key) * sr + hk * sh +
                              c * 8) = o;
  }
}

// Sum of the query-range partials of the column-sum dBias: part [nsplit][B][h_k][keys_r] fp32 -> 16-bit
// (B, h_k, 1, dbias_keys); keys beyond Sk are zero.
template <bool kBf16>
__global__ void __launch_bounds__(256) bwd_reduce_dbias_kernel(const float* __restrict__ part, void* __restrict__ dst,
                                                                int nsplit, int B, int Hk, int dbias_keys, int Sk,
                                                                int keys_r, int64_t sb, int64_t sh) {
  const int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (i >= static_cast<int64_t>(B) * Hk * dbias_keys) return;
  const int key = static_cast<int>(i % dbias_keys);
  const int hk = static_cast<int>((i / dbias_keys) % Hk);
  const int b = static_cast<int>(i / (static_cast<int64_t>(dbias_keys) * Hk));
  float acc = 0.f;
  if (key < Sk)
    for (int s = 0; s < nsplit; ++s) acc += part[((static_cast<int64_t>(s) * B + b) * Hk + hk) * keys_r + key];
  reinterpret_cast<uint16_t*>(dst)[b * sb + hk * sh + key] = float_to_raw16<kBf16>(acc);
}

struct BwdPlan {
  bool bcast;
  bool needs_act;
  int dbias_mode;
  int sq_r;
  int nsplit;
  size_t lse2_off, dsum_off, dq_off, act_off, dbias_off, part_off, dbpart_off, total;
};

// Query-range splits per key tile. A grid of (key tiles x kv heads x batch) CTAs that cannot fill the GPU twice
// (eight times when causal masking makes the CTAs unequal) is cut along the query dimension until about eight CTAs
// per SM exist, so that the causal imbalance between key tiles evens out; every split keeps at least 32 steps.
int pick_nsplit(const fdma_fwd_params& p) {
  const int64_t ctas = static_cast<int64_t>((p.seqlen_k + kBN - 1) / kBN) * p.h_k * p.b;
  const bool causal = p.is_causal != 0 && p.seqlen_q > 1;
  if (ctas >= (causal ? 8 : 2) * sm_count()) return 1;
  const int64_t steps = static_cast<int64_t>((p.seqlen_q + kBM - 1) / kBM) * (p.h / p.h_k);
  const int64_t want = (8 * sm_count() + ctas - 1) / ctas;
  const int64_t cap = std::max<int64_t>(1, steps / 32);
  return static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(std::min(want, cap), 64)));
}

BwdPlan plan(const fdma_bwd_params& bp) {
  const fdma_fwd_params& p = bp.f;
  BwdPlan pl;
  const bool mask_b = !p.mask || p.mask_row_stride == 0 || p.seqlen_q == 1;
  const bool bias_b = !p.bias || p.bias_row_stride == 0 || p.seqlen_q == 1;
  pl.bcast = mask_b && bias_b;
  pl.needs_act = p.mask != nullptr && !mask_b;
  pl.sq_r = static_cast<int>(round_up(p.seqlen_q, kBM));
  const int G = p.h / p.h_k;
  if (!bp.dbias) {
    pl.dbias_mode = kDbNone;
  } else if (bp.dbias_b == p.b && bp.dbias_rows == 1 && p.seqlen_q >= 1 &&
             (bp.dbias_h == p.h_k || (bp.dbias_h == p.h && G == 1))) {
    pl.dbias_mode = kDbColsum;
  } else if (bp.dbias_b == p.b && bp.dbias_rows == p.seqlen_q && (bp.dbias_h == p.h_k || bp.dbias_h == p.h)) {
    pl.dbias_mode = kDbDirect;
  } else {
    pl.dbias_mode = kDbAtomic;
  }
  // per-(query, key) dBias is written by the per-query kernel, whose softmax threads keep one query range per step
  if (pl.dbias_mode == kDbDirect) pl.bcast = false;
  size_t o = 0;
  const size_t rows = static_cast<size_t>(p.b) * p.h * pl.sq_r;
  pl.lse2_off = o; o += align256(rows * 4);
  pl.dsum_off = o; o += align256(rows * 4);
  pl.dq_off = o;   o += align256(static_cast<size_t>(p.b) * p.seqlen_q * p.h * kD * (bp.deterministic ? 8 : 4));
  pl.act_off = o;
  if (pl.needs_act)
    o += align256(static_cast<size_t>(p.b) * p.h_mask * ((p.seqlen_q + 127) / 128) * ((p.seqlen_k + 127) / 128));
  pl.dbias_off = o;
  if (pl.dbias_mode == kDbAtomic)
    o += align256(static_cast<size_t>(bp.dbias_b) * bp.dbias_h * bp.dbias_rows * bp.dbias_keys * 4);
  pl.nsplit = pick_nsplit(p);
  pl.part_off = pl.dbpart_off = o;
  if (pl.nsplit > 1) {
    const size_t keys_r = round_up(p.seqlen_k, kBN);
    o += align256(static_cast<size_t>(2) * pl.nsplit * p.b * p.h_k * keys_r * kD * 4);
    pl.dbpart_off = o;
    if (pl.dbias_mode == kDbColsum) o += align256(static_cast<size_t>(pl.nsplit) * p.b * p.h_k * keys_r * 4);
  }
  pl.total = o;
  return pl;
}

bool aligned16(const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15u) == 0; }

template <bool kBf16>
int launch(const fdma_bwd_params& bp, const BwdPlan& pl, cudaStream_t stream) {
  const fdma_fwd_params& p = bp.f;
  if (!p.workspace || p.workspace_bytes < pl.total) return FDMA_ERR_WORKSPACE;
  char* ws = static_cast<char*>(p.workspace);
  BwdKernelParams kp;
  auto encode = [&](CUtensorMap* tm, const void* base, int heads, int rows, int box_rows, int64_t sb, int64_t sr,
                    int64_t sh) {
    if (heads == 1) sh = p.d;
    if (rows == 1) sr = static_cast<int64_t>(heads) * p.d;
    if (p.b == 1) sb = static_cast<int64_t>(rows) * heads * p.d;
    const uint64_t dims[4] = {static_cast<uint64_t>(p.d), static_cast<uint64_t>(heads), static_cast<uint64_t>(rows),
                              static_cast<uint64_t>(p.b)};
    const uint64_t str[3] = {static_cast<uint64_t>(sh) * 2, static_cast<uint64_t>(sr) * 2,
                             static_cast<uint64_t>(sb) * 2};
    const uint32_t box[4] = {64, 1, static_cast<uint32_t>(box_rows), 1};
    return encode_tmap_4d(tm, base, 2, dims, str, box);
  };
  int st = encode(&kp.tm_q, p.q, p.h, p.seqlen_q, kBM, p.q_batch_stride, p.q_row_stride, p.q_head_stride);
  if (st) return st;
  st = encode(&kp.tm_do, bp.dout, p.h, p.seqlen_q, kBM, bp.do_batch_stride, bp.do_row_stride, bp.do_head_stride);
  if (st) return st;
  st = encode(&kp.tm_k, p.k, p.h_k, p.seqlen_k, kBN, p.k_batch_stride, p.k_row_stride, p.k_head_stride);
  if (st) return st;
  st = encode(&kp.tm_v, p.v, p.h_k, p.seqlen_k, kBN, p.v_batch_stride, p.v_row_stride, p.v_head_stride);
  if (st) return st;

  float* lse2 = reinterpret_cast<float*>(ws + pl.lse2_off);
  float* dsum = reinterpret_cast<float*>(ws + pl.dsum_off);
  float* dq_acc = reinterpret_cast<float*>(ws + pl.dq_off);
  const size_t dq_bytes = static_cast<size_t>(p.b) * p.seqlen_q * p.h * kD * (bp.deterministic ? 8 : 4);
  cudaError_t e = cudaMemsetAsync(dq_acc, 0, dq_bytes, stream);
  if (e != cudaSuccess) return static_cast<int>(e);
  {
    const int64_t warps = static_cast<int64_t>(p.b) * p.h * (pl.sq_r / 8);
    const int64_t blocks = (warps * 32 + 255) / 256;
    bwd_prep_kernel<kBf16><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
        p.out, bp.dout, p.lse, lse2, dsum, p.b, p.h, p.seqlen_q, pl.sq_r, p.o_batch_stride, p.o_row_stride,
        p.o_head_stride, bp.do_batch_stride, bp.do_row_stride, bp.do_head_stride);
    e = cudaGetLastError();
    if (e != cudaSuccess) return static_cast<int>(e);
    st = export_softmax_d(bp, dsum, pl.sq_r, stream);
    if (st) return st;
  }
  kp.act = nullptr;
  kp.mask_bits = p.mask ? p.mask_bits : 0;
  if (pl.needs_act && p.tile_activity) {
    kp.act = p.tile_activity;
  } else if (pl.needs_act) {
    uint8_t* act = reinterpret_cast<uint8_t*>(ws + pl.act_off);
    st = launch_tile_activity(p, act, stream);
    if (st) return st;
    kp.act = act;
  }
  kp.dbias_acc = nullptr;
  if (pl.dbias_mode == kDbAtomic) {
    kp.dbias_acc = reinterpret_cast<float*>(ws + pl.dbias_off);
    e = cudaMemsetAsync(kp.dbias_acc, 0,
                        static_cast<size_t>(bp.dbias_b) * bp.dbias_h * bp.dbias_rows * bp.dbias_keys * 4, stream);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  kp.nsplit = pl.nsplit;
  kp.dkv_part = reinterpret_cast<float*>(ws + pl.part_off);
  kp.dbias_part = reinterpret_cast<float*>(ws + pl.dbpart_off);
  kp.mask = static_cast<const uint8_t*>(p.mask);
  kp.bias = p.bias;
  kp.lse2 = lse2;
  kp.dsum = dsum;
  kp.dq_acc = dq_acc;
  kp.dk = bp.dk;
  kp.dv = bp.dv;
  kp.dbias = bp.dbias;
  kp.status = kernel_status_ptr();
  if (!kp.status) return FDMA_ERR_DRIVER;
  kp.mask_batch_stride = p.mask_batch_stride; kp.mask_head_stride = p.mask_head_stride;
  kp.mask_row_stride = p.seqlen_q == 1 ? 0 : p.mask_row_stride;
  kp.bias_batch_stride = p.bias_batch_stride; kp.bias_head_stride = p.bias_head_stride;
  kp.bias_row_stride = p.seqlen_q == 1 ? 0 : p.bias_row_stride;
  kp.dk_batch_stride = bp.dk_batch_stride; kp.dk_row_stride = bp.dk_row_stride; kp.dk_head_stride = bp.dk_head_stride;
  kp.dv_batch_stride = bp.dv_batch_stride; kp.dv_row_stride = bp.dv_row_stride; kp.dv_head_stride = bp.dv_head_stride;
  kp.dbias_batch_stride = bp.dbias_batch_stride; kp.dbias_head_stride = bp.dbias_head_stride;
  kp.dbias_row_stride = bp.dbias_row_stride;
  kp.b = p.b; kp.seqlen_q = p.seqlen_q; kp.seqlen_k = p.seqlen_k; kp.sq_r = pl.sq_r; kp.h = p.h; kp.h_k = p.h_k;
  kp.h_mask = p.h_mask; kp.h_bias = p.h_bias;
  kp.dbias_b = bp.dbias_b; kp.dbias_h = bp.dbias_h; kp.dbias_rows = bp.dbias_rows; kp.dbias_keys = bp.dbias_keys;
  kp.dbias_mode = pl.dbias_mode;
  kp.is_causal = p.is_causal;
  kp.key_pos = p.key_pos;
  kp.pos_batch_stride = p.key_pos_batch_stride; kp.pos_head_stride = p.key_pos_head_stride;
  kp.h_pos = p.h_pos; kp.causal_shift = p.causal_shift;
  kp.scale_log2 = p.softmax_scale * kLog2e;
  kp.scale = p.softmax_scale;

  auto kern = bp.deterministic ? (pl.bcast ? bwd_kernel<kBf16, true, true> : bwd_kernel<kBf16, false, true>)
                               : (pl.bcast ? bwd_kernel<kBf16, true, false> : bwd_kernel<kBf16, false, false>);
  const int smem_bytes = SmemB::kAlloc;
  e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
  if (e != cudaSuccess) return static_cast<int>(e);
  dim3 grid(((p.seqlen_k + kBN - 1) / kBN) * pl.nsplit, p.h_k, p.b);
  cudaEvent_t ev0, ev1;
  take_timing_events(&ev0, &ev1);
  if (ev0) cudaEventRecord(ev0, stream);
  kern<<<grid, kThreads, smem_bytes, stream>>>(kp);
  if (ev1) cudaEventRecord(ev1, stream);
  e = cudaGetLastError();
  if (e != cudaSuccess) return static_cast<int>(e);

  if (pl.nsplit > 1) {
    const int keys_r = static_cast<int>(round_up(p.seqlen_k, kBN));
    const int64_t n_vec = static_cast<int64_t>(p.b) * p.h_k * p.seqlen_k * (kD / 8);
    const unsigned g = static_cast<unsigned>(std::min<int64_t>((n_vec + 255) / 256, sm_count() * 32));
    for (int which = 0; which < 2; ++which) {  // 0: dV, 1: dK
      const float* part = kp.dkv_part + static_cast<size_t>(which) * pl.nsplit * p.b * p.h_k * keys_r * kD;
      bwd_reduce_dkv_kernel<kBf16><<<g, 256, 0, stream>>>(
          part, which == 0 ? bp.dv : bp.dk, pl.nsplit, p.b, p.h_k, p.seqlen_k, keys_r,
          which == 0 ? bp.dv_batch_stride : bp.dk_batch_stride, which == 0 ? bp.dv_row_stride : bp.dk_row_stride,
          which == 0 ? bp.dv_head_stride : bp.dk_head_stride);
    }
    if (pl.dbias_mode == kDbColsum) {
      const int64_t nk = static_cast<int64_t>(p.b) * p.h_k * bp.dbias_keys;
      bwd_reduce_dbias_kernel<kBf16><<<static_cast<unsigned>((nk + 255) / 256), 256, 0, stream>>>(
          kp.dbias_part, bp.dbias, pl.nsplit, p.b, p.h_k, bp.dbias_keys, p.seqlen_k, keys_r, bp.dbias_batch_stride,
          bp.dbias_head_stride);
    }
    e = cudaGetLastError();
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  {
    const int64_t n_vec = static_cast<int64_t>(p.b) * p.seqlen_q * p.h * kD / 8;
    const unsigned g = static_cast<unsigned>(std::min<int64_t>((n_vec + 255) / 256, sm_count() * 32));
    if (bp.deterministic)
      bwd_convert_dq_fixed_kernel<kBf16><<<g, 256, 0, stream>>>(reinterpret_cast<const long long*>(dq_acc), bp.dq,
                                                              n_vec, p.seqlen_q, p.h, bp.dq_batch_stride,
                                                              bp.dq_row_stride, bp.dq_head_stride, p.softmax_scale,
                                                              dsum, pl.sq_r);
    else
      bwd_convert_dq_kernel<kBf16><<<g, 256, 0, stream>>>(dq_acc, bp.dq, n_vec, p.seqlen_q, p.h, bp.dq_batch_stride,
                                                          bp.dq_row_stride, bp.dq_head_stride, p.softmax_scale);
    e = cudaGetLastError();
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  if (pl.dbias_mode == kDbAtomic) {
    const int64_t ndb = static_cast<int64_t>(bp.dbias_b) * bp.dbias_h * bp.dbias_rows * bp.dbias_keys;
    const unsigned g = static_cast<unsigned>(std::min<int64_t>((ndb + 255) / 256, sm_count() * 32));
    bwd_convert_dbias_kernel<kBf16><<<g, 256, 0, stream>>>(kp.dbias_acc, bp.dbias, bp.dbias_b, bp.dbias_h,
                                                           bp.dbias_rows, bp.dbias_keys, bp.dbias_batch_stride,
                                                           bp.dbias_head_stride, bp.dbias_row_stride);
    e = cudaGetLastError();
  }
  return static_cast<int>(e);
}

}  // namespace

bool tc_bwd_supported(const fdma_bwd_params& bp) {
  const fdma_fwd_params& p = bp.f;
  if (p.d == 256) return tc_bwd256_supported(bp);
  if (!tc_fwd_supported(p)) return false;
  if (p.d != kD) return false;
  if (p.h_k > 65535) return false;
  if (p.key_pos && p.is_causal && p.h_pos == p.h && p.h != p.h_k) return false;  // positions per kv head at most
  const int G = p.h / p.h_k;
  const int act_g = (p.mask && p.h_mask == p.h && G > 1) ? G : 1;
  if (static_cast<int64_t>(act_g) * ((p.seqlen_q + 127) / 128) > kMaxAct) return false;
  const void* ptrs[4] = {bp.dout, bp.dq, bp.dk, bp.dv};
  for (const void* x : ptrs)
    if (!aligned16(x)) return false;
  const int64_t strides[12] = {bp.do_batch_stride, bp.do_row_stride, bp.do_head_stride, bp.dq_batch_stride,
                               bp.dq_row_stride,   bp.dq_head_stride, bp.dk_batch_stride, bp.dk_row_stride,
                               bp.dk_head_stride,  bp.dv_batch_stride, bp.dv_row_stride,  bp.dv_head_stride};
  for (int64_t s : strides)
    if (s % 8 != 0 || s < 0) return false;
  if (p.seqlen_q > 1 && bp.do_row_stride == 0) return false;
  if (bp.dbias && bp.dbias_keys > round_up(p.seqlen_k, kBN)) return false;
  return true;
}

size_t tc_bwd_workspace_bytes(const fdma_bwd_params& p) {
  return p.f.d == 256 ? tc_bwd256_workspace_bytes(p) : plan(p).total;
}

int tc_bwd(const fdma_bwd_params& p, cudaStream_t stream) {
  if (p.f.d == 256) return tc_bwd256(p, stream);
  const BwdPlan pl = plan(p);
  return p.f.dtype == FDMA_BF16 ? launch<true>(p, pl, stream) : launch<false>(p, pl, stream);
}

}  // namespace fdma

#ifdef FDMA_PROF
// Tracing build only: copies the backward kernel's 64 wait-cycle counters to `out` and clears them.
// Slots: [0,8) producer, [8,16) MMA issuer, [16,24) one softmax thread, [24,32) one dQ-writer thread; slot 7 of
// each group is the role's lifetime in cycles, the others are per-wait totals in the order of the source.
extern "C" int fdma_prof_read_bwd(unsigned long long* out) {
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return static_cast<int>(e);
  e = cudaMemcpyFromSymbol(out, fdma::g_prof, sizeof(unsigned long long) * 64);
  if (e != cudaSuccess) return static_cast<int>(e);
  static const unsigned long long zeros[64] = {};
  return static_cast<int>(cudaMemcpyToSymbol(fdma::g_prof, zeros, sizeof(zeros)));
}
#endif
