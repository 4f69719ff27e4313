// Dynamic-mask attention backward for head dim 256 on Blackwell tensor cores (tcgen05 + TMEM + TMA), for
// row-broadcast masks and biases (the shape create_mask produces from a (B, Hk, 1, Sk) bias).
//
// Same mathematics and the same transposed products as the head-dim-128 kernel next door (fdma_bwd_sm100.cu; the
// reference kernel is csrc/flash_sparse_attn/src/flash_bwd_kernel.h:79-1142):
//     St = K Q^T, dPt = V dO^T, P = exp2(St*scale*log2e + bias*log2e - LSE*log2e), dS = P o (dPt - D),
//     dV += P^T dO, dK += dS^T Q (x scale at the end), dQ^T = K^T dS^T (x scale in the convert pass),
//     dBias[key] = sum over queries and the head group of dS.
// What differs is the budget. At d = 256 the dK and dV accumulators of a 128-key tile need 256 TMEM columns EACH, all
// 512 there are, and K + V + one Q/dO step fill 192 KiB of shared memory. So a CTA walks its (query tile, head) steps
// TWICE, recomputing St / dPt / dS:
//     pass A: TMEM  St | dPt | dQ^T low | dQ^T high | dV (256)   -> dV, dQ, dBias
//     pass B: TMEM  St | dPt |     (free)           | dK (256)   -> dK
// and the Q/dO ring has ONE slot: a step is load -> St, dPt -> softmax -> dV (+ dQ) or dK -> next load. That is 14
// GEMM units per step pair instead of the 10 a single pass would need, and no overlap between the steps of one CTA;
// it still beats the CUDA-core kernel, the only other implementation at this head dim, by two orders of magnitude.
// Query-range splits (fp32 partial dK / dV / column sums + a reduction kernel) spread small grids over the GPU as in
// the d = 128 kernel. Every mbarrier wait is bounded.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math_constants.h>

#include <algorithm>

#include "fdma_internal.h"
#include "fdma_ptx.cuh"

namespace fdma {
namespace {

constexpr int kD = 256;
constexpr int kBN = 128;  // keys per CTA
constexpr int kBM = 64;   // query rows per step
constexpr int kThreads = 512;
constexpr float kLog2e = 1.4426950408889634f;

enum WaitCode256 {
  kW256Kv = 301, kW256StageEmpty = 302, kW256StageFull = 303, kW256SFull = 304, kW256Pds = 305, kW256DqFull = 306,
  kW256DqEmpty = 307, kW256DsEmpty = 308, kW256AccFree = 309, kW256Final = 310
};

struct Bwd256Params {
  CUtensorMap tm_q, tm_do, tm_k, tm_v;  // q/do: 64-row boxes, k/v: 128-row boxes, 64 elements wide
  const uint8_t* mask;
  const void* bias;
  const float* lse2;   // (B,H,Sq_r) LSE * log2(e); +inf for empty and padded rows
  const float* dsum;   // (B,H,Sq_r) D = rowsum(dO o O)
  float* dq_acc;       // (B,H,2,Sq,128) fp32: the two halves of d kept apart so that 16 query rows are contiguous
  void* dk;
  void* dv;
  void* dbias;
  float* dkv_part;     // nsplit > 1: fp32 partials [2: dV, dK][nsplit][B][h_k][NT*128][256]
  float* dbias_part;   // nsplit > 1: fp32 partials [nsplit][B][h_k][NT*128]
  int* status;
  int64_t mask_batch_stride, mask_head_stride, bias_batch_stride, bias_head_stride;
  int64_t dk_batch_stride, dk_row_stride, dk_head_stride;
  int64_t dv_batch_stride, dv_row_stride, dv_head_stride;
  int64_t dbias_batch_stride, dbias_head_stride;
  int b, seqlen_q, seqlen_k, sq_r, h, h_k, h_mask, h_bias;
  int dbias_keys, want_dbias, nsplit, is_causal;
  const int32_t* key_pos;
  int64_t pos_batch_stride, pos_head_stride;
  int h_pos, causal_shift;
  float scale_log2, scale;
};

struct Smem256 {
  static constexpr int kKOff = 0;                                   // 4 blocks of [128 keys][64 d]
  static constexpr int kVOff = kBN * kD * 2;                        // 64 KB
  static constexpr int kQOff = 2 * kBN * kD * 2;                    // 128 KB: Q step, 4 blocks of [64 q][64 d]
  static constexpr int kQBytes = kBM * kD * 2;                      // 32 KB
  static constexpr int kDoOff = kQOff + kQBytes;                    // dO step
  static constexpr int kDsOff = kDoOff + kQBytes;                   // 192 KB: dS^T tile [128 keys][64 q] 16-bit
  static constexpr int kDsBytes = kBN * kBM * 2;                    // 16 KB
  static constexpr int kDqOff = kDsOff + kDsBytes;                  // [16 q][128 d] fp32 staging tile of the dQ writer
  static constexpr int kDqRows = 16;
  static constexpr int kLdOff = kDqOff + kDqRows * 128 * 4;         // 64 x LSE*log2e, 64 x D (fp32)
  static constexpr int kLdBytes = 2 * kBM * 4;
  static constexpr int kRedOff = kLdOff + kLdBytes;
  static constexpr int kBarOff = kRedOff + kBN * 4;
  static constexpr int kNumBars = 12;
  static constexpr int kMiscOff = kBarOff + kNumBars * 8;
  static constexpr int kTotal = kMiscOff + 32;
  static constexpr int kAlloc = kTotal + 1024;  // slack to align the base to 1024 B
};
static_assert(Smem256::kAlloc <= 232448, "shared memory budget of one CTA");

template <bool kBf16>
__device__ __forceinline__ float raw16_to_f(uint16_t u) {
  if (kBf16) return __uint_as_float(static_cast<uint32_t>(u) << 16);
  return __half2float(__ushort_as_half(u));
}
template <bool kBf16>
__device__ __forceinline__ uint16_t f_to_raw16(float x) {
  return static_cast<uint16_t>(pack_16x2<kBf16>(x, 0.f) & 0xFFFFu);
}

// D = rowsum(dO o O), LSE in log2 units; rows [Sq, Sq_r) are padding (+inf / 0). One warp per (b, h, row): 32 lanes
// x 8 elements = 256.
template <bool kBf16>
__global__ void __launch_bounds__(256) bwd256_prep_kernel(const void* __restrict__ out, const void* __restrict__ dout,
                                                           const float* __restrict__ lse, float* __restrict__ lse2,
                                                           float* __restrict__ dsum, int B, int H, int Sq, int Sq_r,
                                                           int64_t ob, int64_t orow, int64_t oh, int64_t gb,
                                                           int64_t grow, int64_t gh) {
  const int lane = threadIdx.x & 31;
  const int64_t w = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5;
  const int64_t total = static_cast<int64_t>(B) * H * Sq_r;
  if (w >= total) return;
  const int q = static_cast<int>(w % Sq_r);
  const int h = static_cast<int>((w / Sq_r) % H);
  const int b = static_cast<int>(w / (static_cast<int64_t>(Sq_r) * H));
  if (q >= Sq) {
    if (lane == 0) {
      lse2[w] = CUDART_INF_F;
      dsum[w] = 0.f;
    }
    return;
  }
  const uint4 a = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(out) + b * ob +
                                                  static_cast<int64_t>(q) * orow + h * oh + lane * 8);
  const uint4 c = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(dout) + b * gb +
                                                  static_cast<int64_t>(q) * grow + h * gh + lane * 8);
  const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, cw[4] = {c.x, c.y, c.z, c.w};
  float acc = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    acc = fmaf(raw16_to_f<kBf16>(static_cast<uint16_t>(aw[j] & 0xFFFFu)),
               raw16_to_f<kBf16>(static_cast<uint16_t>(cw[j] & 0xFFFFu)), acc);
    acc = fmaf(raw16_to_f<kBf16>(static_cast<uint16_t>(aw[j] >> 16)), raw16_to_f<kBf16>(static_cast<uint16_t>(cw[j] >> 16)),
               acc);
  }
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
  if (lane == 0) {
    lse2[w] = lse[(static_cast<int64_t>(b) * H + h) * Sq + q] * kLog2e;
    dsum[w] = acc;
  }
}

// fp32 dQ accumulator (B,H,2,Sq,128) * scale -> dq (B,Sq,H,256 strided, 16-bit)
template <bool kBf16>
__global__ void bwd256_convert_dq_kernel(const float* __restrict__ acc, void* __restrict__ dq, int64_t n_vec, int Sq,
                                         int H, int64_t sb, int64_t sr, int64_t sh, float scale) {
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n_vec;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t e = i * 8;
    const int dd = static_cast<int>(e % 128);
    const int q = static_cast<int>((e / 128) % Sq);
    const int dh = static_cast<int>((e / (static_cast<int64_t>(128) * Sq)) % 2);
    const int h = static_cast<int>((e / (static_cast<int64_t>(256) * Sq)) % H);
    const int b = static_cast<int>(e / (static_cast<int64_t>(256) * Sq * H));
    const float4 x = *reinterpret_cast<const float4*>(acc + e);
    const float4 y = *reinterpret_cast<const float4*>(acc + e + 4);
    uint4 o;
    o.x = pack_16x2<kBf16>(x.x * scale, x.y * scale);
    o.y = pack_16x2<kBf16>(x.z * scale, x.w * scale);
    o.z = pack_16x2<kBf16>(y.x * scale, y.y * scale);
    o.w = pack_16x2<kBf16>(y.z * scale, y.w * scale);
    *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(dq) + b * sb + static_cast<int64_t>(q) * sr + h * sh +
                              dh * 128 + dd) = o;
  }
}

// Deterministic mode: the accumulator holds 64-bit fixed point (kDetFracBits256 fractional bits) instead of fp32.
constexpr int kDetFracBits256 = 40;
template <bool kBf16>
__global__ void bwd256_convert_dq_fixed_kernel(const long long* __restrict__ acc, void* __restrict__ dq, int64_t n_vec,
                                               int Sq, int H, int64_t sb, int64_t sr, int64_t sh, float scale,
                                               const float* __restrict__ dsum, int sq_r) {
  const float unit = scale * (1.0f / static_cast<float>(1ll << kDetFracBits256));
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n_vec;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t e = i * 8;
    const int dd = static_cast<int>(e % 128);
    const int q = static_cast<int>((e / 128) % Sq);
    const int dh = static_cast<int>((e / (static_cast<int64_t>(128) * Sq)) % 2);
    const int h = static_cast<int>((e / (static_cast<int64_t>(256) * Sq)) % H);
    const int b = static_cast<int>(e / (static_cast<int64_t>(256) * Sq * H));
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
    *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(dq) + b * sb + static_cast<int64_t>(q) * sr + h * sh +
                              dh * 128 + dd) = o;
  }
}

// Sum of the query-range partials of dK or dV: part [nsplit][B][h_k][keys_r][256] fp32 -> 16-bit (B, Sk, h_k, 256).
template <bool kBf16>
__global__ void __launch_bounds__(256) bwd256_reduce_dkv_kernel(const float* __restrict__ part, void* __restrict__ dst,
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
__global__ void __launch_bounds__(256) bwd256_reduce_dbias_kernel(const float* __restrict__ part, void* __restrict__ dst,
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
  reinterpret_cast<uint16_t*>(dst)[b * sb + hk * sh + key] = f_to_raw16<kBf16>(acc);
}

template <bool kBf16, bool kDet>
__global__ void __launch_bounds__(kThreads, 1) bwd256_kernel(const __grid_constant__ Bwd256Params p) {
  using L = Smem256;
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) &
                                                         ~static_cast<uintptr_t>(1023));
  unsigned char* s_k = smem + L::kKOff;
  unsigned char* s_v = smem + L::kVOff;
  unsigned char* s_q = smem + L::kQOff;
  unsigned char* s_do = smem + L::kDoOff;
  unsigned char* s_ds = smem + L::kDsOff;
  float* s_dq = reinterpret_cast<float*>(smem + L::kDqOff);
  float* s_ld = reinterpret_cast<float*>(smem + L::kLdOff);
  float* s_red = reinterpret_cast<float*>(smem + L::kRedOff);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* bar_kv = bars;
  uint64_t* bar_stage_full = bars + 1;
  uint64_t* bar_stage_empty = bars + 2;
  uint64_t* bar_s_full = bars + 3;
  uint64_t* bar_pds = bars + 4;
  uint64_t* bar_dq_full = bars + 5;
  uint64_t* bar_dq_empty = bars + 6;
  uint64_t* bar_ds_empty = bars + 7;
  uint64_t* bar_acc_free = bars + 8;
  uint64_t* bar_final = bars + 9;  // [2]: end of pass A, end of pass B
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(smem + L::kMiscOff);
  volatile int* s_abort = reinterpret_cast<volatile int*>(smem + L::kMiscOff + 4);
  int* s_active = reinterpret_cast<int*>(smem + L::kMiscOff + 8);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int hk = blockIdx.y, b = blockIdx.z;
  const int G = p.h / p.h_k;
  const int Sq = p.seqlen_q, Sk = p.seqlen_k;
  const int off = Sk - Sq;
  const int NT = (Sk + kBN - 1) / kBN;
  // blockIdx.x = (query-range split, key tile): the CTA covers the 64-row query tiles [m_start, M64) of its key tile;
  // with more than one split it leaves fp32 partials. The last ranges, never emptied by causal masking, run first.
  const int n = blockIdx.x % NT;
  const int split = p.nsplit - 1 - blockIdx.x / NT;
  const int M64_all = (Sq + kBM - 1) / kBM;
  const int m_chunk = (M64_all + p.nsplit - 1) / p.nsplit;
  const int m_lo = split * m_chunk;
  const int M64 = min(M64_all, m_lo + m_chunk);
  const bool causal = p.is_causal != 0;
  const int32_t* pos_row = nullptr;  // compacted keys: the causal test runs on their original positions
  if (causal && p.key_pos)
    pos_row = p.key_pos + b * p.pos_batch_stride + (p.h_pos == p.h_k ? hk : 0) * p.pos_head_stride;
  const int coff = pos_row ? p.causal_shift : off;
  int m_start = 0;
  if (pos_row) {
    const int64_t first = (static_cast<int64_t>(pos_row[n * kBN]) - coff) / kBM;
    m_start = static_cast<int>(max(static_cast<int64_t>(0), min(first, static_cast<int64_t>(M64))));
  } else if (causal) {
    m_start = max(0, (n * kBN - off) / kBM);
  }
  m_start = max(m_start, m_lo);
  const WaitCtl ctl{s_abort, p.status};
  const int hm = p.h_mask == p.h_k ? hk : 0;  // heads of mask / bias are 1 or h_k here (or h == h_k)
  const int hb = p.h_bias == p.h_k ? hk : 0;

  // ---------------- set-up ----------------
  if (tid == 0) {
    *s_abort = 0;
    mbar_init(bar_kv, 1);
    mbar_init(bar_stage_full, 1);
    mbar_init(bar_stage_empty, 1);
    mbar_init(bar_s_full, 1);
    mbar_init(bar_pds, 256);
    mbar_init(bar_dq_full, 1);
    mbar_init(bar_dq_empty, 128);
    mbar_init(bar_ds_empty, 1);
    mbar_init(bar_acc_free, 256);
    mbar_init(bar_final + 0, 1);
    mbar_init(bar_final + 1, 1);
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
  if (warp == 2) {  // does this key tile hold a kept key at all?
    bool any = true;
    if (p.mask) {
      const uint8_t* mrow = p.mask + b * p.mask_batch_stride + hm * p.mask_head_stride + n * kBN;
      any = false;
      for (int i = lane; i < kBN; i += 32) any = any || (n * kBN + i < Sk && mrow[i] != 0);
      any = __any_sync(0xffffffffu, any);
    }
    if (lane == 0) *s_active = any ? 1 : 0;
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *s_tmem;
  const int n_steps = (*s_active && M64 > m_start) ? (M64 - m_start) * G : 0;  // per pass
  constexpr uint32_t kColSt = 0, kColDp = 64, kColDq = 128, kColAcc = 256;

  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
    if (warp == 0) {
      // ---------------- TMA producer ----------------
      if (lane == 0 && n_steps > 0) {
        mbar_arrive_expect_tx(bar_kv, 2 * kBN * kD * 2);
#pragma unroll
        for (int kb = 0; kb < kD / 64; ++kb) {
          tma_load_4d(s_k + kb * (kBN * 128), &p.tm_k, bar_kv, kb * 64, hk, n * kBN, b);
          tma_load_4d(s_v + kb * (kBN * 128), &p.tm_v, bar_kv, kb * 64, hk, n * kBN, b);
        }
        int it = 0;
        bool ok = true;
        for (int pass = 0; pass < 2 && ok; ++pass) {
          for (int m = m_start; m < M64 && ok; ++m) {
            for (int g = 0; g < G; ++g) {
              ok = mbar_wait(bar_stage_empty, (it & 1) ^ 1, ctl, kW256StageEmpty);
              if (!ok) break;
              mbar_arrive_expect_tx(bar_stage_full, 2 * L::kQBytes + L::kLdBytes);
              const int h = hk * G + g;
              const int64_t row0 = (static_cast<int64_t>(b) * p.h + h) * p.sq_r + m * kBM;
              bulk_load_1d(s_ld, p.lse2 + row0, kBM * 4, bar_stage_full);
              bulk_load_1d(s_ld + kBM, p.dsum + row0, kBM * 4, bar_stage_full);
#pragma unroll
              for (int kb = 0; kb < kD / 64; ++kb) {
                tma_load_4d(s_q + kb * (kBM * 128), &p.tm_q, bar_stage_full, kb * 64, h, m * kBM, b);
                tma_load_4d(s_do + kb * (kBM * 128), &p.tm_do, bar_stage_full, kb * 64, h, m * kBM, b);
              }
              ++it;
            }
          }
        }
      }
    } else if (warp == 1) {
      // ---------------- MMA issuer (whole warp, uniform control flow; the issue wrappers elect one lane) -------
      if (n_steps > 0) {
        constexpr uint32_t idesc_s = umma_idesc(kBN, kBM, kBf16, false, false);  // St/dPt: 128 x 64, K-major
        constexpr uint32_t idesc_g = umma_idesc(kBN, kD, kBf16, false, true);    // dV/dK: A from TMEM, B MN-major
        constexpr uint32_t idesc_q = umma_idesc(128, kBM, kBf16, true, true);    // dQ^T half: both MN-major
        const uint32_t k_addr = smem_u32(s_k), v_addr = smem_u32(s_v), q_addr = smem_u32(s_q),
                       do_addr = smem_u32(s_do), ds_addr = smem_u32(s_ds);
        bool ok = __all_sync(0xffffffffu, mbar_wait(bar_kv, 0, ctl, kW256Kv));
        int it = 0;
        for (int pass = 0; pass < 2 && ok; ++pass) {
          for (int i = 0; i < n_steps && ok; ++i, ++it) {
            ok = __all_sync(0xffffffffu, mbar_wait(bar_stage_full, it & 1, ctl, kW256StageFull));
            if (!ok) break;
            tc_fence_after_sync();
#pragma unroll
            for (int kk = 0; kk < kD / 16; ++kk) {  // St = K Q^T
              const uint32_t ko = (kk >> 2) * (kBN * 128) + (kk & 3) * 32;
              const uint32_t qo = (kk >> 2) * (kBM * 128) + (kk & 3) * 32;
              umma_ss(tmem_base + kColSt, umma_desc_sw128(k_addr + ko, 16, 1024), umma_desc_sw128(q_addr + qo, 16, 1024),
                      idesc_s, kk > 0 ? 1u : 0u);
            }
#pragma unroll
            for (int kk = 0; kk < kD / 16; ++kk) {  // dPt = V dO^T
              const uint32_t ko = (kk >> 2) * (kBN * 128) + (kk & 3) * 32;
              const uint32_t qo = (kk >> 2) * (kBM * 128) + (kk & 3) * 32;
              umma_ss(tmem_base + kColDp, umma_desc_sw128(v_addr + ko, 16, 1024),
                      umma_desc_sw128(do_addr + qo, 16, 1024), idesc_s, kk > 0 ? 1u : 0u);
            }
            umma_commit(bar_s_full);
            ok = __all_sync(0xffffffffu, mbar_wait(bar_pds, it & 1, ctl, kW256Pds));
            if (!ok) break;
            tc_fence_after_sync();
            const uint32_t acc = i > 0 ? 1u : 0u;
            // A operands from TMEM: queries 0-31 sit in columns [0,16) of the St / dPt block, queries 32-63 in
            // columns [32,48) (each softmax warpgroup writes back into the columns it read).
            if (pass == 0) {
#pragma unroll
              for (int s = 0; s < 4; ++s) {  // dV += P^T dO
                const uint32_t a_col = (s < 2 ? s * 8 : 32 + (s - 2) * 8);
                umma_ts(tmem_base + kColAcc, tmem_base + kColSt + a_col,
                        umma_desc_sw128(do_addr + s * 2048, kBM * 128, 1024), idesc_g, (acc || s > 0) ? 1u : 0u);
              }
              if (i > 0) {
                ok = __all_sync(0xffffffffu, mbar_wait(bar_dq_empty, (i - 1) & 1, ctl, kW256DqEmpty));
                if (!ok) break;
                tc_fence_after_sync();
              }
#pragma unroll
              for (int dh = 0; dh < 2; ++dh) {  // dQ^T halves = K_half^T dS^T : 8 k-steps of 16 keys
#pragma unroll
                for (int s = 0; s < kBN / 16; ++s) {
                  umma_ss(tmem_base + kColDq + dh * kBM,
                          umma_desc_sw128(k_addr + dh * 2 * (kBN * 128) + s * 2048, kBN * 128, 1024),
                          umma_desc_sw128(ds_addr + s * 2048, 16, 1024), idesc_q, s > 0 ? 1u : 0u);
                }
              }
              umma_commit(bar_dq_full);
              umma_commit(bar_ds_empty);
            } else {
              if (i == 0) {  // the dV accumulator has been read out: its columns now take dK
                ok = __all_sync(0xffffffffu, mbar_wait(bar_acc_free, 0, ctl, kW256AccFree));
                if (!ok) break;
                tc_fence_after_sync();
              }
#pragma unroll
              for (int s = 0; s < 4; ++s) {  // dK += dS^T Q
                const uint32_t a_col = (s < 2 ? s * 8 : 32 + (s - 2) * 8);
                umma_ts(tmem_base + kColAcc, tmem_base + kColDp + a_col,
                        umma_desc_sw128(q_addr + s * 2048, kBM * 128, 1024), idesc_g, (acc || s > 0) ? 1u : 0u);
              }
            }
            umma_commit(bar_stage_empty);
          }
          if (ok) umma_commit(bar_final + pass);
        }
      }
    }
  } else if (warp < 12) {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 176;");
    // ---------------- softmax warpgroups: thread = key = TMEM lane; warpgroup `half` takes 32 of the 64 queries ----
    const int half = (warp - 4) >> 2;
    const int krow = (warp & 3) * 32 + lane;
    const int key = n * kBN + krow;
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const bool key_ok = key < Sk;
    // value compared with q + coff in the causal test: the key's position (clamped so that ckey - coff cannot
    // overflow; padding slots of a gathered key list hold INT_MAX and are masked out anyway)
    const int ckey = pos_row ? (key_ok ? min(pos_row[key], 0x3FFFFFFF) : 0x3FFFFFFF) : key;
    const int ckey_wmax = pos_row ? __shfl_sync(0xffffffffu, ckey, 31) : n * kBN + (warp & 3) * 32 + 31;
    float bv = -CUDART_INF_F;  // bias*log2e of this key, or -inf when the key is masked out
    {
      bool kp = key_ok;
      if (p.mask && kp) kp = p.mask[b * p.mask_batch_stride + hm * p.mask_head_stride + key] != 0;
      if (kp)
        bv = p.bias ? raw16_to_f<kBf16>(reinterpret_cast<const uint16_t*>(
                          p.bias)[b * p.bias_batch_stride + hb * p.bias_head_stride + key]) * kLog2e
                    : 0.f;
    }
    const int m_begin = n_steps > 0 ? m_start : M64;
    float colsum = 0.f;
    int it = 0;
    bool ok = true;
    for (int pass = 0; pass < 2; ++pass) {
      int i = 0;  // step inside the pass
      for (int m = m_begin; m < M64 && ok; ++m) {
        const int q0 = m * kBM + half * 32;
        for (int g = 0; g < G && ok; ++g, ++i, ++it) {
          const bool diag = causal && static_cast<int64_t>(ckey_wmax) > static_cast<int64_t>(q0) + coff;  // warp-uniform
          float2 bias2[16];
          if (diag) {
#pragma unroll
            for (int j = 0; j < 16; ++j)
              bias2[j] = make_float2(ckey - coff > q0 + 2 * j ? -CUDART_INF_F : bv,
                                     ckey - coff > q0 + 2 * j + 1 ? -CUDART_INF_F : bv);
          }
          const float* lrow = s_ld + half * 32;
          const float* drow = lrow + kBM;
          // the stage barrier makes the bulk-copied LSE / D values visible; s_full covers St and dPt
          ok = __all_sync(0xffffffffu, mbar_wait(bar_stage_full, it & 1, ctl, kW256StageFull));
          if (!ok) break;
          ok = __all_sync(0xffffffffu, mbar_wait(bar_s_full, it & 1, ctl, kW256SFull));
          if (!ok) break;
          tc_fence_after_sync();
          uint32_t dsk[16], pk[16];
          {
            uint32_t rs[32], rp[32];
            tmem_ld_x32(tmem_base + lane_addr + kColSt + half * 32, rs);
            tmem_ld_x32(tmem_base + lane_addr + kColDp + half * 32, rp);
            tmem_wait_ld();
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
                const int j = j4 * 2 + e;  // pair of queries
                const float2 lv = e == 0 ? make_float2(l4.x, l4.y) : make_float2(l4.z, l4.w);
                const float2 dv = e == 0 ? make_float2(d4.x, d4.y) : make_float2(d4.z, d4.w);
                const float2 addend = __ffma2_rn(lv, neg1, diag ? bias2[j] : bv2);  // bias - LSE
                const float2 x = __ffma2_rn(
                    make_float2(__uint_as_float(rs[2 * j]), __uint_as_float(rs[2 * j + 1])), sc2, addend);
                const float2 pj = make_float2(fast_exp2(x.x), fast_exp2(x.y));
                const float2 dpd =
                    __ffma2_rn(dv, neg1, make_float2(__uint_as_float(rp[2 * j]), __uint_as_float(rp[2 * j + 1])));
                const float2 ds = __fmul2_rn(pj, dpd);
                part[e] = __fadd2_rn(part[e], ds);
                pk[j] = pack_16x2<kBf16>(pj.x, pj.y);
                dsk[j] = pack_16x2<kBf16>(ds.x, ds.y);
              }
            }
            if (pass == 0) colsum += (part[0].x + part[0].y) + (part[1].x + part[1].y);
          }
          if (pass == 0) tmem_st_x16(tmem_base + lane_addr + kColSt + half * 32, pk);
          tmem_st_x16(tmem_base + lane_addr + kColDp + half * 32, dsk);
          if (pass == 0) {
            // dS^T tile to shared memory for the dQ products: row = key, 64 queries x 2 B = 128 B, 128-byte swizzle.
            // The previous step's dQ products must have finished reading the tile.
            ok = __all_sync(0xffffffffu, mbar_wait(bar_ds_empty, (i & 1) ^ 1, ctl, kW256DsEmpty));
            if (!ok) break;
            unsigned char* rowp = s_ds + krow * 128;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              const int chunk = (half * 4 + c) ^ (krow & 7);
              *reinterpret_cast<uint4*>(rowp + chunk * 16) =
                  make_uint4(dsk[c * 4], dsk[c * 4 + 1], dsk[c * 4 + 2], dsk[c * 4 + 3]);
            }
          }
          tmem_wait_st();
          fence_proxy_async_smem();
          tc_fence_before_sync();
          mbar_arrive(bar_pds);
        }
      }
      // ---------------- end of the pass: dV (pass A) or dK (pass B); column-sum dBias after pass A ----------------
      if (pass == 0 && p.want_dbias) {
        if (half == 1) s_red[krow] = colsum;
        named_bar_sync(1, 256);
        if (half == 0 && key < p.dbias_keys) {
          const float tot = key_ok ? colsum + s_red[krow] : 0.f;
          if (p.nsplit > 1)
            p.dbias_part[((static_cast<int64_t>(split) * p.b + b) * p.h_k + hk) * (NT * kBN) + key] = tot;
          else
            reinterpret_cast<uint16_t*>(p.dbias)[b * p.dbias_batch_stride + hk * p.dbias_head_stride + key] =
                f_to_raw16<kBf16>(tot);
        }
      }
      if (ok && n_steps > 0) ok = __all_sync(0xffffffffu, mbar_wait(bar_final + pass, 0, ctl, kW256Final));
      tc_fence_after_sync();
      if (ok) {
        const float mul = pass == 0 ? 1.f : p.scale;
        const int64_t krow_g = static_cast<int64_t>(min(key, Sk - 1));
        uint16_t* dst = pass == 0 ? reinterpret_cast<uint16_t*>(p.dv) + b * p.dv_batch_stride + hk * p.dv_head_stride +
                                        krow_g * p.dv_row_stride
                                  : reinterpret_cast<uint16_t*>(p.dk) + b * p.dk_batch_stride + hk * p.dk_head_stride +
                                        krow_g * p.dk_row_stride;
        // partial: part[dv|dk][split][b][hk][key][256]
        float* part = p.dkv_part + ((((static_cast<int64_t>(pass) * p.nsplit + split) * p.b + b) * p.h_k + hk) *
                                        (NT * kBN) + key) * kD;
#pragma unroll
        for (int c = 0; c < 4; ++c) {  // this warpgroup's 128 of the 256 columns
          const int col = half * 128 + c * 32;
          uint32_t r[32];
          if (n_steps > 0) {
            tmem_ld_x32(tmem_base + lane_addr + kColAcc + col, r);
            tmem_wait_ld();
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) r[j] = 0u;
          }
          if (p.nsplit > 1) {
#pragma unroll
            for (int v4 = 0; v4 < 8; ++v4)
              *reinterpret_cast<float4*>(part + col + v4 * 4) =
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
              *reinterpret_cast<uint4*>(dst + col + v4 * 8) = o;
            }
          }
        }
        if (pass == 0 && n_steps > 0) {  // the accumulator columns may now take dK
          tc_fence_before_sync();
          mbar_arrive(bar_acc_free);
        }
      }
    }
  } else {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 104;");
    // ---------------- dQ writer (pass A only): thread = head-dim index inside a half of d (row of dQ^T) ----------
    // Each half of dQ^T (128 d x 64 q, fp32) leaves TMEM in four pieces of 16 queries: transposed into a
    // [16 q][128 d] fp32 staging tile in shared memory, then ONE bulk reduce-add per piece into the fp32 dQ buffer,
    // whose (B,H,2,Sq,128) layout makes the 16 rows contiguous.
    const int dl = (warp & 3) * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const int m_begin = n_steps > 0 ? m_start : M64;
    int i = 0;
    bool ok = true;
    for (int m = m_begin; m < M64 && ok; ++m) {
      for (int g = 0; g < G && ok; ++g, ++i) {
        const int h = hk * G + g;
        ok = __all_sync(0xffffffffu, mbar_wait(bar_dq_full, i & 1, ctl, kW256DqFull));
        if (!ok) break;
        tc_fence_after_sync();
#pragma unroll
        for (int dh = 0; dh < 2; ++dh) {
          uint32_t r0[32], r1[32];
          tmem_ld_x32(tmem_base + lane_addr + kColDq + dh * kBM, r0);
          tmem_ld_x32(tmem_base + lane_addr + kColDq + dh * kBM + 32, r1);
          tmem_wait_ld();
          if (dh == 1) {  // both halves are in registers: the dQ^T columns may be overwritten by the next step
            tc_fence_before_sync();
            mbar_arrive(bar_dq_empty);
          }
          float* gdst = p.dq_acc + (((static_cast<int64_t>(b) * p.h + h) * 2 + dh) * Sq + m * kBM) * 128;
          if constexpr (kDet) {
            // 64-bit fixed point: integer sums are the same in any order. 8 queries fill the staging tile.
            long long* s_dq64 = reinterpret_cast<long long*>(s_dq);
            long long* gdst64 = reinterpret_cast<long long*>(p.dq_acc) +
                                (((static_cast<int64_t>(b) * p.h + h) * 2 + dh) * Sq + m * kBM) * 128;
            constexpr float kFix = static_cast<float>(1ll << kDetFracBits256);
#pragma unroll
            for (int c = 0; c < 8; ++c) {
              if (tid == 384) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
              named_bar_sync(2, 128);
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const uint32_t raw = c < 4 ? r0[(c & 3) * 8 + j] : r1[(c & 3) * 8 + j];
                s_dq64[j * 128 + dl] = __float2ll_rn(__uint_as_float(raw) * kFix);
              }
              fence_proxy_async_smem();
              named_bar_sync(3, 128);
              if (tid == 384) {
                const int rows = min(8, Sq - (m * kBM + c * 8));
                if (rows > 0) {
                  asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.u64 [%0], [%1], %2;"
                               :
                               : "l"(reinterpret_cast<uint64_t>(gdst64 + c * 8 * 128)), "r"(smem_u32(s_dq)),
                                 "r"(static_cast<uint32_t>(rows * 128 * 8))
                               : "memory");
                }
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
              }
            }
            continue;
          }
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            if (tid == 384) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");  // staging tile free again
            named_bar_sync(2, 128);
#pragma unroll
            for (int j = 0; j < 16; ++j)
              s_dq[j * 128 + dl] = __uint_as_float(c < 2 ? r0[(c & 1) * 16 + j] : r1[(c & 1) * 16 + j]);
            fence_proxy_async_smem();
            named_bar_sync(3, 128);
            if (tid == 384) {
              const int rows = min(16, Sq - (m * kBM + c * 16));
              if (rows > 0) {
                asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;"
                             :
                             : "l"(reinterpret_cast<uint64_t>(gdst + c * 16 * 128)), "r"(smem_u32(s_dq)),
                               "r"(static_cast<uint32_t>(rows * 128 * 4))
                             : "memory");
              }
              asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
          }
        }
      }
    }
    if (tid == 384) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  }

  // ---------------- tear-down ----------------
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

struct Plan256 {
  int sq_r, nsplit;
  bool want_dbias;
  size_t lse2_off, dsum_off, dq_off, part_off, dbpart_off, total;
};

// Query-range splits per key tile: as in the d = 128 kernel, a grid that cannot fill the GPU twice is cut along the
// query dimension until about eight CTAs per SM exist; every split keeps at least 32 steps.
int pick_nsplit256(const fdma_fwd_params& p) {
  const int64_t ctas = static_cast<int64_t>((p.seqlen_k + kBN - 1) / kBN) * p.h_k * p.b;
  if (ctas >= 2 * sm_count()) return 1;
  const int64_t steps = static_cast<int64_t>((p.seqlen_q + kBM - 1) / kBM) * (p.h / p.h_k);
  const int64_t want = (8 * sm_count() + ctas - 1) / ctas;
  const int64_t cap = std::max<int64_t>(1, steps / 32);
  return static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(std::min(want, cap), 64)));
}

Plan256 plan256(const fdma_bwd_params& bp) {
  const fdma_fwd_params& p = bp.f;
  Plan256 pl;
  pl.sq_r = static_cast<int>(round_up(p.seqlen_q, kBM));
  pl.nsplit = pick_nsplit256(p);
  pl.want_dbias = bp.dbias != nullptr;
  size_t o = 0;
  const size_t rows = static_cast<size_t>(p.b) * p.h * pl.sq_r;
  pl.lse2_off = o; o += align256(rows * 4);
  pl.dsum_off = o; o += align256(rows * 4);
  pl.dq_off = o;   o += align256(static_cast<size_t>(p.b) * p.seqlen_q * p.h * kD * (bp.deterministic ? 8 : 4));
  pl.part_off = pl.dbpart_off = o;
  if (pl.nsplit > 1) {
    const size_t keys_r = round_up(p.seqlen_k, kBN);
    o += align256(static_cast<size_t>(2) * pl.nsplit * p.b * p.h_k * keys_r * kD * 4);
    pl.dbpart_off = o;
    if (pl.want_dbias) o += align256(static_cast<size_t>(pl.nsplit) * p.b * p.h_k * keys_r * 4);
  }
  pl.total = o;
  return pl;
}

bool aligned16(const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15u) == 0; }

template <bool kBf16>
int launch256(const fdma_bwd_params& bp, const Plan256& pl, cudaStream_t stream) {
  const fdma_fwd_params& p = bp.f;
  if (!p.workspace || p.workspace_bytes < pl.total) return FDMA_ERR_WORKSPACE;
  char* ws = static_cast<char*>(p.workspace);
  Bwd256Params kp;
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
  cudaError_t e = cudaMemsetAsync(dq_acc, 0, static_cast<size_t>(p.b) * p.seqlen_q * p.h * kD * (bp.deterministic ? 8 : 4),
                                  stream);
  if (e != cudaSuccess) return static_cast<int>(e);
  {
    const int64_t warps = static_cast<int64_t>(p.b) * p.h * pl.sq_r;
    const int64_t blocks = (warps * 32 + 255) / 256;
    bwd256_prep_kernel<kBf16><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
        p.out, bp.dout, p.lse, lse2, dsum, p.b, p.h, p.seqlen_q, pl.sq_r, p.o_batch_stride, p.o_row_stride,
        p.o_head_stride, bp.do_batch_stride, bp.do_row_stride, bp.do_head_stride);
    e = cudaGetLastError();
    if (e != cudaSuccess) return static_cast<int>(e);
    st = export_softmax_d(bp, dsum, pl.sq_r, stream);
    if (st) return st;
  }
  kp.mask = static_cast<const uint8_t*>(p.mask);
  kp.bias = p.bias;
  kp.lse2 = lse2;
  kp.dsum = dsum;
  kp.dq_acc = dq_acc;
  kp.dk = bp.dk;
  kp.dv = bp.dv;
  kp.dbias = bp.dbias;
  kp.dkv_part = reinterpret_cast<float*>(ws + pl.part_off);
  kp.dbias_part = reinterpret_cast<float*>(ws + pl.dbpart_off);
  kp.status = kernel_status_ptr();
  if (!kp.status) return FDMA_ERR_DRIVER;
  kp.mask_batch_stride = p.mask_batch_stride; kp.mask_head_stride = p.mask_head_stride;
  kp.bias_batch_stride = p.bias_batch_stride; kp.bias_head_stride = p.bias_head_stride;
  kp.dk_batch_stride = bp.dk_batch_stride; kp.dk_row_stride = bp.dk_row_stride; kp.dk_head_stride = bp.dk_head_stride;
  kp.dv_batch_stride = bp.dv_batch_stride; kp.dv_row_stride = bp.dv_row_stride; kp.dv_head_stride = bp.dv_head_stride;
  kp.dbias_batch_stride = bp.dbias_batch_stride; kp.dbias_head_stride = bp.dbias_head_stride;
  kp.b = p.b; kp.seqlen_q = p.seqlen_q; kp.seqlen_k = p.seqlen_k; kp.sq_r = pl.sq_r; kp.h = p.h; kp.h_k = p.h_k;
  // head extents equal to h only occur here with h == h_k (see tc_bwd256_supported): fold them onto h_k
  kp.h_mask = p.h_mask == p.h ? p.h_k : p.h_mask;
  kp.h_bias = p.h_bias == p.h ? p.h_k : p.h_bias;
  kp.dbias_keys = bp.dbias ? bp.dbias_keys : 0;
  kp.want_dbias = pl.want_dbias ? 1 : 0;
  kp.nsplit = pl.nsplit;
  kp.is_causal = p.is_causal;
  kp.key_pos = p.key_pos;
  kp.pos_batch_stride = p.key_pos_batch_stride; kp.pos_head_stride = p.key_pos_head_stride;
  kp.h_pos = p.h_pos == p.h ? p.h_k : p.h_pos;
  kp.causal_shift = p.causal_shift;
  kp.scale_log2 = p.softmax_scale * kLog2e;
  kp.scale = p.softmax_scale;

  auto kern = bp.deterministic ? bwd256_kernel<kBf16, true> : bwd256_kernel<kBf16, false>;
  e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem256::kAlloc);
  if (e != cudaSuccess) return static_cast<int>(e);
  dim3 grid(((p.seqlen_k + kBN - 1) / kBN) * pl.nsplit, p.h_k, p.b);
  cudaEvent_t ev0, ev1;
  take_timing_events(&ev0, &ev1);
  if (ev0) cudaEventRecord(ev0, stream);
  kern<<<grid, kThreads, Smem256::kAlloc, stream>>>(kp);
  if (ev1) cudaEventRecord(ev1, stream);
  e = cudaGetLastError();
  if (e != cudaSuccess) return static_cast<int>(e);

  if (pl.nsplit > 1) {
    const int keys_r = static_cast<int>(round_up(p.seqlen_k, kBN));
    const int64_t n_vec = static_cast<int64_t>(p.b) * p.h_k * p.seqlen_k * (kD / 8);
    const unsigned g = static_cast<unsigned>(std::min<int64_t>((n_vec + 255) / 256, sm_count() * 32));
    for (int which = 0; which < 2; ++which) {  // 0: dV, 1: dK
      const float* part = kp.dkv_part + static_cast<size_t>(which) * pl.nsplit * p.b * p.h_k * keys_r * kD;
      bwd256_reduce_dkv_kernel<kBf16><<<g, 256, 0, stream>>>(
          part, which == 0 ? bp.dv : bp.dk, pl.nsplit, p.b, p.h_k, p.seqlen_k, keys_r,
          which == 0 ? bp.dv_batch_stride : bp.dk_batch_stride, which == 0 ? bp.dv_row_stride : bp.dk_row_stride,
          which == 0 ? bp.dv_head_stride : bp.dk_head_stride);
    }
    if (pl.want_dbias) {
      const int64_t nk = static_cast<int64_t>(p.b) * p.h_k * bp.dbias_keys;
      bwd256_reduce_dbias_kernel<kBf16><<<static_cast<unsigned>((nk + 255) / 256), 256, 0, stream>>>(
          kp.dbias_part, bp.dbias, pl.nsplit, p.b, p.h_k, bp.dbias_keys, p.seqlen_k, keys_r, bp.dbias_batch_stride,
          bp.dbias_head_stride);
    }
    e = cudaGetLastError();
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  const int64_t n_vec = static_cast<int64_t>(p.b) * p.seqlen_q * p.h * kD / 8;
  const unsigned g = static_cast<unsigned>(std::min<int64_t>((n_vec + 255) / 256, sm_count() * 32));
  if (bp.deterministic)
    bwd256_convert_dq_fixed_kernel<kBf16><<<g, 256, 0, stream>>>(reinterpret_cast<const long long*>(dq_acc), bp.dq, n_vec,
                                                               p.seqlen_q, p.h, bp.dq_batch_stride, bp.dq_row_stride,
                                                               bp.dq_head_stride, p.softmax_scale, dsum, pl.sq_r);
  else
    bwd256_convert_dq_kernel<kBf16><<<g, 256, 0, stream>>>(dq_acc, bp.dq, n_vec, p.seqlen_q, p.h, bp.dq_batch_stride,
                                                           bp.dq_row_stride, bp.dq_head_stride, p.softmax_scale);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace

// Head dim 256 on the tensor-core backward: row-broadcast mask and bias with one row per kv head at most, dBias (if
// asked for) of shape (B, h_k, 1, keys); everything else at this head dim stays on the CUDA-core kernels.
bool tc_bwd256_supported(const fdma_bwd_params& bp) {
  const fdma_fwd_params& p = bp.f;
  if (p.d != kD || !tc_fwd_supported(p)) return false;
  if (p.h_k > 65535 || p.b > 65535) return false;
  const int G = p.h / p.h_k;
  const bool mask_b = !p.mask || p.mask_row_stride == 0 || p.seqlen_q == 1;
  const bool bias_b = !p.bias || p.bias_row_stride == 0 || p.seqlen_q == 1;
  if (!mask_b || !bias_b) return false;
  if (G > 1 && ((p.mask && p.h_mask == p.h) || (p.bias && p.h_bias == p.h))) return false;
  if (p.key_pos && p.is_causal && p.h_pos == p.h && G > 1) return false;
  if (bp.dbias) {
    if (!p.bias) return false;
    const bool colsum = bp.dbias_b == p.b && bp.dbias_rows == 1 && (bp.dbias_h == p.h_k || (bp.dbias_h == p.h && G == 1));
    if (!colsum) return false;
  }
  const void* ptrs[4] = {bp.dout, bp.dq, bp.dk, bp.dv};
  for (const void* x : ptrs)
    if (!aligned16(x)) return false;
  const int64_t strides[12] = {bp.do_batch_stride, bp.do_row_stride, bp.do_head_stride, bp.dq_batch_stride,
                               bp.dq_row_stride,   bp.dq_head_stride, bp.dk_batch_stride, bp.dk_row_stride,
                               bp.dk_head_stride,  bp.dv_batch_stride, bp.dv_row_stride,  bp.dv_head_stride};
  for (int64_t s : strides)
    if (s % 8) return false;
  return true;
}

size_t tc_bwd256_workspace_bytes(const fdma_bwd_params& bp) { return plan256(bp).total; }

int tc_bwd256(const fdma_bwd_params& bp, cudaStream_t stream) {
  const Plan256 pl = plan256(bp);
  return bp.f.dtype == FDMA_BF16 ? launch256<true>(bp, pl, stream) : launch256<false>(bp, pl, stream);
}

}  // namespace fdma
