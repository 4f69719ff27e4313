// Single-query (decode) forward: HBM-bound, so the unit of skipping is the KEY ROW, not the 128-key tile.
//
// The reference runs decode through its split-KV kernel (csrc/flash_sparse_attn/src/flash_fwd_kernel.h:808-1587,
// merge :1618-1813) and, at 64- or 128-key tiles, streams every K/V row because a top-w mask leaves some kept key
// in nearly every tile. Here each warp scans the bool mask of its key range (1 byte per key), queues the kept keys,
// and reads only their K and V rows (one 2*d-byte row per warp-wide load, fully coalesced). The G query heads that
// share a kv head are processed together, so each kept row is read once per kv head. Every warp keeps an online
// softmax state (max, sum, d accumulators per head) and writes it as one partial; `decode_merge_kernel` combines
// the partials with the log-sum-exp rule. Scratch: partials (B, H, P, d + 2) fp32, P = splits x warps per CTA.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math_constants.h>

#include <algorithm>

#include "fdma_internal.h"

namespace fdma {
namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kMaxGroup = 8;   // query heads processed together per kv head
constexpr int kBatch = 4;      // kept rows in flight per warp (a K and a V row each)
constexpr int kQueue = 64;     // per-warp queue of kept key indices

template <bool kBf16>
__device__ __forceinline__ float raw_to_f(uint16_t u) {
  if (kBf16) return __uint_as_float(static_cast<uint32_t>(u) << 16);
  return __half2float(__ushort_as_half(u));
}
template <bool kBf16>
__device__ __forceinline__ uint16_t f_to_raw(float x) {
  if (kBf16) return __bfloat16_as_ushort(__float2bfloat16_rn(x));
  return __half_as_ushort(__float2half_rn(x));
}

struct DecodeParams {
  const void* q; const void* k; const void* v; const uint8_t* mask; const void* bias;
  float* partial;  // (B, H, P, D + 2): acc[D], max (log2 units), sum
  int64_t q_batch_stride, q_head_stride;
  int64_t k_batch_stride, k_row_stride, k_head_stride;
  int64_t v_batch_stride, v_row_stride, v_head_stride;
  int64_t mask_batch_stride, mask_head_stride, bias_batch_stride, bias_head_stride;
  int b, seqlen_k, h, h_k, h_mask, h_bias, group, nsplit;
  float scale_log2;
};

// EPL = head-dim elements per lane (D = 32 * EPL), G = query heads handled together.
template <int EPL, int G, bool kBf16>
__global__ void __launch_bounds__(kThreads) decode_kernel(const DecodeParams p) {
  constexpr int D = 32 * EPL;
  __shared__ int s_queue[kWarps][kQueue];
  __shared__ float s_qbias[kWarps][kQueue];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int split = blockIdx.x, b = blockIdx.z;
  const int h0 = blockIdx.y * G;                     // first query head of this CTA
  const int hk = h0 / p.group;
  const int hm = p.h_mask == p.h ? h0 : (p.h_mask == p.h_k ? hk : 0);
  const int hb = p.h_bias == p.h ? h0 : (p.h_bias == p.h_k ? hk : 0);
  const uint8_t* mrow = p.mask ? p.mask + b * p.mask_batch_stride + hm * p.mask_head_stride : nullptr;
  const uint16_t* brow = p.bias ? reinterpret_cast<const uint16_t*>(p.bias) + b * p.bias_batch_stride + hb * p.bias_head_stride
                                : nullptr;
  const uint16_t* kbase = reinterpret_cast<const uint16_t*>(p.k) + b * p.k_batch_stride + hk * p.k_head_stride + lane * EPL;
  const uint16_t* vbase = reinterpret_cast<const uint16_t*>(p.v) + b * p.v_batch_stride + hk * p.v_head_stride + lane * EPL;

  float qv[G][EPL];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const uint16_t* qp = reinterpret_cast<const uint16_t*>(p.q) + b * p.q_batch_stride + (h0 + g) * p.q_head_stride + lane * EPL;
#pragma unroll
    for (int e = 0; e < EPL; ++e) qv[g][e] = raw_to_f<kBf16>(qp[e]) * p.scale_log2;
  }
  float m[G], l[G], acc[G][EPL];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = -CUDART_INF_F;
    l[g] = 0.f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) acc[g][e] = 0.f;
  }

  auto load_row = [&](const uint16_t* base, int64_t row_stride, int key, float (&out)[EPL]) {
    const uint16_t* rp = base + static_cast<int64_t>(key) * row_stride;
    if (EPL == 8) {
      const uint4 r = *reinterpret_cast<const uint4*>(rp);
      const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        out[2 * i] = raw_to_f<kBf16>(static_cast<uint16_t>(w[i] & 0xFFFFu));
        out[2 * i + 1] = raw_to_f<kBf16>(static_cast<uint16_t>(w[i] >> 16));
      }
    } else if (EPL == 4) {
      const uint2 r = *reinterpret_cast<const uint2*>(rp);
      out[0] = raw_to_f<kBf16>(static_cast<uint16_t>(r.x & 0xFFFFu));
      out[1] = raw_to_f<kBf16>(static_cast<uint16_t>(r.x >> 16));
      out[2] = raw_to_f<kBf16>(static_cast<uint16_t>(r.y & 0xFFFFu));
      out[3] = raw_to_f<kBf16>(static_cast<uint16_t>(r.y >> 16));
    } else {
      const uint32_t r = *reinterpret_cast<const uint32_t*>(rp);
      out[0] = raw_to_f<kBf16>(static_cast<uint16_t>(r & 0xFFFFu));
      out[1] = raw_to_f<kBf16>(static_cast<uint16_t>(r >> 16));
    }
  };

  // kept rows [first, first + n) of the queue: scores, online softmax, value accumulation
  auto process = [&](int first, int n) {
    float kr[kBatch][EPL], vr[kBatch][EPL], sc[kBatch][G];
    int keys[kBatch];
#pragma unroll
    for (int t = 0; t < kBatch; ++t) {
      keys[t] = s_queue[warp][first + min(t, n - 1)];
      load_row(kbase, p.k_row_stride, keys[t], kr[t]);
      load_row(vbase, p.v_row_stride, keys[t], vr[t]);
    }
#pragma unroll
    for (int t = 0; t < kBatch; ++t) {
      const float bias2 = s_qbias[warp][first + min(t, n - 1)];
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float d = 0.f;
#pragma unroll
        for (int e = 0; e < EPL; ++e) d = fmaf(qv[g][e], kr[t][e], d);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
        sc[t][g] = t < n ? d + bias2 : -CUDART_INF_F;
      }
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float mx = m[g];
#pragma unroll
      for (int t = 0; t < kBatch; ++t) mx = fmaxf(mx, sc[t][g]);
      const float corr = m[g] == -CUDART_INF_F ? 0.f : exp2f(m[g] - mx);
      float pw[kBatch], psum = 0.f;
#pragma unroll
      for (int t = 0; t < kBatch; ++t) {
        pw[t] = mx == -CUDART_INF_F ? 0.f : exp2f(sc[t][g] - mx);
        psum += pw[t];
      }
      l[g] = l[g] * corr + psum;
      m[g] = mx;
#pragma unroll
      for (int e = 0; e < EPL; ++e) {
        float a = acc[g][e] * corr;
#pragma unroll
        for (int t = 0; t < kBatch; ++t) a = fmaf(pw[t], vr[t][e], a);
        acc[g][e] = a;
      }
    }
  };

  // key range of this CTA, in 32-key chunks dealt round-robin to the warps
  const int chunks_total = (p.seqlen_k + 31) / 32;
  const int chunks_per_split = (chunks_total + p.nsplit - 1) / p.nsplit;
  const int c_begin = split * chunks_per_split, c_end = min(chunks_total, c_begin + chunks_per_split);
  int qn = 0;
  for (int c = c_begin + warp; c < c_end; c += kWarps) {
    const int key = c * 32 + lane;
    bool keep = key < p.seqlen_k;
    if (keep && mrow) keep = mrow[key] != 0;
    const uint32_t bits = __ballot_sync(0xffffffffu, keep);
    if (bits == 0) continue;
    if (keep) {
      const int pos = qn + __popc(bits & ((1u << lane) - 1u));
      s_queue[warp][pos] = key;
      s_qbias[warp][pos] = brow ? raw_to_f<kBf16>(brow[key]) * 1.4426950408889634f : 0.f;
    }
    qn += __popc(bits);
    __syncwarp();
    if (qn > kQueue - 32) {  // not enough room for another full chunk: drain
      int done = 0;
      for (; done + kBatch <= qn; done += kBatch) process(done, kBatch);
      const int rest = qn - done;
      if (rest > 0) {  // move the tail to the front
        int kk = 0;
        float bb = 0.f;
        if (lane < rest) {
          kk = s_queue[warp][done + lane];
          bb = s_qbias[warp][done + lane];
        }
        __syncwarp();
        if (lane < rest) {
          s_queue[warp][lane] = kk;
          s_qbias[warp][lane] = bb;
        }
        __syncwarp();
      }
      qn = rest;
    }
  }
  for (int done = 0; done < qn; done += kBatch) process(done, min(kBatch, qn - done));

  // one partial per warp
  const int P = p.nsplit * kWarps;
#pragma unroll
  for (int g = 0; g < G; ++g) {
    float* dst = p.partial + ((static_cast<int64_t>(b) * p.h + h0 + g) * P + split * kWarps + warp) * (D + 2);
#pragma unroll
    for (int e = 0; e < EPL; ++e) dst[lane * EPL + e] = acc[g][e];
    if (lane == 0) {
      dst[D] = m[g];
      dst[D + 1] = l[g];
    }
  }
}

// O = sum_i 2^(m_i - M) acc_i / sum_i 2^(m_i - M) l_i, LSE = (M + log2(sum)) * ln2; one warp per (b, h).
template <bool kBf16>
__global__ void decode_merge_kernel(const float* __restrict__ partial, void* __restrict__ out, float* __restrict__ lse,
                                    int B, int H, int P, int D, int64_t ob, int64_t oh) {
  const int lane = threadIdx.x & 31;
  const int64_t w = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5;
  if (w >= static_cast<int64_t>(B) * H) return;
  const int h = static_cast<int>(w % H), b = static_cast<int>(w / H);
  const float* base = partial + w * P * (D + 2);
  float M = -CUDART_INF_F;
  for (int i = lane; i < P; i += 32) M = fmaxf(M, base[i * (D + 2) + D]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
  float L = 0.f;
  for (int i = lane; i < P; i += 32) {
    const float mi = base[i * (D + 2) + D];
    if (mi != -CUDART_INF_F) L += exp2f(mi - M) * base[i * (D + 2) + D + 1];
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) L += __shfl_xor_sync(0xffffffffu, L, o);
  uint16_t* op = reinterpret_cast<uint16_t*>(out) + b * ob + h * oh;
  const float inv = L > 0.f ? 1.f / L : 0.f;
  for (int dd = lane; dd < D; dd += 32) {
    float a = 0.f;
    for (int i = 0; i < P; ++i) {
      const float mi = base[i * (D + 2) + D];
      if (mi != -CUDART_INF_F) a = fmaf(exp2f(mi - M), base[i * (D + 2) + dd], a);
    }
    op[dd] = f_to_raw<kBf16>(a * inv);
  }
  if (lane == 0) lse[w] = L > 0.f ? (M + log2f(L)) * 0.6931471805599453f : CUDART_INF_F;
}

int pick_splits(const fdma_fwd_params& p, int ctas_per_split) {
  // aim at ~4 CTAs per SM; every split needs at least a few 32-key chunks per warp
  const int target = 148 * 4;
  int ns = std::max(1, target / std::max(1, ctas_per_split));
  const int max_by_len = std::max(1, (p.seqlen_k + 32 * kWarps * 4 - 1) / (32 * kWarps * 4));
  return std::min(std::min(ns, max_by_len), 64);
}

bool group_shares_mask_bias(const fdma_fwd_params& p) {
  const int G = p.h / p.h_k;
  if (G == 1) return true;
  return (!p.mask || p.h_mask != p.h) && (!p.bias || p.h_bias != p.h);
}

int group_size(const fdma_fwd_params& p) {
  const int G = p.h / p.h_k;
  if (!group_shares_mask_bias(p)) return 1;
  if (G <= kMaxGroup && (G == 1 || G == 2 || G == 4 || G == 8)) return G;
  return 1;
}

template <int EPL, bool kBf16>
int launch_epl(const DecodeParams& dp, int G, dim3 grid, cudaStream_t stream) {
  switch (G) {
    case 1: decode_kernel<EPL, 1, kBf16><<<grid, kThreads, 0, stream>>>(dp); break;
    case 2: decode_kernel<EPL, 2, kBf16><<<grid, kThreads, 0, stream>>>(dp); break;
    case 4: decode_kernel<EPL, 4, kBf16><<<grid, kThreads, 0, stream>>>(dp); break;
    default:
      if (EPL <= 4) decode_kernel<(EPL <= 4 ? EPL : 4), 8, kBf16><<<grid, kThreads, 0, stream>>>(dp);
      else return FDMA_ERR_UNSUPPORTED;
      break;
  }
  return static_cast<int>(cudaGetLastError());
}

}  // namespace

bool decode_supported(const fdma_fwd_params& p) {
  if (p.seqlen_q != 1 || p.seqlen_k <= 0) return false;
  if (p.d != 64 && p.d != 128 && p.d != 256) return false;
  const int epl = p.d / 32;
  // vector loads of EPL 16-bit elements per lane
  const int64_t need = epl;  // elements
  const void* ptrs[3] = {p.q, p.k, p.v};
  for (const void* x : ptrs)
    if (reinterpret_cast<uintptr_t>(x) % (2 * need) != 0) return false;
  const int64_t strides[7] = {p.q_batch_stride, p.q_head_stride, p.k_batch_stride, p.k_row_stride,
                              p.k_head_stride,  p.v_row_stride,  p.v_head_stride};
  for (int64_t s : strides)
    if (s % need != 0) return false;
  if (p.v_batch_stride % need != 0) return false;
  if (p.h / p.h_k > 1 && group_size(p) == 8 && epl > 4) return false;  // register budget
  if (p.b > 65535 || p.h > 65535) return false;
  return true;
}

size_t decode_workspace_bytes(const fdma_fwd_params& p) {
  const int G = group_size(p);
  const int ns = pick_splits(p, p.b * (p.h / G));
  return align256(static_cast<size_t>(p.b) * p.h * ns * kWarps * (p.d + 2) * sizeof(float));
}

int decode_fwd(const fdma_fwd_params& p, cudaStream_t stream) {
  const int G = group_size(p);
  const int ns = pick_splits(p, p.b * (p.h / G));
  const size_t need = decode_workspace_bytes(p);
  if (!p.workspace || p.workspace_bytes < need) return FDMA_ERR_WORKSPACE;
  DecodeParams dp;
  dp.q = p.q; dp.k = p.k; dp.v = p.v; dp.mask = static_cast<const uint8_t*>(p.mask); dp.bias = p.bias;
  dp.partial = static_cast<float*>(p.workspace);
  dp.q_batch_stride = p.q_batch_stride; dp.q_head_stride = p.q_head_stride;
  dp.k_batch_stride = p.k_batch_stride; dp.k_row_stride = p.k_row_stride; dp.k_head_stride = p.k_head_stride;
  dp.v_batch_stride = p.v_batch_stride; dp.v_row_stride = p.v_row_stride; dp.v_head_stride = p.v_head_stride;
  dp.mask_batch_stride = p.mask_batch_stride; dp.mask_head_stride = p.mask_head_stride;
  dp.bias_batch_stride = p.bias_batch_stride; dp.bias_head_stride = p.bias_head_stride;
  dp.b = p.b; dp.seqlen_k = p.seqlen_k; dp.h = p.h; dp.h_k = p.h_k; dp.h_mask = p.h_mask; dp.h_bias = p.h_bias;
  dp.group = p.h / p.h_k; dp.nsplit = ns;
  dp.scale_log2 = p.softmax_scale * 1.4426950408889634f;
  dim3 grid(ns, p.h / G, p.b);
  const bool bf = p.dtype == FDMA_BF16;
  int st;
  if (p.d == 64) st = bf ? launch_epl<2, true>(dp, G, grid, stream) : launch_epl<2, false>(dp, G, grid, stream);
  else if (p.d == 128) st = bf ? launch_epl<4, true>(dp, G, grid, stream) : launch_epl<4, false>(dp, G, grid, stream);
  else st = bf ? launch_epl<8, true>(dp, G, grid, stream) : launch_epl<8, false>(dp, G, grid, stream);
  if (st) return st;
  const int64_t warps = static_cast<int64_t>(p.b) * p.h;
  const unsigned blocks = static_cast<unsigned>((warps * 32 + 255) / 256);
  if (bf)
    decode_merge_kernel<true><<<blocks, 256, 0, stream>>>(dp.partial, p.out, p.lse, p.b, p.h, ns * kWarps, p.d,
                                                          p.o_batch_stride, p.o_head_stride);
  else
    decode_merge_kernel<false><<<blocks, 256, 0, stream>>>(dp.partial, p.out, p.lse, p.b, p.h, ns * kWarps, p.d,
                                                           p.o_batch_stride, p.o_head_stride);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace fdma
