// CUDA-core kernels for dynamic-mask attention: one warp per query row, fp32 arithmetic throughout.
// They cover every head dim (multiple of 8, <= 256), every stride/broadcast combination and unaligned
// pointers, i.e. the shapes the tcgen05 kernels decline. Same math as the reference's
// compute_attn_1rowblock (csrc/flash_sparse_attn/src/flash_fwd_kernel.h:53-804) and
// compute_dq_dk_dv_1colblock (src/flash_bwd_kernel.h:79-1142), restated row-wise.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math_constants.h>

#include <algorithm>

#include "fdma_internal.h"

namespace fdma {
namespace {

constexpr int kWarpsPerBlock = 4;
constexpr int kMaxD = 256;
constexpr int kDimsPerLane = kMaxD / 32;

template <typename T>
__device__ __forceinline__ float to_f32(T x);
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 x) {
  return __bfloat162float(x);
}
template <>
__device__ __forceinline__ float to_f32<__half>(__half x) {
  return __half2float(x);
}
template <typename T>
__device__ __forceinline__ T from_f32(float x);
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) {
  return __float2bfloat16_rn(x);
}
template <>
__device__ __forceinline__ __half from_f32<__half>(float x) {
  return __float2half_rn(x);
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

struct RowCtx {
  int b, h, q, hk;
  int k_limit;  // keys [0, k_limit) pass the causal / length test
  const uint8_t* mask_row;
  const void* bias_row;
  const int32_t* pos_row;  // key positions (compacted keys) or null
  int pos_limit;           // with pos_row and causal: key k is visible iff pos_row[k] <= pos_limit
};

template <typename T>
__device__ __forceinline__ bool locate_row(const fdma_fwd_params& p, int64_t row_id, RowCtx& c) {
  const int64_t total = static_cast<int64_t>(p.b) * p.h * p.seqlen_q;
  if (row_id >= total) return false;
  c.q = static_cast<int>(row_id % p.seqlen_q);
  c.h = static_cast<int>((row_id / p.seqlen_q) % p.h);
  c.b = static_cast<int>(row_id / (static_cast<int64_t>(p.seqlen_q) * p.h));
  c.hk = c.h / (p.h / p.h_k);
  const bool causal = p.is_causal && p.seqlen_q > 1;
  int lim = p.seqlen_k;
  c.pos_row = nullptr;
  c.pos_limit = 0x7FFFFFFF;
  if (causal && p.key_pos) {
    const int hp = p.h_pos == p.h ? c.h : (p.h_pos == p.h_k ? c.hk : 0);
    c.pos_row = p.key_pos + c.b * p.key_pos_batch_stride + hp * p.key_pos_head_stride;
    c.pos_limit = c.q + p.causal_shift;
  } else if (causal) {
    lim = min(lim, c.q + 1 + p.seqlen_k - p.seqlen_q);
  }
  c.k_limit = max(lim, 0);
  c.mask_row = nullptr;
  c.bias_row = nullptr;
  if (p.mask) {
    const int hm = c.h / (p.h / p.h_mask);
    c.mask_row = static_cast<const uint8_t*>(p.mask) + c.b * p.mask_batch_stride + hm * p.mask_head_stride +
                 c.q * p.mask_row_stride;
  }
  if (p.bias) {
    const int hb = c.h / (p.h / p.h_bias);
    c.bias_row = static_cast<const T*>(p.bias) + c.b * p.bias_batch_stride + hb * p.bias_head_stride +
                 c.q * p.bias_row_stride;
  }
  return true;
}

template <typename T>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) simt_fwd_kernel(const fdma_fwd_params p) {
  __shared__ float s_q[kWarpsPerBlock][kMaxD];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  RowCtx c;
  if (!locate_row<T>(p, static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + warp, c)) return;
  const int d = p.d;
  const T* qp = static_cast<const T*>(p.q) + c.b * p.q_batch_stride + c.q * p.q_row_stride + c.h * p.q_head_stride;
  for (int i = lane; i < d; i += 32) s_q[warp][i] = to_f32(qp[i]);
  __syncwarp();
  const T* kbase = static_cast<const T*>(p.k) + c.b * p.k_batch_stride + c.hk * p.k_head_stride;
  const T* vbase = static_cast<const T*>(p.v) + c.b * p.v_batch_stride + c.hk * p.v_head_stride;
  const T* bias_row = static_cast<const T*>(c.bias_row);

  float m = -CUDART_INF_F, l = 0.f;
  float acc[kDimsPerLane];
#pragma unroll
  for (int i = 0; i < kDimsPerLane; ++i) acc[i] = 0.f;

  for (int k0 = 0; k0 < c.k_limit; k0 += 32) {
    const int k = k0 + lane;
    bool valid = k < c.k_limit;
    if (valid && c.mask_row) valid = c.mask_row[k] != 0;
    if (valid && c.pos_row) valid = c.pos_row[k] <= c.pos_limit;
    if (!__any_sync(0xffffffffu, valid)) continue;  // skipped 32-key granule
    float s = -CUDART_INF_F;
    if (valid) {
      const T* kr = kbase + static_cast<int64_t>(k) * p.k_row_stride;
      float dot = 0.f;
      for (int i = 0; i < d; ++i) dot = fmaf(s_q[warp][i], to_f32(kr[i]), dot);
      s = dot * p.softmax_scale + (bias_row ? to_f32(bias_row[k]) : 0.f);
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float pv = valid ? __expf(s - m_new) : 0.f;
    const float corr = (m == -CUDART_INF_F) ? 0.f : __expf(m - m_new);
    l = l * corr + warp_sum(pv);
#pragma unroll
    for (int i = 0; i < kDimsPerLane; ++i) acc[i] *= corr;
    for (int kk = 0; kk < 32; ++kk) {
      const float pk = __shfl_sync(0xffffffffu, pv, kk);
      if (pk == 0.f) continue;
      const T* vr = vbase + static_cast<int64_t>(k0 + kk) * p.v_row_stride;
#pragma unroll
      for (int i = 0; i < kDimsPerLane; ++i) {
        const int dd = lane + 32 * i;
        if (dd < d) acc[i] = fmaf(pk, to_f32(vr[dd]), acc[i]);
      }
    }
    m = m_new;
  }
  T* op = static_cast<T*>(p.out) + c.b * p.o_batch_stride + c.q * p.o_row_stride + c.h * p.o_head_stride;
  const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
  for (int i = 0; i < kDimsPerLane; ++i) {
    const int dd = lane + 32 * i;
    if (dd < d) op[dd] = from_f32<T>(acc[i] * inv);
  }
  if (lane == 0) {
    p.lse[(static_cast<int64_t>(c.b) * p.h + c.h) * p.seqlen_q + c.q] = l > 0.f ? m + logf(l) : CUDART_INF_F;
  }
}

// Backward, one warp per query row. dQ is owned by the warp; dK, dV and dBias are accumulated with fp32
// atomics into scratch buffers, which the convert kernel below rounds once to the output dtype.
template <typename T>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
    simt_bwd_kernel(const fdma_bwd_params bp, float* __restrict__ dk_acc, float* __restrict__ dv_acc,
                    float* __restrict__ dbias_acc) {
  const fdma_fwd_params& p = bp.f;
  __shared__ float s_q[kWarpsPerBlock][kMaxD];
  __shared__ float s_do[kWarpsPerBlock][kMaxD];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  RowCtx c;
  if (!locate_row<T>(p, static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + warp, c)) return;
  const int d = p.d;
  const T* qp = static_cast<const T*>(p.q) + c.b * p.q_batch_stride + c.q * p.q_row_stride + c.h * p.q_head_stride;
  const T* op = static_cast<const T*>(p.out) + c.b * p.o_batch_stride + c.q * p.o_row_stride + c.h * p.o_head_stride;
  const T* dop =
      static_cast<const T*>(bp.dout) + c.b * bp.do_batch_stride + c.q * bp.do_row_stride + c.h * bp.do_head_stride;
  float dsum = 0.f;
  for (int i = lane; i < d; i += 32) {
    const float g = to_f32(dop[i]);
    s_q[warp][i] = to_f32(qp[i]);
    s_do[warp][i] = g;
    dsum = fmaf(g, to_f32(op[i]), dsum);
  }
  const float D = warp_sum(dsum);
  if (bp.softmax_d && lane == 0)
    bp.softmax_d[(static_cast<int64_t>(c.b) * p.h + c.h) * ((p.seqlen_q + 127) / 128 * 128) + c.q] = D;
  __syncwarp();
  const float lse = p.lse[(static_cast<int64_t>(c.b) * p.h + c.h) * p.seqlen_q + c.q];
  const T* kbase = static_cast<const T*>(p.k) + c.b * p.k_batch_stride + c.hk * p.k_head_stride;
  const T* vbase = static_cast<const T*>(p.v) + c.b * p.v_batch_stride + c.hk * p.v_head_stride;
  const T* bias_row = static_cast<const T*>(c.bias_row);
  const int64_t kv_acc_row = static_cast<int64_t>(p.h_k) * d;  // scratch layout (B, Sk, Hk, d)
  float* dk_b = dk_acc + (static_cast<int64_t>(c.b) * p.seqlen_k * p.h_k + c.hk) * d;
  float* dv_b = dv_acc + (static_cast<int64_t>(c.b) * p.seqlen_k * p.h_k + c.hk) * d;
  float* db_row = nullptr;
  if (dbias_acc) {
    const int b2 = bp.dbias_b == 1 ? 0 : c.b;
    const int h2 = c.h / (p.h / bp.dbias_h);
    const int r2 = bp.dbias_rows == 1 ? 0 : c.q;
    db_row = dbias_acc + ((static_cast<int64_t>(b2) * bp.dbias_h + h2) * bp.dbias_rows + r2) * bp.dbias_keys;
  }

  float dq[kDimsPerLane];
#pragma unroll
  for (int i = 0; i < kDimsPerLane; ++i) dq[i] = 0.f;

  const bool row_alive = lse != CUDART_INF_F;
  for (int k0 = 0; row_alive && k0 < c.k_limit; k0 += 32) {
    const int k = k0 + lane;
    bool valid = k < c.k_limit;
    if (valid && c.mask_row) valid = c.mask_row[k] != 0;
    if (valid && c.pos_row) valid = c.pos_row[k] <= c.pos_limit;
    if (!__any_sync(0xffffffffu, valid)) continue;
    float pr = 0.f, ds = 0.f;
    if (valid) {
      const T* kr = kbase + static_cast<int64_t>(k) * p.k_row_stride;
      const T* vr = vbase + static_cast<int64_t>(k) * p.v_row_stride;
      float dot = 0.f, dp = 0.f;
      for (int i = 0; i < d; ++i) {
        dot = fmaf(s_q[warp][i], to_f32(kr[i]), dot);
        dp = fmaf(s_do[warp][i], to_f32(vr[i]), dp);
      }
      const float s = dot * p.softmax_scale + (bias_row ? to_f32(bias_row[k]) : 0.f);
      pr = __expf(s - lse);
      ds = pr * (dp - D);
      if (db_row) atomicAdd(db_row + k, ds);
    }
    for (int kk = 0; kk < 32; ++kk) {
      const float pk = __shfl_sync(0xffffffffu, pr, kk);
      const float dsk = __shfl_sync(0xffffffffu, ds, kk);
      if (pk == 0.f && dsk == 0.f) continue;
      const int krow = k0 + kk;
      const T* kr = kbase + static_cast<int64_t>(krow) * p.k_row_stride;
      float* dkr = dk_b + krow * kv_acc_row;
      float* dvr = dv_b + krow * kv_acc_row;
      const float dss = dsk * p.softmax_scale;
#pragma unroll
      for (int i = 0; i < kDimsPerLane; ++i) {
        const int dd = lane + 32 * i;
        if (dd < d) {
          dq[i] = fmaf(dss, to_f32(kr[dd]), dq[i]);
          atomicAdd(dkr + dd, dss * s_q[warp][dd]);
          atomicAdd(dvr + dd, pk * s_do[warp][dd]);
        }
      }
    }
  }
  T* dqp = static_cast<T*>(bp.dq) + c.b * bp.dq_batch_stride + c.q * bp.dq_row_stride + c.h * bp.dq_head_stride;
#pragma unroll
  for (int i = 0; i < kDimsPerLane; ++i) {
    const int dd = lane + 32 * i;
    if (dd < d) dqp[dd] = from_f32<T>(dq[i]);
  }
}

// fp32 scratch (B,S,Hk,d) -> strided output tensor of dtype T.
template <typename T>
__global__ void convert_kv_grad_kernel(const float* __restrict__ acc, T* __restrict__ out, int B, int S, int Hk,
                                       int d, int64_t sb, int64_t sr, int64_t sh) {
  const int64_t n = static_cast<int64_t>(B) * S * Hk * d;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int dd = static_cast<int>(i % d);
    const int hh = static_cast<int>((i / d) % Hk);
    const int ss = static_cast<int>((i / (static_cast<int64_t>(d) * Hk)) % S);
    const int bb = static_cast<int>(i / (static_cast<int64_t>(d) * Hk * S));
    out[bb * sb + ss * sr + hh * sh + dd] = from_f32<T>(acc[i]);
  }
}

// fp32 scratch (b,h,rows,keys) contiguous -> strided dbias of dtype T.
template <typename T>
__global__ void convert_dbias_kernel(const float* __restrict__ acc, T* __restrict__ out, int nb, int nh, int nr,
                                     int nk, int64_t sb, int64_t sh, int64_t sr) {
  const int64_t n = static_cast<int64_t>(nb) * nh * nr * nk;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int kk = static_cast<int>(i % nk);
    const int rr = static_cast<int>((i / nk) % nr);
    const int hh = static_cast<int>((i / (static_cast<int64_t>(nk) * nr)) % nh);
    const int bb = static_cast<int>(i / (static_cast<int64_t>(nk) * nr * nh));
    out[bb * sb + hh * sh + rr * sr + kk] = from_f32<T>(acc[i]);
  }
}

struct BwdScratch {
  size_t dk_off, dv_off, dbias_off, total;
};
BwdScratch bwd_scratch_layout(const fdma_bwd_params& bp) {
  const fdma_fwd_params& p = bp.f;
  BwdScratch s;
  const size_t kv = align256(static_cast<size_t>(p.b) * p.seqlen_k * p.h_k * p.d * sizeof(float));
  s.dk_off = 0;
  s.dv_off = kv;
  s.dbias_off = 2 * kv;
  const size_t db = bp.dbias ? align256(static_cast<size_t>(bp.dbias_b) * bp.dbias_h * bp.dbias_rows *
                                        bp.dbias_keys * sizeof(float))
                             : 0;
  s.total = 2 * kv + db;
  return s;
}

template <typename T>
int simt_fwd_t(const fdma_fwd_params& p, cudaStream_t stream) {
  const int64_t rows = static_cast<int64_t>(p.b) * p.h * p.seqlen_q;
  if (rows == 0) return 0;
  const int64_t blocks = (rows + kWarpsPerBlock - 1) / kWarpsPerBlock;
  simt_fwd_kernel<T><<<static_cast<unsigned>(blocks), kWarpsPerBlock * 32, 0, stream>>>(p);
  return static_cast<int>(cudaGetLastError());
}

template <typename T>
int simt_bwd_t(const fdma_bwd_params& bp, cudaStream_t stream) {
  const fdma_fwd_params& p = bp.f;
  const BwdScratch lay = bwd_scratch_layout(bp);
  if (lay.total > 0 && (bp.f.workspace == nullptr || bp.f.workspace_bytes < lay.total)) return FDMA_ERR_WORKSPACE;
  char* ws = static_cast<char*>(p.workspace);
  cudaError_t e = cudaSuccess;
  if (lay.total > 0) {
    e = cudaMemsetAsync(ws, 0, lay.total, stream);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  if (bp.softmax_d && p.seqlen_q % 128 != 0) {  // padding columns read as zero
    e = cudaMemsetAsync(bp.softmax_d, 0, static_cast<size_t>(p.b) * p.h * round_up(p.seqlen_q, 128) * sizeof(float), stream);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  float* dk_acc = reinterpret_cast<float*>(ws + lay.dk_off);
  float* dv_acc = reinterpret_cast<float*>(ws + lay.dv_off);
  float* db_acc = bp.dbias ? reinterpret_cast<float*>(ws + lay.dbias_off) : nullptr;
  const int64_t rows = static_cast<int64_t>(p.b) * p.h * p.seqlen_q;
  if (rows > 0) {
    const int64_t blocks = (rows + kWarpsPerBlock - 1) / kWarpsPerBlock;
    simt_bwd_kernel<T><<<static_cast<unsigned>(blocks), kWarpsPerBlock * 32, 0, stream>>>(bp, dk_acc, dv_acc, db_acc);
    e = cudaGetLastError();
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  const int64_t nkv = static_cast<int64_t>(p.b) * p.seqlen_k * p.h_k * p.d;
  if (nkv > 0) {
    const unsigned g = static_cast<unsigned>(std::min<int64_t>((nkv + 255) / 256, sm_count() * 16));
    convert_kv_grad_kernel<T><<<g, 256, 0, stream>>>(dk_acc, static_cast<T*>(bp.dk), p.b, p.seqlen_k, p.h_k, p.d,
                                                     bp.dk_batch_stride, bp.dk_row_stride, bp.dk_head_stride);
    convert_kv_grad_kernel<T><<<g, 256, 0, stream>>>(dv_acc, static_cast<T*>(bp.dv), p.b, p.seqlen_k, p.h_k, p.d,
                                                     bp.dv_batch_stride, bp.dv_row_stride, bp.dv_head_stride);
  }
  if (bp.dbias) {
    const int64_t ndb = static_cast<int64_t>(bp.dbias_b) * bp.dbias_h * bp.dbias_rows * bp.dbias_keys;
    if (ndb > 0) {
      const unsigned g = static_cast<unsigned>(std::min<int64_t>((ndb + 255) / 256, sm_count() * 16));
      convert_dbias_kernel<T><<<g, 256, 0, stream>>>(db_acc, static_cast<T*>(bp.dbias), bp.dbias_b, bp.dbias_h,
                                                     bp.dbias_rows, bp.dbias_keys, bp.dbias_batch_stride,
                                                     bp.dbias_head_stride, bp.dbias_row_stride);
    }
  }
  return static_cast<int>(cudaGetLastError());
}

}  // namespace

size_t simt_bwd_workspace_bytes(const fdma_bwd_params& p) { return bwd_scratch_layout(p).total; }

int simt_fwd(const fdma_fwd_params& p, cudaStream_t stream) {
  if (p.dtype == FDMA_BF16) return simt_fwd_t<__nv_bfloat16>(p, stream);
  if (p.dtype == FDMA_FP16) return simt_fwd_t<__half>(p, stream);
  return FDMA_ERR_UNSUPPORTED;
}

int simt_bwd(const fdma_bwd_params& p, cudaStream_t stream) {
  if (p.f.dtype == FDMA_BF16) return simt_bwd_t<__nv_bfloat16>(p, stream);
  if (p.f.dtype == FDMA_FP16) return simt_bwd_t<__half>(p, stream);
  return FDMA_ERR_UNSUPPORTED;
}

}  // namespace fdma
