// create_mask on the GPU: per row, mark the `window` largest bias values (radix select on
// order-preserving integer keys, ties at the threshold taken in ascending key index), never marking a
// value equal to the caller's min_dtype. Restates topk_mask / relu_mask / block_smooth of
// flash_sparse_attn/utils/mask.py:47-160 without the int64 index tensor and scatter of torch.topk.
//
// One CTA per row. The row's keys are staged once in shared memory (when they fit), so HBM traffic is
// the algorithmic minimum: bias row in, (pre-mask row in,) bool row out.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>

#include "fdma_internal.h"

namespace fdma {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kPerThread = 8;                     // keys per thread per chunk in the write pass
constexpr int kChunk = kThreads * kPerThread;     // 2048 keys
constexpr size_t kMaxStageBytes = 160 * 1024;     // rows up to this size are staged in shared memory

// Order-preserving map from the IEEE bit pattern to an unsigned key (larger value <-> larger key);
// NaN maps to the largest key, which is where torch.topk puts it.
__device__ __forceinline__ uint32_t key16(uint16_t u, uint16_t exp_mask, uint16_t man_mask) {
  if ((u & exp_mask) == exp_mask && (u & man_mask)) return 0xFFFFu;
  return (u & 0x8000u) ? static_cast<uint16_t>(~u) : static_cast<uint16_t>(u | 0x8000u);
}
__device__ __forceinline__ uint32_t key32(uint32_t u) {
  if ((u & 0x7F800000u) == 0x7F800000u && (u & 0x007FFFFFu)) return 0xFFFFFFFFu;
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

template <int DT>
struct KeyTraits;
template <>
struct KeyTraits<FDMA_BF16> {
  using raw_t = uint16_t;
  using key_t = uint16_t;
  static constexpr int kBits = 16;
  static __device__ __forceinline__ uint32_t key(raw_t u) { return key16(u, 0x7F80u, 0x007Fu); }
  static __device__ __forceinline__ raw_t from_float(float f) { return __bfloat16_as_ushort(__float2bfloat16_rn(f)); }
  static __device__ __forceinline__ bool positive(raw_t u) { return __bfloat162float(__ushort_as_bfloat16(u)) > 0.f; }
};
template <>
struct KeyTraits<FDMA_FP16> {
  using raw_t = uint16_t;
  using key_t = uint16_t;
  static constexpr int kBits = 16;
  static __device__ __forceinline__ uint32_t key(raw_t u) { return key16(u, 0x7C00u, 0x03FFu); }
  static __device__ __forceinline__ raw_t from_float(float f) { return __half_as_ushort(__float2half_rn(f)); }
  static __device__ __forceinline__ bool positive(raw_t u) { return __half2float(__ushort_as_half(u)) > 0.f; }
};
template <>
struct KeyTraits<FDMA_FP32> {
  using raw_t = uint32_t;
  using key_t = uint32_t;
  static constexpr int kBits = 32;
  static __device__ __forceinline__ uint32_t key(raw_t u) { return key32(u); }
  static __device__ __forceinline__ raw_t from_float(float f) { return __float_as_uint(f); }
  static __device__ __forceinline__ bool positive(raw_t u) { return __uint_as_float(u) > 0.f; }
};

struct RowPtrs {
  const void* bias;
  const uint8_t* pm;
  uint8_t* out;
};

__device__ __forceinline__ RowPtrs locate(const fdma_mask_params& p, int64_t row, int elem_bytes) {
  const int r = static_cast<int>(row % p.out_rows);
  const int h = static_cast<int>((row / p.out_rows) % p.out_h);
  const int b = static_cast<int>(row / (static_cast<int64_t>(p.out_rows) * p.out_h));
  RowPtrs rp;
  rp.bias = static_cast<const char*>(p.bias) +
            (b * p.bias_batch_stride + h * p.bias_head_stride + r * p.bias_row_stride) * elem_bytes;
  rp.pm = p.premask ? static_cast<const uint8_t*>(p.premask) + b * p.pm_batch_stride + h * p.pm_head_stride +
                          r * p.pm_row_stride
                    : nullptr;
  rp.out = static_cast<uint8_t*>(p.out) + row * p.keys;
  return rp;
}

template <int DT, bool STAGED>
__global__ void __launch_bounds__(kThreads) topk_mask_kernel(const fdma_mask_params p) {
  using KT = KeyTraits<DT>;
  using raw_t = typename KT::raw_t;
  using key_t = typename KT::key_t;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  key_t* s_keys = reinterpret_cast<key_t*>(smem_raw);
  __shared__ int s_hist[kWarps][256];
  __shared__ int s_scan[kWarps];
  __shared__ uint32_t s_prefix;
  __shared__ int s_need;
  __shared__ int s_eq_total;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n = p.keys;
  const RowPtrs rp = locate(p, blockIdx.x, sizeof(raw_t));
  const raw_t* bias = static_cast<const raw_t*>(rp.bias);
  const raw_t min_raw = KT::from_float(p.min_value);
  const uint32_t min_key = KT::key(min_raw);

  auto key_at = [&](int k) -> uint32_t {
    if (STAGED) return s_keys[k];
    raw_t u = bias[k];
    if (rp.pm && !rp.pm[k]) u = min_raw;
    return KT::key(u);
  };

  if (STAGED) {
    for (int k = tid; k < n; k += kThreads) {
      raw_t u = bias[k];
      if (rp.pm && !rp.pm[k]) u = min_raw;
      s_keys[k] = static_cast<key_t>(KT::key(u));
    }
  }
  if (tid == 0) {
    s_prefix = 0;
    s_need = min(p.window, n);
  }
  __syncthreads();

  // Radix select, most significant digit first: after each pass `prefix` holds the leading digits of the
  // window-th largest key and `need` the rank still to be found among keys that share the prefix.
  for (int shift = KT::kBits - 8; shift >= 0; shift -= 8) {
    for (int i = lane; i < 256; i += 32) s_hist[warp][i] = 0;
    __syncwarp();
    const uint32_t prefix = s_prefix;
    const uint32_t hi_mask = (shift + 8 >= 32) ? 0u : (0xFFFFFFFFu << (shift + 8));
    for (int k = tid; k < n; k += kThreads) {
      const uint32_t key = key_at(k);
      if ((key & hi_mask) == prefix) atomicAdd(&s_hist[warp][(key >> shift) & 0xFFu], 1);
    }
    __syncthreads();
    // thread t owns digit t: total count of that digit, then a suffix sum from the top digit down
    int cnt = 0;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) cnt += s_hist[w][tid];
    __syncthreads();
    s_hist[0][tid] = cnt;
    __syncthreads();
    if (warp == 0) {
      // 256 digits, 8 per lane, highest digits in lane 31
      int local[8];
      int sum = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        local[j] = s_hist[0][lane * 8 + j];
        sum += local[j];
      }
      // suffix sum across lanes: above = count of digits in higher lanes
      int above = sum;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_down_sync(0xffffffffu, above, o);
        if (lane + o < 32) above += v;
      }
      above -= sum;
      const int need = s_need;
      __syncwarp();
      int run = above;
#pragma unroll
      for (int j = 7; j >= 0; --j) {
        const int c = local[j];
        if (run < need && run + c >= need) {
          s_prefix = prefix | (static_cast<uint32_t>(lane * 8 + j) << shift);
          s_need = need - run;
          s_eq_total = c;
        }
        run += c;
      }
    }
    __syncthreads();
  }
  const uint32_t thr = s_prefix;  // key of the window-th largest value
  const int need_eq = s_need;     // how many keys equal to thr are selected (>= 1)
  const bool all_eq = need_eq >= s_eq_total;

  // Write pass, kPerThread consecutive keys per thread, ties ranked by a block-wide running count.
  int base_eq = 0;
  for (int c0 = 0; c0 < n; c0 += kChunk) {
    const int k0 = c0 + tid * kPerThread;
    uint32_t keys[kPerThread];
    int eq_cnt = 0;
#pragma unroll
    for (int j = 0; j < kPerThread; ++j) {
      const int k = k0 + j;
      keys[j] = k < n ? key_at(k) : 0u;
      eq_cnt += (k < n && keys[j] == thr) ? 1 : 0;
    }
    int rank0 = 0;
    if (!all_eq) {
      int incl = eq_cnt;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
      }
      if (lane == 31) s_scan[warp] = incl;
      __syncthreads();
      int warp_base = 0, total = 0;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) {
        const int v = s_scan[w];
        if (w < warp) warp_base += v;
        total += v;
      }
      rank0 = base_eq + warp_base + incl - eq_cnt;
      base_eq += total;
      __syncthreads();
    }
    uint8_t o[kPerThread];
#pragma unroll
    for (int j = 0; j < kPerThread; ++j) {
      const uint32_t key = keys[j];
      bool sel = key > thr;
      if (key == thr) {
        sel = all_eq || rank0 < need_eq;
        ++rank0;
      }
      o[j] = (sel && key != min_key) ? 1 : 0;
    }
    if (k0 + kPerThread <= n && ((reinterpret_cast<uintptr_t>(rp.out + k0) & 7u) == 0)) {
      uint2 v;
      v.x = o[0] | (o[1] << 8) | (o[2] << 16) | (o[3] << 24);
      v.y = o[4] | (o[5] << 8) | (o[6] << 16) | (o[7] << 24);
      *reinterpret_cast<uint2*>(rp.out + k0) = v;
    } else {
#pragma unroll
      for (int j = 0; j < kPerThread; ++j)
        if (k0 + j < n) rp.out[k0 + j] = o[j];
    }
  }
}

template <int DT>
__global__ void relu_mask_kernel(const fdma_mask_params p) {
  using KT = KeyTraits<DT>;
  using raw_t = typename KT::raw_t;
  const RowPtrs rp = locate(p, blockIdx.x, sizeof(raw_t));
  const raw_t* bias = static_cast<const raw_t*>(rp.bias);
  const raw_t min_raw = KT::from_float(p.min_value);
  for (int k = threadIdx.x; k < p.keys; k += blockDim.x) {
    raw_t u = bias[k];
    if (rp.pm && !rp.pm[k]) u = min_raw;
    rp.out[k] = KT::positive(u) ? 1 : 0;
  }
}

// Majority vote per block of `block_size` keys, in place; one warp per (row, block).
__global__ void block_smooth_kernel(uint8_t* __restrict__ out, int64_t rows, int keys, int block_size) {
  const int nblk = (keys + block_size - 1) / block_size;
  const int64_t total = rows * nblk;
  const int lane = threadIdx.x & 31;
  for (int64_t w = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5; w < total;
       w += (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5) {
    const int64_t row = w / nblk;
    const int blk = static_cast<int>(w % nblk);
    uint8_t* base = out + row * keys + static_cast<int64_t>(blk) * block_size;
    const int len = min(block_size, keys - blk * block_size);
    int cnt = 0;
    for (int i = lane; i < len; i += 32) cnt += base[i] ? 1 : 0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
    const uint8_t keep = (2 * cnt > len) ? 1 : 0;
    __syncwarp();
    for (int i = lane; i < len; i += 32) base[i] = keep;
  }
}

template <int DT>
int launch_mask(const fdma_mask_params& p, cudaStream_t stream) {
  using KT = KeyTraits<DT>;
  const int64_t rows = static_cast<int64_t>(p.out_b) * p.out_h * p.out_rows;
  if (rows == 0 || p.keys == 0) return 0;
  if (rows > 0x7FFFFFFF) return FDMA_ERR_UNSUPPORTED;
  if (p.kind == FDMA_MASK_RELU) {
    relu_mask_kernel<DT><<<static_cast<unsigned>(rows), kThreads, 0, stream>>>(p);
  } else {
    const size_t stage = static_cast<size_t>(p.keys) * sizeof(typename KT::key_t);
    if (stage <= kMaxStageBytes) {
      auto kern = topk_mask_kernel<DT, true>;
      if (stage > 32 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             static_cast<int>(kMaxStageBytes));
        if (e != cudaSuccess) return static_cast<int>(e);
      }
      kern<<<static_cast<unsigned>(rows), kThreads, stage, stream>>>(p);
    } else {
      topk_mask_kernel<DT, false><<<static_cast<unsigned>(rows), kThreads, 0, stream>>>(p);
    }
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return static_cast<int>(e);
  if (p.block_size > 1) {
    const int nblk = (p.keys + p.block_size - 1) / p.block_size;
    const int64_t warps = rows * nblk;
    const unsigned g = static_cast<unsigned>(std::min<int64_t>((warps + 7) / 8, 148 * 32));
    block_smooth_kernel<<<g, 256, 0, stream>>>(static_cast<uint8_t*>(p.out), rows, p.keys, p.block_size);
    e = cudaGetLastError();
  }
  return static_cast<int>(e);
}

}  // namespace

int create_mask(const fdma_mask_params& p, cudaStream_t stream) {
  switch (p.dtype) {
    case FDMA_BF16: return launch_mask<FDMA_BF16>(p, stream);
    case FDMA_FP16: return launch_mask<FDMA_FP16>(p, stream);
    case FDMA_FP32: return launch_mask<FDMA_FP32>(p, stream);
    default: return FDMA_ERR_UNSUPPORTED;
  }
}

}  // namespace fdma
