// fdma_merge_partials: folds one partial attention result (output + log-sum-exp over a subset of the keys) into a
// running fp32 result, with the rule the reference's split-KV combine kernel uses
// (csrc/flash_sparse_attn/src/flash_fwd_kernel.h:1695-1727):
//     lse' = log(exp(lse) + exp(lse_p)),   acc' = exp(lse - lse') acc + exp(lse_p - lse') out_p.
// The KV-ring context-parallel path calls it once per visible (query chunk, key chunk) pair. HBM-bound: one warp per
// (batch, query, head) row, 16-byte loads of the partial, 32-byte read-modify-write of the accumulator.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math_constants.h>

#include "fdma_internal.h"

namespace fdma {
namespace {

template <bool kBf16>
__global__ void __launch_bounds__(256) merge_partials_kernel(const fdma_merge_params p) {
  const int64_t w = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int64_t total = static_cast<int64_t>(p.b) * p.seqlen_q * p.h;
  if (w >= total) return;
  const int h = static_cast<int>(w % p.h);
  const int q = static_cast<int>((w / p.h) % p.seqlen_q);
  const int b = static_cast<int>(w / (static_cast<int64_t>(p.h) * p.seqlen_q));
  const int64_t li = (static_cast<int64_t>(b) * p.h + h) * p.seqlen_q + q;
  const float la = p.lse_acc[li];                      // -inf: nothing accumulated yet
  float lp = p.lse_part[li];
  if (lp == CUDART_INF_F) lp = -CUDART_INF_F;          // the forward reports rows without a visible key as +inf
  const float mx = fmaxf(la, lp);
  float wa = 0.f, wp = 0.f, ln = -CUDART_INF_F;
  if (mx != -CUDART_INF_F) {
    const float ea = __expf(la - mx), ep = __expf(lp - mx);
    ln = mx + __logf(ea + ep);
    wa = __expf(la - ln);
    wp = __expf(lp - ln);
  }
  float* arow = p.acc + w * p.d;
  const uint16_t* prow = static_cast<const uint16_t*>(p.part) + b * p.part_batch_stride +
                         static_cast<int64_t>(q) * p.part_row_stride + h * p.part_head_stride;
  for (int c = lane * 8; c < p.d; c += 256) {
    const uint4 raw = *reinterpret_cast<const uint4*>(prow + c);
    const uint32_t wds[4] = {raw.x, raw.y, raw.z, raw.w};
    float4 a0 = *reinterpret_cast<const float4*>(arow + c);
    float4 a1 = *reinterpret_cast<const float4*>(arow + c + 4);
    float o[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (kBf16) {
        o[2 * j] = __uint_as_float(wds[j] << 16);
        o[2 * j + 1] = __uint_as_float(wds[j] & 0xFFFF0000u);
      } else {
        const __half2 hh = *reinterpret_cast<const __half2*>(&wds[j]);
        o[2 * j] = __low2float(hh);
        o[2 * j + 1] = __high2float(hh);
      }
    }
    a0 = make_float4(a0.x * wa + o[0] * wp, a0.y * wa + o[1] * wp, a0.z * wa + o[2] * wp, a0.w * wa + o[3] * wp);
    a1 = make_float4(a1.x * wa + o[4] * wp, a1.y * wa + o[5] * wp, a1.z * wa + o[6] * wp, a1.w * wa + o[7] * wp);
    *reinterpret_cast<float4*>(arow + c) = a0;
    *reinterpret_cast<float4*>(arow + c + 4) = a1;
  }
  if (lane == 0) p.lse_acc[li] = ln;
}

}  // namespace
}  // namespace fdma

extern "C" int fdma_merge_partials(const fdma_merge_params* p, void* stream) {
  using namespace fdma;
  if (!p || !p->acc || !p->lse_acc || !p->part || !p->lse_part) return FDMA_ERR_BAD_ARG;
  if (p->b <= 0 || p->seqlen_q <= 0 || p->h <= 0 || p->d <= 0) return FDMA_ERR_BAD_ARG;
  if (p->d % 8 || p->d > 256) return FDMA_ERR_UNSUPPORTED;
  if (p->dtype != FDMA_BF16 && p->dtype != FDMA_FP16) return FDMA_ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(p->part) & 15u) || (reinterpret_cast<uintptr_t>(p->acc) & 15u) ||
      p->part_batch_stride % 8 || p->part_row_stride % 8 || p->part_head_stride % 8)
    return FDMA_ERR_UNSUPPORTED;
  const int64_t warps = static_cast<int64_t>(p->b) * p->seqlen_q * p->h;
  const int64_t blocks = (warps * 32 + 255) / 256;
  if (blocks > 0x7FFFFFFF) return FDMA_ERR_TOO_LARGE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (p->dtype == FDMA_BF16) merge_partials_kernel<true><<<static_cast<unsigned>(blocks), 256, 0, s>>>(*p);
  else merge_partials_kernel<false><<<static_cast<unsigned>(blocks), 256, 0, s>>>(*p);
  return static_cast<int>(cudaGetLastError());
}
