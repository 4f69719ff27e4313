// Key compaction for row-broadcast masks: when every query of a (batch, head) shares one keep-set of W keys out of
// Sk, attention over the W kept keys gives the same result as attention over all Sk keys, as long as the causal
// test still runs on the keys' ORIGINAL positions. This file builds the ascending position list of each mask row
// (fdma_compact_index), gathers the kept K / V / bias rows into dense tensors (fdma_gather_rows) and scatters the
// gradients of the compact tensors back into zero-filled full-size ones (fdma_scatter_rows). The attention kernels
// take the position list through fdma_fwd_params::key_pos.
//
// The reference's CUDA backend has no such path; its Triton prototype gathers keys by top-k index
// (flash_sparse_attn/flash_dmattn_triton.py:49-211). All three kernels are plain HBM-bound copies.
#include <cstdint>
#include <utility>
#include <cuda_runtime.h>

#include "fdma_internal.h"

namespace fdma {
namespace {

constexpr int kIdxThreads = 256;
constexpr int kIdxPerThread = 16;  // mask bytes scanned per thread and round

// One CTA per mask row: running exclusive scan of the keep flags; kept key k lands in slot (number of kept keys
// before it). Slots beyond the count are filled with INT32_MAX, mask_out marks the filled slots.
__global__ void __launch_bounds__(kIdxThreads) compact_index_kernel(const uint8_t* __restrict__ mask, int64_t sb,
                                                                     int64_t sh, int Hm, int Sk, int cap,
                                                                     int32_t* __restrict__ key_pos,
                                                                     int32_t* __restrict__ count,
                                                                     uint8_t* __restrict__ mask_out) {
  __shared__ int s_warp[kIdxThreads / 32];
  __shared__ int s_base;
  const int row = blockIdx.x;
  const int b = row / Hm, hm = row % Hm;
  const uint8_t* mrow = mask + b * sb + hm * sh;
  int32_t* prow = key_pos + static_cast<int64_t>(row) * cap;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) s_base = 0;
  __syncthreads();
  const bool vec_ok = (reinterpret_cast<uintptr_t>(mrow) & 15u) == 0;
  for (int k0 = 0; k0 < Sk; k0 += kIdxThreads * kIdxPerThread) {
    const int k = k0 + tid * kIdxPerThread;
    uint32_t bits = 0;  // bit i = key k + i kept
    if (vec_ok && k + kIdxPerThread <= Sk) {
      const uint4 v = *reinterpret_cast<const uint4*>(mrow + k);
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int i = 0; i < 16; ++i)
        if ((w[i >> 2] >> ((i & 3) * 8)) & 0xFFu) bits |= 1u << i;
    } else {
      for (int i = 0; i < kIdxPerThread; ++i)
        if (k + i < Sk && mrow[k + i]) bits |= 1u << i;
    }
    const int mine = __popc(bits);
    int incl = mine;
#pragma unroll
    for (int s = 1; s < 32; s <<= 1) {
      const int o = __shfl_up_sync(0xffffffffu, incl, s);
      if (lane >= s) incl += o;
    }
    if (lane == 31) s_warp[warp] = incl;
    __syncthreads();
    int before = s_base + incl - mine;
    for (int w = 0; w < warp; ++w) before += s_warp[w];
    while (bits) {
      const int i = __ffs(bits) - 1;
      bits &= bits - 1;
      if (before < cap) prow[before] = k + i;
      ++before;
    }
    __syncthreads();
    if (tid == kIdxThreads - 1) s_base = before;  // the last thread's running total is the row's
    __syncthreads();
  }
  const int total = s_base;
  if (tid == 0) count[row] = total;
  for (int s = tid; s < cap; s += kIdxThreads) {
    if (s >= total) prow[s] = 0x7FFFFFFF;
    if (mask_out) mask_out[static_cast<int64_t>(row) * cap + s] = s < total ? 1 : 0;
  }
}

struct RowsArgs {
  const unsigned char* src;
  unsigned char* dst;
  const int32_t* key_pos;
  int64_t pos_sb, pos_sh;
  int64_t src_sb, src_sr, src_sh;  // bytes
  int64_t dst_sb, dst_sr, dst_sh;  // bytes
  int b, heads, h_pos, rows_full, cap, row_bytes;
};

// Gather (kScatter = false): dst[b][slot][h] = src[b][pos[slot]][h], zero for padding slots.
// Scatter (kScatter = true): dst[b][pos[slot]][h] = src[b][slot][h] for filled slots (dst was zero-filled before).
// One warp per (b, slot, h) row, kVec bytes per lane and step.
template <bool kScatter, int kVec>
__global__ void __launch_bounds__(256) rows_kernel(const RowsArgs a) {
  const int64_t w = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int64_t total = static_cast<int64_t>(a.b) * a.cap * a.heads;
  if (w >= total) return;
  const int h = static_cast<int>(w % a.heads);
  const int slot = static_cast<int>((w / a.heads) % a.cap);
  const int b = static_cast<int>(w / (static_cast<int64_t>(a.heads) * a.cap));
  const int hp = h / (a.heads / a.h_pos);
  const int pos = a.key_pos[b * a.pos_sb + hp * a.pos_sh + slot];
  const bool filled = pos >= 0 && pos < a.rows_full;
  const unsigned char* s;
  unsigned char* d;
  if (kScatter) {
    if (!filled) return;
    s = a.src + b * a.src_sb + static_cast<int64_t>(slot) * a.src_sr + h * a.src_sh;
    d = a.dst + b * a.dst_sb + static_cast<int64_t>(pos) * a.dst_sr + h * a.dst_sh;
  } else {
    s = a.src + b * a.src_sb + static_cast<int64_t>(filled ? pos : 0) * a.src_sr + h * a.src_sh;
    d = a.dst + b * a.dst_sb + static_cast<int64_t>(slot) * a.dst_sr + h * a.dst_sh;
  }
  for (int o = lane * kVec; o < a.row_bytes; o += 32 * kVec) {
    if (kVec == 16) {
      uint4 v = make_uint4(0, 0, 0, 0);
      if (kScatter || filled) v = *reinterpret_cast<const uint4*>(s + o);
      *reinterpret_cast<uint4*>(d + o) = v;
    } else {
      uint16_t v = 0;
      if (kScatter || filled) v = *reinterpret_cast<const uint16_t*>(s + o);
      *reinterpret_cast<uint16_t*>(d + o) = v;
    }
  }
}

// Zero fill of a strided (b, rows, heads, row_bytes) tensor, one warp per row.
template <int kVec>
__global__ void __launch_bounds__(256) zero_rows_kernel(unsigned char* dst, int64_t sb, int64_t sr, int64_t sh, int b,
                                                         int rows, int heads, int row_bytes) {
  const int64_t w = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int64_t total = static_cast<int64_t>(b) * rows * heads;
  if (w >= total) return;
  const int h = static_cast<int>(w % heads);
  const int r = static_cast<int>((w / heads) % rows);
  const int bb = static_cast<int>(w / (static_cast<int64_t>(heads) * rows));
  unsigned char* d = dst + bb * sb + static_cast<int64_t>(r) * sr + h * sh;
  for (int o = lane * kVec; o < row_bytes; o += 32 * kVec) {
    if (kVec == 16) *reinterpret_cast<uint4*>(d + o) = make_uint4(0, 0, 0, 0);
    else *reinterpret_cast<uint16_t*>(d + o) = 0;
  }
}

bool all16(const fdma_rows_params& p, int eb) {
  auto a16 = [](const void* x) { return (reinterpret_cast<uintptr_t>(x) & 15u) == 0; };
  const int64_t strides[6] = {p.src_batch_stride, p.src_row_stride, p.src_head_stride,
                              p.dst_batch_stride, p.dst_row_stride, p.dst_head_stride};
  for (int64_t s : strides)
    if ((s * eb) % 16) return false;
  return a16(p.src) && a16(p.dst) && (static_cast<int64_t>(p.row_elems) * eb) % 16 == 0;
}

// True when the destination's elements form one contiguous block (any order of the dimensions), so that the zero
// fill of a scatter can be a single memset.
bool dst_is_dense(const fdma_rows_params& p) {
  const int64_t ext_all[4] = {p.b, p.rows_full, p.heads, p.row_elems};
  const int64_t str_all[4] = {p.dst_batch_stride, p.dst_row_stride, p.dst_head_stride, 1};
  int64_t ext[4], str[4];
  int n = 0;
  for (int i = 0; i < 4; ++i)
    if (ext_all[i] != 1) {  // a dimension of extent 1 is never stepped over
      ext[n] = ext_all[i];
      str[n] = str_all[i];
      ++n;
    }
  for (int i = 1; i < n; ++i)  // insertion sort by stride
    for (int j = i; j > 0 && str[j] < str[j - 1]; --j) {
      std::swap(ext[j], ext[j - 1]);
      std::swap(str[j], str[j - 1]);
    }
  int64_t expect = 1;
  for (int i = 0; i < n; ++i) {
    if (str[i] != expect) return false;
    expect *= ext[i];
  }
  return true;
}

int check_rows(const fdma_rows_params* p) {
  if (!p || !p->src || !p->dst || !p->key_pos) return FDMA_ERR_BAD_ARG;
  if (p->b <= 0 || p->heads <= 0 || p->h_pos <= 0 || p->rows_full <= 0 || p->capacity <= 0 || p->row_elems <= 0)
    return FDMA_ERR_BAD_ARG;
  if (p->heads % p->h_pos) return FDMA_ERR_BAD_ARG;
  if (p->dtype != FDMA_BF16 && p->dtype != FDMA_FP16) return FDMA_ERR_UNSUPPORTED;
  return 0;
}

RowsArgs make_args(const fdma_rows_params& p) {
  const int eb = 2;
  RowsArgs a;
  a.src = static_cast<const unsigned char*>(p.src);
  a.dst = static_cast<unsigned char*>(p.dst);
  a.key_pos = p.key_pos;
  a.pos_sb = p.key_pos_batch_stride; a.pos_sh = p.key_pos_head_stride;
  a.src_sb = p.src_batch_stride * eb; a.src_sr = p.src_row_stride * eb; a.src_sh = p.src_head_stride * eb;
  a.dst_sb = p.dst_batch_stride * eb; a.dst_sr = p.dst_row_stride * eb; a.dst_sh = p.dst_head_stride * eb;
  a.b = p.b; a.heads = p.heads; a.h_pos = p.h_pos; a.rows_full = p.rows_full; a.cap = p.capacity;
  a.row_bytes = p.row_elems * eb;
  return a;
}

}  // namespace
}  // namespace fdma

extern "C" int fdma_compact_index(const fdma_compact_params* p, void* stream) {
  using namespace fdma;
  if (!p || !p->mask || !p->key_pos || !p->count) return FDMA_ERR_BAD_ARG;
  if (p->b_mask <= 0 || p->h_mask <= 0 || p->seqlen_k <= 0 || p->capacity <= 0) return FDMA_ERR_BAD_ARG;
  const int64_t rows = static_cast<int64_t>(p->b_mask) * p->h_mask;
  if (rows > 0x7FFFFFFF) return FDMA_ERR_TOO_LARGE;
  compact_index_kernel<<<static_cast<unsigned>(rows), kIdxThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(p->mask), p->mask_batch_stride, p->mask_head_stride, p->h_mask, p->seqlen_k,
      p->capacity, p->key_pos, p->count, static_cast<uint8_t*>(p->mask_out));
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fdma_gather_rows(const fdma_rows_params* p, void* stream) {
  using namespace fdma;
  if (int st = check_rows(p)) return st;
  const RowsArgs a = make_args(*p);
  const int64_t warps = static_cast<int64_t>(p->b) * p->capacity * p->heads;
  const unsigned blocks = static_cast<unsigned>((warps * 32 + 255) / 256);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (all16(*p, 2)) rows_kernel<false, 16><<<blocks, 256, 0, s>>>(a);
  else rows_kernel<false, 2><<<blocks, 256, 0, s>>>(a);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fdma_scatter_rows(const fdma_rows_params* p, void* stream) {
  using namespace fdma;
  if (int st = check_rows(p)) return st;
  const RowsArgs a = make_args(*p);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool v16 = all16(*p, 2);
  if (dst_is_dense(*p)) {
    const size_t bytes = static_cast<size_t>(p->b) * p->rows_full * p->heads * a.row_bytes;
    const cudaError_t e = cudaMemsetAsync(a.dst, 0, bytes, s);
    if (e != cudaSuccess) return static_cast<int>(e);
  } else {
    const int64_t zwarps = static_cast<int64_t>(p->b) * p->rows_full * p->heads;
    const unsigned zblocks = static_cast<unsigned>((zwarps * 32 + 255) / 256);
    if (v16) zero_rows_kernel<16><<<zblocks, 256, 0, s>>>(a.dst, a.dst_sb, a.dst_sr, a.dst_sh, a.b, a.rows_full, a.heads, a.row_bytes);
    else zero_rows_kernel<2><<<zblocks, 256, 0, s>>>(a.dst, a.dst_sb, a.dst_sr, a.dst_sh, a.b, a.rows_full, a.heads, a.row_bytes);
  }
  const int64_t warps = static_cast<int64_t>(p->b) * p->capacity * p->heads;
  const unsigned blocks = static_cast<unsigned>((warps * 32 + 255) / 256);
  if (v16) rows_kernel<true, 16><<<blocks, 256, 0, s>>>(a);
  else rows_kernel<true, 2><<<blocks, 256, 0, s>>>(a);
  return static_cast<int>(cudaGetLastError());
}
