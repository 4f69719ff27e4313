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
  // 32-bit divisions (row counts are validated to fit): 64-bit ones cost several hundred instructions per row
  const uint32_t row32 = static_cast<uint32_t>(row);
  const uint32_t bh = row32 / static_cast<uint32_t>(p.out_rows);
  const int r = static_cast<int>(row32 - bh * static_cast<uint32_t>(p.out_rows));
  const uint32_t b32 = bh / static_cast<uint32_t>(p.out_h);
  const int h = static_cast<int>(bh - b32 * static_cast<uint32_t>(p.out_h));
  const int64_t b = b32;
  RowPtrs rp;
  rp.bias = static_cast<const char*>(p.bias) +
            (b * p.bias_batch_stride + h * p.bias_head_stride + r * p.bias_row_stride) * elem_bytes;
  rp.pm = p.premask ? static_cast<const uint8_t*>(p.premask) + b * p.pm_batch_stride + h * p.pm_head_stride +
                          r * p.pm_row_stride
                    : nullptr;
  rp.out = p.out ? static_cast<uint8_t*>(p.out) + row * p.keys : nullptr;
  return rp;
}

// Position output of a row, after its selected keys were written to slots [0, total): the row's count, INT32_MAX in
// the unused slots, and the optional slot mask (slot < count).
__device__ __forceinline__ void finish_positions(const fdma_mask_params& p, int64_t row, int total, int tid,
                                                 int nthreads) {
  if (tid == 0) p.count[row] = total;
  int32_t* prow = p.key_pos + row * p.capacity;
  uint8_t* mrow = p.slot_mask ? static_cast<uint8_t*>(p.slot_mask) + row * p.capacity : nullptr;
  for (int s = tid; s < p.capacity; s += nthreads) {
    if (s >= total) prow[s] = 0x7FFFFFFF;
    if (mrow) mrow[s] = s < total ? 1 : 0;
  }
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
  int base_eq = 0, base_sel = 0;
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
    if (rp.out) {
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
    if (p.key_pos) {  // ascending positions of the selected keys: block-wide running count of selections
      int cnt = 0;
#pragma unroll
      for (int j = 0; j < kPerThread; ++j) cnt += (k0 + j < n && o[j]) ? 1 : 0;
      int incl = cnt;
#pragma unroll
      for (int s = 1; s < 32; s <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, s);
        if (lane >= s) incl += v;
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
      int slot = base_sel + warp_base + incl - cnt;
      int32_t* prow = p.key_pos + static_cast<int64_t>(blockIdx.x) * p.capacity;
#pragma unroll
      for (int j = 0; j < kPerThread; ++j) {
        if (k0 + j < n && o[j]) {
          if (slot < p.capacity) prow[slot] = k0 + j;
          ++slot;
        }
      }
      base_sel += total;
      __syncthreads();
    }
  }
  if (p.key_pos) finish_positions(p, blockIdx.x, base_sel, tid, kThreads);
}


// ---------------------------------------------------------------------------------------------------------
// Fast path for 16-bit biases with rows of at most 32768 keys: the whole row lives in REGISTERS as packed pairs
// of integer keys (8 keys per thread and 2048-key chunk, loaded with one 16-byte access), the key transform and
// the final comparisons run two keys per instruction (SIMD-in-a-word intrinsics), and shared memory holds only
// the radix histograms. About 4x fewer instructions per key than the staged kernel, which is issue-bound.
// ---------------------------------------------------------------------------------------------------------
template <int DT>
__device__ __forceinline__ uint32_t key_pair16(uint32_t u) {
  // per half: negative -> ~u, non-negative -> u | 0x8000; NaN (either sign) -> 0xFFFF. Plain 32-bit operations on
  // both halves at once (the SIMD-in-a-word compare intrinsics expand to several instructions each).
  constexpr uint32_t kExp = (DT == FDMA_BF16) ? 0x7F807F80u : 0x7C007C00u;
  const uint32_t neg = ((u >> 15) & 0x00010001u) * 0xFFFFu;     // 0xFFFF in every half whose sign bit is set
  const uint32_t key = u ^ (neg | 0x80008000u);
  // a magnitude above infinity makes (magnitude + 0x7FFF - infinity) reach bit 15 of its half; the sum stays below
  // 0x10000, so nothing carries into the other half
  const uint32_t t = (u & 0x7FFF7FFFu) + (0x7FFF7FFFu - kExp);
  const uint32_t nan = ((t >> 15) & 0x00010001u) * 0xFFFFu;
  return key | nan;
}

constexpr int kTieSlots = 32;  // up to this many keys tied at the threshold are ranked by one warp

// kPos: also (or, with a null `out`, only) writes the ascending positions of the selected keys.
template <int DT, int CHUNKS, bool kPos>
__global__ void __launch_bounds__(kThreads, CHUNKS <= 4 ? 4 : 1) topk16_reg_kernel(const fdma_mask_params p) {
  using KT = KeyTraits<DT>;
  __shared__ int s_hist[kWarps][256];
  __shared__ int s_scan[CHUNKS * kWarps];
  __shared__ uint32_t s_prefix;
  __shared__ int s_need;
  __shared__ int s_eq_total;
  __shared__ int s_tie[kTieSlots];  // indices of the keys tied at the threshold, when they are few
  __shared__ int s_tie_n;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n = p.keys;
  const int64_t total_rows = static_cast<int64_t>(p.out_b) * p.out_h * p.out_rows;
  const uint32_t min_key = KT::key(KT::from_float(p.min_value));
  const uint32_t min2 = min_key | (min_key << 16);

  // One row per CTA when launched with one CTA per row (the default); the loop also serves smaller grids.
  uint4 raw[CHUNKS];
  uint2 rawm[CHUNKS];
  auto fetch = [&](int64_t row) {
    if (row >= total_rows) return;
    const RowPtrs r = locate(p, row, 2);
    const uint16_t* b16 = static_cast<const uint16_t*>(r.bias);
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      const int k = c * kChunk + tid * kPerThread;
      if (k < n) {
        raw[c] = *reinterpret_cast<const uint4*>(b16 + k);
        if (r.pm) rawm[c] = *reinterpret_cast<const uint2*>(r.pm + k);
      }
    }
  };
  // (Fetching the next row while this one is processed was measured on B200: more registers, fewer CTAs, slower.)
  for (int64_t row = blockIdx.x; row < total_rows; row += gridDim.x) {
  const RowPtrs rp = locate(p, row, 2);
  // bit-packed output: this row's bits as bytes (key k -> bit k & 7 of byte k >> 3, the little-endian view of the
  // uint32 words)
  uint8_t* bits_row = nullptr;
  if (p.bits) bits_row = reinterpret_cast<uint8_t*>(p.bits + row * (((n + 127) / 128) * 4));
  fetch(row);
  // ---- transform: chunk c holds keys [c*2048 + tid*8, +8) of the row ----
  uint32_t kw[CHUNKS][4];
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    const int k = c * kChunk + tid * kPerThread;
    if (k < n) {
      const uint4 v = raw[c];
      kw[c][0] = key_pair16<DT>(v.x);
      kw[c][1] = key_pair16<DT>(v.y);
      kw[c][2] = key_pair16<DT>(v.z);
      kw[c][3] = key_pair16<DT>(v.w);
      if (rp.pm) {  // pre-mask: a masked key takes the value min_dtype
        const uint32_t mb[2] = {rawm[c].x, rawm[c].y};
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          const uint32_t two = mb[w >> 1] >> ((w & 1) * 16);          // bytes of keys 2w, 2w+1
          const uint32_t keep = ((two & 0xFFu) ? 0x0000FFFFu : 0u) | ((two & 0xFF00u) ? 0xFFFF0000u : 0u);
          kw[c][w] = (kw[c][w] & keep) | (min2 & ~keep);
        }
      }
    } else {
      kw[c][0] = kw[c][1] = kw[c][2] = kw[c][3] = 0u;  // below every real key, never counted, never written
    }
  }
  for (int i = lane; i < 256; i += 32) s_hist[warp][i] = 0;
  if (tid == 0) {
    s_prefix = 0;
    s_need = min(p.window, n);
    s_tie_n = 0;
  }
  __syncwarp();
  // ---- pass 1: histogram of the high byte ----
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    if (c * kChunk + tid * kPerThread < n) {
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        atomicAdd(&s_hist[warp][__byte_perm(kw[c][w], 0, 0x4441)], 1);
        atomicAdd(&s_hist[warp][kw[c][w] >> 24], 1);
      }
    }
  }
  // digit selection shared by both passes: finds the digit that holds rank `need` counted from the top
  auto select_digit = [&](int shift) {
    __syncthreads();
    int cnt = 0;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) cnt += s_hist[w][tid];
    __syncthreads();
    s_hist[0][tid] = cnt;
    __syncthreads();
    if (warp == 0) {
      int local[8];
      int sum = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        local[j] = s_hist[0][lane * 8 + j];
        sum += local[j];
      }
      int above = sum;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_down_sync(0xffffffffu, above, o);
        if (lane + o < 32) above += v;
      }
      above -= sum;
      const int need = s_need;
      const uint32_t prefix = s_prefix;
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
  };
  select_digit(8);
  // ---- pass 2: histogram of the low byte among keys whose high byte matches ----
  const uint32_t hi = s_prefix >> 8;
  for (int i = lane; i < 256; i += 32) s_hist[warp][i] = 0;
  __syncwarp();
#pragma unroll
  for (int c = 0; c < CHUNKS; ++c) {
    if (c * kChunk + tid * kPerThread < n) {
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const uint32_t x = kw[c][w];
        if (__byte_perm(x, 0, 0x4441) == hi) atomicAdd(&s_hist[warp][x & 0xFFu], 1);
        if ((x >> 24) == hi) atomicAdd(&s_hist[warp][__byte_perm(x, 0, 0x4442)], 1);
      }
    }
  }
  select_digit(0);
  const uint32_t thr = s_prefix;
  const int need_eq = s_need;
  const bool all_eq = need_eq >= s_eq_total;
  const bool check_min = thr <= min_key;  // only then can a selected key hold the value min_dtype

  // ---- write pass: two output bytes per packed word (bit 0 = low key, bit 8 = high key) ----
  uint32_t selbits[(CHUNKS + 3) / 4];
#pragma unroll
  for (int i = 0; i < (CHUNKS + 3) / 4; ++i) selbits[i] = 0u;
  auto emit = [&](int c, uint32_t (&ob)[4]) {
    const int k = c * kChunk + tid * kPerThread;
    if (k >= n) return;
    if (check_min) {  // a value equal to min_dtype is never marked
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        if ((kw[c][w] & 0xFFFFu) == min_key) ob[w] &= ~1u;
        if ((kw[c][w] >> 16) == min_key) ob[w] &= ~0x100u;
      }
    }
    uint2 o;
    o.x = ob[0] | (ob[1] << 16);
    o.y = ob[2] | (ob[3] << 16);
    if (rp.out) *reinterpret_cast<uint2*>(rp.out + k) = o;
    if (kPos || bits_row) {  // bit j of the chunk's byte = key k + j selected
      const uint32_t b8 = (((o.x & 0x01010101u) * 0x01020408u) >> 24) | ((((o.y & 0x01010101u) * 0x01020408u) >> 24) << 4);
      if (kPos) selbits[c >> 2] |= b8 << ((c & 3) * 8);
      if (bits_row) bits_row[k >> 3] = static_cast<uint8_t>(b8);  // every byte of keys [0, n); the caller zeroed the rest
    }
  };
  if (all_eq) {  // every key equal to the threshold is kept
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      uint32_t ob[4];
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const uint32_t lo = kw[c][w] & 0xFFFFu, hi2 = kw[c][w] >> 16;
        ob[w] = (lo >= thr ? 1u : 0u) | (hi2 >= thr ? 0x100u : 0u);
      }
      emit(c, ob);
    }
  } else if (!kPos && s_eq_total <= kTieSlots) {
    // A handful of keys tied at the threshold (the usual case): the lowest key indices win. Every thread writes the
    // keys above the threshold and drops the index of each tied key of its own into a short list; after a barrier
    // warp 0 ranks the list (one entry per lane, 32 shuffles) and sets the bytes of the winners itself. The
    // block-wide scans of the general path below cost a quarter of the kernel's time.
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      uint32_t ob[4];
      const int k = c * kChunk + tid * kPerThread;
      bool any = false;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const uint32_t lo = kw[c][w] & 0xFFFFu, hi2 = kw[c][w] >> 16;
        ob[w] = (lo > thr ? 1u : 0u) | (hi2 > thr ? 0x100u : 0u);
        any |= lo == thr || hi2 == thr;
      }
      emit(c, ob);
      if (any && k < n) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint32_t key = (j & 1) ? (kw[c][j >> 1] >> 16) : (kw[c][j >> 1] & 0xFFFFu);
          if (key == thr) s_tie[atomicAdd(&s_tie_n, 1)] = k + j;
        }
      }
    }
    __syncthreads();  // the list is complete, and every byte of the row has been written once
    if (warp == 0 && thr != min_key) {  // (keys equal to min_dtype are never marked)
      const int nt = s_tie_n;  // == s_eq_total
      const int mine = lane < nt ? s_tie[lane] : 0x7FFFFFFF;
      int rank = 0;
#pragma unroll
      for (int j = 0; j < 32; ++j) rank += __shfl_sync(0xffffffffu, mine, j) < mine ? 1 : 0;
      if (lane < nt && rank < need_eq) {
        if (rp.out) rp.out[mine] = 1;
        if (bits_row) {
          atomicOr(reinterpret_cast<unsigned*>(bits_row) + (mine >> 5), 1u << (mine & 31));
        }
      }
    }
  } else {
    // ties at the threshold: the lowest key indices win. Keys are ranked chunk by chunk, thread by thread; one
    // block-wide scan of the per-(chunk, thread) tie counts gives every thread the rank of its first tie.
    int excl[CHUNKS];
    uint32_t has_eq = 0;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      int cnt = 0;
      if (c * kChunk + tid * kPerThread < n) {
#pragma unroll
        for (int w = 0; w < 4; ++w)
          cnt += ((kw[c][w] & 0xFFFFu) == thr ? 1 : 0) + ((kw[c][w] >> 16) == thr ? 1 : 0);
      }
      if (cnt) has_eq |= 1u << c;
      int incl = cnt;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
      }
      excl[c] = incl - cnt;
      if (lane == 31) s_scan[c * kWarps + warp] = incl;
    }
    __syncthreads();
    int base = 0;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      uint32_t ob[4];
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const uint32_t lo = kw[c][w] & 0xFFFFu, hi2 = kw[c][w] >> 16;
        ob[w] = (lo > thr ? 1u : 0u) | (hi2 > thr ? 0x100u : 0u);
      }
      int warp_base = 0, total = 0;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) {
        const int v = s_scan[c * kWarps + w];
        if (w < warp) warp_base += v;
        total += v;
      }
      if ((has_eq >> c) & 1u) {
        int rank = base + warp_base + excl[c];
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          if ((kw[c][w] & 0xFFFFu) == thr) {
            if (rank < need_eq) ob[w] |= 1u;
            ++rank;
          }
          if ((kw[c][w] >> 16) == thr) {
            if (rank < need_eq) ob[w] |= 0x100u;
            ++rank;
          }
        }
      }
      base += total;
      emit(c, ob);
    }
  }
  if (kPos) {
    // ascending positions: selections are counted chunk by chunk, thread by thread, with one block-wide scan
    __syncthreads();  // s_scan may still be read by the tie ranking above
    int excl[CHUNKS];
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      const int cnt = __popc((selbits[c >> 2] >> ((c & 3) * 8)) & 0xFFu);
      int incl = cnt;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
      }
      excl[c] = incl - cnt;
      if (lane == 31) s_scan[c * kWarps + warp] = incl;
    }
    __syncthreads();
    int32_t* prow = p.key_pos + row * p.capacity;
    int base = 0;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
      int warp_base = 0, total = 0;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) {
        const int v = s_scan[c * kWarps + w];
        if (w < warp) warp_base += v;
        total += v;
      }
      uint32_t bits = (selbits[c >> 2] >> ((c & 3) * 8)) & 0xFFu;
      int slot = base + warp_base + excl[c];
      const int k = c * kChunk + tid * kPerThread;
      while (bits) {
        const int j = __ffs(bits) - 1;
        bits &= bits - 1;
        if (slot < p.capacity) prow[slot] = k + j;
        ++slot;
      }
      base += total;
    }
    finish_positions(p, row, base, tid, kThreads);
  }
  __syncthreads();  // the shared selection state is rewritten at the top of the next row
  }  // row loop
}

// Tile activity of a bit-packed mask: act[bh][mt][nt] = 1 iff some row of query tile mt has a bit set among the 128
// keys of key tile nt. One warp per tile, four rows per lane, 16 bytes per row.
__global__ void activity_from_bits_kernel(const uint32_t* __restrict__ bits, uint8_t* __restrict__ act, int bh_count,
                                          int rows, int key_tiles) {
  const int lane = threadIdx.x & 31;
  const int row_tiles = (rows + 127) / 128;
  const int64_t total = static_cast<int64_t>(bh_count) * row_tiles * key_tiles;
  const int64_t w = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5;
  if (w >= total) return;
  const int nt = static_cast<int>(w % key_tiles);
  const int mt = static_cast<int>((w / key_tiles) % row_tiles);
  const int64_t bh = w / (static_cast<int64_t>(key_tiles) * row_tiles);
  uint32_t any = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = mt * 128 + i * 32 + lane;
    if (r < rows) {
      const uint4 v = *reinterpret_cast<const uint4*>(bits + ((bh * rows + r) * key_tiles + nt) * 4);
      any |= v.x | v.y | v.z | v.w;
    }
  }
  const bool set = __any_sync(0xffffffffu, any != 0);
  if (lane == 0) act[w] = set ? 1 : 0;
}

template <int DT>
bool reg_path_ok(const fdma_mask_params& p) {
  if (DT == FDMA_FP32) return false;
  if (p.keys % kPerThread != 0 || p.keys > 16 * kChunk) return false;
  if (reinterpret_cast<uintptr_t>(p.bias) & 15u) return false;
  if (p.bias_batch_stride % 8 || p.bias_head_stride % 8 || p.bias_row_stride % 8) return false;
  if (p.premask) {
    if (reinterpret_cast<uintptr_t>(p.premask) & 7u) return false;
    if (p.pm_batch_stride % 8 || p.pm_head_stride % 8 || p.pm_row_stride % 8) return false;
  }
  return (reinterpret_cast<uintptr_t>(p.out) & 7u) == 0;  // a null `out` (positions only) passes
}

template <int DT, bool kPos>
void launch_reg_p(const fdma_mask_params& p, unsigned rows, cudaStream_t stream) {
  const int chunks = (p.keys + kChunk - 1) / kChunk;
  if (chunks <= 1) topk16_reg_kernel<DT, 1, kPos><<<rows, kThreads, 0, stream>>>(p);
  else if (chunks <= 2) topk16_reg_kernel<DT, 2, kPos><<<rows, kThreads, 0, stream>>>(p);
  else if (chunks <= 4) topk16_reg_kernel<DT, 4, kPos><<<rows, kThreads, 0, stream>>>(p);
  else if (chunks <= 8) topk16_reg_kernel<DT, 8, kPos><<<rows, kThreads, 0, stream>>>(p);
  else topk16_reg_kernel<DT, 16, kPos><<<rows, kThreads, 0, stream>>>(p);
}
template <int DT>
void launch_reg(const fdma_mask_params& p, unsigned rows, cudaStream_t stream) {
  if (p.key_pos) launch_reg_p<DT, true>(p, rows, stream);
  else launch_reg_p<DT, false>(p, rows, stream);
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
  if (p.bits && (p.kind != FDMA_MASK_TOPK || !reg_path_ok<DT>(p))) return FDMA_ERR_UNSUPPORTED;  // register kernel only
  if (p.kind == FDMA_MASK_RELU) {
    relu_mask_kernel<DT><<<static_cast<unsigned>(rows), kThreads, 0, stream>>>(p);
  } else if (reg_path_ok<DT>(p)) {
    if constexpr (DT != FDMA_FP32) launch_reg<DT>(p, static_cast<unsigned>(rows), stream);
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
  if (p.bits) {
    const int key_tiles = (p.keys + 127) / 128;
    const int64_t tiles = static_cast<int64_t>(p.out_b) * p.out_h * ((p.out_rows + 127) / 128) * key_tiles;
    activity_from_bits_kernel<<<static_cast<unsigned>((tiles * 32 + 255) / 256), 256, 0, stream>>>(
        p.bits, p.activity, p.out_b * p.out_h, p.out_rows, key_tiles);
    e = cudaGetLastError();
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  if (p.block_size > 1) {
    const int nblk = (p.keys + p.block_size - 1) / p.block_size;
    const int64_t warps = rows * nblk;
    const unsigned g = static_cast<unsigned>(std::min<int64_t>((warps + 7) / 8, sm_count() * 32));
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
