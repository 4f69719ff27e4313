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
  int heads_per_cta;  // query heads that share one pass over the rows (decode_mma_kernel reads it at run time)
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

// ---- pipelined tensor-core variant: head dim 64 / 128, up to 8 query heads per kv head ----------------------------
// Same scan / queue / partial scheme as decode_kernel, with two changes that matter when the kernel is bound by the
// latency of scattered row reads and by instruction issue:
//  * rows travel global -> shared memory with cp.async into a ring of batches (8 K rows + 8 V rows) per warp, so the
//    next batch is in flight (holding no registers) while the current one is computed;
//  * the G query heads that share the rows are the M rows of mma.sync.m16n8k16 (rows >= G are zero): S = Q K^T and
//    O += P V of a batch take 4 + 4 ldmatrix and 8 + 16 mma per 8 keys instead of per-lane dot products, a cross-lane
//    butterfly and per-lane value accumulation (which cost about 110 instructions per key). Shared-memory rows are
//    padded by 16 bytes so that the eight rows of an ldmatrix tile fall into different banks.
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(smem))),
               "l"(gmem)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

template <int D>
struct MmaSmem {
  static constexpr int kRows = 8;
  static constexpr int kRowBytes = D * 2 + 16;
  static constexpr int kStageBytes = 2 * kRows * kRowBytes;  // K rows then V rows
  static constexpr int kStages = 2;                          // row batches per warp: one computed, one in flight (3: slower)
  static constexpr int kWarpBytes = kStages * kStageBytes;
  static constexpr int kTotal = kWarps * kWarpBytes;
};
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
// Rows 8-15 of every product here are zero (A rows 8-15 are zero), so all accumulators share one pair of registers
// (z0, z1) for them.
template <bool kBf16>
__device__ __forceinline__ void mma_16816(float& c0, float& c1, float& z0, float& z1, uint32_t a0, uint32_t a2,
                                          uint32_t b0, uint32_t b1) {
  if (kBf16)
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%5}, {%7,%8}, {%0,%1,%2,%3};"
                 : "+f"(c0), "+f"(c1), "+f"(z0), "+f"(z1) : "r"(a0), "r"(0u), "r"(a2), "r"(b0), "r"(b1));
  else
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%5}, {%7,%8}, {%0,%1,%2,%3};"
                 : "+f"(c0), "+f"(c1), "+f"(z0), "+f"(z1) : "r"(a0), "r"(0u), "r"(a2), "r"(b0), "r"(b1));
}
template <bool kBf16>
__device__ __forceinline__ uint32_t pack_pair(float lo, float hi) {
  if (kBf16) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
  }
  const __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

template <int D, bool kBf16>
__global__ void __launch_bounds__(kThreads, 2) decode_mma_kernel(const DecodeParams p) {
  using L = MmaSmem<D>;
  constexpr int R = L::kRows;
  const int G = p.heads_per_cta;                            // 1, 2, 4 or 8 query heads share the rows
  constexpr int kChunksPerRow = D / 8;                      // 16-byte pieces of a row
  constexpr int kRowsPerCopy = 32 / kChunksPerRow;          // rows covered by one warp-wide cp.async
  extern __shared__ __align__(16) unsigned char s_rows[];
  __shared__ int s_queue[kWarps][kQueue];
  __shared__ float s_qbias[kWarps][kQueue];
  __shared__ float s_pbias[kWarps][L::kStages][R];         // bias of the rows of each stage
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int split = blockIdx.x, b = blockIdx.z;
  const int h0 = blockIdx.y * G;
  const int hk = h0 / p.group;
  const int hm = p.h_mask == p.h ? h0 : (p.h_mask == p.h_k ? hk : 0);
  const int hb = p.h_bias == p.h ? h0 : (p.h_bias == p.h_k ? hk : 0);
  const uint8_t* mrow = p.mask ? p.mask + b * p.mask_batch_stride + hm * p.mask_head_stride : nullptr;
  const uint16_t* brow = p.bias ? reinterpret_cast<const uint16_t*>(p.bias) + b * p.bias_batch_stride + hb * p.bias_head_stride
                                : nullptr;
  const uint16_t* kbase = reinterpret_cast<const uint16_t*>(p.k) + b * p.k_batch_stride + hk * p.k_head_stride;
  const uint16_t* vbase = reinterpret_cast<const uint16_t*>(p.v) + b * p.v_batch_stride + hk * p.v_head_stride;
  unsigned char* my_rows = s_rows + warp * L::kWarpBytes;

  // Fragments of mma.sync.m16n8k16 (row.col): the M = 16 rows are the query heads (rows >= G are zero), so a
  // lane's quad index g = lane >> 2 is its head and lanes of quads >= G carry zeros.
  //   A: a0 = (row g, k = 2c, 2c+1), a2 = (row g, k + 8), a1 / a3 = rows g + 8 (always zero here)   [c = lane & 3]
  //   B: b0 = (k = 2c, 2c+1; n = g), b1 = (k + 8; n = g)
  //   C: c0, c1 = (row g, n = 2c, 2c+1), c2, c3 = rows g + 8 (unused)
  const int quad = lane >> 2, c2 = (lane & 3) * 2;
  uint32_t qa[D / 16][2];
  {
    const uint16_t* qp = reinterpret_cast<const uint16_t*>(p.q) + b * p.q_batch_stride + (h0 + min(quad, G - 1)) * p.q_head_stride;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      qa[ks][0] = quad < G ? *reinterpret_cast<const uint32_t*>(qp + ks * 16 + c2) : 0u;
      qa[ks][1] = quad < G ? *reinterpret_cast<const uint32_t*>(qp + ks * 16 + 8 + c2) : 0u;
    }
  }
  float o[D / 8][2];                                         // O[head g][d = nt * 8 + 2c, +1]
#pragma unroll
  for (int nt = 0; nt < D / 8; ++nt) o[nt][0] = o[nt][1] = 0.f;
  float z0 = 0.f, z1 = 0.f;                                  // rows 8-15 of every accumulator: always zero
  float my_m = -CUDART_INF_F, my_l = 0.f;                   // running max / sum of head g (same in the quad's lanes)

  // queue entries [first, first + n) -> stage: start the row copies, remember the rows' biases
  auto issue = [&](int first, int n, int stage) {
    unsigned char* dst = my_rows + stage * L::kStageBytes;
    const int sub = lane / kChunksPerRow, chunk = lane % kChunksPerRow;
#pragma unroll
    for (int r0 = 0; r0 < R; r0 += kRowsPerCopy) {
      const int t = r0 + sub;
      if (t < R) {
        const int64_t key = s_queue[warp][first + min(t, n - 1)];
        cp_async16(dst + t * L::kRowBytes + chunk * 16, kbase + key * p.k_row_stride + chunk * 8);
        cp_async16(dst + (R + t) * L::kRowBytes + chunk * 16, vbase + key * p.v_row_stride + chunk * 8);
      }
    }
    cp_async_commit();
    if (lane < R) s_pbias[warp][stage][lane] = lane < n ? s_qbias[warp][first + lane] : -CUDART_INF_F;
  };

  // the rows of `stage` have landed: S = Q K^T on the tensor cores (rows = heads, columns = the 8 keys), online
  // softmax on the accumulator fragment, which is also the A fragment of O += P V (keys 8-15 of its k = 16 are zero)
  auto consume = [&](int stage) {
    __syncwarp();
    const uint32_t kaddr = static_cast<uint32_t>(__cvta_generic_to_shared(my_rows + stage * L::kStageBytes)) +
                           (lane & 7) * L::kRowBytes + (lane >> 3) * 16;
    const uint32_t vaddr = kaddr + R * L::kRowBytes;
    float s0 = 0.f, s1 = 0.f;
#pragma unroll
    for (int ks2 = 0; ks2 < D / 32; ++ks2) {  // one ldmatrix.x4 = the B fragments of two k-steps
      uint32_t bf[4];
      ldmatrix_x4(bf, kaddr + ks2 * 64);
      mma_16816<kBf16>(s0, s1, z0, z1, qa[2 * ks2][0], qa[2 * ks2][1], bf[0], bf[1]);
      mma_16816<kBf16>(s0, s1, z0, z1, qa[2 * ks2 + 1][0], qa[2 * ks2 + 1][1], bf[2], bf[3]);
    }
    const float sc0 = fmaf(s0, p.scale_log2, s_pbias[warp][stage][c2]);      // -inf for padding rows
    const float sc1 = fmaf(s1, p.scale_log2, s_pbias[warp][stage][c2 + 1]);
    float mx = fmaxf(sc0, sc1);
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float m_new = fmaxf(my_m, mx);
    const float p0 = m_new == -CUDART_INF_F ? 0.f : exp2f(sc0 - m_new);
    const float p1 = m_new == -CUDART_INF_F ? 0.f : exp2f(sc1 - m_new);
    const float corr = my_m == -CUDART_INF_F ? 0.f : exp2f(my_m - m_new);
    float psum = p0 + p1;
    psum += __shfl_xor_sync(0xffffffffu, psum, 1);
    psum += __shfl_xor_sync(0xffffffffu, psum, 2);
    my_l = my_l * corr + psum;
    my_m = m_new;
    const uint32_t pa = pack_pair<kBf16>(p0, p1);
#pragma unroll
    for (int nt = 0; nt < D / 8; ++nt) {
      o[nt][0] *= corr;
      o[nt][1] *= corr;
    }
#pragma unroll
    for (int nt4 = 0; nt4 < D / 32; ++nt4) {  // one transposed ldmatrix.x4 = the B fragments of four d-tiles
      uint32_t bf[4];
      ldmatrix_x4_trans(bf, vaddr + nt4 * 64);
#pragma unroll
      for (int j = 0; j < 4; ++j) mma_16816<kBf16>(o[nt4 * 4 + j][0], o[nt4 * 4 + j][1], z0, z1, pa, 0u, bf[j], 0u);
    }
    __syncwarp();
  };

  // Scan in pieces of 512 keys per warp: every lane fetches the 16 mask bytes and 16 biases of 16 consecutive keys
  // with three independent vector loads, then the warp walks the 16 byte positions without touching global memory
  // (position j of all lanes forms one 32-key group; the order in which kept keys are queued does not matter).
  // The loop below has ONE copy of the scan step and ONE of issue / consume: with the phases of a warp's life
  // sharing code, the warps of an SM partition stay inside the instruction cache.
  constexpr int kPiece = 512;
  const int pieces_total = (p.seqlen_k + kPiece - 1) / kPiece;
  const int pieces_per_split = (pieces_total + p.nsplit - 1) / p.nsplit;
  const int c_end = min(pieces_total, (split + 1) * pieces_per_split);
  int c = split * pieces_per_split + warp;  // next piece of this warp
  int left = 0, gi = 0, base = 0;           // 32-key groups left in the loaded piece, index of the current one
  uint32_t mw[4] = {0u, 0u, 0u, 0u};        // mw[0] / bw[0..1] always hold the word the current group is in
  uint32_t bw[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
  int head = 0, qn = 0;                     // queue entries [head, qn) wait for their batch
  int pend = 0, st_w = 0, st_r = 0;         // batches in flight, stage to fill next, stage to compute next
  for (;;) {
    while (qn - head < R && (left > 0 || c < c_end)) {
      if (left == 0) {
        base = c * kPiece + lane * 16;
        c += kWarps;
        left = 16;
        gi = 0;
        if (base + 16 <= p.seqlen_k) {
          mw[0] = mw[1] = mw[2] = mw[3] = 0x01010101u;
          if (mrow) {
            const uint4 mv = *reinterpret_cast<const uint4*>(mrow + base);
            mw[0] = mv.x; mw[1] = mv.y; mw[2] = mv.z; mw[3] = mv.w;
          }
          if (brow) {
            const uint4 b0 = *reinterpret_cast<const uint4*>(brow + base);
            const uint4 b1 = *reinterpret_cast<const uint4*>(brow + base + 8);
            bw[0] = b0.x; bw[1] = b0.y; bw[2] = b0.z; bw[3] = b0.w;
            bw[4] = b1.x; bw[5] = b1.y; bw[6] = b1.z; bw[7] = b1.w;
          }
        } else {  // ragged end of the row: byte by byte, keys beyond the end count as masked
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int key = base + j;
            uint32_t mbyte = 0u, bhalf = 0u;
            if (key < p.seqlen_k) {
              mbyte = mrow ? (mrow[key] != 0 ? 1u : 0u) : 1u;
              if (brow) bhalf = brow[key];
            }
            mw[j >> 2] = (mw[j >> 2] & ~(0xFFu << ((j & 3) * 8))) | (mbyte << ((j & 3) * 8));
            bw[j >> 1] = (bw[j >> 1] & ~(0xFFFFu << ((j & 1) * 16))) | (bhalf << ((j & 1) * 16));
          }
        }
      }
      int adv = 1;
      if ((gi & 3) == 0 && __ballot_sync(0xffffffffu, mw[0] != 0u) == 0u) {
        adv = 4;  // 128 keys without a kept one
      } else {
        const int i = gi & 3;
        const bool keep = ((mw[0] >> (8 * i)) & 0xFFu) != 0u;
        const uint32_t bits = __ballot_sync(0xffffffffu, keep);
        if (bits != 0u) {
          if (qn > kQueue - 32) {  // make room: move the waiting entries (fewer than one batch) to the front
            const int rest = qn - head;
            int kk = 0;
            float bb = 0.f;
            if (lane < rest) {
              kk = s_queue[warp][head + lane];
              bb = s_qbias[warp][head + lane];
            }
            __syncwarp();
            if (lane < rest) {
              s_queue[warp][lane] = kk;
              s_qbias[warp][lane] = bb;
            }
            head = 0;
            qn = rest;
          }
          if (keep) {
            const int pos = qn + __popc(bits & ((1u << lane) - 1u));
            const uint32_t bpair = (i & 2) ? bw[1] : bw[0];
            const uint16_t braw = static_cast<uint16_t>((i & 1) ? (bpair >> 16) : (bpair & 0xFFFFu));
            s_queue[warp][pos] = base + gi;
            s_qbias[warp][pos] = brow ? raw_to_f<kBf16>(braw) * 1.4426950408889634f : 0.f;
          }
          qn += __popc(bits);
          __syncwarp();
        }
      }
      gi += adv;
      left -= adv;
      if ((gi & 3) == 0) {  // next word of the piece moves into place
        mw[0] = mw[1]; mw[1] = mw[2]; mw[2] = mw[3];
        bw[0] = bw[2]; bw[1] = bw[3]; bw[2] = bw[4]; bw[3] = bw[5]; bw[4] = bw[6]; bw[5] = bw[7];
      }
    }
    // one batch goes out; once every stage is taken (or nothing is left to send) the oldest batch is computed
    // while the newer ones load
    const int n = min(R, qn - head);
    if (n > 0) {
      issue(head, n, st_w);
      head += n;
      st_w = st_w + 1 == L::kStages ? 0 : st_w + 1;
      ++pend;
    }
    if (pend == L::kStages || (n == 0 && pend > 0)) {
      static_assert(L::kStages <= 3, "add a wait for deeper rings");
      if (pend >= 3) cp_async_wait<2>();  // all but the newest (pend - 1) groups have landed
      else if (pend == 2) cp_async_wait<1>();
      else cp_async_wait<0>();
      consume(st_r);
      st_r = st_r + 1 == L::kStages ? 0 : st_r + 1;
      --pend;
    }
    if (n == 0 && pend == 0) break;
  }

  // one partial per warp and head: the quad of head g holds O[g][:] (two floats per d-tile and lane), m and l
  const int P = p.nsplit * kWarps;
  if (quad < G) {
    float* dst = p.partial + ((static_cast<int64_t>(b) * p.h + h0 + quad) * P + split * kWarps + warp) * (D + 2);
#pragma unroll
    for (int nt = 0; nt < D / 8; ++nt) *reinterpret_cast<float2*>(dst + nt * 8 + c2) = make_float2(o[nt][0], o[nt][1]);
    if ((lane & 3) == 0) {
      dst[D] = my_m;
      dst[D + 1] = my_l;
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
  // Two CTAs are resident per SM and all CTAs of a launch take about the same time, so the launch lasts
  // ceil(splits * ctas_per_split / slots) rounds of 1 / splits of the work each: pick the split count with the
  // smallest product (a small charge per split covers the extra partials). Every split keeps at least four
  // 512-key pieces per warp... unless the row is shorter than that.
  const int slots = sm_count() * 2;
  const int max_by_len = std::max(1, (p.seqlen_k + 512 * kWarps * 4 - 1) / (512 * kWarps * 4));
  const int limit = std::min(max_by_len, 32);
  int best = 1;
  double best_cost = 1e30;
  for (int ns = 1; ns <= limit; ++ns) {
    const int64_t ctas = static_cast<int64_t>(ns) * std::max(1, ctas_per_split);
    const double rounds = static_cast<double>((ctas + slots - 1) / slots);
    const double cost = rounds / ns + 0.01 * ns;
    if (cost < best_cost) {
      best_cost = cost;
      best = ns;
    }
  }
  return best;
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

// cp.async moves 16-byte pieces: K / V bases and row strides must keep rows 16-byte aligned
bool pipe_ok(const DecodeParams& dp) {
  auto a16 = [](const void* x) { return (reinterpret_cast<uintptr_t>(x) & 15u) == 0; };
  const int64_t strides[6] = {dp.k_batch_stride, dp.k_row_stride, dp.k_head_stride,
                              dp.v_batch_stride, dp.v_row_stride, dp.v_head_stride};
  for (int64_t s : strides)
    if (s % 8) return false;
  // the scan reads 16 mask bytes and 16 biases per lane with 16-byte loads
  if (dp.mask && (!a16(dp.mask) || dp.mask_batch_stride % 16 || dp.mask_head_stride % 16)) return false;
  if (dp.bias && (!a16(dp.bias) || dp.bias_batch_stride % 8 || dp.bias_head_stride % 8)) return false;
  return a16(dp.k) && a16(dp.v);
}

template <int D, bool kBf16>
int launch_mma(const DecodeParams& dp, dim3 grid, cudaStream_t stream) {
  using L = MmaSmem<D>;
  auto kern = decode_mma_kernel<D, kBf16>;
  const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal);
  if (e != cudaSuccess) return static_cast<int>(e);
  kern<<<grid, kThreads, L::kTotal, stream>>>(dp);
  return static_cast<int>(cudaGetLastError());
}

// the A fragments are read from Q with 32-bit loads
bool mma_ok(const DecodeParams& dp) {
  return pipe_ok(dp) && (reinterpret_cast<uintptr_t>(dp.q) & 3u) == 0 && dp.q_batch_stride % 2 == 0 &&
         dp.q_head_stride % 2 == 0;
}

template <int EPL, bool kBf16>
int launch_epl(const DecodeParams& dp, int G, dim3 grid, cudaStream_t stream) {
  if (EPL <= 4 && G <= 8 && mma_ok(dp)) return launch_mma<(EPL <= 4 ? 32 * EPL : 128), kBf16>(dp, grid, stream);
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
  dp.group = p.h / p.h_k; dp.nsplit = ns; dp.heads_per_cta = G;
  dp.scale_log2 = p.softmax_scale * 1.4426950408889634f;
  dim3 grid(ns, p.h / G, p.b);
  const bool bf = p.dtype == FDMA_BF16;
  cudaEvent_t ev0, ev1;
  take_timing_events(&ev0, &ev1);
  if (ev0) cudaEventRecord(ev0, stream);
  int st;
  if (p.d == 64) st = bf ? launch_epl<2, true>(dp, G, grid, stream) : launch_epl<2, false>(dp, G, grid, stream);
  else if (p.d == 128) st = bf ? launch_epl<4, true>(dp, G, grid, stream) : launch_epl<4, false>(dp, G, grid, stream);
  else st = bf ? launch_epl<8, true>(dp, G, grid, stream) : launch_epl<8, false>(dp, G, grid, stream);
  if (ev1) cudaEventRecord(ev1, stream);
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
