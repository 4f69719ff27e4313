// extern "C" entry points of libfdma_sm100.so: argument validation, kernel-family selection and the
// error-code conventions declared in include/fdma.h. Host-side counterpart of the reference's
// mha_fwd / mha_bwd (csrc/flash_sparse_attn/flash_api.cpp:351-554, :792-1050), minus tensor
// allocation, which stays with the caller.
#include <cuda.h>
#include <cuda_runtime.h>

#include <mutex>

#include "fdma_internal.h"

namespace fdma {

namespace {

// Per-device status block: [0] the code of the first bounded wait that gave up (0 = none), [2..3] the address of a
// page-locked host int that mirrors it (so the host can poll without synchronising).
__device__ __align__(16) int g_kernel_status[4] = {0, 0, 0, 0};
std::mutex g_status_mutex;
int* g_status_ptr[64] = {nullptr};
volatile int* g_status_host[64] = {nullptr};

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn g_encode = nullptr;
std::once_flag g_encode_once;

void load_encode() {
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) == cudaSuccess &&
      qres == cudaDriverEntryPointSuccess) {
    g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  }
}

int check_arch() {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  int major = 0;
  e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  return major == 10 ? 0 : FDMA_ERR_ARCH;
}

int validate_fwd(const fdma_fwd_params& p) {
  if (!p.q || !p.k || !p.v || !p.out || !p.lse) return FDMA_ERR_BAD_ARG;
  if (p.b <= 0 || p.seqlen_q <= 0 || p.seqlen_k < 0 || p.h <= 0 || p.h_k <= 0 || p.d <= 0) return FDMA_ERR_BAD_ARG;
  if (p.h % p.h_k != 0) return FDMA_ERR_BAD_ARG;
  if (p.d > 256 || p.d % 8 != 0) return FDMA_ERR_UNSUPPORTED;
  if (p.dtype != FDMA_BF16 && p.dtype != FDMA_FP16) return FDMA_ERR_UNSUPPORTED;
  if (p.mask && !(p.h_mask == 1 || p.h_mask == p.h_k || p.h_mask == p.h)) return FDMA_ERR_BAD_ARG;
  if (p.bias && !(p.h_bias == 1 || p.h_bias == p.h_k || p.h_bias == p.h)) return FDMA_ERR_BAD_ARG;
  if (p.key_pos && !(p.h_pos == 1 || p.h_pos == p.h_k || p.h_pos == p.h)) return FDMA_ERR_BAD_ARG;
  return 0;
}

int validate_bwd(const fdma_bwd_params& p) {
  int st = validate_fwd(p.f);
  if (st) return st;
  if (!p.dout || !p.dq || !p.dk || !p.dv) return FDMA_ERR_BAD_ARG;
  if (p.dbias) {
    if (!p.f.bias) return FDMA_ERR_BAD_ARG;
    if (p.dbias_b <= 0 || p.dbias_h <= 0 || p.dbias_rows <= 0 || p.dbias_keys < p.f.seqlen_k) return FDMA_ERR_BAD_ARG;
    if (!(p.dbias_b == 1 || p.dbias_b == p.f.b)) return FDMA_ERR_BAD_ARG;
    if (!(p.dbias_h == 1 || p.dbias_h == p.f.h_k || p.dbias_h == p.f.h)) return FDMA_ERR_BAD_ARG;
    if (!(p.dbias_rows == 1 || p.dbias_rows == p.f.seqlen_q)) return FDMA_ERR_BAD_ARG;
  }
  return 0;
}

// Normalised copy: absent mask/bias get head count 1 so head-ratio arithmetic never divides by zero, and
// causal is dropped for single-query calls (flash_api.cpp:441).
fdma_fwd_params normalise(const fdma_fwd_params& in) {
  fdma_fwd_params p = in;
  if (!p.mask) p.h_mask = 1;
  if (!p.mask) p.mask_bits = 0;
  if (!p.bias) p.h_bias = 1;
  if (p.seqlen_q == 1) p.is_causal = 0;
  if (!p.key_pos || !p.is_causal) {
    p.key_pos = nullptr;
    p.h_pos = 1;
  }
  return p;
}

}  // namespace

int encode_tmap_4d(void* out_map, const void* base, int elem_bytes, const uint64_t dims[4],
                   const uint64_t strides_bytes[3], const uint32_t box[4]) {
  std::call_once(g_encode_once, load_encode);
  if (!g_encode) return FDMA_ERR_DRIVER;
  cuuint64_t gdims[4] = {dims[0], dims[1], dims[2], dims[3]};
  cuuint64_t gstr[3] = {strides_bytes[0], strides_bytes[1], strides_bytes[2]};
  cuuint32_t bx[4] = {box[0], box[1], box[2], box[3]};
  cuuint32_t es[4] = {1, 1, 1, 1};
  auto encode = [&]() {
    return g_encode(static_cast<CUtensorMap*>(out_map),
                    elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4,
                    const_cast<void*>(base), gdims, gstr, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  };
  CUresult r = encode();
  if (r == CUDA_ERROR_INVALID_CONTEXT) {
    // The encode call is the driver API and wants a context current on THIS thread. A thread that has only been
    // handed cached device memory so far (an autograd worker running its first backward) has none: a runtime call
    // binds the device's primary context, then the encode goes through.
    (void)cudaFree(nullptr);
    r = encode();
  }
  return r == CUDA_SUCCESS ? 0 : FDMA_ERR_DRIVER;
}

namespace {
thread_local cudaEvent_t t_ev_start = nullptr;
thread_local cudaEvent_t t_ev_stop = nullptr;
}  // namespace

void take_timing_events(cudaEvent_t* start, cudaEvent_t* stop) {
  *start = t_ev_start;
  *stop = t_ev_stop;
  t_ev_start = nullptr;
  t_ev_stop = nullptr;
}

int* kernel_status_ptr() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(g_status_mutex);
  if (!g_status_ptr[dev]) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_kernel_status) != cudaSuccess) return nullptr;
    // Host mirror: 4 bytes of mapped page-locked memory per device (host memory, allocated once). If it cannot be
    // had, the mirror stays off and only fdma_last_kernel_status sees a timeout.
    int* host = nullptr;
    void* host_dev = nullptr;
    if (cudaHostAlloc(reinterpret_cast<void**>(&host), sizeof(int), cudaHostAllocMapped | cudaHostAllocPortable) ==
            cudaSuccess &&
        cudaHostGetDevicePointer(&host_dev, host, 0) == cudaSuccess) {
      *host = 0;
      if (cudaMemcpy(static_cast<int*>(ptr) + 2, &host_dev, sizeof(void*), cudaMemcpyHostToDevice) == cudaSuccess)
        g_status_host[dev] = host;
    } else {
      (void)cudaGetLastError();
    }
    g_status_ptr[dev] = static_cast<int*>(ptr);
  }
  return g_status_ptr[dev];
}

int export_softmax_d(const fdma_bwd_params& bp, const float* dsum, int sq_r, cudaStream_t stream) {
  if (!bp.softmax_d) return 0;
  const fdma_fwd_params& p = bp.f;
  const size_t rows = static_cast<size_t>(p.b) * p.h;
  const size_t r128 = static_cast<size_t>(round_up(p.seqlen_q, 128));
  cudaError_t e = cudaSuccess;
  if (r128 > static_cast<size_t>(p.seqlen_q)) e = cudaMemsetAsync(bp.softmax_d, 0, rows * r128 * sizeof(float), stream);
  if (e != cudaSuccess) return static_cast<int>(e);
  e = cudaMemcpy2DAsync(bp.softmax_d, r128 * sizeof(float), dsum, static_cast<size_t>(sq_r) * sizeof(float),
                        static_cast<size_t>(p.seqlen_q) * sizeof(float), rows, cudaMemcpyDeviceToDevice, stream);
  return static_cast<int>(e);
}

int sm_count() {
  static std::mutex mu;
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  std::lock_guard<std::mutex> lock(mu);
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

}  // namespace fdma

using namespace fdma;

extern "C" {

int fdma_version(void) { return FDMA_VERSION; }

const char* fdma_strerror(int status) {
  switch (status) {
    case FDMA_OK: return "success";
    case FDMA_ERR_BAD_ARG: return "fdma: invalid argument (null pointer, bad size or inconsistent head counts)";
    case FDMA_ERR_UNSUPPORTED: return "fdma: unsupported shape, dtype or kernel path for these arguments";
    case FDMA_ERR_WORKSPACE: return "fdma: workspace missing or smaller than *_workspace_bytes()";
    case FDMA_ERR_ARCH: return "fdma: device is not compute capability 10.x (sm_100a required)";
    case FDMA_ERR_DRIVER: return "fdma: cuTensorMapEncodeTiled unavailable or rejected the tensor map";
    case FDMA_ERR_TIMEOUT: return "fdma: a bounded in-kernel wait timed out";
    case FDMA_ERR_TOO_LARGE: return "fdma: problem exceeds the static scratch limit of this entry point";
    default: break;
  }
  if (status > 0) return cudaGetErrorString(static_cast<cudaError_t>(status));
  return "fdma: unknown status";
}

size_t fdma_fwd_workspace_bytes(const fdma_fwd_params* pp) {
  if (!pp || validate_fwd(*pp)) return 0;
  const fdma_fwd_params p = normalise(*pp);
  if ((p.path == FDMA_PATH_AUTO || p.path == FDMA_PATH_DECODE) && decode_supported(p)) return decode_workspace_bytes(p);
  if (p.path != FDMA_PATH_SIMT && p.path != FDMA_PATH_DECODE && tc_fwd_supported(p)) return tc_fwd_workspace_bytes(p);
  return 0;
}

int fdma_fwd(const fdma_fwd_params* pp, void* stream_) {
  if (!pp) return FDMA_ERR_BAD_ARG;
  int st = validate_fwd(*pp);
  if (st) return st;
  st = check_arch();
  if (st) return st;
  const fdma_fwd_params p = normalise(*pp);
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (p.path == FDMA_PATH_AUTO || p.path == FDMA_PATH_DECODE) {
    if (decode_supported(p) && !(p.mask && p.mask_bits)) return decode_fwd(p, stream);
    if (p.path == FDMA_PATH_DECODE) return FDMA_ERR_UNSUPPORTED;
  }
  const bool tc_ok = tc_fwd_supported(p);
  if (p.path == FDMA_PATH_TCGEN05 && !tc_ok) return FDMA_ERR_UNSUPPORTED;
  if (p.path != FDMA_PATH_SIMT && tc_ok) return tc_fwd(p, stream);
  if (p.mask && p.mask_bits) return FDMA_ERR_UNSUPPORTED;  // only the tcgen05 kernels read a bit-packed mask
  return simt_fwd(p, stream);
}

size_t fdma_bwd_workspace_bytes(const fdma_bwd_params* pp) {
  if (!pp || validate_bwd(*pp)) return 0;
  fdma_bwd_params p = *pp;
  p.f = normalise(pp->f);
  if (p.f.path != FDMA_PATH_SIMT && tc_bwd_supported(p)) return tc_bwd_workspace_bytes(p);
  return simt_bwd_workspace_bytes(p);
}

int fdma_bwd(const fdma_bwd_params* pp, void* stream_) {
  if (!pp) return FDMA_ERR_BAD_ARG;
  int st = validate_bwd(*pp);
  if (st) return st;
  st = check_arch();
  if (st) return st;
  fdma_bwd_params p = *pp;
  p.f = normalise(pp->f);
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const bool tc_ok = tc_bwd_supported(p);
  if (p.f.path == FDMA_PATH_TCGEN05 && !tc_ok) return FDMA_ERR_UNSUPPORTED;
  if (p.f.path != FDMA_PATH_SIMT && tc_ok) return tc_bwd(p, stream);
  if (p.f.mask && p.f.mask_bits) return FDMA_ERR_UNSUPPORTED;  // only the tcgen05 kernels read a bit-packed mask
  return simt_bwd(p, stream);
}

int fdma_create_mask(const fdma_mask_params* p, void* stream_) {
  if (!p || !p->bias || (!p->out && !p->key_pos && !p->bits)) return FDMA_ERR_BAD_ARG;
  if (p->out_b < 0 || p->out_h < 0 || p->out_rows < 0 || p->keys < 0) return FDMA_ERR_BAD_ARG;
  if (p->kind != FDMA_MASK_TOPK && p->kind != FDMA_MASK_RELU) return FDMA_ERR_BAD_ARG;
  if (p->key_pos) {  // position output: top-k selection without block smoothing, every selection must fit
    if (!p->count || p->capacity <= 0) return FDMA_ERR_BAD_ARG;
    if (p->kind != FDMA_MASK_TOPK || p->block_size > 1) return FDMA_ERR_UNSUPPORTED;
    if (p->window <= 0 || p->capacity < (p->window < p->keys ? p->window : p->keys)) return FDMA_ERR_BAD_ARG;
  }
  if (p->bits) {  // bit-packed output: top-k selection without block smoothing, with its tile activity
    if (!p->activity) return FDMA_ERR_BAD_ARG;
    if (p->kind != FDMA_MASK_TOPK || p->block_size > 1 || p->window <= 0 || p->key_pos) return FDMA_ERR_UNSUPPORTED;
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (p->kind == FDMA_MASK_TOPK && p->window <= 0) {
    const size_t n = static_cast<size_t>(p->out_b) * p->out_h * p->out_rows * p->keys;
    return n ? static_cast<int>(cudaMemsetAsync(p->out, 0, n, stream)) : 0;
  }
  return create_mask(*p, stream);
}

void fdma_time_next_kernel(void* start_event, void* stop_event) {
  t_ev_start = static_cast<cudaEvent_t>(start_event);
  t_ev_stop = static_cast<cudaEvent_t>(stop_event);
}

int fdma_poll_kernel_status(int32_t* detail) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  volatile int* host = g_status_host[dev];
  const int v = host ? *host : 0;
  if (detail) *detail = v;
  return v != 0 ? FDMA_ERR_TIMEOUT : 0;
}

int fdma_last_kernel_status(void* stream_, int32_t* detail) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  int v = 0;
  cudaError_t e = cudaMemcpyFromSymbolAsync(&v, g_kernel_status, sizeof(int), 0, cudaMemcpyDeviceToHost, stream);
  if (e != cudaSuccess) return static_cast<int>(e);
  e = cudaStreamSynchronize(stream);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (detail) *detail = v;
  if (v != 0) {
    const int zero = 0;
    e = cudaMemcpyToSymbolAsync(g_kernel_status, &zero, sizeof(int), 0, cudaMemcpyHostToDevice, stream);
    if (e != cudaSuccess) return static_cast<int>(e);
    e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) return static_cast<int>(e);
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < 64 && g_status_host[dev]) *g_status_host[dev] = 0;
    return FDMA_ERR_TIMEOUT;
  }
  return 0;
}

}  // extern "C"
