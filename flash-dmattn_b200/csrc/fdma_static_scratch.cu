// fdma_fwd_static_scratch: the forward pass for hosts that cannot hand the library a scratch buffer.
//
// fdma_fwd needs caller-provided scratch in two cases: when the mask differs per query row (one activity byte per
// 128x128 tile, written by a small pre-kernel and read by the attention kernel), and for single-query (decode) calls
// (per-split partial results that a merge kernel combines). Some hosts have no way to provide it at call
// time: an engine whose device memory is carved up once at start-up and that exposes no allocator to its
// operators, or a latency-critical loop in which cudaMalloc (which may synchronise the whole device) is off
// limits. For them this entry point keeps the scratch in a fixed array that is part of the library image.
//
// Properties a caller has to know
//  * Limit: kStaticScratchBytes (1 MiB) of scratch, compared with fdma_fwd_workspace_bytes(p): for a per-query mask
//    B * h_mask * ceil(Sq/128) * ceil(Sk/128) activity bytes; for a single-query call the decode partials
//    B * H * splits * 8 * (d + 2) * 4 bytes. Larger problems are refused with FDMA_ERR_TOO_LARGE before anything is
//    launched.
//  * Cost: every GPU on which the library is loaded holds this 1 MiB until the process exits.
//  * The first call on each device looks up the array's device address (one cudaGetSymbolAddress); make that first
//    call outside any stream capture. No call allocates or frees memory.
//  * All calls on a device share the one array, and it keeps whatever the previous call left in it. Every byte a
//    call later reads it has written itself first (the activity pre-kernel covers all tiles, every decode warp
//    writes its own partial), so nothing needs clearing between calls -- but two calls
//    whose GPU work overlaps (different streams, or different host threads) race on it. Serialise them.
#include <cuda_runtime.h>

#include <mutex>

#include "fdma_internal.h"

namespace {

constexpr size_t kStaticScratchBytes = 1u << 20;
constexpr int kMaxDevices = 64;

// The scratch itself. In host code this name is only a handle for cudaGetSymbolAddress, never a usable pointer.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

std::mutex g_setup_mutex;
void* g_scratch_ptr[kMaxDevices] = {nullptr};

// Device address of g_static_scratch on the CURRENT device, resolved once per device.
int scratch_for_current_device(void** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 0 || dev >= kMaxDevices) return FDMA_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (!g_scratch_ptr[dev]) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (e != cudaSuccess) return static_cast<int>(e);
    g_scratch_ptr[dev] = ptr;
  }
  *out = g_scratch_ptr[dev];
  return 0;
}

}  // namespace

extern "C" {

size_t fdma_static_scratch_limit(void) { return kStaticScratchBytes; }

int fdma_fwd_static_scratch(const fdma_fwd_params* p, void* stream) {
  if (!p) return FDMA_ERR_BAD_ARG;
  fdma_fwd_params q = *p;
  q.workspace = nullptr;
  q.workspace_bytes = 0;
  const size_t need = fdma_fwd_workspace_bytes(&q);  // 0 also when the arguments are invalid: fdma_fwd reports that
  if (need > kStaticScratchBytes) return FDMA_ERR_TOO_LARGE;
  if (need > 0) {
    void* ptr = nullptr;
    const int st = scratch_for_current_device(&ptr);
    if (st) return st;
    q.workspace = ptr;
    q.workspace_bytes = kStaticScratchBytes;
  }
  return fdma_fwd(&q, stream);
}

}  // extern "C"
