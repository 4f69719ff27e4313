// Internal declarations shared by the translation units of libfdma_sm100.so.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/fdma.h"

namespace fdma {

constexpr int kKeyPad = 128;  // mask/bias rows are readable up to round_up(Sk, kKeyPad) keys

inline int64_t round_up(int64_t x, int64_t m) { return (x + m - 1) / m * m; }
inline size_t align256(size_t x) { return (x + 255) & ~static_cast<size_t>(255); }

// ---- CUDA-core ("SIMT") kernels: any head dim <= 256 that is a multiple of 8 -------------------
size_t simt_bwd_workspace_bytes(const fdma_bwd_params& p);
int simt_fwd(const fdma_fwd_params& p, cudaStream_t stream);
int simt_bwd(const fdma_bwd_params& p, cudaStream_t stream);

// ---- tcgen05 / TMA kernels ---------------------------------------------------------------------
bool tc_fwd_supported(const fdma_fwd_params& p);
size_t tc_fwd_workspace_bytes(const fdma_fwd_params& p);
int tc_fwd(const fdma_fwd_params& p, cudaStream_t stream);

// Per-tile mask activity map for per-query masks: act[b][h_mask][ceil(Sq/128)][ceil(Sk/128)] bytes.
int launch_tile_activity(const fdma_fwd_params& p, uint8_t* act, cudaStream_t stream);

// head dim 256, row-broadcast mask / bias (fdma_bwd256_sm100.cu); reached through the three tc_bwd entry points
bool tc_bwd256_supported(const fdma_bwd_params& p);
size_t tc_bwd256_workspace_bytes(const fdma_bwd_params& p);
int tc_bwd256(const fdma_bwd_params& p, cudaStream_t stream);

bool tc_bwd_supported(const fdma_bwd_params& p);
size_t tc_bwd_workspace_bytes(const fdma_bwd_params& p);
int tc_bwd(const fdma_bwd_params& p, cudaStream_t stream);

// ---- single-query (decode) forward: row-granular skipping, split over keys + merge -------------
bool decode_supported(const fdma_fwd_params& p);
size_t decode_workspace_bytes(const fdma_fwd_params& p);
int decode_fwd(const fdma_fwd_params& p, cudaStream_t stream);

// ---- create_mask -------------------------------------------------------------------------------
int create_mask(const fdma_mask_params& p, cudaStream_t stream);

// ---- helpers -----------------------------------------------------------------------------------
// Device address of the current device's kernel status word (written by bounded waits that give up).
int* kernel_status_ptr();

// Copies D = rowsum(dO o O) from a kernel's scratch layout (B*H rows of `sq_r` floats, zeros beyond Sq) into the
// caller's optional fdma_bwd_params::softmax_d (B, H, round_up(Sq,128)); no-op when that pointer is null.
int export_softmax_d(const fdma_bwd_params& bp, const float* dsum, int sq_r, cudaStream_t stream);

// Number of SMs of the current device (cudaDevAttrMultiProcessorCount, cached per device).
int sm_count();

// Events registered by fdma_time_next_kernel for this host thread (both null when none); take_* clears them.
void take_timing_events(cudaEvent_t* start, cudaEvent_t* stop);

// Encodes a 4-D tiled tensor map (dims innermost first) with 128-byte swizzle; returns 0 or a status.
int encode_tmap_4d(void* out_map, const void* base, int elem_bytes, const uint64_t dims[4],
                   const uint64_t strides_bytes[3], const uint32_t box[4]);

}  // namespace fdma
