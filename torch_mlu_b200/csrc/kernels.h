// Internal launch interface between the C-ABI front end (sdpa_api.cu) and the kernel files.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "../../include/sdpa_b200.h"

namespace sdpa_b200 {

// First 256 bytes of every workspace: word 0 is the device status, the rest is reserved.
constexpr size_t kWorkspaceHeaderBytes = 256;

// Thread-local error text (set by whoever returns a non-OK status).
void set_error(const char* fmt, ...);
void count_launch(int n = 1);

// Builds a 4-D tensor map over 16-bit elements (f16 or bf16) {head_dim, rows, heads, batch} with a
// {64, box_rows, 1, 1} box and 128-byte swizzle. Strides are in ELEMENTS. Returns an SDPA_B200_* status.
int make_tensor_map_16(bool f16, CUtensorMap* map, const void* base, int head_dim, int64_t rows,
                       int64_t heads, int64_t batch, int64_t row_stride, int64_t head_stride,
                       int64_t batch_stride, int box_rows);

// Prefill forward (TMA + tcgen05), a persistent kernel with one CTA per SM.
int launch_fwd_prefill(const sdpa_b200_params& p, void* workspace, cudaStream_t stream);

// Forward for head dims above 128 (up to 256): one CTA per 128 query rows, Q in tensor memory (d256_sm100.cu).
int launch_fwd_d256(const sdpa_b200_params& p, void* workspace, cudaStream_t stream);
// Backward for the same head dims: a pre-pass and one kernel each for dV, dK and dQ (d256_sm100.cu).
size_t bwd_d256_workspace_bytes(const sdpa_b200_params& p);
int launch_bwd_d256(const sdpa_b200_params& p, void* workspace, cudaStream_t stream);

// Number of SMs of the current device (cached per device), <= 0 on error.
int sm_count();

// Split-KV decode forward. Workspace layout is private to decode_splitkv.cu.
size_t decode_workspace_bytes(const sdpa_b200_params& p, int* num_splits_out);
int launch_fwd_decode(const sdpa_b200_params& p, void* workspace, size_t workspace_bytes,
                      cudaStream_t stream);

// Argument checks of the forward entry point (no device is touched) and the device check, for entry
// points defined outside sdpa_api.cu. Each returns an SDPA_B200_* status and sets the error text.
int validate_forward_args(const sdpa_b200_params* p);
int check_device();

// Refuses what the split-KV decode kernels have no code for (packed tensors, seqlen_q != 1, head dims other
// than 64 and 128, dropout, bias). Touches no device.
int check_decode_request(const sdpa_b200_params& p);

// round(dropout_p * 256), the byte threshold of the dropout keep-masks (dropout_mask.cu)
uint32_t dropout_drop_byte(float dropout_p);

// Backward: delta pre-pass + dK/dV kernel + dQ kernel.
size_t bwd_workspace_bytes(const sdpa_b200_params& p);
int launch_bwd(const sdpa_b200_params& p, void* workspace, size_t workspace_bytes,
               cudaStream_t stream);

}  // namespace sdpa_b200
