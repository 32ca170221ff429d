// C-ABI front end of libsdpa_b200.so: argument validation (the checks mha_varlen_fwd/bwd make
// at torch_mlu/csrc/aten/operators/cnnl/internal/FlashAttention_internal.cpp:73-127, 291-366,
// plus the dispatcher constraints of .../transformers/sdp_utils.h:231-255, 371-431 that apply
// to this path), workspace sizing, kernel selection and TMA descriptor construction.
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <atomic>
#include <mutex>

#include "kernels.h"
#include "ptx_sm100.cuh"

namespace sdpa_b200 {

namespace {
thread_local char g_error[512] = "";
std::atomic<uint64_t> g_launches{0};

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t err = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres);
    if (err == cudaSuccess && qres == cudaDriverEntryPointSuccess) fn = reinterpret_cast<EncodeTiledFn>(ptr);
    (void)cudaGetLastError();
  });
  return fn;
}
}  // namespace

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

void count_launch(int n) { g_launches.fetch_add(static_cast<uint64_t>(n), std::memory_order_relaxed); }

int make_tensor_map_16(bool f16, CUtensorMap* map, const void* base, int head_dim, int64_t rows,
                       int64_t heads, int64_t batch, int64_t row_stride, int64_t head_stride,
                       int64_t batch_stride, int box_rows) {
  EncodeTiledFn encode = get_encode_fn();
  if (encode == nullptr) {
    set_error("cuTensorMapEncodeTiled is not available from the CUDA driver");
    return SDPA_B200_NO_DEVICE;
  }
  if (rows < 1) rows = 1;
  cuuint64_t dims[4] = {static_cast<cuuint64_t>(head_dim), static_cast<cuuint64_t>(rows),
                        static_cast<cuuint64_t>(heads), static_cast<cuuint64_t>(batch)};
  // a size-1 dimension never advances, but its stride must still be a legal value
  if (heads == 1 && (head_stride <= 0)) head_stride = row_stride;
  if (batch == 1) batch_stride = row_stride;
  cuuint64_t strides[3] = {static_cast<cuuint64_t>(row_stride) * 2, static_cast<cuuint64_t>(head_stride) * 2,
                           static_cast<cuuint64_t>(batch_stride) * 2};
  cuuint32_t box[4] = {64, static_cast<cuuint32_t>(box_rows), 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = encode(map, f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box,
                      estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed (CUresult %d): dims {%d,%lld,%lld,%lld} strides(elements) "
              "{row %lld, head %lld, batch %lld}",
              static_cast<int>(r), head_dim, (long long)rows, (long long)heads, (long long)batch,
              (long long)row_stride, (long long)head_stride, (long long)batch_stride);
    return SDPA_B200_INVALID_ARG;
  }
  return SDPA_B200_OK;
}

namespace {

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// strides must keep every row 16-byte aligned (TMA and 128-bit loads/stores)
bool stride_ok(int64_t s) { return s > 0 && (s % 8) == 0; }

int check_tensor(const char* name, const void* ptr, int64_t bs, int64_t hs, int64_t rs, bool varlen,
                 int64_t batch, int64_t heads) {
  if (ptr == nullptr) {
    set_error("%s is NULL", name);
    return SDPA_B200_INVALID_ARG;
  }
  if (!aligned16(ptr)) {
    set_error("%s must be 16-byte aligned", name);
    return SDPA_B200_INVALID_ARG;
  }
  if (!stride_ok(rs) || (heads > 1 && !stride_ok(hs)) || (!varlen && batch > 1 && !stride_ok(bs))) {
    set_error("%s: row/head/batch strides must be positive multiples of 8 elements with unit head_dim "
              "stride (got batch %lld, head %lld, row %lld)",
              name, (long long)bs, (long long)hs, (long long)rs);
    return SDPA_B200_INVALID_ARG;
  }
  return SDPA_B200_OK;
}

// Checks shared by forward and backward.
int validate_common(const sdpa_b200_params* p) {
  if (p == nullptr) {
    set_error("params is NULL");
    return SDPA_B200_INVALID_ARG;
  }
  if (p->dtype != SDPA_B200_BF16 && p->dtype != SDPA_B200_F16) {
    set_error("q/k/v must be bf16 or f16 (dtype code %d)", p->dtype);
    return SDPA_B200_UNSUPPORTED;
  }
  if (p->dropout_p != 0.f) {
    if (!(p->dropout_p > 0.f) || !(p->dropout_p < 1.f)) {
      set_error("dropout_p must be 0 or inside (0, 1) (got %g)", static_cast<double>(p->dropout_p));
      return SDPA_B200_INVALID_ARG;
    }
    if (p->kernel == SDPA_B200_KERNEL_DECODE) {
      set_error("the decode kernel has no dropout");
      return SDPA_B200_UNSUPPORTED;
    }
    if (p->keep_rows == nullptr || (reinterpret_cast<uintptr_t>(p->keep_rows) & 15u) != 0) {
      set_error("dropout_p > 0 needs keep_rows from sdpa_b200_dropout_keep_mask (16-byte aligned)");
      return SDPA_B200_INVALID_ARG;
    }
    if (static_cast<int64_t>(p->batch) * p->heads_q > 65535) {
      set_error("dropout: batch * heads_q must be at most 65535");
      return SDPA_B200_UNSUPPORTED;
    }
  }
  if (p->batch <= 0 || p->heads_q <= 0 || p->heads_kv <= 0) {
    set_error("batch, heads_q and heads_kv must be positive (got %d, %d, %d)", p->batch, p->heads_q, p->heads_kv);
    return SDPA_B200_INVALID_ARG;
  }
  if (p->heads_q % p->heads_kv != 0) {
    set_error("Number of heads in key/value must divide number of heads in query (%d vs %d)", p->heads_kv,
              p->heads_q);
    return SDPA_B200_INVALID_ARG;
  }
  if (p->head_dim <= 0 || p->head_dim % 8 != 0 || p->head_dim > 256) {
    set_error("head_dim must be a multiple of 8 and at most 256 (got %d)", p->head_dim);
    return SDPA_B200_INVALID_ARG;
  }
  if (p->head_dim > 128 && (p->bias != nullptr || p->kernel == SDPA_B200_KERNEL_DECODE)) {
    set_error("head dims above 128 (got %d) run in the tile kernels, without a bias", p->head_dim);
    return SDPA_B200_UNSUPPORTED;
  }
  if (!(p->softmax_scale > 0.f) || !(p->softmax_scale < 3.0e38f)) {
    set_error("softmax_scale must be positive and finite (got %g)", static_cast<double>(p->softmax_scale));
    return SDPA_B200_INVALID_ARG;
  }
  const bool varlen = p->cu_seqlens_q != nullptr || p->cu_seqlens_k != nullptr;
  if (varlen && (p->cu_seqlens_q == nullptr || p->cu_seqlens_k == nullptr)) {
    set_error("cu_seqlens_q and cu_seqlens_k must both be given or both be NULL");
    return SDPA_B200_INVALID_ARG;
  }
  if (p->max_seqlen_q <= 0 || p->max_seqlen_k <= 0) {
    set_error("sequence lengths must be positive (max_seqlen_q %d, max_seqlen_k %d)", p->max_seqlen_q,
              p->max_seqlen_k);
    return SDPA_B200_INVALID_ARG;
  }
  if (varlen && (p->total_q <= 0 || p->total_k <= 0)) {
    set_error("varlen needs total_q and total_k > 0 (got %d, %d)", p->total_q, p->total_k);
    return SDPA_B200_INVALID_ARG;
  }
  if (p->bias != nullptr) {
    if (p->kernel == SDPA_B200_KERNEL_DECODE) {
      set_error("an additive bias is built for the tile kernels only");
      return SDPA_B200_UNSUPPORTED;
    }
    auto bad = [](int64_t s) { return s < 0 || (s % 8) != 0; };
    if (!aligned16(p->bias) || bad(p->bias_batch_stride) || bad(p->bias_head_stride) || bad(p->bias_row_stride)) {
      set_error("bias must be 16-byte aligned with batch / head / row strides that are 0 or multiples of 8 elements "
                "(got %lld, %lld, %lld)",
                (long long)p->bias_batch_stride, (long long)p->bias_head_stride, (long long)p->bias_row_stride);
      return SDPA_B200_INVALID_ARG;
    }
  }
  if (p->sm_margin < 0) {
    set_error("sm_margin must not be negative (got %d)", p->sm_margin);
    return SDPA_B200_INVALID_ARG;
  }
  if ((reinterpret_cast<uintptr_t>(p->device_status) & 3u) != 0) {
    set_error("device_status must be 4-byte aligned");
    return SDPA_B200_INVALID_ARG;
  }
  if (p->dropout_p == 0.f && (p->keep_rows != nullptr || p->keep_cols != nullptr)) {
    set_error("keep_rows / keep_cols must be NULL when dropout_p is 0");
    return SDPA_B200_INVALID_ARG;
  }
  int st;
  if ((st = check_tensor("q", p->q, p->q_batch_stride, p->q_head_stride, p->q_row_stride, varlen, p->batch,
                         p->heads_q)) != SDPA_B200_OK)
    return st;
  if ((st = check_tensor("k", p->k, p->k_batch_stride, p->k_head_stride, p->k_row_stride, varlen, p->batch,
                         p->heads_kv)) != SDPA_B200_OK)
    return st;
  if ((st = check_tensor("v", p->v, p->v_batch_stride, p->v_head_stride, p->v_row_stride, varlen, p->batch,
                         p->heads_kv)) != SDPA_B200_OK)
    return st;
  if ((st = check_tensor("out", p->out, p->o_batch_stride, p->o_head_stride, p->o_row_stride, varlen, p->batch,
                         p->heads_q)) != SDPA_B200_OK)
    return st;
  if (p->lse == nullptr) {
    set_error("lse is NULL");
    return SDPA_B200_INVALID_ARG;
  }
  return SDPA_B200_OK;
}

int validate_workspace(void* workspace, size_t have, size_t need) {
  if (workspace == nullptr || (reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) {
    set_error("workspace must be a non-NULL device pointer aligned to 256 bytes");
    return SDPA_B200_INVALID_ARG;
  }
  if (have < need) {
    set_error("workspace too small: %zu bytes given, %zu needed", have, need);
    return SDPA_B200_INVALID_ARG;
  }
  return SDPA_B200_OK;
}

// Decode is chosen when there are too few query rows to fill a 128-row MMA tile.
bool use_decode(const sdpa_b200_params* p) {
  if (p->kernel == SDPA_B200_KERNEL_DECODE) return true;
  if (p->kernel == SDPA_B200_KERNEL_PREFILL || p->dropout_p != 0.f || p->bias != nullptr) return false;
  // the streaming kernel reads whole 64- or 128-element rows; other head dims take the tile kernel,
  // whose TMA loads pad the head dim with zeros
  return p->cu_seqlens_q == nullptr && p->max_seqlen_q == 1 && (p->head_dim == 64 || p->head_dim == 128);
}

}  // namespace

int sm_count() {
  static std::mutex mu;
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -1;
  std::lock_guard<std::mutex> lock(mu);
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return -1;
    cached[dev] = n;
  }
  return cached[dev];
}

int validate_forward_args(const sdpa_b200_params* p) { return validate_common(p); }

// The compute capability is looked up once per device; the table is shared by all host threads.
int check_device() {
  static std::mutex mu;
  static int8_t major_of[64] = {0};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    (void)cudaGetLastError();
    set_error("no CUDA device is available; this library has no CPU path");
    return SDPA_B200_NO_DEVICE;
  }
  int major = 0;
  {
    std::lock_guard<std::mutex> lock(mu);
    if (major_of[dev] == 0) {
      int m = 0;
      if (cudaDeviceGetAttribute(&m, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) {
        (void)cudaGetLastError();
        m = -1;
      }
      major_of[dev] = static_cast<int8_t>(m);
    }
    major = major_of[dev];
  }
  if (major != 10) {
    set_error("device %d has compute capability %d.x; sm_100 is required", dev, major);
    return SDPA_B200_NO_DEVICE;
  }
  return SDPA_B200_OK;
}

}  // namespace sdpa_b200

namespace sdpa_b200 {
namespace {
// One warp, one barrier that nothing arrives on: the wait runs out after `budget_ns`, lane 0 records the status the
// way the attention kernels do, and the kernel returns.
__global__ void selftest_wait_timeout_kernel(uint32_t* status, uint64_t budget_ns) {
  __shared__ uint64_t barrier;
  __shared__ uint32_t abort_word;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&barrier), 1);
    abort_word = 0;
    fence_mbar_init();
  }
  __syncwarp();
  const bool ok = mbar_wait_budget(smem_u32(&barrier), 0, &abort_word, budget_ns);
  __syncwarp();
  if (threadIdx.x == 0 && (!ok || abort_word != 0)) atomicExch(status, static_cast<uint32_t>(SDPA_B200_DEVICE_TIMEOUT));
}
}  // namespace
}  // namespace sdpa_b200

using namespace sdpa_b200;

extern "C" {

int sdpa_b200_selftest_wait_timeout(uint32_t* device_status, uint32_t budget_us, void* stream) {
  if (device_status == nullptr || (reinterpret_cast<uintptr_t>(device_status) & 3u) != 0) {
    set_error("device_status must be a 4-byte aligned device pointer");
    return SDPA_B200_INVALID_ARG;
  }
  if (budget_us == 0 || budget_us > 1000000u) {
    set_error("budget_us must be between 1 and 1000000 (got %u)", budget_us);
    return SDPA_B200_INVALID_ARG;
  }
  int st = check_device();
  if (st != SDPA_B200_OK) return st;
  selftest_wait_timeout_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(device_status,
                                                                                static_cast<uint64_t>(budget_us) * 1000ull);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) {
    set_error("selftest: launch failed: %s", cudaGetErrorString(err));
    return SDPA_B200_LAUNCH_FAILED;
  }
  count_launch();
  return SDPA_B200_OK;
}

int sdpa_b200_version(void) { return SDPA_B200_VERSION; }

const char* sdpa_b200_status_string(int status) {
  switch (status) {
    case SDPA_B200_OK: return "ok";
    case SDPA_B200_INVALID_ARG: return "invalid argument";
    case SDPA_B200_UNSUPPORTED: return "unsupported configuration";
    case SDPA_B200_LAUNCH_FAILED: return "CUDA launch failed";
    case SDPA_B200_DEVICE_TIMEOUT: return "a bounded wait inside a kernel ran out";
    case SDPA_B200_NO_DEVICE: return "no sm_100 CUDA device";
    default: return "unknown status";
  }
}

const char* sdpa_b200_last_error(void) { return g_error; }

uint64_t sdpa_b200_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int sdpa_b200_fwd_workspace_bytes(const sdpa_b200_params* p, size_t* bytes) {
  if (bytes == nullptr) {
    set_error("bytes is NULL");
    return SDPA_B200_INVALID_ARG;
  }
  int st = validate_common(p);
  if (st != SDPA_B200_OK) return st;
  size_t need = kWorkspaceHeaderBytes;
  if (use_decode(p)) need += decode_workspace_bytes(*p, nullptr);
  *bytes = need;
  return SDPA_B200_OK;
}

int sdpa_b200_bwd_workspace_bytes(const sdpa_b200_params* p, size_t* bytes) {
  if (bytes == nullptr) {
    set_error("bytes is NULL");
    return SDPA_B200_INVALID_ARG;
  }
  int st = validate_common(p);
  if (st != SDPA_B200_OK) return st;
  *bytes = kWorkspaceHeaderBytes + (p->head_dim > 128 ? bwd_d256_workspace_bytes(*p) : bwd_workspace_bytes(*p));
  return SDPA_B200_OK;
}

int sdpa_b200_fwd(const sdpa_b200_params* p, void* workspace, size_t workspace_bytes, void* stream) {
  int st = validate_common(p);
  if (st != SDPA_B200_OK) return st;
  if (use_decode(p) && (st = check_decode_request(*p)) != SDPA_B200_OK) return st;
  size_t need = 0;
  st = sdpa_b200_fwd_workspace_bytes(p, &need);
  if (st != SDPA_B200_OK) return st;
  st = validate_workspace(workspace, workspace_bytes, need);
  if (st != SDPA_B200_OK) return st;
  st = check_device();
  if (st != SDPA_B200_OK) return st;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (cudaMemsetAsync(workspace, 0, kWorkspaceHeaderBytes, s) != cudaSuccess) {
    set_error("clearing the workspace header failed: %s", cudaGetErrorString(cudaGetLastError()));
    return SDPA_B200_LAUNCH_FAILED;
  }
  if (use_decode(p)) return launch_fwd_decode(*p, workspace, workspace_bytes, s);
  if (p->head_dim > 128) return launch_fwd_d256(*p, workspace, s);
  return launch_fwd_prefill(*p, workspace, s);
}

int sdpa_b200_bwd(const sdpa_b200_params* p, void* workspace, size_t workspace_bytes, void* stream) {
  int st = validate_common(p);
  if (st != SDPA_B200_OK) return st;

  if (p->bias_t != nullptr) {
    auto bad = [](int64_t s) { return s < 0 || (s % 8) != 0; };
    if (p->bias == nullptr || !aligned16(p->bias_t) || bad(p->bias_t_batch_stride) || bad(p->bias_t_head_stride) ||
        bad(p->bias_t_row_stride)) {
      set_error("bias_t needs a bias, 16-byte alignment and strides that are 0 or multiples of 8 elements");
      return SDPA_B200_INVALID_ARG;
    }
  }
  if (p->dbias != nullptr) {
    const int64_t need = (static_cast<int64_t>(p->max_seqlen_k) + 7) / 8 * 8;
    if (p->bias == nullptr || !aligned16(p->dbias) || p->dbias_row_stride < need || (p->dbias_row_stride % 8) != 0 ||
        (p->dbias_head_stride % 8) != 0 || (p->dbias_batch_stride % 8) != 0 || p->dbias_head_stride <= 0 ||
        (p->batch > 1 && p->dbias_batch_stride <= 0)) {
      set_error("dbias needs a bias, 16-byte alignment, strides that are multiples of 8 and a row stride of at least "
                "seqlen_k rounded up to 8");
      return SDPA_B200_INVALID_ARG;
    }
  }
  if (p->dropout_p != 0.f && (p->keep_cols == nullptr || (reinterpret_cast<uintptr_t>(p->keep_cols) & 15u) != 0)) {
    set_error("dropout_p > 0 needs keep_cols from sdpa_b200_dropout_keep_mask (16-byte aligned) in the backward");
    return SDPA_B200_INVALID_ARG;
  }
  const bool varlen = p->cu_seqlens_q != nullptr;
  if ((st = check_tensor("dout", p->dout, p->do_batch_stride, p->do_head_stride, p->do_row_stride, varlen,
                         p->batch, p->heads_q)) != SDPA_B200_OK)
    return st;
  if ((st = check_tensor("dq", p->dq, p->dq_batch_stride, p->dq_head_stride, p->dq_row_stride, varlen, p->batch,
                         p->heads_q)) != SDPA_B200_OK)
    return st;
  if ((st = check_tensor("dk", p->dk, p->dk_batch_stride, p->dk_head_stride, p->dk_row_stride, varlen, p->batch,
                         p->heads_kv)) != SDPA_B200_OK)
    return st;
  if ((st = check_tensor("dv", p->dv, p->dv_batch_stride, p->dv_head_stride, p->dv_row_stride, varlen, p->batch,
                         p->heads_kv)) != SDPA_B200_OK)
    return st;
  const size_t need = kWorkspaceHeaderBytes + (p->head_dim > 128 ? bwd_d256_workspace_bytes(*p) : bwd_workspace_bytes(*p));
  st = validate_workspace(workspace, workspace_bytes, need);
  if (st != SDPA_B200_OK) return st;
  st = check_device();
  if (st != SDPA_B200_OK) return st;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (cudaMemsetAsync(workspace, 0, kWorkspaceHeaderBytes, s) != cudaSuccess) {
    set_error("clearing the workspace header failed: %s", cudaGetErrorString(cudaGetLastError()));
    return SDPA_B200_LAUNCH_FAILED;
  }
  if (p->head_dim > 128) return launch_bwd_d256(*p, workspace, s);
  return launch_bwd(*p, workspace, workspace_bytes, s);
}

int sdpa_b200_read_device_status(const void* workspace, void* stream, int* device_status) {
  if (workspace == nullptr || device_status == nullptr) {
    set_error("workspace and device_status must be non-NULL");
    return SDPA_B200_INVALID_ARG;
  }
  uint32_t word = 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t err = cudaMemcpyAsync(&word, workspace, sizeof(word), cudaMemcpyDeviceToHost, s);
  if (err == cudaSuccess) err = cudaStreamSynchronize(s);
  if (err != cudaSuccess) {
    set_error("reading the device status failed: %s", cudaGetErrorString(err));
    return SDPA_B200_LAUNCH_FAILED;
  }
  *device_status = static_cast<int>(word);
  return SDPA_B200_OK;
}

}  // extern "C"
