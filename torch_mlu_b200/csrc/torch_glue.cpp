// Thin PyTorch dispatcher glue over the C ABI of libsdpa_b200.so.
//
// Stands where torch_mlu's generated registration (codegen/templates/RegisterMLU.cpp:185-188,
// schemas from codegen/mlu_functions.yaml:1313-1316) binds the attention operators of
// torch_mlu/csrc/aten/operators/cnnl/transformers/attention.cpp:
//   * TORCH_LIBRARY(b200_sdpa): the four operators with the reference's exact (torch 2.1)
//     schemas, implemented for the CUDA key.
//   * b200_sdpa::_install_aten_overrides(): registers CUDA-key kernels for the same four aten
//     operators with the INSTALLED torch's schemas, so F.scaled_dot_product_attention under the
//     flash backend, and upstream autograd, land in these kernels.
// Nothing here copies or re-packs tensors (the reference wrappers make five contiguous copies,
// attention.cpp:124-129, 260-269): strides go straight into sdpa_b200_params. torch supplies
// device memory (outputs, workspace) and the current stream only.
#include <ATen/ATen.h>
#include <ATen/autocast_mode.h>
#include <ATen/cuda/CUDAContext.h>
#include <ATen/cuda/CUDAGeneratorImpl.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include <cmath>
#include <memory>
#include <mutex>
#include <tuple>

#include "../../include/sdpa_b200.h"

namespace {

using at::Tensor;

void check_status(int st, const char* what) {
  TORCH_CHECK(st == SDPA_B200_OK, what, ": ", sdpa_b200_status_string(st), ": ", sdpa_b200_last_error());
}

// FlashAttention_internal.cpp:73-108: device, dtype and last-dim stride checks
void check_input(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be on a CUDA device (this path has no CPU fallback)");
  TORCH_CHECK(t.scalar_type() == at::kBFloat16 || t.scalar_type() == at::kHalf,
              "FlashAttention only support fp16 and bf16 data type (", name, " is ", t.scalar_type(), ")");
  TORCH_CHECK(t.stride(-1) == 1, "Input tensor must have contiguous last dimension (", name, ")");
}

double scale_or_default(const Tensor& q, c10::optional<double> scale) {  // sdp_utils.h:40-47
  return scale.has_value() ? *scale : 1.0 / std::sqrt(static_cast<double>(q.size(-1)));
}

void set_bhld(int64_t& bs, int64_t& hs, int64_t& rs, const Tensor& t) {
  bs = t.stride(0);
  hs = t.stride(1);
  rs = t.stride(2);
}

void set_thd(int64_t& bs, int64_t& hs, int64_t& rs, const Tensor& t) {
  bs = 0;
  hs = t.stride(1);
  rs = t.stride(0);
}

void base_params(sdpa_b200_params& p, const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& out,
                 const Tensor& lse, bool causal, double scale) {
  std::memset(&p, 0, sizeof(p));
  p.q = q.data_ptr();
  p.k = k.data_ptr();
  p.v = v.data_ptr();
  p.out = out.data_ptr();
  p.lse = lse.data_ptr<float>();
  p.softmax_scale = static_cast<float>(scale);
  p.is_causal = causal ? 1 : 0;
  TORCH_CHECK(k.scalar_type() == q.scalar_type() && v.scalar_type() == q.scalar_type(),
              "query, key, and value must have the same dtype");
  p.dtype = q.scalar_type() == at::kHalf ? SDPA_B200_F16 : SDPA_B200_BF16;
  p.kernel = SDPA_B200_KERNEL_AUTO;
}

void dense_params(sdpa_b200_params& p, const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& out,
                  const Tensor& lse, bool causal, double scale) {
  base_params(p, q, k, v, out, lse, causal, scale);
  p.batch = static_cast<int32_t>(q.size(0));
  p.heads_q = static_cast<int32_t>(q.size(1));
  p.heads_kv = static_cast<int32_t>(k.size(1));
  p.head_dim = static_cast<int32_t>(q.size(3));
  p.max_seqlen_q = static_cast<int32_t>(q.size(2));
  p.max_seqlen_k = static_cast<int32_t>(k.size(2));
  set_bhld(p.q_batch_stride, p.q_head_stride, p.q_row_stride, q);
  set_bhld(p.k_batch_stride, p.k_head_stride, p.k_row_stride, k);
  set_bhld(p.v_batch_stride, p.v_head_stride, p.v_row_stride, v);
  set_bhld(p.o_batch_stride, p.o_head_stride, p.o_row_stride, out);
}

void varlen_params(sdpa_b200_params& p, const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& out,
                   const Tensor& lse, const Tensor& cu_q, const Tensor& cu_k, int64_t max_q, int64_t max_k, bool causal,
                   double scale) {
  base_params(p, q, k, v, out, lse, causal, scale);
  p.cu_seqlens_q = cu_q.data_ptr<int32_t>();
  p.cu_seqlens_k = cu_k.data_ptr<int32_t>();
  p.batch = static_cast<int32_t>(cu_q.numel() - 1);
  p.heads_q = static_cast<int32_t>(q.size(1));
  p.heads_kv = static_cast<int32_t>(k.size(1));
  p.head_dim = static_cast<int32_t>(q.size(2));
  p.max_seqlen_q = static_cast<int32_t>(max_q);
  p.max_seqlen_k = static_cast<int32_t>(max_k);
  p.total_q = static_cast<int32_t>(q.size(0));
  p.total_k = static_cast<int32_t>(k.size(0));
  p.kernel = SDPA_B200_KERNEL_PREFILL;
  set_thd(p.q_batch_stride, p.q_head_stride, p.q_row_stride, q);
  set_thd(p.k_batch_stride, p.k_head_stride, p.k_row_stride, k);
  set_thd(p.v_batch_stride, p.v_head_stride, p.v_row_stride, v);
  set_thd(p.o_batch_stride, p.o_head_stride, p.o_row_stride, out);
}

// One int32 per device that every call made through this glue hands to the kernels (sdpa_b200_params.device_status):
// a kernel whose bounded wait runs out leaves SDPA_B200_DEVICE_TIMEOUT in it, and it stays there, whatever happens
// to the per-call workspaces, until b200_sdpa::_device_status reads and clears it.
Tensor& status_word(int device) {
  static std::mutex mu;
  static Tensor words[64];
  TORCH_CHECK(device >= 0 && device < 64, "device index out of range");
  std::lock_guard<std::mutex> lock(mu);
  if (!words[device].defined())
    words[device] = at::zeros({1}, at::TensorOptions().dtype(at::kInt).device(at::kCUDA, device));
  return words[device];
}

int64_t device_status(int64_t device) {
  if (device < 0) device = at::cuda::current_device();
  c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device));
  Tensor& word = status_word(static_cast<int>(device));
  int st = 0;
  check_status(sdpa_b200_read_device_status(word.data_ptr(), at::cuda::getCurrentCUDAStream(device).stream(), &st),
               "sdpa_b200_read_device_status");
  if (st != 0) word.zero_();
  return st;
}

void run(const sdpa_b200_params& params, bool backward, const Tensor& like) {
  sdpa_b200_params p = params;
  p.device_status = reinterpret_cast<uint32_t*>(status_word(like.get_device()).data_ptr());
  // torch.use_deterministic_algorithms(True) selects the backward with a fixed summation order
  p.deterministic = at::globalContext().deterministicAlgorithms() ? 1 : 0;
  size_t bytes = 0;
  check_status(backward ? sdpa_b200_bwd_workspace_bytes(&p, &bytes) : sdpa_b200_fwd_workspace_bytes(&p, &bytes),
               "sdpa_b200 workspace query");
  Tensor ws = at::empty({static_cast<int64_t>(bytes)}, like.options().dtype(at::kByte));
  void* stream = at::cuda::getCurrentCUDAStream(like.get_device()).stream();
  check_status(backward ? sdpa_b200_bwd(&p, ws.data_ptr(), bytes, stream) : sdpa_b200_fwd(&p, ws.data_ptr(), bytes, stream),
               backward ? "sdpa_b200_bwd" : "sdpa_b200_fwd");
}

void check_varlen(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& cu_q, const Tensor& cu_k) {
  // FlashAttention_internal.cpp:81-84, 112-127
  TORCH_CHECK(q.dim() == 3 && k.dim() == 3 && v.dim() == 3,
              "varlen query, key and value must be packed [total_tokens, heads, head_dim]");
  TORCH_CHECK(cu_q.scalar_type() == at::kInt, "cu_seqlens_q must have dtype int32");
  TORCH_CHECK(cu_k.scalar_type() == at::kInt, "cu_seqlens_k must have dtype int32");
  TORCH_CHECK(cu_q.is_cuda() && cu_k.is_cuda() && cu_q.is_contiguous() && cu_k.is_contiguous(),
              "cu_seqlens must be contiguous device tensors");
  TORCH_CHECK(cu_q.numel() == cu_k.numel() && cu_q.numel() >= 2, "cu_seqlens_q and cu_seqlens_k must have batch+1 entries");
  TORCH_CHECK(k.size(1) == v.size(1) && q.size(1) % k.size(1) == 0,
              "Number of heads in key/value must divide number of heads in query");
  check_input(q, "query");
  check_input(k, "key");
  check_input(v, "value");
}

// ------------------------------------------------------------------------- dropout pattern
// One bit per (query, key) pair in both orientations, written by the library from a Philox seed / offset pair
// (the reference draws the pattern inside its kernel from such a pair and hands the pair to the backward
// operator, FlashAttention_internal.cpp:190-214).
struct KeepMasks {
  Tensor rows, cols;  // int32 [B*H, Lq_pad, Lk_pad/32] and [B*H, Lk_pad, Lq_pad/32]
  double p = 0.0;
};

KeepMasks make_keep_masks(const Tensor& q, int64_t seqlen_k, double dropout_p, uint64_t seed, uint64_t offset, bool causal) {
  TORCH_CHECK(dropout_p > 0.0 && dropout_p < 1.0, "dropout_p must be inside [0, 1)");
  c10::cuda::CUDAGuard guard(q.device());
  const int64_t BH = q.size(0) * q.size(1), Lq = q.size(2);
  const int64_t lq_pad = (Lq + 127) / 128 * 128, lk_pad = (seqlen_k + 127) / 128 * 128;
  KeepMasks m;
  m.p = dropout_p;
  m.rows = at::empty({BH, lq_pad, lk_pad / 32}, q.options().dtype(at::kInt));
  m.cols = at::empty({BH, lk_pad, lq_pad / 32}, q.options().dtype(at::kInt));
  check_status(sdpa_b200_dropout_keep_mask(seed, offset, static_cast<float>(dropout_p), static_cast<int32_t>(q.size(0)),
                                           static_cast<int32_t>(q.size(1)), static_cast<int32_t>(Lq),
                                           static_cast<int32_t>(seqlen_k), causal ? 1 : 0,
                                           reinterpret_cast<uint32_t*>(m.rows.data_ptr()),
                                           reinterpret_cast<uint32_t*>(m.cols.data_ptr()),
                                           at::cuda::getCurrentCUDAStream().stream()),
               "sdpa_b200_dropout_keep_mask");
  return m;
}

// The masks of the most recent forward call per device stay here, so that the backward operator that is handed the same
// Philox pair (and shapes) takes them instead of drawing the whole pattern again; any other pair is drawn afresh.
struct KeepKey {
  int device = -1;
  uint64_t seed = 0, offset = 0;
  double p = 0.0;
  int64_t a = 0, b = 0, c = 0, d = 0;  // dense: batch, heads, Lq, Lk; packed: heads, total_q, total_k, max_q * 2^32 + max_k
  bool causal = false, packed = false;
  const void* cu_q = nullptr;
  bool operator==(const KeepKey& o) const {
    return device == o.device && seed == o.seed && offset == o.offset && p == o.p && a == o.a && b == o.b && c == o.c &&
           d == o.d && causal == o.causal && packed == o.packed && cu_q == o.cu_q;
  }
};

struct KeepCache {
  std::mutex mu;
  KeepKey key[64];
  KeepMasks masks[64];
  void put(const KeepKey& k, const KeepMasks& m) {
    if (k.device < 0 || k.device >= 64) return;
    std::lock_guard<std::mutex> lock(mu);
    key[k.device] = k;
    masks[k.device] = m;
  }
  bool take(const KeepKey& k, KeepMasks* m) {
    if (k.device < 0 || k.device >= 64) return false;
    std::lock_guard<std::mutex> lock(mu);
    if (!(key[k.device] == k) || !masks[k.device].rows.defined()) return false;
    *m = masks[k.device];
    key[k.device] = KeepKey();  // one forward, one backward: drop the reference so the memory can go back
    masks[k.device] = KeepMasks();
    return true;
  }
};
KeepCache g_keep_cache;

KeepKey dense_keep_key(const Tensor& q, int64_t seqlen_k, double p, uint64_t seed, uint64_t offset, bool causal) {
  KeepKey k;
  k.device = q.get_device();
  k.seed = seed;
  k.offset = offset;
  k.p = p;
  k.a = q.size(0);
  k.b = q.size(1);
  k.c = q.size(2);
  k.d = seqlen_k;
  k.causal = causal;
  return k;
}

KeepKey packed_keep_key(const Tensor& q, const Tensor& k_, const Tensor& cu_q, int64_t max_q, int64_t max_k, double p,
                        uint64_t seed, uint64_t offset, bool causal) {
  KeepKey k;
  k.device = q.get_device();
  k.seed = seed;
  k.offset = offset;
  k.p = p;
  k.a = q.size(1);
  k.b = q.size(0);
  k.c = k_.size(0);
  k.d = (max_q << 32) + max_k;
  k.causal = causal;
  k.packed = true;
  k.cu_q = cu_q.data_ptr();
  return k;
}

// (seed, offset) of the device's default generator, advanced like any other Philox consumer
std::pair<uint64_t, uint64_t> draw_philox(const Tensor& q, int64_t elements) {
  auto gen = at::get_generator_or_default<at::CUDAGeneratorImpl>(c10::nullopt,
                                                                 at::cuda::detail::getDefaultCUDAGenerator(q.get_device()));
  std::lock_guard<std::mutex> lock(gen->mutex_);
  return gen->philox_engine_inputs(static_cast<uint64_t>((elements + 3) / 4));
}

Tensor cpu_i64(uint64_t v) { return at::scalar_tensor(at::Scalar(static_cast<int64_t>(v)), at::dtype(at::kLong)); }

// > 0 where a pair was kept, in q's dtype, [B, H, Lq, Lk] (the debug mask of FlashAttention_internal.cpp:141-146)
Tensor debug_mask_of(const KeepMasks& m, const Tensor& q, int64_t seqlen_k) {
  Tensor bits = at::bitwise_and(at::bitwise_right_shift(m.rows.unsqueeze(-1), at::arange(32, m.rows.options())), 1);
  return bits.reshape({m.rows.size(0), m.rows.size(1), -1})
      .slice(1, 0, q.size(2))
      .slice(2, 0, seqlen_k)
      .reshape({q.size(0), q.size(1), q.size(2), seqlen_k})
      .to(q.scalar_type());
}

void set_dropout(sdpa_b200_params& p, const KeepMasks* keep) {
  if (keep == nullptr) return;
  p.dropout_p = static_cast<float>(keep->p);
  p.keep_rows = reinterpret_cast<const uint32_t*>(keep->rows.data_ptr());
  p.keep_cols = reinterpret_cast<const uint32_t*>(keep->cols.data_ptr());
}

// ------------------------------------------------------------------------- dense [B,H,L,D]
std::tuple<Tensor, Tensor> dense_forward(const Tensor& q, const Tensor& k, const Tensor& v, bool causal, double scale,
                                         bool allow_gqa, const KeepMasks* keep = nullptr) {
  // attention.cpp:70-100
  TORCH_CHECK(q.dim() == 4 && k.dim() == 4 && v.dim() == 4,
              "query, key and value must be 4-dimensional [batch, heads, seq_len, head_dim]");
  TORCH_CHECK(q.size(0) == k.size(0) && q.size(0) == v.size(0), "query, key and value must have the same batch size");
  TORCH_CHECK(k.size(2) == v.size(2), "Key and Value must have the same sequence length");
  if (allow_gqa) {
    TORCH_CHECK(k.size(1) == v.size(1) && q.size(1) % k.size(1) == 0,
                "Number of heads in key/value must divide number of heads in query");
  } else {
    TORCH_CHECK(q.size(1) == k.size(1) && q.size(1) == v.size(1), "query, key and value must have the same number of heads");
  }
  TORCH_CHECK(q.size(3) == k.size(3) && q.size(3) == v.size(3), "query, key and value must have the same head_dim");
  check_input(q, "query");
  check_input(k, "key");
  check_input(v, "value");
  c10::cuda::CUDAGuard guard(q.device());
  const int64_t B = q.size(0), H = q.size(1), L = q.size(2), D = q.size(3);
  // [B,H,L,D] view of a [B,L,H,D] buffer, as the reference returns (attention.cpp:146-148)
  Tensor out = at::empty({B, L, H, D}, q.options()).transpose(1, 2);
  Tensor lse = at::empty({B, H, L}, q.options().dtype(at::kFloat));
  sdpa_b200_params p;
  dense_params(p, q, k, v, out, lse, causal, scale);
  set_dropout(p, keep);
  run(p, false, q);
  return {out, lse};
}

std::tuple<Tensor, Tensor, Tensor> dense_backward(const Tensor& dout_in, const Tensor& q, const Tensor& k, const Tensor& v,
                                                  const Tensor& out, const Tensor& lse, bool causal, double scale,
                                                  const KeepMasks* keep = nullptr) {
  Tensor dout = dout_in.stride(-1) == 1 ? dout_in : dout_in.contiguous();
  check_input(dout, "grad_out");
  check_input(q, "query");
  check_input(k, "key");
  check_input(v, "value");
  check_input(out, "out");
  TORCH_CHECK(lse.scalar_type() == at::kFloat && lse.is_contiguous() && lse.dim() == 3 && lse.size(0) == q.size(0) &&
                  lse.size(1) == q.size(1) && lse.size(2) == q.size(2),
              "logsumexp must be contiguous fp32 [batch, heads, seqlen_q]");
  c10::cuda::CUDAGuard guard(q.device());
  const int64_t B = q.size(0), D = q.size(3);
  Tensor dq = at::empty({B, q.size(2), q.size(1), D}, q.options()).transpose(1, 2);
  Tensor dk = at::empty({B, k.size(2), k.size(1), D}, k.options()).transpose(1, 2);
  Tensor dv = at::empty({B, v.size(2), v.size(1), D}, v.options()).transpose(1, 2);
  sdpa_b200_params p;
  dense_params(p, q, k, v, out, lse, causal, scale);
  p.dout = dout.data_ptr();
  p.dq = dq.data_ptr();
  p.dk = dk.data_ptr();
  p.dv = dv.data_ptr();
  set_bhld(p.do_batch_stride, p.do_head_stride, p.do_row_stride, dout);
  set_bhld(p.dq_batch_stride, p.dq_head_stride, p.dq_row_stride, dq);
  set_bhld(p.dk_batch_stride, p.dk_head_stride, p.dk_row_stride, dk);
  set_bhld(p.dv_batch_stride, p.dv_head_stride, p.dv_row_stride, dv);
  set_dropout(p, keep);
  run(p, true, q);
  return {dq, dk, dv};
}

// The dense operator pair with dropout: the forward draws a Philox pair, returns it as two CPU int64 scalars
// (and the pattern on request); the backward draws the same pattern again from them.
struct DenseDropoutResult {
  Tensor out, lse, seed, offset, debug;
};

DenseDropoutResult dense_forward_with_dropout(const Tensor& q, const Tensor& k, const Tensor& v, double dropout_p,
                                              bool causal, bool return_debug_mask, double scale, bool allow_gqa) {
  TORCH_CHECK(dropout_p >= 0.0 && dropout_p < 1.0, "dropout_p must be inside [0, 1)");
  DenseDropoutResult r;
  r.seed = at::empty({0}, q.options().dtype(at::kLong));
  r.offset = at::empty({0}, q.options().dtype(at::kLong));
  r.debug = at::empty({0}, q.options());
  if (dropout_p == 0.0) {
    std::tie(r.out, r.lse) = dense_forward(q, k, v, causal, scale, allow_gqa);
    return r;
  }
  TORCH_CHECK(q.dim() == 4 && k.dim() == 4, "query, key and value must be 4-dimensional [batch, heads, seq_len, head_dim]");
  auto [seed, offset] = draw_philox(q, q.size(0) * q.size(1) * q.size(2) * k.size(2));
  KeepMasks keep = make_keep_masks(q, k.size(2), dropout_p, seed, offset, causal);
  std::tie(r.out, r.lse) = dense_forward(q, k, v, causal, scale, allow_gqa, &keep);
  g_keep_cache.put(dense_keep_key(q, k.size(2), dropout_p, seed, offset, causal), keep);
  r.seed = cpu_i64(seed);
  r.offset = cpu_i64(offset);
  if (return_debug_mask) r.debug = debug_mask_of(keep, q, k.size(2));
  return r;
}

std::tuple<Tensor, Tensor, Tensor> dense_backward_with_dropout(const Tensor& grad_out, const Tensor& q, const Tensor& k,
                                                               const Tensor& v, const Tensor& out, const Tensor& lse,
                                                               double dropout_p, bool causal, const Tensor& philox_seed,
                                                               const Tensor& philox_offset, double scale) {
  TORCH_CHECK(dropout_p >= 0.0 && dropout_p < 1.0, "dropout_p must be inside [0, 1)");
  if (dropout_p == 0.0) return dense_backward(grad_out, q, k, v, out, lse, causal, scale);
  TORCH_CHECK(philox_seed.numel() == 1 && philox_offset.numel() == 1,
              "dropout_p > 0 needs the philox_seed and philox_offset the forward operator returned");
  const uint64_t seed = static_cast<uint64_t>(philox_seed.item<int64_t>());
  const uint64_t offset = static_cast<uint64_t>(philox_offset.item<int64_t>());
  KeepMasks keep;
  if (!g_keep_cache.take(dense_keep_key(q, k.size(2), dropout_p, seed, offset, causal), &keep))
    keep = make_keep_masks(q, k.size(2), dropout_p, seed, offset, causal);
  return dense_backward(grad_out, q, k, v, out, lse, causal, scale, &keep);
}

// ------------------------------------------------------------------ packed [total,H,D]
// packed form of the pattern: rows by packed token index, see sdpa_b200_dropout_keep_mask_varlen
KeepMasks make_keep_masks_varlen(const Tensor& q, const Tensor& k, const Tensor& cu_q, const Tensor& cu_k, int64_t max_q,
                                 int64_t max_k, double dropout_p, uint64_t seed, uint64_t offset, bool causal) {
  TORCH_CHECK(dropout_p > 0.0 && dropout_p < 1.0, "dropout_p must be inside [0, 1)");
  c10::cuda::CUDAGuard guard(q.device());
  KeepMasks m;
  m.p = dropout_p;
  const int64_t H = q.size(1);
  m.rows = at::zeros({H, q.size(0) + 128, (max_k + 127) / 128 * 4}, q.options().dtype(at::kInt));
  m.cols = at::zeros({H, k.size(0) + 128, (max_q + 127) / 128 * 4}, q.options().dtype(at::kInt));
  check_status(sdpa_b200_dropout_keep_mask_varlen(
                   seed, offset, static_cast<float>(dropout_p), static_cast<int32_t>(cu_q.numel() - 1), static_cast<int32_t>(H),
                   cu_q.data_ptr<int32_t>(), cu_k.data_ptr<int32_t>(), static_cast<int32_t>(q.size(0)),
                   static_cast<int32_t>(k.size(0)), static_cast<int32_t>(max_q), static_cast<int32_t>(max_k), causal ? 1 : 0,
                   reinterpret_cast<uint32_t*>(m.rows.data_ptr()), reinterpret_cast<uint32_t*>(m.cols.data_ptr()),
                   at::cuda::getCurrentCUDAStream().stream()),
               "sdpa_b200_dropout_keep_mask_varlen");
  return m;
}

std::tuple<Tensor, Tensor> varlen_forward(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& cu_q,
                                          const Tensor& cu_k, int64_t max_q, int64_t max_k, bool causal, double scale,
                                          const KeepMasks* keep = nullptr) {
  check_varlen(q, k, v, cu_q, cu_k);
  c10::cuda::CUDAGuard guard(q.device());
  Tensor out = at::empty(q.sizes(), q.options());
  Tensor lse = at::empty({q.size(1), q.size(0)}, q.options().dtype(at::kFloat));  // FlashAttention_internal.cpp:129
  sdpa_b200_params p;
  varlen_params(p, q, k, v, out, lse, cu_q, cu_k, max_q, max_k, causal, scale);
  set_dropout(p, keep);
  run(p, false, q);
  return {out, lse};
}

std::tuple<Tensor, Tensor, Tensor> varlen_backward(const Tensor& dout_in, const Tensor& q, const Tensor& k, const Tensor& v,
                                                   const Tensor& out, const Tensor& lse, const Tensor& cu_q,
                                                   const Tensor& cu_k, int64_t max_q, int64_t max_k, bool causal,
                                                   double scale, const KeepMasks* keep = nullptr) {
  check_varlen(q, k, v, cu_q, cu_k);
  Tensor dout = dout_in.stride(-1) == 1 ? dout_in : dout_in.contiguous();
  check_input(dout, "grad_out");
  check_input(out, "out");
  TORCH_CHECK(lse.scalar_type() == at::kFloat && lse.is_contiguous() && lse.dim() == 2 && lse.size(0) == q.size(1) &&
                  lse.size(1) == q.size(0),
              "logsumexp must be contiguous fp32 [heads_q, total_q]");
  c10::cuda::CUDAGuard guard(q.device());
  Tensor dq = at::empty(q.sizes(), q.options());
  Tensor dk = at::empty(k.sizes(), k.options());
  Tensor dv = at::empty(v.sizes(), v.options());
  sdpa_b200_params p;
  varlen_params(p, q, k, v, out, lse, cu_q, cu_k, max_q, max_k, causal, scale);
  p.dout = dout.data_ptr();
  p.dq = dq.data_ptr();
  p.dk = dk.data_ptr();
  p.dv = dv.data_ptr();
  set_thd(p.do_batch_stride, p.do_head_stride, p.do_row_stride, dout);
  set_thd(p.dq_batch_stride, p.dq_head_stride, p.dq_row_stride, dq);
  set_thd(p.dk_batch_stride, p.dk_head_stride, p.dk_row_stride, dk);
  set_thd(p.dv_batch_stride, p.dv_head_stride, p.dv_row_stride, dv);
  set_dropout(p, keep);
  run(p, true, q);
  return {dq, dk, dv};
}

// The debug mask of a packed call: [B, Hq, max_q, max_k] in q's dtype, > 0 where a pair was kept and 0 outside a
// sequence (attention.cpp:178-196 normalises the vendor kernel's mask to the same form). Reads cu_seqlens back
// to the host: a debugging aid, not a hot path.
Tensor debug_mask_of_varlen(const KeepMasks& m, const Tensor& q, const Tensor& cu_q, const Tensor& cu_k, int64_t max_q,
                            int64_t max_k) {
  Tensor hq = cu_q.cpu(), hk = cu_k.cpu();
  const int32_t* cq = hq.data_ptr<int32_t>();
  const int32_t* ck = hk.data_ptr<int32_t>();
  const int64_t B = cu_q.numel() - 1, H = q.size(1);
  Tensor out = at::zeros({B, H, max_q, max_k}, q.options());
  Tensor shifts = at::arange(32, m.rows.options());
  for (int64_t b = 0; b < B; ++b) {
    const int64_t lq = cq[b + 1] - cq[b], lk = ck[b + 1] - ck[b];
    if (lq <= 0 || lk <= 0) continue;
    Tensor words = m.rows.slice(1, cq[b], cq[b + 1]);  // [H, lq, words]
    Tensor bits = at::bitwise_and(at::bitwise_right_shift(words.unsqueeze(-1), shifts), 1).reshape({H, lq, -1}).slice(2, 0, lk);
    out.select(0, b).slice(1, 0, lq).slice(2, 0, lk).copy_(bits);
  }
  return out;
}

// The packed operator pair with dropout.
struct VarlenDropoutResult {
  Tensor out, lse, seed, offset, debug;
};

VarlenDropoutResult varlen_forward_with_dropout(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& cu_q,
                                                const Tensor& cu_k, int64_t max_q, int64_t max_k, double dropout_p, bool causal,
                                                double scale, bool return_debug_mask = false) {
  TORCH_CHECK(dropout_p >= 0.0 && dropout_p < 1.0, "dropout_p must be inside [0, 1)");
  VarlenDropoutResult r;
  r.seed = at::empty({0}, q.options().dtype(at::kLong));
  r.offset = at::empty({0}, q.options().dtype(at::kLong));
  r.debug = at::empty({0}, q.options());
  if (dropout_p == 0.0) {
    std::tie(r.out, r.lse) = varlen_forward(q, k, v, cu_q, cu_k, max_q, max_k, causal, scale);
    return r;
  }
  check_varlen(q, k, v, cu_q, cu_k);
  auto [seed, offset] = draw_philox(q, (cu_q.numel() - 1) * q.size(1) * max_q * max_k);
  KeepMasks keep = make_keep_masks_varlen(q, k, cu_q, cu_k, max_q, max_k, dropout_p, seed, offset, causal);
  std::tie(r.out, r.lse) = varlen_forward(q, k, v, cu_q, cu_k, max_q, max_k, causal, scale, &keep);
  g_keep_cache.put(packed_keep_key(q, k, cu_q, max_q, max_k, dropout_p, seed, offset, causal), keep);
  if (return_debug_mask) r.debug = debug_mask_of_varlen(keep, q, cu_q, cu_k, max_q, max_k);
  r.seed = cpu_i64(seed);
  r.offset = cpu_i64(offset);
  return r;
}

std::tuple<Tensor, Tensor, Tensor> varlen_backward_with_dropout(const Tensor& grad_out, const Tensor& q, const Tensor& k,
                                                                const Tensor& v, const Tensor& out, const Tensor& lse,
                                                                const Tensor& cu_q, const Tensor& cu_k, int64_t max_q,
                                                                int64_t max_k, double dropout_p, bool causal,
                                                                const Tensor& philox_seed, const Tensor& philox_offset,
                                                                double scale) {
  TORCH_CHECK(dropout_p >= 0.0 && dropout_p < 1.0, "dropout_p must be inside [0, 1)");
  if (dropout_p == 0.0) return varlen_backward(grad_out, q, k, v, out, lse, cu_q, cu_k, max_q, max_k, causal, scale);
  TORCH_CHECK(philox_seed.numel() == 1 && philox_offset.numel() == 1,
              "dropout_p > 0 needs the philox_seed and philox_offset the forward operator returned");
  check_varlen(q, k, v, cu_q, cu_k);
  const uint64_t seed = static_cast<uint64_t>(philox_seed.item<int64_t>());
  const uint64_t offset = static_cast<uint64_t>(philox_offset.item<int64_t>());
  KeepMasks keep;
  if (!g_keep_cache.take(packed_keep_key(q, k, cu_q, max_q, max_k, dropout_p, seed, offset, causal), &keep))
    keep = make_keep_masks_varlen(q, k, cu_q, cu_k, max_q, max_k, dropout_p, seed, offset, causal);
  return varlen_backward(grad_out, q, k, v, out, lse, cu_q, cu_k, max_q, max_k, causal, scale, &keep);
}

// ------------------------------------------------ operators with the reference's schemas
std::tuple<Tensor, Tensor, Tensor, Tensor, int64_t, int64_t, Tensor, Tensor, Tensor> ref_sdpa_flash(
    const Tensor& q, const Tensor& k, const Tensor& v, double dropout_p, bool is_causal, bool return_debug_mask,
    c10::optional<double> scale) {
  C10_LOG_API_USAGE_ONCE("torch.sdpa.flash_attention");  // attention.cpp:67
  auto r = dense_forward_with_dropout(q, k, v, dropout_p, is_causal, return_debug_mask, scale_or_default(q, scale),
                                      /*allow_gqa=*/false);
  const int64_t B = q.size(0), Lq = q.size(2), Lk = k.size(2);
  auto iopt = q.options().dtype(at::kInt);
  Tensor cum_q = at::arange(0, (B + 1) * Lq, Lq, iopt);  // attention.cpp:109-119
  Tensor cum_k = at::arange(0, (B + 1) * Lk, Lk, iopt);
  // the reference hands back the logsumexp with its last dimension rounded up to 16 (FlashAttention_internal.cpp:261-265);
  // the padding holds zeros here and the backward operator cuts it off again (:374-375)
  Tensor lse = r.lse;
  const int64_t lq16 = (Lq + 15) / 16 * 16;
  if (lq16 != Lq) lse = at::constant_pad_nd(lse, {0, lq16 - Lq}, 0);
  return {r.out, lse, cum_q, cum_k, Lq, Lk, r.seed, r.offset, r.debug};
}

std::tuple<Tensor, Tensor, Tensor> ref_sdpa_flash_backward(const Tensor& grad_out, const Tensor& q, const Tensor& k,
                                                           const Tensor& v, const Tensor& out, const Tensor& lse,
                                                           const Tensor& cum_q, const Tensor& cum_k, int64_t max_q,
                                                           int64_t max_k, double dropout_p, bool is_causal,
                                                           const Tensor& philox_seed, const Tensor& philox_offset,
                                                           c10::optional<double> scale) {
  (void)cum_q; (void)cum_k; (void)max_q; (void)max_k;
  Tensor lse_q = lse;
  if (lse.dim() == 3 && lse.size(2) != q.size(2)) lse_q = lse.slice(2, 0, q.size(2)).contiguous();
  return dense_backward_with_dropout(grad_out, q, k, v, out, lse_q, dropout_p, is_causal, philox_seed, philox_offset,
                                     scale_or_default(q, scale));
}

std::tuple<Tensor, Tensor, Tensor, Tensor, Tensor> ref_flash_forward(const Tensor& q, const Tensor& k, const Tensor& v,
                                                                     const Tensor& cum_q, const Tensor& cum_k,
                                                                     int64_t max_q, int64_t max_k, double dropout_p,
                                                                     bool is_causal, bool return_debug_mask,
                                                                     c10::optional<double> scale) {
  auto r = varlen_forward_with_dropout(q, k, v, cum_q, cum_k, max_q, max_k, dropout_p, is_causal, scale_or_default(q, scale),
                                       return_debug_mask);
  return {r.out, r.lse, r.seed, r.offset, r.debug};
}

std::tuple<Tensor, Tensor, Tensor> ref_flash_backward(const Tensor& grad_out, const Tensor& q, const Tensor& k,
                                                      const Tensor& v, const Tensor& out, const Tensor& lse,
                                                      const Tensor& cum_q, const Tensor& cum_k, int64_t max_q,
                                                      int64_t max_k, double dropout_p, bool is_causal,
                                                      const Tensor& philox_seed, const Tensor& philox_offset,
                                                      c10::optional<double> scale) {
  return varlen_backward_with_dropout(grad_out, q, k, v, out, lse, cum_q, cum_k, max_q, max_k, dropout_p, is_causal,
                                      philox_seed, philox_offset, scale_or_default(q, scale));
}

// ------------------------------------ CUDA-key kernels for the installed torch's aten schemas
std::tuple<Tensor, Tensor, Tensor, Tensor, c10::SymInt, c10::SymInt, Tensor, Tensor, Tensor> aten_sdpa_flash(
    const Tensor& q, const Tensor& k, const Tensor& v, double dropout_p, bool is_causal, bool return_debug_mask,
    c10::optional<double> scale) {
  auto r = dense_forward_with_dropout(q, k, v, dropout_p, is_causal, return_debug_mask, scale_or_default(q, scale),
                                      /*allow_gqa=*/true);
  Tensor none = at::empty({0}, q.options().dtype(at::kInt));
  // the installed torch names the two slots rng_state and unused; its autograd hands both back to the backward
  return {r.out, r.lse, none, none, c10::SymInt(q.size(2)), c10::SymInt(k.size(2)), r.seed, r.offset, r.debug};
}

std::tuple<Tensor, Tensor, Tensor> aten_sdpa_flash_backward(const Tensor& grad_out, const Tensor& q, const Tensor& k,
                                                            const Tensor& v, const Tensor& out, const Tensor& lse,
                                                            const Tensor& cum_q, const Tensor& cum_k, c10::SymInt max_q,
                                                            c10::SymInt max_k, double dropout_p, bool is_causal,
                                                            const Tensor& philox_seed, const Tensor& philox_offset,
                                                            c10::optional<double> scale) {
  (void)cum_q; (void)cum_k; (void)max_q; (void)max_k;
  return dense_backward_with_dropout(grad_out, q, k, v, out, lse, dropout_p, is_causal, philox_seed, philox_offset,
                                     scale_or_default(q, scale));
}

void check_unsupported_kwargs(const c10::optional<c10::SymInt>& wl, const c10::optional<c10::SymInt>& wr, bool causal) {
  // a causal call arrives as window (-1, 0); anything else is a sliding window
  const bool left_ok = !wl.has_value() || wl->expect_int() < 0;
  const bool right_ok = !wr.has_value() || wr->expect_int() < 0 || (causal && wr->expect_int() == 0);
  TORCH_CHECK(left_ok && right_ok, "sliding-window attention (window_size_left/right) is not built in this library");
}

std::tuple<Tensor, Tensor, Tensor, Tensor, Tensor> aten_flash_forward(
    const Tensor& q, const Tensor& k, const Tensor& v, const c10::optional<Tensor>& cum_q, const c10::optional<Tensor>& cum_k,
    c10::SymInt max_q, c10::SymInt max_k, double dropout_p, bool is_causal, bool return_debug_mask,
    c10::optional<double> scale, c10::optional<c10::SymInt> window_size_left, c10::optional<c10::SymInt> window_size_right,
    const c10::optional<Tensor>& seqused_k, const c10::optional<Tensor>& alibi_slopes) {
  check_unsupported_kwargs(window_size_left, window_size_right, is_causal);
  TORCH_CHECK(!seqused_k.has_value() || !seqused_k->defined(), "seqused_k is not built in this library");
  TORCH_CHECK(!alibi_slopes.has_value() || !alibi_slopes->defined(), "alibi_slopes is not built in this library");
  const double sc = scale_or_default(q, scale);
  if (cum_q.has_value() && cum_q->defined()) {
    TORCH_CHECK(cum_k.has_value() && cum_k->defined(), "cum_seq_q and cum_seq_k must be given together");
    auto r = varlen_forward_with_dropout(q, k, v, *cum_q, *cum_k, max_q.expect_int(), max_k.expect_int(), dropout_p, is_causal, sc,
                                         return_debug_mask);
    return {r.out, r.lse, r.seed, r.offset, r.debug};
  }
  // dense form of the installed torch: [batch, seq, heads, head_dim]
  TORCH_CHECK(q.dim() == 4, "dense _flash_attention_forward expects [batch, seq_len, heads, head_dim]");
  auto r = dense_forward_with_dropout(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), dropout_p, is_causal,
                                      return_debug_mask, sc, /*allow_gqa=*/true);
  return {r.out.transpose(1, 2), r.lse, r.seed, r.offset, r.debug};
}

std::tuple<Tensor, Tensor, Tensor> aten_flash_backward(
    const Tensor& grad_out, const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& out, const Tensor& lse,
    const Tensor& cum_q, const Tensor& cum_k, c10::SymInt max_q, c10::SymInt max_k, double dropout_p, bool is_causal,
    const Tensor& rng_state, const Tensor& unused, c10::optional<double> scale, c10::optional<c10::SymInt> window_size_left,
    c10::optional<c10::SymInt> window_size_right) {
  check_unsupported_kwargs(window_size_left, window_size_right, is_causal);
  const double sc = scale_or_default(q, scale);
  if (cum_q.defined() && cum_q.numel() > 0) {
    return varlen_backward_with_dropout(grad_out, q, k, v, out, lse, cum_q, cum_k, max_q.expect_int(), max_k.expect_int(),
                                        dropout_p, is_causal, rng_state, unused, sc);
  }
  auto [dq, dk, dv] = dense_backward_with_dropout(grad_out.transpose(1, 2), q.transpose(1, 2), k.transpose(1, 2),
                                                  v.transpose(1, 2), out.transpose(1, 2), lse, dropout_p, is_causal, rng_state,
                                                  unused, sc);
  return {dq.transpose(1, 2), dk.transpose(1, 2), dv.transpose(1, 2)};
}

std::unique_ptr<torch::Library> g_aten_overrides;

void install_aten_overrides() {
  if (g_aten_overrides) return;
  g_aten_overrides = std::make_unique<torch::Library>(torch::Library::IMPL, "aten", c10::DispatchKey::CUDA, __FILE__, __LINE__);
  g_aten_overrides->impl("_scaled_dot_product_flash_attention", aten_sdpa_flash);
  g_aten_overrides->impl("_scaled_dot_product_flash_attention_backward", aten_sdpa_flash_backward);
  g_aten_overrides->impl("_flash_attention_forward", aten_flash_forward);
  g_aten_overrides->impl("_flash_attention_backward", aten_flash_backward);
}

void remove_aten_overrides() { g_aten_overrides.reset(); }

int64_t launch_count() { return static_cast<int64_t>(sdpa_b200_launch_count()); }

// ------------------------------------------------ autocast (aten/autocast_mode.cpp:147: lower_precision_fp)
// Under torch.autocast("cuda") fp32 query/key/value are cast to the autocast dtype (fp16 or bf16)
// before the kernels run, as the reference does for _scaled_dot_product_flash_attention.
Tensor to_autocast_dtype(const Tensor& t) {
  return at::autocast::cached_cast(at::autocast::get_autocast_dtype(at::kCUDA), t, c10::DeviceType::CUDA);
}

std::tuple<Tensor, Tensor, Tensor, Tensor, int64_t, int64_t, Tensor, Tensor, Tensor> autocast_sdpa_flash(
    const Tensor& q, const Tensor& k, const Tensor& v, double dropout_p, bool is_causal, bool return_debug_mask,
    c10::optional<double> scale) {
  c10::impl::ExcludeDispatchKeyGuard no_autocast(c10::DispatchKey::AutocastCUDA);
  static auto op = c10::Dispatcher::singleton()
                       .findSchemaOrThrow("b200_sdpa::_scaled_dot_product_flash_attention", "")
                       .typed<decltype(autocast_sdpa_flash)>();
  return op.call(to_autocast_dtype(q), to_autocast_dtype(k), to_autocast_dtype(v), dropout_p, is_causal,
                 return_debug_mask, scale);
}

std::tuple<Tensor, Tensor, Tensor, Tensor, Tensor> autocast_flash_forward(
    const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& cu_q, const Tensor& cu_k, int64_t max_q,
    int64_t max_k, double dropout_p, bool is_causal, bool return_debug_mask, c10::optional<double> scale) {
  c10::impl::ExcludeDispatchKeyGuard no_autocast(c10::DispatchKey::AutocastCUDA);
  static auto op = c10::Dispatcher::singleton()
                       .findSchemaOrThrow("b200_sdpa::_flash_attention_forward", "")
                       .typed<decltype(autocast_flash_forward)>();
  return op.call(to_autocast_dtype(q), to_autocast_dtype(k), to_autocast_dtype(v), cu_q, cu_k, max_q, max_k, dropout_p,
                 is_causal, return_debug_mask, scale);
}

}  // namespace

TORCH_LIBRARY(b200_sdpa, m) {
  // codegen/mlu_functions.yaml:1313-1316, verbatim argument lists
  m.def("_scaled_dot_product_flash_attention(Tensor query, Tensor key, Tensor value, float dropout_p=0.0, bool is_causal=False, "
        "bool return_debug_mask=False, *, float? scale=None) -> (Tensor ouput, Tensor logsumexp, Tensor cum_seq_q, "
        "Tensor cum_seq_k, int max_q, int max_k, Tensor philox_seed, Tensor philox_offset, Tensor debug_attn_mask)");
  m.def("_scaled_dot_product_flash_attention_backward(Tensor grad_out, Tensor query, Tensor key, Tensor value, Tensor out, "
        "Tensor logsumexp, Tensor cum_seq_q, Tensor cum_seq_k, int max_q, int max_k, float dropout_p, bool is_causal, "
        "Tensor philox_seed, Tensor philox_offset, *, float? scale=None) -> (Tensor grad_query, Tensor grad_key, Tensor grad_value)");
  m.def("_flash_attention_forward(Tensor query, Tensor key, Tensor value, Tensor cum_seq_q, Tensor cum_seq_k, int max_q, "
        "int max_k, float dropout_p, bool is_causal, bool return_debug_mask, *, float? scale=None) -> (Tensor output, "
        "Tensor softmax_logsumexp, Tensor philox_seed, Tensor philox_offset, Tensor debug_attn_mask)");
  m.def("_flash_attention_backward(Tensor grad_out, Tensor query, Tensor key, Tensor value, Tensor out, Tensor logsumexp, "
        "Tensor cum_seq_q, Tensor cum_seq_k, int max_q, int max_k, float dropout_p, bool is_causal, Tensor philox_seed, "
        "Tensor philox_offset, *, float? scale=None) -> (Tensor, Tensor, Tensor)");
  m.def("_install_aten_overrides() -> ()", install_aten_overrides);
  m.def("_remove_aten_overrides() -> ()", remove_aten_overrides);
  m.def("_launch_count() -> int", launch_count);
  // status word of `device` (-1 = current): 0, or 4 when a kernel gave up a bounded wait since the last read; clears it
  m.def("_device_status(int device=-1) -> int", device_status);
}

TORCH_LIBRARY_IMPL(b200_sdpa, AutocastCUDA, m) {
  m.impl("_scaled_dot_product_flash_attention", autocast_sdpa_flash);
  m.impl("_flash_attention_forward", autocast_flash_forward);
}

TORCH_LIBRARY_IMPL(b200_sdpa, CUDA, m) {
  m.impl("_scaled_dot_product_flash_attention", ref_sdpa_flash);
  m.impl("_scaled_dot_product_flash_attention_backward", ref_sdpa_flash_backward);
  m.impl("_flash_attention_forward", ref_flash_forward);
  m.impl("_flash_attention_backward", ref_flash_backward);
}
