// torch custom-op layer over the C ABI of libcoda_b200.so (include/coda_b200.h).
//
// Registers torch.ops.coda_b200.* with a Tensor(x!) annotation on every tensor an op writes (state arena planes,
// outputs, scratch, status word), checks devices / dtypes / shapes with TORCH_CHECK (a c10::Error surfaces as a
// Python RuntimeError), picks up the current CUDA stream of the tensors' device under a CUDAGuard and forwards
// raw pointers.  The same role upstream's kernels/coda_diff_epilogue/torch-ext/torch_binding.cpp:72-139,203-213
// plays for its epilogue kernel.  No computation happens here and there is no CPU implementation: the ops are
// registered for the CUDA dispatch key only.
//
// A layer's hyper-parameters travel as two lists in the field order of struct coda_layer_cfg:
//   cfg_i (19 ints): B H Hkv Dh W Me Ms dtype angle_dtype rope_interleaved head_norm_full mask_unused gated
//                    refresh_on_hit overwrite_on_insert Te Ts active_exact active_summary
//   cfg_f (6 floats): tau_gate_exact tau_gate_summary tau_match tau_novel eps energy_scale
// Activations may be row-strided views (slices of a fused projection); the innermost (feature) dimension must be
// dense.  State tensors must be contiguous.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>
#include <torch/types.h>

#include <cstdarg>
#include <cstdio>
#include <optional>
#include <string>

#include "coda_b200.h"

namespace {

using torch::Tensor;
using OptTensor = std::optional<Tensor>;

// Error texts are composed with snprintf and handed to TORCH_CHECK as one string: numbers never go through the
// C++ stream formatting of whichever libstdc++ copy happens to be first in the process's symbol scope.
std::string text(const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  return std::string(buf);
}

static_assert(sizeof(coda_layer_cfg) == 25 * 4, "coda_layer_cfg is 19 int32 fields followed by 6 floats");

coda_layer_cfg make_cfg(c10::IntArrayRef ci, c10::ArrayRef<double> cf) {
  TORCH_CHECK(ci.size() == 19, text("cfg_i must hold the 19 integer fields of coda_layer_cfg, got %zu", ci.size()));
  TORCH_CHECK(cf.size() == 6, text("cfg_f must hold the 6 float fields of coda_layer_cfg, got %zu", cf.size()));
  coda_layer_cfg c;
  int32_t* ip = &c.B;
  for (int i = 0; i < 19; ++i) ip[i] = static_cast<int32_t>(ci[i]);
  float* fp = &c.tau_gate_exact;
  for (int i = 0; i < 6; ++i) fp[i] = static_cast<float>(cf[i]);
  return c;
}

at::ScalarType model_dtype(const coda_layer_cfg& c) { return c.dtype == CODA_BF16 ? at::kBFloat16 : at::kFloat; }

void on_device(const Tensor& t, const Tensor& like, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor (this library has no CPU path)");
  TORCH_CHECK(t.device() == like.device(), text("%s is on cuda:%d but the state is on cuda:%d", name, int(t.device().index()), int(like.device().index())));
}

void dense_rows(const Tensor& t, const char* name) {
  TORCH_CHECK(t.dim() >= 1 && t.stride(-1) == 1, name, " must be dense along its last dimension");
}

void failed(int rc, const char* what) {
  TORCH_CHECK(rc == 0, text("%s rejected the call (%d): %s", what, rc, coda_b200_last_error()));
}

// The state planes of one layer, validated against the configuration (absent tensors: nullptr).
coda_state_ptrs bind_state(const coda_layer_cfg& c, const Tensor& k_buf, const Tensor& v_buf, const Tensor& allowed,
                           const Tensor* g_recent, const Tensor* mem_last_exact, const Tensor* exact_v_norm,
                           const Tensor* sum_lf_k_norm) {
  const int64_t Lbuf = int64_t(c.W) + c.Me + c.Ms;
  const auto dt = model_dtype(c);
  TORCH_CHECK(k_buf.is_cuda(), "k_buf must be a CUDA tensor (this library has no CPU path)");
  on_device(v_buf, k_buf, "v_buf");
  on_device(allowed, k_buf, "allowed");
  TORCH_CHECK(k_buf.scalar_type() == dt && v_buf.scalar_type() == dt, "k_buf / v_buf must have the configuration's dtype");
  const bool shape_ok = k_buf.dim() == 4 && k_buf.size(0) == c.B && k_buf.size(1) == c.Hkv && k_buf.size(2) == Lbuf &&
                        k_buf.size(3) == c.Dh && v_buf.dim() == 4 && v_buf.size(0) == c.B && v_buf.size(1) == c.Hkv &&
                        v_buf.size(2) == Lbuf && v_buf.size(3) == c.Dh;
  TORCH_CHECK(shape_ok, text("k_buf / v_buf must be [B, Hkv, W+Me+Ms, Dh] = [%d, %d, %lld, %d]", c.B, c.Hkv, (long long)Lbuf, c.Dh));
  TORCH_CHECK(k_buf.is_contiguous() && v_buf.is_contiguous() && allowed.is_contiguous(), "state tensors must be contiguous");
  TORCH_CHECK(allowed.element_size() == 1 && allowed.numel() == c.B * Lbuf, "allowed must be [B, W+Me+Ms] of 1-byte elements");
  coda_state_ptrs p;
  p.k_buf = k_buf.data_ptr();
  p.v_buf = v_buf.data_ptr();
  p.allowed = static_cast<uint8_t*>(allowed.data_ptr());
  p.g_recent = nullptr;
  p.mem_last_exact = nullptr;
  p.exact_v_norm = nullptr;
  p.sum_lf_k_norm = nullptr;
  p.events = nullptr;
  if (g_recent != nullptr) {
    on_device(*g_recent, k_buf, "g_recent");
    TORCH_CHECK(g_recent->scalar_type() == at::kFloat && g_recent->is_contiguous() && g_recent->numel() == int64_t(c.B) * c.W,
                "g_recent must be a contiguous float32 [B, W]");
    p.g_recent = g_recent->data_ptr<float>();
  }
  if (mem_last_exact != nullptr && mem_last_exact->numel() > 0) {
    on_device(*mem_last_exact, k_buf, "mem_last_exact");
    TORCH_CHECK(mem_last_exact->scalar_type() == at::kLong && mem_last_exact->is_contiguous() &&
                    mem_last_exact->numel() == int64_t(c.B) * c.Me, "mem_last_exact must be a contiguous int64 [B, Me]");
    p.mem_last_exact = mem_last_exact->data_ptr<int64_t>();
  }
  if (exact_v_norm != nullptr) {
    on_device(*exact_v_norm, k_buf, "exact_v_norm");
    TORCH_CHECK(exact_v_norm->scalar_type() == dt && exact_v_norm->is_contiguous() &&
                    exact_v_norm->numel() == int64_t(c.B) * c.Hkv * c.Me * c.Dh, "exact_v_norm must be [B, Hkv, Me, Dh] in the model dtype");
    p.exact_v_norm = exact_v_norm->data_ptr();
  }
  if (sum_lf_k_norm != nullptr) {
    on_device(*sum_lf_k_norm, k_buf, "sum_lf_k_norm");
    TORCH_CHECK(sum_lf_k_norm->scalar_type() == dt && sum_lf_k_norm->is_contiguous() &&
                    sum_lf_k_norm->numel() == int64_t(c.B) * c.Hkv * c.Ms * (c.Dh - c.Dh / 2),
                "sum_lf_k_norm must be [B, Hkv, Ms, Dh/2] in the model dtype");
    p.sum_lf_k_norm = sum_lf_k_norm->data_ptr();
  }
  return p;
}

const Tensor* opt_ref(const OptTensor& t) { return t.has_value() ? &t.value() : nullptr; }

void check_act(const Tensor& t, const Tensor& like, const coda_layer_cfg& c, int64_t rows, int64_t feat, const char* name) {
  on_device(t, like, name);
  dense_rows(t, name);
  TORCH_CHECK(t.scalar_type() == model_dtype(c), name, " must have the configuration's dtype");
  TORCH_CHECK(t.dim() == 3 && t.size(0) == c.B && t.size(1) == rows && t.size(2) == feat,
              text("%s must be [%d, %lld, %lld] (got %lld dimensions)", name, c.B, (long long)rows, (long long)feat, (long long)t.dim()));
}

const void* opt_ptr(const OptTensor& t) { return t ? t->data_ptr() : nullptr; }

// ---------------------------------------------------------------------------------------------------------------
void prep(Tensor& q, const OptTensor& k, Tensor& q_noise, const Tensor& lam_logit, Tensor& lam,
          const OptTensor& gate_logit, const OptTensor& gate, const Tensor& inv_freq, const Tensor& cos_theta,
          const Tensor& sin_theta, int64_t pos, c10::IntArrayRef ci, c10::ArrayRef<double> cf) {
  auto c = make_cfg(ci, cf);
  TORCH_CHECK(q.is_cuda(), "q must be a CUDA tensor (this library has no CPU path)");
  TORCH_CHECK(q.dim() == 3, "q must be [B, L, H*Dh]");
  const int64_t L = q.size(1);
  check_act(q, q, c, L, int64_t(c.H) * c.Dh, "q");
  if (k) check_act(*k, q, c, L, int64_t(c.Hkv) * c.Dh, "k");
  check_act(q_noise, q, c, L, int64_t(c.H) * c.Dh, "q_noise");
  TORCH_CHECK(q_noise.is_contiguous(), "q_noise must be contiguous");
  check_act(lam_logit, q, c, L, c.H, "lam_logit");
  on_device(lam, q, "lam");
  TORCH_CHECK(lam.scalar_type() == at::kFloat && lam.is_contiguous() && lam.numel() == c.B * L * c.H, "lam must be a contiguous float32 [B, L, H]");
  // With the "none" write policy there are no gate logits and `gate` is filled with ones.
  TORCH_CHECK(!gate_logit || gate, "gate_logit given without a gate output");
  TORCH_CHECK(!(c.gated && gate && !gate_logit), "a gated write policy needs gate logits to fill gate");
  if (gate_logit) {
    on_device(*gate_logit, q, "gate_logit");
    TORCH_CHECK(gate_logit->scalar_type() == model_dtype(c) && gate_logit->dim() == 3 && gate_logit->size(0) == c.B &&
                    gate_logit->size(1) == L && gate_logit->size(2) == 1, "gate_logit must be [B, L, 1] in the model dtype");
  }
  if (gate) {
    on_device(*gate, q, "gate");
    TORCH_CHECK(gate->scalar_type() == at::kFloat && gate->is_contiguous() && gate->numel() == c.B * L, "gate must be a contiguous float32 [B, L]");
  }
  on_device(inv_freq, q, "inv_freq");
  TORCH_CHECK(inv_freq.scalar_type() == at::kFloat && inv_freq.numel() == c.Dh / 2, "inv_freq must be float32 [Dh/2]");
  TORCH_CHECK(cos_theta.numel() == int64_t(c.H) * (c.Dh / 2) && sin_theta.numel() == cos_theta.numel(), "cos/sin theta must be [H, Dh/2]");
  const at::cuda::CUDAGuard guard(q.device());
  coda_ring_pos rp{pos, 0, 0, nullptr};
  failed(coda_b200_prep(&c, int32_t(L), rp, q.data_ptr(), q.stride(0), q.stride(1), k ? k->data_ptr() : nullptr,
                        k ? k->stride(0) : 0, k ? k->stride(1) : 0, q_noise.data_ptr(), lam_logit.data_ptr(),
                        lam_logit.stride(0), lam_logit.stride(1), lam.data_ptr<float>(), opt_ptr(gate_logit),
                        gate_logit ? gate_logit->stride(0) : 0, gate_logit ? gate_logit->stride(1) : 0,
                        gate ? gate->data_ptr<float>() : nullptr, inv_freq.data_ptr<float>(), cos_theta.data_ptr(),
                        sin_theta.data_ptr(), at::cuda::getCurrentCUDAStream()),
         "coda_b200_prep");
}

void attend(Tensor& out, const Tensor& k_buf, const Tensor& v_buf, const Tensor& allowed, const Tensor& q,
            const Tensor& q_noise, const Tensor& lam, const OptTensor& k_blk, const OptTensor& v_blk,
            const OptTensor& norm_w, c10::IntArrayRef ci, c10::ArrayRef<double> cf) {
  auto c = make_cfg(ci, cf);
  const coda_state_ptrs st = bind_state(c, k_buf, v_buf, allowed, nullptr, nullptr, nullptr, nullptr);
  TORCH_CHECK(q.dim() == 3, "q must be [B, Lq, H*Dh]");
  const int64_t Lq = q.size(1);
  check_act(q, k_buf, c, Lq, int64_t(c.H) * c.Dh, "q");
  check_act(q_noise, k_buf, c, Lq, int64_t(c.H) * c.Dh, "q_noise");
  check_act(out, k_buf, c, Lq, int64_t(c.H) * c.Dh, "out");
  on_device(lam, k_buf, "lam");
  TORCH_CHECK(lam.scalar_type() == at::kFloat && lam.dim() == 3 && lam.size(1) == Lq && lam.size(2) == c.H && lam.stride(2) == 1, "lam must be float32 [B, Lq, H]");
  TORCH_CHECK(bool(k_blk) == bool(v_blk), "k_blk and v_blk come together");
  if (k_blk) {
    check_act(*k_blk, k_buf, c, Lq, int64_t(c.Hkv) * c.Dh, "k_blk");
    check_act(*v_blk, k_buf, c, Lq, int64_t(c.Hkv) * c.Dh, "v_blk");
  }
  if (norm_w) TORCH_CHECK(norm_w->is_cuda() && norm_w->numel() == c.Dh && norm_w->scalar_type() == model_dtype(c), "norm_w must be [Dh] in the model dtype");
  const at::cuda::CUDAGuard guard(k_buf.device());
  failed(coda_b200_attend(&c, &st, int32_t(Lq), q.data_ptr(), q.stride(0), q.stride(1), q_noise.data_ptr(),
                          q_noise.stride(0), q_noise.stride(1), lam.data_ptr<float>(), lam.stride(0), lam.stride(1),
                          opt_ptr(k_blk), k_blk ? k_blk->stride(0) : 0, k_blk ? k_blk->stride(1) : 0, opt_ptr(v_blk),
                          v_blk ? v_blk->stride(0) : 0, v_blk ? v_blk->stride(1) : 0, opt_ptr(norm_w), out.data_ptr(),
                          out.stride(0), out.stride(1), at::cuda::getCurrentCUDAStream()),
         "coda_b200_attend");
}

void decode_attend(Tensor& out, const Tensor& k_buf, const Tensor& v_buf, const Tensor& allowed, const Tensor& q_raw,
                   const Tensor& lam_logit, const Tensor& inv_freq, const Tensor& cos_theta, const Tensor& sin_theta,
                   const OptTensor& norm_w, Tensor& qrec, Tensor& status, int64_t pos, int64_t recent_idx,
                   int64_t recent_filled, int64_t token_already_written, c10::IntArrayRef ci, c10::ArrayRef<double> cf) {
  auto c = make_cfg(ci, cf);
  TORCH_CHECK(coda_b200_decode_attend_supported(&c), "decode_attend: this configuration is not covered by the fused decode kernel "
              "(needs bfloat16, head_dim 64 or 128, at most 8 query heads per KV head); use attend");
  const coda_state_ptrs st = bind_state(c, k_buf, v_buf, allowed, nullptr, nullptr, nullptr, nullptr);
  check_act(q_raw, k_buf, c, 1, int64_t(c.H) * c.Dh, "q_raw");
  check_act(lam_logit, k_buf, c, 1, c.H, "lam_logit");
  check_act(out, k_buf, c, 1, int64_t(c.H) * c.Dh, "out");
  on_device(qrec, k_buf, "qrec");
  on_device(status, k_buf, "status");
  TORCH_CHECK(qrec.is_contiguous() && int64_t(qrec.numel() * qrec.element_size()) >= coda_b200_decode_record_bytes(&c) &&
                  reinterpret_cast<uintptr_t>(qrec.data_ptr()) % 16 == 0,
              text("qrec must be a contiguous, 16-byte aligned buffer of at least %lld bytes", (long long)coda_b200_decode_record_bytes(&c)));
  TORCH_CHECK(status.scalar_type() == at::kInt && status.numel() >= 1, "status must be an int32 tensor");
  TORCH_CHECK(inv_freq.is_cuda() && inv_freq.scalar_type() == at::kFloat && inv_freq.numel() == c.Dh / 2, "inv_freq must be float32 [Dh/2]");
  TORCH_CHECK(cos_theta.numel() == int64_t(c.H) * (c.Dh / 2) && sin_theta.numel() == cos_theta.numel(), "cos/sin theta must be [H, Dh/2]");
  const at::cuda::CUDAGuard guard(k_buf.device());
  coda_ring_pos rp{pos, int32_t(recent_idx), int32_t(recent_filled), nullptr};
  failed(coda_b200_decode_attend(&c, &st, rp, int32_t(token_already_written), q_raw.data_ptr(), q_raw.stride(0),
                                 lam_logit.data_ptr(), lam_logit.stride(0), inv_freq.data_ptr<float>(), cos_theta.data_ptr(),
                                 sin_theta.data_ptr(), opt_ptr(norm_w), qrec.data_ptr(), out.data_ptr(), out.stride(0),
                                 status.data_ptr<int32_t>(), at::cuda::getCurrentCUDAStream()),
         "coda_b200_decode_attend");
}

void prefill_attend(Tensor& out, const Tensor& k_buf, const Tensor& v_buf, const Tensor& allowed, const Tensor& q,
                    const Tensor& q_noise, const Tensor& lam, const Tensor& k_seq, const Tensor& v_seq,
                    const OptTensor& norm_w, Tensor& status, int64_t t0, int64_t blk, c10::IntArrayRef ci,
                    c10::ArrayRef<double> cf) {
  auto c = make_cfg(ci, cf);
  TORCH_CHECK(coda_b200_prefill_attend_supported(&c), "prefill_attend: this configuration is not covered by the tensor-core "
              "prefill kernel (needs bfloat16 and head_dim 64 or 128); use attend");
  const coda_state_ptrs st = bind_state(c, k_buf, v_buf, allowed, nullptr, nullptr, nullptr, nullptr);
  TORCH_CHECK(q.dim() == 3, "q must be [B, L, H*Dh]");
  const int64_t L = q.size(1);
  TORCH_CHECK(t0 >= 0 && blk > 0 && t0 + blk <= L, "rows t0 .. t0+blk must lie inside the chunk");
  check_act(q, k_buf, c, L, int64_t(c.H) * c.Dh, "q");
  check_act(q_noise, k_buf, c, L, int64_t(c.H) * c.Dh, "q_noise");
  check_act(k_seq, k_buf, c, L, int64_t(c.Hkv) * c.Dh, "k_seq");
  check_act(v_seq, k_buf, c, L, int64_t(c.Hkv) * c.Dh, "v_seq");
  check_act(out, k_buf, c, L, int64_t(c.H) * c.Dh, "out");
  for (const Tensor* t : {&q, &q_noise, &k_seq, &v_seq})
    TORCH_CHECK(reinterpret_cast<uintptr_t>(t->data_ptr()) % 16 == 0 && t->stride(0) % 8 == 0 && t->stride(1) % 8 == 0,
                "q / q_noise / k_seq / v_seq must be 16-byte aligned with strides that are multiples of 8 elements (TMA)");
  TORCH_CHECK(lam.is_cuda() && lam.scalar_type() == at::kFloat && lam.dim() == 3 && lam.size(1) == L && lam.stride(2) == 1, "lam must be float32 [B, L, H]");
  on_device(status, k_buf, "status");
  TORCH_CHECK(status.scalar_type() == at::kInt && status.numel() >= 1, "status must be an int32 tensor");
  const at::cuda::CUDAGuard guard(k_buf.device());
  failed(coda_b200_prefill_attend(&c, &st, int32_t(L), int32_t(t0), int32_t(blk), q.data_ptr(), q.stride(0), q.stride(1),
                                  q_noise.data_ptr(), q_noise.stride(0), q_noise.stride(1), lam.data_ptr<float>(),
                                  lam.stride(0), lam.stride(1), k_seq.data_ptr(), k_seq.stride(0), k_seq.stride(1),
                                  v_seq.data_ptr(), v_seq.stride(0), v_seq.stride(1), opt_ptr(norm_w), out.data_ptr(),
                                  out.stride(0), out.stride(1), status.data_ptr<int32_t>(), at::cuda::getCurrentCUDAStream()),
         "coda_b200_prefill_attend");
}

void step_write(Tensor& k_buf, Tensor& v_buf, Tensor& allowed, Tensor& g_recent, Tensor& mem_last_exact,
                const OptTensor& exact_v_norm, const OptTensor& sum_lf_k_norm, const Tensor& k_new, const Tensor& v_new,
                const Tensor& gate, const Tensor& eta_logit, int64_t pos, int64_t recent_idx, int64_t recent_filled,
                c10::IntArrayRef ci, c10::ArrayRef<double> cf) {
  auto c = make_cfg(ci, cf);
  const coda_state_ptrs st = bind_state(c, k_buf, v_buf, allowed, &g_recent, &mem_last_exact, opt_ref(exact_v_norm), opt_ref(sum_lf_k_norm));
  check_act(k_new, k_buf, c, 1, int64_t(c.Hkv) * c.Dh, "k_new");
  check_act(v_new, k_buf, c, 1, int64_t(c.Hkv) * c.Dh, "v_new");
  on_device(gate, k_buf, "gate");
  on_device(eta_logit, k_buf, "eta_logit");
  TORCH_CHECK(gate.scalar_type() == at::kFloat && gate.is_contiguous() && gate.numel() == c.B, "gate must be a contiguous float32 [B]");
  TORCH_CHECK(eta_logit.scalar_type() == at::kFloat && eta_logit.numel() == c.Hkv, "eta_logit must be float32 [Hkv]");
  TORCH_CHECK(recent_filled >= 0 && recent_filled <= c.W && recent_idx >= 0 && recent_idx < c.W, "ring scalars out of range");
  const at::cuda::CUDAGuard guard(k_buf.device());
  coda_ring_pos rp{pos, int32_t(recent_idx), int32_t(recent_filled), nullptr};
  failed(coda_b200_step_write(&c, &st, rp, k_new.data_ptr(), k_new.stride(0), v_new.data_ptr(), v_new.stride(0),
                              gate.data_ptr<float>(), eta_logit.data_ptr<float>(), at::cuda::getCurrentCUDAStream()),
         "coda_b200_step_write");
}

void select_candidates(Tensor& cand, const Tensor& gates, int64_t ring_fill0, int64_t L, int64_t block,
                       c10::IntArrayRef ci, c10::ArrayRef<double> cf) {
  auto c = make_cfg(ci, cf);
  TORCH_CHECK(gates.is_cuda() && cand.is_cuda() && gates.device() == cand.device(), "gates and cand must be CUDA tensors on one device");
  TORCH_CHECK(gates.scalar_type() == at::kFloat && gates.dim() == 2 && gates.size(0) == c.B && gates.size(1) == ring_fill0 + L &&
                  gates.stride(1) == 1, "gates must be float32 [B, ring_fill0 + L]");
  TORCH_CHECK(block > 0 && L > 0, "L and block must be positive");
  const int64_t nblk = (L + block - 1) / block;
  TORCH_CHECK(cand.scalar_type() == at::kInt && cand.dim() == 3 && cand.is_contiguous() && cand.size(0) == c.B && cand.size(1) == nblk,
              "cand must be a contiguous int32 [B, ceil(L/block), T]");
  const at::cuda::CUDAGuard guard(gates.device());
  failed(coda_b200_select_candidates(&c, gates.data_ptr<float>(), gates.stride(0), int32_t(ring_fill0), int32_t(L),
                                     int32_t(block), cand.data_ptr<int32_t>(), int32_t(cand.size(2)),
                                     at::cuda::getCurrentCUDAStream()),
         "coda_b200_select_candidates");
}

void route_block(Tensor& k_buf, Tensor& v_buf, Tensor& allowed, Tensor& g_recent, Tensor& mem_last_exact,
                 const OptTensor& exact_v_norm, const OptTensor& sum_lf_k_norm, const Tensor& k_blk, const Tensor& v_blk,
                 const Tensor& gates, const Tensor& cand, const Tensor& eta_logit, Tensor& scratch, int64_t ring_fill,
                 int64_t pos0, int64_t gate_ev0, c10::IntArrayRef ci, c10::ArrayRef<double> cf) {
  auto c = make_cfg(ci, cf);
  const coda_state_ptrs st = bind_state(c, k_buf, v_buf, allowed, &g_recent, &mem_last_exact, opt_ref(exact_v_norm), opt_ref(sum_lf_k_norm));
  TORCH_CHECK(k_blk.dim() == 3, "k_blk must be [B, blk, Hkv*Dh]");
  const int64_t blk = k_blk.size(1);
  check_act(k_blk, k_buf, c, blk, int64_t(c.Hkv) * c.Dh, "k_blk");
  check_act(v_blk, k_buf, c, blk, int64_t(c.Hkv) * c.Dh, "v_blk");
  on_device(gates, k_buf, "gates");
  on_device(cand, k_buf, "cand");
  on_device(eta_logit, k_buf, "eta_logit");
  on_device(scratch, k_buf, "scratch");
  TORCH_CHECK(gates.scalar_type() == at::kFloat && gates.dim() == 2 && gates.size(0) == c.B && gates.stride(1) == 1, "gates must be float32 [B, n]");
  TORCH_CHECK(cand.scalar_type() == at::kInt && cand.dim() == 2 && cand.size(0) == c.B && cand.stride(1) == 1, "cand must be int32 [B, T]");
  TORCH_CHECK(eta_logit.scalar_type() == at::kFloat && eta_logit.numel() == c.Hkv, "eta_logit must be float32 [Hkv]");
  TORCH_CHECK(ring_fill >= 0 && ring_fill <= c.W, "ring_fill out of range");
  TORCH_CHECK(scratch.is_contiguous() && int64_t(scratch.numel() * scratch.element_size()) >= coda_b200_route_scratch_bytes(&c),
              text("scratch must hold at least %lld bytes", (long long)coda_b200_route_scratch_bytes(&c)));
  const at::cuda::CUDAGuard guard(k_buf.device());
  failed(coda_b200_route_block(&c, &st, int32_t(ring_fill), int32_t(blk), pos0, k_blk.data_ptr(), k_blk.stride(0),
                               k_blk.stride(1), v_blk.data_ptr(), v_blk.stride(0), v_blk.stride(1), gates.data_ptr<float>(),
                               gates.stride(0), gate_ev0, cand.data_ptr<int32_t>(), cand.stride(0),
                               eta_logit.data_ptr<float>(), scratch.data_ptr(), at::cuda::getCurrentCUDAStream()),
         "coda_b200_route_block");
}

}  // namespace

TORCH_LIBRARY(coda_b200, m) {
  m.def("prep(Tensor(a!) q, Tensor(b!)? k, Tensor(c!) q_noise, Tensor lam_logit, Tensor(d!) lam, Tensor? gate_logit, "
        "Tensor(e!)? gate, Tensor inv_freq, Tensor cos_theta, Tensor sin_theta, int pos, int[] cfg_i, float[] cfg_f) -> ()");
  m.def("attend(Tensor(a!) out, Tensor k_buf, Tensor v_buf, Tensor allowed, Tensor q, Tensor q_noise, Tensor lam, "
        "Tensor? k_blk, Tensor? v_blk, Tensor? norm_w, int[] cfg_i, float[] cfg_f) -> ()");
  m.def("decode_attend(Tensor(a!) out, Tensor k_buf, Tensor v_buf, Tensor allowed, Tensor q_raw, Tensor lam_logit, "
        "Tensor inv_freq, Tensor cos_theta, Tensor sin_theta, Tensor? norm_w, Tensor(b!) qrec, Tensor(c!) status, int pos, "
        "int recent_idx, int recent_filled, int token_already_written, int[] cfg_i, float[] cfg_f) -> ()");
  m.def("prefill_attend(Tensor(a!) out, Tensor k_buf, Tensor v_buf, Tensor allowed, Tensor q, Tensor q_noise, Tensor lam, "
        "Tensor k_seq, Tensor v_seq, Tensor? norm_w, Tensor(b!) status, int t0, int blk, int[] cfg_i, float[] cfg_f) -> ()");
  m.def("step_write(Tensor(a!) k_buf, Tensor(b!) v_buf, Tensor(c!) allowed, Tensor(d!) g_recent, Tensor(e!) mem_last_exact, "
        "Tensor(f!)? exact_v_norm, Tensor(g!)? sum_lf_k_norm, Tensor k_new, Tensor v_new, Tensor gate, Tensor eta_logit, "
        "int pos, int recent_idx, int recent_filled, int[] cfg_i, float[] cfg_f) -> ()");
  m.def("select_candidates(Tensor(a!) cand, Tensor gates, int ring_fill0, int L, int block, int[] cfg_i, float[] cfg_f) -> ()");
  m.def("route_block(Tensor(a!) k_buf, Tensor(b!) v_buf, Tensor(c!) allowed, Tensor(d!) g_recent, Tensor(e!) mem_last_exact, "
        "Tensor(f!)? exact_v_norm, Tensor(g!)? sum_lf_k_norm, Tensor k_blk, Tensor v_blk, Tensor gates, Tensor cand, "
        "Tensor eta_logit, Tensor(h!) scratch, int ring_fill, int pos0, int gate_ev0, int[] cfg_i, float[] cfg_f) -> ()");
}

TORCH_LIBRARY_IMPL(coda_b200, CUDA, m) {
  m.impl("prep", &prep);
  m.impl("attend", &attend);
  m.impl("decode_attend", &decode_attend);
  m.impl("prefill_attend", &prefill_attend);
  m.impl("step_write", &step_write);
  m.impl("select_candidates", &select_candidates);
  m.impl("route_block", &route_block);
}
