// C-ABI glue: error channel, dispatch of coda_b200_attend, the step counter and the host-side
// selection-order helpers.
#include "coda_common.cuh"
#include "topk_order.h"
#include "tma_utils.cuh"
#include <stdarg.h>
#include <vector>

static thread_local char g_err[512] = "";

void coda_set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

extern "C" const char* coda_b200_last_error(void) { return g_err; }
extern "C" int coda_b200_version(void) { return 1; }

int coda_attend_generic(const coda_layer_cfg* cfg, const coda_state_ptrs* st, int32_t Lq,
                        const void* q, int64_t q_bs, int64_t q_rs,
                        const void* q_noise, int64_t qn_bs, int64_t qn_rs,
                        const float* lam, int64_t lam_bs, int64_t lam_rs,
                        const void* k_blk, int64_t kb_bs, int64_t kb_rs,
                        const void* v_blk, int64_t vb_bs, int64_t vb_rs,
                        const void* norm_w, void* out, int64_t out_bs, int64_t out_rs, cudaStream_t s);

extern "C" int coda_b200_attend(const coda_layer_cfg* cfg, const coda_state_ptrs* st, int32_t Lq,
                                const void* q, int64_t q_bs, int64_t q_rs,
                                const void* q_noise, int64_t qn_bs, int64_t qn_rs,
                                const float* lam, int64_t lam_bs, int64_t lam_rs,
                                const void* k_blk, int64_t kb_bs, int64_t kb_rs,
                                const void* v_blk, int64_t vb_bs, int64_t vb_rs,
                                const void* norm_w,
                                void* out, int64_t out_bs, int64_t out_rs,
                                coda_stream_t stream) {
  CODA_REQUIRE(coda_cfg_ok(cfg) && st, CODA_ERR_ARG, "attend: invalid layer configuration");
  CODA_REQUIRE(Lq > 0, CODA_ERR_ARG, "attend: Lq must be positive");
  CODA_REQUIRE(q && q_noise && lam && out && st->k_buf && st->v_buf && st->allowed, CODA_ERR_ARG, "attend: null pointer");
  CODA_REQUIRE((k_blk == nullptr) == (v_blk == nullptr), CODA_ERR_ARG, "attend: k_blk and v_blk must be given together");
  CODA_REQUIRE(!cfg->head_norm_full || norm_w, CODA_ERR_ARG, "attend: head-norm weight missing");
  return coda_attend_generic(cfg, st, Lq, q, q_bs, q_rs, q_noise, qn_bs, qn_rs, lam, lam_bs, lam_rs,
                             k_blk, kb_bs, kb_rs, v_blk, vb_bs, vb_rs, norm_w, out, out_bs, out_rs,
                             (cudaStream_t)stream);
}

__global__ void advance_steps_kernel(long long* ctr, long long n) { *ctr += n; }

extern "C" int coda_b200_advance_steps(int64_t* step_dev, int64_t n, coda_stream_t stream) {
  CODA_REQUIRE(step_dev, CODA_ERR_ARG, "advance_steps: null counter");
  advance_steps_kernel<<<1, 1, 0, (cudaStream_t)stream>>>((long long*)step_dev, (long long)n);
  CODA_CHECK_LAUNCH("advance_steps");
  return CODA_OK;
}

// Self-test of the bounded waits every pipelined kernel here is built on (tma::mbar_wait).  One CTA, two barriers
// that nobody ever arrives at.  Thread 0 waits on the first with `poll_limit` polls: the wait must give up, record
// its code in the status word and set the CTA's abort word.  Thread 32 waits on the second with the kernels' full
// limit: it must leave as soon as it sees the abort word, long before its own limit.  Nothing traps, nothing spins
// without a bound, and the context stays usable.
__global__ void selftest_wait_kernel(int poll_limit, int* status, int* report) {
  __shared__ uint64_t bars[2];
  __shared__ int s_abort;
  if (threadIdx.x == 0) {
    s_abort = 0;
    tma::mbar_init(&bars[0], 1);
    tma::mbar_init(&bars[1], 1);
    tma::fence_barrier_init();
  }
  __syncthreads();
  if (threadIdx.x == 0 || threadIdx.x == 32) {
    const int who = threadIdx.x / 32;
    const long long t0 = clock64();
    const bool ok = tma::mbar_wait(&bars[who], 0, status, 77 + who, &s_abort, who == 0 ? poll_limit : tma::WAIT_LIMIT);
    const long long dt = clock64() - t0;
    report[2 * who] = ok ? 1 : 0;
    report[2 * who + 1] = dt > 0x7fffffffLL ? 0x7fffffff : (int)dt;
  }
  __syncthreads();
  if (threadIdx.x == 0) report[4] = s_abort;
}

extern "C" int coda_b200_selftest_bounded_wait(int32_t poll_limit, int32_t* status, int32_t* report, coda_stream_t stream) {
  CODA_REQUIRE(status && report, CODA_ERR_ARG, "selftest_bounded_wait: null pointer");
  CODA_REQUIRE(poll_limit > 0 && poll_limit <= (1 << 16), CODA_ERR_ARG, "selftest_bounded_wait: poll_limit must be in 1..65536");
  selftest_wait_kernel<<<1, 64, 0, (cudaStream_t)stream>>>(poll_limit, status, report);
  CODA_CHECK_LAUNCH("selftest_bounded_wait");
  return CODA_OK;
}

template <typename V>
static int host_topk(const V* v, int n, int k, int largest, int sorted, int32_t* out) {
  if (!v || !out || n < 0 || k < 0 || k > n) { coda_set_error("host_topk: bad arguments"); return CODA_ERR_ARG; }
  std::vector<topk_order::Item<V>> q((size_t)(n > 0 ? n : 1));
  for (int j = 0; j < n; ++j) { q[j].v = v[j]; q[j].i = j; }
  if (largest) topk_order::topk_queue<V, true>(q.data(), n, k, sorted != 0);
  else topk_order::topk_queue<V, false>(q.data(), n, k, sorted != 0);
  for (int j = 0; j < k; ++j) out[j] = q[j].i;
  return CODA_OK;
}

extern "C" int coda_b200_host_topk_f32(const float* v, int32_t n, int32_t k, int32_t largest, int32_t sorted, int32_t* out) {
  return host_topk<float>(v, n, k, largest, sorted, out);
}
extern "C" int coda_b200_host_topk_i64(const int64_t* v, int32_t n, int32_t k, int32_t largest, int32_t sorted, int32_t* out) {
  return host_topk<long long>((const long long*)v, n, k, largest, sorted, out);
}

// The default decode step between its two GEMMs as ONE library call: coda_b200_step_write_fused, then
// coda_b200_decode_attend_prepared on the records it left.  Two launches as before; a caller that drives the step
// eagerly from an interpreter pays one foreign call per layer instead of two.
extern "C" int coda_b200_step_write_attend(const coda_layer_cfg* cfg, const coda_state_ptrs* st, coda_ring_pos rp,
                                           const void* k_raw, int64_t k_bs, const void* v_new, int64_t v_bs,
                                           const void* gate_logit, int64_t gate_bs, const float* inv_freq,
                                           const float* eta_logit,
                                           const void* q_raw, int64_t q_bs, const void* lam_logit, int64_t lam_bs,
                                           const void* cos_theta, const void* sin_theta, void* qrec,
                                           const void* norm_w, void* out, int64_t out_bs, int32_t* status,
                                           coda_stream_t stream) {
  const int rc = coda_b200_step_write_fused(cfg, st, rp, k_raw, k_bs, v_new, v_bs, gate_logit, gate_bs, inv_freq, eta_logit,
                                            q_raw, q_bs, lam_logit, lam_bs, cos_theta, sin_theta, qrec, stream);
  if (rc != CODA_OK) return rc;
  return coda_b200_decode_attend_prepared(cfg, st, qrec, norm_w, out, out_bs, status, stream);
}
