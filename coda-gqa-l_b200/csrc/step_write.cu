// Decode-step cache write: ring FIFO + routing of the evicted token into the exact and summary banks.
// One CTA per state.  Reads the two unit-norm routing caches once, rewrites at most one slot per bank.
#include "coda_common.cuh"
#include "tma_utils.cuh"
#include "bank_score.cuh"

struct StepParams {
  coda_layer_cfg c;
  coda_state_ptrs st;
  coda_ring_pos rp;
  const void* k_new; long long k_bs;
  const void* v_new; long long v_bs;
  const float* gate; const float* eta_logit;
  // raw mode: k_new is the un-rotated key projection and the gate comes as a logit; RoPE and the
  // sigmoid are applied here (saves the separate post-processing launch on the decode path)
  int raw; const float* inv_freq; const void* gate_logit; long long gate_bs;
  // stage != 0: both routing caches of the state (contiguous per state) are brought into shared memory by
  // two bulk copies issued at kernel entry, so that scoring does not wait on one global round trip per row
  int stage; int stage_off;       // byte offset of the staged caches inside dynamic shared memory
  int* status;
};

// RoPE'd element d of head-row `row` (Dh values, un-rotated) given cos/sin tables of Dh/2 entries.
template <typename T>
__device__ __forceinline__ float rope_elem(const T* row, int d, int Dh, int interleaved, const float* cs, const float* sn) {
  const int half = Dh >> 1;
  if (interleaved) {                                   // primitives.py:99-106
    const int i = d >> 1;
    const float xe = El<T>::ld(row + 2 * i), xo = El<T>::ld(row + 2 * i + 1);
    return (d & 1) ? t_add<T>(t_mul<T>(xe, sn[i]), t_mul<T>(xo, cs[i])) : t_sub<T>(t_mul<T>(xe, cs[i]), t_mul<T>(xo, sn[i]));
  }
  const int i = d < half ? d : d - half;               // primitives.py:108-113
  const float x1 = El<T>::ld(row + i), x2 = El<T>::ld(row + i + half);
  return d < half ? t_add<T>(t_mul<T>(x1, cs[i]), t_mul<T>(-x2, sn[i])) : t_add<T>(t_mul<T>(x2, cs[i]), t_mul<T>(x1, sn[i]));
}

template <typename T>
__global__ void __launch_bounds__(512) step_write_kernel(StepParams p) {
  extern __shared__ float sm[];
  const coda_layer_cfg& c = p.c;
  const int b = blockIdx.x, tid = threadIdx.x, NT = blockDim.x;
  const int lane = tid & 31, warp = tid >> 5, NW = NT >> 5;
  const int W = c.W, Me = c.Me, Ms = c.Ms, Hkv = c.Hkv, Dh = c.Dh;
  const int Lbuf = W + Me + Ms, HD = Hkv * Dh, lf = Dh / 2, lfd = Dh - lf;
  const RingNow r = ring_now(p.rp, W);

  T* kb = (T*)p.st.k_buf + (long long)b * Hkv * Lbuf * Dh;
  T* vb = (T*)p.st.v_buf + (long long)b * Hkv * Lbuf * Dh;
  uint8_t* al = p.st.allowed + (long long)b * Lbuf;
  float* gr = p.st.g_recent + (long long)b * W;
  const T* kn = (const T*)p.k_new + (long long)b * p.k_bs;
  const T* vn = (const T*)p.v_new + (long long)b * p.v_bs;
  float g_new;
  float* cs = sm + 3 * HD + Hkv * lfd + (Me > Ms ? Me : Ms) + 1;   // [Dh/2] cos, then [Dh/2] sin (raw mode)
  float* sn = cs + Dh / 2;
  if (p.raw) {
    g_new = 1.0f;
    if (c.gated) g_new = t_sigmoid<T>(El<T>::ld((const T*)p.gate_logit + (long long)b * p.gate_bs));
    const bool abf = c.angle_dtype == CODA_BF16;
    for (int i = tid; i < Dh / 2; i += NT) {
      float ta = (float)r.pos, inv = p.inv_freq[i];
      if (abf) { ta = bf16_round(ta); inv = bf16_round(inv); }
      float ang = __fmul_rn(ta, inv);
      if (abf) ang = bf16_round(ang);
      float cc = cosf(ang), ss = sinf(ang);
      if (abf) { cc = bf16_round(cc); ss = bf16_round(ss); }
      cs[i] = El<T>::rnd(cc); sn[i] = El<T>::rnd(ss);
    }
    __syncthreads();
  } else {
    g_new = p.gate[b];
  }
  // element e = h*Dh + d of the new (rotated) key
  auto new_k = [&](int e) -> float {
    if (!p.raw) return El<T>::ld(kn + e);
    const int h = e / Dh, d = e % Dh;
    return rope_elem<T>(kn + h * Dh, d, Dh, c.rope_interleaved, cs, sn);
  };

  if (r.filled < W) {                                   // memory_banks.py:195-201
    const int slot = r.filled;
    for (int e = tid; e < HD; e += NT) {
      const int h = e / Dh, d = e % Dh;
      El<T>::st(kb + ((long long)h * Lbuf + slot) * Dh + d, new_k(e));
      vb[((long long)h * Lbuf + slot) * Dh + d] = vn[e];
    }
    if (tid == 0) { gr[slot] = g_new; al[slot] = 1; }
    return;
  }

  // ---- ring full: evict slot ev (memory_banks.py:203-222) ----
  const int ev = r.idx;
  const long long pos_e = r.pos - W;
  float* ke = sm;                 // [HD] evicted key
  float* ve = ke + HD;            // [HD] evicted value
  float* vhat = ve + HD;          // [HD] unit-norm value   (later: new V row for re-normalising)
  float* khat = vhat + HD;        // [Hkv*lfd] unit-norm LF key (later: new LF key row)
  float* sc = khat + Hkv * lfd;   // [max(Me,Ms)] scores
  long long* s_last = reinterpret_cast<long long*>((reinterpret_cast<uintptr_t>(sn + Dh / 2) + 7) & ~(uintptr_t)7);  // [Me] LRU stamps
  unsigned char* s_used = reinterpret_cast<unsigned char*>(s_last + Me);             // [Me + Ms] slot-in-use flags
  float* dots = reinterpret_cast<float*>((reinterpret_cast<uintptr_t>(s_used + Me + Ms) + 15) & ~(uintptr_t)15);  // [max(Me,Ms)*Hkv]
  __shared__ int s_idx, s_flag;
  __shared__ float s_eta_keep;
  const size_t vbytes = (size_t)Hkv * Me * Dh * sizeof(T), kbytes = (size_t)Hkv * Ms * lfd * sizeof(T);
  T* cacheV = reinterpret_cast<T*>(reinterpret_cast<unsigned char*>(sm) + p.stage_off);
  T* cacheK = reinterpret_cast<T*>(reinterpret_cast<unsigned char*>(cacheV) + vbytes);
  __shared__ __align__(8) uint64_t s_bar;
  if (p.stage) {
    if (tid == 0) { tma::mbar_init(&s_bar, 1); tma::fence_barrier_init(); }
    __syncthreads();
    if (tid == 0) {
      tma::mbar_expect_tx(&s_bar, (uint32_t)(vbytes + kbytes));
      const unsigned char* gv = reinterpret_cast<const unsigned char*>(p.st.exact_v_norm) + (size_t)b * vbytes;
      const unsigned char* gk = reinterpret_cast<const unsigned char*>(p.st.sum_lf_k_norm) + (size_t)b * kbytes;
      for (size_t o = 0; o < vbytes; o += 32768)
        tma::bulk_load(reinterpret_cast<unsigned char*>(cacheV) + o, gv + o, (uint32_t)(vbytes - o < 32768 ? vbytes - o : 32768), &s_bar);
      for (size_t o = 0; o < kbytes; o += 32768)
        tma::bulk_load(reinterpret_cast<unsigned char*>(cacheK) + o, gk + o, (uint32_t)(kbytes - o < 32768 ? kbytes - o : 32768), &s_bar);
    }
  }
  for (int m = tid; m < Me + Ms; m += NT) s_used[m] = al[W + m];
  for (int m = tid; m < Me; m += NT) s_last[m] = ((const long long*)p.st.mem_last_exact)[(long long)b * Me + m];

  for (int e = tid; e < HD; e += NT) {
    const int h = e / Dh, d = e % Dh;
    ke[e] = El<T>::ld(kb + ((long long)h * Lbuf + ev) * Dh + d);
    ve[e] = El<T>::ld(vb + ((long long)h * Lbuf + ev) * Dh + d);
  }
  const float g_e = gr[ev];
  __syncthreads();
  // unit vectors: x / max(||x||, 1e-6) per head (F.normalize, memory_banks.py:258,372)
  for (int h = warp; h < Hkv; h += NW) {
    float ssv = 0.f, ssk = 0.f;
    for (int d = lane; d < Dh; d += 32) {
      const float v = ve[h * Dh + d]; ssv += v * v;
      if (d >= lf) { const float k = ke[h * Dh + d]; ssk += k * k; }
    }
    ssv = warp_sum(ssv); ssk = warp_sum(ssk);
    const float dv = fmaxf(El<T>::rnd(sqrtf(ssv)), 1e-6f), dk = fmaxf(El<T>::rnd(sqrtf(ssk)), 1e-6f);
    for (int d = lane; d < Dh; d += 32) {
      vhat[h * Dh + d] = t_div<T>(ve[h * Dh + d], dv);
      if (d >= lf) khat[h * lfd + d - lf] = t_div<T>(ke[h * Dh + d], dk);
    }
  }
  __syncthreads();

  if (p.stage) tma::mbar_wait(&s_bar, 0, p.status, 3);

  // ================= exact bank (memory_banks.py:230-337) =================
  if (Me > 0) {
    const int Ae = c.active_exact;
    const T* vnorm = p.stage ? cacheV : (const T*)p.st.exact_v_norm + (long long)b * Hkv * Me * Dh;
    bank_scores_one<T>(vhat, vnorm, Me, Dh, Hkv, dots, sc, tid, NT);
    for (int m = tid; m < Me; m += NT) sc[m] = (m >= Ae || !s_used[m]) ? -1e9f : El<T>::rnd(sc[m] / (float)Hkv);
    __syncthreads();
    if (tid == 0) {
      long long* last = (long long*)p.st.mem_last_exact + (long long)b * Me;
      float best = sc[0]; int bi = 0;
      for (int m = 1; m < Me; ++m) if (sc[m] > best) { best = sc[m]; bi = m; }
      bool any_used = false; int free_i = -1; int lru_i = 0; long long lru_v = 0x7fffffffffffffffLL;
      for (int m = 0; m < Me; ++m) {
        const bool used = s_used[m] != 0, act = m < Ae;
        if (act && used) any_used = true;
        if (act && !used && free_i < 0) free_i = m;
        const long long key = (used && act) ? s_last[m] : (1LL << 62);
        if (key < lru_v) { lru_v = key; lru_i = m; }
      }
      const bool novel = !any_used || best < El<T>::rnd(c.tau_novel);
      const bool hit = any_used && best >= El<T>::rnd(c.tau_match);
      const bool keep = c.gated ? (g_e >= c.tau_gate_exact) : true;
      const int idx = novel ? (free_i >= 0 ? free_i : lru_i) : bi;
      const bool ow = (novel || (c.refresh_on_hit && hit)) && keep;
      if (keep) last[idx] = pos_e;                       // memory_banks.py:325-331
      s_idx = idx; s_flag = ow ? 1 : 0;
    }
    __syncthreads();
    if (s_flag) {
      const int slot = W + s_idx;
      for (int e = tid; e < HD; e += NT) {
        const int h = e / Dh, d = e % Dh;
        T* pk = kb + ((long long)h * Lbuf + slot) * Dh + d;
        T* pv = vb + ((long long)h * Lbuf + slot) * Dh + d;
        const float ok = El<T>::ld(pk), ov = El<T>::ld(pv);
        El<T>::st(pk, t_add<T>(ok, t_sub<T>(ke[e], ok)));  // mem + 1*(x - mem), memory_banks.py:301-302
        const float nv = t_add<T>(ov, t_sub<T>(ve[e], ov));
        El<T>::st(pv, nv);
        vhat[e] = nv;
      }
      if (tid == 0) al[slot] = 1;
      __syncthreads();
      T* vnorm_w = (T*)p.st.exact_v_norm + (long long)b * Hkv * Me * Dh;
      for (int h = warp; h < Hkv; h += NW) {              // re-normalise the written slot only
        float ss = 0.f;
        for (int d = lane; d < Dh; d += 32) { const float v = vhat[h * Dh + d]; ss += v * v; }
        const float den = fmaxf(El<T>::rnd(sqrtf(warp_sum(ss))), 1e-6f);
        for (int d = lane; d < Dh; d += 32)
          El<T>::st(vnorm_w + ((long long)h * Me + s_idx) * Dh + d, t_div<T>(vhat[h * Dh + d], den));
      }
    }
    __syncthreads();
  }

  // ================= summary bank (memory_banks.py:343-432) =================
  if (Ms > 0) {
    const int As = c.active_summary;
    const T* knorm = p.stage ? cacheK : (const T*)p.st.sum_lf_k_norm + (long long)b * Hkv * Ms * lfd;
    bank_scores_one<T>(khat, knorm, Ms, lfd, Hkv, dots, sc, tid, NT);
    for (int m = tid; m < Ms; m += NT) sc[m] = (m >= As) ? -1e9f : El<T>::rnd(sc[m] / (float)Hkv);
    __syncthreads();
    if (tid == 0) {
      float best = sc[0]; int bi = 0;
      for (int m = 1; m < Ms; ++m) if (sc[m] > best) { best = sc[m]; bi = m; }
      const bool is_new = s_used[Me + bi] == 0;
      const bool keep = c.gated ? (g_e >= c.tau_gate_summary) : true;
      s_idx = bi; s_flag = (c.overwrite_on_insert && is_new) ? 1 : 0;
      s_eta_keep = keep ? 1.f : 0.f;
      if (keep) al[W + Me + bi] = 1;
    }
    __syncthreads();
    const int slot = W + Me + s_idx;
    const float gT = El<T>::rnd(g_e);
    for (int e = tid; e < HD; e += NT) {
      const int h = e / Dh, d = e % Dh;
      float eta = t_sigmoid<T>(p.eta_logit[h]);
      if (c.gated) eta = t_mul<T>(eta, gT);
      if (s_flag) eta = 1.f;
      eta = t_mul<T>(eta, s_eta_keep);
      T* pk = kb + ((long long)h * Lbuf + slot) * Dh + d;
      T* pv = vb + ((long long)h * Lbuf + slot) * Dh + d;
      const float ok = El<T>::ld(pk), ov = El<T>::ld(pv);
      if (d >= lf) {                                     // phase-safe EMA: LF band only
        const float inc = El<T>::rnd(__fmul_rn(ke[e], c.energy_scale));
        const float nk = t_add<T>(ok, t_mul<T>(eta, t_sub<T>(inc, ok)));
        El<T>::st(pk, nk);
        khat[h * lfd + d - lf] = nk;
      }
      El<T>::st(pv, t_add<T>(ov, t_mul<T>(eta, t_sub<T>(ve[e], ov))));
    }
    __syncthreads();
    T* knorm_w = (T*)p.st.sum_lf_k_norm + (long long)b * Hkv * Ms * lfd;
    for (int h = warp; h < Hkv; h += NW) {
      float ss = 0.f;
      for (int d = lane; d < lfd; d += 32) { const float k = khat[h * lfd + d]; ss += k * k; }
      const float den = fmaxf(El<T>::rnd(sqrtf(warp_sum(ss))), 1e-6f);
      for (int d = lane; d < lfd; d += 32)
        El<T>::st(knorm_w + ((long long)h * Ms + s_idx) * lfd + d, t_div<T>(khat[h * lfd + d], den));
    }
  }

  // ---- the new token takes the evicted slot (memory_banks.py:219-222) ----
  for (int e = tid; e < HD; e += NT) {
    const int h = e / Dh, d = e % Dh;
    El<T>::st(kb + ((long long)h * Lbuf + ev) * Dh + d, new_k(e));
    vb[((long long)h * Lbuf + ev) * Dh + d] = vn[e];
  }
  if (tid == 0) gr[ev] = g_new;
}

static int step_write_impl(const coda_layer_cfg* cfg, const coda_state_ptrs* st, coda_ring_pos rp,
                           const void* k_new, int64_t k_bs, const void* v_new, int64_t v_bs,
                           const float* gate, const float* eta_logit, int raw, const float* inv_freq,
                           const void* gate_logit, int64_t gate_bs, coda_stream_t stream) {
  CODA_REQUIRE(coda_cfg_ok(cfg) && st, CODA_ERR_ARG, "step_write: invalid layer configuration");
  CODA_REQUIRE(st->k_buf && st->v_buf && st->allowed && st->g_recent && k_new && v_new, CODA_ERR_ARG,
               "step_write: null pointer");
  CODA_REQUIRE(raw ? (inv_freq && (!cfg->gated || gate_logit)) : (gate != nullptr), CODA_ERR_ARG,
               "step_write: gate / frequency inputs missing");
  CODA_REQUIRE(cfg->Me == 0 || (st->mem_last_exact && st->exact_v_norm), CODA_ERR_ARG, "step_write: exact bank pointers missing");
  CODA_REQUIRE(cfg->Ms == 0 || (st->sum_lf_k_norm && eta_logit), CODA_ERR_ARG, "step_write: summary bank pointers missing");
  CODA_REQUIRE(rp.recent_idx >= 0 && rp.recent_idx < cfg->W && rp.recent_filled >= 0 && rp.recent_filled <= cfg->W,
               CODA_ERR_ARG, "step_write: ring scalars out of range");
  StepParams p; p.c = *cfg; p.st = *st; p.rp = rp;
  p.k_new = k_new; p.k_bs = k_bs; p.v_new = v_new; p.v_bs = v_bs; p.gate = gate; p.eta_logit = eta_logit;
  p.raw = raw; p.inv_freq = inv_freq; p.gate_logit = gate_logit; p.gate_bs = gate_bs;
  const int HD = cfg->Hkv * cfg->Dh, lfd = cfg->Dh - cfg->Dh / 2;
  const int mx = cfg->Me > cfg->Ms ? cfg->Me : cfg->Ms;
  size_t smem = sizeof(float) * (size_t)(3 * HD + cfg->Hkv * lfd + mx + 1 + cfg->Dh + 2) +
                8 * (size_t)cfg->Me + (size_t)(cfg->Me + cfg->Ms) + 32 + sizeof(float) * (size_t)mx * cfg->Hkv;
  const size_t es = cfg->dtype == CODA_F32 ? 4 : 2;
  const size_t vbytes = (size_t)cfg->Hkv * cfg->Me * cfg->Dh * es, kbytes = (size_t)cfg->Hkv * cfg->Ms * lfd * es;
  p.stage = 0; p.stage_off = 0; p.status = nullptr;
  if (vbytes % 16 == 0 && kbytes % 16 == 0 && vbytes + kbytes > 0 && vbytes + kbytes < (1u << 20) &&
      (cfg->Me == 0 || (uintptr_t)st->exact_v_norm % 16 == 0) && (cfg->Ms == 0 || (uintptr_t)st->sum_lf_k_norm % 16 == 0) &&
      ((smem + 127) / 128 * 128) + vbytes + kbytes <= 226 * 1024) {
    p.stage = 1;
    p.stage_off = (int)((smem + 127) / 128 * 128);
    smem = (size_t)p.stage_off + vbytes + kbytes;
  }
  CODA_REQUIRE(smem <= 226 * 1024, CODA_ERR_LIMIT, "step_write: Hkv*Dh = %d too large for one CTA", HD);
  cudaStream_t s = (cudaStream_t)stream;
  if (cfg->dtype == CODA_F32) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(step_write_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    step_write_kernel<float><<<cfg->B, 512, smem, s>>>(p);
  } else {
    if (smem > 48 * 1024) cudaFuncSetAttribute(step_write_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    step_write_kernel<bf16><<<cfg->B, 512, smem, s>>>(p);
  }
  CODA_CHECK_LAUNCH("step_write");
  return CODA_OK;
}

extern "C" int coda_b200_step_write(const coda_layer_cfg* cfg, const coda_state_ptrs* st, coda_ring_pos rp,
                                    const void* k_new, int64_t k_bs, const void* v_new, int64_t v_bs,
                                    const float* gate, const float* eta_logit, coda_stream_t stream) {
  return step_write_impl(cfg, st, rp, k_new, k_bs, v_new, v_bs, gate, eta_logit, 0, nullptr, nullptr, 0, stream);
}

extern "C" int coda_b200_step_write_raw(const coda_layer_cfg* cfg, const coda_state_ptrs* st, coda_ring_pos rp,
                                        const void* k_raw, int64_t k_bs, const void* v_new, int64_t v_bs,
                                        const void* gate_logit, int64_t gate_bs, const float* inv_freq,
                                        const float* eta_logit, coda_stream_t stream) {
  return step_write_impl(cfg, st, rp, k_raw, k_bs, v_new, v_bs, nullptr, eta_logit, 1, inv_freq, gate_logit, gate_bs, stream);
}
