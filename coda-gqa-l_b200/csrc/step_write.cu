// Decode-step cache write: ring FIFO + routing of the evicted token into the exact and summary banks.
// One CTA per state.  Reads the two unit-norm routing caches once, rewrites at most one slot per bank.
#include <cstring>
#include <vector>
#include "coda_common.cuh"
#include "tma_utils.cuh"
#include "bank_score.cuh"
#include "decode_record.h"

#ifndef CODA_STEP_PREFETCH
#define CODA_STEP_PREFETCH 1   // fused decode write: ask the head's K/V planes into L2 for the attention that follows
#endif

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
  // fused mode (cluster kernel, bf16): the decode record of each plane is written as well
  const void* q_raw; long long q_bs; const void* lam_logit; long long lam_bs;
  const void* cos_t; const void* sin_t; unsigned char* qrec;
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
      float cc, ss; sincos_call(ang, &ss, &cc);
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

  // routing-event record of this call (optional): cleared here, filled by the deciding thread
  int32_t* evw = p.st.events != nullptr ? p.st.events + (long long)b * CODA_EVENT_WORDS : nullptr;
  if (evw != nullptr && tid < CODA_EVENT_WORDS) evw[tid] = 0;
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
      if (evw != nullptr) {
        evw[0] = (c.gated && !keep) ? 1 : 0;
        evw[1] = hit ? 1 : 0;
        evw[2] = (novel && keep) ? 1 : 0;
        evw[3] = ow ? 1 : 0;
        evw[4] = (novel && keep && free_i < 0) ? 1 : 0;
      }
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
      if (evw != nullptr) {
        bool all_used = true;                              // every active slot in use after this write?
        for (int m = 0; m < As; ++m) all_used = all_used && (s_used[Me + m] != 0 || (m == bi && keep));
        evw[5] = keep ? 1 : 0;
        evw[6] = (is_new && keep) ? 1 : 0;
        evw[7] = all_used ? 1 : 0;
        evw[8] = keep ? 1 : 0;
      }
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


// ------------------------------------------------------------------------------------------------------------
// Cluster variant: one CTA per (state, KV head), the Hkv CTAs of a state forming one thread-block cluster.
// The work of a decode write is a chain of short dependent steps (evicted row -> unit vectors -> scores ->
// decision -> slot update); one CTA per state leaves it on 1/5 of the SMs with every global round trip on
// the critical path.  Here each CTA touches one head only: its slice of both routing caches is requested
// into registers at kernel entry (two threads per bank row), the exact- and summary-bank scores are
// computed together, the per-head dot products are exchanged through distributed shared memory (every CTA
// stores its values into all CTAs of the cluster, one cluster barrier), and each CTA then takes both routing
// decisions redundantly, warp-parallel, before rewriting its own head's rows.
//
// MODE splits the step in two launches: the routing of the evicted token depends on the state alone and can
// run beside the projection GEMM that produces the new token, off the critical path.
//   0: everything (route the evicted token, then the new token takes its ring slot; fused mode: + record)
//   1: routing only: banks, routing caches, LRU stamps, slot flags, event record; the ring is left alone
//   2: the new token only, after a MODE 1 launch on the same ring position: ring slot, gate, record
//
// STAGE: both routing caches of the head (contiguous, 16-byte aligned) are brought into shared memory by two
// bulk copies issued by the first thread at entry instead of into registers by every thread: the scoring loop
// reads them from there, no thread holds cache chunks across the entry phase, and more CTAs fit an SM.  The
// launcher adds their bytes (rounded up to 16) to the dynamic shared memory and picks STAGE only when they fit.
template <typename T, int DH, int MODE, bool STAGE = false>
__device__ __forceinline__ void step_cluster_body(const StepParams& p) {
  constexpr bool ROUTE = MODE != 2, APPEND = MODE != 1;
  static_assert(!STAGE || MODE == 1, "staged caches are for the routing-only launch");
  constexpr int NT = 256, LF = DH / 2, LFD = DH - LF;
  constexpr int EPV = 16 / (int)sizeof(T);                // elements per 16-byte chunk
  constexpr int CE = DH / EPV, CS = LFD / EPV;            // chunks per exact / summary routing-cache row (powers of two <= 32)
  constexpr int PE = 4, PS = 2;                           // chunks per thread requested at kernel entry
  extern __shared__ float sm[];
  const coda_layer_cfg& c = p.c;
  const int h = blockIdx.x, b = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int W = c.W, Me = c.Me, Ms = c.Ms, Hkv = c.Hkv;
  const int Lbuf = W + Me + Ms, MM = Me + Ms;

  __shared__ float ke[DH], ve[DH], vhat[DH], khat[LFD], cs[DH / 2], sn[DH / 2], s_den[2];
  // unit vectors for the scoring loop: the second half of each starts 4 words further, so that the two halves
  // (read by alternate lanes) fall into different banks
  __shared__ __align__(16) float hv[DH + DH / 8], hk[LFD + LFD / 8];   // element e sits at e + 4 * (e / 32)
  __shared__ int s_eidx, s_eflag, s_sidx, s_sflag;
  __shared__ float s_keep;
  float* xdots = sm;                                      // [Hkv][MM] per-head dots of every CTA of the cluster
  float* sc = xdots + Hkv * MM;                           // [MM] reduced scores
  long long* s_last = reinterpret_cast<long long*>((reinterpret_cast<uintptr_t>(sc + MM) + 7) & ~(uintptr_t)7);  // [Me]
  unsigned char* s_al = reinterpret_cast<unsigned char*>(s_last + Me);                                           // [Lbuf] slot flags before the write
  unsigned char* s_used = s_al + W;                                                                              // [MM] the banks' part
  unsigned char* stage_e = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(s_al + Lbuf) + 15) & ~(uintptr_t)15);   // STAGE: [Me][DH] T
  unsigned char* stage_s = stage_e + (size_t)Me * DH * sizeof(T);                                                // STAGE: [Ms][LFD] T
  __shared__ __align__(8) uint64_t s_stage_bar;

  T* kb = (T*)p.st.k_buf + ((long long)b * Hkv + h) * Lbuf * DH;       // this head's planes
  T* vb = (T*)p.st.v_buf + ((long long)b * Hkv + h) * Lbuf * DH;
  uint8_t* al = p.st.allowed + (long long)b * Lbuf;
  float* gr = p.st.g_recent + (long long)b * W;
  const T* kn = (const T*)p.k_new + (long long)b * p.k_bs + h * DH;
  const T* vn = (const T*)p.v_new + (long long)b * p.v_bs + h * DH;

  // Distributed shared memory of a CTA may be written only once that CTA runs: every CTA announces itself
  // here and waits for the others just before its first remote store (or before it leaves).
  asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
  // Everything below is a chain of memory round trips, so requests go out as early as their addresses are known
  // and nothing is converted or otherwise touched before the next batch of requests is out (a warp issues in
  // order: the first use of a pending load holds up every request behind it).
  const long long nsteps = ring_steps(p.rp);             // the ring position hangs on it: asked for first

  // routing-event record of this call (optional): cleared here, filled by the deciding lanes of head 0
  int32_t* evw = (ROUTE && p.st.events != nullptr && h == 0) ? p.st.events + (long long)b * CODA_EVENT_WORDS : nullptr;
  if (evw != nullptr && tid < CODA_EVENT_WORDS) evw[tid] = 0;

  // ---- requests that depend on nothing but (b, h): issued first, consumed later ----
  // Both routing caches of this head are contiguous: thread t takes the 16-byte chunks t, t + NT, ... of each
  // (coalesced; CE / CS chunks make a row, held by CE / CS neighbouring lanes).  The first PE / PS passes --
  // 64 rows of each bank at bf16, Dh 128 -- are requested here; larger banks load the rest in the scoring loop.
  const T* vnorm = (const T*)p.st.exact_v_norm + ((long long)b * Hkv + h) * Me * DH;
  const T* knorm = (const T*)p.st.sum_lf_k_norm + ((long long)b * Hkv + h) * Ms * LFD;
  const uint4* vn4 = reinterpret_cast<const uint4*>(vnorm);
  const uint4* kn4 = reinterpret_cast<const uint4*>(knorm);
  const int nce = Me * CE, ncs = Ms * CS;
  uint4 pe[PE], ps[PS];
  if constexpr (STAGE) {
    if (tid == 0) {
      tma::mbar_init(&s_stage_bar, 1);
      tma::fence_barrier_init();
      const uint32_t be = (uint32_t)((size_t)Me * DH * sizeof(T)), bs = (uint32_t)((size_t)Ms * LFD * sizeof(T));
      tma::mbar_expect_tx(&s_stage_bar, be + bs);
      if (be > 0) tma::bulk_load(stage_e, vnorm, be, &s_stage_bar);
      if (bs > 0) tma::bulk_load(stage_s, knorm, bs, &s_stage_bar);
    }
  } else {
#pragma unroll
    for (int j = 0; j < PE; ++j) pe[j] = (ROUTE && tid + j * NT < nce) ? vn4[tid + j * NT] : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
    for (int j = 0; j < PS; ++j) ps[j] = (ROUTE && tid + j * NT < ncs) ? kn4[tid + j * NT] : make_uint4(0u, 0u, 0u, 0u);
  }
  // slot flags and LRU stamps: requested into registers now, parked in shared memory once every other request
  // is out (a load -> shared-store loop would cost one memory round trip per loop); Lbuf <= 4 * NT, Me <= NT
  uint8_t alr[4];
#pragma unroll
  for (int a = 0; a < 4; ++a) { const int m = tid + a * NT; alr[a] = m < Lbuf ? al[m] : (uint8_t)0; }
  const long long lastr = (ROUTE && tid < Me) ? ((const long long*)p.st.mem_last_exact)[(long long)b * Me + tid] : 0;
  // the new token's row (element tid < DH: key, DH <= tid < 2*DH: value)
  T nk_a_raw = T(), nk_b_raw = T(), glog_raw = T();
  float nv_x = 0.f, eta_raw = 0.f, glog = 0.f;
  const bool is_k = tid < DH, is_v = tid >= DH && tid < 2 * DH;
  const int d = is_k ? tid : tid - DH;
  int ri = 0;                                             // RoPE pair index of key element d
  if (APPEND && is_k) {
    if (p.raw) {
      int ia, ib;
      if (c.rope_interleaved) { ri = d >> 1; ia = 2 * ri; ib = ia + 1; }
      else { ri = d < LF ? d : d - LF; ia = ri; ib = ri + LF; }
      nk_a_raw = kn[ia]; nk_b_raw = kn[ib];
    } else {
      nk_a_raw = kn[d];
    }
  }
  T nv_raw = T();
  if (APPEND && is_v) nv_raw = vn[d];
  (void)nv_x;
  if (ROUTE && Ms > 0) eta_raw = p.eta_logit[h];
  const float inv_f = (APPEND && p.raw && tid < DH / 2) ? p.inv_freq[tid] : 0.f;
  if (APPEND) {
    if (p.raw) { if (c.gated) glog_raw = ((const T*)p.gate_logit)[(long long)b * p.gate_bs]; }
    else glog = p.gate[b];
  }

  // fused mode: raw query pairs, theta tables and lambda logit (requested now, used last)
  constexpr int QI = (8 * (DH / 2) + NT - 1) / NT;        // (head, pair) items per thread, G <= 8
  const bool fused = APPEND && p.qrec != nullptr;
  const int G = c.H / Hkv;
  uint32_t fq0[QI], fq1[QI]; bf16 fct[QI], fst[QI];
  float flam = 0.f;
  bf16 flam_raw = __float2bfloat16_rn(0.f);
  if (fused) {
    const bf16* qrow = (const bf16*)p.q_raw + (long long)b * p.q_bs + (long long)h * G * DH;
#pragma unroll
    for (int it = 0; it < QI; ++it) {
      const int w = tid + it * NT;
      fq0[it] = fq1[it] = 0u; fct[it] = fst[it] = __float2bfloat16_rn(0.f);
      if (w < G * (DH / 2)) {
        const int g = w / (DH / 2), i = w % (DH / 2);
        const bf16* qh = qrow + g * DH;
        if (c.rope_interleaved) {
          fq0[it] = *reinterpret_cast<const uint32_t*>(qh + 2 * i);
        } else {
          const int pi = 2 * i < DH / 2 ? 2 * i : 2 * i - DH / 2;
          fq0[it] = *reinterpret_cast<const uint32_t*>(qh + pi);
          fq1[it] = *reinterpret_cast<const uint32_t*>(qh + pi + DH / 2);
        }
        fct[it] = ((const bf16*)p.cos_t)[(h * G + g) * (DH / 2) + i];
        fst[it] = ((const bf16*)p.sin_t)[(h * G + g) * (DH / 2) + i];
      }
    }
    if (tid < G) flam_raw = ((const bf16*)p.lam_logit)[(long long)b * p.lam_bs + h * G + tid];
  }

  const RingNow r = ring_after(p.rp, W, nsteps);
  const bool full = r.filled >= W;
  const int ev = full ? r.idx : r.filled;                 // the ring slot the new token takes
  T ke_raw = T(), ve_raw = T();
  float g_e = 0.f;
  if (ROUTE && full) {                                    // evicted row of this head
    if (is_k) ke_raw = kb[(long long)ev * DH + d];
    if (is_v) ve_raw = vb[(long long)ev * DH + d];
    g_e = gr[ev];
  }
#if CODA_STEP_PREFETCH
  // Fused mode is followed at once by the decode attention, which reads this head's whole K and V planes: the
  // routing below is a chain of memory round trips that leaves HBM idle, so the planes are asked into L2
  // meanwhile (a hint: no completion, nothing depends on it).  Issued after this CTA's own latency-critical
  // requests; the bank slots -- whose rows the routing is about to read -- go first.
  if (fused) {
    constexpr unsigned CH = 16384;
    const unsigned plane_bytes = (unsigned)Lbuf * DH * (unsigned)sizeof(T);      // a multiple of 128
    const unsigned nch = (plane_bytes + CH - 1) / CH;
    for (unsigned i = tid; i < 2 * nch; i += NT) {
      const unsigned cidx = nch - 1 - (i >> 1);                                   // from the end of the plane (banks) backwards
      const unsigned off = cidx * CH, sz = plane_bytes - off < CH ? plane_bytes - off : CH;
      const char* base = reinterpret_cast<const char*>((i & 1) ? vb : kb) + off;
      asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(base), "r"(sz) : "memory");
    }
  }
#endif
  // ---- the first batch of requests is out: from here on values may be used ----
  const float nk_a = El<T>::ld(&nk_a_raw), nk_b = El<T>::ld(&nk_b_raw);
  if (p.raw && c.gated) glog = El<T>::ld(&glog_raw);
  flam = __bfloat162float(flam_raw);
  float g_new = 0.f;
  if (!APPEND) {
  } else if (p.raw) {
    g_new = c.gated ? t_sigmoid<T>(glog) : 1.0f;
    const bool abf = c.angle_dtype == CODA_BF16;
    if (tid < DH / 2) {
      float ta = (float)r.pos, inv = inv_f;
      if (abf) { ta = bf16_round(ta); inv = bf16_round(inv); }
      float ang = __fmul_rn(ta, inv);
      if (abf) ang = bf16_round(ang);
      float cc, ss; sincos_call(ang, &ss, &cc);
      if (abf) { cc = bf16_round(cc); ss = bf16_round(ss); }
      cs[tid] = El<T>::rnd(cc); sn[tid] = El<T>::rnd(ss);
    }
  } else {
    g_new = glog;
  }
  if (ROUTE && full) {
    if (is_k) ke[d] = El<T>::ld(&ke_raw);
    if (is_v) ve[d] = El<T>::ld(&ve_raw);
  }
#pragma unroll
  for (int a = 0; a < 4; ++a) { const int m = tid + a * NT; if (m < Lbuf) s_al[m] = alr[a]; }
  if (tid < Me) s_last[tid] = lastr;
  __syncthreads();
  // rotated key element d (primitives.py:99-113)
  float new_k = nk_a;
  if (is_k && p.raw) {
    const float cc = cs[ri], ss = sn[ri];
    if (c.rope_interleaved) new_k = (d & 1) ? t_add<T>(t_mul<T>(nk_a, ss), t_mul<T>(nk_b, cc)) : t_sub<T>(t_mul<T>(nk_a, cc), t_mul<T>(nk_b, ss));
    else new_k = d < LF ? t_add<T>(t_mul<T>(nk_a, cc), t_mul<T>(-nk_b, ss)) : t_add<T>(t_mul<T>(nk_b, cc), t_mul<T>(nk_a, ss));
  }

  // Decode record of this plane (queries of the token being written, lambda, visibility mask after the write).
  // `e_on`/`s_on`: bank slots switched on by this write (-1: none).
  auto write_record = [&](int e_on, int s_on) {
    if constexpr (sizeof(T) == 2) {
      constexpr int HALF = DH / 2, QSTR = DH + 8;
      unsigned char* rec = p.qrec + ((long long)b * Hkv + h) * DecodeRecord::bytes(G, DH, Lbuf);
      bf16* q_s = reinterpret_cast<bf16*>(rec);
#pragma unroll
      for (int it = 0; it < QI; ++it) {
        const int w = tid + it * NT;
        if (w < G * HALF) {
          const int g = w / HALF, i = w % HALF;
          const float a0 = __uint_as_float(fq0[it] << 16), a1 = __uint_as_float(fq0[it] & 0xffff0000u);
          const float b0 = __uint_as_float(fq1[it] << 16), b1 = __uint_as_float(fq1[it] & 0xffff0000u);
          float e0, e1;                                    // RoPE'd elements 2i, 2i+1 (primitives.py:99-113)
          if (c.rope_interleaved) {
            e0 = t_sub<T>(t_mul<T>(a0, cs[i]), t_mul<T>(a1, sn[i]));
            e1 = t_add<T>(t_mul<T>(a0, sn[i]), t_mul<T>(a1, cs[i]));
          } else {
            const bool lo = 2 * i < HALF;
            const int pi = lo ? 2 * i : 2 * i - HALF;
            e0 = lo ? t_add<T>(t_mul<T>(a0, cs[pi]), t_mul<T>(-b0, sn[pi])) : t_add<T>(t_mul<T>(b0, cs[pi]), t_mul<T>(a0, sn[pi]));
            e1 = lo ? t_add<T>(t_mul<T>(a1, cs[pi + 1]), t_mul<T>(-b1, sn[pi + 1])) : t_add<T>(t_mul<T>(b1, cs[pi + 1]), t_mul<T>(a1, sn[pi + 1]));
          }
          const float ct = __bfloat162float(fct[it]), st = __bfloat162float(fst[it]);
          const float n0 = t_sub<T>(t_mul<T>(e0, ct), t_mul<T>(e1, st));
          const float n1 = t_add<T>(t_mul<T>(e0, st), t_mul<T>(e1, ct));
          __nv_bfloat162 sv = __floats2bfloat162_rn(e0, e1), nv2 = __floats2bfloat162_rn(n0, n1);
          *reinterpret_cast<__nv_bfloat162*>(q_s + g * QSTR + 2 * i) = sv;
          *reinterpret_cast<__nv_bfloat162*>(q_s + (G + g) * QSTR + 2 * i) = nv2;
        }
      }
      const int rows = DecodeRecord::qrows(G);
      #pragma unroll 1
      for (int w = tid; w < (rows - 2 * G) * HALF; w += NT)   // unused rows of the query tile: zero
        *reinterpret_cast<uint32_t*>(q_s + (2 * G + w / HALF) * QSTR + 2 * (w % HALF)) = 0u;
      float* lam = reinterpret_cast<float*>(rec + DecodeRecord::lam_off(G, DH));
      if (tid < 8) lam[tid] = tid < G ? t_sigmoid<T>(flam) : 0.f;
      uint8_t* mk = rec + DecodeRecord::mask_off(G, DH);
      #pragma unroll 1
      for (int i = tid; i < DecodeRecord::mask_bytes(Lbuf); i += NT) {
        uint8_t v = 0;
        if (i < Lbuf) v = (i == ev || (e_on >= 0 && i == W + e_on) || (s_on >= 0 && i == W + Me + s_on)) ? 1 : s_al[i];
        mk[i] = v;
      }
    }
  };

  if (!full || !ROUTE) {                                  // ring still filling (memory_banks.py:195-201; uniform over the grid), or routing done by an earlier launch
    if (fused) write_record(-1, -1);
    asm volatile("barrier.cluster.wait.aligned;" ::: "memory");
    if constexpr (STAGE) tma::mbar_wait(&s_stage_bar, 0, p.status, 31);    // no copy may be in flight into a CTA that leaves
    if (APPEND) {
      if (is_k) El<T>::st(kb + (long long)ev * DH + d, new_k);
      if (is_v) vb[(long long)ev * DH + d] = nv_raw;
      if (h == 0 && tid == 0) { gr[ev] = g_new; if (!full) al[ev] = 1; }
    }
    return;
  }

  // ---- ring full: the evicted token is routed (memory_banks.py:203-222) ----
  const long long pos_e = r.pos - W;
  // unit vectors x / max(||x||, 1e-6) (F.normalize, memory_banks.py:258,372): warp 0 value, warp 1 LF key
  if (warp < 2) {
    float ss = 0.f;
    if (warp == 0) { for (int i = lane; i < DH; i += 32) ss += ve[i] * ve[i]; }
    else { for (int i = LF + lane; i < DH; i += 32) ss += ke[i] * ke[i]; }
    ss = warp_sum(ss);
    if (lane == 0) s_den[warp] = fmaxf(El<T>::rnd(sqrtf(ss)), 1e-6f);
  }
  __syncthreads();
  if (is_v) hv[d + 4 * (d >> 5)] = t_div<T>(ve[d], s_den[0]);
  if (is_k && d >= LF) hk[(d - LF) + 4 * ((d - LF) >> 5)] = t_div<T>(ke[d], s_den[1]);
  __syncthreads();

  asm volatile("barrier.cluster.wait.aligned;" ::: "memory");       // all CTAs of the cluster are running
  // ---- per-head dot products of both banks, sent to every CTA of the cluster ----
  // dot of one chunk with the matching EPV elements of a unit vector (two accumulation chains)
  auto chunk_dot = [&](const uint4& v, const float* a) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    float f[EPV];
    if (sizeof(T) == 2) {
#pragma unroll
      for (int q = 0; q < 4; ++q) { f[2 * q] = __uint_as_float(w[q] << 16); f[2 * q + 1] = __uint_as_float(w[q] & 0xffff0000u); }
    } else {
#pragma unroll
      for (int q = 0; q < 4; ++q) f[q] = __uint_as_float(w[q]);
    }
    float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
    for (int q4 = 0; q4 < EPV; q4 += 4) {
      const float4 av = *reinterpret_cast<const float4*>(a + q4);
      acc0 = fmaf(av.x, f[q4], acc0); acc1 = fmaf(av.y, f[q4 + 1], acc1);
      acc0 = fmaf(av.z, f[q4 + 2], acc0); acc1 = fmaf(av.w, f[q4 + 3], acc1);
    }
    return acc0 + acc1;
  };
  // The rounded per-head dot of bank slot m goes to every CTA of the cluster.  After the butterfly reduction all
  // `per` lanes of the row hold the sum, so lane `first` of the row serves ranks first, first + per, ...: one
  // remote store per lane at the sizes in use (Hkv <= lanes per row) instead of a loop over the ranks in one lane.
  auto send = [&](int m, float acc, int first, int per) {
    const float v = El<T>::rnd(acc);
    const uint32_t local = tma::smem_u32(xdots + h * MM + m);
    #pragma unroll 1
    for (int rk = first; rk < Hkv; rk += per) {
      uint32_t remote;
      asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rk));
      asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(v) : "memory");
    }
  };
  {
    // this thread's chunk position inside a row is the same in every pass (NT is a multiple of CE and CS)
    const int ce = tid % CE, cs_ = tid % CS;
    const float* ae = hv + ce * EPV + 4 * ((ce * EPV) >> 5);
    const float* as = hk + cs_ * EPV + 4 * ((cs_ * EPV) >> 5);
    auto exact_pass = [&](const uint4& v, int j) {
      const int ch = tid + j * NT;
      float acc = ch < nce ? chunk_dot(v, ae) : 0.f;
#pragma unroll
      for (int o = CE / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (ch < nce) send(ch / CE, acc, ce, CE);
    };
    auto summary_pass = [&](const uint4& v, int j) {
      const int ch = tid + j * NT;
      float acc = ch < ncs ? chunk_dot(v, as) : 0.f;
#pragma unroll
      for (int o = CS / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (ch < ncs) send(Me + ch / CS, acc, cs_, CS);
    };
    if constexpr (STAGE) {
      tma::mbar_wait(&s_stage_bar, 0, p.status, 31);
      const uint4* se4 = reinterpret_cast<const uint4*>(stage_e);
      const uint4* ss4 = reinterpret_cast<const uint4*>(stage_s);
      #pragma unroll 2
      for (int j = 0; j * NT < nce; ++j) {
        const int ch = tid + j * NT;
        exact_pass(ch < nce ? se4[ch] : make_uint4(0u, 0u, 0u, 0u), j);
      }
      #pragma unroll 2
      for (int j = 0; j * NT < ncs; ++j) {
        const int ch = tid + j * NT;
        summary_pass(ch < ncs ? ss4[ch] : make_uint4(0u, 0u, 0u, 0u), j);
      }
    } else {
#pragma unroll
    for (int j = 0; j < PE; ++j) if (j * NT < nce) exact_pass(pe[j], j);
    #pragma unroll 1
    for (int j = PE; j * NT < nce; ++j) {
      const int ch = tid + j * NT;
      exact_pass(ch < nce ? vn4[ch] : make_uint4(0u, 0u, 0u, 0u), j);
    }
#pragma unroll
    for (int j = 0; j < PS; ++j) if (j * NT < ncs) summary_pass(ps[j], j);
    #pragma unroll 1
    for (int j = PS; j * NT < ncs; ++j) {
      const int ch = tid + j * NT;
      summary_pass(ch < ncs ? kn4[ch] : make_uint4(0u, 0u, 0u, 0u), j);
    }
    }
  }
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");

  // ---- scores: sum over heads of the rounded per-head dots, mean, masks ----
  const int Ae = c.active_exact, As = c.active_summary;
  #pragma unroll 1
  for (int m = tid; m < MM; m += NT) {
    float tot = 0.f;
    #pragma unroll 1
    for (int hh = 0; hh < Hkv; ++hh) tot += xdots[hh * MM + m];
    const float mean = El<T>::rnd(tot / (float)Hkv);
    sc[m] = m < Me ? ((m >= Ae || !s_used[m]) ? -1e9f : mean) : ((m - Me >= As) ? -1e9f : mean);
  }
  __syncthreads();
  // ---- decisions, taken redundantly by every CTA: warp 0 exact bank, warp 1 summary bank ----
  auto arg_best = [&](const float* v, int n, float& best, int& bi) {     // first index of the maximum
    best = -INFINITY; bi = 0x7fffffff;
    #pragma unroll 1
    for (int m = lane; m < n; m += 32) if (v[m] > best || bi == 0x7fffffff) { best = v[m]; bi = m; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > best || (ov == best && oi < bi))) { best = ov; bi = oi; }
    }
  };
  if (warp == 0 && Me > 0) {                              // memory_banks.py:230-337
    float best; int bi;
    arg_best(sc, Me, best, bi);
    int free_i = 0x7fffffff, lru_i = 0x7fffffff; long long lru_v = 0x7fffffffffffffffLL; bool any_used = false;
    #pragma unroll 1
    for (int m = lane; m < Me; m += 32) {
      const bool used = s_used[m] != 0, act = m < Ae;
      if (act && used) any_used = true;
      if (act && !used && m < free_i) free_i = m;
      const long long key = (used && act) ? s_last[m] : (1LL << 62);
      if (key < lru_v) { lru_v = key; lru_i = m; }
    }
    any_used = __any_sync(0xffffffffu, any_used);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      free_i = min(free_i, __shfl_xor_sync(0xffffffffu, free_i, o));
      const long long ov = __shfl_xor_sync(0xffffffffu, lru_v, o);
      const int oi = __shfl_xor_sync(0xffffffffu, lru_i, o);
      if (ov < lru_v || (ov == lru_v && oi < lru_i)) { lru_v = ov; lru_i = oi; }
    }
    if (lane == 0) {
      const bool novel = !any_used || best < El<T>::rnd(c.tau_novel);
      const bool hit = any_used && best >= El<T>::rnd(c.tau_match);
      const bool keep = c.gated ? (g_e >= c.tau_gate_exact) : true;
      const int idx = novel ? (free_i != 0x7fffffff ? free_i : lru_i) : bi;
      const bool ow = (novel || (c.refresh_on_hit && hit)) && keep;
      if (keep && h == 0) ((long long*)p.st.mem_last_exact)[(long long)b * Me + idx] = pos_e;   // memory_banks.py:325-331
      if (ow && h == 0) al[W + idx] = 1;
      s_eidx = idx; s_eflag = ow ? 1 : 0;
      if (evw != nullptr) {
        evw[0] = (c.gated && !keep) ? 1 : 0;
        evw[1] = hit ? 1 : 0;
        evw[2] = (novel && keep) ? 1 : 0;
        evw[3] = ow ? 1 : 0;
        evw[4] = (novel && keep && free_i == 0x7fffffff) ? 1 : 0;
      }
    }
  }
  if (warp == 1 && Ms > 0) {                              // memory_banks.py:343-432
    float best; int bi;
    arg_best(sc + Me, Ms, best, bi);
    const bool keep_s = c.gated ? (g_e >= c.tau_gate_summary) : true;
    bool all_used = true;                                  // every active slot in use after this write?
    #pragma unroll 1
    for (int m = lane; m < As; m += 32) all_used = all_used && (s_used[Me + m] != 0 || (m == bi && keep_s));
    all_used = __all_sync(0xffffffffu, all_used);
    if (lane == 0) {
      const bool is_new = s_used[Me + bi] == 0;
      const bool keep = keep_s;
      s_sidx = bi; s_sflag = (c.overwrite_on_insert && is_new) ? 1 : 0;
      s_keep = keep ? 1.f : 0.f;
      if (keep && h == 0) al[W + Me + bi] = 1;
      if (evw != nullptr) {
        evw[5] = keep ? 1 : 0;
        evw[6] = (is_new && keep) ? 1 : 0;
        evw[7] = all_used ? 1 : 0;
        evw[8] = keep ? 1 : 0;
      }
    }
  }
  __syncthreads();

  // ---- slot updates of this head: the old rows of both banks are requested together ----
  const bool do_e = Me > 0 && s_eflag != 0, do_s = Ms > 0;
  const long long eoff = (long long)(W + s_eidx) * DH + d, soff = (long long)(W + Me + s_sidx) * DH + d;
  T eo_raw = T(), so_raw = T();
  if (do_e && (is_k || is_v)) eo_raw = ((is_k ? kb : vb))[eoff];
  if (do_s && (is_v || (is_k && d >= LF))) so_raw = ((is_k ? kb : vb))[soff];
  // the record is written while the old rows travel
  if (fused) write_record(do_e ? s_eidx : -1, (do_s && s_keep != 0.f) ? s_sidx : -1);
  const float eo = El<T>::ld(&eo_raw), so = El<T>::ld(&so_raw);
  if (do_e) {
    if (is_k) El<T>::st(kb + eoff, t_add<T>(eo, t_sub<T>(ke[d], eo)));       // mem + 1*(x - mem), memory_banks.py:301-302
    if (is_v) { const float nv = t_add<T>(eo, t_sub<T>(ve[d], eo)); El<T>::st(vb + eoff, nv); vhat[d] = nv; }
  }
  if (do_s) {
    float eta = t_sigmoid<T>(eta_raw);
    if (c.gated) eta = t_mul<T>(eta, El<T>::rnd(g_e));
    if (s_sflag) eta = 1.f;
    eta = t_mul<T>(eta, s_keep);
    if (is_k && d >= LF) {                                // phase-safe EMA: LF band only
      const float inc = El<T>::rnd(__fmul_rn(ke[d], c.energy_scale));
      const float nk = t_add<T>(so, t_mul<T>(eta, t_sub<T>(inc, so)));
      El<T>::st(kb + soff, nk);
      khat[d - LF] = nk;
    }
    if (is_v) El<T>::st(vb + soff, t_add<T>(so, t_mul<T>(eta, t_sub<T>(ve[d], so))));
  }
  __syncthreads();
  // re-normalise the two rewritten rows of the routing caches
  if (warp == 0 && do_e) {
    float ss = 0.f;
    #pragma unroll 1
    for (int i = lane; i < DH; i += 32) ss += vhat[i] * vhat[i];
    const float den = fmaxf(El<T>::rnd(sqrtf(warp_sum(ss))), 1e-6f);
    T* dst = (T*)p.st.exact_v_norm + (((long long)b * Hkv + h) * Me + s_eidx) * DH;
    #pragma unroll 1
    for (int i = lane; i < DH; i += 32) El<T>::st(dst + i, t_div<T>(vhat[i], den));
  }
  if (warp == 1 && do_s) {
    float ss = 0.f;
    #pragma unroll 1
    for (int i = lane; i < LFD; i += 32) ss += khat[i] * khat[i];
    const float den = fmaxf(El<T>::rnd(sqrtf(warp_sum(ss))), 1e-6f);
    T* dst = (T*)p.st.sum_lf_k_norm + (((long long)b * Hkv + h) * Ms + s_sidx) * LFD;
    #pragma unroll 1
    for (int i = lane; i < LFD; i += 32) El<T>::st(dst + i, t_div<T>(khat[i], den));
  }
  // ---- the new token takes the evicted slot (memory_banks.py:219-222) ----
  if (APPEND) {
    if (is_k) El<T>::st(kb + (long long)ev * DH + d, new_k);
    if (is_v) vb[(long long)ev * DH + d] = nv_raw;
    if (h == 0 && tid == 0) gr[ev] = g_new;
  }
}

// ------------------------------------------------------------------------------------------------------------
// The new token's half of a split decode step (bf16, raw inputs, after the routing of the same ring position):
// RoPE of the key, ring slot, gate, decode record.  What step_cluster_body<MODE 2> does, without the routing
// code around it and without a cluster: eight warps work, a ninth does nothing but hand the L2 prefetch of the
// head's planes to the copy engine (~2 K cycles of issue that would otherwise sit on the kernel's only chain).
template <int DH>
__global__ void __launch_bounds__(288) step_append_kernel(StepParams p) {
  using T = bf16;
  constexpr int NT = 256, LF = DH / 2, HALF = DH / 2, QSTR = DH + 8;
  constexpr int QI = (8 * (DH / 2) + NT - 1) / NT;        // (head, pair) items per thread, G <= 8
  const coda_layer_cfg& c = p.c;
  const int h = blockIdx.x, b = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int W = c.W, Me = c.Me, Ms = c.Ms, Hkv = c.Hkv, Lbuf = W + Me + Ms, G = c.H / Hkv;
  __shared__ float cs[DH / 2], sn[DH / 2];
  __shared__ unsigned char s_al[1024];                    // Lbuf <= 1024 (fused-mode limit)
  T* kb = (T*)p.st.k_buf + ((long long)b * Hkv + h) * Lbuf * DH;
  T* vb = (T*)p.st.v_buf + ((long long)b * Hkv + h) * Lbuf * DH;
  // the kernel after this one (the decode attention) may start its prologue now; it waits for this grid to
  // complete before it reads anything
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const long long nsteps = ring_steps(p.rp);             // the ring position hangs on it: asked for first
  if (warp == NT / 32) {
    constexpr unsigned CH = 16384;
    const unsigned plane_bytes = (unsigned)Lbuf * DH * (unsigned)sizeof(T);      // a multiple of 128
    const unsigned nch = (plane_bytes + CH - 1) / CH;
    for (unsigned i = lane; i < 2 * nch; i += 32) {
      const unsigned cidx = i >> 1, off = cidx * CH, sz = plane_bytes - off < CH ? plane_bytes - off : CH;
      const char* base = reinterpret_cast<const char*>((i & 1) ? vb : kb) + off;
      asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(base), "r"(sz) : "memory");
    }
    return;
  }
  uint8_t* al = p.st.allowed + (long long)b * Lbuf;
  float* gr = p.st.g_recent + (long long)b * W;
  const T* kn = (const T*)p.k_new + (long long)b * p.k_bs + h * DH;
  const T* vn = (const T*)p.v_new + (long long)b * p.v_bs + h * DH;
  // ---- every request first (a warp issues in order: the first use of a pending load holds up those behind it) ----
  uint8_t alr[4];
#pragma unroll
  for (int a = 0; a < 4; ++a) { const int m = tid + a * NT; alr[a] = m < Lbuf ? al[m] : (uint8_t)0; }
  const bool is_k = tid < DH, is_v = tid >= DH && tid < 2 * DH;
  const int d = is_k ? tid : tid - DH;
  int ri = 0;
  T nk_a_raw = T(), nk_b_raw = T(), nv_raw = T(), glog_raw = T();
  if (is_k) {
    int ia, ib;
    if (c.rope_interleaved) { ri = d >> 1; ia = 2 * ri; ib = ia + 1; }
    else { ri = d < LF ? d : d - LF; ia = ri; ib = ri + LF; }
    nk_a_raw = kn[ia]; nk_b_raw = kn[ib];
  }
  if (is_v) nv_raw = vn[d];
  const float inv_f = tid < DH / 2 ? p.inv_freq[tid] : 0.f;
  if (c.gated) glog_raw = ((const T*)p.gate_logit)[(long long)b * p.gate_bs];
  uint32_t fq0[QI], fq1[QI]; bf16 fct[QI], fst[QI];
  bf16 flam_raw = __float2bfloat16_rn(0.f);
  {
    const bf16* qrow = (const bf16*)p.q_raw + (long long)b * p.q_bs + (long long)h * G * DH;
#pragma unroll
    for (int it = 0; it < QI; ++it) {
      const int w = tid + it * NT;
      fq0[it] = fq1[it] = 0u; fct[it] = fst[it] = __float2bfloat16_rn(0.f);
      if (w < G * HALF) {
        const int g = w / HALF, i = w % HALF;
        const bf16* qh = qrow + g * DH;
        if (c.rope_interleaved) {
          fq0[it] = *reinterpret_cast<const uint32_t*>(qh + 2 * i);
        } else {
          const int pi = 2 * i < HALF ? 2 * i : 2 * i - HALF;
          fq0[it] = *reinterpret_cast<const uint32_t*>(qh + pi);
          fq1[it] = *reinterpret_cast<const uint32_t*>(qh + pi + HALF);
        }
        fct[it] = ((const bf16*)p.cos_t)[(h * G + g) * HALF + i];
        fst[it] = ((const bf16*)p.sin_t)[(h * G + g) * HALF + i];
      }
    }
    if (tid < G) flam_raw = ((const bf16*)p.lam_logit)[(long long)b * p.lam_bs + h * G + tid];
  }
  const RingNow r = ring_after(p.rp, W, nsteps);
  const bool full = r.filled >= W;
  const int ev = full ? r.idx : r.filled;                 // the ring slot the new token takes
  // ---- cos / sin of the position, gate ----
  const bool abf = c.angle_dtype == CODA_BF16;
  if (tid < DH / 2) {
    float ta = (float)r.pos, inv = inv_f;
    if (abf) { ta = bf16_round(ta); inv = bf16_round(inv); }
    float ang = __fmul_rn(ta, inv);
    if (abf) ang = bf16_round(ang);
    float cc, ss; sincos_call(ang, &ss, &cc);
    if (abf) { cc = bf16_round(cc); ss = bf16_round(ss); }
    cs[tid] = El<T>::rnd(cc); sn[tid] = El<T>::rnd(ss);
  }
#pragma unroll
  for (int a = 0; a < 4; ++a) { const int m = tid + a * NT; if (m < Lbuf) s_al[m] = alr[a]; }
  asm volatile("bar.sync 1, 256;" ::: "memory");         // the eight working warps only
  // ---- key: RoPE (primitives.py:99-113), ring slot ----
  if (is_k) {
    const float nk_a = __bfloat162float(nk_a_raw), nk_b = __bfloat162float(nk_b_raw);
    const float cc = cs[ri], ss = sn[ri];
    float new_k;
    if (c.rope_interleaved) new_k = (d & 1) ? t_add<T>(t_mul<T>(nk_a, ss), t_mul<T>(nk_b, cc)) : t_sub<T>(t_mul<T>(nk_a, cc), t_mul<T>(nk_b, ss));
    else new_k = d < LF ? t_add<T>(t_mul<T>(nk_a, cc), t_mul<T>(-nk_b, ss)) : t_add<T>(t_mul<T>(nk_b, cc), t_mul<T>(nk_a, ss));
    El<T>::st(kb + (long long)ev * DH + d, new_k);
  }
  if (is_v) vb[(long long)ev * DH + d] = nv_raw;
  if (h == 0 && tid == 0) {
    gr[ev] = c.gated ? t_sigmoid<T>(__bfloat162float(glog_raw)) : 1.0f;
    if (!full) al[ev] = 1;
  }
  // ---- decode record of this plane: queries, lambda, visibility mask after the write ----
  unsigned char* rec = p.qrec + ((long long)b * Hkv + h) * DecodeRecord::bytes(G, DH, Lbuf);
  bf16* q_s = reinterpret_cast<bf16*>(rec);
#pragma unroll
  for (int it = 0; it < QI; ++it) {
    const int w = tid + it * NT;
    if (w < G * HALF) {
      const int g = w / HALF, i = w % HALF;
      const float a0 = __uint_as_float(fq0[it] << 16), a1 = __uint_as_float(fq0[it] & 0xffff0000u);
      const float b0 = __uint_as_float(fq1[it] << 16), b1 = __uint_as_float(fq1[it] & 0xffff0000u);
      float e0, e1;
      if (c.rope_interleaved) {
        e0 = t_sub<T>(t_mul<T>(a0, cs[i]), t_mul<T>(a1, sn[i]));
        e1 = t_add<T>(t_mul<T>(a0, sn[i]), t_mul<T>(a1, cs[i]));
      } else {
        const bool lo = 2 * i < HALF;
        const int pi = lo ? 2 * i : 2 * i - HALF;
        e0 = lo ? t_add<T>(t_mul<T>(a0, cs[pi]), t_mul<T>(-b0, sn[pi])) : t_add<T>(t_mul<T>(b0, cs[pi]), t_mul<T>(a0, sn[pi]));
        e1 = lo ? t_add<T>(t_mul<T>(a1, cs[pi + 1]), t_mul<T>(-b1, sn[pi + 1])) : t_add<T>(t_mul<T>(b1, cs[pi + 1]), t_mul<T>(a1, sn[pi + 1]));
      }
      const float ct = __bfloat162float(fct[it]), st = __bfloat162float(fst[it]);
      const float n0 = t_sub<T>(t_mul<T>(e0, ct), t_mul<T>(e1, st));
      const float n1 = t_add<T>(t_mul<T>(e0, st), t_mul<T>(e1, ct));
      *reinterpret_cast<__nv_bfloat162*>(q_s + g * QSTR + 2 * i) = __floats2bfloat162_rn(e0, e1);
      *reinterpret_cast<__nv_bfloat162*>(q_s + (G + g) * QSTR + 2 * i) = __floats2bfloat162_rn(n0, n1);
    }
  }
  const int rows = DecodeRecord::qrows(G);
  #pragma unroll 1
  for (int w = tid; w < (rows - 2 * G) * HALF; w += NT)   // unused rows of the query tile: zero
    *reinterpret_cast<uint32_t*>(q_s + (2 * G + w / HALF) * QSTR + 2 * (w % HALF)) = 0u;
  float* lam = reinterpret_cast<float*>(rec + DecodeRecord::lam_off(G, DH));
  if (tid < 8) lam[tid] = tid < G ? t_sigmoid<T>(__bfloat162float(flam_raw)) : 0.f;
  uint8_t* mk = rec + DecodeRecord::mask_off(G, DH);
  #pragma unroll 1
  for (int i = tid; i < DecodeRecord::mask_bytes(Lbuf); i += NT) mk[i] = i < Lbuf ? (i == ev ? (uint8_t)1 : s_al[i]) : (uint8_t)0;
}

template <typename T, int DH, int MODE>
__global__ void __launch_bounds__(256) step_write_cluster_kernel(StepParams p) { step_cluster_body<T, DH, MODE>(p); }

// Routing (MODE 1) of MANY layers' states in one launch: blockIdx.z picks the layer's parameter block from a
// device array.  The routing of one layer is a latency chain that keeps an SM's resources while it waits; all
// layers' chains side by side fill the machine and are bounded by memory bandwidth instead.
template <typename T, int DH, bool STAGE, int NCTA>
__global__ void __launch_bounds__(256, NCTA) step_route_batched_kernel(const StepParams* __restrict__ layers) {
  __shared__ StepParams sp;
  static_assert(sizeof(StepParams) % 4 == 0, "StepParams is copied word by word");
  const uint32_t* src = reinterpret_cast<const uint32_t*>(layers + blockIdx.z);
  for (int i = threadIdx.x; i < (int)(sizeof(StepParams) / 4); i += 256) reinterpret_cast<uint32_t*>(&sp)[i] = src[i];
  __syncthreads();
  step_cluster_body<T, DH, 1, STAGE>(sp);
}

template <typename T, int DH, int MODE>
static int launch_step_cluster(const StepParams& p, cudaStream_t s) {
  const coda_layer_cfg& c = p.c;
  const int MM = c.Me + c.Ms;
  const size_t smem = sizeof(float) * ((size_t)c.Hkv * MM + MM) + 8 + 8 * (size_t)c.Me + (size_t)(c.W + MM) + 16;
  cudaLaunchConfig_t lc = {};
  lc.gridDim = dim3(c.Hkv, c.B, 1);
  lc.blockDim = dim3(256, 1, 1);
  lc.dynamicSmemBytes = smem;
  lc.stream = s;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = c.Hkv; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
  lc.attrs = at; lc.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&lc, step_write_cluster_kernel<T, DH, MODE>, p);
  if (e != cudaSuccess) { coda_set_error("step_write (cluster): %s", cudaGetErrorString(e)); return CODA_ERR_LAUNCH; }
  return CODA_OK;
}

static int step_write_impl(const coda_layer_cfg* cfg, const coda_state_ptrs* st, coda_ring_pos rp,
                           const void* k_new, int64_t k_bs, const void* v_new, int64_t v_bs,
                           const float* gate, const float* eta_logit, int raw, const float* inv_freq,
                           const void* gate_logit, int64_t gate_bs, coda_stream_t stream,
                           const StepParams* fused = nullptr, int mode = 0) {
  CODA_REQUIRE(coda_cfg_ok(cfg) && st, CODA_ERR_ARG, "step_write: invalid layer configuration");
  CODA_REQUIRE(st->k_buf && st->v_buf && st->allowed && st->g_recent && (mode == 1 || (k_new && v_new)), CODA_ERR_ARG,
               "step_write: null pointer");
  CODA_REQUIRE(mode == 1 || (raw ? (inv_freq && (!cfg->gated || gate_logit)) : (gate != nullptr)), CODA_ERR_ARG,
               "step_write: gate / frequency inputs missing");
  CODA_REQUIRE(cfg->Me == 0 || (st->mem_last_exact && st->exact_v_norm), CODA_ERR_ARG, "step_write: exact bank pointers missing");
  CODA_REQUIRE(cfg->Ms == 0 || (st->sum_lf_k_norm && (mode == 2 || eta_logit)), CODA_ERR_ARG, "step_write: summary bank pointers missing");
  CODA_REQUIRE(rp.recent_idx >= 0 && rp.recent_idx < cfg->W && rp.recent_filled >= 0 && rp.recent_filled <= cfg->W,
               CODA_ERR_ARG, "step_write: ring scalars out of range");
  StepParams p; p.c = *cfg; p.st = *st; p.rp = rp;
  p.k_new = k_new; p.k_bs = k_bs; p.v_new = v_new; p.v_bs = v_bs; p.gate = gate; p.eta_logit = eta_logit;
  p.raw = raw; p.inv_freq = inv_freq; p.gate_logit = gate_logit; p.gate_bs = gate_bs;
  p.q_raw = nullptr; p.q_bs = 0; p.lam_logit = nullptr; p.lam_bs = 0; p.cos_t = nullptr; p.sin_t = nullptr; p.qrec = nullptr;
  if (fused) {
    p.q_raw = fused->q_raw; p.q_bs = fused->q_bs; p.lam_logit = fused->lam_logit; p.lam_bs = fused->lam_bs;
    p.cos_t = fused->cos_t; p.sin_t = fused->sin_t; p.qrec = fused->qrec;
  }
  cudaStream_t s = (cudaStream_t)stream;
  {
    // cluster variant: one CTA per (state, head); needs a portable cluster size and vector-aligned cache rows
    const size_t es0 = cfg->dtype == CODA_F32 ? 4 : 2;
    const int MM = cfg->Me + cfg->Ms;
    const size_t csm = sizeof(float) * ((size_t)cfg->Hkv * MM + MM) + 8 + 8 * (size_t)cfg->Me + (size_t)(cfg->W + MM) + 16;
    const bool ok = cfg->Hkv <= 8 && (cfg->Dh == 64 || cfg->Dh == 128) && csm <= 40 * 1024 && cfg->B <= 65535 &&
                    cfg->W + MM <= 1024 && cfg->Me <= 256 &&
                    (cfg->Me == 0 || (uintptr_t)st->exact_v_norm % 16 == 0) && (cfg->Ms == 0 || (uintptr_t)st->sum_lf_k_norm % 16 == 0) &&
                    ((size_t)cfg->Dh / 4 * es0) % 16 == 0;
    if (ok) {
      p.stage = 0; p.stage_off = 0; p.status = nullptr;
      if (mode == 1) return cfg->Dh == 128 ? launch_step_cluster<bf16, 128, 1>(p, s) : launch_step_cluster<bf16, 64, 1>(p, s);
      if (mode == 2) {
        if (cfg->Dh == 128) step_append_kernel<128><<<dim3(cfg->Hkv, cfg->B), 288, 0, s>>>(p);
        else step_append_kernel<64><<<dim3(cfg->Hkv, cfg->B), 288, 0, s>>>(p);
        CODA_CHECK_LAUNCH("step_append");
        return CODA_OK;
      }
      if (cfg->dtype == CODA_F32) return cfg->Dh == 128 ? launch_step_cluster<float, 128, 0>(p, s) : launch_step_cluster<float, 64, 0>(p, s);
      return cfg->Dh == 128 ? launch_step_cluster<bf16, 128, 0>(p, s) : launch_step_cluster<bf16, 64, 0>(p, s);
    }
    CODA_REQUIRE(!fused && mode == 0, CODA_ERR_ARG, "step_write_fused: configuration not covered by the cluster kernel");
  }
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

// The fused write + query preparation runs on the cluster kernel only (bf16, Hkv <= 8, head_dim 64 / 128).
extern "C" int coda_b200_step_write_fused_supported(const coda_layer_cfg* cfg) {
  if (!coda_cfg_ok(cfg)) return 0;
  const int MM = cfg->Me + cfg->Ms, G = cfg->H / cfg->Hkv;
  const size_t csm = sizeof(float) * ((size_t)cfg->Hkv * MM + MM) + 8 + 8 * (size_t)cfg->Me + (size_t)(cfg->W + MM) + 16;
  return cfg->dtype == CODA_BF16 && cfg->Hkv <= 8 && G <= 8 && (cfg->Dh == 64 || cfg->Dh == 128) && csm <= 40 * 1024 &&
         cfg->B <= 65535 && cfg->W + MM <= 1024 && cfg->Me <= 256;
}

extern "C" int coda_b200_step_write_fused(const coda_layer_cfg* cfg, const coda_state_ptrs* st, coda_ring_pos rp,
                                          const void* k_raw, int64_t k_bs, const void* v_new, int64_t v_bs,
                                          const void* gate_logit, int64_t gate_bs, const float* inv_freq,
                                          const float* eta_logit,
                                          const void* q_raw, int64_t q_bs, const void* lam_logit, int64_t lam_bs,
                                          const void* cos_theta, const void* sin_theta, void* qrec,
                                          coda_stream_t stream) {
  CODA_REQUIRE(coda_b200_step_write_fused_supported(cfg), CODA_ERR_ARG,
               "step_write_fused: needs bf16, at most 8 KV heads and 8 query heads per KV head, head_dim 64 or 128");
  CODA_REQUIRE(q_raw && lam_logit && cos_theta && sin_theta && qrec && ((uintptr_t)qrec % 16 == 0) && ((uintptr_t)q_raw % 4 == 0) &&
               (q_bs % 2 == 0), CODA_ERR_ARG, "step_write_fused: query-side pointers missing or misaligned");
  CODA_REQUIRE(st && (cfg->Me == 0 || (uintptr_t)st->exact_v_norm % 16 == 0) && (cfg->Ms == 0 || (uintptr_t)st->sum_lf_k_norm % 16 == 0),
               CODA_ERR_ARG, "step_write_fused: routing caches must be 16-byte aligned");
  StepParams f;
  f.q_raw = q_raw; f.q_bs = q_bs; f.lam_logit = lam_logit; f.lam_bs = lam_bs; f.cos_t = cos_theta; f.sin_t = sin_theta;
  f.qrec = (unsigned char*)qrec;
  return step_write_impl(cfg, st, rp, k_raw, k_bs, v_new, v_bs, nullptr, eta_logit, 1, inv_freq, gate_logit, gate_bs, stream, &f);
}

// The same step in two launches (configurations of coda_b200_step_write_fused_supported): the routing of the
// token the ring is about to evict needs nothing of the new token ...
extern "C" int coda_b200_step_route(const coda_layer_cfg* cfg, const coda_state_ptrs* st, coda_ring_pos rp,
                                    const float* eta_logit, coda_stream_t stream) {
  CODA_REQUIRE(coda_b200_step_write_fused_supported(cfg), CODA_ERR_ARG,
               "step_route: needs bf16, at most 8 KV heads and 8 query heads per KV head, head_dim 64 or 128");
  CODA_REQUIRE(st && (cfg->Me == 0 || (uintptr_t)st->exact_v_norm % 16 == 0) && (cfg->Ms == 0 || (uintptr_t)st->sum_lf_k_norm % 16 == 0),
               CODA_ERR_ARG, "step_route: routing caches must be 16-byte aligned");
  return step_write_impl(cfg, st, rp, nullptr, 0, nullptr, 0, nullptr, eta_logit, 1, nullptr, nullptr, 0, stream, nullptr, 1);
}

// ... and the new token then takes the ring slot (and leaves its decode record), with the same `rp`.
extern "C" int coda_b200_step_append_fused(const coda_layer_cfg* cfg, const coda_state_ptrs* st, coda_ring_pos rp,
                                           const void* k_raw, int64_t k_bs, const void* v_new, int64_t v_bs,
                                           const void* gate_logit, int64_t gate_bs, const float* inv_freq,
                                           const void* q_raw, int64_t q_bs, const void* lam_logit, int64_t lam_bs,
                                           const void* cos_theta, const void* sin_theta, void* qrec,
                                           coda_stream_t stream) {
  CODA_REQUIRE(coda_b200_step_write_fused_supported(cfg), CODA_ERR_ARG,
               "step_append_fused: needs bf16, at most 8 KV heads and 8 query heads per KV head, head_dim 64 or 128");
  CODA_REQUIRE(q_raw && lam_logit && cos_theta && sin_theta && qrec && ((uintptr_t)qrec % 16 == 0) && ((uintptr_t)q_raw % 4 == 0) &&
               (q_bs % 2 == 0), CODA_ERR_ARG, "step_append_fused: query-side pointers missing or misaligned");
  CODA_REQUIRE(st && (cfg->Me == 0 || (uintptr_t)st->exact_v_norm % 16 == 0) && (cfg->Ms == 0 || (uintptr_t)st->sum_lf_k_norm % 16 == 0),
               CODA_ERR_ARG, "step_append_fused: routing caches must be 16-byte aligned");
  StepParams f;
  f.q_raw = q_raw; f.q_bs = q_bs; f.lam_logit = lam_logit; f.lam_bs = lam_bs; f.cos_t = cos_theta; f.sin_t = sin_theta;
  f.qrec = (unsigned char*)qrec;
  return step_write_impl(cfg, st, rp, k_raw, k_bs, v_new, v_bs, nullptr, nullptr, 1, inv_freq, gate_logit, gate_bs, stream, &f, 2);
}

// ---- routing of several layers' states in one launch -------------------------------------------------------
// A plan is the device array of per-layer parameter blocks the batched kernel indexes with blockIdx.z.  It is
// written once (pointers and ring scalars at that moment plus the device step counter, as for a captured
// step) and then serves every launch / graph replay.
extern "C" int64_t coda_b200_step_route_plan_bytes(int32_t n_layers) {
  return n_layers > 0 ? (int64_t)n_layers * (int64_t)sizeof(StepParams) : 0;
}

extern "C" int coda_b200_step_route_plan(const coda_layer_cfg* cfg, const coda_state_ptrs* sts, const coda_ring_pos* rps,
                                         const float* const* eta_logits, int32_t n_layers, void* plan_dev,
                                         coda_stream_t stream) {
  CODA_REQUIRE(coda_b200_step_write_fused_supported(cfg), CODA_ERR_ARG,
               "step_route_plan: needs bf16, at most 8 KV heads and 8 query heads per KV head, head_dim 64 or 128");
  CODA_REQUIRE(sts && rps && eta_logits && plan_dev && n_layers > 0 && n_layers <= 65535, CODA_ERR_ARG,
               "step_route_plan: null pointer or layer count out of range");
  std::vector<StepParams> host((size_t)n_layers);
  for (int i = 0; i < n_layers; ++i) {
    const coda_state_ptrs& st = sts[i];
    CODA_REQUIRE(st.k_buf && st.v_buf && st.allowed && st.g_recent, CODA_ERR_ARG, "step_route_plan: null state pointer (layer %d)", i);
    CODA_REQUIRE(cfg->Me == 0 || (st.mem_last_exact && st.exact_v_norm && (uintptr_t)st.exact_v_norm % 16 == 0), CODA_ERR_ARG,
                 "step_route_plan: exact bank pointers missing or misaligned (layer %d)", i);
    CODA_REQUIRE(cfg->Ms == 0 || (st.sum_lf_k_norm && eta_logits[i] && (uintptr_t)st.sum_lf_k_norm % 16 == 0), CODA_ERR_ARG,
                 "step_route_plan: summary bank pointers missing or misaligned (layer %d)", i);
    CODA_REQUIRE(rps[i].recent_idx >= 0 && rps[i].recent_idx < cfg->W && rps[i].recent_filled >= 0 && rps[i].recent_filled <= cfg->W,
                 CODA_ERR_ARG, "step_route_plan: ring scalars out of range (layer %d)", i);
    StepParams p;
    memset(&p, 0, sizeof(p));
    p.c = *cfg; p.st = st; p.rp = rps[i]; p.eta_logit = eta_logits[i]; p.raw = 1;
    host[(size_t)i] = p;
  }
  cudaStream_t s = (cudaStream_t)stream;
  cudaError_t e = cudaMemcpyAsync(plan_dev, host.data(), host.size() * sizeof(StepParams), cudaMemcpyHostToDevice, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);       // `host` goes away with this call
  if (e != cudaSuccess) { coda_set_error("step_route_plan: %s", cudaGetErrorString(e)); return CODA_ERR_LAUNCH; }
  return CODA_OK;
}

extern "C" int coda_b200_step_route_batched(const coda_layer_cfg* cfg, const void* plan_dev, int32_t n_layers,
                                            coda_stream_t stream) {
  CODA_REQUIRE(coda_b200_step_write_fused_supported(cfg), CODA_ERR_ARG,
               "step_route_batched: needs bf16, at most 8 KV heads and 8 query heads per KV head, head_dim 64 or 128");
  CODA_REQUIRE(plan_dev && n_layers > 0 && n_layers <= 65535 && (uintptr_t)plan_dev % 8 == 0, CODA_ERR_ARG,
               "step_route_batched: plan missing or layer count out of range");
  const int MM = cfg->Me + cfg->Ms;
  cudaLaunchConfig_t lc = {};
  lc.gridDim = dim3(cfg->Hkv, cfg->B, n_layers);
  lc.blockDim = dim3(256, 1, 1);
  lc.dynamicSmemBytes = sizeof(float) * ((size_t)cfg->Hkv * MM + MM) + 8 + 8 * (size_t)cfg->Me + (size_t)(cfg->W + MM) + 16;
  lc.stream = (cudaStream_t)stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = cfg->Hkv; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
  lc.attrs = at; lc.numAttrs = 1;
  const StepParams* plan = (const StepParams*)plan_dev;
  // both routing caches of a head in shared memory when they fit beside the rest (six CTAs per SM at the 7B shape)
  const size_t stage_bytes = ((size_t)cfg->Me * cfg->Dh + (size_t)cfg->Ms * (cfg->Dh - cfg->Dh / 2)) * 2;
  const bool stage = stage_bytes > 0 && stage_bytes % 16 == 0 && ((size_t)cfg->Me * cfg->Dh * 2) % 16 == 0 &&
                     lc.dynamicSmemBytes + 16 + stage_bytes <= 30 * 1024;
  cudaError_t e;
  if (stage) {
    lc.dynamicSmemBytes += 16 + stage_bytes;
    // five CTAs per SM measured best at the 7B shape (4: 122 us, 5: 111 us, 6: 114 us for 32 layers x 32 states)
    e = cfg->Dh == 128 ? cudaLaunchKernelEx(&lc, step_route_batched_kernel<bf16, 128, true, 5>, plan)
                       : cudaLaunchKernelEx(&lc, step_route_batched_kernel<bf16, 64, true, 5>, plan);
  } else {
    e = cfg->Dh == 128 ? cudaLaunchKernelEx(&lc, step_route_batched_kernel<bf16, 128, false, 4>, plan)
                       : cudaLaunchKernelEx(&lc, step_route_batched_kernel<bf16, 64, false, 4>, plan);
  }
  if (e != cudaSuccess) { coda_set_error("step_route_batched: %s", cudaGetErrorString(e)); return CODA_ERR_LAUNCH; }
  return CODA_OK;
}
