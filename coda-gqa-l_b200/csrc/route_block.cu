// Bank + ring update with one prefill block, as three launches:
//   route_score   grid (candidate groups, B): cosine scores of each candidate against the
//                 routing caches as they were before the block; per candidate the best exact
//                 slot/score and the summary argmax go to a small global scratch.
//   route_commit  grid (B): the order-dependent decisions (LRU victim ranking, novel-rank
//                 assignment, stamps) on one thread, then the slot writes and cache re-normalisation.
//   ring_rewrite  grid (Hkv, B): kept ring rows shift to the front, the block's tail is appended.
// Semantics: upstream memory_banks.py:438-564 (block write), 633-742 (exact), 853-932 (summary).
#include "coda_common.cuh"
#include "topk_order.h"

struct RouteParams {
  coda_layer_cfg c;
  coda_state_ptrs st;
  int fill, blk, n_ev, te, ts;          // ring occupancy before the block; evicted count; candidates used
  long long pos_first;                  // position of evicted token 0
  const void* kblk; long long kb_bs, kb_rs;
  const void* vblk; long long vb_bs, vb_rs;
  const float* gates; long long gates_bs, gate_ev0;
  const int* cand; long long cand_bs;
  const float* eta_logit;
  float* ex_best; int* ex_bi; int* su_idx;   // scratch: [B][Te], [B][Te], [B][Ts]
};

// Row of evicted token e (ring slot e when e < fill, else row e-fill of the block), head h.
template <typename T>
__device__ __forceinline__ const T* src_row(const RouteParams& p, const void* buf, const void* blkp,
                                            long long bbs, long long brs, int b, int e, int h) {
  const int Lbuf = p.c.W + p.c.Me + p.c.Ms, Dh = p.c.Dh;
  if (e < p.fill) return (const T*)buf + (((long long)b * p.c.Hkv + h) * Lbuf + e) * Dh;
  return (const T*)blkp + (long long)b * bbs + (long long)(e - p.fill) * brs + (long long)h * Dh;
}

constexpr int RS_WARPS = 8;

template <typename T>
__global__ void __launch_bounds__(RS_WARPS * 32) route_score_kernel(RouteParams p) {
  extern __shared__ float sm[];
  const coda_layer_cfg& c = p.c;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int b = blockIdx.y;
  const int Hkv = c.Hkv, Dh = c.Dh, lf = Dh / 2, lfd = Dh - lf, Me = c.Me, Ms = c.Ms, W = c.W;
  const int ge = (p.te + RS_WARPS - 1) / RS_WARPS;          // groups of exact candidates
  const bool exact = (int)blockIdx.x < ge;
  const int t = (exact ? blockIdx.x : blockIdx.x - ge) * RS_WARPS + warp;
  if (t >= (exact ? p.te : p.ts)) return;
  float* hat = sm + (size_t)warp * Hkv * Dh;                // this warp's unit-norm candidate
  const int e = p.cand[(long long)b * p.cand_bs + t];
  const uint8_t* al = p.st.allowed + (long long)b * (W + Me + Ms);
  if (exact) {
    for (int h = 0; h < Hkv; ++h) {                         // v_hat = v / max(||v||, 1e-6)  (:498)
      const T* row = src_row<T>(p, p.st.v_buf, p.vblk, p.vb_bs, p.vb_rs, b, e, h);
      float ss = 0.f;
      for (int d = lane; d < Dh; d += 32) { const float v = El<T>::ld(row + d); hat[h * Dh + d] = v; ss += v * v; }
      const float den = fmaxf(El<T>::rnd(sqrtf(warp_sum(ss))), 1e-6f);
      for (int d = lane; d < Dh; d += 32) hat[h * Dh + d] = t_div<T>(hat[h * Dh + d], den);
    }
    __syncwarp();
    const T* vnorm = (const T*)p.st.exact_v_norm + (long long)b * Hkv * Me * Dh;
    float best = 0.f; int bi = 0;
    for (int m = 0; m < Me; ++m) {
      float tot = 0.f;
      for (int h = 0; h < Hkv; ++h) {
        const T* row = vnorm + ((long long)h * Me + m) * Dh;
        float part = 0.f;
        for (int d = lane; d < Dh; d += 32) part += hat[h * Dh + d] * El<T>::ld(row + d);
        tot += El<T>::rnd(warp_sum(part));
      }
      float s = El<T>::rnd(tot / (float)Hkv);
      if (m >= c.active_exact || !al[W + m]) s = -1e9f;      // (:646-650)
      if (m == 0 || s > best) { best = s; bi = m; }
    }
    if (lane == 0) { p.ex_best[(long long)b * c.Te + t] = best; p.ex_bi[(long long)b * c.Te + t] = bi; }
  } else {
    for (int h = 0; h < Hkv; ++h) {                         // k_hat over the LF band (:500)
      const T* row = src_row<T>(p, p.st.k_buf, p.kblk, p.kb_bs, p.kb_rs, b, e, h) + lf;
      float ss = 0.f;
      for (int d = lane; d < lfd; d += 32) { const float v = El<T>::ld(row + d); hat[h * lfd + d] = v; ss += v * v; }
      const float den = fmaxf(El<T>::rnd(sqrtf(warp_sum(ss))), 1e-6f);
      for (int d = lane; d < lfd; d += 32) hat[h * lfd + d] = t_div<T>(hat[h * lfd + d], den);
    }
    __syncwarp();
    const T* knorm = (const T*)p.st.sum_lf_k_norm + (long long)b * Hkv * Ms * lfd;
    float best = 0.f; int bi = 0;
    for (int m = 0; m < Ms; ++m) {
      float tot = 0.f;
      for (int h = 0; h < Hkv; ++h) {
        const T* row = knorm + ((long long)h * Ms + m) * lfd;
        float part = 0.f;
        for (int d = lane; d < lfd; d += 32) part += hat[h * lfd + d] * El<T>::ld(row + d);
        tot += El<T>::rnd(warp_sum(part));
      }
      float s = El<T>::rnd(tot / (float)Hkv);
      if (m >= c.active_summary) s = -1e9f;                  // (:875-877)
      if (m == 0 || s > best) { best = s; bi = m; }
    }
    if (lane == 0) p.su_idx[(long long)b * c.Ts + t] = bi;
  }
}

template <typename T>
__global__ void __launch_bounds__(256) route_commit_kernel(RouteParams p) {
  extern __shared__ unsigned char smraw[];
  const coda_layer_cfg& c = p.c;
  const int b = blockIdx.x, tid = threadIdx.x, NT = blockDim.x, lane = tid & 31, warp = tid >> 5, NW = NT >> 5;
  const int Hkv = c.Hkv, Dh = c.Dh, HD = Hkv * Dh, lf = Dh / 2, lfd = Dh - lf;
  const int Me = c.Me, Ms = c.Ms, W = c.W, Lbuf = W + Me + Ms;
  const int te = p.te, ts = p.ts, tmax = te > ts ? te : ts;
  // shared layout
  typedef topk_order::Item<long long> It64;
  It64* lruq = reinterpret_cast<It64*>(smraw);                       // [Me]
  float* stash = reinterpret_cast<float*>(lruq + (Me > 0 ? Me : 1)); // [HD] new row for re-normalising
  float* c_g = stash + HD;                                           // [tmax] gates
  float* s_w = c_g + tmax;                                           // [ts] summary weights
  float* s_cnt = s_w + (ts > 0 ? ts : 1);                            // [Ms] per-slot weight sum
  int* c_e = reinterpret_cast<int*>(s_cnt + (Ms > 0 ? Ms : 1));      // [tmax] evicted index
  int* e_tgt = c_e + tmax;                                           // [te] exact target slot
  int* e_ow = e_tgt + (te > 0 ? te : 1);                             // [te] overwrite flag
  int* s_ord = e_ow + (te > 0 ? te : 1);                             // [ts] candidates grouped by slot
  int* s_start = s_ord + (ts > 0 ? ts : 1);                          // [Ms+1]
  int* s_was = s_start + Ms + 1;                                     // [Ms] slot was used before the block

  uint8_t* al = p.st.allowed + (long long)b * Lbuf;
  T* kb = (T*)p.st.k_buf + (long long)b * Hkv * Lbuf * Dh;
  T* vb = (T*)p.st.v_buf + (long long)b * Hkv * Lbuf * Dh;

  for (int t = tid; t < tmax; t += NT) {
    const int e = p.cand[(long long)b * p.cand_bs + t];
    c_e[t] = e;
    c_g[t] = p.gates[(long long)b * p.gates_bs + p.gate_ev0 + e];
  }
  __syncthreads();

  if (tid == 0 && te > 0 && Me > 0) {
    // ---- exact bank decisions (memory_banks.py:635-697) ----
    long long* last = (long long*)p.st.mem_last_exact + (long long)b * Me;
    const int Ae = c.active_exact;
    bool any_used = false;
    for (int m = 0; m < Me; ++m) {
      const bool used = al[W + m] != 0;
      any_used |= used;
      lruq[m].v = (used && m < Ae) ? last[m] : -(1LL << 62);
      lruq[m].i = m;
    }
    const int n_lru = te < Ae ? te : Ae;
    topk_order::topk_queue<long long, false>(lruq, Me, n_lru, true);   // victims = lruq[0..n_lru).i
    const float tn = El<T>::rnd(c.tau_novel), tm = El<T>::rnd(c.tau_match);
    int rank = -1;
    for (int t = 0; t < te; ++t) {
      const float best = p.ex_best[(long long)b * c.Te + t];
      const int bi = p.ex_bi[(long long)b * c.Te + t];
      const bool keep = c.gated ? (c_g[t] >= c.tau_gate_exact) : true;
      const bool novel = !any_used || best < tn;
      const bool hit = any_used && best >= tm;
      const bool nk = novel && keep;
      if (nk) ++rank;
      const bool capped = nk && rank < Ae;
      int r = rank < 0 ? 0 : rank;
      if (r > n_lru - 1) r = n_lru - 1 > 0 ? n_lru - 1 : 0;
      const int tgt = capped ? lruq[r].i : bi;
      const bool touch = keep && (!novel || capped);
      e_tgt[t] = tgt;
      e_ow[t] = (c.refresh_on_hit ? (keep && (capped || hit)) : capped) ? 1 : 0;
      // bit 1 of e_ow marks "touch" for the stamp pass below
      if (touch) e_ow[t] |= 2;
    }
    // stamps: per slot the largest position among touching candidates replaces the old stamp
    for (int t = 0; t < te; ++t) {
      if (!(e_ow[t] & 2)) continue;
      bool first = true;
      for (int u = 0; u < t; ++u) if ((e_ow[u] & 2) && e_tgt[u] == e_tgt[t]) { first = false; break; }
      if (!first) continue;
      long long mx = p.pos_first + c_e[t];
      for (int u = t + 1; u < te; ++u)
        if ((e_ow[u] & 2) && e_tgt[u] == e_tgt[t]) { const long long pu = p.pos_first + c_e[u]; if (pu > mx) mx = pu; }
      last[e_tgt[t]] = mx;
    }
  }
  if (tid == 32 % NT && ts > 0 && Ms > 0) {
    // ---- summary bank bookkeeping (memory_banks.py:880-885, 906): weights, per-slot lists ----
    for (int m = 0; m < Ms; ++m) { s_cnt[m] = 0.f; s_start[m] = 0; s_was[m] = al[W + Me + m] != 0; }
    s_start[Ms] = 0;
    for (int t = 0; t < ts; ++t) {
      float w = El<T>::rnd(c_g[t]);
      if (c.gated && !(c_g[t] >= c.tau_gate_summary)) w = 0.f;           // (:518-523)
      s_w[t] = w;
      const int m = p.su_idx[(long long)b * c.Ts + t];
      s_cnt[m] = t_add<T>(s_cnt[m], w);
      s_start[m + 1] += 1;
    }
    for (int m = 0; m < Ms; ++m) s_start[m + 1] += s_start[m];
    // stable grouping by slot (fill positions from a running cursor kept in s_ord's tail-free pass)
    for (int m = 0; m < Ms; ++m) {
      int w_ = s_start[m];
      for (int t = 0; t < ts; ++t) if (p.su_idx[(long long)b * c.Ts + t] == m) s_ord[w_++] = t;
    }
  }
  __syncthreads();

  // ---- exact bank writes (memory_banks.py:707-742) ----
  if (te > 0 && Me > 0) {
    T* vnorm = (T*)p.st.exact_v_norm + (long long)b * Hkv * Me * Dh;
    for (int t = 0; t < te; ++t) {
      if (!(e_ow[t] & 1)) continue;
      const int slot = e_tgt[t];
      bool leader = true;
      for (int u = 0; u < t; ++u) if ((e_ow[u] & 1) && e_tgt[u] == slot) { leader = false; break; }
      if (!leader) continue;                                             // CTA-uniform
      for (int e = tid; e < HD; e += NT) {
        const int h = e / Dh, d = e % Dh;
        T* pk = kb + ((long long)h * Lbuf + W + slot) * Dh + d;
        T* pv = vb + ((long long)h * Lbuf + W + slot) * Dh + d;
        const float ok = El<T>::ld(pk), ov = El<T>::ld(pv);
        float ck = 0.f, cv = 0.f;                                        // scatter_add of deltas, candidate order
        for (int u = t; u < te; ++u) {
          if (!(e_ow[u] & 1) || e_tgt[u] != slot) continue;
          const float xk = El<T>::ld(src_row<T>(p, p.st.k_buf, p.kblk, p.kb_bs, p.kb_rs, b, c_e[u], h) + d);
          const float xv = El<T>::ld(src_row<T>(p, p.st.v_buf, p.vblk, p.vb_bs, p.vb_rs, b, c_e[u], h) + d);
          ck = t_add<T>(ck, t_sub<T>(xk, ok));
          cv = t_add<T>(cv, t_sub<T>(xv, ov));
        }
        El<T>::st(pk, t_add<T>(ok, ck));
        const float nv = t_add<T>(ov, cv);
        El<T>::st(pv, nv);
        stash[e] = nv;
      }
      if (tid == 0) al[W + slot] = 1;
      __syncthreads();
      for (int h = warp; h < Hkv; h += NW) {
        float ss = 0.f;
        for (int d = lane; d < Dh; d += 32) { const float v = stash[h * Dh + d]; ss += v * v; }
        const float den = fmaxf(El<T>::rnd(sqrtf(warp_sum(ss))), 1e-6f);
        for (int d = lane; d < Dh; d += 32)
          El<T>::st(vnorm + ((long long)h * Me + slot) * Dh + d, t_div<T>(stash[h * Dh + d], den));
      }
      __syncthreads();
    }
  }

  // ---- summary bank EMA (memory_banks.py:887-932) ----
  if (ts > 0 && Ms > 0) {
    T* knorm = (T*)p.st.sum_lf_k_norm + (long long)b * Hkv * Ms * lfd;
    const float cmin = El<T>::rnd(1e-6f);
    for (int m = 0; m < Ms; ++m) {
      const float cnt = s_cnt[m];
      if (!(cnt > 0.f)) continue;                                        // CTA-uniform
      const int a0 = s_start[m], a1 = s_start[m + 1];
      const float cden = fmaxf(cnt, cmin);
      const bool fresh = c.overwrite_on_insert && !s_was[m];
      for (int e = tid; e < HD; e += NT) {
        const int h = e / Dh, d = e % Dh;
        float sk = 0.f, sv = 0.f;
        for (int a = a0; a < a1; ++a) {
          const int t = s_ord[a];
          const float w = s_w[t];
          const float xk = El<T>::ld(src_row<T>(p, p.st.k_buf, p.kblk, p.kb_bs, p.kb_rs, b, c_e[t], h) + d);
          const float xv = El<T>::ld(src_row<T>(p, p.st.v_buf, p.vblk, p.vb_bs, p.vb_rs, b, c_e[t], h) + d);
          sk = t_add<T>(sk, t_mul<T>(xk, w));
          sv = t_add<T>(sv, t_mul<T>(xv, w));
        }
        const float eta = fresh ? 1.f : t_sigmoid<T>(p.eta_logit[h]);
        T* pk = kb + ((long long)h * Lbuf + W + Me + m) * Dh + d;
        T* pv = vb + ((long long)h * Lbuf + W + Me + m) * Dh + d;
        const float ov = El<T>::ld(pv);
        El<T>::st(pv, t_add<T>(ov, t_mul<T>(eta, t_sub<T>(t_div<T>(sv, cden), ov))));
        if (d >= lf) {
          const float ok = El<T>::ld(pk);
          const float inc = El<T>::rnd(__fmul_rn(t_div<T>(sk, cden), c.energy_scale));
          const float nk = t_add<T>(ok, t_mul<T>(eta, t_sub<T>(inc, ok)));
          El<T>::st(pk, nk);
          stash[h * lfd + d - lf] = nk;
        }
      }
      if (tid == 0) al[W + Me + m] = 1;
      __syncthreads();
      for (int h = warp; h < Hkv; h += NW) {
        float ss = 0.f;
        for (int d = lane; d < lfd; d += 32) { const float v = stash[h * lfd + d]; ss += v * v; }
        const float den = fmaxf(El<T>::rnd(sqrtf(warp_sum(ss))), 1e-6f);
        for (int d = lane; d < lfd; d += 32)
          El<T>::st(knorm + ((long long)h * Ms + m) * lfd + d, t_div<T>(stash[h * lfd + d], den));
      }
      __syncthreads();
    }
  }
}

// Ring rewrite (memory_banks.py:152-177, 554-563): with the ring in chronological order the kept
// rows [drop, fill) move down to [0, fill-drop) and block rows [bstart, blk) follow them.
constexpr int RR_PER = 8;
template <typename T>
__global__ void __launch_bounds__(256) ring_rewrite_kernel(RouteParams p) {
  const coda_layer_cfg& c = p.c;
  const int h = blockIdx.x, b = blockIdx.y, tid = threadIdx.x, NT = blockDim.x;
  const int W = c.W, Dh = c.Dh, Lbuf = W + c.Me + c.Ms;
  const int drop = p.n_ev < p.fill ? p.n_ev : p.fill;
  const int kept = p.fill - drop;
  const int bstart = p.n_ev > p.fill ? p.n_ev - p.fill : 0;
  const int nnew = p.blk - bstart;
  for (int pass = 0; pass < 2; ++pass) {
    T* ring = (T*)(pass ? p.st.v_buf : p.st.k_buf) + ((long long)b * c.Hkv + h) * Lbuf * Dh;
    if (drop > 0 && kept > 0) {
      const long long n = (long long)kept * Dh, off = (long long)drop * Dh;
      for (long long c0 = 0; c0 < n; c0 += (long long)NT * RR_PER) {
        T tmp[RR_PER];
#pragma unroll
        for (int i = 0; i < RR_PER; ++i) { const long long x = c0 + (long long)i * NT + tid; if (x < n) tmp[i] = ring[off + x]; }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < RR_PER; ++i) { const long long x = c0 + (long long)i * NT + tid; if (x < n) ring[x] = tmp[i]; }
        __syncthreads();
      }
    }
    const T* src = (const T*)(pass ? p.vblk : p.kblk) + (long long)b * (pass ? p.vb_bs : p.kb_bs) + (long long)h * Dh;
    const long long rs = pass ? p.vb_rs : p.kb_rs;
    for (long long x = tid; x < (long long)nnew * Dh; x += NT) {
      const int r = (int)(x / Dh), d = (int)(x % Dh);
      ring[(long long)(kept + r) * Dh + d] = src[(long long)(bstart + r) * rs + d];
    }
  }
  if (h == 0) {
    float* gr = p.st.g_recent + (long long)b * W;
    uint8_t* al = p.st.allowed + (long long)b * Lbuf;
    if (drop > 0 && kept > 0) {
      for (int c0 = 0; c0 < kept; c0 += NT) {
        const int x = c0 + tid;
        float tmp = 0.f;
        if (x < kept) tmp = gr[drop + x];
        __syncthreads();
        if (x < kept) gr[x] = tmp;
        __syncthreads();
      }
    }
    const float* gsrc = p.gates + (long long)b * p.gates_bs + p.gate_ev0 + p.fill + bstart;
    for (int x = tid; x < nnew; x += NT) gr[kept + x] = gsrc[x];
    for (int x = tid; x < kept + nnew; x += NT) al[x] = 1;
  }
}

static size_t route_scratch_bytes(const coda_layer_cfg* c) {
  const size_t te = c->Te > 0 ? c->Te : 0, ts = c->Ts > 0 ? c->Ts : 0;
  return (size_t)c->B * (te * 8 + ts * 4) + 64;
}

extern "C" int64_t coda_b200_route_scratch_bytes(const coda_layer_cfg* cfg) {
  if (!coda_cfg_ok(cfg)) return -1;
  return (int64_t)route_scratch_bytes(cfg);
}

template <typename T>
static int launch_route(RouteParams& p, cudaStream_t s) {
  const coda_layer_cfg& c = p.c;
  const int HD = c.Hkv * c.Dh;
  if (p.te > 0 || p.ts > 0) {
    const int groups = (p.te + RS_WARPS - 1) / RS_WARPS + (p.ts + RS_WARPS - 1) / RS_WARPS;
    const size_t smem1 = sizeof(float) * (size_t)RS_WARPS * HD;
    CODA_REQUIRE(smem1 <= 200 * 1024, CODA_ERR_LIMIT, "route_block: Hkv*Dh = %d too large", HD);
    if (smem1 > 48 * 1024) cudaFuncSetAttribute(route_score_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1);
    route_score_kernel<T><<<dim3(groups, c.B), RS_WARPS * 32, smem1, s>>>(p);
    CODA_CHECK_LAUNCH("route_block (score)");
    const int tmax = p.te > p.ts ? p.te : p.ts;
    const size_t smem2 = 16 * (size_t)(c.Me > 0 ? c.Me : 1) + 4 * ((size_t)HD + tmax + (p.ts > 0 ? p.ts : 1) + (c.Ms > 0 ? c.Ms : 1) +
                         tmax + 2 * (size_t)(p.te > 0 ? p.te : 1) + (p.ts > 0 ? p.ts : 1) + c.Ms + 1 + c.Ms) + 64;
    CODA_REQUIRE(smem2 <= 200 * 1024, CODA_ERR_LIMIT, "route_block: commit stage needs %zu bytes of shared memory", smem2);
    if (smem2 > 48 * 1024) cudaFuncSetAttribute(route_commit_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2);
    route_commit_kernel<T><<<c.B, 256, smem2, s>>>(p);
    CODA_CHECK_LAUNCH("route_block (commit)");
  }
  ring_rewrite_kernel<T><<<dim3(c.Hkv, c.B), 256, 0, s>>>(p);
  CODA_CHECK_LAUNCH("route_block (ring)");
  return CODA_OK;
}

extern "C" int coda_b200_route_block(const coda_layer_cfg* cfg, const coda_state_ptrs* st,
                                     int32_t ring_fill, int32_t blk, int64_t pos0,
                                     const void* k_blk, int64_t kb_bs, int64_t kb_rs,
                                     const void* v_blk, int64_t vb_bs, int64_t vb_rs,
                                     const float* gates, int64_t gates_bs, int64_t gate_ev0,
                                     const int32_t* cand, int64_t cand_bs,
                                     const float* eta_logit, void* scratch, coda_stream_t stream) {
  CODA_REQUIRE(coda_cfg_ok(cfg) && st, CODA_ERR_ARG, "route_block: invalid layer configuration");
  CODA_REQUIRE(blk > 0 && ring_fill >= 0 && ring_fill <= cfg->W, CODA_ERR_ARG, "route_block: bad block / ring sizes");
  CODA_REQUIRE(st->k_buf && st->v_buf && st->allowed && st->g_recent && k_blk && v_blk && gates, CODA_ERR_ARG,
               "route_block: null pointer");
  RouteParams p;
  p.c = *cfg; p.st = *st; p.fill = ring_fill; p.blk = blk;
  const int total = ring_fill + blk;
  const int keep = total < cfg->W ? total : cfg->W;
  p.n_ev = total - keep;
  const bool do_e = cfg->Me > 0 && cfg->Te > 0, do_s = cfg->Ms > 0 && cfg->Ts > 0;
  p.te = do_e ? (cfg->Te < p.n_ev ? cfg->Te : p.n_ev) : 0;
  p.ts = do_s ? (cfg->Ts < p.n_ev ? cfg->Ts : p.n_ev) : 0;
  p.pos_first = pos0 - ring_fill;
  p.kblk = k_blk; p.kb_bs = kb_bs; p.kb_rs = kb_rs; p.vblk = v_blk; p.vb_bs = vb_bs; p.vb_rs = vb_rs;
  p.gates = gates; p.gates_bs = gates_bs; p.gate_ev0 = gate_ev0;
  p.cand = cand; p.cand_bs = cand_bs; p.eta_logit = eta_logit;
  if (p.te > 0 || p.ts > 0) {
    CODA_REQUIRE(cand && scratch, CODA_ERR_ARG, "route_block: candidate list / scratch missing");
    CODA_REQUIRE(!do_e || (st->mem_last_exact && st->exact_v_norm), CODA_ERR_ARG, "route_block: exact bank pointers missing");
    CODA_REQUIRE(!do_s || (st->sum_lf_k_norm && eta_logit), CODA_ERR_ARG, "route_block: summary bank pointers missing");
    const size_t te_all = cfg->Te > 0 ? cfg->Te : 0;
    char* sp = (char*)scratch;
    p.ex_best = (float*)sp; sp += (size_t)cfg->B * te_all * 4;
    p.ex_bi = (int*)sp; sp += (size_t)cfg->B * te_all * 4;
    p.su_idx = (int*)sp;
  } else {
    p.ex_best = nullptr; p.ex_bi = nullptr; p.su_idx = nullptr;
  }
  cudaStream_t s = (cudaStream_t)stream;
  return cfg->dtype == CODA_F32 ? launch_route<float>(p, s) : launch_route<bf16>(p, s);
}
