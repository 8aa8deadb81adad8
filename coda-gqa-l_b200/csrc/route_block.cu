// Bank + ring update with one prefill block, as four launches:
//   route_score   grid (2, B): cosine scores of every candidate against the routing caches as they were
//                 before the block (a register-tiled fp32 mini-GEMM per bank); per candidate the best
//                 exact slot/score and the summary argmax go to a small global scratch.
//   route_decide  grid (B): the order-dependent decisions (LRU victim ranking, novel-rank assignment,
//                 stamps, per-slot candidate lists) -> a small per-state plan in global scratch.
//   route_apply   grid (written slots, B): one CTA per written bank slot: values + cache re-normalisation.
//   ring_rewrite  grid (2*Hkv, B): kept ring rows shift to the front, the block's tail is appended.
// Semantics: upstream memory_banks.py:438-564 (block write), 633-742 (exact), 853-932 (summary).
#include "coda_common.cuh"
#include "topk_order.h"
#include "tma_utils.cuh"
#include "bank_score.cuh"
#include <mutex>

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
  int* plan;                                 // scratch: per-state plan (see Plan)
};

// Row of evicted token e (ring slot e when e < fill, else row e-fill of the block), head h.
template <typename T>
__device__ __forceinline__ const T* src_row(const RouteParams& p, const void* buf, const void* blkp,
                                            long long bbs, long long brs, int b, int e, int h) {
  const int Lbuf = p.c.W + p.c.Me + p.c.Ms, Dh = p.c.Dh;
  if (e < p.fill) return (const T*)buf + (((long long)b * p.c.Hkv + h) * Lbuf + e) * Dh;
  return (const T*)blkp + (long long)b * bbs + (long long)(e - p.fill) * brs + (long long)h * Dh;
}

// ---- scores: a register-tiled fp32 mini-GEMM per state and bank ----
// S[candidate][slot] = mean over heads of the dtype-rounded per-head dot products of the unit-norm candidate
// with the bank's unit-norm cache row; the kernel keeps only the row-wise first-index argmax (and, for the
// exact bank, the best score).  Grid (2, B): x = 0 exact bank (V rows, n = Dh), x = 1 summary bank (LF half of
// the K rows, n = Dh/2).  Tiles: RS_ROWS candidates x 64 slots x 64-element K chunks of one head, staged
// transposed ([k][row]) in shared memory as fp32; 256 threads, each TM x 4 outputs.
constexpr int RS_KC = 64;
constexpr int RS_COLS = 64;

template <typename T, int TM>
__device__ __forceinline__ void route_score_bank(const RouteParams& p, int b, bool exact, float* sm) {
  constexpr int ROWS = 16 * TM;
  const coda_layer_cfg& c = p.c;
  const int tid = threadIdx.x;
  const int Hkv = c.Hkv, Dh = c.Dh, lf = Dh / 2, W = c.W, Me = c.Me, Ms = c.Ms;
  const int n = exact ? Dh : Dh - lf, M = exact ? Me : Ms, Tn = exact ? p.te : p.ts;
  const int active = exact ? c.active_exact : c.active_summary;
  const T* cache = exact ? (const T*)p.st.exact_v_norm + (long long)b * Hkv * Me * Dh
                         : (const T*)p.st.sum_lf_k_norm + (long long)b * Hkv * Ms * n;
  const uint8_t* al = p.st.allowed + (long long)b * (W + Me + Ms);
  float* As = sm;                                  // [RS_KC][ROWS]
  float* Bs = As + RS_KC * ROWS;                   // [RS_KC][RS_COLS]
  float* Ss = Bs + RS_KC * RS_COLS;                // [ROWS][RS_COLS + 1]
  float* den = Ss + ROWS * (RS_COLS + 1);          // [ROWS][Hkv]
  int* cidx = reinterpret_cast<int*>(den + ROWS * Hkv);   // [ROWS]
  const int ty = tid >> 4, tx = tid & 15;          // 16 x 16 thread grid

  for (int r0 = 0; r0 < Tn; r0 += ROWS) {
    const int nrows = min(ROWS, Tn - r0);
    __syncthreads();
    for (int r = tid; r < ROWS; r += 256) cidx[r] = r < nrows ? p.cand[(long long)b * p.cand_bs + r0 + r] : -1;
    __syncthreads();
    // ||x|| of every (candidate, head) of the tile: one thread per pair, batched loads  (memory_banks.py:498-500)
    for (int it = tid; it < ROWS * Hkv; it += 256) {
      const int r = it / Hkv, h = it % Hkv;
      float ss = 0.f;
      if (cidx[r] >= 0) {
        const T* row = exact ? src_row<T>(p, p.st.v_buf, p.vblk, p.vb_bs, p.vb_rs, b, cidx[r], h)
                             : src_row<T>(p, p.st.k_buf, p.kblk, p.kb_bs, p.kb_rs, b, cidx[r], h) + lf;
        int d = 0;
        for (; d + 16 <= n; d += 16) {
          float x[16];
          load_run<T, 16>(row + d, x);
#pragma unroll
          for (int i = 0; i < 16; ++i) ss = fmaf(x[i], x[i], ss);
        }
        for (; d < n; ++d) { const float v = El<T>::ld(row + d); ss = fmaf(v, v, ss); }
      }
      den[it] = fmaxf(El<T>::rnd(sqrtf(ss)), 1e-6f);
    }
    float best = 0.f; int bi = 0;                  // running first-index argmax of row `tid` (tid < ROWS)
    for (int c0 = 0; c0 < M; c0 += RS_COLS) {
      float tot[TM][4];
#pragma unroll
      for (int i = 0; i < TM; ++i) { tot[i][0] = tot[i][1] = tot[i][2] = tot[i][3] = 0.f; }
      for (int h = 0; h < Hkv; ++h) {
        float acc[TM][4];
#pragma unroll
        for (int i = 0; i < TM; ++i) { acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f; }
        for (int k0 = 0; k0 < n; k0 += RS_KC) {
          __syncthreads();
          // stage: candidates (normalised, dtype-rounded) and cache rows, both transposed to [k][row];
          // every thread owns a run of KRUN consecutive k of one row and loads it in one batch
          {
            constexpr int KRUN_A = RS_KC * ROWS / 256;          // 16 (64-row tile) or 4 (16-row tile)
            const int r = tid % ROWS, kq0 = (tid / ROWS) * KRUN_A;
            float x[KRUN_A];
#pragma unroll
            for (int i = 0; i < KRUN_A; ++i) x[i] = 0.f;
            if (cidx[r] >= 0) {
              const T* row = exact ? src_row<T>(p, p.st.v_buf, p.vblk, p.vb_bs, p.vb_rs, b, cidx[r], h)
                                   : src_row<T>(p, p.st.k_buf, p.kblk, p.kb_bs, p.kb_rs, b, cidx[r], h) + lf;
              if (k0 + kq0 + KRUN_A <= n) load_run<T, KRUN_A>(row + k0 + kq0, x);
              else
                for (int i = 0; i < KRUN_A; ++i) if (k0 + kq0 + i < n) x[i] = El<T>::ld(row + k0 + kq0 + i);
              const float dn = den[r * Hkv + h];
#pragma unroll
              for (int i = 0; i < KRUN_A; ++i) x[i] = t_div<T>(x[i], dn);
            }
#pragma unroll
            for (int i = 0; i < KRUN_A; ++i) As[(kq0 + i) * ROWS + r] = x[i];
          }
          {
            constexpr int KRUN_B = RS_KC * RS_COLS / 256;       // 16
            const int col = tid % RS_COLS, kq0 = (tid / RS_COLS) * KRUN_B, m = c0 + col;
            float x[KRUN_B];
#pragma unroll
            for (int i = 0; i < KRUN_B; ++i) x[i] = 0.f;
            if (m < M) {
              const T* row = cache + ((long long)h * M + m) * n;
              if (k0 + kq0 + KRUN_B <= n) load_run<T, KRUN_B>(row + k0 + kq0, x);
              else
                for (int i = 0; i < KRUN_B; ++i) if (k0 + kq0 + i < n) x[i] = El<T>::ld(row + k0 + kq0 + i);
            }
#pragma unroll
            for (int i = 0; i < KRUN_B; ++i) Bs[(kq0 + i) * RS_COLS + col] = x[i];
          }
          __syncthreads();
#pragma unroll 8
          for (int kq = 0; kq < RS_KC; ++kq) {
            float a[TM];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[kq * ROWS + ty * TM + i];
            const float4 bv = *reinterpret_cast<const float4*>(Bs + kq * RS_COLS + tx * 4);
#pragma unroll
            for (int i = 0; i < TM; ++i) {
              acc[i][0] = fmaf(a[i], bv.x, acc[i][0]); acc[i][1] = fmaf(a[i], bv.y, acc[i][1]);
              acc[i][2] = fmaf(a[i], bv.z, acc[i][2]); acc[i][3] = fmaf(a[i], bv.w, acc[i][3]);
            }
          }
        }
#pragma unroll
        for (int i = 0; i < TM; ++i)
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) tot[i][jj] += El<T>::rnd(acc[i][jj]);
      }
      __syncthreads();
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
          const int m = c0 + tx * 4 + jj;
          float s = El<T>::rnd(tot[i][jj] / (float)Hkv);
          if (m >= M) s = -INFINITY;                                   // padding column: never wins
          else if (m >= active || (exact && !al[W + m])) s = -1e9f;    // (:646-650, :875-877)
          Ss[(ty * TM + i) * (RS_COLS + 1) + tx * 4 + jj] = s;
        }
      __syncthreads();
      if (tid < nrows) {
        for (int col = 0; col < RS_COLS && c0 + col < M; ++col) {
          const float s = Ss[tid * (RS_COLS + 1) + col];
          if ((c0 == 0 && col == 0) || s > best) { best = s; bi = c0 + col; }
        }
      }
    }
    if (tid < nrows) {
      if (exact) { p.ex_best[(long long)b * c.Te + r0 + tid] = best; p.ex_bi[(long long)b * c.Te + r0 + tid] = bi; }
      else p.su_idx[(long long)b * c.Ts + r0 + tid] = bi;
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256) route_score_kernel(RouteParams p) {
  extern __shared__ float sm[];
  const bool exact = blockIdx.x == 0;
  if (exact) { if (p.te > 0 && p.c.Me > 0) route_score_bank<T, 1>(p, blockIdx.y, true, sm); }
  else if (p.ts > 0 && p.c.Ms > 0) route_score_bank<T, 4>(p, blockIdx.y, false, sm);
}

// ---- the same scores with the KV heads side by side: one CTA per (bank, state, head), the heads of a state in one cluster ----
// route_score_bank walks the heads one after the other (2 x Hkv tile loads per output tile, each a memory round
// trip); here CTA h computes head h's rounded dot products only, leaves them in its shared memory, and after one
// cluster barrier every CTA finishes the output rows r with r % Hkv == h: it adds the Hkv partials in head order
// (the order route_score_bank adds them in, so the results are the same bits), takes the mean, applies the slot
// masks and keeps the running first-index argmax of its rows.
template <typename T, int TM>
__device__ __forceinline__ void route_score_bank_heads(const RouteParams& p, int b, bool exact, float* sm) {
  constexpr int ROWS = 16 * TM;
  const coda_layer_cfg& c = p.c;
  const int tid = threadIdx.x, h = blockIdx.z;
  const int Hkv = c.Hkv, Dh = c.Dh, lf = Dh / 2, W = c.W, Me = c.Me, Ms = c.Ms;
  const int n = exact ? Dh : Dh - lf, M = exact ? Me : Ms, Tn = exact ? p.te : p.ts;
  const int active = exact ? c.active_exact : c.active_summary;
  const T* cache = exact ? (const T*)p.st.exact_v_norm + (long long)b * Hkv * Me * Dh
                         : (const T*)p.st.sum_lf_k_norm + (long long)b * Hkv * Ms * n;
  const uint8_t* al = p.st.allowed + (long long)b * (W + Me + Ms);
  float* As = sm;                                  // [RS_KC][ROWS]
  float* Bs = As + RS_KC * ROWS;                   // [RS_KC][RS_COLS]
  float* Ps = Bs + RS_KC * RS_COLS;                // [ROWS][RS_COLS]   this head's rounded dots (read by the whole cluster)
  float* Fs = Ps + ROWS * RS_COLS;                 // [ROWS / Hkv + 1][RS_COLS + 1]  final scores of the rows this CTA owns
  float* den = Fs + (ROWS / Hkv + 1) * (RS_COLS + 1);   // [ROWS]
  int* cidx = reinterpret_cast<int*>(den + ROWS);  // [ROWS]
  const int ty = tid >> 4, tx = tid & 15;          // 16 x 16 thread grid
  const int nown_max = ROWS / Hkv + 1;

  for (int r0 = 0; r0 < Tn; r0 += ROWS) {
    const int nrows = min(ROWS, Tn - r0);
    __syncthreads();
    for (int r = tid; r < ROWS; r += 256) cidx[r] = r < nrows ? p.cand[(long long)b * p.cand_bs + r0 + r] : -1;
    __syncthreads();
    // ||x|| of every candidate of the tile for this head, batched loads  (memory_banks.py:498-500).  One thread per
    // row (every fourth): the fp32 sum of squares runs over the elements in order, as route_score_bank's does.
    {
      const int r = tid >> 2, part = tid & 3;
      float ss = 0.f;
      if (r < ROWS && cidx[r] >= 0) {
        const T* row = exact ? src_row<T>(p, p.st.v_buf, p.vblk, p.vb_bs, p.vb_rs, b, cidx[r], h)
                             : src_row<T>(p, p.st.k_buf, p.kblk, p.kb_bs, p.kb_rs, b, cidx[r], h) + lf;
        if (part == 0) {
          int d = 0;
          for (; d + 16 <= n; d += 16) {
            float x[16];
            load_run<T, 16>(row + d, x);
#pragma unroll
            for (int i = 0; i < 16; ++i) ss = fmaf(x[i], x[i], ss);
          }
          for (; d < n; ++d) { const float v = El<T>::ld(row + d); ss = fmaf(v, v, ss); }
        }
      }
      if (r < ROWS && part == 0) den[r] = fmaxf(El<T>::rnd(sqrtf(ss)), 1e-6f);
    }
    float best = 0.f; int bi = 0;                  // running first-index argmax of owned row `tid` (tid < rows owned)
    for (int c0 = 0; c0 < M; c0 += RS_COLS) {
      float acc[TM][4];
#pragma unroll
      for (int i = 0; i < TM; ++i) { acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f; }
      for (int k0 = 0; k0 < n; k0 += RS_KC) {
        __syncthreads();
        {
          constexpr int KRUN_A = RS_KC * ROWS / 256;          // 16 (64-row tile) or 4 (16-row tile)
          const int r = tid % ROWS, kq0 = (tid / ROWS) * KRUN_A;
          float x[KRUN_A];
#pragma unroll
          for (int i = 0; i < KRUN_A; ++i) x[i] = 0.f;
          if (cidx[r] >= 0) {
            const T* row = exact ? src_row<T>(p, p.st.v_buf, p.vblk, p.vb_bs, p.vb_rs, b, cidx[r], h)
                                 : src_row<T>(p, p.st.k_buf, p.kblk, p.kb_bs, p.kb_rs, b, cidx[r], h) + lf;
            if (k0 + kq0 + KRUN_A <= n) load_run<T, KRUN_A>(row + k0 + kq0, x);
            else
              for (int i = 0; i < KRUN_A; ++i) if (k0 + kq0 + i < n) x[i] = El<T>::ld(row + k0 + kq0 + i);
            const float dn = den[r];
#pragma unroll
            for (int i = 0; i < KRUN_A; ++i) x[i] = t_div<T>(x[i], dn);
          }
#pragma unroll
          for (int i = 0; i < KRUN_A; ++i) As[(kq0 + i) * ROWS + r] = x[i];
        }
        {
          constexpr int KRUN_B = RS_KC * RS_COLS / 256;       // 16
          const int col = tid % RS_COLS, kq0 = (tid / RS_COLS) * KRUN_B, m = c0 + col;
          float x[KRUN_B];
#pragma unroll
          for (int i = 0; i < KRUN_B; ++i) x[i] = 0.f;
          if (m < M) {
            const T* row = cache + ((long long)h * M + m) * n;
            if (k0 + kq0 + KRUN_B <= n) load_run<T, KRUN_B>(row + k0 + kq0, x);
            else
              for (int i = 0; i < KRUN_B; ++i) if (k0 + kq0 + i < n) x[i] = El<T>::ld(row + k0 + kq0 + i);
          }
#pragma unroll
          for (int i = 0; i < KRUN_B; ++i) Bs[(kq0 + i) * RS_COLS + col] = x[i];
        }
        __syncthreads();
#pragma unroll 8
        for (int kq = 0; kq < RS_KC; ++kq) {
          float a[TM];
#pragma unroll
          for (int i = 0; i < TM; ++i) a[i] = As[kq * ROWS + ty * TM + i];
          const float4 bv = *reinterpret_cast<const float4*>(Bs + kq * RS_COLS + tx * 4);
#pragma unroll
          for (int i = 0; i < TM; ++i) {
            acc[i][0] = fmaf(a[i], bv.x, acc[i][0]); acc[i][1] = fmaf(a[i], bv.y, acc[i][1]);
            acc[i][2] = fmaf(a[i], bv.z, acc[i][2]); acc[i][3] = fmaf(a[i], bv.w, acc[i][3]);
          }
        }
      }
      // every CTA of the cluster has read the previous tile's partials before they are overwritten
      asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) Ps[(ty * TM + i) * RS_COLS + tx * 4 + jj] = El<T>::rnd(acc[i][jj]);
      asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
      // rows r = h, h + Hkv, ... of the tile are finished here: partials of all heads, in head order
      for (int o = tid; o < nown_max * RS_COLS; o += 256) {
        const int lr = o / RS_COLS, col = o % RS_COLS, r = h + lr * Hkv;
        if (r < ROWS) {
          const uint32_t local = tma::smem_u32(Ps + r * RS_COLS + col);
          float pv[8];                                 // all requests first, then the sum in head order
#pragma unroll
          for (int hh = 0; hh < 8; ++hh) {
            pv[hh] = 0.f;
            if (hh < Hkv) {
              uint32_t remote;
              asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(hh));
              asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(pv[hh]) : "r"(remote) : "memory");
            }
          }
          float tot = 0.f;
#pragma unroll
          for (int hh = 0; hh < 8; ++hh) if (hh < Hkv) tot += pv[hh];
          const int m = c0 + col;
          float sc = El<T>::rnd(tot / (float)Hkv);
          if (m >= M) sc = -INFINITY;                                   // padding column: never wins
          else if (m >= active || (exact && !al[W + m])) sc = -1e9f;    // (:646-650, :875-877)
          Fs[lr * (RS_COLS + 1) + col] = sc;
        }
      }
      __syncthreads();
      {
        const int r = h + tid * Hkv;                 // owned row `tid`
        if (tid < nown_max && r < nrows) {
          for (int col = 0; col < RS_COLS && c0 + col < M; ++col) {
            const float sc = Fs[tid * (RS_COLS + 1) + col];
            if ((c0 == 0 && col == 0) || sc > best) { best = sc; bi = c0 + col; }
          }
        }
      }
    }
    {
      const int r = h + tid * Hkv;
      if (tid < nown_max && r < nrows) {
        if (exact) { p.ex_best[(long long)b * c.Te + r0 + r] = best; p.ex_bi[(long long)b * c.Te + r0 + r] = bi; }
        else p.su_idx[(long long)b * c.Ts + r0 + r] = bi;
      }
    }
  }
  // no CTA may leave while another still reads its partials
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

template <typename T>
__global__ void __launch_bounds__(256) route_score_heads_kernel(RouteParams p) {
  extern __shared__ float sm[];
  const bool exact = blockIdx.x == 0;
  // (both branches are uniform over a cluster: its CTAs differ in blockIdx.z only)
  if (exact) { if (p.te > 0 && p.c.Me > 0) route_score_bank_heads<T, 1>(p, blockIdx.y, true, sm); }
  else if (p.ts > 0 && p.c.Ms > 0) route_score_bank_heads<T, 4>(p, blockIdx.y, false, sm);
}

// Per-state plan written by route_decide and consumed by route_apply (all int32 / fp32, in global scratch).
struct Plan {
  int* e_tgt; int* e_flag;            // [Te]  target slot; bit0 overwrite, bit1 touch, bit2 first overwriter of its slot
  float* s_w; int* s_ord;             // [Ts]  summary weights; candidates grouped by slot
  int* s_start; float* s_cnt; int* s_was;   // [Ms+1], [Ms], [Ms]
};
__device__ __forceinline__ Plan plan_of(const RouteParams& p, int b) {
  const int Te = p.c.Te > 0 ? p.c.Te : 0, Ts = p.c.Ts > 0 ? p.c.Ts : 0, Ms = p.c.Ms;
  const size_t per = (size_t)(2 * Te + 2 * Ts + 3 * Ms + 1);
  int* base = p.plan + (size_t)b * per;
  Plan pl;
  pl.e_tgt = base; pl.e_flag = base + Te;
  pl.s_w = reinterpret_cast<float*>(base + 2 * Te); pl.s_ord = base + 2 * Te + Ts;
  pl.s_start = base + 2 * Te + 2 * Ts; pl.s_cnt = reinterpret_cast<float*>(pl.s_start + Ms + 1);
  pl.s_was = pl.s_start + Ms + 1 + Ms;
  return pl;
}

// ---- decisions: the order-dependent part, one small CTA per state ----
// Inputs are staged into shared memory by all threads, the two serial sections (exact bank on thread 0,
// summary bank on thread 32) work on shared memory only, and the plan is copied out cooperatively.
template <typename T>
__global__ void __launch_bounds__(64) route_decide_kernel(RouteParams p) {
  extern __shared__ unsigned char smraw[];
  const coda_layer_cfg& c = p.c;
  const int b = blockIdx.x, tid = threadIdx.x, NT = blockDim.x;
  const int Me = c.Me, Ms = c.Ms, W = c.W, Lbuf = W + Me + Ms;
  const int te = (Me > 0) ? p.te : 0, ts = (Ms > 0) ? p.ts : 0, tmax = te > ts ? te : ts;
  typedef topk_order::Item<long long> It64;
  It64* lruq = reinterpret_cast<It64*>(smraw);                       // [Me]
  long long* s_last = reinterpret_cast<long long*>(lruq + (Me > 0 ? Me : 1));   // [Me]
  long long* n_last = s_last + (Me > 0 ? Me : 1);                    // [Me] new stamps
  float* c_g = reinterpret_cast<float*>(n_last + (Me > 0 ? Me : 1)); // [tmax] gates
  float* x_best = c_g + (tmax > 0 ? tmax : 1);                       // [te]
  float* w_s = x_best + (te > 0 ? te : 1);                           // [ts] summary weights
  float* cnt_s = w_s + (ts > 0 ? ts : 1);                            // [Ms]
  int* c_e = reinterpret_cast<int*>(cnt_s + (Ms > 0 ? Ms : 1));      // [tmax] evicted index
  int* x_bi = c_e + (tmax > 0 ? tmax : 1);                           // [te]
  int* tgt_s = x_bi + (te > 0 ? te : 1);                             // [te]
  int* flag_s = tgt_s + (te > 0 ? te : 1);                           // [te]
  int* s_idx = flag_s + (te > 0 ? te : 1);                           // [ts]
  int* ord_s = s_idx + (ts > 0 ? ts : 1);                            // [ts]
  int* start_s = ord_s + (ts > 0 ? ts : 1);                          // [Ms+1]
  int* s_cur = start_s + Ms + 1;                                     // [Ms]
  unsigned char* s_used = reinterpret_cast<unsigned char*>(s_cur + (Ms > 0 ? Ms : 1));   // [Me + Ms]
  const uint8_t* al = p.st.allowed + (long long)b * Lbuf;
  long long* last = (long long*)p.st.mem_last_exact + (long long)b * Me;
  Plan pl = plan_of(p, b);
  for (int t = tid; t < tmax; t += NT) {
    const int e = p.cand[(long long)b * p.cand_bs + t];
    c_e[t] = e;
    c_g[t] = p.gates[(long long)b * p.gates_bs + p.gate_ev0 + e];
  }
  for (int t = tid; t < te; t += NT) { x_best[t] = p.ex_best[(long long)b * c.Te + t]; x_bi[t] = p.ex_bi[(long long)b * c.Te + t]; }
  for (int t = tid; t < ts; t += NT) s_idx[t] = p.su_idx[(long long)b * c.Ts + t];
  for (int m = tid; m < Me + Ms; m += NT) s_used[m] = al[W + m];
  for (int m = tid; m < Me; m += NT) { s_last[m] = last[m]; n_last[m] = last[m]; }
  __syncthreads();

  // routing-event record of this call (optional): cleared here, filled by the two deciding threads below
  int32_t* evw = p.st.events != nullptr ? p.st.events + (long long)b * CODA_EVENT_WORDS : nullptr;
  if (evw != nullptr && tid < CODA_EVENT_WORDS) evw[tid] = 0;
  __syncthreads();
  if (tid == 0 && te > 0) {
    // ---- exact bank (memory_banks.py:635-697) ----
    const int Ae = c.active_exact;
    int n_gated = 0, n_hit = 0, n_ins = 0, n_ow = 0, n_frus = 0;
    bool any_used = false;
    for (int m = 0; m < Me; ++m) {
      const bool used = s_used[m] != 0;
      any_used |= used;
      lruq[m].v = (used && m < Ae) ? s_last[m] : -(1LL << 62);
      lruq[m].i = m;
    }
    const int n_lru = te < Ae ? te : Ae;
    topk_order::topk_queue<long long, false>(lruq, Me, n_lru, true);   // victims = lruq[0..n_lru).i
    const float tn = El<T>::rnd(c.tau_novel), tm = El<T>::rnd(c.tau_match);
    int rank = -1;
    for (int t = 0; t < te; ++t) {
      const float best = x_best[t];
      const bool keep = c.gated ? (c_g[t] >= c.tau_gate_exact) : true;
      const bool novel = !any_used || best < tn;
      const bool hit = any_used && best >= tm;
      const bool nk = novel && keep;
      if (nk) ++rank;
      const bool capped = nk && rank < Ae;
      int r = rank < 0 ? 0 : rank;
      if (r > n_lru - 1) r = n_lru - 1 > 0 ? n_lru - 1 : 0;
      const int tgt = capped ? lruq[r].i : x_bi[t];
      const bool touch = keep && (!novel || capped);
      const bool ow = c.refresh_on_hit ? (keep && (capped || hit)) : capped;
      int flag = (ow ? 1 : 0) | (touch ? 2 : 0);
      if (ow) {
        bool first = true;
        for (int u = 0; u < t; ++u) if ((flag_s[u] & 1) && tgt_s[u] == tgt) { first = false; break; }
        if (first) flag |= 4;
      }
      tgt_s[t] = tgt;
      flag_s[t] = flag;
      n_gated += (c.gated && !keep) ? 1 : 0; n_hit += (hit && keep) ? 1 : 0; n_ins += capped ? 1 : 0;
      n_ow += ow ? 1 : 0; n_frus += (nk && !capped) ? 1 : 0;
    }
    if (evw != nullptr) { evw[0] = n_gated; evw[1] = n_hit; evw[2] = n_ins; evw[3] = n_ow; evw[4] = n_frus; }
    // stamps: per slot the largest position among touching candidates replaces the old stamp (:682-697)
    for (int t = 0; t < te; ++t) {
      if (!(flag_s[t] & 2)) continue;
      const int tgt = tgt_s[t];
      bool first = true;
      for (int u = 0; u < t; ++u) if ((flag_s[u] & 2) && tgt_s[u] == tgt) { first = false; break; }
      if (!first) continue;
      long long mx = p.pos_first + c_e[t];
      for (int u = t + 1; u < te; ++u)
        if ((flag_s[u] & 2) && tgt_s[u] == tgt) { const long long pu = p.pos_first + c_e[u]; if (pu > mx) mx = pu; }
      n_last[tgt] = mx;
    }
  }
  if (tid == 32 && ts > 0) {
    // ---- summary bank bookkeeping (memory_banks.py:880-885, 906): weights, per-slot candidate lists ----
    for (int m = 0; m < Ms; ++m) { cnt_s[m] = 0.f; start_s[m] = 0; }
    start_s[Ms] = 0;
    for (int t = 0; t < ts; ++t) {
      float w = El<T>::rnd(c_g[t]);
      if (c.gated && !(c_g[t] >= c.tau_gate_summary)) w = 0.f;           // (:518-523)
      w_s[t] = w;
      const int m = s_idx[t];
      cnt_s[m] = t_add<T>(cnt_s[m], w);
      start_s[m + 1] += 1;
    }
    for (int m = 0; m < Ms; ++m) start_s[m + 1] += start_s[m];
    for (int m = 0; m < Ms; ++m) s_cur[m] = start_s[m];
    for (int t = 0; t < ts; ++t) ord_s[s_cur[s_idx[t]]++] = t;            // stable grouping by slot
    if (evw != nullptr) {
      const int As = c.active_summary;
      int n_upd = 0, n_new = 0; bool all_used = true, incoming = false;
      for (int m = 0; m < Ms; ++m) {
        const bool got = cnt_s[m] > 0.f, was = s_used[Me + m] != 0;
        n_upd += got ? 1 : 0; n_new += (got && !was) ? 1 : 0;
        if (m < As) { all_used = all_used && (was || got); incoming = incoming || got; }
      }
      evw[5] = n_upd; evw[6] = n_new; evw[7] = all_used ? 1 : 0; evw[8] = incoming ? 1 : 0;
    }
  }
  __syncthreads();
  for (int t = tid; t < te; t += NT) { pl.e_tgt[t] = tgt_s[t]; pl.e_flag[t] = flag_s[t]; }
  for (int m = tid; m < Me; m += NT) if (te > 0 && n_last[m] != s_last[m]) last[m] = n_last[m];
  for (int t = tid; t < ts; t += NT) { pl.s_w[t] = w_s[t]; pl.s_ord[t] = ord_s[t]; }
  if (ts > 0) {
    for (int m = tid; m <= Ms; m += NT) pl.s_start[m] = start_s[m];
    for (int m = tid; m < Ms; m += NT) { pl.s_cnt[m] = cnt_s[m]; pl.s_was[m] = s_used[Me + m] != 0; }
  }
}

// ---- slot writes: one CTA per written slot (exact: per overwriting candidate group; summary: per slot) ----
// Each thread owns runs of 8 consecutive elements of the slot's [Hkv*Dh] row pair and loads old values and
// candidate rows in batches.
template <typename T>
__global__ void __launch_bounds__(128) route_apply_kernel(RouteParams p) {
  extern __shared__ float stash[];                                   // [Hkv*Dh] new row for re-normalising, then the slot's candidate list
  const coda_layer_cfg& c = p.c;
  const int b = blockIdx.y, tid = threadIdx.x, NT = blockDim.x, lane = tid & 31, warp = tid >> 5, NW = NT >> 5;
  const int Hkv = c.Hkv, Dh = c.Dh, HD = Hkv * Dh, lf = Dh / 2, lfd = Dh - lf;
  // Every candidate of the block may land on one slot (a one-slot summary bank, clustered keys), so the list
  // staged per slot holds max(te, ts) entries: nothing is ever dropped from a slot's sum.
  const int TMAX = max(max(p.te, p.ts), 1);
  int* s_cand = reinterpret_cast<int*>(stash + HD);
  float* s_wt = reinterpret_cast<float*>(s_cand + TMAX);
  const int Me = c.Me, Ms = c.Ms, W = c.W, Lbuf = W + Me + Ms;
  const int te = (Me > 0) ? p.te : 0;
  uint8_t* al = p.st.allowed + (long long)b * Lbuf;
  T* kb = (T*)p.st.k_buf + (long long)b * Hkv * Lbuf * Dh;
  T* vb = (T*)p.st.v_buf + (long long)b * Hkv * Lbuf * Dh;
  const Plan pl = plan_of(p, b);
  __shared__ int s_n;
  const bool exact = (int)blockIdx.x < te;
  int slot;                                                          // slot index inside its bank
  float cden = 1.f; bool fresh = false;
  if (exact) {
    // ---- exact bank write (memory_banks.py:707-742): candidates that overwrite this slot, in list order ----
    const int t = blockIdx.x;
    if ((pl.e_flag[t] & 5) != 5) return;                               // not the first overwriter of its slot
    slot = pl.e_tgt[t];
    if (tid == 0) {
      int nn = 0;
      for (int u = t; u < te; ++u)
        if ((pl.e_flag[u] & 1) && pl.e_tgt[u] == slot) { s_cand[nn] = p.cand[(long long)b * p.cand_bs + u]; s_wt[nn] = 1.f; ++nn; }
      s_n = nn;
    }
  } else {
    // ---- summary bank EMA of one slot (memory_banks.py:887-932) ----
    slot = blockIdx.x - te;
    if (slot >= Ms || p.ts <= 0) return;
    const float cnt = pl.s_cnt[slot];
    if (!(cnt > 0.f)) return;
    cden = fmaxf(cnt, El<T>::rnd(1e-6f));
    fresh = c.overwrite_on_insert && !pl.s_was[slot];
    if (tid == 0) {
      const int a0 = pl.s_start[slot], a1 = pl.s_start[slot + 1];
      int nn = 0;
      for (int a = a0; a < a1; ++a) {
        const int t = pl.s_ord[a];
        s_cand[nn] = p.cand[(long long)b * p.cand_bs + t]; s_wt[nn] = pl.s_w[t]; ++nn;
      }
      s_n = nn;
    }
  }
  __syncthreads();
  const int nn = s_n;
  const int gslot = W + (exact ? 0 : Me) + slot;
  constexpr int R = 8;
  const bool runs = (Dh % R) == 0;
  for (int e0 = tid * R; e0 < HD; e0 += NT * R) {
    const int h = e0 / Dh, d0 = e0 % Dh;
    T* pk = kb + ((long long)h * Lbuf + gslot) * Dh + d0;
    T* pv = vb + ((long long)h * Lbuf + gslot) * Dh + d0;
    float ok[R], ov[R], ak[R], av[R];
    if (runs) { load_run<T, R>(pk, ok); load_run<T, R>(pv, ov); }
    else for (int i = 0; i < R; ++i) { ok[i] = (e0 + i < HD) ? El<T>::ld(kb + ((long long)((e0 + i) / Dh) * Lbuf + gslot) * Dh + (e0 + i) % Dh) : 0.f;
                                       ov[i] = (e0 + i < HD) ? El<T>::ld(vb + ((long long)((e0 + i) / Dh) * Lbuf + gslot) * Dh + (e0 + i) % Dh) : 0.f; }
#pragma unroll
    for (int i = 0; i < R; ++i) { ak[i] = 0.f; av[i] = 0.f; }
    for (int q = 0; q < nn; ++q) {
      const int ce = s_cand[q];
      const float w = s_wt[q];
      float xk[R], xv[R];
      if (runs) {
        load_run<T, R>(src_row<T>(p, p.st.k_buf, p.kblk, p.kb_bs, p.kb_rs, b, ce, h) + d0, xk);
        load_run<T, R>(src_row<T>(p, p.st.v_buf, p.vblk, p.vb_bs, p.vb_rs, b, ce, h) + d0, xv);
      } else {
        for (int i = 0; i < R; ++i) {
          const int hh = (e0 + i) / Dh, dd = (e0 + i) % Dh;
          xk[i] = (e0 + i < HD) ? El<T>::ld(src_row<T>(p, p.st.k_buf, p.kblk, p.kb_bs, p.kb_rs, b, ce, hh) + dd) : 0.f;
          xv[i] = (e0 + i < HD) ? El<T>::ld(src_row<T>(p, p.st.v_buf, p.vblk, p.vb_bs, p.vb_rs, b, ce, hh) + dd) : 0.f;
        }
      }
#pragma unroll
      for (int i = 0; i < R; ++i) {
        if (exact) { ak[i] = t_add<T>(ak[i], t_sub<T>(xk[i], ok[i])); av[i] = t_add<T>(av[i], t_sub<T>(xv[i], ov[i])); }
        else { ak[i] = t_add<T>(ak[i], t_mul<T>(xk[i], w)); av[i] = t_add<T>(av[i], t_mul<T>(xv[i], w)); }
      }
    }
    // the slot's EMA rate depends on the head only: one sigmoid per run, not one per element
    const float eta_run = (exact || fresh) ? 1.f : t_sigmoid<T>(p.eta_logit[h]);
#pragma unroll
    for (int i = 0; i < R; ++i) {
      const int e = e0 + i;
      if (e >= HD) break;
      const int hh = runs ? h : e / Dh, dd = runs ? d0 + i : e % Dh;
      T* qk = runs ? pk + i : kb + ((long long)hh * Lbuf + gslot) * Dh + dd;
      T* qv = runs ? pv + i : vb + ((long long)hh * Lbuf + gslot) * Dh + dd;
      if (exact) {                                                     // mem + sum of deltas
        El<T>::st(qk, t_add<T>(ok[i], ak[i]));
        const float nv = t_add<T>(ov[i], av[i]);
        El<T>::st(qv, nv);
        stash[e] = nv;
      } else {                                                         // phase-safe EMA
        const float eta = fresh ? 1.f : (runs ? eta_run : t_sigmoid<T>(p.eta_logit[hh]));
        El<T>::st(qv, t_add<T>(ov[i], t_mul<T>(eta, t_sub<T>(t_div<T>(av[i], cden), ov[i]))));
        if (dd >= lf) {
          const float inc = El<T>::rnd(__fmul_rn(t_div<T>(ak[i], cden), c.energy_scale));
          const float nk = t_add<T>(ok[i], t_mul<T>(eta, t_sub<T>(inc, ok[i])));
          El<T>::st(qk, nk);
          stash[hh * lfd + dd - lf] = nk;
        }
      }
    }
  }
  if (tid == 0) al[gslot] = 1;
  __syncthreads();
  const int nn_norm = exact ? Dh : lfd;
  T* cachep = exact ? (T*)p.st.exact_v_norm + (long long)b * Hkv * Me * Dh : (T*)p.st.sum_lf_k_norm + (long long)b * Hkv * Ms * lfd;
  const int Mb = exact ? Me : Ms;
  for (int h = warp; h < Hkv; h += NW) {
    float ss = 0.f;
    for (int d = lane; d < nn_norm; d += 32) { const float v = stash[h * nn_norm + d]; ss += v * v; }
    const float den = fmaxf(El<T>::rnd(sqrtf(warp_sum(ss))), 1e-6f);
    for (int d = lane; d < nn_norm; d += 32)
      El<T>::st(cachep + ((long long)h * Mb + slot) * nn_norm + d, t_div<T>(stash[h * nn_norm + d], den));
  }
}

// Ring rewrite (memory_banks.py:152-177, 554-563): with the ring in chronological order the kept rows
// [drop, fill) move down to [0, fill-drop) and block rows [bstart, blk) follow them.  One CTA per
// (plane, K|V); 16-byte vectors when rows allow it; the in-place shift goes chunk by chunk in ascending order.
template <typename T, typename V>
__device__ __forceinline__ void ring_plane(T* ring, const T* src, long long src_rs, int Dh, int drop, int kept,
                                           int bstart, int nnew, int tid, int NT) {
  constexpr int PER = 4;
  constexpr int EV = sizeof(V) / sizeof(T);
  const int rowv = Dh / EV;                                            // vectors per row
  V* rv = reinterpret_cast<V*>(ring);
  if (drop > 0 && kept > 0) {
    const long long n = (long long)kept * rowv, off = (long long)drop * rowv;
    for (long long c0 = 0; c0 < n; c0 += (long long)NT * PER) {
      V tmp[PER];
#pragma unroll
      for (int i = 0; i < PER; ++i) { const long long x = c0 + (long long)i * NT + tid; if (x < n) tmp[i] = rv[off + x]; }
      __syncthreads();
#pragma unroll
      for (int i = 0; i < PER; ++i) { const long long x = c0 + (long long)i * NT + tid; if (x < n) rv[x] = tmp[i]; }
      __syncthreads();
    }
  }
  for (long long x = tid; x < (long long)nnew * rowv; x += NT) {
    const int r = (int)(x / rowv), dv = (int)(x % rowv);
    rv[(long long)(kept + r) * rowv + dv] = *reinterpret_cast<const V*>(src + (long long)(bstart + r) * src_rs + (long long)dv * EV);
  }
}

template <typename T>
__global__ void __launch_bounds__(256) ring_rewrite_kernel(RouteParams p, int vec16) {
  const coda_layer_cfg& c = p.c;
  const int h = blockIdx.x >> 1, pass = blockIdx.x & 1, b = blockIdx.y, tid = threadIdx.x, NT = blockDim.x;
  const int W = c.W, Dh = c.Dh, Lbuf = W + c.Me + c.Ms;
  const int drop = p.n_ev < p.fill ? p.n_ev : p.fill;
  const int kept = p.fill - drop;
  const int bstart = p.n_ev > p.fill ? p.n_ev - p.fill : 0;
  const int nnew = p.blk - bstart;
  T* ring = (T*)(pass ? p.st.v_buf : p.st.k_buf) + ((long long)b * c.Hkv + h) * Lbuf * Dh;
  const T* src = (const T*)(pass ? p.vblk : p.kblk) + (long long)b * (pass ? p.vb_bs : p.kb_bs) + (long long)h * Dh;
  const long long rs = pass ? p.vb_rs : p.kb_rs;
  if (vec16) ring_plane<T, uint4>(ring, src, rs, Dh, drop, kept, bstart, nnew, tid, NT);
  else ring_plane<T, T>(ring, src, rs, Dh, drop, kept, bstart, nnew, tid, NT);
  if (blockIdx.x == 0) {
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
  const size_t te = c->Te > 0 ? c->Te : 0, ts = c->Ts > 0 ? c->Ts : 0, ms = c->Ms;
  return (size_t)c->B * 4 * (2 * te + ts + (2 * te + 2 * ts + 3 * ms + 1)) + 64;
}

extern "C" int64_t coda_b200_route_scratch_bytes(const coda_layer_cfg* cfg) {
  if (!coda_cfg_ok(cfg)) return -1;
  return (int64_t)route_scratch_bytes(cfg);
}

template <typename T>
// phase 0: everything; 1: scores and decisions only (they read the state and write the scratch and the LRU
// stamps: nothing the attention of the same block reads is touched); 2: slot updates and the ring rewrite only.
static int launch_route(RouteParams& p, cudaStream_t s, int phase = 0) {
  const coda_layer_cfg& c = p.c;
  const int HD = c.Hkv * c.Dh;
  if ((p.te > 0 || p.ts > 0) && phase != 2) {
    const size_t smem1 = sizeof(float) * (size_t)(RS_KC * 64 + RS_KC * RS_COLS + 64 * (RS_COLS + 1) + 64 * c.Hkv + 64);
    CODA_REQUIRE(smem1 <= 200 * 1024, CODA_ERR_LIMIT, "route_block: %d KV heads too many for the scoring tile", c.Hkv);
    if (smem1 > 48 * 1024) cudaFuncSetAttribute(route_score_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1);
    if (c.Hkv >= 2 && c.Hkv <= 8 && c.B <= 65535) {
      // the heads of a state side by side: clusters of Hkv CTAs along z
      const size_t smemh = sizeof(float) * (size_t)(RS_KC * 64 + RS_KC * RS_COLS + 64 * RS_COLS + (64 / c.Hkv + 1) * (RS_COLS + 1) + 64 + 64);
      if (smemh > 48 * 1024) cudaFuncSetAttribute(route_score_heads_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smemh);
      cudaLaunchConfig_t lc = {};
      lc.gridDim = dim3(2, c.B, c.Hkv);
      lc.blockDim = dim3(256, 1, 1);
      lc.dynamicSmemBytes = smemh;
      lc.stream = s;
      cudaLaunchAttribute at[1];
      at[0].id = cudaLaunchAttributeClusterDimension;
      at[0].val.clusterDim.x = 1; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = c.Hkv;
      lc.attrs = at; lc.numAttrs = 1;
      cudaError_t e = cudaLaunchKernelEx(&lc, route_score_heads_kernel<T>, p);
      if (e != cudaSuccess) { coda_set_error("route_block (score): %s", cudaGetErrorString(e)); return CODA_ERR_LAUNCH; }
    } else {
      route_score_kernel<T><<<dim3(2, c.B), 256, smem1, s>>>(p);
      CODA_CHECK_LAUNCH("route_block (score)");
    }
    const int tmax = p.te > p.ts ? p.te : p.ts;
    const size_t smem2 = 32 * (size_t)(c.Me > 0 ? c.Me : 1) + 4 * ((size_t)2 * (tmax + 1) + 4 * (size_t)(p.te + 1) + 4 * (size_t)(p.ts + 1) +
                         3 * (size_t)(c.Ms + 1) + 2) + c.Me + c.Ms + 64;
    CODA_REQUIRE(smem2 <= 200 * 1024, CODA_ERR_LIMIT, "route_block: decision stage needs %zu bytes of shared memory", smem2);
    if (smem2 > 48 * 1024) cudaFuncSetAttribute(route_decide_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2);
    route_decide_kernel<T><<<c.B, 64, smem2, s>>>(p);
    CODA_CHECK_LAUNCH("route_block (decide)");
  }
  if (phase == 1) return CODA_OK;
  if (p.te > 0 || p.ts > 0) {
    const int tmax = p.te > p.ts ? p.te : p.ts;
    const size_t smem3 = sizeof(float) * (size_t)HD + 8 * (size_t)(tmax > 0 ? tmax : 1);   // new row + the slot's candidate list
    CODA_REQUIRE(smem3 <= 200 * 1024, CODA_ERR_LIMIT, "route_block: Hkv*Dh = %d with %d candidates per block needs %zu bytes of shared memory", HD, tmax, smem3);
    if (smem3 > 48 * 1024) cudaFuncSetAttribute(route_apply_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem3);
    const int nslots = (c.Me > 0 ? p.te : 0) + (p.ts > 0 ? c.Ms : 0);
    if (nslots > 0) {
      route_apply_kernel<T><<<dim3(nslots, c.B), 128, smem3, s>>>(p);
      CODA_CHECK_LAUNCH("route_block (apply)");
    }
  }
  const int vec16 = (c.Dh * sizeof(T)) % 16 == 0 && ((uintptr_t)p.st.k_buf % 16 == 0) && ((uintptr_t)p.st.v_buf % 16 == 0) &&
                    ((uintptr_t)p.kblk % 16 == 0) && ((uintptr_t)p.vblk % 16 == 0) && (p.kb_rs * sizeof(T)) % 16 == 0 &&
                    (p.vb_rs * sizeof(T)) % 16 == 0 && (p.kb_bs * sizeof(T)) % 16 == 0 && (p.vb_bs * sizeof(T)) % 16 == 0;
  ring_rewrite_kernel<T><<<dim3(2 * c.Hkv, c.B), 256, 0, s>>>(p, vec16);
  CODA_CHECK_LAUNCH("route_block (ring)");
  return CODA_OK;
}

// ---- allocation-free variant -------------------------------------------------------------------------------
// Scratch for callers that are not allowed to allocate device memory: a fixed array in the library's own
// device image.  Every GPU that loads the library carries these bytes until the process exits.
constexpr size_t CODA_STATIC_SCRATCH_BYTES = 1u << 20;
static __device__ __align__(256) unsigned char g_route_scratch[CODA_STATIC_SCRATCH_BYTES];

extern "C" int64_t coda_b200_route_static_scratch_bytes(void) { return (int64_t)CODA_STATIC_SCRATCH_BYTES; }

// In host code `g_route_scratch` is only a handle for the symbol, not a device address; the address is looked
// up once per device (with that device current) and remembered.
static void* static_scratch_for_current_device() {
  constexpr int MAX_DEV = 64;
  static void* ptrs[MAX_DEV] = {nullptr};
  static std::mutex mu;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEV) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (ptrs[dev] == nullptr) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_route_scratch) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    ptrs[dev] = ptr;
  }
  return ptrs[dev];
}

extern "C" int coda_b200_route_block(const coda_layer_cfg* cfg, const coda_state_ptrs* st,
                                     int32_t ring_fill, int32_t blk, int64_t pos0,
                                     const void* k_blk, int64_t kb_bs, int64_t kb_rs,
                                     const void* v_blk, int64_t vb_bs, int64_t vb_rs,
                                     const float* gates, int64_t gates_bs, int64_t gate_ev0,
                                     const int32_t* cand, int64_t cand_bs,
                                     const float* eta_logit, void* scratch, coda_stream_t stream);

extern "C" int coda_b200_route_block_noalloc(const coda_layer_cfg* cfg, const coda_state_ptrs* st,
                                             int32_t ring_fill, int32_t blk, int64_t pos0,
                                             const void* k_blk, int64_t kb_bs, int64_t kb_rs,
                                             const void* v_blk, int64_t vb_bs, int64_t vb_rs,
                                             const float* gates, int64_t gates_bs, int64_t gate_ev0,
                                             const int32_t* cand, int64_t cand_bs,
                                             const float* eta_logit, coda_stream_t stream) {
  CODA_REQUIRE(coda_cfg_ok(cfg), CODA_ERR_ARG, "route_block_noalloc: invalid layer configuration");
  const size_t need = route_scratch_bytes(cfg);
  CODA_REQUIRE(need <= CODA_STATIC_SCRATCH_BYTES, CODA_ERR_LIMIT,
               "route_block_noalloc: this configuration needs %zu bytes of scratch, the built-in buffer holds %zu "
               "(fewer states per call, or use coda_b200_route_block with caller-provided scratch)",
               need, CODA_STATIC_SCRATCH_BYTES);
  void* scratch = static_scratch_for_current_device();
  CODA_REQUIRE(scratch != nullptr, CODA_ERR_LAUNCH, "route_block_noalloc: cudaGetSymbolAddress failed for the built-in scratch");
  return coda_b200_route_block(cfg, st, ring_fill, blk, pos0, k_blk, kb_bs, kb_rs, v_blk, vb_bs, vb_rs,
                               gates, gates_bs, gate_ev0, cand, cand_bs, eta_logit, scratch, stream);
}

extern "C" int coda_b200_route_block(const coda_layer_cfg* cfg, const coda_state_ptrs* st,
                                     int32_t ring_fill, int32_t blk, int64_t pos0,
                                     const void* k_blk, int64_t kb_bs, int64_t kb_rs,
                                     const void* v_blk, int64_t vb_bs, int64_t vb_rs,
                                     const float* gates, int64_t gates_bs, int64_t gate_ev0,
                                     const int32_t* cand, int64_t cand_bs,
                                     const float* eta_logit, void* scratch, coda_stream_t stream) {
  return coda_b200_route_block_phase(cfg, st, ring_fill, blk, pos0, k_blk, kb_bs, kb_rs, v_blk, vb_bs, vb_rs, gates, gates_bs,
                                     gate_ev0, cand, cand_bs, eta_logit, scratch, 0, stream);
}

extern "C" int coda_b200_route_block_phase(const coda_layer_cfg* cfg, const coda_state_ptrs* st,
                                           int32_t ring_fill, int32_t blk, int64_t pos0,
                                           const void* k_blk, int64_t kb_bs, int64_t kb_rs,
                                           const void* v_blk, int64_t vb_bs, int64_t vb_rs,
                                           const float* gates, int64_t gates_bs, int64_t gate_ev0,
                                           const int32_t* cand, int64_t cand_bs,
                                           const float* eta_logit, void* scratch, int32_t phase, coda_stream_t stream) {
  CODA_REQUIRE(coda_cfg_ok(cfg) && st, CODA_ERR_ARG, "route_block: invalid layer configuration");
  CODA_REQUIRE(phase >= 0 && phase <= 2, CODA_ERR_ARG, "route_block: phase %d is not 0, 1 or 2", phase);
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
    p.su_idx = (int*)sp; sp += (size_t)cfg->B * (cfg->Ts > 0 ? cfg->Ts : 0) * 4;
    p.plan = (int*)sp;
  } else {
    p.ex_best = nullptr; p.ex_bi = nullptr; p.su_idx = nullptr; p.plan = nullptr;
  }
  cudaStream_t s = (cudaStream_t)stream;
  return cfg->dtype == CODA_F32 ? launch_route<float>(p, s, phase) : launch_route<bf16>(p, s, phase);
}
