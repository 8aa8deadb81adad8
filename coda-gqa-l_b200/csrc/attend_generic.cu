// Shape-generic differential attention (any Dh <= 256, any slot count, fp32 or bf16 storage,
// fp32 arithmetic).  One warp owns one query row and carries both streams (signal and noise)
// through the same K/V tiles, so each tile staged in shared memory is used twice.  This is the
// exact-arithmetic path used for fp32 parity and for shapes the tuned kernels do not cover.
#include "coda_common.cuh"

struct AttnParams {
  int B, H, Hkv, Dh, Lbuf, Lq, mask_unused, norm_full;
  float eps, scale_log2;
  const void* q; long long q_bs, q_rs;
  const void* qn; long long qn_bs, qn_rs;
  const float* lam; long long lam_bs, lam_rs;
  const void* kbuf; const void* vbuf; const uint8_t* allowed;
  const void* kblk; long long kb_bs, kb_rs;
  const void* vblk; long long vb_bs, vb_rs;
  const void* norm_w;
  void* out; long long out_bs, out_rs;
};

constexpr int AG_WARPS = 4;     // query rows per CTA
constexpr int AG_TK = 32;       // keys per tile (one per lane)
constexpr int AG_MAXD = 8;      // Dh <= 32*8

template <typename T>
__global__ void __launch_bounds__(AG_WARPS * 32) attend_generic_kernel(AttnParams p) {
  extern __shared__ float sm[];
  const int Dh = p.Dh, DP = Dh + 1;
  float* Ks = sm;                           // [TK][Dh+1]
  float* Vs = Ks + AG_TK * DP;              // [TK][Dh]
  float* Qs = Vs + AG_TK * Dh;              // [WARPS][2][Dh]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int b = blockIdx.z, h = blockIdx.y, hk = h / (p.H / p.Hkv);
  const int row0 = blockIdx.x * AG_WARPS;
  const int row = row0 + warp;
  const bool row_ok = row < p.Lq;
  const int nd = (Dh + 31) / 32;

  float* qs = Qs + (warp * 2) * Dh;
  float* qns = qs + Dh;
  if (row_ok) {
    const T* qp = (const T*)p.q + (long long)b * p.q_bs + (long long)row * p.q_rs + h * Dh;
    const T* qnp = (const T*)p.qn + (long long)b * p.qn_bs + (long long)row * p.qn_rs + h * Dh;
    for (int d = lane; d < Dh; d += 32) { qs[d] = El<T>::ld(qp + d); qns[d] = El<T>::ld(qnp + d); }
  }
  float m_s = -INFINITY, m_n = -INFINITY, l_s = 0.f, l_n = 0.f;
  float acc_s[AG_MAXD], acc_n[AG_MAXD];
#pragma unroll
  for (int i = 0; i < AG_MAXD; ++i) { acc_s[i] = 0.f; acc_n[i] = 0.f; }

  const bool has_blk = p.kblk != nullptr;
  const int last_row = min(row0 + AG_WARPS, p.Lq) - 1;
  const int nkeys = p.Lbuf + (has_blk ? last_row + 1 : 0);
  const T* kbase = (const T*)p.kbuf + ((long long)b * p.Hkv + hk) * p.Lbuf * Dh;
  const T* vbase = (const T*)p.vbuf + ((long long)b * p.Hkv + hk) * p.Lbuf * Dh;
  const uint8_t* al = p.allowed + (long long)b * p.Lbuf;

  for (int j0 = 0; j0 < nkeys; j0 += AG_TK) {
    __syncthreads();
    for (int e = tid; e < AG_TK * Dh; e += AG_WARPS * 32) {
      const int kk = e / Dh, d = e % Dh, j = j0 + kk;
      float kv = 0.f, vv = 0.f;
      if (j < p.Lbuf) {
        kv = El<T>::ld(kbase + (long long)j * Dh + d);
        vv = El<T>::ld(vbase + (long long)j * Dh + d);
      } else if (j < nkeys) {
        const int t = j - p.Lbuf;
        kv = El<T>::ld((const T*)p.kblk + (long long)b * p.kb_bs + (long long)t * p.kb_rs + hk * Dh + d);
        vv = El<T>::ld((const T*)p.vblk + (long long)b * p.vb_bs + (long long)t * p.vb_rs + hk * Dh + d);
      }
      Ks[kk * DP + d] = kv;
      Vs[kk * Dh + d] = vv;
    }
    __syncthreads();
    if (!row_ok) continue;
    const int j = j0 + lane;
    bool vis;
    if (j < p.Lbuf) vis = !p.mask_unused || al[j] != 0;          // attention.py:485-497, 687-692
    else vis = has_blk && (j - p.Lbuf) <= row;                  // causal inside the block (:562)
    float ss = 0.f, sn = 0.f;
    const float* kr = Ks + lane * DP;
    for (int d = 0; d < Dh; ++d) { const float kv = kr[d]; ss = fmaf(qs[d], kv, ss); sn = fmaf(qns[d], kv, sn); }
    ss = vis ? ss * p.scale_log2 : -INFINITY;
    sn = vis ? sn * p.scale_log2 : -INFINITY;
    const float tm_s = warp_max(ss), tm_n = warp_max(sn);
    if (tm_s == -INFINITY) continue;                            // whole tile masked (same mask for both streams)
    const float nm_s = fmaxf(m_s, tm_s), nm_n = fmaxf(m_n, tm_n);
    const float a_s = exp2f(m_s - nm_s), a_n = exp2f(m_n - nm_n);
    const float p_s = exp2f(ss - nm_s), p_n = exp2f(sn - nm_n);
    l_s = l_s * a_s + warp_sum(p_s);
    l_n = l_n * a_n + warp_sum(p_n);
    m_s = nm_s; m_n = nm_n;
#pragma unroll
    for (int i = 0; i < AG_MAXD; ++i) { acc_s[i] *= a_s; acc_n[i] *= a_n; }
    for (int kk = 0; kk < AG_TK; ++kk) {
      const float ws = __shfl_sync(0xffffffffu, p_s, kk), wn = __shfl_sync(0xffffffffu, p_n, kk);
#pragma unroll
      for (int i = 0; i < AG_MAXD; ++i) {
        if (i < nd) {
          const int d = lane + 32 * i;
          const float vv = d < Dh ? Vs[kk * Dh + d] : 0.f;
          acc_s[i] = fmaf(ws, vv, acc_s[i]);
          acc_n[i] = fmaf(wn, vv, acc_n[i]);
        }
      }
    }
  }
  if (!row_ok) return;

  // ---- epilogue: sig - lam*noise, optional RMSNorm over Dh (attention.py:463-464, primitives.py:23-27)
  const float lam = El<T>::rnd(p.lam[(long long)b * p.lam_bs + (long long)row * p.lam_rs + h]);
  const float il_s = l_s > 0.f ? 1.f / l_s : 0.f, il_n = l_n > 0.f ? 1.f / l_n : 0.f;
  float diff[AG_MAXD];
  float sq = 0.f;
#pragma unroll
  for (int i = 0; i < AG_MAXD; ++i) {
    diff[i] = 0.f;
    const int d = lane + 32 * i;
    if (i < nd && d < Dh) {
      const float os = El<T>::rnd(acc_s[i] * il_s), on = El<T>::rnd(acc_n[i] * il_n);
      diff[i] = t_sub<T>(os, t_mul<T>(lam, on));
      sq += El<T>::rnd(diff[i] * diff[i]);
    }
  }
  T* op = (T*)p.out + (long long)b * p.out_bs + (long long)row * p.out_rs + h * Dh;
  if (p.norm_full) {
    const float var = El<T>::rnd(warp_sum(sq) / (float)Dh);
    const float rs = El<T>::rnd(rsqrtf(El<T>::rnd(var + p.eps)));
#pragma unroll
    for (int i = 0; i < AG_MAXD; ++i) {
      const int d = lane + 32 * i;
      if (i < nd && d < Dh) El<T>::st(op + d, t_mul<T>(t_mul<T>(diff[i], rs), El<T>::ld((const T*)p.norm_w + d)));
    }
  } else {
#pragma unroll
    for (int i = 0; i < AG_MAXD; ++i) {
      const int d = lane + 32 * i;
      if (i < nd && d < Dh) El<T>::st(op + d, diff[i]);
    }
  }
}

int coda_attend_generic(const coda_layer_cfg* cfg, const coda_state_ptrs* st, int32_t Lq,
                        const void* q, int64_t q_bs, int64_t q_rs,
                        const void* q_noise, int64_t qn_bs, int64_t qn_rs,
                        const float* lam, int64_t lam_bs, int64_t lam_rs,
                        const void* k_blk, int64_t kb_bs, int64_t kb_rs,
                        const void* v_blk, int64_t vb_bs, int64_t vb_rs,
                        const void* norm_w, void* out, int64_t out_bs, int64_t out_rs, cudaStream_t s) {
  CODA_REQUIRE(cfg->Dh <= 32 * AG_MAXD, CODA_ERR_LIMIT, "attend: head_dim %d > %d unsupported", cfg->Dh, 32 * AG_MAXD);
  AttnParams p;
  p.B = cfg->B; p.H = cfg->H; p.Hkv = cfg->Hkv; p.Dh = cfg->Dh; p.Lbuf = cfg->W + cfg->Me + cfg->Ms; p.Lq = Lq;
  p.mask_unused = cfg->mask_unused; p.norm_full = cfg->head_norm_full; p.eps = cfg->eps;
  p.scale_log2 = 1.4426950408889634f / sqrtf((float)cfg->Dh);
  p.q = q; p.q_bs = q_bs; p.q_rs = q_rs; p.qn = q_noise; p.qn_bs = qn_bs; p.qn_rs = qn_rs;
  p.lam = lam; p.lam_bs = lam_bs; p.lam_rs = lam_rs;
  p.kbuf = st->k_buf; p.vbuf = st->v_buf; p.allowed = st->allowed;
  p.kblk = k_blk; p.kb_bs = kb_bs; p.kb_rs = kb_rs; p.vblk = v_blk; p.vb_bs = vb_bs; p.vb_rs = vb_rs;
  p.norm_w = norm_w; p.out = out; p.out_bs = out_bs; p.out_rs = out_rs;
  const size_t smem = sizeof(float) * (size_t)(AG_TK * (cfg->Dh + 1) + AG_TK * cfg->Dh + AG_WARPS * 2 * cfg->Dh);
  dim3 grid((Lq + AG_WARPS - 1) / AG_WARPS, cfg->H, cfg->B);
  if (cfg->dtype == CODA_F32) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(attend_generic_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    attend_generic_kernel<float><<<grid, AG_WARPS * 32, smem, s>>>(p);
  } else {
    if (smem > 48 * 1024) cudaFuncSetAttribute(attend_generic_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    attend_generic_kernel<bf16><<<grid, AG_WARPS * 32, smem, s>>>(p);
  }
  CODA_CHECK_LAUNCH("attend (generic)");
  return CODA_OK;
}
