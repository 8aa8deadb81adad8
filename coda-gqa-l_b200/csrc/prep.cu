// Projection post-processing: RoPE on q/k, the theta-rotated noise query, lambda / gate sigmoids.
// One CTA per token; HBM-bound elementwise work (reads q,k once, writes q,k,q_noise once).
// Two kernels with the same arithmetic: prep_vec_kernel moves 16-byte vectors (a thread owns whole RoPE pairs AND
// whole noise-rotation pairs, so nothing crosses threads) and is used whenever rows are 16-byte aligned and the head
// dimension allows; prep_kernel is the element-wise fallback for any layout.
#include "coda_common.cuh"

struct PrepParams {
  int B, L, H, Hkv, Dh, interleaved, gated;
  coda_ring_pos rp; int W;
  void* q; long long q_bs, q_rs;
  void* k; long long k_bs, k_rs;
  void* qn;
  const void* lam_logit; long long lam_bs, lam_rs; float* lam;
  const void* gate_logit; long long gate_bs, gate_rs; float* gate;
  const float* inv_freq; const void* cos_t; const void* sin_t;
};

// T: activation dtype, A: dtype the angles are evaluated in.
template <typename T, typename A>
__global__ void __launch_bounds__(256) prep_kernel(PrepParams p) {
  extern __shared__ float sm[];
  const int half = p.Dh >> 1;
  float* cs = sm;                 // [half] cos, rounded to T
  float* sn = sm + half;          // [half] sin
  float* qrow = sm + 2 * half;    // [H*Dh] rotated query row (noise rotation pairs cross RoPE pairs)
  const int tid = threadIdx.x, NT = blockDim.x;
  const long long ntok = (long long)p.B * p.L;
  // In a decode graph the position comes from the step counter; prefill passes step_dev == NULL.
  const long long pos_base = ring_now(p.rp, p.W).pos;
  for (long long tok = blockIdx.x; tok < ntok; tok += gridDim.x) {
    const int b = (int)(tok / p.L), t = (int)(tok % p.L);
    const long long pos = pos_base + t;
    for (int i = tid; i < half; i += NT) {
      // upstream primitives.py:51-54: t = arange(dtype=inv_freq.dtype); freqs = t (x) inv_freq; cos().to(dtype)
      float ta = El<A>::rnd((float)pos);
      float inv = El<A>::rnd(p.inv_freq[i]);
      float ang = El<A>::rnd(__fmul_rn(ta, inv));
      cs[i] = El<T>::rnd(El<A>::rnd(cosf(ang)));
      sn[i] = El<T>::rnd(El<A>::rnd(sinf(ang)));
    }
    __syncthreads();
    T* qt = (T*)p.q + (long long)b * p.q_bs + (long long)t * p.q_rs;
    T* kt = p.k ? (T*)p.k + (long long)b * p.k_bs + (long long)t * p.k_rs : nullptr;
    const int nq = p.H * half, nk = p.k ? p.Hkv * half : 0;
    for (int w = tid; w < nq + nk; w += NT) {
      const bool isq = w < nq;
      const int ww = isq ? w : w - nq;
      const int h = ww / half, i = ww % half;
      T* row = (isq ? qt : kt) + h * p.Dh;
      const float c = cs[i], s = sn[i];
      int ia, ib;
      float oa, ob;
      if (p.interleaved) {                  // primitives.py:99-106
        ia = 2 * i; ib = 2 * i + 1;
        const float xe = El<T>::ld(row + ia), xo = El<T>::ld(row + ib);
        oa = t_sub<T>(t_mul<T>(xe, c), t_mul<T>(xo, s));
        ob = t_add<T>(t_mul<T>(xe, s), t_mul<T>(xo, c));
      } else {                              // primitives.py:108-113: x*cos_full + rotate_half(x)*sin_full
        ia = i; ib = i + half;
        const float x1 = El<T>::ld(row + ia), x2 = El<T>::ld(row + ib);
        oa = t_add<T>(t_mul<T>(x1, c), t_mul<T>(-x2, s));
        ob = t_add<T>(t_mul<T>(x2, c), t_mul<T>(x1, s));
      }
      El<T>::st(row + ia, oa);
      El<T>::st(row + ib, ob);
      if (isq) { qrow[h * p.Dh + ia] = oa; qrow[h * p.Dh + ib] = ob; }
    }
    __syncthreads();
    T* qnt = (T*)p.qn + tok * (long long)(p.H * p.Dh);
    for (int w = tid; w < nq; w += NT) {    // primitives.py:58-80, always (even, odd) pairs
      const int h = w / half, i = w % half;
      const float qe = qrow[h * p.Dh + 2 * i], qo = qrow[h * p.Dh + 2 * i + 1];
      const float ct = El<T>::ld((const T*)p.cos_t + h * half + i);
      const float st = El<T>::ld((const T*)p.sin_t + h * half + i);
      El<T>::st(qnt + h * p.Dh + 2 * i, t_sub<T>(t_mul<T>(qe, ct), t_mul<T>(qo, st)));
      El<T>::st(qnt + h * p.Dh + 2 * i + 1, t_add<T>(t_mul<T>(qe, st), t_mul<T>(qo, ct)));
    }
    for (int h = tid; h < p.H; h += NT) {
      const float z = El<T>::ld((const T*)p.lam_logit + (long long)b * p.lam_bs + (long long)t * p.lam_rs + h);
      p.lam[tok * p.H + h] = t_sigmoid<T>(z);
    }
    if (tid == 0 && p.gate != nullptr) {
      float g = 1.0f;                       // write_policy "none": attention.py:407-408
      if (p.gated) g = t_sigmoid<T>(El<T>::ld((const T*)p.gate_logit + (long long)b * p.gate_bs + (long long)t * p.gate_rs));
      p.gate[tok] = g;
    }
    __syncthreads();
  }
}

// 16-byte vectors of T <-> fp32
template <typename T> struct Vec16;
template <> struct Vec16<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void ld(const float* p, float (&o)[4]) { const float4 v = *reinterpret_cast<const float4*>(p); o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w; }
  static __device__ __forceinline__ void st(float* p, const float (&o)[4]) { *reinterpret_cast<float4*>(p) = make_float4(o[0], o[1], o[2], o[3]); }
};
template <> struct Vec16<bf16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void ld(const bf16* p, float (&o)[8]) {
    const uint4 v = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) { o[2 * j] = __uint_as_float(w[j] << 16); o[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u); }
  }
  static __device__ __forceinline__ void st(bf16* p, const float (&o)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) { __nv_bfloat162 t = __floats2bfloat162_rn(o[2 * j], o[2 * j + 1]); w[j] = *reinterpret_cast<uint32_t*>(&t); }
    *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
  }
};

// Vectorised variant.  Work item = one 16-byte chunk of a head row (interleaved pairs) or the two chunks c and
// c + Dh/2 that hold each other's RoPE partners (half-split pairs).  The noise query always rotates (even, odd)
// neighbours of the ROTATED row (primitives.py:58-80), which lie inside one chunk, so an item is self-contained.
template <typename T, typename A>
__global__ void __launch_bounds__(320) prep_vec_kernel(PrepParams p) {
  constexpr int N = Vec16<T>::N;
  extern __shared__ float sm[];
  const int half = p.Dh >> 1;
  float* cs = sm;                 // [half] cos, rounded to T
  float* sn = sm + half;          // [half] sin
  bf16* csb = reinterpret_cast<bf16*>(sm + 2 * half);   // bf16 activations: the same tables as bf16, [half] cos | [half] sin
  bf16* snb = csb + half;
  constexpr bool PACKED = sizeof(T) == 2;
  const int tid = threadIdx.x, NT = blockDim.x;
  const long long ntok = (long long)p.B * p.L;
  const long long pos_base = ring_now(p.rp, p.W).pos;
  const int per_head = p.interleaved ? p.Dh / N : half / N;       // items per head row
  const int nq = p.H * per_head, nk = p.k ? p.Hkv * per_head : 0;
  for (long long tok = blockIdx.x; tok < ntok; tok += gridDim.x) {
    const int b = (int)(tok / p.L), t = (int)(tok % p.L);
    const long long pos = pos_base + t;
    __syncthreads();                                               // the previous token's table is no longer read
    for (int i = tid; i < half; i += NT) {
      float ta = El<A>::rnd((float)pos);
      float inv = El<A>::rnd(p.inv_freq[i]);
      float ang = El<A>::rnd(__fmul_rn(ta, inv));
      cs[i] = El<T>::rnd(El<A>::rnd(cosf(ang)));
      sn[i] = El<T>::rnd(El<A>::rnd(sinf(ang)));
      if (PACKED) { csb[i] = __float2bfloat16_rn(cs[i]); snb[i] = __float2bfloat16_rn(sn[i]); }
    }
    __syncthreads();
    T* qt = (T*)p.q + (long long)b * p.q_bs + (long long)t * p.q_rs;
    T* kt = p.k ? (T*)p.k + (long long)b * p.k_bs + (long long)t * p.k_rs : nullptr;
    T* qnt = (T*)p.qn + tok * (long long)(p.H * p.Dh);
    for (int w = tid; w < nq + nk; w += NT) {
      const bool isq = w < nq;
      const int ww = isq ? w : w - nq;
      const int h = ww / per_head, c = ww % per_head;
      T* row = (isq ? qt : kt) + h * p.Dh;
      const T* cth = (const T*)p.cos_t + h * half;
      const T* sth = (const T*)p.sin_t + h * half;
      if (PACKED) {
        // eight elements per 16-byte vector, four words of two; the tables' entries come four at a time (8 bytes)
        if (p.interleaved) {                // word j = pair i = 4c + j, rotated by the position's angle i
          uint4 xv = *reinterpret_cast<const uint4*>(row + c * N);
          const uint2 cw = *reinterpret_cast<const uint2*>(csb + 4 * c), sw = *reinterpret_cast<const uint2*>(snb + 4 * c);
          uint4 ov;
          ov.x = brot(xv.x, bdup_lo(cw.x), bdup_lo(sw.x)); ov.y = brot(xv.y, bdup_hi(cw.x), bdup_hi(sw.x));
          ov.z = brot(xv.z, bdup_lo(cw.y), bdup_lo(sw.y)); ov.w = brot(xv.w, bdup_hi(cw.y), bdup_hi(sw.y));
          *reinterpret_cast<uint4*>(row + c * N) = ov;
          if (isq) {
            const uint2 ct = *reinterpret_cast<const uint2*>(cth + 4 * c), st = *reinterpret_cast<const uint2*>(sth + 4 * c);
            uint4 nv;
            nv.x = brot(ov.x, bdup_lo(ct.x), bdup_lo(st.x)); nv.y = brot(ov.y, bdup_hi(ct.x), bdup_hi(st.x));
            nv.z = brot(ov.z, bdup_lo(ct.y), bdup_lo(st.y)); nv.w = brot(ov.w, bdup_hi(ct.y), bdup_hi(st.y));
            *reinterpret_cast<uint4*>(qnt + h * p.Dh + c * N) = nv;
          }
        } else {                            // x1 = elements 8c.., x2 = their partners half + 8c..; angles 8c..8c+7
          const uint4 x1 = *reinterpret_cast<const uint4*>(row + c * N), x2 = *reinterpret_cast<const uint4*>(row + half + c * N);
          const uint4 cv = *reinterpret_cast<const uint4*>(csb + c * N), sv = *reinterpret_cast<const uint4*>(snb + c * N);
          uint4 oa, ob;                       // x1 c + (-x2) s ; x2 c + x1 s
          oa.x = badd2(bmul2(x1.x, cv.x), bmul2(bneg2(x2.x), sv.x)); ob.x = badd2(bmul2(x2.x, cv.x), bmul2(x1.x, sv.x));
          oa.y = badd2(bmul2(x1.y, cv.y), bmul2(bneg2(x2.y), sv.y)); ob.y = badd2(bmul2(x2.y, cv.y), bmul2(x1.y, sv.y));
          oa.z = badd2(bmul2(x1.z, cv.z), bmul2(bneg2(x2.z), sv.z)); ob.z = badd2(bmul2(x2.z, cv.z), bmul2(x1.z, sv.z));
          oa.w = badd2(bmul2(x1.w, cv.w), bmul2(bneg2(x2.w), sv.w)); ob.w = badd2(bmul2(x2.w, cv.w), bmul2(x1.w, sv.w));
          *reinterpret_cast<uint4*>(row + c * N) = oa;
          *reinterpret_cast<uint4*>(row + half + c * N) = ob;
          if (isq) {                        // (even, odd) neighbours of the rotated row: pairs 4c.. and half/2 + 4c..
            const uint2 cta = *reinterpret_cast<const uint2*>(cth + 4 * c), sta = *reinterpret_cast<const uint2*>(sth + 4 * c);
            const uint2 ctb = *reinterpret_cast<const uint2*>(cth + (half >> 1) + 4 * c), stb = *reinterpret_cast<const uint2*>(sth + (half >> 1) + 4 * c);
            uint4 na, nb;
            na.x = brot(oa.x, bdup_lo(cta.x), bdup_lo(sta.x)); na.y = brot(oa.y, bdup_hi(cta.x), bdup_hi(sta.x));
            na.z = brot(oa.z, bdup_lo(cta.y), bdup_lo(sta.y)); na.w = brot(oa.w, bdup_hi(cta.y), bdup_hi(sta.y));
            nb.x = brot(ob.x, bdup_lo(ctb.x), bdup_lo(stb.x)); nb.y = brot(ob.y, bdup_hi(ctb.x), bdup_hi(stb.x));
            nb.z = brot(ob.z, bdup_lo(ctb.y), bdup_lo(stb.y)); nb.w = brot(ob.w, bdup_hi(ctb.y), bdup_hi(stb.y));
            *reinterpret_cast<uint4*>(qnt + h * p.Dh + c * N) = na;
            *reinterpret_cast<uint4*>(qnt + h * p.Dh + half + c * N) = nb;
          }
        }
      } else if (p.interleaved) {                  // primitives.py:99-106: pairs (2i, 2i+1) share cos/sin i
        float x[N], o[N];
        Vec16<T>::ld(row + c * N, x);
#pragma unroll
        for (int e = 0; e < N; e += 2) {
          const int i = (c * N + e) >> 1;
          const float cc = cs[i], ss = sn[i];
          o[e] = t_sub<T>(t_mul<T>(x[e], cc), t_mul<T>(x[e + 1], ss));
          o[e + 1] = t_add<T>(t_mul<T>(x[e], ss), t_mul<T>(x[e + 1], cc));
        }
        Vec16<T>::st(row + c * N, o);
        if (isq) {
          float n[N];
#pragma unroll
          for (int e = 0; e < N; e += 2) {
            const int i = (c * N + e) >> 1;
            const float ct = El<T>::ld(cth + i), st = El<T>::ld(sth + i);
            n[e] = t_sub<T>(t_mul<T>(o[e], ct), t_mul<T>(o[e + 1], st));
            n[e + 1] = t_add<T>(t_mul<T>(o[e], st), t_mul<T>(o[e + 1], ct));
          }
          Vec16<T>::st(qnt + h * p.Dh + c * N, n);
        }
      } else {                              // primitives.py:108-113: x*cos_full + rotate_half(x)*sin_full
        float x1[N], x2[N], oa[N], ob[N];
        Vec16<T>::ld(row + c * N, x1);
        Vec16<T>::ld(row + half + c * N, x2);
#pragma unroll
        for (int e = 0; e < N; ++e) {
          const float cc = cs[c * N + e], ss = sn[c * N + e];
          oa[e] = t_add<T>(t_mul<T>(x1[e], cc), t_mul<T>(-x2[e], ss));
          ob[e] = t_add<T>(t_mul<T>(x2[e], cc), t_mul<T>(x1[e], ss));
        }
        Vec16<T>::st(row + c * N, oa);
        Vec16<T>::st(row + half + c * N, ob);
        if (isq) {
          float na[N], nb[N];
#pragma unroll
          for (int e = 0; e < N; e += 2) {
            const int ia = (c * N + e) >> 1, ib = (half + c * N + e) >> 1;
            const float cta = El<T>::ld(cth + ia), sta = El<T>::ld(sth + ia);
            const float ctb = El<T>::ld(cth + ib), stb = El<T>::ld(sth + ib);
            na[e] = t_sub<T>(t_mul<T>(oa[e], cta), t_mul<T>(oa[e + 1], sta));
            na[e + 1] = t_add<T>(t_mul<T>(oa[e], sta), t_mul<T>(oa[e + 1], cta));
            nb[e] = t_sub<T>(t_mul<T>(ob[e], ctb), t_mul<T>(ob[e + 1], stb));
            nb[e + 1] = t_add<T>(t_mul<T>(ob[e], stb), t_mul<T>(ob[e + 1], ctb));
          }
          Vec16<T>::st(qnt + h * p.Dh + c * N, na);
          Vec16<T>::st(qnt + h * p.Dh + half + c * N, nb);
        }
      }
    }
    for (int h = tid; h < p.H; h += NT) {
      const float z = El<T>::ld((const T*)p.lam_logit + (long long)b * p.lam_bs + (long long)t * p.lam_rs + h);
      p.lam[tok * p.H + h] = t_sigmoid<T>(z);
    }
    if (tid == 0 && p.gate != nullptr) {
      float g = 1.0f;                       // write_policy "none": attention.py:407-408
      if (p.gated) g = t_sigmoid<T>(El<T>::ld((const T*)p.gate_logit + (long long)b * p.gate_bs + (long long)t * p.gate_rs));
      p.gate[tok] = g;
    }
  }
}

extern "C" int coda_b200_prep(const coda_layer_cfg* cfg, int32_t L, coda_ring_pos rp,
                              void* q, int64_t q_bs, int64_t q_rs,
                              void* k, int64_t k_bs, int64_t k_rs,
                              void* q_noise,
                              const void* lam_logit, int64_t lam_bs, int64_t lam_rs, float* lam,
                              const void* gate_logit, int64_t gate_bs, int64_t gate_rs, float* gate,
                              const float* inv_freq, const void* cos_theta, const void* sin_theta,
                              coda_stream_t stream) {
  CODA_REQUIRE(coda_cfg_ok(cfg), CODA_ERR_ARG, "prep: invalid layer configuration");
  CODA_REQUIRE(L >= 0, CODA_ERR_ARG, "prep: negative L");
  if (L == 0) return CODA_OK;
  CODA_REQUIRE(q && q_noise && lam_logit && lam && inv_freq && cos_theta && sin_theta, CODA_ERR_ARG, "prep: null pointer");
  CODA_REQUIRE(!(cfg->gated && gate && !gate_logit), CODA_ERR_ARG, "prep: gated write policy needs gate logits");
  PrepParams p;
  p.B = cfg->B; p.L = L; p.H = cfg->H; p.Hkv = cfg->Hkv; p.Dh = cfg->Dh;
  p.interleaved = cfg->rope_interleaved; p.gated = cfg->gated; p.rp = rp; p.W = cfg->W;
  p.q = q; p.q_bs = q_bs; p.q_rs = q_rs; p.k = k; p.k_bs = k_bs; p.k_rs = k_rs; p.qn = q_noise;
  p.lam_logit = lam_logit; p.lam_bs = lam_bs; p.lam_rs = lam_rs; p.lam = lam;
  p.gate_logit = gate_logit; p.gate_bs = gate_bs; p.gate_rs = gate_rs; p.gate = gate;
  p.inv_freq = inv_freq; p.cos_t = cos_theta; p.sin_t = sin_theta;
  const long long ntok = (long long)cfg->B * L;
  const int grid = (int)(ntok < 148LL * 16 ? ntok : 148LL * 16);
  const size_t smem = sizeof(float) * (size_t)(cfg->Dh + cfg->H * cfg->Dh);
  CODA_REQUIRE(smem <= 200 * 1024, CODA_ERR_LIMIT, "prep: H*Dh = %d exceeds the shared-memory row limit", cfg->H * cfg->Dh);
  cudaStream_t s = (cudaStream_t)stream;
  // 16-byte vectors need aligned rows and chunks that do not straddle a RoPE half / head row
  const int vn = cfg->dtype == CODA_F32 ? 4 : 8;
  const bool vec = ((cfg->rope_interleaved ? cfg->Dh : cfg->Dh / 2) % vn) == 0 && ((uintptr_t)q | (uintptr_t)q_noise) % 16 == 0 &&
                   (q_bs | q_rs) % vn == 0 && (k == nullptr || ((uintptr_t)k % 16 == 0 && (k_bs | k_rs) % vn == 0));
#define LAUNCH(T, A) do { \
    if (vec) { prep_vec_kernel<T, A><<<grid, 320, sizeof(float) * (size_t)cfg->Dh + 2 * sizeof(bf16) * (size_t)(cfg->Dh / 2), s>>>(p); break; } \
    if (smem > 48 * 1024) cudaFuncSetAttribute(prep_kernel<T, A>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    prep_kernel<T, A><<<grid, 256, smem, s>>>(p); } while (0)
  if (cfg->dtype == CODA_F32) {
    CODA_REQUIRE(cfg->angle_dtype == CODA_F32, CODA_ERR_ARG, "prep: fp32 activations need fp32 angles");
    LAUNCH(float, float);
  } else if (cfg->angle_dtype == CODA_BF16) {
    LAUNCH(bf16, bf16);
  } else {
    LAUNCH(bf16, float);
  }
#undef LAUNCH
  CODA_CHECK_LAUNCH("prep");
  return CODA_OK;
}
