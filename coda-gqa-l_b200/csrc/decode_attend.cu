// Fused decode attention for bf16 states (head_dim 64 or 128, up to 8 query heads per KV head).
//
// Persistent kernel: one CTA per SM, each walking over (state, KV head) planes plane = blockIdx.x, + gridDim.x, ...
// The K and V planes of a head -- all W+Me+Ms slots -- are read from HBM exactly once, by TMA
// (cp.async.bulk.tensor, 128-byte swizzle) into a 4-stage ring of 64-slot tiles in shared memory.  The producer
// warp streams tiles continuously ACROSS plane boundaries, so the ring never drains between work items and
// HBM stays busy while the consumers merge / write one plane and prepare the queries of the next (whose
// inputs are prefetched into registers one plane ahead).  Two groups of four consumer warps take alternate
// tiles; inside a group each warp owns 16 slots of the tile.  All query heads of the GQA group and both streams (signal and
// theta-rotated noise) share the staged tiles: they form the 16 rows of the m16n8k16 tensor-core tiles used
// for Q.K^T and P.V.  Per plane the prologue applies RoPE and the learned per-head rotation to the raw query
// projection and evaluates the lambda sigmoid; softmax is an online, per-warp one (quad shuffles), merged
// across the eight warps at the end; the epilogue subtracts lambda * noise and applies the head RMSNorm.
//
// HBM traffic per plane = the two planes (2 * Lbuf * Dh * 2 bytes) + a few hundred bytes of q, lambda, mask
// and output: the kernel is bandwidth-bound by construction.  Every mbarrier wait is bounded; on expiry a
// status word is set and the kernel finishes (with undefined output) instead of hanging.
#include "coda_common.cuh"
#include "tma_utils.cuh"
#include "tensor_maps.h"

namespace {

constexpr int DA_TILE = 64;          // slots per stage
constexpr int DA_STAGES = 4;
constexpr int DA_CWARPS = 8;         // consumer warps (two groups of four)
constexpr int DA_THREADS = (DA_CWARPS + 1) * 32;

struct DecodeParams {
  int B, H, Hkv, G, Lbuf, mask_unused, norm_full, interleaved, angle_bf16;
  float eps, scale_log2;
  coda_ring_pos rp; int W; int pos_minus_one;     // query position = ring position (- 1 when the token was written first)
  const bf16* q; long long q_bs;                  // raw query projection [B][H*Dh]
  const bf16* lam_logit; long long lam_bs;        // [B][H]
  const float* inv_freq; const bf16* cos_t; const bf16* sin_t;
  const uint8_t* allowed;
  const bf16* norm_w;
  bf16* out; long long out_bs;
  int* status;
};

using tma::smem_u32; using tma::mbar_init; using tma::mbar_expect_tx; using tma::mbar_arrive; using tma::mbar_try;
__device__ __forceinline__ void mbar_wait(uint64_t* bar, uint32_t parity, int* status, int code) { tma::mbar_wait(bar, parity, status, code); }
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
               ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ void bar_consumers() { asm volatile("bar.sync 1, %0;" ::"n"(DA_CWARPS * 32) : "memory"); }

// Byte offset of 16-byte chunk `c` of row `s` inside a [64 x DH] bf16 tile written by TMA as DH/64
// boxes of 64 rows x 128 bytes with the 128-byte swizzle (chunk index XOR row mod 8).
template <int DH>
__device__ __forceinline__ uint32_t tile_off(int s, int c) {
  return (uint32_t)((c >> 3) * (DA_TILE * 128) + s * 128 + (((c & 7) ^ (s & 7)) << 4));
}

template <int DH>
__global__ void __launch_bounds__(DA_THREADS, 1)
decode_attend_kernel(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap, DecodeParams p) {
  constexpr int HALF = DH / 2;
  constexpr int KSTEPS = DH / 16;            // k-steps of Q.K^T
  constexpr int NT_O = DH / 8;               // n-tiles of the output
  constexpr int TILE_BYTES = DA_TILE * DH * 2;
  constexpr int QSTR = DH + 8;               // padded row stride of the staged queries (elements)
  constexpr int CT = DA_CWARPS * 32;         // consumer threads

  extern __shared__ unsigned char smem_raw[];
  // the swizzled TMA tiles need a 1024-byte aligned base; the launch reserves the slack
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  unsigned char* stage0 = smem;                                            // DA_STAGES * 2 * TILE_BYTES
  float* comb = reinterpret_cast<float*>(smem + DA_STAGES * 2 * TILE_BYTES);   // [DA_CWARPS][16][DH] partial outputs
  bf16* sQ = reinterpret_cast<bf16*>(comb + DA_CWARPS * 16 * DH);          // [16][QSTR]
  float* sML = reinterpret_cast<float*>(sQ + 16 * QSTR);                   // [2][DA_CWARPS][16]  (m, l)
  float* sLam = sML + 2 * DA_CWARPS * 16;                                  // [8]
  float* sCS = sLam + 8;                                                   // [HALF] cos, [HALF] sin
  uint64_t* full = reinterpret_cast<uint64_t*>(sCS + 2 * HALF);            // [DA_STAGES]
  uint64_t* empty = full + DA_STAGES;                                      // [DA_STAGES]
  uint8_t* sAl = reinterpret_cast<uint8_t*>(empty + DA_STAGES);            // [Lbuf rounded up to a tile]

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int G = p.G;
  const int nst = (p.Lbuf + DA_TILE - 1) / DA_TILE;
  const int nplanes = p.B * p.Hkv;

  if (tid == 0) {
    for (int i = 0; i < DA_STAGES; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], 4); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  if (warp == DA_CWARPS) {
    // ---------------- producer: keep the ring of K/V tiles full, across plane boundaries ----------------
    if (lane == 0) {
      int t = 0;                                           // tiles issued by this CTA so far (all planes)
      for (int plane = blockIdx.x; plane < nplanes; plane += gridDim.x) {
        for (int s = 0; s < nst; ++s, ++t) {
          const int bi = t % DA_STAGES;
          if (t >= DA_STAGES) mbar_wait(&empty[bi], ((t / DA_STAGES) - 1) & 1, p.status, 1);
          mbar_expect_tx(&full[bi], 2 * TILE_BYTES);
          unsigned char* kd = stage0 + bi * 2 * TILE_BYTES;
          unsigned char* vd = kd + TILE_BYTES;
#pragma unroll
          for (int hf = 0; hf < DH / 64; ++hf) {
            tma_load_3d(kd + hf * (DA_TILE * 128), &kmap, &full[bi], hf * 64, s * DA_TILE, plane);
            tma_load_3d(vd + hf * (DA_TILE * 128), &vmap, &full[bi], hf * 64, s * DA_TILE, plane);
          }
        }
      }
    }
    return;
  }

  // ---------------- consumers: two groups of four warps, each taking every other tile ----------------
  const int grp = warp >> 2, gw = warp & 3;            // group, warp inside the group (owns slots gw*16..+15 of a tile)
  // RoPE cos/sin of the query position: the same for every plane
  const long long qpos = ring_now(p.rp, p.W).pos - p.pos_minus_one;
  for (int i = tid; i < HALF; i += CT) {
    float ta = (float)qpos, inv = p.inv_freq[i];
    if (p.angle_bf16) { ta = bf16_round(ta); inv = bf16_round(inv); }
    float ang = __fmul_rn(ta, inv);
    if (p.angle_bf16) ang = bf16_round(ang);
    float c = cosf(ang), s = sinf(ang);
    if (p.angle_bf16) { c = bf16_round(c); s = bf16_round(s); }
    sCS[i] = bf16_round(c);
    sCS[HALF + i] = bf16_round(s);
  }
  for (int i = tid; i < 16 * QSTR; i += CT) sQ[i] = __float2bfloat16_rn(0.f);   // rows >= 2G stay zero

  // Per-plane inputs are fetched one plane ahead into registers, so that only the first plane's prologue
  // waits on global memory.  Work split of the G*HALF (head, pair) items: item w = tid, tid + CT, ...
  constexpr int ITEMS = (8 * HALF + CT - 1) / CT;      // G <= 8
  constexpr int ALW = (4096 / CT + 3) / 4;             // allowed mask words per thread (Lbuf <= 4096)
  float pre_qa[ITEMS], pre_qb[ITEMS], pre_ct[ITEMS], pre_st[ITEMS], pre_lam = 0.f;
  uint32_t pre_al[ALW];
  auto prefetch = [&](int plane) {
    const int b = plane / p.Hkv, hk = plane % p.Hkv;
    const bf16* qrow = p.q + (long long)b * p.q_bs + (long long)hk * G * DH;
#pragma unroll
    for (int it = 0; it < ITEMS; ++it) {
      const int w = tid + it * CT;
      pre_qa[it] = pre_qb[it] = pre_ct[it] = pre_st[it] = 0.f;
      if (w < G * HALF) {
        const int g = w / HALF, i = w % HALF;
        const int ia = p.interleaved ? 2 * i : i, ib = p.interleaved ? 2 * i + 1 : i + HALF;
        pre_qa[it] = __bfloat162float(qrow[g * DH + ia]);
        pre_qb[it] = __bfloat162float(qrow[g * DH + ib]);
        pre_ct[it] = __bfloat162float(p.cos_t[(hk * G + g) * HALF + i]);
        pre_st[it] = __bfloat162float(p.sin_t[(hk * G + g) * HALF + i]);
      }
    }
    if (tid < G) pre_lam = __bfloat162float(p.lam_logit[(long long)b * p.lam_bs + hk * G + tid]);
#pragma unroll
    for (int a = 0; a < ALW; ++a) {
      const int i0 = (tid + a * CT) * 4;
      uint32_t wv = 0;
      if (i0 + 3 < p.Lbuf && ((reinterpret_cast<uintptr_t>(p.allowed + (long long)b * p.Lbuf + i0) & 3) == 0)) {
        wv = *reinterpret_cast<const uint32_t*>(p.allowed + (long long)b * p.Lbuf + i0);
      } else {
        for (int e = 0; e < 4; ++e) if (i0 + e < p.Lbuf) wv |= (uint32_t)p.allowed[(long long)b * p.Lbuf + i0 + e] << (8 * e);
      }
      pre_al[a] = wv;
    }
  };
  if ((int)blockIdx.x < nplanes) prefetch(blockIdx.x);
  bar_consumers();

  int tbase = 0;                                           // tiles consumed before the current plane
  for (int plane = blockIdx.x; plane < nplanes; plane += gridDim.x, tbase += nst) {
    const int b = plane / p.Hkv, hk = plane % p.Hkv;
    // ---- prologue: RoPE -> signal rows, learned (even, odd) rotation -> noise rows, lambda, mask ----
#pragma unroll
    for (int it = 0; it < ITEMS; ++it) {
      const int w = tid + it * CT;
      if (w < G * HALF) {
        const int g = w / HALF, i = w % HALF;
        const float c = sCS[i], s = sCS[HALF + i];
        float oa, ob; int ia, ib;
        if (p.interleaved) {
          ia = 2 * i; ib = 2 * i + 1;
          oa = t_sub<bf16>(t_mul<bf16>(pre_qa[it], c), t_mul<bf16>(pre_qb[it], s));
          ob = t_add<bf16>(t_mul<bf16>(pre_qa[it], s), t_mul<bf16>(pre_qb[it], c));
        } else {
          ia = i; ib = i + HALF;
          oa = t_add<bf16>(t_mul<bf16>(pre_qa[it], c), t_mul<bf16>(-pre_qb[it], s));
          ob = t_add<bf16>(t_mul<bf16>(pre_qb[it], c), t_mul<bf16>(pre_qa[it], s));
        }
        sQ[g * QSTR + ia] = __float2bfloat16_rn(oa);
        sQ[g * QSTR + ib] = __float2bfloat16_rn(ob);
      }
    }
    if (tid < G) sLam[tid] = t_sigmoid<bf16>(pre_lam);
#pragma unroll
    for (int a = 0; a < ALW; ++a) {
      const int i0 = (tid + a * CT) * 4;
      if (i0 < nst * DA_TILE) *reinterpret_cast<uint32_t*>(sAl + i0) = pre_al[a];
    }
    bar_consumers();
#pragma unroll
    for (int it = 0; it < ITEMS; ++it) {
      const int w = tid + it * CT;
      if (w < G * HALF) {
        const int g = w / HALF, i = w % HALF;
        const float qe = __bfloat162float(sQ[g * QSTR + 2 * i]), qo = __bfloat162float(sQ[g * QSTR + 2 * i + 1]);
        sQ[(G + g) * QSTR + 2 * i] = __float2bfloat16_rn(t_sub<bf16>(t_mul<bf16>(qe, pre_ct[it]), t_mul<bf16>(qo, pre_st[it])));
        sQ[(G + g) * QSTR + 2 * i + 1] = __float2bfloat16_rn(t_add<bf16>(t_mul<bf16>(qe, pre_st[it]), t_mul<bf16>(qo, pre_ct[it])));
      }
    }
    bar_consumers();
    // inputs of the next plane: in flight while this plane's tiles are processed
    if (plane + (int)gridDim.x < nplanes) prefetch(plane + gridDim.x);

    uint32_t qf[KSTEPS][4];
    {
      const uint32_t qbase = smem_u32(sQ) + (uint32_t)(((lane & 15) * QSTR + (lane >> 4) * 8) * 2);
#pragma unroll
      for (int kk = 0; kk < KSTEPS; ++kk) ldsm_x4(qf[kk], qbase + kk * 32);
    }
    float oacc[NT_O][4];
#pragma unroll
    for (int j = 0; j < NT_O; ++j) { oacc[j][0] = oacc[j][1] = oacc[j][2] = oacc[j][3] = 0.f; }
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;   // rows lane/4 and lane/4 + 8
    const int li = lane >> 3, lr = lane & 7;

    for (int s = grp; s < nst; s += 2) {
      const int t = tbase + s;
      const int bi = t % DA_STAGES;
      mbar_wait(&full[bi], (t / DA_STAGES) & 1, p.status, 2);
      const uint32_t kb = smem_u32(stage0 + bi * 2 * TILE_BYTES);
      const uint32_t vb = kb + TILE_BYTES;
      // ---- S = Q K^T over this warp's 16 slots (two accumulation chains per n-tile) ----
      float sc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
      float sd[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
      const int krow = gw * 16 + (li >> 1) * 8 + lr;
#pragma unroll
      for (int kk = 0; kk < KSTEPS; kk += 2) {
        uint32_t kf[4], kg[4];
        ldsm_x4(kf, kb + tile_off<DH>(krow, kk * 2 + (li & 1)));
        ldsm_x4(kg, kb + tile_off<DH>(krow, (kk + 1) * 2 + (li & 1)));
        mma_bf16(sc[0], qf[kk], kf[0], kf[1]);
        mma_bf16(sc[1], qf[kk], kf[2], kf[3]);
        mma_bf16(sd[0], qf[kk + 1], kg[0], kg[1]);
        mma_bf16(sd[1], qf[kk + 1], kg[2], kg[3]);
      }
      // ---- mask + online softmax (rows r0 = lane/4, r1 = r0 + 8) ----
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int slot = s * DA_TILE + gw * 16 + nt * 8 + 2 * (lane & 3) + e;
          const bool vis = slot < p.Lbuf && (!p.mask_unused || sAl[slot] != 0);
          sc[nt][e] = vis ? (sc[nt][e] + sd[nt][e]) * p.scale_log2 : -INFINITY;
          sc[nt][2 + e] = vis ? (sc[nt][2 + e] + sd[nt][2 + e]) * p.scale_log2 : -INFINITY;
          mx0 = fmaxf(mx0, sc[nt][e]);
          mx1 = fmaxf(mx1, sc[nt][2 + e]);
        }
      }
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      const float nm0 = fmaxf(m0, mx0), nm1 = fmaxf(m1, mx1);
      const float ref0 = nm0 == -INFINITY ? 0.f : nm0, ref1 = nm1 == -INFINITY ? 0.f : nm1;
      const float a0 = exp2f(m0 - ref0), a1 = exp2f(m1 - ref1);
      m0 = nm0; m1 = nm1;
      uint32_t pf[4];
      {
        const float p00 = exp2f(sc[0][0] - ref0), p01 = exp2f(sc[0][1] - ref0), p02 = exp2f(sc[0][2] - ref1), p03 = exp2f(sc[0][3] - ref1);
        const float p10 = exp2f(sc[1][0] - ref0), p11 = exp2f(sc[1][1] - ref0), p12 = exp2f(sc[1][2] - ref1), p13 = exp2f(sc[1][3] - ref1);
        l0 = l0 * a0 + (p00 + p01 + p10 + p11);
        l1 = l1 * a1 + (p02 + p03 + p12 + p13);
        pf[0] = pack_bf16(p00, p01); pf[1] = pack_bf16(p02, p03); pf[2] = pack_bf16(p10, p11); pf[3] = pack_bf16(p12, p13);
      }
      if (a0 != 1.f || a1 != 1.f) {
#pragma unroll
        for (int j = 0; j < NT_O; ++j) { oacc[j][0] *= a0; oacc[j][1] *= a0; oacc[j][2] *= a1; oacc[j][3] *= a1; }
      }
      // ---- O += P V ----
      const int vrow = gw * 16 + (li & 1) * 8 + lr;
#pragma unroll
      for (int j = 0; j < NT_O; j += 2) {
        uint32_t vf[4];
        ldsm_x4_t(vf, vb + tile_off<DH>(vrow, j + (li >> 1)));
        mma_bf16(oacc[j], pf, vf[0], vf[1]);
        mma_bf16(oacc[j + 1], pf, vf[2], vf[3]);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[bi]);
    }

    // ---- merge the eight warps' partial softmaxes ----
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    if ((lane & 3) == 0) {
      const int r = lane >> 2;
      sML[warp * 16 + r] = m0; sML[warp * 16 + r + 8] = m1;
      sML[DA_CWARPS * 16 + warp * 16 + r] = l0; sML[DA_CWARPS * 16 + warp * 16 + r + 8] = l1;
    }
    {
      // only the 2G live rows are exchanged (row r and r + 8 of the accumulator tile)
      const int r = lane >> 2, cb = 2 * (lane & 3);
#pragma unroll
      for (int j = 0; j < NT_O; ++j) {
        if (r < 2 * G) {
          float* d0 = comb + ((warp * 16 + r) * DH + j * 8 + cb);
          d0[0] = oacc[j][0]; d0[1] = oacc[j][1];
        }
        if (r + 8 < 2 * G) {
          float* d1 = comb + ((warp * 16 + r + 8) * DH + j * 8 + cb);
          d1[0] = oacc[j][2]; d1[1] = oacc[j][3];
        }
      }
    }
    bar_consumers();

    // ---- epilogue: one warp per query head: sig - lam*noise, optional RMSNorm, bf16 store ----
    for (int g = warp; g < G; g += DA_CWARPS) {
      float os[DH / 32], on[DH / 32];
#pragma unroll
      for (int st = 0; st < 2; ++st) {
        const int row = st * G + g;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < DA_CWARPS; ++w) M = fmaxf(M, sML[w * 16 + row]);
        float f[DA_CWARPS], L = 0.f;
#pragma unroll
        for (int w = 0; w < DA_CWARPS; ++w) {
          const float mw = sML[w * 16 + row];
          f[w] = (mw == -INFINITY) ? 0.f : exp2f(mw - M);
          L += f[w] * sML[DA_CWARPS * 16 + w * 16 + row];
        }
        const float inv = L > 0.f ? 1.f / L : 0.f;
#pragma unroll
        for (int i = 0; i < DH / 32; ++i) {
          const int d = lane + 32 * i;
          float acc = 0.f;
#pragma unroll
          for (int w = 0; w < DA_CWARPS; ++w) acc += f[w] * comb[(w * 16 + row) * DH + d];
          const float v = bf16_round(acc * inv);
          if (st == 0) os[i] = v; else on[i] = v;
        }
      }
      const float lam = sLam[g];
      float diff[DH / 32], sq = 0.f;
#pragma unroll
      for (int i = 0; i < DH / 32; ++i) {
        diff[i] = t_sub<bf16>(os[i], t_mul<bf16>(lam, on[i]));
        sq += bf16_round(diff[i] * diff[i]);
      }
      bf16* op = p.out + (long long)b * p.out_bs + (long long)(hk * G + g) * DH;
      if (p.norm_full) {
        const float var = bf16_round(warp_sum(sq) / (float)DH);
        const float rs = bf16_round(rsqrtf(bf16_round(var + p.eps)));
#pragma unroll
        for (int i = 0; i < DH / 32; ++i) {
          const int d = lane + 32 * i;
          op[d] = __float2bfloat16_rn(t_mul<bf16>(t_mul<bf16>(diff[i], rs), __bfloat162float(p.norm_w[d])));
        }
      } else {
#pragma unroll
        for (int i = 0; i < DH / 32; ++i) op[lane + 32 * i] = __float2bfloat16_rn(diff[i]);
      }
    }
    bar_consumers();                       // sQ / sML / comb / sAl are rewritten by the next plane's prologue
  }  // plane loop
}

template <int DH>
size_t decode_smem(int Lbuf) {
  const int nst = (Lbuf + DA_TILE - 1) / DA_TILE;
  return (size_t)DA_STAGES * 2 * DA_TILE * DH * 2 + (size_t)DA_CWARPS * 16 * DH * 4 + 16 * (DH + 8) * 2 + (2 * DA_CWARPS * 16 + 8 + DH) * 4 +
         2 * DA_STAGES * 8 + (size_t)nst * DA_TILE + 16 + 1024;
}

template <int DH>
int launch_decode(const CUtensorMap& km, const CUtensorMap& vm, const DecodeParams& p, cudaStream_t s) {
  const size_t smem = decode_smem<DH>(p.Lbuf);
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(decode_attend_kernel<DH>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024);
    configured = true;
  }
  CODA_REQUIRE(smem <= 226 * 1024, CODA_ERR_LIMIT, "decode_attend: %d slots need %zu bytes of shared memory", p.Lbuf, smem);
  static int num_sms = 0;
  if (num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || num_sms <= 0) num_sms = 148;
  }
  const int nplanes = p.B * p.Hkv;
  decode_attend_kernel<DH><<<nplanes < num_sms ? nplanes : num_sms, DA_THREADS, smem, s>>>(km, vm, p);
  CODA_CHECK_LAUNCH("decode_attend");
  return CODA_OK;
}

}  // namespace

// True when the tuned kernel covers this configuration; otherwise callers use the generic kernels.
extern "C" int coda_b200_decode_attend_supported(const coda_layer_cfg* cfg) {
  if (!coda_cfg_ok(cfg)) return 0;
  const int G = cfg->H / cfg->Hkv;
  return cfg->dtype == CODA_BF16 && (cfg->Dh == 64 || cfg->Dh == 128) && G <= 8 &&
         (size_t)(cfg->W + cfg->Me + cfg->Ms) <= 4096 && tmaps::available();
}

extern "C" int coda_b200_decode_attend(const coda_layer_cfg* cfg, const coda_state_ptrs* st, coda_ring_pos rp,
                                       int32_t token_already_written,
                                       const void* q_raw, int64_t q_bs, const void* lam_logit, int64_t lam_bs,
                                       const float* inv_freq, const void* cos_theta, const void* sin_theta,
                                       const void* norm_w, void* out, int64_t out_bs, int32_t* status,
                                       coda_stream_t stream) {
  CODA_REQUIRE(coda_cfg_ok(cfg) && st, CODA_ERR_ARG, "decode_attend: invalid layer configuration");
  CODA_REQUIRE(coda_b200_decode_attend_supported(cfg), CODA_ERR_ARG,
               "decode_attend: needs bf16, head_dim 64 or 128 and at most 8 query heads per KV head");
  CODA_REQUIRE(q_raw && lam_logit && inv_freq && cos_theta && sin_theta && out && st->k_buf && st->v_buf && st->allowed,
               CODA_ERR_ARG, "decode_attend: null pointer");
  CODA_REQUIRE(!cfg->head_norm_full || norm_w, CODA_ERR_ARG, "decode_attend: head-norm weight missing");
  CODA_REQUIRE(((uintptr_t)st->k_buf % 16 == 0) && ((uintptr_t)st->v_buf % 16 == 0), CODA_ERR_ARG,
               "decode_attend: k_buf / v_buf must be 16-byte aligned");
  const int Lbuf = cfg->W + cfg->Me + cfg->Ms;
  CUtensorMap km, vm;
  CODA_REQUIRE(tmaps::plane_map(&km, st->k_buf, cfg->B * cfg->Hkv, Lbuf, cfg->Dh) &&
               tmaps::plane_map(&vm, st->v_buf, cfg->B * cfg->Hkv, Lbuf, cfg->Dh), CODA_ERR_LAUNCH,
               "decode_attend: cuTensorMapEncodeTiled failed");
  DecodeParams p;
  p.B = cfg->B; p.H = cfg->H; p.Hkv = cfg->Hkv; p.G = cfg->H / cfg->Hkv; p.Lbuf = Lbuf;
  p.mask_unused = cfg->mask_unused; p.norm_full = cfg->head_norm_full; p.interleaved = cfg->rope_interleaved;
  p.angle_bf16 = cfg->angle_dtype == CODA_BF16; p.eps = cfg->eps;
  p.scale_log2 = 1.4426950408889634f / sqrtf((float)cfg->Dh);
  p.rp = rp; p.W = cfg->W; p.pos_minus_one = token_already_written ? 1 : 0;
  p.q = (const bf16*)q_raw; p.q_bs = q_bs; p.lam_logit = (const bf16*)lam_logit; p.lam_bs = lam_bs;
  p.inv_freq = inv_freq; p.cos_t = (const bf16*)cos_theta; p.sin_t = (const bf16*)sin_theta;
  p.allowed = st->allowed; p.norm_w = (const bf16*)norm_w; p.out = (bf16*)out; p.out_bs = out_bs; p.status = status;
  cudaStream_t s = (cudaStream_t)stream;
  return cfg->Dh == 128 ? launch_decode<128>(km, vm, p, s) : launch_decode<64>(km, vm, p, s);
}
