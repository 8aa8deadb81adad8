// Fused decode attention for bf16 states (head_dim 64 or 128, up to 8 query heads per KV head).
//
// Persistent kernel: one CTA per SM, each walking over (state, KV head) planes plane = blockIdx.x, + gridDim.x, ...
// The K and V planes of a head -- all W+Me+Ms slots -- are read from HBM exactly once, by TMA
// (cp.async.bulk.tensor, 128-byte swizzle) into a ring of 64-slot tiles in shared memory.  Three roles:
//   * one producer warp streams tiles continuously ACROSS plane boundaries, so the ring never drains between
//     work items;
//   * eight consumer warps (two groups of four taking alternate tiles; inside a group each warp owns 16 slots
//     of the tile) do nothing but tensor-core work: all query heads of the GQA group and both streams (signal
//     and theta-rotated noise) share the staged tiles as the 16 rows of the m16n8k16 tiles used for Q.K^T and
//     P.V, with an online per-warp softmax (quad shuffles);
//   * four auxiliary warps prepare the queries of the NEXT plane (RoPE, learned per-head rotation, lambda
//     sigmoid, visibility mask; double-buffered) and finish the PREVIOUS one (merge of the eight partial
//     softmaxes, signal - lambda * noise, head RMSNorm, store) while the consumers are already on the next
//     plane's tiles.
// The roles meet only through mbarriers in shared memory.
//
// HBM traffic per plane = the two planes (2 * Lbuf * Dh * 2 bytes) + a few hundred bytes of q, lambda, mask
// and output: the kernel is bandwidth-bound by construction.  Every mbarrier wait is bounded; on expiry a
// status word is set and the kernel finishes (with undefined output) instead of hanging.
#include "coda_common.cuh"
#include "tma_utils.cuh"
#include "tensor_maps.h"

namespace {

constexpr int DA_TILE = 64;          // slots per stage
constexpr int DA_MAX_STAGES = 8;
constexpr int DA_CWARPS = 8;         // consumer warps (two groups of four)
constexpr int DA_AWARPS = 4;         // auxiliary warps (query preparation, merge + epilogue)
constexpr int DA_THREADS = (DA_CWARPS + DA_AWARPS + 4) * 32;   // the producer's warpgroup has one working warp

struct DecodeParams {
  int B, H, Hkv, G, Lbuf, mask_unused, norm_full, interleaved, angle_bf16, stages;
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
__device__ __forceinline__ uint32_t movmatrix_t(uint32_t x) {
  uint32_t y;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(y) : "r"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ void bar_aux() { asm volatile("bar.sync 2, %0;" ::"n"(DA_AWARPS * 32) : "memory"); }

// Byte offset of 16-byte chunk `c` of row `s` inside a [64 x DH] bf16 tile written by TMA as DH/64
// boxes of 64 rows x 128 bytes with the 128-byte swizzle (chunk index XOR row mod 8).
template <int DH>
__device__ __forceinline__ uint32_t tile_off(int s, int c) {
  return (uint32_t)((c >> 3) * (DA_TILE * 128) + s * 128 + (((c & 7) ^ (s & 7)) << 4));
}

// Shared-memory carve-up, the same on host and device.  RL = live query rows (2 * G).
template <int DH>
struct DecodeSmem {
  static constexpr int TILE_BYTES = DA_TILE * DH * 2;
  static constexpr int QSTR = DH + 8;               // padded row stride of the staged queries (elements)
  int comb, sq, sml, slam, scs, bars, sal, total;
  __host__ __device__ DecodeSmem(int stages, int G, int nst) {
    int o = stages * 2 * TILE_BYTES;
    comb = o; o += DA_CWARPS * 2 * G * DH * 4;      // [DA_CWARPS][2G][DH] partial outputs
    sq = o;   o += 2 * 16 * QSTR * 2;               // [2][16][QSTR] staged queries (double-buffered)
    sml = o;  o += 2 * DA_CWARPS * 16 * 4;          // [2][DA_CWARPS][16]  (m, l)
    slam = o; o += 2 * 8 * 4;                       // [2][8] lambda
    scs = o;  o += DH * 4;                          // [DH/2] cos, [DH/2] sin
    bars = o; o += (2 * DA_MAX_STAGES + 4) * 8;     // full[], empty[], q_ready[2], comb_full, comb_free
    sal = o;  o += 2 * nst * DA_TILE;               // [2][nst * DA_TILE] visibility mask
    total = o;
  }
};

template <int DH, int NQ>
__global__ void __launch_bounds__(DA_THREADS, 1)
decode_attend_kernel(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap, DecodeParams p) {
  constexpr int HALF = DH / 2;
  constexpr int KSTEPS = DH / 16;            // k-steps of Q.K^T
  constexpr int MT_O = DH / 16;              // m-tiles of the (transposed) output
  constexpr int TILE_BYTES = DA_TILE * DH * 2;
  constexpr int QSTR = DH + 8;
  constexpr int AT = DA_AWARPS * 32;         // auxiliary threads

  extern __shared__ unsigned char smem_raw[];
  // the swizzled TMA tiles need a 1024-byte aligned base; the launch reserves the slack
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int G = p.G, RL = 2 * G, S = p.stages;
  const int nst = (p.Lbuf + DA_TILE - 1) / DA_TILE;
  const int nplanes = p.B * p.Hkv;
  const DecodeSmem<DH> L(S, G, nst);
  unsigned char* stage0 = smem;
  float* comb = reinterpret_cast<float*>(smem + L.comb);
  bf16* sQ = reinterpret_cast<bf16*>(smem + L.sq);
  float* sML = reinterpret_cast<float*>(smem + L.sml);
  float* sLam = reinterpret_cast<float*>(smem + L.slam);
  float* sCS = reinterpret_cast<float*>(smem + L.scs);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L.bars);
  uint64_t* empty = full + DA_MAX_STAGES;
  uint64_t* q_ready = empty + DA_MAX_STAGES;       // [2]
  uint64_t* comb_full = q_ready + 2;
  uint64_t* comb_free = comb_full + 1;
  uint8_t* sAl = smem + L.sal;
  const int al_stride = nst * DA_TILE;

  // ---- auxiliary warps: first requests, issued before the producer starts to fill the ring ----
  const bool is_aux = warp >= DA_CWARPS && warp < DA_CWARPS + DA_AWARPS;
  const int at = tid - DA_CWARPS * 32, aw = warp - DA_CWARPS;
  // Global loads of these warps queue behind the tile traffic of the whole chip (a few thousand cycles when
  // the ring is being filled), so every input of a plane is requested in ONE batch into registers
  // (fetch), long before it is consumed (stage).  Item (g, i): RoPE'd elements 2i and 2i+1 of head g
  // (signal row g) and their learned (even, odd) rotation by theta (noise row G + g).
  constexpr int ITEMS = (8 * HALF + AT - 1) / AT;        // G <= 8
  constexpr int ALW = (4096 / 4 + AT - 1) / AT;          // mask words per thread (Lbuf <= 4096)
  struct Inputs { uint32_t q0[ITEMS], q1[ITEMS], al[ALW]; bf16 ct[ITEMS], st[ITEMS]; float lam; };
  // Two sets: set (k % 2) holds the inputs of this CTA's k-th plane.  A request stands behind everything the
  // producer has in flight for this SM (a full ring: several microseconds at this SM's share of the HBM
  // bandwidth), so it is made two planes ahead.
  Inputs inA, inB;
  auto fetch = [&](int plane, Inputs& in) {
    const int b = plane / p.Hkv, hk = plane % p.Hkv;
    const bf16* qrow = p.q + (long long)b * p.q_bs + (long long)hk * G * DH;
#pragma unroll
    for (int it = 0; it < ITEMS; ++it) {
      const int w = at + it * AT;
      in.q0[it] = in.q1[it] = 0u;
      in.ct[it] = in.st[it] = __float2bfloat16_rn(0.f);
      if (w < G * HALF) {
        const int g = w / HALF, i = w % HALF;
        const bf16* qh = qrow + g * DH;
        if (p.interleaved) {
          in.q0[it] = *reinterpret_cast<const uint32_t*>(qh + 2 * i);
        } else {
          const int pi = 2 * i < HALF ? 2 * i : 2 * i - HALF;        // pair index of element 2i (2i+1: the next)
          in.q0[it] = *reinterpret_cast<const uint32_t*>(qh + pi);
          in.q1[it] = *reinterpret_cast<const uint32_t*>(qh + pi + HALF);
        }
        in.ct[it] = p.cos_t[(hk * G + g) * HALF + i];
        in.st[it] = p.sin_t[(hk * G + g) * HALF + i];
      }
    }
    in.lam = 0.f;
    if (at < G) in.lam = __bfloat162float(p.lam_logit[(long long)b * p.lam_bs + hk * G + at]);
    const uint8_t* alb = p.allowed + (long long)b * p.Lbuf;
    const bool al4 = (reinterpret_cast<uintptr_t>(alb) & 3) == 0;
#pragma unroll
    for (int a = 0; a < ALW; ++a) {
      const int i0 = (at + a * AT) * 4;
      uint32_t wv = 0;
      if (i0 < p.Lbuf) {
        if (al4 && i0 + 3 < p.Lbuf) wv = *reinterpret_cast<const uint32_t*>(alb + i0);
        else for (int e = 0; e < 4; ++e) if (i0 + e < p.Lbuf) wv |= (uint32_t)alb[i0 + e] << (8 * e);
      }
      in.al[a] = wv;
    }
  };
  constexpr int DV = 4;                                  // output dims per lane in the epilogue: 4*lane .. 4*lane+3
  const bool dact = 4 * lane < DH;                       // (head_dim 64: the upper half-warp idles there)
  float nw[DV], inv_pre = 0.f;
  long long steps_pre = 0;
  if (is_aux) {
    if ((int)blockIdx.x < nplanes) fetch(blockIdx.x, inA);
    if ((int)(blockIdx.x + gridDim.x) < nplanes) fetch(blockIdx.x + gridDim.x, inB);
    if (at < HALF) inv_pre = p.inv_freq[at];
    if (p.rp.step_dev != nullptr) steps_pre = *p.rp.step_dev;
#pragma unroll
    for (int k = 0; k < DV; ++k) nw[k] = (p.norm_full && dact) ? __bfloat162float(p.norm_w[4 * lane + k]) : 1.f;
  }

  if (tid == 0) {
    for (int i = 0; i < S; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], 4); }
    mbar_init(&q_ready[0], DA_AWARPS); mbar_init(&q_ready[1], DA_AWARPS);
    mbar_init(comb_full, DA_CWARPS); mbar_init(comb_free, DA_AWARPS);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // The producer starts only here, after the auxiliary warps have made their first requests: whatever is
  // requested later (instruction and constant fetches included) stands behind a ring's worth of tile traffic.
  __syncthreads();

  // Registers follow the roles (per warpgroup): the consumers hold the output accumulators and the query
  // fragments, the other warps need little.
  if (warp >= DA_CWARPS + DA_AWARPS) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
    if (warp > DA_CWARPS + DA_AWARPS) return;
    // ---------------- producer: keep the ring of K/V tiles full, across plane boundaries ----------------
    if (lane == 0) {
      int bi = 0, round = 0;                               // ring slot and how often the ring has wrapped
      for (int plane = blockIdx.x; plane < nplanes; plane += gridDim.x) {
        for (int s = 0; s < nst; ++s) {
          if (round > 0) mbar_wait(&empty[bi], (round - 1) & 1, p.status, 1);
          mbar_expect_tx(&full[bi], 2 * TILE_BYTES);
          unsigned char* kd = stage0 + bi * 2 * TILE_BYTES;
          unsigned char* vd = kd + TILE_BYTES;
#pragma unroll
          for (int hf = 0; hf < DH / 64; ++hf) {
            tma_load_3d(kd + hf * (DA_TILE * 128), &kmap, &full[bi], hf * 64, s * DA_TILE, plane);
            tma_load_3d(vd + hf * (DA_TILE * 128), &vmap, &full[bi], hf * 64, s * DA_TILE, plane);
          }
          if (++bi == S) { bi = 0; ++round; }
        }
      }
    }
    return;
  }

  if (warp >= DA_CWARPS) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 104;");
    // ---------------- auxiliary warps: queries of the next plane, merge + epilogue of the previous ----------------
    auto stage = [&](int buf, const Inputs& in) {
      bf16* q_s = sQ + buf * 16 * QSTR;
#pragma unroll
      for (int it = 0; it < ITEMS; ++it) {
        const int w = at + it * AT;
        if (w < G * HALF) {
          const int g = w / HALF, i = w % HALF;
          const float a0 = __uint_as_float(in.q0[it] << 16), a1 = __uint_as_float(in.q0[it] & 0xffff0000u);
          const float b0 = __uint_as_float(in.q1[it] << 16), b1 = __uint_as_float(in.q1[it] & 0xffff0000u);
          float e0, e1;                                    // RoPE'd elements 2i, 2i+1 (primitives.py:99-113)
          if (p.interleaved) {
            const float c = sCS[i], s = sCS[HALF + i];
            e0 = t_sub<bf16>(t_mul<bf16>(a0, c), t_mul<bf16>(a1, s));
            e1 = t_add<bf16>(t_mul<bf16>(a0, s), t_mul<bf16>(a1, c));
          } else {
            const bool lo = 2 * i < HALF;
            const int pi = lo ? 2 * i : 2 * i - HALF;
            const float c0 = sCS[pi], s0 = sCS[HALF + pi], c1 = sCS[pi + 1], s1 = sCS[HALF + pi + 1];
            e0 = lo ? t_add<bf16>(t_mul<bf16>(a0, c0), t_mul<bf16>(-b0, s0)) : t_add<bf16>(t_mul<bf16>(b0, c0), t_mul<bf16>(a0, s0));
            e1 = lo ? t_add<bf16>(t_mul<bf16>(a1, c1), t_mul<bf16>(-b1, s1)) : t_add<bf16>(t_mul<bf16>(b1, c1), t_mul<bf16>(a1, s1));
          }
          const float ct = __bfloat162float(in.ct[it]), st = __bfloat162float(in.st[it]);
          const float n0 = t_sub<bf16>(t_mul<bf16>(e0, ct), t_mul<bf16>(e1, st));
          const float n1 = t_add<bf16>(t_mul<bf16>(e0, st), t_mul<bf16>(e1, ct));
          *reinterpret_cast<uint32_t*>(q_s + g * QSTR + 2 * i) = pack_bf16(e0, e1);
          *reinterpret_cast<uint32_t*>(q_s + (G + g) * QSTR + 2 * i) = pack_bf16(n0, n1);
        }
      }
      if (at < G) sLam[buf * 8 + at] = t_sigmoid<bf16>(in.lam);
      uint8_t* al_s = sAl + buf * al_stride;
#pragma unroll
      for (int a = 0; a < ALW; ++a) {
        const int i0 = (at + a * AT) * 4;
        if (i0 < al_stride) *reinterpret_cast<uint32_t*>(al_s + i0) = in.al[a];
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&q_ready[buf]);
    };

    {
      // RoPE cos/sin of the query position (ring position + device step counter): the same for every plane
      const long long qpos = p.rp.pos + steps_pre - p.pos_minus_one;
      if (at < HALF) {
        float ta = (float)qpos, inv = inv_pre;
        if (p.angle_bf16) { ta = bf16_round(ta); inv = bf16_round(inv); }
        float ang = __fmul_rn(ta, inv);
        if (p.angle_bf16) ang = bf16_round(ang);
        float c = cosf(ang), s = sinf(ang);
        if (p.angle_bf16) { c = bf16_round(c); s = bf16_round(s); }
        sCS[at] = bf16_round(c);
        sCS[HALF + at] = bf16_round(s);
      }
      for (int i = at; i < 2 * 16 * QSTR; i += AT) sQ[i] = __float2bfloat16_rn(0.f);   // rows >= 2G stay zero
      bar_aux();
    }
    const int gstep = (int)gridDim.x;
    if ((int)blockIdx.x < nplanes) stage(0, inA);
    if ((int)blockIdx.x + 2 * gstep < nplanes) fetch(blockIdx.x + 2 * gstep, inA);

    // One plane of this CTA (its i-th); `nxt` is the input set of the following one.
    auto aux_plane = [&](int i, int plane, Inputs& nxt) {
      // queries of the next plane (requested two planes ago) first, then the request for the plane that will
      // use the same set: both are off the consumers' critical path, which is inside the current plane's tiles
      if (plane + gstep < nplanes) stage((i + 1) & 1, nxt);
      if (plane + 3 * gstep < nplanes) fetch(plane + 3 * gstep, nxt);
      // ---- merge of the eight partial softmaxes; one warp per query head: sig - lam*noise, RMSNorm, store ----
      mbar_wait(comb_full, i & 1, p.status, 5);
      const int b = plane / p.Hkv, hk = plane % p.Hkv;
      for (int g = aw; g < G; g += DA_AWARPS) {
        // lanes 0-7: partial w = lane of the signal row g; lanes 8-15: of the noise row G + g (16-31 mirror them)
        const int mrow = ((lane >> 3) & 1) * G + g, mw = lane & 7;
        const float m_w = sML[mw * 16 + mrow], l_w = sML[DA_CWARPS * 16 + mw * 16 + mrow];
        float M = m_w;
#pragma unroll
        for (int o = 1; o < 8; o <<= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
        const float f_w = (m_w == -INFINITY) ? 0.f : exp2f(m_w - M);
        float Lsum = f_w * l_w;
#pragma unroll
        for (int o = 1; o < 8; o <<= 1) Lsum += __shfl_xor_sync(0xffffffffu, Lsum, o);
        const float inv_w = Lsum > 0.f ? 1.f / Lsum : 0.f;
        float v[2][DV];                                    // [stream][dims 4*lane .. 4*lane+3 (+128 ...)]
#pragma unroll
        for (int st = 0; st < 2; ++st) {
          const int row = st * G + g;
          const int sw = ((row >> 1) & 3) << 3;            // column swizzle of the partials (see the consumer)
          const float inv = __shfl_sync(0xffffffffu, inv_w, st * 8);
          float acc[DV];
#pragma unroll
          for (int k = 0; k < DV; ++k) acc[k] = 0.f;
#pragma unroll
          for (int w = 0; w < DA_CWARPS; ++w) {
            const float f = __shfl_sync(0xffffffffu, f_w, st * 8 + w);
            const float4 c4 = *reinterpret_cast<const float4*>(comb + (w * RL + row) * DH + (dact ? ((4 * lane) ^ sw) : 0));
            acc[0] += f * c4.x; acc[1] += f * c4.y; acc[2] += f * c4.z; acc[3] += f * c4.w;
          }
#pragma unroll
          for (int k = 0; k < DV; ++k) v[st][k] = bf16_round(acc[k] * inv);
        }
        const float lam = sLam[(i & 1) * 8 + g];
        float diff[DV], sq = 0.f;
#pragma unroll
        for (int k = 0; k < DV; ++k) {
          diff[k] = t_sub<bf16>(v[0][k], t_mul<bf16>(lam, v[1][k]));
          if (dact) sq += bf16_round(diff[k] * diff[k]);
        }
        bf16* op = p.out + (long long)b * p.out_bs + (long long)(hk * G + g) * DH;
        if (p.norm_full) {
          const float var = bf16_round(warp_sum(sq) / (float)DH);
          const float rs = bf16_round(rsqrtf(bf16_round(var + p.eps)));
#pragma unroll
          for (int k = 0; k < DV; ++k) diff[k] = t_mul<bf16>(t_mul<bf16>(diff[k], rs), nw[k]);
        }
        if (dact) {
          uint2 o2;
          o2.x = pack_bf16(diff[0], diff[1]); o2.y = pack_bf16(diff[2], diff[3]);
          *reinterpret_cast<uint2*>(op + 4 * lane) = o2;
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(comb_free);
    };
    for (int i = 0, plane = blockIdx.x; plane < nplanes; i += 2, plane += 2 * gstep) {
      aux_plane(i, plane, inB);
      if (plane + gstep < nplanes) aux_plane(i + 1, plane + gstep, inA);
    }
    return;
  }

  // ---------------- consumers: two groups of four warps, each taking every other tile ----------------
  // Tensor-core tiles are laid out with the SLOTS as the m dimension and the queries as n = 8:
  //   S^T[16 slots x 8 q] = K[16 x Dh] . Q^T,   O^T[Dh x 8 q] += V^T[16 dh x 16 slots] . P^T
  // so that the 2G <= 8 live query rows fill an n-tile exactly (NQ = 2 n-tiles for 8 < 2G <= 16); with the
  // queries as m = 16 half of every tile would be padding, and the legacy tensor path is what bounds a tile.
  asm volatile("setmaxnreg.inc.sync.aligned.u32 152;");
  const int grp = warp >> 2, gw = warp & 3;            // group, warp inside the group (owns slots gw*16..+15 of a tile)
  const int li = lane >> 3, lr = lane & 7;
  const int qa = 2 * (lane & 3);                        // this thread's query columns: nq*8 + qa + {0, 1}
  int i = 0;
  for (int plane = blockIdx.x; plane < nplanes; plane += gridDim.x, ++i) {
    const int buf = i & 1;
    mbar_wait(&q_ready[buf], (i >> 1) & 1, p.status, 3);
    const uint8_t* al_s = sAl + buf * al_stride;
    // B fragments of Q^T: one ldmatrix.x4 covers two k-steps of one n-tile (matrices: dh chunks 4j .. 4j+3)
    uint32_t qf[NQ][KSTEPS / 2][4];
#pragma unroll
    for (int nq = 0; nq < NQ; ++nq) {
      const uint32_t qbase = smem_u32(sQ + buf * 16 * QSTR) + (uint32_t)(((nq * 8 + lr) * QSTR + li * 8) * 2);
#pragma unroll
      for (int j = 0; j < KSTEPS / 2; ++j) ldsm_x4(qf[nq][j], qbase + j * 64);
    }
    float oacc[NQ][MT_O][4];
#pragma unroll
    for (int nq = 0; nq < NQ; ++nq)
#pragma unroll
      for (int j = 0; j < MT_O; ++j) { oacc[nq][j][0] = oacc[nq][j][1] = oacc[nq][j][2] = oacc[nq][j][3] = 0.f; }
    float mrun[NQ][2], lrun[NQ][2];                       // running max / (per-thread partial) sum of columns qa, qa+1
#pragma unroll
    for (int nq = 0; nq < NQ; ++nq) { mrun[nq][0] = mrun[nq][1] = -INFINITY; lrun[nq][0] = lrun[nq][1] = 0.f; }
    // tile s of this CTA's i-th plane is the (i * nst + s)-th tile through the ring
    int bi = (i * nst + grp) % S, round = (i * nst + grp) / S;

    for (int s = grp; s < nst; s += 2) {
      mbar_wait(&full[bi], round & 1, p.status, 2);
      const uint32_t kb = smem_u32(stage0 + bi * 2 * TILE_BYTES);
      const uint32_t vb = kb + TILE_BYTES;
      // ---- S^T = K Q^T over this warp's 16 slots (two accumulation chains per n-tile) ----
      float sc[NQ][4], sd[NQ][4];
#pragma unroll
      for (int nq = 0; nq < NQ; ++nq) { sc[nq][0] = sc[nq][1] = sc[nq][2] = sc[nq][3] = 0.f; sd[nq][0] = sd[nq][1] = sd[nq][2] = sd[nq][3] = 0.f; }
      const int krow = gw * 16 + (li & 1) * 8 + lr;
#pragma unroll
      for (int kk = 0; kk < KSTEPS; kk += 2) {
        uint32_t kf[4], kg[4];
        ldsm_x4(kf, kb + tile_off<DH>(krow, kk * 2 + (li >> 1)));
        ldsm_x4(kg, kb + tile_off<DH>(krow, (kk + 1) * 2 + (li >> 1)));
#pragma unroll
        for (int nq = 0; nq < NQ; ++nq) {
          mma_bf16(sc[nq], kf, qf[nq][kk / 2][0], qf[nq][kk / 2][1]);
          mma_bf16(sd[nq], kg, qf[nq][kk / 2][2], qf[nq][kk / 2][3]);
        }
      }
      // ---- mask + online softmax; this thread: slots r0 = lane/4 and r0 + 8, columns qa, qa + 1 ----
      const int slot0 = s * DA_TILE + gw * 16 + (lane >> 2);
      const bool vis0 = slot0 < p.Lbuf && (!p.mask_unused || al_s[slot0] != 0);
      const bool vis1 = slot0 + 8 < p.Lbuf && (!p.mask_unused || al_s[slot0 + 8] != 0);
      uint32_t pb[NQ][2];                                  // B fragments of P^T
#pragma unroll
      for (int nq = 0; nq < NQ; ++nq) {
        float x[4];
        x[0] = vis0 ? (sc[nq][0] + sd[nq][0]) * p.scale_log2 : -INFINITY;
        x[1] = vis0 ? (sc[nq][1] + sd[nq][1]) * p.scale_log2 : -INFINITY;
        x[2] = vis1 ? (sc[nq][2] + sd[nq][2]) * p.scale_log2 : -INFINITY;
        x[3] = vis1 ? (sc[nq][3] + sd[nq][3]) * p.scale_log2 : -INFINITY;
        float mx0 = fmaxf(x[0], x[2]), mx1 = fmaxf(x[1], x[3]);
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) {
          mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, o));
          mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, o));
        }
        const float nm0 = fmaxf(mrun[nq][0], mx0), nm1 = fmaxf(mrun[nq][1], mx1);
        const float ref0 = nm0 == -INFINITY ? 0.f : nm0, ref1 = nm1 == -INFINITY ? 0.f : nm1;
        const float a0 = exp2f(mrun[nq][0] - ref0), a1 = exp2f(mrun[nq][1] - ref1);
        mrun[nq][0] = nm0; mrun[nq][1] = nm1;
        const float p0 = exp2f(x[0] - ref0), p1 = exp2f(x[1] - ref1), p2 = exp2f(x[2] - ref0), p3 = exp2f(x[3] - ref1);
        lrun[nq][0] = lrun[nq][0] * a0 + (p0 + p2);
        lrun[nq][1] = lrun[nq][1] * a1 + (p1 + p3);
        // [slot][q] fragments -> [q][slot] (the B operand of P^T): 8x8 transposes across the warp
        pb[nq][0] = movmatrix_t(pack_bf16(p0, p1));
        pb[nq][1] = movmatrix_t(pack_bf16(p2, p3));
        if (a0 != 1.f || a1 != 1.f) {
#pragma unroll
          for (int j = 0; j < MT_O; ++j) { oacc[nq][j][0] *= a0; oacc[nq][j][1] *= a1; oacc[nq][j][2] *= a0; oacc[nq][j][3] *= a1; }
        }
      }
      // ---- O^T += V^T P^T ----
      const int vrow = gw * 16 + (li >> 1) * 8 + lr;
#pragma unroll
      for (int j = 0; j < MT_O; ++j) {
        uint32_t vf[4];
        ldsm_x4_t(vf, vb + tile_off<DH>(vrow, 2 * j + (li & 1)));
#pragma unroll
        for (int nq = 0; nq < NQ; ++nq) mma_bf16(oacc[nq][j], vf, pb[nq][0], pb[nq][1]);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[bi]);
      bi += 2;
      if (bi >= S) { bi -= S; ++round; }
    }

    // ---- hand the partial softmax of this warp to the auxiliary warps ----
#pragma unroll
    for (int nq = 0; nq < NQ; ++nq)
#pragma unroll
      for (int o = 4; o < 32; o <<= 1) {
        lrun[nq][0] += __shfl_xor_sync(0xffffffffu, lrun[nq][0], o);
        lrun[nq][1] += __shfl_xor_sync(0xffffffffu, lrun[nq][1], o);
      }
    if (i >= 1) mbar_wait(comb_free, (i - 1) & 1, p.status, 4);
    if (lane < 4) {
#pragma unroll
      for (int nq = 0; nq < NQ; ++nq)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int q = nq * 8 + qa + e;
          sML[warp * 16 + q] = mrun[nq][e];
          sML[DA_CWARPS * 16 + warp * 16 + q] = lrun[nq][e];
        }
    }
    {
      // comb[warp][q][dh]; the dh index is XOR-swizzled with (q / 2) % 4 = lane % 4, so that the four query
      // pairs a warp stores at once fall into different banks.  Only the 2G live rows are exchanged.
      const int sw = (lane & 3) << 3;
#pragma unroll
      for (int nq = 0; nq < NQ; ++nq)
#pragma unroll
        for (int j = 0; j < MT_O; ++j) {
          const int d0 = (j * 16 + (lane >> 2)) ^ sw, d1 = (j * 16 + 8 + (lane >> 2)) ^ sw;
          const int q = nq * 8 + qa;
          if (q < RL) {
            comb[(warp * RL + q) * DH + d0] = oacc[nq][j][0];
            comb[(warp * RL + q) * DH + d1] = oacc[nq][j][2];
          }
          if (q + 1 < RL) {
            comb[(warp * RL + q + 1) * DH + d0] = oacc[nq][j][1];
            comb[(warp * RL + q + 1) * DH + d1] = oacc[nq][j][3];
          }
        }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(comb_full);
  }  // plane loop
}

template <int DH, int NQ>
int launch_decode(const CUtensorMap& km, const CUtensorMap& vm, DecodeParams p, cudaStream_t s) {
  constexpr int BUDGET = 226 * 1024;
  const int nst = (p.Lbuf + DA_TILE - 1) / DA_TILE;
  // as many ring stages as fit beside the fixed buffers (at least 2, at most DA_MAX_STAGES)
  const int fixed = DecodeSmem<DH>(0, p.G, nst).total + 1024;
  int stages = (BUDGET - fixed) / (2 * DecodeSmem<DH>::TILE_BYTES);
  if (stages > DA_MAX_STAGES) stages = DA_MAX_STAGES;
  CODA_REQUIRE(stages >= 2, CODA_ERR_LIMIT, "decode_attend: %d slots leave no room for the tile ring in shared memory", p.Lbuf);
  p.stages = stages;
  const size_t smem = (size_t)DecodeSmem<DH>(stages, p.G, nst).total + 1024;
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(decode_attend_kernel<DH, NQ>, cudaFuncAttributeMaxDynamicSharedMemorySize, BUDGET);
    configured = true;
  }
  static int num_sms = 0;
  if (num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || num_sms <= 0) num_sms = 148;
  }
  const int nplanes = p.B * p.Hkv;
  decode_attend_kernel<DH, NQ><<<nplanes < num_sms ? nplanes : num_sms, DA_THREADS, smem, s>>>(km, vm, p);
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
  if (p.G <= 4) return cfg->Dh == 128 ? launch_decode<128, 1>(km, vm, p, s) : launch_decode<64, 1>(km, vm, p, s);
  return cfg->Dh == 128 ? launch_decode<128, 2>(km, vm, p, s) : launch_decode<64, 2>(km, vm, p, s);
}
