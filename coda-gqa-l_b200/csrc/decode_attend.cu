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
#include "decode_record.h"

extern "C" int coda_b200_decode_attend_supported(const coda_layer_cfg* cfg);

// Whether the decode attention kernels let the kernel after them be brought onto the SMs as these become free
// (griddepcontrol.launch_dependents right after their own dependency wait).  On by default; a benchmark that times a
// train of these launches switches it off so that consecutive launches do not overlap.
static int g_early_trigger = 1;
extern "C" void coda_b200_decode_set_early_trigger(int32_t on) { g_early_trigger = on ? 1 : 0; }

namespace {

constexpr int DA_TILE = 64;          // slots per stage
constexpr int DA_MAX_STAGES = 8;
constexpr int DA_CWARPS = 8;         // consumer warps (two groups of four)
constexpr int DA_AWARPS = 4;         // auxiliary warps (query preparation, merge + epilogue)
constexpr int DA_THREADS = (DA_CWARPS + DA_AWARPS + 1) * 32;   // 8 consumer, 4 auxiliary, 1 producer warp

struct DecodeParams {
  int B, H, Hkv, G, Lbuf, mask_unused, norm_full, interleaved, angle_bf16, stages;
  float eps, scale_log2;
  coda_ring_pos rp; int W;                        // (preparation kernel only)
  unsigned char* qrec;                            // decode records, one per (state, KV head) plane
  const uint8_t* allowed;                         // (preparation kernel only)
  const bf16* norm_w;
  bf16* out; long long out_bs;
  int* status;
  // APPEND variant only: the new token (raw projections of this step) and the state buffers it is written to
  const bf16* k_raw; long long k_bs; const bf16* v_new; long long v_bs;
  const bf16* gate_logit; long long gate_bs; int gated;
  const float* inv_freq;
  const bf16* q_raw; long long q_bs; const bf16* lam_logit; long long lam_bs;
  const bf16* cos_t; const bf16* sin_t;
  const float* rope_cs;                           // optional: cos [Dh/2] | sin [Dh/2] of the token's position, precomputed
  bf16* k_buf; bf16* v_buf; uint8_t* allowed_w; float* g_recent;
  int early_trigger;
  unsigned int hkv_magic;                         // ceil(2^32 / Hkv): plane -> (state, KV head) without a division
};

// plane = b * Hkv + hk for plane < 2^20 and Hkv < 2^8 (then the rounded-up reciprocal is exact)
__device__ __forceinline__ void plane_split(const DecodeParams& p, int plane, int& b, int& hk) {
  b = p.Hkv == 1 ? plane : (int)__umulhi((unsigned int)plane, p.hkv_magic);
  hk = plane - b * p.Hkv;
}

using tma::smem_u32; using tma::mbar_init; using tma::mbar_expect_tx; using tma::mbar_arrive; using tma::mbar_try;
__device__ __forceinline__ void mbar_wait(uint64_t* bar, uint32_t parity, int* status, int code, int* abort) { tma::mbar_wait(bar, parity, status, code, abort); }
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
  int comb, rec, rec_stride, sml, nkv, cs, bars, total;
  __host__ __device__ DecodeSmem(int stages, int G, int Lbuf) {
    int o = stages * 2 * TILE_BYTES;
    comb = o; o += DA_CWARPS * 2 * G * DH * 4;      // [DA_CWARPS][2G][DH] partial outputs
    rec_stride = (DecodeRecord::bytes(G, DH, Lbuf) + 127) / 128 * 128;
    rec = o;  o += 2 * rec_stride;                  // [2] decode records (double-buffered)
    sml = o;  o += 2 * DA_CWARPS * 16 * 4;          // [2][DA_CWARPS][16]  (m, l)
    nkv = o;  o += 2 * 4 * DH;                      // [2][K row | V row] of the new token (APPEND variant)
    cs = o;   o += 4 * DH + 16 + 2 * DH;            // cos | sin of the position (floats), the ring slot (int), cos | sin again as bf16
    bars = o; o += (2 * DA_MAX_STAGES + 8) * 8;     // full[], empty[], q_ready[2], q_free[2], comb_full, comb_free, row_ready[2]
    total = o;
  }
};

// Decode record of one plane from the raw query projection (used when the cache write has not prepared it).
template <int DH>
__global__ void __launch_bounds__(128) decode_prep_kernel(DecodeParams p, const bf16* q, long long q_bs, const bf16* lam_logit,
                                                          long long lam_bs, const float* inv_freq, const bf16* cos_t,
                                                          const bf16* sin_t, int pos_minus_one) {
  constexpr int HALF = DH / 2, QSTR = DH + 8;
  __shared__ float sCS[DH];
  const int plane = blockIdx.x, b = plane / p.Hkv, hk = plane % p.Hkv, tid = threadIdx.x, G = p.G;
  unsigned char* rec = p.qrec + (long long)plane * DecodeRecord::bytes(G, DH, p.Lbuf);
  bf16* q_s = reinterpret_cast<bf16*>(rec);
  const long long qpos = ring_now(p.rp, p.W).pos - pos_minus_one;
  for (int i = tid; i < HALF; i += blockDim.x) {
    float ta = (float)qpos, inv = inv_freq[i];
    if (p.angle_bf16) { ta = bf16_round(ta); inv = bf16_round(inv); }
    float ang = __fmul_rn(ta, inv);
    if (p.angle_bf16) ang = bf16_round(ang);
    float c, s; sincos_call(ang, &s, &c);
    if (p.angle_bf16) { c = bf16_round(c); s = bf16_round(s); }
    sCS[i] = bf16_round(c);
    sCS[HALF + i] = bf16_round(s);
  }
  __syncthreads();
  const bf16* qrow = q + (long long)b * q_bs + (long long)hk * G * DH;
  const int rows = DecodeRecord::qrows(G);
  // item (g, i): RoPE'd elements 2i, 2i+1 of head g (primitives.py:99-113) and their rotation by theta
  for (int w = tid; w < rows * HALF; w += blockDim.x) {
    const int g = w / HALF, i = w % HALF;
    if (g >= G) {
      if (g >= 2 * G) *reinterpret_cast<uint32_t*>(q_s + g * QSTR + 2 * i) = 0u;
      continue;
    }
    const bf16* qh = qrow + g * DH;
    float e0, e1;
    if (p.interleaved) {
      const float a0 = __bfloat162float(qh[2 * i]), a1 = __bfloat162float(qh[2 * i + 1]);
      const float c = sCS[i], s = sCS[HALF + i];
      e0 = t_sub<bf16>(t_mul<bf16>(a0, c), t_mul<bf16>(a1, s));
      e1 = t_add<bf16>(t_mul<bf16>(a0, s), t_mul<bf16>(a1, c));
    } else {
      const bool lo = 2 * i < HALF;
      const int pi = lo ? 2 * i : 2 * i - HALF;
      const float a0 = __bfloat162float(qh[pi]), a1 = __bfloat162float(qh[pi + 1]);
      const float b0 = __bfloat162float(qh[pi + HALF]), b1 = __bfloat162float(qh[pi + HALF + 1]);
      const float c0 = sCS[pi], s0 = sCS[HALF + pi], c1 = sCS[pi + 1], s1 = sCS[HALF + pi + 1];
      e0 = lo ? t_add<bf16>(t_mul<bf16>(a0, c0), t_mul<bf16>(-b0, s0)) : t_add<bf16>(t_mul<bf16>(b0, c0), t_mul<bf16>(a0, s0));
      e1 = lo ? t_add<bf16>(t_mul<bf16>(a1, c1), t_mul<bf16>(-b1, s1)) : t_add<bf16>(t_mul<bf16>(b1, c1), t_mul<bf16>(a1, s1));
    }
    const float ct = __bfloat162float(cos_t[(hk * G + g) * HALF + i]), st = __bfloat162float(sin_t[(hk * G + g) * HALF + i]);
    const float n0 = t_sub<bf16>(t_mul<bf16>(e0, ct), t_mul<bf16>(e1, st));
    const float n1 = t_add<bf16>(t_mul<bf16>(e0, st), t_mul<bf16>(e1, ct));
    *reinterpret_cast<uint32_t*>(q_s + g * QSTR + 2 * i) = pack_bf16(e0, e1);
    *reinterpret_cast<uint32_t*>(q_s + (G + g) * QSTR + 2 * i) = pack_bf16(n0, n1);
  }
  float* lam = reinterpret_cast<float*>(rec + DecodeRecord::lam_off(G, DH));
  if (tid < 8) lam[tid] = tid < G ? t_sigmoid<bf16>(__bfloat162float(lam_logit[(long long)b * lam_bs + hk * G + tid])) : 0.f;
  uint8_t* mk = rec + DecodeRecord::mask_off(G, DH);
  const uint8_t* alb = p.allowed + (long long)b * p.Lbuf;
  for (int i = tid; i < DecodeRecord::mask_bytes(p.Lbuf); i += blockDim.x) mk[i] = i < p.Lbuf ? alb[i] : 0;
}

// APPEND: the kernel also writes the step's new token (what step_append_kernel does): the auxiliary warps build
// each plane's decode record in shared memory themselves instead of receiving it by bulk copy, write the token's
// RoPE'd key / value row to the ring slot in global memory, and leave a copy in shared memory with which the
// consumer warp that owns the slot overwrites that row of the staged tile (the tile was requested from HBM
// before the row was written).
template <int DH, int NQ, bool APPEND>
__global__ void __launch_bounds__(DA_THREADS, 1)
decode_attend_kernel(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap, DecodeParams p) {
  constexpr int KSTEPS = DH / 16;            // k-steps of Q.K^T
  constexpr int MT_O = DH / 16;              // m-tiles of the (transposed) output
  constexpr int TILE_BYTES = DA_TILE * DH * 2;
  constexpr int QSTR = DH + 8;

  extern __shared__ unsigned char smem_raw[];
  // the swizzled TMA tiles need a 1024-byte aligned base; the launch reserves the slack
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int G = p.G, RL = 2 * G, S = p.stages;
  const int nst = (p.Lbuf + DA_TILE - 1) / DA_TILE;
  const int nplanes = p.B * p.Hkv;
  const DecodeSmem<DH> L(S, G, p.Lbuf);
  const int rec_bytes = DecodeRecord::bytes(G, DH, p.Lbuf);
  const int lam_off = DecodeRecord::lam_off(G, DH), mask_off = DecodeRecord::mask_off(G, DH);
  unsigned char* stage0 = smem;
  float* comb = reinterpret_cast<float*>(smem + L.comb);
  unsigned char* rec0 = smem + L.rec;
  float* sML = reinterpret_cast<float*>(smem + L.sml);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L.bars);
  uint64_t* empty = full + DA_MAX_STAGES;
  uint64_t* q_ready = empty + DA_MAX_STAGES;       // [2] record of the plane has landed
  uint64_t* q_free = q_ready + 2;                  // [2] record buffer may be overwritten
  uint64_t* comb_full = q_free + 2;
  uint64_t* comb_free = comb_full + 1;
  uint64_t* row_ready = comb_free + 1;             // [2] APPEND: the new token's row of the plane is in shared memory

  __shared__ int s_abort;                          // set by the first bounded wait of this CTA that expires
  int* const abortw = &s_abort;
  if (tid == 0) {
    s_abort = 0;
    for (int i = 0; i < S; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], 4); }
    mbar_init(&q_ready[0], APPEND ? DA_AWARPS : 1); mbar_init(&q_ready[1], APPEND ? DA_AWARPS : 1);
    mbar_init(&q_free[0], DA_CWARPS + DA_AWARPS); mbar_init(&q_free[1], DA_CWARPS + DA_AWARPS);
    mbar_init(comb_full, DA_CWARPS); mbar_init(comb_free, DA_AWARPS);
    mbar_init(&row_ready[0], DA_AWARPS); mbar_init(&row_ready[1], DA_AWARPS);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (APPEND && warp >= DA_CWARPS && warp < DA_CWARPS + DA_AWARPS) {
    // rows of the two query tiles that no head uses stay zero for the whole launch (the records are built in place)
    const int rows = DecodeRecord::qrows(G), at0 = tid - DA_CWARPS * 32;
    for (int buf = 0; buf < 2; ++buf) {
      bf16* q_s = reinterpret_cast<bf16*>(rec0 + buf * L.rec_stride);
      for (int w = at0; w < (rows - 2 * G) * (DH / 2); w += DA_AWARPS * 32)
        *reinterpret_cast<uint32_t*>(q_s + (2 * G + w / (DH / 2)) * QSTR + 2 * (w % (DH / 2))) = 0u;
    }
  }
  // everything above touched no global memory: from here on the previous kernel's results are needed
  asm volatile("griddepcontrol.wait;" ::: "memory");
  // The kernel after this one may be brought onto the SMs as they become free (its own griddepcontrol.wait holds
  // it back from this kernel's results until the whole grid has finished): the CTAs with one plane fewer leave early.
  if (p.early_trigger) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  // ---- APPEND: the new token's inputs of one plane, as the auxiliary threads hold them between request and use ----
  constexpr int HALF = DH / 2;
  constexpr int QI = (8 * HALF + DA_AWARPS * 32 - 1) / (DA_AWARPS * 32);   // (head, RoPE pair) items per auxiliary thread, G <= 8
  constexpr int MB = 8;                                                     // mask bytes per auxiliary thread (Lbuf <= 1024)
  // fq0 / fq1: raw query pairs of this thread's QI CONSECUTIVE (head, RoPE pair) items (one 16- or 8-byte request
  // each); fct / fst: the matching cos / sin of the learned rotation, two bf16 per word
  // lam0 / lam1: lambda logits of the two query heads this thread's warp finishes in the epilogue (aw, aw + 4)
  struct AppIn { uint32_t fq0[QI], fq1[QI], fct[QI / 2], fst[QI / 2]; bf16 ka, kb, vv, lam0, lam1, gate; uint8_t am[MB]; };
  static_assert(QI == 2 || QI == 4, "vector widths below assume 2 or 4 items per auxiliary thread");
  auto ld_words = [](uint32_t* dst, const void* src, int n) {       // n = 1, 2 or 4 words, naturally aligned
    if (n == 4) { const uint4 t = *reinterpret_cast<const uint4*>(src); dst[0] = t.x; dst[1] = t.y; dst[2] = t.z; dst[3] = t.w; }
    else if (n == 2) { const uint2 t = *reinterpret_cast<const uint2*>(src); dst[0] = t.x; dst[1] = t.y; }
    else dst[0] = *reinterpret_cast<const uint32_t*>(src);
  };
  AppIn in;
  long long nsteps = 0;
  float inv_f = 0.f;
  const int at = tid - DA_CWARPS * 32;                   // index among the 128 auxiliary threads
  auto load_inputs = [&](int plane, AppIn& a) {
    int b, hk; plane_split(p, plane, b, hk);
    const bf16* qrow = p.q_raw + (long long)b * p.q_bs + (long long)hk * G * DH;
#pragma unroll
    for (int it = 0; it < QI; ++it) a.fq0[it] = a.fq1[it] = 0u;
#pragma unroll
    for (int it = 0; it < QI / 2; ++it) a.fct[it] = a.fst[it] = 0u;
    const int w0 = at * QI;                                // items w0 .. w0 + QI - 1: one head, consecutive pairs
    if (w0 < G * HALF) {
      const int g = w0 / HALF, i0 = w0 % HALF;
      const bf16* qh = qrow + g * DH;
      if (p.interleaved) {
        ld_words(a.fq0, qh + 2 * i0, QI);
      } else {
        const int pi0 = 2 * i0 < HALF ? 2 * i0 : 2 * i0 - HALF;
        ld_words(a.fq0, qh + pi0, QI);
        ld_words(a.fq1, qh + pi0 + HALF, QI);
      }
      ld_words(a.fct, p.cos_t + (hk * G + g) * HALF + i0, QI / 2);
      ld_words(a.fst, p.sin_t + (hk * G + g) * HALF + i0, QI / 2);
    }
    a.ka = a.kb = a.vv = a.lam0 = a.lam1 = a.gate = __float2bfloat16_rn(0.f);
    if (at < DH) {
      const bf16* kn = p.k_raw + (long long)b * p.k_bs + hk * DH;
      int ia, ib;
      if (p.interleaved) { ia = 2 * (at >> 1); ib = ia + 1; }
      else { ia = at < HALF ? at : at - HALF; ib = ia + HALF; }
      a.ka = kn[ia]; a.kb = kn[ib];
      a.vv = p.v_new[(long long)b * p.v_bs + hk * DH + at];
    }
    {
      const int aw_ = at >> 5;
      if (aw_ < G) a.lam0 = p.lam_logit[(long long)b * p.lam_bs + hk * G + aw_];
      if (aw_ + DA_AWARPS < G) a.lam1 = p.lam_logit[(long long)b * p.lam_bs + hk * G + aw_ + DA_AWARPS];
    }
    if (at == 0 && p.gated) a.gate = p.gate_logit[(long long)b * p.gate_bs];
#pragma unroll
    for (int k = 0; k < MB; ++k) {
      if (k * (DA_AWARPS * 32) >= p.Lbuf) break;           // (the same for every thread)
      const int m = at + k * (DA_AWARPS * 32); a.am[k] = m < p.Lbuf ? p.allowed[(long long)b * p.Lbuf + m] : (uint8_t)0;
    }
  };
  if (APPEND) {
    // requested before the block barrier below, i.e. before the producer's first tile: a small load issued behind
    // a ring's worth of tile traffic would wait for all of it
    if (warp >= DA_CWARPS && warp < DA_CWARPS + DA_AWARPS) {
      nsteps = ring_steps(p.rp);
      if (p.rope_cs != nullptr) { if (at < DH) inv_f = p.rope_cs[at]; }      // the table entry itself
      else if (at < HALF) inv_f = p.inv_freq[at];
      if ((int)blockIdx.x < nplanes) load_inputs(blockIdx.x, in);
    }
    __syncthreads();
  }

  if (warp >= DA_CWARPS + DA_AWARPS) {
    // ---------------- producer: records first, then the ring of K/V tiles, across plane boundaries ----------------
    if (lane == 0) {
      int bi = 0, round = 0, i = 0;                        // ring slot, how often the ring has wrapped, plane count
      // k-th plane of this CTA -> record buffer k % 2; the buffer was last used by plane k - 2
      auto record_free = [&](int k) { return k < 2 || mbar_try(&q_free[k & 1], ((k >> 1) - 1) & 1); };
      auto load_record = [&](int plane, int k) {
        const int buf = k & 1;
        mbar_expect_tx(&q_ready[buf], rec_bytes);
        tma::bulk_load(rec0 + buf * L.rec_stride, p.qrec + (long long)plane * rec_bytes, rec_bytes, &q_ready[buf]);
      };
      if (!APPEND && (int)blockIdx.x < nplanes) load_record(blockIdx.x, 0);
      for (int plane = blockIdx.x; plane < nplanes; plane += gridDim.x, ++i) {
        // The next plane's record is requested as soon as its buffer is free -- normally before this plane's
        // first tile, so that it never stands behind a ring's worth of tile traffic -- without holding up the tiles.
        // (APPEND: the auxiliary warps build the records, nothing to request.)
        bool pending = !APPEND && plane + (int)gridDim.x < nplanes;
        for (int s = 0; s < nst; ++s) {
          if (pending && record_free(i + 1)) { load_record(plane + gridDim.x, i + 1); pending = false; }
          if (round > 0) mbar_wait(&empty[bi], (round - 1) & 1, p.status, 1, abortw);
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
        if (pending) {
          mbar_wait(&q_free[(i + 1) & 1], (((i + 1) >> 1) - 1) & 1, p.status, 6, abortw);
          load_record(plane + gridDim.x, i + 1);
        }
      }
    }
    return;
  }

  if (warp >= DA_CWARPS) {
    // ---------------- auxiliary warps: merge of the eight partial softmaxes + epilogue, one warp per query head ----------------
    const int aw = warp - DA_CWARPS;
    constexpr int DV = 4;                                  // output dims per lane: 4*lane .. 4*lane+3
    const bool dact = 4 * lane < DH;                       // (head_dim 64: the upper half-warp idles)
    float nw[DV];
#pragma unroll
    for (int k = 0; k < DV; ++k) nw[k] = (p.norm_full && dact) ? __bfloat162float(p.norm_w[4 * lane + k]) : 1.f;
    // ---- APPEND: record + new token row of a plane, from the inputs requested earlier ----
    float* sCS = reinterpret_cast<float*>(smem + L.cs);    // cos [HALF] | sin [HALF] of the token's position
    int* s_ev = reinterpret_cast<int*>(smem + L.cs + 4 * DH);
    bf16* sCSb = reinterpret_cast<bf16*>(smem + L.cs + 4 * DH + 16);       // the same table as bf16 (its entries are bf16 values)
    int ev = 0; bool ring_full = false;
    float lam_next[2] = {0.f, 0.f}, lam_cur[2] = {0.f, 0.f};     // APPEND: sigma(lambda) of heads aw, aw + 4: plane being built / plane in its epilogue
    auto build_record = [&](int plane, int buf, const AppIn& a) {
      using T = bf16;
      int b, hk; plane_split(p, plane, b, hk);
      unsigned char* rec = rec0 + buf * L.rec_stride;
      bf16* q_s = reinterpret_cast<bf16*>(rec);
      const int w0 = at * QI;
      if (w0 < G * HALF) {
        const int g = w0 / HALF, i0 = w0 % HALF;
        // Packed bf16 arithmetic (one instruction per element pair, each result the bf16 rounding of the exact
        // product or sum, as the reference's op-by-op bf16 arithmetic gives it): this chain stands between the
        // token's inputs and the consumers' first tile.
        const uint32_t* cw32 = reinterpret_cast<const uint32_t*>(sCSb);         // (cos[2j], cos[2j+1])
        const uint32_t* sw32 = cw32 + HALF / 2;
        uint32_t sv[QI], nv[QI];
#pragma unroll
        for (int it = 0; it < QI; ++it) {
          const int i = i0 + it;
          uint32_t e;                                      // RoPE'd elements 2i, 2i+1 (primitives.py:99-113)
          if (p.interleaved) {                             // the pair (2i, 2i+1) turns by the position's angle i
            const uint32_t cp = cw32[i >> 1], sp = sw32[i >> 1];
            e = brot(a.fq0[it], (i & 1) ? bdup_hi(cp) : bdup_lo(cp), (i & 1) ? bdup_hi(sp) : bdup_lo(sp));
          } else {                                         // x cos + rotate_half(x) sin, two neighbouring elements at once
            const bool lo = 2 * i < HALF;
            const int pi = lo ? 2 * i : 2 * i - HALF;
            const uint32_t c2 = cw32[pi >> 1], s2 = sw32[pi >> 1];
            e = lo ? badd2(bmul2(a.fq0[it], c2), bmul2(bneg2(a.fq1[it]), s2)) : badd2(bmul2(a.fq1[it], c2), bmul2(a.fq0[it], s2));
          }
          const uint32_t cw = a.fct[it >> 1], sw = a.fst[it >> 1];
          sv[it] = e;
          nv[it] = brot(e, (it & 1) ? bdup_hi(cw) : bdup_lo(cw), (it & 1) ? bdup_hi(sw) : bdup_lo(sw));   // the learned rotation of the pair
        }
        bf16* srow = q_s + g * QSTR + 2 * i0;              // 4 * i0 bytes into a 272-byte row: aligned to QI words
        bf16* nrow = q_s + (G + g) * QSTR + 2 * i0;
        if (QI == 4) {
          *reinterpret_cast<uint4*>(srow) = make_uint4(sv[0], sv[1], sv[2], sv[3]);
          *reinterpret_cast<uint4*>(nrow) = make_uint4(nv[0], nv[1], nv[2], nv[3]);
        } else {
          *reinterpret_cast<uint2*>(srow) = make_uint2(sv[0], sv[1]);
          *reinterpret_cast<uint2*>(nrow) = make_uint2(nv[0], nv[1]);
        }
      }
      uint8_t* mk = rec + mask_off;
#pragma unroll
      for (int k = 0; k < MB; ++k) {
        if (k * (DA_AWARPS * 32) >= DecodeRecord::mask_bytes(p.Lbuf)) break;   // (the same for every thread)
        const int m = at + k * (DA_AWARPS * 32);
        if (m < DecodeRecord::mask_bytes(p.Lbuf)) mk[m] = m < p.Lbuf ? (m == ev ? (uint8_t)1 : a.am[k]) : (uint8_t)0;
      }
      // queries and mask are what the consumers wait for: everything else of the plane follows behind the barrier
      __syncwarp();
      if (lane == 0) mbar_arrive(&q_ready[buf]);
      // the token's own row: ring slot in global memory, and a copy for the consumer warp that patches the tile
      if (at < DH) {
        const int d = at;
        const float ka = __bfloat162float(a.ka), kb = __bfloat162float(a.kb);
        const int ri = p.interleaved ? (d >> 1) : (d < HALF ? d : d - HALF);
        const float cc = sCS[ri], ss = sCS[HALF + ri];
        float nk;
        if (p.interleaved) nk = (d & 1) ? t_add<T>(t_mul<T>(ka, ss), t_mul<T>(kb, cc)) : t_sub<T>(t_mul<T>(ka, cc), t_mul<T>(kb, ss));
        else nk = d < HALF ? t_add<T>(t_mul<T>(ka, cc), t_mul<T>(-kb, ss)) : t_add<T>(t_mul<T>(kb, cc), t_mul<T>(ka, ss));
        const bf16 nkb = __float2bfloat16_rn(nk);
        bf16* nkv = reinterpret_cast<bf16*>(smem + L.nkv + buf * 4 * DH);
        nkv[d] = nkb; nkv[DH + d] = a.vv;
        const long long row = ((long long)plane * p.Lbuf + ev) * DH + d;
        p.k_buf[row] = nkb; p.v_buf[row] = a.vv;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&row_ready[buf]);
      if (hk == 0 && at == 0) {
        p.g_recent[(long long)b * p.W + ev] = p.gated ? t_sigmoid<T>(__bfloat162float(a.gate)) : 1.0f;
        if (!ring_full) p.allowed_w[(long long)b * p.Lbuf + ev] = 1;
      }
      // sigma(lambda) of this warp's two heads, kept in registers for the plane's epilogue
      if (aw < G) lam_next[0] = t_sigmoid<T>(__bfloat162float(a.lam0));
      if (aw + DA_AWARPS < G) lam_next[1] = t_sigmoid<T>(__bfloat162float(a.lam1));
    };
    if (APPEND && (int)blockIdx.x < nplanes) {
      const RingNow r = ring_after(p.rp, p.W, nsteps);
      ring_full = r.filled >= p.W;
      ev = ring_full ? r.idx : r.filled;
      if (at == 0) *s_ev = ev;
      if (p.rope_cs != nullptr) {
        if (at < DH) { sCS[at] = inv_f; sCSb[at] = __float2bfloat16_rn(inv_f); }   // computed once per step for all layers (coda_b200_rope_table)
      } else if (at < HALF) {
        float ta = (float)r.pos, inv = inv_f;
        if (p.angle_bf16) { ta = bf16_round(ta); inv = bf16_round(inv); }
        float ang = __fmul_rn(ta, inv);
        if (p.angle_bf16) ang = bf16_round(ang);
        float cc, ss; sincos_call(ang, &ss, &cc);
        if (p.angle_bf16) { cc = bf16_round(cc); ss = bf16_round(ss); }
        sCS[at] = bf16_round(cc); sCS[HALF + at] = bf16_round(ss);
        sCSb[at] = __float2bfloat16_rn(cc); sCSb[HALF + at] = __float2bfloat16_rn(ss);
      }
      asm volatile("bar.sync 2, 128;" ::: "memory");       // the four auxiliary warps
      build_record(blockIdx.x, 0, in);
      if ((int)(blockIdx.x + gridDim.x) < nplanes) load_inputs(blockIdx.x + gridDim.x, in);
    }
    int i = 0;
    for (int plane = blockIdx.x; plane < nplanes; plane += gridDim.x, ++i) {
      if (APPEND) {
        lam_cur[0] = lam_next[0]; lam_cur[1] = lam_next[1];
        // the NEXT plane's record, while the consumers are on this plane's tiles (its inputs were requested a plane ago)
        const int next = plane + gridDim.x;
        if (next < nplanes) {
          if (i + 1 >= 2) mbar_wait(&q_free[(i + 1) & 1], (((i + 1) >> 1) - 1) & 1, p.status, 6, abortw);
          build_record(next, (i + 1) & 1, in);
          if (next + (int)gridDim.x < nplanes) load_inputs(next + gridDim.x, in);
        }
      }
      mbar_wait(&q_ready[i & 1], (i >> 1) & 1, p.status, 7, abortw);   // lambda comes from the plane's record (a bulk copy: observed through its own barrier)
      mbar_wait(comb_full, i & 1, p.status, 5, abortw);
      int b, hk; plane_split(p, plane, b, hk);
      const float* sLam = reinterpret_cast<const float*>(rec0 + (i & 1) * L.rec_stride + lam_off);
      const float lam_a = APPEND ? lam_cur[0] : sLam[aw];                 // heads aw and aw + 4 of the group (G <= 8)
      const float lam_b = APPEND ? lam_cur[1] : sLam[(aw + DA_AWARPS) & 7];
      __syncwarp();
      if (lane == 0) mbar_arrive(&q_free[i & 1]);          // the record buffer is no longer needed by this warp
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
        const float lam = g == aw ? lam_a : lam_b;
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
    }
    return;
  }

  // ---------------- consumers: two groups of four warps, each taking every other tile ----------------
  // Tensor-core tiles are laid out with the SLOTS as the m dimension and the queries as n = 8:
  //   S^T[16 slots x 8 q] = K[16 x Dh] . Q^T,   O^T[Dh x 8 q] += V^T[16 dh x 16 slots] . P^T
  // so that the 2G <= 8 live query rows fill an n-tile exactly (NQ = 2 n-tiles for 8 < 2G <= 16); with the
  // queries as m = 16 half of every tile would be padding, and the legacy tensor path is what bounds a tile.
  const int grp = warp >> 2, gw = warp & 3;            // group, warp inside the group (owns slots gw*16..+15 of a tile)
  const int li = lane >> 3, lr = lane & 7;
  const int qa = 2 * (lane & 3);                        // this thread's query columns: nq*8 + qa + {0, 1}
  int i = 0;
  for (int plane = blockIdx.x; plane < nplanes; plane += gridDim.x, ++i) {
    const int buf = i & 1;
    mbar_wait(&q_ready[buf], (i >> 1) & 1, p.status, 3, abortw);
    const unsigned char* rec = rec0 + buf * L.rec_stride;
    const uint8_t* al_s = rec + mask_off;
    // B fragments of Q^T: one ldmatrix.x4 covers two k-steps of one n-tile (matrices: dh chunks 4j .. 4j+3)
    uint32_t qf[NQ][KSTEPS / 2][4];
#pragma unroll
    for (int nq = 0; nq < NQ; ++nq) {
      const uint32_t qbase = smem_u32(rec) + (uint32_t)(((nq * 8 + lr) * QSTR + li * 8) * 2);
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
    // Tile s of this CTA's i-th plane is the t = (i * nst + s)-th tile through the ring (stage t % S).  A group
    // takes the tiles of ITS parity of t, and S is even, so a ring stage is only ever consumed by one group:
    // a parity wait tells "this phase or the one before" apart, nothing more, and a group that met a stage
    // whose previous use belonged to the other group could run past a phase it never observed (TMA tiles
    // need not land in issue order).
    const int s0 = (grp ^ (i * nst)) & 1;
    int bi = (i * nst + s0) % S, round = (i * nst + s0) / S;

    for (int s = s0; s < nst; s += 2) {
      mbar_wait(&full[bi], round & 1, p.status, 2, abortw);
      const uint32_t kb = smem_u32(stage0 + bi * 2 * TILE_BYTES);
      const uint32_t vb = kb + TILE_BYTES;
      if (APPEND) {
        // the tile may have left HBM before the new token's row was written: the warp that owns the ring slot
        // puts the row (left in shared memory by the auxiliary warps) over it -- only this warp reads these rows
        const int ev = *reinterpret_cast<const int*>(smem + L.cs + 4 * DH);
        if (s == ev / DA_TILE && gw == (ev % DA_TILE) / 16) {
          mbar_wait(&row_ready[buf], (i >> 1) & 1, p.status, 8, abortw);
          constexpr int CPR = DH / 8;                      // 16-byte chunks per row
          if (lane < 2 * CPR) {
            const int which = lane / CPR, c = lane % CPR;
            const uint4 v = *reinterpret_cast<const uint4*>(smem + L.nkv + buf * 4 * DH + which * 2 * DH + c * 16);
            *reinterpret_cast<uint4*>(stage0 + bi * 2 * TILE_BYTES + which * TILE_BYTES + tile_off<DH>(ev % DA_TILE, c)) = v;
          }
          __syncwarp();
        }
      }
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

    __syncwarp();
    if (lane == 0) mbar_arrive(&q_free[buf]);              // queries are in registers, the mask is no longer read
    // ---- hand the partial softmax of this warp to the auxiliary warps ----
#pragma unroll
    for (int nq = 0; nq < NQ; ++nq)
#pragma unroll
      for (int o = 4; o < 32; o <<= 1) {
        lrun[nq][0] += __shfl_xor_sync(0xffffffffu, lrun[nq][0], o);
        lrun[nq][1] += __shfl_xor_sync(0xffffffffu, lrun[nq][1], o);
      }
    if (i >= 1) mbar_wait(comb_free, (i - 1) & 1, p.status, 4, abortw);
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

template <int DH, int NQ, bool APPEND>
int launch_decode(const CUtensorMap& km, const CUtensorMap& vm, DecodeParams p, cudaStream_t s) {
  constexpr int BUDGET = 226 * 1024;
  // as many ring stages as fit beside the fixed buffers (at least 2, at most DA_MAX_STAGES)
  const int fixed = DecodeSmem<DH>(0, p.G, p.Lbuf).total + 1024;
  int stages = (BUDGET - fixed) / (2 * DecodeSmem<DH>::TILE_BYTES);
  if (stages > DA_MAX_STAGES) stages = DA_MAX_STAGES;
  stages &= ~1;                                      // even: each ring stage belongs to one consumer group (see the kernel)
  CODA_REQUIRE(stages >= 2, CODA_ERR_LIMIT, "decode_attend: %d slots leave no room for the tile ring in shared memory", p.Lbuf);
  p.stages = stages;
  const size_t smem = (size_t)DecodeSmem<DH>(stages, p.G, p.Lbuf).total + 1024;
  static coda_device_once once;
  const int num_sms = coda_on_first_use(once, [] {
    cudaFuncSetAttribute(decode_attend_kernel<DH, NQ, APPEND>, cudaFuncAttributeMaxDynamicSharedMemorySize, BUDGET);
  });
  const int nplanes = p.B * p.Hkv;
  // Programmatic dependent launch: the CTAs may start (shared-memory carve-up, barrier initialisation) while the
  // kernel before this one on the stream is still finishing; they wait for it (griddepcontrol.wait) before the
  // first global access.
  cudaLaunchConfig_t lc = {};
  lc.gridDim = dim3(nplanes < num_sms ? nplanes : num_sms, 1, 1);
  lc.blockDim = dim3(DA_THREADS, 1, 1);
  lc.dynamicSmemBytes = smem;
  lc.stream = s;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  lc.attrs = at; lc.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&lc, decode_attend_kernel<DH, NQ, APPEND>, km, vm, p);
  if (e != cudaSuccess) { coda_set_error("decode_attend: %s", cudaGetErrorString(e)); return CODA_ERR_LAUNCH; }
  return CODA_OK;
}

int check_common(const coda_layer_cfg* cfg, const coda_state_ptrs* st, const void* qrec, const void* norm_w, const void* out) {
  CODA_REQUIRE(coda_cfg_ok(cfg) && st, CODA_ERR_ARG, "decode_attend: invalid layer configuration");
  CODA_REQUIRE(coda_b200_decode_attend_supported(cfg), CODA_ERR_ARG,
               "decode_attend: needs bf16, head_dim 64 or 128 and at most 8 query heads per KV head");
  CODA_REQUIRE(qrec && out && st->k_buf && st->v_buf && st->allowed, CODA_ERR_ARG, "decode_attend: null pointer");
  CODA_REQUIRE(!cfg->head_norm_full || norm_w, CODA_ERR_ARG, "decode_attend: head-norm weight missing");
  CODA_REQUIRE(((uintptr_t)st->k_buf % 16 == 0) && ((uintptr_t)st->v_buf % 16 == 0) && ((uintptr_t)qrec % 16 == 0), CODA_ERR_ARG,
               "decode_attend: k_buf / v_buf / record buffer must be 16-byte aligned");
  // (the kernel splits a plane index into state and KV head by a reciprocal multiply, exact below this bound)
  CODA_REQUIRE((long long)cfg->B * cfg->Hkv * cfg->Hkv < (1ll << 32), CODA_ERR_LIMIT, "decode_attend: %d states x %d KV heads exceed the plane index range", cfg->B, cfg->Hkv);
  return CODA_OK;
}

DecodeParams make_params(const coda_layer_cfg* cfg, const coda_state_ptrs* st, void* qrec, const void* norm_w, void* out,
                         int64_t out_bs, int32_t* status) {
  DecodeParams p;
  p.B = cfg->B; p.H = cfg->H; p.Hkv = cfg->Hkv; p.G = cfg->H / cfg->Hkv; p.Lbuf = cfg->W + cfg->Me + cfg->Ms;
  p.hkv_magic = (unsigned int)((0x100000000ull + (unsigned long long)cfg->Hkv - 1) / (unsigned long long)cfg->Hkv);
  p.mask_unused = cfg->mask_unused; p.norm_full = cfg->head_norm_full; p.interleaved = cfg->rope_interleaved;
  p.angle_bf16 = cfg->angle_dtype == CODA_BF16; p.stages = 0; p.eps = cfg->eps;
  p.scale_log2 = 1.4426950408889634f / sqrtf((float)cfg->Dh);
  p.rp = coda_ring_pos{0, 0, 0, nullptr}; p.W = cfg->W;
  p.qrec = (unsigned char*)qrec; p.allowed = st->allowed; p.norm_w = (const bf16*)norm_w;
  p.out = (bf16*)out; p.out_bs = out_bs; p.status = status;
  p.k_raw = nullptr; p.k_bs = 0; p.v_new = nullptr; p.v_bs = 0; p.gate_logit = nullptr; p.gate_bs = 0; p.gated = 0;
  p.inv_freq = nullptr; p.q_raw = nullptr; p.q_bs = 0; p.lam_logit = nullptr; p.lam_bs = 0; p.cos_t = nullptr; p.sin_t = nullptr;
  p.rope_cs = nullptr;
  p.k_buf = nullptr; p.v_buf = nullptr; p.allowed_w = nullptr; p.g_recent = nullptr;
  p.early_trigger = g_early_trigger;
  return p;
}

int launch_main(const coda_layer_cfg* cfg, const coda_state_ptrs* st, const DecodeParams& p, cudaStream_t s, bool append = false) {
  CUtensorMap km, vm;
  CODA_REQUIRE(tmaps::plane_map(&km, st->k_buf, cfg->B * cfg->Hkv, p.Lbuf, cfg->Dh) &&
               tmaps::plane_map(&vm, st->v_buf, cfg->B * cfg->Hkv, p.Lbuf, cfg->Dh), CODA_ERR_LAUNCH,
               "decode_attend: cuTensorMapEncodeTiled failed");
  if (append) {
    if (p.G <= 4) return cfg->Dh == 128 ? launch_decode<128, 1, true>(km, vm, p, s) : launch_decode<64, 1, true>(km, vm, p, s);
    return cfg->Dh == 128 ? launch_decode<128, 2, true>(km, vm, p, s) : launch_decode<64, 2, true>(km, vm, p, s);
  }
  if (p.G <= 4) return cfg->Dh == 128 ? launch_decode<128, 1, false>(km, vm, p, s) : launch_decode<64, 1, false>(km, vm, p, s);
  return cfg->Dh == 128 ? launch_decode<128, 2, false>(km, vm, p, s) : launch_decode<64, 2, false>(km, vm, p, s);
}

}  // namespace

// True when the tuned kernel covers this configuration; otherwise callers use the generic kernels.
extern "C" int coda_b200_decode_attend_supported(const coda_layer_cfg* cfg) {
  if (!coda_cfg_ok(cfg)) return 0;
  const int G = cfg->H / cfg->Hkv;
  return cfg->dtype == CODA_BF16 && (cfg->Dh == 64 || cfg->Dh == 128) && G <= 8 &&
         (size_t)(cfg->W + cfg->Me + cfg->Ms) <= 4096 && tmaps::available();
}

// Bytes of the decode-record buffer (one record per state and KV head) for this configuration.
extern "C" int64_t coda_b200_decode_record_bytes(const coda_layer_cfg* cfg) {
  if (!coda_cfg_ok(cfg)) return 0;
  return (int64_t)cfg->B * cfg->Hkv * DecodeRecord::bytes(cfg->H / cfg->Hkv, cfg->Dh, cfg->W + cfg->Me + cfg->Ms);
}

extern "C" int coda_b200_decode_attend(const coda_layer_cfg* cfg, const coda_state_ptrs* st, coda_ring_pos rp,
                                       int32_t token_already_written,
                                       const void* q_raw, int64_t q_bs, const void* lam_logit, int64_t lam_bs,
                                       const float* inv_freq, const void* cos_theta, const void* sin_theta,
                                       const void* norm_w, void* qrec, void* out, int64_t out_bs, int32_t* status,
                                       coda_stream_t stream) {
  int rc = check_common(cfg, st, qrec, norm_w, out);
  if (rc != CODA_OK) return rc;
  CODA_REQUIRE(q_raw && lam_logit && inv_freq && cos_theta && sin_theta, CODA_ERR_ARG, "decode_attend: null pointer");
  DecodeParams p = make_params(cfg, st, qrec, norm_w, out, out_bs, status);
  p.rp = rp;
  cudaStream_t s = (cudaStream_t)stream;
  const int nplanes = cfg->B * cfg->Hkv;
  if (cfg->Dh == 128)
    decode_prep_kernel<128><<<nplanes, 128, 0, s>>>(p, (const bf16*)q_raw, q_bs, (const bf16*)lam_logit, lam_bs, inv_freq,
                                                    (const bf16*)cos_theta, (const bf16*)sin_theta, token_already_written ? 1 : 0);
  else
    decode_prep_kernel<64><<<nplanes, 128, 0, s>>>(p, (const bf16*)q_raw, q_bs, (const bf16*)lam_logit, lam_bs, inv_freq,
                                                   (const bf16*)cos_theta, (const bf16*)sin_theta, token_already_written ? 1 : 0);
  CODA_CHECK_LAUNCH("decode_prep");
  return launch_main(cfg, st, p, s);
}

extern "C" int coda_b200_decode_attend_prepared(const coda_layer_cfg* cfg, const coda_state_ptrs* st, const void* qrec,
                                                const void* norm_w, void* out, int64_t out_bs, int32_t* status,
                                                coda_stream_t stream) {
  int rc = check_common(cfg, st, qrec, norm_w, out);
  if (rc != CODA_OK) return rc;
  const DecodeParams p = make_params(cfg, st, const_cast<void*>(qrec), norm_w, out, out_bs, status);
  return launch_main(cfg, st, p, (cudaStream_t)stream);
}

// The decode attention that also writes the step's new token (the second half of a split step, in place of
// coda_b200_step_append_fused + coda_b200_decode_attend_prepared): ring slot, gate, slot flag, and the queries,
// lambda and mask the attention itself needs, built in shared memory.  Same arguments as the two calls together;
// the routing of the token the ring evicts (coda_b200_step_route / _batched with the same rp) must have run.
extern "C" int coda_b200_decode_attend_append_supported(const coda_layer_cfg* cfg) {
  return coda_b200_decode_attend_supported(cfg) && cfg->W + cfg->Me + cfg->Ms <= 1024;
}

extern "C" int coda_b200_decode_attend_append(const coda_layer_cfg* cfg, const coda_state_ptrs* st, coda_ring_pos rp,
                                              const void* k_raw, int64_t k_bs, const void* v_new, int64_t v_bs,
                                              const void* gate_logit, int64_t gate_bs, const float* inv_freq,
                                              const void* q_raw, int64_t q_bs, const void* lam_logit, int64_t lam_bs,
                                              const void* cos_theta, const void* sin_theta, const float* rope_cs,
                                              const void* norm_w,
                                              void* out, int64_t out_bs, int32_t* status, coda_stream_t stream) {
  CODA_REQUIRE(coda_cfg_ok(cfg) && st, CODA_ERR_ARG, "decode_attend_append: invalid layer configuration");
  CODA_REQUIRE(coda_b200_decode_attend_append_supported(cfg), CODA_ERR_ARG,
               "decode_attend_append: needs bf16, head_dim 64 or 128, at most 8 query heads per KV head and 1024 slots");
  CODA_REQUIRE(out && st->k_buf && st->v_buf && st->allowed && st->g_recent && k_raw && v_new && inv_freq && q_raw && lam_logit &&
               cos_theta && sin_theta && (!cfg->gated || gate_logit), CODA_ERR_ARG, "decode_attend_append: null pointer");
  CODA_REQUIRE(!cfg->head_norm_full || norm_w, CODA_ERR_ARG, "decode_attend_append: head-norm weight missing");
  CODA_REQUIRE(((uintptr_t)st->k_buf % 16 == 0) && ((uintptr_t)st->v_buf % 16 == 0) && ((uintptr_t)q_raw % 16 == 0) && (q_bs % 8 == 0) &&
               ((uintptr_t)cos_theta % 8 == 0) && ((uintptr_t)sin_theta % 8 == 0), CODA_ERR_ARG,
               "decode_attend_append: k_buf / v_buf / q_raw must be 16-byte aligned (q stride a multiple of 8 elements), the theta tables 8-byte aligned");
  CODA_REQUIRE(rp.recent_idx >= 0 && rp.recent_idx < cfg->W && rp.recent_filled >= 0 && rp.recent_filled <= cfg->W,
               CODA_ERR_ARG, "decode_attend_append: ring scalars out of range");
  DecodeParams p = make_params(cfg, st, nullptr, norm_w, out, out_bs, status);
  p.rp = rp;
  p.k_raw = (const bf16*)k_raw; p.k_bs = k_bs; p.v_new = (const bf16*)v_new; p.v_bs = v_bs;
  p.gate_logit = (const bf16*)gate_logit; p.gate_bs = gate_bs; p.gated = cfg->gated;
  p.inv_freq = inv_freq; p.q_raw = (const bf16*)q_raw; p.q_bs = q_bs; p.lam_logit = (const bf16*)lam_logit; p.lam_bs = lam_bs;
  p.cos_t = (const bf16*)cos_theta; p.sin_t = (const bf16*)sin_theta; p.rope_cs = rope_cs;
  p.k_buf = (bf16*)st->k_buf; p.v_buf = (bf16*)st->v_buf; p.allowed_w = st->allowed; p.g_recent = st->g_recent;
  return launch_main(cfg, st, p, (cudaStream_t)stream, true);
}

// cos [Dh/2] | sin [Dh/2] of the position the ring scalars `rp` (+ device step counter) name, rounded as the decode
// kernels round them (primitives.py:30-64 in bf16: angle dtype, then the K/V dtype): layers that share head_dim,
// RoPE base and dtype can compute it once per step and hand it to coda_b200_decode_attend_append.
__global__ void rope_table_kernel(coda_ring_pos rp, int W, const float* inv_freq, int half, int angle_bf16, float* out) {
  const int i = threadIdx.x;
  if (i >= half) return;
  const RingNow r = ring_now(rp, W);
  float ta = (float)r.pos, inv = inv_freq[i];
  if (angle_bf16) { ta = bf16_round(ta); inv = bf16_round(inv); }
  float ang = __fmul_rn(ta, inv);
  if (angle_bf16) ang = bf16_round(ang);
  float cc, ss; sincos_call(ang, &ss, &cc);
  if (angle_bf16) { cc = bf16_round(cc); ss = bf16_round(ss); }
  out[i] = bf16_round(cc); out[half + i] = bf16_round(ss);
}

extern "C" int coda_b200_rope_table(const coda_layer_cfg* cfg, coda_ring_pos rp, const float* inv_freq, float* out,
                                    coda_stream_t stream) {
  CODA_REQUIRE(coda_cfg_ok(cfg) && inv_freq && out && cfg->Dh / 2 <= 1024, CODA_ERR_ARG, "rope_table: invalid arguments");
  rope_table_kernel<<<1, (cfg->Dh / 2 + 31) / 32 * 32, 0, (cudaStream_t)stream>>>(rp, cfg->W, inv_freq, cfg->Dh / 2,
                                                                                cfg->angle_dtype == CODA_BF16, out);
  CODA_CHECK_LAUNCH("rope_table");
  return CODA_OK;
}
