// Y[M x N] = X[M x K] . W[N x K]^T (+ R), bf16 in / fp32 accumulate / bf16 out, for M <= 32 rows: the decode
// step's output projection (upstream attention.py:514, `self.o_proj(...)`, with the decoder's residual added
// in the same pass).  With so few rows the GEMM is a stream of the weight matrix: 2*N*K bytes from HBM once.
//
// One thread-block cluster of two CTAs per 64 weight rows; the pair splits K.  Each CTA keeps ITS half of X in
// shared memory for the whole kernel (TMA, 128-byte swizzle: 32 rows x 64 elements per box) and streams its half
// of the 64 weight rows through a ring of 64 x 64 boxes.  Tensor-core tiles take the WEIGHT rows as m = 16 and the
// X rows as n = 8 (Y^T = W . X^T), so that M = 32 fills four n-tiles with no padding.  Eight consumer warps: warp w
// owns weight rows (w % 4) * 16 .. + 15 and k-steps 2 * (w / 4), + 1 of every box.  At the end the two k-step halves
// meet in shared memory, the second CTA's sum crosses to the first through distributed shared memory, and the
// first adds the residual and writes the 32 x 64 output tile with 16-byte stores.
// Every mbarrier wait is bounded (status word); the cluster barriers are hardware barriers among co-scheduled CTAs.
#include "coda_common.cuh"
#include "tma_utils.cuh"
#include "tensor_maps.h"

namespace {

constexpr int SG_BN = 64;            // weight rows per cluster
constexpr int SG_BK = 64;            // elements per box row (128 bytes)
constexpr int SG_MAXM = 32;          // rows of X
constexpr int SG_STAGES = 11;        // ring of weight boxes (8 KB each)
constexpr int SG_CWARPS = 8;
constexpr int SG_THREADS = (SG_CWARPS + 1) * 32;
constexpr int SG_XGROUP = 4;         // X boxes per arrival barrier
constexpr int SG_MAXXG = 8;          // (K / 2 / 64) / SG_XGROUP at K = 4096
constexpr int SG_WBOX = SG_BN * 128; // bytes of a weight box
constexpr int SG_XBOX = SG_MAXM * 128;

struct SkinnyParams {
  int M, N, K;
  const bf16* res; long long res_rs;   // optional residual [M][N]
  const bf16* bias;                    // optional bias [N] (four-way kernel)
  bf16* y; long long y_rs;
  int* status;
};

using tma::smem_u32;

__device__ __forceinline__ void sg_tma_load(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
               ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(0) : "memory");
}
__device__ __forceinline__ void sg_ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void sg_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t bf16_pack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
// byte offset of 16-byte chunk c (0..7) of row r inside a box of 128-byte rows written with the 128-byte swizzle
__device__ __forceinline__ uint32_t sg_off(int r, int c) { return (uint32_t)(r * 128 + ((c ^ (r & 7)) << 4)); }

// shared-memory carve-up (after 1024-byte alignment): X half | weight ring | exchange tile | barriers
struct SkinnySmem {
  int x, ring, xchg, bars, total;
  __host__ __device__ explicit SkinnySmem(int khalf) {
    x = 0;
    ring = x + (khalf / SG_BK) * SG_XBOX;
    xchg = ring + SG_STAGES * SG_WBOX;                 // [32][64] fp32 from the other CTA of the pair
    bars = xchg + SG_MAXM * SG_BN * 4;
    total = bars + (2 * SG_STAGES + SG_MAXXG) * 8;
  }
};

__global__ void __launch_bounds__(SG_THREADS, 1)
skinny_gemm_kernel(const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap wmap, SkinnyParams p) {
  extern __shared__ unsigned char sg_raw[];
  unsigned char* smem = sg_raw + ((1024u - (smem_u32(sg_raw) & 1023u)) & 1023u);   // swizzled boxes need 1024-byte alignment
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int rank = blockIdx.x;                           // position in the pair = cluster rank (cluster dims (2,1,1))
  const int n0 = blockIdx.y * SG_BN;
  const int khalf = p.K / 2, kbase = rank * khalf, nbox = khalf / SG_BK;
  const SkinnySmem L(khalf);
  unsigned char* xs = smem + L.x;
  unsigned char* ring = smem + L.ring;
  float* xchg = reinterpret_cast<float*>(smem + L.xchg);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L.bars);
  uint64_t* empty = full + SG_STAGES;
  uint64_t* xbar = empty + SG_STAGES;

  // The other CTA's shared memory may be written only once that CTA runs: announce here, wait before the exchange.
  asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
  __shared__ int s_abort;                          // set by the first bounded wait of this CTA that expires
  int* const abortw = &s_abort;
  if (tid == 0) {
    s_abort = 0;
    for (int i = 0; i < SG_STAGES; ++i) { tma::mbar_init(&full[i], 1); tma::mbar_init(&empty[i], SG_CWARPS); }
    for (int i = 0; i < SG_MAXXG; ++i) tma::mbar_init(&xbar[i], 1);
    tma::fence_barrier_init();
  }
  __syncthreads();

  float acc[4][4];
#pragma unroll
  for (int mt = 0; mt < 4; ++mt) acc[mt][0] = acc[mt][1] = acc[mt][2] = acc[mt][3] = 0.f;
  const int rb = warp & 3, kp = (warp >> 2) & 1;         // consumer warp: weight rows rb*16.., k-steps 2*kp, 2*kp+1 of a box
  const int li = lane >> 3, lr = lane & 7;

  if (warp == SG_CWARPS) {
    // ---------------- producer: this CTA's half of X, then the ring of weight boxes ----------------
    if (lane == 0) {
      for (int i = 0; i < nbox; ++i) {
        // X travels in groups of SG_XGROUP boxes, each just ahead of the weight boxes that need it, so that the
        // first tiles do not wait for all of X
        if (i % SG_XGROUP == 0) {
          const int g = i / SG_XGROUP, nb = min(SG_XGROUP, nbox - i);
          tma::mbar_expect_tx(&xbar[g], (uint32_t)nb * SG_XBOX);
          for (int j = 0; j < nb; ++j) sg_tma_load(xs + (i + j) * SG_XBOX, &xmap, &xbar[g], kbase + (i + j) * SG_BK, 0);
        }
        const int s = i % SG_STAGES, round = i / SG_STAGES;
        if (round > 0) tma::mbar_wait(&empty[s], (round - 1) & 1, p.status, 21, abortw);
        tma::mbar_expect_tx(&full[s], SG_WBOX);
        sg_tma_load(ring + s * SG_WBOX, &wmap, &full[s], kbase + i * SG_BK, n0);
      }
    }
    __syncwarp();
  } else {
    // ---------------- consumers ----------------
    const uint32_t xs_u = smem_u32(xs), ring_u = smem_u32(ring);
    for (int i = 0; i < nbox; ++i) {
      if (i % SG_XGROUP == 0) tma::mbar_wait(&xbar[i / SG_XGROUP], 0, p.status, 22, abortw);   // each X barrier completes once
      const int s = i % SG_STAGES, round = i / SG_STAGES;
      tma::mbar_wait(&full[s], round & 1, p.status, 23, abortw);
      const uint32_t wb = ring_u + s * SG_WBOX, xb = xs_u + i * SG_XBOX;
      uint32_t a0[4], a1[4];                               // weight fragments of the two k-steps
      const int wrow = rb * 16 + (li & 1) * 8 + lr;
      sg_ldsm_x4(a0, wb + sg_off(wrow, (2 * kp) * 2 + (li >> 1)));
      sg_ldsm_x4(a1, wb + sg_off(wrow, (2 * kp + 1) * 2 + (li >> 1)));
#pragma unroll
      for (int mt = 0; mt < 4; ++mt) {
        uint32_t bx[4];                                    // X^T fragments: {k 0-7, k 8-15} of both k-steps
        sg_ldsm_x4(bx, xb + sg_off(mt * 8 + lr, 4 * kp + li));
        sg_mma(acc[mt], a0, bx[0], bx[1]);
        sg_mma(acc[mt], a1, bx[2], bx[3]);
      }
      __syncwarp();
      if (lane == 0) tma::mbar_arrive(&empty[s]);
    }
    // ---- the two k-step halves meet in shared memory (the ring is free: every box has been consumed) ----
    asm volatile("bar.sync 1, 256;" ::: "memory");
    float* red = reinterpret_cast<float*>(ring);           // [2][32][64]
#pragma unroll
    for (int mt = 0; mt < 4; ++mt) {
      const int n = rb * 16 + (lane >> 2), m = mt * 8 + 2 * (lane & 3);
      float* r0 = red + (kp * SG_MAXM + m) * SG_BN + n;
      r0[0] = acc[mt][0]; r0[SG_BN] = acc[mt][1]; r0[8] = acc[mt][2]; r0[SG_BN + 8] = acc[mt][3];
    }
    asm volatile("bar.sync 1, 256;" ::: "memory");
  }

  // ---- pair exchange: the second CTA's sums cross to the first, which finishes the tile ----
  asm volatile("barrier.cluster.wait.aligned;" ::: "memory");          // (pairs with the arrive at entry)
  const int m = tid >> 3, n8 = (tid & 7) * 8;                          // this thread's 8 outputs (consumer threads only)
  float sum[8];
  if (warp < SG_CWARPS) {
    const float* red = reinterpret_cast<const float*>(ring);
    const float4 u0 = *reinterpret_cast<const float4*>(red + m * SG_BN + n8), u1 = *reinterpret_cast<const float4*>(red + m * SG_BN + n8 + 4);
    const float4 v0 = *reinterpret_cast<const float4*>(red + (SG_MAXM + m) * SG_BN + n8), v1 = *reinterpret_cast<const float4*>(red + (SG_MAXM + m) * SG_BN + n8 + 4);
    sum[0] = u0.x + v0.x; sum[1] = u0.y + v0.y; sum[2] = u0.z + v0.z; sum[3] = u0.w + v0.w;
    sum[4] = u1.x + v1.x; sum[5] = u1.y + v1.y; sum[6] = u1.z + v1.z; sum[7] = u1.w + v1.w;
    if (rank == 1) {
      uint32_t remote;
      asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(xchg + m * SG_BN + n8)), "r"(0));
      asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(remote), "f"(sum[0]), "f"(sum[1]), "f"(sum[2]), "f"(sum[3]) : "memory");
      asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(remote + 16), "f"(sum[4]), "f"(sum[5]), "f"(sum[6]), "f"(sum[7]) : "memory");
    }
  }
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
  if (rank == 0 && warp < SG_CWARPS && m < p.M) {
    const float4 o0 = *reinterpret_cast<const float4*>(xchg + m * SG_BN + n8), o1 = *reinterpret_cast<const float4*>(xchg + m * SG_BN + n8 + 4);
    float t[8] = {sum[0] + o0.x, sum[1] + o0.y, sum[2] + o0.z, sum[3] + o0.w, sum[4] + o1.x, sum[5] + o1.y, sum[6] + o1.z, sum[7] + o1.w};
    if (p.res != nullptr) {
      const uint4 rv = *reinterpret_cast<const uint4*>(p.res + (long long)m * p.res_rs + n0 + n8);
      const uint32_t rw[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        // the product is rounded to bf16 first, as a GEMM followed by a separate add would
        t[2 * q] = bf16_round(t[2 * q]) + __uint_as_float(rw[q] << 16);
        t[2 * q + 1] = bf16_round(t[2 * q + 1]) + __uint_as_float(rw[q] & 0xffff0000u);
      }
    }
    uint4 ov;
    ov.x = bf16_pack(t[0], t[1]); ov.y = bf16_pack(t[2], t[3]); ov.z = bf16_pack(t[4], t[5]); ov.w = bf16_pack(t[6], t[7]);
    *reinterpret_cast<uint4*>(p.y + (long long)m * p.y_rs + n0 + n8) = ov;
  }
}


// ---- the same product with K split four ways -------------------------------------------------------------------
// A CTA takes in its weight rows AND its share of X, and what bounds the kernel is the bytes one SM can take in
// (about 45 GB/s).  With a pair per 64 rows every CTA reads half of X: a third of its traffic.  Here a cluster of
// FOUR CTAs shares a tile of `bn` weight rows (the smallest multiple of 16 with which all clusters are resident at
// once, as the occupancy query of the device says: 128 at N = 4096 where 32 clusters of four fit), each CTA reads
// a quarter of K -- a quarter of X.  Consumer warp w owns
// weight rows 16 w .. 16 w + 15 of the tile and all four k-steps of a box.  At the end the 16-row groups of the tile
// are dealt out to the four CTAs (group g to CTA g % 4): every CTA sends its partial sums of a group to the group's
// owner through distributed shared memory, and the owner adds the four partials (in rank order), bias or residual,
// and writes.  Launched as a programmatic dependent: the first ring pass of WEIGHT boxes goes out before the wait
// for the kernel that produces X, and the kernel after this one is let onto the SMs from the start.
// CW: consumer warps (tiles of up to 16 CW rows); STAGES ring slots of 16 CW x 128 bytes.
constexpr int S4_CL = 4;

template <int CW, int STAGES>
struct Skinny4Smem {
  static constexpr int SLOT = CW * 16 * 128;
  static constexpr int XCH_BYTES = S4_CL * ((CW + 3) / 4) * SG_MAXM * 16 * 4;   // partial sums [src rank][group slot][token][row] fp32
  // The exchange space is the instance's own where X at its largest, the ring and it fit one CTA; otherwise it
  // lies over the ring, which must then be drained in every CTA of the cluster before the first partial sum lands.
  static constexpr bool OWN_XCH = SG_XGROUP * SG_MAXXG / 2 * SG_XBOX + STAGES * SLOT + XCH_BYTES + 2048 <= 226 * 1024;
  int x, ring, xch, bars, total;
  __host__ __device__ explicit Skinny4Smem(int kq) {
    x = 0;
    ring = x + (kq / SG_BK) * SG_XBOX;
    xch = OWN_XCH ? ring + STAGES * SLOT : ring;
    bars = ring + STAGES * SLOT + (OWN_XCH ? XCH_BYTES : 0);
    total = bars + (2 * STAGES + SG_MAXXG) * 8;
  }
};

template <int CW, int STAGES>
__global__ void __launch_bounds__((CW + 1) * 32, 1)
skinny_gemm4_kernel(const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap wmap, SkinnyParams p, int bn) {
  constexpr int SLOT = Skinny4Smem<CW, STAGES>::SLOT;
  extern __shared__ unsigned char sg_raw[];
  unsigned char* smem = sg_raw + ((1024u - (smem_u32(sg_raw) & 1023u)) & 1023u);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int rank = blockIdx.x;                           // cluster rank (cluster dims (4,1,1))
  const int n0 = blockIdx.y * bn;
  const int kq = p.K / S4_CL, kbase = rank * kq, nbox = kq / SG_BK;
  const int ngrp = bn / 16;                              // 16-row groups of the tile = working consumer warps
  const Skinny4Smem<CW, STAGES> L(kq);
  unsigned char* xs = smem + L.x;
  unsigned char* ring = smem + L.ring;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L.bars);
  uint64_t* empty = full + STAGES;
  uint64_t* xbar = empty + STAGES;
  const uint32_t wbox_bytes = (uint32_t)bn * 128;

  asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  __shared__ int s_abort;
  int* const abortw = &s_abort;
  if (tid == 0) {
    s_abort = 0;
    for (int i = 0; i < STAGES; ++i) { tma::mbar_init(&full[i], 1); tma::mbar_init(&empty[i], ngrp); }
    for (int i = 0; i < SG_MAXXG; ++i) tma::mbar_init(&xbar[i], 1);
    tma::fence_barrier_init();
  }
  __syncthreads();

  float acc[4][4];
#pragma unroll
  for (int mt = 0; mt < 4; ++mt) acc[mt][0] = acc[mt][1] = acc[mt][2] = acc[mt][3] = 0.f;
  const int li = lane >> 3, lr = lane & 7;

  if (warp == CW) {
    if (lane == 0) {
      // The weights do not depend on the kernel before this one: the first pass of the ring is requested BEFORE
      // waiting for it, X -- that kernel's output -- after.
      const int pre = min(nbox, STAGES);
      for (int i = 0; i < pre; ++i) {
        tma::mbar_expect_tx(&full[i], wbox_bytes);
        sg_tma_load(ring + i * SLOT, &wmap, &full[i], kbase + i * SG_BK, n0);
      }
      asm volatile("griddepcontrol.wait;" ::: "memory");
      for (int i = 0; i < nbox; ++i) {
        if (i % SG_XGROUP == 0) {
          const int g = i / SG_XGROUP, nb = min(SG_XGROUP, nbox - i);
          tma::mbar_expect_tx(&xbar[g], (uint32_t)nb * SG_XBOX);
          for (int j = 0; j < nb; ++j) sg_tma_load(xs + (i + j) * SG_XBOX, &xmap, &xbar[g], kbase + (i + j) * SG_BK, 0);
        }
        if (i < pre) continue;
        const int s = i % STAGES, round = i / STAGES;
        if (round > 0) tma::mbar_wait(&empty[s], (round - 1) & 1, p.status, 24, abortw);
        tma::mbar_expect_tx(&full[s], wbox_bytes);
        sg_tma_load(ring + s * SLOT, &wmap, &full[s], kbase + i * SG_BK, n0);
      }
    }
    __syncwarp();
  } else if (warp < ngrp) {
    const uint32_t xs_u = smem_u32(xs), ring_u = smem_u32(ring);
    const int wrow = warp * 16 + (li & 1) * 8 + lr;
    for (int i = 0; i < nbox; ++i) {
      if (i % SG_XGROUP == 0) tma::mbar_wait(&xbar[i / SG_XGROUP], 0, p.status, 25, abortw);
      const int s = i % STAGES, round = i / STAGES;
      tma::mbar_wait(&full[s], round & 1, p.status, 26, abortw);
      const uint32_t wb = ring_u + s * SLOT, xb = xs_u + i * SG_XBOX;
      uint32_t a[4][4];                                  // weight fragments of the box's four k-steps
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) sg_ldsm_x4(a[ks], wb + sg_off(wrow, ks * 2 + (li >> 1)));
#pragma unroll
      for (int mt = 0; mt < 4; ++mt) {
        uint32_t b0[4], b1[4];                           // X^T fragments: k 0-31 and k 32-63 of the box
        sg_ldsm_x4(b0, xb + sg_off(mt * 8 + lr, li));
        sg_ldsm_x4(b1, xb + sg_off(mt * 8 + lr, 4 + li));
        sg_mma(acc[mt], a[0], b0[0], b0[1]);
        sg_mma(acc[mt], a[1], b0[2], b0[3]);
        sg_mma(acc[mt], a[2], b1[0], b1[1]);
        sg_mma(acc[mt], a[3], b1[2], b1[3]);
      }
      __syncwarp();
      if (lane == 0) tma::mbar_arrive(&empty[s]);
    }
  }

  // ---- exchange: partial sums go to the owners' shared memory.  Where that space lies over the ring, every CTA of the
  // cluster must have consumed its ring first (cluster barrier); where it is the instance's own, a warp sends its sums
  // as soon as it has them, under the other CTAs' last boxes ----
  asm volatile("griddepcontrol.wait;" ::: "memory");                   // (bias, residual and output belong to this kernel's place in the stream)
  asm volatile("barrier.cluster.wait.aligned;" ::: "memory");          // (pairs with the arrive at entry: all CTAs run)
  if (!Skinny4Smem<CW, STAGES>::OWN_XCH)
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
  // xch[src rank][owner's group slot gs][token 32][row 16] fp32, in the OWNER's shared memory
  constexpr int GS = (CW + 3) / 4;                                     // group slots per owner
  float* xch = reinterpret_cast<float*>(smem + L.xch);
  if (warp < ngrp) {
    const int g = warp, owner = g & 3, gs = g >> 2;
    const uint32_t base_local = smem_u32(xch + ((rank * GS + gs) * SG_MAXM) * 16);
    uint32_t base_remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(base_remote) : "r"(base_local), "r"(owner));
#pragma unroll
    for (int mt = 0; mt < 4; ++mt) {
      const int tok = mt * 8 + 2 * (lane & 3), nl = lane >> 2;         // C fragment: rows nl, nl + 8 of the group; tokens tok, tok + 1
      const uint32_t a0 = base_remote + (uint32_t)((tok * 16 + nl) * 4);
      asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(a0), "f"(acc[mt][0]) : "memory");
      asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(a0 + 16 * 4), "f"(acc[mt][1]) : "memory");
      asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(a0 + 8 * 4), "f"(acc[mt][2]) : "memory");
      asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(a0 + (16 + 8) * 4), "f"(acc[mt][3]) : "memory");
    }
  }
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
  // ---- the owner of a group adds the four partials, bias / residual, and writes 4 consecutive outputs per thread ----
  if (warp < CW) {
    const int gs = tid >> 7, g = rank + 4 * gs;                        // group slot, group of the tile
    const int m = (tid & 127) >> 2, nq = (tid & 3) * 4;                // token, first of 4 rows inside the group
    const int n = n0 + g * 16 + nq;
    if (gs < GS && g < ngrp && m < p.M && n < p.N) {
      float t[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int src = 0; src < S4_CL; ++src) {
        const float4 v = *reinterpret_cast<const float4*>(xch + ((src * GS + gs) * SG_MAXM + m) * 16 + nq);
        t[0] += v.x; t[1] += v.y; t[2] += v.z; t[3] += v.w;
      }
      if (p.bias != nullptr) {                                         // fp32 sum + bias, one rounding (a linear layer's epilogue)
        const uint2 bv = *reinterpret_cast<const uint2*>(p.bias + n);
        t[0] += __uint_as_float(bv.x << 16); t[1] += __uint_as_float(bv.x & 0xffff0000u);
        t[2] += __uint_as_float(bv.y << 16); t[3] += __uint_as_float(bv.y & 0xffff0000u);
      }
      if (p.res != nullptr) {
        const uint2 rv = *reinterpret_cast<const uint2*>(p.res + (long long)m * p.res_rs + n);
        // the product is rounded to bf16 first, as a GEMM followed by a separate add would
        t[0] = bf16_round(t[0]) + __uint_as_float(rv.x << 16);
        t[1] = bf16_round(t[1]) + __uint_as_float(rv.x & 0xffff0000u);
        t[2] = bf16_round(t[2]) + __uint_as_float(rv.y << 16);
        t[3] = bf16_round(t[3]) + __uint_as_float(rv.y & 0xffff0000u);
      }
      uint2 ov;
      ov.x = bf16_pack(t[0], t[1]); ov.y = bf16_pack(t[2], t[3]);
      *reinterpret_cast<uint2*>(p.y + (long long)m * p.y_rs + n) = ov;
    }
  }
}

// One instance of the four-way kernel: set-up once per device, clusters that fit at once, launch.
template <int CW, int STAGES>
struct Skinny4 {
  static int max_clusters(size_t smem) {
    static coda_device_once once;
    static int mc[64];
    const int dev = coda_current_device();
    coda_on_first_use(once, [smem, dev] {
      cudaFuncSetAttribute(skinny_gemm4_kernel<CW, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024);
      cudaLaunchConfig_t q = {};
      q.gridDim = dim3(S4_CL, 64, 1); q.blockDim = dim3((CW + 1) * 32, 1, 1); q.dynamicSmemBytes = smem;
      cudaLaunchAttribute qa[1];
      qa[0].id = cudaLaunchAttributeClusterDimension;
      qa[0].val.clusterDim.x = S4_CL; qa[0].val.clusterDim.y = 1; qa[0].val.clusterDim.z = 1;
      q.attrs = qa; q.numAttrs = 1;
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, skinny_gemm4_kernel<CW, STAGES>, &q) != cudaSuccess) { n = 0; cudaGetLastError(); }
      if (dev >= 0 && dev < 64) mc[dev] = n;
    });
    return (dev >= 0 && dev < 64) ? mc[dev] : 0;
  }
  static int launch(const CUtensorMap& xm, const void* w, const SkinnyParams& p, int bn, size_t smem, cudaStream_t stream) {
    CUtensorMap wm;
    CODA_REQUIRE(tmaps::plane_map(&wm, w, 1, p.N, p.K, bn), CODA_ERR_LAUNCH, "skinny_gemm: cuTensorMapEncodeTiled failed");
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3(S4_CL, (p.N + bn - 1) / bn, 1);
    lc.blockDim = dim3((CW + 1) * 32, 1, 1);
    lc.dynamicSmemBytes = smem;
    lc.stream = stream;
    cudaLaunchAttribute at[2];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = S4_CL; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
    at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[1].val.programmaticStreamSerializationAllowed = 1;
    lc.attrs = at; lc.numAttrs = 2;
    cudaError_t e = cudaLaunchKernelEx(&lc, skinny_gemm4_kernel<CW, STAGES>, xm, wm, p, bn);
    if (e != cudaSuccess) { coda_set_error("skinny_gemm (four-way): %s", cudaGetErrorString(e)); return CODA_ERR_LAUNCH; }
    return CODA_OK;
  }
};

// ---- two dependent products behind one launch -------------------------------------------------------------------
// A decode step's output projection (with the residual) is followed by the next layer's input projection, whose X is
// the first product's Y.  As two launches the second pays its own ramp: launch, barrier set-up, first boxes.  Here
// the same CTAs run both products (phase A, then phase B) with a barrier across the whole grid in between:
//   * the grid is one wave (the launcher sizes the tiles so that all clusters are resident at once), so every CTA
//     reaches the barrier; the wait is bounded all the same and reports through the status word;
//   * phase B's first ring pass of WEIGHT boxes goes out before the barrier -- the weights depend on nothing --
//     and streams while the slower CTAs finish phase A;
//   * phase A's outputs are written with generic stores, fenced, and read in phase B by TMA behind a proxy fence.
// `gsync`: two words of device memory, zero before the first launch: arrival count and generation.  Launches that
// share them must be ordered on one stream.
__device__ __forceinline__ void sg_grid_barrier(unsigned int* gsync, unsigned int nctas, int* status) {
  unsigned int gen, now;
  asm volatile("ld.acquire.gpu.u32 %0, [%1];" : "=r"(gen) : "l"(gsync + 1) : "memory");
  __threadfence();
  const unsigned int old = atomicAdd(gsync, 1u);
  if (old == nctas - 1) {
    gsync[0] = 0u;
    __threadfence();
    atomicAdd(gsync + 1, 1u);
    return;
  }
  for (int it = 0; it < (1 << 24); ++it) {
    asm volatile("ld.acquire.gpu.u32 %0, [%1];" : "=r"(now) : "l"(gsync + 1) : "memory");
    if (now != gen) return;
  }
  if (status) atomicCAS(status, 0, 27);                                // gave up: the results of phase B are not valid
}

template <int CW, int STAGES>
struct ChainSmem {
  static constexpr int SLOT = CW * 16 * 128;
  static constexpr int GS = (CW + 3) / 4;                // group slots per owner
  static constexpr int NBAR = 2 * STAGES + 2 * SG_MAXXG; // full, empty, X arrivals of phase A and of phase B
  int x, ring, xch, bars, total;
  __host__ __device__ explicit ChainSmem(int kq_max) {
    x = 0;
    ring = x + (kq_max / SG_BK) * SG_XBOX;
    xch = ring + STAGES * SLOT;                          // partial sums [src rank][group slot][token 32][row 16] fp32
    bars = xch + S4_CL * GS * SG_MAXM * 16 * 4;
    total = bars + NBAR * 8;
  }
};

template <int CW, int STAGES>
__global__ void __launch_bounds__((CW + 1) * 32, 1)
skinny_gemm4_chain_kernel(const __grid_constant__ CUtensorMap xmapA, const __grid_constant__ CUtensorMap wmapA, SkinnyParams pA, int bnA,
                          const __grid_constant__ CUtensorMap xmapB, const __grid_constant__ CUtensorMap wmapB, SkinnyParams pB, int bnB,
                          unsigned int* gsync, int kq_max) {
  using SM = ChainSmem<CW, STAGES>;
  constexpr int SLOT = SM::SLOT, GS = SM::GS;
  extern __shared__ unsigned char sg_raw[];
  unsigned char* smem = sg_raw + ((1024u - (smem_u32(sg_raw) & 1023u)) & 1023u);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int rank = blockIdx.x;                           // cluster rank (cluster dims (4,1,1))
  const SM L(kq_max);
  unsigned char* xs = smem + L.x;
  unsigned char* ring = smem + L.ring;
  float* xch = reinterpret_cast<float*>(smem + L.xch);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L.bars);
  uint64_t* empty = full + STAGES;
  uint64_t* xbars = empty + STAGES;                      // [2 phases][SG_MAXXG]

  asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  __shared__ int s_abort;
  int* const abortw = &s_abort;
  if (tid == 0) {
    s_abort = 0;
    // one ring for both phases: every consumer warp takes part in its hand-shake, also where a phase's tile leaves
    // it without rows, so that the arrival count of a slot does not depend on the phase
    for (int i = 0; i < STAGES; ++i) { tma::mbar_init(&full[i], 1); tma::mbar_init(&empty[i], CW); }
    for (int i = 0; i < 2 * SG_MAXXG; ++i) tma::mbar_init(&xbars[i], 1);
    tma::fence_barrier_init();
  }
  __syncthreads();
  const int li = lane >> 3, lr = lane & 7;
  const unsigned int nctas = gridDim.x * gridDim.y;
  const int n0A = blockIdx.y * bnA, n0B = blockIdx.y * bnB;
  const bool activeA = n0A < pA.N, activeB = n0B < pB.N; // (a phase with fewer tiles leaves the last clusters idle)
  const int nboxA = pA.K / S4_CL / SG_BK, nboxB = pB.K / S4_CL / SG_BK;
  int gi = 0;                                            // boxes through the ring so far (producer and consumers count alike)

  // producer: box i of a phase into the next ring slot, behind the consumers' release of that slot
  auto issue_w = [&](const CUtensorMap* wmap, int kcoord, int n0, uint32_t bytes, int* status) {
    const int s = gi % STAGES, round = gi / STAGES;
    if (round > 0) tma::mbar_wait(&empty[s], (round - 1) & 1, status, 24, abortw);
    tma::mbar_expect_tx(&full[s], bytes);
    sg_tma_load(ring + s * SLOT, wmap, &full[s], kcoord, n0);
    ++gi;
  };

#pragma unroll 1
  for (int ph = 0; ph < 2; ++ph) {
    const CUtensorMap* xmap = ph ? &xmapB : &xmapA;
    const CUtensorMap* wmap = ph ? &wmapB : &wmapA;
    const SkinnyParams& p = ph ? pB : pA;
    const int bn = ph ? bnB : bnA;
    const int n0 = ph ? n0B : n0A;
    const bool active = ph ? activeB : activeA;
    const int kq = p.K / S4_CL, kbase = rank * kq, nbox = ph ? nboxB : nboxA;
    const int ngrp = bn / 16;                            // 16-row groups of the tile = consumer warps with rows
    uint64_t* xbar = xbars + ph * SG_MAXXG;
    const uint32_t wbox_bytes = (uint32_t)bn * 128;
    float acc[4][4];
#pragma unroll
    for (int mt = 0; mt < 4; ++mt) acc[mt][0] = acc[mt][1] = acc[mt][2] = acc[mt][3] = 0.f;

    if (warp == CW) {
      if (lane == 0) {
        // Weights depend on nothing that runs before.  Phase A: the first ring pass goes out BEFORE the wait for
        // the kernel that produces X.  Phase B: its first ring pass was requested at the end of phase A (below), so
        // the ring refills while this CTA's last boxes, its exchange and the barrier across the grid go by.
        const int pre = active ? min(nbox, STAGES) : 0;
        if (ph == 0) {
          for (int i = 0; i < pre; ++i) issue_w(wmap, kbase + i * SG_BK, n0, wbox_bytes, p.status);
          asm volatile("griddepcontrol.wait;" ::: "memory");
        } else {
          sg_grid_barrier(gsync, nctas, p.status);
          asm volatile("fence.proxy.async;" ::: "memory");
        }
        for (int i = 0; active && i < nbox; ++i) {
          if (i % SG_XGROUP == 0) {
            const int g = i / SG_XGROUP, nb = min(SG_XGROUP, nbox - i);
            tma::mbar_expect_tx(&xbar[g], (uint32_t)nb * SG_XBOX);
            for (int j = 0; j < nb; ++j) sg_tma_load(xs + (i + j) * SG_XBOX, xmap, &xbar[g], kbase + (i + j) * SG_BK, 0);
          }
          if (i >= pre) issue_w(wmap, kbase + i * SG_BK, n0, wbox_bytes, p.status);
        }
        if (ph == 0 && activeB) {                        // phase B's first ring pass, into the slots phase A's consumers free
          const int preB = min(nboxB, STAGES), kqB = pB.K / S4_CL;
          for (int i = 0; i < preB; ++i) issue_w(&wmapB, rank * kqB + i * SG_BK, n0B, (uint32_t)bnB * 128, pB.status);
        }
      }
      __syncwarp();
    } else if (active) {
      const uint32_t xs_u = smem_u32(xs), ring_u = smem_u32(ring);
      const int wrow = warp * 16 + (li & 1) * 8 + lr;
      const bool rows = warp < ngrp;
      for (int i = 0; i < nbox; ++i, ++gi) {
        if (rows && i % SG_XGROUP == 0) tma::mbar_wait(&xbar[i / SG_XGROUP], 0, p.status, 25, abortw);
        const int s = gi % STAGES, round = gi / STAGES;
        tma::mbar_wait(&full[s], round & 1, p.status, 26, abortw);
        if (rows) {
          const uint32_t wb = ring_u + s * SLOT, xb = xs_u + i * SG_XBOX;
          uint32_t a[4][4];                                // weight fragments of the box's four k-steps
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) sg_ldsm_x4(a[ks], wb + sg_off(wrow, ks * 2 + (li >> 1)));
#pragma unroll
          for (int mt = 0; mt < 4; ++mt) {
            uint32_t b0[4], b1[4];                         // X^T fragments: k 0-31 and k 32-63 of the box
            sg_ldsm_x4(b0, xb + sg_off(mt * 8 + lr, li));
            sg_ldsm_x4(b1, xb + sg_off(mt * 8 + lr, 4 + li));
            sg_mma(acc[mt], a[0], b0[0], b0[1]);
            sg_mma(acc[mt], a[1], b0[2], b0[3]);
            sg_mma(acc[mt], a[2], b1[0], b1[1]);
            sg_mma(acc[mt], a[3], b1[2], b1[3]);
          }
        }
        __syncwarp();
        if (lane == 0) tma::mbar_arrive(&empty[s]);
      }
    }

    // ---- exchange through the owners' shared memory (its own space: the ring already holds the next phase) ----
    if (ph == 0) {
      asm volatile("griddepcontrol.wait;" ::: "memory");               // (residual and output belong to this kernel's place in the stream)
      asm volatile("barrier.cluster.wait.aligned;" ::: "memory");      // (pairs with the arrive at entry: all CTAs run)
    }
    if (active) {                                                      // (the whole cluster: same tile index)
      // every owner has read the previous phase's partial sums
      asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
      if (warp < ngrp) {
        const int g = warp, owner = g & 3, gs = g >> 2;
        const uint32_t base_local = smem_u32(xch + ((rank * GS + gs) * SG_MAXM) * 16);
        uint32_t base_remote;
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(base_remote) : "r"(base_local), "r"(owner));
#pragma unroll
        for (int mt = 0; mt < 4; ++mt) {
          const int tok = mt * 8 + 2 * (lane & 3), nl = lane >> 2;     // C fragment: rows nl, nl + 8 of the group; tokens tok, tok + 1
          const uint32_t a0 = base_remote + (uint32_t)((tok * 16 + nl) * 4);
          asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(a0), "f"(acc[mt][0]) : "memory");
          asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(a0 + 16 * 4), "f"(acc[mt][1]) : "memory");
          asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(a0 + 8 * 4), "f"(acc[mt][2]) : "memory");
          asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(a0 + (16 + 8) * 4), "f"(acc[mt][3]) : "memory");
        }
      }
      asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
      if (warp < CW) {
        const int gs = tid >> 7, g = rank + 4 * gs;                    // group slot, group of the tile
        const int m = (tid & 127) >> 2, nq = (tid & 3) * 4;            // token, first of 4 rows inside the group
        const int n = n0 + g * 16 + nq;
        if (gs < GS && g < ngrp && m < p.M && n < p.N) {
          float t[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int src = 0; src < S4_CL; ++src) {
            const float4 v = *reinterpret_cast<const float4*>(xch + ((src * GS + gs) * SG_MAXM + m) * 16 + nq);
            t[0] += v.x; t[1] += v.y; t[2] += v.z; t[3] += v.w;
          }
          if (p.bias != nullptr) {                                     // fp32 sum + bias, one rounding (a linear layer's epilogue)
            const uint2 bv = *reinterpret_cast<const uint2*>(p.bias + n);
            t[0] += __uint_as_float(bv.x << 16); t[1] += __uint_as_float(bv.x & 0xffff0000u);
            t[2] += __uint_as_float(bv.y << 16); t[3] += __uint_as_float(bv.y & 0xffff0000u);
          }
          if (p.res != nullptr) {
            const uint2 rv = *reinterpret_cast<const uint2*>(p.res + (long long)m * p.res_rs + n);
            // the product is rounded to bf16 first, as a GEMM followed by a separate add would
            t[0] = bf16_round(t[0]) + __uint_as_float(rv.x << 16);
            t[1] = bf16_round(t[1]) + __uint_as_float(rv.x & 0xffff0000u);
            t[2] = bf16_round(t[2]) + __uint_as_float(rv.y << 16);
            t[3] = bf16_round(t[3]) + __uint_as_float(rv.y & 0xffff0000u);
          }
          uint2 ov;
          ov.x = bf16_pack(t[0], t[1]); ov.y = bf16_pack(t[2], t[3]);
          *reinterpret_cast<uint2*>(p.y + (long long)m * p.y_rs + n) = ov;
        }
      }
    }
    if (ph == 0) {
      // everything this CTA wrote in phase A is out and fenced before its producer joins the barrier across the grid;
      // phase A's X is no longer read
      __threadfence();
      __syncthreads();
    }
  }
}

// Tile height for the four-way kernel: the smallest multiple of 16 rows with which the clusters fit the device at
// once; 0 when no instance covers it.  `cw` receives the instance (8 or 12 consumer warps).
static int skinny4_plan(int K, int N, int* cw) {
  if (K % 256 != 0 || K / 4 / SG_BK > SG_XGROUP * SG_MAXXG || N % 16 != 0) return 0;
  const int kq = K / 4;
  const int mc8 = Skinny4<8, 8>::max_clusters((size_t)Skinny4Smem<8, 8>(kq).total + 1024);
  if (mc8 > 0) {
    const int bn = ((N + mc8 - 1) / mc8 + 15) / 16 * 16;
    if (bn <= 128) { *cw = 8; return bn < 16 ? 16 : bn; }
  }
  const int mc12 = Skinny4<12, 6>::max_clusters((size_t)Skinny4Smem<12, 6>(kq).total + 1024);
  if (mc12 > 0) {
    const int bn = ((N + mc12 - 1) / mc12 + 15) / 16 * 16;
    if (bn <= 192) { *cw = 12; return bn; }
  }
  return 0;
}

}  // namespace

// Shapes the kernel covers: up to 32 rows, K a multiple of 128 and at most 4096 (each CTA of a pair keeps K/2
// columns of X in shared memory), N a multiple of 64.
extern "C" int coda_b200_skinny_gemm_supported(int32_t M, int32_t K, int32_t N) {
  return M >= 1 && M <= SG_MAXM && K >= 128 && K % 128 == 0 && K <= 4096 && N >= SG_BN && N % SG_BN == 0 && N / SG_BN <= 65535 &&
         tmaps::available();
}

extern "C" int coda_b200_skinny_gemm(const void* x, int32_t M, int32_t K, const void* w, int32_t N,
                                     const void* residual, int64_t res_rs, void* y, int64_t y_rs,
                                     int32_t* status, coda_stream_t stream) {
  return coda_b200_skinny_gemm_bias(x, M, K, w, N, nullptr, residual, res_rs, y, y_rs, status, stream);
}

extern "C" int coda_b200_skinny_gemm_bias(const void* x, int32_t M, int32_t K, const void* w, int32_t N, const void* bias,
                                          const void* residual, int64_t res_rs, void* y, int64_t y_rs,
                                          int32_t* status, coda_stream_t stream) {
  CODA_REQUIRE(coda_b200_skinny_gemm_supported(M, K, N), CODA_ERR_ARG,
               "skinny_gemm: needs 1..32 rows, K a multiple of 128 up to 4096, N a multiple of 64 (got %d x %d -> %d)", M, K, N);
  CODA_REQUIRE(x && w && y && (uintptr_t)x % 16 == 0 && (uintptr_t)w % 16 == 0 && (uintptr_t)y % 16 == 0 && y_rs % 8 == 0 && y_rs >= N,
               CODA_ERR_ARG, "skinny_gemm: null or misaligned pointer / output stride");
  CODA_REQUIRE(!residual || ((uintptr_t)residual % 16 == 0 && res_rs % 8 == 0 && res_rs >= N), CODA_ERR_ARG,
               "skinny_gemm: misaligned residual");
  CODA_REQUIRE(!bias || (uintptr_t)bias % 16 == 0, CODA_ERR_ARG, "skinny_gemm: misaligned bias");
  CUtensorMap xm, wm;
  CODA_REQUIRE(tmaps::plane_map(&xm, x, 1, M, K, SG_MAXM), CODA_ERR_LAUNCH, "skinny_gemm: cuTensorMapEncodeTiled failed");
  SkinnyParams p;
  p.M = M; p.N = N; p.K = K; p.res = (const bf16*)residual; p.res_rs = res_rs; p.bias = (const bf16*)bias;
  p.y = (bf16*)y; p.y_rs = y_rs; p.status = status;
  // The four-way split whenever an instance covers the shape with its clusters resident at once
  int cw = 0;
  const int bn = skinny4_plan(K, N, &cw);
  if (bn != 0) {
    if (cw == 8) return Skinny4<8, 8>::launch(xm, w, p, bn, (size_t)Skinny4Smem<8, 8>(K / 4).total + 1024, (cudaStream_t)stream);
    return Skinny4<12, 6>::launch(xm, w, p, bn, (size_t)Skinny4Smem<12, 6>(K / 4).total + 1024, (cudaStream_t)stream);
  }
  CODA_REQUIRE(!bias, CODA_ERR_LIMIT, "skinny_gemm: the bias epilogue needs the four-way kernel, which does not cover %d x %d -> %d here", M, K, N);
  CODA_REQUIRE(tmaps::plane_map(&wm, w, 1, N, K, SG_BN), CODA_ERR_LAUNCH, "skinny_gemm: cuTensorMapEncodeTiled failed");
  const size_t smem = (size_t)SkinnySmem(K / 2).total + 1024;
  static coda_device_once once;
  coda_on_first_use(once, [] {
    cudaFuncSetAttribute(skinny_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024);
  });
  cudaLaunchConfig_t lc = {};
  lc.gridDim = dim3(2, N / SG_BN, 1);
  lc.blockDim = dim3(SG_THREADS, 1, 1);
  lc.dynamicSmemBytes = smem;
  lc.stream = (cudaStream_t)stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
  lc.attrs = at; lc.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&lc, skinny_gemm_kernel, xm, wm, p);
  if (e != cudaSuccess) { coda_set_error("skinny_gemm: %s", cudaGetErrorString(e)); return CODA_ERR_LAUNCH; }
  return CODA_OK;
}

// ---- the chain: Y_A = X_A . W_A^T + R (phase A), Y_B = Y_A . W_B^T + bias (phase B), one launch ----------------------
namespace {
constexpr int CH_CW = 12, CH_STAGES = 5;
size_t chain_smem(int kq_max) { return (size_t)ChainSmem<CH_CW, CH_STAGES>(kq_max).total + 1024; }
// clusters of four CTAs of the chain kernel that are resident at once on the current device (0: unknown)
int chain_max_clusters(int kq_max) {
  static coda_device_once once;
  static int mc[64][3];                                  // by kq_max / 512 - 1 (K = 2048, 4096 in use)
  const int dev = coda_current_device();
  coda_on_first_use(once, [dev] {
    cudaFuncSetAttribute(skinny_gemm4_chain_kernel<CH_CW, CH_STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024);
    for (int k = 0; k < 3; ++k) {
      const int kq = 512 * (k + 1) <= 1024 ? 512 * (k + 1) : 1024;
      cudaLaunchConfig_t q = {};
      q.gridDim = dim3(S4_CL, 64, 1); q.blockDim = dim3((CH_CW + 1) * 32, 1, 1); q.dynamicSmemBytes = chain_smem(kq);
      cudaLaunchAttribute qa[1];
      qa[0].id = cudaLaunchAttributeClusterDimension;
      qa[0].val.clusterDim.x = S4_CL; qa[0].val.clusterDim.y = 1; qa[0].val.clusterDim.z = 1;
      q.attrs = qa; q.numAttrs = 1;
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, skinny_gemm4_chain_kernel<CH_CW, CH_STAGES>, &q) != cudaSuccess) { n = 0; cudaGetLastError(); }
      if (dev >= 0 && dev < 64) mc[dev][k] = n;
    }
  });
  if (dev < 0 || dev >= 64) return 0;
  return mc[dev][kq_max <= 512 ? 0 : 1];
}
// tile heights of the two phases such that the larger tile count still is one wave; false when a phase does not fit
bool chain_plan(int KA, int NA, int NB, int* bnA, int* bnB, int* clusters) {
  if (KA % 256 != 0 || NA % 256 != 0 || NA % 16 != 0 || NB % 16 != 0 || KA > 4096 || NA > 4096) return false;
  const int kq_max = (KA > NA ? KA : NA) / 4;
  if (kq_max / SG_BK > SG_XGROUP * SG_MAXXG) return false;
  const int mc = chain_max_clusters(kq_max);
  if (mc <= 0) return false;
  int a = ((NA + mc - 1) / mc + 15) / 16 * 16, b = ((NB + mc - 1) / mc + 15) / 16 * 16;
  if (a < 16) a = 16;
  if (b < 16) b = 16;
  if (a > 16 * CH_CW || b > 16 * CH_CW) return false;
  const int ca = (NA + a - 1) / a, cb = (NB + b - 1) / b;
  *bnA = a; *bnB = b; *clusters = ca > cb ? ca : cb;
  return *clusters <= mc;
}
}  // namespace

extern "C" int coda_b200_skinny_gemm_chain_supported(int32_t M, int32_t KA, int32_t NA, int32_t NB) {
  if (!(M >= 1 && M <= SG_MAXM && tmaps::available())) return 0;
  int a, b, c;
  return chain_plan(KA, NA, NB, &a, &b, &c) ? 1 : 0;
}

extern "C" int coda_b200_skinny_gemm_chain(const void* xA, int32_t M, int32_t KA, const void* wA, int32_t NA,
                                           const void* residualA, int64_t res_rs, void* yA,
                                           const void* wB, int32_t NB, const void* biasB, void* yB, int64_t yB_rs,
                                           uint32_t* gsync, int32_t* status, coda_stream_t stream) {
  int bnA = 0, bnB = 0, clusters = 0;
  CODA_REQUIRE(M >= 1 && M <= SG_MAXM && tmaps::available() && chain_plan(KA, NA, NB, &bnA, &bnB, &clusters), CODA_ERR_ARG,
               "skinny_gemm_chain: %d x %d -> %d -> %d is not covered on this device", M, KA, NA, NB);
  CODA_REQUIRE(xA && wA && yA && wB && yB && gsync, CODA_ERR_ARG, "skinny_gemm_chain: null pointer");
  const uintptr_t al = (uintptr_t)xA | (uintptr_t)wA | (uintptr_t)yA | (uintptr_t)wB | (uintptr_t)yB | (uintptr_t)residualA | (uintptr_t)biasB;
  CODA_REQUIRE(al % 16 == 0 && (uintptr_t)gsync % 8 == 0 && yB_rs % 8 == 0 && yB_rs >= NB && (!residualA || (res_rs % 8 == 0 && res_rs >= NA)),
               CODA_ERR_ARG, "skinny_gemm_chain: misaligned pointer or stride");
  CUtensorMap xmA, wmA, xmB, wmB;
  const bool ok = tmaps::plane_map(&xmA, xA, 1, M, KA, SG_MAXM) && tmaps::plane_map(&wmA, wA, 1, NA, KA, bnA) &&
                  tmaps::plane_map(&xmB, yA, 1, M, NA, SG_MAXM) && tmaps::plane_map(&wmB, wB, 1, NB, NA, bnB);
  CODA_REQUIRE(ok, CODA_ERR_LAUNCH, "skinny_gemm_chain: cuTensorMapEncodeTiled failed");
  SkinnyParams pA, pB;
  pA.M = M; pA.N = NA; pA.K = KA; pA.res = (const bf16*)residualA; pA.res_rs = res_rs; pA.bias = nullptr;
  pA.y = (bf16*)yA; pA.y_rs = NA; pA.status = status;
  pB.M = M; pB.N = NB; pB.K = NA; pB.res = nullptr; pB.res_rs = 0; pB.bias = (const bf16*)biasB;
  pB.y = (bf16*)yB; pB.y_rs = yB_rs; pB.status = status;
  const int kq_max = (KA > NA ? KA : NA) / 4;
  cudaLaunchConfig_t lc = {};
  lc.gridDim = dim3(S4_CL, clusters, 1);
  lc.blockDim = dim3((CH_CW + 1) * 32, 1, 1);
  lc.dynamicSmemBytes = chain_smem(kq_max);
  lc.stream = (cudaStream_t)stream;
  cudaLaunchAttribute at[2];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = S4_CL; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
  at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[1].val.programmaticStreamSerializationAllowed = 1;
  lc.attrs = at; lc.numAttrs = 2;
  cudaError_t e = cudaLaunchKernelEx(&lc, skinny_gemm4_chain_kernel<CH_CW, CH_STAGES>, xmA, wmA, pA, bnA, xmB, wmB, pB, bnB,
                                     (unsigned int*)gsync, kq_max);
  if (e != cudaSuccess) { coda_set_error("skinny_gemm_chain: %s", cudaGetErrorString(e)); return CODA_ERR_LAUNCH; }
  return CODA_OK;
}

// How the four-way kernel would cover a shape on the current device: tile height in weight rows (0: not covered) and
// the number of clusters of four CTAs it launches.
extern "C" int coda_b200_skinny_gemm_plan(int32_t K, int32_t N, int32_t* tile_rows, int32_t* clusters) {
  int cw = 0;
  const int bn = skinny4_plan(K, N, &cw);
  if (tile_rows) *tile_rows = bn;
  if (clusters) *clusters = bn ? (N + bn - 1) / bn : 0;
  return bn != 0;
}

// Whether coda_b200_skinny_gemm_bias can take a bias for this shape on the current device (the four-way kernel covers it).
extern "C" int coda_b200_skinny_gemm_bias_supported(int32_t M, int32_t K, int32_t N) {
  if (!coda_b200_skinny_gemm_supported(M, K, N)) return 0;
  int cw = 0;
  return skinny4_plan(K, N, &cw) != 0;
}
