// Y[M x N] = X[M x K] . W[N x K]^T (+ bias[N]) (+ R[M x N]), bf16 in / fp32 accumulate / bf16 out, for the few rows
// of a decode step (M <= 64 tokens): the fused [q | k | v | lambda | gate] input projection and the output
// projection of upstream attention.py:396-410,467-470,514 (`nn.Linear` weights, [out][in], used as they are), the
// latter with the decoder's residual added in the same pass.  With so few rows the GEMM is one pass over the weight
// matrix: 2*N*K bytes from HBM, and nothing else matters.
//
// Swapped operands on the 5th-generation tensor cores: the WEIGHT rows are the MMA's M (128 per tile), the tokens
// its N (32 or 64), so a tile's accumulator is 32 / 64 TMEM columns and no tensor work is spent on padding:
//     D[128 weight rows][tokens] += W_tile[128][64] . X[tokens][64]^T        tcgen05.mma, A and B K-major from smem
// Work split ("stream-K"): the tiles' k-blocks (64 columns of K each) are laid end to end, tile after tile, and cut
// into one equal contiguous run per SM, so every SM streams the same number of weight bytes whatever N is; a run
// that crosses a tile boundary is two segments with their own accumulators (TMEM is double-buffered).  A tile cut
// over several CTAs is summed without anybody waiting: each contributor leaves its fp32 partial tile in a global
// workspace and bumps the tile's counter; whoever arrives last adds the partials in a fixed order, applies bias /
// residual and writes the bf16 rows.  No clusters, no spinning.
// Per CTA: warp 0 = TMA producer (a ring of stages, each KPS weight boxes + KPS X boxes on one mbarrier; 128-byte
// swizzle), warp 1 = MMA issuer and TMEM owner, warps 2-5 = epilogue.  The weights do not depend on the kernel before
// this one on the stream, so with a programmatic dependent launch the producer fills the whole ring with weight boxes
// BEFORE griddepcontrol.wait; only the X boxes, the residual, the workspace and the stores wait for the predecessor.
// Every mbarrier wait is bounded (status word + CTA abort word).  No multicast anywhere.
#include "coda_common.cuh"
#include "tma_utils.cuh"
#include "tensor_maps.h"
#include <stdlib.h>

namespace {

constexpr int PG_BN = 128;           // weight rows per tile (MMA M)
constexpr int PG_BK = 64;            // elements per k-block (128 bytes: one swizzle row)
constexpr int PG_WBOX = PG_BN * 128; // bytes of a weight box
constexpr int PG_THREADS = 192;      // producer warp, MMA warp, four epilogue warps
constexpr int PG_CNT_BYTES = 4096;   // tile counters at the head of the workspace (up to 1024 tiles)

struct ProjParams {
  int M, N, K, nkb, tiles, maxc;     // nkb = K / 64; maxc = partial slots per tile
  const bf16* bias;                  // [N] or null
  const bf16* res; long long res_rs; // [M][N] or null
  bf16* y; long long y_rs;
  int* counters;                     // [tiles], zero between launches
  float* partials;                   // [tiles][maxc][NTOK][128]
  int* status;
};

using tma::smem_u32;

__device__ __forceinline__ void pg_tma_load(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
               ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(0) : "memory");
}
__device__ __forceinline__ void pg_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void pg_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void pg_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void pg_mma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void pg_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
               "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                 "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                 "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                 "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
               : "r"(taddr));
}
// K-major shared-memory operand, 128-byte swizzle (rows of 64 bf16, 8-row groups 1024 bytes apart), descriptor version 1
__device__ __forceinline__ uint64_t pg_desc(uint32_t addr) {
  return (uint64_t)((addr >> 4) & 0x3FFF) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// fp32 accumulate, bf16 x bf16, M = 128, N = n, both operands K-major
__device__ __forceinline__ constexpr uint32_t pg_idesc(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(PG_BN >> 4) << 24);
}

// Work of one CTA: a list of segments, each a k-range of one weight tile with its own accumulator.
//   tiles < CTAs: every CTA works on ONE tile; the tile's k-blocks are cut evenly over its `nparts` CTAs (the first
//                 G % T tiles get one CTA more than the others, so all G CTAs are used);
//   tiles >= CTAs: CTA g takes whole tiles g, g + G, ... one after the other.
struct Seg { int tile, kb0, kb1, part, nparts; };
__device__ __forceinline__ bool pg_seg(int idx, int g, int G, int T, int nkb, Seg& s) {
  if (T >= G) {
    s.tile = g + idx * G; s.kb0 = 0; s.kb1 = nkb; s.part = 0; s.nparts = 1;
    return s.tile < T;
  }
  if (idx > 0) return false;
  const int base = G / T, extra = G % T, big = extra * (base + 1);
  if (g < big) { s.tile = g / (base + 1); s.part = g % (base + 1); s.nparts = base + 1; }
  else { const int r = g - big; s.tile = extra + r / base; s.part = r % base; s.nparts = base; }
  s.kb0 = nkb * s.part / s.nparts;
  s.kb1 = nkb * (s.part + 1) / s.nparts;
  return true;
}

// NTOK = token columns of the MMA (32 or 64), STAGES = ring depth, KPS = k-blocks per stage.  A stage is one mbarrier
// phase; measured on B200, a phase costs some hundred cycles whatever it carries, so a stage holds several boxes.
template <int NTOK, int STAGES, int KPS>
__global__ void __launch_bounds__(PG_THREADS, 1)
proj_gemm_kernel(const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap wmap, ProjParams p) {
  constexpr int XBOX = NTOK * 128;
  constexpr int STAGE_BYTES = KPS * (PG_WBOX + XBOX);
  extern __shared__ unsigned char pg_raw[];
  unsigned char* smem = pg_raw + ((1024u - (smem_u32(pg_raw) & 1023u)) & 1023u);   // swizzled boxes need 1024-byte alignment
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;                   // [2] accumulator of a segment complete
  uint64_t* acc_empty = acc_full + 2;                    // [2] accumulator read out, may be overwritten
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  int* s_last = reinterpret_cast<int*>(tmem_slot + 1);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int G = gridDim.x, g = blockIdx.x;

  __shared__ int s_abort;                                // set by the first bounded wait of this CTA that expires
  int* const abortw = &s_abort;
  if (tid == 0) {
    s_abort = 0;
    for (int i = 0; i < STAGES; ++i) { tma::mbar_init(&full[i], 1); tma::mbar_init(&empty[i], 1); }
    for (int i = 0; i < 2; ++i) { tma::mbar_init(&acc_full[i], 1); tma::mbar_init(&acc_empty[i], 4); }
    tma::fence_barrier_init();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)(2 * NTOK)) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    pg_fence_before();
  }
  __syncthreads();
  pg_fence_after();
  const uint32_t tmem = *tmem_slot;
  // the kernel after this one on the stream may start its own prologue now
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  if (warp == 0) {
    // =========================== TMA producer ===========================
    if (lane == 0) {
      // The stages of all segments in order: stage n of the CTA = k-blocks [kb, kb + nb) of segment `si`.
      Seg sg; int si = 0, kb = 0; bool have = pg_seg(0, g, G, p.tiles, p.nkb, sg);
      if (have) kb = sg.kb0;
      auto next_stage = [&](int& tile, int& k0, int& nb) {
        while (have && kb >= sg.kb1) { have = pg_seg(++si, g, G, p.tiles, p.nkb, sg); if (have) kb = sg.kb0; }
        if (!have) return false;
        tile = sg.tile; k0 = kb; nb = sg.kb1 - kb < KPS ? sg.kb1 - kb : KPS; kb += nb;
        return true;
      };
      int tiles_[STAGES], k0s[STAGES], nbs[STAGES];
      int n = 0;
      // weights first: they are not produced by the predecessor kernel
      for (; n < STAGES && next_stage(tiles_[n], k0s[n], nbs[n]); ++n) {
        tma::mbar_expect_tx(&full[n], nbs[n] * (PG_WBOX + XBOX));
        for (int j = 0; j < nbs[n]; ++j) pg_tma_load(smem + n * STAGE_BYTES + j * PG_WBOX, &wmap, &full[n], (k0s[n] + j) * PG_BK, tiles_[n] * PG_BN);
      }
      asm volatile("griddepcontrol.wait;" ::: "memory");
      for (int i = 0; i < n; ++i)
        for (int j = 0; j < nbs[i]; ++j) pg_tma_load(smem + i * STAGE_BYTES + KPS * PG_WBOX + j * XBOX, &xmap, &full[i], (k0s[i] + j) * PG_BK, 0);
      int tile, k0, nb;
      for (int i = n; next_stage(tile, k0, nb); ++i) {
        const int st = i % STAGES;
        tma::mbar_wait(&empty[st], ((i / STAGES) - 1) & 1, p.status, 31, abortw);
        tma::mbar_expect_tx(&full[st], nb * (PG_WBOX + XBOX));
        for (int j = 0; j < nb; ++j) {
          pg_tma_load(smem + st * STAGE_BYTES + j * PG_WBOX, &wmap, &full[st], (k0 + j) * PG_BK, tile * PG_BN);
          pg_tma_load(smem + st * STAGE_BYTES + KPS * PG_WBOX + j * XBOX, &xmap, &full[st], (k0 + j) * PG_BK, 0);
        }
      }
    }
  } else if (warp == 1) {
    // =========================== MMA issuer ===========================
    if (lane == 0) {
      constexpr uint32_t IDESC = pg_idesc(NTOK);
      Seg sg;
      int i = 0;
      for (int seg = 0; pg_seg(seg, g, G, p.tiles, p.nkb, sg); ++seg) {
        if (seg >= 2) { tma::mbar_wait(&acc_empty[seg & 1], ((seg >> 1) - 1) & 1, p.status, 34, abortw); pg_fence_after(); }
        const uint32_t dcol = tmem + (uint32_t)((seg & 1) * NTOK);
        for (int kb = sg.kb0; kb < sg.kb1; kb += KPS, ++i) {
          const int st = i % STAGES;
          const int nb = sg.kb1 - kb < KPS ? sg.kb1 - kb : KPS;
          tma::mbar_wait(&full[st], (i / STAGES) & 1, p.status, 32, abortw);
          pg_fence_after();
          for (int j = 0; j < nb; ++j) {
            const uint32_t wbase = smem_u32(smem + st * STAGE_BYTES + j * PG_WBOX);
            const uint32_t xbase = smem_u32(smem + st * STAGE_BYTES + KPS * PG_WBOX + j * XBOX);
#pragma unroll
            for (int kk = 0; kk < PG_BK / 16; ++kk)
              pg_mma(dcol, pg_desc(wbase + kk * 32), pg_desc(xbase + kk * 32), IDESC, (kb > sg.kb0 || j > 0 || kk > 0) ? 1u : 0u);
          }
          pg_commit(&empty[st]);                          // the stage is free once these MMAs have read it
        }
        pg_commit(&acc_full[seg & 1]);
      }
    }
  } else {
    // =========================== epilogue ===========================
    asm volatile("griddepcontrol.wait;" ::: "memory");   // residual, workspace and output follow the predecessor
    const int quarter = warp & 3;                         // TMEM lane quarter this warp may touch
    const int row = quarter * 32 + lane;                  // weight row inside the tile
    const int et = tid - 64;                              // 0..127 among the epilogue threads
    Seg sg;
    for (int seg = 0; pg_seg(seg, g, G, p.tiles, p.nkb, sg); ++seg) {
      const int tile = sg.tile;
      const int buf = seg & 1;
      const int nc = sg.nparts;                            // contributors of this tile, in k order
      const int n = tile * PG_BN + row;
      const int nn = n < p.N ? n : 0;                      // rows past N read row 0 and store nothing
      // bias and residual do not depend on the accumulator: requested before the wait for it
      const bool has_res = p.res != nullptr;
      const float bias = p.bias != nullptr ? __bfloat162float(p.bias[nn]) : 0.f;
      float rv[NTOK];
#pragma unroll
      for (int t = 0; t < NTOK; ++t) {
        const int tt = t < p.M ? t : 0;                    // rows past M re-read row 0: no branch around the load
        rv[t] = has_res ? __bfloat162float(p.res[(long long)tt * p.res_rs + nn]) : 0.f;
      }
      tma::mbar_wait(&acc_full[buf], (seg >> 1) & 1, p.status, 33, abortw);
      pg_fence_after();
      float acc[NTOK];
#pragma unroll
      for (int c = 0; c < NTOK / 32; ++c) {
        uint32_t v[32];
        pg_ld32(tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * NTOK + c * 32), v);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int t = 0; t < 32; ++t) acc[c * 32 + t] = __uint_as_float(v[t]);
      }
      pg_fence_before();
      __syncwarp();
      if (lane == 0) tma::mbar_arrive(&acc_empty[buf]);   // the MMA warp may reuse this accumulator
      bool reduce = true;
      if (nc > 1) {
        float* slot = p.partials + ((long long)tile * p.maxc + sg.part) * (NTOK * PG_BN);
#pragma unroll
        for (int t = 0; t < NTOK; ++t) __stcg(slot + t * PG_BN + row, acc[t]);     // all token columns: no branches, the stores pipeline
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (et == 0) {
          const int old = atomicAdd(&p.counters[tile], 1);
          *s_last = (old == nc - 1) ? 1 : 0;
          if (old == nc - 1) p.counters[tile] = 0;        // ready for the next launch
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        reduce = *s_last != 0;
        if (reduce) {
          __threadfence();
          const float* base = p.partials + (long long)tile * p.maxc * (NTOK * PG_BN) + row;
#pragma unroll
          for (int t = 0; t < NTOK; ++t) acc[t] = 0.f;
          // fixed order c = 0, 1, ...: the sum does not depend on who came last.  Two slots are requested per round
          // trip, every load of a round in flight before the first add.
          for (int c = 0; c < nc; c += 2) {
            const float* s0 = base + (long long)c * (NTOK * PG_BN);
            const float* s1 = base + (long long)(c + 1 < nc ? c + 1 : c) * (NTOK * PG_BN);
            float v0[NTOK], v1[NTOK];
#pragma unroll
            for (int t = 0; t < NTOK; ++t) { v0[t] = __ldcg(s0 + t * PG_BN); v1[t] = __ldcg(s1 + t * PG_BN); }
            const float keep = c + 1 < nc ? 1.f : 0.f;
#pragma unroll
            for (int t = 0; t < NTOK; ++t) { acc[t] += v0[t]; acc[t] += keep * v1[t]; }
          }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");    // s_last is rewritten by the next segment
      }
      if (reduce && n < p.N) {
#pragma unroll
        for (int t = 0; t < NTOK; ++t) {
          float out = bf16_round(acc[t] + bias);
          if (has_res) out = bf16_round(out + rv[t]);
          if (t < p.M) p.y[(long long)t * p.y_rs + n] = __float2bfloat16_rn(out);
        }
      }
    }
  }
  __syncthreads();
  if (warp == 1) {
    pg_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)(2 * NTOK)) : "memory");
  }
}

struct ProjGeometry { int tiles, nkb, grid, maxc; };
static ProjGeometry proj_geometry(int K, int N, int num_sms) {
  ProjGeometry q;
  q.tiles = (N + PG_BN - 1) / PG_BN;
  q.nkb = K / PG_BK;
  if (q.tiles >= num_sms) { q.grid = num_sms; q.maxc = 1; return q; }
  const long long U = (long long)q.tiles * q.nkb;
  q.grid = U < num_sms ? (int)U : num_sms;              // never more parts than a tile has k-blocks
  q.maxc = q.grid / q.tiles + (q.grid % q.tiles ? 1 : 0);
  return q;
}

template <int NTOK, int STAGES, int KPS>
int launch_proj(const CUtensorMap& xm, const CUtensorMap& wm, ProjParams& p, void* workspace, cudaStream_t s) {
  constexpr size_t SMEM = (size_t)STAGES * KPS * (PG_WBOX + NTOK * 128) + (2 * STAGES + 4) * 8 + 16 + 1024;
  static_assert(SMEM <= 227 * 1024, "ring does not fit in shared memory");
  static coda_device_once once;
  const int num_sms = coda_on_first_use(once, [] {
    cudaFuncSetAttribute(proj_gemm_kernel<NTOK, STAGES, KPS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM);
  });
  const ProjGeometry q = proj_geometry(p.K, p.N, num_sms);
  CODA_REQUIRE((size_t)q.tiles * 4 <= PG_CNT_BYTES, CODA_ERR_LIMIT, "proj_gemm: %d weight tiles (at most %d)", q.tiles, PG_CNT_BYTES / 4);
  p.tiles = q.tiles; p.nkb = q.nkb; p.maxc = q.maxc;
  p.counters = reinterpret_cast<int*>(workspace);
  p.partials = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(workspace) + PG_CNT_BYTES);
  cudaLaunchConfig_t lc = {};
  lc.gridDim = dim3(q.grid, 1, 1);
  lc.blockDim = dim3(PG_THREADS, 1, 1);
  lc.dynamicSmemBytes = SMEM;
  lc.stream = s;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  lc.attrs = at;
  lc.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&lc, proj_gemm_kernel<NTOK, STAGES, KPS>, xm, wm, p);
  if (e != cudaSuccess) { coda_set_error("proj_gemm: %s", cudaGetErrorString(e)); cudaGetLastError(); return CODA_ERR_LAUNCH; }
  return CODA_OK;
}

}  // namespace

extern "C" int coda_b200_proj_gemm_supported(int32_t M, int32_t K, int32_t N) {
  return M >= 1 && M <= 64 && K >= PG_BK && K % PG_BK == 0 && N >= 1 && (N + PG_BN - 1) / PG_BN * 4 <= PG_CNT_BYTES &&
         tmaps::available();
}

extern "C" int64_t coda_b200_proj_gemm_workspace_bytes(int32_t M, int32_t K, int32_t N) {
  if (!(M >= 1 && M <= 64 && K >= PG_BK && K % PG_BK == 0 && N >= 1)) return -1;
  // sized for any SM count: a tile is never cut into more pieces than it has k-blocks, nor than 1 + k-blocks per shortest run
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) {
    cudaGetLastError();
    sms = 148;
  }
  const ProjGeometry q = proj_geometry(K, N, sms);
  const int ntok = M <= 32 ? 32 : 64;
  return (int64_t)PG_CNT_BYTES + (int64_t)q.tiles * q.maxc * ntok * PG_BN * 4;
}

extern "C" int coda_b200_proj_gemm(const void* x, int64_t x_rs, int32_t M, int32_t K, const void* w, int32_t N, const void* bias,
                                   const void* residual, int64_t res_rs, void* y, int64_t y_rs, void* workspace,
                                   int32_t* status, coda_stream_t stream) {
  CODA_REQUIRE(x && w && y && workspace, CODA_ERR_ARG, "proj_gemm: null pointer");
  CODA_REQUIRE(coda_b200_proj_gemm_supported(M, K, N), CODA_ERR_ARG,
               "proj_gemm: needs 1 <= M <= 64, K a multiple of 64 (M=%d K=%d N=%d)", M, K, N);
  CODA_REQUIRE(((uintptr_t)x | (uintptr_t)w | (uintptr_t)workspace) % 16 == 0, CODA_ERR_ARG, "proj_gemm: x, w and workspace must be 16-byte aligned");
  CODA_REQUIRE(y_rs >= N && (residual == nullptr || res_rs >= N) && x_rs >= K && x_rs % 8 == 0, CODA_ERR_ARG,
               "proj_gemm: row strides shorter than a row (or x's not a multiple of 8 elements)");
  const int ntok = M <= 32 ? 32 : 64;
  CUtensorMap xm, wm;
  CODA_REQUIRE(tmaps::matrix_map(&xm, x, M, K, x_rs, ntok) && tmaps::matrix_map(&wm, w, N, K, K, PG_BN), CODA_ERR_LAUNCH,
               "proj_gemm: cuTensorMapEncodeTiled failed");
  ProjParams p;
  p.M = M; p.N = N; p.K = K; p.bias = (const bf16*)bias; p.res = (const bf16*)residual; p.res_rs = res_rs;
  p.y = (bf16*)y; p.y_rs = y_rs; p.status = status;
  if (ntok == 64) return launch_proj<64, 4, 2>(xm, wm, p, workspace, (cudaStream_t)stream);
  return launch_proj<32, 5, 2>(xm, wm, p, workspace, (cudaStream_t)stream);
}
