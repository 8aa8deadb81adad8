// Y[M x N] = X[M x K] . W[N x K]^T (+ bias[N]) (+ R[M x N]), bf16 in / fp32 accumulate / bf16 out, for the few rows
// of a decode step (M <= 64 tokens): the fused [q | k | v | lambda | gate] input projection and the output
// projection of upstream attention.py:396-410,467-470,514 (`nn.Linear` weights, [out][in]), the latter with the
// decoder's residual added in the same pass.  With so few rows the GEMM is one pass over the weight matrix:
// 2*N*K bytes from HBM, and nothing else matters.
//
// Swapped operands on the 5th-generation tensor cores: the WEIGHT rows are the MMA's M (128 per tile), the tokens
// its N (32 or 64), so a tile's accumulator is 32 / 64 TMEM columns and no tensor work is spent on padding:
//     D[128 weight rows][tokens] += W_tile[128][64] . X[tokens][64]^T        tcgen05.mma, A and B K-major from smem
// Grid: one cluster per 128-row weight tile; the cluster's S CTAs split K (S chosen so that tiles x S fills the
// SMs once).  Per CTA: warp 0 = TMA producer (a ring of {16 KB weight box, X box} stages, 128-byte swizzle), warp
// 1 = MMA issuer and TMEM owner, warps 2-5 = epilogue.  The weights do not depend on the kernel before this one
// on the stream, so with a programmatic dependent launch the producer fills the whole ring with weight boxes BEFORE
// griddepcontrol.wait and only the X boxes, the residual and the stores wait for the predecessor.
// Split-K reduction inside the cluster: every CTA leaves its fp32 partial tile in its own shared memory, one
// hardware cluster barrier, then CTA r sums tokens r, r+S, ... over all CTAs through distributed shared memory, adds
// bias / residual and writes bf16 rows (128 consecutive outputs per token: coalesced).
// Every mbarrier wait is bounded (status word + CTA abort word); cluster barriers are hardware barriers among
// co-scheduled CTAs.  No multicast anywhere.
#include "coda_common.cuh"
#include "tma_utils.cuh"
#include "tensor_maps.h"

namespace {

constexpr int PG_BN = 128;           // weight rows per tile (MMA M)
constexpr int PG_BK = 64;            // elements per stage along K (128 bytes: one swizzle row)
constexpr int PG_WBOX = PG_BN * 128; // bytes of a weight box
constexpr int PG_THREADS = 192;      // producer warp, MMA warp, four epilogue warps
constexpr int PG_MAX_SPLIT = 8;      // portable cluster size

struct ProjParams {
  int M, N, K, nkb;                  // nkb = K / 64
  const bf16* bias;                  // [N] or null
  const bf16* res; long long res_rs; // [M][N] or null
  bf16* y; long long y_rs;
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
__device__ __forceinline__ uint32_t pg_mapa(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ float pg_ld_cluster(uint32_t addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ void pg_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// NTOK = token columns of the MMA (32 or 64), STAGES = ring depth
template <int NTOK, int STAGES>
__global__ void __launch_bounds__(PG_THREADS, 1)
proj_gemm_kernel(const __grid_constant__ CUtensorMap xmap, const __grid_constant__ CUtensorMap wmap, ProjParams p) {
  constexpr int XBOX = NTOK * 128;
  constexpr int STAGE_BYTES = PG_WBOX + XBOX;
  extern __shared__ unsigned char pg_raw[];
  unsigned char* smem = pg_raw + ((1024u - (smem_u32(pg_raw) & 1023u)) & 1023u);   // swizzled boxes need 1024-byte alignment
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
  float* part = reinterpret_cast<float*>(smem);          // [NTOK][128] fp32 partial tile; reuses the ring once the MMAs are done

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int S = gridDim.x, rank = blockIdx.x;            // cluster = the S CTAs of one weight tile (cluster dims (S,1,1))
  const int n0 = blockIdx.y * PG_BN;
  const int kb0 = (int)(((long long)p.nkb * rank) / S), kb1 = (int)(((long long)p.nkb * (rank + 1)) / S);
  const int nkb = kb1 - kb0;

  __shared__ int s_abort;                                // set by the first bounded wait of this CTA that expires
  int* const abortw = &s_abort;
  if (tid == 0) {
    s_abort = 0;
    for (int i = 0; i < STAGES; ++i) { tma::mbar_init(&full[i], 1); tma::mbar_init(&empty[i], 1); }
    tma::mbar_init(acc_full, 1);
    tma::fence_barrier_init();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)NTOK) : "memory");
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
      const int first = nkb < STAGES ? nkb : STAGES;
      // weights first: they are not produced by the predecessor kernel
      for (int i = 0; i < first; ++i) {
        tma::mbar_expect_tx(&full[i], STAGE_BYTES);
        pg_tma_load(smem + i * STAGE_BYTES, &wmap, &full[i], (kb0 + i) * PG_BK, n0);
      }
      asm volatile("griddepcontrol.wait;" ::: "memory");
      for (int i = 0; i < first; ++i)
        pg_tma_load(smem + i * STAGE_BYTES + PG_WBOX, &xmap, &full[i], (kb0 + i) * PG_BK, 0);
      for (int i = first; i < nkb; ++i) {
        const int st = i % STAGES;
        tma::mbar_wait(&empty[st], ((i / STAGES) - 1) & 1, p.status, 31, abortw);
        tma::mbar_expect_tx(&full[st], STAGE_BYTES);
        pg_tma_load(smem + st * STAGE_BYTES, &wmap, &full[st], (kb0 + i) * PG_BK, n0);
        pg_tma_load(smem + st * STAGE_BYTES + PG_WBOX, &xmap, &full[st], (kb0 + i) * PG_BK, 0);
      }
    }
  } else if (warp == 1) {
    // =========================== MMA issuer ===========================
    if (lane == 0) {
      constexpr uint32_t IDESC = pg_idesc(NTOK);
      for (int i = 0; i < nkb; ++i) {
        const int st = i % STAGES;
        tma::mbar_wait(&full[st], (i / STAGES) & 1, p.status, 32, abortw);
        pg_fence_after();
        const uint32_t wbase = smem_u32(smem + st * STAGE_BYTES), xbase = wbase + PG_WBOX;
#pragma unroll
        for (int kk = 0; kk < PG_BK / 16; ++kk)
          pg_mma(tmem, pg_desc(wbase + kk * 32), pg_desc(xbase + kk * 32), IDESC, (i > 0 || kk > 0) ? 1u : 0u);
        pg_commit(&empty[st]);                            // the stage is free once these MMAs have read it
      }
      pg_commit(acc_full);
    }
  } else {
    // =========================== epilogue ===========================
    asm volatile("griddepcontrol.wait;" ::: "memory");   // residual reads and output writes follow the predecessor
    const int quarter = warp & 3;                         // TMEM lane quarter this warp may touch
    const int row = quarter * 32 + lane;                  // weight row inside the tile
    if (nkb > 0) {
      tma::mbar_wait(acc_full, 0, p.status, 33, abortw);
      pg_fence_after();
#pragma unroll
      for (int c = 0; c < NTOK / 32; ++c) {
        uint32_t v[32];
        pg_ld32(tmem + ((uint32_t)(quarter * 32) << 16) + c * 32, v);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int t = 0; t < 32; ++t) part[(c * 32 + t) * PG_BN + row] = __uint_as_float(v[t]);
      }
      pg_fence_before();
    } else {
#pragma unroll
      for (int t = 0; t < NTOK; ++t) part[t * PG_BN + row] = 0.f;
    }
  }
  // every CTA of the cluster has its partial tile in shared memory
  __syncwarp();
  pg_cluster_sync();
  if (warp >= 2) {
    const int row = (warp & 3) * 32 + lane, n = n0 + row;
    if (n < p.N) {
      const float bias = p.bias != nullptr ? __bfloat162float(p.bias[n]) : 0.f;
      const uint32_t mine = smem_u32(part);
      for (int t = rank; t < p.M; t += S) {
        float acc = 0.f;
        for (int c = 0; c < S; ++c) acc += pg_ld_cluster(pg_mapa(mine, (uint32_t)c) + (uint32_t)(t * PG_BN + row) * 4u);
        float out = bf16_round(acc + bias);
        if (p.res != nullptr) out = bf16_round(out + __bfloat162float(p.res[(long long)t * p.res_rs + n]));
        p.y[(long long)t * p.y_rs + n] = __float2bfloat16_rn(out);
      }
    }
  }
  // nobody leaves while a peer may still read its partial tile
  __syncwarp();
  pg_cluster_sync();
  if (warp == 1) {
    pg_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)NTOK) : "memory");
  }
}

template <int NTOK, int STAGES>
int launch_proj(const CUtensorMap& xm, const CUtensorMap& wm, const ProjParams& p, cudaStream_t s) {
  constexpr size_t SMEM = (size_t)STAGES * (PG_WBOX + NTOK * 128) + (2 * STAGES + 1) * 8 + 16 + 1024;
  static_assert(SMEM <= 227 * 1024, "ring does not fit in shared memory");
  static_assert((size_t)NTOK * PG_BN * 4 <= (size_t)STAGES * (PG_WBOX + NTOK * 128), "partial tile must fit in the ring");
  static coda_device_once once;
  const int num_sms = coda_on_first_use(once, [] {
    cudaFuncSetAttribute(proj_gemm_kernel<NTOK, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM);
  });
  const int tiles = (p.N + PG_BN - 1) / PG_BN;
  int split = num_sms / tiles;                         // tiles x split CTAs fill the SMs once
  if (split > PG_MAX_SPLIT) split = PG_MAX_SPLIT;
  if (split > p.nkb) split = p.nkb;
  if (split < 1) split = 1;
  cudaLaunchConfig_t lc = {};
  lc.gridDim = dim3(split, tiles, 1);
  lc.blockDim = dim3(PG_THREADS, 1, 1);
  lc.dynamicSmemBytes = SMEM;
  lc.stream = s;
  cudaLaunchAttribute at[2];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = split; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
  at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[1].val.programmaticStreamSerializationAllowed = 1;
  lc.attrs = at;
  lc.numAttrs = 2;
  cudaError_t e = cudaLaunchKernelEx(&lc, proj_gemm_kernel<NTOK, STAGES>, xm, wm, p);
  if (e != cudaSuccess) { coda_set_error("proj_gemm: %s", cudaGetErrorString(e)); cudaGetLastError(); return CODA_ERR_LAUNCH; }
  return CODA_OK;
}

}  // namespace

extern "C" int coda_b200_proj_gemm_supported(int32_t M, int32_t K, int32_t N) {
  return M >= 1 && M <= 64 && K >= PG_BK && K % PG_BK == 0 && N >= 1 && tmaps::available();
}

extern "C" int coda_b200_proj_gemm(const void* x, int64_t x_rs, int32_t M, int32_t K, const void* w, int32_t N, const void* bias,
                                   const void* residual, int64_t res_rs, void* y, int64_t y_rs, int32_t* status,
                                   coda_stream_t stream) {
  CODA_REQUIRE(x && w && y, CODA_ERR_ARG, "proj_gemm: null pointer");
  CODA_REQUIRE(coda_b200_proj_gemm_supported(M, K, N), CODA_ERR_ARG,
               "proj_gemm: needs 1 <= M <= 64, K a multiple of 64 (M=%d K=%d N=%d)", M, K, N);
  CODA_REQUIRE(((uintptr_t)x | (uintptr_t)w) % 16 == 0, CODA_ERR_ARG, "proj_gemm: x and w must be 16-byte aligned");
  CODA_REQUIRE(y_rs >= N && (residual == nullptr || res_rs >= N) && x_rs >= K && x_rs % 8 == 0, CODA_ERR_ARG,
               "proj_gemm: row strides shorter than a row (or x's not a multiple of 8 elements)");
  const int ntok = M <= 32 ? 32 : 64;
  CUtensorMap xm, wm;
  CODA_REQUIRE(tmaps::matrix_map(&xm, x, M, K, x_rs, ntok) && tmaps::matrix_map(&wm, w, N, K, K, PG_BN), CODA_ERR_LAUNCH,
               "proj_gemm: cuTensorMapEncodeTiled failed");
  ProjParams p;
  p.M = M; p.N = N; p.K = K; p.nkb = K / PG_BK; p.bias = (const bf16*)bias; p.res = (const bf16*)residual; p.res_rs = res_rs;
  p.y = (bf16*)y; p.y_rs = y_rs; p.status = status;
  return ntok == 32 ? launch_proj<32, 10>(xm, wm, p, (cudaStream_t)stream) : launch_proj<64, 8>(xm, wm, p, (cudaStream_t)stream);
}
