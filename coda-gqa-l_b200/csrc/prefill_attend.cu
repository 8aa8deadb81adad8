// Chunked-prefill differential attention on the 5th-generation tensor cores (tcgen05 + TMEM), bf16.
//
// One CTA = one (state, query head, 128-row query tile) and BOTH streams: signal Q and theta-rotated noise Q
// share every K/V tile.  Keys are the layer's Lbuf slots (masked by `allowed`) followed by the block's own
// tokens (causal).  Per 128-key tile and stream:
//     S = Q . K^T          tcgen05.mma  M=128 N=128 K=Dh   A, B from shared memory, S in TMEM
//     P = exp2(S - m)      softmax warps: tcgen05.ld, lazy-rescaled online softmax, bf16 P written back over S
//     O += P . V           tcgen05.mma  M=128 N=Dh  K=128  A = P straight from TMEM, B = V from shared memory
// Warp roles: warps 0-3 = softmax / correction / epilogue of the signal stream, warps 4-7 = the same for the
// noise stream (one thread per query row, the whole row of S in registers: setmaxnreg gives these two
// warpgroups 208 registers), warp 8 = TMA producer (cp.async.bulk.tensor, 128-byte swizzle, 2-stage ring of
// 128-key K/V tiles), warp 9 = MMA issuer and TMEM owner.  The two streams ping-pong on the
// tensor core: while one stream is in softmax the other's P.V and next Q.K^T run.  Keeping P in TMEM halves
// the shared-memory operand traffic of P.V and N=128 tiles keep Q.K^T at the operand-bandwidth limit.
// TMEM map (512 columns): S_sig 0..127 (P_sig aliases 0..63), S_noise 128..255, O_sig 256.., O_noise 256+Dh..
// Epilogue: O/l per stream, sig - lambda*noise, optional RMSNorm over Dh, bf16 rows written in the (B, L, H*Dh)
// layout the output projection reads.  All mbarrier waits are bounded (status word, no hang, TMEM is freed).
#include "coda_common.cuh"
#include "tma_utils.cuh"
#include "tensor_maps.h"

namespace {

constexpr int PF_BM = 128;       // query rows per CTA
constexpr int PF_BN = 128;       // keys per tile
// Register split after launch (setmaxnreg): the two softmax warpgroups grow, the third warpgroup shrinks.  A
// warpgroup that asks for more than the CTA's pool (threads x registers at launch) can give waits forever, so the
// launcher checks the sum against the kernel's compiled register count and refuses to launch otherwise.
constexpr int PF_REGS_SOFTMAX = 208, PF_REGS_AUX = 72;
constexpr int PF_REGS_TOTAL = 256 * PF_REGS_SOFTMAX + 128 * PF_REGS_AUX;
constexpr int PF_THREADS = 384;  // warps 0-3 / 4-7: softmax of the signal / noise stream, 8: TMA, 9: MMA issuer, 10-11 idle
constexpr int PF_STAGES = 2;     // K/V tiles in flight
constexpr float PF_RESCALE_GAP = 8.0f;   // log2 units the running max may lag before O is rescaled

struct PrefillParams {
  int B, H, Hkv, Lbuf, blk, t0, mask_unused, norm_full;
  float eps, scale_log2;
  const float* lam; long long lam_bs, lam_rs;
  const uint8_t* allowed;
  const bf16* norm_w;
  bf16* out; long long out_bs, out_rs;
  int* status;
};

using tma::smem_u32;

__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
               ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
               ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}

// ---- tcgen05 wrappers ----
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc]
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem desc]
__device__ __forceinline__ void tc_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
               "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                 "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                 "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                 "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
               : "r"(taddr));
}
__device__ __forceinline__ void tc_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
               "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
               ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                 "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
                 "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
                 "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
               : "memory");
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                 "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
               : "r"(taddr));
}
__device__ __forceinline__ void tc_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
               ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                 "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
               : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor, 128-byte swizzle, version 1 (Blackwell).  K-major operands (rows of 64
// bf16 = 128 bytes, 8-row groups 1024 bytes apart): lbo unused (1), sbo = 1024.  MN-major operands (rows are
// the K index, 64 MN elements per 128-byte row): lbo = distance between 64-element MN groups, sbo = 1024.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  return (uint64_t)((addr >> 4) & 0x3FFF) | ((uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16) |
         ((uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor: fp32 accumulate, bf16 x bf16, M = 128, N = n, A K-major, B K-major or MN-major.
__device__ __forceinline__ constexpr uint32_t instr_desc(int n, bool b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn_major ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(PF_BM >> 4) << 24);
}
// 2^x for x <= 0 on the special-function unit (one MUFU op).
__device__ __forceinline__ float ex2_mufu(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Packed fp32 pairs (one instruction for two lanes of a register pair) and the three-input maximum.
__device__ __forceinline__ uint64_t pk64(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpk64(uint64_t v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t add2_rm(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rm.ftz.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
// 2^x for a pair of arguments on the FMA / integer pipes (x = n + f, n = floor(x) left in the low mantissa bits
// by a round-down add of 1.5 * 2^23; 2^f by a cubic, relative error < 1e-4, far below the bf16 rounding of P;
// n added into the exponent field).  The special-function unit delivers one warp of exponentials per 8 cycles
// per scheduler; a third of the exponentials go this way so that neither pipe bounds the softmax.
__device__ __forceinline__ void ex2_poly2(float x0, float x1, float& y0, float& y1) {
  const uint64_t x = pk64(fmaxf(x0, -127.0f), fmaxf(x1, -127.0f));
  const uint64_t magic = pk64(12582912.0f, 12582912.0f), nmagic = pk64(-12582912.0f, -12582912.0f);
  const uint64_t t = add2_rm(x, magic);
  const uint64_t fl = add2(t, nmagic);                           // floor(x), exact
  const uint64_t mone = pk64(-1.0f, -1.0f);
  const uint64_t f = fma2(fl, mone, x);                          // x - floor(x), exact
  uint64_t r = fma2(f, pk64(0.077119089663028717f, 0.077119089663028717f), pk64(0.227564394474029541f, 0.227564394474029541f));
  r = fma2(r, f, pk64(0.695146143436431885f, 0.695146143436431885f));
  r = fma2(r, f, pk64(1.0f, 1.0f));
  float r0, r1, t0, t1;
  unpk64(r, r0, r1);
  unpk64(t, t0, t1);
  y0 = __int_as_float(__float_as_int(r0) + (__float_as_int(t0) << 23));
  y1 = __int_as_float(__float_as_int(r1) + (__float_as_int(t1) << 23));
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}
__device__ __forceinline__ void bar_softmax_all() { asm volatile("bar.sync 1, 256;" ::: "memory"); }
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

template <int DH>
__global__ void __launch_bounds__(PF_THREADS, 1)
prefill_attend_kernel(const __grid_constant__ CUtensorMap qmap, const __grid_constant__ CUtensorMap qnmap,
                      const __grid_constant__ CUtensorMap kpmap, const __grid_constant__ CUtensorMap vpmap,
                      const __grid_constant__ CUtensorMap kbmap, const __grid_constant__ CUtensorMap vbmap,
                      PrefillParams p) {
  constexpr int HALVES = DH / 64;                 // 64-element (128-byte) column groups per row
  constexpr int Q_HALF = PF_BM * 128;             // bytes of one Q half tile
  constexpr int Q_BYTES = HALVES * Q_HALF;
  constexpr int KV_HALF = PF_BN * 128;
  constexpr int KV_BYTES = HALVES * KV_HALF;      // one K (or V) tile
  constexpr int KSTEPS_QK = DH / 16;
  constexpr int KSTEPS_PV = PF_BN / 16;
  constexpr uint32_t TM_SN = 128, TM_OS = 256, TM_ON = 256 + DH;   // TMEM column offsets (S_sig at 0)

  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  unsigned char* sQs = smem;
  unsigned char* sQn = sQs + Q_BYTES;
  unsigned char* sK = sQn + Q_BYTES;               // [PF_STAGES][KV_BYTES]
  unsigned char* sV = sK + PF_STAGES * KV_BYTES;   // [PF_STAGES][KV_BYTES]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + PF_STAGES * KV_BYTES);
  uint64_t* q_full = bars;                          // 1
  uint64_t* kv_full = bars + 1;                     // PF_STAGES
  uint64_t* kv_empty = kv_full + PF_STAGES;         // PF_STAGES
  uint64_t* s_full = kv_empty + PF_STAGES;          // [stream]
  uint64_t* p_full = s_full + 2;                    // [stream]
  uint64_t* pv_done = p_full + 2;                   // [stream]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pv_done + 2);
  uint32_t* sMask = tmem_slot + 2;                  // visibility bits of the prefix slots, 32 per word

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int r0 = blockIdx.x * PF_BM, h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.H / p.Hkv);
  const int NP = (p.Lbuf + PF_BN - 1) / PF_BN;                                   // prefix tiles
  const int last_row = min(r0 + PF_BM, p.blk) - 1;
  const int NB = last_row / PF_BN + 1;                                            // block tiles (causal limit)
  const int NT = NP + NB;

  __shared__ int s_abort;                          // set by the first bounded wait of this CTA that expires
  int* const abortw = &s_abort;
  if (tid == 0) {
    s_abort = 0;
    tma::mbar_init(q_full, 1);
    for (int i = 0; i < PF_STAGES; ++i) { tma::mbar_init(&kv_full[i], 1); tma::mbar_init(&kv_empty[i], 1); }
    for (int i = 0; i < 2; ++i) { tma::mbar_init(&s_full[i], 1); tma::mbar_init(&p_full[i], 4); tma::mbar_init(&pv_done[i], 1); }
    tma::fence_barrier_init();
  }
  if (warp == 9) {                                   // TMEM: all 512 columns, owned by the MMA warp
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    tc_fence_before();
  }
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  // Registers follow the roles, per warpgroup: a softmax thread keeps a whole row of S (128 values) in registers.
  if (warp >= 8) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(PF_REGS_AUX));
  if (warp == 8) {
    // =========================== TMA producer ===========================
    if (lane == 0) {
      tma::mbar_expect_tx(q_full, 2 * Q_BYTES);
#pragma unroll
      for (int hf = 0; hf < HALVES; ++hf) {
        tma_load_4d(sQs + hf * Q_HALF, &qmap, q_full, hf * 64, h, p.t0 + r0, b);
        tma_load_4d(sQn + hf * Q_HALF, &qnmap, q_full, hf * 64, h, p.t0 + r0, b);
      }
      for (int j = 0; j < NT; ++j) {
        const int st = j % PF_STAGES;
        if (j >= PF_STAGES) tma::mbar_wait(&kv_empty[st], ((j / PF_STAGES) - 1) & 1, p.status, 11, abortw);
        tma::mbar_expect_tx(&kv_full[st], 2 * KV_BYTES);
        unsigned char* kd = sK + st * KV_BYTES;
        unsigned char* vd = sV + st * KV_BYTES;
#pragma unroll
        for (int hf = 0; hf < HALVES; ++hf) {
          if (j < NP) {
            tma_load_3d(kd + hf * KV_HALF, &kpmap, &kv_full[st], hf * 64, j * PF_BN, b * p.Hkv + hk);
            tma_load_3d(vd + hf * KV_HALF, &vpmap, &kv_full[st], hf * 64, j * PF_BN, b * p.Hkv + hk);
          } else {
            tma_load_4d(kd + hf * KV_HALF, &kbmap, &kv_full[st], hf * 64, hk, p.t0 + (j - NP) * PF_BN, b);
            tma_load_4d(vd + hf * KV_HALF, &vbmap, &kv_full[st], hf * 64, hk, p.t0 + (j - NP) * PF_BN, b);
          }
        }
      }
    }
  } else if (warp == 9) {
    // =========================== MMA issuer ===========================
    if (lane == 0) {
      constexpr uint32_t IDESC_QK = instr_desc(PF_BN, false);
      constexpr uint32_t IDESC_PV = instr_desc(DH, true);
      // S_s = Q_s . K_j^T  (the stream's S columns are free: its previous P.V, which read P from them, was
      // issued earlier by this same thread and the tensor pipe executes in order)
      auto issue_qk = [&](int j, int s) {
        const uint32_t kbase = smem_u32(sK + (j % PF_STAGES) * KV_BYTES);
        const uint32_t qbase = smem_u32(s ? sQn : sQs);
        const uint32_t dcol = tmem + (s ? TM_SN : 0u);
#pragma unroll
        for (int kk = 0; kk < KSTEPS_QK; ++kk) {
          const uint64_t ad = smem_desc(qbase + (kk >> 2) * Q_HALF + (kk & 3) * 32, 16, 1024);
          const uint64_t bd = smem_desc(kbase + (kk >> 2) * KV_HALF + (kk & 3) * 32, 16, 1024);
          tc_mma(dcol, ad, bd, IDESC_QK, kk > 0 ? 1u : 0u);
        }
        tc_commit(&s_full[s]);
      };
      tma::mbar_wait(q_full, 0, p.status, 13, abortw);
      tma::mbar_wait(&kv_full[0], 0, p.status, 14, abortw);
      tc_fence_after();
      issue_qk(0, 0);
      issue_qk(0, 1);
      for (int j = 0; j < NT; ++j) {
        const int st = j % PF_STAGES;
        const uint32_t vbase = smem_u32(sV + st * KV_BYTES);
        if (j + 1 < NT) tma::mbar_wait(&kv_full[(j + 1) % PF_STAGES], ((j + 1) / PF_STAGES) & 1, p.status, 14, abortw);
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          tma::mbar_wait(&p_full[s], j & 1, p.status, 12, abortw);
          tc_fence_after();
          const uint32_t pcol = tmem + (s ? TM_SN : 0u);          // P (bf16 pairs) sits in the first 64 S columns
          const uint32_t dcol = tmem + (s ? TM_ON : TM_OS);
#pragma unroll
          for (int kk = 0; kk < KSTEPS_PV; ++kk) {
            const uint64_t bd = smem_desc(vbase + kk * 2048, KV_HALF, 1024);
            tc_mma_ts(dcol, pcol + kk * 8, bd, IDESC_PV, (j > 0 || kk > 0) ? 1u : 0u);
          }
          tc_commit(&pv_done[s]);
          if (s == 1) tc_commit(&kv_empty[st]);
          if (j + 1 < NT) issue_qk(j + 1, s);
        }
      }
    }
  }
    __syncthreads();                                   // every role meets here once all tensor work is done
    if (warp == 9) {
      tc_fence_after();
      asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
    }
    return;
  }
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(PF_REGS_SOFTMAX));
  {
    // =========================== softmax / correction / epilogue (one stream per warp group) ===========================
    const int s = warp >> 2;                              // 0 = signal, 1 = noise
    const int sw = warp & 3;                              // warp index inside its group
    const int quarter = warp & 3;                         // TMEM lane quarter this warp may touch
    const int row = quarter * 32 + lane;                  // row of the query tile
    const int grow = r0 + row;                            // row inside the block
    const uint32_t lane_addr = tmem + ((uint32_t)(quarter * 32) << 16);
    const uint32_t s_col = lane_addr + (s ? TM_SN : 0u);
    const uint32_t o_col = lane_addr + (s ? TM_ON : TM_OS);
    if (s == 0) {                                         // visibility bits of the prefix slots
      for (int w32 = sw; w32 < NP * 4; w32 += 4) {
        const int c = w32 * 32 + lane;
        const bool vis = c < p.Lbuf && (!p.mask_unused || p.allowed[(long long)b * p.Lbuf + c] != 0);
        const unsigned bits = __ballot_sync(0xffffffffu, vis);
        if (lane == 0) sMask[w32] = bits;
      }
    }
    bar_softmax_all();

    float mb = -INFINITY;                                 // exponent base (lags the true max by < GAP)
    float l = 0.f;
    for (int j = 0; j < NT; ++j) {
      tma::mbar_wait(&s_full[s], j & 1, p.status, 16, abortw);
      tc_fence_after();
      // Visibility per group of 32 keys.  cls: 2 = all visible, 0 = none, 1 = mixed; the class is the same for
      // every lane of a warp: prefix slots carry one mask per state, and in a block tile the 32 rows of a warp
      // meet the causal diagonal inside one group only.
      uint32_t vis[4]; int cls[4];
      if (j < NP) {
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          vis[q4] = sMask[4 * j + q4];
          cls[q4] = vis[q4] == 0xffffffffu ? 2 : (vis[q4] == 0u ? 0 : 1);
        }
      } else {
        const int nvis = grow - (j - NP) * PF_BN + 1;     // key c0+i visible iff c0+i <= grow
        const int qd = (r0 + quarter * 32 - (j - NP) * PF_BN) >> 5;    // group holding this warp's diagonal
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const int nq = nvis - 32 * q4;
          vis[q4] = nq >= 32 ? 0xffffffffu : (nq <= 0 ? 0u : ((1u << nq) - 1u));
          cls[q4] = q4 < qd ? 2 : (q4 == qd ? 1 : 0);
        }
      }
      // S is read from TMEM once, all 128 keys of the row into registers (TMEM -> register bandwidth, not
      // arithmetic, bounds a two-pass softmax here); groups without a visible key are not read at all.
      uint32_t v[4][32];
#pragma unroll
      for (int g = 0; g < 4; ++g) if (cls[g] != 0) tc_ld32(s_col + g * 32, v[g]);
      tc_wait_ld();
      // row maximum over the visible keys
      float mx = -INFINITY;
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        float m0 = -INFINITY, m1 = -INFINITY;
        if (cls[g] == 2) {
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            m0 = max3(m0, __uint_as_float(v[g][i]), __uint_as_float(v[g][i + 1]));
            m1 = max3(m1, __uint_as_float(v[g][i + 2]), __uint_as_float(v[g][i + 3]));
          }
        } else if (cls[g] == 1) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            if (!((vis[g] >> i) & 1u)) v[g][i] = 0xff800000u;       // -inf: exp gives 0 below
            m0 = fmaxf(m0, __uint_as_float(v[g][i]));
          }
        }
        mx = max3(mx, m0, m1);
      }
      mx *= p.scale_log2;                                  // scale > 0: max commutes with the scaling
      float alpha = 1.f;
      if (mx > mb + PF_RESCALE_GAP || (mb == -INFINITY && mx > -INFINITY)) {
        alpha = (mb == -INFINITY) ? 0.f : exp2f(mb - mx);
        mb = mx;
        l *= alpha;
      }
      // rescale O when some row of this warp moved its exponent base (not for the first tile: the first
      // P.V overwrites O instead of accumulating); O must be quiescent: wait for the previous P.V
      if (__any_sync(0xffffffffu, (alpha != 1.f) && j > 0)) {
        tma::mbar_wait(&pv_done[s], (j - 1) & 1, p.status, 19, abortw);
        tc_fence_after();
#pragma unroll 1
        for (int c = 0; c < DH / 16; ++c) {
          uint32_t o[16];
          tc_ld16(o_col + c * 16, o);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tc_st16(o_col + c * 16, o);
        }
      }
      // probabilities, written back over S as packed bf16 (key 2i, 2i+1 -> column i); every S column has been
      // read by now
      const float nref = mb == -INFINITY ? 0.f : -mb;
      const uint64_t scale2 = pk64(p.scale_log2, p.scale_log2), nref2 = pk64(nref, nref);
      uint64_t sum0 = 0ull, sum1 = 0ull, sum2 = 0ull, sum3 = 0ull;     // four independent chains of packed pairs
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        uint32_t pk[16];
        if (cls[g] == 0) {
#pragma unroll
          for (int i = 0; i < 16; ++i) pk[i] = 0u;
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            // exponent arguments of two keys per instruction; two pairs in three on the special-function
            // unit, the third on the FMA pipe
            float x0, x1, a0, a1;
            unpk64(fma2(pk64(__uint_as_float(v[g][2 * i]), __uint_as_float(v[g][2 * i + 1])), scale2, nref2), x0, x1);
            if (i % 3 == 2) { ex2_poly2(x0, x1, a0, a1); } else { a0 = ex2_mufu(x0); a1 = ex2_mufu(x1); }
            const uint64_t pr = pk64(a0, a1);
            if ((i & 3) == 0) sum0 = add2(sum0, pr); else if ((i & 3) == 1) sum1 = add2(sum1, pr);
            else if ((i & 3) == 2) sum2 = add2(sum2, pr); else sum3 = add2(sum3, pr);
            pk[i] = pack2(a0, a1);
          }
        }
        tc_st16(s_col + g * 16, pk);
      }
      {
        float t0, t1;
        unpk64(add2(add2(sum0, sum1), add2(sum2, sum3)), t0, t1);
        l += t0 + t1;
      }
      tc_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) tma::mbar_arrive(&p_full[s]);
    }

    // ---- epilogue: signal / l_s - lambda * noise / l_n, head RMSNorm, store ----
    // Both accumulators of a row sit in the same TMEM lane, so a thread reads both streams directly; the two
    // warp groups split the head dimension (group s takes columns s*Dh/2 ..) and exchange only the row sums
    // (1/l of each stream, partial sums of squares) through the shared memory of the query tiles, which are
    // dead once every Q.K^T has completed.  fp32 end to end with a single rounding of the result.
    const bool valid = grow < p.blk;
    float lam = 0.f;
    if (valid) lam = bf16_round(p.lam[(long long)b * p.lam_bs + (long long)(p.t0 + grow) * p.lam_rs + h]);
    constexpr int HC = DH / 2;                             // columns per thread
    float nwv[HC];
    if (p.norm_full) {
#pragma unroll
      for (int i = 0; i < HC / 2; ++i) {
        const __nv_bfloat162 wv = reinterpret_cast<const __nv_bfloat162*>(p.norm_w)[(s * HC) / 2 + i];
        nwv[2 * i] = __low2float(wv); nwv[2 * i + 1] = __high2float(wv);
      }
    }
    // Each group waits for ITS stream's last P.V only -- a barrier whose phases it has followed in order; a
    // parity wait on the other stream's barrier could pass on a phase two tiles back.  The block barrier below
    // then carries "both streams are complete" across the groups.
    tma::mbar_wait(&pv_done[s], (NT - 1) & 1, p.status, 18, abortw);
    tc_fence_after();
    float* xch = reinterpret_cast<float*>(sQs);            // [2][128] 1/l, then [2][128] partial sums of squares
    xch[s * PF_BM + row] = l > 0.f ? 1.f / l : 0.f;
    tc_fence_before();
    bar_softmax_all();
    tc_fence_after();
    const float inv_s = xch[row], inv_n = xch[PF_BM + row];
    float dv[HC];                                          // sig - lam * noise of this thread's columns
    float sq = 0.f;
#pragma unroll
    for (int c = 0; c < HC / 32; ++c) {
      uint32_t os[32], on[32];
      tc_ld32(lane_addr + TM_OS + s * HC + c * 32, os);
      tc_ld32(lane_addr + TM_ON + s * HC + c * 32, on);
      tc_wait_ld();
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const float d = fmaf(-lam, __uint_as_float(on[i]) * inv_n, __uint_as_float(os[i]) * inv_s);
        sq = fmaf(d, d, sq);
        dv[c * 32 + i] = d;
      }
    }
    xch[2 * PF_BM + s * PF_BM + row] = sq;
    bar_softmax_all();
    if (valid) {
      const float sq_row = xch[2 * PF_BM + row] + xch[3 * PF_BM + row];
      bf16* op = p.out + (long long)b * p.out_bs + (long long)(p.t0 + grow) * p.out_rs + (long long)h * DH + s * HC;
      const float rs = p.norm_full ? rsqrtf(sq_row / (float)DH + p.eps) : 1.f;
#pragma unroll
      for (int i = 0; i < HC / 8; ++i) {
        uint32_t w[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float y0 = dv[8 * i + 2 * e] * rs, y1 = dv[8 * i + 2 * e + 1] * rs;
          if (p.norm_full) { y0 *= nwv[8 * i + 2 * e]; y1 *= nwv[8 * i + 2 * e + 1]; }
          w[e] = pack2(y0, y1);
        }
        reinterpret_cast<uint4*>(op)[i] = make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
    tc_fence_before();
  }

  __syncthreads();
}

template <int DH>
size_t prefill_smem(int Lbuf) {
  const int NP = (Lbuf + PF_BN - 1) / PF_BN;
  return (size_t)2 * (DH / 64) * PF_BM * 128 + 2 * PF_STAGES * (size_t)(DH / 64) * PF_BN * 128 +
         (7 + 2 * PF_STAGES) * 8 + 8 + (size_t)NP * 4 * 4 + 1024 + 64;
}

template <int DH>
int launch_prefill(const CUtensorMap* maps, const PrefillParams& p, cudaStream_t s) {
  const size_t smem = prefill_smem<DH>(p.Lbuf);
  CODA_REQUIRE(smem <= 226 * 1024, CODA_ERR_LIMIT, "prefill_attend: %d slots need %zu bytes of shared memory", p.Lbuf, smem);
  static coda_device_once once;
  coda_on_first_use(once, [] {
    cudaFuncSetAttribute(prefill_attend_kernel<DH>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024);
  });
  dim3 grid((p.blk + PF_BM - 1) / PF_BM, p.H, p.B);
  {
    static int pool = 0;
    if (pool == 0) {
      cudaFuncAttributes fa;
      CODA_REQUIRE(cudaFuncGetAttributes(&fa, prefill_attend_kernel<DH>) == cudaSuccess, CODA_ERR_LAUNCH, "prefill_attend: cudaFuncGetAttributes failed");
      pool = fa.numRegs * PF_THREADS;
    }
    CODA_REQUIRE(pool >= PF_REGS_TOTAL, CODA_ERR_LAUNCH, "prefill_attend: register pool %d below the %d the roles ask for", pool, PF_REGS_TOTAL);
  }
  prefill_attend_kernel<DH><<<grid, PF_THREADS, smem, s>>>(maps[0], maps[1], maps[2], maps[3], maps[4], maps[5], p);
  CODA_CHECK_LAUNCH("prefill_attend");
  return CODA_OK;
}

}  // namespace

extern "C" int coda_b200_prefill_attend_supported(const coda_layer_cfg* cfg) {
  if (!coda_cfg_ok(cfg)) return 0;
  return cfg->dtype == CODA_BF16 && (cfg->Dh == 64 || cfg->Dh == 128) && tmaps::available();
}

extern "C" int coda_b200_prefill_attend(const coda_layer_cfg* cfg, const coda_state_ptrs* st,
                                        int32_t L, int32_t t0, int32_t blk,
                                        const void* q, int64_t q_bs, int64_t q_rs,
                                        const void* q_noise, int64_t qn_bs, int64_t qn_rs,
                                        const float* lam, int64_t lam_bs, int64_t lam_rs,
                                        const void* k_seq, int64_t k_bs, int64_t k_rs,
                                        const void* v_seq, int64_t v_bs, int64_t v_rs,
                                        const void* norm_w, void* out, int64_t out_bs, int64_t out_rs,
                                        int32_t* status, coda_stream_t stream) {
  CODA_REQUIRE(coda_cfg_ok(cfg) && st, CODA_ERR_ARG, "prefill_attend: invalid layer configuration");
  CODA_REQUIRE(coda_b200_prefill_attend_supported(cfg), CODA_ERR_ARG, "prefill_attend: needs bf16 and head_dim 64 or 128");
  CODA_REQUIRE(L > 0 && blk > 0 && t0 >= 0 && t0 + blk <= L, CODA_ERR_ARG, "prefill_attend: block [%d, %d) outside the %d tokens", t0, t0 + blk, L);
  CODA_REQUIRE(q && q_noise && lam && k_seq && v_seq && out && st->k_buf && st->v_buf && st->allowed, CODA_ERR_ARG,
               "prefill_attend: null pointer");
  CODA_REQUIRE(!cfg->head_norm_full || norm_w, CODA_ERR_ARG, "prefill_attend: head-norm weight missing");
  const uintptr_t al = (uintptr_t)q | (uintptr_t)q_noise | (uintptr_t)k_seq | (uintptr_t)v_seq | (uintptr_t)out |
                       (uintptr_t)st->k_buf | (uintptr_t)st->v_buf;
  CODA_REQUIRE(al % 16 == 0 && (q_bs | q_rs | qn_bs | qn_rs | k_bs | k_rs | v_bs | v_rs | out_bs | out_rs) % 8 == 0, CODA_ERR_ARG,
               "prefill_attend: pointers must be 16-byte aligned and strides multiples of 8 elements");
  const int Lbuf = cfg->W + cfg->Me + cfg->Ms, Dh = cfg->Dh;
  CUtensorMap maps[6];
  const bool ok = tmaps::token_map(&maps[0], q, cfg->B, L, cfg->H, Dh, q_bs, q_rs, PF_BM) &&
                  tmaps::token_map(&maps[1], q_noise, cfg->B, L, cfg->H, Dh, qn_bs, qn_rs, PF_BM) &&
                  tmaps::plane_map(&maps[2], st->k_buf, cfg->B * cfg->Hkv, Lbuf, Dh, PF_BN) &&
                  tmaps::plane_map(&maps[3], st->v_buf, cfg->B * cfg->Hkv, Lbuf, Dh, PF_BN) &&
                  tmaps::token_map(&maps[4], k_seq, cfg->B, L, cfg->Hkv, Dh, k_bs, k_rs, PF_BN) &&
                  tmaps::token_map(&maps[5], v_seq, cfg->B, L, cfg->Hkv, Dh, v_bs, v_rs, PF_BN);
  CODA_REQUIRE(ok, CODA_ERR_LAUNCH, "prefill_attend: cuTensorMapEncodeTiled failed");
  PrefillParams p;
  p.B = cfg->B; p.H = cfg->H; p.Hkv = cfg->Hkv; p.Lbuf = Lbuf; p.blk = blk; p.t0 = t0;
  p.mask_unused = cfg->mask_unused; p.norm_full = cfg->head_norm_full; p.eps = cfg->eps;
  p.scale_log2 = 1.4426950408889634f / sqrtf((float)Dh);
  p.lam = lam; p.lam_bs = lam_bs; p.lam_rs = lam_rs; p.allowed = st->allowed; p.norm_w = (const bf16*)norm_w;
  p.out = (bf16*)out; p.out_bs = out_bs; p.out_rs = out_rs; p.status = status;
  cudaStream_t s = (cudaStream_t)stream;
  return Dh == 128 ? launch_prefill<128>(maps, p, s) : launch_prefill<64>(maps, p, s);
}
