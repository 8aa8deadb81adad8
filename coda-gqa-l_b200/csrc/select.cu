// Candidate selection for all blocks of one prefill call.
// Which tokens leave the ring in block j depends only on counts, and their write gates are
// known before the block loop starts, so the per-block top-k (upstream memory_banks.py:486-552)
// is hoisted out of the sequential chain: one warp per (state, block) stages the gates of the
// evicted run in shared memory and lane 0 replays the host selection algorithm on them.
#include "coda_common.cuh"
#include "topk_order.h"

struct SelectParams {
  const float* gates; long long gates_bs;
  int B, W, Te, Ts, ring_fill0, L, block, nblk;
  int* cand; int cand_stride;
};

constexpr int SEL_WARPS = 4;

__global__ void __launch_bounds__(SEL_WARPS * 32) select_kernel(SelectParams p, int cap) {
  extern __shared__ unsigned char sel_sm[];
  typedef topk_order::Item<float> It;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  It* q = reinterpret_cast<It*>(sel_sm) + (size_t)warp * cap;
  const long long prob = (long long)blockIdx.x * SEL_WARPS + warp;
  if (prob >= (long long)p.B * p.nblk) return;
  const int b = (int)(prob / p.nblk), j = (int)(prob % p.nblk);
  // counts before block j (memory_banks.py:459-466)
  const long long t0 = (long long)j * p.block;
  const long long seen = p.ring_fill0 + t0;                 // tokens of the stream before the block
  const int fill = (int)(seen < p.W ? seen : p.W);          // ring occupancy before the block
  const int blk = (int)((p.L - t0) < p.block ? (p.L - t0) : p.block);
  const int n_ev = max(0, fill + blk - p.W);
  const int te = min(p.Te, n_ev), ts = min(p.Ts, n_ev);
  const int k = max(te, ts);
  int* out = p.cand + ((long long)b * p.nblk + j) * p.cand_stride;
  if (k == 0) return;
  const float* g = p.gates + (long long)b * p.gates_bs + (seen - fill);   // first evicted token
  for (int i = lane; i < n_ev; i += 32) { q[i].v = g[i]; q[i].i = i; }
  __syncwarp();
  if (lane == 0) topk_order::topk_queue<float, true>(q, n_ev, k, false);
  __syncwarp();
  for (int i = lane; i < k; i += 32) out[i] = q[i].i;
}

extern "C" int coda_b200_select_candidates(const coda_layer_cfg* cfg, const float* gates, int64_t gates_bs,
                                           int32_t ring_fill0, int32_t L, int32_t block,
                                           int32_t* cand, int32_t cand_stride, coda_stream_t stream) {
  CODA_REQUIRE(coda_cfg_ok(cfg), CODA_ERR_ARG, "select_candidates: invalid layer configuration");
  CODA_REQUIRE(gates && cand && L > 0 && block > 0, CODA_ERR_ARG, "select_candidates: bad arguments");
  CODA_REQUIRE(ring_fill0 >= 0 && ring_fill0 <= cfg->W, CODA_ERR_ARG, "select_candidates: ring_fill0 out of range");
  SelectParams p;
  p.gates = gates; p.gates_bs = gates_bs; p.B = cfg->B; p.W = cfg->W;
  p.Te = (cfg->Me > 0) ? cfg->Te : 0; p.Ts = (cfg->Ms > 0) ? cfg->Ts : 0;
  p.ring_fill0 = ring_fill0; p.L = L; p.block = block; p.nblk = (L + block - 1) / block;
  p.cand = cand; p.cand_stride = cand_stride;
  const int tmax = p.Te > p.Ts ? p.Te : p.Ts;
  CODA_REQUIRE(cand_stride >= (tmax < block ? tmax : block), CODA_ERR_ARG, "select_candidates: cand_stride too small");
  if (tmax == 0) return CODA_OK;
  const int cap = block;                                       // evict_len <= block
  const size_t smem = (size_t)SEL_WARPS * cap * sizeof(topk_order::Item<float>);
  CODA_REQUIRE(smem <= 200 * 1024, CODA_ERR_LIMIT, "select_candidates: block_size %d exceeds the limit of %d tokens",
               block, (int)(200 * 1024 / (SEL_WARPS * sizeof(topk_order::Item<float>))));
  if (smem > 48 * 1024) cudaFuncSetAttribute(select_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  const long long nprob = (long long)cfg->B * p.nblk;
  const int grid = (int)((nprob + SEL_WARPS - 1) / SEL_WARPS);
  select_kernel<<<grid, SEL_WARPS * 32, smem, (cudaStream_t)stream>>>(p, cap);
  CODA_CHECK_LAUNCH("select_candidates");
  return CODA_OK;
}
