/*
 * coda_b200.h -- C ABI of the B200 (sm_100a) kernels for bounded-cache differential attention.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream, launches
 * asynchronously on that stream, allocates nothing and never synchronises.  It returns 0 on
 * success and a negative code when an argument is rejected; coda_b200_last_error() then
 * gives the reason.  The library has no CPU fallback: all pointers must be device pointers.
 *
 * Upstream paths below are relative to the CoDA-GQA-L project root.  The binding pattern
 * (raw pointers + cudaStream_t behind extern "C") follows upstream's own native layer,
 * kernels/coda_diff_epilogue/kernel_src/diff_epilogue.cu:465-568.
 *
 * Tensor layouts (row-major, innermost dimension last):
 *   k_buf, v_buf      [B][Hkv][Lbuf][Dh]   Lbuf = W + Me + Ms, slot order [ring | exact | summary]
 *   allowed           [B][Lbuf]            1 byte per slot, non-zero = slot holds valid data
 *   g_recent          [B][W]               fp32 write gate of each ring slot
 *   mem_last_exact    [B][Me]              int64 LRU stamp (position of the last touch)
 *   exact_v_norm      [B][Hkv][Me][Dh]     unit-norm copy of the exact bank's V rows
 *   sum_lf_k_norm     [B][Hkv][Ms][Dh/2]   unit-norm copy of the summary bank's low-frequency K band
 * Activations q/k/v are [B][L][heads][Dh] with Dh contiguous, heads Dh apart, and explicit
 * token (row) and batch strides in elements, so a slice of a fused projection can be passed.
 */
#ifndef CODA_B200_H
#define CODA_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* coda_stream_t; /* == cudaStream_t */

enum { CODA_F32 = 0, CODA_BF16 = 1 };

enum {
  CODA_OK = 0,
  CODA_ERR_ARG = -1,      /* bad size / null pointer / unsupported combination */
  CODA_ERR_LAUNCH = -2,   /* the CUDA runtime refused the launch */
  CODA_ERR_LIMIT = -3     /* a documented size limit was exceeded */
};

/* Hyper-parameters of one layer; mirrors the constructor arguments of upstream
 * CoDAGQALandmarkPerf2 (src/coda_gqa_l/attention.py:89-141) that the kernels need. */
typedef struct coda_layer_cfg {
  int32_t B, H, Hkv, Dh;
  int32_t W, Me, Ms;
  int32_t dtype;               /* CODA_F32 / CODA_BF16: k_buf, v_buf, norm caches, q, k, v, out */
  int32_t angle_dtype;         /* dtype RoPE angles are evaluated in (dtype of upstream's inv_freq buffer) */
  int32_t rope_interleaved;    /* 1: pairs (2i,2i+1); 0: pairs (i, i+Dh/2) */
  int32_t head_norm_full;      /* 1: RMSNorm over Dh in the epilogue; 0: plain subtraction */
  int32_t mask_unused;         /* 1: slots with allowed==0 are invisible to attention */
  int32_t gated;               /* 1: write_policy "gated"; 0: "none" (gate == 1, no thresholds) */
  int32_t refresh_on_hit;
  int32_t overwrite_on_insert;
  int32_t Te, Ts;              /* exact / summary candidates per block */
  int32_t active_exact, active_summary;
  float tau_gate_exact, tau_gate_summary, tau_match, tau_novel;
  float eps;                   /* head-norm epsilon */
  float energy_scale;          /* sqrt(Dh / (Dh - Dh/2)) */
} coda_layer_cfg;

/* Device pointers of one layer's state; the fields of upstream's state dataclass
 * (src/coda_gqa_l/state.py:23-54). Pointers of absent banks (Me==0 / Ms==0) may be NULL. */
typedef struct coda_state_ptrs {
  void* k_buf;
  void* v_buf;
  uint8_t* allowed;
  float* g_recent;
  int64_t* mem_last_exact;
  void* exact_v_norm;
  void* sum_lf_k_norm;
  /* Optional routing-event record, int32 [B][CODA_EVENT_WORDS], or NULL.  Each cache write (step_write*,
   * route_block*) overwrites the words it owns with what happened to the state IN THAT CALL; the host turns
   * them into upstream's metrics counters (src/coda_gqa_l/attention.py:319-336) and into the pressure signals
   * of dynamic bank expansion (attention.py:358-390, memory_banks.py:333-337,416-420,744-760,934-940):
   *   [0] exact: candidates below the write gate        [1] exact: hits (decode: hit; block: hit and kept)
   *   [2] exact: inserts (novel, kept, within capacity) [3] exact: overwrites
   *   [4] exact: novel kept candidates that found no free active slot (decode) / beyond the capacity (block)
   *   [5] summary: updates (decode: kept; block: slots that received weight)   [6] summary: first fills
   *   [7] summary: every active slot in use after the call (0/1)              [8] summary: something came in */
  int32_t* events;
} coda_state_ptrs;
#define CODA_EVENT_WORDS 16

/* Ring scalars (state.py:28-36).  They are deterministic functions of the number of tokens
 * written, so the host keeps them as integers.  When step_dev is non-NULL the kernels add the
 * int64 it points to (a count of decode steps taken since the scalars were read) before use,
 * which lets a captured CUDA graph be replayed without re-baking the scalars. */
typedef struct coda_ring_pos {
  int64_t pos;
  int32_t recent_idx;
  int32_t recent_filled;
  const int64_t* step_dev;
} coda_ring_pos;

const char* coda_b200_last_error(void);
int coda_b200_version(void);

/* Projection post-processing for L tokens per state: RoPE on q and k in place, the
 * theta-rotated noise query, sigmoid of the lambda and write-gate logits.
 * Replaces RotaryEmbedding.forward + apply_rope + _apply_pairwise_rotation
 * (src/coda_gqa_l/primitives.py:43-113) and the sigmoids of attention.py:406-410,508,603.
 * q [B][L][H][Dh], k [B][L][Hkv][Dh] strided; q_noise [B][L][H][Dh] contiguous;
 * lam_logit [B][L][H] strided (dtype) -> lam [B][L][H] fp32; gate_logit [B][L] strided
 * (dtype, NULL when !gated) -> gate [B][L] fp32.  inv_freq fp32[Dh/2]; cos_theta/sin_theta
 * [H][Dh/2] in dtype.  Positions are rp.pos .. rp.pos+L-1.  k may be NULL (query only). */
int coda_b200_prep(const coda_layer_cfg* cfg, int32_t L, coda_ring_pos rp,
                   void* q, int64_t q_bs, int64_t q_rs,
                   void* k, int64_t k_bs, int64_t k_rs,
                   void* q_noise,
                   const void* lam_logit, int64_t lam_bs, int64_t lam_rs, float* lam,
                   const void* gate_logit, int64_t gate_bs, int64_t gate_rs, float* gate,
                   const float* inv_freq, const void* cos_theta, const void* sin_theta,
                   coda_stream_t stream);

/* One decode token per state: ring FIFO write, and when the ring is full the evicted token is
 * routed to the exact bank (value-space cosine novelty, first-free-else-LRU slot) and the
 * summary bank (low-frequency-key cosine argmax, phase-safe EMA).
 * Replaces _write_one / _exact_update_one / _summary_update_one
 * (src/coda_gqa_l/memory_banks.py:183-224, 230-337, 343-432).
 * k_new (already rotated), v_new: [B][Hkv][Dh] with batch stride; gate fp32[B];
 * eta_logit fp32[Hkv] (summary_eta_logit).  rp holds the scalars BEFORE the write. */
int coda_b200_step_write(const coda_layer_cfg* cfg, const coda_state_ptrs* st, coda_ring_pos rp,
                         const void* k_new, int64_t k_bs, const void* v_new, int64_t v_bs,
                         const float* gate, const float* eta_logit, coda_stream_t stream);

/* Same as coda_b200_step_write, but takes the un-rotated key projection and the gate LOGIT (dtype,
 * batch stride gate_bs; NULL when !gated): RoPE at position rp.pos (primitives.py:43-113) and the gate
 * sigmoid (attention.py:406-410) are applied inside the kernel. */
int coda_b200_step_write_raw(const coda_layer_cfg* cfg, const coda_state_ptrs* st, coda_ring_pos rp,
                             const void* k_raw, int64_t k_bs, const void* v_new, int64_t v_bs,
                             const void* gate_logit, int64_t gate_bs, const float* inv_freq,
                             const float* eta_logit, coda_stream_t stream);

/* Same as coda_b200_step_write_raw and, in the same launch, prepares the decode attention of the token being
 * written (the query side of attend_step, src/coda_gqa_l/attention.py:476-514): RoPE of the raw query
 * projection at position rp.pos, the learned theta rotation, the lambda sigmoid and the slot visibility mask
 * AFTER this write go into `qrec`, one record per (state, KV head), for coda_b200_decode_attend_prepared.
 * bf16 only; q_raw [B][H*Dh], lam_logit [B][H] with batch strides; cos_theta/sin_theta [H][Dh/2];
 * qrec: device buffer of coda_b200_decode_record_bytes(cfg) bytes, 16-byte aligned.  Needs a configuration
 * for which coda_b200_decode_attend_supported() is true and Hkv <= 8. */
int coda_b200_step_write_fused(const coda_layer_cfg* cfg, const coda_state_ptrs* st, coda_ring_pos rp,
                               const void* k_raw, int64_t k_bs, const void* v_new, int64_t v_bs,
                               const void* gate_logit, int64_t gate_bs, const float* inv_freq,
                               const float* eta_logit,
                               const void* q_raw, int64_t q_bs, const void* lam_logit, int64_t lam_bs,
                               const void* cos_theta, const void* sin_theta, void* qrec,
                               coda_stream_t stream);
int coda_b200_step_write_fused_supported(const coda_layer_cfg* cfg);

/* coda_b200_step_write_fused in two launches, for callers that want the routing off their critical path: the
 * token the ring is about to evict is routed into the banks from the state alone (coda_b200_step_route: may run
 * beside the projection GEMM that produces the new token, e.g. on another stream), then the new token takes the
 * ring slot and leaves its decode record (coda_b200_step_append_fused; same rp; must follow the route launch of
 * the same step).  The pair leaves the state exactly as the single launch does.  Same configurations as
 * coda_b200_step_write_fused_supported. */
int coda_b200_step_route(const coda_layer_cfg* cfg, const coda_state_ptrs* st, coda_ring_pos rp,
                         const float* eta_logit, coda_stream_t stream);
/* coda_b200_step_route for n_layers states of the same configuration in ONE launch (a decoder stack routes all
 * its layers' evicted tokens at the start of a step: one layer's routing is a chain of memory round trips, many
 * side by side are bound by bandwidth).  sts / rps / eta_logits are HOST arrays of n_layers entries;
 * coda_b200_step_route_plan copies what the kernel needs to `plan_dev` (device,
 * coda_b200_step_route_plan_bytes(n_layers) bytes, 8-byte aligned) and returns when the copy is done -- call it
 * outside stream capture; coda_b200_step_route_batched launches on a plan and may be captured and replayed
 * (with rp.step_dev set, as for any captured step). */
int64_t coda_b200_step_route_plan_bytes(int32_t n_layers);
int coda_b200_step_route_plan(const coda_layer_cfg* cfg, const coda_state_ptrs* sts, const coda_ring_pos* rps,
                              const float* const* eta_logits, int32_t n_layers, void* plan_dev,
                              coda_stream_t stream);
int coda_b200_step_route_batched(const coda_layer_cfg* cfg, const void* plan_dev, int32_t n_layers,
                                 coda_stream_t stream);
int coda_b200_step_append_fused(const coda_layer_cfg* cfg, const coda_state_ptrs* st, coda_ring_pos rp,
                                const void* k_raw, int64_t k_bs, const void* v_new, int64_t v_bs,
                                const void* gate_logit, int64_t gate_bs, const float* inv_freq,
                                const void* q_raw, int64_t q_bs, const void* lam_logit, int64_t lam_bs,
                                const void* cos_theta, const void* sin_theta, void* qrec,
                                coda_stream_t stream);

/* Fused decode attention (bf16, head_dim 64/128, <= 8 query heads per KV head): for every state and KV
 * head the K and V planes are read once (TMA into shared memory) and serve all query heads of the group
 * and both streams; RoPE at position rp.pos (- 1 if token_already_written), the theta rotation, the lambda
 * sigmoid, the lambda-gated subtraction and the head RMSNorm are fused.  Same result as
 * coda_b200_prep + coda_b200_attend with Lq = 1; replaces attend_step (src/coda_gqa_l/attention.py:476-514)
 * with _sdpa_stacked_two_stream (:416-465).  q_raw [B][H*Dh] and lam_logit [B][H] are bf16 with batch
 * strides; out [B][H*Dh] bf16.  qrec: device scratch of coda_b200_decode_record_bytes(cfg) bytes (16-byte
 * aligned) that receives the prepared queries.  status: optional device int, set non-zero if a bounded wait
 * expired.  coda_b200_decode_attend_supported() tells whether this configuration is covered.
 * coda_b200_decode_attend_prepared is the second half alone, on records already written by
 * coda_b200_step_write_fused. */
int coda_b200_decode_attend_supported(const coda_layer_cfg* cfg);
int64_t coda_b200_decode_record_bytes(const coda_layer_cfg* cfg);
int coda_b200_decode_attend(const coda_layer_cfg* cfg, const coda_state_ptrs* st, coda_ring_pos rp,
                            int32_t token_already_written,
                            const void* q_raw, int64_t q_bs, const void* lam_logit, int64_t lam_bs,
                            const float* inv_freq, const void* cos_theta, const void* sin_theta,
                            const void* norm_w, void* qrec, void* out, int64_t out_bs, int32_t* status,
                            coda_stream_t stream);
int coda_b200_decode_attend_prepared(const coda_layer_cfg* cfg, const coda_state_ptrs* st, const void* qrec,
                                     const void* norm_w, void* out, int64_t out_bs, int32_t* status,
                                     coda_stream_t stream);

/* Process-wide switch (default 1): the decode attention kernels signal `griddepcontrol.launch_dependents` right
 * after their own dependency wait, so that a following kernel launched as a programmatic dependent (the output
 * projection coda_b200_skinny_gemm is) is brought onto SMs as they become free and can stream its weights while the
 * attention's last planes finish; such a kernel still waits for the whole attention grid before it reads its
 * result.  0 restores the implicit trigger at grid completion (used to time a train of attention launches without
 * overlap between them).  Applies to launches made after the call. */
void coda_b200_decode_set_early_trigger(int32_t on);

/* coda_b200_step_write_fused followed by coda_b200_decode_attend_prepared on the records it wrote, as one call
 * (the default `step` of src/coda_gqa_l/attention.py:516-547 between its projections): same arguments, same two
 * launches, same results; for hosts where a foreign call costs more than the launch it makes. */
int coda_b200_step_write_attend(const coda_layer_cfg* cfg, const coda_state_ptrs* st, coda_ring_pos rp,
                                const void* k_raw, int64_t k_bs, const void* v_new, int64_t v_bs,
                                const void* gate_logit, int64_t gate_bs, const float* inv_freq,
                                const float* eta_logit,
                                const void* q_raw, int64_t q_bs, const void* lam_logit, int64_t lam_bs,
                                const void* cos_theta, const void* sin_theta, void* qrec,
                                const void* norm_w, void* out, int64_t out_bs, int32_t* status,
                                coda_stream_t stream);

/* y[M][N] = x[M][K] . w[N][K]^T (+ residual[M][N]), bf16 with fp32 accumulation, for the decode step's few rows
 * (M <= 32): the output projection of src/coda_gqa_l/attention.py:514 (`self.o_proj`, an nn.Linear without bias,
 * weight [N][K]) with the decoder's residual added in the same pass (the product is rounded to bf16 before the
 * add, as a GEMM followed by an add would).  x and w are dense row-major; y and residual have row strides in
 * elements.  coda_b200_skinny_gemm_supported tells whether the shape is covered (K a multiple of 128 up to 4096,
 * N a multiple of 64); status: optional device int, set non-zero if a bounded wait expired. */
int coda_b200_skinny_gemm_supported(int32_t M, int32_t K, int32_t N);
int coda_b200_skinny_gemm(const void* x, int32_t M, int32_t K, const void* w, int32_t N,
                          const void* residual, int64_t res_rs, void* y, int64_t y_rs,
                          int32_t* status, coda_stream_t stream);

/* The same product with a bias[N] added to the fp32 sum before its one rounding: the decode step's fused input
 * projection (the nn.Linear calls of src/coda_gqa_l/attention.py:396-410,508 as one [q|k|v|lambda|gate] matrix).
 * Runs on the variant of the kernel that splits K over clusters of four CTAs; coda_b200_skinny_gemm_bias_supported
 * tells whether that variant covers the shape on the current device (its clusters must be resident at once).
 * bias may be NULL (then this is coda_b200_skinny_gemm). */
int coda_b200_skinny_gemm_bias_supported(int32_t M, int32_t K, int32_t N);
/* How the four-way variant covers K x N on the current device: tile height in weight rows (0 when it does not)
 * and the number of clusters of four CTAs launched; returns whether it is covered. */
int coda_b200_skinny_gemm_plan(int32_t K, int32_t N, int32_t* tile_rows, int32_t* clusters);
int coda_b200_skinny_gemm_bias(const void* x, int32_t M, int32_t K, const void* w, int32_t N, const void* bias,
                               const void* residual, int64_t res_rs, void* y, int64_t y_rs,
                               int32_t* status, coda_stream_t stream);

/* A layer's output projection and the NEXT layer's fused input projection behind one launch:
 *   y_a[M][Na] = x_a[M][Ka] . w_a[Na][Ka]^T (+ residual_a, as coda_b200_skinny_gemm adds it), then
 *   y_b[M][Nb] = y_a . w_b[Nb][Na]^T + bias_b (as coda_b200_skinny_gemm_bias).
 * (src/coda_gqa_l/attention.py:514 of one layer followed by :396-410,508 of the next in a decoder that chains layers
 * as h <- h + layer(h).)  The same CTAs run both products with a barrier across the grid in between; the second
 * product's first weight boxes stream while the slower CTAs finish the first.  y_a is written densely (row stride Na).
 * gsync: two 32-bit words of device memory, zero before the first call and owned by the calls that share them, which
 * must be ordered on one stream.  coda_b200_skinny_gemm_chain_supported: whether both products fit the device as one
 * wave of clusters (needed for the barrier).  A barrier wait that runs out stores code 27 in the status word. */
int coda_b200_skinny_gemm_chain_supported(int32_t M, int32_t Ka, int32_t Na, int32_t Nb);
int coda_b200_skinny_gemm_chain(const void* x_a, int32_t M, int32_t Ka, const void* w_a, int32_t Na,
                                const void* residual_a, int64_t res_rs, void* y_a,
                                const void* w_b, int32_t Nb, const void* bias_b, void* y_b, int64_t y_b_rs,
                                uint32_t* gsync, int32_t* status, coda_stream_t stream);

/* The decode step's two projections on the tcgen05 tensor cores: y[M][N] = x[M][K] . w[N][K]^T (+ bias[N]) (+ residual[M][N]),
 * bf16 with fp32 accumulation, M <= 64 rows.  Replaces the nn.Linear calls of src/coda_gqa_l/attention.py:396-410,508 (the
 * q / k / v / lambda / write-gate projections, given here as ONE weight matrix whose rows are the five weights stacked,
 * bias likewise) and :467-470,514 (o_proj; `residual` adds the decoder's skip connection in the same pass: the product
 * (+ bias) is rounded to bf16 before the add, as a GEMM followed by an add would).  w is the nn.Linear weight as it is
 * ([out][in], dense, 16-byte aligned); x, y and residual have row strides in elements (x's a multiple of 8, x 16-byte
 * aligned); bias may be NULL.  K must be a multiple of 64.
 * The weight rows are the MMA's M (tiles of 128), the tokens its N.  All tiles' k-blocks, laid end to end, are cut into one
 * equal run per SM; a tile shared by several CTAs is summed through `workspace`: every contributor stores its fp32 partial
 * tile there, and the one that arrives last (a counter per tile, nobody waits) adds them in a fixed order and writes the
 * rows, so results are bit-reproducible.  workspace: coda_b200_proj_gemm_workspace_bytes(M, K, N) bytes on the device,
 * 16-byte aligned, its first 4096 bytes ZERO before the first use (the kernel leaves them zero); one workspace may serve
 * every call made on one stream (of the largest size asked for), calls that overlap on the GPU need their own.
 * Launched as a programmatic dependent launch: the weight stream starts before the kernel ahead of it on the stream has
 * finished; x, residual, workspace and y are touched only after it has.  status: optional device int, set non-zero if a
 * bounded wait expired. */
int coda_b200_proj_gemm_supported(int32_t M, int32_t K, int32_t N);
int64_t coda_b200_proj_gemm_workspace_bytes(int32_t M, int32_t K, int32_t N);
int coda_b200_proj_gemm(const void* x, int64_t x_rs, int32_t M, int32_t K, const void* w, int32_t N, const void* bias,
                        const void* residual, int64_t res_rs, void* y, int64_t y_rs, void* workspace, int32_t* status,
                        coda_stream_t stream);

/* coda_b200_step_append_fused and coda_b200_decode_attend_prepared as ONE launch: the attention kernel's
 * auxiliary warps write the new token (ring slot, gate, slot flag) and build each plane's queries / lambda / mask
 * in shared memory; the consumer warp owning the ring slot overwrites that row of the staged tile.  Saves a
 * launch and the record's round trip through global memory.  The token the ring evicts must have been routed
 * before (coda_b200_step_route or coda_b200_step_route_batched, same rp).  <= 1024 slots. */
int coda_b200_decode_attend_append_supported(const coda_layer_cfg* cfg);
int coda_b200_decode_attend_append(const coda_layer_cfg* cfg, const coda_state_ptrs* st, coda_ring_pos rp,
                                   const void* k_raw, int64_t k_bs, const void* v_new, int64_t v_bs,
                                   const void* gate_logit, int64_t gate_bs, const float* inv_freq,
                                   const void* q_raw, int64_t q_bs, const void* lam_logit, int64_t lam_bs,
                                   const void* cos_theta, const void* sin_theta, const float* rope_cs,
                                   const void* norm_w,
                                   void* out, int64_t out_bs, int32_t* status, coda_stream_t stream);
/* rope_cs (optional, may be NULL): cos [Dh/2] | sin [Dh/2] of the token's position from coda_b200_rope_table --
 * layers of a stack that share head_dim, RoPE base and dtype compute it once per step instead of once per CTA. */
int coda_b200_rope_table(const coda_layer_cfg* cfg, coda_ring_pos rp, const float* inv_freq, float* out,
                         coda_stream_t stream);

/* Differential attention of Lq query rows per state over [all Lbuf slots | optional block].
 * out = head_norm( softmax(q K^T) V - lam * softmax(q_noise K^T) V ), GQA by head index.
 * Slots are masked by `allowed` (when mask_unused); block key j is visible to row i iff j <= i.
 * Replaces _sdpa_stacked_two_stream + HeadwiseRMSNorm + the mask construction of
 * attend_step / prefill_chunked (src/coda_gqa_l/attention.py:416-465, 476-514, 553-565,
 * 612-701) and upstream's triton_diff_flash / coda_diff_epilogue accelerators.
 * q, q_noise [B][Lq][H][Dh] strided; lam fp32 [B][Lq][H] with strides; k_blk, v_blk
 * [B][Lq][Hkv][Dh] strided or NULL (decode); norm_w [Dh] in dtype or NULL;
 * out [B][Lq][H*Dh] with strides. */
int coda_b200_attend(const coda_layer_cfg* cfg, const coda_state_ptrs* st, int32_t Lq,
                     const void* q, int64_t q_bs, int64_t q_rs,
                     const void* q_noise, int64_t qn_bs, int64_t qn_rs,
                     const float* lam, int64_t lam_bs, int64_t lam_rs,
                     const void* k_blk, int64_t kb_bs, int64_t kb_rs,
                     const void* v_blk, int64_t vb_bs, int64_t vb_rs,
                     const void* norm_w,
                     void* out, int64_t out_bs, int64_t out_rs,
                     coda_stream_t stream);

/* Tensor-core prefill attention (bf16, head_dim 64/128): same result as coda_b200_attend for one block of `blk`
 * query rows starting at token t0 of an L-token chunk, computed with tcgen05.mma (accumulators in TMEM) on
 * TMA-staged tiles; both streams of a query head share every K/V tile.  Replaces the prefix+block attention of
 * prefill_chunked (src/coda_gqa_l/attention.py:612-701, _sdpa_stacked_two_stream :416-465, mask :553-565) and
 * upstream's triton_diff_flash kernel.  q, q_noise [B][L][H][Dh], k_seq, v_seq [B][L][Hkv][Dh] are the WHOLE
 * chunk's tensors (bf16, 16-byte aligned, strides multiples of 8 elements); lam fp32 [B][L][H]; out [B][L][H*Dh]
 * (rows t0 .. t0+blk-1 are written).  status: optional device int set when a bounded wait expires. */
int coda_b200_prefill_attend_supported(const coda_layer_cfg* cfg);
int coda_b200_prefill_attend(const coda_layer_cfg* cfg, const coda_state_ptrs* st,
                             int32_t L, int32_t t0, int32_t blk,
                             const void* q, int64_t q_bs, int64_t q_rs,
                             const void* q_noise, int64_t qn_bs, int64_t qn_rs,
                             const float* lam, int64_t lam_bs, int64_t lam_rs,
                             const void* k_seq, int64_t k_bs, int64_t k_rs,
                             const void* v_seq, int64_t v_bs, int64_t v_rs,
                             const void* norm_w, void* out, int64_t out_bs, int64_t out_rs,
                             int32_t* status, coda_stream_t stream);

/* Candidate selection for every block of one prefill call: for block j the tokens that leave
 * the ring are a contiguous run of the token stream; their fp32 gates are ranked exactly like
 * the host top-k upstream uses (memory_banks.py:486-552, torch.topk largest, unsorted), tie
 * order included, and the first T_max indices are written.
 * gates [B][ring_fill0 + L] (gates of the ring's tokens in chronological order, then the new
 * tokens); cand int32 [B][nblk][cand_stride]; nblk = ceil(L / block).  T_max per block is
 * max(Te', Ts') with Te' = min(Te, evict_len) (0 if that bank is off). */
int coda_b200_select_candidates(const coda_layer_cfg* cfg, const float* gates, int64_t gates_bs,
                                int32_t ring_fill0, int32_t L, int32_t block,
                                int32_t* cand, int32_t cand_stride, coda_stream_t stream);

/* Bank + ring update with one prefill block.  Requires recent_idx == 0 (ring stored in
 * chronological order; rotate it first if a decode phase moved the pointer).
 * Replaces _write_block_fast / _exact_update_block_vectorized / _summary_update_block_hard /
 * _set_recent_from_sequence (src/coda_gqa_l/memory_banks.py:438-564, 570-774, 780-950,
 * 152-177; PyTorch branches, not the Triton ones).
 * k_blk, v_blk [B][blk][Hkv][Dh] strided (k rotated); gates as for select_candidates with
 * gate_ev0 = index in `gates` rows of the first evicted token; cand int32 [B][*] with batch
 * stride cand_bs (this block's list); ring_fill = tokens in the ring before the block;
 * pos0 = position of the block's first token; scratch: coda_b200_route_scratch_bytes() bytes. */
int64_t coda_b200_route_scratch_bytes(const coda_layer_cfg* cfg);
int coda_b200_route_block(const coda_layer_cfg* cfg, const coda_state_ptrs* st,
                          int32_t ring_fill, int32_t blk, int64_t pos0,
                          const void* k_blk, int64_t kb_bs, int64_t kb_rs,
                          const void* v_blk, int64_t vb_bs, int64_t vb_rs,
                          const float* gates, int64_t gates_bs, int64_t gate_ev0,
                          const int32_t* cand, int64_t cand_bs,
                          const float* eta_logit, void* scratch, coda_stream_t stream);

/* The same block update in two halves, for callers that overlap the first with the block's attention:
 * phase 1 = scores and decisions (reads the state; writes only the scratch and the exact bank's LRU stamps, which
 * no attention kernel reads), phase 2 = slot updates and the ring rewrite (after phase 1 AND after the block's
 * attention have finished, same arguments, same scratch); phase 0 = both, i.e. coda_b200_route_block. */
int coda_b200_route_block_phase(const coda_layer_cfg* cfg, const coda_state_ptrs* st,
                                int32_t ring_fill, int32_t blk, int64_t pos0,
                                const void* k_blk, int64_t kb_bs, int64_t kb_rs,
                                const void* v_blk, int64_t vb_bs, int64_t vb_rs,
                                const float* gates, int64_t gates_bs, int64_t gate_ev0,
                                const int32_t* cand, int64_t cand_bs,
                                const float* eta_logit, void* scratch, int32_t phase, coda_stream_t stream);

/* coda_b200_route_block for callers that may not allocate device memory -- code running where cudaMalloc is
 * forbidden or unavailable: inside a serving engine whose memory pool is frozen after start-up, under a
 * framework that owns all allocations, or in a latency-critical loop where an allocation could stall.  It has no
 * counterpart in the reference (which allocates freely through PyTorch).  The per-state plan and score scratch
 * lives in a fixed array inside the library's device image; coda_b200_route_static_scratch_bytes() (1 MiB)
 * is its size, and a configuration whose coda_b200_route_scratch_bytes() exceeds it is rejected with
 * CODA_ERR_LIMIT (at the 7B shape that is reached beyond ~600 states per call).  Every GPU that loads the
 * library carries the array until the process exits.  The first call on a device looks up the array's address
 * (cudaGetSymbolAddress, with that device current): make that first call outside any stream capture.  All
 * calls on a device share the one array: the kernels overwrite every word they later read, so nothing has to be
 * cleared between calls, but two calls that overlap on the GPU (different streams) race on it.  Inputs and
 * outputs are the caller's, exactly as for coda_b200_route_block; no allocation happens on any path. */
int64_t coda_b200_route_static_scratch_bytes(void);
int coda_b200_route_block_noalloc(const coda_layer_cfg* cfg, const coda_state_ptrs* st,
                                  int32_t ring_fill, int32_t blk, int64_t pos0,
                                  const void* k_blk, int64_t kb_bs, int64_t kb_rs,
                                  const void* v_blk, int64_t vb_bs, int64_t vb_rs,
                                  const float* gates, int64_t gates_bs, int64_t gate_ev0,
                                  const int32_t* cand, int64_t cand_bs,
                                  const float* eta_logit, coda_stream_t stream);

/* Adds `n` to the int64 step counter that coda_ring_pos.step_dev points to (one thread). */
int coda_b200_advance_steps(int64_t* step_dev, int64_t n, coda_stream_t stream);

/* Self-test of the bounded device-side waits (no reference counterpart: the reference has no device-side waits).
 * Every pipelined kernel here waits on shared-memory barriers through one helper that gives up after a fixed
 * number of polls, records a code in the kernel's status word and sets a CTA-wide abort word that makes every other
 * wait of the CTA return at once; the kernel then runs out on meaningless data and exits normally (tensor memory
 * freed), and the host finds the code in the status word.  This entry point runs that helper on two barriers that
 * nobody arrives at: thread 0 with `poll_limit` polls (1..65536), thread 32 with the kernels' full limit.
 * status: device int32, zero before the call, 77 afterwards (the code of the wait that gave up first).
 * report: device int32[5] = {thread 0 saw its barrier complete (0), its cycles, thread 32 saw its barrier complete (0),
 * its cycles, the abort word (77)}.  Returns after the launch like every other entry point. */
int coda_b200_selftest_bounded_wait(int32_t poll_limit, int32_t* status, int32_t* report, coda_stream_t stream);

/* Host-only helpers (no GPU needed): the selection order used by select_candidates and by
 * the LRU victim ranking, exposed so that CPU tests can compare it with torch.topk. */
int coda_b200_host_topk_f32(const float* v, int32_t n, int32_t k, int32_t largest, int32_t sorted, int32_t* out);
int coda_b200_host_topk_i64(const int64_t* v, int32_t n, int32_t k, int32_t largest, int32_t sorted, int32_t* out);

#ifdef __cplusplus
}
#endif
#endif /* CODA_B200_H */
