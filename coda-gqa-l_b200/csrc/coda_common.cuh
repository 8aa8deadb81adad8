// Shared device helpers: element-type traits with "round like a tensor op" arithmetic,
// warp reductions, ring-scalar arithmetic and the host-side error channel.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>
#include "coda_b200.h"

typedef __nv_bfloat16 bf16;

// ---- element traits -------------------------------------------------------------------------
// The reference path runs as a chain of separate tensor ops; each op rounds its result to the
// tensor dtype.  rnd() applies that rounding to an fp32 intermediate (identity for fp32), and
// the rn intrinsics keep the compiler from contracting a*b+c into one fused rounding.
template <typename T> struct El;
template <> struct El<float> {
  static __device__ __forceinline__ float ld(const float* p) { return *p; }
  static __device__ __forceinline__ void st(float* p, float x) { *p = x; }
  static __device__ __forceinline__ float rnd(float x) { return x; }
};
template <> struct El<bf16> {
  static __device__ __forceinline__ float ld(const bf16* p) { return __bfloat162float(*p); }
  static __device__ __forceinline__ void st(bf16* p, float x) { *p = __float2bfloat16_rn(x); }
  static __device__ __forceinline__ float rnd(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
};

template <typename T> __device__ __forceinline__ float t_mul(float a, float b) { return El<T>::rnd(__fmul_rn(a, b)); }
template <typename T> __device__ __forceinline__ float t_add(float a, float b) { return El<T>::rnd(__fadd_rn(a, b)); }
template <typename T> __device__ __forceinline__ float t_sub(float a, float b) { return El<T>::rnd(__fsub_rn(a, b)); }
// Packed bf16 arithmetic: one instruction for two elements, each result the correctly rounded bf16 of the exact
// product / sum -- the same value as the fp32 operation followed by a rounding to bf16 that the scalar code spells
// out (a product of two bf16 is exact in fp32; a sum of two bf16 is exact in fp32 unless their exponents are more
// than 16 apart, and then it is more than a bf16 rounding step away from any tie).
__device__ __forceinline__ uint32_t bmul2(uint32_t a, uint32_t b) { uint32_t d; asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d; }
__device__ __forceinline__ uint32_t badd2(uint32_t a, uint32_t b) { uint32_t d; asm("add.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d; }
__device__ __forceinline__ uint32_t bneg2(uint32_t a) { return a ^ 0x80008000u; }
__device__ __forceinline__ uint32_t bdup_lo(uint32_t a) { return __byte_perm(a, a, 0x1010); }     // (x, y) -> (x, x)
__device__ __forceinline__ uint32_t bdup_hi(uint32_t a) { return __byte_perm(a, a, 0x3232); }     // (x, y) -> (y, y)
// (x, y) -> (-y, x): the second addend of a plane rotation (a, b) -> (a c - b s, b c + a s) written as
// (a, b) * (c, c) + (-(b s), a s)
__device__ __forceinline__ uint32_t bswap_neg(uint32_t a) { return __byte_perm(a, a, 0x1032) ^ 0x00008000u; }
// rotation of the pair held in one word by the angle (c, s) given as duplicated words
__device__ __forceinline__ uint32_t brot(uint32_t xy, uint32_t cc, uint32_t ss) { return badd2(bmul2(xy, cc), bswap_neg(bmul2(xy, ss))); }

// The correctly rounded division, exp and sin/cos expand to long instruction sequences (slow paths included).
// Kernels that run every instruction once pay for their code size in instruction fetches, so these live in
// one out-of-line copy per kernel.
static __device__ __noinline__ float div_rn_call(float a, float b) { return __fdiv_rn(a, b); }
static __device__ __noinline__ float sigmoid_call(float z) { return __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-z))); }
static __device__ __noinline__ void sincos_call(float x, float* s, float* c) { *s = sinf(x); *c = cosf(x); }

template <typename T> __device__ __forceinline__ float t_div(float a, float b) { return El<T>::rnd(div_rn_call(a, b)); }

// sigmoid of a value held in dtype T, result rounded to T
template <typename T> __device__ __forceinline__ float t_sigmoid(float z) { return El<T>::rnd(sigmoid_call(z)); }

__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

// ---- batched loads ---------------------------------------------------------------------------
// CNT consecutive elements starting at p, converted to fp32.  All loads are issued before any use (one
// memory round trip instead of CNT dependent ones); 16-byte vectors when the run is aligned.
template <typename T, int CNT>
__device__ __forceinline__ void load_run(const T* __restrict__ p, float (&out)[CNT]) {
  constexpr int BYTES = CNT * (int)sizeof(T);
  if constexpr (BYTES % 16 == 0) {
    if ((reinterpret_cast<uintptr_t>(p) & 15) == 0) {
      uint4 v[BYTES / 16];
#pragma unroll
      for (int i = 0; i < BYTES / 16; ++i) v[i] = reinterpret_cast<const uint4*>(p)[i];
#pragma unroll
      for (int i = 0; i < BYTES / 16; ++i) {
        const uint32_t w[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
        if (sizeof(T) == 2) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            out[i * 8 + 2 * j] = __uint_as_float(w[j] << 16);
            out[i * 8 + 2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j) out[i * 4 + j] = __uint_as_float(w[j]);
        }
      }
      return;
    }
  } else if constexpr (BYTES == 8 && sizeof(T) == 2) {
    if ((reinterpret_cast<uintptr_t>(p) & 7) == 0) {
      const uint2 v = *reinterpret_cast<const uint2*>(p);
      out[0] = __uint_as_float(v.x << 16); out[1] = __uint_as_float(v.x & 0xffff0000u);
      out[2] = __uint_as_float(v.y << 16); out[3] = __uint_as_float(v.y & 0xffff0000u);
      return;
    }
  }
  T raw[CNT];
#pragma unroll
  for (int i = 0; i < CNT; ++i) raw[i] = p[i];
#pragma unroll
  for (int i = 0; i < CNT; ++i) out[i] = El<T>::ld(&raw[i]);
}

// ---- warp helpers ---------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// ---- ring scalars ---------------------------------------------------------------------------
struct RingNow { long long pos; int idx; int filled; };

// Scalars after `n` more single-token writes (memory_banks.py:195-224): the ring fills slot by
// slot, then the eviction pointer walks round it.
__device__ __forceinline__ RingNow ring_after(const coda_ring_pos& rp, int W, long long n) {
  RingNow r; r.pos = rp.pos; r.idx = rp.recent_idx; r.filled = rp.recent_filled;
  if (n != 0) {
    long long to_fill = (long long)W - r.filled;
    if (to_fill < 0) to_fill = 0;
    long long nf = n < to_fill ? n : to_fill;
    r.filled += (int)nf;
    // steps past the fill wrap around the ring: 32-bit arithmetic whenever the count fits (a 64-bit remainder
    // is a long software routine, and every thread of every CTA on a latency chain runs this)
    const long long adv = (long long)r.idx + (n - nf);
    r.idx = adv < 0x7fffffffLL ? (int)((unsigned)adv % (unsigned)W) : (int)(adv % W);
    r.pos += n;
  }
  return r;
}
// The device step counter (0 without one): a kernel on a latency chain requests it first of all ...
__device__ __forceinline__ long long ring_steps(const coda_ring_pos& rp) { return rp.step_dev != nullptr ? *rp.step_dev : 0; }
// ... and uses it once its other requests are out.
__device__ __forceinline__ RingNow ring_now(const coda_ring_pos& rp, int W) { return ring_after(rp, W, ring_steps(rp)); }

// ---- host error channel ---------------------------------------------------------------------
void coda_set_error(const char* fmt, ...);
#define CODA_REQUIRE(cond, code, ...) do { if (!(cond)) { coda_set_error(__VA_ARGS__); return (code); } } while (0)
#define CODA_CHECK_LAUNCH(what) do { cudaError_t e__ = cudaGetLastError(); if (e__ != cudaSuccess) { \
  coda_set_error("%s: %s", what, cudaGetErrorString(e__)); return CODA_ERR_LAUNCH; } } while (0)

// ---- per-device launch set-up ------------------------------------------------------------------
// cudaFuncSetAttribute and the SM count belong to a device, not to the process: a process that drives several
// GPUs (a model spread over devices, one thread per GPU) repeats them for every device it launches on.
// `once` is a launcher's own table; returns true exactly once per device for it, holding off concurrent callers
// on the same table until the first one has finished its set-up (the caller does the set-up while `lock` lives).
#include <mutex>
constexpr int CODA_MAX_DEVICES = 64;
struct coda_device_once {
  std::mutex mu;
  bool done[CODA_MAX_DEVICES] = {};
  int sms[CODA_MAX_DEVICES] = {};
};
static inline int coda_current_device() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= CODA_MAX_DEVICES) return -1;
  return dev;
}
// Runs `setup` the first time this table sees the current device; returns that device's SM count.
template <typename F>
static inline int coda_on_first_use(coda_device_once& once, F&& setup) {
  const int dev = coda_current_device();
  std::lock_guard<std::mutex> lock(once.mu);
  if (dev < 0) { setup(); return 148; }               // unknown ordinal: configure every time
  if (!once.done[dev]) {
    setup();
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    once.sms[dev] = n;
    once.done[dev] = true;
  }
  return once.sms[dev];
}

static inline bool coda_cfg_ok(const coda_layer_cfg* c) {
  return c && c->B > 0 && c->H > 0 && c->Hkv > 0 && c->H % c->Hkv == 0 && c->Dh > 0 && (c->Dh % 2) == 0 &&
         c->W > 0 && c->Me >= 0 && c->Ms >= 0 && (c->dtype == CODA_F32 || c->dtype == CODA_BF16);
}
