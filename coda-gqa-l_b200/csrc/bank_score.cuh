// Cosine scoring of unit-norm candidates against a bank's unit-norm routing cache.
#pragma once
#include "coda_common.cuh"

// Scores of ONE candidate against every slot of a bank (decode path).
//   hat   [Hkv][n] fp32 in shared memory: the candidate's unit vectors
//   cache [Hkv][M][n] (shared or global): the bank's unit-norm rows
//   dots  [M*Hkv] fp32 scratch in shared memory
//   out   [M]: sum over heads of the dtype-rounded per-head dot products
// One thread per (slot, head) pair walks its row sequentially -- no cross-lane reduction -- starting at a
// lane-dependent rotation so that the 32 rows a warp reads (all a multiple of 32 banks apart) hit different
// banks.  A second pass adds the Hkv per-head values of each slot.
template <typename T>
__device__ __forceinline__ void bank_scores_one(const float* __restrict__ hat, const T* __restrict__ cache, int M, int n,
                                                int Hkv, float* __restrict__ dots, float* __restrict__ out, int tid, int NT) {
  const int items = M * Hkv;
  const bool vec = (n % 4 == 0) && ((reinterpret_cast<uintptr_t>(cache) % 16) == 0) && ((reinterpret_cast<uintptr_t>(hat) % 16) == 0);
  for (int it = tid; it < items; it += NT) {
    const int m = it / Hkv, h = it % Hkv;
    const T* row = cache + ((long long)h * M + m) * n;
    const float* a = hat + h * n;
    float acc = 0.f;
    if (vec) {
      const int nq = n >> 2;                                 // 4-element chunks
      int q = (tid & 31) % nq;
#pragma unroll 4
      for (int j = 0; j < nq; ++j) {
        const float4 av = *reinterpret_cast<const float4*>(a + 4 * q);
        float r0, r1, r2, r3;
        if (sizeof(T) == 2) {
          const uint2 u = *reinterpret_cast<const uint2*>(reinterpret_cast<const unsigned char*>(row) + 8 * q);
          r0 = __uint_as_float(u.x << 16); r1 = __uint_as_float(u.x & 0xffff0000u);
          r2 = __uint_as_float(u.y << 16); r3 = __uint_as_float(u.y & 0xffff0000u);
        } else {
          const float4 rv = *reinterpret_cast<const float4*>(reinterpret_cast<const unsigned char*>(row) + 16 * q);
          r0 = rv.x; r1 = rv.y; r2 = rv.z; r3 = rv.w;
        }
        acc = fmaf(av.x, r0, acc); acc = fmaf(av.y, r1, acc); acc = fmaf(av.z, r2, acc); acc = fmaf(av.w, r3, acc);
        q = (q + 1 == nq) ? 0 : q + 1;
      }
    } else {
      for (int d = 0; d < n; ++d) acc = fmaf(a[d], El<T>::ld(row + d), acc);
    }
    dots[it] = El<T>::rnd(acc);
  }
  __syncthreads();
  for (int m = tid; m < M; m += NT) {
    float tot = 0.f;
    for (int h = 0; h < Hkv; ++h) tot += dots[m * Hkv + h];
    out[m] = tot;
  }
  __syncthreads();
}
