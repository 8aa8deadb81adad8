// Per-plane "decode record": everything the decode attention kernel needs for one (state, KV head) plane
// besides the K/V planes themselves, laid out exactly as the kernel keeps it in shared memory, so that one
// bulk copy brings it in:
//   [rows][Dh + 8] bf16   prepared queries: rows 0..G-1 the RoPE'd query heads of the group (signal), rows
//                         G..2G-1 their learned (even, odd) rotation by theta (noise), remaining rows zero;
//                         rows = 8 for G <= 4, else 16; the 8 pad columns keep ldmatrix free of bank conflicts
//   8 floats              lambda = sigmoid(lambda logit) of the G heads (rest zero)
//   ceil(Lbuf / 64) * 64  bytes of the slot visibility mask (zero past Lbuf)
// Written by the decode-step cache write (which has the position's cos/sin table at hand) or by a small
// preparation kernel; read by decode_attend_kernel.
#pragma once

struct DecodeRecord {
  static __host__ __device__ int qrows(int G) { return 2 * G <= 8 ? 8 : 16; }
  static __host__ __device__ int qstr(int Dh) { return Dh + 8; }
  static __host__ __device__ int lam_off(int G, int Dh) { return qrows(G) * qstr(Dh) * 2; }
  static __host__ __device__ int mask_off(int G, int Dh) { return lam_off(G, Dh) + 32; }
  static __host__ __device__ int mask_bytes(int Lbuf) { return (Lbuf + 63) / 64 * 64; }
  static __host__ __device__ int bytes(int G, int Dh, int Lbuf) { return mask_off(G, Dh) + mask_bytes(Lbuf); }
};
