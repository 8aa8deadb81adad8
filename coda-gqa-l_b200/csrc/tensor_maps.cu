#include "tensor_maps.h"
#include <map>
#include <mutex>
#include <tuple>

namespace tmaps {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  });
  return fn;
}

bool available() { return encode_fn() != nullptr; }

typedef std::tuple<const void*, long long, long long, long long, long long, long long, long long, int> Key;
static std::mutex g_mu;
static std::map<Key, CUtensorMap> g_cache;

static bool encode(CUtensorMap* out, const Key& key, int rank, const void* base, const cuuint64_t* dims,
                   const cuuint64_t* strides, const cuuint32_t* box) {
  std::lock_guard<std::mutex> lock(g_mu);
  auto it = g_cache.find(key);
  if (it != g_cache.end()) { *out = it->second; return true; }
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUtensorMap m;
  CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  if (g_cache.size() > 4096) g_cache.clear();
  g_cache[key] = m;
  *out = m;
  return true;
}

bool plane_map(CUtensorMap* out, const void* base, int planes, int rows, int Dh, int box_rows) {
  cuuint64_t dims[3] = {(cuuint64_t)Dh, (cuuint64_t)rows, (cuuint64_t)planes};
  cuuint64_t strides[2] = {(cuuint64_t)Dh * 2, (cuuint64_t)rows * Dh * 2};
  cuuint32_t box[3] = {64, (cuuint32_t)box_rows, 1};
  return encode(out, Key(base, planes, rows, Dh, 0, 0, box_rows, 3), 3, base, dims, strides, box);
}

bool matrix_map(CUtensorMap* out, const void* base, int rows, int cols, long long row_stride, int box_rows) {
  cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, 1};
  cuuint64_t strides[2] = {(cuuint64_t)row_stride * 2, (cuuint64_t)rows * (cuuint64_t)row_stride * 2};
  cuuint32_t box[3] = {64, (cuuint32_t)box_rows, 1};
  return encode(out, Key(base, -1, rows, cols, row_stride, 0, box_rows, 3), 3, base, dims, strides, box);
}

bool token_map(CUtensorMap* out, const void* base, int B, int L, int heads, int Dh, long long bs, long long rs,
               int box_rows) {
  cuuint64_t dims[4] = {(cuuint64_t)Dh, (cuuint64_t)heads, (cuuint64_t)L, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)Dh * 2, (cuuint64_t)rs * 2, (cuuint64_t)bs * 2};
  cuuint32_t box[4] = {64, 1, (cuuint32_t)box_rows, 1};
  return encode(out, Key(base, B, L, (long long)heads * 1000 + Dh, bs, rs, box_rows, 4), 4, base, dims, strides, box);
}

}  // namespace tmaps
