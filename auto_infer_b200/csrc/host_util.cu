// Host-side plumbing shared by the entry points: error text, device queries and
// the tensor-map encoder (driver entry point fetched at run time, so the library
// links against the CUDA runtime only).
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <vector>

#include "common.cuh"

namespace b200 {

static thread_local char g_last_error[512] = "";

void set_last_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
}

int check_cuda(cudaError_t err, const char* what) {
  if (err == cudaSuccess) return B200_OK;
  set_last_error("%s: %s", what, cudaGetErrorString(err));
  return B200_ECUDA;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

struct MapKey {
  const void* ptr;
  int num_blocks, block_size, heads, dim, box_tokens, device;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && num_blocks == o.num_blocks && block_size == o.block_size &&
           heads == o.heads && dim == o.dim && box_tokens == o.box_tokens && device == o.device;
  }
};
struct MapEntry {
  MapKey key;
  CUtensorMap map;
};

int get_cache_tensor_map(const void* cache, int num_blocks, int block_size, int heads, int dim,
                         int box_tokens, CUtensorMap* out) {
  static std::mutex mu;
  static std::vector<MapEntry> cache_entries;
  int device = 0;
  cudaGetDevice(&device);
  MapKey key{cache, num_blocks, block_size, heads, dim, box_tokens, device};
  {
    std::lock_guard<std::mutex> lock(mu);
    for (const MapEntry& e : cache_entries)
      if (e.key == key) {
        *out = e.map;
        return B200_OK;
      }
  }
  EncodeTiledFn fn = encode_fn();
  if (!fn) {
    set_last_error("cuTensorMapEncodeTiled is not available from this driver");
    return B200_ECUDA;
  }
  if (reinterpret_cast<uintptr_t>(cache) % 16 != 0) {
    set_last_error("paged cache base must be 16-byte aligned for TMA");
    return B200_EALIGN;
  }
  // innermost first: dim, head, token-in-block, block
  cuuint64_t dims[4] = {(cuuint64_t)dim, (cuuint64_t)heads, (cuuint64_t)block_size,
                        (cuuint64_t)num_blocks};
  cuuint64_t strides[3] = {(cuuint64_t)dim * 2, (cuuint64_t)heads * dim * 2,
                           (cuuint64_t)block_size * heads * dim * 2};
  cuuint32_t box[4] = {64, 1, (cuuint32_t)box_tokens, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUtensorMap map;
  CUresult r = fn(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(cache), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_last_error("cuTensorMapEncodeTiled failed with CUresult %d (blocks=%d bs=%d heads=%d dim=%d)",
                   (int)r, num_blocks, block_size, heads, dim);
    return B200_ECUDA;
  }
  {
    std::lock_guard<std::mutex> lock(mu);
    if (cache_entries.size() >= 256) cache_entries.erase(cache_entries.begin());
    cache_entries.push_back(MapEntry{key, map});
  }
  *out = map;
  return B200_OK;
}

struct QMapKey {
  const void* ptr;
  int num_tokens, heads, group, device;
  int64_t token_stride;
  bool operator==(const QMapKey& o) const {
    return ptr == o.ptr && num_tokens == o.num_tokens && heads == o.heads && group == o.group &&
           device == o.device && token_stride == o.token_stride;
  }
};
struct QMapEntry {
  QMapKey key;
  CUtensorMap map;
};

int get_query_tensor_map(const void* q, int num_tokens, int heads, int64_t token_stride, int group,
                         CUtensorMap* out) {
  static std::mutex mu;
  static std::vector<QMapEntry> entries;
  int device = 0;
  cudaGetDevice(&device);
  QMapKey key{q, num_tokens, heads, group, device, token_stride};
  {
    std::lock_guard<std::mutex> lock(mu);
    for (const QMapEntry& e : entries)
      if (e.key == key) {
        *out = e.map;
        return B200_OK;
      }
  }
  EncodeTiledFn fn = encode_fn();
  if (!fn) {
    set_last_error("cuTensorMapEncodeTiled is not available from this driver");
    return B200_ECUDA;
  }
  // innermost first: dim, head, token
  cuuint64_t dims[3] = {128, (cuuint64_t)heads, (cuuint64_t)num_tokens};
  cuuint64_t strides[2] = {128 * 2, (cuuint64_t)token_stride * 2};
  cuuint32_t box[3] = {64, (cuuint32_t)group, (cuuint32_t)(128 / group)};
  cuuint32_t estr[3] = {1, 1, 1};
  CUtensorMap map;
  CUresult r = fn(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(q), dims, strides, box,
                  estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_last_error("cuTensorMapEncodeTiled failed with CUresult %d (query: tokens=%d heads=%d group=%d)",
                   (int)r, num_tokens, heads, group);
    return B200_ECUDA;
  }
  {
    std::lock_guard<std::mutex> lock(mu);
    if (entries.size() >= 64) entries.erase(entries.begin());
    entries.push_back(QMapEntry{key, map});
  }
  *out = map;
  return B200_OK;
}

}  // namespace b200

extern "C" {

const char* b200_version(void) { return "b200-attention 0.1 sm_100a"; }

const char* b200_last_error(void) { return b200::g_last_error; }

int b200_sm_count(void) {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -1;
  if (dev < 64 && cached[dev] > 0) return cached[dev];
  int n = 0;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return -1;
  if (dev < 64) cached[dev] = n;
  return n;
}

}  // extern "C"
