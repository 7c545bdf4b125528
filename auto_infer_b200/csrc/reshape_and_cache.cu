// KV-cache slot write: cache[slot / bs, slot % bs, :, :] = x[t] for K and V.
// Bit-exact byte copy; 16-byte vector path when every row is 16-byte aligned,
// 2-byte path otherwise.  HBM-bound and tiny (a few KB to a few MB per step):
// one CTA per token keeps every store of a row coalesced.
#include "common.cuh"

namespace b200 {

template <typename Vec>
__global__ void __launch_bounds__(256)
reshape_and_cache_kernel(const Vec* __restrict__ key, const Vec* __restrict__ value,
                         Vec* __restrict__ key_cache, Vec* __restrict__ value_cache,
                         const int32_t* __restrict__ slot_mapping, int64_t key_stride,
                         int64_t value_stride, int k_row, int v_row, int64_t total_slots,
                         int32_t* status) {
  grid_dep_launch();              // the attention kernel may set itself up while rows are copied
  grid_dep_wait();                // the rows come from the kernel before this one
  const int t = blockIdx.x;
  const int64_t slot = slot_mapping[t];
  if (slot < 0) return;  // padding row
  if (slot >= total_slots) {
    if (threadIdx.x == 0 && status) atomicOr(status, B200_STATUS_BAD_SLOT);
    return;
  }
  const Vec* ksrc = key + (int64_t)t * key_stride;
  Vec* kdst = key_cache + slot * k_row;
  for (int i = threadIdx.x; i < k_row; i += blockDim.x) kdst[i] = ksrc[i];
  if (value != nullptr) {
    const Vec* vsrc = value + (int64_t)t * value_stride;
    Vec* vdst = value_cache + slot * v_row;
    for (int i = threadIdx.x; i < v_row; i += blockDim.x) vdst[i] = vsrc[i];
  }
}

}  // namespace b200

extern "C" int b200_reshape_and_cache(const void* key, const void* value, void* key_cache,
                                      void* value_cache, const int32_t* slot_mapping,
                                      int num_tokens, int num_kv_heads, int k_dim, int v_dim,
                                      int64_t key_stride, int64_t value_stride, int block_size,
                                      int num_blocks, int32_t* status, void* stream) {
  using namespace b200;
  if (num_tokens == 0) return B200_OK;
  if (!key || !key_cache || !slot_mapping || num_tokens < 0 || num_kv_heads <= 0 || k_dim <= 0 ||
      block_size <= 0 || num_blocks <= 0) {
    set_last_error("reshape_and_cache: null pointer or non-positive size");
    return B200_EINVAL;
  }
  if ((value == nullptr) != (value_cache == nullptr) || (value && v_dim <= 0)) {
    set_last_error("reshape_and_cache: value and value_cache must be given together");
    return B200_EINVAL;
  }
  const int64_t k_row = (int64_t)num_kv_heads * k_dim;
  const int64_t v_row = value ? (int64_t)num_kv_heads * v_dim : 0;
  if (key_stride < k_row || (value && value_stride < v_row)) {
    set_last_error("reshape_and_cache: token stride smaller than a row");
    return B200_EINVAL;
  }
  const int64_t total_slots = (int64_t)num_blocks * block_size;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  auto aligned16 = [](const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
  const bool vec = aligned16(key) && aligned16(key_cache) && (k_row % 8 == 0) && (key_stride % 8 == 0) &&
                   (!value || (aligned16(value) && aligned16(value_cache) && (v_row % 8 == 0) &&
                               (value_stride % 8 == 0)));
  if (vec) {
    const int row16 = (int)(k_row / 8);
    const int threads = row16 >= 256 ? 256 : (row16 >= 128 ? 128 : 64);
    return check_cuda(
        launch_pdl(reshape_and_cache_kernel<uint4>, dim3(num_tokens), dim3(threads), 0, s,
                   (const uint4*)key, (const uint4*)value, (uint4*)key_cache, (uint4*)value_cache,
                   slot_mapping, key_stride / 8, value_stride / 8, (int)(k_row / 8), (int)(v_row / 8),
                   total_slots, status),
        "reshape_and_cache launch");
  }
  return check_cuda(
      launch_pdl(reshape_and_cache_kernel<uint16_t>, dim3(num_tokens), dim3(256), 0, s,
                 (const uint16_t*)key, (const uint16_t*)value, (uint16_t*)key_cache,
                 (uint16_t*)value_cache, slot_mapping, key_stride, value_stride, (int)k_row, (int)v_row,
                 total_slots, status),
      "reshape_and_cache launch");
}
