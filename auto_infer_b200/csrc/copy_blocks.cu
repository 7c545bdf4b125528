// Copy of selected pages between two paged caches of identical layout: the transfer a
// prefill instance makes to a decode instance (auto_infer/pd/connector.py:30-51 copies the
// blocks one by one with a tensor copy each).  One launch moves all listed pages of one
// cache tensor; source and target may live on different GPUs of a node when the target (or
// the source) is peer-mapped into the calling device: only plain loads and stores cross the
// link.  Bit-exact, HBM / NVLink bound: bytes = 2 * pages * page_bytes.
#include "common.cuh"

namespace b200 {

constexpr int kCopyThreads = 256;

__global__ void __launch_bounds__(kCopyThreads)
copy_blocks_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst,
                   const int32_t* __restrict__ src_ids, const int32_t* __restrict__ dst_ids,
                   int num_ids, int64_t page_vec, int num_src_blocks, int num_dst_blocks,
                   int chunks_per_page, int32_t* status) {
  grid_dep_wait();
  const int page = blockIdx.x / chunks_per_page;
  const int chunk = blockIdx.x % chunks_per_page;
  if (page >= num_ids) return;
  const int s = src_ids[page];
  const int d = dst_ids ? dst_ids[page] : s;
  if (s < 0 || s >= num_src_blocks || d < 0 || d >= num_dst_blocks) {
    if (threadIdx.x == 0 && status) atomicOr(status, B200_STATUS_BAD_BLOCK);
    return;
  }
  const int64_t per_chunk = (page_vec + chunks_per_page - 1) / chunks_per_page;
  const int64_t lo = chunk * per_chunk;
  const int64_t hi = lo + per_chunk < page_vec ? lo + per_chunk : page_vec;
  const uint4* sp = src + (int64_t)s * page_vec;
  uint4* dp = dst + (int64_t)d * page_vec;
  // four independent 16-byte loads in flight per thread
  int64_t i = lo + threadIdx.x;
  for (; i + 3 * kCopyThreads < hi; i += 4 * kCopyThreads) {
    const uint4 a = sp[i], b = sp[i + kCopyThreads], c = sp[i + 2 * kCopyThreads], e = sp[i + 3 * kCopyThreads];
    dp[i] = a;
    dp[i + kCopyThreads] = b;
    dp[i + 2 * kCopyThreads] = c;
    dp[i + 3 * kCopyThreads] = e;
  }
  for (; i < hi; i += kCopyThreads) dp[i] = sp[i];
}

}  // namespace b200

extern "C" int b200_copy_blocks(const void* src_cache, void* dst_cache, const int32_t* src_block_ids,
                                const int32_t* dst_block_ids, int num_ids, int64_t page_bytes,
                                int num_src_blocks, int num_dst_blocks, int32_t* status, void* stream) {
  using namespace b200;
  if (num_ids == 0) return B200_OK;
  if (!src_cache || !dst_cache || !src_block_ids || num_ids < 0 || page_bytes <= 0 || num_src_blocks <= 0 ||
      num_dst_blocks <= 0) {
    set_last_error("copy_blocks: null pointer or non-positive size");
    return B200_EINVAL;
  }
  if (page_bytes % 16 || reinterpret_cast<uintptr_t>(src_cache) % 16 || reinterpret_cast<uintptr_t>(dst_cache) % 16) {
    set_last_error("copy_blocks: page size and cache bases must be multiples of 16 bytes");
    return B200_EALIGN;
  }
  const int64_t page_vec = page_bytes / 16;
  // enough CTAs to fill the machine also when few pages move: a page is cut into chunks of
  // at least 16 KiB
  int chunks = 1;
  int sms = b200_sm_count();
  if (sms <= 0) sms = 148;
  while (chunks < 16 && (int64_t)num_ids * chunks < 4LL * sms && page_bytes / (chunks * 2) >= 16384) chunks *= 2;
  const int64_t grid = (int64_t)num_ids * chunks;
  if (grid > INT32_MAX) {
    set_last_error("copy_blocks: %d pages exceed one launch", num_ids);
    return B200_ETOOLARGE;
  }
  return check_cuda(launch_pdl(copy_blocks_kernel, dim3((unsigned)grid), dim3(kCopyThreads), 0,
                               static_cast<cudaStream_t>(stream), (const uint4*)src_cache, (uint4*)dst_cache,
                               src_block_ids, dst_block_ids, num_ids, page_vec, num_src_blocks, num_dst_blocks,
                               chunks, status),
                    "copy_blocks launch");
}
