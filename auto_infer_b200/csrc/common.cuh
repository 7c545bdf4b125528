// Shared device helpers for the sm_100a paged-attention kernels: mbarrier and
// TMA wrappers with bounded waits, ldmatrix / mma.sync fragments, small math.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/b200_attention.h"

namespace b200 {

// ---- host-side error text -------------------------------------------------
void set_last_error(const char* fmt, ...);
int check_cuda(cudaError_t err, const char* what);

// Encodes (and memoises) a 4-D tiled tensor map over a paged cache
// (num_blocks, block_size, heads, dim) bf16 with the dim axis cut into
// 64-element (128-byte) boxes under the 128-byte swizzle.
int get_cache_tensor_map(const void* cache, int num_blocks, int block_size, int heads, int dim,
                         int box_tokens, CUtensorMap* out);

// Encodes (and memoises) a 3-D tiled tensor map over the query activations
// (num_tokens, heads, 128) bf16 whose box is one 128-row query tile of a kv
// group: 64 dims x group heads x (128 / group) tokens, 128-byte swizzle.
int get_query_tensor_map(const void* q, int num_tokens, int heads, int64_t token_stride, int group,
                         CUtensorMap* out);

// ---- device ---------------------------------------------------------------
#ifdef __CUDACC__

// Launch with programmatic stream serialisation: the kernel may be scheduled
// while its predecessor in the stream is still draining, and synchronises with
// it itself through grid_dep_wait().  Saves the launch latency between the
// back-to-back kernels of a layer-step (slot write -> attention -> merge).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                              cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// Blocks until every kernel this one depends on has completed and its writes are
// visible (no-op when the kernel was launched the ordinary way).
__device__ __forceinline__ void grid_dep_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}
// Lets the next kernel of the stream be scheduled from now on.
__device__ __forceinline__ void grid_dep_launch() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Waits for a phase of an mbarrier, but never for ever: after `limit_ns` the
// wait gives up, raises the CTA-wide abort flag (every later wait in the CTA
// then returns at once, so control flow stays uniform and the kernel drains to
// its end) and records B200_STATUS_WAIT_TIMEOUT for the host.
// The spinning part lives in one out-of-line copy: the kernels have dozens of wait sites
// and their instruction footprint matters more than a call on the slow path.  A kernel that
// moves registers between its warps (setmaxnreg) cannot contain calls: its translation unit
// defines B200_INLINE_WAITS before including this header.
#ifdef B200_INLINE_WAITS
static __device__ __forceinline__ void mbar_wait_slow(
#else
static __device__ __noinline__ void mbar_wait_slow(
#endif
    uint64_t* bar, uint32_t parity, volatile int* cta_abort,
                                            int32_t* status, uint64_t limit_ns) {
  const uint64_t t0 = global_timer_ns();
  uint32_t spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 63u) == 0) {
      if (*cta_abort) return;
      if (global_timer_ns() - t0 > limit_ns) {
        *cta_abort = 1;
        if (status) atomicOr(status, B200_STATUS_WAIT_TIMEOUT);
        return;
      }
    }
  }
}
__device__ __forceinline__ void mbar_wait_bounded(uint64_t* bar, uint32_t parity,
                                                  volatile int* cta_abort, int32_t* status,
                                                  uint64_t limit_ns = 2000000000ull) {
  if (mbar_try_wait(bar, parity)) return;
  mbar_wait_slow(bar, parity, cta_abort, status, limit_ns);
}

// Orders this thread's earlier generic-proxy accesses to shared memory before later
// accesses by the async proxy (TMA) to the same bytes.
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// One 4-D tiled TMA load (no multicast) into this CTA's shared memory,
// completion counted in bytes on `bar`.
__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* map, uint64_t* bar,
                                            int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)),
        "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

// Hint: bring one 4-D box into L2 (nothing lands in shared memory, nothing completes on a
// barrier).  Out-of-range coordinates touch no memory.
__device__ __forceinline__ void tma_prefetch_4d(const CUtensorMap* map, int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.prefetch.tensor.4d.L2.global.tile [%0, {%1, %2, %3, %4}];"
               ::"l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
               : "memory");
}

__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, uint64_t* bar,
                                            int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)),
        "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

__device__ __forceinline__ void named_bar_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

// D(16x8, fp32) += A(16x16, bf16, row) * B(16x8, bf16, col)
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                               uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Byte offset of (row, 16-byte chunk) inside a [rows][64 x bf16] tile written by
// TMA under the 128-byte swizzle (tile base 1024-byte aligned).
__device__ __forceinline__ uint32_t swz128(int row, int chunk) {
  return static_cast<uint32_t>(row * 128 + ((chunk ^ (row & 7)) << 4));
}

#endif  // __CUDACC__
}  // namespace b200
