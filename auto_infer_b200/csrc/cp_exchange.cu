// Context-parallel exchange fused with the merge: every rank pushes its packed
// partial record [o | lse] straight into the receive buffers of all ranks with
// peer-to-peer stores over NVLink, raises flags in each of them, waits (bounded)
// for the flags of all ranks in its own buffer and merges the R records by
// log-sum-exp from local memory.  One kernel replaces the NCCL all-gather and the
// merge kernel of a layer-step; nothing but plain stores and loads crosses the link
// (no multicast, no remote TMA).
//
// The rows are dealt to the blocks of the grid in contiguous slices.  A block pushes
// ITS slice of this rank's record to every rank, raises ITS flag there, waits for the
// same slice's flag from every rank and merges that slice: blocks never wait for one
// another, only for the same block of the peers, so no block of a rank is a funnel
// for the others and all blocks need not even be resident together.
//
// Receive buffer of a rank (symmetric: same layout on every rank, mapped into
// every peer):  [2 slots][R sources][slot_floats] fp32, then R x kExMaxBlocks
// uint32 flags (source-major).  The slot is the parity of the step number, which
// lives in device memory and is advanced by the kernel itself, so a captured step
// replays correctly.  A rank cannot get two steps ahead of a peer (it needs that
// peer's flags of the next step first), so two slots are enough and no "consumed"
// handshake is needed.
#include "common.cuh"

namespace b200 {

constexpr int kExThreads = 256;
constexpr int kExMaxBlocks = 64;
constexpr uint64_t kExDefaultWaitNs = 1000000000ull;   // 1 s: a peer is gone

struct ExchangeParams {
  const float* local;              // this rank's record: rows*D floats of o, then rows floats of lse
  const uint64_t* recv_ptrs;       // device array: receive-buffer base of every rank (peer mapped)
  uint32_t* state;                 // [0] step number, [2] blocks done with the step
  int rank, world;
  int64_t rows;
  int64_t rows_per_block;
  int dim;
  int64_t slot_floats;             // capacity of one (slot, source) record
  int64_t flags_offset;            // in floats from the buffer base
  uint64_t wait_limit_ns;
  void* out;
  float* lse_out;
  int32_t* status;
  int out_is_f32;
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(kExThreads)
cp_exchange_combine_kernel(const ExchangeParams p) {
  __shared__ int s_timeout;
  if (threadIdx.x == 0) s_timeout = 0;
  grid_dep_wait();                                   // the local record comes from the decode kernel
  const uint32_t seq = p.state[0] + 1;               // advanced at the very end by the last block
  const int slot = seq & 1u;
  const int nblk = gridDim.x;
  const int64_t row0 = (int64_t)blockIdx.x * p.rows_per_block;
  const int64_t row1 = row0 + p.rows_per_block < p.rows ? row0 + p.rows_per_block : p.rows;
  const int64_t lse_base = p.rows * p.dim;           // offset of the lse part inside a record

  // ---- 1. push my slice of this rank's record into every rank's receive buffer (mine included)
  if (row0 < row1) {
    const int64_t n4 = (row1 - row0) * p.dim >> 2;   // dim is a multiple of 4 (checked on the host)
    const float4* src = reinterpret_cast<const float4*>(p.local + row0 * p.dim);
    for (int r = 0; r < p.world; ++r) {
      const int peer = (p.rank + r) % p.world;       // start with myself, spread the links
      float* rec = reinterpret_cast<float*>(p.recv_ptrs[peer]) + ((int64_t)slot * p.world + p.rank) * p.slot_floats;
      float4* dst = reinterpret_cast<float4*>(rec + row0 * p.dim);
      for (int64_t i = threadIdx.x; i < n4; i += kExThreads) dst[i] = src[i];
      for (int64_t i = row0 + threadIdx.x; i < row1; i += kExThreads) rec[lse_base + i] = p.local[lse_base + i];
    }
  }
  __threadfence_system();
  __syncthreads();
  // ---- 2. raise my block's flag in every rank's buffer; 3. wait, bounded, for the same
  // block's flag of every rank in my own buffer
  if (threadIdx.x < p.world) {
    const int r = threadIdx.x;
    uint32_t* theirs = reinterpret_cast<uint32_t*>(reinterpret_cast<float*>(p.recv_ptrs[r]) + p.flags_offset) +
                       p.rank * kExMaxBlocks + blockIdx.x;
    st_release_sys(theirs, seq);
    const uint32_t* mine = reinterpret_cast<const uint32_t*>(reinterpret_cast<const float*>(p.recv_ptrs[p.rank]) +
                                                           p.flags_offset) + r * kExMaxBlocks + blockIdx.x;
    const uint64_t t0 = global_timer_ns();
    uint32_t spins = 0;
    while ((int32_t)(ld_acquire_sys(mine) - seq) < 0) {
      if ((++spins & 63u) == 0 && global_timer_ns() - t0 > p.wait_limit_ns) {     // the peer is gone
        s_timeout = 1;
        if (p.status) atomicOr(p.status, B200_STATUS_WAIT_TIMEOUT);
        break;
      }
    }
  }
  __syncthreads();
  // ---- 4. merge the R records of my slice: one warp per row, lane = float4 column group
  if (!s_timeout) {
    const float* base = reinterpret_cast<const float*>(p.recv_ptrs[p.rank]) + (int64_t)slot * p.world * p.slot_floats;
    const int lane = threadIdx.x & 31;
    const int warps = kExThreads >> 5;
    for (int64_t row = row0 + (threadIdx.x >> 5); row < row1; row += warps) {
      float mx = -INFINITY;
      for (int r = 0; r < p.world; ++r) mx = fmaxf(mx, base[r * p.slot_floats + lse_base + row]);
      float wsum = 0.f;
      for (int r = 0; r < p.world; ++r) {
        const float l = base[r * p.slot_floats + lse_base + row];
        wsum += (l == -INFINITY) ? 0.f : __expf(l - mx);
      }
      const float inv = wsum > 0.f ? 1.f / wsum : 0.f;
      for (int c = lane * 4; c < p.dim; c += 128) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int r = 0; r < p.world; ++r) {
          const float l = base[r * p.slot_floats + lse_base + row];
          const float w = (l == -INFINITY) ? 0.f : __expf(l - mx) * inv;
          const float4 x = *reinterpret_cast<const float4*>(base + r * p.slot_floats + row * p.dim + c);
          acc.x += w * x.x; acc.y += w * x.y; acc.z += w * x.z; acc.w += w * x.w;
        }
        if (p.out_is_f32) {
          *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out) + row * p.dim + c) = acc;
        } else {
          uint2 pk;
          pk.x = pack_bf16(acc.x, acc.y);
          pk.y = pack_bf16(acc.z, acc.w);
          *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p.out) + row * p.dim + c) = pk;
        }
      }
      if (p.lse_out && lane == 0) p.lse_out[row] = wsum > 0.f ? mx + __logf(wsum) : -INFINITY;
    }
  }
  // ---- 5. the last block to finish advances the step number (also after a timeout: the
  // next call then starts a fresh step instead of finding half of this one)
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(&p.state[2], 1u) == (uint32_t)nblk - 1) {
      p.state[2] = 0;
      p.state[0] = seq;
      __threadfence();
    }
  }
}

static int exchange_blocks(int64_t rows) {
  int64_t blocks = (rows + 7) / 8;                   // a warp per row, eight rows at a time
  if (blocks > kExMaxBlocks) blocks = kExMaxBlocks;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

}  // namespace b200

extern "C" size_t b200_cp_exchange_buffer_bytes(int world, int64_t rows, int head_dim) {
  if (world <= 0 || rows < 0 || head_dim <= 0) return 0;
  const int64_t rec = rows * (head_dim + 1);
  const int64_t slot_floats = (rec + 63) / 64 * 64;
  return (size_t)(2 * (int64_t)world * slot_floats + (int64_t)world * b200::kExMaxBlocks) * sizeof(float);
}

extern "C" int b200_cp_exchange_combine(const float* local_record, const uint64_t* recv_ptrs_dev,
                                        uint32_t* state_dev, int rank, int world, int64_t rows,
                                        int head_dim, int64_t wait_limit_ns, void* out,
                                        int out_is_f32, float* lse_out, int32_t* status,
                                        void* stream) {
  using namespace b200;
  if (rows == 0) return B200_OK;
  if (!local_record || !recv_ptrs_dev || !state_dev || !out || world <= 0 || world > kExThreads ||
      rank < 0 || rank >= world || rows < 0 || head_dim <= 0 || wait_limit_ns < 0) {
    set_last_error("cp_exchange_combine: null pointer, bad rank/world, non-positive size or negative wait limit");
    return B200_EINVAL;
  }
  if (head_dim % 4 || reinterpret_cast<uintptr_t>(local_record) % 16 ||
      reinterpret_cast<uintptr_t>(out) % 16) {
    set_last_error("cp_exchange_combine: head_dim must be a multiple of 4, pointers 16-byte aligned");
    return B200_EALIGN;
  }
  const int blocks = exchange_blocks(rows);
  ExchangeParams p;
  p.local = local_record;
  p.recv_ptrs = recv_ptrs_dev;
  p.state = state_dev;
  p.rank = rank;
  p.world = world;
  p.rows = rows;
  p.rows_per_block = (rows + blocks - 1) / blocks;
  p.dim = head_dim;
  const int64_t rec = rows * ((int64_t)head_dim + 1);
  p.slot_floats = (rec + 63) / 64 * 64;
  p.flags_offset = 2 * (int64_t)world * p.slot_floats;
  p.wait_limit_ns = wait_limit_ns > 0 ? (uint64_t)wait_limit_ns : kExDefaultWaitNs;
  p.out = out;
  p.lse_out = lse_out;
  p.status = status;
  p.out_is_f32 = out_is_f32;
  return check_cuda(launch_pdl(cp_exchange_combine_kernel, dim3(blocks), dim3(kExThreads), 0,
                               static_cast<cudaStream_t>(stream), p),
                    "cp_exchange_combine launch");
}
