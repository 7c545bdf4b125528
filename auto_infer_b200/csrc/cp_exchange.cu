// Context-parallel exchange fused with the merge: every rank pushes its partial record
// [o | lse] straight into the receive buffers of all ranks with peer-to-peer stores over
// NVLink and merges the R records that arrive in its own buffer by log-sum-exp.  One kernel
// replaces the NCCL all-gather and the merge kernel of a layer-step; nothing but plain stores
// and loads crosses the link (no multicast, no remote TMA).
//
// The records travel in flagged 16-byte lines, {payload, step, payload, step}: a line is
// valid when both of its step words equal the step being exchanged, so the data needs no
// separate "ready" flag and the sender no fence that waits for its stores to be
// acknowledged across the link - the receiver simply polls the lines it is about to merge,
// and the latency of an exchange is one store's trip instead of three dependent ones (data,
// acknowledgement, flag).  A payload word holds two bf16 values of o (the partial rows are
// normalised, |o| is of the order of the values; the merged row is rounded to bf16 anyway),
// the row's log-sum-exp travels as fp32 in a line of its own.  Every rank merges what is in
// its receive buffer, its own record included, so all ranks compute the same bits.
//
// Receive buffer of a rank (symmetric: same layout on every rank, mapped into every peer):
// [2 slots][R sources][rows][dim / 4 + 1 lines].  The slot is the parity of the step number,
// which lives in device memory and is advanced by the kernel itself, so a captured step
// replays correctly.  A rank cannot get two steps ahead of a peer (it needs that peer's lines
// of the next step first), so two slots are enough and no "consumed" handshake is needed;
// lines left over from two steps ago carry an older step number and never match.
#include "common.cuh"

namespace b200 {

constexpr int kExThreads = 256;
constexpr int kExMaxBlocks = 64;
constexpr int kExMaxLinesPerLane = 4;                  // rows of up to 512 values
constexpr uint64_t kExDefaultWaitNs = 1000000000ull;   // 1 s: a peer is gone

struct ExchangeParams {
  const float* local;              // this rank's record: rows*D floats of o, then rows floats of lse
  const uint64_t* recv_ptrs;       // device array: receive-buffer base of every rank (peer mapped)
  uint32_t* state;                 // [0] step number, [2] blocks done with the step
  int rank, world;
  int64_t rows;
  int64_t rows_per_block;
  int dim;
  int lines_per_row;               // dim / 4 payload lines + 1 line for the lse
  uint64_t wait_limit_ns;
  void* out;
  float* lse_out;
  int32_t* status;
  int out_is_f32;
};

__device__ __forceinline__ void st_line(uint4* p, uint4 v) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}
__device__ __forceinline__ uint4 ld_line(const uint4* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

// Polls one line until both step words match; gives up after the limit (returns false).
__device__ __forceinline__ bool wait_line(const uint4* p, uint32_t seq, uint64_t limit_ns, uint4& v) {
  v = ld_line(p);
  if (v.y == seq && v.w == seq) return true;
  const uint64_t t0 = global_timer_ns();
  uint32_t spins = 0;
  for (;;) {
    v = ld_line(p);
    if (v.y == seq && v.w == seq) return true;
    if ((++spins & 63u) == 0 && global_timer_ns() - t0 > limit_ns) return false;
  }
}

__device__ __forceinline__ float2 unpack_bf16(uint32_t w) {
  const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(&w);
  return make_float2(__low2float(v), __high2float(v));
}

__global__ void __launch_bounds__(kExThreads)
cp_exchange_combine_kernel(const ExchangeParams p) {
  grid_dep_launch();                                 // the next kernel may set itself up meanwhile (it waits for this grid itself)
  grid_dep_wait();                                   // the local record comes from the decode kernel
  const uint32_t seq = p.state[0] + 1;               // advanced at the very end by the last block
  const int slot = seq & 1u;
  const int nblk = gridDim.x;
  const int64_t row0 = (int64_t)blockIdx.x * p.rows_per_block;
  const int64_t row1 = row0 + p.rows_per_block < p.rows ? row0 + p.rows_per_block : p.rows;
  const int64_t lse_base = p.rows * p.dim;           // offset of the lse part inside the local record
  const int lpr = p.lines_per_row;
  const int64_t src_lines = p.rows * lpr;            // lines of one (slot, source) record

  // ---- 1. push my slice of this rank's record, as flagged lines, into every rank's buffer
  for (int64_t i = threadIdx.x; i < (row1 - row0) * lpr; i += kExThreads) {
    const int64_t row = row0 + i / lpr;
    const int line = (int)(i % lpr);
    uint4 v;
    v.y = v.w = seq;
    if (line < lpr - 1) {
      const float4 x = *reinterpret_cast<const float4*>(p.local + row * p.dim + line * 4);
      v.x = pack_bf16(x.x, x.y);
      v.z = pack_bf16(x.z, x.w);
    } else {
      v.x = __float_as_uint(p.local[lse_base + row]);
      v.z = 0u;
    }
    for (int r = 0; r < p.world; ++r) {
      const int peer = (p.rank + r) % p.world;       // start with myself, spread the links
      uint4* dst = reinterpret_cast<uint4*>(p.recv_ptrs[peer]) + ((int64_t)slot * p.world + p.rank) * src_lines +
                   row * lpr + line;
      st_line(dst, v);
    }
  }
  // ---- 2. merge the R records of my slice as their lines arrive: one warp per row, a lane
  // takes every 32nd payload line (4 columns each); every lane reads the row's lse lines
  // itself.  A row is written only when the whole warp has all of its lines.
  {
    const uint4* base = reinterpret_cast<const uint4*>(p.recv_ptrs[p.rank]) + (int64_t)slot * p.world * src_lines;
    const int lane = threadIdx.x & 31;
    const int warps = kExThreads >> 5;
    for (int64_t row = row0 + (threadIdx.x >> 5); row < row1; row += warps) {
      // The lines of the R sources are independent: four loads are issued together and only a
      // line that has not arrived yet is polled, so a row costs about R / 4 trips to memory
      // instead of R.
      bool ok = true;
      float mx = -INFINITY;
      const uint4* lse_line = base + row * lpr + (lpr - 1);
      for (int r0 = 0; r0 < p.world && ok; r0 += 4) {
        uint4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (r0 + u < p.world) v[u] = ld_line(lse_line + (int64_t)(r0 + u) * src_lines);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (r0 + u >= p.world || !ok) continue;
          if (v[u].y != seq || v[u].w != seq)
            ok = wait_line(lse_line + (int64_t)(r0 + u) * src_lines, seq, p.wait_limit_ns, v[u]);
          mx = fmaxf(mx, __uint_as_float(v[u].x));
        }
      }
      float wsum = 0.f;
      for (int r = 0; r < p.world && ok; ++r) {
        const float l = __uint_as_float(ld_line(lse_line + (int64_t)r * src_lines).x);
        wsum += (l == -INFINITY) ? 0.f : __expf(l - mx);
      }
      const float inv = wsum > 0.f ? 1.f / wsum : 0.f;
      float4 acc[kExMaxLinesPerLane];
#pragma unroll
      for (int k = 0; k < kExMaxLinesPerLane; ++k) {
        acc[k] = make_float4(0.f, 0.f, 0.f, 0.f);
        const int line = lane + 32 * k;
        if (line >= lpr - 1) continue;
        const uint4* pay = base + row * lpr + line;
        for (int r0 = 0; r0 < p.world && ok; r0 += 4) {
          uint4 v[4], lv[4];
#pragma unroll
          for (int u = 0; u < 4; ++u)
            if (r0 + u < p.world) {
              v[u] = ld_line(pay + (int64_t)(r0 + u) * src_lines);
              lv[u] = ld_line(lse_line + (int64_t)(r0 + u) * src_lines);
            }
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            if (r0 + u >= p.world || !ok) continue;
            if (v[u].y != seq || v[u].w != seq)
              ok = wait_line(pay + (int64_t)(r0 + u) * src_lines, seq, p.wait_limit_ns, v[u]);
            const float l = __uint_as_float(lv[u].x);
            const float w = (l == -INFINITY) ? 0.f : __expf(l - mx) * inv;
            const float2 a = unpack_bf16(v[u].x), b = unpack_bf16(v[u].z);
            acc[k].x += w * a.x; acc[k].y += w * a.y; acc[k].z += w * b.x; acc[k].w += w * b.y;
          }
        }
      }
      if (!__all_sync(0xffffffffu, ok)) {              // a peer is gone: this and the remaining rows stay as they are
        if (lane == 0 && p.status) atomicOr(p.status, B200_STATUS_WAIT_TIMEOUT);
        break;
      }
#pragma unroll
      for (int k = 0; k < kExMaxLinesPerLane; ++k) {
        const int line = lane + 32 * k;
        if (line >= lpr - 1) continue;
        const int c = line * 4;
        if (p.out_is_f32) {
          *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out) + row * p.dim + c) = acc[k];
        } else {
          uint2 pk;
          pk.x = pack_bf16(acc[k].x, acc[k].y);
          pk.y = pack_bf16(acc[k].z, acc[k].w);
          *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p.out) + row * p.dim + c) = pk;
        }
      }
      if (p.lse_out && lane == 0) p.lse_out[row] = wsum > 0.f ? mx + __logf(wsum) : -INFINITY;
    }
  }
  // ---- 3. the last block to finish advances the step number (also after a timeout: the
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
  const int64_t lines = rows * (head_dim / 4 + 1);
  return (size_t)(2 * (int64_t)world * lines) * 16 + 256;
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
  if (head_dim > 128 * kExMaxLinesPerLane) {
    set_last_error("cp_exchange_combine: rows of %d values exceed the %d the kernel is built for", head_dim,
                   128 * kExMaxLinesPerLane);
    return B200_EUNSUPPORTED;
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
  p.lines_per_row = head_dim / 4 + 1;
  p.wait_limit_ns = wait_limit_ns > 0 ? (uint64_t)wait_limit_ns : kExDefaultWaitNs;
  p.out = out;
  p.lse_out = lse_out;
  p.status = status;
  p.out_is_f32 = out_is_f32;
  return check_cuda(launch_pdl(cp_exchange_combine_kernel, dim3(blocks), dim3(kExThreads), 0,
                               static_cast<cudaStream_t>(stream), p),
                    "cp_exchange_combine launch");
}
