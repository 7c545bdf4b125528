// Log-sum-exp merge of uniformly shaped partial results (context-parallel
// ranks): out[row] = sum_r exp(lse_r - lse) * o_r, lse = logsumexp_r lse_r.
// One warp per row; each lane owns float4 columns, so a 128-wide row is one
// coalesced 512-byte read per part.  HBM/latency-bound and tiny.
#include "common.cuh"

namespace b200 {

__global__ void __launch_bounds__(256)
lse_combine_kernel(const float* __restrict__ o_parts, const float* __restrict__ lse_parts,
                   int64_t stride_o, int64_t stride_lse, int n_parts, int64_t rows, int dim,
                   void* __restrict__ out, int out_is_f32, float* __restrict__ lse_out) {
  grid_dep_launch();              // the next kernel may set itself up meanwhile (it waits for this grid itself)
  grid_dep_wait();                // the parts come from the kernel (or collective) before this one
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  float mx = -INFINITY;
  for (int r = 0; r < n_parts; ++r) mx = fmaxf(mx, lse_parts[r * stride_lse + row]);
  float wsum = 0.f;
  for (int r = 0; r < n_parts; ++r) {
    const float l = lse_parts[r * stride_lse + row];
    wsum += (l == -INFINITY) ? 0.f : __expf(l - mx);
  }
  const float inv = wsum > 0.f ? 1.f / wsum : 0.f;
  for (int c = lane * 4; c < dim; c += 128) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r = 0; r < n_parts; ++r) {
      const float l = lse_parts[r * stride_lse + row];
      const float w = (l == -INFINITY) ? 0.f : __expf(l - mx) * inv;
      const float4 x = *reinterpret_cast<const float4*>(o_parts + r * stride_o + row * dim + c);
      acc.x += w * x.x; acc.y += w * x.y; acc.z += w * x.z; acc.w += w * x.w;
    }
    if (out_is_f32) {
      *reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + row * dim + c) = acc;
    } else {
      uint2 pk;
      pk.x = pack_bf16(acc.x, acc.y);
      pk.y = pack_bf16(acc.z, acc.w);
      *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(out) + row * dim + c) = pk;
    }
  }
  if (lse_out && lane == 0) lse_out[row] = wsum > 0.f ? mx + __logf(wsum) : -INFINITY;
}

}  // namespace b200

extern "C" int b200_lse_combine(const float* o_parts, const float* lse_parts, int64_t part_stride_o,
                                int64_t part_stride_lse, int n_parts, int64_t rows, int head_dim,
                                void* out, int out_is_f32, float* lse_out, void* stream) {
  using namespace b200;
  if (rows == 0) return B200_OK;
  if (!o_parts || !lse_parts || !out || n_parts <= 0 || rows < 0 || head_dim <= 0) {
    set_last_error("lse_combine: null pointer or non-positive size");
    return B200_EINVAL;
  }
  if (head_dim % 4 || part_stride_o % 4 || reinterpret_cast<uintptr_t>(o_parts) % 16 ||
      reinterpret_cast<uintptr_t>(out) % 16) {
    set_last_error("lse_combine: head_dim and part stride must be multiples of 4 and pointers 16-byte aligned");
    return B200_EALIGN;
  }
  const int warps = 8;
  const int64_t blocks = (rows + warps - 1) / warps;
  return check_cuda(launch_pdl(lse_combine_kernel, dim3((unsigned)blocks), dim3(warps * 32), 0,
                               static_cast<cudaStream_t>(stream), o_parts, lse_parts, part_stride_o,
                               part_stride_lse, n_parts, rows, head_dim, out, out_is_f32, lse_out),
                    "lse_combine launch");
}
