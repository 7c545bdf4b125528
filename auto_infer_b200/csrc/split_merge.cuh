// Merge of the split-KV partial (o, lse) records of the (sequence, kv head) pairs
// that were cut across CTAs.  One CTA of 128 threads per 512 output floats: a
// whole row when the value width is 512 (MLA), four rows when it is 128 (GQA);
// each thread owns one float4 column group and walks the pair's records with
// four loads in flight, so a pair cut into many records (small batch, long
// context) is merged by rows * D / 512 CTAs in parallel instead of one.
#pragma once
#include "common.cuh"
#include "decode_plan.h"

namespace b200 {

template <int kDim>
__global__ void __launch_bounds__(128)
split_merge_kernel(const int32_t* __restrict__ plan, const float* __restrict__ part_o,
                   const float* __restrict__ part_lse, void* __restrict__ out,
                   float* __restrict__ lse_out, int num_q_heads, int group, int out_is_f32) {
  grid_dep_launch();                                 // the next kernel may set itself up meanwhile (it waits for this grid itself)
  grid_dep_wait();                                   // the partial records come from the decode kernel
  constexpr int kRowsPerCta = 512 / kDim;            // 1 (MLA) or 4 (GQA)
  constexpr int kThreadsPerRow = kDim / 4;
  constexpr int kCtasPerPair = kMaxRows / kRowsPerCta;
  // a replayable launch has the grid of the largest plan: CTAs past this plan's cut pairs leave
  if ((int)(blockIdx.x / kCtasPerPair) >= plan[kHdrNumMulti]) return;
  const MultiGroup g = reinterpret_cast<const MultiGroup*>(plan + plan[kHdrOffMulti])[blockIdx.x / kCtasPerPair];
  const int rows = g.q_len * group;
  const int row = (blockIdx.x % kCtasPerPair) * kRowsPerCta + threadIdx.x / kThreadsPerRow;
  const int col = (threadIdx.x % kThreadsPerRow) * 4;
  if (row >= rows) return;          // warp-uniform: a warp never spans two rows
  const int n = g.part_end - g.part_begin;
  const float* lse_base = part_lse + (int64_t)g.part_begin * kMaxRows + row;
  const float* o_base = part_o + ((int64_t)g.part_begin * kMaxRows + row) * kDim + col;
  // The lse values of the row are fetched 32 at a time, one per lane (all lanes of
  // a warp work on the same row), so the maximum costs one round of loads and a
  // shuffle tree instead of n dependent loads; the weights then travel by shuffle.
  const int lane = threadIdx.x & 31;
  float mx = -INFINITY;
  for (int i = lane; i < n; i += 32) mx = fmaxf(mx, lse_base[(int64_t)i * kMaxRows]);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
  float4 acc[4];
  float wsum[4];
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    acc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
    wsum[u] = 0.f;
  }
  for (int base = 0; base < n; base += 32) {
    float wl = 0.f;
    if (base + lane < n) {
      const float l = lse_base[(int64_t)(base + lane) * kMaxRows];
      wl = (l == -INFINITY) ? 0.f : __expf(l - mx);
    }
    const int cnt = min(32, n - base);
    for (int i = 0; i < cnt; i += 4) {
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const float w = __shfl_sync(0xffffffffu, wl, (i + u) & 31);
        if (i + u < cnt) {
          const float4 x = *reinterpret_cast<const float4*>(o_base + (int64_t)(base + i + u) * kMaxRows * kDim);
          wsum[u] += w;
          acc[u].x += w * x.x; acc[u].y += w * x.y; acc[u].z += w * x.z; acc[u].w += w * x.w;
        }
      }
    }
  }
  const float ws = (wsum[0] + wsum[1]) + (wsum[2] + wsum[3]);
  const float inv = ws > 0.f ? 1.f / ws : 0.f;
  float4 r;
  r.x = ((acc[0].x + acc[1].x) + (acc[2].x + acc[3].x)) * inv;
  r.y = ((acc[0].y + acc[1].y) + (acc[2].y + acc[3].y)) * inv;
  r.z = ((acc[0].z + acc[1].z) + (acc[2].z + acc[3].z)) * inv;
  r.w = ((acc[0].w + acc[1].w) + (acc[2].w + acc[3].w)) * inv;
  const int64_t tok = g.q_start + row / group;
  const int head = g.kv_head * group + row % group;
  const int64_t off = (tok * num_q_heads + head) * kDim + col;
  if (out_is_f32) {
    *reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + off) = r;
  } else {
    uint2 pk;
    pk.x = pack_bf16(r.x, r.y);
    pk.y = pack_bf16(r.z, r.w);
    *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(out) + off) = pk;
  }
  if (lse_out && (threadIdx.x % kThreadsPerRow) == 0)
    lse_out[tok * num_q_heads + head] = ws > 0.f ? mx + __logf(ws) : -INFINITY;
}

template <int kDim>
inline int split_merge_grid(int num_multi) { return num_multi * (kMaxRows / (512 / kDim)); }

}  // namespace b200
