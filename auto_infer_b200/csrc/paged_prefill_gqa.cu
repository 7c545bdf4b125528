// Paged GQA attention for wide query blocks (chunked prefill, multi-token
// verify): any q_len, bottom-right causal over the paged prefix.
//
// Work item = 128 packed query rows of one (sequence, kv head) pair, a row being
// (query position, head within the kv group), so the G heads that share a kv
// head also share every K/V tile in shared memory.  One persistent CTA per SM
// takes items from a list sorted by decreasing key count (host plan):
//   * warp 8 streams 64-token K and V tiles through a 4-stage TMA ring exactly
//     as the decode kernel does (same tensor maps, same 128-byte swizzle);
//   * warps 0-7 each own 16 of the 128 rows and walk every tile: S = Q K^T and
//     O += P V on mma.sync m16n8k16 with an fp32 online softmax per row; tiles
//     entirely above a warp's causal frontier are skipped, tiles entirely below
//     it skip the mask.
// Tensor-bound: flops = 4 * D * sum over rows of visible keys.
#include <algorithm>
#include <vector>

#include "common.cuh"
#include "decode_plan.h"

namespace b200 {

constexpr int kPfHeadDim = 128;
constexpr int kPfStages = 4;
constexpr int kPfRows = 128;                                   // packed query rows per item
constexpr int kPfWarps = 8;
constexpr int kPfThreads = kPfWarps * 32 + 32;
constexpr int kPfHalfTileBytes = kTileTokens * 128;
constexpr int kPfTileBytes = 2 * kPfHalfTileBytes;
constexpr int kPfStageBytes = 2 * kPfTileBytes;
constexpr int kPfItemInts = 8;
constexpr int kPfMagic = 0x70663030;

struct PrefillItem {
  int32_t seq, kv_head, row0, n_tiles;        // row0: first packed row of the pair this item owns
  int32_t kv_len, q_start, q_len, causal_base;
};
static_assert(sizeof(PrefillItem) == kPfItemInts * 4, "item layout");

struct __align__(1024) PrefillSmem {
  uint8_t stage[kPfStages][kPfStageBytes];
  uint64_t full[kPfStages];
  uint64_t empty[kPfStages];
  int abort_flag;
};

struct PrefillParams {
  const __nv_bfloat16* q;
  int64_t q_stride;
  const int32_t* block_table;
  int64_t bt_stride;
  const PrefillItem* items;
  int num_items;
  void* out;
  float* lse_out;
  int32_t* status;
  int num_q_heads, group;
  int block_size, block_shift, num_blocks, box_tokens, boxes_per_tile;
  int out_is_f32;
  float scale, scale_log2;
};

__global__ void __launch_bounds__(kPfThreads, 1)
paged_prefill_gqa_kernel(const __grid_constant__ CUtensorMap k_map,
                         const __grid_constant__ CUtensorMap v_map, const PrefillParams p) {
  extern __shared__ uint8_t smem_raw[];
  PrefillSmem& sm = *reinterpret_cast<PrefillSmem*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    sm.abort_flag = 0;
    for (int s = 0; s < kPfStages; ++s) {
      mbar_init(&sm.full[s], 1);
      mbar_init(&sm.empty[s], kPfWarps);
    }
    mbar_fence_init();
  }
  __syncthreads();
  volatile int* abort_flag = &sm.abort_flag;

  if (warp == kPfWarps) {
    // ------------------------------ producer ------------------------------
    if (lane == 0) {
      tma_prefetch_desc(&k_map);
      tma_prefetch_desc(&v_map);
    }
    uint32_t it = 0;
    const int nbox = p.boxes_per_tile;
    for (int idx = blockIdx.x; idx < p.num_items; idx += gridDim.x) {
      const PrefillItem item = p.items[idx];
      const int last_block = (item.kv_len - 1) >> p.block_shift;
      for (int tile = 0; tile < item.n_tiles; ++tile, ++it) {
        int bid = 0;
        if (lane < nbox) {
          int lb = ((tile * kTileTokens) >> p.block_shift) + lane;
          lb = lb > last_block ? last_block : lb;
          bid = __ldg(p.block_table + (int64_t)item.seq * p.bt_stride + lb);
        }
        const int s = it % kPfStages;
        if (lane == 0) {
          mbar_wait_bounded(&sm.empty[s], ((it / kPfStages) & 1u) ^ 1u, abort_flag, p.status);
          mbar_arrive_expect_tx(&sm.full[s], kPfStageBytes);
        }
        __syncwarp();
        if (lane < nbox) {
          if (bid < 0 || bid >= p.num_blocks) {
            if (p.status) atomicOr(p.status, B200_STATUS_BAD_BLOCK);
            bid = p.num_blocks;
          }
          const int tok = (tile * kTileTokens + lane * p.box_tokens) & (p.block_size - 1);
          uint8_t* dst = sm.stage[s] + lane * p.box_tokens * 128;
          tma_load_4d(dst, &k_map, &sm.full[s], 0, item.kv_head, tok, bid);
          tma_load_4d(dst + kPfHalfTileBytes, &k_map, &sm.full[s], 64, item.kv_head, tok, bid);
          tma_load_4d(dst + kPfTileBytes, &v_map, &sm.full[s], 0, item.kv_head, tok, bid);
          tma_load_4d(dst + kPfTileBytes + kPfHalfTileBytes, &v_map, &sm.full[s], 64, item.kv_head, tok, bid);
        }
        __syncwarp();
      }
    }
    if (lane == 0) {
      const uint32_t n = it < (uint32_t)kPfStages ? it : (uint32_t)kPfStages;
      for (uint32_t k = 0; k < n; ++k) {
        const uint32_t j = it - 1 - k;
        mbar_wait_bounded(&sm.full[j % kPfStages], (j / kPfStages) & 1u, abort_flag, p.status);
      }
    }
    return;
  }

  // -------------------------------- consumers --------------------------------
  const int quad = lane >> 2;
  const int qlane = lane & 3;
  const int G = p.group;
  // ldmatrix lane addressing for a 16-token slice `ts` of the tile
  const int k_tok_l = ((lane >> 4) << 3) + (lane & 7);
  const int k_chunk_sel = (lane >> 3) & 1;
  const int v_tok_l = (((lane >> 3) & 1) << 3) + (lane & 7);
  const int v_chunk_sel = lane >> 4;

  uint32_t it = 0;
  for (int idx = blockIdx.x; idx < p.num_items; idx += gridDim.x) {
    const PrefillItem item = p.items[idx];
    const int rows_total = item.q_len * G;
    const int r0 = item.row0 + warp * 16 + quad;
    const int r1 = r0 + 8;
    const bool v0 = r0 < rows_total, v1 = r1 < rows_total;
    uint32_t qf[8][4];
    {
      const __nv_bfloat16* q0 = v0 ? p.q + (int64_t)(item.q_start + r0 / G) * p.q_stride +
                                         (int64_t)(item.kv_head * G + r0 % G) * kPfHeadDim
                                   : nullptr;
      const __nv_bfloat16* q1 = v1 ? p.q + (int64_t)(item.q_start + r1 / G) * p.q_stride +
                                         (int64_t)(item.kv_head * G + r1 % G) * kPfHeadDim
                                   : nullptr;
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        const int c = ks * 16 + qlane * 2;
        qf[ks][0] = q0 ? __ldg(reinterpret_cast<const uint32_t*>(q0 + c)) : 0u;
        qf[ks][1] = q1 ? __ldg(reinterpret_cast<const uint32_t*>(q1 + c)) : 0u;
        qf[ks][2] = q0 ? __ldg(reinterpret_cast<const uint32_t*>(q0 + c + 8)) : 0u;
        qf[ks][3] = q1 ? __ldg(reinterpret_cast<const uint32_t*>(q1 + c + 8)) : 0u;
      }
    }
    const int lim0 = v0 ? min(item.causal_base + r0 / G, item.kv_len - 1) : -1;
    const int lim1 = v1 ? min(item.causal_base + r1 / G, item.kv_len - 1) : -1;
    // warp-wide frontier: rows of a warp are consecutive, limits are monotone
    int wmax = max(lim0, lim1), wmin = min(v0 ? lim0 : INT32_MAX, v1 ? lim1 : INT32_MAX);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      wmax = max(wmax, __shfl_xor_sync(0xffffffffu, wmax, off));
      wmin = min(wmin, __shfl_xor_sync(0xffffffffu, wmin, off));
    }

    float o[16][4];
#pragma unroll
    for (int n = 0; n < 16; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

    for (int tile = 0; tile < item.n_tiles; ++tile, ++it) {
      const int s = it % kPfStages;
      const int tbase = tile * kTileTokens;
      // every warp observes every phase, also of tiles it skips: a warp that ran
      // ahead could otherwise arrive twice within one phase of the empty barrier
      mbar_wait_bounded(&sm.full[s], (it / kPfStages) & 1u, abort_flag, p.status);
      if (tbase <= wmax) {                      // otherwise the whole tile is above this warp's frontier
        const uint32_t kbase = smem_u32(sm.stage[s]);
        const uint32_t vbase = kbase + kPfTileBytes;
        const bool need_mask = tbase + kTileTokens - 1 > wmin;
#pragma unroll
        for (int half = 0; half < 2; ++half) {   // 32 tokens at a time keeps S at 16 registers
          float sacc[4][4];
#pragma unroll
          for (int n = 0; n < 4; ++n) sacc[n][0] = sacc[n][1] = sacc[n][2] = sacc[n][3] = 0.f;
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            const int chunk = ks * 2 + k_chunk_sel;
#pragma unroll
            for (int ts = 0; ts < 2; ++ts) {
              uint32_t kb[4];
              const int tok = half * 32 + ts * 16 + k_tok_l;
              ldmatrix_x4(kb, kbase + (chunk >> 3) * kPfHalfTileBytes + swz128(tok, chunk & 7));
              mma_bf16_16816(sacc[2 * ts], qf[ks], kb[0], kb[1]);
              mma_bf16_16816(sacc[2 * ts + 1], qf[ks], kb[2], kb[3]);
            }
          }
          float mx0 = -INFINITY, mx1 = -INFINITY;
          if (need_mask) {
            const int tok0 = tbase + half * 32 + qlane * 2;
#pragma unroll
            for (int n = 0; n < 4; ++n) {
#pragma unroll
              for (int e = 0; e < 2; ++e) {
                const int j = tok0 + n * 8 + e;
                if (j > lim0) sacc[n][e] = -INFINITY;
                if (j > lim1) sacc[n][2 + e] = -INFINITY;
              }
            }
          }
#pragma unroll
          for (int n = 0; n < 4; ++n) {
            mx0 = fmaxf(mx0, fmaxf(sacc[n][0], sacc[n][1]));
            mx1 = fmaxf(mx1, fmaxf(sacc[n][2], sacc[n][3]));
          }
          mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
          mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
          mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
          mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
          const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
          const float ms0 = (mn0 == -INFINITY) ? 0.f : mn0 * p.scale_log2;
          const float ms1 = (mn1 == -INFINITY) ? 0.f : mn1 * p.scale_log2;
          if (__any_sync(0xffffffffu, (mn0 != m0) || (mn1 != m1))) {
            const float c0 = fast_exp2(m0 * p.scale_log2 - ms0);
            const float c1 = fast_exp2(m1 * p.scale_log2 - ms1);
            l0 *= c0;
            l1 *= c1;
#pragma unroll
            for (int n = 0; n < 16; ++n) {
              o[n][0] *= c0; o[n][1] *= c0; o[n][2] *= c1; o[n][3] *= c1;
            }
            m0 = mn0;
            m1 = mn1;
          }
          uint32_t pf[2][4];
#pragma unroll
          for (int ts = 0; ts < 2; ++ts) {
            float pr[2][4];
#pragma unroll
            for (int n = 0; n < 2; ++n) {
              pr[n][0] = fast_exp2(fmaf(sacc[2 * ts + n][0], p.scale_log2, -ms0));
              pr[n][1] = fast_exp2(fmaf(sacc[2 * ts + n][1], p.scale_log2, -ms0));
              pr[n][2] = fast_exp2(fmaf(sacc[2 * ts + n][2], p.scale_log2, -ms1));
              pr[n][3] = fast_exp2(fmaf(sacc[2 * ts + n][3], p.scale_log2, -ms1));
              l0 += pr[n][0] + pr[n][1];
              l1 += pr[n][2] + pr[n][3];
            }
            pf[ts][0] = pack_bf16(pr[0][0], pr[0][1]);
            pf[ts][1] = pack_bf16(pr[0][2], pr[0][3]);
            pf[ts][2] = pack_bf16(pr[1][0], pr[1][1]);
            pf[ts][3] = pack_bf16(pr[1][2], pr[1][3]);
          }
#pragma unroll
          for (int ts = 0; ts < 2; ++ts) {
            const int tok = half * 32 + ts * 16 + v_tok_l;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const int chunk = j * 2 + v_chunk_sel;
              uint32_t vb[4];
              ldmatrix_x4_trans(vb, vbase + (chunk >> 3) * kPfHalfTileBytes + swz128(tok, chunk & 7));
              mma_bf16_16816(o[2 * j], pf[ts], vb[0], vb[1]);
              mma_bf16_16816(o[2 * j + 1], pf[ts], vb[2], vb[3]);
            }
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&sm.empty[s]);
    }

    // ---- normalise and store this warp's 16 rows
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float inv0 = l0 > 0.f ? 1.f / l0 : 0.f;
    const float inv1 = l1 > 0.f ? 1.f / l1 : 0.f;
    if (v0) {
      const int64_t tok = item.q_start + r0 / G;
      const int head = item.kv_head * G + r0 % G;
      const int64_t off = (tok * p.num_q_heads + head) * kPfHeadDim + qlane * 2;
#pragma unroll
      for (int n = 0; n < 16; ++n) {
        if (p.out_is_f32)
          *reinterpret_cast<float2*>(reinterpret_cast<float*>(p.out) + off + n * 8) =
              make_float2(o[n][0] * inv0, o[n][1] * inv0);
        else
          *reinterpret_cast<uint32_t*>(reinterpret_cast<__nv_bfloat16*>(p.out) + off + n * 8) =
              pack_bf16(o[n][0] * inv0, o[n][1] * inv0);
      }
      if (p.lse_out && qlane == 0)
        p.lse_out[tok * p.num_q_heads + head] = l0 > 0.f ? m0 * p.scale + __logf(l0) : -INFINITY;
    }
    if (v1) {
      const int64_t tok = item.q_start + r1 / G;
      const int head = item.kv_head * G + r1 % G;
      const int64_t off = (tok * p.num_q_heads + head) * kPfHeadDim + qlane * 2;
#pragma unroll
      for (int n = 0; n < 16; ++n) {
        if (p.out_is_f32)
          *reinterpret_cast<float2*>(reinterpret_cast<float*>(p.out) + off + n * 8) =
              make_float2(o[n][2] * inv1, o[n][3] * inv1);
        else
          *reinterpret_cast<uint32_t*>(reinterpret_cast<__nv_bfloat16*>(p.out) + off + n * 8) =
              pack_bf16(o[n][2] * inv1, o[n][3] * inv1);
      }
      if (p.lse_out && qlane == 0)
        p.lse_out[tok * p.num_q_heads + head] = l1 > 0.f ? m1 * p.scale + __logf(l1) : -INFINITY;
    }
  }
}

}  // namespace b200

using namespace b200;

extern "C" size_t b200_prefill_plan_bytes(int num_seqs, int num_tokens, int num_q_heads,
                                          int num_kv_heads) {
  if (num_seqs < 0 || num_tokens < 0 || num_q_heads <= 0 || num_kv_heads <= 0) return 0;
  const size_t group = (size_t)num_q_heads / num_kv_heads;
  const size_t items = ((size_t)num_tokens * group / kPfRows + num_seqs) * num_kv_heads;
  return (kPlanHeaderInts + kPfItemInts * items) * sizeof(int32_t);
}

extern "C" int b200_prefill_plan(const int32_t* cu_q, const int32_t* kv_lens,
                                 const int32_t* causal_base, int num_seqs, int num_q_heads,
                                 int num_kv_heads, int min_rows, int32_t* plan, size_t plan_bytes,
                                 b200_prefill_plan_info* info) {
  if (!plan || !info || num_seqs < 0 || (num_seqs > 0 && (!cu_q || !kv_lens)) || num_q_heads <= 0 ||
      num_kv_heads <= 0 || num_q_heads % num_kv_heads != 0) {
    set_last_error("prefill_plan: bad argument (null pointer, heads not divisible, or size <= 0)");
    return B200_EINVAL;
  }
  const int group = num_q_heads / num_kv_heads;
  const int num_tokens = num_seqs ? cu_q[num_seqs - 1] : 0;
  if (plan_bytes < b200_prefill_plan_bytes(num_seqs, num_tokens, num_q_heads, num_kv_heads)) {
    set_last_error("prefill_plan: plan buffer of %zu bytes is smaller than b200_prefill_plan_bytes()",
                   plan_bytes);
    return B200_EPLAN;
  }
  std::vector<PrefillItem> items;
  int64_t total_tiles = 0;
  int prev = 0;
  for (int b = 0; b < num_seqs; ++b) {
    const int q_start = prev;
    const int q_len = cu_q[b] - prev;
    prev = cu_q[b];
    if (q_len < 0 || kv_lens[b] < 0) {
      set_last_error("prefill_plan: sequence %d has negative length", b);
      return B200_EINVAL;
    }
    const int rows = q_len * group;
    if (q_len == 0 || kv_lens[b] == 0 || rows <= min_rows) continue;
    const int base = causal_base ? causal_base[b] : kv_lens[b] - q_len;
    for (int row0 = 0; row0 < rows; row0 += kPfRows) {
      const int last_row = std::min(row0 + kPfRows, rows) - 1;
      const int lim = std::min(base + last_row / group, kv_lens[b] - 1);   // last visible key of the item
      const int n_tiles = lim < 0 ? 0 : lim / kTileTokens + 1;
      for (int h = 0; h < num_kv_heads; ++h) {
        items.push_back(PrefillItem{b, h, row0, n_tiles, kv_lens[b], q_start, q_len, base});
        total_tiles += n_tiles;
      }
    }
  }
  // longest first: with round-robin assignment the tail is made of short items
  std::stable_sort(items.begin(), items.end(),
                   [](const PrefillItem& a, const PrefillItem& b) { return a.n_tiles > b.n_tiles; });
  plan[0] = kPfMagic;
  plan[1] = (int32_t)items.size();
  for (int i = 2; i < kPlanHeaderInts; ++i) plan[i] = 0;
  if (!items.empty())
    memcpy(plan + kPlanHeaderInts, items.data(), items.size() * sizeof(PrefillItem));
  info->num_items = (int32_t)items.size();
  info->total_tiles = total_tiles > INT32_MAX ? INT32_MAX : (int32_t)total_tiles;
  info->plan_ints = kPlanHeaderInts + kPfItemInts * (int32_t)items.size();
  info->reserved = 0;
  return B200_OK;
}

extern "C" int b200_paged_prefill_gqa(const void* q, int64_t q_stride, const void* key_cache,
                                      const void* value_cache, int num_blocks, int block_size,
                                      const int32_t* block_table, int64_t bt_stride,
                                      const int32_t* plan_dev, const b200_prefill_plan_info* info,
                                      int num_q_heads, int num_kv_heads, int head_dim, float scale,
                                      void* out, int out_is_f32, float* lse_out, int32_t* status,
                                      void* stream) {
  if (!info) {
    set_last_error("paged_prefill_gqa: plan info is null");
    return B200_EINVAL;
  }
  if (info->num_items == 0) return B200_OK;
  if (!q || !key_cache || !value_cache || !block_table || !plan_dev || !out || num_blocks <= 0 ||
      num_q_heads <= 0 || num_kv_heads <= 0 || num_q_heads % num_kv_heads) {
    set_last_error("paged_prefill_gqa: null pointer or bad head counts");
    return B200_EINVAL;
  }
  if (head_dim != kPfHeadDim) {
    set_last_error("paged_prefill_gqa: head_dim %d unsupported (kernel is built for 128)", head_dim);
    return B200_EUNSUPPORTED;
  }
  if (block_size < 8 || (block_size & (block_size - 1))) {
    set_last_error("paged_prefill_gqa: block_size %d must be a power of two >= 8", block_size);
    return B200_EUNSUPPORTED;
  }
  if (reinterpret_cast<uintptr_t>(q) % 4 || (q_stride % 2) || q_stride < (int64_t)num_q_heads * head_dim ||
      reinterpret_cast<uintptr_t>(out) % 16) {
    set_last_error("paged_prefill_gqa: q must be 4-byte aligned with an even stride >= Hq*D, out 16-byte aligned");
    return B200_EALIGN;
  }
  const int box_tokens = block_size < kTileTokens ? block_size : kTileTokens;
  CUtensorMap k_map, v_map;
  int rc = get_cache_tensor_map(key_cache, num_blocks, block_size, num_kv_heads, head_dim, box_tokens, &k_map);
  if (rc) return rc;
  rc = get_cache_tensor_map(value_cache, num_blocks, block_size, num_kv_heads, head_dim, box_tokens, &v_map);
  if (rc) return rc;

  PrefillParams p;
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.q_stride = q_stride;
  p.block_table = block_table;
  p.bt_stride = bt_stride;
  p.items = reinterpret_cast<const PrefillItem*>(plan_dev + kPlanHeaderInts);
  p.num_items = info->num_items;
  p.out = out;
  p.lse_out = lse_out;
  p.status = status;
  p.num_q_heads = num_q_heads;
  p.group = num_q_heads / num_kv_heads;
  p.block_size = block_size;
  p.block_shift = __builtin_ctz(block_size);
  p.num_blocks = num_blocks;
  p.box_tokens = box_tokens;
  p.boxes_per_tile = kTileTokens / box_tokens;
  p.out_is_f32 = out_is_f32;
  p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;

  const size_t smem = sizeof(PrefillSmem) + 1024;
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 64 || !attr_set[dev]) {
    rc = check_cuda(cudaFuncSetAttribute(paged_prefill_gqa_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem),
                    "paged_prefill_gqa smem attribute");
    if (rc) return rc;
    if (dev < 64) attr_set[dev] = true;
  }
  int grid = b200_sm_count();
  if (grid <= 0) grid = 148;
  if (grid > info->num_items) grid = info->num_items;
  paged_prefill_gqa_kernel<<<grid, kPfThreads, smem, static_cast<cudaStream_t>(stream)>>>(k_map, v_map, p);
  return check_cuda(cudaGetLastError(), "paged_prefill_gqa launch");
}
