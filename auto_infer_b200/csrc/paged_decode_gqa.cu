// Split-KV paged GQA decode / MTP-verify attention for sm_100a.
//
// HBM-bound: every key/value byte is read exactly once, so the kernel is built
// around keeping enough loads in flight per SM.  One persistent CTA per SM:
//   * warp 8 (producer) walks the CTA's work items and streams 64-token K and V
//     tiles of the (sequence, kv head) pair into a 6-stage shared-memory ring
//     with TMA (cp.async.bulk.tensor, 128-byte swizzle), block ids coming from
//     the block table; it runs ahead across item boundaries, so the ring never
//     drains between items;
//   * warps 0-7 (consumers) are two groups of four that take alternate tiles;
//     inside a tile each warp owns 16 tokens: S = Q K^T and O += P V run on
//     mma.sync m16n8k16 (all q_len*group <= 16 query rows of the pair share the
//     tile), with a warp-shuffle online softmax in fp32;
//   * at the end of an item the eight warps merge their (m, l, O) through shared
//     memory in a fixed order (deterministic) and write either the final bf16
//     rows (the item covered the whole pair) or one fp32 partial (o, lse).
// A second small kernel (split_merge.cuh, launched with programmatic dependent
// launch) merges the partials of pairs that were cut; merging inside this kernel
// by the last-arriving CTA was tried and put the merge's dependent L2 loads on the
// consumers' critical path for no gain.
//
// Algorithmic bytes per launch: sum_b kv_len_b * 2 * Hkv * 128 * 2 B (+ q, o).
#include "common.cuh"
#include "decode_plan.h"
#include "split_merge.cuh"

namespace b200 {

constexpr int kHeadDim = 128;
// The stage count must be even: the two consumer groups take alternate tiles, and
// with an even ring each stage (and its pair of mbarriers) belongs to one group
// for ever, so that group observes every phase of its barriers in order.  With an
// odd ring a group would revisit a stage only every second phase, and a parity
// wait cannot tell phase n from phase n-2.
constexpr int kStages = 6;
static_assert(kStages % 2 == 0, "each stage must always be consumed by the same warp group");
constexpr int kConsumerWarps = 8;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kDecodeThreads = kConsumerThreads + 32;
constexpr int kHalfTileBytes = kTileTokens * 128;            // [64 tokens][64 dims] bf16
constexpr int kTileBytes = 2 * kHalfTileBytes;               // K or V tile of one stage
constexpr int kStageBytes = 2 * kTileBytes;                  // K + V
constexpr int kSlotFloats = kMaxRows * kHeadDim;             // one warp's O in the merge buffer

struct __align__(1024) DecodeSmem {
  uint8_t stage[kStages][kStageBytes];                       // [K lo | K hi | V lo | V hi]
  float slots[4][kSlotFloats];                               // merge buffer, 4 warps at a time
  float red_m[kConsumerWarps][kMaxRows];
  float red_l[kConsumerWarps][kMaxRows];
  uint64_t full[kStages];
  uint64_t empty[kStages];
  int abort_flag;
};

static_assert(sizeof(DecodeSmem) + 1024 <= 227 * 1024, "shared memory budget of one CTA");

struct DecodeParams {
  const __nv_bfloat16* q;
  int64_t q_stride;                 // elements between query tokens
  const int32_t* block_table;
  int64_t bt_stride;
  int32_t* plan;                    // the pairs' arrival counters in it are updated by the kernel
  float* part_o;                    // (num_partials, 16, 128) fp32
  float* part_lse;                  // (num_partials, 16)
  void* out;                        // (T, Hq, 128) bf16 or fp32
  float* lse_out;                   // (T, Hq) or null
  int32_t* status;
#ifdef B200_TRACE
  long long* trace;                 // %globaltimer samples, 16 per CTA (debug builds)
#endif
  int num_q_heads, num_kv_heads, group;
  int block_size, block_shift, num_blocks;
  int box_tokens, boxes_per_tile;
  int out_is_f32;
  int off_cta, off_items, off_multi;   // plan offsets (derivable from the grid size and item count)
  float scale, scale_log2;
};

// Walks the CTA's (item, tile) sequence; identical in producer and consumers.
struct TileWalker {
  const DecodeItem* items;
  int item, item_end, tile, tile_end;
  DecodeItem cur;
  __device__ __forceinline__ void load() {
    if (item < item_end) {
      const int4* p = reinterpret_cast<const int4*>(items + item);
      int4 a = __ldg(p), b = __ldg(p + 1), c = __ldg(p + 2);
      cur.seq = a.x; cur.kv_head = a.y; cur.tile_begin = a.z; cur.tile_end = a.w;
      cur.kv_len = b.x; cur.q_start = b.y; cur.q_len = b.z; cur.causal_base = b.w;
      cur.partial_idx = c.x; cur.direct = c.y; cur.multi_idx = c.z;
      tile = cur.tile_begin;
      tile_end = cur.tile_end;
    }
  }
};

__global__ void __launch_bounds__(kDecodeThreads, 1)
paged_decode_gqa_kernel(const __grid_constant__ CUtensorMap k_map,
                        const __grid_constant__ CUtensorMap v_map, const DecodeParams p) {
  extern __shared__ uint8_t smem_raw[];
  DecodeSmem& sm = *reinterpret_cast<DecodeSmem*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int32_t* plan = p.plan;
  const int32_t* cta_off = plan + p.off_cta;
  const DecodeItem* items = reinterpret_cast<const DecodeItem*>(plan + p.off_items);
  const int item_begin = cta_off[blockIdx.x];
  const int item_end = cta_off[blockIdx.x + 1];

  if (threadIdx.x == 0) {
    sm.abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&sm.full[s], 1);
      mbar_init(&sm.empty[s], 4);     // one arrival per warp of the consuming group
    }
    mbar_fence_init();
  }
  __syncthreads();
#ifdef B200_TRACE
  if (p.trace && threadIdx.x == 0) p.trace[blockIdx.x * 16 + 0] = (long long)global_timer_ns();
#endif
  grid_dep_launch();              // the next kernel may be scheduled; it waits for this grid itself
  grid_dep_wait();                // q and the step's new cache rows come from earlier kernels
#ifdef B200_TRACE
  if (p.trace && threadIdx.x == 0) p.trace[blockIdx.x * 16 + 1] = (long long)global_timer_ns();
#endif
  if (item_begin >= item_end) return;
  volatile int* abort_flag = &sm.abort_flag;

  if (warp == kConsumerWarps) {
    // ------------------------------ producer ------------------------------
    if (lane == 0) {
      tma_prefetch_desc(&k_map);
      tma_prefetch_desc(&v_map);
    }
    TileWalker w{items, item_begin, item_end, 0, 0, {}};
    w.load();
    uint32_t it = 0;
    const int nbox = p.boxes_per_tile;
    // block id of this lane's box for the current tile (lane < nbox)
    auto fetch_block = [&](const TileWalker& tw) -> int {
      if (lane >= nbox) return 0;
      const int last_block = (tw.cur.kv_len - 1) >> p.block_shift;
      int lb = ((tw.tile * kTileTokens) >> p.block_shift) + lane;
      lb = lb > last_block ? last_block : lb;       // tail boxes re-read the last valid page
      return __ldg(p.block_table + (int64_t)tw.cur.seq * p.bt_stride + lb);
    };
    int bid = fetch_block(w);
    while (w.item < w.item_end) {
      // look one tile ahead so the block-table read overlaps the wait below
      TileWalker nxt = w;
      ++nxt.tile;
      if (nxt.tile >= nxt.tile_end) {
        ++nxt.item;
        nxt.load();
      }
      int bid_next = 0;
      if (nxt.item < nxt.item_end) bid_next = fetch_block(nxt);

      const int s = it % kStages;
      const uint32_t ph = (it / kStages) & 1u;
      if (lane == 0) {
        mbar_wait_bounded(&sm.empty[s], ph ^ 1u, abort_flag, p.status);
        mbar_arrive_expect_tx(&sm.full[s], kStageBytes);
      }
      __syncwarp();
      if (lane < nbox) {
        int b = bid;
        if (b < 0 || b >= p.num_blocks) {           // out-of-pool id: TMA zero-fills, flag it
          if (p.status) atomicOr(p.status, B200_STATUS_BAD_BLOCK);
          b = p.num_blocks;
        }
        const int tok = (w.tile * kTileTokens + lane * p.box_tokens) & (p.block_size - 1);
        uint8_t* dst = sm.stage[s] + lane * p.box_tokens * 128;
        const int h = w.cur.kv_head;
#ifdef B200_TRACE
        if (p.trace && lane == 0 && it == 0) p.trace[blockIdx.x * 16 + 2] = (long long)global_timer_ns();
#endif
        tma_load_4d(dst, &k_map, &sm.full[s], 0, h, tok, b);
        tma_load_4d(dst + kHalfTileBytes, &k_map, &sm.full[s], 64, h, tok, b);
        tma_load_4d(dst + kTileBytes, &v_map, &sm.full[s], 0, h, tok, b);
        tma_load_4d(dst + kTileBytes + kHalfTileBytes, &v_map, &sm.full[s], 64, h, tok, b);
      }
      __syncwarp();
      ++it;
      w = nxt;
      bid = bid_next;
    }
    // drain: do not leave while copies may still land in this CTA's shared memory
    if (lane == 0) {
      const uint32_t n = it < (uint32_t)kStages ? it : (uint32_t)kStages;
      for (uint32_t k = 0; k < n; ++k) {
        const uint32_t j = it - 1 - k;
        mbar_wait_bounded(&sm.full[j % kStages], (j / kStages) & 1u, abort_flag, p.status);
      }
    }
    return;
  }

  // -------------------------------- consumers --------------------------------
  const int grp = warp >> 2;          // which tiles (parity of the running tile counter)
  const int wslice = warp & 3;        // 16-token slice of the tile
  const int quad = lane >> 2;         // fragment row (and row + 8)
  const int qlane = lane & 3;
  const int G = p.group;

  // ldmatrix lane addressing (byte offsets inside a 64-token half tile, before swizzle)
  const int k_tok = wslice * 16 + ((lane >> 4) << 3) + (lane & 7);   // K: matrices 2,3 -> tokens +8
  const int k_chunk_sel = (lane >> 3) & 1;                           // K: matrices 1,3 -> dims +8
  const int v_tok = wslice * 16 + (((lane >> 3) & 1) << 3) + (lane & 7);  // V: matrices 1,3 -> tokens +8
  const int v_chunk_sel = lane >> 4;                                 // V: matrices 2,3 -> dims +8

  TileWalker w{items, item_begin, item_end, 0, 0, {}};
  w.load();
  uint32_t it = 0;

  // Q fragments of an item: 8 k-steps x 4 registers, rows beyond q_len*group are zero.
  // They are fetched for the NEXT item right after the tile loop, so the global
  // loads fly while the warps merge and write the current item.
  uint32_t qf[8][4];
  auto load_q = [&](const DecodeItem& qi) {
    const int qrows = qi.q_len * G;
    const int r0 = quad, r1 = quad + 8;
    const __nv_bfloat16* q0 = nullptr;
    const __nv_bfloat16* q1 = nullptr;
    if (r0 < qrows)
      q0 = p.q + (int64_t)(qi.q_start + r0 / G) * p.q_stride + (int64_t)(qi.kv_head * G + r0 % G) * kHeadDim;
    if (r1 < qrows)
      q1 = p.q + (int64_t)(qi.q_start + r1 / G) * p.q_stride + (int64_t)(qi.kv_head * G + r1 % G) * kHeadDim;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      const int c = ks * 16 + qlane * 2;
      qf[ks][0] = q0 ? __ldg(reinterpret_cast<const uint32_t*>(q0 + c)) : 0u;
      qf[ks][1] = q1 ? __ldg(reinterpret_cast<const uint32_t*>(q1 + c)) : 0u;
      qf[ks][2] = q0 ? __ldg(reinterpret_cast<const uint32_t*>(q0 + c + 8)) : 0u;
      qf[ks][3] = q1 ? __ldg(reinterpret_cast<const uint32_t*>(q1 + c + 8)) : 0u;
    }
  };
  load_q(w.cur);

  while (w.item < w.item_end) {
    const DecodeItem item = w.cur;
    const int rows = item.q_len * G;
    // last visible key per fragment row (-1: row unused, everything masked)
    const int lim0 = quad < rows ? min(item.causal_base + quad / G, item.kv_len - 1) : -1;
    const int lim1 = quad + 8 < rows ? min(item.causal_base + (quad + 8) / G, item.kv_len - 1) : -1;

    float o[16][4];
#pragma unroll
    for (int n = 0; n < 16; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

    for (int tile = item.tile_begin; tile < item.tile_end; ++tile, ++it) {
      if ((int)(it & 1u) != grp) continue;
      const int s = it % kStages;
      mbar_wait_bounded(&sm.full[s], (it / kStages) & 1u, abort_flag, p.status);
      const uint32_t kbase = smem_u32(sm.stage[s]);
      const uint32_t vbase = kbase + kTileBytes;

      // ---- S = Q K^T for this warp's 16 tokens (two n-tiles of 8)
      float sacc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        const int chunk = ks * 2 + k_chunk_sel;          // 16-byte chunk of the 128-dim row
        uint32_t kb[4];
        ldmatrix_x4(kb, kbase + (chunk >> 3) * kHalfTileBytes + swz128(k_tok, chunk & 7));
        mma_bf16_16816(sacc[0], qf[ks], kb[0], kb[1]);
        mma_bf16_16816(sacc[1], qf[ks], kb[2], kb[3]);
      }
      // ---- mask + online softmax (fp32, exp2 domain)
      const int tok0 = tile * kTileTokens + wslice * 16 + qlane * 2;
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int n = 0; n < 2; ++n) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int j = tok0 + n * 8 + e;
          if (j > lim0) sacc[n][e] = -INFINITY;
          if (j > lim1) sacc[n][2 + e] = -INFINITY;
          mx0 = fmaxf(mx0, sacc[n][e]);
          mx1 = fmaxf(mx1, sacc[n][2 + e]);
        }
      }
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
      const float ms0 = (mn0 == -INFINITY) ? 0.f : mn0 * p.scale_log2;
      const float ms1 = (mn1 == -INFINITY) ? 0.f : mn1 * p.scale_log2;
      if (__any_sync(0xffffffffu, (mn0 != m0) || (mn1 != m1))) {
        const float c0 = fast_exp2(m0 * p.scale_log2 - ms0);   // m = -inf -> exp2(-inf) = 0
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
      uint32_t pf[4];
      {
        float pr[2][4];
#pragma unroll
        for (int n = 0; n < 2; ++n) {
          pr[n][0] = fast_exp2(fmaf(sacc[n][0], p.scale_log2, -ms0));
          pr[n][1] = fast_exp2(fmaf(sacc[n][1], p.scale_log2, -ms0));
          pr[n][2] = fast_exp2(fmaf(sacc[n][2], p.scale_log2, -ms1));
          pr[n][3] = fast_exp2(fmaf(sacc[n][3], p.scale_log2, -ms1));
          l0 += pr[n][0] + pr[n][1];
          l1 += pr[n][2] + pr[n][3];
        }
        pf[0] = pack_bf16(pr[0][0], pr[0][1]);
        pf[1] = pack_bf16(pr[0][2], pr[0][3]);
        pf[2] = pack_bf16(pr[1][0], pr[1][1]);
        pf[3] = pack_bf16(pr[1][2], pr[1][3]);
      }
      // ---- O += P V (k = this warp's 16 tokens, n = 128 dims)
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int chunk = j * 2 + v_chunk_sel;
        uint32_t vb[4];
        ldmatrix_x4_trans(vb, vbase + (chunk >> 3) * kHalfTileBytes + swz128(v_tok, chunk & 7));
        mma_bf16_16816(o[2 * j], pf, vb[0], vb[1]);
        mma_bf16_16816(o[2 * j + 1], pf, vb[2], vb[3]);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&sm.empty[s]);
#ifdef B200_TRACE
      if (p.trace && lane == 0 && warp < 2) {
        if (it < 2) p.trace[blockIdx.x * 16 + 3 + warp * 4] = (long long)global_timer_ns();   // first tile done
        p.trace[blockIdx.x * 16 + 4 + warp * 4] = (long long)global_timer_ns();               // latest tile done
        p.trace[blockIdx.x * 16 + 6] = it + 1;
      }
#endif
    }

    // ---- next item's Q on its way, then merge the eight warps (fixed order) and write the result
    ++w.item;
    w.load();
    if (w.item < w.item_end) load_q(w.cur);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    if (qlane == 0) {
      sm.red_m[warp][quad] = m0;
      sm.red_m[warp][quad + 8] = m1;
      sm.red_l[warp][quad] = l0;
      sm.red_l[warp][quad + 8] = l1;
    }
    named_bar_sync(1, kConsumerThreads);
    {
      float g0 = -INFINITY, g1 = -INFINITY;
#pragma unroll
      for (int ww = 0; ww < kConsumerWarps; ++ww) {
        g0 = fmaxf(g0, sm.red_m[ww][quad]);
        g1 = fmaxf(g1, sm.red_m[ww][quad + 8]);
      }
      const float f0 = (m0 == -INFINITY) ? 0.f : fast_exp2((m0 - g0) * p.scale_log2);
      const float f1 = (m1 == -INFINITY) ? 0.f : fast_exp2((m1 - g1) * p.scale_log2);
#pragma unroll
      for (int n = 0; n < 16; ++n) {
        o[n][0] *= f0; o[n][1] *= f0; o[n][2] *= f1; o[n][3] *= f1;
      }
    }
    auto store_slot = [&](float* slot) {
#pragma unroll
      for (int n = 0; n < 16; ++n) {
        const int col = n * 8 + qlane * 2;
        *reinterpret_cast<float2*>(slot + quad * kHeadDim + col) = make_float2(o[n][0], o[n][1]);
        *reinterpret_cast<float2*>(slot + (quad + 8) * kHeadDim + col) = make_float2(o[n][2], o[n][3]);
      }
    };
    if (warp >= 4) store_slot(sm.slots[warp - 4]);
    named_bar_sync(1, kConsumerThreads);
    if (warp < 4) {
      const float* slot = sm.slots[warp];
#pragma unroll
      for (int n = 0; n < 16; ++n) {
        const int col = n * 8 + qlane * 2;
        const float2 a = *reinterpret_cast<const float2*>(slot + quad * kHeadDim + col);
        const float2 b = *reinterpret_cast<const float2*>(slot + (quad + 8) * kHeadDim + col);
        o[n][0] += a.x; o[n][1] += a.y; o[n][2] += b.x; o[n][3] += b.y;
      }
    }
    named_bar_sync(1, kConsumerThreads);
    if (warp < 4) store_slot(sm.slots[warp]);
    named_bar_sync(1, kConsumerThreads);
    {
      // 256 threads: thread -> (row, 8 columns)
      const int t = threadIdx.x;
      const int row = t >> 4;
      const int col = (t & 15) * 8;
      if (row < rows) {
        float g = -INFINITY;
#pragma unroll
        for (int ww = 0; ww < kConsumerWarps; ++ww) g = fmaxf(g, sm.red_m[ww][row]);
        float lsum = 0.f;
#pragma unroll
        for (int ww = 0; ww < kConsumerWarps; ++ww) {
          const float mw = sm.red_m[ww][row];
          lsum += (mw == -INFINITY) ? 0.f : sm.red_l[ww][row] * fast_exp2((mw - g) * p.scale_log2);
        }
        const float inv = lsum > 0.f ? 1.f / lsum : 0.f;
        float v[8];
#pragma unroll
        for (int c = 0; c < 8; c += 4) {
          float4 acc = *reinterpret_cast<const float4*>(&sm.slots[0][row * kHeadDim + col + c]);
#pragma unroll
          for (int sl = 1; sl < 4; ++sl) {
            const float4 x = *reinterpret_cast<const float4*>(&sm.slots[sl][row * kHeadDim + col + c]);
            acc.x += x.x; acc.y += x.y; acc.z += x.z; acc.w += x.w;
          }
          v[c] = acc.x * inv; v[c + 1] = acc.y * inv; v[c + 2] = acc.z * inv; v[c + 3] = acc.w * inv;
        }
        const float lse = lsum > 0.f ? g * p.scale + __logf(lsum) : -INFINITY;
        if (item.direct) {
          const int64_t tok = item.q_start + row / G;
          const int head = item.kv_head * G + row % G;
          const int64_t off = (tok * p.num_q_heads + head) * kHeadDim + col;
          if (p.out_is_f32) {
            float* dst = reinterpret_cast<float*>(p.out) + off;
            *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
            *reinterpret_cast<float4*>(dst + 4) = make_float4(v[4], v[5], v[6], v[7]);
          } else {
            uint4 pk;
            pk.x = pack_bf16(v[0], v[1]); pk.y = pack_bf16(v[2], v[3]);
            pk.z = pack_bf16(v[4], v[5]); pk.w = pack_bf16(v[6], v[7]);
            *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.out) + off) = pk;
          }
          if (p.lse_out && (t & 15) == 0) p.lse_out[tok * p.num_q_heads + head] = lse;
        } else {
          float* dst = p.part_o + ((int64_t)item.partial_idx * kMaxRows + row) * kHeadDim + col;
          *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
          *reinterpret_cast<float4*>(dst + 4) = make_float4(v[4], v[5], v[6], v[7]);
          if ((t & 15) == 0) p.part_lse[(int64_t)item.partial_idx * kMaxRows + row] = lse;
        }
      }
    }
#ifdef B200_TRACE
    if (p.trace && threadIdx.x == 0) p.trace[blockIdx.x * 16 + 5] = (long long)global_timer_ns();   // item written
#endif
    // the next item's first shared-memory write of the merge area comes after
    // its own first barrier, which no thread passes before finishing the reads above
  }
}

}  // namespace b200

#ifdef B200_TRACE
static long long* g_trace = nullptr;
extern "C" void b200_debug_set_trace(void* dev_ptr) { g_trace = static_cast<long long*>(dev_ptr); }
#endif

extern "C" int b200_paged_decode_gqa(const void* q, int64_t q_stride, const void* key_cache,
                                     const void* value_cache, int num_blocks, int block_size,
                                     const int32_t* block_table, int64_t bt_stride,
                                     int32_t* plan_dev, const b200_decode_plan_info* info,
                                     int num_q_heads, int num_kv_heads, int head_dim, float scale,
                                     void* workspace, size_t workspace_bytes, void* out,
                                     int out_is_f32, float* lse_out, int32_t* status,
                                     void* stream) {
  using namespace b200;
  if (!info) {
    set_last_error("paged_decode_gqa: plan info is null");
    return B200_EINVAL;
  }
  if (info->num_items == 0) return B200_OK;
  if (!q || !key_cache || !value_cache || !block_table || !plan_dev || !out || !workspace ||
      num_blocks <= 0 || num_q_heads <= 0 || num_kv_heads <= 0 || num_q_heads % num_kv_heads) {
    set_last_error("paged_decode_gqa: null pointer or bad head counts");
    return B200_EINVAL;
  }
  if (head_dim != kHeadDim) {
    set_last_error("paged_decode_gqa: head_dim %d unsupported (kernel is built for 128)", head_dim);
    return B200_EUNSUPPORTED;
  }
  if (block_size < 8 || (block_size & (block_size - 1))) {
    set_last_error("paged_decode_gqa: block_size %d must be a power of two >= 8", block_size);
    return B200_EUNSUPPORTED;
  }
  if (reinterpret_cast<uintptr_t>(q) % 4 || (q_stride % 2) || q_stride < (int64_t)num_q_heads * head_dim) {
    set_last_error("paged_decode_gqa: q must be 4-byte aligned with an even token stride >= Hq*D");
    return B200_EALIGN;
  }
  if (reinterpret_cast<uintptr_t>(out) % 16 || reinterpret_cast<uintptr_t>(workspace) % 16) {
    set_last_error("paged_decode_gqa: out and workspace must be 16-byte aligned");
    return B200_EALIGN;
  }
  const size_t need = (size_t)info->num_partials * (kMaxRows * (size_t)kHeadDim + kMaxRows) * sizeof(float);
  if (workspace_bytes < need) {
    set_last_error("paged_decode_gqa: workspace %zu bytes < %zu needed", workspace_bytes, need);
    return B200_EPLAN;
  }
  const int box_tokens = block_size < kTileTokens ? block_size : kTileTokens;
  CUtensorMap k_map, v_map;
  int rc = get_cache_tensor_map(key_cache, num_blocks, block_size, num_kv_heads, head_dim, box_tokens, &k_map);
  if (rc) return rc;
  rc = get_cache_tensor_map(value_cache, num_blocks, block_size, num_kv_heads, head_dim, box_tokens, &v_map);
  if (rc) return rc;

  DecodeParams p;
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.q_stride = q_stride;
  p.block_table = block_table;
  p.bt_stride = bt_stride;
  p.plan = plan_dev;
  p.off_cta = kPlanHeaderInts;
  p.off_items = p.off_cta + round_up4(info->num_ctas + 1);
  p.off_multi = p.off_items + kItemInts * info->num_items;
  p.part_o = static_cast<float*>(workspace);
  p.part_lse = p.part_o + (size_t)info->num_partials * kMaxRows * kHeadDim;
  p.out = out;
  p.lse_out = lse_out;
  p.status = status;
#ifdef B200_TRACE
  p.trace = g_trace;
#endif
  p.num_q_heads = num_q_heads;
  p.num_kv_heads = num_kv_heads;
  p.group = num_q_heads / num_kv_heads;
  p.block_size = block_size;
  p.block_shift = __builtin_ctz(block_size);
  p.num_blocks = num_blocks;
  p.box_tokens = box_tokens;
  p.boxes_per_tile = kTileTokens / box_tokens;
  p.out_is_f32 = out_is_f32;
  p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;

  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const size_t smem = sizeof(DecodeSmem) + 1024;
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 64 || !attr_set[dev]) {
    rc = check_cuda(cudaFuncSetAttribute(paged_decode_gqa_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem),
                    "paged_decode_gqa smem attribute");
    if (rc) return rc;
    if (dev < 64) attr_set[dev] = true;
  }
  rc = check_cuda(launch_pdl(paged_decode_gqa_kernel, dim3(info->num_ctas), dim3(kDecodeThreads), smem, s,
                             k_map, v_map, p),
                  "paged_decode_gqa launch");
  if (rc) return rc;
  if (info->num_multi > 0) {
    rc = check_cuda(launch_pdl(split_merge_kernel<kHeadDim>, dim3(split_merge_grid<kHeadDim>(info->num_multi)),
                               dim3(128), 0, s, (const int32_t*)plan_dev, (const float*)p.part_o,
                               (const float*)p.part_lse, out, lse_out, num_q_heads, p.group, out_is_f32),
                    "decode_merge launch");
  }
  return rc;
}

// ---------------------------------------------------------------------------
// Allocation-free variant.  Some hosts of this library may not allocate device
// memory when a step runs: a serving engine that gave every free byte of HBM to
// its paged KV pool at start-up has nothing left to allocate from, and a decode
// loop that must keep its latency cannot afford the device-wide synchronisation
// an allocation or a free implies.  For them the split-KV partial records live
// in a fixed array that is part of the loaded module: it exists on every GPU
// that loads the library, from load to exit, whether or not this entry point is
// ever called.
// ---------------------------------------------------------------------------
namespace b200 {
constexpr int kStaticMaxPartials = 1024;   // (o, lse) records; 8 256 B each -> 8.06 MiB in total
constexpr size_t kStaticScratchFloats = (size_t)kStaticMaxPartials * (kMaxRows * kHeadDim + kMaxRows);
static __device__ __align__(256) float g_decode_scratch[kStaticScratchFloats];
}  // namespace b200

extern "C" int b200_paged_decode_gqa_static(const void* q, int64_t q_stride, const void* key_cache,
                                            const void* value_cache, int num_blocks, int block_size,
                                            const int32_t* block_table, int64_t bt_stride,
                                            int32_t* plan_dev,
                                            const b200_decode_plan_info* info, int num_q_heads,
                                            int num_kv_heads, int head_dim, float scale, void* out,
                                            int out_is_f32, float* lse_out, int32_t* status,
                                            void* stream) {
  using namespace b200;
  if (!info) {
    set_last_error("paged_decode_gqa_static: plan info is null");
    return B200_EINVAL;
  }
  if (info->num_partials > kStaticMaxPartials) {
    set_last_error("paged_decode_gqa_static: the plan needs %d partial records but the built-in scratch "
                   "holds %d; plan with fewer CTAs or use b200_paged_decode_gqa with a caller workspace",
                   info->num_partials, kStaticMaxPartials);
    return B200_ETOOLARGE;
  }
  // In host code the array's name is only a handle; the device address has to be
  // asked for, once per device, with that device current.
  static float* scratch_addr[64] = {nullptr};
  int dev = 0;
  int rc = check_cuda(cudaGetDevice(&dev), "paged_decode_gqa_static cudaGetDevice");
  if (rc) return rc;
  if (dev < 0 || dev >= 64) {
    set_last_error("paged_decode_gqa_static: device ordinal %d outside the supported 0..63", dev);
    return B200_EUNSUPPORTED;
  }
  if (scratch_addr[dev] == nullptr) {
    float* addr = nullptr;
    rc = check_cuda(cudaGetSymbolAddress(reinterpret_cast<void**>(&addr), g_decode_scratch),
                    "paged_decode_gqa_static cudaGetSymbolAddress");
    if (rc) return rc;
    scratch_addr[dev] = addr;
  }
  return b200_paged_decode_gqa(q, q_stride, key_cache, value_cache, num_blocks, block_size, block_table,
                               bt_stride, plan_dev, info, num_q_heads, num_kv_heads, head_dim, scale,
                               scratch_addr[dev], kStaticScratchFloats * sizeof(float), out, out_is_f32,
                               lse_out, status, stream);
}
