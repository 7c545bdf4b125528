// Absorbed-MLA decode attention for sm_100a: all heads attend one shared latent
// "kv head" of width kv_lora_rank + rope (512 + 64), stored ONCE per token; the
// same shared-memory tile serves as K (576 wide) and as V (its first 512 dims).
//
// HBM-bound at 16 heads (34 816 flop per 1 152-byte latent row = 30 flop/B), so
// the design is the split-KV streaming design of the GQA decode kernel:
//   * host plan: 32-token latent tiles of all sequences laid end to end and cut
//     into one equal range per CTA (persistent CTA per SM);
//   * producer warp: nine 4 KB TMA boxes (64 dims x 32 tokens, 128-byte swizzle)
//     per tile into a 4-stage ring (36 KB per stage);
//   * two consumer groups of four warps take alternate tiles (even ring: a stage
//     always belongs to one group).  Inside a group every warp computes a
//     quarter of S = Q K^T (16 of the tile's 32 tokens x half of the 576 dims;
//     q_len*heads <= 16 rows form the M of mma.sync m16n8k16, Q fragments come
//     from shared memory), the four partial score blocks meet in shared memory
//     behind ONE barrier per tile, every warp then holds the full 16 x 32 scores
//     in MMA-fragment layout, runs the same online softmax (identical row state
//     in all four warps, nothing else to exchange) and accumulates O += P V for
//     its 128 of the 512 value dims with P straight from registers;
//   * the groups' (m, l, O) are merged in a fixed order at the end of an item.
// Algorithmic bytes per launch: sum_b kv_len_b * 1 152 B (+ q, o).
#include <algorithm>

#include "common.cuh"
#include "decode_plan.h"
#include "split_merge.cuh"

namespace b200 {

constexpr int kLatentDim = 576;
constexpr int kValueDim = 512;
constexpr int kMlaSub = kLatentDim / 64;                      // 64-dim sub-tiles per latent row
constexpr int kMlaSubBytes = kMlaTileTokens * 128;            // [32 tokens][64 dims] bf16
constexpr int kMlaStageBytes = kMlaSub * kMlaSubBytes;        // 36 864
constexpr int kMlaStages = 4;
// Tiles alternate between the two consumer groups.  With an even ring a group meets every
// phase of the stages it uses; with an odd ring it would meet every other phase only, and a
// parity wait cannot tell phase k from phase k + 2: a group running ahead would read a stage
// before its tile has landed.
static_assert(kMlaStages % 2 == 0, "each stage must always be consumed by the same warp group");
constexpr int kMlaWarps = 8;
constexpr int kMlaConsumerThreads = kMlaWarps * 32;
constexpr int kMlaThreads = kMlaConsumerThreads + 32;
constexpr int kQPitch = kLatentDim * 2 + 16;                  // bytes per Q row in shared memory

struct __align__(1024) MlaSmem {
  uint8_t stage[kMlaStages][kMlaStageBytes];
  float slots[4][kMaxRows * 128];                             // merge buffer: one 128-dim slice per warp pair
  __align__(16) uint8_t qbuf[kMaxRows * kQPitch];
  float s_part[2][2][4][32 * 8];                              // [group][tile parity][warp][lane x 8] partial scores
  float red_m[2][kMaxRows];
  float red_l[kMlaWarps][kMaxRows];
  uint64_t full[kMlaStages];
  uint64_t empty[kMlaStages];
  int abort_flag;
};
static_assert(sizeof(MlaSmem) + 1024 <= 227 * 1024, "shared memory budget of one CTA");

struct MlaParams {
  const __nv_bfloat16* q;          // (T, H, 576)
  int64_t q_stride;
  const int32_t* block_table;
  int64_t bt_stride;
  const int32_t* plan;
  float* part_o;                   // (num_partials, 16, 512)
  float* part_lse;                 // (num_partials, 16)
  void* out;                       // (T, H, 512) bf16 or fp32
  float* lse_out;
  int32_t* status;
  int num_heads;
  int max_partials;                // records the workspace holds
  int block_size, block_shift, num_blocks, box_tokens, boxes_per_tile;
  int out_is_f32;
  float scale, scale_log2;
#ifdef B200_TRACE
  long long* trace;                // clock samples of CTA 0, 8 per tile (debug builds)
#endif
};

#ifdef B200_TRACE
#define MLA_TRACE(slot, tileno)                                                                  \
  do {                                                                                           \
    if (p.trace && blockIdx.x == 0 && lane == 0 && (tileno) < 64) p.trace[(tileno) * 8 + (slot)] = clock64(); \
  } while (0)
// per-CTA time stamps (ns): entry, dependency met, first / last tile consumed, end; tiles, items
#define MLA_CTA_TRACE(slot, value)                                                               \
  do {                                                                                           \
    if (p.trace && threadIdx.x == 0) p.trace[4096 + blockIdx.x * 8 + (slot)] = (long long)(value); \
  } while (0)
#else
#define MLA_TRACE(slot, tileno) do {} while (0)
#define MLA_CTA_TRACE(slot, value) do {} while (0)
#endif

struct MlaWalker {
  const DecodeItem* items;
  int item, item_end, tile, tile_end;
  DecodeItem cur;
  __device__ __forceinline__ void load() {
    if (item < item_end) {
      const int4* p = reinterpret_cast<const int4*>(items + item);
      int4 a = __ldg(p), b = __ldg(p + 1), c = __ldg(p + 2);
      cur.seq = a.x; cur.kv_head = a.y; cur.tile_begin = a.z; cur.tile_end = a.w;
      cur.kv_len = b.x; cur.q_start = b.y; cur.q_len = b.z; cur.causal_base = b.w;
      cur.partial_idx = c.x; cur.direct = c.y;
      tile = cur.tile_begin;
      tile_end = cur.tile_end;
    }
  }
};

__global__ void __launch_bounds__(kMlaThreads, 1)
mla_decode_kernel(const __grid_constant__ CUtensorMap lat_map, const MlaParams p) {
  extern __shared__ uint8_t smem_raw[];
  MlaSmem& sm = *reinterpret_cast<MlaSmem*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int32_t* plan = p.plan;
  const CtaRecord* cta_rec = reinterpret_cast<const CtaRecord*>(plan + plan[kHdrOffCta]) + blockIdx.x;
  const DecodeItem* items = reinterpret_cast<const DecodeItem*>(plan + plan[kHdrOffItems]);
  const int item_begin = cta_rec->item_begin;
  const int item_end = cta_rec->item_end;
  // read ahead of the dependency wait like the rest of the plan: it reaches the device by a copy,
  // never by the kernel in front
  const bool plan_ok = plan[kHdrMagic] == kPlanMagic && plan[kHdrNumCtas] == (int)gridDim.x;

  if (threadIdx.x == 0) {
    sm.abort_flag = 0;
    for (int s = 0; s < kMlaStages; ++s) {
      mbar_init(&sm.full[s], 1);
      mbar_init(&sm.empty[s], 4);
    }
    mbar_fence_init();
  }
  __syncthreads();
  MLA_CTA_TRACE(0, global_timer_ns());
  // While the kernels in front drain (the previous layer's merge, this step's slot write): the
  // first tiles of this CTA's first item are asked into L2 (hints only: block ids read past the
  // L1 and used for nothing but the prefetch addresses; the loads proper follow the dependency
  // wait and find a warm L2).
  if (warp == kMlaWarps && item_begin < item_end) {
    constexpr int kHintTiles = 3;
    const DecodeItem& f = cta_rec->first;
    const int nbox = p.boxes_per_tile;
    const int n_hint = min(f.tile_end - f.tile_begin, kHintTiles) * nbox;
    if (lane < n_hint && f.kv_len > 0) {
      const int tile = f.tile_begin + lane / nbox, box = lane % nbox;
      int lb = ((tile * kMlaTileTokens) >> p.block_shift) + box;
      const int last_block = (f.kv_len - 1) >> p.block_shift;
      lb = lb > last_block ? last_block : lb;
      const int bid = __ldcg(p.block_table + (int64_t)f.seq * p.bt_stride + lb);
      if (bid >= 0 && bid < p.num_blocks) {
        const int tok = (tile * kMlaTileTokens + box * p.box_tokens) & (p.block_size - 1);
#pragma unroll
        for (int c = 0; c < kMlaSub; ++c) tma_prefetch_4d(&lat_map, c * 64, 0, tok, bid);
      }
    }
  }
  grid_dep_launch();              // the merge kernel may be scheduled; it waits for this grid itself
  grid_dep_wait();                // q and the step's new latent rows come from earlier kernels
  MLA_CTA_TRACE(1, global_timer_ns());
  if (!plan_ok) {                 // not a plan for this launch
    if (threadIdx.x == 0 && p.status) atomicOr(p.status, B200_STATUS_BAD_LAUNCH);
    return;
  }
  if (item_begin >= item_end) return;
  volatile int* abort_flag = &sm.abort_flag;

  if (warp == kMlaWarps) {
    // ------------------------------ producer ------------------------------
    if (lane == 0) tma_prefetch_desc(&lat_map);
    MlaWalker w{items, item_begin, item_end, 0, 0, {}};
    w.load();
    uint32_t it = 0;
    const int nbox = p.boxes_per_tile;
    auto fetch_block = [&](const MlaWalker& tw) -> int {
      if (lane >= nbox) return 0;
      const int last_block = (tw.cur.kv_len - 1) >> p.block_shift;
      int lb = ((tw.tile * kMlaTileTokens) >> p.block_shift) + lane;
      lb = lb > last_block ? last_block : lb;
      return __ldg(p.block_table + (int64_t)tw.cur.seq * p.bt_stride + lb);
    };
    int bid = fetch_block(w);
    while (w.item < w.item_end) {
      MlaWalker nxt = w;
      ++nxt.tile;
      if (nxt.tile >= nxt.tile_end) {
        ++nxt.item;
        nxt.load();
      }
      int bid_next = 0;
      if (nxt.item < nxt.item_end) bid_next = fetch_block(nxt);
      const int s = it % kMlaStages;
      if (lane == 0) {
        mbar_wait_bounded(&sm.empty[s], ((it / kMlaStages) & 1u) ^ 1u, abort_flag, p.status);
        mbar_arrive_expect_tx(&sm.full[s], kMlaStageBytes);
        MLA_TRACE(6, it);
      }
      __syncwarp();
      // box i of the tile by lane i; each lane issues its nine 64-dim slices
      if (lane < nbox) {
        int b = bid;
        if (b < 0 || b >= p.num_blocks) {
          if (p.status) atomicOr(p.status, B200_STATUS_BAD_BLOCK);
          b = p.num_blocks;
        }
        const int tok = (w.tile * kMlaTileTokens + lane * p.box_tokens) & (p.block_size - 1);
        uint8_t* dst = sm.stage[s] + lane * p.box_tokens * 128;
#pragma unroll
        for (int c = 0; c < kMlaSub; ++c)
          tma_load_4d(dst + c * kMlaSubBytes, &lat_map, &sm.full[s], c * 64, 0, tok, b);
      }
      __syncwarp();
      ++it;
      w = nxt;
      bid = bid_next;
    }
    if (lane == 0) {
      const uint32_t n = it < (uint32_t)kMlaStages ? it : (uint32_t)kMlaStages;
      for (uint32_t k = 0; k < n; ++k) {
        const uint32_t j = it - 1 - k;
        mbar_wait_bounded(&sm.full[j % kMlaStages], (j / kMlaStages) & 1u, abort_flag, p.status);
      }
    }
    return;
  }

  // -------------------------------- consumers --------------------------------
  const int grp = warp >> 2;
  const int gw = warp & 3;             // warp within the group: S slice (0,1) and value-dim slice (0..3)
  const int quad = lane >> 2;
  const int qlane = lane & 3;
  const int G = p.num_heads;
  const int gbar = 1 + grp;            // named barrier of the group (128 threads)

  // ldmatrix lane addressing
  const int slice = gw & 1;            // 16-token slice of the tile this warp scores
  const int khalf = gw >> 1;           // latent sub-tiles [0,5) or [5,9)
  const int k_tok = slice * 16 + ((lane >> 4) << 3) + (lane & 7);     // K operand
  const int k_chunk_sel = (lane >> 3) & 1;
  const int v_tok_l = (((lane >> 3) & 1) << 3) + (lane & 7);          // V operand
  const int v_chunk_sel = lane >> 4;
  // A operands from row-major shared memory: matrices (r0-7,k0-7) (r8-15,k0-7) (r0-7,k8-15) (r8-15,k8-15)
  const int a_row = (lane & 7) + (((lane >> 3) & 1) << 3);
  const int a_koff = (lane >> 4) << 3;

  MlaWalker w{items, item_begin, item_end, 0, 0, {}};
  w.load();
  uint32_t it = 0;

  while (w.item < w.item_end) {
    const DecodeItem item = w.cur;
    const int rows = item.q_len * G;
    // ---- stage Q (rows x 576, zero padded to 16 rows) in shared memory: all loads of a
    // thread are issued before its first store, so their latencies overlap
    {
      constexpr int kChunks = kMaxRows * (kLatentDim / 8);              // 16-byte chunks
      constexpr int kPerThread = (kChunks + kMlaConsumerThreads - 1) / kMlaConsumerThreads;
      uint4 qv[kPerThread];
#pragma unroll
      for (int u = 0; u < kPerThread; ++u) {
        const int i = threadIdx.x + u * kMlaConsumerThreads;
        const int r = i / (kLatentDim / 8), c = i % (kLatentDim / 8);
        qv[u] = make_uint4(0u, 0u, 0u, 0u);
        if (i < kChunks && r < rows)
          qv[u] = __ldg(reinterpret_cast<const uint4*>(p.q + (int64_t)(item.q_start + r / G) * p.q_stride +
                                                       (int64_t)(r % G) * kLatentDim + c * 8));
      }
#pragma unroll
      for (int u = 0; u < kPerThread; ++u) {
        const int i = threadIdx.x + u * kMlaConsumerThreads;
        if (i < kChunks)
          *reinterpret_cast<uint4*>(sm.qbuf + (i / (kLatentDim / 8)) * kQPitch + (i % (kLatentDim / 8)) * 16) = qv[u];
      }
    }
    named_bar_sync(3, kMlaConsumerThreads);

    const int lim0 = quad < rows ? min(item.causal_base + quad / G, item.kv_len - 1) : -1;
    const int lim1 = quad + 8 < rows ? min(item.causal_base + (quad + 8) / G, item.kv_len - 1) : -1;
    float o[16][4];
#pragma unroll
    for (int n = 0; n < 16; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    const uint32_t qbase = smem_u32(sm.qbuf) + a_row * kQPitch + a_koff * 2;

    for (int tile = item.tile_begin; tile < item.tile_end; ++tile, ++it) {
      if ((int)(it & 1u) != grp) continue;
      const int s = it % kMlaStages;
      if (gw == 0) MLA_TRACE(0, it);
      mbar_wait_bounded(&sm.full[s], (it / kMlaStages) & 1u, abort_flag, p.status);
      if (gw == 0) MLA_TRACE(1, it);
      const uint32_t sbase = smem_u32(sm.stage[s]);

      // ---- this warp's quarter of S = Q K^T: 16 tokens x sub-tiles [sub0, sub1); four
      // accumulator sets per n-tile keep the dependent mma chain short
      float part[4][2][4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int n = 0; n < 2; ++n) part[u][n][0] = part[u][n][1] = part[u][n][2] = part[u][n][3] = 0.f;
      // sub-tiles [0,5) or [5,9), 4 k-steps each.  The inline-asm loads and MMAs keep
      // program order, so the operand loads are software-pipelined by hand: the fragments
      // of k-step st+2 are requested before the MMAs of k-step st are issued.
      const int sub0 = khalf ? 5 : 0;
      const int nsteps = (khalf ? kMlaSub - 5 : 5) * 4;
      uint32_t qa[3][4], kb[3][4];
      auto load_step = [&](int st, int buf) {
        const int sub = sub0 + (st >> 2), u = st & 3;
        ldmatrix_x4(qa[buf], qbase + (sub * 4 + u) * 32);
        ldmatrix_x4(kb[buf], sbase + sub * kMlaSubBytes + swz128(k_tok, u * 2 + k_chunk_sel));
      };
      load_step(0, 0);
      load_step(1, 1);
#pragma unroll
      for (int st = 0; st < 20; ++st) {
        if (st < nsteps) {
          if (st + 2 < nsteps) load_step(st + 2, (st + 2) % 3);
          mma_bf16_16816(part[st & 3][0], qa[st % 3], kb[st % 3][0], kb[st % 3][1]);
          mma_bf16_16816(part[st & 3][1], qa[st % 3], kb[st % 3][2], kb[st % 3][3]);
        }
      }
      float* my_part = sm.s_part[grp][(it >> 1) & 1][gw] + lane * 8;
#pragma unroll
      for (int n = 0; n < 2; ++n)
        *reinterpret_cast<float4*>(my_part + n * 4) =
            make_float4((part[0][n][0] + part[1][n][0]) + (part[2][n][0] + part[3][n][0]),
                        (part[0][n][1] + part[1][n][1]) + (part[2][n][1] + part[3][n][1]),
                        (part[0][n][2] + part[1][n][2]) + (part[2][n][2] + part[3][n][2]),
                        (part[0][n][3] + part[1][n][3]) + (part[2][n][3] + part[3][n][3]));
      if (gw == 0) MLA_TRACE(2, it);
      named_bar_sync(gbar, 128);
      if (gw == 0) MLA_TRACE(3, it);
      // ---- full scores of the tile in fragment layout: sacc[kt][n] = tokens kt*16 + n*8 ...
      float sacc[2][2][4];
      {
        const float (*pp)[32 * 8] = sm.s_part[grp][(it >> 1) & 1];
#pragma unroll
        for (int kt = 0; kt < 2; ++kt)
#pragma unroll
          for (int n = 0; n < 2; ++n) {
            const float4 a = *reinterpret_cast<const float4*>(pp[kt] + lane * 8 + n * 4);       // dims [0,320)
            const float4 c = *reinterpret_cast<const float4*>(pp[kt + 2] + lane * 8 + n * 4);   // dims [320,576)
            sacc[kt][n][0] = a.x + c.x; sacc[kt][n][1] = a.y + c.y;
            sacc[kt][n][2] = a.z + c.z; sacc[kt][n][3] = a.w + c.w;
          }
      }
      const int tok0 = tile * kMlaTileTokens + qlane * 2;
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int kt = 0; kt < 2; ++kt)
#pragma unroll
        for (int n = 0; n < 2; ++n)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int j = tok0 + kt * 16 + n * 8 + e;
            if (j > lim0) sacc[kt][n][e] = -INFINITY;
            if (j > lim1) sacc[kt][n][2 + e] = -INFINITY;
            mx0 = fmaxf(mx0, sacc[kt][n][e]);
            mx1 = fmaxf(mx1, sacc[kt][n][2 + e]);
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
      for (int kt = 0; kt < 2; ++kt) {
        float pr[2][4];
#pragma unroll
        for (int n = 0; n < 2; ++n) {
          pr[n][0] = fast_exp2(fmaf(sacc[kt][n][0], p.scale_log2, -ms0));
          pr[n][1] = fast_exp2(fmaf(sacc[kt][n][1], p.scale_log2, -ms0));
          pr[n][2] = fast_exp2(fmaf(sacc[kt][n][2], p.scale_log2, -ms1));
          pr[n][3] = fast_exp2(fmaf(sacc[kt][n][3], p.scale_log2, -ms1));
          l0 += pr[n][0] + pr[n][1];
          l1 += pr[n][2] + pr[n][3];
        }
        pf[kt][0] = pack_bf16(pr[0][0], pr[0][1]);
        pf[kt][1] = pack_bf16(pr[0][2], pr[0][3]);
        pf[kt][2] = pack_bf16(pr[1][0], pr[1][1]);
        pf[kt][3] = pack_bf16(pr[1][2], pr[1][3]);
      }
      if (gw == 0) MLA_TRACE(4, it);
      // ---- O[:, 128*gw .. +128) += P V over the tile's 32 tokens
      {
        // 16 V fragments (2 token halves x 8 dim pairs), loads two steps ahead of the MMAs
        uint32_t vb[3][4];
        auto load_v = [&](int st, int buf) {
          const int kt = st >> 3, j = st & 7;
          const int tok = kt * 16 + v_tok_l;
          const int chunk = (j & 3) * 2 + v_chunk_sel;
          const int sub = gw * 2 + (j >> 2);
          ldmatrix_x4_trans(vb[buf], sbase + sub * kMlaSubBytes + swz128(tok, chunk));
        };
        load_v(0, 0);
        load_v(1, 1);
#pragma unroll
        for (int st = 0; st < 16; ++st) {
          if (st + 2 < 16) load_v(st + 2, (st + 2) % 3);
          const int kt = st >> 3, j = st & 7;
          mma_bf16_16816(o[2 * j], pf[kt], vb[st % 3][0], vb[st % 3][1]);
          mma_bf16_16816(o[2 * j + 1], pf[kt], vb[st % 3][2], vb[st % 3][3]);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&sm.empty[s]);
      if (gw == 0) MLA_TRACE(5, it);
#ifdef B200_TRACE
      if (it == 0) MLA_CTA_TRACE(2, global_timer_ns());
      if (grp == 0) MLA_CTA_TRACE(3, global_timer_ns());
      if (grp == 0) MLA_CTA_TRACE(5, it + 1);
#endif
    }

    // ---- merge the two groups in a fixed order, write the item's result
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    if (qlane == 0) {
      if (gw == 0) {
        sm.red_m[grp][quad] = m0;
        sm.red_m[grp][quad + 8] = m1;
      }
      sm.red_l[warp][quad] = (gw == 0) ? l0 : 0.f;   // all four warps of a group hold the same row sums
      sm.red_l[warp][quad + 8] = (gw == 0) ? l1 : 0.f;
    }
    named_bar_sync(3, kMlaConsumerThreads);
    const float ga0 = fmaxf(sm.red_m[0][quad], sm.red_m[1][quad]);
    const float ga1 = fmaxf(sm.red_m[0][quad + 8], sm.red_m[1][quad + 8]);
    {
      const float f0 = (m0 == -INFINITY) ? 0.f : fast_exp2((m0 - ga0) * p.scale_log2);
      const float f1 = (m1 == -INFINITY) ? 0.f : fast_exp2((m1 - ga1) * p.scale_log2);
#pragma unroll
      for (int n = 0; n < 16; ++n) {
        o[n][0] *= f0; o[n][1] *= f0; o[n][2] *= f1; o[n][3] *= f1;
      }
    }
    if (grp == 1) {
      float* slot = sm.slots[gw];
#pragma unroll
      for (int n = 0; n < 16; ++n) {
        const int col = n * 8 + qlane * 2;
        *reinterpret_cast<float2*>(slot + quad * 128 + col) = make_float2(o[n][0], o[n][1]);
        *reinterpret_cast<float2*>(slot + (quad + 8) * 128 + col) = make_float2(o[n][2], o[n][3]);
      }
    }
    named_bar_sync(3, kMlaConsumerThreads);
    const bool record_fits = item.direct || item.partial_idx < p.max_partials;
    if (!record_fits && threadIdx.x == 0 && p.status)
      atomicOr(p.status, B200_STATUS_BAD_LAUNCH);              // workspace smaller than the plan needs
    if (grp == 0 && record_fits) {
      const float* slot = sm.slots[gw];
      // row sums over both groups
      float ls0 = 0.f, ls1 = 0.f;
#pragma unroll
      for (int g2 = 0; g2 < 2; ++g2) {
        const float mg0 = sm.red_m[g2][quad], mg1 = sm.red_m[g2][quad + 8];
        const float s0 = (mg0 == -INFINITY) ? 0.f : fast_exp2((mg0 - ga0) * p.scale_log2);
        const float s1 = (mg1 == -INFINITY) ? 0.f : fast_exp2((mg1 - ga1) * p.scale_log2);
#pragma unroll
        for (int ww = 0; ww < 4; ++ww) {
          ls0 += sm.red_l[g2 * 4 + ww][quad] * s0;
          ls1 += sm.red_l[g2 * 4 + ww][quad + 8] * s1;
        }
      }
      const float inv0 = ls0 > 0.f ? 1.f / ls0 : 0.f;
      const float inv1 = ls1 > 0.f ? 1.f / ls1 : 0.f;
      const float lse0 = ls0 > 0.f ? ga0 * p.scale + __logf(ls0) : -INFINITY;
      const float lse1 = ls1 > 0.f ? ga1 * p.scale + __logf(ls1) : -INFINITY;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int row = quad + half * 8;
        if (row >= rows) continue;
        const float inv = half ? inv1 : inv0;
        const int64_t tok = item.q_start + row / G;
        const int head = row % G;
#pragma unroll
        for (int n = 0; n < 16; ++n) {
          const int col = n * 8 + qlane * 2;
          const float2 other = *reinterpret_cast<const float2*>(slot + row * 128 + col);
          const float x = (o[n][half * 2] + other.x) * inv;
          const float y = (o[n][half * 2 + 1] + other.y) * inv;
          const int vcol = gw * 128 + col;
          if (item.direct) {
            const int64_t off = (tok * p.num_heads + head) * kValueDim + vcol;
            if (p.out_is_f32)
              *reinterpret_cast<float2*>(reinterpret_cast<float*>(p.out) + off) = make_float2(x, y);
            else
              *reinterpret_cast<uint32_t*>(reinterpret_cast<__nv_bfloat16*>(p.out) + off) = pack_bf16(x, y);
          } else {
            float* dst = p.part_o + ((int64_t)item.partial_idx * kMaxRows + row) * kValueDim + vcol;
            *reinterpret_cast<float2*>(dst) = make_float2(x, y);
          }
        }
        if (gw == 0 && qlane == 0) {
          const float lse = half ? lse1 : lse0;
          if (item.direct) {
            if (p.lse_out) p.lse_out[tok * p.num_heads + head] = lse;
          } else {
            p.part_lse[(int64_t)item.partial_idx * kMaxRows + row] = lse;
          }
        }
      }
    }
    // the Q staging of the next item waits on barrier 3 again; nobody can still be
    // reading qbuf / slots of this item by then (all reads precede a barrier above
    // or belong to warps that must reach the next barrier themselves)
    named_bar_sync(3, kMlaConsumerThreads);
    MLA_CTA_TRACE(4, global_timer_ns());
    MLA_CTA_TRACE(6, w.item - item_begin + 1);
    ++w.item;
    w.load();
  }
}

}  // namespace b200

#ifdef B200_TRACE
static long long* g_mla_trace = nullptr;
extern "C" void b200_debug_set_mla_trace(void* dev_ptr) { g_mla_trace = static_cast<long long*>(dev_ptr); }
#endif

namespace b200 {

// `info` given: the launch is sized by the plan (its CTAs, its partial records, its cut pairs).
// `info` null: the replayable form - grid num_ctas, the workspace cut for as many records as it
// holds, the merge launched for the most cut pairs a plan of num_ctas CTAs can have; counts and
// offsets are read from the plan on the device.
static int launch_mla(const char* who, const void* q_latent, int64_t q_stride, const void* latent_cache,
                      int num_blocks, int block_size, const int32_t* block_table, int64_t bt_stride,
                      const int32_t* plan_dev, const b200_decode_plan_info* info, int num_ctas, int num_heads,
                      int kv_lora_rank, int rope_dim, float scale, void* workspace, size_t workspace_bytes,
                      void* out, int out_is_f32, float* lse_out, int32_t* status, void* stream) {
  if (!q_latent || !latent_cache || !block_table || !plan_dev || !out || !workspace ||
      num_blocks <= 0 || num_heads <= 0 || num_ctas <= 0) {
    set_last_error("%s: null pointer or non-positive size", who);
    return B200_EINVAL;
  }
  if (kv_lora_rank != kValueDim || rope_dim != kLatentDim - kValueDim) {
    set_last_error("%s: latent %d+%d unsupported (kernel is built for 512+64)", who, kv_lora_rank, rope_dim);
    return B200_EUNSUPPORTED;
  }
  if (num_heads > kMaxRows) {
    set_last_error("%s: %d heads exceed the 16 query rows of one MMA tile", who, num_heads);
    return B200_EUNSUPPORTED;
  }
  if (block_size < 8 || (block_size & (block_size - 1))) {
    set_last_error("%s: block_size %d must be a power of two >= 8", who, block_size);
    return B200_EUNSUPPORTED;
  }
  if (reinterpret_cast<uintptr_t>(q_latent) % 16 || (q_stride % 8) ||
      q_stride < (int64_t)num_heads * kLatentDim || reinterpret_cast<uintptr_t>(out) % 16 ||
      reinterpret_cast<uintptr_t>(workspace) % 16) {
    set_last_error("%s: q, out and workspace must be 16-byte aligned, q stride a multiple of 8", who);
    return B200_EALIGN;
  }
  const size_t record_bytes = (kMaxRows * (size_t)kValueDim + kMaxRows) * sizeof(float);
  int max_partials;
  if (info) {
    max_partials = info->num_partials;
    if (workspace_bytes < (size_t)max_partials * record_bytes) {
      set_last_error("%s: workspace %zu bytes < %zu needed", who, workspace_bytes, (size_t)max_partials * record_bytes);
      return B200_EPLAN;
    }
  } else {
    max_partials = (int)std::min<size_t>(workspace_bytes / record_bytes, (size_t)1 << 24);
    if (max_partials < num_ctas) {
      set_last_error("%s: workspace %zu bytes holds fewer than num_ctas = %d records; size it with "
                     "b200_mla_decode_workspace_bytes", who, workspace_bytes, num_ctas);
      return B200_EPLAN;
    }
  }
  const int box_tokens = block_size < kMlaTileTokens ? block_size : kMlaTileTokens;
  CUtensorMap lat_map;
  int rc = get_cache_tensor_map(latent_cache, num_blocks, block_size, 1, kLatentDim, box_tokens, &lat_map);
  if (rc) return rc;

  MlaParams p;
  p.q = static_cast<const __nv_bfloat16*>(q_latent);
  p.q_stride = q_stride;
  p.block_table = block_table;
  p.bt_stride = bt_stride;
  p.plan = plan_dev;
  p.part_o = static_cast<float*>(workspace);
  p.part_lse = p.part_o + (size_t)max_partials * kMaxRows * kValueDim;
  p.out = out;
  p.lse_out = lse_out;
  p.status = status;
  p.num_heads = num_heads;
  p.max_partials = max_partials;
  p.block_size = block_size;
  p.block_shift = __builtin_ctz(block_size);
  p.num_blocks = num_blocks;
  p.box_tokens = box_tokens;
  p.boxes_per_tile = kMlaTileTokens / box_tokens;
  p.out_is_f32 = out_is_f32;
  p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;
#ifdef B200_TRACE
  p.trace = g_mla_trace;
#endif

  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const size_t smem = sizeof(MlaSmem) + 1024;
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 64 || !attr_set[dev]) {
    rc = check_cuda(cudaFuncSetAttribute(mla_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem),
                    "mla_decode smem attribute");
    if (rc) return rc;
    if (dev < 64) attr_set[dev] = true;
  }
  rc = check_cuda(launch_pdl(mla_decode_kernel, dim3(num_ctas), dim3(kMlaThreads), smem, s, lat_map, p),
                  "mla_decode launch");
  if (rc) return rc;
  const int merge_pairs = info ? info->num_multi : num_ctas;     // a plan of n CTAs cuts at most n pairs
  if (merge_pairs > 0) {
    rc = check_cuda(launch_pdl(split_merge_kernel<kValueDim>, dim3(split_merge_grid<kValueDim>(merge_pairs)),
                               dim3(128), 0, s, plan_dev, (const float*)p.part_o, (const float*)p.part_lse,
                               out, lse_out, num_heads, num_heads, out_is_f32),
                    "mla_merge launch");
  }
  return rc;
}

}  // namespace b200

extern "C" int b200_mla_decode_absorbed(const void* q_latent, int64_t q_stride,
                                        const void* latent_cache, int num_blocks, int block_size,
                                        const int32_t* block_table, int64_t bt_stride,
                                        const int32_t* plan_dev, const b200_decode_plan_info* info,
                                        int num_heads, int kv_lora_rank, int rope_dim, float scale,
                                        void* workspace, size_t workspace_bytes, void* out,
                                        int out_is_f32, float* lse_out, int32_t* status,
                                        void* stream) {
  using namespace b200;
  if (!info) {
    set_last_error("mla_decode_absorbed: plan info is null");
    return B200_EINVAL;
  }
  if (info->num_items == 0) return B200_OK;
  return launch_mla("mla_decode_absorbed", q_latent, q_stride, latent_cache, num_blocks, block_size, block_table,
                    bt_stride, plan_dev, info, info->num_ctas, num_heads, kv_lora_rank, rope_dim, scale, workspace,
                    workspace_bytes, out, out_is_f32, lse_out, status, stream);
}

extern "C" int b200_mla_decode_absorbed_replayable(const void* q_latent, int64_t q_stride,
                                                   const void* latent_cache, int num_blocks, int block_size,
                                                   const int32_t* block_table, int64_t bt_stride,
                                                   const int32_t* plan_dev, int num_ctas, int num_heads,
                                                   int kv_lora_rank, int rope_dim, float scale,
                                                   void* workspace, size_t workspace_bytes, void* out,
                                                   int out_is_f32, float* lse_out, int32_t* status,
                                                   void* stream) {
  using namespace b200;
  return launch_mla("mla_decode_absorbed_replayable", q_latent, q_stride, latent_cache, num_blocks, block_size,
                    block_table, bt_stride, plan_dev, nullptr, num_ctas, num_heads, kv_lora_rank, rope_dim, scale,
                    workspace, workspace_bytes, out, out_is_f32, lse_out, status, stream);
}
