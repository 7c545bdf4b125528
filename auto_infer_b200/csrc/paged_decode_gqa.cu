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
// The partial records of a pair that was cut are merged by the CTA whose record
// arrives last (one arrival counter per cut pair in the plan).  That CTA only notes
// the pair and carries on with its own items; the merges it owes run once, after its
// last item, so the dependent L2 loads of a merge never sit between two items and a
// layer-step needs no second kernel.
//
// Algorithmic bytes per launch: sum_b kv_len_b * 2 * Hkv * 128 * 2 B (+ q, o).
#include "common.cuh"
#include "decode_plan.h"

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
constexpr int kRecFloats = kMaxRows * kHeadDim + kMaxRows;   // partial record: o (16 x 128), then lse (16)

struct __align__(1024) DecodeSmem {
  uint8_t stage[kStages][kStageBytes];                       // [K lo | K hi | V lo | V hi]
  float slots[4][kSlotFloats];                               // merge buffer, 4 warps at a time
  float red_m[kConsumerWarps][kMaxRows];
  float red_l[kConsumerWarps][kMaxRows];
  uint64_t full[kStages];
  uint64_t empty[kStages];
  int abort_flag;
  int merge_count;                                           // cut pairs whose last record this CTA wrote
  int merge_list[kMaxDeferred];
};

static_assert(sizeof(DecodeSmem) + 1024 <= 227 * 1024, "shared memory budget of one CTA");

struct DecodeParams {
  const __nv_bfloat16* q;
  int64_t q_stride;                 // elements between query tokens
  const int32_t* block_table;
  int64_t bt_stride;
  int32_t* plan;                    // the arrival counters of its cut pairs are counted up and put back to zero
  float* part;                      // partial records, kRecFloats each
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
  int max_partials;                 // records the workspace holds
  float scale, scale_log2;
};

// Fused slot write (the kWrite instantiation): the step's new K/V rows and where they go
struct WriteParams {
  const __nv_bfloat16* k_new;
  const __nv_bfloat16* v_new;
  int64_t k_new_stride, v_new_stride;   // elements between tokens
  const int32_t* slot_mapping;
  __nv_bfloat16* key_cache;
  __nv_bfloat16* value_cache;
  int64_t total_slots;
};

// Walks the CTA's (item, tile) sequence; identical in producer and consumers.
struct TileWalker {
  const DecodeItem* items;
  int item, item_end, tile, tile_end;
  DecodeItem cur;
  __device__ __forceinline__ void set(const int4& a, const int4& b, const int4& c) {
    cur.seq = a.x; cur.kv_head = a.y; cur.tile_begin = a.z; cur.tile_end = a.w;
    cur.kv_len = b.x; cur.q_start = b.y; cur.q_len = b.z; cur.causal_base = b.w;
    cur.partial_idx = c.x; cur.direct = c.y; cur.multi_idx = c.z;
    tile = cur.tile_begin;
    tile_end = cur.tile_end;
  }
  __device__ __forceinline__ void load() {
    if (item < item_end) {
      const int4* p = reinterpret_cast<const int4*>(items + item);
      set(__ldg(p), __ldg(p + 1), __ldg(p + 2));
    }
  }
};

// Merge of the partial records of the cut pairs a CTA has noted, by its 256 consumer
// threads: thread -> (row, 8 columns) of the pair's 16 x 128 result.  Records are read
// with L2 loads (other CTAs wrote them) in record order, so the sum does not depend on
// which CTA happens to run the merge.
__device__ __forceinline__ void merge_noted_pairs(const DecodeParams& p, const int* list, int count,
                                               int off_multi) {
  const int t = threadIdx.x;
  const int row = t >> 4;
  const int col = (t & 15) * 8;
  const int G = p.group;
  for (int e = 0; e < count; ++e) {
    const MultiGroup* mg = reinterpret_cast<const MultiGroup*>(p.plan + off_multi) + list[e];
    const int pb = __ldcg(&mg->part_begin), pe = __ldcg(&mg->part_end);
    const int q_start = __ldcg(&mg->q_start), q_len = __ldcg(&mg->q_len), kv_head = __ldcg(&mg->kv_head);
    if (row >= q_len * G) continue;
    const float* rec = p.part + (int64_t)pb * kRecFloats;
    const int n = pe - pb;
    float mx = -INFINITY;
#pragma unroll 4
    for (int i = 0; i < n; ++i) mx = fmaxf(mx, __ldcg(rec + (int64_t)i * kRecFloats + kMaxRows * kHeadDim + row));
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    float wsum = 0.f;
#pragma unroll 4
    for (int i = 0; i < n; ++i) {
      const float* r = rec + (int64_t)i * kRecFloats;
      const float l = __ldcg(r + kMaxRows * kHeadDim + row);
      const float wgt = (l == -INFINITY) ? 0.f : __expf(l - mx);
      const float4* src = reinterpret_cast<const float4*>(r + row * kHeadDim + col);
      const float4 a = __ldcg(src), b = __ldcg(src + 1);
      wsum += wgt;
      acc[0] += wgt * a.x; acc[1] += wgt * a.y; acc[2] += wgt * a.z; acc[3] += wgt * a.w;
      acc[4] += wgt * b.x; acc[5] += wgt * b.y; acc[6] += wgt * b.z; acc[7] += wgt * b.w;
    }
    const float inv = wsum > 0.f ? 1.f / wsum : 0.f;
    const int64_t tok = q_start + row / G;
    const int head = kv_head * G + row % G;
    const int64_t off = (tok * p.num_q_heads + head) * kHeadDim + col;
    if (p.out_is_f32) {
      float* dst = reinterpret_cast<float*>(p.out) + off;
      *reinterpret_cast<float4*>(dst) = make_float4(acc[0] * inv, acc[1] * inv, acc[2] * inv, acc[3] * inv);
      *reinterpret_cast<float4*>(dst + 4) = make_float4(acc[4] * inv, acc[5] * inv, acc[6] * inv, acc[7] * inv);
    } else {
      uint4 pk;
      pk.x = pack_bf16(acc[0] * inv, acc[1] * inv); pk.y = pack_bf16(acc[2] * inv, acc[3] * inv);
      pk.z = pack_bf16(acc[4] * inv, acc[5] * inv); pk.w = pack_bf16(acc[6] * inv, acc[7] * inv);
      *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.out) + off) = pk;
    }
    if (p.lse_out && (t & 15) == 0)
      p.lse_out[tok * p.num_q_heads + head] = wsum > 0.f ? mx + __logf(wsum) : -INFINITY;
  }
}

// kWrite: the form that also performs the step's KV slot write.  The new rows of a sequence
// (local positions j >= causal_base, row j - causal_base of k_new / v_new) belong to exactly one
// CTA per kv head - the one that streams the tile they fall in.  Their cache slots have not been
// written when the tile is loaded, so the warp that owns them puts the rows into the shared-memory
// tile itself and stores them to their slots in the cache: no write kernel in front of this one.
// It is an instantiation of its own so that the plain form carries none of its code or registers.
template <bool kWrite>
__global__ void __launch_bounds__(kDecodeThreads, 1)
paged_decode_gqa_kernel(const __grid_constant__ CUtensorMap k_map,
                        const __grid_constant__ CUtensorMap v_map, const DecodeParams p,
                        const WriteParams wp) {
  extern __shared__ uint8_t smem_raw[];
  DecodeSmem& sm = *reinterpret_cast<DecodeSmem*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // The plan is host-built and reaches the device by a copy, never by the kernel in
  // front of this one: its words may be read before the grid dependency is resolved.
  const int32_t* plan = p.plan;
  const int4* rec = reinterpret_cast<const int4*>(plan + kPlanHeaderInts + kCtaInts * blockIdx.x);
  const int4 r0 = __ldg(rec), r1 = __ldg(rec + 1), r2 = __ldg(rec + 2), r3 = __ldg(rec + 3);
  const int4 hdr0 = __ldg(reinterpret_cast<const int4*>(plan));
  const int4 hdr1 = __ldg(reinterpret_cast<const int4*>(plan) + 1);
  const int item_begin = r0.x;
  const int item_end = r0.y;
  const DecodeItem* items = reinterpret_cast<const DecodeItem*>(plan + hdr1.z);   // kHdrOffItems

  if (threadIdx.x == 0) {
    sm.abort_flag = 0;
    sm.merge_count = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&sm.full[s], 1);
      mbar_init(&sm.empty[s], 4);     // one arrival per warp of the consuming group
    }
    mbar_fence_init();
  }
  __syncthreads();
#ifdef B200_TRACE
  if (p.trace && threadIdx.x == 0) {
    p.trace[blockIdx.x * 16 + 0] = (long long)global_timer_ns();
    p.trace[blockIdx.x * 16 + 15] = clock64();
  }
#endif
  // While the kernel in front drains: the first tiles of this CTA's first item are asked into
  // L2.  Hints only - the block ids are read past the L1 (nothing stale can stick there) and used
  // for nothing but the prefetch addresses; the loads proper follow the dependency wait and then
  // find a warm L2 instead of paying the cold trip to HBM (the table and the cache rows are
  // normally written long before; if the kernel in front does write them, the hint is merely
  // wasted).
  if (warp == kConsumerWarps && item_begin < item_end) {
    constexpr int kHintTiles = 4;
    const int nbox = p.boxes_per_tile;
    const int n_hint = min(r1.w - r1.z, kHintTiles) * nbox;          // tile_end - tile_begin of the first item
    if (lane < n_hint && r2.x > 0) {
      const int tile = r1.z + lane / nbox, box = lane % nbox;
      int lb = ((tile * kTileTokens) >> p.block_shift) + box;
      const int last_block = (r2.x - 1) >> p.block_shift;
      lb = lb > last_block ? last_block : lb;
      const int bid = __ldcg(p.block_table + (int64_t)r1.x * p.bt_stride + lb);
      if (bid >= 0 && bid < p.num_blocks) {
        const int tok = (tile * kTileTokens + box * p.box_tokens) & (p.block_size - 1);
        tma_prefetch_4d(&k_map, 0, r1.y, tok, bid);
        tma_prefetch_4d(&k_map, 64, r1.y, tok, bid);
        tma_prefetch_4d(&v_map, 0, r1.y, tok, bid);
        tma_prefetch_4d(&v_map, 64, r1.y, tok, bid);
      }
    }
  }
  grid_dep_launch();              // the next kernel may be scheduled; it waits for this grid itself
  grid_dep_wait();                // q, the block table and the step's new cache rows come from earlier kernels
#ifdef B200_TRACE
  if (p.trace && threadIdx.x == 0) p.trace[blockIdx.x * 16 + 1] = (long long)global_timer_ns();
#endif
  if (hdr0.x != kPlanMagic || hdr0.y != (int)gridDim.x) {      // not a plan for this launch
    if (threadIdx.x == 0 && p.status) atomicOr(p.status, B200_STATUS_BAD_LAUNCH);
    return;
  }
  if (item_begin >= item_end) return;
  volatile int* abort_flag = &sm.abort_flag;

  if (warp == kConsumerWarps) {
    // ------------------------------ producer ------------------------------
    if (lane == 0) {
      tma_prefetch_desc(&k_map);
      tma_prefetch_desc(&v_map);
    }
    TileWalker w{items, item_begin, item_end, 0, 0, {}};
    w.set(r1, r2, r3);
    uint32_t it = 0;
    const int nbox = p.boxes_per_tile;
    // Block ids come out of a register window: lane l holds the id of logical block
    // win_base + l of the current sequence (32 blocks = 64 tiles at block_size 128), and the
    // window after it is already on its way.  A tile's boxes never straddle a window (the box
    // count divides 32), so one shuffle per tile replaces a dependent trip to L2 per tile,
    // which would hold a CTA that streams alone to one tile per round trip.
    int win_seq = -1, win_base = 0, win_ids = 0, nxt_ids = 0;
    // the item after the current one is fetched when the current one starts
    int4 na = r1, nb = r2, nc = r3;
    auto prefetch_item = [&](int idx) {
      if (idx < item_end) {
        const int4* ip = reinterpret_cast<const int4*>(items + idx);
        na = __ldg(ip); nb = __ldg(ip + 1); nc = __ldg(ip + 2);
      }
    };
    prefetch_item(item_begin + 1);
    auto load_window = [&](int seq, int base, int kv_len) -> int {
      const int last_block = (kv_len - 1) >> p.block_shift;
      int lb = base + lane;
      lb = lb > last_block ? last_block : lb;         // past the end: any valid entry of the row
      return __ldg(p.block_table + (int64_t)seq * p.bt_stride + lb);
    };
    while (w.item < w.item_end) {
      if (w.tile >= w.tile_end) {                    // item done (or without any tile: an empty key range)
        ++w.item;
        if (w.item < w.item_end) {
          w.set(na, nb, nc);
          prefetch_item(w.item + 1);
        }
        continue;
      }
      const int first_lb = (w.tile * kTileTokens) >> p.block_shift;
      const int base = first_lb & ~31;
      if (w.cur.seq != win_seq || base != win_base) {
        if (w.cur.seq == win_seq && base == win_base + 32) {
          win_ids = nxt_ids;                          // the prefetched window
        } else {
          win_ids = load_window(w.cur.seq, base, w.cur.kv_len);
        }
        win_seq = w.cur.seq;
        win_base = base;
        nxt_ids = load_window(w.cur.seq, base + 32, w.cur.kv_len);   // used 32 blocks from now, if at all
      }
      // this lane's box of the tile (lanes >= nbox idle); tail boxes re-read the last valid page
      const int last_block = (w.cur.kv_len - 1) >> p.block_shift;
      int lb = first_lb + (lane < nbox ? lane : 0);
      lb = lb > last_block ? last_block : lb;
      const int bid = __shfl_sync(0xffffffffu, win_ids, lb - win_base);

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
      ++w.tile;
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
  w.set(r1, r2, r3);
  uint32_t it = 0;

  // Q fragments of an item: 8 k-steps x 4 registers, rows beyond q_len*group are zero.
  // They are fetched for the NEXT item right after the tile loop, so the global
  // loads fly while the warps merge and write the current item.
  uint32_t qf[8][4];
  auto load_q = [&](const DecodeItem& qi) {
    if constexpr (kWrite) {
      // the item's new K / V rows (if its tiles hold them) are asked into L1 now, so that the
      // patch of the tile they fall in does not wait for a trip to L2
      if (qi.tile_end * kTileTokens >= qi.kv_len && warp < 4) {
        const int row = warp;                                  // one row per warp, the first four
        if (row < qi.q_len) {
          const int64_t tok = qi.q_start + row;
          const __nv_bfloat16* src = (lane >= 16 ? wp.v_new + tok * wp.v_new_stride : wp.k_new + tok * wp.k_new_stride) +
                                     qi.kv_head * kHeadDim + (lane & 15) * 8;
          asm volatile("prefetch.global.L1 [%0];" ::"l"(src));
        }
      }
    }
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

  // A partial record is announced (arrival counter of its pair) one item late, or at the end
  // of the CTA's work: by then its stores have long left the SM and the fence that must
  // precede the announcement costs nothing, where a fence right behind the stores would
  // hold all eight warps for a round trip through a loaded memory system.
  int pending_multi = -1;
  const int off_multi = hdr1.w;
  auto announce = [&](int multi_idx) {            // thread 0, after a fence by all and a barrier
    MultiGroup* mg = reinterpret_cast<MultiGroup*>(p.plan + off_multi) + multi_idx;
    const int n_parts = mg->part_end - mg->part_begin;
    if (atomicAdd(&mg->arrivals, 1) == n_parts - 1) {
      mg->arrivals = 0;                           // ready for the next launch on this plan
      __threadfence();                            // the other CTAs' records are visible from here on
      if (sm.merge_count < kMaxDeferred) {
        sm.merge_list[sm.merge_count] = multi_idx;
        sm.merge_count = sm.merge_count + 1;
      } else if (p.status) {                      // the planner never gives a CTA this many cut pieces
        atomicOr(p.status, B200_STATUS_BAD_LAUNCH);
      }
    }
  };
  // the record of the item after the current one, fetched while the current one streams
  // (its first two quarters: what the Q fetch needs; the rest is read at the hand-over and
  // not used before the item ends)
  int4 na = r1, nb = r2;
  auto prefetch_item = [&](int idx) {
    if (idx < item_end) {
      const int4* ip = reinterpret_cast<const int4*>(items + idx);
      na = __ldg(ip); nb = __ldg(ip + 1);
    }
  };
  prefetch_item(item_begin + 1);

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
      if constexpr (kWrite) {
        const int row_lo = tile * kTileTokens + wslice * 16;
        const int j_lo = max(max(item.causal_base, 0), row_lo);
        const int j_hi = min(min(item.kv_len, item.causal_base + item.q_len), row_lo + 16);
        if (j_lo < j_hi) {
          const int chunk = lane & 15;                    // 16-byte chunk of the 256-byte row
          const bool is_v = lane >= 16;                   // lanes 0-15 carry K, lanes 16-31 V
          for (int j = j_lo; j < j_hi; ++j) {
            const int64_t tok = item.q_start + (j - item.causal_base);
            const __nv_bfloat16* src = (is_v ? wp.v_new + tok * wp.v_new_stride : wp.k_new + tok * wp.k_new_stride) +
                                       item.kv_head * kHeadDim + chunk * 8;
            const uint4 val = *reinterpret_cast<const uint4*>(src);
            *reinterpret_cast<uint4*>(sm.stage[s] + (is_v ? kTileBytes : 0) + (chunk >> 3) * kHalfTileBytes +
                                      swz128(j - tile * kTileTokens, chunk & 7)) = val;
            const int64_t slot = wp.slot_mapping[tok];
            if (slot >= 0 && slot < wp.total_slots) {
              __nv_bfloat16* cache = is_v ? wp.value_cache : wp.key_cache;
              *reinterpret_cast<uint4*>(cache + (slot * p.num_kv_heads + item.kv_head) * kHeadDim + chunk * 8) = val;
            } else if (slot >= wp.total_slots && lane == 0 && p.status) {
              atomicOr(p.status, B200_STATUS_BAD_SLOT);
            }
          }
          __syncwarp();
        }
      }

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
      // ---- rows past the sequence's end carry weight 0, but 0 x NaN is NaN: whatever bytes
      // an unwritten cache slot holds must not reach the MMA.  Only a pair's last tile has
      // such rows; the warp clears its own 16 of them in shared memory.
      const bool ragged = (tile + 1) * kTileTokens > item.kv_len;
      if (ragged) {
        const int first_bad = item.kv_len - tile * kTileTokens;          // first row of the tile past the end
        for (int idx = lane; idx < 16 * 16; idx += 32) {
          const int row = wslice * 16 + (idx >> 4), chunk = idx & 15;
          if (row >= first_bad)
            *reinterpret_cast<uint4*>(sm.stage[s] + kTileBytes + (chunk >> 3) * kHalfTileBytes +
                                      swz128(row, chunk & 7)) = make_uint4(0u, 0u, 0u, 0u);
        }
        __syncwarp();
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
      // the stage goes back to TMA: order this warp's stores into it before TMA's writes
      if constexpr (kWrite) {
        if (ragged || (tile + 1) * kTileTokens > max(item.causal_base, 0)) fence_proxy_async();
      } else {
        if (ragged) fence_proxy_async();
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

#ifdef B200_TRACE_PHASES
    if (p.trace && threadIdx.x == 0) p.trace[blockIdx.x * 16 + 14] = (long long)global_timer_ns();
#endif
    // ---- next item's Q on its way, then merge the eight warps (fixed order) and write the result
    ++w.item;
    if (w.item < w.item_end) {
      w.set(na, nb, __ldg(reinterpret_cast<const int4*>(items + w.item) + 2));
      prefetch_item(w.item + 1);
      load_q(w.cur);
    }
    if (pending_multi >= 0) __threadfence();      // stores of the PREVIOUS partial record (long done)
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    if (qlane == 0) {
      sm.red_m[warp][quad] = m0;
      sm.red_m[warp][quad + 8] = m1;
    }
    named_bar_sync(1, kConsumerThreads);                       // (1) every warp's row maxima are in place
#ifdef B200_TRACE_PHASES
    if (p.trace && threadIdx.x == 0) p.trace[blockIdx.x * 16 + 10] = (long long)global_timer_ns();
#endif
    if (pending_multi >= 0) {
      if (threadIdx.x == 0) announce(pending_multi);
      pending_multi = -1;
    }
    {
      // bring this warp's sums and accumulators to the rows' common maximum; the scaled
      // sums go to red_l, so that the row total later is eight loads and adds
      float g0 = -INFINITY, g1 = -INFINITY;
#pragma unroll
      for (int ww = 0; ww < kConsumerWarps; ++ww) {
        g0 = fmaxf(g0, sm.red_m[ww][quad]);
        g1 = fmaxf(g1, sm.red_m[ww][quad + 8]);
      }
      const float f0 = (m0 == -INFINITY) ? 0.f : fast_exp2((m0 - g0) * p.scale_log2);
      const float f1 = (m1 == -INFINITY) ? 0.f : fast_exp2((m1 - g1) * p.scale_log2);
      if (qlane == 0) {
        sm.red_l[warp][quad] = l0 * f0;
        sm.red_l[warp][quad + 8] = l1 * f1;
      }
#pragma unroll
      for (int n = 0; n < 16; ++n) {
        o[n][0] *= f0; o[n][1] *= f0; o[n][2] *= f1; o[n][3] *= f1;
      }
    }
    // Merge-buffer rows are 128 floats, a multiple of the 32 banks: the eight fragment rows a
    // warp stores at once would all land in the same banks.  Column groups of 8 floats are
    // XOR-ed with the row number (mod 4), which spreads them over all banks.
    const int swz = (quad & 3) << 3;              // same for row quad and row quad + 8
    if (warp >= 4) {
      float* slot = sm.slots[warp - 4];
#pragma unroll
      for (int n = 0; n < 16; ++n) {
        const int col = (n * 8 + qlane * 2) ^ swz;
        *reinterpret_cast<float2*>(slot + quad * kHeadDim + col) = make_float2(o[n][0], o[n][1]);
        *reinterpret_cast<float2*>(slot + (quad + 8) * kHeadDim + col) = make_float2(o[n][2], o[n][3]);
      }
    }
    named_bar_sync(1, kConsumerThreads);                       // (2) warps 4-7 have parked their sums
#ifdef B200_TRACE_PHASES
    if (p.trace && threadIdx.x == 0) p.trace[blockIdx.x * 16 + 11] = (long long)global_timer_ns();
#endif
    if (warp < 4) {
      // Add the partner warp's sums in place: a thread rewrites exactly the words it read.  The
      // loads of four column groups are issued together before any of their stores: written as
      // load-add-store per word, every load would wait behind the store before it (the compiler
      // must assume they alias) and the warp would pay one shared-memory latency per word.
      float* slot = sm.slots[warp];
#pragma unroll
      for (int n0 = 0; n0 < 16; n0 += 4) {
        float2 a[4], b[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int col = ((n0 + u) * 8 + qlane * 2) ^ swz;
          a[u] = *reinterpret_cast<const float2*>(slot + quad * kHeadDim + col);
          b[u] = *reinterpret_cast<const float2*>(slot + (quad + 8) * kHeadDim + col);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int col = ((n0 + u) * 8 + qlane * 2) ^ swz;
          *reinterpret_cast<float2*>(slot + quad * kHeadDim + col) =
              make_float2(a[u].x + o[n0 + u][0], a[u].y + o[n0 + u][1]);
          *reinterpret_cast<float2*>(slot + (quad + 8) * kHeadDim + col) =
              make_float2(b[u].x + o[n0 + u][2], b[u].y + o[n0 + u][3]);
        }
      }
    }
    // 256 threads: thread -> rows (t / 32) and (t / 32 + 8), 4 columns each, so a warp reads and
    // writes whole rows.  The rows' maxima and scaled sums are taken from red_m / red_l
    // BEFORE barrier (3): no warp writes those arrays again (next item) until every thread
    // has passed (3), i.e. has finished reading them.
    const int t = threadIdx.x;
    const int col = (t & 31) * 4;
    float inv_r[2], lse_r[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int row = (t >> 5) + h * 8;
      float g = -INFINITY, lsum = 0.f;
#pragma unroll
      for (int ww = 0; ww < kConsumerWarps; ++ww) {
        g = fmaxf(g, sm.red_m[ww][row]);
        lsum += sm.red_l[ww][row];
      }
      inv_r[h] = lsum > 0.f ? 1.f / lsum : 0.f;
      lse_r[h] = lsum > 0.f ? g * p.scale + __logf(lsum) : -INFINITY;
    }
    named_bar_sync(1, kConsumerThreads);                       // (3) the four slots hold the warp-pair sums
#ifdef B200_TRACE_PHASES
    if (p.trace && threadIdx.x == 0) p.trace[blockIdx.x * 16 + 13] = (long long)global_timer_ns();
#endif
    const bool record_fits = item.direct || item.partial_idx < p.max_partials;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int row = (t >> 5) + h * 8;
      if (row >= rows || !record_fits) continue;
      const int pcol = col ^ ((row & 3) << 3);
      float4 acc = *reinterpret_cast<const float4*>(&sm.slots[0][row * kHeadDim + pcol]);
#pragma unroll
      for (int sl = 1; sl < 4; ++sl) {
        const float4 x = *reinterpret_cast<const float4*>(&sm.slots[sl][row * kHeadDim + pcol]);
        acc.x += x.x; acc.y += x.y; acc.z += x.z; acc.w += x.w;
      }
      const float inv = inv_r[h];
      const float4 v = make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv);
      if (item.direct) {
        const int64_t tok = item.q_start + row / G;
        const int head = item.kv_head * G + row % G;
        const int64_t off = (tok * p.num_q_heads + head) * kHeadDim + col;
        if (p.out_is_f32) {
          *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out) + off) = v;
        } else {
          uint2 pk;
          pk.x = pack_bf16(v.x, v.y);
          pk.y = pack_bf16(v.z, v.w);
          *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p.out) + off) = pk;
        }
        if (p.lse_out && (t & 31) == 0) p.lse_out[tok * p.num_q_heads + head] = lse_r[h];
      } else {
        float* rec = p.part + (int64_t)item.partial_idx * kRecFloats;
        *reinterpret_cast<float4*>(rec + row * kHeadDim + col) = v;
        if ((t & 31) == 0) rec[kMaxRows * kHeadDim + row] = lse_r[h];
      }
    }
    if (!item.direct) {
      if (record_fits) {
        pending_multi = item.multi_idx;
      } else if (t == 0 && p.status) {
        atomicOr(p.status, B200_STATUS_BAD_LAUNCH);            // workspace smaller than the plan needs
      }
    }
#ifdef B200_TRACE
    if (p.trace && threadIdx.x == 0) p.trace[blockIdx.x * 16 + 5] = (long long)global_timer_ns();   // item written
#endif
    // The next item's first write to red_m comes after barrier (3) above, and its first write to
    // red_l and to the slots after its own barrier (1), which no thread passes before it has
    // finished the reads of this item.
  }

  // ---- the last record's announcement, then the merges this CTA owes: the cut pairs
  // whose last record it wrote
  if (pending_multi >= 0) {
    __threadfence();
    named_bar_sync(1, kConsumerThreads);
    if (threadIdx.x == 0) announce(pending_multi);
  }
  named_bar_sync(1, kConsumerThreads);
  if (sm.merge_count > 0) merge_noted_pairs(p, sm.merge_list, sm.merge_count, off_multi);
#ifdef B200_TRACE
  if (p.trace && threadIdx.x == 0) {
    p.trace[blockIdx.x * 16 + 9] = (long long)global_timer_ns();   // merges done
    p.trace[blockIdx.x * 16 + 15] = clock64() - p.trace[blockIdx.x * 16 + 15];
  }
#endif
}

}  // namespace b200

#ifdef B200_TRACE
static long long* g_trace = nullptr;
extern "C" void b200_debug_set_trace(void* dev_ptr) { g_trace = static_cast<long long*>(dev_ptr); }
#endif

namespace b200 {

// Shared launcher.  With `info` the counts of the step are known on the host (nothing
// is launched for an empty plan, the workspace only has to hold the records the plan
// uses).  Without it every count is read from the plan on the device: the launch then
// depends on num_ctas alone and can be recorded once and replayed for other steps.
struct NewKv {
  const void* k;
  int64_t k_stride;
  const void* v;
  int64_t v_stride;
  const int32_t* slot_mapping;
};

static int launch_decode(const char* who, const void* q, int64_t q_stride, const void* key_cache,
                         const void* value_cache, int num_blocks, int block_size,
                         const int32_t* block_table, int64_t bt_stride, int32_t* plan_dev,
                         const b200_decode_plan_info* info, int num_ctas, int num_q_heads,
                         int num_kv_heads, int head_dim, float scale, void* workspace,
                         size_t workspace_bytes, void* out, int out_is_f32, float* lse_out,
                         int32_t* status, void* stream, const NewKv* new_kv = nullptr) {
  if (new_kv) {
    if (!new_kv->k || !new_kv->v || !new_kv->slot_mapping) {
      set_last_error("%s: new K/V rows and the slot mapping must all be given", who);
      return B200_EINVAL;
    }
    if (reinterpret_cast<uintptr_t>(new_kv->k) % 16 || reinterpret_cast<uintptr_t>(new_kv->v) % 16 ||
        new_kv->k_stride % 8 || new_kv->v_stride % 8 || new_kv->k_stride < (int64_t)num_kv_heads * head_dim ||
        new_kv->v_stride < (int64_t)num_kv_heads * head_dim) {
      set_last_error("%s: new K/V rows must be 16-byte aligned with token strides that are multiples of 8 elements", who);
      return B200_EALIGN;
    }
  }
  if (!q || !key_cache || !value_cache || !block_table || !plan_dev || !out || !workspace ||
      num_blocks <= 0 || num_q_heads <= 0 || num_kv_heads <= 0 || num_q_heads % num_kv_heads ||
      num_ctas <= 0) {
    set_last_error("%s: null pointer, bad head counts or no CTAs", who);
    return B200_EINVAL;
  }
  if (head_dim != kHeadDim) {
    set_last_error("%s: head_dim %d unsupported (kernel is built for 128)", who, head_dim);
    return B200_EUNSUPPORTED;
  }
  if (block_size < 8 || (block_size & (block_size - 1))) {
    set_last_error("%s: block_size %d must be a power of two >= 8", who, block_size);
    return B200_EUNSUPPORTED;
  }
  if (reinterpret_cast<uintptr_t>(q) % 4 || (q_stride % 2) || q_stride < (int64_t)num_q_heads * head_dim) {
    set_last_error("%s: q must be 4-byte aligned with an even token stride >= Hq*D", who);
    return B200_EALIGN;
  }
  if (reinterpret_cast<uintptr_t>(out) % 16 || reinterpret_cast<uintptr_t>(workspace) % 16 ||
      reinterpret_cast<uintptr_t>(plan_dev) % 16) {
    set_last_error("%s: out, workspace and plan must be 16-byte aligned", who);
    return B200_EALIGN;
  }
  const size_t max_partials = workspace_bytes / (kRecFloats * sizeof(float));
  if (info && (size_t)info->num_partials > max_partials) {
    set_last_error("%s: workspace %zu bytes < %zu needed", who, workspace_bytes,
                   (size_t)info->num_partials * kRecFloats * sizeof(float));
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
  p.part = static_cast<float*>(workspace);
  p.max_partials = max_partials > (size_t)INT32_MAX ? INT32_MAX : (int)max_partials;
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
  WriteParams wp{};
  if (new_kv) {
    wp.k_new = static_cast<const __nv_bfloat16*>(new_kv->k);
    wp.v_new = static_cast<const __nv_bfloat16*>(new_kv->v);
    wp.k_new_stride = new_kv->k_stride;
    wp.v_new_stride = new_kv->v_stride;
    wp.slot_mapping = new_kv->slot_mapping;
    wp.key_cache = static_cast<__nv_bfloat16*>(const_cast<void*>(key_cache));
    wp.value_cache = static_cast<__nv_bfloat16*>(const_cast<void*>(value_cache));
    wp.total_slots = (int64_t)num_blocks * block_size;
  }

  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const size_t smem = sizeof(DecodeSmem) + 1024;
  static bool attr_set[2][64] = {{false}, {false}};
  auto kernel = new_kv ? paged_decode_gqa_kernel<true> : paged_decode_gqa_kernel<false>;
  const int which = new_kv ? 1 : 0;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 64 || !attr_set[which][dev]) {
    rc = check_cuda(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem),
                    "paged_decode_gqa smem attribute");
    if (rc) return rc;
    if (dev < 64) attr_set[which][dev] = true;
  }
  return check_cuda(launch_pdl(kernel, dim3(num_ctas), dim3(kDecodeThreads), smem, s, k_map, v_map, p, wp),
                    "paged_decode_gqa launch");
}

}  // namespace b200

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
  return launch_decode("paged_decode_gqa", q, q_stride, key_cache, value_cache, num_blocks, block_size,
                       block_table, bt_stride, plan_dev, info, info->num_ctas, num_q_heads, num_kv_heads,
                       head_dim, scale, workspace, workspace_bytes, out, out_is_f32, lse_out, status,
                       stream);
}

extern "C" int b200_paged_decode_gqa_replayable(const void* q, int64_t q_stride, const void* key_cache,
                                                const void* value_cache, int num_blocks, int block_size,
                                                const int32_t* block_table, int64_t bt_stride,
                                                int32_t* plan_dev, int num_ctas, int num_q_heads,
                                                int num_kv_heads, int head_dim, float scale,
                                                void* workspace, size_t workspace_bytes, void* out,
                                                int out_is_f32, float* lse_out, int32_t* status,
                                                void* stream) {
  using namespace b200;
  return launch_decode("paged_decode_gqa_replayable", q, q_stride, key_cache, value_cache, num_blocks,
                       block_size, block_table, bt_stride, plan_dev, nullptr, num_ctas, num_q_heads,
                       num_kv_heads, head_dim, scale, workspace, workspace_bytes, out, out_is_f32,
                       lse_out, status, stream);
}

extern "C" int b200_paged_decode_gqa_write(const void* q, int64_t q_stride, const void* k_new,
                                           int64_t k_new_stride, const void* v_new, int64_t v_new_stride,
                                           const int32_t* slot_mapping, void* key_cache, void* value_cache,
                                           int num_blocks, int block_size, const int32_t* block_table,
                                           int64_t bt_stride, int32_t* plan_dev,
                                           const b200_decode_plan_info* info, int num_ctas,
                                           int num_q_heads, int num_kv_heads, int head_dim, float scale,
                                           void* workspace, size_t workspace_bytes, void* out,
                                           int out_is_f32, float* lse_out, int32_t* status, void* stream) {
  using namespace b200;
  if (info && info->skipped_seqs != 0) {
    set_last_error("paged_decode_gqa_write: the plan leaves %d sequences to the wide-query kernel, whose new "
                   "rows this call would not write; use b200_reshape_and_cache for such a step",
                   info->skipped_seqs);
    return B200_EUNSUPPORTED;
  }
  if (info && info->num_items == 0) return B200_OK;
  NewKv nk{k_new, k_new_stride, v_new, v_new_stride, slot_mapping};
  return launch_decode("paged_decode_gqa_write", q, q_stride, key_cache, value_cache, num_blocks, block_size,
                       block_table, bt_stride, plan_dev, info, info ? info->num_ctas : num_ctas, num_q_heads,
                       num_kv_heads, head_dim, scale, workspace, workspace_bytes, out, out_is_f32, lse_out,
                       status, stream, &nk);
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
constexpr size_t kStaticScratchFloats = (size_t)kStaticMaxPartials * kRecFloats;
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
