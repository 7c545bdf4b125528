// Paged GQA attention for wide query blocks (chunked prefill, multi-token
// verify): any q_len, bottom-right causal over the paged prefix, on the
// Blackwell tensor cores (tcgen05.mma with accumulators in tensor memory).
//
// Work item = 128 packed query rows of one (sequence, kv head) pair, a row being
// (query position, head within the kv group), so the G heads that share a kv
// head also share every K/V tile in shared memory.  Items are sorted by
// decreasing key count on the host and handed out through a work queue to one
// persistent CTA per SM.
// Tensor-bound: flops = 4 * D * sum over rows of visible keys.
#include <algorithm>
#include <vector>

#define B200_INLINE_WAITS
#include "common.cuh"
#include "decode_plan.h"
#include "tc05.cuh"

namespace b200 {

constexpr int kPfHeadDim = 128;
constexpr int kPfRows = 128;                                   // packed query rows per item
constexpr int kPfTile = 128;                                    // KV tokens per tile
constexpr int kPfHalfTileBytes = kPfTile * 128;                 // [128 tokens][64 dims] bf16
constexpr int kPfTileBytes = 2 * kPfHalfTileBytes;              // K or V tile: 32 KB
constexpr int kPfItemInts = 8;
constexpr int kPfMagic = 0x70663030;

struct PrefillItem {
  int32_t seq, kv_head, row0, n_tiles;        // row0: first packed row of the pair this item owns
  int32_t kv_len, q_start, q_len, causal_base;
};
static_assert(sizeof(PrefillItem) == kPfItemInts * 4, "item layout");

// The order in which an item walks its KV tiles is free (online softmax), so every item
// starts at a different tile and wraps around: the row tiles of one (sequence, kv head)
// pair run on different SMs at the same time, and walking in step they would all ask the
// L2 for the same lines at the same moment.
constexpr int kPfTileRotation = 5;
__device__ __forceinline__ int first_tile(const PrefillItem& item) {
  return item.n_tiles > 0 ? ((item.row0 / kPfRows) * kPfTileRotation) % item.n_tiles : 0;
}

struct PrefillParams {
  const __nv_bfloat16* q;
  int64_t q_stride;
  const int32_t* block_table;
  int64_t bt_stride;
  const PrefillItem* items;
  int* work_counter;                // two plan words: next item to hand out, CTAs that have left
                                    // (the word before them is the number of items)
  void* out;
  float* lse_out;
  int32_t* status;
  int num_q_heads, group;
  int block_size, block_shift, num_blocks, box_tokens, boxes_per_tile;
  int out_is_f32;
  int q_by_tma;                     // the Q tile is one TMA box (else copied row by row)
  float scale, scale_log2;
#ifdef B200_TRACE
  long long* trace;                 // clock64 samples of CTA 0 (debug builds)
#endif
};

#ifdef B200_TRACE
#define PF_TRACE(slot, tileno)                                                                \
  do {                                                                                        \
    if (p.trace && blockIdx.x == 0 && (tileno) < 96) p.trace[(tileno) * 16 + (slot)] = clock64(); \
  } while (0)
#else
#define PF_TRACE(slot, tileno) do {} while (0)
#endif


// ============================================================================
// One 128-row query tile per work item, S and O accumulated in tensor memory by
// tcgen05.mma.  Warp roles (512 threads = four warpgroups, one CTA per SM):
//   warps 0-3   softmax group A     thread r owns query row r (TMEM lane r)
//   warps 4-7   softmax group B     same rows, the other half of the KV tiles
//   warp  8     TMA producer: Q tile, 128-token K and V tiles (separate rings), work queue
//   warp  9     tensor-memory owner, issues S = Q K^T
//   warp  10    issues O += P V          (warp 11 only completes the warpgroup)
//   warps 12-15 epilogue: thread e takes row e of O out of tensor memory and stores it
// After set-up the warpgroups trade registers (setmaxnreg): 200 per softmax thread, which
// holds a whole 128-column score row, 40 / 72 for the others.
// The s-th KV tile an item works on (running count over the CTA's items) belongs to group
// s & 1 and uses S buffer s & 1: S = Q K^T (M 128, N 128, 8 x K16, both operands in shared
// memory) lands there, the group's threads read their row with tcgen05.ld (a thread holds a
// whole row: no shuffles), hand the buffer straight back, and write P as packed bf16 into
// the group's own P buffer in tensor memory; the MMA reads it from there as its A operand:
// O (+)= P V (M 128, N 128, 8 x K16, V read MN-major from the TMA tile).  Both groups
// accumulate into ONE O under ONE running maximum per row, handed from the owner of one
// step to the owner of the next through shared memory right after the row maximum is
// known.  Each group keeps its own row sum; the sums are merged by the epilogue warps,
// which work on item k while the softmax groups are already in item k + 1 (the P V issuer
// waits for them before it overwrites O).  O is rescaled in tensor memory only when a row
// maximum grows by more than 2^8 (the stale maximum is kept otherwise).
// Measured on the part: an M 128 x N 128 x K 16 MMA takes 67 cycles with both operands in
// shared memory (8 KB read: all the bandwidth an SM has) and 100 cycles with A in tensor
// memory whatever N <= 128 is, so Q stays in shared memory and only P, which the threads
// produce in registers anyway, goes through tensor memory.
// N = 128 per MMA on purpose: a tcgen05.mma costs ~50 cycles to issue whatever its
// size, so N = 64 instructions (32 cycles of math) would leave the pipe waiting.
// ============================================================================
// Ring depths and the K lead were chosen by A/B timing on the part (2 + 4 and 4 + 2 stages and
// leads of 0 and 1 were each 0.5-2 % slower).
constexpr int kTcKStages = 3;             // 32 KB per stage
constexpr int kTcVStages = 3;
constexpr int kTcKLead = 2;               // K loads run this many tiles ahead of the V loads
constexpr int kTcSoftmaxThreads = 256;
constexpr int kTcEpilogueThreads = 128;
constexpr int kTcThreads = kTcSoftmaxThreads + 128 + kTcEpilogueThreads;   // whole warpgroups: 512 = 4 x 128
// registers per thread after the hand-over below: 256 * 200 + 128 * 40 + 128 * 72 = 512 * 128
constexpr int kTcRegsSoftmax = 200;

__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
constexpr int kTcRegsOther = 40;
constexpr int kTcRegsEpilogue = 72;
constexpr int kTcTmemCols = 512;          // S0 [0,128) S1 [128,256) O [256,384) P_A [384,448) P_B [448,512)
constexpr int kTcOCol = 256;
constexpr int kTcPCol = 384;
constexpr int kTcQBytes = 2 * kPfRows * 128;

struct __align__(1024) TcSmem {
  uint8_t q[kTcQBytes];                    // [dim half][128 rows][128 B], swizzled
  uint8_t k[kTcKStages][kPfTileBytes];     // [dims 0-63 | dims 64-127], 128 tokens x 128 B each
  uint8_t v[kTcVStages][kPfTileBytes];
  float row_l[2][kPfRows];                 // end of item: the groups' row sums, scaled to the final maximum
  float row_mfin[kPfRows];                 // end of item: the final row maximum
  float row_ms[2][kPfRows];                // running row maximum after tile j, slot j & 1
  uint64_t k_full[kTcKStages];
  uint64_t k_empty[kTcKStages];
  uint64_t v_full[kTcVStages];
  uint64_t v_empty[kTcVStages];
  uint64_t s_full[2];
  uint64_t s_empty[2];                     // softmax threads: the tile's scores are in registers
  uint64_t p_full[2];                      // per group
  uint64_t pv_done[2];                     // per tile parity
  uint64_t m_ready[2];                     // per tile parity: row_ms[parity] is written
  uint64_t o_done;                         // P V issuer -> epilogue warps: the item's O is complete
  uint64_t o_free;                         // epilogue warps -> P V issuer: O is in registers
  uint64_t l_full;                         // softmax threads -> epilogue warps: row_l / row_mfin written
  uint64_t l_empty;                        // and read
  uint64_t q_full;                         // producer warp: the item's Q tile is staged
  uint64_t q_empty;                        // all S MMAs of the item have run
  uint64_t item_full[2];                   // work-queue hand-off: producer warp -> the other roles
  uint64_t item_empty[2];
  alignas(16) PrefillItem next_rec[2];     // the mailbox carries the whole item record (read as int4)
  int next_item[2];
  uint32_t tmem_base;
  int abort_flag;
};
static_assert(sizeof(TcSmem) <= 227 * 1024, "shared memory budget of one CTA");

__global__ void __launch_bounds__(kTcThreads, 1)
paged_prefill_tc_kernel(const __grid_constant__ CUtensorMap k_map,
                        const __grid_constant__ CUtensorMap v_map,
                        const __grid_constant__ CUtensorMap q_map, const PrefillParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  TcSmem& sm = *reinterpret_cast<TcSmem*>(smem_raw);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  if (smem_u32(smem_raw) & 1023u) {       // the swizzled tiles need a 1024-byte aligned base
    if (threadIdx.x == 0 && p.status) atomicOr(p.status, B200_STATUS_BAD_LAUNCH);
    return;
  }

  if (threadIdx.x == 0) {
    sm.abort_flag = 0;
    for (int s = 0; s < kTcKStages; ++s) {
      mbar_init(&sm.k_full[s], 1);
      mbar_init(&sm.k_empty[s], 1);
    }
    for (int s = 0; s < kTcVStages; ++s) {
      mbar_init(&sm.v_full[s], 1);
      mbar_init(&sm.v_empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&sm.s_full[b], 1);
      mbar_init(&sm.s_empty[b], 128);
      mbar_init(&sm.p_full[b], 128);
      mbar_init(&sm.pv_done[b], 1);
      mbar_init(&sm.m_ready[b], 128);
      mbar_init(&sm.item_full[b], 1);
      mbar_init(&sm.item_empty[b], kTcSoftmaxThreads + 2 + kTcEpilogueThreads);   // all consumers of the mailbox
    }
    mbar_init(&sm.o_done, 1);
    mbar_init(&sm.o_free, kTcEpilogueThreads);
    mbar_init(&sm.l_full, kTcSoftmaxThreads);
    mbar_init(&sm.l_empty, kTcEpilogueThreads);
    mbar_init(&sm.q_full, 32);
    mbar_init(&sm.q_empty, 1);
    mbar_fence_init();
  }
  if (warp == 9) {
    tmem_alloc(&sm.tmem_base, kTcTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  // The softmax threads keep a whole 128-column score row in registers (reading it from
  // tensor memory twice cost 13 % of the kernel); the warps that only issue TMA loads and
  // MMAs give them the registers for it (setmaxnreg below, executed by whole warpgroups).
  grid_dep_wait();                // q and the step's new cache rows come from earlier kernels
  const uint32_t tmem = sm.tmem_base;
  volatile int* abort_flag = &sm.abort_flag;
  // Items are handed out dynamically, longest first: the producer warp draws the
  // next index from a global counter and passes it to the other roles through a
  // two-slot mailbox.  -1 ends the CTA.
  auto take_item = [&](uint32_t k, PrefillItem& rec) -> int {
    mbar_wait_bounded(&sm.item_full[k & 1u], (k >> 1) & 1u, abort_flag, p.status);
    const int idx = *reinterpret_cast<volatile int*>(&sm.next_item[k & 1u]);
    const int4* src = reinterpret_cast<const int4*>(&sm.next_rec[k & 1u]);
    const int4 lo = src[0], hi = src[1];
    rec = PrefillItem{lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
    mbar_arrive(&sm.item_empty[k & 1u]);
    return (*abort_flag || idx < 0) ? -1 : idx;      // the producer has mapped an index past the list to -1
  };

  if (warp >= 8 && warp < 12) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kTcRegsOther));
  if (warp == 8) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      tma_prefetch_desc(&k_map);
      tma_prefetch_desc(&v_map);
      if (p.q_by_tma) tma_prefetch_desc(&q_map);
    }
    uint32_t it = 0;
    const int nbox = p.boxes_per_tile;
    for (uint32_t k = 0;; ++k) {
      int idx = -1;
      if (lane == 0) {
        // the first item of a CTA is its own index (no round trip to the counter before
        // the first load); the rest of the list is handed out dynamically
        idx = (k == 0) ? (int)blockIdx.x : (int)gridDim.x + atomicAdd(p.work_counter, 1);
        // the item count lives in the plan, not in the launch: a recorded launch serves other steps
        if (idx >= __ldg(p.work_counter - 1) || *abort_flag) idx = -1;
        mbar_wait_bounded(&sm.item_empty[k & 1u], ((k >> 1) & 1u) ^ 1u, abort_flag, p.status);
        if (idx >= 0) {
          const int4* src = reinterpret_cast<const int4*>(p.items + idx);
          int4* dst = reinterpret_cast<int4*>(&sm.next_rec[k & 1u]);
          dst[0] = __ldg(src);
          dst[1] = __ldg(src + 1);
        }
        sm.next_item[k & 1u] = idx;
        mbar_arrive(&sm.item_full[k & 1u]);     // release semantics: index and record are visible to waiters
      }
      idx = __shfl_sync(0xffffffffu, idx, 0);
      if (idx < 0) break;
      const PrefillItem item = sm.next_rec[k & 1u];   // not overwritten before this warp draws item k + 2
      // ---- stage the item's Q tile (K-major, 128-byte swizzle) as soon as the previous item's
      // last S MMA has run, about a tile and an epilogue before it is needed.  Rows are (token, head of the kv group) pairs, head
      // fastest: exactly one TMA box of group heads x 128 / group tokens per half of the
      // dims when 128 is a multiple of the group (rows past the sequence then hold other
      // tokens' queries or zeros: their scores are masked and nothing of them is stored).
      {
        if (lane == 0) mbar_wait_bounded(&sm.q_empty, (k & 1u) ^ 1u, abort_flag, p.status);
        __syncwarp();
        if (p.q_by_tma) {
          if (lane == 0) {
            mbar_arrive_expect_tx(&sm.q_full, kTcQBytes);
            const int tok0 = item.q_start + item.row0 / p.group;
            tma_load_3d(sm.q, &q_map, &sm.q_full, 0, item.kv_head * p.group, tok0);
            tma_load_3d(sm.q + kPfRows * 128, &q_map, &sm.q_full, 64, item.kv_head * p.group, tok0);
          } else {
            mbar_arrive(&sm.q_full);
          }
        } else {
          // lane l copies rows l, l+32, ... (zero for unused rows), four 16-byte chunks in
          // flight: this warp runs on few registers
          const int rows_total = item.q_len * p.group;
#pragma unroll 1
          for (int r = lane; r < kPfRows; r += 32) {
            const int rg = item.row0 + r;
            const bool valid = rg < rows_total;
            const uint4* src = reinterpret_cast<const uint4*>(
                p.q + (int64_t)(item.q_start + (valid ? rg / p.group : 0)) * p.q_stride +
                (int64_t)(item.kv_head * p.group + (valid ? rg % p.group : 0)) * kPfHeadDim);
#pragma unroll 1
            for (int c0 = 0; c0 < 16; c0 += 4) {
              uint4 v[4];
#pragma unroll
              for (int c = 0; c < 4; ++c) v[c] = valid ? __ldg(src + c0 + c) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
              for (int c = 0; c < 4; ++c)
                *reinterpret_cast<uint4*>(sm.q + ((c0 + c) >> 3) * (kPfRows * 128) + swz128(r, (c0 + c) & 7)) = v[c];
            }
          }
          fence_proxy_async_smem();
          mbar_arrive(&sm.q_full);
        }
      }
      const int last_block = (item.kv_len - 1) >> p.block_shift;
      // K and V travel through separate rings: a K stage is free again as soon as
      // S = Q K^T has run, long before the V stage of the same tile (held until P V has
      // run).  So the K loads run kTcKLead tiles ahead of the V loads: a full V ring does
      // not keep the next K, which the S MMA needs first, from being requested.
      const int rot = first_tile(item);
      auto issue = [&](bool is_k, int step, uint32_t itx) {
        int bid = 0;
        int tile = step + rot;
        if (tile >= item.n_tiles) tile -= item.n_tiles;
        const int token0 = tile * kPfTile + lane * p.box_tokens;     // first token of this lane's box
        if (lane < nbox) {
          int lb = token0 >> p.block_shift;
          lb = lb > last_block ? last_block : lb;                  // tail boxes re-read the last valid page
          bid = __ldg(p.block_table + (int64_t)item.seq * p.bt_stride + lb);
        }
        if (bid < 0 || bid >= p.num_blocks) {
          if (lane < nbox && p.status) atomicOr(p.status, B200_STATUS_BAD_BLOCK);
          bid = p.num_blocks;
        }
        const int tok = token0 & (p.block_size - 1);
        if (is_k) {
          const int sk = itx % kTcKStages;
          if (lane == 0) {
            mbar_wait_bounded(&sm.k_empty[sk], ((itx / kTcKStages) & 1u) ^ 1u, abort_flag, p.status);
            mbar_arrive_expect_tx(&sm.k_full[sk], kPfTileBytes);
          }
          __syncwarp();
          if (lane < nbox) {
            uint8_t* dst = sm.k[sk] + lane * p.box_tokens * 128;
            tma_load_4d(dst, &k_map, &sm.k_full[sk], 0, item.kv_head, tok, bid);
            tma_load_4d(dst + kPfHalfTileBytes, &k_map, &sm.k_full[sk], 64, item.kv_head, tok, bid);
          }
        } else {
          const int sv = itx % kTcVStages;
          if (lane == 0) {
            mbar_wait_bounded(&sm.v_empty[sv], ((itx / kTcVStages) & 1u) ^ 1u, abort_flag, p.status);
            mbar_arrive_expect_tx(&sm.v_full[sv], kPfTileBytes);
          }
          __syncwarp();
          if (lane < nbox) {
            uint8_t* dst = sm.v[sv] + lane * p.box_tokens * 128;
            tma_load_4d(dst, &v_map, &sm.v_full[sv], 0, item.kv_head, tok, bid);
            tma_load_4d(dst + kPfHalfTileBytes, &v_map, &sm.v_full[sv], 64, item.kv_head, tok, bid);
          }
        }
        __syncwarp();
      };
      int kt = 0;                                  // next K tile to request
      for (int tile = 0; tile < item.n_tiles; ++tile) {
        for (; kt < item.n_tiles && kt <= tile + kTcKLead; ++kt) issue(true, kt, it + kt);
        issue(false, tile, it + tile);
      }
      it += item.n_tiles;
    }
    if (lane == 0) {   // drain: nothing may still be landing when the CTA leaves
      for (uint32_t k = 0; k < (uint32_t)kTcKStages && k < it; ++k) {
        const uint32_t j = it - 1 - k;
        mbar_wait_bounded(&sm.k_full[j % kTcKStages], (j / kTcKStages) & 1u, abort_flag, p.status);
      }
      for (uint32_t k = 0; k < (uint32_t)kTcVStages && k < it; ++k) {
        const uint32_t j = it - 1 - k;
        mbar_wait_bounded(&sm.v_full[j % kTcVStages], (j / kTcVStages) & 1u, abort_flag, p.status);
      }
    }
  } else if (warp == 9) {
    // ------------------------- MMA issuer: S = Q K^T -------------------------
    if (lane == 0) {
      constexpr uint32_t idesc_qk = umma_idesc_bf16(kPfRows, kPfTile, false);
      // descriptors differ only in their start-address field: build once, add offsets
      const uint64_t dq = umma_desc_sw128(smem_u32(sm.q), 16, 1024);
      const uint64_t dk = umma_desc_sw128(smem_u32(sm.k[0]), 16, 1024);
      const uint32_t dq_lo = (uint32_t)dq, dq_hi = (uint32_t)(dq >> 32);
      const uint32_t dk_lo = (uint32_t)dk, dk_hi = (uint32_t)(dk >> 32);
      uint32_t it = 0;
      for (uint32_t item_no = 0;; ++item_no) {
        PrefillItem rec;
        if (take_item(item_no, rec) < 0) break;
        const int n_tiles = rec.n_tiles;
        mbar_wait_bounded(&sm.q_full, item_no & 1u, abort_flag, p.status);
        const uint32_t q_lo = dq_lo;
        if (n_tiles == 0) umma_commit(&sm.q_empty);
        for (int tile = 0; tile < n_tiles; ++tile, ++it) {
          const int s = it % kTcKStages;
          const int b = it & 1u;
          mbar_wait_bounded(&sm.k_full[s], (it / kTcKStages) & 1u, abort_flag, p.status);
          PF_TRACE(13, it);
          mbar_wait_bounded(&sm.s_empty[b], ((it >> 1) & 1u) ^ 1u, abort_flag, p.status);
          PF_TRACE(15, it);
          tc_fence_after();
          const uint32_t k_lo = dk_lo + (uint32_t)((s * kPfTileBytes) >> 4);
          const uint32_t d_tmem = tmem + b * 128;
          umma_bf16_ss_lo<false>(d_tmem, q_lo, dq_hi, k_lo, dk_hi, idesc_qk);
#pragma unroll
          for (int ks = 1; ks < kPfHeadDim / 16; ++ks) {
            const int half = ks >> 2;
            umma_bf16_ss_lo<true>(d_tmem, q_lo + (uint32_t)((half * (kPfRows * 128) + (ks & 3) * 32) >> 4),
                                  dq_hi, k_lo + (uint32_t)((half * kPfHalfTileBytes + (ks & 3) * 32) >> 4),
                                  dk_hi, idesc_qk);
          }
          umma_commit(&sm.s_full[b]);
          umma_commit(&sm.k_empty[s]);
          if (tile == n_tiles - 1) umma_commit(&sm.q_empty);   // the Q buffer may be refilled
          PF_TRACE(4, it);
        }
      }
    }
    __syncwarp();
  } else if (warp == 10) {
    // ------------------------- MMA issuer: O += P V --------------------------
    if (lane == 0) {
      constexpr uint32_t idesc_pv = umma_idesc_bf16(kPfRows, kPfHeadDim, true);
      const uint64_t dv = umma_desc_sw128(smem_u32(sm.v[0]), kPfHalfTileBytes, 1024);
      const uint32_t dv_lo = (uint32_t)dv, dv_hi = (uint32_t)(dv >> 32);
      uint32_t it = 0;
      for (uint32_t item_no = 0;; ++item_no) {
        PrefillItem rec;
        if (take_item(item_no, rec) < 0) break;
        const int n_tiles = rec.n_tiles;
        for (int tile = 0; tile < n_tiles; ++tile, ++it) {
          const int s = it % kTcVStages;
          const int g = it & 1u;                            // the group that owns this tile
          mbar_wait_bounded(&sm.v_full[s], (it / kTcVStages) & 1u, abort_flag, p.status);
          mbar_wait_bounded(&sm.p_full[g], (it >> 1) & 1u, abort_flag, p.status);
          if (tile == 0 && item_no > 0)                     // the previous item's O has been read
            mbar_wait_bounded(&sm.o_free, (item_no - 1) & 1u, abort_flag, p.status);
          tc_fence_after();
          PF_TRACE(5, it);
          const uint32_t v_lo = dv_lo + (uint32_t)((s * kPfTileBytes) >> 4);
          const uint32_t p_tmem = tmem + kTcPCol + g * 64;  // P of the tile: 128 tokens as bf16 pairs
          const uint32_t d_tmem = tmem + kTcOCol;
          if (tile == 0)                                    // the first tile of the item overwrites
            umma_bf16_ts_lo<false>(d_tmem, p_tmem, v_lo, dv_hi, idesc_pv);
          else
            umma_bf16_ts_lo<true>(d_tmem, p_tmem, v_lo, dv_hi, idesc_pv);
#pragma unroll
          for (int ks = 1; ks < kPfTile / 16; ++ks)
            umma_bf16_ts_lo<true>(d_tmem, p_tmem + ks * 8, v_lo + (uint32_t)((ks * 2048) >> 4), dv_hi, idesc_pv);
          umma_commit(&sm.pv_done[g]);
          umma_commit(&sm.v_empty[s]);
          PF_TRACE(6, it);
        }
        umma_commit(&sm.o_done);
      }
    }
    __syncwarp();
  }
  } else if (warp < 8) {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kTcRegsSoftmax));
    // --------------------------- softmax + epilogue ---------------------------
    const int g = warp >> 2;                         // group: KV tiles whose running index & 1 == g
    const int r = threadIdx.x & 127;                 // query row of the tile == TMEM lane
    const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    const uint32_t o_col = lane_base + kTcOCol;
    const uint32_t p_col = lane_base + kTcPCol + g * 64;
    const int G = p.group;
    uint32_t it = 0;
    for (uint32_t item_no = 0;; ++item_no) {
      PrefillItem item;
      if (take_item(item_no, item) < 0) break;
      const int rows_total = item.q_len * G;
      const int rg = item.row0 + r;
      const bool valid = rg < rows_total;
      const int64_t tok = item.q_start + (valid ? rg / G : 0);
      const int head = item.kv_head * G + (valid ? rg % G : 0);
      const int lim = valid ? min(item.causal_base + rg / G, item.kv_len - 1) : -1;
      const int rot = first_tile(item);
      float m_ref = -INFINITY;       // maximum this group's row sum is scaled to
      float l = 0.f;
      for (int tile = 0; tile < item.n_tiles; ++tile, ++it) {
        if ((int)(it & 1u) != g) continue;             // the other group's tile
        const uint32_t sb = it & 1u;
        const uint32_t s_col = lane_base + sb * 128;
        if (r == 0) PF_TRACE(0, it);
        mbar_wait_bounded(&sm.s_full[sb], (it >> 1) & 1u, abort_flag, p.status);
        tc_fence_after();
        if (r == 0) PF_TRACE(1, it);
        int kv_tile = tile + rot;                      // the KV tile this step works on
        if (kv_tile >= item.n_tiles) kv_tile -= item.n_tiles;
        const int tbase = kv_tile * kPfTile;
        const bool need_mask = tbase + kPfTile - 1 > lim;
        // The whole score row goes to registers in one go and the S buffer straight back to
        // the MMA issuer.
        uint32_t sv[4][32];
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) tmem_ld32(s_col + q4 * 32, sv[q4]);
        tmem_wait_ld();
        tc_fence_before();
        mbar_arrive(&sm.s_empty[sb]);
        if (r == 0) PF_TRACE(10, it);
        if (need_mask) {
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4)
#pragma unroll
            for (int c = 0; c < 32; ++c)
              if (tbase + q4 * 32 + c > lim) sv[q4][c] = __float_as_uint(-INFINITY);
        }
        // The softmax warps are bound by instruction issue (two of them share a scheduler):
        // three-input maxima and, below, packed two-element fp32 multiply-adds and adds halve
        // the count of the row maximum, the scaling and the row sum.
        float mx;
        {
          float mq[8];                      // eight independent chains instead of one of 128
#pragma unroll
          for (int u = 0; u < 8; ++u) mq[u] = __uint_as_float(sv[0][u]);
#pragma unroll
          for (int c = 8; c < 120; c += 16)
#pragma unroll
            for (int u = 0; u < 8; ++u)
              mq[u] = fmax3(mq[u], __uint_as_float(sv[(c + u) >> 5][(c + u) & 31]),
                            __uint_as_float(sv[(c + 8 + u) >> 5][(c + 8 + u) & 31]));
#pragma unroll
          for (int u = 0; u < 8; ++u) mq[u] = fmaxf(mq[u], __uint_as_float(sv[3][24 + u]));
          mx = fmaxf(fmax3(mq[0], mq[1], mq[2]), fmax3(fmax3(mq[3], mq[4], mq[5]), mq[6], mq[7]));
        }
        // the maximum O is scaled to after the previous tile (owned by the other group)
        float m_in = -INFINITY;
        if (tile > 0) {
          mbar_wait_bounded(&sm.m_ready[(it - 1) & 1u], ((it - 1) >> 1) & 1u, abort_flag, p.status);
          m_in = sm.row_ms[(it - 1) & 1u][r];
        }
        // lazy rescale: only when some row of the warp outgrew the stale maximum by 2^8
        const bool grow = (mx - m_in) * p.scale_log2 > 8.f || (m_in == -INFINITY && mx > -INFINITY);
        const bool rescale = __any_sync(0xffffffffu, grow);
        const float m_used = rescale ? fmaxf(m_in, mx) : m_in;
        sm.row_ms[it & 1u][r] = m_used;
        mbar_arrive(&sm.m_ready[it & 1u]);             // release: the next tile's owner may go on
        if (r == 0) PF_TRACE(11, it);
        if (m_used != m_ref) {                         // bring this group's row sum to the new reference
          l *= (m_ref == -INFINITY) ? 0.f : fast_exp2((m_ref - m_used) * p.scale_log2);
          m_ref = m_used;
        }
        const float ms = (m_used == -INFINITY) ? 0.f : m_used * p.scale_log2;
        // The group's P buffer is free once the P V of its previous tile (of this item or the
        // one before) has run.  The group waited for the one before that two tiles ago, so
        // the parity wait cannot be off by a phase.
        if (it >= 2) {
          mbar_wait_bounded(&sm.pv_done[g], ((it - 2) >> 1) & 1u, abort_flag, p.status);
          tc_fence_after();
        }
        // O may be touched once the previous tile's P V (the other group's) has run: rare path
        if (rescale && tile > 0) {
          const float corr = (m_in == -INFINITY) ? 0.f : fast_exp2((m_in - m_used) * p.scale_log2);
          mbar_wait_bounded(&sm.pv_done[g ^ 1], ((it - 1) >> 1) & 1u, abort_flag, p.status);
          tc_fence_after();
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t orow[32];
            tmem_ld32(o_col + c * 32, orow);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) orow[i] = __float_as_uint(__uint_as_float(orow[i]) * corr);
            tmem_st32(o_col + c * 32, orow);
          }
        }
        // Probabilities, software-pipelined by a quarter of the row: the exponentials of
        // quarter q are issued while quarter q - 1 is summed and packed, so nothing waits for a
        // MUFU result.  P (bf16 pairs) goes to the group's buffer 64 columns at a time.
        float2 ls[4] = {{0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}};
        const float2 scale2 = make_float2(p.scale_log2, p.scale_log2), shift2 = make_float2(-ms, -ms);
        uint32_t pk[32];
#pragma unroll
        for (int q4 = 0; q4 <= 4; ++q4) {
#pragma unroll
          for (int c = 0; c < 32; c += 2) {
            if (q4 < 4) {
              const float2 x = __ffma2_rn(make_float2(__uint_as_float(sv[q4][c]), __uint_as_float(sv[q4][c + 1])),
                                          scale2, shift2);
              sv[q4][c] = __float_as_uint(fast_exp2(x.x));
              sv[q4][c + 1] = __float_as_uint(fast_exp2(x.y));
            }
            if (q4 > 0) {
              const float2 pp = make_float2(__uint_as_float(sv[q4 - 1][c]), __uint_as_float(sv[q4 - 1][c + 1]));
              ls[(c >> 1) & 3] = __fadd2_rn(ls[(c >> 1) & 3], pp);
              pk[((q4 - 1) & 1) * 16 + (c >> 1)] = pack_bf16(pp.x, pp.y);
            }
          }
          if (q4 == 2) tmem_st32(p_col, pk);
          if (q4 == 4) tmem_st32(p_col + 32, pk);
        }
        {
          const float2 a = __fadd2_rn(ls[0], ls[1]), b = __fadd2_rn(ls[2], ls[3]);
          l += (a.x + a.y) + (b.x + b.y);
        }
        if (r == 0) PF_TRACE(2, it);
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(&sm.p_full[g]);
        if (r == 0) PF_TRACE(3, it);
      }
      if (r == 0 && g == 0) PF_TRACE(7, it > 0 ? it - 1 : 0);
      // ---- hand the row sums to the epilogue warps and go on with the next item
      // the maxima only grow along the tiles: the last tile's is what O is scaled to
      float mm = -INFINITY;
      if (item.n_tiles > 0) {
        mbar_wait_bounded(&sm.m_ready[(it - 1) & 1u], ((it - 1) >> 1) & 1u, abort_flag, p.status);
        mm = sm.row_ms[(it - 1) & 1u][r];
      }
      if (item_no > 0) mbar_wait_bounded(&sm.l_empty, (item_no - 1) & 1u, abort_flag, p.status);
      sm.row_l[g][r] = (m_ref == -INFINITY) ? 0.f : l * fast_exp2((m_ref - mm) * p.scale_log2);
      if (g == 0) sm.row_mfin[r] = mm;
      mbar_arrive(&sm.l_full);
    }
  } else {
    // ------------------------------- epilogue --------------------------------
    // Thread e owns query row e (TMEM lane e): it takes O out of tensor memory as soon as
    // the item's last P V has run, frees the accumulator for the next item (whose first
    // tiles the softmax groups are already working on) and normalises and stores the row.
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kTcRegsEpilogue));
    const int r = threadIdx.x - (kTcThreads - kTcEpilogueThreads);
    const uint32_t o_col = tmem + ((uint32_t)((warp & 3) * 32) << 16) + kTcOCol;
    const int G = p.group;
    for (uint32_t item_no = 0;; ++item_no) {
      PrefillItem item;
      if (take_item(item_no, item) < 0) break;
      const int rg = item.row0 + r;
      const bool valid = rg < item.q_len * G;
      const int64_t tok = item.q_start + (valid ? rg / G : 0);
      const int head = item.kv_head * G + (valid ? rg % G : 0);
      mbar_wait_bounded(&sm.l_full, item_no & 1u, abort_flag, p.status);
      const float lsum = sm.row_l[0][r] + sm.row_l[1][r];
      const float mm = sm.row_mfin[r];
      mbar_arrive(&sm.l_empty);
      const float inv = lsum > 0.f ? 1.f / lsum : 0.f;
      mbar_wait_bounded(&sm.o_done, item_no & 1u, abort_flag, p.status);
      tc_fence_after();
      if (r == 0) PF_TRACE(9, 95 - item_no);
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t o[32];
        tmem_ld32(o_col + c * 32, o);
        tmem_wait_ld();
        if (c == 3) {                        // the whole row is out of tensor memory
          tc_fence_before();
          mbar_arrive(&sm.o_free);
        }
        if (!(lsum > 0.f)) {                 // no visible key: zeros, whatever the accumulator holds
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 0u;
        }
        if (valid) {
          const int64_t off = (tok * p.num_q_heads + head) * kPfHeadDim + c * 32;
          if (p.out_is_f32) {
            float* dst = reinterpret_cast<float*>(p.out) + off;
#pragma unroll
            for (int i = 0; i < 32; i += 4)
              *reinterpret_cast<float4*>(dst + i) =
                  make_float4(__uint_as_float(o[i]) * inv, __uint_as_float(o[i + 1]) * inv,
                              __uint_as_float(o[i + 2]) * inv, __uint_as_float(o[i + 3]) * inv);
          } else {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.out) + off;
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              uint4 v;
              v.x = pack_bf16(__uint_as_float(o[i]) * inv, __uint_as_float(o[i + 1]) * inv);
              v.y = pack_bf16(__uint_as_float(o[i + 2]) * inv, __uint_as_float(o[i + 3]) * inv);
              v.z = pack_bf16(__uint_as_float(o[i + 4]) * inv, __uint_as_float(o[i + 5]) * inv);
              v.w = pack_bf16(__uint_as_float(o[i + 6]) * inv, __uint_as_float(o[i + 7]) * inv);
              *reinterpret_cast<uint4*>(dst + i) = v;
            }
          }
        }
      }
      if (valid && p.lse_out)
        p.lse_out[tok * p.num_q_heads + head] = lsum > 0.f ? mm * p.scale + __logf(lsum) : -INFINITY;
      if (r == 0) PF_TRACE(8, 95 - item_no);
    }
  }
  // ---- teardown: everyone is done with tensor memory before it is released
  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tmem, kTcTmemCols);
  }
  // the last CTA to leave puts the queue back to zero for the next launch on this plan
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(p.work_counter + 1, 1) == (int)gridDim.x - 1) {
      p.work_counter[0] = 0;
      p.work_counter[1] = 0;
      __threadfence();
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
    // a sequence without keys (the empty slice of a context-parallel rank) is planned too:
    // its items have no tile and come out as zeros with lse = -inf
    if (q_len == 0 || rows <= min_rows) continue;
    const int base = causal_base ? causal_base[b] : kv_lens[b] - q_len;
    for (int row0 = 0; row0 < rows; row0 += kPfRows) {
      const int last_row = std::min(row0 + kPfRows, rows) - 1;
      const int lim = std::min(base + last_row / group, kv_lens[b] - 1);   // last visible key of the item
      const int n_tiles = lim < 0 ? 0 : lim / kPfTile + 1;
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
  info->num_tokens = num_tokens;
  return B200_OK;
}


#ifdef B200_TRACE
static long long* g_pf_trace = nullptr;
extern "C" void b200_debug_set_pf_trace(void* dev_ptr) { g_pf_trace = static_cast<long long*>(dev_ptr); }
#endif

// Shared launcher.  With `info` the step's item count is known on the host (no launch for an
// empty plan, a grid no larger than the item list); without it the launch depends only on the
// device and on num_tokens (the rows q holds), and the kernel reads the count from the plan.
static int launch_prefill(const char* who, const void* q, int64_t q_stride, const void* key_cache,
                          const void* value_cache, int num_blocks, int block_size,
                          const int32_t* block_table, int64_t bt_stride, int32_t* plan_dev,
                          const b200_prefill_plan_info* info, int num_tokens, int num_q_heads,
                          int num_kv_heads, int head_dim, float scale, void* out, int out_is_f32,
                          float* lse_out, int32_t* status, void* stream, int max_ctas = 0) {
  if (!q || !key_cache || !value_cache || !block_table || !plan_dev || !out || num_blocks <= 0 ||
      num_q_heads <= 0 || num_kv_heads <= 0 || num_q_heads % num_kv_heads || num_tokens < 0 || max_ctas < 0) {
    set_last_error("%s: null pointer or bad head counts", who);
    return B200_EINVAL;
  }
  if (head_dim != kPfHeadDim) {
    set_last_error("%s: head_dim %d unsupported (kernel is built for 128)", who, head_dim);
    return B200_EUNSUPPORTED;
  }
  if (block_size < 8 || (block_size & (block_size - 1))) {
    set_last_error("%s: block_size %d must be a power of two >= 8", who, block_size);
    return B200_EUNSUPPORTED;
  }
  if (reinterpret_cast<uintptr_t>(q) % 16 || (q_stride % 8) || q_stride < (int64_t)num_q_heads * head_dim ||
      reinterpret_cast<uintptr_t>(out) % 16 || reinterpret_cast<uintptr_t>(plan_dev) % 16) {
    set_last_error("%s: q, out and the plan must be 16-byte aligned, the q token stride a multiple of 8 elements and >= Hq*D", who);
    return B200_EALIGN;
  }
  const int box_tokens = block_size < 64 ? block_size : 64;
  CUtensorMap k_map, v_map;
  int rc = get_cache_tensor_map(key_cache, num_blocks, block_size, num_kv_heads, head_dim, box_tokens, &k_map);
  if (rc) return rc;
  rc = get_cache_tensor_map(value_cache, num_blocks, block_size, num_kv_heads, head_dim, box_tokens, &v_map);
  if (rc) return rc;

  // One TMA box per Q tile needs a group that divides 128.
  const int group = num_q_heads / num_kv_heads;
  const bool q_by_tma = kPfRows % group == 0 && num_tokens > 0;
  CUtensorMap q_map = k_map;      // placeholder when the tile is copied row by row
  if (q_by_tma) {
    rc = get_query_tensor_map(q, num_tokens, num_q_heads, q_stride, group, &q_map);
    if (rc) return rc;
  }

  PrefillParams p;
  p.q_by_tma = q_by_tma ? 1 : 0;
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.q_stride = q_stride;
  p.block_table = block_table;
  p.bt_stride = bt_stride;
  p.items = reinterpret_cast<const PrefillItem*>(plan_dev + kPlanHeaderInts);
  p.work_counter = plan_dev + 2;
  p.out = out;
  p.lse_out = lse_out;
  p.status = status;
  p.num_q_heads = num_q_heads;
  p.group = num_q_heads / num_kv_heads;
  p.block_size = block_size;
  p.block_shift = __builtin_ctz(block_size);
  p.num_blocks = num_blocks;
  p.box_tokens = box_tokens;
  p.boxes_per_tile = kPfTile / box_tokens;
  p.out_is_f32 = out_is_f32;
  p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;
#ifdef B200_TRACE
  p.trace = g_pf_trace;
#endif

  const size_t smem_tc = sizeof(TcSmem);
  static bool attr_tc[64] = {false};
  int dev_tc = 0;
  cudaGetDevice(&dev_tc);
  if (dev_tc >= 64 || !attr_tc[dev_tc]) {
    rc = check_cuda(cudaFuncSetAttribute(paged_prefill_tc_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_tc),
                    "paged_prefill_gqa smem attribute");
    if (rc) return rc;
    if (dev_tc < 64) attr_tc[dev_tc] = true;
  }
  int grid = b200_sm_count();
  if (grid <= 0) grid = 148;
  if (info && grid > info->num_items) grid = info->num_items;
  if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;     // the rest of the SMs are left to another kernel
  return check_cuda(launch_pdl(paged_prefill_tc_kernel, dim3(grid), dim3(kTcThreads), smem_tc,
                               static_cast<cudaStream_t>(stream), k_map, v_map, q_map, p),
                    "paged_prefill_gqa launch");
}

extern "C" int b200_paged_prefill_gqa(const void* q, int64_t q_stride, const void* key_cache,
                                      const void* value_cache, int num_blocks, int block_size,
                                      const int32_t* block_table, int64_t bt_stride,
                                      int32_t* plan_dev, const b200_prefill_plan_info* info,
                                      int num_q_heads, int num_kv_heads, int head_dim, float scale,
                                      void* out, int out_is_f32, float* lse_out, int32_t* status,
                                      void* stream) {
  if (!info) {
    set_last_error("paged_prefill_gqa: plan info is null");
    return B200_EINVAL;
  }
  if (info->num_items == 0) return B200_OK;
  return launch_prefill("paged_prefill_gqa", q, q_stride, key_cache, value_cache, num_blocks, block_size,
                        block_table, bt_stride, plan_dev, info, info->num_tokens, num_q_heads, num_kv_heads,
                        head_dim, scale, out, out_is_f32, lse_out, status, stream);
}

extern "C" int b200_paged_prefill_gqa_replayable(const void* q, int64_t q_stride, const void* key_cache,
                                                 const void* value_cache, int num_blocks, int block_size,
                                                 const int32_t* block_table, int64_t bt_stride,
                                                 int32_t* plan_dev, int num_tokens, int num_q_heads,
                                                 int num_kv_heads, int head_dim, float scale, void* out,
                                                 int out_is_f32, float* lse_out, int32_t* status,
                                                 void* stream) {
  return launch_prefill("paged_prefill_gqa_replayable", q, q_stride, key_cache, value_cache, num_blocks,
                        block_size, block_table, bt_stride, plan_dev, nullptr, num_tokens, num_q_heads,
                        num_kv_heads, head_dim, scale, out, out_is_f32, lse_out, status, stream);
}

extern "C" int b200_paged_prefill_gqa_on(const void* q, int64_t q_stride, const void* key_cache,
                                         const void* value_cache, int num_blocks, int block_size,
                                         const int32_t* block_table, int64_t bt_stride,
                                         int32_t* plan_dev, const b200_prefill_plan_info* info, int max_ctas,
                                         int num_q_heads, int num_kv_heads, int head_dim, float scale,
                                         void* out, int out_is_f32, float* lse_out, int32_t* status,
                                         void* stream) {
  if (!info) {
    set_last_error("paged_prefill_gqa_on: plan info is null");
    return B200_EINVAL;
  }
  if (info->num_items == 0) return B200_OK;
  return launch_prefill("paged_prefill_gqa_on", q, q_stride, key_cache, value_cache, num_blocks, block_size,
                        block_table, bt_stride, plan_dev, info, info->num_tokens, num_q_heads, num_kv_heads,
                        head_dim, scale, out, out_is_f32, lse_out, status, stream, max_ctas);
}
