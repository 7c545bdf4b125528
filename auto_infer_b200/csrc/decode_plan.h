// Layout of the split-KV decode plan shared by the host planner and the kernels.
//
//   [header: kPlanHeaderInts]
//   [one CtaRecord per CTA]                      fixed offset, fixed size
//   [MultiGroup records, capacity max_multi]     fixed offset
//   [DecodeItem records, n_items used]           fixed offset, variable length
//
// Every offset depends only on (num_ctas, num_seqs, num_kv_heads), never on the
// step's lengths, so a kernel launch recorded once (CUDA graph) stays valid when the
// buffer is refilled with another step's plan.
#pragma once
#include <stdint.h>

namespace b200 {

constexpr int kTileTokens = 64;      // KV tokens per pipeline stage (GQA kernels)
constexpr int kMlaTileTokens = 32;   // latent tokens per pipeline stage (MLA decode)
constexpr int kItemOverheadTiles = 5;   // planner's cost of one work item, in tiles (streaming cut)
constexpr int kMaxRows = 16;         // q_len * group rows one MMA tile holds
constexpr int kMaxDeferred = 8;      // cut pieces one CTA may hold (each may leave it a merge to run)
constexpr int kPlanMagic = 0x62323031;
constexpr int kPlanHeaderInts = 16;
constexpr int kCtaInts = 16;
constexpr int kItemInts = 12;
constexpr int kMultiInts = 8;

// header words
enum PlanHeader {
  kHdrMagic = 0, kHdrNumCtas, kHdrNumItems, kHdrNumPartials, kHdrNumMulti,
  kHdrOffCta, kHdrOffItems, kHdrOffMulti, kHdrTotalTiles, kHdrMaxPartials, kHdrMode
};

// One contiguous run of KV tiles of one (sequence, kv head) pair, owned by one CTA.
struct DecodeItem {
  int32_t seq, kv_head, tile_begin, tile_end;
  int32_t kv_len, q_start, q_len, causal_base;   // key j visible to row i iff j <= causal_base + i
  int32_t partial_idx, direct, multi_idx, pad1;  // direct: item covers the whole pair, write final output;
                                                 // multi_idx: the pair's MultiGroup record when it is cut
};
static_assert(sizeof(DecodeItem) == kItemInts * 4, "item layout");

// What a CTA needs to start: its item range and a copy of its first item, in one
// 64-byte record (one round trip to memory instead of range -> item).
struct CtaRecord {
  int32_t item_begin, item_end, pad0, pad1;
  DecodeItem first;
};
static_assert(sizeof(CtaRecord) == kCtaInts * 4, "cta record layout");

// A (sequence, kv head) pair split over several items.  `arrivals` counts, on the
// device, the items of the pair whose record has been written; the CTA that brings
// it to part_end - part_begin merges the records and puts the counter back to zero.
struct MultiGroup {
  int32_t q_start, q_len, kv_head, part_begin, part_end;
  int32_t arrivals;
  int32_t pad1, pad2;
};
static_assert(sizeof(MultiGroup) == kMultiInts * 4, "group layout");

inline int plan_max_items(int num_seqs, int num_kv_heads, int num_ctas) {
  return num_ctas + num_seqs * num_kv_heads;
}
inline int plan_max_multi(int num_seqs, int num_kv_heads, int num_ctas) {
  const int pairs = num_seqs * num_kv_heads;
  return pairs < num_ctas ? pairs : num_ctas;
}
inline int plan_off_cta() { return kPlanHeaderInts; }
inline int plan_off_multi(int num_ctas) { return kPlanHeaderInts + kCtaInts * num_ctas; }
inline int plan_off_items(int num_seqs, int num_kv_heads, int num_ctas) {
  return plan_off_multi(num_ctas) + kMultiInts * plan_max_multi(num_seqs, num_kv_heads, num_ctas);
}

}  // namespace b200
