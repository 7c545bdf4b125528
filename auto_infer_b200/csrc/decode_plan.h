// Layout of the split-KV decode plan shared by the host planner and the kernels.
#pragma once
#include <stdint.h>

namespace b200 {

constexpr int kTileTokens = 64;      // KV tokens per pipeline stage (GQA kernels)
constexpr int kMlaTileTokens = 32;   // latent tokens per pipeline stage (MLA decode)
constexpr int kItemOverheadTiles = 5;   // planner's cost of one work item, in tiles
constexpr int kMaxRows = 16;         // q_len * group rows one MMA tile holds
constexpr int kPlanMagic = 0x62323030;
constexpr int kPlanHeaderInts = 16;
constexpr int kItemInts = 12;
constexpr int kMultiInts = 8;

// header words
enum PlanHeader {
  kHdrMagic = 0, kHdrNumCtas, kHdrNumItems, kHdrNumPartials, kHdrNumMulti,
  kHdrOffCta, kHdrOffItems, kHdrOffMulti, kHdrTotalTiles
};

// One contiguous run of KV tiles of one (sequence, kv head) pair, owned by one CTA.
struct DecodeItem {
  int32_t seq, kv_head, tile_begin, tile_end;
  int32_t kv_len, q_start, q_len, causal_base;   // key j visible to row i iff j <= causal_base + i
  int32_t partial_idx, direct, multi_idx, pad1;  // direct: item covers the whole pair, write final output;
                                                 // multi_idx: the pair's MultiGroup record when it is cut
};
static_assert(sizeof(DecodeItem) == kItemInts * 4, "item layout");

// A (sequence, kv head) pair split over several items; merged by the combine pass.
struct MultiGroup {
  int32_t q_start, q_len, kv_head, part_begin, part_end;
  int32_t arrivals;    // device-side: items of the pair that have written their record (GQA decode merges in-kernel)
  int32_t pad1, pad2;
};
static_assert(sizeof(MultiGroup) == kMultiInts * 4, "group layout");

inline int round_up4(int x) { return (x + 3) & ~3; }

}  // namespace b200
