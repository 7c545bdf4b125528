// Host planner of the split-KV decode kernel: lays the 64-token KV tiles of all
// (sequence, kv head) pairs end to end and cuts the line into one equal range
// per CTA, so every SM streams the same number of bytes whatever the context
// length distribution (the per-step host lists it consumes are the ones
// auto_infer/worker/model_runner.py:126-136 builds).
#include <cstring>

#include "common.cuh"
#include "decode_plan.h"

using namespace b200;

extern "C" size_t b200_decode_plan_bytes(int num_seqs, int num_kv_heads, int num_ctas) {
  if (num_seqs < 0 || num_kv_heads <= 0 || num_ctas <= 0) return 0;
  const size_t groups = (size_t)num_seqs * num_kv_heads;
  const size_t ints = kPlanHeaderInts + round_up4(num_ctas + 1) + kItemInts * (num_ctas + groups) +
                      kMultiInts * groups + 4;
  return ints * sizeof(int32_t);
}

extern "C" size_t b200_decode_workspace_bytes(int num_seqs, int num_kv_heads, int num_ctas,
                                              int head_dim) {
  if (num_seqs < 0 || num_kv_heads <= 0 || num_ctas <= 0 || head_dim <= 0) return 0;
  const size_t parts = (size_t)num_ctas + (size_t)num_seqs * num_kv_heads;
  return parts * (kMaxRows * (size_t)head_dim + kMaxRows) * sizeof(float) + 256;
}

static int build_split_plan(const char* who, int tile_tokens, const int32_t* cu_q,
                            const int32_t* kv_lens, const int32_t* causal_base, int num_seqs,
                            int num_q_heads, int num_kv_heads, int num_ctas, int32_t* plan,
                            size_t plan_bytes, b200_decode_plan_info* info);

extern "C" int b200_decode_plan(const int32_t* cu_q, const int32_t* kv_lens,
                                const int32_t* causal_base, int num_seqs, int num_q_heads,
                                int num_kv_heads, int num_ctas, int32_t* plan, size_t plan_bytes,
                                b200_decode_plan_info* info) {
  return build_split_plan("decode_plan", kTileTokens, cu_q, kv_lens, causal_base, num_seqs,
                          num_q_heads, num_kv_heads, num_ctas, plan, plan_bytes, info);
}

// The latent (MLA) decode kernel streams 32-token tiles of one shared latent head.
extern "C" int b200_mla_decode_plan(const int32_t* cu_q, const int32_t* kv_lens,
                                    const int32_t* causal_base, int num_seqs, int num_heads,
                                    int num_ctas, int32_t* plan, size_t plan_bytes,
                                    b200_decode_plan_info* info) {
  return build_split_plan("mla_decode_plan", kMlaTileTokens, cu_q, kv_lens, causal_base, num_seqs,
                          num_heads, 1, num_ctas, plan, plan_bytes, info);
}

extern "C" size_t b200_mla_decode_workspace_bytes(int num_seqs, int num_ctas, int kv_lora_rank) {
  if (num_seqs < 0 || num_ctas <= 0 || kv_lora_rank <= 0) return 0;
  const size_t parts = (size_t)num_ctas + (size_t)num_seqs;
  return parts * (kMaxRows * (size_t)kv_lora_rank + kMaxRows) * sizeof(float) + 256;
}

static int build_split_plan(const char* who, int tile_tokens, const int32_t* cu_q,
                            const int32_t* kv_lens, const int32_t* causal_base, int num_seqs,
                            int num_q_heads, int num_kv_heads, int num_ctas, int32_t* plan,
                            size_t plan_bytes, b200_decode_plan_info* info) {
  if (!plan || !info || num_seqs < 0 || (num_seqs > 0 && (!cu_q || !kv_lens)) || num_q_heads <= 0 ||
      num_kv_heads <= 0 || num_ctas <= 0 || num_q_heads % num_kv_heads != 0) {
    set_last_error("%s: bad argument (null pointer, heads not divisible, or size <= 0)", who);
    return B200_EINVAL;
  }
  if (plan_bytes < b200_decode_plan_bytes(num_seqs, num_kv_heads, num_ctas)) {
    set_last_error("%s: plan buffer of %zu bytes is smaller than b200_decode_plan_bytes()", who,
                   plan_bytes);
    return B200_EPLAN;
  }
  const int group = num_q_heads / num_kv_heads;
  memset(info, 0, sizeof(*info));

  // pass 1: tiles per sequence
  int64_t total = 0;
  int skipped = 0;
  int prev = 0;
  for (int b = 0; b < num_seqs; ++b) {
    const int q_len = cu_q[b] - prev;
    prev = cu_q[b];
    if (q_len < 0 || kv_lens[b] < 0) {
      set_last_error("%s: sequence %d has negative length", who, b);
      return B200_EINVAL;
    }
    if (q_len == 0 || kv_lens[b] == 0) continue;
    if (q_len * group > kMaxRows) {
      ++skipped;
      continue;
    }
    total += (int64_t)((kv_lens[b] + tile_tokens - 1) / tile_tokens) * num_kv_heads;
  }
  if (total > INT32_MAX) {
    set_last_error("%s: %lld tiles exceed the int32 plan format", who, (long long)total);
    return B200_ETOOLARGE;
  }

  const int off_cta = kPlanHeaderInts;
  const int off_items = off_cta + round_up4(num_ctas + 1);
  int32_t* cta_off = plan + off_cta;
  DecodeItem* items = reinterpret_cast<DecodeItem*>(plan + off_items);

  // Every item costs its tiles plus a fixed overhead (merge of the warps' partial
  // states, the record or output write, the next Q): ranges are cut to equal COST, so
  // a CTA whose range crosses pair boundaries gets fewer tiles.  The number of items
  // is about pairs + CTAs; any rounding error only shortens the last ranges.
  int64_t pairs = 0;
  {
    int pv = 0;
    for (int b = 0; b < num_seqs; ++b) {
      const int q_len = cu_q[b] - pv;
      pv = cu_q[b];
      if (q_len > 0 && kv_lens[b] > 0 && q_len * group <= kMaxRows) pairs += num_kv_heads;
    }
  }
  const int64_t item_cost = total >= 8 * (int64_t)num_ctas ? kItemOverheadTiles : 0;   // tiny steps: pure tile balance
  const int64_t total_cost = total + item_cost * (pairs + num_ctas);
  const int64_t quota_lo = total_cost / num_ctas;
  const int rem = (int)(total_cost % num_ctas);
  auto quota = [&](int c) -> int64_t { return quota_lo + (c < rem ? 1 : 0); };

  int n_items = 0, n_parts = 0, n_multi = 0;
  int cta = 0;
  int64_t cap = quota(0);
  cta_off[0] = 0;
  // the multi-group records are staged after the worst-case item area
  const size_t max_items = (size_t)num_ctas + (size_t)num_seqs * num_kv_heads;
  MultiGroup* multi = reinterpret_cast<MultiGroup*>(plan + off_items + kItemInts * max_items);

  prev = 0;
  for (int b = 0; b < num_seqs && total > 0; ++b) {
    const int q_start = prev;
    const int q_len = cu_q[b] - prev;
    prev = cu_q[b];
    if (q_len == 0 || kv_lens[b] == 0 || q_len * group > kMaxRows) continue;
    const int tiles = (kv_lens[b] + tile_tokens - 1) / tile_tokens;
    const int base = causal_base ? causal_base[b] : kv_lens[b] - q_len;
    for (int h = 0; h < num_kv_heads; ++h) {
      int t = 0;
      int first_part = n_parts;
      while (t < tiles) {
        while (cap <= item_cost && cta + 1 < num_ctas) {  // no room for an item plus a tile: next CTA
          ++cta;
          cta_off[cta] = n_items;
          cap = quota(cta);
        }
        int64_t room = cap - item_cost;
        if (room < 1 || cta + 1 == num_ctas) room = tiles - t;       // the last CTA takes what is left
        const int take = (int)((tiles - t) < room ? (tiles - t) : room);
        DecodeItem& it = items[n_items++];
        it.seq = b;
        it.kv_head = h;
        it.tile_begin = t;
        it.tile_end = t + take;
        it.kv_len = kv_lens[b];
        it.q_start = q_start;
        it.q_len = q_len;
        it.causal_base = base;
        it.direct = (take == tiles) ? 1 : 0;
        it.partial_idx = it.direct ? -1 : n_parts++;
        it.multi_idx = -1;
        it.pad1 = 0;
        t += take;
        cap -= take + item_cost;
      }
      if (n_parts > first_part) {
        // the items of this pair are the last ones emitted: point them at the pair's record
        for (int k = n_items - 1; k >= 0 && items[k].seq == b && items[k].kv_head == h; --k)
          items[k].multi_idx = n_multi;
        MultiGroup& g = multi[n_multi++];
        g.q_start = q_start;
        g.q_len = q_len;
        g.kv_head = h;
        g.part_begin = first_part;
        g.part_end = n_parts;
        g.arrivals = 0;
        g.pad1 = g.pad2 = 0;
      }
    }
  }
  for (int c = cta + 1; c <= num_ctas; ++c) cta_off[c] = n_items;

  // compact: move the multi-group records right behind the items actually used
  const int off_multi = off_items + kItemInts * n_items;
  memmove(plan + off_multi, multi, sizeof(MultiGroup) * n_multi);

  plan[kHdrMagic] = kPlanMagic;
  plan[kHdrNumCtas] = num_ctas;
  plan[kHdrNumItems] = n_items;
  plan[kHdrNumPartials] = n_parts;
  plan[kHdrNumMulti] = n_multi;
  plan[kHdrOffCta] = off_cta;
  plan[kHdrOffItems] = off_items;
  plan[kHdrOffMulti] = off_multi;
  plan[kHdrTotalTiles] = (int32_t)total;
  for (int i = kHdrTotalTiles + 1; i < kPlanHeaderInts; ++i) plan[i] = 0;

  info->num_ctas = num_ctas;
  info->num_items = n_items;
  info->num_partials = n_parts;
  info->num_multi = n_multi;
  info->total_tiles = (int32_t)total;
  info->skipped_seqs = skipped;
  info->plan_ints = off_multi + kMultiInts * n_multi;
  return B200_OK;
}
