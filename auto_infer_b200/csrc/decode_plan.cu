// Host planner of the split-KV decode kernels.  The per-step host lists it consumes
// are the ones auto_infer/worker/model_runner.py:126-136 builds (cumulative query
// lengths, per-sequence kv lengths).  Two ways of dealing the KV tiles of the
// (sequence, kv head) pairs to the persistent CTAs:
//
//   * whole pieces: every pair stays whole, or is cut into a few equal pieces when it
//     is much longer than a CTA's fair share, and the pieces are packed onto the CTAs
//     longest first.  Few work items, few or no partial records.  Chosen for small
//     steps (latency-bound: a CTA that finishes early leaves its memory bandwidth to
//     the others, so a moderate imbalance costs nothing) and whenever the packing
//     comes out balanced anyway (many pairs);
//   * streaming cut: the tiles of all pairs are laid end to end and the line is cut
//     into one range of equal cost per CTA, so every SM streams the same number of
//     bytes whatever the length distribution.  Chosen for long steps that the first
//     scheme would leave unbalanced.
#include <algorithm>
#include <cstring>
#include <queue>
#include <vector>

#include "common.cuh"
#include "decode_plan.h"

using namespace b200;

extern "C" size_t b200_decode_plan_bytes(int num_seqs, int num_kv_heads, int num_ctas) {
  if (num_seqs < 0 || num_kv_heads <= 0 || num_ctas <= 0) return 0;
  const size_t ints = (size_t)plan_off_items(num_seqs, num_kv_heads, num_ctas) +
                      (size_t)kItemInts * plan_max_items(num_seqs, num_kv_heads, num_ctas) + 4;
  return ints * sizeof(int32_t);
}

extern "C" size_t b200_decode_workspace_bytes(int num_seqs, int num_kv_heads, int num_ctas,
                                              int head_dim) {
  if (num_seqs < 0 || num_kv_heads <= 0 || num_ctas <= 0 || head_dim <= 0) return 0;
  const size_t parts = (size_t)plan_max_items(num_seqs, num_kv_heads, num_ctas);
  return parts * (kMaxRows * (size_t)head_dim + kMaxRows) * sizeof(float) + 256;
}

static int build_split_plan(const char* who, int tile_tokens, bool bandwidth_shared,
                            const int32_t* cu_q, const int32_t* kv_lens, const int32_t* causal_base,
                            int num_seqs, int num_q_heads, int num_kv_heads, int num_ctas,
                            int32_t* plan, size_t plan_bytes, b200_decode_plan_info* info);

extern "C" int b200_decode_plan(const int32_t* cu_q, const int32_t* kv_lens,
                                const int32_t* causal_base, int num_seqs, int num_q_heads,
                                int num_kv_heads, int num_ctas, int32_t* plan, size_t plan_bytes,
                                b200_decode_plan_info* info) {
  // the GQA kernel is bound by HBM bandwidth, which the CTAs share: uneven pieces are fine in a small step
  return build_split_plan("decode_plan", kTileTokens, true, cu_q, kv_lens, causal_base, num_seqs,
                          num_q_heads, num_kv_heads, num_ctas, plan, plan_bytes, info);
}

// The latent (MLA) decode kernel streams 32-token tiles of one shared latent head.
extern "C" int b200_mla_decode_plan(const int32_t* cu_q, const int32_t* kv_lens,
                                    const int32_t* causal_base, int num_seqs, int num_heads,
                                    int num_ctas, int32_t* plan, size_t plan_bytes,
                                    b200_decode_plan_info* info) {
  // the latent kernel runs at the pace of its own warps: only a balanced packing is as fast as the cut
  return build_split_plan("mla_decode_plan", kMlaTileTokens, false, cu_q, kv_lens, causal_base, num_seqs,
                          num_heads, 1, num_ctas, plan, plan_bytes, info);
}

extern "C" size_t b200_mla_decode_workspace_bytes(int num_seqs, int num_ctas, int kv_lora_rank) {
  if (num_seqs < 0 || num_ctas <= 0 || kv_lora_rank <= 0) return 0;
  const size_t parts = (size_t)plan_max_items(num_seqs, 1, num_ctas);
  return parts * (kMaxRows * (size_t)kv_lora_rank + kMaxRows) * sizeof(float) + 256;
}

namespace {

struct Pair {
  int seq, head, tiles, q_start, q_len, kv_len, base;
};

struct Piece {
  int pair, tile_begin, tile_end;
};

// Steps whose fair share per CTA is at most this many tiles are "short": fixed costs (pipeline
// ramp, the hand-over between two items of a CTA, the merge of a cut pair) weigh more than a
// moderate imbalance, because the memory bandwidth is shared: a CTA streaming next to idle SMs
// runs up to ~1.4x faster than its fair share (bounded by the bytes its ring keeps in flight).
constexpr int kShortStepTiles = 256;
// In a short step a piece may be this much longer than the fair share (x / 100); in a very
// short one (a few tens of microseconds) more, because every extra item and every cut pair
// costs microseconds of its own there.
constexpr int kPieceSlackPercent = 130;
constexpr int kTinyStepTiles = 64;
constexpr int kTinyPieceSlackPercent = 160;
// A longer step takes the whole-piece packing only if its longest CTA stays within this much
// of the fair share (x / 100): tighter for a kernel whose CTAs run at their own pace than for
// one whose CTAs share the memory bandwidth.
constexpr int kBalancedPercent = 104;
constexpr int kSharedBalancedPercent = 115;

DecodeItem make_item(const Pair& p, int tile_begin, int tile_end) {
  DecodeItem it;
  it.seq = p.seq;
  it.kv_head = p.head;
  it.tile_begin = tile_begin;
  it.tile_end = tile_end;
  it.kv_len = p.kv_len;
  it.q_start = p.q_start;
  it.q_len = p.q_len;
  it.causal_base = p.base;
  it.direct = (tile_begin == 0 && tile_end == p.tiles) ? 1 : 0;
  it.partial_idx = -1;
  it.multi_idx = -1;
  it.pad1 = 0;
  return it;
}

// Whole-piece packing.  Returns false when it does not apply (too many pieces for
// the plan format, or a larger step that it would leave unbalanced).
bool pack_whole_pieces(const std::vector<Pair>& pairs, int64_t total, int num_ctas, int max_items,
                       bool bandwidth_shared, std::vector<std::vector<Piece>>* per_cta) {
  const int64_t fair = (total + num_ctas - 1) / num_ctas;
  const bool small_step = bandwidth_shared && fair <= kShortStepTiles;
  int64_t cap = fair;
  if (small_step) cap = (fair * (fair <= kTinyStepTiles ? kTinyPieceSlackPercent : kPieceSlackPercent) + 99) / 100;
  if (cap < 4) cap = 4;
  std::vector<Piece> pieces;
  pieces.reserve(pairs.size() + num_ctas);
  for (size_t i = 0; i < pairs.size(); ++i) {
    const int t = pairs[i].tiles;
    const int k = t > 0 ? (int)((t + cap - 1) / cap) : 1;
    const int lo = t / k, rem = t % k;
    int at = 0;
    for (int j = 0; j < k; ++j) {
      const int len = lo + (j < rem ? 1 : 0);
      pieces.push_back(Piece{(int)i, at, at + len});
      at += len;
    }
    if ((int)pieces.size() > max_items) return false;
  }
  // longest first onto the least loaded CTA; ties broken by index, so the plan is deterministic
  std::vector<int> order(pieces.size());
  for (size_t i = 0; i < order.size(); ++i) order[i] = (int)i;
  std::stable_sort(order.begin(), order.end(), [&](int a, int b) {
    return pieces[a].tile_end - pieces[a].tile_begin > pieces[b].tile_end - pieces[b].tile_begin;
  });
  typedef std::pair<int64_t, int> Load;   // (tiles so far, cta)
  std::priority_queue<Load, std::vector<Load>, std::greater<Load>> heap;
  for (int c = 0; c < num_ctas; ++c) heap.push(Load(0, c));
  per_cta->assign(num_ctas, std::vector<Piece>());
  int64_t longest = 0;
  for (int idx : order) {
    Load l = heap.top();
    heap.pop();
    const Piece& pc = pieces[idx];
    // a second and later item of a CTA costs a hand-over (merge of the warps, Q reload)
    l.first += (pc.tile_end - pc.tile_begin) + ((*per_cta)[l.second].empty() ? 0 : 2);
    (*per_cta)[l.second].push_back(pc);
    longest = std::max(longest, l.first);
    heap.push(l);
  }
  for (const std::vector<Piece>& mine : *per_cta) {        // the kernel notes at most kMaxDeferred merges per CTA
    int cut = 0;
    for (const Piece& pc : mine) cut += (pc.tile_begin != 0 || pc.tile_end != pairs[pc.pair].tiles) ? 1 : 0;
    if (cut > kMaxDeferred) return false;
  }
  if (small_step) return true;
  const int64_t handovers = (int64_t)pieces.size() > num_ctas ? 2 * ((int64_t)pieces.size() - num_ctas) : 0;
  const int64_t fair_cost = (total + handovers + num_ctas - 1) / num_ctas;
#ifdef B200_FORCE_STREAMING_CUT
  return false;                                              // A/B builds only
#endif
  return longest * 100 <= fair_cost * (bandwidth_shared ? kSharedBalancedPercent : kBalancedPercent);
}

}  // namespace

static int build_split_plan(const char* who, int tile_tokens, bool bandwidth_shared,
                            const int32_t* cu_q, const int32_t* kv_lens, const int32_t* causal_base,
                            int num_seqs, int num_q_heads, int num_kv_heads, int num_ctas,
                            int32_t* plan, size_t plan_bytes, b200_decode_plan_info* info) {
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

  // pass 1: the (sequence, kv head) pairs this kernel takes
  std::vector<Pair> pairs;
  pairs.reserve((size_t)num_seqs * num_kv_heads);
  int64_t total = 0;
  int skipped = 0;
  int prev = 0;
  for (int b = 0; b < num_seqs; ++b) {
    const int q_start = prev;
    const int q_len = cu_q[b] - prev;
    prev = cu_q[b];
    if (q_len < 0 || kv_lens[b] < 0) {
      set_last_error("%s: sequence %d has negative length", who, b);
      return B200_EINVAL;
    }
    if (q_len == 0) continue;
    if (q_len * group > kMaxRows) {
      ++skipped;
      continue;
    }
    // A sequence without keys (the empty slice of a context-parallel rank) still gets an
    // item per kv head, with no tile: its rows come out as zeros with lse = -inf, so the
    // output of a step is fully written whatever the lengths.  (GQA kernel only.)
    if (kv_lens[b] == 0 && !bandwidth_shared) continue;
    const int tiles = (kv_lens[b] + tile_tokens - 1) / tile_tokens;
    const int base = causal_base ? causal_base[b] : kv_lens[b] - q_len;
    for (int h = 0; h < num_kv_heads; ++h)
      pairs.push_back(Pair{b, h, tiles, q_start, q_len, kv_lens[b], base});
    total += (int64_t)tiles * num_kv_heads;
  }
  if (total > INT32_MAX) {
    set_last_error("%s: %lld tiles exceed the int32 plan format", who, (long long)total);
    return B200_ETOOLARGE;
  }

  const int max_items = plan_max_items(num_seqs, num_kv_heads, num_ctas);
  const int max_multi = plan_max_multi(num_seqs, num_kv_heads, num_ctas);
  const int off_cta = plan_off_cta();
  const int off_multi = plan_off_multi(num_ctas);
  const int off_items = plan_off_items(num_seqs, num_kv_heads, num_ctas);
  CtaRecord* ctas = reinterpret_cast<CtaRecord*>(plan + off_cta);
  MultiGroup* multi = reinterpret_cast<MultiGroup*>(plan + off_multi);
  DecodeItem* items = reinterpret_cast<DecodeItem*>(plan + off_items);
  memset(ctas, 0, sizeof(CtaRecord) * num_ctas);

  int n_items = 0;
  int mode = 0;
  std::vector<std::vector<Piece>> per_cta;
  if (!pairs.empty() && pack_whole_pieces(pairs, total, num_ctas, max_items, bandwidth_shared, &per_cta)) {
    mode = 1;
    for (int c = 0; c < num_ctas; ++c) {
      ctas[c].item_begin = n_items;
      for (const Piece& pc : per_cta[c]) items[n_items++] = make_item(pairs[pc.pair], pc.tile_begin, pc.tile_end);
      ctas[c].item_end = n_items;
    }
  } else if (!pairs.empty()) {
    // Streaming cut.  Every item costs its tiles plus a fixed overhead (merge of the
    // warps' partial states, the record or output write, the next Q): ranges are cut to
    // equal COST, so a CTA whose range crosses pair boundaries gets fewer tiles.  The
    // number of items is about pairs + CTAs; any rounding error only shortens the last
    // ranges.
    const int64_t item_cost = total >= 8 * (int64_t)num_ctas ? kItemOverheadTiles : 0;
    const int64_t total_cost = total + item_cost * ((int64_t)pairs.size() + num_ctas);
    const int64_t quota_lo = total_cost / num_ctas;
    const int rem = (int)(total_cost % num_ctas);
    auto quota = [&](int c) -> int64_t { return quota_lo + (c < rem ? 1 : 0); };
    int cta = 0;
    int64_t cap = quota(0);
    ctas[0].item_begin = 0;
    for (const Pair& pr : pairs) {
      int t = 0;
      if (pr.tiles == 0) {                                   // an empty key range: one item without tiles
        items[n_items++] = make_item(pr, 0, 0);
        cap -= item_cost;
      }
      while (t < pr.tiles) {
        while (cap <= item_cost && cta + 1 < num_ctas) {  // no room for an item plus a tile: next CTA
          ctas[cta].item_end = n_items;
          ++cta;
          ctas[cta].item_begin = n_items;
          cap = quota(cta);
        }
        int64_t room = cap - item_cost;
        if (room < 1 || cta + 1 == num_ctas) room = pr.tiles - t;       // the last CTA takes what is left
        const int take = (int)((pr.tiles - t) < room ? (pr.tiles - t) : room);
        items[n_items++] = make_item(pr, t, t + take);
        t += take;
        cap -= take + item_cost;
      }
    }
    ctas[cta].item_end = n_items;
    for (int c = cta + 1; c < num_ctas; ++c) ctas[c].item_begin = ctas[c].item_end = n_items;
  }

  // partial records and groups: the pieces of a cut pair get consecutive record numbers
  // in tile order, whichever CTAs own them, so the merge order is fixed
  int n_parts = 0, n_multi = 0;
  {
    std::vector<int> first_part(pairs.size(), -1), n_pieces(pairs.size(), 0), group_of(pairs.size(), -1);
    // pairs are emitted seq-major, head-minor: index = position in `pairs`
    std::vector<int> pair_index((size_t)num_seqs * num_kv_heads, -1);
    for (size_t i = 0; i < pairs.size(); ++i) pair_index[(size_t)pairs[i].seq * num_kv_heads + pairs[i].head] = (int)i;
    for (int k = 0; k < n_items; ++k)
      if (!items[k].direct) ++n_pieces[pair_index[(size_t)items[k].seq * num_kv_heads + items[k].kv_head]];
    for (size_t i = 0; i < pairs.size(); ++i) {
      if (n_pieces[i] == 0) continue;
      if (n_multi >= max_multi) {
        set_last_error("%s: internal error, %d cut pairs exceed the plan format", who, n_multi + 1);
        return B200_EPLAN;
      }
      first_part[i] = n_parts;
      group_of[i] = n_multi;
      MultiGroup& g = multi[n_multi++];
      g.q_start = pairs[i].q_start;
      g.q_len = pairs[i].q_len;
      g.kv_head = pairs[i].head;
      g.part_begin = n_parts;
      g.part_end = n_parts + n_pieces[i];
      g.arrivals = 0;
      g.pad1 = g.pad2 = 0;
      n_parts += n_pieces[i];
    }
    // record number of a piece = first record of its pair + rank of its tile_begin among the pair's pieces
    std::vector<std::vector<std::pair<int, int>>> by_pair(pairs.size());   // (tile_begin, item)
    for (int k = 0; k < n_items; ++k)
      if (!items[k].direct)
        by_pair[pair_index[(size_t)items[k].seq * num_kv_heads + items[k].kv_head]].push_back({items[k].tile_begin, k});
    for (size_t i = 0; i < pairs.size(); ++i) {
      std::sort(by_pair[i].begin(), by_pair[i].end());
      for (size_t j = 0; j < by_pair[i].size(); ++j) {
        DecodeItem& it = items[by_pair[i][j].second];
        it.partial_idx = first_part[i] + (int)j;
        it.multi_idx = group_of[i];
      }
    }
  }
  for (int c = 0; c < num_ctas; ++c)
    if (ctas[c].item_end > ctas[c].item_begin) ctas[c].first = items[ctas[c].item_begin];

  plan[kHdrMagic] = kPlanMagic;
  plan[kHdrNumCtas] = num_ctas;
  plan[kHdrNumItems] = n_items;
  plan[kHdrNumPartials] = n_parts;
  plan[kHdrNumMulti] = n_multi;
  plan[kHdrOffCta] = off_cta;
  plan[kHdrOffItems] = off_items;
  plan[kHdrOffMulti] = off_multi;
  plan[kHdrTotalTiles] = (int32_t)total;
  plan[kHdrMaxPartials] = max_items;
  plan[kHdrMode] = mode;
  for (int i = kHdrMode + 1; i < kPlanHeaderInts; ++i) plan[i] = 0;

  info->num_ctas = num_ctas;
  info->num_items = n_items;
  info->num_partials = n_parts;
  info->num_multi = n_multi;
  info->total_tiles = (int32_t)total;
  info->skipped_seqs = skipped;
  info->plan_ints = off_items + kItemInts * n_items;
  info->mode = mode;
  return B200_OK;
}
