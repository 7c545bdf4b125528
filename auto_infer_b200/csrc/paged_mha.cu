// Paged multi-head attention with unequal key / value widths (192 / 128) for sm_100a: the
// non-absorbed form of MLA, where every head has its own decompressed K = [k_nope | k_pe]
// (192 wide) and V (128 wide) in the cache (auto_infer/layers/attention/mla.py:23-64).  One
// kernel serves decode rows and prefill chunks of any q_len, bottom-right causal.
//
// A work item is one block of up to 64 query positions of one (sequence, head) pair and one
// contiguous share ("split") of the 64-token KV tiles those positions can see.  One CTA per item:
//   * producer warp: per tile three K boxes and two V boxes (64 dims x 64 tokens, 128-byte
//     swizzle) by TMA into a ring of 40 KB stages;
//   * four consumer warps: S = Q K^T with mma.sync m16n8k16 (Q fragments in registers, K by
//     ldmatrix), online softmax in fp32 (exp2 domain), O += P V with P straight from registers
//     and V by ldmatrix.trans.
// Two instantiations.  "Wide" (any step): every warp owns 16 query rows and all 64 tokens of a
// tile (a warp without rows only keeps the ring moving), two stages, two CTAs per SM.  "Narrow"
// (a step in which every block has at most 16 rows: decode, verify): HBM-bound, so one CTA per SM
// with a five-stage ring (four tiles, 160 KB, in flight), all four warps on the same 16 rows and a
// quarter of each tile's tokens each, their (m, l, O) merged through shared memory at the end.
// With one split the rows are written as bf16 (or fp32) results; with more, every split writes
// a normalised fp32 row and its log-sum-exp, and b200_lse_combine merges the splits in a fixed
// order.  The host plan picks the number of splits so that a decode batch of a few sequences
// still fills the SMs.  Algorithmic bytes: sum over (sequence, head) of kv_len * 640 B.
#include <algorithm>
#include <vector>

#include "common.cuh"

namespace b200 {

constexpr int kMhaTile = 64;                                  // KV tokens per stage
constexpr int kMhaKDim = 192;
constexpr int kMhaVDim = 128;
constexpr int kMhaKSub = kMhaKDim / 64;                       // 64-dim sub-tiles of a K row
constexpr int kMhaVSub = kMhaVDim / 64;
constexpr int kMhaSubBytes = kMhaTile * 128;                  // [64 tokens][64 dims] bf16
constexpr int kMhaKBytes = kMhaKSub * kMhaSubBytes;
constexpr int kMhaStageBytes = (kMhaKSub + kMhaVSub) * kMhaSubBytes;   // 40 960
constexpr int kMhaWideStages = 2;
constexpr int kMhaNarrowStages = 5;
constexpr int kMhaWarps = 4;
constexpr int kMhaConsumerThreads = kMhaWarps * 32;
constexpr int kMhaThreads = kMhaConsumerThreads + 32;
constexpr int kMhaRows = 16 * kMhaWarps;                      // query positions per item
constexpr int kMhaMaxSplits = 8;
constexpr int kMhaMagic = 0x6d686131;
constexpr int kMhaHeaderInts = 16;
constexpr int kMhaItemInts = 12;

struct MhaItem {
  int32_t seq, head, tok0, n_rows;          // tok0: packed token index of the block's first row
  int32_t tile_begin, tile_end, kv_len;
  int32_t limit0;                           // last key row 0 may see (row i: limit0 + i)
  int32_t split, pad0, pad1, pad2;
};
static_assert(sizeof(MhaItem) == kMhaItemInts * 4, "item layout");

template <int kStages>
struct __align__(1024) MhaSmem {
  uint8_t stage[kStages][kMhaStageBytes];
  uint64_t full[kStages];
  uint64_t empty[kStages];
  int abort_flag;
};

struct MhaParams {
  const __nv_bfloat16* q;          // (T, H, 192)
  int64_t q_stride;
  const int32_t* block_table;
  int64_t bt_stride;
  const int32_t* plan;
  float* part_o;                   // (splits, T, H, 128) when splits > 1
  float* part_lse;                 // (splits, T, H)
  void* out;                       // (T, H, 128) bf16 or fp32
  float* lse_out;
  int32_t* status;
  int num_heads, num_tokens, num_splits;
  int block_size, block_shift, num_blocks, box_tokens, boxes_per_tile;
  int out_is_f32;
  float scale, scale_log2;
};

template <bool kNarrow>
__global__ void __launch_bounds__(kMhaThreads, kNarrow ? 1 : 2)
paged_mha_kernel(const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map,
                 const MhaParams p) {
  constexpr int kMhaStages = kNarrow ? kMhaNarrowStages : kMhaWideStages;
  extern __shared__ uint8_t smem_raw[];
  MhaSmem<kMhaStages>& sm =
      *reinterpret_cast<MhaSmem<kMhaStages>*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  MhaItem item;
  {
    const int4* ip = reinterpret_cast<const int4*>(p.plan + kMhaHeaderInts + (int64_t)blockIdx.x * kMhaItemInts);
    const int4 a = __ldg(ip), b = __ldg(ip + 1), c = __ldg(ip + 2);
    item.seq = a.x; item.head = a.y; item.tok0 = a.z; item.n_rows = a.w;
    item.tile_begin = b.x; item.tile_end = b.y; item.kv_len = b.z; item.limit0 = b.w;
    item.split = c.x;
  }
  if (threadIdx.x == 0) {
    sm.abort_flag = 0;
    for (int s = 0; s < kMhaStages; ++s) {
      mbar_init(&sm.full[s], 1);
      mbar_init(&sm.empty[s], kMhaWarps);
    }
    mbar_fence_init();
  }
  __syncthreads();
  grid_dep_launch();
  grid_dep_wait();                 // q and the step's new K / V rows come from earlier kernels
  volatile int* abort_flag = &sm.abort_flag;
  const int n_tiles = item.tile_end - item.tile_begin;

  if (warp == kMhaWarps) {
    // ------------------------------ producer ------------------------------
    if (lane == 0) {
      tma_prefetch_desc(&k_map);
      tma_prefetch_desc(&v_map);
    }
    const int nbox = p.boxes_per_tile;
    const int last_block = (item.kv_len - 1) >> p.block_shift;
    for (int it = 0; it < n_tiles; ++it) {
      const int tile = item.tile_begin + it;
      const int s = it % kMhaStages;
      int bid = 0;
      if (lane < nbox) {
        int lb = ((tile * kMhaTile) >> p.block_shift) + lane;
        lb = lb > last_block ? last_block : lb;       // boxes past the sequence's last page re-read it (masked)
        bid = __ldg(p.block_table + (int64_t)item.seq * p.bt_stride + lb);
        if (bid < 0 || bid >= p.num_blocks) {
          if (p.status) atomicOr(p.status, B200_STATUS_BAD_BLOCK);
          bid = p.num_blocks;                         // out of range: TMA fills zeros
        }
      }
      if (lane == 0) {
        mbar_wait_bounded(&sm.empty[s], ((it / kMhaStages) & 1u) ^ 1u, abort_flag, p.status);
        mbar_arrive_expect_tx(&sm.full[s], kMhaStageBytes);
      }
      __syncwarp();
      if (lane < nbox) {
        const int tok = (tile * kMhaTile + lane * p.box_tokens) & (p.block_size - 1);
        uint8_t* dst = sm.stage[s] + lane * p.box_tokens * 128;
#pragma unroll
        for (int c = 0; c < kMhaKSub; ++c)
          tma_load_4d(dst + c * kMhaSubBytes, &k_map, &sm.full[s], c * 64, item.head, tok, bid);
#pragma unroll
        for (int c = 0; c < kMhaVSub; ++c)
          tma_load_4d(dst + kMhaKBytes + c * kMhaSubBytes, &v_map, &sm.full[s], c * 64, item.head, tok, bid);
      }
      __syncwarp();
    }
    if (lane == 0) {               // every copy has landed before the CTA may leave
      const int n = n_tiles < kMhaStages ? n_tiles : kMhaStages;
      for (int k = 0; k < n; ++k) {
        const int j = n_tiles - 1 - k;
        mbar_wait_bounded(&sm.full[j % kMhaStages], (j / kMhaStages) & 1u, abort_flag, p.status);
      }
    }
    return;
  }

  // -------------------------------- consumers --------------------------------
  const int quad = lane >> 2;
  const int qlane = lane & 3;
  const int r0 = (kNarrow ? 0 : warp * 16) + quad, r1 = r0 + 8;
  const bool active = kNarrow || warp * 16 < item.n_rows;      // the whole warp, not the lane
  // ldmatrix lane addressing inside a 64-token sub-tile (before the swizzle)
  const int k_tok_l = ((lane >> 4) << 3) + (lane & 7);        // K: matrices 2,3 -> tokens +8
  const int k_chunk_sel = (lane >> 3) & 1;                    // K: matrices 1,3 -> dims +8
  const int v_tok_l = (((lane >> 3) & 1) << 3) + (lane & 7);  // V: matrices 1,3 -> tokens +8
  const int v_chunk_sel = lane >> 4;                          // V: matrices 2,3 -> dims +8

  uint32_t qf[kMhaKDim / 16][4];
  {
    const __nv_bfloat16* q0 = nullptr;
    const __nv_bfloat16* q1 = nullptr;
    if (r0 < item.n_rows) q0 = p.q + (int64_t)(item.tok0 + r0) * p.q_stride + (int64_t)item.head * kMhaKDim;
    if (r1 < item.n_rows) q1 = p.q + (int64_t)(item.tok0 + r1) * p.q_stride + (int64_t)item.head * kMhaKDim;
#pragma unroll
    for (int ks = 0; ks < kMhaKDim / 16; ++ks) {
      const int c = ks * 16 + qlane * 2;
      qf[ks][0] = q0 ? __ldg(reinterpret_cast<const uint32_t*>(q0 + c)) : 0u;
      qf[ks][1] = q1 ? __ldg(reinterpret_cast<const uint32_t*>(q1 + c)) : 0u;
      qf[ks][2] = q0 ? __ldg(reinterpret_cast<const uint32_t*>(q0 + c + 8)) : 0u;
      qf[ks][3] = q1 ? __ldg(reinterpret_cast<const uint32_t*>(q1 + c + 8)) : 0u;
    }
  }
  // last visible key per fragment row (-1: row unused, everything masked)
  const int lim0 = r0 < item.n_rows ? min(item.limit0 + r0, item.kv_len - 1) : -1;
  const int lim1 = r1 < item.n_rows ? min(item.limit0 + r1, item.kv_len - 1) : -1;

  float o[kMhaVDim / 8][4];
#pragma unroll
  for (int n = 0; n < kMhaVDim / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

  for (int it = 0; it < n_tiles; ++it) {
    const int tile = item.tile_begin + it;
    const int s = it % kMhaStages;
    mbar_wait_bounded(&sm.full[s], (it / kMhaStages) & 1u, abort_flag, p.status);
    const uint32_t kbase = smem_u32(sm.stage[s]);
    const uint32_t vbase = kbase + kMhaKBytes;
    // Rows past the sequence's end carry weight 0, but 0 x NaN is NaN: whatever bytes an
    // unwritten cache slot holds must not reach the MMA.  Only the sequence's last tile has
    // such rows; each warp clears 16 of them for all.
    const bool ragged = (tile + 1) * kMhaTile > item.kv_len;
    if (ragged) {
      const int first_bad = item.kv_len - tile * kMhaTile;
      for (int idx = lane; idx < 16 * 16; idx += 32) {
        const int row = warp * 16 + (idx >> 4), chunk = idx & 15;
        if (row >= first_bad)
          *reinterpret_cast<uint4*>(sm.stage[s] + kMhaKBytes + (chunk >> 3) * kMhaSubBytes + swz128(row, chunk & 7)) =
              make_uint4(0u, 0u, 0u, 0u);
      }
      named_bar_sync(1, kMhaConsumerThreads);
    }
    if constexpr (kNarrow) {
      // ---- this warp's 16 tokens of the tile: S (12 k-steps x 2 n-tiles), softmax, O += P V
      float sacc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
      for (int ks = 0; ks < kMhaKDim / 16; ++ks) {
        const int chunk = ks * 2 + k_chunk_sel;
        uint32_t kb[4];
        ldmatrix_x4(kb, kbase + (chunk >> 3) * kMhaSubBytes + swz128(warp * 16 + k_tok_l, chunk & 7));
        mma_bf16_16816(sacc[0], qf[ks], kb[0], kb[1]);
        mma_bf16_16816(sacc[1], qf[ks], kb[2], kb[3]);
      }
      const int tok0 = tile * kMhaTile + warp * 16 + qlane * 2;
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
        const float c0 = fast_exp2(m0 * p.scale_log2 - ms0);
        const float c1 = fast_exp2(m1 * p.scale_log2 - ms1);
        l0 *= c0;
        l1 *= c1;
#pragma unroll
        for (int n = 0; n < kMhaVDim / 8; ++n) {
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
#pragma unroll
      for (int j = 0; j < kMhaVDim / 16; ++j) {
        const int chunk = j * 2 + v_chunk_sel;
        uint32_t vb[4];
        ldmatrix_x4_trans(vb, vbase + (chunk >> 3) * kMhaSubBytes + swz128(warp * 16 + v_tok_l, chunk & 7));
        mma_bf16_16816(o[2 * j], pf, vb[0], vb[1]);
        mma_bf16_16816(o[2 * j + 1], pf, vb[2], vb[3]);
      }
    } else if (active) {
      // ---- S = Q K^T: 16 rows x 64 tokens (eight n-tiles of 8)
      float sacc[8][4];
#pragma unroll
      for (int n = 0; n < 8; ++n) sacc[n][0] = sacc[n][1] = sacc[n][2] = sacc[n][3] = 0.f;
#pragma unroll
      for (int ks = 0; ks < kMhaKDim / 16; ++ks) {
        const int chunk = ks * 2 + k_chunk_sel;            // 16-byte chunk of the 384-byte row
        const uint32_t sub = kbase + (chunk >> 3) * kMhaSubBytes;
#pragma unroll
        for (int tp = 0; tp < 4; ++tp) {
          uint32_t kb[4];
          ldmatrix_x4(kb, sub + swz128(tp * 16 + k_tok_l, chunk & 7));
          mma_bf16_16816(sacc[2 * tp], qf[ks], kb[0], kb[1]);
          mma_bf16_16816(sacc[2 * tp + 1], qf[ks], kb[2], kb[3]);
        }
      }
      // ---- mask + online softmax (fp32, exp2 domain)
      const int tok0 = tile * kMhaTile + qlane * 2;
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int n = 0; n < 8; ++n) {
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
        for (int n = 0; n < kMhaVDim / 8; ++n) {
          o[n][0] *= c0; o[n][1] *= c0; o[n][2] *= c1; o[n][3] *= c1;
        }
        m0 = mn0;
        m1 = mn1;
      }
      uint32_t pf[4][4];
#pragma unroll
      for (int kt = 0; kt < 4; ++kt) {
        float pr[2][4];
#pragma unroll
        for (int n = 0; n < 2; ++n) {
          pr[n][0] = fast_exp2(fmaf(sacc[2 * kt + n][0], p.scale_log2, -ms0));
          pr[n][1] = fast_exp2(fmaf(sacc[2 * kt + n][1], p.scale_log2, -ms0));
          pr[n][2] = fast_exp2(fmaf(sacc[2 * kt + n][2], p.scale_log2, -ms1));
          pr[n][3] = fast_exp2(fmaf(sacc[2 * kt + n][3], p.scale_log2, -ms1));
          l0 += pr[n][0] + pr[n][1];
          l1 += pr[n][2] + pr[n][3];
        }
        pf[kt][0] = pack_bf16(pr[0][0], pr[0][1]);
        pf[kt][1] = pack_bf16(pr[0][2], pr[0][3]);
        pf[kt][2] = pack_bf16(pr[1][0], pr[1][1]);
        pf[kt][3] = pack_bf16(pr[1][2], pr[1][3]);
      }
      // ---- O += P V (k = 64 tokens in four steps, n = 128 dims)
#pragma unroll
      for (int kt = 0; kt < 4; ++kt) {
#pragma unroll
        for (int j = 0; j < kMhaVDim / 16; ++j) {
          const int chunk = j * 2 + v_chunk_sel;
          uint32_t vb[4];
          ldmatrix_x4_trans(vb, vbase + (chunk >> 3) * kMhaSubBytes + swz128(kt * 16 + v_tok_l, chunk & 7));
          mma_bf16_16816(o[2 * j], pf[kt], vb[0], vb[1]);
          mma_bf16_16816(o[2 * j + 1], pf[kt], vb[2], vb[3]);
        }
      }
    }
    if (ragged) fence_proxy_async();   // the stage goes back to TMA: order the cleared rows before its writes
    __syncwarp();
    if (lane == 0) mbar_arrive(&sm.empty[s]);
  }

  // ---- rows of this warp: normalise and store
  if (!active) return;
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  if constexpr (kNarrow) {
    // merge of the four token slices in a fixed order through the (now idle) first stage:
    // [warp][16 rows][128] sums scaled to the warp's own maximum, then [warp][16] maxima and sums
    float* mo = reinterpret_cast<float*>(sm.stage[0]);
    float* mm = mo + kMhaWarps * 16 * kMhaVDim;
    float* ml = mm + kMhaWarps * 16;
    named_bar_sync(1, kMhaConsumerThreads);          // every warp has left the tile loop
#pragma unroll
    for (int n = 0; n < kMhaVDim / 8; ++n) {
      *reinterpret_cast<float2*>(mo + (warp * 16 + quad) * kMhaVDim + n * 8 + qlane * 2) = make_float2(o[n][0], o[n][1]);
      *reinterpret_cast<float2*>(mo + (warp * 16 + quad + 8) * kMhaVDim + n * 8 + qlane * 2) =
          make_float2(o[n][2], o[n][3]);
    }
    if (qlane == 0) {
      mm[warp * 16 + quad] = m0; mm[warp * 16 + quad + 8] = m1;
      ml[warp * 16 + quad] = l0; ml[warp * 16 + quad + 8] = l1;
    }
    named_bar_sync(1, kMhaConsumerThreads);
    const int t = threadIdx.x;                       // 128 threads: row t / 8, 16 columns each
    const int row = t >> 3, col = (t & 7) * 16;
    if (row >= item.n_rows) return;
    float g = -INFINITY;
#pragma unroll
    for (int w2 = 0; w2 < kMhaWarps; ++w2) g = fmaxf(g, mm[w2 * 16 + row]);
    float wgt[kMhaWarps], lsum = 0.f;
#pragma unroll
    for (int w2 = 0; w2 < kMhaWarps; ++w2) {
      const float mw = mm[w2 * 16 + row];
      wgt[w2] = (mw == -INFINITY) ? 0.f : fast_exp2((mw - g) * p.scale_log2);
      lsum += ml[w2 * 16 + row] * wgt[w2];
    }
    const float inv = lsum > 0.f ? 1.f / lsum : 0.f;
    const float lse = lsum > 0.f ? g * p.scale + __logf(lsum) : -INFINITY;
    float acc[16];
#pragma unroll
    for (int c = 0; c < 16; ++c) acc[c] = 0.f;
#pragma unroll
    for (int w2 = 0; w2 < kMhaWarps; ++w2) {
      const float4* src = reinterpret_cast<const float4*>(mo + (w2 * 16 + row) * kMhaVDim + col);
#pragma unroll
      for (int c4 = 0; c4 < 4; ++c4) {
        const float4 x = src[c4];
        acc[c4 * 4] += wgt[w2] * x.x; acc[c4 * 4 + 1] += wgt[w2] * x.y;
        acc[c4 * 4 + 2] += wgt[w2] * x.z; acc[c4 * 4 + 3] += wgt[w2] * x.w;
      }
    }
    const int64_t rix = (int64_t)(item.tok0 + row) * p.num_heads + item.head;
    if (p.num_splits > 1) {
      const int64_t prow = (int64_t)item.split * p.num_tokens * p.num_heads + rix;
      float* dst = p.part_o + prow * kMhaVDim + col;
#pragma unroll
      for (int c4 = 0; c4 < 4; ++c4)
        *reinterpret_cast<float4*>(dst + c4 * 4) = make_float4(acc[c4 * 4] * inv, acc[c4 * 4 + 1] * inv,
                                                               acc[c4 * 4 + 2] * inv, acc[c4 * 4 + 3] * inv);
      if ((t & 7) == 0) p.part_lse[prow] = lse;
    } else {
      const int64_t off = rix * kMhaVDim + col;
      if (p.out_is_f32) {
#pragma unroll
        for (int c4 = 0; c4 < 4; ++c4)
          *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out) + off + c4 * 4) =
              make_float4(acc[c4 * 4] * inv, acc[c4 * 4 + 1] * inv, acc[c4 * 4 + 2] * inv, acc[c4 * 4 + 3] * inv);
      } else {
        uint32_t pk[8];
#pragma unroll
        for (int c2 = 0; c2 < 8; ++c2) pk[c2] = pack_bf16(acc[c2 * 2] * inv, acc[c2 * 2 + 1] * inv);
        uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.out) + off);
        dst[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        dst[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
      }
      if (p.lse_out && (t & 7) == 0) p.lse_out[rix] = lse;
    }
  } else {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int row = half ? r1 : r0;
      if (row >= item.n_rows) continue;
      const float l = half ? l1 : l0, m = half ? m1 : m0;
      const float inv = l > 0.f ? 1.f / l : 0.f;
      const float lse = l > 0.f ? m * p.scale + __logf(l) : -INFINITY;
      const int64_t rix = (int64_t)(item.tok0 + row) * p.num_heads + item.head;
      if (p.num_splits > 1) {
        const int64_t prow = (int64_t)item.split * p.num_tokens * p.num_heads + rix;
        float* dst = p.part_o + prow * kMhaVDim;
#pragma unroll
        for (int n = 0; n < kMhaVDim / 8; ++n)
          *reinterpret_cast<float2*>(dst + n * 8 + qlane * 2) =
              make_float2(o[n][half * 2] * inv, o[n][half * 2 + 1] * inv);
        if (qlane == 0) p.part_lse[prow] = lse;
      } else {
#pragma unroll
        for (int n = 0; n < kMhaVDim / 8; ++n) {
          const float x = o[n][half * 2] * inv, y = o[n][half * 2 + 1] * inv;
          const int64_t off = rix * kMhaVDim + n * 8 + qlane * 2;
          if (p.out_is_f32)
            *reinterpret_cast<float2*>(reinterpret_cast<float*>(p.out) + off) = make_float2(x, y);
          else
            *reinterpret_cast<uint32_t*>(reinterpret_cast<__nv_bfloat16*>(p.out) + off) = pack_bf16(x, y);
        }
        if (p.lse_out && qlane == 0) p.lse_out[rix] = lse;
      }
    }
  }
}

}  // namespace b200

// ---------------------------------------------------------------------------
// Host plan
// ---------------------------------------------------------------------------
extern "C" size_t b200_mha_plan_bytes(int num_seqs, int num_tokens, int num_heads) {
  using namespace b200;
  if (num_seqs < 0 || num_tokens < 0 || num_heads <= 0) return 0;
  const int64_t blocks = (int64_t)num_seqs + num_tokens / kMhaRows;       // >= sum of ceil(q_len / 64)
  return (size_t)(kMhaHeaderInts + blocks * num_heads * kMhaMaxSplits * kMhaItemInts) * sizeof(int32_t);
}

extern "C" size_t b200_mha_workspace_bytes(int num_tokens, int num_heads) {
  using namespace b200;
  if (num_tokens < 0 || num_heads <= 0) return 0;
  return (size_t)kMhaMaxSplits * num_tokens * num_heads * (kMhaVDim + 1) * sizeof(float) + 16;
}

extern "C" int b200_mha_plan(const int32_t* cu_q, const int32_t* kv_lens, const int32_t* causal_base,
                             int num_seqs, int num_heads, int num_ctas, int32_t* plan_host,
                             size_t plan_bytes, b200_mha_plan_info* info) {
  using namespace b200;
  if (!info || !plan_host || num_seqs < 0 || num_heads <= 0 || num_ctas <= 0 || (num_seqs > 0 && (!cu_q || !kv_lens))) {
    set_last_error("mha_plan: null pointer or non-positive size");
    return B200_EINVAL;
  }
  struct Block { int seq, tok0, n_rows, kv_len, limit0, n_tiles; };
  std::vector<Block> blocks;
  int prev = 0, max_tiles = 0;
  int64_t total_tiles = 0;
  for (int b = 0; b < num_seqs; ++b) {
    const int q_len = cu_q[b] - prev;
    const int kv_len = kv_lens[b];
    if (q_len < 0 || kv_len < 0) {
      set_last_error("mha_plan: sequence %d has negative q_len or kv_len", b);
      return B200_EINVAL;
    }
    const int base = causal_base ? causal_base[b] : kv_len - q_len;
    for (int r = 0; r < q_len; r += kMhaRows) {
      const int n_rows = std::min(kMhaRows, q_len - r);
      int last = std::min(base + r + n_rows - 1, kv_len - 1);          // last key any row of the block sees
      const int n_tiles = last < 0 ? 0 : last / kMhaTile + 1;
      blocks.push_back(Block{b, prev + r, n_rows, kv_len, base + r, n_tiles});
      max_tiles = std::max(max_tiles, n_tiles);
      total_tiles += n_tiles;
    }
    prev = cu_q[b];
  }
  const int num_tokens = prev;
  const int64_t base_items = (int64_t)blocks.size() * num_heads;
  bool narrow = true;
  for (const Block& blk : blocks) narrow &= blk.n_rows <= 16;
  int splits = 1;
  if (base_items > 0) {
    // wide: two CTAs per SM, and twice that many items to even out their lengths; narrow: one
    // CTA per SM, three items each
    const int64_t want = (narrow ? 3LL : 4LL) * num_ctas;
    splits = (int)std::min<int64_t>(kMhaMaxSplits, (want + base_items - 1) / base_items);
    splits = std::max(1, std::min(splits, max_tiles / 4));             // at least four tiles per split
  }
  const size_t need = (size_t)(kMhaHeaderInts + base_items * splits * kMhaItemInts) * sizeof(int32_t);
  if (plan_bytes < need) {
    set_last_error("mha_plan: plan buffer %zu bytes < %zu needed", plan_bytes, need);
    return B200_EPLAN;
  }
  std::vector<MhaItem> items;
  items.reserve((size_t)base_items * splits);
  for (const Block& blk : blocks) {
    const int per = (blk.n_tiles + splits - 1) / splits;
    for (int h = 0; h < num_heads; ++h)
      for (int s = 0; s < splits; ++s) {
        const int t0 = std::min(blk.n_tiles, s * per), t1 = std::min(blk.n_tiles, (s + 1) * per);
        items.push_back(MhaItem{blk.seq, h, blk.tok0, blk.n_rows, t0, t1, blk.kv_len, blk.limit0, s, 0, 0, 0});
      }
  }
  std::stable_sort(items.begin(), items.end(), [](const MhaItem& a, const MhaItem& b) {
    return a.tile_end - a.tile_begin > b.tile_end - b.tile_begin;     // long items first
  });
  std::fill(plan_host, plan_host + kMhaHeaderInts, 0);
  plan_host[0] = kMhaMagic;
  plan_host[1] = (int32_t)items.size();
  plan_host[2] = splits;
  plan_host[3] = num_tokens;
  plan_host[4] = narrow ? 1 : 0;
  if (!items.empty())
    std::copy(reinterpret_cast<const int32_t*>(items.data()),
              reinterpret_cast<const int32_t*>(items.data()) + items.size() * kMhaItemInts,
              plan_host + kMhaHeaderInts);
  info->num_items = (int32_t)items.size();
  info->num_splits = splits;
  info->num_tokens = num_tokens;
  info->narrow = narrow ? 1 : 0;
  info->plan_ints = (int32_t)(kMhaHeaderInts + items.size() * kMhaItemInts);
  info->total_tiles = total_tiles * num_heads;
  return B200_OK;
}

extern "C" int b200_paged_mha(const void* q, int64_t q_stride, const void* key_cache, const void* value_cache,
                              int num_blocks, int block_size, const int32_t* block_table, int64_t bt_stride,
                              const int32_t* plan_dev, const b200_mha_plan_info* info, int num_heads,
                              int k_dim, int v_dim, float scale, void* workspace, size_t workspace_bytes,
                              void* out, int out_is_f32, float* lse_out, int32_t* status, void* stream) {
  using namespace b200;
  if (!info) {
    set_last_error("paged_mha: plan info is null");
    return B200_EINVAL;
  }
  if (info->num_items == 0) return B200_OK;
  if (!q || !key_cache || !value_cache || !block_table || !plan_dev || !out || num_blocks <= 0 || num_heads <= 0) {
    set_last_error("paged_mha: null pointer or non-positive size");
    return B200_EINVAL;
  }
  if (k_dim != kMhaKDim || v_dim != kMhaVDim) {
    set_last_error("paged_mha: head widths %d / %d unsupported (kernel is built for 192 / 128)", k_dim, v_dim);
    return B200_EUNSUPPORTED;
  }
  if (block_size < 8 || (block_size & (block_size - 1))) {
    set_last_error("paged_mha: block_size %d must be a power of two >= 8", block_size);
    return B200_EUNSUPPORTED;
  }
  if (reinterpret_cast<uintptr_t>(q) % 4 || (q_stride % 2) || q_stride < (int64_t)num_heads * kMhaKDim ||
      reinterpret_cast<uintptr_t>(out) % 8) {
    set_last_error("paged_mha: q must be 4-byte aligned with an even token stride, out 8-byte aligned");
    return B200_EALIGN;
  }
  const int splits = info->num_splits;
  const int64_t rows = (int64_t)info->num_tokens * num_heads;
  float* part_o = nullptr;
  float* part_lse = nullptr;
  if (splits > 1) {
    const size_t need = (size_t)splits * rows * (kMhaVDim + 1) * sizeof(float);
    if (!workspace || workspace_bytes < need || reinterpret_cast<uintptr_t>(workspace) % 16) {
      set_last_error("paged_mha: workspace %zu bytes < %zu needed (or missing / not 16-byte aligned)",
                     workspace_bytes, need);
      return B200_EPLAN;
    }
    part_o = static_cast<float*>(workspace);
    part_lse = part_o + (size_t)splits * rows * kMhaVDim;
  }
  const int box_tokens = block_size < kMhaTile ? block_size : kMhaTile;
  CUtensorMap k_map, v_map;
  int rc = get_cache_tensor_map(key_cache, num_blocks, block_size, num_heads, kMhaKDim, box_tokens, &k_map);
  if (rc) return rc;
  rc = get_cache_tensor_map(value_cache, num_blocks, block_size, num_heads, kMhaVDim, box_tokens, &v_map);
  if (rc) return rc;

  MhaParams p;
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.q_stride = q_stride;
  p.block_table = block_table;
  p.bt_stride = bt_stride;
  p.plan = plan_dev;
  p.part_o = part_o;
  p.part_lse = part_lse;
  p.out = out;
  p.lse_out = lse_out;
  p.status = status;
  p.num_heads = num_heads;
  p.num_tokens = info->num_tokens;
  p.num_splits = splits;
  p.block_size = block_size;
  p.block_shift = __builtin_ctz(block_size);
  p.num_blocks = num_blocks;
  p.box_tokens = box_tokens;
  p.boxes_per_tile = kMhaTile / box_tokens;
  p.out_is_f32 = out_is_f32;
  p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;

  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int which = info->narrow ? 1 : 0;
  auto kernel = which ? paged_mha_kernel<true> : paged_mha_kernel<false>;
  const size_t smem = (which ? sizeof(MhaSmem<kMhaNarrowStages>) : sizeof(MhaSmem<kMhaWideStages>)) + 1024;
  static bool attr_set[2][64] = {{false}, {false}};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 64 || !attr_set[which][dev]) {
    rc = check_cuda(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem),
                    "paged_mha smem attribute");
    if (rc) return rc;
    if (dev < 64) attr_set[which][dev] = true;
  }
  rc = check_cuda(launch_pdl(kernel, dim3(info->num_items), dim3(kMhaThreads), smem, s, k_map, v_map, p),
                  "paged_mha launch");
  if (rc || splits == 1) return rc;
  return b200_lse_combine(part_o, part_lse, rows * kMhaVDim, rows, splits, rows, kMhaVDim, out, out_is_f32,
                          lse_out, stream);
}
