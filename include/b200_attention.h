/*
 * b200_attention.h — C ABI of the B200 (sm_100a) paged-attention library.
 *
 * Every entry point takes raw device pointers, plain sizes and a CUDA stream
 * (passed as void*; NULL = the legacy default stream).  None of them allocates
 * device memory unless its comment says so; the caller owns inputs, outputs and
 * workspaces.  Return value: 0 on success, a negative B200_E* code when an
 * argument is rejected (nothing is launched then).  Faults found on the device
 * (a block id outside the pool, a slot outside the cache, a wait that ran out)
 * never trap: the offending access is skipped and a bit is OR-ed into the int32
 * status word the caller passed (may be NULL).
 *
 * The functions replace the two vendor operators auto-infer's attention
 * backends call, plus the pieces a split / context-parallel run needs:
 *
 *   b200_reshape_and_cache      auto_infer/layers/attention/base.py:41-45   (write_kv)
 *   b200_paged_decode_gqa       auto_infer/layers/attention/base.py:48-61   (paged_fia, q_len*group <= 16)
 *   b200_paged_prefill_gqa      auto_infer/layers/attention/base.py:48-61   (paged_fia, any q_len)
 *   b200_mla_decode_absorbed    auto_infer/layers/attention/mla.py:115-120  (paged_fia over the 576-wide latent)
 *   b200_paged_mha              auto_infer/layers/attention/mla.py:56-63    (paged_fia, K 192 / V 128 per head)
 *   b200_lse_combine            no vendor counterpart; merges what graph_fia.py:41 calls [o, lse]
 *   b200_decode_plan*           host-side replacement of the per-step host length lists
 *                               (auto_infer/worker/model_runner.py:126-136)
 */
#ifndef B200_ATTENTION_H_
#define B200_ATTENTION_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- return codes ------------------------------------------------------ */
#define B200_OK               0
#define B200_EINVAL          -1   /* null pointer, negative size, bad stride        */
#define B200_EUNSUPPORTED    -2   /* shape outside what the kernels are built for   */
#define B200_EALIGN          -3   /* pointer / stride not aligned as required       */
#define B200_ECUDA           -4   /* a CUDA runtime / driver call failed            */
#define B200_ETOOLARGE       -5   /* exceeds a stated fixed capacity                */
#define B200_EPLAN           -6   /* plan buffer too small or inconsistent          */

/* ---- bits OR-ed into the device status word ------------------------------ */
#define B200_STATUS_BAD_SLOT      1   /* slot outside [0, num_blocks*block_size)   */
#define B200_STATUS_BAD_BLOCK     2   /* block id outside [0, num_blocks)          */
#define B200_STATUS_WAIT_TIMEOUT  4   /* a bounded barrier wait ran out            */
#define B200_STATUS_BAD_LAUNCH    8   /* a kernel found its launch state unusable  */

/* Library / build identification: "b200-attention <ver> sm_100a". */
const char* b200_version(void);
/* Text of the last rejected call on this thread (never NULL). */
const char* b200_last_error(void);
/* Number of SMs of the current device (persistent kernels launch one CTA each). */
int b200_sm_count(void);

/* ------------------------------------------------------------------------ *
 * KV-cache slot write.  Replaces write_kv
 * (auto_infer/layers/attention/base.py:41-45; callers gqa.py:76-79,
 * mla.py:113,243-245).
 *   key   (T, Hkv, k_dim) bf16, row t starts at key + t*key_stride (elements)
 *   value (T, Hkv, v_dim) bf16 or NULL (latent cache stored once)
 *   caches (num_blocks, block_size, Hkv, dim) bf16, contiguous
 *   slot_mapping (T,) int32: slot = block*block_size + offset; negative slots
 *   are skipped silently (padding rows), slots past the pool set BAD_SLOT.
 * Bit-exact copy. */
int b200_reshape_and_cache(const void* key, const void* value,
                           void* key_cache, void* value_cache,
                           const int32_t* slot_mapping,
                           int num_tokens, int num_kv_heads, int k_dim, int v_dim,
                           int64_t key_stride, int64_t value_stride,
                           int block_size, int num_blocks,
                           int32_t* status, void* stream);

/* ------------------------------------------------------------------------ *
 * Split-KV decode plan (host).  The reference hands the vendor op two host
 * lists per step (cumulative query lengths, per-sequence kv lengths:
 * auto_infer/worker/model_runner.py:126-136, forward_context.py:15-16).  Here
 * the same two lists are turned, once per step and for all layers, into a flat
 * work list of 64-token KV tile runs of the (sequence, kv head) pairs, dealt to
 * num_ctas persistent CTAs: whole pairs (or a few equal pieces of a long pair)
 * packed longest first when the step is small or the packing comes out
 * balanced, otherwise all tiles laid end to end and cut into num_ctas ranges of
 * equal cost, so that every CTA streams the same number of bytes whatever the
 * length distribution.
 *
 * Sequences whose q_len * (Hq/Hkv) exceeds 16 rows are left out (they belong to
 * b200_paged_prefill_gqa); their count is reported in info->skipped_seqs.
 *
 * causal_base may be NULL (then kv_len - q_len is used): key j of sequence b is
 * visible to its query row i iff j <= causal_base[b] + i.  A context-parallel
 * rank passes its local kv lengths and a base shifted by its slice offset.
 *
 * Every offset inside the plan depends on (num_seqs, num_kv_heads, num_ctas)
 * only, so a buffer of b200_decode_plan_bytes() can be refilled step after step
 * at one device address (see b200_paged_decode_gqa_replayable).
 */
typedef struct b200_decode_plan_info {
  int32_t num_ctas;        /* grid of the decode kernel                         */
  int32_t num_items;       /* work items (tile runs)                            */
  int32_t num_partials;    /* partial (o, lse) records the kernel writes        */
  int32_t num_multi;       /* (seq, kv head) pairs cut into several items       */
  int32_t total_tiles;     /* KV tiles over all pairs                           */
  int32_t skipped_seqs;    /* sequences too wide for the decode kernel          */
  int32_t plan_ints;       /* int32 words of the plan actually used             */
  int32_t mode;            /* 1: whole pieces packed, 0: streaming cut          */
} b200_decode_plan_info;

/* Upper bounds for sizing buffers before the lengths are known. */
size_t b200_decode_plan_bytes(int num_seqs, int num_kv_heads, int num_ctas);
size_t b200_decode_workspace_bytes(int num_seqs, int num_kv_heads, int num_ctas, int head_dim);

int b200_decode_plan(const int32_t* cu_seqlens_q_host, const int32_t* seqlens_kv_host,
                     const int32_t* causal_base_host,
                     int num_seqs, int num_q_heads, int num_kv_heads, int num_ctas,
                     int32_t* plan_host, size_t plan_bytes,
                     b200_decode_plan_info* info);

/* ------------------------------------------------------------------------ *
 * Paged GQA decode / MTP-verify attention, q_len * (Hq/Hkv) <= 16 per
 * sequence.  Replaces paged_fia (auto_infer/layers/attention/base.py:48-61) as
 * called from GqaFIABackend._attn (gqa.py:81-94) for decode-shaped rows.
 *   q (T, Hq, 128) bf16, row stride q_stride elements
 *   caches (num_blocks, block_size, Hkv, 128) bf16; block_size a power of two >= 8
 *   block_table (B, >= blocks needed) int32, row stride bt_stride
 *   plan_dev: device copy of the plan built by b200_decode_plan (info->plan_ints words),
 *             16-byte aligned; it must reach the device by a copy, not be written by the
 *             kernel launched just before this call.  Not const: it holds one arrival
 *             counter per cut pair, which the kernel counts up and puts back to zero (the
 *             CTA that completes a pair's records merges them, so there is no second
 *             kernel); one plan serves all layers of a step as long as calls sharing it
 *             do not overlap on the GPU
 *   workspace: room for info->num_partials records of 16*128+16 floats
 *             (b200_decode_workspace_bytes() is the upper bound for any plan of that
 *             geometry), 16-byte aligned
 *   out: (T, Hq, 128) bf16 when out_is_f32 == 0, fp32 otherwise (the fp32 form
 *        is one context-parallel rank's partial); lse_out (T, Hq) fp32 or NULL
 * Mask: bottom-right causal (sparse_mode 3 of the vendor op).  Cache rows past a
 * sequence's kv_len (the unwritten tail of its last page) are never read into the
 * arithmetic: they may hold any bytes. */
int b200_paged_decode_gqa(const void* q, int64_t q_stride,
                          const void* key_cache, const void* value_cache,
                          int num_blocks, int block_size,
                          const int32_t* block_table, int64_t bt_stride,
                          int32_t* plan_dev, const b200_decode_plan_info* info,
                          int num_q_heads, int num_kv_heads, int head_dim, float scale,
                          void* workspace, size_t workspace_bytes,
                          void* out, int out_is_f32, float* lse_out,
                          int32_t* status, void* stream);

/* ------------------------------------------------------------------------ *
 * The same attention as a launch that can be recorded once and replayed for
 * other steps (CUDA graph).  Replaces what the reference's graph mode does on
 * the host for every layer of every replay: re-issuing the attention task with
 * the step's length lists (GraphFiaLifecycle.update / update_many,
 * auto_infer/layers/attention/graph_fia.py:70-104).  Here the lengths live in
 * the plan on the device; nothing about the launch depends on them:
 *   - the grid is num_ctas, the counts and offsets are read from plan_dev by the
 *     kernel, nothing is skipped for an empty plan;
 *   - plan_dev has b200_decode_plan_bytes(num_seqs, Hkv, num_ctas) bytes and the
 *     workspace b200_decode_workspace_bytes(num_seqs, Hkv, num_ctas, 128) bytes,
 *     so that any later plan built for at most num_seqs sequences with the same
 *     num_ctas fits; before each replay the caller copies the new plan (its
 *     info->plan_ints words) to the same address, on the same stream or as a
 *     copy node of the graph from a fixed pinned buffer.
 * A plan built for another num_ctas sets B200_STATUS_BAD_LAUNCH and nothing is
 * computed. */
int b200_paged_decode_gqa_replayable(const void* q, int64_t q_stride,
                                     const void* key_cache, const void* value_cache,
                                     int num_blocks, int block_size,
                                     const int32_t* block_table, int64_t bt_stride,
                                     int32_t* plan_dev, int num_ctas,
                                     int num_q_heads, int num_kv_heads, int head_dim, float scale,
                                     void* workspace, size_t workspace_bytes,
                                     void* out, int out_is_f32, float* lse_out,
                                     int32_t* status, void* stream);

/* ------------------------------------------------------------------------ *
 * Slot write and attention of a step in one launch.  Replaces the pair
 * write_kv + paged_fia that every layer issues back to back
 * (auto_infer/layers/attention/base.py:41-61, called from
 * layers/attention/gqa.py:94-113): the new K/V rows of a sequence are the last
 * q_len keys of its own attention, so the CTA that streams the KV tile they fall
 * in takes them from k_new / v_new instead of from the (not yet written) cache
 * rows, and stores them to their slots itself.  One kernel less per layer and
 * no wait between the write and the first tile load.
 *   k_new / v_new (T, Hkv, 128) bf16, token strides k_new_stride / v_new_stride
 *       elements (multiples of 8, 16-byte aligned bases): row t of the packed
 *       query is the key at position kv_len - q_len + (t - q_start) of its
 *       sequence;
 *   slot_mapping (T,) int32 as b200_reshape_and_cache (negative: the row is
 *       not stored - it still takes part in the attention; past the pool:
 *       B200_STATUS_BAD_SLOT);
 *   key_cache / value_cache are written; everything else as
 *       b200_paged_decode_gqa.  With info == NULL the launch is the replayable
 *       one (grid num_ctas, counts read from the plan).
 * The result equals b200_reshape_and_cache followed by b200_paged_decode_gqa bit
 * for bit, provided slot_mapping names the rows the block table gives for those
 * positions (the reference computes both from the same table,
 * auto_infer/worker/model_runner.py:100-124).  Only sequences the plan covers are
 * written: a plan with info->skipped_seqs != 0 is refused (B200_EUNSUPPORTED);
 * with info == NULL that is the caller's to ensure.  Not for context-parallel
 * plans (a rank's causal_base is shifted there). */
int b200_paged_decode_gqa_write(const void* q, int64_t q_stride,
                                const void* k_new, int64_t k_new_stride,
                                const void* v_new, int64_t v_new_stride,
                                const int32_t* slot_mapping,
                                void* key_cache, void* value_cache,
                                int num_blocks, int block_size,
                                const int32_t* block_table, int64_t bt_stride,
                                int32_t* plan_dev, const b200_decode_plan_info* info, int num_ctas,
                                int num_q_heads, int num_kv_heads, int head_dim, float scale,
                                void* workspace, size_t workspace_bytes,
                                void* out, int out_is_f32, float* lse_out,
                                int32_t* status, void* stream);

/* ------------------------------------------------------------------------ *
 * Paged GQA attention for wide query blocks: chunked prefill over a cached
 * prefix and multi-token verify, any q_len, bottom-right causal.  Replaces
 * paged_fia (auto_infer/layers/attention/base.py:48-61) for the rows the decode
 * kernel leaves out.  The host plan cuts every (sequence, kv head) pair into
 * items of 128 packed query rows (row = query position x head within the kv
 * group) and sorts them by decreasing key count.
 *   min_rows: only sequences with q_len * (Hq/Hkv) > min_rows are planned
 *             (16 complements b200_decode_plan; 0 plans every sequence).
 * Arguments of the run call are those of b200_paged_decode_gqa without the
 * workspace (this kernel needs none).  plan_dev is not const: two of its header
 * words serve as the kernel's work-queue counters and are back at zero when the
 * kernel ends, so one plan serves all layers of a step as long as the calls that
 * share it do not overlap on the GPU.  q, out and plan_dev must be 16-byte
 * aligned and q_stride a multiple of 8 elements (B200_EALIGN otherwise); q must
 * hold at least info->num_tokens rows. */
typedef struct b200_prefill_plan_info {
  int32_t num_items;       /* 128-row work items                               */
  int32_t total_tiles;     /* 128-token KV tiles summed over the items          */
  int32_t plan_ints;       /* int32 words of the plan actually used            */
  int32_t num_tokens;      /* rows of q the plan covers (the last cu_seqlens_q) */
} b200_prefill_plan_info;

size_t b200_prefill_plan_bytes(int num_seqs, int num_tokens, int num_q_heads, int num_kv_heads);

int b200_prefill_plan(const int32_t* cu_seqlens_q_host, const int32_t* seqlens_kv_host,
                      const int32_t* causal_base_host,
                      int num_seqs, int num_q_heads, int num_kv_heads, int min_rows,
                      int32_t* plan_host, size_t plan_bytes,
                      b200_prefill_plan_info* info);

int b200_paged_prefill_gqa(const void* q, int64_t q_stride,
                           const void* key_cache, const void* value_cache,
                           int num_blocks, int block_size,
                           const int32_t* block_table, int64_t bt_stride,
                           int32_t* plan_dev, const b200_prefill_plan_info* info,
                           int num_q_heads, int num_kv_heads, int head_dim, float scale,
                           void* out, int out_is_f32, float* lse_out,
                           int32_t* status, void* stream);

/* The same on at most max_ctas SMs (0 = all), for a mixed step whose decode rows
 * and prefill chunks run side by side: the decode kernel is bound by memory
 * bandwidth and the wide-query kernel by the tensor pipe and shared memory, so a
 * step that gives each its share of the SMs (decode plan built for the other
 * num_ctas, the two launches on two streams) finishes sooner than one that runs
 * them one after the other on all SMs.  The kernels do not wait on one another. */
int b200_paged_prefill_gqa_on(const void* q, int64_t q_stride,
                              const void* key_cache, const void* value_cache,
                              int num_blocks, int block_size,
                              const int32_t* block_table, int64_t bt_stride,
                              int32_t* plan_dev, const b200_prefill_plan_info* info, int max_ctas,
                              int num_q_heads, int num_kv_heads, int head_dim, float scale,
                              void* out, int out_is_f32, float* lse_out,
                              int32_t* status, void* stream);

/* The wide-query attention as a launch that can be recorded once and replayed
 * for other steps (the prefill gears of the reference's graph runner,
 * auto_infer/worker/graph_decode_runner.py:360-414): the grid is the SM count,
 * the item count is read from the plan on the device.  plan_dev holds
 * b200_prefill_plan_bytes(num_seqs, num_tokens, Hq, Hkv) bytes for the largest
 * step of the gear and is refilled in place (the plan's first info->plan_ints
 * words) before each replay; q holds num_tokens rows (the gear's static buffer).
 * A refilled plan with no item at all is fine: every CTA leaves at once. */
int b200_paged_prefill_gqa_replayable(const void* q, int64_t q_stride,
                                      const void* key_cache, const void* value_cache,
                                      int num_blocks, int block_size,
                                      const int32_t* block_table, int64_t bt_stride,
                                      int32_t* plan_dev, int num_tokens,
                                      int num_q_heads, int num_kv_heads, int head_dim, float scale,
                                      void* out, int out_is_f32, float* lse_out,
                                      int32_t* status, void* stream);

/* ------------------------------------------------------------------------ *
 * Same attention as b200_paged_decode_gqa for callers that may not allocate
 * device memory.  (No counterpart in the reference: its vendor op manages its
 * own workspace.)  Two kinds of host are meant: a serving engine that handed
 * all free HBM to the paged KV pool at start-up, so that an allocation made
 * while a step runs can fail; and a latency-bound decode loop that cannot take
 * the device-wide synchronisation an allocation or a free brings.  The split-KV
 * partial records go to a fixed 8.06 MiB array inside the loaded module instead
 * of a caller workspace; every GPU that loads the library carries that array
 * until the process exits.  The call itself allocates nothing on the device
 * and frees nothing.
 *   - Limit: plans with more than 1024 partial records (info->num_partials;
 *     at most num_ctas + num_seqs * Hkv) are refused with B200_ETOOLARGE and
 *     nothing is launched.
 *   - The first call on each device looks the array's device address up (and,
 *     as any first launch does, loads the kernels); make that call during
 *     start-up, with the device current, before any stream capture begins.
 *   - All calls on a device share the one array and it keeps whatever the last
 *     call left.  Nothing in it has to start at zero: every record is written
 *     in full before it is read.  Two calls whose kernels overlap on the GPU
 *     (different streams) race on it; keep such calls on one stream or order
 *     them with events.
 *   - The looked-up address is kept per device in a table that is filled without
 *     a lock: two threads making the first call at once both look the same
 *     address up and store the same value.
 * All other arguments, outputs and return codes are those of
 * b200_paged_decode_gqa. */
int b200_paged_decode_gqa_static(const void* q, int64_t q_stride,
                                 const void* key_cache, const void* value_cache,
                                 int num_blocks, int block_size,
                                 const int32_t* block_table, int64_t bt_stride,
                                 int32_t* plan_dev, const b200_decode_plan_info* info,
                                 int num_q_heads, int num_kv_heads, int head_dim, float scale,
                                 void* out, int out_is_f32, float* lse_out,
                                 int32_t* status, void* stream);

/* ------------------------------------------------------------------------ *
 * Absorbed-MLA decode attention over the latent cache.  Replaces the paged_fia
 * call of mla_paged_absorbed (auto_infer/layers/attention/mla.py:115-120): one
 * shared latent head of width kv_lora_rank + rope_dim = 512 + 64 per token,
 * attended by all query heads, output = first kv_lora_rank columns.  The latent
 * is cached ONCE, (num_blocks, block_size, 1, 576) bf16 (the reference keeps a
 * second copy as V, mla.py:210-212, only because its vendor op wants symmetric
 * K and V); the tile in shared memory serves as K and as V.
 *   q_latent (T, H, 576) bf16 = [q_nope W_UK | q_pe], row stride q_stride
 *   sequences need q_len * H <= 16 (plan with b200_mla_decode_plan, which uses
 *   32-token tiles; buffers sized with b200_decode_plan_bytes(num_seqs, 1, ctas)
 *   and b200_mla_decode_workspace_bytes)
 *   out (T, H, 512) bf16 or fp32; lse_out (T, H) or NULL
 * scale is the model's softmax scale, (qk_nope + qk_rope)^-0.5 * yarn factor
 * (auto_infer/models/deepseek_v2.py:67,74), applied to the 576-wide products. */
int b200_mla_decode_plan(const int32_t* cu_seqlens_q_host, const int32_t* seqlens_kv_host,
                         const int32_t* causal_base_host,
                         int num_seqs, int num_heads, int num_ctas,
                         int32_t* plan_host, size_t plan_bytes,
                         b200_decode_plan_info* info);

size_t b200_mla_decode_workspace_bytes(int num_seqs, int num_ctas, int kv_lora_rank);

int b200_mla_decode_absorbed(const void* q_latent, int64_t q_stride,
                             const void* latent_cache, int num_blocks, int block_size,
                             const int32_t* block_table, int64_t bt_stride,
                             const int32_t* plan_dev, const b200_decode_plan_info* info,
                             int num_heads, int kv_lora_rank, int rope_dim, float scale,
                             void* workspace, size_t workspace_bytes,
                             void* out, int out_is_f32, float* lse_out,
                             int32_t* status, void* stream);

/* The same attention as a launch that can be recorded once and replayed for other
 * steps (CUDA graph), as b200_paged_decode_gqa_replayable: the grid is num_ctas,
 * counts and offsets are read from plan_dev; plan_dev has
 * b200_decode_plan_bytes(num_seqs, 1, num_ctas) bytes and the workspace
 * b200_mla_decode_workspace_bytes(num_seqs, num_ctas, 512) bytes for the largest
 * step the recording has to serve; before each replay the caller copies the new
 * plan to the same address.  The merge of cut sequences is launched for the most
 * cut sequences such a plan can have and leaves early for the rest.  A plan built
 * for another num_ctas, or one that needs more records than the workspace holds,
 * sets B200_STATUS_BAD_LAUNCH. */
int b200_mla_decode_absorbed_replayable(const void* q_latent, int64_t q_stride,
                                        const void* latent_cache, int num_blocks, int block_size,
                                        const int32_t* block_table, int64_t bt_stride,
                                        const int32_t* plan_dev, int num_ctas,
                                        int num_heads, int kv_lora_rank, int rope_dim, float scale,
                                        void* workspace, size_t workspace_bytes,
                                        void* out, int out_is_f32, float* lse_out,
                                        int32_t* status, void* stream);

/* ------------------------------------------------------------------------ *
 * Paged attention of the non-absorbed MLA form: one decompressed K (192 wide,
 * [k_nope | k_pe]) and V (128 wide) row per head and token, every query head
 * its own kv head.  Replaces the paged_fia call of mla_paged and of
 * MlaFIABackend._attn (auto_infer/layers/attention/mla.py:56-63, 243-254) with
 * the caches of MlaFIABackend.alloc_kv_caches (mla.py:214-216):
 *   key_cache (num_blocks, block_size, H, 192), value_cache (.., H, 128) bf16
 *   q (T, H, 192) bf16, token stride q_stride elements (even)
 *   out (T, H, 128) bf16 or fp32; lse_out (T, H) or NULL
 * Decode rows and prefill chunks of any q_len in one launch, bottom-right
 * causal; causal_base as in b200_decode_plan.  The host plan cuts every
 * sequence into blocks of 64 query positions per head and, when that gives too
 * few items for the SMs, every block's keys into up to 8 equal splits whose
 * normalised rows are merged by b200_lse_combine (launched by this call).
 *   plan buffer: b200_mha_plan_bytes(num_seqs, num_tokens, H) bytes (upper bound)
 *   workspace:   b200_mha_workspace_bytes(num_tokens, H) bytes (used when the
 *                plan has more than one split; may be NULL otherwise)
 * Cache rows past a sequence's kv_len may hold any bytes. */
typedef struct b200_mha_plan_info {
  int32_t num_items;     /* CTAs of the launch                                   */
  int32_t num_splits;    /* key splits per (block of rows, head), 1..8           */
  int32_t num_tokens;    /* packed query tokens the plan covers                  */
  int32_t plan_ints;     /* int32 words of the plan to copy to the device        */
  int32_t narrow;        /* 1: every block has <= 16 rows (decode / verify step)  */
  int32_t reserved;
  int64_t total_tiles;   /* 64-token tiles streamed by all items                 */
} b200_mha_plan_info;

size_t b200_mha_plan_bytes(int num_seqs, int num_tokens, int num_heads);
size_t b200_mha_workspace_bytes(int num_tokens, int num_heads);

int b200_mha_plan(const int32_t* cu_seqlens_q_host, const int32_t* seqlens_kv_host,
                  const int32_t* causal_base_host,
                  int num_seqs, int num_heads, int num_ctas,
                  int32_t* plan_host, size_t plan_bytes, b200_mha_plan_info* info);

int b200_paged_mha(const void* q, int64_t q_stride,
                   const void* key_cache, const void* value_cache,
                   int num_blocks, int block_size,
                   const int32_t* block_table, int64_t bt_stride,
                   const int32_t* plan_dev, const b200_mha_plan_info* info,
                   int num_heads, int k_dim, int v_dim, float scale,
                   void* workspace, size_t workspace_bytes,
                   void* out, int out_is_f32, float* lse_out,
                   int32_t* status, void* stream);

/* ------------------------------------------------------------------------ *
 * Merge n_parts normalised partial results by log-sum-exp:
 *   o_parts (n_parts, rows, D) fp32, lse_parts (n_parts, rows) fp32 (natural
 *   log, -inf = empty part)  ->  out (rows, D) bf16 (or fp32 if out_is_f32),
 *   lse_out (rows) or NULL.
 * part_stride_o / part_stride_lse are element strides between parts, so the
 * buffer an all-gather filled with per-rank [o | lse] records can be merged in
 * place.  Used for context-parallel partials; D must be a multiple of 4. */
int b200_lse_combine(const float* o_parts, const float* lse_parts,
                     int64_t part_stride_o, int64_t part_stride_lse,
                     int n_parts, int64_t rows, int head_dim,
                     void* out, int out_is_f32, float* lse_out, void* stream);

/* ------------------------------------------------------------------------ *
 * Context-parallel exchange fused with the merge (no counterpart in the
 * reference, whose only CP code all-gathers K and V per layer,
 * auto_infer/models/qwen2.py:211-212).  Every rank pushes its packed fp32
 * record [o (rows*D) | lse (rows)] into the receive buffers of all ranks with
 * peer-to-peer stores and merges the records that arrive in its own buffer.
 * The records travel as flagged 16-byte lines {payload, step, payload, step}
 * (two bf16 values of o per payload word, the row's lse as fp32 in a line of its
 * own): a receiver polls the lines it is about to merge, so no separate flag and
 * no acknowledgement round trip is needed.  The rows are dealt to the blocks of
 * the grid; a block waits only for the lines of its own rows.
 *   recv_ptrs_dev: device array of `world` pointers, entry r = base of rank r's
 *     receive buffer as mapped in this process (symmetric memory; the caller
 *     sets it up, zero-filled, b200_cp_exchange_buffer_bytes() bytes per rank)
 *   state_dev: 4 uint32 of local device memory, zero-filled once
 *   wait_limit_ns: how long a block waits for a peer's flag; 0 = one second.
 *     When it runs out the block sets B200_STATUS_WAIT_TIMEOUT and leaves the
 *     rows it has not merged yet unwritten; the step number still advances, so the next call
 *     starts a fresh step.  Ranks should therefore be lined up (a host barrier
 *     after set-up) before the first exchange.
 * All ranks must call it once per step with the same shapes. */
size_t b200_cp_exchange_buffer_bytes(int world, int64_t rows, int head_dim);

int b200_cp_exchange_combine(const float* local_record, const uint64_t* recv_ptrs_dev,
                             uint32_t* state_dev, int rank, int world,
                             int64_t rows, int head_dim, int64_t wait_limit_ns,
                             void* out, int out_is_f32, float* lse_out,
                             int32_t* status, void* stream);

/* ------------------------------------------------------------------------ *
 * Fused prologue of the GQA attention sub-block: what auto-infer runs between
 * the QKV projection and the attention call as separate elementwise ops
 * (auto_infer/layers/attention/gqa.py:40-47): optional per-head RMSNorm of q and
 * k (Qwen3; layers/norm.py:5-9), NeoX rotary embedding of q and k
 * (layers/rotary_embedding/__init__.py:10-12) and the slot write of k and v
 * (base.py:41-45).
 *   q / k / v: (T, H*, 128) bf16 views of the packed projection, token strides in
 *     elements; cos / sin (T, 1, 128) bf16, token stride cos_sin_stride
 *   q_norm_weight / k_norm_weight: (128) bf16, both or neither
 *   q_out (T, Hq, 128) bf16 (token stride q_out_stride): the rotated queries
 *   k_out (T, Hkv, 128) bf16 or NULL: the rotated keys, for callers that want them
 *   caches / slot_mapping: as b200_reshape_and_cache
 * Rounds to bf16 where the eager chain of bf16 tensors does, so q_out and the
 * cache rows equal that chain's. */
int b200_gqa_rope_cache(const void* q, int64_t q_stride, const void* k, int64_t k_stride,
                        const void* v, int64_t v_stride,
                        const void* cos, const void* sin, int64_t cos_sin_stride,
                        const void* q_norm_weight, const void* k_norm_weight, float eps,
                        void* q_out, int64_t q_out_stride, void* k_out,
                        void* key_cache, void* value_cache, const int32_t* slot_mapping,
                        int num_tokens, int num_q_heads, int num_kv_heads, int head_dim,
                        int block_size, int num_blocks, int32_t* status, void* stream);

/* Fused prologue of the absorbed-MLA sub-block (auto_infer/layers/attention/
 * mla.py:96-113): RMSNorm of the 512-wide latent, interleaved-to-halves
 * regrouping (layers/rotary_embedding/__init__.py:15-23) and rotary embedding
 * of the 64-wide decoupled key and of every head's q_pe, and the slot write of
 * the latent row [ckv | k_pe] into the single latent cache.
 *   ckv_full (T, 576) bf16: output of kv_a_proj_with_mqa, token stride ckv_stride
 *   q_pe (T, H, 64) bf16 view (token / head strides in elements) -> q_pe_out, a
 *     view of the same shape (e.g. the last 64 columns of the q_latent buffer)
 *   k_latent_out (T, 576) bf16 or NULL: the row as cached */
int b200_mla_rope_norm_cache(const void* ckv_full, int64_t ckv_stride,
                             const void* norm_weight, float eps,
                             const void* q_pe, int64_t q_pe_stride_t, int64_t q_pe_stride_h,
                             void* q_pe_out, int64_t q_out_stride_t, int64_t q_out_stride_h,
                             const void* cos, const void* sin, int64_t cos_sin_stride,
                             void* latent_cache, void* k_latent_out, const int32_t* slot_mapping,
                             int num_tokens, int num_heads, int kv_lora_rank, int rope_dim,
                             int block_size, int num_blocks, int32_t* status, void* stream);

/* ------------------------------------------------------------------------ *
 * Copy of selected pages between two paged caches of identical page layout (one
 * K or V tensor per call): the prefill-to-decode block transfer of
 * auto_infer/pd/connector.py:30-51 (copy_blocks), which copies block by block
 * with one tensor copy each.  Page i of the list goes from block
 * src_block_ids[i] of src_cache to block dst_block_ids[i] of dst_cache
 * (dst_block_ids NULL = the same ids, the reference's form).  The two caches
 * may sit on different GPUs of a node if one of them is peer-mapped into the
 * current device.  page_bytes = block_size * Hkv * dim * 2 must be a multiple of
 * 16.  Ids outside a pool are skipped and set B200_STATUS_BAD_BLOCK.  Bit-exact. */
int b200_copy_blocks(const void* src_cache, void* dst_cache,
                     const int32_t* src_block_ids, const int32_t* dst_block_ids, int num_ids,
                     int64_t page_bytes, int num_src_blocks, int num_dst_blocks,
                     int32_t* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif  /* B200_ATTENTION_H_ */
