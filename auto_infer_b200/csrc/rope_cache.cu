// Prologue of the attention sub-block, fused: what sits between the QKV projection and the
// attention call in auto-infer's backends.
//
//   GQA (auto_infer/layers/attention/gqa.py:40-47): optional per-head RMSNorm of q and k
//   (Qwen3), NeoX rotary embedding of q and k
//   (auto_infer/layers/rotary_embedding/__init__.py:10-12), then the slot write of k and v.
//   MLA (auto_infer/layers/attention/mla.py:96-113): RMSNorm of the 512-wide latent, the
//   interleaved-to-halves regrouping (rotary_embedding/__init__.py:15-23) and rotary
//   embedding of the 64-wide decoupled key and of every head's q_pe, then the slot write of
//   the latent row [ckv | k_pe].
//
// The reference runs these as six to eight elementwise launches on bf16 tensors.  Every
// intermediate of that chain is a bf16 tensor, and the kernels here round at exactly the
// same places (x*cos, rot(x)*sin and their sum are each rounded to bf16; the norm is taken
// in fp32, rounded, then scaled by the weight and rounded again), so the cache rows equal
// the eager chain's bit for bit wherever the fp32 sum of squares does (it is summed in
// another order: a last-place difference of the rsqrt can flip one bf16 rounding).
//
// One warp per (token, head) row.  Latency-bound and tiny: bytes = rows read once, written
// once (q) or twice (k: cache and, if asked for, the rotated copy).
#include "common.cuh"

namespace b200 {

__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

struct GqaRopeParams {
  const __nv_bfloat16* q;
  const __nv_bfloat16* k;
  const __nv_bfloat16* v;
  int64_t q_stride, k_stride, v_stride;        // elements between tokens
  const __nv_bfloat16* cos;
  const __nv_bfloat16* sin;
  int64_t cs_stride;                           // elements between tokens of cos / sin
  const __nv_bfloat16* q_norm_w;               // (128) or null
  const __nv_bfloat16* k_norm_w;
  float eps;
  __nv_bfloat16* q_out;
  int64_t q_out_stride;
  __nv_bfloat16* k_out;                        // (T, Hkv, 128) or null
  __nv_bfloat16* key_cache;
  __nv_bfloat16* value_cache;
  const int32_t* slot_mapping;
  int num_tokens, num_q_heads, num_kv_heads;
  int64_t total_slots;
  int32_t* status;
};

// 128-wide rows: lane l holds dims 4l .. 4l+3; the rotation partner of dim d is d +- 64,
// i.e. the same registers of lane l ^ 16.
__global__ void __launch_bounds__(256)
gqa_rope_cache_kernel(const GqaRopeParams p) {
  grid_dep_launch();              // the attention kernel may set itself up meanwhile (it waits for this grid itself)
  grid_dep_wait();
  const int lane = threadIdx.x & 31;
  const int heads = p.num_q_heads + p.num_kv_heads;
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= (int64_t)p.num_tokens * heads) return;
  const int t = (int)(row / heads);
  const int h = (int)(row % heads);
  const bool is_q = h < p.num_q_heads;
  const int hk = h - p.num_q_heads;
  const __nv_bfloat16* src = is_q ? p.q + (int64_t)t * p.q_stride + (int64_t)h * 128
                                  : p.k + (int64_t)t * p.k_stride + (int64_t)hk * 128;
  const uint2 raw = *reinterpret_cast<const uint2*>(src + lane * 4);
  float x[4];
  {
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    x[0] = __low2float(a); x[1] = __high2float(a); x[2] = __low2float(b); x[3] = __high2float(b);
  }
  const __nv_bfloat16* nw = is_q ? p.q_norm_w : p.k_norm_w;
  if (nw != nullptr) {
    float ss = x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
    const float r = rsqrtf(ss * (1.f / 128.f) + p.eps);
#pragma unroll
    for (int i = 0; i < 4; ++i)
      x[i] = bf16_round(bf16_round(x[i] * r) * __bfloat162float(nw[lane * 4 + i]));
  }
  const __nv_bfloat16* cs = p.cos + (int64_t)t * p.cs_stride + lane * 4;
  const __nv_bfloat16* sn = p.sin + (int64_t)t * p.cs_stride + lane * 4;
  float y[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float other = __shfl_xor_sync(0xffffffffu, x[i], 16);
    const float rot = lane < 16 ? -other : other;              // rotate_half: (-x2, x1)
    y[i] = bf16_round(bf16_round(x[i] * __bfloat162float(cs[i])) + bf16_round(rot * __bfloat162float(sn[i])));
  }
  uint2 packed;
  packed.x = pack_bf16(y[0], y[1]);
  packed.y = pack_bf16(y[2], y[3]);
  if (is_q) {
    *reinterpret_cast<uint2*>(p.q_out + (int64_t)t * p.q_out_stride + (int64_t)h * 128 + lane * 4) = packed;
    return;
  }
  if (p.k_out) *reinterpret_cast<uint2*>(p.k_out + ((int64_t)t * p.num_kv_heads + hk) * 128 + lane * 4) = packed;
  const int64_t slot = p.slot_mapping[t];
  if (slot < 0) return;                                        // padding row
  if (slot >= p.total_slots) {
    if (lane == 0 && p.status) atomicOr(p.status, B200_STATUS_BAD_SLOT);
    return;
  }
  const int64_t dst = (slot * p.num_kv_heads + hk) * 128 + lane * 4;
  *reinterpret_cast<uint2*>(p.key_cache + dst) = packed;
  *reinterpret_cast<uint2*>(p.value_cache + dst) =
      *reinterpret_cast<const uint2*>(p.v + (int64_t)t * p.v_stride + (int64_t)hk * 128 + lane * 4);
}

struct MlaRopeParams {
  const __nv_bfloat16* ckv_full;               // (T, kvl + rope): output of kv_a_proj_with_mqa
  int64_t ckv_stride;
  const __nv_bfloat16* norm_w;                 // (kvl)
  float eps;
  const __nv_bfloat16* q_pe;                   // (T, H, rope) view: token / head strides in elements
  int64_t q_pe_stride_t, q_pe_stride_h;
  __nv_bfloat16* q_pe_out;                     // same shape, own strides
  int64_t q_out_stride_t, q_out_stride_h;
  const __nv_bfloat16* cos;
  const __nv_bfloat16* sin;
  int64_t cs_stride;
  __nv_bfloat16* latent_cache;
  __nv_bfloat16* k_latent_out;                 // (T, kvl + rope) or null
  const int32_t* slot_mapping;
  int num_tokens, num_heads;
  int64_t total_slots;
  int32_t* status;
};

constexpr int kMlaKvl = 512;
constexpr int kMlaRope = 64;

// Rotary part of a 64-wide row held interleaved (pairs (2j, 2j+1)): regrouped into halves
// [x0 x2 .. x62 | x1 x3 .. x63] and rotated NeoX style.  Lane l holds the pair (2l, 2l+1):
// after regrouping, element l of the first half is x[2l], element l of the second half is
// x[2l+1], so the rotation partner lives in the same lane.
__device__ __forceinline__ void rope_interleaved_pair(float even, float odd, float cos_lo, float sin_lo,
                                                      float cos_hi, float sin_hi, float& out_lo, float& out_hi) {
  out_lo = bf16_round(bf16_round(even * cos_lo) + bf16_round(-odd * sin_lo));   // first half: x1*cos - x2*sin
  out_hi = bf16_round(bf16_round(odd * cos_hi) + bf16_round(even * sin_hi));    // second half: x2*cos + x1*sin
}

__global__ void __launch_bounds__(256)
mla_rope_norm_cache_kernel(const MlaRopeParams p) {
  grid_dep_launch();              // the attention kernel may set itself up meanwhile (it waits for this grid itself)
  grid_dep_wait();
  const int lane = threadIdx.x & 31;
  const int rows_per_token = p.num_heads + 1;                  // every head's q_pe, then the latent row
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= (int64_t)p.num_tokens * rows_per_token) return;
  const int t = (int)(row / rows_per_token);
  const int h = (int)(row % rows_per_token);
  const __nv_bfloat16* cs = p.cos + (int64_t)t * p.cs_stride;
  const __nv_bfloat16* sn = p.sin + (int64_t)t * p.cs_stride;
  const float cos_lo = __bfloat162float(cs[lane]), cos_hi = __bfloat162float(cs[lane + 32]);
  const float sin_lo = __bfloat162float(sn[lane]), sin_hi = __bfloat162float(sn[lane + 32]);
  if (h < p.num_heads) {
    const __nv_bfloat16* src = p.q_pe + (int64_t)t * p.q_pe_stride_t + (int64_t)h * p.q_pe_stride_h;
    const __nv_bfloat162 pr = *reinterpret_cast<const __nv_bfloat162*>(src + 2 * lane);
    float lo, hi;
    rope_interleaved_pair(__low2float(pr), __high2float(pr), cos_lo, sin_lo, cos_hi, sin_hi, lo, hi);
    __nv_bfloat16* dst = p.q_pe_out + (int64_t)t * p.q_out_stride_t + (int64_t)h * p.q_out_stride_h;
    dst[lane] = __float2bfloat16_rn(lo);
    dst[lane + 32] = __float2bfloat16_rn(hi);
    return;
  }
  // ---- latent row: RMSNorm of the first 512 columns, rotary on the last 64
  const __nv_bfloat16* src = p.ckv_full + (int64_t)t * p.ckv_stride;
  float x[16];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {                                // 4 x (4 columns) per lane, coalesced 8-byte loads
    const uint2 raw = *reinterpret_cast<const uint2*>(src + i * 128 + lane * 4);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    x[i * 4 + 0] = __low2float(a); x[i * 4 + 1] = __high2float(a);
    x[i * 4 + 2] = __low2float(b); x[i * 4 + 3] = __high2float(b);
#pragma unroll
    for (int j = 0; j < 4; ++j) ss += x[i * 4 + j] * x[i * 4 + j];
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
  const float r = rsqrtf(ss * (1.f / kMlaKvl) + p.eps);
  const __nv_bfloat162 pr = *reinterpret_cast<const __nv_bfloat162*>(src + kMlaKvl + 2 * lane);
  float lo, hi;
  rope_interleaved_pair(__low2float(pr), __high2float(pr), cos_lo, sin_lo, cos_hi, sin_hi, lo, hi);

  const int64_t slot = p.slot_mapping[t];
  __nv_bfloat16* cache_row = nullptr;
  if (slot >= p.total_slots) {
    if (lane == 0 && p.status) atomicOr(p.status, B200_STATUS_BAD_SLOT);
  } else if (slot >= 0) {
    cache_row = p.latent_cache + slot * (kMlaKvl + kMlaRope);
  }
  __nv_bfloat16* copy_row = p.k_latent_out ? p.k_latent_out + (int64_t)t * (kMlaKvl + kMlaRope) : nullptr;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float y[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
      y[j] = bf16_round(bf16_round(x[i * 4 + j] * r) * __bfloat162float(p.norm_w[i * 128 + lane * 4 + j]));
    uint2 packed;
    packed.x = pack_bf16(y[0], y[1]);
    packed.y = pack_bf16(y[2], y[3]);
    if (cache_row) *reinterpret_cast<uint2*>(cache_row + i * 128 + lane * 4) = packed;
    if (copy_row) *reinterpret_cast<uint2*>(copy_row + i * 128 + lane * 4) = packed;
  }
  if (cache_row) {
    cache_row[kMlaKvl + lane] = __float2bfloat16_rn(lo);
    cache_row[kMlaKvl + 32 + lane] = __float2bfloat16_rn(hi);
  }
  if (copy_row) {
    copy_row[kMlaKvl + lane] = __float2bfloat16_rn(lo);
    copy_row[kMlaKvl + 32 + lane] = __float2bfloat16_rn(hi);
  }
}

}  // namespace b200

extern "C" int b200_gqa_rope_cache(const void* q, int64_t q_stride, const void* k, int64_t k_stride,
                                   const void* v, int64_t v_stride, const void* cos, const void* sin,
                                   int64_t cos_sin_stride, const void* q_norm_weight,
                                   const void* k_norm_weight, float eps, void* q_out,
                                   int64_t q_out_stride, void* k_out, void* key_cache,
                                   void* value_cache, const int32_t* slot_mapping, int num_tokens,
                                   int num_q_heads, int num_kv_heads, int head_dim, int block_size,
                                   int num_blocks, int32_t* status, void* stream) {
  using namespace b200;
  if (num_tokens == 0) return B200_OK;
  if (!q || !k || !v || !cos || !sin || !q_out || !key_cache || !value_cache || !slot_mapping ||
      num_tokens < 0 || num_q_heads <= 0 || num_kv_heads <= 0 || block_size <= 0 || num_blocks <= 0 ||
      (q_norm_weight == nullptr) != (k_norm_weight == nullptr)) {
    set_last_error("gqa_rope_cache: null pointer, non-positive size, or only one of the two norm weights");
    return B200_EINVAL;
  }
  if (head_dim != 128) {
    set_last_error("gqa_rope_cache: head_dim %d unsupported (kernel is built for 128)", head_dim);
    return B200_EUNSUPPORTED;
  }
  auto mis = [](const void* ptr) { return reinterpret_cast<uintptr_t>(ptr) % 8 != 0; };
  if (mis(q) || mis(k) || mis(v) || mis(q_out) || mis(key_cache) || mis(value_cache) || (k_out && mis(k_out)) ||
      q_stride % 4 || k_stride % 4 || v_stride % 4 || q_out_stride % 4) {
    set_last_error("gqa_rope_cache: rows must be 8-byte aligned (pointers and token strides)");
    return B200_EALIGN;
  }
  GqaRopeParams p;
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.k = static_cast<const __nv_bfloat16*>(k);
  p.v = static_cast<const __nv_bfloat16*>(v);
  p.q_stride = q_stride; p.k_stride = k_stride; p.v_stride = v_stride;
  p.cos = static_cast<const __nv_bfloat16*>(cos);
  p.sin = static_cast<const __nv_bfloat16*>(sin);
  p.cs_stride = cos_sin_stride;
  p.q_norm_w = static_cast<const __nv_bfloat16*>(q_norm_weight);
  p.k_norm_w = static_cast<const __nv_bfloat16*>(k_norm_weight);
  p.eps = eps;
  p.q_out = static_cast<__nv_bfloat16*>(q_out);
  p.q_out_stride = q_out_stride;
  p.k_out = static_cast<__nv_bfloat16*>(k_out);
  p.key_cache = static_cast<__nv_bfloat16*>(key_cache);
  p.value_cache = static_cast<__nv_bfloat16*>(value_cache);
  p.slot_mapping = slot_mapping;
  p.num_tokens = num_tokens;
  p.num_q_heads = num_q_heads;
  p.num_kv_heads = num_kv_heads;
  p.total_slots = (int64_t)num_blocks * block_size;
  p.status = status;
  const int64_t rows = (int64_t)num_tokens * (num_q_heads + num_kv_heads);
  const int64_t blocks = (rows + 7) / 8;
  return check_cuda(launch_pdl(gqa_rope_cache_kernel, dim3((unsigned)blocks), dim3(256), 0,
                               static_cast<cudaStream_t>(stream), p),
                    "gqa_rope_cache launch");
}

extern "C" int b200_mla_rope_norm_cache(const void* ckv_full, int64_t ckv_stride, const void* norm_weight,
                                        float eps, const void* q_pe, int64_t q_pe_stride_t,
                                        int64_t q_pe_stride_h, void* q_pe_out, int64_t q_out_stride_t,
                                        int64_t q_out_stride_h, const void* cos, const void* sin,
                                        int64_t cos_sin_stride, void* latent_cache, void* k_latent_out,
                                        const int32_t* slot_mapping, int num_tokens, int num_heads,
                                        int kv_lora_rank, int rope_dim, int block_size, int num_blocks,
                                        int32_t* status, void* stream) {
  using namespace b200;
  if (num_tokens == 0) return B200_OK;
  if (!ckv_full || !norm_weight || !q_pe || !q_pe_out || !cos || !sin || !latent_cache || !slot_mapping ||
      num_tokens < 0 || num_heads <= 0 || block_size <= 0 || num_blocks <= 0) {
    set_last_error("mla_rope_norm_cache: null pointer or non-positive size");
    return B200_EINVAL;
  }
  if (kv_lora_rank != kMlaKvl || rope_dim != kMlaRope) {
    set_last_error("mla_rope_norm_cache: latent %d + %d unsupported (kernel is built for 512 + 64)",
                   kv_lora_rank, rope_dim);
    return B200_EUNSUPPORTED;
  }
  auto mis = [](const void* ptr, int a) { return reinterpret_cast<uintptr_t>(ptr) % a != 0; };
  if (mis(ckv_full, 8) || mis(latent_cache, 8) || (k_latent_out && mis(k_latent_out, 8)) || mis(q_pe, 4) ||
      ckv_stride % 4 || q_pe_stride_t % 2 || q_pe_stride_h % 2) {
    set_last_error("mla_rope_norm_cache: latent rows must be 8-byte aligned and q_pe rows 4-byte aligned");
    return B200_EALIGN;
  }
  MlaRopeParams p;
  p.ckv_full = static_cast<const __nv_bfloat16*>(ckv_full);
  p.ckv_stride = ckv_stride;
  p.norm_w = static_cast<const __nv_bfloat16*>(norm_weight);
  p.eps = eps;
  p.q_pe = static_cast<const __nv_bfloat16*>(q_pe);
  p.q_pe_stride_t = q_pe_stride_t;
  p.q_pe_stride_h = q_pe_stride_h;
  p.q_pe_out = static_cast<__nv_bfloat16*>(q_pe_out);
  p.q_out_stride_t = q_out_stride_t;
  p.q_out_stride_h = q_out_stride_h;
  p.cos = static_cast<const __nv_bfloat16*>(cos);
  p.sin = static_cast<const __nv_bfloat16*>(sin);
  p.cs_stride = cos_sin_stride;
  p.latent_cache = static_cast<__nv_bfloat16*>(latent_cache);
  p.k_latent_out = static_cast<__nv_bfloat16*>(k_latent_out);
  p.slot_mapping = slot_mapping;
  p.num_tokens = num_tokens;
  p.num_heads = num_heads;
  p.total_slots = (int64_t)num_blocks * block_size;
  p.status = status;
  const int64_t rows = (int64_t)num_tokens * (num_heads + 1);
  const int64_t blocks = (rows + 7) / 8;
  return check_cuda(launch_pdl(mla_rope_norm_cache_kernel, dim3((unsigned)blocks), dim3(256), 0,
                               static_cast<cudaStream_t>(stream), p),
                    "mla_rope_norm_cache launch");
}
