// Rotary position embedding of fresh query / key rows fused with the key / value cache update.
//
// What the flow-matching loop does between the q/k/v projection and the attention of every layer:
// rotate q and k (apply_rotary_pos_emb, models/pi05/modeling_gemma.py:178-209), bring q into
// [batch, heads, tokens, dim] order, and append the rotated keys and the values behind the cached
// prefix (the reference's fused form: fused_cache_update_rope_bf16,
// blackwell/csrc/fp4_cutlass_linear.cu:478-588).  As a chain of tensor ops this is about fourteen
// launches per layer; here it is one.  The cache buffers are preallocated for prefix + tokens rows
// and already hold the prefix, so only the new rows are written.
//
// Arithmetic (identical to bf16 tensor ops and to the reference's rope_element,
// fp4_cutlass_linear.cu:96-126): out = bf16( bf16(x * cos) + bf16(r * sin) ), r = -x[j + d/2] for
// j < d/2 and x[j - d/2] otherwise; three roundings to bf16, fp32 in between.
//
// One warp per (row, head): lane l handles the eight elements [8 l, 8 l + 8) of the head and of its
// rotation partner (16-byte loads and stores); head_dim is a multiple of 16, at most 512.

#include <cuda_bf16.h>

#include "rk_common.cuh"
#include "rk_host.h"

namespace rk {
namespace {

__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }
__device__ __forceinline__ float round_bf16(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  const uint32_t l = __bfloat16_as_ushort(__float2bfloat16_rn(lo));
  const uint32_t h = __bfloat16_as_ushort(__float2bfloat16_rn(hi));
  return l | (h << 16);
}

// eight rotated elements: x and partner are the raw words, `negate` says whether the partner enters negated
__device__ __forceinline__ uint4 rotate8(const uint4& x, const uint4& partner, const uint4& c, const uint4& s, bool negate) {
  const uint32_t xw[4] = {x.x, x.y, x.z, x.w}, pw[4] = {partner.x, partner.y, partner.z, partner.w};
  const uint32_t cw[4] = {c.x, c.y, c.z, c.w}, sw[4] = {s.x, s.y, s.z, s.w};
  uint32_t o[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float sign = negate ? -1.0f : 1.0f;
    const float a0 = round_bf16(__fmul_rn(bf16_lo(xw[i]), bf16_lo(cw[i])));
    const float a1 = round_bf16(__fmul_rn(bf16_hi(xw[i]), bf16_hi(cw[i])));
    const float b0 = round_bf16(__fmul_rn(sign * bf16_lo(pw[i]), bf16_lo(sw[i])));
    const float b1 = round_bf16(__fmul_rn(sign * bf16_hi(pw[i]), bf16_hi(sw[i])));
    o[i] = pack2(__fadd_rn(a0, b0), __fadd_rn(a1, b1));
  }
  return make_uint4(o[0], o[1], o[2], o[3]);
}

struct RopeParams {
  const __nv_bfloat16 *q, *k, *v;        // rows of [heads * dim], [kv_heads * dim], [kv_heads * dim]
  long long q_stride, k_stride, v_stride;  // row strides in elements
  const __nv_bfloat16 *cos, *sin;        // [batch, tokens, dim]
  __nv_bfloat16 *q_out;                  // [batch, heads, tokens, dim], or [batch, tokens, heads, dim] (token_major)
  __nv_bfloat16 *k_all, *v_all;          // [batch, kv_heads, cache_rows, dim]
  __nv_bfloat16 *vt_all;                 // optional transposed values [batch, kv_heads, dim, vt_pitch]
  long long vt_pitch;
  int batch, tokens, heads, kv_heads, dim, cache_rows, prefix, token_major;
};

__global__ void __launch_bounds__(256)
rope_cache_update_kernel(const RopeParams p) {
  pdl_launch_dependents();  // every thread, before any return: see launch_pdl
  pdl_wait();
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const int units = p.heads + 2 * p.kv_heads;  // per row: query heads, key heads, value heads
  const long long job = static_cast<long long>(blockIdx.x) * warps_per_block + (threadIdx.x >> 5);
  const long long jobs = static_cast<long long>(p.batch) * p.tokens * units;
  if (job >= jobs) return;
  const int unit = static_cast<int>(job % units);
  const long long row = job / units;  // batch * tokens + token
  const int token = static_cast<int>(row % p.tokens);
  const int b = static_cast<int>(row / p.tokens);
  const int half = p.dim >> 1;
  const __nv_bfloat16* cs = p.cos + row * p.dim;
  const __nv_bfloat16* sn = p.sin + row * p.dim;
  for (int j = lane * 8; j < p.dim; j += 256) {
    if (unit < p.heads + p.kv_heads) {
      const bool is_q = unit < p.heads;
      const int head = is_q ? unit : unit - p.heads;
      const __nv_bfloat16* src = (is_q ? p.q + row * p.q_stride : p.k + row * p.k_stride) + head * p.dim;
      const int jp = j < half ? j + half : j - half;
      const uint4 x = *reinterpret_cast<const uint4*>(src + j);
      const uint4 partner = *reinterpret_cast<const uint4*>(src + jp);
      const uint4 c = *reinterpret_cast<const uint4*>(cs + j);
      const uint4 s = *reinterpret_cast<const uint4*>(sn + j);
      const uint4 o = rotate8(x, partner, c, s, j < half);
      __nv_bfloat16* dst =
          is_q ? p.q_out + (p.token_major ? (row * p.heads + head) * p.dim
                                          : ((static_cast<long long>(b) * p.heads + head) * p.tokens + token) * p.dim)
               : p.k_all + ((static_cast<long long>(b) * p.kv_heads + head) * p.cache_rows + p.prefix + token) * p.dim;
      *reinterpret_cast<uint4*>(dst + j) = o;
    } else {
      const int head = unit - p.heads - p.kv_heads;
      const __nv_bfloat16* src = p.v + row * p.v_stride + head * p.dim;
      __nv_bfloat16* dst = p.v_all + ((static_cast<long long>(b) * p.kv_heads + head) * p.cache_rows + p.prefix + token) * p.dim;
      const uint4 x = *reinterpret_cast<const uint4*>(src + j);
      *reinterpret_cast<uint4*>(dst + j) = x;
      if (p.vt_all != nullptr) {
        // the same eight values into column (prefix + token) of the transposed cache
        unsigned short* const col = reinterpret_cast<unsigned short*>(p.vt_all) +
                                    (static_cast<long long>(b) * p.kv_heads + head) * p.dim * p.vt_pitch + p.prefix + token;
        const uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          col[(j + 2 * e) * p.vt_pitch] = static_cast<unsigned short>(w[e] & 0xFFFFu);
          col[(j + 2 * e + 1) * p.vt_pitch] = static_cast<unsigned short>(w[e] >> 16);
        }
      }
    }
  }
}

}  // namespace
}  // namespace rk

static int rope_cache_update_impl(const void* q, int64_t q_stride, const void* k, int64_t k_stride, const void* v,
                                  int64_t v_stride, const void* cos, const void* sin, int64_t batch, int64_t tokens,
                                  int64_t heads, int64_t kv_heads, int64_t head_dim, void* q_out, int q_token_major,
                                  void* k_cache, void* v_cache, int64_t cache_rows, int64_t prefix, void* vt_cache,
                                  int64_t vt_pitch, void* stream, const char* who) {
  using namespace rk;
  if (vt_cache != nullptr && (vt_pitch < prefix + tokens || (reinterpret_cast<uintptr_t>(vt_cache) & 1u)))
    return fail(RK_EINVAL, "%s: the transposed value cache needs a pitch of at least prefix + tokens", who);
  if (!q || !k || !v || !cos || !sin || !q_out || !k_cache || !v_cache) return fail(RK_EINVAL, "%s: null pointer", who);
  if (batch < 1 || tokens < 1 || heads < 1 || kv_heads < 1) return fail(RK_EINVAL, "%s: empty problem", who);
  if (head_dim < 16 || head_dim % 16 != 0 || head_dim > 512)
    return fail(RK_EINVAL, "%s: head_dim must be a multiple of 16 up to 512", who);
  if (prefix < 0 || prefix + tokens > cache_rows) return fail(RK_EINVAL, "%s: the cache holds %lld rows, %lld + %lld needed", who,
                                                           static_cast<long long>(cache_rows), static_cast<long long>(prefix),
                                                           static_cast<long long>(tokens));
  if (q_stride % 8 || k_stride % 8 || v_stride % 8 || q_stride < heads * head_dim || k_stride < kv_heads * head_dim ||
      v_stride < kv_heads * head_dim)
    return fail(RK_EINVAL, "%s: row strides must cover a row and be multiples of 8 elements", who);
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(cos) || !aligned16(sin) || !aligned16(q_out) ||
      !aligned16(k_cache) || !aligned16(v_cache))
    return fail(RK_EINVAL, "%s: pointers must be 16-byte aligned", who);
  if (batch * tokens * (heads + 2 * kv_heads) > (1ll << 31)) return fail(RK_EUNSUPPORTED, "%s: problem too large", who);
  RopeParams p{};
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.k = static_cast<const __nv_bfloat16*>(k);
  p.v = static_cast<const __nv_bfloat16*>(v);
  p.q_stride = q_stride;
  p.k_stride = k_stride;
  p.v_stride = v_stride;
  p.cos = static_cast<const __nv_bfloat16*>(cos);
  p.sin = static_cast<const __nv_bfloat16*>(sin);
  p.q_out = static_cast<__nv_bfloat16*>(q_out);
  p.k_all = static_cast<__nv_bfloat16*>(k_cache);
  p.v_all = static_cast<__nv_bfloat16*>(v_cache);
  p.vt_all = static_cast<__nv_bfloat16*>(vt_cache);
  p.vt_pitch = vt_pitch;
  p.batch = static_cast<int>(batch);
  p.tokens = static_cast<int>(tokens);
  p.heads = static_cast<int>(heads);
  p.kv_heads = static_cast<int>(kv_heads);
  p.dim = static_cast<int>(head_dim);
  p.cache_rows = static_cast<int>(cache_rows);
  p.prefix = static_cast<int>(prefix);
  p.token_major = q_token_major ? 1 : 0;
  const long long jobs = batch * tokens * (heads + 2 * kv_heads);
  const int warps = 8;
  const unsigned blocks = static_cast<unsigned>((jobs + warps - 1) / warps);
  launch_pdl(rope_cache_update_kernel, blocks, warps * 32, as_stream(stream), p);
  return check_launch(who);
}


extern "C" int rk_rope_cache_update(const void* q, int64_t q_stride, const void* k, int64_t k_stride, const void* v,
                                    int64_t v_stride, const void* cos, const void* sin, int64_t batch, int64_t tokens,
                                    int64_t heads, int64_t kv_heads, int64_t head_dim, void* q_out, int q_token_major,
                                    void* k_cache, void* v_cache, int64_t cache_rows, int64_t prefix, void* stream) {
  return rope_cache_update_impl(q, q_stride, k, k_stride, v, v_stride, cos, sin, batch, tokens, heads, kv_heads, head_dim,
                                q_out, q_token_major, k_cache, v_cache, cache_rows, prefix, nullptr, 0, stream,
                                "rk_rope_cache_update");
}

extern "C" int rk_rope_cache_update_vt(const void* q, int64_t q_stride, const void* k, int64_t k_stride, const void* v,
                                       int64_t v_stride, const void* cos, const void* sin, int64_t batch, int64_t tokens,
                                       int64_t heads, int64_t kv_heads, int64_t head_dim, void* q_out, int q_token_major,
                                       void* k_cache, void* v_cache, int64_t cache_rows, int64_t prefix, void* vt_cache,
                                       int64_t vt_pitch, void* stream) {
  if (!vt_cache) return rk::fail(RK_EINVAL, "rk_rope_cache_update_vt: null transposed cache");
  return rope_cache_update_impl(q, q_stride, k, k_stride, v, v_stride, cos, sin, batch, tokens, heads, kv_heads, head_dim,
                                q_out, q_token_major, k_cache, v_cache, cache_rows, prefix, vt_cache, vt_pitch, stream,
                                "rk_rope_cache_update_vt");
}
