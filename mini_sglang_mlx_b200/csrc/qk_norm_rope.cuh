// The step in front of the attention op, fused: per-head RMSNorm of q and k, rotary
// position embedding of both, and the scatter of the new K/V rows into the paged pool.
//
// In the reference these are separate array ops around the kernel boundary
// (mini_sglang_mlx/models/qwen3.py:58-68: q_norm, k_norm, rope on q and on k, then
// AttnBackend.forward stores K/V with store_kv_cache before attention), i.e. q and k make
// three HBM round trips and k a fourth for the store.  Here every row is read once and
// written once: q in place, k straight into k_cache[out_loc], v into v_cache[out_loc].
//
// Arithmetic follows the reference's building blocks: RMSNorm y = x * rsqrt(mean(x^2) + eps) * w
// in fp32, rounded to the 16-bit type (the reference materialises that array); RoPE in the
// non-interleaved layout (pairs (i, i + rd/2), angle = position * base^(-2i/rd)) in fp32,
// rounded once more.  head_dim 128, rotary_dim 64 or 128.
//
// One CTA of four warps per token, the warps independent of one another (no shared memory,
// no CTA barrier): each takes four (token, head) rows at a time with the next four already
// in flight (the kernel is bound by HBM and needs the bytes in flight), and computes the two
// rotary angles its lanes need itself.  Lane l holds elements 2l, 2l+1 and 64+2l, 65+2l of a
// row: 128-byte warp accesses, and for rotary_dim 128 both members of a rotary pair sit in
// the same lane (for rotary_dim 64 the partner is lane l ^ 16).
#pragma once

#include "common.cuh"

namespace msgl {

struct QkNormRopeParams {
  void* q;                 // (n, hq, 128), normalised and rotated in place
  const void* k;           // (n, hkv, 128)
  const void* v;           // (n, hkv, 128)
  const void* q_weight;    // (128) or null: no q norm
  const void* k_weight;    // (128) or null: no k norm
  const int32_t* positions;
  const int32_t* out_loc;  // slot of each token's K/V row
  void* k_cache;
  void* v_cache;
  int n, hq, hkv, rotary_dim;
  int64_t q_stride, k_stride, v_stride;  // elements between consecutive tokens
  int64_t cache_stride;                  // elements between consecutive slots
  int64_t num_slots;
  float log2_base, eps;
};

template <typename T>
__device__ __forceinline__ float to_f32(T x);
template <>
__device__ __forceinline__ float to_f32(__nv_bfloat16 x) { return __bfloat162float(x); }
template <>
__device__ __forceinline__ float to_f32(__half x) { return __half2float(x); }

// sin and cos of an angle of up to ~2*10^5 rad: the multiple of 2*pi is taken off with a
// two-constant fused multiply-add (exact to about 3e-7 rad at that size), the rest goes to
// the hardware approximations, whose absolute error on [-pi, pi] is about 5e-7 -- three
// orders below the 16-bit rounding of the result.
__device__ __forceinline__ void sincos_reduced(float x, float& s, float& c) {
  const float k = rintf(x * 0.15915494309189535f);
  float r = fmaf(-k, 6.2831854820251465f, x);
  r = fmaf(-k, -1.7484556000744883e-7f, r);
  __sincosf(r, &s, &c);
}

template <typename T>
struct Pair16;
template <>
struct Pair16<__nv_bfloat16> {
  using type = __nv_bfloat162;
  __device__ __forceinline__ static float2 unpack(type v) { return __bfloat1622float2(v); }
  __device__ __forceinline__ static type pack(float a, float b) { return __floats2bfloat162_rn(a, b); }
};
template <>
struct Pair16<__half> {
  using type = __half2;
  __device__ __forceinline__ static float2 unpack(type v) { return __half22float2(v); }
  __device__ __forceinline__ static type pack(float a, float b) { return __floats2half2_rn(a, b); }
};

template <typename T>
__global__ void __launch_bounds__(128) qk_norm_rope_store_kernel(const QkNormRopeParams p) {
  constexpr int HD = 128;
  constexpr int RU = 4;  // rows a warp has in flight
  using P2 = typename Pair16<T>::type;
  const int tok = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int half = p.rotary_dim >> 1;
  const int n_qk = p.hq + p.hkv, rows = n_qk + p.hkv;
  auto row_ptr = [&](int row) -> const T* {
    if (row < p.hq) return static_cast<const T*>(p.q) + tok * p.q_stride + row * HD;
    if (row < n_qk) return static_cast<const T*>(p.k) + tok * p.k_stride + (row - p.hq) * HD;
    return static_cast<const T*>(p.v) + tok * p.v_stride + (row - n_qk) * HD;
  };
  auto load_rows = [&](int row0, P2 (&lo)[RU], P2 (&hi)[RU]) {
#pragma unroll
    for (int u = 0; u < RU; ++u) {
      if (row0 + u < rows) {
        const P2* src = reinterpret_cast<const P2*>(row_ptr(row0 + u));
        lo[u] = src[lane];
        hi[u] = src[32 + lane];
      }
    }
  };
  // the first rows are on their way while the token's angles are worked out
  P2 lo[RU], hi[RU];
  load_rows(warp * RU, lo, hi);
  const int slot = p.out_loc[tok];
  const bool slot_ok = slot >= 0 && slot < p.num_slots;
  // this lane's two rotary frequencies: pairs (2l, 2l+1) of the first half for rotary_dim 128,
  // (2(l & 15), +1) for rotary_dim 64.  angle = position * base^(-2i/rd): the product is taken
  // in fp32 as the reference does.
  const int f0 = half == 64 ? 2 * lane : 2 * (lane & 15);
  const float posf = static_cast<float>(p.positions[tok]);
  const float inv_rd = 1.f / static_cast<float>(p.rotary_dim);
  float c0, s0, c1, s1;
  sincos_reduced(posf * exp2f(-p.log2_base * (static_cast<float>(2 * f0) * inv_rd)), s0, c0);
  sincos_reduced(posf * exp2f(-p.log2_base * (static_cast<float>(2 * f0 + 2) * inv_rd)), s1, c1);
  float w_lo[2][2], w_hi[2][2];  // [q or k][element of the pair]
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const T* w = static_cast<const T*>(t == 0 ? p.q_weight : p.k_weight);
    if (w) {
      const float2 a = Pair16<T>::unpack(reinterpret_cast<const P2*>(w)[lane]);
      const float2 b = Pair16<T>::unpack(reinterpret_cast<const P2*>(w)[32 + lane]);
      w_lo[t][0] = a.x; w_lo[t][1] = a.y; w_hi[t][0] = b.x; w_hi[t][1] = b.y;
    } else {
      w_lo[t][0] = w_lo[t][1] = w_hi[t][0] = w_hi[t][1] = 0.f;
    }
  }

  for (int row0 = warp * RU; row0 < rows; row0 += nwarps * RU) {
    P2 nlo[RU], nhi[RU];   // the next four rows, in flight while these are processed
    load_rows(row0 + nwarps * RU, nlo, nhi);
#pragma unroll
    for (int u = 0; u < RU; ++u) {
      const int row = row0 + u;
      if (row >= rows) break;
      if (row >= n_qk) {
        // ---- V row: copy into the pool
        if (slot_ok) {
          T* dst = static_cast<T*>(p.v_cache) + slot * p.cache_stride + (row - n_qk) * HD;
          reinterpret_cast<P2*>(dst)[lane] = lo[u];
          reinterpret_cast<P2*>(dst)[32 + lane] = hi[u];
        }
        continue;
      }
      const bool is_q = row < p.hq;
      if (!is_q && !slot_ok) continue;
      T* dst = is_q ? static_cast<T*>(p.q) + tok * p.q_stride + row * HD
                    : static_cast<T*>(p.k_cache) + slot * p.cache_stride + (row - p.hq) * HD;
      const int wi = is_q ? 0 : 1;
      float2 a = Pair16<T>::unpack(lo[u]), b = Pair16<T>::unpack(hi[u]);
      if ((is_q ? p.q_weight : p.k_weight) != nullptr) {
        float ss = a.x * a.x + a.y * a.y + b.x * b.x + b.y * b.y;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        const float inv = rsqrtf(ss * (1.f / HD) + p.eps);
        // rounded as the reference's materialised norm output is
        a = Pair16<T>::unpack(Pair16<T>::pack(a.x * inv * w_lo[wi][0], a.y * inv * w_lo[wi][1]));
        b = Pair16<T>::unpack(Pair16<T>::pack(b.x * inv * w_hi[wi][0], b.y * inv * w_hi[wi][1]));
      }
      if (half == 64) {
        // pairs (2l, 64+2l) and (2l+1, 65+2l), both in this lane
        const float ax = a.x * c0 - b.x * s0, bx = a.x * s0 + b.x * c0;
        const float ay = a.y * c1 - b.y * s1, by = a.y * s1 + b.y * c1;
        a = make_float2(ax, ay);
        b = make_float2(bx, by);
      } else {
        // rotary_dim 64: pairs (i, i+32) inside the first 64 elements; lanes 0-15 hold the
        // first members, lanes 16-31 the second; the upper 64 elements pass through
        const float ox = __shfl_xor_sync(0xffffffffu, a.x, 16);
        const float oy = __shfl_xor_sync(0xffffffffu, a.y, 16);
        if (lane < 16) a = make_float2(a.x * c0 - ox * s0, a.y * c1 - oy * s1);
        else a = make_float2(ox * s0 + a.x * c0, oy * s1 + a.y * c1);
      }
      reinterpret_cast<P2*>(dst)[lane] = Pair16<T>::pack(a.x, a.y);
      reinterpret_cast<P2*>(dst)[32 + lane] = Pair16<T>::pack(b.x, b.y);
    }
#pragma unroll
    for (int u = 0; u < RU; ++u) {
      lo[u] = nlo[u];
      hi[u] = nhi[u];
    }
  }
}

}  // namespace msgl
