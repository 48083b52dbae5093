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
// One CTA per token, its warps independent of one another (no shared memory, no CTA
// barrier).  A half-warp owns a row: lane hl of it holds elements 4hl..4hl+3 and
// 64+4hl..64+4hl+3 (8-byte accesses, 128 bytes per half-warp), so for rotary_dim 128 both
// members of a rotary pair sit in the same lane (for rotary_dim 64 the partner is lane ^ 8).
// A warp has eight rows in flight and the next eight prefetched (the kernel is bound by HBM
// and needs the bytes in flight), and computes the four rotary angles its lanes need itself.
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
  __device__ __forceinline__ static float2 from_bits(uint32_t v) {
    return make_float2(__uint_as_float(v << 16), __uint_as_float(v & 0xffff0000u));
  }
  __device__ __forceinline__ static type pack(float a, float b) { return __floats2bfloat162_rn(a, b); }
};
template <>
struct Pair16<__half> {
  using type = __half2;
  __device__ __forceinline__ static float2 unpack(type v) { return __half22float2(v); }
  __device__ __forceinline__ static float2 from_bits(uint32_t v) {
    return make_float2(__half2float(__ushort_as_half(static_cast<unsigned short>(v & 0xffffu))),
                       __half2float(__ushort_as_half(static_cast<unsigned short>(v >> 16))));
  }
  __device__ __forceinline__ static type pack(float a, float b) { return __floats2half2_rn(a, b); }
};

template <typename T>
__global__ void __launch_bounds__(256) qk_norm_rope_store_kernel(const QkNormRopeParams p) {
  constexpr int HD = 128;
  constexpr int RU = 4;  // row pairs a warp has in flight (a half-warp per row)
  using P2 = typename Pair16<T>::type;
  const int tok = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int hl = lane & 15, side = lane >> 4;   // position inside the half-warp, which row of the pair
  const int half = p.rotary_dim >> 1;
  const int n_qk = p.hq + p.hkv, rows = n_qk + p.hkv;
  auto row_ptr = [&](int row) -> const T* {
    if (row < p.hq) return static_cast<const T*>(p.q) + tok * p.q_stride + row * HD;
    if (row < n_qk) return static_cast<const T*>(p.k) + tok * p.k_stride + (row - p.hq) * HD;
    return static_cast<const T*>(p.v) + tok * p.v_stride + (row - n_qk) * HD;
  };
  // lane (side, hl) holds elements 4hl..4hl+3 and 64+4hl..64+4hl+3 of row (first + 2u + side)
  auto load_rows = [&](int first, uint2 (&lo)[RU], uint2 (&hi)[RU]) {
#pragma unroll
    for (int u = 0; u < RU; ++u) {
      const int row = first + 2 * u + side;
      if (row < rows) {
        const uint2* src = reinterpret_cast<const uint2*>(row_ptr(row));
        lo[u] = src[hl];
        hi[u] = src[16 + hl];
      }
    }
  };
  // the first rows are on their way while the token's angles are worked out
  uint2 lo[RU], hi[RU];
  load_rows(warp * 2 * RU, lo, hi);
  const int slot = p.out_loc[tok];
  const bool slot_ok = slot >= 0 && slot < p.num_slots;
  // this lane's four rotary frequencies: pair index i = 4hl + e of the first half for
  // rotary_dim 128, 4(hl & 7) + e for rotary_dim 64.  angle = position * base^(-2i/rd): the
  // product is taken in fp32 as the reference does.
  const int f0 = half == 64 ? 4 * hl : 4 * (hl & 7);
  const float posf = static_cast<float>(p.positions[tok]);
  const float inv_rd = 1.f / static_cast<float>(p.rotary_dim);
  float cs[4], sn[4];
#pragma unroll
  for (int e = 0; e < 4; ++e)
    sincos_reduced(posf * exp2f(-p.log2_base * (static_cast<float>(2 * (f0 + e)) * inv_rd)), sn[e], cs[e]);
  // norm weights and rotation factors as packed pairs of floats: elements (0,1) and (2,3) of
  // the lane's low and high quadruple
  uint64_t wq[4], wk[4];   // [lo01, lo23, hi01, hi23]
  {
    const T* w = static_cast<const T*>(p.q_weight);
    const T* x = static_cast<const T*>(p.k_weight);
#pragma unroll
    for (int h2 = 0; h2 < 4; ++h2) {
      const int e0 = (h2 >> 1) * 64 + 4 * hl + (h2 & 1) * 2;
      wq[h2] = w ? pack_f32x2(to_f32(w[e0]), to_f32(w[e0 + 1])) : 0ull;
      wk[h2] = x ? pack_f32x2(to_f32(x[e0]), to_f32(x[e0 + 1])) : 0ull;
    }
  }
  const uint64_t cs01 = pack_f32x2(cs[0], cs[1]), cs23 = pack_f32x2(cs[2], cs[3]);
  const uint64_t sn01 = pack_f32x2(sn[0], sn[1]), sn23 = pack_f32x2(sn[2], sn[3]);
  const uint64_t ng01 = pack_f32x2(-sn[0], -sn[1]), ng23 = pack_f32x2(-sn[2], -sn[3]);
  auto from_bits2 = [](uint32_t v) -> uint64_t {
    const float2 f = Pair16<T>::from_bits(v);
    return pack_f32x2(f.x, f.y);
  };
  auto to_bits2 = [](uint64_t v) -> uint32_t {
    float x, y;
    unpack_f32x2(v, x, y);
    return MmaOp<T>::pack(x, y);
  };

  for (int first = warp * 2 * RU; first < rows; first += nwarps * 2 * RU) {
    uint2 nlo[RU], nhi[RU];   // the next rows, in flight while these are processed
    load_rows(first + nwarps * 2 * RU, nlo, nhi);
#pragma unroll
    for (int u = 0; u < RU; ++u) {
      const int row = first + 2 * u + side;
      const bool live = row < rows;
      if (first + 2 * u >= n_qk) {
        // ---- both rows of the pair are V rows (or past the end): copy into the pool
        if (live && slot_ok) {
          T* dst = static_cast<T*>(p.v_cache) + slot * p.cache_stride + (row - n_qk) * HD;
          reinterpret_cast<uint2*>(dst)[hl] = lo[u];
          reinterpret_cast<uint2*>(dst)[16 + hl] = hi[u];
        }
        continue;
      }
      // the two half-warps may still hold rows of different kinds (last q row / first k row,
      // last k row / first v row): every decision below is per half-warp, the shuffles stay
      // inside it
      const bool is_v = live && row >= n_qk;
      const bool is_q = live && row < p.hq;
      const bool has_w = live && !is_v && (is_q ? p.q_weight : p.k_weight) != nullptr;
      uint64_t a01 = from_bits2(live ? lo[u].x : 0u), a23 = from_bits2(live ? lo[u].y : 0u);
      uint64_t b01 = from_bits2(live ? hi[u].x : 0u), b23 = from_bits2(live ? hi[u].y : 0u);
      float ss;
      {
        uint64_t acc = mul_f32x2(a01, a01);
        acc = fma_f32x2(a23, a23, acc);
        acc = fma_f32x2(b01, b01, acc);
        acc = fma_f32x2(b23, b23, acc);
        float s0, s1;
        unpack_f32x2(acc, s0, s1);
        ss = s0 + s1;
      }
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      if (has_w) {
        const float inv = rsqrtf(ss * (1.f / HD) + p.eps);
        const uint64_t inv2 = pack_f32x2(inv, inv);
        // (x * inv) * w, rounded to the 16-bit type as the reference's materialised norm output is
        a01 = from_bits2(to_bits2(mul_f32x2(mul_f32x2(a01, inv2), is_q ? wq[0] : wk[0])));
        a23 = from_bits2(to_bits2(mul_f32x2(mul_f32x2(a23, inv2), is_q ? wq[1] : wk[1])));
        b01 = from_bits2(to_bits2(mul_f32x2(mul_f32x2(b01, inv2), is_q ? wq[2] : wk[2])));
        b23 = from_bits2(to_bits2(mul_f32x2(mul_f32x2(b23, inv2), is_q ? wq[3] : wk[3])));
      }
      if (half == 64) {
        if (!is_v) {
          // pairs (4hl+e, 64+4hl+e), both in this lane: a' = a cos - b sin, b' = a sin + b cos
          const uint64_t x01 = a01, x23 = a23;
          a01 = fma_f32x2(b01, ng01, mul_f32x2(x01, cs01));
          a23 = fma_f32x2(b23, ng23, mul_f32x2(x23, cs23));
          b01 = fma_f32x2(b01, cs01, mul_f32x2(x01, sn01));
          b23 = fma_f32x2(b23, cs23, mul_f32x2(x23, sn23));
        }
      } else {
        // rotary_dim 64: pairs (i, i+32) inside the first 64 elements; lanes hl < 8 hold the
        // first members, hl >= 8 the second (partner lane ^ 8); the upper 64 pass through
        float a[4], other[4];
        unpack_f32x2(a01, a[0], a[1]);
        unpack_f32x2(a23, a[2], a[3]);
#pragma unroll
        for (int e = 0; e < 4; ++e) other[e] = __shfl_xor_sync(0xffffffffu, a[e], 8);
        if (!is_v) {
#pragma unroll
          for (int e = 0; e < 4; ++e)
            a[e] = hl < 8 ? a[e] * cs[e] - other[e] * sn[e] : other[e] * sn[e] + a[e] * cs[e];
        }
        a01 = pack_f32x2(a[0], a[1]);
        a23 = pack_f32x2(a[2], a[3]);
      }
      if (!live) continue;
      T* dst;
      if (is_q) {
        dst = static_cast<T*>(p.q) + tok * p.q_stride + row * HD;
      } else {
        if (!slot_ok) continue;
        dst = is_v ? static_cast<T*>(p.v_cache) + slot * p.cache_stride + (row - n_qk) * HD
                   : static_cast<T*>(p.k_cache) + slot * p.cache_stride + (row - p.hq) * HD;
      }
      reinterpret_cast<uint2*>(dst)[hl] = is_v ? lo[u] : make_uint2(to_bits2(a01), to_bits2(a23));
      reinterpret_cast<uint2*>(dst)[16 + hl] = is_v ? hi[u] : make_uint2(to_bits2(b01), to_bits2(b23));
    }
#pragma unroll
    for (int u = 0; u < RU; ++u) {
      lo[u] = nlo[u];
      hi[u] = nhi[u];
    }
  }
}

}  // namespace msgl
