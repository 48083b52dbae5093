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
// rounded once more.  head_dim 128 or 256; rotary_dim = head_dim, head_dim/2 or head_dim/4
// (the reference's Qwen3 layers rotate the whole head, its Qwen3.5 layers a quarter of it).
//
// Work items are (token, head) rows, a half-warp each, in a grid-stride loop.  Lane hl of the
// half-warp holds E = head_dim/32 consecutive elements of the lower half of the row and the
// E elements half a row further on (8- or 16-byte accesses), so with rotary_dim == head_dim
// both members of a rotary pair sit in the same lane (with a smaller rotary_dim the partner
// is a lane of the same half-warp).  The rotary frequencies of a lane are constants; the
// angles are recomputed per row from the token's position (cheaper than keeping a token's
// rows together: what this kernel needs is many independent rows in flight).
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

template <int BYTES>
struct RowVec;
template <>
struct RowVec<8> { using type = uint2; };
template <>
struct RowVec<16> { using type = uint4; };

// heads per work item: sixteen bytes of row data in flight per lane and head either way
__host__ __device__ constexpr int qk_rows_per_item(int head_dim) { return head_dim == 256 ? 2 : 4; }

template <typename T, int HD>
__global__ void __launch_bounds__(256) qk_norm_rope_store_kernel(const QkNormRopeParams p) {
  static_assert(HD == 128 || HD == 256, "head_dim 128 or 256");
  constexpr int E = HD / 32;             // elements of a lane in each half of the row
  constexpr int W = E / 2;               // 32-bit words (16-bit pairs) of those
  constexpr int R = qk_rows_per_item(HD);
  using Vec = typename RowVec<E * 2>::type;
  const int lane = threadIdx.x & 31;
  const int hl = lane & 15;                                   // position inside the half-warp
  const uint32_t hmask = (lane & 16) ? 0xffff0000u : 0x0000ffffu;   // the half-warps run apart
  const int half = p.rotary_dim >> 1;
  // Rotary pairs are (i, i + half).  With rotary_dim == head_dim the partner of a lane's lower
  // element is its own upper element.  With a smaller rotary_dim the pairs lie inside the
  // lower half of the row: lanes below xm hold first members, the partner is lane ^ xm, and
  // lanes from 2*xm on (and the whole upper half) pass through.
  const bool in_lane = p.rotary_dim == HD;
  const int xm = in_lane ? 0 : half / E;
  const bool rot_lane = in_lane || hl < 2 * xm;
  const int f0 = in_lane ? E * hl : E * (hl & (xm - 1));
  // this lane's rotary frequencies base^(-2i/rd): the same for every token
  float freq[E];
  {
    const float inv_rd = 1.f / static_cast<float>(p.rotary_dim);
#pragma unroll
    for (int e = 0; e < E; ++e) freq[e] = exp2f(-p.log2_base * (static_cast<float>(2 * (f0 + e)) * inv_rd));
  }
  auto word = [](const Vec& v, int i) -> uint32_t { return reinterpret_cast<const uint32_t*>(&v)[i]; };
  auto from_bits2 = [](uint32_t v) -> uint64_t {
    const float2 f = Pair16<T>::from_bits(v);
    return pack_f32x2(f.x, f.y);
  };
  auto to_bits2 = [](uint64_t v) -> uint32_t {
    float x, y;
    unpack_f32x2(v, x, y);
    return MmaOp<T>::pack(x, y);
  };

  // A work item is up to R consecutive heads of one token and one kind (q, k or v), handled by
  // a half-warp; items are taken in a grid-stride loop.  The kernel has to retire a row every
  // ~24 cycles per SM to keep up with HBM, i.e. it is bound by instruction issue as much as by
  // latency: the angles, the norm weights and the index arithmetic are per item, not per row,
  // and V items are plain copies.
  const uint32_t gq = (p.hq + R - 1) / R, gk = (p.hkv + R - 1) / R;
  const uint32_t groups = gq + 2 * gk;
  const uint32_t total = static_cast<uint32_t>(p.n) * groups;
  const uint32_t stride = gridDim.x * (blockDim.x >> 4);
  for (uint32_t item = (blockIdx.x * blockDim.x + threadIdx.x) >> 4; item < total; item += stride) {
    const uint32_t tok = item / groups;
    const uint32_t g = item - tok * groups;
    const bool is_q = g < gq, is_v = g >= gq + gk;
    const int h0 = static_cast<int>(is_q ? g : is_v ? g - gq - gk : g - gq) * R;   // first head
    const int cnt = min(R, (is_q ? p.hq : p.hkv) - h0);
    const T* src = is_q   ? static_cast<const T*>(p.q) + tok * p.q_stride
                   : is_v ? static_cast<const T*>(p.v) + tok * p.v_stride
                          : static_cast<const T*>(p.k) + tok * p.k_stride;
    src += h0 * HD;
    Vec lo[R], hi[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      if (r < cnt) {
        lo[r] = reinterpret_cast<const Vec*>(src + r * HD)[hl];
        hi[r] = reinterpret_cast<const Vec*>(src + r * HD)[16 + hl];
      }
    }
    T* dst;
    if (is_q) {
      dst = static_cast<T*>(p.q) + tok * p.q_stride + h0 * HD;
    } else {
      const int slot = p.out_loc[tok];
      if (slot < 0 || slot >= p.num_slots) continue;
      dst = static_cast<T*>(is_v ? p.v_cache : p.k_cache) + slot * p.cache_stride + h0 * HD;
    }
    if (is_v) {
#pragma unroll
      for (int r = 0; r < R; ++r) {
        if (r < cnt) {
          reinterpret_cast<Vec*>(dst + r * HD)[hl] = lo[r];
          reinterpret_cast<Vec*>(dst + r * HD)[16 + hl] = hi[r];
        }
      }
      continue;
    }
    // angle = position * freq: the product is taken in fp32 as the reference does
    const float posf = static_cast<float>(p.positions[tok]);
    // a' = a cos + other * sa, where other is the pair's second member with sa = -sin for a
    // first member, and the first member with sa = +sin for a second member held by another
    // lane; with both members in this lane b' = b cos + a * sb, sb = +sin.
    uint64_t cs2[W], sa2[W], sb2[W];
#pragma unroll
    for (int w = 0; w < W; ++w) {
      float c0, s0, c1, s1;
      sincos_reduced(posf * freq[2 * w], s0, c0);
      sincos_reduced(posf * freq[2 * w + 1], s1, c1);
      cs2[w] = pack_f32x2(c0, c1);
      sb2[w] = pack_f32x2(s0, s1);
      sa2[w] = (!in_lane && hl >= xm) ? sb2[w] : pack_f32x2(-s0, -s1);
    }
    const T* wt = static_cast<const T*>(is_q ? p.q_weight : p.k_weight);
    uint64_t wl[W], wh[W];
    if (wt != nullptr) {
      const Vec l = reinterpret_cast<const Vec*>(wt)[hl], h = reinterpret_cast<const Vec*>(wt)[16 + hl];
#pragma unroll
      for (int w = 0; w < W; ++w) {
        wl[w] = from_bits2(word(l, w));
        wh[w] = from_bits2(word(h, w));
      }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
      if (r >= cnt) break;
      uint64_t a[W], b[W];
#pragma unroll
      for (int w = 0; w < W; ++w) {
        a[w] = from_bits2(word(lo[r], w));
        b[w] = from_bits2(word(hi[r], w));
      }
      if (wt != nullptr) {
        uint64_t acc = mul_f32x2(a[0], a[0]);
        acc = fma_f32x2(b[0], b[0], acc);
#pragma unroll
        for (int w = 1; w < W; ++w) {
          acc = fma_f32x2(a[w], a[w], acc);
          acc = fma_f32x2(b[w], b[w], acc);
        }
        float s0, s1;
        unpack_f32x2(acc, s0, s1);
        float ss = s0 + s1;
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(hmask, ss, o);
        const float inv = rsqrtf(ss * (1.f / HD) + p.eps);
        const uint64_t inv2 = pack_f32x2(inv, inv);
        // (x * inv) * w, rounded to the 16-bit type as the reference's materialised norm output is
#pragma unroll
        for (int w = 0; w < W; ++w) {
          a[w] = from_bits2(to_bits2(mul_f32x2(mul_f32x2(a[w], inv2), wl[w])));
          b[w] = from_bits2(to_bits2(mul_f32x2(mul_f32x2(b[w], inv2), wh[w])));
        }
      }
      if (in_lane) {
#pragma unroll
        for (int w = 0; w < W; ++w) {
          const uint64_t x = a[w];
          a[w] = fma_f32x2(b[w], sa2[w], mul_f32x2(x, cs2[w]));
          b[w] = fma_f32x2(x, sb2[w], mul_f32x2(b[w], cs2[w]));
        }
      } else {
#pragma unroll
        for (int w = 0; w < W; ++w) {
          float x0, x1;
          unpack_f32x2(a[w], x0, x1);
          const uint64_t other = pack_f32x2(__shfl_xor_sync(hmask, x0, xm), __shfl_xor_sync(hmask, x1, xm));
          if (rot_lane) a[w] = fma_f32x2(other, sa2[w], mul_f32x2(a[w], cs2[w]));
        }
      }
      Vec olo, ohi;
#pragma unroll
      for (int w = 0; w < W; ++w) {
        reinterpret_cast<uint32_t*>(&olo)[w] = to_bits2(a[w]);
        reinterpret_cast<uint32_t*>(&ohi)[w] = to_bits2(b[w]);
      }
      reinterpret_cast<Vec*>(dst + r * HD)[hl] = olo;
      reinterpret_cast<Vec*>(dst + r * HD)[16 + hl] = ohi;
    }
  }
}

}  // namespace msgl
