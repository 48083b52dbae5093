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
// One CTA per token, its warps independent of one another (no shared memory, no CTA
// barrier).  A half-warp owns a row: lane hl of it holds E = head_dim/32 consecutive elements
// of the lower half of the row and the E elements half a row further on (8- or 16-byte
// accesses), so with rotary_dim == head_dim both members of a rotary pair sit in the same lane
// (with a smaller rotary_dim the partner is a lane of the same half-warp).  A warp has eight
// rows in flight (four at head_dim 256) and as many prefetched (the kernel needs the bytes in
// flight), and computes the rotary angles its lanes need itself.
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

template <typename T, int HD>
__global__ void __launch_bounds__(256) qk_norm_rope_store_kernel(const QkNormRopeParams p) {
  static_assert(HD == 128 || HD == 256, "head_dim 128 or 256");
  constexpr int RU = HD == 128 ? 4 : 2;  // row pairs a warp has in flight (a half-warp per row)
  constexpr int E = HD / 32;             // elements of a lane in each half of the row
  constexpr int W = E / 2;               // 32-bit words (16-bit pairs) of those
  using Vec = typename RowVec<E * 2>::type;
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
  // lane (side, hl) holds elements E*hl .. E*hl+E-1 of the lower and of the upper half of
  // row (first + 2u + side)
  auto load_rows = [&](int first, Vec (&lo)[RU], Vec (&hi)[RU]) {
#pragma unroll
    for (int u = 0; u < RU; ++u) {
      const int row = first + 2 * u + side;
      if (row < rows) {
        const Vec* src = reinterpret_cast<const Vec*>(row_ptr(row));
        lo[u] = src[hl];
        hi[u] = src[16 + hl];
      }
    }
  };
  auto word = [](const Vec& v, int i) -> uint32_t { return reinterpret_cast<const uint32_t*>(&v)[i]; };
  // the first rows are on their way while the token's angles are worked out
  Vec lo[RU], hi[RU];
  load_rows(warp * 2 * RU, lo, hi);
  const int slot = p.out_loc[tok];
  const bool slot_ok = slot >= 0 && slot < p.num_slots;
  // Rotary pairs are (i, i + half).  With rotary_dim == head_dim the partner of a lane's lower
  // element is its own upper element.  With a smaller rotary_dim the pairs lie inside the
  // lower half of the row: lanes below xm hold first members, the partner is lane ^ xm, and
  // lanes from 2*xm on (and the whole upper half) pass through.  angle = position *
  // base^(-2i/rd): the product is taken in fp32 as the reference does.
  const bool in_lane = p.rotary_dim == HD;
  const int xm = in_lane ? 0 : half / E;
  const bool rot_lane = in_lane || hl < 2 * xm;
  const int f0 = in_lane ? E * hl : E * (hl & (xm - 1));
  const float posf = static_cast<float>(p.positions[tok]);
  const float inv_rd = 1.f / static_cast<float>(p.rotary_dim);
  uint64_t cs2[W], sn2[W], ng2[W];
#pragma unroll
  for (int w = 0; w < W; ++w) {
    float c0, s0, c1, s1;
    sincos_reduced(posf * exp2f(-p.log2_base * (static_cast<float>(2 * (f0 + 2 * w)) * inv_rd)), s0, c0);
    sincos_reduced(posf * exp2f(-p.log2_base * (static_cast<float>(2 * (f0 + 2 * w + 1)) * inv_rd)), s1, c1);
    cs2[w] = pack_f32x2(c0, c1);
    sn2[w] = pack_f32x2(s0, s1);
    ng2[w] = pack_f32x2(-s0, -s1);
  }
  // norm weights as packed pairs of floats: [lower words, upper words]
  uint64_t wq[2 * W], wk[2 * W];
  {
    const T* w = static_cast<const T*>(p.q_weight);
    const T* x = static_cast<const T*>(p.k_weight);
#pragma unroll
    for (int i = 0; i < 2 * W; ++i) {
      const int e0 = (i / W) * (HD / 2) + E * hl + (i % W) * 2;
      wq[i] = w ? pack_f32x2(to_f32(w[e0]), to_f32(w[e0 + 1])) : 0ull;
      wk[i] = x ? pack_f32x2(to_f32(x[e0]), to_f32(x[e0 + 1])) : 0ull;
    }
  }
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
    Vec nlo[RU], nhi[RU];   // the next rows, in flight while these are processed
    load_rows(first + nwarps * 2 * RU, nlo, nhi);
#pragma unroll
    for (int u = 0; u < RU; ++u) {
      const int row = first + 2 * u + side;
      const bool live = row < rows;
      if (first + 2 * u >= n_qk) {
        // ---- both rows of the pair are V rows (or past the end): copy into the pool
        if (live && slot_ok) {
          T* dst = static_cast<T*>(p.v_cache) + slot * p.cache_stride + (row - n_qk) * HD;
          reinterpret_cast<Vec*>(dst)[hl] = lo[u];
          reinterpret_cast<Vec*>(dst)[16 + hl] = hi[u];
        }
        continue;
      }
      // the two half-warps may still hold rows of different kinds (last q row / first k row,
      // last k row / first v row): every decision below is per half-warp, the shuffles stay
      // inside it
      const bool is_v = live && row >= n_qk;
      const bool is_q = live && row < p.hq;
      const bool has_w = live && !is_v && (is_q ? p.q_weight : p.k_weight) != nullptr;
      uint64_t a[W], b[W];
#pragma unroll
      for (int w = 0; w < W; ++w) {
        a[w] = from_bits2(live ? word(lo[u], w) : 0u);
        b[w] = from_bits2(live ? word(hi[u], w) : 0u);
      }
      float ss;
      {
        uint64_t acc = mul_f32x2(a[0], a[0]);
        acc = fma_f32x2(b[0], b[0], acc);
#pragma unroll
        for (int w = 1; w < W; ++w) {
          acc = fma_f32x2(a[w], a[w], acc);
          acc = fma_f32x2(b[w], b[w], acc);
        }
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
#pragma unroll
        for (int w = 0; w < W; ++w) {
          a[w] = from_bits2(to_bits2(mul_f32x2(mul_f32x2(a[w], inv2), is_q ? wq[w] : wk[w])));
          b[w] = from_bits2(to_bits2(mul_f32x2(mul_f32x2(b[w], inv2), is_q ? wq[W + w] : wk[W + w])));
        }
      }
      if (in_lane) {
        if (!is_v) {
          // a' = a cos - b sin, b' = a sin + b cos
#pragma unroll
          for (int w = 0; w < W; ++w) {
            const uint64_t x = a[w];
            a[w] = fma_f32x2(b[w], ng2[w], mul_f32x2(x, cs2[w]));
            b[w] = fma_f32x2(b[w], cs2[w], mul_f32x2(x, sn2[w]));
          }
        }
      } else {
#pragma unroll
        for (int w = 0; w < W; ++w) {
          float x0, x1;
          unpack_f32x2(a[w], x0, x1);
          const uint64_t other = pack_f32x2(__shfl_xor_sync(0xffffffffu, x0, xm),
                                            __shfl_xor_sync(0xffffffffu, x1, xm));
          if (!is_v && rot_lane) {
            a[w] = hl < xm ? fma_f32x2(other, ng2[w], mul_f32x2(a[w], cs2[w]))     // first member
                           : fma_f32x2(other, sn2[w], mul_f32x2(a[w], cs2[w]));    // second member
          }
        }
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
      Vec olo, ohi;
#pragma unroll
      for (int w = 0; w < W; ++w) {
        reinterpret_cast<uint32_t*>(&olo)[w] = to_bits2(a[w]);
        reinterpret_cast<uint32_t*>(&ohi)[w] = to_bits2(b[w]);
      }
      reinterpret_cast<Vec*>(dst)[hl] = is_v ? lo[u] : olo;
      reinterpret_cast<Vec*>(dst)[16 + hl] = is_v ? hi[u] : ohi;
    }
#pragma unroll
    for (int u = 0; u < RU; ++u) {
      lo[u] = nlo[u];
      hi[u] = nhi[u];
    }
  }
}

}  // namespace msgl
