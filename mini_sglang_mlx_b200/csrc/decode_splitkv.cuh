// Split-KV flash-decoding for one query token per sequence (sm_100a).
//
// Pass 1 (decode_partial_kernel): one CTA per (split, kv_head, sequence).  The
// G = Hq/Hkv query heads of the KV head are the rows of a 16-row tensor-core
// tile.  Each warp of the CTA walks its own 16-token groups of the split's
// token range: the K and V rows of a group (256 bytes per token per head at
// head_dim 128) are gathered through the per-token slot ids with 16-byte
// cp.async copies (16 lanes cover one row) into a warp-private ring of
// swizzled shared-memory tiles, then S = Q K^T and O += P V run as
// m16n8k16 mma.sync with fp32 accumulation and a base-2 online softmax whose
// row reductions are warp shuffles.  The warps' (max, sum, O) triples are
// merged through shared memory; the CTA writes a normalised fp32 partial and
// its log-sum-exp, or the final bf16/f16 row when the sequence has one split.
// Pass 2 (decode_merge_kernel): one CTA per (q_head, sequence) merges the
// partials by log-sum-exp.
//
// Semantics follow the reference stages
// (mini-sglang-mlx-kernel/csrc/paged_decode_attention.metal:313-506 and
// 512-586): slot addressing row = kv_indices[kv_indptr[b] + t], normalised
// partials, lse in natural-log units, merge out = sum_s e^{lse_s-M} O_s /
// sum_s e^{lse_s-M}.  Address arithmetic is 64-bit.
#pragma once

#include "common.cuh"

namespace msgl {

struct DecodeParams {
  const void* q;
  const void* k_cache;
  const void* v_cache;
  const int32_t* kv_indptr;
  const int32_t* kv_indices;
  const int32_t* num_kv_splits;  // may be null
  void* out;
  const void* gate;  // (batch, hq, D) or null: out *= sigmoid(gate)
  float* part_o;    // (batch, hq, max_splits, D)
  float* part_lse;  // (batch, hq, max_splits)
  int* status;      // device status word (0 = ok); may be null
  int batch, hq, hkv, group;
  int max_splits;
  int64_t num_slots;
  float scale_log2;  // sm_scale * log2(e)
};

constexpr int kDecodeGroupTokens = 16;  // tokens a warp consumes per step

// Split count actually used for a sequence of length L: the caller's hint
// clamped to [1, max_splits] and to the number of CTA-wide token tiles.
__device__ __forceinline__ int decode_effective_splits(int L, const int32_t* hints, int b,
                                                       int max_splits, int cta_tokens) {
  int s = hints ? hints[b] : max_splits;
  s = min(s, max_splits);
  s = min(s, ceil_div(L, cta_tokens));
  return max(s, 1);
}

template <typename T, int HD, int NWARPS, int NSTAGES>
__global__ void __launch_bounds__(NWARPS * 32)
    decode_partial_kernel(const DecodeParams p) {
  constexpr int CH = HD / 8;                              // 16-byte chunks per token row
  constexpr int ROW_BYTES = HD * 2;
  constexpr int TILE_BYTES = kDecodeGroupTokens * ROW_BYTES;  // one K (or V) group tile
  constexpr int CTA_TOKENS = NWARPS * kDecodeGroupTokens;
  constexpr int KSTEPS = HD / 16;
  constexpr int NT = HD / 8;  // output n-tiles
  static_assert(CH == 16 || CH == 32, "head_dim must be 128 or 256");

  extern __shared__ __align__(128) unsigned char smem_raw[];

  const int split = blockIdx.x;
  const int h = blockIdx.y;
  const int b = blockIdx.z;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int kv_begin = p.kv_indptr[b];
  const int L = p.kv_indptr[b + 1] - kv_begin;
  const int splits = decode_effective_splits(L, p.num_kv_splits, b, p.max_splits, CTA_TOKENS);
  if (split >= splits) return;
  const int per = ceil_div(ceil_div(L, splits), CTA_TOKENS) * CTA_TOKENS;
  const int t_begin = split * per;
  const int t_end = min(L, t_begin + per);

  const int G = p.group;
  const T* __restrict__ q = static_cast<const T*>(p.q);
  const unsigned char* __restrict__ kbase = static_cast<const unsigned char*>(p.k_cache);
  const unsigned char* __restrict__ vbase = static_cast<const unsigned char*>(p.v_cache);
  const int64_t slot_stride = static_cast<int64_t>(p.hkv) * ROW_BYTES;
  const int64_t head_off = static_cast<int64_t>(h) * ROW_BYTES;

  // ---- Q fragments: rows = query heads of this KV head (rows >= G are zero)
  uint32_t qf[KSTEPS][4];
  {
    const int r0 = lane >> 2;
    const int c0 = (lane & 3) * 2;
    const uint32_t* q0 = reinterpret_cast<const uint32_t*>(
        q + (static_cast<int64_t>(b) * p.hq + static_cast<int64_t>(h) * G + r0) * HD);
    const uint32_t* q1 = q0 + 8 * HD / 2;
    const bool v0 = r0 < G;
    const bool v1 = (r0 + 8) < G;
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
      const int w = (ks * 16 + c0) >> 1;
      qf[ks][0] = v0 ? q0[w] : 0u;
      qf[ks][1] = v1 ? q1[w] : 0u;
      qf[ks][2] = v0 ? q0[w + 4] : 0u;
      qf[ks][3] = v1 ? q1[w + 4] : 0u;
    }
  }

  // ---- warp-private ring of K/V group tiles
  const uint32_t ring = smem_u32(smem_raw) + warp * (NSTAGES * 2 * TILE_BYTES);

  // group g of this warp covers tokens [t_begin + (g*NWARPS + warp)*16, +16)
  const int first = t_begin + warp * kDecodeGroupTokens;
  const int nsteps = first < t_end ? ceil_div(t_end - first, CTA_TOKENS) : 0;

  auto load_idx = [&](int step) -> int {
    int slot = -1;
    if (step < nsteps && lane < kDecodeGroupTokens) {
      const int t = first + step * CTA_TOKENS + lane;
      if (t < t_end) {
        slot = p.kv_indices[kv_begin + t];
        if (slot < 0 || static_cast<int64_t>(slot) >= p.num_slots) {
          if (p.status) atomicExch(p.status, 2);  // out-of-range slot: treated as absent
          slot = -1;
        }
      }
    }
    return slot;
  };

  auto issue = [&](int stage, int my_slot) {
    const uint32_t kdst = ring + stage * (2 * TILE_BYTES);
    const uint32_t vdst = kdst + TILE_BYTES;
    constexpr int ROWS_PER_PASS = 32 / CH == 0 ? 1 : 32 / CH;  // 2 at HD=128, 1 at HD=256
    constexpr int PASSES = kDecodeGroupTokens / ROWS_PER_PASS;
    const int chunk = lane % CH;
    const int rsub = lane / CH;
#pragma unroll
    for (int i = 0; i < PASSES; ++i) {
      const int row = i * ROWS_PER_PASS + rsub;
      const int slot = __shfl_sync(0xffffffffu, my_slot, row);
      const bool ok = slot >= 0;
      const int64_t off = (ok ? static_cast<int64_t>(slot) * slot_stride + head_off : 0) + chunk * 16;
      const uint32_t so = swz_offset<CH>(row, chunk);
      cp_async_16(kdst + so, kbase + off, ok ? 16 : 0);
      cp_async_16(vdst + so, vbase + off, ok ? 16 : 0);
    }
  };

  float o[NT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

  // prologue: NSTAGES-1 groups in flight
  int next_slot = load_idx(0);
#pragma unroll
  for (int s = 0; s < NSTAGES - 1; ++s) {
    if (s < nsteps) issue(s, next_slot);
    cp_async_commit();
    next_slot = load_idx(s + 1);
  }

  for (int step = 0; step < nsteps; ++step) {
    cp_async_wait<NSTAGES - 2>();
    __syncwarp();
    // refill the stage consumed in the previous iteration
    {
      const int nstep = step + NSTAGES - 1;
      if (nstep < nsteps) issue(nstep % NSTAGES, next_slot);
      cp_async_commit();
      next_slot = load_idx(nstep + 1);
    }
    const uint32_t kt = ring + (step % NSTAGES) * (2 * TILE_BYTES);
    const uint32_t vt = kt + TILE_BYTES;
    const int tok0 = first + step * CTA_TOKENS;

    // S = Q K^T for 16 tokens: two n-tiles of 8 tokens
    float s[2][4];
#pragma unroll
    for (int i = 0; i < 2; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
    {
      const int mat = lane >> 3;
      const int row = (lane & 7) + ((mat >> 1) << 3);
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks) {
        uint32_t kf[4];
        ldmatrix_x4(kf, kt + swz_offset<CH>(row, 2 * ks + (mat & 1)));
        MmaOp<T>::run(s[0], qf[ks], kf[0], kf[1]);
        MmaOp<T>::run(s[1], qf[ks], kf[2], kf[3]);
      }
    }
    // scale to base-2 logits, mask the tail of the range
    const int nvalid = t_end - tok0;  // >= 1
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int col = nt * 8 + (lane & 3) * 2 + (e & 1);
        s[nt][e] = (col < nvalid) ? s[nt][e] * p.scale_log2 : -INFINITY;
      }
    }
    float mx0 = quad_max(fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1])));
    float mx1 = quad_max(fmaxf(fmaxf(s[0][2], s[0][3]), fmaxf(s[1][2], s[1][3])));
    const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);  // finite: column 0 is valid
    const float a0 = fast_exp2(m0 - mn0), a1 = fast_exp2(m1 - mn1);
    m0 = mn0;
    m1 = mn1;
    float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      s[nt][0] = fast_exp2(s[nt][0] - mn0);
      s[nt][1] = fast_exp2(s[nt][1] - mn0);
      s[nt][2] = fast_exp2(s[nt][2] - mn1);
      s[nt][3] = fast_exp2(s[nt][3] - mn1);
      ps0 += s[nt][0] + s[nt][1];
      ps1 += s[nt][2] + s[nt][3];
    }
    l0 = l0 * a0 + ps0;
    l1 = l1 * a1 + ps1;
#pragma unroll
    for (int i = 0; i < NT; ++i) {
      o[i][0] *= a0;
      o[i][1] *= a0;
      o[i][2] *= a1;
      o[i][3] *= a1;
    }
    uint32_t pa[4];
    pa[0] = MmaOp<T>::pack(s[0][0], s[0][1]);
    pa[1] = MmaOp<T>::pack(s[0][2], s[0][3]);
    pa[2] = MmaOp<T>::pack(s[1][0], s[1][1]);
    pa[3] = MmaOp<T>::pack(s[1][2], s[1][3]);
    // O += P V
    {
      const int mat = lane >> 3;
      const int row = (lane & 7) + ((mat & 1) << 3);
#pragma unroll
      for (int j = 0; j < NT / 2; ++j) {
        uint32_t vf[4];
        ldmatrix_x4_trans(vf, vt + swz_offset<CH>(row, 2 * j + (mat >> 1)));
        MmaOp<T>::run(o[2 * j], pa, vf[0], vf[1]);
        MmaOp<T>::run(o[2 * j + 1], pa, vf[2], vf[3]);
      }
    }
  }
  cp_async_wait<0>();
  l0 = quad_sum(l0);
  l1 = quad_sum(l1);
  __syncthreads();  // every warp is done with its ring: reuse it for the merge

  // ---- merge the warps' partials
  float* sm_m = reinterpret_cast<float*>(smem_raw);          // [NWARPS][16]
  float* sm_l = sm_m + NWARPS * 16;                          // [NWARPS][16]
  float* sm_o = sm_l + NWARPS * 16;                          // [NWARPS][16][HD]
  {
    const int r0 = lane >> 2;
    if ((lane & 3) == 0) {
      sm_m[warp * 16 + r0] = m0;
      sm_m[warp * 16 + r0 + 8] = m1;
      sm_l[warp * 16 + r0] = l0;
      sm_l[warp * 16 + r0 + 8] = l1;
    }
    float* ow = sm_o + warp * 16 * HD;
#pragma unroll
    for (int i = 0; i < NT; ++i) {
      const int c = i * 8 + (lane & 3) * 2;
      if (r0 < G) *reinterpret_cast<float2*>(ow + r0 * HD + c) = make_float2(o[i][0], o[i][1]);
      if (r0 + 8 < G)
        *reinterpret_cast<float2*>(ow + (r0 + 8) * HD + c) = make_float2(o[i][2], o[i][3]);
    }
  }
  __syncthreads();

  T* out = static_cast<T*>(p.out);
  for (int g = 0; g < G; ++g) {
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < NWARPS; ++w) M = fmaxf(M, sm_m[w * 16 + g]);
    float wgt[NWARPS];
    float den = 0.f;
#pragma unroll
    for (int w = 0; w < NWARPS; ++w) {
      wgt[w] = (M == -INFINITY) ? 0.f : fast_exp2(sm_m[w * 16 + g] - M);
      den += wgt[w] * sm_l[w * 16 + g];
    }
    const float inv = den > 0.f ? 1.f / den : 0.f;
    const int64_t hq_idx = static_cast<int64_t>(b) * p.hq + static_cast<int64_t>(h) * G + g;
    for (int d = threadIdx.x; d < HD; d += NWARPS * 32) {
      float num = 0.f;
#pragma unroll
      for (int w = 0; w < NWARPS; ++w) num += wgt[w] * sm_o[(w * 16 + g) * HD + d];
      const float val = num * inv;
      if (splits == 1) {
        out[hq_idx * HD + d] = p.gate ? apply_gate<T>(val, static_cast<const T*>(p.gate)[hq_idx * HD + d])
                                      : MmaOp<T>::from_float(val);
      } else {
        p.part_o[(hq_idx * p.max_splits + split) * HD + d] = val;
      }
    }
    if (splits > 1 && threadIdx.x == 0) {
      p.part_lse[hq_idx * p.max_splits + split] =
          den > 0.f ? M * kLn2 + __logf(den) : -INFINITY;
    }
  }
}

template <typename T, int HD, int CTA_TOKENS>
__global__ void __launch_bounds__(HD) decode_merge_kernel(const DecodeParams p) {
  const int hq = blockIdx.x;
  const int b = blockIdx.y;
  const int L = p.kv_indptr[b + 1] - p.kv_indptr[b];
  const int splits = decode_effective_splits(L, p.num_kv_splits, b, p.max_splits, CTA_TOKENS);
  if (splits <= 1) return;  // pass 1 already wrote the final row
  grid_dependency_wait();   // the partials come from pass 1
  const int64_t hq_idx = static_cast<int64_t>(b) * p.hq + hq;
  const float* lse = p.part_lse + hq_idx * p.max_splits;
  const float* po = p.part_o + hq_idx * p.max_splits * HD;
  float M = -INFINITY;
  for (int s = 0; s < splits; ++s) M = fmaxf(M, lse[s]);
  const int d = threadIdx.x;
  float num = 0.f, den = 0.f;
  if (M != -INFINITY) {
    for (int s = 0; s < splits; ++s) {
      const float w = __expf(lse[s] - M);
      den += w;
      num += w * po[s * HD + d];
    }
  }
  const float val = den > 0.f ? num / den : 0.f;
  static_cast<T*>(p.out)[hq_idx * HD + d] =
      p.gate ? apply_gate<T>(val, static_cast<const T*>(p.gate)[hq_idx * HD + d]) : MmaOp<T>::from_float(val);
}

}  // namespace msgl
