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
// Merge: the CTA of a (sequence, KV head) that finishes last (an arrival counter per pair)
// combines the splits' partials by log-sum-exp and writes the final rows; there is no second
// launch.
//
// Page-granular form (PAGED): a warp's 16-token group is one page (or a 16-row slice of a
// larger page), contiguous in the pool, so lane 0 fetches its K and V rows with TMA box copies
// (cp.async.bulk.tensor.2d, 16 rows x 64 elements, 128-byte swizzle) straight from the page id
// and the warp waits on the stage's mbarrier; only a sequence's ragged last page is copied row
// by row (rows past the length are zero-filled).
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
  // page-granular addressing (kv_lens != null): see PrefillParams
  const int32_t* page_indptr;
  const int32_t* page_indices;
  const int32_t* kv_lens;
  int page_size;
  void* out;
  const void* gate;  // (batch, hq, D) or null: out *= sigmoid(gate)
  float* part_o;    // (batch, hq, max_splits, D)
  float* part_lse;  // (batch, hq, max_splits)
  // (batch, hkv) arrival counters of the splits of a (sequence, KV head): the CTA that arrives
  // last merges the partials and puts the counter back to zero.  Zero before the first launch.
  int* tickets;
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

// Length in tokens of sequence b (page-granular: clamped to the tokens its pages hold).
__device__ __forceinline__ int decode_seq_len(const DecodeParams& p, int b) {
  if (p.kv_lens) {
    const int64_t cap =
        static_cast<int64_t>(max(p.page_indptr[b + 1] - p.page_indptr[b], 0)) * p.page_size;
    return static_cast<int>(min(static_cast<int64_t>(max(p.kv_lens[b], 0)), cap));
  }
  return p.kv_indptr[b + 1] - p.kv_indptr[b];
}

template <typename T, int HD, int NWARPS, int NSTAGES, bool PAGED = false>
__global__ void __launch_bounds__(NWARPS * 32)
    decode_partial_kernel(const DecodeParams p, const __grid_constant__ CUtensorMap tm_k,
                          const __grid_constant__ CUtensorMap tm_v) {
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
#ifdef MSGL_TRACE
  const int tr_id = (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
#define MSGL_TRD(slot, value) do { if (threadIdx.x == 0 && tr_id < kTraceCtas) g_cta_trace[tr_id][slot] = (value); } while (0)
  MSGL_TRD(0, trace_wall());
  MSGL_TRD(1, clock64());
  MSGL_TRD(2, trace_smid());
  MSGL_TRD(10, 0);
#else
#define MSGL_TRD(slot, value) do { } while (0)
#endif

  const int G = p.group;
  const T* __restrict__ q = static_cast<const T*>(p.q);
  // (issued before the sequence's length is looked up: the two round trips to memory overlap)
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

  const int kv_begin = PAGED ? p.page_indptr[b] : p.kv_indptr[b];   // pages / tokens
  const int L = decode_seq_len(p, b);
  if (PAGED && split == 0 && h == 0 && threadIdx.x == 0 && p.status) {
    const int len = p.kv_lens[b];   // negative or beyond the sequence's pages: clamped, reported
    if (len < 0 || len > L) atomicExch(p.status, 2);
  }
  const int splits = decode_effective_splits(L, p.num_kv_splits, b, p.max_splits, CTA_TOKENS);
  if (split >= splits) return;
  MSGL_TRD(3, clock64());      // lengths known
  const int per = ceil_div(ceil_div(L, splits), CTA_TOKENS) * CTA_TOKENS;
  const int t_begin = split * per;
  const int t_end = min(L, t_begin + per);

  const unsigned char* __restrict__ kbase = static_cast<const unsigned char*>(p.k_cache);
  const unsigned char* __restrict__ vbase = static_cast<const unsigned char*>(p.v_cache);
  const int64_t slot_stride = static_cast<int64_t>(p.hkv) * ROW_BYTES;
  const int64_t head_off = static_cast<int64_t>(h) * ROW_BYTES;

  // ---- warp-private ring of K/V group tiles
  // PAGED: tiles are TMA destinations with the 128-byte swizzle, which is a function of the
  // shared-memory address: the ring starts on a 1024-byte boundary.  A tile is HD/64 column
  // blocks of 16 rows x 128 bytes.
  const uint32_t smem_pad = PAGED ? ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u) : 0u;
  unsigned char* smem_al = smem_raw + smem_pad;
  const uint32_t ring = smem_u32(smem_al) + warp * (NSTAGES * 2 * TILE_BYTES);
  auto toff = [](int row, int chunk) -> uint32_t {
    if constexpr (PAGED)
      return static_cast<uint32_t>((chunk >> 3) * (kDecodeGroupTokens * 128) + (row << 7) +
                                   (((chunk & 7) ^ (row & 7)) << 4));
    else
      return swz_offset<CH>(row, chunk);
  };
  __shared__ uint64_t s_bar[PAGED ? NWARPS * NSTAGES : 1];
  if constexpr (PAGED) {
    if (threadIdx.x == 0) {
      for (int i = 0; i < NWARPS * NSTAGES; ++i) mbar_init(smem_u32(&s_bar[i]), 1);
      fence_mbar_init();
      prefetch_tensormap(&tm_k);
      prefetch_tensormap(&tm_v);
    }
    __syncthreads();
  }

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

  // ---- PAGED: page of a step -> first pool row y and number of valid rows n (all lanes agree)
  const int32_t* __restrict__ pages = PAGED ? p.page_indices + kv_begin : nullptr;
  auto load_page = [&](int step, int& y, int& n) {
    y = 0;
    n = 0;
    if (step < nsteps) {
      const int t = first + step * CTA_TOKENS;
      const int pg = __ldg(pages + t / p.page_size);
      const int64_t row0 = static_cast<int64_t>(pg) * p.page_size + t % p.page_size;
      const int nv = min(kDecodeGroupTokens, L - t);
      if (pg < 0 || row0 + nv > p.num_slots) {
        if (p.status && lane == 0) atomicExch(p.status, 2);   // page outside the pool: zeros
      } else {
        y = static_cast<int>(row0);
        n = nv;
      }
    }
  };
  auto bar_of = [&](int stage) { return smem_u32(&s_bar[warp * NSTAGES + stage]); };
  auto issue_page = [&](int stage, int y, int n) {
    const uint32_t kdst = ring + stage * (2 * TILE_BYTES);
    const uint32_t vdst = kdst + TILE_BYTES;
    const uint32_t bar = bar_of(stage);
    if (n == kDecodeGroupTokens) {
      if (lane == 0) {
        mbar_arrive_expect_tx(bar, 2 * TILE_BYTES);
#pragma unroll
        for (int c = 0; c < HD / 64; ++c) {
          tma_load_2d(kdst + c * (kDecodeGroupTokens * 128), &tm_k, h * HD + c * 64, y, bar);
          tma_load_2d(vdst + c * (kDecodeGroupTokens * 128), &tm_v, h * HD + c * 64, y, bar);
        }
      }
    } else {
      // ragged last page of the sequence (or a page outside the pool): valid rows by 16-byte
      // copies, the rest zeros; waited for on the spot (once per sequence and KV head)
#pragma unroll
      for (int k = 0; k < kDecodeGroupTokens * CH / 32; ++k) {
        const int e = k * 32 + lane;
        const int row = e / CH, chunk = e % CH;
        const bool ok = row < n;
        const int64_t off =
            (ok ? static_cast<int64_t>(y + row) * slot_stride + head_off : 0) + chunk * 16;
        cp_async_16(kdst + toff(row, chunk), kbase + off, ok ? 16 : 0);
        cp_async_16(vdst + toff(row, chunk), vbase + off, ok ? 16 : 0);
      }
      cp_async_commit();
      cp_async_wait<0>();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar);
    }
  };

  // prologue: NSTAGES-1 groups in flight
  int next_slot = 0, next_y = 0, next_n = 0;
  if constexpr (PAGED) {
    int py[NSTAGES], pn[NSTAGES];
#pragma unroll
    for (int s = 0; s < NSTAGES; ++s) load_page(s, py[s], pn[s]);   // independent loads, in flight together
#pragma unroll
    for (int s = 0; s < NSTAGES - 1; ++s)
      if (s < nsteps) issue_page(s, py[s], pn[s]);
    next_y = py[NSTAGES - 1];
    next_n = pn[NSTAGES - 1];
  } else {
    next_slot = load_idx(0);
#pragma unroll
    for (int s = 0; s < NSTAGES - 1; ++s) {
      if (s < nsteps) issue(s, next_slot);
      cp_async_commit();
      next_slot = load_idx(s + 1);
    }
  }

  MSGL_TRD(4, clock64());      // Q in registers, first copies issued
  bool alive = true;
  for (int step = 0; step < nsteps; ++step) {
    if (step == 1) MSGL_TRD(5, clock64());   // first group consumed
    if constexpr (PAGED) {
      // bounded wait for this step's stage
      const uint32_t bar = bar_of(step % NSTAGES);
      const uint32_t parity = (step / NSTAGES) & 1;
      bool ok = mbar_try_wait(bar, parity);
      if (!ok) {
        const long long t0 = clock64();
        while (!(ok = mbar_try_wait(bar, parity)) && clock64() - t0 < kTcWaitCycles) {
        }
      }
      alive = __all_sync(0xffffffffu, ok ? 1 : 0) != 0;
      if (!alive) break;
      // refill the stage consumed in the previous iteration
      const int nstep = step + NSTAGES - 1;
      if (nstep < nsteps) issue_page(nstep % NSTAGES, next_y, next_n);
      load_page(nstep + 1, next_y, next_n);
    } else {
      cp_async_wait<NSTAGES - 2>();
      __syncwarp();
      // refill the stage consumed in the previous iteration
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
        ldmatrix_x4(kf, kt + toff(row, 2 * ks + (mat & 1)));
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
        ldmatrix_x4_trans(vf, vt + toff(row, 2 * j + (mat >> 1)));
        MmaOp<T>::run(o[2 * j], pa, vf[0], vf[1]);
        MmaOp<T>::run(o[2 * j + 1], pa, vf[2], vf[3]);
      }
    }
  }
  MSGL_TRD(6, clock64());      // main loop done
  cp_async_wait<0>();
  if (PAGED && !alive && p.status && lane == 0) atomicExch(p.status, 1);   // a wait ran out
  l0 = quad_sum(l0);
  l1 = quad_sum(l1);
  __syncthreads();  // every warp is done with its ring: reuse it for the merge

  // ---- merge the warps' partials
  float* sm_m = reinterpret_cast<float*>(smem_al);           // [NWARPS][16]
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
  constexpr int VPL = HD / 32, NV = VPL / 4;   // columns (16-byte pieces) of a row per lane
  // a warp per query head (heads warp, warp + NWARPS, ...), a lane per VPL consecutive columns
  for (int g = warp; g < G; g += NWARPS) {
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
    float4 num[NV];
#pragma unroll
    for (int e4 = 0; e4 < NV; ++e4) num[e4] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int w = 0; w < NWARPS; ++w) {
      const float4* row = reinterpret_cast<const float4*>(sm_o + (w * 16 + g) * HD + lane * VPL);
#pragma unroll
      for (int e4 = 0; e4 < NV; ++e4) {
        const float4 x = row[e4];
        num[e4].x += wgt[w] * x.x;
        num[e4].y += wgt[w] * x.y;
        num[e4].z += wgt[w] * x.z;
        num[e4].w += wgt[w] * x.w;
      }
    }
#pragma unroll
    for (int e4 = 0; e4 < NV; ++e4) {
      num[e4].x *= inv;
      num[e4].y *= inv;
      num[e4].z *= inv;
      num[e4].w *= inv;
    }
    if (splits == 1) {
      const int64_t oi = hq_idx * HD + lane * VPL;
      alignas(16) T vals[VPL];
#pragma unroll
      for (int e4 = 0; e4 < NV; ++e4) {
        const float f[4] = {num[e4].x, num[e4].y, num[e4].z, num[e4].w};
#pragma unroll
        for (int e = 0; e < 4; ++e)
          vals[4 * e4 + e] = p.gate ? apply_gate<T>(f[e], static_cast<const T*>(p.gate)[oi + 4 * e4 + e])
                                    : MmaOp<T>::from_float(f[e]);
      }
      if constexpr (VPL == 4)
        *reinterpret_cast<uint2*>(out + oi) = *reinterpret_cast<const uint2*>(vals);
      else
        *reinterpret_cast<uint4*>(out + oi) = *reinterpret_cast<const uint4*>(vals);
    } else {
      float4* dst = reinterpret_cast<float4*>(p.part_o + (hq_idx * p.max_splits + split) * HD + lane * VPL);
#pragma unroll
      for (int e4 = 0; e4 < NV; ++e4) dst[e4] = num[e4];
      if (lane == 0)
        p.part_lse[hq_idx * p.max_splits + split] = den > 0.f ? M * kLn2 + __logf(den) : -INFINITY;
    }
  }
  MSGL_TRD(7, clock64());      // partial (or final rows) written
  MSGL_TRD(10, trace_wall());
  if (splits == 1) return;

  // ---- the split that arrives last merges: out = sum_s e^(lse_s - M) O_s / sum_s e^(lse_s - M)
  // (the second stage of the reference, paged_decode_attention.metal:512-586, without a launch)
  __shared__ int s_last;
  __threadfence();      // this thread's partials are visible device-wide before the arrival
  __syncthreads();
  if (threadIdx.x == 0) {
    int* ticket = p.tickets + static_cast<int64_t>(b) * p.hkv + h;
    const int arrived = atomicAdd(ticket, 1);
    s_last = (arrived == splits - 1) ? 1 : 0;
    if (s_last) *ticket = 0;
  }
  __syncthreads();
  MSGL_TRD(8, clock64());      // arrival counted
  MSGL_TRD(10, trace_wall());
  MSGL_TRD(11, s_last);
  if (s_last == 0) return;
  __threadfence();
  // a warp per query head, a lane per 4 (8) output columns; the splits' rows come straight from
  // scratch (L2), four splits in flight per lane
  constexpr int SIF = HD == 256 ? 8 : 16;   // splits in flight per lane
  for (int g = warp; g < G; g += NWARPS) {
    const int64_t hq_idx = static_cast<int64_t>(b) * p.hq + static_cast<int64_t>(h) * G + g;
    const float* lse = p.part_lse + hq_idx * p.max_splits;
    const float* po = p.part_o + hq_idx * p.max_splits * HD + lane * VPL;
    float ls[SIF];
    float4 x[SIF][NV];
    auto load_splits = [&](int s0) {
#pragma unroll
      for (int u = 0; u < SIF; ++u) {
        const int sp = min(s0 + u, splits - 1);
        ls[u] = __ldcg(lse + sp);
#pragma unroll
        for (int e4 = 0; e4 < NV; ++e4)
          x[u][e4] = __ldcg(reinterpret_cast<const float4*>(po + static_cast<int64_t>(sp) * HD) + e4);
      }
    };
    load_splits(0);   // in flight while the largest log-sum-exp is found
    float M = -INFINITY;
    for (int s = lane; s < splits; s += 32) M = fmaxf(M, __ldcg(lse + s));
#pragma unroll
    for (int o2 = 16; o2 > 0; o2 >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o2));
    float num[VPL];
#pragma unroll
    for (int e = 0; e < VPL; ++e) num[e] = 0.f;
    float den = 0.f;
    if (M != -INFINITY) {
      for (int s0 = 0; s0 < splits; s0 += SIF) {
        if (s0 > 0) load_splits(s0);
#pragma unroll
        for (int u = 0; u < SIF; ++u) {
          if (s0 + u >= splits) break;
          const float w = __expf(ls[u] - M);
          den += w;
#pragma unroll
          for (int e4 = 0; e4 < NV; ++e4) {
            num[4 * e4 + 0] += w * x[u][e4].x;
            num[4 * e4 + 1] += w * x[u][e4].y;
            num[4 * e4 + 2] += w * x[u][e4].z;
            num[4 * e4 + 3] += w * x[u][e4].w;
          }
        }
      }
    }
    const float inv = den > 0.f ? 1.f / den : 0.f;
    const int64_t oi = hq_idx * HD + lane * VPL;
    alignas(16) T vals[VPL];
#pragma unroll
    for (int e = 0; e < VPL; ++e) {
      const float val = num[e] * inv;
      vals[e] = p.gate ? apply_gate<T>(val, static_cast<const T*>(p.gate)[oi + e]) : MmaOp<T>::from_float(val);
    }
    if constexpr (VPL == 4)
      *reinterpret_cast<uint2*>(out + oi) = *reinterpret_cast<const uint2*>(vals);
    else
      *reinterpret_cast<uint4*>(out + oi) = *reinterpret_cast<const uint4*>(vals);
  }
  MSGL_TRD(9, clock64());      // merged rows written
  MSGL_TRD(10, trace_wall());
}

}  // namespace msgl
