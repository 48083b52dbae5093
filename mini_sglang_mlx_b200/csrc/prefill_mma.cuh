// Paged prefill / extend / verify attention on warp-level tensor-core tiles
// (mma.sync m16n8k16, fp32 accumulation) with GQA-packed query rows.
//
// One CTA (4 warps) owns a tile of 64 packed query rows of one KV head and
// walks the visible key range of that tile in 64-token steps.  K and V rows
// are gathered through the per-token slot ids with 16-byte cp.async copies
// into a three-stage ring of swizzled shared-memory tiles shared by the four
// warps; each warp keeps its 16 query rows as register fragments.  Tiles
// that lie wholly inside every row's visible range skip the mask.  With
// kv_chunk > 0 the key range is cut into splits whose unnormalised partials
// (O, max, sum) go to scratch and are combined by prefill_merge_kernel.
#pragma once

#include "prefill_tiles.cuh"

namespace msgl {

constexpr int kMmaBM = 64;
constexpr int kMmaBN = 64;
constexpr int kMmaWarps = 4;
constexpr int kMmaStages = 3;

template <typename T, int HD>
__global__ void __launch_bounds__(kMmaWarps * 32)
    prefill_mma_kernel(const PrefillParams p) {
  constexpr int BM = kMmaBM, BN = kMmaBN, NTHREADS = kMmaWarps * 32;
  constexpr int CH = HD / 8;
  constexpr int ROW_BYTES = HD * 2;
  constexpr int TILE_BYTES = BN * ROW_BYTES;
  constexpr int KSTEPS = HD / 16;
  constexpr int NT = HD / 8;
  constexpr int ROWS_PER_PASS = NTHREADS / CH;  // token rows covered by one pass of the CTA
  constexpr int PASSES = BN / ROWS_PER_PASS;

  extern __shared__ __align__(128) unsigned char smem_raw[];
  const uint32_t smem0 = smem_u32(smem_raw);

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int h = blockIdx.y;
  const int G = p.group;

  int b, local, base;
  // heaviest (last) items first: later q tiles of a causal chunk see more keys
  const int item = static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x);
  if (!find_item<NTHREADS>(p, item, BM, b, local, base)) return;
  const SeqShape sq = load_seq_shape(p, b, BM);
  const int qt = local / sq.nsplit;
  const int split = local % sq.nsplit;
  if (p.plan && local == 0 && h == 0 && tid == 0) {
    p.plan[2 * b] = base;
    p.plan[2 * b + 1] = sq.nsplit;
  }

  // packed rows of this tile
  const int pk0 = qt * BM;
  const int tok_first = pk0 / G;
  const int tok_last = min(sq.tq - 1, (pk0 + BM - 1) / G);
  const int pos_first = sq.prefix + tok_first;
  const int pos_last = sq.prefix + tok_last;
  // key range of the tile, then of the split
  int kv_lo = p.window > 0 ? max(0, pos_first - p.window + 1) : 0;
  int kv_hi = p.is_cross ? sq.L : min(sq.L, pos_last + 1);
  if (p.kv_chunk > 0) {
    kv_lo = max(kv_lo, sq.lo + split * p.kv_chunk);
    kv_hi = min(kv_hi, sq.lo + (split + 1) * p.kv_chunk);
  }
  kv_lo = (kv_lo / BN) * BN;  // tile-aligned start; the mask trims the front
  const int ntiles = kv_hi > kv_lo ? ceil_div(kv_hi - kv_lo, BN) : 0;

  const T* __restrict__ q = static_cast<const T*>(p.q);
  const unsigned char* __restrict__ kbase = static_cast<const unsigned char*>(p.k_cache);
  const unsigned char* __restrict__ vbase = static_cast<const unsigned char*>(p.v_cache);
  const int64_t slot_stride = static_cast<int64_t>(p.hkv) * ROW_BYTES;
  const int64_t head_off = static_cast<int64_t>(h) * ROW_BYTES;

  // ---- Q tile -> shared (stage 0 area) -> A fragments in registers
  {
    constexpr int QPASSES = BM / ROWS_PER_PASS;
    const int chunk = tid % CH, rsub = tid / CH;
#pragma unroll
    for (int i = 0; i < QPASSES; ++i) {
      const int row = i * ROWS_PER_PASS + rsub;
      const int pk = pk0 + row;
      const int tl = pk / G, g = pk - tl * G;
      const bool ok = tl < sq.tq;
      const int64_t off =
          ok ? ((static_cast<int64_t>(sq.q_begin + tl) * p.hq + static_cast<int64_t>(h) * G + g) * HD)
             : 0;
      cp_async_16(smem0 + swz_offset<CH>(row, chunk),
                  reinterpret_cast<const unsigned char*>(q + off) + chunk * 16, ok ? 16 : 0);
    }
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();
  }
  uint32_t qf[KSTEPS][4];
  {
    const int mat = lane >> 3;
    const int row = warp * 16 + (lane & 7) + ((mat & 1) << 3);
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks)
      ldmatrix_x4(qf[ks], smem0 + swz_offset<CH>(row, 2 * ks + (mat >> 1)));
  }
  __syncthreads();  // Q area is free for the K/V ring

  // ---- per-lane row geometry (two rows per lane)
  const int r0 = warp * 16 + (lane >> 2), r1 = r0 + 8;
  const int tl0 = (pk0 + r0) / G, tl1 = (pk0 + r1) / G;
  const int pos0 = sq.prefix + tl0, pos1 = sq.prefix + tl1;
  const int hi0 = p.is_cross ? sq.L - 1 : min(pos0, sq.L - 1);
  const int hi1 = p.is_cross ? sq.L - 1 : min(pos1, sq.L - 1);
  const int lo0 = p.window > 0 ? pos0 - p.window + 1 : 0;
  const int lo1 = p.window > 0 ? pos1 - p.window + 1 : 0;
  // split bounds also clip visibility
  const int s_lo = p.kv_chunk > 0 ? sq.lo + split * p.kv_chunk : 0;
  const int s_hi = p.kv_chunk > 0 ? sq.lo + (split + 1) * p.kv_chunk - 1 : 0x7fffffff;
  const int vlo0 = max(lo0, s_lo), vlo1 = max(lo1, s_lo);
  const int vhi0 = min(hi0, s_hi), vhi1 = min(hi1, s_hi);
  // bounds inside which every row of the CTA sees every key
  const int all_lo = max(p.window > 0 ? pos_last - p.window + 1 : 0, s_lo);
  const int all_hi = min(min(p.is_cross ? sq.L - 1 : pos_first, sq.L - 1), s_hi);

  // ---- K/V ring
  const int chunk = tid % CH, rsub = tid / CH;
  int slots[PASSES];
  auto load_slots = [&](int tile) {
#pragma unroll
    for (int i = 0; i < PASSES; ++i) {
      const int t = kv_lo + tile * BN + i * ROWS_PER_PASS + rsub;
      int slot = -1;
      if (tile < ntiles && t < kv_hi) {
        slot = p.kv_indices[sq.kv_begin + t];
        if (slot < 0 || static_cast<int64_t>(slot) >= p.num_slots) {
          if (p.status) atomicExch(p.status, 2);
          slot = -1;
        }
      }
      slots[i] = slot;
    }
  };
  auto issue = [&](int stage) {
    const uint32_t kdst = smem0 + stage * (2 * TILE_BYTES);
    const uint32_t vdst = kdst + TILE_BYTES;
#pragma unroll
    for (int i = 0; i < PASSES; ++i) {
      const int row = i * ROWS_PER_PASS + rsub;
      const bool ok = slots[i] >= 0;
      const int64_t off =
          (ok ? static_cast<int64_t>(slots[i]) * slot_stride + head_off : 0) + chunk * 16;
      const uint32_t so = swz_offset<CH>(row, chunk);
      cp_async_16(kdst + so, kbase + off, ok ? 16 : 0);
      cp_async_16(vdst + so, vbase + off, ok ? 16 : 0);
    }
  };

  float o[NT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

  load_slots(0);
#pragma unroll
  for (int s = 0; s < kMmaStages - 1; ++s) {
    if (s < ntiles) issue(s);
    cp_async_commit();
    load_slots(s + 1);
  }

  for (int tile = 0; tile < ntiles; ++tile) {
    cp_async_wait<kMmaStages - 2>();
    __syncthreads();  // tile `tile` landed for all threads; stage (tile-1) is free
    {
      const int nt_ = tile + kMmaStages - 1;
      if (nt_ < ntiles) issue(nt_ % kMmaStages);
      cp_async_commit();
      load_slots(nt_ + 1);
    }
    const uint32_t kt = smem0 + (tile % kMmaStages) * (2 * TILE_BYTES);
    const uint32_t vt = kt + TILE_BYTES;
    const int k0 = kv_lo + tile * BN;

    float s[BN / 8][4];
#pragma unroll
    for (int i = 0; i < BN / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
    {
      const int mat = lane >> 3;
      const int rowin = (lane & 7) + ((mat >> 1) << 3);
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
        for (int np = 0; np < BN / 16; ++np) {
          uint32_t kf[4];
          ldmatrix_x4(kf, kt + swz_offset<CH>(np * 16 + rowin, 2 * ks + (mat & 1)));
          MmaOp<T>::run(s[2 * np], qf[ks], kf[0], kf[1]);
          MmaOp<T>::run(s[2 * np + 1], qf[ks], kf[2], kf[3]);
        }
      }
    }
    const bool full = (k0 >= all_lo) && (k0 + BN - 1 <= all_hi);
    if (full) {
#pragma unroll
      for (int i = 0; i < BN / 8; ++i) {
#pragma unroll
        for (int e = 0; e < 4; ++e) s[i][e] *= p.scale_log2;
      }
    } else {
#pragma unroll
      for (int i = 0; i < BN / 8; ++i) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int kpos = k0 + i * 8 + (lane & 3) * 2 + (e & 1);
          const bool vis = (e < 2) ? (kpos >= vlo0 && kpos <= vhi0) : (kpos >= vlo1 && kpos <= vhi1);
          s[i][e] = vis ? s[i][e] * p.scale_log2 : -INFINITY;
        }
      }
    }
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int i = 0; i < BN / 8; ++i) {
      mx0 = fmaxf(mx0, fmaxf(s[i][0], s[i][1]));
      mx1 = fmaxf(mx1, fmaxf(s[i][2], s[i][3]));
    }
    mx0 = quad_max(mx0);
    mx1 = quad_max(mx1);
    const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
    // a row with no visible key so far keeps max = -inf; use 0 as the
    // subtrahend so that exp2(-inf - 0) = 0 instead of NaN
    const float mu0 = (mn0 == -INFINITY) ? 0.f : mn0;
    const float mu1 = (mn1 == -INFINITY) ? 0.f : mn1;
    const float a0 = fast_exp2(m0 - mu0), a1 = fast_exp2(m1 - mu1);
    m0 = mn0;
    m1 = mn1;
    float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
    for (int i = 0; i < BN / 8; ++i) {
      s[i][0] = fast_exp2(s[i][0] - mu0);
      s[i][1] = fast_exp2(s[i][1] - mu0);
      s[i][2] = fast_exp2(s[i][2] - mu1);
      s[i][3] = fast_exp2(s[i][3] - mu1);
      ps0 += s[i][0] + s[i][1];
      ps1 += s[i][2] + s[i][3];
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
    {
      const int mat = lane >> 3;
      const int rowin = (lane & 7) + ((mat & 1) << 3);
#pragma unroll
      for (int kk = 0; kk < BN / 16; ++kk) {
        uint32_t pa[4];
        pa[0] = MmaOp<T>::pack(s[2 * kk][0], s[2 * kk][1]);
        pa[1] = MmaOp<T>::pack(s[2 * kk][2], s[2 * kk][3]);
        pa[2] = MmaOp<T>::pack(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        pa[3] = MmaOp<T>::pack(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int j = 0; j < NT / 2; ++j) {
          uint32_t vf[4];
          ldmatrix_x4_trans(vf, vt + swz_offset<CH>(kk * 16 + rowin, 2 * j + (mat >> 1)));
          MmaOp<T>::run(o[2 * j], pa, vf[0], vf[1]);
          MmaOp<T>::run(o[2 * j + 1], pa, vf[2], vf[3]);
        }
      }
    }
  }
  cp_async_wait<0>();
  l0 = quad_sum(l0);
  l1 = quad_sum(l1);

  // ---- epilogue
  const int g0 = (pk0 + r0) - tl0 * G, g1 = (pk0 + r1) - tl1 * G;
  const bool ok0 = tl0 < sq.tq, ok1 = tl1 < sq.tq;
  if (p.kv_chunk == 0) {
    T* out = static_cast<T*>(p.out);
    const float i0 = l0 > 0.f ? 1.f / l0 : 0.f, i1 = l1 > 0.f ? 1.f / l1 : 0.f;
    T* o0 = out + (static_cast<int64_t>(sq.q_begin + tl0) * p.hq + static_cast<int64_t>(h) * G + g0) * HD;
    T* o1 = out + (static_cast<int64_t>(sq.q_begin + tl1) * p.hq + static_cast<int64_t>(h) * G + g1) * HD;
#pragma unroll
    for (int i = 0; i < NT; ++i) {
      const int c = i * 8 + (lane & 3) * 2;
      if (ok0) *reinterpret_cast<uint32_t*>(o0 + c) = MmaOp<T>::pack(o[i][0] * i0, o[i][1] * i0);
      if (ok1) *reinterpret_cast<uint32_t*>(o1 + c) = MmaOp<T>::pack(o[i][2] * i1, o[i][3] * i1);
    }
  } else {
    const int64_t slot = static_cast<int64_t>(item) * p.hkv + h;
    float* po = p.part_o + slot * BM * HD;
    float* pml = p.part_ml + slot * BM * 2;
    if ((lane & 3) == 0) {
      if (ok0) *reinterpret_cast<float2*>(pml + r0 * 2) = make_float2(m0, l0);
      if (ok1) *reinterpret_cast<float2*>(pml + r1 * 2) = make_float2(m1, l1);
    }
#pragma unroll
    for (int i = 0; i < NT; ++i) {
      const int c = i * 8 + (lane & 3) * 2;
      if (ok0) *reinterpret_cast<float2*>(po + r0 * HD + c) = make_float2(o[i][0], o[i][1]);
      if (ok1) *reinterpret_cast<float2*>(po + r1 * HD + c) = make_float2(o[i][2], o[i][3]);
    }
  }
}

// Combines the kv-split partials of one (query token, query head).
// grid = (total_q, hq), block = HD threads.
template <typename T, int HD, int BM>
__global__ void __launch_bounds__(HD) prefill_merge_kernel(const PrefillParams p) {
  const int tok = blockIdx.x;
  const int hq = blockIdx.y;
  // sequence of this token: last b with qo_indptr[b] <= tok
  int lo = 0, hi = p.batch;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (p.qo_indptr[mid] <= tok) lo = mid; else hi = mid;
  }
  const int b = lo;
  const int q_begin = p.qo_indptr[b];
  if (tok < q_begin || tok >= p.qo_indptr[b + 1]) return;  // token not covered by any sequence
  const int G = p.group;
  const int h = hq / G, g = hq - h * G;
  const int pk = (tok - q_begin) * G + g;
  const int qt = pk / BM, r = pk - qt * BM;
  const int base = p.plan[2 * b], nsplit = p.plan[2 * b + 1];
  const int d = threadIdx.x;
  float M = -INFINITY;
  for (int s = 0; s < nsplit; ++s) {
    const int64_t slot = static_cast<int64_t>(base + qt * nsplit + s) * p.hkv + h;
    M = fmaxf(M, p.part_ml[(slot * BM + r) * 2]);
  }
  float num = 0.f, den = 0.f;
  if (M != -INFINITY) {
    for (int s = 0; s < nsplit; ++s) {
      const int64_t slot = static_cast<int64_t>(base + qt * nsplit + s) * p.hkv + h;
      const float2 ml = *reinterpret_cast<const float2*>(p.part_ml + (slot * BM + r) * 2);
      const float w = fast_exp2(ml.x - M);  // exp2(-inf) = 0 for empty splits
      den += w * ml.y;
      num += w * p.part_o[(slot * BM + r) * HD + d];
    }
  }
  static_cast<T*>(p.out)[(static_cast<int64_t>(tok) * p.hq + hq) * HD + d] =
      MmaOp<T>::from_float(den > 0.f ? num / den : 0.f);
}

}  // namespace msgl
