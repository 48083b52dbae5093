// Work decomposition shared by the paged prefill kernels and their merge pass.
//
// Query rows of one sequence and one KV head are "packed": packed index
// pk = token_local * G + g addresses query token token_local and query head
// kv_head * G + g, so that all G heads sharing a KV head sit in the same tile
// and K/V is read once per KV head.  A tile is BM consecutive packed rows.
// A work item is (sequence, q tile, kv split); items are numbered densely in
// sequence order and a CTA finds its item from blockIdx.x with a block-wide
// scan over the sequences' item counts (no planning launch, no host sync).
//
// Mask semantics are those of the reference kernel
// (mini-sglang-mlx-kernel/csrc/paged_prefill_attention.metal:324-350 and
// 446-450): query row p of a sequence sits at absolute position
// prefix_len + p; key t is visible iff t < kv_len, (cross or t <= pos) and
// (W == 0 or t >= pos - W + 1).
#pragma once

#include "common.cuh"

namespace msgl {

struct PrefillParams {
  const void* q;
  const void* k_cache;
  const void* v_cache;
  const int32_t* qo_indptr;
  const int32_t* kv_indptr;
  const int32_t* kv_indices;
  const int32_t* prefix_lens;
  void* out;
  float* part_o;   // (items, hkv, BM, D) unnormalised fp32 partial outputs
  float* part_ml;  // (items, hkv, BM, 2) running max (base-2 units) and sum
  int* plan;       // (batch, 2): first item id and split count of each sequence
  int* status;
  int batch, total_q, hq, hkv, group;
  int64_t num_slots;
  float scale_log2;
  int is_cross, window;
  int kv_chunk;  // tokens per kv split; 0 = never split
};

struct SeqShape {
  int q_begin, tq, kv_begin, L, prefix;
  int lo, hi;      // union over the sequence's rows of the visible key range [lo, hi)
  int nqt, nsplit;
};

__device__ __forceinline__ SeqShape load_seq_shape(const PrefillParams& p, int b, int BM) {
  SeqShape s;
  s.q_begin = p.qo_indptr[b];
  s.tq = max(p.qo_indptr[b + 1] - s.q_begin, 0);
  s.kv_begin = p.kv_indptr[b];
  s.L = max(p.kv_indptr[b + 1] - s.kv_begin, 0);
  s.prefix = p.prefix_lens[b];
  s.lo = p.window > 0 ? max(0, s.prefix - p.window + 1) : 0;
  s.hi = p.is_cross ? s.L : min(s.L, s.prefix + s.tq);
  s.hi = max(s.hi, s.lo);
  s.nqt = ceil_div(s.tq * p.group, BM);
  s.nsplit = p.kv_chunk > 0 ? max(1, ceil_div(s.hi - s.lo, p.kv_chunk)) : 1;
  return s;
}

// Block-wide search for the sequence that owns flat item id `item`.
// Returns false (for the whole block) if item is past the last one.
// On success: b = sequence, local = item index inside it, base = its first item.
template <int NTHREADS>
__device__ __forceinline__ bool find_item(const PrefillParams& p, int item, int BM, int& b_out,
                                          int& local_out, int& base_out) {
  __shared__ int s_warp_tot[NTHREADS / 32];
  __shared__ int s_found[3];
  const int tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;
  if (tid == 0) s_found[0] = -1;
  __syncthreads();
  int running = 0;
  for (int b0 = 0; b0 < p.batch; b0 += NTHREADS) {
    const int b = b0 + tid;
    int items = 0;
    if (b < p.batch) {
      const SeqShape s = load_seq_shape(p, b, BM);
      items = s.nqt * s.nsplit;
    }
    int incl = items;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    if (lane == 31) s_warp_tot[warp] = incl;
    __syncthreads();
    int warp_base = 0, total = 0;
#pragma unroll
    for (int w = 0; w < NTHREADS / 32; ++w) {
      const int t = s_warp_tot[w];
      if (w < warp) warp_base += t;
      total += t;
    }
    const int excl = running + warp_base + incl - items;
    if (items > 0 && item >= excl && item < excl + items) {
      s_found[0] = b;
      s_found[1] = item - excl;
      s_found[2] = excl;
    }
    running += total;
    __syncthreads();
    if (running > item) break;
  }
  __syncthreads();
  b_out = s_found[0];
  local_out = s_found[1];
  base_out = s_found[2];
  return b_out >= 0;
}

// Upper bound (host side) on the number of work items.
inline int64_t prefill_item_bound(int batch, int total_q, int64_t total_kv, int group, int BM,
                                  int max_len_extend, int kv_chunk) {
  const int64_t packed = static_cast<int64_t>(total_q) * group;
  const int64_t qtiles = packed / BM + batch;  // sum of ceil(tq*G/BM)
  if (kv_chunk <= 0) return qtiles;
  const int64_t nqt_max =
      (static_cast<int64_t>(max_len_extend) * group + BM - 1) / BM;
  // sum_b nqt_b * ceil(span_b / chunk) <= nqt_max * (total_kv / chunk + batch)
  return nqt_max * (total_kv / kv_chunk + batch);
}

}  // namespace msgl
