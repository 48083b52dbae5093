// Work decomposition shared by the paged prefill kernels and the merge of their key-range splits.
//
// Query rows of one sequence and one KV head are "packed": packed index
// pk = token_local * G + g addresses query token token_local and query head
// kv_head * G + g, so that all G heads sharing a KV head sit in the same tile
// and K/V is read once per KV head.  A tile is BM consecutive packed rows.
// A work item is (sequence, q tile, kv split); items are numbered densely and a
// CTA finds its item from its launch rank with a block-wide pass over the
// sequences' item counts (no planning launch, no host sync).
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
  // Page-granular addressing (kv_lens != null): sequence b owns pages
  // page_indices[page_indptr[b] .. page_indptr[b+1]) of page_size tokens each, token t of the
  // sequence sits in slot page_indices[page_indptr[b] + t / page_size] * page_size + t % page_size,
  // and kv_lens[b] is its length in tokens.  kv_indptr / kv_indices are unused then.
  const int32_t* page_indptr;
  const int32_t* page_indices;
  const int32_t* kv_lens;
  int page_size;
  void* out;
  const void* gate;  // (total_q, hq, D) or null: out *= sigmoid(gate)
  float* part_o;   // (items, hkv, BM, D) unnormalised fp32 partial outputs
  float* part_ml;  // (items, hkv, BM, 2) running max (base-2 units) and sum
  // Arrival counters of the kv splits of a (sequence, q tile, head) unit, one per unit (units
  // are numbered densely; the key range is split only while there are at most kPrefillTickets
  // of them): the CTA that arrives last merges the partials and puts the counter back to zero.
  // They live in the workspace header and read zero whenever no call is in flight.
  int* tickets;
  int q_tma;       // PAGED: the query rows are described by a tensor map (TMA loads)
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
  if (p.kv_lens) {
    // page-granular: kv_begin counts pages; a length beyond the sequence's pages is clamped
    s.kv_begin = p.page_indptr[b];
    const int64_t cap = static_cast<int64_t>(max(p.page_indptr[b + 1] - s.kv_begin, 0)) * p.page_size;
    s.L = static_cast<int>(min(static_cast<int64_t>(max(p.kv_lens[b], 0)), cap));
  } else {
    s.kv_begin = p.kv_indptr[b];
    s.L = max(p.kv_indptr[b + 1] - s.kv_begin, 0);
  }
  s.prefix = p.prefix_lens[b];
  s.lo = p.window > 0 ? max(0, s.prefix - p.window + 1) : 0;
  s.hi = p.is_cross ? s.L : min(s.L, s.prefix + s.tq);
  s.hi = max(s.hi, s.lo);
  s.nqt = ceil_div(s.tq * p.group, BM);
  s.nsplit = p.kv_chunk > 0 ? max(1, ceil_div(s.hi - s.lo, p.kv_chunk)) : 1;
  return s;
}

// Which (sequence, kv head, q tile, kv split) a CTA works on.
struct ItemCoord {
  int b, h, qt, split;
  int base;    // id of the sequence's first item; an item's scratch slot is base + qt*nsplit + split
  int qt_base; // q tiles of the sequences in front: (qt_base + qt) * hkv + h numbers the
               // (sequence, q tile, head) units densely (arrival counters of the kv splits)
  bool first;  // exactly one CTA per sequence has this set (it reports a clamped length)
};

constexpr int kSortedBatchMax = 128;
constexpr int kPrefillTickets = 1024;   // arrival counters the prefill op may use

// Block-wide mapping from a launch rank (blockIdx.x; 0 is scheduled first) to a work item.
// Returns false (for the whole block) if the rank is past the last item.
// Order: sequence, then kv head, then q tile / kv split.  CTAs that run at the same
// time then mostly share one sequence's K/V of one or two heads (L2 reuse), and heavy
// work gets low ranks so that the hardware's in-order CTA dispatch approximates
// longest-first scheduling: with at most kSortedBatchMax sequences they are taken by
// visible key length, longest first, and inside a (sequence, head) the last (causally
// longest) q tile comes first; larger batches keep the natural order, reversed.
// `scratch` is block-shared memory the caller does not need yet (4*kSortedBatchMax ints).
template <int NTHREADS>
__device__ __forceinline__ bool find_item(const PrefillParams& p, int rank, int BM, int* scratch,
                                          ItemCoord& out) {
  __shared__ int s_res[7];
  const int tid = threadIdx.x;
  if (tid == 0) s_res[0] = -1;
  if (p.batch <= kSortedBatchMax) {
    int* s_key = scratch;
    int* s_cnt = scratch + kSortedBatchMax;
    int* s_nsplit = scratch + 2 * kSortedBatchMax;
    int* s_nqt = scratch + 3 * kSortedBatchMax;
    if (tid < p.batch) {
      const SeqShape s = load_seq_shape(p, tid, BM);
      s_key[tid] = s.hi - s.lo;
      s_cnt[tid] = s.nqt * s.nsplit;
      s_nsplit[tid] = s.nsplit;
      s_nqt[tid] = s.nqt;
    }
    __syncthreads();
    if (tid < p.batch) {
      // rank of this sequence in the order (longest first) and the items of all sequences in
      // front of it, in one pass; the sequence whose item range holds `rank` publishes the result
      const int key = s_key[tid];
      int running = 0, running_qt = 0;
      for (int k = 0; k < p.batch; ++k) {
        const int kk = s_key[k];
        if (kk > key || (kk == key && k < tid)) {
          running += s_cnt[k];
          running_qt += s_nqt[k];
        }
      }
      const int c = s_cnt[tid];
      if (c > 0 && rank >= running * p.hkv && rank < (running + c) * p.hkv) {
        const int off = rank - running * p.hkv;
        const int local = off % c;
        const int nsplit = s_nsplit[tid];
        s_res[0] = tid;
        s_res[1] = c / nsplit - 1 - local / nsplit;  // last q tile first
        s_res[2] = local % nsplit;
        s_res[3] = running;
        s_res[4] = off == 0;
        s_res[5] = off / c;
        s_res[6] = running_qt;
      }
    }
    __syncthreads();
  } else {
    // natural order, reversed: flat id = (CTAs launched) - 1 - rank
    __shared__ int s_warp_tot[NTHREADS / 32];
    const int flat = static_cast<int>(gridDim.x) - 1 - rank;
    const int lane = tid & 31, warp = tid >> 5;
    __syncthreads();
    __shared__ int s_warp_qt[NTHREADS / 32];
    int running = 0, running_qt = 0;
    for (int b0 = 0; b0 < p.batch; b0 += NTHREADS) {
      const int b = b0 + tid;
      int items = 0, nsplit = 1, nqt = 0;
      if (b < p.batch) {
        const SeqShape s = load_seq_shape(p, b, BM);
        items = s.nqt * s.nsplit;
        nsplit = s.nsplit;
        nqt = s.nqt;
      }
      int incl = items, incl_qt = nqt;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        const int vq = __shfl_up_sync(0xffffffffu, incl_qt, o);
        if (lane >= o) {
          incl += v;
          incl_qt += vq;
        }
      }
      if (lane == 31) {
        s_warp_tot[warp] = incl;
        s_warp_qt[warp] = incl_qt;
      }
      __syncthreads();
      int warp_base = 0, total = 0, warp_base_qt = 0, total_qt = 0;
#pragma unroll
      for (int w = 0; w < NTHREADS / 32; ++w) {
        const int t = s_warp_tot[w], tq = s_warp_qt[w];
        if (w < warp) {
          warp_base += t;
          warp_base_qt += tq;
        }
        total += t;
        total_qt += tq;
      }
      const int excl = running + warp_base + incl - items;
      const int excl_qt = running_qt + warp_base_qt + incl_qt - nqt;
      if (items > 0 && flat >= excl * p.hkv && flat < (excl + items) * p.hkv) {
        const int off = flat - excl * p.hkv;
        const int local = off % items;
        s_res[0] = b;
        s_res[1] = local / nsplit;
        s_res[2] = local % nsplit;
        s_res[3] = excl;
        s_res[4] = off == 0;
        s_res[5] = off / items;
        s_res[6] = excl_qt;
      }
      running += total;
      running_qt += total_qt;
      __syncthreads();
      if (running * p.hkv > flat) break;
    }
    __syncthreads();
  }
  out.b = s_res[0];
  out.qt = s_res[1];
  out.split = s_res[2];
  out.base = s_res[3];
  out.first = s_res[4] != 0;
  out.h = s_res[5];
  out.qt_base = s_res[6];
  return out.b >= 0;
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
