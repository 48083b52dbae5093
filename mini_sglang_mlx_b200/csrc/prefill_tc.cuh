// Paged prefill / extend / verify attention on the 5th-generation tensor
// cores: tcgen05.mma with accumulators in tensor memory (TMEM), sm_100a only.
//
// One CTA owns 256 GQA-packed query rows of one KV head (two sub-tiles of 128
// rows) and walks the visible key range in tiles of BN tokens.  Two variants:
// BN = 128 (S single-buffered; the two sub-tiles ping-pong on the tensor pipe)
// for long query chunks, BN = 64 (S double-buffered, S runs two key tiles
// ahead of PV) for short query blocks where only one sub-tile has rows.
//
//   warps 0-3    softmax group 0: thread r owns row r of sub-tile 0 (TMEM lane r)
//   warps 4-7    softmax group 1: the same for sub-tile 1
//   warp  8      MMA issuer (one elected lane issues every tcgen05.mma / commit)
//   warps 9-15   producers: gather Q rows and paged K/V token rows with 16-byte
//                cp.async into 128-byte-swizzled shared-memory tiles
// The softmax warps raise their register budget (setmaxnreg) so that a thread can
// hold a whole 128-column score row; the other warps lower theirs.
// A one-sub-tile shape (128 rows: softmax warps 0-3, MMA warp 4, producers 5-11,
// half the TMEM and under half the shared memory, two CTAs per SM) serves query
// blocks that fill at most one sub-tile.  Those shapes are bound by HBM, and a warp
// sustains only about one 512-byte cp.async instruction per 150 cycles (measured), so
// the shape keeps as many producer warps as the two-sub-tile one.
//
// Per key tile j and sub-tile i:  S_i[j] = Q_i K_j^T  (SS MMA M128 N=BN, fp32 in TMEM)
//   -> softmax group i reads its BN-column row (tcgen05.ld), masks boundary
//      tiles, keeps a running reference max (O is rescaled lazily, only when the
//      max grows by more than 2^8), writes P as 16-bit pairs over the first BN/2
//      of those columns (tcgen05.st)
//   -> O_i += P V_j  (TS MMA M128 N128: A from TMEM, V as an MN-major shared operand).
// S_i[j+LA] is issued right after PV_i[j] (LA = 1 for BN 128, 2 for BN 64 where
// S has two buffers per sub-tile).  All hand-offs are mbarriers; every wait is
// bounded and reports through the status word instead of hanging.
// TMEM columns: S_i[b] at 128 i + BN b (b = j mod 2 if double-buffered), O_i after the S tiles.
//
// Shared-memory tile layout (Q sub-tile, K tile and V tile alike): two halves,
// half h holding elements [64h, 64h+64) of every row; inside a half row r sits
// at (r/8)*1024 + (r%8)*128 and its 16-byte chunk c at position c ^ (r%8).
// This is the canonical 128-byte-swizzle layout, K-major for Q and K (rows =
// M/N index) and MN-major for V (rows = K index).
//
// Page-granular form (PAGED): the pool is addressed by pages of 16 tokens (or a multiple), so
// the 16 token rows of a page are contiguous in the pool and one TMA box copy
// (cp.async.bulk.tensor.2d, 16 rows x 64 elements, 128-byte swizzle = exactly the tile layout
// above) moves a quarter of a 64-key tile's K or V half.  One lane per page issues the copies
// straight from the page ids, completion is counted in bytes on the tile's mbarrier; the seven
// copying warps and the per-token id staging go away.  Only the ragged last page of a sequence
// (and the pages of a tile past the sequence's end) are filled with 16-byte cp.async copies, so
// that rows past the sequence's length are zeros rather than whatever the pool holds there.
//
// Key-range splits (few query tiles: verify, draft blocks, short chunks over long prefixes): a
// CTA writes an unnormalised fp32 partial (O rows and their (max, sum)) to scratch; the
// partials of a (sequence, query tile, head) unit are reduced row by row straight from scratch
// (merge_kv_splits), either by the CTA that arrives last at the unit's arrival counter, inside
// the same launch, or -- units whose partials exceed 64 KB -- by prefill_merge_kernel, a second
// launch chained with programmatic stream serialization that spreads the rows over the grid.
#pragma once

#include <type_traits>

#include "prefill_tiles.cuh"

namespace msgl {

constexpr int kTcSub = 128;       // rows per sub-tile (= MMA M)

// Shape of a CTA.  NSUB = 2: 256 query rows, 16 warps, all 512 TMEM columns, 160 KB K/V
// ring, one CTA per SM.  NSUB = 1: 128 rows, 12 warps, 256 TMEM columns, 64 KB ring, two
// CTAs per SM (short query blocks are bandwidth-bound: two independent pipelines per SM
// keep more copies in flight).
//
// PAGED: the softmax warps, the MMA warp and three producer warps (the first issues the TMA
// copies, all three load Q): 4*NSUB + 4 warps.
template <int NSUB, int HD = 128, bool PAGED = false>
struct TcShape {
  static_assert(HD == 128 || (HD == 256 && NSUB == 1), "head_dim 256 runs the one-sub-tile shape");
  static constexpr int kBM = NSUB * kTcSub;                       // packed query rows per CTA
  static constexpr int kRowBytes = HD * 2;                        // one token row of one head
  static constexpr int kQTileBytes = kTcSub * kRowBytes;          // one 128-row query sub-tile
  static constexpr int kWarps = PAGED ? 4 * NSUB + 4 : (NSUB == 2 ? 16 : 12);
  static constexpr int kThreads = kWarps * 32;
  static constexpr int kMmaWarp = 4 * NSUB;                       // after the softmax warps
  static constexpr int kProducerWarp0 = kMmaWarp + 1;             // ... the rest copy
  static constexpr int kRingBytes = NSUB == 2 ? 5 * 128 * 256 : 4 * 64 * kRowBytes;
  static constexpr int kSmemBytes = NSUB * kQTileBytes + kRingBytes + 1024;  // + alignment slack
  static constexpr int kTmemCols = HD == 256 ? 512 : NSUB * 256;  // S buffers + O (HD columns per sub-tile)
  static constexpr int kCtasPerSm = (NSUB == 2 || HD == 256) ? 1 : 2;
  // register cap at launch: the one-sub-tile shapes start at 80 registers either way (the
  // setmaxnreg budgets below are written against that pool)
  // (head_dim 256 runs one CTA per SM anyway: its per-token form takes the larger cap, 168
  // registers for every warp, instead of spilling under 80)
  static constexpr int kMinCtasForRegs = (NSUB == 2 || (HD == 256 && !PAGED)) ? 1 : 2;
  // The CTA's register pool is threads x registers at launch; setmaxnreg moves registers between
  // the softmax warps and the others inside that pool.  The PAGED one-sub-tile shape (256 threads
  // at 128 registers, two CTAs per SM = the whole register file) already gives its softmax warps
  // what they need: no re-balancing there.
  static constexpr bool kRebalanceRegs = !(PAGED && NSUB == 1) && !(HD == 256 && !PAGED);
};

// ---------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void tc_mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void tc_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]),
        "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]),
        "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]),
        "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]),
        "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_st() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

template <int N>
__device__ __forceinline__ void reg_inc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void reg_dec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}
// Ties the registers written by an asynchronous tcgen05.ld to the wait that
// precedes this call: no instruction, only a scheduling dependency.
template <int N>
__device__ __forceinline__ void reg_fence(uint32_t (&r)[N]) {
#pragma unroll
  for (int e = 0; e < N; ++e) asm volatile("" : "+r"(r[e])::"memory");
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// 32 columns of this thread's TMEM lane into r[OFF .. OFF+32)
template <int OFF, int N>
__device__ __forceinline__ void tmem_ld32_at(uint32_t taddr, uint32_t (&r)[N]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[OFF + 0]), "=r"(r[OFF + 1]), "=r"(r[OFF + 2]), "=r"(r[OFF + 3]), "=r"(r[OFF + 4]),
        "=r"(r[OFF + 5]), "=r"(r[OFF + 6]), "=r"(r[OFF + 7]), "=r"(r[OFF + 8]), "=r"(r[OFF + 9]),
        "=r"(r[OFF + 10]), "=r"(r[OFF + 11]), "=r"(r[OFF + 12]), "=r"(r[OFF + 13]),
        "=r"(r[OFF + 14]), "=r"(r[OFF + 15]), "=r"(r[OFF + 16]), "=r"(r[OFF + 17]),
        "=r"(r[OFF + 18]), "=r"(r[OFF + 19]), "=r"(r[OFF + 20]), "=r"(r[OFF + 21]),
        "=r"(r[OFF + 22]), "=r"(r[OFF + 23]), "=r"(r[OFF + 24]), "=r"(r[OFF + 25]),
        "=r"(r[OFF + 26]), "=r"(r[OFF + 27]), "=r"(r[OFF + 28]), "=r"(r[OFF + 29]),
        "=r"(r[OFF + 30]), "=r"(r[OFF + 31])
      : "r"(taddr)
      : "memory");
}

// One lane of a converged warp (the same lane every time for a full mask).
__device__ __forceinline__ uint32_t elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t.reg .b32 rx;\n\t.reg .pred px;\n\t"
      "elect.sync rx|px, %1;\n\t"
      "@px mov.s32 %0, 1;\n\t}"
      : "+r"(pred)
      : "r"(0xFFFFFFFFu));
  return pred;
}

// Shared-memory matrix descriptor, 128-byte swizzle, descriptor version 1.
// lbo / sbo are byte offsets (leading / stride dimension).
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((lbo >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo >> 4) & 0x3FFFu) << 32;
  d |= 1ull << 46;
  d |= 2ull << 61;
  return d;
}

// Instruction descriptor of kind::f16: fp32 accumulate, A/B both bf16 or both f16,
// A K-major, B K-major (b_mn = 0) or MN-major (b_mn = 1), M = 128, N = n.
template <typename T>
__device__ __forceinline__ uint32_t idesc_m128(uint32_t n, uint32_t b_mn) {
  const uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
  return (1u << 4) | (fmt << 7) | (fmt << 10) | (b_mn << 16) | ((n >> 3) << 17) |
         ((128u >> 4) << 24);
}

// Byte offset of 16-byte chunk `chunk` (0..15) of row `row` inside a tile of ROWS rows.
template <int ROWS>
__device__ __forceinline__ uint32_t tc_tile_offset(int row, int chunk) {
  return static_cast<uint32_t>((chunk >> 3) * (ROWS * 128) + ((row >> 3) << 10) + ((row & 7) << 7) +
                               (((chunk & 7) ^ (row & 7)) << 4));
}

// Position of a tile in the order the MMA warp consumes the ring when S runs LA
// key tiles ahead of PV:  K_0 .. K_{LA-1}, then V_0 K_LA V_1 K_{LA+1} ...
template <int LA>
__device__ __forceinline__ int ring_seq_k(int t) { return t < LA ? t : 2 * t - LA + 1; }
template <int LA>
__device__ __forceinline__ int ring_seq_v(int j) { return 2 * j + LA; }

struct TcBarriers {
  uint64_t q_full;
  uint64_t idx_sync;  // producers only: guards the staged slot ids
  uint64_t full[10], empty[10];
  // [sub-tile][S buffer]: a softmax group may finish tile j+1 before the MMA warp has
  // looked at tile j, so both hand-offs are per S buffer (tiles j and j+2 never overlap)
  // (with one PV barrier a group that waits only now and then could not tell completion
  // j-2 from j by parity alone)
  uint64_t s_full[2][2], p_full[2][2], pv_done[2][2];
  // kv splits: stage[i] synchronises the 128 threads of softmax group i around the staging
  // buffer of its partial
  uint64_t stage[2];
};

// Merge of rows [row_lo, row_hi) of the kv-split partials of one (sequence, q tile, head) unit,
// run by NSW warps: all rows by the CTA that arrived last at the unit's counter, or (large
// units: one SM would pull megabytes through its own L2 port) a slice of the rows by each CTA
// of a second, dependent launch.  A warp owns RU rows at a time and a lane 4 or 8 columns
// of a row; per row it takes the largest split maximum M (lane-strided loads of the (m, l)
// pairs, one warp reduction), then walks the splits once: out = sum_s 2^(m_s - M) O_s /
// sum_s 2^(m_s - M) l_s, the rows of O_s read straight from scratch (they sit in L2: the
// splits have just written them), all splits of the RU rows in flight together.  No shared
// memory, no synchronisation between warps.
// (The few fields of the launch parameters it needs come by value: taking the address of the
// kernel's parameter block would make the kernel keep a local copy of it.)
struct MergeArgs {
  const float* part_o;
  const float* part_ml;
  void* out;
  const void* gate;
  int hq, group;
};
template <typename T, int HD, int NSW, int BM, int RU, int SU>
__device__ __noinline__ void merge_kv_splits(const MergeArgs p, int nsp, int64_t slot0,
                                             int64_t slot_stride, int row_lo, int row_hi, int pk0,
                                             int q_begin, int h) {
  // partial sp of the unit sits in scratch slot slot0 + sp * slot_stride; in scratch the
  // 16-byte chunk c of row r sits at chunk position c ^ (r & 31) of the row
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = p.group;
  __threadfence();
  constexpr int VPL = HD / 32;          // output columns per lane
  constexpr int NV = VPL / 4;           // 16-byte pieces per lane
  // RU rows a warp works on at a time, SU splits whose loads are issued together
  T* out = static_cast<T*>(p.out);
  const T* gate = static_cast<const T*>(p.gate);
  for (int r0 = row_lo + warp * RU; r0 < row_hi; r0 += NSW * RU) {
    int rr[RU];
#pragma unroll
    for (int k = 0; k < RU; ++k) rr[k] = min(r0 + k, row_hi - 1);
    float2 ml[SU][RU];
    float4 x[SU][RU][NV];
    auto load_splits = [&](int s0) {   // splits s0 .. s0+SU-1 of the RU rows (clamped: re-reads the last)
#pragma unroll
      for (int u = 0; u < SU; ++u) {
        const int sp = min(s0 + u, nsp - 1);
        const int64_t row0 = (slot0 + sp * slot_stride) * BM;
#pragma unroll
        for (int k = 0; k < RU; ++k) {
          ml[u][k] = __ldcg(reinterpret_cast<const float2*>(p.part_ml + (row0 + rr[k]) * 2));
#pragma unroll
          for (int e4 = 0; e4 < NV; ++e4) {
            const int pos = ((lane * NV + e4) ^ (rr[k] & 31)) << 2;   // in floats
            x[u][k][e4] = __ldcg(reinterpret_cast<const float4*>(p.part_o + (row0 + rr[k]) * HD + pos));
          }
        }
      }
    };
    load_splits(0);   // in flight while the row maxima are found
    float M[RU], L[RU];
#pragma unroll
    for (int k = 0; k < RU; ++k) {
      float m = -INFINITY;
      for (int sp = lane; sp < nsp; sp += 32)
        m = fmaxf(m, __ldcg(p.part_ml + ((slot0 + sp * slot_stride) * BM + rr[k]) * 2));
      M[k] = m;
      L[k] = 0.f;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
      for (int k = 0; k < RU; ++k) M[k] = fmaxf(M[k], __shfl_xor_sync(0xffffffffu, M[k], o));
    }
    float4 acc[RU][NV];
#pragma unroll
    for (int k = 0; k < RU; ++k)
#pragma unroll
      for (int e4 = 0; e4 < NV; ++e4) acc[k][e4] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s0 = 0; s0 < nsp; s0 += SU) {
      if (s0 > 0) load_splits(s0);
#pragma unroll
      for (int u = 0; u < SU; ++u) {
        if (s0 + u >= nsp) break;
#pragma unroll
        for (int k = 0; k < RU; ++k) {
          const float w = ml[u][k].x == -INFINITY ? 0.f : fast_exp2(ml[u][k].x - M[k]);
          L[k] += w * ml[u][k].y;
#pragma unroll
          for (int e4 = 0; e4 < NV; ++e4) {
            acc[k][e4].x += w * x[u][k][e4].x;
            acc[k][e4].y += w * x[u][k][e4].y;
            acc[k][e4].z += w * x[u][k][e4].z;
            acc[k][e4].w += w * x[u][k][e4].w;
          }
        }
      }
    }
#pragma unroll
    for (int k = 0; k < RU; ++k) {
      if (r0 + k >= row_hi) break;
      const float invd = L[k] > 0.f ? 1.f / L[k] : 0.f;
      const int pkr = pk0 + r0 + k;
      const int tlr = pkr / G, gr = pkr - tlr * G;
      const int64_t oi =
          (static_cast<int64_t>(q_begin + tlr) * p.hq + static_cast<int64_t>(h) * G + gr) * HD +
          lane * VPL;
      alignas(16) T vals[VPL];
#pragma unroll
      for (int e4 = 0; e4 < NV; ++e4) {
        const float f[4] = {acc[k][e4].x * invd, acc[k][e4].y * invd, acc[k][e4].z * invd,
                            acc[k][e4].w * invd};
#pragma unroll
        for (int e = 0; e < 4; ++e)
          vals[4 * e4 + e] =
              gate ? apply_gate<T>(f[e], gate[oi + 4 * e4 + e]) : MmaOp<T>::from_float(f[e]);
      }
      if constexpr (VPL == 4)
        *reinterpret_cast<uint2*>(out + oi) = *reinterpret_cast<const uint2*>(vals);
      else
        *reinterpret_cast<uint4*>(out + oi) = *reinterpret_cast<const uint4*>(vals);
    }
  }
}

template <typename T, int BN, int NSUB, int HD = 128, bool PAGED = false>
__global__ void __launch_bounds__(TcShape<NSUB, HD, PAGED>::kThreads,
                                  TcShape<NSUB, HD, PAGED>::kMinCtasForRegs)
    prefill_tc_kernel(const PrefillParams p, const __grid_constant__ CUtensorMap tm_k,
                      const __grid_constant__ CUtensorMap tm_v,
                      const __grid_constant__ CUtensorMap tm_q) {
  static_assert(BN == 64 || BN == 128, "key tile of 64 or 128 tokens");
  static_assert(NSUB == 2 || BN == 64, "the one-sub-tile shape has TMEM for 64-column score tiles only");
  using Shape = TcShape<NSUB, HD, PAGED>;
  constexpr int kTcQTileBytes = Shape::kQTileBytes;
  constexpr int CPR = HD / 8;                          // 16-byte chunks of a token row
  constexpr int BM = Shape::kBM, SUB = kTcSub;
  constexpr int kTcThreads = Shape::kThreads;
  constexpr int kMmaWarp = Shape::kMmaWarp;
  constexpr int kTcProducerWarp0 = Shape::kProducerWarp0;
  constexpr int NPROD = (Shape::kWarps - kTcProducerWarp0) * 32;  // producer threads
  constexpr int PROWS = NPROD / CPR;                    // token rows covered by one pass of the producers
  constexpr int LA = BN == 64 ? 2 : 1;        // key tiles S runs ahead of PV (= S buffers per sub-tile)
  constexpr int kTcKvTileBytes = BN * Shape::kRowBytes;
  constexpr int kTcBufs = Shape::kRingBytes / kTcKvTileBytes;
  constexpr uint32_t kOCol = NSUB * 128;      // first TMEM column of the O accumulators

  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ TcBarriers bars;
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;
  __shared__ int s_slots[(LA + 1) * BN];  // slot ids of the key tiles being copied / next to copy

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int G = p.group;
#ifdef MSGL_TRACE
  if (tid == 0) {
    MSGL_TR(0, trace_wall());
    MSGL_TR(1, clock64());
    MSGL_TR(2, trace_smid());
  }
#endif

  // ---- barriers and tensor memory first: neither depends on which work item this CTA gets
  const uint32_t bar_q = smem_u32(&bars.q_full);
  auto bar_full = [&](int bf) { return smem_u32(&bars.full[bf]); };
  auto bar_empty = [&](int bf) { return smem_u32(&bars.empty[bf]); };
  auto bar_sf = [&](int i, int sb) { return smem_u32(&bars.s_full[i][sb]); };
  auto bar_pf = [&](int i, int sb) { return smem_u32(&bars.p_full[i][sb]); };
  auto bar_pv = [&](int i, int sb) { return smem_u32(&bars.pv_done[i][sb]); };
  // Q arrives as TMA boxes when the caller could describe it (query heads per KV head a power
  // of two), else as 16-byte copies by the producer threads
  const bool q_tma = PAGED && p.q_tma != 0;

  if (tid == 0) {
    s_abort = 0;
    mbar_init(bar_q, q_tma ? 1 : NPROD);
    mbar_init(smem_u32(&bars.idx_sync), NPROD);
    for (int bf = 0; bf < kTcBufs; ++bf) {
      // PAGED: the 32 lanes of the copying warp (their cp.async arrivals) + the arrival that
      // announces the TMA bytes
      mbar_init(bar_full(bf), PAGED ? 33 : NPROD);
      mbar_init(bar_empty(bf), 1);
    }
    for (int i = 0; i < NSUB; ++i) {
      mbar_init(smem_u32(&bars.stage[i]), SUB / 32);     // one arrival per warp of the group
      mbar_init(bar_sf(i, 0), 1);
      mbar_init(bar_sf(i, 1), 1);
      mbar_init(bar_pf(i, 0), SUB / 32);
      mbar_init(bar_pf(i, 1), SUB / 32);
      mbar_init(bar_pv(i, 0), 1);
      mbar_init(bar_pv(i, 1), 1);
    }
    fence_mbar_init();
  }
  if (warp == kMmaWarp) {
    tmem_alloc(smem_u32(&s_tmem_base), Shape::kTmemCols);
    tmem_relinquish();
  }

  ItemCoord it;
  const bool have_item =
      find_item<kTcThreads>(p, static_cast<int>(blockIdx.x), BM, reinterpret_cast<int*>(smem_raw), it);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (!have_item) {  // block-uniform: a launch rank past the last item
    if (warp == kMmaWarp) tmem_dealloc(s_tmem_base, Shape::kTmemCols);
    return;
  }
  const int h = it.h;
  const SeqShape sq = load_seq_shape(p, it.b, BM);
  const int qt = it.qt, split = it.split;
  const int slot_item = it.base + qt * sq.nsplit + split;   // where this item's kv-split partial goes
  if (PAGED && it.first && tid == 0 && p.status) {
    // a length that is negative or exceeds the sequence's pages was clamped: report it
    const int64_t cap = static_cast<int64_t>(p.page_indptr[it.b + 1] - p.page_indptr[it.b]) * p.page_size;
    const int len = p.kv_lens[it.b];
    if (len < 0 || len > cap) atomicExch(p.status, 2);
  }

  // ---- geometry of the CTA's rows and of each sub-tile
  const int pk0 = qt * BM;
  const int rows_valid = min(BM, sq.tq * G - pk0);              // >= 1
  const int nsub = (NSUB == 2 && rows_valid > SUB) ? 2 : 1;
  const int tok_first = pk0 / G;
  const int s_lo = p.kv_chunk > 0 ? sq.lo + split * p.kv_chunk : 0;
  const int s_hi = p.kv_chunk > 0 ? sq.lo + (split + 1) * p.kv_chunk : 0x7fffffff;  // exclusive
  int kv_lo = p.window > 0 ? max(0, sq.prefix + tok_first - p.window + 1) : 0;
  kv_lo = max(kv_lo, s_lo);
  kv_lo = (kv_lo / BN) * BN;
  int ntiles_sub[2] = {0, 0};
#pragma unroll
  for (int i = 0; i < NSUB; ++i) {
    const int last_row = min(rows_valid, (i + 1) * SUB) - 1;     // last valid row of the sub-tile
    const int tok_last = (pk0 + last_row) / G;
    int hi = p.is_cross ? sq.L : min(sq.L, sq.prefix + tok_last + 1);
    hi = min(hi, s_hi);
    ntiles_sub[i] = (i < nsub && hi > kv_lo) ? ceil_div(hi - kv_lo, BN) : 0;
  }
  const int ntiles = max(ntiles_sub[0], ntiles_sub[1]);
  // keys past kv_hi_load are never fetched (zero rows in the tile)
  int kv_hi_load = p.is_cross ? sq.L : min(sq.L, sq.prefix + (pk0 + rows_valid - 1) / G + 1);
  kv_hi_load = min(kv_hi_load, s_hi);

  // ---- shared-memory carve-up (1024-byte aligned tiles)
  const uint32_t smem0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t q_smem = smem0;                                   // 2 sub-tiles
  const uint32_t ring = smem0 + NSUB * kTcQTileBytes;              // kTcBufs K/V tiles

  const uint32_t tmem = s_tmem_base;
  volatile int* abort_flag = &s_abort;
#ifdef MSGL_TRACE
  if (tid == 0) {
    MSGL_TR(3, clock64());          // set-up done
    MSGL_TR(4, ntiles);
  }
#endif

  // Register budget: the softmax warps hold a whole score row per thread, the others need
  // little.  Each warpgroup executes one and the same setmaxnreg instruction.
  if (warp >= kMmaWarp) {
  if constexpr (Shape::kRebalanceRegs) reg_dec<56>();
  if (warp >= kTcProducerWarp0) {
    // =========================================================== producers
    const int ptid = tid - kTcProducerWarp0 * 32;  // 0..NPROD-1
    const int chunk = ptid % CPR;          // 16-byte chunk of a token row
    const int rsub = ptid / CPR;           // row inside a pass of PROWS rows
    const T* __restrict__ q = static_cast<const T*>(p.q);
    const unsigned char* __restrict__ kbase = static_cast<const unsigned char*>(p.k_cache);
    const unsigned char* __restrict__ vbase = static_cast<const unsigned char*>(p.v_cache);
    const int64_t slot_stride = static_cast<int64_t>(p.hkv) * (HD * 2);
    const int64_t head_off = static_cast<int64_t>(h) * (HD * 2);

    if (q_tma) {
      // Q: one box per sub-tile and 64-element column block.  The tensor map is
      // (head_dim, query heads, tokens) with a box of 64 x G x 128/G, so the rows land in
      // packed order (token-major, the G heads of this KV head inside a token).  Rows past the
      // sequence's last query token hold a neighbour's rows (or zeros past the last token of
      // the batch); they are computed on and never written out.
      if (warp == kTcProducerWarp0 && lane == 0) {
        prefetch_tensormap(&tm_q);
        mbar_arrive_expect_tx(bar_q, nsub * kTcQTileBytes);
        for (int i = 0; i < nsub; ++i)
#pragma unroll
          for (int c = 0; c < HD / 64; ++c)
            tma_load_3d(q_smem + i * kTcQTileBytes + c * (SUB * 128), &tm_q, c * 64, h * G,
                        sq.q_begin + tok_first + i * (SUB / G), bar_q);
      }
    } else {
      // Q: rows_valid packed rows, the rest zero
      for (int i = 0; i < (BM + PROWS - 1) / PROWS; ++i) {
        const int row = i * PROWS + rsub;  // 0..255
        if (row >= nsub * SUB) break;
        const int pk = pk0 + row;
        const int tl = pk / G, g = pk - tl * G;
        const bool ok = row < rows_valid;
        const int64_t off =
            ok ? ((static_cast<int64_t>(sq.q_begin + tl) * p.hq + static_cast<int64_t>(h) * G + g) * HD)
               : 0;
        cp_async_16(q_smem + (row >> 7) * kTcQTileBytes + tc_tile_offset<128>(row & 127, chunk),
                    reinterpret_cast<const unsigned char*>(q + off) + chunk * 16, ok ? 16 : 0);
      }
      cp_async_mbar_arrive(bar_q);
    }

    bool alive = true;
    if constexpr (PAGED) {
      // ------------------------------------------------ page-granular: TMA boxes from the page ids
      if (warp == kTcProducerWarp0) {
        constexpr int PPT = BN / kTmaBoxRows;            // boxes (= lanes at work) per tile
        constexpr int NQ = HD / 64;                      // 128-byte column blocks of a token row
        constexpr uint32_t kBoxBytes = kTmaBoxRows * 128;
        const int32_t* __restrict__ pages = p.page_indices + sq.kv_begin;
        const int x0 = h * HD;
        if (lane == 0) {
          prefetch_tensormap(&tm_k);
          prefetch_tensormap(&tm_v);
        }
        // Lane i < PPT owns box i of a tile (tokens [16 i, 16 i + 16) of the tile): y = its first
        // pool row, n = how many of its rows belong to the sequence (16: a TMA box; fewer: rows
        // by cp.async, the rest zero-filled; 0: all zeros).
        auto fetch_box = [&](int tile, int& y, int& n) {
          y = 0;
          n = 0;
          const int t0 = kv_lo + tile * BN + lane * kTmaBoxRows;
          if (lane < PPT && tile < ntiles && t0 < kv_hi_load) {
            const int pg = __ldg(pages + t0 / p.page_size);
            const int64_t row0 = static_cast<int64_t>(pg) * p.page_size + t0 % p.page_size;
            const int nv = min(kTmaBoxRows, sq.L - t0);
            if (pg < 0 || row0 + nv > p.num_slots) {
              if (p.status) atomicExch(p.status, 2);   // page outside the pool: rows read as zeros
            } else {
              y = static_cast<int>(row0);
              n = nv;
            }
          }
        };
        int issued_seq = -1;   // ring sequence number of the last tile whose copies were issued
        auto produce = [&](int seq, const CUtensorMap* tm, const unsigned char* src_base, int y, int n) {
          const int bf = seq % kTcBufs;
          alive = mbar_wait_warp(bar_empty(bf), ((seq / kTcBufs) & 1) ^ 1, abort_flag);
          if (!alive) return;
          const uint32_t dst = ring + bf * kTcKvTileBytes;
          const uint32_t bar = bar_full(bf);
          const bool full = n == kTmaBoxRows;
          const uint32_t full_mask = __ballot_sync(0xffffffffu, full);
          if (lane == 0) mbar_arrive_expect_tx(bar, __popc(full_mask) * (kTmaBoxRows * HD * 2));
          __syncwarp();
          if (full) {
#pragma unroll
            for (int c = 0; c < NQ; ++c)
              tma_load_2d(dst + c * (BN * 128) + lane * kBoxBytes, tm, x0 + c * 64, y, bar);
          }
          uint32_t rest = ~full_mask & ((1u << PPT) - 1u);
          while (rest) {   // warp-uniform
            const int i = __ffs(rest) - 1;
            rest &= rest - 1;
            const int yi = __shfl_sync(0xffffffffu, y, i), ni = __shfl_sync(0xffffffffu, n, i);
#pragma unroll
            for (int k = 0; k < kTmaBoxRows * CPR / 32; ++k) {
              const int e = k * 32 + lane;
              const int row = e / CPR, chunk = e % CPR;
              const bool ok = row < ni;
              const int64_t off =
                  (ok ? static_cast<int64_t>(yi + row) * slot_stride + head_off : 0) + chunk * 16;
              cp_async_16(dst + tc_tile_offset<BN>(i * kTmaBoxRows + row, chunk), src_base + off,
                          ok ? 16 : 0);
            }
          }
          cp_async_mbar_arrive(bar);
          issued_seq = seq;
        };
        // window of the boxes of tiles j .. j+LA (tile j: V next, tile j+LA: K next)
        int wy[LA + 1], wn[LA + 1];
#pragma unroll
        for (int t = 0; t <= LA; ++t) fetch_box(t, wy[t], wn[t]);
#pragma unroll
        for (int t = 0; t < LA; ++t)
          if (t < ntiles && alive) produce(ring_seq_k<LA>(t), &tm_k, kbase, wy[t], wn[t]);
#pragma unroll 1
        for (int j = 0; j < ntiles && alive; ++j) {
          int ny, nn;
          fetch_box(j + LA + 1, ny, nn);   // in flight while this step's copies are issued
          produce(ring_seq_v<LA>(j), &tm_v, vbase, wy[0], wn[0]);
          if (!alive) break;
          if (j + LA < ntiles) {
            produce(ring_seq_k<LA>(j + LA), &tm_k, kbase, wy[LA], wn[LA]);
            if (!alive) break;
          }
#pragma unroll
          for (int t = 0; t < LA; ++t) {
            wy[t] = wy[t + 1];
            wn[t] = wn[t + 1];
          }
          wy[LA] = ny;
          wn[LA] = nn;
        }
        if (!alive) {
          // gave up: let the bulk copies still in flight (at most a ring's worth) land before the
          // CTA's shared memory goes away; bounded
          const long long t0 = clock64();
          for (int sq_i = max(0, issued_seq - kTcBufs + 1); sq_i <= issued_seq; ++sq_i) {
            while (!mbar_try_wait(bar_full(sq_i % kTcBufs), (sq_i / kTcBufs) & 1) &&
                   clock64() - t0 < 2000000LL) {
            }
          }
        }
      }
    } else {
      constexpr int RPT = (BN + PROWS - 1) / PROWS;  // passes over a tile
      // Slot ids are staged in shared memory: thread r fetches the id of row r of a tile (one
      // coalesced load per tile, two tiles ahead of its use), out-of-range ids are reported
      // once and stored as -1 (row treated as absent).  Tile t lives in s_slots[(t % (LA+1)) * BN ..].
      const int32_t* __restrict__ idx = p.kv_indices + sq.kv_begin;
      auto fetch_slot = [&](int tile) -> int {
        const int t = kv_lo + tile * BN + ptid;
        return (ptid < BN && tile < ntiles && t < kv_hi_load) ? __ldg(idx + t) : -1;
      };
      auto stage_slot = [&](int tile, int slot) {
        if (ptid < BN) {
          if (slot < -1 || static_cast<int64_t>(slot) >= p.num_slots) {
            if (p.status) atomicExch(p.status, 2);
            slot = -1;
          }
          s_slots[(tile % (LA + 1)) * BN + ptid] = slot;
        }
      };
      uint32_t idx_phase = 0;
      const uint32_t bar_idx = smem_u32(&bars.idx_sync);
      auto producers_sync = [&]() {  // bounded barrier among the 128 producer threads
        mbar_arrive(bar_idx);
        alive = mbar_wait_warp(bar_idx, idx_phase, abort_flag);
        idx_phase ^= 1;
      };
      // copy one tile into the ring buffer of sequence number `seq`
      auto produce = [&](int seq, const unsigned char* src_base, int tile) {
        const int bf = seq % kTcBufs;
        alive = mbar_wait_warp(bar_empty(bf), ((seq / kTcBufs) & 1) ^ 1, abort_flag);
        if (!alive) return;
        const uint32_t dst = ring + bf * kTcKvTileBytes;
        const int* slots = s_slots + (tile % (LA + 1)) * BN;
  #pragma unroll
        for (int i = 0; i < RPT; ++i) {
          const int row = i * PROWS + rsub;
          if (BN % PROWS != 0 && row >= BN) break;
          const int slot = slots[row];
          const bool ok = slot >= 0;
          const int64_t off =
              (ok ? static_cast<int64_t>(slot) * slot_stride + head_off : 0) + chunk * 16;
          cp_async_16(dst + tc_tile_offset<BN>(row, chunk), src_base + off, ok ? 16 : 0);
        }
        cp_async_mbar_arrive(bar_full(bf));
      };
  #pragma unroll
      for (int t = 0; t <= LA; ++t) stage_slot(t, fetch_slot(t));
      producers_sync();
      for (int t = 0; t < LA && t < ntiles && alive; ++t) produce(ring_seq_k<LA>(t), kbase, t);
  #pragma unroll 1
      for (int j = 0; j < ntiles && alive; ++j) {
        const int next_slot = fetch_slot(j + LA + 1);  // in flight while this tile's copies are issued
        produce(ring_seq_v<LA>(j), vbase, j);
        if (!alive) break;
        if (j + LA < ntiles) {
          produce(ring_seq_k<LA>(j + LA), kbase, j + LA);
          if (!alive) break;
        }
        producers_sync();               // every producer is done reading tile j's ids
        if (!alive) break;
        stage_slot(j + LA + 1, next_slot);  // reuses tile j's place
        producers_sync();
      }
    }
    cp_async_wait<0>();
    if (!alive && p.status && ptid == 0) atomicExch(p.status, 1);
  } else if (warp == kMmaWarp) {
    // =========================================================== MMA issuer
    {
    const uint32_t idesc_s = idesc_m128<T>(BN, 0);
    const uint32_t idesc_pv = idesc_m128<T>(HD, 1);
    bool alive = true;
    // Descriptors are computed by the whole (converged) warp so that they stay
    // warp-uniform values; only the elected lane issues the instructions.
    const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem, 0);
    const uint64_t desc_hi_k = smem_desc_sw128(0, 16, 1024);                 // Q / K: K-major
    const uint64_t desc_hi_v = smem_desc_sw128(0, BN * 128, 1024);           // V: MN-major
    // The MMAs of one step (PV of tile t_pv and/or S of tile t_s, sub-tile i) are issued by
    // one elected lane in one go, each group followed by its commit.
    auto issue_step = [&](int i, bool do_pv, int t_pv, int buf_v, bool do_s, int t_s, int buf_k) {
      const uint32_t vb = (ring + buf_v * kTcKvTileBytes) >> 4;
      const uint32_t o_tm = tmem_u + kOCol + i * HD;
      const uint32_t p_tm = tmem_u + i * 128 + (t_pv % LA) * BN;
      const uint32_t qa = (q_smem + i * kTcQTileBytes) >> 4;
      const uint32_t kb = (ring + buf_k * kTcKvTileBytes) >> 4;
      const uint32_t s_tm = tmem_u + i * 128 + (t_s % LA) * BN;
      const uint32_t bar_o = bar_pv(i, t_pv % LA);
      const uint32_t bar_s = bar_sf(i, t_s % LA);
      if (elect_one()) {
        if (do_pv) {
          // O_i (+)= P V_t : k-steps of 16 tokens; A = P from TMEM, B = V MN-major
#pragma unroll
          for (int ks = 0; ks < BN / 16; ++ks) {
            tc_mma_ts(o_tm, p_tm + ks * 8, desc_hi_v | (vb + ks * (2048 >> 4)), idesc_pv,
                      (t_pv == 0 && ks == 0) ? 0u : 1u);
          }
          tc_commit(bar_o);
        }
        if (do_s) {
          // S_i[t] = Q_i K_t^T : HD/16 k-steps of 16 elements; both operands K-major
#pragma unroll
          for (int ks = 0; ks < HD / 16; ++ks) {
            const uint32_t qoff = ((ks >> 2) * (128 * 128) + (ks & 3) * 32) >> 4;
            const uint32_t koff = ((ks >> 2) * (BN * 128) + (ks & 3) * 32) >> 4;
            tc_mma_ss(s_tm, desc_hi_k | (qa + qoff), desc_hi_k | (kb + koff), idesc_s,
                      ks > 0 ? 1u : 0u);
          }
          tc_commit(bar_s);
        }
      }
      __syncwarp();
    };
    // wait for ring item `seq`, make its bytes visible to the tensor pipe
    auto acquire = [&](int seq) {
      alive = mbar_wait_warp(bar_full(seq % kTcBufs), (seq / kTcBufs) & 1, abort_flag);
      if (alive) {
        fence_proxy_async_smem();
        tc_fence_after();
      }
    };
    if (ntiles > 0) {
      alive = mbar_wait_warp(bar_q, 0, abort_flag);
      for (int t = 0; t < LA && t < ntiles && alive; ++t) {
        const int sk = ring_seq_k<LA>(t);
        acquire(sk);
        if (!alive) break;
        for (int i = 0; i < nsub; ++i)
          issue_step(i, false, 0, 0, t < ntiles_sub[i], t, sk % kTcBufs);
        if (elect_one()) tc_commit(bar_empty(sk % kTcBufs));
        __syncwarp();
      }
    }
#pragma unroll 1
    for (int j = 0; j < ntiles && alive; ++j) {
      // Both tiles of this step are acquired before the wait for P: the hand-off
      // P -> PV -> next S of a sub-tile is the chain that bounds the kernel.
      const int sv = ring_seq_v<LA>(j), sk = ring_seq_k<LA>(j + LA);
      const bool have_k = j + LA < ntiles;
      acquire(sv);
      if (!alive) break;
      if (have_k) {
        acquire(sk);
        if (!alive) break;
      }
      for (int i = 0; i < nsub && alive; ++i) {
        const bool do_pv = j < ntiles_sub[i], do_s = j + LA < ntiles_sub[i];
        if (do_pv) {
          alive = mbar_wait_warp(bar_pf(i, j % LA), (j / LA) & 1, abort_flag);
          if (!alive) break;
          tc_fence_after();
        }
        if (do_pv || do_s) issue_step(i, do_pv, j, sv % kTcBufs, do_s, j + LA, sk % kTcBufs);
      }
      if (!alive) break;
      if (elect_one()) {
        tc_commit(bar_empty(sv % kTcBufs));
        if (have_k) tc_commit(bar_empty(sk % kTcBufs));
      }
      __syncwarp();
    }
    if (!alive && p.status && lane == 0) atomicExch(p.status, 1);
    }
  }
  } else {
    // =========================================================== softmax groups
    if constexpr (Shape::kRebalanceRegs) {
      if (NSUB == 2) reg_inc<200>(); else reg_inc<128>();
    }
    const int i = warp >> 2;                 // sub-tile
    const int r = tid & 127;                 // row inside the sub-tile == TMEM lane
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t s_tm = tmem + lane_base + i * 128;
    const uint32_t o_tm = tmem + lane_base + kOCol + i * HD;
    const int row = i * SUB + r;
    const int pk = pk0 + row;
    const int tl = pk / G;
    const bool valid = row < rows_valid;
    const int pos = sq.prefix + tl;
    const int vhi = min(p.is_cross ? sq.L - 1 : min(pos, sq.L - 1), s_hi - 1);
    const int vlo = max(p.window > 0 ? pos - p.window + 1 : 0, s_lo);
    const int my_tiles = ntiles_sub[i];
    float m_ref = -INFINITY, l = 0.f;
    bool alive = true;
    const bool sc_neg = !(p.scale_log2 > 0.f);
    const float sc = sc_neg ? 1.f : p.scale_log2;

#pragma unroll 1
    for (int j = 0; j < my_tiles; ++j) {
      const int sb = j % LA;
      alive = mbar_wait_warp(bar_sf(i, sb), (j / LA) & 1, abort_flag);
      if (!alive) break;
      tc_fence_after();
#ifdef MSGL_TRACE
      if (tid == 0 && j == 0) MSGL_TR(5, clock64());   // first scores ready
      if (tid == 0 && j == 8) MSGL_TR(9, clock64());   // ninth
#endif
      const int k0 = kv_lo + j * BN;
      const bool need_mask = !(k0 >= vlo && k0 + BN - 1 <= vhi);
      // ---- the score row of this tile into registers
      uint32_t v[BN];
      tmem_ld32_at<0>(s_tm + sb * BN, v);
      tmem_ld32_at<32>(s_tm + sb * BN + 32, v);
      if (BN == 128) {
        tmem_ld32_at<BN - 64>(s_tm + sb * BN + 64, v);
        tmem_ld32_at<BN - 32>(s_tm + sb * BN + 96, v);
      }
      tmem_wait_ld();
      reg_fence(v);
      if (sc_neg) {  // a non-positive scale: fold it into the scores so that max() commutes
#pragma unroll
        for (int e = 0; e < BN; ++e) v[e] = __float_as_uint(__uint_as_float(v[e]) * p.scale_log2);
      }
      if (need_mask) {
#pragma unroll
        for (int e = 0; e < BN; ++e) {
          const int kpos = k0 + e;
          if (!(kpos >= vlo && kpos <= vhi)) v[e] = 0xff800000u;  // -inf
        }
      }
      float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int e = 0; e < BN; e += 8) {
#pragma unroll
        for (int c = 0; c < 4; ++c)
          mx[c] = max3(mx[c], __uint_as_float(v[e + 2 * c]), __uint_as_float(v[e + 2 * c + 1]));
      }
      const float mt = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * sc;
      // ---- lazy rescale of the accumulator
      float alpha = 1.f;
      bool resc = false;
      if (mt > m_ref + 8.f) {
        if (m_ref != -INFINITY) {
          alpha = fast_exp2(m_ref - mt);
          resc = true;
        }
        m_ref = mt;
      }
      if (j > 0 && __any_sync(0xffffffffu, resc)) {
        alive = mbar_wait_warp(bar_pv(i, (j - 1) % LA), ((j - 1) / LA) & 1, abort_flag);
        if (!alive) break;
        tc_fence_after();
#pragma unroll 1
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t o[32];
          tmem_ld32(o_tm + c * 32, o);
          tmem_wait_ld();
          reg_fence(o);
#pragma unroll
          for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
          tmem_st32(o_tm + c * 32, o);
        }
        tmem_wait_st();
      }
      l *= alpha;
      const float nmu = (m_ref == -INFINITY) ? 0.f : -m_ref;
      // ---- P = exp2(s*scale - m_ref) as packed 16-bit pairs over the S columns
      // (scale-and-shift and the row sum run as packed two-float operations: the loop is
      // bounded by instruction issue next to the special-function unit)
      const uint64_t sc2 = pack_f32x2(sc, sc), nmu2 = pack_f32x2(nmu, nmu);
      uint64_t la = pack_f32x2(0.f, 0.f), lb = la;
#pragma unroll
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t pk16[16];
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          float x0, x1;
          unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(v[c * 32 + e]),
                                            __uint_as_float(v[c * 32 + e + 1])), sc2, nmu2), x0, x1);
          const float p0 = fast_exp2(x0);
          const float p1 = fast_exp2(x1);
          if (e & 2) lb = add_f32x2(lb, pack_f32x2(p0, p1));
          else la = add_f32x2(la, pack_f32x2(p0, p1));
          pk16[e >> 1] = MmaOp<T>::pack(p0, p1);
        }
        tmem_st16(s_tm + sb * BN + c * 16, pk16);  // P columns [16c, 16c+16) of this S buffer
      }
      {
        float l0, l1;
        unpack_f32x2(add_f32x2(la, lb), l0, l1);
        l += l0 + l1;
      }
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_pf(i, sb));
    }

#ifdef MSGL_TRACE
    if (tid == 0) MSGL_TR(6, clock64());               // last P handed over
#endif
    // ---- epilogue
    if (alive && my_tiles > 0) {
      alive = mbar_wait_warp(bar_pv(i, (my_tiles - 1) % LA), ((my_tiles - 1) / LA) & 1, abort_flag);
      if (alive) tc_fence_after();
    }
    if (alive) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      if (p.kv_chunk == 0 || sq.nsplit == 1) {
        // Each warp stages its 32 output rows (HD*2 bytes each) in the Q sub-tile's shared memory,
        // free once the last S MMA has completed, then writes them out as whole rows (two per
        // instruction at head_dim 128); chunk c of row r sits at chunk position c ^ (r & 15)
        // (conflict-free).
        constexpr int RB = HD * 2;
        unsigned char* stage = smem_raw + (smem0 - smem_u32(smem_raw)) + i * kTcQTileBytes;
#pragma unroll 1
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t v[32];
          if (my_tiles > 0) {
            tmem_ld32(o_tm + c * 32, v);
            tmem_wait_ld();
            reg_fence(v);
          } else {
#pragma unroll
            for (int e = 0; e < 32; ++e) v[e] = 0u;
          }
#pragma unroll
          for (int e = 0; e < 32; e += 8) {
            uint4 w;
            w.x = MmaOp<T>::pack(__uint_as_float(v[e]) * inv, __uint_as_float(v[e + 1]) * inv);
            w.y = MmaOp<T>::pack(__uint_as_float(v[e + 2]) * inv, __uint_as_float(v[e + 3]) * inv);
            w.z = MmaOp<T>::pack(__uint_as_float(v[e + 4]) * inv, __uint_as_float(v[e + 5]) * inv);
            w.w = MmaOp<T>::pack(__uint_as_float(v[e + 6]) * inv, __uint_as_float(v[e + 7]) * inv);
            const int chunk = c * 4 + (e >> 3);
            *reinterpret_cast<uint4*>(stage + r * RB + ((chunk ^ (r & 15)) << 4)) = w;
          }
        }
        __syncwarp();
        {
          const int wrow0 = (warp & 3) * 32;   // first row of this warp inside the sub-tile
          const int chunk = lane % CPR;
#pragma unroll 4
          for (int rr = lane / CPR; rr < 32; rr += 32 / CPR) {
            const int rloc = wrow0 + rr;
            const int prow = i * SUB + rloc;
            if (prow < rows_valid) {
              const int pkr = pk0 + prow;
              const int tlr = pkr / G, gr = pkr - tlr * G;
              T* dst = static_cast<T*>(p.out) +
                       (static_cast<int64_t>(sq.q_begin + tlr) * p.hq + static_cast<int64_t>(h) * G + gr) * HD;
              uint4 w =
                  *reinterpret_cast<const uint4*>(stage + rloc * RB + ((chunk ^ (rloc & 15)) << 4));
              if (p.gate) {
                const T* grow = static_cast<const T*>(p.gate) + (dst - static_cast<T*>(p.out));
                const uint4 gv = *reinterpret_cast<const uint4*>(
                    reinterpret_cast<const unsigned char*>(grow) + chunk * 16);
                T* wo = reinterpret_cast<T*>(&w);
                const T* wg = reinterpret_cast<const T*>(&gv);
#pragma unroll
                for (int e = 0; e < 8; ++e) wo[e] = apply_gate<T>(to_f32(wo[e]), wg[e]);
              }
              *reinterpret_cast<uint4*>(reinterpret_cast<unsigned char*>(dst) + chunk * 16) = w;
            }
          }
        }
      } else {
        // Unnormalised partial of this kv split (empty split: max = -inf, sum = 0).  (m, l) go
        // straight to scratch; the fp32 rows of O are staged, 64 rows at a time, in the
        // sub-tile's Q buffer (free: every S MMA of the sub-tile is done) and leave as ONE bulk
        // copy per 64 rows.  In the staging buffer (and so in scratch) the 16-byte chunk c of
        // row r sits at chunk position c ^ (r & 31): conflict-free for the row-per-thread
        // writes here and for the row-per-warp reads of the merge.
        const int64_t slot = static_cast<int64_t>(slot_item) * p.hkv + h;
        if (valid) {
          *reinterpret_cast<float2*>(p.part_ml + (slot * BM + row) * 2) =
              make_float2(my_tiles > 0 ? m_ref : -INFINITY, my_tiles > 0 ? l : 0.f);
        }
        constexpr int RBF = HD * 4;                       // bytes of an fp32 row
        const uint32_t stage_u = q_smem + i * kTcQTileBytes;   // 64 rows x RBF = one Q sub-tile
        unsigned char* stage = smem_raw + (stage_u - smem_u32(smem_raw));
        const int rows_sub = rows_valid - i * SUB;        // valid rows of this sub-tile (group-uniform)
        const uint32_t bar_st = smem_u32(&bars.stage[i]);
        uint32_t st_phase = 0;
        for (int hb = 0; hb < 2 && alive; ++hb) {
          if (rows_sub <= hb * 64) break;
          if ((r >> 6) == hb) {                           // warp-uniform
            const int rr = r & 63;
#pragma unroll 1
            for (int c = 0; c < HD / 32; ++c) {
              uint32_t v[32];
              if (my_tiles > 0) {
                tmem_ld32(o_tm + c * 32, v);
                tmem_wait_ld();
                reg_fence(v);
              } else {
#pragma unroll
                for (int e = 0; e < 32; ++e) v[e] = 0u;
              }
#pragma unroll
              for (int e = 0; e < 32; e += 4) {
                const int chunk = c * 8 + (e >> 2);
                *reinterpret_cast<uint4*>(stage + rr * RBF + ((chunk ^ (rr & 31)) << 4)) =
                    make_uint4(v[e], v[e + 1], v[e + 2], v[e + 3]);
              }
            }
            fence_proxy_async_smem();   // the rows are visible to the bulk copy
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_st);
          alive = mbar_wait_warp(bar_st, st_phase, abort_flag);
          st_phase ^= 1;
          if (!alive) break;
          if (r == hb * 64) {
            bulk_store(p.part_o + (slot * BM + i * SUB + hb * 64) * HD, stage_u, 64 * RBF);
            bulk_commit();
            bulk_wait_all();            // the copy has read the buffer and written scratch
            fence_proxy_async_all();
            __threadfence();            // ... device-wide, before this CTA's arrival is counted
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_st);
          alive = mbar_wait_warp(bar_st, st_phase, abort_flag);
          st_phase ^= 1;
        }
        __threadfence();                // (m, l) of this row
#ifdef MSGL_TRACE
        if (tid == 0) MSGL_TR(15, clock64());
#endif
      }
    }
    if (!alive && p.status && r == 0) atomicExch(p.status, 1);
#ifdef MSGL_TRACE
    if (tid == 0) MSGL_TR(7, clock64());               // output written
#endif
  }

  // ---- teardown: every role is past its last TMEM access
  tc_fence_before();
  __syncthreads();
#ifdef MSGL_TRACE
  if (tid == 0) {
    MSGL_TR(8, clock64());
    MSGL_TR(10, trace_wall());
  }
#endif
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem, Shape::kTmemCols);
  }

  // ---- kv splits: the CTA that arrives last at the unit's counter merges the partials
  // (out = sum_s 2^(m_s - M) O_s / sum_s 2^(m_s - M) l_s) and writes the output rows; no second
  // launch.  The counter goes back to zero for the next call.
  if (p.kv_chunk > 0 && sq.nsplit > 1 && p.tickets != nullptr) {
    __shared__ int s_last;
    const int nsp = sq.nsplit;
    const int64_t slot0 = static_cast<int64_t>(it.base + qt * nsp) * p.hkv + h;  // split s: slot0 + s * hkv
    if (tid == 0) {
      MSGL_TR(11, clock64());
      int* ticket = p.tickets + (it.qt_base + qt) * p.hkv + h;
      __threadfence();
      const int arrived = atomicAdd(ticket, 1);
      s_last = (arrived == nsp - 1) ? 1 : 0;
      if (s_last) *ticket = 0;
    }
    __syncthreads();
#ifdef MSGL_TRACE
    if (tid == 0) {
      MSGL_TR(12, clock64());
      MSGL_TR(13, s_last);
    }
#endif
    // (where the register pool was re-balanced only the softmax warps have the registers)
    constexpr int kMergers = Shape::kRebalanceRegs ? kMmaWarp : Shape::kWarps;
    if (s_last != 0 && warp < kMergers) {
      // the softmax warps merge (a function of its own: its registers do not weigh on the main loop)
      const MergeArgs ma{p.part_o, p.part_ml, p.out, p.gate, p.hq, p.group};
      // (rows x 2 splits in flight per lane: what the register cap of the main kernel holds)
      constexpr int kMergeRows = (!Shape::kRebalanceRegs && HD == 128) ? 4 : 2;
      merge_kv_splits<T, HD, kMergers, BM, kMergeRows, 2>(ma, nsp, slot0, p.hkv, 0, rows_valid,
                                                                    pk0, sq.q_begin, h);
#ifdef MSGL_TRACE
      if (tid == 0) MSGL_TR(14, clock64());
#endif
    }
  }
}

// Second launch of a split call whose units are too large for one CTA to merge: same grid as the
// attention kernel; the CTA that maps to split s of a unit merges the s-th slice of the unit's
// rows (gridDim.y CTAs share a slice), so the work is spread over as many SMs as the attention
// itself was, a row or two per warp.
constexpr int kMergeWarps = 8;
constexpr int kMergeSlices = 4;
template <typename T, int HD, int BM>
__global__ void __launch_bounds__(kMergeWarps * 32) prefill_merge_kernel(const PrefillParams p) {
  __shared__ int s_scratch[4 * kSortedBatchMax];
  grid_dependency_wait();   // the partials come from the attention kernel
  ItemCoord it;
  if (!find_item<kMergeWarps * 32>(p, static_cast<int>(blockIdx.x), BM, s_scratch, it)) return;
  const SeqShape sq = load_seq_shape(p, it.b, BM);
  const int nsp = sq.nsplit;
  if (nsp <= 1) return;     // an unsplit unit's rows were written by the attention kernel
  const int pk0 = it.qt * BM;
  const int rows_valid = min(BM, sq.tq * p.group - pk0);
  const int parts = nsp * static_cast<int>(gridDim.y);
  const int per = (rows_valid + parts - 1) / parts;
  const int row_lo = (it.split * static_cast<int>(gridDim.y) + static_cast<int>(blockIdx.y)) * per;
  const int row_hi = min(rows_valid, row_lo + per);
  if (row_lo >= row_hi) return;
  const int64_t slot0 = static_cast<int64_t>(it.base + it.qt * nsp) * p.hkv + it.h;
  const MergeArgs ma{p.part_o, p.part_ml, p.out, p.gate, p.hq, p.group};
  merge_kv_splits<T, HD, kMergeWarps, BM, 2, 4>(ma, nsp, slot0, p.hkv, row_lo, row_hi, pk0, sq.q_begin,
                                                 it.h);
}

}  // namespace msgl
