// C-ABI entry points of the B200 paged-attention library: argument
// validation (same rules and message prefixes as the reference host wrappers),
// scratch layout, launch configuration.  Declarations: include/msgl_b200.h.
#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>

#include "../../include/msgl_b200.h"
#include "decode_splitkv.cuh"
#include "prefill_tc.cuh"
#include "qk_norm_rope.cuh"

namespace {

thread_local std::string g_last_error;

int fail(int code, const std::string& msg) {
  g_last_error = msg;
  return code;
}

int cuda_fail(const char* op, cudaError_t e) {
  return fail(MSGL_CUDA_ERROR, std::string(op) + ": CUDA error: " + cudaGetErrorString(e));
}

// Head of every workspace: the device status word (first 256 bytes), then kTicketSlots arrival
// counters of split-KV pieces at a fixed place, so that a buffer re-used by calls of different
// shapes never finds anything but the zeros the kernels leave there.
constexpr size_t kTicketSlots = 16384;
constexpr size_t kStatusBytes = 256 + kTicketSlots * sizeof(int);

// Scratch of msgl_paged_decode_attention_static: lives in the library's image,
// so every GPU that loads the library holds these bytes until the process exits.
static __device__ __align__(256) unsigned char g_static_decode_scratch[MSGL_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
std::mutex g_static_mutex;
void* g_static_scratch_ptr[kMaxDevices] = {};  // device address of the array, per device

// Device address of the static scratch on the current device.  In host code the
// array's name is only a handle; the address a kernel can use comes from
// cudaGetSymbolAddress, asked once per device with that device current.
int static_scratch_for_current_device(void** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail("paged_decode_attention_static", e);
  if (dev < 0 || dev >= kMaxDevices)
    return fail(MSGL_BAD_ARG, "paged_decode_attention_static: device ordinal out of range");
  std::lock_guard<std::mutex> lock(g_static_mutex);
  if (g_static_scratch_ptr[dev] == nullptr) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_static_decode_scratch);
    if (e != cudaSuccess) return cuda_fail("paged_decode_attention_static", e);
    if (ptr == nullptr)
      return fail(MSGL_CUDA_ERROR, "paged_decode_attention_static: no device address for the scratch");
    g_static_scratch_ptr[dev] = ptr;
  }
  *out = g_static_scratch_ptr[dev];
  return MSGL_OK;
}

constexpr int kDecWarps = 4;
constexpr int kDecStages = 3;
constexpr int kDecCtaTokens = kDecWarps * msgl::kDecodeGroupTokens;

int sm_count_cached() {
  static thread_local int cached_dev = -1;
  static thread_local int cached_sms = 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -1;
  if (dev != cached_dev) {
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return -1;
    cached_dev = dev;
    cached_sms = sms;
  }
  return cached_sms;
}

template <typename K>
cudaError_t allow_smem(K kernel, int bytes) {
  return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
}

// ---- TMA tensor maps over a K or V pool (page-granular entries)
// The encoder is a driver-API function; it is looked up through the runtime, so the library
// needs no link against libcuda.
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn tensor_map_encoder() {
  static EncodeTiledFn fn = [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      f = nullptr;
    return reinterpret_cast<EncodeTiledFn>(f);
  }();
  return fn;
}

// 2-D map over a pool (num_slots rows of num_kv_heads * head_dim 16-bit elements): a box is
// 16 token rows x 64 elements (128 bytes) of one head, written to shared memory with the
// 128-byte swizzle, i.e. in the layout the tensor-core descriptors of the kernels expect.
// Rows outside the pool read as zeros.  The last map per (pointer, shape) is kept per thread.
bool make_pool_tensor_map(CUtensorMap* out, const void* base, int64_t num_slots, int num_kv_heads,
                          int head_dim, int dtype) {
  struct Cached {
    const void* base;
    int64_t num_slots;
    int hkv, hd, dtype;
    CUtensorMap map;
  };
  static thread_local Cached cache[4] = {};
  static thread_local int next = 0;
  for (const Cached& c : cache)
    if (c.base == base && c.num_slots == num_slots && c.hkv == num_kv_heads && c.hd == head_dim &&
        c.dtype == dtype && base != nullptr) {
      *out = c.map;
      return true;
    }
  EncodeTiledFn enc = tensor_map_encoder();
  if (!enc || num_slots <= 0 || reinterpret_cast<uintptr_t>(base) % 16 != 0) return false;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(num_kv_heads) * head_dim,
                              static_cast<cuuint64_t>(num_slots)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(num_kv_heads) * head_dim * 2};
  const cuuint32_t box[2] = {64, static_cast<cuuint32_t>(msgl::kTmaBoxRows)};
  const cuuint32_t elem_strides[2] = {1, 1};
  CUtensorMap m;
  const CUresult r = enc(&m, dtype == MSGL_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                      : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                         2, const_cast<void*>(base), dims, strides, box, elem_strides,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  cache[next] = Cached{base, num_slots, num_kv_heads, head_dim, dtype, m};
  next = (next + 1) % 4;
  *out = m;
  return true;
}

// 3-D map over the query tensor (tokens, query heads, head_dim): a box is 64 elements x the
// `group` heads of one KV head x 128 / group tokens, i.e. the 128 packed rows of a query
// sub-tile in the order the kernel numbers them.  Needs a group that divides 128.
bool make_query_tensor_map(CUtensorMap* out, const void* q, int total_q, int num_q_heads, int group,
                           int head_dim, int dtype) {
  EncodeTiledFn enc = tensor_map_encoder();
  if (!enc || total_q <= 0 || group <= 0 || 128 % group != 0 || num_q_heads % group != 0 ||
      reinterpret_cast<uintptr_t>(q) % 16 != 0)
    return false;
  const cuuint64_t dims[3] = {static_cast<cuuint64_t>(head_dim), static_cast<cuuint64_t>(num_q_heads),
                              static_cast<cuuint64_t>(total_q)};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(head_dim) * 2,
                                 static_cast<cuuint64_t>(num_q_heads) * head_dim * 2};
  const cuuint32_t box[3] = {64, static_cast<cuuint32_t>(group), static_cast<cuuint32_t>(128 / group)};
  const cuuint32_t elem_strides[3] = {1, 1, 1};
  const CUresult r = enc(out, dtype == MSGL_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                        : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                         3, const_cast<void*>(q), dims, strides, box, elem_strides,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// Launches `kernel` so that its CTAs may be scheduled while the previous kernel of the
// stream drains (programmatic dependent launch); the kernel itself waits for the previous
// kernel's memory with griddepcontrol.wait before it reads anything that kernel wrote.
template <typename P, typename K>
cudaError_t launch_dependent(K kernel, dim3 grid, dim3 block, cudaStream_t s, const P& params) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = 0;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, params);
}

// ---- prefill scheduling decision (shared by the workspace query and the launch)
struct PrefillPlan {
  int kv_chunk;        // 0 = no kv split
  int64_t items;       // grid.x
  size_t part_o_bytes, part_ml_bytes, plan_bytes;
  bool fused_merge;    // the CTA that arrives last at a unit merges it (else: a second launch)
};


// Query blocks that fill at most one 128-row sub-tile (verify, draft blocks) run the
// one-sub-tile shape (64-token key tiles, two CTAs per SM); longer chunks the two-sub-tile
// shape with 128-token key tiles.  head_dim 256 always runs the one-sub-tile shape (its
// output accumulator alone takes 256 of the 512 TMEM columns), one CTA per SM.
bool prefill_short_q(int max_len_extend, int group, int head_dim) {
  return head_dim == 256 || static_cast<int64_t>(max_len_extend) * group <= msgl::kTcSub;
}

PrefillPlan plan_prefill(int batch, int total_q, int64_t total_kv, int hq, int hkv, int head_dim,
                         int max_len_extend, int window, int sms) {
  // The key range is split only when the query tiles alone cannot give every CTA slot of the
  // GPU a CTA; then about two CTAs per slot are made.
  PrefillPlan pl{};
  const int G = hq / hkv;
  const bool short_q = prefill_short_q(max_len_extend, G, head_dim);
  const int BM = short_q ? msgl::TcShape<1>::kBM : msgl::TcShape<2>::kBM;
  const int slots = sms * (head_dim == 256 ? msgl::TcShape<1, 256>::kCtasPerSm
                           : short_q       ? msgl::TcShape<1>::kCtasPerSm
                                           : msgl::TcShape<2>::kCtasPerSm);
  int64_t qtiles = msgl::prefill_item_bound(batch, total_q, total_kv, G, BM, max_len_extend, 0);
  {  // the other upper bound on the number of query tiles: every sequence at the longest length
    const int64_t per_seq = (static_cast<int64_t>(max_len_extend) * G + BM - 1) / BM;
    if (per_seq * batch < qtiles) qtiles = per_seq * batch;
  }
  int64_t visible = total_kv;
  if (window > 0) {
    const int64_t w = static_cast<int64_t>(batch) * (static_cast<int64_t>(window) + max_len_extend);
    if (w < visible) visible = w;
  }
  pl.kv_chunk = 0;
  // Split the key range only when the query tiles fill at most half of the CTA slots: a
  // nearly full single wave beats more, shorter CTAs plus a merge pass.
  if (qtiles * hkv * 2 <= slots && qtiles * hkv <= msgl::kPrefillTickets && visible > 0) {
    // One wave: every (sequence, head, query tile) unit is cut into as many equal pieces as
    // the CTA slots allow for a sequence of average length.  Measured on the draft-block and
    // verify configurations and on the small-chunk points of the prefill grid (chunk x prefix
    // 128 x 32768: 9 pieces of 3712 keys 94 us against 121 us with 2048-key pieces; 256 x 8192:
    // 4 pieces 67 us against 83; 512 x 16384: 2 pieces 172 us against 231; 16 query tokens over
    // a 4096 window: 2 pieces of 2176 keys 88 us against 98 with 2048 + 2048 + 16): a second,
    // partial wave and the start-up of more CTAs cost more than the longer pieces.
    const int64_t pieces = slots / (qtiles * hkv);                 // >= 2 here
    int64_t chunk = (visible / batch + pieces - 1) / pieces;
    if (chunk < 1024) chunk = 1024;
    chunk = (chunk + 127) / 128 * 128;
    if (chunk < visible) pl.kv_chunk = static_cast<int>(chunk);
    // One CTA merges a unit at the pace of one SM's L2 port (about 17 GB/s measured with the
    // rows of the other splits in flight): fine for the draft-block and verify units (64 rows x 2
    // pieces x 512 B = 64 KB, a few us, and no second launch), not for a 256-row unit (chunk 512
    // in 2 pieces: 256 KB, 15 us; 128 query tokens over 32768 keys in 9 pieces: 1.2 MB, 70 us
    // against 4 us spread over the grid of a second launch).
    // (sized for a sequence of average length: the lengths themselves are device data)
    const int64_t rows = std::min<int64_t>(BM, static_cast<int64_t>(max_len_extend) * G);
    const int64_t pieces_used = (visible / batch + chunk - 1) / chunk;
    pl.fused_merge = pieces_used * rows * head_dim * 4 <= 64 * 1024;
  }
#ifdef MSGL_TRACE
  // development builds only: a key-range piece length to try instead of the policy's
  if (const char* env = std::getenv("MSGL_KV_CHUNK")) {
    const int forced = std::atoi(env);
    if (forced >= 0) pl.kv_chunk = forced / 128 * 128;
  }
#endif
  pl.items = msgl::prefill_item_bound(batch, total_q, total_kv, G, BM, max_len_extend, pl.kv_chunk);
  if (pl.kv_chunk > 0) {
    const size_t slots_n = static_cast<size_t>(pl.items) * hkv;
    pl.part_o_bytes = slots_n * BM * head_dim * sizeof(float);
    pl.part_ml_bytes = slots_n * BM * 2 * sizeof(float);
    pl.plan_bytes = 0;
  }
  return pl;
}

// The waiting pattern of the attention kernels on a barrier that nothing completes: two warps wait
// (bounded), the first to run out raises the CTA's abort flag, the other sees it and leaves too,
// the status word gets 1 and the kernel returns normally.
__global__ void bounded_wait_selftest_kernel(int* status, long long limit_cycles) {
  __shared__ uint64_t bar;
  __shared__ int s_abort;
  if (threadIdx.x == 0) {
    s_abort = 0;
    msgl::mbar_init(msgl::smem_u32(&bar), 1);
    msgl::fence_mbar_init();
  }
  __syncthreads();
  // the second warp gets a far longer limit: it must leave through the abort flag
  const long long limit = threadIdx.x < 32 ? limit_cycles : limit_cycles * 1000;
  const bool ok = msgl::mbar_wait_limit(msgl::smem_u32(&bar), 0, &s_abort, limit);
  const bool all_out = __all_sync(0xffffffffu, !ok);
  __syncthreads();
  if (threadIdx.x == 0) msgl::mbar_inval(msgl::smem_u32(&bar));
  if (all_out && (threadIdx.x & 31) == 0) atomicExch(status, 1);
}

// ---- small data-movement kernels
template <int VEC_BYTES>
__global__ void store_kv_kernel(unsigned char* __restrict__ kc, unsigned char* __restrict__ vc,
                                const int32_t* __restrict__ indices,
                                const unsigned char* __restrict__ k,
                                const unsigned char* __restrict__ v, int length, int vec_per_row,
                                int64_t cache_row_bytes, int64_t input_row_bytes,
                                int64_t num_slots, int* status) {
  using V = typename std::conditional<VEC_BYTES == 16, uint4, uint2>::type;
  const int64_t total = static_cast<int64_t>(length) * vec_per_row;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int r = static_cast<int>(i / vec_per_row);
    const int c = static_cast<int>(i - static_cast<int64_t>(r) * vec_per_row);
    const int slot = indices[r];
    if (slot < 0 || slot >= num_slots) {
      if (status) atomicExch(status, 2);
      continue;
    }
    const int64_t src = r * input_row_bytes + static_cast<int64_t>(c) * VEC_BYTES;
    const int64_t dst = slot * cache_row_bytes + static_cast<int64_t>(c) * VEC_BYTES;
    *reinterpret_cast<V*>(kc + dst) = *reinterpret_cast<const V*>(k + src);
    *reinterpret_cast<V*>(vc + dst) = *reinterpret_cast<const V*>(v + src);
  }
}

// Rows and columns of the table and the size of the output are checked: a table row id outside
// [0, num_rows), a length beyond num_cols or an output position beyond total_kv is skipped and
// reported (status word 2) instead of being dereferenced.
__global__ void gather_kv_indices_kernel(const int32_t* __restrict__ page_table,
                                         int64_t row_stride, const int32_t* __restrict__ table_idx,
                                         const int32_t* __restrict__ kv_indptr,
                                         int32_t* __restrict__ kv_indices, int batch,
                                         int64_t num_rows, int64_t num_cols, int64_t total_kv,
                                         int* status) {
  const int b = blockIdx.y;
  const int64_t begin = kv_indptr[b];
  int64_t len = static_cast<int64_t>(kv_indptr[b + 1]) - begin;
  const int64_t r = table_idx[b];
  bool bad = begin < 0 || len < 0 || r < 0 || r >= num_rows;
  if (!bad && (len > num_cols || begin + len > total_kv)) {
    len = max(static_cast<int64_t>(0), min(num_cols, total_kv - begin));
    if (status && threadIdx.x == 0 && blockIdx.x == 0) atomicExch(status, 2);
  }
  if (bad) {
    if (status && threadIdx.x == 0 && blockIdx.x == 0) atomicExch(status, 2);
    return;
  }
  const int32_t* row = page_table + r * row_stride;
  for (int64_t t = blockIdx.x * blockDim.x + threadIdx.x; t < len; t += gridDim.x * blockDim.x)
    kv_indices[begin + t] = row[t];
}

// All index arrays of a step in one launch.  `req` holds, for the batch's sequences in order,
// the new-token counts, the KV lengths and the page-table rows: [extend | kv | row], 3 * batch
// int32.  CTA (x, b) sums the lengths of the sequences in front of b (a block-wide reduction:
// batch^2 / 2 additions in total, nothing next to one K/V tile), CTA (0, b) writes b's entries
// of the pointer arrays, and all CTAs of b copy its slot ids / page ids and write its
// positions.  Everything is bounds-checked against the sizes the host allocated; a violation
// sets status word 2 and is skipped.
struct MetadataParams {
  const int32_t* req;
  const int32_t* page_table;
  int64_t row_stride, table_rows, table_cols;
  int batch, page_size, split_chunk, max_kv_splits;
  int64_t total_q, total_kv, total_pages;
  int32_t *qo_indptr, *kv_indptr, *prefix_lens, *num_kv_splits, *positions;
  int32_t *kv_indices;     // may be null
  int32_t *page_indptr, *page_indices;   // may be null (page_size 1)
  int* status;
};

__global__ void __launch_bounds__(256) build_metadata_kernel(const MetadataParams p) {
  __shared__ long long s_red[3][8];
  const int b = blockIdx.y, tid = threadIdx.x;
  const int32_t* ext = p.req;
  const int32_t* kvl = p.req + p.batch;
  const int32_t* rows = p.req + 2 * p.batch;
  long long q0 = 0, k0 = 0, g0 = 0;
  for (int i = tid; i < b; i += 256) {
    const int e = max(ext[i], 0), k = max(kvl[i], 0);
    q0 += e;
    k0 += k;
    g0 += (k + p.page_size - 1) / p.page_size;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    q0 += __shfl_xor_sync(0xffffffffu, q0, o);
    k0 += __shfl_xor_sync(0xffffffffu, k0, o);
    g0 += __shfl_xor_sync(0xffffffffu, g0, o);
  }
  if ((tid & 31) == 0) {
    s_red[0][tid >> 5] = q0;
    s_red[1][tid >> 5] = k0;
    s_red[2][tid >> 5] = g0;
  }
  __syncthreads();
  q0 = k0 = g0 = 0;
#pragma unroll
  for (int w = 0; w < 8; ++w) {
    q0 += s_red[0][w];
    k0 += s_red[1][w];
    g0 += s_red[2][w];
  }
  const int e = max(ext[b], 0), k = max(kvl[b], 0);
  const int npg = (k + p.page_size - 1) / p.page_size;
  const long long r = rows[b];
  bool bad = ext[b] < 0 || kvl[b] < 0 || e > k || r < 0 || r >= p.table_rows || k > p.table_cols ||
             q0 + e > p.total_q || k0 + k > p.total_kv || (p.page_indices && g0 + npg > p.total_pages);
  if (blockIdx.x == 0 && tid == 0) {
    p.qo_indptr[b] = static_cast<int32_t>(q0);
    p.kv_indptr[b] = static_cast<int32_t>(k0);
    if (p.page_indptr) p.page_indptr[b] = static_cast<int32_t>(g0);
    if (b == p.batch - 1) {
      p.qo_indptr[p.batch] = static_cast<int32_t>(q0 + e);
      p.kv_indptr[p.batch] = static_cast<int32_t>(k0 + k);
      if (p.page_indptr) p.page_indptr[p.batch] = static_cast<int32_t>(g0 + npg);
    }
    p.prefix_lens[b] = k - e;
    const int chunk = p.split_chunk > 0 ? p.split_chunk : 128;
    p.num_kv_splits[b] = min(p.max_kv_splits, max(1, (k + chunk - 1) / chunk));
    if (bad && p.status) atomicExch(p.status, 2);
  }
  if (bad) return;
  const int32_t* row = p.page_table + r * p.row_stride;
  const int stride = gridDim.x * 256;
  for (int t = blockIdx.x * 256 + tid; t < k; t += stride) {
    const int32_t slot = row[t];
    if (p.kv_indices) p.kv_indices[k0 + t] = slot;
    if (p.page_indices && t % p.page_size == 0) {
      if (slot < 0 || slot % p.page_size != 0) {
        if (p.status) atomicExch(p.status, 2);     // a sequence that does not start its pages on page boundaries
        p.page_indices[g0 + t / p.page_size] = -1;
      } else {
        p.page_indices[g0 + t / p.page_size] = slot / p.page_size;
      }
    }
  }
  for (int t = blockIdx.x * 256 + tid; t < e; t += stride) p.positions[q0 + t] = k - e + t;
}

// Page-granular index entries: kv_indptr = exclusive scan of the sequence lengths (one CTA),
// then one slot id per token, slot = page * page_size + offset inside the page.  A length that
// is negative or longer than the sequence's pages is reported in the status word and clamped.
__global__ void __launch_bounds__(1024) page_lens_scan_kernel(const int32_t* __restrict__ kv_lens,
                                                              const int32_t* __restrict__ page_indptr,
                                                              int batch, int page_size,
                                                              int32_t* __restrict__ kv_indptr,
                                                              int* status) {
  __shared__ int s_sum[1024];
  __shared__ int s_carry;
  const int tid = threadIdx.x;
  if (tid == 0) {
    s_carry = 0;
    kv_indptr[0] = 0;
  }
  __syncthreads();
  for (int base = 0; base < batch; base += 1024) {
    const int i = base + tid;
    int len = 0;
    if (i < batch) {
      len = kv_lens[i];
      const int64_t cap = static_cast<int64_t>(page_indptr[i + 1] - page_indptr[i]) * page_size;
      if (len < 0 || len > cap) {
        if (status) atomicExch(status, 2);
        len = len < 0 ? 0 : static_cast<int>(cap < 0 ? 0 : cap);
      }
    }
    s_sum[tid] = len;
    __syncthreads();
    for (int off = 1; off < 1024; off <<= 1) {
      const int v = tid >= off ? s_sum[tid - off] : 0;
      __syncthreads();
      s_sum[tid] += v;
      __syncthreads();
    }
    if (i < batch) kv_indptr[i + 1] = s_carry + s_sum[tid];
    __syncthreads();
    if (tid == 1023) s_carry += s_sum[1023];
    __syncthreads();
  }
}

// A page id whose slots would fall outside [0, num_slots) gives slot id -1 (the attention
// kernels read such a row as zeros and report it); the slot is computed in 64 bits so that a
// corrupt id cannot wrap into the pool.
__global__ void expand_page_indices_kernel(const int32_t* __restrict__ page_indptr,
                                           const int32_t* __restrict__ page_indices,
                                           const int32_t* __restrict__ kv_indptr, int page_size,
                                           int64_t total_pages, int64_t num_slots,
                                           int32_t* __restrict__ kv_indices, int* status) {
  const int b = blockIdx.y;
  const int begin = kv_indptr[b];
  const int len = kv_indptr[b + 1] - begin;
  const int64_t first = page_indptr[b];
  if (first < 0 || first > total_pages) {
    if (status && threadIdx.x == 0 && blockIdx.x == 0) atomicExch(status, 2);
    for (int t = blockIdx.x * blockDim.x + threadIdx.x; t < len; t += gridDim.x * blockDim.x)
      kv_indices[begin + t] = -1;
    return;
  }
  const int32_t* pages = page_indices + first;
  for (int t = blockIdx.x * blockDim.x + threadIdx.x; t < len; t += gridDim.x * blockDim.x) {
    const int pg = t / page_size;
    int64_t slot = -1;
    if (first + pg < total_pages) slot = static_cast<int64_t>(pages[pg]) * page_size + (t - pg * page_size);
    if (slot < 0 || slot >= num_slots) {
      if (status) atomicExch(status, 2);
      slot = -1;
    }
    kv_indices[begin + t] = static_cast<int32_t>(slot);
  }
}

template <typename T>
int launch_decode(const msgl::DecodeParams& p, int head_dim, cudaStream_t s, const CUtensorMap& tm_k,
                  const CUtensorMap& tm_v) {
  dim3 grid1(p.max_splits, p.hkv, p.batch);
  const bool paged = p.kv_lens != nullptr;
  auto launch = [&](auto k1, int smem) -> int {
    cudaError_t e = allow_smem(k1, smem);
    if (e != cudaSuccess) return cuda_fail("paged_decode_attention", e);
    k1<<<grid1, kDecWarps * 32, smem, s>>>(p, tm_k, tm_v);
    e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail("paged_decode_attention", e);
    return MSGL_OK;
  };
  // page-granular: the same ring plus the slack that puts it on a 1024-byte boundary
  if (head_dim == 128) {
    constexpr int smem = kDecWarps * kDecStages * 2 * msgl::kDecodeGroupTokens * 256;
    return paged ? launch(msgl::decode_partial_kernel<T, 128, kDecWarps, kDecStages, true>, smem + 1024)
                 : launch(msgl::decode_partial_kernel<T, 128, kDecWarps, kDecStages>, smem);
  }
  // head_dim 256: 512-byte token rows, 16 KB per stage
  constexpr int kStages256 = 3;   // 192 KB of the 227 KB: one CTA per SM, three 16-token groups in flight per warp
  constexpr int smem = kDecWarps * kStages256 * 2 * msgl::kDecodeGroupTokens * 512;
  return paged ? launch(msgl::decode_partial_kernel<T, 256, kDecWarps, kStages256, true>, smem + 1024)
               : launch(msgl::decode_partial_kernel<T, 256, kDecWarps, kStages256>, smem);
}

// Page-granular addressing of a call (null: per-token kv_indptr / kv_indices).
struct PageIndex {
  const int32_t* page_indptr;
  const int32_t* page_indices;
  const int32_t* kv_lens;
  int page_size;
};

}  // namespace

// Arrival counters of the decode op: one per (sequence, KV head).  They sit in the workspace
// header when there are at most kTicketSlots of them; a larger batch gets a region of its own
// behind the header, cleared by every call (the workspace query is not told the KV head
// count, so it sizes that region for the query heads).
static bool aligned16(const void* ptr) { return reinterpret_cast<uintptr_t>(ptr) % 16 == 0; }

static size_t decode_ticket_bytes(int batch, int num_q_heads) {
  const size_t n = static_cast<size_t>(batch) * num_q_heads;
  return n <= kTicketSlots ? 0 : (n * sizeof(int) + 255) / 256 * 256;
}

extern "C" {

int msgl_abi_version(void) { return MSGL_ABI_VERSION; }

const char* msgl_last_error_string(void) { return g_last_error.c_str(); }

int msgl_device_sm_count(void) { return sm_count_cached(); }

size_t msgl_decode_workspace_bytes(int batch, int num_q_heads, int head_dim, int max_kv_splits) {
  if (batch <= 0 || num_q_heads <= 0 || head_dim <= 0 || max_kv_splits <= 0) return kStatusBytes;
  const size_t rows = static_cast<size_t>(batch) * num_q_heads * max_kv_splits;
  return kStatusBytes + decode_ticket_bytes(batch, num_q_heads) + rows * head_dim * sizeof(float) +
         rows * sizeof(float);
}

static int decode_impl(const void* q, const void* k_cache, const void* v_cache,
                       const int32_t* kv_indptr, const int32_t* kv_indices,
                       const int32_t* num_kv_splits, const void* gate, void* out, void* workspace,
                       size_t workspace_bytes, int batch, int num_q_heads, int num_kv_heads,
                       int head_dim, int64_t num_slots, int dtype, float sm_scale,
                       int max_kv_splits, void* stream, const PageIndex* pages = nullptr) {
  const char* op = "paged_decode_attention: ";
  if (batch < 0 || num_q_heads <= 0 || num_kv_heads <= 0 || num_slots < 0)
    return fail(MSGL_BAD_SHAPE, std::string(op) + "q must be 3D (batch, num_q_heads, head_dim)");
  if (head_dim != 128 && head_dim != 256)
    return fail(MSGL_UNSUPPORTED_HEAD_DIM, std::string(op) + "head_dim must be 128 or 256");
  if (num_q_heads % num_kv_heads != 0)
    return fail(MSGL_BAD_GQA, std::string(op) + "num_q_heads must be a multiple of num_kv_heads");
  if (num_q_heads / num_kv_heads > 16)
    return fail(MSGL_BAD_GQA, std::string(op) + "only q_heads/kv_heads <= 16 is supported");
  if (dtype != MSGL_DTYPE_BF16 && dtype != MSGL_DTYPE_F16)
    return fail(MSGL_BAD_DTYPE, std::string(op) + "unsupported dtype, must be float16 or bfloat16");
  if (max_kv_splits < 1 || max_kv_splits > MSGL_MAX_KV_SPLITS)
    return fail(MSGL_BAD_ARG, std::string(op) + "max_kv_splits must be in [1, 128]");
  if (batch == 0) return MSGL_OK;
  if (batch > 65535 || num_kv_heads > 65535)
    return fail(MSGL_BAD_SHAPE, std::string(op) + "batch and num_kv_heads must be <= 65535");
  if (!q || !k_cache || !v_cache || !out || (!pages && (!kv_indptr || !kv_indices)))
    return fail(MSGL_BAD_ARG, std::string(op) + "null tensor pointer");
  if (!aligned16(q) || !aligned16(k_cache) || !aligned16(v_cache) || !aligned16(out) ||
      !aligned16(gate) || !aligned16(workspace))
    return fail(MSGL_BAD_ARG, std::string(op) + "q, the pools, out, gate and the workspace must be "
                                                "16-byte aligned");
  CUtensorMap tm_k, tm_v;
  std::memset(&tm_k, 0, sizeof(tm_k));
  std::memset(&tm_v, 0, sizeof(tm_v));
  if (pages && (!make_pool_tensor_map(&tm_k, k_cache, num_slots, num_kv_heads, head_dim, dtype) ||
                !make_pool_tensor_map(&tm_v, v_cache, num_slots, num_kv_heads, head_dim, dtype)))
    return fail(MSGL_CUDA_ERROR, std::string(op) + "cannot build the tensor maps of the K/V pool");
  const size_t need = msgl_decode_workspace_bytes(batch, num_q_heads, head_dim, max_kv_splits);
  if (!workspace || workspace_bytes < need)
    return fail(MSGL_BAD_ARG, std::string(op) + "workspace too small");

  msgl::DecodeParams p{};
  p.q = q;
  p.k_cache = k_cache;
  p.v_cache = v_cache;
  p.kv_indptr = kv_indptr;
  p.kv_indices = kv_indices;
  p.num_kv_splits = num_kv_splits;
  if (pages) {
    p.page_indptr = pages->page_indptr;
    p.page_indices = pages->page_indices;
    p.kv_lens = pages->kv_lens;
    p.page_size = pages->page_size;
  }
  p.out = out;
  p.gate = gate;
  unsigned char* ws = static_cast<unsigned char*>(workspace);
  p.status = reinterpret_cast<int*>(ws);
  const size_t own_tickets = decode_ticket_bytes(batch, num_q_heads);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (own_tickets == 0) {
    p.tickets = reinterpret_cast<int*>(ws + 256);
  } else {
    p.tickets = reinterpret_cast<int*>(ws + kStatusBytes);
    cudaError_t e = cudaMemsetAsync(p.tickets, 0, own_tickets, s);
    if (e != cudaSuccess) return cuda_fail("paged_decode_attention", e);
  }
  p.part_o = reinterpret_cast<float*>(ws + kStatusBytes + own_tickets);
  p.part_lse = p.part_o + static_cast<size_t>(batch) * num_q_heads * max_kv_splits * head_dim;
  p.batch = batch;
  p.hq = num_q_heads;
  p.hkv = num_kv_heads;
  p.group = num_q_heads / num_kv_heads;
  p.max_splits = max_kv_splits;
  p.num_slots = num_slots;
  p.scale_log2 = sm_scale * msgl::kLog2e;
  if (dtype == MSGL_DTYPE_BF16) return launch_decode<__nv_bfloat16>(p, head_dim, s, tm_k, tm_v);
  return launch_decode<__half>(p, head_dim, s, tm_k, tm_v);
}

int msgl_paged_decode_attention(const void* q, const void* k_cache, const void* v_cache,
                                const int32_t* kv_indptr, const int32_t* kv_indices,
                                const int32_t* num_kv_splits, void* out, void* workspace,
                                size_t workspace_bytes, int batch, int num_q_heads,
                                int num_kv_heads, int head_dim, int64_t num_slots, int dtype,
                                float sm_scale, int max_kv_splits, void* stream) {
  return decode_impl(q, k_cache, v_cache, kv_indptr, kv_indices, num_kv_splits, nullptr, out, workspace,
                     workspace_bytes, batch, num_q_heads, num_kv_heads, head_dim, num_slots, dtype,
                     sm_scale, max_kv_splits, stream);
}

int msgl_paged_decode_attention_gated(const void* q, const void* k_cache, const void* v_cache,
                                      const int32_t* kv_indptr, const int32_t* kv_indices,
                                      const int32_t* num_kv_splits, const void* gate, void* out,
                                      void* workspace, size_t workspace_bytes, int batch,
                                      int num_q_heads, int num_kv_heads, int head_dim,
                                      int64_t num_slots, int dtype, float sm_scale,
                                      int max_kv_splits, void* stream) {
  if (!gate && batch > 0) return fail(MSGL_BAD_ARG, "paged_decode_attention: null gate pointer");
  return decode_impl(q, k_cache, v_cache, kv_indptr, kv_indices, num_kv_splits, gate, out, workspace,
                     workspace_bytes, batch, num_q_heads, num_kv_heads, head_dim, num_slots, dtype,
                     sm_scale, max_kv_splits, stream);
}

int msgl_paged_decode_attention_static(const void* q, const void* k_cache, const void* v_cache,
                                       const int32_t* kv_indptr, const int32_t* kv_indices,
                                       const int32_t* num_kv_splits, void* out, int batch,
                                       int num_q_heads, int num_kv_heads, int head_dim,
                                       int64_t num_slots, int dtype, float sm_scale,
                                       int max_kv_splits, void* stream) {
  // Size check first: it needs no device and must fail clearly.
  if (batch > 0 && num_q_heads > 0 && head_dim > 0 && max_kv_splits > 0) {
    const size_t need = msgl_decode_workspace_bytes(batch, num_q_heads, head_dim, max_kv_splits);
    if (need > static_cast<size_t>(MSGL_STATIC_SCRATCH_BYTES))
      return fail(MSGL_BAD_ARG,
                  "paged_decode_attention_static: needs " + std::to_string(need) +
                      " bytes of scratch, the built-in array holds " +
                      std::to_string(static_cast<size_t>(MSGL_STATIC_SCRATCH_BYTES)) +
                      "; lower batch * num_q_heads * max_kv_splits or use "
                      "msgl_paged_decode_attention with a caller-supplied workspace");
  }
  if (batch == 0) return MSGL_OK;
  void* scratch = nullptr;
  const int rc = static_scratch_for_current_device(&scratch);
  if (rc != MSGL_OK) return rc;
  // What has to start at zero does: the array is zero when the library is loaded, the arrival
  // counters behind the status word are put back to zero by the CTA that merges, every partial
  // and log-sum-exp that a merge reads is written earlier in the same call, and the status
  // word at the head is sticky by design.
  return msgl_paged_decode_attention(q, k_cache, v_cache, kv_indptr, kv_indices, num_kv_splits, out,
                                     scratch, MSGL_STATIC_SCRATCH_BYTES, batch, num_q_heads,
                                     num_kv_heads, head_dim, num_slots, dtype, sm_scale,
                                     max_kv_splits, stream);
}

int msgl_read_status(void* workspace, int clear, int* status_out, void* stream) {
  void* word = workspace;
  if (!word) {
    const int rc = static_scratch_for_current_device(&word);
    if (rc != MSGL_OK) return rc;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int value = 0;
  cudaError_t e = cudaMemcpyAsync(&value, word, sizeof(int), cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess && clear) e = cudaMemsetAsync(word, 0, sizeof(int), s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  if (e != cudaSuccess) return cuda_fail("read_status", e);
  if (status_out) *status_out = value;
  if (value == 0) return MSGL_OK;
  return fail(MSGL_DEVICE_STATUS,
              value == 1 ? "read_status: a bounded wait inside a kernel ran out (results are not valid)"
              : value == 2
                  ? "read_status: a slot or page id outside the pool, or a length beyond a sequence's "
                    "pages, was met (those rows were read as zeros)"
                  : "read_status: unknown device status " + std::to_string(value));
}

int msgl_selftest_bounded_wait(void* workspace, int limit_us, void* stream) {
  if (!workspace) return fail(MSGL_BAD_ARG, "selftest_bounded_wait: null workspace");
  if (limit_us < 1 || limit_us > 100000)
    return fail(MSGL_BAD_ARG, "selftest_bounded_wait: limit_us must be in [1, 100000]");
  // about 2 cycles per nanosecond: the wait gives up after limit_us at the latest
  bounded_wait_selftest_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<int*>(workspace), static_cast<long long>(limit_us) * 2000);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail("selftest_bounded_wait", e);
  return MSGL_OK;
}

size_t msgl_prefill_workspace_bytes(int batch, int total_q, int64_t total_kv, int num_q_heads,
                                    int num_kv_heads, int head_dim, int max_len_extend,
                                    int sliding_window_size) {
  if (batch <= 0 || total_q <= 0 || num_q_heads <= 0 || num_kv_heads <= 0 ||
      num_q_heads % num_kv_heads != 0)
    return kStatusBytes;
  const int sms = sm_count_cached();
  const PrefillPlan pl = plan_prefill(batch, total_q, total_kv, num_q_heads, num_kv_heads,
                                      head_dim, max_len_extend, sliding_window_size,
                                      sms > 0 ? sms : 148);
  return kStatusBytes + pl.plan_bytes + pl.part_ml_bytes + pl.part_o_bytes;
}

int msgl_prefill_launch_count(int batch, int total_q, int64_t total_kv, int num_q_heads,
                              int num_kv_heads, int head_dim, int max_len_extend,
                              int sliding_window_size, int page_granular) {
  if (batch <= 0 || total_q <= 0 || num_q_heads <= 0 || num_kv_heads <= 0 ||
      num_q_heads % num_kv_heads != 0)
    return 1;
  const int sms = sm_count_cached();
  (void)page_granular;   // both index granularities split alike
  const PrefillPlan pl = plan_prefill(batch, total_q, total_kv, num_q_heads, num_kv_heads,
                                      head_dim, max_len_extend, sliding_window_size,
                                      sms > 0 ? sms : 148);
  return (pl.kv_chunk > 0 && !pl.fused_merge) ? 2 : 1;
}

static int prefill_impl(const void* q, const void* k_cache, const void* v_cache,
                        const int32_t* qo_indptr, const int32_t* kv_indptr,
                        const int32_t* kv_indices, const int32_t* prefix_lens, const void* gate,
                        void* out, void* workspace, size_t workspace_bytes, int batch, int total_q,
                        int64_t total_kv, int num_q_heads, int num_kv_heads, int head_dim,
                        int64_t num_slots, int dtype, float sm_scale, int max_len_extend,
                        int is_cross_attention, int sliding_window_size, void* stream,
                        const PageIndex* pages = nullptr) {
  const char* op = "paged_prefill_attention: ";
  if (total_q < 0 || num_q_heads <= 0 || num_kv_heads <= 0 || num_slots < 0 || total_kv < 0)
    return fail(MSGL_BAD_SHAPE,
                std::string(op) + "q must be 3D (total_q_tokens, num_q_heads, head_dim)");
  if (head_dim != 128 && head_dim != 256)
    return fail(MSGL_UNSUPPORTED_HEAD_DIM, std::string(op) + "head_dim must be 128 or 256");
  if (num_q_heads % num_kv_heads != 0)
    return fail(MSGL_BAD_GQA, std::string(op) + "num_q_heads must be a multiple of num_kv_heads");
  if (sliding_window_size < 0)
    return fail(MSGL_BAD_ARG, std::string(op) + "sliding_window_size must be >= 0");
  if (batch <= 0) return fail(MSGL_BAD_SHAPE, std::string(op) + "batch must be > 0");
  if (dtype != MSGL_DTYPE_BF16 && dtype != MSGL_DTYPE_F16)
    return fail(MSGL_BAD_DTYPE, std::string(op) + "unsupported dtype, must be float16 or bfloat16");
  if (total_q == 0) return MSGL_OK;
  if (num_kv_heads > 65535)
    return fail(MSGL_BAD_SHAPE, std::string(op) + "num_kv_heads must be <= 65535");
  if (max_len_extend < 1) max_len_extend = 1;
  if (!q || !k_cache || !v_cache || !qo_indptr || !prefix_lens || !out ||
      (!pages && (!kv_indptr || !kv_indices)))
    return fail(MSGL_BAD_ARG, std::string(op) + "null tensor pointer");
  if (!aligned16(q) || !aligned16(k_cache) || !aligned16(v_cache) || !aligned16(out) ||
      !aligned16(gate) || !aligned16(workspace))
    return fail(MSGL_BAD_ARG, std::string(op) + "q, the pools, out, gate and the workspace must be "
                                                "16-byte aligned");
  const int sms = sm_count_cached();
  if (sms <= 0) return fail(MSGL_CUDA_ERROR, std::string(op) + "cannot query the device");
  CUtensorMap tm_k, tm_v;
  std::memset(&tm_k, 0, sizeof(tm_k));
  std::memset(&tm_v, 0, sizeof(tm_v));
  if (pages && (!make_pool_tensor_map(&tm_k, k_cache, num_slots, num_kv_heads, head_dim, dtype) ||
                !make_pool_tensor_map(&tm_v, v_cache, num_slots, num_kv_heads, head_dim, dtype)))
    return fail(MSGL_CUDA_ERROR, std::string(op) + "cannot build the tensor maps of the K/V pool");
  CUtensorMap tm_q;
  std::memset(&tm_q, 0, sizeof(tm_q));
  const bool q_tma = pages && make_query_tensor_map(&tm_q, q, total_q, num_q_heads,
                                                    num_q_heads / num_kv_heads, head_dim, dtype);
  const PrefillPlan pl = plan_prefill(batch, total_q, total_kv, num_q_heads, num_kv_heads,
                                      head_dim, max_len_extend, sliding_window_size, sms);
  const size_t need = kStatusBytes + pl.plan_bytes + pl.part_ml_bytes + pl.part_o_bytes;
  if (!workspace || workspace_bytes < need)
    return fail(MSGL_BAD_ARG, std::string(op) + "workspace too small");
  if (pl.items * num_kv_heads > 0x7fffffffLL || num_q_heads > 65535)
    return fail(MSGL_BAD_SHAPE, std::string(op) + "problem too large for one launch");

  msgl::PrefillParams p{};
  p.q = q;
  p.k_cache = k_cache;
  p.v_cache = v_cache;
  p.qo_indptr = qo_indptr;
  p.kv_indptr = kv_indptr;
  p.kv_indices = kv_indices;
  p.prefix_lens = prefix_lens;
  if (pages) {
    p.page_indptr = pages->page_indptr;
    p.page_indices = pages->page_indices;
    p.kv_lens = pages->kv_lens;
    p.page_size = pages->page_size;
  }
  p.q_tma = q_tma ? 1 : 0;
  p.out = out;
  p.gate = gate;
  unsigned char* ws = static_cast<unsigned char*>(workspace);
  p.status = reinterpret_cast<int*>(ws);
  if (pl.kv_chunk > 0) {
    // at most kPrefillTickets units when split; no counters = the merge is a launch of its own
    p.tickets = pl.fused_merge ? reinterpret_cast<int*>(ws + 256) : nullptr;
    p.part_ml = reinterpret_cast<float*>(ws + kStatusBytes + pl.plan_bytes);
    p.part_o = reinterpret_cast<float*>(ws + kStatusBytes + pl.plan_bytes + pl.part_ml_bytes);
  }
  p.batch = batch;
  p.total_q = total_q;
  p.hq = num_q_heads;
  p.hkv = num_kv_heads;
  p.group = num_q_heads / num_kv_heads;
  p.num_slots = num_slots;
  p.scale_log2 = sm_scale * msgl::kLog2e;
  p.is_cross = is_cross_attention ? 1 : 0;
  p.window = sliding_window_size;
  p.kv_chunk = pl.kv_chunk;
  cudaStream_t s = static_cast<cudaStream_t>(stream);

  dim3 grid(static_cast<unsigned>(pl.items * num_kv_heads));
  const bool short_q = prefill_short_q(max_len_extend, p.group, head_dim);
  cudaError_t e;
  auto launch = [&](auto kernel, auto merge, int threads, int smem) -> cudaError_t {
    cudaError_t err = allow_smem(kernel, smem);
    if (err != cudaSuccess) return err;
    kernel<<<grid, threads, smem, s>>>(p, tm_k, tm_v, tm_q);
    if (pl.kv_chunk > 0 && !pl.fused_merge)
      return launch_dependent(merge, dim3(grid.x, msgl::kMergeSlices), dim3(msgl::kMergeWarps * 32), s, p);
    return cudaSuccess;
  };
  // per element type: head_dim 256 / short query blocks / long chunks, each per-token or paged
  auto dispatch = [&](auto tag) -> cudaError_t {
    using T = decltype(tag);
    using S1 = msgl::TcShape<1>;
    using S2 = msgl::TcShape<2>;
    using S1w = msgl::TcShape<1, 256>;
    using P1 = msgl::TcShape<1, 128, true>;
    using P2 = msgl::TcShape<2, 128, true>;
    using P1w = msgl::TcShape<1, 256, true>;
    auto m1w = msgl::prefill_merge_kernel<T, 256, S1w::kBM>;
    auto m1 = msgl::prefill_merge_kernel<T, 128, S1::kBM>;
    auto m2 = msgl::prefill_merge_kernel<T, 128, S2::kBM>;
    if (head_dim == 256)
      return pages ? launch(msgl::prefill_tc_kernel<T, 64, 1, 256, true>, m1w, P1w::kThreads, P1w::kSmemBytes)
                   : launch(msgl::prefill_tc_kernel<T, 64, 1, 256>, m1w, S1w::kThreads, S1w::kSmemBytes);
    if (short_q)
      return pages ? launch(msgl::prefill_tc_kernel<T, 64, 1, 128, true>, m1, P1::kThreads, P1::kSmemBytes)
                   : launch(msgl::prefill_tc_kernel<T, 64, 1>, m1, S1::kThreads, S1::kSmemBytes);
    return pages ? launch(msgl::prefill_tc_kernel<T, 128, 2, 128, true>, m2, P2::kThreads, P2::kSmemBytes)
                 : launch(msgl::prefill_tc_kernel<T, 128, 2>, m2, S2::kThreads, S2::kSmemBytes);
  };
  e = dtype == MSGL_DTYPE_BF16 ? dispatch(__nv_bfloat16{}) : dispatch(__half{});
  if (e != cudaSuccess) return cuda_fail("paged_prefill_attention", e);
  if ((e = cudaGetLastError()) != cudaSuccess) return cuda_fail("paged_prefill_attention", e);
  return MSGL_OK;
}

int msgl_paged_prefill_attention(const void* q, const void* k_cache, const void* v_cache,
                                 const int32_t* qo_indptr, const int32_t* kv_indptr,
                                 const int32_t* kv_indices, const int32_t* prefix_lens, void* out,
                                 void* workspace, size_t workspace_bytes, int batch, int total_q,
                                 int64_t total_kv, int num_q_heads, int num_kv_heads,
                                 int head_dim, int64_t num_slots, int dtype, float sm_scale,
                                 int max_len_extend, int is_cross_attention,
                                 int sliding_window_size, void* stream) {
  return prefill_impl(q, k_cache, v_cache, qo_indptr, kv_indptr, kv_indices, prefix_lens, nullptr, out,
                      workspace, workspace_bytes, batch, total_q, total_kv, num_q_heads, num_kv_heads,
                      head_dim, num_slots, dtype, sm_scale, max_len_extend, is_cross_attention,
                      sliding_window_size, stream);
}

int msgl_paged_prefill_attention_gated(const void* q, const void* k_cache, const void* v_cache,
                                       const int32_t* qo_indptr, const int32_t* kv_indptr,
                                       const int32_t* kv_indices, const int32_t* prefix_lens,
                                       const void* gate, void* out, void* workspace,
                                       size_t workspace_bytes, int batch, int total_q,
                                       int64_t total_kv, int num_q_heads, int num_kv_heads,
                                       int head_dim, int64_t num_slots, int dtype, float sm_scale,
                                       int max_len_extend, int is_cross_attention,
                                       int sliding_window_size, void* stream) {
  if (!gate && total_q > 0) return fail(MSGL_BAD_ARG, "paged_prefill_attention: null gate pointer");
  return prefill_impl(q, k_cache, v_cache, qo_indptr, kv_indptr, kv_indices, prefix_lens, gate, out,
                      workspace, workspace_bytes, batch, total_q, total_kv, num_q_heads, num_kv_heads,
                      head_dim, num_slots, dtype, sm_scale, max_len_extend, is_cross_attention,
                      sliding_window_size, stream);
}

int msgl_store_kv_cache(void* k_cache, void* v_cache, const int32_t* indices, const void* k,
                        const void* v, int length, int num_kv_heads, int head_dim,
                        int64_t num_slots, int64_t cache_row_stride, int64_t input_row_stride,
                        int dtype, void* status_word, void* stream) {
  const char* op = "store_kv_cache: ";
  if (length < 0 || num_kv_heads <= 0 || head_dim <= 0 || num_slots < 0)
    return fail(MSGL_BAD_SHAPE,
                std::string(op) + "k and v shape must be (length, num_kv_heads, head_dim)");
  if (head_dim % 4 != 0)
    return fail(MSGL_BAD_SHAPE, std::string(op) + "head_dim must be a multiple of 4");
  if (dtype != MSGL_DTYPE_BF16 && dtype != MSGL_DTYPE_F16)
    return fail(MSGL_BAD_DTYPE, std::string(op) + "k_cache, v_cache, k, v must have the same dtype");
  const int64_t row_elems = static_cast<int64_t>(num_kv_heads) * head_dim;
  if (cache_row_stride < row_elems || input_row_stride < row_elems)
    return fail(MSGL_BAD_SHAPE, std::string(op) + "row stride smaller than num_kv_heads*head_dim");
  if (length == 0) return MSGL_OK;
  if (!k_cache || !v_cache || !indices || !k || !v)
    return fail(MSGL_BAD_ARG, std::string(op) + "null tensor pointer");
  const int64_t row_bytes = row_elems * 2;
  const int64_t crb = cache_row_stride * 2, irb = input_row_stride * 2;
  auto aligned = [](const void* ptr, int64_t a) { return reinterpret_cast<uintptr_t>(ptr) % a == 0; };
  const bool vec16 = row_bytes % 16 == 0 && crb % 16 == 0 && irb % 16 == 0 && aligned(k_cache, 16) &&
                     aligned(v_cache, 16) && aligned(k, 16) && aligned(v, 16);
  const bool vec8 = crb % 8 == 0 && irb % 8 == 0 && aligned(k_cache, 8) && aligned(v_cache, 8) &&
                    aligned(k, 8) && aligned(v, 8);
  if (!vec16 && !vec8)
    return fail(MSGL_BAD_ARG, std::string(op) + "tensors must be 8-byte aligned");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int vec = vec16 ? 16 : 8;
  const int vec_per_row = static_cast<int>(row_bytes / vec);
  const int64_t total = static_cast<int64_t>(length) * vec_per_row;
  const int threads = 256;
  int sms = sm_count_cached();
  if (sms <= 0) sms = 148;
  int64_t blocks = (total + threads - 1) / threads;
  if (blocks > static_cast<int64_t>(sms) * 16) blocks = static_cast<int64_t>(sms) * 16;
  if (vec16)
    store_kv_kernel<16><<<static_cast<unsigned>(blocks), threads, 0, s>>>(
        static_cast<unsigned char*>(k_cache), static_cast<unsigned char*>(v_cache), indices,
        static_cast<const unsigned char*>(k), static_cast<const unsigned char*>(v), length,
        vec_per_row, crb, irb, num_slots, static_cast<int*>(status_word));
  else
    store_kv_kernel<8><<<static_cast<unsigned>(blocks), threads, 0, s>>>(
        static_cast<unsigned char*>(k_cache), static_cast<unsigned char*>(v_cache), indices,
        static_cast<const unsigned char*>(k), static_cast<const unsigned char*>(v), length,
        vec_per_row, crb, irb, num_slots, static_cast<int*>(status_word));
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail("store_kv_cache", e);
  return MSGL_OK;
}

int msgl_qk_norm_rope_store(void* q, const void* k, const void* v, const void* q_weight,
                            const void* k_weight, const int32_t* positions,
                            const int32_t* out_loc, void* k_cache, void* v_cache, int n_tokens,
                            int num_q_heads, int num_kv_heads, int head_dim, int rotary_dim,
                            float rope_base, float eps, int64_t num_slots, int64_t q_token_stride,
                            int64_t k_token_stride, int64_t v_token_stride,
                            int64_t cache_row_stride, int dtype, void* stream) {
  const char* op = "qk_norm_rope_store: ";
  if (n_tokens < 0 || num_q_heads <= 0 || num_kv_heads <= 0 || num_slots < 0)
    return fail(MSGL_BAD_SHAPE, std::string(op) +
                "q must be (n_tokens, num_q_heads, head_dim), k and v (n_tokens, num_kv_heads, head_dim)");
  if (head_dim != 128 && head_dim != 256)
    return fail(MSGL_UNSUPPORTED_HEAD_DIM, std::string(op) + "head_dim must be 128 or 256");
  if (rotary_dim != head_dim && rotary_dim != head_dim / 2 && rotary_dim != head_dim / 4)
    return fail(MSGL_BAD_ARG,
                std::string(op) + "rotary_dim must be head_dim, head_dim/2 or head_dim/4");
  if (dtype != MSGL_DTYPE_BF16 && dtype != MSGL_DTYPE_F16)
    return fail(MSGL_BAD_DTYPE, std::string(op) + "q, k, v, the weights and the caches must be bf16 or f16");
  if (!(rope_base > 1.f) || !(eps >= 0.f))
    return fail(MSGL_BAD_ARG, std::string(op) + "rope_base must be > 1 and eps >= 0");
  const int64_t kv_row = static_cast<int64_t>(num_kv_heads) * head_dim;
  if (q_token_stride < static_cast<int64_t>(num_q_heads) * head_dim || k_token_stride < kv_row ||
      v_token_stride < kv_row || cache_row_stride < kv_row)
    return fail(MSGL_BAD_SHAPE, std::string(op) + "a token or slot stride is smaller than its row");
  if (n_tokens == 0) return MSGL_OK;
  if (!q || !k || !v || !positions || !out_loc || !k_cache || !v_cache)
    return fail(MSGL_BAD_ARG, std::string(op) + "null tensor pointer");
  const int va = head_dim == 256 ? 16 : 8;   // bytes of one lane's access
  auto aligned = [va](const void* ptr) { return reinterpret_cast<uintptr_t>(ptr) % va == 0; };
  const int64_t ve = va / 2;
  if (!aligned(q) || !aligned(k) || !aligned(v) || !aligned(k_cache) || !aligned(v_cache) ||
      q_token_stride % ve != 0 || k_token_stride % ve != 0 || v_token_stride % ve != 0 ||
      cache_row_stride % ve != 0)
    return fail(MSGL_BAD_ARG, std::string(op) + "q, k, v and cache rows must be 8-byte aligned "
                                                "(16-byte at head_dim 256)");
  msgl::QkNormRopeParams p{};
  p.q = q;
  p.k = k;
  p.v = v;
  p.q_weight = q_weight;
  p.k_weight = k_weight;
  p.positions = positions;
  p.out_loc = out_loc;
  p.k_cache = k_cache;
  p.v_cache = v_cache;
  p.n = n_tokens;
  p.hq = num_q_heads;
  p.hkv = num_kv_heads;
  p.rotary_dim = rotary_dim;
  p.q_stride = q_token_stride;
  p.k_stride = k_token_stride;
  p.v_stride = v_token_stride;
  p.cache_stride = cache_row_stride;
  p.num_slots = num_slots;
  p.log2_base = log2f(rope_base);
  p.eps = eps;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int threads = 256;                          // sixteen half-warps, an item each per pass
  int sms = sm_count_cached();
  if (sms <= 0) sms = 148;
  const int kR = msgl::qk_rows_per_item(head_dim);
  const int64_t items = static_cast<int64_t>(n_tokens) *
                        ((num_q_heads + kR - 1) / kR + 2 * ((num_kv_heads + kR - 1) / kR));
  if (items >= (1ll << 31)) return fail(MSGL_BAD_ARG, "qk_norm_rope_store: too many rows for one call");
  const int64_t want = (items + 15) / 16;
  const int n_ctas = static_cast<int>(std::min<int64_t>(want, static_cast<int64_t>(sms) * 16));
  if (head_dim == 256) {
    if (dtype == MSGL_DTYPE_BF16)
      msgl::qk_norm_rope_store_kernel<__nv_bfloat16, 256><<<n_ctas, threads, 0, s>>>(p);
    else
      msgl::qk_norm_rope_store_kernel<__half, 256><<<n_ctas, threads, 0, s>>>(p);
  } else if (dtype == MSGL_DTYPE_BF16) {
    msgl::qk_norm_rope_store_kernel<__nv_bfloat16, 128><<<n_ctas, threads, 0, s>>>(p);
  } else {
    msgl::qk_norm_rope_store_kernel<__half, 128><<<n_ctas, threads, 0, s>>>(p);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail("qk_norm_rope_store", e);
  return MSGL_OK;
}

size_t msgl_page_index_workspace_bytes(int batch, int64_t total_pages, int page_size) {
  if (batch <= 0 || total_pages <= 0 || page_size <= 0) return 256;
  const size_t n = static_cast<size_t>(batch) + 1 + static_cast<size_t>(total_pages) * page_size;
  return (n * sizeof(int32_t) + 255) / 256 * 256;
}

// Builds kv_indptr and per-token kv_indices in `index_ws`; *total_kv_bound = total_pages * page_size.
static int expand_page_index(const char* op_name, const int32_t* page_indptr,
                             const int32_t* page_indices, const int32_t* kv_lens, int batch,
                             int64_t total_pages, int page_size, int64_t num_slots, void* index_ws,
                             int* status, const int32_t** kv_indptr, const int32_t** kv_indices,
                             int64_t* total_kv_bound, void* stream) {
  const std::string op = std::string(op_name) + ": ";
  if (batch < 0 || total_pages < 0) return fail(MSGL_BAD_SHAPE, op + "negative size");
  if (page_size <= 0) return fail(MSGL_BAD_ARG, op + "page_size must be > 0");
  if (batch > 65535) return fail(MSGL_BAD_SHAPE, op + "batch must be <= 65535");
  if (total_pages * page_size >= (1ll << 31))
    return fail(MSGL_BAD_SHAPE, op + "total_pages * page_size must be < 2^31");
  if (batch > 0 && (!page_indptr || !kv_lens || (total_pages > 0 && !page_indices)))
    return fail(MSGL_BAD_ARG, op + "null tensor pointer");
  int32_t* indptr = static_cast<int32_t*>(index_ws);
  int32_t* indices = indptr + batch + 1;
  *kv_indptr = indptr;
  *kv_indices = indices;
  *total_kv_bound = total_pages * page_size;
  if (batch == 0) return MSGL_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  page_lens_scan_kernel<<<1, 1024, 0, s>>>(kv_lens, page_indptr, batch, page_size, indptr, status);
  if (total_pages > 0) {
    const int64_t avg = *total_kv_bound / batch + 1;
    int bx = static_cast<int>((avg + 255) / 256);
    if (bx > 64) bx = 64;
    expand_page_indices_kernel<<<dim3(bx, batch), 256, 0, s>>>(page_indptr, page_indices, indptr,
                                                                page_size, total_pages, num_slots,
                                                                indices, status);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(op_name, e);
  return MSGL_OK;
}

int msgl_paged_decode_attention_p16(const void* q, const void* k_cache, const void* v_cache,
                                    const int32_t* page_indptr, const int32_t* page_indices,
                                    const int32_t* kv_lens, const int32_t* num_kv_splits,
                                    const void* gate, void* out,
                                    void* workspace, size_t workspace_bytes, int batch,
                                    int num_q_heads, int num_kv_heads, int head_dim,
                                    int64_t num_slots, int dtype, float sm_scale, int max_kv_splits,
                                    int page_size, int64_t total_pages, void* stream) {
  const char* op = "paged_decode_attention_p16";
  if (batch < 0 || num_q_heads <= 0 || head_dim <= 0 || max_kv_splits <= 0 || total_pages < 0 ||
      page_size <= 0)
    return fail(MSGL_BAD_SHAPE, std::string(op) + ": bad sizes");
  const size_t op_ws = (msgl_decode_workspace_bytes(batch, num_q_heads, head_dim, max_kv_splits) + 255) / 256 * 256;
  const size_t idx_ws = msgl_page_index_workspace_bytes(batch, total_pages, page_size);
  if (!workspace || workspace_bytes < op_ws + idx_ws)
    return fail(MSGL_BAD_ARG, std::string(op) + ": workspace too small: need " +
                                  std::to_string(op_ws + idx_ws) + " bytes, got " +
                                  std::to_string(workspace_bytes));
  if (page_size % msgl::kTmaBoxRows == 0 && tensor_map_encoder() != nullptr) {
    // Fast path: a warp's 16-token group is one TMA box copy per K/V half straight from the
    // page id; no per-token index is built.
    if (batch > 0 && (!page_indptr || !kv_lens || (total_pages > 0 && !page_indices)))
      return fail(MSGL_BAD_ARG, std::string(op) + ": null tensor pointer");
    if (total_pages * page_size >= (1ll << 31))
      return fail(MSGL_BAD_SHAPE, std::string(op) + ": total_pages * page_size must be < 2^31");
    const PageIndex pages{page_indptr, page_indices, kv_lens, page_size};
    return decode_impl(q, k_cache, v_cache, nullptr, nullptr, num_kv_splits, gate, out, workspace,
                       op_ws, batch, num_q_heads, num_kv_heads, head_dim, num_slots, dtype, sm_scale,
                       max_kv_splits, stream, &pages);
  }
  const int32_t *kv_indptr = nullptr, *kv_indices = nullptr;
  int64_t bound = 0;
  int rc = expand_page_index(op, page_indptr, page_indices, kv_lens, batch, total_pages, page_size,
                             num_slots, static_cast<unsigned char*>(workspace) + op_ws,
                             static_cast<int*>(workspace), &kv_indptr, &kv_indices, &bound, stream);
  if (rc != MSGL_OK) return rc;
  return decode_impl(q, k_cache, v_cache, kv_indptr, kv_indices, num_kv_splits, gate, out, workspace,
                     op_ws, batch, num_q_heads, num_kv_heads, head_dim, num_slots, dtype, sm_scale,
                     max_kv_splits, stream);
}

size_t msgl_prefill_workspace_bytes_p16(int batch, int total_q, int64_t total_pages, int page_size,
                                        int num_q_heads, int num_kv_heads, int head_dim,
                                        int max_len_extend, int sliding_window_size) {
  if (total_pages < 0 || page_size <= 0) return 0;
  const size_t op_ws = (msgl_prefill_workspace_bytes(batch, total_q, total_pages * page_size, num_q_heads,
                                                     num_kv_heads, head_dim, max_len_extend,
                                                     sliding_window_size) + 255) / 256 * 256;
  return op_ws + msgl_page_index_workspace_bytes(batch, total_pages, page_size);
}

int msgl_paged_prefill_attention_p16(const void* q, const void* k_cache, const void* v_cache,
                                     const int32_t* qo_indptr, const int32_t* page_indptr,
                                     const int32_t* page_indices, const int32_t* kv_lens,
                                     const int32_t* prefix_lens, const void* gate, void* out,
                                     void* workspace, size_t workspace_bytes, int batch, int total_q,
                                     int num_q_heads,
                                     int num_kv_heads, int head_dim, int64_t num_slots, int dtype,
                                     float sm_scale, int max_len_extend, int is_cross_attention,
                                     int sliding_window_size, int page_size, int64_t total_pages,
                                     void* stream) {
  const char* op = "paged_prefill_attention_p16";
  if (batch < 0 || total_q < 0 || num_q_heads <= 0 || num_kv_heads <= 0 || total_pages < 0 ||
      page_size <= 0)
    return fail(MSGL_BAD_SHAPE, std::string(op) + ": bad sizes");
  const size_t idx_ws = msgl_page_index_workspace_bytes(batch, total_pages, page_size);
  const size_t total = msgl_prefill_workspace_bytes_p16(batch, total_q, total_pages, page_size,
                                                        num_q_heads, num_kv_heads, head_dim,
                                                        max_len_extend, sliding_window_size);
  if (!workspace || workspace_bytes < total)
    return fail(MSGL_BAD_ARG, std::string(op) + ": workspace too small: need " +
                                  std::to_string(total) + " bytes, got " +
                                  std::to_string(workspace_bytes));
  const size_t op_ws = total - idx_ws;
  if (page_size % msgl::kTmaBoxRows == 0 && tensor_map_encoder() != nullptr) {
    // Fast path: the 16 token rows of a page (or of a 16-row slice of a larger page) are
    // contiguous in the pool, so the kernel copies them as TMA boxes straight from the page
    // ids; no per-token index is built.
    if (batch > 0 && (!page_indptr || !kv_lens || (total_pages > 0 && !page_indices)))
      return fail(MSGL_BAD_ARG, std::string(op) + ": null tensor pointer");
    if (total_pages * page_size >= (1ll << 31))
      return fail(MSGL_BAD_SHAPE, std::string(op) + ": total_pages * page_size must be < 2^31");
    const PageIndex pages{page_indptr, page_indices, kv_lens, page_size};
    return prefill_impl(q, k_cache, v_cache, qo_indptr, nullptr, nullptr, prefix_lens, gate, out,
                        workspace, op_ws, batch, total_q, total_pages * page_size, num_q_heads,
                        num_kv_heads, head_dim, num_slots, dtype, sm_scale, max_len_extend,
                        is_cross_attention, sliding_window_size, stream, &pages);
  }
  const int32_t *kv_indptr = nullptr, *kv_indices = nullptr;
  int64_t bound = 0;
  int rc = expand_page_index(op, page_indptr, page_indices, kv_lens, batch, total_pages, page_size,
                             num_slots, static_cast<unsigned char*>(workspace) + op_ws,
                             static_cast<int*>(workspace), &kv_indptr, &kv_indices, &bound, stream);
  if (rc != MSGL_OK) return rc;
  return prefill_impl(q, k_cache, v_cache, qo_indptr, kv_indptr, kv_indices, prefix_lens, gate, out,
                      workspace, op_ws, batch, total_q, bound, num_q_heads, num_kv_heads, head_dim,
                      num_slots, dtype, sm_scale, max_len_extend, is_cross_attention,
                      sliding_window_size, stream);
}

#ifdef MSGL_TRACE
// Development builds only: copies the per-CTA trace of the last prefill launch to host memory.
int msgl_debug_read_cta_trace(void* dst, int n_ctas) {
  if (n_ctas > msgl::kTraceCtas) n_ctas = msgl::kTraceCtas;
  cudaError_t e = cudaMemcpyFromSymbol(dst, msgl::g_cta_trace, sizeof(long long) * 32 * n_ctas);
  return e == cudaSuccess ? MSGL_OK : cuda_fail("debug_read_cta_trace", e);
}
#endif

int64_t msgl_fast_compare_key(const void* a, const void* b, int64_t len_a, int64_t len_b,
                              int elem_bytes) {
  // host memory; first index at which the two keys differ (their common length if none)
  if (!a || !b || len_a <= 0 || len_b <= 0) return 0;
  const int64_t n = len_a < len_b ? len_a : len_b;
  if (elem_bytes == 8) {
    const int64_t* x = static_cast<const int64_t*>(a);
    const int64_t* y = static_cast<const int64_t*>(b);
    int64_t i = 0;
    while (i < n && x[i] == y[i]) ++i;
    return i;
  }
  if (elem_bytes == 4) {
    const int32_t* x = static_cast<const int32_t*>(a);
    const int32_t* y = static_cast<const int32_t*>(b);
    int64_t i = 0;
    // eight ids per step while whole blocks agree, then element by element
    while (i + 8 <= n && std::memcmp(x + i, y + i, 32) == 0) i += 8;
    while (i < n && x[i] == y[i]) ++i;
    return i;
  }
  g_last_error = "fast_compare_key: Arrays must be int32 or int64.";
  return -1;
}

int msgl_build_attn_metadata(const int32_t* req, const int32_t* page_table, int64_t table_row_stride,
                             int64_t table_rows, int64_t table_cols, int batch, int page_size,
                             int split_chunk, int max_kv_splits, int64_t total_q, int64_t total_kv,
                             int64_t total_pages, int32_t* qo_indptr, int32_t* kv_indptr,
                             int32_t* prefix_lens, int32_t* num_kv_splits, int32_t* positions,
                             int32_t* kv_indices, int32_t* page_indptr, int32_t* page_indices,
                             void* status_word, void* stream) {
  const char* op = "build_attn_metadata: ";
  if (batch < 0 || table_rows < 0 || table_cols < 0 || table_row_stride < 0 || total_q < 0 ||
      total_kv < 0 || total_pages < 0)
    return fail(MSGL_BAD_SHAPE, std::string(op) + "negative size");
  if (page_size < 1 || max_kv_splits < 1 || split_chunk < 0)
    return fail(MSGL_BAD_ARG, std::string(op) + "page_size and max_kv_splits must be >= 1, split_chunk >= 0");
  if (batch > 65535) return fail(MSGL_BAD_SHAPE, std::string(op) + "batch must be <= 65535");
  if (total_q >= (1ll << 31) || total_kv >= (1ll << 31))
    return fail(MSGL_BAD_SHAPE, std::string(op) + "totals must be < 2^31");
  if (batch == 0) return MSGL_OK;
  if (!req || !page_table || !qo_indptr || !kv_indptr || !prefix_lens || !num_kv_splits ||
      (total_q > 0 && !positions) || (page_indptr && total_pages > 0 && !page_indices))
    return fail(MSGL_BAD_ARG, std::string(op) + "null tensor pointer");
  MetadataParams p{};
  p.req = req;
  p.page_table = page_table;
  p.row_stride = table_row_stride;
  p.table_rows = table_rows;
  p.table_cols = table_cols;
  p.batch = batch;
  p.page_size = page_size;
  p.split_chunk = split_chunk;
  p.max_kv_splits = max_kv_splits;
  p.total_q = total_q;
  p.total_kv = total_kv;
  p.total_pages = total_pages;
  p.qo_indptr = qo_indptr;
  p.kv_indptr = kv_indptr;
  p.prefix_lens = prefix_lens;
  p.num_kv_splits = num_kv_splits;
  p.positions = positions;
  p.kv_indices = kv_indices;
  p.page_indptr = page_indptr;
  p.page_indices = page_indptr ? page_indices : nullptr;
  p.status = static_cast<int*>(status_word);
  const int64_t avg = total_kv / batch + 1;
  int bx = static_cast<int>((avg + 255) / 256);
  if (bx > 32) bx = 32;
  if (bx < 1) bx = 1;
  build_metadata_kernel<<<dim3(bx, batch), 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail("build_attn_metadata", e);
  return MSGL_OK;
}

int msgl_gather_kv_indices(const int32_t* page_table, int64_t table_row_stride,
                           const int32_t* table_idx, const int32_t* kv_indptr,
                           int32_t* kv_indices, int batch, int64_t total_kv, int64_t table_rows,
                           int64_t table_cols, void* status_word, void* stream) {
  const char* op = "gather_kv_indices: ";
  if (batch < 0 || total_kv < 0 || table_row_stride < 0 || table_rows < 0 || table_cols < 0)
    return fail(MSGL_BAD_SHAPE, std::string(op) + "negative size");
  if (batch == 0 || total_kv == 0) return MSGL_OK;
  if (batch > 65535) return fail(MSGL_BAD_SHAPE, std::string(op) + "batch must be <= 65535");
  if (!page_table || !table_idx || !kv_indptr || !kv_indices)
    return fail(MSGL_BAD_ARG, std::string(op) + "null tensor pointer");
  const int64_t avg = total_kv / batch + 1;
  int bx = static_cast<int>((avg + 255) / 256);
  if (bx > 64) bx = 64;
  dim3 grid(bx, batch);
  gather_kv_indices_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      page_table, table_row_stride, table_idx, kv_indptr, kv_indices, batch, table_rows, table_cols,
      total_kv, static_cast<int*>(status_word));
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail("gather_kv_indices", e);
  return MSGL_OK;
}

}  // extern "C"
