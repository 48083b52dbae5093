/*
 * msgl_b200.h — C ABI of the B200 (sm_100a) paged-attention library.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream
 * handle (passed as void*, i.e. a cudaStream_t).  No entry point retains a
 * pointer past the call or allocates device memory, and none but
 * msgl_read_status synchronises the host with the device: scratch space is
 * supplied by the caller (query its size with the *_workspace_bytes
 * functions; msgl_paged_decode_attention_static uses an array inside the
 * library instead).  Launches are asynchronous on `stream`.
 *
 * Workspaces.  A workspace starts with a header of MSGL_WORKSPACE_HEADER_BYTES.
 * Its first word is a sticky device status (0 = fine, 1 = a bounded wait inside
 * a kernel ran out, 2 = a slot or page id outside the pool, or a length beyond
 * a sequence's pages, was met: such rows are read as zero keys and values).
 * From byte 256 on it holds the arrival counters of the attention ops'
 * split-KV pieces (the piece that arrives last merges the partials).  The
 * kernels leave the counters at zero, but they must BE zero at the first call:
 * clear at least the header once after allocating a workspace
 * (cudaMemsetAsync), use one workspace per stream, and let nothing else write
 * to the header.  After a call that reported status 1 clear it again.
 *
 * Each function replaces one operator of the reference extension
 * `mini_sglang_mlx_kernel` (mini-sglang-mlx-kernel/csrc/bindings.cpp); the
 * citation beside each declaration names the reference host wrapper whose
 * argument meaning, validation and error text it keeps.
 *
 * Tensors (row-major, innermost stride 1):
 *   q / out of decode      (batch, num_q_heads, head_dim)
 *   q / out of prefill     (total_q_tokens, num_q_heads, head_dim)
 *   k_cache / v_cache      (num_slots, num_kv_heads, head_dim)   one slot = one KV token
 *   kv_indptr, qo_indptr   (batch + 1) int32, CSR row pointers
 *   kv_indices             (kv_indptr[batch]) int32, slot id of every KV token
 *   prefix_lens            (batch) int32, absolute position of a sequence's first query row
 *   num_kv_splits          (batch) int32, split-KV hint per sequence
 * Grouped-query mapping: kv_head = q_head / (num_q_heads / num_kv_heads).
 * q, out, gate, the pools and every workspace must be 16-byte aligned (the
 * kernels move them in 16-byte pieces); the attention ops return MSGL_BAD_ARG
 * otherwise.
 */
#ifndef MSGL_B200_H_
#define MSGL_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MSGL_ABI_VERSION 2

/* Status codes returned by every int-valued entry point. */
enum {
  MSGL_OK = 0,
  MSGL_BAD_SHAPE = 1,
  MSGL_BAD_DTYPE = 2,
  MSGL_UNSUPPORTED_HEAD_DIM = 3,
  MSGL_BAD_GQA = 4,
  MSGL_BAD_ARG = 5,
  MSGL_CUDA_ERROR = 6,
  MSGL_DEVICE_STATUS = 7 /* a kernel reported a bounded-wait timeout or an out-of-range slot */
};

/* Element types of q / k_cache / v_cache / out. */
enum { MSGL_DTYPE_BF16 = 0, MSGL_DTYPE_F16 = 1 };

/* Bytes of the header every workspace starts with: status word (256 bytes) and 16384
 * arrival counters. */
#define MSGL_WORKSPACE_HEADER_BYTES (256 + 16384 * 4)

/* Largest split count the decode workspace layout supports. */
#define MSGL_MAX_KV_SPLITS 128

int msgl_abi_version(void);

/* Message of the last non-OK status returned on the calling thread ("" if none). */
const char* msgl_last_error_string(void);

/* Number of SMs of the current device (cached per device); <0 on CUDA error. */
int msgl_device_sm_count(void);

/*
 * Bytes of scratch the decode op needs: the header, fp32 partial outputs
 * (batch, num_q_heads, max_kv_splits, head_dim) and fp32 log-sum-exp (batch,
 * num_q_heads, max_kv_splits); a batch of more than 16384 (sequence, head)
 * pairs gets a counter region of its own in front of the partials, which every
 * call clears.
 * Replaces the two temporaries of PagedDecodeAttention::eval_gpu
 * (mini-sglang-mlx-kernel/csrc/paged_decode_attention.cpp:119-131).
 */
size_t msgl_decode_workspace_bytes(int batch, int num_q_heads, int head_dim, int max_kv_splits);

/*
 * Paged decode attention: one query token per sequence over all of its KV
 * tokens, split over the KV range; the piece of a (sequence, KV head) that
 * finishes last merges the partials by log-sum-exp (one launch).
 * Replaces paged_decode_attention
 * (mini-sglang-mlx-kernel/csrc/paged_decode_attention.cpp:15-73, binding
 * csrc/bindings.cpp:36-44) and its two Metal stages
 * (csrc/paged_decode_attention.metal:313-506, 512-586).
 * num_kv_splits may be NULL (then every sequence uses max_kv_splits capped by
 * its length).  Sequences of length 0 produce zeros.
 */
int msgl_paged_decode_attention(
    const void* q, const void* k_cache, const void* v_cache,
    const int32_t* kv_indptr, const int32_t* kv_indices, const int32_t* num_kv_splits,
    void* out, void* workspace, size_t workspace_bytes,
    int batch, int num_q_heads, int num_kv_heads, int head_dim, int64_t num_slots,
    int dtype, float sm_scale, int max_kv_splits, void* stream);

/* Size of the scratch array built into the library for the entry point below. */
#define MSGL_STATIC_SCRATCH_BYTES (32u << 20)

/*
 * Paged decode attention for callers that cannot allocate device memory.
 * No counterpart in the reference: it exists for hosts that hold no allocator
 * at the call site, for example a serving loop that runs inside a memory
 * budget fixed at start-up, a plugin that is forbidden to call cudaMalloc
 * because another runtime owns the device heap, or code running where an
 * allocation would synchronise the device.  Same arguments and result as
 * msgl_paged_decode_attention, minus the workspace: the split-KV partials go
 * to a fixed array of MSGL_STATIC_SCRATCH_BYTES (32 MiB) inside the library,
 * which every GPU that loads the library keeps until the process exits.
 *  - Limit: msgl_decode_workspace_bytes(batch, num_q_heads, head_dim,
 *    max_kv_splits) must not exceed MSGL_STATIC_SCRATCH_BYTES, i.e. about
 *    batch * num_q_heads * max_kv_splits <= 65 000 at head_dim 128; larger
 *    problems are rejected with MSGL_BAD_ARG and a message giving both sizes.
 *  - The first call on each device looks up the array's device address
 *    (cudaGetSymbolAddress, with that device current); make that first call
 *    outside any stream capture.  No call allocates or frees memory.
 *  - All calls on a device share the one array and it keeps the previous
 *    call's contents; calls that overlap on the GPU (different streams) race
 *    on it, so issue them on one stream or order them with events.
 *  - The array is laid out like a workspace (status word, arrival counters,
 *    partials); it is zero when the library is loaded.  Read its status word
 *    with msgl_read_status(NULL, ...).  The cached device address belongs to
 *    the device's primary context: after cudaDeviceReset the library has to
 *    be loaded afresh.
 */
int msgl_paged_decode_attention_static(
    const void* q, const void* k_cache, const void* v_cache,
    const int32_t* kv_indptr, const int32_t* kv_indices, const int32_t* num_kv_splits,
    void* out, int batch, int num_q_heads, int num_kv_heads, int head_dim, int64_t num_slots,
    int dtype, float sm_scale, int max_kv_splits, void* stream);

/*
 * Reads the sticky device status word of `workspace` (NULL: of the array behind
 * msgl_paged_decode_attention_static on the current device): waits for the work
 * queued on `stream`, copies the word to the host, clears it on the device if
 * `clear` is non-zero.  Returns MSGL_OK if it was 0, else MSGL_DEVICE_STATUS with
 * a message that names the condition; *status_out (may be NULL) receives the raw
 * word.  The only entry point that waits for the device.  No counterpart in the
 * reference (its kernels do not check slot ids).
 */
int msgl_read_status(void* workspace, int clear, int* status_out, void* stream);

/*
 * Self-test of the bounded waits: launches one small CTA whose warps wait, the way the
 * attention kernels do, on a barrier that nothing completes; the wait gives up after about
 * limit_us microseconds (1 .. 100000), the kernel sets the status word of `workspace` to 1
 * and returns, and the context stays usable.  Read the result with msgl_read_status.  For
 * deployment checks and tests; no counterpart in the reference.
 */
int msgl_selftest_bounded_wait(void* workspace, int limit_us, void* stream);

/*
 * msgl_paged_decode_attention with the output gate of the reference's Qwen3.5 attention
 * layer fused into the final write: out = attention * sigmoid(gate), gate (batch,
 * num_q_heads, head_dim) in the data dtype, both factors rounded to that dtype before the
 * product as the reference's array ops do (mini_sglang_mlx/models/qwen3_5.py:91-110).
 * No operator of the reference does this (the gate is an array op after its kernel).
 */
int msgl_paged_decode_attention_gated(
    const void* q, const void* k_cache, const void* v_cache,
    const int32_t* kv_indptr, const int32_t* kv_indices, const int32_t* num_kv_splits,
    const void* gate, void* out, void* workspace, size_t workspace_bytes,
    int batch, int num_q_heads, int num_kv_heads, int head_dim, int64_t num_slots,
    int dtype, float sm_scale, int max_kv_splits, void* stream);

/*
 * Bytes of scratch the prefill op needs for the given problem (split-KV
 * partials when there are too few query tiles to fill the GPU, plus a small
 * planning area).  total_kv = kv_indptr[batch] = length of kv_indices.
 * No counterpart in the reference (its prefill kernel never splits KV).
 */
size_t msgl_prefill_workspace_bytes(int batch, int total_q, int64_t total_kv, int num_q_heads,
                                    int num_kv_heads, int head_dim, int max_len_extend,
                                    int sliding_window_size);

/*
 * Kernel launches one prefill call of this shape makes: 1, or 2 when the key
 * range is split and a (sequence, query tile, head) unit is too large for the
 * CTA that finishes last to merge (the merge is then a second launch, chained
 * to the first with programmatic stream serialization).  page_granular != 0
 * asks for the *_p16 entry points.  No counterpart in the reference.
 */
int msgl_prefill_launch_count(int batch, int total_q, int64_t total_kv, int num_q_heads,
                              int num_kv_heads, int head_dim, int max_len_extend,
                              int sliding_window_size, int page_granular);

/*
 * Paged prefill / extend attention over prefix + new tokens with the four
 * mask modes (causal, full, causal+window, bidirectional+window); also the
 * speculative-verify and draft-block shapes.
 * Replaces paged_prefill_attention
 * (mini-sglang-mlx-kernel/csrc/paged_prefill_attention.cpp:18-87, binding
 * csrc/bindings.cpp:45-55) and its Metal kernel
 * (csrc/paged_prefill_attention.metal:382-640).
 * Key t of a sequence is visible to query row p iff t < kv_len and
 * (is_cross_attention or t <= prefix_len + p) and
 * (sliding_window_size == 0 or t >= prefix_len + p - sliding_window_size + 1).
 * Rows with no visible key produce zeros.  head_dim 128 or 256, as the reference.
 */
int msgl_paged_prefill_attention(
    const void* q, const void* k_cache, const void* v_cache,
    const int32_t* qo_indptr, const int32_t* kv_indptr, const int32_t* kv_indices,
    const int32_t* prefix_lens, void* out, void* workspace, size_t workspace_bytes,
    int batch, int total_q, int64_t total_kv, int num_q_heads, int num_kv_heads, int head_dim,
    int64_t num_slots, int dtype, float sm_scale, int max_len_extend,
    int is_cross_attention, int sliding_window_size, void* stream);

/*
 * msgl_paged_prefill_attention with out = attention * sigmoid(gate) fused into the final
 * write (see msgl_paged_decode_attention_gated); gate (total_q_tokens, num_q_heads, head_dim).
 */
int msgl_paged_prefill_attention_gated(
    const void* q, const void* k_cache, const void* v_cache,
    const int32_t* qo_indptr, const int32_t* kv_indptr, const int32_t* kv_indices,
    const int32_t* prefix_lens, const void* gate, void* out, void* workspace, size_t workspace_bytes,
    int batch, int total_q, int64_t total_kv, int num_q_heads, int num_kv_heads, int head_dim,
    int64_t num_slots, int dtype, float sm_scale, int max_len_extend,
    int is_cross_attention, int sliding_window_size, void* stream);

/*
 * Scatter new keys/values into the pool: k_cache[indices[r]] = k[r],
 * v_cache[indices[r]] = v[r] for r < length.  Row strides are in elements.
 * A row whose index is outside [0, num_slots) is dropped; if status_word (a
 * device int, e.g. the head of a workspace; may be NULL) is given it is set
 * to 2 then.
 * Replaces store_kv_cache
 * (mini-sglang-mlx-kernel/csrc/store_kv_cache.cpp:13-107, kernel
 * csrc/store_kv_cache.metal:7-31).
 */
int msgl_store_kv_cache(void* k_cache, void* v_cache, const int32_t* indices, const void* k,
                        const void* v, int length, int num_kv_heads, int head_dim,
                        int64_t num_slots, int64_t cache_row_stride, int64_t input_row_stride,
                        int dtype, void* status_word, void* stream);

/*
 * CSR metadata from a page table: for sequence b, copies
 * page_table[table_idx[b], 0:kv_lens[b]] to kv_indices[kv_indptr[b]:...]
 * in one launch.  kv_indptr (batch+1) must already hold the exclusive prefix
 * sum of kv_lens.  The table has table_rows x table_cols entries and the
 * output total_kv: a row id, a length or an output position outside them is
 * skipped (clamped) and sets status_word (a device int, may be NULL) to 2.
 * Replaces the per-request slice-and-concatenate loops of
 * AttnBackend.build_prefill_metadata / build_decode_metadata
 * (mini_sglang_mlx/attention/backend.py:239-244, 279-284).
 */
int msgl_gather_kv_indices(const int32_t* page_table, int64_t table_row_stride,
                           const int32_t* table_idx, const int32_t* kv_indptr,
                           int32_t* kv_indices, int batch, int64_t total_kv, int64_t table_rows,
                           int64_t table_cols, void* status_word, void* stream);

/*
 * All index arrays of one step from the page table in ONE launch (one host-to-device copy of
 * `req` in front of it).  req (3 * batch int32, device): for the batch's sequences in order the
 * number of new tokens [0, batch), the KV lengths including them [batch, 2 batch) and the
 * page-table rows [2 batch, 3 batch) (a decode step has one new token per sequence).  Outputs:
 * qo_indptr / kv_indptr (batch+1), prefix_lens = kv - new (batch), num_kv_splits =
 * min(max_kv_splits, max(1, ceil(kv / split_chunk))) (batch; split_chunk 0 = the reference's 128),
 * positions (total_q: kv - new + i for the i-th new token), kv_indices (total_kv per-token slot
 * ids copied from the table rows; NULL to skip) and, with page_size > 1, page_indptr (batch+1)
 * and page_indices (total_pages: slot of the page's first token / page_size; both NULL to
 * skip).  total_* are the sizes the caller allocated; anything outside them or outside the
 * table sets status_word (a device int, may be NULL) to 2 and is skipped.
 * Replaces the host loops of AttnBackend.build_prefill_metadata / build_decode_metadata and
 * _compute_num_kv_splits (mini_sglang_mlx/attention/backend.py:205-307).
 */
int msgl_build_attn_metadata(const int32_t* req, const int32_t* page_table, int64_t table_row_stride,
                             int64_t table_rows, int64_t table_cols, int batch, int page_size,
                             int split_chunk, int max_kv_splits, int64_t total_q, int64_t total_kv,
                             int64_t total_pages, int32_t* qo_indptr, int32_t* kv_indptr,
                             int32_t* prefix_lens, int32_t* num_kv_splits, int32_t* positions,
                             int32_t* kv_indices, int32_t* page_indptr, int32_t* page_indices,
                             void* status_word, void* stream);

/*
 * Page-granular index entries.  The reference hard-wires one token per page
 * (mini_sglang_mlx/engine/engine.py:103) and hands the ops one slot id per token
 * (kv_indices, mini_sglang_mlx/attention/backend.py:239-244, 279-284).  A pool
 * allocated in pages of page_size tokens (slot = page * page_size + offset) is
 * described more compactly by one id per PAGE: page_indptr (batch+1),
 * page_indices (total_pages) and the token lengths kv_lens (batch), all int32
 * device arrays.  These entries take that form.  With a page size that is a
 * multiple of 16 they are the fast path: the 16 token rows of a page (or of a
 * 16-row slice of a larger page) are contiguous in the pool, and the kernels
 * fetch them as TMA box copies (16 rows x 64 elements, 128-byte swizzle, one
 * instruction per box, completion counted on an mbarrier) straight from the
 * page ids; the query tile of the prefill op is fetched the same way.  Other
 * page sizes build kv_indptr and the per-token slot ids on the device first (a
 * scan of the lengths and one 4-byte store per token) and run the per-token
 * kernels.  A length that is negative or exceeds page_size * (pages of the
 * sequence) sets the device status word to 2 and is clamped; so does a page id
 * outside the pool, whose rows then read as zeros.  The pools must be 16-byte
 * aligned.
 *
 * Workspace: the op's own scratch followed by the index scratch,
 *   decode : round_up(msgl_decode_workspace_bytes(...), 256)
 *            + msgl_page_index_workspace_bytes(batch, total_pages, page_size)
 *   prefill: msgl_prefill_workspace_bytes_p16(...)
 * total_pages * page_size must be below 2^31.
 */
size_t msgl_page_index_workspace_bytes(int batch, int64_t total_pages, int page_size);

int msgl_paged_decode_attention_p16(
    const void* q, const void* k_cache, const void* v_cache,
    const int32_t* page_indptr, const int32_t* page_indices, const int32_t* kv_lens,
    const int32_t* num_kv_splits, const void* gate /* may be NULL, see *_gated */,
    void* out, void* workspace, size_t workspace_bytes,
    int batch, int num_q_heads, int num_kv_heads, int head_dim, int64_t num_slots,
    int dtype, float sm_scale, int max_kv_splits, int page_size, int64_t total_pages,
    void* stream);

size_t msgl_prefill_workspace_bytes_p16(int batch, int total_q, int64_t total_pages, int page_size,
                                        int num_q_heads, int num_kv_heads, int head_dim,
                                        int max_len_extend, int sliding_window_size);

int msgl_paged_prefill_attention_p16(
    const void* q, const void* k_cache, const void* v_cache,
    const int32_t* qo_indptr, const int32_t* page_indptr, const int32_t* page_indices,
    const int32_t* kv_lens, const int32_t* prefix_lens, const void* gate /* may be NULL */,
    void* out, void* workspace,
    size_t workspace_bytes, int batch, int total_q, int num_q_heads, int num_kv_heads,
    int head_dim, int64_t num_slots, int dtype, float sm_scale, int max_len_extend,
    int is_cross_attention, int sliding_window_size, int page_size, int64_t total_pages,
    void* stream);

/*
 * Length of the common prefix of two token-id keys in HOST memory (the first
 * index at which they differ), elem_bytes 4 (int32) or 8 (int64); -1 for any
 * other element size.  Used by the radix prefix cache when it walks an edge.
 * Replaces fast_compare_key
 * (mini-sglang-mlx-kernel/csrc/fast_compare_key.cpp:9-45, binding
 * csrc/bindings.cpp:33-35).
 */
int64_t msgl_fast_compare_key(const void* a, const void* b, int64_t len_a, int64_t len_b,
                              int elem_bytes);

/*
 * The step in front of the attention op, fused into one pass over q, k and v: per-head
 * RMSNorm of q and k (weights of head_dim elements, same dtype as the data; a null weight
 * skips that norm), rotary embedding of both (non-interleaved pairs (i, i + rotary_dim/2),
 * angle = positions[t] * rope_base^(-2i/rotary_dim)), q written back in place, the k rows
 * written to k_cache[out_loc[t]] and the v rows copied to v_cache[out_loc[t]].
 * Replaces, for a caller that adopts it, the array ops of
 * mini_sglang_mlx/models/qwen3.py:58-68 (q_norm, k_norm, rope, rope) plus the
 * store_kv_cache call of attention/backend.py:117-121; the reference has no fused
 * operator of this kind (its extension stops at store_kv_cache).
 * q (n_tokens, Hq, D), k and v (n_tokens, Hkv, D) with the given token strides in
 * elements (rows of a fused qkv projection are fine); caches (num_slots, Hkv, D) with
 * cache_row_stride elements per slot.  head_dim 128 or 256; rotary_dim = head_dim, head_dim/2
 * or head_dim/4 (the first rotary_dim elements of a head are rotated, the rest pass through).
 * Tokens whose out_loc is outside [0, num_slots) get their q processed and their k/v dropped.
 */
int msgl_qk_norm_rope_store(void* q, const void* k, const void* v, const void* q_weight,
                            const void* k_weight, const int32_t* positions,
                            const int32_t* out_loc, void* k_cache, void* v_cache, int n_tokens,
                            int num_q_heads, int num_kv_heads, int head_dim, int rotary_dim,
                            float rope_base, float eps, int64_t num_slots, int64_t q_token_stride,
                            int64_t k_token_stride, int64_t v_token_stride,
                            int64_t cache_row_stride, int dtype, void* stream);

#ifdef __cplusplus
}
#endif

#endif /* MSGL_B200_H_ */
