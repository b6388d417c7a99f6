/*
 * flash_moba_b200 — C ABI of the B200 (sm_100a) MoBA sparse-attention kernels.
 *
 * One shared library, libflashmoba_b200.so.  Every entry point takes plain device
 * pointers, sizes and a CUDA stream; it never allocates or frees device memory and, unless
 * its description says "synchronising", never synchronises the host with the device.  All
 * outputs and workspaces are allocated by the caller; `*_workspace_bytes` tells how much.
 * All work is enqueued on `stream` of the CURRENT device (the caller sets the device).
 *
 * State the library keeps (everything else lives in the caller's buffers):
 *   - per host thread: the text behind fmb_last_error(); the one-shot offers made with
 *     fmb_attn_rows_offer, fmb_attn_lists_load, fmb_attn_status_mirror and fmb_attn_key_spans,
 *     consumed by that thread's next attention call;
 *   - per process: the engine selected with fmb_set_engine, the launch counter and the event
 *     records of fmb_launch_count / fmb_profile_*;
 *   - per device: the gating kernel's status word (fmb_gate_status) and the 8 MiB scratch array
 *     of fmb_build_csc_static.
 * Calls on different streams or from different host threads are independent apart from these.
 *
 * Return value: 0 on success, otherwise one of FMB_ERR_*; `fmb_last_error()` then
 * returns a thread-local, human readable message.
 *
 * Each function names the entry point of the reference project (mit-han-lab/flash-moba)
 * whose work it replaces, as `file:line` inside that project.
 *
 * Conventions
 *   - q/k/v/out/dout/dq/dk/dv are (tokens, heads, head_dim) with head_dim contiguous;
 *     `*_row_stride` / `*_head_stride` are in ELEMENTS.
 *   - cu_seqlens_* are int32[batch+1] on the device.
 *   - dtype: FMB_BF16 or FMB_FP16.
 *   - pattern ("CSC"): col_offsets int64[batch][heads][ncol], col_nnz int32[batch][heads][ncol],
 *     indices int32[n_indices]; column (b,h,c) lists, ascending, the sequence-local query
 *     rows that attend key chunk c:  indices[col_offsets[b,h,c] .. + col_nnz[b,h,c]).
 */
#ifndef FLASH_MOBA_B200_H_
#define FLASH_MOBA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* fmb_stream_t; /* a cudaStream_t */

enum { FMB_BF16 = 0, FMB_FP16 = 1 };

enum {
  FMB_OK = 0,
  FMB_ERR_BAD_ARG = 1,      /* shape / stride / size rule violated            */
  FMB_ERR_UNSUPPORTED = 2,  /* valid in the reference, not built here          */
  FMB_ERR_WORKSPACE = 3,    /* workspace pointer null or too small             */
  FMB_ERR_CUDA = 4,         /* a CUDA runtime call or kernel launch failed     */
  FMB_ERR_TIMEOUT = 5       /* a bounded device-side wait expired              */
};

/* Library version (major*10000 + minor*100 + patch). */
int fmb_version(void);

/* Message of the last failing call made by this thread ("" if none). */
const char* fmb_last_error(void);

/* ------------------------------------------------------------------ stage P: mean-pool
 * cu_seqlens_km[b] = sum_{b'<b} ceil(len_k[b'] / chunk); one tiny launch, no host sync.
 * Replaces the ATen prologue of flash_moba/triton_mean_pool.py:134-138 (which syncs with
 * `.item()` at :140). */
int fmb_chunk_offsets(const int32_t* cu_seqlens_k, int batch, int chunk,
                      int32_t* cu_seqlens_km, fmb_stream_t stream);

/* km[cu_seqlens_km[b] + n, hk, :] = mean over the rows of chunk n of sequence b of k[:, hk, :]
 * (fp32 accumulation, divided by the true length of a short last chunk, rounded to dtype).
 * km is contiguous (km_rows, heads_k, head_dim); rows of km that belong to no chunk are
 * not written.  Replaces mean_pool_kernel / flash_topk_mean_pool,
 * flash_moba/triton_mean_pool.py:41-109, 112-157. */
int fmb_mean_pool(const void* k, int64_t k_row_stride, int64_t k_head_stride,
                  const int32_t* cu_seqlens_k, const int32_t* cu_seqlens_km, void* km,
                  int batch, int heads_k, int head_dim, int max_seqlen_k, int chunk,
                  int dtype, fmb_stream_t stream);

/* fmb_chunk_offsets and fmb_mean_pool in one call: cu_seqlens_km is an OUTPUT here.  For batches of
 * at most 64 sequences it is one launch (every warp of the pool kernel derives its sequence's first
 * centroid row from cu_seqlens_k itself); larger batches take the two launches above. */
int fmb_mean_pool_offsets(const void* k, int64_t k_row_stride, int64_t k_head_stride,
                          const int32_t* cu_seqlens_k, int32_t* cu_seqlens_km, void* km,
                          int batch, int heads_k, int head_dim, int max_seqlen_k, int chunk,
                          int dtype, fmb_stream_t stream);

/* ------------------------------------------------------------------ stage G: gating top-k
 * For every query row and q head: scores q . km (fp32, unscaled) against the centroids of
 * its sequence (kv head = h / (heads/heads_k)), causal chunk rule, top-k.
 *   topk_idx int32 [row][head][topk]: chunk ids by descending score, -1 = unused; entry
 *            (row, h, j) lives at row*topk_row_stride + h*topk_head_stride + j (elements),
 *            so both (total_q, heads, topk) and (heads, total_q, topk) storage work.
 *   topk_val float, same addressing, or NULL: the scores (+inf for the own chunk).
 * Rule under `causal`, p = row + len_k - len_q: chunk p/chunk is always selected first;
 * chunk n competes only if (n+1)*chunk-1 < p; rows with p < 0 select nothing.  Equal
 * scores: the higher chunk id ranks first.  1 <= topk <= 64.
 * Replaces moba_fused_topk's main kernel, csrc/flash_topk/flash_topk_api.cpp:130-258 and
 * csrc/flash_topk/src/flash_topk_kernel.h:31-357. */
int fmb_gate_topk(const void* q, int64_t q_row_stride, int64_t q_head_stride,
                  const void* km, /* contiguous (km_rows, heads_k, head_dim) */
                  const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k,
                  const int32_t* cu_seqlens_km, int32_t* topk_idx, float* topk_val,
                  int64_t topk_row_stride, int64_t topk_head_stride,
                  int batch, int heads, int heads_k, int head_dim, int max_seqlen_q,
                  int max_seqlen_k, int topk, int chunk, int causal, int dtype,
                  fmb_stream_t stream);

/* ------------------------------------------------------------------ stages O/E/S: pattern
 * Bytes of scratch `fmb_build_csc` needs. */
size_t fmb_build_csc_workspace_bytes(int batch, int heads, int max_seqlen_q, int ncol);

/* Top-k lists -> CSC pattern, deterministic, columns come out sorted (no sort pass).
 *   col_offsets[b,h,c] = (cu_q[b]*heads + len_q[b]*h)*topk + sum_{c'<c} col_nnz[b,h,c']
 *   indices has total_q*heads*topk entries; the unused tail of each (b,h) region is 0.
 * Replaces compute_topk_offset + compute_topk_epilogue_1rowblock
 * (csrc/flash_topk/src/flash_topk_kernel.h:376-402, 407-478) and varlen_sort
 * (csrc/flash_topk/src/varlen_sort.cu:127-162). */
int fmb_build_csc(const int32_t* topk_idx, int64_t topk_row_stride, int64_t topk_head_stride,
                  const int32_t* cu_seqlens_q, int64_t* col_offsets,
                  int32_t* col_nnz, int32_t* indices, void* workspace, size_t workspace_bytes,
                  int batch, int heads, int topk, int max_seqlen_q, int ncol,
                  fmb_stream_t stream);

/* fmb_build_csc that also writes the row-major view of the pattern it builds: row_slots
 * (uint32, total_q*heads*topk, index ((h*total_q + token)*topk + j)) receives, for place j of the
 * top-k list of (token, head h), the position in `indices` where that (row, chunk) pair was put, or
 * 0xffffffff for an empty place (chunk id < 0 or >= ncol).  Rows of sequences shorter than
 * max_seqlen_q and all tokens of the batch are covered; a list must not name a chunk twice (the
 * lists of fmb_gate_topk never do).  fmb_attn_rows_offer hands row_slots to the next fmb_attn_fwd
 * or fmb_attn_bwd call made by the same host thread: if that call's geometry matches (total_q,
 * heads, n_indices = total_q*heads*topk) and its workspace holds all heads in one pass, it uses an
 * entry's position in `indices` as its partial-result slot and these row lists, and launches none
 * of its own list-building kernels (the reference rebuilds nothing either: its kernels are
 * query-block-major, csrc/flash_moba/src/flash_fwd_kernel.h:232-769).  The offer is consumed by
 * that one call whether it is used or not; passing NULL withdraws it.  The pattern must be the
 * one fmb_build_csc_rows wrote together with row_slots (columns that do not overlap). */
int fmb_build_csc_rows(const int32_t* topk_idx, int64_t topk_row_stride, int64_t topk_head_stride,
                       const int32_t* cu_seqlens_q, int64_t* col_offsets, int32_t* col_nnz,
                       int32_t* indices, uint32_t* row_slots, void* workspace, size_t workspace_bytes,
                       int batch, int heads, int topk, int64_t total_q, int max_seqlen_q, int ncol,
                       fmb_stream_t stream);
int fmb_attn_rows_offer(const uint32_t* row_slots, int64_t total_q, int heads, int topk);

/* fmb_build_csc for callers that cannot allocate device memory.  This entry point has no
 * counterpart in the reference (there the C++ side allocates with torch::empty).  It is for
 * hosts that may not call cudaMalloc once they are running — a serving runtime that took
 * all device memory at start-up, a thin foreign-language shim that can only forward the
 * pointers it was handed — and so cannot supply the workspace fmb_build_csc wants.  The
 * scratch is a device array built into the library instead: 8 MiB
 * (fmb_build_csc_static_capacity()), held by every GPU that loads the library until the
 * process ends.  Inputs and outputs are still the caller's.  Limits and rules:
 *   - fmb_build_csc_workspace_bytes(batch, heads, max_seqlen_q, ncol) must not exceed the
 *     capacity, otherwise FMB_ERR_WORKSPACE is returned and nothing is launched;
 *   - all calls share the array; calls that overlap on the GPU (two streams, two host
 *     threads) race — keep them on one stream or order them with events;
 *   - the first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress); make that first call outside any stream capture.
 * It allocates nothing and gives bit-identical results to fmb_build_csc. */
size_t fmb_build_csc_static_capacity(void);
int fmb_build_csc_static(const int32_t* topk_idx, int64_t topk_row_stride, int64_t topk_head_stride,
                         const int32_t* cu_seqlens_q, int64_t* col_offsets, int32_t* col_nnz,
                         int32_t* indices, int batch, int heads, int topk, int max_seqlen_q, int ncol,
                         fmb_stream_t stream);

/* Ascending sort of int32 keys inside each segment [starts[i], ends[i]) of src into dst
 * (dst is first filled with 0).  Kept for callers of the reference's stand-alone
 * varlen_sort, csrc/flash_topk/src/varlen_sort.cu:127-162. */
int fmb_varlen_sort(const int64_t* starts, const int64_t* ends, const int32_t* src, int32_t* dst,
                    int64_t num_segments, int64_t num_items, fmb_stream_t stream);

/* ------------------------------------------------------------------ stage F: forward
 * Scratch for fmb_attn_fwd / fmb_attn_bwd.  The kernels keep one partial result per
 * (pattern entry, 128-key block of its chunk) in the workspace and work through the query
 * heads in passes, so the workspace only has to hold one pass:
 *   heads_per_pass <= 0 : bytes for a single pass over all heads (fastest);
 *   heads_per_pass  > 0 : bytes for passes of that many query heads (rounded down to whole
 *                         kv-head groups, at least one group).
 * fmb_attn_fwd / fmb_attn_bwd accept any workspace of at least the one-group size and use the
 * largest pass that fits.  n_indices = entries of `indices`; chunk = lg_block_n of the call. */
size_t fmb_attn_fwd_workspace_bytes(int64_t total_q, int heads, int heads_k, int head_dim,
                                    int64_t n_indices, int batch, int max_seqlen_k, int chunk,
                                    int heads_per_pass);
size_t fmb_attn_bwd_workspace_bytes(int64_t total_q, int heads, int heads_k, int head_dim,
                                    int64_t n_indices, int batch, int max_seqlen_k, int chunk,
                                    int heads_per_pass);

/* out[row,h] = softmax over the visible keys (scale * q.k) . v, where key col of the row's
 * sequence is visible iff chunk col/chunk is in the row's pattern, col < len_k and, if
 * causal, col <= row + len_k - len_q.  lse float (heads, total_q) = log-sum-exp of the
 * scaled scores; rows without visible keys give out = 0, lse = +inf.
 * head_dim: 64, 128 or 256 (the Python layer zero-pads anything else up to the next); chunk: a multiple of 64.
 * Replaces moba_varlen_fwd, csrc/flash_moba/flash_moba_api.cpp:375-596 and
 * csrc/flash_moba/src/flash_fwd_kernel.h:232-769. */
int fmb_attn_fwd(const void* q, int64_t q_row_stride, int64_t q_head_stride,
                 const void* k, int64_t k_row_stride, int64_t k_head_stride,
                 const void* v, int64_t v_row_stride, int64_t v_head_stride,
                 void* out, int64_t o_row_stride, int64_t o_head_stride, float* lse,
                 const int64_t* col_offsets, const int32_t* col_nnz, const int32_t* indices,
                 int64_t n_indices, const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k,
                 void* workspace, size_t workspace_bytes, int batch, int heads, int heads_k,
                 int head_dim, int64_t total_q, int max_seqlen_q, int max_seqlen_k, int chunk,
                 float softmax_scale, int causal, int dtype, fmb_stream_t stream);

/* Keys of a sequence that do not start at cu_seqlens_k[b] or end at cu_seqlens_k[b+1]: the next
 * fmb_attn_fwd call of this host thread reads sequence b's keys from rows [k_begin[b], k_end[b]) of
 * k and v (device int32[batch] each) instead; cu_seqlens_k is then only checked for NULL.  This is
 * how the reference's `leftpad_k` (k_begin[b] = cu_seqlens_k[b] + leftpad_k[b]) and `seqused_k`
 * (k_end[b] = cu_seqlens_k[b] + seqused_k[b]) arguments of its forward op are served
 * (csrc/flash_moba/src/block_info.h:19-26, csrc/flash_moba/flash_moba_api.cpp:477-482,558-564);
 * like there, the backward call has no such arguments.  max_seqlen_k must bound k_end - k_begin.
 * One-shot; (NULL, NULL) withdraws it. */
int fmb_attn_key_spans(const int32_t* k_begin, const int32_t* k_end);

/* ------------------------------------------------------------------ stage B: backward
 * dq/dk/dv for the forward above (dk/dv summed over the q heads of a kv head).
 * softmax_d float (heads, total_q) receives rowsum(dout*out).  Atomics-free and
 * deterministic.  Replaces moba_varlen_bwd, csrc/flash_moba/flash_moba_api.cpp:610-848,
 * csrc/flash_moba/src/flash_bwd_kernel.h:99-874 and
 * csrc/flash_moba/src/flash_bwd_preprocess_kernel.h:59-140, 146-232. */
int fmb_attn_bwd(const void* dout, int64_t do_row_stride, int64_t do_head_stride,
                 const void* q, int64_t q_row_stride, int64_t q_head_stride,
                 const void* k, int64_t k_row_stride, int64_t k_head_stride,
                 const void* v, int64_t v_row_stride, int64_t v_head_stride,
                 const void* out, int64_t o_row_stride, int64_t o_head_stride,
                 const float* lse, void* dq, int64_t dq_row_stride, int64_t dq_head_stride,
                 void* dk, int64_t dk_row_stride, int64_t dk_head_stride,
                 void* dv, int64_t dv_row_stride, int64_t dv_head_stride, float* softmax_d,
                 const int64_t* col_offsets, const int32_t* col_nnz, const int32_t* indices,
                 int64_t n_indices, const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k,
                 void* workspace, size_t workspace_bytes, int batch, int heads, int heads_k,
                 int head_dim, int64_t total_q, int64_t total_k, int max_seqlen_q,
                 int max_seqlen_k, int chunk, float softmax_scale, int causal, int dtype,
                 fmb_stream_t stream);

/* Selects the engine of the attention and gating kernels for this process: 0 = CUDA-core kernels,
 * 1 = tcgen05 tensor-core kernels (the default).  Testing aid; returns the engine now in use. */
int fmb_set_engine(int engine);

/* Which engine fmb_attn_fwd (backward = 0) or fmb_attn_bwd (backward = 1) will use for this
 * chunk size and head dimension under the current fmb_set_engine setting: 1 = tcgen05,
 * 0 = CUDA cores. */
int fmb_attn_engine(int chunk, int head_dim, int backward);

/* Same for fmb_gate_topk (tcgen05 for head_dim 64/128/256 and topk <= 32). */
int fmb_gate_engine(int head_dim, int topk);

/* Synchronising read of the gating kernel's device-side status word of the current device into
 * *host_status: 0 = ok, non-zero = a bounded wait expired in some gating launch since the last
 * read.  The word is cleared by the read.  Returns FMB_ERR_TIMEOUT when it was non-zero. */
int fmb_gate_status(int* host_status);

/* Synchronising read of the status word that fmb_attn_fwd / fmb_attn_bwd left in the first 4
 * bytes of `workspace` (see below), after the work enqueued on `stream` so far has completed.
 * *host_status receives the word; the return value is FMB_OK for 0, FMB_ERR_TIMEOUT for an
 * expired wait (1..6, 8), FMB_ERR_WORKSPACE for 7 and FMB_ERR_CUDA for 9. */
int fmb_attn_status(const void* workspace, int* host_status, fmb_stream_t stream);

/* Self test of the tcgen05 path, no counterpart in the reference: d[128][128] (float) =
 * a[128][128] . b, where b is [n][k] (k contiguous) if b_mn_major == 0, or [k][n]
 * (n contiguous) if 1; uses the same shared-memory descriptors as the attention kernels.
 * *status (device int, zeroed by the caller) receives a non-zero code if a bounded wait on
 * the device expired. */
int fmb_selftest_umma(const void* a, const void* b, float* d, int b_mn_major, int dtype, int* status,
                      fmb_stream_t stream);

/* Self test of the bounded wait every kernel of this library uses: one warp waits on an mbarrier
 * that nobody arrives at, gives up, records code 5 in *status (device int, set to 0 by the call
 * first) and the nanoseconds the wait lasted in *elapsed_ns (device uint64), and exits normally.
 * Nothing else runs in the kernel, so no copy or MMA is in flight when it gives up. */
int fmb_selftest_wait_expiry(int* status, unsigned long long* elapsed_ns, fmb_stream_t stream);

/* Optional hand-over of the pattern's slot and row lists (the CSR transpose that both attention
 * calls build in their workspace) from a forward call to the backward call of the same pattern.
 * No counterpart in the reference, whose kernels walk the pattern query-block-major and need no
 * transpose.  After fmb_attn_fwd: fmb_attn_lists_save copies the lists out of the forward
 * workspace into `lists` (fmb_attn_lists_bytes of device memory).  Before fmb_attn_bwd, on the
 * same host thread: fmb_attn_lists_load copies them into the backward workspace; the next
 * fmb_attn_bwd of this thread on that workspace and geometry then skips its own build (64K
 * tokens x 32 heads: 0.24 ms of 11).  Both return 0 when done, 1 when the workspace makes the
 * call run in several passes over the heads (nothing copied, fmb_attn_bwd builds its own lists),
 * an FMB_ERR_* code on bad arguments.  Same stream order as the attention calls. */
size_t fmb_attn_lists_bytes(int64_t total_q, int heads, int heads_k, int head_dim, int64_t n_indices,
                            int batch, int max_seqlen_k, int chunk);
int fmb_attn_lists_save(const void* fwd_workspace, size_t workspace_bytes, int64_t total_q, int heads,
                        int heads_k, int head_dim, int64_t n_indices, int batch, int max_seqlen_k,
                        int chunk, void* lists, size_t lists_bytes, fmb_stream_t stream);
int fmb_attn_lists_load(void* bwd_workspace, size_t workspace_bytes, int64_t total_q, int heads,
                        int heads_k, int head_dim, int64_t n_indices, int batch, int max_seqlen_k,
                        int chunk, const void* lists, size_t lists_bytes, fmb_stream_t stream);

/* The first 4 bytes of the workspace given to fmb_attn_fwd / fmb_attn_bwd hold a device-side
 * status word after the call: 0 = ok; 1..6 and 8 = a bounded wait inside a kernel expired
 * (FMB_ERR_TIMEOUT condition); 7 = the pattern's columns overlap or exceed the slots of a pass
 * (give a larger workspace); 9 = the kernel found its shared memory misaligned (a build problem).
 * Results are invalid when it is non-zero. */

/* Reading that word without a copy in the stream: fmb_attn_status_mirror(p) makes the next
 * fmb_attn_fwd / fmb_attn_bwd call of this host thread store its status word to *p once its main
 * kernels have completed (one store by one thread of its merge kernel; p must be writable by
 * the device and readable by the host, typically mapped pinned host memory).  The caller sets *p
 * to a "pending" value before the call and polls it, or looks at it after an event recorded
 * behind the call.  One-shot; NULL withdraws it.  (A 4-byte device-to-host copy in the stream
 * queues behind large copies of other streams on the same copy engine: measured 55 -> 61 ms per
 * step in a pipeline that overlaps result copies with kernels.) */
int fmb_attn_status_mirror(int* mirror);

/* ------------------------------------------------------------------ measurement aids
 * No counterpart in the reference (it is timed from Python with torch.utils.benchmark,
 * flash_moba/utils/benchmark.py:120-156).
 * Kernel launches made by this library in this process so far. */
unsigned long long fmb_launch_count(void);

/* CUDA-event timing of the dominant kernels on the launching stream.  While enabled, up to
 * 256 launches per kind are bracketed by events (no synchronisation is added); enabling
 * also clears the record.  kind: 0 forward main kernel, 1 backward main kernel, 2 gating
 * kernel, 3 mean-pool kernel, 4 forward combine, 5 backward combine, 6 pattern build (its
 * three kernels together), 7 dO.O.  After the caller has synchronised, fmb_profile_read stores
 * the elapsed milliseconds of each recorded launch and returns how many (or -1). */
int fmb_profile_enable(int on);
int fmb_profile_read(int kind, float* ms, int max_entries);
/* Restricts the bracketing to the kinds whose bit is set in `mask` (bit k = kind k; all kinds after
 * fmb_profile_enable): two event records per launch between short kernels are not free, and a
 * caller that times whole steps may want only the dominant kernel bracketed meanwhile. */
int fmb_profile_kinds(unsigned mask);

/* Strided host<->device copy of a head range: `rows` rows of `width_bytes` bytes, `src_pitch` /
 * `dst_pitch` bytes apart, enqueued on `stream` (cudaMemcpy2DAsync; the host side should be
 * pinned).  direction: 0 host->device, 1 device->host.  Used by the host pipeline that overlaps
 * the copies of one head group with the kernels of another.  No counterpart in the reference,
 * whose operands are device tensors. */
int fmb_copy_rows_async(void* dst, size_t dst_pitch, const void* src, size_t src_pitch, size_t width_bytes,
                        size_t rows, int direction, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FLASH_MOBA_B200_H_ */
