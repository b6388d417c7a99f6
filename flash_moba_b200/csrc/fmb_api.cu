// The C ABI (include/flash_moba_b200.h): argument validation, error reporting, dispatch.
#include <cstring>

#include "fmb_attn.cuh"

namespace fmb {

static thread_local char g_err[512] = "";
char* error_buffer() { return g_err; }

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

static int g_engine = 1;

static unsigned long long g_launches = 0;
void note_launch() { __atomic_fetch_add(&g_launches, 1ull, __ATOMIC_RELAXED); }

// ---- optional event timing of the dominant kernels ------------------------------------
constexpr int kProfKinds = 8, kProfRing = 256;
struct ProfState {
  bool on = false;
  unsigned kinds = ~0u;       // bit k: launches of kind k are bracketed
  cudaEvent_t ev[kProfKinds][kProfRing][2] = {};
  int count[kProfKinds] = {};
};
static ProfState g_prof;
void prof_begin(int kind, cudaStream_t s) {
  if (!g_prof.on || !((g_prof.kinds >> kind) & 1u) || g_prof.count[kind] >= kProfRing) return;
  cudaEvent_t& e = g_prof.ev[kind][g_prof.count[kind]][0];
  if (!e) cudaEventCreate(&e);
  cudaEventRecord(e, s);
}
void prof_end(int kind, cudaStream_t s) {
  if (!g_prof.on || !((g_prof.kinds >> kind) & 1u) || g_prof.count[kind] >= kProfRing) return;
  cudaEvent_t& e = g_prof.ev[kind][g_prof.count[kind]][1];
  if (!e) cudaEventCreate(&e);
  cudaEventRecord(e, s);
  ++g_prof.count[kind];
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

static int check_tensor(const char* name, const void* p, int64_t rs, int64_t hs, int d) {
  if (p == nullptr) return fail(FMB_ERR_BAD_ARG, "%s: null pointer", name);
  if (!aligned16(p) || rs % 8 != 0 || hs % 8 != 0)
    return fail(FMB_ERR_BAD_ARG, "%s: base pointer and row/head strides must be 16-byte aligned "
                "(strides %lld, %lld elements)", name, (long long)rs, (long long)hs);
  if (hs < d && hs != 0 && rs < d) return fail(FMB_ERR_BAD_ARG, "%s: overlapping strides", name);
  return FMB_OK;
}

static int check_common(const char* op, int heads, int heads_k, int d, int dtype) {
  if (dtype != FMB_BF16 && dtype != FMB_FP16)
    return fail(FMB_ERR_BAD_ARG, "%s: only fp16 and bf16 data types are supported", op);
  if (d <= 0 || d > 256) return fail(FMB_ERR_BAD_ARG, "%s: head dimension must be in (0, 256], got %d", op, d);
  if (d % 8 != 0) return fail(FMB_ERR_BAD_ARG, "%s: head dimension must be a multiple of 8, got %d", op, d);
  if (heads <= 0 || heads_k <= 0 || heads % heads_k != 0)
    return fail(FMB_ERR_BAD_ARG, "%s: number of heads in key/value must divide number of heads in query "
                "(%d, %d)", op, heads, heads_k);
  return FMB_OK;
}

}  // namespace fmb

using namespace fmb;

extern "C" {

int fmb_version(void) { return 100; }

const char* fmb_last_error(void) { return error_buffer(); }

unsigned long long fmb_launch_count(void) { return __atomic_load_n(&g_launches, __ATOMIC_RELAXED); }

int fmb_profile_enable(int on) {
  g_prof.on = on != 0;
  g_prof.kinds = ~0u;
  for (int k = 0; k < kProfKinds; ++k) g_prof.count[k] = 0;
  return FMB_OK;
}

int fmb_profile_kinds(unsigned mask) {
  g_prof.kinds = mask;
  return FMB_OK;
}

int fmb_profile_read(int kind, float* ms, int max_entries) {
  if (kind < 0 || kind >= kProfKinds || (!ms && max_entries > 0)) return -1;
  int n = g_prof.count[kind] < max_entries ? g_prof.count[kind] : max_entries;
  for (int i = 0; i < n; ++i) {
    if (cudaEventElapsedTime(&ms[i], g_prof.ev[kind][i][0], g_prof.ev[kind][i][1]) != cudaSuccess) {
      cudaGetLastError();
      return -1;
    }
  }
  return n;
}

int fmb_copy_rows_async(void* dst, size_t dst_pitch, const void* src, size_t src_pitch, size_t width_bytes,
                        size_t rows, int direction, void* stream) {
  if (rows == 0 || width_bytes == 0) return FMB_OK;
  if (!dst || !src || width_bytes > dst_pitch || width_bytes > src_pitch || (direction != 0 && direction != 1))
    return fail(FMB_ERR_BAD_ARG, "copy_rows: bad pointers, pitches (%zu, %zu) narrower than the width %zu, or direction %d",
                dst_pitch, src_pitch, width_bytes, direction);
  FMB_CUDA(cudaMemcpy2DAsync(dst, dst_pitch, src, src_pitch, width_bytes, rows,
                             direction == 0 ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToHost, (cudaStream_t)stream));
  return FMB_OK;
}

int fmb_attn_engine(int chunk, int head_dim, int backward) {
  AttnArgs a;
  memset(&a, 0, sizeof(a));
  a.chunk = chunk; a.d = head_dim; a.heads = 1;
  a.q_rs = a.do_rs = head_dim; a.q_hs = a.do_hs = head_dim;   // a packed layout
  return (g_engine == 1 && (tc_supported(a, backward != 0) || tc_wide_supported(a, backward != 0))) ? 1 : 0;
}

int fmb_selftest_umma(const void* a, const void* b, float* d, int b_mn_major, int dtype, int* status,
                      fmb_stream_t stream) {
  FMB_CHECK_ARG(a && b && d && status, "selftest_umma: null pointer");
  FMB_CHECK_ARG(dtype == FMB_BF16 || dtype == FMB_FP16, "selftest_umma: only fp16 and bf16");
  return launch_selftest_umma(a, b, d, b_mn_major, dtype, status, (cudaStream_t)stream);
}

int fmb_set_engine(int engine) {
  if (engine == 0 || engine == 1) {
    g_engine = engine;
    set_gate_engine(engine);
  }
  return g_engine;
}

int fmb_gate_engine(int head_dim, int topk) { return (g_engine == 1 && gate_tc_supported(head_dim, topk)) ? 1 : 0; }

int fmb_gate_status(int* host_status) {
  FMB_CHECK_ARG(host_status, "gate_status: null pointer");
  const int rc = read_gate_status(host_status);
  if (rc) return rc;
  if (*host_status != 0)
    return fail(FMB_ERR_TIMEOUT, "gate_topk: a bounded device-side wait expired (code %d)", *host_status);
  return FMB_OK;
}

int fmb_attn_status(const void* workspace, int* host_status, fmb_stream_t stream) {
  FMB_CHECK_ARG(workspace && host_status, "attn_status: null pointer");
  FMB_CUDA(cudaMemcpyAsync(host_status, workspace, sizeof(int), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
  FMB_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
  const int code = *host_status;
  if (code == 0) return FMB_OK;
  if (code == 7)
    return fail(FMB_ERR_WORKSPACE, "attention: the pattern does not fit the slots of a pass (columns that overlap, "
                "or a workspace too small for this pattern)");
  if (code == 9) return fail(FMB_ERR_CUDA, "attention: a kernel found its shared memory misaligned");
  return fail(FMB_ERR_TIMEOUT, "attention: a bounded device-side wait expired (code %d)", code);
}

int fmb_attn_status_mirror(int* mirror) {
  attn_status_mirror(mirror);
  return FMB_OK;
}

int fmb_selftest_wait_expiry(int* status, unsigned long long* elapsed_ns, fmb_stream_t stream) {
  FMB_CHECK_ARG(status && elapsed_ns, "selftest_wait_expiry: null pointer");
  return launch_selftest_wait_expiry(status, elapsed_ns, (cudaStream_t)stream);
}

int fmb_chunk_offsets(const int32_t* cu_seqlens_k, int batch, int chunk, int32_t* cu_seqlens_km,
                      fmb_stream_t stream) {
  FMB_CHECK_ARG(cu_seqlens_k && cu_seqlens_km, "chunk_offsets: null pointer");
  FMB_CHECK_ARG(batch >= 0 && chunk > 0, "chunk_offsets: batch >= 0 and chunk > 0 required");
  return launch_chunk_offsets(cu_seqlens_k, batch, chunk, cu_seqlens_km, (cudaStream_t)stream);
}

int fmb_mean_pool(const void* k, int64_t k_row_stride, int64_t k_head_stride, const int32_t* cu_seqlens_k,
                  const int32_t* cu_seqlens_km, void* km, int batch, int heads_k, int head_dim,
                  int max_seqlen_k, int chunk, int dtype, fmb_stream_t stream) {
  int rc = check_common("mean_pool", heads_k, heads_k, head_dim, dtype);
  if (rc) return rc;
  FMB_CHECK_ARG(chunk > 0 && batch >= 0 && max_seqlen_k >= 0, "mean_pool: bad sizes");
  FMB_CHECK_ARG(cu_seqlens_k && cu_seqlens_km, "mean_pool: null cu_seqlens");
  if (batch == 0 || max_seqlen_k == 0) return FMB_OK;
  if ((rc = check_tensor("mean_pool: k", k, k_row_stride, k_head_stride, head_dim))) return rc;
  FMB_CHECK_ARG(km && aligned16(km), "mean_pool: km must be non-null and 16-byte aligned");
  FMB_CHECK_ARG(heads_k <= 65535 && batch <= 65535, "mean_pool: heads_k and batch must be <= 65535");
  return launch_mean_pool(k, k_row_stride, k_head_stride, cu_seqlens_k, const_cast<int32_t*>(cu_seqlens_km), km, batch,
                          heads_k, head_dim, max_seqlen_k, chunk, dtype, (cudaStream_t)stream);
}

int fmb_mean_pool_offsets(const void* k, int64_t k_row_stride, int64_t k_head_stride, const int32_t* cu_seqlens_k,
                          int32_t* cu_seqlens_km, void* km, int batch, int heads_k, int head_dim,
                          int max_seqlen_k, int chunk, int dtype, fmb_stream_t stream) {
  int rc = check_common("mean_pool", heads_k, heads_k, head_dim, dtype);
  if (rc) return rc;
  FMB_CHECK_ARG(chunk > 0 && batch >= 0 && max_seqlen_k >= 0, "mean_pool: bad sizes");
  FMB_CHECK_ARG(cu_seqlens_k && cu_seqlens_km, "mean_pool: null cu_seqlens");
  if (batch == 0 || max_seqlen_k == 0)     // nothing to pool: the offsets alone
    return launch_chunk_offsets(cu_seqlens_k, batch, chunk, cu_seqlens_km, (cudaStream_t)stream);
  if ((rc = check_tensor("mean_pool: k", k, k_row_stride, k_head_stride, head_dim))) return rc;
  FMB_CHECK_ARG(km && aligned16(km), "mean_pool: km must be non-null and 16-byte aligned");
  FMB_CHECK_ARG(heads_k <= 65535 && batch <= 65535, "mean_pool: heads_k and batch must be <= 65535");
  return launch_mean_pool(k, k_row_stride, k_head_stride, cu_seqlens_k, cu_seqlens_km, km, batch, heads_k, head_dim,
                          max_seqlen_k, chunk, dtype, (cudaStream_t)stream, true);
}

int fmb_gate_topk(const void* q, int64_t q_row_stride, int64_t q_head_stride, const void* km,
                  const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k, const int32_t* cu_seqlens_km,
                  int32_t* topk_idx, float* topk_val, int64_t topk_row_stride, int64_t topk_head_stride,
                  int batch, int heads, int heads_k, int head_dim, int max_seqlen_q, int max_seqlen_k,
                  int topk, int chunk, int causal, int dtype, fmb_stream_t stream) {
  int rc = check_common("gate_topk", heads, heads_k, head_dim, dtype);
  if (rc) return rc;
  FMB_CHECK_ARG(topk >= 1 && topk <= 64, "gate_topk: moba_topk must be in [1, 64], got %d", topk);
  FMB_CHECK_ARG(chunk > 0, "gate_topk: moba_chunk_size must be positive");
  FMB_CHECK_ARG(cu_seqlens_q && cu_seqlens_k && cu_seqlens_km && topk_idx, "gate_topk: null pointer");
  FMB_CHECK_ARG(batch >= 0 && max_seqlen_q >= 0 && max_seqlen_k >= 0, "gate_topk: bad sizes");
  if (batch == 0 || max_seqlen_q == 0) return FMB_OK;
  if ((rc = check_tensor("gate_topk: q", q, q_row_stride, q_head_stride, head_dim))) return rc;
  FMB_CHECK_ARG(max_seqlen_k == 0 || (km && aligned16(km)), "gate_topk: km must be 16-byte aligned");
  FMB_CHECK_ARG(heads <= 65535 && batch <= 65535, "gate_topk: heads and batch must be <= 65535");
  GateArgs a;
  a.q = q; a.q_rs = q_row_stride; a.q_hs = q_head_stride; a.km = km;
  a.cu_q = cu_seqlens_q; a.cu_k = cu_seqlens_k; a.cu_km = cu_seqlens_km;
  a.topk_idx = topk_idx; a.topk_val = topk_val; a.t_rs = topk_row_stride; a.t_hs = topk_head_stride;
  a.batch = batch; a.heads = heads; a.heads_k = heads_k; a.d = head_dim; a.max_q = max_seqlen_q;
  a.max_k = max_seqlen_k; a.topk = topk; a.chunk = chunk; a.causal = causal; a.dtype = dtype;
  return launch_gate_topk(a, (cudaStream_t)stream);
}

size_t fmb_build_csc_workspace_bytes(int batch, int heads, int max_seqlen_q, int ncol) {
  return csc_workspace_bytes(batch, heads, max_seqlen_q, ncol);
}

int fmb_build_csc(const int32_t* topk_idx, int64_t topk_row_stride, int64_t topk_head_stride,
                  const int32_t* cu_seqlens_q, int64_t* col_offsets, int32_t* col_nnz, int32_t* indices,
                  void* workspace, size_t workspace_bytes, int batch, int heads, int topk, int max_seqlen_q,
                  int ncol, fmb_stream_t stream) {
  FMB_CHECK_ARG(batch >= 0 && heads >= 0 && topk >= 1 && max_seqlen_q >= 0 && ncol >= 0, "build_csc: bad sizes");
  if (batch == 0 || heads == 0 || ncol == 0) return FMB_OK;
  FMB_CHECK_ARG(topk_idx && cu_seqlens_q && col_offsets && col_nnz && indices, "build_csc: null pointer");
  FMB_CHECK_ARG(max_seqlen_q / 512 < 65535, "build_csc: max_seqlen_q too large");
  return launch_build_csc(topk_idx, topk_row_stride, topk_head_stride, cu_seqlens_q, col_offsets, col_nnz,
                          indices, workspace, workspace_bytes, batch, heads, topk, max_seqlen_q, ncol,
                          (cudaStream_t)stream);
}

int fmb_build_csc_rows(const int32_t* topk_idx, int64_t topk_row_stride, int64_t topk_head_stride,
                       const int32_t* cu_seqlens_q, int64_t* col_offsets, int32_t* col_nnz, int32_t* indices,
                       uint32_t* row_slots, void* workspace, size_t workspace_bytes, int batch, int heads, int topk,
                       int64_t total_q, int max_seqlen_q, int ncol, fmb_stream_t stream) {
  FMB_CHECK_ARG(batch >= 0 && heads >= 0 && topk >= 1 && max_seqlen_q >= 0 && ncol >= 0 && total_q >= 0,
                "build_csc_rows: bad sizes");
  FMB_CHECK_ARG(total_q * heads * topk < (int64_t)0xffffffffll, "build_csc_rows: more than 2^32 - 1 pattern entries");
  if (batch == 0 || heads == 0) return FMB_OK;
  FMB_CHECK_ARG(topk_idx && cu_seqlens_q && col_offsets && col_nnz && indices && row_slots, "build_csc_rows: null pointer");
  FMB_CHECK_ARG(max_seqlen_q / 512 < 65535, "build_csc_rows: max_seqlen_q too large");
  if (ncol == 0) {   // no columns at all: every place of every row list is empty
    FMB_CUDA(cudaMemsetAsync(row_slots, 0xff, (size_t)total_q * heads * topk * sizeof(uint32_t), (cudaStream_t)stream));
    return FMB_OK;
  }
  return launch_build_csc(topk_idx, topk_row_stride, topk_head_stride, cu_seqlens_q, col_offsets, col_nnz,
                          indices, workspace, workspace_bytes, batch, heads, topk, max_seqlen_q, ncol,
                          (cudaStream_t)stream, row_slots, total_q);
}

int fmb_attn_rows_offer(const uint32_t* row_slots, int64_t total_q, int heads, int topk) {
  FMB_CHECK_ARG(row_slots == nullptr || (total_q >= 0 && heads > 0 && topk > 0), "attn_rows_offer: bad sizes");
  attn_rows_offer(row_slots, total_q, heads, topk);
  return FMB_OK;
}

size_t fmb_build_csc_static_capacity(void) { return csc_static_scratch_bytes(); }

int fmb_build_csc_static(const int32_t* topk_idx, int64_t topk_row_stride, int64_t topk_head_stride,
                         const int32_t* cu_seqlens_q, int64_t* col_offsets, int32_t* col_nnz, int32_t* indices,
                         int batch, int heads, int topk, int max_seqlen_q, int ncol, fmb_stream_t stream) {
  FMB_CHECK_ARG(batch >= 0 && heads >= 0 && topk >= 1 && max_seqlen_q >= 0 && ncol >= 0,
                "build_csc_static: bad sizes");
  if (batch == 0 || heads == 0 || ncol == 0) return FMB_OK;
  FMB_CHECK_ARG(topk_idx && cu_seqlens_q && col_offsets && col_nnz && indices, "build_csc_static: null pointer");
  FMB_CHECK_ARG(max_seqlen_q / 512 < 65535, "build_csc_static: max_seqlen_q too large");
  return launch_build_csc_static(topk_idx, topk_row_stride, topk_head_stride, cu_seqlens_q, col_offsets, col_nnz,
                                 indices, batch, heads, topk, max_seqlen_q, ncol, (cudaStream_t)stream);
}

int fmb_varlen_sort(const int64_t* starts, const int64_t* ends, const int32_t* src, int32_t* dst,
                    int64_t num_segments, int64_t num_items, fmb_stream_t stream) {
  FMB_CHECK_ARG(num_segments >= 0 && num_items >= 0, "varlen_sort: bad sizes");
  if (num_items == 0) return FMB_OK;
  FMB_CHECK_ARG(src && dst && (num_segments == 0 || (starts && ends)), "varlen_sort: null pointer");
  return launch_varlen_sort(starts, ends, src, dst, num_segments, num_items, (cudaStream_t)stream);
}

size_t fmb_attn_fwd_workspace_bytes(int64_t total_q, int heads, int heads_k, int head_dim, int64_t n_indices,
                                    int batch, int max_seqlen_k, int chunk, int heads_per_pass) {
  return attn_workspace_bytes(total_q, heads, heads_k, head_dim, n_indices, batch, max_seqlen_k, chunk,
                              heads_per_pass, false);
}
size_t fmb_attn_bwd_workspace_bytes(int64_t total_q, int heads, int heads_k, int head_dim, int64_t n_indices,
                                    int batch, int max_seqlen_k, int chunk, int heads_per_pass) {
  return attn_workspace_bytes(total_q, heads, heads_k, head_dim, n_indices, batch, max_seqlen_k, chunk,
                              heads_per_pass, true);
}

static AttnArgs lists_geometry(const void* ws, size_t ws_bytes, int64_t total_q, int heads, int heads_k,
                               int head_dim, int64_t n_indices, int batch, int max_seqlen_k, int chunk) {
  AttnArgs a;
  memset(&a, 0, sizeof(a));
  a.ws = const_cast<void*>(ws); a.ws_bytes = ws_bytes;
  a.total_q = total_q; a.heads = heads; a.heads_k = heads_k > 0 ? heads_k : heads; a.d = head_dim;
  a.n_indices = n_indices; a.batch = batch; a.chunk = chunk > 0 ? chunk : 128;
  a.ncol = ceil_div(max_seqlen_k, a.chunk);
  return a;
}
size_t fmb_attn_lists_bytes(int64_t total_q, int heads, int heads_k, int head_dim, int64_t n_indices, int batch,
                            int max_seqlen_k, int chunk) {
  if (heads <= 0) return 0;
  return attn_lists_bytes(lists_geometry(nullptr, 0, total_q, heads, heads_k, head_dim, n_indices, batch,
                                         max_seqlen_k, chunk));
}
int fmb_attn_lists_save(const void* fwd_workspace, size_t workspace_bytes, int64_t total_q, int heads, int heads_k,
                        int head_dim, int64_t n_indices, int batch, int max_seqlen_k, int chunk, void* lists,
                        size_t lists_bytes, fmb_stream_t stream) {
  FMB_CHECK_ARG(heads > 0 && chunk > 0 && chunk % 64 == 0, "attn_lists_save: bad geometry");
  return attn_lists_save(lists_geometry(fwd_workspace, workspace_bytes, total_q, heads, heads_k, head_dim, n_indices,
                                        batch, max_seqlen_k, chunk),
                         lists, lists_bytes, (cudaStream_t)stream);
}
int fmb_attn_lists_load(void* bwd_workspace, size_t workspace_bytes, int64_t total_q, int heads, int heads_k,
                        int head_dim, int64_t n_indices, int batch, int max_seqlen_k, int chunk, const void* lists,
                        size_t lists_bytes, fmb_stream_t stream) {
  FMB_CHECK_ARG(heads > 0 && chunk > 0 && chunk % 64 == 0, "attn_lists_load: bad geometry");
  return attn_lists_load(lists_geometry(bwd_workspace, workspace_bytes, total_q, heads, heads_k, head_dim, n_indices,
                                        batch, max_seqlen_k, chunk),
                         lists, lists_bytes, (cudaStream_t)stream);
}

static int check_attn(const char* op, const AttnArgs& a) {
  int rc = check_common(op, a.heads, a.heads_k, a.d, a.dtype);
  if (rc) return rc;
  FMB_CHECK_ARG(a.chunk > 0 && a.chunk % 64 == 0, "%s: lg_block_n (chunk) must be a multiple of 64, got %d", op,
                a.chunk);
  FMB_CHECK_ARG(a.batch >= 0 && a.total_q >= 0 && a.max_q >= 0 && a.max_k >= 0 && a.n_indices >= 0,
                "%s: bad sizes", op);
  FMB_CHECK_ARG(a.n_indices < (int64_t)0xffffffffll, "%s: pattern has too many entries", op);
  FMB_CHECK_ARG(a.total_q * a.heads < (int64_t)0xfffffffell, "%s: too many (token, head) rows", op);
  FMB_CHECK_ARG(a.cu_q && a.cu_k, "%s: null cu_seqlens", op);
  FMB_CHECK_ARG(a.ncol == 0 || (a.col_offsets && a.col_nnz), "%s: null pattern", op);
  FMB_CHECK_ARG(a.n_indices == 0 || a.indices, "%s: null pattern indices", op);
  FMB_CHECK_ARG(a.heads <= 65535 && a.batch <= 65535, "%s: heads and batch must be <= 65535", op);
  return FMB_OK;
}

static thread_local const int32_t* g_key_spans[2] = {nullptr, nullptr};

int fmb_attn_key_spans(const int32_t* k_begin, const int32_t* k_end) {
  FMB_CHECK_ARG((k_begin == nullptr) == (k_end == nullptr), "attn_key_spans: give both arrays or neither");
  g_key_spans[0] = k_begin;
  g_key_spans[1] = k_end;
  return FMB_OK;
}

int fmb_attn_fwd(const void* q, int64_t q_row_stride, int64_t q_head_stride, const void* k,
                 int64_t k_row_stride, int64_t k_head_stride, const void* v, int64_t v_row_stride,
                 int64_t v_head_stride, void* out, int64_t o_row_stride, int64_t o_head_stride, float* lse,
                 const int64_t* col_offsets, const int32_t* col_nnz, const int32_t* indices, int64_t n_indices,
                 const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k, void* workspace,
                 size_t workspace_bytes, int batch, int heads, int heads_k, int head_dim, int64_t total_q,
                 int max_seqlen_q, int max_seqlen_k, int chunk, float softmax_scale, int causal, int dtype,
                 fmb_stream_t stream) {
  AttnArgs a;
  memset(&a, 0, sizeof(a));
  a.q = q; a.k = k; a.v = v; a.o = out;
  a.q_rs = q_row_stride; a.q_hs = q_head_stride; a.k_rs = k_row_stride; a.k_hs = k_head_stride;
  a.v_rs = v_row_stride; a.v_hs = v_head_stride; a.o_rs = o_row_stride; a.o_hs = o_head_stride;
  a.lse = lse; a.col_offsets = col_offsets; a.col_nnz = col_nnz; a.indices = indices; a.n_indices = n_indices;
  a.cu_q = cu_seqlens_q; a.cu_k = cu_seqlens_k; a.ws = workspace; a.ws_bytes = workspace_bytes;
  a.k_begin = cu_seqlens_k; a.k_end = cu_seqlens_k ? cu_seqlens_k + 1 : nullptr;
  if (g_key_spans[0] != nullptr) {      // one-shot: spans given for this call (fmb_attn_key_spans)
    a.k_begin = g_key_spans[0]; a.k_end = g_key_spans[1];
    g_key_spans[0] = g_key_spans[1] = nullptr;
  }
  a.batch = batch; a.heads = heads; a.heads_k = heads_k; a.d = head_dim; a.total_q = total_q;
  a.max_q = max_seqlen_q; a.max_k = max_seqlen_k; a.chunk = chunk;
  a.ncol = chunk > 0 ? ceil_div(max_seqlen_k, chunk) : 0;
  a.scale = softmax_scale; a.causal = causal; a.dtype = dtype;
  int rc = check_attn("attn_fwd", a);
  if (rc) return rc;
  if (total_q == 0 || batch == 0) return FMB_OK;
  if ((rc = check_tensor("attn_fwd: q", q, q_row_stride, q_head_stride, head_dim))) return rc;
  if (max_seqlen_k > 0) {
    if ((rc = check_tensor("attn_fwd: k", k, k_row_stride, k_head_stride, head_dim))) return rc;
    if ((rc = check_tensor("attn_fwd: v", v, v_row_stride, v_head_stride, head_dim))) return rc;
  }
  if ((rc = check_tensor("attn_fwd: out", out, o_row_stride, o_head_stride, head_dim))) return rc;
  FMB_CHECK_ARG(lse, "attn_fwd: null lse");
  return launch_attn_fwd(a, g_engine, (cudaStream_t)stream);
}

int fmb_attn_bwd(const void* dout, int64_t do_row_stride, int64_t do_head_stride, const void* q,
                 int64_t q_row_stride, int64_t q_head_stride, const void* k, int64_t k_row_stride,
                 int64_t k_head_stride, const void* v, int64_t v_row_stride, int64_t v_head_stride,
                 const void* out, int64_t o_row_stride, int64_t o_head_stride, const float* lse, void* dq,
                 int64_t dq_row_stride, int64_t dq_head_stride, void* dk, int64_t dk_row_stride,
                 int64_t dk_head_stride, void* dv, int64_t dv_row_stride, int64_t dv_head_stride,
                 float* softmax_d, const int64_t* col_offsets, const int32_t* col_nnz, const int32_t* indices,
                 int64_t n_indices, const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k, void* workspace,
                 size_t workspace_bytes, int batch, int heads, int heads_k, int head_dim, int64_t total_q,
                 int64_t total_k, int max_seqlen_q, int max_seqlen_k, int chunk, float softmax_scale,
                 int causal, int dtype, fmb_stream_t stream) {
  AttnArgs a;
  memset(&a, 0, sizeof(a));
  a.q = q; a.k = k; a.v = v; a.o = out; a.dout = dout;
  a.q_rs = q_row_stride; a.q_hs = q_head_stride; a.k_rs = k_row_stride; a.k_hs = k_head_stride;
  a.v_rs = v_row_stride; a.v_hs = v_head_stride; a.o_rs = o_row_stride; a.o_hs = o_head_stride;
  a.do_rs = do_row_stride; a.do_hs = do_head_stride;
  a.dq = dq; a.dk = dk; a.dv = dv;
  a.dq_rs = dq_row_stride; a.dq_hs = dq_head_stride; a.dk_rs = dk_row_stride; a.dk_hs = dk_head_stride;
  a.dv_rs = dv_row_stride; a.dv_hs = dv_head_stride;
  a.lse = const_cast<float*>(lse); a.softmax_d = softmax_d;
  a.col_offsets = col_offsets; a.col_nnz = col_nnz; a.indices = indices; a.n_indices = n_indices;
  a.cu_q = cu_seqlens_q; a.cu_k = cu_seqlens_k; a.ws = workspace; a.ws_bytes = workspace_bytes;
  a.k_begin = cu_seqlens_k; a.k_end = cu_seqlens_k ? cu_seqlens_k + 1 : nullptr;
  a.batch = batch; a.heads = heads; a.heads_k = heads_k; a.d = head_dim; a.total_q = total_q;
  a.total_k = total_k; a.max_q = max_seqlen_q; a.max_k = max_seqlen_k; a.chunk = chunk;
  a.ncol = chunk > 0 ? ceil_div(max_seqlen_k, chunk) : 0;
  a.scale = softmax_scale; a.causal = causal; a.dtype = dtype;
  int rc = check_attn("attn_bwd", a);
  if (rc) return rc;
  if (batch == 0 || (total_q == 0 && total_k == 0)) return FMB_OK;
  if (total_q > 0) {
    if ((rc = check_tensor("attn_bwd: dout", dout, do_row_stride, do_head_stride, head_dim))) return rc;
    if ((rc = check_tensor("attn_bwd: q", q, q_row_stride, q_head_stride, head_dim))) return rc;
    if ((rc = check_tensor("attn_bwd: out", out, o_row_stride, o_head_stride, head_dim))) return rc;
    if ((rc = check_tensor("attn_bwd: dq", dq, dq_row_stride, dq_head_stride, head_dim))) return rc;
    FMB_CHECK_ARG(lse && softmax_d, "attn_bwd: null lse / softmax_d");
  }
  if (total_k > 0) {
    if ((rc = check_tensor("attn_bwd: k", k, k_row_stride, k_head_stride, head_dim))) return rc;
    if ((rc = check_tensor("attn_bwd: v", v, v_row_stride, v_head_stride, head_dim))) return rc;
    if ((rc = check_tensor("attn_bwd: dk", dk, dk_row_stride, dk_head_stride, head_dim))) return rc;
    if ((rc = check_tensor("attn_bwd: dv", dv, dv_row_stride, dv_head_stride, head_dim))) return rc;
  }
  return launch_attn_bwd(a, g_engine, (cudaStream_t)stream);
}

}  // extern "C"
