// Shared pieces of the block-sparse attention (stages F and B).
//
// Both passes are KEY-CHUNK-MAJOR: a CTA owns one key chunk of one (sequence, head) and
// walks the chunk's CSC column, i.e. the gathered list of query rows that selected it, in
// dense tiles.  A (row, chunk) pair is item `pos` of the flat `indices` array, and that
// position is also where the pair's partial result lives in the workspace:
//   forward : part_o[pos][d]  (chunk-local softmax(QK^T)V, normalised, in the I/O dtype)
//             part_lse[pos]   (chunk-local log-sum-exp, natural log, of the scaled scores)
//   backward: part_dq[pos][d] (softmax_scale * dS.K of that chunk, in the I/O dtype)
// A row-major "combine" kernel then merges the partials of each row in ascending `pos`
// order, found through a CSR transpose of the pattern (row_ptr / row_pos) that is rebuilt
// per call with integer atomics; the merge order is fixed by sorting, so results are
// run-to-run deterministic and no floating-point atomics are used anywhere.
#pragma once
#include "fmb_common.cuh"

namespace fmb {

// Partial rows are stored with their 16-byte chunks permuted: chunk c of the pair at position
// `pos` sits at chunk (c ^ (pos & 7)).  The tensor-core kernels stage a tile of partial rows
// in shared memory before one bulk copy per warp; with this permutation the 32 lanes of a
// warp (consecutive positions) write their rows without bank conflicts, and the linear copy
// preserves it.  Writers and the combine kernels use part_col() for the element index.
__host__ __device__ __forceinline__ int part_col(int64_t pos, int col, int elems_per_chunk) {
  const int chunk = col / elems_per_chunk;
  return ((chunk ^ (int)(pos & 7)) * elems_per_chunk) + (col % elems_per_chunk);
}

// A call is processed in one or more PASSES over ranges of query heads [h0, h0+nh), so that the
// per-pair partials need memory for one pass only.  Inside a pass, column (b, h, c) owns the
// slots [slot_base, slot_base + nnz) of every partial array ("slot" = running count of pattern
// entries over the pass's columns in (b, h, c) order), and a key chunk wider than the kernels'
// key block KB is handled as nsub = chunk / KB sub-blocks, each with its own plane of `cap`
// slots: the partial of (entry j of the column, sub-block sb) lives at sb*cap + slot_base + j.
struct AttnWorkspace {
  int* status;          // first word: 0, or where a bounded device wait gave up (1-6, 8) / 7 = slot overflow / 9 = misaligned shared memory
  void* part_o;         // nsub*cap*d elements of the I/O dtype (fwd: O partials, bwd: dQ partials)
  float* part_lse;      // fwd only: nsub*cap
  uint32_t* slot_base;  // batch*nh*ncol + 1
  uint32_t* row_ptr;    // nh*total_q + 1
  uint32_t* row_fill;   // nh*total_q
  uint32_t* row_pos;    // cap: slots of a row's entries
  uint32_t* scan_tmp;   // block sums of the scans
  int fixed_k;          // > 0: row lists handed over by the pattern builder (see attn_rows_offer)
  int* mirror;          // where the call's status word is copied at its end (see attn_status_mirror), or nullptr
  int nh;               // heads per pass
  int nsub, kb;         // sub-blocks per chunk, keys per sub-block
  int64_t cap;          // slots per plane
  size_t bytes;
  size_t lists_off, lists_bytes;   // slot_base .. row_pos: what a backward call can take over from a forward call
};

// Pass geometry + pattern access shared by every attention kernel
struct PassParams {
  const int64_t* col_offsets; const int32_t* col_nnz; const int32_t* indices; int64_t n_indices;
  const uint32_t* slot_base;
  int heads, ncol, h0, nh, nsub, kb, chunk;
  int64_t cap;
  int64_t slot_shift;   // without a slot table: slot = position in `indices` - slot_shift (the first position
                        // of the pass's heads; single sequences only, whose heads are contiguous in `indices`)
  int* status;
};
struct ColRef {
  int nnz;          // 0 if the column is empty, malformed or does not fit the pass's slots
  int64_t off;      // first entry in `indices`
  int64_t slot;     // first slot of the column in the pass
};
__device__ __forceinline__ ColRef column_of(const PassParams& r, int b, int h, int c) {
  ColRef o{0, 0, 0};
  if (c >= r.ncol) return o;
  const int64_t ci = ((int64_t)b * r.heads + h) * r.ncol + c;
  const int nnz = r.col_nnz[ci];
  const int64_t off = r.col_offsets[ci];
  if (nnz <= 0 || off < 0 || off + nnz > r.n_indices) return o;   // malformed: ignored, never read
  // no slot table: the pattern builder vouches for columns that do not overlap, and an entry's
  // slot is simply its position in `indices`
  const int64_t slot = r.slot_base ? (int64_t)r.slot_base[((int64_t)b * r.nh + (h - r.h0)) * r.ncol + c]
                                   : off - r.slot_shift;
  if (slot < 0 || slot + nnz > r.cap) {          // cannot happen for a pattern whose columns do not overlap
    atomicCAS(r.status, 0, 7);
    return o;
  }
  o.nnz = nnz; o.off = off; o.slot = slot;
  return o;
}

// A key block that starts beyond the sequence's keys contributes nothing: its dQ partials are
// zero (the combine still reads them).  Called by a whole CTA of the backward kernels (or, _by, by `nthreads` threads numbered `tid`).
template <typename T>
__device__ __forceinline__ void zero_dq_partials_by(const PassParams& r, T* part_dq, int64_t plane, int b, int hk,
                                                    int group, int c, int d, int tid, int nthreads) {
  for (int hg = 0; hg < group; ++hg) {
    const ColRef col = column_of(r, b, hk * group + hg, c);
    if (col.nnz <= 0) continue;
    uint4* dst = reinterpret_cast<uint4*>(part_dq + (plane + col.slot) * d);
    const int64_t n16 = (int64_t)col.nnz * d * (int64_t)sizeof(T) / 16;
    for (int64_t i = tid; i < n16; i += nthreads) dst[i] = make_uint4(0, 0, 0, 0);
  }
}
template <typename T>
__device__ __forceinline__ void zero_dq_partials(const PassParams& r, T* part_dq, int64_t plane, int b, int hk,
                                                 int group, int c, int d) {
  zero_dq_partials_by<T>(r, part_dq, plane, b, hk, group, c, d, threadIdx.x, blockDim.x);
}

AttnWorkspace carve_attn_workspace(void* base, size_t bytes_available, const AttnArgs& a, size_t part_elem_bytes,
                                   bool with_lse, int heads_per_pass);
PassParams make_pass(const AttnArgs& a, const AttnWorkspace& w, int h0, int nh);

// The slot and row lists depend on the pattern alone, so a backward call can take over the lists
// the forward call of the same pattern built, when both run in one pass over all heads.
// attn_lists_save copies them out of a forward workspace; attn_lists_load copies them into a
// backward workspace and arms the next launch_attn_bwd of this thread on that workspace to skip
// its own build.  Both return 1 (and do nothing) when the workspace makes the call multi-pass.
size_t attn_lists_bytes(const AttnArgs& geometry);
int attn_lists_save(const AttnArgs& geometry_and_ws, void* dst, size_t dst_bytes, cudaStream_t s);
int attn_lists_load(const AttnArgs& geometry_and_ws, const void* src, size_t src_bytes, cudaStream_t s);

// The pattern builder can hand over the row-major view of its pattern (fmb_build_csc_rows): for
// entry j of row (h, token)'s top-k list, the position in `indices` of that (row, chunk) pair, or
// 0xffffffff.  attn_rows_offer arms the next attention call of this thread (forward or backward,
// one pass over all heads, same geometry) to use positions in `indices` as slots and these rows
// instead of building slot and row lists.
void attn_rows_offer(const uint32_t* row_slots, int64_t total_q, int heads, int topk);
// One-shot, per host thread: the next attention call copies its status word to *mirror (memory the
// device can write and the host can read, e.g. mapped pinned memory) when its main kernels are done.
void attn_status_mirror(int* mirror);

// Builds slot_base and row_ptr / row_pos (CSR transpose of the pass's part of the pattern).
// Row id = (h - h0)*total_q + token.
int build_row_lists(const AttnArgs& a, const AttnWorkspace& w, const PassParams& ps, cudaStream_t s);

// out/lse from the forward partials
int launch_fwd_combine(const AttnArgs& a, const AttnWorkspace& w, const PassParams& ps, cudaStream_t s);
// dq = sum of the row's backward partials (already scaled)
int launch_bwd_combine(const AttnArgs& a, const AttnWorkspace& w, const PassParams& ps, cudaStream_t s);
// softmax_d[h, t] = sum_d dout*out
int launch_dot_do_o(const AttnArgs& a, cudaStream_t s);

// engines: main kernels that produce the partials (and dk/dv in backward)
int launch_fwd_main_simt(const AttnArgs& a, const AttnWorkspace& w, const PassParams& ps, cudaStream_t s);
int launch_bwd_main_simt(const AttnArgs& a, const AttnWorkspace& w, const PassParams& ps, cudaStream_t s);
int launch_fwd_main_tc(const AttnArgs& a, const AttnWorkspace& w, const PassParams& ps, cudaStream_t s);
int launch_bwd_main_tc(const AttnArgs& a, const AttnWorkspace& w, const PassParams& ps, cudaStream_t s);
bool tc_supported(const AttnArgs& a, bool backward);
// tcgen05 kernels for head dims 192 and 256 (fmb_attn_tc_wide.cu)
int launch_fwd_main_tc_wide(const AttnArgs& a, const AttnWorkspace& w, const PassParams& ps, cudaStream_t s);
int launch_bwd_main_tc_wide(const AttnArgs& a, const AttnWorkspace& w, const PassParams& ps, cudaStream_t s);
bool tc_wide_supported(const AttnArgs& a, bool backward);
int sm_count();   // SMs of the current device
int launch_selftest_wait_expiry(int* status, unsigned long long* elapsed_ns, cudaStream_t s);
int launch_selftest_umma(const void* a, const void* b, float* d, int b_mn_major, int dtype, int* status,
                         cudaStream_t s);

}  // namespace fmb
