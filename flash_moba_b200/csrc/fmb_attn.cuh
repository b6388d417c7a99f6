// Shared pieces of the block-sparse attention (stages F and B).
//
// Both passes are KEY-CHUNK-MAJOR: a CTA owns one key chunk of one (sequence, head) and
// walks the chunk's CSC column, i.e. the gathered list of query rows that selected it, in
// dense tiles.  A (row, chunk) pair is item `pos` of the flat `indices` array, and that
// position is also where the pair's partial result lives in the workspace:
//   forward : part_o[pos][d]  (chunk-local softmax(QK^T)V, normalised, in the I/O dtype)
//             part_lse[pos]   (chunk-local log-sum-exp, natural log, of the scaled scores)
//   backward: part_dq[pos][d] (fp32, unscaled dS.K of that chunk)
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

struct AttnWorkspace {
  int* status;         // first word of the workspace: 0, or where a bounded device wait gave up
  void* part_o;        // fwd: n_indices * d elements of the I/O dtype;  bwd: n_indices * d floats
  float* part_lse;     // fwd only: n_indices
  uint32_t* row_ptr;   // heads*total_q + 1
  uint32_t* row_fill;  // heads*total_q
  uint32_t* row_pos;   // n_indices
  uint32_t* scan_tmp;  // block sums of the scan
  size_t bytes;
};

AttnWorkspace carve_attn_workspace(void* base, int64_t total_q, int heads, int d, int64_t n_indices,
                                   size_t part_elem_bytes, bool with_lse);

// Builds row_ptr / row_pos (CSR transpose of the CSC pattern).  Row id = h*total_q + token.
int build_row_lists(const AttnArgs& a, const AttnWorkspace& w, cudaStream_t s);

// out/lse from the forward partials
int launch_fwd_combine(const AttnArgs& a, const AttnWorkspace& w, cudaStream_t s);
// dq from the backward partials (multiplies by softmax_scale)
int launch_bwd_combine(const AttnArgs& a, const AttnWorkspace& w, cudaStream_t s);
// softmax_d[h, t] = sum_d dout*out
int launch_dot_do_o(const AttnArgs& a, cudaStream_t s);

// forward partials of pattern entries whose chunk starts beyond the sequence's keys
int launch_fwd_dead_columns(const AttnArgs& a, const AttnWorkspace& w, cudaStream_t s);

// engines: main kernels that produce the partials (and dk/dv in backward)
int launch_fwd_main_simt(const AttnArgs& a, const AttnWorkspace& w, cudaStream_t s);
int launch_bwd_main_simt(const AttnArgs& a, const AttnWorkspace& w, cudaStream_t s);
int launch_fwd_main_tc(const AttnArgs& a, const AttnWorkspace& w, cudaStream_t s);
int launch_bwd_main_tc(const AttnArgs& a, const AttnWorkspace& w, cudaStream_t s);
bool tc_supported(const AttnArgs& a, bool backward);
int launch_selftest_gather(const void* a, int a_rows, const int* idx, const void* b, float* d, int dtype,
                           int* status, cudaStream_t s);
int launch_selftest_umma(const void* a, const void* b, float* d, int b_mn_major, int dtype, int* status,
                         cudaStream_t s);

}  // namespace fmb
