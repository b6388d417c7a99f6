// Stages O/E/S: per-row top-k lists -> key-block-major CSC pattern, without atomics on
// global memory and without a sort pass.
//
// The reference counts with global atomics, scans with one thread, scatters with global
// atomics (unordered) and then runs a segmented sort
// (csrc/flash_topk/src/flash_topk_kernel.h:303-312, 376-402, 407-478;
//  csrc/flash_topk/src/varlen_sort.cu:29-124).  Here:
//   1. tile_hist : a CTA takes kTileRows query rows of one (b,h) and a range of columns,
//                  marks (column,row) bits in a shared-memory bitmap and pop-counts each
//                  column -> hist[bh][tile][col]
//   2. col_scan  : per (b,h): running sum over tiles per column (hist becomes the tile's
//                  write cursor), col_nnz, exclusive scan over columns -> col_offsets,
//                  zero of the region's unused tail
//   3. scatter   : rebuild the bitmap; a half-warp per column walks its bits in row
//                  order and writes them at col_offsets + cursor -> columns come out
//                  ascending, bit-exact and run-to-run deterministic.  On request the same
//                  kernel also writes, for entry j of every row's top-k list, the position
//                  in `indices` where that (row, chunk) pair landed (row_slots): the
//                  row-major view of the pattern that the attention kernels' combine pass
//                  needs, so that an attention call on this pattern builds no lists of its own.
// HBM bound.  Algorithmic bytes: 4*nnz read + 4*nnz written + 12*B*H*ncol.
#include <mutex>

#include "fmb_common.cuh"

namespace fmb {

constexpr int kTileRows = 512;                 // query rows per tile
constexpr int kTileWords = kTileRows / 32;     // bitmap words per column
constexpr int kBmStride = kTileWords + 1;      // padded: conflict-free column walks
constexpr int kMaxColsPerCta = 1024;
constexpr int kCscThreads = 512;

struct CscParams {
  const int32_t* topk_idx; int64_t idx_rs, idx_hs;   // element strides of (row, head)
  const int32_t* cu_q;
  int64_t* col_offsets; int32_t* col_nnz; int32_t* indices;
  int32_t* hist;                                      // [B*H][ntiles][ncol]
  uint32_t* row_slots;                                // optional: [(h*total_q + token)*topk + j], 0xffffffff = no entry
  int64_t total_q;
  int heads, topk, ncol, ntiles, cols_per_cta;
};

// marks the bits of this CTA's (tile, column range); returns through smem `bm`
__device__ __forceinline__ void build_bitmap(const CscParams& p, uint32_t* bm, int b, int h, int tile,
                                             int c0, int ncols, int len_q, int seq0) {
  const int words = ncols * kBmStride;
  for (int i = threadIdx.x; i < words; i += blockDim.x) bm[i] = 0u;
  __syncthreads();
  const int r0 = tile * kTileRows;
  const int rows = min(kTileRows, len_q - r0);
  const int n = rows * p.topk;
  const int32_t* src = p.topk_idx + (int64_t)(seq0 + r0) * p.idx_rs + (int64_t)h * p.idx_hs;
  for (int e = threadIdx.x; e < n; e += blockDim.x) {
    const int r = e / p.topk, s = e - r * p.topk;
    const int c = src[(int64_t)r * p.idx_rs + s] - c0;
    if (c >= 0 && c < ncols) atomicOr(&bm[c * kBmStride + (r >> 5)], 1u << (r & 31));
  }
  __syncthreads();
}

__global__ void __launch_bounds__(kCscThreads) csc_tile_hist_kernel(CscParams p) {
  extern __shared__ uint32_t bm[];
  const int bh = blockIdx.x, tile = blockIdx.y, c0 = blockIdx.z * p.cols_per_cta;
  const int b = bh / p.heads, h = bh - b * p.heads;
  const int seq0 = p.cu_q[b], len_q = p.cu_q[b + 1] - seq0;
  const int ncols = min(p.cols_per_cta, p.ncol - c0);
  int32_t* hist = p.hist + ((int64_t)bh * p.ntiles + tile) * p.ncol + c0;
  if (tile * kTileRows >= len_q) {   // tile beyond this sequence: empty counts
    for (int c = threadIdx.x; c < ncols; c += blockDim.x) hist[c] = 0;
    return;
  }
  build_bitmap(p, bm, b, h, tile, c0, ncols, len_q, seq0);
  for (int c = threadIdx.x; c < ncols; c += blockDim.x) {
    int cnt = 0;
#pragma unroll
    for (int w = 0; w < kTileWords; ++w) cnt += __popc(bm[c * kBmStride + w]);
    hist[c] = cnt;
  }
}

__global__ void __launch_bounds__(1024) csc_col_scan_kernel(CscParams p) {
  __shared__ int64_t warp_sums[32];
  __shared__ int64_t carry_s;
  const int bh = blockIdx.x;
  const int b = bh / p.heads, h = bh - b * p.heads;
  const int seq0 = p.cu_q[b], len_q = p.cu_q[b + 1] - seq0;
  const int ntiles_b = (len_q + kTileRows - 1) / kTileRows;
  const int64_t base = ((int64_t)seq0 * p.heads + (int64_t)len_q * h) * p.topk;
  int32_t* hist = p.hist + (int64_t)bh * p.ntiles * p.ncol;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) carry_s = 0;
  __syncthreads();
  for (int c0 = 0; c0 < p.ncol; c0 += blockDim.x) {
    const int c = c0 + threadIdx.x;
    int run = 0;
    if (c < p.ncol) {
      // tiles beyond the sequence hold zeros.  Sixteen counters are fetched at a time so that the
      // loads overlap: one dependent load-add-store chain per tile would cost a memory latency each
      for (int t0 = 0; t0 < ntiles_b; t0 += 16) {
        int x[16];
#pragma unroll
        for (int u = 0; u < 16; ++u) x[u] = (t0 + u < ntiles_b) ? hist[(int64_t)(t0 + u) * p.ncol + c] : 0;
#pragma unroll
        for (int u = 0; u < 16; ++u) {
          if (t0 + u < ntiles_b) hist[(int64_t)(t0 + u) * p.ncol + c] = run;
          run += x[u];
        }
      }
    }
    // block-wide exclusive scan of `run` over this group of columns
    int64_t x = run;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int64_t y = __shfl_up_sync(0xffffffffu, x, o);
      if (lane >= o) x += y;
    }
    if (lane == 31) warp_sums[warp] = x;
    __syncthreads();
    if (warp == 0) {
      int64_t w = warp_sums[lane];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        int64_t y = __shfl_up_sync(0xffffffffu, w, o);
        if (lane >= o) w += y;
      }
      warp_sums[lane] = w;   // inclusive over warps
    }
    __syncthreads();
    const int64_t carry = carry_s;
    const int64_t excl = carry + (warp ? warp_sums[warp - 1] : 0) + x - run;
    if (c < p.ncol) {
      p.col_offsets[(int64_t)bh * p.ncol + c] = base + excl;
      p.col_nnz[(int64_t)bh * p.ncol + c] = run;
    }
    __syncthreads();
    if (threadIdx.x == blockDim.x - 1) carry_s = carry + warp_sums[31];
    __syncthreads();
  }
  // unused tail of this (b,h) region stays zero, as in the reference's zero-initialised
  // buffer (csrc/flash_topk/flash_topk_api.cpp:217)
  const int64_t total = carry_s, region = (int64_t)len_q * p.topk;
  for (int64_t i = total + threadIdx.x; i < region; i += blockDim.x) p.indices[base + i] = 0;
}

__global__ void __launch_bounds__(kCscThreads) csc_scatter_kernel(CscParams p) {
  extern __shared__ uint32_t bm[];
  const int bh = blockIdx.x, tile = blockIdx.y, c0 = blockIdx.z * p.cols_per_cta;
  const int b = bh / p.heads, h = bh - b * p.heads;
  const int seq0 = p.cu_q[b], len_q = p.cu_q[b + 1] - seq0;
  if (tile * kTileRows >= len_q) return;
  const int ncols = min(p.cols_per_cta, p.ncol - c0);
  build_bitmap(p, bm, b, h, tile, c0, ncols, len_q, seq0);
  const int32_t* cursor = p.hist + ((int64_t)bh * p.ntiles + tile) * p.ncol + c0;
  const int64_t* offs = p.col_offsets + (int64_t)bh * p.ncol + c0;
  // a half-warp per column: lane w of the half owns bitmap word w (32 rows)
  static_assert(kTileWords == 16, "half-warp mapping assumes 16 words per column");
  const int half = threadIdx.x >> 4, hl = threadIdx.x & 15;
  const int nhalves = blockDim.x >> 4;
  const unsigned hmask = 0xffffu << (threadIdx.x & 16);
  for (int c = half; c < ncols; c += nhalves) {
    uint32_t bits = bm[c * kBmStride + hl];
    int cnt = __popc(bits), x = cnt;
#pragma unroll
    for (int o = 1; o < 16; o <<= 1) {
      int y = __shfl_up_sync(hmask, x, o, 16);
      if (hl >= o) x += y;
    }
    int32_t* dst = p.indices + offs[c] + cursor[c] + (x - cnt);
    const int rbase = tile * kTileRows + hl * 32;
    while (bits) {
      const int bit = __ffs(bits) - 1;
      bits &= bits - 1;
      *dst++ = rbase + bit;
    }
  }
  if (p.row_slots == nullptr) return;
  // Row-major pass: entry (row r, list place j) with chunk c in this CTA's column range sits at
  // col_offsets[c] + cursor[c] + (rows of this tile below r that also selected c).
  const int r0 = tile * kTileRows;
  const int rows = min(kTileRows, len_q - r0);
  const int32_t* src = p.topk_idx + (int64_t)(seq0 + r0) * p.idx_rs + (int64_t)h * p.idx_hs;
  uint32_t* out = p.row_slots + ((int64_t)h * p.total_q + seq0 + r0) * p.topk;
  for (int e = threadIdx.x; e < rows * p.topk; e += blockDim.x) {
    const int r = e / p.topk, j = e - r * p.topk;
    const int cg = src[(int64_t)r * p.idx_rs + j];
    const int c = cg - c0;
    if (c >= 0 && c < ncols) {
      const uint32_t* col = bm + c * kBmStride;
      int below = __popc(col[r >> 5] & ((1u << (r & 31)) - 1u));
      for (int w = 0; w < (r >> 5); ++w) below += __popc(col[w]);
      out[e] = (uint32_t)(offs[c] + cursor[c] + below);
    } else if (blockIdx.z == 0 && (cg < 0 || cg >= p.ncol)) {
      out[e] = 0xffffffffu;     // empty place of the list (or a chunk id outside the pattern)
    }
  }
}

static int csc_ntiles(int max_q) { return max(1, ceil_div(max_q, kTileRows)); }

size_t csc_workspace_bytes(int batch, int heads, int max_q, int ncol) {
  return align_up((size_t)batch * heads * csc_ntiles(max_q) * (size_t)max(ncol, 1) * sizeof(int32_t), 256);
}

int launch_build_csc(const int32_t* topk_idx, int64_t idx_rs, int64_t idx_hs, const int32_t* cu_q, int64_t* col_offsets, int32_t* col_nnz,
                     int32_t* indices, void* ws, size_t ws_bytes, int batch, int heads, int topk, int max_q,
                     int ncol, cudaStream_t s, uint32_t* row_slots, int64_t total_q) {
  if (batch == 0 || heads == 0 || ncol == 0) return FMB_OK;
  if (ws == nullptr || ws_bytes < csc_workspace_bytes(batch, heads, max_q, ncol))
    return fail(FMB_ERR_WORKSPACE, "build_csc: workspace too small (%zu < %zu)", ws_bytes,
                csc_workspace_bytes(batch, heads, max_q, ncol));
  CscParams p;
  p.topk_idx = topk_idx;
  p.idx_rs = idx_rs;
  p.idx_hs = idx_hs;
  p.cu_q = cu_q; p.col_offsets = col_offsets; p.col_nnz = col_nnz; p.indices = indices;
  p.hist = static_cast<int32_t*>(ws);
  p.row_slots = row_slots; p.total_q = total_q;
  p.heads = heads; p.topk = topk; p.ncol = ncol; p.ntiles = csc_ntiles(max_q);
  p.cols_per_cta = min(kMaxColsPerCta, ncol);
  const int ncr = ceil_div(ncol, p.cols_per_cta);
  const size_t smem = (size_t)p.cols_per_cta * kBmStride * sizeof(uint32_t);
  // the attribute belongs to the current device: set on every call (cheap, idempotent, thread-safe)
  FMB_CUDA(cudaFuncSetAttribute(csc_tile_hist_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                kMaxColsPerCta * kBmStride * 4));
  FMB_CUDA(cudaFuncSetAttribute(csc_scatter_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                kMaxColsPerCta * kBmStride * 4));
  dim3 grid(batch * heads, p.ntiles, ncr);
  prof_begin(6, s);
  csc_tile_hist_kernel<<<grid, kCscThreads, smem, s>>>(p);
  FMB_LAUNCH_CHECK("csc_tile_hist_kernel");
  csc_col_scan_kernel<<<batch * heads, 1024, 0, s>>>(p);
  FMB_LAUNCH_CHECK("csc_col_scan_kernel");
  csc_scatter_kernel<<<grid, kCscThreads, smem, s>>>(p);
  prof_end(6, s);
  FMB_LAUNCH_CHECK("csc_scatter_kernel");
  return FMB_OK;
}

// ---------------------------------------------------------------------------------------
// Pattern build for callers that cannot allocate device memory.
//
// Some hosts of this library have no way to hand over a workspace: a serving runtime that
// claims all device memory at start-up and forbids cudaMalloc afterwards (the call
// synchronises the whole device and can fail once the arena owns the memory), or a thin
// FFI shim in another language that only forwards the pointers it was given.  For them the
// tile-histogram scratch of the builder lives in this file-scope device array instead.
//   * capacity: kStaticScratchBytes (8 MiB), i.e. batch*heads*ceil(max_seqlen_q/512)*ncol
//     <= 2,097,152 counters (e.g. one 64K-token sequence x 32 heads x 512 chunks); larger
//     problems are rejected with FMB_ERR_WORKSPACE and must use fmb_build_csc;
//   * every GPU that loads the library holds the array until the process exits;
//   * the array is shared by all calls and keeps the previous call's contents.  Nothing has
//     to start at zero: the histogram kernel writes every counter the later kernels read;
//   * two calls that overlap on the GPU (different streams, or different host threads)
//     race on the array: issue them on one stream, or order them with events.
// In host code the array's name is only a stand-in; the device address is obtained once per
// device with cudaGetSymbolAddress, on the first call made with that device current.  That
// first call should therefore be made outside any stream capture.
// ---------------------------------------------------------------------------------------
constexpr size_t kStaticScratchBytes = 8u << 20;
static __device__ __align__(256) int32_t g_csc_static_scratch[kStaticScratchBytes / sizeof(int32_t)];

static int csc_static_scratch_ptr(int32_t** out) {
  constexpr int kMaxDevices = 64;
  static std::mutex mu;
  static int32_t* ptrs[kMaxDevices] = {};
  int dev = 0;
  FMB_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail(FMB_ERR_CUDA, "build_csc_static: device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lock(mu);
  if (ptrs[dev] == nullptr) {
    int32_t* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_csc_static_scratch);
    if (e != cudaSuccess || p == nullptr)
      return fail(FMB_ERR_CUDA, "build_csc_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
    ptrs[dev] = p;
  }
  *out = ptrs[dev];
  return FMB_OK;
}

size_t csc_static_scratch_bytes() { return kStaticScratchBytes; }

int launch_build_csc_static(const int32_t* topk_idx, int64_t idx_rs, int64_t idx_hs, const int32_t* cu_q,
                            int64_t* col_offsets, int32_t* col_nnz, int32_t* indices, int batch, int heads,
                            int topk, int max_q, int ncol, cudaStream_t s) {
  if (batch == 0 || heads == 0 || ncol == 0) return FMB_OK;
  const size_t need = csc_workspace_bytes(batch, heads, max_q, ncol);
  if (need > kStaticScratchBytes)
    return fail(FMB_ERR_WORKSPACE,
                "build_csc_static: this problem needs %zu bytes of scratch, the built-in array holds %zu "
                "(batch*heads*ceil(max_seqlen_q/512)*ncol must be <= %zu); use fmb_build_csc with a workspace",
                need, kStaticScratchBytes, kStaticScratchBytes / sizeof(int32_t));
  int32_t* scratch = nullptr;
  const int rc = csc_static_scratch_ptr(&scratch);
  if (rc) return rc;
  return launch_build_csc(topk_idx, idx_rs, idx_hs, cu_q, col_offsets, col_nnz, indices, scratch,
                          kStaticScratchBytes, batch, heads, topk, max_q, ncol, s);
}

// ---------------------------------------------------------------------------------------
// Stand-alone segmented ascending sort (the reference's varlen_sort entry point,
// csrc/flash_topk/src/varlen_sort.cu:127-162).  The pattern builder above never needs it;
// it exists for callers that sort their own column lists.  One CTA per segment runs a
// direction-free bitonic network in place on dst: every compare-exchange puts the smaller
// key at the lower index, so virtual +inf padding above the segment end never moves.
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) varlen_sort_kernel(const int64_t* __restrict__ starts,
                                                          const int64_t* __restrict__ ends,
                                                          const int32_t* __restrict__ src,
                                                          int32_t* __restrict__ dst, int64_t nitems) {
  const int64_t s0 = starts[blockIdx.x], s1 = ends[blockIdx.x];
  if (s1 <= s0 || s0 < 0 || s1 > nitems) return;
  const int64_t n = s1 - s0;
  int32_t* a = dst + s0;
  for (int64_t i = threadIdx.x; i < n; i += blockDim.x) a[i] = src[s0 + i];
  __syncthreads();
  int64_t N = 1;
  while (N < n) N <<= 1;
  for (int64_t k = 2; k <= N; k <<= 1) {
    for (int64_t j = k >> 1; j >= 1; j >>= 1) {
      const bool flip = (j == (k >> 1));
      for (int64_t i = threadIdx.x; i < N; i += blockDim.x) {
        const int64_t l = flip ? (i ^ (k - 1)) : (i ^ j);
        if (l > i && l < n) {
          const int32_t x = a[i], y = a[l];
          if (x > y) { a[i] = y; a[l] = x; }
        }
      }
      __syncthreads();
    }
  }
}

int launch_varlen_sort(const int64_t* starts, const int64_t* ends, const int32_t* src, int32_t* dst,
                       int64_t nseg, int64_t nitems, cudaStream_t s) {
  FMB_CUDA(cudaMemsetAsync(dst, 0, (size_t)nitems * sizeof(int32_t), s));
  if (nseg == 0 || nitems == 0) return FMB_OK;
  FMB_CHECK_ARG(nseg <= 0x7fffffff, "varlen_sort: too many segments");
  varlen_sort_kernel<<<(unsigned)nseg, 256, 0, s>>>(starts, ends, src, dst, nitems);
  FMB_LAUNCH_CHECK("varlen_sort_kernel");
  return FMB_OK;
}

}  // namespace fmb
