// Row lists (CSR transpose of the pattern), the row-major combine kernels and the
// forward / backward drivers shared by both attention engines.
#include "fmb_attn.cuh"

namespace fmb {

// ------------------------------------------------------------------ workspace layout
static size_t scan_tmp_elems(int64_t n) { return (size_t)ceil_div64(n, 4096) + 1; }

AttnWorkspace carve_attn_workspace(void* base, int64_t total_q, int heads, int d, int64_t n_indices,
                                   size_t part_elem_bytes, bool with_lse) {
  AttnWorkspace w;
  size_t off = 0;
  auto take = [&](size_t bytes) {
    void* p = base ? static_cast<char*>(base) + off : nullptr;
    off += align_up(bytes, 256);
    return p;
  };
  const int64_t rows = total_q * heads;
  w.status = static_cast<int*>(take(512));
  w.part_o = take((size_t)n_indices * d * part_elem_bytes);
  w.part_lse = static_cast<float*>(take(with_lse ? (size_t)n_indices * sizeof(float) : 0));
  w.row_ptr = static_cast<uint32_t*>(take((size_t)(rows + 1) * sizeof(uint32_t)));
  w.row_fill = static_cast<uint32_t*>(take((size_t)rows * sizeof(uint32_t)));
  w.row_pos = static_cast<uint32_t*>(take((size_t)n_indices * sizeof(uint32_t)));
  w.scan_tmp = static_cast<uint32_t*>(take(scan_tmp_elems(rows + 1) * sizeof(uint32_t)));
  w.bytes = off;
  return w;
}

size_t attn_fwd_workspace_bytes(int64_t total_q, int heads, int d, int64_t n_indices) {
  return carve_attn_workspace(nullptr, total_q, heads, d, n_indices, 2, true).bytes;
}
size_t attn_bwd_workspace_bytes(int64_t total_q, int heads, int d, int64_t n_indices) {
  return carve_attn_workspace(nullptr, total_q, heads, d, n_indices, 4, false).bytes;
}

// ------------------------------------------------------------------ row lists
struct RowListParams {
  const int64_t* col_offsets; const int32_t* col_nnz; const int32_t* indices; int64_t n_indices;
  const int32_t* cu_q;
  uint32_t *row_ptr, *row_fill, *row_pos;
  int heads, ncol; int64_t total_q;
};

// grid (ncol, heads, batch): one CTA per column
template <bool kFill>
__global__ void __launch_bounds__(256) row_list_kernel(RowListParams p) {
  const int c = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int64_t ci = ((int64_t)b * p.heads + h) * p.ncol + c;
  const int nnz = p.col_nnz[ci];
  if (nnz <= 0) return;
  const int64_t off = p.col_offsets[ci];
  if (off < 0 || off + nnz > p.n_indices) return;   // malformed pattern: ignored, never read out of bounds
  const int q0 = p.cu_q[b], len_q = p.cu_q[b + 1] - q0;
  const int64_t rbase = (int64_t)h * p.total_q + q0;
  for (int j = threadIdx.x; j < nnz; j += blockDim.x) {
    const int r = p.indices[off + j];
    if (r < 0 || r >= len_q) continue;
    if (!kFill) {
      atomicAdd(&p.row_ptr[rbase + r + 1], 1u);     // counts, shifted by one for the scan
    } else {
      const uint32_t slot = atomicAdd(&p.row_fill[rbase + r], 1u);
      p.row_pos[p.row_ptr[rbase + r] + slot] = (uint32_t)(off + j);
    }
  }
}

// inclusive scan of u32 in place, three phases, 4096 items per block
constexpr int kScanItems = 4096;
__global__ void __launch_bounds__(1024) scan_block_kernel(uint32_t* data, int64_t n, uint32_t* block_sums) {
  __shared__ uint32_t wsum[32];
  const int64_t base = (int64_t)blockIdx.x * kScanItems + threadIdx.x * 4;
  uint32_t v[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) v[i] = (base + i < n) ? data[base + i] : 0u;
  v[1] += v[0]; v[2] += v[1]; v[3] += v[2];
  uint32_t x = v[3];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    uint32_t y = __shfl_up_sync(0xffffffffu, x, o);
    if (lane >= o) x += y;
  }
  if (lane == 31) wsum[warp] = x;
  __syncthreads();
  if (warp == 0) {
    uint32_t w = wsum[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      uint32_t y = __shfl_up_sync(0xffffffffu, w, o);
      if (lane >= o) w += y;
    }
    wsum[lane] = w;
  }
  __syncthreads();
  const uint32_t excl = (warp ? wsum[warp - 1] : 0u) + x - v[3];
#pragma unroll
  for (int i = 0; i < 4; ++i)
    if (base + i < n) data[base + i] = v[i] + excl;
  if (threadIdx.x == 1023) block_sums[blockIdx.x] = wsum[31];
}
__global__ void __launch_bounds__(1024) scan_sums_kernel(uint32_t* block_sums, int nblocks) {
  // single block: serial over groups of 1024 with a running carry (exclusive result)
  __shared__ uint32_t wsum[32];
  __shared__ uint32_t carry_s;
  if (threadIdx.x == 0) carry_s = 0;
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int g = 0; g < nblocks; g += 1024) {
    const int i = g + threadIdx.x;
    const uint32_t v = i < nblocks ? block_sums[i] : 0u;
    uint32_t x = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      uint32_t y = __shfl_up_sync(0xffffffffu, x, o);
      if (lane >= o) x += y;
    }
    if (lane == 31) wsum[warp] = x;
    __syncthreads();
    if (warp == 0) {
      uint32_t w = wsum[lane];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        uint32_t y = __shfl_up_sync(0xffffffffu, w, o);
        if (lane >= o) w += y;
      }
      wsum[lane] = w;
    }
    __syncthreads();
    const uint32_t carry = carry_s;
    if (i < nblocks) block_sums[i] = carry + (warp ? wsum[warp - 1] : 0u) + x - v;
    __syncthreads();
    if (threadIdx.x == 1023) carry_s = carry + wsum[31];
    __syncthreads();
  }
}
__global__ void __launch_bounds__(1024) scan_add_kernel(uint32_t* data, int64_t n, const uint32_t* block_sums) {
  const int64_t base = (int64_t)blockIdx.x * kScanItems + threadIdx.x * 4;
  const uint32_t add = block_sums[blockIdx.x];
#pragma unroll
  for (int i = 0; i < 4; ++i)
    if (base + i < n) data[base + i] += add;
}

int build_row_lists(const AttnArgs& a, const AttnWorkspace& w, cudaStream_t s) {
  const int64_t rows = a.total_q * a.heads;
  FMB_CUDA(cudaMemsetAsync(w.status, 0, 512, s));
  FMB_CUDA(cudaMemsetAsync(w.row_ptr, 0, (size_t)(rows + 1) * sizeof(uint32_t), s));
  FMB_CUDA(cudaMemsetAsync(w.row_fill, 0, (size_t)rows * sizeof(uint32_t), s));
  if (a.ncol == 0 || a.batch == 0) return FMB_OK;
  RowListParams p;
  p.col_offsets = a.col_offsets; p.col_nnz = a.col_nnz; p.indices = a.indices; p.n_indices = a.n_indices;
  p.cu_q = a.cu_q; p.row_ptr = w.row_ptr; p.row_fill = w.row_fill; p.row_pos = w.row_pos;
  p.heads = a.heads; p.ncol = a.ncol; p.total_q = a.total_q;
  dim3 grid(a.ncol, a.heads, a.batch);
  row_list_kernel<false><<<grid, 256, 0, s>>>(p);
  FMB_LAUNCH_CHECK("row_list_kernel<count>");
  const int64_t n = rows + 1;
  const int nblocks = (int)ceil_div64(n, kScanItems);
  scan_block_kernel<<<nblocks, 1024, 0, s>>>(w.row_ptr, n, w.scan_tmp);
  FMB_LAUNCH_CHECK("scan_block_kernel");
  if (nblocks > 1) {
    scan_sums_kernel<<<1, 1024, 0, s>>>(w.scan_tmp, nblocks);
    FMB_LAUNCH_CHECK("scan_sums_kernel");
    scan_add_kernel<<<nblocks, 1024, 0, s>>>(w.row_ptr, n, w.scan_tmp);
    FMB_LAUNCH_CHECK("scan_add_kernel");
  }
  row_list_kernel<true><<<grid, 256, 0, s>>>(p);
  FMB_LAUNCH_CHECK("row_list_kernel<fill>");
  return FMB_OK;
}

// ------------------------------------------------------------------ combine kernels
// A warp per (token, head).  The row's partials are visited in ascending `pos`.
// next_pos(): smallest position of the row that is greater than `last` (-1 first).
__device__ __forceinline__ int64_t next_pos(const uint32_t* rp, int n, int64_t last, int lane) {
  int64_t best = INT64_MAX;
  for (int j = lane; j < n; j += 32) {
    const int64_t x = rp[j];
    if (x > last && x < best) best = x;
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) {
    const int64_t y = __shfl_xor_sync(0xffffffffu, best, o);
    best = y < best ? y : best;
  }
  return best;
}

template <typename T>
__global__ void __launch_bounds__(256) fwd_combine_kernel(const T* __restrict__ part_o,
                                                          const float* __restrict__ part_lse,
                                                          const uint32_t* __restrict__ row_ptr,
                                                          const uint32_t* __restrict__ row_pos, T* out,
                                                          int64_t o_rs, int64_t o_hs, float* lse,
                                                          int64_t total_q, int heads, int d,
                                                          const int* only_if, int min_n) {
  using T2 = typename Elem<T>::T2;
  if (only_if && *only_if == 0) return;   // the earlier stages met no row they had to leave
  const int64_t wid = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= total_q * heads) return;
  const int64_t t = wid / heads;
  const int h = (int)(wid - t * heads);
  const int64_t rid = (int64_t)h * total_q + t;
  const uint32_t p0 = row_ptr[rid];
  const int n = (int)(row_ptr[rid + 1] - p0);
  if (n < min_n) return;
  const uint32_t* rp = row_pos + p0;
  // pass 1: maximum of the partial log-sum-exps
  float m = -CUDART_INF_F;
  for (int j = lane; j < n; j += 32) m = fmaxf(m, part_lse[rp[j]]);
#pragma unroll
  for (int o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  float2 acc[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) acc[i] = make_float2(0.f, 0.f);
  float ssum = 0.f;
  if (m > -CUDART_INF_F) {
    int64_t last = -1;
    for (int r = 0; r < n; ++r) {
      const int64_t pos = next_pos(rp, n, last, lane);
      last = pos;
      const float wgt = __expf(part_lse[pos] - m);
      ssum += wgt;
      const T* src = part_o + pos * d;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int c = lane * 2 + i * 64;
        if (c < d) {
          const float2 x = Elem<T>::to_f2(*reinterpret_cast<const T2*>(src + part_col(pos, c, 8)));
          acc[i].x = fmaf(wgt, x.x, acc[i].x);
          acc[i].y = fmaf(wgt, x.y, acc[i].y);
        }
      }
    }
  }
  const float inv = ssum > 0.f ? 1.f / ssum : 0.f;
  T* dst = out + t * o_rs + (int64_t)h * o_hs;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int c = lane * 2 + i * 64;
    if (c < d) *reinterpret_cast<T2*>(dst + c) = Elem<T>::from_f2(acc[i].x * inv, acc[i].y * inv);
  }
  if (lane == 0) lse[rid] = ssum > 0.f ? m + logf(ssum) : CUDART_INF_F;
}

template <typename T>
__global__ void __launch_bounds__(256) bwd_combine_kernel(const float* __restrict__ part_dq,
                                                          const uint32_t* __restrict__ row_ptr,
                                                          const uint32_t* __restrict__ row_pos, T* dq,
                                                          int64_t rs, int64_t hs, int64_t total_q, int heads,
                                                          int d, float scale, const int* only_if, int min_n) {
  using T2 = typename Elem<T>::T2;
  if (only_if && *only_if == 0) return;
  const int64_t wid = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= total_q * heads) return;
  const int64_t t = wid / heads;
  const int h = (int)(wid - t * heads);
  const int64_t rid = (int64_t)h * total_q + t;
  const uint32_t p0 = row_ptr[rid];
  const int n = (int)(row_ptr[rid + 1] - p0);
  if (n < min_n) return;
  const uint32_t* rp = row_pos + p0;
  float2 acc[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) acc[i] = make_float2(0.f, 0.f);
  int64_t last = -1;
  for (int r = 0; r < n; ++r) {
    const int64_t pos = next_pos(rp, n, last, lane);
    last = pos;
    const float* src = part_dq + pos * d;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int c = lane * 2 + i * 64;
      if (c < d) {
        const float2 x = *reinterpret_cast<const float2*>(src + part_col(pos, c, 4));
        acc[i].x += x.x;
        acc[i].y += x.y;
      }
    }
  }
  T* dst = dq + t * rs + (int64_t)h * hs;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int c = lane * 2 + i * 64;
    if (c < d) *reinterpret_cast<T2*>(dst + c) = Elem<T>::from_f2(acc[i].x * scale, acc[i].y * scale);
  }
}

// ------------------------------------------------------------------ fast combine (rows of <= G partials)
// G lanes per (token, head) row, 32/G rows per warp.  Lane j of a group first fetches the
// position and log-sum-exp of the row's j-th partial; the group ranks the positions (merge
// order = ascending position, whatever order the atomics of the row-list build produced);
// then every lane fetches its d/G elements of ALL the row's partial rows before the ordered
// accumulation.  Several rows per warp and all loads of a row in flight at once hide the
// chain of dependent, scattered reads.  Rows with more than G partials set *overflow and are
// left to the next kernel (larger G, finally the generic one).
template <int G>
__device__ __forceinline__ unsigned group_mask(int lane) {
  return G == 32 ? 0xffffffffu : (((1u << G) - 1u) << (lane & ~(G - 1)));
}

template <typename T, int G, int EPL>
__global__ void __launch_bounds__(256) fwd_combine_group_kernel(const T* __restrict__ part_o,
                                                                const float* __restrict__ part_lse,
                                                                const uint32_t* __restrict__ row_ptr,
                                                                const uint32_t* __restrict__ row_pos, T* out,
                                                                int64_t o_rs, int64_t o_hs, float* lse,
                                                                int64_t total_q, int heads, int min_n,
                                                                const int* only_if, int* overflow) {
  constexpr int d = G * EPL;
  constexpr int NV = EPL / 8;                 // 16-byte loads per partial row per lane
  static_assert(EPL % 8 == 0, "a lane owns whole 16-byte chunks");
  if (only_if && *only_if == 0) return;
  const int lane = threadIdx.x & 31, gl = lane & (G - 1);
  const int64_t gid = (((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5) * (32 / G) + (lane / G);
  const bool row_ok = gid < total_q * heads;
  const unsigned gm = group_mask<G>(lane);
  const int64_t t = row_ok ? gid / heads : 0;
  const int h = row_ok ? (int)(gid - t * heads) : 0;
  const int64_t rid = (int64_t)h * total_q + t;
  uint32_t p0 = 0;
  int n = 0;
  if (row_ok) {
    p0 = row_ptr[rid];
    n = (int)(row_ptr[rid + 1] - p0);
  }
  bool mine = row_ok && n >= min_n;           // rows below min_n were done by the previous kernel
  if (n > G) {
    if (gl == 0) *overflow = 1;
    mine = false;
  }
  if (!mine) n = 0;
  const bool valid = gl < n;
  const uint32_t pos = valid ? row_pos[p0 + gl] : 0xffffffffu;
  const float l = valid ? part_lse[pos] : -CUDART_INF_F;
  float m = l;
#pragma unroll
  for (int o = G / 2; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(gm, m, o, G));
  const float w = (valid && m > -CUDART_INF_F) ? __expf(l - m) : 0.f;
  int rank = 0;
#pragma unroll
  for (int i = 0; i < G; ++i) rank += (__shfl_sync(gm, pos, i, G) < pos) ? 1 : 0;
  float acc[EPL];
#pragma unroll
  for (int i = 0; i < EPL; ++i) acc[i] = 0.f;
  float ssum = 0.f;
  constexpr int B = G < 8 ? G : 8;            // partial rows in flight per step
#pragma unroll
  for (int r0 = 0; r0 < G; r0 += B) {
    uint4 x[B][NV];
    float wk[B];
#pragma unroll
    for (int k = 0; k < B; ++k) {
      // the lane of this group whose partial has rank r0+k (none if the row is shorter)
      const unsigned hit = __ballot_sync(0xffffffffu, valid && rank == r0 + k) & gm;
      const int src = hit ? (__ffs(hit) - 1) : lane;
      const uint32_t pk = __shfl_sync(0xffffffffu, pos, src);
      wk[k] = hit ? __shfl_sync(0xffffffffu, w, src) : 0.f;
      if (hit && wk[k] > 0.f) {
        const T* row = part_o + (int64_t)pk * d;
#pragma unroll
        for (int v = 0; v < NV; ++v) x[k][v] = *reinterpret_cast<const uint4*>(row + part_col(pk, gl * EPL + 8 * v, 8));
      } else {
#pragma unroll
        for (int v = 0; v < NV; ++v) x[k][v] = make_uint4(0, 0, 0, 0);
      }
    }
#pragma unroll
    for (int k = 0; k < B; ++k) {
      ssum += wk[k];
#pragma unroll
      for (int v = 0; v < NV; ++v) {
        float f[8];
        unpack8<T>(x[k][v], f);
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[8 * v + e] = fmaf(wk[k], f[e], acc[8 * v + e]);
      }
    }
  }
  if (mine) {
    const float inv = ssum > 0.f ? 1.f / ssum : 0.f;
    T* dst = out + t * o_rs + (int64_t)h * o_hs + gl * EPL;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[8 * v + e] *= inv;
      *reinterpret_cast<uint4*>(dst + 8 * v) = pack8<T>(acc + 8 * v);
    }
    if (gl == 0) lse[rid] = ssum > 0.f ? m + logf(ssum) : CUDART_INF_F;
  }
}

template <typename T, int G, int EPL>
__global__ void __launch_bounds__(256) bwd_combine_group_kernel(const float* __restrict__ part_dq,
                                                                const uint32_t* __restrict__ row_ptr,
                                                                const uint32_t* __restrict__ row_pos, T* dq,
                                                                int64_t rs, int64_t hs, int64_t total_q,
                                                                int heads, float scale, int min_n,
                                                                const int* only_if, int* overflow) {
  constexpr int d = G * EPL;
  constexpr int NV = EPL / 4;                 // 16-byte (4 float) loads per partial row per lane
  static_assert(EPL % 8 == 0, "a lane owns whole 16-byte chunks of the output");
  if (only_if && *only_if == 0) return;
  const int lane = threadIdx.x & 31, gl = lane & (G - 1);
  const int64_t gid = (((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5) * (32 / G) + (lane / G);
  const bool row_ok = gid < total_q * heads;
  const unsigned gm = group_mask<G>(lane);
  const int64_t t = row_ok ? gid / heads : 0;
  const int h = row_ok ? (int)(gid - t * heads) : 0;
  const int64_t rid = (int64_t)h * total_q + t;
  uint32_t p0 = 0;
  int n = 0;
  if (row_ok) {
    p0 = row_ptr[rid];
    n = (int)(row_ptr[rid + 1] - p0);
  }
  bool mine = row_ok && n >= min_n;
  if (n > G) {
    if (gl == 0) *overflow = 1;
    mine = false;
  }
  if (!mine) n = 0;
  const bool valid = gl < n;
  const uint32_t pos = valid ? row_pos[p0 + gl] : 0xffffffffu;
  int rank = 0;
#pragma unroll
  for (int i = 0; i < G; ++i) rank += (__shfl_sync(gm, pos, i, G) < pos) ? 1 : 0;
  float acc[EPL];
#pragma unroll
  for (int i = 0; i < EPL; ++i) acc[i] = 0.f;
  constexpr int B = 4;
#pragma unroll
  for (int r0 = 0; r0 < G; r0 += B) {
    float4 x[B][NV];
#pragma unroll
    for (int k = 0; k < B; ++k) {
      const unsigned hit = __ballot_sync(0xffffffffu, valid && rank == r0 + k) & gm;
      const int src = hit ? (__ffs(hit) - 1) : lane;
      const uint32_t pk = __shfl_sync(0xffffffffu, pos, src);
      if (hit) {
        const float* row = part_dq + (int64_t)pk * d;
#pragma unroll
        for (int v = 0; v < NV; ++v) x[k][v] = *reinterpret_cast<const float4*>(row + part_col(pk, gl * EPL + 4 * v, 4));
      } else {
#pragma unroll
        for (int v = 0; v < NV; ++v) x[k][v] = make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
#pragma unroll
    for (int k = 0; k < B; ++k) {
#pragma unroll
      for (int v = 0; v < NV; ++v) {
        acc[4 * v] += x[k][v].x; acc[4 * v + 1] += x[k][v].y; acc[4 * v + 2] += x[k][v].z; acc[4 * v + 3] += x[k][v].w;
      }
    }
  }
  if (mine) {
    T* dst = dq + t * rs + (int64_t)h * hs + gl * EPL;
#pragma unroll
    for (int v = 0; v < EPL / 8; ++v) {
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[8 * v + e] *= scale;
      *reinterpret_cast<uint4*>(dst + 8 * v) = pack8<T>(acc + 8 * v);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256) dot_do_o_kernel(const T* __restrict__ dout, int64_t do_rs, int64_t do_hs,
                                                       const T* __restrict__ o, int64_t o_rs, int64_t o_hs,
                                                       float* softmax_d, int64_t total_q, int heads, int d) {
  using T2 = typename Elem<T>::T2;
  const int64_t wid = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= total_q * heads) return;
  const int64_t t = wid / heads;
  const int h = (int)(wid - t * heads);
  const T* a = dout + t * do_rs + (int64_t)h * do_hs;
  const T* b = o + t * o_rs + (int64_t)h * o_hs;
  float s = 0.f;
  for (int c = lane * 2; c < d; c += 64) {
    const float2 x = Elem<T>::to_f2(*reinterpret_cast<const T2*>(a + c));
    const float2 y = Elem<T>::to_f2(*reinterpret_cast<const T2*>(b + c));
    s = fmaf(x.x, y.x, s);
    s = fmaf(x.y, y.y, s);
  }
#pragma unroll
  for (int o2 = 16; o2; o2 >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o2);
  if (lane == 0) softmax_d[(int64_t)h * total_q + t] = s;
}

static unsigned warp_grid(int64_t warps) { return (unsigned)ceil_div64(warps, 8); }

// Cascade: G = 8 (rows of <= 8 partials), 16, 32, then the generic kernel; each later stage
// runs only the rows the earlier ones left and exits at once if there were none.
static unsigned group_grid(int64_t rows, int G) { return (unsigned)ceil_div64(ceil_div64(rows, 32 / G), 8); }

template <typename T, int D>
static int fwd_combine_dispatch(const AttnArgs& a, const AttnWorkspace& w, cudaStream_t s) {
  const int64_t rows = a.total_q * a.heads;
  int* ovf = w.status + 1;   // words 1..3 of the status block, zeroed with it
  const T* po = (const T*)w.part_o;
  T* out = (T*)a.o;
  fwd_combine_group_kernel<T, 8, D / 8><<<group_grid(rows, 8), 256, 0, s>>>(
      po, w.part_lse, w.row_ptr, w.row_pos, out, a.o_rs, a.o_hs, a.lse, a.total_q, a.heads, 0, nullptr, ovf);
  FMB_LAUNCH_CHECK("fwd_combine_group_kernel<8>");
  fwd_combine_group_kernel<T, 16, D / 16><<<group_grid(rows, 16), 256, 0, s>>>(
      po, w.part_lse, w.row_ptr, w.row_pos, out, a.o_rs, a.o_hs, a.lse, a.total_q, a.heads, 9, ovf, ovf + 1);
  FMB_LAUNCH_CHECK("fwd_combine_group_kernel<16>");
  fwd_combine_kernel<T><<<warp_grid(rows), 256, 0, s>>>(po, w.part_lse, w.row_ptr, w.row_pos, out, a.o_rs, a.o_hs,
                                                        a.lse, a.total_q, a.heads, a.d, ovf + 1, 17);
  FMB_LAUNCH_CHECK("fwd_combine_kernel");
  return FMB_OK;
}

template <typename T>
static int fwd_combine_any(const AttnArgs& a, const AttnWorkspace& w, cudaStream_t s) {
  if (a.d == 128) return fwd_combine_dispatch<T, 128>(a, w, s);
  if (a.d == 256) return fwd_combine_dispatch<T, 256>(a, w, s);
  const int64_t rows = a.total_q * a.heads;
  fwd_combine_kernel<T><<<warp_grid(rows), 256, 0, s>>>((const T*)w.part_o, w.part_lse, w.row_ptr, w.row_pos,
                                                        (T*)a.o, a.o_rs, a.o_hs, a.lse, a.total_q, a.heads, a.d,
                                                        nullptr, 0);
  FMB_LAUNCH_CHECK("fwd_combine_kernel");
  return FMB_OK;
}

int launch_fwd_combine(const AttnArgs& a, const AttnWorkspace& w, cudaStream_t s) {
  if (a.total_q * a.heads == 0) return FMB_OK;
  return a.dtype == FMB_BF16 ? fwd_combine_any<__nv_bfloat16>(a, w, s) : fwd_combine_any<__half>(a, w, s);
}

template <typename T, int D>
static int bwd_combine_dispatch(const AttnArgs& a, const AttnWorkspace& w, cudaStream_t s) {
  const int64_t rows = a.total_q * a.heads;
  int* ovf = w.status + 1;
  const float* pd = (const float*)w.part_o;
  T* dq = (T*)a.dq;
  bwd_combine_group_kernel<T, 8, D / 8><<<group_grid(rows, 8), 256, 0, s>>>(
      pd, w.row_ptr, w.row_pos, dq, a.dq_rs, a.dq_hs, a.total_q, a.heads, a.scale, 0, nullptr, ovf);
  FMB_LAUNCH_CHECK("bwd_combine_group_kernel<8>");
  bwd_combine_group_kernel<T, 16, D / 16><<<group_grid(rows, 16), 256, 0, s>>>(
      pd, w.row_ptr, w.row_pos, dq, a.dq_rs, a.dq_hs, a.total_q, a.heads, a.scale, 9, ovf, ovf + 1);
  FMB_LAUNCH_CHECK("bwd_combine_group_kernel<16>");
  bwd_combine_kernel<T><<<warp_grid(rows), 256, 0, s>>>(pd, w.row_ptr, w.row_pos, dq, a.dq_rs, a.dq_hs, a.total_q,
                                                        a.heads, a.d, a.scale, ovf + 1, 17);
  FMB_LAUNCH_CHECK("bwd_combine_kernel");
  return FMB_OK;
}

template <typename T>
static int bwd_combine_any(const AttnArgs& a, const AttnWorkspace& w, cudaStream_t s) {
  if (a.d == 128) return bwd_combine_dispatch<T, 128>(a, w, s);
  if (a.d == 256) return bwd_combine_dispatch<T, 256>(a, w, s);
  const int64_t rows = a.total_q * a.heads;
  bwd_combine_kernel<T><<<warp_grid(rows), 256, 0, s>>>((const float*)w.part_o, w.row_ptr, w.row_pos, (T*)a.dq,
                                                        a.dq_rs, a.dq_hs, a.total_q, a.heads, a.d, a.scale, nullptr, 0);
  FMB_LAUNCH_CHECK("bwd_combine_kernel");
  return FMB_OK;
}

int launch_bwd_combine(const AttnArgs& a, const AttnWorkspace& w, cudaStream_t s) {
  if (a.total_q * a.heads == 0) return FMB_OK;
  return a.dtype == FMB_BF16 ? bwd_combine_any<__nv_bfloat16>(a, w, s) : bwd_combine_any<__half>(a, w, s);
}

int launch_dot_do_o(const AttnArgs& a, cudaStream_t s) {
  const int64_t rows = a.total_q * a.heads;
  if (rows == 0) return FMB_OK;
  if (a.dtype == FMB_BF16)
    dot_do_o_kernel<__nv_bfloat16><<<warp_grid(rows), 256, 0, s>>>(
        (const __nv_bfloat16*)a.dout, a.do_rs, a.do_hs, (const __nv_bfloat16*)a.o, a.o_rs, a.o_hs, a.softmax_d,
        a.total_q, a.heads, a.d);
  else
    dot_do_o_kernel<__half><<<warp_grid(rows), 256, 0, s>>>((const __half*)a.dout, a.do_rs, a.do_hs,
                                                           (const __half*)a.o, a.o_rs, a.o_hs, a.softmax_d,
                                                           a.total_q, a.heads, a.d);
  FMB_LAUNCH_CHECK("dot_do_o_kernel");
  return FMB_OK;
}

// ------------------------------------------------------------------ drivers
int launch_attn_fwd(const AttnArgs& a, int engine, cudaStream_t s) {
  AttnWorkspace w = carve_attn_workspace(a.ws, a.total_q, a.heads, a.d, a.n_indices, 2, true);
  if (a.ws == nullptr || a.ws_bytes < w.bytes)
    return fail(FMB_ERR_WORKSPACE, "attn_fwd: workspace too small (%zu < %zu)", a.ws_bytes, w.bytes);
  int rc = build_row_lists(a, w, s);
  if (rc) return rc;
  prof_begin(0, s);
  if (engine == 1 && tc_supported(a, false)) rc = launch_fwd_main_tc(a, w, s);
  else rc = launch_fwd_main_simt(a, w, s);
  prof_end(0, s);
  if (rc) return rc;
  return launch_fwd_combine(a, w, s);
}

int launch_attn_bwd(const AttnArgs& a, int engine, cudaStream_t s) {
  AttnWorkspace w = carve_attn_workspace(a.ws, a.total_q, a.heads, a.d, a.n_indices, 4, false);
  if (a.ws == nullptr || a.ws_bytes < w.bytes)
    return fail(FMB_ERR_WORKSPACE, "attn_bwd: workspace too small (%zu < %zu)", a.ws_bytes, w.bytes);
  int rc = build_row_lists(a, w, s);
  if (rc) return rc;
  rc = launch_dot_do_o(a, s);
  if (rc) return rc;
  prof_begin(1, s);
  if (engine == 1 && tc_supported(a, true)) rc = launch_bwd_main_tc(a, w, s);
  else rc = launch_bwd_main_simt(a, w, s);
  prof_end(1, s);
  if (rc) return rc;
  return launch_bwd_combine(a, w, s);
}

}  // namespace fmb
