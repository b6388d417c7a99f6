// Pass planning, slot and row lists (CSR transpose of the pattern), the row-major combine
// kernels and the forward / backward drivers shared by both attention engines.
#include "fmb_attn.cuh"

namespace fmb {

// ------------------------------------------------------------------ workspace layout / passes
static size_t scan_tmp_elems(int64_t n) { return (size_t)ceil_div64(n, 4096) + 1; }

static size_t layout(AttnWorkspace& w, void* base, const AttnArgs& a, size_t part_elem_bytes, bool with_lse, int nh) {
  size_t off = 0;
  auto take = [&](size_t bytes) {
    void* p = base ? static_cast<char*>(base) + off : nullptr;
    off += align_up(bytes, 256);
    return p;
  };
  w.nh = nh;
  w.fixed_k = 0;
  w.mirror = nullptr;
  // key block: 128 keys when the chunk is a multiple of 128, except in the backward pass of head
  // dim 256, whose dK and dV accumulators for 128 keys would not fit in TMEM (with_lse = forward)
  w.kb = (a.chunk % 128 == 0 && (a.d <= 128 || with_lse)) ? 128 : 64;
  w.nsub = a.chunk / w.kb;
  // one pass over all heads can never need more slots than the pattern has entries; a pass over a
  // share of the heads is given that share (exact for the top-k packing), rounded up
  w.cap = nh >= a.heads ? a.n_indices : ceil_div64(a.n_indices * nh, a.heads) + 128;
  w.cap = ceil_div64(w.cap, 8) * 8;
  const int64_t rows = a.total_q * nh;
  const int64_t ncols = (int64_t)a.batch * nh * a.ncol;
  w.status = static_cast<int*>(take(512));
  w.part_o = take((size_t)w.nsub * w.cap * a.d * part_elem_bytes);
  w.part_lse = static_cast<float*>(take(with_lse ? (size_t)w.nsub * w.cap * sizeof(float) : 0));
  w.lists_off = off;
  w.slot_base = static_cast<uint32_t*>(take((size_t)(ncols + 1) * sizeof(uint32_t)));
  w.row_ptr = static_cast<uint32_t*>(take((size_t)(rows + 1) * sizeof(uint32_t)));
  w.row_fill = static_cast<uint32_t*>(take((size_t)rows * sizeof(uint32_t)));
  w.row_pos = static_cast<uint32_t*>(take((size_t)w.cap * sizeof(uint32_t)));
  w.lists_bytes = off - w.lists_off;
  const int64_t longest = rows + 1 > ncols + 1 ? rows + 1 : ncols + 1;
  w.scan_tmp = static_cast<uint32_t*>(take(scan_tmp_elems(longest) * sizeof(uint32_t)));
  w.bytes = off;
  return off;
}

AttnWorkspace carve_attn_workspace(void* base, size_t bytes_available, const AttnArgs& a, size_t part_elem_bytes,
                                   bool with_lse, int heads_per_pass) {
  AttnWorkspace w;
  const int group = a.heads / a.heads_k;
  int nh = a.heads;
  if (heads_per_pass > 0) {
    nh = min(a.heads, max(group, heads_per_pass / group * group));
  } else if (base != nullptr) {   // the largest pass (whole kv-head groups) that fits what the caller gave
    while (nh > group && layout(w, nullptr, a, part_elem_bytes, with_lse, nh) > bytes_available) nh -= group;
  }
  layout(w, base, a, part_elem_bytes, with_lse, nh);
  return w;
}

size_t attn_workspace_bytes(int64_t total_q, int heads, int heads_k, int d, int64_t n_indices, int batch, int max_k,
                            int chunk, int heads_per_pass, bool backward) {
  AttnArgs a;
  memset(&a, 0, sizeof(a));
  a.total_q = total_q; a.heads = heads; a.heads_k = heads_k > 0 ? heads_k : heads; a.d = d; a.n_indices = n_indices;
  a.batch = batch; a.chunk = chunk > 0 ? chunk : 128; a.ncol = ceil_div(max_k, a.chunk);
  return carve_attn_workspace(nullptr, 0, a, 2, !backward, heads_per_pass > 0 ? heads_per_pass : heads)
      .bytes;
}

PassParams make_pass(const AttnArgs& a, const AttnWorkspace& w, int h0, int nh) {
  PassParams r;
  r.col_offsets = a.col_offsets; r.col_nnz = a.col_nnz; r.indices = a.indices; r.n_indices = a.n_indices;
  r.slot_base = w.slot_base;
  r.heads = a.heads; r.ncol = a.ncol; r.h0 = h0; r.nh = nh; r.nsub = w.nsub; r.kb = w.kb; r.chunk = a.chunk;
  r.cap = w.cap; r.status = w.status;
  r.slot_shift = w.fixed_k > 0 ? (int64_t)h0 * a.total_q * w.fixed_k : 0;
  return r;
}

// ------------------------------------------------------------------ slot and row lists
// slot_base[i + 1] = entries of the i-th column of the pass (0 if the column is malformed);
// an inclusive scan then turns the array into first slots
__global__ void __launch_bounds__(256) slot_count_kernel(PassParams r, uint32_t* slot_base, int batch) {
  const int64_t n = (int64_t)batch * r.nh * r.ncol;
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i == 0) slot_base[0] = 0;
  if (i >= n) return;
  const int c = (int)(i % r.ncol);
  const int hr = (int)((i / r.ncol) % r.nh);
  const int b = (int)(i / ((int64_t)r.ncol * r.nh));
  const int64_t ci = ((int64_t)b * r.heads + r.h0 + hr) * r.ncol + c;
  const int nnz = r.col_nnz[ci];
  const int64_t off = r.col_offsets[ci];
  slot_base[i + 1] = (nnz > 0 && off >= 0 && off + nnz <= r.n_indices) ? (uint32_t)nnz : 0u;
}

struct RowListParams {
  PassParams r;
  const int32_t* cu_q;
  uint32_t *row_ptr, *row_fill, *row_pos;
  int64_t total_q;
};

// grid (ncol, nh, batch): one CTA per column of the pass
template <bool kFill>
__global__ void __launch_bounds__(256) row_list_kernel(RowListParams p) {
  const int c = blockIdx.x, hr = blockIdx.y, b = blockIdx.z;
  const ColRef col = column_of(p.r, b, p.r.h0 + hr, c);
  if (col.nnz <= 0) return;
  const int q0 = p.cu_q[b], len_q = p.cu_q[b + 1] - q0;
  const int64_t rbase = (int64_t)hr * p.total_q + q0;
  for (int j = threadIdx.x; j < col.nnz; j += blockDim.x) {
    const int r = p.r.indices[col.off + j];
    if (r < 0 || r >= len_q) continue;
    if (!kFill) {
      atomicAdd(&p.row_ptr[rbase + r + 1], 1u);     // counts, shifted by one for the scan
    } else {
      const uint32_t k = atomicAdd(&p.row_fill[rbase + r], 1u);
      p.row_pos[p.row_ptr[rbase + r] + k] = (uint32_t)(col.slot + j);
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

static int inclusive_scan(uint32_t* data, int64_t n, uint32_t* tmp, cudaStream_t s) {
  const int nblocks = (int)ceil_div64(n, kScanItems);
  scan_block_kernel<<<nblocks, 1024, 0, s>>>(data, n, tmp);
  FMB_LAUNCH_CHECK("scan_block_kernel");
  if (nblocks > 1) {
    scan_sums_kernel<<<1, 1024, 0, s>>>(tmp, nblocks);
    FMB_LAUNCH_CHECK("scan_sums_kernel");
    scan_add_kernel<<<nblocks, 1024, 0, s>>>(data, n, tmp);
    FMB_LAUNCH_CHECK("scan_add_kernel");
  }
  return FMB_OK;
}

int build_row_lists(const AttnArgs& a, const AttnWorkspace& w, const PassParams& ps, cudaStream_t s) {
  const int64_t rows = a.total_q * ps.nh;
  const int64_t ncols = (int64_t)a.batch * ps.nh * a.ncol;
  // row_ptr and row_fill are neighbours in the workspace: one clear for both
  FMB_CUDA(cudaMemsetAsync(w.row_ptr, 0, (size_t)((char*)(w.row_fill + rows) - (char*)w.row_ptr), s));
  if (ncols == 0) return FMB_OK;
  slot_count_kernel<<<(unsigned)ceil_div64(ncols + 1, 256), 256, 0, s>>>(ps, w.slot_base, a.batch);
  FMB_LAUNCH_CHECK("slot_count_kernel");
  int rc = inclusive_scan(w.slot_base, ncols + 1, w.scan_tmp, s);
  if (rc) return rc;
  RowListParams p;
  p.r = ps; p.cu_q = a.cu_q; p.row_ptr = w.row_ptr; p.row_fill = w.row_fill; p.row_pos = w.row_pos;
  p.total_q = a.total_q;
  dim3 grid(a.ncol, ps.nh, a.batch);
  row_list_kernel<false><<<grid, 256, 0, s>>>(p);
  FMB_LAUNCH_CHECK("row_list_kernel<count>");
  rc = inclusive_scan(w.row_ptr, rows + 1, w.scan_tmp, s);
  if (rc) return rc;
  row_list_kernel<true><<<grid, 256, 0, s>>>(p);
  FMB_LAUNCH_CHECK("row_list_kernel<fill>");
  return FMB_OK;
}

// ------------------------------------------------------------------ combine kernels
// What a combine kernel needs to know about the pass
struct CombineParams {
  const uint32_t* row_ptr; const uint32_t* row_pos;
  int64_t total_q, cap;
  int heads_out;   // heads of the output tensor's row (for nothing but documentation)
  int h0, nh, nsub, d;
  int fixed_k;     // > 0: row lists handed over by the pattern builder: row `rid` owns the fixed_k places
                   // row_pos[rid*fixed_k ..], empty places hold 0xffffffff; row_ptr is not used
  int64_t slot_shift;               // handed-over rows hold positions in `indices`: slot = position - slot_shift
  const int* status; int* mirror;   // mirror != nullptr: the first combine kernel of the call's last pass copies
                                    // the call's status word there (see attn_status_mirror)
};
// The main kernels, which set the status word, have completed when a combine kernel starts.
__device__ __forceinline__ void mirror_status(const CombineParams& c) {
  if (c.mirror != nullptr && blockIdx.x == 0 && threadIdx.x == 0) *c.mirror = *c.status;
}
// first place and number of places of row `rid` in row_pos
__device__ __forceinline__ void row_span(const CombineParams& c, int64_t rid, int64_t& p0, int& n) {
  if (c.fixed_k > 0) {
    p0 = rid * c.fixed_k;
    n = c.fixed_k;
  } else {
    p0 = c.row_ptr[rid];
    n = (int)(c.row_ptr[rid + 1] - (uint32_t)p0);
  }
}
constexpr uint32_t kNoSlot = 0xffffffffu;

// Generic kernel: a warp per (token, head of the pass).  The row's partials are visited plane by
// plane, inside a plane in ascending slot order = ascending (sb*cap + slot).
// next_slot(): smallest slot of the row that is greater than `last` (-1 first).
__device__ __forceinline__ int64_t next_slot(const uint32_t* rp, int n, int64_t last, int lane) {
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

// The combine kernels walk "virtual blocks" of 256 threads with a grid-stride loop, so that the
// later stages of the cascade can be launched with a small grid: they usually find their flag
// clear and must cost microseconds, not a scan of the whole block range.
template <typename T>
__device__ __forceinline__ void fwd_combine_body(int64_t vblock, const T* __restrict__ part_o,
                                                 const float* __restrict__ part_lse, const CombineParams& c,
                                                 T* out, int64_t o_rs, int64_t o_hs, float* lse, int min_n) {
  using T2 = typename Elem<T>::T2;
  const int64_t wid = (vblock * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= c.total_q * c.nh) return;
  const int64_t t = wid / c.nh;
  const int hr = (int)(wid - t * c.nh);
  const int64_t rid = (int64_t)hr * c.total_q + t;
  int64_t p0;
  int n;
  row_span(c, rid, p0, n);
  if (n * c.nsub < min_n) return;
  const uint32_t* rp = c.row_pos + p0;
  float m = -CUDART_INF_F;
  for (int sb = 0; sb < c.nsub; ++sb)
    for (int j = lane; j < n; j += 32)
      if (rp[j] != kNoSlot) m = fmaxf(m, part_lse[(int64_t)sb * c.cap + rp[j] - c.slot_shift]);
#pragma unroll
  for (int o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  float2 acc[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) acc[i] = make_float2(0.f, 0.f);
  float ssum = 0.f;
  if (m > -CUDART_INF_F) {
    for (int sb = 0; sb < c.nsub; ++sb) {
      int64_t last = -1;
      for (int r = 0; r < n; ++r) {
        const int64_t raw = next_slot(rp, n, last, lane);
        if (raw >= (int64_t)kNoSlot) break;      // the remaining places of the row are empty
        last = raw;
        const int64_t slot = raw - c.slot_shift;
        const int64_t pp = (int64_t)sb * c.cap + slot;
        const float wgt = __expf(part_lse[pp] - m);
        ssum += wgt;
        const T* src = part_o + pp * c.d;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int col = lane * 2 + i * 64;
          if (col < c.d) {
            const float2 x = Elem<T>::to_f2(*reinterpret_cast<const T2*>(src + part_col(slot, col, 8)));
            acc[i].x = fmaf(wgt, x.x, acc[i].x);
            acc[i].y = fmaf(wgt, x.y, acc[i].y);
          }
        }
      }
    }
  }
  const float inv = ssum > 0.f ? 1.f / ssum : 0.f;
  const int h = c.h0 + hr;
  T* dst = out + t * o_rs + (int64_t)h * o_hs;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int col = lane * 2 + i * 64;
    if (col < c.d) *reinterpret_cast<T2*>(dst + col) = Elem<T>::from_f2(acc[i].x * inv, acc[i].y * inv);
  }
  if (lane == 0) lse[(int64_t)h * c.total_q + t] = ssum > 0.f ? m + logf(ssum) : CUDART_INF_F;
}
template <typename T>
__global__ void __launch_bounds__(256) fwd_combine_kernel(const T* __restrict__ part_o,
                                                          const float* __restrict__ part_lse, CombineParams c,
                                                          T* out, int64_t o_rs, int64_t o_hs, float* lse,
                                                          const int* only_if, int min_n, int64_t nvb) {
  mirror_status(c);
  if (only_if && *only_if == 0) return;   // the earlier stages met no row they had to leave
  for (int64_t vb = blockIdx.x; vb < nvb; vb += gridDim.x)
    fwd_combine_body<T>(vb, part_o, part_lse, c, out, o_rs, o_hs, lse, min_n);
}

template <typename T>
__device__ __forceinline__ void bwd_combine_body(int64_t vblock, const T* __restrict__ part_dq, const CombineParams& c,
                                                 T* dq, int64_t rs, int64_t hs, int min_n) {
  using T2 = typename Elem<T>::T2;
  const int64_t wid = (vblock * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= c.total_q * c.nh) return;
  const int64_t t = wid / c.nh;
  const int hr = (int)(wid - t * c.nh);
  const int64_t rid = (int64_t)hr * c.total_q + t;
  int64_t p0;
  int n;
  row_span(c, rid, p0, n);
  if (n * c.nsub < min_n) return;
  const uint32_t* rp = c.row_pos + p0;
  float2 acc[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) acc[i] = make_float2(0.f, 0.f);
  for (int sb = 0; sb < c.nsub; ++sb) {
    int64_t last = -1;
    for (int r = 0; r < n; ++r) {
      const int64_t raw = next_slot(rp, n, last, lane);
      if (raw >= (int64_t)kNoSlot) break;        // the remaining places of the row are empty
      last = raw;
      const int64_t slot = raw - c.slot_shift;
      const T* src = part_dq + ((int64_t)sb * c.cap + slot) * c.d;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int col = lane * 2 + i * 64;
        if (col < c.d) {
          const float2 x = Elem<T>::to_f2(*reinterpret_cast<const T2*>(src + part_col(slot, col, 8)));
          acc[i].x += x.x;
          acc[i].y += x.y;
        }
      }
    }
  }
  T* dst = dq + t * rs + (int64_t)(c.h0 + hr) * hs;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int col = lane * 2 + i * 64;
    if (col < c.d) *reinterpret_cast<T2*>(dst + col) = Elem<T>::from_f2(acc[i].x, acc[i].y);
  }
}
template <typename T>
__global__ void __launch_bounds__(256) bwd_combine_kernel(const T* __restrict__ part_dq, CombineParams c, T* dq,
                                                          int64_t rs, int64_t hs, const int* only_if, int min_n,
                                                          int64_t nvb) {
  mirror_status(c);
  if (only_if && *only_if == 0) return;
  for (int64_t vb = blockIdx.x; vb < nvb; vb += gridDim.x) bwd_combine_body<T>(vb, part_dq, c, dq, rs, hs, min_n);
}

// ------------------------------------------------------------------ fast combine (rows of <= G partials)
// G lanes per (token, head) row, 32/G rows per warp.  Lane j of a group first fetches the plane
// position (sb*cap + slot) and log-sum-exp of the row's j-th partial; the group ranks the positions
// (merge order = ascending position, whatever order the atomics of the row-list build produced);
// then every lane fetches its d/G elements of ALL the row's partial rows before the ordered
// accumulation.  Several rows per warp and all loads of a row in flight at once hide the chain of
// dependent, scattered reads.  Rows with more than G partials set *overflow and are left to the
// next kernel (larger G, finally the generic one).
template <int G>
__device__ __forceinline__ unsigned group_mask(int lane) {
  return G == 32 ? 0xffffffffu : (((1u << G) - 1u) << (lane & ~(G - 1)));
}

// common prologue: the row of this lane group and the plane position held by this lane
struct GroupRow {
  int64_t t; int hr; int64_t rid; int n; bool mine; bool valid; uint32_t pos; uint32_t slot;
};
template <int G>
__device__ __forceinline__ GroupRow group_row(int64_t vblock, const CombineParams& c, int min_n, int* overflow) {
  GroupRow g;
  const int lane = threadIdx.x & 31, gl = lane & (G - 1);
  const int64_t gid = ((vblock * blockDim.x + threadIdx.x) >> 5) * (32 / G) + (lane / G);
  const bool row_ok = gid < c.total_q * c.nh;
  g.t = row_ok ? gid / c.nh : 0;
  g.hr = row_ok ? (int)(gid - g.t * c.nh) : 0;
  g.rid = (int64_t)g.hr * c.total_q + g.t;
  int64_t p0 = 0;
  int n_e = 0;
  if (row_ok) row_span(c, g.rid, p0, n_e);
  g.n = n_e * c.nsub;                       // partials of the row
  g.mine = row_ok && g.n >= min_n;          // rows below min_n were done by the previous kernel
  if (g.n > G) {
    if (gl == 0) *overflow = 1;
    g.mine = false;
  }
  if (!g.mine) g.n = 0;
  g.valid = gl < g.n;
  g.slot = g.valid ? c.row_pos[p0 + gl / c.nsub] : 0u;
  if (g.slot == kNoSlot) g.valid = false;      // an empty place of a handed-over row list
  else g.slot -= (uint32_t)c.slot_shift;
  g.pos = g.valid ? (uint32_t)((gl % c.nsub) * c.cap) + g.slot : 0xffffffffu;
  return g;
}

template <typename T, int G, int EPL>
__device__ __forceinline__ void fwd_combine_group_body(int64_t vblock, const T* __restrict__ part_o,
                                                       const float* __restrict__ part_lse, const CombineParams& c,
                                                       T* out, int64_t o_rs, int64_t o_hs, float* lse, int min_n,
                                                       int* overflow) {
  constexpr int d = G * EPL;
  constexpr int NV = EPL / 8;                 // 16-byte loads per partial row per lane
  static_assert(EPL % 8 == 0, "a lane owns whole 16-byte chunks");
  const int lane = threadIdx.x & 31, gl = lane & (G - 1);
  const unsigned gm = group_mask<G>(lane);
  const GroupRow g = group_row<G>(vblock, c, min_n, overflow);
  // the log-sum-exp of this lane's partial: requested first, used last (the partial rows are
  // requested before anything waits for it, so that there is ONE round trip to memory, not two)
  const float l = g.valid ? part_lse[g.pos] : -CUDART_INF_F;
  int rank = 0;
#pragma unroll
  for (int i = 0; i < G; ++i) rank += (__shfl_sync(gm, g.pos, i, G) < g.pos) ? 1 : 0;
  float acc[EPL];
#pragma unroll
  for (int i = 0; i < EPL; ++i) acc[i] = 0.f;
  float ssum = 0.f;
  float m = -CUDART_INF_F, w = 0.f;
  constexpr int B = G < 8 ? G : 8;            // partial rows in flight per step
#pragma unroll
  for (int r0 = 0; r0 < G; r0 += B) {
    uint4 x[B][NV];
    int srcs[B];
#pragma unroll
    for (int k = 0; k < B; ++k) {
      // the lane of this group whose partial has rank r0+k (none if the row is shorter).  Every
      // partial row of a listed slot has been written (zeros for a row that saw no key), so it is
      // fetched whatever its weight turns out to be.
      const unsigned hit = __ballot_sync(0xffffffffu, g.valid && rank == r0 + k) & gm;
      const int src = hit ? (__ffs(hit) - 1) : lane;
      srcs[k] = hit ? src : -1;
      const uint32_t pk = __shfl_sync(0xffffffffu, g.pos, src);
      const uint32_t sk = __shfl_sync(0xffffffffu, g.slot, src);
      if (hit) {
        const T* row = part_o + (int64_t)pk * d;
#pragma unroll
        for (int v = 0; v < NV; ++v) x[k][v] = *reinterpret_cast<const uint4*>(row + part_col(sk, gl * EPL + 8 * v, 8));
      } else {
#pragma unroll
        for (int v = 0; v < NV; ++v) x[k][v] = make_uint4(0, 0, 0, 0);
      }
    }
    if (r0 == 0) {   // weights: the row maximum of the partial log-sum-exps
      m = l;
#pragma unroll
      for (int o = G / 2; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(gm, m, o, G));
      w = (g.valid && m > -CUDART_INF_F) ? __expf(l - m) : 0.f;
    }
#pragma unroll
    for (int k = 0; k < B; ++k) {
      // executed by every lane: groups of one warp differ in srcs[k] when their rows have
      // different numbers of partials
      const float w_src = __shfl_sync(0xffffffffu, w, srcs[k] < 0 ? lane : srcs[k]);
      const float wk = srcs[k] < 0 ? 0.f : w_src;
      ssum += wk;
#pragma unroll
      for (int v = 0; v < NV; ++v) {
        float f[8];
        unpack8<T>(x[k][v], f);
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[8 * v + e] = fmaf(wk, f[e], acc[8 * v + e]);
      }
    }
  }
  if (g.mine) {
    const float inv = ssum > 0.f ? 1.f / ssum : 0.f;
    const int h = c.h0 + g.hr;
    T* dst = out + g.t * o_rs + (int64_t)h * o_hs + gl * EPL;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[8 * v + e] *= inv;
      *reinterpret_cast<uint4*>(dst + 8 * v) = pack8<T>(acc + 8 * v);
    }
    if (gl == 0) lse[(int64_t)h * c.total_q + g.t] = ssum > 0.f ? m + logf(ssum) : CUDART_INF_F;
  }
}
template <typename T, int G, int EPL>
__global__ void __launch_bounds__(256, EPL <= 8 ? 3 : 2) fwd_combine_group_kernel(const T* __restrict__ part_o,
                                                                const float* __restrict__ part_lse,
                                                                CombineParams c, T* out, int64_t o_rs, int64_t o_hs,
                                                                float* lse, int min_n, const int* only_if,
                                                                int* overflow, int64_t nvb) {
  mirror_status(c);
  if (only_if && *only_if == 0) return;
  for (int64_t vb = blockIdx.x; vb < nvb; vb += gridDim.x)
    fwd_combine_group_body<T, G, EPL>(vb, part_o, part_lse, c, out, o_rs, o_hs, lse, min_n, overflow);
}

template <typename T, int G, int EPL>
__device__ __forceinline__ void bwd_combine_group_body(int64_t vblock, const T* __restrict__ part_dq,
                                                       const CombineParams& c, T* dq, int64_t rs, int64_t hs,
                                                       int min_n, int* overflow) {
  constexpr int d = G * EPL;
  constexpr int NV = EPL / 8;                 // 16-byte loads per partial row per lane
  static_assert(EPL % 8 == 0, "a lane owns whole 16-byte chunks");
  const int lane = threadIdx.x & 31, gl = lane & (G - 1);
  const unsigned gm = group_mask<G>(lane);
  const GroupRow g = group_row<G>(vblock, c, min_n, overflow);
  int rank = 0;
#pragma unroll
  for (int i = 0; i < G; ++i) rank += (__shfl_sync(gm, g.pos, i, G) < g.pos) ? 1 : 0;
  float acc[EPL];
#pragma unroll
  for (int i = 0; i < EPL; ++i) acc[i] = 0.f;
  constexpr int B = G < 8 ? G : 8;            // partial rows in flight per step
#pragma unroll
  for (int r0 = 0; r0 < G; r0 += B) {
    uint4 x[B][NV];
#pragma unroll
    for (int k = 0; k < B; ++k) {
      const unsigned hit = __ballot_sync(0xffffffffu, g.valid && rank == r0 + k) & gm;
      const int src = hit ? (__ffs(hit) - 1) : lane;
      const uint32_t pk = __shfl_sync(0xffffffffu, g.pos, src);
      const uint32_t sk = __shfl_sync(0xffffffffu, g.slot, src);
      if (hit) {
        const T* row = part_dq + (int64_t)pk * d;
#pragma unroll
        for (int v = 0; v < NV; ++v) x[k][v] = *reinterpret_cast<const uint4*>(row + part_col(sk, gl * EPL + 8 * v, 8));
      } else {
#pragma unroll
        for (int v = 0; v < NV; ++v) x[k][v] = make_uint4(0, 0, 0, 0);
      }
    }
#pragma unroll
    for (int k = 0; k < B; ++k) {
#pragma unroll
      for (int v = 0; v < NV; ++v) {
        float f[8];
        unpack8<T>(x[k][v], f);
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[8 * v + e] += f[e];
      }
    }
  }
  if (g.mine) {
    T* dst = dq + g.t * rs + (int64_t)(c.h0 + g.hr) * hs + gl * EPL;
#pragma unroll
    for (int v = 0; v < NV; ++v) *reinterpret_cast<uint4*>(dst + 8 * v) = pack8<T>(acc + 8 * v);
  }
}
template <typename T, int G, int EPL>
__global__ void __launch_bounds__(256) bwd_combine_group_kernel(const T* __restrict__ part_dq, CombineParams c,
                                                                T* dq, int64_t rs, int64_t hs, int min_n,
                                                                const int* only_if, int* overflow, int64_t nvb) {
  mirror_status(c);
  if (only_if && *only_if == 0) return;
  for (int64_t vb = blockIdx.x; vb < nvb; vb += gridDim.x)
    bwd_combine_group_body<T, G, EPL>(vb, part_dq, c, dq, rs, hs, min_n, overflow);
}

// ------------------------------------------------------------------ wide combine (rows of <= 32 partials)
// A warp per (token, head) row.  Lane j fetches the position and log-sum-exp of the row's j-th
// partial and the warp ranks the positions, as above.  A partial row is D/8 16-byte chunks, so D/8
// lanes fetch one partial row and the warp fetches 32/(D/8) partial rows per step, eight steps in
// flight; lane group s accumulates the partials of rank s, s + 32/(D/8), ... in ascending order and
// the groups are added at the end in a fixed order.  FWD weights the partials by
// exp(lse_j - max lse) and writes the row's log-sum-exp; the backward form is a plain sum.
template <typename T, int D, bool FWD>
__device__ __forceinline__ void combine_wide_body(int64_t vblock, const T* __restrict__ part,
                                                  const float* __restrict__ part_lse, const CombineParams& c,
                                                  T* out, int64_t rs, int64_t hs, float* lse, int min_n,
                                                  int* overflow) {
  constexpr int LPR = D / 8;                  // lanes per partial row
  constexpr int PPS = 32 / LPR;               // partial rows per step
  constexpr int B = 8;                        // steps in flight
  static_assert(D == 64 || D == 128 || D == 256, "a partial row is 8, 16 or 32 chunks");
  const int lane = threadIdx.x & 31, sub = lane / LPR, ch = lane % LPR;
  const GroupRow g = group_row<32>(vblock, c, min_n, overflow);
  if (!g.mine) return;                        // the same for every lane of the warp
  float l = -CUDART_INF_F;
  if (FWD && g.valid) l = part_lse[g.pos];
  int rank = 0;
#pragma unroll
  for (int i = 0; i < 32; ++i) rank += (__shfl_sync(0xffffffffu, g.pos, i) < g.pos) ? 1 : 0;
  // the row's partials in use (a handed-over row list may have empty places: they rank last)
  const int nv = __popc(__ballot_sync(0xffffffffu, g.valid));
  int inv = 0;                                // the lane that holds the partial of rank `lane`
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const int ri = __shfl_sync(0xffffffffu, rank, i);
    const bool vi = (__shfl_sync(0xffffffffu, (int)g.valid, i) != 0);
    if (vi && ri == lane) inv = i;
  }
  float m = 0.f, w = 1.f, ssum = 1.f;
  if (FWD) {
    m = l;
#pragma unroll
    for (int o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    w = (g.valid && m > -CUDART_INF_F) ? __expf(l - m) : 0.f;
    // summed with the weights in rank order: the order in which the row's partials sit in the
    // lanes is that of the row list, which the atomics of its build leave undefined
    const float w_ranked = __shfl_sync(0xffffffffu, w, inv);
    ssum = lane < nv ? w_ranked : 0.f;
#pragma unroll
    for (int o = 16; o; o >>= 1) ssum += __shfl_xor_sync(0xffffffffu, ssum, o);
  }
  float acc[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) acc[e] = 0.f;
  for (int r0 = 0; r0 < nv; r0 += PPS * B) {
    uint4 x[B];
    float wk[B];
#pragma unroll
    for (int k = 0; k < B; ++k) {
      const int want = r0 + k * PPS + sub;
      const bool hit = want < nv;
      const int src = __shfl_sync(0xffffffffu, inv, want & 31);
      const uint32_t pk = __shfl_sync(0xffffffffu, g.pos, src);
      const uint32_t sk = __shfl_sync(0xffffffffu, g.slot, src);
      const float ws = __shfl_sync(0xffffffffu, w, src);
      wk[k] = hit ? ws : 0.f;
      x[k] = hit ? *reinterpret_cast<const uint4*>(part + (int64_t)pk * D + part_col(sk, ch * 8, 8))
                 : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int k = 0; k < B; ++k) {
      float f[8];
      unpack8<T>(x[k], f);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] = FWD ? fmaf(wk[k], f[e], acc[e]) : acc[e] + f[e];   // x is 0 past the row's end
    }
  }
#pragma unroll
  for (int o = LPR; o < 32; o <<= 1) {
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], o);
  }
  const int h = c.h0 + g.hr;
  if (sub == 0) {
    const float inv_s = FWD ? (ssum > 0.f ? 1.f / ssum : 0.f) : 1.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] *= inv_s;
    *reinterpret_cast<uint4*>(out + g.t * rs + (int64_t)h * hs + ch * 8) = pack8<T>(acc);
  }
  if (FWD && lane == 0) lse[(int64_t)h * c.total_q + g.t] = ssum > 0.f ? m + logf(ssum) : CUDART_INF_F;
}
template <typename T, int D, bool FWD>
__global__ void __launch_bounds__(256) combine_wide_kernel(const T* __restrict__ part,
                                                           const float* __restrict__ part_lse, CombineParams c,
                                                           T* out, int64_t rs, int64_t hs, float* lse, int min_n,
                                                           const int* only_if, int* overflow, int64_t nvb) {
  mirror_status(c);
  if (only_if && *only_if == 0) return;
  for (int64_t vb = blockIdx.x; vb < nvb; vb += gridDim.x)
    combine_wide_body<T, D, FWD>(vb, part, part_lse, c, out, rs, hs, lse, min_n, overflow);
}

// D[h, t] = sum_d dO.O.  LPR lanes per row, each with one 16-byte load of dO and of O (LPR = d / 8
// when that is a power of two); LPR = 0 selects the generic warp-per-row form.
template <typename T, int LPR>
__global__ void __launch_bounds__(256) dot_do_o_kernel(const T* __restrict__ dout, int64_t do_rs, int64_t do_hs,
                                                       const T* __restrict__ o, int64_t o_rs, int64_t o_hs,
                                                       float* softmax_d, int64_t total_q, int heads, int d) {
  using T2 = typename Elem<T>::T2;
  const int lane = threadIdx.x & 31;
  const int64_t wid = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (LPR > 0) {
    constexpr int L = LPR > 0 ? LPR : 32;
    const int64_t row = wid * (32 / L) + lane / L;
    float s = 0.f;
    if (row < total_q * heads) {
      const int64_t t = row / heads;
      const int h = (int)(row - t * heads);
      const int c = (lane % L) * 8;
      float x[8], y[8];
      unpack8<T>(ldg_nc_16(dout + t * do_rs + (int64_t)h * do_hs + c), x);
      unpack8<T>(ldg_nc_16(o + t * o_rs + (int64_t)h * o_hs + c), y);
#pragma unroll
      for (int e = 0; e < 8; ++e) s = fmaf(x[e], y[e], s);
    }
#pragma unroll
    for (int o2 = L / 2; o2; o2 >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o2);
    if (row < total_q * heads && lane % L == 0) {
      const int64_t t = row / heads;
      softmax_d[(int64_t)(row - t * heads) * total_q + t] = s;
    }
    return;
  }
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

static int64_t warp_grid(int64_t warps) { return ceil_div64(warps, 8); }

// Cascade: lane groups of 8 (rows of <= 8 partials), of 16 (<= 16, head dims of 128 and more), the
// warp-per-row wide kernel (<= 32), then the generic kernel; each later stage runs only the rows the earlier ones left and exits at once if
// there were none.
static int64_t group_grid(int64_t rows, int G) { return ceil_div64(ceil_div64(rows, 32 / G), 8); }
int sm_count() {
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
    n = 148;
  return n;
}

// First cascade stage: persistent CTAs, as many as are resident (2 per SM at 128 registers); measured
// at 64K tokens 0.24 ms per step faster than one CTA per block of rows (65,536 short-lived CTAs).
// (Prefetching the next blocks' row lists inside the loop was tried and lost 0.7 ms to spills; with the
// pattern builder's fixed-stride rows the prefetch is one register and changed nothing: 0.94 against
// 0.92 ms in the backward combine, which reads its 4.8 GB at 80 % of the measured copy bandwidth.)
static unsigned first_grid(int64_t nvb, int ctas_per_sm = 2) {
  const int64_t cap = (int64_t)sm_count() * ctas_per_sm;
  return (unsigned)(nvb < cap ? nvb : cap);
}
// grid of a later cascade stage: enough CTAs to fill the GPU if it does have work
static unsigned late_grid(int64_t nvb) {
  const int64_t cap = (int64_t)sm_count() * 8;
  return (unsigned)(nvb < cap ? (nvb > 0 ? nvb : 1) : cap);
}

static CombineParams make_combine(const AttnArgs& a, const AttnWorkspace& w, const PassParams& ps) {
  CombineParams c;
  c.row_ptr = w.row_ptr; c.row_pos = w.row_pos; c.total_q = a.total_q; c.cap = w.cap; c.heads_out = a.heads;
  c.h0 = ps.h0; c.nh = ps.nh; c.nsub = w.nsub; c.d = a.d;
  c.fixed_k = w.fixed_k;
  c.slot_shift = ps.slot_shift;
  if (w.fixed_k > 0) c.row_pos = w.row_pos + (int64_t)ps.h0 * a.total_q * w.fixed_k;   // the pass's heads
  c.status = w.status;
  c.mirror = (ps.h0 + ps.nh >= a.heads) ? w.mirror : nullptr;   // the call's last pass
  return c;
}

template <typename T, int D>
static int fwd_combine_dispatch(const AttnArgs& a, const AttnWorkspace& w, const PassParams& ps, cudaStream_t s) {
  const int64_t rows = a.total_q * ps.nh;
  const CombineParams c = make_combine(a, w, ps);
  int* ovf = w.status + 1;   // words 1..3 of the status block, zeroed with it
  const T* po = (const T*)w.part_o;
  T* out = (T*)a.o;
  const int64_t nb8 = group_grid(rows, 8), nbw = warp_grid(rows);
  if (c.fixed_k > 0) {   // every row has fixed_k * nsub places: the stage is known on the host, one launch
    const int places = c.fixed_k * c.nsub;
    // 8 lanes per row while a lane's share of a partial row is at most 32 bytes (at d = 128, 16 lanes
    // for these rows: 1.57 ms against 1.21 ms at 64K; at d = 256, 8 lanes would hold 128 registers of
    // loads in flight each: 3.5 ms against the 16-lane form's time for the same bytes)
    if (places <= 8 && D <= 128) {
      fwd_combine_group_kernel<T, 8, D / 8><<<first_grid(nb8), 256, 0, s>>>(po, w.part_lse, c, out, a.o_rs, a.o_hs, a.lse,
                                                                          0, nullptr, ovf, nb8);
      FMB_LAUNCH_CHECK("fwd_combine_group_kernel<8>");
    } else if (D >= 128 && places <= 16) {
      if constexpr (D >= 128) {
        const int64_t nb16 = group_grid(rows, 16);
        fwd_combine_group_kernel<T, 16, D / 16><<<first_grid(nb16, D / 16 <= 8 ? 3 : 2), 256, 0, s>>>(
            po, w.part_lse, c, out, a.o_rs, a.o_hs, a.lse, 0, nullptr, ovf, nb16);
        FMB_LAUNCH_CHECK("fwd_combine_group_kernel<16>");
      }
    } else if (places <= 32) {
      combine_wide_kernel<T, D, true><<<late_grid(nbw), 256, 0, s>>>(po, w.part_lse, c, out, a.o_rs, a.o_hs, a.lse, 0,
                                                                     nullptr, ovf, nbw);
      FMB_LAUNCH_CHECK("combine_wide_kernel<fwd>");
    } else {
      fwd_combine_kernel<T><<<late_grid(nbw), 256, 0, s>>>(po, w.part_lse, c, out, a.o_rs, a.o_hs, a.lse, nullptr, 0, nbw);
      FMB_LAUNCH_CHECK("fwd_combine_kernel");
    }
    return FMB_OK;
  }
  int* left = ovf;            // flag set by the stage before; rows of at least min_n partials are left
  int min_n = 9;
  if constexpr (D <= 128) {
    fwd_combine_group_kernel<T, 8, D / 8><<<first_grid(nb8), 256, 0, s>>>(po, w.part_lse, c, out, a.o_rs, a.o_hs, a.lse, 0,
                                                                        nullptr, ovf, nb8);
    FMB_LAUNCH_CHECK("fwd_combine_group_kernel<8>");
  }
  if constexpr (D >= 128) {   // 16 lanes of a row own whole 16-byte chunks: two rows per warp
    const int64_t nb16 = group_grid(rows, 16);
    if constexpr (D <= 128)
      fwd_combine_group_kernel<T, 16, D / 16><<<late_grid(nb16), 256, 0, s>>>(po, w.part_lse, c, out, a.o_rs, a.o_hs,
                                                                             a.lse, 9, ovf, ovf + 1, nb16);
    else                      // d = 256: the first stage
      fwd_combine_group_kernel<T, 16, D / 16><<<first_grid(nb16), 256, 0, s>>>(po, w.part_lse, c, out, a.o_rs, a.o_hs,
                                                                              a.lse, 0, nullptr, ovf + 1, nb16);
    FMB_LAUNCH_CHECK("fwd_combine_group_kernel<16>");
    left = ovf + 1;
    min_n = 17;
  }
  combine_wide_kernel<T, D, true><<<late_grid(nbw), 256, 0, s>>>(po, w.part_lse, c, out, a.o_rs, a.o_hs, a.lse, min_n,
                                                                 left, ovf + 2, nbw);
  FMB_LAUNCH_CHECK("combine_wide_kernel<fwd>");
  fwd_combine_kernel<T><<<late_grid(nbw), 256, 0, s>>>(po, w.part_lse, c, out, a.o_rs, a.o_hs, a.lse, ovf + 2, 33, nbw);
  FMB_LAUNCH_CHECK("fwd_combine_kernel");
  return FMB_OK;
}

template <typename T>
static int fwd_combine_any(const AttnArgs& a, const AttnWorkspace& w, const PassParams& ps, cudaStream_t s) {
  if (a.d == 64) return fwd_combine_dispatch<T, 64>(a, w, ps, s);
  if (a.d == 128) return fwd_combine_dispatch<T, 128>(a, w, ps, s);
  if (a.d == 256) return fwd_combine_dispatch<T, 256>(a, w, ps, s);
  const int64_t rows = a.total_q * ps.nh;
  fwd_combine_kernel<T><<<warp_grid(rows), 256, 0, s>>>((const T*)w.part_o, w.part_lse, make_combine(a, w, ps),
                                                        (T*)a.o, a.o_rs, a.o_hs, a.lse, nullptr, 0, warp_grid(rows));
  FMB_LAUNCH_CHECK("fwd_combine_kernel");
  return FMB_OK;
}

int launch_fwd_combine(const AttnArgs& a, const AttnWorkspace& w, const PassParams& ps, cudaStream_t s) {
  if (a.total_q * ps.nh == 0) return FMB_OK;
  return a.dtype == FMB_BF16 ? fwd_combine_any<__nv_bfloat16>(a, w, ps, s) : fwd_combine_any<__half>(a, w, ps, s);
}

template <typename T, int D>
static int bwd_combine_dispatch(const AttnArgs& a, const AttnWorkspace& w, const PassParams& ps, cudaStream_t s) {
  const int64_t rows = a.total_q * ps.nh;
  const CombineParams c = make_combine(a, w, ps);
  int* ovf = w.status + 1;
  const T* pd = (const T*)w.part_o;
  T* dq = (T*)a.dq;
  const int64_t nb8 = group_grid(rows, 8), nbw = warp_grid(rows);
  if (c.fixed_k > 0) {   // every row has fixed_k * nsub places: the stage is known on the host, one launch
    const int places = c.fixed_k * c.nsub;
    if (places <= 8 && D <= 128) {
      bwd_combine_group_kernel<T, 8, D / 8><<<first_grid(nb8), 256, 0, s>>>(pd, c, dq, a.dq_rs, a.dq_hs, 0, nullptr, ovf, nb8);
      FMB_LAUNCH_CHECK("bwd_combine_group_kernel<8>");
    } else if (D >= 128 && places <= 16) {
      if constexpr (D >= 128) {
        const int64_t nb16 = group_grid(rows, 16);
        bwd_combine_group_kernel<T, 16, D / 16><<<first_grid(nb16), 256, 0, s>>>(pd, c, dq, a.dq_rs, a.dq_hs, 0, nullptr,
                                                                                ovf, nb16);
        FMB_LAUNCH_CHECK("bwd_combine_group_kernel<16>");
      }
    } else if (places <= 32) {
      combine_wide_kernel<T, D, false><<<late_grid(nbw), 256, 0, s>>>(pd, nullptr, c, dq, a.dq_rs, a.dq_hs, nullptr, 0,
                                                                      nullptr, ovf, nbw);
      FMB_LAUNCH_CHECK("combine_wide_kernel<bwd>");
    } else {
      bwd_combine_kernel<T><<<late_grid(nbw), 256, 0, s>>>(pd, c, dq, a.dq_rs, a.dq_hs, nullptr, 0, nbw);
      FMB_LAUNCH_CHECK("bwd_combine_kernel");
    }
    return FMB_OK;
  }
  int* left = ovf;
  int min_n = 9;
  if constexpr (D <= 128) {
    bwd_combine_group_kernel<T, 8, D / 8><<<first_grid(nb8), 256, 0, s>>>(pd, c, dq, a.dq_rs, a.dq_hs, 0, nullptr, ovf, nb8);
    FMB_LAUNCH_CHECK("bwd_combine_group_kernel<8>");
  }
  if constexpr (D >= 128) {
    const int64_t nb16 = group_grid(rows, 16);
    if constexpr (D <= 128)
      bwd_combine_group_kernel<T, 16, D / 16><<<late_grid(nb16), 256, 0, s>>>(pd, c, dq, a.dq_rs, a.dq_hs, 9, ovf, ovf + 1,
                                                                             nb16);
    else
      bwd_combine_group_kernel<T, 16, D / 16><<<first_grid(nb16), 256, 0, s>>>(pd, c, dq, a.dq_rs, a.dq_hs, 0, nullptr,
                                                                              ovf + 1, nb16);
    FMB_LAUNCH_CHECK("bwd_combine_group_kernel<16>");
    left = ovf + 1;
    min_n = 17;
  }
  combine_wide_kernel<T, D, false><<<late_grid(nbw), 256, 0, s>>>(pd, nullptr, c, dq, a.dq_rs, a.dq_hs, nullptr, min_n,
                                                                  left, ovf + 2, nbw);
  FMB_LAUNCH_CHECK("combine_wide_kernel<bwd>");
  bwd_combine_kernel<T><<<late_grid(nbw), 256, 0, s>>>(pd, c, dq, a.dq_rs, a.dq_hs, ovf + 2, 33, nbw);
  FMB_LAUNCH_CHECK("bwd_combine_kernel");
  return FMB_OK;
}

template <typename T>
static int bwd_combine_any(const AttnArgs& a, const AttnWorkspace& w, const PassParams& ps, cudaStream_t s) {
  if (a.d == 64) return bwd_combine_dispatch<T, 64>(a, w, ps, s);
  if (a.d == 128) return bwd_combine_dispatch<T, 128>(a, w, ps, s);
  if (a.d == 256) return bwd_combine_dispatch<T, 256>(a, w, ps, s);
  const int64_t rows = a.total_q * ps.nh;
  bwd_combine_kernel<T><<<warp_grid(rows), 256, 0, s>>>((const T*)w.part_o, make_combine(a, w, ps), (T*)a.dq,
                                                        a.dq_rs, a.dq_hs, nullptr, 0, warp_grid(rows));
  FMB_LAUNCH_CHECK("bwd_combine_kernel");
  return FMB_OK;
}

int launch_bwd_combine(const AttnArgs& a, const AttnWorkspace& w, const PassParams& ps, cudaStream_t s) {
  if (a.total_q * ps.nh == 0) return FMB_OK;
  return a.dtype == FMB_BF16 ? bwd_combine_any<__nv_bfloat16>(a, w, ps, s) : bwd_combine_any<__half>(a, w, ps, s);
}

template <typename T>
static int dot_do_o_dispatch(const AttnArgs& a, cudaStream_t s) {
  const int64_t rows = a.total_q * a.heads;
  const T* dout = (const T*)a.dout;
  const T* o = (const T*)a.o;
#define FMB_DOT(LPR_)                                                                                        \
  dot_do_o_kernel<T, LPR_><<<(unsigned)warp_grid(ceil_div64(rows, LPR_ ? 32 / (LPR_ ? LPR_ : 1) : 1)), 256, 0, s>>>( \
      dout, a.do_rs, a.do_hs, o, a.o_rs, a.o_hs, a.softmax_d, a.total_q, a.heads, a.d)
  if (a.d == 128) FMB_DOT(16);
  else if (a.d == 64) FMB_DOT(8);
  else if (a.d == 256) FMB_DOT(32);
  else FMB_DOT(0);
#undef FMB_DOT
  FMB_LAUNCH_CHECK("dot_do_o_kernel");
  return FMB_OK;
}

int launch_dot_do_o(const AttnArgs& a, cudaStream_t s) {
  if (a.total_q * a.heads == 0) return FMB_OK;
  return a.dtype == FMB_BF16 ? dot_do_o_dispatch<__nv_bfloat16>(a, s) : dot_do_o_dispatch<__half>(a, s);
}

// ------------------------------------------------------------------ drivers
// Each pass: slot and row lists of its heads, main kernel (partials), combine.  The status block
// is cleared once per call, so a failure in any pass stays visible.
static int check_pass_sizes(const char* op, const AttnArgs& a, const AttnWorkspace& w, size_t need_one_group) {
  if (a.ws == nullptr || a.ws_bytes < w.bytes)
    return fail(FMB_ERR_WORKSPACE, "%s: workspace too small (%zu bytes given; a pass over one kv-head group needs %zu)",
                op, a.ws_bytes, need_one_group);
  if ((int64_t)w.nsub * w.cap >= (int64_t)0xffffffffll)
    return fail(FMB_ERR_BAD_ARG, "%s: too many partial slots in one pass; give a smaller workspace", op);
  return FMB_OK;
}

// ------------------------------------------------------------------ rows handed over by the pattern builder
struct RowsTicket {
  const uint32_t* rows; int64_t total_q; int heads, topk; bool armed;
};
static thread_local RowsTicket g_rows = {nullptr, 0, 0, 0, false};

void attn_rows_offer(const uint32_t* row_slots, int64_t total_q, int heads, int topk) {
  g_rows = RowsTicket{row_slots, total_q, heads, topk, row_slots != nullptr && topk > 0};
}
// Consumes the ticket; true if this call (matching geometry; one pass over all heads, or a single
// sequence, whose heads lie one after the other in `indices`) runs on it: slots are positions in
// `indices` (less the pass's first), the row lists are the builder's.
static bool take_rows(const AttnArgs& a, AttnWorkspace& w) {
  const RowsTicket t = g_rows;
  g_rows.armed = false;
  w.fixed_k = 0;
  if (!t.armed || t.total_q != a.total_q || t.heads != a.heads || (w.nh < a.heads && a.batch != 1) ||
      (int64_t)t.total_q * t.heads * t.topk != a.n_indices || a.n_indices >= (int64_t)0xffffffffll)
    return false;
  w.fixed_k = t.topk;
  w.row_pos = const_cast<uint32_t*>(t.rows);
  w.slot_base = nullptr;
  return true;
}

// ------------------------------------------------------------------ status word mirrored for the host
static thread_local int* g_mirror = nullptr;
void attn_status_mirror(int* mirror) { g_mirror = mirror; }
static int* take_mirror() {
  int* m = g_mirror;
  g_mirror = nullptr;
  return m;
}

int launch_attn_fwd(const AttnArgs& a, int engine, cudaStream_t s) {
  AttnWorkspace w = carve_attn_workspace(a.ws, a.ws_bytes, a, 2, true, 0);
  w.mirror = take_mirror();
  int rc = check_pass_sizes("attn_fwd", a, w, w.bytes);
  if (rc) return rc;
  const bool rows_given = take_rows(a, w);
  FMB_CUDA(cudaMemsetAsync(w.status, 0, 512, s));
  for (int h0 = 0; h0 < a.heads; h0 += w.nh) {
    const PassParams ps = make_pass(a, w, h0, min(w.nh, a.heads - h0));
    if (!rows_given && (rc = build_row_lists(a, w, ps, s))) return rc;
    prof_begin(0, s);
    if (engine == 1 && tc_supported(a, false)) rc = launch_fwd_main_tc(a, w, ps, s);
    else if (engine == 1 && tc_wide_supported(a, false)) rc = launch_fwd_main_tc_wide(a, w, ps, s);
    else rc = launch_fwd_main_simt(a, w, ps, s);
    prof_end(0, s);
    if (rc) return rc;
    prof_begin(4, s);
    rc = launch_fwd_combine(a, w, ps, s);
    prof_end(4, s);
    if (rc) return rc;
  }
  return FMB_OK;
}

// ------------------------------------------------------------------ lists handed from forward to backward
struct ListsTicket {
  const void* ws; int64_t total_q, n_indices; int heads, batch, ncol, chunk; bool armed;
};
static thread_local ListsTicket g_ticket = {nullptr, 0, 0, 0, 0, 0, 0, false};

size_t attn_lists_bytes(const AttnArgs& a) {
  return carve_attn_workspace(nullptr, 0, a, 2, false, a.heads).lists_bytes;
}
int attn_lists_save(const AttnArgs& a, void* dst, size_t dst_bytes, cudaStream_t s) {
  const AttnWorkspace w = carve_attn_workspace(a.ws, a.ws_bytes, a, 2, true, 0);
  if (a.ws == nullptr || a.ws_bytes < w.bytes || w.nh < a.heads) return 1;
  if (dst == nullptr || dst_bytes < w.lists_bytes)
    return fail(FMB_ERR_WORKSPACE, "attn_lists_save: buffer too small (%zu bytes given, %zu needed)", dst_bytes,
                w.lists_bytes);
  FMB_CUDA(cudaMemcpyAsync(dst, static_cast<const char*>(a.ws) + w.lists_off, w.lists_bytes,
                           cudaMemcpyDeviceToDevice, s));
  return FMB_OK;
}
int attn_lists_load(const AttnArgs& a, const void* src, size_t src_bytes, cudaStream_t s) {
  const AttnWorkspace w = carve_attn_workspace(a.ws, a.ws_bytes, a, 2, false, 0);
  if (a.ws == nullptr || a.ws_bytes < w.bytes || w.nh < a.heads) return 1;
  if (src == nullptr || src_bytes < w.lists_bytes)
    return fail(FMB_ERR_WORKSPACE, "attn_lists_load: buffer too small (%zu bytes given, %zu needed)", src_bytes,
                w.lists_bytes);
  FMB_CUDA(cudaMemcpyAsync(static_cast<char*>(a.ws) + w.lists_off, src, w.lists_bytes, cudaMemcpyDeviceToDevice, s));
  g_ticket = ListsTicket{a.ws, a.total_q, a.n_indices, a.heads, a.batch, a.ncol, a.chunk, true};
  return FMB_OK;
}

int launch_attn_bwd(const AttnArgs& a, int engine, cudaStream_t s) {
  AttnWorkspace w = carve_attn_workspace(a.ws, a.ws_bytes, a, 2, false, 0);
  w.mirror = take_mirror();
  int rc = check_pass_sizes("attn_bwd", a, w, w.bytes);
  if (rc) return rc;
  // lists loaded into this very workspace for this very problem, one pass: no build of our own
  const bool lists_given = g_ticket.armed && g_ticket.ws == a.ws && g_ticket.total_q == a.total_q &&
                           g_ticket.n_indices == a.n_indices && g_ticket.heads == a.heads &&
                           g_ticket.batch == a.batch && g_ticket.ncol == a.ncol && g_ticket.chunk == a.chunk &&
                           w.nh >= a.heads;
  g_ticket.armed = false;
  const bool rows_given = take_rows(a, w);
  FMB_CUDA(cudaMemsetAsync(w.status, 0, 512, s));
  prof_begin(7, s);
  rc = launch_dot_do_o(a, s);
  prof_end(7, s);
  if (rc) return rc;
  for (int h0 = 0; h0 < a.heads; h0 += w.nh) {
    const PassParams ps = make_pass(a, w, h0, min(w.nh, a.heads - h0));
    if (!lists_given && !rows_given && (rc = build_row_lists(a, w, ps, s))) return rc;
    prof_begin(1, s);
    if (engine == 1 && tc_supported(a, true)) rc = launch_bwd_main_tc(a, w, ps, s);
    else if (engine == 1 && tc_wide_supported(a, true)) rc = launch_bwd_main_tc_wide(a, w, ps, s);
    else rc = launch_bwd_main_simt(a, w, ps, s);
    prof_end(1, s);
    if (rc) return rc;
    prof_begin(5, s);
    rc = launch_bwd_combine(a, w, ps, s);
    prof_end(5, s);
    if (rc) return rc;
  }
  return FMB_OK;
}

}  // namespace fmb
