// Stage G: fused gating.  scores = Q . centroid^T (fp32, unscaled) -> causal chunk rule ->
// per-row top-k, in one kernel; the score matrix never reaches HBM.
//
// Replaces csrc/flash_topk/src/flash_topk_kernel.h:31-357 of the reference (one thread per
// row doing a serial insertion over every score of every tile).  Here a CTA owns 128 query
// rows of one (sequence, head); for each tile of 128 centroids the score tile is produced
// into shared memory and then a WARP owns a row: its 32 lanes test 32 scores at once
// against the row's current k-th best (one compare + one ballot per 32 scores), and only
// the rare survivors are inserted into the sorted list, which lives distributed across the
// lanes (lane j holds rank j and rank j+32).  Ordering rule = the reference's: descending
// score, and on equal scores the higher chunk id first
// (csrc/flash_topk/src/flash_topk_kernel.h:261-285).
#include "fmb_common.cuh"

namespace fmb {

constexpr int kGateM = 128;          // query rows per CTA
constexpr int kGateN = 128;          // centroids per score tile
constexpr int kGateThreads = 256;
constexpr int kGateDSlab = 128;      // head-dim slab staged in shared memory
constexpr int kGateSStride = kGateN + 4;

struct GateParams {
  const void* q; int64_t q_rs, q_hs;
  const void* km;
  const int32_t *cu_q, *cu_k, *cu_km;
  int32_t* topk_idx; float* topk_val; int64_t t_rs, t_hs;
  int heads, heads_k, d, topk, chunk, causal;
};

// true if entry a ranks ahead of entry b
__device__ __forceinline__ bool ranks_ahead(float va, int ia, float vb, int ib) {
  return va > vb || (va == vb && ia > ib);
}

// Sorted list of one row, distributed over the warp: lane j holds ranks j and j+32.
struct RowList {
  float v0, v1;
  int i0, i1;
};

template <bool kTwoHalves>
__device__ __forceinline__ void list_insert(RowList& L, float v, int n, int topk, int lane) {
  const unsigned full = 0xffffffffu;
  const unsigned m0 = __ballot_sync(full, ranks_ahead(L.v0, L.i0, v, n));
  int pos = __popc(m0);
  if (kTwoHalves) pos += __popc(__ballot_sync(full, ranks_ahead(L.v1, L.i1, v, n)));
  // shift the tail down by one rank and drop the new entry in at `pos`
  const float pv0 = __shfl_up_sync(full, L.v0, 1);
  const int pi0 = __shfl_up_sync(full, L.i0, 1);
  if (kTwoHalves) {
    const float cv = __shfl_sync(full, L.v0, 31);
    const int ci = __shfl_sync(full, L.i0, 31);
    float pv1 = __shfl_up_sync(full, L.v1, 1);
    int pi1 = __shfl_up_sync(full, L.i1, 1);
    if (lane == 0) { pv1 = cv; pi1 = ci; }
    const int r1 = lane + 32;
    if (r1 == pos) { L.v1 = v; L.i1 = n; }
    else if (r1 > pos) { L.v1 = pv1; L.i1 = pi1; }
    if (r1 >= topk) { L.v1 = -CUDART_INF_F; L.i1 = -1; }
  }
  if (lane == pos) { L.v0 = v; L.i0 = n; }
  else if (lane > pos) { L.v0 = pv0; L.i0 = pi0; }
  if (lane >= topk) { L.v0 = -CUDART_INF_F; L.i0 = -1; }
}

// Offer 32 scores (one per lane) of one row to its list.
template <bool kTwoHalves>
__device__ __forceinline__ void list_offer(RowList& L, float v, int n, bool eligible, int topk, int lane) {
  const unsigned full = 0xffffffffu;
  const int kl = (topk - 1) & 31;
  float tv = __shfl_sync(full, (kTwoHalves && topk > 32) ? L.v1 : L.v0, kl);
  int ti = __shfl_sync(full, (kTwoHalves && topk > 32) ? L.i1 : L.i0, kl);
  bool cand = eligible && v > -CUDART_INF_F && ranks_ahead(v, n, tv, ti);
  unsigned m = __ballot_sync(full, cand);
  while (m) {
    const int src = __ffs(m) - 1;
    const float nv = __shfl_sync(full, v, src);
    const int nn = __shfl_sync(full, n, src);
    list_insert<kTwoHalves>(L, nv, nn, topk, lane);
    tv = __shfl_sync(full, (kTwoHalves && topk > 32) ? L.v1 : L.v0, kl);
    ti = __shfl_sync(full, (kTwoHalves && topk > 32) ? L.i1 : L.i0, kl);
    cand = cand && lane != src && ranks_ahead(v, n, tv, ti);
    m = __ballot_sync(full, cand);
  }
}

// CUDA-core score tile: S[128][128] = Qt^T . Kt over one head-dim slab (operands transposed
// in shared memory so that each thread reads 16 contiguous bytes per operand per step).
template <typename T>
__device__ __forceinline__ void score_tile_fma(const T* sQt, const T* sKt, int dlen, float (&acc)[8][8]) {
  const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
  for (int dd = 0; dd < dlen; ++dd) {
    float a[8], b[8];
    unpack8<T>(*reinterpret_cast<const uint4*>(sQt + dd * kGateM + ty * 8), a);
    unpack8<T>(*reinterpret_cast<const uint4*>(sKt + dd * kGateN + tx * 8), b);
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
  }
}

// stage rows [r0, r0+128) x dims [d0, d0+dlen) of a (rows, stride) matrix, transposed
template <typename T>
__device__ __forceinline__ void stage_transposed(T* dst, const T* src, int64_t row_stride, int rows_valid,
                                                 int d0, int dlen) {
  // lane -> row (conflict-free transposed stores), loop over 16-byte column groups
  const int ngroups = dlen / 8;
  for (int e = threadIdx.x; e < 128 * ngroups; e += blockDim.x) {
    const int r = e & 127, g = e >> 7;
    uint4 u = make_uint4(0, 0, 0, 0);
    if (r < rows_valid) u = ldg_nc_16(src + (int64_t)r * row_stride + d0 + g * 8);
    const T* x = reinterpret_cast<const T*>(&u);
#pragma unroll
    for (int i = 0; i < 8; ++i) dst[(g * 8 + i) * 128 + r] = x[i];
  }
}

template <typename T, bool kTwoHalves>
__global__ void __launch_bounds__(kGateThreads) gate_topk_kernel(GateParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* sQt = reinterpret_cast<T*>(smem_raw);                         // [128 dd][128 rows]
  T* sKt = sQt + kGateDSlab * kGateM;                              // [128 dd][128 centroids]
  float* sS = reinterpret_cast<float*>(sKt + kGateDSlab * kGateN); // [128][132]
  float* sTV = sS + kGateM * kGateSStride;                         // [128][topk]
  int* sTI = reinterpret_cast<int*>(sTV + kGateM * p.topk);        // [128][topk]

  const int mt = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int q0 = p.cu_q[b], len_q = p.cu_q[b + 1] - q0;
  const int len_k = p.cu_k[b + 1] - p.cu_k[b];
  const int km0 = p.cu_km[b], nchunks = p.cu_km[b + 1] - km0;
  const int r0 = mt * kGateM;
  if (r0 >= len_q) return;
  const int rows = min(kGateM, len_q - r0);
  const int hk = h / (p.heads / p.heads_k);
  const int shift = len_k - len_q;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int topk = p.topk;

  // initial lists: empty, or the row's own chunk pinned at rank 0 under the causal rule
  for (int e = threadIdx.x; e < kGateM * topk; e += blockDim.x) {
    const int r = e / topk, j = e - r * topk;
    float v = -CUDART_INF_F;
    int i = -1;
    const int pos = r0 + r + shift;
    if (p.causal && j == 0 && r < rows && pos >= 0 && nchunks > 0) { v = CUDART_INF_F; i = pos / p.chunk; }
    sTV[e] = v;
    sTI[e] = i;
  }

  // centroids that any row of this CTA may still select
  int n_end = nchunks;
  if (p.causal) {
    const int pmax = r0 + rows - 1 + shift;
    n_end = pmax < 0 ? 0 : min(nchunks, pmax / p.chunk);   // candidate n: (n+1)*chunk <= p
  }
  const T* qbase = static_cast<const T*>(p.q) + (int64_t)(q0 + r0) * p.q_rs + (int64_t)h * p.q_hs;
  const T* kmbase = static_cast<const T*>(p.km) + ((int64_t)km0 * p.heads_k + hk) * p.d;
  const int64_t km_rs = (int64_t)p.heads_k * p.d;
  const bool single_slab = p.d <= kGateDSlab;
  if (single_slab && n_end > 0) stage_transposed<T>(sQt, qbase, p.q_rs, rows, 0, p.d);
  __syncthreads();

  for (int n0 = 0; n0 < n_end; n0 += kGateN) {
    const int ncols = min(kGateN, n_end - n0);
    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;
    for (int d0 = 0; d0 < p.d; d0 += kGateDSlab) {
      const int dlen = min(kGateDSlab, p.d - d0);
      if (!single_slab) stage_transposed<T>(sQt, qbase, p.q_rs, rows, d0, dlen);
      stage_transposed<T>(sKt, kmbase + (int64_t)n0 * km_rs, km_rs, ncols, d0, dlen);
      __syncthreads();
      score_tile_fma<T>(sQt, sKt, dlen, acc);
      __syncthreads();
    }
    {
      const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float* dst = sS + (ty * 8 + i) * kGateSStride + tx * 8;
        *reinterpret_cast<float4*>(dst) = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
        *reinterpret_cast<float4*>(dst + 4) = make_float4(acc[i][4], acc[i][5], acc[i][6], acc[i][7]);
      }
    }
    __syncthreads();
    // selection: warp w owns rows w*16 .. w*16+15
    for (int rr = 0; rr < 16; ++rr) {
      const int r = warp * 16 + rr;
      if (r >= rows) break;
      const int pos = r0 + r + shift;
      RowList L;
      L.v0 = lane < topk ? sTV[r * topk + lane] : -CUDART_INF_F;
      L.i0 = lane < topk ? sTI[r * topk + lane] : -1;
      L.v1 = -CUDART_INF_F; L.i1 = -1;
      if (kTwoHalves && lane + 32 < topk) { L.v1 = sTV[r * topk + lane + 32]; L.i1 = sTI[r * topk + lane + 32]; }
      for (int g = 0; g < kGateN; g += 32) {
        if (g >= ncols) break;
        const int n = n0 + g + lane;
        const float v = sS[r * kGateSStride + g + lane];
        const bool ok = (g + lane < ncols) && (!p.causal || ((n + 1) * p.chunk - 1 < pos));
        list_offer<kTwoHalves>(L, v, n, ok, topk, lane);
      }
      if (lane < topk) { sTV[r * topk + lane] = L.v0; sTI[r * topk + lane] = L.i0; }
      if (kTwoHalves && lane + 32 < topk) { sTV[r * topk + lane + 32] = L.v1; sTI[r * topk + lane + 32] = L.i1; }
    }
    __syncthreads();
  }
  __syncthreads();
  // write the lists
  for (int e = threadIdx.x; e < rows * topk; e += blockDim.x) {
    const int r = e / topk, j = e - r * topk;
    const int64_t o = (int64_t)(q0 + r0 + r) * p.t_rs + (int64_t)h * p.t_hs + j;
    p.topk_idx[o] = sTI[e];
    if (p.topk_val) p.topk_val[o] = sTV[e];
  }
}

template <typename T>
static int gate_dispatch(const GateParams& p, int batch, int max_q, cudaStream_t s) {
  const size_t smem = (size_t)kGateDSlab * (kGateM + kGateN) * sizeof(T) +
                      (size_t)kGateM * kGateSStride * sizeof(float) + (size_t)kGateM * p.topk * 8;
  dim3 grid(ceil_div(max_q, kGateM), p.heads, batch);
  if (p.topk > 32) {
    auto kern = gate_topk_kernel<T, true>;
    FMB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<grid, kGateThreads, smem, s>>>(p);
  } else {
    auto kern = gate_topk_kernel<T, false>;
    FMB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<grid, kGateThreads, smem, s>>>(p);
  }
  FMB_LAUNCH_CHECK("gate_topk_kernel");
  return FMB_OK;
}

int launch_gate_topk(const GateArgs& a, cudaStream_t s) {
  if (a.batch == 0 || a.max_q == 0 || a.heads == 0) return FMB_OK;
  GateParams p;
  p.q = a.q; p.q_rs = a.q_rs; p.q_hs = a.q_hs; p.km = a.km;
  p.cu_q = a.cu_q; p.cu_k = a.cu_k; p.cu_km = a.cu_km;
  p.topk_idx = a.topk_idx; p.topk_val = a.topk_val; p.t_rs = a.t_rs; p.t_hs = a.t_hs;
  p.heads = a.heads; p.heads_k = a.heads_k; p.d = a.d; p.topk = a.topk; p.chunk = a.chunk; p.causal = a.causal;
  prof_begin(2, s);
  const int rc = a.dtype == FMB_BF16 ? gate_dispatch<__nv_bfloat16>(p, a.batch, a.max_q, s)
                                     : gate_dispatch<__half>(p, a.batch, a.max_q, s);
  prof_end(2, s);
  return rc;
}

}  // namespace fmb
