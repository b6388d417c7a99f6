// Stage G: fused gating.  scores = Q . centroid^T (fp32, unscaled) -> causal chunk rule ->
// per-row top-k, in one kernel; the score matrix never reaches HBM.
//
// Replaces csrc/flash_topk/src/flash_topk_kernel.h:31-357 of the reference (one thread per
// row doing a serial insertion over every score of every tile).  Two kernels:
//   * gate_topk_tc_kernel (head dims 64 / 128, top-k <= 32): the score tile is a tcgen05 MMA with
//     the accumulator in TMEM; TMEM lane = query row, so a thread reads its row's scores straight
//     from TMEM and keeps the row's list in registers as 64-bit ordered keys;
//   * gate_topk_kernel (other shapes, and the cross-check of the first): CUDA-core score tile in
//     shared memory, a warp per row, the list distributed over the lanes.
// Ordering rule = the reference's: descending score, and on equal scores the higher chunk id
// first (csrc/flash_topk/src/flash_topk_kernel.h:261-285).
#include "fmb_common.cuh"
#include "fmb_tc.cuh"

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

// One score tile (rows x ncols in sS) offered to the rows' lists; warp w owns rows w*R..,
// R = 128 / number of warps.
template <bool kTwoHalves>
__device__ __forceinline__ void select_tile(const float* sS, float* sTV, int* sTI, int r0, int rows, int n0,
                                            int ncols, int shift, int topk, int chunk, int causal) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rows_per_warp = kGateM / (blockDim.x >> 5);
  for (int rr = 0; rr < rows_per_warp; ++rr) {
    const int r = warp * rows_per_warp + rr;
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
      const bool ok = (g + lane < ncols) && (!causal || ((n + 1) * chunk - 1 < pos));
      list_offer<kTwoHalves>(L, v, n, ok, topk, lane);
    }
    if (lane < topk) { sTV[r * topk + lane] = L.v0; sTI[r * topk + lane] = L.i0; }
    if (kTwoHalves && lane + 32 < topk) { sTV[r * topk + lane + 32] = L.v1; sTI[r * topk + lane + 32] = L.i1; }
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

  // late row tiles see the most candidate chunks under a causal mask: they are scheduled first
  const int mt = gridDim.x - 1 - blockIdx.x, h = blockIdx.y, b = blockIdx.z;
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
    select_tile<kTwoHalves>(sS, sTV, sTI, r0, rows, n0, ncols, shift, topk, p.chunk, p.causal);
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

// ---------------------------------------------------------------------------------------
// Tensor-core variant (head_dim 64, 128 or 256, top-k <= 32).  The score tile is a tcgen05 MMA
// with the accumulator in TMEM; TMEM lane = query row, so thread t reads row t's scores
// straight from TMEM (no shared-memory staging of scores) and keeps that row's top-k list
// in registers: val[] = order-preserving 32-bit images of the fp32 scores, descending, and
// idx[] = their chunk ids.  A thread meets its candidates in ascending chunk order, so "the
// higher chunk id ranks first on equal scores" (the reference's rule) is simply: a candidate
// goes ahead of every entry it is greater than OR EQUAL to, one 32-bit compare per slot; the
// values move with a min/max pair, the ids with two selects.  Slots that must never be
// displaced (the row's own chunk, and the unused head of a list shorter than KMAX) hold the image
// 0xffffffff, which no score that passes the "> -inf" test can reach; the empty slot holds the
// image of -inf.  Q is staged once; centroid tiles and TMEM accumulators are double-buffered so
// the MMA of tile n+1 runs under the selection of tile n; two CTAs share an SM.  All waits are
// bounded (status word g_gate_status).
// ---------------------------------------------------------------------------------------
__device__ int g_gate_status = 0;

__device__ __forceinline__ uint32_t score_to_ordered(float v) {
  const uint32_t b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float ordered_to_score(uint32_t o) {
  return __uint_as_float((o & 0x80000000u) ? (o & 0x7fffffffu) : ~o);
}

// NQ threads share a row (TMEM lane): warps w, w+4, w+8, ... may all read lane quarter w%4, so
// each of them scans 128/NQ of a tile's columns into a private list; the NQ lists of a row are
// merged once at the end.  More warps per row hide the latency of the (divergent) insertions.
template <typename T, int D, int KMAX, int NQ>
__global__ void __launch_bounds__(128 * NQ) gate_topk_tc_kernel(GateParams p) {
  using namespace tc;
  constexpr uint32_t kBlock = 128 * 128;       // bytes between 64-element blocks of a 128-row tile
  constexpr uint32_t kTile = 128 * D * 2;
  extern __shared__ unsigned char smem_raw[];
  __shared__ uint64_t bar[2];
  __shared__ uint32_t tmem_base_s;
  // the two threads of a row tell each other the eight best images they hold (NQ == 2)
  __shared__ uint32_t sX[NQ == 2 ? 2 : 1][NQ == 2 ? 8 : 1][NQ == 2 ? 128 : 1];
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  unsigned char* sQ = smem;
  unsigned char* sKM = sQ + kTile;             // two buffers

  // late row tiles see the most candidate chunks under a causal mask: they are scheduled first
  const int mt = gridDim.x - 1 - blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int q0 = p.cu_q[b], len_q = p.cu_q[b + 1] - q0;
  const int len_k = p.cu_k[b + 1] - p.cu_k[b];
  const int km0 = p.cu_km[b], nchunks = p.cu_km[b + 1] - km0;
  const int r0 = mt * kGateM;
  if (r0 >= len_q) return;
  const int rows = min(kGateM, len_q - r0);
  const int hk = h / (p.heads / p.heads_k);
  const int shift = len_k - len_q;
  const int tid = threadIdx.x, warp = tid >> 5;
  const int lt = tid & 127, qd = tid >> 7;     // row, and which share of the columns
  const int topk = p.topk;

  // this thread's row: list of KMAX keys, descending; the first KMAX-topk are sentinels
  const int pos = r0 + lt + shift;
  const bool row_ok = lt < rows;
  int nlim = nchunks;                          // candidate chunks of the row: n < nlim
  if (p.causal) nlim = pos < 0 ? 0 : min(nchunks, pos / p.chunk);
  if (!row_ok) nlim = 0;
  constexpr uint32_t kFixed = 0xffffffffu;     // image of a slot no candidate may displace
  constexpr uint32_t kEmptyVal = 0x007fffffu;  // image of -inf: the empty slot
  constexpr int kBlockedId = -2;               // id of the unused head of a list shorter than KMAX
  const bool own = p.causal && row_ok && pos >= 0 && nchunks > 0 && qd == 0;
  uint32_t val[KMAX];
  int idx[KMAX];
#pragma unroll
  for (int j = 0; j < KMAX; ++j) {   // static indices only: the list must stay in registers
    const bool blocked = j < KMAX - topk, is_own = (j == KMAX - topk) && own;
    val[j] = (blocked || is_own) ? kFixed : kEmptyVal;
    idx[j] = blocked ? kBlockedId : (is_own ? pos / p.chunk : -1);
  }
  // val[j] for a j that depends on the run-time top-k (selects: the list must stay in registers)
  auto val_at = [&](int j) {
    if (topk == KMAX) return val[j < KMAX ? j : 0];   // (callers pass compile-time j: no selects in the common case)
    uint32_t x = val[0];
#pragma unroll
    for (int y = 1; y < KMAX; ++y) x = (j == y) ? val[y] : x;
    return x;
  };
  // candidate (image ox, chunk n) into the list; every entry already there has a lower chunk id
  auto insert = [&](uint32_t ox, int n) {
    bool ge[KMAX];
#pragma unroll
    for (int y = 0; y < KMAX; ++y) ge[y] = ox >= val[y];
#pragma unroll
    for (int y = KMAX - 1; y > 0; --y) {
      idx[y] = ge[y - 1] ? idx[y - 1] : (ge[y] ? n : idx[y]);
      val[y] = min(val[y - 1], max(val[y], ox));
    }
    idx[0] = ge[0] ? n : idx[0];
    val[0] = max(val[0], ox);
  };

  int n_end = nchunks;
  if (p.causal) {
    const int pmax = r0 + rows - 1 + shift;
    n_end = pmax < 0 ? 0 : min(nchunks, pmax / p.chunk);
  }
  const int ntiles = (n_end + kGateN - 1) / kGateN;
  if (ntiles > 0) {   // CTA-uniform
    if (warp == 0) tmem_alloc(&tmem_base_s, 256);
    if (tid == 0) {
      mbar_init(&bar[0], 1);
      mbar_init(&bar[1], 1);
      mbar_fence_init();
    }
    const T* qbase = static_cast<const T*>(p.q) + (int64_t)(q0 + r0) * p.q_rs + (int64_t)h * p.q_hs;
    const T* kmbase = static_cast<const T*>(p.km) + ((int64_t)km0 * p.heads_k + hk) * p.d;
    const int64_t km_rs = (int64_t)p.heads_k * p.d;
    // The Q tile and the first two centroid tiles are copied with cp.async (no registers, all in
    // flight at once); inside the loop the tile two steps ahead is copied while this step's scores
    // are examined, and its MMA is issued at the step's end, so that neither a copy nor an MMA is
    // waited for in the steady state.
    auto stage_km = [&](int t) {
      const int n1 = t * kGateN, nc = min(kGateN, n_end - n1);
      dense_cp_async<T, D / 8, kGateN, 128 * NQ>(tid, sKM + (t & 1) * kTile, kBlock, kmbase + (int64_t)n1 * km_rs, km_rs, nc);
    };
    dense_cp_async<T, D / 8, kGateM, 128 * NQ>(tid, sQ, kBlock, qbase, p.q_rs, rows);
    stage_km(0);
    if (ntiles > 1) stage_km(1);
    cp_async_wait_all();
    fence_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = tmem_base_s;
    const uint32_t sQ_a = smem_u32(sQ), sKM_a = smem_u32(sKM);
    constexpr uint32_t idesc = make_idesc(FmtOf<T>::v, 128, 128, 0, 0);
    auto issue = [&](int buf) {
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        const uint32_t o = (ks >> 2) * kBlock + (ks & 3) * 32;
        umma_ss(tmem_base + buf * 128, make_desc_sw128(sQ_a + o, 16, 1024),
                make_desc_sw128(sKM_a + buf * kTile + o, 16, 1024), idesc, ks > 0);
      }
      umma_commit(&bar[buf]);
    };
    if (tid == 0) {
      issue(0);
      if (ntiles > 1) issue(1);
    }
    uint32_t phases = 0;   // bit b = parity to wait for on bar[b]
    float floor_thr_row = -CUDART_INF_F;   // what the k-th best of the row is known to reach
    for (int t = 0; t < ntiles; ++t) {
      const int buf = t & 1;
      const int n0 = t * kGateN;
      const bool ok = mbar_wait(&bar[buf], (phases >> buf) & 1u, &g_gate_status, 1);
      phases ^= 1u << buf;
      if (!__syncthreads_and(ok)) break;
      tc_fence_after_sync();
      // MMA t has completed: its centroid buffer takes the tile two steps ahead
      const bool ahead = t + 2 < ntiles;
      if (ahead) stage_km(t + 2);
      constexpr int kCols = kGateN / NQ;        // columns of a tile examined by this thread
      const uint32_t taddr = tmem_base + buf * 128 + qd * kCols + ((uint32_t)((warp & 3) * 32) << 16);
      // 16 scores per step; the next 16 are fetched while these are examined.  A step first marks,
      // without branching, the scores that reach the row's current k-th best (a superset of the
      // scores that enter the list: the threshold is not updated inside the step).  Then every lane
      // works through ITS OWN marked scores, so the (long) insertion code runs max-over-lanes of
      // the marked counts times per step instead of once per position that any lane marked.
      const bool tail = n0 + kGateN > nlim;     // this tile crosses the row's candidate limit
      // A list that is still empty lets every score in.  For the first tile of a row the thread
      // therefore first finds a floor for its k-th best: the maxima of its groups of 4 scores are
      // different candidates, so their k-th largest cannot exceed the k-th largest score (lists of
      // 8 with 16 or 32 groups, lists of 16 with 32 groups).  Only the scores that reach the floor
      // are then looked at one by one, a dozen instead of some forty while a list of 8 fills (the
      // scores are read from TMEM a second time for it).
      float floor_thr = floor_thr_row;
      constexpr int kGroups = kCols / 4;
      constexpr bool kColdFloor = (KMAX == 8 && kGroups == 16) || (KMAX == 16 && kGroups == 32);
      if (kColdFloor && t == 0) {
        float gm[kGroups];
#pragma unroll
        for (int i = 0; i < kCols / 16; ++i) {
          float w[16];
          tmem_ld16(taddr + i * 16, w);
          tmem_ld_wait();
          if (tail) {
            const int left = nlim - (n0 + qd * kCols + i * 16);
#pragma unroll
            for (int j = 0; j < 16; ++j) w[j] = j < left ? w[j] : -CUDART_INF_F;
          }
#pragma unroll
          for (int g4 = 0; g4 < 4; ++g4)
            gm[i * 4 + g4] = fmaxf(fmaxf(fmaxf(w[g4 * 4], w[g4 * 4 + 1]), fmaxf(w[g4 * 4 + 2], w[g4 * 4 + 3])),
                                   -CUDART_INF_F);   // (a group of NaNs counts as -inf: fmaxf drops NaN operands)
        }
        // descending sorting networks on registers: 8 values in 19 compare-exchanges; 16 values as
        // two sorted eights and a bitonic merge
#define FMB_CE(x, i, j) { const float hi_ = fmaxf(x[i], x[j]), lo_ = fminf(x[i], x[j]); x[i] = hi_; x[j] = lo_; }
        auto sort8 = [](float* x) {
          FMB_CE(x, 0, 1) FMB_CE(x, 2, 3) FMB_CE(x, 4, 5) FMB_CE(x, 6, 7)
          FMB_CE(x, 0, 2) FMB_CE(x, 1, 3) FMB_CE(x, 4, 6) FMB_CE(x, 5, 7)
          FMB_CE(x, 1, 2) FMB_CE(x, 5, 6) FMB_CE(x, 0, 4) FMB_CE(x, 3, 7)
          FMB_CE(x, 1, 5) FMB_CE(x, 2, 6)
          FMB_CE(x, 1, 4) FMB_CE(x, 3, 6)
          FMB_CE(x, 2, 4) FMB_CE(x, 3, 5)
          FMB_CE(x, 3, 4)
        };
        auto sort16 = [&](float* x) {
          sort8(x);
          sort8(x + 8);
#pragma unroll
          for (int i = 0; i < 8; ++i) FMB_CE(x, i, 15 - i)
#pragma unroll
          for (int h8 = 0; h8 < 16; h8 += 8) {
#pragma unroll
            for (int i = 0; i < 4; ++i) FMB_CE(x, h8 + i, h8 + i + 4)
#pragma unroll
            for (int i = 0; i < 8; i += 4) { FMB_CE(x, h8 + i, h8 + i + 2) FMB_CE(x, h8 + i + 1, h8 + i + 3) }
#pragma unroll
            for (int i = 0; i < 8; i += 2) FMB_CE(x, h8 + i, h8 + i + 1)
          }
        };
        float kth = CUDART_INF_F;
        if constexpr (KMAX == 8) {
          // 8th largest of the 16 group maxima: both halves sorted, then min over i of max(a[i], b[7 - i]);
          // those eight maxima, sorted, are also what the row's other thread needs
          sort8(gm);
          sort8(gm + 8);
          float c8[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) c8[i] = fmaxf(gm[i], gm[15 - i]);
          if constexpr (NQ == 2) {
            // the 8th largest of the 32 groups of the whole tile is the floor for both threads
            sort8(c8);
#pragma unroll
            for (int i = 0; i < 8; ++i) sX[qd][i][lt] = __float_as_uint(c8[i]);
            bar_sync(1 + (warp & 3), 64);         // warps w and w + 4 hold the same rows
#pragma unroll
            for (int i = 0; i < 8; ++i) kth = fminf(kth, fmaxf(c8[i], __uint_as_float(sX[qd ^ 1][7 - i][lt])));
            bar_sync(1 + (warp & 3), 64);         // both have read before the buffer is written again
          } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) kth = fminf(kth, c8[i]);
          }
        } else {
          // 16th largest of the 32 group maxima
          sort16(gm);
          sort16(gm + 16);
#pragma unroll
          for (int i = 0; i < 16; ++i) kth = fminf(kth, fmaxf(gm[i], gm[31 - i]));
        }
#undef FMB_CE
        floor_thr = kth;
        floor_thr_row = kth;
      }
      float v[2][16];
      tmem_ld16(taddr, v[0]);
#pragma unroll 1
      for (int i = 0; i < kCols / 16; i += 2) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          tmem_ld_wait();
          if (i + half + 1 < kCols / 16) tmem_ld16(taddr + (i + half + 1) * 16, v[half ^ 1]);
          const int nb = n0 + qd * kCols + (i + half) * 16;
          const float thr = val[KMAX - 1] == kFixed ? CUDART_INF_F : fmaxf(floor_thr, ordered_to_score(val[KMAX - 1]));
          uint32_t m = 0;
#pragma unroll
          for (int j = 0; j < 16; ++j) m |= (v[half][j] >= thr) ? (1u << j) : 0u;
          if (tail) {
            const int left = nlim - nb;           // candidates are n < nlim
            m = left <= 0 ? 0u : (left >= 16 ? m : (m & ((1u << left) - 1u)));
          }
          while (__any_sync(0xffffffffu, m != 0u)) {
            if (m != 0u) {
              const int j = __ffs(m) - 1;
              m &= m - 1u;
              // v[half][j] for a run-time j: a 4-level select tree (the array must stay in registers)
              float a8[8], a4[4];
#pragma unroll
              for (int e = 0; e < 8; ++e) a8[e] = (j & 8) ? v[half][8 + e] : v[half][e];
#pragma unroll
              for (int e = 0; e < 4; ++e) a4[e] = (j & 4) ? a8[4 + e] : a8[e];
              const float a2a = (j & 2) ? a4[2] : a4[0], a2b = (j & 2) ? a4[3] : a4[1];
              const float x = (j & 1) ? a2b : a2a;
              const uint32_t ox = score_to_ordered(x);
              if (x > -CUDART_INF_F && ox >= val[KMAX - 1]) insert(ox, nb + j);
            }
          }
        }
      }
      if (ahead) {             // CTA-uniform
        if (NQ == 2 && KMAX == 8) {   // this thread's list without the slots of a list shorter than KMAX
#pragma unroll
          for (int j = 0; j < 8; ++j) sX[qd][j][lt] = (j + (KMAX - topk) < KMAX) ? val_at(j + (KMAX - topk)) : kEmptyVal;
        }
        cp_async_wait_all();
        fence_async_smem();
        tc_fence_before_sync();
        __syncthreads();       // tile t + 2 staged; every thread has finished reading TMEM buffer buf
        if (tid == 0) {
          tc_fence_after_sync();
          issue(buf);
        }
        if (NQ == 2 && KMAX == 8) {
          // The k-th best of the row so far is at least the k-th largest of the two threads' lists
          // together (both sorted: min over i of max(a[i], b[k - 1 - i])): a floor for the next tiles
          // that roughly halves the scores each thread still has to look at one by one.  (The
          // barrier at the top of the next tile separates these reads from the next writes.)
          uint32_t kth = kFixed;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const uint32_t mine = (i + (KMAX - topk) < KMAX) ? val_at(i + (KMAX - topk)) : kEmptyVal;
            kth = min(kth, max(mine, sX[qd ^ 1][7 - i][lt]));
          }
          if (kth != kFixed) floor_thr_row = fmaxf(floor_thr_row, ordered_to_score(kth));
        }
      }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base, 256);
    if (NQ > 1) {   // merge the row's NQ lists (the centroid buffers are free: every MMA has completed)
      uint64_t* sMerge = reinterpret_cast<uint64_t*>(sKM);
      if (qd > 0) {
#pragma unroll
        for (int j = 0; j < KMAX; ++j) sMerge[((qd - 1) * KMAX + j) * 128 + lt] = ((uint64_t)val[j] << 32) | (uint32_t)idx[j];
      }
      __syncthreads();
      if (qd == 0) {
        for (int e = 0; e < (NQ - 1) * KMAX; ++e) {
          const uint64_t cand = sMerge[e * 128 + lt];
          const uint32_t ox = (uint32_t)(cand >> 32);
          const int n = (int)(uint32_t)cand;
          // blocked and empty slots of the other lists are skipped.  The lists meet in no particular
          // chunk order, so the order is the full one here: score first, then the higher chunk id.
          if (n >= 0 && (ox > val[KMAX - 1] || (ox == val[KMAX - 1] && n > idx[KMAX - 1]))) {
            bool gt[KMAX];
#pragma unroll
            for (int y = 0; y < KMAX; ++y) gt[y] = ox > val[y] || (ox == val[y] && n > idx[y]);
#pragma unroll
            for (int y = KMAX - 1; y > 0; --y) {
              idx[y] = gt[y - 1] ? idx[y - 1] : (gt[y] ? n : idx[y]);
              val[y] = gt[y - 1] ? val[y - 1] : (gt[y] ? ox : val[y]);
            }
            idx[0] = gt[0] ? n : idx[0];
            val[0] = gt[0] ? ox : val[0];
          }
        }
      }
    }
  }
  if (row_ok && qd == 0) {
    const int64_t o = (int64_t)(q0 + r0 + lt) * p.t_rs + (int64_t)h * p.t_hs;
#pragma unroll
    for (int j = 0; j < KMAX; ++j) {
      const int slot = j - (KMAX - topk);
      if (slot >= 0) {
        p.topk_idx[o + slot] = idx[j];
        if (p.topk_val) p.topk_val[o + slot] = val[j] == kFixed ? CUDART_INF_F : ordered_to_score(val[j]);
      }
    }
  }
}

static int g_gate_engine = 1;
void set_gate_engine(int e) { g_gate_engine = e; }
bool gate_tc_supported(int d, int topk) { return (d == 64 || d == 128 || d == 256) && topk <= 32; }

// reads the word (synchronising) and clears it, so that one expired wait is reported once
int read_gate_status(int* out) {
  FMB_CUDA(cudaMemcpyFromSymbol(out, g_gate_status, sizeof(int)));
  if (*out != 0) {
    const int zero = 0;
    FMB_CUDA(cudaMemcpyToSymbol(g_gate_status, &zero, sizeof(int)));
  }
  return FMB_OK;
}

template <typename T, int D, int KMAX, int NQ>
static int gate_tc_launch(const GateParams& p, int batch, int max_q, cudaStream_t s) {
  // 2 CTAs per SM at most (256 TMEM columns each): keep dynamic shared memory above a third of the SM's
  size_t smem = 1024 + (size_t)3 * 128 * D * 2;
  if (smem < 80 * 1024) smem = 80 * 1024;
  static_assert(NQ == 1 || (size_t)(NQ - 1) * KMAX * 128 * 8 <= (size_t)2 * 128 * D * 2, "merge buffer fits the centroid tiles");
  auto kern = gate_topk_tc_kernel<T, D, KMAX, NQ>;
  FMB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  kern<<<dim3(ceil_div(max_q, kGateM), p.heads, batch), 128 * NQ, smem, s>>>(p);
  FMB_LAUNCH_CHECK("gate_topk_tc_kernel");
  return FMB_OK;
}
template <typename T, int D>
static int gate_tc_pick(const GateParams& p, int batch, int max_q, cudaStream_t s) {
  // threads per row (each scans its share of a tile's columns with its own list, merged at the
  // end).  Measured at 64K tokens, top-k 8: 1.77 ms with one, 1.67 ms with two, 2.68 ms with four.
  if (p.topk <= 8) return gate_tc_launch<T, D, 8, 2>(p, batch, max_q, s);
  if (p.topk <= 16) return gate_tc_launch<T, D, 16, 1>(p, batch, max_q, s);
  return gate_tc_launch<T, D, 32, 1>(p, batch, max_q, s);
}

template <typename T>
static int gate_dispatch(const GateParams& p, int batch, int max_q, cudaStream_t s) {
  const size_t smem = (size_t)kGateDSlab * (kGateM + kGateN) * sizeof(T) +
                      (size_t)kGateM * kGateSStride * sizeof(float) + (size_t)kGateM * p.topk * 8;
  dim3 grid(ceil_div(max_q, kGateM), p.heads, batch);
  if (g_gate_engine == 1 && gate_tc_supported(p.d, p.topk)) {
    if (p.d == 64) return gate_tc_pick<T, 64>(p, batch, max_q, s);
    if (p.d == 128) return gate_tc_pick<T, 128>(p, batch, max_q, s);
    return gate_tc_pick<T, 256>(p, batch, max_q, s);     // one CTA per SM: Q and two centroid tiles are 192 KB
  }
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
