// tcgen05 main kernels of the block-sparse attention for head dim 256 (the host pads 129 ... 255 up to it).
//
// The kernels of fmb_attn_tc.cu keep dK and dV of a 128-key block in the SM's 512 TMEM columns,
// which a head dim of 128 already fills, and their shared-memory tiles assume d <= 128.  Wider heads
// run here (forward: key blocks of 128 keys where the chunk allows, else 64; backward: 64), in a
// simpler shape: one CTA of 256 threads per work item (key block, head or kv head, sequence), every
// thread takes part in every phase, one thread issues the MMAs, and the only overlap is the
// cp.async gather of the next tile's rows under the rest of the current tile's work (the row
// gathers, 512 bytes per row, bound these kernels).  Same workspace contract (slots, per-entry
// partials) and the same merge kernels as the other engines.  Every mbarrier wait is bounded
// (status word of the workspace).
//
// Forward, per tile of 128 gathered query rows:
//     S = Q.K^T (K dimension d)  ->  the Q tile is refilled with the next tile's rows
//     chunk-local softmax in one pass (32 or 64 scores per thread), P (I/O dtype) to shared memory
//     O = P.V  (N = d)           ->  O / l written from registers (256 contiguous bytes per thread)
// Backward (head dim 256), work item = key block of one kv head, tiles = the q heads of its group
// times the 128-row tiles of each head's column.  dK and dV are accumulated TRANSPOSED (TMEM lane =
// head-dim index, two halves of 128; column = key), which takes 2 x 128 columns instead of the
// 2 x 256 of a key-per-lane layout; S | dP share 128 columns with the two halves of dQ, which are
// computed and written one after the other:
//     S = Q.K^T, dP = dO.V^T -> P = exp2(S.scale - LSE), dS = P o (dP - D) to shared memory
//     dV^T += dO^T.P, dK^T += Q^T.dS (Q, dO as M-major A operands), dQ = dS.K per half
//     once those have completed the Q and dO tiles are refilled with the next tile's rows while the
//     dQ halves are read out and written from registers
#include "fmb_attn.cuh"
#include "fmb_tc.cuh"

namespace fmb {

using namespace tc;

namespace {

constexpr int kM = 128;               // gathered rows per tile = TMEM lanes
constexpr int kC = 64;                // keys per block
constexpr int kThreads = 256;         // two threads per row: each owns half of the columns
constexpr float kLog2e = 1.4426950408889634f;

struct WideParams {
  const void *q, *k, *v, *dout;
  int64_t q_rs, q_hs, k_rs, k_hs, v_rs, v_hs, do_rs, do_hs;
  void *dk, *dv; int64_t dk_rs, dk_hs, dv_rs, dv_hs;
  const float *lse, *softmax_d;
  PassParams ps;
  const int32_t *cu_q, *k_begin, *k_end;
  void* part_o; float* part_lse; int* status;
  int heads, heads_k; int64_t total_q;
  float scale; int causal;
};

// threads that take part in the 16-byte copies of rows of D elements: eight rows per pass
template <int D> struct Copiers { static constexpr int n = (D / 8) * 8; };

template <typename T, int C, int D>
__global__ void __launch_bounds__(kThreads) fwd_wide_tc_kernel(WideParams p) {
  constexpr int NCH = D / 8;                    // 16-byte chunks of a row
  constexpr int NT = Copiers<D>::n;             // copying threads
  constexpr uint32_t kKBlock = C * 128;         // bytes between 64-element blocks of the K / V tiles
  constexpr uint32_t kQBlock = kM * 128;        // same for the 128-row Q and P tiles
  constexpr int CH = C / 2, DH = D / 2;         // keys / head-dim columns per thread
  static_assert(D == 256 && (C == 64 || C == 128), "head dim 256, key blocks of 64 or 128");
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  __shared__ uint64_t bar_s, bar_o;
  __shared__ uint32_t tmem_base_s;
  __shared__ int sRow[kM];
  __shared__ float sMax[2][kM], sSum[2][kM];

  // with 128-key blocks the tiles and the arrays above fill the 227 KB: no room for alignment padding
  unsigned char* smem = smem_raw;
  if ((smem_u32(smem_raw) & 1023u) != 0) {
    if (threadIdx.x == 0) atomicCAS(p.status, 0, 9);
    return;
  }
  unsigned char* sK = smem;                     // [C][D]
  unsigned char* sV = sK + C * D * 2;           // [C][D]
  unsigned char* sQ = sV + C * D * 2;           // [128][D]: refilled as soon as the tile's S has been computed
  unsigned char* sP = sQ + kM * D * 2;          // [128][C]

  const int tid = threadIdx.x, warp = tid >> 5;
  const int lt = tid & (kM - 1), hf = tid >> 7;
  const int c = blockIdx.x / p.ps.nsub, sb = blockIdx.x % p.ps.nsub, h = p.ps.h0 + blockIdx.y, b = blockIdx.z;
  const ColRef col = column_of(p.ps, b, h, c);
  if (col.nnz <= 0) return;                     // CTA-uniform
  const int64_t slot0 = (int64_t)sb * p.ps.cap + col.slot;
  const int q0 = p.cu_q[b], len_q = p.cu_q[b + 1] - q0;
  const int k0 = p.k_begin[b], len_k = p.k_end[b] - k0;
  const int key0 = c * p.ps.chunk + sb * C;
  const int keys_valid = max(0, min(C, len_k - key0));
  const int hk = h / (p.heads / p.heads_k);
  const int shift = len_k - len_q;
  const float scale_log2 = p.scale * kLog2e;
  const int ntiles = (col.nnz + kM - 1) / kM;
  const T* qbase = static_cast<const T*>(p.q) + (int64_t)q0 * p.q_rs + (int64_t)h * p.q_hs;
  T* part_o = static_cast<T*>(p.part_o);

  if (warp == 0) tmem_alloc(&tmem_base_s, 512);
  if (tid == 0) {
    mbar_init(&bar_s, 1);
    mbar_init(&bar_o, 1);
    mbar_fence_init();
  }
  // row ids of tile t (-1 = none)
  auto load_rows = [&](int t) {
    if (tid < kM) {
      int r = -1;
      if (t < ntiles && t * kM + tid < col.nnz) {
        r = p.ps.indices[col.off + t * kM + tid];
        if (r < 0 || r >= len_q) r = -1;
      }
      sRow[tid] = r;
    }
  };
  load_rows(0);
  if (tid < NT) {
    const T* kbase = static_cast<const T*>(p.k) + (int64_t)(k0 + key0) * p.k_rs + (int64_t)hk * p.k_hs;
    const T* vbase = static_cast<const T*>(p.v) + (int64_t)(k0 + key0) * p.v_rs + (int64_t)hk * p.v_hs;
    dense_cp_async<T, NCH, C, NT>(tid, sK, kKBlock, kbase, p.k_rs, keys_valid);
    dense_cp_async<T, NCH, C, NT>(tid, sV, kKBlock, vbase, p.v_rs, keys_valid);
  }
  tc_fence_before_sync();
  __syncthreads();                              // row ids of tile 0, the TMEM base, the barriers
  tc_fence_after_sync();
  if (tid < NT) gather_cp_async<T, NCH, NT>(tid, sQ, kQBlock, qbase, p.q_rs, sRow);
  const uint32_t tmem_base = tmem_base_s;
  const uint32_t tS = tmem_base, tO = tmem_base + 256;
  const uint32_t lane_sel = (uint32_t)((warp & 3) * 32) << 16;
  constexpr uint32_t idesc_s = make_idesc(FmtOf<T>::v, kM, C, 0, 0);
  constexpr uint32_t idesc_o = make_idesc(FmtOf<T>::v, kM, D, 0, 1);
  const uint32_t hi = desc_hi_sw128(1024);
  const uint32_t q_km = desc_lo_sw128(smem_u32(sQ), 16), k_km = desc_lo_sw128(smem_u32(sK), 16);
  const uint32_t v_mn = desc_lo_sw128(smem_u32(sV), kKBlock), p_km = desc_lo_sw128(smem_u32(sP), 16);
  bool good = true;

#pragma unroll 1
  for (int i = 0; i < ntiles && good; ++i) {
    const int t0 = i * kM;
    const int rows = min(kM, col.nnz - t0);
    // Q(i) (with K and V on the first tile) has landed
    const int r = sRow[lt];                     // this tile's row, before the next tile's ids replace it
    cp_async_wait_all();
    fence_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    if (tid == 0) {
      umma_gemm<D / 16>(tS, q_km, hi, 2, kQBlock >> 4, k_km, hi, 2, kKBlock >> 4, idesc_s, 0);
      umma_commit(&bar_s);
    }
    load_rows(i + 1);                           // (every thread has read its row id above)
    good = mbar_wait(&bar_s, i & 1, p.status, 1);
    __syncthreads();                            // the next tile's row ids
    tc_fence_after_sync();
    // S is complete, so the Q tile is free: the next tile's rows are gathered under the rest of this
    // tile's work (the row gather, not the arithmetic, is what bounds these kernels)
    if (i + 1 < ntiles && tid < NT) gather_cp_async<T, NCH, NT>(tid, sQ, kQBlock, qbase, p.q_rs, sRow);

    // ---- chunk-local softmax of row `lt`, this thread's half of the keys, in one pass over the scores
    const int lim = r < 0 ? 0 : (p.causal ? min(keys_valid, r + shift - key0 + 1) : keys_valid);
    float s[CH];
#pragma unroll
    for (int q4 = 0; q4 < CH / 32; ++q4) tmem_ld32(tS + lane_sel + hf * CH + q4 * 32, s + q4 * 32);
    tmem_ld_wait();
    tc_fence_before_sync();
    float mx = -CUDART_INF_F;
#pragma unroll
    for (int jj = 0; jj < CH; ++jj) mx = fmaxf(mx, hf * CH + jj < lim ? s[jj] : -CUDART_INF_F);
    sMax[hf][lt] = mx;
    good = __syncthreads_and(good);
    if (!good) break;
    mx = fmaxf(mx, sMax[hf ^ 1][lt]);
    const float mref = lim > 0 ? mx * scale_log2 : 0.f;
    float sum = 0.f;
#pragma unroll
    for (int jj = 0; jj < CH; ++jj) {
      const float e = exp2f(s[jj] * scale_log2 - mref);
      s[jj] = (hf * CH + jj < lim) ? e : 0.f;
      sum += s[jj];
    }
#pragma unroll
    for (int jj = 0; jj < CH / 8; ++jj)
      *reinterpret_cast<uint4*>(sP + sw128_offset(lt, hf * (CH / 8) + jj, kQBlock)) = pack8<T>(s + jj * 8);
    sSum[hf][lt] = sum;
    fence_async_smem();
    tc_fence_before_sync();
    __syncthreads();                            // P complete; S has been read by every thread
    tc_fence_after_sync();
    if (tid == 0) {
      umma_gemm<C / 16>(tO, p_km, hi, 2, kQBlock >> 4, v_mn, hi, 128, 512, idesc_o, 0);
      umma_commit(&bar_o);
    }
    sum += sSum[hf ^ 1][lt];
    const float inv = sum > 0.f ? 1.f / sum : 0.f;
    if (hf == 0 && lt < rows) p.part_lse[slot0 + t0 + lt] = sum > 0.f ? mx * p.scale + logf(sum) : -CUDART_INF_F;
    good = mbar_wait(&bar_o, i & 1, p.status, 2);
    tc_fence_after_sync();

    // ---- normalised partial O of row `lt`, this thread's half of the head dim (256 contiguous
    // bytes of the row's slot), written from registers; 16-byte chunks permuted like every partial
    {
      const int key = (int)((slot0 + t0 + lt) & 7);
      T* dst = part_o + (slot0 + t0 + lt) * D;
#pragma unroll
      for (int q4 = 0; q4 < DH / 32; ++q4) {
        float o[32];
        tmem_ld32(tO + lane_sel + hf * DH + q4 * 32, o);
        tmem_ld_wait();
        if (lt < rows) {
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) {
#pragma unroll
            for (int e = 0; e < 8; ++e) o[jj * 8 + e] *= inv;
            *reinterpret_cast<uint4*>(dst + (((hf * (DH / 8) + q4 * 4 + jj) ^ key) << 3)) = pack8<T>(o + jj * 8);
          }
        }
      }
      tc_fence_before_sync();
    }
    // (the barrier at the top of the next tile keeps its P.V, which overwrites O, behind these reads)
  }
  cp_async_wait_all();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == 0) tmem_dealloc(tmem_base, 512);
}

template <typename T, int D>
__global__ void __launch_bounds__(kThreads) bwd_wide_tc_kernel(WideParams p) {
  static_assert(D == 256, "two head-dim halves of 128 TMEM lanes");
  constexpr int NCH = D / 8;
  constexpr int NT = Copiers<D>::n;
  constexpr uint32_t kKBlock = kC * 128;
  constexpr uint32_t kQBlock = kM * 128;
  constexpr uint32_t kQTile = kM * D * 2;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  __shared__ uint64_t bar_a, bar_b, bar_c;
  __shared__ uint32_t tmem_base_s;
  __shared__ int sRow[kM];
  __shared__ float sLse[kM], sDsum[kM];

  // the tiles fill the 227 KB together with the static arrays above: no room for alignment padding
  unsigned char* smem = smem_raw;
  if ((smem_u32(smem_raw) & 1023u) != 0) {
    if (threadIdx.x == 0) atomicCAS(p.status, 0, 9);
    return;
  }
  unsigned char* sK = smem;                     // [64][D]
  unsigned char* sV = sK + kC * D * 2;          // [64][D]
  unsigned char* sQ = sV + kC * D * 2;          // [128][D]
  unsigned char* sdO = sQ + kQTile;             // [128][D]
  unsigned char* sP = sdO + kQTile;             // [128][64]
  unsigned char* sdS = sP + kM * kC * 2;        // [128][64]

  const int tid = threadIdx.x, warp = tid >> 5;
  const int lt = tid & (kM - 1), hf = tid >> 7;
  const int group = p.heads / p.heads_k;
  const int c = blockIdx.x / p.ps.nsub, sb = blockIdx.x % p.ps.nsub, hk = p.ps.h0 / group + blockIdx.y, b = blockIdx.z;
  const int64_t plane = (int64_t)sb * p.ps.cap;
  const int q0 = p.cu_q[b], len_q = p.cu_q[b + 1] - q0;
  const int k0 = p.k_begin[b], len_k = p.k_end[b] - k0;
  const int key0 = c * p.ps.chunk + sb * kC;
  T* part_dq = static_cast<T*>(p.part_o);
  if (key0 >= len_k) {                          // CTA-uniform: the key block starts past the sequence's last key
    zero_dq_partials<T>(p.ps, part_dq, plane, b, hk, group, c, D);
    return;
  }
  const int keys_valid = min(kC, len_k - key0);
  const int shift = len_k - len_q;
  const float scale_log2 = p.scale * kLog2e;

  if (warp == 0) tmem_alloc(&tmem_base_s, 512);
  if (tid == 0) {
    mbar_init(&bar_a, 1);
    mbar_init(&bar_b, 1);
    mbar_init(&bar_c, 1);
    mbar_fence_init();
  }
  if (tid < NT) {
    const T* kbase = static_cast<const T*>(p.k) + (int64_t)(k0 + key0) * p.k_rs + (int64_t)hk * p.k_hs;
    const T* vbase = static_cast<const T*>(p.v) + (int64_t)(k0 + key0) * p.v_rs + (int64_t)hk * p.v_hs;
    dense_cp_async<T, NCH, kC, NT>(tid, sK, kKBlock, kbase, p.k_rs, keys_valid);
    dense_cp_async<T, NCH, kC, NT>(tid, sV, kKBlock, vbase, p.v_rs, keys_valid);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_base_s;
  const uint32_t tS = tmem_base, tdP = tmem_base + 64, tdQ = tmem_base;      // dQ halves over S | dP
  const uint32_t tdK = tmem_base + 128, tdV = tmem_base + 256;                // [half][64 keys]
  const uint32_t lane_sel = (uint32_t)((warp & 3) * 32) << 16;
  constexpr uint32_t idesc_s = make_idesc(FmtOf<T>::v, kM, kC, 0, 0);         // rows x keys
  constexpr uint32_t idesc_t = make_idesc(FmtOf<T>::v, 128, kC, 1, 1);        // head-dim half x keys, both M/N-major
  constexpr uint32_t idesc_dq = make_idesc(FmtOf<T>::v, kM, 128, 0, 1);       // rows x head-dim half
  const uint32_t hi = desc_hi_sw128(1024);
  const uint32_t k_km = desc_lo_sw128(smem_u32(sK), 16), v_km = desc_lo_sw128(smem_u32(sV), 16);
  const uint32_t q_km = desc_lo_sw128(smem_u32(sQ), 16), do_km = desc_lo_sw128(smem_u32(sdO), 16);
  const uint32_t ds_km = desc_lo_sw128(smem_u32(sdS), 16);
  const uint32_t p_mn = desc_lo_sw128(smem_u32(sP), kQBlock), ds_mn = desc_lo_sw128(smem_u32(sdS), kQBlock);
  bool good = true;
  uint32_t g = 0;                               // tiles so far (phase of the three barriers)

  // The item's tiles as one sequence over the q heads of the group and the 128-row tiles of each
  // head's column: `cur` is the tile being worked on, `nxt` the one whose rows are gathered under
  // the end of it.
  struct Tile { int hg, t0, nnz; int64_t off, slot; bool valid; };
  auto seek = [&](Tile& t) {                    // first head >= t.hg with a column; t.t0 = 0
    t.valid = false;
    for (; t.hg < group; ++t.hg) {
      const ColRef col = column_of(p.ps, b, hk * group + t.hg, c);
      if (col.nnz > 0) { t.nnz = col.nnz; t.off = col.off; t.slot = col.slot; t.t0 = 0; t.valid = true; return; }
    }
  };
  auto advance = [&](Tile t) {
    t.t0 += kM;
    if (t.t0 >= t.nnz) { ++t.hg; seek(t); }
    return t;
  };
  // row ids, log-sum-exps and dO.O sums of a tile into shared memory (the first 128 threads)
  auto load_rows = [&](const Tile& t) {
    if (tid < kM) {
      int r = -1;
      float l = CUDART_INF_F, dd = 0.f;
      if (t.valid && t.t0 + tid < t.nnz) {
        r = p.ps.indices[t.off + t.t0 + tid];
        if (r < 0 || r >= len_q) r = -1;
        else {
          const int64_t at = (int64_t)(hk * group + t.hg) * p.total_q + q0 + r;
          l = p.lse[at];
          dd = p.softmax_d[at];
        }
      }
      sRow[tid] = r; sLse[tid] = l; sDsum[tid] = dd;
    }
  };
  auto gather = [&](const Tile& t) {
    if (tid < NT) {
      const int h = hk * group + t.hg;
      gather_cp_async<T, NCH, NT>(tid, sQ, kQBlock, static_cast<const T*>(p.q) + (int64_t)q0 * p.q_rs + (int64_t)h * p.q_hs,
                                  p.q_rs, sRow);
      gather_cp_async<T, NCH, NT>(tid, sdO, kQBlock,
                                  static_cast<const T*>(p.dout) + (int64_t)q0 * p.do_rs + (int64_t)h * p.do_hs, p.do_rs, sRow);
    }
  };
  Tile cur{0, 0, 0, 0, 0, false};
  seek(cur);
  if (cur.valid) {
    load_rows(cur);
    __syncthreads();
    gather(cur);
  }
#pragma unroll 1
  for (; cur.valid; ++g) {
    const int rows = min(kM, cur.nnz - cur.t0);
    const int64_t slot0 = plane + cur.slot + cur.t0;
    cp_async_wait_all();                        // Q and dO rows of the tile (and K, V on the item's first)
    fence_async_smem();
    tc_fence_before_sync();
    good = __syncthreads_and(good);             // (a wait that gave up in the tile before ends the loop for every thread)
    if (!good) break;
    tc_fence_after_sync();
    if (tid == 0) {
      umma_gemm<D / 16>(tS, q_km, hi, 2, kQBlock >> 4, k_km, hi, 2, kKBlock >> 4, idesc_s, 0);
      umma_gemm<D / 16>(tdP, do_km, hi, 2, kQBlock >> 4, v_km, hi, 2, kKBlock >> 4, idesc_s, 0);
      umma_commit(&bar_a);
    }
    const Tile nxt = advance(cur);              // (global loads of the next column's header, under the MMAs)
    good = mbar_wait(&bar_a, g & 1, p.status, 3);
    tc_fence_after_sync();

    // ---- P and dS of row `lt`, this thread's 32 keys
    {
      const int r = sRow[lt];
      const float lse2 = sLse[lt] * kLog2e, dd = sDsum[lt];
      const int lim = r < 0 ? 0 : (p.causal ? min(keys_valid, r + shift - key0 + 1) : keys_valid);
      float pr[32], dp[32];
      tmem_ld32(tS + lane_sel + hf * 32, pr);
      tmem_ld32(tdP + lane_sel + hf * 32, dp);
      tmem_ld_wait();
      tc_fence_before_sync();
#pragma unroll
      for (int jj = 0; jj < 32; ++jj) {
        pr[jj] = (hf * 32 + jj < lim) ? exp2f(pr[jj] * scale_log2 - lse2) : 0.f;
        dp[jj] = pr[jj] * (dp[jj] - dd);
      }
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        *reinterpret_cast<uint4*>(sP + sw128_offset(lt, hf * 4 + jj, kQBlock)) = pack8<T>(pr + jj * 8);
        *reinterpret_cast<uint4*>(sdS + sw128_offset(lt, hf * 4 + jj, kQBlock)) = pack8<T>(dp + jj * 8);
      }
    }
    fence_async_smem();
    tc_fence_before_sync();
    good = __syncthreads_and(good);             // P, dS complete; S, dP and the row data have been read by every thread
    if (!good) break;
    tc_fence_after_sync();
    if (tid == 0) {
      const uint32_t acc = g > 0 ? 1u : 0u;     // the item's first tile starts the accumulators
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        // dV^T[half] += dO^T.P, dK^T[half] += Q^T.dS : M = 128 head-dim columns, N = keys, K = the rows
        umma_gemm<kM / 16>(tdV + hh * 64, desc_lo_sw128(smem_u32(sdO) + hh * 2 * kQBlock, kQBlock), hi, 128, 512,
                           p_mn, hi, 128, 512, idesc_t, acc);
        umma_gemm<kM / 16>(tdK + hh * 64, desc_lo_sw128(smem_u32(sQ) + hh * 2 * kQBlock, kQBlock), hi, 128, 512,
                           ds_mn, hi, 128, 512, idesc_t, acc);
      }
      // dQ[first half of the head dim] = dS.K over the columns S and dP occupied
      umma_gemm<kC / 16>(tdQ, ds_km, hi, 2, 0, desc_lo_sw128(smem_u32(sK), kKBlock), hi, 128, 512, idesc_dq, 0);
      umma_commit(&bar_b);
    }
    load_rows(nxt);                             // the next tile's row data, under these MMAs
    good = mbar_wait(&bar_b, g & 1, p.status, 4);
    good = __syncthreads_and(good);             // (also publishes the row data)
    if (!good) break;
    tc_fence_after_sync();
    // dV^T, dK^T and the first dQ half are complete: the Q and dO tiles are free, and the next
    // tile's rows are gathered while dQ is read out (the gathers bound this kernel)
    if (nxt.valid) gather(nxt);
    // ---- dQ partial of row `lt`: per head-dim half, this thread's 64 columns (128 contiguous bytes
    // of the row's slot): scaled, rounded, written from registers, 16-byte chunks permuted like every partial
    const int key = (int)((slot0 + lt) & 7);
    T* dst = part_dq + (slot0 + lt) * D;
#pragma unroll 1
    for (int hh = 0; hh < 2; ++hh) {
#pragma unroll
      for (int i2 = 0; i2 < 2; ++i2) {
        float o[32];
        tmem_ld32(tdQ + lane_sel + hf * 64 + i2 * 32, o);
        tmem_ld_wait();
        if (lt < rows) {
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) {
#pragma unroll
            for (int e = 0; e < 8; ++e) o[jj * 8 + e] *= p.scale;
            *reinterpret_cast<uint4*>(dst + (((hh * 16 + hf * 8 + i2 * 4 + jj) ^ key) << 3)) = pack8<T>(o + jj * 8);
          }
        }
      }
      tc_fence_before_sync();
      if (hh == 0) {
        __syncthreads();                        // the first half has been read out of TMEM
        tc_fence_after_sync();
        if (tid == 0) {
          umma_gemm<kC / 16>(tdQ, ds_km, hi, 2, 0, desc_lo_sw128(smem_u32(sK) + 2 * kKBlock, kKBlock), hi, 128, 512,
                             idesc_dq, 0);
          umma_commit(&bar_c);
        }
        good = mbar_wait(&bar_c, g & 1, p.status, 4);
        tc_fence_after_sync();
      }
    }
    cur = nxt;
    // (the barrier at the top of the next tile keeps its S and dP, which overwrite dQ, behind these reads)
  }
  cp_async_wait_all();                          // (K and V of an item without tiles)
  // ---- dK (scaled) and dV of this key block: TMEM lane = head-dim index of this thread's half,
  // column = key; consecutive lanes write consecutive elements of a key's row
  if (good) {
    tc_fence_after_sync();
    T* dkp = static_cast<T*>(p.dk) + (int64_t)(k0 + key0) * p.dk_rs + (int64_t)hk * p.dk_hs + hf * 128 + lt;
    T* dvp = static_cast<T*>(p.dv) + (int64_t)(k0 + key0) * p.dv_rs + (int64_t)hk * p.dv_hs + hf * 128 + lt;
#pragma unroll 1
    for (int i2 = 0; i2 < 2; ++i2) {
      float a[32], bq[32];
      if (g > 0) {
        tmem_ld32(tdK + hf * 64 + lane_sel + i2 * 32, a);
        tmem_ld32(tdV + hf * 64 + lane_sel + i2 * 32, bq);
        tmem_ld_wait();
      } else {                                   // no tile at all: the gradients of these keys are zero
#pragma unroll
        for (int jj = 0; jj < 32; ++jj) { a[jj] = 0.f; bq[jj] = 0.f; }
      }
#pragma unroll
      for (int jj = 0; jj < 32; ++jj) {
        const int kk = i2 * 32 + jj;
        if (kk < keys_valid) {
          dkp[(int64_t)kk * p.dk_rs] = Elem<T>::from_f(a[jj] * p.scale);
          dvp[(int64_t)kk * p.dv_rs] = Elem<T>::from_f(bq[jj]);
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == 0) tmem_dealloc(tmem_base, 512);
}

WideParams make_wide_params(const AttnArgs& a, const AttnWorkspace& w, const PassParams& ps) {
  WideParams p;
  p.q = a.q; p.k = a.k; p.v = a.v; p.dout = a.dout;
  p.q_rs = a.q_rs; p.q_hs = a.q_hs; p.k_rs = a.k_rs; p.k_hs = a.k_hs; p.v_rs = a.v_rs; p.v_hs = a.v_hs;
  p.do_rs = a.do_rs; p.do_hs = a.do_hs;
  p.dk = a.dk; p.dv = a.dv; p.dk_rs = a.dk_rs; p.dk_hs = a.dk_hs; p.dv_rs = a.dv_rs; p.dv_hs = a.dv_hs;
  p.lse = a.lse; p.softmax_d = a.softmax_d;
  p.ps = ps;
  p.cu_q = a.cu_q; p.k_begin = a.k_begin; p.k_end = a.k_end;
  p.part_o = w.part_o; p.part_lse = w.part_lse; p.status = w.status;
  p.heads = a.heads; p.heads_k = a.heads_k; p.total_q = a.total_q;
  p.scale = a.scale; p.causal = a.causal;
  return p;
}

template <typename T, int C, int D>
int fwd_wide_launch(const AttnArgs& a, const AttnWorkspace& w, const PassParams& ps, cudaStream_t s) {
  const WideParams p = make_wide_params(a, w, ps);
  const size_t smem = (size_t)2 * C * D * 2 + (size_t)kM * D * 2 + (size_t)kM * C * 2;   // K, V, Q, P
  auto kern = fwd_wide_tc_kernel<T, C, D>;
  FMB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  kern<<<dim3(a.ncol * ps.nsub, ps.nh, a.batch), kThreads, smem, s>>>(p);
  FMB_LAUNCH_CHECK("fwd_wide_tc_kernel");
  return FMB_OK;
}

template <typename T, int D>
int bwd_wide_launch(const AttnArgs& a, const AttnWorkspace& w, const PassParams& ps, cudaStream_t s) {
  const WideParams p = make_wide_params(a, w, ps);
  // K, V, Q, dO, P, dS: with d = 256 that and the kernel's static arrays are the 227 KB a CTA may have
  const size_t smem = (size_t)2 * kC * D * 2 + (size_t)2 * kM * D * 2 + (size_t)2 * kM * kC * 2;
  auto kern = bwd_wide_tc_kernel<T, D>;
  FMB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const int nchunk = max(a.ncol, ceil_div(a.max_k, a.chunk));
  kern<<<dim3(nchunk * ps.nsub, ps.nh / (a.heads / a.heads_k), a.batch), kThreads, smem, s>>>(p);
  FMB_LAUNCH_CHECK("bwd_wide_tc_kernel");
  return FMB_OK;
}

}  // namespace

bool tc_wide_supported(const AttnArgs& a, bool backward) {
  if (a.chunk % 64 != 0) return false;
  return a.d == 256;
}

int launch_bwd_main_tc_wide(const AttnArgs& a, const AttnWorkspace& w, const PassParams& ps, cudaStream_t s) {
  if (a.batch == 0 || a.heads == 0) return FMB_OK;
  if (w.kb != kC) return fail(FMB_ERR_UNSUPPORTED, "wide-head backward: key block %d (64 expected)", w.kb);
  if (a.d == 256)
    return a.dtype == FMB_BF16 ? bwd_wide_launch<__nv_bfloat16, 256>(a, w, ps, s) : bwd_wide_launch<__half, 256>(a, w, ps, s);
  return fail(FMB_ERR_UNSUPPORTED, "wide-head backward: head_dim %d not built", a.d);
}

int launch_fwd_main_tc_wide(const AttnArgs& a, const AttnWorkspace& w, const PassParams& ps, cudaStream_t s) {
  if (a.ncol == 0 || a.batch == 0 || a.heads == 0) return FMB_OK;
  if (a.d == 256 && w.kb == 128)
    return a.dtype == FMB_BF16 ? fwd_wide_launch<__nv_bfloat16, 128, 256>(a, w, ps, s)
                               : fwd_wide_launch<__half, 128, 256>(a, w, ps, s);
  if (a.d == 256 && w.kb == 64)
    return a.dtype == FMB_BF16 ? fwd_wide_launch<__nv_bfloat16, 64, 256>(a, w, ps, s)
                               : fwd_wide_launch<__half, 64, 256>(a, w, ps, s);
  return fail(FMB_ERR_UNSUPPORTED, "wide-head forward: key block %d / head_dim %d not built", w.kb, a.d);
}

}  // namespace fmb
