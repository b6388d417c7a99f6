// tcgen05 tensor-core engine of the block-sparse attention main kernels.
//
// Key-chunk-major: a work item is one key block of one (sequence, head) (backward: kv head); its
// K and V tiles sit in shared memory (128-byte-swizzled UMMA tiles) while the item's CSC column,
// i.e. the gathered list of query rows that selected the chunk, is walked in dense tiles of 128
// rows.  One persistent CTA per SM (all 512 TMEM columns, nearly all shared memory) runs through
// its work items as one stream of tiles; the roles (compute warps, one MMA-issuing thread, loader
// warps that gather rows with 16-byte cp.async copies, a scout warp that decodes items ahead and
// stages K / V) hand tiles to each other through mbarriers.  Forward and backward kernels are
// described at their definitions below.
// Every mbarrier wait is bounded; a wait that expires records where in the status word of the
// workspace and the CTA leaves through the normal exit (TMEM released).
#include "fmb_attn.cuh"
#include "fmb_tma.cuh"

namespace fmb {

using namespace tc;

constexpr int kTcM = 128;   // gathered rows per tile = TMEM lanes

constexpr float kLog2eTc = 1.4426950408889634f;

struct TcParams {
  const void *q, *k, *v, *dout;
  int64_t q_rs, q_hs, k_rs, k_hs, v_rs, v_hs, do_rs, do_hs;
  void *dk, *dv; int64_t dk_rs, dk_hs, dv_rs, dv_hs;
  const float *lse, *softmax_d;
  PassParams ps;
  const int32_t *cu_q, *k_begin, *k_end;
  void* part_o; float* part_lse; int* status;
  int heads, heads_k; int64_t total_q;
  float scale; int causal;
  // persistent CTAs: work items (key block, head or kv head, sequence) are handed out through a
  // counter in the workspace status block.  Order: one (head, sequence) after the other, so that
  // the CTAs running at the same time gather rows of few heads (their Q / dO rows stay in L2);
  // inside a head the key blocks ascend (under a causal mask the early key blocks have the
  // longest columns, so a head's long items start first and its short ones fill the end).
  // The first `items_heavy` key blocks of every head (the longest columns) come before all of
  // that, so that no long item starts late in the launch.
  int* work; int n_items, items_x, items_y, items_z, items_heavy;
  // 1: whole key blocks are staged with TMA tensor-map loads (K and V laid out so that one 2-D map
  // covers all kv heads of a token row); a sequence's short last block takes the cp.async path
  int kv_tma;
};

// One key block (C rows x D columns of kv head `hk`, first row `row0`) -> the swizzled K-major
// tile at `tile`, as D/64 tensor-map loads that complete `bar` (whose one arrival is the
// expect_tx made here).  One thread.
template <int C, int D>
__device__ __forceinline__ void tma_stage_block(unsigned char* tile, const CUtensorMap* map, int64_t head_col, int row0,
                                                uint64_t* bar, uint32_t expect_bytes) {
  if (expect_bytes) mbar_expect_tx(bar, expect_bytes);
#pragma unroll
  for (int hb = 0; hb < D / 64; ++hb)
    tma_load_2d(tile + hb * (C * 128), map, (int)head_col + hb * 64, row0, bar);
}

// work item -> (key block index, head/sequence index)
__device__ __forceinline__ void decode_item(const TcParams& p, int item, int& bx, int& rem) {
  const int yz = p.items_y * p.items_z, n_a = p.items_heavy * yz;
  if (item < n_a) {
    bx = item / yz;
    rem = item - bx * yz;
  } else {
    const int j = item - n_a, rest = p.items_x - p.items_heavy;
    rem = j / rest;
    bx = p.items_heavy + (j - rem * rest);
  }
}

__host__ __device__ constexpr int next_pow2_cols(int x) { return x <= 32 ? 32 : x <= 64 ? 64 : x <= 128 ? 128 : x <= 256 ? 256 : 512; }

// ======================================================================== forward
// Work item = key block c of one (sequence, head); 704 threads, warp-specialised, one persistent
// CTA per SM that runs through its work items as ONE stream of 128-row tiles:
//   warps 0-7 / 8-15  compute group 0 / 1 (two threads per row, each owns half of the columns).
//                     The groups take alternate tiles of an item's CSC column; each has its own Q
//                     tile, P/O-staging tile, 256 TMEM columns (S | O) and mbarriers.
//                     Per tile: wait S -> chunk-local softmax (row maximum, then exponentials) ->
//                     P (bf16) to shared memory -> P_ready;  wait O -> O / l staged and written
//                     with one bulk copy per warp, log-sum-exp beside it.
//   warp 16           one thread issues every MMA of both groups.  It polls the groups' barriers in
//                     turn (P_ready -> O = P.V; Q tile landed -> next S = Q.K^T), so that a late
//                     gather never stalls a compute warp.
//   warps 17-18 / 19-20  loaders of group 0 / 1: row ids of the next tile, then its Q rows with
//                     16-byte cp.async copies straight into the swizzled UMMA tile, as soon as
//                     the group's previous S GEMM has released the Q tile.
//   warp 21           scout: takes work items from the counter, decodes them (a chain of dependent
//                     global loads) one item ahead and publishes them in shared memory; stages an
//                     item's K tile once the S GEMMs of the item before it have completed and its V
//                     tile once the P.V GEMMs have.
// No role waits for another at an item boundary except through the data it needs: the barriers are
// initialised once and their phases counted per group across items.
constexpr int kFwdGroups = 2;
constexpr int kFwdGroupThreads = 256;
constexpr int kFwdLoaderWarps = 2;              // loader warps per compute group
constexpr int kFwdLoaderSet = 32 * kFwdLoaderWarps;  // loader threads per compute group
constexpr int kFwdIssuerWarp = kFwdGroups * kFwdGroupThreads / 32;
constexpr int kFwdScoutWarp = kFwdIssuerWarp + 1 + kFwdGroups * kFwdLoaderWarps;
constexpr int kFwdThreads = kFwdGroups * kFwdGroupThreads + 32 + kFwdGroups * kFwdLoaderSet + 32;

// a decoded work item as the scout publishes it
struct FwdItem {
  int nnz;            // entries of the column (0: the stream has ended)
  int64_t off;        // first entry in `indices`
  int64_t slot;       // first slot of the column, plane included
  int q0, len_q, h;   // the sequence's first query token and length, the head
  int key0, keys_valid, shift;
};

template <typename T, int C, int D>
__global__ void __launch_bounds__(kFwdThreads) fwd_main_tc_kernel(TcParams p, const __grid_constant__ CUtensorMap map_k,
                                                                  const __grid_constant__ CUtensorMap map_v) {
  constexpr int QP = (C > D ? C : D);
  constexpr uint32_t kKBlock = C * 128;        // bytes between 64-element blocks of the K / V tiles
  constexpr uint32_t kQBlock = kTcM * 128;     // same for the 128-row Q / P tiles
  constexpr int NCOLS = 512;
  constexpr int CH = C / 2, DH = D / 2;        // columns per thread in the softmax / epilogue
  extern __shared__ unsigned char smem_raw[];
  __shared__ uint64_t bar_s[kFwdGroups], bar_o[kFwdGroups], bar_full[kFwdGroups], bar_qfree[kFwdGroups];
  __shared__ uint64_t bar_pready[kFwdGroups], bar_k, bar_v, bar_sfin, bar_fin, bar_info[4];
  __shared__ uint32_t tmem_base_s;
  __shared__ int s_info[4][12];
  __shared__ int sRow[kFwdGroups][2][kTcM];
  __shared__ float sMax[kFwdGroups][2][kTcM], sSum[kFwdGroups][2][kTcM];

  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  unsigned char* sK = smem;
  unsigned char* sV = sK + C * D * 2;
  unsigned char* sQg = sV + C * D * 2;                         // [group][128][D]
  unsigned char* sPOg = sQg + kFwdGroups * kTcM * D * 2;       // [group][128][max(C,D)]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const float scale_log2 = p.scale * kLog2eTc;
  if (warp == 0) tmem_alloc(&tmem_base_s, NCOLS);
  if (tid == 0) {
    for (int i = 0; i < kFwdGroups; ++i) {
      mbar_init(&bar_s[i], 1);
      mbar_init(&bar_o[i], 1);
      mbar_init(&bar_full[i], kFwdLoaderSet / 32);       // one arrival per loader warp
      mbar_init(&bar_qfree[i], 1);
      mbar_init(&bar_pready[i], kFwdGroupThreads / 32);  // one arrival per compute warp
    }
    mbar_init(&bar_k, 1); mbar_init(&bar_v, 1); mbar_init(&bar_sfin, 1); mbar_init(&bar_fin, 1);
    for (int i = 0; i < 4; ++i) mbar_init(&bar_info[i], 1);
    mbar_fence_init();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_base_s;

  // n-th item of this CTA's stream; false: the wait gave up (error recorded).  it.nnz == 0: the end.
  auto read_info = [&](uint32_t n, FwdItem& it) -> bool {
    if (!mbar_wait(&bar_info[n & 3], (n >> 2) & 1, p.status, 8)) {
      it.nnz = 0;
      return false;
    }
    const volatile int* f = s_info[n & 3];
    it.nnz = f[0];
    it.off = (int64_t)(((uint64_t)(uint32_t)f[2] << 32) | (uint32_t)f[1]);
    it.slot = (int64_t)(((uint64_t)(uint32_t)f[4] << 32) | (uint32_t)f[3]);
    it.q0 = f[5]; it.len_q = f[6]; it.h = f[7]; it.key0 = f[8]; it.keys_valid = f[9]; it.shift = f[10];
    return true;
  };

  if (warp == kFwdScoutWarp) {
    // =============================================================== scout: items, K and V tiles
    bool ok = true;
    const T* kbase = nullptr;
    const T* vbase = nullptr;
    int keys_valid = 0, key_row0 = 0;
    int64_t k_col = 0, v_col = 0;
    // takes items from the counter until one has entries, publishes it as item n of the stream
    auto scout_item = [&](uint32_t n) -> bool {
      FwdItem it;
      it.nnz = 0;
      for (;;) {
        int item = 0;
        if (lane == 0) item = atomicAdd(p.work, 1);
        item = __shfl_sync(0xffffffffu, item, 0);
        if (item >= p.n_items) { it.nnz = 0; break; }
        int bx, rem;
        decode_item(p, item, bx, rem);
        // C is the key block: chunk c of the pattern is covered by nsub blocks of C keys
        const int c = bx / p.ps.nsub, sb = bx % p.ps.nsub, h = p.ps.h0 + rem % p.items_y, b = rem / p.items_y;
        const ColRef col = column_of(p.ps, b, h, c);
        if (col.nnz <= 0) continue;
        const int q0 = p.cu_q[b], len_q = p.cu_q[b + 1] - q0;
        const int k0 = p.k_begin[b], len_k = p.k_end[b] - k0;
        const int hk = h / (p.heads / p.heads_k);
        it.nnz = col.nnz; it.off = col.off; it.slot = (int64_t)sb * p.ps.cap + col.slot;
        it.q0 = q0; it.len_q = len_q; it.h = h;
        it.key0 = c * p.ps.chunk + sb * C;
        it.keys_valid = max(0, min(C, len_k - it.key0));
        it.shift = len_k - len_q;
        kbase = static_cast<const T*>(p.k) + (int64_t)(k0 + it.key0) * p.k_rs + (int64_t)hk * p.k_hs;
        vbase = static_cast<const T*>(p.v) + (int64_t)(k0 + it.key0) * p.v_rs + (int64_t)hk * p.v_hs;
        keys_valid = it.keys_valid;
        key_row0 = k0 + it.key0;
        k_col = (int64_t)hk * p.k_hs;
        v_col = (int64_t)hk * p.v_hs;
        break;
      }
      if (lane == 0) {
        volatile int* f = s_info[n & 3];
        f[1] = (int)(uint32_t)((uint64_t)it.off & 0xffffffffu); f[2] = (int)(uint32_t)((uint64_t)it.off >> 32);
        f[3] = (int)(uint32_t)((uint64_t)it.slot & 0xffffffffu); f[4] = (int)(uint32_t)((uint64_t)it.slot >> 32);
        f[5] = it.q0; f[6] = it.len_q; f[7] = it.h; f[8] = it.key0; f[9] = it.keys_valid; f[10] = it.shift;
        f[0] = it.nnz;
        mbar_arrive(&bar_info[n & 3]);
      }
      return it.nnz > 0;
    };
    bool more = scout_item(0);
#pragma unroll 1
    for (uint32_t n = 0; more && ok; ++n) {
      // K of item n: every S GEMM of item n - 1 has completed; V: every P.V GEMM has
      if (n > 0) ok = mbar_wait(&bar_sfin, (n - 1) & 1, p.status, 8);
      if (!ok) break;
      const bool by_tma = p.kv_tma && keys_valid == C;     // warp-uniform
      if (by_tma) {
        if (lane == 0) tma_stage_block<C, D>(sK, &map_k, k_col, key_row0, &bar_k, C * D * 2);
      } else {
        dense_cp_async<T, D / 8, C, 32>(lane, sK, kKBlock, kbase, p.k_rs, keys_valid);
        cp_async_wait_all();
        fence_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar_k);
      }
      if (n > 0) ok = mbar_wait(&bar_fin, (n - 1) & 1, p.status, 8);
      if (!ok) break;
      if (by_tma) {
        if (lane == 0) tma_stage_block<C, D>(sV, &map_v, v_col, key_row0, &bar_v, C * D * 2);
      } else {
        dense_cp_async<T, D / 8, C, 32>(lane, sV, kKBlock, vbase, p.v_rs, keys_valid);
        cp_async_wait_all();
        fence_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar_v);
      }
      more = scout_item(n + 1);
    }
  } else if (warp == kFwdIssuerWarp) {
    // =============================================================== MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc(FmtOf<T>::v, kTcM, C, 0, 0);
      constexpr uint32_t idesc_o = make_idesc(FmtOf<T>::v, kTcM, D, 0, 1);
      const uint32_t hi = desc_hi_sw128(1024);
      const uint32_t k_km = desc_lo_sw128(smem_u32(sK), 16), v_mn = desc_lo_sw128(smem_u32(sV), kKBlock);
      constexpr uint32_t kQB = kQBlock >> 4, kKB = kKBlock >> 4;
      uint32_t cs[kFwdGroups] = {0, 0}, cp[kFwdGroups] = {0, 0};   // S / P.V GEMMs issued per group so far
      bool ok = true;
#pragma unroll 1
      for (uint32_t n = 0; ok; ++n) {
        FwdItem it;
        if (!(ok = read_info(n, it)) || it.nnz <= 0) break;
        const int ntiles = (it.nnz + kTcM - 1) / kTcM;
        int ts[kFwdGroups], tp[kFwdGroups];     // next tile whose S / P.V GEMM is to be issued
#pragma unroll
        for (int g = 0; g < kFwdGroups; ++g) { ts[g] = g; tp[g] = g; }
        if (!(ok = mbar_wait(&bar_k, n & 1, p.status, 6))) break;
        bool have_v = false, s_open = true;
        uint32_t idle = 0;
        while (ok && (tp[0] < ntiles || tp[1] < ntiles)) {
          bool progress = false;
          if (!have_v && mbar_test(&bar_v, n & 1)) have_v = true;
#pragma unroll
          for (int g = 0; g < kFwdGroups; ++g) {
            const uint32_t tS = tmem_base + g * 256, tO = tS + 128;
            const uint32_t q_km = desc_lo_sw128(smem_u32(sQg + g * (kTcM * D * 2)), 16);
            const uint32_t p_km = desc_lo_sw128(smem_u32(sPOg + g * (kTcM * QP * 2)), 16);
            // O = P.V of tile tp: P is in shared memory and S has been read
            if (have_v && tp[g] < ntiles && tp[g] < ts[g] && mbar_test(&bar_pready[g], cp[g] & 1)) {
              tc_fence_after_sync();
              umma_gemm<C / 16>(tO, p_km, hi, 2, kQB, v_mn, hi, 128, 512, idesc_o, 0);
              umma_commit(&bar_o[g]);
              tp[g] += kFwdGroups;
              ++cp[g];
              progress = true;
            }
            // S = Q.K^T of tile ts: its Q rows have landed, and S of the group's previous tile has been read
            if (ts[g] < ntiles && ts[g] < tp[g] + kFwdGroups && mbar_test(&bar_full[g], cs[g] & 1)) {
              tc_fence_after_sync();
              umma_gemm<D / 16>(tS, q_km, hi, 2, kQB, k_km, hi, 2, kKB, idesc_s, 0);
              umma_commit(&bar_qfree[g]);   // the loaders may refill the Q tile
              umma_commit(&bar_s[g]);
              ts[g] += kFwdGroups;
              ++cs[g];
              progress = true;
            }
          }
          if (s_open && ts[0] >= ntiles && ts[1] >= ntiles) {   // the item's last S GEMM has been issued
            umma_commit(&bar_sfin);
            s_open = false;
          }
          if (progress) idle = 0;
          else if (++idle > (kSpinLimit << 4)) {   // bounded like every other wait
            atomicCAS(p.status, 0, 6);
            ok = false;
          }
        }
        if (ok) umma_commit(&bar_fin);             // the item's last P.V GEMM has been issued
      }
    }
  } else if (warp > kFwdIssuerWarp) {
    // =============================================================== loader warps
    // two independent sets of 64 threads, one per compute group
    const int lt0 = tid - (kFwdIssuerWarp + 1) * 32;
    const int gi = lt0 / kFwdLoaderSet;        // the group this set serves
    const int st = lt0 % kFwdLoaderSet;
    uint32_t m = 0;                            // tiles of this group so far
    bool ok = true;
#pragma unroll 1
    for (uint32_t n = 0; ok; ++n) {
      FwdItem it;
      ok = read_info(n, it);
      ok = bar_and(4 + gi, kFwdLoaderSet, ok);   // the set goes on, or leaves, together
      if (!ok || it.nnz <= 0) break;
      const int ntiles = (it.nnz + kTcM - 1) / kTcM;
      const T* qbase = static_cast<const T*>(p.q) + (int64_t)it.q0 * p.q_rs + (int64_t)it.h * p.q_hs;
      // row id of entry e of a tile (-1 = none): the load only; the range check happens at the use
      auto row_raw = [&](int tile, int e) {
        return (e < kTcM && tile < ntiles && tile * kTcM + e < it.nnz) ? p.ps.indices[it.off + tile * kTcM + e] : -1;
      };
      int r_a = row_raw(gi, st), r_b = row_raw(gi, st + kFwdLoaderSet);   // the set's first tile of the item
#pragma unroll 1
      for (int i = gi; i < ntiles; i += kFwdGroups, ++m) {
        int* rows = sRow[gi][m & 1];
        if (m > 0) {   // the group's previous S GEMM must have finished reading its Q tile; it is
                       // issued after the softmax of the tile before, the last reader of rows[]
          ok = mbar_wait(&bar_qfree[gi], (m - 1) & 1, p.status, 5);
        }
        rows[st] = (r_a < 0 || r_a >= it.len_q) ? -1 : r_a;
        if (st + kFwdLoaderSet < kTcM) rows[st + kFwdLoaderSet] = (r_b < 0 || r_b >= it.len_q) ? -1 : r_b;
        r_a = row_raw(i + kFwdGroups, st);                  // next tile's row ids, in flight meanwhile
        r_b = row_raw(i + kFwdGroups, st + kFwdLoaderSet);
        ok = bar_and(4 + gi, kFwdLoaderSet, ok);   // also publishes the row ids inside the set
        if (!ok) break;
        gather_cp_async<T, D / 8, kFwdLoaderSet>(st, sQg + gi * (kTcM * D * 2), kQBlock, qbase, p.q_rs, rows);
        cp_async_wait_all();
        fence_async_smem();   // the copies are generic-proxy writes; the MMAs read through the async proxy
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar_full[gi]);
      }
    }
  } else {
    // =============================================================== compute groups
    const int g = tid / kFwdGroupThreads;      // compute group
    const int gt = tid % kFwdGroupThreads;     // thread inside the group
    const int lt = tid & (kTcM - 1);           // row (TMEM lane)
    const int hf = (gt >> 7) & 1;              // column half
    const int gw = gt >> 5;                    // warp inside the group (0..7)
    unsigned char* sPO = sPOg + g * (kTcM * QP * 2);
    const uint32_t tS = tmem_base + g * 256, tO = tS + 128;
    const uint32_t lane_sel = (uint32_t)((warp & 3) * 32) << 16;
    T* part_o = static_cast<T*>(p.part_o);
    const int bar_id = 2 + g;
    bool good = true;
    uint32_t m = 0;                            // tiles of this group so far

#pragma unroll 1
    for (uint32_t n = 0; good; ++n) {
      FwdItem it;
      good = read_info(n, it);
      good = bar_and(bar_id, kFwdGroupThreads, good);   // the group goes on, or leaves, together
      if (!good || it.nnz <= 0) break;
      const int ntiles = (it.nnz + kTcM - 1) / kTcM;
#pragma unroll 1
      for (int i = g; i < ntiles; i += kFwdGroups, ++m) {
        const int t0 = i * kTcM;
        const int rows = min(kTcM, it.nnz - t0);
        if (gw < 4 && lane == 0) bulk_wait_read();   // the previous tile's O staging has been read out
        if (good) good = mbar_wait(&bar_s[g], m & 1, p.status, 1);   // on failure: run on to the barrier
        tc_fence_after_sync();

        // ---- chunk-local softmax of row `lt`, this thread's half of the keys
        const int r = sRow[g][m & 1][lt];
        const int lim = r < 0 ? 0 : (p.causal ? min(it.keys_valid, r + it.shift - it.key0 + 1) : it.keys_valid);
        // two passes over the row's scores in TMEM (maximum, then exponentials), 32 at a time: keeps
        // the thread at 32 live scores, which is what the register budget of 22 warps allows
        float mx = -CUDART_INF_F;
#pragma unroll
        for (int q4 = 0; q4 < CH / 32; ++q4) {
          float s[32];
          tmem_ld32(tS + lane_sel + hf * CH + q4 * 32, s);
          tmem_ld_wait();
          if (lim >= C) {   // nothing masked: the common case away from the causal diagonal
#pragma unroll
            for (int jj = 0; jj < 32; ++jj) mx = fmaxf(mx, s[jj]);
          } else {
#pragma unroll
            for (int jj = 0; jj < 32; ++jj) mx = fmaxf(mx, hf * CH + q4 * 32 + jj < lim ? s[jj] : -CUDART_INF_F);
          }
        }
        sMax[g][hf][lt] = mx;
        good = bar_and(bar_id, kFwdGroupThreads, good);   // also: the previous bulk reads are done
        if (!good) break;
        mx = fmaxf(mx, sMax[g][hf ^ 1][lt]);
        const float mref = lim > 0 ? mx * scale_log2 : 0.f;
        float sum = 0.f;
#pragma unroll
        for (int q4 = 0; q4 < CH / 32; ++q4) {
          float s[32];
          tmem_ld32(tS + lane_sel + hf * CH + q4 * 32, s);
          tmem_ld_wait();
          if (lim >= C) {
#pragma unroll
            for (int jj = 0; jj < 32; ++jj) {
              s[jj] = exp2f(s[jj] * scale_log2 - mref);
              sum += s[jj];
            }
          } else {
#pragma unroll
            for (int jj = 0; jj < 32; ++jj) {
              const float e = exp2f(s[jj] * scale_log2 - mref);
              s[jj] = (hf * CH + q4 * 32 + jj < lim) ? e : 0.f;
              sum += s[jj];
            }
          }
#pragma unroll
          for (int jj = 0; jj < 4; ++jj)
            *reinterpret_cast<uint4*>(sPO + sw128_offset(lt, hf * (CH / 8) + q4 * 4 + jj, kQBlock)) = pack8<T>(s + jj * 8);
        }
        tc_fence_before_sync();
        sSum[g][hf][lt] = sum;
        fence_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar_pready[g]);   // S has been read, P is in shared memory
        bar_sync(bar_id, kFwdGroupThreads);           // the other half's sum
        sum += sSum[g][hf ^ 1][lt];
        const float inv = sum > 0.f ? 1.f / sum : 0.f;
        if (hf == 0 && lt < rows) p.part_lse[it.slot + t0 + lt] = sum > 0.f ? mx * p.scale + logf(sum) : -CUDART_INF_F;
        if (good) good = mbar_wait(&bar_o[g], m & 1, p.status, 2);
        tc_fence_after_sync();

        // ---- epilogue: normalised partial O of row `lt`, this thread's half of the head dim,
        // staged in the P tile (its MMAs have completed); one bulk copy per 32 rows
        {
          const int key = (int)((it.slot + t0 + lt) & 7);
          unsigned char* srow = sPO + lt * (D * 2);
          float o[DH];
#pragma unroll
          for (int q4 = 0; q4 < DH / 32; ++q4) tmem_ld32(tO + lane_sel + hf * DH + q4 * 32, o + q4 * 32);
          tmem_ld_wait();
#pragma unroll
          for (int jj = 0; jj < DH; ++jj) o[jj] *= inv;
#pragma unroll
          for (int jj = 0; jj < DH / 8; ++jj)
            *reinterpret_cast<uint4*>(srow + (((hf * (DH / 8) + jj) ^ key) << 4)) = pack8<T>(o + jj * 8);
          tc_fence_before_sync();
          fence_async_smem();
        }
        good = bar_and(bar_id, kFwdGroupThreads, good);   // both halves of every row staged
        if (!good) break;
        if (gw < 4) {
          const int wrows = min(32, rows - gw * 32);   // a warp's rows are contiguous in the workspace
          if (lane == 0 && wrows > 0) {
            bulk_store(part_o + (it.slot + t0 + gw * 32) * D, sPO + gw * 32 * (D * 2), (uint32_t)wrows * D * 2);
            bulk_commit();   // its reads are waited for before the next tile's P is stored
          }
        }
      }
    }
    if (gw < 4 && lane == 0) bulk_wait_read();
  }
  tc_fence_before_sync();
  __syncthreads();         // every role is done with its tiles, barriers and TMEM columns
  tc_fence_after_sync();
  if (warp == 0) tmem_dealloc(tmem_base, NCOLS);
}


// ======================================================================== backward
// Work item = key block c of (sequence b, kv head hk); 512 threads, warp-specialised, one
// persistent CTA per SM that runs through its work items as ONE stream of 128-row tiles:
//   warps 0-7   compute.  TMEM lane = gathered query row (at the end: key); warps w and w+4 share
//               a lane quarter and split the columns in halves.  They issue no global loads.
//   warp 8      one thread issues every MMA; it alone waits for operand tiles, so a late gather
//               never stalls a compute warp that still has work.
//   warps 9-10  Q loader, warps 11-14 dO loader: 16-byte cp.async copies of the tile's rows
//               straight into the swizzled UMMA tiles (no registers; measured ~4x the throughput
//               of loads into registers, and ~3.5x that of TMA tile::gather4 row gathers for these
//               isolated 256-byte rows).  Q is double buffered (its loader has two tiles of slack);
//               dO is refilled as soon as the dV GEMM of the previous tile has completed.  Ahead of
//               the dO tile its loader leaves the rows' query positions, log-sum-exps, dO.O sums
//               and the tile's slot range in shared memory for the compute warps.
//   warp 15     scout: decodes item n + 1 (geometry, first tile: a chain of dependent global
//               loads) while item n runs and publishes it in a shared-memory ring; stages an
//               item's K and V tiles as soon as every GEMM of the item before it has completed.
// An item's tiles are the q heads of the kv head's group and the 128-row tiles of each head's CSC
// column.  Per tile, five GEMMs:
//     S  = Q.K^T          dP = dO.V^T                       (both K-major operands)
//     dV += P^T.dO        dK += dS^T.Q   (A and B consumed MN-major from the row-major tiles)
//     dQ_partial = dS.K   (K consumed MN-major)             -> workspace at the entry's slot
// dK and dV stay in TMEM (fp32) for the whole item: no atomics, no cross-head reduction pass; they
// are written out while the next item's first GEMMs run.  TMEM columns: [0,C) S, [C,2C) dP then
// dQ, [2C,2C+D) dV, [2C+D,2C+2D) dK.
//
// All hand-offs are mbarriers, initialised once; their phases are counted over the stream.  Per
// tile g (the tensor pipe executes the GEMMs in issue order):
//   compute:  wait S(g)  -> P = exp2(S.scale.log2e - LSE.log2e) -> shared (bf16) + registers      -> P_ready
//             wait dP(g) -> dS = P.(dP - D) -> shared (bf16)                                        -> dS_ready
//             wait dQ(g) -> dQ partial: TMEM -> registers -> staging -> global (scaled, I/O dtype)  -> dQ_free
//   issuer:   P_ready(g)  -> dV(g) [its completion frees dO and P], S(g+1) once Q(g+1) has landed
//             dS_ready(g) -> dQ(g) over dP's columns, dK(g) [its completion frees this Q buffer]
//             dO(g+1) landed and dQ_free(g) -> dP(g+1)
//   at an item's end the issuer commits "item finished"; the scout then loads the next K, V, the
//   compute warps read dK, dV out of TMEM.
constexpr int kBwdCompute = 256;
// Loader warps.  Measured at 64K tokens (backward main kernel, before the item stream): 1 + 2 warps
// 5.14 ms, 2 + 2 warps 4.98 ms, 2 + 4 warps 4.63 ms, 1 + 4 warps 5.2 ms: the gathers are latency
// bound per warp; with the item stream 3 + 3 warps 4.14 ms against 4.08 ms for 2 + 4.  Sixteen
// warps are the most that keep 128 registers per thread (registers are allocated to warps in
// groups of four: a seventeenth warp would bring the limit down to 96).
constexpr int kBwdQLoaders = 32 * 2;          // threads gathering Q rows
constexpr int kBwdOLoaders = 32 * 4;          // threads gathering dO rows
constexpr int kBwdScoutWarp = (kBwdCompute + 32 + kBwdQLoaders + kBwdOLoaders) / 32;   // K/V loader and item scout
constexpr int kBwdThreads = kBwdCompute + 32 + kBwdQLoaders + kBwdOLoaders + 32;

struct BwdTile {
  int hg;        // head within the group
  int t0;        // first entry of the tile inside the head's column
  int nnz;       // entries of the head's column
  int64_t off;   // the column's first entry in `indices`
  int64_t slot;  // the column's first slot in the pass
};

// first head >= it.hg of the kv head's group whose column of key block c is not empty
__device__ __forceinline__ bool bwd_seek_head(const PassParams& ps, int b, int hk, int group, int c, BwdTile& it) {
  for (; it.hg < group; ++it.hg) {
    const ColRef col = column_of(ps, b, hk * group + it.hg, c);
    if (col.nnz > 0) {
      it.nnz = col.nnz; it.off = col.off; it.slot = col.slot; it.t0 = 0;
      return true;
    }
  }
  it.hg = group;
  return false;
}
__device__ __forceinline__ bool bwd_next_tile(const PassParams& ps, int b, int hk, int group, int c, BwdTile& it) {
  it.t0 += kTcM;
  if (it.t0 < it.nnz) return true;
  ++it.hg;
  return bwd_seek_head(ps, b, hk, group, c, it);
}

// One work item's geometry, derived by every role from the item number alone
struct BwdItem {
  int c, hk, b, q0, len_q, k0, len_k, key0, keys_valid, shift;
  int64_t plane;
  bool skip;       // the key block starts past the sequence's last key
};
__device__ __forceinline__ void bwd_decode_item(const TcParams& p, int item, int group, BwdItem& I) {
  int bx, rem;
  decode_item(p, item, bx, rem);
  const int sb = bx % p.ps.nsub;
  I.c = bx / p.ps.nsub;
  I.hk = p.ps.h0 / group + rem % p.items_y;
  I.b = rem / p.items_y;
  I.plane = (int64_t)sb * p.ps.cap;
  I.q0 = p.cu_q[I.b];
  I.len_q = p.cu_q[I.b + 1] - I.q0;
  I.k0 = p.k_begin[I.b];
  I.len_k = p.k_end[I.b] - I.k0;
  // The kernel always works on 128 key lanes; with 64-key blocks (chunks that are not a multiple of
  // 128) the upper 64 lanes are zero-filled and masked: twice the tensor work per key, still several
  // times faster than the CUDA-core backward, and the tensor pipe is mostly idle anyway.
  I.key0 = I.c * p.ps.chunk + sb * p.ps.kb;
  I.skip = I.key0 >= I.len_k;
  I.keys_valid = min(p.ps.kb, I.len_k - I.key0);
  I.shift = I.len_k - I.len_q;
}

template <typename T, int C, int D>
__global__ void __launch_bounds__(kBwdThreads) bwd_main_tc_kernel(TcParams p, const __grid_constant__ CUtensorMap map_k,
                                                                  const __grid_constant__ CUtensorMap map_v) {
  static_assert(C == 128, "tensor-core backward keeps one key per TMEM lane");
  constexpr uint32_t kKBlock = C * 128;
  constexpr uint32_t kQBlock = kTcM * 128;
  constexpr uint32_t kQTile = kTcM * D * 2;
  constexpr int NCOLS = 512;
  constexpr int DH = D / 2;                       // head-dim columns per thread in the epilogues
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  __shared__ uint64_t bar_s, bar_p, bar_dq, bar_dv, bar_fin, bar_fulldo, bar_dk[2], bar_fullq[2];
  __shared__ uint64_t bar_pready, bar_dsready, bar_dqfree, bar_kv, bar_rows, bar_item[4];
  __shared__ float sLse[kTcM], sDsum[kTcM];        // log-sum-exp and dO.O of the rows of the dO tile
  __shared__ int s_tile[4];                       // that tile's valid rows, first slot (64 bit), "another tile follows"
  __shared__ uint32_t tmem_base_s;
  __shared__ uint64_t bar_info[4];
  __shared__ int s_items[4];                      // ring of work items, fetched two ahead
  __shared__ int s_info[4][20];                   // ring of decoded work items (geometry, first tile)
  __shared__ int s_prev[4];                       // key row, kv head, valid keys of the item whose dK / dV are in TMEM
  __shared__ int sRowQ[kTcM], sRowO[kTcM];        // row ids of the tile a loader group is fetching

  // the swizzled tiles need a 1024-byte aligned base; static and dynamic shared memory together use
  // the whole 227 KB, so there is no room for padding: checked here, reported through the status word
  unsigned char* smem = smem_raw;
  if ((smem_u32(smem_raw) & 1023u) != 0) {
    if (threadIdx.x == 0) atomicCAS(p.status, 0, 9);
    return;
  }
  unsigned char* sK = smem;                       // [C][D]
  unsigned char* sV = sK + C * D * 2;             // [C][D]
  unsigned char* sQ = sV + C * D * 2;             // 2 x [128][D]
  unsigned char* sdO = sQ + 2 * kQTile;           // [128][D]
  unsigned char* sP = sdO + kQTile;               // [128][C]
  unsigned char* sdS = sP + kTcM * C * 2;         // [128][C]

  const int group = p.heads / p.heads_k;
  const float scale_log2 = p.scale * kLog2eTc;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int lt = tid & (kTcM - 1);                // row (TMEM lane) of a compute thread
  const int hf = (tid >> 7) & 1;                  // column half of a compute thread

  if (warp == 0) tmem_alloc(&tmem_base_s, NCOLS);
  if (tid == 0) {
    mbar_init(&bar_s, 1); mbar_init(&bar_p, 1); mbar_init(&bar_dq, 1); mbar_init(&bar_dv, 1); mbar_init(&bar_fin, 1);
    mbar_init(&bar_dk[0], 1); mbar_init(&bar_dk[1], 1);
    mbar_init(&bar_fullq[0], kBwdQLoaders / 32); mbar_init(&bar_fullq[1], kBwdQLoaders / 32);
    mbar_init(&bar_fulldo, kBwdOLoaders / 32);   // one arrival per loader warp
    mbar_init(&bar_pready, kBwdCompute / 32); mbar_init(&bar_dsready, kBwdCompute / 32);
    mbar_init(&bar_dqfree, kBwdCompute / 32);   // one arrival per compute warp
    mbar_init(&bar_kv, 1);
    mbar_init(&bar_rows, kBwdOLoaders / 32);
#pragma unroll
    for (int k = 0; k < 4; ++k) { mbar_init(&bar_item[k], 1); mbar_init(&bar_info[k], 1); }
    mbar_fence_init();
    s_items[0] = atomicAdd(p.work, 1);
    s_items[1] = atomicAdd(p.work, 1);
    mbar_arrive(&bar_item[0]);
    mbar_arrive(&bar_item[1]);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_base_s;
  const uint32_t tS = tmem_base, tdP = tmem_base + C, tdV = tmem_base + 2 * C, tdK = tmem_base + 2 * C + D;
  const uint32_t tdQ = tdP;

  // The CTA is persistent and its roles run through the work items as ONE stream of tiles: no
  // role waits for another at an item boundary except through the data it needs.  Every barrier
  // is initialised once; phases are counted with stream-wide counters (n: items, nk: items with
  // keys, g / m: tiles) that every role advances in the same way.
  // n-th item of this CTA (p.n_items or more: the counter has run out); read by the scout warp only
  auto get_item = [&](uint32_t n, int& item) -> bool {
    if (!mbar_wait(&bar_item[n & 3], (n >> 2) & 1, p.status, 8)) {
      item = p.n_items;
      return false;
    }
    item = *reinterpret_cast<volatile int*>(&s_items[n & 3]);
    return true;
  };
  // The scout warp decodes every item ahead of the other roles (the geometry and the first tile
  // cost a chain of three dependent global loads) and publishes it in s_info.
  // state: 0 = the stream has ended, 1 = item with tiles or keys, 2 = key block past the sequence's end
  auto read_info = [&](uint32_t n, BwdItem& I, BwdTile& it, bool& have) -> int {
    if (!mbar_wait(&bar_info[n & 3], (n >> 2) & 1, p.status, 8)) return -1;
    const volatile int* f = s_info[n & 3];
    const int state = f[0];
    I.c = f[1]; I.hk = f[2]; I.b = f[3]; I.q0 = f[4]; I.len_q = f[5]; I.k0 = f[6]; I.len_k = f[7];
    I.key0 = f[8]; I.keys_valid = f[9]; I.shift = f[10]; I.plane = (int64_t)f[11] * p.ps.cap; I.skip = state == 2;
    have = f[12] != 0;
    it.hg = f[13]; it.t0 = 0; it.nnz = f[14];
    it.off = (int64_t)(((uint64_t)(uint32_t)f[16] << 32) | (uint32_t)f[15]);
    it.slot = (int64_t)(((uint64_t)(uint32_t)f[18] << 32) | (uint32_t)f[17]);
    return state;
  };
  // ---- an item's tile sequence
  auto seek_head = [&](const BwdItem& I, BwdTile& it) { return bwd_seek_head(p.ps, I.b, I.hk, group, I.c, it); };
  auto next_tile = [&](const BwdItem& I, BwdTile& it) { return bwd_next_tile(p.ps, I.b, I.hk, group, I.c, it); };
  // sequence-local query row of entry i of the tile (-1 = none).  row_raw() only issues the load;
  // row_checked() is applied where the value is used, so that a prefetch does not wait for it.
  auto row_raw = [&](const BwdTile& it, int i) {
    return (it.t0 + i < it.nnz) ? ldg_s32_here(p.ps.indices + it.off + it.t0 + i) : -1;
  };
  auto row_checked = [&](const BwdItem& I, int r) { return (r < 0 || r >= I.len_q) ? -1 : r; };

  if (warp == 8) {
    // =============================================================== MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc(FmtOf<T>::v, kTcM, C, 0, 0);     // rows x keys
      constexpr uint32_t idesc_kv = make_idesc(FmtOf<T>::v, C, D, 1, 1);       // keys x d, both MN-major
      constexpr uint32_t idesc_dq = make_idesc(FmtOf<T>::v, kTcM, D, 0, 1);    // rows x d
      // descriptor halves of every operand view, built once
      const uint32_t hi = desc_hi_sw128(1024);
      const uint32_t k_km = desc_lo_sw128(smem_u32(sK), 16), v_km = desc_lo_sw128(smem_u32(sV), 16);
      const uint32_t k_mn = desc_lo_sw128(smem_u32(sK), kKBlock);
      const uint32_t q_km = desc_lo_sw128(smem_u32(sQ), 16), q_mn = desc_lo_sw128(smem_u32(sQ), kQBlock);
      const uint32_t do_km = desc_lo_sw128(smem_u32(sdO), 16), do_mn = desc_lo_sw128(smem_u32(sdO), kQBlock);
      const uint32_t p_mn = desc_lo_sw128(smem_u32(sP), kQBlock);
      const uint32_t ds_km = desc_lo_sw128(smem_u32(sdS), 16), ds_mn = desc_lo_sw128(smem_u32(sdS), kQBlock);
      constexpr uint32_t kQBuf = kQTile >> 4;        // second Q buffer, in descriptor address units
      constexpr uint32_t kQB = kQBlock >> 4, kKB = kKBlock >> 4;
      uint32_t g = 0, nk = 0;          // tiles and items with keys so far
      bool ok = true;
      // S(g) = Q(g).K^T once Q(g) has landed; S's columns are free since P_ready(g-1)
      auto issue_s = [&]() {
        if (!(ok = mbar_wait(&bar_fullq[g & 1], (g >> 1) & 1, p.status, 6))) return;
        tc_fence_after_sync();
        umma_gemm<D / 16>(tS, q_km + (g & 1) * kQBuf, hi, 2, kQB, k_km, hi, 2, kKB, idesc_s, 0);
        umma_commit(&bar_s);
      };
      // dP(g) = dO(g).V^T once dO(g) has landed and dQ(g-1) has been read out of these columns
      auto issue_dp = [&]() {
        if (!(ok = mbar_wait(&bar_fulldo, g & 1, p.status, 6))) return;
        if (g > 0 && !(ok = mbar_wait(&bar_dqfree, (g - 1) & 1, p.status, 6))) return;
        tc_fence_after_sync();
        umma_gemm<D / 16>(tdP, do_km, hi, 2, kQB, v_km, hi, 2, kKB, idesc_s, 0);
        umma_commit(&bar_p);
      };
#pragma unroll 1
      for (uint32_t n = 0; ok; ++n) {
        BwdItem I;
        BwdTile it;
        bool have;
        const int state = read_info(n, I, it, have);
        if (state < 0) ok = false;
        if (state <= 0) break;
        if (I.skip) continue;
        // K and V of this item are in place (the scout warp loads them once every GEMM of the
        // previous item has completed)
        if (!(ok = mbar_wait(&bar_kv, nk & 1, p.status, 6))) break;
        if (have) {
          issue_s();
          if (ok) issue_dp();
          uint32_t acc = 0;
#pragma unroll 1
          while (ok) {
            const bool more = next_tile(I, it);
            // dV += P^T.dO : M = keys, N = d, K = the 128 gathered rows
            if (!(ok = mbar_wait(&bar_pready, g & 1, p.status, 1))) break;
            tc_fence_after_sync();
            umma_gemm<kTcM / 16>(tdV, p_mn, hi, 128, 512, do_mn, hi, 128, 512, idesc_kv, acc);
            umma_commit(&bar_dv);        // dO is free once this completes: the dO loader's signal
            if (!(ok = mbar_wait(&bar_dsready, g & 1, p.status, 2))) break;
            tc_fence_after_sync();
            // dQ partial = dS.K : M = rows, N = d, K = keys
            umma_gemm<C / 16>(tdQ, ds_km, hi, 2, kQB, k_mn, hi, 128, 512, idesc_dq, 0);
            umma_commit(&bar_dq);
            // dK += dS^T.Q
            umma_gemm<kTcM / 16>(tdK, ds_mn, hi, 128, 512, q_mn + (g & 1) * kQBuf, hi, 128, 512, idesc_kv, acc);
            umma_commit(&bar_dk[g & 1]); // this Q buffer is free once it completes: the Q loader's signal
            ++g;
            acc = 1;
            if (!more) break;
            issue_s();
            if (ok) issue_dp();
          }
        }
        if (ok) umma_commit(&bar_fin);   // every GEMM of the item has completed: K, V, dK, dV may be reused
        ++nk;
      }
    }
  } else if (warp == kBwdScoutWarp) {
    // =============================================================== scout: items and K / V tiles
    // Decodes item n + 1 and publishes it while item n is being worked on, and loads an item's K
    // and V tiles as soon as every GEMM of the item before it has completed.
    BwdItem I;
    BwdTile it{0, 0, 0, 0, 0};
    bool ok = true;
    // returns 1 if item n exists (I, it describe it), 0 at the end of the stream
    auto scout_item = [&](uint32_t n) -> int {
      int item;
      if (!get_item(n, item)) { ok = false; return 0; }
      int state = 0, have = 0;
      it = BwdTile{0, 0, 0, 0, 0};
      I.skip = true;
      if (item < p.n_items) {
        bwd_decode_item(p, item, group, I);
        state = I.skip ? 2 : 1;
        if (!I.skip) have = seek_head(I, it) ? 1 : 0;
      }
      if (lane == 0) {
        volatile int* f = s_info[n & 3];
        f[1] = I.c; f[2] = I.hk; f[3] = I.b; f[4] = I.q0; f[5] = I.len_q; f[6] = I.k0; f[7] = I.len_k;
        f[8] = I.key0; f[9] = I.keys_valid; f[10] = I.shift; f[11] = (int)(p.ps.cap ? I.plane / p.ps.cap : 0);
        f[12] = have; f[13] = it.hg; f[14] = it.nnz;
        f[15] = (int)(uint32_t)((uint64_t)it.off & 0xffffffffu); f[16] = (int)(uint32_t)((uint64_t)it.off >> 32);
        f[17] = (int)(uint32_t)((uint64_t)it.slot & 0xffffffffu); f[18] = (int)(uint32_t)((uint64_t)it.slot >> 32);
        f[0] = state;
        mbar_arrive(&bar_info[n & 3]);
      }
      return state != 0;
    };
    int more = scout_item(0);
    uint32_t nk = 0;                 // items with keys so far
#pragma unroll 1
    for (uint32_t n = 0; more && ok; ++n) {
      const bool skip = I.skip;
      if (!skip) {
        const T* kbase = static_cast<const T*>(p.k) + (int64_t)(I.k0 + I.key0) * p.k_rs + (int64_t)I.hk * p.k_hs;
        const T* vbase = static_cast<const T*>(p.v) + (int64_t)(I.k0 + I.key0) * p.v_rs + (int64_t)I.hk * p.v_hs;
        if (p.kv_tma && I.keys_valid == C) {   // warp-uniform
          if (lane == 0) {
            tma_stage_block<C, D>(sK, &map_k, (int64_t)I.hk * p.k_hs, I.k0 + I.key0, &bar_kv, 2 * C * D * 2);
            tma_stage_block<C, D>(sV, &map_v, (int64_t)I.hk * p.v_hs, I.k0 + I.key0, &bar_kv, 0);
          }
        } else {
          dense_cp_async<T, D / 8, C, 32>(lane, sK, kKBlock, kbase, p.k_rs, I.keys_valid);
          dense_cp_async<T, D / 8, C, 32>(lane, sV, kKBlock, vbase, p.v_rs, I.keys_valid);
          cp_async_wait_all();
          fence_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(&bar_kv);
        }
      }
      more = scout_item(n + 1);
      if (!skip) {                   // every GEMM of item n has completed: its K and V tiles are free
        if (ok) ok = mbar_wait(&bar_fin, nk & 1, p.status, 8);
        ++nk;
      }
    }
  } else if (warp >= 9) {
    // =============================================================== loader warps
    const bool q_side = warp < 9 + kBwdQLoaders / 32;
    const int nt = q_side ? kBwdQLoaders : kBwdOLoaders;
    const int t = q_side ? tid - (kBwdCompute + 32) : tid - (kBwdCompute + 32 + kBwdQLoaders);
    int* sRow = q_side ? sRowQ : sRowO;
    const int bar_id = q_side ? 3 : 4;
    uint32_t m = 0;                  // tiles so far
    bool ok = true;
#pragma unroll 1
    for (uint32_t n = 0; ok; ++n) {
      BwdItem I;
      BwdTile it;
      bool have;
      const int state = read_info(n, I, it, have);
      ok = bar_and(bar_id, nt, state >= 0);  // the group goes on, or leaves, together
      if (!ok || state == 0) break;
      if (I.skip) continue;
#pragma unroll 1
      for (; have; ++m) {
        // the tile's row ids, fetched before the wait for the buffer
        int rid[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) rid[k] = (t + k * nt < kTcM) ? row_checked(I, row_raw(it, t + k * nt)) : -1;
        const int h = I.hk * group + it.hg;
        BwdTile nx = it;
        const bool more = next_tile(I, nx);
        if (q_side) {
          if (m >= 2) ok = mbar_wait(&bar_dk[m & 1], ((m >> 1) - 1) & 1, p.status, 5);   // dK(m-2) has read Q
        } else {
          // What the compute warps need to know about the tile's rows (so that they issue no global
          // loads of their own) goes ahead of the tile: it may be written as soon as they have copied
          // the previous tile's values to registers, which they do before P_ready.
          if (m >= 1) ok = mbar_wait(&bar_pready, (m - 1) & 1, p.status, 5);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            if (t + k * nt < kTcM) {
              float l = CUDART_INF_F, dd = 0.f;
              if (rid[k] >= 0) {
                const int64_t at = (int64_t)h * p.total_q + I.q0 + rid[k];
                l = p.lse[at];
                dd = p.softmax_d[at];
              }
              sRow[t + k * nt] = rid[k];
              sLse[t + k * nt] = l;
              sDsum[t + k * nt] = dd;
            }
          }
          if (t == 0) {
            const int64_t slot = it.slot + it.t0;
            s_tile[0] = min(kTcM, it.nnz - it.t0);
            s_tile[1] = (int)(uint32_t)((uint64_t)slot & 0xffffffffu);
            s_tile[2] = (int)(uint32_t)((uint64_t)slot >> 32);
            s_tile[3] = more ? 1 : 0;
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(&bar_rows);
          if (ok && m >= 1) ok = mbar_wait(&bar_dv, (m - 1) & 1, p.status, 5);           // dV(m-1) has read dO
        }
        if (q_side) {
#pragma unroll
          for (int k = 0; k < 4; ++k)
            if (t + k * nt < kTcM) sRow[t + k * nt] = rid[k];
        }
        ok = bar_and(bar_id, nt, ok);                // also publishes the row ids to the group
        if (!ok) break;
        if (q_side) {
          const T* qbase = static_cast<const T*>(p.q) + (int64_t)I.q0 * p.q_rs + (int64_t)h * p.q_hs;
          gather_cp_async<T, D / 8, kBwdQLoaders>(t, sQ + (m & 1) * kQTile, kQBlock, qbase, p.q_rs, sRow);
        } else {
          const T* dobase = static_cast<const T*>(p.dout) + (int64_t)I.q0 * p.do_rs + (int64_t)h * p.do_hs;
          gather_cp_async<T, D / 8, kBwdOLoaders>(t, sdO, kQBlock, dobase, p.do_rs, sRow);
        }
        cp_async_wait_all();
        fence_async_smem();        // the copies are generic-proxy writes; the MMAs read through the async proxy
        __syncwarp();
        if (lane == 0) mbar_arrive(q_side ? &bar_fullq[m & 1] : &bar_fulldo);
        bar_sync(bar_id, nt);                        // every thread has read the row ids
        it = nx;
        have = more;
      }
    }
  } else {
    // =============================================================== compute warps
    const uint32_t lane_sel = (uint32_t)((warp & 3) * 32) << 16;
    T* part_dq = static_cast<T*>(p.part_o);
    bool good = true;
    uint32_t g = 0, nk = 0;          // tiles and items with keys so far
    // the item whose dK / dV are still in TMEM
    bool prev = false, prev_any = false;

#pragma unroll 1
    for (uint32_t n = 0;; ++n) {
      BwdItem I;
      BwdTile it;
      bool have;
      const int state = read_info(n, I, it, have);
      good = bar_and(2, kBwdCompute, good && state >= 0);
      const bool done = !good || state == 0;
      int fetched = 0;
      if (tid == 0 && !done) fetched = atomicAdd(p.work, 1);      // item n + 2, published below
      const bool run = !done && !I.skip;
      have = have && run;

      // ---- the previous item's GEMMs have completed: its dK and dV are final
      if (prev) {
        if (warp < 4) bulk_wait_read();
        if (good) good = mbar_wait(&bar_fin, (nk - 1) & 1, p.status, 4);
        good = bar_and(2, kBwdCompute, good);
        tc_fence_after_sync();
      }
      // ---- dK and dV of key `lt` of the previous item, this thread's half of the head dim: staged in
      // the P / dS tiles (free between items) with rows 16 bytes apart from a multiple of 128, which
      // keeps the 16-byte stores of a warp off each other's banks, then one bulk copy per key row.
      // dK first, then dV through the same staging area.
      if (prev && good) {
        // (written by thread 0 after the item's last tile; the barrier at the top of this iteration orders the read)
        const int64_t prev_row = s_prev[0];
        const int prev_hk = s_prev[1], prev_keys = s_prev[2];
        constexpr int kPitch = D * 2 + 16;
        static_assert(kTcM * kPitch <= 2 * kTcM * C * 2, "staging area = the P and dS tiles");
        unsigned char* srow = sP + lt * kPitch;
#pragma unroll
        for (int which = 0; which < 2; ++which) {
          if (which == 1) {            // the dK rows have been read out of the staging area
            if (hf == 0) bulk_wait_read();
            good = bar_and(2, kBwdCompute, good);
          }
#pragma unroll
          for (int i2 = 0; i2 < DH / 32; ++i2) {
            float o[32];
            if (prev_any) {
              tmem_ld32((which == 0 ? tdK : tdV) + lane_sel + hf * DH + i2 * 32, o);
              tmem_ld_wait();
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) o[j] = 0.f;
            }
            if (which == 0) {
#pragma unroll
              for (int j = 0; j < 32; ++j) o[j] *= p.scale;
            }
#pragma unroll
            for (int j = 0; j < 4; ++j)
              *reinterpret_cast<uint4*>(srow + (hf * DH + i2 * 32 + j * 8) * 2) = pack8<T>(o + j * 8);
          }
          fence_async_smem();
          good = bar_and(2, kBwdCompute, good);   // both halves of every row staged
          if (good && hf == 0 && lt < prev_keys) {
            T* dst = which == 0
                         ? static_cast<T*>(p.dk) + (prev_row + lt) * p.dk_rs + (int64_t)prev_hk * p.dk_hs
                         : static_cast<T*>(p.dv) + (prev_row + lt) * p.dv_rs + (int64_t)prev_hk * p.dv_hs;
            bulk_store(dst, srow, D * 2);
            bulk_commit();
          }
        }
        tc_fence_before_sync();
      }
      if (tid == 0 && !done) {
        *reinterpret_cast<volatile int*>(&s_items[(n + 2) & 3]) = fetched;
        mbar_arrive(&bar_item[(n + 2) & 3]);
      }
      prev = false;
      prev_any = false;
      if (done) break;
      if (I.skip) {
        zero_dq_partials_by<T>(p.ps, part_dq, I.plane, I.b, I.hk, group, I.c, D, tid, kBwdCompute);
        continue;
      }

      // The compute warps issue no global loads inside an item: the dO loader leaves the rows' query
      // positions, log-sum-exps and dO.O sums and the tile's slot range in shared memory.
      bool more = have;
#pragma unroll 1
      for (; more && good; ++g) {
        // ---- P of row `lt`, this thread's 64 keys
        if (good) good = mbar_wait(&bar_s, g & 1, p.status, 3);   // on failure: run on to the barriers, leave there
        if (good) good = mbar_wait(&bar_rows, g & 1, p.status, 3);   // row data of the tile (long landed)
        tc_fence_after_sync();
        const int r_cur = sRowO[lt];
        const float lse2 = sLse[lt] * kLog2eTc, dd_cur = sDsum[lt];
        const int rows = s_tile[0];
        const int64_t slot0 = (int64_t)(((uint64_t)(uint32_t)s_tile[2] << 32) | (uint32_t)s_tile[1]);
        more = s_tile[3] != 0;
        const int lim = r_cur < 0 ? 0 : (p.causal ? min(I.keys_valid, r_cur + I.shift - I.key0 + 1) : I.keys_valid);
        // P is kept as the rounded values the dV GEMM uses (32 registers instead of 64 fp32): the
        // registers saved let the CTA run more loader warps without spilling
        uint4 pp[8];
#pragma unroll
        for (int i2 = 0; i2 < 2; ++i2) {
          const int col0 = hf * 64 + i2 * 32;
          float pr[32];
          tmem_ld32(tS + lane_sel + col0, pr);
          tmem_ld_wait();
          if (i2 == 1) tc_fence_before_sync();
#pragma unroll
          for (int jj = 0; jj < 32; ++jj) pr[jj] = (col0 + jj < lim) ? exp2f(pr[jj] * scale_log2 - lse2) : 0.f;
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) pp[i2 * 4 + jj] = pack8<T>(pr + jj * 8);
          if (i2 == 0) {               // the previous tile's dQ staging / the dK, dV staging has been read out
            if (warp < 4) bulk_wait_read();
            good = bar_and(2, kBwdCompute, good);
          }
#pragma unroll
          for (int jj = 0; jj < 4; ++jj)
            *reinterpret_cast<uint4*>(sP + sw128_offset(lt, col0 / 8 + jj, kQBlock)) = pp[i2 * 4 + jj];
        }
        tc_fence_before_sync();
        fence_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar_pready);      // S has been read, P is in shared memory

        // ---- dS
        if (good) good = mbar_wait(&bar_p, g & 1, p.status, 3);
        tc_fence_after_sync();
#pragma unroll
        for (int i2 = 0; i2 < 2; ++i2) {
          const int col0 = hf * 64 + i2 * 32;
          float dp[32];
          tmem_ld32(tdP + lane_sel + col0, dp);
          tmem_ld_wait();
#pragma unroll
          for (int j8 = 0; j8 < 4; ++j8) {
            float pf[8];
            unpack8<T>(pp[i2 * 4 + j8], pf);
#pragma unroll
            for (int e = 0; e < 8; ++e) dp[j8 * 8 + e] = pf[e] * (dp[j8 * 8 + e] - dd_cur);
          }
#pragma unroll
          for (int jj = 0; jj < 4; ++jj)
            *reinterpret_cast<uint4*>(sdS + sw128_offset(lt, col0 / 8 + jj, kQBlock)) = pack8<T>(dp + jj * 8);
        }
        tc_fence_before_sync();
        fence_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar_dsready);     // dP has been read, dS is in shared memory

        // ---- dQ partial of row `lt`, this thread's half of the head dim: scaled, rounded to the I/O
        // dtype, stored at the entry's slot (16-byte chunks permuted like the forward partials)
        if (good) good = mbar_wait(&bar_dq, g & 1, p.status, 4);
        tc_fence_after_sync();
        {
          // staged in the P tile (free: dV(g) completed before dQ(g)), 16-byte chunks permuted like the
          // forward partials; one bulk copy per 32 rows, whose reads are waited for before the next P
          // is stored.  32 columns at a time keep the register footprint small.
          constexpr int NCH = DH / 8;               // 16-byte chunks of this thread's half row
          const int key = (int)((slot0 + lt) & 7);
          unsigned char* srow = sP + lt * (D * 2);
#pragma unroll
          for (int i2 = 0; i2 < DH / 32; ++i2) {
            float o[32];
            tmem_ld32(tdQ + lane_sel + hf * DH + i2 * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
#pragma unroll
              for (int e = 0; e < 8; ++e) o[jj * 8 + e] *= p.scale;
              *reinterpret_cast<uint4*>(srow + (((hf * NCH + i2 * 4 + jj) ^ key) << 4)) = pack8<T>(o + jj * 8);
            }
          }
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&bar_dqfree);    // dQ has been read out of dP's columns
          fence_async_smem();
          good = bar_and(2, kBwdCompute, good);     // both halves of every row staged
          if (good && warp < 4 && lane == 0) {
            const int wrows = min(32, rows - warp * 32);
            if (wrows > 0) {
              bulk_store(part_dq + (I.plane + slot0 + warp * 32) * D, sP + warp * 32 * (D * 2),
                         (uint32_t)wrows * D * 2);
              bulk_commit();
            }
          }
        }
        prev_any = true;
      }
      prev = true;
      if (tid == 0) { s_prev[0] = I.k0 + I.key0; s_prev[1] = I.hk; s_prev[2] = I.keys_valid; }
      ++nk;
    }
    if (warp < 4) bulk_wait_read();
  }
  tc_fence_before_sync();
  __syncthreads();         // every role is done with its tiles, barriers and TMEM columns
  tc_fence_after_sync();
  if (warp == 0) tmem_dealloc(tmem_base, NCOLS);
}

// ------------------------------------------------------------------ self test of the bounded wait
__global__ void __launch_bounds__(32) selftest_wait_expiry_kernel(int* status, unsigned long long* elapsed_ns) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    mbar_fence_init();
  }
  __syncwarp();
  unsigned long long t0, t1;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  const bool ok = mbar_wait(&bar, 0, status, 5);     // nobody arrives: gives up after kSpinLimit polls
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
  if (threadIdx.x == 0) *elapsed_ns = ok ? 0ull : t1 - t0;
}

int launch_selftest_wait_expiry(int* status, unsigned long long* elapsed_ns, cudaStream_t s) {
  FMB_CUDA(cudaMemsetAsync(status, 0, sizeof(int), s));
  selftest_wait_expiry_kernel<<<1, 32, 0, s>>>(status, elapsed_ns);
  FMB_LAUNCH_CHECK("selftest_wait_expiry_kernel");
  return FMB_OK;
}

// ------------------------------------------------------------------ self test of the MMA path
// D[128][128] (fp32) = A[128][128] . B, with B given [N][K] (K contiguous) when b_mn_major == 0
// or [K][N] (N contiguous) when 1.  Exercises exactly the descriptors the attention kernels use.
template <typename T>
__global__ void __launch_bounds__(128) selftest_umma_kernel(const T* a, const T* b, float* d, int b_mn_major,
                                                            int* status) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_base_s;
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  unsigned char* sA = smem;
  unsigned char* sB = smem + 128 * 128 * 2;
  const int tid = threadIdx.x, warp = tid >> 5;
  if (warp == 0) tmem_alloc(&tmem_base_s, 128);
  if (tid == 0) { mbar_init(&bar, 1); mbar_fence_init(); }
  stage_tile_sw128<T, 16>(sA, 128 * 128, a, 128, 128, [](int r) { return (int64_t)r; });
  stage_tile_sw128<T, 16>(sB, 128 * 128, b, 128, 128, [](int r) { return (int64_t)r; });
  fence_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tD = tmem_base_s;
  if (tid == 0) {
    const uint32_t idesc = make_idesc(FmtOf<T>::v, 128, 128, 0, b_mn_major);
    for (int ks = 0; ks < 8; ++ks) {
      const uint64_t ad = make_desc_sw128(smem_u32(sA) + (ks >> 2) * 16384 + (ks & 3) * 32, 16, 1024);
      const uint64_t bd = b_mn_major ? make_desc_sw128(smem_u32(sB) + ks * 2048, 16384, 1024)
                                     : make_desc_sw128(smem_u32(sB) + (ks >> 2) * 16384 + (ks & 3) * 32, 16, 1024);
      umma_ss(tD, ad, bd, idesc, ks > 0);
    }
    umma_commit(&bar);
  }
  const bool ok = mbar_wait(&bar, 0, status, 9);
  if (__syncthreads_and(ok)) {
    tc_fence_after_sync();
    for (int i = 0; i < 4; ++i) {
      float o[32];
      tmem_ld32(tD + ((uint32_t)(warp * 32) << 16) + i * 32, o);
      tmem_ld_wait();
      for (int j = 0; j < 32; ++j) d[tid * 128 + i * 32 + j] = o[j];
    }
    tc_fence_before_sync();
  }
  __syncthreads();
  if (warp == 0) tmem_dealloc(tD, 128);
}

int launch_selftest_umma(const void* a, const void* b, float* d, int b_mn_major, int dtype, int* status,
                         cudaStream_t s) {
  const size_t smem = 2 * 128 * 128 * 2 + 1024;
  if (dtype == FMB_BF16) {
    auto kern = selftest_umma_kernel<__nv_bfloat16>;
    FMB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<1, 128, smem, s>>>((const __nv_bfloat16*)a, (const __nv_bfloat16*)b, d, b_mn_major, status);
  } else {
    auto kern = selftest_umma_kernel<__half>;
    FMB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<1, 128, smem, s>>>((const __half*)a, (const __half*)b, d, b_mn_major, status);
  }
  FMB_LAUNCH_CHECK("selftest_umma_kernel");
  return FMB_OK;
}

// ------------------------------------------------------------------ launchers
static TcParams make_tc_params(const AttnArgs& a, const AttnWorkspace& w, const PassParams& ps) {
  TcParams p;
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

// When the gathered rows of the whole pass (Q, and dO in the backward pass) fit in L2 whatever the
// order of the work items, the key blocks are handed out longest columns first throughout: a launch
// of few items per CTA (one rank's share of a multi-GPU run) is balanced best that way.  Measured:
// 64K tokens x 4 heads 1.69 -> 1.62 ms per step; 512K tokens x 4 heads (1 GB of rows) 1 % slower,
// hence the size test.
static bool rows_fit_l2(const AttnArgs& a, const PassParams& ps) {
  return (int64_t)a.total_q * a.d * 2 * 2 * ps.nh <= (int64_t)160 << 20;
}

// Tensor maps of K and V for the key-block loads: one 2-D map per tensor over (columns of a token
// row, token rows), box 64 columns x C rows, 128-byte swizzle.  Possible when all kv heads of a
// token lie inside its row stride; the row extent is left open because only blocks that lie wholly
// inside their sequence are loaded this way.  Tensor maps over this GPU's own memory only, plain
// per-CTA loads (no multicast: the kernels also run in multi-GPU jobs).
static int make_kv_maps(const AttnArgs& a, int C, CUtensorMap* mk, CUtensorMap* mv, int* usable) {
  *usable = 0;
  memset(mk, 0, sizeof(*mk));
  memset(mv, 0, sizeof(*mv));
  auto fits = [&](int64_t rs, int64_t hs) { return hs >= 0 && rs > 0 && (int64_t)(a.heads_k - 1) * hs + a.d <= rs; };
  if (a.k == nullptr || a.v == nullptr || !fits(a.k_rs, a.k_hs) || !fits(a.v_rs, a.v_hs)) return FMB_OK;
  const uint64_t rows = (uint64_t)1 << 31;
  int rc = make_tmap_2d(mk, a.k, a.dtype, (uint64_t)((a.heads_k - 1) * a.k_hs + a.d), rows, (uint64_t)a.k_rs * 2, 64, C);
  if (rc == FMB_OK) rc = make_tmap_2d(mv, a.v, a.dtype, (uint64_t)((a.heads_k - 1) * a.v_hs + a.d), rows, (uint64_t)a.v_rs * 2, 64, C);
  if (rc != FMB_OK) return FMB_OK;     // no driver support for tensor maps: the cp.async path serves every block
  *usable = 1;
  return FMB_OK;
}

template <typename T, int C, int D>
static int fwd_tc_launch(const AttnArgs& a, const AttnWorkspace& w, const PassParams& ps, cudaStream_t s) {
  TcParams p = make_tc_params(a, w, ps);
  CUtensorMap map_k, map_v;
  make_kv_maps(a, C, &map_k, &map_v, &p.kv_tma);
  constexpr int QP = (C > D ? C : D);
  // K, V, and per compute group a Q tile and a P / O-staging tile; one CTA per SM by size
  // (all 512 TMEM columns are allocated)
  size_t smem = (size_t)2 * C * D * 2 + (size_t)kFwdGroups * kTcM * (D + QP) * 2 + 1024;
  if (smem < 120 * 1024) smem = 120 * 1024;
  auto kern = fwd_main_tc_kernel<T, C, D>;
  FMB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  // persistent CTAs, one per SM
  p.work = w.status + 4;
  p.items_x = a.ncol * ps.nsub; p.items_y = ps.nh; p.items_z = a.batch;
  p.items_heavy = !a.causal ? 0 : (rows_fit_l2(a, ps) ? p.items_x : min(p.items_x, 16 * ps.nsub));
  p.n_items = p.items_x * p.items_y * p.items_z;
  if (ps.h0 > 0) FMB_CUDA(cudaMemsetAsync(p.work, 0, sizeof(int), s));   // first pass: cleared with the status block
  kern<<<min(p.n_items, sm_count()), kFwdThreads, smem, s>>>(p, map_k, map_v);
  FMB_LAUNCH_CHECK("fwd_main_tc_kernel");
  return FMB_OK;
}

template <typename T, int C, int D>
static int bwd_tc_launch(const AttnArgs& a, const AttnWorkspace& w, const PassParams& ps, cudaStream_t s) {
  TcParams p = make_tc_params(a, w, ps);
  CUtensorMap map_k, map_v;
  make_kv_maps(a, C, &map_k, &map_v, &p.kv_tma);
  // K, V, two Q tiles, one dO tile, P and dS: with d = 128 that and the kernel's 3 KB of static shared
  // memory are exactly the 227 KB a CTA may have (the dynamic part is declared 1024-byte aligned)
  const size_t smem = (size_t)2 * C * D * 2 + (size_t)3 * kTcM * D * 2 + (size_t)2 * kTcM * C * 2;
  auto kern = bwd_main_tc_kernel<T, C, D>;
  FMB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const int nchunk = max(a.ncol, ceil_div(a.max_k, a.chunk));
  // persistent CTAs, one per SM
  p.work = w.status + 4;
  p.items_x = nchunk * ps.nsub; p.items_y = ps.nh / (a.heads / a.heads_k); p.items_z = a.batch;
  p.items_heavy = !a.causal ? 0 : (rows_fit_l2(a, ps) ? p.items_x : min(p.items_x, 16 * ps.nsub));
  p.n_items = p.items_x * p.items_y * p.items_z;
  if (ps.h0 > 0) FMB_CUDA(cudaMemsetAsync(p.work, 0, sizeof(int), s));   // first pass: cleared with the status block
  kern<<<min(p.n_items, sm_count()), kBwdThreads, smem, s>>>(p, map_k, map_v);
  FMB_LAUNCH_CHECK("bwd_main_tc_kernel");
  return FMB_OK;
}

bool tc_supported(const AttnArgs& a, bool backward) {
  // key block = 128 keys when the chunk is a multiple of 128, else 64
  return a.chunk % 64 == 0 && (a.d == 64 || a.d == 128);
}

int launch_fwd_main_tc(const AttnArgs& a, const AttnWorkspace& w, const PassParams& ps, cudaStream_t s) {
  if (a.ncol == 0 || a.batch == 0 || a.heads == 0) return FMB_OK;
#define FMB_TC_FWD(TT)                                                          \
  if (w.kb == 64 && a.d == 64) return fwd_tc_launch<TT, 64, 64>(a, w, ps, s);     \
  if (w.kb == 64 && a.d == 128) return fwd_tc_launch<TT, 64, 128>(a, w, ps, s);   \
  if (w.kb == 128 && a.d == 64) return fwd_tc_launch<TT, 128, 64>(a, w, ps, s);   \
  if (w.kb == 128 && a.d == 128) return fwd_tc_launch<TT, 128, 128>(a, w, ps, s);
  if (a.dtype == FMB_BF16) { FMB_TC_FWD(__nv_bfloat16) } else { FMB_TC_FWD(__half) }
#undef FMB_TC_FWD
  return fail(FMB_ERR_UNSUPPORTED, "tensor-core forward: head_dim %d not built", a.d);
}

int launch_bwd_main_tc(const AttnArgs& a, const AttnWorkspace& w, const PassParams& ps, cudaStream_t s) {
  if (a.batch == 0 || a.heads == 0) return FMB_OK;
  // 64-key blocks run on the same 128-lane kernel with the upper lanes masked
  if ((w.kb == 128 || w.kb == 64) && a.d == 64)
    return a.dtype == FMB_BF16 ? bwd_tc_launch<__nv_bfloat16, 128, 64>(a, w, ps, s)
                               : bwd_tc_launch<__half, 128, 64>(a, w, ps, s);
  if ((w.kb == 128 || w.kb == 64) && a.d == 128)
    return a.dtype == FMB_BF16 ? bwd_tc_launch<__nv_bfloat16, 128, 128>(a, w, ps, s)
                               : bwd_tc_launch<__half, 128, 128>(a, w, ps, s);
  return fail(FMB_ERR_UNSUPPORTED, "tensor-core backward: key block %d / head_dim %d not built", w.kb, a.d);
}

}  // namespace fmb
