// CUDA-core ("SIMT") engine of the block-sparse attention: a plain fp32-FMA implementation
// of the key-chunk-major main kernels for every shape the tensor-core engines serve (key blocks
// of 64 / 128 keys with head dims 64 / 128; key blocks of 64 keys with head dim 256, where the
// backward tiles are 32 rows so that K, V and the row tiles fit in shared memory).  It is a
// cross-check, not a fallback: the GPU tests run both engines (fmb_set_engine(0) selects this
// one) against the CPU oracle and against each other through the same workspace contract and the
// same merge kernels.  Mathematics follows the
// reference kernels (csrc/flash_moba/src/flash_fwd_kernel.h:535-640, flash_bwd_kernel.h:552-803,
// softmax.h:259-319, mask.h:139-176); the tiling is this library's own.
#include "fmb_attn.cuh"

namespace fmb {

// gathered query rows per tile: 16 row groups x M/16 rows per thread (M = 64, or 32 where the
// backward's tiles would not fit in shared memory otherwise)
constexpr int kSimtThreads = 256;
constexpr float kLog2e = 1.4426950408889634f;

struct SimtParams {
  const void *q, *k, *v, *dout;
  int64_t q_rs, q_hs, k_rs, k_hs, v_rs, v_hs, do_rs, do_hs;
  void *dk, *dv; int64_t dk_rs, dk_hs, dv_rs, dv_hs;
  const float *lse, *softmax_d;
  PassParams ps;
  const int32_t *cu_q, *k_begin, *k_end;
  void* part_o; float* part_lse;
  int heads, heads_k; int64_t total_q;
  float scale; int causal;
};

// stage `rows_valid` gathered rows (ids in sRow, -1 = padding) transposed: dst[dd][m]
template <typename T, int D, int M>
__device__ __forceinline__ void stage_rows_transposed(T* dst, const T* base, int64_t row_stride,
                                                      const int* sRow, int rows_valid) {
  constexpr int G = D / 8;
  for (int e = threadIdx.x; e < M * G; e += blockDim.x) {
    const int r = e % M, g = e / M;
    uint4 u = make_uint4(0, 0, 0, 0);
    if (r < rows_valid && sRow[r] >= 0) u = ldg_nc_16(base + (int64_t)sRow[r] * row_stride + g * 8);
    const T* x = reinterpret_cast<const T*>(&u);
#pragma unroll
    for (int i = 0; i < 8; ++i) dst[(g * 8 + i) * M + r] = x[i];
  }
}
// natural layout dst[m][D]
template <typename T, int D, int M>
__device__ __forceinline__ void stage_rows(T* dst, const T* base, int64_t row_stride, const int* sRow,
                                           int rows_valid) {
  constexpr int G = D / 8;
  for (int e = threadIdx.x; e < M * G; e += blockDim.x) {
    const int r = e / G, g = e % G;
    uint4 u = make_uint4(0, 0, 0, 0);
    if (r < rows_valid && sRow[r] >= 0) u = ldg_nc_16(base + (int64_t)sRow[r] * row_stride + g * 8);
    *reinterpret_cast<uint4*>(dst + r * D + g * 8) = u;
  }
}
// key chunk: natural dst[key][D] and/or transposed dstT[dd][C]
template <typename T, int C, int D>
__device__ __forceinline__ void stage_keys(T* dst, T* dstT, const T* base, int64_t row_stride, int keys_valid) {
  constexpr int G = D / 8;
  for (int e = threadIdx.x; e < C * G; e += blockDim.x) {
    const int r = e % C, g = e / C;
    uint4 u = make_uint4(0, 0, 0, 0);
    if (r < keys_valid) u = ldg_nc_16(base + (int64_t)r * row_stride + g * 8);
    if (dst) *reinterpret_cast<uint4*>(dst + r * D + g * 8) = u;
    if (dstT) {
      const T* x = reinterpret_cast<const T*>(&u);
#pragma unroll
      for (int i = 0; i < 8; ++i) dstT[(g * 8 + i) * C + r] = x[i];
    }
  }
}

// acc[M/16][C/16] += At^T Bt : rows ty*(M/16).., cols tx*(C/16)..   (At [D][M], Bt [D][C])
template <typename T, int C, int D, int M>
__device__ __forceinline__ void gemm_rows_keys(const T* At, const T* Bt, float (&acc)[M / 16][C / 16]) {
  constexpr int TN = C / 16, RM = M / 16;
  const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
#pragma unroll 4
  for (int dd = 0; dd < D; ++dd) {
    float a[RM], b[TN];
#pragma unroll
    for (int i = 0; i < RM; ++i) a[i] = Elem<T>::to_f(At[dd * M + ty * RM + i]);
#pragma unroll
    for (int j = 0; j < TN; ++j) b[j] = Elem<T>::to_f(Bt[dd * C + tx * TN + j]);
#pragma unroll
    for (int i = 0; i < RM; ++i)
#pragma unroll
      for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
  }
}

// ======================================================================== forward
template <typename T, int C, int D, int M>
__global__ void __launch_bounds__(kSimtThreads) fwd_main_simt_kernel(SimtParams p) {
  constexpr int TN = C / 16, TD = D / 16, SS = C + 4, RM = M / 16;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* sKt = reinterpret_cast<T*>(smem_raw);          // [D][C]
  T* sV = sKt + D * C;                              // [C][D]
  T* sQt = sV + C * D;                              // [D][M]
  float* sS = reinterpret_cast<float*>(sQt + D * M);   // [M][C+4]
  int* sRow = reinterpret_cast<int*>(sS + M * SS);     // [M]
  float* sInv = reinterpret_cast<float*>(sRow + M);    // [M]

  // C is the key block: chunk c of the pattern is covered by nsub blocks of C keys
  const int c = blockIdx.x / p.ps.nsub, sb = blockIdx.x % p.ps.nsub, h = p.ps.h0 + blockIdx.y, b = blockIdx.z;
  const ColRef col = column_of(p.ps, b, h, c);
  const int nnz = col.nnz;
  if (nnz <= 0) return;
  const int64_t off = col.off;
  const int64_t slot0 = col.slot, plane = (int64_t)sb * p.ps.cap;
  const int q0 = p.cu_q[b], len_q = p.cu_q[b + 1] - q0;
  const int k0 = p.k_begin[b], len_k = p.k_end[b] - k0;
  const int key0 = c * p.ps.chunk + sb * C;
  const int keys_valid = max(0, min(C, len_k - key0));
  const int hk = h / (p.heads / p.heads_k);
  const int shift = len_k - len_q;
  const float scale_log2 = p.scale * kLog2e;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;

  const T* kbase = static_cast<const T*>(p.k) + (int64_t)(k0 + key0) * p.k_rs + (int64_t)hk * p.k_hs;
  const T* vbase = static_cast<const T*>(p.v) + (int64_t)(k0 + key0) * p.v_rs + (int64_t)hk * p.v_hs;
  const T* qbase = static_cast<const T*>(p.q) + (int64_t)q0 * p.q_rs + (int64_t)h * p.q_hs;
  stage_keys<T, C, D>(nullptr, sKt, kbase, p.k_rs, keys_valid);
  stage_keys<T, C, D>(sV, nullptr, vbase, p.v_rs, keys_valid);
  T* part_o = static_cast<T*>(p.part_o);

  for (int t0 = 0; t0 < nnz; t0 += M) {
    const int rows = min(M, nnz - t0);
    __syncthreads();
    if (threadIdx.x < M) {
      int r = -1;
      if (threadIdx.x < rows) {
        r = p.ps.indices[off + t0 + threadIdx.x];
        if (r < 0 || r >= len_q) r = -1;
      }
      sRow[threadIdx.x] = r;
    }
    __syncthreads();
    stage_rows_transposed<T, D, M>(sQt, qbase, p.q_rs, sRow, rows);
    __syncthreads();
    float acc[RM][TN];
#pragma unroll
    for (int i = 0; i < RM; ++i)
#pragma unroll
      for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;
    gemm_rows_keys<T, C, D, M>(sQt, sKt, acc);
#pragma unroll
    for (int i = 0; i < RM; ++i)
#pragma unroll
      for (int j = 0; j < TN; ++j) sS[(ty * RM + i) * SS + tx * TN + j] = acc[i][j];
    __syncthreads();
    // chunk-local softmax: warp w owns rows w*(M/8)..
    for (int rr = 0; rr < M / 8; ++rr) {
      const int m = warp * (M / 8) + rr;
      const int r = sRow[m];
      const int lim = p.causal ? min(keys_valid, r + shift - key0 + 1) : keys_valid;  // visible keys: j < lim
      float mx = -CUDART_INF_F;
      for (int j = lane; j < C; j += 32) {
        const float s = (r >= 0 && j < lim) ? sS[m * SS + j] : -CUDART_INF_F;
        mx = fmaxf(mx, s);
      }
#pragma unroll
      for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      float sum = 0.f;
      for (int j = lane; j < C; j += 32) {
        float pr = 0.f;
        if (r >= 0 && j < lim) pr = exp2f((sS[m * SS + j] - mx) * scale_log2);
        sS[m * SS + j] = pr;
        sum += pr;
      }
#pragma unroll
      for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      if (lane == 0) {
        sInv[m] = sum > 0.f ? 1.f / sum : 0.f;
        if (m < rows) p.part_lse[plane + slot0 + t0 + m] = sum > 0.f ? mx * p.scale + logf(sum) : -CUDART_INF_F;
      }
    }
    __syncthreads();
    // partial O = P.V / l
    float o[RM][TD];
#pragma unroll
    for (int i = 0; i < RM; ++i)
#pragma unroll
      for (int j = 0; j < TD; ++j) o[i][j] = 0.f;
    for (int j = 0; j < C; ++j) {
      float pr[RM], vv[TD];
#pragma unroll
      for (int i = 0; i < RM; ++i) pr[i] = sS[(ty * RM + i) * SS + j];
#pragma unroll
      for (int x = 0; x < TD; ++x) vv[x] = Elem<T>::to_f(sV[j * D + tx * TD + x]);
#pragma unroll
      for (int i = 0; i < RM; ++i)
#pragma unroll
        for (int x = 0; x < TD; ++x) o[i][x] = fmaf(pr[i], vv[x], o[i][x]);
    }
#pragma unroll
    for (int i = 0; i < RM; ++i) {
      const int m = ty * RM + i;
      if (m < rows) {
        const float inv = sInv[m];
        const int64_t slot = slot0 + t0 + m;
        T* dst = part_o + (plane + slot) * D;
#pragma unroll
        for (int x = 0; x < TD; ++x) dst[part_col(slot, tx * TD + x, 8)] = Elem<T>::from_f(o[i][x] * inv);
      }
    }
  }
}

// ======================================================================== backward
template <typename T, int C, int D, int M>
__global__ void __launch_bounds__(kSimtThreads) bwd_main_simt_kernel(SimtParams p) {
  constexpr int TN = C / 16, TD = D / 16, SS = C + 4, RM = M / 16;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* sKt = reinterpret_cast<T*>(smem_raw);          // [D][C]
  T* sVt = sKt + D * C;                             // [D][C]
  T* sK = sVt + D * C;                              // [C][D]
  T* sQt = sK + C * D;                              // [D][M]
  T* sdOt = sQt + D * M;                       // [D][M]
  T* sQ = sdOt + D * M;                        // [M][D]
  T* sdO = sQ + M * D;                         // [M][D]
  float* sP = reinterpret_cast<float*>(sdO + M * D);   // [M][C+4]
  float* sdS = sP + M * SS;                            // [M][C+4]
  int* sRow = reinterpret_cast<int*>(sdS + M * SS);    // [M]
  float* sLse = reinterpret_cast<float*>(sRow + M);    // [M]
  float* sD = sLse + M;                                // [M]

  const int group = p.heads / p.heads_k;
  const int c = blockIdx.x / p.ps.nsub, sb = blockIdx.x % p.ps.nsub, hk = p.ps.h0 / group + blockIdx.y, b = blockIdx.z;
  const int64_t plane = (int64_t)sb * p.ps.cap;
  const int q0 = p.cu_q[b], len_q = p.cu_q[b + 1] - q0;
  const int k0 = p.k_begin[b], len_k = p.k_end[b] - k0;
  const int key0 = c * p.ps.chunk + sb * C;
  if (key0 >= len_k) {
    zero_dq_partials<T>(p.ps, static_cast<T*>(p.part_o), plane, b, hk, group, c, D);
    return;
  }
  const int keys_valid = min(C, len_k - key0);
  const int shift = len_k - len_q;
  const float scale_log2 = p.scale * kLog2e;
  const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;

  const T* kbase = static_cast<const T*>(p.k) + (int64_t)(k0 + key0) * p.k_rs + (int64_t)hk * p.k_hs;
  const T* vbase = static_cast<const T*>(p.v) + (int64_t)(k0 + key0) * p.v_rs + (int64_t)hk * p.v_hs;
  stage_keys<T, C, D>(sK, sKt, kbase, p.k_rs, keys_valid);
  stage_keys<T, C, D>(nullptr, sVt, vbase, p.v_rs, keys_valid);
  T* part_dq = static_cast<T*>(p.part_o);

  // dK/dV accumulators: keys ty*TN.., dims tx*TD..
  float dk[TN][TD], dv[TN][TD];
#pragma unroll
  for (int i = 0; i < TN; ++i)
#pragma unroll
    for (int j = 0; j < TD; ++j) { dk[i][j] = 0.f; dv[i][j] = 0.f; }

  for (int hg = 0; hg < group; ++hg) {
    const int h = hk * group + hg;
    const ColRef col = column_of(p.ps, b, h, c);
    const int nnz = col.nnz;
    const int64_t off = col.off, slot0 = col.slot;
    if (nnz <= 0) continue;
    const T* qbase = static_cast<const T*>(p.q) + (int64_t)q0 * p.q_rs + (int64_t)h * p.q_hs;
    const T* dobase = static_cast<const T*>(p.dout) + (int64_t)q0 * p.do_rs + (int64_t)h * p.do_hs;
    const float* lse = p.lse + (int64_t)h * p.total_q + q0;
    const float* dsum = p.softmax_d + (int64_t)h * p.total_q + q0;

    for (int t0 = 0; t0 < nnz; t0 += M) {
      const int rows = min(M, nnz - t0);
      __syncthreads();
      if (threadIdx.x < M) {
        int r = -1;
        float l = CUDART_INF_F, dd = 0.f;
        if (threadIdx.x < rows) {
          r = p.ps.indices[off + t0 + threadIdx.x];
          if (r < 0 || r >= len_q) r = -1;
          else { l = lse[r]; dd = dsum[r]; }
        }
        sRow[threadIdx.x] = r; sLse[threadIdx.x] = l; sD[threadIdx.x] = dd;
      }
      __syncthreads();
      stage_rows_transposed<T, D, M>(sQt, qbase, p.q_rs, sRow, rows);
      stage_rows_transposed<T, D, M>(sdOt, dobase, p.do_rs, sRow, rows);
      stage_rows<T, D, M>(sQ, qbase, p.q_rs, sRow, rows);
      stage_rows<T, D, M>(sdO, dobase, p.do_rs, sRow, rows);
      __syncthreads();
      {
        float s[RM][TN], dp[RM][TN];
#pragma unroll
        for (int i = 0; i < RM; ++i)
#pragma unroll
          for (int j = 0; j < TN; ++j) { s[i][j] = 0.f; dp[i][j] = 0.f; }
        gemm_rows_keys<T, C, D, M>(sQt, sKt, s);
        gemm_rows_keys<T, C, D, M>(sdOt, sVt, dp);
#pragma unroll
        for (int i = 0; i < RM; ++i) {
          const int m = ty * RM + i;
          const int r = sRow[m];
          const int lim = p.causal ? min(keys_valid, r + shift - key0 + 1) : keys_valid;
          const float l2 = sLse[m] * kLog2e, dd = sD[m];
#pragma unroll
          for (int j = 0; j < TN; ++j) {
            const int col = tx * TN + j;
            float pr = 0.f;
            if (r >= 0 && col < lim) pr = exp2f(s[i][j] * scale_log2 - l2);
            sP[m * SS + col] = pr;
            sdS[m * SS + col] = pr * (dp[i][j] - dd);
          }
        }
      }
      __syncthreads();
      // dV += P^T dO ; dK += dS^T Q        (keys ty*TN.., dims tx*TD..)
      for (int m = 0; m < M; ++m) {
        float pv[TN], ds[TN], dov[TD], qv[TD];
#pragma unroll
        for (int i = 0; i < TN; ++i) { pv[i] = sP[m * SS + ty * TN + i]; ds[i] = sdS[m * SS + ty * TN + i]; }
#pragma unroll
        for (int j = 0; j < TD; ++j) {
          dov[j] = Elem<T>::to_f(sdO[m * D + tx * TD + j]);
          qv[j] = Elem<T>::to_f(sQ[m * D + tx * TD + j]);
        }
#pragma unroll
        for (int i = 0; i < TN; ++i)
#pragma unroll
          for (int j = 0; j < TD; ++j) {
            dv[i][j] = fmaf(pv[i], dov[j], dv[i][j]);
            dk[i][j] = fmaf(ds[i], qv[j], dk[i][j]);
          }
      }
      // partial dQ = dS . K  (rows ty*4.., dims tx*TD..), unscaled
      {
        float dq[RM][TD];
#pragma unroll
        for (int i = 0; i < RM; ++i)
#pragma unroll
          for (int j = 0; j < TD; ++j) dq[i][j] = 0.f;
        for (int key = 0; key < C; ++key) {
          float ds[RM], kv[TD];
#pragma unroll
          for (int i = 0; i < RM; ++i) ds[i] = sdS[(ty * RM + i) * SS + key];
#pragma unroll
          for (int j = 0; j < TD; ++j) kv[j] = Elem<T>::to_f(sK[key * D + tx * TD + j]);
#pragma unroll
          for (int i = 0; i < RM; ++i)
#pragma unroll
            for (int j = 0; j < TD; ++j) dq[i][j] = fmaf(ds[i], kv[j], dq[i][j]);
        }
#pragma unroll
        for (int i = 0; i < RM; ++i) {
          const int m = ty * RM + i;
          if (m < rows) {
            const int64_t slot = slot0 + t0 + m;
            T* dst = part_dq + (plane + slot) * D;
#pragma unroll
            for (int j = 0; j < TD; ++j) dst[part_col(slot, tx * TD + j, 8)] = Elem<T>::from_f(dq[i][j] * p.scale);
          }
        }
      }
    }
  }
  // write dK (scaled) and dV of this chunk
  T* dkp = static_cast<T*>(p.dk) + (int64_t)(k0 + key0) * p.dk_rs + (int64_t)hk * p.dk_hs;
  T* dvp = static_cast<T*>(p.dv) + (int64_t)(k0 + key0) * p.dv_rs + (int64_t)hk * p.dv_hs;
#pragma unroll
  for (int i = 0; i < TN; ++i) {
    const int key = ty * TN + i;
    if (key < keys_valid) {
#pragma unroll
      for (int j = 0; j < TD; ++j) {
        dkp[(int64_t)key * p.dk_rs + tx * TD + j] = Elem<T>::from_f(dk[i][j] * p.scale);
        dvp[(int64_t)key * p.dv_rs + tx * TD + j] = Elem<T>::from_f(dv[i][j]);
      }
    }
  }
}

static SimtParams make_params(const AttnArgs& a, const AttnWorkspace& w, const PassParams& ps) {
  SimtParams p;
  p.q = a.q; p.k = a.k; p.v = a.v; p.dout = a.dout;
  p.q_rs = a.q_rs; p.q_hs = a.q_hs; p.k_rs = a.k_rs; p.k_hs = a.k_hs; p.v_rs = a.v_rs; p.v_hs = a.v_hs;
  p.do_rs = a.do_rs; p.do_hs = a.do_hs;
  p.dk = a.dk; p.dv = a.dv; p.dk_rs = a.dk_rs; p.dk_hs = a.dk_hs; p.dv_rs = a.dv_rs; p.dv_hs = a.dv_hs;
  p.lse = a.lse; p.softmax_d = a.softmax_d;
  p.ps = ps;
  p.cu_q = a.cu_q; p.k_begin = a.k_begin; p.k_end = a.k_end; p.part_o = w.part_o; p.part_lse = w.part_lse;
  p.heads = a.heads; p.heads_k = a.heads_k; p.total_q = a.total_q;
  p.scale = a.scale; p.causal = a.causal;
  return p;
}

template <typename T, int C, int D>
static int fwd_launch(const AttnArgs& a, const AttnWorkspace& w, const PassParams& ps, cudaStream_t s) {
  SimtParams p = make_params(a, w, ps);
  constexpr int M = 64;
  const size_t smem = (size_t)(2 * C * D + D * M) * sizeof(T) + (size_t)M * (C + 4) * 4 + M * 8;
  auto kern = fwd_main_simt_kernel<T, C, D, M>;
  FMB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  kern<<<dim3(a.ncol * ps.nsub, ps.nh, a.batch), kSimtThreads, smem, s>>>(p);
  FMB_LAUNCH_CHECK("fwd_main_simt_kernel");
  return FMB_OK;
}
template <typename T, int C, int D>
static int bwd_launch(const AttnArgs& a, const AttnWorkspace& w, const PassParams& ps, cudaStream_t s) {
  SimtParams p = make_params(a, w, ps);
  constexpr int M = D > 128 ? 32 : 64;    // 64-row tiles of d = 256 would need 264 KB of shared memory
  const size_t smem = (size_t)(3 * C * D + 4 * D * M) * sizeof(T) + (size_t)2 * M * (C + 4) * 4 +
                      M * 12;
  auto kern = bwd_main_simt_kernel<T, C, D, M>;
  FMB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const int nchunk = max(a.ncol, ceil_div(a.max_k, a.chunk));
  kern<<<dim3(nchunk * ps.nsub, ps.nh / (a.heads / a.heads_k), a.batch), kSimtThreads, smem, s>>>(p);
  FMB_LAUNCH_CHECK("bwd_main_simt_kernel");
  return FMB_OK;
}

#define FMB_SIMT_DISPATCH(FN, FWD)                                                             \
  if (a.dtype == FMB_BF16) {                                                                \
    if (w.kb == 64 && a.d == 64) return FN<__nv_bfloat16, 64, 64>(a, w, ps, s);             \
    if (w.kb == 64 && a.d == 128) return FN<__nv_bfloat16, 64, 128>(a, w, ps, s);           \
    if (w.kb == 128 && a.d == 64) return FN<__nv_bfloat16, 128, 64>(a, w, ps, s);           \
    if (w.kb == 128 && a.d == 128) return FN<__nv_bfloat16, 128, 128>(a, w, ps, s);         \
    if (w.kb == 64 && a.d == 256) return FN<__nv_bfloat16, 64, 256>(a, w, ps, s);           \
    if (FWD && w.kb == 128 && a.d == 256) return fwd_launch<__nv_bfloat16, 128, 256>(a, w, ps, s);   \
  } else {                                                                                  \
    if (w.kb == 64 && a.d == 64) return FN<__half, 64, 64>(a, w, ps, s);                    \
    if (w.kb == 64 && a.d == 128) return FN<__half, 64, 128>(a, w, ps, s);                  \
    if (w.kb == 128 && a.d == 64) return FN<__half, 128, 64>(a, w, ps, s);                  \
    if (w.kb == 128 && a.d == 128) return FN<__half, 128, 128>(a, w, ps, s);                \
    if (w.kb == 64 && a.d == 256) return FN<__half, 64, 256>(a, w, ps, s);                  \
    if (FWD && w.kb == 128 && a.d == 256) return fwd_launch<__half, 128, 256>(a, w, ps, s);          \
  }                                                                                         \
  return fail(FMB_ERR_UNSUPPORTED, "attention (CUDA-core engine): head_dim %d not built "  \
              "(head_dim in {64,128,256})", a.d);

int launch_fwd_main_simt(const AttnArgs& a, const AttnWorkspace& w, const PassParams& ps, cudaStream_t s) {
  if (a.ncol == 0 || a.batch == 0 || a.heads == 0) return FMB_OK;
  FMB_SIMT_DISPATCH(fwd_launch, true)
}
int launch_bwd_main_simt(const AttnArgs& a, const AttnWorkspace& w, const PassParams& ps, cudaStream_t s) {
  if (a.batch == 0 || a.heads == 0) return FMB_OK;
  FMB_SIMT_DISPATCH(bwd_launch, false)
}

}  // namespace fmb
