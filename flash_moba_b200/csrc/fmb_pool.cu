// Stage P: per-chunk key mean-pool (centroids), a 128-bit HBM-streaming kernel.
//
// Replaces the reference's Triton kernel (flash_moba/triton_mean_pool.py:41-109) and its
// host prologue (:134-142).  HBM bound: reads K once (T*Hk*d*2 bytes), writes one row per
// chunk.  One warp owns one (chunk, kv head): lanes cover the head dimension with 16-byte
// loads, several rows per iteration, four independent loads in flight per lane, fp32
// accumulation, one shuffle reduction at the end.
#include "fmb_common.cuh"

namespace fmb {

__global__ void chunk_offsets_kernel(const int32_t* __restrict__ cu_k, int batch, int chunk,
                                     int32_t* __restrict__ cu_km) {
  // one warp, chunked inclusive scan over the batch
  const int lane = threadIdx.x;
  int carry = 0;
  if (lane == 0) cu_km[0] = 0;
  for (int b0 = 0; b0 < batch; b0 += 32) {
    int b = b0 + lane;
    int n = 0;
    if (b < batch) n = (cu_k[b + 1] - cu_k[b] + chunk - 1) / chunk;
    int x = n;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int y = __shfl_up_sync(0xffffffffu, x, o);
      if (lane >= o) x += y;
    }
    if (b < batch) cu_km[b + 1] = carry + x;
    carry += __shfl_sync(0xffffffffu, x, 31);
  }
}

int launch_chunk_offsets(const int32_t* cu_k, int batch, int chunk, int32_t* cu_km, cudaStream_t s) {
  chunk_offsets_kernel<<<1, 32, 0, s>>>(cu_k, batch, chunk, cu_km);
  FMB_LAUNCH_CHECK("chunk_offsets_kernel");
  return FMB_OK;
}

constexpr int kPoolWarps = 4;

// batches up to this many sequences have their chunk offsets computed inside the pool kernel
// (every warp sums the chunk counts of the sequences before its own: two rounds of loads at most)
constexpr int kPoolInlineOffsets = 64;

// LPR = lanes per row (power of two >= d/8), RPI = rows per warp iteration = 32 / LPR.
// OFFS: cu_km is an OUTPUT: the warp derives its sequence's first centroid row from cu_k itself and
// the first warp of every sequence publishes it (no separate offsets launch).
template <typename T, int LPR, bool OFFS>
__global__ void __launch_bounds__(kPoolWarps * 32)
mean_pool_kernel(const T* __restrict__ k, int64_t row_stride, int64_t head_stride,
                 const int32_t* __restrict__ cu_k, int32_t* cu_km,
                 T* __restrict__ km, int heads_k, int d, int chunk) {
  constexpr int RPI = 32 / LPR;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * kPoolWarps + warp;  // chunk of this sequence
  const int hk = blockIdx.y, b = blockIdx.z;
  const int seq0 = cu_k[b];
  const int len = cu_k[b + 1] - seq0;
  int km_row0;                                   // first centroid row of this sequence
  if (OFFS) {
    int sum = 0;
    for (int b0 = 0; b0 < b; b0 += 32) {
      const int bb = b0 + lane;
      sum += bb < b ? (cu_k[bb + 1] - cu_k[bb] + chunk - 1) / chunk : 0;
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    km_row0 = sum;
    if (n == 0 && hk == 0 && lane == 0) {
      if (b == 0) cu_km[0] = 0;
      cu_km[b + 1] = sum + (len + chunk - 1) / chunk;
    }
  } else {
    km_row0 = cu_km[b];
  }
  const int row0 = n * chunk;
  if (row0 >= len) return;
  const int rows = min(chunk, len - row0);
  const int sub = lane / LPR;   // which of the RPI rows of an iteration
  const int col = lane % LPR;   // 16-byte column
  const bool col_ok = col * 8 < d;

  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;

  const T* base = k + (int64_t)(seq0 + row0) * row_stride + (int64_t)hk * head_stride + col * 8;
  if (col_ok) {
    int r = sub;
    // four independent 16-byte loads in flight per lane
    for (; r + 3 * RPI < rows; r += 4 * RPI) {
      uint4 u0 = ldg_nc_16(base + (int64_t)(r) * row_stride);
      uint4 u1 = ldg_nc_16(base + (int64_t)(r + RPI) * row_stride);
      uint4 u2 = ldg_nc_16(base + (int64_t)(r + 2 * RPI) * row_stride);
      uint4 u3 = ldg_nc_16(base + (int64_t)(r + 3 * RPI) * row_stride);
      float f[8];
      unpack8<T>(u0, f);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += f[i];
      unpack8<T>(u1, f);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += f[i];
      unpack8<T>(u2, f);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += f[i];
      unpack8<T>(u3, f);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += f[i];
    }
    for (; r < rows; r += RPI) {
      uint4 u0 = ldg_nc_16(base + (int64_t)r * row_stride);
      float f[8];
      unpack8<T>(u0, f);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += f[i];
    }
  }
  // reduce the RPI partial rows (lanes with equal `col`)
#pragma unroll
  for (int o = LPR; o < 32; o <<= 1) {
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], o);
  }
  if (sub == 0 && col_ok) {
    const float inv = 1.0f / (float)rows;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] *= inv;
    T* dst = km + ((int64_t)(km_row0 + n) * heads_k + hk) * d + col * 8;
    *reinterpret_cast<uint4*>(dst) = pack8<T>(acc);
  }
}

template <typename T>
static int pool_dispatch(const void* k, int64_t rs, int64_t hs, const int32_t* cu_k, int32_t* cu_km,
                         void* km, int batch, int heads_k, int d, int max_seqlen_k, int chunk,
                         bool offsets, cudaStream_t s) {
  const int nchunk = ceil_div(max_seqlen_k, chunk);
  if (nchunk == 0 || batch == 0) return FMB_OK;
  dim3 grid(ceil_div(nchunk, kPoolWarps), heads_k, batch), block(kPoolWarps * 32);
  const int lanes = d / 8;
  const T* kp = static_cast<const T*>(k);
  T* kmp = static_cast<T*>(km);
#define FMB_POOL(L)                                                                                              \
  do {                                                                                                           \
    if (offsets) mean_pool_kernel<T, L, true><<<grid, block, 0, s>>>(kp, rs, hs, cu_k, cu_km, kmp, heads_k, d, chunk);   \
    else mean_pool_kernel<T, L, false><<<grid, block, 0, s>>>(kp, rs, hs, cu_k, cu_km, kmp, heads_k, d, chunk);  \
  } while (0)
  if (lanes <= 1) FMB_POOL(1);
  else if (lanes <= 2) FMB_POOL(2);
  else if (lanes <= 4) FMB_POOL(4);
  else if (lanes <= 8) FMB_POOL(8);
  else if (lanes <= 16) FMB_POOL(16);
  else FMB_POOL(32);
#undef FMB_POOL
  FMB_LAUNCH_CHECK("mean_pool_kernel");
  return FMB_OK;
}

// offsets: cu_km is written (by the pool kernel itself for small batches, by the offsets kernel
// first otherwise) instead of read
int launch_mean_pool(const void* k, int64_t rs, int64_t hs, const int32_t* cu_k, int32_t* cu_km,
                     void* km, int batch, int heads_k, int d, int max_seqlen_k, int chunk, int dtype,
                     cudaStream_t s, bool offsets) {
  prof_begin(3, s);
  bool inline_offsets = false;
  int rc = FMB_OK;
  if (offsets) {
    // a batch without keys launches no pool kernel: the offsets kernel then writes the zeros
    inline_offsets = batch <= kPoolInlineOffsets && ceil_div(max_seqlen_k, chunk) > 0;
    if (!inline_offsets) rc = launch_chunk_offsets(cu_k, batch, chunk, cu_km, s);
  }
  if (rc == FMB_OK)
    rc = dtype == FMB_BF16
        ? pool_dispatch<__nv_bfloat16>(k, rs, hs, cu_k, cu_km, km, batch, heads_k, d, max_seqlen_k, chunk, inline_offsets, s)
        : pool_dispatch<__half>(k, rs, hs, cu_k, cu_km, km, batch, heads_k, d, max_seqlen_k, chunk, inline_offsets, s);
  prof_end(3, s);
  return rc;
}

}  // namespace fmb
