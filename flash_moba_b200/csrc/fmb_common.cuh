// Shared helpers of the flash_moba_b200 kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/flash_moba_b200.h"

namespace fmb {

// ---- error reporting (thread-local message behind fmb_last_error) -------------------
char* error_buffer();          // defined in fmb_api.cu
int fail(int code, const char* fmt, ...);
void note_launch();            // counts kernel launches (fmb_launch_count)
// optional CUDA-event timing of the kernels (fmb_profile_*); kind 0 = forward main kernel,
// 1 = backward main kernel, 2 = gating kernel, 3 = mean-pool kernel, 4 = forward combine,
// 5 = backward combine, 6 = pattern build (three kernels), 7 = dO.O
void prof_begin(int kind, cudaStream_t s);
void prof_end(int kind, cudaStream_t s);

#define FMB_CHECK_ARG(cond, ...)                                   \
  do {                                                             \
    if (!(cond)) return ::fmb::fail(FMB_ERR_BAD_ARG, __VA_ARGS__); \
  } while (0)

#define FMB_CUDA(call)                                                                  \
  do {                                                                                  \
    cudaError_t e_ = (call);                                                            \
    if (e_ != cudaSuccess)                                                              \
      return ::fmb::fail(FMB_ERR_CUDA, "%s failed: %s", #call, cudaGetErrorString(e_)); \
  } while (0)

#define FMB_LAUNCH_CHECK(name)                                                           \
  do {                                                                                   \
    cudaError_t e_ = cudaGetLastError();                                                 \
    if (e_ != cudaSuccess)                                                               \
      return ::fmb::fail(FMB_ERR_CUDA, "launch of %s failed: %s", name,                  \
                         cudaGetErrorString(e_));                                        \
    ::fmb::note_launch();                                                                \
  } while (0)

// ---- small device helpers -----------------------------------------------------------
template <typename T> struct Elem;
template <> struct Elem<__nv_bfloat16> {
  using T2 = __nv_bfloat162;
  static __device__ __forceinline__ float to_f(__nv_bfloat16 x) { return __bfloat162float(x); }
  static __device__ __forceinline__ __nv_bfloat16 from_f(float x) { return __float2bfloat16_rn(x); }
  static __device__ __forceinline__ float2 to_f2(__nv_bfloat162 x) { return __bfloat1622float2(x); }
  static __device__ __forceinline__ __nv_bfloat162 from_f2(float a, float b) {
    return __floats2bfloat162_rn(a, b);
  }
};
template <> struct Elem<__half> {
  using T2 = __half2;
  static __device__ __forceinline__ float to_f(__half x) { return __half2float(x); }
  static __device__ __forceinline__ __half from_f(float x) { return __float2half_rn(x); }
  static __device__ __forceinline__ float2 to_f2(__half2 x) { return __half22float2(x); }
  static __device__ __forceinline__ __half2 from_f2(float a, float b) {
    return __floats2half2_rn(a, b);
  }
};

// 8 packed 16-bit values (one 128-bit access) -> 8 floats
template <typename T>
__device__ __forceinline__ void unpack8(const uint4& u, float* f) {
  using T2 = typename Elem<T>::T2;
  const T2* p = reinterpret_cast<const T2*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = Elem<T>::to_f2(p[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
template <typename T>
__device__ __forceinline__ uint4 pack8(const float* f) {
  using T2 = typename Elem<T>::T2;
  uint4 u;
  T2* p = reinterpret_cast<T2*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) p[i] = Elem<T>::from_f2(f[2 * i], f[2 * i + 1]);
  return u;
}

__device__ __forceinline__ uint4 ldg_nc_16(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}

__host__ __device__ __forceinline__ int ceil_div(int a, int b) { return (a + b - 1) / b; }
__host__ __device__ __forceinline__ int64_t ceil_div64(int64_t a, int64_t b) { return (a + b - 1) / b; }
__host__ __device__ __forceinline__ size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// ---- launchers implemented in the .cu files, called from fmb_api.cu ------------------
int launch_chunk_offsets(const int32_t* cu_k, int batch, int chunk, int32_t* cu_km, cudaStream_t s);
int launch_mean_pool(const void* k, int64_t rs, int64_t hs, const int32_t* cu_k, int32_t* cu_km,
                     void* km, int batch, int heads_k, int d, int max_seqlen_k, int chunk, int dtype,
                     cudaStream_t s, bool offsets = false);

struct GateArgs {
  const void* q; int64_t q_rs, q_hs;
  const void* km;
  const int32_t *cu_q, *cu_k, *cu_km;
  int32_t* topk_idx; float* topk_val; int64_t t_rs, t_hs;
  int batch, heads, heads_k, d, max_q, max_k, topk, chunk, causal, dtype;
};
int launch_gate_topk(const GateArgs& a, cudaStream_t s);
void set_gate_engine(int e);
bool gate_tc_supported(int d, int topk);
int read_gate_status(int* out);

size_t csc_workspace_bytes(int batch, int heads, int max_q, int ncol);
int launch_build_csc(const int32_t* topk_idx, int64_t idx_rs, int64_t idx_hs, const int32_t* cu_q, int64_t* col_offsets, int32_t* col_nnz,
                     int32_t* indices, void* ws, size_t ws_bytes, int batch, int heads, int topk, int max_q,
                     int ncol, cudaStream_t s, uint32_t* row_slots = nullptr, int64_t total_q = 0);
size_t csc_static_scratch_bytes();
int launch_build_csc_static(const int32_t* topk_idx, int64_t idx_rs, int64_t idx_hs, const int32_t* cu_q,
                            int64_t* col_offsets, int32_t* col_nnz, int32_t* indices, int batch, int heads,
                            int topk, int max_q, int ncol, cudaStream_t s);
int launch_varlen_sort(const int64_t* starts, const int64_t* ends, const int32_t* src, int32_t* dst,
                       int64_t nseg, int64_t nitems, cudaStream_t s);

struct AttnArgs {
  const void *q, *k, *v, *o, *dout;   // o: forward output (written in fwd, read in bwd)
  int64_t q_rs, q_hs, k_rs, k_hs, v_rs, v_hs, o_rs, o_hs, do_rs, do_hs;
  void *dq, *dk, *dv;
  int64_t dq_rs, dq_hs, dk_rs, dk_hs, dv_rs, dv_hs;
  float* lse;        // (heads, total_q)
  float* softmax_d;  // (heads, total_q)
  const int64_t* col_offsets; const int32_t* col_nnz; const int32_t* indices; int64_t n_indices;
  const int32_t *cu_q, *cu_k;
  // first key row and one-past-last key row of every sequence: cu_k and cu_k + 1 unless the caller
  // gave its own spans (left padding / fewer keys in use than stored; forward only)
  const int32_t *k_begin, *k_end;
  void* ws; size_t ws_bytes;
  int batch, heads, heads_k, d; int64_t total_q, total_k; int max_q, max_k, chunk, ncol;
  float scale; int causal, dtype;
};
size_t attn_workspace_bytes(int64_t total_q, int heads, int heads_k, int d, int64_t n_indices, int batch, int max_k,
                            int chunk, int heads_per_pass, bool backward);
int launch_attn_fwd(const AttnArgs& a, int engine, cudaStream_t s);
int launch_attn_bwd(const AttnArgs& a, int engine, cudaStream_t s);

}  // namespace fmb
