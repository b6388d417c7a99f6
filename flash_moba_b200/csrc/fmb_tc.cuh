// Blackwell (sm_100a) primitives used by the tensor-core kernels: tcgen05 MMA with TMEM
// accumulators, shared-memory matrix descriptors, mbarriers with BOUNDED waits, proxy fences.
// Inline PTX only; no library templates.
#pragma once
#include "fmb_common.cuh"

namespace fmb {
namespace tc {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- mbarrier ------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// non-blocking test of a phase (for a thread that serves several barriers in turn)
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: gives up after kSpinLimit polls, records `where` in *status and returns false.
// The caller then leaves the kernel through its normal exit path (TMEM is still released).
// A poll blocks for a hardware-defined time, so the bound is one in time too: measured on a B200
// by fmb_selftest_wait_expiry (an mbarrier nobody arrives at), which the GPU tests run.  The loop is
// kept this small on purpose: the attention kernels have about twenty-five call sites, and a
// second register in the loop (a clock-based bound) cost the backward kernel 7 % through spills.
constexpr uint32_t kSpinLimit = 1u << 17;
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* status, int where) {
#pragma unroll 1   // the compiler otherwise unrolls the poll 32 times at every call site
  for (uint32_t i = 0; i < kSpinLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
  }
  if (status) atomicCAS(status, 0, where);
  return false;
}

// ---- a load that is issued where it is written
// A plain load of read-only data may be moved by the compiler down to its first use (it does so
// under register pressure), which turns a prefetch into a full-latency stall.  This is a volatile
// asm statement: it keeps its place among the other volatile statements (barrier waits).
__device__ __forceinline__ int ldg_s32_here(const int* ptr) {
  int v;
  asm volatile("ld.global.nc.s32 %0, [%1];" : "=r"(v) : "l"(ptr));
  return v;
}

// ---- named barriers for groups of warps inside a CTA (id 1..15; count a multiple of 32)
__device__ __forceinline__ void bar_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}
// barrier + AND-reduction of a predicate over the group
__device__ __forceinline__ bool bar_and(int id, int nthreads, bool pred) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 q, %3, 0;\n\t"
      "bar.red.and.pred p, %1, %2, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(r)
      : "r"(id), "r"(nthreads), "r"((uint32_t)pred)
      : "memory");
  return r != 0;
}

// ---- register budget per warpgroup ------------------------------------------------------
// A CTA is launched with one register count for every thread; warp-specialised kernels hand
// registers from the warps that only copy or issue to the warps that compute.  Executed by all
// four warps of a warpgroup (warps 4i..4i+3) with the same value, a multiple of 8.
template <int N>
__device__ __forceinline__ void reg_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N>
__device__ __forceinline__ void reg_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }

// ---- fences --------------------------------------------------------------------------
// generic-proxy writes to shared memory -> visible to the async proxy (tcgen05.mma, TMA)
__device__ __forceinline__ void fence_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ---- TMEM ----------------------------------------------------------------------------
// whole warp; ncols power of two in [32, 512]; the base address lands in *dst_smem
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)),
               "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// 32 lanes x 32 consecutive fp32 columns: thread t of the warp gets lane (t), columns c..c+31
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float* v) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]),
        "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]),
        "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float* v) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---- shared-memory matrix descriptors (128-byte swizzle) ------------------------------
// Tiles are stored as rows of 128 bytes (64 16-bit elements); 16-byte chunk j of row r sits
// at r*128 + ((j ^ (r & 7)) << 4); a tile wider than 64 elements is a sequence of such
// blocks.  Tile bases are 1024-byte aligned.
//   lbo/sbo in bytes.  K-major: sbo = distance between 8-row groups (1024), lbo unused.
//   MN-major: lbo = distance between 64-element blocks along M/N, sbo = distance between
//   8-row groups along K.
__device__ __forceinline__ uint64_t make_desc_sw128(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3ffffu) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3fffu) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3fffu) << 32;
  d |= (uint64_t)1 << 46;   // descriptor version (Blackwell)
  d |= (uint64_t)2 << 61;   // SWIZZLE_128B
  return d;
}

// instruction descriptor, kind::f16, fp32 accumulate.  fmt: 0 = fp16, 1 = bf16.
__host__ __device__ constexpr uint32_t make_idesc(int fmt, int M, int N, int a_mn_major, int b_mn_major) {
  return (1u << 4) | ((uint32_t)fmt << 7) | ((uint32_t)fmt << 10) | ((uint32_t)a_mn_major << 15) |
         ((uint32_t)b_mn_major << 16) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// D[tmem] (+)= A[smem] . B[smem]; issued by ONE thread
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      :
      : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
// The same instruction with the two descriptors given as 32-bit halves.  The low word holds the
// start address (in 16-byte units) and the leading-dimension offset, the high word the stride
// offset, version and swizzle mode: stepping through the K dimension only adds to the low word,
// which keeps the issuing thread's instruction count per MMA small (it is a single thread whose
// issue latency is on the kernel's critical path).
__device__ __forceinline__ uint32_t desc_lo_sw128(uint32_t smem_addr, uint32_t lbo_bytes) {
  return ((smem_addr & 0x3ffffu) >> 4) | (((lbo_bytes >> 4) & 0x3fffu) << 16);
}
__device__ __forceinline__ uint32_t desc_hi_sw128(uint32_t sbo_bytes) {
  return ((sbo_bytes >> 4) & 0x3fffu) | (1u << 14) | (2u << 29);
}
__device__ __forceinline__ void umma_ss_lohi(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo,
                                             uint32_t b_hi, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "mov.b64 da, {%1, %2};\n\t"
      "mov.b64 db, {%3, %4};\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, {%7, %7, %7, %7}, p;\n\t}"
      :
      : "r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
// One GEMM of NK k-steps (16 elements each).  Operand offsets per k-step, in 16-byte units:
// K-major tiles advance 2 inside a 64-element block and `blk` between blocks; MN-major tiles
// advance 128 per step (blk = 512).
template <int NK>
__device__ __forceinline__ void umma_gemm(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t a_step,
                                          uint32_t a_blk, uint32_t b_lo, uint32_t b_hi, uint32_t b_step,
                                          uint32_t b_blk, uint32_t idesc, uint32_t accumulate) {
#pragma unroll
  for (int ks = 0; ks < NK; ++ks) {
    umma_ss_lohi(d_tmem, a_lo + (ks >> 2) * a_blk + (ks & 3) * a_step, a_hi,
                 b_lo + (ks >> 2) * b_blk + (ks & 3) * b_step, b_hi, idesc, accumulate | (ks > 0));
  }
}
// the mbarrier receives one arrival when every MMA issued so far by this thread has completed
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}

// byte offset of 16-byte chunk `j` (0.. row_bytes/16) of row `r` in a swizzled tile whose
// 64-element blocks are `block_stride` bytes apart
__device__ __forceinline__ uint32_t sw128_offset(int r, int j, uint32_t block_stride) {
  return (uint32_t)(j >> 3) * block_stride + (uint32_t)r * 128u + (uint32_t)(((j & 7) ^ (r & 7)) << 4);
}

// rows x (NCHUNK*8 elements) from global memory into a swizzled UMMA tile.
// row_of(r) gives the source row (or -1 for zero fill).
template <typename T, int NCHUNK, typename RowFn>
__device__ __forceinline__ void stage_tile_sw128(unsigned char* tile, uint32_t block_stride, const T* base,
                                                 int64_t row_stride, int nrows, RowFn row_of) {
  for (int e = threadIdx.x; e < nrows * NCHUNK; e += blockDim.x) {
    const int r = e / NCHUNK, j = e % NCHUNK;
    const int64_t src = row_of(r);
    uint4 u = make_uint4(0, 0, 0, 0);
    if (src >= 0) u = ldg_nc_16(base + src * row_stride + j * 8);
    *reinterpret_cast<uint4*>(tile + sw128_offset(r, j, block_stride)) = u;
  }
}

// ---- cp.async (16-byte global -> shared copies that bypass registers) ------------------
// Measured on B200: a 128-thread group gathers random 256-byte rows about four times faster
// with these than with loads into registers (whose number in flight per warp is small).
__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gsrc, bool valid) {
  const uint32_t n = valid ? 16u : 0u;   // src-size 0: the 16 bytes are zero-filled, nothing is read
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(n)
               : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
  asm volatile("cp.async.commit_group;" ::: "memory");
  asm volatile("cp.async.wait_group 0;" ::: "memory");
}
// one 128-row x NCHUNK*16-byte tile gathered by a group of NT threads (t = index in the group);
// rows[] holds the source row of each tile row, -1 = zero fill
template <typename T, int NCHUNK, int NT = 128>
__device__ __forceinline__ void gather_cp_async(int t, unsigned char* tile, uint32_t block_stride, const T* base,
                                                int64_t row_stride, const int* rows) {
  static_assert(NT % NCHUNK == 0, "a thread keeps one 16-byte chunk column");
  constexpr int RPP = NT / NCHUNK;           // rows per pass
  constexpr int PASSES = (128 + RPP - 1) / RPP;
  const int j = t % NCHUNK, rb = t / NCHUNK;
  // partly unrolled on purpose: the loader warps run beside other roles and the kernel's code has
  // to stay small enough for the instruction cache
#pragma unroll 4
  for (int i = 0; i < PASSES; ++i) {
    const int r = rb + RPP * i;
    if (128 % RPP != 0 && r >= 128) break;   // thread groups that do not tile the 128 rows evenly
    const int src = rows[r];
    cp_async_16(tile + sw128_offset(r, j, block_stride), base + (int64_t)(src < 0 ? 0 : src) * row_stride + j * 8,
                src >= 0);
  }
}

// NROWS x NCHUNK*16-byte dense tile (rows `row_stride` apart, rows >= rows_valid zero-filled) copied
// by a group of NT threads with 16-byte cp.async copies
template <typename T, int NCHUNK, int NROWS, int NT>
__device__ __forceinline__ void dense_cp_async(int t, unsigned char* tile, uint32_t block_stride, const T* base,
                                               int64_t row_stride, int rows_valid) {
  constexpr int RPP = NT / NCHUNK;           // rows per pass
  static_assert(NT % NCHUNK == 0 && NROWS % RPP == 0, "thread group does not tile the rows");
  const int j = t % NCHUNK, rb = t / NCHUNK;
#pragma unroll 4
  for (int i = 0; i < NROWS / RPP; ++i) {
    const int r = rb + RPP * i;
    const bool ok = r < rows_valid;
    cp_async_16(tile + sw128_offset(r, j, block_stride), base + (int64_t)(ok ? r : 0) * row_stride + j * 8, ok);
  }
}

// ---- bulk (TMA, non-tensor) shared -> global stores -----------------------------------
// 16-byte aligned addresses, size a multiple of 16.  The issuing thread commits its copies
// as a group and must wait for the group's READS before the shared-memory source is reused
// (or the CTA exits).
__device__ __forceinline__ void bulk_store(void* gdst, const void* ssrc, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_u32(ssrc)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }

template <typename T> struct FmtOf;
template <> struct FmtOf<__nv_bfloat16> { static constexpr int v = 1; };
template <> struct FmtOf<__half> { static constexpr int v = 0; };


}  // namespace tc
}  // namespace fmb
