// TMA (tensor-map) support: host-side descriptor builder and device-side issue wrappers.
// Only plain per-CTA tiled loads are used (the K / V key blocks of the attention kernels),
// completion through an mbarrier's transaction count.  No multicast.
#pragma once
#include <cuda.h>

#include "fmb_tc.cuh"

namespace fmb {

// 2-D tensor map over a row-major matrix of 16-bit elements: `cols` contiguous elements per
// row, `rows` rows, rows `row_stride_bytes` apart; box = box_cols x box_rows; 128-byte swizzle
// (box_cols must be 64); out-of-range elements read as zero.  Returns FMB_OK or an error.
int make_tmap_2d(CUtensorMap* map, const void* base, int dtype, uint64_t cols, uint64_t rows,
                 uint64_t row_stride_bytes, uint32_t box_cols, uint32_t box_rows);

namespace tc {

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}

// box (box_cols x box_rows) whose first element is (x, y) -> shared memory
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}

__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

}  // namespace tc
}  // namespace fmb
