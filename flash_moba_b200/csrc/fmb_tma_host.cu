// Host side of the TMA support: cuTensorMapEncodeTiled is looked up through the runtime
// (cudaGetDriverEntryPoint), so the library does not link against libcuda.
#include <mutex>

#include "fmb_tma.cuh"

namespace fmb {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

int make_tmap_2d(CUtensorMap* map, const void* base, int dtype, uint64_t cols, uint64_t rows,
                 uint64_t row_stride_bytes, uint32_t box_cols, uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(FMB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  if (rows == 0) rows = 1;   // an empty tensor still needs a valid descriptor; it is never read
  const cuuint64_t gdim[2] = {cols, rows};
  const cuuint64_t gstride[1] = {row_stride_bytes};
  const cuuint32_t box[2] = {box_cols, box_rows};
  const cuuint32_t estride[2] = {1, 1};
  const CUresult r = fn(map, dtype == FMB_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                        2, const_cast<void*>(base), gdim, gstride, box, estride, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(FMB_ERR_CUDA, "cuTensorMapEncodeTiled failed (code %d): cols %llu rows %llu stride %llu box %ux%u",
                (int)r, (unsigned long long)cols, (unsigned long long)rows, (unsigned long long)row_stride_bytes,
                box_cols, box_rows);
  return FMB_OK;
}

}  // namespace fmb
