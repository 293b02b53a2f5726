#include "tma_host.h"

#include <mutex>

namespace b200 {
namespace k {

namespace {
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

Status get_encode_fn(EncodeTiledFn* out) {
  static std::mutex mu;
  static EncodeTiledFn fn = nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !p) {
      cudaGetLastError();
      return Status::Cuda("cuTensorMapEncodeTiled is not available from this driver");
    }
    fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  *out = fn;
  return Status::OK();
}
}  // namespace

Status encode_tma_4d_16bit(CUtensorMap* map, const void* base, bool f16, const uint64_t dims[4], const uint64_t strides_bytes[3],
                           const uint32_t box[4], int swizzle_bytes) {
  EncodeTiledFn fn;
  B200_TRY(get_encode_fn(&fn));
  cuuint64_t d[4] = {dims[0], dims[1], dims[2], dims[3]};
  cuuint64_t s[3] = {strides_bytes[0], strides_bytes[1], strides_bytes[2]};
  cuuint32_t bx[4] = {box[0], box[1], box[2], box[3]};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(map, f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), d, s, bx, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return Status::Cuda(strfmt("cuTensorMapEncodeTiled failed with code %d", (int)r));
  return Status::OK();
}

}  // namespace k
}  // namespace b200
