// Gather: embedding-row lookup (the fast path) and general XLA Gather.
//
// The reference broadcasts the index tensor to the full output size and calls
// gatherAlongAxis (mpsgraph gather.go:156-170), or transposes the operand and
// uses gatherND (gather.go:190-434).  Here the row path moves whole rows with
// 128-bit copies straight from the table, and the general path computes every
// output element's source address from the XLA Gather rule.  Payload is copied
// bit-exactly; start indices are clamped so a slice never leaves the operand
// (XLA semantics).  HBM-bound: bytes = 2 * output bytes + index bytes.
#include "../kernels.h"

namespace b200 {
namespace k {

namespace {

template <typename I>
__device__ __forceinline__ int64_t load_index(const void* ids, int64_t i) {
  return (int64_t) reinterpret_cast<const I*>(ids)[i];
}
__device__ __forceinline__ int64_t load_index_dt(const void* ids, int dt, int64_t i) {
  switch (dt) {
    case B200_INT32: return load_index<int32_t>(ids, i);
    case B200_INT64: return load_index<int64_t>(ids, i);
    case B200_UINT32: return load_index<uint32_t>(ids, i);
    case B200_UINT64: {   // saturate: an index above INT64_MAX clamps to the last row, not to row 0
      const uint64_t v = reinterpret_cast<const uint64_t*>(ids)[i];
      return v > (uint64_t)INT64_MAX ? INT64_MAX : (int64_t)v;
    }
    case B200_INT16: return load_index<int16_t>(ids, i);
    case B200_UINT16: return load_index<uint16_t>(ids, i);
    case B200_INT8: return load_index<int8_t>(ids, i);
    case B200_UINT8: return load_index<uint8_t>(ids, i);
  }
  return 0;
}

// One warp per gathered row, rows of row_vecs 16-byte vectors.
__global__ void __launch_bounds__(256) gather_rows_kernel(const uint4* table, const void* ids, int ids_dtype, uint4* y,
                                                           int64_t num_ids, int64_t num_rows, int64_t row_vecs) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * 8;
  for (int64_t i = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5); i < num_ids; i += warps) {
    int64_t r = load_index_dt(ids, ids_dtype, i);
    r = r < 0 ? 0 : (r >= num_rows ? num_rows - 1 : r);
    const uint4* src = table + r * row_vecs;
    uint4* dst = y + i * row_vecs;
    for (int64_t v = lane; v < row_vecs; v += 32) dst[v] = src[v];
  }
}

template <typename T>
__global__ void __launch_bounds__(256) gather_general_kernel(const __grid_constant__ GatherParams p, int64_t total) {
  const T* operand = reinterpret_cast<const T*>(p.operand);
  T* y = reinterpret_cast<T*>(p.y);
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t rem = i;
    int64_t batch_coord[kMaxDims];
    int64_t offset_by_axis[kMaxDims];
    for (int d = 0; d < p.operand_rank; ++d) offset_by_axis[d] = 0;
    for (int d = p.out_rank - 1; d >= 0; --d) {
      const int64_t c = rem % p.out_dims[d];
      rem /= p.out_dims[d];
      if (p.out_offset_operand_axis[d] >= 0) offset_by_axis[p.out_offset_operand_axis[d]] = c;
      else batch_coord[p.out_batch_pos[d]] = c;
    }
    int64_t ibase = 0;
    for (int b = 0; b < p.num_batch_dims; ++b) ibase += batch_coord[b] * p.batch_index_strides[b];
    int64_t start[kMaxDims];
    for (int d = 0; d < p.operand_rank; ++d) start[d] = 0;
    for (int c = 0; c < p.num_index_components; ++c) {
      const int ax = p.start_index_map[c];
      int64_t s = load_index_dt(p.indices, p.ids_dtype, ibase + c * p.index_vector_stride);
      const int64_t hi = p.operand_dims[ax] - p.slice_sizes[ax];
      s = s < 0 ? 0 : (s > hi ? hi : s);
      start[ax] = s;
    }
    int64_t src = 0;
    for (int d = 0; d < p.operand_rank; ++d) src += (start[d] + offset_by_axis[d]) * p.operand_strides[d];
    y[i] = operand[src];
  }
}

}  // namespace

Status gather_rows(Device* dev, const void* table, const void* ids, int ids_dtype, void* y, int64_t num_ids, int64_t num_rows,
                   int64_t row_bytes) {
  if (num_ids == 0 || row_bytes == 0) return Status::OK();
  if (row_bytes % 16 != 0 || (reinterpret_cast<uintptr_t>(table) & 15) || (reinterpret_cast<uintptr_t>(y) & 15))
    return Status::Invalid("gather_rows: rows must be 16-byte multiples and aligned");
  B200_TRY(dev->MakeCurrent());
  int64_t blocks = (num_ids + 7) / 8;
  const int64_t cap = (int64_t)dev->sm_count() * 16;
  if (blocks > cap) blocks = cap;
  gather_rows_kernel<<<(unsigned)blocks, 256, 0, dev->stream()>>>((const uint4*)table, ids, ids_dtype, (uint4*)y, num_ids, num_rows,
                                                                  row_bytes / 16);
  return dev->CheckLaunch("gather_rows");
}

Status gather_general(Device* dev, const GatherParams& p) {
  int64_t total = 1;
  for (int d = 0; d < p.out_rank; ++d) total *= p.out_dims[d];
  if (total == 0) return Status::OK();
  B200_TRY(dev->MakeCurrent());
  int64_t blocks = (total + 255) / 256;
  const int64_t cap = (int64_t)dev->sm_count() * 32;
  if (blocks > cap) blocks = cap;
  cudaStream_t s = dev->stream();
  switch (p.elt_size) {
    case 1: gather_general_kernel<uint8_t><<<(unsigned)blocks, 256, 0, s>>>(p, total); break;
    case 2: gather_general_kernel<uint16_t><<<(unsigned)blocks, 256, 0, s>>>(p, total); break;
    case 4: gather_general_kernel<uint32_t><<<(unsigned)blocks, 256, 0, s>>>(p, total); break;
    case 8: gather_general_kernel<uint64_t><<<(unsigned)blocks, 256, 0, s>>>(p, total); break;
    default: return Status::Invalid("gather: element size");
  }
  return dev->CheckLaunch("gather_general");
}

}  // namespace k
}  // namespace b200
