// Data-movement kernels: strided copy (Transpose / Slice / Reverse /
// BroadcastInDim / Concatenate / Pad), tiled 2-D transpose, fill, iota, cast.
//
// The reference realises a permutation as a chain of pairwise axis swaps, each
// a full pass over the tensor (mpsgraph bridge.m:425-465).  Here any
// permutation, slice, reversal or broadcast is ONE pass: the output is walked
// densely and the input address is computed from strides.  All HBM-bound:
// bytes = input bytes touched + output bytes.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "../kernels.h"
#include "pdl.cuh"

namespace b200 {
namespace k {

namespace {

struct ScArgs {
  const void* x;
  void* y;
  int rank;
  int64_t dims[kMaxDims];
  int64_t in_strides[kMaxDims];
  int64_t out_strides[kMaxDims];
  int64_t in_offset, out_offset;
  int64_t total;
};

// One thread per output element; T is an unsigned integer of the element size.
template <typename T>
__global__ void __launch_bounds__(256) strided_copy_kernel(const __grid_constant__ ScArgs a) {
  const T* x = reinterpret_cast<const T*>(a.x);
  T* y = reinterpret_cast<T*>(a.y);
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < a.total; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t rem = i, in = a.in_offset, out = a.out_offset;
    for (int d = a.rank - 1; d >= 0; --d) {
      const int64_t c = rem % a.dims[d];
      rem /= a.dims[d];
      in += c * a.in_strides[d];
      out += c * a.out_strides[d];
    }
    y[out] = x[in];
  }
}

// Same walk, but the innermost dim is contiguous on both sides and a multiple
// of VEC elements: moves 16 bytes per thread.
template <int ELT>
__global__ void __launch_bounds__(256) strided_copy_vec_kernel(const __grid_constant__ ScArgs a) {
  constexpr int VEC = 16 / ELT;
  const char* x = reinterpret_cast<const char*>(a.x);
  char* y = reinterpret_cast<char*>(a.y);
  const int64_t inner_vecs = a.dims[a.rank - 1] / VEC;
  const int64_t total_vecs = a.total / VEC;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total_vecs; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t rem = i / inner_vecs;
    const int64_t cv = i % inner_vecs;
    int64_t in = a.in_offset + cv * VEC, out = a.out_offset + cv * VEC;
    for (int d = a.rank - 2; d >= 0; --d) {
      const int64_t c = rem % a.dims[d];
      rem /= a.dims[d];
      in += c * a.in_strides[d];
      out += c * a.out_strides[d];
    }
    *reinterpret_cast<uint4*>(y + out * ELT) = *reinterpret_cast<const uint4*>(x + in * ELT);
  }
}

// x[batch, rows, cols] -> y[batch, cols, rows] through a padded 32x32 tile.
template <typename T>
__global__ void __launch_bounds__(256) transpose_2d_kernel(const T* x, T* y, int64_t rows, int64_t cols) {
  __shared__ T tile[32][33];
  const int64_t b = blockIdx.z;
  const T* xb = x + b * rows * cols;
  T* yb = y + b * rows * cols;
  const int64_t c0 = (int64_t)blockIdx.x * 32, r0 = (int64_t)blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
#pragma unroll
  for (int i = 0; i < 32; i += 8) {
    const int64_t r = r0 + ty + i, c = c0 + tx;
    if (r < rows && c < cols) tile[ty + i][tx] = xb[r * cols + c];
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 32; i += 8) {
    const int64_t c = c0 + ty + i, r = r0 + tx;
    if (r < rows && c < cols) yb[c * rows + r] = tile[tx][ty + i];
  }
}

template <typename T>
__global__ void __launch_bounds__(256) fill_kernel(T* y, int64_t n, T v) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) y[i] = v;
}

template <typename T> __device__ __forceinline__ T from_index(int64_t i) { return (T)i; }
template <> __device__ __forceinline__ __nv_bfloat16 from_index<__nv_bfloat16>(int64_t i) { return __float2bfloat16_rn((float)i); }
template <> __device__ __forceinline__ __half from_index<__half>(int64_t i) { return __float2half_rn((float)i); }

template <typename T>
__global__ void __launch_bounds__(256) iota_kernel(T* y, int64_t total, int64_t n, int64_t inner) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x)
    y[i] = from_index<T>((i / inner) % n);
}

// Dense [rows, cols] from rows stored with a pitch: every thread produces one ALIGNED 16-byte vector of the destination
// (the destination as a whole is one contiguous array, so its vectors never straddle anything but a row seam).  The
// source bytes of a vector lie at an arbitrary even offset: two aligned 16-byte loads and a funnel shift.  Vectors
// that straddle a row seam, and the tail, go element by element.
template <typename E>
__global__ void __launch_bounds__(256) unpad_rows_kernel(const E* __restrict__ src, E* __restrict__ dst, int64_t total, int64_t cols,
                                                         int64_t pitch) {
  constexpr int V = 16 / (int)sizeof(E);
  const int64_t nvec = (total + V - 1) / V;
  for (int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; t < nvec; t += (int64_t)gridDim.x * blockDim.x) {
    const int64_t i0 = t * V;
    const int64_t r = i0 / cols;
    const int64_t c = i0 - r * cols;
    if (c + V <= cols && i0 + V <= total) {
      const uintptr_t addr = reinterpret_cast<uintptr_t>(src + r * pitch + c);
      const uint4* a = reinterpret_cast<const uint4*>(addr & ~uintptr_t(15));
      const uint32_t sh = (uint32_t)(addr & 15);
      const uint4 v0 = __ldg(a);
      uint4 out = v0;
      if (sh != 0) {
        const uint4 v1 = __ldg(a + 1);
        const uint32_t w[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
        const uint32_t bits = (sh & 3) * 8;
        switch (sh >> 2) {
          case 0: out = make_uint4(__funnelshift_r(w[0], w[1], bits), __funnelshift_r(w[1], w[2], bits), __funnelshift_r(w[2], w[3], bits), __funnelshift_r(w[3], w[4], bits)); break;
          case 1: out = make_uint4(__funnelshift_r(w[1], w[2], bits), __funnelshift_r(w[2], w[3], bits), __funnelshift_r(w[3], w[4], bits), __funnelshift_r(w[4], w[5], bits)); break;
          case 2: out = make_uint4(__funnelshift_r(w[2], w[3], bits), __funnelshift_r(w[3], w[4], bits), __funnelshift_r(w[4], w[5], bits), __funnelshift_r(w[5], w[6], bits)); break;
          default: out = make_uint4(__funnelshift_r(w[3], w[4], bits), __funnelshift_r(w[4], w[5], bits), __funnelshift_r(w[5], w[6], bits), __funnelshift_r(w[6], w[7], bits)); break;
        }
      }
      *reinterpret_cast<uint4*>(dst + i0) = out;
    } else {
      int64_t rr = r, cc = c;
      for (int e = 0; e < V && i0 + e < total; ++e) {
        dst[i0 + e] = src[rr * pitch + cc];
        if (++cc == cols) { cc = 0; ++rr; }
      }
    }
  }
}

struct DynArgs {
  const void* x;
  const void* u;
  void* y;
  int rank;
  int64_t x_dims[kMaxDims], b_dims[kMaxDims];
  int64_t u_strides[kMaxDims];   // of the update block, in elements
  const void* starts[kMaxDims];
  int start_dtypes[kMaxDims];
};
// The update block's strides: the caller's, or dense.
static void fill_update_strides(const DynSliceParams& p, DynArgs* a) {
  int64_t dense = 1;
  for (int d = kMaxDims - 1; d >= 0; --d) {
    if (d >= p.rank) { a->u_strides[d] = 0; continue; }
    a->u_strides[d] = p.u_strided ? p.u_strides[d] : dense;
    dense *= p.b_dims[d];
  }
}
__device__ __forceinline__ int64_t load_index(const void* p, int dtype) {
  switch (dtype) {
    case B200_INT8: return *reinterpret_cast<const int8_t*>(p);
    case B200_INT16: return *reinterpret_cast<const int16_t*>(p);
    case B200_INT32: return *reinterpret_cast<const int32_t*>(p);
    case B200_INT64: return *reinterpret_cast<const int64_t*>(p);
    case B200_UINT8: return *reinterpret_cast<const uint8_t*>(p);
    case B200_UINT16: return *reinterpret_cast<const uint16_t*>(p);
    case B200_UINT32: return *reinterpret_cast<const uint32_t*>(p);
    default: {
      const uint64_t v = *reinterpret_cast<const uint64_t*>(p);
      return v > (uint64_t)INT64_MAX ? INT64_MAX : (int64_t)v;
    }
  }
}
// Clamped start of the block on every axis, computed once per CTA.
__device__ __forceinline__ void block_starts(const DynArgs& a, int64_t* start_sh) {
  if (threadIdx.x < a.rank) {
    const int d = threadIdx.x;
    int64_t v = load_index(a.starts[d], a.start_dtypes[d]);
    const int64_t hi = a.x_dims[d] - a.b_dims[d];
    v = v < 0 ? 0 : (v > hi ? hi : v);
    start_sh[d] = v;
  }
  __syncthreads();
}
template <typename E>
__global__ void __launch_bounds__(256) dynamic_slice_kernel(const DynArgs a, int64_t total) {
  __shared__ int64_t start[kMaxDims];
  block_starts(a, start);
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t rem = i, src = 0, stride = 1;
    for (int d = a.rank - 1; d >= 0; --d) {
      const int64_t c = rem % a.b_dims[d];
      rem /= a.b_dims[d];
      src += (c + start[d]) * stride;
      stride *= a.x_dims[d];
    }
    reinterpret_cast<E*>(a.y)[i] = reinterpret_cast<const E*>(a.x)[src];
  }
}
template <typename E>
__global__ void __launch_bounds__(256) dynamic_update_slice_kernel(const DynArgs a, int64_t total) {
  __shared__ int64_t start[kMaxDims];
  block_starts(a, start);
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t rem = i, usrc = 0;
    bool inside = true;
    for (int d = a.rank - 1; d >= 0; --d) {
      const int64_t c = rem % a.x_dims[d];
      rem /= a.x_dims[d];
      const int64_t r = c - start[d];
      inside = inside && r >= 0 && r < a.b_dims[d];
      usrc += r * a.u_strides[d];
    }
    reinterpret_cast<E*>(a.y)[i] = inside ? reinterpret_cast<const E*>(a.u)[usrc] : reinterpret_cast<const E*>(a.x)[i];
  }
}

struct ConcatFlatArgs {
  const void* src[kMaxConcatFlat];
  int64_t end[kMaxConcatFlat];   // running element count after each operand
  int n;
  void* dst;
};
template <typename E>
__global__ void __launch_bounds__(256) concat_flat_kernel(const ConcatFlatArgs a) {
  const int64_t total = a.end[a.n - 1];
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    int k = 0;
    while (i >= a.end[k]) ++k;
    const int64_t start = k ? a.end[k - 1] : 0;
    reinterpret_cast<E*>(a.dst)[i] = reinterpret_cast<const E*>(a.src[k])[i - start];
  }
}

unsigned grid_for(Device* dev, int64_t work_items) {
  const int64_t blocks = (work_items + 255) / 256;
  const int64_t cap = (int64_t)dev->sm_count() * 32;
  return (unsigned)(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
}

}  // namespace

Status strided_copy(Device* dev, const StridedCopyParams& p) {
  ScArgs a;
  a.x = p.x; a.y = p.y; a.in_offset = p.in_offset; a.out_offset = p.out_offset;
  // Collapse neighbouring dims that are contiguous on both sides; drop size-1 dims.
  int r = 0;
  int64_t total = 1;
  for (int d = 0; d < p.rank; ++d) {
    total *= p.dims[d];
    if (p.dims[d] == 1) continue;
    if (r > 0 && a.in_strides[r - 1] == p.in_strides[d] * p.dims[d] && a.out_strides[r - 1] == p.out_strides[d] * p.dims[d]) {
      a.dims[r - 1] *= p.dims[d];
      a.in_strides[r - 1] = p.in_strides[d];
      a.out_strides[r - 1] = p.out_strides[d];
    } else {
      a.dims[r] = p.dims[d];
      a.in_strides[r] = p.in_strides[d];
      a.out_strides[r] = p.out_strides[d];
      ++r;
    }
  }
  if (total == 0) return Status::OK();
  if (r == 0) { a.dims[0] = 1; a.in_strides[0] = 1; a.out_strides[0] = 1; r = 1; }
  a.rank = r;
  a.total = total;
  B200_TRY(dev->MakeCurrent());
  cudaStream_t s = dev->stream();
  const int es = p.elt_size;
  const int vec = 16 / es;
  bool vec_ok = a.in_strides[r - 1] == 1 && a.out_strides[r - 1] == 1 && a.dims[r - 1] % vec == 0 &&
                (a.in_offset % vec) == 0 && (a.out_offset % vec) == 0 &&
                (reinterpret_cast<uintptr_t>(a.x) & 15) == 0 && (reinterpret_cast<uintptr_t>(a.y) & 15) == 0;
  for (int d = 0; d + 1 < r && vec_ok; ++d) vec_ok = (a.in_strides[d] % vec == 0) && (a.out_strides[d] % vec == 0);
  if (vec_ok) {
    const unsigned grid = grid_for(dev, total / vec);
    switch (es) {
      case 1: strided_copy_vec_kernel<1><<<grid, 256, 0, s>>>(a); break;
      case 2: strided_copy_vec_kernel<2><<<grid, 256, 0, s>>>(a); break;
      case 4: strided_copy_vec_kernel<4><<<grid, 256, 0, s>>>(a); break;
      case 8: strided_copy_vec_kernel<8><<<grid, 256, 0, s>>>(a); break;
      default: return Status::Invalid("strided_copy: element size");
    }
  } else {
    const unsigned grid = grid_for(dev, total);
    switch (es) {
      case 1: strided_copy_kernel<uint8_t><<<grid, 256, 0, s>>>(a); break;
      case 2: strided_copy_kernel<uint16_t><<<grid, 256, 0, s>>>(a); break;
      case 4: strided_copy_kernel<uint32_t><<<grid, 256, 0, s>>>(a); break;
      case 8: strided_copy_kernel<uint64_t><<<grid, 256, 0, s>>>(a); break;
      default: return Status::Invalid("strided_copy: element size");
    }
  }
  return dev->CheckLaunch("strided_copy");
}

template <typename E>
__global__ void __launch_bounds__(256) dynamic_update_inplace_kernel(const DynArgs a, int64_t total) {
  __shared__ int64_t start[kMaxDims];
  block_starts(a, start);
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t rem = i, dst = 0, src = 0, stride = 1;
    for (int d = a.rank - 1; d >= 0; --d) {
      const int64_t c = rem % a.b_dims[d];
      rem /= a.b_dims[d];
      dst += (c + start[d]) * stride;
      src += c * a.u_strides[d];
      stride *= a.x_dims[d];
    }
    reinterpret_cast<E*>(a.y)[dst] = reinterpret_cast<const E*>(a.u)[src];
  }
}

// Two in-place updates of the same geometry (a layer's key and value caches) in one launch: blockIdx.y picks the pair.
template <typename E>
__global__ void __launch_bounds__(256) dynamic_update_inplace2_kernel(const DynArgs a0, const DynArgs a1, int64_t total) {
  __shared__ int64_t start[kMaxDims];
  pdl_launch_dependents();
  pdl_wait();
  const DynArgs& a = blockIdx.y ? a1 : a0;
  block_starts(a, start);
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t rem = i, dst = 0, src = 0, stride = 1;
    for (int d = a.rank - 1; d >= 0; --d) {
      const int64_t c = rem % a.b_dims[d];
      rem /= a.b_dims[d];
      dst += (c + start[d]) * stride;
      src += c * a.u_strides[d];
      stride *= a.x_dims[d];
    }
    reinterpret_cast<E*>(a.y)[dst] = reinterpret_cast<const E*>(a.u)[src];
  }
}

static int64_t fill_inplace_args(const DynSliceParams& p, DynArgs* a) {
  a->x = p.y; a->u = p.u; a->y = p.y; a->rank = p.rank;
  fill_update_strides(p, a);
  int64_t total = 1;
  for (int d = 0; d < kMaxDims; ++d) {
    a->x_dims[d] = d < p.rank ? p.x_dims[d] : 1;
    a->b_dims[d] = d < p.rank ? p.b_dims[d] : 1;
    a->starts[d] = d < p.rank ? p.starts[d] : nullptr;
    a->start_dtypes[d] = d < p.rank ? p.start_dtypes[d] : B200_INT32;
    if (d < p.rank) total *= p.b_dims[d];
  }
  return total;
}

Status dynamic_update_slice_inplace2(Device* dev, const DynSliceParams& p0, const DynSliceParams& p1) {
  if (p0.rank < 0 || p0.rank > kMaxDims || p1.rank != p0.rank || p1.elt_size != p0.elt_size) return Status::Invalid("dynamic slice: rank");
  DynArgs a0, a1;
  const int64_t total = fill_inplace_args(p0, &a0);
  if (fill_inplace_args(p1, &a1) != total) return Status::Invalid("dynamic slice: the two updates differ in size");
  if (total == 0) return Status::OK();
  B200_TRY(dev->MakeCurrent());
  const dim3 grid(grid_for(dev, total), 2);
  cudaStream_t s = dev->stream();
  cudaError_t e;   // launched as a programmatic dependent (a decoding step is a chain of such small kernels)
  switch (p0.elt_size) {
    case 1: e = launch_dependent_dims(dynamic_update_inplace2_kernel<uint8_t>, grid, dim3(256), 0, s, a0, a1, total); break;
    case 2: e = launch_dependent_dims(dynamic_update_inplace2_kernel<uint16_t>, grid, dim3(256), 0, s, a0, a1, total); break;
    case 4: e = launch_dependent_dims(dynamic_update_inplace2_kernel<uint32_t>, grid, dim3(256), 0, s, a0, a1, total); break;
    case 8: e = launch_dependent_dims(dynamic_update_inplace2_kernel<uint64_t>, grid, dim3(256), 0, s, a0, a1, total); break;
    default: return Status::Invalid("dynamic slice: element size");
  }
  if (e != cudaSuccess) {
    cudaGetLastError();
    return Status::Cuda(strfmt("dynamic_update_slice_inplace2: %s", cudaGetErrorString(e)));
  }
  return dev->CheckLaunch("dynamic_update_slice_inplace2");
}

Status dynamic_update_slice_inplace(Device* dev, const DynSliceParams& p) {
  if (p.rank < 0 || p.rank > kMaxDims) return Status::Invalid("dynamic slice: rank");
  DynArgs a;
  const int64_t total = fill_inplace_args(p, &a);
  if (total == 0) return Status::OK();
  B200_TRY(dev->MakeCurrent());
  const unsigned grid = grid_for(dev, total);
  cudaStream_t s = dev->stream();
  switch (p.elt_size) {
    case 1: dynamic_update_inplace_kernel<uint8_t><<<grid, 256, 0, s>>>(a, total); break;
    case 2: dynamic_update_inplace_kernel<uint16_t><<<grid, 256, 0, s>>>(a, total); break;
    case 4: dynamic_update_inplace_kernel<uint32_t><<<grid, 256, 0, s>>>(a, total); break;
    case 8: dynamic_update_inplace_kernel<uint64_t><<<grid, 256, 0, s>>>(a, total); break;
    default: return Status::Invalid("dynamic slice: element size");
  }
  return dev->CheckLaunch("dynamic_update_slice_inplace");
}

static Status dyn_launch(Device* dev, const DynSliceParams& p, bool update) {
  if (p.rank < 0 || p.rank > kMaxDims) return Status::Invalid("dynamic slice: rank");
  DynArgs a;
  a.x = p.x; a.u = p.u; a.y = p.y; a.rank = p.rank;
  fill_update_strides(p, &a);
  int64_t total = 1;
  for (int d = 0; d < kMaxDims; ++d) {
    a.x_dims[d] = d < p.rank ? p.x_dims[d] : 1;
    a.b_dims[d] = d < p.rank ? p.b_dims[d] : 1;
    a.starts[d] = d < p.rank ? p.starts[d] : nullptr;
    a.start_dtypes[d] = d < p.rank ? p.start_dtypes[d] : B200_INT32;
    if (d < p.rank) total *= update ? p.x_dims[d] : p.b_dims[d];
  }
  if (total == 0) return Status::OK();
  B200_TRY(dev->MakeCurrent());
  const unsigned grid = grid_for(dev, total);
  cudaStream_t s = dev->stream();
#define B200_DYN(E)                                                              \
  do {                                                                           \
    if (update) dynamic_update_slice_kernel<E><<<grid, 256, 0, s>>>(a, total);   \
    else dynamic_slice_kernel<E><<<grid, 256, 0, s>>>(a, total);                 \
  } while (0)
  switch (p.elt_size) {
    case 1: B200_DYN(uint8_t); break;
    case 2: B200_DYN(uint16_t); break;
    case 4: B200_DYN(uint32_t); break;
    case 8: B200_DYN(uint64_t); break;
    default: return Status::Invalid("dynamic slice: element size");
  }
#undef B200_DYN
  return dev->CheckLaunch(update ? "dynamic_update_slice" : "dynamic_slice");
}
Status dynamic_slice(Device* dev, const DynSliceParams& p) { return dyn_launch(dev, p, false); }
Status dynamic_update_slice(Device* dev, const DynSliceParams& p) { return dyn_launch(dev, p, true); }

Status concat_flat(Device* dev, const void* const* src, const int64_t* counts, int n, void* y, int elt_size) {
  if (n < 1 || n > kMaxConcatFlat) return Status::Invalid("concat_flat: 1 to 8 operands");
  ConcatFlatArgs a;
  int64_t run = 0;
  for (int i = 0; i < n; ++i) { a.src[i] = src[i]; run += counts[i]; a.end[i] = run; }
  for (int i = n; i < kMaxConcatFlat; ++i) { a.src[i] = nullptr; a.end[i] = run; }
  a.n = n;
  a.dst = y;
  if (run == 0) return Status::OK();
  B200_TRY(dev->MakeCurrent());
  const unsigned grid = grid_for(dev, run);
  cudaStream_t s = dev->stream();
  switch (elt_size) {
    case 1: concat_flat_kernel<uint8_t><<<grid, 256, 0, s>>>(a); break;
    case 2: concat_flat_kernel<uint16_t><<<grid, 256, 0, s>>>(a); break;
    case 4: concat_flat_kernel<uint32_t><<<grid, 256, 0, s>>>(a); break;
    case 8: concat_flat_kernel<uint64_t><<<grid, 256, 0, s>>>(a); break;
    default: return Status::Invalid("concat_flat: element size");
  }
  return dev->CheckLaunch("concat_flat");
}

// The source must be readable for 16 bytes past its last element (the second aligned load of the last vector).
Status unpad_rows(Device* dev, const void* src, void* dst, int64_t rows, int64_t cols, int64_t src_pitch, int elt_size) {
  const int64_t total = rows * cols;
  if (total == 0) return Status::OK();
  if (!(elt_size == 2 || elt_size == 4) || src_pitch < cols) return Status::Invalid("unpad_rows: 2- or 4-byte elements, pitch >= cols");
  if ((reinterpret_cast<uintptr_t>(dst) & 15) != 0 || (reinterpret_cast<uintptr_t>(src) & (uintptr_t)(elt_size - 1)) != 0)
    return Status::Invalid("unpad_rows: destination must be 16-byte aligned");
  B200_TRY(dev->MakeCurrent());
  const unsigned grid = grid_for(dev, (total + 16 / elt_size - 1) / (16 / elt_size));
  if (elt_size == 2) unpad_rows_kernel<uint16_t><<<grid, 256, 0, dev->stream()>>>((const uint16_t*)src, (uint16_t*)dst, total, cols, src_pitch);
  else unpad_rows_kernel<uint32_t><<<grid, 256, 0, dev->stream()>>>((const uint32_t*)src, (uint32_t*)dst, total, cols, src_pitch);
  return dev->CheckLaunch("unpad_rows");
}

Status transpose_2d(Device* dev, const void* x, void* y, int64_t batch, int64_t rows, int64_t cols, int elt_size) {
  if (batch * rows * cols == 0) return Status::OK();
  if (batch > 65535 || (rows + 31) / 32 > 65535) return Status::Unsupported("transpose_2d: grid too large");
  B200_TRY(dev->MakeCurrent());
  dim3 grid((unsigned)((cols + 31) / 32), (unsigned)((rows + 31) / 32), (unsigned)batch);
  cudaStream_t s = dev->stream();
  switch (elt_size) {
    case 1: transpose_2d_kernel<uint8_t><<<grid, 256, 0, s>>>((const uint8_t*)x, (uint8_t*)y, rows, cols); break;
    case 2: transpose_2d_kernel<uint16_t><<<grid, 256, 0, s>>>((const uint16_t*)x, (uint16_t*)y, rows, cols); break;
    case 4: transpose_2d_kernel<uint32_t><<<grid, 256, 0, s>>>((const uint32_t*)x, (uint32_t*)y, rows, cols); break;
    case 8: transpose_2d_kernel<uint64_t><<<grid, 256, 0, s>>>((const uint64_t*)x, (uint64_t*)y, rows, cols); break;
    default: return Status::Invalid("transpose_2d: element size");
  }
  return dev->CheckLaunch("transpose_2d");
}

Status fill(Device* dev, void* y, int64_t n, int elt_size, uint64_t pattern) {
  if (n == 0) return Status::OK();
  B200_TRY(dev->MakeCurrent());
  const unsigned grid = grid_for(dev, n);
  cudaStream_t s = dev->stream();
  switch (elt_size) {
    case 1: fill_kernel<uint8_t><<<grid, 256, 0, s>>>((uint8_t*)y, n, (uint8_t)pattern); break;
    case 2: fill_kernel<uint16_t><<<grid, 256, 0, s>>>((uint16_t*)y, n, (uint16_t)pattern); break;
    case 4: fill_kernel<uint32_t><<<grid, 256, 0, s>>>((uint32_t*)y, n, (uint32_t)pattern); break;
    case 8: fill_kernel<uint64_t><<<grid, 256, 0, s>>>((uint64_t*)y, n, pattern); break;
    default: return Status::Invalid("fill: element size");
  }
  return dev->CheckLaunch("fill");
}

Status iota(Device* dev, void* y, int dtype, int64_t outer, int64_t n, int64_t inner) {
  const int64_t total = outer * n * inner;
  if (total == 0) return Status::OK();
  B200_TRY(dev->MakeCurrent());
  const unsigned grid = grid_for(dev, total);
  cudaStream_t s = dev->stream();
#define IOTA_CASE(DT, T) case DT: iota_kernel<T><<<grid, 256, 0, s>>>((T*)y, total, n, inner); break;
  switch (dtype) {
    IOTA_CASE(B200_INT8, int8_t) IOTA_CASE(B200_INT16, int16_t) IOTA_CASE(B200_INT32, int32_t)
    IOTA_CASE(B200_INT64, int64_t) IOTA_CASE(B200_UINT8, uint8_t) IOTA_CASE(B200_UINT16, uint16_t)
    IOTA_CASE(B200_UINT32, uint32_t) IOTA_CASE(B200_UINT64, uint64_t) IOTA_CASE(B200_FLOAT32, float)
    IOTA_CASE(B200_FLOAT64, double) IOTA_CASE(B200_BFLOAT16, __nv_bfloat16) IOTA_CASE(B200_FLOAT16, __half)
    default: return Status::Unsupported(strfmt("iota: dtype %s", dtype_name(dtype)));
  }
#undef IOTA_CASE
  return dev->CheckLaunch("iota");
}

Status cast(Device* dev, const void* x, int src_dtype, void* y, int dst_dtype, int64_t n) {
  // A cast is a one-instruction elementwise program.
  EwProgram p;
  p.rank = 1;
  p.dims[0] = n;
  p.num_leaves = 1;
  p.leaves[0].ptr = x;
  p.leaves[0].dtype = src_dtype;
  for (int d = 0; d < kMaxDims; ++d) p.leaves[0].strides[d] = 0;
  p.leaves[0].strides[0] = 1;
  p.num_instr = 2;
  p.instr[0] = EwInstr{EW_LOAD, 0, (uint8_t)src_dtype, (uint8_t)src_dtype, 0, 0, 0, 0, 0};
  p.instr[1] = EwInstr{EW_CAST, 0, (uint8_t)dst_dtype, (uint8_t)src_dtype, 1, 0, 0, 0, 0};
  p.num_regs = 2;
  p.out_reg = 1;
  p.out_dtype = dst_dtype;
  p.out = y;
  p.wide = dtype_size(src_dtype) == 8 || dtype_size(dst_dtype) == 8;
  return ewise_run(dev, p);
}

}  // namespace k
}  // namespace b200
