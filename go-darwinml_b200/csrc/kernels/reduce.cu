// Reductions (sum / product / max / min) and arg-min/max.
//
// The input is viewed as [outer, n, inner] and reduced over n.  The reference
// calls MPSGraph's reductionSum/Product/Maximum/Minimum (mpsgraph bridge.m:706-738),
// keeps the reduced dims as 1 and reshapes them away (function.go:1164-1181);
// ArgMin/ArgMax at bridge.m:823-863.  Semantics kept: empty-axes = all axes is
// resolved by the caller; here the axis is always explicit.
//
// Accumulator types: fp32 for F16/BF16/F32, f64 for F64, the 32/64-bit integer
// of matching signedness for integers (result wraps to the storage type).
// Float max/min propagate NaN.  When outer*inner offers too little parallelism
// the n axis is split across CTAs: phase one writes partial accumulators to a
// caller-provided scratch buffer, phase two folds them.
// HBM-bound: bytes = input bytes + output bytes (+ partials, negligible).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <limits>
#include <type_traits>

#include "../kernels.h"
#include "sm100_ptx.cuh"

namespace b200 {
namespace k {

namespace {

constexpr int64_t kTargetCtas = 148 * 8;

template <typename T> struct AccOf { using type = T; };
template <> struct AccOf<__nv_bfloat16> { using type = float; };
template <> struct AccOf<__half> { using type = float; };
template <> struct AccOf<int8_t> { using type = int32_t; };
template <> struct AccOf<int16_t> { using type = int32_t; };
template <> struct AccOf<uint8_t> { using type = uint32_t; };
template <> struct AccOf<uint16_t> { using type = uint32_t; };

template <typename T, typename A> __device__ __forceinline__ A to_acc(T v) { return (A)v; }
template <> __device__ __forceinline__ float to_acc<__nv_bfloat16, float>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_acc<__half, float>(__half v) { return __half2float(v); }
template <typename A, typename T> __device__ __forceinline__ T from_acc(A v) { return (T)v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_acc<float, __nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_acc<float, __half>(float v) { return __float2half_rn(v); }

template <typename A> __device__ __forceinline__ A acc_identity(int rt) {
  switch (rt) {
    case B200_REDUCE_SUM: return (A)0;
    case B200_REDUCE_PRODUCT: return (A)1;
    case B200_REDUCE_MAX:
      if (std::is_floating_point<A>::value) return (A)(-INFINITY);
      return std::numeric_limits<A>::lowest();
    default:
      if (std::is_floating_point<A>::value) return (A)(INFINITY);
      return std::numeric_limits<A>::max();
  }
}
template <typename A> __device__ __forceinline__ A acc_combine(int rt, A a, A b) {
  switch (rt) {
    case B200_REDUCE_SUM: return a + b;
    case B200_REDUCE_PRODUCT: return a * b;
    case B200_REDUCE_MAX:
      if (std::is_floating_point<A>::value && (a != a || b != b)) return a + b;
      return a > b ? a : b;
    default:
      if (std::is_floating_point<A>::value && (a != a || b != b)) return a + b;
      return a < b ? a : b;
  }
}

template <typename A> __device__ __forceinline__ A shfl_xor_any(A v, int o) {
  if constexpr (sizeof(A) == 8) {
    long long x = *reinterpret_cast<long long*>(&v);
    x = __shfl_xor_sync(0xffffffffu, x, o);
    return *reinterpret_cast<A*>(&x);
  } else {
    int x = *reinterpret_cast<int*>(&v);
    x = __shfl_xor_sync(0xffffffffu, x, o);
    return *reinterpret_cast<A*>(&x);
  }
}
template <typename A> __device__ __forceinline__ A warp_fold(int rt, A v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = acc_combine<A>(rt, v, shfl_xor_any<A>(v, o));
  return v;
}
// Folds over the 256 threads of a CTA; result valid in thread 0.
template <typename A> __device__ __forceinline__ A cta_fold(int rt, A v) {
  __shared__ unsigned long long sm[8];
  v = warp_fold<A>(rt, v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) *reinterpret_cast<A*>(&sm[warp]) = v;
  __syncthreads();
  A t = (lane < 8) ? *reinterpret_cast<A*>(&sm[lane]) : acc_identity<A>(rt);
  return warp_fold<A>(rt, t);
}

// inner == 1.  grid = (chunks, outer); each CTA folds one chunk of one row.
// chunks == 1: writes T to y[row]; else writes A to partial[row * chunks + chunk].
template <typename T, typename A>
__global__ void __launch_bounds__(256) reduce_rows_kernel(const T* x, void* out, int rt, int64_t n, int64_t chunk_len, int chunks) {
  const int64_t row = blockIdx.y, chunk = blockIdx.x;
  const int64_t lo = chunk * chunk_len;
  int64_t hi = lo + chunk_len;
  if (hi > n) hi = n;
  const T* xr = x + row * n;
  A acc = acc_identity<A>(rt);
  int64_t j = lo + threadIdx.x;
  for (; j + 768 < hi; j += 1024) {
    const A a0 = to_acc<T, A>(xr[j]), a1 = to_acc<T, A>(xr[j + 256]), a2 = to_acc<T, A>(xr[j + 512]), a3 = to_acc<T, A>(xr[j + 768]);
    acc = acc_combine<A>(rt, acc, acc_combine<A>(rt, acc_combine<A>(rt, a0, a1), acc_combine<A>(rt, a2, a3)));
  }
  for (; j < hi; j += 256) acc = acc_combine<A>(rt, acc, to_acc<T, A>(xr[j]));
  acc = cta_fold<A>(rt, acc);
  if (threadIdx.x == 0) {
    if (chunks == 1) reinterpret_cast<T*>(out)[row] = from_acc<A, T>(acc);
    else reinterpret_cast<A*>(out)[row * chunks + chunk] = acc;
  }
}

// inner == 1, short rows: one warp per row, 8 rows per CTA.
template <typename T, typename A>
__global__ void __launch_bounds__(256) reduce_rows_warp_kernel(const T* x, T* y, int rt, int64_t outer, int64_t n) {
  const int64_t row = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= outer) return;
  const int lane = threadIdx.x & 31;
  const T* xr = x + row * n;
  A acc = acc_identity<A>(rt);
  for (int64_t j = lane; j < n; j += 32) acc = acc_combine<A>(rt, acc, to_acc<T, A>(xr[j]));
  acc = warp_fold<A>(rt, acc);
  if (lane == 0) y[row] = from_acc<A, T>(acc);
}

// inner > 1.  One thread per (outer, inner) pair; grid.y splits n into chunks.
template <typename T, typename A>
__global__ void __launch_bounds__(256) reduce_cols_kernel(const T* x, void* out, int rt, int64_t outer, int64_t n, int64_t inner,
                                                           int64_t chunk_len, int chunks) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= outer * inner) return;
  const int64_t o = idx / inner, i = idx % inner;
  const int64_t chunk = blockIdx.y;
  const int64_t lo = chunk * chunk_len;
  int64_t hi = lo + chunk_len;
  if (hi > n) hi = n;
  const T* xp = x + o * n * inner + i;
  A acc = acc_identity<A>(rt);
  int64_t j = lo;
  for (; j + 3 < hi; j += 4) {
    const A a0 = to_acc<T, A>(xp[j * inner]), a1 = to_acc<T, A>(xp[(j + 1) * inner]), a2 = to_acc<T, A>(xp[(j + 2) * inner]),
            a3 = to_acc<T, A>(xp[(j + 3) * inner]);
    acc = acc_combine<A>(rt, acc, acc_combine<A>(rt, acc_combine<A>(rt, a0, a1), acc_combine<A>(rt, a2, a3)));
  }
  for (; j < hi; ++j) acc = acc_combine<A>(rt, acc, to_acc<T, A>(xp[j * inner]));
  if (chunks == 1) reinterpret_cast<T*>(out)[idx] = from_acc<A, T>(acc);
  else reinterpret_cast<A*>(out)[chunk * outer * inner + idx] = acc;
}

// y[j] = fold_c partial[j * stride_j + c * stride_c]
template <typename T, typename A>
__global__ void __launch_bounds__(256) reduce_finalize_kernel(const A* partial, T* y, int rt, int64_t count, int chunks,
                                                               int64_t stride_j, int64_t stride_c) {
  const int64_t j = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= count) return;
  A acc = acc_identity<A>(rt);
  for (int c = 0; c < chunks; ++c) acc = acc_combine<A>(rt, acc, partial[j * stride_j + c * stride_c]);
  y[j] = from_acc<A, T>(acc);
}

struct Split {
  int chunks;
  int64_t chunk_len;
};
Split plan_split(int64_t outer, int64_t n, int64_t inner) {
  int64_t chunks = 1;
  if (n <= 0) return Split{1, 1};
  if (inner == 1) {
    if (outer < kTargetCtas && n >= 8192) {
      chunks = (kTargetCtas + outer - 1) / outer;
      const int64_t max_chunks = (n + 4095) / 4096;
      if (chunks > max_chunks) chunks = max_chunks;
    }
  } else {
    const int64_t blocks_x = (outer * inner + 255) / 256;
    if (blocks_x < kTargetCtas && n >= 256) {
      chunks = (kTargetCtas + blocks_x - 1) / blocks_x;
      const int64_t max_chunks = (n + 63) / 64;
      if (chunks > max_chunks) chunks = max_chunks;
    }
  }
  if (chunks < 1) chunks = 1;
  if (chunks > 65535) chunks = 65535;
  int64_t chunk_len = (n + chunks - 1) / chunks;
  chunks = (int)((n + chunk_len - 1) / chunk_len);
  return Split{(int)chunks, chunk_len};
}

template <typename T>
Status reduce_typed(Device* dev, const void* xv, void* yv, int rt, int64_t outer, int64_t n, int64_t inner, void* scratch,
                    int64_t scratch_bytes) {
  using A = typename AccOf<T>::type;
  const T* x = reinterpret_cast<const T*>(xv);
  T* y = reinterpret_cast<T*>(yv);
  cudaStream_t s = dev->stream();
  const Split sp = plan_split(outer, n, inner);
  if (sp.chunks > 1) {
    const int64_t need = outer * inner * sp.chunks * (int64_t)sizeof(A);
    if (!scratch || scratch_bytes < need) return Status::Invalid("reduce: scratch buffer too small");
  }
  if (inner == 1) {
    if (outer > 65535 || (sp.chunks == 1 && n <= 1024 && outer >= 64)) {
      if (sp.chunks != 1) return Status::Unsupported("reduce: too many rows for a split reduction");
      reduce_rows_warp_kernel<T, A><<<(unsigned)((outer + 7) / 8), 256, 0, s>>>(x, y, rt, outer, n);
      return dev->CheckLaunch("reduce_rows_warp");
    }
    dim3 grid((unsigned)sp.chunks, (unsigned)outer);
    reduce_rows_kernel<T, A><<<grid, 256, 0, s>>>(x, sp.chunks == 1 ? (void*)y : scratch, rt, n, sp.chunk_len, sp.chunks);
    B200_TRY(dev->CheckLaunch("reduce_rows"));
    if (sp.chunks > 1) {
      reduce_finalize_kernel<T, A><<<(unsigned)((outer + 255) / 256), 256, 0, s>>>(reinterpret_cast<const A*>(scratch), y, rt, outer,
                                                                                 sp.chunks, sp.chunks, 1);
      return dev->CheckLaunch("reduce_finalize");
    }
    return Status::OK();
  }
  const int64_t count = outer * inner;
  dim3 grid((unsigned)((count + 255) / 256), (unsigned)sp.chunks);
  reduce_cols_kernel<T, A><<<grid, 256, 0, s>>>(x, sp.chunks == 1 ? (void*)y : scratch, rt, outer, n, inner, sp.chunk_len, sp.chunks);
  B200_TRY(dev->CheckLaunch("reduce_cols"));
  if (sp.chunks > 1) {
    reduce_finalize_kernel<T, A><<<(unsigned)((count + 255) / 256), 256, 0, s>>>(reinterpret_cast<const A*>(scratch), y, rt, count,
                                                                               sp.chunks, 1, count);
    return dev->CheckLaunch("reduce_finalize");
  }
  return Status::OK();
}

// ---- arg-min / arg-max ------------------------------------------------------
// Ordering: lowest index wins ties; NaN counts as the extreme for both min and
// max (so the first NaN wins), which is NumPy's argmax/argmin behaviour.
template <typename A> struct Best {
  A v;
  int64_t i;
};
template <typename A> __device__ __forceinline__ bool better(bool is_min, A cv, int64_t ci, A bv, int64_t bi) {
  // is (cv, ci) better than (bv, bi)?
  if (bi < 0) return true;
  if (ci < 0) return false;
  const bool cn = (cv != cv), bn = (bv != bv);
  if (cn || bn) {
    if (cn && bn) return ci < bi;
    return cn;
  }
  if (cv == bv) return ci < bi;
  return is_min ? (cv < bv) : (cv > bv);
}

// One row per cluster (grid (outer, C), cluster (1, C)): a CTA scans its share of the row, four independent loads per
// thread in flight, and the CTAs' winners meet in CTA 0 through distributed shared memory.  A long row with few rows in
// all (an argmax over the vocabulary of a decoding step) would otherwise be one CTA's serial scan.
template <typename T, typename A, typename O>
__global__ void __launch_bounds__(1024) argminmax_rows_kernel(const T* x, O* y, bool is_min, int64_t outer, int64_t n) {
  __shared__ unsigned long long sv[32];
  __shared__ long long si[32];
  __shared__ unsigned long long cta_v;
  __shared__ long long cta_i;
  const int64_t row = blockIdx.x;
  const int rank = blockIdx.y, csize = gridDim.y;
  const int64_t chunk = (n + csize - 1) / csize;
  const int64_t begin = rank * chunk, end = begin + chunk < n ? begin + chunk : n;
  const T* xr = x + row * n;
  A bv = (A)0;
  int64_t bi = -1;
  const int64_t step = blockDim.x;
  for (int64_t j = begin + threadIdx.x; j < end; j += 4 * step) {
    A v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) v[u] = j + u * step < end ? to_acc<T, A>(xr[j + u * step]) : (A)0;
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (j + u * step < end && better<A>(is_min, v[u], j + u * step, bv, bi)) { bv = v[u]; bi = j + u * step; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const A ov = shfl_xor_any<A>(bv, o);
    const int64_t oi = __shfl_xor_sync(0xffffffffu, (long long)bi, o);
    if (better<A>(is_min, ov, oi, bv, bi)) { bv = ov; bi = oi; }
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  if (lane == 0) { sv[warp] = 0; *reinterpret_cast<A*>(&sv[warp]) = bv; si[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    bv = (lane < warps) ? *reinterpret_cast<A*>(&sv[lane]) : (A)0;
    bi = (lane < warps) ? si[lane] : -1;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const A ov = shfl_xor_any<A>(bv, o);
      const int64_t oi = __shfl_xor_sync(0xffffffffu, (long long)bi, o);
      if (better<A>(is_min, ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) {
      if (csize == 1) y[row] = (O)bi;
      else { cta_v = 0; *reinterpret_cast<A*>(&cta_v) = bv; cta_i = bi; }
    }
  }
  if (csize == 1) return;
  sm100::cluster_sync_all();
  if (rank == 0 && threadIdx.x == 0) {
    const uint32_t va = sm100::smem_u32(&cta_v), ia = sm100::smem_u32(&cta_i);
    for (int r = 1; r < csize; ++r) {
      unsigned long long rv;
      long long ri;
      asm volatile("ld.shared::cluster.u64 %0, [%1];" : "=l"(rv) : "r"(sm100::map_to_cta(va, (uint32_t)r)) : "memory");
      asm volatile("ld.shared::cluster.s64 %0, [%1];" : "=l"(ri) : "r"(sm100::map_to_cta(ia, (uint32_t)r)) : "memory");
      const A ov = *reinterpret_cast<A*>(&rv);
      if (better<A>(is_min, ov, (int64_t)ri, bv, bi)) { bv = ov; bi = ri; }
    }
    y[row] = (O)bi;
  }
  sm100::cluster_sync_all();   // nobody leaves while its winner may still be read
}

template <typename T, typename A, typename O>
__global__ void __launch_bounds__(256) argminmax_cols_kernel(const T* x, O* y, bool is_min, int64_t outer, int64_t n, int64_t inner) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= outer * inner) return;
  const int64_t o = idx / inner, i = idx % inner;
  const T* xp = x + o * n * inner + i;
  A bv = (A)0;
  int64_t bi = -1;
  for (int64_t j = 0; j < n; ++j) {
    const A v = to_acc<T, A>(xp[j * inner]);
    if (better<A>(is_min, v, j, bv, bi)) { bv = v; bi = j; }
  }
  y[idx] = (O)bi;
}

template <typename T, typename O>
Status argminmax_typed2(Device* dev, const void* xv, void* yv, bool is_min, int64_t outer, int64_t n, int64_t inner) {
  using A = typename AccOf<T>::type;
  cudaStream_t s = dev->stream();
  if (inner == 1) {
    // CTAs per row: enough to give every SM a share when the rows are few and long; at least 4096 elements each
    int64_t c = 1;
    if (outer < dev->sm_count() && n >= 8192) {
      c = (dev->sm_count() + outer - 1) / outer;
      if (c > 8) c = 8;
      if (c > n / 4096) c = n / 4096;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)outer, (unsigned)c);
    cfg.blockDim = dim3(n >= 4096 ? 1024 : 256);
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1; attr[0].val.clusterDim.y = (unsigned)c; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, argminmax_rows_kernel<T, A, O>, (const T*)xv, (O*)yv, is_min, outer, n);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return Status::Cuda(strfmt("argminmax_rows: %s", cudaGetErrorString(e)));
    }
    return dev->CheckLaunch("argminmax_rows");
  }
  const int64_t count = outer * inner;
  argminmax_cols_kernel<T, A, O><<<(unsigned)((count + 255) / 256), 256, 0, s>>>((const T*)xv, (O*)yv, is_min, outer, n, inner);
  return dev->CheckLaunch("argminmax_cols");
}
template <typename T>
Status argminmax_typed(Device* dev, const void* x, void* y, int out_dtype, bool is_min, int64_t outer, int64_t n, int64_t inner) {
  switch (out_dtype) {
    case B200_INT32: case B200_UINT32: return argminmax_typed2<T, int32_t>(dev, x, y, is_min, outer, n, inner);
    case B200_INT64: case B200_UINT64: return argminmax_typed2<T, int64_t>(dev, x, y, is_min, outer, n, inner);
    case B200_INT16: case B200_UINT16: return argminmax_typed2<T, int16_t>(dev, x, y, is_min, outer, n, inner);
    case B200_INT8: case B200_UINT8: return argminmax_typed2<T, int8_t>(dev, x, y, is_min, outer, n, inner);
    default: return Status::Unsupported(strfmt("ArgMinMax: output dtype %s", dtype_name(out_dtype)));
  }
}

}  // namespace

int64_t reduce_scratch_bytes(int dtype, int64_t outer, int64_t n, int64_t inner) {
  (void)dtype;
  const Split sp = plan_split(outer, n, inner);
  if (sp.chunks <= 1) return 0;
  return outer * inner * sp.chunks * 8;
}

Status reduce(Device* dev, const void* x, void* y, int dtype, int reduce_type, int64_t outer, int64_t n, int64_t inner,
              void* scratch, int64_t scratch_bytes) {
  if (outer * inner == 0) return Status::OK();
  if (reduce_type < 0 || reduce_type > 3) return Status::Invalid("reduce: bad reduce type");
  B200_TRY(dev->MakeCurrent());
#define RCASE(DT, T) case DT: return reduce_typed<T>(dev, x, y, reduce_type, outer, n, inner, scratch, scratch_bytes);
  switch (dtype) {
    RCASE(B200_FLOAT32, float) RCASE(B200_FLOAT64, double) RCASE(B200_BFLOAT16, __nv_bfloat16) RCASE(B200_FLOAT16, __half)
    RCASE(B200_INT8, int8_t) RCASE(B200_INT16, int16_t) RCASE(B200_INT32, int32_t) RCASE(B200_INT64, int64_t)
    RCASE(B200_UINT8, uint8_t) RCASE(B200_UINT16, uint16_t) RCASE(B200_UINT32, uint32_t) RCASE(B200_UINT64, uint64_t)
    RCASE(B200_BOOL, uint8_t)
    default: return Status::Unsupported(strfmt("reduce: dtype %s", dtype_name(dtype)));
  }
#undef RCASE
}

Status arg_min_max(Device* dev, const void* x, void* y, int dtype, int out_dtype, bool is_min, int64_t outer, int64_t n,
                   int64_t inner) {
  if (outer * inner == 0) return Status::OK();
  if (n == 0) return Status::Invalid("ArgMinMax: reduced axis has size 0");
  if (inner == 1 && outer > 0x7fffffffLL) return Status::Unsupported("ArgMinMax: too many rows");
  B200_TRY(dev->MakeCurrent());
#define ACASE(DT, T) case DT: return argminmax_typed<T>(dev, x, y, out_dtype, is_min, outer, n, inner);
  switch (dtype) {
    ACASE(B200_FLOAT32, float) ACASE(B200_FLOAT64, double) ACASE(B200_BFLOAT16, __nv_bfloat16) ACASE(B200_FLOAT16, __half)
    ACASE(B200_INT8, int8_t) ACASE(B200_INT16, int16_t) ACASE(B200_INT32, int32_t) ACASE(B200_INT64, int64_t)
    ACASE(B200_UINT8, uint8_t) ACASE(B200_UINT16, uint16_t) ACASE(B200_UINT32, uint32_t) ACASE(B200_UINT64, uint64_t)
    default: return Status::Unsupported(strfmt("ArgMinMax: dtype %s", dtype_name(dtype)));
  }
#undef ACASE
}

}  // namespace k
}  // namespace b200
