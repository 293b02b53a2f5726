// ScatterSum / ScatterMax / ScatterMin: XLA scatter with a combiner.
//
// The reference lowers these to MPSGraph's scatterAlongAxis (one indexed axis; the index tensor is first broadcast
// to the updates' full shape) or scatterND after transposing the operand (mpsgraph gather.go:441-641).  Here one
// kernel handles every form: the result starts as a copy of the operand, then one thread per element of `updates`
// works out the operand position its scatter indices name and combines the value in with an atomic: native atomics
// where the hardware has them (add on f32 / f64 / 16-bit floats / 32- and 64-bit integers, max / min on 32- and 64-bit
// integers), otherwise a compare-and-swap loop on the enclosing 32- or 64-bit word.  Float max / min propagate NaN.
// An element whose position falls outside the operand is dropped.
// Order of combination is whatever the hardware makes it: integer results and max / min are exact; a float sum that
// receives several updates in one position can differ in its last bits from run to run.
// HBM-bound: bytes = operand in + out, updates and indices once, plus the atomics' read-modify-writes (L2).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "../kernels.h"

namespace b200 {
namespace k {

namespace {

__device__ __forceinline__ int64_t load_index(const void* p, int dtype, int64_t i) {
  switch (dtype) {
    case B200_INT8: return reinterpret_cast<const int8_t*>(p)[i];
    case B200_INT16: return reinterpret_cast<const int16_t*>(p)[i];
    case B200_INT32: return reinterpret_cast<const int32_t*>(p)[i];
    case B200_INT64: return reinterpret_cast<const int64_t*>(p)[i];
    case B200_UINT8: return reinterpret_cast<const uint8_t*>(p)[i];
    case B200_UINT16: return reinterpret_cast<const uint16_t*>(p)[i];
    case B200_UINT32: return reinterpret_cast<const uint32_t*>(p)[i];
    default: {
      const uint64_t v = reinterpret_cast<const uint64_t*>(p)[i];
      return v > (uint64_t)INT64_MAX ? INT64_MAX : (int64_t)v;
    }
  }
}

// combine(old, v) for one element type; F = float-like (NaN rules), MODE: 0 sum, 1 max, 2 min
template <typename T, int MODE> __device__ __forceinline__ T combine(T a, T b) {
  if (MODE == 0) return a + b;
  if (MODE == 1) return a > b ? a : b;
  return a < b ? a : b;
}
template <int MODE> __device__ __forceinline__ float combine_f(float a, float b) {
  if (MODE == 0) return a + b;
  if (a != a || b != b) return a + b;
  return MODE == 1 ? fmaxf(a, b) : fminf(a, b);
}
template <int MODE> __device__ __forceinline__ double combine_d(double a, double b) {
  if (MODE == 0) return a + b;
  if (a != a || b != b) return a + b;
  return MODE == 1 ? fmax(a, b) : fmin(a, b);
}

// Compare-and-swap loop on the 32-bit word that holds a 1-, 2- or 4-byte element.  conv: bits -> bits.
template <typename F>
__device__ __forceinline__ void cas_update(void* base, int64_t elem, int elt_bytes, F f) {
  const uintptr_t addr = reinterpret_cast<uintptr_t>(base) + (uintptr_t)elem * elt_bytes;
  unsigned int* word = reinterpret_cast<unsigned int*>(addr & ~uintptr_t(3));
  const unsigned shift = (unsigned)(addr & 3) * 8;
  const unsigned int mask = elt_bytes == 4 ? 0xffffffffu : (((1u << (elt_bytes * 8)) - 1u) << shift);
  unsigned int old = *word, assumed;
  do {
    assumed = old;
    const unsigned int cur = (assumed & mask) >> shift;
    const unsigned int next = (f(cur) << shift) & mask;
    if (next == (assumed & mask)) return;   // nothing to change (max / min that keeps the old value)
    old = atomicCAS(word, assumed, (assumed & ~mask) | next);
  } while (old != assumed);
}
template <typename F>
__device__ __forceinline__ void cas_update64(void* base, int64_t elem, F f) {
  unsigned long long* word = reinterpret_cast<unsigned long long*>(base) + elem;
  unsigned long long old = *word, assumed;
  do {
    assumed = old;
    const unsigned long long next = f(assumed);
    if (next == assumed) return;
    old = atomicCAS(word, assumed, next);
  } while (old != assumed);
}

template <int MODE>
__device__ __forceinline__ void apply(void* out, int64_t pos, const void* upd, int64_t ui, int dtype) {
  switch (dtype) {
    case B200_FLOAT32: {
      const float v = reinterpret_cast<const float*>(upd)[ui];
      if (MODE == 0) atomicAdd(reinterpret_cast<float*>(out) + pos, v);
      else cas_update(out, pos, 4, [v](unsigned int c) { return __float_as_uint(combine_f<MODE>(__uint_as_float(c), v)); });
      break;
    }
    case B200_FLOAT64: {
      const double v = reinterpret_cast<const double*>(upd)[ui];
      if (MODE == 0) atomicAdd(reinterpret_cast<double*>(out) + pos, v);
      else cas_update64(out, pos, [v](unsigned long long c) { return (unsigned long long)__double_as_longlong(combine_d<MODE>(__longlong_as_double((long long)c), v)); });
      break;
    }
    case B200_BFLOAT16: {
      const __nv_bfloat16 v = reinterpret_cast<const __nv_bfloat16*>(upd)[ui];
      if (MODE == 0) atomicAdd(reinterpret_cast<__nv_bfloat16*>(out) + pos, v);
      else {
        const float fv = __bfloat162float(v);
        cas_update(out, pos, 2, [fv](unsigned int c) {
          const float r = combine_f<MODE>(__uint_as_float(c << 16), fv);
          return (unsigned int)(__float_as_uint(r) >> 16);   // the result is one of the two 16-bit inputs (or a NaN): the shift is exact
        });
      }
      break;
    }
    case B200_FLOAT16: {
      const __half v = reinterpret_cast<const __half*>(upd)[ui];
      if (MODE == 0) atomicAdd(reinterpret_cast<__half*>(out) + pos, v);
      else {
        const float fv = __half2float(v);
        cas_update(out, pos, 2, [fv](unsigned int c) {
          const float r = combine_f<MODE>(__half2float(__ushort_as_half((unsigned short)c)), fv);
          return (unsigned int)__half_as_ushort(__float2half_rn(r));
        });
      }
      break;
    }
    case B200_INT32: {
      const int v = reinterpret_cast<const int*>(upd)[ui];
      int* p = reinterpret_cast<int*>(out) + pos;
      if (MODE == 0) atomicAdd(p, v); else if (MODE == 1) atomicMax(p, v); else atomicMin(p, v);
      break;
    }
    case B200_UINT32: {
      const unsigned v = reinterpret_cast<const unsigned*>(upd)[ui];
      unsigned* p = reinterpret_cast<unsigned*>(out) + pos;
      if (MODE == 0) atomicAdd(p, v); else if (MODE == 1) atomicMax(p, v); else atomicMin(p, v);
      break;
    }
    case B200_INT64: {
      const long long v = reinterpret_cast<const long long*>(upd)[ui];
      long long* p = reinterpret_cast<long long*>(out) + pos;
      if (MODE == 0) atomicAdd(reinterpret_cast<unsigned long long*>(p), (unsigned long long)v);
      else if (MODE == 1) atomicMax(p, v); else atomicMin(p, v);
      break;
    }
    case B200_UINT64: {
      const unsigned long long v = reinterpret_cast<const unsigned long long*>(upd)[ui];
      unsigned long long* p = reinterpret_cast<unsigned long long*>(out) + pos;
      if (MODE == 0) atomicAdd(p, v); else if (MODE == 1) atomicMax(p, v); else atomicMin(p, v);
      break;
    }
    case B200_INT8: {
      const int v = reinterpret_cast<const int8_t*>(upd)[ui];
      cas_update(out, pos, 1, [v](unsigned int c) { return (unsigned int)(uint8_t)combine<int, MODE>((int)(int8_t)c, v); });
      break;
    }
    case B200_UINT8: {
      const unsigned v = reinterpret_cast<const uint8_t*>(upd)[ui];
      cas_update(out, pos, 1, [v](unsigned int c) { return (unsigned int)(uint8_t)combine<unsigned, MODE>(c, v); });
      break;
    }
    case B200_INT16: {
      const int v = reinterpret_cast<const int16_t*>(upd)[ui];
      cas_update(out, pos, 2, [v](unsigned int c) { return (unsigned int)(uint16_t)combine<int, MODE>((int)(int16_t)c, v); });
      break;
    }
    case B200_UINT16: {
      const unsigned v = reinterpret_cast<const uint16_t*>(upd)[ui];
      cas_update(out, pos, 2, [v](unsigned int c) { return (unsigned int)(uint16_t)combine<unsigned, MODE>(c, v); });
      break;
    }
    default: break;
  }
}

template <int MODE>
__global__ void __launch_bounds__(256) scatter_kernel(const __grid_constant__ ScatterParams p, int64_t total) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    // coordinates of this update element
    int64_t rem = i;
    int64_t u[kMaxDims];
    for (int d = p.update_rank - 1; d >= 0; --d) {
      u[d] = rem % p.update_dims[d];
      rem /= p.update_dims[d];
    }
    // its index vector
    int64_t ibase = 0;
    for (int k = 0; k < p.num_batch_dims; ++k) ibase += u[p.batch_update_axis[k]] * p.batch_index_strides[k];
    int64_t coord[kMaxDims];
    for (int d = 0; d < p.operand_rank; ++d) coord[d] = 0;
    for (int c = 0; c < p.num_index_components; ++c)
      coord[p.scatter_axes_to_operand_axes[c]] = load_index(p.indices, p.ids_dtype, ibase + c * p.index_vector_stride);
    for (int j = 0; j < p.num_window_axes; ++j) coord[p.window_operand_axis[j]] += u[p.window_update_axis[j]];
    int64_t pos = 0;
    bool inside = true;
    for (int d = 0; d < p.operand_rank; ++d) {
      inside = inside && coord[d] >= 0 && coord[d] < p.operand_dims[d];
      pos += coord[d] * p.operand_strides[d];
    }
    if (inside) apply<MODE>(p.y, pos, p.updates, i, p.dtype);
  }
}

}  // namespace

Status scatter(Device* dev, const ScatterParams& p) {
  int64_t total = 1;
  for (int d = 0; d < p.update_rank; ++d) total *= p.update_dims[d];
  if (total == 0) return Status::OK();
  B200_TRY(dev->MakeCurrent());
  int64_t blocks = (total + 255) / 256;
  const int64_t cap = (int64_t)dev->sm_count() * 16;
  if (blocks > cap) blocks = cap;
  cudaStream_t s = dev->stream();
  switch (p.mode) {
    case 0: scatter_kernel<0><<<(unsigned)blocks, 256, 0, s>>>(p, total); break;
    case 1: scatter_kernel<1><<<(unsigned)blocks, 256, 0, s>>>(p, total); break;
    default: scatter_kernel<2><<<(unsigned)blocks, 256, 0, s>>>(p, total); break;
  }
  return dev->CheckLaunch("scatter");
}

}  // namespace k
}  // namespace b200
