// Rotary position embedding, rotate-half form, as one pass:
//   y = x * c + swap_halves(x) * s          on the last axis, per head of `head_dim` elements,
// each product and the sum rounded to the storage type (the value a Mul, Mul, Add chain gives).  The reference has no
// such op: GoMLX models spell it with Slice, Concatenate, Mul and Add, which the reference runs as separate MPSGraph
// nodes (mpsgraph function.go:1026-1125 for the slicing, :658-963 for the arithmetic).
//
// HBM-bound: reads x once (from inside a wider buffer when the caller says so: the QKV projection's output), the
// tables (L2-resident: they repeat per batch entry), writes y once.  16-byte vectors; a vector and its partner half
// a head away are both loaded by the same thread.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "../kernels.h"
#include "pdl.cuh"

namespace b200 {
namespace k {

namespace {

template <typename T> struct RopeCvt;
template <> struct RopeCvt<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void unpack(const uint4& q, float* v) {
    v[0] = __uint_as_float(q.x); v[1] = __uint_as_float(q.y); v[2] = __uint_as_float(q.z); v[3] = __uint_as_float(q.w);
  }
  static __device__ __forceinline__ uint4 pack(const float* v) {
    return make_uint4(__float_as_uint(v[0]), __float_as_uint(v[1]), __float_as_uint(v[2]), __float_as_uint(v[3]));
  }
  static __device__ __forceinline__ float round(float v) { return v; }
  // intrinsics: the compiler must not contract the products into an FMA (fp32 would round once)
  static __device__ __forceinline__ uint4 combine(const uint4& qx, const uint4& qp, const uint4& qc, const uint4& qs) {
    float x[4], p[4], c[4], s[4], r[4];
    unpack(qx, x); unpack(qp, p); unpack(qc, c); unpack(qs, s);
#pragma unroll
    for (int e = 0; e < 4; ++e) r[e] = __fadd_rn(__fmul_rn(x[e], c[e]), __fmul_rn(p[e], s[e]));
    return pack(r);
  }
};
template <> struct RopeCvt<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void unpack(const uint4& q, float* v) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
  }
  static __device__ __forceinline__ uint4 pack(const float* v) {
    uint4 q;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    return q;
  }
  static __device__ __forceinline__ float round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
  // The two products are rounded to the storage type by the packed 16-bit multiply itself (the exact product of two
  // 8-bit significands, rounded once: the value fp32 multiply + conversion gives); the sum is taken in fp32 and rounded
  // by the packing conversion.  One conversion per PAIR instead of seven per pair: scalar conversions run at a fraction of
  // the ALU rate and made this kernel compute-bound at a third of the memory rate.
  static __device__ __forceinline__ uint4 combine(const uint4& qx, const uint4& qp, const uint4& qc, const uint4& qs) {
    const __nv_bfloat162* x = reinterpret_cast<const __nv_bfloat162*>(&qx);
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&qp);
    const __nv_bfloat162* c = reinterpret_cast<const __nv_bfloat162*>(&qc);
    const __nv_bfloat162* s = reinterpret_cast<const __nv_bfloat162*>(&qs);
    uint4 q;
    __nv_bfloat162* r = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 a = __bfloat1622float2(__hmul2_rn(x[i], c[i])), b = __bfloat1622float2(__hmul2_rn(p[i], s[i]));
      r[i] = __floats2bfloat162_rn(__fadd_rn(a.x, b.x), __fadd_rn(a.y, b.y));
    }
    return q;
  }
};
template <> struct RopeCvt<__half> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void unpack(const uint4& q, float* v) {
    const __half2* h = reinterpret_cast<const __half2*>(&q);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __half22float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
  }
  static __device__ __forceinline__ uint4 pack(const float* v) {
    uint4 q;
    __half2* h = reinterpret_cast<__half2*>(&q);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
    return q;
  }
  static __device__ __forceinline__ float round(float v) { return __half2float(__float2half_rn(v)); }
  // as for bf16: an 11-bit by 11-bit product is exact in fp32, so the packed multiply rounds it exactly once
  static __device__ __forceinline__ uint4 combine(const uint4& qx, const uint4& qp, const uint4& qc, const uint4& qs) {
    const __half2* x = reinterpret_cast<const __half2*>(&qx);
    const __half2* p = reinterpret_cast<const __half2*>(&qp);
    const __half2* c = reinterpret_cast<const __half2*>(&qc);
    const __half2* s = reinterpret_cast<const __half2*>(&qs);
    uint4 q;
    __half2* r = reinterpret_cast<__half2*>(&q);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 a = __half22float2(__hmul2_rn(x[i], c[i])), b = __half22float2(__hmul2_rn(p[i], s[i]));
      r[i] = __floats2half2_rn(__fadd_rn(a.x, b.x), __fadd_rn(a.y, b.y));
    }
    return q;
  }
};

struct RopeArgs {
  const uint4* x;
  const uint4* c;
  const uint4* s;
  uint4* y;
  int64_t rows;
  int64_t total_vecs;     // rows * cols / N
  uint32_t row_vecs;      // cols / N
  uint32_t head_vecs;     // head_dim / N
  int64_t x_pitch_vecs;
  int64_t c_period_vecs, s_period_vecs;
  uint32_t c_head_rows, s_head_rows;      // > 0: the table is [that many rows, head_dim], shared by the heads
  uint32_t c_period_rows, s_period_rows;  // > 0: the table repeats every that many whole rows of x
};

// Thread (tx, ty) owns vector tx (+ k * blockDim.x) of the rows blockIdx.x * blockDim.y + ty (+ grid stride): the column
// work (position inside the head, the partner half a head away) is done once per thread, the row work is one 32-bit
// modulo for the table row, and nothing divides per vector.  Two rows per iteration, all eight loads issued before the
// first use, keep enough bytes in flight.
template <typename T>
__global__ void __launch_bounds__(256) rope_kernel(const RopeArgs a) {
  using C = RopeCvt<T>;
  pdl_launch_dependents();
  pdl_wait();
  const uint32_t half = a.head_vecs >> 1;
  const uint32_t row_stride = gridDim.x * blockDim.y;
  const uint32_t rows = (uint32_t)a.rows;
  struct Loaded { uint4 x, p, c, s; };
  for (uint32_t j = threadIdx.x; j < a.row_vecs; j += blockDim.x) {   // one trip unless a row has more than 256 vectors
    const uint32_t in_head = j % a.head_vecs;
    const uint32_t jp = in_head < half ? j + half : j - half;   // the partner half a head away
    auto table_index = [&](uint32_t row, uint32_t head_rows, uint32_t period_rows, int64_t period_vecs) -> int64_t {
      if (head_rows) return (int64_t)(row % head_rows) * a.head_vecs + in_head;          // [positions, head_dim]
      if (period_rows) return (int64_t)(row % period_rows) * a.row_vecs + j;             // repeats every whole number of rows
      const int64_t flat = (int64_t)row * a.row_vecs + j;
      return period_vecs == a.total_vecs ? flat : flat % period_vecs;
    };
    auto load = [&](uint32_t row) {
      const uint4* xr = a.x + (int64_t)row * a.x_pitch_vecs;
      Loaded l;
      l.x = __ldg(xr + j);
      l.p = __ldg(xr + jp);
      l.c = __ldg(a.c + table_index(row, a.c_head_rows, a.c_period_rows, a.c_period_vecs));
      l.s = __ldg(a.s + table_index(row, a.s_head_rows, a.s_period_rows, a.s_period_vecs));
      return l;
    };
    for (uint32_t row = blockIdx.x * blockDim.y + threadIdx.y; row < rows; row += 2 * row_stride) {
      const uint32_t row1 = row + row_stride;
      const bool two = row1 < rows;
      const Loaded l0 = load(row);
      Loaded l1 = l0;
      if (two) l1 = load(row1);
      a.y[(int64_t)row * a.row_vecs + j] = C::combine(l0.x, l0.p, l0.c, l0.s);
      if (two) a.y[(int64_t)row1 * a.row_vecs + j] = C::combine(l1.x, l1.p, l1.c, l1.s);
    }
  }
}

}  // namespace

Status rope(Device* dev, const RopeParams& p) {
  const bool ok_type = p.dtype == B200_FLOAT32 || p.dtype == B200_BFLOAT16 || p.dtype == B200_FLOAT16;
  if (!ok_type) return Status::Unsupported("rope: needs a 16- or 32-bit float type");
  const int n = p.dtype == B200_FLOAT32 ? 4 : 8;
  if (p.rows <= 0 || p.cols <= 0) return Status::OK();
  auto al = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  if (p.head_dim <= 0 || p.cols % p.head_dim != 0 || (p.head_dim / 2) % n != 0 || p.x_pitch % n != 0 || p.c_period % n != 0 ||
      p.s_period % n != 0 || p.c_period <= 0 || p.s_period <= 0 ||
      (p.c_per_head ? (p.c_period % p.head_dim != 0 || p.rows % (p.c_period / p.head_dim) != 0) : (p.rows * p.cols) % p.c_period != 0) ||
      (p.s_per_head ? (p.s_period % p.head_dim != 0 || p.rows % (p.s_period / p.head_dim) != 0) : (p.rows * p.cols) % p.s_period != 0) ||
      !al(p.x) || !al(p.c) || !al(p.s) || !al(p.y))
    return Status::Unsupported("rope: half a head must be a whole number of 16-byte vectors, and every operand 16-byte aligned");
  if (p.cols / n > 0x7fffffffLL || p.rows > 0x3fffffffLL) return Status::Unsupported("rope: more than 2^30 rows, or a row too long");
  B200_TRY(dev->MakeCurrent());
  RopeArgs a;
  a.x = reinterpret_cast<const uint4*>(p.x);
  a.c = reinterpret_cast<const uint4*>(p.c);
  a.s = reinterpret_cast<const uint4*>(p.s);
  a.y = reinterpret_cast<uint4*>(p.y);
  a.rows = p.rows;
  a.total_vecs = p.rows * p.cols / n;
  a.row_vecs = (uint32_t)(p.cols / n);
  a.head_vecs = (uint32_t)(p.head_dim / n);
  a.x_pitch_vecs = p.x_pitch / n;
  a.c_period_vecs = p.c_period / n;
  a.s_period_vecs = p.s_period / n;
  a.c_head_rows = p.c_per_head ? (uint32_t)(p.c_period / p.head_dim) : 0;
  a.s_head_rows = p.s_per_head ? (uint32_t)(p.s_period / p.head_dim) : 0;
  auto period_rows = [&](int64_t period_vecs) -> uint32_t {
    return (period_vecs % a.row_vecs == 0 && period_vecs / a.row_vecs <= 0x3fffffffLL) ? (uint32_t)(period_vecs / a.row_vecs) : 0;
  };
  a.c_period_rows = p.c_per_head ? 0 : period_rows(a.c_period_vecs);
  a.s_period_rows = p.s_per_head ? 0 : period_rows(a.s_period_vecs);
  // 256 threads: as many along the row as it has vectors (a power of two up to 256), the rest across rows
  unsigned tx = 1;
  while (tx < 256 && tx < a.row_vecs) tx *= 2;
  const dim3 block(tx, 256 / tx);
  int64_t blocks = (p.rows + 2 * block.y - 1) / (2 * block.y);   // two rows per thread and iteration
  const int64_t cap = (int64_t)dev->sm_count() * 16;
  if (blocks > cap) blocks = cap;
  // launched as a programmatic dependent: the launch itself runs under the previous kernel's tail
  cudaError_t e;
  if (p.dtype == B200_FLOAT32) e = launch_dependent_dims(rope_kernel<float>, dim3((unsigned)blocks), block, 0, dev->stream(), a);
  else if (p.dtype == B200_BFLOAT16) e = launch_dependent_dims(rope_kernel<__nv_bfloat16>, dim3((unsigned)blocks), block, 0, dev->stream(), a);
  else e = launch_dependent_dims(rope_kernel<__half>, dim3((unsigned)blocks), block, 0, dev->stream(), a);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return Status::Cuda(strfmt("rope: %s", cudaGetErrorString(e)));
  }
  return dev->CheckLaunch("rope");
}

}  // namespace k
}  // namespace b200
