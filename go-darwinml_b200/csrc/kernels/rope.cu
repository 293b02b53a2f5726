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
};

struct RopeArgs {
  const uint4* x;
  const uint4* c;
  const uint4* s;
  uint4* y;
  int64_t total_vecs;     // rows * cols / N
  uint32_t row_vecs;      // cols / N
  uint32_t head_vecs;     // head_dim / N
  int64_t x_pitch_vecs;
  int64_t c_period_vecs, s_period_vecs;
};

template <typename T>
__global__ void __launch_bounds__(256) rope_kernel(const RopeArgs a) {
  using C = RopeCvt<T>;
  constexpr int N = C::N;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const uint32_t half = a.head_vecs >> 1;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < a.total_vecs; i += stride) {
    const int64_t row = i / a.row_vecs;
    const uint32_t j = (uint32_t)(i - row * a.row_vecs);
    const uint32_t in_head = j % a.head_vecs;
    const uint32_t jp = in_head < half ? j + half : j - half;   // the partner half a head away
    const uint4* xr = a.x + row * a.x_pitch_vecs;
    const uint4 qx = __ldg(xr + j), qp = __ldg(xr + jp);
    const uint4 qc = __ldg(a.c + (a.c_period_vecs == a.total_vecs ? i : i % a.c_period_vecs));
    const uint4 qs = __ldg(a.s + (a.s_period_vecs == a.total_vecs ? i : i % a.s_period_vecs));
    float x[N], p[N], c[N], s[N], r[N];
    C::unpack(qx, x); C::unpack(qp, p); C::unpack(qc, c); C::unpack(qs, s);
#pragma unroll
    for (int e = 0; e < N; ++e)   // intrinsics: the compiler must not contract the products into an FMA (fp32 would round once)
      r[e] = C::round(__fadd_rn(C::round(__fmul_rn(x[e], c[e])), C::round(__fmul_rn(p[e], s[e]))));
    a.y[i] = C::pack(r);
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
      p.s_period % n != 0 || p.c_period <= 0 || p.s_period <= 0 || (p.rows * p.cols) % p.c_period != 0 || (p.rows * p.cols) % p.s_period != 0 ||
      !al(p.x) || !al(p.c) || !al(p.s) || !al(p.y))
    return Status::Unsupported("rope: half a head must be a whole number of 16-byte vectors, and every operand 16-byte aligned");
  if (p.cols / n > 0x7fffffffLL) return Status::Unsupported("rope: row too long");
  B200_TRY(dev->MakeCurrent());
  RopeArgs a;
  a.x = reinterpret_cast<const uint4*>(p.x);
  a.c = reinterpret_cast<const uint4*>(p.c);
  a.s = reinterpret_cast<const uint4*>(p.s);
  a.y = reinterpret_cast<uint4*>(p.y);
  a.total_vecs = p.rows * p.cols / n;
  a.row_vecs = (uint32_t)(p.cols / n);
  a.head_vecs = (uint32_t)(p.head_dim / n);
  a.x_pitch_vecs = p.x_pitch / n;
  a.c_period_vecs = p.c_period / n;
  a.s_period_vecs = p.s_period / n;
  int64_t blocks = (a.total_vecs + 255) / 256;
  const int64_t cap = (int64_t)dev->sm_count() * 16;
  if (blocks > cap) blocks = cap;
  if (p.dtype == B200_FLOAT32) rope_kernel<float><<<(unsigned)blocks, 256, 0, dev->stream()>>>(a);
  else if (p.dtype == B200_BFLOAT16) rope_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, dev->stream()>>>(a);
  else rope_kernel<__half><<<(unsigned)blocks, 256, 0, dev->stream()>>>(a);
  return dev->CheckLaunch("rope");
}

}  // namespace k
}  // namespace b200
