// Fused masked softmax.
//
//   y[r, j] = exp(s[r, j] - max_j s[r, j]) / sum_j exp(s[r, j] - max_j s[r, j]),
//   s[r, j] = scale * x[r, j] (+ float mask) , or -inf where a bool mask is
//   false or (causal) j > q(r), with q(r) = r mod seq_q.
//
// This replaces the reference's softMaxWithTensor call (mpsgraph bridge.m:1448-1461)
// together with the scale / Where(-inf) / Add(mask) ops that its SDPA lowering
// emits in front of it (function.go:2768-2894): no mask tensor is ever built.
//
// Fast path ("rows in registers"): one row group (32..1024 threads) per row,
// the whole row is read ONCE with 128-bit streaming loads, kept in registers,
// reduced with warp shuffles, and written once.  Under a causal mask the
// 16-byte vectors that lie entirely right of the diagonal are never loaded
// (their output is 0), so a causal launch reads about half of x.
// HBM-bound: algorithmic bytes = 2 * rows * cols * sizeof(T).
#include "../kernels.h"
#include "rowwise.cuh"

namespace b200 {
namespace k {

namespace {

struct SmArgs {
  const void* x;
  void* y;
  int64_t rows, cols;
  float scale;
  int causal;
  int64_t seq_q;
  const void* mask;
  int mask_kind;  // 0 none, 1 bool (uint8), 2 float of x's dtype
  int64_t heads;  // rows = batch * heads * seq_q (mask addressing only)
  int64_t m_b, m_h, m_q, m_k;  // mask strides in elements (0 = broadcast)
};

// exp(x) as one multiply and one MUFU op.  The flush-to-zero form: without it the compiler wraps the instruction in a
// range test and two rescaling multiplies for results below 2^-126, which no tolerance of a softmax can see.
__device__ __forceinline__ float exp_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x * 1.4426950408889634f));
  return y;
}

// Offset of a row's first mask element (the row's batch, head and query position taken apart ONCE per row: three 64-bit
// divisions that, left inside the per-element code, made a 192 x 1024 masked softmax take 49 us).
__device__ __forceinline__ int64_t mask_row_offset(const SmArgs& a, int64_t row) {
  if (a.mask_kind == 0) return 0;
  const int64_t q = row % a.seq_q;
  const int64_t h = (row / a.seq_q) % a.heads;
  const int64_t b = row / (a.seq_q * a.heads);
  return b * a.m_b + h * a.m_h + q * a.m_q;
}

// scale and the explicit mask, without the causal limit; mrow = mask_row_offset of the row
template <typename T>
__device__ __forceinline__ float scaled_score(const SmArgs& a, float xv, int64_t mrow, int64_t j) {
  float s = xv * a.scale;
  if (a.mask_kind != 0) {
    const int64_t off = mrow + j * a.m_k;
    if (a.mask_kind == 1) {
      if (!reinterpret_cast<const uint8_t*>(a.mask)[off]) s = -INFINITY;
    } else {
      s += Cvt<T>::load1(reinterpret_cast<const T*>(a.mask) + off);
    }
  }
  return s;
}
template <typename T>
__device__ __forceinline__ float masked_score(const SmArgs& a, float xv, int64_t mrow, int64_t j, int64_t limit) {
  return j >= limit ? -INFINITY : scaled_score<T>(a, xv, mrow, j);
}

template <typename T, int ITERS, int TPR>
__global__ void __launch_bounds__(TPR > 256 ? TPR : 256, TPR > 256 ? 1 : ((sizeof(T) == 4 || ITERS <= 4) ? 4 : 2)) softmax_rows_kernel(const SmArgs a) {
  constexpr int V = Cvt<T>::N;
  __shared__ float red[32];
  const int rows_per_cta = blockDim.x / TPR;
  int64_t row = (int64_t)blockIdx.x * rows_per_cta + threadIdx.x / TPR;
  const int t = threadIdx.x % TPR;
  const bool active = row < a.rows;
  if (!active) row = a.rows - 1;  // keep every thread in the barriers of group_reduce
  int64_t limit = a.cols;
  if (a.causal) {
    const int64_t q = row % a.seq_q;
    limit = (q + 1 < a.cols) ? q + 1 : a.cols;
  }
  const T* xr = reinterpret_cast<const T*>(a.x) + row * a.cols;
  T* yr = reinterpret_cast<T*>(a.y) + row * a.cols;
  const int64_t mrow = mask_row_offset(a, row);

  // 16-bit rows: vectors wholly right of the causal limit take no arithmetic (their exponentials are exactly 0), measured
  // 6 % faster; on fp32 rows the same branches cost registers (spills at the 64-register cap) and measured 2 % slower, so
  // there every vector runs the straight-line code on -inf.
  constexpr bool SKIP = sizeof(T) == 2;
  float v[ITERS][V];
  Raw16 raw[ITERS];
  // Issue every load of the row before touching any of them.
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const int64_t c0 = (int64_t)(it * TPR + t) * V;
    if (c0 < limit) raw[it] = ld_stream16(xr + c0);
  }
  float mx = -INFINITY;
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const int64_t c0 = (int64_t)(it * TPR + t) * V;
    if (c0 < limit) {
      Cvt<T>::unpack(raw[it], v[it]);
      const int keep = (limit - c0) < V ? (int)(limit - c0) : V;   // elements of this vector left of the limit (32-bit compares below)
      if (a.mask_kind == 0) {
#pragma unroll
        for (int e = 0; e < V; ++e) {
          v[it][e] = e < keep ? v[it][e] * a.scale : -INFINITY;
          mx = fmaxf(mx, v[it][e]);
        }
      } else {
#pragma unroll
        for (int e = 0; e < V; ++e) {
          v[it][e] = e < keep ? scaled_score<T>(a, v[it][e], mrow, c0 + e) : -INFINITY;
          mx = fmaxf(mx, v[it][e]);
        }
      }
    } else if constexpr (!SKIP) {
#pragma unroll
      for (int e = 0; e < V; ++e) v[it][e] = -INFINITY;
    }
  }
  mx = group_reduce<TPR>(mx, MaxOp(), -INFINITY, red);
  float sum = 0.f;
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const int64_t c0 = (int64_t)(it * TPR + t) * V;
    if (!SKIP || c0 < limit) {
#pragma unroll
      for (int e = 0; e < V; ++e) {
        // A fully masked row has mx = -inf: (-inf) - (-inf) = NaN, as IEEE gives.
        v[it][e] = exp_fast(v[it][e] - mx);
        sum += v[it][e];
      }
    }
  }
  sum = group_reduce<TPR>(sum, SumOp(), 0.f, red);
  const float inv = 1.0f / sum;
  if (!active) return;
  const float zero = 0.f * inv;   // 0, or NaN in a fully masked row (what exp(-inf - mx) * inv gives there)
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const int64_t c0 = (int64_t)(it * TPR + t) * V;
    if (c0 < a.cols) {
      if (!SKIP || c0 < limit) {
#pragma unroll
        for (int e = 0; e < V; ++e) v[it][e] *= inv;
      } else {
#pragma unroll
        for (int e = 0; e < V; ++e) v[it][e] = zero;
      }
      Raw16 o;
      Cvt<T>::pack(v[it], o);
      st_stream16(yr + c0, o);
    }
  }
}

// Any cols, any alignment: one CTA per row, three streaming passes.
template <typename T>
__global__ void __launch_bounds__(256) softmax_generic_row_kernel(const SmArgs a) {
  __shared__ float red[32];
  const int64_t row = blockIdx.x;
  int64_t limit = a.cols;
  if (a.causal) {
    const int64_t q = row % a.seq_q;
    limit = (q + 1 < a.cols) ? q + 1 : a.cols;
  }
  const T* xr = reinterpret_cast<const T*>(a.x) + row * a.cols;
  T* yr = reinterpret_cast<T*>(a.y) + row * a.cols;
  const int64_t mrow = mask_row_offset(a, row);
  float mx = -INFINITY;
  for (int64_t j = threadIdx.x; j < limit; j += blockDim.x)
    mx = fmaxf(mx, masked_score<T>(a, Cvt<T>::load1(xr + j), mrow, j, limit));
  mx = group_reduce<256>(mx, MaxOp(), -INFINITY, red);
  float sum = 0.f;
  for (int64_t j = threadIdx.x; j < limit; j += blockDim.x)
    sum += expf(masked_score<T>(a, Cvt<T>::load1(xr + j), mrow, j, limit) - mx);
  sum = group_reduce<256>(sum, SumOp(), 0.f, red);
  const float inv = 1.0f / sum;
  for (int64_t j = threadIdx.x; j < a.cols; j += blockDim.x) {
    float s = (j < limit) ? masked_score<T>(a, Cvt<T>::load1(xr + j), mrow, j, limit) : -INFINITY;
    Cvt<T>::store1(yr + j, expf(s - mx) * inv);
  }
}

// Softmax over a middle axis: x viewed as [outer, n, inner], inner > 1.  One
// thread per (outer, inner) pair; neighbouring threads touch neighbouring
// addresses, so every pass is coalesced.
template <typename T>
__global__ void __launch_bounds__(256) softmax_strided_kernel(const T* x, T* y, int64_t outer, int64_t n, int64_t inner) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= outer * inner) return;
  const int64_t o = idx / inner, i = idx % inner;
  const T* xp = x + o * n * inner + i;
  T* yp = y + o * n * inner + i;
  float mx = -INFINITY;
  for (int64_t j = 0; j < n; ++j) mx = fmaxf(mx, Cvt<T>::load1(xp + j * inner));
  float sum = 0.f;
  for (int64_t j = 0; j < n; ++j) sum += expf(Cvt<T>::load1(xp + j * inner) - mx);
  const float inv = 1.0f / sum;
  for (int64_t j = 0; j < n; ++j) Cvt<T>::store1(yp + j * inner, expf(Cvt<T>::load1(xp + j * inner) - mx) * inv);
}

template <typename T, int TPR>
void launch_rows_tpr(const SmArgs& a, int iters, cudaStream_t s) {
  const int block = TPR > 256 ? TPR : 256;
  const int rows_per_cta = block / TPR;
  const unsigned grid = (unsigned)((a.rows + rows_per_cta - 1) / rows_per_cta);
  switch (iters) {
    case 1: softmax_rows_kernel<T, 1, TPR><<<grid, block, 0, s>>>(a); break;
    case 2: softmax_rows_kernel<T, 2, TPR><<<grid, block, 0, s>>>(a); break;
    case 4: softmax_rows_kernel<T, 4, TPR><<<grid, block, 0, s>>>(a); break;
    default: softmax_rows_kernel<T, 8, TPR><<<grid, block, 0, s>>>(a); break;
  }
}

template <typename T>
void launch_typed(const SmArgs& a, cudaStream_t s) {
  constexpr int V = Cvt<T>::N;
  const bool vec_ok = (a.cols % V == 0) && ((reinterpret_cast<uintptr_t>(a.x) & 15) == 0) &&
                      ((reinterpret_cast<uintptr_t>(a.y) & 15) == 0) && a.cols <= (int64_t)1024 * V * 8;
  if (!vec_ok) {
    softmax_generic_row_kernel<T><<<(unsigned)a.rows, 256, 0, s>>>(a);
    return;
  }
  const int64_t vecs = a.cols / V;
  int tpr = 32;
  if (vecs > 32 * 8) tpr = 256;
  if (vecs > 256 * 8) tpr = 1024;
  int iters = 1;
  while ((int64_t)iters * tpr < vecs) iters *= 2;
  if (tpr == 32) launch_rows_tpr<T, 32>(a, iters, s);
  else if (tpr == 256) launch_rows_tpr<T, 256>(a, iters, s);
  else launch_rows_tpr<T, 1024>(a, iters, s);
}

}  // namespace

Status softmax_rows(Device* dev, const SoftmaxParams& p) {
  if (p.rows == 0 || p.cols == 0) return Status::OK();
  if (p.rows > 0x7fffffffLL) return Status::Unsupported("softmax: more than 2^31-1 rows");
  SmArgs a;
  a.x = p.x; a.y = p.y; a.rows = p.rows; a.cols = p.cols;
  a.scale = (float)p.scale; a.causal = p.causal ? 1 : 0;
  a.seq_q = p.seq_q > 0 ? p.seq_q : p.rows;
  a.mask = p.mask; a.mask_kind = p.mask ? p.mask_kind : 0;
  a.heads = p.heads > 0 ? p.heads : 1;
  a.m_b = p.mask_strides[0]; a.m_h = p.mask_strides[1]; a.m_q = p.mask_strides[2]; a.m_k = p.mask_strides[3];
  B200_TRY(dev->MakeCurrent());
  switch (p.dtype) {
    case B200_FLOAT32: launch_typed<float>(a, dev->stream()); break;
    case B200_BFLOAT16: launch_typed<__nv_bfloat16>(a, dev->stream()); break;
    case B200_FLOAT16: launch_typed<__half>(a, dev->stream()); break;
    default: return Status::Unsupported(strfmt("softmax: dtype %s", dtype_name(p.dtype)));
  }
  return dev->CheckLaunch("softmax_rows");
}

Status softmax_strided(Device* dev, const void* x, void* y, int64_t outer, int64_t n, int64_t inner, int dtype) {
  if (outer * n * inner == 0) return Status::OK();
  B200_TRY(dev->MakeCurrent());
  const int64_t threads = outer * inner;
  const unsigned grid = (unsigned)((threads + 255) / 256);
  switch (dtype) {
    case B200_FLOAT32: softmax_strided_kernel<float><<<grid, 256, 0, dev->stream()>>>((const float*)x, (float*)y, outer, n, inner); break;
    case B200_BFLOAT16: softmax_strided_kernel<__nv_bfloat16><<<grid, 256, 0, dev->stream()>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, outer, n, inner); break;
    case B200_FLOAT16: softmax_strided_kernel<__half><<<grid, 256, 0, dev->stream()>>>((const __half*)x, (__half*)y, outer, n, inner); break;
    default: return Status::Unsupported(strfmt("softmax: dtype %s", dtype_name(dtype)));
  }
  return dev->CheckLaunch("softmax_strided");
}

}  // namespace k
}  // namespace b200
