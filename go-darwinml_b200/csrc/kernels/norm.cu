// LayerNorm and RMSNorm row kernels.
//
//   LayerNorm: two passes over the row held in registers: m = sum(x)/n; d = x - m; var = sum(d*d)/n (biased);
//              y = d * rsqrt(var + eps) [* gamma] [+ beta]
//              (the formula of the reference's FusedLayerNorm lowering, mpsgraph function.go:2430-2558, which spends
//              ~12 graph ops on it).  The one-pass forms (sum and sum of squares together, with or without a shift)
//              cancel when a row has an outlier or a mean far from its spread; with the row in registers the second
//              pass costs one more reduction round and no memory traffic.
//   RMSNorm:   y = x * rsqrt(sum(x*x)/n + eps) [* gamma]   (no reference counterpart)
//
// Statistics are accumulated in fp32 whatever the storage type; the result is
// rounded once.
//
// Design (HBM-bound; algorithmic bytes = 2 * rows * cols * sizeof(T), gamma and
// beta are read once per CTA):
//   * persistent grid: a multiple of the SM count of CTAs, each walking rows
//     with a grid stride, so there is no wave-quantisation tail at 16k rows;
//   * a row group of TPR threads (32..1024, chosen so that a thread owns at
//     most 32 elements) cooperates on a row; groups of one CTA synchronise with
//     their own named barrier, never with the whole CTA;
//   * the row is loaded once with 128-bit streaming loads, unpacked ONCE to
//     fp32 registers and reused by the mean / variance / output passes;
//   * gamma (unpacked) and beta (packed) are loaded to registers once per CTA,
//     outside the row loop: at 2 bytes per element the kernel is as close to
//     the instruction-issue limit as to the HBM limit, so every per-element
//     instruction counts;
//   * the next row's loads are issued before the current row is reduced;
//   * one reduction round per row for RMSNorm, two for LayerNorm (mean, then centred sum of squares); the per-warp
//     partials are double-buffered in shared memory so a round costs ONE named barrier, and the cross-warp step is
//     a few broadcast reads instead of a second shuffle tree.
#include "../kernels.h"
#include "pdl.cuh"
#include "rowwise.cuh"

namespace b200 {
namespace k {

namespace {

struct NArgs {
  const void* x;
  const void* gamma;
  const void* beta;
  void* y;
  int64_t rows, cols;
  float eps;
};

// Sums of NV values over the TPR threads of a row group; all of them get the results.  `slots` is this group's private
// area of 2 x NV x WPR floats, used alternately by successive calls (`phase`), which is what lets one barrier per call
// suffice: a warp can only reach the call after next, which reuses a buffer, once every warp has passed this call's
// barrier and therefore finished reading the call before.
template <int TPR, int NV>
__device__ __forceinline__ void group_sum_n(float (&v)[NV], float* slots, int bar, int& phase) {
#pragma unroll
  for (int i = 0; i < NV; ++i) v[i] = warp_reduce(v[i], SumOp());
  if constexpr (TPR > 32) {
    constexpr int WPR = TPR / 32;
    const int lane = threadIdx.x & 31, w = (threadIdx.x % TPR) >> 5;
    float* buf = slots + phase * (NV * WPR);
    phase ^= 1;
    if (lane == 0) {
#pragma unroll
      for (int i = 0; i < NV; ++i) buf[i * WPR + w] = v[i];
    }
    asm volatile("bar.sync %0, %1;" ::"r"(bar), "r"(TPR) : "memory");
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      float t = 0.f;
#pragma unroll
      for (int k = 0; k < WPR; ++k) t += buf[i * WPR + k];   // same address for every lane: broadcast reads
      v[i] = t;
    }
  }
}

// CTAs per SM the kernel is compiled for: short rows (few vectors per thread) need few registers, and more resident
// rows are what hides the memory latency when a row is only a kilobyte or two.
template <int ITERS, int TPR> struct NormOcc { static constexpr int kCtas = TPR > 256 ? 1 : (ITERS <= 2 ? 4 : (ITERS == 3 ? 3 : 2)); };

template <typename T, int ITERS, int TPR, bool RMS, bool HAS_G, bool HAS_B>
__global__ void __launch_bounds__(TPR > 256 ? TPR : 256, NormOcc<ITERS, TPR>::kCtas) norm_rows_kernel(const NArgs a) {
  constexpr int V = Cvt<T>::N;
  constexpr int BLOCK = TPR > 256 ? TPR : 256;
  constexpr int GROUPS = BLOCK / TPR;
  pdl_launch_dependents();   // the next kernel may be scheduled as SMs fall free; it waits for this one in its own pdl_wait
  pdl_wait();                // launched as a programmatic dependent: the kernel before this one has completed
  __shared__ float red[2 * 32];   // per group: 2 phases x warps per row
  const int group = threadIdx.x / TPR;
  const int t = threadIdx.x % TPR;
  float* slot = red + group * (2 * (TPR / 32));
  int phase = 0;
  const int bar = 1 + group;
  const float inv_n = 1.0f / (float)a.cols;

  // per-thread column offsets and validity are the same for every row
  bool valid[ITERS];
  int64_t c0[ITERS];
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    c0[it] = (int64_t)(it * TPR + t) * V;
    valid[it] = c0[it] < a.cols;
  }
  // LayerNorm with both gamma and beta keeps BOTH packed (16 bytes per vector) and unpacks them per row: with gamma
  // unpacked as well the kernel sat at its 128-register cap and spilled inside the row loop.
  constexpr bool PACKED_G = HAS_G && HAS_B && !RMS && sizeof(T) == 2;
  float g[PACKED_G ? 1 : ITERS][V];
  Raw16 gq[PACKED_G ? ITERS : 1];
  Raw16 bq[ITERS];  // beta stays packed (16 bytes per vector): unpacking it per row is cheaper than 32 more registers
  if constexpr (HAS_G) {
#pragma unroll
    for (int it = 0; it < ITERS; ++it)
      if (valid[it]) {
        if constexpr (PACKED_G) gq[it] = ld_cached16(reinterpret_cast<const T*>(a.gamma) + c0[it]);
        else Cvt<T>::unpack(ld_cached16(reinterpret_cast<const T*>(a.gamma) + c0[it]), g[it]);
      }
  }
  if constexpr (HAS_B && !RMS) {
#pragma unroll
    for (int it = 0; it < ITERS; ++it)
      if (valid[it]) bq[it] = ld_cached16(reinterpret_cast<const T*>(a.beta) + c0[it]);
  }

  const int64_t row_stride = (int64_t)gridDim.x * GROUPS;
  int64_t row = (int64_t)blockIdx.x * GROUPS + group;
  Raw16 raw[ITERS];
  if (row < a.rows) {
    const T* xr = reinterpret_cast<const T*>(a.x) + row * a.cols;
#pragma unroll
    for (int it = 0; it < ITERS; ++it)
      if (valid[it]) raw[it] = ld_stream16(xr + c0[it]);
  }
  for (; row < a.rows; row += row_stride) {
    float f[ITERS][V];
#pragma unroll
    for (int it = 0; it < ITERS; ++it)
      if (valid[it]) Cvt<T>::unpack(raw[it], f[it]);
    // prefetch the next row of this group while this one is reduced
    const int64_t next = row + row_stride;
    if (next < a.rows) {
      const T* xn = reinterpret_cast<const T*>(a.x) + next * a.cols;
#pragma unroll
      for (int it = 0; it < ITERS; ++it)
        if (valid[it]) raw[it] = ld_stream16(xn + c0[it]);
    }
    float rstd;
    float acc[1] = {0.f};
    if constexpr (!RMS) {
#pragma unroll
      for (int it = 0; it < ITERS; ++it)
        if (valid[it]) {
#pragma unroll
          for (int e = 0; e < V; ++e) acc[0] += f[it][e];
        }
      group_sum_n<TPR, 1>(acc, slot, bar, phase);
      const float mean = acc[0] * inv_n;
      acc[0] = 0.f;
#pragma unroll
      for (int it = 0; it < ITERS; ++it)
        if (valid[it]) {
#pragma unroll
          for (int e = 0; e < V; ++e) f[it][e] -= mean;   // the output pass multiplies the centred value
        }
    }
#pragma unroll
    for (int it = 0; it < ITERS; ++it)
      if (valid[it]) {
#pragma unroll
        for (int e = 0; e < V; ++e) acc[0] += f[it][e] * f[it][e];
      }
    group_sum_n<TPR, 1>(acc, slot, bar, phase);
    rstd = rsqrtf(acc[0] * inv_n + a.eps);
    T* yr = reinterpret_cast<T*>(a.y) + row * a.cols;
#pragma unroll
    for (int it = 0; it < ITERS; ++it)
      if (valid[it]) {
        // the empty asm makes the packed words opaque per row: otherwise the compiler hoists the (row-invariant)
        // unpacking out of the row loop and keeps the 32-bit copies in registers after all
        float b[V];
        if constexpr (HAS_B && !RMS) {
          asm volatile("" : "+r"(bq[it].w[0]), "+r"(bq[it].w[1]), "+r"(bq[it].w[2]), "+r"(bq[it].w[3]));
          Cvt<T>::unpack(bq[it], b);
        }
        float gu[V];
        if constexpr (PACKED_G) {
          asm volatile("" : "+r"(gq[it].w[0]), "+r"(gq[it].w[1]), "+r"(gq[it].w[2]), "+r"(gq[it].w[3]));
          Cvt<T>::unpack(gq[it], gu);
        }
#pragma unroll
        for (int e = 0; e < V; ++e) {
          float v = f[it][e] * rstd;
          if constexpr (PACKED_G) v *= gu[e];
          else if constexpr (HAS_G) v *= g[it][e];
          if constexpr (HAS_B && !RMS) v += b[e];
          f[it][e] = v;
        }
        Raw16 o;
        Cvt<T>::pack(f[it], o);
        st_stream16(yr + c0[it], o);
      }
  }
}

// Any cols / alignment: one CTA per row, three passes with scalar accesses.
template <typename T, bool RMS>
__global__ void __launch_bounds__(256) norm_generic_kernel(const NArgs a) {
  __shared__ float red[32];
  const int64_t row = blockIdx.x;
  const T* xr = reinterpret_cast<const T*>(a.x) + row * a.cols;
  T* yr = reinterpret_cast<T*>(a.y) + row * a.cols;
  const float inv_n = 1.0f / (float)a.cols;
  float mean = 0.f;
  if (!RMS) {
    float s = 0.f;
    for (int64_t j = threadIdx.x; j < a.cols; j += blockDim.x) s += Cvt<T>::load1(xr + j);
    mean = group_reduce<256>(s, SumOp(), 0.f, red) * inv_n;
  }
  float sq = 0.f;
  for (int64_t j = threadIdx.x; j < a.cols; j += blockDim.x) {
    const float d = Cvt<T>::load1(xr + j) - mean;
    sq += d * d;
  }
  sq = group_reduce<256>(sq, SumOp(), 0.f, red);
  const float rstd = rsqrtf(sq * inv_n + a.eps);
  for (int64_t j = threadIdx.x; j < a.cols; j += blockDim.x) {
    float v = (Cvt<T>::load1(xr + j) - mean) * rstd;
    if (a.gamma) v *= Cvt<T>::load1(reinterpret_cast<const T*>(a.gamma) + j);
    if (!RMS && a.beta) v += Cvt<T>::load1(reinterpret_cast<const T*>(a.beta) + j);
    Cvt<T>::store1(yr + j, v);
  }
}

template <typename T, int ITERS, int TPR, bool RMS>
void launch_params(const NArgs& a, unsigned grid, cudaStream_t s) {
  constexpr int BLOCK = TPR > 256 ? TPR : 256;
  const bool hg = a.gamma != nullptr, hb = a.beta != nullptr && !RMS;
  if (hg && hb) launch_dependent(norm_rows_kernel<T, ITERS, TPR, RMS, true, true>, grid, BLOCK, 0, s, a);
  else if (hg) launch_dependent(norm_rows_kernel<T, ITERS, TPR, RMS, true, false>, grid, BLOCK, 0, s, a);
  else if (hb) launch_dependent(norm_rows_kernel<T, ITERS, TPR, RMS, false, true>, grid, BLOCK, 0, s, a);
  else launch_dependent(norm_rows_kernel<T, ITERS, TPR, RMS, false, false>, grid, BLOCK, 0, s, a);
}

template <typename T, int TPR, bool RMS>
void launch_tpr(Device* dev, const NArgs& a, int iters, cudaStream_t s) {
  constexpr int BLOCK = TPR > 256 ? TPR : 256;
  constexpr int GROUPS = BLOCK / TPR;
  const int64_t ctas_needed = (a.rows + GROUPS - 1) / GROUPS;
  // persistent: a few CTAs per SM, never more than there are row slots
  auto grid_for = [&](int ctas_per_sm) {
    int64_t grid = (int64_t)dev->sm_count() * ctas_per_sm;
    return (unsigned)(grid > ctas_needed ? ctas_needed : grid);
  };
  switch (iters) {
    case 1: launch_params<T, 1, TPR, RMS>(a, grid_for(NormOcc<1, TPR>::kCtas), s); break;
    case 2: launch_params<T, 2, TPR, RMS>(a, grid_for(NormOcc<2, TPR>::kCtas), s); break;
    case 3: launch_params<T, 3, TPR, RMS>(a, grid_for(NormOcc<3, TPR>::kCtas), s); break;
    default: launch_params<T, 4, TPR, RMS>(a, grid_for(NormOcc<4, TPR>::kCtas), s); break;
  }
}

template <typename T, bool RMS>
void launch_typed(Device* dev, const NArgs& a, cudaStream_t s) {
  constexpr int V = Cvt<T>::N;
  constexpr int MAX_ITERS = 4;
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  const bool vec_ok = (a.cols % V == 0) && al16(a.x) && al16(a.y) && al16(a.gamma) && al16(a.beta) &&
                      a.cols <= (int64_t)1024 * V * MAX_ITERS;
  if (!vec_ok) {
    norm_generic_kernel<T, RMS><<<(unsigned)a.rows, 256, 0, s>>>(a);
    return;
  }
  const int64_t vecs = a.cols / V;
  int tpr = 32;
  while ((int64_t)tpr * MAX_ITERS < vecs) tpr *= 2;
  const int iters = (int)((vecs + tpr - 1) / tpr);   // 1 .. MAX_ITERS vectors per thread
  switch (tpr) {
    case 32: launch_tpr<T, 32, RMS>(dev, a, iters, s); break;
    case 64: launch_tpr<T, 64, RMS>(dev, a, iters, s); break;
    case 128: launch_tpr<T, 128, RMS>(dev, a, iters, s); break;
    case 256: launch_tpr<T, 256, RMS>(dev, a, iters, s); break;
    case 512: launch_tpr<T, 512, RMS>(dev, a, iters, s); break;
    default: launch_tpr<T, 1024, RMS>(dev, a, iters, s); break;
  }
}

}  // namespace

Status norm_rows(Device* dev, const NormParams& p) {
  if (p.rows == 0 || p.cols == 0) return Status::OK();
  if (p.rows > 0x7fffffffLL) return Status::Unsupported("norm: more than 2^31-1 rows");
  NArgs a{p.x, p.gamma, p.rms ? nullptr : p.beta, p.y, p.rows, p.cols, (float)p.epsilon};
  B200_TRY(dev->MakeCurrent());
  cudaStream_t s = dev->stream();
  switch (p.dtype) {
    case B200_FLOAT32: p.rms ? launch_typed<float, true>(dev, a, s) : launch_typed<float, false>(dev, a, s); break;
    case B200_BFLOAT16: p.rms ? launch_typed<__nv_bfloat16, true>(dev, a, s) : launch_typed<__nv_bfloat16, false>(dev, a, s); break;
    case B200_FLOAT16: p.rms ? launch_typed<__half, true>(dev, a, s) : launch_typed<__half, false>(dev, a, s); break;
    default: return Status::Unsupported(strfmt("norm: dtype %s", dtype_name(p.dtype)));
  }
  return dev->CheckLaunch(p.rms ? "rms_norm" : "layer_norm");
}

}  // namespace k
}  // namespace b200
