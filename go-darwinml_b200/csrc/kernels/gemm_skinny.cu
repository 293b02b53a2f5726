// C[M, N] = act(X[M, K] W[K, N] + bias) (+ / * residual) for a handful of rows (M <= 64): a decoding step's projections.
//
// Such a product is bound by reading W once (2 K N bytes); the 128 x 256 tensor-core tile gives it N / 256 CTAs, each
// streaming its whole K through one SM's load path (28 us for K = 3072, N = 768).  Here many CTAs share W: a CTA owns
// 64 columns and one slice of K and streams the slice through a four-stage ring of 64-row chunks in shared memory
// (128-row chunks when the CTAs are few; 16-byte asynchronous copies, always three chunks ahead of the arithmetic; a
// slice that fits the ring is simply in flight at once), multiplies with mma.sync m16n8k16 (X as one, two or four 16-row operands, rows past M zero), and
// holds an M x 64 fp32 partial.  A slab's (at most 8) slices are the CTAs of one cluster: the partials meet through
// distributed shared memory, added in slice order (the same sum on every run), each CTA finishing a share of the
// outputs (bias, activation, residual).  The other reduction (B200MLX_GEMM_SKINNY_CLUSTER=0: up to 16 slices, no
// cluster) goes through global memory: the CTA that arrives last on its slab's counter adds the partials, again in
// slice order, and writes C; it leaves the counter at zero for the next launch.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <map>
#include <mutex>

#include "../kernels.h"
#include "gemm_common.cuh"
#include "pdl.cuh"
#include "sm100_ptx.cuh"

namespace b200 {
namespace k {

namespace {

constexpr int SK_THREADS = 128;
constexpr int SK_BN = 64;
constexpr int SK_MAX_ROWS = 64;
constexpr int SK_MAX_SPLITS = 16;   // reduction through global memory: the last CTA adds the slices' partial sums in two rounds of eight loads at most
constexpr int SK_STAGES = 4;   // at most; three when that lets the whole grid be resident at once
constexpr int SK_X_PAD = 8;   // elements: the X rows' pitch is an odd number of 16-byte units, conflict-free for ldmatrix

struct SkArgs {
  const void* x;
  const void* w;
  const void* w2;   // DUAL: the second weight
  const void* gamma;   // RMS: the norm's gain [K]
  float rms_eps;
  void* c;
  const void* bias;
  const void* residual;
  float* partial;       // [splits, 16 / 32 / 64 rows, N] (reduction through global memory only)
  unsigned* counters;   // [N / 64], zero between launches
  int M, N, K, kc, kch, stages, splits, act, residual_mul;   // kc: K per slice; kch: rows of K per ring stage; stages: 3 or 4 (the kernel's S)
  int w_static;   // W may be fetched before the previous kernel on the stream has finished
};

__device__ __forceinline__ void sk_cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void sk_cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
__device__ __forceinline__ void sk_cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void sk_cp_async_wait_group() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void sk_ldmatrix_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void sk_ldmatrix_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
template <typename T> __device__ __forceinline__ void sk_mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <> __device__ __forceinline__ void sk_mma<__nv_bfloat16>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <> __device__ __forceinline__ void sk_mma<__half>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <typename T> __device__ __forceinline__ float2 sk_unpack2(uint32_t w);
template <> __device__ __forceinline__ float2 sk_unpack2<__nv_bfloat16>(uint32_t w) { return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u)); }
template <> __device__ __forceinline__ float2 sk_unpack2<__half>(uint32_t w) { return __half22float2(*reinterpret_cast<const __half2*>(&w)); }
template <typename T> __device__ __forceinline__ uint32_t sk_mul2(uint32_t a, uint32_t b);   // two 16-bit products, each rounded
template <> __device__ __forceinline__ uint32_t sk_mul2<__nv_bfloat16>(uint32_t a, uint32_t b) {
  const __nv_bfloat162 r = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&a), *reinterpret_cast<const __nv_bfloat162*>(&b));
  return *reinterpret_cast<const uint32_t*>(&r);
}
template <> __device__ __forceinline__ uint32_t sk_mul2<__half>(uint32_t a, uint32_t b) {
  const __half2 r = __hmul2(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&b));
  return *reinterpret_cast<const uint32_t*>(&r);
}
template <typename T> __device__ __forceinline__ float sk_to_f(T v);
template <> __device__ __forceinline__ float sk_to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float sk_to_f(__half v) { return __half2float(v); }
template <typename T> __device__ __forceinline__ T sk_from_f(float v);
template <> __device__ __forceinline__ __nv_bfloat16 sk_from_f(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half sk_from_f(float v) { return __float2half_rn(v); }

// CLUSTER: the slab's K slices are the CTAs of one cluster (at most 8); their partial sums stay in shared memory and
// meet through distributed shared memory, each CTA finishing an equal share of the slab's outputs.  Otherwise (K too
// long for 8 slices) the partial sums go through global memory and the slab's last CTA finishes them.
// MT: 16-row tiles of X (1, 2 or 4: up to 16, 32 or 64 rows); W's fragments are loaded once per k-step for all of them.
// NK: W is stored [N, K] (an LM head tied to the embedding table): a stage holds [64 columns][kch] instead of [kch][64], its
// fragments come from ldmatrix without .trans, and N need not be a multiple of 64 (columns past N are zero in shared
// memory and never stored).
// DUAL (cluster reduction, W as [K, N] only): a second weight W2 of the same shape streams beside W and the result is
// round(act(X W + bias)) * round(X W2), rounded again -- a gated MLP's act(x W1) * (x W2) in one launch, bit for bit what
// the two launches (X W2 first, then act(X W) with a multiplying residual) produce.
// RMS (cluster reduction, W as [K, N] only): X is the INPUT of an RMSNorm with gain gamma whose output the product takes:
// rms_norm(x)[m, :] W = rstd[m] * ((x[m, :] * gamma) W), so the gain is applied to X's fragments on their way into the MMAs,
// the rows' sums of squares are collected from the same fragments (each K slice its share; the slices' shares meet
// through distributed shared memory with the partial sums), and rstd scales the finished sums.  One launch and one pass
// over X fewer than norm + product; the product of x and gamma is rounded to the 16-bit type, the scaling by rstd is not
// (the two-launch form rounds x * rstd * gamma once).
template <typename T, bool CLUSTER, int MT, bool NK, int S, bool DUAL, bool RMS>
__global__ void __launch_bounds__(SK_THREADS) gemm_skinny_kernel(const SkArgs g) {
  constexpr int ROWS = 16 * MT;
  extern __shared__ __align__(128) unsigned char sk_smem[];
  __shared__ int s_last;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int slab = blockIdx.x, split = blockIdx.y;
  const int n0 = slab * SK_BN;
  const int k0 = split * g.kc;
  const int kc = g.K - k0 < g.kc ? g.K - k0 : g.kc;   // this slice's length, a multiple of 16
  // The slice streams through a ring of SK_STAGES stages of g.kch rows of K: W rows [kch][64] with 16-byte units
  // XOR-swizzled by (row & 7), then X [ROWS][kch + 8].  Chunk c + SK_STAGES is requested as soon as chunk c has been
  // multiplied, so loads stay SK_STAGES - 1 chunks ahead of the arithmetic; a slice that fits the ring is in flight at once.
  const int kch = g.kch;
  const int x_pitch = (kch + SK_X_PAD) * 2;           // bytes
  const int w_bytes = (NK ? (kch + 63) / 64 * 64 : kch) * SK_BN * 2;   // a stage's W part (NK: whole 128-byte groups per column, it swizzles within them)
  const int x_off = (DUAL ? 2 : 1) * w_bytes;   // DUAL: W2's part follows W's
  const int g_off = x_off + ROWS * x_pitch;           // RMS: the chunk of gamma follows X
  const int stage_bytes = g_off + (RMS ? kch * 2 : 0);
  const uint32_t ring_u = sm100::smem_u32(sk_smem);
  const int nch = (kc + kch - 1) / kch;
  const T* Wg = NK ? reinterpret_cast<const T*>(g.w) + (int64_t)n0 * g.K + k0 : reinterpret_cast<const T*>(g.w) + (int64_t)k0 * g.N + n0;
  const T* Xg = reinterpret_cast<const T*>(g.x) + k0;
  const int w_pitch = (kch + 63) / 64 * 128;   // NK: bytes per column's row of a stage, whole 128-byte groups
  // W as [K, N]: this thread's unit of the chunk's first 16 rows, in memory and (swizzled) in a stage; 16 rows further: w_step
  const T* w_thread = Wg + (int64_t)(tid >> 3) * g.N + (tid & 7) * 8;
  const T* w2_thread = DUAL ? reinterpret_cast<const T*>(g.w2) + (int64_t)k0 * g.N + n0 + (int64_t)(tid >> 3) * g.N + (tid & 7) * 8 : nullptr;
  const int64_t w_step = 16 * (int64_t)g.N;
  const uint32_t w_dst0 = (tid >> 3) * 128 + (((tid & 7) ^ ((tid >> 3) & 7)) << 4);
  // X: with 64 or 128 rows of K per stage a row of the chunk is 8 or 16 units, so (row, unit) of a thread are shifts
  const bool x_fast = kch == 64 || kch == 128;
  const int x_shift = kch == 64 ? 3 : 4;
  auto issue_w = [&](int c) {
    if (c >= nch) return;
    const int rows = kc - c * kch < kch ? kc - c * kch : kch;
    const uint32_t wst = ring_u + (c % S) * stage_bytes;
    if constexpr (NK) {
      // 64 columns x (rows / 8) units of 16 bytes; the unit's low 3 bits XOR (column & 7)
      const int upr = rows >> 3;
      const T* W = Wg + c * kch;
      for (int idx = tid; idx < SK_BN * upr; idx += SK_THREADS) {
        const int n = idx / upr, u = idx - n * upr;
        const uint32_t dst = wst + n * w_pitch + (((u & ~7) | ((u ^ n) & 7)) << 4);
        if (n0 + n < g.N) sk_cp_async16(dst, W + (int64_t)n * g.K + u * 8);
        else asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(dst), "r"(0u) : "memory");
      }
    } else {
      // thread (wr, wc) copies unit wc of rows wr, wr + 16, ...: its source and destination advance by constants
      const int64_t chunk_off = (int64_t)c * kch * g.N;
      const T* src = w_thread + chunk_off;
      uint32_t dst = wst + w_dst0;
      for (int row = tid >> 3; row < rows; row += 16, src += w_step, dst += 16 * 128) sk_cp_async16(dst, src);
      if constexpr (DUAL) {
        const T* src2 = w2_thread + chunk_off;
        dst = wst + w_bytes + w_dst0;
        for (int row = tid >> 3; row < rows; row += 16, src2 += w_step, dst += 16 * 128) sk_cp_async16(dst, src2);
      }
    }
  };
  auto issue_x = [&](int c) {
    if (c >= nch) return;
    const int rows = kc - c * kch < kch ? kc - c * kch : kch;
    unsigned char* xst = sk_smem + (c % S) * stage_bytes + x_off;
    const uint32_t xst_u = sm100::smem_u32(xst);
    const T* X = Xg + c * kch;
    const int xch = rows >> 3;
    if constexpr (RMS) {
      if (tid < xch) sk_cp_async16(ring_u + (c % S) * stage_bytes + g_off + tid * 16, reinterpret_cast<const T*>(g.gamma) + k0 + c * kch + tid * 8);
    }
    if (x_fast) {
      const int ch = tid & ((1 << x_shift) - 1), rstep = SK_THREADS >> x_shift;
      if (ch < xch) {
        for (int row = tid >> x_shift; row < ROWS; row += rstep) {
          if (row < g.M) sk_cp_async16(xst_u + row * x_pitch + ch * 16, X + (int64_t)row * g.K + ch * 8);
          else *reinterpret_cast<uint4*>(xst + row * x_pitch + ch * 16) = make_uint4(0, 0, 0, 0);
        }
      }
    } else {
      for (int idx = tid; idx < ROWS * xch; idx += SK_THREADS) {
        const int row = idx / xch, ch = idx - row * xch;
        if (row < g.M) sk_cp_async16(xst_u + row * x_pitch + ch * 16, X + (int64_t)row * g.K + ch * 8);
        else *reinterpret_cast<uint4*>(xst + row * x_pitch + ch * 16) = make_uint4(0, 0, 0, 0);
      }
    }
  };
  pdl_launch_dependents();
  // Weights that nothing in flight can be writing are requested before the previous kernel's results are waited for.
  if (g.w_static) {
#pragma unroll 1
    for (int c = 0; c < S; ++c) issue_w(c);
    pdl_wait();
#pragma unroll 1
    for (int c = 0; c < S; ++c) { issue_x(c); sk_cp_async_commit(); }   // (group 0 also holds every W chunk of the prologue)
  } else {
    pdl_wait();
#pragma unroll 1
    for (int c = 0; c < S; ++c) { issue_w(c); issue_x(c); sk_cp_async_commit(); }
  }
  // warp w: columns [16 w, 16 w + 16) of the slab, all rows, all of the slice's k
  float acc[MT][2][4];
  float acc2[DUAL ? MT : 1][2][4];   // DUAL: X W2
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int t = 0; t < 2; ++t)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        acc[mt][t][i] = 0.f;
        if (DUAL) acc2[DUAL ? mt : 0][t][i] = 0.f;
      }
  float ss[RMS ? MT : 1][2];   // RMS: this slice's sums of squares of rows 16 mt + lane / 4 (+ 8), this thread's columns only
#pragma unroll
  for (int mt = 0; mt < (RMS ? MT : 1); ++mt) ss[mt][0] = ss[mt][1] = 0.f;
  {
    const int mi = lane >> 3, r = lane & 7;
    const uint32_t a_off = x_off + (lane & 15) * x_pitch + (lane >> 4) * 16;
    const int b_k = (mi & 1) * 8 + r;          // k within the 16-step; (k & 7) == r
    const int b_ch = warp * 2 + (mi >> 1);     // 16-byte unit within the 128-byte row
    const uint32_t b_off = b_k * 128 + ((b_ch ^ r) << 4);
    // NK: matrix mi covers column tile mi / 2 and k half mi % 2; lane r of it reads column 16 w + 8 (mi / 2) + r
    const uint32_t nk_row = (warp * 16 + (mi >> 1) * 8 + r) * w_pitch;
#pragma unroll 1
    for (int c = 0; c < nch; ++c) {
      sk_cp_async_wait_group<S - 1>();   // chunk c has landed (one group per chunk, complete in order)
      __syncthreads();
      const uint32_t st = ring_u + (c % S) * stage_bytes;
      const int rows = kc - c * kch < kch ? kc - c * kch : kch;
#pragma unroll 2
      for (int kk = 0; kk < rows; kk += 16) {
        uint32_t bq[4], bq2[4];
        if constexpr (DUAL) sk_ldmatrix_x4_trans(st + w_bytes + b_off + kk * 128, bq2);
        if constexpr (NK) {
          const int u = (kk >> 3) + (mi & 1);   // the 16-byte unit of this k half within the column's row
          sk_ldmatrix_x4(st + nk_row + (((u & ~7) | ((u ^ r) & 7)) << 4), bq);
        } else {
          sk_ldmatrix_x4_trans(st + b_off + kk * 128, bq);
        }
        uint32_t gk0 = 0, gk1 = 0;   // RMS: gamma at this thread's fragment columns kk + 2 (lane % 4) + {0, 1} and + 8
        if constexpr (RMS) {
          asm volatile("ld.shared.u32 %0, [%1];" : "=r"(gk0) : "r"(st + g_off + (kk + 2 * (lane & 3)) * 2));
          asm volatile("ld.shared.u32 %0, [%1];" : "=r"(gk1) : "r"(st + g_off + (kk + 8 + 2 * (lane & 3)) * 2));
        }
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          uint32_t a[4];
          sk_ldmatrix_x4(st + a_off + mt * 16 * x_pitch + kk * 2, a);
          if constexpr (RMS) {
            if (((kk >> 4) & 3) == warp) {   // every warp holds the same X fragments: they take turns counting
              const float2 x0 = sk_unpack2<T>(a[0]), x1 = sk_unpack2<T>(a[1]), x2 = sk_unpack2<T>(a[2]), x3 = sk_unpack2<T>(a[3]);
              ss[mt][0] += x0.x * x0.x + x0.y * x0.y + x2.x * x2.x + x2.y * x2.y;
              ss[mt][1] += x1.x * x1.x + x1.y * x1.y + x3.x * x3.x + x3.y * x3.y;
            }
            a[0] = sk_mul2<T>(a[0], gk0);
            a[1] = sk_mul2<T>(a[1], gk0);
            a[2] = sk_mul2<T>(a[2], gk1);
            a[3] = sk_mul2<T>(a[3], gk1);
          }
          sk_mma<T>(acc[mt][0], a, bq[0], bq[1]);
          sk_mma<T>(acc[mt][1], a, bq[2], bq[3]);
          if constexpr (DUAL) {
            sk_mma<T>(acc2[DUAL ? mt : 0][0], a, bq2[0], bq2[1]);
            sk_mma<T>(acc2[DUAL ? mt : 0][1], a, bq2[2], bq2[3]);
          }
        }
      }
      __syncthreads();   // everybody is done with the stage: it takes chunk c + SK_STAGES
      issue_w(c + S);
      issue_x(c + S);
      sk_cp_async_commit();
    }
    sk_cp_async_wait_all();
  }
  // the slice's partial: rows 16 mt + lane / 4 (+ 8), columns 16 w + 8 t + 2 (lane % 4) + {0, 1}
  if constexpr (CLUSTER) {
    __syncthreads();   // everybody is done with the operand tiles: the partial takes their place
    float* psm = reinterpret_cast<float*>(sk_smem);   // [ROWS][64]
    const int r0 = lane >> 2, c0 = warp * 16 + 2 * (lane & 3);
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        *reinterpret_cast<float2*>(psm + (16 * mt + r0) * SK_BN + c0 + 8 * t) = make_float2(acc[mt][t][0], acc[mt][t][1]);
        *reinterpret_cast<float2*>(psm + (16 * mt + r0 + 8) * SK_BN + c0 + 8 * t) = make_float2(acc[mt][t][2], acc[mt][t][3]);
        if constexpr (DUAL) {   // the second product's partial follows the first's
          float* psm2 = psm + ROWS * SK_BN;
          *reinterpret_cast<float2*>(psm2 + (16 * mt + r0) * SK_BN + c0 + 8 * t) = make_float2(acc2[DUAL ? mt : 0][t][0], acc2[DUAL ? mt : 0][t][1]);
          *reinterpret_cast<float2*>(psm2 + (16 * mt + r0 + 8) * SK_BN + c0 + 8 * t) = make_float2(acc2[DUAL ? mt : 0][t][2], acc2[DUAL ? mt : 0][t][3]);
        }
      }
    float* ssq = psm + (DUAL ? 2 : 1) * ROWS * SK_BN;   // RMS: [ROWS] sums of squares of this slice, then the warps' [4][ROWS]
    if constexpr (RMS) {
      float* ssw = ssq + ROWS + warp * ROWS;
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        float s0 = ss[mt][0], s1 = ss[mt][1];
        s0 += __shfl_xor_sync(0xffffffffu, s0, 1);
        s0 += __shfl_xor_sync(0xffffffffu, s0, 2);
        s1 += __shfl_xor_sync(0xffffffffu, s1, 1);
        s1 += __shfl_xor_sync(0xffffffffu, s1, 2);
        if ((lane & 3) == 0) { ssw[16 * mt + r0] = s0; ssw[16 * mt + r0 + 8] = s1; }
      }
      __syncthreads();
      if (tid < ROWS) ssq[tid] = (ssq[ROWS + tid] + ssq[2 * ROWS + tid]) + (ssq[3 * ROWS + tid] + ssq[4 * ROWS + tid]);
    }
    sm100::cluster_sync_all();
    const int csize = g.splits;
    const int per = ROWS * SK_BN / csize;   // outputs this CTA finishes (csize is 1, 2, 4 or 8), four per thread and step
    const uint32_t psm_u = sm100::smem_u32(psm);
    for (int e = split * per + 4 * tid; e < (split + 1) * per; e += 4 * SK_THREADS) {
      const int row = e >> 6, col = e & 63;
      if (row < g.M && (!NK || n0 + col < g.N)) {
        float4 pv[8];   // every slice's four values requested before any is used
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          pv[c] = make_float4(0.f, 0.f, 0.f, 0.f);
          if (c < csize)
            asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                         : "=f"(pv[c].x), "=f"(pv[c].y), "=f"(pv[c].z), "=f"(pv[c].w)
                         : "r"(sm100::map_to_cta(psm_u + e * 4u, (uint32_t)c))
                         : "memory");
        }
        float v[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int c = 0; c < 8; ++c) {   // slice order: the same sum on every run (absent slices add +0)
          v[0] += pv[c].x; v[1] += pv[c].y; v[2] += pv[c].z; v[3] += pv[c].w;
        }
        float v2[4] = {0.f, 0.f, 0.f, 0.f};
        if constexpr (DUAL) {
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            pv[c] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (c < csize)
              asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                           : "=f"(pv[c].x), "=f"(pv[c].y), "=f"(pv[c].z), "=f"(pv[c].w)
                           : "r"(sm100::map_to_cta(psm_u + (ROWS * SK_BN + e) * 4u, (uint32_t)c))
                           : "memory");
          }
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            v2[0] += pv[c].x; v2[1] += pv[c].y; v2[2] += pv[c].z; v2[3] += pv[c].w;
          }
        }
        const bool whole = !NK || (g.N & 3) == 0;   // rows of C (bias, residual) are 8-byte aligned at every fourth column (always so for W as [K, N])
        const int64_t at = (int64_t)row * g.N + n0 + col;
        const int valid = g.N - (n0 + col) < 4 ? g.N - (n0 + col) : 4;
        if constexpr (RMS) {   // the row's mean square over all of K: the slices' shares in slice order
          const uint32_t sq_u = sm100::smem_u32(ssq + row);
          float tot = 0.f, part[8];
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            part[c] = 0.f;
            if (c < csize) asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(part[c]) : "r"(sm100::map_to_cta(sq_u, (uint32_t)c)) : "memory");
          }
#pragma unroll
          for (int c = 0; c < 8; ++c) tot += part[c];
          const float rstd = rsqrtf(tot / (float)g.K + g.rms_eps);
#pragma unroll
          for (int j = 0; j < 4; ++j) { v[j] *= rstd; v2[j] *= rstd; }
        }
        if (g.bias) {
          uint2 bq = make_uint2(0, 0);
          T* bt = reinterpret_cast<T*>(&bq);
          if (whole) bq = *reinterpret_cast<const uint2*>(reinterpret_cast<const T*>(g.bias) + n0 + col);
          else if constexpr (NK) {
#pragma unroll
            for (int j = 0; j < 4; ++j)
              if (j < valid) bt[j] = reinterpret_cast<const T*>(g.bias)[n0 + col + j];
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) v[j] += sk_to_f<T>(bt[j]);
        }
        apply_activation_n<4, true>(g.act, v);
        uint2 out;
        T* ot = reinterpret_cast<T*>(&out);
#pragma unroll
        for (int j = 0; j < 4; ++j) ot[j] = sk_from_f<T>(v[j]);
        if constexpr (DUAL) {   // both products rounded, multiplied, rounded again
#pragma unroll
          for (int j = 0; j < 4; ++j) ot[j] = sk_from_f<T>(sk_to_f<T>(ot[j]) * sk_to_f<T>(sk_from_f<T>(v2[j])));
        }
        if (g.residual) {   // the rounded value combined with the residual, rounded again
          uint2 rq = make_uint2(0, 0);
          T* rt = reinterpret_cast<T*>(&rq);
          if (whole) rq = *reinterpret_cast<const uint2*>(reinterpret_cast<const T*>(g.residual) + at);
          else if constexpr (NK) {
#pragma unroll
            for (int j = 0; j < 4; ++j)
              if (j < valid) rt[j] = reinterpret_cast<const T*>(g.residual)[at + j];
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float a = sk_to_f<T>(ot[j]), r = sk_to_f<T>(rt[j]);
            ot[j] = sk_from_f<T>(g.residual_mul ? a * r : a + r);
          }
        }
        if (whole) *reinterpret_cast<uint2*>(reinterpret_cast<T*>(g.c) + at) = out;
        else if constexpr (NK) {
#pragma unroll
          for (int j = 0; j < 4; ++j)
            if (j < valid) reinterpret_cast<T*>(g.c)[at + j] = ot[j];
        }
      }
    }
    sm100::cluster_sync_all();   // nobody leaves while its partial may still be read
    return;
  }
  {
    float* P = g.partial + (int64_t)split * ROWS * g.N + n0 + warp * 16 + 2 * (lane & 3);
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      const int r0 = 16 * mt + (lane >> 2);
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        if (r0 < g.M) __stcg(reinterpret_cast<float2*>(P + (int64_t)r0 * g.N + 8 * t), make_float2(acc[mt][t][0], acc[mt][t][1]));
        if (r0 + 8 < g.M) __stcg(reinterpret_cast<float2*>(P + (int64_t)(r0 + 8) * g.N + 8 * t), make_float2(acc[mt][t][2], acc[mt][t][3]));
      }
    }
  }
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const unsigned old = atomicAdd(g.counters + slab, 1u);
    const int last = old == (unsigned)(g.splits - 1);
    if (last) g.counters[slab] = 0;   // everybody has arrived: ready for the next launch
    s_last = last;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  // the slab's last CTA: thread t owns rows t / 8 + 16 mt, columns [8 (t % 8), 8 (t % 8) + 8)
  const int64_t pstride = (int64_t)ROWS * g.N;
  for (int mt = 0; mt < MT; ++mt) {
    const int row = 16 * mt + (tid >> 3), col = n0 + (tid & 7) * 8;
    if (row >= g.M) break;
    float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    const float* P = g.partial + (int64_t)row * g.N + col;
    int s = 0;
    for (; s + 8 <= g.splits; s += 8) {   // eight slices' loads in flight (each round costs one trip to L2), added in slice order
      float4 q[16];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        q[2 * u] = __ldcg(reinterpret_cast<const float4*>(P + (s + u) * pstride));
        q[2 * u + 1] = __ldcg(reinterpret_cast<const float4*>(P + (s + u) * pstride + 4));
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        v[0] += q[2 * u].x; v[1] += q[2 * u].y; v[2] += q[2 * u].z; v[3] += q[2 * u].w;
        v[4] += q[2 * u + 1].x; v[5] += q[2 * u + 1].y; v[6] += q[2 * u + 1].z; v[7] += q[2 * u + 1].w;
      }
    }
    for (; s < g.splits; ++s) {
      const float4 q0 = __ldcg(reinterpret_cast<const float4*>(P + s * pstride)), q1 = __ldcg(reinterpret_cast<const float4*>(P + s * pstride + 4));
      v[0] += q0.x; v[1] += q0.y; v[2] += q0.z; v[3] += q0.w;
      v[4] += q1.x; v[5] += q1.y; v[6] += q1.z; v[7] += q1.w;
    }
    if (g.bias) {
      const uint4 bq = *reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(g.bias) + col);
      const T* bt = reinterpret_cast<const T*>(&bq);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] += sk_to_f<T>(bt[j]);
    }
    apply_activation_n<8, true>(g.act, v);
    uint4 out;
    T* ot = reinterpret_cast<T*>(&out);
#pragma unroll
    for (int j = 0; j < 8; ++j) ot[j] = sk_from_f<T>(v[j]);
    if (g.residual) {   // the rounded value combined with the residual, rounded again
      const uint4 rq = *reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(g.residual) + (int64_t)row * g.N + col);
      const T* rt = reinterpret_cast<const T*>(&rq);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float a = sk_to_f<T>(ot[j]), r = sk_to_f<T>(rt[j]);
        ot[j] = sk_from_f<T>(g.residual_mul ? a * r : a + r);
      }
    }
    *reinterpret_cast<uint4*>(reinterpret_cast<T*>(g.c) + (int64_t)row * g.N + col) = out;
  }
}

struct SkPlan { int splits, kc, kch, stages, mt; bool cluster; };

int sk_tiles(int64_t m) { return m <= 16 ? 1 : (m <= 32 ? 2 : 4); }
size_t sk_smem_bytes(int kch, int mt, int stages, bool nk, bool dual = false, bool rms = false) {
  const size_t ring = (size_t)stages * ((size_t)(nk ? (kch + 63) / 64 * 64 : kch) * SK_BN * 2 * (dual ? 2 : 1) + (size_t)16 * mt * (kch + SK_X_PAD) * 2 +
                                        (rms ? (size_t)kch * 2 : 0)),
               partial = (size_t)16 * mt * SK_BN * 4 * (dual ? 2 : 1) + (rms ? (size_t)16 * mt * 4 * 5 : 0);
  return ring > partial ? ring : partial;   // the partial takes the ring's place
}

bool sk_cluster_on() {
  static const bool on = []() { const char* v = getenv("B200MLX_GEMM_SKINNY_CLUSTER"); return !(v && v[0] == '0'); }();
  return on;
}

bool sk_shape_ok(const GemmParams& p) {
  static const bool on = []() { const char* v = getenv("B200MLX_GEMM_SKINNY"); return !(v && v[0] == '0'); }();
  if (!on) return false;
  if (p.dtype != B200_BFLOAT16 && p.dtype != B200_FLOAT16) return false;
  if (p.batch != 1 || p.m < 1 || p.m > SK_MAX_ROWS || !p.a_k_major) return false;
  // W as [K, N]: whole 64-column slabs; as [N, K]: any N, through the cluster reduction only (its epilogue handles a ragged N)
  // (and only up to 32768 columns: beyond that the 128 x 256 tensor-core tile has a CTA for every SM and measured faster --
  // GPT-2's 50257 x 768 LM head 34 us there, 47 us here, where a column's K is visited 128 bytes at a time)
  if (p.b_k_major ? (!sk_cluster_on() || p.n > 32768) : p.n % SK_BN != 0) return false;
  if (p.k % 16 != 0 || p.n < SK_BN || p.k < 16 || p.n > (1 << 20) || p.k > (1 << 20)) return false;
  if (p.ldc != 0 && p.ldc != p.n) return false;
  return p.num_c_extra == 0;
}

SkPlan sk_plan(const GemmParams& p, int sm_count) {
  const int64_t slabs = (p.n + SK_BN - 1) / SK_BN;
  const int mt = sk_tiles(p.m);
  const bool cluster_on = sk_cluster_on();
  int64_t splits, kc;
  if (cluster_on) {
    // a power of two of slices, at most 8 (one cluster), up to four CTAs per SM in all -- eight from 32 M weights on (measured:
    // 4096 x 11008 takes 21.6 us so and 29.5 at four per SM, while 3072 x 768 takes 5.4 against 4.6) --, at least 64 of K
    // each (all of it when shorter)
    splits = 8;
    const int64_t per_sm = p.k * p.n >= (32LL << 20) ? 8 : 4;
    while (splits > 1 && (slabs * splits > per_sm * (int64_t)sm_count || p.k / splits < 64)) splits /= 2;
    kc = ((p.k + splits - 1) / splits + 15) / 16 * 16;
    while (splits > 1 && (splits - 1) * kc >= p.k) { splits /= 2; kc = ((p.k + splits - 1) / splits + 15) / 16 * 16; }   // every slice has some of K
  } else {
    splits = (2 * (int64_t)sm_count + slabs - 1) / slabs;
    if (splits < 1) splits = 1;
    if (splits > p.k / 16) splits = p.k / 16;
    if (splits > SK_MAX_SPLITS) splits = SK_MAX_SPLITS;
    kc = ((p.k + splits - 1) / splits + 15) / 16 * 16;
    splits = (p.k + kc - 1) / kc;
  }
  // rows of K per ring stage: 64 (a 10 KB stage at 16 rows of X: five CTAs per SM; 32 measured 30 - 70 % slower), 128 when
  // the CTAs are fewer than two per SM (fewer, longer steps per CTA: 768 x 3072 takes 4.7 us so and 5.3 with 64); never
  // more than the slice
  int64_t kch = slabs * splits < 2 * (int64_t)sm_count ? 128 : 64;
  if (kch > kc) kch = kc;
  // Four stages, or three when the grid fits the SMs at once with three and not with four (a second, nearly empty wave
  // costs a whole CTA's time: 786 slabs of a 50257-column LM head against 740 places)
  auto places = [&](int stages) { return (int64_t)sm_count * (int64_t)((227 * 1024) / (sk_smem_bytes((int)kch, mt, stages, p.b_k_major, p.b2 != nullptr, p.rms_gamma != nullptr) + 1024)); };
  const int64_t ctas = slabs * splits;
  const bool dual = p.b2 != nullptr;
  const int stages = ((p.b_k_major || dual) && ctas > places(SK_STAGES) && ctas <= places(3)) ? 3 : SK_STAGES;
  return SkPlan{(int)splits, (int)kc, (int)kch, stages, mt, cluster_on};
}

template <typename T, bool CLUSTER, bool NK, int S, bool DUAL = false, bool RMS = false>
auto sk_kernel_for2(int mt) -> void (*)(const SkArgs) {
  return mt == 1 ? gemm_skinny_kernel<T, CLUSTER, 1, NK, S, DUAL, RMS>
                 : (mt == 2 ? gemm_skinny_kernel<T, CLUSTER, 2, NK, S, DUAL, RMS> : gemm_skinny_kernel<T, CLUSTER, 4, NK, S, DUAL, RMS>);
}
template <typename T, bool CLUSTER>
auto sk_kernel_for(int mt, bool nk, int stages, bool dual, bool rms) -> void (*)(const SkArgs) {
  if constexpr (CLUSTER) {
    if (rms) {   // (at most 32 rows, like the gated pair)
      if (dual) return stages == 3 ? sk_kernel_for2<T, true, false, 3, true, true>(mt) : sk_kernel_for2<T, true, false, SK_STAGES, true, true>(mt);
      return sk_kernel_for2<T, true, false, SK_STAGES, false, true>(mt);
    }
    if (dual) return stages == 3 ? sk_kernel_for2<T, true, false, 3, true>(mt) : sk_kernel_for2<T, true, false, SK_STAGES, true>(mt);
    if (nk) return stages == 3 ? sk_kernel_for2<T, true, true, 3>(mt) : sk_kernel_for2<T, true, true, SK_STAGES>(mt);   // three stages: W as [N, K] only
    return sk_kernel_for2<T, true, false, SK_STAGES>(mt);
  } else {
    return sk_kernel_for2<T, false, false, SK_STAGES>(mt);   // W as [N, K] always takes the cluster reduction
  }
}

}  // namespace

int64_t gemm_skinny_scratch_bytes(const GemmParams& p, int sm_count) {
  if (!sk_shape_ok(p)) return 0;
  const SkPlan pl = sk_plan(p, sm_count);
  return pl.cluster ? 16 : (int64_t)pl.splits * 16 * pl.mt * p.n * 4;   // (16: "taken", nothing goes through it)
}
// Whether act(A B + bias) * (A B2) can be one launch for this shape (B2 of B's shape and layout).
bool gemm_skinny_dual_ok(const GemmParams& p) { return sk_shape_ok(p) && sk_cluster_on() && !p.b_k_major && p.m <= 32; }
int64_t gemm_skinny_counter_bytes(const GemmParams& p) { return sk_shape_ok(p) ? (p.n + SK_BN - 1) / SK_BN * 4 : 0; }

Status gemm_skinny(Device* dev, const GemmParams& p, bool* taken) {
  *taken = false;
  if (!sk_shape_ok(p) || !p.split_scratch || !p.skinny_counters) return Status::OK();
  const SkPlan pl = sk_plan(p, dev->sm_count());
  if (!pl.cluster && p.split_scratch_bytes < (int64_t)pl.splits * 16 * pl.mt * p.n * 4) return Status::OK();
  auto al = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  if (!al(p.a) || !al(p.b) || !al(p.c) || !al(p.bias) || !al(p.residual) || !al(p.split_scratch)) return Status::OK();
  B200_TRY(dev->MakeCurrent());
  SkArgs g;
  const bool dual = p.b2 != nullptr, rms = p.rms_gamma != nullptr;
  if (dual && (!pl.cluster || p.b_k_major || p.residual || !al(p.b2))) return Status::OK();
  if (rms && (!pl.cluster || p.b_k_major || p.m > 32 || !al(p.rms_gamma))) return Status::OK();   // (likewise: the caller falls back)   // (gemm_skinny_dual_ok said otherwise: the caller falls back)
  g.gamma = p.rms_gamma; g.rms_eps = (float)p.rms_eps;
  g.x = p.a; g.w = p.b; g.w2 = p.b2; g.c = p.c; g.bias = p.bias; g.residual = p.residual;
  g.partial = reinterpret_cast<float*>(p.split_scratch);
  g.counters = reinterpret_cast<unsigned*>(p.skinny_counters);
  g.M = (int)p.m; g.N = (int)p.n; g.K = (int)p.k; g.kc = pl.kc; g.kch = pl.kch; g.stages = pl.stages; g.splits = pl.splits;
  g.act = p.activation; g.residual_mul = p.residual_op;
  g.w_static = p.b_static ? 1 : 0;
  const size_t smem = sk_smem_bytes(pl.kch, pl.mt, pl.stages, p.b_k_major, dual, rms);
  auto kern = p.dtype == B200_FLOAT16 ? (pl.cluster ? sk_kernel_for<__half, true>(pl.mt, p.b_k_major, pl.stages, dual, rms) : sk_kernel_for<__half, false>(pl.mt, false, SK_STAGES, false, false))
                                      : (pl.cluster ? sk_kernel_for<__nv_bfloat16, true>(pl.mt, p.b_k_major, pl.stages, dual, rms) : sk_kernel_for<__nv_bfloat16, false>(pl.mt, false, SK_STAGES, false, false));
  static std::mutex mu;
  static std::map<std::pair<int, const void*>, bool> configured;   // per device and kernel
  {
    std::lock_guard<std::mutex> lk(mu);
    bool& done = configured[{dev->ordinal(), (const void*)kern}];
    if (!done) {
      B200_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sk_smem_bytes(128, 2, SK_STAGES, true, true, true)));
      done = true;
    }
  }
  static const bool pdl_on = []() { const char* v = getenv("B200MLX_PDL"); return !(v && v[0] == '0'); }();
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)((p.n + SK_BN - 1) / SK_BN), (unsigned)pl.splits);
  cfg.blockDim = dim3(SK_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = dev->stream();
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (pl.cluster) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = 1; attr[na].val.clusterDim.y = (unsigned)pl.splits; attr[na].val.clusterDim.z = 1;
    ++na;
  }
  if (pdl_on) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kern, g);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return Status::Cuda(strfmt("gemm_skinny: %s", cudaGetErrorString(e)));
  }
  *taken = true;
  return dev->CheckLaunch("gemm_skinny");
}

}  // namespace k
}  // namespace b200
