// Fused scaled-dot-product attention (flash style) on tcgen05 tensor cores.
//
//   O = softmax(scale * Q K^T + causal mask) V        per (batch, head), head dim 64,
// for Q [B, Sq, H, 64] / K, V [B, Sk, Hkv, 64] in either BSHD or BHSD order, with
// grouped-query attention (query head h reads KV head h / (H / Hkv)).
//
// The reference lowers FusedScaledDotProductAttention to two batched matmuls
// around a softmax and materialises the [B, H, Sq, Sk] score tensor, a causal
// mask built from two iotas, repeated K/V heads for GQA and up to four layout
// transposes (mpsgraph function.go:2697-2907).  Here none of those tensors
// exists: one CTA owns 128 query rows of one head and walks the keys in blocks of
// 64 with an online softmax, reading Q, K and V in place through TMA.
//
// Per key block:  S = Q K_j^T   (tcgen05.mma 128 x 64 x 16, four per block, fp32 in TMEM)
//                 each of the 128 threads owns one query row: tcgen05.ld its 64 scores,
//                 mask, running max / sum in base 2, P = exp2(...) rounded to the input
//                 type and written to shared memory in the 128-byte-swizzled K-major layout
//                 O_j = P V_j   (tcgen05.mma 128 x 64 x 16, four per block; V is read as an
//                 MN-major operand, so it needs no transpose)
//                 O = O * alpha + O_j in registers.
// K/V blocks are double-buffered; three CTAs fit on an SM, so one CTA's softmax
// overlaps another's MMAs.  Causal launches skip key blocks right of the diagonal.
// Tensor-bound in flops (4 * Sq * Sk * 64 per head, half that when causal), with
// the exponentials (one MUFU op per score) as the co-limiter.
// Every mbarrier wait is bounded; a wait that gives up sets the device's error word.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <mutex>

#include "../kernels.h"
#include "sm100_ptx.cuh"
#include "tma_host.h"

namespace b200 {
namespace k {

namespace {

using namespace sm100;

constexpr int HD = 64;           // head dim
constexpr int BQ = 128;          // query rows per CTA (UMMA M)
constexpr int BKV = 64;          // keys per step (UMMA N of the score MMA, K of the PV MMA)
constexpr int Q_BYTES = BQ * HD * 2;     // 16 KiB
constexpr int KV_BYTES = BKV * HD * 2;   // 8 KiB
constexpr int P_BYTES = BQ * BKV * 2;    // 16 KiB
constexpr int ATT_SMEM = Q_BYTES + 4 * KV_BYTES + P_BYTES + 1024 + 128;
constexpr int ATT_THREADS = 128;
constexpr int ATT_TMEM_COLS = 128;       // 64 score columns + 64 output columns

struct AttArgs {
  void* o;
  int64_t o_sb, o_sh, o_ss;   // element strides of O along batch, head, sequence (head dim contiguous)
  int B, H, Hkv, Sq, Sk;
  int causal;
  int is_f16;
  float scale_log2e;          // scale * log2(e)
  int* err_flag;
};

template <typename T> __device__ __forceinline__ uint32_t pack2(float a, float b);
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <> __device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <typename T>
__global__ void __launch_bounds__(ATT_THREADS, 3)
attention_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                 const __grid_constant__ CUtensorMap tm_v, const AttArgs g) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* sQ = base;
  unsigned char* sK = sQ + Q_BYTES;            // two buffers
  unsigned char* sV = sK + 2 * KV_BYTES;       // two buffers
  unsigned char* sP = sV + 2 * KV_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + P_BYTES);
  uint64_t* q_full = bars;          // [1]
  uint64_t* kv_full = bars + 1;     // [2]
  uint64_t* s_done = bars + 3;      // [1] score MMAs finished
  uint64_t* pv_done = bars + 4;     // [1] PV MMAs finished
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 5);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* err = g.err_flag;

  // work item: heavy (late) query blocks first so the causal tail is short
  const int nq = (g.Sq + BQ - 1) / BQ;
  const int64_t item = blockIdx.x;
  const int qb = nq - 1 - (int)(item % nq);
  const int h = (int)((item / nq) % g.H);
  const int b = (int)(item / ((int64_t)nq * g.H));
  const int hkv = h / (g.H / g.Hkv);
  const int q0 = qb * BQ;
  int kv_end = g.Sk;
  if (g.causal) kv_end = (q0 + BQ < g.Sk) ? q0 + BQ : g.Sk;   // keys beyond the block's last row are masked for every row
  const int nkv = (kv_end + BKV - 1) / BKV;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(&kv_full[0], 1);
    mbar_init(&kv_full[1], 1);
    mbar_init(s_done, 1);
    mbar_init(pv_done, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, ATT_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_s = tmem_base, tmem_o = tmem_base + 64;
  const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;   // this warp's 32 TMEM lanes

  // instruction descriptors: fp32 accumulate, M = 128, N = 64
  const uint32_t fmt = g.is_f16 ? 0u : 1u;
  const uint32_t idesc_common = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(64 >> 3) << 17) | ((uint32_t)(BQ >> 4) << 24);
  const uint32_t idesc_s = idesc_common;                 // Q (K-major) x K_j (K-major)
  const uint32_t idesc_pv = idesc_common | (1u << 16);   // P (K-major) x V_j (MN-major)

  bool ok = true;
  bool issued = true;   // thread 0: false once one of its own waits gave up
  if (threadIdx.x == 0) {
    mbar_expect_tx(q_full, Q_BYTES);
    tma_load_4d(sQ, &tm_q, q_full, 0, q0, h, b);
    mbar_expect_tx(&kv_full[0], 2 * KV_BYTES);
    tma_load_4d(sK, &tm_k, &kv_full[0], 0, 0, hkv, b);
    tma_load_4d(sV, &tm_v, &kv_full[0], 0, 0, hkv, b);
  }

  const int row = warp * 32 + lane;      // query row inside the block
  const int q_row = q0 + row;
  float o_acc[HD];
#pragma unroll
  for (int d = 0; d < HD; ++d) o_acc[d] = 0.f;
  float m_run = -INFINITY, l_run = 0.f;

  for (int j = 0; j < nkv; ++j) {
    const int buf = j & 1;
    const uint32_t par = (uint32_t)(j & 1);
    if (threadIdx.x == 0) {
      // prefetch the next key/value block into the other buffer (its last readers, the PV MMAs of step j-1, are done)
      if (j + 1 < nkv) {
        mbar_expect_tx(&kv_full[buf ^ 1], 2 * KV_BYTES);
        tma_load_4d(sK + (buf ^ 1) * KV_BYTES, &tm_k, &kv_full[buf ^ 1], 0, (j + 1) * BKV, hkv, b);
        tma_load_4d(sV + (buf ^ 1) * KV_BYTES, &tm_v, &kv_full[buf ^ 1], 0, (j + 1) * BKV, hkv, b);
      }
      bool landed = (j > 0) || mbar_wait(q_full, 0, err, 1);
      landed = landed && mbar_wait(&kv_full[buf], (uint32_t)((j >> 1) & 1), err, 3);
      issued = landed;
      if (landed) {
        tc_fence_after();
        const uint32_t a0 = smem_u32(sQ), b0 = smem_u32(sK + buf * KV_BYTES);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k)
          umma_f16(tmem_s, make_smem_desc(a0 + k * 32, 16, 1024), make_smem_desc(b0 + k * 32, 16, 1024), idesc_s, k != 0 ? 1u : 0u);
      }
      tc_commit(s_done);   // also arrives when nothing was issued, so the other threads never wait on a dead step
    }
    // ---- scores -> probabilities ----
    {
      const bool landed = mbar_wait(s_done, par, err, 4);
      if (!__syncthreads_and((landed && issued) ? 1 : 0)) { ok = false; break; }
    }
    tc_fence_after();
    uint32_t sr[64];
    tmem_ld32(tmem_s + lane_addr, sr);
    tmem_ld32(tmem_s + lane_addr + 32, sr + 32);
    tmem_ld_wait();
    const int kv0 = j * BKV;
    int limit = g.Sk - kv0;                               // columns >= limit are masked
    if (g.causal && q_row + 1 - kv0 < limit) limit = q_row + 1 - kv0;
    float mx = m_run;
#pragma unroll
    for (int c = 0; c < 64; ++c) {
      float t = __uint_as_float(sr[c]) * g.scale_log2e;
      t = (c < limit) ? t : -INFINITY;
      sr[c] = __float_as_uint(t);
      mx = fmaxf(mx, t);
    }
    // a row with nothing visible yet keeps m = -inf; use 0 as the reference point so exp2 sees -inf, not NaN
    const float m_ref = (mx == -INFINITY) ? 0.f : mx;
    const float alpha = fast_exp2(m_run - m_ref);
    float psum = 0.f;
    uint32_t packed[32];
#pragma unroll
    for (int c = 0; c < 64; c += 2) {
      const float p0 = fast_exp2(__uint_as_float(sr[c]) - m_ref);
      const float p1 = fast_exp2(__uint_as_float(sr[c + 1]) - m_ref);
      psum += p0 + p1;
      packed[c >> 1] = pack2<T>(p0, p1);
    }
    l_run = l_run * alpha + psum;
    m_run = mx;
    // P row -> shared memory, K-major with 128-byte swizzle: 16-byte chunk c of row r lives at chunk (c ^ (r & 7))
    {
      unsigned char* prow = sP + row * 128;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        uint4 q = make_uint4(packed[4 * c], packed[4 * c + 1], packed[4 * c + 2], packed[4 * c + 3]);
        *reinterpret_cast<uint4*>(prow + ((c ^ (row & 7)) << 4)) = q;
      }
    }
    fence_proxy_async_smem();
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0) {
      tc_fence_after();
      const uint32_t a0 = smem_u32(sP), b0 = smem_u32(sV + buf * KV_BYTES);
#pragma unroll
      for (int k = 0; k < BKV / 16; ++k)
        umma_f16(tmem_o, make_smem_desc(a0 + k * 32, 16, 1024), make_smem_desc(b0 + k * 2048, 8192, 1024), idesc_pv, k != 0 ? 1u : 0u);
      tc_commit(pv_done);
    }
    // rescale the running output while the PV MMAs run
#pragma unroll
    for (int d = 0; d < HD; ++d) o_acc[d] *= alpha;
    {
      const bool landed = mbar_wait(pv_done, par, err, 2);
      if (!__syncthreads_and(landed ? 1 : 0)) { ok = false; break; }
    }
    tc_fence_after();
    uint32_t pr[64];
    tmem_ld32(tmem_o + lane_addr, pr);
    tmem_ld32(tmem_o + lane_addr + 32, pr + 32);
    tmem_ld_wait();
#pragma unroll
    for (int d = 0; d < HD; ++d) o_acc[d] += __uint_as_float(pr[d]);
    tc_fence_before();
    // the next step's score MMA overwrites tmem_s and its PV MMA overwrites tmem_o and sP: every thread has finished
    // reading them once it passes the __syncthreads_and at the top of the next step (score) / the one above (PV).
  }

  if (ok && q_row < g.Sq) {
    const float inv = 1.0f / l_run;   // a fully masked row (l = 0) yields NaN, as the unfused path does
    T* orow = reinterpret_cast<T*>(g.o) + (int64_t)b * g.o_sb + (int64_t)h * g.o_sh + (int64_t)q_row * g.o_ss;
#pragma unroll
    for (int d = 0; d < HD; d += 8) {
      uint4 q;
      q.x = pack2<T>(o_acc[d] * inv, o_acc[d + 1] * inv);
      q.y = pack2<T>(o_acc[d + 2] * inv, o_acc[d + 3] * inv);
      q.z = pack2<T>(o_acc[d + 4] * inv, o_acc[d + 5] * inv);
      q.w = pack2<T>(o_acc[d + 6] * inv, o_acc[d + 7] * inv);
      *reinterpret_cast<uint4*>(orow + d) = q;
    }
  }

  tc_fence_before();
  __shared__ int failed;
  if (threadIdx.x == 0) failed = ok ? 0 : 1;
  __syncthreads();
  if (failed != 0) {
    const unsigned long long t0 = global_ns();
    while (global_ns() - t0 < 200000ull) {}
    __syncthreads();
  }
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, ATT_TMEM_COLS);
  }
}

}  // namespace

bool attention_supported(const AttentionParams& p) {
  const bool is16 = p.dtype == B200_BFLOAT16 || p.dtype == B200_FLOAT16;
  if (!is16 || p.head_dim != HD) return false;
  if (p.B <= 0 || p.H <= 0 || p.Hkv <= 0 || p.Sq <= 0 || p.Sk <= 0 || p.H % p.Hkv != 0) return false;
  auto al = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  return al(p.q) && al(p.k) && al(p.v) && al(p.o);
}

Status attention(Device* dev, const AttentionParams& p) {
  if (!attention_supported(p)) return Status::Unsupported("attention: needs 16-bit floats, head dim 64 and 16-byte aligned tensors");
  B200_TRY(dev->MakeCurrent());
  const bool f16 = p.dtype == B200_FLOAT16;
  // element strides (batch, head, sequence) of a [B, S, Hx, 64] (BSHD) or [B, Hx, S, 64] (BHSD) tensor
  auto strides = [&](int64_t S, int64_t Hx, int64_t* sb, int64_t* sh, int64_t* ss) {
    if (p.bshd) { *ss = Hx * HD; *sh = HD; *sb = S * Hx * HD; }
    else { *ss = HD; *sh = S * HD; *sb = Hx * S * HD; }
  };
  auto make_map = [&](CUtensorMap* map, const void* base, int64_t S, int64_t Hx, int rows, const int64_t* custom) -> Status {
    int64_t sb, sh, ss;
    strides(S, Hx, &sb, &sh, &ss);
    if (custom[0] | custom[1] | custom[2]) { sb = custom[0]; sh = custom[1]; ss = custom[2]; }
    if ((sb % 8) | (sh % 8) | (ss % 8)) return Status::Unsupported("attention: operand strides must be multiples of 8 elements");
    const uint64_t dims[4] = {(uint64_t)HD, (uint64_t)S, (uint64_t)Hx, (uint64_t)p.B};
    const uint64_t st[3] = {(uint64_t)ss * 2, (uint64_t)sh * 2, (uint64_t)sb * 2};
    const uint32_t box[4] = {(uint32_t)HD, (uint32_t)rows, 1, 1};
    return encode_tma_4d_16bit(map, base, f16, dims, st, box);
  };
  CUtensorMap tq, tk, tv;
  B200_TRY(make_map(&tq, p.q, p.Sq, p.H, BQ, p.q_strides));
  B200_TRY(make_map(&tk, p.k, p.Sk, p.Hkv, BKV, p.k_strides));
  B200_TRY(make_map(&tv, p.v, p.Sk, p.Hkv, BKV, p.v_strides));
  AttArgs g;
  g.o = p.o;
  strides(p.Sq, p.H, &g.o_sb, &g.o_sh, &g.o_ss);
  g.B = (int)p.B; g.H = (int)p.H; g.Hkv = (int)p.Hkv; g.Sq = (int)p.Sq; g.Sk = (int)p.Sk;
  g.causal = p.causal ? 1 : 0;
  g.is_f16 = f16 ? 1 : 0;
  g.scale_log2e = (float)(p.scale * 1.4426950408889634);
  g.err_flag = dev->kernel_error_flag();
  const int64_t nq = (p.Sq + BQ - 1) / BQ;
  const int64_t grid = nq * p.H * p.B;
  if (grid > 0x7fffffffLL) return Status::Unsupported("attention: too many work items");
  static std::mutex attr_mu;
  static bool attr_done[2][64] = {};
  cudaError_t e = cudaSuccess;
  {
    std::lock_guard<std::mutex> lock(attr_mu);
    const int slot = f16 ? 1 : 0;
    if (!attr_done[slot][dev->ordinal()]) {
      e = f16 ? cudaFuncSetAttribute(attention_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, ATT_SMEM)
              : cudaFuncSetAttribute(attention_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, ATT_SMEM);
      attr_done[slot][dev->ordinal()] = (e == cudaSuccess);
    }
  }
  if (e == cudaSuccess) {
    if (f16) attention_kernel<__half><<<(unsigned)grid, ATT_THREADS, ATT_SMEM, dev->stream()>>>(tq, tk, tv, g);
    else attention_kernel<__nv_bfloat16><<<(unsigned)grid, ATT_THREADS, ATT_SMEM, dev->stream()>>>(tq, tk, tv, g);
  } else {
    cudaGetLastError();
    return Status::Cuda(strfmt("attention: %s", cudaGetErrorString(e)));
  }
  return dev->CheckLaunch("attention");
}

}  // namespace k
}  // namespace b200
