// Attention of ONE query position per (batch, head) over a key / value cache: the decoding step.
//
//   o[b, h, :] = softmax_k( scale * q[b, h, :] . K[b, h / group, k, :] + mask[b, h, k] ) V[b, h / group, k, :]     head dim 64
//
// The general lowering runs this as two batched matrix-vector products around a masked softmax (four launches, the
// scores and probabilities through memory); here it is one launch that reads K and V once.  Bandwidth-bound: bytes =
// the cache (2 * Sk * 128 B per KV head and batch entry).
//
// A cluster of up to 8 CTAs owns one (batch, head) and splits the keys.  A CTA walks its keys 256 at a time; eight
// lanes share a key (16 bytes of its K row and of its V row each), so after a 3-step shuffle all eight hold the key's
// score and P.V needs no exchange.  All of a chunk's K and V loads are issued first, as asynchronous copies into the
// thread's own slots of shared memory (64 KB in flight per CTA at no register cost: three CTAs per SM), and each warp
// keeps an online softmax of its own keys, so nothing in the loop waits for another warp.  The warps', then the
// CTAs', (maximum, sum, partial output) meet at the end, the CTAs' through distributed shared memory; CTA 0 writes the row.
// A row with every key masked yields NaN, as the general lowering does.
// When 2 to 16 query heads share a KV head, attention_decode_mma_kernel (below) takes the launch instead.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <map>
#include <mutex>

#include "../kernels.h"
#include "pdl.cuh"
#include "sm100_ptx.cuh"

namespace b200 {
namespace k {

namespace {

constexpr int DEC_THREADS = 256;
constexpr int DEC_CHUNK = 256;     // keys per pass
constexpr int DEC_D = 64;
constexpr int DEC_MAX_SPLITS = 8;
constexpr int DEC_SMEM_BYTES = 2 * (DEC_CHUNK / 32) * DEC_THREADS * 16;   // the chunk in flight: K and V, 16 bytes per thread and key round
constexpr int DEC_WARPS = DEC_THREADS / 32;

struct DecArgs {
  const void* q;
  const void* k;
  const void* v;
  void* o;
  const void* mask;
  int mask_kind;                     // 0 none, 1 Bool (false = masked), 2 additive, of the tensors' dtype
  int64_t m_b, m_h, m_k;             // mask element strides (0 on broadcast dims)
  int B, H, group, Sk;
  int64_t q_sb, q_sh, k_sb, k_sh, k_ss, v_sb, v_sh, v_ss, o_sb, o_sh;   // element strides
  float scale_log2e;
  int keys_per_cta;
};

template <typename T> __device__ __forceinline__ float2 dec_unpack2(uint32_t w);
template <> __device__ __forceinline__ float2 dec_unpack2<__nv_bfloat16>(uint32_t w) {
  return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}
template <> __device__ __forceinline__ float2 dec_unpack2<__half>(uint32_t w) { return __half22float2(*reinterpret_cast<const __half2*>(&w)); }
template <typename T> __device__ __forceinline__ float dec_to_f(T v);
template <> __device__ __forceinline__ float dec_to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float dec_to_f(__half v) { return __half2float(v); }
template <typename T> __device__ __forceinline__ T dec_from_f(float v);
template <> __device__ __forceinline__ __nv_bfloat16 dec_from_f(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half dec_from_f(float v) { return __float2half_rn(v); }

__device__ __forceinline__ float dec_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float dec_ld_cluster(uint32_t addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
  return v;
}

// 16 bytes (eight 16-bit elements) as four float pairs
template <typename T>
__device__ __forceinline__ void dec_unpack8(const uint4& r, float2 (&f)[4]) {
  f[0] = dec_unpack2<T>(r.x);
  f[1] = dec_unpack2<T>(r.y);
  f[2] = dec_unpack2<T>(r.z);
  f[3] = dec_unpack2<T>(r.w);
}

// CONTIG: key rows of K and V are 64 elements apart (a BHSD cache), so every load's offset is an immediate.
template <typename T, bool CONTIG>
__global__ void __launch_bounds__(DEC_THREADS, 3) attention_decode_kernel(const DecArgs g) {
  extern __shared__ __align__(128) unsigned char dec_smem[];   // the chunk in flight: 2 x [8][256] x 16 bytes
  __shared__ float wm[DEC_WARPS], wl[DEC_WARPS];   // each warp's running maximum (log2 units) and sum
  __shared__ float wacc[DEC_WARPS][DEC_D];         // and unnormalised output
  __shared__ float part[DEC_D + 2];                // this CTA's result: output (unnormalised), maximum, sum
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bh = blockIdx.x, rank = blockIdx.y, csize = gridDim.y;
  const int b = bh / g.H, h = bh - b * g.H, hkv = h / g.group;
  pdl_launch_dependents();
  pdl_wait();
  const int64_t kss = CONTIG ? DEC_D : g.k_ss, vss = CONTIG ? DEC_D : g.v_ss;
  const int key_begin = rank * g.keys_per_cta;
  const int key_end = key_begin + g.keys_per_cta < g.Sk ? key_begin + g.keys_per_cta : g.Sk;
  // Lane (kq, part) of warp w: keys 32 it + 4 w + kq of every 256-key chunk (it = 0..7), dims [8 part, 8 part + 8) of
  // both K and V.  The eight lanes of a key all end up with its score, so P.V needs no exchange, and a warp keeps an
  // online softmax of its own keys: nothing in the loop waits for another warp.
  const int kq = lane >> 3, dpart = lane & 7;
  const int key0 = warp * 4 + kq;
  const T* Kt = reinterpret_cast<const T*>(g.k) + (int64_t)b * g.k_sb + (int64_t)hkv * g.k_sh + (int64_t)(key_begin + key0) * kss + dpart * 8;
  const T* Vt = reinterpret_cast<const T*>(g.v) + (int64_t)b * g.v_sb + (int64_t)hkv * g.v_sh + (int64_t)(key_begin + key0) * vss + dpart * 8;
  const int64_t mrow = (int64_t)b * g.m_b + (int64_t)h * g.m_h;
  float2 qf[4];   // the query's eight dims, pre-multiplied by scale * log2(e)
  {
    const uint4 qv = *reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(g.q) + (int64_t)b * g.q_sb + (int64_t)h * g.q_sh + dpart * 8);
    dec_unpack8<T>(qv, qf);
    const float2 sl = make_float2(g.scale_log2e, g.scale_log2e);
#pragma unroll
    for (int i = 0; i < 4; ++i) qf[i] = __fmul2_rn(qf[i], sl);
  }
  float m_run = -INFINITY, l_run = 0.f;
  float2 acc[4] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
  constexpr int ITS = DEC_CHUNK / 32;
  for (int c0 = key_begin; c0 < key_end; c0 += DEC_CHUNK, Kt += DEC_CHUNK * kss, Vt += DEC_CHUNK * vss) {
    const bool full = c0 + DEC_CHUNK <= key_end;
    // Every load of the chunk is issued up front (V does not depend on the scores), as asynchronous copies into the
    // thread's own 16-byte slots of shared memory: the chunk in flight costs no registers, which is what lets three
    // CTAs share an SM.  A thread reads back only what it copied itself, so its own wait is all the ordering needed.
    uint4* kslot = reinterpret_cast<uint4*>(dec_smem) + threadIdx.x;   // [ITS][256] for K, then the same for V
    uint4* vslot = kslot + ITS * DEC_THREADS;
    {
      const uint32_t ks = sm100::smem_u32(kslot), vs = sm100::smem_u32(vslot);
#pragma unroll
      for (int it = 0; it < ITS; ++it) {
        const bool in = full || c0 + it * 32 + key0 < key_end;
        if (in) {
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(ks + it * DEC_THREADS * 16), "l"(Kt + it * 32 * kss) : "memory");
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(vs + it * DEC_THREADS * 16), "l"(Vt + it * 32 * vss) : "memory");
        } else {
          kslot[it * DEC_THREADS] = make_uint4(0, 0, 0, 0);
          vslot[it * DEC_THREADS] = make_uint4(0, 0, 0, 0);
        }
      }
    }
    float s[ITS];
    // the keys' mask terms, in log2 units (the eight lanes of a key read the same element)
#pragma unroll
    for (int it = 0; it < ITS; ++it) {
      const int key = c0 + it * 32 + key0;
      s[it] = key < key_end ? 0.f : -INFINITY;
      if (g.mask_kind != 0 && key < key_end) {
        if (g.mask_kind == 1) s[it] = reinterpret_cast<const uint8_t*>(g.mask)[mrow + (int64_t)key * g.m_k] ? 0.f : -INFINITY;
        else s[it] = dec_to_f<T>(reinterpret_cast<const T*>(g.mask)[mrow + (int64_t)key * g.m_k]) * 1.4426950408889634f;
      }
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
    // scores
    float cmax = -INFINITY;
#pragma unroll
    for (int it = 0; it < ITS; ++it) {
      float2 kf[4];
      dec_unpack8<T>(kslot[it * DEC_THREADS], kf);
      float2 d2 = __fmul2_rn(kf[0], qf[0]);
#pragma unroll
      for (int i = 1; i < 4; ++i) d2 = __ffma2_rn(kf[i], qf[i], d2);
      float d = d2.x + d2.y;
      d += __shfl_xor_sync(0xffffffffu, d, 1);
      d += __shfl_xor_sync(0xffffffffu, d, 2);
      d += __shfl_xor_sync(0xffffffffu, d, 4);
      s[it] += d;
      cmax = fmaxf(cmax, s[it]);
    }
    cmax = fmaxf(cmax, __shfl_xor_sync(0xffffffffu, cmax, 8));
    cmax = fmaxf(cmax, __shfl_xor_sync(0xffffffffu, cmax, 16));
    const float m_new = fmaxf(m_run, cmax);
    const float m_safe = m_new == -INFINITY ? 0.f : m_new;   // every key so far masked: keep the arithmetic finite
    const float alpha = dec_exp2(m_run - m_safe);            // 0 on the first chunk (m_run = -inf)
    m_run = m_new;
    const float2 a2 = make_float2(alpha, alpha);
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[i] = __fmul2_rn(acc[i], a2);
    float lsum = 0.f;
#pragma unroll
    for (int it = 0; it < ITS; ++it) {
      const float pk = dec_exp2(s[it] - m_safe);   // 0 for a masked key and past the end
      lsum += pk;
      float2 vf[4];
      dec_unpack8<T>(vslot[it * DEC_THREADS], vf);
      const float2 p2 = make_float2(pk, pk);
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[i] = __ffma2_rn(p2, vf[i], acc[i]);
    }
    l_run = fmaf(l_run, alpha, lsum);   // this lane group's keys only; the groups meet below
  }
  // the warp's four key groups (they share m_run), then the CTA's warps, meet in a fixed order
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 8);
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 16);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    acc[i].x += __shfl_xor_sync(0xffffffffu, acc[i].x, 8);
    acc[i].y += __shfl_xor_sync(0xffffffffu, acc[i].y, 8);
    acc[i].x += __shfl_xor_sync(0xffffffffu, acc[i].x, 16);
    acc[i].y += __shfl_xor_sync(0xffffffffu, acc[i].y, 16);
  }
  if (kq == 0) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      wacc[warp][dpart * 8 + 2 * i] = acc[i].x;
      wacc[warp][dpart * 8 + 2 * i + 1] = acc[i].y;
    }
    if (dpart == 0) { wm[warp] = m_run; wl[warp] = l_run; }
  }
  __syncthreads();
  if (threadIdx.x < DEC_D) {
    float M = wm[0];
#pragma unroll
    for (int w = 1; w < DEC_WARPS; ++w) M = fmaxf(M, wm[w]);
    const float Ms = M == -INFINITY ? 0.f : M;
    float L = 0.f, O = 0.f;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) {
      const float wgt = dec_exp2(wm[w] - Ms);
      L = fmaf(wl[w], wgt, L);
      O = fmaf(wacc[w][threadIdx.x], wgt, O);
    }
    part[threadIdx.x] = O;
    if (threadIdx.x == 0) { part[DEC_D] = M; part[DEC_D + 1] = L; }
  }
  __syncthreads();
  // the CTAs' results meet through distributed shared memory; CTA 0 writes the row
  if (csize > 1) sm100::cluster_sync_all();
  if (rank == 0 && threadIdx.x < DEC_D) {
    const uint32_t base = sm100::smem_u32(&part[0]);
    float M = -INFINITY;
    for (int r = 0; r < csize; ++r) M = fmaxf(M, csize > 1 ? dec_ld_cluster(sm100::map_to_cta(base + DEC_D * 4u, (uint32_t)r)) : part[DEC_D]);
    const float Ms = M == -INFINITY ? 0.f : M;
    float L = 0.f, O = 0.f;
    for (int r = 0; r < csize; ++r) {
      const uint32_t pb = csize > 1 ? sm100::map_to_cta(base, (uint32_t)r) : 0u;
      const float mr = csize > 1 ? dec_ld_cluster(pb + DEC_D * 4u) : part[DEC_D];
      const float lr = csize > 1 ? dec_ld_cluster(pb + (DEC_D + 1) * 4u) : part[DEC_D + 1];
      const float orr = csize > 1 ? dec_ld_cluster(pb + threadIdx.x * 4u) : part[threadIdx.x];
      const float wgt = dec_exp2(mr - Ms);
      L = fmaf(lr, wgt, L);
      O = fmaf(orr, wgt, O);
    }
    T* Op = reinterpret_cast<T*>(g.o) + (int64_t)b * g.o_sb + (int64_t)h * g.o_sh;
    Op[threadIdx.x] = dec_from_f<T>(O / L);   // L = 0 (every key masked): NaN
  }
  if (csize > 1) sm100::cluster_sync_all();   // nobody leaves while its result may still be read
}

// ---- the group's heads as the rows of a tensor-core product ----------------------------------------------------
// One cluster per (batch, KV head); the group's query heads (up to 16) are the 16 rows of mma.sync m16n8k16 products:
// S = Q K^T with K's rows as the column operand, O += P V with V through ldmatrix.trans and P taken from the score
// accumulators in registers.  The FMA kernel above spends about 20 instructions per head and key, which binds grouped-
// query attention on instruction issue rather than on the cache's bytes; here a warp's 32 keys cost 32 MMAs and a
// two-row softmax whatever the group size.  Chunks of 128 keys (K and V, 32 KB) stream through a ring of three
// XOR-swizzled buffers in shared memory, two chunks always in flight under the arithmetic; warp w owns keys
// [16 w, 16 w + 16) of a chunk and an online softmax of its own.
template <typename T> __device__ __forceinline__ uint32_t dec_pack2(float lo, float hi);
template <> __device__ __forceinline__ uint32_t dec_pack2<__nv_bfloat16>(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}
template <> __device__ __forceinline__ uint32_t dec_pack2<__half>(float lo, float hi) {
  const __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}
template <typename T> __device__ __forceinline__ void dec_mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <> __device__ __forceinline__ void dec_mma<__nv_bfloat16>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <> __device__ __forceinline__ void dec_mma<__half>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void dec_ldmatrix_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void dec_ldmatrix_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

constexpr int DEC_GROUP_ROWS = 16;
constexpr int DEC_MMA_CHUNK = 128;                                   // keys per ring buffer: 16 per warp
constexpr int DEC_MMA_BUFS = 3;
constexpr int DEC_MMA_BUF_BYTES = 2 * DEC_MMA_CHUNK * DEC_D * 2;      // K and V of one chunk
constexpr int DEC_MMA_SMEM_BYTES = DEC_MMA_BUFS * DEC_MMA_BUF_BYTES;  // 96 KB: two CTAs per SM

template <typename T>
__global__ void __launch_bounds__(DEC_THREADS, 2) attention_decode_mma_kernel(const DecArgs g) {
  extern __shared__ __align__(128) unsigned char dec_smem[];   // three buffers of K [128][128 B] + V [128][128 B]; 16-byte units XOR (row & 7)
  __shared__ __align__(128) unsigned char qsm[DEC_GROUP_ROWS * DEC_D * 2];   // the group's queries (rows past the group zero), same swizzle
  __shared__ float wm[DEC_WARPS][DEC_GROUP_ROWS], wl[DEC_WARPS][DEC_GROUP_ROWS];
  __shared__ float part[DEC_GROUP_ROWS][DEC_D + 2];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int rank = blockIdx.y, csize = gridDim.y;
  const int G = g.group;
  const int hkv_count = g.H / G;
  const int b = blockIdx.x / hkv_count, hkv = blockIdx.x - b * hkv_count;
  const int h0 = hkv * G;
  pdl_launch_dependents();
  pdl_wait();
  const int key_begin = rank * g.keys_per_cta;
  const int key_end = key_begin + g.keys_per_cta < g.Sk ? key_begin + g.keys_per_cta : g.Sk;
  const T* Kb = reinterpret_cast<const T*>(g.k) + (int64_t)b * g.k_sb + (int64_t)hkv * g.k_sh;
  const T* Vb = reinterpret_cast<const T*>(g.v) + (int64_t)b * g.v_sb + (int64_t)hkv * g.v_sh;
  const uint32_t ring_u = sm100::smem_u32(dec_smem), qsm_u = sm100::smem_u32(qsm);
  // the queries: 16 rows x 8 units of 16 bytes
  if (tid < DEC_GROUP_ROWS * 8) {
    const int row = tid >> 3, c = tid & 7;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (row < G) v = *reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(g.q) + (int64_t)b * g.q_sb + (int64_t)(h0 + row) * g.q_sh + c * 8);
    *reinterpret_cast<uint4*>(qsm + row * 128 + ((c ^ (row & 7)) << 4)) = v;
  }
  __syncthreads();
  uint32_t qa[4][4];   // Q as the row operand, four k-steps of 16 dims
  {
    const int mi = lane >> 3, row = (mi & 1) * 8 + (lane & 7);
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) dec_ldmatrix_x4(qsm_u + row * 128 + (((2 * kk + (mi >> 1)) ^ (row & 7)) << 4), qa[kk]);
  }
  // this thread's rows (heads) hr0 = lane / 4 and hr0 + 8; its columns within an 8-key tile 2 (lane % 4) + {0, 1}
  const int hr0 = lane >> 2, hr1 = hr0 + 8, kc2 = 2 * (lane & 3);
  const int64_t mrow0 = (int64_t)b * g.m_b + (int64_t)(h0 + hr0) * g.m_h, mrow1 = (int64_t)b * g.m_b + (int64_t)(h0 + hr1) * g.m_h;
  const bool row0_real = hr0 < G, row1_real = hr1 < G;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  float o[8][4];
#pragma unroll
  for (int n = 0; n < 8; ++n)
#pragma unroll
    for (int i = 0; i < 4; ++i) o[n][i] = 0.f;
  // A ring of three buffers of 128 keys (K 16 KB + V 16 KB each): chunk c + 2 is requested before chunk c is multiplied,
  // so two chunks are always in flight under the arithmetic and one barrier per chunk is all the ordering needed (the
  // buffer that takes chunk c + 2 held chunk c - 1, which every warp finished before this iteration's barrier).
  const int nchunks = (key_end - key_begin + DEC_MMA_CHUNK - 1) / DEC_MMA_CHUNK;
  // Thread (lk, lc) copies 16-byte unit lc of keys lk, lk + 32, lk + 64, lk + 96 of a chunk: its offset in a buffer
  // (the swizzle depends on lk & 7 only) and its sources advance by constants.
  const int lk = tid >> 3, lc = tid & 7;
  const uint32_t l_off = lk * 128 + ((lc ^ (lk & 7)) << 4);
  const T* k_thread = Kb + (int64_t)(key_begin + lk) * g.k_ss + lc * 8;
  const T* v_thread = Vb + (int64_t)(key_begin + lk) * g.v_ss + lc * 8;
  const int64_t k_step = 32 * g.k_ss, v_step = 32 * g.v_ss;
  auto issue = [&](int c) {
    if (c < nchunks) {
      const int c0 = key_begin + c * DEC_MMA_CHUNK;
      const uint32_t kb_u = ring_u + (c % DEC_MMA_BUFS) * DEC_MMA_BUF_BYTES + l_off, vb_u = kb_u + DEC_MMA_CHUNK * DEC_D * 2;
      const T* ks = k_thread + (int64_t)c * DEC_MMA_CHUNK * g.k_ss;
      const T* vs = v_thread + (int64_t)c * DEC_MMA_CHUNK * g.v_ss;
      if (c0 + DEC_MMA_CHUNK <= key_end) {   // a whole chunk: no guards
#pragma unroll
        for (int it = 0; it < 4; ++it) {
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(kb_u + it * 32 * 128), "l"(ks + it * k_step) : "memory");
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(vb_u + it * 32 * 128), "l"(vs + it * v_step) : "memory");
        }
      } else {
#pragma unroll
        for (int it = 0; it < 4; ++it) {
          if (c0 + lk + 32 * it < key_end) {
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(kb_u + it * 32 * 128), "l"(ks + it * k_step) : "memory");
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(vb_u + it * 32 * 128), "l"(vs + it * v_step) : "memory");
          } else {
            const uint32_t z = 0;
            asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(kb_u + it * 32 * 128), "r"(z) : "memory");
            asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(vb_u + it * 32 * 128), "r"(z) : "memory");
          }
        }
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");   // one group per chunk index, empty past the end
  };
  issue(0);
  issue(1);
  for (int c = 0; c < nchunks; ++c) {
    const int c0 = key_begin + c * DEC_MMA_CHUNK;
    // the mask terms of this thread's 2 rows x 4 keys, in log2 units, requested before the wait
    const int wkey = c0 + warp * 16;   // the warp's first key
    float mk[2][4];
    const int64_t mkey = (int64_t)(wkey + kc2) * g.m_k;   // the thread's first key of the chunk in the mask
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int key = wkey + 8 * j + kc2 + (i & 1);
        const bool real = (i < 2 ? row0_real : row1_real);
        float t = key < key_end ? 0.f : -INFINITY;
        if (g.mask_kind != 0 && key < key_end && real) {
          const int64_t at = (i < 2 ? mrow0 : mrow1) + mkey + (8 * j + (i & 1)) * g.m_k;
          if (g.mask_kind == 1) t = reinterpret_cast<const uint8_t*>(g.mask)[at] ? 0.f : -INFINITY;
          else t = dec_to_f<T>(reinterpret_cast<const T*>(g.mask)[at]) * 1.4426950408889634f;
        }
        mk[j][i] = t;
      }
    asm volatile("cp.async.wait_group 1;" ::: "memory");   // chunk c has landed (groups complete in order)
    __syncthreads();
    issue(c + 2);
    if (wkey >= key_end) continue;   // nothing of this chunk is this warp's (warp-uniform; the barrier is above)
    const uint32_t kbuf_u = ring_u + (c % DEC_MMA_BUFS) * DEC_MMA_BUF_BYTES, vbuf_u = kbuf_u + DEC_MMA_CHUNK * DEC_D * 2;
    // S = Q K^T for the warp's 16 keys: two 8-key tiles x four k-steps
    float sc[2][4];
    {
      const int mi = lane >> 3, r = lane & 7;
#pragma unroll
      for (int j = 0; j < 2; ++j) {
#pragma unroll
        for (int i = 0; i < 4; ++i) sc[j][i] = 0.f;
        const uint32_t rowaddr = kbuf_u + (warp * 16 + 8 * j + r) * 128;
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          uint32_t kb[4];
          dec_ldmatrix_x4(rowaddr + (((4 * hh + mi) ^ r) << 4), kb);
          dec_mma<T>(sc[j], qa[2 * hh], kb[0], kb[1]);
          dec_mma<T>(sc[j], qa[2 * hh + 1], kb[2], kb[3]);
        }
      }
    }
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
#pragma unroll
      for (int i = 0; i < 4; ++i) sc[j][i] = fmaf(sc[j][i], g.scale_log2e, mk[j][i]);
      mx0 = fmaxf(mx0, fmaxf(sc[j][0], sc[j][1]));
      mx1 = fmaxf(mx1, fmaxf(sc[j][2], sc[j][3]));
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
    const float ms0 = mn0 == -INFINITY ? 0.f : mn0, ms1 = mn1 == -INFINITY ? 0.f : mn1;   // every key so far masked: stay finite
    const float al0 = dec_exp2(m0 - ms0), al1 = dec_exp2(m1 - ms1);
    m0 = mn0;
    m1 = mn1;
    float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      sc[j][0] = dec_exp2(sc[j][0] - ms0);
      sc[j][1] = dec_exp2(sc[j][1] - ms0);
      sc[j][2] = dec_exp2(sc[j][2] - ms1);
      sc[j][3] = dec_exp2(sc[j][3] - ms1);
      ps0 += sc[j][0] + sc[j][1];
      ps1 += sc[j][2] + sc[j][3];
    }
    l0 = fmaf(l0, al0, ps0);   // this thread's keys only; the quad meets at the end
    l1 = fmaf(l1, al1, ps1);
#pragma unroll
    for (int n = 0; n < 8; ++n) { o[n][0] *= al0; o[n][1] *= al0; o[n][2] *= al1; o[n][3] *= al1; }
    // O += P V: one k-step of 16 keys; P from the score registers, V through ldmatrix.trans
    {
      const int mi = lane >> 3, r = lane & 7;
      uint32_t pa[4];
      pa[0] = dec_pack2<T>(sc[0][0], sc[0][1]);
      pa[1] = dec_pack2<T>(sc[0][2], sc[0][3]);
      pa[2] = dec_pack2<T>(sc[1][0], sc[1][1]);
      pa[3] = dec_pack2<T>(sc[1][2], sc[1][3]);
      const uint32_t rowaddr = vbuf_u + (warp * 16 + (mi & 1) * 8 + r) * 128;
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        uint32_t vb[4];
        dec_ldmatrix_x4_trans(rowaddr + (((2 * u + (mi >> 1)) ^ r) << 4), vb);
        dec_mma<T>(o[2 * u], pa, vb[0], vb[1]);
        dec_mma<T>(o[2 * u + 1], pa, vb[2], vb[3]);
      }
    }
  }
  asm volatile("cp.async.wait_all;" ::: "memory");
  // the quad's sums, then the warps' (maximum, sum, output) through shared memory (the outputs take the chunk's place)
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  __syncthreads();
  float (*wo)[DEC_GROUP_ROWS][DEC_D] = reinterpret_cast<float (*)[DEC_GROUP_ROWS][DEC_D]>(dec_smem);   // [8][16][64] floats = 32 KB
#pragma unroll
  for (int n = 0; n < 8; ++n) {
    *reinterpret_cast<float2*>(&wo[warp][hr0][8 * n + kc2]) = make_float2(o[n][0], o[n][1]);
    *reinterpret_cast<float2*>(&wo[warp][hr1][8 * n + kc2]) = make_float2(o[n][2], o[n][3]);
  }
  if ((lane & 3) == 0) { wm[warp][hr0] = m0; wm[warp][hr1] = m1; wl[warp][hr0] = l0; wl[warp][hr1] = l1; }
  __syncthreads();
  for (int e = tid; e < G * DEC_D; e += DEC_THREADS) {
    const int gi = e >> 6, d = e & 63;
    float M = wm[0][gi];
#pragma unroll
    for (int w = 1; w < DEC_WARPS; ++w) M = fmaxf(M, wm[w][gi]);
    const float Ms = M == -INFINITY ? 0.f : M;
    float L = 0.f, O = 0.f;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) {
      const float wgt = dec_exp2(wm[w][gi] - Ms);
      L = fmaf(wl[w][gi], wgt, L);
      O = fmaf(wo[w][gi][d], wgt, O);
    }
    part[gi][d] = O;
    if (d == 0) { part[gi][DEC_D] = M; part[gi][DEC_D + 1] = L; }
  }
  __syncthreads();
  if (csize > 1) sm100::cluster_sync_all();
  if (rank == 0) {
    for (int e = tid; e < G * DEC_D; e += DEC_THREADS) {
      const int gi = e >> 6, d = e & 63;
      const uint32_t base = sm100::smem_u32(&part[gi][0]);
      float M = -INFINITY;
      for (int r = 0; r < csize; ++r) M = fmaxf(M, csize > 1 ? dec_ld_cluster(sm100::map_to_cta(base + DEC_D * 4u, (uint32_t)r)) : part[gi][DEC_D]);
      const float Ms = M == -INFINITY ? 0.f : M;
      float L = 0.f, O = 0.f;
      for (int r = 0; r < csize; ++r) {
        const uint32_t pb = csize > 1 ? sm100::map_to_cta(base, (uint32_t)r) : 0u;
        const float mr = csize > 1 ? dec_ld_cluster(pb + DEC_D * 4u) : part[gi][DEC_D];
        const float lr = csize > 1 ? dec_ld_cluster(pb + (DEC_D + 1) * 4u) : part[gi][DEC_D + 1];
        const float orr = csize > 1 ? dec_ld_cluster(pb + d * 4u) : part[gi][d];
        const float wgt = dec_exp2(mr - Ms);
        L = fmaf(lr, wgt, L);
        O = fmaf(orr, wgt, O);
      }
      T* Op = reinterpret_cast<T*>(g.o) + (int64_t)b * g.o_sb + (int64_t)(h0 + gi) * g.o_sh;
      Op[d] = dec_from_f<T>(O / L);   // L = 0 (every key masked): NaN
    }
  }
  if (csize > 1) sm100::cluster_sync_all();   // nobody leaves while its result may still be read
}

}  // namespace

bool attention_decode_supported(const AttentionParams& p) {
  static const bool on = []() { const char* v = getenv("B200MLX_DECODE_ATTENTION"); return !(v && v[0] == '0'); }();
  const bool is16 = p.dtype == B200_BFLOAT16 || p.dtype == B200_FLOAT16;
  if (!on || !is16 || p.head_dim != DEC_D || p.Sq != 1 || p.causal) return false;
  if (p.B <= 0 || p.H <= 0 || p.Hkv <= 0 || p.Sk <= 0 || p.H % p.Hkv != 0 || p.B * p.H > 0x7fffffffLL || p.Sk > 0x7fffffffLL) return false;
  return p.scale > 0 && p.scale < 1e30;
}

Status attention_decode(Device* dev, const AttentionParams& p) {
  if (!attention_decode_supported(p)) return Status::Unsupported("attention_decode: needs one query position, head dim 64, 16-bit floats, no causal flag");
  auto al = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  if (!al(p.q) || !al(p.k) || !al(p.v)) return Status::Unsupported("attention_decode: operands must be 16-byte aligned");
  B200_TRY(dev->MakeCurrent());
  DecArgs g;
  g.q = p.q; g.k = p.k; g.v = p.v; g.o = p.o;
  g.mask = p.mask; g.mask_kind = p.mask ? p.mask_kind : 0;
  g.m_b = p.m_b; g.m_h = p.m_h; g.m_k = p.m_k;
  g.B = (int)p.B; g.H = (int)p.H; g.group = (int)(p.H / p.Hkv); g.Sk = (int)p.Sk;
  auto strides = [&](int64_t S, int64_t Hx, const int64_t* custom, int64_t* sb, int64_t* sh, int64_t* ss) {
    if (custom[0] | custom[1] | custom[2]) { *sb = custom[0]; *sh = custom[1]; *ss = custom[2]; return; }
    if (p.bshd) { *ss = Hx * DEC_D; *sh = DEC_D; *sb = S * Hx * DEC_D; }
    else { *ss = DEC_D; *sh = S * DEC_D; *sb = Hx * S * DEC_D; }
  };
  int64_t q_ss, o_ss;
  const int64_t none[3] = {0, 0, 0};
  strides(1, p.H, p.q_strides, &g.q_sb, &g.q_sh, &q_ss);
  strides(p.Sk, p.Hkv, p.k_strides, &g.k_sb, &g.k_sh, &g.k_ss);
  strides(p.Sk, p.Hkv, p.v_strides, &g.v_sb, &g.v_sh, &g.v_ss);
  strides(1, p.H, none, &g.o_sb, &g.o_sh, &o_ss);
  if ((g.q_sb | g.q_sh | g.k_sb | g.k_sh | g.k_ss | g.v_sb | g.v_sh) % 8 != 0 || g.v_ss % 8 != 0)
    return Status::Unsupported("attention_decode: operand strides must be multiples of 8 elements");
  g.scale_log2e = (float)(p.scale * 1.4426950408889634);
  // Which kernel: the group's heads as the rows of tensor-core products (one cluster per KV head) from B200MLX_DECODE_ATTENTION_MMA
  // heads per group on (default 2; 1 = always, 0 = never), else one cluster per head on the FMA pipe.
  static const int mma_from = []() { const char* v = getenv("B200MLX_DECODE_ATTENTION_MMA"); return v ? atoi(v) : 2; }();
  const bool use_mma = mma_from > 0 && g.group >= mma_from && g.group <= DEC_GROUP_ROWS;
  // CTAs per cluster: as many as keep the whole grid resident at once (three CTAs of 64 KB per SM; two of the tensor-
  // core kernel) -- a second wave of short CTAs costs more than longer CTAs do --, whole 256-key chunks, at most 8
  const int64_t bh = use_mma ? p.B * p.Hkv : p.B * p.H;
  int64_t splits = (use_mma ? 2 : 3) * (int64_t)dev->sm_count() / bh;
  if (splits < 1) splits = 1;
  if (splits > DEC_MAX_SPLITS) splits = DEC_MAX_SPLITS;
  if (splits > (p.Sk + DEC_CHUNK - 1) / DEC_CHUNK) splits = (p.Sk + DEC_CHUNK - 1) / DEC_CHUNK;
  if (splits < 1) splits = 1;
  int64_t per = ((p.Sk + splits - 1) / splits + DEC_CHUNK - 1) / DEC_CHUNK * DEC_CHUNK;
  splits = (p.Sk + per - 1) / per;
  g.keys_per_cta = (int)per;
  static const bool pdl_on = []() { const char* v = getenv("B200MLX_PDL"); return !(v && v[0] == '0'); }();
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)bh, (unsigned)splits);
  cfg.blockDim = dim3(DEC_THREADS);
  cfg.dynamicSmemBytes = use_mma ? DEC_MMA_SMEM_BYTES : DEC_SMEM_BYTES;
  cfg.stream = dev->stream();
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1; attr[0].val.clusterDim.y = (unsigned)splits; attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_on ? 2 : 1;
  const bool contig = g.k_ss == DEC_D && g.v_ss == DEC_D;
  void (*kern)(const DecArgs) = p.dtype == B200_FLOAT16 ? (contig ? attention_decode_kernel<__half, true> : attention_decode_kernel<__half, false>)
                                                        : (contig ? attention_decode_kernel<__nv_bfloat16, true> : attention_decode_kernel<__nv_bfloat16, false>);
  if (use_mma) kern = p.dtype == B200_FLOAT16 ? attention_decode_mma_kernel<__half> : attention_decode_mma_kernel<__nv_bfloat16>;
  {
    static std::mutex mu;
    static std::map<std::pair<int, const void*>, bool> configured;   // the shared-memory opt-in is per device and kernel
    std::lock_guard<std::mutex> lk(mu);
    bool& done = configured[{dev->ordinal(), (const void*)kern}];
    if (!done) {
      B200_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, use_mma ? DEC_MMA_SMEM_BYTES : DEC_SMEM_BYTES));
      done = true;
    }
  }
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kern, g);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return Status::Cuda(strfmt("attention_decode: %s", cudaGetErrorString(e)));
  }
  return dev->CheckLaunch("attention_decode");
}

}  // namespace k
}  // namespace b200
