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
// exists: one CTA owns 256 query rows of one head (two tiles of 128) and walks
// the keys in blocks of 64 with an online softmax, reading Q, K and V in place
// through TMA.
//
// Persistent CTAs (two per SM) walk the work items; the next item's queries are loaded while this one is computed.
// Warp roles (320 threads):
//   warp 0      loader: Q once, then K_j / V_j blocks into a 3-stage ring;
//   warp 1      issuer: S_t = Q_t K_j^T (tcgen05.mma 128 x 64 x 16, fp32 in TMEM) and O_t += P_t V_j for both tiles
//               (V read as an MN-major operand, so it needs no transpose); the two tiles alternate, so one tile's
//               MMAs run under the other tile's softmax;
//   warps 2-5   softmax of tile 0, warps 6-9 of tile 1: each thread owns one query row: tcgen05.ld its 64 scores,
//               running max / sum in base 2 with the scale folded into the exponent's FMA, P = exp2(...) rounded to
//               the input type and written back over S in TENSOR MEMORY (tcgen05.st), where the PV MMA reads it as its
//               A operand: P never touches shared memory.
// The output accumulates in TMEM across key blocks.  Its reference maximum is only moved when a row's maximum grew by
// more than 2^8 since the last move (then the row of O is rescaled in TMEM); P stays below 2^8 and the final division
// by the row sum cancels the common factor, so nothing is lost and most blocks skip the rescale.
// Causal launches skip key blocks right of the diagonal.  Tensor-bound in flops (4 * Sq * Sk * 64 per head, half that
// when causal) with the exponentials (one MUFU op per score, 16 per clock per SM) as the real limiter at head dim 64.
// Every mbarrier wait is bounded; a wait that gives up sets the device's error word.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <mutex>

#include "../kernels.h"
#include "pdl.cuh"
#include "sm100_ptx.cuh"
#include "tma_host.h"

namespace b200 {
namespace k {

namespace {

using namespace sm100;

constexpr int HD = 64;           // head dim
constexpr int BQ = 128;          // query rows per tile (UMMA M)
constexpr int QT = 2;            // query tiles per CTA
constexpr int BKV = 64;          // keys per step (UMMA N of the score MMA, K of the PV MMA)
constexpr int KV_STAGES = 3;
constexpr int Q_BYTES = BQ * HD * 2;     // 16 KiB per tile
constexpr int KV_BYTES = BKV * HD * 2;   // 8 KiB (K or V)
constexpr int Q_BUFS = 2;             // the next work item's queries are loaded while this one is computed
constexpr int ATT_TILE_BYTES = Q_BUFS * QT * Q_BYTES + KV_STAGES * 2 * KV_BYTES;  // 112 KiB: P never touches shared memory
constexpr int ATT_SMEM = ATT_TILE_BYTES + 256;   // + barriers; the dynamic window itself is 1024-byte aligned (checked)
constexpr int ATT_THREADS = 320;
constexpr int ATT_TMEM_COLS = 256;       // S0, S1, O0, O1: 64 columns each
constexpr float kRescaleThreshold = 8.f; // log2 units
// every ATT_POLY_MOD-th pair of scores takes its exp2 from the FMA pipe (measured at S = 2048, B = 8, not causal: none 728,
// every 5th 760, 4th 794, 3rd 805, 2nd 748 TFLOP/s: past a third the softmax warps run out of issue slots)
constexpr int ATT_POLY_MOD = 3;

struct AttArgs {
  void* o;
  int64_t o_sb, o_sh, o_ss;   // element strides of O along batch, head, sequence (head dim contiguous)
  int B, H, Hkv, Sq, Sk;
  int group;                  // query heads per KV head: H / Hkv
  int causal;
  int is_f16;
  float scale_log2e;          // scale * log2(e), > 0
  int* err_flag;
  int* next_item;             // [0] work items beyond the first of each CTA are taken from here; [1] CTAs that have finished
};

// The work-item counter of a launch and the count of its finished CTAs (one pair per device: the array lives in each
// device's copy of the module).  Both are zero between launches: the last CTA to finish puts them back, so no memset
// has to sit between this kernel and the one before it (which would keep it from starting under that kernel's tail).
// Launches of one device are ordered on its stream.
__device__ int g_next_item[4];

template <typename T> __device__ __forceinline__ uint32_t pack2(float a, float b);
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <> __device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float y;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(y) : "f"(a), "f"(b), "f"(c));
  return y;
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// 2^x for a pair of fp32 values without the special-function unit.  x <= 8 here (the rescale threshold bounds it);
// x below -126 (a masked score is -inf) is clamped, which yields 2^-126 instead of 0: it vanishes in every sum.
__device__ __forceinline__ float2 exp2_fma_pair(float2 x) {
  const float2 magic = make_float2(12582912.f, 12582912.f);   // 1.5 * 2^23: adding it rounds x to an integer in the low mantissa bits
  const float2 neg_magic = make_float2(-12582912.f, -12582912.f);
  x.x = fmaxf(x.x, -126.f);
  x.y = fmaxf(x.y, -126.f);
  const float2 xf = __fadd2_rn(x, magic);
  const float2 r = __ffma2_rn(__fadd2_rn(xf, neg_magic), make_float2(-1.f, -1.f), x);   // x - round(x), in [-1/2, 1/2]
  // minimax cubic for 2^r on [-1/2, 1/2]: relative error 7.5e-5
  const float2 k3 = make_float2(0.05517093f, 0.05517093f), k2 = make_float2(0.24260931f, 0.24260931f);
  const float2 k1 = make_float2(0.69326094f, 0.69326094f), k0 = make_float2(0.99992819f, 0.99992819f);
  float2 pl = __ffma2_rn(r, k3, k2);
  pl = __ffma2_rn(pl, r, k1);
  pl = __ffma2_rn(pl, r, k0);
  // the integer sits in the low bits of xf: shifted into the exponent field and added (the constant part of magic's
  // bit pattern has no bits below bit 9, so it shifts out)
  float2 out;
  out.x = __uint_as_float(__float_as_uint(pl.x) + (__float_as_uint(xf.x) << 23));
  out.y = __uint_as_float(__float_as_uint(pl.y) + (__float_as_uint(xf.y) << 23));
  return out;
}

template <typename T>
__global__ void __launch_bounds__(ATT_THREADS, 2)
attention_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                 const __grid_constant__ CUtensorMap tm_v, const AttArgs g) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* sQ = smem_raw;                          // [Q_BUFS][QT] tiles
  unsigned char* sKV = sQ + Q_BUFS * QT * Q_BYTES;       // [KV_STAGES] x (K, V)
  uint64_t* bars = reinterpret_cast<uint64_t*>(sKV + KV_STAGES * 2 * KV_BYTES);
  uint64_t* q_full = bars;                       // [Q_BUFS] the item's queries landed
  uint64_t* q_empty = q_full + Q_BUFS;           // [Q_BUFS] the item's score MMAs are done AND its 8 softmax warps have staged O through the buffer
  uint64_t* kv_full = q_empty + Q_BUFS;          // [KV_STAGES] bytes of K_j and V_j landed
  uint64_t* kv_empty = kv_full + KV_STAGES;      // [KV_STAGES] every MMA that reads the stage is done
  uint64_t* s_full = kv_empty + KV_STAGES;       // [QT] scores of the current block are in TMEM
  uint64_t* p_ready = s_full + QT;               // [QT] P is in tensor memory (and S has been read): 4 warp arrivals
  uint64_t* o_done = p_ready + QT;               // [QT] the PV MMAs of the current block are done
  uint64_t* item_ready = o_done + QT;            // [Q_BUFS] the loader has published the work item that will use this Q buffer
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(item_ready + Q_BUFS);
  int* failed = reinterpret_cast<int*>(tmem_slot + 1);
  volatile int* s_item = reinterpret_cast<volatile int*>(tmem_slot + 2);   // [Q_BUFS] work item per Q buffer; -1: no more work

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* err = g.err_flag;

  // Persistent CTAs: the fixed cost of a CTA -- launch, TMEM allocation, the first loads, the drain -- is paid once per
  // CTA instead of once per work item (256 query rows of one head; it measured 7.5 us per item against 1.5 us per key
  // block).  Items are ordered heaviest first (latest query block under a causal mask).  A CTA starts with item
  // blockIdx.x and takes every further one from a global counter when it gets there, so a CTA that drew light items
  // simply does more of them: with a fixed round-robin deal, GPT-2's shape (768 items of 4..16 key-block steps on 296
  // CTAs) left the busiest CTA with 32 steps against a mean of 26.  The loader draws the item and publishes it to the
  // other warps through shared memory (item_ready); barrier phases keep counting across items.
  const int nq = (g.Sq + QT * BQ - 1) / (QT * BQ);
  const int64_t heads_total = (int64_t)g.H * g.B;
  const int64_t num_items = (int64_t)nq * heads_total;
  struct Item {
    int h, b, hkv, q0, nkv0, nkv1, nkv_max;
  };
  auto decode = [&](int64_t item) {
    Item it;
    // 32-bit unsigned arithmetic (the launcher refuses 2^31 items and more): this runs once per item in the
    // single-thread loader and issuer, where a 64-bit division is some hundred dependent instructions
    const uint32_t item32 = (uint32_t)item, ht32 = (uint32_t)heads_total, H32 = (uint32_t)g.H;
    const uint32_t qi = item32 / ht32;
    const uint32_t hb = item32 - qi * ht32;
    const uint32_t bi = hb / H32;
    const int qb = nq - 1 - (int)qi;
    it.h = (int)(hb - bi * H32);
    it.b = (int)bi;
    it.hkv = (int)((uint32_t)it.h / (uint32_t)g.group);
    it.q0 = qb * QT * BQ;
    // key blocks each tile walks: under a causal mask keys beyond the tile's last row are masked for every row
    auto blocks_of = [&](int t) {
      const int first = it.q0 + t * BQ;
      int kv_end = g.Sk;
      if (g.causal && first + BQ < kv_end) kv_end = first + BQ;
      return first < g.Sq ? (kv_end + BKV - 1) / BKV : 0;   // a tile wholly past the last query row does nothing
    };
    it.nkv0 = blocks_of(0);
    it.nkv1 = blocks_of(1);
    it.nkv_max = it.nkv0 > it.nkv1 ? it.nkv0 : it.nkv1;
    return it;
  };

  if (threadIdx.x == 0) {
    for (int q = 0; q < Q_BUFS; ++q) { mbar_init(&q_full[q], 1); mbar_init(&q_empty[q], 1 + QT * 4); mbar_init(&item_ready[q], 1); }
    for (int s = 0; s < KV_STAGES; ++s) { mbar_init(&kv_full[s], 1); mbar_init(&kv_empty[s], 1); }
    for (int t = 0; t < QT; ++t) { mbar_init(&s_full[t], 1); mbar_init(&p_ready[t], 4); mbar_init(&o_done[t], 1); }
    *failed = 0;
    if ((smem_u32(smem_raw) & 1023u) != 0) { atomicCAS((int*)g.err_flag, 0, 5); *failed = 1; }  // swizzled tiles need the alignment
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, ATT_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const bool misaligned = *failed != 0;
  // everything above ran under the tail of the kernel before this one (when launched as its programmatic dependent)
  pdl_launch_dependents();
  pdl_wait();

  if (misaligned) {
    // nothing was issued; fall through to the teardown
  } else if (warp == 0) {
    // -------------------------------------------------------------------- loader ---
    if (lane == 0) {
      int s = 0;
      uint32_t phase = 0, n_item = 0;
      bool ok = true;
      for (int64_t item = blockIdx.x; ok; ++n_item) {
        const int qbuf = (int)(n_item & 1);
        if (!mbar_wait(&q_empty[qbuf], ((n_item >> 1) & 1) ^ 1, err, 1)) break;   // the slot's previous item is finished everywhere
        const bool more = item < num_items;
        s_item[qbuf] = more ? (int)item : -1;
        mbar_arrive(&item_ready[qbuf]);   // release: the store above is visible to whoever sees this phase complete
        if (!more) break;
        const Item it = decode(item);
        mbar_expect_tx(&q_full[qbuf], QT * Q_BYTES);
#pragma unroll
        for (int t = 0; t < QT; ++t) tma_load_4d(sQ + (qbuf * QT + t) * Q_BYTES, &tm_q, &q_full[qbuf], 0, it.q0 + t * BQ, it.h, it.b);
        for (int j = 0; j < it.nkv_max; ++j) {
          if (!mbar_wait(&kv_empty[s], phase ^ 1, err, 1)) { ok = false; break; }
          unsigned char* dst = sKV + s * 2 * KV_BYTES;
          mbar_expect_tx(&kv_full[s], 2 * KV_BYTES);
          tma_load_4d(dst, &tm_k, &kv_full[s], 0, j * BKV, it.hkv, it.b);
          tma_load_4d(dst + KV_BYTES, &tm_v, &kv_full[s], 0, j * BKV, it.hkv, it.b);
          if (++s == KV_STAGES) { s = 0; phase ^= 1; }
        }
        item = (int64_t)gridDim.x + atomicAdd(g.next_item, 1);
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------------- issuer ---
    if (lane == 0) {
      // instruction descriptors: fp32 accumulate, M = 128, N = 64
      const uint32_t fmt = g.is_f16 ? 0u : 1u;
      const uint32_t idesc_s = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(64 >> 3) << 17) | ((uint32_t)(BQ >> 4) << 24);
      const uint32_t idesc_pv = idesc_s | (1u << 16);   // P (K-major) x V_j (MN-major)
      const uint64_t dq0 = make_smem_desc(smem_u32(sQ), 16, 1024);
      const uint64_t dk0 = make_smem_desc(smem_u32(sKV), 16, 1024);
      const uint64_t dv0 = make_smem_desc(smem_u32(sKV) + KV_BYTES, 8192, 1024);
      int qbuf = 0;
      auto issue_scores = [&](int t, int stage) {   // S_t = Q_t K^T
        const uint64_t dq = dq0 + (uint64_t)(((qbuf * QT + t) * Q_BYTES) >> 4), dk = dk0 + (uint64_t)((stage * 2 * KV_BYTES) >> 4);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) umma_f16(tmem_base + t * 64, dq + (uint64_t)((k * 32) >> 4), dk + (uint64_t)((k * 32) >> 4), idesc_s, k != 0 ? 1u : 0u);
        tc_commit(&s_full[t]);
      };
      int s = 0;
      uint32_t phase = 0, n_item = 0;
      uint32_t done[QT] = {0, 0};   // key blocks each tile has finished so far, over all items: the phase of its barriers
      bool ok = true;
      for (;; ++n_item) {
        qbuf = (int)(n_item & 1);
        if (!mbar_wait(&item_ready[qbuf], (n_item >> 1) & 1, err, 2)) break;
        const int item = s_item[qbuf];
        if (item < 0) break;
        const Item it = decode(item);
        if (it.nkv_max == 0) { tc_commit(&q_empty[qbuf]); continue; }   // the loader loaded Q anyway: hand the buffer back
        ok = mbar_wait(&q_full[qbuf], (n_item >> 1) & 1, err, 2);
        if (ok) ok = mbar_wait(&kv_full[s], phase, err, 3);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int t = 0; t < QT; ++t)
          if ((t ? it.nkv1 : it.nkv0) > 0) issue_scores(t, s);
        for (int j = 0; j < it.nkv_max && ok; ++j) {
          const int s_next = (s + 1 == KV_STAGES) ? 0 : s + 1;
          const uint32_t phase_next = (s + 1 == KV_STAGES) ? (phase ^ 1) : phase;
          bool next_landed = false;
#pragma unroll
          for (int t = 0; t < QT; ++t) {
            const int nt = t ? it.nkv1 : it.nkv0;
            if (j >= nt) continue;
            if (!mbar_wait(&p_ready[t], done[t] & 1, err, 4)) { ok = false; break; }
            tc_fence_after();
            // O_t (+)= P_t V_j.  P_t lies in the first 32 columns of S_t (two 16-bit values per column): 16 keys per MMA = 8 columns
            const uint64_t dv = dv0 + (uint64_t)((s * 2 * KV_BYTES) >> 4);
#pragma unroll
            for (int k = 0; k < BKV / 16; ++k)
              umma_f16_ts(tmem_base + 128 + t * 64, tmem_base + t * 64 + k * 8, dv + (uint64_t)((k * 2048) >> 4), idesc_pv, (j | k) != 0 ? 1u : 0u);
            tc_commit(&o_done[t]);
            ++done[t];
            // the tile's next scores go out at once: its softmax warps have read S_t (they said so with p_ready)
            if (j + 1 < nt) {
              if (!next_landed) {
                if (!mbar_wait(&kv_full[s_next], phase_next, err, 3)) { ok = false; break; }
                tc_fence_after();
                next_landed = true;
              }
              issue_scores(t, s_next);
            }
          }
          if (!ok) break;
          tc_commit(&kv_empty[s]);   // every MMA that reads stage s has been issued before this point
          s = s_next;
          phase = phase_next;
        }
        if (!ok) break;
        tc_commit(&q_empty[qbuf]);   // every score MMA of this item has been issued: Q may be replaced when they are done
      }
    }
  } else {
    // ------------------------------------------------------------------- softmax ---
    const int t = (warp - 2) >> 2;          // query tile
    const int quarter = warp & 3;           // TMEM lanes [32 * quarter, +32) are this warp's
    const int row = quarter * 32 + lane;    // row inside the tile
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const uint32_t tmem_s = tmem_base + t * 64 + lane_addr, tmem_o = tmem_base + 128 + t * 64 + lane_addr;
    const float c = g.scale_log2e;
    uint32_t done = 0;                      // key blocks this tile has finished so far, over all items: the barriers' phase
    uint32_t n_item = 0;
    bool ok = true;
    for (; ok; ++n_item) {
    {
      const bool published = mbar_wait(&item_ready[n_item & 1], (n_item >> 1) & 1, err, 6);
      if (!__all_sync(0xffffffffu, published)) break;
    }
    const int item = s_item[n_item & 1];
    if (item < 0) break;
    const Item it = decode(item);
    const int h = it.h, b = it.b;
    const int q_row = it.q0 + t * BQ + row;   // the row this thread's softmax works on
    float m_ref = 0.f, l_run = 0.f;         // p = exp2(c * s - m_ref)
    const int n = t ? it.nkv1 : it.nkv0;
    for (int j = 0; j < n; ++j) {
      {
        const bool landed = mbar_wait(&s_full[t], done & 1, err, 6);
        if (!__all_sync(0xffffffffu, landed)) { ok = false; break; }   // tcgen05.ld is warp-collective: leave together
      }
      tc_fence_after();
      const int kv0 = j * BKV;
      int limit = g.Sk - kv0;                               // columns >= limit are masked
      if (g.causal && q_row + 1 - kv0 < limit) limit = q_row + 1 - kv0;
      // The block's 64 scores of this row stay in registers from the maximum (pass 1) to the exponentials (pass 2): a
      // TMEM read costs some 300 cycles of pure latency on the tile's critical path.  Only when the reference maximum
      // moves (the first block of an item, then rarely) are they dropped across the rescale of O and read again.
      uint32_t sr[64];
      auto load_scores = [&]() {
        tmem_ld32(tmem_s, sr);
        tmem_ld32(tmem_s + 32, sr + 32);
        tmem_ld_wait();
        if (limit < 64) {
#pragma unroll
          for (int cidx = 0; cidx < 64; ++cidx)
            if (cidx >= limit) sr[cidx] = 0xff800000u;   // -inf
        }
      };
      load_scores();
      // Pass 1: the row maximum: three-input maximum (sm_100), 32 instructions in four independent chains
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
      for (int cidx = 0; cidx < 64; cidx += 8) {
        mx0 = max3(mx0, __uint_as_float(sr[cidx]), __uint_as_float(sr[cidx + 1]));
        mx1 = max3(mx1, __uint_as_float(sr[cidx + 2]), __uint_as_float(sr[cidx + 3]));
        mx2 = max3(mx2, __uint_as_float(sr[cidx + 4]), __uint_as_float(sr[cidx + 5]));
        mx3 = max3(mx3, __uint_as_float(sr[cidx + 6]), __uint_as_float(sr[cidx + 7]));
      }
      const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
      const float m_new = mx * c;                           // c > 0: the maximum commutes with the scale
      // Move the reference only when some row of the warp needs it (tcgen05.ld / st are warp-collective).
      const bool grow = (j == 0) ? true : (m_new > m_ref + kRescaleThreshold);
      if (__any_sync(0xffffffffu, grow)) {
        const float m_next = grow ? (m_new == -INFINITY ? 0.f : m_new) : m_ref;
        if (j > 0) {
          // the PV MMAs of block j-1 must have landed before O is touched
          const bool landed = mbar_wait(&o_done[t], (done - 1) & 1, err, 7);
          if (!__all_sync(0xffffffffu, landed)) { ok = false; break; }
          tc_fence_after();
          const float alpha = fast_exp2(m_ref - m_next);    // 1 for rows that keep their reference
          l_run *= alpha;
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            uint32_t orow[32];
            tmem_ld32(tmem_o + half * 32, orow);
            tmem_ld_wait();
#pragma unroll
            for (int d = 0; d < 32; ++d) orow[d] = __float_as_uint(__uint_as_float(orow[d]) * alpha);
            tmem_st32(tmem_o + half * 32, orow);
          }
          tmem_st_wait();
          load_scores();   // the registers were given to the row of O
        }
        m_ref = m_next;
      }
      // Pass 2: P = exp2(c * s - m_ref), rounded to the input type, written over the first 32 columns of S_t, where the
      // PV MMA reads it as its A operand (the PV MMAs of block j-1 read the previous P there, but they were issued
      // before the score MMAs that produced this S, and MMAs run in issue order: they are done).
      float psum0 = 0.f, psum1 = 0.f;
      {
        // One exponential per score makes the special-function unit (16 per clock per SM) the kernel's limiter at head
        // dim 64, so every third pair of scores takes its exp2 from the FMA pipe instead: round to the nearest integer n
        // with the 1.5 * 2^23 trick, a cubic for 2^r on r in [-1/2, 1/2] (relative error 7.5e-5, below half an ulp of
        // the 16-bit P), n added into the exponent field.  Scale, sums and the cubic use the packed two-lane fp32 forms.
        const float2 c2 = make_float2(c, c), nm2 = make_float2(-m_ref, -m_ref);
        float2 psum = make_float2(0.f, 0.f);
#pragma unroll
        for (int cidx = 0; cidx < 64; cidx += 2) {
          const float2 x = __ffma2_rn(make_float2(__uint_as_float(sr[cidx]), __uint_as_float(sr[cidx + 1])), c2, nm2);
          float2 pr;
          if ((cidx >> 1) % ATT_POLY_MOD == ATT_POLY_MOD - 1) pr = exp2_fma_pair(x);
          else pr = make_float2(fast_exp2(x.x), fast_exp2(x.y));
          psum = __fadd2_rn(psum, pr);
          sr[cidx >> 1] = pack2<T>(pr.x, pr.y);   // in place: entry cidx / 2 has been consumed
        }
        psum0 = psum.x;
        psum1 = psum.y;
        tmem_st32(tmem_s, sr);
        tmem_st_wait();
      }
      l_run += psum0 + psum1;
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_ready[t]);
      ++done;
    }
    // Epilogue.  A thread owns a whole output row, so storing from registers would scatter every store instruction over
    // 32 rows.  The item's query tile in shared memory is dead by now (every score MMA has finished), so the warp
    // stages its 32 normalised rows there (16-byte chunks XOR-swizzled by row: conflict-free) and writes them back
    // transposed, 4 rows x 128 contiguous bytes per instruction.  The buffer goes back to the loader only when the
    // issuer AND all eight softmax warps have released it (q_empty counts nine arrivals).
    const int qbuf = (int)(n_item & 1);
    if (ok && n > 0) {
      const bool landed = mbar_wait(&o_done[t], (done - 1) & 1, err, 7);
      if (!__all_sync(0xffffffffu, landed)) {
        ok = false;
      } else {
        tc_fence_after();
        const float inv = 1.0f / l_run;   // a fully masked row (l = 0) yields NaN, as the unfused path does
        unsigned char* stage = sQ + (qbuf * QT + t) * Q_BYTES + quarter * 32 * 128;   // this warp's 32 rows x 128 bytes
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t orow[32];
          tmem_ld32(tmem_o + half * 32, orow);
          tmem_ld_wait();
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 v;
            v.x = pack2<T>(__uint_as_float(orow[8 * q]) * inv, __uint_as_float(orow[8 * q + 1]) * inv);
            v.y = pack2<T>(__uint_as_float(orow[8 * q + 2]) * inv, __uint_as_float(orow[8 * q + 3]) * inv);
            v.z = pack2<T>(__uint_as_float(orow[8 * q + 4]) * inv, __uint_as_float(orow[8 * q + 5]) * inv);
            v.w = pack2<T>(__uint_as_float(orow[8 * q + 6]) * inv, __uint_as_float(orow[8 * q + 7]) * inv);
            *reinterpret_cast<uint4*>(stage + lane * 128 + (((half * 4 + q) ^ (lane & 7)) << 4)) = v;
          }
        }
        __syncwarp();
        const int chunk = lane & 7;
#pragma unroll
        for (int pass = 0; pass < 8; ++pass) {
          const int rl = pass * 4 + (lane >> 3);              // row inside the warp's 32
          const int64_t qr = (int64_t)it.q0 + t * BQ + quarter * 32 + rl;
          const uint4 v = *reinterpret_cast<const uint4*>(stage + rl * 128 + ((chunk ^ (rl & 7)) << 4));
          if (qr < g.Sq)
            *reinterpret_cast<uint4*>(reinterpret_cast<T*>(g.o) + (int64_t)b * g.o_sb + (int64_t)h * g.o_sh + qr * g.o_ss + chunk * 8) = v;
        }
        fence_proxy_async_smem();   // the next writer of this buffer is a TMA load
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&q_empty[qbuf]);   // also for an idle tile and after a failed wait: the loader counts nine
    if (!ok) break;
    }   // items
  }

  // ---------------------------------------------------------------------- teardown ---
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *err != 0) *failed = 1;
  __syncthreads();
  if (*failed != 0) {
    // a wait gave up: let copies and MMAs still in flight settle before the tiles and TMEM go away
    const unsigned long long t0 = global_ns();
    while (global_ns() - t0 < 200000ull) {}
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, ATT_TMEM_COLS);
  }
  // the last CTA out zeroes the counters for the next launch (every CTA's draws from next_item precede its arrival here)
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(g.next_item + 1, 1) == (int)gridDim.x - 1) {
      g.next_item[0] = 0;
      g.next_item[1] = 0;
      __threadfence();
    }
  }
}

}  // namespace

bool attention_supported(const AttentionParams& p) {
  const bool is16 = p.dtype == B200_BFLOAT16 || p.dtype == B200_FLOAT16;
  if (!is16 || p.head_dim != HD) return false;
  if (p.B <= 0 || p.H <= 0 || p.Hkv <= 0 || p.Sq <= 0 || p.Sk <= 0 || p.H % p.Hkv != 0) return false;
  if (!(p.scale > 0) || !(p.scale < 1e30)) return false;   // the kernel takes the row maximum before scaling
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
  g.group = (int)(p.H / p.Hkv);
  g.causal = p.causal ? 1 : 0;
  g.is_f16 = f16 ? 1 : 0;
  g.scale_log2e = (float)(p.scale * 1.4426950408889634);
  g.err_flag = dev->kernel_error_flag();
  {
    void* ctr = nullptr;
    B200_CUDA_TRY(cudaGetSymbolAddress(&ctr, g_next_item));
    g.next_item = reinterpret_cast<int*>(ctr);
  }
  const int64_t nq = (p.Sq + QT * BQ - 1) / (QT * BQ);
  const int64_t items = nq * p.H * p.B;
  if (items >= 2147483648LL) return Status::Unsupported("attention: more than 2^31 work items");
  const int64_t resident = (int64_t)dev->sm_count() * 2;   // persistent: two CTAs per SM walk the work items
  const int64_t grid = items < resident ? items : resident;
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
    e = f16 ? launch_dependent(attention_kernel<__half>, (unsigned)grid, ATT_THREADS, ATT_SMEM, dev->stream(), tq, tk, tv, g)
            : launch_dependent(attention_kernel<__nv_bfloat16>, (unsigned)grid, ATT_THREADS, ATT_SMEM, dev->stream(), tq, tk, tv, g);
  }
  if (e != cudaSuccess) {
    cudaGetLastError();
    return Status::Cuda(strfmt("attention: %s", cudaGetErrorString(e)));
  }
  return dev->CheckLaunch("attention");
}

}  // namespace k
}  // namespace b200
