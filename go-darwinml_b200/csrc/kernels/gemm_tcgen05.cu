// DotGeneral's dense contraction on the 5th-generation tensor cores.
//
//   C[b, m, n] = act( sum_k A(b, m, k) * B(b, k, n) + bias[n] )     fp32 accumulation,
//   one rounding to the storage type in the epilogue (output dtype = input dtype,
//   as the reference's matmul does: mpsgraph dotgeneral.go:52, bridge.m:684-700).
//
// Both operands are read IN PLACE in either storage order:
//   A as [batch, M, K] ("K-major")  or [batch, K, M] ("MN-major"),
//   B as [batch, N, K] ("K-major")  or [batch, K, N] ("MN-major"),
// because the UMMA instruction descriptor carries a major bit per operand.  The
// reference materialises up to three transposes per DotGeneral instead
// (dotgeneral.go:110-142).
//
// Structure (one CTA per SM, persistent over output tiles of 128 x 256):
//   warp 0     producer: one lane issues TMA tile loads (128-byte swizzle) into a
//              4-stage shared-memory ring, signalling "full" mbarriers by byte count;
//   warp 1     issuer: one lane issues tcgen05.mma (M=128, N=256, K=16 per instruction)
//              from shared-memory descriptors into a TMEM accumulator; tcgen05.commit
//              releases ring stages ("empty") and publishes finished accumulators;
//   warps 2-17 epilogue: tcgen05.ld the accumulator (a warp reaches the 32 TMEM lanes of its quarter), add bias,
//              apply the activation, round, and hand the rows to a TMA tile store (16-bit results with aligned rows) or
//              write them out through a staging transpose as 16-byte vectors.  Sixteen warps of 64 columns each, in the
//              single-CTA kernel and in the CTA-pair kernel below: with short K the epilogue is the critical path.
// TMEM holds two 256-column accumulators, so the epilogue of tile i overlaps the
// main loop of tile i+1.  Tensor-core bound: flops = 2 * batch * M * N * K.
//
// fp32 operands use the same kernel through a 3-way bf16 split (see gemm_split3
// below): a = a1 + a2 + a3 with 8 significant bits each, six partial products
// accumulated in fp32 -- about fp32 accuracy at 1/6 of the bf16 rate.
//
// Every wait on an mbarrier is bounded (about two seconds of wall time); a wait
// that gives up raises a flag in global memory, every role leaves its loop, the
// TMEM allocation is released and the host reports B200_ERR_TIMEOUT.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdlib>
#include <mutex>

#include "../kernels.h"
#include "gemm_common.cuh"
#include "pdl.cuh"
#include "sm100_ptx.cuh"
#include "tma_host.h"

namespace b200 {
namespace k {

namespace {

using namespace sm100;

constexpr int BM = 128;        // tile rows  (UMMA M)
constexpr int BN = 256;        // tile cols  (UMMA N)
constexpr int BK = 64;         // K elements per stage = one 128-byte swizzle row of 16-bit elements
constexpr int UMMA_K = 16;     // K elements per tcgen05.mma for 16-bit types
constexpr int STAGES = 4;
constexpr int A_STAGE_BYTES = BM * BK * 2;  // 16 KiB
constexpr int B_STAGE_BYTES = BN * BK * 2;  // 32 KiB
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int TMEM_COLS = 512;
// sixteen epilogue warps, four per TMEM lane quarter (64 columns each)
constexpr int S_EPI_WARPS = 16;
constexpr int S_EPI_PITCH = 20;                      // words per scratch row: 16 + 4
// per warp: 32 rows x 16 words (2 KiB), the source box of a tile store {32 columns of 16 bits, 32 rows} with 64-byte
// swizzle; the write-out through registers uses the first 16 x 20 words of it
constexpr int S_EPI_STAGE_WORDS = 32 * 16;
constexpr int S_BAR_BYTES = 1024;   // barriers and the TMEM slot, padded so that the staging area stays 1024-byte aligned
constexpr int S_SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + S_BAR_BYTES + S_EPI_WARPS * S_EPI_STAGE_WORDS * 4;
static_assert(S_SMEM_BYTES <= 232448, "single-CTA GEMM: shared memory over the per-block limit");
constexpr int S_NUM_THREADS = 64 + 32 * S_EPI_WARPS;   // producer warp, issuer warp, epilogue warps

}  // namespace

namespace {

struct TcArgs {
  void* c;
  const void* bias;
  const void* residual;   // same shape as C, or null
  void* c_extra[GemmParams::kMaxExtraC];   // further copies of C (other ranks' buffers), same pitch
  int num_c_extra;
  int residual_mul;       // combine by * instead of +
  int64_t M, N, K, ldc;
  int batch;
  int a_kmajor, b_kmajor;
  int activation;
  int in_f16;       // operands are F16 (else BF16)
  int out_dtype;    // B200_BFLOAT16, B200_FLOAT16 or B200_FLOAT32
  int tiles_m, tiles_n;
  int64_t total_tiles;
  int k_blocks;     // ceil(K / BK)
  int segs;         // 1, or 6 partial products of the 3-way split
  // fp32 operands only: a tile's K range is cut into num_chunks chunks of chunk_blocks k-blocks.  Each chunk is accumulated
  // from zero in TMEM and the epilogue adds it to C in fp32 (round to nearest), so no TMEM accumulator ever holds more
  // than a short partial sum.  The tensor core's fp32 accumulate TRUNCATES (measured: on all-positive data the error of a
  // K = 8192 product is one-sided and 35 times the tolerance of 1e-5 of the result's RMS; on N(0,1) data 4.8 times),
  // and that bias grows with the number of accumulations times the magnitude of the running sum; chunks of 512 keep it
  // below 0.3 of the tolerance at every K (better than a plain fp32 FFMA GEMM, which is at 1.8 at K = 8192).
  int num_chunks, chunk_blocks;
  int vec_store;    // rows of C start 16-byte aligned and N is a multiple of the vector width
  // Ragged rows (16-bit C, dense, N not a multiple of 8, M a multiple of 8): row r of C starts (r * N) mod 8 elements off
  // the 16-byte grid, the same for every row of one residue class r mod 8.  The problem is cut into 8 classes; a class's
  // tiles take every 8th row of A (a 4-D map) and a column window shifted left by the class's offset, so every vector of
  // a tile is aligned in memory and only the first and last vector of a ROW are partial (written element by element).
  // m-tile index = 8 * (tile within the class) + class.  rag_q = N mod 8.
  int rag, rag_q;
  // single-CTA kernel, 16-bit C with aligned rows: the epilogue hands its staged rows to a tile store (tm_c) instead of
  // reading them back and storing from registers
  int tma_store;
  int* err_flag;
};

// Where a tile's rows live in C.  Plain: batch b, pitch ldc.  Ragged rows: class `kres` of batch b, pitch 8 N, base moved
// left by the class's shift so that the tile's column j is element j of a 16-byte aligned row image.
template <typename OutT>
struct CView {
  OutT* base;
  int64_t ld, rows, col_lo, col_hi;   // valid tile columns are [col_lo, col_hi)
};
template <typename OutT>
__device__ __forceinline__ CView<OutT> c_view(const TcArgs& g, int b, int kres) {
  CView<OutT> v;
  if (g.rag) {
    const int64_t shift = (kres * g.rag_q) & 7;
    v.base = reinterpret_cast<OutT*>(g.c) + ((int64_t)b * g.M + kres) * g.N - shift;
    v.ld = 8 * g.N;
    v.rows = g.M >> 3;
    v.col_lo = shift;
    v.col_hi = g.N + shift;
  } else {
    v.base = reinterpret_cast<OutT*>(g.c) + (int64_t)b * g.M * g.ldc;
    v.ld = g.ldc;
    v.rows = g.M;
    v.col_lo = 0;
    v.col_hi = g.N;
  }
  return v;
}

// The valid elements of a 16-byte vector that straddles the start or the end of a ragged row, as 2-byte stores.
template <typename OutT>
__device__ __forceinline__ void store_partial_vector(OutT* dst, uint4 q, int64_t col, int64_t col_lo, int64_t col_hi) {
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
  uint16_t* d16 = reinterpret_cast<uint16_t*>(dst);
#pragma unroll
  for (int e = 0; e < 8; ++e)
    if (col + e >= col_lo && col + e < col_hi) d16[e] = (uint16_t)(w[e >> 1] >> (16 * (e & 1)));
}

// plane of A / B used by each of the six partial products of the 3-way split,
// smallest terms first: a1*b3, a3*b1, a2*b2, a1*b2, a2*b1, a1*b1
__constant__ int kPlaneA[6] = {0, 2, 1, 0, 1, 0};
__constant__ int kPlaneB[6] = {2, 0, 1, 1, 0, 0};

// Runs once per tile in the producer thread and in every epilogue warp (a few hundred dependent instructions with
// 64-bit divisions): 32-bit unsigned arithmetic, three divisions, the remainders by multiply-subtract.  The launcher
// refuses tile counts of 2^31 and more.
__device__ __forceinline__ void tile_coords(const TcArgs& g, int64_t t64, int* b, int* m_t, int* n_t) {
  constexpr uint32_t GROUP = 16;  // m-tiles per super-row: CTAs running together share A and B panels in L2
  const uint32_t t = (uint32_t)t64;
  const uint32_t tiles_m = (uint32_t)g.tiles_m, tiles_n = (uint32_t)g.tiles_n;
  const uint32_t per_batch = tiles_m * tiles_n;
  const uint32_t bi = t / per_batch;
  const uint32_t r = t - bi * per_batch;
  const uint32_t group_size = GROUP * tiles_n;
  const uint32_t gidx = r / group_size;
  const uint32_t in_group = r - gidx * group_size;
  const uint32_t first_m = gidx * GROUP;
  const uint32_t gm = (tiles_m - first_m) < GROUP ? (tiles_m - first_m) : GROUP;
  const uint32_t ni = in_group / gm;
  *b = (int)bi;
  *m_t = (int)(first_m + in_group - ni * gm);
  *n_t = (int)ni;
}

template <typename OutT> __device__ __forceinline__ float load_bias(const void* bias, int64_t col) {
  return 0.f;
}
template <> __device__ __forceinline__ float load_bias<float>(const void* bias, int64_t col) { return reinterpret_cast<const float*>(bias)[col]; }
template <> __device__ __forceinline__ float load_bias<__nv_bfloat16>(const void* bias, int64_t col) {
  return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(bias)[col]);
}
template <> __device__ __forceinline__ float load_bias<__half>(const void* bias, int64_t col) {
  return __half2float(reinterpret_cast<const __half*>(bias)[col]);
}

template <typename OutT> struct OutTraits;
template <> struct OutTraits<float> { static constexpr int kColsPerWord = 1; static constexpr bool kFast = false; };
template <> struct OutTraits<__nv_bfloat16> { static constexpr int kColsPerWord = 2; static constexpr bool kFast = true; };
template <> struct OutTraits<__half> { static constexpr int kColsPerWord = 2; static constexpr bool kFast = true; };

template <typename OutT> __device__ __forceinline__ uint32_t pack_word(float a, float b);
template <> __device__ __forceinline__ uint32_t pack_word<float>(float a, float) { return __float_as_uint(a); }
template <> __device__ __forceinline__ uint32_t pack_word<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <> __device__ __forceinline__ uint32_t pack_word<__half>(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

// word (one fp32 or two 16-bit values, already rounded) combined with the residual word (+ or *), rounded again
template <typename OutT> __device__ __forceinline__ uint32_t add_residual_word(uint32_t w, uint32_t r, int mul);
template <> __device__ __forceinline__ uint32_t add_residual_word<float>(uint32_t w, uint32_t r, int mul) {
  return __float_as_uint(mul ? __uint_as_float(w) * __uint_as_float(r) : __uint_as_float(w) + __uint_as_float(r));
}
template <> __device__ __forceinline__ uint32_t add_residual_word<__nv_bfloat16>(uint32_t w, uint32_t r, int mul) {
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r));
  return mul ? pack_word<__nv_bfloat16>(a.x * b.x, a.y * b.y) : pack_word<__nv_bfloat16>(a.x + b.x, a.y + b.y);
}
template <> __device__ __forceinline__ uint32_t add_residual_word<__half>(uint32_t w, uint32_t r, int mul) {
  const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&w));
  const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&r));
  return mul ? pack_word<__half>(a.x * b.x, a.y * b.y) : pack_word<__half>(a.x + b.x, a.y + b.y);
}

// NC consecutive bias values starting at col (col is a multiple of NC; col + NC <= N is NOT assumed: tail guarded).
template <typename OutT, int NC>
__device__ __forceinline__ void add_bias_n(const TcArgs& g, int64_t col, float* v) {
  if (g.vec_store && col + NC <= g.N) {
    // 16-byte loads; every lane reads the same addresses (one broadcast transaction each)
    const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const OutT*>(g.bias) + col);
    constexpr int kPerVec = 16 / (int)sizeof(OutT);
#pragma unroll
    for (int q = 0; q < NC / kPerVec; ++q) {
      const uint4 w = __ldg(src + q);
      const OutT* e = reinterpret_cast<const OutT*>(&w);
#pragma unroll
      for (int i = 0; i < kPerVec; ++i) v[q * kPerVec + i] += (float)e[i];
    }
  } else {
#pragma unroll
    for (int j = 0; j < NC; ++j)
      if (col + j < g.N) v[j] += load_bias<OutT>(g.bias, col + j);
  }
}
template <typename OutT>
__device__ __forceinline__ void add_bias32(const TcArgs& g, int64_t col, float* v) { add_bias_n<OutT, 32>(g, col, v); }

// 16 bytes of C read back through the coherent path (never ld.global.nc: the line was written by this kernel)
__device__ __forceinline__ uint4 ld_c16(const void* p) {
  uint4 q;
  asm volatile("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(q.x), "=r"(q.y), "=r"(q.z), "=r"(q.w) : "l"(p) : "memory");
  return q;
}

// fp32 chunked accumulation, applied to one word of the write-out: adds the value C already holds (chunks after the
// first), and on a tile's last chunk does what the plain epilogue did before staging: bias, activation, residual.
__device__ __forceinline__ uint32_t combine_chunk_word(const TcArgs& g, uint32_t acc, uint32_t c_old, bool first, bool last, int64_t col,
                                                       const float* residual_elem) {
  float v = __uint_as_float(acc);
  if (!first) v += __uint_as_float(c_old);
  if (last) {
    if (g.bias) v += reinterpret_cast<const float*>(g.bias)[col];
    float one[1] = {v};
    apply_activation_n<1, false>(g.activation, one);
    v = one[0];
    if (residual_elem) v = g.residual_mul ? v * *residual_elem : v + *residual_elem;
  }
  return __float_as_uint(v);
}

// The epilogue of both kernels.  With short K a tile's main loop is no longer than its epilogue, and the epilogue is a
// chain of dependent instructions (TMEM read, rounding, staging, write-out) that a scheduler with two warps cannot keep
// issuing: SIXTEEN warps share a CTA's 128 x 256 accumulator, four per TMEM lane quarter, 64 columns each, in sub-steps
// of 16 words per row (32 16-bit columns or 16 fp32 columns) so that a thread stays under 112 registers.
// A thread holds one ROW of the accumulator, so storing from registers would scatter every store instruction over 32
// rows (32 cache lines).  16-bit results with aligned rows go to a 32 x 64-byte staging box per warp and from there to C
// as one TMA tile store per sub-step (measured on M = 16384, N = 3072: the epilogue alone, K = 64, 54 -> 32 us; a warp's
// drain of a tile 7100 -> 2800 cycles).  Everything else (fp32 and its chunked accumulation, ragged rows, extra
// destinations) is staged 16 rows x 16 words at a time (20-word pitch) and written back transposed, 8 rows x 64
// contiguous bytes per store instruction.
template <typename OutT>
__device__ __forceinline__ void drain_accumulator_narrow(const TcArgs& g, const CUtensorMap* tm_c, const CUtensorMap* tm_r, uint64_t* rbar,
                                                         uint32_t& rphase, uint32_t tmem_acc, int64_t row0, int64_t n0, int b, int kres,
                                                         int quarter, int cq, int lane, uint32_t* stage, int chunk) {
  using Tr = OutTraits<OutT>;
  constexpr int CPW = Tr::kColsPerWord;
  constexpr int SUB_COLS = 16 * CPW;            // columns per sub-step: 16 words per row
  constexpr int WARP_COLS = BN / 4;             // columns per warp
  constexpr int SUBS = WARP_COLS / SUB_COLS;
  const uint32_t taddr = tmem_acc + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(cq * WARP_COLS);
  const int64_t row_base = row0 + quarter * 32;
  const CView<OutT> cv = c_view<OutT>(g, b, kres);
  const int64_t ld = cv.ld, col_hi = cv.col_hi;
  OutT* cbase = cv.base + row_base * ld;
  const OutT* rbase = g.residual ? reinterpret_cast<const OutT*>(g.residual) + ((int64_t)b * g.M + row_base) * g.ldc : nullptr;   // never with ragged rows
  const bool chunked = CPW == 1 && g.num_chunks > 1;   // fp32 chunked accumulation, as in drain_accumulator
  const bool first_chunk = chunk == 0, last_chunk = chunk == g.num_chunks - 1;
  const int wg = (lane & 3) * 4;                // write-out: this lane's 4 words of a 16-word row
  const int rsub = lane >> 2;                   // write-out: row within a pass of 8 rows
  // per-store work is kept to a pointer increment and a 32-bit compare: the epilogue is bound by instruction issue
  const int rows_left = (int)((cv.rows - row_base) < 32 ? (cv.rows - row_base) : 32);
  const int64_t pass_stride = 8 * ld;
#pragma unroll 1
  for (int sub = 0; sub < SUBS; ++sub) {
    const int64_t col0 = n0 + cq * WARP_COLS + sub * SUB_COLS;
    if (col0 >= col_hi) break;  // uniform across the warp
    const int64_t col = col0 + (int64_t)wg * CPW;
    // the residual block of this sub-step, fetched first in the write-out layout (latency hides under the TMEM read)
    const bool col_ok = col < col_hi;
    const int64_t first = (int64_t)rsub * ld + col;   // element offset of this lane's vector in pass 0
    const bool partial = CPW == 2 && g.rag && (col < cv.col_lo || col + 8 > col_hi);   // the vector straddles an end of a ragged row
    uint4 rv[4];
    if (CPW == 2 && g.tma_store) {
      // The residual's 32 x 64-byte block of this sub-step comes into the warp's staging box by a tile load (a thread
      // owns a row, so loads from registers would touch 32 lines per instruction), under the TMEM read and the
      // arithmetic below; the box is free once the previous tile store has read it.
      if (rbase && lane == 0) {
        bulk_wait_read_all();
        mbar_expect_tx(rbar, 32 * 64);
        tma_load_4d(stage, tm_r, rbar, (int)col0, (int)row_base, b, 0);
      }
    } else if (chunked) {
      if (!first_chunk && g.vec_store) {
#pragma unroll
        for (int pass = 0; pass < 4; ++pass)
          rv[pass] = (col_ok && pass * 8 + rsub < rows_left) ? ld_c16(cbase + first + pass * pass_stride)
                                                             : make_uint4(0, 0, 0, 0);
      }
    } else if (rbase && g.vec_store) {
#pragma unroll
      for (int pass = 0; pass < 4; ++pass)
        rv[pass] = (col_ok && pass * 8 + rsub < rows_left) ? __ldg(reinterpret_cast<const uint4*>(rbase + first + pass * pass_stride))
                                                           : make_uint4(0, 0, 0, 0);
    }
    uint32_t words[16];
    {
      uint32_t r[SUB_COLS];
      if constexpr (CPW == 2) tmem_ld32(taddr + sub * SUB_COLS, r);
      else tmem_ld16(taddr + sub * SUB_COLS, r);
      tmem_ld_wait();
      float v[SUB_COLS];
#pragma unroll
      for (int j = 0; j < SUB_COLS; ++j) v[j] = __uint_as_float(r[j]);
      if (!chunked) {
        if (g.bias) add_bias_n<OutT, SUB_COLS>(g, col0, v);
        apply_activation_n<SUB_COLS, Tr::kFast>(g.activation, v);
      }
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        if constexpr (CPW == 2) words[j] = pack_word<OutT>(v[2 * j], v[2 * j + 1]);
        else words[j] = pack_word<OutT>(v[j], 0.f);
      }
    }
    if (CPW == 2 && g.tma_store) {
      // The warp's 32 rows x 64 bytes go to its staging box and from there to C as ONE tile store, issued by lane 0:
      // nothing is read back, no store instruction or address arithmetic per row, and rows / columns past the edge of
      // C are clipped by the copy.  64-byte swizzle: the 16-byte chunk j of row r sits at chunk j ^ ((r >> 1) & 3), so the
      // eight rows a store instruction's quarter-warp covers fall in eight different bank groups.
      uint32_t* srow = stage + lane * 16;
      const int sw = (lane >> 1) & 3;
      if (rbase) {
        mbar_wait(rbar, rphase, g.err_flag, 8);   // the residual block has landed (a wait that gives up raises the error word)
        rphase ^= 1;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint4 rq = *reinterpret_cast<const uint4*>(srow + ((j ^ sw) << 2));
          words[4 * j] = add_residual_word<OutT>(words[4 * j], rq.x, g.residual_mul);
          words[4 * j + 1] = add_residual_word<OutT>(words[4 * j + 1], rq.y, g.residual_mul);
          words[4 * j + 2] = add_residual_word<OutT>(words[4 * j + 2], rq.z, g.residual_mul);
          words[4 * j + 3] = add_residual_word<OutT>(words[4 * j + 3], rq.w, g.residual_mul);
        }
      } else {
        if (lane == 0) bulk_wait_read_all();   // the previous store has finished reading the box
        __syncwarp();
      }
#pragma unroll
      for (int j = 0; j < 4; ++j)
        *reinterpret_cast<uint4*>(srow + ((j ^ sw) << 2)) = make_uint4(words[4 * j], words[4 * j + 1], words[4 * j + 2], words[4 * j + 3]);
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        tma_store_4d(tm_c, stage, (int)col0, (int)row_base, b, 0);
        bulk_commit_group();
      }
      continue;
    }
#pragma unroll
    for (int round = 0; round < 2; ++round) {
      if ((lane >> 4) == round) {
#pragma unroll
        for (int j = 0; j < 16; j += 4)
          *reinterpret_cast<uint4*>(stage + (lane & 15) * S_EPI_PITCH + j) = make_uint4(words[j], words[j + 1], words[j + 2], words[j + 3]);
      }
      __syncwarp();
      if (g.vec_store) {
#pragma unroll
        for (int pass = 0; pass < 2; ++pass) {
          const int rl = pass * 8 + rsub;
          const int rr = round * 16 + rl;
          uint4 q = *reinterpret_cast<const uint4*>(stage + rl * S_EPI_PITCH + wg);
          if (col_ok && rr < rows_left) {
            if (chunked) {
              const uint4 rq = first_chunk ? make_uint4(0, 0, 0, 0) : rv[round * 2 + pass];
              const float* re = (last_chunk && rbase) ? reinterpret_cast<const float*>(rbase) + first + (round * 2 + pass) * pass_stride : nullptr;
              q.x = combine_chunk_word(g, q.x, rq.x, first_chunk, last_chunk, col, re);
              q.y = combine_chunk_word(g, q.y, rq.y, first_chunk, last_chunk, col + 1, re ? re + 1 : nullptr);
              q.z = combine_chunk_word(g, q.z, rq.z, first_chunk, last_chunk, col + 2, re ? re + 2 : nullptr);
              q.w = combine_chunk_word(g, q.w, rq.w, first_chunk, last_chunk, col + 3, re ? re + 3 : nullptr);
            } else if (rbase) {
              const uint4 rq = rv[round * 2 + pass];
              q.x = add_residual_word<OutT>(q.x, rq.x, g.residual_mul);
              q.y = add_residual_word<OutT>(q.y, rq.y, g.residual_mul);
              q.z = add_residual_word<OutT>(q.z, rq.z, g.residual_mul);
              q.w = add_residual_word<OutT>(q.w, rq.w, g.residual_mul);
            }
            const int64_t off = first + (round * 2 + pass) * pass_stride;
            if (partial) store_partial_vector<OutT>(cbase + off, q, col, cv.col_lo, col_hi);
            else *reinterpret_cast<uint4*>(cbase + off) = q;
            if (g.num_c_extra > 0) {
              // the same vector to every other rank's copy: plain stores to peer-mapped memory (NVLink)
              for (int x = 0; x < g.num_c_extra; ++x)
                *reinterpret_cast<uint4*>(reinterpret_cast<OutT*>(g.c_extra[x]) + ((int64_t)b * g.M + row_base) * g.ldc + off) = q;
            }
          }
        }
      } else {
        // Rows of C do not start 16-byte aligned: 4 bytes per lane, two rows per store instruction (lanes 0-15 one row,
        // lanes 16-31 the next).  A 16-bit row that starts on an odd element is 2 bytes off the word grid: its words are
        // re-cut from neighbouring staged words (funnel shift) and the two end elements go out as 2-byte stores.
        const int l16 = lane & 15;
#pragma unroll 2
        for (int it = 0; it < 8; ++it) {
          const int rl = it * 2 + (lane >> 4);
          const int rr = round * 16 + rl;
          if (row_base + rr >= g.M) continue;
          OutT* crow = cbase + (int64_t)rr * g.ldc;
          const OutT* rrow = rbase ? rbase + (int64_t)rr * g.ldc : nullptr;
          if constexpr (CPW == 1) {
            const int64_t c1 = col0 + l16;
            if (c1 < g.N) {
              uint32_t w = stage[rl * S_EPI_PITCH + l16];
              if (chunked) {
                const uint32_t c_old = first_chunk ? 0u : reinterpret_cast<const volatile uint32_t*>(crow)[c1];
                w = combine_chunk_word(g, w, c_old, first_chunk, last_chunk, c1, (last_chunk && rbase) ? reinterpret_cast<const float*>(rrow) + c1 : nullptr);
              } else if (rbase) w = add_residual_word<OutT>(w, reinterpret_cast<const uint32_t*>(rrow)[c1], g.residual_mul);
              reinterpret_cast<uint32_t*>(crow)[c1] = w;
            }
          } else {
            const uint32_t odd = (uint32_t)((((int64_t)b * g.M + row_base + rr) * g.ldc + col0) & 1);
            const uint32_t w0 = stage[rl * S_EPI_PITCH + l16];
            const uint32_t w1 = stage[rl * S_EPI_PITCH + l16 + 1];  // lane 15 reads a pad word: unused
            uint32_t w = odd ? __funnelshift_r(w0, w1, 16) : w0;    // elements (2 l16 + odd, 2 l16 + odd + 1)
            const int64_t c1 = col0 + 2 * l16 + odd;
            uint16_t* c16 = reinterpret_cast<uint16_t*>(crow);
            const uint16_t* r16 = reinterpret_cast<const uint16_t*>(rrow);
            const bool pair_ok = c1 + 1 < g.N && !(odd && l16 == 15);
            if (pair_ok) {
              if (rbase) w = add_residual_word<OutT>(w, (uint32_t)r16[c1] | ((uint32_t)r16[c1 + 1] << 16), g.residual_mul);
              *reinterpret_cast<uint32_t*>(c16 + c1) = w;   // (row start + 2 l16 + odd) is even: 4-byte aligned
            } else if (c1 < g.N) {
              uint32_t lo = w & 0xffffu;                    // the last column of the row, or element 31 of an odd row
              if (rbase) lo = add_residual_word<OutT>(lo, r16[c1], g.residual_mul) & 0xffffu;
              c16[c1] = (uint16_t)lo;
            }
            if (odd && l16 == 0 && col0 < g.N) {           // element 0 of an odd row
              uint32_t lo = w0 & 0xffffu;
              if (rbase) lo = add_residual_word<OutT>(lo, r16[col0], g.residual_mul) & 0xffffu;
              c16[col0] = (uint16_t)lo;
            }
          }
        }
      }
      __syncwarp();
    }
  }
}

template <typename OutT>
__global__ void __launch_bounds__(S_NUM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b, const __grid_constant__ CUtensorMap tm_c,
                    const __grid_constant__ CUtensorMap tm_r, const TcArgs g) {
  extern __shared__ unsigned char smem_raw[];
  // operand tiles need 1024-byte alignment for the 128-byte swizzle
  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + STAGES * STAGE_BYTES);
  uint64_t* full = bars;                    // [STAGES]  TMA bytes landed
  uint64_t* empty = bars + STAGES;          // [STAGES]  MMAs that read the stage are done
  uint64_t* acc_full = bars + 2 * STAGES;   // [2]       accumulator complete
  uint64_t* acc_empty = bars + 2 * STAGES + 2;  // [2]   accumulator drained by the epilogue
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  uint64_t* res_bar = bars + 32;            // [S_EPI_WARPS] an epilogue warp's residual block has landed
  uint32_t* epi_stage = reinterpret_cast<uint32_t*>(tiles + STAGES * STAGE_BYTES + S_BAR_BYTES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* err = g.err_flag;
  // only fp32 results cut the K range into chunks; for 16-bit results these fold to constants and the chunk loops vanish
  const int NCH = sizeof(OutT) == 4 ? g.num_chunks : 1;
  const int CHB = sizeof(OutT) == 4 ? g.chunk_blocks : g.k_blocks;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], S_EPI_WARPS); }
    for (int w = 0; w < S_EPI_WARPS; ++w) mbar_init(&res_bar[w], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // everything above ran under the tail of the kernel before this one (when launched as its programmatic dependent);
  // from here on its results are read and its operands' memory may be overwritten
  pdl_launch_dependents();
  pdl_wait();

  if (warp == 0) {
    // ------------------------------------------------------------------ producer ---
    if (lane == 0) {
      // one thread, about 500 cycles per stage: no divisions in the loop, (seg, kb) advance by increments
      int s = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int64_t t = blockIdx.x; t < g.total_tiles && ok; t += gridDim.x) {
        int b, m_t, n_t;
        tile_coords(g, t, &b, &m_t, &n_t);
        int kres = 0, shift = 0;
        if (g.rag) { kres = m_t & 7; m_t >>= 3; shift = (kres * g.rag_q) & 7; }
        const int m0 = m_t * BM, n0 = n_t * BN - shift;   // ragged rows: the class's column window starts `shift` columns early
        // coordinates 3 and 4 of A: (batch, plane), or with ragged rows (row class, batch)
        const int a3 = g.rag ? kres : b, a4_rag = b;
        for (int chunk = 0; chunk < NCH && ok; ++chunk) {
        const int kb_begin = chunk * CHB;
        const int kb_end = kb_begin + CHB < g.k_blocks ? kb_begin + CHB : g.k_blocks;
        for (int seg = 0; seg < g.segs && ok; ++seg) {
          const int pa = g.segs > 1 ? kPlaneA[seg] : 0, pb = g.segs > 1 ? kPlaneB[seg] : 0;
          for (int kb = kb_begin; kb < kb_end; ++kb) {
            if (!mbar_wait(&empty[s], phase ^ 1, err, 1)) { ok = false; break; }
            unsigned char* sa = tiles + s * STAGE_BYTES;
            unsigned char* sb = sa + A_STAGE_BYTES;
            const int k0 = kb * BK;
            mbar_expect_tx(&full[s], STAGE_BYTES);
            if (g.a_kmajor) {
              // box {64 k, 128 m}: 128 rows of 128 bytes
              tma_load_4d(sa, &tm_a, &full[s], k0, m0, a3, g.rag ? a4_rag : pa);
            } else {
              // two boxes {64 m, 64 k}: 64 k-rows of 128 bytes each, one box per 64-wide block of M
              tma_load_4d(sa, &tm_a, &full[s], m0, k0, b, pa);
              tma_load_4d(sa + 8192, &tm_a, &full[s], m0 + 64, k0, b, pa);
            }
            if (g.b_kmajor) {
              tma_load_4d(sb, &tm_b, &full[s], k0, n0, b, pb);
            } else {
#pragma unroll
              for (int j = 0; j < 4; ++j) tma_load_4d(sb + j * 8192, &tm_b, &full[s], n0 + j * 64, k0, b, pb);
            }
            if (++s == STAGES) { s = 0; phase ^= 1; }
          }
        }
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------------- issuer ---
    if (lane == 0) {
      // instruction descriptor: fp32 accumulate, operand format, majors, N and M
      uint32_t idesc = 0;
      idesc |= 1u << 4;                                  // D format: F32
      idesc |= (g.in_f16 ? 0u : 1u) << 7;                // A format: F16 = 0, BF16 = 1
      idesc |= (g.in_f16 ? 0u : 1u) << 10;               // B format
      idesc |= (g.a_kmajor ? 0u : 1u) << 15;             // A major: 0 = K, 1 = MN
      idesc |= (g.b_kmajor ? 0u : 1u) << 16;             // B major
      idesc |= (uint32_t)(BN >> 3) << 17;
      idesc |= (uint32_t)(BM >> 4) << 24;
      // K-major tile: rows of 128 bytes, 8-row groups 1024 bytes apart; 16 k-elements = 32 bytes along the row.
      // MN-major tile: 64-wide blocks 8192 bytes apart (LBO), 8-k-row groups 1024 bytes apart (SBO); 16 k = 2 groups.
      const uint32_t a_lbo = g.a_kmajor ? 16u : 8192u, b_lbo = g.b_kmajor ? 16u : 8192u;
      const uint32_t a_kstep = g.a_kmajor ? 32u : 2048u, b_kstep = g.b_kmajor ? 32u : 2048u;
      // per stage the descriptors differ only in the 14-bit address field (shared memory is below 256 KiB: no carry)
      const uint64_t da0 = make_smem_desc(smem_u32(tiles), a_lbo, 1024), db0 = make_smem_desc(smem_u32(tiles) + A_STAGE_BYTES, b_lbo, 1024);
      int s = 0;
      uint32_t phase = 0;
      bool ok = true;
      // one work item = one chunk of one tile (a whole tile when the K range is not cut): items alternate between the
      // two accumulators
      int local_tile = 0;
      for (int64_t t = blockIdx.x; t < g.total_tiles && ok; t += gridDim.x)
      for (int chunk = 0; chunk < NCH && ok; ++chunk, ++local_tile) {
        const int acc = local_tile & 1;
        const uint32_t acc_phase = (local_tile >> 1) & 1;
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1, err, 2)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        const int kb_begin = chunk * CHB;
        const int kb_end = kb_begin + CHB < g.k_blocks ? kb_begin + CHB : g.k_blocks;
        const int iters = (kb_end - kb_begin) * g.segs;
        for (int it = 0; it < iters; ++it) {
          if (!mbar_wait(&full[s], phase, err, 3)) { ok = false; break; }
          tc_fence_after();
          const uint64_t da_s = da0 + (uint64_t)((s * STAGE_BYTES) >> 4), db_s = db0 + (uint64_t)((s * STAGE_BYTES) >> 4);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_f16(d_tmem, da_s + (uint64_t)((k * a_kstep) >> 4), db_s + (uint64_t)((k * b_kstep) >> 4), idesc, (it | k) != 0 ? 1u : 0u);
          tc_commit(&empty[s]);  // frees the stage once these MMAs have read it
          if (++s == STAGES) { s = 0; phase ^= 1; }
        }
        if (ok) tc_commit(&acc_full[acc]);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue ---
    const int quarter = warp & 3;              // TMEM lanes [32*quarter, 32*quarter + 32) belong to this warp
    bool ok = true;
    int local_tile = 0;
    uint32_t rphase = 0;
    for (int64_t t = blockIdx.x; t < g.total_tiles && ok; t += gridDim.x) {
      int b, m_t, n_t;
      tile_coords(g, t, &b, &m_t, &n_t);
      int kres = 0;
      if (g.rag) { kres = m_t & 7; m_t >>= 3; }
      for (int chunk = 0; chunk < NCH && ok; ++chunk, ++local_tile) {
      const int acc = local_tile & 1;
      const uint32_t acc_phase = (local_tile >> 1) & 1;
      const bool landed = mbar_wait(&acc_full[acc], acc_phase, err, 4);
      if (!__all_sync(0xffffffffu, landed)) { ok = false; break; }  // the warp leaves together: tcgen05.ld is warp-collective
      tc_fence_after();
      drain_accumulator_narrow<OutT>(g, &tm_c, &tm_r, &res_bar[warp - 2], rphase, tmem_base + acc * BN, (int64_t)m_t * BM, (int64_t)n_t * BN, b, kres, quarter, (warp - 2) >> 2, lane,
                                     epi_stage + (warp - 2) * S_EPI_STAGE_WORDS, chunk);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[acc]);
      }
    }
    if (g.tma_store && lane == 0) bulk_wait_all();   // this warp's tile stores are done before its staging memory goes away
  }

  // ---------------------------------------------------------------------- teardown ---
  tc_fence_before();
  __shared__ int failed;
  if (threadIdx.x == 0) failed = *err;
  __syncthreads();
  if (failed != 0) {
    // a wait gave up: let copies and MMAs still in flight settle before the tiles and TMEM go away
    const unsigned long long t0 = global_ns();
    while (global_ns() - t0 < 200000ull) {}
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------------------------------------------------------
// CTA-pair variant: two CTAs of a cluster (neighbouring SMs) compute one 256 x 256 tile with tcgen05.mma
// cta_group::2.  Each CTA loads its 128 rows of A and HALF of the tile's B columns (128), so a CTA pulls 32 KiB per
// 64-deep K block from L2 instead of 48 KiB; its TMEM holds the 128 x 256 accumulator of its own rows.  The CTA of
// even rank (the leader) issues every MMA.  Barriers:
//   full[s]      leader only; counts the bytes of BOTH CTAs' tile loads (the peer's loads name it by cluster address)
//   empty[s]     one per CTA; the leader commits to both once the MMAs that read stage s are done
//   acc_full[a]  one per CTA; the leader commits to both when a tile's accumulator is complete
//   acc_empty[a] leader only; the 8 + 8 epilogue warps of both CTAs arrive when they have drained it
// The pair joins at a cluster barrier before either releases TMEM or exits, so no CTA's shared memory or barriers
// are touched after it has gone.
constexpr int P_STAGES = 6;
constexpr int P_BN_HALF = BN / 2;                         // B columns held per CTA
constexpr int P_B_STAGE_BYTES = P_BN_HALF * BK * 2;       // 16 KiB
constexpr int P_STAGE_BYTES = A_STAGE_BYTES + P_B_STAGE_BYTES;  // 32 KiB
constexpr int P_SMEM_BYTES = P_STAGES * P_STAGE_BYTES + 1024 + S_BAR_BYTES + S_EPI_WARPS * S_EPI_STAGE_WORDS * 4;
static_assert(P_SMEM_BYTES <= 232448, "CTA-pair GEMM: shared memory over the per-block limit");

__device__ __forceinline__ void pair_tile_coords(const TcArgs& g, int64_t t, int* b, int* m_t, int* n_t) {
  // same grouping as tile_coords over tiles of 256 rows: g.tiles_m counts 256-row tiles here
  tile_coords(g, t, b, m_t, n_t);
}

template <typename OutT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(S_NUM_THREADS, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b, const __grid_constant__ CUtensorMap tm_c,
                         const __grid_constant__ CUtensorMap tm_r, const TcArgs g) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + P_STAGES * P_STAGE_BYTES);
  uint64_t* full = bars;                          // [P_STAGES]
  uint64_t* empty = bars + P_STAGES;              // [P_STAGES]
  uint64_t* acc_full = bars + 2 * P_STAGES;       // [2]
  uint64_t* acc_empty = bars + 2 * P_STAGES + 2;  // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * P_STAGES + 4);
  uint64_t* res_bar = bars + 32;                  // [S_EPI_WARPS] an epilogue warp's residual block has landed
  uint32_t* epi_stage = reinterpret_cast<uint32_t*>(tiles + P_STAGES * P_STAGE_BYTES + S_BAR_BYTES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int64_t pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  volatile int* err = g.err_flag;
  // only fp32 results cut the K range into chunks; for 16-bit results these fold to constants and the chunk loops vanish
  const int NCH = sizeof(OutT) == 4 ? g.num_chunks : 1;
  const int CHB = sizeof(OutT) == 4 ? g.chunk_blocks : g.k_blocks;

  if (threadIdx.x == 0) {
    for (int s = 0; s < P_STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], 2 * S_EPI_WARPS); }
    for (int w = 0; w < S_EPI_WARPS; ++w) mbar_init(&res_bar[w], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before either signals the other's
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // everything above ran under the tail of the kernel before this one (when launched as its programmatic dependent);
  // from here on its results are read and its operands' memory may be overwritten
  pdl_launch_dependents();
  pdl_wait();

  if (warp == 0) {
    // ------------------------------------------------------------------ producer ---
    if (lane == 0) {
      // A single thread runs this loop and every stage has about 500 cycles, so it carries no divisions: the cursor
      // (tile, seg, kb) advances by increments.  (Measured: with a division per k-block the loop itself cost 10 % of
      // the kernel's throughput; asking L2 to prefetch tiles ahead of the ring halved it, the requests compete with the loads.)
      struct Cursor {
        int64_t t;        // global tile index
        int b, m0, n0;    // this CTA's rows of A / columns of B in that tile
        int kres;         // ragged rows: the tile's row class
        int seg, kb;
        int chunk, kb_end;   // the chunk of the tile's K range being loaded and its last k-block + 1
      };
      auto place = [&](Cursor& c) {
        int m_t, n_t;
        pair_tile_coords(g, c.t, &c.b, &m_t, &n_t);
        int shift = 0;
        c.kres = 0;
        if (g.rag) { c.kres = m_t & 7; m_t >>= 3; shift = (c.kres * g.rag_q) & 7; }
        c.m0 = m_t * 2 * BM + (int)rank * BM;
        c.n0 = n_t * BN + (int)rank * P_BN_HALF - shift;
      };
      auto chunk_range = [&](Cursor& c) {
        c.kb = c.chunk * CHB;
        c.kb_end = c.kb + CHB < g.k_blocks ? c.kb + CHB : g.k_blocks;
      };
      auto advance = [&](Cursor& c) {  // returns false past the last item; order: tile, chunk, segment, k-block
        if (++c.kb == c.kb_end) {
          if (++c.seg == g.segs) {
            c.seg = 0;
            if (++c.chunk == NCH) {
              c.chunk = 0;
              c.t += num_pairs;
              if (c.t >= g.total_tiles) return false;
              place(c);
            }
          }
          chunk_range(c);
        }
        return true;
      };
      auto issue = [&](unsigned char* sa, uint32_t bar, const Cursor& c) {
        const int pa = g.segs > 1 ? kPlaneA[c.seg] : 0, pb = g.segs > 1 ? kPlaneB[c.seg] : 0;
        const int k0 = c.kb * BK;
        unsigned char* sb = sa + A_STAGE_BYTES;
        if (g.a_kmajor) {
          tma_load_4d_pair(sa, &tm_a, bar, k0, c.m0, g.rag ? c.kres : c.b, g.rag ? c.b : pa);
        } else {
          tma_load_4d_pair(sa, &tm_a, bar, c.m0, k0, c.b, pa);
          tma_load_4d_pair(sa + 8192, &tm_a, bar, c.m0 + 64, k0, c.b, pa);
        }
        if (g.b_kmajor) {
          tma_load_4d_pair(sb, &tm_b, bar, k0, c.n0, c.b, pb);
        } else {
          tma_load_4d_pair(sb, &tm_b, bar, c.n0, k0, c.b, pb);
          tma_load_4d_pair(sb + 8192, &tm_b, bar, c.n0 + 64, k0, c.b, pb);
        }
      };
      if (pair < g.total_tiles) {
        Cursor ld{pair, 0, 0, 0, 0, 0, 0, 0, 0};
        place(ld);
        chunk_range(ld);
        // full[s] of the leader, as a cluster address: the same offset for every stage
        const uint32_t full0 = map_to_cta(smem_u32(&full[0]), 0);
        int s = 0;
        uint32_t phase = 0;
        for (;;) {
          if (!mbar_wait_cluster(&empty[s], phase ^ 1, err, 1)) break;
          if (leader) mbar_expect_tx(&full[s], 2 * P_STAGE_BYTES);
          issue(tiles + s * P_STAGE_BYTES, full0 + s * 8, ld);
          if (++s == P_STAGES) { s = 0; phase ^= 1; }
          if (!advance(ld)) break;
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------------- issuer ---
    if (lane == 0 && leader) {
      uint32_t idesc = 0;
      idesc |= 1u << 4;
      idesc |= (g.in_f16 ? 0u : 1u) << 7;
      idesc |= (g.in_f16 ? 0u : 1u) << 10;
      idesc |= (g.a_kmajor ? 0u : 1u) << 15;
      idesc |= (g.b_kmajor ? 0u : 1u) << 16;
      idesc |= (uint32_t)(BN >> 3) << 17;
      idesc |= (uint32_t)((2 * BM) >> 4) << 24;   // M = 256 across the pair
      const uint32_t a_lbo = g.a_kmajor ? 16u : 8192u, b_lbo = g.b_kmajor ? 16u : 8192u;
      const uint32_t a_kstep = g.a_kmajor ? 32u : 2048u, b_kstep = g.b_kmajor ? 32u : 2048u;
      const uint32_t empty_own = map_to_cta(smem_u32(&empty[0]), 0), empty_peer = map_to_cta(smem_u32(&empty[0]), 1);
      const uint64_t da0 = make_smem_desc(smem_u32(tiles), a_lbo, 1024), db0 = make_smem_desc(smem_u32(tiles) + A_STAGE_BYTES, b_lbo, 1024);
      int s = 0;
      uint32_t phase = 0;
      bool ok = true;
      int local_tile = 0;   // counts work items: one per chunk of a tile
      for (int64_t t = pair; t < g.total_tiles && ok; t += num_pairs)
      for (int chunk = 0; chunk < NCH && ok; ++chunk, ++local_tile) {
        const int acc = local_tile & 1;
        const uint32_t acc_phase = (local_tile >> 1) & 1;
        if (!mbar_wait_cluster(&acc_empty[acc], acc_phase ^ 1, err, 2)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        const int kb_begin = chunk * CHB;
        const int kb_end = kb_begin + CHB < g.k_blocks ? kb_begin + CHB : g.k_blocks;
        const int iters = (kb_end - kb_begin) * g.segs;
        for (int it = 0; it < iters; ++it) {
          if (!mbar_wait_cluster(&full[s], phase, err, 3)) { ok = false; break; }
          tc_fence_after();
          // the descriptors differ from stage 0's only in the 14-bit address field (shared memory is below 256 KiB: no carry)
          const uint64_t da_s = da0 + (uint64_t)((s * P_STAGE_BYTES) >> 4), db_s = db0 + (uint64_t)((s * P_STAGE_BYTES) >> 4);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_f16_pair(d_tmem, da_s + (uint64_t)((k * a_kstep) >> 4), db_s + (uint64_t)((k * b_kstep) >> 4), idesc, (it | k) != 0 ? 1u : 0u);
          // the stage is free in BOTH CTAs once these MMAs have read it
          tc_commit_pair(empty_own + s * 8);
          tc_commit_pair(empty_peer + s * 8);
          if (++s == P_STAGES) { s = 0; phase ^= 1; }
        }
        if (ok) {
          tc_commit_pair(map_to_cta(smem_u32(&acc_full[acc]), 0));
          tc_commit_pair(map_to_cta(smem_u32(&acc_full[acc]), 1));
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue ---
    const int quarter = warp & 3;
    bool ok = true;
    int local_tile = 0;
    uint32_t rphase = 0;
    for (int64_t t = pair; t < g.total_tiles && ok; t += num_pairs) {
      int b, m_t, n_t;
      pair_tile_coords(g, t, &b, &m_t, &n_t);
      int kres = 0;
      if (g.rag) { kres = m_t & 7; m_t >>= 3; }
      for (int chunk = 0; chunk < NCH && ok; ++chunk, ++local_tile) {
        const int acc = local_tile & 1;
        const uint32_t acc_phase = (local_tile >> 1) & 1;
        const bool landed = mbar_wait_cluster(&acc_full[acc], acc_phase, err, 4);
        if (!__all_sync(0xffffffffu, landed)) { ok = false; break; }
        tc_fence_after();
        drain_accumulator_narrow<OutT>(g, &tm_c, &tm_r, &res_bar[warp - 2], rphase, tmem_base + acc * BN, (int64_t)m_t * 2 * BM + (int64_t)rank * BM, (int64_t)n_t * BN, b, kres,
                                       quarter, (warp - 2) >> 2, lane, epi_stage + (warp - 2) * S_EPI_STAGE_WORDS, chunk);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty[acc]), 0));
      }
    }
    if (g.tma_store && lane == 0) bulk_wait_all();   // this warp's tile stores are done before its staging memory goes away
  }

  // ---------------------------------------------------------------------- teardown ---
  tc_fence_before();
  __shared__ int failed;
  if (threadIdx.x == 0) failed = *err;
  __syncthreads();
  if (failed != 0) {
    const unsigned long long t0 = global_ns();
    while (global_ns() - t0 < 200000ull) {}
    __syncthreads();
  }
  cluster_sync_all();  // the peer has issued its last load, MMA and remote arrive
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

}  // namespace

namespace {

// ---- fp32 -> three bf16 planes (hi, mid, lo): x = p0 + p1 + p2 up to 2^-24 relative ----
__global__ void __launch_bounds__(256) split3_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ planes, int64_t n) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const float v = x[i];
    const __nv_bfloat16 h0 = __float2bfloat16_rn(v);
    const float r1 = v - __bfloat162float(h0);
    const __nv_bfloat16 h1 = __float2bfloat16_rn(r1);
    const float r2 = r1 - __bfloat162float(h1);
    planes[i] = h0;
    planes[n + i] = h1;
    planes[2 * n + i] = __float2bfloat16_rn(r2);
  }
}

// 4-D map {inner, outer, batch, plane} over 16-bit elements with a {64, box_outer, 1, 1} box and 128-byte swizzle.
Status make_operand_map(CUtensorMap* map, const void* base, bool f16, int64_t inner, int64_t outer, int64_t ld, int64_t batch,
                        int64_t batch_stride, int64_t planes, int64_t plane_stride, int box_outer) {
  const uint64_t dims[4] = {(uint64_t)inner, (uint64_t)outer, (uint64_t)batch, (uint64_t)planes};
  const uint64_t strides[3] = {(uint64_t)ld * 2, (uint64_t)batch_stride * 2, (uint64_t)plane_stride * 2};
  const uint32_t box[4] = {64, (uint32_t)box_outer, 1, 1};
  return encode_tma_4d_16bit(map, base, f16, dims, strides, box);
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }


}  // namespace

// Ragged rows (see TcArgs::rag): a dense 16-bit result whose row length is not a multiple of 8, written with aligned
// 16-byte vectors all the same.  Needs both operands K-major (the shifted column window moves B's N coordinate, which
// must not be the contiguous one; A's rows are taken with a stride of 8), whole classes (M a multiple of 8), classes
// of at least one full tile, and nothing fused that is indexed by column or laid out like C.
bool gemm_tcgen05_ragged_rows(const GemmParams& p, bool has_bias, bool has_residual) {
  const bool is16 = p.dtype == B200_BFLOAT16 || p.dtype == B200_FLOAT16;
  static const bool on = []() { const char* v = getenv("B200MLX_GEMM_RAGGED"); return !(v && v[0] == '0'); }();
  return on && is16 && p.a_k_major && p.b_k_major && p.m % 8 == 0 && p.m >= 8 * BM && p.n % 8 != 0 && p.k % 8 == 0 && !has_bias &&
         !has_residual && p.num_c_extra == 0 && (p.ldc <= 0 || p.ldc == p.n) && p.a_batch_stride < 0 && p.b_batch_stride < 0;
}

Status gemm_tcgen05(Device* dev, const GemmParams& p, bool* taken) {
  *taken = false;
  const bool is16 = p.dtype == B200_BFLOAT16 || p.dtype == B200_FLOAT16;
  const bool is32 = p.dtype == B200_FLOAT32;
  if (!is16 && !is32) return Status::OK();
  if (p.batch <= 0 || p.m <= 0 || p.n <= 0 || p.k <= 0) return Status::OK();
  if (p.a_batch_stride >= 0 || p.b_batch_stride >= 0) return Status::OK();  // only dense batches here
  // TMA needs 16-byte aligned bases and row pitches: the contiguous extent of each operand must be a multiple of 8 elements.
  const int64_t a_inner = p.a_k_major ? p.k : p.m, b_inner = p.b_k_major ? p.k : p.n;
  if (a_inner % 8 != 0 || b_inner % 8 != 0) return Status::OK();
  if (!aligned16(p.a) || !aligned16(p.b)) return Status::OK();
  if (p.m > 0x7fffffffLL || p.n > 0x7fffffffLL || p.k > 0x7fffffffLL || p.batch > 0x7fffffffLL) return Status::OK();
  // tiny problems are latency-bound either way; leave them to the SIMT kernel
  if ((double)p.batch * p.m * p.n * p.k < 64.0 * 64.0 * 64.0) return Status::OK();
  // tile coordinates are computed in 32-bit arithmetic on the device
  if ((double)p.batch * (double)((p.m + BM - 1) / BM + 8) * (double)((p.n + 7 + BN - 1) / BN) >= 2147483648.0) return Status::OK();
  *taken = true;

  B200_TRY(dev->MakeCurrent());
  cudaStream_t stream = dev->stream();
  const void* a = p.a;
  const void* b = p.b;
  void* tmp_a = nullptr;
  void* tmp_b = nullptr;
  int64_t planes = 1, a_plane_stride = 0, b_plane_stride = 0;
  const int64_t a_elems = p.batch * p.m * p.k, b_elems = p.batch * p.k * p.n;
  void* planes_a = nullptr;
  void* planes_b = nullptr;
  if (is32) {
    // three bf16 planes per operand: in the caller's scratch when it gave one, else allocated for this launch
    if (p.split_scratch && p.split_scratch_bytes >= gemm_split_scratch_bytes(p.batch, p.m, p.n, p.k) && aligned16(p.split_scratch)) {
      planes_a = p.split_scratch;
      planes_b = reinterpret_cast<char*>(p.split_scratch) + (a_elems * 6 + 255) / 256 * 256;
    } else {
      Status s = dev->Alloc(a_elems * 6, &tmp_a);
      if (s.ok()) s = dev->Alloc(b_elems * 6, &tmp_b);
      if (!s.ok()) { dev->Free(tmp_a); return s; }
      planes_a = tmp_a;
      planes_b = tmp_b;
    }
    auto grid_for = [&](int64_t n) { int64_t g = (n + 255) / 256, cap = (int64_t)dev->sm_count() * 16; return (unsigned)(g < cap ? g : cap); };
    split3_kernel<<<grid_for(a_elems), 256, 0, stream>>>((const float*)p.a, (__nv_bfloat16*)planes_a, a_elems);
    split3_kernel<<<grid_for(b_elems), 256, 0, stream>>>((const float*)p.b, (__nv_bfloat16*)planes_b, b_elems);
    a = planes_a; b = planes_b;
    planes = 3; a_plane_stride = a_elems; b_plane_stride = b_elems;
  }
  auto cleanup = [&]() { dev->Free(tmp_a); dev->Free(tmp_b); };

  // CTA pairs (256-row tiles) whenever there is more than one 128-row tile of M to share B with
  static const int pair_mode = []() { const char* v = getenv("B200MLX_GEMM_PAIR"); return v ? atoi(v) : 1; }();   // 0 never, 1 by shape, 2 always
  const bool pair_allowed = pair_mode != 0;
  // Pairs pay off once a tile's main loop is long enough to hide the cross-CTA hand-offs (measured: K = 512 is 8 % slower on
  // pairs, K >= 4096 is 5 - 10 % faster) and there are enough tiles to fill the GPU either way.
  const int64_t k_iters = (p.k + BK - 1) / BK * (is32 ? 6 : 1);
  const bool rag = gemm_tcgen05_ragged_rows(p, p.bias != nullptr, p.residual != nullptr) && aligned16(p.c);
  const int64_t m_rows = rag ? p.m / 8 : p.m;            // rows of one tile grid (a row class, or all of M)
  const int64_t n_cols = rag ? p.n + 7 : p.n;            // its columns (a class's window may start up to 7 columns early)
  const int64_t grids = rag ? 8 : 1;
  const int64_t pair_tiles = ((m_rows + 2 * BM - 1) / (2 * BM)) * ((n_cols + BN - 1) / BN) * p.batch * grids;
  const bool use_pair = pair_allowed && m_rows > BM && (pair_mode == 2 || (k_iters >= 16 && pair_tiles >= 32));

  CUtensorMap tm_a, tm_b;
  Status s;
  const bool f16 = p.dtype == B200_FLOAT16;
  const int b_box = use_pair ? P_BN_HALF : BN;
  if (rag) s = make_operand_map(&tm_a, a, f16, p.k, p.m / 8, 8 * p.k, 8, p.k, p.batch, p.m * p.k, BM);   // {K, row in class, class, batch}
  else if (p.a_k_major) s = make_operand_map(&tm_a, a, f16, p.k, p.m, p.k, p.batch, p.m * p.k, planes, planes > 1 ? a_plane_stride : p.m * p.k * p.batch, BM);
  else s = make_operand_map(&tm_a, a, f16, p.m, p.k, p.m, p.batch, p.m * p.k, planes, planes > 1 ? a_plane_stride : p.m * p.k * p.batch, 64);
  if (s.ok()) {
    if (p.b_k_major) s = make_operand_map(&tm_b, b, f16, p.k, p.n, p.k, p.batch, p.n * p.k, planes, planes > 1 ? b_plane_stride : p.n * p.k * p.batch, b_box);
    else s = make_operand_map(&tm_b, b, f16, p.n, p.k, p.n, p.batch, p.n * p.k, planes, planes > 1 ? b_plane_stride : p.n * p.k * p.batch, 64);
  }
  if (!s.ok()) { cleanup(); return s; }

  TcArgs g;
  g.c = p.c; g.bias = p.bias; g.residual = p.residual; g.residual_mul = p.residual_op;
  g.num_c_extra = p.num_c_extra;
  for (int x = 0; x < GemmParams::kMaxExtraC; ++x) g.c_extra[x] = x < p.num_c_extra ? p.c_extra[x] : nullptr;
  g.M = p.m; g.N = p.n; g.K = p.k; g.ldc = p.ldc > 0 ? p.ldc : p.n;
  g.batch = (int)p.batch;
  g.a_kmajor = p.a_k_major ? 1 : 0; g.b_kmajor = p.b_k_major ? 1 : 0;
  g.activation = p.activation;
  g.in_f16 = f16 ? 1 : 0;
  g.out_dtype = p.dtype;
  const int tile_rows = use_pair ? 2 * BM : BM;
  g.tiles_m = (int)((m_rows + tile_rows - 1) / tile_rows * grids);   // ragged rows: 8 * (tile within the class) + class
  g.tiles_n = (int)((n_cols + BN - 1) / BN);
  g.rag = rag ? 1 : 0;
  g.rag_q = (int)(p.n & 7);
  g.total_tiles = (int64_t)g.tiles_m * g.tiles_n * p.batch;
  g.k_blocks = (int)((p.k + BK - 1) / BK);
  g.segs = is32 ? 6 : 1;
  // fp32: chunks of at most 8 k-blocks (512 elements of K), balanced over the K range (see TcArgs::num_chunks)
  static const int chunk_cap = []() { const char* v = getenv("B200MLX_GEMM_F32_CHUNK_BLOCKS"); return v ? atoi(v) : 8; }();   // 0 = never cut
  g.num_chunks = (is32 && chunk_cap > 0) ? (g.k_blocks + chunk_cap - 1) / chunk_cap : 1;
  g.chunk_blocks = (g.k_blocks + g.num_chunks - 1) / g.num_chunks;
  const int out_vec = is32 ? 4 : 8;
  g.vec_store = (rag || (g.ldc % out_vec == 0 && g.ldc >= (p.n + out_vec - 1) / out_vec * out_vec && aligned16(p.c) && aligned16(p.residual))) ? 1 : 0;
  if (p.num_c_extra > 0) {
    bool ok = g.vec_store != 0 && !is32;
    for (int x = 0; x < p.num_c_extra; ++x) ok = ok && aligned16(p.c_extra[x]);
    if (!ok) { cleanup(); return Status::Unsupported("gemm: extra destinations need 16-byte aligned rows and a 16-bit type"); }
  }
  g.err_flag = dev->kernel_error_flag();
  // C as a tile-store destination {N, M, batch}: boxes of 32 columns x 32 rows, 64-byte swizzle
  static const bool tma_store_on = []() { const char* v = getenv("B200MLX_GEMM_TMA_STORE"); return !(v && v[0] == '0'); }();
  g.tma_store = (tma_store_on && is16 && g.vec_store && !rag && p.num_c_extra == 0) ? 1 : 0;
  CUtensorMap tm_c = tm_a, tm_r = tm_a;   // valid maps when unused
  if (g.tma_store) {
    const uint64_t cdims[4] = {(uint64_t)p.n, (uint64_t)p.m, (uint64_t)p.batch, 1};
    const uint64_t cstrides[3] = {(uint64_t)g.ldc * 2, (uint64_t)p.m * (uint64_t)g.ldc * 2, (uint64_t)p.m * (uint64_t)g.ldc * 2 * (uint64_t)p.batch};
    const uint32_t cbox[4] = {32, 32, 1, 1};
    s = encode_tma_4d_16bit(&tm_c, p.c, f16, cdims, cstrides, cbox, 64);
    if (s.ok() && p.residual) s = encode_tma_4d_16bit(&tm_r, p.residual, f16, cdims, cstrides, cbox, 64);   // same shape and pitch as C
    if (!s.ok()) { cleanup(); return s; }
  }

  cudaError_t e = cudaSuccess;
  // the dynamic shared memory opt-in is per function and per device; do it once
  static std::mutex attr_mu;
  static bool attr_done[6][64] = {};
  static int max_pairs[6][64] = {};
#define LAUNCH_TC(OutT, SLOT)                                                                                               \
  do {                                                                                                                      \
    {                                                                                                                       \
      std::lock_guard<std::mutex> lock(attr_mu);                                                                            \
      if (!attr_done[SLOT][dev->ordinal()]) {                                                                               \
        e = cudaFuncSetAttribute(gemm_tcgen05_kernel<OutT>, cudaFuncAttributeMaxDynamicSharedMemorySize, S_SMEM_BYTES);       \
        attr_done[SLOT][dev->ordinal()] = (e == cudaSuccess);                                                               \
      }                                                                                                                     \
    }                                                                                                                       \
    const int64_t grid = g.total_tiles < dev->sm_count() ? g.total_tiles : dev->sm_count();                                 \
    if (e == cudaSuccess) e = launch_dependent(gemm_tcgen05_kernel<OutT>, (unsigned)grid, S_NUM_THREADS, S_SMEM_BYTES, stream, tm_a, tm_b, tm_c, tm_r, g); \
  } while (0)
#define LAUNCH_TC_PAIR(OutT, SLOT)                                                                                          \
  do {                                                                                                                      \
    {                                                                                                                       \
      std::lock_guard<std::mutex> lock(attr_mu);                                                                            \
      if (!attr_done[SLOT][dev->ordinal()]) {                                                                               \
        e = cudaFuncSetAttribute(gemm_tcgen05_pair_kernel<OutT>, cudaFuncAttributeMaxDynamicSharedMemorySize, P_SMEM_BYTES); \
        attr_done[SLOT][dev->ordinal()] = (e == cudaSuccess);                                                               \
        /* how many pairs can be resident at once: the persistent grid is that many clusters */                             \
        int clusters = 0;                                                                                                   \
        cudaLaunchConfig_t cfg = {};                                                                                        \
        cfg.gridDim = dim3((unsigned)(dev->sm_count() & ~1));                                                               \
        cfg.blockDim = dim3(S_NUM_THREADS);                                                                                 \
        cfg.dynamicSmemBytes = P_SMEM_BYTES;                                                                                \
        cudaLaunchAttribute attr[1];                                                                                        \
        attr[0].id = cudaLaunchAttributeClusterDimension;                                                                   \
        attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;                           \
        cfg.attrs = attr; cfg.numAttrs = 1;                                                                                 \
        if (e == cudaSuccess && cudaOccupancyMaxActiveClusters(&clusters, gemm_tcgen05_pair_kernel<OutT>, &cfg) != cudaSuccess) { \
          cudaGetLastError();                                                                                               \
          clusters = 0;                                                                                                     \
        }                                                                                                                   \
        if (clusters <= 0 || clusters > dev->sm_count() / 2) clusters = dev->sm_count() / 2;                                \
        max_pairs[SLOT][dev->ordinal()] = clusters;                                                                         \
      }                                                                                                                     \
    }                                                                                                                       \
    const int64_t cap = max_pairs[SLOT][dev->ordinal()];                                                                    \
    const int64_t pairs = g.total_tiles < cap ? g.total_tiles : cap;                                                        \
    if (e == cudaSuccess)                                                                                                   \
      e = launch_dependent(gemm_tcgen05_pair_kernel<OutT>, (unsigned)(2 * pairs), S_NUM_THREADS, P_SMEM_BYTES, stream, tm_a, tm_b, tm_c, tm_r, g); \
  } while (0)
  if (use_pair) {
    if (is32) LAUNCH_TC_PAIR(float, 3);
    else if (f16) LAUNCH_TC_PAIR(__half, 4);
    else LAUNCH_TC_PAIR(__nv_bfloat16, 5);
  } else {
    if (is32) LAUNCH_TC(float, 0);
    else if (f16) LAUNCH_TC(__half, 1);
    else LAUNCH_TC(__nv_bfloat16, 2);
  }
#undef LAUNCH_TC
#undef LAUNCH_TC_PAIR
  cleanup();  // stream-ordered: the blocks are reused only by work enqueued after this kernel
  if (e != cudaSuccess) {
    cudaGetLastError();
    return Status::Cuda(strfmt("gemm_tcgen05: %s", cudaGetErrorString(e)));
  }
  return dev->CheckLaunch("gemm_tcgen05");
}

}  // namespace k
}  // namespace b200
