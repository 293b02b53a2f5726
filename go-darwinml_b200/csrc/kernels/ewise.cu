// Fused elementwise chains: one interpreter kernel evaluates a whole
// straight-line program (loads with broadcast strides, iotas, immediates,
// unary / binary / compare / select / clamp / cast) per output element, so a
// chain of N graph ops costs one read of each distinct input and one write of
// the result instead of N round trips through HBM.  The reference issues one
// MPSGraph op per primitive (mpsgraph bridge.m:265-401 macros) and leaves
// fusion to Apple's compiler; here the lowering pass builds the program and this
// kernel runs it.
//
// Virtual registers live in shared memory as [reg][vector][element][thread]:
// dynamic register numbers cost nothing to index, and for a fixed element the
// threads of a warp touch consecutive banks, so no access conflicts.
// Register representation:
//   F16/BF16/F32 -> float bits      (16-bit floats are re-rounded after every op,
//                                    so a fused chain equals the op-by-op result)
//   F64 -> double bits (wide programs only)
//   I8/I16/I32, U8/U16/U32, Bool -> 32-bit integer, sign/zero extended
//   I64/U64 -> 64-bit integer (wide programs only)
// HBM-bound: bytes = sum of distinct leaf bytes + output bytes.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <utility>

#include "../kernels.h"

namespace b200 {
namespace k {

namespace {

constexpr int kBlock = 128;

#include "ewise_ops.cuh"

// The interpreter decodes an instruction once and calls these out of line; the run-time compiled kernels inline the cores.
template <typename R>
__device__ __noinline__ R eval_op(const EwInstr& in, R a, R b, R c) { return eval_op_core<R>(in.op, in.sdtype, a, b, c); }
template <typename R>
__device__ __noinline__ R eval_cast(int from, int to, R a) { return eval_cast_core<R>(from, to, a); }

// One thread owns U vectors of VEC consecutive output elements (vector u of a thread is kBlock vectors after
// vector u-1, so a warp's accesses stay coalesced).  Each program instruction is decoded ONCE per thread and
// applied to all U*VEC elements; the hottest float ops are dispatched outside the element loop.
// RANK is the compile-time rank of the (collapsed) output index space: the host pads leading dims of size 1 up to
// the next instantiated rank, so index arithmetic is RANK-1 divisions and RANK multiply-adds, fully unrolled.
template <typename R, int VEC, int U, int RANK>
__global__ void __launch_bounds__(kBlock, 4) ewise_kernel(const __grid_constant__ EwProgram p, int64_t total_vecs) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  R* regs = reinterpret_cast<R*>(smem_raw);  // [reg][U][VEC][kBlock]: consecutive threads hit consecutive banks
  const int tid = threadIdx.x;
  constexpr int rank = RANK;
  const int64_t first_vec = (int64_t)blockIdx.x * (kBlock * U) + tid;
  // multi-index of the first element of each of this thread's vectors (32-bit: callers split larger tensors)
  int idx[U][RANK];
  bool live[U];
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const int64_t vi = first_vec + (int64_t)u * kBlock;
    live[u] = vi < total_vecs;
    // statically indexed (fully unrolled) so that idx stays in registers
    uint32_t rem = (uint32_t)(vi * VEC);
#pragma unroll
    for (int d = RANK - 1; d > 0; --d) {
      const uint32_t dim = (uint32_t)p.dims[d];
      const uint32_t q = rem / dim;
      idx[u][d] = (int)(rem - q * dim);
      rem = q;
    }
    idx[u][0] = (int)rem;
  }
#define REG(r, u, v) regs[(((r) * U + (u)) * VEC + (v)) * kBlock + tid]
#define FOR_ALL(...)                                                \
  _Pragma("unroll") for (int u = 0; u < U; ++u) {                   \
    if (!live[u]) continue;                                         \
    _Pragma("unroll") for (int v = 0; v < VEC; ++v) { __VA_ARGS__ } \
  }
  for (int pc = 0; pc < p.num_instr; ++pc) {
    const EwInstr in = p.instr[pc];
    switch (in.kind) {
      case EW_LOAD: {
        const EwLeaf& lf = p.leaves[in.a];
        const int64_t si = lf.strides[RANK - 1];
        const bool al16 = (reinterpret_cast<uintptr_t>(lf.ptr) & 15) == 0;
#pragma unroll
        for (int u = 0; u < U; ++u) {
          if (!live[u]) continue;
          int64_t off = 0;
#pragma unroll
          for (int d = 0; d < RANK; ++d) off += (int64_t)idx[u][d] * lf.strides[d];
          if (VEC == 4 && si == 1 && (off & 3) == 0 && al16 &&
              (lf.dtype == B200_FLOAT32 || lf.dtype == B200_INT32 || lf.dtype == B200_UINT32)) {
            const uint4 q = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint32_t*>(lf.ptr) + off);
            REG(in.dst, u, 0) = (R)q.x; REG(in.dst, u, 1 % VEC) = (R)q.y; REG(in.dst, u, 2 % VEC) = (R)q.z; REG(in.dst, u, 3 % VEC) = (R)q.w;
          } else if (VEC == 4 && si == 1 && (off & 3) == 0 && al16 && lf.dtype == B200_BFLOAT16) {
            const uint2 q = *reinterpret_cast<const uint2*>(reinterpret_cast<const uint16_t*>(lf.ptr) + off);
            REG(in.dst, u, 0) = (R)(q.x << 16); REG(in.dst, u, 1 % VEC) = (R)(q.x & 0xffff0000u);
            REG(in.dst, u, 2 % VEC) = (R)(q.y << 16); REG(in.dst, u, 3 % VEC) = (R)(q.y & 0xffff0000u);
          } else if (si == 0) {
            const R r = load_elem<R>(lf.ptr, off, lf.dtype);
#pragma unroll
            for (int v = 0; v < VEC; ++v) REG(in.dst, u, v) = r;
          } else {
#pragma unroll
            for (int v = 0; v < VEC; ++v) REG(in.dst, u, v) = load_elem<R>(lf.ptr, off + v * si, lf.dtype);
          }
        }
        break;
      }
      case EW_IMM:
        FOR_ALL(REG(in.dst, u, v) = (R)in.imm;)
        break;
      case EW_IOTA: {
        const int d = in.a;
        FOR_ALL({
          int64_t coord = 0;
          _Pragma("unroll") for (int dd = 0; dd < RANK; ++dd) if (dd == d) coord = idx[u][dd];
          coord += (d == rank - 1) ? v : 0;
          R r;
          if (in.dtype == B200_FLOAT64) { if constexpr (RegTraits<R>::wide) r = from_d((double)coord); else r = 0; }
          else if (dtype_is_float(in.dtype)) r = from_f<R>(round_to(in.dtype, (float)coord));
          else if (in.dtype == B200_INT64 || in.dtype == B200_UINT64) r = (R)(uint64_t)coord;
          else r = (R)wrap_i32(in.dtype, (uint32_t)coord);
          REG(in.dst, u, v) = r;
        })
        break;
      }
      case EW_CAST:
        FOR_ALL(REG(in.dst, u, v) = eval_cast<R>(in.sdtype, in.dtype, REG(in.a, u, v));)
        break;
      default: {
        const int sd = in.sdtype;
        const bool f32cls = sd == B200_FLOAT32 || sd == B200_BFLOAT16 || sd == B200_FLOAT16;
#define FAST2(EXPR)                                                                                          \
  if (sd == B200_FLOAT32) {                                                                                  \
    FOR_ALL({ const float x = as_f(REG(in.a, u, v)), y = as_f(REG(in.b, u, v)); REG(in.dst, u, v) = from_f<R>((EXPR)); })      \
  } else if (sd == B200_BFLOAT16) {                                                                          \
    FOR_ALL({ const float x = as_f(REG(in.a, u, v)), y = as_f(REG(in.b, u, v));                              \
              REG(in.dst, u, v) = from_f<R>(__bfloat162float(__float2bfloat16_rn((EXPR)))); })               \
  } else {                                                                                                   \
    FOR_ALL({ const float x = as_f(REG(in.a, u, v)), y = as_f(REG(in.b, u, v));                              \
              REG(in.dst, u, v) = from_f<R>(__half2float(__float2half_rn((EXPR)))); })                       \
  }                                                                                                          \
  break;
#define FAST1(EXPR)                                                                                          \
  if (sd == B200_FLOAT32) {                                                                                  \
    FOR_ALL({ const float x = as_f(REG(in.a, u, v)); REG(in.dst, u, v) = from_f<R>((EXPR)); })               \
  } else if (sd == B200_BFLOAT16) {                                                                          \
    FOR_ALL({ const float x = as_f(REG(in.a, u, v)); REG(in.dst, u, v) = from_f<R>(__bfloat162float(__float2bfloat16_rn((EXPR)))); }) \
  } else {                                                                                                   \
    FOR_ALL({ const float x = as_f(REG(in.a, u, v)); REG(in.dst, u, v) = from_f<R>(__half2float(__float2half_rn((EXPR)))); })         \
  }                                                                                                          \
  break;
        bool done = f32cls;
        if (f32cls) {
          switch ((Op)in.op) {
            case Op::Add: FAST2(x + y)
            case Op::Sub: FAST2(x - y)
            case Op::Mul: FAST2(x * y)
            case Op::Div: FAST2(x / y)
            case Op::Neg: FAST1(-x)
            case Op::Exp: FAST1(expf(x))
            case Op::Tanh: FAST1(tanhf(x))
            case Op::Rsqrt: FAST1(1.0f / sqrtf(x))
            case Op::Sigmoid: FAST1(1.0f / (1.0f + expf(-x)))
            case Op::Silu: FAST1(x / (1.0f + expf(-x)))
            case Op::Relu: FAST1(fmaxf(x, 0.0f))
            case Op::GeluTanh: FAST1(0.5f * x * (1.0f + tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x))))
            default: done = false; break;
          }
        }
#undef FAST1
#undef FAST2
        if (!done) {
          FOR_ALL(REG(in.dst, u, v) = eval_op<R>(in, REG(in.a, u, v), REG(in.b, u, v), REG(in.c, u, v));)
        }
        break;
      }
    }
  }
  const bool out_al = (reinterpret_cast<uintptr_t>(p.out) & 15) == 0;
#pragma unroll
  for (int u = 0; u < U; ++u) {
    if (!live[u]) continue;
    const int64_t out0 = (first_vec + (int64_t)u * kBlock) * VEC;
    if (VEC == 4 && out_al && (p.out_dtype == B200_FLOAT32 || p.out_dtype == B200_INT32 || p.out_dtype == B200_UINT32)) {
      uint4 q;
      q.x = (uint32_t)REG(p.out_reg, u, 0); q.y = (uint32_t)REG(p.out_reg, u, 1 % VEC);
      q.z = (uint32_t)REG(p.out_reg, u, 2 % VEC); q.w = (uint32_t)REG(p.out_reg, u, 3 % VEC);
      *reinterpret_cast<uint4*>(reinterpret_cast<uint32_t*>(p.out) + out0) = q;
    } else if (VEC == 4 && out_al && p.out_dtype == B200_BFLOAT16) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(as_f(REG(p.out_reg, u, 0)), as_f(REG(p.out_reg, u, 1 % VEC)));
      __nv_bfloat162 hi = __floats2bfloat162_rn(as_f(REG(p.out_reg, u, 2 % VEC)), as_f(REG(p.out_reg, u, 3 % VEC)));
      uint2 q;
      q.x = *reinterpret_cast<uint32_t*>(&lo); q.y = *reinterpret_cast<uint32_t*>(&hi);
      *reinterpret_cast<uint2*>(reinterpret_cast<uint16_t*>(p.out) + out0) = q;
    } else {
#pragma unroll
      for (int v = 0; v < VEC; ++v) store_elem<R>(p.out, out0 + v, p.out_dtype, REG(p.out_reg, u, v));
    }
  }
#undef FOR_ALL
#undef REG
}


inline bool is_bin_host(int op) { return op >= (int)Op::Add && op <= (int)Op::ShiftRightLogical; }

// ---- fast path: out = op(a, b) on one storage type, a dense, b dense or repeating with a period -------------
// (residual adds, bias adds, gated multiplies).  16-byte vectors, grid-stride, no shared memory.
template <typename T> struct FastCvt;
template <> struct FastCvt<float> {
  static constexpr int N = 4;
  __device__ __forceinline__ static void unpack(const uint4& q, float* f) {
    f[0] = __uint_as_float(q.x); f[1] = __uint_as_float(q.y); f[2] = __uint_as_float(q.z); f[3] = __uint_as_float(q.w);
  }
  __device__ __forceinline__ static uint4 pack(const float* f) {
    return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
  }
};
template <> struct FastCvt<__nv_bfloat16> {
  static constexpr int N = 8;
  __device__ __forceinline__ static void unpack(const uint4& q, float* f) {
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { f[2 * i] = __uint_as_float(w[i] << 16); f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
  }
  __device__ __forceinline__ static uint4 pack(const float* f) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) { __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]); w[i] = *reinterpret_cast<uint32_t*>(&h); }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
};
template <> struct FastCvt<__half> {
  static constexpr int N = 8;
  __device__ __forceinline__ static void unpack(const uint4& q, float* f) {
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { float2 v = __half22float2(*reinterpret_cast<const __half2*>(&w[i])); f[2 * i] = v.x; f[2 * i + 1] = v.y; }
  }
  __device__ __forceinline__ static uint4 pack(const float* f) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) { __half2 h = __floats2half2_rn(f[2 * i], f[2 * i + 1]); w[i] = *reinterpret_cast<uint32_t*>(&h); }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
};

template <typename T, int OPC>
__global__ void __launch_bounds__(256) ewise_binary_fast_kernel(const uint4* __restrict__ a, const uint4* __restrict__ b, uint4* __restrict__ out,
                                                                int64_t nvec, int64_t b_period_vecs) {
  constexpr int N = FastCvt<T>::N;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    const uint4 qa = a[i];
    const uint4 qb = b[b_period_vecs == nvec ? i : (nvec <= 0xffffffffLL ? (int64_t)((uint32_t)i % (uint32_t)b_period_vecs) : i % b_period_vecs)];
    float x[N], y[N];
    FastCvt<T>::unpack(qa, x);
    FastCvt<T>::unpack(qb, y);
#pragma unroll
    for (int e = 0; e < N; ++e) {
      if (OPC == 0) x[e] = x[e] + y[e];
      else if (OPC == 1) x[e] = x[e] - y[e];
      else if (OPC == 2) x[e] = x[e] * y[e];
      else x[e] = x[e] / y[e];
    }
    out[i] = FastCvt<T>::pack(x);
  }
}

// Recognises LOAD a, LOAD b, OP(a, b) over one float type with a dense and b dense-or-periodic; launches the fast kernel.
bool try_binary_fast(Device* dev, const EwProgram& p, int64_t n) {
  if (p.num_instr != 3 || p.num_leaves != 2) return false;
  const EwInstr &i0 = p.instr[0], &i1 = p.instr[1], &i2 = p.instr[2];
  if (i0.kind != EW_LOAD || i1.kind != EW_LOAD || i2.kind != EW_OP) return false;
  int opc;
  switch ((Op)i2.op) {
    case Op::Add: opc = 0; break;
    case Op::Sub: opc = 1; break;
    case Op::Mul: opc = 2; break;
    case Op::Div: opc = 3; break;
    default: return false;
  }
  const int dt = p.out_dtype;
  if (!(dt == B200_FLOAT32 || dt == B200_BFLOAT16 || dt == B200_FLOAT16)) return false;
  if (i2.dtype != dt || i2.sdtype != dt || p.leaves[0].dtype != dt || p.leaves[1].dtype != dt) return false;
  if (p.out_reg != i2.dst) return false;
  // which leaf feeds which operand
  int la = -1, lb = -1;
  if (i2.a == i0.dst && i2.b == i1.dst) { la = i0.a; lb = i1.a; }
  else if (i2.a == i1.dst && i2.b == i0.dst) { la = i1.a; lb = i0.a; }
  else return false;
  // dense strides of the (collapsed) output
  int64_t dense[kMaxDims];
  int64_t acc = 1;
  for (int d = p.rank - 1; d >= 0; --d) { dense[d] = acc; acc *= p.dims[d]; }
  auto is_dense = [&](const EwLeaf& lf) {
    for (int d = 0; d < p.rank; ++d)
      if (p.dims[d] != 1 && lf.strides[d] != dense[d]) return false;
    return true;
  };
  // periodic: zero strides on leading dims, dense on the trailing ones; returns the period in elements (0 = no)
  auto period_of = [&](const EwLeaf& lf) -> int64_t {
    int d = 0;
    while (d < p.rank && (lf.strides[d] == 0 || p.dims[d] == 1)) ++d;
    int64_t per = 1;
    for (int e = d; e < p.rank; ++e) {
      if (p.dims[e] != 1 && lf.strides[e] != dense[e]) return 0;
      per *= p.dims[e];
    }
    return per;
  };
  bool swapped = false;
  if (!is_dense(p.leaves[la])) {
    if ((opc == 0 || opc == 2) && is_dense(p.leaves[lb])) { std::swap(la, lb); swapped = true; }  // commutative ops only
    else return false;
  }
  (void)swapped;
  const int64_t period = is_dense(p.leaves[lb]) ? n : period_of(p.leaves[lb]);
  const int vecn = 16 / dtype_size(dt);
  if (period <= 0 || n % vecn != 0 || period % vecn != 0) return false;
  auto al = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  if (!al(p.leaves[la].ptr) || !al(p.leaves[lb].ptr) || !al(p.out)) return false;
  const int64_t nvec = n / vecn, pvec = period / vecn;
  int64_t blocks = (nvec + 255) / 256;
  const int64_t cap = (int64_t)dev->sm_count() * 16;
  if (blocks > cap) blocks = cap;
  const uint4* a = reinterpret_cast<const uint4*>(p.leaves[la].ptr);
  const uint4* b = reinterpret_cast<const uint4*>(p.leaves[lb].ptr);
  uint4* o = reinterpret_cast<uint4*>(p.out);
  cudaStream_t s = dev->stream();
#define FAST_OP(T)                                                                                         \
  switch (opc) {                                                                                           \
    case 0: ewise_binary_fast_kernel<T, 0><<<(unsigned)blocks, 256, 0, s>>>(a, b, o, nvec, pvec); break;    \
    case 1: ewise_binary_fast_kernel<T, 1><<<(unsigned)blocks, 256, 0, s>>>(a, b, o, nvec, pvec); break;    \
    case 2: ewise_binary_fast_kernel<T, 2><<<(unsigned)blocks, 256, 0, s>>>(a, b, o, nvec, pvec); break;    \
    default: ewise_binary_fast_kernel<T, 3><<<(unsigned)blocks, 256, 0, s>>>(a, b, o, nvec, pvec); break;   \
  }
  if (dt == B200_FLOAT32) { FAST_OP(float) }
  else if (dt == B200_BFLOAT16) { FAST_OP(__nv_bfloat16) }
  else { FAST_OP(__half) }
#undef FAST_OP
  return true;
}


// ---- fast path 2: small expression trees over dense / periodic / scalar leaves -------------------------------
//   form A:  out = post( op1( op0(L0, L1), L2 ) )            e.g. x*w + b, tanh(x*w + b), (a + b) * c
//   form B:  out = post( op2( op0(L0, L1), op1(L2, L3) ) )   e.g. x*cos + r*sin
// ops in {Add, Sub, Mul, Div}; post in {none, a few activations}.  One pass, 16-byte vectors, registers only.
// 16-bit results are re-rounded after every op, like the interpreter, so results equal the op-by-op evaluation.
struct TreeLeaf {
  const uint4* ptr;      // null: immediate
  int64_t period_vecs;   // == nvec: dense
  float imm;
};
struct TreeArgs {
  TreeLeaf leaf[4];
  int form;              // 0 = A, 1 = B
  int op[3];             // 0 add, 1 sub, 2 mul, 3 div; operands may be swapped (see swap)
  int swap[3];           // op k computes f(rhs, lhs) instead of f(lhs, rhs)
  int post;              // 0 none, else an Op code of a unary float op
  uint4* out;
  int64_t nvec;
};
template <typename T> __device__ __forceinline__ float round_like(float v);
template <> __device__ __forceinline__ float round_like<float>(float v) { return v; }
template <> __device__ __forceinline__ float round_like<__nv_bfloat16>(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
template <> __device__ __forceinline__ float round_like<__half>(float v) { return __half2float(__float2half_rn(v)); }

template <typename T, int N>
__device__ __forceinline__ void tree_apply(int op, int swap, const float* a, const float* b, float* r) {
  const float* x = swap ? b : a;
  const float* y = swap ? a : b;
#pragma unroll
  for (int e = 0; e < N; ++e) {
    float v;
    switch (op) {
      case 0: v = x[e] + y[e]; break;
      case 1: v = x[e] - y[e]; break;
      case 2: v = x[e] * y[e]; break;
      default: v = x[e] / y[e]; break;
    }
    r[e] = round_like<T>(v);
  }
}

template <typename T>
__global__ void __launch_bounds__(256) ewise_tree_fast_kernel(const TreeArgs g) {
  constexpr int N = FastCvt<T>::N;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int nleaf = g.form == 0 ? 3 : 4;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < g.nvec; i += stride) {
    float L[4][N];
#pragma unroll
    for (int l = 0; l < 4; ++l) {
      if (l >= nleaf) continue;
      if (g.leaf[l].ptr) {
        const int64_t pv = g.leaf[l].period_vecs;
        const int64_t j = pv == g.nvec ? i : (g.nvec <= 0xffffffffLL ? (int64_t)((uint32_t)i % (uint32_t)pv) : i % pv);
        FastCvt<T>::unpack(g.leaf[l].ptr[j], L[l]);
      } else {
#pragma unroll
        for (int e = 0; e < N; ++e) L[l][e] = g.leaf[l].imm;
      }
    }
    float t0[N], r[N];
    tree_apply<T, N>(g.op[0], g.swap[0], L[0], L[1], t0);
    if (g.form == 0) {
      tree_apply<T, N>(g.op[1], g.swap[1], t0, L[2], r);
    } else {
      float t1[N];
      tree_apply<T, N>(g.op[1], g.swap[1], L[2], L[3], t1);
      tree_apply<T, N>(g.op[2], g.swap[2], t0, t1, r);
    }
    if (g.post != 0) {
#pragma unroll
      for (int e = 0; e < N; ++e) r[e] = round_like<T>(sizeof(T) == 2 ? f_unary_to16(g.post, r[e]) : f_unary<float>(g.post, r[e]));
    }
    g.out[i] = FastCvt<T>::pack(r);
  }
}

// Matches the two tree forms in a program; on success fills TreeArgs and launches.
bool try_tree_fast(Device* dev, const EwProgram& p, int64_t n) {
  const int dt = p.out_dtype;
  if (!(dt == B200_FLOAT32 || dt == B200_BFLOAT16 || dt == B200_FLOAT16)) return false;
  if (p.num_instr < 5 || p.num_instr > 8) return false;
  // instruction that defines each register at the end of the (straight-line, SSA-allocated) program: walk backwards
  // from the output; registers are reused, so resolve a register to the LAST instruction before `at` that writes it.
  auto def_of = [&](int reg, int at) -> int {
    for (int i = at - 1; i >= 0; --i)
      if (p.instr[i].dst == reg) return i;
    return -1;
  };
  auto binop = [&](const EwInstr& in, int* code) -> bool {
    if (in.kind != EW_OP || in.dtype != dt || in.sdtype != dt) return false;
    switch ((Op)in.op) {
      case Op::Add: *code = 0; return true;
      case Op::Sub: *code = 1; return true;
      case Op::Mul: *code = 2; return true;
      case Op::Div: *code = 3; return true;
      default: return false;
    }
  };
  int64_t dense[kMaxDims];
  int64_t acc = 1;
  for (int d = p.rank - 1; d >= 0; --d) { dense[d] = acc; acc *= p.dims[d]; }
  const int vecn = 16 / dtype_size(dt);
  if (n % vecn != 0) return false;
  const int64_t nvec = n / vecn;
  auto al = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  // leaf instruction -> TreeLeaf (dense, periodic, or immediate)
  auto make_leaf = [&](int instr_index, TreeLeaf* out) -> bool {
    if (instr_index < 0) return false;
    const EwInstr& in = p.instr[instr_index];
    if (in.kind == EW_IMM) {
      if (in.dtype != dt) return false;
      uint32_t bits = (uint32_t)in.imm;
      float f;
      memcpy(&f, &bits, 4);
      *out = TreeLeaf{nullptr, nvec, f};
      return true;
    }
    if (in.kind != EW_LOAD) return false;
    const EwLeaf& lf = p.leaves[in.a];
    if (lf.dtype != dt || !al(lf.ptr)) return false;
    int d = 0;
    while (d < p.rank && (lf.strides[d] == 0 || p.dims[d] == 1)) ++d;
    int64_t per = 1;
    for (int e = d; e < p.rank; ++e) {
      if (p.dims[e] != 1 && lf.strides[e] != dense[e]) return false;
      per *= p.dims[e];
    }
    if (per % vecn != 0) return false;
    *out = TreeLeaf{reinterpret_cast<const uint4*>(lf.ptr), per / vecn, 0.f};
    return true;
  };
  TreeArgs g;
  g.post = 0;
  g.swap[0] = g.swap[1] = g.swap[2] = 0;
  int root = def_of(p.out_reg, p.num_instr);
  if (root < 0) return false;
  // optional unary post-op
  if (p.instr[root].kind == EW_OP && !is_bin_host(p.instr[root].op)) {
    const EwInstr& u = p.instr[root];
    if (u.dtype != dt || u.sdtype != dt) return false;
    switch ((Op)u.op) {
      case Op::Tanh: case Op::Exp: case Op::Sigmoid: case Op::Silu: case Op::Relu: case Op::GeluTanh: case Op::GeluExact: case Op::Neg:
      case Op::Rsqrt: case Op::Sqrt: case Op::Abs:
        g.post = u.op;
        break;
      default: return false;
    }
    root = def_of(u.a, root);
    if (root < 0) return false;
  }
  int top_code;
  if (!binop(p.instr[root], &top_code)) return false;
  const int ia = def_of(p.instr[root].a, root), ib = def_of(p.instr[root].b, root);
  if (ia < 0 || ib < 0) return false;
  int ca, cb;
  const bool a_is_op = binop(p.instr[ia], &ca), b_is_op = binop(p.instr[ib], &cb);
  if (a_is_op && b_is_op) {
    // form B
    g.form = 1;
    g.op[0] = ca; g.op[1] = cb; g.op[2] = top_code;
    if (!make_leaf(def_of(p.instr[ia].a, ia), &g.leaf[0]) || !make_leaf(def_of(p.instr[ia].b, ia), &g.leaf[1])) return false;
    if (!make_leaf(def_of(p.instr[ib].a, ib), &g.leaf[2]) || !make_leaf(def_of(p.instr[ib].b, ib), &g.leaf[3])) return false;
  } else if (a_is_op != b_is_op) {
    // form A: inner op on one side, a leaf on the other
    g.form = 0;
    const int inner = a_is_op ? ia : ib, other = a_is_op ? ib : ia;
    g.op[0] = a_is_op ? ca : cb;
    g.op[1] = top_code;
    g.swap[1] = a_is_op ? 0 : 1;  // top = f(inner, leaf) when the inner op is the left operand, else f(leaf, inner)
    if (!make_leaf(def_of(p.instr[inner].a, inner), &g.leaf[0]) || !make_leaf(def_of(p.instr[inner].b, inner), &g.leaf[1])) return false;
    if (!make_leaf(other, &g.leaf[2])) return false;
    g.leaf[3] = TreeLeaf{nullptr, nvec, 0.f};
  } else {
    return false;
  }
  if (!al(p.out)) return false;
  g.out = reinterpret_cast<uint4*>(p.out);
  g.nvec = nvec;
  int64_t blocks = (nvec + 255) / 256;
  const int64_t cap = (int64_t)dev->sm_count() * 16;
  if (blocks > cap) blocks = cap;
  cudaStream_t s = dev->stream();
  if (dt == B200_FLOAT32) ewise_tree_fast_kernel<float><<<(unsigned)blocks, 256, 0, s>>>(g);
  else if (dt == B200_BFLOAT16) ewise_tree_fast_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, s>>>(g);
  else ewise_tree_fast_kernel<__half><<<(unsigned)blocks, 256, 0, s>>>(g);
  return true;
}

}  // namespace

Status ewise_run_fast(Device* dev, const EwProgram& prog_in, bool* taken, bool trees) {
  *taken = false;
  int64_t n = 1;
  for (int d = 0; d < prog_in.rank; ++d) n *= prog_in.dims[d];
  if (n == 0) { *taken = true; return Status::OK(); }
  B200_TRY(dev->MakeCurrent());
  if (try_binary_fast(dev, prog_in, n)) { *taken = true; return dev->CheckLaunch("ewise_binary_fast"); }
  if (trees && try_tree_fast(dev, prog_in, n)) { *taken = true; return dev->CheckLaunch("ewise_tree_fast"); }
  return Status::OK();
}

Status ewise_run(Device* dev, const EwProgram& prog_in) {
  int64_t n = 1;
  for (int d = 0; d < prog_in.rank; ++d) n *= prog_in.dims[d];
  if (n == 0) return Status::OK();
  if (prog_in.num_regs > kEwMaxRegs || prog_in.num_instr > kEwMaxInstr || prog_in.num_leaves > kEwMaxLeaves)
    return Status::Invalid("ewise: program exceeds interpreter limits");
  bool taken = false;
  B200_TRY(ewise_run_fast(dev, prog_in, &taken));
  if (taken) return Status::OK();
  if (n > 0x7fffffffLL) return Status::Unsupported("ewise: more than 2^31-1 elements in one launch");
  // pad leading dims of size 1 up to the next instantiated rank (1, 2, 3, 4 or 8)
  EwProgram prog = prog_in;
  const int r0 = prog_in.rank < 1 ? 1 : prog_in.rank;
  const int krank = r0 <= 4 ? r0 : kMaxDims;
  const int shift = krank - prog_in.rank;
  if (shift > 0) {
    for (int d = krank - 1; d >= 0; --d) {
      const int sd = d - shift;
      prog.dims[d] = sd >= 0 ? prog_in.dims[sd] : 1;
      for (int l = 0; l < prog.num_leaves; ++l) prog.leaves[l].strides[d] = sd >= 0 ? prog_in.leaves[l].strides[sd] : 0;
    }
    for (int i = 0; i < prog.num_instr; ++i)
      if (prog.instr[i].kind == EW_IOTA) prog.instr[i].a = (uint8_t)(prog.instr[i].a + shift);
    prog.rank = krank;
  }
  const int64_t inner = prog.dims[krank - 1];
  const int vec = (inner % 4 == 0) ? 4 : 1;
  const int64_t total_vecs = n / vec;
  const size_t reg_bytes = prog.wide ? 8 : 4;
  // vectors per thread: as many as the shared-memory register file allows (up to 4), fewer for small tensors
  int unroll = 4;
  while (unroll > 1 && ((size_t)prog.num_regs * unroll * kBlock * vec * reg_bytes > 64 * 1024 ||
                        total_vecs < (int64_t)kBlock * unroll * dev->sm_count() * 2))
    unroll /= 2;
  if (vec == 1 || unroll == 2) unroll = 1;
  const size_t smem = (size_t)prog.num_regs * unroll * kBlock * vec * reg_bytes;
  const int64_t per_block = (int64_t)kBlock * unroll;
  const int64_t grid64 = (total_vecs + per_block - 1) / per_block;
  cudaStream_t s = dev->stream();
#define LAUNCH(R, V, UU, RK)                                                                                       \
  do {                                                                                                             \
    if (smem > 48 * 1024)                                                                                          \
      B200_CUDA_TRY(cudaFuncSetAttribute(ewise_kernel<R, V, UU, RK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
    ewise_kernel<R, V, UU, RK><<<(unsigned)grid64, kBlock, smem, s>>>(prog, total_vecs);                           \
  } while (0)
#define LAUNCH_RK(R, V, UU)                                               \
  do {                                                                    \
    switch (krank) {                                                      \
      case 1: LAUNCH(R, V, UU, 1); break;                                 \
      case 2: LAUNCH(R, V, UU, 2); break;                                 \
      case 3: LAUNCH(R, V, UU, 3); break;                                 \
      case 4: LAUNCH(R, V, UU, 4); break;                                 \
      default: LAUNCH(R, V, UU, 8); break;                                \
    }                                                                     \
  } while (0)
#define LAUNCH_U(R)                                                       \
  do {                                                                    \
    if (vec == 1) LAUNCH_RK(R, 1, 1);                                     \
    else if (unroll == 4) LAUNCH_RK(R, 4, 4);                             \
    else LAUNCH_RK(R, 4, 1);                                              \
  } while (0)
  if (prog.wide) LAUNCH_U(uint64_t);
  else LAUNCH_U(uint32_t);
#undef LAUNCH_U
#undef LAUNCH_RK
#undef LAUNCH
  return dev->CheckLaunch("ewise_kernel");
}

}  // namespace k
}  // namespace b200
