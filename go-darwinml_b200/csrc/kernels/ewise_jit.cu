// Run-time compiled kernels for fused elementwise chains (and, through the same generated body, for reductions whose
// operand is such a chain).
//
// The lowering pass hands over a straight-line program (EwProgram: loads through broadcast / permute / slice strides of
// the output index space, iotas, immediates, unary / binary / compare / select / clamp / cast instructions).  The
// interpreter kernel of ewise.cu decodes that program for every element; here the program is turned into CUDA C once,
// at b200_compile time, compiled with NVRTC for sm_100a and cached by its source text:
//   * every instruction becomes one statement over real registers, calling the SAME op functions (ewise_ops.cuh) with
//     literal op codes and dtypes, so the result is the interpreter's, op by op (NVRTC runs with --fmad=false so that
//     separate ops are never contracted into one);
//   * the output shape and every leaf's strides are literals: index arithmetic is multiply-shift, dense leaves use the
//     linear index, broadcast dims cost nothing;
//   * a thread owns VEC consecutive elements (16 bytes of the narrowest dense operand) of UNR vectors: dense leaves and
//     the result move as 128-bit accesses, a leaf that is constant along the last axis is loaded once per vector.
// The reference leaves fusion to Apple's graph compiler (mpsgraph function.go:658-963 issues one graph op per primitive).
//
// NVRTC is looked up at run time (dlopen); when it is missing, or a compile fails, the caller keeps using the
// interpreter kernel, which needs nothing but this library.
#include <cuda_fp16.h>
#include <dlfcn.h>

#include <cstring>

#include <mutex>
#include <sstream>
#include <unordered_map>

#include "../kernels.h"

namespace b200 {
namespace k {

namespace {

// The text of ewise_ops.cuh, generated next to the objects by the build script.
const char* const kOpsSource =
#include "ewise_ops_src.inc"
    ;

// ------------------------------------------------------------------------------------------------ NVRTC, by dlopen ---
struct Nvrtc {
  void* handle = nullptr;
  int (*CreateProgram)(void**, const char*, const char*, int, const char* const*, const char* const*) = nullptr;
  int (*CompileProgram)(void*, int, const char* const*) = nullptr;
  int (*GetProgramLogSize)(void*, size_t*) = nullptr;
  int (*GetProgramLog)(void*, char*) = nullptr;
  int (*GetCUBINSize)(void*, size_t*) = nullptr;
  int (*GetCUBIN)(void*, char*) = nullptr;
  int (*DestroyProgram)(void**) = nullptr;
  const char* (*GetErrorString)(int) = nullptr;
  std::string why;   // why it is unavailable
};

Nvrtc* nvrtc() {
  static Nvrtc n;
  static std::once_flag once;
  std::call_once(once, [] {
    const char* env = getenv("B200MLX_NVRTC");
    const char* names[] = {env, "libnvrtc.so.12", "/usr/local/cuda/lib64/libnvrtc.so.12", "libnvrtc.so", "/usr/local/cuda/lib64/libnvrtc.so"};
    for (const char* name : names) {
      if (!name || !*name) continue;
      n.handle = dlopen(name, RTLD_NOW | RTLD_LOCAL);
      if (n.handle) break;
    }
    if (!n.handle) { n.why = "libnvrtc.so.12 not found (set B200MLX_NVRTC to its path)"; return; }
    auto sym = [&](const char* s) { return dlsym(n.handle, s); };
    n.CreateProgram = reinterpret_cast<decltype(n.CreateProgram)>(sym("nvrtcCreateProgram"));
    n.CompileProgram = reinterpret_cast<decltype(n.CompileProgram)>(sym("nvrtcCompileProgram"));
    n.GetProgramLogSize = reinterpret_cast<decltype(n.GetProgramLogSize)>(sym("nvrtcGetProgramLogSize"));
    n.GetProgramLog = reinterpret_cast<decltype(n.GetProgramLog)>(sym("nvrtcGetProgramLog"));
    n.GetCUBINSize = reinterpret_cast<decltype(n.GetCUBINSize)>(sym("nvrtcGetCUBINSize"));
    n.GetCUBIN = reinterpret_cast<decltype(n.GetCUBIN)>(sym("nvrtcGetCUBIN"));
    n.DestroyProgram = reinterpret_cast<decltype(n.DestroyProgram)>(sym("nvrtcDestroyProgram"));
    n.GetErrorString = reinterpret_cast<decltype(n.GetErrorString)>(sym("nvrtcGetErrorString"));
    if (!n.CreateProgram || !n.CompileProgram || !n.GetProgramLogSize || !n.GetProgramLog || !n.GetCUBINSize || !n.GetCUBIN ||
        !n.DestroyProgram || !n.GetErrorString) {
      n.why = "libnvrtc lacks an expected entry point";
      n.handle = nullptr;
    }
  });
  return &n;
}

// ------------------------------------------------------------------------------------------------- code generation ---
const char* kDtypeConst[] = {"B200_BOOL", "B200_INT8", "B200_INT16", "B200_INT32", "B200_INT64", "B200_FLOAT16", "B200_BFLOAT16",
                             "B200_FLOAT32", "B200_FLOAT64", "B200_UINT8", "B200_UINT16", "B200_UINT32", "B200_UINT64"};

// What the including translation unit gives ewise_ops.cuh under nvcc: integer typedefs, dtype constants, the op enum.
std::string Preamble() {
  std::ostringstream o;
  o << "typedef signed char int8_t; typedef short int16_t; typedef int int32_t; typedef long long int64_t;\n"
       "typedef unsigned char uint8_t; typedef unsigned short uint16_t; typedef unsigned int uint32_t; typedef unsigned long long uint64_t;\n"
       "typedef unsigned long long uintptr_t;\n";
  o << "enum {";
  for (int d = 0; d <= 12; ++d) o << kDtypeConst[d] << " = " << d << (d < 12 ? ", " : "");
  o << "};\nenum class Op : int {";
  for (int i = 0; i < (int)Op::kNumOps; ++i) o << op_name((Op)i) << ", ";
  o << "kNumOps};\n";
  o << "__device__ __forceinline__ int dtype_size(int dt) {\n"
       "  switch (dt) {\n"
       "    case B200_BOOL: case B200_INT8: case B200_UINT8: return 1;\n"
       "    case B200_INT16: case B200_UINT16: case B200_FLOAT16: case B200_BFLOAT16: return 2;\n"
       "    case B200_INT32: case B200_UINT32: case B200_FLOAT32: return 4;\n"
       "    default: return 8;\n"
       "  }\n"
       "}\n"
       "__device__ __forceinline__ bool dtype_is_float(int dt) {\n"
       "  return dt == B200_FLOAT16 || dt == B200_BFLOAT16 || dt == B200_FLOAT32 || dt == B200_FLOAT64;\n"
       "}\n";
  return o.str();
}

// Helpers of the generated kernels that sit on top of ewise_ops.cuh: raw element bits <-> register representation.
const char* const kGlue = R"GLUE(
template <typename R> __device__ __forceinline__ R ew_from_raw(uint64_t bits, int dt) {
  switch (dt) {
    case B200_BFLOAT16: return (R)((uint32_t)bits << 16);
    case B200_FLOAT16: return from_f<R>(ew_f16_to_f((uint16_t)bits));
    case B200_INT8: return (R)(uint32_t)(int32_t)(int8_t)bits;
    case B200_INT16: return (R)(uint32_t)(int32_t)(int16_t)bits;
    case B200_BOOL: return (R)((bits & 0xff) ? 1u : 0u);
    default: return (R)bits;   // 32- and 64-bit types, U8, U16: the bits themselves
  }
}
template <typename R> __device__ __forceinline__ uint64_t ew_to_raw(R r, int dt) {
  switch (dt) {
    case B200_BFLOAT16: return ew_f_to_bf16(as_f(r));
    case B200_FLOAT16: return ew_f_to_f16(as_f(r));
    case B200_BOOL: return r ? 1 : 0;
    case B200_INT8: case B200_UINT8: return (uint64_t)r & 0xff;
    case B200_INT16: case B200_UINT16: return (uint64_t)r & 0xffff;
    case B200_INT32: case B200_UINT32: case B200_FLOAT32: return (uint64_t)r & 0xffffffffull;
    default: return (uint64_t)r;
  }
}
// Two 16-bit float results as one 32-bit word (low half first).  The registers already hold values of the 16-bit type
// (every op rounds), so bf16 is a matter of taking the upper halves; f16 takes one packed conversion.
template <typename R> __device__ __forceinline__ uint32_t ew_pack_pair(R a, R b, int dt) {
  if (dt == B200_BFLOAT16) return ((uint32_t)a >> 16) | ((uint32_t)b & 0xffff0000u);
  uint32_t p;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(p) : "f"(as_f(b)), "f"(as_f(a)));
  return p;
}
// ---- packed mode: a chain whose every value is of ONE 16-bit float type keeps two elements per 32-bit register (low
// half = the even element).  Add / Sub / Mul / Max / Min / Neg / Abs are single packed instructions with one IEEE
// rounding of the exact result; every other op unpacks to fp32, computes as the unpacked path does, and repacks with
// one packed conversion.  Loads and stores move the registers as they are.
__device__ __forceinline__ float ew_p2_lo(uint32_t p, int dt) { return dt == B200_BFLOAT16 ? __uint_as_float(p << 16) : ew_f16_to_f((uint16_t)(p & 0xffffu)); }
__device__ __forceinline__ float ew_p2_hi(uint32_t p, int dt) { return dt == B200_BFLOAT16 ? __uint_as_float(p & 0xffff0000u) : ew_f16_to_f((uint16_t)(p >> 16)); }
__device__ __forceinline__ uint32_t ew_p2_pack(float lo, float hi, int dt) {
  uint32_t p;
  if (dt == B200_BFLOAT16) asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(p) : "f"(hi), "f"(lo));
  else asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(p) : "f"(hi), "f"(lo));
  return p;
}
#define EW_P2_BIN(NAME, BF, HF)                                                                       \
  __device__ __forceinline__ uint32_t NAME(uint32_t a, uint32_t b, int dt) {                          \
    uint32_t r;                                                                                       \
    if (dt == B200_BFLOAT16) asm(BF " %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));                      \
    else asm(HF " %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));                                          \
    return r;                                                                                         \
  }
EW_P2_BIN(ew_p2_add, "add.rn.bf16x2", "add.rn.f16x2")
EW_P2_BIN(ew_p2_sub, "sub.rn.bf16x2", "sub.rn.f16x2")
EW_P2_BIN(ew_p2_mul, "mul.rn.bf16x2", "mul.rn.f16x2")
EW_P2_BIN(ew_p2_max, "max.NaN.bf16x2", "max.NaN.f16x2")
EW_P2_BIN(ew_p2_min, "min.NaN.bf16x2", "min.NaN.f16x2")
__device__ __forceinline__ uint32_t ew_p2_op(int op, int dt, uint32_t a, uint32_t b, uint32_t c) {
  switch ((Op)op) {
    case Op::Add: return ew_p2_add(a, b, dt);
    case Op::Sub: return ew_p2_sub(a, b, dt);
    case Op::Mul: return ew_p2_mul(a, b, dt);
    case Op::Max: return ew_p2_max(a, b, dt);
    case Op::Min: return ew_p2_min(a, b, dt);
    case Op::Neg: return a ^ 0x80008000u;
    case Op::Abs: return a & 0x7fff7fffu;
    case Op::Identity: return a;
    default: {
      const float lo = as_f(eval_op_unrounded<uint32_t>(op, dt, from_f<uint32_t>(ew_p2_lo(a, dt)), from_f<uint32_t>(ew_p2_lo(b, dt)),
                                                        from_f<uint32_t>(ew_p2_lo(c, dt))));
      const float hi = as_f(eval_op_unrounded<uint32_t>(op, dt, from_f<uint32_t>(ew_p2_hi(a, dt)), from_f<uint32_t>(ew_p2_hi(b, dt)),
                                                        from_f<uint32_t>(ew_p2_hi(c, dt))));
      return ew_p2_pack(lo, hi, dt);
    }
  }
}
template <typename R> __device__ __forceinline__ R ew_iota(long long coord, int dt) {
  if (dt == B200_FLOAT64) return (R)from_d((double)coord);
  if (dtype_is_float(dt)) return from_f<R>(round_to(dt, (float)coord));
  if (dt == B200_INT64 || dt == B200_UINT64) return (R)(uint64_t)coord;
  return (R)wrap_i32(dt, (uint32_t)coord);
}
struct EwPtrs { const void* leaf[8]; void* out; };

// ---- reductions: accumulator types and combination rules of reduce.cu (fp32 for 16/32-bit floats, f64 for F64, the
// 32/64-bit integer of matching signedness for integers and Bool; float max / min propagate NaN) ----
template <typename A> struct RdAcc;
template <> struct RdAcc<float> {
  template <typename R> static __device__ __forceinline__ float in(R r, int) { return as_f(r); }
  template <typename R> static __device__ __forceinline__ R out(float a, int dt) { return from_f<R>(round_to(dt, a)); }
  static __device__ __forceinline__ float lowest() { return -ew_inf(); }
  static __device__ __forceinline__ float highest() { return ew_inf(); }
  static constexpr bool is_float = true;
};
template <> struct RdAcc<double> {
  template <typename R> static __device__ __forceinline__ double in(R r, int) { return as_d((uint64_t)r); }
  template <typename R> static __device__ __forceinline__ R out(double a, int) { return (R)from_d(a); }
  static __device__ __forceinline__ double lowest() { return -(double)ew_inf(); }
  static __device__ __forceinline__ double highest() { return (double)ew_inf(); }
  static constexpr bool is_float = true;
};
template <> struct RdAcc<int32_t> {
  template <typename R> static __device__ __forceinline__ int32_t in(R r, int) { return (int32_t)(uint32_t)r; }
  template <typename R> static __device__ __forceinline__ R out(int32_t a, int dt) { return (R)wrap_i32(dt, (uint32_t)a); }
  static __device__ __forceinline__ int32_t lowest() { return (int32_t)0x80000000u; }
  static __device__ __forceinline__ int32_t highest() { return 0x7fffffff; }
  static constexpr bool is_float = false;
};
template <> struct RdAcc<uint32_t> {
  template <typename R> static __device__ __forceinline__ uint32_t in(R r, int) { return (uint32_t)r; }
  template <typename R> static __device__ __forceinline__ R out(uint32_t a, int dt) { return (R)wrap_i32(dt == B200_BOOL ? B200_UINT8 : dt, a); }
  static __device__ __forceinline__ uint32_t lowest() { return 0u; }
  static __device__ __forceinline__ uint32_t highest() { return 0xffffffffu; }
  static constexpr bool is_float = false;
};
template <> struct RdAcc<int64_t> {
  template <typename R> static __device__ __forceinline__ int64_t in(R r, int) { return (int64_t)(uint64_t)r; }
  template <typename R> static __device__ __forceinline__ R out(int64_t a, int) { return (R)(uint64_t)a; }
  static __device__ __forceinline__ int64_t lowest() { return (int64_t)0x8000000000000000ull; }
  static __device__ __forceinline__ int64_t highest() { return 0x7fffffffffffffffll; }
  static constexpr bool is_float = false;
};
template <> struct RdAcc<uint64_t> {
  template <typename R> static __device__ __forceinline__ uint64_t in(R r, int) { return (uint64_t)r; }
  template <typename R> static __device__ __forceinline__ R out(uint64_t a, int) { return (R)a; }
  static __device__ __forceinline__ uint64_t lowest() { return 0ull; }
  static __device__ __forceinline__ uint64_t highest() { return 0xffffffffffffffffull; }
  static constexpr bool is_float = false;
};
template <typename A> __device__ __forceinline__ A rd_identity(int rt) {
  return rt == 0 ? (A)0 : rt == 1 ? (A)1 : rt == 2 ? RdAcc<A>::lowest() : RdAcc<A>::highest();
}
template <typename A> __device__ __forceinline__ A rd_combine(int rt, A a, A b) {
  if (rt == 0) return a + b;
  if (rt == 1) return a * b;
  if (RdAcc<A>::is_float && (a != a || b != b)) return a + b;
  return rt == 2 ? (a > b ? a : b) : (a < b ? a : b);
}
template <typename A> __device__ __forceinline__ A rd_shfl_xor(A v, int o) {
  if (sizeof(A) == 8) {
    long long x = *reinterpret_cast<long long*>(&v);
    x = __shfl_xor_sync(0xffffffffu, x, o);
    return *reinterpret_cast<A*>(&x);
  } else {
    int x = *reinterpret_cast<int*>(&v);
    x = __shfl_xor_sync(0xffffffffu, x, o);
    return *reinterpret_cast<A*>(&x);
  }
}
template <typename A> __device__ __forceinline__ A rd_warp(int rt, A v) {
  _Pragma("unroll") for (int o = 16; o > 0; o >>= 1) v = rd_combine<A>(rt, v, rd_shfl_xor<A>(v, o));
  return v;
}
)GLUE";

bool IsBinOp(int op) { return op >= (int)Op::Add && op <= (int)Op::ShiftRightLogical; }
bool IsCmpOp(int op) { return op >= (int)Op::Equal && op <= (int)Op::GreaterOrEqual; }

struct LeafPlan {
  enum Kind { kDense, kVector, kBroadcast, kStrided } kind = kStrided;
  bool wide_offset = false;   // offsets need 64 bits
  int64_t last_stride = 0;
};

struct GenConfig {
  int vec = 1;        // elements per thread and vector
  int unroll = 1;     // vectors per thread
  bool wide_index = false;   // more than 2^32 - 1 elements
  bool packed = false;       // every value is of one 16-bit float type: two elements per register
  int packed_dtype = 0;
};

// Packed mode applies when every leaf, every instruction and the result are of the same 16-bit float type and no
// instruction produces or consumes anything else (compares, selects, casts, integer iotas keep the unpacked form).
bool CanPack(const EwProgram& p, int* dtype) {
  const int dt = p.out_dtype;
  if (dt != B200_BFLOAT16 && dt != B200_FLOAT16) return false;
  for (int l = 0; l < p.num_leaves; ++l)
    if (p.leaves[l].dtype != dt) return false;
  for (int i = 0; i < p.num_instr; ++i) {
    const EwInstr& in = p.instr[i];
    if (in.dtype != dt || in.sdtype != dt) return false;
    if (in.kind == EW_CAST) return false;
    if (in.kind == EW_OP) {
      const int op = in.op;
      if ((op >= (int)Op::Equal && op <= (int)Op::GreaterOrEqual) || op == (int)Op::Where || op == (int)Op::IsFinite || op == (int)Op::IsNaN)
        return false;
    }
  }
  *dtype = dt;
  return true;
}
uint32_t FloatBitsTo16(uint32_t float_bits, int dt) {   // host: a value already representable in the 16-bit type
  if (dt == B200_BFLOAT16) return float_bits >> 16;
  float f;
  memcpy(&f, &float_bits, 4);
  const __half h = __float2half_rn(f);
  uint16_t b;
  memcpy(&b, &h, 2);
  return b;
}

int64_t NumElements(const EwProgram& p) {
  int64_t n = 1;
  for (int d = 0; d < p.rank; ++d) n *= p.dims[d];
  return n;
}

LeafPlan PlanLeaf(const EwProgram& p, const EwLeaf& lf, int vec) {
  LeafPlan lp;
  const int last = p.rank - 1;
  lp.last_stride = lf.strides[last];
  int64_t acc = 1, max_off = 0;
  bool dense = true, other_multiple = true;
  for (int d = last; d >= 0; --d) {
    if (p.dims[d] != 1 && lf.strides[d] != acc) dense = false;
    if (d != last && lf.strides[d] % vec != 0) other_multiple = false;
    const int64_t s = lf.strides[d] < 0 ? -lf.strides[d] : lf.strides[d];
    max_off += (p.dims[d] - 1) * s;
    acc *= p.dims[d];
  }
  lp.wide_offset = max_off >= 0x7fffffffLL;
  if (dense) lp.kind = LeafPlan::kDense;
  else if (lp.last_stride == 1 && other_multiple) lp.kind = LeafPlan::kVector;
  else if (lp.last_stride == 0) lp.kind = LeafPlan::kBroadcast;
  else lp.kind = LeafPlan::kStrided;
  if (vec == 1 && lp.kind == LeafPlan::kVector) lp.kind = LeafPlan::kStrided;
  return lp;
}

// Emits `n` contiguous bytes at byte pointer expression `ptr` loaded into uint32_t words named w<tag>[]; n is 1, 2, 4, 8 or
// a multiple of 16.
void EmitVectorLoad(std::ostringstream& o, const std::string& ptr, int nbytes, const std::string& w) {
  const int words = nbytes >= 4 ? nbytes / 4 : 1;
  o << "        uint32_t " << w << "[" << words << "];\n";
  if (nbytes >= 16) {
    for (int i = 0; i < nbytes / 16; ++i)
      o << "        { const uint4 q = reinterpret_cast<const uint4*>(" << ptr << ")[" << i << "]; " << w << "[" << 4 * i << "] = q.x; " << w << "["
        << 4 * i + 1 << "] = q.y; " << w << "[" << 4 * i + 2 << "] = q.z; " << w << "[" << 4 * i + 3 << "] = q.w; }\n";
  } else if (nbytes == 8) {
    o << "        { const uint2 q = *reinterpret_cast<const uint2*>(" << ptr << "); " << w << "[0] = q.x; " << w << "[1] = q.y; }\n";
  } else if (nbytes == 4) {
    o << "        " << w << "[0] = *reinterpret_cast<const uint32_t*>(" << ptr << ");\n";
  } else if (nbytes == 2) {
    o << "        " << w << "[0] = *reinterpret_cast<const uint16_t*>(" << ptr << ");\n";
  } else {
    o << "        " << w << "[0] = *reinterpret_cast<const uint8_t*>(" << ptr << ");\n";
  }
}
// Expression for the raw bits of element v (of elt bytes) inside words w[].
std::string RawElem(const std::string& w, int v, int elt) {
  std::ostringstream o;
  if (elt == 8) o << "((uint64_t)" << w << "[" << 2 * v << "] | ((uint64_t)" << w << "[" << 2 * v + 1 << "] << 32))";
  else if (elt == 4) o << "(uint64_t)" << w << "[" << v << "]";
  else if (elt == 2) o << "(uint64_t)((" << w << "[" << v / 2 << "] >> " << 16 * (v % 2) << ") & 0xffffu)";
  else o << "(uint64_t)((" << w << "[" << v / 4 << "] >> " << 8 * (v % 4) << ") & 0xffu)";
  return o.str();
}

// The statements that compute every register of the program for the vectors vi[u] (u < UNR, guarded by live[u]); the result
// is left in r<out_reg>[u][v].  Shared by the elementwise and the reduction skeletons.
void EmitBody(std::ostringstream& o, const EwProgram& p, const GenConfig& cfg) {
  const int last = p.rank - 1;
  const char* idx_t = cfg.wide_index ? "uint64_t" : "uint32_t";
  // multi-index of the first element of each vector
  o << "      " << idx_t << " ix[UNR][" << p.rank << "];\n";
  o << "      _Pragma(\"unroll\") for (int u = 0; u < UNR; ++u) {\n";
  o << "        " << idx_t << " rem = vi[u] * VEC;\n";
  const char* sfx = cfg.wide_index ? "ull" : "u";
  for (int d = last; d > 0; --d) {
    o << "        { const " << idx_t << " q = rem / " << p.dims[d] << sfx << "; ix[u][" << d << "] = rem - q * " << p.dims[d] << sfx << "; rem = q; }\n";
  }
  o << "        ix[u][0] = rem;\n      }\n";
  if (cfg.packed) {
    for (int r = 0; r < p.num_regs; ++r) o << "      uint32_t r" << r << "[UNR][VEC / 2];\n";
  } else {
    for (int r = 0; r < p.num_regs; ++r) o << "      R r" << r << "[UNR][VEC];\n";
  }
  for (int pc = 0; pc < p.num_instr; ++pc) {
    const EwInstr& in = p.instr[pc];
    if (cfg.packed) {
      const int dt = cfg.packed_dtype;
      o << "      // " << pc << " (packed)\n";
      o << "      _Pragma(\"unroll\") for (int u = 0; u < UNR; ++u) {\n        if (!live[u]) continue;\n";
      if (in.kind == EW_LOAD) {
        const EwLeaf& lf = p.leaves[in.a];
        const LeafPlan lp = PlanLeaf(p, lf, cfg.vec);
        const char* off_t = lp.wide_offset || cfg.wide_index ? "long long" : "int";
        std::ostringstream off;
        if (lp.kind == LeafPlan::kDense) {
          off << "(" << (cfg.wide_index ? "long long" : "unsigned") << ")(vi[u] * VEC)";
        } else {
          off << "(";
          bool any = false;
          for (int d = 0; d < p.rank; ++d) {
            if (lf.strides[d] == 0 || p.dims[d] == 1) continue;
            off << (any ? " + " : "") << "(" << off_t << ")ix[u][" << d << "] * (" << off_t << ")" << lf.strides[d] << "ll";
            any = true;
          }
          if (!any) off << "0";
          off << ")";
        }
        const std::string base = "reinterpret_cast<const uint16_t*>(P.leaf[" + std::to_string(in.a) + "])";
        if (lp.kind == LeafPlan::kDense || lp.kind == LeafPlan::kVector) {
          o << "        const unsigned char* src = reinterpret_cast<const unsigned char*>(" << base << " + (long long)" << off.str() << ");\n";
          EmitVectorLoad(o, "src", cfg.vec * 2, "w");
          for (int i = 0; i < cfg.vec / 2; ++i) o << "        r" << (int)in.dst << "[u][" << i << "] = w[" << i << "];\n";
        } else if (lp.kind == LeafPlan::kBroadcast) {
          o << "        const uint32_t x = " << base << "[(long long)" << off.str() << "];\n";
          o << "        _Pragma(\"unroll\") for (int i = 0; i < VEC / 2; ++i) r" << (int)in.dst << "[u][i] = x | (x << 16);\n";
        } else {
          o << "        const long long off = (long long)" << off.str() << ";\n";
          o << "        _Pragma(\"unroll\") for (int i = 0; i < VEC / 2; ++i) r" << (int)in.dst << "[u][i] = (uint32_t)" << base << "[off + (2 * i) * "
            << lp.last_stride << "ll] | ((uint32_t)" << base << "[off + (2 * i + 1) * " << lp.last_stride << "ll] << 16);\n";
        }
      } else if (in.kind == EW_IMM) {
        const uint32_t h = FloatBitsTo16((uint32_t)in.imm, dt);
        o << "        _Pragma(\"unroll\") for (int i = 0; i < VEC / 2; ++i) r" << (int)in.dst << "[u][i] = 0x" << std::hex << (h | (h << 16)) << std::dec << "u;\n";
      } else if (in.kind == EW_IOTA) {
        o << "        _Pragma(\"unroll\") for (int i = 0; i < VEC / 2; ++i) r" << (int)in.dst << "[u][i] = ew_p2_pack((float)((long long)ix[u][" << (int)in.a
          << "]" << ((int)in.a == last ? " + 2 * i" : "") << "), (float)((long long)ix[u][" << (int)in.a << "]" << ((int)in.a == last ? " + 2 * i + 1" : "")
          << "), " << dt << ");\n";
      } else {
        const int op = in.op;
        const bool three = op == (int)Op::Clamp;
        const bool two = three || IsBinOp(op);
        o << "        _Pragma(\"unroll\") for (int i = 0; i < VEC / 2; ++i) r" << (int)in.dst << "[u][i] = ew_p2_op(" << op << ", " << dt << ", r"
          << (int)in.a << "[u][i], " << (two ? "r" + std::to_string((int)in.b) + "[u][i]" : std::string("0u")) << ", "
          << (three ? "r" + std::to_string((int)in.c) + "[u][i]" : std::string("0u")) << ");\n";
      }
      o << "      }\n";
      continue;
    }
    o << "      // " << pc << "\n";
    o << "      _Pragma(\"unroll\") for (int u = 0; u < UNR; ++u) {\n        if (!live[u]) continue;\n";
    switch (in.kind) {
      case EW_LOAD: {
        const EwLeaf& lf = p.leaves[in.a];
        const LeafPlan lp = PlanLeaf(p, lf, cfg.vec);
        const int elt = dtype_size(lf.dtype);
        const char* off_t = lp.wide_offset || cfg.wide_index ? "long long" : "int";
        std::ostringstream off;
        if (lp.kind == LeafPlan::kDense) {
          off << "(" << (cfg.wide_index ? "long long" : "unsigned") << ")(vi[u] * VEC)";
        } else {
          off << "(";
          bool any = false;
          for (int d = 0; d < p.rank; ++d) {
            if (lf.strides[d] == 0 || p.dims[d] == 1) continue;
            off << (any ? " + " : "") << "(" << off_t << ")ix[u][" << d << "] * (" << off_t << ")" << lf.strides[d] << "ll";
            any = true;
          }
          if (!any) off << "0";
          off << ")";
        }
        const std::string base = "reinterpret_cast<const unsigned char*>(P.leaf[" + std::to_string(in.a) + "])";
        if (lp.kind == LeafPlan::kDense || lp.kind == LeafPlan::kVector) {
          o << "        const unsigned char* src = " << base << " + (long long)" << off.str() << " * " << elt << ";\n";
          if (cfg.vec == 1) {
            o << "        r" << (int)in.dst << "[u][0] = load_elem<R>(src, 0, " << lf.dtype << ");\n";
          } else {
            EmitVectorLoad(o, "src", cfg.vec * elt, "w");
            for (int v = 0; v < cfg.vec; ++v)
              o << "        r" << (int)in.dst << "[u][" << v << "] = ew_from_raw<R>(" << RawElem("w", v, elt) << ", " << lf.dtype << ");\n";
          }
        } else if (lp.kind == LeafPlan::kBroadcast) {
          o << "        const R x = load_elem<R>(" << base << ", (long long)" << off.str() << ", " << lf.dtype << ");\n";
          o << "        _Pragma(\"unroll\") for (int v = 0; v < VEC; ++v) r" << (int)in.dst << "[u][v] = x;\n";
        } else {
          o << "        const long long off = (long long)" << off.str() << ";\n";
          o << "        _Pragma(\"unroll\") for (int v = 0; v < VEC; ++v) r" << (int)in.dst << "[u][v] = load_elem<R>(" << base << ", off + v * "
            << lp.last_stride << "ll, " << lf.dtype << ");\n";
        }
        break;
      }
      case EW_IMM:
        o << "        _Pragma(\"unroll\") for (int v = 0; v < VEC; ++v) r" << (int)in.dst << "[u][v] = (R)0x" << std::hex << in.imm << std::dec << "ull;\n";
        break;
      case EW_IOTA:
        o << "        _Pragma(\"unroll\") for (int v = 0; v < VEC; ++v) r" << (int)in.dst << "[u][v] = ew_iota<R>((long long)ix[u][" << (int)in.a << "]"
          << ((int)in.a == last ? " + v" : "") << ", " << (int)in.dtype << ");\n";
        break;
      case EW_CAST:
        o << "        _Pragma(\"unroll\") for (int v = 0; v < VEC; ++v) r" << (int)in.dst << "[u][v] = eval_cast_core<R>(" << (int)in.sdtype << ", "
          << (int)in.dtype << ", r" << (int)in.a << "[u][v]);\n";
        break;
      default: {
        const int op = in.op;
        const bool three = op == (int)Op::Where || op == (int)Op::Clamp;
        const bool two = three || IsBinOp(op) || IsCmpOp(op);
        // a 16-bit float result is rounded after the op: two elements per packed conversion
        const bool is16 = in.dtype == B200_BFLOAT16 || in.dtype == B200_FLOAT16;
        const bool float_result = !IsCmpOp(op) && op != (int)Op::IsFinite && op != (int)Op::IsNaN && op != (int)Op::Where;
        const bool pair = is16 && float_result && cfg.vec % 2 == 0 && (in.sdtype == B200_BFLOAT16 || in.sdtype == B200_FLOAT16);
        auto call = [&](const char* fn, const std::string& v) {
          std::ostringstream c;
          c << fn << "<R>(" << op << ", " << (int)in.sdtype << ", r" << (int)in.a << "[u][" << v << "], ";
          if (two) c << "r" << (int)in.b << "[u][" << v << "], "; else c << "(R)0, ";
          if (three) c << "r" << (int)in.c << "[u][" << v << "])"; else c << "(R)0)";
          return c.str();
        };
        if (pair) {
          o << "        _Pragma(\"unroll\") for (int v = 0; v < VEC; v += 2) {\n";
          o << "          float t0 = as_f(" << call("eval_op_unrounded", "v") << "), t1 = as_f(" << call("eval_op_unrounded", "v + 1") << ");\n";
          o << "          ew_round_pair(" << (int)in.dtype << ", t0, t1);\n";
          o << "          r" << (int)in.dst << "[u][v] = from_f<R>(t0); r" << (int)in.dst << "[u][v + 1] = from_f<R>(t1);\n        }\n";
        } else {
          o << "        _Pragma(\"unroll\") for (int v = 0; v < VEC; ++v) r" << (int)in.dst << "[u][v] = " << call("eval_op_core", "v") << ";\n";
        }
        break;
      }
    }
    o << "      }\n";
  }
}

GenConfig ChooseConfig(const EwProgram& p, int sm_count, bool allow_vector) {
  GenConfig cfg;
  const int64_t n = NumElements(p);
  cfg.wide_index = n > 0xffffffffLL;
  int min_elt = dtype_size(p.out_dtype);
  for (int l = 0; l < p.num_leaves; ++l) min_elt = dtype_size(p.leaves[l].dtype) < min_elt ? dtype_size(p.leaves[l].dtype) : min_elt;
  int vec = 16 / min_elt;
  if (vec > 8) vec = 8;
  // wide programs hold 64-bit registers: halve the vector so the register file is not swamped
  if (p.wide && vec > 2) vec = dtype_size(p.out_dtype) == 8 ? 2 : 4;
  const int64_t inner = p.dims[p.rank - 1];
  while (vec > 1 && inner % vec != 0) vec /= 2;
  if (!allow_vector) vec = 1;
  cfg.vec = vec;
  cfg.packed = vec >= 2 && CanPack(p, &cfg.packed_dtype);
  const int64_t nvec = n / vec;
  cfg.unroll = (vec > 1 && p.num_regs * vec <= (cfg.packed ? 96 : 48) && nvec >= (int64_t)sm_count * 256 * 8) ? 2 : 1;
  return cfg;
}

}  // namespace

std::string ewise_jit_source(const EwProgram& p, int sm_count, bool allow_vector) {
  const GenConfig cfg = ChooseConfig(p, sm_count, allow_vector);
  const int64_t nvec = NumElements(p) / cfg.vec;
  const char* idx_t = cfg.wide_index ? "uint64_t" : "uint32_t";
  std::ostringstream o;
  o << Preamble() << kOpsSource << kGlue;
  o << "typedef " << (p.wide ? "uint64_t" : "uint32_t") << " R;\n";
  o << "#define VEC " << cfg.vec << "\n#define UNR " << cfg.unroll << "\n";
  o << "extern \"C\" __global__ void __launch_bounds__(256) ew_kernel(const EwPtrs P) {\n";
  o << "  const " << idx_t << " nvec = " << nvec << "ull;\n";
  o << "  for (" << idx_t << " base = (" << idx_t << ")blockIdx.x * (256 * UNR); base < nvec; base += (" << idx_t << ")gridDim.x * (256 * UNR)) {\n";
  o << "      " << idx_t << " vi[UNR];\n      bool live[UNR];\n";
  o << "      _Pragma(\"unroll\") for (int u = 0; u < UNR; ++u) { vi[u] = base + u * 256 + threadIdx.x; live[u] = vi[u] < nvec; }\n";
  EmitBody(o, p, cfg);
  // store
  const int elt = dtype_size(p.out_dtype);
  o << "      _Pragma(\"unroll\") for (int u = 0; u < UNR; ++u) {\n        if (!live[u]) continue;\n";
  if (cfg.vec == 1) {
    o << "        store_elem<R>(P.out, (long long)vi[u], " << p.out_dtype << ", r" << p.out_reg << "[u][0]);\n";
  } else {
    const int nbytes = cfg.vec * elt;
    const int words = nbytes >= 4 ? nbytes / 4 : 1;
    o << "        uint32_t w[" << words << "];\n";
    for (int wi = 0; wi < words; ++wi) {
      if (cfg.packed) {
        o << "        w[" << wi << "] = r" << p.out_reg << "[u][" << wi << "];\n";
        continue;
      }
      o << "        w[" << wi << "] = ";
      if (elt == 8) {
        o << "(uint32_t)(ew_to_raw<R>(r" << p.out_reg << "[u][" << wi / 2 << "], " << p.out_dtype << ") >> " << 32 * (wi % 2) << ");\n";
      } else if (elt == 2 && (p.out_dtype == B200_BFLOAT16 || p.out_dtype == B200_FLOAT16)) {
        o << "ew_pack_pair<R>(r" << p.out_reg << "[u][" << 2 * wi << "], r" << p.out_reg << "[u][" << 2 * wi + 1 << "], " << p.out_dtype << ");\n";
      } else {
        const int per = 4 / elt;
        for (int e = 0; e < per; ++e)
          o << (e ? " | " : "") << "((uint32_t)ew_to_raw<R>(r" << p.out_reg << "[u][" << wi * per + e << "], " << p.out_dtype << ") << " << 8 * elt * e << ")";
        o << ";\n";
      }
    }
    o << "        unsigned char* dst = reinterpret_cast<unsigned char*>(P.out) + (long long)(vi[u] * VEC) * " << elt << ";\n";
    if (nbytes >= 16) {
      for (int i = 0; i < nbytes / 16; ++i)
        o << "        reinterpret_cast<uint4*>(dst)[" << i << "] = make_uint4(w[" << 4 * i << "], w[" << 4 * i + 1 << "], w[" << 4 * i + 2 << "], w["
          << 4 * i + 3 << "]);\n";
    } else if (nbytes == 8) {
      o << "        *reinterpret_cast<uint2*>(dst) = make_uint2(w[0], w[1]);\n";
    } else if (nbytes == 4) {
      o << "        *reinterpret_cast<uint32_t*>(dst) = w[0];\n";
    } else {
      o << "        *reinterpret_cast<uint16_t*>(dst) = (uint16_t)w[0];\n";
    }
  }
  o << "      }\n  }\n}\n";
  return o.str();
}

Status ewise_jit_nvrtc(const std::string& source, std::vector<char>* cubin) {
  Nvrtc* n = nvrtc();
  if (!n->handle) return Status::Unsupported("run-time compilation unavailable: " + n->why);
  void* prog = nullptr;
  int rc = n->CreateProgram(&prog, source.c_str(), "ewise_chain.cu", 0, nullptr, nullptr);
  if (rc != 0) return Status::Cuda(strfmt("nvrtcCreateProgram: %s", n->GetErrorString(rc)));
  const char* opts[] = {"--gpu-architecture=sm_100a", "--std=c++17", "--fmad=false", "-default-device"};
  rc = n->CompileProgram(prog, 4, opts);
  if (rc != 0) {
    size_t len = 0;
    n->GetProgramLogSize(prog, &len);
    std::string log(len, '\0');
    if (len) n->GetProgramLog(prog, &log[0]);
    n->DestroyProgram(&prog);
    if (log.size() > 1500) log.resize(1500);
    return Status::Cuda(strfmt("nvrtcCompileProgram: %s\n%s", n->GetErrorString(rc), log.c_str()));
  }
  size_t size = 0;
  rc = n->GetCUBINSize(prog, &size);
  if (rc == 0 && size > 0) {
    cubin->resize(size);
    rc = n->GetCUBIN(prog, cubin->data());
  }
  n->DestroyProgram(&prog);
  if (rc != 0 || size == 0) return Status::Cuda("nvrtc produced no device code for sm_100a");
  return Status::OK();
}

// One compiled chain: the loaded module, its kernel and what the launcher needs to know about the specialisation.
struct EwJit {
  cudaLibrary_t lib = nullptr;
  cudaKernel_t kernel = nullptr;
  int vec = 1, unroll = 1;
  int64_t nvec = 0;
  int num_leaves = 0;
  int align_bytes[kEwMaxLeaves] = {0};   // required alignment of each leaf pointer (vector loads), 0 = none
  int out_align = 0;
  EwJit* scalar = nullptr;               // the VEC = 1 build, made on first need (a pointer that is not aligned enough)
  EwProgram prog;                        // kept for that second build
  int sm_count = 148;
  // reductions of a chain (ewise_jit_reduce_prepare)
  bool is_reduce = false;
  int reduce_type = 0;
  int64_t outer = 1, n = 1, inner = 1;
  int64_t grid_units = 0;                // CTAs wanted before the persistent cap
};

namespace {
std::mutex g_jit_mu;
std::unordered_map<std::string, EwJit*> g_jit_cache;   // source text -> kernel, for the life of the process

Status BuildJit(const EwProgram& p, int sm_count, bool allow_vector, EwJit** out) {
  const std::string src = ewise_jit_source(p, sm_count, allow_vector);
  {
    std::lock_guard<std::mutex> lock(g_jit_mu);
    auto it = g_jit_cache.find(src);
    if (it != g_jit_cache.end()) { *out = it->second; return Status::OK(); }
  }
  if (const char* dir = getenv("B200MLX_JIT_DUMP")) {
    static int serial = 0;
    const std::string path = std::string(dir) + "/ewise_chain_" + std::to_string(serial++) + ".cu";
    if (FILE* f = fopen(path.c_str(), "w")) { fputs(src.c_str(), f); fclose(f); }
  }
  std::vector<char> cubin;
  B200_TRY(ewise_jit_nvrtc(src, &cubin));
  std::unique_ptr<EwJit> j(new EwJit());
  B200_CUDA_TRY(cudaLibraryLoadData(&j->lib, cubin.data(), nullptr, nullptr, 0, nullptr, nullptr, 0));
  B200_CUDA_TRY(cudaLibraryGetKernel(&j->kernel, j->lib, "ew_kernel"));
  const GenConfig cfg = ChooseConfig(p, sm_count, allow_vector);
  j->vec = cfg.vec;
  j->unroll = cfg.unroll;
  j->nvec = NumElements(p) / cfg.vec;
  j->num_leaves = p.num_leaves;
  j->prog = p;
  j->sm_count = sm_count;
  if (cfg.vec > 1) {
    auto align_of = [](int bytes) { return bytes >= 16 ? 16 : bytes; };
    for (int l = 0; l < p.num_leaves; ++l) {
      const LeafPlan lp = PlanLeaf(p, p.leaves[l], cfg.vec);
      if (lp.kind == LeafPlan::kDense || lp.kind == LeafPlan::kVector) j->align_bytes[l] = align_of(cfg.vec * dtype_size(p.leaves[l].dtype));
    }
    j->out_align = align_of(cfg.vec * dtype_size(p.out_dtype));
  }
  std::lock_guard<std::mutex> lock(g_jit_mu);
  auto ins = g_jit_cache.emplace(src, j.get());
  if (ins.second) j.release();   // else another thread built the same text meanwhile: keep theirs, drop ours
  *out = ins.first->second;
  return Status::OK();
}
}  // namespace

Status ewise_jit_prepare(Device* dev, const EwProgram& prog, EwJit** out) {
  *out = nullptr;
  const char* off = getenv("B200MLX_JIT");
  if (off && off[0] == '0') return Status::Unsupported("run-time compilation switched off (B200MLX_JIT=0)");
  if (NumElements(prog) == 0) return Status::Unsupported("empty result");
  B200_TRY(dev->MakeCurrent());
  return BuildJit(prog, dev->sm_count(), true, out);
}

// ---------------------------------------------------------------------------------------- reductions of a chain ---
// The program's index space is [outer, n, inner] (its dims refine that split); the kernel folds over n.
//   inner == 1: a row group (one warp, or a CTA of 256 threads for long rows) walks its row in vectors, UNR vectors in
//               flight per thread, and folds by shuffle; rows are dealt to groups with a grid stride;
//   inner  > 1: a thread owns VEC neighbouring columns and walks n; neighbouring threads read neighbouring vectors.
namespace {

const char* AccType(int dtype) {
  switch (dtype) {
    case B200_FLOAT64: return "double";
    case B200_FLOAT32: case B200_BFLOAT16: case B200_FLOAT16: return "float";
    case B200_INT8: case B200_INT16: case B200_INT32: return "int32_t";
    case B200_INT64: return "int64_t";
    case B200_UINT64: return "uint64_t";
    default: return "uint32_t";   // U8 U16 U32 Bool
  }
}

struct ReduceGeom {
  int64_t outer = 1, n = 1, inner = 1;
  int vec = 1, unroll = 1, tpr = 32;   // tpr: threads per row (inner == 1)
  bool rows = true;                    // inner == 1
};

ReduceGeom ChooseReduce(const EwProgram& p, int64_t outer, int64_t n, int64_t inner, bool allow_vector) {
  ReduceGeom g;
  g.outer = outer; g.n = n; g.inner = inner;
  g.rows = inner == 1;
  int min_elt = 8;
  for (int l = 0; l < p.num_leaves; ++l) min_elt = dtype_size(p.leaves[l].dtype) < min_elt ? dtype_size(p.leaves[l].dtype) : min_elt;
  if (p.num_leaves == 0) min_elt = 4;
  int vec = 16 / min_elt;
  if (vec > 8) vec = 8;
  if (p.wide && vec > 2) vec = 2;
  const int64_t contiguous = g.rows ? n : inner;
  while (vec > 1 && (contiguous % vec != 0 || p.dims[p.rank - 1] % vec != 0)) vec /= 2;
  if (!allow_vector) vec = 1;
  g.vec = vec;
  if (g.rows) {
    const int64_t vecs = n / vec;
    g.tpr = vecs <= 1024 ? 32 : 256;
    // vectors in flight per thread: a row group waits for its loads before it can fold them, so the loads of one
    // iteration are all the memory parallelism it has
    g.unroll = 1;
    while (g.unroll < 4 && vecs >= 2 * g.unroll * g.tpr && p.num_regs * vec * 2 * g.unroll <= 64) g.unroll *= 2;
  }
  return g;
}

std::string ReduceSource(const EwProgram& p, int rt, const ReduceGeom& g, int out_dtype) {
  GenConfig cfg;
  cfg.vec = g.vec;
  cfg.unroll = g.unroll;
  cfg.wide_index = NumElements(p) > 0xffffffffLL;
  cfg.packed = g.vec >= 2 && CanPack(p, &cfg.packed_dtype);
  const char* idx_t = cfg.wide_index ? "uint64_t" : "uint32_t";
  const char* acc_t = AccType(out_dtype);
  // the value of element v of vector u as an accumulator
  auto elem_acc = [&](const std::string& v_even_odd_index) {
    std::ostringstream e;
    if (cfg.packed) e << "(A)(((" << v_even_odd_index << ") & 1) ? ew_p2_hi(r" << p.out_reg << "[u][(" << v_even_odd_index << ") >> 1], " << out_dtype
                      << ") : ew_p2_lo(r" << p.out_reg << "[u][(" << v_even_odd_index << ") >> 1], " << out_dtype << "))";
    else e << "RdAcc<A>::in(r" << p.out_reg << "[u][" << v_even_odd_index << "], " << out_dtype << ")";
    return e.str();
  };
  std::ostringstream o;
  o << Preamble() << kOpsSource << kGlue;
  o << "typedef " << (p.wide ? "uint64_t" : "uint32_t") << " R;\ntypedef " << acc_t << " A;\n";
  o << "#define VEC " << cfg.vec << "\n#define UNR " << cfg.unroll << "\n#define RT " << rt << "\n";
  o << "extern \"C\" __global__ void __launch_bounds__(256) ew_kernel(const EwPtrs P) {\n";
  if (g.rows) {
    const int64_t vecs = g.n / g.vec;
    o << "  const int TPR = " << g.tpr << ";\n";
    o << "  const " << idx_t << " vecs = " << vecs << "ull, rows = " << g.outer << "ull;\n";
    o << "  const int t = threadIdx.x % TPR;\n";
    o << "  __shared__ A part[8];\n";
    o << "  for (" << idx_t << " row = (" << idx_t << ")blockIdx.x * (256 / TPR) + threadIdx.x / TPR; row < rows; row += (" << idx_t
      << ")gridDim.x * (256 / TPR)) {\n";
    o << "    A acc = rd_identity<A>(RT);\n";
    o << "    for (" << idx_t << " v0 = t; v0 < vecs; v0 += TPR * UNR) {\n";
    o << "      " << idx_t << " vi[UNR];\n      bool live[UNR];\n";
    o << "      _Pragma(\"unroll\") for (int u = 0; u < UNR; ++u) { live[u] = v0 + u * TPR < vecs; vi[u] = row * vecs + v0 + u * TPR; }\n";
    EmitBody(o, p, cfg);
    o << "      _Pragma(\"unroll\") for (int u = 0; u < UNR; ++u) {\n        if (!live[u]) continue;\n";
    o << "        _Pragma(\"unroll\") for (int v = 0; v < VEC; ++v) acc = rd_combine<A>(RT, acc, " << elem_acc("v") << ");\n      }\n    }\n";
    o << "    acc = rd_warp<A>(RT, acc);\n";
    if (g.tpr == 256) {
      // one row per CTA and iteration: every thread takes part in both barriers
      o << "    __syncthreads();\n    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = acc;\n    __syncthreads();\n";
      o << "    if (threadIdx.x < 32) {\n      A x = threadIdx.x < 8 ? part[threadIdx.x] : rd_identity<A>(RT);\n      x = rd_warp<A>(RT, x);\n";
      o << "      if (threadIdx.x == 0) store_elem<R>(P.out, (long long)row, " << out_dtype << ", RdAcc<A>::out<R>(x, " << out_dtype << "));\n    }\n";
    } else {
      o << "    if (t == 0) store_elem<R>(P.out, (long long)row, " << out_dtype << ", RdAcc<A>::out<R>(acc, " << out_dtype << "));\n";
    }
    o << "  }\n}\n";
  } else {
    // thread per VEC columns of one outer slice
    const int64_t ivecs = g.inner / g.vec;
    o << "  const " << idx_t << " ivecs = " << ivecs << "ull, count = " << g.outer * ivecs << "ull, n = " << g.n << "ull;\n";
    o << "  for (" << idx_t << " c = (" << idx_t << ")blockIdx.x * 256 + threadIdx.x; c < count; c += (" << idx_t << ")gridDim.x * 256) {\n";
    o << "    const " << idx_t << " ob = c / ivecs, iv = c - ob * ivecs;\n";
    o << "    A acc[VEC];\n    _Pragma(\"unroll\") for (int v = 0; v < VEC; ++v) acc[v] = rd_identity<A>(RT);\n";
    o << "    for (" << idx_t << " j = 0; j < n; j += UNR) {\n";
    o << "      " << idx_t << " vi[UNR];\n      bool live[UNR];\n";
    o << "      _Pragma(\"unroll\") for (int u = 0; u < UNR; ++u) { live[u] = j + u < n; vi[u] = (ob * n + j + u) * ivecs + iv; }\n";
    EmitBody(o, p, cfg);
    o << "      _Pragma(\"unroll\") for (int u = 0; u < UNR; ++u) {\n        if (!live[u]) continue;\n";
    o << "        _Pragma(\"unroll\") for (int v = 0; v < VEC; ++v) acc[v] = rd_combine<A>(RT, acc[v], " << elem_acc("v") << ");\n      }\n    }\n";
    o << "    _Pragma(\"unroll\") for (int v = 0; v < VEC; ++v) store_elem<R>(P.out, (long long)(c * VEC + v), " << out_dtype
      << ", RdAcc<A>::out<R>(acc[v], " << out_dtype << "));\n";
    o << "  }\n}\n";
  }
  return o.str();
}

}  // namespace

std::string ewise_jit_reduce_source(const EwProgram& p, int reduce_type, int64_t outer, int64_t n, int64_t inner, bool allow_vector) {
  ReduceGeom g = ChooseReduce(p, outer, n, inner, allow_vector);
  if (!g.rows) g.unroll = (n >= 4 && p.num_regs * g.vec <= 32) ? 2 : 1;
  return ReduceSource(p, reduce_type, g, p.out_dtype);
}

bool ewise_jit_reduce_fits(int64_t outer, int64_t n, int64_t inner, int sm_count) {
  // no split across CTAs here: there must be enough rows (or columns) to fill the GPU, or little enough work not to care
  if (inner == 1) return outer >= (int64_t)sm_count * 2 || n <= 16384;
  return outer * inner >= (int64_t)sm_count * 256 || n <= 512;
}

Status ewise_jit_reduce_prepare(Device* dev, const EwProgram& prog, int reduce_type, int64_t outer, int64_t n, int64_t inner, EwJit** out) {
  *out = nullptr;
  const char* off = getenv("B200MLX_JIT");
  if (off && off[0] == '0') return Status::Unsupported("run-time compilation switched off (B200MLX_JIT=0)");
  if (outer * n * inner == 0) return Status::Unsupported("empty reduction");
  if (!ewise_jit_reduce_fits(outer, n, inner, dev->sm_count())) return Status::Unsupported("reduction needs a split across CTAs");
  B200_TRY(dev->MakeCurrent());
  // vector form first; the scalar form is built only if the vector form cannot be used at all (pointer alignment is
  // checked at launch, where a misaligned leaf switches to a scalar build made on demand)
  const std::string src = ewise_jit_reduce_source(prog, reduce_type, outer, n, inner, true);
  {
    std::lock_guard<std::mutex> lock(g_jit_mu);
    auto it = g_jit_cache.find(src);
    if (it != g_jit_cache.end()) { *out = it->second; return Status::OK(); }
  }
  if (const char* dir = getenv("B200MLX_JIT_DUMP")) {
    static int serial = 0;
    const std::string path = std::string(dir) + "/reduce_chain_" + std::to_string(serial++) + ".cu";
    if (FILE* f = fopen(path.c_str(), "w")) { fputs(src.c_str(), f); fclose(f); }
  }
  std::vector<char> cubin;
  B200_TRY(ewise_jit_nvrtc(src, &cubin));
  std::unique_ptr<EwJit> j(new EwJit());
  B200_CUDA_TRY(cudaLibraryLoadData(&j->lib, cubin.data(), nullptr, nullptr, 0, nullptr, nullptr, 0));
  B200_CUDA_TRY(cudaLibraryGetKernel(&j->kernel, j->lib, "ew_kernel"));
  const ReduceGeom g = ChooseReduce(prog, outer, n, inner, true);
  j->vec = g.vec;
  j->num_leaves = prog.num_leaves;
  j->prog = prog;
  j->sm_count = dev->sm_count();
  j->is_reduce = true;
  j->reduce_type = reduce_type;
  j->outer = outer; j->n = n; j->inner = inner;
  if (g.rows) j->grid_units = (outer + (256 / g.tpr) - 1) / (256 / g.tpr);
  else j->grid_units = (outer * (inner / g.vec) + 255) / 256;
  if (g.vec > 1) {
    auto align_of = [](int bytes) { return bytes >= 16 ? 16 : bytes; };
    for (int l = 0; l < prog.num_leaves; ++l) {
      const LeafPlan lp = PlanLeaf(prog, prog.leaves[l], g.vec);
      if (lp.kind == LeafPlan::kDense || lp.kind == LeafPlan::kVector) j->align_bytes[l] = align_of(g.vec * dtype_size(prog.leaves[l].dtype));
    }
  }
  j->out_align = 1;
  std::lock_guard<std::mutex> lock(g_jit_mu);
  auto ins = g_jit_cache.emplace(src, j.get());
  if (ins.second) j.release();
  *out = ins.first->second;
  return Status::OK();
}

namespace {
// The VEC = 1 build of a reduction kernel, for operands that are not aligned for vector loads.
Status BuildReduceScalar(EwJit* jit, EwJit** out) {
  const std::string src = ewise_jit_reduce_source(jit->prog, jit->reduce_type, jit->outer, jit->n, jit->inner, false);
  {
    std::lock_guard<std::mutex> lock(g_jit_mu);
    auto it = g_jit_cache.find(src);
    if (it != g_jit_cache.end()) { *out = it->second; return Status::OK(); }
  }
  std::vector<char> cubin;
  B200_TRY(ewise_jit_nvrtc(src, &cubin));
  std::unique_ptr<EwJit> j(new EwJit());
  B200_CUDA_TRY(cudaLibraryLoadData(&j->lib, cubin.data(), nullptr, nullptr, 0, nullptr, nullptr, 0));
  B200_CUDA_TRY(cudaLibraryGetKernel(&j->kernel, j->lib, "ew_kernel"));
  const ReduceGeom g = ChooseReduce(jit->prog, jit->outer, jit->n, jit->inner, false);
  j->vec = 1;
  j->num_leaves = jit->num_leaves;
  j->is_reduce = true;
  if (g.rows) j->grid_units = (jit->outer + (256 / g.tpr) - 1) / (256 / g.tpr);
  else j->grid_units = (jit->outer * jit->inner + 255) / 256;
  std::lock_guard<std::mutex> lock(g_jit_mu);
  auto ins = g_jit_cache.emplace(src, j.get());
  if (ins.second) j.release();
  *out = ins.first->second;
  return Status::OK();
}
}  // namespace

Status ewise_jit_run(Device* dev, EwJit* jit, const EwProgram& prog) {
  B200_TRY(dev->MakeCurrent());
  EwJit* use = jit;
  if (jit->vec > 1) {
    bool aligned = jit->out_align <= 1 || (reinterpret_cast<uintptr_t>(prog.out) % (unsigned)jit->out_align) == 0;
    for (int l = 0; l < jit->num_leaves && aligned; ++l)
      if (jit->align_bytes[l] && reinterpret_cast<uintptr_t>(prog.leaves[l].ptr) % (unsigned)jit->align_bytes[l] != 0) aligned = false;
    if (!aligned) {
      if (!jit->scalar) {
        EwJit* s = nullptr;
        if (jit->is_reduce) B200_TRY(BuildReduceScalar(jit, &s));
        else B200_TRY(BuildJit(jit->prog, jit->sm_count, false, &s));
        jit->scalar = s;
      }
      use = jit->scalar;
    }
  }
  struct { const void* leaf[8]; void* out; } ptrs;
  for (int l = 0; l < 8; ++l) ptrs.leaf[l] = l < prog.num_leaves ? prog.leaves[l].ptr : nullptr;
  ptrs.out = prog.out;
  const int64_t per_block = 256 * (int64_t)use->unroll;
  int64_t blocks = use->is_reduce ? use->grid_units : (use->nvec + per_block - 1) / per_block;
  // elementwise kernels run a persistent grid; row reductions get one CTA per 256 / TPR rows (short CTAs that the
  // hardware deals out as SMs free up balance better than a static stride when there are only a few rows per row group)
  const int64_t cap = use->is_reduce ? 0x7fffffffLL : (int64_t)dev->sm_count() * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  void* args[] = {&ptrs};
  B200_CUDA_TRY(cudaLaunchKernel(reinterpret_cast<const void*>(use->kernel), dim3((unsigned)blocks), dim3(256), args, 0, dev->stream()));
  return Status::OK();
}


bool ewise_jit_available(std::string* why) {
  Nvrtc* n = nvrtc();
  if (why) *why = n->why;
  return n->handle != nullptr;
}

}  // namespace k
}  // namespace b200
