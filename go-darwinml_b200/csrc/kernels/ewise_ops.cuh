// Semantics of the fused elementwise programs: register representation, loads / stores of one element, every unary /
// binary / compare / select / clamp op and every conversion, as always-inline device functions of (op, dtype, values).
//
// Two users compile this text: ewise.cu with nvcc (the interpreter kernel calls it with run-time op codes), and the
// run-time compiler of ewise_jit.cu, which hands it to NVRTC in front of a generated straight-line kernel that calls the
// same functions with literal op codes, so that both paths compute every op with the same expressions.  For that
// reason this file includes nothing and uses only built-in types, inline PTX and the CUDA math functions that NVRTC
// declares by itself; the integer typedefs, the dtype constants (B200_*), `enum class Op`, dtype_size() and
// dtype_is_float() come from the including translation unit (common.h under nvcc, a generated preamble under NVRTC).
//
// Register representation:
//   F16/BF16/F32 -> float bits      (16-bit floats are re-rounded after every op,
//                                    so a fused chain equals the op-by-op result)
//   F64 -> double bits (wide programs only)
//   I8/I16/I32, U8/U16/U32, Bool -> 32-bit integer, sign/zero extended
//   I64/U64 -> 64-bit integer (wide programs only)

// ---- what <type_traits>, <cmath> and the 16-bit float headers would have given ----
template <typename I> struct EwInt;
template <> struct EwInt<int32_t> { typedef uint32_t U; static constexpr bool is_signed = true; };
template <> struct EwInt<uint32_t> { typedef uint32_t U; static constexpr bool is_signed = false; };
template <> struct EwInt<int64_t> { typedef uint64_t U; static constexpr bool is_signed = true; };
template <> struct EwInt<uint64_t> { typedef uint64_t U; static constexpr bool is_signed = false; };
__device__ __forceinline__ float ew_inf() { return __int_as_float(0x7f800000); }
__device__ __forceinline__ uint16_t ew_f_to_bf16(float v) {   // round to nearest even, NaN kept
  uint16_t h;
  asm("cvt.rn.bf16.f32 %0, %1;" : "=h"(h) : "f"(v));
  return h;
}
__device__ __forceinline__ float ew_bf16_to_f(uint16_t h) { return __uint_as_float((uint32_t)h << 16); }
__device__ __forceinline__ uint16_t ew_f_to_f16(float v) {
  uint16_t h;
  asm("cvt.rn.f16.f32 %0, %1;" : "=h"(h) : "f"(v));
  return h;
}
__device__ __forceinline__ float ew_f16_to_f(uint16_t h) {
  float f;
  asm("cvt.f32.f16 %0, %1;" : "=f"(f) : "h"(h));
  return f;
}
__device__ __forceinline__ float ew_round_bf16(float v) { return ew_bf16_to_f(ew_f_to_bf16(v)); }
__device__ __forceinline__ float ew_round_f16(float v) { return ew_f16_to_f(ew_f_to_f16(v)); }

template <typename R> struct RegTraits;
template <> struct RegTraits<uint32_t> { static constexpr bool wide = false; };
template <> struct RegTraits<uint64_t> { static constexpr bool wide = true; };

// ---- representation helpers ------------------------------------------------
template <typename R> __device__ __forceinline__ float as_f(R r) { return __uint_as_float((uint32_t)r); }
template <typename R> __device__ __forceinline__ R from_f(float f) { return (R)__float_as_uint(f); }
__device__ __forceinline__ double as_d(uint64_t r) { return __longlong_as_double((long long)r); }
__device__ __forceinline__ uint64_t from_d(double d) { return (uint64_t)__double_as_longlong(d); }

__device__ __forceinline__ float round_to(int dtype, float v) {
  if (dtype == B200_BFLOAT16) return ew_round_bf16(v);
  if (dtype == B200_FLOAT16) return ew_round_f16(v);
  return v;
}
__device__ __forceinline__ uint32_t wrap_i32(int dtype, uint32_t v) {
  switch (dtype) {
    case B200_INT8: return (uint32_t)(int32_t)(int8_t)v;
    case B200_INT16: return (uint32_t)(int32_t)(int16_t)v;
    case B200_UINT8: return v & 0xffu;
    case B200_UINT16: return v & 0xffffu;
    case B200_BOOL: return v ? 1u : 0u;
  }
  return v;
}

template <typename R>
__device__ __forceinline__ R load_elem(const void* base, int64_t off, int dtype) {
  switch (dtype) {
    case B200_FLOAT32: return from_f<R>(reinterpret_cast<const float*>(base)[off]);
    case B200_BFLOAT16: return from_f<R>(ew_bf16_to_f(reinterpret_cast<const uint16_t*>(base)[off]));
    case B200_FLOAT16: return from_f<R>(ew_f16_to_f(reinterpret_cast<const uint16_t*>(base)[off]));
    case B200_INT32: case B200_UINT32: return (R) reinterpret_cast<const uint32_t*>(base)[off];
    case B200_INT8: return (R)(uint32_t)(int32_t) reinterpret_cast<const int8_t*>(base)[off];
    case B200_INT16: return (R)(uint32_t)(int32_t) reinterpret_cast<const int16_t*>(base)[off];
    case B200_UINT8: return (R) reinterpret_cast<const uint8_t*>(base)[off];
    case B200_BOOL: return (R)(reinterpret_cast<const uint8_t*>(base)[off] ? 1u : 0u);
    case B200_UINT16: return (R) reinterpret_cast<const uint16_t*>(base)[off];
    default:
      if constexpr (RegTraits<R>::wide) return (R) reinterpret_cast<const uint64_t*>(base)[off];  // I64/U64/F64
      return 0;
  }
}
template <typename R>
__device__ __forceinline__ void store_elem(void* base, int64_t off, int dtype, R r) {
  switch (dtype) {
    case B200_FLOAT32: reinterpret_cast<float*>(base)[off] = as_f(r); break;
    case B200_BFLOAT16: reinterpret_cast<uint16_t*>(base)[off] = ew_f_to_bf16(as_f(r)); break;
    case B200_FLOAT16: reinterpret_cast<uint16_t*>(base)[off] = ew_f_to_f16(as_f(r)); break;
    case B200_INT32: case B200_UINT32: reinterpret_cast<uint32_t*>(base)[off] = (uint32_t)r; break;
    case B200_INT8: case B200_UINT8: reinterpret_cast<uint8_t*>(base)[off] = (uint8_t)r; break;
    case B200_BOOL: reinterpret_cast<uint8_t*>(base)[off] = r ? 1 : 0; break;
    case B200_INT16: case B200_UINT16: reinterpret_cast<uint16_t*>(base)[off] = (uint16_t)r; break;
    default:
      if constexpr (RegTraits<R>::wide) reinterpret_cast<uint64_t*>(base)[off] = (uint64_t)r;
      break;
  }
}

// ---- arithmetic on one computational type ----------------------------------
template <typename F> __device__ __forceinline__ F f_unary(int op, F x) {
  switch ((Op)op) {
    case Op::Abs: return fabs(x);
    case Op::Neg: return -x;
    case Op::Sqrt: return sqrt(x);
    case Op::Rsqrt: return F(1) / sqrt(x);
    case Op::Exp: return exp(x);
    case Op::Expm1: return exp(x) - F(1);      // naive form, as the reference builds it (bridge.m:315-333)
    case Op::Log: return log(x);
    case Op::Log1p: return log(F(1) + x);      // naive form (bridge.m:336-354)
    case Op::Sin: return sin(x);
    case Op::Cos: return cos(x);
    case Op::Tanh: return tanh(x);
    case Op::Sigmoid: return F(1) / (F(1) + exp(-x));
    case Op::Erf: return erf(x);
    case Op::Floor: return floor(x);
    case Op::Ceil: return ceil(x);
    case Op::Round: return rint(x);
    case Op::Sign: return (x > F(0)) ? F(1) : ((x < F(0)) ? F(-1) : x);  // keeps +-0 and NaN
    case Op::Identity: return x;
    case Op::GeluExact: return F(0.5) * x * (F(1) + erf(x * F(0.7071067811865475)));
    case Op::GeluTanh: return F(0.5) * x * (F(1) + tanh(F(0.7978845608028654) * (x + F(0.044715) * x * x * x)));
    case Op::Relu: return fmax(x, F(0));
    case Op::Silu: return x / (F(1) + exp(-x));
    default: return x;
  }
}
// Unary float ops whose result is rounded to a 16-bit float (8 or 11 significant bits): the hardware approximations
// (tanh.approx, ex2.approx, rsqrt.approx: relative error about 2^-11 .. 2^-22) are then below the rounding step, and a
// chain over 16-bit data is bound by instruction issue, not by memory (8 elements per 16-byte vector).  Ops without a
// cheap form fall through to the exact one.
__device__ __forceinline__ float ew_tanh_approx(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float f_unary_to16(int op, float x) {
  switch ((Op)op) {
    case Op::Tanh: return ew_tanh_approx(x);
    case Op::Exp: return __expf(x);
    case Op::Sigmoid: return __fdividef(1.0f, 1.0f + __expf(-x));
    case Op::Silu: return __fdividef(x, 1.0f + __expf(-x));
    case Op::Rsqrt: return rsqrtf(x);
    case Op::GeluTanh: {
      const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
      return 0.5f * x * (1.0f + ew_tanh_approx(u));
    }
    default: return f_unary<float>(op, x);
  }
}
// max / min that return NaN when either operand is NaN (one instruction)
__device__ __forceinline__ float ew_max_nan(float a, float b) {
  float r;
  asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ float ew_min_nan(float a, float b) {
  float r;
  asm("min.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}

template <typename F> __device__ __forceinline__ F f_binary(int op, F a, F b) {
  switch ((Op)op) {
    case Op::Add: return a + b;
    case Op::Sub: return a - b;
    case Op::Mul: return a * b;
    case Op::Div: return a / b;
    case Op::Rem: return fmod(a, b);
    case Op::Pow: return pow(a, b);
    // NaN-propagating max/min, like XLA and NumPy maximum/minimum
    case Op::Max: return (a != a || b != b) ? (a + b) : fmax(a, b);
    case Op::Min: return (a != a || b != b) ? (a + b) : fmin(a, b);
    case Op::Atan2: return atan2(a, b);
    default: return a;
  }
}
template <typename I> __device__ __forceinline__ I i_unary(int op, I x) {
  using U = typename EwInt<I>::U;
  switch ((Op)op) {
    case Op::Abs: return EwInt<I>::is_signed ? (I)(x < 0 ? (I)(U(0) - U(x)) : x) : x;
    case Op::Neg: return (I)(U(0) - U(x));
    case Op::Sign: return EwInt<I>::is_signed ? (I)((x > 0) - (x < 0)) : (I)(x != 0);
    case Op::BitwiseNot: return (I)~U(x);
    case Op::LogicalNot: return (I)(x == 0);
    case Op::Relu: return x > 0 ? x : (I)0;
    default: return x;
  }
}
template <typename I> __device__ __forceinline__ I i_binary(int op, I a, I b) {
  using U = typename EwInt<I>::U;
  constexpr int bits = sizeof(I) * 8;
  switch ((Op)op) {
    case Op::Add: return (I)(U(a) + U(b));
    case Op::Sub: return (I)(U(a) - U(b));
    case Op::Mul: return (I)(U(a) * U(b));
    case Op::Div:
      if (b == 0) return (I)-1;
      if (EwInt<I>::is_signed && b == (I)-1) return (I)(U(0) - U(a));
      return a / b;
    case Op::Rem:
      if (b == 0) return a;
      if (EwInt<I>::is_signed && b == (I)-1) return 0;
      return a % b;
    case Op::Pow: {
      if (EwInt<I>::is_signed && b < 0) return (a == 1) ? (I)1 : ((a == (I)-1) ? ((b & 1) ? (I)-1 : (I)1) : (I)0);
      U r = 1, base = U(a), e = U(b);
      while (e) { if (e & 1) r *= base; base *= base; e >>= 1; }
      return (I)r;
    }
    case Op::Max: return a > b ? a : b;
    case Op::Min: return a < b ? a : b;
    case Op::LogicalAnd: return (I)((a != 0) && (b != 0));
    case Op::LogicalOr: return (I)((a != 0) || (b != 0));
    case Op::LogicalXor: return (I)((a != 0) != (b != 0));
    case Op::BitwiseAnd: return (I)(U(a) & U(b));
    case Op::BitwiseOr: return (I)(U(a) | U(b));
    case Op::BitwiseXor: return (I)(U(a) ^ U(b));
    case Op::ShiftLeft: return (U(b) >= (U)bits) ? (I)0 : (I)(U(a) << U(b));
    case Op::ShiftRight:
      if (U(b) >= (U)bits) return (EwInt<I>::is_signed && a < 0) ? (I)-1 : (I)0;
      return (I)(a >> b);
    case Op::ShiftRightLogical: return (U(b) >= (U)bits) ? (I)0 : (I)(U(a) >> U(b));
    default: return a;
  }
}
template <typename T> __device__ __forceinline__ bool cmp(int op, T a, T b) {
  switch ((Op)op) {
    case Op::Equal: return a == b;
    case Op::NotEqual: return a != b;
    case Op::LessThan: return a < b;
    case Op::LessOrEqual: return a <= b;
    case Op::GreaterThan: return a > b;
    case Op::GreaterOrEqual: return a >= b;
    default: return false;
  }
}

__device__ __forceinline__ bool is_cmp_op(int op) { return op >= (int)Op::Equal && op <= (int)Op::GreaterOrEqual; }
__device__ __forceinline__ bool is_bin_op(int op) { return op >= (int)Op::Add && op <= (int)Op::ShiftRightLogical; }

// Narrow value of `dtype` held in r -> signed 32-bit view / float view are both r itself.
template <typename R>
__device__ __forceinline__ R eval_op_impl(const int op, const int sd, R a, R b, R c, const bool round16) {
  if (op == (int)Op::Where) return a ? b : c;  // a is a Bool register
  if (op == (int)Op::IsFinite || op == (int)Op::IsNaN) {
    if (sd == B200_FLOAT64) {
      if constexpr (RegTraits<R>::wide) {
        const double x = as_d(a);
        return (R)(op == (int)Op::IsNaN ? (x != x) : (x == x && fabs(x) != ew_inf()));
      }
      return 0;
    }
    if (dtype_is_float(sd)) {
      const float x = as_f(a);
      return (R)(op == (int)Op::IsNaN ? (x != x) : (x == x && fabsf(x) != ew_inf()));
    }
    return (R)(op == (int)Op::IsNaN ? 0 : 1);
  }
  switch (sd) {
    case B200_FLOAT32: case B200_BFLOAT16: case B200_FLOAT16: {
      const float x = as_f(a), y = as_f(b), z = as_f(c);
      if (is_cmp_op(op)) return (R)cmp<float>(op, x, y);
      float r;
      if (op == (int)Op::Clamp) r = fminf(fmaxf(y, x), z);  // (min=a, x=b, max=c)
      else if (op == (int)Op::Max) r = ew_max_nan(x, y);
      else if (op == (int)Op::Min) r = ew_min_nan(x, y);
      else if (is_bin_op(op)) r = f_binary<float>(op, x, y);
      else if (sd != B200_FLOAT32) r = f_unary_to16(op, x);
      else r = f_unary<float>(op, x);
      return from_f<R>(round16 ? round_to(sd, r) : r);
    }
    case B200_FLOAT64:
      if constexpr (RegTraits<R>::wide) {
        const double x = as_d(a), y = as_d(b), z = as_d(c);
        if (is_cmp_op(op)) return (R)cmp<double>(op, x, y);
        double r;
        if (op == (int)Op::Clamp) r = fmin(fmax(y, x), z);
        else if (is_bin_op(op)) r = f_binary<double>(op, x, y);
        else r = f_unary<double>(op, x);
        return from_d(r);
      }
      return 0;
    case B200_INT64:
      if constexpr (RegTraits<R>::wide) {
        const int64_t x = (int64_t)a, y = (int64_t)b, z = (int64_t)c;
        if (is_cmp_op(op)) return (R)cmp<int64_t>(op, x, y);
        if (op == (int)Op::Clamp) return (R)(y < x ? x : (y > z ? z : y));
        return (R)(is_bin_op(op) ? i_binary<int64_t>(op, x, y) : i_unary<int64_t>(op, x));
      }
      return 0;
    case B200_UINT64:
      if constexpr (RegTraits<R>::wide) {
        const uint64_t x = a, y = b, z = c;
        if (is_cmp_op(op)) return (R)cmp<uint64_t>(op, x, y);
        if (op == (int)Op::Clamp) return (R)(y < x ? x : (y > z ? z : y));
        return (R)(is_bin_op(op) ? i_binary<uint64_t>(op, x, y) : i_unary<uint64_t>(op, x));
      }
      return 0;
    case B200_INT8: case B200_INT16: case B200_INT32: {
      const int32_t x = (int32_t)(uint32_t)a, y = (int32_t)(uint32_t)b, z = (int32_t)(uint32_t)c;
      if (is_cmp_op(op)) return (R)cmp<int32_t>(op, x, y);
      int32_t r;
      if (op == (int)Op::Clamp) r = (y < x ? x : (y > z ? z : y));
      else if (op == (int)Op::ShiftLeft || op == (int)Op::ShiftRight || op == (int)Op::ShiftRightLogical) {
        // shifts act on the value's own width
        const int bits = dtype_size(sd) * 8;
        const uint32_t mask = bits == 32 ? 0xffffffffu : ((1u << bits) - 1u);
        const uint32_t ux = (uint32_t)x & mask, sh = (uint32_t)y;
        if (sh >= (uint32_t)bits) r = (op == (int)Op::ShiftRight && x < 0) ? -1 : 0;
        else if (op == (int)Op::ShiftLeft) r = (int32_t)(ux << sh);
        else if (op == (int)Op::ShiftRight) r = x >> sh;
        else r = (int32_t)(ux >> sh);
      } else r = is_bin_op(op) ? i_binary<int32_t>(op, x, y) : i_unary<int32_t>(op, x);
      return (R)wrap_i32(sd, (uint32_t)r);
    }
    default: {  // U8 U16 U32 Bool
      const uint32_t x = (uint32_t)a, y = (uint32_t)b, z = (uint32_t)c;
      if (is_cmp_op(op)) return (R)cmp<uint32_t>(op, x, y);
      uint32_t r;
      if (op == (int)Op::Clamp) r = (y < x ? x : (y > z ? z : y));
      else if (op == (int)Op::ShiftLeft || op == (int)Op::ShiftRight || op == (int)Op::ShiftRightLogical) {
        const int bits = dtype_size(sd) * 8;
        r = (y >= (uint32_t)bits) ? 0u : (op == (int)Op::ShiftLeft ? (x << y) : (x >> y));
      } else r = is_bin_op(op) ? i_binary<uint32_t>(op, x, y) : i_unary<uint32_t>(op, x);
      return (R)wrap_i32(sd, r);
    }
  }
}

template <typename R>
__device__ __forceinline__ R eval_op_core(const int op, const int sd, R a, R b, R c) { return eval_op_impl<R>(op, sd, a, b, c, true); }
// The same without the final rounding of a 16-bit float result: the caller rounds two results at once (ew_round_pair).
template <typename R>
__device__ __forceinline__ R eval_op_unrounded(const int op, const int sd, R a, R b, R c) { return eval_op_impl<R>(op, sd, a, b, c, false); }
// Rounds two fp32 values to the 16-bit float type dt (round to nearest even, as round_to does) with ONE packed
// conversion.  The scalar conversion instruction is issued at a quarter of the arithmetic rate; a chain over 16-bit
// data rounds after every op and was bound by exactly that.
__device__ __forceinline__ void ew_round_pair(int dt, float& a, float& b) {
  uint32_t p;
  if (dt == B200_BFLOAT16) {
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(p) : "f"(b), "f"(a));   // upper half <- b, lower half <- a
    a = __uint_as_float(p << 16);
    b = __uint_as_float(p & 0xffff0000u);
  } else {
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(p) : "f"(b), "f"(a));
    a = ew_f16_to_f((uint16_t)(p & 0xffffu));
    b = ew_f16_to_f((uint16_t)(p >> 16));
  }
}

// Conversion between register representations.  Float -> integer truncates
// toward zero and saturates (NaN -> 0), which is what the cvt.rzi instructions
// do; integer -> narrower integer wraps; anything -> Bool is (x != 0).
template <typename R>
__device__ __forceinline__ R eval_cast_core(int from, int to, R a) {
  if (from == to) return a;
  const bool wide = RegTraits<R>::wide;
  // source as one of: float, double, int64, uint64
  if (to == B200_BOOL) {
    if (from == B200_FLOAT64) { if constexpr (wide) return (R)(as_d(a) != 0.0); return 0; }
    if (dtype_is_float(from)) return (R)(as_f(a) != 0.0f);
    if (from == B200_INT64 || from == B200_UINT64) return (R)(a != 0);
    return (R)((uint32_t)a != 0u);
  }
  if (dtype_is_float(from) && from != B200_FLOAT64) {
    const float x = as_f(a);
    switch (to) {
      case B200_FLOAT32: return a;
      case B200_BFLOAT16: case B200_FLOAT16: return from_f<R>(round_to(to, x));
      case B200_FLOAT64: if constexpr (wide) return from_d((double)x); return 0;
      case B200_INT64: if constexpr (wide) return (R)(int64_t)__float2ll_rz(x); return 0;
      case B200_UINT64: if constexpr (wide) return (R)__float2ull_rz(x); return 0;
      case B200_UINT32: return (R)__float2uint_rz(x);
      case B200_UINT8: case B200_UINT16: {
        const uint32_t lim = to == B200_UINT8 ? 0xffu : 0xffffu;
        const uint32_t v = __float2uint_rz(x);
        return (R)(v > lim ? lim : v);
      }
      case B200_INT32: return (R)(uint32_t)__float2int_rz(x);
      default: {  // I8 I16 saturate
        const int32_t lo = to == B200_INT8 ? -128 : -32768, hi = to == B200_INT8 ? 127 : 32767;
        int32_t v = __float2int_rz(x);
        v = v < lo ? lo : (v > hi ? hi : v);
        return (R)(uint32_t)v;
      }
    }
  }
  if (from == B200_FLOAT64) {
    if constexpr (wide) {
      const double x = as_d(a);
      switch (to) {
        case B200_FLOAT32: return from_f<R>((float)x);
        case B200_BFLOAT16: case B200_FLOAT16: return from_f<R>(round_to(to, (float)x));
        case B200_INT64: return (R)(int64_t)__double2ll_rz(x);
        case B200_UINT64: return (R)__double2ull_rz(x);
        case B200_UINT32: return (R)__double2uint_rz(x);
        case B200_INT32: return (R)(uint32_t)__double2int_rz(x);
        case B200_UINT8: case B200_UINT16: {
          const uint32_t lim = to == B200_UINT8 ? 0xffu : 0xffffu;
          const uint32_t v = __double2uint_rz(x);
          return (R)(v > lim ? lim : v);
        }
        default: {
          const int32_t lo = to == B200_INT8 ? -128 : -32768, hi = to == B200_INT8 ? 127 : 32767;
          int32_t v = __double2int_rz(x);
          v = v < lo ? lo : (v > hi ? hi : v);
          return (R)(uint32_t)v;
        }
      }
    }
    return 0;
  }
  // integer (or Bool) source
  const bool src64 = (from == B200_INT64 || from == B200_UINT64);
  const bool src_signed = (from == B200_INT8 || from == B200_INT16 || from == B200_INT32 || from == B200_INT64);
  int64_t sv;
  uint64_t uv;
  if (src64) { uv = (uint64_t)a; sv = (int64_t)uv; }
  else if (src_signed) { sv = (int64_t)(int32_t)(uint32_t)a; uv = (uint64_t)sv; }
  else { uv = (uint64_t)(uint32_t)a; sv = (int64_t)uv; }
  switch (to) {
    case B200_FLOAT32: return from_f<R>(src_signed ? (float)sv : (float)uv);
    case B200_BFLOAT16: case B200_FLOAT16: return from_f<R>(round_to(to, src_signed ? (float)sv : (float)uv));
    case B200_FLOAT64: if constexpr (wide) return from_d(src_signed ? (double)sv : (double)uv); return 0;
    case B200_INT64: case B200_UINT64: if constexpr (wide) return (R)uv; return 0;
    default: return (R)wrap_i32(to, (uint32_t)uv);
  }
}
