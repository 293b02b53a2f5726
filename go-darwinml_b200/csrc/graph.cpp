// Graph construction: the b200_* op functions of the C ABI.  Each validates its
// operands, infers the result shape and appends one node (fused ops that are
// pure rewrites append several).  No device work happens here.
//
// Counterpart in the reference: the Go Function methods (mpsgraph
// function.go:288-3075, dotgeneral.go, gather.go) together with the native
// graph-op wrappers they call (bridge.m:197-1106).  Shape rules follow those
// call sites; GoMLX's shapeinference package itself is not part of that tree.
#include <algorithm>
#include <cmath>
#include <functional>
#include <set>
#include <unordered_map>
#include <unordered_set>

#include "common.h"

namespace b200 {

const char* op_name(Op op) {
  static const char* names[] = {
      "Parameter", "Constant", "Iota",
      "Abs", "Neg", "Sqrt", "Rsqrt", "Exp", "Expm1", "Log", "Log1p", "Sin", "Cos", "Tanh", "Sigmoid", "Erf", "Floor",
      "Ceil", "Round", "Sign", "LogicalNot", "BitwiseNot", "IsFinite", "IsNaN", "Identity",
      "GeluExact", "GeluTanh", "Relu", "Silu",
      "Add", "Sub", "Mul", "Div", "Rem", "Pow", "Max", "Min", "Atan2", "LogicalAnd", "LogicalOr", "LogicalXor",
      "BitwiseAnd", "BitwiseOr", "BitwiseXor", "ShiftLeft", "ShiftRight", "ShiftRightLogical",
      "Equal", "NotEqual", "LessThan", "LessOrEqual", "GreaterThan", "GreaterOrEqual",
      "Where", "Clamp",
      "Cast", "Reshape", "Transpose", "BroadcastInDim", "Slice", "Concatenate", "Reverse", "Pad", "DynamicSlice", "DynamicUpdateSlice",
      "DotGeneral", "Reduce", "ArgMinMax", "Gather",
      "Softmax", "SoftmaxMasked", "LayerNorm", "RmsNorm", "Attention", "Rope", "Scatter", "RngBits",
      "ClosureParam", "While", "WhileResult", "ArgSort", "If", "IfResult"};
  static_assert(sizeof(names) / sizeof(names[0]) == (size_t)Op::kNumOps, "op_name table out of date");
  return names[(int)op];
}
bool op_is_unary(Op op) { return op >= Op::Abs && op <= Op::Silu; }
bool op_is_binary(Op op) { return op >= Op::Add && op <= Op::ShiftRightLogical; }
bool op_is_compare(Op op) { return op >= Op::Equal && op <= Op::GreaterOrEqual; }
bool op_is_elementwise(Op op) {
  return op_is_unary(op) || op_is_binary(op) || op_is_compare(op) || op == Op::Where || op == Op::Clamp || op == Op::Cast;
}

namespace {

std::string dims_str(const std::vector<int64_t>& d) {
  std::string s = "[";
  for (size_t i = 0; i < d.size(); ++i) s += (i ? "," : "") + std::to_string(d[i]);
  return s + "]";
}

Status check_node(B200Context ctx, B200Value v, const char* what, Node** out) {
  if (!ctx) return Status::Invalid(std::string(what) + ": null context");
  if (!v) return Status::Invalid(std::string(what) + ": null value");
  Node* n = reinterpret_cast<Node*>(v);
  Ctx* c = reinterpret_cast<Ctx*>(ctx);
  if (n->graph != &c->graph || n->id < 0 || n->id >= (int)c->graph.nodes.size() || c->graph.nodes[n->id].get() != n)
    return Status::Invalid(std::string(what) + ": value does not belong to this context");
  *out = n;
  return Status::OK();
}

Status broadcast_shapes(const char* what, const std::vector<int64_t>& a, const std::vector<int64_t>& b,
                        std::vector<int64_t>* out) {
  const size_t r = std::max(a.size(), b.size());
  out->assign(r, 1);
  for (size_t i = 0; i < r; ++i) {
    const int64_t da = i < r - a.size() ? 1 : a[i - (r - a.size())];
    const int64_t db = i < r - b.size() ? 1 : b[i - (r - b.size())];
    if (da != db && da != 1 && db != 1)
      return Status::Invalid(strfmt("%s: shapes %s and %s do not broadcast", what, dims_str(a).c_str(), dims_str(b).c_str()));
    (*out)[i] = (da == 1) ? db : da;
  }
  return Status::OK();
}

B200Value ret(B200Error* err, const Status& s, Node* n) {
  set_error(err, s);
  return s.ok() ? reinterpret_cast<B200Value>(n) : nullptr;
}

Status unary_impl(B200Context ctx, Op op, B200Value x, Node** out) {
  Node* n;
  const char* name = op_name(op);
  B200_TRY(check_node(ctx, x, name, &n));
  Graph& g = reinterpret_cast<Ctx*>(ctx)->graph;
  int out_dtype = n->dtype;
  switch (op) {
    case Op::Sqrt: case Op::Rsqrt: case Op::Exp: case Op::Expm1: case Op::Log: case Op::Log1p: case Op::Sin: case Op::Cos:
    case Op::Tanh: case Op::Sigmoid: case Op::Erf: case Op::Floor: case Op::Ceil: case Op::Round: case Op::GeluExact:
    case Op::GeluTanh: case Op::Silu:
      if (!dtype_is_float(n->dtype)) return Status::Invalid(strfmt("%s: needs a float operand, got %s", name, dtype_name(n->dtype)));
      break;
    case Op::LogicalNot:
      if (n->dtype != B200_BOOL) return Status::Invalid(strfmt("%s: needs a Bool operand, got %s", name, dtype_name(n->dtype)));
      break;
    case Op::BitwiseNot:
      if (dtype_is_float(n->dtype)) return Status::Invalid(strfmt("%s: needs an integer or Bool operand", name));
      break;
    case Op::Abs: case Op::Neg: case Op::Sign: case Op::Relu:
      if (n->dtype == B200_BOOL) return Status::Invalid(strfmt("%s: Bool operand", name));
      break;
    case Op::IsFinite: case Op::IsNaN:
      out_dtype = B200_BOOL;
      break;
    default: break;
  }
  *out = g.Add(op, out_dtype, n->dims, {n});
  return Status::OK();
}

Status binary_impl(B200Context ctx, Op op, B200Value lhs, B200Value rhs, Node** out) {
  Node *a, *b;
  const char* name = op_name(op);
  B200_TRY(check_node(ctx, lhs, name, &a));
  B200_TRY(check_node(ctx, rhs, name, &b));
  if (a->dtype != b->dtype)
    return Status::Invalid(strfmt("%s: operand dtypes differ (%s vs %s)", name, dtype_name(a->dtype), dtype_name(b->dtype)));
  const int dt = a->dtype;
  switch (op) {
    case Op::LogicalAnd: case Op::LogicalOr: case Op::LogicalXor:
      if (dt != B200_BOOL) return Status::Invalid(strfmt("%s: needs Bool operands, got %s", name, dtype_name(dt)));
      break;
    case Op::BitwiseAnd: case Op::BitwiseOr: case Op::BitwiseXor:
      if (dtype_is_float(dt)) return Status::Invalid(strfmt("%s: needs integer or Bool operands", name));
      break;
    case Op::ShiftLeft: case Op::ShiftRight: case Op::ShiftRightLogical:
      if (!dtype_is_int(dt)) return Status::Invalid(strfmt("%s: needs integer operands", name));
      break;
    case Op::Atan2:
      if (!dtype_is_float(dt)) return Status::Invalid(strfmt("%s: needs float operands", name));
      break;
    default:
      if (dt == B200_BOOL && !op_is_compare(op) && op != Op::Max && op != Op::Min)
        return Status::Invalid(strfmt("%s: Bool operands", name));
      break;
  }
  std::vector<int64_t> dims;
  B200_TRY(broadcast_shapes(name, a->dims, b->dims, &dims));
  Graph& g = reinterpret_cast<Ctx*>(ctx)->graph;
  *out = g.Add(op, op_is_compare(op) ? (int)B200_BOOL : dt, dims, {a, b});
  return Status::OK();
}

Status normalize_axis(const char* what, int axis, int rank, int* out) {
  int a = axis < 0 ? axis + rank : axis;
  if (a < 0 || a >= rank) return Status::Invalid(strfmt("%s: axis %d out of range for rank %d", what, axis, rank));
  *out = a;
  return Status::OK();
}

Status check_shape(const char* what, const int64_t* shape, int rank) {
  if (rank < 0 || rank > 16) return Status::Invalid(strfmt("%s: rank %d not supported", what, rank));
  if (rank > 0 && !shape) return Status::Invalid(strfmt("%s: null shape", what));
  for (int i = 0; i < rank; ++i)
    if (shape[i] < 0) return Status::Invalid(strfmt("%s: negative dimension", what));
  return Status::OK();
}

Node* make_scalar_const(Graph& g, int dtype, double v);

}  // namespace

// Scalar constant of `dtype` holding v.  The reference makes helper scalars as
// Float32 and casts them (function.go:212-231); the value therefore passes
// through float32 first, and so it does here.
namespace {
Node* make_scalar_const(Graph& g, int dtype, double v) {
  const float f32 = (float)v;
  Node* n = g.Add(Op::Constant, B200_FLOAT32, {}, {});
  n->data.resize(4);
  memcpy(n->data.data(), &f32, 4);
  if (dtype != B200_FLOAT32) n = g.Add(Op::Cast, dtype, {}, {n});
  return n;
}
}  // namespace

}  // namespace b200

using namespace b200;

extern "C" {

const char* b200_version(void) { return "b200mlx 0.1 (sm_100a)"; }

int b200_device_count(B200Error* err) {
  clear_error(err);
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess) {
    cudaGetLastError();
    set_error(err, Status::Cuda(strfmt("cudaGetDeviceCount: %s", cudaGetErrorString(e))));
    return -1;
  }
  return n;
}

B200Context b200_create_context(int device, B200Error* err) {
  clear_error(err);
  Device* dev = nullptr;
  Status s = Device::Get(device, &dev);
  if (!s.ok()) { set_error(err, s); return nullptr; }
  Ctx* c = new Ctx();
  c->graph.device = device;
  c->dev = dev;
  return c;
}
void b200_destroy_context(B200Context ctx) { delete reinterpret_cast<Ctx*>(ctx); }
const char* b200_device_name(B200Context ctx) {
  if (!ctx) return nullptr;
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, reinterpret_cast<Ctx*>(ctx)->graph.device) != cudaSuccess) return strdup("unknown");
  return strdup(prop.name);
}
int b200_context_device(B200Context ctx) { return ctx ? reinterpret_cast<Ctx*>(ctx)->graph.device : -1; }

int b200_value_dtype(B200Value v) { return v ? reinterpret_cast<Node*>(v)->dtype : -1; }
int b200_value_rank(B200Value v) { return v ? reinterpret_cast<Node*>(v)->rank() : -1; }
int b200_value_shape(B200Value v, int64_t* dims, int cap) {
  if (!v) return -1;
  Node* n = reinterpret_cast<Node*>(v);
  for (int i = 0; i < n->rank() && i < cap; ++i) dims[i] = n->dims[i];
  return n->rank();
}

// ---- leaves -----------------------------------------------------------------
B200Value b200_placeholder(B200Context ctx, int dtype, const int64_t* shape, int rank, B200Error* err) {
  clear_error(err);
  if (!ctx) return ret(err, Status::Invalid("placeholder: null context"), nullptr);
  if (!dtype_valid(dtype)) return ret(err, Status::Invalid("placeholder: bad dtype"), nullptr);
  Status s = check_shape("placeholder", shape, rank);
  if (!s.ok()) return ret(err, s, nullptr);
  Graph& g = reinterpret_cast<Ctx*>(ctx)->graph;
  return ret(err, Status::OK(), g.Add(Op::Parameter, dtype, std::vector<int64_t>(shape, shape + rank), {}));
}

B200Value b200_constant(B200Context ctx, const void* data, int64_t nbytes, int dtype, const int64_t* shape, int rank,
                        B200Error* err) {
  clear_error(err);
  if (!ctx) return ret(err, Status::Invalid("constant: null context"), nullptr);
  if (!dtype_valid(dtype)) return ret(err, Status::Invalid("constant: bad dtype"), nullptr);
  Status s = check_shape("constant", shape, rank);
  if (!s.ok()) return ret(err, s, nullptr);
  int64_t n = 1;
  for (int i = 0; i < rank; ++i) n *= shape[i];
  if (nbytes != n * dtype_size(dtype))
    return ret(err, Status::Invalid(strfmt("constant: %lld bytes given, shape needs %lld", (long long)nbytes, (long long)(n * dtype_size(dtype)))), nullptr);
  if (nbytes > 0 && !data) return ret(err, Status::Invalid("constant: null data"), nullptr);
  Graph& g = reinterpret_cast<Ctx*>(ctx)->graph;
  Node* node = g.Add(Op::Constant, dtype, std::vector<int64_t>(shape, shape + rank), {});
  node->data.assign((const uint8_t*)data, (const uint8_t*)data + nbytes);
  return ret(err, Status::OK(), node);
}

B200Value b200_iota(B200Context ctx, int dtype, const int64_t* shape, int rank, int axis, B200Error* err) {
  clear_error(err);
  if (!ctx) return ret(err, Status::Invalid("Iota: null context"), nullptr);
  if (!dtype_valid(dtype) || dtype == B200_BOOL) return ret(err, Status::Invalid("Iota: bad dtype"), nullptr);
  Status s = check_shape("Iota", shape, rank);
  if (!s.ok()) return ret(err, s, nullptr);
  int a;
  s = normalize_axis("Iota", axis, rank, &a);
  if (!s.ok()) return ret(err, s, nullptr);
  Graph& g = reinterpret_cast<Ctx*>(ctx)->graph;
  Node* n = g.Add(Op::Iota, dtype, std::vector<int64_t>(shape, shape + rank), {});
  n->ia = {a};
  return ret(err, Status::OK(), n);
}

// ---- unary / binary / compare -------------------------------------------------
#define B200_UNARY(fn, OP)                                           \
  B200Value fn(B200Context ctx, B200Value x, B200Error* err) {       \
    clear_error(err);                                                \
    Node* n = nullptr;                                               \
    Status s = unary_impl(ctx, Op::OP, x, &n);                       \
    return ret(err, s, n);                                           \
  }
B200_UNARY(b200_abs, Abs) B200_UNARY(b200_neg, Neg) B200_UNARY(b200_sqrt, Sqrt) B200_UNARY(b200_rsqrt, Rsqrt)
B200_UNARY(b200_exp, Exp) B200_UNARY(b200_expm1, Expm1) B200_UNARY(b200_log, Log) B200_UNARY(b200_log1p, Log1p)
B200_UNARY(b200_sin, Sin) B200_UNARY(b200_cos, Cos) B200_UNARY(b200_tanh, Tanh) B200_UNARY(b200_sigmoid, Sigmoid)
B200_UNARY(b200_erf, Erf) B200_UNARY(b200_floor, Floor) B200_UNARY(b200_ceil, Ceil) B200_UNARY(b200_round, Round)
B200_UNARY(b200_sign, Sign) B200_UNARY(b200_logical_not, LogicalNot) B200_UNARY(b200_bitwise_not, BitwiseNot)
B200_UNARY(b200_is_finite, IsFinite) B200_UNARY(b200_is_nan, IsNaN) B200_UNARY(b200_identity, Identity)
#undef B200_UNARY

#define B200_BINARY(fn, OP)                                                        \
  B200Value fn(B200Context ctx, B200Value lhs, B200Value rhs, B200Error* err) {    \
    clear_error(err);                                                              \
    Node* n = nullptr;                                                             \
    Status s = binary_impl(ctx, Op::OP, lhs, rhs, &n);                             \
    return ret(err, s, n);                                                         \
  }
B200_BINARY(b200_add, Add) B200_BINARY(b200_sub, Sub) B200_BINARY(b200_mul, Mul) B200_BINARY(b200_div, Div)
B200_BINARY(b200_rem, Rem) B200_BINARY(b200_pow, Pow) B200_BINARY(b200_max, Max) B200_BINARY(b200_min, Min)
B200_BINARY(b200_atan2, Atan2) B200_BINARY(b200_logical_and, LogicalAnd) B200_BINARY(b200_logical_or, LogicalOr)
B200_BINARY(b200_logical_xor, LogicalXor) B200_BINARY(b200_bitwise_and, BitwiseAnd) B200_BINARY(b200_bitwise_or, BitwiseOr)
B200_BINARY(b200_bitwise_xor, BitwiseXor) B200_BINARY(b200_shift_left, ShiftLeft) B200_BINARY(b200_shift_right, ShiftRight)
B200_BINARY(b200_shift_right_logical, ShiftRightLogical)
B200_BINARY(b200_equal, Equal) B200_BINARY(b200_not_equal, NotEqual) B200_BINARY(b200_less_than, LessThan)
B200_BINARY(b200_less_or_equal, LessOrEqual) B200_BINARY(b200_greater_than, GreaterThan)
B200_BINARY(b200_greater_or_equal, GreaterOrEqual)
#undef B200_BINARY

// ---- shape ops ----------------------------------------------------------------
B200Value b200_reshape(B200Context ctx, B200Value x, const int64_t* shape, int rank, B200Error* err) {
  clear_error(err);
  Node* n;
  Status s = check_node(ctx, x, "Reshape", &n);
  if (s.ok()) s = check_shape("Reshape", shape, rank);
  if (!s.ok()) return ret(err, s, nullptr);
  int64_t count = 1;
  for (int i = 0; i < rank; ++i) count *= shape[i];
  if (count != n->num_elements())
    return ret(err, Status::Invalid(strfmt("Reshape: %s has %lld elements, target %s has %lld", dims_str(n->dims).c_str(),
                                           (long long)n->num_elements(), dims_str(std::vector<int64_t>(shape, shape + rank)).c_str(),
                                           (long long)count)), nullptr);
  Graph& g = reinterpret_cast<Ctx*>(ctx)->graph;
  return ret(err, Status::OK(), g.Add(Op::Reshape, n->dtype, std::vector<int64_t>(shape, shape + rank), {n}));
}

B200Value b200_transpose(B200Context ctx, B200Value x, const int* permutation, int rank, B200Error* err) {
  clear_error(err);
  Node* n;
  Status s = check_node(ctx, x, "Transpose", &n);
  if (!s.ok()) return ret(err, s, nullptr);
  if (rank != n->rank()) return ret(err, Status::Invalid(strfmt("Transpose: %d permutation entries for rank %d", rank, n->rank())), nullptr);
  std::vector<bool> seen(rank, false);
  std::vector<int64_t> dims(rank);
  Graph& g = reinterpret_cast<Ctx*>(ctx)->graph;
  std::vector<int64_t> perm(rank);
  for (int i = 0; i < rank; ++i) {
    const int p = permutation[i];
    if (p < 0 || p >= rank || seen[p]) return ret(err, Status::Invalid("Transpose: not a permutation"), nullptr);
    seen[p] = true;
    dims[i] = n->dims[p];
    perm[i] = p;
  }
  Node* t = g.Add(Op::Transpose, n->dtype, dims, {n});
  t->ia = perm;
  return ret(err, Status::OK(), t);
}

B200Value b200_cast(B200Context ctx, B200Value x, int dtype, B200Error* err) {
  clear_error(err);
  Node* n;
  Status s = check_node(ctx, x, "ConvertDType", &n);
  if (!s.ok()) return ret(err, s, nullptr);
  if (!dtype_valid(dtype)) return ret(err, Status::Invalid("ConvertDType: bad dtype"), nullptr);
  Graph& g = reinterpret_cast<Ctx*>(ctx)->graph;
  if (dtype == n->dtype) return ret(err, Status::OK(), g.Add(Op::Identity, dtype, n->dims, {n}));
  return ret(err, Status::OK(), g.Add(Op::Cast, dtype, n->dims, {n}));
}

B200Value b200_broadcast_in_dim(B200Context ctx, B200Value x, const int64_t* shape, int rank, const int* broadcast_axes,
                                int num_axes, B200Error* err) {
  clear_error(err);
  Node* n;
  Status s = check_node(ctx, x, "BroadcastInDim", &n);
  if (s.ok()) s = check_shape("BroadcastInDim", shape, rank);
  if (!s.ok()) return ret(err, s, nullptr);
  if (num_axes != n->rank())
    return ret(err, Status::Invalid(strfmt("BroadcastInDim: %d broadcast axes for operand rank %d", num_axes, n->rank())), nullptr);
  std::vector<int64_t> axes(num_axes);
  std::vector<bool> seen(rank, false);
  for (int i = 0; i < num_axes; ++i) {
    const int a = broadcast_axes[i];
    if (a < 0 || a >= rank || seen[a]) return ret(err, Status::Invalid("BroadcastInDim: bad broadcast axis"), nullptr);
    seen[a] = true;
    if (n->dims[i] != 1 && n->dims[i] != shape[a])
      return ret(err, Status::Invalid(strfmt("BroadcastInDim: operand dim %d (%lld) does not match output dim %d (%lld)", i,
                                             (long long)n->dims[i], a, (long long)shape[a])), nullptr);
    axes[i] = a;
  }
  Graph& g = reinterpret_cast<Ctx*>(ctx)->graph;
  Node* b = g.Add(Op::BroadcastInDim, n->dtype, std::vector<int64_t>(shape, shape + rank), {n});
  b->ia = axes;
  return ret(err, Status::OK(), b);
}

B200Value b200_broadcast_to(B200Context ctx, B200Value x, const int64_t* shape, int rank, B200Error* err) {
  clear_error(err);
  Node* n;
  Status s = check_node(ctx, x, "BroadcastTo", &n);
  if (!s.ok()) return ret(err, s, nullptr);
  if (rank < n->rank()) return ret(err, Status::Invalid("BroadcastTo: target rank smaller than operand rank"), nullptr);
  std::vector<int> axes(n->rank());
  for (int i = 0; i < n->rank(); ++i) axes[i] = rank - n->rank() + i;
  return b200_broadcast_in_dim(ctx, x, shape, rank, axes.data(), n->rank(), err);
}

B200Value b200_slice(B200Context ctx, B200Value x, const int64_t* starts, const int64_t* ends, const int64_t* strides,
                     int rank, B200Error* err) {
  clear_error(err);
  Node* n;
  Status s = check_node(ctx, x, "Slice", &n);
  if (!s.ok()) return ret(err, s, nullptr);
  if (rank != n->rank()) return ret(err, Status::Invalid(strfmt("Slice: %d bounds for rank %d", rank, n->rank())), nullptr);
  std::vector<int64_t> dims(rank), attrs;
  for (int i = 0; i < rank; ++i) {
    const int64_t st = strides ? strides[i] : 1;
    if (st < 1 || starts[i] < 0 || ends[i] > n->dims[i] || starts[i] > ends[i])
      return ret(err, Status::Invalid(strfmt("Slice: axis %d bounds [%lld:%lld:%lld] invalid for dim %lld", i, (long long)starts[i],
                                             (long long)ends[i], (long long)st, (long long)n->dims[i])), nullptr);
    dims[i] = (ends[i] - starts[i] + st - 1) / st;
    attrs.push_back(starts[i]);
    attrs.push_back(st);
  }
  Graph& g = reinterpret_cast<Ctx*>(ctx)->graph;
  Node* o = g.Add(Op::Slice, n->dtype, dims, {n});
  o->ia = attrs;  // (start, stride) per axis
  return ret(err, Status::OK(), o);
}

B200Value b200_concatenate(B200Context ctx, const B200Value* tensors, int num_tensors, int axis, B200Error* err) {
  clear_error(err);
  if (num_tensors < 1 || !tensors) return ret(err, Status::Invalid("Concatenate: no operands"), nullptr);
  std::vector<Node*> in(num_tensors);
  for (int i = 0; i < num_tensors; ++i) {
    Status s = check_node(ctx, tensors[i], "Concatenate", &in[i]);
    if (!s.ok()) return ret(err, s, nullptr);
  }
  int a;
  Status s = normalize_axis("Concatenate", axis, in[0]->rank(), &a);
  if (!s.ok()) return ret(err, s, nullptr);
  std::vector<int64_t> dims = in[0]->dims;
  for (int i = 1; i < num_tensors; ++i) {
    if (in[i]->dtype != in[0]->dtype || in[i]->rank() != in[0]->rank())
      return ret(err, Status::Invalid("Concatenate: operands differ in dtype or rank"), nullptr);
    for (int d = 0; d < in[0]->rank(); ++d)
      if (d != a && in[i]->dims[d] != in[0]->dims[d]) return ret(err, Status::Invalid("Concatenate: operand shapes differ off the axis"), nullptr);
    dims[a] += in[i]->dims[a];
  }
  Graph& g = reinterpret_cast<Ctx*>(ctx)->graph;
  Node* o = g.Add(Op::Concatenate, in[0]->dtype, dims, in);
  o->ia = {a};
  return ret(err, Status::OK(), o);
}

// ---- dynamic slices (ref function.go:1571-1621) ------------------------------------------------
static Status dynamic_starts(B200Context ctx, const char* what, Node* operand, const B200Value* start_indices, int num_indices,
                             std::vector<Node*>* starts) {
  if (num_indices != operand->rank()) return Status::Invalid(strfmt("%s: %d start indices for an operand of rank %d", what, num_indices, operand->rank()));
  if (operand->rank() > 8) return Status::Unsupported(strfmt("%s: more than 8 dims", what));
  for (int i = 0; i < num_indices; ++i) {
    Node* n;
    B200_TRY(check_node(ctx, start_indices[i], what, &n));
    if (n->num_elements() != 1 || !dtype_is_int(n->dtype)) return Status::Invalid(strfmt("%s: start index %d must be one integer value", what, i));
    starts->push_back(n);
  }
  return Status::OK();
}

B200Value b200_dynamic_slice(B200Context ctx, B200Value operand, const B200Value* start_indices, int num_indices,
                             const int64_t* slice_sizes, int rank, B200Error* err) {
  clear_error(err);
  Node* n;
  Status s = check_node(ctx, operand, "DynamicSlice", &n);
  if (!s.ok()) return ret(err, s, nullptr);
  if (rank != n->rank() || (rank > 0 && !slice_sizes)) return ret(err, Status::Invalid("DynamicSlice: one slice size per axis"), nullptr);
  std::vector<Node*> starts;
  s = dynamic_starts(ctx, "DynamicSlice", n, start_indices, num_indices, &starts);
  if (!s.ok()) return ret(err, s, nullptr);
  std::vector<int64_t> dims(rank);
  for (int i = 0; i < rank; ++i) {
    if (slice_sizes[i] < 0 || slice_sizes[i] > n->dims[i])
      return ret(err, Status::Invalid(strfmt("DynamicSlice: slice size %lld on axis %d exceeds dim %lld", (long long)slice_sizes[i], i, (long long)n->dims[i])), nullptr);
    dims[i] = slice_sizes[i];
  }
  std::vector<Node*> in = {n};
  in.insert(in.end(), starts.begin(), starts.end());
  Graph& g = reinterpret_cast<Ctx*>(ctx)->graph;
  return ret(err, Status::OK(), g.Add(Op::DynamicSlice, n->dtype, dims, in));
}

B200Value b200_dynamic_update_slice(B200Context ctx, B200Value operand, B200Value update, const B200Value* start_indices,
                                    int num_indices, B200Error* err) {
  clear_error(err);
  Node *n, *u;
  Status s = check_node(ctx, operand, "DynamicUpdateSlice: operand", &n);
  if (s.ok()) s = check_node(ctx, update, "DynamicUpdateSlice: update", &u);
  if (!s.ok()) return ret(err, s, nullptr);
  if (u->dtype != n->dtype || u->rank() != n->rank()) return ret(err, Status::Invalid("DynamicUpdateSlice: update differs from the operand in dtype or rank"), nullptr);
  for (int i = 0; i < n->rank(); ++i)
    if (u->dims[i] > n->dims[i]) return ret(err, Status::Invalid(strfmt("DynamicUpdateSlice: update dim %d (%lld) exceeds operand dim %lld", i, (long long)u->dims[i], (long long)n->dims[i])), nullptr);
  std::vector<Node*> starts;
  s = dynamic_starts(ctx, "DynamicUpdateSlice", n, start_indices, num_indices, &starts);
  if (!s.ok()) return ret(err, s, nullptr);
  std::vector<Node*> in = {n, u};
  in.insert(in.end(), starts.begin(), starts.end());
  Graph& g = reinterpret_cast<Ctx*>(ctx)->graph;
  return ret(err, Status::OK(), g.Add(Op::DynamicUpdateSlice, n->dtype, n->dims, in));
}

B200Value b200_reverse(B200Context ctx, B200Value x, const int* axes, int num_axes, B200Error* err) {
  clear_error(err);
  Node* n;
  Status s = check_node(ctx, x, "Reverse", &n);
  if (!s.ok()) return ret(err, s, nullptr);
  std::vector<int64_t> ax;
  for (int i = 0; i < num_axes; ++i) {
    int a;
    s = normalize_axis("Reverse", axes[i], n->rank(), &a);
    if (!s.ok()) return ret(err, s, nullptr);
    ax.push_back(a);
  }
  Graph& g = reinterpret_cast<Ctx*>(ctx)->graph;
  Node* o = g.Add(Op::Reverse, n->dtype, n->dims, {n});
  o->ia = ax;
  return ret(err, Status::OK(), o);
}

B200Value b200_pad(B200Context ctx, B200Value x, B200Value pad_value, const int64_t* pad_before, const int64_t* pad_after,
                   int rank, B200Error* err) {
  clear_error(err);
  Node *n, *pv;
  Status s = check_node(ctx, x, "Pad", &n);
  if (s.ok()) s = check_node(ctx, pad_value, "Pad", &pv);
  if (!s.ok()) return ret(err, s, nullptr);
  if (rank != n->rank()) return ret(err, Status::Invalid("Pad: rank mismatch"), nullptr);
  if (pv->num_elements() != 1 || pv->dtype != n->dtype) return ret(err, Status::Invalid("Pad: fill value must be one element of the operand dtype"), nullptr);
  std::vector<int64_t> dims(rank), attrs;
  for (int i = 0; i < rank; ++i) {
    if (pad_before[i] < 0 || pad_after[i] < 0) return ret(err, Status::Unsupported("Pad: negative padding"), nullptr);
    dims[i] = n->dims[i] + pad_before[i] + pad_after[i];
    attrs.push_back(pad_before[i]);
  }
  Graph& g = reinterpret_cast<Ctx*>(ctx)->graph;
  Node* o = g.Add(Op::Pad, n->dtype, dims, {n, pv});
  o->ia = attrs;
  return ret(err, Status::OK(), o);
}

// ---- selection ----------------------------------------------------------------
B200Value b200_where(B200Context ctx, B200Value cond, B200Value on_true, B200Value on_false, B200Error* err) {
  clear_error(err);
  Node *c, *t, *f;
  Status s = check_node(ctx, cond, "Where", &c);
  if (s.ok()) s = check_node(ctx, on_true, "Where", &t);
  if (s.ok()) s = check_node(ctx, on_false, "Where", &f);
  if (!s.ok()) return ret(err, s, nullptr);
  if (c->dtype != B200_BOOL) return ret(err, Status::Invalid("Where: condition must be Bool"), nullptr);
  if (t->dtype != f->dtype) return ret(err, Status::Invalid("Where: branch dtypes differ"), nullptr);
  std::vector<int64_t> d1, d2;
  s = broadcast_shapes("Where", t->dims, f->dims, &d1);
  if (s.ok()) s = broadcast_shapes("Where", c->dims, d1, &d2);
  if (!s.ok()) return ret(err, s, nullptr);
  Graph& g = reinterpret_cast<Ctx*>(ctx)->graph;
  return ret(err, Status::OK(), g.Add(Op::Where, t->dtype, d2, {c, t, f}));
}

B200Value b200_clamp(B200Context ctx, B200Value min_val, B200Value x, B200Value max_val, B200Error* err) {
  clear_error(err);
  Node *lo, *n, *hi;
  Status s = check_node(ctx, min_val, "Clamp", &lo);
  if (s.ok()) s = check_node(ctx, x, "Clamp", &n);
  if (s.ok()) s = check_node(ctx, max_val, "Clamp", &hi);
  if (!s.ok()) return ret(err, s, nullptr);
  if (lo->dtype != n->dtype || hi->dtype != n->dtype) return ret(err, Status::Invalid("Clamp: dtypes differ"), nullptr);
  std::vector<int64_t> d1, d2;
  s = broadcast_shapes("Clamp", lo->dims, n->dims, &d1);
  if (s.ok()) s = broadcast_shapes("Clamp", d1, hi->dims, &d2);
  if (!s.ok()) return ret(err, s, nullptr);
  Graph& g = reinterpret_cast<Ctx*>(ctx)->graph;
  return ret(err, Status::OK(), g.Add(Op::Clamp, n->dtype, d2, {lo, n, hi}));
}

// ---- contraction ----------------------------------------------------------------
B200Value b200_dot_general(B200Context ctx, B200Value lhs, const int* lhs_contracting, int num_lhs_contracting,
                           const int* lhs_batch, int num_lhs_batch, B200Value rhs, const int* rhs_contracting,
                           int num_rhs_contracting, const int* rhs_batch, int num_rhs_batch, B200Error* err) {
  clear_error(err);
  Node *a, *b;
  Status s = check_node(ctx, lhs, "DotGeneral", &a);
  if (s.ok()) s = check_node(ctx, rhs, "DotGeneral", &b);
  if (!s.ok()) return ret(err, s, nullptr);
  if (a->dtype != b->dtype)
    return ret(err, Status::Invalid(strfmt("DotGeneral: operand dtypes differ (%s vs %s)", dtype_name(a->dtype), dtype_name(b->dtype))), nullptr);
  if (a->dtype == B200_BOOL) return ret(err, Status::Invalid("DotGeneral: Bool operands"), nullptr);
  if (num_lhs_contracting != num_rhs_contracting || num_lhs_batch != num_rhs_batch)
    return ret(err, Status::Invalid("DotGeneral: lhs and rhs must name the same number of contracting and of batch axes"), nullptr);
  auto norm = [&](const int* axes, int n, int rank, std::vector<int64_t>* out) -> Status {
    for (int i = 0; i < n; ++i) {
      int ax;
      B200_TRY(normalize_axis("DotGeneral", axes[i], rank, &ax));
      out->push_back(ax);
    }
    return Status::OK();
  };
  std::vector<int64_t> lc, lb, rc, rb;
  s = norm(lhs_contracting, num_lhs_contracting, a->rank(), &lc);
  if (s.ok()) s = norm(lhs_batch, num_lhs_batch, a->rank(), &lb);
  if (s.ok()) s = norm(rhs_contracting, num_rhs_contracting, b->rank(), &rc);
  if (s.ok()) s = norm(rhs_batch, num_rhs_batch, b->rank(), &rb);
  if (!s.ok()) return ret(err, s, nullptr);
  std::set<int64_t> lset(lc.begin(), lc.end()), rset(rc.begin(), rc.end());
  lset.insert(lb.begin(), lb.end());
  rset.insert(rb.begin(), rb.end());
  if (lset.size() != lc.size() + lb.size() || rset.size() != rc.size() + rb.size())
    return ret(err, Status::Invalid("DotGeneral: an axis is named twice"), nullptr);
  for (size_t i = 0; i < lc.size(); ++i)
    if (a->dims[lc[i]] != b->dims[rc[i]])
      return ret(err, Status::Invalid(strfmt("DotGeneral: contracting dims differ (%lld vs %lld)", (long long)a->dims[lc[i]], (long long)b->dims[rc[i]])), nullptr);
  for (size_t i = 0; i < lb.size(); ++i)
    if (a->dims[lb[i]] != b->dims[rb[i]])
      return ret(err, Status::Invalid(strfmt("DotGeneral: batch dims differ (%lld vs %lld)", (long long)a->dims[lb[i]], (long long)b->dims[rb[i]])), nullptr);
  // Output dims: batch ++ lhs free ++ rhs free (ref dotgeneral.go:34-50).
  std::vector<int64_t> dims;
  for (auto ax : lb) dims.push_back(a->dims[ax]);
  for (int i = 0; i < a->rank(); ++i)
    if (!lset.count(i)) dims.push_back(a->dims[i]);
  for (int i = 0; i < b->rank(); ++i)
    if (!rset.count(i)) dims.push_back(b->dims[i]);
  Graph& g = reinterpret_cast<Ctx*>(ctx)->graph;
  Node* o = g.Add(Op::DotGeneral, a->dtype, dims, {a, b});
  // ia = [nc, nb, lc..., lb..., rc..., rb...]; optional bias is in[2]; fa[0] = activation
  o->ia = {(int64_t)lc.size(), (int64_t)lb.size()};
  o->ia.insert(o->ia.end(), lc.begin(), lc.end());
  o->ia.insert(o->ia.end(), lb.begin(), lb.end());
  o->ia.insert(o->ia.end(), rc.begin(), rc.end());
  o->ia.insert(o->ia.end(), rb.begin(), rb.end());
  o->fa = {(double)B200_ACT_NONE};
  return ret(err, Status::OK(), o);
}

B200Value b200_matmul(B200Context ctx, B200Value lhs, B200Value rhs, B200Error* err) {
  clear_error(err);
  Node *a, *b;
  Status s = check_node(ctx, lhs, "MatMul", &a);
  if (s.ok()) s = check_node(ctx, rhs, "MatMul", &b);
  if (!s.ok()) return ret(err, s, nullptr);
  if (a->rank() < 2 || a->rank() != b->rank()) return ret(err, Status::Invalid("MatMul: operands need equal rank >= 2"), nullptr);
  const int r = a->rank();
  std::vector<int> batch(r - 2);
  for (int i = 0; i < r - 2; ++i) batch[i] = i;
  const int lc = r - 1, rc = r - 2;
  return b200_dot_general(ctx, lhs, &lc, 1, batch.data(), r - 2, rhs, &rc, 1, batch.data(), r - 2, err);
}

// ---- reductions -----------------------------------------------------------------
B200Value b200_reduce(B200Context ctx, B200Value x, int reduce_type, const int* axes, int num_axes, B200Error* err) {
  clear_error(err);
  Node* n;
  Status s = check_node(ctx, x, "Reduce", &n);
  if (!s.ok()) return ret(err, s, nullptr);
  if (reduce_type < 0 || reduce_type > 3) return ret(err, Status::Invalid("Reduce: bad reduce type"), nullptr);
  std::set<int64_t> ax;
  if (num_axes == 0) {
    for (int i = 0; i < n->rank(); ++i) ax.insert(i);  // empty = all (ref function.go:1153-1158)
  } else {
    for (int i = 0; i < num_axes; ++i) {
      int a;
      s = normalize_axis("Reduce", axes[i], n->rank(), &a);
      if (!s.ok()) return ret(err, s, nullptr);
      if (!ax.insert(a).second) return ret(err, Status::Invalid("Reduce: axis named twice"), nullptr);
    }
  }
  std::vector<int64_t> dims;
  for (int i = 0; i < n->rank(); ++i)
    if (!ax.count(i)) dims.push_back(n->dims[i]);
  Graph& g = reinterpret_cast<Ctx*>(ctx)->graph;
  Node* o = g.Add(Op::Reduce, n->dtype, dims, {n});
  o->ia = {reduce_type};
  o->ia.insert(o->ia.end(), ax.begin(), ax.end());
  return ret(err, Status::OK(), o);
}

static B200Value argminmax(B200Context ctx, B200Value x, int axis, int output_dtype, bool is_min, B200Error* err) {
  clear_error(err);
  Node* n;
  Status s = check_node(ctx, x, "ArgMinMax", &n);
  if (!s.ok()) return ret(err, s, nullptr);
  int a;
  s = normalize_axis("ArgMinMax", axis, n->rank(), &a);
  if (!s.ok()) return ret(err, s, nullptr);
  if (!dtype_is_int(output_dtype)) return ret(err, Status::Invalid("ArgMinMax: output dtype must be an integer type"), nullptr);
  if (n->dtype == B200_BOOL) return ret(err, Status::Invalid("ArgMinMax: Bool operand"), nullptr);
  if (n->dims[a] == 0) return ret(err, Status::Invalid("ArgMinMax: reduced axis has size 0"), nullptr);
  std::vector<int64_t> dims;
  for (int i = 0; i < n->rank(); ++i)
    if (i != a) dims.push_back(n->dims[i]);
  Graph& g = reinterpret_cast<Ctx*>(ctx)->graph;
  Node* o = g.Add(Op::ArgMinMax, output_dtype, dims, {n});
  o->ia = {a, is_min ? 1 : 0};
  return ret(err, Status::OK(), o);
}
B200Value b200_argmin(B200Context ctx, B200Value x, int axis, int output_dtype, B200Error* err) {
  return argminmax(ctx, x, axis, output_dtype, true, err);
}
B200Value b200_argmax(B200Context ctx, B200Value x, int axis, int output_dtype, B200Error* err) {
  return argminmax(ctx, x, axis, output_dtype, false, err);
}

// ---- gather ---------------------------------------------------------------------
B200Value b200_gather(B200Context ctx, B200Value operand, B200Value start_indices, int index_vector_axis,
                      const int* offset_output_axes, int num_offset_output_axes, const int* collapsed_slice_axes,
                      int num_collapsed_slice_axes, const int* start_index_map, int num_start_index_map,
                      const int64_t* slice_sizes, int num_slice_sizes, bool indices_are_sorted, B200Error* err) {
  (void)indices_are_sorted;
  clear_error(err);
  Node *op, *idx;
  Status s = check_node(ctx, operand, "Gather", &op);
  if (s.ok()) s = check_node(ctx, start_indices, "Gather", &idx);
  if (!s.ok()) return ret(err, s, nullptr);
  if (!dtype_is_int(idx->dtype)) return ret(err, Status::Invalid("Gather: start indices must be integers"), nullptr);
  const int orank = op->rank(), irank = idx->rank();
  if (num_slice_sizes != orank) return ret(err, Status::Invalid("Gather: sliceSizes must have one entry per operand axis"), nullptr);
  if (index_vector_axis < 0 || index_vector_axis > irank) return ret(err, Status::Invalid("Gather: indexVectorAxis out of range"), nullptr);
  // indexVectorAxis == rank means an implicit trailing axis of size 1.
  const int64_t ncomp = index_vector_axis == irank ? 1 : idx->dims[index_vector_axis];
  if (ncomp != num_start_index_map) return ret(err, Status::Invalid("Gather: startIndexMap length must equal the index vector size"), nullptr);
  std::set<int> collapsed;
  for (int i = 0; i < num_collapsed_slice_axes; ++i) {
    const int a = collapsed_slice_axes[i];
    if (a < 0 || a >= orank || !collapsed.insert(a).second) return ret(err, Status::Invalid("Gather: bad collapsedSliceAxes"), nullptr);
    if (slice_sizes[a] != 1) return ret(err, Status::Invalid("Gather: a collapsed axis must have slice size 1"), nullptr);
  }
  for (int i = 0; i < orank; ++i)
    if (slice_sizes[i] < 0 || slice_sizes[i] > op->dims[i]) return ret(err, Status::Invalid("Gather: slice size out of range"), nullptr);
  for (int i = 0; i < num_start_index_map; ++i)
    if (start_index_map[i] < 0 || start_index_map[i] >= orank) return ret(err, Status::Invalid("Gather: bad startIndexMap"), nullptr);
  if (num_offset_output_axes != orank - num_collapsed_slice_axes)
    return ret(err, Status::Invalid("Gather: offsetOutputAxes must have one entry per non-collapsed operand axis"), nullptr);
  const int batch_rank = index_vector_axis == irank ? irank : irank - 1;
  const int out_rank = batch_rank + num_offset_output_axes;
  std::set<int> offset_axes;
  for (int i = 0; i < num_offset_output_axes; ++i) {
    const int a = offset_output_axes[i];
    if (a < 0 || a >= out_rank || !offset_axes.insert(a).second) return ret(err, Status::Invalid("Gather: bad offsetOutputAxes"), nullptr);
    if (i > 0 && offset_output_axes[i] <= offset_output_axes[i - 1]) return ret(err, Status::Invalid("Gather: offsetOutputAxes must ascend"), nullptr);
  }
  std::vector<int64_t> batch_dims, offset_dims, dims(out_rank);
  for (int i = 0; i < irank; ++i)
    if (i != index_vector_axis) batch_dims.push_back(idx->dims[i]);
  for (int i = 0; i < orank; ++i)
    if (!collapsed.count(i)) offset_dims.push_back(slice_sizes[i]);
  size_t bi = 0, oi = 0;
  for (int d = 0; d < out_rank; ++d) dims[d] = offset_axes.count(d) ? offset_dims[oi++] : batch_dims[bi++];
  Graph& g = reinterpret_cast<Ctx*>(ctx)->graph;
  Node* o = g.Add(Op::Gather, op->dtype, dims, {op, idx});
  // ia = [index_vector_axis, n_off, off..., n_col, col..., n_map, map..., n_ss, ss...]
  o->ia = {index_vector_axis, num_offset_output_axes};
  for (int i = 0; i < num_offset_output_axes; ++i) o->ia.push_back(offset_output_axes[i]);
  o->ia.push_back(num_collapsed_slice_axes);
  for (int i = 0; i < num_collapsed_slice_axes; ++i) o->ia.push_back(collapsed_slice_axes[i]);
  o->ia.push_back(num_start_index_map);
  for (int i = 0; i < num_start_index_map; ++i) o->ia.push_back(start_index_map[i]);
  o->ia.push_back(num_slice_sizes);
  for (int i = 0; i < num_slice_sizes; ++i) o->ia.push_back(slice_sizes[i]);
  return ret(err, Status::OK(), o);
}

// out[..., i, ...] = x[..., indices[..., i, ...], ...] along `axis`; indices has x's rank.
// Expressed as an XLA gather over flattened coordinates is awkward, so it is
// lowered to: Iota coordinates for the other axes are implicit in the general
// gather kernel through a full index tensor built here from primitives.
B200Value b200_gather_along_axis(B200Context ctx, B200Value x, B200Value indices, int axis, B200Error* err) {
  clear_error(err);
  Node *n, *idx;
  Status s = check_node(ctx, x, "GatherAlongAxis", &n);
  if (s.ok()) s = check_node(ctx, indices, "GatherAlongAxis", &idx);
  if (!s.ok()) return ret(err, s, nullptr);
  int a;
  s = normalize_axis("GatherAlongAxis", axis, n->rank(), &a);
  if (!s.ok()) return ret(err, s, nullptr);
  if (idx->rank() != n->rank() || !dtype_is_int(idx->dtype)) return ret(err, Status::Invalid("GatherAlongAxis: indices must be integers of the operand's rank"), nullptr);
  for (int d = 0; d < n->rank(); ++d)
    if (d != a && idx->dims[d] != n->dims[d]) return ret(err, Status::Invalid("GatherAlongAxis: index shape must match the operand off the axis"), nullptr);
  // Build a [.., rank] coordinate tensor: coordinate d is Iota(d) except on `axis`, where it is the index.
  const int r = n->rank();
  std::vector<int64_t> ext = idx->dims;
  ext.push_back(1);
  std::vector<B200Value> parts;
  for (int d = 0; d < r; ++d) {
    B200Value c;
    if (d == a) c = b200_reshape(ctx, indices, ext.data(), r + 1, err);
    else c = b200_iota(ctx, idx->dtype, ext.data(), r + 1, d, err);
    if (!c) return nullptr;
    parts.push_back(c);
  }
  B200Value coords = b200_concatenate(ctx, parts.data(), r, r, err);
  if (!coords) return nullptr;
  std::vector<int> collapsed(r), map(r);
  std::vector<int64_t> ss(r, 1);
  for (int d = 0; d < r; ++d) collapsed[d] = map[d] = d;
  return b200_gather(ctx, x, coords, r, nullptr, 0, collapsed.data(), r, map.data(), r, ss.data(), r, false, err);
}

// ---- fused ops ------------------------------------------------------------------
B200Value b200_softmax(B200Context ctx, B200Value x, int axis, B200Error* err) {
  clear_error(err);
  Node* n;
  Status s = check_node(ctx, x, "FusedSoftmax", &n);
  if (!s.ok()) return ret(err, s, nullptr);
  int a;
  s = normalize_axis("FusedSoftmax", axis, n->rank(), &a);
  if (!s.ok()) return ret(err, s, nullptr);
  if (!dtype_is_float(n->dtype)) return ret(err, Status::Invalid("FusedSoftmax: needs a float operand"), nullptr);
  Graph& g = reinterpret_cast<Ctx*>(ctx)->graph;
  Node* o = g.Add(Op::Softmax, n->dtype, n->dims, {n});
  o->ia = {a};
  return ret(err, Status::OK(), o);
}

B200Value b200_softmax_masked(B200Context ctx, B200Value x, double scale, int causal, B200Value mask, B200Error* err) {
  clear_error(err);
  Node *n, *m = nullptr;
  Status s = check_node(ctx, x, "SoftmaxMasked", &n);
  if (s.ok() && mask) s = check_node(ctx, mask, "SoftmaxMasked", &m);
  if (!s.ok()) return ret(err, s, nullptr);
  if (!dtype_is_float(n->dtype) || n->dtype == B200_FLOAT64) return ret(err, Status::Invalid("SoftmaxMasked: needs a 16/32-bit float operand"), nullptr);
  if (n->rank() < 2) return ret(err, Status::Invalid("SoftmaxMasked: operand needs rank >= 2 ([..., Sq, Sk])"), nullptr);
  if (m) {
    if (m->dtype != B200_BOOL && m->dtype != n->dtype) return ret(err, Status::Invalid("SoftmaxMasked: mask must be Bool or of the operand dtype"), nullptr);
    if (m->rank() > n->rank()) return ret(err, Status::Invalid("SoftmaxMasked: mask rank exceeds operand rank"), nullptr);
    const int off = n->rank() - m->rank();
    for (int i = 0; i < m->rank(); ++i)
      if (m->dims[i] != 1 && m->dims[i] != n->dims[off + i]) return ret(err, Status::Invalid("SoftmaxMasked: mask does not broadcast to the scores"), nullptr);
  }
  Graph& g = reinterpret_cast<Ctx*>(ctx)->graph;
  std::vector<Node*> in = {n};
  if (m) in.push_back(m);
  Node* o = g.Add(Op::SoftmaxMasked, n->dtype, n->dims, in);
  o->ia = {causal ? 1 : 0};
  o->fa = {scale};
  return ret(err, Status::OK(), o);
}

static Status norm_common(B200Context ctx, const char* what, B200Value x, const int* axes, int num_axes, Node** xn,
                          std::vector<int64_t>* ax) {
  B200_TRY(check_node(ctx, x, what, xn));
  if (!dtype_is_float((*xn)->dtype)) return Status::Invalid(strfmt("%s: needs a float operand", what));
  if (num_axes < 1) return Status::Invalid(strfmt("%s: no axes", what));
  std::set<int64_t> seen;
  for (int i = 0; i < num_axes; ++i) {
    int a;
    B200_TRY(normalize_axis(what, axes[i], (*xn)->rank(), &a));  // negative axes allowed (ref function.go:2417-2428)
    if (!seen.insert(a).second) return Status::Invalid(strfmt("%s: axis named twice", what));
  }
  ax->assign(seen.begin(), seen.end());
  return Status::OK();
}

// gamma / beta of lower rank are laid onto the normalised axes in order
// (ref function.go:2499-2530); equal-rank ones broadcast as they are.
static Status check_scale(const char* what, Node* x, Node* p, const std::vector<int64_t>& axes) {
  if (p->dtype != x->dtype) return Status::Invalid(strfmt("%s: gamma/beta dtype differs from the operand", what));
  if (p->rank() >= x->rank()) {
    if (p->rank() > x->rank()) return Status::Invalid(strfmt("%s: gamma/beta rank exceeds operand rank", what));
    for (int i = 0; i < x->rank(); ++i)
      if (p->dims[i] != 1 && p->dims[i] != x->dims[i]) return Status::Invalid(strfmt("%s: gamma/beta does not broadcast", what));
    return Status::OK();
  }
  if (p->rank() > (int)axes.size()) return Status::Invalid(strfmt("%s: gamma/beta rank exceeds the number of normalised axes", what));
  for (int i = 0; i < p->rank(); ++i)
    if (p->dims[i] != 1 && p->dims[i] != x->dims[axes[i]]) return Status::Invalid(strfmt("%s: gamma/beta does not match the normalised axes", what));
  return Status::OK();
}

B200Value b200_layer_norm(B200Context ctx, B200Value x, const int* axes, int num_axes, double epsilon, B200Value gamma,
                          B200Value beta, B200Error* err) {
  clear_error(err);
  Node *n, *g_ = nullptr, *b_ = nullptr;
  std::vector<int64_t> ax;
  Status s = norm_common(ctx, "FusedLayerNorm", x, axes, num_axes, &n, &ax);
  if (s.ok() && gamma) s = check_node(ctx, gamma, "FusedLayerNorm: gamma", &g_);
  if (s.ok() && beta) s = check_node(ctx, beta, "FusedLayerNorm: beta", &b_);
  if (s.ok() && g_) s = check_scale("FusedLayerNorm", n, g_, ax);
  if (s.ok() && b_) s = check_scale("FusedLayerNorm", n, b_, ax);
  if (!s.ok()) return ret(err, s, nullptr);
  Graph& g = reinterpret_cast<Ctx*>(ctx)->graph;
  // A full-rank gamma/beta that varies along a non-normalised axis cannot be a
  // per-column vector: normalise first, then scale and shift as elementwise ops.
  auto varies_off_axes = [&](Node* p) {
    if (!p || p->rank() < n->rank()) return false;
    for (int i = 0; i < n->rank(); ++i)
      if (p->dims[i] != 1 && !std::count(ax.begin(), ax.end(), (int64_t)i)) return true;
    return false;
  };
  const bool split = varies_off_axes(g_) || varies_off_axes(b_);
  std::vector<Node*> in = {n};
  // ia = [has_gamma, has_beta, axes...]
  if (g_ && !split) in.push_back(g_);
  if (b_ && !split) in.push_back(b_);
  Node* o = g.Add(Op::LayerNorm, n->dtype, n->dims, in);
  o->ia = {(g_ && !split) ? 1 : 0, (b_ && !split) ? 1 : 0};
  o->ia.insert(o->ia.end(), ax.begin(), ax.end());
  o->fa = {epsilon};
  if (split) {
    B200Value y = reinterpret_cast<B200Value>(o);
    if (g_) { y = b200_mul(ctx, y, gamma, err); if (!y) return nullptr; }
    if (b_) { y = b200_add(ctx, y, beta, err); if (!y) return nullptr; }
    return y;
  }
  return ret(err, Status::OK(), o);
}

B200Value b200_rms_norm(B200Context ctx, B200Value x, const int* axes, int num_axes, double epsilon, B200Value gamma,
                        B200Error* err) {
  clear_error(err);
  Node *n, *g_ = nullptr;
  std::vector<int64_t> ax;
  Status s = norm_common(ctx, "RMSNorm", x, axes, num_axes, &n, &ax);
  if (s.ok() && gamma) s = check_node(ctx, gamma, "RMSNorm: gamma", &g_);
  if (s.ok() && g_) s = check_scale("RMSNorm", n, g_, ax);
  if (!s.ok()) return ret(err, s, nullptr);
  Graph& g = reinterpret_cast<Ctx*>(ctx)->graph;
  std::vector<Node*> in = {n};
  if (g_) in.push_back(g_);
  Node* o = g.Add(Op::RmsNorm, n->dtype, n->dims, in);
  o->ia = {g_ ? 1 : 0, 0};
  o->ia.insert(o->ia.end(), ax.begin(), ax.end());
  o->fa = {epsilon};
  return ret(err, Status::OK(), o);
}

B200Value b200_gelu(B200Context ctx, B200Value x, int exact, B200Error* err) {
  clear_error(err);
  Node* n = nullptr;
  Status s = unary_impl(ctx, exact ? Op::GeluExact : Op::GeluTanh, x, &n);
  return ret(err, s, n);
}

B200Value b200_dense(B200Context ctx, B200Value x, B200Value weight, B200Value bias, int activation, B200Error* err) {
  clear_error(err);
  Node *xn, *wn, *bn = nullptr;
  Status s = check_node(ctx, x, "FusedDense: x", &xn);
  if (s.ok()) s = check_node(ctx, weight, "FusedDense: weight", &wn);
  if (s.ok() && bias) s = check_node(ctx, bias, "FusedDense: bias", &bn);
  if (!s.ok()) return ret(err, s, nullptr);
  if (xn->rank() < 1 || wn->rank() < 2)
    return ret(err, Status::Invalid(strfmt("FusedDense: x must have rank >= 1 (got %d), weight must have rank >= 2 (got %d)", xn->rank(), wn->rank())), nullptr);
  if (xn->dims.back() != wn->dims[0])
    return ret(err, Status::Invalid(strfmt("FusedDense: x's last dim (%lld) must match weight's first dim (%lld)", (long long)xn->dims.back(), (long long)wn->dims[0])), nullptr);
  if (activation < B200_ACT_NONE || activation > B200_ACT_TANH)
    return ret(err, Status::Invalid(strfmt("FusedDense: unsupported activation type %d", activation)), nullptr);
  const int lc = xn->rank() - 1, rc = 0;
  B200Value y = b200_dot_general(ctx, x, &lc, 1, nullptr, 0, weight, &rc, 1, nullptr, 0, err);
  if (!y) return nullptr;
  Node* yn = reinterpret_cast<Node*>(y);
  const bool float_epilogue = yn->dtype == B200_FLOAT32 || yn->dtype == B200_BFLOAT16 || yn->dtype == B200_FLOAT16;
  if (bn) {
    if (bn->dtype != yn->dtype || bn->rank() > yn->rank()) return ret(err, Status::Invalid("FusedDense: bias dtype or rank"), nullptr);
    // trailing-axis broadcast (ref function.go:2604-2612)
    const int off = yn->rank() - bn->rank();
    for (int i = 0; i < bn->rank(); ++i)
      if (bn->dims[i] != yn->dims[off + i]) return ret(err, Status::Invalid("FusedDense: bias shape does not match the output's trailing dims"), nullptr);
  }
  // The GEMM epilogue takes a bias vector over the N axis and an activation.
  const bool simple_bias = !bn || (bn->rank() == 1 && wn->rank() == 2);
  if (float_epilogue && simple_bias) {
    if (bn) yn->in.push_back(bn);
    yn->fa[0] = (double)activation;
    return y;
  }
  if (bn) {
    std::vector<int> axes(bn->rank());
    for (int i = 0; i < bn->rank(); ++i) axes[i] = yn->rank() - bn->rank() + i;
    B200Value bb = b200_broadcast_in_dim(ctx, bias, yn->dims.data(), yn->rank(), axes.data(), bn->rank(), err);
    if (!bb) return nullptr;
    y = b200_add(ctx, y, bb, err);
    if (!y) return nullptr;
  }
  Node* act = nullptr;
  Status as = Status::OK();
  switch (activation) {
    case B200_ACT_GELU: as = unary_impl(ctx, Op::GeluTanh, y, &act); break;
    case B200_ACT_RELU: as = unary_impl(ctx, Op::Relu, y, &act); break;
    case B200_ACT_SILU: as = unary_impl(ctx, Op::Silu, y, &act); break;
    case B200_ACT_TANH: as = unary_impl(ctx, Op::Tanh, y, &act); break;
    default: return y;
  }
  return ret(err, as, act);
}

bool b200_attention_qkv_projection(B200Context ctx, B200Value x, B200Value w_qkv, B200Value bias_q, B200Value bias_k,
                                   B200Value bias_v, int query_dim, int key_value_dim, B200Value* out_q, B200Value* out_k,
                                   B200Value* out_v, B200Error* err) {
  clear_error(err);
  Node *xn, *wn;
  Status s = check_node(ctx, x, "FusedAttentionQKVProjection: x", &xn);
  if (s.ok()) s = check_node(ctx, w_qkv, "FusedAttentionQKVProjection: wQKV", &wn);
  if (!s.ok()) { set_error(err, s); return false; }
  if (xn->rank() < 1) { set_error(err, Status::Invalid("FusedAttentionQKVProjection: x must have rank >= 1")); return false; }
  if (wn->rank() != 2 || wn->dims[1] != query_dim + 2 * (int64_t)key_value_dim) {
    set_error(err, Status::Invalid("FusedAttentionQKVProjection: wQKV must be [in, queryDim + 2*keyValueDim]"));
    return false;
  }
  const int lc = xn->rank() - 1, rc = 0;
  B200Value combined = b200_dot_general(ctx, x, &lc, 1, nullptr, 0, w_qkv, &rc, 1, nullptr, 0, err);
  if (!combined) return false;
  Node* cn = reinterpret_cast<Node*>(combined);
  const int r = cn->rank();
  // When every bias present is a plain vector of the right length, the three biases become ONE vector added in the
  // GEMM epilogue (absent ones are zeros), instead of three separate elementwise adds after the slices.
  bool fold = (bias_q || bias_k || bias_v) && (cn->dtype == B200_FLOAT32 || cn->dtype == B200_BFLOAT16 || cn->dtype == B200_FLOAT16);
  const int64_t want[3] = {query_dim, key_value_dim, key_value_dim};
  B200Value biases[3] = {bias_q, bias_k, bias_v};
  for (int i = 0; i < 3 && fold; ++i) {
    if (!biases[i]) continue;
    Node* bn;
    Status bs = check_node(ctx, biases[i], "FusedAttentionQKVProjection: bias", &bn);
    if (!bs.ok()) { set_error(err, bs); return false; }
    fold = bn->rank() == 1 && bn->dims[0] == want[i] && bn->dtype == cn->dtype;
  }
  if (fold) {
    Graph& g = reinterpret_cast<Ctx*>(ctx)->graph;
    B200Value parts[3];
    for (int i = 0; i < 3; ++i) {
      if (biases[i]) { parts[i] = biases[i]; continue; }
      Node* z = g.Add(Op::Constant, cn->dtype, {want[i]}, {});
      z->data.assign((size_t)want[i] * dtype_size(cn->dtype), 0);
      parts[i] = reinterpret_cast<B200Value>(z);
    }
    B200Value all = b200_concatenate(ctx, parts, 3, 0, err);
    if (!all) return false;
    cn->in.push_back(reinterpret_cast<Node*>(all));
    bias_q = bias_k = bias_v = nullptr;
  }
  auto part = [&](int64_t lo, int64_t hi, B200Value bias, B200Value* out) -> bool {
    std::vector<int64_t> st(r, 0), en(cn->dims), sd(r, 1);
    st[r - 1] = lo;
    en[r - 1] = hi;
    B200Value v = b200_slice(ctx, combined, st.data(), en.data(), sd.data(), r, err);
    if (!v) return false;
    if (bias) {
      Node* bn;
      Status bs = check_node(ctx, bias, "FusedAttentionQKVProjection: bias", &bn);
      if (!bs.ok()) { set_error(err, bs); return false; }
      Node* vn = reinterpret_cast<Node*>(v);
      std::vector<int> axes(bn->rank());
      for (int i = 0; i < bn->rank(); ++i) axes[i] = r - bn->rank() + i;
      B200Value bb = b200_broadcast_in_dim(ctx, bias, vn->dims.data(), r, axes.data(), bn->rank(), err);
      if (!bb) return false;
      v = b200_add(ctx, v, bb, err);
      if (!v) return false;
    }
    *out = v;
    return true;
  };
  return part(0, query_dim, bias_q, out_q) && part(query_dim, query_dim + key_value_dim, bias_k, out_k) &&
         part(query_dim + key_value_dim, query_dim + 2 * (int64_t)key_value_dim, bias_v, out_v);
}

B200Value b200_scaled_dot_product_attention(B200Context ctx, B200Value query, B200Value key, B200Value value, B200Value mask,
                                            int num_heads, int num_kv_heads, int axes_layout, double scale, int causal,
                                            B200Error* err) {
  clear_error(err);
  Node *q, *k, *v, *m = nullptr;
  Status s = check_node(ctx, query, "SDPA: query", &q);
  if (s.ok()) s = check_node(ctx, key, "SDPA: key", &k);
  if (s.ok()) s = check_node(ctx, value, "SDPA: value", &v);
  if (s.ok() && mask) s = check_node(ctx, mask, "SDPA: mask", &m);
  if (!s.ok()) return ret(err, s, nullptr);
  if (q->rank() != 4) return ret(err, Status::Invalid(strfmt("SDPA: query must have rank 4, got %d", q->rank())), nullptr);
  if (k->rank() != 4 || v->rank() != 4) return ret(err, Status::Invalid("SDPA: key and value must have rank 4"), nullptr);
  if (num_heads <= 0 || num_kv_heads <= 0 || num_heads % num_kv_heads != 0)
    return ret(err, Status::Invalid(strfmt("SDPA: numHeads (%d) must be positive and divisible by numKVHeads (%d)", num_heads, num_kv_heads)), nullptr);
  const bool bshd = axes_layout == B200_LAYOUT_BSHD;
  // Fused path: no mask tensor (or one query position), head dim 64, 16-bit floats.  One kernel reads Q, K and V in the layout they come
  // in; neither the scores, nor a mask, nor repeated K/V heads, nor a transposed copy is ever written.
  {
    const int s_ax = bshd ? 1 : 2, h_ax = bshd ? 2 : 1;
    const bool shapes_ok = k->dims == v->dims && q->dims[0] == k->dims[0] && q->dims[3] == k->dims[3] &&
                           q->dims[h_ax] == num_heads && k->dims[h_ax] == num_kv_heads && q->dtype == k->dtype && q->dtype == v->dtype;
    if (!shapes_ok) return ret(err, Status::Invalid("SDPA: query / key / value shapes, dtypes or head counts do not agree"), nullptr);
    const bool fusable = q->dims[3] == 64 && (q->dtype == B200_BFLOAT16 || q->dtype == B200_FLOAT16) && q->dims[s_ax] > 0 && k->dims[s_ax] > 0;
    // One query position (a decoding step) takes a mask tensor too: any mask that broadcasts to [B, H, 1, Sk].
    static const bool decode_on = []() { const char* e = getenv("B200MLX_DECODE_ATTENTION"); return !(e && e[0] == '0'); }();
    bool mask_ok = !m;
    if (m && decode_on && fusable && q->dims[s_ax] == 1 && !causal && scale > 0 && scale < 1e30 && (m->dtype == B200_BOOL || m->dtype == q->dtype) && m->rank() <= 4) {
      const int64_t full[4] = {q->dims[0], bshd && m->rank() == 4 ? 1 : (int64_t)num_heads, bshd && m->rank() == 4 ? (int64_t)num_heads : 1, k->dims[s_ax]};
      mask_ok = true;
      for (int i = 0; i < m->rank(); ++i) {
        const int64_t want = full[4 - m->rank() + i];
        if (m->dims[i] != 1 && m->dims[i] != want) mask_ok = false;
      }
    }
    if (mask_ok && fusable) {
      Graph& gr = reinterpret_cast<Ctx*>(ctx)->graph;
      Node* o = m ? gr.Add(Op::Attention, q->dtype, q->dims, {q, k, v, m}) : gr.Add(Op::Attention, q->dtype, q->dims, {q, k, v});
      o->ia = {num_heads, num_kv_heads, bshd ? 1 : 0, causal ? 1 : 0};
      o->fa = {scale};
      return ret(err, Status::OK(), o);
    }
  }
  // Work in BHSD like the reference (function.go:2697-2726).
  const int perm[4] = {0, 2, 1, 3};
  B200Value Q = query, K = key, V = value, M = mask;
  if (bshd) {
    Q = b200_transpose(ctx, Q, perm, 4, err); if (!Q) return nullptr;
    K = b200_transpose(ctx, K, perm, 4, err); if (!K) return nullptr;
    V = b200_transpose(ctx, V, perm, 4, err); if (!V) return nullptr;
    if (m && m->rank() == 4) { M = b200_transpose(ctx, M, perm, 4, err); if (!M) return nullptr; }
  }
  Node* qn = reinterpret_cast<Node*>(Q);
  Node* kn = reinterpret_cast<Node*>(K);
  if (qn->dims[1] != num_heads || kn->dims[1] != num_kv_heads)
    return ret(err, Status::Invalid("SDPA: head counts do not match the tensors"), nullptr);
  // GQA: query head h reads KV head h / repeats (each KV head repeated `repeats`
  // times consecutively, ref function.go:2910-2955).  Q is regrouped to
  // [B, Hkv, repeats*Sq, D] so K and V are used as they are, never copied.
  const int64_t B = qn->dims[0], H = num_heads, Hkv = num_kv_heads, Sq = qn->dims[2], D = qn->dims[3], Sk = kn->dims[2];
  const int64_t rep = H / Hkv;
  B200Value Qg = Q;
  if (rep > 1) {
    const int64_t g4[4] = {B, Hkv, rep * Sq, D};
    Qg = b200_reshape(ctx, Q, g4, 4, err);
    if (!Qg) return nullptr;
  }
  const int c3 = 3, bt[2] = {0, 1};
  B200Value scores = b200_dot_general(ctx, Qg, &c3, 1, bt, 2, K, &c3, 1, bt, 2, err);  // [B, Hkv, rep*Sq, Sk]
  if (!scores) return nullptr;
  const int64_t s4[4] = {B, H, Sq, Sk};
  if (rep > 1) { scores = b200_reshape(ctx, scores, s4, 4, err); if (!scores) return nullptr; }
  B200Value probs = b200_softmax_masked(ctx, scores, scale, causal, M, err);
  if (!probs) return nullptr;
  if (rep > 1) {
    const int64_t p4[4] = {B, Hkv, rep * Sq, Sk};
    probs = b200_reshape(ctx, probs, p4, 4, err);
    if (!probs) return nullptr;
  }
  const int c2 = 2;
  B200Value out = b200_dot_general(ctx, probs, &c3, 1, bt, 2, V, &c2, 1, bt, 2, err);  // [B, Hkv, rep*Sq, D]
  if (!out) return nullptr;
  const int64_t o4[4] = {B, H, Sq, reinterpret_cast<Node*>(V)->dims[3]};
  if (rep > 1) { out = b200_reshape(ctx, out, o4, 4, err); if (!out) return nullptr; }
  if (bshd) out = b200_transpose(ctx, out, perm, 4, err);
  return out;
}

B200Value b200_batch_norm_inference(B200Context ctx, B200Value input, B200Value mean, B200Value variance, B200Value gamma,
                                    B200Value beta, float epsilon, int feature_axis, B200Error* err) {
  clear_error(err);
  Node* n;
  Status s = check_node(ctx, input, "BatchNormForInference", &n);
  if (!s.ok()) return ret(err, s, nullptr);
  int a;
  s = normalize_axis("BatchNormForInference", feature_axis, n->rank(), &a);
  if (!s.ok()) return ret(err, s, nullptr);
  Graph& g = reinterpret_cast<Ctx*>(ctx)->graph;
  auto bc = [&](B200Value p) -> B200Value { return b200_broadcast_in_dim(ctx, p, n->dims.data(), n->rank(), &a, 1, err); };
  B200Value m = bc(mean); if (!m) return nullptr;
  B200Value var = bc(variance); if (!var) return nullptr;
  B200Value eps = reinterpret_cast<B200Value>(make_scalar_const(g, n->dtype, epsilon));
  B200Value d = b200_sub(ctx, input, m, err); if (!d) return nullptr;
  B200Value ve = b200_add(ctx, var, eps, err); if (!ve) return nullptr;
  B200Value r = b200_rsqrt(ctx, ve, err); if (!r) return nullptr;
  B200Value y = b200_mul(ctx, d, r, err); if (!y) return nullptr;
  if (gamma) { B200Value gg = bc(gamma); if (!gg) return nullptr; y = b200_mul(ctx, y, gg, err); if (!y) return nullptr; }
  if (beta) { B200Value bb = bc(beta); if (!bb) return nullptr; y = b200_add(ctx, y, bb, err); if (!y) return nullptr; }
  return y;
}

// ---- training-side ops ------------------------------------------------------------------------------------
// BatchNormForTraining (ref mpsgraph function.go:1263-1375): batch statistics over every axis but the feature axis,
// biased variance of the centred value (two-pass), rsqrt(var + eps), scale, offset; mean and variance come back as
// [feature] vectors.  Built from graph primitives like the reference's, so the lowering fuses the elementwise parts
// and the reductions read their operand chains in place.  scale / offset are laid along the FEATURE axis (the
// reference relies on trailing-axis broadcasting, which coincides when the feature axis is the last one).
bool b200_batch_norm_training(B200Context ctx, B200Value operand, B200Value scale, B200Value offset, float epsilon, int feature_axis,
                              B200Value* out_normalized, B200Value* out_mean, B200Value* out_variance, B200Error* err) {
  clear_error(err);
  Node *n, *sc, *of;
  Status s = check_node(ctx, operand, "BatchNormForTraining: operand", &n);
  if (s.ok()) s = check_node(ctx, scale, "BatchNormForTraining: scale", &sc);
  if (s.ok()) s = check_node(ctx, offset, "BatchNormForTraining: offset", &of);
  int a = 0;
  if (s.ok()) s = normalize_axis("BatchNormForTraining", feature_axis, n->rank(), &a);
  if (s.ok() && !dtype_is_float(n->dtype)) s = Status::Invalid("BatchNormForTraining: needs a float operand");
  if (s.ok() && (sc->num_elements() != n->dims[a] || of->num_elements() != n->dims[a]))
    s = Status::Invalid(strfmt("BatchNormForTraining: scale and offset must hold %lld elements (the feature axis)", (long long)n->dims[a]));
  if (!s.ok()) { set_error(err, s); return false; }
  if (!out_normalized || !out_mean || !out_variance) { set_error(err, Status::Invalid("BatchNormForTraining: null output pointer")); return false; }
  Graph& g = reinterpret_cast<Ctx*>(ctx)->graph;
  std::vector<int> batch_axes;
  int64_t count = 1;
  for (int i = 0; i < n->rank(); ++i)
    if (i != a) { batch_axes.push_back(i); count *= n->dims[i]; }
  const int64_t fdim[1] = {n->dims[a]};
  auto over_batch = [&](B200Value v) -> B200Value {   // sum over the batch axes -> [feature]
    if (batch_axes.empty()) return b200_reshape(ctx, v, fdim, 1, err);
    return b200_reduce(ctx, v, B200_REDUCE_SUM, batch_axes.data(), (int)batch_axes.size(), err);
  };
  auto along_feature = [&](B200Value v) -> B200Value {   // [feature] -> operand shape
    B200Value flat = b200_reshape(ctx, v, fdim, 1, err);
    if (!flat) return nullptr;
    return b200_broadcast_in_dim(ctx, flat, n->dims.data(), n->rank(), &a, 1, err);
  };
  B200Value cnt = reinterpret_cast<B200Value>(make_scalar_const(g, n->dtype, (double)count));
  B200Value eps = reinterpret_cast<B200Value>(make_scalar_const(g, n->dtype, (double)epsilon));
  B200Value sum = over_batch(operand); if (!sum) return false;
  B200Value mean = b200_div(ctx, sum, cnt, err); if (!mean) return false;
  B200Value mean_b = along_feature(mean); if (!mean_b) return false;
  B200Value diff = b200_sub(ctx, operand, mean_b, err); if (!diff) return false;
  B200Value sq = b200_mul(ctx, diff, diff, err); if (!sq) return false;
  B200Value vsum = over_batch(sq); if (!vsum) return false;
  B200Value var = b200_div(ctx, vsum, cnt, err); if (!var) return false;
  B200Value ve = b200_add(ctx, var, eps, err); if (!ve) return false;
  B200Value inv = b200_rsqrt(ctx, ve, err); if (!inv) return false;
  B200Value inv_b = along_feature(inv); if (!inv_b) return false;
  B200Value y = b200_mul(ctx, diff, inv_b, err); if (!y) return false;
  B200Value sc_b = along_feature(scale); if (!sc_b) return false;
  y = b200_mul(ctx, y, sc_b, err); if (!y) return false;
  B200Value of_b = along_feature(offset); if (!of_b) return false;
  y = b200_add(ctx, y, of_b, err); if (!y) return false;
  *out_normalized = y;
  *out_mean = mean;
  *out_variance = var;
  return true;
}

// BatchNormGradient (ref mpsgraph function.go:1377-1527):
//   xhat = (x - mean) * rsqrt(var + eps);  gradOffset = sum(dy);  gradScale = sum(dy * xhat);
//   gradOperand = (1 / N) * scale * rsqrt(var + eps) * (N * dy - gradOffset - xhat * gradScale)       sums over the batch axes
bool b200_batch_norm_gradient(B200Context ctx, B200Value operand, B200Value scale, B200Value mean, B200Value variance, B200Value grad_output,
                              float epsilon, int feature_axis, B200Value* out_grad_operand, B200Value* out_grad_scale,
                              B200Value* out_grad_offset, B200Error* err) {
  clear_error(err);
  Node *n, *sc, *mn, *vr, *dy;
  Status s = check_node(ctx, operand, "BatchNormGradient: operand", &n);
  if (s.ok()) s = check_node(ctx, scale, "BatchNormGradient: scale", &sc);
  if (s.ok()) s = check_node(ctx, mean, "BatchNormGradient: mean", &mn);
  if (s.ok()) s = check_node(ctx, variance, "BatchNormGradient: variance", &vr);
  if (s.ok()) s = check_node(ctx, grad_output, "BatchNormGradient: gradOutput", &dy);
  int a = 0;
  if (s.ok()) s = normalize_axis("BatchNormGradient", feature_axis, n->rank(), &a);
  if (s.ok() && !dtype_is_float(n->dtype)) s = Status::Invalid("BatchNormGradient: needs a float operand");
  if (s.ok() && dy->dims != n->dims) s = Status::Invalid("BatchNormGradient: gradOutput must have the operand's shape");
  if (s.ok())
    for (Node* p : {sc, mn, vr})
      if (p->num_elements() != n->dims[a]) s = Status::Invalid(strfmt("BatchNormGradient: scale, mean and variance must hold %lld elements", (long long)n->dims[a]));
  if (!s.ok()) { set_error(err, s); return false; }
  if (!out_grad_operand || !out_grad_scale || !out_grad_offset) { set_error(err, Status::Invalid("BatchNormGradient: null output pointer")); return false; }
  Graph& g = reinterpret_cast<Ctx*>(ctx)->graph;
  std::vector<int> batch_axes;
  int64_t count = 1;
  for (int i = 0; i < n->rank(); ++i)
    if (i != a) { batch_axes.push_back(i); count *= n->dims[i]; }
  const int64_t fdim[1] = {n->dims[a]};
  auto over_batch = [&](B200Value v) -> B200Value {
    if (batch_axes.empty()) return b200_reshape(ctx, v, fdim, 1, err);
    return b200_reduce(ctx, v, B200_REDUCE_SUM, batch_axes.data(), (int)batch_axes.size(), err);
  };
  auto along_feature = [&](B200Value v) -> B200Value {
    B200Value flat = b200_reshape(ctx, v, fdim, 1, err);
    if (!flat) return nullptr;
    return b200_broadcast_in_dim(ctx, flat, n->dims.data(), n->rank(), &a, 1, err);
  };
  B200Value eps = reinterpret_cast<B200Value>(make_scalar_const(g, n->dtype, (double)epsilon));
  B200Value n_c = reinterpret_cast<B200Value>(make_scalar_const(g, n->dtype, (double)count));
  B200Value inv_n = reinterpret_cast<B200Value>(make_scalar_const(g, n->dtype, 1.0 / (double)count));
  B200Value ve = b200_add(ctx, variance, eps, err); if (!ve) return false;
  B200Value inv = b200_rsqrt(ctx, ve, err); if (!inv) return false;
  B200Value inv_b = along_feature(inv); if (!inv_b) return false;
  B200Value mean_b = along_feature(mean); if (!mean_b) return false;
  B200Value centered = b200_sub(ctx, operand, mean_b, err); if (!centered) return false;
  B200Value xhat = b200_mul(ctx, centered, inv_b, err); if (!xhat) return false;
  B200Value g_off = over_batch(grad_output); if (!g_off) return false;
  B200Value dyx = b200_mul(ctx, grad_output, xhat, err); if (!dyx) return false;
  B200Value g_sc = over_batch(dyx); if (!g_sc) return false;
  B200Value t1 = b200_mul(ctx, n_c, grad_output, err); if (!t1) return false;
  B200Value g_off_b = along_feature(g_off); if (!g_off_b) return false;
  t1 = b200_sub(ctx, t1, g_off_b, err); if (!t1) return false;
  B200Value g_sc_b = along_feature(g_sc); if (!g_sc_b) return false;
  B200Value t3 = b200_mul(ctx, xhat, g_sc_b, err); if (!t3) return false;
  t1 = b200_sub(ctx, t1, t3, err); if (!t1) return false;
  B200Value go = b200_mul(ctx, inv_n, t1, err); if (!go) return false;
  B200Value sc_b = along_feature(scale); if (!sc_b) return false;
  go = b200_mul(ctx, sc_b, go, err); if (!go) return false;
  go = b200_mul(ctx, inv_b, go, err); if (!go) return false;
  *out_grad_operand = go;
  *out_grad_scale = g_sc;
  *out_grad_offset = g_off;
  return true;
}

// ScatterSum / ScatterMax / ScatterMin (ref mpsgraph gather.go:441-641): XLA scatter with a combiner.  The result is the
// operand with every element of `updates` combined into the position its scatter indices name:
//   update index u = (scatter coordinates s, window coordinates w);  index vector i = indices[s along index_vector_axis];
//   operand position: axis scatter_axes_to_operand_axes[k] starts at i[k]; window axis j of the update walks the j-th operand
//   axis that is not an inserted window axis.  An element whose position falls outside the operand is dropped.
B200Value b200_scatter(B200Context ctx, int mode, B200Value operand, B200Value scatter_indices, B200Value updates, int index_vector_axis,
                       const int* update_window_axes, int num_update_window_axes, const int* inserted_window_axes,
                       int num_inserted_window_axes, const int* scatter_axes_to_operand_axes, int num_scatter_axes,
                       bool indices_are_sorted, bool unique_indices, B200Error* err) {
  (void)indices_are_sorted;
  clear_error(err);
  const char* what = mode == 0 ? "ScatterSum" : mode == 1 ? "ScatterMax" : "ScatterMin";
  if (mode < 0 || mode > 2) return ret(err, Status::Invalid("Scatter: mode must be 0 (sum), 1 (max) or 2 (min)"), nullptr);
  Node *op, *idx, *upd;
  Status s = check_node(ctx, operand, what, &op);
  if (s.ok()) s = check_node(ctx, scatter_indices, what, &idx);
  if (s.ok()) s = check_node(ctx, updates, what, &upd);
  if (!s.ok()) return ret(err, s, nullptr);
  if (!dtype_is_int(idx->dtype)) return ret(err, Status::Invalid(std::string(what) + ": scatter indices must be integers"), nullptr);
  if (upd->dtype != op->dtype) return ret(err, Status::Invalid(std::string(what) + ": updates must have the operand's dtype"), nullptr);
  if (op->dtype == B200_BOOL) return ret(err, Status::Invalid(std::string(what) + ": Bool operand"), nullptr);
  const int orank = op->rank(), irank = idx->rank(), urank = upd->rank();
  if (orank > 8 || urank > 8 || irank > 8) return ret(err, Status::Unsupported(std::string(what) + ": more than 8 dims"), nullptr);
  if (index_vector_axis < 0 || index_vector_axis > irank) return ret(err, Status::Invalid(std::string(what) + ": indexVectorAxis out of range"), nullptr);
  const int64_t ncomp = index_vector_axis == irank ? 1 : idx->dims[index_vector_axis];
  if (ncomp != num_scatter_axes) return ret(err, Status::Invalid(std::string(what) + ": scatterAxesToOperandAxes length must equal the index vector size"), nullptr);
  std::set<int> inserted, window_upd, mapped;
  for (int i = 0; i < num_inserted_window_axes; ++i)
    if (inserted_window_axes[i] < 0 || inserted_window_axes[i] >= orank || !inserted.insert(inserted_window_axes[i]).second)
      return ret(err, Status::Invalid(std::string(what) + ": bad insertedWindowAxes"), nullptr);
  for (int i = 0; i < num_update_window_axes; ++i) {
    if (update_window_axes[i] < 0 || update_window_axes[i] >= urank || !window_upd.insert(update_window_axes[i]).second)
      return ret(err, Status::Invalid(std::string(what) + ": bad updateWindowAxes"), nullptr);
    if (i > 0 && update_window_axes[i] <= update_window_axes[i - 1]) return ret(err, Status::Invalid(std::string(what) + ": updateWindowAxes must ascend"), nullptr);
  }
  for (int i = 0; i < num_scatter_axes; ++i)
    if (scatter_axes_to_operand_axes[i] < 0 || scatter_axes_to_operand_axes[i] >= orank || !mapped.insert(scatter_axes_to_operand_axes[i]).second)
      return ret(err, Status::Invalid(std::string(what) + ": bad scatterAxesToOperandAxes"), nullptr);
  if (num_update_window_axes != orank - num_inserted_window_axes)
    return ret(err, Status::Invalid(std::string(what) + ": updateWindowAxes must have one entry per operand axis that is not an inserted window axis"), nullptr);
  // window axis j of the update <-> j-th operand axis that is not inserted; its extent must fit the operand
  std::vector<int> window_operand_axis;
  for (int i = 0; i < orank; ++i)
    if (!inserted.count(i)) window_operand_axis.push_back(i);
  for (int j = 0; j < num_update_window_axes; ++j)
    if (upd->dims[update_window_axes[j]] > op->dims[window_operand_axis[j]])
      return ret(err, Status::Invalid(std::string(what) + ": an update window is larger than the operand"), nullptr);
  // the update's scatter dims are the indices' batch dims, in order
  std::vector<int64_t> batch_dims, scatter_dims;
  for (int i = 0; i < irank; ++i)
    if (i != index_vector_axis) batch_dims.push_back(idx->dims[i]);
  for (int i = 0; i < urank; ++i)
    if (!window_upd.count(i)) scatter_dims.push_back(upd->dims[i]);
  if (batch_dims != scatter_dims) return ret(err, Status::Invalid(std::string(what) + ": the updates' scatter dims must equal the indices' batch dims"), nullptr);
  Graph& g = reinterpret_cast<Ctx*>(ctx)->graph;
  Node* o = g.Add(Op::Scatter, op->dtype, op->dims, {op, idx, upd});
  // ia = [mode, index_vector_axis, unique, n_uw, uw..., n_iw, iw..., n_map, map...]
  o->ia = {mode, index_vector_axis, unique_indices ? 1 : 0, num_update_window_axes};
  for (int i = 0; i < num_update_window_axes; ++i) o->ia.push_back(update_window_axes[i]);
  o->ia.push_back(num_inserted_window_axes);
  for (int i = 0; i < num_inserted_window_axes; ++i) o->ia.push_back(inserted_window_axes[i]);
  o->ia.push_back(num_scatter_axes);
  for (int i = 0; i < num_scatter_axes; ++i) o->ia.push_back(scatter_axes_to_operand_axes[i]);
  return ret(err, Status::OK(), o);
}

// RNGBitGenerator (ref mpsgraph function.go:1627-1692): state is [3] Uint64; returns the advanced state (every word + 1,
// as the reference advances it) and values of the requested dtype and shape.  The reference takes its values from
// MPSGraph's own generator, which ignores the state; here they are a pure function of the state: Philox4x32-10 keyed by
// state[0], counter (state[1], state[2]) + block number, four 32-bit words per block.  Integer dtypes get the raw bits
// (64-bit types two words), float dtypes a uniform value in [0, 1) from the top bits.
bool b200_rng_bit_generator(B200Context ctx, B200Value state, int dtype, const int64_t* shape, int rank, B200Value* out_new_state,
                            B200Value* out_values, B200Error* err) {
  clear_error(err);
  Node* st;
  Status s = check_node(ctx, state, "RNGBitGenerator: state", &st);
  if (s.ok() && (st->dtype != B200_UINT64 || st->rank() != 1 || st->dims[0] != 3))
    s = Status::Invalid("RNGBitGenerator: expected state shape (Uint64)[3]");
  if (s.ok() && (!dtype_valid(dtype) || dtype == B200_BOOL)) s = Status::Invalid("RNGBitGenerator: unsupported dtype");
  if (s.ok()) s = check_shape("RNGBitGenerator", shape, rank);
  if (!s.ok()) { set_error(err, s); return false; }
  if (!out_new_state || !out_values) { set_error(err, Status::Invalid("RNGBitGenerator: null output pointer")); return false; }
  Graph& g = reinterpret_cast<Ctx*>(ctx)->graph;
  Node* v = g.Add(Op::RngBits, dtype, std::vector<int64_t>(shape, shape + rank), {st});
  const uint64_t one_bits = 1;
  Node* one = g.Add(Op::Constant, B200_UINT64, {}, {});
  one->data.resize(8);
  memcpy(one->data.data(), &one_bits, 8);
  const int64_t three[1] = {3};
  B200Value one_b = b200_broadcast_in_dim(ctx, reinterpret_cast<B200Value>(one), three, 1, nullptr, 0, err);
  if (!one_b) return false;
  B200Value ns = b200_add(ctx, state, one_b, err);
  if (!ns) return false;
  *out_new_state = ns;
  *out_values = reinterpret_cast<B200Value>(v);
  return true;
}

// ---- control flow over closures (ref mpsgraph function.go:354-652; the reference runs these on the host, one control-flow
// op per function, executable.go:219-480) -------------------------------------------------------------------------
// A closure is a sub-graph of the SAME graph: its parameters are ClosureParam nodes, its results ordinary values, and it
// captures outer values simply by using them.  Call inlines the callee; If computes both branches and selects (the
// branches are pure); While keeps cond and body as sub-graphs that the executor compiles into two sub-plans; Sort
// recognises a comparator that orders by its first operand and becomes ArgSort + one gather per input.
B200Value b200_closure_parameter(B200Context ctx, int dtype, const int64_t* shape, int rank, B200Error* err) {
  clear_error(err);
  if (!ctx) return ret(err, Status::Invalid("closure parameter: null context"), nullptr);
  if (!dtype_valid(dtype)) return ret(err, Status::Invalid("closure parameter: bad dtype"), nullptr);
  Status s = check_shape("closure parameter", shape, rank);
  if (!s.ok()) return ret(err, s, nullptr);
  Graph& g = reinterpret_cast<Ctx*>(ctx)->graph;
  return ret(err, Status::OK(), g.Add(Op::ClosureParam, dtype, std::vector<int64_t>(shape, shape + rank), {}));
}

static Status closure_nodes(B200Context ctx, const char* what, const B200Value* vals, int n, std::vector<Node*>* out) {
  for (int i = 0; i < n; ++i) {
    Node* x;
    B200_TRY(check_node(ctx, vals[i], what, &x));
    out->push_back(x);
  }
  return Status::OK();
}

bool b200_call(B200Context ctx, const B200Value* params, int num_params, const B200Value* outputs, int num_outputs,
               const B200Value* inputs, B200Value* results, B200Error* err) {
  clear_error(err);
  std::vector<Node*> ps, outs, ins;
  Status s = closure_nodes(ctx, "Call: parameter", params, num_params, &ps);
  if (s.ok()) s = closure_nodes(ctx, "Call: output", outputs, num_outputs, &outs);
  if (s.ok()) s = closure_nodes(ctx, "Call: input", inputs, num_params, &ins);
  for (int i = 0; s.ok() && i < num_params; ++i) {
    if (ps[i]->op != Op::ClosureParam) s = Status::Invalid("Call: parameter is not a function parameter");
    else if (ps[i]->dtype != ins[i]->dtype || ps[i]->dims != ins[i]->dims)
      s = Status::Invalid(strfmt("Call: parameter %d shape mismatch", i));
  }
  if (s.ok() && (num_outputs < 1 || !results)) s = Status::Invalid("Call: the function returns nothing");
  if (!s.ok()) { set_error(err, s); return false; }
  Graph& g = reinterpret_cast<Ctx*>(ctx)->graph;
  std::vector<Node*> cloned;
  s = CloneClosure(g, ps, ins, outs, &cloned, nullptr, nullptr);
  if (!s.ok()) { set_error(err, s); return false; }
  for (int i = 0; i < num_outputs; ++i) results[i] = reinterpret_cast<B200Value>(cloned[i]);
  return true;
}

bool b200_if(B200Context ctx, B200Value pred, const B200Value* true_outputs, const B200Value* false_outputs, int num_outputs,
             B200Value* results, B200Error* err) {
  clear_error(err);
  Node* p;
  std::vector<Node*> t, f;
  Status s = check_node(ctx, pred, "If: pred", &p);
  if (s.ok() && (p->dtype != B200_BOOL || p->num_elements() != 1 || p->rank() != 0)) s = Status::Invalid("If: pred must be scalar bool");
  if (s.ok()) s = closure_nodes(ctx, "If: trueBranch output", true_outputs, num_outputs, &t);
  if (s.ok()) s = closure_nodes(ctx, "If: falseBranch output", false_outputs, num_outputs, &f);
  for (int i = 0; s.ok() && i < num_outputs; ++i)
    if (t[i]->dtype != f[i]->dtype || t[i]->dims != f[i]->dims) s = Status::Invalid(strfmt("If: output %d shapes must match", i));
  if (s.ok() && (num_outputs < 1 || !results)) s = Status::Invalid("If: the branches return nothing");
  if (!s.ok()) { set_error(err, s); return false; }
  // Light branches (elementwise work on small values) are both evaluated and the outputs selected: no hand-off, and the
  // select fuses into whatever consumes it.  A branch that holds a contraction, a reduction, a row kernel, a gather or
  // a loop, or that produces a lot of data, is worth skipping: then each branch becomes a sub-graph and one of the two
  // sub-plans runs (on the host's say-so on a plan's first runs, as a conditional graph node when the plan is replayed).
  {
    Ctx* c = reinterpret_cast<Ctx*>(ctx);
    Graph& g = c->graph;
    std::unordered_set<Node*> seen;
    int64_t weight = 0;
    bool heavy = false;
    std::function<void(Node*)> walk = [&](Node* n) {
      if (!seen.insert(n).second) return;
      // what was built before the predicate exists whether or not a branch runs (the branches are built after it)
      if (n->id <= p->id || n->op == Op::Parameter || n->op == Op::ClosureParam || n->op == Op::Constant) return;
      switch (n->op) {
        case Op::DotGeneral: case Op::Reduce: case Op::ArgMinMax: case Op::Gather: case Op::Scatter: case Op::Softmax: case Op::SoftmaxMasked:
        case Op::LayerNorm: case Op::RmsNorm: case Op::Attention: case Op::While: case Op::WhileResult: case Op::ArgSort: case Op::RngBits:
        case Op::If: case Op::IfResult:
          heavy = true;
          break;
        default: break;
      }
      weight += n->num_elements();
      if (seen.size() > 4096) { heavy = true; return; }
      for (Node* i : n->in) walk(i);
    };
    for (Node* o : t) walk(o);
    for (Node* o : f) walk(o);
    static const int64_t kSelectLimit = []() { const char* v = getenv("B200MLX_IF_SELECT_ELEMENTS"); return v ? atoll(v) : (int64_t)(1 << 20); }();
    if (heavy || weight > kSelectLimit) {
      auto extract = [&](const std::vector<Node*>& outs, std::vector<Node*>* caps) -> int {
        std::unique_ptr<SubGraph> sg(new SubGraph());
        sg->graph.device = g.device;
        std::vector<Node*> cap_params;
        s = CloneClosure(sg->graph, {}, {}, outs, &sg->targets, caps, &cap_params);
        if (!s.ok()) return -1;
        sg->feeds = cap_params;
        c->subgraphs.push_back(std::move(sg));
        return (int)c->subgraphs.size() - 1;
      };
      std::vector<Node*> t_caps, f_caps;
      const int t_sg = extract(t, &t_caps);
      const int f_sg = t_sg >= 0 ? extract(f, &f_caps) : -1;
      if (t_sg < 0 || f_sg < 0) { set_error(err, s); return false; }
      std::vector<Node*> operands = {p};
      operands.insert(operands.end(), t_caps.begin(), t_caps.end());
      operands.insert(operands.end(), f_caps.begin(), f_caps.end());
      Node* branch = g.Add(Op::If, B200_BOOL, {}, operands);
      // ia = [n_outputs, true sub-graph, false sub-graph, n true captures, n false captures]
      branch->ia = {num_outputs, t_sg, f_sg, (int64_t)t_caps.size(), (int64_t)f_caps.size()};
      for (int i = 0; i < num_outputs; ++i) {
        Node* r = g.Add(Op::IfResult, t[i]->dtype, t[i]->dims, {branch});
        r->ia = {i};
        results[i] = reinterpret_cast<B200Value>(r);
      }
      return true;
    }
  }
  for (int i = 0; i < num_outputs; ++i) {
    B200Value cond = b200_broadcast_in_dim(ctx, pred, t[i]->dims.data(), t[i]->rank(), nullptr, 0, err);
    if (!cond) return false;
    results[i] = b200_where(ctx, cond, true_outputs[i], false_outputs[i], err);
    if (!results[i]) return false;
  }
  return true;
}

bool b200_while(B200Context ctx, const B200Value* cond_params, B200Value cond_output, const B200Value* body_params,
                const B200Value* body_outputs, int num_state, const B200Value* initial_state, B200Value* results, B200Error* err) {
  clear_error(err);
  std::vector<Node*> cp, bp, bo, init;
  Node* co = nullptr;
  Status s = num_state >= 1 ? Status::OK() : Status::Invalid("While: requires at least one initial state value");
  if (s.ok()) s = closure_nodes(ctx, "While: cond parameter", cond_params, num_state, &cp);
  if (s.ok()) s = closure_nodes(ctx, "While: body parameter", body_params, num_state, &bp);
  if (s.ok()) s = closure_nodes(ctx, "While: body output", body_outputs, num_state, &bo);
  if (s.ok()) s = closure_nodes(ctx, "While: initial state", initial_state, num_state, &init);
  if (s.ok()) s = check_node(ctx, cond_output, "While: cond output", &co);
  if (s.ok() && (co->dtype != B200_BOOL || co->rank() != 0)) s = Status::Invalid("While: cond must return scalar bool");
  for (int i = 0; s.ok() && i < num_state; ++i) {
    auto same = [&](Node* a) { return a->dtype == init[i]->dtype && a->dims == init[i]->dims; };
    if (cp[i]->op != Op::ClosureParam || bp[i]->op != Op::ClosureParam) s = Status::Invalid("While: cond / body parameter is not a closure parameter");
    else if (!same(cp[i])) s = Status::Invalid(strfmt("While: cond parameter %d doesn't match state shape", i));
    else if (!same(bp[i])) s = Status::Invalid(strfmt("While: body parameter %d doesn't match state shape", i));
    else if (!same(bo[i])) s = Status::Invalid(strfmt("While: body output %d must match state shape", i));
  }
  if (s.ok() && !results) s = Status::Invalid("While: null result pointer");
  if (!s.ok()) { set_error(err, s); return false; }
  Ctx* c = reinterpret_cast<Ctx*>(ctx);
  Graph& g = c->graph;
  // cond and body each become a graph of their own (compiled into a sub-plan when the parent is compiled): parameters
  // first, then the outer values they capture, which the While node lists after its initial state so that they are
  // live and materialised in the parent
  auto extract = [&](const std::vector<Node*>& params, const std::vector<Node*>& outs, std::vector<Node*>* caps) -> int {
    std::unique_ptr<SubGraph> sg(new SubGraph());
    sg->graph.device = g.device;
    std::vector<Node*> feeds, cap_params;
    for (Node* p : params) feeds.push_back(sg->graph.Add(Op::Parameter, p->dtype, p->dims, {}));
    s = CloneClosure(sg->graph, params, feeds, outs, &sg->targets, caps, &cap_params);
    if (!s.ok()) return -1;
    feeds.insert(feeds.end(), cap_params.begin(), cap_params.end());
    sg->feeds = feeds;
    c->subgraphs.push_back(std::move(sg));
    return (int)c->subgraphs.size() - 1;
  };
  std::vector<Node*> cond_caps, body_caps;
  const int cond_sg = extract(cp, {co}, &cond_caps);
  const int body_sg = cond_sg >= 0 ? extract(bp, bo, &body_caps) : -1;
  if (cond_sg < 0 || body_sg < 0) { set_error(err, s); return false; }
  std::vector<Node*> operands = init;
  operands.insert(operands.end(), cond_caps.begin(), cond_caps.end());
  operands.insert(operands.end(), body_caps.begin(), body_caps.end());
  Node* w = g.Add(Op::While, B200_BOOL, {}, operands);
  // ia = [n_state, cond subgraph, body subgraph, n_cond_captures, n_body_captures]
  w->ia = {num_state, cond_sg, body_sg, (int64_t)cond_caps.size(), (int64_t)body_caps.size()};
  for (int i = 0; i < num_state; ++i) {
    Node* r = g.Add(Op::WhileResult, init[i]->dtype, init[i]->dims, {w});
    r->ia = {i};
    results[i] = reinterpret_cast<B200Value>(r);
  }
  return true;
}

// The comparator must order by its FIRST operand alone: output = LessThan / LessOrEqual (ascending) or GreaterThan /
// GreaterOrEqual (descending) of parameters 0 and 1, in either order, which is what GoMLX's Sort helper builds.
bool b200_sort(B200Context ctx, const B200Value* comparator_params, int num_params, B200Value comparator_output, int axis, bool is_stable,
               const B200Value* inputs, int num_inputs, B200Value* results, B200Error* err) {
  (void)is_stable;   // the sort is always stable
  clear_error(err);
  std::vector<Node*> cp, ins;
  Node* co = nullptr;
  Status s = num_inputs >= 1 ? Status::OK() : Status::Invalid("Sort: requires at least one input tensor");
  if (s.ok() && num_params != 2 * num_inputs) s = Status::Invalid(strfmt("Sort: comparator must have %d parameters, got %d", 2 * num_inputs, num_params));
  if (s.ok()) s = closure_nodes(ctx, "Sort: comparator parameter", comparator_params, num_params, &cp);
  if (s.ok()) s = closure_nodes(ctx, "Sort: input", inputs, num_inputs, &ins);
  if (s.ok()) s = check_node(ctx, comparator_output, "Sort: comparator output", &co);
  if (s.ok() && (co->dtype != B200_BOOL || co->rank() != 0)) s = Status::Invalid("Sort: comparator must return scalar bool");
  for (int i = 0; s.ok() && i < num_inputs; ++i) {
    if (ins[i]->dims != ins[0]->dims) s = Status::Invalid("Sort: all inputs must have same dimensions");
    for (int j = 0; s.ok() && j < 2; ++j) {
      Node* q = cp[2 * i + j];
      if (q->op != Op::ClosureParam || q->rank() != 0) s = Status::Invalid(strfmt("Sort: comparator parameter %d must be scalar", 2 * i + j));
      else if (q->dtype != ins[i]->dtype) s = Status::Invalid(strfmt("Sort: comparator parameter %d dtype must match input dtype", 2 * i + j));
    }
  }
  int a = 0;
  if (s.ok()) s = normalize_axis("Sort", axis, ins[0]->rank(), &a);
  bool descending = false;
  if (s.ok()) {
    Node* c = co;
    while (c->op == Op::Identity || c->op == Op::Reshape) c = c->in[0];
    const bool lt = c->op == Op::LessThan || c->op == Op::LessOrEqual, gt = c->op == Op::GreaterThan || c->op == Op::GreaterOrEqual;
    if ((lt || gt) && c->in[0] == cp[0] && c->in[1] == cp[1]) descending = gt;
    else if ((lt || gt) && c->in[0] == cp[1] && c->in[1] == cp[0]) descending = lt;
    else s = Status::Unsupported("Sort: only comparators that order by the first input (LessThan / GreaterThan of its two parameters) are supported");
  }
  if (s.ok() && dtype_size(ins[0]->dtype) == 8) s = Status::Unsupported("Sort: 64-bit keys are not supported");
  if (s.ok() && !results) s = Status::Invalid("Sort: null result pointer");
  if (!s.ok()) { set_error(err, s); return false; }
  Graph& g = reinterpret_cast<Ctx*>(ctx)->graph;
  Node* perm = g.Add(Op::ArgSort, B200_INT32, ins[0]->dims, {ins[0]});
  perm->ia = {a, descending ? 1 : 0};
  for (int i = 0; i < num_inputs; ++i) {
    results[i] = b200_gather_along_axis(ctx, inputs[i], reinterpret_cast<B200Value>(perm), a, err);
    if (!results[i]) return false;
  }
  return true;
}

}  // extern "C"

namespace b200 {

Status CloneClosure(Graph& dst, const std::vector<Node*>& params, const std::vector<Node*>& subst, const std::vector<Node*>& outputs,
                    std::vector<Node*>* cloned_outputs, std::vector<Node*>* captures, std::vector<Node*>* capture_params) {
  if (outputs.empty()) return Status::Invalid("closure: no outputs");
  Graph* src = outputs[0]->graph;
  const bool same_graph = src == &dst;
  std::unordered_map<Node*, Node*> map;
  for (size_t i = 0; i < params.size(); ++i) map[params[i]] = subst[i];
  // does a node depend on a parameter of THIS closure?  (memoised; another closure's parameter counts as outside)
  std::unordered_map<Node*, bool> dep;
  std::function<bool(Node*)> depends = [&](Node* n) -> bool {
    auto it = dep.find(n);
    if (it != dep.end()) return it->second;
    bool d = map.count(n) && n->op == Op::ClosureParam;
    for (Node* i : n->in) d = depends(i) || d;
    return dep[n] = d;
  };
  // computed from constants and iotas alone (cheap to copy into another graph)
  std::function<bool(Node*)> constant_only = [&](Node* n) -> bool {
    if (n->op == Op::Constant || n->op == Op::Iota) return true;
    if (n->op == Op::Parameter || n->op == Op::ClosureParam || n->in.empty()) return false;
    if (n->op == Op::While || n->op == Op::WhileResult || n->op == Op::If || n->op == Op::IfResult || n->num_elements() > 4096)
      return false;   // an outer loop's or branch's result is fed, not re-run
    for (Node* i : n->in)
      if (!constant_only(i)) return false;
    return true;
  };
  Status failed = Status::OK();
  std::function<Node*(Node*)> clone = [&](Node* n) -> Node* {
    auto it = map.find(n);
    if (it != map.end()) return it->second;
    // a While (and the picks of its results) is copied like any other node: its cond / body sub-graphs belong to the
    // context and are named by index, its operands (initial state and captured values) are cloned or captured in turn
    // (a parameter of an ENCLOSING closure is an outer value like any other: shared when inlining, fed when extracting)
    if (!depends(n)) {
      if (same_graph) return map[n] = n;
      if (!constant_only(n)) {   // an outer value: feed it
        Node* p = dst.Add(Op::Parameter, n->dtype, n->dims, {});
        if (captures) captures->push_back(n);
        if (capture_params) capture_params->push_back(p);
        return map[n] = p;
      }
    }
    std::vector<Node*> in;
    for (Node* i : n->in) in.push_back(clone(i));
    Node* c = dst.Add(n->op, n->dtype, n->dims, in);
    c->ia = n->ia;
    c->fa = n->fa;
    c->data = n->data;
    return map[n] = c;
  };
  for (Node* o : outputs) {
    Node* c = clone(o);
    if (!failed.ok()) return failed;
    cloned_outputs->push_back(c);
  }
  return Status::OK();
}

}  // namespace b200
