// Shared internal declarations of libb200mlx: dtypes, errors, the device
// runtime (stream + caching allocator), buffers, the graph IR and the kernel
// launchers.  Nothing here is part of the C ABI; see include/b200mlx.h for that.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <atomic>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/b200mlx.h"

#ifdef __CUDACC__
#define B200_HD __host__ __device__
#else
#define B200_HD
#endif

namespace b200 {

// ---------------------------------------------------------------- dtypes ---
B200_HD inline int dtype_size(int dt) {
  switch (dt) {
    case B200_BOOL: case B200_INT8: case B200_UINT8: return 1;
    case B200_INT16: case B200_UINT16: case B200_FLOAT16: case B200_BFLOAT16: return 2;
    case B200_INT32: case B200_UINT32: case B200_FLOAT32: return 4;
    case B200_INT64: case B200_UINT64: case B200_FLOAT64: return 8;
  }
  return 0;
}
B200_HD inline bool dtype_valid(int dt) { return dt >= 0 && dt <= 12; }
B200_HD inline bool dtype_is_float(int dt) {
  return dt == B200_FLOAT16 || dt == B200_BFLOAT16 || dt == B200_FLOAT32 || dt == B200_FLOAT64;
}
B200_HD inline bool dtype_is_int(int dt) { return dtype_valid(dt) && !dtype_is_float(dt) && dt != B200_BOOL; }
B200_HD inline bool dtype_is_unsigned(int dt) {
  return dt == B200_UINT8 || dt == B200_UINT16 || dt == B200_UINT32 || dt == B200_UINT64 || dt == B200_BOOL;
}
const char* dtype_name(int dt);

// ---------------------------------------------------------------- errors ---
struct Status {
  int code = 0;
  std::string msg;
  bool ok() const { return code == 0; }
  static Status OK() { return Status(); }
  static Status Invalid(const std::string& m) { return Status{B200_ERR_INVALID, m}; }
  static Status Cuda(const std::string& m) { return Status{B200_ERR_CUDA, m}; }
  static Status Unsupported(const std::string& m) { return Status{B200_ERR_UNSUPPORTED, m}; }
  static Status Oom(const std::string& m) { return Status{B200_ERR_OOM, m}; }
  static Status Timeout(const std::string& m) { return Status{B200_ERR_TIMEOUT, m}; }
};
std::string strfmt(const char* fmt, ...);
inline void clear_error(B200Error* e) {
  if (e) { e->code = 0; e->message = nullptr; }
}
inline void set_error(B200Error* e, const Status& s) {
  if (!e) return;
  e->code = s.code;
  e->message = s.ok() ? nullptr : strdup(s.msg.c_str());
}
#define B200_CUDA_TRY(expr)                                                                         \
  do {                                                                                              \
    cudaError_t _e = (expr);                                                                        \
    if (_e != cudaSuccess)                                                                          \
      return ::b200::Status::Cuda(::b200::strfmt("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), \
                                                 __FILE__, __LINE__));                              \
  } while (0)
#define B200_TRY(expr)          \
  do {                          \
    ::b200::Status _s = (expr); \
    if (!_s.ok()) return _s;    \
  } while (0)

// --------------------------------------------------------------- runtime ---
// One Device object per CUDA ordinal, created on first use and kept until
// process exit.  It owns the stream every launch of this library goes to and a
// stream-ordered caching allocator (blocks are reused only on that stream, so
// freeing needs no synchronisation).
class Device {
 public:
  static Status Get(int ordinal, Device** out);
  int ordinal() const { return ordinal_; }
  // The stream work is enqueued on: the device's one compute stream, except inside a StreamOverride of the calling
  // thread (used to record a launch plan into a CUDA graph on a private stream, so that work other threads enqueue on
  // the compute stream meanwhile is not swept into the recording).
  cudaStream_t stream() const;
  cudaStream_t compute_stream() const { return stream_; }
  Status CaptureStream(cudaStream_t* out);
  // A second private stream: the body of a While loop is recorded on it into the loop's conditional graph node while
  // the plan around the loop is being recorded on the capture stream (same holder of capture_mutex).
  // One such stream per nesting depth of loops (0 = outermost), at most kMaxLoopDepth.
  static constexpr int kMaxLoopDepth = 4;
  Status LoopStream(int depth, cudaStream_t* out);
  // Held from cudaStreamBeginCapture to cudaStreamEndCapture on the capture stream: the device has one such stream,
  // and two executables reaching their recording run at the same time would otherwise begin a capture on a stream
  // that is already capturing.
  std::mutex& capture_mutex() { return capture_mu_; }
  // Two extra streams for host<->device copies that overlap the compute stream (created on first use).
  Status CopyStreams(cudaStream_t* in, cudaStream_t* out);
  int sm_count() const { return sm_count_; }
  Status Alloc(int64_t nbytes, void** out);
  void Free(void* p);
  int64_t BytesReserved();
  void Trim();
  Status MakeCurrent();
  Status Synchronize();
  // Launch status: any launch helper calls this after a kernel launch.
  Status CheckLaunch(const char* what);
  // A word of device memory that kernels with bounded waits set when a wait
  // gives up.  Read back (and cleared) at synchronisation points, and only when
  // a kernel that can set it was launched since the last check.
  int* kernel_error_flag() {
    error_check_pending_ = true;
    return error_flag_;
  }
  Status CheckKernelErrors();
  // A small pinned staging area used by synchronous host<->device copies.
 private:
  Device() = default;
  int ordinal_ = 0;
  int sm_count_ = 148;
  cudaStream_t stream_ = nullptr;
  cudaStream_t copy_in_ = nullptr, copy_out_ = nullptr, capture_ = nullptr, loop_[kMaxLoopDepth] = {};
  int* error_flag_ = nullptr;
  std::atomic<bool> error_check_pending_{false};   // set by launching threads, read at synchronisation points
  std::mutex mu_, capture_mu_;
  std::multimap<int64_t, void*> free_blocks_;  // size -> ptr
  std::map<void*, int64_t> live_blocks_;       // ptr -> size
  int64_t reserved_ = 0;
};

// Code a device-resident While loop writes to the device's error word when it stops at its iteration limit (codes 1..8
// are the bounded waits of the tensor-core kernels).
constexpr int kErrWhileLimit = 100;

// While alive, Device::stream() of `dev` returns `s` on this thread only.
class StreamOverride {
 public:
  StreamOverride(const Device* dev, cudaStream_t s);
  ~StreamOverride();   // restores what was in force before (overrides nest)
  StreamOverride(const StreamOverride&) = delete;
  StreamOverride& operator=(const StreamOverride&) = delete;

 private:
  const Device* prev_dev_;
  cudaStream_t prev_stream_;
};

struct Buffer {
  int device = 0;
  int dtype = B200_FLOAT32;
  std::vector<int64_t> dims;
  void* ptr = nullptr;
  int64_t nbytes = 0;
  bool owned = true;
  bool ipc = false;   // mapped from another process: unmapped, not freed
  int64_t num_elements() const {
    int64_t n = 1;
    for (auto d : dims) n *= d;
    return n;
  }
};

// ------------------------------------------------------------------- IR ----
enum class Op : int {
  // leaves
  Parameter, Constant, Iota,
  // unary
  Abs, Neg, Sqrt, Rsqrt, Exp, Expm1, Log, Log1p, Sin, Cos, Tanh, Sigmoid, Erf, Floor, Ceil, Round, Sign,
  LogicalNot, BitwiseNot, IsFinite, IsNaN, Identity,
  GeluExact, GeluTanh, Relu, Silu,  // activations, produced by b200_gelu / b200_dense
  // binary
  Add, Sub, Mul, Div, Rem, Pow, Max, Min, Atan2, LogicalAnd, LogicalOr, LogicalXor, BitwiseAnd, BitwiseOr,
  BitwiseXor, ShiftLeft, ShiftRight, ShiftRightLogical,
  // compare
  Equal, NotEqual, LessThan, LessOrEqual, GreaterThan, GreaterOrEqual,
  // ternary
  Where, Clamp,
  // data movement
  Cast, Reshape, Transpose, BroadcastInDim, Slice, Concatenate, Reverse, Pad, DynamicSlice, DynamicUpdateSlice,
  // contraction / reduction / indexing
  DotGeneral, Reduce, ArgMinMax, Gather,
  // fused
  Softmax, SoftmaxMasked, LayerNorm, RmsNorm, Attention,
  // produced only by the compile-time rewrites: x * c + swap_halves(x) * s on the last axis (rotary embedding)
  Rope,
  // training side: XLA scatter with a combiner (sum / max / min), and random bits from a counter-based generator
  Scatter, RngBits,
  // control flow over closures (sub-graphs of the same graph whose inputs are ClosureParam nodes): While is the loop itself
  // (no value), WhileResult picks one of its final state values; ArgSort is the permutation a Sort applies to its inputs
  ClosureParam, While, WhileResult, ArgSort,
  // If with branches too heavy to evaluate both: runs one of two sub-plans; IfResult picks one of its outputs
  If, IfResult,
  kNumOps
};
const char* op_name(Op op);
bool op_is_unary(Op op);
bool op_is_binary(Op op);
bool op_is_compare(Op op);
// Ops the elementwise interpreter can evaluate inside a fused chain.
bool op_is_elementwise(Op op);

struct Graph;

struct Node {
  Graph* graph = nullptr;
  int id = 0;
  Op op = Op::Parameter;
  int dtype = B200_FLOAT32;
  std::vector<int64_t> dims;
  std::vector<Node*> in;
  // generic attributes; meaning depends on op (documented where each op is built)
  std::vector<int64_t> ia;            // integer attributes
  std::vector<double> fa;             // floating attributes
  std::vector<uint8_t> data;          // constant payload (host copy)
  int64_t num_elements() const {
    int64_t n = 1;
    for (auto d : dims) n *= d;
    return n;
  }
  int rank() const { return (int)dims.size(); }
};

struct Graph {
  int device = 0;
  std::vector<std::unique_ptr<Node>> nodes;
  Node* Add(Op op, int dtype, std::vector<int64_t> dims, std::vector<Node*> in) {
    auto n = std::make_unique<Node>();
    n->graph = this;
    n->id = (int)nodes.size();
    n->op = op;
    n->dtype = dtype;
    n->dims = std::move(dims);
    n->in = std::move(in);
    nodes.push_back(std::move(n));
    return nodes.back().get();
  }
};

// Compile-time rewrite: turns RMSNorm spelled in primitives (x * rsqrt(mean(x^2, last) + eps) [* gamma]) into one
// RmsNorm node.  Returns the number of patterns rewritten.  Defined in rewrite.cpp.
int RewriteRmsNorm(Graph& graph, const std::vector<Node*>& targets);   // also LayerNorm: the same chain around x - mean(x)
// Compile-time rewrite: Div(Exp(x - rowmax(x)), rowsum(Exp(x - rowmax(x)))) over the last axis becomes one Softmax node.
int RewriteSoftmax(Graph& graph, const std::vector<Node*>& targets);
// Compile-time rewrite: Add(DotGeneral(...), r) or Mul(DotGeneral(...), r) where the product has no other user becomes one
// DotGeneral node that combines with r in its epilogue (rounding the product first, so the value is the op-by-op one).  Returns the number of rewrites.
int RewriteGemmResidual(Graph& graph, const std::vector<Node*>& targets);
// Compile-time rewrite: Add(Mul(x, c), Mul(Concatenate(upper half of x, lower half of x), s)) on the last axis becomes one
// Rope node (inputs x, c, s): one pass over x instead of two slices, a concatenation and a three-op chain.
int RewriteRope(Graph& graph, const std::vector<Node*>& targets);

// Copies the sub-graph that computes `outputs` from the closure parameters `params` into graph `dst` (which may be the
// graph they live in): parameter i becomes subst[i]; a node that does not depend on any parameter is shared when dst
// is its own graph, else cloned if it is a constant / iota (or computed from those alone) and otherwise turned into a
// fresh Parameter of dst and appended to *captures (the value the caller must feed).  Defined in graph.cpp.
Status CloneClosure(Graph& dst, const std::vector<Node*>& params, const std::vector<Node*>& subst, const std::vector<Node*>& outputs,
                    std::vector<Node*>* cloned_outputs, std::vector<Node*>* captures, std::vector<Node*>* capture_params);

// What a B200Context handle points to: one graph under construction and its device.
// A closure extracted into a graph of its own (the cond or the body of a While): its feeds are the closure's parameters
// followed by the outer values it captures, in the order the While node lists them among its operands.
struct SubGraph {
  Graph graph;
  std::vector<Node*> feeds, targets;
};

struct Ctx {
  Graph graph;
  Device* dev = nullptr;
  std::vector<std::unique_ptr<SubGraph>> subgraphs;   // owned by the context; a While node names two of them by index
};

}  // namespace b200
