// The lowering pass: graph -> launch plan, and the executor that replays it.
//
// Counterpart in the reference: Builder.Compile / compileSimple (mpsgraph
// builder.go:72-109) hands the graph to MPSGraph's compiler, and
// Executable.Execute (executable.go:50-112) copies every input in, waits, and
// copies every output out.  Here compile() walks the graph once and emits a
// list of kernel launches with a static memory plan; execute() only binds
// pointers and enqueues.
//
// What the pass does:
//   * dead-code elimination from the targets;
//   * Reshape / Identity become views (no launch);
//   * chains of elementwise ops, broadcasts, transposes, slices, reversals,
//     iotas and scalar constants are fused into ONE interpreter program per
//     materialised result (kernels/ewise.cu);
//   * DotGeneral picks the operand-major form the GEMM reads in place, so no
//     transpose is materialised for the [B,M,K]x[B,K,N], [B,K,M]x[B,K,N],
//     QK^T and PV forms; bias and activation ride in the GEMM epilogue;
//   * Softmax / SoftmaxMasked / LayerNorm / RMSNorm / Reduce / ArgMinMax /
//     Gather go to their dedicated kernels;
//   * intermediates get offsets in one arena by a liveness scan (a value's
//     bytes are reused after its last reader), outputs are fresh allocations.
#include <algorithm>
#include <array>
#include <cmath>
#include <cstdlib>
#include <functional>
#include <sstream>
#include <unordered_map>

#include "common.h"
#include "kernels.h"

namespace b200 {

namespace k {
Status gemm_simt(Device* dev, const GemmParams& p);
}

namespace {

enum class SlotKind { Input, Const, Arena, Output, Scratch };

struct Slot {
  SlotKind kind = SlotKind::Arena;
  int index = 0;        // input / output ordinal, or constant ordinal
  int64_t nbytes = 0;
  int64_t offset = 0;   // arena offset (Arena / Scratch)
  int first_step = -1, last_step = -1;
};

struct Step {
  std::string desc;
  std::vector<int> reads, writes;
  int launches = 1;
  bool capturable = true;   // false when run() allocates or frees device memory (its pointers would be stale in a replay)
  bool wants_graph = false; // a step that is much cheaper inside a replayed graph (a While loop then runs on the device)
  std::function<Status(Device*, void* const*)> run;  // ptrs indexed by slot
};

// One instantiated CUDA graph of a whole launch plan, valid for one set of input / output addresses.
struct PlanGraph {
  std::vector<void*> key;
  cudaGraphExec_t exec = nullptr;
  uint64_t last_used = 0;
};

struct OutputDesc {
  int slot;
  int dtype;
  std::vector<int64_t> dims;
  int64_t nbytes;
};

struct Exec {
  Device* dev = nullptr;
  std::vector<Slot> slots;
  std::vector<Step> steps;
  std::vector<OutputDesc> inputs;   // slot = the input's slot
  std::vector<OutputDesc> outputs;
  std::vector<void*> const_ptrs;
  void* arena = nullptr;
  int64_t arena_bytes = 0;
  int num_launches = 0;
  std::mutex mu;
  // Launch-bound plans replay as one CUDA graph: the second time a plan runs on the same input and output addresses
  // (a serving loop that frees its outputs gets the same blocks back from the caching allocator) its steps are
  // captured from the stream instead of launched, and later calls with those addresses are one cudaGraphLaunch.
  // output j may take over the memory of donated input donate_alias[j] (-1: never): see EmitDynamicSlice
  std::vector<int> donate_alias;
  bool capturable = false;
  std::vector<PlanGraph> graphs;
  std::vector<void*> last_key;
  uint64_t tick = 0;
  // sub-plans of While loops (cond, body); run by the While step through RunSubPlan, never from outside
  std::vector<std::unique_ptr<Exec>> children;
  ~Exec() {
    for (auto& g : graphs)
      if (g.exec) cudaGraphExecDestroy(g.exec);
    if (dev) {
      for (void* p : const_ptrs) dev->Free(p);
      dev->Free(arena);
    }
  }
};

int64_t align_up(int64_t v, int64_t a) { return (v + a - 1) / a * a; }

std::vector<int64_t> dense_strides(const std::vector<int64_t>& dims) {
  std::vector<int64_t> s(dims.size());
  int64_t acc = 1;
  for (int i = (int)dims.size() - 1; i >= 0; --i) {
    s[i] = acc;
    acc *= dims[i];
  }
  return s;
}

// Per-dimension affine map from a node's index space into the index space of
// the fused kernel's output: node_idx[i] = a[i] * out_idx[m[i]] + b[i]
// (m[i] == -1: the coordinate is the constant b[i]).
struct IndexMap {
  std::vector<int> m;
  std::vector<int64_t> a, b;
  std::string key() const {
    std::string s;
    for (size_t i = 0; i < m.size(); ++i) s += std::to_string(m[i]) + ":" + std::to_string(a[i]) + ":" + std::to_string(b[i]) + ",";
    return s;
  }
  static IndexMap Identity(int rank) {
    IndexMap im;
    for (int i = 0; i < rank; ++i) { im.m.push_back(i); im.a.push_back(1); im.b.push_back(0); }
    return im;
  }
};

// Rewrites + plan + arena for one graph (the context's own, or a While's cond / body sub-graph of `owner`).
Status CompileGraph(Ctx* owner, Graph& graph, std::vector<Node*> feeds, std::vector<Node*> targets, std::unique_ptr<Exec>* out, int loop_depth = 0);

// Runs a sub-plan's steps on the device's stream with caller-provided input and output addresses.
Status RunSubPlan(Exec* ex, void* const* in_ptrs, void* const* out_ptrs) {
  std::vector<void*> ptrs(ex->slots.size(), nullptr);
  for (size_t i = 0; i < ex->inputs.size(); ++i) ptrs[ex->inputs[i].slot] = in_ptrs[i];
  for (size_t i = 0; i < ex->outputs.size(); ++i) ptrs[ex->outputs[i].slot] = out_ptrs[i];
  for (size_t s = 0; s < ex->slots.size(); ++s) {
    const Slot& sl = ex->slots[s];
    if (sl.kind == SlotKind::Arena) ptrs[s] = (char*)ex->arena + sl.offset;
    else if (sl.kind == SlotKind::Const) ptrs[s] = ex->const_ptrs[sl.index];
  }
  for (auto& st : ex->steps) {
    Status rs = st.run(ex->dev, ptrs.data());
    if (!rs.ok()) return Status{rs.code, st.desc + ": " + rs.msg};
  }
  return Status::OK();
}

constexpr int kWhileMaxIterations = 1000000;   // the reference's limit (ref mpsgraph executable.go:241)

// Sets the condition of a device-resident While loop for its next trip: the cond sub-plan's byte, unless the trip limit
// is reached (then the loop stops and the device's error word says why).  One thread.
__global__ void while_set_cond_kernel(cudaGraphConditionalHandle handle, const unsigned char* pred, int* trips, int limit, int* err_flag) {
  unsigned go = *pred != 0 ? 1u : 0u;
  const int t = *trips;
  if (go && t >= limit) {
    atomicCAS(err_flag, 0, kErrWhileLimit);
    go = 0;
  }
  *trips = t + 1;
  cudaGraphSetConditional(handle, go);
}

// Sets the conditions of the two conditional IF nodes of a branch: one runs when the predicate byte is set, the other
// when it is not.  One thread.
__global__ void if_set_cond_kernel(cudaGraphConditionalHandle on_true, cudaGraphConditionalHandle on_false, const unsigned char* pred) {
  const unsigned v = *pred != 0 ? 1u : 0u;
  cudaGraphSetConditional(on_true, v);
  cudaGraphSetConditional(on_false, 1u - v);
}

// Records a two-way branch into the CUDA graph that `dev->stream()` is being captured into: two conditional IF nodes, one
// per branch, whose body graphs are recorded on the loop stream of this nesting depth.
Status RecordIfNodes(Device* dev, int depth, const unsigned char* pred, const std::function<Status()>& run_true,
                     const std::function<Status()>& run_false) {
  cudaStream_t ps = dev->stream();
  cudaStream_t ls = nullptr;
  B200_TRY(dev->LoopStream(depth, &ls));
  cudaStreamCaptureStatus status;
  unsigned long long id = 0;
  cudaGraph_t parent = nullptr;
  const cudaGraphNode_t* deps = nullptr;
  size_t num_deps = 0;
  B200_CUDA_TRY(cudaStreamGetCaptureInfo_v2(ps, &status, &id, &parent, &deps, &num_deps));
  if (status != cudaStreamCaptureStatusActive || !parent) return Status::Invalid("If: the stream is not being recorded");
  cudaGraphConditionalHandle handles[2];
  for (int b = 0; b < 2; ++b) B200_CUDA_TRY(cudaGraphConditionalHandleCreate(&handles[b], parent, 0, cudaGraphCondAssignDefault));
  if_set_cond_kernel<<<1, 1, 0, ps>>>(handles[0], handles[1], pred);
  B200_TRY(dev->CheckLaunch("if_set_cond"));
  for (int b = 0; b < 2; ++b) {
    B200_CUDA_TRY(cudaStreamGetCaptureInfo_v2(ps, &status, &id, &parent, &deps, &num_deps));
    cudaGraphNodeParams params = {};
    params.type = cudaGraphNodeTypeConditional;
    params.conditional.handle = handles[b];
    params.conditional.type = cudaGraphCondTypeIf;
    params.conditional.size = 1;
    cudaGraphNode_t node = nullptr;
    B200_CUDA_TRY(cudaGraphAddNode(&node, parent, deps, num_deps, &params));
    cudaGraph_t body = params.conditional.phGraph_out[0];
    B200_CUDA_TRY(cudaStreamUpdateCaptureDependencies(ps, &node, 1, cudaStreamSetCaptureDependencies));
    B200_CUDA_TRY(cudaStreamBeginCaptureToGraph(ls, body, nullptr, nullptr, 0, cudaStreamCaptureModeThreadLocal));
    Status st = Status::OK();
    {
      StreamOverride in_body(dev, ls);
      st = b == 0 ? run_true() : run_false();
    }
    cudaGraph_t ended = nullptr;
    const cudaError_t ce = cudaStreamEndCapture(ls, &ended);   // always: the loop stream must not stay in capture mode
    B200_TRY(st);
    if (ce != cudaSuccess) { cudaGetLastError(); return Status::Cuda(strfmt("If: recording a branch failed: %s", cudaGetErrorString(ce))); }
  }
  return Status::OK();
}

// Records a While loop into the CUDA graph that `dev->stream()` is being captured into, as a conditional WHILE node:
// cond runs once in front of the node; the node's body graph (recorded on the device's loop stream) runs body, copies the
// new state over the current one, runs cond again and sets the node's condition, all on the device.  `run_cond` and
// `run_body` launch the sub-plans on dev->stream(), whatever it is at the time.
Status RecordWhileNode(Device* dev, int depth, const std::function<Status()>& run_cond, const std::function<Status()>& run_body_and_advance,
                       const unsigned char* pred, int* trips) {
  cudaStream_t ps = dev->stream();
  cudaStream_t ls = nullptr;
  B200_TRY(dev->LoopStream(depth, &ls));   // a loop inside this loop's body records on the next depth's stream
  B200_CUDA_TRY(cudaMemsetAsync(trips, 0, sizeof(int), ps));
  B200_TRY(run_cond());
  cudaStreamCaptureStatus status;
  unsigned long long id = 0;
  cudaGraph_t parent = nullptr;
  const cudaGraphNode_t* deps = nullptr;
  size_t num_deps = 0;
  B200_CUDA_TRY(cudaStreamGetCaptureInfo_v2(ps, &status, &id, &parent, &deps, &num_deps));
  if (status != cudaStreamCaptureStatusActive || !parent) return Status::Invalid("While: the stream is not being recorded");
  cudaGraphConditionalHandle handle;
  B200_CUDA_TRY(cudaGraphConditionalHandleCreate(&handle, parent, 0, cudaGraphCondAssignDefault));
  int* err_flag = dev->kernel_error_flag();
  while_set_cond_kernel<<<1, 1, 0, ps>>>(handle, pred, trips, kWhileMaxIterations, err_flag);
  B200_TRY(dev->CheckLaunch("while_set_cond"));
  B200_CUDA_TRY(cudaStreamGetCaptureInfo_v2(ps, &status, &id, &parent, &deps, &num_deps));
  cudaGraphNodeParams params = {};
  params.type = cudaGraphNodeTypeConditional;
  params.conditional.handle = handle;
  params.conditional.type = cudaGraphCondTypeWhile;
  params.conditional.size = 1;
  cudaGraphNode_t node = nullptr;
  B200_CUDA_TRY(cudaGraphAddNode(&node, parent, deps, num_deps, &params));
  cudaGraph_t body = params.conditional.phGraph_out[0];
  B200_CUDA_TRY(cudaStreamUpdateCaptureDependencies(ps, &node, 1, cudaStreamSetCaptureDependencies));
  B200_CUDA_TRY(cudaStreamBeginCaptureToGraph(ls, body, nullptr, nullptr, 0, cudaStreamCaptureModeThreadLocal));
  Status st = Status::OK();
  {
    StreamOverride in_body(dev, ls);
    st = run_body_and_advance();
    if (st.ok()) st = run_cond();
    if (st.ok()) {
      while_set_cond_kernel<<<1, 1, 0, ls>>>(handle, pred, trips, kWhileMaxIterations, err_flag);
      st = dev->CheckLaunch("while_set_cond");
    }
  }
  cudaGraph_t ended = nullptr;
  const cudaError_t ce = cudaStreamEndCapture(ls, &ended);   // always: the loop stream must not stay in capture mode
  B200_TRY(st);
  if (ce != cudaSuccess) { cudaGetLastError(); return Status::Cuda(strfmt("While: recording the loop body failed: %s", cudaGetErrorString(ce))); }
  return Status::OK();
}

class Planner {
 public:
  Planner(Ctx* ctx, Graph& graph, Exec* exec, int loop_depth = 0) : ctx_(ctx), ex_(exec), g_(graph), loop_depth_(loop_depth) {}

  Status Run(const std::vector<Node*>& feeds, const std::vector<Node*>& targets) {
    const int n = (int)g_.nodes.size();
    live_.assign(n, false);
    uses_.assign(n, 0);
    slot_of_.assign(n, -1);
    // liveness + use counts
    std::vector<Node*> stack(targets.begin(), targets.end());
    while (!stack.empty()) {
      Node* x = stack.back();
      stack.pop_back();
      if (live_[x->id]) continue;
      live_[x->id] = true;
      for (Node* i : x->in) stack.push_back(i);
    }
    for (int i = 0; i < n; ++i)
      if (live_[i]) {
        // A Rope node's table operands do not count as uses: EmitRope reads the table underneath their broadcasts
        // (PeriodicOperand) and materialises only what it really reads, so a table broadcast over the batch that feeds
        // every layer's Rope must not be written out just because it has many users.
        const size_t counted = g_.nodes[i]->op == Op::Rope ? 1 : g_.nodes[i]->in.size();
        for (size_t k = 0; k < counted; ++k) uses_[g_.nodes[i]->in[k]->id]++;
      }
    for (Node* t : targets) uses_[t->id]++;
    // inputs
    for (size_t i = 0; i < feeds.size(); ++i) {
      Node* f = feeds[i];
      if (f->op != Op::Parameter) return Status::Invalid("compile: feed is not a placeholder");
      if (slot_of_[f->id] >= 0) return Status::Invalid("compile: placeholder listed twice");
      const int s = NewSlot(SlotKind::Input, (int)i, f->num_elements() * dtype_size(f->dtype));
      slot_of_[f->id] = s;
      ex_->inputs.push_back(OutputDesc{s, f->dtype, f->dims, ex_->slots[s].nbytes});
    }
    for (int i = 0; i < n; ++i)
      if (live_[i] && g_.nodes[i]->op == Op::Parameter && slot_of_[i] < 0)
        return Status::Invalid("compile: a placeholder used by the targets is not among the feeds");
    // Which node's storage becomes which output: the first target whose base
    // (through views) is a computed node claims that node's slot.
    target_of_base_.clear();
    std::vector<int> target_base(targets.size(), -1);
    for (size_t t = 0; t < targets.size(); ++t) {
      Node* b = ViewBase(targets[t]);
      if (b->op != Op::Parameter && !(b->op == Op::Constant) && !target_of_base_.count(b->id)) {
        target_of_base_[b->id] = (int)t;
        target_base[t] = b->id;
      }
    }
    // Emit in creation order (operands always precede users), materialising
    // what must exist in memory; fused producers are pulled in on demand.
    // ... except the second product of a gated pair act(a W1) * (a W2): it waits for its consumer, which either takes both
    // weights in one launch or asks for it then.
    std::vector<bool> deferred(n, false);
    for (int i = 0; i < n; ++i) {
      if (!live_[i]) continue;
      Node* x = g_.nodes[i].get();
      if (Node* second = GatedSecondProduct(x)) deferred[second->id] = true;
    }
    // ... and an RMSNorm over the last axis whose every user is a DotGeneral taking it as the left operand: a product
    // of a few rows applies the norm itself (EmitDotGeneral); any user that does not asks for the norm then.
    rms_deferred_.assign(n, false);
    {
      std::vector<int> bad(n, 0), users(n, 0);
      for (int i = 0; i < n; ++i) {
        if (!live_[i]) continue;
        Node* u = g_.nodes[i].get();
        for (size_t j = 0; j < u->in.size(); ++j) {
          Node* b = ViewBase(u->in[j]);
          if (b->op != Op::RmsNorm || IsView(u)) continue;   // (a view's own users are seen through it)
          ++users[b->id];
          if (u->op != Op::DotGeneral || j != 0) ++bad[b->id];
        }
      }
      for (int i = 0; i < n; ++i) {
        if (!live_[i]) continue;
        Node* r = g_.nodes[i].get();
        static const bool rms_on = []() { const char* v = getenv("B200MLX_GEMM_SKINNY_RMS"); return !(v && v[0] == '0'); }();
        if (!rms_on || r->op != Op::RmsNorm || bad[i] || users[i] == 0 || target_of_base_.count(i)) continue;
        if (r->dtype != B200_BFLOAT16 && r->dtype != B200_FLOAT16) continue;
        const bool one_last_axis = r->ia.size() == 3 && r->ia[0] != 0 && r->ia[1] == 0 && r->ia[2] == r->rank() - 1;
        if (!one_last_axis || r->in.size() < 2 || r->in[1]->num_elements() != r->dims.back() || r->in[1]->dtype != r->dtype) continue;
        rms_deferred_[i] = true;
        deferred[i] = true;
      }
    }
    for (int i = 0; i < n; ++i) {
      if (!live_[i]) continue;
      Node* x = g_.nodes[i].get();
      if (MustMaterialize(x) && !deferred[i]) B200_TRY(EnsureMaterialized(x));
    }
    // Outputs.
    for (size_t t = 0; t < targets.size(); ++t) {
      Node* x = targets[t];
      B200_TRY(EnsureMaterialized(x));
      int s = slot_of_[ViewBase(x)->id];
      const int64_t nbytes = x->num_elements() * dtype_size(x->dtype);
      if (target_base[t] < 0) {
        // target is (a view of) an input, a constant, or storage another output owns: copy
        const int o = NewSlot(SlotKind::Output, (int)t, nbytes);
        const int src = s;
        Step st;
        st.desc = "copy -> output " + std::to_string(t);
        st.reads = {src};
        st.writes = {o};
        st.run = [src, o, nbytes](Device* dev, void* const* p) -> Status {
          if (nbytes == 0) return Status::OK();
          B200_CUDA_TRY(cudaMemcpyAsync(p[o], p[src], (size_t)nbytes, cudaMemcpyDeviceToDevice, dev->stream()));
          return Status::OK();
        };
        st.launches = 0;
        ex_->steps.push_back(std::move(st));
        s = o;
      }
      ex_->outputs.push_back(OutputDesc{s, x->dtype, x->dims, nbytes});
    }
    PlanArena();
    ex_->num_launches = 0;
    for (auto& st : ex_->steps) ex_->num_launches += st.launches;
    return Status::OK();
  }

 private:
  Ctx* ctx_;
  Exec* ex_;
  Graph& g_;
  int loop_depth_;   // how many While loops enclose the graph being planned
  std::vector<bool> live_;
  std::vector<int> uses_;
  std::vector<int> slot_of_;  // node id -> slot (materialised nodes; views resolve through ViewBase)
  std::unordered_map<int, int> target_of_base_;

  int NewSlot(SlotKind kind, int index, int64_t nbytes) {
    Slot s;
    s.kind = kind;
    s.index = index;
    s.nbytes = nbytes;
    ex_->slots.push_back(s);
    return (int)ex_->slots.size() - 1;
  }
  int NewValueSlot(Node* x) {
    const int64_t nbytes = x->num_elements() * dtype_size(x->dtype);
    auto it = target_of_base_.find(x->id);
    const int s = (it != target_of_base_.end()) ? NewSlot(SlotKind::Output, it->second, nbytes) : NewSlot(SlotKind::Arena, 0, nbytes);
    slot_of_[x->id] = s;
    return s;
  }
  int NewTemp(int64_t nbytes) { return NewSlot(SlotKind::Arena, 0, nbytes); }

  static bool IsView(Node* x) { return x->op == Op::Reshape || x->op == Op::Identity; }
  static Node* ViewBase(Node* x) {
    while (IsView(x)) x = x->in[0];
    return x;
  }
  static bool IsScalarConst(Node* x) { return x->op == Op::Constant && x->num_elements() == 1; }
  // A Reshape whose non-1 dims are the operand's non-1 dims in the same order.
  static bool UnitReshape(Node* x) {
    if (x->op != Op::Reshape) return false;
    std::vector<int64_t> a, b;
    for (auto d : x->dims) if (d != 1) a.push_back(d);
    for (auto d : x->in[0]->dims) if (d != 1) b.push_back(d);
    return a == b;
  }
  // Ops that can be evaluated inside an elementwise program.
  static bool Fusible(Node* x) {
    if (op_is_elementwise(x->op)) return true;
    switch (x->op) {
      case Op::BroadcastInDim: case Op::Transpose: case Op::Slice: case Op::Reverse: case Op::Iota: return true;
      case Op::Constant: return IsScalarConst(x);
      default: return false;
    }
  }
  // Cheap enough to recompute in every consumer instead of storing.
  bool Cheap(Node* x) const {
    if (x->op == Op::Iota || IsScalarConst(x)) return true;
    if ((x->op == Op::BroadcastInDim || x->op == Op::Cast || IsView(x)) && Cheap(x->in[0])) return true;
    return false;
  }
  bool MustMaterialize(Node* x) const {
    if (x->op == Op::Parameter) return false;       // already in memory
    if (IsView(x)) return false;                    // resolved through its base
    if (IsScalarConst(x)) return false;             // becomes an immediate (materialised on demand if a kernel needs memory)
    if (!Fusible(x)) return true;
    if (target_of_base_.count(x->id)) return true;
    if (uses_[x->id] > 1 && !Cheap(x)) return true;
    return false;                                   // inlined into its consumer, or pulled in on demand
  }

  // x = DotGeneral(a, W1)[+ bias][activation] multiplied (the compile-time rewrite's fa[1] == 2) by a plain
  // DotGeneral(a, W2) of the same shapes that feeds nothing else and is no output: returns that second product.
  Node* GatedSecondProduct(Node* x) const {
    if (x->op != Op::DotGeneral || x->fa.size() < 2 || x->fa[1] != 2.0 || x->in.size() < 3) return nullptr;
    Node* r = x->in.back();
    if (r->op != Op::DotGeneral || uses_[r->id] != 1 || target_of_base_.count(r->id) || r->in.size() != 2 || r->in[0] != x->in[0] ||
        r->ia != x->ia || r->in[1]->dims != x->in[1]->dims || r->in[1]->dtype != x->in[1]->dtype || r->dtype != x->dtype)
      return nullptr;
    if ((!r->fa.empty() && r->fa[0] != 0) || (r->fa.size() > 1 && r->fa[1] != 0)) return nullptr;
    if (x->dtype != B200_BFLOAT16 && x->dtype != B200_FLOAT16) return nullptr;
    return r;
  }

  Status EnsureMaterialized(Node* x) {
    Node* b = ViewBase(x);
    if (slot_of_[b->id] >= 0) return Status::OK();
    return Materialize(b);
  }
  int SlotOf(Node* x) const { return slot_of_[ViewBase(x)->id]; }

  // ------------------------------------------------------------ dispatch ---
  Status Materialize(Node* x) {
    switch (x->op) {
      case Op::Parameter: return Status::Invalid("compile: unbound placeholder");
      case Op::Constant: return EmitConstant(x);
      case Op::DotGeneral: return EmitDotGeneral(x);
      case Op::Reduce: return EmitReduce(x);
      case Op::ArgMinMax: return EmitArgMinMax(x);
      case Op::Gather: return EmitGather(x);
      case Op::Scatter: return EmitScatter(x);
      case Op::RngBits: return EmitRngBits(x);
      case Op::ArgSort: return EmitArgSort(x);
      case Op::While: return EmitWhile(x);
      case Op::WhileResult:
        B200_TRY(EnsureMaterialized(x->in[0]));
        return slot_of_[x->id] >= 0 ? Status::OK() : Status::Invalid("compile: While did not produce its result");
      case Op::If: return EmitIf(x);
      case Op::IfResult:
        B200_TRY(EnsureMaterialized(x->in[0]));
        return slot_of_[x->id] >= 0 ? Status::OK() : Status::Invalid("compile: If did not produce its result");
      case Op::ClosureParam: return Status::Invalid("compile: a closure's parameter is used outside its closure");
      case Op::Softmax: return EmitSoftmax(x);
      case Op::SoftmaxMasked: return EmitSoftmaxMasked(x);
      case Op::LayerNorm: case Op::RmsNorm: return EmitNorm(x);
      case Op::Attention: return EmitAttention(x);
      case Op::Rope: return EmitRope(x);
      case Op::Concatenate: return EmitConcatenate(x);
      case Op::Pad: return EmitPad(x);
      case Op::DynamicSlice: case Op::DynamicUpdateSlice: return EmitDynamicSlice(x);
      case Op::Transpose: case Op::Slice: case Op::Reverse: case Op::BroadcastInDim:
        if (ViewBase(x->in[0])->op == Op::Parameter || slot_of_[ViewBase(x->in[0])->id] >= 0 || !Fusible(ViewBase(x->in[0])) ||
            IsView(x->in[0]))
          return EmitMovement(x);
        return EmitEwise(x);
      default:
        if (Fusible(x)) return EmitEwise(x);
        return Status::Unsupported(strfmt("compile: no lowering for %s", op_name(x->op)));
    }
  }

  // Device memory of the plan's own, zeroed once when the plan is built (counters that their kernel leaves at zero).
  Status NewZeroedConst(int64_t nbytes, int* slot) {
    void* p = nullptr;
    B200_TRY(ex_->dev->Alloc(nbytes > 0 ? nbytes : 1, &p));
    ex_->const_ptrs.push_back(p);
    B200_TRY(ex_->dev->MakeCurrent());
    B200_CUDA_TRY(cudaMemsetAsync(p, 0, (size_t)(nbytes > 0 ? nbytes : 1), ex_->dev->stream()));
    B200_CUDA_TRY(cudaStreamSynchronize(ex_->dev->stream()));
    *slot = NewSlot(SlotKind::Const, (int)ex_->const_ptrs.size() - 1, nbytes);
    return Status::OK();
  }

  Status EmitConstant(Node* x) {
    void* p = nullptr;
    const int64_t nbytes = (int64_t)x->data.size();
    B200_TRY(ex_->dev->Alloc(nbytes > 0 ? nbytes : 1, &p));
    if (nbytes > 0) {
      B200_TRY(ex_->dev->MakeCurrent());
      B200_CUDA_TRY(cudaMemcpyAsync(p, x->data.data(), (size_t)nbytes, cudaMemcpyHostToDevice, ex_->dev->stream()));
      B200_CUDA_TRY(cudaStreamSynchronize(ex_->dev->stream()));
    }
    ex_->const_ptrs.push_back(p);
    slot_of_[x->id] = NewSlot(SlotKind::Const, (int)ex_->const_ptrs.size() - 1, nbytes);
    return Status::OK();
  }

  // ------------------------------------------------- elementwise programs ---
  struct EwBuild {
    k::EwProgram prog;
    std::vector<int> leaf_slots;
    std::unordered_map<std::string, int> memo;  // (node id, index map) -> virtual register
    int next_vreg = 0;
    int op_budget = 0;
    bool overflow = false;
    std::vector<bool> dim_used_by_iota;
    std::vector<std::array<int, 3>> vreg_ops;  // per instruction (= virtual register): operand vregs, -1 = none
    std::vector<int64_t> leaf_offsets;         // element offset added to each leaf's base pointer
  };

  static uint64_t ImmBits(int dtype, const uint8_t* data) {
    // register representation of one element (see kernels/ewise.cu)
    switch (dtype) {
      case B200_FLOAT32: { uint32_t u; memcpy(&u, data, 4); return u; }
      case B200_BFLOAT16: { uint16_t h; memcpy(&h, data, 2); return (uint32_t)h << 16; }
      case B200_FLOAT16: {
        uint16_t h; memcpy(&h, data, 2);
        const uint32_t sign = (h >> 15) & 1, exp = (h >> 10) & 0x1f, man = h & 0x3ff;
        float f;
        if (exp == 0) f = ldexpf((float)man, -24);
        else if (exp == 31) f = man ? NAN : INFINITY;
        else f = ldexpf((float)(man | 0x400), (int)exp - 25);
        if (sign) f = -f;
        uint32_t u; memcpy(&u, &f, 4); return u;
      }
      case B200_FLOAT64: case B200_INT64: case B200_UINT64: { uint64_t u; memcpy(&u, data, 8); return u; }
      case B200_INT32: case B200_UINT32: { uint32_t u; memcpy(&u, data, 4); return u; }
      case B200_INT16: { int16_t v; memcpy(&v, data, 2); return (uint32_t)(int32_t)v; }
      case B200_UINT16: { uint16_t v; memcpy(&v, data, 2); return v; }
      case B200_INT8: return (uint32_t)(int32_t)(int8_t)data[0];
      case B200_UINT8: return data[0];
      case B200_BOOL: return data[0] ? 1 : 0;
    }
    return 0;
  }

  int PushInstr(EwBuild& b, k::EwInstr in) {
    if (b.prog.num_instr >= k::kEwMaxInstr) { b.overflow = true; return 0; }
    in.dst = 0;
    const int v = b.next_vreg++;
    b.prog.instr[b.prog.num_instr++] = in;
    return v;
  }

  // Emits code computing node x under index map im; returns the virtual register.
  Status BuildExpr(EwBuild& b, Node* x, const IndexMap& im, int* out_vreg) {
    if (b.overflow) { *out_vreg = 0; return Status::OK(); }
    const std::string key = std::to_string(x->id) + "|" + im.key();
    auto it = b.memo.find(key);
    if (it != b.memo.end()) { *out_vreg = it->second; return Status::OK(); }
    int v = -1;
    Node* base = ViewBase(x);
    const bool in_memory = base->op == Op::Parameter || slot_of_[base->id] >= 0;
    if (!in_memory && IsView(x) && Fusible(ViewBase(x->in[0])) && (x->op == Op::Identity || UnitReshape(x))) {
      // A view that only adds or drops size-1 dims of a value that is not in
      // memory: carry the index map through instead of forcing a store.
      Node* src = x->in[0];
      IndexMap sm;
      int xi = 0;
      for (int j = 0; j < src->rank(); ++j) {
        if (src->dims[j] == 1 && x->op != Op::Identity) { sm.m.push_back(-1); sm.a.push_back(0); sm.b.push_back(0); continue; }
        if (x->op != Op::Identity)
          while (x->dims[xi] == 1) ++xi;
        sm.m.push_back(im.m[xi]); sm.a.push_back(im.a[xi]); sm.b.push_back(im.b[xi]);
        ++xi;
      }
      return BuildExprMemo(b, key, src, sm, out_vreg);
    }
    const bool inline_it = !in_memory && !IsView(x) && Fusible(x) && (b.op_budget > 0 || Cheap(x));
    if (!inline_it) {
      // leaf: load from memory through the index map
      if (!in_memory) B200_TRY(Materialize(base));
      if (b.prog.num_leaves >= k::kEwMaxLeaves) { b.overflow = true; *out_vreg = 0; return Status::OK(); }
      const int slot = slot_of_[base->id];
      k::EwLeaf& lf = b.prog.leaves[b.prog.num_leaves];
      lf.ptr = nullptr;
      lf.dtype = x->dtype;
      for (int d = 0; d < k::kMaxDims; ++d) lf.strides[d] = 0;
      const std::vector<int64_t> cs = dense_strides(x->dims);
      int64_t base_off = 0;
      for (int i = 0; i < x->rank(); ++i) {
        base_off += cs[i] * im.b[i];
        if (im.m[i] >= 0) lf.strides[im.m[i]] += cs[i] * im.a[i];
      }
      b.leaf_offsets.push_back(base_off);
      b.leaf_slots.push_back(slot);
      k::EwInstr in{};
      in.kind = k::EW_LOAD;
      in.dtype = in.sdtype = (uint8_t)x->dtype;
      in.a = (uint8_t)b.prog.num_leaves;
      b.prog.num_leaves++;
      b.vreg_ops.push_back({-1, -1, -1});
      v = PushInstr(b, in);
    } else if (x->op == Op::Constant) {
      k::EwInstr in{};
      in.kind = k::EW_IMM;
      in.dtype = in.sdtype = (uint8_t)x->dtype;
      in.imm = ImmBits(x->dtype, x->data.data());
      b.vreg_ops.push_back({-1, -1, -1});
      v = PushInstr(b, in);
    } else if (x->op == Op::Iota) {
      const int ax = (int)x->ia[0];
      k::EwInstr in{};
      in.dtype = in.sdtype = (uint8_t)x->dtype;
      if (im.m[ax] < 0 || b.prog.dims[im.m[ax]] == 1) {
        // constant coordinate
        in.kind = k::EW_IMM;
        in.imm = IotaImm(x->dtype, im.b[ax]);
      } else if (im.a[ax] == 1 && im.b[ax] == 0) {
        in.kind = k::EW_IOTA;
        in.a = (uint8_t)im.m[ax];
        b.dim_used_by_iota[im.m[ax]] = true;
      } else {
        // strided / offset iota: not expressible as a plain coordinate; keep it in memory
        B200_TRY(Materialize(x));
        return BuildExpr(b, x, im, out_vreg);
      }
      b.vreg_ops.push_back({-1, -1, -1});
      v = PushInstr(b, in);
    } else if (x->op == Op::BroadcastInDim) {
      Node* src = x->in[0];
      IndexMap sm;
      for (int i = 0; i < src->rank(); ++i) {
        const int oa = (int)x->ia[i];
        if (src->dims[i] == 1 && x->dims[oa] != 1) { sm.m.push_back(-1); sm.a.push_back(0); sm.b.push_back(0); }
        else { sm.m.push_back(im.m[oa]); sm.a.push_back(im.a[oa]); sm.b.push_back(im.b[oa]); }
      }
      return BuildExprMemo(b, key, src, sm, out_vreg);
    } else if (x->op == Op::Transpose) {
      Node* src = x->in[0];
      IndexMap sm;
      sm.m.resize(src->rank()); sm.a.resize(src->rank()); sm.b.resize(src->rank());
      for (int i = 0; i < x->rank(); ++i) {
        const int p = (int)x->ia[i];
        sm.m[p] = im.m[i]; sm.a[p] = im.a[i]; sm.b[p] = im.b[i];
      }
      return BuildExprMemo(b, key, src, sm, out_vreg);
    } else if (x->op == Op::Slice) {
      Node* src = x->in[0];
      IndexMap sm = im;
      for (int i = 0; i < x->rank(); ++i) {
        const int64_t start = x->ia[2 * i], stride = x->ia[2 * i + 1];
        sm.a[i] = im.a[i] * stride;
        sm.b[i] = im.b[i] * stride + start;
      }
      return BuildExprMemo(b, key, src, sm, out_vreg);
    } else if (x->op == Op::Reverse) {
      Node* src = x->in[0];
      IndexMap sm = im;
      for (int64_t ax : x->ia) {
        sm.a[ax] = -im.a[ax];
        sm.b[ax] = x->dims[ax] - 1 - im.b[ax];
      }
      return BuildExprMemo(b, key, src, sm, out_vreg);
    } else {
      // unary / binary / compare / where / clamp / cast
      b.op_budget--;
      int r[3] = {-1, -1, -1};
      for (size_t i = 0; i < x->in.size() && i < 3; ++i) {
        Node* o = x->in[i];
        // NumPy-style broadcast: operand dims right-aligned to the result's
        IndexMap om;
        const int off = x->rank() - o->rank();
        for (int d = 0; d < o->rank(); ++d) {
          if (o->dims[d] == 1 && x->dims[off + d] != 1) { om.m.push_back(-1); om.a.push_back(0); om.b.push_back(0); }
          else { om.m.push_back(im.m[off + d]); om.a.push_back(im.a[off + d]); om.b.push_back(im.b[off + d]); }
        }
        B200_TRY(BuildExpr(b, o, om, &r[i]));
        if (b.overflow) { *out_vreg = 0; return Status::OK(); }
      }
      k::EwInstr in{};
      if (x->op == Op::Cast) {
        in.kind = k::EW_CAST;
        in.dtype = (uint8_t)x->dtype;
        in.sdtype = (uint8_t)x->in[0]->dtype;
      } else {
        in.kind = k::EW_OP;
        in.op = (uint8_t)x->op;
        in.dtype = (uint8_t)x->dtype;
        in.sdtype = (uint8_t)((x->op == Op::Where) ? x->in[1]->dtype : x->in[0]->dtype);
      }
      b.vreg_ops.push_back({r[0], r[1], r[2]});
      v = PushInstr(b, in);
    }
    b.memo[key] = v;
    *out_vreg = v;
    return Status::OK();
  }
  Status BuildExprMemo(EwBuild& b, const std::string& key, Node* src, const IndexMap& sm, int* out_vreg) {
    B200_TRY(BuildExpr(b, src, sm, out_vreg));
    b.memo[key] = *out_vreg;
    return Status::OK();
  }
  static uint64_t IotaImm(int dtype, int64_t v) {
    switch (dtype) {
      case B200_FLOAT32: case B200_BFLOAT16: case B200_FLOAT16: { float f = (float)v; uint32_t u; memcpy(&u, &f, 4); return u; }
      case B200_FLOAT64: { double d = (double)v; uint64_t u; memcpy(&u, &d, 8); return u; }
      case B200_INT64: case B200_UINT64: return (uint64_t)v;
      case B200_INT8: return (uint32_t)(int32_t)(int8_t)v;
      case B200_INT16: return (uint32_t)(int32_t)(int16_t)v;
      case B200_UINT8: return (uint32_t)(uint8_t)v;
      case B200_UINT16: return (uint32_t)(uint16_t)v;
      default: return (uint32_t)v;
    }
  }

  Status EmitEwise(Node* x) {
    if (x->rank() > k::kMaxDims) return Status::Unsupported("compile: elementwise result with more than 8 dims");
    // Try with a generous inlining budget; on overflow of the interpreter's
    // limits retry with a smaller one (deeper operands then become kernels of their own).
    for (int budget = 24; budget >= 1; budget /= 2) {
      EwBuild b;
      b.op_budget = budget;
      b.dim_used_by_iota.assign(x->rank() + 1, false);
      b.prog.rank = x->rank();
      for (int d = 0; d < x->rank(); ++d) b.prog.dims[d] = x->dims[d];
      int root = 0;
      // The root itself must be computed here even when it has a slot pending.
      B200_TRY(BuildRoot(b, x, &root));
      if (b.overflow) continue;
      if (!AssignRegisters(b, root)) continue;
      return FinishEwise(b, x);
    }
    return Status::Unsupported(strfmt("compile: elementwise node %s does not fit the interpreter", op_name(x->op)));
  }

  Status BuildRoot(EwBuild& b, Node* x, int* root) {
    // x has no slot yet, so BuildExpr would inline it if budget allows; force that.
    if (b.op_budget < 1) b.op_budget = 1;
    return BuildExpr(b, x, IndexMap::Identity(x->rank()), root);
  }

  // Linear-scan allocation of physical registers from virtual ones.
  bool AssignRegisters(EwBuild& b, int root_vreg) {
    const int ni = b.prog.num_instr;
    std::vector<int> last_use(ni, -1), phys(ni, -1);
    for (int i = 0; i < ni; ++i)
      for (int o : b.vreg_ops[i])
        if (o >= 0) last_use[o] = i;
    last_use[root_vreg] = ni;  // live to the end
    std::vector<int> free_regs;
    int next = 0;
    for (int i = 0; i < ni; ++i) {
      // operands whose last use is this instruction free their register AFTER it reads them,
      // but the destination may reuse such a register only if it is not also read here by
      // another element of the vector -- each thread reads all operands before writing, so reuse is safe.
      k::EwInstr& in = b.prog.instr[i];
      const auto& ops = b.vreg_ops[i];
      if (in.kind == k::EW_OP || in.kind == k::EW_CAST) {
        in.a = (uint8_t)(ops[0] >= 0 ? phys[ops[0]] : 0);
        in.b = (uint8_t)(ops[1] >= 0 ? phys[ops[1]] : 0);
        in.c = (uint8_t)(ops[2] >= 0 ? phys[ops[2]] : 0);
      }
      int dst;
      if (!free_regs.empty()) { dst = free_regs.back(); free_regs.pop_back(); }
      else dst = next++;
      if (dst >= k::kEwMaxRegs) return false;
      phys[i] = dst;
      in.dst = (uint8_t)dst;
      for (int o : ops)
        if (o >= 0 && last_use[o] == i) {
          bool dup = false;
          for (int f : free_regs) dup |= (f == phys[o]);
          if (!dup) free_regs.push_back(phys[o]);
        }
      if (last_use[i] < 0) free_regs.push_back(dst);  // value never read
    }
    b.prog.num_regs = next;
    b.prog.out_reg = phys[root_vreg];
    return true;
  }

  // Drops size-1 dims and collapses neighbouring output dims that every leaf walks contiguously.  `fences` lists dims d
  // (of the uncollapsed space) that must not be merged with dim d - 1: a reduction keeps the boundaries of its reduced
  // run.  Returns, through remap_out, where each original dim went.
  static void CollapseProgram(const EwBuild& b, k::EwProgram& prog, const std::vector<int>& fences, int* remap_out = nullptr) {
    int r = 0;
    int remap[k::kMaxDims];
    int64_t dims[k::kMaxDims];
    int64_t strides[k::kEwMaxLeaves][k::kMaxDims];
    bool kept_iota[k::kMaxDims];
    bool fence_pending = false;
    for (int d = 0; d < prog.rank; ++d) {
      remap[d] = r > 0 ? r - 1 : 0;
      for (int f : fences) fence_pending |= (f == d);
      if (prog.dims[d] == 1) continue;  // never an iota dim (BuildExpr turns those into immediates)
      bool merge = r > 0 && !fence_pending && !b.dim_used_by_iota[d] && !kept_iota[r - 1];
      if (merge)
        for (int l = 0; l < prog.num_leaves; ++l) merge &= (strides[l][r - 1] == prog.leaves[l].strides[d] * prog.dims[d]);
      if (merge) {
        dims[r - 1] *= prog.dims[d];
        for (int l = 0; l < prog.num_leaves; ++l) strides[l][r - 1] = prog.leaves[l].strides[d];
        remap[d] = r - 1;
      } else {
        dims[r] = prog.dims[d];
        for (int l = 0; l < prog.num_leaves; ++l) strides[l][r] = prog.leaves[l].strides[d];
        kept_iota[r] = b.dim_used_by_iota[d];
        remap[d] = r;
        ++r;
      }
      fence_pending = false;
    }
    if (r == 0) {
      dims[0] = 1;
      for (int l = 0; l < prog.num_leaves; ++l) strides[l][0] = 0;
      r = 1;
    }
    for (int i = 0; i < prog.num_instr; ++i)
      if (prog.instr[i].kind == k::EW_IOTA) prog.instr[i].a = (uint8_t)remap[prog.instr[i].a];
    if (remap_out)
      for (int d = 0; d < prog.rank; ++d) remap_out[d] = remap[d];
    prog.rank = r;
    for (int d = 0; d < k::kMaxDims; ++d) {
      prog.dims[d] = d < r ? dims[d] : 0;
      for (int l = 0; l < prog.num_leaves; ++l) prog.leaves[l].strides[d] = d < r ? strides[l][d] : 0;
    }
  }

  Status FinishEwise(EwBuild& b, Node* x) {
    k::EwProgram prog = b.prog;
    prog.out_dtype = x->dtype;
    prog.wide = dtype_size(x->dtype) == 8;
    for (int i = 0; i < prog.num_instr; ++i)
      if (dtype_size(prog.instr[i].dtype) == 8 || dtype_size(prog.instr[i].sdtype) == 8) prog.wide = true;
    CollapseProgram(b, prog, {});
    const int out_slot = NewValueSlot(x);
    // The chain as one straight-line kernel, compiled now (NVRTC) and cached by its text; without NVRTC the interpreter
    // kernel runs the program.  The two templated fast shapes keep priority at launch time (they depend on pointers).
    k::EwJit* jit = nullptr;
    if (!k::ewise_jit_prepare(ex_->dev, prog, &jit).ok()) jit = nullptr;
    Step st;
    std::ostringstream os;
    os << "ewise[" << op_name(x->op) << " instr=" << prog.num_instr << " leaves=" << prog.num_leaves << " regs=" << prog.num_regs
       << (prog.wide ? " wide" : "") << (jit ? " compiled" : " interpreted") << "]";
    st.desc = os.str();
    st.reads = b.leaf_slots;
    st.writes = {out_slot};
    std::vector<int> leaf_slots = b.leaf_slots;
    std::vector<int64_t> leaf_offsets = b.leaf_offsets;
    st.run = [prog, leaf_slots, leaf_offsets, out_slot, jit](Device* dev, void* const* p) -> Status {
      k::EwProgram q = prog;
      for (int l = 0; l < q.num_leaves; ++l)
        q.leaves[l].ptr = (const char*)p[leaf_slots[l]] + leaf_offsets[l] * dtype_size(q.leaves[l].dtype);
      q.out = p[out_slot];
      if (!jit) return k::ewise_run(dev, q);
      // x op y keeps its templated kernel (0.92 - 0.97 of the copy rate); everything else, the small trees included, runs
      // the compiled chain, which rounds 16-bit results two at a time
      bool taken = false;
      B200_TRY(k::ewise_run_fast(dev, q, &taken, /*trees=*/false));
      if (taken) return Status::OK();
      return k::ewise_jit_run(dev, jit, q);
    };
    ex_->steps.push_back(std::move(st));
    return Status::OK();
  }

  // --------------------------------------------------------- data movement ---
  // A lone Transpose / Slice / Reverse / BroadcastInDim of something already in memory.
  Status EmitMovement(Node* x) {
    Node* src = x->in[0];
    B200_TRY(EnsureMaterialized(src));
    if (x->rank() > k::kMaxDims) return Status::Unsupported("compile: more than 8 dims");
    const int in_slot = SlotOf(src);
    k::StridedCopyParams p;
    p.elt_size = dtype_size(x->dtype);
    p.rank = x->rank();
    const std::vector<int64_t> cs = dense_strides(src->dims), os = dense_strides(x->dims);
    for (int d = 0; d < x->rank(); ++d) { p.dims[d] = x->dims[d]; p.out_strides[d] = os[d]; p.in_strides[d] = 0; }
    switch (x->op) {
      case Op::Transpose:
        for (int d = 0; d < x->rank(); ++d) p.in_strides[d] = cs[x->ia[d]];
        break;
      case Op::Slice:
        for (int d = 0; d < x->rank(); ++d) { p.in_strides[d] = cs[d] * x->ia[2 * d + 1]; p.in_offset += cs[d] * x->ia[2 * d]; }
        break;
      case Op::Reverse:
        for (int d = 0; d < x->rank(); ++d) p.in_strides[d] = cs[d];
        for (int64_t ax : x->ia) { p.in_strides[ax] = -cs[ax]; p.in_offset += cs[ax] * (x->dims[ax] - 1); }
        break;
      default:  // BroadcastInDim
        for (int i = 0; i < src->rank(); ++i) {
          const int oa = (int)x->ia[i];
          p.in_strides[oa] = (src->dims[i] == 1 && x->dims[oa] != 1) ? 0 : cs[i];
        }
        break;
    }
    // Batched swap of the two innermost dims goes through the tiled transpose.
    bool tiled = false;
    int64_t tb = 1, trows = 0, tcols = 0;
    if (x->op == Op::Transpose && x->rank() >= 2) {
      const int r = x->rank();
      tiled = x->ia[r - 1] == r - 2 && x->ia[r - 2] == r - 1;
      for (int d = 0; d < r - 2 && tiled; ++d) { tiled = x->ia[d] == d; tb *= x->dims[d]; }
      trows = src->dims[r - 2];
      tcols = src->dims[r - 1];
      if (tb > 65535 || (trows + 31) / 32 > 65535) tiled = false;
    }
    const int out_slot = NewValueSlot(x);
    Step st;
    st.desc = std::string("move[") + op_name(x->op) + (tiled ? " tiled" : "") + "]";
    st.reads = {in_slot};
    st.writes = {out_slot};
    const int es = p.elt_size;
    if (tiled) {
      st.run = [=](Device* dev, void* const* ptrs) -> Status { return k::transpose_2d(dev, ptrs[in_slot], ptrs[out_slot], tb, trows, tcols, es); };
    } else {
      st.run = [p, in_slot, out_slot](Device* dev, void* const* ptrs) -> Status {
        k::StridedCopyParams q = p;
        q.x = ptrs[in_slot];
        q.y = ptrs[out_slot];
        return k::strided_copy(dev, q);
      };
    }
    ex_->steps.push_back(std::move(st));
    return Status::OK();
  }

  // Copies `src` (any materialised node) into a sub-block of slot `out_slot`.
  void EmitBlockCopy(Node* src, int out_slot, const std::vector<int64_t>& out_dims, const std::vector<int64_t>& out_start,
                     const char* what) {
    k::StridedCopyParams p;
    p.elt_size = dtype_size(src->dtype);
    p.rank = src->rank();
    const std::vector<int64_t> cs = dense_strides(src->dims), os = dense_strides(out_dims);
    for (int d = 0; d < src->rank(); ++d) {
      p.dims[d] = src->dims[d];
      p.in_strides[d] = cs[d];
      p.out_strides[d] = os[d];
      p.out_offset += os[d] * out_start[d];
    }
    const int in_slot = SlotOf(src);
    Step st;
    st.desc = std::string("move[") + what + "]";
    st.reads = {in_slot};
    st.writes = {out_slot};
    st.run = [p, in_slot, out_slot](Device* dev, void* const* ptrs) -> Status {
      k::StridedCopyParams q = p;
      q.x = ptrs[in_slot];
      q.y = ptrs[out_slot];
      return k::strided_copy(dev, q);
    };
    ex_->steps.push_back(std::move(st));
  }

  Status EmitConcatenate(Node* x) {
    if (x->rank() > k::kMaxDims) return Status::Unsupported("compile: more than 8 dims");
    // An operand that is a not-yet-stored Slice of something in memory is copied straight from its source.
    auto direct_slice = [&](Node* in) {
      return in->op == Op::Slice && slot_of_[in->id] < 0 && uses_[in->id] == 1;
    };
    for (Node* in : x->in) B200_TRY(EnsureMaterialized(direct_slice(in) ? in->in[0] : in));
    const int out_slot = NewValueSlot(x);
    const int ax = (int)x->ia[0];
    {
      // Small operands laid end to end (everything before the axis has extent 1): one launch instead of one per operand.
      bool flat = (int)x->in.size() <= k::kMaxConcatFlat && x->num_elements() * dtype_size(x->dtype) <= (1 << 20);
      for (int d = 0; d < ax && flat; ++d) flat = x->dims[d] == 1;
      for (Node* in : x->in) flat = flat && !direct_slice(in);
      if (flat) {
        std::vector<int> slots;
        std::vector<int64_t> counts;
        for (Node* in : x->in) { slots.push_back(SlotOf(in)); counts.push_back(in->num_elements()); }
        const int es = dtype_size(x->dtype);
        Step st;
        st.desc = strfmt("move[Concatenate x%d flat]", (int)x->in.size());
        st.reads = slots;
        st.writes = {out_slot};
        st.run = [slots, counts, out_slot, es](Device* dev, void* const* ptrs) -> Status {
          const void* src[k::kMaxConcatFlat];
          for (size_t i = 0; i < slots.size(); ++i) src[i] = ptrs[slots[i]];
          return k::concat_flat(dev, src, counts.data(), (int)slots.size(), ptrs[out_slot], es);
        };
        ex_->steps.push_back(std::move(st));
        return Status::OK();
      }
    }
    int64_t pos = 0;
    for (Node* in : x->in) {
      std::vector<int64_t> start(x->rank(), 0);
      start[ax] = pos;
      if (direct_slice(in)) {
        Node* src = in->in[0];
        k::StridedCopyParams p;
        p.elt_size = dtype_size(in->dtype);
        p.rank = in->rank();
        const std::vector<int64_t> cs = dense_strides(src->dims), os = dense_strides(x->dims);
        for (int d = 0; d < in->rank(); ++d) {
          p.dims[d] = in->dims[d];
          p.in_strides[d] = cs[d] * in->ia[2 * d + 1];
          p.in_offset += cs[d] * in->ia[2 * d];
          p.out_strides[d] = os[d];
          p.out_offset += os[d] * start[d];
        }
        const int in_slot = SlotOf(src);
        Step st;
        st.desc = "move[Concatenate of Slice]";
        st.reads = {in_slot};
        st.writes = {out_slot};
        st.run = [p, in_slot, out_slot](Device* dev, void* const* ptrs) -> Status {
          k::StridedCopyParams q = p;
          q.x = ptrs[in_slot];
          q.y = ptrs[out_slot];
          return k::strided_copy(dev, q);
        };
        ex_->steps.push_back(std::move(st));
      } else {
        EmitBlockCopy(in, out_slot, x->dims, start, "Concatenate");
      }
      pos += in->dims[ax];
    }
    return Status::OK();
  }

  // The most recent DynamicUpdateSlice step, kept so that a twin that follows it directly can join it.
  struct LastDus {
    int step = -1;
    std::vector<int> start_slots;
    int rank = 0, elt_size = 0, out_slot = -1, x_slot = -1;
    int64_t x_dims[k::kMaxDims] = {0}, b_dims[k::kMaxDims] = {0};
    std::function<k::DynSliceParams(void* const*)> bind;
  } last_dus_;

  // DynamicSlice (inputs: operand, starts...) and DynamicUpdateSlice (operand, update, starts...): the start scalars are
  // read on the device, so the launch plan stays static.
  Status EmitDynamicSlice(Node* x) {
    const bool update = x->op == Op::DynamicUpdateSlice;
    Node* operand = x->in[0];
    Node* upd = update ? x->in[1] : nullptr;
    const size_t first = update ? 2 : 1;
    B200_TRY(EnsureMaterialized(operand));
    // an update block that is a column range of a wider tensor (the K or V part of a fused projection) is read in place
    Node* upd_src = nullptr;
    int64_t upd_off = 0;
    std::vector<int64_t> upd_strides;
    if (upd && ColumnRangeView(upd, &upd_src, &upd_off, &upd_strides)) B200_TRY(EnsureMaterialized(upd_src));
    else upd_src = nullptr;
    if (upd && !upd_src) B200_TRY(EnsureMaterialized(upd));
    for (size_t i = first; i < x->in.size(); ++i) B200_TRY(EnsureMaterialized(x->in[i]));
    k::DynSliceParams dp;
    dp.elt_size = dtype_size(x->dtype);
    dp.rank = operand->rank();
    for (int d = 0; d < dp.rank; ++d) {
      dp.x_dims[d] = operand->dims[d];
      dp.b_dims[d] = update ? upd->dims[d] : x->dims[d];
      dp.start_dtypes[d] = x->in[first + d]->dtype;
    }
    std::vector<int> start_slots;
    for (size_t i = first; i < x->in.size(); ++i) start_slots.push_back(SlotOf(x->in[i]));
    const int x_slot = SlotOf(operand), u_slot = upd ? SlotOf(upd_src ? upd_src : upd) : -1, out_slot = NewValueSlot(x);
    const int64_t u_byte_off = upd_off * dtype_size(x->dtype);
    if (upd_src) {
      dp.u_strided = true;
      for (int d = 0; d < dp.rank; ++d) dp.u_strides[d] = upd_strides[d];
    }
    Step st;
    st.desc = strfmt("move[%s rank=%d%s]", update ? "DynamicUpdateSlice" : "DynamicSlice", dp.rank, upd_src ? " update read in place" : "");
    st.reads = start_slots;
    st.reads.push_back(x_slot);
    if (upd) st.reads.push_back(u_slot);
    st.writes = {out_slot};
    // DynamicUpdateSlice straight from a placeholder into an output, the placeholder feeding nothing else: when the caller
    // donates that input, execute binds the output to the input's memory and this step only writes the block.
    if (update && operand->op == Op::Parameter && uses_[operand->id] == 1 && ex_->slots[out_slot].kind == SlotKind::Output &&
        ex_->slots[x_slot].kind == SlotKind::Input) {
      if (ex_->donate_alias.size() <= (size_t)ex_->slots[out_slot].index) ex_->donate_alias.resize(ex_->slots[out_slot].index + 1, -1);
      ex_->donate_alias[ex_->slots[out_slot].index] = ex_->slots[x_slot].index;
    }
    auto bind = [dp, start_slots, x_slot, u_slot, out_slot, u_byte_off](void* const* p) {
      k::DynSliceParams q = dp;
      q.x = p[x_slot];
      q.u = u_slot >= 0 ? (const char*)p[u_slot] + u_byte_off : nullptr;
      q.y = p[out_slot];
      for (size_t i = 0; i < start_slots.size(); ++i) q.starts[i] = p[start_slots[i]];
      return q;
    };
    auto run_one = [update](Device* dev, const k::DynSliceParams& q) -> Status {
      if (update && q.x == q.y) return k::dynamic_update_slice_inplace(dev, q);
      return update ? k::dynamic_update_slice(dev, q) : k::dynamic_slice(dev, q);
    };
    // A second update with the same start indices and block geometry right after the first (a layer's key cache, then its
    // value cache): one step, and one launch when both turn out to be in place.
    // (never an update OF the first one's result or FROM it: the two run side by side)
    if (update && last_dus_.step == (int)ex_->steps.size() - 1 && last_dus_.step >= 0 && last_dus_.start_slots == start_slots &&
        last_dus_.rank == dp.rank && last_dus_.elt_size == dp.elt_size && x_slot != last_dus_.out_slot && u_slot != last_dus_.out_slot &&
        out_slot != last_dus_.out_slot && x_slot != last_dus_.x_slot &&
        std::equal(dp.x_dims, dp.x_dims + dp.rank, last_dus_.x_dims) && std::equal(dp.b_dims, dp.b_dims + dp.rank, last_dus_.b_dims)) {
      Step& prev = ex_->steps.back();
      prev.desc.insert(prev.desc.size() - 1, upd_src ? " + a second one, read in place" : " + a second one");
      prev.reads.insert(prev.reads.end(), st.reads.begin(), st.reads.end());
      prev.writes.push_back(out_slot);
      auto first = last_dus_.bind;
      prev.run = [first, bind, run_one](Device* dev, void* const* p) -> Status {
        const k::DynSliceParams q0 = first(p), q1 = bind(p);
        if (q0.x == q0.y && q1.x == q1.y) return k::dynamic_update_slice_inplace2(dev, q0, q1);
        B200_TRY(run_one(dev, q0));
        return run_one(dev, q1);
      };
      last_dus_.step = -1;   // pairs only
      return Status::OK();
    }
    st.run = [bind, run_one](Device* dev, void* const* p) -> Status { return run_one(dev, bind(p)); };
    ex_->steps.push_back(std::move(st));
    if (update) {
      last_dus_.step = (int)ex_->steps.size() - 1;
      last_dus_.start_slots = start_slots;
      last_dus_.rank = dp.rank;
      last_dus_.elt_size = dp.elt_size;
      last_dus_.out_slot = out_slot;
      last_dus_.x_slot = x_slot;
      std::copy(dp.x_dims, dp.x_dims + k::kMaxDims, last_dus_.x_dims);
      std::copy(dp.b_dims, dp.b_dims + k::kMaxDims, last_dus_.b_dims);
      last_dus_.bind = bind;
    }
    return Status::OK();
  }

  Status EmitPad(Node* x) {
    if (x->rank() > k::kMaxDims) return Status::Unsupported("compile: more than 8 dims");
    Node* src = x->in[0];
    Node* pv = x->in[1];
    B200_TRY(EnsureMaterialized(src));
    B200_TRY(EnsureMaterialized(pv));
    const int out_slot = NewValueSlot(x);
    const int pv_slot = SlotOf(pv);
    {
      // fill = broadcast of the one-element pad value
      k::StridedCopyParams p;
      p.elt_size = dtype_size(x->dtype);
      p.rank = 1;
      p.dims[0] = x->num_elements();
      p.in_strides[0] = 0;
      p.out_strides[0] = 1;
      Step st;
      st.desc = "move[Pad fill]";
      st.reads = {pv_slot};
      st.writes = {out_slot};
      st.run = [p, pv_slot, out_slot](Device* dev, void* const* ptrs) -> Status {
        k::StridedCopyParams q = p;
        q.x = ptrs[pv_slot];
        q.y = ptrs[out_slot];
        return k::strided_copy(dev, q);
      };
      ex_->steps.push_back(std::move(st));
    }
    std::vector<int64_t> start(x->ia.begin(), x->ia.end());
    EmitBlockCopy(src, out_slot, x->dims, start, "Pad body");
    ex_->steps.back().reads.push_back(out_slot);  // ordered after the fill
    return Status::OK();
  }

  // Makes a dense copy of `src` permuted by `perm` into a temp slot; returns the slot.
  int EmitPermutedTemp(Node* src, const std::vector<int>& perm, const char* what) {
    k::StridedCopyParams p;
    p.elt_size = dtype_size(src->dtype);
    p.rank = src->rank();
    const std::vector<int64_t> cs = dense_strides(src->dims);
    std::vector<int64_t> od(src->rank());
    for (int d = 0; d < src->rank(); ++d) od[d] = src->dims[perm[d]];
    const std::vector<int64_t> os = dense_strides(od);
    for (int d = 0; d < src->rank(); ++d) { p.dims[d] = od[d]; p.in_strides[d] = cs[perm[d]]; p.out_strides[d] = os[d]; }
    const int in_slot = SlotOf(src);
    const int tmp = NewTemp(src->num_elements() * dtype_size(src->dtype));
    Step st;
    st.desc = std::string("move[") + what + "]";
    st.reads = {in_slot};
    st.writes = {tmp};
    st.run = [p, in_slot, tmp](Device* dev, void* const* ptrs) -> Status {
      k::StridedCopyParams q = p;
      q.x = ptrs[in_slot];
      q.y = ptrs[tmp];
      return k::strided_copy(dev, q);
    };
    ex_->steps.push_back(std::move(st));
    return tmp;
  }

  // ------------------------------------------------------------ DotGeneral ---
  // Decides whether an operand, as it lies in memory, is [batch, free, contract]
  // (K-major) or [batch, contract, free] (MN-major) with the batch and
  // contracting axes in the required order.  Returns 1, 0, or -1 (needs a copy).
  static int OperandMajor(Node* t, const std::vector<int64_t>& batch, const std::vector<int64_t>& contract) {
    const int r = t->rank();
    std::vector<int> role(r, 0);  // 0 free, 1 batch, 2 contracting
    for (auto a : batch) role[a] = 1;
    for (auto a : contract) role[a] = 2;
    // size-1 axes can sit anywhere; ignore them when reading the order
    std::vector<int> order;
    for (int i = 0; i < r; ++i)
      if (t->dims[i] != 1) {
        if (order.empty() || order.back() != role[i]) order.push_back(role[i]);
      }
    auto ascending = [&](const std::vector<int64_t>& axes) {
      int64_t prev = -1;
      for (auto a : axes) {
        if (t->dims[a] == 1) continue;
        if (a < prev) return false;
        prev = a;
      }
      return true;
    };
    if (!ascending(batch) || !ascending(contract)) return -1;
    // strip a leading batch group
    size_t i = 0;
    if (i < order.size() && order[i] == 1) ++i;
    std::vector<int> rest(order.begin() + i, order.end());
    for (int v : rest)
      if (v == 1) return -1;  // batch axes not leading
    if (rest.empty()) return 1;
    if (rest.size() == 1) return 1;  // only free or only contracting: either reading works; call it K-major
    if (rest.size() == 2) return (rest[0] == 0 && rest[1] == 2) ? 1 : ((rest[0] == 2 && rest[1] == 0) ? 0 : -1);
    return -1;
  }

  std::vector<bool> rms_deferred_;   // RMSNorm nodes left to their consumers (see the emission loop)

  Status EmitDotGeneral(Node* x) {
    Node* a = x->in[0];
    Node* b = x->in[1];
    // the left operand is an RMSNorm that nobody has asked for yet: candidate for the norm applied inside the product
    Node* rms = nullptr;
    if (Node* ab = ViewBase(a); ab->op == Op::RmsNorm && (size_t)ab->id < rms_deferred_.size() && rms_deferred_[ab->id] && slot_of_[ab->id] < 0) rms = ab;
    // inputs: lhs, rhs, [bias], [residual]; fa = {activation, has_residual (set by the compile-time rewrite)}
    const bool has_residual = x->fa.size() > 1 && x->fa[1] != 0;
    Node* residual = has_residual ? x->in.back() : nullptr;
    Node* bias = (int)x->in.size() - (has_residual ? 1 : 0) > 2 ? x->in[2] : nullptr;
    if (!rms) B200_TRY(EnsureMaterialized(a));
    B200_TRY(EnsureMaterialized(b));
    if (bias) B200_TRY(EnsureMaterialized(bias));
    // act(a W1) * (a W2), the second product a plain DotGeneral of the same operand that feeds nothing else (a gated MLP):
    // candidate for ONE launch with two weights when the shape is the few-rows kernel's (decided below)
    Node* dual_w2 = nullptr;
    if (residual && GatedSecondProduct(x) == residual && slot_of_[residual->id] < 0) dual_w2 = residual->in[1];
    const int nc = (int)x->ia[0], nb = (int)x->ia[1];
    std::vector<int64_t> lc(x->ia.begin() + 2, x->ia.begin() + 2 + nc);
    std::vector<int64_t> lb(x->ia.begin() + 2 + nc, x->ia.begin() + 2 + nc + nb);
    std::vector<int64_t> rc(x->ia.begin() + 2 + nc + nb, x->ia.begin() + 2 + 2 * nc + nb);
    std::vector<int64_t> rb(x->ia.begin() + 2 + 2 * nc + nb, x->ia.begin() + 2 + 2 * nc + 2 * nb);
    int64_t B = 1, K = 1;
    for (auto ax : lb) B *= a->dims[ax];
    for (auto ax : lc) K *= a->dims[ax];
    const int64_t M = (B * K) ? a->num_elements() / (B * K) : 0;
    const int64_t N = (B * K) ? b->num_elements() / (B * K) : 0;
    int a_major = OperandMajor(a, lb, lc);
    int b_major = OperandMajor(b, rb, rc);  // 1: [B,N,K]; 0: [B,K,N]
    if (rms) {
      k::GemmParams probe;
      probe.batch = B; probe.m = M; probe.n = N; probe.k = K;
      probe.a_k_major = a_major == 1; probe.b_k_major = b_major != 0; probe.dtype = x->dtype;
      const bool last_axis_only = lc.size() == 1 && lc[0] == a->rank() - 1 && K == rms->dims.back() && lb.empty();
      // (not into a product that streams a large weight through every CTA's whole K, such as an LM head: the norm's extra
      // work per k-step sits on that kernel's critical path -- 128256 x 2048: 128 us against 107 -- and saves one launch)
      if (!last_axis_only || a_major != 1 || b_major != 0 || !k::gemm_skinny_dual_ok(probe) || N * K > (64LL << 20)) {
        rms = nullptr;
        B200_TRY(EnsureMaterialized(a));   // the norm on its own after all
      } else {
        B200_TRY(EnsureMaterialized(rms->in[0]));
        B200_TRY(EnsureMaterialized(rms->in[1]));
      }
    }
    if (dual_w2) {
      k::GemmParams probe;
      probe.batch = B; probe.m = M; probe.n = N; probe.k = K;
      probe.a_k_major = a_major == 1; probe.b_k_major = b_major != 0; probe.dtype = x->dtype;
      if (a_major != 1 || b_major != 0 || OperandMajor(dual_w2, rb, rc) != 0 || !k::gemm_skinny_dual_ok(probe)) dual_w2 = nullptr;
    }
    if (dual_w2) {
      B200_TRY(EnsureMaterialized(dual_w2));
      residual = nullptr;   // never computed on its own
    } else if (residual) {
      B200_TRY(EnsureMaterialized(residual));
    }
    // With several contracting (or batch) axes both sides must walk them in the same order.
    auto same_order = [](Node* t1, const std::vector<int64_t>& ax1, Node* t2, const std::vector<int64_t>& ax2) {
      std::vector<size_t> idx;
      for (size_t i = 0; i < ax1.size(); ++i)
        if (t1->dims[ax1[i]] != 1) idx.push_back(i);
      for (size_t i = 1; i < idx.size(); ++i)
        if ((ax1[idx[i]] > ax1[idx[i - 1]]) != (ax2[idx[i]] > ax2[idx[i - 1]])) return false;
      return true;
    };
    if (!same_order(a, lc, b, rc) || !same_order(a, lb, b, rb)) b_major = -1;
    int a_slot = rms ? SlotOf(rms->in[0]) : SlotOf(a), b_slot = SlotOf(b);
    auto canonical = [&](Node* t, const std::vector<int64_t>& batch, const std::vector<int64_t>& contract) {
      std::vector<int> perm;
      std::vector<bool> used(t->rank(), false);
      for (auto ax : batch) { perm.push_back((int)ax); used[ax] = true; }
      for (auto ax : contract) used[ax] = true;
      for (int i = 0; i < t->rank(); ++i)
        if (!used[i]) perm.push_back(i);
      for (auto ax : contract) perm.push_back((int)ax);
      return perm;
    };
    if (a_major < 0) {
      if (a->rank() > k::kMaxDims) return Status::Unsupported("DotGeneral: more than 8 dims");
      a_slot = EmitPermutedTemp(a, canonical(a, lb, lc), "DotGeneral lhs -> [B,M,K]");
      a_major = 1;
    }
    if (b_major < 0) {
      if (b->rank() > k::kMaxDims) return Status::Unsupported("DotGeneral: more than 8 dims");
      b_slot = EmitPermutedTemp(b, canonical(b, rb, rc), "DotGeneral rhs -> [B,N,K]");
      b_major = 1;
    }
    const int out_slot = NewValueSlot(x);
    // A large result whose rows are not a whole number of 16-byte vectors (GPT-2's 50257-column logits): the GEMM writes
    // it with a padded row pitch, where its epilogue can use full-line vector stores, and one packing pass makes it
    // dense.  Writing the ragged rows straight from the epilogue splits every 32-byte sector between two stores and
    // measured 2.2x slower than GEMM + packing pass.
    const int64_t es_out = dtype_size(x->dtype);
    const int64_t vec_out = 16 / es_out;
    const bool float_out = x->dtype == B200_FLOAT32 || x->dtype == B200_BFLOAT16 || x->dtype == B200_FLOAT16;
    k::GemmParams gp;
    gp.batch = B; gp.m = M; gp.n = N; gp.k = K;
    gp.a_k_major = a_major == 1;
    gp.b_k_major = b_major == 1;
    gp.dtype = x->dtype;
    // ... unless the tensor-core kernel can write the ragged rows with aligned vectors itself (row classes: both operands
    // K-major, M a multiple of 8, nothing fused)
    const bool ragged_direct = k::gemm_tcgen05_ragged_rows(gp, bias != nullptr, residual != nullptr);
    const bool pad_rows = float_out && !residual && !ragged_direct && N % vec_out != 0 && B * M * N * es_out >= (int64_t)(8 << 20);
    const int64_t ldc = pad_rows ? (N + vec_out - 1) / vec_out * vec_out : 0;
    const int gemm_out = pad_rows ? NewTemp(B * M * ldc * es_out + 16) : out_slot;
    gp.ldc = ldc;
    gp.activation = (int)x->fa[0];
    gp.residual_op = (has_residual && x->fa[1] == 2.0 && !dual_w2) ? 1 : 0;
    const int bias_slot = bias ? SlotOf(bias) : -1;
    const int res_slot = residual ? SlotOf(residual) : -1;
    Step st;
    st.desc = strfmt("gemm[B=%lld M=%lld N=%lld K=%lld %s a:%s b:%s%s%s act=%d]", (long long)B, (long long)M, (long long)N, (long long)K,
                     dtype_name(x->dtype), gp.a_k_major ? "MK" : "KM", gp.b_k_major ? "NK" : "KN", bias ? " bias" : "",
                     dual_w2 ? " *second-product" : (residual ? (gp.residual_op ? " *residual" : " +residual") : ""), gp.activation);
    if (ragged_direct && k::gemm_skinny_scratch_bytes(gp, ex_->dev->sm_count()) == 0) st.desc.insert(st.desc.size() - 1, " ragged-rows");
    st.reads = {a_slot, b_slot};
    if (bias) st.reads.push_back(bias_slot);
    if (residual) st.reads.push_back(res_slot);
    // two weights in one launch; should the kernel decline at run time (an unaligned buffer), the two products run one
    // after the other through a small temporary
    const int gamma_slot = rms ? SlotOf(rms->in[1]) : -1;
    const int rms_tmp = rms ? NewTemp(M * K * es_out + 16) : -1;
    const double rms_eps = rms ? rms->fa[0] : 0.0;
    if (rms) {
      st.reads.push_back(gamma_slot);
      st.writes.push_back(rms_tmp);
      st.desc.insert(st.desc.size() - 1, " of-rms-norm");
    }
    const int w2_slot = dual_w2 ? SlotOf(dual_w2) : -1;
    const int dual_tmp = dual_w2 ? NewTemp(B * M * N * es_out + 16) : -1;
    if (dual_w2) {
      st.reads.push_back(w2_slot);
      st.writes.push_back(dual_tmp);
    }
    st.writes.insert(st.writes.begin(), gemm_out);
    // fp32 on the tensor cores splits both operands into bf16 planes: their room comes from the plan's arena, so the step
    // allocates nothing and can be recorded
    // A 16-bit product of a handful of rows splits K over many CTAs: fp32 partial sums in the arena and a few counters
    // of the step's own (zeroed once; the kernel leaves them at zero).
    // weights that are an input or a constant of this plan: nothing this plan launches writes them (an input that a
    // DynamicUpdateSlice updates in place feeds nothing else)
    auto never_written = [&](int slot) { return ex_->slots[slot].kind == SlotKind::Input || ex_->slots[slot].kind == SlotKind::Const; };
    gp.b_static = never_written(b_slot) && (w2_slot < 0 || never_written(w2_slot));   // (a gated pair: both weights)
    const int64_t skinny_bytes = k::gemm_skinny_scratch_bytes(gp, ex_->dev->sm_count());
    const int64_t split_bytes = x->dtype == B200_FLOAT32 ? k::gemm_split_scratch_bytes(B, M, N, K) : skinny_bytes;
    const int split_slot = split_bytes > 0 ? NewTemp(split_bytes) : -1;
    if (split_slot >= 0) st.writes.push_back(split_slot);
    int counter_slot = -1;
    if (skinny_bytes > 0) {
      B200_TRY(NewZeroedConst(k::gemm_skinny_counter_bytes(gp), &counter_slot));
      st.desc.insert(st.desc.size() - 1, " few-rows");
    }
    st.run = [gp, a_slot, b_slot, bias_slot, res_slot, gemm_out, split_slot, split_bytes, counter_slot, w2_slot, dual_tmp, gamma_slot, rms_tmp,
              rms_eps](Device* dev, void* const* p) -> Status {
      k::GemmParams q = gp;
      if (split_slot >= 0) { q.split_scratch = p[split_slot]; q.split_scratch_bytes = split_bytes; }
      if (counter_slot >= 0) q.skinny_counters = p[counter_slot];
      q.a = p[a_slot];
      q.b = p[b_slot];
      q.c = p[gemm_out];
      q.bias = bias_slot >= 0 ? p[bias_slot] : nullptr;
      q.residual = res_slot >= 0 ? p[res_slot] : nullptr;
      if (w2_slot >= 0 || gamma_slot >= 0) {
        if (w2_slot >= 0) q.b2 = p[w2_slot];
        if (gamma_slot >= 0) { q.rms_gamma = p[gamma_slot]; q.rms_eps = rms_eps; }
        bool taken = false;
        B200_TRY(k::gemm_skinny(dev, q, &taken));
        if (taken) return Status::OK();
        if (gamma_slot >= 0) {   // the norm on its own into the temporary, then the product of that
          k::NormParams np;
          np.x = p[a_slot]; np.gamma = p[gamma_slot]; np.y = p[rms_tmp];
          np.rows = gp.m; np.cols = gp.k; np.dtype = gp.dtype; np.epsilon = rms_eps; np.rms = true;
          B200_TRY(k::norm_rows(dev, np));
          q.a = p[rms_tmp];
          q.rms_gamma = nullptr;
        }
        if (w2_slot < 0) return k::gemm(dev, q);
        k::GemmParams second = q;   // X W2 on its own ...
        second.b = p[w2_slot]; second.b2 = nullptr; second.c = p[dual_tmp]; second.bias = nullptr; second.activation = B200_ACT_NONE;
        B200_TRY(k::gemm(dev, second));
        q.b2 = nullptr;             // ... then act(X W + bias) times it
        q.residual = p[dual_tmp];
        q.residual_op = 1;
      }
      return k::gemm(dev, q);
    };
    ex_->steps.push_back(std::move(st));
    if (pad_rows) {
      Step up;
      up.desc = strfmt("move[pack rows=%lld cols=%lld pitch=%lld]", (long long)(B * M), (long long)N, (long long)ldc);
      up.reads = {gemm_out};
      up.writes = {out_slot};
      const int64_t rows = B * M;
      const int es_i = (int)es_out;
      up.run = [gemm_out, out_slot, rows, N, ldc, es_i](Device* dev, void* const* p) -> Status {
        return k::unpad_rows(dev, p[gemm_out], p[out_slot], rows, N, ldc, es_i);
      };
      ex_->steps.push_back(std::move(up));
    }
    return Status::OK();
  }

  // ------------------------------------------------------------ reductions ---
  // A reduction over ONE run of neighbouring axes whose operand is an elementwise chain (or a plain tensor): the chain
  // is evaluated inside the reduction kernel, which is compiled at plan time, so the chain's value never goes to memory
  // and the operand is read with 128-bit loads.  Sets *done when the step was emitted; otherwise nothing has changed and
  // the caller materialises the operand and uses the precompiled reduction kernels.
  Status TryEmitFusedReduce(Node* x, int rt, int lo, int hi, bool* done) {
    *done = false;
    Node* src = x->in[0];
    if (src->rank() > k::kMaxDims || src->rank() == 0) return Status::OK();
    std::string why;
    if (!k::ewise_jit_available(&why)) return Status::OK();
    int64_t outer = 1, n = 1, inner = 1;
    for (int d = 0; d < lo; ++d) outer *= src->dims[d];
    for (int d = lo; d <= hi; ++d) n *= src->dims[d];
    for (int d = hi + 1; d < src->rank(); ++d) inner *= src->dims[d];
    if (outer * n * inner == 0 || !k::ewise_jit_reduce_fits(outer, n, inner, ex_->dev->sm_count())) return Status::OK();
    for (int budget = 24; budget >= 1; budget /= 2) {
      EwBuild b;
      b.op_budget = budget;
      b.dim_used_by_iota.assign(src->rank() + 1, false);
      b.prog.rank = src->rank();
      for (int d = 0; d < src->rank(); ++d) b.prog.dims[d] = src->dims[d];
      int root = 0;
      B200_TRY(BuildExpr(b, src, IndexMap::Identity(src->rank()), &root));
      if (b.overflow) continue;
      if (!AssignRegisters(b, root)) continue;
      k::EwProgram prog = b.prog;
      prog.out_dtype = src->dtype;
      prog.wide = dtype_size(src->dtype) == 8;
      for (int i = 0; i < prog.num_instr; ++i)
        if (dtype_size(prog.instr[i].dtype) == 8 || dtype_size(prog.instr[i].sdtype) == 8) prog.wide = true;
      CollapseProgram(b, prog, {lo, hi + 1});
      k::EwJit* jit = nullptr;
      if (!k::ewise_jit_reduce_prepare(ex_->dev, prog, rt, outer, n, inner, &jit).ok() || !jit) return Status::OK();
      const int out_slot = NewValueSlot(x);
      Step st;
      st.desc = strfmt("reduce[type=%d outer=%lld n=%lld inner=%lld %s fused instr=%d leaves=%d compiled]", rt, (long long)outer, (long long)n,
                       (long long)inner, dtype_name(src->dtype), prog.num_instr, prog.num_leaves);
      st.reads = b.leaf_slots;
      st.writes = {out_slot};
      std::vector<int> leaf_slots = b.leaf_slots;
      std::vector<int64_t> leaf_offsets = b.leaf_offsets;
      st.run = [prog, leaf_slots, leaf_offsets, out_slot, jit](Device* dev, void* const* p) -> Status {
        k::EwProgram q = prog;
        for (int l = 0; l < q.num_leaves; ++l)
          q.leaves[l].ptr = (const char*)p[leaf_slots[l]] + leaf_offsets[l] * dtype_size(q.leaves[l].dtype);
        q.out = p[out_slot];
        return k::ewise_jit_run(dev, jit, q);
      };
      ex_->steps.push_back(std::move(st));
      *done = true;
      return Status::OK();
    }
    return Status::OK();
  }

  Status EmitReduce(Node* x) {
    Node* src = x->in[0];
    const int rt = (int)x->ia[0];
    std::vector<int64_t> axes(x->ia.begin() + 1, x->ia.end());
    std::sort(axes.begin(), axes.end());
    {
      bool one_run = !axes.empty();
      for (size_t i = 1; i < axes.size(); ++i) one_run = one_run && axes[i] == axes[i - 1] + 1;
      if (one_run) {
        bool done = false;
        B200_TRY(TryEmitFusedReduce(x, rt, (int)axes.front(), (int)axes.back(), &done));
        if (done) return Status::OK();
      }
    }
    B200_TRY(EnsureMaterialized(src));
    // Runs of neighbouring reduced axes, folded from the innermost run outwards.
    struct Run { int lo, hi; };
    std::vector<Run> runs;
    for (auto ax : axes) {
      if (!runs.empty() && runs.back().hi + 1 == (int)ax) runs.back().hi = (int)ax;
      else runs.push_back(Run{(int)ax, (int)ax});
    }
    std::vector<int64_t> cur = src->dims;
    int cur_slot = SlotOf(src);
    if (runs.empty()) {
      // nothing to reduce (rank-0 operand): copy through
      const int out_slot = NewValueSlot(x);
      const int64_t nbytes = x->num_elements() * dtype_size(x->dtype);
      Step st;
      st.desc = "copy[Reduce of scalar]";
      st.reads = {cur_slot};
      st.writes = {out_slot};
      st.launches = 0;
      st.run = [=](Device* dev, void* const* p) -> Status {
        B200_CUDA_TRY(cudaMemcpyAsync(p[out_slot], p[cur_slot], (size_t)nbytes, cudaMemcpyDeviceToDevice, dev->stream()));
        return Status::OK();
      };
      ex_->steps.push_back(std::move(st));
      return Status::OK();
    }
    for (int ri = (int)runs.size() - 1; ri >= 0; --ri) {
      int64_t outer = 1, n = 1, inner = 1;
      for (int d = 0; d < runs[ri].lo; ++d) outer *= cur[d];
      for (int d = runs[ri].lo; d <= runs[ri].hi; ++d) n *= cur[d];
      for (int d = runs[ri].hi + 1; d < (int)cur.size(); ++d) inner *= cur[d];
      const bool last = ri == 0;
      const int64_t out_bytes = outer * inner * dtype_size(x->dtype);
      const int out_slot = last ? NewValueSlot(x) : NewTemp(out_bytes);
      const int64_t sb = k::reduce_scratch_bytes(x->dtype, outer, n, inner);
      const int scratch_slot = sb > 0 ? NewTemp(sb) : -1;
      const int in_slot = cur_slot, dt = x->dtype;
      Step st;
      st.desc = strfmt("reduce[type=%d outer=%lld n=%lld inner=%lld %s%s]", rt, (long long)outer, (long long)n, (long long)inner,
                       dtype_name(dt), sb > 0 ? " split" : "");
      st.reads = {in_slot};
      st.writes = {out_slot};
      if (scratch_slot >= 0) st.writes.push_back(scratch_slot);
      st.launches = sb > 0 ? 2 : 1;
      st.run = [=](Device* dev, void* const* p) -> Status {
        return k::reduce(dev, p[in_slot], p[out_slot], dt, rt, outer, n, inner, scratch_slot >= 0 ? p[scratch_slot] : nullptr, sb);
      };
      ex_->steps.push_back(std::move(st));
      cur.erase(cur.begin() + runs[ri].lo, cur.begin() + runs[ri].hi + 1);
      cur_slot = out_slot;
    }
    return Status::OK();
  }

  Status EmitArgMinMax(Node* x) {
    Node* src = x->in[0];
    B200_TRY(EnsureMaterialized(src));
    const int ax = (int)x->ia[0];
    const bool is_min = x->ia[1] != 0;
    int64_t outer = 1, inner = 1;
    for (int d = 0; d < ax; ++d) outer *= src->dims[d];
    for (int d = ax + 1; d < src->rank(); ++d) inner *= src->dims[d];
    const int64_t n = src->dims[ax];
    const int in_slot = SlotOf(src), out_slot = NewValueSlot(x);
    const int dt = src->dtype, odt = x->dtype;
    Step st;
    st.desc = strfmt("arg%s[outer=%lld n=%lld inner=%lld %s -> %s]", is_min ? "min" : "max", (long long)outer, (long long)n,
                     (long long)inner, dtype_name(dt), dtype_name(odt));
    st.reads = {in_slot};
    st.writes = {out_slot};
    st.run = [=](Device* dev, void* const* p) -> Status { return k::arg_min_max(dev, p[in_slot], p[out_slot], dt, odt, is_min, outer, n, inner); };
    ex_->steps.push_back(std::move(st));
    return Status::OK();
  }

  // ---------------------------------------------------------------- gather ---
  Status EmitGather(Node* x) {
    Node* op = x->in[0];
    Node* idx = x->in[1];
    B200_TRY(EnsureMaterialized(op));
    B200_TRY(EnsureMaterialized(idx));
    size_t pos = 0;
    const int iva = (int)x->ia[pos++];
    auto take = [&]() { const int n = (int)x->ia[pos++]; std::vector<int64_t> v(x->ia.begin() + pos, x->ia.begin() + pos + n); pos += n; return v; };
    const std::vector<int64_t> off_axes = take(), collapsed = take(), sim = take(), ss = take();
    const int orank = op->rank(), irank = idx->rank();
    if (orank > k::kMaxDims || x->rank() > k::kMaxDims || irank > k::kMaxDims) return Status::Unsupported("Gather: more than 8 dims");
    const int op_slot = SlotOf(op), idx_slot = SlotOf(idx), out_slot = NewValueSlot(x);
    const int es = dtype_size(op->dtype), idt = idx->dtype;
    // Fast path: whole rows of the leading axis (embedding lookup; ref gather.go:61-91).
    bool rows = sim.size() == 1 && sim[0] == 0 && collapsed.size() == 1 && collapsed[0] == 0 && ss[0] == 1 &&
                (iva == irank || iva == irank - 1);
    for (int d = 1; d < orank && rows; ++d) rows = ss[d] == op->dims[d];
    const int batch_rank = iva == irank ? irank : irank - 1;
    for (size_t i = 0; i < off_axes.size() && rows; ++i) rows = off_axes[i] == (int64_t)(batch_rank + i);
    int64_t row_bytes = es;
    for (int d = 1; d < orank; ++d) row_bytes *= op->dims[d];
    rows = rows && (row_bytes % 16 == 0) && orank >= 1;
    if (rows) {
      const int64_t num_ids = idx->num_elements(), num_rows = op->dims[0];
      Step st;
      st.desc = strfmt("gather_rows[ids=%lld rows=%lld row_bytes=%lld]", (long long)num_ids, (long long)num_rows, (long long)row_bytes);
      st.reads = {op_slot, idx_slot};
      st.writes = {out_slot};
      st.run = [=](Device* dev, void* const* p) -> Status { return k::gather_rows(dev, p[op_slot], p[idx_slot], idt, p[out_slot], num_ids, num_rows, row_bytes); };
      ex_->steps.push_back(std::move(st));
      return Status::OK();
    }
    k::GatherParams gp;
    gp.elt_size = es;
    gp.ids_dtype = idt;
    gp.out_rank = x->rank();
    gp.operand_rank = orank;
    const std::vector<int64_t> ostr = dense_strides(op->dims), istr = dense_strides(idx->dims);
    for (int d = 0; d < orank; ++d) { gp.operand_dims[d] = op->dims[d]; gp.operand_strides[d] = ostr[d]; gp.slice_sizes[d] = ss[d]; }
    std::vector<int> offset_operand_axes;  // non-collapsed operand axes in order
    for (int d = 0; d < orank; ++d)
      if (!std::count(collapsed.begin(), collapsed.end(), (int64_t)d)) offset_operand_axes.push_back(d);
    int bpos = 0;
    for (int d = 0; d < x->rank(); ++d) {
      gp.out_dims[d] = x->dims[d];
      auto it = std::find(off_axes.begin(), off_axes.end(), (int64_t)d);
      if (it != off_axes.end()) { gp.out_offset_operand_axis[d] = offset_operand_axes[it - off_axes.begin()]; gp.out_batch_pos[d] = -1; }
      else { gp.out_offset_operand_axis[d] = -1; gp.out_batch_pos[d] = bpos++; }
    }
    gp.num_batch_dims = bpos;
    int bi = 0;
    for (int d = 0; d < irank; ++d)
      if (d != iva) gp.batch_index_strides[bi++] = istr[d];
    gp.index_vector_stride = iva < irank ? istr[iva] : 0;
    gp.num_index_components = (int)sim.size();
    for (size_t i = 0; i < sim.size(); ++i) gp.start_index_map[i] = (int)sim[i];
    Step st;
    st.desc = "gather_general";
    st.reads = {op_slot, idx_slot};
    st.writes = {out_slot};
    st.run = [gp, op_slot, idx_slot, out_slot](Device* dev, void* const* p) -> Status {
      k::GatherParams q = gp;
      q.operand = p[op_slot];
      q.indices = p[idx_slot];
      q.y = p[out_slot];
      return k::gather_general(dev, q);
    };
    ex_->steps.push_back(std::move(st));
    return Status::OK();
  }

  // ------------------------------------------------- scatter, random bits ---
  Status EmitScatter(Node* x) {
    Node* op = x->in[0];
    Node* idx = x->in[1];
    Node* upd = x->in[2];
    B200_TRY(EnsureMaterialized(op));
    B200_TRY(EnsureMaterialized(idx));
    B200_TRY(EnsureMaterialized(upd));
    size_t pos = 0;
    const int mode = (int)x->ia[pos++], iva = (int)x->ia[pos++];
    pos++;  // unique_indices: the atomics are correct either way
    auto take = [&]() { const int n = (int)x->ia[pos++]; std::vector<int64_t> v(x->ia.begin() + pos, x->ia.begin() + pos + n); pos += n; return v; };
    const std::vector<int64_t> uw = take(), iw = take(), map = take();
    const int orank = op->rank(), irank = idx->rank(), urank = upd->rank();
    const int op_slot = SlotOf(op), idx_slot = SlotOf(idx), upd_slot = SlotOf(upd), out_slot = NewValueSlot(x);
    k::ScatterParams sp;
    sp.dtype = op->dtype;
    sp.ids_dtype = idx->dtype;
    sp.mode = mode;
    sp.operand_rank = orank;
    sp.update_rank = urank;
    const std::vector<int64_t> ostr = dense_strides(op->dims), istr = dense_strides(idx->dims);
    for (int d = 0; d < orank; ++d) { sp.operand_dims[d] = op->dims[d]; sp.operand_strides[d] = ostr[d]; }
    for (int d = 0; d < urank; ++d) sp.update_dims[d] = upd->dims[d];
    int nb = 0;
    for (int d = 0; d < urank; ++d)
      if (!std::count(uw.begin(), uw.end(), (int64_t)d)) sp.batch_update_axis[nb++] = d;
    sp.num_batch_dims = nb;
    int bi = 0;
    for (int d = 0; d < irank; ++d)
      if (d != iva) sp.batch_index_strides[bi++] = istr[d];
    sp.index_vector_stride = iva < irank ? istr[iva] : 0;
    sp.num_index_components = (int)map.size();
    for (size_t i = 0; i < map.size(); ++i) sp.scatter_axes_to_operand_axes[i] = (int)map[i];
    int nw = 0;
    for (int d = 0; d < orank; ++d)
      if (!std::count(iw.begin(), iw.end(), (int64_t)d)) {
        sp.window_operand_axis[nw] = d;
        sp.window_update_axis[nw] = (int)uw[nw];
        ++nw;
      }
    sp.num_window_axes = nw;
    const int64_t nbytes = x->num_elements() * dtype_size(x->dtype);
    Step st;
    st.desc = strfmt("scatter[mode=%d operand=%lld updates=%lld %s]", mode, (long long)op->num_elements(), (long long)upd->num_elements(),
                     dtype_name(op->dtype));
    st.reads = {op_slot, idx_slot, upd_slot};
    st.writes = {out_slot};
    st.launches = 1;
    st.run = [sp, op_slot, idx_slot, upd_slot, out_slot, nbytes](Device* dev, void* const* p) -> Status {
      if (nbytes > 0 && p[out_slot] != p[op_slot])
        B200_CUDA_TRY(cudaMemcpyAsync(p[out_slot], p[op_slot], (size_t)nbytes, cudaMemcpyDeviceToDevice, dev->stream()));
      k::ScatterParams q = sp;
      q.y = p[out_slot];
      q.indices = p[idx_slot];
      q.updates = p[upd_slot];
      return k::scatter(dev, q);
    };
    ex_->steps.push_back(std::move(st));
    return Status::OK();
  }

  // The stable sorting permutation of in[0] along ia[0] (ia[1]: descending), int32.
  Status EmitArgSort(Node* x) {
    Node* a = x->in[0];
    B200_TRY(EnsureMaterialized(a));
    const int axis = (int)x->ia[0];
    const bool descending = x->ia[1] != 0;
    int64_t outer = 1, inner = 1;
    for (int i = 0; i < axis; ++i) outer *= a->dims[i];
    for (int i = axis + 1; i < a->rank(); ++i) inner *= a->dims[i];
    const int64_t n = a->rank() ? a->dims[axis] : 1;
    const int sa = SlotOf(a);
    const int so = NewValueSlot(x);
    const int64_t scratch_bytes = k::arg_sort_scratch_bytes(outer, n, inner, ex_->dev->sm_count());
    const int sc = scratch_bytes > 0 ? NewTemp(scratch_bytes) : -1;
    const int dt = a->dtype;
    Step st;
    st.desc = strfmt("argsort[%s rows=%lld n=%lld inner=%lld %s]", dtype_name(dt), (long long)outer, (long long)n, (long long)inner,
                     descending ? "descending" : "ascending");
    st.reads = {sa};
    st.writes = {so};
    if (sc >= 0) st.writes.push_back(sc);
    st.run = [=](Device* dev, void* const* p) -> Status {
      return k::arg_sort(dev, p[sa], p[so], dt, outer, n, inner, descending, sc >= 0 ? p[sc] : nullptr, scratch_bytes);
    };
    ex_->steps.push_back(std::move(st));
    return Status::OK();
  }

  // If with heavy branches: in = predicate, then the outer values the true branch captures, then those of the false branch;
  // ia = [n outputs, true sub-graph, false sub-graph, n true captures, n false captures].  Each branch compiles into a
  // sub-plan that writes the result slots; the step runs ONE of them: on a plan's first runs the host reads the
  // predicate byte and launches the chosen sub-plan, in a replayed plan two conditional IF graph nodes do it on the
  // device.  The reference reads the predicate on the host and runs the chosen branch's executable
  // (ref mpsgraph executable.go:286-318).
  Status EmitIf(Node* w) {
    if (loop_depth_ >= Device::kMaxLoopDepth) return Status::Unsupported("compile: control flow nested deeper than 4");
    const int n_out = (int)w->ia[0];
    const int n_tc = (int)w->ia[3], n_fc = (int)w->ia[4];
    if (w->ia[1] < 0 || w->ia[2] < 0 || (size_t)w->ia[1] >= ctx_->subgraphs.size() || (size_t)w->ia[2] >= ctx_->subgraphs.size())
      return Status::Invalid("compile: If names a sub-graph the context does not hold");
    for (Node* i : w->in) B200_TRY(EnsureMaterialized(i));
    std::unique_ptr<Exec> on_true, on_false;
    SubGraph* tsg = ctx_->subgraphs[(size_t)w->ia[1]].get();
    SubGraph* fsg = ctx_->subgraphs[(size_t)w->ia[2]].get();
    Status s = CompileGraph(ctx_, tsg->graph, tsg->feeds, tsg->targets, &on_true, loop_depth_ + 1);
    if (!s.ok()) return Status{s.code, "If trueBranch: " + s.msg};
    s = CompileGraph(ctx_, fsg->graph, fsg->feeds, fsg->targets, &on_false, loop_depth_ + 1);
    if (!s.ok()) return Status{s.code, "If falseBranch: " + s.msg};
    Exec* te = on_true.get();
    Exec* fe = on_false.get();
    ex_->children.push_back(std::move(on_true));
    ex_->children.push_back(std::move(on_false));
    std::vector<int> in_slots, res_slots;
    for (Node* i : w->in) in_slots.push_back(SlotOf(i));
    std::vector<Node*> result_node(n_out, nullptr);
    for (auto& up : g_.nodes)
      if (up->op == Op::IfResult && up->in[0] == w && live_[up->id]) result_node[(size_t)up->ia[0]] = up.get();
    for (int i = 0; i < n_out; ++i) {
      const OutputDesc& od = te->outputs[(size_t)i];
      res_slots.push_back(result_node[i] ? NewValueSlot(result_node[i]) : NewTemp(od.nbytes));
    }
    slot_of_[w->id] = in_slots[0];   // the branch node itself has no value of its own
    static const bool device_loops = []() { const char* v = getenv("B200MLX_DEVICE_LOOPS"); return !(v && v[0] == '0'); }();
    bool recordable = device_loops;
    for (const Step& cs : te->steps) recordable = recordable && cs.capturable;
    for (const Step& cs : fe->steps) recordable = recordable && cs.capturable;
    if (recordable) {
      cudaStream_t ls = nullptr;
      B200_TRY(ex_->dev->LoopStream(loop_depth_, &ls));   // created now: not while a recording is under way
    }
    Step st;
    st.desc = strfmt("if[outputs=%d true: %d steps, %d captures; false: %d steps, %d captures%s]", n_out, (int)te->steps.size(), n_tc,
                     (int)fe->steps.size(), n_fc, recordable ? "; on the device when replayed" : "");
    st.reads = in_slots;
    st.writes = res_slots;
    st.capturable = recordable;
    st.wants_graph = recordable;
    st.launches = 0;
    const int depth = loop_depth_;
    st.run = [=](Device* dev, void* const* p) -> Status {
      B200_TRY(dev->MakeCurrent());
      std::vector<void*> tin(n_tc), fin(n_fc), outs(n_out);
      for (int i = 0; i < n_tc; ++i) tin[i] = p[in_slots[1 + i]];
      for (int i = 0; i < n_fc; ++i) fin[i] = p[in_slots[1 + n_tc + i]];
      for (int i = 0; i < n_out; ++i) outs[i] = p[res_slots[i]];
      const unsigned char* pred = reinterpret_cast<const unsigned char*>(p[in_slots[0]]);
      cudaStreamCaptureStatus recording = cudaStreamCaptureStatusNone;
      B200_CUDA_TRY(cudaStreamIsCapturing(dev->stream(), &recording));
      if (recording == cudaStreamCaptureStatusActive)
        return RecordIfNodes(dev, depth, pred, [&]() { return RunSubPlan(te, tin.data(), outs.data()); },
                             [&]() { return RunSubPlan(fe, fin.data(), outs.data()); });
      unsigned char go = 0;
      B200_CUDA_TRY(cudaMemcpyAsync(&go, pred, 1, cudaMemcpyDeviceToHost, dev->stream()));
      B200_CUDA_TRY(cudaStreamSynchronize(dev->stream()));
      return go ? RunSubPlan(te, tin.data(), outs.data()) : RunSubPlan(fe, fin.data(), outs.data());
    };
    ex_->steps.push_back(std::move(st));
    return Status::OK();
  }

  // While: in = initial state, then the outer values cond captures, then those body captures;
  // ia = [n_state, cond sub-graph, body sub-graph, n cond captures, n body captures] (sub-graphs are owned by the context).
  // cond and body compile into two sub-plans.  The step copies the initial state into the result slots, then loops on the
  // host: run cond, read its one byte back, stop or run body into a second set of state buffers and swap.  The reference
  // also loops on the host, re-entering a whole executable per iteration (ref mpsgraph executable.go:219-300).
  Status EmitWhile(Node* w) {
    if (loop_depth_ >= Device::kMaxLoopDepth) return Status::Unsupported("compile: While loops nested deeper than 4");
    const int n_state = (int)w->ia[0];
    const int n_cc = (int)w->ia[3], n_bc = (int)w->ia[4];
    if (w->ia[1] < 0 || w->ia[2] < 0 || (size_t)w->ia[1] >= ctx_->subgraphs.size() || (size_t)w->ia[2] >= ctx_->subgraphs.size())
      return Status::Invalid("compile: While names a sub-graph the context does not hold");
    for (Node* i : w->in) B200_TRY(EnsureMaterialized(i));
    std::unique_ptr<Exec> cond, body;
    SubGraph* csg = ctx_->subgraphs[(size_t)w->ia[1]].get();
    SubGraph* bsg = ctx_->subgraphs[(size_t)w->ia[2]].get();
    Status s = CompileGraph(ctx_, csg->graph, csg->feeds, csg->targets, &cond, loop_depth_ + 1);
    if (!s.ok()) return Status{s.code, "While cond: " + s.msg};
    s = CompileGraph(ctx_, bsg->graph, bsg->feeds, bsg->targets, &body, loop_depth_ + 1);
    if (!s.ok()) return Status{s.code, "While body: " + s.msg};
    Exec* ce = cond.get();
    Exec* be = body.get();
    ex_->children.push_back(std::move(cond));
    ex_->children.push_back(std::move(body));

    std::vector<int> in_slots, res_slots, tmp_slots;
    std::vector<int64_t> nbytes;
    for (Node* i : w->in) in_slots.push_back(SlotOf(i));
    // the WhileResult nodes that exist for this loop claim their slots now; a state value nobody reads still needs memory
    std::vector<Node*> result_node(n_state, nullptr);
    for (auto& up : g_.nodes)
      if (up->op == Op::WhileResult && up->in[0] == w && live_[up->id]) result_node[(size_t)up->ia[0]] = up.get();
    for (int i = 0; i < n_state; ++i) {
      const int64_t nb = w->in[i]->num_elements() * dtype_size(w->in[i]->dtype);
      nbytes.push_back(nb);
      res_slots.push_back(result_node[i] ? NewValueSlot(result_node[i]) : NewTemp(nb));
      // A state value that body only updates in place (its new value is DynamicUpdateSlice of its parameter, which
      // feeds nothing else: a KV cache that gets one more entry per trip) lives in ONE buffer: body is handed the same
      // address for the value and its successor and writes just the block.  The others alternate between two buffers.
      const bool in_place = (size_t)i < be->donate_alias.size() && be->donate_alias[(size_t)i] == i;
      tmp_slots.push_back(in_place ? -1 : NewTemp(nb));
    }
    const int pred_slot = NewTemp(256);
    slot_of_[w->id] = pred_slot;

    // The loop runs on the device (a conditional WHILE node) when the plan is replayed as a CUDA graph, which needs every
    // step of both sub-plans to be recordable; otherwise, and on a plan's first runs, the host drives it.
    static const bool device_loops = []() { const char* v = getenv("B200MLX_DEVICE_LOOPS"); return !(v && v[0] == '0'); }();
    bool recordable = device_loops;
    for (const Step& cs : ce->steps) recordable = recordable && cs.capturable;
    for (const Step& bs : be->steps) recordable = recordable && bs.capturable;
    if (recordable) {
      cudaStream_t ls = nullptr;
      B200_TRY(ex_->dev->LoopStream(loop_depth_, &ls));   // created now: not while a recording is under way
    }
    Step st;
    int n_in_place = 0;
    for (int t : tmp_slots) n_in_place += t < 0 ? 1 : 0;
    st.desc = strfmt("while[state=%d (%d updated in place) cond: %d steps, %d captures; body: %d steps, %d captures%s]", n_state, n_in_place,
                     (int)ce->steps.size(), n_cc, (int)be->steps.size(), n_bc, recordable ? "; on the device when replayed" : "");
    st.reads = in_slots;
    st.writes = res_slots;
    for (int t : tmp_slots)
      if (t >= 0) st.writes.push_back(t);
    st.writes.push_back(pred_slot);
    st.capturable = recordable;
    st.wants_graph = recordable;
    st.launches = 0;         // counted per run: unknown at compile time
    const int depth = loop_depth_;
    st.run = [=](Device* dev, void* const* p) -> Status {
      B200_TRY(dev->MakeCurrent());
      std::vector<void*> cur(n_state), nxt(n_state);
      for (int i = 0; i < n_state; ++i) {
        cur[i] = p[res_slots[i]];
        nxt[i] = tmp_slots[i] >= 0 ? p[tmp_slots[i]] : cur[i];   // updated in place: one buffer
        if (nbytes[i] > 0) B200_CUDA_TRY(cudaMemcpyAsync(cur[i], p[in_slots[i]], (size_t)nbytes[i], cudaMemcpyDeviceToDevice, dev->stream()));
      }
      std::vector<void*> cin(n_state + n_cc), bin(n_state + n_bc);
      for (int i = 0; i < n_cc; ++i) cin[n_state + i] = p[in_slots[n_state + i]];
      for (int i = 0; i < n_bc; ++i) bin[n_state + i] = p[in_slots[n_state + n_cc + i]];
      void* pred = p[pred_slot];
      cudaStreamCaptureStatus recording = cudaStreamCaptureStatusNone;
      B200_CUDA_TRY(cudaStreamIsCapturing(dev->stream(), &recording));
      if (recording == cudaStreamCaptureStatusActive) {
        // fixed addresses: body writes the second set of state buffers and the new state is copied over the current one
        for (int i = 0; i < n_state; ++i) cin[i] = bin[i] = cur[i];
        auto run_cond = [&]() { return RunSubPlan(ce, cin.data(), &pred); };
        auto run_body = [&]() -> Status {
          B200_TRY(RunSubPlan(be, bin.data(), nxt.data()));
          for (int i = 0; i < n_state; ++i)
            if (nbytes[i] > 0 && cur[i] != nxt[i])
              B200_CUDA_TRY(cudaMemcpyAsync(cur[i], nxt[i], (size_t)nbytes[i], cudaMemcpyDeviceToDevice, dev->stream()));
          return Status::OK();
        };
        dev->kernel_error_flag();   // the loop may raise the error word: have the next synchronisation point read it
        return RecordWhileNode(dev, depth, run_cond, run_body, reinterpret_cast<const unsigned char*>(pred),
                               reinterpret_cast<int*>(reinterpret_cast<char*>(pred) + 64));
      }
      for (int64_t iter = 0;; ++iter) {
        if (iter >= kWhileMaxIterations) return Status::Invalid("While: exceeded maximum iterations (1000000)");
        for (int i = 0; i < n_state; ++i) cin[i] = bin[i] = cur[i];
        B200_TRY(RunSubPlan(ce, cin.data(), &pred));
        unsigned char go = 0;
        B200_CUDA_TRY(cudaMemcpyAsync(&go, pred, 1, cudaMemcpyDeviceToHost, dev->stream()));
        B200_CUDA_TRY(cudaStreamSynchronize(dev->stream()));
        if (!go) break;
        B200_TRY(RunSubPlan(be, bin.data(), nxt.data()));
        cur.swap(nxt);
      }
      for (int i = 0; i < n_state; ++i)
        if (cur[i] != p[res_slots[i]] && nbytes[i] > 0)
          B200_CUDA_TRY(cudaMemcpyAsync(p[res_slots[i]], cur[i], (size_t)nbytes[i], cudaMemcpyDeviceToDevice, dev->stream()));
      return Status::OK();
    };
    ex_->steps.push_back(std::move(st));
    return Status::OK();
  }

  Status EmitRngBits(Node* x) {
    Node* state = x->in[0];
    B200_TRY(EnsureMaterialized(state));
    const int st_slot = SlotOf(state), out_slot = NewValueSlot(x);
    const int dt = x->dtype;
    const int64_t n = x->num_elements();
    Step st;
    st.desc = strfmt("rng_bits[n=%lld %s]", (long long)n, dtype_name(dt));
    st.reads = {st_slot};
    st.writes = {out_slot};
    st.run = [=](Device* dev, void* const* p) -> Status { return k::rng_bits(dev, p[st_slot], p[out_slot], dt, n); };
    ex_->steps.push_back(std::move(st));
    return Status::OK();
  }

  // ----------------------------------------------------------- softmax etc. ---
  Status EmitSoftmax(Node* x) {
    Node* src = x->in[0];
    B200_TRY(EnsureMaterialized(src));
    const int ax = (int)x->ia[0];
    int64_t outer = 1, inner = 1;
    for (int d = 0; d < ax; ++d) outer *= src->dims[d];
    for (int d = ax + 1; d < src->rank(); ++d) inner *= src->dims[d];
    const int64_t n = src->dims[ax];
    const int in_slot = SlotOf(src), out_slot = NewValueSlot(x), dt = x->dtype;
    Step st;
    st.desc = strfmt("softmax[outer=%lld n=%lld inner=%lld %s]", (long long)outer, (long long)n, (long long)inner, dtype_name(dt));
    st.reads = {in_slot};
    st.writes = {out_slot};
    if (inner == 1 && dt != B200_FLOAT64) {
      st.run = [=](Device* dev, void* const* p) -> Status {
        k::SoftmaxParams sp;
        sp.x = p[in_slot]; sp.y = p[out_slot]; sp.rows = outer; sp.cols = n; sp.dtype = dt;
        return k::softmax_rows(dev, sp);
      };
    } else {
      if (dt == B200_FLOAT64) return Status::Unsupported("FusedSoftmax: Float64");
      st.run = [=](Device* dev, void* const* p) -> Status { return k::softmax_strided(dev, p[in_slot], p[out_slot], outer, n, inner, dt); };
    }
    ex_->steps.push_back(std::move(st));
    return Status::OK();
  }

  Status EmitSoftmaxMasked(Node* x) {
    Node* src = x->in[0];
    Node* mask = x->in.size() > 1 ? x->in[1] : nullptr;
    B200_TRY(EnsureMaterialized(src));
    if (mask) B200_TRY(EnsureMaterialized(mask));
    const int r = src->rank();
    const int64_t cols = src->dims[r - 1], seq_q = src->dims[r - 2];
    const int64_t heads = r >= 3 ? src->dims[r - 3] : 1;
    int64_t rows = 1;
    for (int d = 0; d < r - 1; ++d) rows *= src->dims[d];
    k::SoftmaxParams sp;
    sp.rows = rows; sp.cols = cols; sp.dtype = x->dtype; sp.scale = x->fa[0]; sp.causal = x->ia[0] != 0;
    sp.seq_q = seq_q; sp.heads = heads;
    if (mask) {
      sp.mask_kind = mask->dtype == B200_BOOL ? 1 : 2;
      const std::vector<int64_t> ms = dense_strides(mask->dims);
      const int off = r - mask->rank();
      // positions: batch (everything left of heads, must be one dim or broadcast), head, q, k
      auto stride_at = [&](int xdim) -> int64_t {
        const int md = xdim - off;
        if (md < 0 || mask->dims[md] == 1) return 0;
        return ms[md];
      };
      sp.mask_strides[3] = stride_at(r - 1);
      sp.mask_strides[2] = stride_at(r - 2);
      sp.mask_strides[1] = r >= 3 ? stride_at(r - 3) : 0;
      int64_t bstride = 0;
      int nonbroadcast_batch_dims = 0;
      for (int d = 0; d < r - 3; ++d)
        if (stride_at(d) != 0) { nonbroadcast_batch_dims++; bstride = stride_at(d); }
      if (nonbroadcast_batch_dims > 1 || (nonbroadcast_batch_dims == 1 && r - 3 > 1))
        return Status::Unsupported("SoftmaxMasked: mask varies over more than one leading batch axis");
      sp.mask_strides[0] = bstride;
    }
    const int in_slot = SlotOf(src), out_slot = NewValueSlot(x), mask_slot = mask ? SlotOf(mask) : -1;
    Step st;
    st.desc = strfmt("softmax_masked[rows=%lld cols=%lld %s scale=%g causal=%d mask=%d]", (long long)rows, (long long)cols,
                     dtype_name(x->dtype), sp.scale, (int)sp.causal, sp.mask_kind);
    st.reads = {in_slot};
    if (mask) st.reads.push_back(mask_slot);
    st.writes = {out_slot};
    st.run = [sp, in_slot, out_slot, mask_slot](Device* dev, void* const* p) -> Status {
      k::SoftmaxParams q = sp;
      q.x = p[in_slot];
      q.y = p[out_slot];
      q.mask = mask_slot >= 0 ? p[mask_slot] : nullptr;
      return k::softmax_rows(dev, q);
    };
    ex_->steps.push_back(std::move(st));
    return Status::OK();
  }

  // Recognises t = Reshape[B,S,H,D](Slice(X[B,S,W], last axis [lo, lo + H*D))) with X in (or going to) memory:
  // the attention kernel can then read t in place inside X.  Fills the source node, the element offset and the
  // (batch, head, sequence) strides.
  bool StridedProjectionView(Node* t, bool bshd, Node** src, int64_t* offset, int64_t strides[3]) {
    if (!bshd || t->op != Op::Reshape || t->rank() != 4) return false;
    Node* sl = t->in[0];
    if (sl->op != Op::Slice || sl->rank() != 3) return false;
    Node* X = sl->in[0];
    if (X->rank() != 3 || slot_of_[ViewBase(sl)->id] >= 0) return false;  // already copied: nothing to gain
    for (int d = 0; d < 3; ++d)
      if (sl->ia[2 * d + 1] != 1) return false;
    if (sl->ia[0] != 0 || sl->ia[2] != 0 || sl->dims[0] != X->dims[0] || sl->dims[1] != X->dims[1]) return false;
    const int64_t B = t->dims[0], S = t->dims[1], H = t->dims[2], D = t->dims[3], W = X->dims[2];
    if (sl->dims[0] != B || sl->dims[1] != S || sl->dims[2] != H * D) return false;
    const int64_t lo = sl->ia[4];
    if (lo % 8 != 0 || W % 8 != 0) return false;  // TMA: 16-byte aligned base and pitches
    Node* base = ViewBase(X);
    if (!(base->op == Op::Parameter || slot_of_[base->id] >= 0 || MustMaterialize(base))) return false;
    *src = X;
    *offset = lo;
    strides[0] = S * W;
    strides[1] = D;
    strides[2] = W;
    return true;
  }

  // Recognises t = Reshape*(Slice(X)) where the slice keeps every axis of X whole except a unit-stride range [lo, lo + w)
  // of the last one, the slice has not been copied yet, and the reshapes keep the split "rows of X | columns of the
  // range" (leading dims of t multiply to X's row count, the rest to w).  t can then be read in place inside X: fills
  // the source node, the element offset and t's element strides.
  bool ColumnRangeView(Node* t, Node** src, int64_t* offset, std::vector<int64_t>* strides) {
    Node* sl = t;
    while (sl->op == Op::Reshape) sl = sl->in[0];
    if (sl->op != Op::Slice || sl->rank() < 1 || t->rank() < 1 || slot_of_[ViewBase(t)->id] >= 0 || slot_of_[ViewBase(sl)->id] >= 0) return false;
    Node* X = sl->in[0];
    const int r = sl->rank();
    for (int d = 0; d < r; ++d) {
      if (sl->ia[2 * d + 1] != 1) return false;
      if (d < r - 1 && (sl->ia[2 * d] != 0 || sl->dims[d] != X->dims[d])) return false;
    }
    const int64_t W = X->dims[r - 1], w = sl->dims[r - 1], lo = sl->ia[2 * (r - 1)];
    int64_t rows = 1;
    for (int d = 0; d < r - 1; ++d) rows *= X->dims[d];
    if (w <= 0 || rows <= 0 || w == W) return false;
    int j = 0;
    int64_t lead = 1;
    while (j < t->rank() && lead < rows) lead *= t->dims[j++];
    if (lead != rows) return false;
    int64_t rest = 1;
    for (int d = j; d < t->rank(); ++d) rest *= t->dims[d];
    if (rest != w) return false;
    Node* base = ViewBase(X);
    if (!(base->op == Op::Parameter || slot_of_[base->id] >= 0 || MustMaterialize(base))) return false;
    strides->assign(t->rank(), 0);
    int64_t st = 1;
    for (int d = t->rank() - 1; d >= j; --d) { (*strides)[d] = st; st *= t->dims[d]; }
    st = W;
    for (int d = j - 1; d >= 0; --d) { (*strides)[d] = st; st *= t->dims[d]; }
    *src = X;
    *offset = lo;
    return true;
  }

  Status EmitAttention(Node* x) {
    Node* q = x->in[0];
    Node* kk = x->in[1];
    Node* v = x->in[2];
    const bool bshd = x->ia[2] != 0;
    Node* srcs[3] = {q, kk, v};
    int64_t offs[3] = {0, 0, 0};
    int64_t strd[3][3] = {{0, 0, 0}, {0, 0, 0}, {0, 0, 0}};
    k::AttentionParams probe;
    probe.B = q->dims[0]; probe.H = x->ia[0]; probe.Hkv = x->ia[1];
    probe.Sq = q->dims[bshd ? 1 : 2]; probe.Sk = kk->dims[bshd ? 1 : 2];
    probe.head_dim = q->dims[3]; probe.causal = x->ia[3] != 0; probe.scale = x->fa[0]; probe.dtype = x->dtype;
    const bool decode_shape = k::attention_decode_supported(probe);
    if (x->dtype == B200_BFLOAT16 || x->dtype == B200_FLOAT16) {
      for (int i = 0; i < 3; ++i) {
        Node* src;
        int64_t off, st3[3];
        std::vector<int64_t> st4;
        if (StridedProjectionView(srcs[i], bshd, &src, &off, st3)) {
          srcs[i] = src;
          offs[i] = off;
          for (int j = 0; j < 3; ++j) strd[i][j] = st3[j];
        } else if (i == 0 && decode_shape && ColumnRangeView(q, &src, &off, &st4) &&
                   st4[3] == 1 && off % 8 == 0 && st4[0] % 8 == 0 && st4[bshd ? 2 : 1] % 8 == 0) {
          // one query position: the cache-reading kernel takes the query in place inside the fused projection
          srcs[i] = src;
          offs[i] = off;
          strd[i][0] = st4[0];
          strd[i][1] = st4[bshd ? 2 : 1];
          strd[i][2] = st4[0];   // one position only: never multiplied by anything but 0
        }
      }
    }
    B200_TRY(EnsureMaterialized(srcs[0]));
    B200_TRY(EnsureMaterialized(srcs[1]));
    B200_TRY(EnsureMaterialized(srcs[2]));
    k::AttentionParams ap;
    ap.B = q->dims[0];
    ap.H = x->ia[0];
    ap.Hkv = x->ia[1];
    ap.Sq = q->dims[bshd ? 1 : 2];
    ap.Sk = kk->dims[bshd ? 1 : 2];
    ap.head_dim = q->dims[3];
    ap.bshd = bshd;
    ap.causal = x->ia[3] != 0;
    ap.scale = x->fa[0];
    ap.dtype = x->dtype;
    for (int j = 0; j < 3; ++j) { ap.q_strides[j] = strd[0][j]; ap.k_strides[j] = strd[1][j]; ap.v_strides[j] = strd[2][j]; }
    // One query position: the cache-reading kernel, which also takes the mask (dims aligned to the trailing dims of
    // [B, H, 1, Sk]; of [B, 1, H, Sk] for a rank-4 mask in the BSHD layout).
    const bool decode = k::attention_decode_supported(ap);
    Node* mk = x->in.size() > 3 ? x->in[3] : nullptr;
    if (mk && !decode) return Status::Unsupported("attention with a mask tensor needs one query position");
    int ms = -1;
    if (mk) {
      B200_TRY(EnsureMaterialized(mk));
      ms = SlotOf(mk);
      ap.mask_kind = mk->dtype == B200_BOOL ? 1 : 2;
      const int r = mk->rank();
      const int h_pos = bshd && r == 4 ? 2 : 1;   // position of the head dim among the four
      int64_t stride = 1;
      for (int i = r - 1; i >= 0; --i) {
        const int pos = 4 - r + i;   // position among the four dims
        const int64_t st1 = mk->dims[i] == 1 ? 0 : stride;
        if (pos == 3) ap.m_k = st1;
        else if (pos == h_pos) ap.m_h = st1;
        else if (pos == 0) ap.m_b = st1;
        stride *= mk->dims[i];
      }
    }
    const int qs = SlotOf(srcs[0]), ks = SlotOf(srcs[1]), vs = SlotOf(srcs[2]), os = NewValueSlot(x);
    const int64_t es = dtype_size(x->dtype);
    const int64_t qo = offs[0] * es, ko = offs[1] * es, vo = offs[2] * es;
    Step st;
    st.desc = strfmt("%s[B=%lld H=%lld Hkv=%lld Sq=%lld Sk=%lld D=%lld %s %s causal=%d%s]", decode ? "attention_decode" : "attention",
                     (long long)ap.B, (long long)ap.H, (long long)ap.Hkv, (long long)ap.Sq, (long long)ap.Sk, (long long)ap.head_dim,
                     dtype_name(ap.dtype), bshd ? "BSHD" : "BHSD", (int)ap.causal, mk ? (ap.mask_kind == 1 ? " mask=Bool" : " mask=additive") : "");
    st.reads = {qs, ks, vs};
    if (ms >= 0) st.reads.push_back(ms);
    st.writes = {os};
    st.run = [ap, qs, ks, vs, os, ms, qo, ko, vo, decode](Device* dev, void* const* p) -> Status {
      k::AttentionParams a = ap;
      a.q = (const char*)p[qs] + qo;
      a.k = (const char*)p[ks] + ko;
      a.v = (const char*)p[vs] + vo;
      a.o = p[os];
      a.mask = ms >= 0 ? p[ms] : nullptr;
      return decode ? k::attention_decode(dev, a) : k::attention(dev, a);
    };
    ex_->steps.push_back(std::move(st));
    return Status::OK();
  }

  // A table operand of Rope: when it is a broadcast of a smaller tensor over LEADING axes only (the same table for every
  // batch entry), the kernel reads the small tensor with a period instead of a materialised copy.
  // *per_head (when asked for): the table is [positions, head_dim], spread over the heads by a broadcast
  // [S, D] -> [S, heads, D] and over the batch by a second one; the kernel then indexes it by (row mod S, column mod D)
  // and neither broadcast is materialised.
  Status PeriodicOperand(Node* t, int* slot, int64_t* period, int64_t head_dim = 0, bool* per_head = nullptr) {
    Node* b = t;
    while (b->op == Op::Identity) b = b->in[0];
    if (per_head) *per_head = false;
    if (b->op == Op::BroadcastInDim) {
      Node* src = b->in[0];
      const int r = b->rank(), k = src->rank();
      bool trailing = k <= r && k > 0;
      for (int i = 0; i < k && trailing; ++i) trailing = b->ia[i] == r - k + i && src->dims[i] == b->dims[r - k + i];
      if (trailing && per_head && head_dim > 0) {
        // [S, D] -> [S, heads, D] underneath?  (x is [.., S, heads, D] with rows = (.., S): the row number mod S is the position)
        Node* inner = src;
        while (inner->op == Op::Identity) inner = inner->in[0];
        if (inner->op == Op::BroadcastInDim && inner->rank() == 3 && inner->in[0]->rank() == 2 && inner->ia.size() == 2 &&
            inner->ia[0] == 0 && inner->ia[1] == 2 && inner->in[0]->dims[0] == inner->dims[0] &&
            inner->in[0]->dims[1] == inner->dims[2] && inner->dims[2] == head_dim && k == 3 && src->dims == inner->dims) {
          Node* table = inner->in[0];
          B200_TRY(EnsureMaterialized(table));
          *slot = SlotOf(table);
          *period = table->num_elements();
          *per_head = true;
          return Status::OK();
        }
      }
      if (trailing && src->num_elements() > 0) {
        B200_TRY(EnsureMaterialized(src));
        *slot = SlotOf(src);
        *period = src->num_elements();
        return Status::OK();
      }
    }
    B200_TRY(EnsureMaterialized(t));
    *slot = SlotOf(t);
    *period = t->num_elements();
    return Status::OK();
  }

  Status EmitRope(Node* x) {
    Node* src = x->in[0];
    k::RopeParams rp;
    rp.dtype = x->dtype;
    rp.head_dim = x->dims.back();
    Node* base = src;
    int64_t offset = 0, st3[3];
    bool in_place_range = false;
    const int64_t vec = 16 / dtype_size(x->dtype);
    if (src->rank() == 4 && StridedProjectionView(src, true, &base, &offset, st3) && offset % vec == 0 && st3[2] % vec == 0) {
      rp.rows = src->dims[0] * src->dims[1];
      rp.cols = src->dims[2] * src->dims[3];
      rp.x_pitch = st3[2];
    } else if (std::vector<int64_t> vs; ColumnRangeView(src, &base, &offset, &vs) && vs.back() == 1 && offset % vec == 0 &&
               base->dims.back() % vec == 0 && (src->num_elements() / (base->num_elements() / base->dims.back())) % rp.head_dim == 0) {
      // a column range of a wider tensor (the Q or K part of a decoding step's fused projection): its rows in place
      rp.x_pitch = base->dims.back();
      rp.rows = base->num_elements() / rp.x_pitch;
      rp.cols = src->num_elements() / rp.rows;
      in_place_range = true;
    } else {
      base = src;
      offset = 0;
      // rows of (heads x head_dim) when there is a head axis, so that a row number is a position (per-head tables below)
      rp.cols = src->rank() >= 3 ? src->dims[src->rank() - 2] * src->dims.back() : src->dims.back();
      rp.rows = src->num_elements() / rp.cols;
      rp.x_pitch = rp.cols;
    }
    B200_TRY(EnsureMaterialized(base));
    int c_slot, s_slot;
    // a per-head table needs x's rows to be (batch.., position) and its columns (head, head_dim): rank >= 3 with the
    // position on axis rank - 3
    const bool rows_are_positions = !in_place_range && src->rank() >= 3 && rp.cols == src->dims[src->rank() - 2] * src->dims[src->rank() - 1];
    B200_TRY(PeriodicOperand(x->in[1], &c_slot, &rp.c_period, rows_are_positions ? rp.head_dim : 0, &rp.c_per_head));
    B200_TRY(PeriodicOperand(x->in[2], &s_slot, &rp.s_period, rows_are_positions ? rp.head_dim : 0, &rp.s_per_head));
    const int x_slot = SlotOf(base), out_slot = NewValueSlot(x);
    const int64_t x_off = offset * dtype_size(x->dtype);
    Step st;
    st.desc = strfmt("rope[rows=%lld cols=%lld head=%lld %s pitch=%lld table_period=%lld%s]", (long long)rp.rows, (long long)rp.cols,
                     (long long)rp.head_dim, dtype_name(x->dtype), (long long)rp.x_pitch, (long long)rp.c_period,
                     rp.c_per_head ? " per-head" : "");
    st.reads = {x_slot, c_slot, s_slot};
    st.writes = {out_slot};
    st.run = [rp, x_slot, c_slot, s_slot, out_slot, x_off](Device* dev, void* const* p) -> Status {
      k::RopeParams q = rp;
      q.x = (const char*)p[x_slot] + x_off;
      q.c = p[c_slot];
      q.s = p[s_slot];
      q.y = p[out_slot];
      return k::rope(dev, q);
    };
    ex_->steps.push_back(std::move(st));
    return Status::OK();
  }

  // A [cols] vector for gamma / beta: the parameter itself when it already is
  // one, else a broadcast copy laid over the normalised axes.
  Status NormParamSlot(Node* x, Node* p, const std::vector<int64_t>& axes, int64_t cols, int* slot) {
    B200_TRY(EnsureMaterialized(p));
    if (p->num_elements() == cols) {
      // dims (ignoring 1s) must follow the normalised axes in order: true when counts match, because
      // check_scale() aligned it either to the axes (lower rank) or to the full shape (equal rank).
      *slot = SlotOf(p);
      return Status::OK();
    }
    // broadcast inside the normalised axes
    std::vector<int64_t> nd;
    for (auto ax : axes) nd.push_back(x->dims[ax]);
    k::StridedCopyParams sc;
    sc.elt_size = dtype_size(p->dtype);
    sc.rank = (int)nd.size();
    if (sc.rank > k::kMaxDims) return Status::Unsupported("norm: more than 8 normalised axes");
    const std::vector<int64_t> os = dense_strides(nd), ps = dense_strides(p->dims);
    for (int d = 0; d < sc.rank; ++d) {
      sc.dims[d] = nd[d];
      sc.out_strides[d] = os[d];
      int pd;
      if (p->rank() >= x->rank()) pd = (int)axes[d];
      else pd = d < p->rank() ? d : -1;
      sc.in_strides[d] = (pd < 0 || p->dims[pd] == 1) ? 0 : ps[pd];
    }
    const int in_slot = SlotOf(p);
    const int tmp = NewTemp(cols * dtype_size(p->dtype));
    Step st;
    st.desc = "move[norm parameter broadcast]";
    st.reads = {in_slot};
    st.writes = {tmp};
    st.run = [sc, in_slot, tmp](Device* dev, void* const* ptrs) -> Status {
      k::StridedCopyParams q = sc;
      q.x = ptrs[in_slot];
      q.y = ptrs[tmp];
      return k::strided_copy(dev, q);
    };
    ex_->steps.push_back(std::move(st));
    *slot = tmp;
    return Status::OK();
  }

  Status EmitNorm(Node* x) {
    Node* src = x->in[0];
    B200_TRY(EnsureMaterialized(src));
    if (x->dtype == B200_FLOAT64) return Status::Unsupported("norm: Float64");
    const bool rms = x->op == Op::RmsNorm;
    const bool has_gamma = x->ia[0] != 0, has_beta = x->ia[1] != 0;
    std::vector<int64_t> axes(x->ia.begin() + 2, x->ia.end());
    const int r = src->rank();
    int64_t cols = 1;
    for (auto ax : axes) cols *= src->dims[ax];
    const int64_t rows = cols ? src->num_elements() / cols : 0;
    // trailing block of axes?
    bool trailing = true;
    for (size_t i = 0; i < axes.size(); ++i) trailing &= axes[i] == (int64_t)(r - (int)axes.size() + (int)i);
    int gamma_slot = -1, beta_slot = -1;
    size_t pi = 1;
    if (has_gamma) B200_TRY(NormParamSlot(src, x->in[pi++], axes, cols, &gamma_slot));
    if (has_beta) B200_TRY(NormParamSlot(src, x->in[pi++], axes, cols, &beta_slot));
    int in_slot = SlotOf(src);
    std::vector<int> perm, inv;
    if (!trailing) {
      if (r > k::kMaxDims) return Status::Unsupported("norm: more than 8 dims");
      std::vector<bool> is_norm(r, false);
      for (auto ax : axes) is_norm[ax] = true;
      for (int d = 0; d < r; ++d)
        if (!is_norm[d]) perm.push_back(d);
      for (auto ax : axes) perm.push_back((int)ax);
      in_slot = EmitPermutedTemp(src, perm, "norm axes -> trailing");
      inv.resize(r);
      for (int d = 0; d < r; ++d) inv[perm[d]] = d;
    }
    const int64_t nbytes = x->num_elements() * dtype_size(x->dtype);
    const int norm_out = trailing ? NewValueSlot(x) : NewTemp(nbytes);
    k::NormParams np;
    np.rows = rows; np.cols = cols; np.dtype = x->dtype; np.epsilon = x->fa[0]; np.rms = rms;
    Step st;
    st.desc = strfmt("%s[rows=%lld cols=%lld %s gamma=%d beta=%d]", rms ? "rms_norm" : "layer_norm", (long long)rows, (long long)cols,
                     dtype_name(x->dtype), (int)has_gamma, (int)has_beta);
    st.reads = {in_slot};
    if (gamma_slot >= 0) st.reads.push_back(gamma_slot);
    if (beta_slot >= 0) st.reads.push_back(beta_slot);
    st.writes = {norm_out};
    st.run = [np, in_slot, gamma_slot, beta_slot, norm_out](Device* dev, void* const* p) -> Status {
      k::NormParams q = np;
      q.x = p[in_slot];
      q.y = p[norm_out];
      q.gamma = gamma_slot >= 0 ? p[gamma_slot] : nullptr;
      q.beta = beta_slot >= 0 ? p[beta_slot] : nullptr;
      return k::norm_rows(dev, q);
    };
    ex_->steps.push_back(std::move(st));
    if (!trailing) {
      // permute back
      std::vector<int64_t> pd(r);
      for (int d = 0; d < r; ++d) pd[d] = src->dims[perm[d]];
      k::StridedCopyParams sc;
      sc.elt_size = dtype_size(x->dtype);
      sc.rank = r;
      const std::vector<int64_t> ps = dense_strides(pd), os = dense_strides(x->dims);
      for (int d = 0; d < r; ++d) { sc.dims[d] = x->dims[d]; sc.out_strides[d] = os[d]; sc.in_strides[d] = ps[inv[d]]; }
      const int out_slot = NewValueSlot(x);
      Step back;
      back.desc = "move[norm axes back]";
      back.reads = {norm_out};
      back.writes = {out_slot};
      back.run = [sc, norm_out, out_slot](Device* dev, void* const* ptrs) -> Status {
        k::StridedCopyParams q = sc;
        q.x = ptrs[norm_out];
        q.y = ptrs[out_slot];
        return k::strided_copy(dev, q);
      };
      ex_->steps.push_back(std::move(back));
    }
    return Status::OK();
  }

  // ----------------------------------------------------------- memory plan ---
  void PlanArena() {
    auto& slots = ex_->slots;
    for (int si = 0; si < (int)ex_->steps.size(); ++si) {
      for (int s : ex_->steps[si].writes) {
        if (slots[s].first_step < 0) slots[s].first_step = si;
        slots[s].last_step = si;
      }
      for (int s : ex_->steps[si].reads) {
        if (slots[s].first_step < 0) slots[s].first_step = si;
        slots[s].last_step = si;
      }
    }
    // Greedy first-fit over time: walk slots by first use, place each at the
    // lowest offset that does not overlap a slot still alive.
    std::vector<int> order;
    for (int s = 0; s < (int)slots.size(); ++s)
      if (slots[s].kind == SlotKind::Arena && slots[s].first_step >= 0) order.push_back(s);
    std::sort(order.begin(), order.end(), [&](int a, int b) { return slots[a].first_step < slots[b].first_step; });
    std::vector<int> placed;
    int64_t top = 0;
    for (int s : order) {
      const int64_t size = align_up(std::max<int64_t>(slots[s].nbytes, 1), 256);
      std::vector<std::pair<int64_t, int64_t>> busy;
      for (int o : placed)
        if (slots[o].last_step >= slots[s].first_step && slots[o].first_step <= slots[s].last_step)
          busy.emplace_back(slots[o].offset, slots[o].offset + align_up(std::max<int64_t>(slots[o].nbytes, 1), 256));
      std::sort(busy.begin(), busy.end());
      int64_t off = 0;
      for (auto& iv : busy) {
        if (off + size <= iv.first) break;
        off = std::max(off, iv.second);
      }
      slots[s].offset = off;
      top = std::max(top, off + size);
      placed.push_back(s);
    }
    ex_->arena_bytes = top;
  }
};

Status CompileGraph(Ctx* owner, Graph& graph, std::vector<Node*> feeds, std::vector<Node*> targets, std::unique_ptr<Exec>* out, int loop_depth) {
  Device* dev = nullptr;
  B200_TRY(Device::Get(graph.device, &dev));
  RewriteRmsNorm(graph, targets);
  RewriteSoftmax(graph, targets);
  RewriteGemmResidual(graph, targets);
  RewriteRope(graph, targets);
  std::unique_ptr<Exec> ex(new Exec());
  ex->dev = dev;
  Planner planner(owner, graph, ex.get(), loop_depth);
  B200_TRY(planner.Run(feeds, targets));
  if (ex->arena_bytes > 0) B200_TRY(ex->dev->Alloc(ex->arena_bytes, &ex->arena));
  static const bool graphs_on = []() { const char* v = getenv("B200MLX_GRAPHS"); return !(v && v[0] == '0'); }();
  bool wanted = ex->steps.size() >= 4;   // short plans are not launch-bound ... unless a step asks
  for (const Step& st : ex->steps) wanted = wanted || st.wants_graph;
  bool all = graphs_on && wanted;
  for (const Step& st : ex->steps) all = all && st.capturable;
  ex->capturable = all;
  *out = std::move(ex);
  return Status::OK();
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

B200Exec b200_compile(B200Context ctx, const B200Value* feeds, int num_feeds, const B200Value* targets, int num_targets,
                      B200Error* err) {
  clear_error(err);
  if (!ctx) { set_error(err, Status::Invalid("compile: null context")); return nullptr; }
  Ctx* c = reinterpret_cast<Ctx*>(ctx);
  if (num_targets < 1 || !targets) { set_error(err, Status::Invalid("compile: no outputs (Return was not called)")); return nullptr; }
  std::vector<Node*> f, t;
  auto own = [&](B200Value v) -> Node* {
    Node* n = reinterpret_cast<Node*>(v);
    if (!n || n->graph != &c->graph) return nullptr;
    return n;
  };
  for (int i = 0; i < num_feeds; ++i) {
    Node* n = own(feeds[i]);
    if (!n) { set_error(err, Status::Invalid("compile: feed does not belong to this context")); return nullptr; }
    f.push_back(n);
  }
  for (int i = 0; i < num_targets; ++i) {
    Node* n = own(targets[i]);
    if (!n) { set_error(err, Status::Invalid("compile: target does not belong to this context")); return nullptr; }
    t.push_back(n);
  }
  std::unique_ptr<Exec> ex;
  Status s = CompileGraph(c, c->graph, f, t, &ex);
  if (!s.ok()) { set_error(err, s); return nullptr; }
  return ex.release();
}

void b200_destroy_exec(B200Exec exec) { delete reinterpret_cast<Exec*>(exec); }
int b200_exec_device(B200Exec exec) { return exec ? reinterpret_cast<Exec*>(exec)->dev->ordinal() : -1; }
int b200_exec_num_inputs(B200Exec exec) { return exec ? (int)reinterpret_cast<Exec*>(exec)->inputs.size() : -1; }
int b200_exec_num_outputs(B200Exec exec) { return exec ? (int)reinterpret_cast<Exec*>(exec)->outputs.size() : -1; }
static int desc_shape(const OutputDesc& d, int* dtype, int64_t* dims, int cap) {
  if (dtype) *dtype = d.dtype;
  for (int i = 0; i < (int)d.dims.size() && i < cap; ++i) dims[i] = d.dims[i];
  return (int)d.dims.size();
}
int b200_exec_output_shape(B200Exec exec, int i, int* dtype, int64_t* dims, int cap) {
  Exec* ex = reinterpret_cast<Exec*>(exec);
  if (!ex || i < 0 || i >= (int)ex->outputs.size()) return -1;
  return desc_shape(ex->outputs[i], dtype, dims, cap);
}
int b200_exec_input_shape(B200Exec exec, int i, int* dtype, int64_t* dims, int cap) {
  Exec* ex = reinterpret_cast<Exec*>(exec);
  if (!ex || i < 0 || i >= (int)ex->inputs.size()) return -1;
  return desc_shape(ex->inputs[i], dtype, dims, cap);
}
int b200_exec_num_launches(B200Exec exec) { return exec ? reinterpret_cast<Exec*>(exec)->num_launches : -1; }
int64_t b200_exec_arena_bytes(B200Exec exec) { return exec ? reinterpret_cast<Exec*>(exec)->arena_bytes : -1; }
int64_t b200_exec_describe(B200Exec exec, char* buf, int64_t cap) {
  Exec* ex = reinterpret_cast<Exec*>(exec);
  if (!ex) return -1;
  // one line per step; the sub-plans of loops and branches follow their step, indented, in the order the step names them
  std::string s;
  std::function<void(const Exec*, const std::string&)> list = [&](const Exec* e, const std::string& indent) {
    size_t child = 0;
    for (auto& st : e->steps) {
      s += indent + st.desc + "\n";
      const bool owns_two = st.desc.compare(0, 6, "while[") == 0 || st.desc.compare(0, 3, "if[") == 0;
      for (int k = 0; owns_two && k < 2 && child < e->children.size(); ++k) list(e->children[child++].get(), indent + "    ");
    }
  };
  list(ex, "");
  if (buf && cap > 0) {
    const int64_t n = std::min<int64_t>(cap - 1, (int64_t)s.size());
    memcpy(buf, s.data(), (size_t)n);
    buf[n] = 0;
  }
  return (int64_t)s.size();
}

static bool execute_impl(B200Exec exec, const B200Buffer* inputs, int num_inputs, B200Buffer* outputs, int num_outputs,
                         std::vector<float>* step_ms, const unsigned char* donate, B200Error* err);

bool b200_execute(B200Exec exec, const B200Buffer* inputs, int num_inputs, B200Buffer* outputs, int num_outputs, B200Error* err) {
  return execute_impl(exec, inputs, num_inputs, outputs, num_outputs, nullptr, nullptr, err);
}

bool b200_execute_donating(B200Exec exec, const B200Buffer* inputs, const unsigned char* donate, int num_inputs, B200Buffer* outputs,
                           int num_outputs, B200Error* err) {
  return execute_impl(exec, inputs, num_inputs, outputs, num_outputs, nullptr, donate, err);
}

int64_t b200_execute_profiled(B200Exec exec, const B200Buffer* inputs, int num_inputs, B200Buffer* outputs, int num_outputs, char* report,
                              int64_t cap, B200Error* err) {
  std::vector<float> ms;
  if (!execute_impl(exec, inputs, num_inputs, outputs, num_outputs, &ms, nullptr, err)) return -1;
  Exec* ex = reinterpret_cast<Exec*>(exec);
  std::string s;
  double total = 0;
  for (float v : ms) total += v;
  for (size_t i = 0; i < ms.size(); ++i) s += strfmt("%9.4f ms  %5.1f%%  ", ms[i], total > 0 ? 100.0 * ms[i] / total : 0.0) + ex->steps[i].desc + "\n";
  s += strfmt("%9.4f ms  total of %d steps\n", total, (int)ms.size());
  if (report && cap > 0) {
    const int64_t n = std::min<int64_t>(cap - 1, (int64_t)s.size());
    memcpy(report, s.data(), (size_t)n);
    report[n] = 0;
  }
  return (int64_t)s.size();
}

static bool execute_impl(B200Exec exec, const B200Buffer* inputs, int num_inputs, B200Buffer* outputs, int num_outputs,
                         std::vector<float>* step_ms, const unsigned char* donate, B200Error* err) {
  clear_error(err);
  Exec* ex = reinterpret_cast<Exec*>(exec);
  if (!ex) { set_error(err, Status::Invalid("Execute: null executable")); return false; }
  if (num_inputs != (int)ex->inputs.size()) {
    set_error(err, Status::Invalid(strfmt("Execute: expected %d inputs, got %d", (int)ex->inputs.size(), num_inputs)));
    return false;
  }
  if (num_outputs != (int)ex->outputs.size()) {
    set_error(err, Status::Invalid(strfmt("Execute: expected %d outputs, got %d", (int)ex->outputs.size(), num_outputs)));
    return false;
  }
  std::lock_guard<std::mutex> lock(ex->mu);  // executions of one executable are serialised (ref executable.go:25, 51)
  std::vector<void*> ptrs(ex->slots.size(), nullptr);
  for (int i = 0; i < num_inputs; ++i) {
    Buffer* b = reinterpret_cast<Buffer*>(inputs[i]);
    const OutputDesc& d = ex->inputs[i];
    if (!b || !b->ptr) { set_error(err, Status::Invalid(strfmt("Execute: input %d is null or finalized", i))); return false; }
    if (b->device != ex->dev->ordinal()) { set_error(err, Status::Invalid(strfmt("Execute: input %d lives on device %d, executable on %d", i, b->device, ex->dev->ordinal()))); return false; }
    if (b->dtype != d.dtype || b->dims != d.dims) {
      set_error(err, Status::Invalid(strfmt("Execute: input %d shape mismatch (buffer %s, expected %s)", i, dtype_name(b->dtype), dtype_name(d.dtype))));
      return false;
    }
    ptrs[d.slot] = b->ptr;
  }
  std::vector<Buffer*> outs;
  std::vector<int> taken_from(num_outputs, -1);   // output j holds the block of donated input taken_from[j]
  auto fail = [&](const Status& s) {
    for (size_t j = 0; j < outs.size(); ++j) {
      if (taken_from[j] < 0) ex->dev->Free(outs[j]->ptr);   // a block taken from an input stays the input's on failure
      delete outs[j];
    }
    set_error(err, s);
    return false;
  };
  // On success donated inputs are finalized: the one an output took over loses its block to it, the others free theirs.
  auto consume_donated = [&]() {
    if (!donate) return;
    for (int i = 0; i < num_inputs; ++i) {
      if (!donate[i]) continue;
      bool dup = false;
      for (int k = 0; k < i; ++k) dup = dup || inputs[k] == inputs[i];
      if (dup) continue;
      Buffer* b = reinterpret_cast<Buffer*>(inputs[i]);
      bool taken = false;
      for (int j = 0; j < num_outputs; ++j) taken = taken || taken_from[j] == i;
      if (taken) b->ptr = nullptr;
      b200_buffer_free(inputs[i]);
    }
  };
  for (int i = 0; i < num_outputs; ++i) {
    const OutputDesc& d = ex->outputs[i];
    Buffer* b = new Buffer();
    b->device = ex->dev->ordinal();
    b->dtype = d.dtype;
    b->dims = d.dims;
    b->nbytes = d.nbytes;
    // a donated input this output may update in place: the output takes over the input's block
    const int alias = (donate && (size_t)i < ex->donate_alias.size()) ? ex->donate_alias[i] : -1;
    Buffer* src = alias >= 0 && donate[alias] ? reinterpret_cast<Buffer*>(inputs[alias]) : nullptr;
    if (src && src->owned && !src->ipc && src->nbytes == d.nbytes) {
      b->ptr = src->ptr;
      taken_from[i] = alias;
      outs.push_back(b);
      ptrs[d.slot] = b->ptr;
      continue;
    }
    Status s = ex->dev->Alloc(d.nbytes > 0 ? d.nbytes : 1, &b->ptr);
    outs.push_back(b);
    if (!s.ok()) return fail(s);
    ptrs[d.slot] = b->ptr;
  }
  for (size_t s = 0; s < ex->slots.size(); ++s) {
    const Slot& sl = ex->slots[s];
    if (sl.kind == SlotKind::Arena) ptrs[s] = (char*)ex->arena + sl.offset;
    else if (sl.kind == SlotKind::Const) ptrs[s] = ex->const_ptrs[sl.index];
  }
  if (!step_ms && ex->capturable) {
    std::vector<void*> key;
    for (int i = 0; i < num_inputs; ++i) key.push_back(reinterpret_cast<Buffer*>(inputs[i])->ptr);
    for (Buffer* b : outs) key.push_back(b->ptr);
    cudaStream_t stream = ex->dev->stream();
    PlanGraph* hit = nullptr;
    for (auto& g : ex->graphs)
      if (g.key == key) hit = &g;
    Status gs = ex->dev->MakeCurrent();
    if (!gs.ok()) return fail(gs);
    if (!hit && key == ex->last_key) {
      // second run on these addresses: record the plan instead of launching it.  The recording happens on a private
      // stream that only this thread sees as the device's stream, so work other threads enqueue on the compute stream
      // meanwhile stays out of it.
      cudaGraph_t graph = nullptr;
      cudaStream_t cs = nullptr;
      std::lock_guard<std::mutex> recording(ex->dev->capture_mutex());   // one capture stream per device
      cudaError_t ce = ex->dev->CaptureStream(&cs).ok() ? cudaSuccess : cudaErrorUnknown;
      if (ce == cudaSuccess) ce = cudaStreamBeginCapture(cs, cudaStreamCaptureModeThreadLocal);
      const bool began = ce == cudaSuccess;
      if (ce == cudaSuccess) {
        Status rs = Status::OK();
        {
          StreamOverride record_on(ex->dev, cs);
          for (auto& st : ex->steps) {
            rs = st.run(ex->dev, ptrs.data());
            if (!rs.ok()) { rs = Status{rs.code, st.desc + ": " + rs.msg}; break; }
          }
        }
        ce = cudaStreamEndCapture(cs, &graph);
        if (!rs.ok() && ce == cudaSuccess) ce = cudaErrorStreamCaptureInvalidated;   // a step refused to record: plain path below
        cudaGraphExec_t gexec = nullptr;
        if (ce == cudaSuccess) ce = cudaGraphInstantiate(&gexec, graph, 0);
        if (graph) cudaGraphDestroy(graph);
        if (ce == cudaSuccess) {
          if (ex->graphs.size() >= 4) {   // keep the four most recently used address sets
            size_t lru = 0;
            for (size_t i = 1; i < ex->graphs.size(); ++i)
              if (ex->graphs[i].last_used < ex->graphs[lru].last_used) lru = i;
            cudaGraphExecDestroy(ex->graphs[lru].exec);
            ex->graphs.erase(ex->graphs.begin() + (long)lru);
          }
          ex->graphs.push_back(PlanGraph{key, gexec, 0});
          hit = &ex->graphs.back();
        }
      }
      if (!hit) {
        cudaGetLastError();
        // A plan that began recording and did not finish cleanly runs step by step from now on (nothing was launched:
        // the plain path below runs it now and reports a real error if there is one).  A capture that could not even
        // begin says nothing about the plan: a later call tries again.
        if (began) ex->capturable = false;
      }
    }
    if (hit) {
      hit->last_used = ++ex->tick;
      ex->dev->kernel_error_flag();   // a replayed kernel can raise the error word too: have the next sync point read it
      cudaError_t ce = cudaGraphLaunch(hit->exec, stream);
      if (ce != cudaSuccess) {
        cudaGetLastError();
        return fail(Status::Cuda(strfmt("Execute: graph launch failed: %s", cudaGetErrorString(ce))));
      }
      for (int i = 0; i < num_outputs; ++i) outputs[i] = outs[i];
      consume_donated();
      return true;
    }
    ex->last_key = key;
  }
  std::vector<cudaEvent_t> events;
  if (step_ms) {
    events.resize(ex->steps.size() + 1);
    for (auto& e : events) cudaEventCreate(&e);
    cudaEventRecord(events[0], ex->dev->stream());
  }
  size_t si = 0;
  for (auto& st : ex->steps) {
    Status s = st.run(ex->dev, ptrs.data());
    if (!s.ok()) {
      for (auto& e : events) cudaEventDestroy(e);
      return fail(Status{s.code, st.desc + ": " + s.msg});
    }
    if (step_ms) cudaEventRecord(events[++si], ex->dev->stream());
  }
  if (step_ms) {
    cudaStreamSynchronize(ex->dev->stream());
    step_ms->resize(ex->steps.size());
    for (size_t i = 0; i < ex->steps.size(); ++i) cudaEventElapsedTime(&(*step_ms)[i], events[i], events[i + 1]);
    for (auto& e : events) cudaEventDestroy(e);
  }
  for (int i = 0; i < num_outputs; ++i) outputs[i] = outs[i];
  consume_donated();
  return true;
}

// Host arrays in, host arrays out, over `num_slices` consecutive leading-axis slices.  The executable is compiled for ONE slice.
// Three streams: the upload of slice s+1, the kernels of slice s and the download of slice s-1 run at the same time, each
// pair ordered by events; two sets of device buffers alternate.
bool b200_execute_host_sliced(B200Exec exec, void** input_data, const int* input_sliced, int num_inputs, void** output_data,
                              int num_outputs, int64_t num_slices, B200Error* err) {
  clear_error(err);
  Exec* ex = reinterpret_cast<Exec*>(exec);
  if (!ex) { set_error(err, Status::Invalid("ExecuteSliced: null executable")); return false; }
  if (num_inputs != (int)ex->inputs.size() || num_outputs != (int)ex->outputs.size()) {
    set_error(err, Status::Invalid(strfmt("ExecuteSliced: expected %d inputs and %d outputs, got %d and %d", (int)ex->inputs.size(),
                                          (int)ex->outputs.size(), num_inputs, num_outputs)));
    return false;
  }
  if (num_slices < 0) { set_error(err, Status::Invalid("ExecuteSliced: negative slice count")); return false; }
  for (int i = 0; i < num_inputs; ++i)
    if (!input_data[i] && ex->inputs[i].nbytes > 0) { set_error(err, Status::Invalid(strfmt("ExecuteSliced: input %d is null", i))); return false; }
  for (int i = 0; i < num_outputs; ++i)
    if (!output_data[i] && ex->outputs[i].nbytes > 0 && num_slices > 0) { set_error(err, Status::Invalid(strfmt("ExecuteSliced: output %d is null", i))); return false; }
  if (num_slices == 0) return true;
  std::lock_guard<std::mutex> lock(ex->mu);
  Device* dev = ex->dev;
  Status st = dev->MakeCurrent();
  cudaStream_t s_in = nullptr, s_out = nullptr;
  if (st.ok()) st = dev->CopyStreams(&s_in, &s_out);
  if (!st.ok()) { set_error(err, st); return false; }
  const cudaStream_t s_main = dev->stream();

  constexpr int kSets = 2;
  std::vector<void*> owned;  // every device block of this call
  std::vector<void*> in_ptr[kSets], out_ptr[kSets];
  cudaEvent_t ev_in[kSets] = {}, ev_done[kSets] = {}, ev_out[kSets] = {}, ev_start = nullptr;
  auto release = [&]() {
    for (void* p : owned) dev->Free(p);
    for (int k = 0; k < kSets; ++k) {
      if (ev_in[k]) cudaEventDestroy(ev_in[k]);
      if (ev_done[k]) cudaEventDestroy(ev_done[k]);
      if (ev_out[k]) cudaEventDestroy(ev_out[k]);
    }
    if (ev_start) cudaEventDestroy(ev_start);
  };
  auto fail = [&](const Status& s) {
    cudaStreamSynchronize(s_in);
    cudaStreamSynchronize(s_main);
    cudaStreamSynchronize(s_out);
    release();
    set_error(err, s);
    return false;
  };
#define B200_SLICED_TRY(expr)                                                                  \
  do {                                                                                         \
    cudaError_t e_ = (expr);                                                                   \
    if (e_ != cudaSuccess) return fail(Status::Cuda(strfmt("%s: %s", #expr, cudaGetErrorString(e_)))); \
  } while (0)

  const int sets = (int)std::min<int64_t>(kSets, num_slices);
  for (int k = 0; k < kSets; ++k) { in_ptr[k].assign(num_inputs, nullptr); out_ptr[k].assign(num_outputs, nullptr); }
  for (int i = 0; i < num_inputs; ++i) {
    const int copies = input_sliced && input_sliced[i] ? sets : 1;
    for (int k = 0; k < copies; ++k) {
      void* p = nullptr;
      st = dev->Alloc(std::max<int64_t>(ex->inputs[i].nbytes, 1), &p);
      if (!st.ok()) return fail(st);
      owned.push_back(p);
      in_ptr[k][i] = p;
    }
    for (int k = copies; k < kSets; ++k) in_ptr[k][i] = in_ptr[0][i];
  }
  for (int i = 0; i < num_outputs; ++i)
    for (int k = 0; k < sets; ++k) {
      void* p = nullptr;
      st = dev->Alloc(std::max<int64_t>(ex->outputs[i].nbytes, 1), &p);
      if (!st.ok()) return fail(st);
      owned.push_back(p);
      out_ptr[k][i] = p;
    }
  for (int k = 0; k < kSets; ++k) {
    B200_SLICED_TRY(cudaEventCreateWithFlags(&ev_in[k], cudaEventDisableTiming));
    B200_SLICED_TRY(cudaEventCreateWithFlags(&ev_done[k], cudaEventDisableTiming));
    B200_SLICED_TRY(cudaEventCreateWithFlags(&ev_out[k], cudaEventDisableTiming));
  }
  B200_SLICED_TRY(cudaEventCreateWithFlags(&ev_start, cudaEventDisableTiming));
  // The blocks above may have been freed by earlier work on the compute stream: the copy streams start after it.
  B200_SLICED_TRY(cudaEventRecord(ev_start, s_main));
  B200_SLICED_TRY(cudaStreamWaitEvent(s_in, ev_start, 0));
  B200_SLICED_TRY(cudaStreamWaitEvent(s_out, ev_start, 0));
  // Inputs shared by every slice (weights, tables) go up once, ahead of slice 0.
  for (int i = 0; i < num_inputs; ++i)
    if (!(input_sliced && input_sliced[i]) && ex->inputs[i].nbytes > 0)
      B200_SLICED_TRY(cudaMemcpyAsync(in_ptr[0][i], input_data[i], (size_t)ex->inputs[i].nbytes, cudaMemcpyHostToDevice, s_in));

  std::vector<void*> ptrs(ex->slots.size(), nullptr);
  for (size_t s = 0; s < ex->slots.size(); ++s) {
    const Slot& sl = ex->slots[s];
    if (sl.kind == SlotKind::Arena) ptrs[s] = (char*)ex->arena + sl.offset;
    else if (sl.kind == SlotKind::Const) ptrs[s] = ex->const_ptrs[sl.index];
  }
  for (int64_t sl = 0; sl < num_slices; ++sl) {
    const int k = (int)(sl % kSets);
    // upload: the set's previous kernels (slice sl - 2) must have finished reading it
    if (sl >= kSets) B200_SLICED_TRY(cudaStreamWaitEvent(s_in, ev_done[k], 0));
    for (int i = 0; i < num_inputs; ++i)
      if (input_sliced && input_sliced[i] && ex->inputs[i].nbytes > 0)
        B200_SLICED_TRY(cudaMemcpyAsync(in_ptr[k][i], (const char*)input_data[i] + sl * ex->inputs[i].nbytes, (size_t)ex->inputs[i].nbytes,
                                        cudaMemcpyHostToDevice, s_in));
    B200_SLICED_TRY(cudaEventRecord(ev_in[k], s_in));
    // kernels: after the upload, and after the download of slice sl - 2 has drained the set's outputs
    B200_SLICED_TRY(cudaStreamWaitEvent(s_main, ev_in[k], 0));
    if (sl >= kSets) B200_SLICED_TRY(cudaStreamWaitEvent(s_main, ev_out[k], 0));
    for (int i = 0; i < num_inputs; ++i) ptrs[ex->inputs[i].slot] = in_ptr[k][i];
    for (int i = 0; i < num_outputs; ++i) ptrs[ex->outputs[i].slot] = out_ptr[k][i];
    for (auto& step : ex->steps) {
      Status s = step.run(dev, ptrs.data());
      if (!s.ok()) return fail(Status{s.code, step.desc + ": " + s.msg});
    }
    B200_SLICED_TRY(cudaEventRecord(ev_done[k], s_main));
    // download
    B200_SLICED_TRY(cudaStreamWaitEvent(s_out, ev_done[k], 0));
    for (int i = 0; i < num_outputs; ++i)
      if (ex->outputs[i].nbytes > 0)
        B200_SLICED_TRY(cudaMemcpyAsync((char*)output_data[i] + sl * ex->outputs[i].nbytes, out_ptr[k][i], (size_t)ex->outputs[i].nbytes,
                                        cudaMemcpyDeviceToHost, s_out));
    B200_SLICED_TRY(cudaEventRecord(ev_out[k], s_out));
  }
  // Join: the compute stream waits for both copy streams so that the blocks can go back to the stream-ordered allocator.
  for (int k = 0; k < sets; ++k) {
    B200_SLICED_TRY(cudaStreamWaitEvent(s_main, ev_in[k], 0));
    B200_SLICED_TRY(cudaStreamWaitEvent(s_main, ev_out[k], 0));
  }
  B200_SLICED_TRY(cudaStreamSynchronize(s_out));
  st = dev->Synchronize();
  if (!st.ok()) return fail(st);
#undef B200_SLICED_TRY
  release();
  return true;
}

}  // extern "C"
