// Launchers of the sm_100a kernels.  Each takes raw device pointers, enqueues on
// the Device's stream and returns a Status; none allocates or synchronises.
#pragma once

#include "common.h"

namespace b200 {
namespace k {

constexpr int kMaxDims = 8;

// ------------------------------------------------------------- softmax -----
struct SoftmaxParams {
  const void* x = nullptr;
  void* y = nullptr;
  int64_t rows = 0, cols = 0;
  int dtype = B200_FLOAT32;
  double scale = 1.0;
  bool causal = false;
  int64_t seq_q = 0;  // rows = batch * heads * seq_q; 0 means rows
  int64_t heads = 1;
  const void* mask = nullptr;
  int mask_kind = 0;                          // 1 bool, 2 float (dtype of x)
  int64_t mask_strides[4] = {0, 0, 0, 0};     // batch, head, q, k (elements)
};
Status softmax_rows(Device* dev, const SoftmaxParams& p);
Status softmax_strided(Device* dev, const void* x, void* y, int64_t outer, int64_t n, int64_t inner, int dtype);

// ---------------------------------------------------------------- norms ----
struct NormParams {
  const void* x = nullptr;
  const void* gamma = nullptr;  // [cols] of x's dtype, or null
  const void* beta = nullptr;   // [cols] of x's dtype, or null (LayerNorm only)
  void* y = nullptr;
  int64_t rows = 0, cols = 0;
  int dtype = B200_FLOAT32;
  double epsilon = 1e-5;
  bool rms = false;
};
Status norm_rows(Device* dev, const NormParams& p);

// ---------------------------------------------- fused elementwise chains ---
// A straight-line program over virtual registers, evaluated per output element
// by one interpreter kernel.  Leaves are loads from dense tensors addressed
// through broadcast strides of the OUTPUT index space, iotas, or immediates.
constexpr int kEwMaxInstr = 48;
constexpr int kEwMaxLeaves = 8;
constexpr int kEwMaxRegs = 24;

enum EwKind : uint8_t { EW_LOAD = 0, EW_IMM = 1, EW_IOTA = 2, EW_OP = 3, EW_CAST = 4 };

struct EwInstr {
  uint8_t kind;   // EwKind
  uint8_t op;     // b200::Op value for EW_OP
  uint8_t dtype;  // dtype of the RESULT (for EW_OP: compares produce Bool but compute in src dtype, see sdtype)
  uint8_t sdtype; // dtype of the operands (EW_OP, EW_CAST)
  uint8_t dst, a, b, c;  // register numbers; for EW_LOAD a = leaf index; for EW_IOTA a = output dim
  uint64_t imm;   // EW_IMM: raw bits of the value already in register representation
};

struct EwLeaf {
  const void* ptr;
  int64_t strides[kMaxDims];  // per OUTPUT dim, in elements; 0 = broadcast
  int dtype;
};

struct EwProgram {
  int num_instr = 0;
  int num_leaves = 0;
  int num_regs = 0;
  int rank = 0;                 // collapsed output rank (<= kMaxDims)
  int64_t dims[kMaxDims] = {0};  // output dims
  EwInstr instr[kEwMaxInstr];
  EwLeaf leaves[kEwMaxLeaves];
  int out_reg = 0;
  int out_dtype = B200_FLOAT32;
  void* out = nullptr;
  bool wide = false;  // needs 64-bit registers (any I64/U64/F64 value)
};
Status ewise_run(Device* dev, const EwProgram& prog);
// The templated fast shapes of ewise_run alone: x op y, and (with trees = true) the small expression trees.  *taken says
// whether one of them was launched.
Status ewise_run_fast(Device* dev, const EwProgram& prog, bool* taken, bool trees = true);

// Run-time compiled form of a program (ewise_jit.cu): one straight-line kernel per distinct program text, built with
// NVRTC at plan time and cached for the life of the process.  ewise_jit_prepare fails with B200_ERR_UNSUPPORTED when
// NVRTC is not installed (the interpreter kernel of ewise_run then does the work).  The handle is never freed.
struct EwJit;
Status ewise_jit_prepare(Device* dev, const EwProgram& prog, EwJit** out);
Status ewise_jit_run(Device* dev, EwJit* jit, const EwProgram& prog);   // prog: the same program with its pointers filled in
bool ewise_jit_available(std::string* why);
// The same for a reduction (B200ReduceType) whose operand is the program: the program's index space is viewed as
// [outer, n, inner] (its dims must refine that split) and folded over n in one pass, so the chain's value is never
// written to memory.  prog.out_dtype is the dtype of the chain's value and of the result; prog.out receives
// [outer, inner].  Fails with B200_ERR_UNSUPPORTED when the shape would need a split across CTAs (ewise_jit_reduce_fits).
bool ewise_jit_reduce_fits(int64_t outer, int64_t n, int64_t inner, int sm_count);
Status ewise_jit_reduce_prepare(Device* dev, const EwProgram& prog, int reduce_type, int64_t outer, int64_t n, int64_t inner, EwJit** out);
std::string ewise_jit_reduce_source(const EwProgram& prog, int reduce_type, int64_t outer, int64_t n, int64_t inner, bool allow_vector);
// The generated CUDA C text and its compilation, separately (tests and tools).
std::string ewise_jit_source(const EwProgram& prog, int sm_count, bool allow_vector);
Status ewise_jit_nvrtc(const std::string& source, std::vector<char>* cubin);

// ---------------------------------------------------------- data movement --
// y[idx] = x[offset + sum_d idx_d * strides_d] over a dense row-major output.
// Covers Transpose, Slice, Reverse, BroadcastInDim (stride 0) and
// Concatenate / Pad (through out_offset and out_strides).
struct StridedCopyParams {
  const void* x = nullptr;
  void* y = nullptr;
  int elt_size = 4;
  int rank = 0;
  int64_t dims[kMaxDims] = {0};
  int64_t in_strides[kMaxDims] = {0};   // elements, may be 0 or negative
  int64_t in_offset = 0;                // elements
  int64_t out_strides[kMaxDims] = {0};  // elements
  int64_t out_offset = 0;
};
Status strided_copy(Device* dev, const StridedCopyParams& p);
// Batched 2-D transpose through shared memory: x[batch, rows, cols] -> y[batch, cols, rows].
Status transpose_2d(Device* dev, const void* x, void* y, int64_t batch, int64_t rows, int64_t cols, int elt_size);
// Slices whose start indices live in device memory (one integer scalar per axis, any integer dtype), clamped so the
// block fits.  dynamic_slice: y[block dims] = x[start + idx].  dynamic_update_slice: y = x with the block `u` written at
// start (one pass: every element of y comes from u or from x).
struct DynSliceParams {
  const void* x = nullptr;       // operand [x_dims]
  const void* u = nullptr;       // update block [b_dims] (update only)
  void* y = nullptr;
  int elt_size = 4;
  int rank = 0;
  int64_t x_dims[kMaxDims] = {0};
  int64_t b_dims[kMaxDims] = {0};  // slice sizes / update dims
  const void* starts[kMaxDims] = {nullptr};
  int start_dtypes[kMaxDims] = {0};
  // update only: element strides of the update block when it is read in place inside a larger tensor (dense otherwise)
  bool u_strided = false;
  int64_t u_strides[kMaxDims] = {0};
};
Status dynamic_slice(Device* dev, const DynSliceParams& p);
Status dynamic_update_slice(Device* dev, const DynSliceParams& p);
// The same when y already holds x (y == x): only the block is written.
Status dynamic_update_slice_inplace(Device* dev, const DynSliceParams& p);
// Two of them with the same block geometry and element size (a layer's key and value caches) in ONE launch.
Status dynamic_update_slice_inplace2(Device* dev, const DynSliceParams& p0, const DynSliceParams& p1);

// Up to 8 contiguous arrays laid end to end into y with ONE launch (small concatenations are launch-bound: a fused QKV
// projection joins three bias vectors per layer).  counts are in elements.
constexpr int kMaxConcatFlat = 8;
Status concat_flat(Device* dev, const void* const* src, const int64_t* counts, int n, void* y, int elt_size);
Status fill(Device* dev, void* y, int64_t n, int elt_size, uint64_t pattern);
// Packs rows of `cols` elements stored with a pitch of `src_pitch` elements into a dense [rows, cols] array, writing
// whole 16-byte vectors of the destination whatever the alignment of its rows.
Status unpad_rows(Device* dev, const void* src, void* dst, int64_t rows, int64_t cols, int64_t src_pitch, int elt_size);
Status iota(Device* dev, void* y, int dtype, int64_t outer, int64_t n, int64_t inner);
Status cast(Device* dev, const void* x, int src_dtype, void* y, int dst_dtype, int64_t n);

// ------------------------------------------------------------ reductions ---
// x viewed as [outer, n, inner] -> y[outer, inner].  Floats accumulate in fp32
// (f64 in f64), integers in their own width.
Status reduce(Device* dev, const void* x, void* y, int dtype, int reduce_type, int64_t outer, int64_t n,
              int64_t inner, void* scratch, int64_t scratch_bytes);
int64_t reduce_scratch_bytes(int dtype, int64_t outer, int64_t n, int64_t inner);
Status arg_min_max(Device* dev, const void* x, void* y, int dtype, int out_dtype, bool is_min, int64_t outer,
                   int64_t n, int64_t inner);

// ---------------------------------------------------------------- gather ---
// Row gather (embedding lookup): y[i, :] = table[clamp(ids[i]), :], rows of row_bytes bytes.
Status gather_rows(Device* dev, const void* table, const void* ids, int ids_dtype, void* y, int64_t num_ids,
                   int64_t num_rows, int64_t row_bytes);
// General XLA gather, one thread per output element.
struct GatherParams {
  const void* operand = nullptr;
  const void* indices = nullptr;
  void* y = nullptr;
  int elt_size = 4;
  int ids_dtype = B200_INT32;
  int out_rank = 0;
  int64_t out_dims[kMaxDims] = {0};
  int operand_rank = 0;
  int64_t operand_dims[kMaxDims] = {0};
  int64_t operand_strides[kMaxDims] = {0};
  int64_t slice_sizes[kMaxDims] = {0};
  // For every output dim: if it is an offset dim, offset_operand_axis >= 0 names the operand axis it walks;
  // else batch_pos names which batch (index) coordinate it is.
  int out_offset_operand_axis[kMaxDims];
  int out_batch_pos[kMaxDims];
  int num_batch_dims = 0;
  int64_t batch_index_strides[kMaxDims] = {0};  // strides of the indices tensor for each batch coordinate
  int64_t index_vector_stride = 0;              // stride along index_vector_axis
  int num_index_components = 0;
  int start_index_map[kMaxDims];
};
Status gather_general(Device* dev, const GatherParams& p);

// --------------------------------------------------------------- scatter ---
// XLA scatter with a combiner (mode 0 sum, 1 max, 2 min): y must already hold a copy of the operand; one thread per
// element of `updates` combines it into the operand position its scatter indices name, out-of-range elements are dropped.
struct ScatterParams {
  void* y = nullptr;              // operand-shaped, pre-filled with the operand
  const void* indices = nullptr;
  const void* updates = nullptr;
  int dtype = B200_FLOAT32;
  int ids_dtype = B200_INT32;
  int mode = 0;
  int operand_rank = 0;
  int64_t operand_dims[kMaxDims] = {0};
  int64_t operand_strides[kMaxDims] = {0};
  int update_rank = 0;
  int64_t update_dims[kMaxDims] = {0};
  int num_batch_dims = 0;                          // update axes that are scatter (batch) axes, in order
  int batch_update_axis[kMaxDims];
  int64_t batch_index_strides[kMaxDims] = {0};     // strides of the indices tensor for each batch coordinate
  int64_t index_vector_stride = 0;
  int num_index_components = 0;
  int scatter_axes_to_operand_axes[kMaxDims];
  int num_window_axes = 0;                         // update window axis j walks operand axis window_operand_axis[j]
  int window_update_axis[kMaxDims];
  int window_operand_axis[kMaxDims];
};
Status scatter(Device* dev, const ScatterParams& p);

// ------------------------------------------------------------------ sort ---
// out (int32, x's shape) = the stable permutation that sorts x, viewed as [outer, n, inner], along n; NaN keys last.
// Rows longer than 4096 keys need arg_sort_scratch_bytes of scratch.
int64_t arg_sort_scratch_bytes(int64_t outer, int64_t n, int64_t inner, int sm_count);
Status arg_sort(Device* dev, const void* x, void* out, int dtype, int64_t outer, int64_t n, int64_t inner, bool descending, void* scratch,
                int64_t scratch_bytes);

// ------------------------------------------------------------------- RNG ---
// n elements of `dtype` from Philox4x32-10 keyed and positioned by the [3] Uint64 state in device memory.
Status rng_bits(Device* dev, const void* state, void* y, int dtype, int64_t n);

// ------------------------------------------------------------------ GEMM ---
struct GemmParams {
  const void* a = nullptr;
  const void* b = nullptr;
  void* c = nullptr;
  int64_t batch = 1, m = 0, n = 0, k = 0;
  bool a_k_major = true;   // A is [batch, M, K] (true) or [batch, K, M]
  bool b_k_major = false;  // B is [batch, N, K] (true) or [batch, K, N]
  int dtype = B200_BFLOAT16;
  const void* bias = nullptr;  // [N] of dtype, or null
  int activation = B200_ACT_NONE;
  // [batch, M, N] of dtype or null: C = round(act(A B + bias)) + residual, rounded again (the op-by-op result of a
  // DotGeneral followed by Add, without the extra pass over C)
  const void* residual = nullptr;
  int residual_op = 0;   // 0: + residual, 1: * residual (a gated MLP's act(x W1) * (x W2))
  // Row pitch of C (and of the residual) in elements; 0 = n.  A pitch rounded up to 16 bytes lets a ragged N use the
  // vector epilogue: the columns between n and the pitch are written with don't-care values.
  int64_t ldc = 0;
  // Further copies of C (same pitch and shape): the epilogue stores every tile to each of them as well.  They may be
  // peer-device memory; only the tensor-core kernels honour them and only with vector stores (gemm_tcgen05 refuses otherwise).
  static constexpr int kMaxExtraC = 7;
  void* c_extra[kMaxExtraC] = {nullptr};
  int num_c_extra = 0;
  // batch strides in elements; 0 on an operand broadcasts it over the batch
  int64_t a_batch_stride = -1, b_batch_stride = -1;  // -1 = dense (m*k, k*n)
  // fp32 on the tensor-core path: room for the three bf16 planes of both operands (gemm_split_scratch_bytes).  Without
  // it the launch allocates them itself, which keeps the step out of recorded plans.
  // A 16-bit product of at most 64 rows (gemm_skinny): split_scratch holds the K slices' fp32 partial sums
  // (gemm_skinny_scratch_bytes) and skinny_counters one zeroed 32-bit counter per 64 columns (gemm_skinny_counter_bytes),
  // which the kernel leaves at zero.  Counters must not be shared by launches that may run at the same time.
  void* split_scratch = nullptr;
  int64_t split_scratch_bytes = 0;
  void* skinny_counters = nullptr;
  // gemm_skinny only: a second weight of B's shape and layout; C = round(act(A B + bias)) * round(A B2), rounded again
  // (a gated MLP in one launch).  Set only where gemm_skinny_dual_ok() holds; without a residual.
  const void* b2 = nullptr;
  // gemm_skinny only (where gemm_skinny_dual_ok() holds): A is the INPUT of an RMSNorm over K with this gain [K] and
  // epsilon, and the product is taken of the norm's output -- the norm costs no launch of its own.
  const void* rms_gamma = nullptr;
  double rms_eps = 0;
  // B is not written by anything that may still be running when this launch starts (a plan input or constant): a
  // kernel launched as a programmatic dependent may then fetch it before the previous kernel has finished.
  bool b_static = false;
};
int64_t gemm_skinny_scratch_bytes(const GemmParams& p, int sm_count);   // 0: not a shape gemm_skinny takes
int64_t gemm_skinny_counter_bytes(const GemmParams& p);
bool gemm_skinny_dual_ok(const GemmParams& p);
// The few-rows path alone: *taken is false (and nothing is launched) when the problem is outside its rules or has no scratch.
Status gemm_skinny(Device* dev, const GemmParams& p, bool* taken);
inline int64_t gemm_split_scratch_bytes(int64_t batch, int64_t m, int64_t n, int64_t k) {
  const int64_t a = (batch * m * k * 6 + 255) / 256 * 256, b = (batch * k * n * 6 + 255) / 256 * 256;
  return a + b;
}
Status gemm(Device* dev, const GemmParams& p);
// The tensor-core path alone: *taken is false (and nothing is launched) when the problem is outside its rules.
Status gemm_tcgen05(Device* dev, const GemmParams& p, bool* taken);
// True when the tensor-core path writes this dense 16-bit result, whose rows are not a whole number of 16-byte vectors,
// with aligned vector stores all the same (pointers aside: shapes, majors and what is fused decide).
bool gemm_tcgen05_ragged_rows(const GemmParams& p, bool has_bias, bool has_residual);

// ------------------------------------------------------------------ rope ---
// y[r, j] = round(round(x[r, j] * c[r, j]) + round(x[r, j ^ half] * s[r, j])) over rows of `cols` elements made of heads of
// `head_dim`: j ^ half swaps the halves of each head.  x may live inside a wider buffer (row pitch x_pitch elements);
// c and s repeat with a period of c_period / s_period elements (a table shared by every batch entry); y is dense.
struct RopeParams {
  const void* x = nullptr;
  const void* c = nullptr;
  const void* s = nullptr;
  void* y = nullptr;
  int64_t rows = 0, cols = 0, head_dim = 0;
  int64_t x_pitch = 0;
  int64_t c_period = 0, s_period = 0;
  // A table shared by every head: it holds [period / head_dim, head_dim] and element (row, col) of x reads
  // table[(row mod (period / head_dim)) * head_dim + col mod head_dim].  Otherwise the table is indexed by the flat element
  // number of x modulo its period.
  bool c_per_head = false, s_per_head = false;
  int dtype = B200_BFLOAT16;
};
Status rope(Device* dev, const RopeParams& p);

// ------------------------------------------------------------- attention ---
// softmax(scale * Q K^T [+ causal mask]) V for Q [B, Sq, H, D] / K, V [B, Sk, Hkv, D] (bshd) or [B, H, Sq, D] (bhsd);
// O has Q's layout.  Query head h reads KV head h / (H / Hkv).
struct AttentionParams {
  const void* q = nullptr;
  const void* k = nullptr;
  const void* v = nullptr;
  void* o = nullptr;
  int64_t B = 0, H = 0, Hkv = 0, Sq = 0, Sk = 0, head_dim = 0;
  bool bshd = true;
  bool causal = false;
  double scale = 1.0;
  int dtype = B200_BFLOAT16;
  // Optional element strides (batch, head, sequence) per input; 0 = dense in the stated layout.  Lets Q, K and V be
  // read straight out of a wider buffer, e.g. the three column blocks of a fused QKV projection.
  int64_t q_strides[3] = {0, 0, 0}, k_strides[3] = {0, 0, 0}, v_strides[3] = {0, 0, 0};
  // One query position only (attention_decode): an optional mask over [batch, head, key], Bool (1: false = masked) or
  // additive in the tensors' dtype (2), with its element strides (0 on a broadcast dim).
  const void* mask = nullptr;
  int mask_kind = 0;
  int64_t m_b = 0, m_h = 0, m_k = 0;
};
bool attention_supported(const AttentionParams& p);
Status attention(Device* dev, const AttentionParams& p);
// One query position per (batch, head) against a key / value cache (Sq == 1, not causal): one bandwidth-bound launch.
bool attention_decode_supported(const AttentionParams& p);
Status attention_decode(Device* dev, const AttentionParams& p);

}  // namespace k
}  // namespace b200
