/*
 * b200mlx.h -- C ABI of the B200-native GoMLX backend library (libb200mlx.so).
 *
 * This header plays the role that mpsgraph/gomlx/internal/bridge/bridge.h plays
 * in the reference (gomlx/go-darwinml): opaque context / value / executable /
 * buffer handles, one graph-building function per op, compile, execute, buffer
 * I/O, and a {code, message} error struct as the last parameter of every
 * fallible call.  Citations "ref:" below are file:line inside the reference
 * project; they name the interface each declaration replaces.
 *
 * Conventions (same as ref bridge.h:16-20, bridge.m:46-58):
 *   - Every fallible call takes a trailing B200Error*.  It is cleared on entry.
 *     On failure the call returns NULL / false / -1, sets code != 0 and sets
 *     message to a malloc'd string that the CALLER frees with free().
 *   - Value handles (B200Value) are non-owning: they stay valid while the
 *     context that made them lives (ref bridge.h:12).
 *   - No call keeps a caller pointer after it returns (cgo rule; ref
 *     bridge.go:772-789, 852-895).
 *   - Plain C types only.  No CUDA, C++ or framework type appears here.
 *
 * There is no CPU fallback: with no usable GPU every device call fails with
 * B200_ERR_CUDA.
 */
#ifndef B200MLX_H
#define B200MLX_H

#include <stdbool.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- handles (ref bridge.h:11-14) ------------------------------------- */
typedef void* B200Context; /* one graph under construction + its device     */
typedef void* B200Value;   /* a node of that graph (non-owning)              */
typedef void* B200Exec;    /* a compiled launch plan                         */
typedef void* B200Buffer;  /* a device allocation with dtype and dims        */

/* ---- errors (ref bridge.h:16-20) -------------------------------------- */
typedef struct {
  int code;            /* 0 = ok, else one of B200ErrCode                    */
  const char* message; /* malloc'd; caller frees                             */
} B200Error;

typedef enum {
  B200_OK = 0,
  B200_ERR_INVALID = 1, /* bad handle, shape, axis, dtype ...                */
  B200_ERR_CUDA = 2,    /* a CUDA runtime/driver call failed                 */
  B200_ERR_UNSUPPORTED = 3,
  B200_ERR_OOM = 4,
  B200_ERR_TIMEOUT = 5, /* a bounded device-side wait gave up                */
} B200ErrCode;

/* ---- dtypes: numeric values kept from ref bridge.h:23-37 so that the Go
 * side's dtypeToBridgeDType (ref buffer.go:90-119) carries over ---------- */
typedef enum {
  B200_BOOL = 0,
  B200_INT8 = 1,
  B200_INT16 = 2,
  B200_INT32 = 3,
  B200_INT64 = 4,
  B200_FLOAT16 = 5,
  B200_BFLOAT16 = 6,
  B200_FLOAT32 = 7,
  B200_FLOAT64 = 8,
  B200_UINT8 = 9,
  B200_UINT16 = 10,
  B200_UINT32 = 11,
  B200_UINT64 = 12,
} B200DType;

/* ref bridge.h:40-45 */
typedef enum {
  B200_REDUCE_SUM = 0,
  B200_REDUCE_PRODUCT = 1,
  B200_REDUCE_MAX = 2,
  B200_REDUCE_MIN = 3,
} B200ReduceType;

/* Activation fused into b200_dense (ref function.go:2624-2664:
 * backends.ActivationNone/Gelu/Relu/Silu/Tanh; Gelu is the tanh form). */
typedef enum {
  B200_ACT_NONE = 0,
  B200_ACT_GELU = 1,
  B200_ACT_RELU = 2,
  B200_ACT_SILU = 3,
  B200_ACT_TANH = 4,
} B200Activation;

/* Attention axes layout (ref function.go:2699: backends.AxesLayoutBSHD / BHSD) */
typedef enum {
  B200_LAYOUT_BHSD = 0,
  B200_LAYOUT_BSHD = 1,
} B200AxesLayout;

/* ---- library / device -------------------------------------------------- */
const char* b200_version(void); /* static string */
/* Number of CUDA devices visible, or -1 with error (ref backend.go:56-57 NumDevices). */
int b200_device_count(B200Error* err);

/* ---- context lifecycle (ref bridge.h:48-52) ----------------------------
 * A context is one graph builder bound to one device (ref backend.go:70-77
 * makes a fresh native context per Builder). */
B200Context b200_create_context(int device, B200Error* err);
void b200_destroy_context(B200Context ctx);
const char* b200_device_name(B200Context ctx); /* malloc'd, caller frees (ref bridge.h:52) */
int b200_context_device(B200Context ctx);

/* ---- leaves (ref bridge.h:55-60) --------------------------------------- */
B200Value b200_placeholder(B200Context ctx, int dtype, const int64_t* shape, int rank, B200Error* err);
/* Copies nbytes of data (ref bridge.m:217-235). */
B200Value b200_constant(B200Context ctx, const void* data, int64_t nbytes, int dtype,
                        const int64_t* shape, int rank, B200Error* err);
B200Value b200_iota(B200Context ctx, int dtype, const int64_t* shape, int rank, int axis, B200Error* err);

/* ---- value introspection (ref builder.go:63-70 OpShape) ----------------- */
int b200_value_dtype(B200Value v);
int b200_value_rank(B200Value v);
/* Writes up to cap dims; returns rank. */
int b200_value_shape(B200Value v, int64_t* dims, int cap);

/* ---- unary ops (ref bridge.h:63-84) ------------------------------------ */
B200Value b200_abs(B200Context ctx, B200Value x, B200Error* err);
B200Value b200_neg(B200Context ctx, B200Value x, B200Error* err);
B200Value b200_sqrt(B200Context ctx, B200Value x, B200Error* err);
B200Value b200_rsqrt(B200Context ctx, B200Value x, B200Error* err);
B200Value b200_exp(B200Context ctx, B200Value x, B200Error* err);
B200Value b200_expm1(B200Context ctx, B200Value x, B200Error* err);
B200Value b200_log(B200Context ctx, B200Value x, B200Error* err);
B200Value b200_log1p(B200Context ctx, B200Value x, B200Error* err);
B200Value b200_sin(B200Context ctx, B200Value x, B200Error* err);
B200Value b200_cos(B200Context ctx, B200Value x, B200Error* err);
B200Value b200_tanh(B200Context ctx, B200Value x, B200Error* err);
B200Value b200_sigmoid(B200Context ctx, B200Value x, B200Error* err);
B200Value b200_erf(B200Context ctx, B200Value x, B200Error* err);
B200Value b200_floor(B200Context ctx, B200Value x, B200Error* err);
B200Value b200_ceil(B200Context ctx, B200Value x, B200Error* err);
B200Value b200_round(B200Context ctx, B200Value x, B200Error* err); /* ties to even (ref bridge.m:293) */
B200Value b200_sign(B200Context ctx, B200Value x, B200Error* err);
B200Value b200_logical_not(B200Context ctx, B200Value x, B200Error* err);
B200Value b200_bitwise_not(B200Context ctx, B200Value x, B200Error* err);
B200Value b200_is_finite(B200Context ctx, B200Value x, B200Error* err);
B200Value b200_is_nan(B200Context ctx, B200Value x, B200Error* err);
B200Value b200_identity(B200Context ctx, B200Value x, B200Error* err);

/* ---- binary ops with NumPy-style broadcasting (ref bridge.h:87-103) ----- */
B200Value b200_add(B200Context ctx, B200Value lhs, B200Value rhs, B200Error* err);
B200Value b200_sub(B200Context ctx, B200Value lhs, B200Value rhs, B200Error* err);
B200Value b200_mul(B200Context ctx, B200Value lhs, B200Value rhs, B200Error* err);
B200Value b200_div(B200Context ctx, B200Value lhs, B200Value rhs, B200Error* err);
B200Value b200_rem(B200Context ctx, B200Value lhs, B200Value rhs, B200Error* err); /* truncated (C fmod) */
B200Value b200_pow(B200Context ctx, B200Value lhs, B200Value rhs, B200Error* err);
B200Value b200_max(B200Context ctx, B200Value lhs, B200Value rhs, B200Error* err);
B200Value b200_min(B200Context ctx, B200Value lhs, B200Value rhs, B200Error* err);
B200Value b200_atan2(B200Context ctx, B200Value lhs, B200Value rhs, B200Error* err);
B200Value b200_logical_and(B200Context ctx, B200Value lhs, B200Value rhs, B200Error* err);
B200Value b200_logical_or(B200Context ctx, B200Value lhs, B200Value rhs, B200Error* err);
B200Value b200_logical_xor(B200Context ctx, B200Value lhs, B200Value rhs, B200Error* err);
B200Value b200_bitwise_and(B200Context ctx, B200Value lhs, B200Value rhs, B200Error* err);
B200Value b200_bitwise_or(B200Context ctx, B200Value lhs, B200Value rhs, B200Error* err);
B200Value b200_bitwise_xor(B200Context ctx, B200Value lhs, B200Value rhs, B200Error* err);
B200Value b200_shift_left(B200Context ctx, B200Value lhs, B200Value rhs, B200Error* err);
B200Value b200_shift_right(B200Context ctx, B200Value lhs, B200Value rhs, B200Error* err); /* arithmetic for signed */
B200Value b200_shift_right_logical(B200Context ctx, B200Value lhs, B200Value rhs, B200Error* err); /* ref function.go ShiftRightLogical */

/* ---- comparisons -> Bool (ref bridge.h:106-111) ------------------------ */
B200Value b200_equal(B200Context ctx, B200Value lhs, B200Value rhs, B200Error* err);
B200Value b200_not_equal(B200Context ctx, B200Value lhs, B200Value rhs, B200Error* err);
B200Value b200_less_than(B200Context ctx, B200Value lhs, B200Value rhs, B200Error* err);
B200Value b200_less_or_equal(B200Context ctx, B200Value lhs, B200Value rhs, B200Error* err);
B200Value b200_greater_than(B200Context ctx, B200Value lhs, B200Value rhs, B200Error* err);
B200Value b200_greater_or_equal(B200Context ctx, B200Value lhs, B200Value rhs, B200Error* err);

/* ---- shape ops (ref bridge.h:114-130) ---------------------------------- */
B200Value b200_reshape(B200Context ctx, B200Value x, const int64_t* shape, int rank, B200Error* err);
B200Value b200_transpose(B200Context ctx, B200Value x, const int* permutation, int rank, B200Error* err);
B200Value b200_cast(B200Context ctx, B200Value x, int dtype, B200Error* err); /* float->int truncates toward zero */
B200Value b200_broadcast_to(B200Context ctx, B200Value x, const int64_t* shape, int rank, B200Error* err);
/* XLA BroadcastInDim: operand axis i maps to output axis broadcast_axes[i]
 * (ref function.go:1021-1041 builds it from reshape + broadcast_to). */
B200Value b200_broadcast_in_dim(B200Context ctx, B200Value x, const int64_t* shape, int rank,
                                const int* broadcast_axes, int num_axes, B200Error* err);
B200Value b200_slice(B200Context ctx, B200Value x, const int64_t* starts, const int64_t* ends,
                     const int64_t* strides, int rank, B200Error* err);
B200Value b200_concatenate(B200Context ctx, const B200Value* tensors, int num_tensors, int axis, B200Error* err);
B200Value b200_reverse(B200Context ctx, B200Value x, const int* axes, int num_axes, B200Error* err);
B200Value b200_pad(B200Context ctx, B200Value x, B200Value pad_value, const int64_t* pad_before,
                   const int64_t* pad_after, int rank, B200Error* err);
/* Slice whose start indices are scalar integer VALUES of the graph, one per axis (ref function.go:1571-1594;
 * bridge.m:918-984 builds it from per-axis gathers).  Out-of-range starts are clamped so that the slice fits, as
 * GoMLX documents for DynamicSlice; the reference bridge does not clamp (its gather reads whatever MPSGraph returns
 * for an out-of-range index), so parity is defined for in-range starts. */
B200Value b200_dynamic_slice(B200Context ctx, B200Value operand, const B200Value* start_indices, int num_indices,
                             const int64_t* slice_sizes, int rank, B200Error* err);
/* operand with the block `update` written at the (clamped) start indices (ref function.go:1596-1621;
 * bridge.m:986-1108 builds it from a mask, per-axis gathers and a select: three passes over the operand). */
B200Value b200_dynamic_update_slice(B200Context ctx, B200Value operand, B200Value update, const B200Value* start_indices,
                                    int num_indices, B200Error* err);

/* ---- selection (ref bridge.h:133-136) ---------------------------------- */
B200Value b200_where(B200Context ctx, B200Value cond, B200Value on_true, B200Value on_false, B200Error* err);
B200Value b200_clamp(B200Context ctx, B200Value min_val, B200Value x, B200Value max_val, B200Error* err);

/* ---- contraction ------------------------------------------------------- */
/* [..,M,K] x [..,K,N] batched matmul (ref bridge.h:139-140). */
B200Value b200_matmul(B200Context ctx, B200Value lhs, B200Value rhs, B200Error* err);
/* First-class DotGeneral: output dims = batch ++ lhs free ++ rhs free, output
 * dtype = lhs dtype, fp32 accumulation (ref dotgeneral.go:15-53, 65-164; there
 * it is lowered to transposes + mpsgraph_matmul, here the GEMM reads both
 * operand layouts directly). */
B200Value b200_dot_general(B200Context ctx, B200Value lhs, const int* lhs_contracting, int num_lhs_contracting,
                           const int* lhs_batch, int num_lhs_batch, B200Value rhs, const int* rhs_contracting,
                           int num_rhs_contracting, const int* rhs_batch, int num_rhs_batch, B200Error* err);

/* ---- reductions (ref bridge.h:143-144, 195-198) ------------------------- */
/* Reduced axes are REMOVED from the result; num_axes == 0 reduces all axes
 * (ref function.go:1147-1183). */
B200Value b200_reduce(B200Context ctx, B200Value x, int reduce_type, const int* axes, int num_axes, B200Error* err);
/* Axis removed; lowest index wins ties; NaN counts as the extreme. */
B200Value b200_argmin(B200Context ctx, B200Value x, int axis, int output_dtype, B200Error* err);
B200Value b200_argmax(B200Context ctx, B200Value x, int axis, int output_dtype, B200Error* err);

/* ---- gather (ref bridge.h:147-152; gather.go:24-434) -------------------- */
/* Full XLA Gather, the signature of backends.Function.Gather (ref gather.go:24-29).
 * Out-of-range start indices are clamped so the slice stays inside the operand. */
B200Value b200_gather(B200Context ctx, B200Value operand, B200Value start_indices, int index_vector_axis,
                      const int* offset_output_axes, int num_offset_output_axes, const int* collapsed_slice_axes,
                      int num_collapsed_slice_axes, const int* start_index_map, int num_start_index_map,
                      const int64_t* slice_sizes, int num_slice_sizes, bool indices_are_sorted, B200Error* err);
B200Value b200_gather_along_axis(B200Context ctx, B200Value x, B200Value indices, int axis, B200Error* err);

/* ---- fused ops: explicit here, where the reference hopes the framework fuses */
/* ref bridge.h:201-202; function.go:2276-2286 */
B200Value b200_softmax(B200Context ctx, B200Value x, int axis, B200Error* err);
/* softmax(scale * x + mask terms) over the LAST axis of x[..., Sq, Sk].
 * causal != 0 masks element (i, j) with j > i to -inf.  mask may be NULL, a Bool
 * tensor (false -> -inf) or a float tensor (added); it is broadcast from its
 * trailing axes (ref function.go:2768-2894, the scale/mask/softmax part of SDPA). */
B200Value b200_softmax_masked(B200Context ctx, B200Value x, double scale, int causal, B200Value mask, B200Error* err);
/* ref function.go:2410-2565.  gamma / beta may be NULL. */
B200Value b200_layer_norm(B200Context ctx, B200Value x, const int* axes, int num_axes, double epsilon,
                          B200Value gamma, B200Value beta, B200Error* err);
/* y = x * rsqrt(mean(x^2 over axes) + eps) * gamma.  No counterpart in the
 * reference (it has no RMSNorm); GoMLX emits it as primitives. */
B200Value b200_rms_norm(B200Context ctx, B200Value x, const int* axes, int num_axes, double epsilon,
                        B200Value gamma, B200Error* err);
/* ref function.go:2288-2408 */
B200Value b200_gelu(B200Context ctx, B200Value x, int exact, B200Error* err);
/* ref function.go:2567-2667.  bias may be NULL. */
B200Value b200_dense(B200Context ctx, B200Value x, B200Value weight, B200Value bias, int activation, B200Error* err);
/* ref function.go:2976-3075.  Writes three values.  Biases may be NULL. */
bool b200_attention_qkv_projection(B200Context ctx, B200Value x, B200Value w_qkv, B200Value bias_q,
                                   B200Value bias_k, B200Value bias_v, int query_dim, int key_value_dim,
                                   B200Value* out_q, B200Value* out_k, B200Value* out_v, B200Error* err);
/* ref function.go:2669-2907.  mask may be NULL. */
B200Value b200_scaled_dot_product_attention(B200Context ctx, B200Value query, B200Value key, B200Value value,
                                            B200Value mask, int num_heads, int num_kv_heads, int axes_layout,
                                            double scale, int causal, B200Error* err);
/* ref bridge.h:189-192 (inference form) */
B200Value b200_batch_norm_inference(B200Context ctx, B200Value input, B200Value mean, B200Value variance,
                                    B200Value gamma, B200Value beta, float epsilon, int feature_axis,
                                    B200Error* err);

/* ---- training-side ops ---------------------------------------------------- */
/* BatchNormForTraining (ref function.go:1263-1375): batch mean and biased variance over every axis but feature_axis,
 * normalised * scale + offset; out_mean / out_variance are [feature] vectors.  false + *err on failure. */
bool b200_batch_norm_training(B200Context ctx, B200Value operand, B200Value scale, B200Value offset, float epsilon,
                              int feature_axis, B200Value* out_normalized, B200Value* out_mean, B200Value* out_variance,
                              B200Error* err);
/* BatchNormGradient (ref function.go:1377-1527): gradients w.r.t. operand, scale and offset. */
bool b200_batch_norm_gradient(B200Context ctx, B200Value operand, B200Value scale, B200Value mean, B200Value variance,
                              B200Value grad_output, float epsilon, int feature_axis, B200Value* out_grad_operand,
                              B200Value* out_grad_scale, B200Value* out_grad_offset, B200Error* err);
/* ScatterSum / ScatterMax / ScatterMin (ref gather.go:441-641; bridge.h:153-155, 233-235), the signature of
 * backends.Function.ScatterSum with the combiner as `mode`: 0 sum, 1 max, 2 min.  Elements whose position falls
 * outside the operand are dropped. */
B200Value b200_scatter(B200Context ctx, int mode, B200Value operand, B200Value scatter_indices, B200Value updates,
                       int index_vector_axis, const int* update_window_axes, int num_update_window_axes,
                       const int* inserted_window_axes, int num_inserted_window_axes,
                       const int* scatter_axes_to_operand_axes, int num_scatter_axes, bool indices_are_sorted,
                       bool unique_indices, B200Error* err);
/* RNGBitGenerator (ref function.go:1627-1692): state is (Uint64)[3]; *out_new_state is the state with every word + 1
 * (as the reference advances it), *out_values are `dtype`[shape] values that are a pure function of the state
 * (Philox4x32-10; the reference's values come from Apple's generator and are not reproducible): raw bits for integer
 * dtypes, uniform [0, 1) for float dtypes. */
bool b200_rng_bit_generator(B200Context ctx, B200Value state, int dtype, const int64_t* shape, int rank,
                            B200Value* out_new_state, B200Value* out_values, B200Error* err);

/* ---- control flow over closures (ref function.go:109-131, 354-652; executable.go:219-480) ----------------
 * A closure (GoMLX's Function.Closure() / Builder.NewFunction()) is built in the SAME context as its parent: its
 * parameters come from b200_closure_parameter, its results are ordinary values, and it captures outer values by
 * using them.  The reference keeps one control-flow op per function and runs it on the host; here there is no
 * such limit. */
B200Value b200_closure_parameter(B200Context ctx, int dtype, const int64_t* shape, int rank, B200Error* err);
/* Call: the callee (params -> outputs) is inlined with `inputs` in place of its parameters. */
bool b200_call(B200Context ctx, const B200Value* params, int num_params, const B200Value* outputs, int num_outputs,
               const B200Value* inputs, B200Value* results, B200Error* err);
/* If: pred is a scalar Bool; the branches take no parameters.  Light (elementwise, small) branches are both evaluated
 * and results[i] selects between them; heavy ones become two sub-plans of which one runs (chosen by the host on the
 * executable's first runs, by conditional graph nodes on the device once the plan replays as a CUDA graph). */
bool b200_if(B200Context ctx, B200Value pred, const B200Value* true_outputs, const B200Value* false_outputs,
             int num_outputs, B200Value* results, B200Error* err);
/* While: state -> cond(state) scalar Bool; state -> body(state) of the same shapes; results = the final state.  cond and
 * body are compiled into two sub-plans when the parent is compiled.  On the executable's first runs the host drives the
 * loop (it reads the one-byte condition back each trip); once the plan replays as a CUDA graph the loop is a
 * conditional node and runs entirely on the device.  At most 1 000 000 trips (ref executable.go:241). */
bool b200_while(B200Context ctx, const B200Value* cond_params, B200Value cond_output, const B200Value* body_params,
                const B200Value* body_outputs, int num_state, const B200Value* initial_state, B200Value* results,
                B200Error* err);
/* Sort along `axis` (always stable): the comparator (2 scalar parameters per input) must order by its first input:
 * LessThan / LessOrEqual / GreaterThan / GreaterOrEqual of its parameters 0 and 1.  Every input is permuted alike.
 * NaN keys sort last.  64-bit keys are not supported. */
bool b200_sort(B200Context ctx, const B200Value* comparator_params, int num_params, B200Value comparator_output, int axis,
               bool is_stable, const B200Value* inputs, int num_inputs, B200Value* results, B200Error* err);

/* ---- compile (ref bridge.h:159-163; builder.go:72-109) ------------------ */
/* feeds are placeholders in Parameter order, targets in Return order. */
B200Exec b200_compile(B200Context ctx, const B200Value* feeds, int num_feeds, const B200Value* targets,
                      int num_targets, B200Error* err);
void b200_destroy_exec(B200Exec exec);
int b200_exec_device(B200Exec exec);
int b200_exec_num_inputs(B200Exec exec);
int b200_exec_num_outputs(B200Exec exec);
/* Shape of output i: writes dims (up to cap), dtype; returns rank (ref executable.go:40-47). */
int b200_exec_output_shape(B200Exec exec, int i, int* dtype, int64_t* dims, int cap);
int b200_exec_input_shape(B200Exec exec, int i, int* dtype, int64_t* dims, int cap);
/* Number of kernel launches one execution enqueues, and bytes of intermediate arena. */
int b200_exec_num_launches(B200Exec exec);
int64_t b200_exec_arena_bytes(B200Exec exec);
/* Writes a NUL-terminated, human-readable launch plan (one line per step) into
 * buf (truncated to cap).  Returns the full length. */
int64_t b200_exec_describe(B200Exec exec, char* buf, int64_t cap);

/* ---- execute ------------------------------------------------------------ */
/* Device buffers in, fresh device buffers out (caller owns them and frees them
 * with b200_buffer_free).  Enqueues on the device's stream and returns without
 * waiting (ref executable.go:50-112 is the blocking, copying counterpart).
 * Inputs are not consumed.  Executions of one B200Exec are serialised. */
bool b200_execute(B200Exec exec, const B200Buffer* inputs, int num_inputs, B200Buffer* outputs, int num_outputs,
                  B200Error* err);
/* b200_execute with GoMLX's `donate` flags (ref executable.go:50-60 accepts and ignores them): donate[i] != 0 hands
 * input i to the call: its handle is finalized by the call (do not free it again) and its memory may become an output.
 * Today one case reuses it: an output that is DynamicUpdateSlice(input i, ...), with input i used by nothing else,
 * is updated IN PLACE -- only the update block is written, which is what makes a KV-cache append cost the size of the
 * new entry instead of a copy of the whole cache.  Other donated inputs are simply released. */
bool b200_execute_donating(B200Exec exec, const B200Buffer* inputs, const unsigned char* donate, int num_inputs, B200Buffer* outputs,
                           int num_outputs, B200Error* err);
/* Like b200_execute, but brackets every step of the launch plan with CUDA events, waits, and writes a
 * NUL-terminated report (one line per step: milliseconds, share, description) into report (truncated to cap).
 * Returns the full report length, or -1 with error.  The reference has no profiling hook (only DEBUG
 * fprintf, ref bridge.m:1218-1236). */
int64_t b200_execute_profiled(B200Exec exec, const B200Buffer* inputs, int num_inputs, B200Buffer* outputs, int num_outputs,
                              char* report, int64_t cap, B200Error* err);
/* Host pointers in, host pointers out: the exact calling shape of
 * mpsgraph_execute (ref bridge.h:167-172; bridge.m:1251-1403).  Copies inputs
 * host->device, runs, copies outputs device->host, and waits. */
bool b200_execute_host(B200Exec exec, void** input_data, const int64_t* input_sizes, const int* input_dtypes,
                       int64_t** input_shapes, const int* input_ranks, int num_inputs, void** output_data,
                       const int64_t* output_sizes, const int* output_dtypes, int64_t** output_shapes,
                       const int* output_ranks, int num_outputs, B200Error* err);
/* The same over num_slices consecutive leading-axis slices of the host arrays, for an executable compiled for ONE
 * slice.  Input i with input_sliced[i] != 0 holds num_slices x (executable input i) back to back and slice s is fed
 * to run s; other inputs (weights, tables) are uploaded once and fed to every run.  Output j receives num_slices x
 * (executable output j) back to back.  The result equals num_slices calls of b200_execute_host, but the upload of
 * slice s+1, the kernels of slice s and the download of slice s-1 run concurrently on three streams (pass pinned
 * memory from b200_host_alloc for the copies to overlap).  Blocks until every output is in host memory.  The
 * reference's execute (ref bridge.m:1293-1391) uploads, runs and downloads strictly in sequence. */
bool b200_execute_host_sliced(B200Exec exec, void** input_data, const int* input_sliced, int num_inputs, void** output_data,
                              int num_outputs, int64_t num_slices, B200Error* err);

/* ---- device buffers (ref bridge.h:175-178; backend.go:103-167) ---------- */
B200Buffer b200_buffer_alloc(int device, int dtype, const int64_t* shape, int rank, B200Error* err);
/* BufferFromFlatData (ref backend.go:140-143): allocates and copies nbytes from host. */
B200Buffer b200_buffer_from_host(int device, const void* data, int64_t nbytes, int dtype, const int64_t* shape,
                                 int rank, B200Error* err);
/* BufferToFlatData (ref backend.go:131-138): waits for pending work on the
 * buffer's device stream, then copies to host. */
bool b200_buffer_to_host(B200Buffer buf, void* data, int64_t nbytes, B200Error* err);
/* Overwrites an existing buffer from host memory, stream-ordered (pinned host memory makes it asynchronous). */
bool b200_buffer_write(B200Buffer buf, const void* data, int64_t nbytes, B200Error* err);
/* BufferCopyToDevice (ref backend.go:164-167 returns an error; here a peer copy). */
B200Buffer b200_buffer_copy_to_device(B200Buffer buf, int device, B200Error* err);
void b200_buffer_free(B200Buffer buf); /* BufferFinalize (ref backend.go:103-115) */
int b200_buffer_dtype(B200Buffer buf);
int b200_buffer_rank(B200Buffer buf);
int b200_buffer_shape(B200Buffer buf, int64_t* dims, int cap);
int64_t b200_buffer_nbytes(B200Buffer buf);
int b200_buffer_device(B200Buffer buf); /* BufferDeviceNum (ref backend.go:126-129) */
void* b200_buffer_device_ptr(B200Buffer buf);
/* Sharing a buffer with the other processes of one host (one process per GPU): export writes a 64-byte handle that
 * another process passes to import, which maps the same device memory (peer access over NVLink is enabled by the
 * mapping).  The imported buffer is unmapped, not freed, by b200_buffer_free; the exporter must outlive every
 * importer's use.  The reference is single-device (ref backend.go:144-167) and has no counterpart. */
#define B200_IPC_HANDLE_BYTES 64
bool b200_buffer_ipc_export(B200Buffer buf, void* handle_out, B200Error* err);
B200Buffer b200_buffer_ipc_import(int device, const void* handle, int dtype, const int64_t* shape, int rank, B200Error* err);
/* Wraps device memory owned by someone else (not freed by b200_buffer_free). */
B200Buffer b200_buffer_wrap(int device, void* device_ptr, int dtype, const int64_t* shape, int rank, B200Error* err);

/* Pinned host staging memory for asynchronous copies. */
void* b200_host_alloc(int64_t nbytes, B200Error* err);
void b200_host_free(void* p);

/* Waits for all work enqueued on the device's stream (ref bridge.m:1339-1340). */
bool b200_device_synchronize(int device, B200Error* err);
/* The CUDA stream (a cudaStream_t, as void*) that this library enqueues on for the device. */
void* b200_device_stream(int device, B200Error* err);
/* Bytes currently held by the device's caching allocator (in use + cached). */
int64_t b200_device_bytes_reserved(int device);
/* Returns cached, unused blocks to the driver. */
void b200_device_trim(int device);

/* ---- direct kernel entry points ----------------------------------------
 * The same launchers the compiled plans use, on raw device pointers and the
 * library's stream for `device`.  They let a caller (and the benchmarks) time
 * one kernel without the graph layer.  All return false + error on bad
 * arguments or a launch failure. */

/* Row softmax over the last axis of x[rows, cols]; row r is treated as query
 * position (r % seq_q) when causal != 0: columns j > (r % seq_q) are -inf.
 * dtype in {F32, BF16, F16}. */
bool b200_k_softmax(int device, const void* x, void* y, int64_t rows, int64_t cols, int dtype, double scale,
                    int causal, int64_t seq_q, B200Error* err);
/* LayerNorm / RMSNorm over the last axis of x[rows, cols]; gamma / beta [cols] or NULL. */
bool b200_k_layer_norm(int device, const void* x, const void* gamma, const void* beta, void* y, int64_t rows,
                       int64_t cols, int dtype, double epsilon, B200Error* err);
bool b200_k_rms_norm(int device, const void* x, const void* gamma, void* y, int64_t rows, int64_t cols, int dtype,
                     double epsilon, B200Error* err);
/* C[b] = op(A[b]) * op(B[b]), fp32 accumulation, output dtype = input dtype.
 * a_k_major: A stored [batch, M, K] (1) or [batch, K, M] (0).
 * b_k_major: B stored [batch, N, K] (1) or [batch, K, N] (0).  C is [batch, M, N].
 * dtype in {BF16, F16, F32}.  bias [N] (may be NULL) and activation are applied in the epilogue. */
bool b200_k_gemm(int device, const void* a, const void* b, void* c, int64_t batch, int64_t m, int64_t n, int64_t k,
                 int a_k_major, int b_k_major, int dtype, const void* bias, int activation, B200Error* err);
/* Column-sharded matmul with the all-gather fused into the GEMM: this rank multiplies A [M, K] by ITS column block of
 * the weight (B stored [K, n_local] when b_k_major == 0, [n_local, K] otherwise) and the epilogue stores the [M, n_local]
 * slab straight into columns [rank * n_local, +n_local) of EVERY rank's full result C_r [M, num_ranks * n_local]:
 * c_all[r] is rank r's C as seen from this device (its own for r == rank, b200_buffer_ipc_import'ed peers otherwise),
 * so the slab crosses NVLink as plain stores while the next tiles are still being multiplied.  No collective call
 * follows; the ranks only have to agree (a host barrier after each has synchronised its stream) that every slab has
 * landed before C is read.  n_local must be a multiple of 8 (16-byte stores).  dtype in {BF16, F16}. */
bool b200_k_gemm_allgather(int device, const void* a, const void* b, void* const* c_all, int num_ranks, int rank, int64_t m,
                           int64_t n_local, int64_t k, int a_k_major, int b_k_major, int dtype, B200Error* err);
/* Fused attention softmax(scale * Q K^T [+ causal mask]) V, the kernel behind
 * b200_scaled_dot_product_attention when no mask tensor is given (ref function.go:2669-2907).
 * Q is [batch, seq_q, heads, 64] (bshd != 0) or [batch, heads, seq_q, 64]; K and V likewise with kv_heads and
 * seq_k; O has Q's layout.  head_dim must be 64, dtype BF16 or F16. */
bool b200_k_attention(int device, const void* q, const void* k, const void* v, void* o, int64_t batch, int64_t heads,
                      int64_t kv_heads, int64_t seq_q, int64_t seq_k, int64_t head_dim, int bshd, int causal, double scale,
                      int dtype, B200Error* err);
/* Sum of all n elements of x (F32) into out[0] (F32).  scratch must hold
 * b200_k_reduce_sum_scratch_bytes(n) bytes of device memory. */
int64_t b200_k_reduce_sum_scratch_bytes(int64_t n);
bool b200_k_reduce_sum_f32(int device, const float* x, float* out, int64_t n, void* scratch, int64_t scratch_bytes,
                           B200Error* err);
/* The same reduction for callers that cannot allocate device memory (fixed
 * memory budgets, latency-critical loops, threads without access to an
 * allocator): the partial sums go to a 16 KiB array built into the library's
 * device image, so no scratch pointer is passed and nothing is allocated.
 * n must be <= 2^30; larger inputs are refused with B200_ERR_INVALID.  The
 * first call on a device looks up the array's address; on a device nothing else
 * has used through this library it also creates the library's stream (no
 * cudaMalloc: the library's status word is a device-image array too).  Make that
 * first call at start-up, before any stream capture.  All calls on a device
 * share the array: overlapping calls would race.
 * This entry point has no counterpart in the reference. */
bool b200_k_reduce_sum_f32_noalloc(int device, const float* x, float* out, int64_t n, B200Error* err);

#ifdef __cplusplus
}
#endif
#endif /* B200MLX_H */
