// Buffer, device and direct-kernel entry points of the C ABI.
//
// Buffers replace the reference's gpuBuffer (a Go slice; mpsgraph buffer.go:20-87)
// and its unused MTLBuffer helpers (bridge.h:175-178): here a buffer IS a device
// allocation, and host<->device traffic happens only in buffer_from_host,
// buffer_to_host, buffer_write and execute_host.
#include "common.h"
#include "kernels.h"

using namespace b200;

namespace {

Status make_buffer(int device, int dtype, const int64_t* shape, int rank, Buffer** out) {
  if (!dtype_valid(dtype)) return Status::Invalid("buffer: bad dtype");
  if (rank < 0 || rank > 16 || (rank > 0 && !shape)) return Status::Invalid("buffer: bad shape");
  Device* dev;
  B200_TRY(Device::Get(device, &dev));
  std::unique_ptr<Buffer> b(new Buffer());
  b->device = device;
  b->dtype = dtype;
  int64_t n = 1;
  for (int i = 0; i < rank; ++i) {
    if (shape[i] < 0) return Status::Invalid("buffer: negative dimension");
    b->dims.push_back(shape[i]);
    n *= shape[i];
  }
  b->nbytes = n * dtype_size(dtype);  // a scalar is stored as one element (ref buffer.go:28-31)
  B200_TRY(dev->Alloc(b->nbytes > 0 ? b->nbytes : 1, &b->ptr));
  *out = b.release();
  return Status::OK();
}

}  // namespace

extern "C" {

B200Buffer b200_buffer_alloc(int device, int dtype, const int64_t* shape, int rank, B200Error* err) {
  clear_error(err);
  Buffer* b = nullptr;
  Status s = make_buffer(device, dtype, shape, rank, &b);
  if (!s.ok()) { set_error(err, s); return nullptr; }
  return b;
}

B200Buffer b200_buffer_from_host(int device, const void* data, int64_t nbytes, int dtype, const int64_t* shape, int rank,
                                 B200Error* err) {
  clear_error(err);
  Buffer* b = nullptr;
  Status s = make_buffer(device, dtype, shape, rank, &b);
  if (!s.ok()) { set_error(err, s); return nullptr; }
  if (nbytes != b->nbytes) {
    s = Status::Invalid(strfmt("BufferFromFlatData: %lld bytes given, shape needs %lld", (long long)nbytes, (long long)b->nbytes));
  } else if (nbytes > 0) {
    if (!data) s = Status::Invalid("BufferFromFlatData: null data");
    else if (!b200_buffer_write(b, data, nbytes, err)) { b200_buffer_free(b); return nullptr; }
  }
  if (!s.ok()) { set_error(err, s); b200_buffer_free(b); return nullptr; }
  return b;
}

bool b200_buffer_write(B200Buffer buf, const void* data, int64_t nbytes, B200Error* err) {
  clear_error(err);
  Buffer* b = reinterpret_cast<Buffer*>(buf);
  if (!b || !b->ptr) { set_error(err, Status::Invalid("buffer_write: null or finalized buffer")); return false; }
  if (nbytes != b->nbytes) { set_error(err, Status::Invalid("buffer_write: size mismatch")); return false; }
  Device* dev;
  Status s = Device::Get(b->device, &dev);
  if (s.ok()) s = dev->MakeCurrent();
  if (s.ok() && nbytes > 0) {
    // Pinned sources copy asynchronously; pageable ones are staged by the driver before this returns.
    cudaError_t e = cudaMemcpyAsync(b->ptr, data, (size_t)nbytes, cudaMemcpyHostToDevice, dev->stream());
    if (e != cudaSuccess) s = Status::Cuda(strfmt("host->device copy failed: %s", cudaGetErrorString(e)));
  }
  if (!s.ok()) { set_error(err, s); return false; }
  return true;
}

bool b200_buffer_to_host(B200Buffer buf, void* data, int64_t nbytes, B200Error* err) {
  clear_error(err);
  Buffer* b = reinterpret_cast<Buffer*>(buf);
  if (!b || !b->ptr) { set_error(err, Status::Invalid("BufferToFlatData: null or finalized buffer")); return false; }
  if (nbytes != b->nbytes) {
    set_error(err, Status::Invalid(strfmt("BufferToFlatData: destination holds %lld bytes, buffer %lld", (long long)nbytes, (long long)b->nbytes)));
    return false;
  }
  Device* dev;
  Status s = Device::Get(b->device, &dev);
  if (s.ok()) s = dev->MakeCurrent();
  if (s.ok() && nbytes > 0) {
    cudaError_t e = cudaMemcpyAsync(data, b->ptr, (size_t)nbytes, cudaMemcpyDeviceToHost, dev->stream());
    if (e != cudaSuccess) s = Status::Cuda(strfmt("device->host copy failed: %s", cudaGetErrorString(e)));
  }
  if (s.ok()) {
    cudaError_t e = cudaStreamSynchronize(dev->stream());
    if (e != cudaSuccess) s = Status::Cuda(strfmt("stream synchronize failed: %s", cudaGetErrorString(e)));
    else s = dev->CheckKernelErrors();
  }
  if (!s.ok()) { set_error(err, s); return false; }
  return true;
}

B200Buffer b200_buffer_copy_to_device(B200Buffer buf, int device, B200Error* err) {
  clear_error(err);
  Buffer* b = reinterpret_cast<Buffer*>(buf);
  if (!b || !b->ptr) { set_error(err, Status::Invalid("BufferCopyToDevice: null or finalized buffer")); return nullptr; }
  Buffer* o = nullptr;
  Status s = make_buffer(device, b->dtype, b->dims.data(), (int)b->dims.size(), &o);
  if (!s.ok()) { set_error(err, s); return nullptr; }
  Device *src, *dst;
  s = Device::Get(b->device, &src);
  if (s.ok()) s = Device::Get(device, &dst);
  if (s.ok() && b->nbytes > 0) {
    // Order the copy after the producer's stream and run it on the consumer's stream; then make the producer's
    // stream wait for the copy.  The source device's allocator hands a freed block out again at once on the
    // grounds that every use of it was enqueued on that device's own stream: without the second wait a caller
    // that finalizes the source right after this call could see its block overwritten while the copy still reads it.
    cudaEvent_t ev = nullptr, done = nullptr;
    cudaError_t e = cudaSetDevice(b->device);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&ev, cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventRecord(ev, src->stream());
    if (e == cudaSuccess) e = cudaSetDevice(device);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(dst->stream(), ev, 0);
    if (e == cudaSuccess) e = cudaMemcpyPeerAsync(o->ptr, device, b->ptr, b->device, (size_t)b->nbytes, dst->stream());
    if (e == cudaSuccess && src != dst) {
      e = cudaEventCreateWithFlags(&done, cudaEventDisableTiming);
      if (e == cudaSuccess) e = cudaEventRecord(done, dst->stream());
      if (e == cudaSuccess) e = cudaSetDevice(b->device);
      if (e == cudaSuccess) e = cudaStreamWaitEvent(src->stream(), done, 0);
    }
    if (ev) cudaEventDestroy(ev);
    if (done) cudaEventDestroy(done);
    if (e != cudaSuccess) s = Status::Cuda(strfmt("peer copy failed: %s", cudaGetErrorString(e)));
  }
  if (!s.ok()) { set_error(err, s); b200_buffer_free(o); return nullptr; }
  return o;
}

void b200_buffer_free(B200Buffer buf) {
  Buffer* b = reinterpret_cast<Buffer*>(buf);
  if (!b) return;
  if (b->ipc && b->ptr) {
    Device* dev;
    if (Device::Get(b->device, &dev).ok() && dev->MakeCurrent().ok()) cudaIpcCloseMemHandle(b->ptr);
  } else if (b->owned && b->ptr) {
    Device* dev;
    if (Device::Get(b->device, &dev).ok()) dev->Free(b->ptr);
  }
  delete b;
}

static_assert(sizeof(cudaIpcMemHandle_t) == B200_IPC_HANDLE_BYTES, "IPC handle size");

bool b200_buffer_ipc_export(B200Buffer buf, void* handle_out, B200Error* err) {
  clear_error(err);
  Buffer* b = reinterpret_cast<Buffer*>(buf);
  if (!b || !b->ptr || !handle_out) { set_error(err, Status::Invalid("ipc_export: null buffer or handle")); return false; }
  if (!b->owned || b->ipc) { set_error(err, Status::Invalid("ipc_export: only a buffer this process allocated can be exported")); return false; }
  Device* dev;
  Status s = Device::Get(b->device, &dev);
  if (s.ok()) s = dev->MakeCurrent();
  if (!s.ok()) { set_error(err, s); return false; }
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, b->ptr);
  if (e != cudaSuccess) {
    cudaGetLastError();
    set_error(err, Status::Cuda(strfmt("cudaIpcGetMemHandle: %s", cudaGetErrorString(e))));
    return false;
  }
  memcpy(handle_out, &h, sizeof(h));
  return true;
}

B200Buffer b200_buffer_ipc_import(int device, const void* handle, int dtype, const int64_t* shape, int rank, B200Error* err) {
  clear_error(err);
  if (!handle || !dtype_valid(dtype) || rank < 0 || rank > 16 || (rank > 0 && !shape)) { set_error(err, Status::Invalid("ipc_import: bad handle, dtype or shape")); return nullptr; }
  Device* dev;
  Status s = Device::Get(device, &dev);
  if (s.ok()) s = dev->MakeCurrent();
  if (!s.ok()) { set_error(err, s); return nullptr; }
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) {
    cudaGetLastError();
    set_error(err, Status::Cuda(strfmt("cudaIpcOpenMemHandle: %s", cudaGetErrorString(e))));
    return nullptr;
  }
  Buffer* b = new Buffer();
  b->device = device;
  b->dtype = dtype;
  int64_t n = 1;
  for (int i = 0; i < rank; ++i) { b->dims.push_back(shape[i]); n *= shape[i]; }
  b->nbytes = n * dtype_size(dtype);
  b->ptr = p;
  b->owned = false;
  b->ipc = true;
  return b;
}

int b200_buffer_dtype(B200Buffer buf) { return buf ? reinterpret_cast<Buffer*>(buf)->dtype : -1; }
int b200_buffer_rank(B200Buffer buf) { return buf ? (int)reinterpret_cast<Buffer*>(buf)->dims.size() : -1; }
int b200_buffer_shape(B200Buffer buf, int64_t* dims, int cap) {
  if (!buf) return -1;
  Buffer* b = reinterpret_cast<Buffer*>(buf);
  for (int i = 0; i < (int)b->dims.size() && i < cap; ++i) dims[i] = b->dims[i];
  return (int)b->dims.size();
}
int64_t b200_buffer_nbytes(B200Buffer buf) { return buf ? reinterpret_cast<Buffer*>(buf)->nbytes : -1; }
int b200_buffer_device(B200Buffer buf) { return buf ? reinterpret_cast<Buffer*>(buf)->device : -1; }
void* b200_buffer_device_ptr(B200Buffer buf) { return buf ? reinterpret_cast<Buffer*>(buf)->ptr : nullptr; }

B200Buffer b200_buffer_wrap(int device, void* device_ptr, int dtype, const int64_t* shape, int rank, B200Error* err) {
  clear_error(err);
  if (!dtype_valid(dtype) || rank < 0 || rank > 16 || (rank > 0 && !shape)) { set_error(err, Status::Invalid("buffer_wrap: bad dtype or shape")); return nullptr; }
  Device* dev;
  Status s = Device::Get(device, &dev);
  if (!s.ok()) { set_error(err, s); return nullptr; }
  Buffer* b = new Buffer();
  b->device = device;
  b->dtype = dtype;
  int64_t n = 1;
  for (int i = 0; i < rank; ++i) { b->dims.push_back(shape[i]); n *= shape[i]; }
  b->nbytes = n * dtype_size(dtype);
  b->ptr = device_ptr;
  b->owned = false;
  return b;
}

void* b200_host_alloc(int64_t nbytes, B200Error* err) {
  clear_error(err);
  void* p = nullptr;
  cudaError_t e = cudaHostAlloc(&p, (size_t)(nbytes > 0 ? nbytes : 1), cudaHostAllocDefault);
  if (e != cudaSuccess) {
    cudaGetLastError();
    set_error(err, Status::Cuda(strfmt("cudaHostAlloc failed: %s", cudaGetErrorString(e))));
    return nullptr;
  }
  return p;
}
void b200_host_free(void* p) {
  if (p) cudaFreeHost(p);
}

bool b200_device_synchronize(int device, B200Error* err) {
  clear_error(err);
  Device* dev;
  Status s = Device::Get(device, &dev);
  if (s.ok()) s = dev->Synchronize();
  if (!s.ok()) { set_error(err, s); return false; }
  return true;
}
void* b200_device_stream(int device, B200Error* err) {
  clear_error(err);
  Device* dev;
  Status s = Device::Get(device, &dev);
  if (!s.ok()) { set_error(err, s); return nullptr; }
  return (void*)dev->stream();
}
int64_t b200_device_bytes_reserved(int device) {
  Device* dev;
  if (!Device::Get(device, &dev).ok()) return -1;
  return dev->BytesReserved();
}
void b200_device_trim(int device) {
  Device* dev;
  if (Device::Get(device, &dev).ok()) dev->Trim();
}

// Host pointers in, host pointers out (the calling shape of mpsgraph_execute,
// ref bridge.h:167-172).
bool b200_execute_host(B200Exec exec, void** input_data, const int64_t* input_sizes, const int* input_dtypes,
                       int64_t** input_shapes, const int* input_ranks, int num_inputs, void** output_data,
                       const int64_t* output_sizes, const int* output_dtypes, int64_t** output_shapes, const int* output_ranks,
                       int num_outputs, B200Error* err) {
  clear_error(err);
  (void)output_dtypes; (void)output_shapes; (void)output_ranks;
  if (!exec) { set_error(err, Status::Invalid("Execute: null executable")); return false; }
  if (num_inputs != b200_exec_num_inputs(exec) || num_outputs != b200_exec_num_outputs(exec)) {
    set_error(err, Status::Invalid("Execute: wrong number of inputs or outputs"));
    return false;
  }
  // The executable knows its device through its inputs' expected placement; use device of context via a probe buffer.
  std::vector<B200Buffer> in(num_inputs, nullptr), out(num_outputs, nullptr);
  auto cleanup = [&]() {
    for (auto b : in) b200_buffer_free(b);
    for (auto b : out) b200_buffer_free(b);
  };
  const int device = b200_exec_device(exec);
  for (int i = 0; i < num_inputs; ++i) {
    in[i] = b200_buffer_from_host(device, input_data[i], input_sizes[i], input_dtypes[i], input_shapes ? input_shapes[i] : nullptr,
                                  input_ranks[i], err);
    if (!in[i]) { cleanup(); return false; }
  }
  if (!b200_execute(exec, in.data(), num_inputs, out.data(), num_outputs, err)) { cleanup(); return false; }
  for (int i = 0; i < num_outputs; ++i) {
    if (!b200_buffer_to_host(out[i], output_data[i], output_sizes[i], err)) { cleanup(); return false; }
  }
  cleanup();
  return true;
}

// ---- direct kernel entry points ---------------------------------------------
bool b200_k_softmax(int device, const void* x, void* y, int64_t rows, int64_t cols, int dtype, double scale, int causal,
                    int64_t seq_q, B200Error* err) {
  clear_error(err);
  Device* dev;
  Status s = Device::Get(device, &dev);
  if (s.ok()) {
    k::SoftmaxParams p;
    p.x = x; p.y = y; p.rows = rows; p.cols = cols; p.dtype = dtype; p.scale = scale; p.causal = causal != 0; p.seq_q = seq_q;
    s = k::softmax_rows(dev, p);
  }
  if (!s.ok()) { set_error(err, s); return false; }
  return true;
}

static bool norm_entry(int device, const void* x, const void* gamma, const void* beta, void* y, int64_t rows, int64_t cols,
                       int dtype, double epsilon, bool rms, B200Error* err) {
  clear_error(err);
  Device* dev;
  Status s = Device::Get(device, &dev);
  if (s.ok()) {
    k::NormParams p;
    p.x = x; p.gamma = gamma; p.beta = beta; p.y = y; p.rows = rows; p.cols = cols; p.dtype = dtype; p.epsilon = epsilon; p.rms = rms;
    s = k::norm_rows(dev, p);
  }
  if (!s.ok()) { set_error(err, s); return false; }
  return true;
}
bool b200_k_layer_norm(int device, const void* x, const void* gamma, const void* beta, void* y, int64_t rows, int64_t cols,
                       int dtype, double epsilon, B200Error* err) {
  return norm_entry(device, x, gamma, beta, y, rows, cols, dtype, epsilon, false, err);
}
bool b200_k_rms_norm(int device, const void* x, const void* gamma, void* y, int64_t rows, int64_t cols, int dtype, double epsilon,
                     B200Error* err) {
  return norm_entry(device, x, gamma, nullptr, y, rows, cols, dtype, epsilon, true, err);
}

bool b200_k_gemm(int device, const void* a, const void* b, void* c, int64_t batch, int64_t m, int64_t n, int64_t k_, int a_k_major,
                 int b_k_major, int dtype, const void* bias, int activation, B200Error* err) {
  clear_error(err);
  Device* dev;
  Status s = Device::Get(device, &dev);
  if (s.ok()) {
    k::GemmParams p;
    p.a = a; p.b = b; p.c = c; p.batch = batch; p.m = m; p.n = n; p.k = k_;
    p.a_k_major = a_k_major != 0; p.b_k_major = b_k_major != 0; p.dtype = dtype; p.bias = bias; p.activation = activation;
    s = k::gemm(dev, p);
  }
  if (!s.ok()) { set_error(err, s); return false; }
  return true;
}

bool b200_k_gemm_allgather(int device, const void* a, const void* b, void* const* c_all, int num_ranks, int rank, int64_t m,
                           int64_t n_local, int64_t k_, int a_k_major, int b_k_major, int dtype, B200Error* err) {
  clear_error(err);
  Device* dev;
  Status s = Device::Get(device, &dev);
  if (s.ok() && (num_ranks < 1 || num_ranks > 1 + k::GemmParams::kMaxExtraC || rank < 0 || rank >= num_ranks || !c_all))
    s = Status::Invalid("gemm_allgather: 1 to 8 ranks, rank inside");
  if (s.ok() && !(dtype == B200_BFLOAT16 || dtype == B200_FLOAT16)) s = Status::Unsupported("gemm_allgather: BF16 or F16");
  if (s.ok() && (n_local % 8 != 0 || m <= 0 || n_local <= 0 || k_ <= 0)) s = Status::Invalid("gemm_allgather: n_local must be a positive multiple of 8");
  if (s.ok()) {
    const int64_t es = dtype_size(dtype);
    k::GemmParams p;
    p.a = a; p.b = b;
    p.batch = 1; p.m = m; p.n = n_local; p.k = k_;
    p.a_k_major = a_k_major != 0; p.b_k_major = b_k_major != 0;
    p.dtype = dtype;
    p.ldc = n_local * num_ranks;
    const int64_t col_bytes = (int64_t)rank * n_local * es;
    for (int r = 0; r < num_ranks && s.ok(); ++r)
      if (!c_all[r]) s = Status::Invalid("gemm_allgather: null destination");
    if (s.ok()) {
      p.c = (char*)c_all[rank] + col_bytes;
      for (int r = 0; r < num_ranks; ++r)
        if (r != rank) p.c_extra[p.num_c_extra++] = (char*)c_all[r] + col_bytes;
      bool taken = false;
      s = k::gemm_tcgen05(dev, p, &taken);
      if (s.ok() && !taken) s = Status::Unsupported("gemm_allgather: shape or alignment outside the tensor-core kernel (K and the operands' contiguous extents must be multiples of 8, 16-byte aligned)");
    }
  }
  if (!s.ok()) { set_error(err, s); return false; }
  return true;
}

bool b200_k_attention(int device, const void* q, const void* k_, const void* v, void* o, int64_t batch, int64_t heads, int64_t kv_heads,
                      int64_t seq_q, int64_t seq_k, int64_t head_dim, int bshd, int causal, double scale, int dtype, B200Error* err) {
  clear_error(err);
  Device* dev;
  Status s = Device::Get(device, &dev);
  if (s.ok()) {
    k::AttentionParams p;
    p.q = q; p.k = k_; p.v = v; p.o = o;
    p.B = batch; p.H = heads; p.Hkv = kv_heads; p.Sq = seq_q; p.Sk = seq_k; p.head_dim = head_dim;
    p.bshd = bshd != 0; p.causal = causal != 0; p.scale = scale; p.dtype = dtype;
    s = k::attention(dev, p);
  }
  if (!s.ok()) { set_error(err, s); return false; }
  return true;
}

int64_t b200_k_reduce_sum_scratch_bytes(int64_t n) { return k::reduce_scratch_bytes(B200_FLOAT32, 1, n, 1); }

bool b200_k_reduce_sum_f32(int device, const float* x, float* out, int64_t n, void* scratch, int64_t scratch_bytes, B200Error* err) {
  clear_error(err);
  Device* dev;
  Status s = Device::Get(device, &dev);
  if (s.ok()) s = k::reduce(dev, x, out, B200_FLOAT32, B200_REDUCE_SUM, 1, n, 1, scratch, scratch_bytes);
  if (!s.ok()) { set_error(err, s); return false; }
  return true;
}

}  // extern "C"
