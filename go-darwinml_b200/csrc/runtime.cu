// Device runtime: one stream and one stream-ordered caching allocator per GPU.
//
// The reference keeps every tensor in a Go slice and copies all inputs to the
// device on every Execute (mpsgraph bridge.m:1293) and all outputs back
// (bridge.m:1391).  Here buffers are device allocations; host<->device copies
// happen only in the buffer_from_host / buffer_to_host / execute_host calls.
#include <cstdarg>
#include <cstdio>

#include "common.h"

namespace b200 {

std::string strfmt(const char* fmt, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  return std::string(buf);
}

const char* dtype_name(int dt) {
  static const char* names[] = {"Bool",    "Int8",    "Int16", "Int32",  "Int64",  "Float16", "BFloat16",
                                "Float32", "Float64", "Uint8", "Uint16", "Uint32", "Uint64"};
  return dtype_valid(dt) ? names[dt] : "InvalidDType";
}

namespace {
constexpr int kMaxDevices = 64;
// The per-device status word that kernels with bounded waits set when a wait gives up.  It lives in the library's
// device image (every GPU that loads the library holds these 256 bytes, zero at load), so device set-up allocates
// nothing; in host code the name is only a stand-in, the device address comes from cudaGetSymbolAddress.
static __device__ __align__(256) int g_status_word[64];
std::mutex g_dev_mu;
Device* g_devices[kMaxDevices] = {nullptr};

int64_t round_size(int64_t n) {
  if (n <= 0) n = 1;
  if (n < (1 << 20)) return (n + 511) & ~int64_t(511);
  const int64_t g = 2 << 20;
  return (n + g - 1) / g * g;
}
}  // namespace

Status Device::Get(int ordinal, Device** out) {
  if (ordinal < 0 || ordinal >= kMaxDevices) return Status::Invalid(strfmt("device ordinal %d out of range", ordinal));
  std::lock_guard<std::mutex> lock(g_dev_mu);
  if (!g_devices[ordinal]) {
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return Status::Cuda(strfmt("no usable CUDA device: %s (this library has no CPU fallback)", cudaGetErrorString(e)));
    }
    if (ordinal >= count) return Status::Invalid(strfmt("device %d requested but only %d visible", ordinal, count));
    B200_CUDA_TRY(cudaSetDevice(ordinal));
    std::unique_ptr<Device> d(new Device());
    d->ordinal_ = ordinal;
    B200_CUDA_TRY(cudaStreamCreateWithFlags(&d->stream_, cudaStreamNonBlocking));
    int sms = 0;
    B200_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, ordinal));
    d->sm_count_ = sms > 0 ? sms : 148;
    B200_CUDA_TRY(cudaGetSymbolAddress((void**)&d->error_flag_, g_status_word));   // with this device current
    g_devices[ordinal] = d.release();
  }
  *out = g_devices[ordinal];
  return Status::OK();
}

namespace {
thread_local const Device* tls_override_dev = nullptr;
thread_local cudaStream_t tls_override_stream = nullptr;
}  // namespace

cudaStream_t Device::stream() const { return (tls_override_dev == this && tls_override_stream) ? tls_override_stream : stream_; }

StreamOverride::StreamOverride(const Device* dev, cudaStream_t s) : prev_dev_(tls_override_dev), prev_stream_(tls_override_stream) {
  tls_override_dev = dev;
  tls_override_stream = s;
}
StreamOverride::~StreamOverride() {
  tls_override_dev = prev_dev_;
  tls_override_stream = prev_stream_;
}

Status Device::LoopStream(int depth, cudaStream_t* out) {
  if (depth < 0 || depth >= kMaxLoopDepth) return Status::Unsupported("While: loops nested deeper than 4");
  std::lock_guard<std::mutex> lock(mu_);
  if (!loop_[depth]) {
    B200_CUDA_TRY(cudaSetDevice(ordinal_));
    B200_CUDA_TRY(cudaStreamCreateWithFlags(&loop_[depth], cudaStreamNonBlocking));
  }
  *out = loop_[depth];
  return Status::OK();
}

Status Device::CaptureStream(cudaStream_t* out) {
  std::lock_guard<std::mutex> lock(mu_);
  if (!capture_) {
    B200_CUDA_TRY(cudaSetDevice(ordinal_));
    B200_CUDA_TRY(cudaStreamCreateWithFlags(&capture_, cudaStreamNonBlocking));
  }
  *out = capture_;
  return Status::OK();
}

Status Device::CopyStreams(cudaStream_t* in, cudaStream_t* out) {
  std::lock_guard<std::mutex> lock(mu_);
  if (!copy_in_) {
    B200_CUDA_TRY(cudaSetDevice(ordinal_));
    B200_CUDA_TRY(cudaStreamCreateWithFlags(&copy_in_, cudaStreamNonBlocking));
    B200_CUDA_TRY(cudaStreamCreateWithFlags(&copy_out_, cudaStreamNonBlocking));
  }
  *in = copy_in_;
  *out = copy_out_;
  return Status::OK();
}

Status Device::MakeCurrent() {
  B200_CUDA_TRY(cudaSetDevice(ordinal_));
  return Status::OK();
}

Status Device::Synchronize() {
  B200_TRY(MakeCurrent());
  B200_CUDA_TRY(cudaStreamSynchronize(stream_));
  return CheckKernelErrors();
}

Status Device::CheckKernelErrors() {
  if (!error_flag_ || !error_check_pending_) return Status::OK();
  error_check_pending_ = false;
  int code = 0;
  B200_CUDA_TRY(cudaMemcpyAsync(&code, error_flag_, sizeof(int), cudaMemcpyDeviceToHost, stream_));
  B200_CUDA_TRY(cudaStreamSynchronize(stream_));
  if (code != 0) {
    B200_CUDA_TRY(cudaMemsetAsync(error_flag_, 0, sizeof(int), stream_));
    static const char* who[] = {"?", "a tile loader waiting for a free stage", "an MMA issuer waiting for a drained accumulator or for Q",
                                "an MMA issuer waiting for operand tiles", "an epilogue or MMA issuer waiting for its producer",
                                "a kernel whose shared-memory window is not 1024-byte aligned", "a softmax warp waiting for scores",
                                "a softmax warp waiting for the output MMAs", "an epilogue warp waiting for its residual block"};
    if (code == kErrWhileLimit) return Status::Invalid("While: exceeded maximum iterations (1000000); the loop was stopped and its results are invalid");
    return Status::Timeout(strfmt("a bounded wait inside a tensor-core kernel gave up (%s); its results are invalid",
                                  (code >= 1 && code <= 8) ? who[code] : who[0]));
  }
  return Status::OK();
}

Status Device::CheckLaunch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return Status::Cuda(strfmt("launch of %s failed: %s", what, cudaGetErrorString(e)));
  return Status::OK();
}

Status Device::Alloc(int64_t nbytes, void** out) {
  const int64_t size = round_size(nbytes);
  {
    std::lock_guard<std::mutex> lock(mu_);
    auto it = free_blocks_.lower_bound(size);
    // Reuse a cached block unless it would waste more than a quarter of itself.
    if (it != free_blocks_.end() && it->first <= size + size / 4 + 4096) {
      *out = it->second;
      live_blocks_[it->second] = it->first;
      free_blocks_.erase(it);
      return Status::OK();
    }
  }
  B200_TRY(MakeCurrent());
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, (size_t)size);
  if (e == cudaErrorMemoryAllocation) {
    cudaGetLastError();
    Trim();
    e = cudaMalloc(&p, (size_t)size);
  }
  if (e != cudaSuccess) {
    cudaGetLastError();
    return Status::Oom(strfmt("cudaMalloc of %lld bytes on device %d failed: %s", (long long)size, ordinal_,
                              cudaGetErrorString(e)));
  }
  std::lock_guard<std::mutex> lock(mu_);
  live_blocks_[p] = size;
  reserved_ += size;
  *out = p;
  return Status::OK();
}

void Device::Free(void* p) {
  if (!p) return;
  std::lock_guard<std::mutex> lock(mu_);
  auto it = live_blocks_.find(p);
  if (it == live_blocks_.end()) return;
  // Every use of the block was enqueued on stream_, and so will the next be:
  // reuse is ordered after the last use without a synchronisation.
  free_blocks_.emplace(it->second, p);
  live_blocks_.erase(it);
}

int64_t Device::BytesReserved() {
  std::lock_guard<std::mutex> lock(mu_);
  return reserved_;
}

void Device::Trim() {
  std::multimap<int64_t, void*> blocks;
  {
    std::lock_guard<std::mutex> lock(mu_);
    blocks.swap(free_blocks_);
  }
  if (blocks.empty()) return;
  cudaSetDevice(ordinal_);
  cudaStreamSynchronize(stream_);
  int64_t freed = 0;
  for (auto& kv : blocks) {
    cudaFree(kv.second);
    freed += kv.first;
  }
  std::lock_guard<std::mutex> lock(mu_);
  reserved_ -= freed;
}

}  // namespace b200
