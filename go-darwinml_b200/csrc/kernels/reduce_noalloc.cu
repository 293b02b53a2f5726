// b200_k_reduce_sum_f32_noalloc: the split (two-launch) fp32 sum reduction of
// reduce.cu for callers that must not allocate device memory.
//
// Who needs this: code that runs where an allocation is forbidden or would
// break an invariant -- a caller whose memory budget is fixed and fully handed
// out up front (an inference server that sized its pools at start-up and must
// never grow), a caller inside a latency-critical loop that cannot afford
// cudaMalloc's implicit device synchronisation, or a host thread that holds no
// handle to this library's allocator.  The regular entry point
// (b200_k_reduce_sum_f32) makes such callers provide a scratch buffer, which is
// exactly the allocation they cannot make.
//
// Here the partial sums go to a fixed array that lives in the library's device
// image: kNoAllocScratchBytes bytes on every GPU that loads the library, held
// until the process exits.  Consequences the caller must know:
//   * n is limited to kNoAllocMaxElements; larger inputs are refused.
//   * The FIRST call on a device looks up the array's device address.  If
//     nothing else has used that device through this library yet, that call
//     also performs the library's one-time device set-up: it creates the
//     library's stream (cudaStreamCreateWithFlags) and looks up the address of
//     the library's status word, which is a __device__ array like the scratch.
//     Neither step calls cudaMalloc, but creating a stream is not free: make
//     that first call at start-up, and before starting any stream capture.
//   * Every call on a device uses the same array and leaves its partial sums
//     behind.  Nothing needs clearing between calls: each launch overwrites
//     every slot it later reads.  Calls issued through this library run one
//     after another on the device's stream; if a caller arranges for two of
//     them to overlap on one GPU they race on the array.
//   * No cudaMalloc, cudaFree or other allocating routine is called here or
//     in the device set-up this may trigger.
#include <mutex>

#include "../kernels.h"

namespace {

constexpr int64_t kNoAllocScratchBytes = 16 * 1024;
constexpr int64_t kNoAllocMaxElements = int64_t(1) << 30;  // 4 GiB of float32
constexpr int kMaxDevices = 64;

// The scratch itself.  In host code this name is only a stand-in for the
// symbol, not a device address: the address comes from cudaGetSymbolAddress.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

std::mutex g_mu;
void* g_scratch_addr[kMaxDevices] = {nullptr};

// Once per device, with that device current.
b200::Status scratch_for(b200::Device* dev, void** out) {
  const int ord = dev->ordinal();
  if (ord < 0 || ord >= kMaxDevices) return b200::Status::Invalid("reduce_sum_noalloc: device ordinal out of range");
  std::lock_guard<std::mutex> lock(g_mu);
  if (!g_scratch_addr[ord]) {
    B200_TRY(dev->MakeCurrent());
    void* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress((void**)&ptr, g_noalloc_scratch);
    if (e != cudaSuccess || !ptr) {
      cudaGetLastError();
      return b200::Status::Cuda(b200::strfmt("reduce_sum_noalloc: cudaGetSymbolAddress failed on device %d: %s", ord, cudaGetErrorString(e)));
    }
    g_scratch_addr[ord] = ptr;
  }
  *out = g_scratch_addr[ord];
  return b200::Status::OK();
}

}  // namespace

extern "C" bool b200_k_reduce_sum_f32_noalloc(int device, const float* x, float* out, int64_t n, B200Error* err) {
  using namespace b200;
  clear_error(err);
  Status s = Status::OK();
  Device* dev = nullptr;
  if (n < 0 || n > kNoAllocMaxElements) {
    s = Status::Invalid(strfmt("reduce_sum_noalloc: n = %lld is outside [0, %lld]; use b200_k_reduce_sum_f32 with a caller-provided scratch buffer",
                               (long long)n, (long long)kNoAllocMaxElements));
  } else if (!x || !out) {
    s = Status::Invalid("reduce_sum_noalloc: null pointer");
  } else {
    s = Device::Get(device, &dev);
  }
  if (s.ok()) {
    const int64_t need = k::reduce_scratch_bytes(B200_FLOAT32, 1, n, 1);
    if (need > kNoAllocScratchBytes) {
      s = Status::Invalid(strfmt("reduce_sum_noalloc: needs %lld bytes of scratch, the built-in array holds %lld", (long long)need,
                                 (long long)kNoAllocScratchBytes));
    } else {
      void* scratch = nullptr;
      s = scratch_for(dev, &scratch);
      if (s.ok()) s = k::reduce(dev, x, out, B200_FLOAT32, B200_REDUCE_SUM, 1, n, 1, scratch, kNoAllocScratchBytes);
    }
  }
  if (!s.ok()) {
    set_error(err, s);
    return false;
  }
  return true;
}
