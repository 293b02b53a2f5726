// ArgSort: the stable permutation that sorts x along one axis, as int32 indices of x's shape.
//
// GoMLX's Sort takes a comparator closure and any number of tensors that are permuted alike (ref mpsgraph
// function.go:562-652; the reference sorts on the host, executable.go:385-480).  The graph layer accepts the
// comparators that order by the first tensor (LessThan / GreaterThan of its two parameters), turns the sort into this
// ArgSort plus one gather per tensor, and so the only sorting kernel is this one.
//
// x is viewed as [outer, n, inner]; every (outer, inner) pair is a row of n keys.  A key becomes a 32-bit unsigned
// integer whose order is the key's (floats: sign-magnitude flipped to two's-complement order, -0 = +0, NaN greatest;
// signed integers: sign bit flipped; for a descending sort the complement, NaN still greatest), the row index goes
// into the low 32 bits of a 64-bit word, and the words are sorted ascending by a bitonic network -- so equal keys keep
// their order (stable) and NaNs land last either way.  One CTA per row at a time; rows of up to 4096 keys sort in
// shared memory, longer ones in a per-CTA slice of a scratch buffer (the network's passes are CTA-wide barriers).
// Bit-exact by construction.  Cost: n log^2 n compare-exchanges per row; this is index work, not a bandwidth kernel.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "../kernels.h"

namespace b200 {
namespace k {

namespace {

constexpr int kSortThreads = 512;
constexpr int64_t kSmemKeys = 4096;

__device__ __forceinline__ uint32_t float_key(float f) {
  if (f != f) return 0xffffffffu;
  uint32_t u = __float_as_uint(f + 0.0f);   // -0 + 0 = +0
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ uint32_t load_key(const void* x, int64_t i, int dtype, bool descending) {
  uint32_t t;
  bool nan = false;
  switch (dtype) {
    case B200_FLOAT32: { const float f = reinterpret_cast<const float*>(x)[i]; nan = f != f; t = float_key(f); break; }
    case B200_BFLOAT16: { const float f = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(x)[i]); nan = f != f; t = float_key(f); break; }
    case B200_FLOAT16: { const float f = __half2float(reinterpret_cast<const __half*>(x)[i]); nan = f != f; t = float_key(f); break; }
    case B200_INT32: t = reinterpret_cast<const uint32_t*>(x)[i] ^ 0x80000000u; break;
    case B200_INT16: t = (uint32_t)(int32_t) reinterpret_cast<const int16_t*>(x)[i] ^ 0x80000000u; break;
    case B200_INT8: t = (uint32_t)(int32_t) reinterpret_cast<const int8_t*>(x)[i] ^ 0x80000000u; break;
    case B200_UINT32: t = reinterpret_cast<const uint32_t*>(x)[i]; break;
    case B200_UINT16: t = reinterpret_cast<const uint16_t*>(x)[i]; break;
    default: t = reinterpret_cast<const uint8_t*>(x)[i]; break;   // U8, Bool
  }
  if (descending && !nan) t = ~t;   // float keys lie in [0x007fffff, 0xff800000], so the complement never meets NaN's key
  return t;
}

__device__ __forceinline__ void bitonic(unsigned long long* buf, int64_t n_pad) {
  for (int64_t k = 2; k <= n_pad; k <<= 1) {
    for (int64_t j = k >> 1; j > 0; j >>= 1) {
      for (int64_t i = threadIdx.x; i < n_pad; i += blockDim.x) {
        const int64_t p = i ^ j;
        if (p > i) {
          const unsigned long long a = buf[i], b = buf[p];
          const bool up = (i & k) == 0;
          if ((a > b) == up) { buf[i] = b; buf[p] = a; }
        }
      }
      __syncthreads();
    }
  }
}

__global__ void __launch_bounds__(kSortThreads) argsort_kernel(const void* x, int32_t* out, int dtype, int64_t outer, int64_t n, int64_t inner,
                                                               int64_t n_pad, bool descending, unsigned long long* scratch) {
  extern __shared__ unsigned long long smem[];
  unsigned long long* buf = scratch ? scratch + (int64_t)blockIdx.x * n_pad : smem;
  const int64_t rows = outer * inner;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const int64_t o = row / inner, in = row - o * inner;
    const int64_t base = o * n * inner + in;
    for (int64_t j = threadIdx.x; j < n_pad; j += blockDim.x)
      buf[j] = j < n ? (((unsigned long long)load_key(x, base + j * inner, dtype, descending) << 32) | (unsigned long long)j) : ~0ull;
    __syncthreads();
    bitonic(buf, n_pad);
    for (int64_t j = threadIdx.x; j < n; j += blockDim.x) out[base + j * inner] = (int32_t)(buf[j] & 0xffffffffull);
    __syncthreads();
  }
}

int64_t pad_pow2(int64_t n) {
  int64_t p = 2;
  while (p < n) p <<= 1;
  return p;
}

}  // namespace

int64_t arg_sort_scratch_bytes(int64_t outer, int64_t n, int64_t inner, int sm_count) {
  const int64_t n_pad = pad_pow2(n);
  if (n_pad <= kSmemKeys) return 0;
  const int64_t rows = outer * inner;
  const int64_t grid = rows < (int64_t)sm_count * 2 ? rows : (int64_t)sm_count * 2;
  return grid * n_pad * 8;
}

Status arg_sort(Device* dev, const void* x, void* out, int dtype, int64_t outer, int64_t n, int64_t inner, bool descending, void* scratch,
                int64_t scratch_bytes) {
  if (outer * n * inner == 0) return Status::OK();
  if (dtype_size(dtype) == 8) return Status::Unsupported("Sort: 64-bit keys are not supported");
  if (n > 0x7fffffffLL) return Status::Unsupported("Sort: more than 2^31-1 keys per row");
  B200_TRY(dev->MakeCurrent());
  const int64_t n_pad = pad_pow2(n);
  const int64_t rows = outer * inner;
  const bool use_smem = n_pad <= kSmemKeys;
  int64_t grid = rows < (int64_t)dev->sm_count() * 2 ? rows : (int64_t)dev->sm_count() * 2;
  if (!use_smem && (!scratch || scratch_bytes < grid * n_pad * 8)) return Status::Invalid("Sort: scratch buffer too small");
  const size_t smem = use_smem ? (size_t)n_pad * 8 : 0;
  argsort_kernel<<<(unsigned)grid, kSortThreads, smem, dev->stream()>>>(x, reinterpret_cast<int32_t*>(out), dtype, outer, n, inner, n_pad, descending,
                                                                      use_smem ? nullptr : reinterpret_cast<unsigned long long*>(scratch));
  return dev->CheckLaunch("argsort");
}

}  // namespace k
}  // namespace b200
