// RNGBitGenerator: random bits as a pure function of the generator state.
//
// The reference takes its random values from MPSGraph's own generator and only advances the state tensor beside it
// (mpsgraph function.go:1627-1692), so its values cannot be reproduced anywhere else.  Here the values are
// Philox4x32-10 (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3", SC'11): key = the two halves of
// state[0], counter = the 128-bit number (state[2] : state[1]) + block number; block b yields the four 32-bit words
// 4b .. 4b+3 of the stream.  Element e of a 1-, 2- or 4-byte type takes word e (low bits), of an 8-byte type words 2e
// and 2e+1; float types map the top bits of their word(s) to a uniform value in [0, 1):
//   F32 (w >> 8) * 2^-24,  BF16 (w >> 24) * 2^-8,  F16 (w >> 21) * 2^-11,  F64 ((w1 : w0) >> 11) * 2^-53.
// One thread per block of four words; HBM-bound on the write (bytes = output bytes).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "../kernels.h"

namespace b200 {
namespace k {

namespace {

__device__ __forceinline__ void philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0, uint32_t k1, uint32_t* out) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
    const uint32_t n0 = hi1 ^ c1 ^ k0, n1 = lo1, n2 = hi0 ^ c3 ^ k1, n3 = lo0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

__device__ __forceinline__ void store_word_elem(void* y, int64_t e, int dtype, uint32_t w) {
  switch (dtype) {
    case B200_INT8: case B200_UINT8: reinterpret_cast<uint8_t*>(y)[e] = (uint8_t)w; break;
    case B200_INT16: case B200_UINT16: reinterpret_cast<uint16_t*>(y)[e] = (uint16_t)w; break;
    case B200_INT32: case B200_UINT32: reinterpret_cast<uint32_t*>(y)[e] = w; break;
    case B200_FLOAT32: reinterpret_cast<float*>(y)[e] = (float)(w >> 8) * 5.9604644775390625e-08f; break;
    case B200_BFLOAT16: reinterpret_cast<__nv_bfloat16*>(y)[e] = __float2bfloat16_rn((float)(w >> 24) * 0.00390625f); break;
    case B200_FLOAT16: reinterpret_cast<__half*>(y)[e] = __float2half_rn((float)(w >> 21) * 0.00048828125f); break;
    default: break;
  }
}

__global__ void __launch_bounds__(256) rng_kernel(const uint64_t* state, void* y, int dtype, int64_t n, int64_t blocks_total) {
  const uint64_t key = state[0], lo = state[1], hi = state[2];
  const bool wide = dtype == B200_INT64 || dtype == B200_UINT64 || dtype == B200_FLOAT64;
  for (int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; b < blocks_total; b += (int64_t)gridDim.x * blockDim.x) {
    const uint64_t c_lo = lo + (uint64_t)b;
    const uint64_t c_hi = hi + (c_lo < lo ? 1ull : 0ull);
    uint32_t w[4];
    philox4x32_10((uint32_t)c_lo, (uint32_t)(c_lo >> 32), (uint32_t)c_hi, (uint32_t)(c_hi >> 32), (uint32_t)key, (uint32_t)(key >> 32), w);
    if (!wide) {
#pragma unroll
      for (int i = 0; i < 4; ++i)
        if (4 * b + i < n) store_word_elem(y, 4 * b + i, dtype, w[i]);
    } else {
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int64_t e = 2 * b + i;
        if (e >= n) continue;
        const uint64_t v = (uint64_t)w[2 * i] | ((uint64_t)w[2 * i + 1] << 32);
        if (dtype == B200_FLOAT64) reinterpret_cast<double*>(y)[e] = (double)(v >> 11) * 1.1102230246251565e-16;
        else reinterpret_cast<uint64_t*>(y)[e] = v;
      }
    }
  }
}

}  // namespace

Status rng_bits(Device* dev, const void* state, void* y, int dtype, int64_t n) {
  if (n == 0) return Status::OK();
  B200_TRY(dev->MakeCurrent());
  const bool wide = dtype_size(dtype) == 8;
  const int64_t per_block = wide ? 2 : 4;
  const int64_t blocks_total = (n + per_block - 1) / per_block;
  int64_t grid = (blocks_total + 255) / 256;
  const int64_t cap = (int64_t)dev->sm_count() * 16;
  if (grid > cap) grid = cap;
  rng_kernel<<<(unsigned)grid, 256, 0, dev->stream()>>>(reinterpret_cast<const uint64_t*>(state), y, dtype, n, blocks_total);
  return dev->CheckLaunch("rng_bits");
}

}  // namespace k
}  // namespace b200
