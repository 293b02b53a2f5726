// GEMM dispatch: the tcgen05/TMEM kernel takes the 16-bit and fp32 float
// problems whose shapes meet its tiling and TMA alignment rules; everything
// else (tiny, ragged, F64, integer) goes to the SIMT kernel.
#include "../kernels.h"

namespace b200 {
namespace k {

Status gemm_simt(Device* dev, const GemmParams& p);
Status gemm_tcgen05(Device* dev, const GemmParams& p, bool* taken);

Status gemm(Device* dev, const GemmParams& p) {
  if (p.batch < 0 || p.m < 0 || p.n < 0 || p.k < 0) return Status::Invalid("gemm: negative size");
  bool taken = false;
  B200_TRY(gemm_skinny(dev, p, &taken));
  if (taken) return Status::OK();
  B200_TRY(gemm_tcgen05(dev, p, &taken));
  if (taken) return Status::OK();
  return gemm_simt(dev, p);
}

}  // namespace k
}  // namespace b200
