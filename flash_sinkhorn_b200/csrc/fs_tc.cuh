// tcgen05 / TMEM / TMA engine interface (implemented in fs_tc.cu).
#pragma once
#include "fs_common.cuh"

namespace fs {
namespace tc {

// Operands staged for the tensor-core path: K-padded, TF32-rounded copies of the
// two clouds with the per-column bias folded into extra K columns.
struct Staged {
  void* impl = nullptr;
};

bool supported(int n, int m, int d, int prec);
size_t staged_bytes(int n, int m, int d, int prec);
cudaError_t stage(Staged& s, char* buf, const float* x, const float* y, int n, int m, int d, int prec,
                  cudaStream_t st);
cudaError_t lse(const Staged& s, int side, const StreamArgs& a, const LseEpilogue& e, cudaStream_t st);

}  // namespace tc
}  // namespace fs
