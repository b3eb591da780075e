#include "fs_tc.cuh"
namespace fs { namespace tc {
bool supported(int, int, int, int) { return false; }
size_t staged_bytes(int, int, int, int) { return 0; }
cudaError_t stage(Staged&, char*, const float*, const float*, int, int, int, int, cudaStream_t) { return cudaErrorNotSupported; }
cudaError_t lse(const Staged&, int, const StreamArgs&, const LseEpilogue&, cudaStream_t) { return cudaErrorNotSupported; }
}}
