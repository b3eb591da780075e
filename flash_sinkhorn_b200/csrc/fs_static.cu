// fs_apply_mat_static: plan-times-matrix for callers that are not allowed to allocate.
//
// Some hosts of this library cannot hand it a workspace: code that runs inside another
// framework's operator callback where the allocator must not be re-entered, real-time or
// latency-critical loops whose memory was fixed at start-up, and plug-ins that receive only
// input and output buffers from their host application and have no right to call cudaMalloc
// in that process. For them this one entry point keeps its single scratch vector (the per-row
// log2 normaliser that the first streaming pass writes and the second pass reads) in a
// file-scope device array that lives in the library image: every GPU that loads the library
// holds kStaticMaxRows floats (256 KiB) until the process exits.
//
// Consequences of the shared, static scratch:
//  * sizes: the output row count (n for axis 1, m for axis 0) must be <= kStaticMaxRows;
//  * the array keeps whatever the previous call left in it. Nothing has to start at zero:
//    entries [0, rows) are fully rewritten by the first pass before the second pass reads them,
//    and entries beyond `rows` are never read;
//  * two calls that overlap on the same GPU (different streams, or different host threads)
//    race on the array. Serialise them (one stream, or events between streams);
//  * the first call on each device resolves the array's device address with
//    cudaGetSymbolAddress (the symbol's name in host code is only a host-side handle, not a
//    device pointer). Make that first call outside any CUDA stream capture.
// It always uses the CUDA-core fp32 engine (the tensor-core engine needs staged operand copies,
// i.e. a workspace).
#include "../../include/flash_sinkhorn_b200.h"
#include "fs_common.cuh"

#include <mutex>

namespace fs {
int report_error(int code, const char* msg);  // fs_api.cu: records the calling thread's error text
void count_launches(int k);                   // fs_api.cu: adds to the count behind fs_launch_count()
}

namespace {

constexpr int kStaticMaxRows = 1 << 16;
constexpr int kMaxDevices = 64;

static __device__ __align__(256) float g_static_row_offsets[kStaticMaxRows];

std::mutex g_mu;
float* g_dev_ptr[kMaxDevices] = {nullptr};

// Device address of the scratch array on the CURRENT device (resolved once per device).
int static_scratch(float** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fs::report_error(FS_ERR_CUDA, "cudaGetDevice failed");
  if (dev < 0 || dev >= kMaxDevices) return fs::report_error(FS_ERR_UNSUPPORTED, "device ordinal out of range");
  std::lock_guard<std::mutex> lock(g_mu);
  if (!g_dev_ptr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_row_offsets);
    if (e != cudaSuccess || !p)
      return fs::report_error(FS_ERR_CUDA, "cudaGetSymbolAddress(static scratch) failed");
    g_dev_ptr[dev] = static_cast<float*>(p);
  }
  *out = g_dev_ptr[dev];
  return FS_OK;
}

}  // namespace

extern "C" int fs_apply_mat_static(const float* x, const float* y, int n, int m, int d, const float* f_hat,
                                   const float* g_hat, const float* log_a, const float* log_b, const float* mat,
                                   int dv, const float* scale, float* out, float eps, int axis, float cost_scale,
                                   void* stream) {
  using namespace fs;
  if (n <= 0 || m <= 0 || d <= 0 || dv <= 0) return report_error(FS_ERR_BAD_ARG, "n, m, d, dv must be positive");
  if (axis != 0 && axis != 1) return report_error(FS_ERR_BAD_ARG, "axis must be 0 or 1");
  const int rows = axis == 1 ? n : m;
  if (rows > kStaticMaxRows)
    return report_error(FS_ERR_BAD_ARG,
                        "fs_apply_mat_static: output rows exceed the static scratch (65536 rows); "
                        "use fs_apply_mat with a caller-provided workspace");
  if (!x || !y || !f_hat || !g_hat || !log_a || !log_b || !mat || !out)
    return report_error(FS_ERR_BAD_ARG, "null argument");
  if (scale && axis != 1) return report_error(FS_ERR_BAD_ARG, "scale is only supported for axis=1");
  if (!(eps > 0.f) || !(cost_scale > 0.f)) return report_error(FS_ERR_BAD_ARG, "eps and cost_scale must be > 0");
  const int arch = fs_device_arch();
  if (arch < 0) return report_error(FS_ERR_CUDA, "cannot query the current CUDA device");
  if (arch / 10 != 10) return report_error(FS_ERR_UNSUPPORTED, "this library is built for sm_100a only");
  float* R = nullptr;
  int st_code = static_scratch(&R);
  if (st_code != FS_OK) return st_code;
  cudaStream_t st = static_cast<cudaStream_t>(stream);

  const int side = axis == 1 ? 0 : 1;
  StreamArgs s;
  s.rows = side == 0 ? x : y;
  s.cols = side == 0 ? y : x;
  s.nr = side == 0 ? n : m;
  s.nc = side == 0 ? m : n;
  s.d = d;
  s.pot = side == 0 ? g_hat : f_hat;
  s.logw = side == 0 ? log_b : log_a;
  s.eps = eps;
  s.cost_scale = cost_scale;
  LseEpilogue ep;
  ep.lse2 = R;  // pass 1: per-row log2 normaliser into the static array
  if (simt_lse(s, ep, st) != cudaSuccess) return report_error(FS_ERR_CUDA, "first streaming pass failed to launch");
  PvArgs a;
  a.R = R; a.V = mat; a.dv = dv; a.colscale = scale; a.epilogue = PV_APPLY;
  a.rowpot = side == 0 ? f_hat : g_hat;
  a.rowlogw = side == 0 ? log_a : log_b;
  a.out = out;
  if (simt_pv(s, a, st) != cudaSuccess) return report_error(FS_ERR_CUDA, "second streaming pass failed to launch");
  count_launches(2);  // the two streaming passes, as fs_apply_mat counts its own
  return FS_OK;
}
