// C-ABI layer: argument checks, workspace carving, the solver/CG drivers and the
// small vector kernels that sit between streaming passes. All device work is
// enqueued on the caller's stream; nothing here allocates or synchronises.
#include "../../include/flash_sinkhorn_b200.h"
#include "fs_common.cuh"
#include "fs_tc.cuh"

#include <atomic>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <vector>

namespace fs {
namespace {

thread_local char g_err[512] = "";

// Kernels enqueued by this library since load (all threads); read by fs_launch_count().
std::atomic<long long> g_launches{0};

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

#define FS_CUDA(expr)                                                                      \
  do {                                                                                     \
    cudaError_t _e = (expr);                                                               \
    if (_e != cudaSuccess)                                                                 \
      return fail(FS_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e),     \
                  __FILE__, __LINE__);                                                     \
  } while (0)

#define FS_TRY(expr)                 \
  do {                               \
    int _s = (expr);                 \
    if (_s != FS_OK) return _s;      \
  } while (0)

// ---------------------------------------------------------------------------
// Workspace: bump allocator; with base == nullptr it only measures.
// ---------------------------------------------------------------------------
struct Ws {
  char* base;
  size_t cap;
  size_t off = 0;
  bool overflow = false;
  Ws(void* b, size_t c) : base(static_cast<char*>(b)), cap(c) {}
  template <typename T>
  T* take(size_t count) {
    size_t bytes = (count * sizeof(T) + 255) & ~size_t(255);
    size_t o = off;
    off += bytes;
    if (!base) return nullptr;
    if (off > cap) { overflow = true; return nullptr; }
    return reinterpret_cast<T*>(base + o);
  }
};

// ---------------------------------------------------------------------------
// Small vector kernels
// ---------------------------------------------------------------------------
// out_i = coef * |row_i|^2, one warp per row.
__global__ void sqnorm_kernel(const float* __restrict__ x, int n, int d, float coef, float* __restrict__ out) {
  int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  int lane = threadIdx.x & 31;
  if (warp >= n) return;
  const float* r = x + (size_t)warp * d;
  float s = 0.f;
  for (int k = lane; k < d; k += 32) { float v = r[k]; s = fmaf(v, v, s); }
#pragma unroll
  for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0) out[warp] = coef * s;
}

// out = ca*a + cb*b (a or b may be null => treated as 0)
__global__ void axpby_kernel(int n, float ca, const float* a, float cb, const float* b, float* out) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float v = 0.f;
  if (a) v += ca * a[i];
  if (b) v += cb * b[i];
  out[i] = v;
}

__global__ void fill_kernel(int n, float v, float* out) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = v;
}

__global__ void ctrl_init_kernel(Ctrl* c, int have_prev) {
  c->delta_bits = 0u;
  c->converged = 0;
  c->have_prev = have_prev;
  c->iters_used = 0;
}

__global__ void bump_iters_kernel(Ctrl* c, int only_if_running) {
  if (only_if_running && c->converged) return;
  c->iters_used += 1;
}

// max |cur - prev| over both potentials -> ctrl->delta_bits
__global__ void delta_kernel(const float* f, const float* pf, int n, const float* g, const float* pg, int m,
                             Ctrl* c) {
  if (c->converged || !c->have_prev) return;
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  float d = 0.f;
  if (i < n) d = fabsf(f[i] - pf[i]);
  else if (i < n + m) d = fabsf(g[i - n] - pg[i - n]);
  // NaN compares false everywhere in the reference's `max(...) < threshold`; map NaN to +inf.
  if (d != d) d = INFINITY;
#pragma unroll
  for (int o = 16; o; o >>= 1) d = fmaxf(d, __shfl_xor_sync(0xffffffffu, d, o));
  if ((threadIdx.x & 31) == 0 && d > 0.f) atomicMax(&c->delta_bits, __float_as_uint(d));
}

__global__ void decide_kernel(Ctrl* c, double threshold) {
  if (c->converged) return;
  if (c->have_prev) {
    float d = __uint_as_float(c->delta_bits);
    if ((double)d < threshold) c->converged = 1;
  }
  c->have_prev = 1;
  c->delta_bits = 0u;
}

__global__ void snapshot_kernel(const float* f, float* pf, int n, const float* g, float* pg, int m,
                                const Ctrl* c) {
  if (c->converged) return;
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) pf[i] = f[i];
  else if (i < n + m) pg[i - n] = g[i - n];
}

__global__ void copy_int_kernel(const int* src, int* dst) { *dst = *src; }

inline dim3 g1(int n, int bs = 256) {
  g_launches.fetch_add(1, std::memory_order_relaxed);  // every small-kernel launch sizes its grid here
  return dim3((n + bs - 1) / bs);
}

// ---------------------------------------------------------------------------
// Problem: the two clouds plus engine selection. Side 0 streams rows of x
// against y (f-update, P v); side 1 streams rows of y against x (g-update, P^T v).
// ---------------------------------------------------------------------------
struct Problem {
  const float* x;
  const float* y;
  int n, m, d;
  float cs;
  int prec;
  cudaStream_t st;
  const int* csr_rp[2] = {nullptr, nullptr};
  const int* csr_ci[2] = {nullptr, nullptr};
  tc::Staged staged;  // tcgen05 operands (valid when use_tc)
  bool use_tc = false;
  LabelCost lab;      // V == 0: plain squared-Euclidean cost
  int nlab = 0;       // label-table columns of the tensor-core operands (3V: the table rides in the contraction)

  StreamArgs stream_args(int side, const float* pot, const float* logw, float eps) const {
    StreamArgs s;
    s.rows = side == 0 ? x : y;
    s.cols = side == 0 ? y : x;
    s.nr = side == 0 ? n : m;
    s.nc = side == 0 ? m : n;
    s.d = d;
    s.pot = pot;
    s.logw = logw;
    s.eps = eps;
    s.cost_scale = cs;
    s.tile_row_ptr = csr_rp[side];
    s.tile_col_idx = csr_ci[side];
    if (lab.V > 0) {
      s.lab_rows = lab.lab[side == 0 ? 0 : 1];
      s.lab_cols = lab.lab[side == 0 ? 1 : 0];
      s.W = lab.W; s.V = lab.V; s.lam_w = lab.lam_w;
      s.w_row_major = side == 0 ? 1 : 0;
    }
    s.row_begin = row_lo[side];
    if (row_hi[side] >= 0 && row_hi[side] < s.nr) s.nr = row_hi[side];
    return s;
  }
  // Row sharding: side `s` only produces rows [row_lo[s], row_hi[s]) (row_hi < 0: to the end).
  int row_lo[2] = {0, 0};
  int row_hi[2] = {-1, -1};

  cudaError_t lse(int side, const float* pot, const float* logw, float eps, const LseEpilogue& ep) const {
    StreamArgs s = stream_args(side, pot, logw, eps);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    // Block-sparse tile lists run on the tensor cores when the shape has a 128 x 128 tile plan and the row
    // range starts on a tile boundary; otherwise the CUDA-core engine walks the list.
    const bool tiles_ok = !s.tile_row_ptr || (tc::csr_supported(d, prec, nlab) && (s.row_begin & 127) == 0);
    if (use_tc && tiles_ok) return tc::lse(staged, side, s, ep, st);
    return simt_lse(s, ep, st);
  }
  // Hard c-transform: min_j(-2cs x_i.y_j + bias_j) and its smallest arg-min, rows of `side`.
  cudaError_t argmin(int side, const float* bias, float* out_val, int* out_idx) const {
    StreamArgs s = stream_args(side, bias, nullptr, 1.0f);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    if (use_tc && !tc::k_streamed(d, prec, nlab)) return tc::argmax(staged, side, s, out_val, out_idx, st);
    return simt_argmin(s, out_val, out_idx, st);
  }
  // Weighted pass. With a row normaliser R (log2 LSE of the same scores, from lse()) and the tensor-core
  // engine available it runs as a one-column matrix pass on tcgen05; otherwise on the CUDA-core engine.
  cudaError_t vec(int side, const float* pot, const float* logw, float eps, const VecArgs& v,
                  const float* R = nullptr) const {
    StreamArgs s = stream_args(side, pot, logw, eps);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    if (vec_on_tc() && R) {
      PvArgs pa;
      pa.R = R; pa.V = v.v; pa.dv = 1; pa.epilogue = PV_APPLY;
      pa.rowpot = v.rowpot; pa.rowlogw = v.rowlogw; pa.out = v.out; pa.skip = v.skip;
      return tc::pv(staged, side, s, pa, pv_scratch, st);
    }
    return simt_vec(s, v, st);
  }
  bool vec_on_tc() const {
    return use_tc && pv_scratch && !csr_rp[0] && tc::pv_supported(d, prec, 1, nlab) &&
           tc::pv_scratch_bytes(n > m ? n : m, d, prec, 1, nlab) <= pv_scratch_bytes;
  }
  cudaError_t pv(int side, const float* pot, const float* logw, float eps, const PvArgs& p) const {
    StreamArgs s = stream_args(side, pot, logw, eps);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    if (use_tc && !s.tile_row_ptr && pv_scratch) {
      const int nm = n > m ? n : m;
      const size_t need = p.rows2 ? tc::mat5_scratch_bytes(nm, nm, d, prec, p.dv, nlab)
                                  : (tc::pv_supported(d, prec, p.dv, nlab) ? tc::pv_scratch_bytes(nm, d, prec, p.dv, nlab) : 0);
      if (need > 0 && need <= pv_scratch_bytes) return tc::pv(staged, side, s, p, pv_scratch, st);
    }
    return simt_pv(s, p, st);
  }
  // Row normaliser R (written) followed by the matrix pass over the same scores: gradient, plan-times-matrix.
  cudaError_t lse_pv(int side, const float* pot, const float* logw, float eps, float* R, PvArgs pa) const {
    pa.R = R;
    if (use_tc && mat_streamed && !pa.rows2 && !csr_rp[0]) {
      StreamArgs s = stream_args(side, pot, logw, eps);
      g_launches.fetch_add(3, std::memory_order_relaxed);
      return tc::kstream_mat(staged, side, s, pa, R, pv_scratch, pv_scratch_bytes, st);
    }
    LseEpilogue ep;
    ep.lse2 = R;
    cudaError_t e = lse(side, pot, logw, eps, ep);
    if (e != cudaSuccess) return e;
    return pv(side, pot, logw, eps, pa);
  }
  char* pv_scratch = nullptr;  // transposed copy of V for the tensor-core matrix pass
  size_t pv_scratch_bytes = 0;
  bool mat_streamed = false;   // wide matrix passes of a K-streamed problem: scores kept, weights materialised
};

int check_common(const void* x, const void* y, int n, int m, int d, float eps, float cost_scale, int prec) {
  if (!x || !y) return fail(FS_ERR_BAD_ARG, "x and y must be non-null device pointers");
  if (n <= 0 || m <= 0 || d <= 0) return fail(FS_ERR_BAD_ARG, "n, m, d must be positive (got %d, %d, %d)", n, m, d);
  if (!(eps > 0.f)) return fail(FS_ERR_BAD_ARG, "eps must be > 0 (got %g)", (double)eps);
  if (!(cost_scale > 0.f)) return fail(FS_ERR_BAD_ARG, "cost_scale must be > 0 (got %g)", (double)cost_scale);
  if (prec != FS_PREC_TF32 && prec != FS_PREC_FP32 && prec != FS_PREC_SIMT)
    return fail(FS_ERR_BAD_ARG, "unknown precision mode %d", prec);
  return FS_OK;
}

int check_device() {
  int arch = fs_device_arch();
  if (arch < 0) return fail(FS_ERR_CUDA, "cannot query the current CUDA device");
  if (arch / 10 != 10) return fail(FS_ERR_UNSUPPORTED, "this library is built for sm_100a only; current device is sm_%d", arch);
  return FS_OK;
}

// Sets up `p` (engine choice + staged tcgen05 operands carved from ws).
// `lse_only` is true for ops that only run LSE passes.
int make_problem(Problem& p, Ws& ws, const float* x, const float* y, int n, int m, int d, float cs, int prec,
                 cudaStream_t st, bool measure_only, int pv_dv = 0, bool run_staging = true,
                 const LabelCost* lab = nullptr, bool exact_width = false, bool mat5 = false) {
  p.x = x; p.y = y; p.n = n; p.m = m; p.d = d; p.cs = cs; p.prec = prec; p.st = st;
  if (lab && lab->V > 0) p.lab = *lab;
  p.nlab = 3 * p.lab.V;
  p.use_tc = (prec != FS_PREC_SIMT) && tc::supported(n, m, d, prec, p.nlab);
  if (p.use_tc) {
    size_t bytes = tc::staged_bytes(n, m, d, prec, p.nlab);
    char* buf = ws.take<char>(bytes);
    if (!measure_only) {
      if (ws.overflow) return fail(FS_ERR_WORKSPACE, "workspace too small");
      // staged label entries: logit = scale2 * S with scale2 = 2cs/eps*log2e, so S gets -lam_w*W/(2cs)
      cudaError_t e = tc::stage(p.staged, buf, x, y, n, m, d, prec, st, run_staging, p.lab.V ? &p.lab : nullptr,
                                -p.lab.lam_w / (2.0f * cs));
      if (e != cudaSuccess) return fail(FS_ERR_CUDA, "staging tcgen05 operands failed: %s", cudaGetErrorString(e));
    }
    // Scratch of the matrix pass (transposed V; scores and weights for K-streamed problems). When only sizes
    // are asked for, the matrix may later have any width up to pv_dv, so the largest need is reported; a run
    // takes the scratch only if it fits and otherwise leaves it null (the CUDA-core engine then serves the pass).
    if (pv_dv > 0) {
      const int nm = n > m ? n : m;
      size_t need = 0;
      if (mat5) {
        need = tc::mat5_scratch_bytes(nm, nm, d, prec, pv_dv, p.nlab);
      } else if (tc::k_streamed(d, prec, p.nlab)) {
        // one-column passes take a padded copy of the vector, wide matrices the score / weight scratch, widths
        // in between the transposed matrix of the TMEM-fed second GEMM; the size query covers them all
        const bool any_width = measure_only && !exact_width;
        const int cand[6] = {1, 32, 64, 96, 128, pv_dv};
        for (int c : cand)
          if (c <= pv_dv && (c == pv_dv || any_width)) {
            const size_t b = tc::pv_scratch_bytes(nm, d, prec, c, p.nlab);
            if (b > need) need = b;
          }
        if (pv_dv > 1 && tc::kstream_mat_supported(pv_dv)) {
          const size_t b = tc::kstream_mat_scratch(nm, nm, pv_dv, prec);
          if (b > need) need = b;
          p.mat_streamed = true;
        }
      } else if (measure_only && !exact_width) {
        const int cand[5] = {32, 64, 96, 128, pv_dv};
        for (int c : cand)
          if (c <= pv_dv && tc::pv_supported(d, prec, c, p.nlab)) {
            const size_t b = tc::pv_scratch_bytes(nm, d, prec, c, p.nlab);
            if (b > need) need = b;
          }
      } else if (tc::pv_supported(d, prec, pv_dv, p.nlab)) {
        need = tc::pv_scratch_bytes(nm, d, prec, pv_dv, p.nlab);
      }
      if (need > 0) {
        if (measure_only) {
          ws.take<char>(need);
        } else if (ws.off + ((need + 255) & ~size_t(255)) <= ws.cap) {
          p.pv_scratch_bytes = need;
          p.pv_scratch = ws.take<char>(need);
        }
      }
      if (!p.pv_scratch) p.mat_streamed = false;
    }
  }
  return FS_OK;
}

struct SolveBufs {
  float *alpha, *beta, *fh[2], *gh[2], *pf, *pg, *zeros_n, *zeros_m;
  Ctrl* ctrl;
};

void carve_solve(Ws& ws, SolveBufs& b, int n, int m) {
  b.ctrl = ws.take<Ctrl>(1);
  b.alpha = ws.take<float>(n);
  b.beta = ws.take<float>(m);
  for (int i = 0; i < 2; ++i) { b.fh[i] = ws.take<float>(n); b.gh[i] = ws.take<float>(m); }
  b.pf = ws.take<float>(n);
  b.pg = ws.take<float>(m);
  b.zeros_n = ws.take<float>(n);
  b.zeros_m = ws.take<float>(m);
}

// C-ABI label-cost descriptor -> engine form. Returns false on an inconsistent descriptor.
// Kernels then run with cost scale cs*lambda_x on the dot term and subtract lambda_y*cs*W/eps from the logit
// (reference kernels/sinkhorn_flashstyle_sqeuclid.py:545-560).
inline bool label_cost_from_abi(const fs_label_cost* in, float cost_scale, LabelCost& out, float& cs_kernel) {
  cs_kernel = cost_scale;
  if (!in || in->V <= 0 || in->lambda_y == 0.f) return true;
  if (!in->label_x || !in->label_y || !in->W || !(in->lambda_x > 0.f)) return false;
  out.lab[0] = in->label_x; out.lab[1] = in->label_y; out.W = in->W; out.V = in->V;
  out.lam_w = in->lambda_y * cost_scale;
  cs_kernel = cost_scale * in->lambda_x;
  return true;
}

inline double dampening(double eps, double rho) {
  if (!(rho >= 0.0)) return 1.0;  // negative or NaN: balanced
  return 1.0 / (1.0 + eps / rho);
}

}  // namespace
}  // namespace fs

namespace fs {
// Lets the other translation units of the library record an error for fs_last_error().
int report_error(int code, const char* msg) { return fail(code, "%s", msg); }
// Lets them add the kernels they enqueue themselves to the count behind fs_launch_count().
void count_launches(int k) { g_launches.fetch_add(k, std::memory_order_relaxed); }
}  // namespace fs

using namespace fs;

extern "C" {

int fs_version(void) { return 200; }  // 0.2.0

long long fs_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int fs_device_error(void) { return tc::read_error_flag(); }

int fs_clear_device_error(void) { return tc::clear_error_flag(); }

size_t fs_apply_mat_plan_bytes(int n, int m, int d, int dv, int prec) {
  if (n <= 0 || m <= 0 || d <= 0 || dv <= 0) return 0;
  // Same carving as fs_apply_mat performs, without a workspace: what a call with this matrix width takes.
  Ws ws(nullptr, 0);
  Problem p;
  make_problem(p, ws, nullptr, nullptr, n, m, d, 1.f, prec, nullptr, true, dv <= d ? dv : 0, true, nullptr, true);
  ws.take<float>(n > m ? n : m);
  return ws.off;
}

int fs_set_cta_limit(int k) { return tc::set_cta_limit(k); }

int fs_set_wide_tile_min_chunks(int k) { return tc::set_wide_tile_min_chunks(k); }

int fs_set_prefer_streamed(int on) { return tc::set_prefer_streamed(on); }

int fs_set_pv_split(int split) { return tc::set_pv_split(split); }

int fs_engine(int n, int m, int d, int prec) {
  if (prec == FS_PREC_SIMT || !tc::supported(n, m, d, prec, 0)) return 0;
  return tc::k_streamed(d, prec, 0) ? 2 : 1;
}

int fs_plan_pv_split(int rows, int cols, int prec, int sms, int* slots) {
  return tc::plan_pv_split(rows, cols, prec, sms, slots);
}

int fs_plan_ctas(int n_row_blocks, int n_col_tiles, int sms, int reserved, int limit) {
  return tc::plan_ctas(n_row_blocks, n_col_tiles, sms, reserved, limit);
}

const char* fs_last_error(void) { return g_err; }

int fs_device_arch(void) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -1;
  int major = 0, minor = 0;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return -1;
  if (cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev) != cudaSuccess) return -1;
  return major * 10 + minor;
}

size_t fs_workspace_bytes(int op, int n, int m, int d, int prec) {
  return fs_workspace_bytes_labels(op, n, m, d, prec, 0);
}

size_t fs_workspace_bytes_labels(int op, int n, int m, int d, int prec, int n_classes) {
  if (n <= 0 || m <= 0 || d <= 0) return 0;
  Ws ws(nullptr, 0);
  Problem p;
  const bool matrix_op = (op == FS_OP_APPLY_MAT || op == FS_OP_GRAD || op == FS_OP_MAT5);
  const bool vector_op = (op == FS_OP_APPLY_VEC || op == FS_OP_SCHUR);
  LabelCost lc;
  lc.V = n_classes > 0 ? n_classes : 0;  // only the class count matters for sizes
  make_problem(p, ws, nullptr, nullptr, n, m, d, 1.f, prec, nullptr, true, matrix_op ? d : (vector_op ? 1 : 0),
               true, &lc, false, op == FS_OP_MAT5);
  size_t nm = (size_t)(n > m ? n : m);
  switch (op) {
    case FS_OP_LSE:
      ws.take<float>(nm);
      break;
    case FS_OP_STEP:
      ws.take<float>(nm);
      break;
    case FS_OP_SOLVE_SYMMETRIC:
    case FS_OP_SOLVE_ALTERNATING: {
      SolveBufs b;
      carve_solve(ws, b, n, m);
      break;
    }
    case FS_OP_APPLY_VEC:
      ws.take<float>(nm);
      break;
    case FS_OP_APPLY_MAT:
      ws.take<float>(nm);
      ws.take<float>(nm);
      break;
    case FS_OP_GRAD:
      ws.take<float>(n); ws.take<float>(m); ws.take<float>(n); ws.take<float>(m);
      break;
    case FS_OP_MAT5:
      ws.take<float>(n); ws.take<float>(m); ws.take<float>(n); ws.take<float>(m); ws.take<float>(m);
      break;
    case FS_OP_SCHUR:
      ws.take<float>(16);
      for (int i = 0; i < 3; ++i) ws.take<float>(m);
      ws.take<float>(n);
      ws.take<float>(n);
      ws.take<float>(m);
      break;
    default:
      return 0;
  }
  return ws.off + 256;
}

int fs_lse(const float* x, const float* y, int n, int m, int d, const float* pot, const float* logw, float* out,
           float eps, float cost_scale, float damping, int prec, void* wsp, size_t ws_bytes, void* stream) {
  FS_TRY(check_common(x, y, n, m, d, eps, cost_scale, prec));
  if (!pot || !out) return fail(FS_ERR_BAD_ARG, "pot and out must be non-null");
  FS_TRY(check_device());
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  Ws ws(wsp, ws_bytes);
  Problem p;
  FS_TRY(make_problem(p, ws, x, y, n, m, d, cost_scale, prec, st, false));
  LseEpilogue ep;
  ep.damping = damping;
  ep.w = 1.f;
  ep.out = out;
  FS_CUDA(p.lse(0, pot, logw, eps, ep));
  return FS_OK;
}

int fs_c_transform(const float* x, const float* y, int n, int m, int d, const float* bias, float cost_scale,
                   float* out_val, int* out_idx, int prec, void* wsp, size_t ws_bytes, void* stream) {
  FS_TRY(check_common(x, y, n, m, d, 1.0f, cost_scale, prec));
  if (!bias || !out_val || !out_idx) return fail(FS_ERR_BAD_ARG, "bias, out_val and out_idx must be non-null");
  FS_TRY(check_device());
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  Ws ws(wsp, ws_bytes);
  Problem p;
  FS_TRY(make_problem(p, ws, x, y, n, m, d, cost_scale, prec, st, false));
  FS_CUDA(p.argmin(0, bias, out_val, out_idx));
  return FS_OK;
}

int fs_symmetric_step(const float* x, const float* y, int n, int m, int d, const float* f_hat, const float* g_hat,
                      const float* log_a, const float* log_b, float* f_out, float* g_out, const float* alpha_x,
                      const float* beta_y, float eps, float w, float damp_f, float damp_g, float cost_scale,
                      int prec, void* wsp, size_t ws_bytes, void* stream, const fs_label_cost* labels) {
  FS_TRY(check_common(x, y, n, m, d, eps, cost_scale, prec));
  if (!f_hat || !g_hat || !log_a || !log_b || !f_out || !g_out)
    return fail(FS_ERR_BAD_ARG, "potentials, log-weights and outputs must be non-null");
  if (f_out == f_hat || g_out == g_hat) return fail(FS_ERR_BAD_ARG, "outputs must not alias the inputs (Jacobi step)");
  FS_TRY(check_device());
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  Ws ws(wsp, ws_bytes);
  Problem p;
  LabelCost lc;
  float cs_kernel;
  if (!label_cost_from_abi(labels, cost_scale, lc, cs_kernel)) return fail(FS_ERR_BAD_ARG, "invalid label cost descriptor");
  FS_TRY(make_problem(p, ws, x, y, n, m, d, cs_kernel, prec, st, false, 0, true, &lc));
  LseEpilogue ef;
  ef.damping = damp_f; ef.old = f_hat; ef.w = w; ef.out = f_out;
  if (alpha_x && damp_f < 1.f) { ef.shift = alpha_x; ef.shiftcoef = w * (1.f - damp_f); }
  LseEpilogue eg;
  eg.damping = damp_g; eg.old = g_hat; eg.w = w; eg.out = g_out;
  if (beta_y && damp_g < 1.f) { eg.shift = beta_y; eg.shiftcoef = w * (1.f - damp_g); }
  FS_CUDA(p.lse(0, g_hat, log_b, eps, ef));
  FS_CUDA(p.lse(1, f_hat, log_a, eps, eg));
  return FS_OK;
}

int fs_solve_symmetric(const float* x, const float* y, int n, int m, int d, const float* log_a, const float* log_b,
                       const double* eps_list, int n_eps, int last_extrapolation, float cost_scale, double rho_x,
                       double rho_y, double threshold, int check_every, const float* f_init, const float* g_init,
                       float* f, float* g, float* f_pre, float* g_pre, int* iters_used, int prec, void* wsp,
                       size_t ws_bytes, void* stream, const fs_label_cost* labels) {
  if (!eps_list || n_eps <= 0) return fail(FS_ERR_BAD_ARG, "eps_list must be non-empty");
  FS_TRY(check_common(x, y, n, m, d, (float)eps_list[0], cost_scale, prec));
  for (int i = 0; i < n_eps; ++i)
    if (!(eps_list[i] > 0.0)) return fail(FS_ERR_BAD_ARG, "eps_list[%d] must be > 0", i);
  if (!log_a || !log_b || !f || !g) return fail(FS_ERR_BAD_ARG, "log_a, log_b, f, g must be non-null");
  const bool early = threshold >= 0.0;
  if (early && check_every <= 0) return fail(FS_ERR_BAD_ARG, "check_every must be positive");
  FS_TRY(check_device());
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  Ws ws(wsp, ws_bytes);
  Problem p;
  LabelCost lc;
  float cs_kernel;
  if (!label_cost_from_abi(labels, cost_scale, lc, cs_kernel)) return fail(FS_ERR_BAD_ARG, "invalid label cost descriptor");
  // lambda_x scales the dot term only; the shifts alpha, beta below keep the plain cost scale (as the reference does)
  FS_TRY(make_problem(p, ws, x, y, n, m, d, cs_kernel, prec, st, false, 0, true, &lc));
  SolveBufs b;
  carve_solve(ws, b, n, m);
  if (ws.overflow) return fail(FS_ERR_WORKSPACE, "workspace too small: need %zu bytes", ws.off);

  ctrl_init_kernel<<<1, 1, 0, st>>>(b.ctrl, 0);
  sqnorm_kernel<<<g1(n * 32), 256, 0, st>>>(x, n, d, cost_scale, b.alpha);
  sqnorm_kernel<<<g1(m * 32), 256, 0, st>>>(y, m, d, cost_scale, b.beta);
  // f_hat = f_init - alpha (or -alpha)
  axpby_kernel<<<g1(n), 256, 0, st>>>(n, 1.f, f_init, -1.f, b.alpha, b.fh[0]);
  axpby_kernel<<<g1(m), 256, 0, st>>>(m, 1.f, g_init, -1.f, b.beta, b.gh[0]);
  FS_CUDA(cudaGetLastError());

  // Self-transport problem (the debiasing terms OT(a,a), OT(b,b)): same cloud, weights, penalties and
  // initial potentials on both sides. Both Jacobi updates then read identical inputs through the same
  // kernel, so g equals f bit for bit after every step: run one soft-min per step and copy its result.
  const bool self_problem = x == y && n == m && log_a == log_b && f_init == g_init && rho_x == rho_y &&
                            lc.V == 0;  // a label table need not be symmetric: keep both sides then

  int cur = 0;
  auto step = [&](double eps, float w, bool in_loop) -> int {
    float df = (float)dampening(eps, rho_x), dg = (float)dampening(eps, rho_y);
    LseEpilogue ef;
    ef.damping = df; ef.old = b.fh[cur]; ef.w = w; ef.out = b.fh[cur ^ 1];
    if (df < 1.f) { ef.shift = b.alpha; ef.shiftcoef = w * (1.f - df); }
    LseEpilogue eg;
    eg.damping = dg; eg.old = b.gh[cur]; eg.w = w; eg.out = b.gh[cur ^ 1];
    if (dg < 1.f) { eg.shift = b.beta; eg.shiftcoef = w * (1.f - dg); }
    if (in_loop && early) { ef.ctrl = b.ctrl; eg.ctrl = b.ctrl; }
    FS_CUDA(p.lse(0, b.gh[cur], log_b, (float)eps, ef));
    if (self_problem) {
      FS_CUDA(cudaMemcpyAsync(b.gh[cur ^ 1], b.fh[cur ^ 1], sizeof(float) * (size_t)n, cudaMemcpyDeviceToDevice, st));
    } else {
      FS_CUDA(p.lse(1, b.fh[cur], log_a, (float)eps, eg));
    }
    bump_iters_kernel<<<1, 1, 0, st>>>(b.ctrl, in_loop && early ? 1 : 0);
    cur ^= 1;
    return FS_OK;
  };

  FS_TRY(step(eps_list[0], 1.0f, false));
  for (int it = 0; it < n_eps; ++it) {
    FS_TRY(step(eps_list[it], 0.5f, true));
    if (early && (it + 1) % check_every == 0) {
      delta_kernel<<<g1(n + m), 256, 0, st>>>(b.fh[cur], b.pf, n, b.gh[cur], b.pg, m, b.ctrl);
      decide_kernel<<<1, 1, 0, st>>>(b.ctrl, threshold);
      snapshot_kernel<<<g1(n + m), 256, 0, st>>>(b.fh[cur], b.pf, n, b.gh[cur], b.pg, m, b.ctrl);
    }
  }
  if (last_extrapolation) {
    if (f_pre) axpby_kernel<<<g1(n), 256, 0, st>>>(n, 1.f, b.fh[cur], 1.f, b.alpha, f_pre);
    if (g_pre) axpby_kernel<<<g1(m), 256, 0, st>>>(m, 1.f, b.gh[cur], 1.f, b.beta, g_pre);
    FS_TRY(step(eps_list[n_eps - 1], 1.0f, false));
  }
  axpby_kernel<<<g1(n), 256, 0, st>>>(n, 1.f, b.fh[cur], 1.f, b.alpha, f);
  axpby_kernel<<<g1(m), 256, 0, st>>>(m, 1.f, b.gh[cur], 1.f, b.beta, g);
  if (!last_extrapolation) {
    if (f_pre) axpby_kernel<<<g1(n), 256, 0, st>>>(n, 1.f, b.fh[cur], 1.f, b.alpha, f_pre);
    if (g_pre) axpby_kernel<<<g1(m), 256, 0, st>>>(m, 1.f, b.gh[cur], 1.f, b.beta, g_pre);
  }
  if (iters_used) copy_int_kernel<<<1, 1, 0, st>>>(&b.ctrl->iters_used, iters_used);
  FS_CUDA(cudaGetLastError());
  return FS_OK;
}

int fs_solve_alternating(const float* x, const float* y, int n, int m, int d, const float* log_a,
                         const float* log_b, const double* eps_list, int n_eps, int iters_per_eps,
                         float cost_scale, double rho_x, double rho_y, int ott_convention, double threshold,
                         int check_every, const int* tile_row_ptr, const int* tile_col_idx,
                         const int* tile_row_ptr_t, const int* tile_col_idx_t, float* f, float* g,
                         int* iters_used, int prec, void* wsp, size_t ws_bytes, void* stream) {
  if (!eps_list || n_eps <= 0) return fail(FS_ERR_BAD_ARG, "eps_list must be non-empty");
  FS_TRY(check_common(x, y, n, m, d, (float)eps_list[0], cost_scale, prec));
  for (int i = 0; i < n_eps; ++i)
    if (!(eps_list[i] > 0.0)) return fail(FS_ERR_BAD_ARG, "eps_list[%d] must be > 0", i);
  if (iters_per_eps < 0) return fail(FS_ERR_BAD_ARG, "iters_per_eps must be >= 0");
  if (!log_a || !log_b || !f || !g) return fail(FS_ERR_BAD_ARG, "log_a, log_b, f, g must be non-null");
  if ((tile_row_ptr != nullptr) != (tile_row_ptr_t != nullptr) || (tile_row_ptr != nullptr) != (tile_col_idx != nullptr) ||
      (tile_row_ptr_t != nullptr) != (tile_col_idx_t != nullptr))
    return fail(FS_ERR_BAD_ARG, "tile lists: pass all four CSR arrays (tile list and its transpose) or none");
  const bool early = threshold >= 0.0;
  if (early && check_every <= 0) return fail(FS_ERR_BAD_ARG, "check_every must be positive");
  FS_TRY(check_device());
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  Ws ws(wsp, ws_bytes);
  Problem p;
  FS_TRY(make_problem(p, ws, x, y, n, m, d, cost_scale, prec, st, false));
  p.csr_rp[0] = tile_row_ptr; p.csr_ci[0] = tile_col_idx;
  p.csr_rp[1] = tile_row_ptr_t; p.csr_ci[1] = tile_col_idx_t;
  SolveBufs b;
  carve_solve(ws, b, n, m);
  if (ws.overflow) return fail(FS_ERR_WORKSPACE, "workspace too small: need %zu bytes", ws.off);

  ctrl_init_kernel<<<1, 1, 0, st>>>(b.ctrl, 1);
  sqnorm_kernel<<<g1(n * 32), 256, 0, st>>>(x, n, d, cost_scale, b.alpha);
  sqnorm_kernel<<<g1(m * 32), 256, 0, st>>>(y, m, d, cost_scale, b.beta);
  float* fh = b.fh[0];
  float* gh = b.gh[0];
  axpby_kernel<<<g1(n), 256, 0, st>>>(n, 0.f, nullptr, -1.f, b.alpha, fh);
  axpby_kernel<<<g1(m), 256, 0, st>>>(m, 0.f, nullptr, -1.f, b.beta, gh);
  if (early) {
    axpby_kernel<<<g1(n), 256, 0, st>>>(n, 1.f, fh, 0.f, nullptr, b.pf);
    axpby_kernel<<<g1(m), 256, 0, st>>>(m, 1.f, gh, 0.f, nullptr, b.pg);
  }
  if (ott_convention) {
    fill_kernel<<<g1(n), 256, 0, st>>>(n, 0.f, b.zeros_n);
    fill_kernel<<<g1(m), 256, 0, st>>>(m, 0.f, b.zeros_m);
  }
  FS_CUDA(cudaGetLastError());

  int global_it = 0;
  for (int e = 0; e < n_eps; ++e) {
    const double eps = eps_list[e];
    const float df = (float)dampening(eps, rho_x), dg = (float)dampening(eps, rho_y);
    for (int it = 0; it < iters_per_eps; ++it, ++global_it) {
      LseEpilogue ef, eg;
      ef.damping = df; ef.w = 1.f; ef.out = fh;
      eg.damping = dg; eg.w = 1.f; eg.out = gh;
      if (early) { ef.ctrl = b.ctrl; eg.ctrl = b.ctrl; }
      if (ott_convention) {
        // g first, log-marginals outside the LSE (sinkhorn_solvers.py:188-217)
        eg.addvec = log_b; eg.addcoef = (float)eps;
        ef.addvec = log_a; ef.addcoef = (float)eps;
        FS_CUDA(p.lse(1, fh, b.zeros_n, (float)eps, eg));
        FS_CUDA(p.lse(0, gh, b.zeros_m, (float)eps, ef));
      } else {
        FS_CUDA(p.lse(0, gh, log_b, (float)eps, ef));
        FS_CUDA(p.lse(1, fh, log_a, (float)eps, eg));
      }
      bump_iters_kernel<<<1, 1, 0, st>>>(b.ctrl, early ? 1 : 0);
      if (early && (global_it + 1) % check_every == 0) {
        delta_kernel<<<g1(n + m), 256, 0, st>>>(fh, b.pf, n, gh, b.pg, m, b.ctrl);
        decide_kernel<<<1, 1, 0, st>>>(b.ctrl, threshold);
        snapshot_kernel<<<g1(n + m), 256, 0, st>>>(fh, b.pf, n, gh, b.pg, m, b.ctrl);
      }
    }
  }
  axpby_kernel<<<g1(n), 256, 0, st>>>(n, 1.f, fh, 1.f, b.alpha, f);
  axpby_kernel<<<g1(m), 256, 0, st>>>(m, 1.f, gh, 1.f, b.beta, g);
  if (iters_used) copy_int_kernel<<<1, 1, 0, st>>>(&b.ctrl->iters_used, iters_used);
  FS_CUDA(cudaGetLastError());
  return FS_OK;
}

int fs_apply_vec(const float* x, const float* y, int n, int m, int d, const float* f_hat, const float* g_hat,
                 const float* log_a, const float* log_b, const float* vec, float* out, float eps, int axis,
                 float cost_scale, int prec, void* wsp, size_t ws_bytes, void* stream) {
  FS_TRY(check_common(x, y, n, m, d, eps, cost_scale, prec));
  if (axis != 0 && axis != 1) return fail(FS_ERR_BAD_ARG, "axis must be 0 or 1");
  if (!f_hat || !g_hat || !log_a || !log_b || !vec || !out) return fail(FS_ERR_BAD_ARG, "null argument");
  FS_TRY(check_device());
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  Ws ws(wsp, ws_bytes);
  Problem p;
  FS_TRY(make_problem(p, ws, x, y, n, m, d, cost_scale, prec, st, false, 1));
  float* R = ws.take<float>(n > m ? n : m);
  if (ws.overflow) return fail(FS_ERR_WORKSPACE, "workspace too small: need %zu bytes", ws.off);
  VecArgs v;
  v.v = vec; v.out = out;
  const int side = axis == 1 ? 0 : 1;
  const float* cpot = side == 0 ? g_hat : f_hat;
  const float* clw = side == 0 ? log_b : log_a;
  v.rowpot = side == 0 ? f_hat : g_hat;
  v.rowlogw = side == 0 ? log_a : log_b;
  const float* Rp = nullptr;
  if (p.vec_on_tc()) {  // normaliser pass first, then the weighted pass re-uses the same scores
    LseEpilogue ep;
    ep.lse2 = R;
    FS_CUDA(p.lse(side, cpot, clw, eps, ep));
    Rp = R;
  }
  FS_CUDA(p.vec(side, cpot, clw, eps, v, Rp));
  return FS_OK;
}

int fs_apply_mat(const float* x, const float* y, int n, int m, int d, const float* f_hat, const float* g_hat,
                 const float* log_a, const float* log_b, const float* mat, int dv, const float* scale, float* out,
                 float eps, int axis, float cost_scale, int prec, void* wsp, size_t ws_bytes, void* stream) {
  FS_TRY(check_common(x, y, n, m, d, eps, cost_scale, prec));
  if (axis != 0 && axis != 1) return fail(FS_ERR_BAD_ARG, "axis must be 0 or 1");
  if (dv <= 0) return fail(FS_ERR_BAD_ARG, "dv must be positive");
  if (scale && axis != 1) return fail(FS_ERR_BAD_ARG, "scale is only supported for axis=1");
  if (!f_hat || !g_hat || !log_a || !log_b || !mat || !out) return fail(FS_ERR_BAD_ARG, "null argument");
  FS_TRY(check_device());
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  Ws ws(wsp, ws_bytes);
  Problem p;
  FS_TRY(make_problem(p, ws, x, y, n, m, d, cost_scale, prec, st, false, dv <= d ? dv : 0));
  const int side = axis == 1 ? 0 : 1;
  const int nr = side == 0 ? n : m;
  float* R = ws.take<float>(n > m ? n : m);
  if (ws.overflow) return fail(FS_ERR_WORKSPACE, "workspace too small: need %zu bytes", ws.off);
  (void)nr;
  const float* cpot = side == 0 ? g_hat : f_hat;
  const float* clw = side == 0 ? log_b : log_a;
  // The normaliser R and the weights must come from the same engine (bit-identical scores).
  if (p.use_tc && !p.pv_scratch) p.use_tc = false;
  PvArgs a;
  a.V = mat; a.dv = dv; a.colscale = scale; a.epilogue = PV_APPLY;
  a.rowpot = side == 0 ? f_hat : g_hat;
  a.rowlogw = side == 0 ? log_a : log_b;
  a.out = out;
  FS_CUDA(p.lse_pv(side, cpot, clw, eps, R, a));
  return FS_OK;
}

int fs_grad(const float* x, const float* y, int n, int m, int d, const float* a, const float* b,
            const float* log_a, const float* log_b, const float* f, const float* g, const float* grad_scale,
            float* grad_x, float* grad_y, float eps, float cost_scale, int prec, void* wsp, size_t ws_bytes,
            void* stream, const fs_label_cost* labels) {
  FS_TRY(check_common(x, y, n, m, d, eps, cost_scale, prec));
  if (!a || !b || !log_a || !log_b || !f || !g) return fail(FS_ERR_BAD_ARG, "null argument");
  FS_TRY(check_device());
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  Ws ws(wsp, ws_bytes);
  Problem p;
  LabelCost lc;
  {
    // The gradient kernels of the reference scale the WHOLE squared distance by lambda_x
    // (kernels/sinkhorn_triton_grad_sqeuclid.py:236, :275): from here on cost_scale means cs*lambda_x.
    const float cs_plain = cost_scale;
    if (!label_cost_from_abi(labels, cs_plain, lc, cost_scale)) return fail(FS_ERR_BAD_ARG, "invalid label cost descriptor");
  }
  FS_TRY(make_problem(p, ws, x, y, n, m, d, cost_scale, prec, st, false, d, true, &lc));
  // The normaliser R and the weights must come from the same engine (bit-identical scores).
  if (p.use_tc && !p.pv_scratch) p.use_tc = false;
  float* fh = ws.take<float>(n);
  float* gh = ws.take<float>(m);
  float* Rn = ws.take<float>(n);
  float* Rm = ws.take<float>(m);
  if (ws.overflow) return fail(FS_ERR_WORKSPACE, "workspace too small: need %zu bytes", ws.off);
  // Shifted potentials: the row-constant part of (g_j - C_ij)/eps cancels in the softmax.
  if (grad_x) {
    sqnorm_kernel<<<g1(m * 32), 256, 0, st>>>(y, m, d, cost_scale, Rm);
    axpby_kernel<<<g1(m), 256, 0, st>>>(m, 1.f, g, -1.f, Rm, gh);
    PvArgs pa;
    pa.V = y; pa.dv = d; pa.epilogue = PV_GRAD; pa.roww = a; pa.gs = grad_scale;
    pa.coef = 2.f * cost_scale; pa.out = grad_x;
    FS_CUDA(p.lse_pv(0, gh, log_b, eps, Rn, pa));
  }
  if (grad_y) {
    sqnorm_kernel<<<g1(n * 32), 256, 0, st>>>(x, n, d, cost_scale, Rn);
    axpby_kernel<<<g1(n), 256, 0, st>>>(n, 1.f, f, -1.f, Rn, fh);
    PvArgs pa;
    pa.V = x; pa.dv = d; pa.epilogue = PV_GRAD; pa.roww = b; pa.gs = grad_scale;
    pa.coef = 2.f * cost_scale; pa.out = grad_y;
    FS_CUDA(p.lse_pv(1, fh, log_a, eps, Rm, pa));
  }
  FS_CUDA(cudaGetLastError());
  return FS_OK;
}

int fs_mat5(const float* x, const float* y, int n, int m, int d, const float* f_ott, const float* g_ott,
            const float* A, float* out, float eps, float cost_scale, int prec, void* wsp, size_t ws_bytes,
            void* stream) {
  FS_TRY(check_common(x, y, n, m, d, eps, cost_scale, prec));
  if (!f_ott || !g_ott || !A || !out) return fail(FS_ERR_BAD_ARG, "null argument");
  FS_TRY(check_device());
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  Ws ws(wsp, ws_bytes);
  Problem p;
  FS_TRY(make_problem(p, ws, x, y, n, m, d, cost_scale, prec, st, false, d, true, nullptr, false, true));
  float* fh = ws.take<float>(n);
  float* gh = ws.take<float>(m);
  float* R = ws.take<float>(n);
  float* tmp = ws.take<float>(m);
  float* zeros_m = ws.take<float>(m);
  if (ws.overflow) return fail(FS_ERR_WORKSPACE, "workspace too small: need %zu bytes", ws.off);
  sqnorm_kernel<<<g1(n * 32), 256, 0, st>>>(x, n, d, cost_scale, R);
  axpby_kernel<<<g1(n), 256, 0, st>>>(n, 1.f, f_ott, -1.f, R, fh);
  sqnorm_kernel<<<g1(m * 32), 256, 0, st>>>(y, m, d, cost_scale, tmp);
  axpby_kernel<<<g1(m), 256, 0, st>>>(m, 1.f, g_ott, -1.f, tmp, gh);
  fill_kernel<<<g1(m), 256, 0, st>>>(m, 0.f, zeros_m);
  LseEpilogue ep;
  ep.lse2 = R;
  FS_CUDA(p.lse(0, gh, zeros_m, eps, ep));
  PvArgs pa;
  pa.R = R; pa.rows2 = A; pa.V = y; pa.dv = d; pa.epilogue = PV_MAT5;
  pa.rowpot = fh; pa.rowlogw = nullptr; pa.coef = -4.f * cost_scale / eps; pa.out = out;
  FS_CUDA(p.pv(0, gh, zeros_m, eps, pa));
  FS_CUDA(cudaGetLastError());
  return FS_OK;
}

}  // extern "C"

extern "C" int fs_symmetric_step_range(const float* x, const float* y, int n, int m, int d, const float* f_hat,
                                       const float* g_hat, const float* log_a, const float* log_b, float* f_out,
                                       float* g_out, const float* alpha_x, const float* beta_y, float eps, float w,
                                       float damp_f, float damp_g, float cost_scale, int f_begin, int f_end,
                                       int g_begin, int g_end, int restage, int prec, void* wsp, size_t ws_bytes,
                                       void* stream) {
  return fs_symmetric_step_range_tiles(x, y, n, m, d, f_hat, g_hat, log_a, log_b, f_out, g_out, alpha_x, beta_y, eps,
                                       w, damp_f, damp_g, cost_scale, f_begin, f_end, g_begin, g_end, restage,
                                       nullptr, nullptr, nullptr, nullptr, prec, wsp, ws_bytes, stream);
}

extern "C" int fs_symmetric_step_range_tiles(const float* x, const float* y, int n, int m, int d, const float* f_hat,
                                             const float* g_hat, const float* log_a, const float* log_b,
                                             float* f_out, float* g_out, const float* alpha_x, const float* beta_y,
                                             float eps, float w, float damp_f, float damp_g, float cost_scale,
                                             int f_begin, int f_end, int g_begin, int g_end, int restage,
                                             const int* tile_row_ptr, const int* tile_col_idx,
                                             const int* tile_row_ptr_t, const int* tile_col_idx_t, int prec,
                                             void* wsp, size_t ws_bytes, void* stream) {
  if ((tile_row_ptr != nullptr) != (tile_row_ptr_t != nullptr) || (tile_row_ptr != nullptr) != (tile_col_idx != nullptr) ||
      (tile_row_ptr_t != nullptr) != (tile_col_idx_t != nullptr))
    return fail(FS_ERR_BAD_ARG, "tile lists: pass all four CSR arrays (tile list and its transpose) or none");
  if (tile_row_ptr && ((f_begin & 127) || (g_begin & 127)))
    return fail(FS_ERR_BAD_ARG, "with tile lists the row ranges must start on multiples of 128");
  FS_TRY(check_common(x, y, n, m, d, eps, cost_scale, prec));
  if (!f_hat || !g_hat || !log_a || !log_b || !f_out || !g_out)
    return fail(FS_ERR_BAD_ARG, "potentials, log-weights and outputs must be non-null");
  if (f_out == f_hat || g_out == g_hat) return fail(FS_ERR_BAD_ARG, "outputs must not alias the inputs (Jacobi step)");
  if (f_begin < 0 || f_end > n || g_begin < 0 || g_end > m || f_begin > f_end || g_begin > g_end)
    return fail(FS_ERR_BAD_ARG, "row ranges must satisfy 0 <= begin <= end <= rows");
  FS_TRY(check_device());
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  Ws ws(wsp, ws_bytes);
  Problem p;
  FS_TRY(make_problem(p, ws, x, y, n, m, d, cost_scale, prec, st, false, 0, restage != 0));
  p.row_lo[0] = f_begin; p.row_hi[0] = f_end;
  p.row_lo[1] = g_begin; p.row_hi[1] = g_end;
  p.csr_rp[0] = tile_row_ptr; p.csr_ci[0] = tile_col_idx;
  p.csr_rp[1] = tile_row_ptr_t; p.csr_ci[1] = tile_col_idx_t;
  LseEpilogue ef;
  ef.damping = damp_f; ef.old = f_hat; ef.w = w; ef.out = f_out;
  if (alpha_x && damp_f < 1.f) { ef.shift = alpha_x; ef.shiftcoef = w * (1.f - damp_f); }
  LseEpilogue eg;
  eg.damping = damp_g; eg.old = g_hat; eg.w = w; eg.out = g_out;
  if (beta_y && damp_g < 1.f) { eg.shift = beta_y; eg.shiftcoef = w * (1.f - damp_g); }
  if (f_end > f_begin) FS_CUDA(p.lse(0, g_hat, log_b, eps, ef));
  if (g_end > g_begin) FS_CUDA(p.lse(1, f_hat, log_a, eps, eg));
  return FS_OK;
}

extern "C" int fs_symmetric_step_multi(const fs_step_item* items, int n_items, int d, int prec, void* stream) {
  constexpr int kMaxItems = 8;
  if (!items || n_items <= 0 || n_items > kMaxItems)
    return fail(FS_ERR_BAD_ARG, "fs_symmetric_step_multi takes 1..%d items", kMaxItems);
  FS_TRY(check_device());
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  Problem probs[kMaxItems];
  tc::MultiPass passes[2 * kMaxItems];
  int n_pass = 0;
  bool all_tc = true;
  for (int i = 0; i < n_items; ++i) {
    const fs_step_item& it = items[i];
    FS_TRY(check_common(it.x, it.y, it.n, it.m, d, it.eps, it.cost_scale, prec));
    if (!it.f_hat || !it.g_hat || !it.log_a || !it.log_b || !it.f_out || !it.g_out)
      return fail(FS_ERR_BAD_ARG, "item %d: potentials, log-weights and outputs must be non-null", i);
    if (it.f_out == it.f_hat || it.g_out == it.g_hat)
      return fail(FS_ERR_BAD_ARG, "item %d: outputs must not alias the inputs (Jacobi step)", i);
    if (it.f_begin < 0 || it.f_end > it.n || it.g_begin < 0 || it.g_end > it.m || it.f_begin > it.f_end ||
        it.g_begin > it.g_end)
      return fail(FS_ERR_BAD_ARG, "item %d: row ranges must satisfy 0 <= begin <= end <= rows", i);
    // Packed potentials: element j of f_hat lives at f_hat[(j / f_shard) * pack_stride + j % f_shard] (same for
    // g_hat, f_out, g_out). The rows a pass produces lie inside ONE shard, so for them - the old values that are
    // averaged in, the outputs - the packed vector is an ordinary contiguous one behind a shifted pointer.
    const bool packed = it.f_shard > 0 || it.g_shard > 0;
    if (packed && (it.f_shard <= 0 || it.g_shard <= 0 || it.pack_stride <= 0))
      return fail(FS_ERR_BAD_ARG, "item %d: packed potentials need f_shard, g_shard and pack_stride > 0", i);
    if (packed && ((it.f_end > it.f_begin && (it.f_end - 1) / it.f_shard != it.f_begin / it.f_shard) ||
                   (it.g_end > it.g_begin && (it.g_end - 1) / it.g_shard != it.g_begin / it.g_shard)))
      return fail(FS_ERR_BAD_ARG, "item %d: a row range must lie inside one shard of the packed layout", i);
    auto rows_alias = [&](const float* base, int shard, int begin) -> const float* {
      if (!packed || !base) return base;
      const long long q = begin / shard;
      return base + q * it.pack_stride - q * shard;
    };
    Ws ws(it.ws, it.ws_bytes);
    Problem& p = probs[i];
    FS_TRY(make_problem(p, ws, it.x, it.y, it.n, it.m, d, it.cost_scale, prec, st, false, 0, it.restage != 0));
    if (packed && !p.use_tc)
      return fail(FS_ERR_UNSUPPORTED, "item %d: packed potentials are read by the tensor-core engine only", i);
    p.row_lo[0] = it.f_begin; p.row_hi[0] = it.f_end;
    p.row_lo[1] = it.g_begin; p.row_hi[1] = it.g_end;
    all_tc = all_tc && p.use_tc;
    for (int side = 0; side < 2; ++side) {
      const int lo = side == 0 ? it.f_begin : it.g_begin, hi = side == 0 ? it.f_end : it.g_end;
      if (hi <= lo) continue;
      tc::MultiPass& mp = passes[n_pass++];
      mp.s = &p.staged;
      mp.side = side;
      mp.a = p.stream_args(side, side == 0 ? it.g_hat : it.f_hat, side == 0 ? it.log_b : it.log_a, it.eps);
      LseEpilogue ep;
      const float damp = side == 0 ? it.damp_f : it.damp_g;
      const float* shift = side == 0 ? it.alpha_x : it.beta_y;
      const int shard = side == 0 ? it.f_shard : it.g_shard;
      ep.damping = damp; ep.w = it.w;
      ep.old = rows_alias(side == 0 ? it.f_hat : it.g_hat, shard, lo);
      ep.out = const_cast<float*>(rows_alias(side == 0 ? it.f_out : it.g_out, shard, lo));
      if (packed) {  // the column potential of this pass is the OTHER side's packed vector
        mp.a.pot_shard = side == 0 ? it.g_shard : it.f_shard;
        mp.a.pot_stride = it.pack_stride;
      }
      if (shift && damp < 1.f) { ep.shift = shift; ep.shiftcoef = it.w * (1.f - damp); }
      mp.e = ep;
    }
  }
  // Groups of passes share a launch when the tensor-core engine takes them that way; otherwise one by one.
  const int group = tc::multi_max();
  for (int k0 = 0; k0 < n_pass; k0 += group) {
    const int cnt = n_pass - k0 < group ? n_pass - k0 : group;
    cudaError_t e = all_tc ? tc::lse_multi(passes + k0, cnt, st) : cudaErrorNotSupported;
    if (e == cudaSuccess) {
      g_launches.fetch_add(2, std::memory_order_relaxed);
      continue;
    }
    if (e != cudaErrorNotSupported)
      return fail(FS_ERR_CUDA, "multi-pass launch failed: %s", cudaGetErrorString(e));
    (void)cudaGetLastError();
    for (int k = k0; k < k0 + cnt; ++k) {
      const tc::MultiPass& mp = passes[k];
      const Problem* owner = nullptr;
      for (int i = 0; i < n_items; ++i)
        if (&probs[i].staged == mp.s) owner = &probs[i];
      g_launches.fetch_add(1, std::memory_order_relaxed);
      // (the stream arguments carry the packed-potential addressing, so they are passed on as they are)
      FS_CUDA(owner->use_tc ? tc::lse(*mp.s, mp.side, mp.a, mp.e, st) : simt_lse(mp.a, mp.e, st));
    }
  }
  return FS_OK;
}

// Several symmetric solves in lockstep (batched inputs, or the three problems of a debiased loss): every step of
// all problems that still have one goes out as fused multi-pass launches, so B small problems cost about one
// solve's worth of launches instead of B. Schedules may differ in length; a finished problem drops out.
extern "C" int fs_solve_symmetric_batched(const fs_batch_item* items, int n_items, int d, int last_extrapolation,
                                          float cost_scale, double rho_x, double rho_y, int prec, void* stream) {
  constexpr int kMaxBatch = 256;
  if (!items || n_items <= 0 || n_items > kMaxBatch)
    return fail(FS_ERR_BAD_ARG, "fs_solve_symmetric_batched takes 1..%d items", kMaxBatch);
  FS_TRY(check_device());
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  struct Item {
    Problem p;
    SolveBufs b;
    int cur = 0, steps = 0;
    bool self_problem = false;
  };
  std::vector<Item> its(n_items);
  int max_steps = 0;
  for (int i = 0; i < n_items; ++i) {
    const fs_batch_item& in = items[i];
    if (!in.eps_list_host || in.n_eps <= 0) return fail(FS_ERR_BAD_ARG, "item %d: eps_list must be non-empty", i);
    FS_TRY(check_common(in.x, in.y, in.n, in.m, d, (float)in.eps_list_host[0], cost_scale, prec));
    for (int k = 0; k < in.n_eps; ++k)
      if (!(in.eps_list_host[k] > 0.0)) return fail(FS_ERR_BAD_ARG, "item %d: eps_list[%d] must be > 0", i, k);
    if (!in.log_a || !in.log_b || !in.f || !in.g) return fail(FS_ERR_BAD_ARG, "item %d: log_a, log_b, f, g must be non-null", i);
    Item& it = its[i];
    Ws ws(in.ws, in.ws_bytes);
    FS_TRY(make_problem(it.p, ws, in.x, in.y, in.n, in.m, d, cost_scale, prec, st, false));
    carve_solve(ws, it.b, in.n, in.m);
    if (ws.overflow) return fail(FS_ERR_WORKSPACE, "item %d: workspace too small: need %zu bytes", i, ws.off);
    it.steps = in.n_eps + 1 + (last_extrapolation ? 1 : 0);
    if (it.steps > max_steps) max_steps = it.steps;
    it.self_problem = in.x == in.y && in.n == in.m && in.log_a == in.log_b && rho_x == rho_y;
    sqnorm_kernel<<<g1(in.n * 32), 256, 0, st>>>(in.x, in.n, d, cost_scale, it.b.alpha);
    sqnorm_kernel<<<g1(in.m * 32), 256, 0, st>>>(in.y, in.m, d, cost_scale, it.b.beta);
    axpby_kernel<<<g1(in.n), 256, 0, st>>>(in.n, 0.f, nullptr, -1.f, it.b.alpha, it.b.fh[0]);
    axpby_kernel<<<g1(in.m), 256, 0, st>>>(in.m, 0.f, nullptr, -1.f, it.b.beta, it.b.gh[0]);
  }
  FS_CUDA(cudaGetLastError());
  std::vector<tc::MultiPass> passes;
  std::vector<int> owner;
  const int group = tc::multi_max();
  for (int t = 0; t < max_steps; ++t) {
    passes.clear();
    owner.clear();
    for (int i = 0; i < n_items; ++i) {
      Item& it = its[i];
      if (t >= it.steps) continue;
      const fs_batch_item& in = items[i];
      const bool first = t == 0, last = last_extrapolation && t == it.steps - 1;
      const double eps = first ? in.eps_list_host[0] : (last ? in.eps_list_host[in.n_eps - 1] : in.eps_list_host[t - 1]);
      const float w = (first || last) ? 1.0f : 0.5f;
      if (last) {  // the potentials before the final extrapolation are part of the result
        if (in.f_pre) axpby_kernel<<<g1(in.n), 256, 0, st>>>(in.n, 1.f, it.b.fh[it.cur], 1.f, it.b.alpha, in.f_pre);
        if (in.g_pre) axpby_kernel<<<g1(in.m), 256, 0, st>>>(in.m, 1.f, it.b.gh[it.cur], 1.f, it.b.beta, in.g_pre);
      }
      const float df = (float)dampening(eps, rho_x), dg = (float)dampening(eps, rho_y);
      for (int side = 0; side < (it.self_problem ? 1 : 2); ++side) {
        tc::MultiPass mp;
        mp.s = &it.p.staged;
        mp.side = side;
        mp.a = it.p.stream_args(side, side == 0 ? it.b.gh[it.cur] : it.b.fh[it.cur], side == 0 ? in.log_b : in.log_a,
                                (float)eps);
        LseEpilogue ep;
        const float damp = side == 0 ? df : dg;
        ep.damping = damp; ep.w = w;
        ep.old = side == 0 ? it.b.fh[it.cur] : it.b.gh[it.cur];
        ep.out = side == 0 ? it.b.fh[it.cur ^ 1] : it.b.gh[it.cur ^ 1];
        if (damp < 1.f) { ep.shift = side == 0 ? it.b.alpha : it.b.beta; ep.shiftcoef = w * (1.f - damp); }
        mp.e = ep;
        passes.push_back(mp);
        owner.push_back(i);
      }
    }
    const int n_pass = (int)passes.size();
    for (int k0 = 0; k0 < n_pass; k0 += group) {
      const int cnt = n_pass - k0 < group ? n_pass - k0 : group;
      bool all_tc = true;
      for (int k = k0; k < k0 + cnt; ++k) all_tc = all_tc && its[owner[k]].p.use_tc;
      cudaError_t e = all_tc ? tc::lse_multi(passes.data() + k0, cnt, st) : cudaErrorNotSupported;
      if (e == cudaSuccess) {
        g_launches.fetch_add(2, std::memory_order_relaxed);
        continue;
      }
      if (e != cudaErrorNotSupported) return fail(FS_ERR_CUDA, "multi-pass launch failed: %s", cudaGetErrorString(e));
      (void)cudaGetLastError();
      for (int k = k0; k < k0 + cnt; ++k) {
        const tc::MultiPass& mp = passes[k];
        const Problem& pr = its[owner[k]].p;
        g_launches.fetch_add(1, std::memory_order_relaxed);
        FS_CUDA(pr.use_tc ? tc::lse(*mp.s, mp.side, mp.a, mp.e, st) : simt_lse(mp.a, mp.e, st));
      }
    }
    for (int i = 0; i < n_items; ++i) {
      Item& it = its[i];
      if (t >= it.steps) continue;
      if (it.self_problem)  // g equals f bit for bit: one soft-min per step, copied
        FS_CUDA(cudaMemcpyAsync(it.b.gh[it.cur ^ 1], it.b.fh[it.cur ^ 1], sizeof(float) * (size_t)items[i].n,
                                cudaMemcpyDeviceToDevice, st));
      it.cur ^= 1;
    }
  }
  for (int i = 0; i < n_items; ++i) {
    const fs_batch_item& in = items[i];
    Item& it = its[i];
    axpby_kernel<<<g1(in.n), 256, 0, st>>>(in.n, 1.f, it.b.fh[it.cur], 1.f, it.b.alpha, in.f);
    axpby_kernel<<<g1(in.m), 256, 0, st>>>(in.m, 1.f, it.b.gh[it.cur], 1.f, it.b.beta, in.g);
    if (!last_extrapolation) {
      if (in.f_pre) axpby_kernel<<<g1(in.n), 256, 0, st>>>(in.n, 1.f, it.b.fh[it.cur], 1.f, it.b.alpha, in.f_pre);
      if (in.g_pre) axpby_kernel<<<g1(in.m), 256, 0, st>>>(in.m, 1.f, it.b.gh[it.cur], 1.f, it.b.beta, in.g_pre);
    }
  }
  FS_CUDA(cudaGetLastError());
  return FS_OK;
}

extern "C" int fs_grad_range(const float* x, const float* y, int n, int m, int d, const float* a, const float* b,
                             const float* log_a, const float* log_b, const float* f, const float* g,
                             const float* grad_scale, float* grad_x, float* grad_y, float eps, float cost_scale,
                             int x_begin, int x_end, int y_begin, int y_end, int prec, void* wsp, size_t ws_bytes,
                             void* stream) {
  FS_TRY(check_common(x, y, n, m, d, eps, cost_scale, prec));
  if (!a || !b || !log_a || !log_b || !f || !g) return fail(FS_ERR_BAD_ARG, "null argument");
  if (x_begin < 0 || x_end > n || y_begin < 0 || y_end > m || x_begin > x_end || y_begin > y_end)
    return fail(FS_ERR_BAD_ARG, "row ranges must satisfy 0 <= begin <= end <= rows");
  FS_TRY(check_device());
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  Ws ws(wsp, ws_bytes);
  Problem p;
  FS_TRY(make_problem(p, ws, x, y, n, m, d, cost_scale, prec, st, false, d));
  if (p.use_tc && !p.pv_scratch) p.use_tc = false;
  p.row_lo[0] = x_begin; p.row_hi[0] = x_end;
  p.row_lo[1] = y_begin; p.row_hi[1] = y_end;
  float* fh = ws.take<float>(n);
  float* gh = ws.take<float>(m);
  float* Rn = ws.take<float>(n);
  float* Rm = ws.take<float>(m);
  if (ws.overflow) return fail(FS_ERR_WORKSPACE, "workspace too small: need %zu bytes", ws.off);
  if (grad_x && x_end > x_begin) {
    sqnorm_kernel<<<g1(m * 32), 256, 0, st>>>(y, m, d, cost_scale, Rm);
    axpby_kernel<<<g1(m), 256, 0, st>>>(m, 1.f, g, -1.f, Rm, gh);
    PvArgs pa;
    pa.V = y; pa.dv = d; pa.epilogue = PV_GRAD; pa.roww = a; pa.gs = grad_scale;
    pa.coef = 2.f * cost_scale; pa.out = grad_x;
    FS_CUDA(p.lse_pv(0, gh, log_b, eps, Rn, pa));
  }
  if (grad_y && y_end > y_begin) {
    sqnorm_kernel<<<g1(n * 32), 256, 0, st>>>(x, n, d, cost_scale, Rn);
    axpby_kernel<<<g1(n), 256, 0, st>>>(n, 1.f, f, -1.f, Rn, fh);
    PvArgs pa;
    pa.V = x; pa.dv = d; pa.epilogue = PV_GRAD; pa.roww = b; pa.gs = grad_scale;
    pa.coef = 2.f * cost_scale; pa.out = grad_y;
    FS_CUDA(p.lse_pv(1, fh, log_a, eps, Rm, pa));
  }
  FS_CUDA(cudaGetLastError());
  return FS_OK;
}

// ---------------------------------------------------------------------------
// Plan session: many applications of ONE transport plan (fixed clouds and potentials) that share the staged
// operands and the two log-normaliser vectors. The Hessian-vector product is the user: its ~50 plan passes
// then cost one streaming pass each.
// ---------------------------------------------------------------------------
namespace fs {
namespace {

struct Session {
  Problem p;
  float* R[2] = {nullptr, nullptr};  // log2 normalisers of the rows of x (side 0) and of y (side 1)
  float* cg = nullptr;               // state and vectors of the Schur CG
  float eps = 1.f;
};

// Lays the session out inside `ws` (identical for every call with the same sizes); stages when asked to.
int open_session(Session& se, Ws& ws, const float* x, const float* y, int n, int m, int d, float eps, float cs,
                 int prec, cudaStream_t st, bool stage, bool measure_only) {
  se.eps = eps;
  Problem& p = se.p;
  FS_TRY(make_problem(p, ws, x, y, n, m, d, cs, prec, st, measure_only, 0, stage));
  if (p.use_tc) {
    const int nm = n > m ? n : m;
    size_t need = tc::mat5_scratch_bytes(nm, nm, d, prec, d, 0);
    const int widths[6] = {1, 32, 64, 96, 128, d};
    for (int w : widths)
      if (w <= d && tc::pv_supported(d, prec, w, 0)) {
        const size_t b = tc::pv_scratch_bytes(nm, d, prec, w, 0);
        if (b > need) need = b;
      }
    if (tc::k_streamed(d, prec, 0) && tc::kstream_mat_supported(d)) {
      const size_t b = tc::kstream_mat_scratch(nm, nm, d, prec);
      if (b > need) need = b;
      p.mat_streamed = true;
    }
    p.pv_scratch_bytes = need;
    p.pv_scratch = ws.take<char>(need);
  }
  se.R[0] = ws.take<float>(n);
  se.R[1] = ws.take<float>(m);
  se.cg = ws.take<float>(16 + 3 * (size_t)m + (size_t)n);
  if (!measure_only && ws.overflow) return fail(FS_ERR_WORKSPACE, "workspace too small: need %zu bytes", ws.off);
  return FS_OK;
}

}  // namespace
}  // namespace fs

extern "C" size_t fs_plan_session_bytes(int n, int m, int d, int prec) {
  if (n <= 0 || m <= 0 || d <= 0) return 0;
  Ws ws(nullptr, 0);
  Session se;
  open_session(se, ws, nullptr, nullptr, n, m, d, 1.f, 1.f, prec, nullptr, false, true);
  return ws.off + 256;
}

extern "C" int fs_plan_session_begin(const float* x, const float* y, int n, int m, int d, const float* f_hat,
                                     const float* g_hat, const float* log_a, const float* log_b, float eps,
                                     float cost_scale, int prec, void* wsp, size_t ws_bytes, void* stream) {
  FS_TRY(check_common(x, y, n, m, d, eps, cost_scale, prec));
  if (!f_hat || !g_hat || !log_a || !log_b) return fail(FS_ERR_BAD_ARG, "null argument");
  FS_TRY(check_device());
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  Ws ws(wsp, ws_bytes);
  Session se;
  FS_TRY(open_session(se, ws, x, y, n, m, d, eps, cost_scale, prec, st, true, false));
  LseEpilogue e0, e1;
  e0.lse2 = se.R[0];
  e1.lse2 = se.R[1];
  FS_CUDA(se.p.lse(0, g_hat, log_b, eps, e0));
  FS_CUDA(se.p.lse(1, f_hat, log_a, eps, e1));
  return FS_OK;
}

// One plan application inside a session. kind 0: vector (operand [cols], out [rows]); 1: matrix with dv columns and
// an optional per-column-point scale (axis 1 only); 2: the Mat5 term (operand A [n, d], axis 1, dv = d).
extern "C" int fs_plan_session_apply(const float* x, const float* y, int n, int m, int d, const float* f_hat,
                                     const float* g_hat, const float* log_a, const float* log_b, int kind,
                                     const float* operand, int dv, const float* scale, float coef, float* out,
                                     int axis, float eps, float cost_scale, int prec, void* wsp, size_t ws_bytes,
                                     void* stream) {
  FS_TRY(check_common(x, y, n, m, d, eps, cost_scale, prec));
  if (!f_hat || !g_hat || !log_a || !log_b || !operand || !out) return fail(FS_ERR_BAD_ARG, "null argument");
  if (axis != 0 && axis != 1) return fail(FS_ERR_BAD_ARG, "axis must be 0 or 1");
  if (kind < 0 || kind > 2) return fail(FS_ERR_BAD_ARG, "kind must be 0 (vector), 1 (matrix) or 2 (Mat5)");
  if (kind == 2 && (axis != 1 || dv != d)) return fail(FS_ERR_BAD_ARG, "Mat5 is an axis-1 pass with dv == d");
  if (kind == 1 && (dv <= 0 || dv > d)) return fail(FS_ERR_BAD_ARG, "matrix passes of a session take 1 <= dv <= d");
  if (scale && (axis != 1 || kind != 1)) return fail(FS_ERR_BAD_ARG, "scale is only supported for axis-1 matrix passes");
  FS_TRY(check_device());
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  Ws ws(wsp, ws_bytes);
  Session se;
  FS_TRY(open_session(se, ws, x, y, n, m, d, eps, cost_scale, prec, st, false, false));
  const int side = axis == 1 ? 0 : 1;
  const float* cpot = side == 0 ? g_hat : f_hat;
  const float* clw = side == 0 ? log_b : log_a;
  const float* rpot = side == 0 ? f_hat : g_hat;
  const float* rlw = side == 0 ? log_a : log_b;
  if (kind == 0) {
    VecArgs v;
    v.v = operand; v.out = out; v.rowpot = rpot; v.rowlogw = rlw;
    FS_CUDA(se.p.vec(side, cpot, clw, eps, v, se.p.vec_on_tc() ? se.R[side] : nullptr));
    return FS_OK;
  }
  PvArgs a;
  a.R = se.R[side]; a.V = kind == 2 ? y : operand; a.dv = dv; a.colscale = scale;
  a.epilogue = kind == 2 ? PV_MAT5 : PV_APPLY;
  a.rows2 = kind == 2 ? operand : nullptr;
  a.rowpot = rpot; a.rowlogw = rlw; a.coef = kind == 2 ? coef : 1.f; a.out = out;
  if (kind == 1 && se.p.mat_streamed) {  // wide matrix of a K-streamed problem: scores are kept, R recomputed
    FS_CUDA(se.p.lse_pv(side, cpot, clw, eps, se.R[side], a));
    return FS_OK;
  }
  FS_CUDA(se.p.pv(side, cpot, clw, eps, a));
  return FS_OK;
}

// ---------------------------------------------------------------------------
// Device-resident conjugate gradient on the Schur complement
// ---------------------------------------------------------------------------
namespace fs {
namespace {

struct CgState {
  float rz_old, tol, res, init_res;
  int done, converged, iters, pad;
};

__device__ float block_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (threadIdx.x < (blockDim.x >> 5)) ? red[threadIdx.x] : 0.f;
  if (w == 0) {
#pragma unroll
    for (int o = 16; o; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (l == 0) red[0] = t;
  }
  __syncthreads();
  return red[0];
}

// z = 0, r = p = rhs, rz_old = |r|^2, tol = max(atol, rtol*|r|).  One block.
__global__ void cg_init_kernel(int m, const float* rhs, float* z, float* r, float* pvec, CgState* s, float rtol,
                               float atol) {
  __shared__ float red[32];
  float acc = 0.f;
  for (int i = threadIdx.x; i < m; i += blockDim.x) {
    float v = rhs[i];
    z[i] = 0.f; r[i] = v; pvec[i] = v;
    acc = fmaf(v, v, acc);
  }
  float rr = block_sum(acc, red);
  if (threadIdx.x == 0) {
    s->rz_old = rr;
    s->init_res = sqrtf(rr);
    s->res = s->init_res;
    s->tol = fmaxf(atol, rtol * s->init_res);
    s->done = 0; s->converged = 0; s->iters = 0;
  }
}

// u = t / diag_x  (skipped once done)
__global__ void cg_div_kernel(int n, const float* t, const float* diag, float* u, const CgState* s) {
  if (s->done) return;
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) u[i] = t[i] / diag[i];
}

// One block: Ap = denom*p - q; alpha = rz/(p.Ap); z += alpha p; r -= alpha Ap; test; p = r + beta p.
__global__ void cg_update_kernel(int m, const float* denom, const float* q, float* z, float* r, float* pvec,
                                 CgState* s, int it) {
  __shared__ float red[32];
  if (s->done) return;
  float acc = 0.f;
  for (int i = threadIdx.x; i < m; i += blockDim.x) {
    float ap = denom[i] * pvec[i] - q[i];
    acc = fmaf(pvec[i], ap, acc);
  }
  float pAp = block_sum(acc, red);
  if (pAp == 0.f) {  // reference: `if denom.abs() == 0: break`
    if (threadIdx.x == 0) s->done = 1;
    return;
  }
  float rz_old = s->rz_old;
  float alpha = rz_old / pAp;
  acc = 0.f;
  for (int i = threadIdx.x; i < m; i += blockDim.x) {
    float pi = pvec[i];
    float ap = denom[i] * pi - q[i];
    z[i] = z[i] + alpha * pi;
    float ri = r[i] - alpha * ap;
    r[i] = ri;
    acc = fmaf(ri, ri, acc);
  }
  float rz_new = block_sum(acc, red);
  float res = sqrtf(rz_new);
  bool conv = res <= s->tol;
  if (!conv) {
    float beta = rz_new / rz_old;
    for (int i = threadIdx.x; i < m; i += blockDim.x) pvec[i] = r[i] + beta * pvec[i];
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    s->res = res;
    s->rz_old = rz_new;
    if (conv) { s->done = 1; s->converged = 1; s->iters = it + 1; }
  }
}

__global__ void cg_finish_kernel(const CgState* s, float* info, int max_iter) {
  info[0] = s->converged ? 1.f : 0.f;
  info[1] = s->converged ? (float)s->iters : (float)max_iter;
  info[2] = s->res;
  info[3] = s->init_res;
}

}  // namespace
}  // namespace fs

extern "C" int fs_schur_cg(const float* x, const float* y, int n, int m, int d, const float* f_hat,
                           const float* g_hat, const float* log_a, const float* log_b, const float* diag_x,
                           const float* denom, const float* rhs, float* z, float* info, float eps,
                           float cost_scale, int max_iter, float rtol, float atol, int prec, void* wsp,
                           size_t ws_bytes, void* stream) {
  FS_TRY(check_common(x, y, n, m, d, eps, cost_scale, prec));
  if (!f_hat || !g_hat || !log_a || !log_b || !diag_x || !denom || !rhs || !z || !info)
    return fail(FS_ERR_BAD_ARG, "null argument");
  if (max_iter < 0) return fail(FS_ERR_BAD_ARG, "max_iter must be >= 0");
  FS_TRY(check_device());
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  Ws ws(wsp, ws_bytes);
  Problem p;
  FS_TRY(make_problem(p, ws, x, y, n, m, d, cost_scale, prec, st, false, 1));
  CgState* s = reinterpret_cast<CgState*>(ws.take<float>(16));
  float* r = ws.take<float>(m);
  float* pv = ws.take<float>(m);
  float* q = ws.take<float>(m);
  float* t = ws.take<float>(n);
  float* R_row = ws.take<float>(n);
  float* R_col = ws.take<float>(m);
  if (ws.overflow) return fail(FS_ERR_WORKSPACE, "workspace too small: need %zu bytes", ws.off);
  const bool on_tc = p.vec_on_tc();
  if (on_tc) {  // the potentials are fixed during CG: both normalisers are computed once
    LseEpilogue e0, e1;
    e0.lse2 = R_row;
    e1.lse2 = R_col;
    FS_CUDA(p.lse(0, g_hat, log_b, eps, e0));
    FS_CUDA(p.lse(1, f_hat, log_a, eps, e1));
  }
  cg_init_kernel<<<1, 1024, 0, st>>>(m, rhs, z, r, pv, s, rtol, atol);
  for (int it = 0; it < max_iter; ++it) {
    VecArgs v1;
    v1.v = pv; v1.rowpot = f_hat; v1.rowlogw = log_a; v1.out = t; v1.skip = &s->done;
    FS_CUDA(p.vec(0, g_hat, log_b, eps, v1, on_tc ? R_row : nullptr));
    cg_div_kernel<<<g1(n), 256, 0, st>>>(n, t, diag_x, t, s);
    VecArgs v0;
    v0.v = t; v0.rowpot = g_hat; v0.rowlogw = log_b; v0.out = q; v0.skip = &s->done;
    FS_CUDA(p.vec(1, f_hat, log_a, eps, v0, on_tc ? R_col : nullptr));
    cg_update_kernel<<<1, 1024, 0, st>>>(m, denom, q, z, r, pv, s, it);
  }
  cg_finish_kernel<<<1, 1, 0, st>>>(s, info, max_iter);
  FS_CUDA(cudaGetLastError());
  return FS_OK;
}

// The Schur-complement CG of the Hessian-vector product inside a plan session: the same device-resident loop as
// fs_schur_cg, without staging and without the two normaliser passes (the session holds both).
extern "C" int fs_plan_session_cg(const float* x, const float* y, int n, int m, int d, const float* f_hat,
                                  const float* g_hat, const float* log_a, const float* log_b, const float* diag_x,
                                  const float* denom, const float* rhs, float* z, float* info, float eps,
                                  float cost_scale, int max_iter, float rtol, float atol, int prec, void* wsp,
                                  size_t ws_bytes, void* stream) {
  FS_TRY(check_common(x, y, n, m, d, eps, cost_scale, prec));
  if (!f_hat || !g_hat || !log_a || !log_b || !diag_x || !denom || !rhs || !z || !info)
    return fail(FS_ERR_BAD_ARG, "null argument");
  if (max_iter < 0) return fail(FS_ERR_BAD_ARG, "max_iter must be >= 0");
  FS_TRY(check_device());
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  Ws ws(wsp, ws_bytes);
  Session se;
  FS_TRY(open_session(se, ws, x, y, n, m, d, eps, cost_scale, prec, st, false, false));
  const Problem& p = se.p;
  CgState* s = reinterpret_cast<CgState*>(se.cg);
  float* r = se.cg + 16;
  float* pv = r + m;
  float* q = pv + m;
  float* t = q + m;
  const bool on_tc = p.vec_on_tc();
  cg_init_kernel<<<1, 1024, 0, st>>>(m, rhs, z, r, pv, s, rtol, atol);
  for (int it = 0; it < max_iter; ++it) {
    VecArgs v1;
    v1.v = pv; v1.rowpot = f_hat; v1.rowlogw = log_a; v1.out = t; v1.skip = &s->done;
    FS_CUDA(p.vec(0, g_hat, log_b, eps, v1, on_tc ? se.R[0] : nullptr));
    cg_div_kernel<<<g1(n), 256, 0, st>>>(n, t, diag_x, t, s);
    VecArgs v0;
    v0.v = t; v0.rowpot = g_hat; v0.rowlogw = log_b; v0.out = q; v0.skip = &s->done;
    FS_CUDA(p.vec(1, f_hat, log_a, eps, v0, on_tc ? se.R[1] : nullptr));
    cg_update_kernel<<<1, 1024, 0, st>>>(m, denom, q, z, r, pv, s, it);
  }
  cg_finish_kernel<<<1, 1, 0, st>>>(s, info, max_iter);
  FS_CUDA(cudaGetLastError());
  return FS_OK;
}
