// CUDA-core (fp32 FMA) streaming engine. Exact-fp32 products, any n, m, d.
//
// It serves the shapes the tcgen05 engine does not take (tiny or very large
// feature dimension, matrix passes in exact-fp32 mode) and is the on-device
// cross-check for it. Same maths as the reference's Triton kernels
// (kernels/sinkhorn_flashstyle_sqeuclid.py:199-419, kernels/apply_flash.py:50-343,
// :595-832, kernels/sinkhorn_triton_grad_sqeuclid.py:102-402,
// kernels/apply_ott.py:35-168) with a different decomposition: every thread keeps
// a private online (max, sum) pair for the columns it owns and the 16 partial
// pairs of a row are merged once at the end, so no per-tile reductions are
// needed; matrix passes take a known per-row offset R and are rescale-free.
#include "fs_common.cuh"

namespace fs {
namespace {

constexpr int TM = 64;    // rows per CTA
constexpr int TN = 64;    // columns per tile
constexpr int TK = 16;    // feature chunk staged in shared memory
constexpr int NT = 256;   // threads: 16 (ty) x 16 (tx), 4x4 outputs each
constexpr int LDS_T = TM + 4;

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Stage rows [r0, r0+64) x features [k0, k0+16) of src (ld = d) transposed: dst[k][r].
__device__ __forceinline__ void stage_tile(float (*dst)[LDS_T], const float* __restrict__ src,
                                           int r0, int nrows, int k0, int d, int tid) {
#pragma unroll
  for (int i = 0; i < (TM * TK) / NT; ++i) {
    int e = tid + i * NT;
    int r = e / TK, k = e % TK;
    int gr = r0 + r, gk = k0 + k;
    float v = 0.f;
    if (gr < nrows && gk < d) v = __ldg(src + (size_t)gr * d + gk);
    dst[k][r] = v;
  }
}

__device__ __forceinline__ void fma_tile(float (&acc)[4][4], const float (*As)[LDS_T],
                                         const float (*Bs)[LDS_T], int ty, int tx) {
#pragma unroll
  for (int k = 0; k < TK; ++k) {
    float4 a = *reinterpret_cast<const float4*>(&As[k][ty * 4]);
    float4 b = *reinterpret_cast<const float4*>(&Bs[k][tx * 4]);
    float av[4] = {a.x, a.y, a.z, a.w};
    float bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
  }
}

__device__ __forceinline__ float col_bias2(const StreamArgs& s, int col, float inv_eps_log2) {
  // Same association as the reference: g*inv_eps*log2e + logw*log2e.
  if (s.logw) return __ldg(s.pot + col) * inv_eps_log2 + __ldg(s.logw + col) * kLog2e;
  return __ldg(s.pot + col) * kLog2e;
}

// Label-cost term of entry (row label lr, column label lc), in log2 units (0 without label cost).
__device__ __forceinline__ float label_term2(const StreamArgs& s, int lr, int lc, float lw2) {
  return lw2 * __ldg(s.W + (s.w_row_major ? lr * s.V + lc : lc * s.V + lr));
}

// Column-tile iteration (dense, or CSR over 128-wide tiles => two 64-wide tiles each).
struct TileIter {
  int pos, end, sub, ntiles;
  const int* idx;
  __device__ TileIter(const StreamArgs& s, int row0) {
    ntiles = (s.nc + TN - 1) / TN;
    sub = 0;
    if (s.tile_row_ptr) {
      int rt = row0 / 128;
      pos = s.tile_row_ptr[rt];
      end = s.tile_row_ptr[rt + 1];
      idx = s.tile_col_idx;
    } else {
      pos = 0;
      end = ntiles;
      idx = nullptr;
    }
  }
  // Returns the next 64-wide column tile index or -1.
  __device__ int next() {
    while (pos < end) {
      if (!idx) return pos++;
      int t = idx[pos] * 2 + sub;
      if (sub == 0) sub = 1; else { sub = 0; ++pos; }
      if (t < ntiles) return t;
    }
    return -1;
  }
};

enum { MODE_LSE = 0, MODE_VEC = 1 };

template <int MODE>
__global__ void __launch_bounds__(NT) simt_stream_kernel(StreamArgs s, LseEpilogue ep, VecArgs va) {
  __shared__ __align__(16) float As[TK][LDS_T];
  __shared__ __align__(16) float Bs[TK][LDS_T];
  __shared__ float bias_s[TN];
  __shared__ float vec_s[TN];
  __shared__ int lab_s[TN];

  const int tid = threadIdx.x, ty = tid / 16, tx = tid % 16;
  const int row0 = s.row_begin + blockIdx.x * TM;

  if (MODE == MODE_LSE && ep.ctrl && ep.ctrl->converged) {
    // Identity step: the solve already stopped; keep buffers consistent.
    if (tid < TM && row0 + tid < s.nr && ep.old) ep.out[row0 + tid] = ep.old[row0 + tid];
    return;
  }
  if (MODE == MODE_VEC && va.skip && *va.skip) return;

  const float inv_eps = 1.0f / s.eps;
  const float inv_eps_log2 = inv_eps * kLog2e;
  const float scale2 = (2.0f * s.cost_scale) * inv_eps * kLog2e;

  float m[4], acc1[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) { m[i] = -INFINITY; acc1[i] = 0.f; }
  const float lw2 = s.lam_w * inv_eps_log2;
  int lr[4] = {0, 0, 0, 0};
  if (s.V) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int r = row0 + ty * 4 + i;
      lr[i] = (r < s.nr) ? __ldg(s.lab_rows + r) : 0;
    }
  }

  TileIter it(s, row0);
  for (int ct = it.next(); ct >= 0; ct = it.next()) {
    const int col0 = ct * TN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    if (tid < TN) {
      int c = col0 + tid;
      bias_s[tid] = (c < s.nc) ? col_bias2(s, c, inv_eps_log2) : -INFINITY;
      if (MODE == MODE_VEC) vec_s[tid] = (c < s.nc) ? __ldg(va.v + c) : 0.f;
      if (s.V) lab_s[tid] = (c < s.nc) ? __ldg(s.lab_cols + c) : 0;
    }
    for (int k0 = 0; k0 < s.d; k0 += TK) {
      __syncthreads();
      stage_tile(As, s.rows, row0, s.nr, k0, s.d, tid);
      stage_tile(Bs, s.cols, col0, s.nc, k0, s.d, tid);
      __syncthreads();
      fma_tile(acc, As, Bs, ty, tx);
    }
    __syncthreads();  // bias_s visible even when d == 0 chunks... (d >= 1 always)

    float bj[4], vj[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      bj[j] = bias_s[tx * 4 + j];
      vj[j] = (MODE == MODE_VEC) ? vec_s[tx * 4 + j] : 1.f;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float t[4];
      float tmax = -INFINITY;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        t[j] = fmaf(acc[i][j], scale2, bj[j]);  // -inf bias masks padded columns
        if (s.V) t[j] -= label_term2(s, lr[i], lab_s[tx * 4 + j], lw2);
        tmax = fmaxf(tmax, t[j]);
      }
      float mn = fmaxf(m[i], tmax);
      if (mn > -INFINITY) {
        float a = acc1[i] * ex2(m[i] - mn);
#pragma unroll
        for (int j = 0; j < 4; ++j) a = fmaf(ex2(t[j] - mn), vj[j], a);
        acc1[i] = a;
        m[i] = mn;
      }
    }
    __syncthreads();  // bias_s / vec_s reused by the next tile
  }

  // Merge the 16 per-thread partials of each row (lanes tx = 0..15 of a half-warp).
#pragma unroll
  for (int i = 0; i < 4; ++i) {
#pragma unroll
    for (int off = 8; off >= 1; off >>= 1) {
      float mo = __shfl_xor_sync(0xffffffffu, m[i], off);
      float ao = __shfl_xor_sync(0xffffffffu, acc1[i], off);
      float mn = fmaxf(m[i], mo);
      if (mn > -INFINITY) {
        acc1[i] = acc1[i] * ex2(m[i] - mn) + ao * ex2(mo - mn);
        m[i] = mn;
      }
    }
  }
  if (tx == 0) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int r = row0 + ty * 4 + i;
      if (r >= s.nr) continue;
      if (MODE == MODE_LSE) {
        float lse2 = m[i] + log2f(fmaxf(acc1[i], 1e-40f));
        if (ep.lse2) ep.lse2[r] = lse2;
        if (ep.out) {
          float cand = -s.eps * ep.damping * (lse2 * kLn2);
          float o = ep.w * cand;
          if (ep.old) o += (1.0f - ep.w) * ep.old[r];
          if (ep.shift) o -= ep.shiftcoef * ep.shift[r];
          if (ep.addvec) o += ep.addcoef * ep.addvec[r];
          ep.out[r] = o;
        }
      } else {
        float rt = (va.rowpot[r] * inv_eps + (va.rowlogw ? va.rowlogw[r] : 0.f)) * kLog2e;
        va.out[r] = (m[i] > -INFINITY) ? ex2(m[i] + rt) * acc1[i] : 0.f;
      }
    }
  }
}

// Plan-times-matrix pass, one 64-wide slice of V's columns per blockIdx.y.
template <bool DOT2>
__global__ void __launch_bounds__(NT) simt_pv_kernel(StreamArgs s, PvArgs p) {
  __shared__ __align__(16) float As[TK][LDS_T];
  __shared__ __align__(16) float Bs[TK][LDS_T];
  __shared__ __align__(16) float A2s[DOT2 ? TK : 1][LDS_T];
  __shared__ float Ws[TM][TN + 1];
  __shared__ __align__(16) float Vs[TN][64];
  __shared__ float bias_s[TN];
  __shared__ float cs_s[TN];
  __shared__ int lab_s[TN];

  const int tid = threadIdx.x, ty = tid / 16, tx = tid % 16;
  const int row0 = s.row_begin + blockIdx.x * TM;
  const int dv0 = blockIdx.y * 64;

  const float inv_eps = 1.0f / s.eps;
  const float inv_eps_log2 = inv_eps * kLog2e;
  const float scale2 = (2.0f * s.cost_scale) * inv_eps * kLog2e;

  float Rr[4];
  int lr[4] = {0, 0, 0, 0};
  const float lw2 = s.lam_w * inv_eps_log2;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int r = row0 + ty * 4 + i;
    Rr[i] = (r < s.nr) ? __ldg(p.R + r) : 0.f;
    if (s.V) lr[i] = (r < s.nr) ? __ldg(s.lab_rows + r) : 0;
  }
  float O[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) O[i][j] = 0.f;

  TileIter it(s, row0);
  for (int ct = it.next(); ct >= 0; ct = it.next()) {
    const int col0 = ct * TN;
    float acc[4][4], acc2[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) { acc[i][j] = 0.f; acc2[i][j] = 0.f; }

    if (tid < TN) {
      int c = col0 + tid;
      bias_s[tid] = (c < s.nc) ? col_bias2(s, c, inv_eps_log2) : -INFINITY;
      cs_s[tid] = (c < s.nc && p.colscale) ? __ldg(p.colscale + c) : 1.f;
      if (s.V) lab_s[tid] = (c < s.nc) ? __ldg(s.lab_cols + c) : 0;
    }
    for (int k0 = 0; k0 < s.d; k0 += TK) {
      __syncthreads();
      stage_tile(As, s.rows, row0, s.nr, k0, s.d, tid);
      stage_tile(Bs, s.cols, col0, s.nc, k0, s.d, tid);
      if (DOT2) stage_tile(A2s, p.rows2, row0, s.nr, k0, s.d, tid);
      __syncthreads();
      fma_tile(acc, As, Bs, ty, tx);
      if (DOT2) fma_tile(acc2, A2s, Bs, ty, tx);
    }
    __syncthreads();
    // V tile: rows col0.., columns dv0..dv0+63 (zero-filled outside).
#pragma unroll
    for (int i = 0; i < (TN * 64) / NT; ++i) {
      int e = tid + i * NT;
      int j = e / 64, c = e % 64;
      int gj = col0 + j, gc = dv0 + c;
      Vs[j][c] = (gj < s.nc && gc < p.dv) ? __ldg(p.V + (size_t)gj * p.dv + gc) : 0.f;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        int cj = tx * 4 + j;
        float tij = fmaf(acc[i][j], scale2, bias_s[cj]);
        if (s.V) tij -= label_term2(s, lr[i], lab_s[cj], lw2);
        float w = ex2(tij - Rr[i]);  // padded columns: 2^-inf = 0
        if (DOT2) w *= acc2[i][j];
        w *= cs_s[cj];
        Ws[ty * 4 + i][cj] = w;
      }
    __syncthreads();
#pragma unroll 8
    for (int j = 0; j < TN; ++j) {
      float4 b = *reinterpret_cast<const float4*>(&Vs[j][tx * 4]);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float a = Ws[ty * 4 + i][j];
        O[i][0] = fmaf(a, b.x, O[i][0]);
        O[i][1] = fmaf(a, b.y, O[i][1]);
        O[i][2] = fmaf(a, b.z, O[i][2]);
        O[i][3] = fmaf(a, b.w, O[i][3]);
      }
    }
    __syncthreads();
  }

  const float gsv = p.gs ? __ldg(p.gs) : 1.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int r = row0 + ty * 4 + i;
    if (r >= s.nr) continue;
    float fac;
    if (p.epilogue == PV_GRAD) {
      fac = (p.coef * gsv) * __ldg(p.roww + r);
    } else {
      float rt = (__ldg(p.rowpot + r) * inv_eps + (p.rowlogw ? __ldg(p.rowlogw + r) : 0.f)) * kLog2e;
      fac = p.coef * ex2(Rr[i] + rt);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int c = dv0 + tx * 4 + j;
      if (c >= p.dv) continue;
      float o = O[i][j];
      if (p.epilogue == PV_GRAD) o = __ldg(s.rows + (size_t)r * s.d + c) - o;
      p.out[(size_t)r * p.dv + c] = fac * o;
    }
  }
}

// Hard c-transform: out_val_i = min_j (-2cs x_i.y_j + bias_j), out_idx_i = the smallest j attaining it
// (reference kernels/c_transform_sqeuclid.py:117-206). s.pot holds the bias. A thread visits its columns in
// increasing order and replaces its candidate only on a strictly smaller value; the 16 candidates of a row
// are merged with "smaller value, then smaller column".
__global__ void __launch_bounds__(NT) simt_argmin_kernel(StreamArgs s, float* __restrict__ out_val,
                                                         int* __restrict__ out_idx) {
  __shared__ __align__(16) float As[TK][LDS_T];
  __shared__ __align__(16) float Bs[TK][LDS_T];
  __shared__ float bias_s[TN];
  const int tid = threadIdx.x, ty = tid / 16, tx = tid % 16;
  const int row0 = s.row_begin + blockIdx.x * TM;
  const float coord = 2.0f * s.cost_scale;
  float best[4];
  int arg[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) { best[i] = INFINITY; arg[i] = 0x7fffffff; }
  const int ntiles = (s.nc + TN - 1) / TN;
  for (int ct = 0; ct < ntiles; ++ct) {
    const int col0 = ct * TN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    if (tid < TN) bias_s[tid] = (col0 + tid < s.nc) ? __ldg(s.pot + col0 + tid) : INFINITY;
    for (int k0 = 0; k0 < s.d; k0 += TK) {
      __syncthreads();
      stage_tile(As, s.rows, row0, s.nr, k0, s.d, tid);
      stage_tile(Bs, s.cols, col0, s.nc, k0, s.d, tid);
      __syncthreads();
      fma_tile(acc, As, Bs, ty, tx);
    }
    __syncthreads();
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float bj = bias_s[tx * 4 + j];  // +inf masks padded columns
      const int c = col0 + tx * 4 + j;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float v = fmaf(-coord, acc[i][j], bj);
        if (v < best[i]) { best[i] = v; arg[i] = c; }
      }
    }
    __syncthreads();  // bias_s is rewritten by the next tile
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
#pragma unroll
    for (int off = 8; off >= 1; off >>= 1) {
      const float vo = __shfl_xor_sync(0xffffffffu, best[i], off);
      const int ao = __shfl_xor_sync(0xffffffffu, arg[i], off);
      if (vo < best[i] || (vo == best[i] && ao < arg[i])) { best[i] = vo; arg[i] = ao; }
    }
  }
  if (tx == 0) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = row0 + ty * 4 + i;
      if (r < s.nr) { out_val[r] = best[i]; out_idx[r] = arg[i]; }
    }
  }
}

}  // namespace

cudaError_t simt_argmin(const StreamArgs& s, float* out_val, int* out_idx, cudaStream_t st) {
  if (s.nr - s.row_begin <= 0) return cudaSuccess;
  dim3 grid((s.nr - s.row_begin + TM - 1) / TM);
  simt_argmin_kernel<<<grid, NT, 0, st>>>(s, out_val, out_idx);
  return cudaGetLastError();
}

cudaError_t simt_lse(const StreamArgs& s, const LseEpilogue& e, cudaStream_t st) {
  if (s.nr - s.row_begin <= 0) return cudaSuccess;
  dim3 grid((s.nr - s.row_begin + TM - 1) / TM);
  simt_stream_kernel<MODE_LSE><<<grid, NT, 0, st>>>(s, e, VecArgs{});
  return cudaGetLastError();
}

cudaError_t simt_vec(const StreamArgs& s, const VecArgs& v, cudaStream_t st) {
  if (s.nr - s.row_begin <= 0) return cudaSuccess;
  dim3 grid((s.nr - s.row_begin + TM - 1) / TM);
  simt_stream_kernel<MODE_VEC><<<grid, NT, 0, st>>>(s, LseEpilogue{}, v);
  return cudaGetLastError();
}

cudaError_t simt_pv(const StreamArgs& s, const PvArgs& p, cudaStream_t st) {
  if (s.nr - s.row_begin <= 0 || p.dv <= 0) return cudaSuccess;
  dim3 grid((s.nr - s.row_begin + TM - 1) / TM, (p.dv + 63) / 64);
  if (p.rows2)
    simt_pv_kernel<true><<<grid, NT, 0, st>>>(s, p);
  else
    simt_pv_kernel<false><<<grid, NT, 0, st>>>(s, p);
  return cudaGetLastError();
}

}  // namespace fs
