// Shared declarations of the streaming-Sinkhorn engine: argument blocks that the
// C-ABI layer (fs_api.cu) fills and the two engines (fs_simt.cu: CUDA-core fp32,
// fs_tc.cu: tcgen05/TMEM/TMA) consume.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stddef.h>

namespace fs {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// Device-side solver control block (lives in caller workspace).
struct Ctrl {
  unsigned int delta_bits;  // max |delta| of the current check, as float bits (non-negative floats order like uints)
  int converged;            // 1 once the early-stop test passed: loop steps become identity
  int have_prev;            // 1 once a snapshot exists
  int iters_used;           // number of executed steps
  int pad[4];
};

// One streaming pass "rows against all cols":
//   t_ij = scale2 * <rows_i, cols_j> + bias2_j        (log2 domain)
//   scale2 = 2*cost_scale*log2e/eps
//   bias2_j = (pot_j/eps + logw_j)*log2e  (logw != nullptr)  or  pot_j*log2e
struct StreamArgs {
  const float* rows = nullptr;  // [nr, d]
  const float* cols = nullptr;  // [nc, d]
  int nr = 0, nc = 0, d = 0;
  int row_begin = 0;            // only rows [row_begin, nr) are produced (row sharding); nr = end of the range
  const float* pot = nullptr;   // [nc]
  const float* logw = nullptr;  // [nc] or nullptr
  // Packed potentials (tensor-core engine only): when pot_shard > 0, element j of the potential is at
  // pot[(j / pot_shard) * pot_stride + j % pot_shard] (slices of several vectors gathered from the ranks of a
  // multi-GPU solve into one [ranks, pot_stride] buffer).
  int pot_shard = 0, pot_stride = 0;
  float eps = 1.f, cost_scale = 1.f;
  // Block-sparse tile list over 128x128 (row-tile, col-tile) pairs, CSR by row tile; nullptr = dense.
  const int* tile_row_ptr = nullptr;
  const int* tile_col_idx = nullptr;
  // Label cost (V > 0): t_ij -= lam_w/eps*log2e * W[a, b] with (a, b) = (label of the x point, label of the
  // y point); w_row_major says whether the ROWS of this pass are the x cloud (index = lab_rows*V + lab_cols)
  // or the y cloud (index = lab_cols*V + lab_rows). The tensor-core engine folds the same term into the
  // contraction when the operands are staged and ignores these fields.
  const int* lab_rows = nullptr;
  const int* lab_cols = nullptr;
  const float* W = nullptr;
  int V = 0;
  int w_row_major = 1;
  float lam_w = 0.f;
};

// Label-augmented ground cost C_ij = cs*lambda_x*|x_i-y_j|^2-like dot term + lam_w * W[label_x_i, label_y_j]
// (reference kernels/sinkhorn_flashstyle_sqeuclid.py:545-560): device labels of both clouds and the V x V table.
struct LabelCost {
  const int* lab[2] = {nullptr, nullptr};  // labels of cloud 0 (x) and cloud 1 (y)
  const float* W = nullptr;                // [V, V] row-major, W[label_x, label_y]
  int V = 0;                               // 0 = no label cost
  float lam_w = 0.f;                       // lambda_y * cost_scale
};

// LSE pass epilogue:
//   cand_i = -eps*damping*ln2*(m_i + log2(max(s_i,1e-40)))
//   out_i  = (old ? (1-w)*old_i : 0) + w*cand_i - shiftcoef*shift_i + addcoef*addvec_i
//   lse2_i = m_i + log2(s_i)   (optional raw log2 normaliser)
// If ctrl && ctrl->converged: out_i = old_i (identity step), lse2 untouched.
struct LseEpilogue {
  float damping = 1.f;
  const float* old = nullptr;
  float w = 1.f;
  const float* shift = nullptr;
  float shiftcoef = 0.f;
  const float* addvec = nullptr;
  float addcoef = 0.f;
  float* out = nullptr;
  float* lse2 = nullptr;
  const Ctrl* ctrl = nullptr;
};

// Weighted pass: out_i = 2^(rowterm2_i) * sum_j 2^(t_ij) * v_j, rowterm2_i = (rowpot_i/eps + rowlogw_i)*log2e
struct VecArgs {
  const float* v = nullptr;        // [nc]
  const float* rowpot = nullptr;   // [nr]
  const float* rowlogw = nullptr;  // [nr]
  float* out = nullptr;            // [nr]
  const int* skip = nullptr;       // device flag: non-zero => the pass is a no-op (finished CG)
};

enum PvEpilogue { PV_APPLY = 0, PV_GRAD = 1, PV_MAT5 = 2 };

// Plan-times-matrix pass with known per-row log2 offsets R (p_ij = 2^(t_ij - R_i)):
//   O_i = sum_j p_ij * e_ij * colscale_j * V_j,  e_ij = <rows2_i, cols_j> if rows2 else 1
//   PV_APPLY: out_i = 2^(R_i + rowterm2_i) * O_i
//   PV_GRAD : out_i = coef * gs * roww_i * (rows_i - O_i)        (needs dv == d, R = exact LSE)
//   PV_MAT5 : out_i = coef * 2^(R_i + rowterm2_i) * O_i
struct PvArgs {
  const float* R = nullptr;        // [nr]
  const float* rows2 = nullptr;    // [nr, d] or nullptr
  const float* V = nullptr;        // [nc, dv]
  int dv = 0;
  const float* colscale = nullptr; // [nc] or nullptr
  int epilogue = PV_APPLY;
  const float* rowpot = nullptr;   // [nr]   (APPLY/MAT5)
  const float* rowlogw = nullptr;  // [nr] or nullptr
  const float* roww = nullptr;     // [nr]   (GRAD: a_i)
  const float* gs = nullptr;       // device scalar or nullptr
  float coef = 1.f;
  float* out = nullptr;            // [nr, dv]
  const int* skip = nullptr;       // device flag: non-zero => the pass is a no-op (finished CG)
};

// --- CUDA-core engine (fs_simt.cu) ---
cudaError_t simt_lse(const StreamArgs& s, const LseEpilogue& e, cudaStream_t st);
cudaError_t simt_vec(const StreamArgs& s, const VecArgs& v, cudaStream_t st);
cudaError_t simt_pv(const StreamArgs& s, const PvArgs& p, cudaStream_t st);
// min_j(-2cs rows_i.cols_j + s.pot[j]) and the smallest j attaining it (s.logw, s.eps unused).
cudaError_t simt_argmin(const StreamArgs& s, float* out_val, int* out_idx, cudaStream_t st);

}  // namespace fs
