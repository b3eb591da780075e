// tcgen05 / TMEM / TMA engine interface (implemented in fs_tc.cu).
//
// The score tile S = rows x cols^T is a dense contraction, so it runs on the 5th-gen
// tensor cores: operands are staged once per call as K-padded, TF32-rounded copies
// (3xTF32 hi/lo splits in exact-fp32 mode) whose last K columns carry the per-column
// bias, split into three TF32 pieces that multiply constant ones on the row side --
// the bias add is done by the MMA itself and the soft-max warps only see finished
// logits (up to a common positive scale).
#pragma once
#include "fs_common.cuh"

#include <cuda.h>

namespace fs {
namespace tc {

struct CloudOps {
  float* opA = nullptr;  // [rows_pad, kp] row-operand form (ones in the bias columns)
  float* opB = nullptr;  // [rows_pad, kp] column-operand form (bias columns rewritten per pass)
  int rows = 0, rows_pad = 0;
};

struct Staged {
  CloudOps cloud[2];  // 0 = x, 1 = y
  int d = 0, nlab = 0, kc = 0, kp = 0, prec = 0;  // nlab: label-table columns staged after the coordinates
  // Per side (0: rows of x, 1: rows of y): [pieces, part_stride] partial scaled maxima and sums of row blocks
  // shared by several CTAs, and [rows_pad / 128] arrival counters of those CTAs (zero at rest).
  float* part_m[2] = {nullptr, nullptr};
  float* part_s[2] = {nullptr, nullptr};
  int part_stride = 0;
  int* tickets[2] = {nullptr, nullptr};
};

// Streaming passes leave `k` SMs unused from now on (process-wide; returns the previous value).
int set_reserved_sms(int k);
// Shapes whose resident-operand plan only fits 64-column score tiles run their soft-min and plan-times-vector
// passes on the K-streamed kernels (on = 1, the default) or on the resident ones (0). Returns the previous value.
int set_prefer_streamed(int on);
// Column shares per row block of the plan-times-matrix kernel with the row operand resident: 0 = as many as fill
// the SMs best (the default), 1..8 = forced where the scratch has room. Test knob; returns the previous value.
int set_pv_split(int split);
// Streaming passes use at most `k` CTAs from now on (0 = no limit; returns the previous value). Test knob.
int set_cta_limit(int k);
// CTA count a streaming pass over nblk row blocks x ntiles column tiles would get on a device with `sms`
// SMs of which `reserved` are left free and with CTA limit `limit` (0 = none). Pure host arithmetic.
int plan_ctas(int nblk, int ntiles, int sms, int reserved, int limit);
// Host arithmetic of the plan-times-matrix kernel with the row operand resident: column shares per row block
// for `rows` output rows against `cols` columns on `sms` SMs (prec 0: 128-column tiles, 1: 64-column tiles), and
// through *slots (may be null) the raw output tiles the scratch holds for clouds of at most max(rows, cols) points.
int plan_pv_split(int rows, int cols, int prec, int sms, int* slots);

bool supported(int n, int m, int d, int prec, int nlab = 0);
size_t staged_bytes(int n, int m, int d, int prec, int nlab = 0);
// run_kernels = false only lays out the pointers inside `buf` (operands staged there by an earlier call
// with the same sizes are re-used: row-sharded solvers stage once and step many times).
// With a label cost (lab->V > 0) the operands get 3V extra columns that carry w_coef * W[label, label']
// through the contraction; every size query for such a problem must then pass nlab = 3V.
cudaError_t stage(Staged& s, char* buf, const float* x, const float* y, int n, int m, int d, int prec,
                  cudaStream_t st, bool run_kernels = true, const LabelCost* lab = nullptr, float w_coef = 0.f);
// One LSE pass: side 0 = rows of x against y, side 1 = rows of y against x.
cudaError_t lse(const Staged& s, int side, const StreamArgs& a, const LseEpilogue& e, cudaStream_t st);

// Several dense LSE passes (of one or several staged problems with the same d, precision and label columns) as
// ONE launch preceded by one bias launch: the (row block, column tile) items of all passes form one list that is
// cut over the SMs, so the ramp and tail of a launch are paid once per group instead of once per pass. At most
// multi_max() passes; cudaErrorNotSupported when a pass is K-streamed, carries a tile list or an early-stop flag
// (the caller then runs the passes one by one).
struct MultiPass {
  const Staged* s;
  int side;
  StreamArgs a;
  LseEpilogue e;
};
int multi_max();
cudaError_t lse_multi(const MultiPass* passes, int n, cudaStream_t st);

// Hard c-transform pass over the same staged operands: out_val_i = min_j(-2cs x_i.y_j + bias_j) and the
// smallest column attaining it (a.pot = bias, a.logw ignored, a.eps unused).
cudaError_t argmax(const Staged& s, int side, const StreamArgs& a, float* out_val, int* out_idx, cudaStream_t st);

// Plan-times-matrix pass on the tensor cores (same staged operands, hence bit-identical scores
// to the LSE passes). `scratch` holds the transposed, TF32-split copy of V (pv_scratch_bytes).
// Scratch of a Mat5 pass (PvArgs::rows2 set: weights multiplied by rows2_i . cols_j), which pv() runs on the
// K-streamed kernel at every shape; 0 when the tensor-core engine does not take the problem.
size_t mat5_scratch_bytes(int nr, int nc, int d, int prec, int dv, int nlab = 0);
bool pv_supported(int d, int prec, int dv, int nlab = 0);
size_t pv_scratch_bytes(int nc, int d, int prec, int dv, int nlab = 0);
cudaError_t pv(const Staged& s, int side, const StreamArgs& a, const PvArgs& p, char* scratch, cudaStream_t st);

// ---- K-streamed passes (fs_tck.cu) --------------------------------------------------------------------
// When the K-padded 128-row operand does not fit in shared memory (large d, or moderate d in the 3xTF32
// mode) both operands stream through shared memory in 32-float K chunks and the score tile accumulates in
// TMEM over the chunks. lse() and pv() route there by themselves; the functions below are their back ends.
bool k_streamed(int d, int prec, int nlab = 0);
// Tuning knob of the K-streamed kernels: contractions of at least k 32-float chunks take 256 x 256 tiles with
// one accumulator per half, shorter ones 256 x 128 tiles with two (returns the previous value).
int set_wide_tile_min_chunks(int k);
// lse() takes a block-sparse list of kept 128 x 128 tiles (StreamArgs::tile_row_ptr / tile_col_idx) for these
// shapes; the row range must then start on a multiple of 128.
bool csr_supported(int d, int prec, int nlab = 0);
// Soft-min pass; with s_out != nullptr the raw scores of rows [row_begin, nr) are also stored, row r at
// s_out + (r - row_begin) * ld_s (the matrix pass turns them into weights instead of recomputing them).
cudaError_t kstream_lse(const Staged& s, int side, const StreamArgs& a, const LseEpilogue& e, float* s_out,
                        long long ld_s, cudaStream_t st);
// out_i = 2^(rowterm_i + R_i) * sum_j 2^(t_ij - R_i) v_j with the known normaliser p.R (p.dv == 1).
cudaError_t kstream_vec(const Staged& s, int side, const StreamArgs& a, const PvArgs& p, char* scratch,
                        cudaStream_t st);
// Whole matrix pass for wide V: per chunk of rows one soft-min pass that keeps its scores, an elementwise
// pass that turns them into TF32 weights, and a K-streamed GEMM against the transposed V. Writes the row
// normalisers to R_out ([nr] floats) on the way. `scratch` must hold kstream_mat_scratch() bytes.
// Matrix pass with the second GEMM fed from TMEM (any contraction length, V in slices of 128 columns): narrow V
// of K-streamed problems, and the Mat5 term of the Hessian (weights multiplied by rows2_i . cols_j) at any shape.
size_t kstream_pv_scratch(int nr, int nc, int kp, int dv, int prec, bool mat5);
cudaError_t kstream_pv(const Staged& s, int side, const StreamArgs& a, const PvArgs& p, char* scratch,
                       size_t scratch_bytes, cudaStream_t st);
bool kstream_mat_supported(int dv);
size_t kstream_mat_scratch(int nr, int nc, int dv, int prec);
cudaError_t kstream_mat(const Staged& s, int side, const StreamArgs& a, const PvArgs& p, float* R_out,
                        char* scratch, size_t scratch_bytes, cudaStream_t st);

// Shared host helpers of the two translation units.
namespace detail {
// 2-D fp32 tensor [rows, kp] whose rows are row_pitch floats apart (0 = kp: densely packed).
bool encode_map(CUtensorMap* map, const float* base, long long rows, long long kp, int box_k, int box_rows,
                CUtensorMapSwizzle swz, long long row_pitch = 0);
int pick_ctas(int nblk, int ntiles);
int sm_count();
// Writes the column bias of a pass (divided by the logit scale, split into three TF32 pieces) into the bias
// columns of the column operand.
void launch_bias(const CloudOps& colc, int kc, int kp, const float* pot, const float* logw, float inv_eps,
                 float inv_scale2, const Ctrl* ctrl, cudaStream_t st, int pot_shard = 0, int pot_stride = 0);
inline int pad256(int r) { return (r + 255) & ~255; }
}  // namespace detail

// Value of the device-global error word (non-zero once a bounded wait gave up); synchronises.
int read_error_flag();
// Resets the word to zero (0 on success, -1 on a CUDA error); synchronises.
int clear_error_flag();

// Average SM cycles per tcgen05.mma (kind::tf32, 128 x n_cols x 8, n_cols in {64,128,256}; A from shared
// memory or from TMEM) when one lane issues 4096 of them back to back on every SM. Allocates a small
// buffer and synchronises; < 0 on error. Diagnostic (roofline denominators).
double micro_mma_cycles(int n_cols, bool a_in_tmem);

}  // namespace tc
}  // namespace fs
