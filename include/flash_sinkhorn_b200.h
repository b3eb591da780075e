/*
 * flash_sinkhorn_b200 -- C ABI of the B200 (sm_100a) streaming-Sinkhorn engine.
 *
 * Every entry point replaces one kernel launcher (or one host loop over
 * launchers) of the reference package ot-triton-lab/flash-sinkhorn; the
 * reference has no FFI of its own, so each declaration cites the Python
 * function whose body it stands in for (paths are relative to the reference's
 * src/flash_sinkhorn/).
 *
 * Conventions
 *  - All pointers are DEVICE pointers to contiguous fp32 (row-major for
 *    matrices) owned by the caller, unless the name ends in _host.
 *  - `stream` is a cudaStream_t passed as void* (NULL = legacy default stream).
 *  - `ws`/`ws_bytes`: caller-owned scratch, at least fs_workspace_bytes() for
 *    the same (op, n, m, d, prec); 256-byte aligned. Nothing is allocated, and
 *    nothing synchronises with the host unless stated.
 *  - Return value: FS_OK or an fs_status; fs_last_error() gives the message of
 *    the calling thread's last failure.
 *  - `prec`: FS_PREC_TF32 (one tcgen05 kind::tf32 pass), FS_PREC_FP32 (3xTF32
 *    split, fp32-equivalent products) or FS_PREC_SIMT (CUDA-core fp32 FMA).
 *  - rho < 0 (or NaN) means "balanced side" (no marginal relaxation).
 *  - Notation: cs = cost_scale, C_ij = cs*|x_i-y_j|^2, alpha_i = cs*|x_i|^2,
 *    beta_j = cs*|y_j|^2, shifted potentials f_hat = f-alpha, g_hat = g-beta.
 */
#ifndef FLASH_SINKHORN_B200_H
#define FLASH_SINKHORN_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  FS_OK = 0,
  FS_ERR_BAD_ARG = 1,
  FS_ERR_UNSUPPORTED = 2,
  FS_ERR_CUDA = 3,
  FS_ERR_TIMEOUT = 4,
  FS_ERR_WORKSPACE = 5
} fs_status;

enum { FS_PREC_TF32 = 0, FS_PREC_FP32 = 1, FS_PREC_SIMT = 2 };

/* op ids for fs_workspace_bytes */
enum {
  FS_OP_LSE = 0,
  FS_OP_STEP = 1,
  FS_OP_SOLVE_SYMMETRIC = 2,
  FS_OP_SOLVE_ALTERNATING = 3,
  FS_OP_APPLY_VEC = 4,
  FS_OP_APPLY_MAT = 5,
  FS_OP_GRAD = 6,
  FS_OP_MAT5 = 7,
  FS_OP_SCHUR = 8
};

/* Library/ABI version (major*10000 + minor*100 + patch); 200 = 0.2.0. */
int fs_version(void);

/* Message of the calling thread's most recent non-FS_OK return ("" if none). */
const char* fs_last_error(void);

/* Compute capability of the current device as major*10+minor (100 on B200);
 * negative on CUDA error. The compute entry points return FS_ERR_UNSUPPORTED
 * on anything that is not sm_100. */
int fs_device_arch(void);

/* Number of kernels this library has enqueued since it was loaded (monotonic, all
 * threads; single-thread <<<1,1>>> bookkeeping kernels are not counted). Lets a caller
 * verify that its work ran on the GPU path: difference two readings around a call. */
long long fs_launch_count(void);

/* Device-side health word of the current device: 0 = fine, 1 = some kernel of this
 * library gave up a bounded wait (its outputs are then invalid), negative = CUDA error
 * while reading it. SYNCHRONISES the device; meant for tests and post-mortems. */
int fs_device_error(void);

/* Resets the health word of the current device to 0 (after the cause of a time-out has been dealt with and the
 * workspaces of the affected calls have been re-staged). Returns 0, or a negative value on a CUDA error.
 * SYNCHRONISES the device. */
int fs_clear_device_error(void);

/* Host arithmetic only: the workspace bytes an fs_apply_mat call with a matrix of `dv` columns carves at these
 * sizes. Never more than fs_workspace_bytes(FS_OP_APPLY_MAT, n, m, d, prec), which is sized for any dv <= d. */
size_t fs_apply_mat_plan_bytes(int n, int m, int d, int dv, int prec);

/* Measurement aid (no reference counterpart): ex2 evaluations per second that this GPU sustains,
 * mode 0 = ex2.approx alone, mode 1 = the soft-max inner loop (max + FFMA + ex2 + FADD per entry) on
 * register data, with `warps_per_sm` resident warps per SM. Used by bench.py as the measured
 * transcendental-pipe peak of the roofline. Allocates 4 bytes and synchronises; < 0 on error. */
double fs_micro_exp_rate(int mode, int warps_per_sm);

/* Micro-benchmark (no reference counterpart): average SM cycles per `tcgen05.mma.kind::tf32`
 * instruction of shape 128 x n_cols x 8 (n_cols in {64, 128, 256}; A operand from shared memory, or from
 * TMEM when a_in_tmem != 0) when one lane per SM issues 4096 of them back to back. The tensor term of
 * the roofline follows from it: entries/s = SMs * clock * 128 * n_cols / (cycles * K-steps per entry
 * tile). Allocates a few KB and synchronises; < 0 on error. */
double fs_micro_mma_cycles(int n_cols, int a_in_tmem);

/* Multi-GPU helper (no reference counterpart): from now on the streaming passes of this process use k SMs
 * fewer than the device has, leaving them to a collective (NCCL all-gather of the previous half-step) that
 * runs next to the pass. A pass is a single wave of one CTA per SM with a static work split, so a CTA that
 * must wait for the collective's CTAs to leave its SM delays the whole pass; k = 2 costs ~1 % when nothing
 * else runs. Returns the previous value; 0 restores the default. */
int fs_set_reserved_sms(int k);

/* Test knob (no reference counterpart): streaming passes of this process use at most k CTAs from now on
 * (0 = no limit, the default). Returns the previous value. Lets tests force the work split of a pass (one
 * CTA covering many row blocks, many CTAs sharing one) without touching the environment. */
int fs_set_cta_limit(int k);

/* Tuning knob (no reference counterpart): K-streamed passes whose contraction has at least k chunks of 32
 * floats use 256 x 256 score tiles with one TMEM accumulator per 128-row half, shorter ones 256 x 128 tiles
 * with two accumulators per half. Returns the previous value. */
int fs_set_wide_tile_min_chunks(int k);

/* Tuning knob (no reference counterpart): shapes whose row operand fits in shared memory only next to
 * 64-column score tiles (e.g. d = 64 in the exact mode) run their soft-min and plan-times-vector passes on the
 * K-streamed kernels (on != 0, the default: larger, MMA-efficient tiles) or on the resident-operand kernels
 * (on = 0). Returns the previous value. */
int fs_set_prefer_streamed(int on);

/* Test knob (no reference counterpart): the plan-times-matrix kernel with the row operand resident in shared
 * memory cuts the column range of a 128-row block into shares, one CTA each; every CTA parks its raw output
 * tile in the scratch and the last to finish adds the shares in share order (run-to-run identical bits).
 * split = 0: as many shares as fill the SMs best (the default); 1..8: that many where the scratch has room.
 * Process-wide; returns the previous value. */
int fs_set_pv_split(int split);

/* Which engine serves a problem of these sizes (no reference counterpart): 0 = CUDA-core fp32 FMA, 1 = tcgen05
 * with the row operand resident in shared memory, 2 = tcgen05 with both operands streamed in K chunks. */
int fs_engine(int n, int m, int d, int prec);

/* Host arithmetic only (no reference counterpart): the CTA count a streaming pass over n_row_blocks x
 * n_col_tiles work items gets on a device with `sms` SMs when `reserved` of them are left free and the CTA
 * limit is `limit` (0 = none). At most 16 CTAs ever share a row block. Returns 0 on non-positive sizes. */
int fs_plan_ctas(int n_row_blocks, int n_col_tiles, int sms, int reserved, int limit);

/* Host arithmetic only (no reference counterpart): the column shares per 128-row block that the plan-times-matrix
 * kernel with the row operand resident uses for `rows` output rows against `cols` columns on a device with `sms`
 * SMs (prec FS_PREC_TF32: 128-column tiles, FS_PREC_FP32: 64-column tiles); *slots (may be NULL) receives the number
 * of raw output tiles the scratch holds for clouds of at most max(rows, cols) points. rows/128 * shares never
 * exceeds it, and a share never has fewer than 8 column tiles. Returns 0 on non-positive sizes. */
int fs_plan_pv_split(int rows, int cols, int prec, int sms, int* slots);

/* Optional label-augmented ground cost (OTDD), reference kernels/sinkhorn_flashstyle_sqeuclid.py:545-560
 * and kernels/sinkhorn_triton_grad_sqeuclid.py:225-236: the logit of entry (i, j) becomes
 *   (lambda_x * 2cs * x_i.y_j - lambda_y * cs * W[label_x_i, label_y_j]) / eps + bias_j.
 * A NULL pointer, V <= 0 or lambda_y == 0 means the plain squared-Euclidean cost. Entry points that take
 * this descriptor size their workspace with fs_workspace_bytes_labels (the tensor-core engine carries the
 * table through the contraction as 3V extra operand columns). All pointers are device pointers. */
typedef struct fs_label_cost {
  const int* label_x;    /* [n] class of every x point, in [0, V) */
  const int* label_y;    /* [m] class of every y point, in [0, V) */
  const float* W;        /* [V, V] row-major label-to-label cost, indexed W[label_x, label_y] */
  int V;
  float lambda_x;        /* weight of the Euclidean term (> 0) */
  float lambda_y;        /* weight of the label term */
} fs_label_cost;

/* Scratch bytes needed by `op` (one of FS_OP_*) at these sizes. */
size_t fs_workspace_bytes(int op, int n, int m, int d, int prec);
/* The same for a call that passes an fs_label_cost with V = n_classes (0 = none). */
size_t fs_workspace_bytes_labels(int op, int n, int m, int d, int prec, int n_classes);

/* Row log-sum-exp potential update.
 *   out_i = -eps*damping * log sum_j exp( (2cs/eps) x_i.y_j + bias_j )
 *   bias_j = pot_j/eps + logw_j   when logw != NULL
 *          = pot_j                when logw == NULL (bias already scaled)
 * Replaces kernels/sinkhorn_flashstyle_sqeuclid.py:815-955 (flashsinkhorn_lse,
 * raw bias) and :958-1090 (flashsinkhorn_lse_fused); the g-update is the same
 * call with (y, x) swapped, as sinkhorn_solvers.py:629-632 does. */
int fs_lse(const float* x, const float* y, int n, int m, int d,
           const float* pot, const float* logw, float* out,
           float eps, float cost_scale, float damping,
           int prec, void* ws, size_t ws_bytes, void* stream);

/* Hard (non-entropic) c-transform, inner minimum:
 *   out_val_i = min_j ( -2*cost_scale * x_i.y_j + bias_j ),   out_idx_i = the smallest j attaining it
 * (the caller adds cost_scale*|x_i|^2 and passes bias_j = cost_scale*|y_j|^2 - psi_j). Same staged
 * operands and tile engine as fs_lse (workspace: fs_workspace_bytes(FS_OP_LSE, ...)); prec selects TF32,
 * 3xTF32 or true-fp32 products. Replaces kernels/c_transform_sqeuclid.py:219-354 (c_transform_kernel). */
int fs_c_transform(const float* x, const float* y, int n, int m, int d,
                   const float* bias, float cost_scale, float* out_val, int* out_idx,
                   int prec, void* ws, size_t ws_bytes, void* stream);

/* One Jacobi (symmetric) step: both sides read the OLD potentials.
 *   f_out = (1-w) f_hat + w * (-eps*damp_f*LSE_j[(2cs/eps)x_i.y_j + g_hat_j/eps + log_b_j])
 *   g_out likewise with roles swapped.
 * When alpha_x/beta_y are non-NULL the unbalanced shift correction
 *   f_out -= w*alpha_x*(1-damp_f),  g_out -= w*beta_y*(1-damp_g)
 * (sinkhorn_solvers.py:509-517) is fused in; pass NULL to get exactly the
 * kernel result of kernels/sinkhorn_flashstyle_sqeuclid.py:1093-1317
 * (flashsinkhorn_symmetric_step). f_out/g_out must not alias f_hat/g_hat. */
int fs_symmetric_step(const float* x, const float* y, int n, int m, int d,
                      const float* f_hat, const float* g_hat,
                      const float* log_a, const float* log_b,
                      float* f_out, float* g_out,
                      const float* alpha_x, const float* beta_y,
                      float eps, float w, float damp_f, float damp_g, float cost_scale,
                      int prec, void* ws, size_t ws_bytes, void* stream,
                      const fs_label_cost* labels);

/* Row-sharded form of fs_symmetric_step for multi-GPU solves (no reference counterpart: the
 * reference is single-GPU). Only rows [f_begin, f_end) of f_out and [g_begin, g_end) of g_out are
 * computed; all inputs are full-size and replicated on every rank, the caller all-gathers the
 * produced slices. `restage` = 0 re-uses the tensor-core operands that an earlier call with the
 * same (x, y, n, m, d, prec) staged into the SAME workspace (x, y constant over a solve), so a
 * step costs only the two streaming passes. */
int fs_symmetric_step_range(const float* x, const float* y, int n, int m, int d,
                            const float* f_hat, const float* g_hat,
                            const float* log_a, const float* log_b,
                            float* f_out, float* g_out,
                            const float* alpha_x, const float* beta_y,
                            float eps, float w, float damp_f, float damp_g, float cost_scale,
                            int f_begin, int f_end, int g_begin, int g_end, int restage,
                            int prec, void* ws, size_t ws_bytes, void* stream);

/* Several row-sharded Jacobi steps - of one problem or of several independent problems with the same feature
 * dimension - enqueued together (no reference counterpart). Each item is one fs_symmetric_step_range call
 * with its own workspace (sized for FS_OP_STEP at its n, m); a side whose row range is empty is skipped.
 * On the tensor-core engine up to four of the resulting soft-min passes share ONE kernel launch (their work
 * items form one list that is cut over the SMs), so the fixed cost of a launch is paid once per group: this is
 * what keeps short per-rank passes efficient when a debiased loss (three problems, four passes per iteration)
 * is sharded over many GPUs. Results are those of the separate calls up to the order in which partial sums
 * of a row are merged. At most 8 items. */
typedef struct fs_step_item {
  const float* x; const float* y; int n, m;
  const float* f_hat; const float* g_hat; const float* log_a; const float* log_b;
  float* f_out; float* g_out;
  const float* alpha_x; const float* beta_y;   /* shift-correction vectors, NULL on balanced sides */
  float eps, w, damp_f, damp_g, cost_scale;
  int f_begin, f_end, g_begin, g_end;
  int restage;                                   /* 0: operands staged by an earlier call into the same ws */
  void* ws; size_t ws_bytes;
  /* Packed potentials (all three 0 = plain contiguous vectors). With f_shard > 0 element j of f_hat and of
   * f_out is at ptr[(j / f_shard) * pack_stride + j % f_shard], likewise g with g_shard: the layout of a
   * [ranks, pack_stride] buffer that one all-gather completes when rank r owns rows [r*shard, (r+1)*shard)
   * of every vector. A row range must then lie inside one shard. Tensor-core engine only. */
  int f_shard, g_shard, pack_stride;
} fs_step_item;
int fs_symmetric_step_multi(const fs_step_item* items, int n_items, int d, int prec, void* stream);

/* Several symmetric solves at once (replaces the Python loop over batch items of the reference,
 * samples_loss.py:515-552, and serves the three solves of a debiased loss): same step sequence per item as
 * fs_solve_symmetric (own eps schedule, lengths may differ), no early stopping, no warm start, no label cost.
 * Every step of all unfinished items goes out as fused multi-pass launches (up to four soft-min passes per
 * launch), so B small problems cost about a quarter of B solves' worth of launches. Results equal the
 * one-at-a-time solves up to the order in which a row's partial sums are merged (rounding level, not bit for
 * bit). Each item brings its own workspace of fs_workspace_bytes(FS_OP_SOLVE_SYMMETRIC, n, m, d, prec) bytes.
 * An item with y == x, log_b == log_a (and rho_x == rho_y) is a self-transport problem: one soft-min per step. */
typedef struct fs_batch_item {
  const float* x; const float* y; int n, m;
  const float* log_a; const float* log_b;
  const double* eps_list_host; int n_eps;
  float* f; float* g; float* f_pre; float* g_pre;   /* outputs [n], [m]; the *_pre pair may be NULL */
  void* ws; size_t ws_bytes;
} fs_batch_item;
int fs_solve_symmetric_batched(const fs_batch_item* items, int n_items, int d, int last_extrapolation,
                               float cost_scale, double rho_x, double rho_y, int prec, void* stream);

/* The same with a block-sparse list of kept 128 x 128 tiles (CSR over the 128-row blocks of x, and the
 * transposed list over the blocks of y, as fs_solve_alternating takes them; all four NULL = dense). No
 * reference counterpart. Row ranges must start on multiples of 128; a multi-GPU caller cuts them so that
 * every rank gets about the same number of kept tiles rather than of rows. */
int fs_symmetric_step_range_tiles(const float* x, const float* y, int n, int m, int d,
                                  const float* f_hat, const float* g_hat,
                                  const float* log_a, const float* log_b,
                                  float* f_out, float* g_out,
                                  const float* alpha_x, const float* beta_y,
                                  float eps, float w, float damp_f, float damp_g, float cost_scale,
                                  int f_begin, int f_end, int g_begin, int g_end, int restage,
                                  const int* tile_row_ptr, const int* tile_col_idx,
                                  const int* tile_row_ptr_t, const int* tile_col_idx_t,
                                  int prec, void* ws, size_t ws_bytes, void* stream);

/* Row-sharded form of fs_grad: rows [x_begin, x_end) of grad_x and [y_begin, y_end) of grad_y. */
int fs_grad_range(const float* x, const float* y, int n, int m, int d,
                  const float* a, const float* b, const float* log_a, const float* log_b,
                  const float* f, const float* g, const float* grad_scale,
                  float* grad_x, float* grad_y, float eps, float cost_scale,
                  int x_begin, int x_end, int y_begin, int y_end,
                  int prec, void* ws, size_t ws_bytes, void* stream);

/* Whole symmetric (GeomLoss-style) solve, enqueued without host synchronisation.
 * Schedule: one step with weight 1 at eps_list[0]; one step with weight 1/2 per
 * entry of eps_list; if last_extrapolation, one more step with weight 1 at
 * eps_list[n_eps-1]. Early stop (threshold >= 0): every check_every loop steps
 * max|delta f_hat|, max|delta g_hat| against the snapshot of the previous check
 * is evaluated ON THE DEVICE; once below threshold the remaining loop steps are
 * skipped (the final extrapolation still runs).
 *   f_init/g_init : standard (unshifted) warm-start potentials or NULL (zeros)
 *   f, g          : final standard potentials
 *   f_pre, g_pre  : potentials before the extrapolation step (may be NULL)
 *   iters_used    : device int, number of steps executed (may be NULL)
 * Replaces sinkhorn_solvers.py:290-707 (sinkhorn_flashstyle_symmetric). */
int fs_solve_symmetric(const float* x, const float* y, int n, int m, int d,
                       const float* log_a, const float* log_b,
                       const double* eps_list_host, int n_eps, int last_extrapolation,
                       float cost_scale, double rho_x, double rho_y,
                       double threshold, int check_every,
                       const float* f_init, const float* g_init,
                       float* f, float* g, float* f_pre, float* g_pre,
                       int* iters_used,
                       int prec, void* ws, size_t ws_bytes, void* stream,
                       const fs_label_cost* labels);

/* Whole alternating (Gauss-Seidel) solve. For each eps of eps_list, iters_per_eps
 * iterations of { f_hat <- LSE(g_hat) ; g_hat <- LSE(new f_hat) } (no averaging,
 * no shift correction), warm-started from the previous eps. With n_eps == 1 this
 * is sinkhorn_solvers.py:30-287 (sinkhorn_flashstyle_alternating) with
 * n_iters = iters_per_eps; ott_convention != 0 selects its :188-228 branch
 * (g first, log-marginals outside the LSE). Early stop as above, counted in
 * iterations across the whole run. tile_row_ptr/tile_col_idx (may be NULL) give a
 * CSR list of kept 128x128 (x-tile, y-tile) pairs: tiles not listed contribute
 * nothing to either LSE (block-sparse skipping; no reference counterpart). */
int fs_solve_alternating(const float* x, const float* y, int n, int m, int d,
                         const float* log_a, const float* log_b,
                         const double* eps_list_host, int n_eps, int iters_per_eps,
                         float cost_scale, double rho_x, double rho_y,
                         int ott_convention, double threshold, int check_every,
                         const int* tile_row_ptr, const int* tile_col_idx,
                         const int* tile_row_ptr_t, const int* tile_col_idx_t,
                         float* f, float* g, int* iters_used,
                         int prec, void* ws, size_t ws_bytes, void* stream);

/* out = P v (axis 1, v has m entries, out n) or P^T v (axis 0), with
 * P_ij = exp( (f_hat_i + g_hat_j + 2cs x_i.y_j)/eps + log_a_i + log_b_j ).
 * Replaces kernels/apply_flash.py:835-951 (apply_plan_vec_flashstyle). */
int fs_apply_vec(const float* x, const float* y, int n, int m, int d,
                 const float* f_hat, const float* g_hat,
                 const float* log_a, const float* log_b,
                 const float* vec, float* out,
                 float eps, int axis, float cost_scale,
                 int prec, void* ws, size_t ws_bytes, void* stream);

/* out = P V (axis 1: V is [m,dv], out [n,dv]; optional scale[m] multiplies the
 * rows of V) or P^T V (axis 0: V is [n,dv], out [m,dv]; scale must be NULL).
 * Replaces kernels/apply_flash.py:360-579 (apply_plan_mat_flashstyle; the
 * reference requires dv == d, this ABI does not). */
int fs_apply_mat(const float* x, const float* y, int n, int m, int d,
                 const float* f_hat, const float* g_hat,
                 const float* log_a, const float* log_b,
                 const float* mat, int dv, const float* scale, float* out,
                 float eps, int axis, float cost_scale,
                 int prec, void* ws, size_t ws_bytes, void* stream);

/* fs_apply_mat for callers that must not allocate. It has no counterpart in the reference.
 * Same result as fs_apply_mat(..., FS_PREC_SIMT, ...) but takes no workspace: its one scratch
 * vector lives in a 256 KiB static device array inside the library (held by every GPU that
 * loads it, until exit). Meant for hosts that cannot provide scratch memory: operator
 * callbacks that may not re-enter their framework's allocator, fixed-memory real-time loops,
 * plug-ins that only ever see their input and output buffers.
 *   - the output row count (n for axis 1, m for axis 0) must be <= 65536, else FS_ERR_BAD_ARG;
 *   - calls that overlap on one GPU race on the shared array: serialise them;
 *   - the first call on a device looks up the array's device address; make that call outside
 *     any stream capture. Nothing in the array needs clearing between calls. */
int fs_apply_mat_static(const float* x, const float* y, int n, int m, int d,
                        const float* f_hat, const float* g_hat,
                        const float* log_a, const float* log_b,
                        const float* mat, int dv, const float* scale, float* out,
                        float eps, int axis, float cost_scale, void* stream);

/* Analytic gradient of the OT cost (barycentric form), standard potentials f, g:
 *   grad_x_i = 2cs*gs*a_i*( x_i - sum_j w_ij y_j / max(sum_j w_ij, 1e-40) ),
 *   w_ij = exp( (g_j - C_ij)/eps + log_b_j );  grad_y symmetric with f, a.
 * grad_scale points to one device float (gs) or is NULL (gs = 1). Either output
 * may be NULL. Any d (no separate large-d entry point). Replaces
 * kernels/sinkhorn_triton_grad_sqeuclid.py:891-1207
 * (sinkhorn_geomloss_online_grad_sqeuclid). */
int fs_grad(const float* x, const float* y, int n, int m, int d,
            const float* a, const float* b, const float* log_a, const float* log_b,
            const float* f, const float* g, const float* grad_scale,
            float* grad_x, float* grad_y,
            float eps, float cost_scale,
            int prec, void* ws, size_t ws_bytes, void* stream,
            const fs_label_cost* labels);

/* out_i = (-4cs/eps) sum_j P_ij (A_i.y_j) y_j with P_ij = exp((f_i+g_j-C_ij)/eps)
 * (OTT-convention potentials, log-weights already inside f, g). Replaces
 * kernels/apply_ott.py:453-566 (mat5_sqeuclid). */
int fs_mat5(const float* x, const float* y, int n, int m, int d,
            const float* f_ott, const float* g_ott, const float* A, float* out,
            float eps, float cost_scale,
            int prec, void* ws, size_t ws_bytes, void* stream);

/* Conjugate gradient on the HVP's Schur complement, entirely on the device:
 *   solve (diag(denom) - P^T diag(1/diag_x) P) z = rhs,  z0 = 0,
 * stopping when |r| <= max(atol, rtol*|r0|) or after max_iter iterations; all
 * dot products, the stopping test and the iteration counter stay on the GPU.
 * info (device, 4 floats): [converged(0/1), iterations, |r|, |r0|].
 * Replaces the loop of cg.py:27-121 (conjugate_gradient) as driven by
 * hvp.py:505-520 (two plan applications per iteration). */
int fs_schur_cg(const float* x, const float* y, int n, int m, int d,
                const float* f_hat, const float* g_hat,
                const float* log_a, const float* log_b,
                const float* diag_x, const float* denom, const float* rhs,
                float* z, float* info,
                float eps, float cost_scale, int max_iter, float rtol, float atol,
                int prec, void* ws, size_t ws_bytes, void* stream);

/* ---- Plan session (no reference counterpart as an API; replaces the repeated launches inside the
 * reference's hvp.py:282-623) ------------------------------------------------------------------------------
 * Many applications of ONE transport plan P = diag(a) exp((f_hat + g_hat + 2cs x.y)/eps) diag(b): the operands
 * are staged and the two log-normaliser vectors computed ONCE (fs_plan_session_begin: two soft-min passes); every
 * later application then costs a single streaming pass. All calls of a session take the same x, y, sizes,
 * potentials, eps, cost_scale, prec and the same workspace of fs_plan_session_bytes() bytes; nothing else may
 * write that workspace in between. The Hessian-vector product uses it: 11 + 2K passes for K CG iterations
 * (the reference launches 10 + 2K kernels, hvp.py:164-623). */
size_t fs_plan_session_bytes(int n, int m, int d, int prec);
int fs_plan_session_begin(const float* x, const float* y, int n, int m, int d,
                          const float* f_hat, const float* g_hat, const float* log_a, const float* log_b,
                          float eps, float cost_scale, int prec, void* ws, size_t ws_bytes, void* stream);
/* kind 0: out = P v (axis 1, operand [m]) or P^T u (axis 0, operand [n]); reference
 * kernels/apply_flash.py:835-951. kind 1: out = P V / P^T V with dv <= d columns and an optional per-point
 * `scale` of V's rows (axis 1 only); kernels/apply_flash.py:360-579. kind 2: the Mat5 term
 * out_i = coef * sum_j P_ij (A_i . y_j) y_j with operand = A [n, d], axis 1, dv = d; kernels/apply_ott.py:453-566
 * (coef = -4 cs / eps there). */
int fs_plan_session_apply(const float* x, const float* y, int n, int m, int d,
                          const float* f_hat, const float* g_hat, const float* log_a, const float* log_b,
                          int kind, const float* operand, int dv, const float* scale, float coef, float* out,
                          int axis, float eps, float cost_scale, int prec, void* ws, size_t ws_bytes, void* stream);
/* fs_schur_cg inside a session (no staging, no normaliser passes): reference hvp.py:505-520, cg.py:27-121. */
int fs_plan_session_cg(const float* x, const float* y, int n, int m, int d,
                       const float* f_hat, const float* g_hat, const float* log_a, const float* log_b,
                       const float* diag_x, const float* denom, const float* rhs, float* z, float* info,
                       float eps, float cost_scale, int max_iter, float rtol, float atol, int prec,
                       void* ws, size_t ws_bytes, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FLASH_SINKHORN_B200_H */
