// tcgen05 / TMEM / TMA streaming engine for sm_100a: LSE pass (potential updates), arg-max pass (hard
// c-transform) and plan-times-matrix pass (gradient, plan applications).
//
// LSE / arg-max pass. Work item = (row block of BM = 128*NHALF rows of the "row" cloud, column tile of BN
// rows of the "column" cloud). The items, row block after row block, are cut into equal contiguous ranges,
// one per CTA, one CTA per SM (a single wave). For each row block it touches ("segment") a CTA keeps the
// K-padded row operand (constant ones in the bias columns) resident in shared memory while column tiles
// stream through an NSTAGE ring of TMA-filled buffers. Warp roles (FlashAttention-style specialisation):
//   warp 0      : TMA producer (one lane)
//   warps 1, 3  : tcgen05.mma issuers, one lane per 128-row half; warp 1 owns the TMEM allocation
//   warp 2      : idle
//   warps 4..   : soft-max warpgroups, one per 128-row half and half of each tile's columns; thread t of a
//                 warpgroup owns score row t (TMEM lane t), so row max / row sum need no shuffles.
// Per column tile and half an MMA lane accumulates S = A_half x B_tile^T (M=128, N=BN, K=8 per instruction,
// kind::tf32) into one of two TMEM buffers of that half, commits to an mbarrier, and the warpgroups drain the
// other buffer with tcgen05.ld meanwhile. Because the bias sits in the contraction, the drained value is
// (logit / scale): max -> one FFMA + one ex2.approx + one FADD per entry. A row block shared by several CTAs
// gets one partial per row from each; the CTA that takes the block's last ticket merges them in a fixed order.
//
// Plan-times-matrix pass: see tc_pv_kernel below (second GEMM with the weights read from TMEM).
//
// Every wait on an mbarrier is bounded (clock64 budget); a wait that runs out raises a
// CTA-wide abort flag, the CTA drains its outstanding copies and MMAs (bounded again),
// frees its TMEM and returns; a device-global error word records the event.
#include "fs_tc.cuh"
#include "fs_ptx.cuh"

#include <cuda.h>
#include <cudaTypedefs.h>
#include <cuda_runtime.h>

#include <cstdlib>
#include <atomic>
#include <mutex>

namespace fs {
namespace tc {

__device__ int g_tc_error = 0;  // non-zero once any bounded wait gave up (read by fs_device_error)

namespace {

// One streaming pass of a launch ("sub-pass"): rows [row_begin, nr) of one cloud against all columns of the other.
struct SubPass {
  CUtensorMap mapA_full, mapA_tail, mapB_full, mapB_tail;
  int nr, nc;        // end of the row range / valid columns
  int row_begin;     // first row of the range (row sharding)
  int ntiles;        // column tiles of BN
  int nblk;          // row blocks of BM rows
  int item0;         // index of this pass's first (row block, column tile) item in the launch's item list
  float scale2;      // 2*cs*log2e/eps: logit = scale2 * S
  float eps;
  LseEpilogue ep;
  // Partial (scale2*max, sum) pairs of row blocks that several CTAs share, and one arrival counter per row
  // block (zero between launches). Passes of one launch never share these.
  float* part_m;
  float* part_s;
  int part_stride;
  int* tickets;
  int* out_idx;  // AM kernels: arg-max column per row (values go to ep.out, multiplied by scale2)
  // CSR kernels: block-sparse list of kept (128-row block, 128-column tile) pairs. csr_rp points at the entry
  // of the first row block of this launch's row range (nblk + 1 entries are read), csr_ci is the whole
  // column-tile array (indexed with the values of csr_rp).
  const int* csr_rp;
  const int* csr_ci;
};

// A launch = up to NSUB passes over operands of the same shape class (same K blocks, tile shape and ring depth).
// Work split: the (row block, column tile) items of all passes, pass after pass and row block after row block,
// are cut into gridDim.x equal contiguous ranges, one per CTA (one CTA per SM, a single wave). A CTA's range may
// end one row block and begin the next (also of the next pass); a row block shared by several CTAs gets one
// partial pair per row from each, and the last of them to finish merges the pairs.
template <int NSUB>
struct Launch {
  int nsub;
  int nfull, ntail;  // K blocks: nfull of 32 floats (128B swizzle) + ntail of 8 floats (32B swizzle)
  int nstage;
  long long total;   // items of all passes (dense passes: sum of nblk * ntiles)
  SubPass sub[NSUB];
};
constexpr int kMaxSub = 4;  // passes per multi-pass launch (keeps the kernel parameters under 4 KB)

// Soft-max warpgroups per 128-row half: each takes half of every tile's 32-column chunks (more warps per
// scheduler to hide the fixed latencies around the chunk max / rescale); their partials merge at the end.
constexpr int kParts = 2;

// AM = false: online log-sum-exp of the scaled scores (potential update). AM = true: running maximum of the
// raw scores and the smallest column attaining it (hard c-transform); no exponentials at all.
// CSR = true: the item list is the list of kept tiles (row block after row block, NHALF = 1, BN = 128) instead
// of all nblk x ntiles pairs; everything else - contiguous ranges per CTA, segments, ticketed merge - is the same.
// NSUB > 1: several dense passes in one launch (no arg-max, no tile list, no device-side early-stop flag).
template <int NHALF, int BN, bool AM, bool CSR = false, int NSUB = 1>
__global__ void __launch_bounds__(128 + 128 * NHALF * kParts, 1)
tc_lse_kernel(const __grid_constant__ Launch<NSUB> P) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  constexpr int BM = 128 * NHALF;
  // This CTA's items [w_begin, w_end) of the flattened (row block, column tile) list.
  static_assert(!CSR || (NHALF == 1 && BN == 128 && !AM), "tile lists are over 128 x 128 tiles");
  static_assert(NSUB == 1 || (!CSR && !AM), "multi-pass launches are dense soft-min passes");
  int sub = 0;  // pass of the segment this thread's role is working on (always 0 when NSUB == 1)
  auto SP = [&]() -> const SubPass& { return P.sub[NSUB == 1 ? 0 : sub]; };
  const SubPass& p = P.sub[0];  // single-pass code paths (CSR, arg-max, early-stop flag) read pass 0
  const int rp0 = CSR ? p.csr_rp[0] : 0;
  const long long total_items = CSR ? (long long)(p.csr_rp[p.nblk] - rp0) : P.total;
  // CTAs that share the items. A sparse list may hold few tiles per CTA; G is then lowered so that a row block
  // (at most ntiles items) is never cut into more pieces than there are partial slots (16).
  int G = (int)gridDim.x;
  if (CSR) {
    long long cap = (12 * total_items) / (p.ntiles > 0 ? p.ntiles : 1);
    if (cap > total_items) cap = total_items;  // no CTA without items inside the list: pieces are counted by owner
    if (cap < 1) cap = 1;
    if (cap < G) G = (int)cap;
  }
  const bool has_work = (int)blockIdx.x < G && total_items > 0;
  const int w_begin = has_work ? (int)((total_items * blockIdx.x) / G) : 0;
  const int w_end = has_work ? (int)((total_items * (blockIdx.x + 1)) / G) : 0;
  // Items of row block b are [row_start(b), row_end(b)); blk_of(w) = row block holding item w.
  // (b counts the row blocks of the current pass; blk_of and next_blk also move `sub` to the pass of the item.)
  auto row_start = [&](int b) { return CSR ? p.csr_rp[b] - rp0 : SP().item0 + b * SP().ntiles; };
  auto row_end = [&](int b) { return CSR ? p.csr_rp[b + 1] - rp0 : SP().item0 + (b + 1) * SP().ntiles; };
  auto blk_of = [&](int w) {
    if (!CSR) {
      if (NSUB > 1) {
        sub = 0;
        while (sub + 1 < P.nsub && P.sub[sub + 1].item0 <= w) ++sub;
      }
      return (w - SP().item0) / SP().ntiles;
    }
    int lo = 0, hi = p.nblk - 1;  // smallest b with row_end(b) > w
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (p.csr_rp[mid + 1] - rp0 > w) hi = mid; else lo = mid + 1;
    }
    return lo;
  };
  auto next_blk = [&](int b, int w) {  // row block of item w, the first item after row block b
    ++b;
    if (CSR) while (row_end(b) <= w) ++b;
    if (NSUB > 1 && b == SP().nblk) {  // dense passes have no empty row block: w opens the next pass
      ++sub;
      b = 0;
    }
    return b;
  };
  auto col_of = [&](int w, int b) { return CSR ? p.csr_ci[rp0 + w] : w - row_start(b); };
  // First item of CTA c; CTA holding item t (largest c whose first item is <= t).
  auto cta_first = [&](int c) { return (int)((total_items * c) / G); };
  auto cta_of = [&](int t) {
    int c = (int)(((long long)t * G) / total_items);
    while (c + 1 < G && cta_first(c + 1) <= t) ++c;
    while (c > 0 && cta_first(c) > t) --c;
    return c;
  };

  if (NSUB == 1 && SP().ep.ctrl && SP().ep.ctrl->converged) {  // solve already stopped: identity step
    if (SP().ep.old && SP().ep.out)
      for (int r = SP().row_begin + blockIdx.x * blockDim.x + tid; r < SP().nr; r += gridDim.x * blockDim.x)
        SP().ep.out[r] = SP().ep.old[r];
    return;
  }

  // ---- shared memory carve-up (all operand blocks 1024-byte aligned) ----
  uint8_t* base = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t a_half_bytes = P.nfull * (128 * 128) + P.ntail * (128 * 32);
  const uint32_t b_stage_bytes = P.nfull * (BN * 128) + P.ntail * (BN * 32);
  uint8_t* a_smem = base;
  uint8_t* b_smem = a_smem + NHALF * a_half_bytes;
  uint64_t* bars = (uint64_t*)(b_smem + P.nstage * b_stage_bytes);
  // barrier indices
  const int B_FULL = 0, B_EMPTY = P.nstage, S_FULL = 2 * P.nstage, S_EMPTY = S_FULL + 2 * NHALF,
            A_FULL = S_EMPTY + 2 * NHALF, A_EMPTY = A_FULL + 1, DRAIN = A_EMPTY + 1, NBARS = DRAIN + 2;
  uint32_t* tmem_slot = (uint32_t*)(bars + NBARS);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
  volatile int* last_flag = (volatile int*)(tmem_slot + 2);  // this CTA took the last ticket of its row block
  float* merge_off = (float*)(tmem_slot + 4);        // [NHALF*128] partials of the second column part
  float* merge_sum = merge_off + NHALF * 128;
  auto bar = [&](int i) { return smem_u32(bars + i); };

  constexpr uint32_t kTmemCols = (2 * NHALF * BN) < 32 ? 32 : (2 * NHALF * BN);

  if (tid == 0) {
    for (int s = 0; s < P.nstage; ++s) {
      mbar_init(bar(B_FULL + s), 1);
      mbar_init(bar(B_EMPTY + s), NHALF);  // one commit per MMA-issuing lane (one lane per 128-row half)
    }
    for (int i = 0; i < 2 * NHALF; ++i) {
      mbar_init(bar(S_FULL + i), 1);
      mbar_init(bar(S_EMPTY + i), 4 * kParts);  // one arrive per soft-max warp reading the buffer
    }
    mbar_init(bar(A_FULL), 1);
    mbar_init(bar(A_EMPTY), NHALF);
    mbar_init(bar(DRAIN), 1);
    mbar_init(bar(DRAIN + 1), 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ===================== TMA producer =====================
    if (lane == 0) {
      int issued = 0, seg = 0;  // column tiles issued so far by this CTA (ring position), segment count
      bool ok = true;
      // Column tile `issued` (a CTA-wide running index) of the segment that starts at item w0.
      auto load_b = [&](int j) -> bool {
        const int s = issued % P.nstage;
        const uint32_t ph = (issued / P.nstage) & 1;
        if (!mbar_wait(bar(B_EMPTY + s), ph ^ 1, abort_flag, 2000)) return false;
        mbar_expect_tx(bar(B_FULL + s), b_stage_bytes);
        uint32_t dst = smem_u32(b_smem + s * b_stage_bytes);
        const int col0 = j * BN;
        for (int kb = 0; kb < P.nfull; ++kb)
          tma_load_2d(dst + kb * (BN * 128), &SP().mapB_full, kb * 32, col0, bar(B_FULL + s));
        for (int t = 0; t < P.ntail; ++t)
          tma_load_2d(dst + P.nfull * (BN * 128) + t * (BN * 32), &SP().mapB_tail, P.nfull * 32 + t * 8, col0,
                      bar(B_FULL + s));
        ++issued;
        return true;
      };
      int pre = 0;  // column tiles of the current segment that were already issued during the previous one
#pragma unroll 1
      int blk = has_work ? blk_of(w_begin) : 0;
#pragma unroll 1
      for (int w = w_begin; ok && w < w_end; ++seg) {
        const int seg_end = row_end(blk) < w_end ? row_end(blk) : w_end;
        const int row0 = SP().row_begin + blk * BM;
        // The row operand of the previous segment must have been read by its last MMA.
        if (!mbar_wait(bar(A_EMPTY), (seg & 1) ^ 1, abort_flag, 2000)) break;
        mbar_expect_tx(bar(A_FULL), NHALF * a_half_bytes);
#pragma unroll 1
        for (int h = 0; h < NHALF; ++h) {
          uint32_t dst = smem_u32(a_smem + h * a_half_bytes);
          for (int kb = 0; kb < P.nfull; ++kb)
            tma_load_2d(dst + kb * (128 * 128), &SP().mapA_full, kb * 32, row0 + h * 128, bar(A_FULL));
          for (int t = 0; t < P.ntail; ++t)
            tma_load_2d(dst + P.nfull * (128 * 128) + t * (128 * 32), &SP().mapA_tail, P.nfull * 32 + t * 8,
                        row0 + h * 128, bar(A_FULL));
        }
#pragma unroll 1
        for (int t = w + pre; ok && t < seg_end; ++t) ok = load_b(col_of(t, blk));
        w = seg_end;
        // Next segment (another row block, columns from 0): its first column tiles do not need the new row
        // operand, so they go into ring slots as this segment's tiles retire - every slot waited for here
        // holds a tile of this or an earlier segment, which the MMA lane consumes without the next A.
        pre = 0;
        if (ok && w < w_end) {
          blk = next_blk(blk, w);
          const int nnext = (row_end(blk) < w_end ? row_end(blk) : w_end) - w;
          const int npre = nnext < P.nstage ? nnext : P.nstage;
#pragma unroll 1
          for (; ok && pre < npre; ++pre) ok = load_b(col_of(w + pre, blk));
        }
      }
      if (*abort_flag) {  // let every copy we issued land before the CTA goes away
        if (seg > 0) mbar_wait_quiet(bar(A_FULL), (seg - 1) & 1);
        for (int j = (issued > P.nstage ? issued - P.nstage : 0); j < issued; ++j)
          mbar_wait_quiet(bar(B_FULL + j % P.nstage), (j / P.nstage) & 1);
      }
    }
  } else if (warp == 1 || (warp == 3 && NHALF == 2)) {
    // ===================== MMA issuers: one warp per 128-row half =====================
    // A stream that shares its scheduler with soft-max warps sustains one MMA per ~90 cycles, the tensor pipe
    // one per 64: with one issuer per half (warps 1 and 3) the score tiles of the next column tile are ready
    // well before the soft-max warps ask for them, instead of just in time. All 32 lanes run the loop and one
    // elected lane issues: descriptor arithmetic is then warp-uniform (uniform registers, which is where
    // tcgen05 instructions take their operands) instead of per-thread values moved over for every MMA. Every
    // exit decision is a warp vote, since elect.sync needs all 32 lanes at the same instruction. Tile lists keep
    // the loop on lane 0 alone (kWarpIssue false): with one MMA per tile (d = 3) and the list look-ups in the
    // loop the converged form measured 15 % slower per pass there.
    constexpr bool kWarpIssue = !CSR;
    auto vote = [&](bool okl) { return kWarpIssue ? (__all_sync(0xffffffffu, okl) != 0) : okl; };
    auto pick = [&]() { return kWarpIssue ? elect_one() : true; };
    if (kWarpIssue || lane == 0) {
      const int h = (warp == 1) ? 0 : 1;
      constexpr uint32_t idesc = make_idesc(BN);
      const uint32_t a_lo0 = desc_lo(smem_u32(a_smem + h * a_half_bytes));
      bool ok = true;
      int jt = 0, seg = 0;  // column tiles processed so far by this CTA (ring / buffer position), segment count
      int blk = has_work ? blk_of(w_begin) : 0;
#pragma unroll 1
      for (int w = w_begin; ok && w < w_end; ++seg) {
        const int nseg = (row_end(blk) < w_end ? row_end(blk) : w_end) - w;
        if (!vote(mbar_wait(bar(A_FULL), seg & 1, abort_flag, 2000))) break;
        tc_fence_after();
#pragma unroll 1
        for (int i = 0; i < nseg; ++i, ++jt) {
          const int s = jt % P.nstage;
          const uint32_t ph = (jt / P.nstage) & 1;
          if (!vote(mbar_wait(bar(B_FULL + s), ph, abort_flag, 2000))) { ok = false; break; }
          const int buf = jt & 1;
          const uint32_t sph = (jt >> 1) & 1;
          if (!vote(mbar_wait(bar(S_EMPTY + h * 2 + buf), sph ^ 1, abort_flag, 2000))) {
            ok = false;
            break;
          }
          tc_fence_after();
          // Descriptors are advanced incrementally: the low word holds (address >> 4), the high word (stride,
          // version, swizzle) is a constant per block class.
          const uint32_t d_tmem = tmem_base + (uint32_t)((h * 2 + buf) * BN);
          uint32_t al = a_lo0, bl = desc_lo(smem_u32(b_smem + s * b_stage_bytes));
          // One election per tile where a tile has few MMAs (the 256-row plans: measured 1.3 % faster per pass,
          // 10 % for the arg-max pass), one per instruction in the 128-row plans with their long K (d = 128:
          // 1.3 % faster that way). kTileElect false: all lanes enter and every instruction is elected.
          constexpr bool kTileElect = (NHALF == 2);
          if (kTileElect ? pick() : true) {
            uint32_t acc = 0;
#pragma unroll 1
            for (int kb = 0; kb < P.nfull; ++kb) {
#pragma unroll
              for (int ks = 0; ks < 4; ++ks) {
                if (kTileElect || pick())
                  umma_tf32(d_tmem, pack_desc(al + 2 * ks, kDescHi128), pack_desc(bl + 2 * ks, kDescHi128), idesc, acc);
                acc = 1;
              }
              al += (128 * 128) >> 4;
              bl += (BN * 128) >> 4;
            }
#pragma unroll 1
            for (int t = 0; t < P.ntail; ++t) {
              if (kTileElect || pick())
                umma_tf32(d_tmem, pack_desc(al, kDescHi32), pack_desc(bl, kDescHi32), idesc, acc);
              acc = 1;
              al += (128 * 32) >> 4;
              bl += (BN * 32) >> 4;
            }
            if (kTileElect || pick()) {
              umma_commit(bar(S_FULL + h * 2 + buf));
              umma_commit(bar(B_EMPTY + s));
            }
          }
          if (kWarpIssue) __syncwarp();
        }
        // the row operand may be replaced once every MMA issued so far retired
        if (pick()) umma_commit(bar(A_EMPTY));
        if (kWarpIssue) __syncwarp();
        w += nseg;
        if (w < w_end) blk = next_blk(blk, w);
      }
      if (kWarpIssue) __syncwarp();
      if (*abort_flag && lane == 0) {  // wait (bounded) for every MMA issued by this warp before TMEM is freed
        umma_commit(bar(DRAIN + h));
        mbar_wait_quiet(bar(DRAIN + h), 0);
      }
    }
  } else if (warp >= 4) {
    // ===================== soft-max warpgroups =====================
    const int wg = (warp - 4) >> 2;      // warpgroup index
    const int h = wg / kParts;           // 128-row half
    const int part = wg % kParts;        // which half of each tile's chunks
    const int q = warp & 3;              // TMEM lane quarter this warp may read
    const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
    // (the soft-max warps set `sub` with blk_of(w_begin) below, before the first chunk is consumed)
    if (has_work) blk_of(w_begin);
    float scale = SP().scale2;  // logit scale of the current segment's pass
    // off_run is the fp32 exponent offset all terms of s_run are relative to: sum = s_run * 2^off_run.
    // It is carried as the ROUNDED value scale*max (not recomputed from the max), so that rescaling by
    // 2^(off_old - off_new) and the final off_run + log2(s_run) are exact identities in fp32.
    float m_run = kRunInit, off_run = __fmul_rn(scale, kRunInit), s_run = 0.f;
    int idx_run = 0;   // AM: column of the running maximum m_run
    int col_tile = CSR ? 0 : w_begin % p.ntiles;  // AM: column tile of the chunk being consumed
    bool ok = true;
    constexpr int CH = BN / 32 / kParts;  // 32-column chunks of a tile owned by this warpgroup
    const int total = (w_end - w_begin) * CH;  // chunks of all segments; g / CH counts the CTA's tiles
    const int c_base = part * CH;
    // One online-softmax update with the 32 scores of a chunk (this thread's row).
    auto consume = [&](const uint32_t (&r)[32], int chunk_in_tile) {
      float v[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
      float t[11];
#pragma unroll
      for (int i = 0; i < 10; ++i) t[i] = max3(v[3 * i], v[3 * i + 1], v[3 * i + 2]);
      t[10] = fmaxf(v[30], v[31]);
      float u0 = max3(t[0], t[1], t[2]), u1 = max3(t[3], t[4], t[5]), u2 = max3(t[6], t[7], t[8]);
      float cm = fmaxf(max3(u0, u1, u2), fmaxf(t[9], t[10]));
      if (AM) {
        // Columns are visited in increasing order by this thread, so a later column only replaces the
        // running maximum when strictly larger; inside the chunk the smallest index attaining cm wins.
        if (cm > m_run) {
          int bi = 31;
#pragma unroll
          for (int i = 30; i >= 0; --i) bi = (v[i] == cm) ? i : bi;
          m_run = cm;
          idx_run = col_tile * BN + (c_base + chunk_in_tile) * 32 + bi;
        }
        return;
      }
      const float m_new = fmaxf(m_run, cm);
      // __fmul_rn: must not be contracted into an FMA with the subtraction below (the residual of the
      // product would leak into the exponent; with the huge init/mask magnitudes it even overflows).
      const float off_new = __fmul_rn(scale, m_new);
      const float nms = -off_new;
      // After the first tiles the running max rarely moves; when it moved for no row of the warp the
      // rescale factor is exactly 2^0 and its ex2 (one slot of the saturated pipe in 33) is skipped.
      float s0 = s_run, s1 = 0.f, s2 = 0.f, s3 = 0.f;
      if (__any_sync(0xffffffffu, off_new != off_run)) s0 *= ex2(off_run - off_new);
#pragma unroll
      for (int i = 0; i < 32; i += 4) {
        s0 += ex2(fmaf(v[i], scale, nms));
        s1 += ex2(fmaf(v[i + 1], scale, nms));
        s2 += ex2(fmaf(v[i + 2], scale, nms));
        s3 += ex2(fmaf(v[i + 3], scale, nms));
      }
      s_run = (s0 + s1) + (s2 + s3);
      m_run = m_new;
      off_run = off_new;
    };
    // Issue the TMEM load of chunk g (first waits for its tile if g starts one). No wait for the data.
    auto issue = [&](int g, uint32_t (&r)[32]) -> bool {
      const int j = g / CH, c = g % CH;
      const int buf = j & 1;
      if (c == 0) {
        if (!mbar_wait(bar(S_FULL + h * 2 + buf), (j >> 1) & 1, abort_flag)) return false;
        __syncwarp();  // lanes leave the poll loop at different times; tcgen05.ld is .sync.aligned
        tc_fence_after();
      }
      tmem_ld32_nowait(lane_addr + (uint32_t)((h * 2 + buf) * BN) + (c_base + c) * 32, r);
      return true;
    };
    // The load of chunk g has landed (tcgen05.wait::ld): if it was the last chunk of its tile,
    // hand the TMEM buffer back to the MMA warp.
    auto landed = [&](int g, uint32_t (&r)[32]) {
      tmem_ld_wait(r);
      if (g % CH == CH - 1) {
        const int j = g / CH;
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(S_EMPTY + h * 2 + (j & 1)));
      }
    };
    // Epilogue of a finished row: raw log2 normaliser and / or the damped, averaged potential update.
    auto store_lse = [&](int r, float lse2) {
      const LseEpilogue& ep = SP().ep;
      if (ep.lse2) ep.lse2[r] = lse2;
      if (ep.out) {
        float cand = -SP().eps * ep.damping * (lse2 * kLn2);
        float o = ep.w * cand;
        if (ep.old) o += (1.0f - ep.w) * ep.old[r];
        if (ep.shift) o -= ep.shiftcoef * ep.shift[r];
        if (ep.addvec) o += ep.addcoef * ep.addvec[r];
        ep.out[r] = o;
      }
    };
    // A row block without any kept tile is visited by no item: its rows get the empty soft-min (log-sum of
    // nothing = -inf), written by the CTAs in turn before they start on their items.
    if (CSR && part == 0) {
#pragma unroll 1
      for (int b = blockIdx.x; b < p.nblk; b += gridDim.x) {
        const int r = SP().row_begin + b * BM + h * 128 + q * 32 + lane;
        if (row_end(b) == row_start(b) && r < SP().nr) store_lse(r, -INFINITY);
      }
    }
    // End of a segment (the part of one row block this CTA covers): merge the two column parts, then either
    // finish the rows (the block is ours alone) or publish the (offset, sum) pair per row; the CTA that
    // publishes last (ticket counter per row block) merges all pairs in piece order - the result does not
    // depend on which CTA that is - and applies the epilogue. Every soft-max warp runs the same barrier
    // sequence for every segment, also after an abort (live = false), so the named barriers always match.
    auto finalize = [&](int blk, bool live) {
      const int r = SP().row_begin + blk * BM + h * 128 + q * 32 + lane;
      // AM: a partial is (maximum, column); the larger maximum wins, equal maxima keep the smaller column.
      auto better = [](float va, int ia, float vb, int ib) { return vb > va || (vb == va && ib < ia); };
      if (part == 1) {  // second column part parks its partial in shared memory
        merge_off[h * 128 + q * 32 + lane] = live ? (AM ? m_run : off_run) : kRunInit;
        merge_sum[h * 128 + q * 32 + lane] = AM ? __int_as_float(idx_run) : (live ? s_run : 0.f);
      }
      asm volatile("bar.sync 1, %0;" ::"n"(128 * NHALF * kParts) : "memory");  // soft-max warps only
      if (part == 0) {
        const float o2 = merge_off[h * 128 + q * 32 + lane], s2 = merge_sum[h * 128 + q * 32 + lane];
        if (AM) {
          if (better(m_run, idx_run, o2, __float_as_int(s2))) { m_run = o2; idx_run = __float_as_int(s2); }
        } else {
          const float on = fmaxf(off_run, o2);
          s_run = s_run * ex2(off_run - on) + s2 * ex2(o2 - on);
          off_run = on;
        }
      }
      const int c_lo = cta_of(row_start(blk)), c_hi = cta_of(row_end(blk) - 1);
      const int pieces = c_hi - c_lo + 1, piece = (int)blockIdx.x - c_lo;
      bool finish = pieces == 1;
      if (pieces > 1) {
        if (live && part == 0 && r < SP().nr) {
          SP().part_m[(size_t)piece * SP().part_stride + r] = AM ? m_run : off_run;
          SP().part_s[(size_t)piece * SP().part_stride + r] = AM ? __int_as_float(idx_run) : s_run;
        }
        __threadfence();  // the pairs must be visible device-wide before the ticket is taken
        asm volatile("bar.sync 1, %0;" ::"n"(128 * NHALF * kParts) : "memory");
        if (warp == 4 && lane == 0) *last_flag = (atomicAdd(SP().tickets + blk, 1) == pieces - 1) ? 1 : 0;
        asm volatile("bar.sync 1, %0;" ::"n"(128 * NHALF * kParts) : "memory");
        finish = *last_flag != 0;
        if (finish) {
          __threadfence();
          if (part == 0 && r < SP().nr) {
            float M = __ldcg(SP().part_m + r);
            if (AM) {
              int I = __float_as_int(__ldcg(SP().part_s + r));
              for (int c = 1; c < pieces; ++c) {
                const float vc = __ldcg(SP().part_m + (size_t)c * SP().part_stride + r);
                const int ic = __float_as_int(__ldcg(SP().part_s + (size_t)c * SP().part_stride + r));
                if (better(M, I, vc, ic)) { M = vc; I = ic; }
              }
              m_run = M;
              idx_run = I;
            } else {
              for (int c = 1; c < pieces; ++c) M = fmaxf(M, __ldcg(SP().part_m + (size_t)c * SP().part_stride + r));
              float S = 0.f;
              for (int c = 0; c < pieces; ++c)
                S += __ldcg(SP().part_s + (size_t)c * SP().part_stride + r) *
                     ex2(__ldcg(SP().part_m + (size_t)c * SP().part_stride + r) - M);
              off_run = M;
              s_run = S;
            }
          }
          if (warp == 4 && lane == 0) SP().tickets[blk] = 0;  // ready for the next launch on this stream
        }
      }
      if (AM) {
        if (finish && live && part == 0 && r < SP().nr && !*abort_flag) {
          SP().ep.out[r] = SP().scale2 * m_run;  // scale2 = -2*cost_scale turns the maximal score into the minimal cost
          SP().out_idx[r] = idx_run;
        }
      } else if (finish && live && part == 0 && r < SP().nr && !*abort_flag) {
        store_lse(r, off_run + log2f(fmaxf(s_run, 1e-40f)));
      }
      // merge_off / merge_sum / last_flag are re-used by the next segment
      asm volatile("bar.sync 1, %0;" ::"n"(128 * NHALF * kParts) : "memory");
      m_run = kRunInit;
      off_run = __fmul_rn(scale, kRunInit);
      s_run = 0.f;
      idx_run = 0;
    };
    // Segment bookkeeping: seg_w = first item of the current segment, seg_end_g = its last chunk + 1.
    int seg_w = w_begin, seg_blk = has_work ? blk_of(w_begin) : 0;
    auto seg_len = [&]() { return (row_end(seg_blk) < w_end ? row_end(seg_blk) : w_end) - seg_w; };
    auto next_seg = [&]() {  // step to the segment after the current one (if any)
      seg_w += seg_len();
      if (seg_w < w_end) {
        seg_blk = next_blk(seg_blk, seg_w);
        if (NSUB > 1) {  // the next segment may belong to another pass, with its own logit scale
          scale = SP().scale2;
          off_run = __fmul_rn(scale, kRunInit);
        }
      }
    };
    int seg_end_g = has_work ? seg_len() * CH : 0;
    auto consumed = [&](int g) {  // chunk g has been folded in: close the segment if it was its last chunk
      if (AM && g % CH == CH - 1) ++col_tile;
      if (g + 1 == seg_end_g) {
        finalize(seg_blk, true);
        next_seg();
        if (seg_w < w_end) seg_end_g += seg_len() * CH;
        if (AM) col_tile = 0;  // every later segment starts a new row block at column 0
      }
    };
    // Software pipeline, two register buffers: the load of chunk g+1 is in flight while chunk g is consumed
    // (also across a segment boundary: the next row block's first scores load during the finalisation).
    uint32_t ra[32], rb[32];
    ok = total > 0 && issue(0, ra);
#pragma unroll 1
    for (int g = 0; ok && g < total; g += 2) {
      landed(g, ra);
      if (g + 1 < total) {
        ok = issue(g + 1, rb);
        if (!ok) break;
      }
      consume(ra, g % CH);
      if (CH == 1) consumed(g);  // with two chunks per tile a segment can only end on the odd chunk
      if (g + 1 >= total) break;
      landed(g + 1, rb);
      if (g + 2 < total) {
        ok = issue(g + 2, ra);
        if (!ok) break;
      }
      consume(rb, (g + 1) % CH);
      consumed(g + 1);
    }
    // After an abort: keep the barrier sequence of the remaining segments (no data is written).
#pragma unroll 1
    while (seg_w < w_end) {
      finalize(seg_blk, false);
      next_seg();
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    __syncwarp();
    tmem_dealloc(tmem_base, kTmemCols);
  }
  if (tid == 0 && *abort_flag) atomicExch(&g_tc_error, 1);
}

// ------------------------------------------------------------------ plan-times-matrix kernel
// out = epilogue( sum_j 2^(logit_ij - R_i) * V_j ) with a known per-row offset R (the exact
// log2-normaliser from an LSE pass over the SAME staged operands, so the scores are
// bit-identical to the ones the potentials were fitted to). FlashAttention-style second GEMM:
//   MMA1 : S = A x B_tile^T           -> TMEM buffer (as in the LSE kernel)
//   warpgroup: W = 2^(scale*S - R), rounded to TF32, stored back over S with tcgen05.st
//   MMA2 : O += W x Vt_tile^T         (A operand from TMEM, B = V^T tile, K-major, in smem)
// No running max and no rescaling of O: R makes every W <= ~1. In SPLIT mode (exact fp32)
// W = Wh + Wl and V = Vh + Vl and MMA2 is issued three times (Wh.Vh + Wl.Vh + Wh.Vl).
// One CTA = 128 rows; TMEM columns: [0, 3*WCOLS) three S/W buffers, then DV_PAD columns of O.
struct PvKernelParams {
  int nr, nc, ntiles, nfull, ntail;
  int nb, nv;            // ring depths: column-operand tiles (freed after the score GEMM) and V tiles
  int row_begin;         // rows [row_begin, nr) are produced
  int dv, dv_pad, dv0;   // real width, padded slice width (multiple of 32, <= 128), first column of this slice
  int ld_out;            // row pitch of out (= full dv of the problem)
  float scale2, eps;
  const float* R;
  int epilogue;          // PvEpilogue
  const float* rowpot; const float* rowlogw; const float* roww; const float* gs; float coef;
  const float* rows_raw; int ld_rows;   // original row cloud (GRAD epilogue: x_i - O_i)
  float* out;
  const int* skip;       // device flag: non-zero => whole launch is a no-op
  // Column split: CTA b serves row block b / nsplit and the column tiles of share b % nsplit; with nsplit > 1
  // every CTA parks its raw O tile in `partial` ([row block][share][128][dv_pad]) and the one that takes
  // the last ticket of the row block adds the shares in share order and applies the epilogue.
  int nsplit;
  float* partial;
  int* tickets;
};


constexpr int kNSW = 3;  // S/W buffers of the plan-times-matrix kernel

template <int BN, bool SPLIT>
__global__ void __launch_bounds__(128 + 128 * kParts, 1)
tc_pv_kernel(const __grid_constant__ CUtensorMap mapA_full, const __grid_constant__ CUtensorMap mapA_tail,
             const __grid_constant__ CUtensorMap mapB_full, const __grid_constant__ CUtensorMap mapB_tail,
             const __grid_constant__ CUtensorMap mapV_hi, const __grid_constant__ CUtensorMap mapV_lo,
             const PvKernelParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int blk = (int)blockIdx.x / p.nsplit, share = (int)blockIdx.x % p.nsplit;
  const int row0 = p.row_begin + blk * 128;
  if (p.skip && *p.skip) return;  // uniform across the grid (set by an earlier kernel of the stream)
  constexpr int WCOLS = SPLIT ? 2 * BN : BN;  // TMEM columns per S/W buffer (Wl lives right after Wh)
  constexpr int NV = SPLIT ? 2 : 1;
  const int j0 = (int)((long long)share * p.ntiles / p.nsplit);
  const int ntl = (int)((long long)(share + 1) * p.ntiles / p.nsplit) - j0;  // column tiles of this CTA

  uint8_t* base = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t a_bytes = p.nfull * (128 * 128) + p.ntail * (128 * 32);
  const uint32_t b_bytes = p.nfull * (BN * 128) + p.ntail * (BN * 32);
  const uint32_t v_blk = (uint32_t)p.dv_pad * 128;        // one 32-column K block of V^T: dv_pad rows x 128 B
  const uint32_t v_bytes = (BN / 32) * v_blk;             // per hi/lo part
  const uint32_t v_stage = NV * v_bytes;
  uint8_t* a_smem = base;
  uint8_t* b_smem = a_smem + a_bytes;
  uint8_t* v_smem = b_smem + p.nb * b_bytes;
  uint64_t* bars = (uint64_t*)(v_smem + p.nv * v_stage);
  // Two independent rings: a column-operand tile is released as soon as its score GEMM retires, a V tile
  // only after the second GEMM, a whole soft-max later; sharing one ring would serialise TMA latency
  // behind the soft-max.
  const int B_FULL = 0, B_EMPTY = p.nb, V_FULL = 2 * p.nb, V_EMPTY = V_FULL + p.nv, S_FULL = V_EMPTY + p.nv,
            W_FULL = S_FULL + kNSW, W_FREE = W_FULL + kNSW, A_FULL = W_FREE + kNSW, O_FULL = A_FULL + 1,
            DRAIN = O_FULL + 1, NBARS = DRAIN + 1;
  uint32_t* tmem_slot = (uint32_t*)(bars + NBARS);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
  volatile int* last_flag = (volatile int*)(tmem_slot + 2);
  auto bar = [&](int i) { return smem_u32(bars + i); };
  constexpr uint32_t kTmemCols = 512;

  if (tid == 0) {
    for (int s = 0; s < p.nb; ++s) {
      mbar_init(bar(B_FULL + s), 1);
      mbar_init(bar(B_EMPTY + s), 1);
    }
    for (int s = 0; s < p.nv; ++s) {
      mbar_init(bar(V_FULL + s), 1);
      mbar_init(bar(V_EMPTY + s), 1);
    }
    for (int i = 0; i < kNSW; ++i) {
      mbar_init(bar(S_FULL + i), 1);
      mbar_init(bar(W_FULL + i), 4 * kParts);
      mbar_init(bar(W_FREE + i), 1);
    }
    mbar_init(bar(A_FULL), 1);
    mbar_init(bar(O_FULL), 1);
    mbar_init(bar(DRAIN), 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t o_tmem = tmem_base + kNSW * WCOLS;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(bar(A_FULL), a_bytes);
      uint32_t dst = smem_u32(a_smem);
      for (int kb = 0; kb < p.nfull; ++kb) tma_load_2d(dst + kb * (128 * 128), &mapA_full, kb * 32, row0, bar(A_FULL));
      for (int t = 0; t < p.ntail; ++t)
        tma_load_2d(dst + p.nfull * (128 * 128) + t * (128 * 32), &mapA_tail, p.nfull * 32 + t * 8, row0, bar(A_FULL));
      int issued = 0;
#pragma unroll 1
      for (int j = 0; j < ntl; ++j) {
        const int s = j % p.nb;
        const uint32_t ph = (j / p.nb) & 1;
        if (!mbar_wait(bar(B_EMPTY + s), ph ^ 1, abort_flag, 2000)) break;
        mbar_expect_tx(bar(B_FULL + s), b_bytes);
        uint32_t d0 = smem_u32(b_smem + s * b_bytes);
        for (int kb = 0; kb < p.nfull; ++kb)
          tma_load_2d(d0 + kb * (BN * 128), &mapB_full, kb * 32, (j0 + j) * BN, bar(B_FULL + s));
        for (int t = 0; t < p.ntail; ++t)
          tma_load_2d(d0 + p.nfull * (BN * 128) + t * (BN * 32), &mapB_tail, p.nfull * 32 + t * 8, (j0 + j) * BN,
                      bar(B_FULL + s));
        issued = j + 1;
      }
      if (*abort_flag) {
        mbar_wait_quiet(bar(A_FULL), 0);
        for (int j = (issued > p.nb ? issued - p.nb : 0); j < issued; ++j)
          mbar_wait_quiet(bar(B_FULL + j % p.nb), (j / p.nb) & 1);
      }
    }
  } else if (warp == 2) {
    if (lane == 0) {  // V^T tiles (hi and, in split mode, lo) on their own ring
      int issued = 0;
#pragma unroll 1
      for (int j = 0; j < ntl; ++j) {
        const int s = j % p.nv;
        const uint32_t ph = (j / p.nv) & 1;
        if (!mbar_wait(bar(V_EMPTY + s), ph ^ 1, abort_flag, 2000)) break;
        mbar_expect_tx(bar(V_FULL + s), v_stage);
        uint32_t dv_dst = smem_u32(v_smem + s * v_stage);
        for (int kb = 0; kb < BN / 32; ++kb) {
          tma_load_2d(dv_dst + kb * v_blk, &mapV_hi, (j0 + j) * BN + kb * 32, p.dv0, bar(V_FULL + s));
          if (SPLIT)
            tma_load_2d(dv_dst + v_bytes + kb * v_blk, &mapV_lo, (j0 + j) * BN + kb * 32, p.dv0, bar(V_FULL + s));
        }
        issued = j + 1;
      }
      if (*abort_flag) {
        for (int j = (issued > p.nv ? issued - p.nv : 0); j < issued; ++j)
          mbar_wait_quiet(bar(V_FULL + j % p.nv), (j / p.nv) & 1);
      }
    }
  } else if (warp == 1) {
    // Score GEMM S_j = A . B_j^T into S/W buffer j%3, issued from this warp, the second GEMM from another:
    // one stream sharing its scheduler with soft-max warps sustains one MMA per ~90 cycles, and the 9 + 16
    // instructions of a tile would otherwise queue behind each other. All 32 lanes run the loop (uniform
    // descriptor arithmetic), one elected lane issues.
    {
      constexpr uint32_t idesc1 = make_idesc(BN);
      // every exit decision is a warp vote: elect.sync needs all 32 lanes at the same instruction
      const bool ok = __all_sync(0xffffffffu, mbar_wait(bar(A_FULL), 0, abort_flag, 2000));
      tc_fence_after();
      const uint32_t a_lo0 = desc_lo(smem_u32(a_smem));
#pragma unroll 1
      for (int j = 0; ok && j < ntl; ++j) {
        const int s = j % p.nb, buf = j % kNSW;
        if (!__all_sync(0xffffffffu, mbar_wait(bar(W_FREE + buf), ((j / kNSW) & 1) ^ 1, abort_flag, 2000))) break;
        if (!__all_sync(0xffffffffu, mbar_wait(bar(B_FULL + s), (j / p.nb) & 1, abort_flag, 2000))) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * WCOLS;
        uint32_t al = a_lo0, bl = desc_lo(smem_u32(b_smem + s * b_bytes));
        if (elect_one()) {  // one election per tile
          uint32_t acc = 0;
#pragma unroll 1
          for (int kb = 0; kb < p.nfull; ++kb) {
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
              umma_tf32(d_tmem, pack_desc(al + 2 * ks, kDescHi128), pack_desc(bl + 2 * ks, kDescHi128), idesc1, acc);
              acc = 1;
            }
            al += (128 * 128) >> 4;
            bl += (BN * 128) >> 4;
          }
#pragma unroll 1
          for (int t = 0; t < p.ntail; ++t) {
            umma_tf32(d_tmem, pack_desc(al, kDescHi32), pack_desc(bl, kDescHi32), idesc1, acc);
            acc = 1;
            al += (128 * 32) >> 4;
            bl += (BN * 32) >> 4;
          }
          umma_commit(bar(S_FULL + buf));
          umma_commit(bar(B_EMPTY + s));
        }
        __syncwarp();
      }
      __syncwarp();
      if (*abort_flag && lane == 0) {  // let every MMA issued by this warp retire before TMEM is freed
        umma_commit(bar(DRAIN));
        mbar_wait_quiet(bar(DRAIN), 0);
      }
    }
  } else if (warp == 3) {
    // Second GEMM O += W_j . V_j (W read from TMEM), once the soft-max warps have written W_j.
    {
      const uint32_t idesc2 = make_idesc(p.dv_pad);
      const uint32_t v_blk_units = v_blk >> 4;
      uint32_t o_acc = 0;
#pragma unroll 1
      for (int j = 0; j < ntl; ++j) {
        const int sv = j % p.nv, buf = j % kNSW;
        if (!__all_sync(0xffffffffu, mbar_wait(bar(V_FULL + sv), (j / p.nv) & 1, abort_flag, 2000))) break;
        if (!__all_sync(0xffffffffu, mbar_wait(bar(W_FULL + buf), (j / kNSW) & 1, abort_flag, 2000))) break;
        tc_fence_after();
        const uint32_t w_tmem = tmem_base + buf * WCOLS;
        const uint32_t v_lo0 = desc_lo(smem_u32(v_smem + sv * v_stage));
        if (elect_one()) {  // one election per tile
          uint32_t acc2 = o_acc;
#pragma unroll 1
          for (int part = 0; part < (SPLIT ? 3 : 1); ++part) {
            // part 0: Wh.Vh   part 1: Wl.Vh   part 2: Wh.Vl
            uint32_t wa = w_tmem + ((part == 1) ? BN : 0);
            uint32_t vl = v_lo0 + ((part == 2) ? (v_bytes >> 4) : 0);
#pragma unroll 1
            for (int kb = 0; kb < BN / 32; ++kb) {
#pragma unroll
              for (int ks = 0; ks < 4; ++ks) {
                umma_tf32_ts(o_tmem, wa + ks * 8, pack_desc(vl + 2 * ks, kDescHi128), idesc2, acc2);
                acc2 = 1;
              }
              wa += 32;
              vl += v_blk_units;
            }
          }
          umma_commit(bar(V_EMPTY + sv));
          umma_commit(bar(W_FREE + buf));
        }
        o_acc = 1;
        __syncwarp();
      }
      __syncwarp();
      if (lane == 0) {
        umma_commit(bar(O_FULL));
        if (*abort_flag) mbar_wait_quiet(bar(O_FULL), 0);
      }
    }
  } else if (warp >= 4) {
    // Two warpgroups share the 128 rows: each takes half of every tile's 32-column chunks.
    const int part = (warp - 4) >> 2;
    const int q = warp & 3;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
    const int r_in = q * 32 + lane;  // row within the block
    const int r = row0 + r_in;
    const float scale = p.scale2;
    const float negR = (r < p.nr) ? -p.R[r] : 0.f;
    bool ok = true;
    constexpr int CH = BN / 32 / kParts;
    const int total = ntl * CH;
    const int c_base = part * CH;
    auto issue = [&](int g, uint32_t (&rg)[32]) -> bool {
      const int j = g / CH, c = g % CH, buf = j % kNSW;
      if (c == 0) {
        if (!mbar_wait(bar(S_FULL + buf), (j / kNSW) & 1, abort_flag)) return false;
        __syncwarp();
        tc_fence_after();
      }
      tmem_ld32_nowait(lane_addr + buf * WCOLS + (c_base + c) * 32, rg);
      return true;
    };
    // Scores of chunk g have landed in rg: turn them into weights, store them back over the scores.
    auto weigh = [&](int g, uint32_t (&rg)[32]) {
      const int j = g / CH, c = g % CH, buf = j % kNSW;
      const uint32_t taddr = lane_addr + buf * WCOLS + (c_base + c) * 32;
      float v[32];
      if (SPLIT) {
        float lo[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float w = ex2(fmaf(__uint_as_float(rg[i]), scale, negR));
          float hi = round_tf32_pos(w);
          lo[i] = round_tf32_pos(w - hi);
          v[i] = hi;
        }
        tmem_st32(taddr + BN, lo);
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = round_tf32_pos(ex2(fmaf(__uint_as_float(rg[i]), scale, negR)));
      }
      tmem_st32(taddr, v);
      if (c == CH - 1) {  // this warp's share of the tile is written: tell the MMA lane
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(W_FULL + buf));
      }
    };
    // One pipeline step: chunk g is in `cur`; the load of chunk g+1 goes to `nxt`. Within a tile the next
    // load is issued before the arithmetic; across tiles only after W_FULL was signalled, so that a warp
    // never sits on the next tile's barrier while the MMA lane waits for its share of this one.
    auto pipe = [&](int g, uint32_t (&cur)[32], uint32_t (&nxt)[32]) -> bool {
      tmem_ld_wait(cur);
      const bool last = (g % CH) == CH - 1;
      const bool more = g + 1 < total;
      if (!last && more && !issue(g + 1, nxt)) return false;
      weigh(g, cur);
      if (last && more && !issue(g + 1, nxt)) return false;
      return true;
    };
    uint32_t ra[32], rb[32];
    ok = total > 0 && issue(0, ra);
#pragma unroll 1
    for (int g = 0; ok && g < total; g += 2) {
      ok = pipe(g, ra, rb);
      if (!ok || g + 1 >= total) break;
      ok = pipe(g + 1, rb, ra);
    }
    if (ok) ok = mbar_wait(bar(O_FULL), 0, abort_flag);
    __syncwarp();
    tc_fence_after();
    // `ok` is warp-uniform (every lane polls the same barrier). tcgen05.ld is .sync.aligned: all 32
    // lanes must execute it together, so rows beyond nr load too and only their stores are masked.
    const float inv_eps = 1.0f / p.eps;
    // Epilogue of one output row: o = sum_j w_ij V_j over ALL columns.
    auto finish_row = [&](int rr, int c, const float (&o)[32], float fac) {
      float* orow = p.out + (size_t)rr * p.ld_out + p.dv0;
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        int col = c * 32 + i;
        if (p.dv0 + col < p.dv) {
          float val = o[i];
          if (p.epilogue == PV_GRAD) val = __ldg(p.rows_raw + (size_t)rr * p.ld_rows + p.dv0 + col) - val;
          orow[col] = fac * val;
        }
      }
    };
    auto row_factor = [&](int rr) {
      if (p.epilogue == PV_GRAD) return p.coef * (p.gs ? __ldg(p.gs) : 1.f) * __ldg(p.roww + rr);
      // Rounding written out (the compiler's choice of fused multiply-adds here moved a CG-bound result by 1e-3).
      const float pot = __ldg(p.rowpot + rr), lw = (p.rowlogw ? __ldg(p.rowlogw + rr) : 0.f);
      const float t = __fadd_rn(__fmul_rn(pot, inv_eps), lw);
      return __fmul_rn(p.coef, ex2(__fmaf_rn(t, kLog2e, -negR)));
    };
    const size_t tile_elems = (size_t)128 * p.dv_pad;
    const bool valid = r < p.nr;
    const int rr = valid ? r : 0;
    if (ok) {
      const float fac = (p.nsplit == 1) ? row_factor(rr) : 0.f;
      float* my_partial = p.nsplit > 1 ? p.partial + ((size_t)blk * p.nsplit + share) * tile_elems : nullptr;
#pragma unroll 1
      for (int c = part; c < p.dv_pad / 32; c += kParts) {  // the warpgroups split the output chunks
        float o[32];
        tmem_ld32(lane_addr + kNSW * WCOLS + c * 32, o);
        if (p.nsplit == 1) {
          if (valid) finish_row(rr, c, o, fac);
        } else {  // raw share of the row, merged below
          float4* dst = reinterpret_cast<float4*>(my_partial + (size_t)r_in * p.dv_pad + c * 32);
#pragma unroll
          for (int i = 0; i < 8; ++i) dst[i] = make_float4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
        }
      }
    }
    if (p.nsplit > 1) {
      // Every soft-max warp runs this barrier sequence, also after an abort; what happens between the barriers
      // is decided by one thread and read back from shared memory, so it is the same for all of them.
      __threadfence();  // the shares must be visible device-wide before the ticket is taken
      asm volatile("bar.sync 1, %0;" ::"n"(128 * kParts) : "memory");
      if (warp == 4 && lane == 0)
        *last_flag = (!*abort_flag && atomicAdd(p.tickets + blk, 1) == p.nsplit - 1) ? 1 : 0;
      asm volatile("bar.sync 1, %0;" ::"n"(128 * kParts) : "memory");
      if (*last_flag) {
        __threadfence();
        if (valid) {
          const float* blk_partial = p.partial + (size_t)blk * p.nsplit * tile_elems;
          const float fac = row_factor(r);
#pragma unroll 1
          for (int c = part; c < p.dv_pad / 32; c += kParts) {
            float o[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = 0.f;
            for (int sh = 0; sh < p.nsplit; ++sh) {  // fixed order: the sum does not depend on who merges
              const float4* src =
                  reinterpret_cast<const float4*>(blk_partial + (size_t)sh * tile_elems + (size_t)r_in * p.dv_pad + c * 32);
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const float4 t = __ldcg(src + i);
                o[4 * i] += t.x; o[4 * i + 1] += t.y; o[4 * i + 2] += t.z; o[4 * i + 3] += t.w;
              }
            }
            finish_row(r, c, o, fac);
          }
        }
        if (warp == 4 && lane == 0) p.tickets[blk] = 0;  // ready for the next launch on this stream
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    __syncwarp();
    tmem_dealloc(tmem_base, kTmemCols);
  }
  if (tid == 0 && *abort_flag) atomicExch(&g_tc_error, 1);
}

// V^T staging: vt[c][j] = tf32(V[j][c] * colscale_j) (hi) and the tf32 residual (lo), zero padded
// to [dv_rows_pad, cols_pad]. One thread per output element, reads along j are strided by dv
// (the matrices involved are O((n+m) d), negligible next to the n*m pass).
__global__ void stage_vt_kernel(const float* __restrict__ V, int nc, int dv, const float* __restrict__ colscale,
                                int rows_pad, int cols_pad, float* __restrict__ vt_hi, float* __restrict__ vt_lo) {
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  size_t total = (size_t)rows_pad * cols_pad;
  if (idx >= total) return;
  int c = (int)(idx / cols_pad), j = (int)(idx % cols_pad);
  float v = 0.f;
  if (c < dv && j < nc) {
    v = V[(size_t)j * dv + c];
    if (colscale) v *= colscale[j];
  }
  float hi = to_tf32(v);
  vt_hi[idx] = hi;
  if (vt_lo) vt_lo[idx] = to_tf32(v - hi);
}

// ------------------------------------------------------------------ staging kernels
// opA/opB for one cloud. Column layout (kp floats per row):
//   TF32 mode : [ x (d) | aug (3) | 0 ... ]                       A-role aug = 1,1,1 ; B-role aug = bias split
//   FP32 mode : A-role [ xh (d) | xh (d) | xl (d) | aug | 0 ...]   B-role [ yh | yl | yh | aug | 0 ... ]
// so that sum_k A_k B_k = xh.yh + xh.yl + xl.yh + bias  (the dropped xl.yl term is ~2^-22 relative).
// Label cost: the coordinate columns are followed by 3V label columns per point, so that the table lookup
// becomes part of the same contraction: in the row role a point of label l carries (1,1,1) in the three
// columns of class l and zeros elsewhere; in the column role it carries, for every class v, the three-piece
// TF32 split of w_coef * W[.,.] between v and its own label (exact in fp32, so the block is staged once in
// either precision mode).
__global__ void stage_kernel(const float* __restrict__ src, int rows, int rows_pad, int d, int kc, int kp, int prec,
                             float* __restrict__ opA, float* __restrict__ opB,
                             const int* __restrict__ labels, const float* __restrict__ W, int V, int cloud,
                             float w_coef) {
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  size_t total = (size_t)rows_pad * kp;
  if (idx >= total) return;
  int r = (int)(idx / kp), k = (int)(idx % kp);
  const int kcoord = (prec == 0) ? d : 3 * d;  // coordinate columns; [kcoord, kc) is the label block
  float va = 0.f, vb = 0.f;
  if (k < kcoord) {
    if (r < rows) {
      int part = k / d, c = k % d;
      float x = src[(size_t)r * d + c];
      float hi = to_tf32(x);
      float lo = to_tf32(x - hi);
      if (prec == 0) { va = hi; vb = hi; }
      else { va = (part == 2) ? lo : hi; vb = (part == 1) ? lo : hi; }
    }
  } else if (k < kc) {
    if (r < rows) {
      const int v = (k - kcoord) / 3, piece = (k - kcoord) % 3;
      const int l = labels[r];
      va = (l == v) ? 1.f : 0.f;
      // cloud 0 (x) as column: rows are y points of label v -> W[l, v]; cloud 1 (y) as column: W[v, l]
      const float w = w_coef * W[cloud == 0 ? l * V + v : v * V + l];
      const float h = to_tf32(w), mid = to_tf32(w - h), low = to_tf32(w - h - mid);
      vb = piece == 0 ? h : (piece == 1 ? mid : low);
    }
  } else if (k < kc + 3) {
    va = 1.f;
    vb = (k == kc && r >= rows) ? kMaskBias : 0.f;  // padded rows are masked for good
  }
  opA[idx] = va;
  opB[idx] = vb;
}

// Writes the bias of a pass, divided by the logit scale and split into 3 TF32 pieces, into opB's aug columns.
__global__ void bias_kernel(float* __restrict__ opB, int rows, int kc, int kp, const float* __restrict__ pot,
                            const float* __restrict__ logw, float inv_eps, float inv_scale2, const Ctrl* ctrl,
                            int pot_shard = 0, int pot_stride = 0) {
  if (ctrl && ctrl->converged) return;
  int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  const float pr = pot_shard > 0 ? pot[(size_t)(r / pot_shard) * pot_stride + r % pot_shard] : pot[r];
  // bias in log2 units, same association as the reference kernels, then / scale2
  float b2 = logw ? (pr * (inv_eps * kLog2e) + logw[r] * kLog2e) : pr * kLog2e;
  float b = b2 * inv_scale2;
  float hi = to_tf32(b);
  float r1 = b - hi;
  float mid = to_tf32(r1);
  float lo = to_tf32(r1 - mid);
  float* row = opB + (size_t)r * kp + kc;
  row[0] = hi; row[1] = mid; row[2] = lo;
}

// ------------------------------------------------------------------ host side
PFN_cuTensorMapEncodeTiled_v12000 get_encode() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(sym);
  });
  return fn;
}

bool encode_map(CUtensorMap* map, const float* base, int rows, int kp, int box_k, int box_rows,
                CUtensorMapSwizzle swz) {
  return detail::encode_map(map, base, rows, kp, box_k, box_rows, swz);
}

struct Shape {
  int kc, kp, nfull, ntail, nhalf, bn, nstage;
  size_t smem;
  bool ok;
  bool streamed;  // the row operand does not fit in shared memory: K-streamed kernels (fs_tck.cu) take the pass
};

// nlab = label-table columns (3 per class), staged once in either precision mode: their values are exact in TF32.
Shape plan_shape(int d, int prec, int nlab = 0) {
  Shape s{};
  s.kc = ((prec == 0) ? d : 3 * d) + nlab;
  s.kp = (s.kc + 3 + 7) & ~7;  // + 3 bias columns, padded to whole K steps of 8
  s.nfull = s.kp / 32;
  s.ntail = (s.kp % 32) / 8;
  const size_t row_bytes = (size_t)s.kp * 4;
  const size_t budget = kSmemMax - 4096;  // barriers, merge buffers, alignment slack
  s.ok = false;
  const int cand[3][2] = {{2, 128}, {1, 128}, {1, 64}};
  for (auto& c : cand) {
    size_t a = (size_t)c[0] * 128 * row_bytes, b = (size_t)c[1] * row_bytes;
    if (a + 2 * b > budget) continue;
    int ns = (int)((budget - a) / b);
    if (ns > 4) ns = 4;
    s.nhalf = c[0]; s.bn = c[1]; s.nstage = ns;
    s.smem = a + ns * b + 4096;
    if (s.smem < (size_t)kSmemMin) s.smem = kSmemMin;
    s.ok = true;
    break;
  }
  if (!s.ok) {  // any K: both operands stream through shared memory in K chunks
    s.ok = true;
    s.streamed = true;
  }
  return s;
}

// Tile lists are over 128 x 128 tiles: one 128-row half per CTA, 128-column tiles.
Shape plan_shape_csr(int d, int prec, int nlab) {
  Shape s = plan_shape(d, prec, nlab);
  if (!s.ok || s.streamed) { s.ok = false; return s; }
  const size_t row_bytes = (size_t)s.kp * 4, budget = kSmemMax - 4096;
  const size_t a = 128 * row_bytes, b = 128 * row_bytes;
  if (a + 2 * b > budget) { s.ok = false; return s; }
  int ns = (int)((budget - a) / b);
  if (ns > 4) ns = 4;
  s.nhalf = 1; s.bn = 128; s.nstage = ns;
  s.smem = a + ns * b + 4096;
  if (s.smem < (size_t)kSmemMin) s.smem = kSmemMin;
  return s;
}

template <int NHALF, int BN, bool AM, bool CSR = false, int NSUB = 1>
cudaError_t launch(const Launch<NSUB>& lp, dim3 grid, size_t smem, cudaStream_t st) {
  auto kern = tc_lse_kernel<NHALF, BN, AM, CSR, NSUB>;
  // Per device (context) attribute; cheap enough to set on every launch.
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemMax);
  if (e != cudaSuccess) return e;
  kern<<<grid, 128 + 128 * NHALF * kParts, smem, st>>>(lp);
  return cudaGetLastError();
}

// Bias columns of up to kMaxSub column operands in one launch (blockIdx.y = job).
struct BiasJobs {
  struct Job {
    float* opB;
    int rows, kc, kp;
    const float* pot;
    const float* logw;
    float inv_eps, inv_scale2;
    int pot_shard, pot_stride;  // packed potential (see StreamArgs), 0 = contiguous
  } job[kMaxSub];
};

__global__ void bias_multi_kernel(const BiasJobs jobs) {
  const BiasJobs::Job& j = jobs.job[blockIdx.y];
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= j.rows) return;
  const float pr = j.pot_shard > 0 ? j.pot[(size_t)(r / j.pot_shard) * j.pot_stride + r % j.pot_shard] : j.pot[r];
  const float b2 = j.logw ? (pr * (j.inv_eps * kLog2e) + j.logw[r] * kLog2e) : pr * kLog2e;
  const float b = b2 * j.inv_scale2;
  const float hi = to_tf32(b);
  const float r1 = b - hi;
  const float mid = to_tf32(r1);
  const float lo = to_tf32(r1 - mid);
  float* row = j.opB + (size_t)r * j.kp + j.kc;
  row[0] = hi; row[1] = mid; row[2] = lo;
}

constexpr int kMaxChunks = 16;

std::atomic<int> g_reserved_sms{0};
std::atomic<int> g_cta_limit{0};
std::atomic<int> g_prefer_streamed{1};
std::atomic<int> g_pv_split{0};  // column shares per row block of the matrix pass. 0: chosen by SM fill, 1..8: forced

}  // namespace

namespace detail {

// 2-D fp32 tensor [rows, kp] (kp contiguous), box = [box_k floats, box_rows rows].
bool encode_map(CUtensorMap* map, const float* base, long long rows, long long kp, int box_k, int box_rows,
                CUtensorMapSwizzle swz, long long row_pitch) {
  auto enc = get_encode();
  if (!enc) return false;
  cuuint64_t dims[2] = {(cuuint64_t)kp, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)(row_pitch > 0 ? row_pitch : kp) * sizeof(float)};
  cuuint32_t box[2] = {(cuuint32_t)box_k, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// SMs of the current device (cached per device index; 148 on B200).
int sm_count() {
  static std::atomic<int> cache[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  int v = cache[dev].load(std::memory_order_relaxed);
  if (v > 0) return v;
  if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) return 148;
  cache[dev].store(v, std::memory_order_relaxed);
  return v;
}

// CTAs of a streaming pass. The nblk*ntiles (row block, column tile) items are cut into equal contiguous
// ranges, one per CTA: a single wave of at most one CTA per SM, at least ~4 tiles each, and no row block
// shared by more than kMaxChunks CTAs (that many partial slots exist per row).
int pick_ctas_for(int nblk, int ntiles, int sms, int reserved, int limit) {
  const long long total = (long long)nblk * ntiles;
  // SMs left free on request (a collective running next to the pass needs a few: a CTA of this kernel
  // fills its SM, and one that has to wait for the collective to leave delays the whole single wave).
  long long g = sms - reserved;
  if (g < 1) g = 1;
  if (limit >= 1 && limit < g) g = limit;
  if (g > (total + 3) / 4) g = (total + 3) / 4;
  if (g > total) g = total;
  if (g < 1) g = 1;
  auto first = [&](long long c) { return (total * c) / g; };
  auto owner = [&](long long t) {
    long long c = (t * g) / total;
    while (c + 1 < g && first(c + 1) <= t) ++c;
    while (c > 0 && first(c) > t) --c;
    return c;
  };
  for (; g > 1; --g) {
    long long worst = 1;
    for (int b = 0; b < nblk && worst <= kMaxChunks; ++b) {
      long long pieces = owner((long long)(b + 1) * ntiles - 1) - owner((long long)b * ntiles) + 1;
      if (pieces > worst) worst = pieces;
    }
    if (worst <= kMaxChunks) break;
  }
  return (int)g;
}

void launch_bias(const CloudOps& colc, int kc, int kp, const float* pot, const float* logw, float inv_eps,
                 float inv_scale2, const Ctrl* ctrl, cudaStream_t st, int pot_shard, int pot_stride) {
  bias_kernel<<<(colc.rows + 255) / 256, 256, 0, st>>>(colc.opB, colc.rows, kc, kp, pot, logw, inv_eps, inv_scale2,
                                                       ctrl, pot_shard, pot_stride);
}

int pick_ctas(int nblk, int ntiles) {
  return pick_ctas_for(nblk, ntiles, sm_count(), g_reserved_sms.load(std::memory_order_relaxed),
                       g_cta_limit.load(std::memory_order_relaxed));
}

}  // namespace detail

namespace {
using detail::pick_ctas;
}  // namespace

int set_reserved_sms(int k) {
  const int sms = detail::sm_count();
  if (k < 0) k = 0;
  if (k > sms - 1) k = sms - 1;
  return g_reserved_sms.exchange(k, std::memory_order_relaxed);
}

int set_cta_limit(int k) {
  if (k < 0) k = 0;
  return g_cta_limit.exchange(k, std::memory_order_relaxed);
}

int set_prefer_streamed(int on) { return g_prefer_streamed.exchange(on ? 1 : 0, std::memory_order_relaxed); }

int set_pv_split(int split) {
  return g_pv_split.exchange(split >= 1 && split <= 8 ? split : 0, std::memory_order_relaxed);
}

int plan_ctas(int nblk, int ntiles, int sms, int reserved, int limit) {
  if (nblk <= 0 || ntiles <= 0 || sms <= 0) return 0;
  return detail::pick_ctas_for(nblk, ntiles, sms, reserved < 0 ? 0 : reserved, limit);
}

bool k_streamed(int d, int prec, int nlab) { return plan_shape(d, prec, nlab).streamed; }

size_t mat5_scratch_bytes(int nr, int nc, int d, int prec, int dv, int nlab) {
  const Shape sh = plan_shape(d, prec, nlab);
  if (!sh.ok || (prec != 0 && prec != 1)) return 0;
  const int nm = nr > nc ? nr : nc;
  return kstream_pv_scratch(nm, nm, sh.kp, dv, prec, true);
}

bool csr_supported(int d, int prec, int nlab) {
  return (prec == 0 || prec == 1) && plan_shape_csr(d, prec, nlab).ok;
}

bool supported(int n, int m, int d, int prec, int nlab) {
  if (prec != 0 && prec != 1) return false;
  if (n <= 0 || m <= 0 || d <= 0) return false;
  // The streaming kernel numbers its (row block, column tile) items with 32-bit integers: with 128-row
  // blocks and 64-column tiles (the smallest it uses) both orientations must stay below 2^31 items,
  // i.e. n*m below about 1.7e13. Larger problems go to the CUDA-core engine, which has no such product.
  const long long blocks_n = ((long long)n + 127) / 128, blocks_m = ((long long)m + 127) / 128;
  const long long tiles_n = ((long long)n + 63) / 64, tiles_m = ((long long)m + 63) / 64;
  if (blocks_n * tiles_m >= (1ll << 31) || blocks_m * tiles_n >= (1ll << 31)) return false;
  return plan_shape(d, prec, nlab).ok;
}

using detail::pad256;

size_t staged_bytes(int n, int m, int d, int prec, int nlab) {
  Shape s = plan_shape(d, prec, nlab);
  if (!s.ok) return 0;
  size_t per_row = (size_t)s.kp * sizeof(float);
  size_t b = 0;
  b += 2 * (((size_t)pad256(n) * per_row + 1023) & ~size_t(1023));
  b += 2 * (((size_t)pad256(m) * per_row + 1023) & ~size_t(1023));
  b += 2 * 2 * (size_t)kMaxChunks * pad256(n > m ? n : m) * sizeof(float);  // column-split partials, per side
  b += 2 * (size_t)(pad256(n > m ? n : m) / 128) * sizeof(int);             // row-block tickets, per side
  return b + 1024;
}

cudaError_t stage(Staged& s, char* buf, const float* x, const float* y, int n, int m, int d, int prec,
                  cudaStream_t st, bool run_kernels, const LabelCost* lab, float w_coef) {
  const int V = (lab && lab->V > 0) ? lab->V : 0;
  Shape sh = plan_shape(d, prec, 3 * V);  // the label table rides along as 3V extra columns (see stage_kernel)
  if (!sh.ok) return cudaErrorNotSupported;
  s.d = d; s.nlab = 3 * V; s.kc = sh.kc; s.kp = sh.kp; s.prec = prec;
  char* p = (char*)(((uintptr_t)buf + 1023) & ~(uintptr_t)1023);
  const float* src[2] = {x, y};
  const int rows[2] = {n, m};
  for (int c = 0; c < 2; ++c) {
    CloudOps& o = s.cloud[c];
    o.rows = rows[c];
    o.rows_pad = pad256(rows[c]);
    size_t bytes = (((size_t)o.rows_pad * sh.kp * sizeof(float)) + 1023) & ~size_t(1023);
    o.opA = reinterpret_cast<float*>(p); p += bytes;
    o.opB = reinterpret_cast<float*>(p); p += bytes;
    size_t total = (size_t)o.rows_pad * sh.kp;
    if (run_kernels)
      stage_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(src[c], o.rows, o.rows_pad, d, sh.kc, sh.kp, prec,
                                                                    o.opA, o.opB, V ? lab->lab[c] : nullptr,
                                                                    V ? lab->W : nullptr, V, c, w_coef);
  }
  s.part_stride = pad256(n > m ? n : m);
  // Each side has its own partial slots and tickets: the two passes of a Jacobi step may share one launch.
  const size_t slots = (size_t)kMaxChunks * s.part_stride;
  float* fp = reinterpret_cast<float*>(p);
  for (int sd = 0; sd < 2; ++sd) {
    s.part_m[sd] = fp + (2 * sd) * slots;
    s.part_s[sd] = fp + (2 * sd + 1) * slots;
  }
  int* tk = reinterpret_cast<int*>(fp + 4 * slots);
  s.tickets[0] = tk;
  s.tickets[1] = tk + s.part_stride / 128;
  if (run_kernels) {
    cudaError_t e = cudaMemsetAsync(tk, 0, 2 * (size_t)(s.part_stride / 128) * sizeof(int), st);
    if (e != cudaSuccess) return e;
  }
  return cudaGetLastError();
}

namespace {
// Tensor maps and geometry of one pass over staged operands (side 0: rows of x against y, side 1: the reverse).
// A boxes are 128 rows, B boxes BN rows; when a K-block class is absent its map still has to be a valid object:
// it is encoded over the first columns (never used by the kernel).
bool fill_subpass(SubPass& kp, const Staged& s, int side, const StreamArgs& a, const LseEpilogue& e, const Shape& sh,
                  float scale2) {
  const CloudOps& rowc = s.cloud[side == 0 ? 0 : 1];
  const CloudOps& colc = s.cloud[side == 0 ? 1 : 0];
  bool ok = true;
  ok &= encode_map(&kp.mapA_full, rowc.opA, rowc.rows_pad, sh.kp, sh.nfull ? 32 : 8, 128,
                   sh.nfull ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_32B);
  ok &= encode_map(&kp.mapA_tail, rowc.opA, rowc.rows_pad, sh.kp, 8, 128, CU_TENSOR_MAP_SWIZZLE_32B);
  ok &= encode_map(&kp.mapB_full, colc.opB, colc.rows_pad, sh.kp, sh.nfull ? 32 : 8, sh.bn,
                   sh.nfull ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_32B);
  ok &= encode_map(&kp.mapB_tail, colc.opB, colc.rows_pad, sh.kp, 8, sh.bn, CU_TENSOR_MAP_SWIZZLE_32B);
  kp.nr = a.nr; kp.nc = a.nc; kp.row_begin = a.row_begin;
  kp.ntiles = (a.nc + sh.bn - 1) / sh.bn;
  const int bm = 128 * sh.nhalf;
  kp.nblk = (a.nr - a.row_begin + bm - 1) / bm;
  kp.item0 = 0;
  kp.scale2 = scale2; kp.eps = a.eps; kp.ep = e;
  kp.part_m = s.part_m[side]; kp.part_s = s.part_s[side]; kp.part_stride = s.part_stride; kp.tickets = s.tickets[side];
  kp.out_idx = nullptr; kp.csr_rp = nullptr; kp.csr_ci = nullptr;
  return ok;
}

// One streaming pass over the staged operands: LSE (out_idx == nullptr) or running arg-max of the raw scores.
cudaError_t stream_pass(const Staged& s, int side, const StreamArgs& a, const LseEpilogue& e, int* out_idx,
                        cudaStream_t st) {
  const bool csr = a.tile_row_ptr != nullptr;
  Shape sh = csr ? plan_shape_csr(s.d, s.prec, s.nlab) : plan_shape(s.d, s.prec, s.nlab);
  if (!sh.ok) return cudaErrorNotSupported;
  const bool am = out_idx != nullptr;
  if (csr && (am || !a.tile_col_idx || (a.row_begin & 127))) return cudaErrorNotSupported;
  if (sh.streamed) return am ? cudaErrorNotSupported : kstream_lse(s, side, a, e, nullptr, 0, st);
  // A resident plan that only fits 64-column tiles issues half-efficient MMAs (N = 64); the K-streamed kernel
  // with its 256 x 128 tiles is faster there (d = 64 in the exact mode: K = 195), unless a knob says otherwise.
  if (sh.bn == 64 && !am && !csr && g_prefer_streamed.load(std::memory_order_relaxed))
    return kstream_lse(s, side, a, e, nullptr, 0, st);
  const CloudOps& rowc = s.cloud[side == 0 ? 0 : 1];
  const CloudOps& colc = s.cloud[side == 0 ? 1 : 0];
  // LSE: logit = scale2 * (x.y + bias/scale2). Arg-max: cost = -2cs * (x.y - bias/(2cs)), so the column
  // "bias" staged next to y is -bias/(2cs) (a.pot holds the raw bias, no log-weights) and scale2 = -2cs.
  const float scale2 = am ? -2.0f * a.cost_scale : (2.0f * a.cost_scale) * (1.0f / a.eps) * kLog2e;
  if (am)
    bias_kernel<<<(colc.rows + 255) / 256, 256, 0, st>>>(colc.opB, colc.rows, sh.kc, sh.kp, a.pot, nullptr, 1.0f,
                                                         1.0f / (scale2 * kLog2e), nullptr);
  else
    bias_kernel<<<(colc.rows + 255) / 256, 256, 0, st>>>(colc.opB, colc.rows, sh.kc, sh.kp, a.pot, a.logw,
                                                         1.0f / a.eps, 1.0f / scale2, e.ctrl, a.pot_shard, a.pot_stride);
  Launch<1> lp{};
  lp.nsub = 1;
  lp.nfull = sh.nfull; lp.ntail = sh.ntail; lp.nstage = sh.nstage;
  SubPass& kp = lp.sub[0];
  if (!fill_subpass(kp, s, side, a, e, sh, scale2)) return cudaErrorInvalidValue;
  if (kp.nblk <= 0) return cudaSuccess;
  lp.total = (long long)kp.nblk * kp.ntiles;
  kp.out_idx = out_idx;
  kp.csr_rp = csr ? a.tile_row_ptr + a.row_begin / 128 : nullptr;
  kp.csr_ci = a.tile_col_idx;
  dim3 grid(pick_ctas(kp.nblk, kp.ntiles));
  if (csr) return launch<1, 128, false, true>(lp, grid, sh.smem, st);
  if (am) {
    if (sh.nhalf == 2) return launch<2, 128, true>(lp, grid, sh.smem, st);
    if (sh.bn == 128) return launch<1, 128, true>(lp, grid, sh.smem, st);
    return launch<1, 64, true>(lp, grid, sh.smem, st);
  }
  if (sh.nhalf == 2) return launch<2, 128, false>(lp, grid, sh.smem, st);
  if (sh.bn == 128) return launch<1, 128, false>(lp, grid, sh.smem, st);
  return launch<1, 64, false>(lp, grid, sh.smem, st);
}
}  // namespace

cudaError_t lse(const Staged& s, int side, const StreamArgs& a, const LseEpilogue& e, cudaStream_t st) {
  return stream_pass(s, side, a, e, nullptr, st);
}

int multi_max() { return kMaxSub; }

cudaError_t lse_multi(const MultiPass* passes, int n, cudaStream_t st) {
  if (n <= 0) return cudaSuccess;
  if (n > kMaxSub || !passes) return cudaErrorInvalidValue;
  const Staged& s0 = *passes[0].s;
  const Shape sh = plan_shape(s0.d, s0.prec, s0.nlab);
  if (!sh.ok || sh.streamed) return cudaErrorNotSupported;
  Launch<kMaxSub> lp{};
  BiasJobs jobs{};
  lp.nfull = sh.nfull; lp.ntail = sh.ntail; lp.nstage = sh.nstage;
  int used = 0, max_cols = 0;
  long long total = 0;
  for (int i = 0; i < n; ++i) {
    const MultiPass& mp = passes[i];
    const Staged& s = *mp.s;
    if (s.d != s0.d || s.prec != s0.prec || s.nlab != s0.nlab || s.kp != s0.kp) return cudaErrorNotSupported;
    if (mp.a.tile_row_ptr || mp.e.ctrl) return cudaErrorNotSupported;
    if (mp.a.nr <= mp.a.row_begin) continue;  // empty row range
    const float scale2 = (2.0f * mp.a.cost_scale) * (1.0f / mp.a.eps) * kLog2e;
    SubPass& kp = lp.sub[used];
    if (!fill_subpass(kp, s, mp.side, mp.a, mp.e, sh, scale2)) return cudaErrorInvalidValue;
    kp.item0 = (int)total;
    total += (long long)kp.nblk * kp.ntiles;
    if (total >= (1ll << 31)) return cudaErrorNotSupported;
    const CloudOps& colc = s.cloud[mp.side == 0 ? 1 : 0];
    BiasJobs::Job& j = jobs.job[used];
    j.opB = colc.opB; j.rows = colc.rows; j.kc = sh.kc; j.kp = sh.kp;
    j.pot = mp.a.pot; j.logw = mp.a.logw; j.inv_eps = 1.0f / mp.a.eps; j.inv_scale2 = 1.0f / scale2;
    j.pot_shard = mp.a.pot_shard; j.pot_stride = mp.a.pot_stride;
    if (colc.rows > max_cols) max_cols = colc.rows;
    // Two passes of one launch must not write the bias columns of the same operand (nor merge in the same
    // partial slots): that is the same side of the same staged problem twice.
    for (int k = 0; k < used; ++k)
      if (lp.sub[k].part_m == kp.part_m) return cudaErrorInvalidValue;
    ++used;
  }
  if (used == 0) return cudaSuccess;
  lp.nsub = used;
  lp.total = total;
  bias_multi_kernel<<<dim3((max_cols + 255) / 256, used), 256, 0, st>>>(jobs);
  // CTAs: one wave, at least ~4 items each, and no row block cut into more pieces than there are slots.
  long long g = detail::sm_count() - g_reserved_sms.load(std::memory_order_relaxed);
  const int limit = g_cta_limit.load(std::memory_order_relaxed);
  if (g < 1) g = 1;
  if (limit >= 1 && limit < g) g = limit;
  if (g > (total + 3) / 4) g = (total + 3) / 4;
  if (g < 1) g = 1;
  int max_tiles = 1;
  for (int k = 0; k < used; ++k) max_tiles = lp.sub[k].ntiles > max_tiles ? lp.sub[k].ntiles : max_tiles;
  while (g > 1 && (long long)max_tiles * g / total + 2 > kMaxChunks) --g;
  dim3 grid((unsigned)g);
  if (sh.nhalf == 2) return launch<2, 128, false, false, kMaxSub>(lp, grid, sh.smem, st);
  if (sh.bn == 128) return launch<1, 128, false, false, kMaxSub>(lp, grid, sh.smem, st);
  return launch<1, 64, false, false, kMaxSub>(lp, grid, sh.smem, st);
}

cudaError_t argmax(const Staged& s, int side, const StreamArgs& a, float* out_val, int* out_idx, cudaStream_t st) {
  if (!out_val || !out_idx) return cudaErrorInvalidValue;
  LseEpilogue e;
  e.out = out_val;
  return stream_pass(s, side, a, e, out_idx, st);
}

// ---- plan-times-matrix host side ----
namespace {

struct PvShape {
  int bn, dv_pad, nslices, nb, nv, cols_pad_mult;
  size_t smem;
  bool split, ok;
};

// Share slots (one raw O tile of a row block each) that the scratch of a matrix pass holds for the column
// split: a function of the larger cloud only, so that sizing and launching agree. No split below 16 column
// tiles; otherwise up to 8 shares per row block, capped at eight 128-row tiles per SM of a 148-SM device.
int pv_share_slots(int nm, int bn) {
  const int ntiles = (nm + bn - 1) / bn;
  const int smax = ntiles / 8 < 8 ? ntiles / 8 : 8;
  if (smax < 2) return 0;
  const long long nblk = (nm + 127) / 128;
  const long long cap = nblk > 1184 ? nblk : 1184;
  const long long want = nblk * smax;
  return (int)(want < cap ? want : cap);
}

// Shares per row block: the smallest count within 2 % of the best SM fill (CTAs / (waves * SMs)).
int pick_pv_split(int nblk, int ntiles, int slots, int sms) {
  if (sms < 1) sms = 1;
  auto fill = [&](int s) {
    const long long ctas = (long long)nblk * s;
    return (double)ctas / (double)(((ctas + sms - 1) / sms) * sms);
  };
  int best = 1;
  double best_fill = fill(1);
  for (int s = 2; s <= 8 && s <= ntiles / 8 && (long long)nblk * s <= slots; ++s)
    if (fill(s) > best_fill + 0.02) { best = s; best_fill = fill(s); }
  const int forced = g_pv_split.load(std::memory_order_relaxed);
  if (forced >= 1 && forced <= 8 && forced <= ntiles && (forced == 1 || (long long)nblk * forced <= slots)) return forced;
  return best;
}

PvShape plan_pv(int d, int prec, int dv, int nlab = 0) {
  PvShape s{};
  Shape sh = plan_shape(d, prec, nlab);
  s.ok = false;
  if (!sh.ok || sh.streamed || dv <= 0) return s;
  s.split = (prec == 1);
  s.bn = s.split ? 64 : 128;
  // TMEM: 3 S/W buffers of 128 columns leave 128 for O, so wider V goes in slices of 128 columns.
  const int w = dv < 128 ? dv : 128;
  s.dv_pad = (w + 31) & ~31;
  s.nslices = (dv + 127) / 128;
  const size_t a = (size_t)128 * sh.kp * 4;
  const size_t b = (size_t)s.bn * sh.kp * 4;
  const size_t v = (size_t)(s.split ? 2 : 1) * (s.bn / 32) * s.dv_pad * 128;
  const size_t budget = kSmemMax - 2048;
  if (a + b + v > budget) return s;
  // Grow the rings alternately (V first: its tiles live through a whole soft-max) up to 3 deep each.
  s.nb = s.nv = 1;
  for (int round = 0; round < 4; ++round) {
    int& ring = (round & 1) ? s.nb : s.nv;
    const size_t unit = (round & 1) ? b : v;
    if (ring < 3 && a + s.nb * b + s.nv * v + unit <= budget) ++ring;
  }
  s.smem = a + s.nb * b + s.nv * v + 2048;
  if (s.smem < (size_t)kSmemMin) s.smem = kSmemMin;
  s.ok = true;
  return s;
}

template <int BN, bool SPLIT>
cudaError_t launch_pv(const CUtensorMap* maps, const PvKernelParams& kp, int grid, size_t smem, cudaStream_t st) {
  auto kern = tc_pv_kernel<BN, SPLIT>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemMax);
  if (e != cudaSuccess) return e;
  kern<<<grid, 128 + 128 * kParts, smem, st>>>(maps[0], maps[1], maps[2], maps[3], maps[4], maps[5], kp);
  return cudaGetLastError();
}

}  // namespace

int plan_pv_split(int rows, int cols, int prec, int sms, int* slots) {
  if (rows <= 0 || cols <= 0 || sms <= 0) return 0;
  const int bn = prec == 1 ? 64 : 128;
  const int nm = rows > cols ? rows : cols;
  const int have = pv_share_slots(nm, bn);
  if (slots) *slots = have;
  return pick_pv_split((rows + 127) / 128, (cols + bn - 1) / bn, have, sms);
}

bool pv_supported(int d, int prec, int dv, int nlab) {
  if (prec != 0 && prec != 1) return false;
  if (plan_shape(d, prec, nlab).streamed) return dv >= 1;  // one column, or V in slices through kstream_pv
  return plan_pv(d, prec, dv, nlab).ok;
}

size_t pv_scratch_bytes(int nc, int d, int prec, int dv, int nlab) {
  const Shape shs = plan_shape(d, prec, nlab);
  if (shs.streamed)
    return dv == 1 ? (size_t)pad256(nc) * sizeof(float) + 1024 : kstream_pv_scratch(nc, nc, shs.kp, dv, prec, false);
  PvShape s = plan_pv(d, prec, dv, nlab);
  if (!s.ok) return 0;
  size_t one = (size_t)s.nslices * s.dv_pad * pad256(nc) * sizeof(float);
  return (s.split ? 2 : 1) * ((one + 1023) & ~size_t(1023)) + 1024 +
         (size_t)pv_share_slots(nc, s.bn) * 128 * s.dv_pad * sizeof(float);
}

cudaError_t pv(const Staged& s, int side, const StreamArgs& a, const PvArgs& pa, char* scratch, cudaStream_t st) {
  Shape sh = plan_shape(s.d, s.prec, s.nlab);
  if (sh.ok && pa.dv == 1 && !pa.rows2 && sh.bn == 64 && !sh.streamed && g_prefer_streamed.load(std::memory_order_relaxed))
    return kstream_vec(s, side, a, pa, scratch, st);
  if (sh.ok && (sh.streamed || pa.rows2)) {
    if (pa.dv == 1 && !pa.rows2) return kstream_vec(s, side, a, pa, scratch, st);
    // the caller sized the scratch with pv_scratch_bytes / mat5_scratch_bytes for these sizes
    const size_t have = kstream_pv_scratch(a.nr > a.nc ? a.nr : a.nc, a.nr > a.nc ? a.nr : a.nc, s.kp, pa.dv, s.prec,
                                           pa.rows2 != nullptr);
    return kstream_pv(s, side, a, pa, scratch, have, st);
  }
  PvShape ps = plan_pv(s.d, s.prec, pa.dv, s.nlab);
  if (!sh.ok || !ps.ok) return cudaErrorNotSupported;
  const CloudOps& rowc = s.cloud[side == 0 ? 0 : 1];
  const CloudOps& colc = s.cloud[side == 0 ? 1 : 0];
  const float scale2 = (2.0f * a.cost_scale) * (1.0f / a.eps) * kLog2e;
  bias_kernel<<<(colc.rows + 255) / 256, 256, 0, st>>>(colc.opB, colc.rows, sh.kc, sh.kp, a.pot, a.logw,
                                                       1.0f / a.eps, 1.0f / scale2, nullptr);
  // V^T (hi / lo), [nslices*dv_pad, cols_pad]
  const int vrows = ps.nslices * ps.dv_pad, vcols = colc.rows_pad;
  char* p = (char*)(((uintptr_t)scratch + 1023) & ~(uintptr_t)1023);
  float* vt_hi = reinterpret_cast<float*>(p);
  size_t one = (((size_t)vrows * vcols * sizeof(float)) + 1023) & ~size_t(1023);
  float* vt_lo = ps.split ? reinterpret_cast<float*>(p + one) : nullptr;
  size_t total = (size_t)vrows * vcols;
  stage_vt_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(pa.V, a.nc, pa.dv, pa.colscale, vrows, vcols,
                                                                   vt_hi, vt_lo);
  CUtensorMap maps[6];
  bool ok = true;
  ok &= encode_map(&maps[0], rowc.opA, rowc.rows_pad, sh.kp, sh.nfull ? 32 : 8, 128,
                   sh.nfull ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_32B);
  ok &= encode_map(&maps[1], rowc.opA, rowc.rows_pad, sh.kp, 8, 128, CU_TENSOR_MAP_SWIZZLE_32B);
  ok &= encode_map(&maps[2], colc.opB, colc.rows_pad, sh.kp, sh.nfull ? 32 : 8, ps.bn,
                   sh.nfull ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_32B);
  ok &= encode_map(&maps[3], colc.opB, colc.rows_pad, sh.kp, 8, ps.bn, CU_TENSOR_MAP_SWIZZLE_32B);
  ok &= encode_map(&maps[4], vt_hi, vrows, vcols, 32, ps.dv_pad, CU_TENSOR_MAP_SWIZZLE_128B);
  ok &= encode_map(&maps[5], ps.split ? vt_lo : vt_hi, vrows, vcols, 32, ps.dv_pad, CU_TENSOR_MAP_SWIZZLE_128B);
  if (!ok) return cudaErrorInvalidValue;
  PvKernelParams kp;
  kp.nr = a.nr; kp.nc = a.nc; kp.row_begin = a.row_begin;
  kp.ntiles = (a.nc + ps.bn - 1) / ps.bn;
  kp.nfull = sh.nfull; kp.ntail = sh.ntail; kp.nb = ps.nb; kp.nv = ps.nv;
  kp.dv = pa.dv; kp.dv_pad = ps.dv_pad; kp.ld_out = pa.dv;
  kp.scale2 = scale2; kp.eps = a.eps; kp.R = pa.R; kp.epilogue = pa.epilogue;
  kp.rowpot = pa.rowpot; kp.rowlogw = pa.rowlogw; kp.roww = pa.roww; kp.gs = pa.gs; kp.coef = pa.coef;
  kp.rows_raw = a.rows; kp.ld_rows = a.d; kp.out = pa.out; kp.skip = pa.skip;
  const int nblk = (a.nr - a.row_begin + 127) / 128;
  if (nblk <= 0) return cudaSuccess;
  // Column shares per row block: as many as fill the SMs best, within the share slots the scratch was sized for.
  const int nm = a.nr > a.nc ? a.nr : a.nc;
  kp.nsplit = pick_pv_split(nblk, kp.ntiles, pv_share_slots(nm, ps.bn),
                            detail::sm_count() - g_reserved_sms.load(std::memory_order_relaxed));
  kp.partial = reinterpret_cast<float*>(p + (ps.split ? 2 : 1) * one);
  kp.tickets = s.tickets[side];
  const int grid = nblk * kp.nsplit;
  for (int sl = 0; sl < ps.nslices; ++sl) {
    kp.dv0 = sl * ps.dv_pad;
    cudaError_t e = ps.split ? launch_pv<64, true>(maps, kp, grid, ps.smem, st)
                             : launch_pv<128, false>(maps, kp, grid, ps.smem, st);
    if (e != cudaSuccess) return e;
  }
  return cudaSuccess;
}

// ---- micro-benchmark: cycles per tcgen05.mma as issued by one lane ----
namespace {

// One lane issues n_mma MMAs (kind::tf32, M=128, K=8, N columns; operands from zero-filled shared memory,
// A optionally from TMEM) back to back, walking the four K slices of a 128-byte swizzle row, commits and
// waits (bounded). out[2*cta] = cycles until the last issue, out[2*cta+1] = cycles until completion.
template <int N, bool TS>
__global__ void __launch_bounds__(128, 1) mma_rate_kernel(int n_mma, long long* out) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* base = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  uint64_t* bars = (uint64_t*)(base + 64 * 1024);
  uint32_t* tmem_slot = (uint32_t*)(bars + 2);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
  for (int i = tid; i < 64 * 1024 / 4; i += 128) ((float*)base)[i] = 0.f;  // A: 16 KB at 0, B: 32 KB at 32 KB
  if (tid == 0) {
    mbar_init(smem_u32(bars), 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  constexpr uint32_t idesc = make_idesc(N);
  const uint32_t al0 = desc_lo(smem_u32(base)), bl0 = desc_lo(smem_u32(base + 32 * 1024));
  const uint32_t a_t = tmem_base + 384;  // TMEM operand columns (contents irrelevant for timing)
  if (warp == 1 && lane == 0) {
    const long long t0 = clock64();
#pragma unroll 1
    for (int i = 0; i < n_mma; i += 8) {
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        const uint32_t off = 2 * (ks & 3);
        if (TS) umma_tf32_ts(tmem_base, a_t + 8 * (ks & 3), pack_desc(bl0 + off, kDescHi128), idesc, 1u);
        else umma_tf32(tmem_base, pack_desc(al0 + off, kDescHi128), pack_desc(bl0 + off, kDescHi128), idesc, 1u);
      }
    }
    const long long t1 = clock64();
    umma_commit(smem_u32(bars));
    mbar_wait(smem_u32(bars), 0, abort_flag, 0);
    const long long t2 = clock64();
    out[blockIdx.x * 2] = t1 - t0;
    out[blockIdx.x * 2 + 1] = t2 - t0;
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    __syncwarp();
    tmem_dealloc(tmem_base, 512);
  }
  if (tid == 0 && *abort_flag) atomicExch(&g_tc_error, 1);
}

template <int N, bool TS>
double run_mma_rate(int sms) {
  const int n_mma = 4096;
  long long* out = nullptr;
  if (cudaMalloc(&out, sizeof(long long) * 2 * sms) != cudaSuccess) return -1.0;
  auto k = mma_rate_kernel<N, TS>;
  const size_t smem = 64 * 1024 + 2048;
  double res = -1.0;
  if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) == cudaSuccess) {
    k<<<sms, 128, smem>>>(64, out);      // warm-up
    k<<<sms, 128, smem>>>(n_mma, out);
    long long* host = new long long[2 * sms];
    if (cudaMemcpy(host, out, sizeof(long long) * 2 * sms, cudaMemcpyDeviceToHost) == cudaSuccess) {
      double tot = 0.0;
      for (int i = 0; i < sms; ++i) tot += (double)host[2 * i + 1];
      res = tot / sms / n_mma;
    }
    delete[] host;
  }
  cudaFree(out);
  return res;
}

}  // namespace

double micro_mma_cycles(int n_cols, bool a_in_tmem) {
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -1.0;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (sms <= 0) return -1.0;
  switch (n_cols) {
    case 64: return a_in_tmem ? run_mma_rate<64, true>(sms) : run_mma_rate<64, false>(sms);
    case 128: return a_in_tmem ? run_mma_rate<128, true>(sms) : run_mma_rate<128, false>(sms);
    case 256: return a_in_tmem ? run_mma_rate<256, true>(sms) : run_mma_rate<256, false>(sms);
    default: return -1.0;
  }
}

int read_error_flag_k();  // fs_tck.cu: the K-streamed kernels keep their own word (no relocatable device code)
int clear_error_flag_k();

int clear_error_flag() {
  const int zero = 0;
  if (cudaMemcpyToSymbol(g_tc_error, &zero, sizeof(int)) != cudaSuccess) return -1;
  return clear_error_flag_k();
}

int read_error_flag() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_tc_error, sizeof(int)) != cudaSuccess) return -1;
  const int k = read_error_flag_k();
  if (k < 0) return -1;
  return (v | k) ? 1 : 0;
}

}  // namespace tc
}  // namespace fs
