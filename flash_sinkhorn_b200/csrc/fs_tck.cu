// K-streamed tcgen05 passes for sm_100a: the score tile S = rows x cols^T accumulates in TMEM while BOTH
// operands stream through shared memory in 32-float K chunks, so the feature dimension is unbounded
// (d = 2048, or d = 128 in the 3xTF32 mode whose contraction is three times as long).
//
// Work item = (row block of BM = 128*NHALF rows, column tile of BN columns). The items, row block after
// row block, are cut into equal contiguous ranges, one per CTA, one CTA per SM. Per item and K chunk the
// producer lane fills one ring stage with the chunk of the row block (NHALF x 128 rows x 128 bytes) and of
// the column tile (BN rows x 128 bytes), both 128-byte swizzled by TMA; one MMA lane per 128-row half issues
// four tcgen05.mma kind::tf32 (M = 128, N = BN, K = 8) per stage into that half's TMEM accumulator and
// commits the stage back to the producer; after the last chunk it commits the accumulator to the epilogue
// warps. Large tiles matter here: a 256 x 256 tile needs 64 flop per operand byte, a 256 x 128 one 43.
// Warp roles: warp 0 producer, warps 1 and 3 MMA issuers (warp 1 owns the TMEM allocation), warps 4.. are
// the epilogue warpgroups, two per 128-row half, each taking half of a tile's 32-column chunks; thread t of
// a warpgroup owns score row t (TMEM lane t).
//
// Epilogues (template parameter):
//   EPI_LSE : online log-sum-exp of the scaled scores, partial (offset, sum) pairs of row blocks shared by
//             several CTAs merged by the CTA that takes the block's last ticket (same scheme as the
//             resident-operand kernel); optionally the raw scores are also written out.
//   EPI_VEC : sum_j 2^(scale*S_ij - R_i) v_j with a known row normaliser R (plan-times-vector).
//   EPI_OUT : plain GEMM tile store with a per-row epilogue (second GEMM of a plan-times-matrix pass, whose
//             "row operand" is the weight matrix and whose "column operand" is the transposed V).
//
// Every mbarrier wait is bounded; on expiry the CTA raises an abort flag, lets its copies and MMAs land,
// frees its TMEM and returns, and a device-global error word records the event.
#include "fs_tc.cuh"
#include "fs_ptx.cuh"

#include <cudaTypedefs.h>

#include <atomic>

namespace fs {
namespace tc {

__device__ int g_tck_error = 0;

namespace {

enum { EPI_LSE = 0, EPI_VEC = 1, EPI_OUT = 2 };
constexpr int kPartsK = 2;  // epilogue warpgroups per 128-row half

struct KParams {
  int nr, nc;       // end of the row range (rows >= nr are padding) / valid columns
  int row_begin;    // first row of the range; row blocks are counted from here
  int ntiles, nblk;
  int nk;           // K chunks of 32 floats
  int klast;        // K steps of 8 in the last chunk (1..4)
  int nstage;
  float scale2, eps;
  LseEpilogue ep;   // EPI_LSE
  float* part_m; float* part_s; int part_stride; int* tickets;
  float* s_out; long long ld_s;  // EPI_LSE: optional raw scores, row r at s_out + (r - row_begin) * ld_s
  // EPI_VEC / EPI_OUT
  const float* R;        // [rows] log2 normaliser
  const float* vpad;     // EPI_VEC: v padded with zeros to a whole number of tiles
  const float* rowpot; const float* rowlogw;
  float* vout;           // EPI_VEC output
  const int* skip;       // device flag: non-zero => the launch is a no-op
  // EPI_OUT: rows of the row operand are local to a chunk; global row = out_row0 + local row
  int epilogue, out_row0, dv, ld_out;
  float* out;
  const float* roww; const float* gs; float coef;
  const float* rows_raw; int ld_rows;
};

template <int NHALF, int BN, int NBUF, int EPI>
__global__ void __launch_bounds__(128 + 128 * NHALF * kPartsK, 1)
tck_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB, const KParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  constexpr int BM = 128 * NHALF;
  constexpr int NSYNC = 128 * NHALF * kPartsK;  // epilogue threads (named barrier 1)
  const long long total_items = (long long)p.nblk * p.ntiles;
  const int w_begin = (int)((total_items * blockIdx.x) / gridDim.x);
  const int w_end = (int)((total_items * (blockIdx.x + 1)) / gridDim.x);
  auto cta_first = [&](int c) { return (int)((total_items * c) / gridDim.x); };
  auto cta_of = [&](int t) {
    int c = (int)(((long long)t * gridDim.x) / total_items);
    while (c + 1 < (int)gridDim.x && cta_first(c + 1) <= t) ++c;
    while (c > 0 && cta_first(c) > t) --c;
    return c;
  };

  if (EPI == EPI_LSE && p.ep.ctrl && p.ep.ctrl->converged) {  // solve already stopped: identity step
    if (p.ep.old && p.ep.out)
      for (int r = p.row_begin + blockIdx.x * blockDim.x + tid; r < p.nr; r += gridDim.x * blockDim.x)
        p.ep.out[r] = p.ep.old[r];
    return;
  }
  if (EPI != EPI_LSE && p.skip && *p.skip) return;  // uniform across the grid

  // ---- shared memory: ring of K-chunk stages, then barriers and small merge buffers ----
  uint8_t* base = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  constexpr uint32_t kAHalf = 128 * 128;                    // 128 rows x 32 floats
  constexpr uint32_t kStage = NHALF * kAHalf + BN * 128;    // row block chunk + column tile chunk
  uint8_t* ring = base;
  uint64_t* bars = (uint64_t*)(ring + (size_t)p.nstage * kStage);
  const int FULL = 0, EMPTY = p.nstage, S_FULL = 2 * p.nstage, S_EMPTY = S_FULL + NHALF * NBUF,
            DRAIN = S_EMPTY + NHALF * NBUF, NBARS = DRAIN + 2;
  uint32_t* tmem_slot = (uint32_t*)(bars + NBARS);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
  volatile int* last_flag = (volatile int*)(tmem_slot + 2);
  float* merge_off = (float*)(tmem_slot + 4);  // [NHALF*128] partials of the second column part
  float* merge_sum = merge_off + NHALF * 128;
  auto bar = [&](int i) { return smem_u32(bars + i); };

  constexpr uint32_t kTmemCols = NHALF * NBUF * BN;  // 128, 256 or 512
  static_assert(kTmemCols >= 32 && kTmemCols <= 512 && (kTmemCols & (kTmemCols - 1)) == 0, "TMEM columns");

  if (tid == 0) {
    for (int s = 0; s < p.nstage; ++s) {
      mbar_init(bar(FULL + s), 1);
      mbar_init(bar(EMPTY + s), NHALF);  // one commit per MMA-issuing lane
    }
    for (int i = 0; i < NHALF * NBUF; ++i) {
      mbar_init(bar(S_FULL + i), 1);
      mbar_init(bar(S_EMPTY + i), 4 * kPartsK);  // one arrive per epilogue warp reading the buffer
    }
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
      int issued = 0;  // stages filled so far (ring position)
      bool ok = true;
#pragma unroll 1
      for (int w = w_begin; ok && w < w_end; ++w) {
        const int blk = w / p.ntiles, j = w - blk * p.ntiles;
        const int row0 = p.row_begin + blk * BM, col0 = j * BN;
#pragma unroll 1
        for (int kc = 0; kc < p.nk; ++kc) {
          const int s = issued % p.nstage;
          const uint32_t ph = (issued / p.nstage) & 1;
          if (!mbar_wait(bar(EMPTY + s), ph ^ 1, abort_flag, 2000)) { ok = false; break; }
          mbar_expect_tx(bar(FULL + s), kStage);
          const uint32_t dst = smem_u32(ring + (size_t)s * kStage);
#pragma unroll
          for (int h = 0; h < NHALF; ++h) tma_load_2d(dst + h * kAHalf, &mapA, kc * 32, row0 + h * 128, bar(FULL + s));
          tma_load_2d(dst + NHALF * kAHalf, &mapB, kc * 32, col0, bar(FULL + s));
          ++issued;
        }
      }
      if (*abort_flag) {  // let every copy we issued land before the CTA goes away
        for (int j = (issued > p.nstage ? issued - p.nstage : 0); j < issued; ++j)
          mbar_wait_quiet(bar(FULL + j % p.nstage), (j / p.nstage) & 1);
      }
    }
  } else if (warp == 1 || (warp == 3 && NHALF == 2)) {
    // ===================== MMA issuers: one warp per 128-row half =====================
    // All 32 lanes run the loop (warp-uniform descriptor arithmetic), one elected lane issues; every exit
    // decision is a warp vote, since elect.sync needs all lanes at the same instruction.
    {
      const int h = (warp == 1) ? 0 : 1;
      constexpr uint32_t idesc = make_idesc(BN);
      bool ok = true;
      int s = 0;
      uint32_t ph = 0;
      int jt = 0;  // items processed so far by this CTA (accumulator buffer position)
#pragma unroll 1
      for (int w = w_begin; ok && w < w_end; ++w, ++jt) {
        const int buf = jt % NBUF;
        const uint32_t sph = (jt / NBUF) & 1;
        if (!__all_sync(0xffffffffu, mbar_wait(bar(S_EMPTY + h * NBUF + buf), sph ^ 1, abort_flag, 2000))) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)((h * NBUF + buf) * BN);
        uint32_t acc = 0;
#pragma unroll 1
        for (int kc = 0; kc < p.nk; ++kc) {
          if (!__all_sync(0xffffffffu, mbar_wait(bar(FULL + s), ph, abort_flag, 2000))) { ok = false; break; }
          tc_fence_after();
          const uint32_t stage_addr = smem_u32(ring + (size_t)s * kStage);
          const uint32_t al = desc_lo(stage_addr + h * kAHalf), bl = desc_lo(stage_addr + NHALF * kAHalf);
          if (kc + 1 < p.nk) {
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
              if (elect_one())
                umma_tf32(d_tmem, pack_desc(al + 2 * ks, kDescHi128), pack_desc(bl + 2 * ks, kDescHi128), idesc, acc);
              acc = 1;
            }
          } else {
#pragma unroll 1
            for (int ks = 0; ks < p.klast; ++ks) {
              if (elect_one())
                umma_tf32(d_tmem, pack_desc(al + 2 * ks, kDescHi128), pack_desc(bl + 2 * ks, kDescHi128), idesc, acc);
              acc = 1;
            }
          }
          if (elect_one()) umma_commit(bar(EMPTY + s));
          __syncwarp();
          if (++s == p.nstage) { s = 0; ph ^= 1; }
        }
        if (!ok) break;
        if (elect_one()) umma_commit(bar(S_FULL + h * NBUF + buf));
        __syncwarp();
      }
      __syncwarp();
      if (*abort_flag && lane == 0) {  // wait (bounded) for every MMA issued by this warp before TMEM is freed
        umma_commit(bar(DRAIN + h));
        mbar_wait_quiet(bar(DRAIN + h), 0);
      }
    }
  } else if (warp >= 4) {
    // ===================== epilogue warpgroups =====================
    const int wg = (warp - 4) >> 2;
    const int h = wg / kPartsK;     // 128-row half
    const int part = wg % kPartsK;  // which half of each tile's chunks
    const int q = warp & 3;         // TMEM lane quarter this warp may read
    const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
    const int trow = h * 128 + q * 32 + lane;  // this thread's row inside a row block
    const float scale = p.scale2;
    constexpr int CH = BN / 32 / kPartsK;  // 32-column chunks of a tile owned by this warpgroup
    const int total = (w_end - w_begin) * CH;
    const int c_base = part * CH;
    // Running state of the current segment (the part of one row block this CTA covers). LSE: sum =
    // s_run * 2^off_run with off_run the rounded value scale*max. VEC: off_run stays 0 and s_run is the signed
    // weighted sum, so the same merge formulas (2^0 = 1 exactly) serve both.
    const float off_init = (EPI == EPI_LSE) ? __fmul_rn(scale, kRunInit) : 0.f;
    float m_run = kRunInit, off_run = off_init, s_run = 0.f;
    int cur_blk = w_begin / p.ntiles, cur_jt = w_begin - cur_blk * p.ntiles;  // item of the chunk being consumed
    bool row_fresh = true;  // per-row constants (negR, fac) belong to another row block
    float negR = 0.f, fac = 0.f;
    bool ok = true;

    auto load_row_consts = [&]() {
      row_fresh = false;
      if (EPI == EPI_VEC) {
        const int r = p.row_begin + cur_blk * BM + trow;
        negR = (r < p.nr) ? -__ldg(p.R + r) : 0.f;
      } else if (EPI == EPI_OUT) {
        const int lr = cur_blk * BM + trow;
        const int gr = p.out_row0 + lr;
        fac = 0.f;
        if (lr < p.nr) {
          if (p.epilogue == PV_GRAD) {
            fac = p.coef * (p.gs ? __ldg(p.gs) : 1.f) * __ldg(p.roww + gr);
          } else {
            const float rt = (__ldg(p.rowpot + gr) * (1.0f / p.eps) + (p.rowlogw ? __ldg(p.rowlogw + gr) : 0.f)) * kLog2e;
            fac = p.coef * ex2(rt + __ldg(p.R + gr));
          }
        }
      }
    };

    auto consume = [&](const uint32_t (&r)[32], int chunk_in_tile) {
      float v[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
      const int col0 = cur_jt * BN + (c_base + chunk_in_tile) * 32;
      if (EPI == EPI_LSE) {
        if (p.s_out) {
          const int lr = cur_blk * BM + trow;
          if (p.row_begin + lr < p.nr) {
            float4* dst = reinterpret_cast<float4*>(p.s_out + (size_t)lr * p.ld_s + col0);
#pragma unroll
            for (int i = 0; i < 8; ++i) dst[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
          }
        }
        float t[11];
#pragma unroll
        for (int i = 0; i < 10; ++i) t[i] = max3(v[3 * i], v[3 * i + 1], v[3 * i + 2]);
        t[10] = fmaxf(v[30], v[31]);
        float u0 = max3(t[0], t[1], t[2]), u1 = max3(t[3], t[4], t[5]), u2 = max3(t[6], t[7], t[8]);
        float cm = fmaxf(max3(u0, u1, u2), fmaxf(t[9], t[10]));
        const float m_new = fmaxf(m_run, cm);
        const float off_new = __fmul_rn(scale, m_new);  // not contracted with the subtraction below
        const float nms = -off_new;
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
      } else if (EPI == EPI_VEC) {
        if (row_fresh) load_row_consts();
        const float4* vv = reinterpret_cast<const float4*>(p.vpad + col0);  // same address for the whole warp
        float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float4 t = __ldg(vv + i);
          a0 = fmaf(ex2(fmaf(v[4 * i], scale, negR)), t.x, a0);
          a1 = fmaf(ex2(fmaf(v[4 * i + 1], scale, negR)), t.y, a1);
          a2 = fmaf(ex2(fmaf(v[4 * i + 2], scale, negR)), t.z, a2);
          a3 = fmaf(ex2(fmaf(v[4 * i + 3], scale, negR)), t.w, a3);
        }
        s_run += (a0 + a1) + (a2 + a3);
      } else {
        if (row_fresh) load_row_consts();
        const int lr = cur_blk * BM + trow;
        if (lr < p.nr && col0 < p.dv) {
          const int gr = p.out_row0 + lr;
          float* orow = p.out + (size_t)gr * p.ld_out + col0;
          const float* xrow = (p.epilogue == PV_GRAD) ? p.rows_raw + (size_t)gr * p.ld_rows + col0 : nullptr;
          const bool vec4 = ((p.ld_out & 3) == 0) && (col0 + 32 <= p.dv) && (!xrow || (p.ld_rows & 3) == 0);
          if (vec4) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              float4 o = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
              if (xrow) {
                const float4 xv = __ldg(reinterpret_cast<const float4*>(xrow) + i);
                o = make_float4(xv.x - o.x, xv.y - o.y, xv.z - o.z, xv.w - o.w);
              }
              reinterpret_cast<float4*>(orow)[i] = make_float4(fac * o.x, fac * o.y, fac * o.z, fac * o.w);
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) {  // unrolled: v[] must stay in registers
              if (col0 + i < p.dv) {
                float val = v[i];
                if (xrow) val = __ldg(xrow + i) - val;
                orow[i] = fac * val;
              }
            }
          }
        }
      }
    };

    // Issue the TMEM load of chunk g (first waits for its tile if g starts one). No wait for the data.
    auto issue = [&](int g, uint32_t (&r)[32]) -> bool {
      const int j = g / CH, c = g % CH;
      const int buf = j % NBUF;
      if (c == 0) {
        if (!mbar_wait(bar(S_FULL + h * NBUF + buf), (j / NBUF) & 1, abort_flag)) return false;
        __syncwarp();  // lanes leave the poll loop at different times; tcgen05.ld is .sync.aligned
        tc_fence_after();
      }
      tmem_ld32_nowait(lane_addr + (uint32_t)((h * NBUF + buf) * BN) + (c_base + c) * 32, r);
      return true;
    };
    // The load of chunk g has landed: if it was the last chunk of its tile, hand the accumulator back.
    auto landed = [&](int g, uint32_t (&r)[32]) {
      tmem_ld_wait(r);
      if (g % CH == CH - 1) {
        const int j = g / CH;
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(S_EMPTY + h * NBUF + (j % NBUF)));
      }
    };
    // End of a segment (LSE / VEC): merge the two column parts, then either finish the rows (the block is
    // ours alone) or publish the (offset, sum) pair per row; the CTA that publishes last merges all pairs in
    // piece order and applies the epilogue. Every epilogue warp runs the same barrier sequence for every
    // segment, also after an abort (live = false), so the named barriers always match.
    auto finalize = [&](int blk, bool live) {
      const int r = p.row_begin + blk * BM + trow;
      if (part == 1) {
        merge_off[trow] = live ? off_run : off_init;
        merge_sum[trow] = live ? s_run : 0.f;
      }
      asm volatile("bar.sync 1, %0;" ::"n"(NSYNC) : "memory");
      if (part == 0) {
        const float o2 = merge_off[trow], s2 = merge_sum[trow];
        const float on = fmaxf(off_run, o2);
        s_run = s_run * ex2(off_run - on) + s2 * ex2(o2 - on);
        off_run = on;
      }
      const int c_lo = cta_of(blk * p.ntiles), c_hi = cta_of((blk + 1) * p.ntiles - 1);
      const int pieces = c_hi - c_lo + 1, piece = (int)blockIdx.x - c_lo;
      bool finish = pieces == 1;
      if (pieces > 1) {
        if (live && part == 0 && r < p.nr) {
          p.part_m[(size_t)piece * p.part_stride + r] = off_run;
          p.part_s[(size_t)piece * p.part_stride + r] = s_run;
        }
        __threadfence();  // the pairs must be visible device-wide before the ticket is taken
        asm volatile("bar.sync 1, %0;" ::"n"(NSYNC) : "memory");
        if (warp == 4 && lane == 0) *last_flag = (atomicAdd(p.tickets + blk, 1) == pieces - 1) ? 1 : 0;
        asm volatile("bar.sync 1, %0;" ::"n"(NSYNC) : "memory");
        finish = *last_flag != 0;
        if (finish) {
          __threadfence();
          if (part == 0 && r < p.nr) {
            float M = __ldcg(p.part_m + r);
            for (int c = 1; c < pieces; ++c) M = fmaxf(M, __ldcg(p.part_m + (size_t)c * p.part_stride + r));
            float S = 0.f;
            for (int c = 0; c < pieces; ++c)
              S += __ldcg(p.part_s + (size_t)c * p.part_stride + r) *
                   ex2(__ldcg(p.part_m + (size_t)c * p.part_stride + r) - M);
            off_run = M;
            s_run = S;
          }
          if (warp == 4 && lane == 0) p.tickets[blk] = 0;  // ready for the next launch on this stream
        }
      }
      if (finish && live && part == 0 && r < p.nr && !*abort_flag) {
        if (EPI == EPI_LSE) {
          const LseEpilogue& ep = p.ep;
          const float lse2 = off_run + log2f(fmaxf(s_run, 1e-40f));
          if (ep.lse2) ep.lse2[r] = lse2;
          if (ep.out) {
            const float cand = -p.eps * ep.damping * (lse2 * kLn2);
            float o = ep.w * cand;
            if (ep.old) o += (1.0f - ep.w) * ep.old[r];
            if (ep.shift) o -= ep.shiftcoef * ep.shift[r];
            if (ep.addvec) o += ep.addcoef * ep.addvec[r];
            ep.out[r] = o;
          }
        } else {
          const float rt = (__ldg(p.rowpot + r) * (1.0f / p.eps) + (p.rowlogw ? __ldg(p.rowlogw + r) : 0.f)) * kLog2e;
          p.vout[r] = ex2(rt + __ldg(p.R + r)) * s_run;
        }
      }
      asm volatile("bar.sync 1, %0;" ::"n"(NSYNC) : "memory");  // merge buffers are re-used by the next segment
      m_run = kRunInit;
      off_run = off_init;
      s_run = 0.f;
    };
    // Segment bookkeeping: seg_w = first item of the current segment, seg_end_g = its last chunk + 1.
    int seg_w = w_begin;
    auto seg_len = [&](int w) {
      const int j0 = w % p.ntiles;
      return (p.ntiles - j0 < w_end - w) ? (p.ntiles - j0) : (w_end - w);
    };
    int seg_end_g = seg_len(seg_w) * CH;
    auto consumed = [&](int g) {  // chunk g has been folded in
      if (g % CH == CH - 1) {     // last chunk of its tile: move on to the next item
        if (++cur_jt == p.ntiles) { cur_jt = 0; ++cur_blk; row_fresh = true; }
      }
      if (g + 1 == seg_end_g) {
        if (EPI != EPI_OUT) finalize(seg_w / p.ntiles, true);
        seg_w += seg_len(seg_w);
        if (seg_w < w_end) seg_end_g += seg_len(seg_w) * CH;
      }
    };
    // Software pipeline, two register buffers: the load of chunk g+1 is in flight while chunk g is consumed.
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
      consumed(g);
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
    if (EPI != EPI_OUT) {
#pragma unroll 1
      while (seg_w < w_end) {
        finalize(seg_w / p.ntiles, false);
        seg_w += seg_len(seg_w);
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
  if (tid == 0 && *abort_flag) atomicExch(&g_tck_error, 1);
}

// ------------------------------------------------------------------ K-streamed plan-times-matrix kernel
// out = epilogue( sum_j 2^(logit_ij - R_i) [* (rows2_i . cols_j)] * V_j ) for narrow V (at most 128 columns per
// launch) when the row operand does not fit in shared memory: the score GEMM streams both operands in K chunks
// (as tck_kernel does), the weights go back to TMEM and feed the second GEMM O += W x V^T with A from TMEM, O
// stays in TMEM for the whole pass (FlashAttention-style). R is the exact log2 normaliser from a soft-min pass
// over the same staged operands, so no running maximum and no rescaling of O are needed.
//   warp 0 : TMA producer of the K-chunk ring (row chunk, optional second row operand chunk, column chunk)
//   warp 2 : TMA producer of the V^T tiles (own ring)
//   warp 1 : score MMAs (S, and E = rows2 x cols^T in MAT5 mode), warp 3 : second GEMM
//   warps 4..11 : two warpgroups turning scores into weights (each half of a tile's 32-column chunks)
// One CTA = 128 rows, column tiles of 64. TMEM: NSW buffers of [S -> Wh | Wl (split) | E (MAT5)], then O.
struct KPvParams {
  int nr, nc, ntiles, row_begin;
  int nk, klast, nstage, nv;   // K chunks, K steps of the last one, ring depths (K chunks / V tiles)
  int dv, dv_pad, dv0, ld_out;
  float scale2, eps;
  const float* R;
  int epilogue;
  const float* rowpot; const float* rowlogw; const float* roww; const float* gs; float coef;
  const float* rows_raw; int ld_rows;
  float* out;
  const int* skip;
};

template <bool SPLIT, bool MAT5>
__global__ void __launch_bounds__(128 + 128 * kPartsK, 1)
tck_pv_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapA2,
              const __grid_constant__ CUtensorMap mapB, const __grid_constant__ CUtensorMap mapV_hi,
              const __grid_constant__ CUtensorMap mapV_lo, const KPvParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int row0 = p.row_begin + blockIdx.x * 128;
  if (p.skip && *p.skip) return;  // uniform across the grid
  constexpr int BN = 64;
  constexpr int WCOLS = SPLIT ? 2 * BN : BN;          // S, overwritten by Wh (and Wl right after it)
  constexpr int BUFCOLS = WCOLS + (MAT5 ? BN : 0);    // + E
  constexpr int NSW = MAT5 ? 2 : 3;                   // score / weight buffers
  constexpr int NVP = SPLIT ? 2 : 1;
  static_assert(NSW * BUFCOLS + 128 <= 512, "TMEM budget");

  uint8_t* base = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  constexpr uint32_t kAChunk = 128 * 128, kBChunk = BN * 128;
  constexpr uint32_t kStage = kAChunk * (MAT5 ? 2 : 1) + kBChunk;
  const uint32_t v_blk = (uint32_t)p.dv_pad * 128;   // one 32-column K block of V^T: dv_pad rows x 128 B
  const uint32_t v_bytes = (BN / 32) * v_blk;        // per hi/lo part
  const uint32_t v_stage = NVP * v_bytes;
  uint8_t* ring = base;
  uint8_t* v_smem = ring + (size_t)p.nstage * kStage;
  uint64_t* bars = (uint64_t*)(v_smem + (size_t)p.nv * v_stage);
  const int FULL = 0, EMPTY = p.nstage, V_FULL = 2 * p.nstage, V_EMPTY = V_FULL + p.nv, S_FULL = V_EMPTY + p.nv,
            W_FULL = S_FULL + NSW, W_FREE = W_FULL + NSW, O_FULL = W_FREE + NSW, DRAIN = O_FULL + 1, NBARS = DRAIN + 1;
  uint32_t* tmem_slot = (uint32_t*)(bars + NBARS);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
  auto bar = [&](int i) { return smem_u32(bars + i); };
  constexpr uint32_t kTmemCols = 512;

  if (tid == 0) {
    for (int s = 0; s < p.nstage; ++s) {
      mbar_init(bar(FULL + s), 1);
      mbar_init(bar(EMPTY + s), 1);
    }
    for (int s = 0; s < p.nv; ++s) {
      mbar_init(bar(V_FULL + s), 1);
      mbar_init(bar(V_EMPTY + s), 1);
    }
    for (int i = 0; i < NSW; ++i) {
      mbar_init(bar(S_FULL + i), 1);
      mbar_init(bar(W_FULL + i), 4 * kPartsK);
      mbar_init(bar(W_FREE + i), 1);
    }
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
  const uint32_t o_tmem = tmem_base + NSW * BUFCOLS;

  if (warp == 0) {
    if (lane == 0) {  // K-chunk ring: for every column tile all chunks of the row block and of the tile
      int issued = 0;
      bool ok = true;
#pragma unroll 1
      for (int j = 0; ok && j < p.ntiles; ++j) {
#pragma unroll 1
        for (int kc = 0; kc < p.nk; ++kc) {
          const int s = issued % p.nstage;
          const uint32_t ph = (issued / p.nstage) & 1;
          if (!mbar_wait(bar(EMPTY + s), ph ^ 1, abort_flag, 2000)) { ok = false; break; }
          mbar_expect_tx(bar(FULL + s), kStage);
          const uint32_t dst = smem_u32(ring + (size_t)s * kStage);
          tma_load_2d(dst, &mapA, kc * 32, row0, bar(FULL + s));
          if (MAT5) tma_load_2d(dst + kAChunk, &mapA2, kc * 32, row0, bar(FULL + s));
          tma_load_2d(dst + kAChunk * (MAT5 ? 2 : 1), &mapB, kc * 32, j * BN, bar(FULL + s));
          ++issued;
        }
      }
      if (*abort_flag) {
        for (int j = (issued > p.nstage ? issued - p.nstage : 0); j < issued; ++j)
          mbar_wait_quiet(bar(FULL + j % p.nstage), (j / p.nstage) & 1);
      }
    }
  } else if (warp == 2) {
    if (lane == 0) {  // V^T tiles (hi and, in split mode, lo) on their own ring
      int issued = 0;
#pragma unroll 1
      for (int j = 0; j < p.ntiles; ++j) {
        const int s = j % p.nv;
        const uint32_t ph = (j / p.nv) & 1;
        if (!mbar_wait(bar(V_EMPTY + s), ph ^ 1, abort_flag, 2000)) break;
        mbar_expect_tx(bar(V_FULL + s), v_stage);
        const uint32_t dv_dst = smem_u32(v_smem + (size_t)s * v_stage);
        for (int kb = 0; kb < BN / 32; ++kb) {
          tma_load_2d(dv_dst + kb * v_blk, &mapV_hi, j * BN + kb * 32, p.dv0, bar(V_FULL + s));
          if (SPLIT) tma_load_2d(dv_dst + v_bytes + kb * v_blk, &mapV_lo, j * BN + kb * 32, p.dv0, bar(V_FULL + s));
        }
        issued = j + 1;
      }
      if (*abort_flag) {
        for (int j = (issued > p.nv ? issued - p.nv : 0); j < issued; ++j)
          mbar_wait_quiet(bar(V_FULL + j % p.nv), (j / p.nv) & 1);
      }
    }
  } else if (warp == 1) {
    {  // score GEMM(s) of tile j into buffer j % NSW, accumulated over the K chunks. All 32 lanes run the loop
       // (warp-uniform descriptor arithmetic), one elected lane issues; exits are warp votes.
      constexpr uint32_t idesc1 = make_idesc(BN);
      bool ok = true;
      int s = 0;
      uint32_t ph = 0;
#pragma unroll 1
      for (int j = 0; ok && j < p.ntiles; ++j) {
        const int buf = j % NSW;
        if (!__all_sync(0xffffffffu, mbar_wait(bar(W_FREE + buf), ((j / NSW) & 1) ^ 1, abort_flag, 2000))) break;
        tc_fence_after();
        const uint32_t s_tmem = tmem_base + buf * BUFCOLS;
        uint32_t acc = 0;
#pragma unroll 1
        for (int kc = 0; kc < p.nk; ++kc) {
          if (!__all_sync(0xffffffffu, mbar_wait(bar(FULL + s), ph, abort_flag, 2000))) { ok = false; break; }
          tc_fence_after();
          const uint32_t stage_addr = smem_u32(ring + (size_t)s * kStage);
          const uint32_t al = desc_lo(stage_addr), a2l = desc_lo(stage_addr + kAChunk),
                         bl = desc_lo(stage_addr + kAChunk * (MAT5 ? 2 : 1));
          const int nks = (kc + 1 < p.nk) ? 4 : p.klast;
#pragma unroll 1
          for (int ks = 0; ks < nks; ++ks) {
            if (elect_one()) {
              umma_tf32(s_tmem, pack_desc(al + 2 * ks, kDescHi128), pack_desc(bl + 2 * ks, kDescHi128), idesc1, acc);
              if (MAT5)
                umma_tf32(s_tmem + WCOLS, pack_desc(a2l + 2 * ks, kDescHi128), pack_desc(bl + 2 * ks, kDescHi128),
                          idesc1, acc);
            }
            acc = 1;
          }
          if (elect_one()) umma_commit(bar(EMPTY + s));
          __syncwarp();
          if (++s == p.nstage) { s = 0; ph ^= 1; }
        }
        if (!ok) break;
        if (elect_one()) umma_commit(bar(S_FULL + buf));
        __syncwarp();
      }
      __syncwarp();
      if (*abort_flag && lane == 0) {
        umma_commit(bar(DRAIN));
        mbar_wait_quiet(bar(DRAIN), 0);
      }
    }
  } else if (warp == 3) {
    {  // second GEMM O += W_j . V_j (W read from TMEM) once the weights of tile j are written
      const uint32_t idesc2 = make_idesc(p.dv_pad);
      const uint32_t v_blk_units = v_blk >> 4;
      uint32_t o_acc = 0;
#pragma unroll 1
      for (int j = 0; j < p.ntiles; ++j) {
        const int sv = j % p.nv, buf = j % NSW;
        if (!__all_sync(0xffffffffu, mbar_wait(bar(V_FULL + sv), (j / p.nv) & 1, abort_flag, 2000))) break;
        if (!__all_sync(0xffffffffu, mbar_wait(bar(W_FULL + buf), (j / NSW) & 1, abort_flag, 2000))) break;
        tc_fence_after();
        const uint32_t w_tmem = tmem_base + buf * BUFCOLS;
        const uint32_t v_lo0 = desc_lo(smem_u32(v_smem + (size_t)sv * v_stage));
#pragma unroll 1
        for (int part = 0; part < (SPLIT ? 3 : 1); ++part) {  // Wh.Vh, Wl.Vh, Wh.Vl
          uint32_t wa = w_tmem + ((part == 1) ? BN : 0);
          uint32_t vl = v_lo0 + ((part == 2) ? (v_bytes >> 4) : 0);
#pragma unroll 1
          for (int kb = 0; kb < BN / 32; ++kb) {
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
              if (elect_one()) umma_tf32_ts(o_tmem, wa + ks * 8, pack_desc(vl + 2 * ks, kDescHi128), idesc2, o_acc);
              o_acc = 1;
            }
            wa += 32;
            vl += v_blk_units;
          }
        }
        if (elect_one()) {
          umma_commit(bar(V_EMPTY + sv));
          umma_commit(bar(W_FREE + buf));
        }
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
    const int r = row0 + q * 32 + lane;
    const float scale = p.scale2;
    const float negR = (r < p.nr) ? -p.R[r] : 0.f;
    bool ok = true;
    constexpr int CH = BN / 32 / kPartsK;
    const int total = p.ntiles * CH;
    const int c_base = part * CH;
    auto issue = [&](int g, uint32_t (&rg)[32]) -> bool {
      const int j = g / CH, c = g % CH, buf = j % NSW;
      if (c == 0) {
        if (!mbar_wait(bar(S_FULL + buf), (j / NSW) & 1, abort_flag)) return false;
        __syncwarp();
        tc_fence_after();
      }
      tmem_ld32_nowait(lane_addr + buf * BUFCOLS + (c_base + c) * 32, rg);
      return true;
    };
    // Scores of chunk g have landed in rg: turn them into weights, store them back over the scores.
    auto weigh = [&](int g, uint32_t (&rg)[32]) {
      const int j = g / CH, c = g % CH, buf = j % NSW;
      const uint32_t taddr = lane_addr + buf * BUFCOLS + (c_base + c) * 32;
      float e[32];
      if (MAT5) tmem_ld32(taddr + WCOLS, e);  // E = rows2 . cols of the same entries
      float v[32];
      if (SPLIT) {
        float lo[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float w = ex2(fmaf(__uint_as_float(rg[i]), scale, negR));
          if (MAT5) w *= e[i];
          const float hi = round_tf32_pos(w);
          lo[i] = round_tf32_pos(w - hi);
          v[i] = hi;
        }
        tmem_st32(taddr + BN, lo);
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float w = ex2(fmaf(__uint_as_float(rg[i]), scale, negR));
          if (MAT5) w *= e[i];
          v[i] = round_tf32_pos(w);
        }
      }
      tmem_st32(taddr, v);
      if (c == CH - 1) {  // this warp's share of the tile is written: tell the MMA lane
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(W_FULL + buf));
      }
    };
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
    // `ok` is warp-uniform. tcgen05.ld is .sync.aligned: rows beyond nr load too, only their stores are masked.
    if (ok) {
      const bool valid = r < p.nr;
      const int rr = valid ? r : 0;
      const float inv_eps = 1.0f / p.eps;
      float fac;
      if (p.epilogue == PV_GRAD) {
        fac = p.coef * (p.gs ? __ldg(p.gs) : 1.f) * __ldg(p.roww + rr);
      } else {
        const float rt = (__ldg(p.rowpot + rr) * inv_eps + (p.rowlogw ? __ldg(p.rowlogw + rr) : 0.f)) * kLog2e;
        fac = p.coef * ex2(rt - negR);
      }
      float* orow = p.out + (size_t)rr * p.ld_out + p.dv0;
#pragma unroll 1
      for (int c = part; c < p.dv_pad / 32; c += kPartsK) {  // the warpgroups split the output chunks
        float o[32];
        tmem_ld32(lane_addr + NSW * BUFCOLS + c * 32, o);
        if (valid) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int col = c * 32 + i;
            if (p.dv0 + col < p.dv) {
              float val = o[i];
              if (p.epilogue == PV_GRAD) val = __ldg(p.rows_raw + (size_t)rr * p.ld_rows + p.dv0 + col) - val;
              orow[col] = fac * val;
            }
          }
        }
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
  if (tid == 0 && *abort_flag) atomicExch(&g_tck_error, 1);
}

// W = 2^(scale2 * S - R_row), rounded to TF32, written over the scores (pitch ld). In split mode the row holds
// [Wh | Wl | Wh] in three blocks of cols_pad columns, which the GEMM pairs with [Vh | Vh | Vl]. Columns beyond
// nc get zero weight without looking at the stored value.
__global__ void wexp_kernel(float* __restrict__ W, long long ld, int rows, int row0, int nc, int cols_pad,
                            const float* __restrict__ R, float scale2, int split, const int* skip) {
  if (skip && *skip) return;
  const int quads = cols_pad >> 2;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)rows * quads) return;
  const int r = (int)(idx / quads), j4 = (int)(idx - (long long)r * quads);
  float* row = W + (size_t)r * ld;
  const float negR = -__ldg(R + row0 + r);
  const float4 s = *reinterpret_cast<const float4*>(row + 4 * j4);
  const float sv[4] = {s.x, s.y, s.z, s.w};
  float hi[4], lo[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float w = (4 * j4 + e < nc) ? ex2(fmaf(sv[e], scale2, negR)) : 0.f;
    hi[e] = round_tf32_pos(w);
    lo[e] = round_tf32_pos(w - hi[e]);
  }
  const float4 h4 = make_float4(hi[0], hi[1], hi[2], hi[3]);
  *reinterpret_cast<float4*>(row + 4 * j4) = h4;
  if (split) {
    *reinterpret_cast<float4*>(row + cols_pad + 4 * j4) = make_float4(lo[0], lo[1], lo[2], lo[3]);
    *reinterpret_cast<float4*>(row + 2 * (size_t)cols_pad + 4 * j4) = h4;
  }
}

// vt[c][part*cols_pad + j] = TF32 pieces of V[j][c] * colscale_j, zero beyond (dv, nc): parts [Vh] (TF32 mode) or
// [Vh | Vh | Vl] (split mode). 32 x 32 tiles through shared memory so that both sides are coalesced.
__global__ void stage_vt_cat_kernel(const float* __restrict__ V, int nc, int dv, const float* __restrict__ colscale,
                                    int dv_rows, int cols_pad, int split, float* __restrict__ vt) {
  __shared__ float tile[32][33];
  const int j0 = blockIdx.x * 32, c0 = blockIdx.y * 32;
  const int tx = threadIdx.x, ty = threadIdx.y;  // 32 x 8
  for (int i = ty; i < 32; i += 8) {
    const int j = j0 + i, c = c0 + tx;
    float v = 0.f;
    if (j < nc && c < dv) {
      v = V[(size_t)j * dv + c];
      if (colscale) v *= colscale[j];
    }
    tile[i][tx] = v;
  }
  __syncthreads();
  const size_t ld = (size_t)cols_pad * (split ? 3 : 1);
  for (int i = ty; i < 32; i += 8) {
    const int c = c0 + i, j = j0 + tx;
    if (c >= dv_rows || j >= cols_pad) continue;
    const float v = tile[tx][i];
    const float hi = to_tf32(v);
    float* row = vt + (size_t)c * ld;
    row[j] = hi;
    if (split) {
      row[cols_pad + j] = hi;
      row[2 * (size_t)cols_pad + j] = to_tf32(v - hi);
    }
  }
}

__global__ void pad_vec_kernel(const float* __restrict__ v, int nc, int cols_pad, float* __restrict__ out,
                               const int* skip) {
  if (skip && *skip) return;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < cols_pad) out[i] = (i < nc) ? v[i] : 0.f;
}

// ------------------------------------------------------------------ host side
struct KPlan {
  int nhalf, bn, nbuf, nstage;
  size_t smem;
};

// Tile shape by contraction length: long contractions take 256 x 256 tiles with a single accumulator per half
// (the epilogue of a tile is a few per cent of its MMA time there), shorter ones 256 x 128 tiles with two
// accumulators per half so that the epilogue of one tile overlaps the MMAs of the next. `ncols` caps the tile
// width for narrow outputs.
std::atomic<int> g_wide_min_chunks{24};

KPlan plan_k(int nk, int ncols) {
  KPlan k{};
  k.nhalf = 2;
  const bool wide = nk >= g_wide_min_chunks.load(std::memory_order_relaxed) && ncols > 128;
  k.bn = wide ? 256 : 128;
  k.nbuf = wide ? 1 : 2;
  const size_t stage = (size_t)(k.nhalf * 128 + k.bn) * 128;
  k.nstage = (int)((kSmemMax - 4096) / stage);
  if (k.nstage > 6) k.nstage = 6;
  k.smem = k.nstage * stage + 4096;
  if (k.smem < (size_t)kSmemMin) k.smem = kSmemMin;
  return k;
}

template <int NHALF, int BN, int NBUF, int EPI>
cudaError_t launch_k(const CUtensorMap& ma, const CUtensorMap& mb, const KParams& kp, int grid, size_t smem,
                     cudaStream_t st) {
  auto kern = tck_kernel<NHALF, BN, NBUF, EPI>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemMax);
  if (e != cudaSuccess) return e;
  kern<<<grid, 128 + 128 * NHALF * kPartsK, smem, st>>>(ma, mb, kp);
  return cudaGetLastError();
}

template <int EPI>
cudaError_t launch_plan(const KPlan& k, const CUtensorMap& ma, const CUtensorMap& mb, const KParams& kp, int grid,
                        cudaStream_t st) {
  if (k.bn == 256) return launch_k<2, 256, 1, EPI>(ma, mb, kp, grid, k.smem, st);
  return launch_k<2, 128, 2, EPI>(ma, mb, kp, grid, k.smem, st);
}

// Operand maps (32-float K chunks, 128-byte swizzle) and the chunk counts of a contraction of kp floats.
bool make_maps(CUtensorMap* ma, CUtensorMap* mb, const float* A, long long rowsA, const float* B, long long rowsB,
               long long kp, int bn) {
  return detail::encode_map(ma, A, rowsA, kp, 32, 128, CU_TENSOR_MAP_SWIZZLE_128B) &&
         detail::encode_map(mb, B, rowsB, kp, 32, bn, CU_TENSOR_MAP_SWIZZLE_128B);
}

void set_chunks(KParams& kp, long long k_floats) {
  kp.nk = (int)((k_floats + 31) / 32);
  const int rem = (int)(k_floats - 32ll * (kp.nk - 1));  // 8..32, a multiple of 8
  kp.klast = (rem + 7) / 8;
}

}  // namespace

int set_wide_tile_min_chunks(int k) {
  if (k < 1) k = 1;
  return g_wide_min_chunks.exchange(k, std::memory_order_relaxed);
}

cudaError_t kstream_lse(const Staged& s, int side, const StreamArgs& a, const LseEpilogue& e, float* s_out,
                        long long ld_s, cudaStream_t st) {
  const CloudOps& rowc = s.cloud[side == 0 ? 0 : 1];
  const CloudOps& colc = s.cloud[side == 0 ? 1 : 0];
  const float scale2 = (2.0f * a.cost_scale) * (1.0f / a.eps) * kLog2e;
  detail::launch_bias(colc, s.kc, s.kp, a.pot, a.logw, 1.0f / a.eps, 1.0f / scale2, e.ctrl, st, a.pot_shard,
                      a.pot_stride);
  KParams kp{};
  set_chunks(kp, s.kp);
  const KPlan k = plan_k(kp.nk, a.nc);
  CUtensorMap ma, mb;
  if (!make_maps(&ma, &mb, rowc.opA, rowc.rows_pad, colc.opB, colc.rows_pad, s.kp, k.bn)) return cudaErrorInvalidValue;
  kp.nr = a.nr; kp.nc = a.nc; kp.row_begin = a.row_begin;
  kp.ntiles = (a.nc + k.bn - 1) / k.bn;
  kp.nstage = k.nstage;
  kp.scale2 = scale2; kp.eps = a.eps; kp.ep = e;
  const int bm = 128 * k.nhalf;
  kp.nblk = (a.nr - a.row_begin + bm - 1) / bm;
  if (kp.nblk <= 0) return cudaSuccess;
  kp.part_m = s.part_m[side]; kp.part_s = s.part_s[side]; kp.part_stride = s.part_stride; kp.tickets = s.tickets[side];
  kp.s_out = s_out; kp.ld_s = ld_s;
  return launch_plan<EPI_LSE>(k, ma, mb, kp, detail::pick_ctas(kp.nblk, kp.ntiles), st);
}

cudaError_t kstream_vec(const Staged& s, int side, const StreamArgs& a, const PvArgs& pa, char* scratch,
                        cudaStream_t st) {
  if (!scratch || !pa.R || !pa.V || !pa.out) return cudaErrorInvalidValue;
  const CloudOps& rowc = s.cloud[side == 0 ? 0 : 1];
  const CloudOps& colc = s.cloud[side == 0 ? 1 : 0];
  const float scale2 = (2.0f * a.cost_scale) * (1.0f / a.eps) * kLog2e;
  detail::launch_bias(colc, s.kc, s.kp, a.pot, a.logw, 1.0f / a.eps, 1.0f / scale2, nullptr, st);
  float* vpad = reinterpret_cast<float*>(((uintptr_t)scratch + 255) & ~(uintptr_t)255);
  pad_vec_kernel<<<(colc.rows_pad + 255) / 256, 256, 0, st>>>(pa.V, a.nc, colc.rows_pad, vpad, pa.skip);
  KParams kp{};
  set_chunks(kp, s.kp);
  const KPlan k = plan_k(kp.nk, a.nc);
  CUtensorMap ma, mb;
  if (!make_maps(&ma, &mb, rowc.opA, rowc.rows_pad, colc.opB, colc.rows_pad, s.kp, k.bn)) return cudaErrorInvalidValue;
  kp.nr = a.nr; kp.nc = a.nc; kp.row_begin = a.row_begin;
  kp.ntiles = (a.nc + k.bn - 1) / k.bn;
  kp.nstage = k.nstage;
  kp.scale2 = scale2; kp.eps = a.eps;
  const int bm = 128 * k.nhalf;
  kp.nblk = (a.nr - a.row_begin + bm - 1) / bm;
  if (kp.nblk <= 0) return cudaSuccess;
  kp.part_m = s.part_m[side]; kp.part_s = s.part_s[side]; kp.part_stride = s.part_stride; kp.tickets = s.tickets[side];
  kp.R = pa.R; kp.vpad = vpad; kp.rowpot = pa.rowpot; kp.rowlogw = pa.rowlogw; kp.vout = pa.out; kp.skip = pa.skip;
  return launch_plan<EPI_VEC>(k, ma, mb, kp, detail::pick_ctas(kp.nblk, kp.ntiles), st);
}

// ---- narrow plan-times-matrix pass (second GEMM from TMEM) -------------------------------------------
namespace {

// Second row operand of the Mat5 term in the row-role layout of the staged clouds: [Ah | Ah | Al | 0 ...] in the
// split mode, [Ah | 0 ...] in TF32 mode, so that its contraction with the staged column operand is A_i . y_j
// (the bias and label columns of the column operand meet zeros).
__global__ void stage_rows2_kernel(const float* __restrict__ A, int rows, int rows_pad, int d, int kp, int split,
                                   float* __restrict__ out) {
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (size_t)rows_pad * kp) return;
  const int r = (int)(idx / kp), k = (int)(idx % kp);
  float v = 0.f;
  if (r < rows && k < (split ? 3 * d : d)) {
    const float a = A[(size_t)r * d + k % d];
    const float hi = to_tf32(a);
    v = (split && k / d == 2) ? to_tf32(a - hi) : hi;
  }
  out[idx] = v;
}

struct KPvPlan {
  int dv_pad, nslices, vrows, cols_pad, parts, nstage, nv;
  long long ld_v;
  size_t vt_bytes, a2_bytes, smem;
  bool ok;
};

KPvPlan plan_kpv(int nr, int nc, int kp, int dv, int prec, bool mat5) {
  KPvPlan k{};
  const bool split = prec == 1;
  const int w = dv < 128 ? dv : 128;
  k.dv_pad = (w + 31) & ~31;
  k.nslices = (dv + 127) / 128;
  k.vrows = k.nslices * k.dv_pad;
  k.cols_pad = detail::pad256(nc);
  k.parts = split ? 3 : 1;
  k.ld_v = (long long)k.cols_pad * k.parts;
  k.vt_bytes = (((size_t)k.vrows * k.ld_v * sizeof(float)) + 1023) & ~size_t(1023);
  k.a2_bytes = mat5 ? ((((size_t)detail::pad256(nr) * kp * sizeof(float)) + 1023) & ~size_t(1023)) : 0;
  const size_t stage = (size_t)(mat5 ? 2 : 1) * 128 * 128 + 64 * 128;
  const size_t v_stage = (size_t)(split ? 2 : 1) * 2 * k.dv_pad * 128;
  const size_t budget = kSmemMax - 2048;
  k.nv = (2 * v_stage + 2 * stage <= budget) ? 2 : 1;
  const size_t rest = budget - k.nv * v_stage;
  k.nstage = (int)(rest / stage);
  if (k.nstage > 4) k.nstage = 4;
  k.ok = k.nstage >= 2;
  k.smem = k.nv * v_stage + k.nstage * stage + 2048;
  if (k.smem < (size_t)kSmemMin) k.smem = kSmemMin;
  return k;
}

template <bool SPLIT, bool MAT5>
cudaError_t launch_kpv(const CUtensorMap* maps, const KPvParams& kp, int grid, size_t smem, cudaStream_t st) {
  auto kern = tck_pv_kernel<SPLIT, MAT5>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemMax);
  if (e != cudaSuccess) return e;
  kern<<<grid, 128 + 128 * kPartsK, smem, st>>>(maps[0], maps[1], maps[2], maps[3], maps[4], kp);
  return cudaGetLastError();
}

}  // namespace

size_t kstream_pv_scratch(int nr, int nc, int kp, int dv, int prec, bool mat5) {
  const KPvPlan k = plan_kpv(nr, nc, kp, dv, prec, mat5);
  return k.ok ? k.vt_bytes + k.a2_bytes + 2048 : 0;
}

cudaError_t kstream_pv(const Staged& s, int side, const StreamArgs& a, const PvArgs& pa, char* scratch,
                       size_t scratch_bytes, cudaStream_t st) {
  if (!scratch || !pa.R || !pa.V || !pa.out) return cudaErrorInvalidValue;
  const CloudOps& rowc = s.cloud[side == 0 ? 0 : 1];
  const CloudOps& colc = s.cloud[side == 0 ? 1 : 0];
  const bool mat5 = pa.rows2 != nullptr, split = s.prec == 1;
  const KPvPlan k = plan_kpv(rowc.rows, a.nc, s.kp, pa.dv, s.prec, mat5);
  if (!k.ok) return cudaErrorNotSupported;
  if (k.vt_bytes + k.a2_bytes + 2048 > scratch_bytes) return cudaErrorInvalidValue;
  const float scale2 = (2.0f * a.cost_scale) * (1.0f / a.eps) * kLog2e;
  detail::launch_bias(colc, s.kc, s.kp, a.pot, a.logw, 1.0f / a.eps, 1.0f / scale2, nullptr, st, a.pot_shard,
                      a.pot_stride);
  char* p0 = (char*)(((uintptr_t)scratch + 1023) & ~(uintptr_t)1023);
  float* vt = reinterpret_cast<float*>(p0);
  float* a2 = mat5 ? reinterpret_cast<float*>(p0 + k.vt_bytes) : nullptr;
  {
    dim3 grid((k.cols_pad + 31) / 32, (k.vrows + 31) / 32), block(32, 8);
    stage_vt_cat_kernel<<<grid, block, 0, st>>>(pa.V, a.nc, pa.dv, pa.colscale, k.vrows, k.cols_pad, split, vt);
  }
  if (mat5) {
    const size_t total = (size_t)rowc.rows_pad * s.kp;
    stage_rows2_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(pa.rows2, rowc.rows, rowc.rows_pad, s.d, s.kp,
                                                                        split, a2);
  }
  CUtensorMap maps[5];
  bool ok = true;
  ok &= detail::encode_map(&maps[0], rowc.opA, rowc.rows_pad, s.kp, 32, 128, CU_TENSOR_MAP_SWIZZLE_128B);
  ok &= detail::encode_map(&maps[1], mat5 ? a2 : rowc.opA, rowc.rows_pad, s.kp, 32, 128, CU_TENSOR_MAP_SWIZZLE_128B);
  ok &= detail::encode_map(&maps[2], colc.opB, colc.rows_pad, s.kp, 32, 64, CU_TENSOR_MAP_SWIZZLE_128B);
  ok &= detail::encode_map(&maps[3], vt, k.vrows, k.cols_pad, 32, k.dv_pad, CU_TENSOR_MAP_SWIZZLE_128B, k.ld_v);
  ok &= detail::encode_map(&maps[4], split ? vt + 2 * (size_t)k.cols_pad : vt, k.vrows, k.cols_pad, 32, k.dv_pad,
                           CU_TENSOR_MAP_SWIZZLE_128B, k.ld_v);
  if (!ok) return cudaErrorInvalidValue;
  KPvParams kp{};
  kp.nr = a.nr; kp.nc = a.nc; kp.row_begin = a.row_begin;
  kp.ntiles = (a.nc + 63) / 64;
  KParams chunks{};
  set_chunks(chunks, s.kp);
  kp.nk = chunks.nk; kp.klast = chunks.klast; kp.nstage = k.nstage; kp.nv = k.nv;
  kp.dv = pa.dv; kp.dv_pad = k.dv_pad; kp.ld_out = pa.dv;
  kp.scale2 = scale2; kp.eps = a.eps; kp.R = pa.R; kp.epilogue = pa.epilogue;
  kp.rowpot = pa.rowpot; kp.rowlogw = pa.rowlogw; kp.roww = pa.roww; kp.gs = pa.gs; kp.coef = pa.coef;
  kp.rows_raw = a.rows; kp.ld_rows = a.d; kp.out = pa.out; kp.skip = pa.skip;
  const int grid = (a.nr - a.row_begin + 127) / 128;
  if (grid <= 0) return cudaSuccess;
  for (int sl = 0; sl < k.nslices; ++sl) {
    kp.dv0 = sl * k.dv_pad;
    cudaError_t e;
    if (mat5) e = split ? launch_kpv<true, true>(maps, kp, grid, k.smem, st) : launch_kpv<false, true>(maps, kp, grid, k.smem, st);
    else e = split ? launch_kpv<true, false>(maps, kp, grid, k.smem, st) : launch_kpv<false, false>(maps, kp, grid, k.smem, st);
    if (e != cudaSuccess) return e;
  }
  return cudaSuccess;
}

// ---- wide plan-times-matrix pass -------------------------------------------------------------------
namespace {
constexpr size_t kWeightCap = size_t(2) << 30;  // bytes of score / weight scratch per chunk of rows

struct MatPlan {
  int cols_pad, parts, dv_rows, rows_chunk;
  long long k2;                 // contraction length of the second GEMM (floats)
  size_t vt_bytes, w_bytes;
};

MatPlan plan_mat(int nr, int nc, int dv, int prec) {
  MatPlan m{};
  m.cols_pad = detail::pad256(nc);
  m.parts = prec == 1 ? 3 : 1;
  m.k2 = (long long)m.cols_pad * m.parts;
  m.dv_rows = detail::pad256(dv);
  m.vt_bytes = (((size_t)m.dv_rows * m.k2 * sizeof(float)) + 1023) & ~size_t(1023);
  const size_t row_bytes = (size_t)m.k2 * sizeof(float);
  long long rc = (long long)(kWeightCap / row_bytes) & ~255ll;
  if (rc < 256) rc = 256;
  if (rc > detail::pad256(nr)) rc = detail::pad256(nr);
  m.rows_chunk = (int)rc;
  m.w_bytes = (((size_t)m.rows_chunk * row_bytes) + 1023) & ~size_t(1023);
  return m;
}
}  // namespace

bool kstream_mat_supported(int dv) { return dv >= 256; }

size_t kstream_mat_scratch(int nr, int nc, int dv, int prec) {
  const MatPlan m = plan_mat(nr, nc, dv, prec);
  return m.vt_bytes + m.w_bytes + 2048;
}

cudaError_t kstream_mat(const Staged& s, int side, const StreamArgs& a, const PvArgs& pa, float* R_out,
                        char* scratch, size_t scratch_bytes, cudaStream_t st) {
  if (!scratch || !R_out || !pa.V || !pa.out || pa.rows2) return cudaErrorInvalidValue;
  const MatPlan m = plan_mat(a.nr - a.row_begin, a.nc, pa.dv, s.prec);
  if (m.vt_bytes + m.w_bytes + 2048 > scratch_bytes) return cudaErrorInvalidValue;
  char* p0 = (char*)(((uintptr_t)scratch + 1023) & ~(uintptr_t)1023);
  float* vt = reinterpret_cast<float*>(p0);
  float* W = reinterpret_cast<float*>(p0 + m.vt_bytes);
  const float scale2 = (2.0f * a.cost_scale) * (1.0f / a.eps) * kLog2e;
  {
    dim3 grid((m.cols_pad + 31) / 32, (m.dv_rows + 31) / 32), block(32, 8);
    stage_vt_cat_kernel<<<grid, block, 0, st>>>(pa.V, a.nc, pa.dv, pa.colscale, m.dv_rows, m.cols_pad, m.parts == 3,
                                                vt);
  }
  KParams g2{};
  set_chunks(g2, m.k2);
  const KPlan k2 = plan_k(g2.nk, pa.dv);
  CUtensorMap ma2, mb2;
  if (!make_maps(&ma2, &mb2, W, m.rows_chunk, vt, m.dv_rows, m.k2, k2.bn)) return cudaErrorInvalidValue;
  for (int r0 = a.row_begin; r0 < a.nr; r0 += m.rows_chunk) {
    const int r1 = (a.nr - r0 > m.rows_chunk) ? r0 + m.rows_chunk : a.nr;
    // 1. soft-min pass over rows [r0, r1): normalisers to R_out, raw scores to W
    StreamArgs ac = a;
    ac.row_begin = r0; ac.nr = r1;
    LseEpilogue ep;
    ep.lse2 = R_out;
    cudaError_t e = kstream_lse(s, side, ac, ep, W, m.k2, st);
    if (e != cudaSuccess) return e;
    // 2. scores -> TF32 weights in place
    const long long quads = (long long)(r1 - r0) * (m.cols_pad / 4);
    wexp_kernel<<<(unsigned)((quads + 255) / 256), 256, 0, st>>>(W, m.k2, r1 - r0, r0, a.nc, m.cols_pad, R_out, scale2,
                                                                 m.parts == 3, pa.skip);
    // 3. out[r0:r1] = epilogue(W x Vt^T)
    g2.nr = r1 - r0; g2.nc = pa.dv; g2.row_begin = 0;
    g2.ntiles = (pa.dv + k2.bn - 1) / k2.bn;
    g2.nstage = k2.nstage;
    g2.scale2 = scale2; g2.eps = a.eps;
    g2.nblk = (g2.nr + 128 * k2.nhalf - 1) / (128 * k2.nhalf);
    g2.R = R_out; g2.rowpot = pa.rowpot; g2.rowlogw = pa.rowlogw; g2.skip = pa.skip;
    g2.epilogue = pa.epilogue; g2.out_row0 = r0; g2.dv = pa.dv; g2.ld_out = pa.dv; g2.out = pa.out;
    g2.roww = pa.roww; g2.gs = pa.gs; g2.coef = pa.coef; g2.rows_raw = a.rows; g2.ld_rows = a.d;
    e = launch_plan<EPI_OUT>(k2, ma2, mb2, g2, detail::pick_ctas(g2.nblk, g2.ntiles), st);
    if (e != cudaSuccess) return e;
  }
  return cudaGetLastError();
}

int clear_error_flag_k() {
  const int zero = 0;
  return cudaMemcpyToSymbol(g_tck_error, &zero, sizeof(int)) == cudaSuccess ? 0 : -1;
}

int read_error_flag_k() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_tck_error, sizeof(int)) != cudaSuccess) return -1;
  return v;
}

}  // namespace tc
}  // namespace fs
