// Micro-benchmarks that give the roofline its measured denominators on the box the bench runs on:
// the issue rate of ex2.approx (the transcendental pipe) alone, and of the soft-max inner loop
// (FFMA + ex2 + FADD + half a 3-input max per entry) with no memory traffic at all.
#include "../../include/flash_sinkhorn_b200.h"
#include "fs_tc.cuh"
#include <cuda_runtime.h>

namespace {

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm volatile("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}

// MODE 0: 8 independent ex2 chains per thread. MODE 1: the soft-max chunk loop on register data.
template <int MODE>
__global__ void micro_kernel(int iters, float seed, float* out) {
  float v[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = seed * (float)(i + 1) + (float)threadIdx.x * 1e-3f;
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f, m_run = -1e30f, off_run = -1e30f;
  const float scale = 1.0001f;
  for (int it = 0; it < iters; ++it) {
    if (MODE == 0) {
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = ex2(v[i] * 0.5f - 1.0f);  // one FFMA + one ex2 per value
    } else {
      float t[11];
#pragma unroll
      for (int i = 0; i < 10; ++i) t[i] = max3(v[3 * i], v[3 * i + 1], v[3 * i + 2]);
      t[10] = fmaxf(v[30], v[31]);
      float u0 = max3(t[0], t[1], t[2]), u1 = max3(t[3], t[4], t[5]), u2 = max3(t[6], t[7], t[8]);
      float cm = fmaxf(max3(u0, u1, u2), fmaxf(t[9], t[10]));
      float m_new = fmaxf(m_run, cm);
      float off_new = __fmul_rn(scale, m_new);
      float nms = -off_new;
      s0 = ((s0 + s1) + (s2 + s3)) * ex2(off_run - off_new);
      s1 = 0.f; s2 = 0.f; s3 = 0.f;
#pragma unroll
      for (int i = 0; i < 32; i += 4) {
        s0 += ex2(fmaf(v[i], scale, nms));
        s1 += ex2(fmaf(v[i + 1], scale, nms));
        s2 += ex2(fmaf(v[i + 2], scale, nms));
        s3 += ex2(fmaf(v[i + 3], scale, nms));
      }
      m_run = m_new; off_run = off_new;
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] += 1e-3f * s0;  // new "scores" next round (keeps the loop live)
    }
  }
  float acc = s0 + s1 + s2 + s3;
#pragma unroll
  for (int i = 0; i < 32; ++i) acc += v[i];
  if (acc == 123.456f) out[0] = acc;  // never true; defeats dead-code elimination
}

}  // namespace

// mode 0: ex2 alone; mode 1: soft-max inner loop. warps_per_sm in {4..32}. Returns ex2 evaluations per second
// (synchronises the device; diagnostic only).
extern "C" double fs_micro_exp_rate(int mode, int warps_per_sm) {
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -1.0;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (warps_per_sm < 1) warps_per_sm = 1;
  if (warps_per_sm > 32) warps_per_sm = 32;
  const int threads = warps_per_sm * 32, iters = 4096;
  float* out = nullptr;
  if (cudaMalloc(&out, 4) != cudaSuccess) return -1.0;
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0); cudaEventCreate(&e1);
  auto launch = [&]() {
    if (mode == 0) micro_kernel<0><<<sms, threads>>>(iters, 1e-3f, out);
    else micro_kernel<1><<<sms, threads>>>(iters, 1e-3f, out);
  };
  launch();
  cudaEventRecord(e0);
  launch();
  cudaEventRecord(e1);
  cudaEventSynchronize(e1);
  float ms = 0.f;
  cudaEventElapsedTime(&ms, e0, e1);
  cudaEventDestroy(e0); cudaEventDestroy(e1);
  cudaFree(out);
  if (cudaGetLastError() != cudaSuccess || ms <= 0.f) return -1.0;
  return (double)sms * threads * 32.0 * iters / (ms * 1e-3);
}

// Cycles per tensor-core instruction of the engine's shape family, measured on the current device.
extern "C" double fs_micro_mma_cycles(int n_cols, int a_in_tmem) {
  return fs::tc::micro_mma_cycles(n_cols, a_in_tmem != 0);
}

// See the header: SMs the streaming passes leave to concurrently running collectives.
extern "C" int fs_set_reserved_sms(int k) { return fs::tc::set_reserved_sms(k); }
