// What a batch of eight tcgen05.mma instructions costs the warp that issues it, in the forms the
// kernels of this package use and in the ones they avoid (sm_100a).  One CTA an SM; the issuing warp
// is warp 1; every figure is clocks per batch (M128 N128 K16 products, a commit after each batch),
// taken from CTA 0.  Run through `python -m qorvix_b200.issue_bench`.
//
//   FORM   0: the loop under `if (lane == 0)`            1: all lanes walk the loop, an elected lane issues
//   WAITS  barrier waits (on a barrier that has long flipped) before each batch
//   MIX    0: SS products only   1: SS batches and TS batches (A from tensor memory, B MN-major) in turn
//   BESIDE 0: nothing   1: sixteen warps polling a barrier   2: eight warps of back-to-back FMAs
//          3: eight warps of back-to-back ex2 (two a scheduler in 2 and 3)
// and, separately, the time from the first issue of a batch to its completion after the tensor pipe
// has idled for a given number of clocks.
#include <cstdio>
#include <cstdlib>
#include "../tc_common.cuh"

namespace {

template <int FORM, int WAITS, int MIX, int BESIDE>
__global__ void __launch_bounds__(640) issue_kernel(long long* out, int iters, int idle, int* err) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t bars[8];
  __shared__ uint32_t slot;
  __shared__ int stop;
  if (threadIdx.x == 0) {
    for (int i = 0; i < 8; ++i) mbar_init(&bars[i], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    mbar_arrive(&bars[7]);                         // bars[7]: phase 0 complete for good
    stop = 0;
  }
  const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&slot)), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  for (int i = threadIdx.x; i < 160 * 1024 / 4; i += blockDim.x) ((uint32_t*)base)[i] = 0;
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = slot;
  if (warp == 1 && (FORM == 1 || lane == 0)) {
    const bool leader = FORM == 1 ? elect_one() : true;
    constexpr uint32_t idesc_ss = umma_idesc(128, 128, 0);
    constexpr uint32_t idesc_ts = umma_idesc(128, 128, 1);
    long long issue = 0, whole = 0;
    const long long t_begin = clock64();
    for (int it = 0; it < iters; ++it) {
      const int s = it % 3;                        // operands from a ring of three stages, as in the kernels
      const bool ts_batch = MIX == 1 && (it & 1);
      for (int w = 0; w < WAITS; ++w) mbar_wait(&bars[7], 0, err, 2);
      tc_fence_after();
      const long long t0 = clock64();
      if (leader) {
        if (ts_batch) {
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            umma_f16_ts(tmem + 256, tmem + (uint32_t)(kk * 8), umma_desc_mn(smem_u32(base + 65536 + s * 32768 + kk * 2048), 16384), idesc_ts, 1u);
        } else {
#pragma unroll
          for (int hf = 0; hf < 2; ++hf) {
            const uint64_t da = umma_desc(smem_u32(base + hf * 16384));
            const uint64_t db = umma_desc(smem_u32(base + 32768 + s * 32768 + hf * 16384));
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) umma_f16(tmem + (uint32_t)((it & 2) * 64), da + 2 * kk, db + 2 * kk, idesc_ss, (hf > 0 || kk > 0) ? 1u : 0u);
          }
        }
        umma_commit(&bars[0]);
      }
      if (FORM == 1) __syncwarp();
      if (idle >= 0) {                             // the batch's completion, then a pause with the pipe empty
        const long long t1 = clock64();
        mbar_wait(&bars[0], (uint32_t)(it & 1), err, 1);
        const long long t2 = clock64();
        issue += t1 - t0;
        whole += t2 - t0;
        while (clock64() - t2 < idle) { }
      }
    }
    const long long t_end = clock64();
    if (idle < 0) {
      if (leader) umma_commit(&bars[6]);
      if (FORM == 1) __syncwarp();
      mbar_wait(&bars[6], 0, err, 1);
    }
    if (lane == 0) {
      out[blockIdx.x * 4] = t_end - t_begin;
      out[blockIdx.x * 4 + 1] = issue;
      out[blockIdx.x * 4 + 2] = whole;
      *(volatile int*)&stop = 1;
    }
  } else if (BESIDE == 1 && warp >= 4) {
    bool got = false;
    for (uint32_t i = 0; i < (1u << 24) && !got && !*(volatile int*)&stop; ++i) got = mbar_try_wait(&bars[5], 0);
  } else if (BESIDE >= 2 && warp >= 4 && warp < 12) {
    float v[16];
#pragma unroll
    for (int u = 0; u < 16; ++u) v[u] = -0.001f * (float)(threadIdx.x + u);
    for (int i = 0; i < (1 << 20) && !*(volatile int*)&stop; ++i) {
#pragma unroll
      for (int rep = 0; rep < 8; ++rep) {
#pragma unroll
        for (int u = 0; u < 16; ++u) {
          if (BESIDE == 2) v[u] = fmaf(v[u], 0.999f, -0.0001f);
          else { float e; asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(v[u])); v[u] = e - 1.0001f; }
        }
      }
    }
    float acc = 0.f;
#pragma unroll
    for (int u = 0; u < 16; ++u) acc += v[u];
    if (acc == 12345.f) out[3] = 1;               // keeps the loop alive
  }
  __syncthreads();
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
}

int failures = 0;

template <int FORM, int WAITS, int MIX, int BESIDE>
void run(const char* name, int idle = -1) {
  static long long* out = nullptr;
  static int* err = nullptr;
  if (!out) { cudaMalloc(&out, 148 * 32); cudaMalloc(&err, 4); }
  cudaMemset(err, 0, 4);
  auto kern = issue_kernel<FORM, WAITS, MIX, BESIDE>;
  cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
  const int iters = 500, threads = BESIDE ? 640 : 128;
  kern<<<148, threads, 200 * 1024>>>(out, 10, idle, err);
  kern<<<148, threads, 200 * 1024>>>(out, iters, idle, err);
  long long h[3];
  int e = 0;
  cudaMemcpy(h, out, sizeof(h), cudaMemcpyDeviceToHost);
  cudaMemcpy(&e, err, 4, cudaMemcpyDeviceToHost);
  const cudaError_t rc = cudaGetLastError();
  if (e || rc != cudaSuccess) ++failures;
  if (idle < 0) printf("%-78s %6.0f clocks a batch (wait code %d, %s)\n", name, (double)h[0] / iters, e, cudaGetErrorString(rc));
  else printf("%-58s idle %5d: issue %4.0f, issue to completion %4.0f clocks (wait code %d, %s)\n", name, idle, (double)h[1] / iters, (double)h[2] / iters, e, cudaGetErrorString(rc));
}

}  // namespace

int main() {
  run<0, 0, 0, 0>("lane-0 branch, SS batches");
  run<1, 0, 0, 0>("elected lane, SS batches");
  run<1, 0, 1, 0>("elected lane, SS and TS batches in turn");
  run<1, 2, 1, 0>("elected lane, SS and TS in turn, two satisfied waits a batch");
  run<0, 2, 1, 0>("lane-0 branch, SS and TS in turn, two satisfied waits a batch");
  run<1, 2, 1, 1>("elected lane, two waits, sixteen polling warps beside");
  run<0, 2, 1, 1>("lane-0 branch, two waits, sixteen polling warps beside");
  run<1, 2, 1, 2>("elected lane, two waits, eight warps of FMAs beside");
  run<1, 2, 1, 3>("elected lane, two waits, eight warps of ex2 beside");
  for (int idle : {0, 300, 1000, 5000}) run<1, 0, 0, 0>("elected lane, SS batch after the pipe idled", idle);
  for (int idle : {0, 300, 1000, 5000}) run<1, 0, 1, 0>("elected lane, SS / TS batch after the pipe idled", idle);
  return failures ? 1 : 0;
}
