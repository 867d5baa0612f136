// Shared helpers for the sm_100a kernels: element types, loads/stores through float,
// warp reductions with a fixed order, and the launch-error convention.
//
// Every entry point is `extern "C" int qv_*(..., void* stream)`: it launches on the given
// stream and returns cudaGetLastError() as an int (0 = launched), or a negative code of
// its own for arguments it refuses (the Python side turns both into exceptions).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <utility>

#define QV_DT_F32 0
#define QV_DT_BF16 1

// Refusals (never a wrong result): negative so they cannot be mistaken for cudaError_t.
#define QV_ERR_UNSUPPORTED (-2)   // a size or dtype this kernel does not take
#define QV_ERR_TOO_LARGE (-3)     // exceeds shared memory / grid limits

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_f(float v) { return v; }
__device__ __forceinline__ float to_f(bf16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum whose order depends only on blockDim (so only on the row length the
// launch was sized for), never on what else is in the batch.
__device__ __forceinline__ float block_sum(float v, float* red /* >= 33 floats */) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarp ? red[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}

static inline int qv_launch_status() { return (int)cudaGetLastError(); }

// Programmatic dependent launch: a kernel launched through qv_launch may be scheduled while the
// kernel before it in the stream is still running; it must call pdl_wait() before it reads or
// writes anything the earlier kernel touches, and what it does before that call (setting up
// barriers, fetching weights, which no kernel writes) overlaps the earlier kernel's tail.
// pdl_launch_dependents() lets the kernel after this one be scheduled likewise.  In a kernel
// launched the ordinary way both calls do nothing.  QORVIX_PDL=0 switches the attribute off.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

static inline bool qv_pdl_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("QORVIX_PDL");
    v = (e && e[0] == '0') ? 0 : 1;
  }
  return v != 0;
}

// As qv_launch, with the grid grouped into thread-block clusters of the given shape.
template <typename... KArgs, typename... Args>
static inline int qv_launch_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, dim3 cluster,
                                    Args&&... args) {
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  int n = 0;
  if (cluster.x * cluster.y * cluster.z > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = cluster.x;
    attr[n].val.clusterDim.y = cluster.y;
    attr[n].val.clusterDim.z = cluster.z;
    ++n;
  }
  if (qv_pdl_enabled()) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return (int)cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

template <typename... KArgs, typename... Args>
static inline int qv_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = qv_pdl_enabled() ? 1 : 0;
  return (int)cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

#define QV_DISPATCH_DT(dt, T, ...)                                   \
  do {                                                               \
    if ((dt) == QV_DT_F32) { typedef float T; __VA_ARGS__; }         \
    else if ((dt) == QV_DT_BF16) { typedef bf16 T; __VA_ARGS__; }    \
    else return QV_ERR_UNSUPPORTED;                                  \
  } while (0)
