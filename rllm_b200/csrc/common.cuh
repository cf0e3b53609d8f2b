// Shared helpers of the sm_100a kernels: storage types, conversions, reductions,
// and the launcher conventions.
//
// Every exported launcher is `extern "C"`, takes raw device pointers, sizes and
// the CUDA stream to launch on, allocates nothing, and returns 0 or a negative
// code for a refused size / a positive cudaError_t of the launch. The Python
// side (rllm_b200/kernels/ops.py) checks shapes and dtypes before the call.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdlib.h>
#include <utility>

#define RLLM_API extern "C" __attribute__((visibility("default")))

namespace rllm {

enum : int { DT_F32 = 0, DT_BF16 = 1 };
enum : int { ERR_BAD_DTYPE = -1, ERR_BAD_SIZE = -2, ERR_BAD_ALIGN = -3, ERR_TOO_LARGE = -4 };

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(bf16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

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

// Sum over a block in a fixed order (warp tree, then warp 0 over the warp sums).
// `red` needs 32 floats of shared memory. All threads get the result.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float r = (lane < nwarps) ? red[lane] : 0.f;
  r = warp_sum(r);
  return r;
}
__device__ __forceinline__ float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float r = (lane < nwarps) ? red[lane] : -INFINITY;
  r = warp_max(r);
  return r;
}

static inline int launch_status() {
  cudaError_t e = cudaPeekAtLastError();
  if (e != cudaSuccess) { cudaGetLastError(); return (int)e; }
  return 0;
}

// ---- programmatic dependent launch
// Every kernel of this library starts with pdl_launch() (its successor in the stream may begin
// its own prologue) and calls pdl_wait() before it reads what its predecessor wrote or writes
// anything. Launched without the attribute both are no-ops. RLLM_B200_NO_PDL=1 turns the
// attribute off (plain stream order).
__device__ __forceinline__ void pdl_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

static inline bool pdl_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("RLLM_B200_NO_PDL");
    v = (e && e[0] == '1') ? 0 : 1;
  }
  return v != 0;
}

// More than 48 KB of dynamic shared memory has to be allowed per kernel, and the permission belongs to a
// device's copy of the kernel: `done` (one static array per kernel instantiation) remembers which devices
// have it. Returns 0 or -5.
template <typename K>
static inline int allow_dynamic_smem(K kernel, int bytes, bool (&done)[64]) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { cudaGetLastError(); return -5; }
  if (!done[dev]) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) {
      cudaGetLastError();
      return -5;
    }
    done[dev] = true;
  }
  return 0;
}

// Launch with the attributes this library uses: programmatic stream serialization, and a
// thread-block cluster of (1, 1, cluster_z) when cluster_z > 1.
template <typename... KArgs, typename... Args>
static inline int launch_ex(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s,
                            int cluster_z, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attrs[2];
  int n = 0;
  if (pdl_enabled()) {
    attrs[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  if (cluster_z > 1) {
    attrs[n].id = cudaLaunchAttributeClusterDimension;
    attrs[n].val.clusterDim.x = 1;
    attrs[n].val.clusterDim.y = 1;
    attrs[n].val.clusterDim.z = (unsigned)cluster_z;
    ++n;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = n;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
  if (e != cudaSuccess) { cudaGetLastError(); return (int)e; }
  return 0;
}

}  // namespace rllm
