// Shared device helpers: element types, conversions, deterministic reductions.
//
// Element type codes used by every extern "C" launcher: 0 = float, 1 = bfloat16.
// Reductions have a fixed shape (xor-shuffle tree inside a warp, then a serial
// sum over warps), so a result never depends on how many rows a launch holds.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define FT_DTYPE_F32 0
#define FT_DTYPE_BF16 1

#define FT_OK 0
#define FT_ERR_DTYPE -101
#define FT_ERR_SHAPE -102

// Run BODY with T bound to the element type named by CODE.
#define FT_DISPATCH(CODE, T, ...)                           \
  switch (CODE) {                                           \
    case FT_DTYPE_F32: { using T = float; __VA_ARGS__; } break;           \
    case FT_DTYPE_BF16: { using T = __nv_bfloat16; __VA_ARGS__; } break;  \
    default: return FT_ERR_DTYPE;                           \
  }

#define FT_LAUNCH_CHECK()                                  \
  do {                                                     \
    cudaError_t e__ = cudaGetLastError();                  \
    if (e__ != cudaSuccess) return (int)e__;               \
  } while (0)

namespace ft {

// Programmatic dependent launch: a kernel launched through launch_pdl() may
// become resident while the kernel before it in the stream is still running;
// pdl_wait() holds it until that kernel has completed and its writes are
// visible.  Every kernel launched this way calls pdl_wait() before it touches
// global memory.  (The reference wraps the same griddepcontrol instructions,
// python/freetoken/kernel/csrc/include/freetoken/utils.cuh:43-57.)
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                              cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

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

// Sum over the block; every thread gets the result.  `scratch` holds 33 floats.
// The order is fixed by blockDim alone.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();  // scratch may still be read from a previous call
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.f;
    for (int w = 0; w < nwarps; ++w) s += scratch[w];
    scratch[32] = s;
  }
  __syncthreads();
  return scratch[32];
}

}  // namespace ft
