// Shared helpers for the sm_100a kernels of this library.
//
// Every launcher is an `extern "C"` function that takes raw device pointers, sizes and a
// cudaStream_t and returns an int: 0 on success, a negative LLMIE_ERR_* code when the
// arguments are refused, or a positive cudaError_t from the launch. Launchers never
// allocate, never synchronise and never touch a stream other than the one they are given.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#define LLMIE_OK 0
#define LLMIE_ERR_BAD_ARG (-1)
#define LLMIE_ERR_UNSUPPORTED_SIZE (-2)
#define LLMIE_ERR_ALIGNMENT (-3)
#define LLMIE_ERR_DTYPE (-4)

// dtype codes shared with the Python wrappers
#define LLMIE_F32 0
#define LLMIE_BF16 1

#define LLMIE_LAUNCH_CHECK()                          \
  do {                                                \
    cudaError_t e__ = cudaGetLastError();             \
    if (e__ != cudaSuccess) return (int)e__;          \
  } while (0)

namespace llmie {

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
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

// Sum over a whole block; every thread gets the result. `scratch` holds 32 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n_warps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();  // scratch may still be read from an earlier call
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = (lane < n_warps) ? scratch[lane] : 0.f;
  return warp_sum(t);
}

// Loads 8 consecutive elements as floats. p must be 16-byte aligned for bf16, 32 for float.
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&out)[8]) {
  uint4 raw = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f = __bfloat1622float2(h[i]);
    out[2 * i] = f.x;
    out[2 * i + 1] = f.y;
  }
}
__device__ __forceinline__ void load8(const float* p, float (&out)[8]) {
  float4 a = *reinterpret_cast<const float4*>(p);
  float4 b = *reinterpret_cast<const float4*>(p + 4);
  out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w;
  out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&v)[8]) {
  uint4 raw;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = raw;
}
__device__ __forceinline__ void store8(float* p, const float (&v)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Programmatic dependent launch: a kernel launched through launch_k may begin while the kernel
// before it in the stream is still draining. Each such kernel calls pdl_launch_dependents() at
// its top (the next kernel may be scheduled) and pdl_wait() before it touches anything an
// earlier kernel wrote (the wait returns when all earlier kernels have completed and their
// writes are visible). What a kernel does before pdl_wait() - index arithmetic, loads of
// weights that no kernel writes - overlaps the previous kernel's tail. Both calls are no-ops
// in a kernel launched the ordinary way. llmie_set_pdl(0) turns the attribute off for this library's launches
// (each kernel library has its own copy of the switch).
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Asks the memory system to bring `bytes` (a multiple of 16, from a 16-byte aligned address) into
// L2. No register, no shared memory and no waiting on the issuing thread: a block can ask for all
// the weights it is going to stream, long before its loads of them, even before pdl_wait().
__device__ __forceinline__ void l2_prefetch(const void* p, unsigned bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}

static int g_pdl_on = 1;      // per library; llmie_set_pdl changes it
static inline bool pdl_enabled() { return g_pdl_on != 0; }

template <typename... KArgs, typename... Args>
static inline void launch_k(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                            Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  const bool pdl = pdl_enabled();
  cfg.attrs = pdl ? attr : nullptr;
  cfg.numAttrs = pdl ? 1 : 0;
  cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);   // errors surface in cudaGetLastError()
}

// The same for a kernel whose blocks form thread-block clusters of `cluster_x` along x (grid.x a multiple of it).
template <typename... KArgs, typename... Args>
static inline void launch_k_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                    unsigned cluster_x, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cluster_x;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace llmie

// Programmatic dependent launch on (1, the default) or off (0) for every launch of this library.
extern "C" void llmie_set_pdl(int on) { llmie::g_pdl_on = on ? 1 : 0; }
