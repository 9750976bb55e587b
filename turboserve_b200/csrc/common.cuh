// Shared helpers of the engine's CUDA sources (sm_100a).
//
// Every library exports plain C entry points: raw device pointers, sizes, a dtype code and
// a stream. An entry point returns 0 on success, a cudaError_t from the launch otherwise,
// or a negative code (TS_ERR_*) when it refuses its arguments; it never falls back.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define TS_EXPORT extern "C" __attribute__((visibility("default")))

enum : int { TS_F32 = 0, TS_BF16 = 1 };
enum : int {
  TS_ERR_DTYPE = -1,      // dtype code not known to this entry point
  TS_ERR_SIZE = -2,       // a size this kernel does not take
  TS_ERR_ALIGN = -3,      // a pointer or stride that is not aligned as the kernel needs
  TS_ERR_ARGUMENT = -4,   // any other refused argument
};

template <typename T> __device__ __forceinline__ float to_float(T v);
template <> __device__ __forceinline__ float to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) v += __shfl_xor_sync(0xffffffffu, v, offset);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1)
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, offset));
  return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result. `scratch` holds 33
// floats of shared memory. The order of additions is fixed by the thread index, so the sum
// of a row does not depend on what else the grid computes.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int num_warps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < num_warps ? scratch[lane] : 0.0f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// The gated feed-forward's activation, fp32: 0 silu, 1 gelu (erf), 2 gelu (tanh approximation).
// FAST (results that are rounded to bfloat16): silu with the hardware exponential and reciprocal,
// a few units in the last place of fp32 off, which bfloat16's eight bits never see; the
// precise form costs as many issue slots as the kernel's memory traffic takes time.
template <bool FAST = false>
__device__ __forceinline__ float activation(float x, int act) {
  if (act == 0) return FAST ? __fdividef(x, 1.0f + __expf(-x)) : x / (1.0f + expf(-x));
  if (act == 1) return 0.5f * x * (1.0f + erff(x * 0.70710678118654752440f));
  const float inner = 0.79788456080286535588f * (x + 0.044715f * x * x * x);
  return 0.5f * x * (1.0f + tanhf(inner));
}

static inline int ts_launch_status() { return (int)cudaGetLastError(); }

// Programmatic dependent launch.  Every kernel of the package is launched with the attribute
// that lets it be set up while the kernel before it in the stream is still draining, and every
// kernel calls pdl_wait() before it reads anything the kernel before it wrote, and before its
// own first write (every block does, so that "the kernel before has completed" holds along the
// whole chain).  What a kernel does before pdl_wait() (index arithmetic, barrier set-up,
// loading weights, which no step ever writes) may overlap the tail of its predecessor.
// TURBOSERVE_B200_PDL=0 switches the attribute off (pdl_wait() is then a no-op).
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// An explicit early trigger (griddepcontrol.launch_dependents right after a kernel's own
// pdl_wait(), which keeps at most one dependent kernel resident) pays where the dependent has
// work to do before its own wait, and costs where it has none or where the triggering kernel
// runs long.  Measured on B200 inside a captured decode step, 3.39 ms with no explicit trigger,
// one kind of kernel triggering at a time:
//   add + norm (dependents: the qkv and gate/up products, which fetch weights first)   3.33 ms
//   register-streaming products (dependents: element-wise kernels)                      3.37 ms
//   decode attention, register-fed kernel (dependent: the output projection)            3.39 ms
//     (the TMA-fed decode kernel does not trigger: 3.42 ms with, 3.21 ms without; triggering after
//     its last key tile, before the join of its parts, costs as much: 3.49 against 3.28 ms)
//   rotation + cache append (dependent: decode attention, launched as clusters)         3.76 ms
//     (with attention launched without clusters the same trigger costs 0.02 ms: it is the
//     early launch of a cluster kernel that is slow)
//   tcgen05 product (dependent: the down projection), after its wait or after its loop  4.54 to 4.67 ms
//     (the same whether or not the down projection fetches weights before its wait; no
//     penalty when the down projection is a library kernel, which is never launched early;
//     the same again with one thread of the dependent waiting and the others parked at a barrier)
//   every kernel, at its top or after its main loop                                     4.9 to 5.1 ms
// The first three together give 3.32 ms and are on by default (mask 2 + 8 + 32); a build with
// -DTS_EARLY_TRIGGER_MASK=<bits> chooses otherwise (0: none).
#ifndef TS_EARLY_TRIGGER_MASK
#define TS_EARLY_TRIGGER_MASK 42
#endif
// GROUP names the kind of kernel: 1 element-wise, 32 add + norm, 64 rotation + cache append, 2
// register-streaming product, 4 tcgen05 product, 8 attention, 16 the rest.
template <int GROUP = 16>
__device__ __forceinline__ void pdl_trigger() {
  if constexpr ((TS_EARLY_TRIGGER_MASK & GROUP) != 0) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

static inline bool ts_pdl_enabled() {
  static int enabled = -1;
  if (enabled < 0) {
    const char* env = getenv("TURBOSERVE_B200_PDL");
    enabled = (env && env[0] == '0') ? 0 : 1;
  }
  return enabled != 0;
}

// The same with the blocks grouped into thread-block clusters of cluster_x along x.
template <typename... KArgs, typename... Args>
static inline void ts_launch_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                     cudaStream_t stream, int cluster_x, Args&&... args) {
  cudaLaunchConfig_t config;
  memset(&config, 0, sizeof(config));
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attributes[2];
  memset(attributes, 0, sizeof(attributes));
  attributes[0].id = cudaLaunchAttributeClusterDimension;
  attributes[0].val.clusterDim.x = (unsigned)cluster_x;
  attributes[0].val.clusterDim.y = 1;
  attributes[0].val.clusterDim.z = 1;
  attributes[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attributes[1].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attributes;
  config.numAttrs = ts_pdl_enabled() ? 2 : 1;
  cudaLaunchKernelEx(&config, kernel, static_cast<KArgs>(args)...);
}

template <typename... KArgs, typename... Args>
static inline void ts_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                             cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t config;
  memset(&config, 0, sizeof(config));
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute;
  memset(&attribute, 0, sizeof(attribute));
  attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute.val.programmaticStreamSerializationAllowed = 1;
  config.attrs = &attribute;
  config.numAttrs = ts_pdl_enabled() ? 1 : 0;
  cudaLaunchKernelEx(&config, kernel, static_cast<KArgs>(args)...);
}
