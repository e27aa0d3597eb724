// Shared helpers of the hand-written sm_100a kernels: element types, loads/stores that widen
// to float, block reductions, and the launch-status convention of the exported C entry points.
//
// Every exported function is `extern "C"`, takes raw device pointers plus sizes and the CUDA
// stream as a `void*`, launches asynchronously on that stream and returns 0 on success or a
// negative code for a refused argument / a positive `cudaError_t` for a failed launch.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define PKV_EXPORT extern "C" __attribute__((visibility("default")))

// element type codes used across the C interface
#define PKV_F32 0
#define PKV_BF16 1

// refusal codes (negative so that they never collide with cudaError_t values)
#define PKV_ERR_DTYPE (-2)
#define PKV_ERR_SIZE (-3)
#define PKV_ERR_ALIGN (-4)
#define PKV_ERR_LIMIT (-5)

namespace pkv {

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_float<bf16>(float v) { return __float2bfloat16_rn(v); }

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

// Sum over a thread block (any multiple of 32 threads up to 1024). `scratch` holds 32 floats.
// The order of additions depends only on the block size, never on the data or the batch.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  const int nwarps = (blockDim.x + 31) >> 5;
  float total = (lane < nwarps) ? scratch[lane] : 0.0f;
  total = warp_sum(total);
  return total;
}

inline int launch_status() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : (int)e;
}

// Programmatic dependent launch. A kernel launched with `chained` may start while the kernel
// before it on the stream is still running, once every block of that kernel has called
// `dependents_may_launch()` (or has ended). It must call `wait_for_prior_kernels()` before it
// reads anything an earlier kernel writes and before it writes anything at all; the call returns
// when the kernel before it has finished and its writes are visible. Because every chained
// kernel waits in this way, a kernel that has passed its wait knows that all earlier work on
// the stream has finished, not only its direct predecessor. Kernels call both at their top
// (the calls do nothing in a kernel launched the ordinary way); only what is constant during a
// step (weights) may be touched before the wait.
#ifdef PKV_TRACE
// Development aid (-DPKV_TRACE): the first thread of every kernel notes the global nanosecond
// timer when it passes `dependents_may_launch()` (what = 0) and when its dependency wait returns
// (what = 1), in a ring that each library keeps; `pkv_trace_read` copies the ring out. The time
// at which a kernel's wait returns is also the time at which the kernel before it had finished.
struct TraceRecord {
  unsigned long long t;
  int what, grid, block, pad;
};
static __device__ TraceRecord trace_ring[8192];
static __device__ unsigned int trace_count;
__device__ __forceinline__ void trace_note(int what) {
  if ((blockIdx.x | blockIdx.y | blockIdx.z | threadIdx.x) == 0) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    const unsigned int i = atomicAdd(&trace_count, 1u) & 8191u;
    trace_ring[i].t = t;
    trace_ring[i].what = what;
    trace_ring[i].grid = (int)(gridDim.x * gridDim.y * gridDim.z);
    trace_ring[i].block = (int)blockDim.x;
  }
}
// the same from the first thread of every block (what >= 16; with -DPKV_TRACE_BLOCKS as well), to
// see how far apart blocks finish
__device__ __forceinline__ void trace_note_block(int what) {
  if (threadIdx.x == 0) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    const unsigned int i = atomicAdd(&trace_count, 1u) & 8191u;
    trace_ring[i].t = t;
    trace_ring[i].what = what;
    trace_ring[i].grid = (int)(gridDim.x * gridDim.y * gridDim.z);
    trace_ring[i].block = (int)blockIdx.x;
  }
}
#define PKV_TRACE_NOTE(what) pkv::trace_note(what)
#ifdef PKV_TRACE_BLOCKS
#define PKV_TRACE_NOTE_BLOCK(what) pkv::trace_note_block(what)
#else
#define PKV_TRACE_NOTE_BLOCK(what)
#endif
#else
#define PKV_TRACE_NOTE(what)
#define PKV_TRACE_NOTE_BLOCK(what)
#endif

__device__ __forceinline__ void dependents_may_launch() {
  PKV_TRACE_NOTE(0);
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void wait_for_prior_kernels() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  PKV_TRACE_NOTE(1);
}

// Launches `kernel`; `chained` as above, `cluster_x` > 0 groups that many blocks along x into a
// thread-block cluster. Returns 0 or the CUDA error.
template <typename... P, typename... A>
inline int launch_kernel(void (*kernel)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, bool chained,
                         int cluster_x, A&&... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attributes[2];
  int n = 0;
  if (cluster_x > 0) {
    attributes[n].id = cudaLaunchAttributeClusterDimension;
    attributes[n].val.clusterDim.x = cluster_x;
    attributes[n].val.clusterDim.y = 1;
    attributes[n].val.clusterDim.z = 1;
    ++n;
  }
#ifdef PKV_NO_CHAIN  // build switch for comparisons: every launch an ordinary one
  chained = false;
#endif
  if (chained) {
    attributes[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attributes[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  config.attrs = attributes;
  config.numAttrs = n;
  cudaError_t e = cudaLaunchKernelEx(&config, kernel, P(args)...);
  return e == cudaSuccess ? launch_status() : (int)e;
}

}  // namespace pkv

#ifdef PKV_TRACE
// Copies the library's trace ring (8192 records of 24 bytes) and its count to the host.
PKV_EXPORT int pkv_trace_read(void* records, unsigned int* count) {
  cudaError_t e = cudaMemcpyFromSymbol(records, pkv::trace_ring, sizeof(pkv::trace_ring));
  if (e == cudaSuccess) e = cudaMemcpyFromSymbol(count, pkv::trace_count, sizeof(unsigned int));
  return (int)e;
}
#endif
