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

// codes kernels record in the device's status word; the host raises on any of them
#define PKV_STATUS_BAD_ID 1        // a token id outside the embedding table
#define PKV_STATUS_GAVE_UP 2       // a bounded wait ran out
#define PKV_STATUS_OUT_OF_RANGE 3  // a page, a cache slot or a position outside its range

namespace pkv {

typedef __nv_bfloat16 bf16;

// A page number read from a block table is a page of the pool or -1 ("no page": its keys read as
// zeros). Anything else is recorded in the status word and treated as no page, so that a table
// the host got wrong never becomes an address.
__device__ __forceinline__ int checked_page(int page, int num_pages, int* status) {
  if (page >= num_pages || page < -1) {
    if (status) atomicExch(status, PKV_STATUS_OUT_OF_RANGE);
    return -1;
  }
  return page;
}

// The same for the kernels that fetch pages with TMA: the pool row where a page's keys of one
// key/value head begin, or `pool_rows` (a row the copy unit reads as zeros) for no page and for a
// page outside the pool, which is recorded.
__device__ __forceinline__ int checked_pool_row(int page, int n_kv, int kvh, int page_size, int pool_rows, int* status) {
  if (page < 0) {
    if (page < -1 && status) atomicExch(status, PKV_STATUS_OUT_OF_RANGE);
    return pool_rows;
  }
  const long long row = ((long long)page * n_kv + kvh) * page_size;
  if (row >= pool_rows) {
    if (status) atomicExch(status, PKV_STATUS_OUT_OF_RANGE);
    return pool_rows;
  }
  return (int)row;
}

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
__device__ __forceinline__ void dependents_may_launch() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void wait_for_prior_kernels() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
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
