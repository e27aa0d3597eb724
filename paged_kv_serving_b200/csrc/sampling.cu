// Token sampling on the device: greedy, temperature and nucleus (top-p), one block per row.
//
// The procedure restates the reference (rouviere-german/paged-kv-serving,
// src/paged_kv_serving/engine/sampling.py:28-74):
//   greedy        argmax, the lowest id on ties (rows whose temperature is below the threshold)
//   temperature   scaled = logits / T in float32; p = exp(double(scaled - max)) / sum -> float32
//   nucleus       tokens in descending probability (lower id first among equals) are kept up to
//                 and including the one whose cumulative mass (float64) reaches top_p; the rest
//                 are zeroed and the kept ones renormalised
//   draw          cum = cumulative sum in float64 in id order; draw = u * cum[-1]; the token is
//                 the first id whose cumulative mass exceeds the draw
// The uniform number u comes from the request's own generator on the host
// (src/paged_kv_serving/engine/sequence.py:165-170), one per sampled token, so a request's
// output does not depend on the batch it was sampled in.
//
// `probs` is scratch memory of n_rows * vocab floats: the kernel writes the (filtered)
// probabilities there and reads them back in later passes. With `status_word` (a device int, may
// be null) `out` has n_rows + 1 elements and the last one receives the word's value, so that the
// host learns of a fault that a kernel of the step recorded in the copy that brings the ids.
#include "common.cuh"

namespace pkv {

constexpr int SAMPLE_THREADS = 1024;

struct ArgMax {
  float v;
  int i;
};

__device__ __forceinline__ ArgMax better(ArgMax a, ArgMax b) {
  if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
  return a;
}

__device__ __forceinline__ double warp_sum_d(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ double block_sum_d(double v, double* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum_d(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  double t = lane < (SAMPLE_THREADS >> 5) ? scratch[lane] : 0.0;
  t = warp_sum_d(t);
  return t;  // the same value in every thread
}

// exclusive prefix sum over the block in thread order; returns the exclusive prefix of this
// thread and stores the block total in *total.
__device__ double block_scan_d(double v, double* scratch, double* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  double inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const double n = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += n;
  }
  __syncthreads();
  if (lane == 31) scratch[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    double w = scratch[lane];
    double winc = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const double n = __shfl_up_sync(0xffffffffu, winc, o);
      if (lane >= o) winc += n;
    }
    scratch[lane] = winc - w;       // exclusive prefix of each warp
    if (lane == 31) scratch[32] = winc;
  }
  __syncthreads();
  *total = scratch[32];
  return scratch[warp] + (inc - v);
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, long long row_stride, const float* __restrict__ temperature,
              const float* __restrict__ top_p, const double* __restrict__ uniform, float* __restrict__ probs,
              int32_t* __restrict__ out, int vocab, float greedy_below, const int* __restrict__ status_word) {
  __shared__ double scratch_d[33];
  __shared__ ArgMax scratch_a[32];
  __shared__ float shared_f;
  __shared__ int shared_i;
  __shared__ int shared_last;
  dependents_may_launch();
  wait_for_prior_kernels();
  const int r = blockIdx.x;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // every kernel of the step has finished (the wait above): what they recorded in the device's
  // status word travels to the host behind the ids, in the same copy
  if (status_word != nullptr && r == 0 && tid == 0) out[gridDim.x] = *status_word;
  const float* row = logits + (size_t)r * row_stride;
  const float temp = temperature[r];

  // ---- maximum (and its lowest index) of the row ----
  ArgMax best = {-INFINITY, 0x7fffffff};
  for (int i = tid; i < vocab; i += SAMPLE_THREADS) {
    const float v = row[i];
    if (v > best.v) best = {v, i};
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax other = {__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
    best = better(best, other);
  }
  if (lane == 0) scratch_a[warp] = best;
  __syncthreads();
  if (warp == 0) {
    best = scratch_a[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      ArgMax other = {__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
      best = better(best, other);
    }
    if (lane == 0) {
      shared_f = best.v;
      shared_i = best.i == 0x7fffffff ? 0 : best.i;
    }
  }
  __syncthreads();
  if (temp < greedy_below) {
    if (tid == 0) out[r] = shared_i;
    return;
  }

  // ---- probabilities: float32 scaling, float64 exponentials ----
  const float scaled_max = shared_f / temp;  // division is monotone: the scaled maximum
  float* p = probs + (size_t)r * vocab;
  double part = 0.0;
  for (int i = tid; i < vocab; i += SAMPLE_THREADS) part += exp((double)(row[i] / temp - scaled_max));
  const double denom = block_sum_d(part, scratch_d);
  for (int i = tid; i < vocab; i += SAMPLE_THREADS)
    p[i] = (float)(exp((double)(row[i] / temp - scaled_max)) / denom);
  __syncthreads();

  const int chunk = (vocab + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
  const int c0 = min(tid * chunk, vocab), c1 = min(c0 + chunk, vocab);

  // ---- nucleus filter ----
  const float tp = top_p[r];
  if (tp < 1.0f) {
    const double target = (double)tp;
    // largest probability value v with mass{p >= v} >= top_p, by bisection on the bit pattern
    unsigned lo = 0u, hi = 0x7f800001u;
    while (hi - lo > 1u) {
      const unsigned mid = lo + ((hi - lo) >> 1);
      const float thr = __uint_as_float(mid);
      double mass = 0.0;
      for (int i = tid; i < vocab; i += SAMPLE_THREADS) {
        const float v = p[i];
        if (v >= thr) mass += (double)v;
      }
      mass = block_sum_d(mass, scratch_d);
      if (mass >= target) lo = mid; else hi = mid;
    }
    const float pstar = __uint_as_float(lo);
    double above = 0.0;
    for (int i = tid; i < vocab; i += SAMPLE_THREADS) {
      const float v = p[i];
      if (v > pstar) above += (double)v;
    }
    above = block_sum_d(above, scratch_d);
    // ties at pstar are kept in id order until the cumulative mass reaches top_p
    long long need = 1;
    if (pstar > 0.0f) {
      need = (long long)ceil((target - above) / (double)pstar);
      if (need < 1) need = 1;
      while (need > 1 && above + (double)(need - 1) * (double)pstar >= target) --need;
      while (above + (double)need * (double)pstar < target && need < vocab) ++need;
    } else {
      need = vocab;  // the whole mass is below top_p: everything is kept
    }
    double ties = 0.0;
    for (int i = c0; i < c1; ++i) ties += (p[i] == pstar) ? 1.0 : 0.0;
    double tie_total;
    double rank = block_scan_d(ties, scratch_d, &tie_total);
    double kept = 0.0;
    for (int i = c0; i < c1; ++i) {
      const float v = p[i];
      bool keep = v > pstar;
      if (v == pstar) {
        keep = rank < (double)need;
        rank += 1.0;
      }
      if (keep) kept += (double)v; else p[i] = 0.0f;
    }
    const float total = (float)block_sum_d(kept, scratch_d);
    if (total > 0.0f)
      for (int i = c0; i < c1; ++i) p[i] = p[i] / total;
    __syncthreads();
  }

  // ---- inverse CDF in id order ----
  double mine = 0.0;
  int last_kept = -1;   // the highest id of this thread's share with a probability above zero
  for (int i = c0; i < c1; ++i) {
    mine += (double)p[i];
    if (p[i] > 0.0f) last_kept = i;
  }
  double total;
  const double before = block_scan_d(mine, scratch_d, &total);
  const double draw = uniform[r] * total;
  if (tid == 0) {
    shared_i = -1;
    shared_last = 0;
  }
  __syncthreads();
  if (last_kept >= 0) atomicMax(&shared_last, last_kept);
  if (last_kept >= 0 && before <= draw && before + mine > draw) {
    // `before` comes from the block's scan and `mine` from this loop: their roundings differ by an
    // ulp, so the loop may end without crossing the draw; the share's last kept id then takes it
    double c = before;
    int token = last_kept;
    for (int i = c0; i < c1; ++i) {
      c += (double)p[i];
      if (c > draw && p[i] > 0.0f) { token = i; break; }
    }
    shared_i = token;
  }
  __syncthreads();
  // a draw at the very top of the distribution (u * total rounding up to the total) is claimed by
  // no share: it belongs to the last id that the filter kept, never to a zeroed one
  if (tid == 0) out[r] = shared_i >= 0 ? shared_i : shared_last;
}

}  // namespace pkv

using namespace pkv;

PKV_EXPORT int pkv_sample(const float* logits, long long row_stride, const float* temperature, const float* top_p,
                          const double* uniform, float* probs, int32_t* out, int n_rows, int vocab,
                          float greedy_below, const int* status_word, void* stream) {
  if (n_rows <= 0) return 0;
  if (vocab <= 0 || row_stride < vocab) return PKV_ERR_SIZE;
  return launch_kernel(sample_kernel, dim3(n_rows), dim3(SAMPLE_THREADS), 0, (cudaStream_t)stream, true, 0, logits, row_stride,
                       temperature, top_p, uniform, probs, out, vocab, greedy_below, status_word);
}

// ---------------------------------------------------------------------------------------------
// The same sampling for callers that cannot allocate: the work area is part of the library image.
// See sampling_noalloc.h for who needs this and for the rules of use.
// ---------------------------------------------------------------------------------------------
#include "sampling_noalloc.h"

// In device code this name is the array itself. In host code it is only a stand-in for it: the
// device address has to be asked for with cudaGetSymbolAddress, once per device.
static __device__ __align__(256) float pkv_sample_static_area[PKV_SAMPLE_STATIC_FLOATS];

namespace {
constexpr int kMaxDevices = 64;
float* static_area_of_device[kMaxDevices] = {};
}  // namespace

PKV_EXPORT int pkv_sample_static_scratch(const float* logits, long long row_stride, const float* temperature,
                                         const float* top_p, const double* uniform, int32_t* out, int n_rows,
                                         int vocab, float greedy_below, void* stream) {
  if (n_rows <= 0) return 0;
  if (vocab <= 0 || row_stride < vocab) return PKV_ERR_SIZE;
  if ((long long)n_rows * vocab > (long long)PKV_SAMPLE_STATIC_FLOATS) return PKV_SAMPLE_STATIC_TOO_LARGE;
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return (int)e;
  if (device < 0 || device >= kMaxDevices) return PKV_SAMPLE_STATIC_DEVICE_INDEX;
  if (!static_area_of_device[device]) {
    // set-up, once per device, with that device current
    float* address = nullptr;
    e = cudaGetSymbolAddress((void**)&address, pkv_sample_static_area);
    if (e != cudaSuccess) return (int)e;
    static_area_of_device[device] = address;
  }
  sample_kernel<<<n_rows, SAMPLE_THREADS, 0, (cudaStream_t)stream>>>(logits, row_stride, temperature, top_p, uniform,
                                                                    static_area_of_device[device], out, vocab,
                                                                    greedy_below, nullptr);
  return launch_status();
}
