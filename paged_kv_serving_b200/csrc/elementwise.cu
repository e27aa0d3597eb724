// Row-wise and element-wise kernels of the decoder: embedding gather, residual add + RMSNorm,
// SiLU(gate) * up, and rotary position encoding fused with the write of keys and values into
// the paged cache. All arithmetic is float32; tensors are float32 or bfloat16 in memory.
//
// Formulas restate the reference (rouviere-german/paged-kv-serving):
//   RMSNorm   src/paged_kv_serving/engine/model.py:43-46   y = (x / sqrt(mean(x^2) + eps)) * w
//   SiLU      src/paged_kv_serving/engine/model.py:49-51   x * 1/(1 + exp(-clip(x, -c, c)))
//   RoPE      src/paged_kv_serving/engine/model.py:70-81   half-split rotation by position
//   KV write  src/paged_kv_serving/engine/runner.py:149-159,194-196  slot = page * size + offset
#include "common.cuh"

namespace pkv {

// ---------------------------------------------------------------------------------------------
// embedding gather: out[t, :] = table[ids[t], :] widened to float32
// ---------------------------------------------------------------------------------------------
template <typename W>
__global__ void embedding_gather_kernel(const W* __restrict__ table, const int32_t* __restrict__ ids,
                                        float* __restrict__ out, int d, int vocab, int* __restrict__ status) {
  const int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 || id >= vocab) {  // never read outside the table: record and use row 0
    if (threadIdx.x == 0) atomicExch(status, 1);
    id = 0;
  }
  const W* row = table + (size_t)id * d;
  float* dst = out + (size_t)t * d;
  for (int i = threadIdx.x; i < d; i += blockDim.x) dst[i] = to_float(row[i]);
}

// ---------------------------------------------------------------------------------------------
// residual add + RMSNorm
//   src = rows ? rows[r] : r
//   x   = hidden[src] + (delta ? delta[src] : 0)        (float32)
//   if (!rows) hidden[src] = x                           (the residual stream is updated in place)
//   out[r] = (x / sqrt(mean(x^2) + eps)) * weight
// One block per output row; the row is kept in shared memory between the two passes.
// ---------------------------------------------------------------------------------------------
template <typename D, typename O>
__global__ void add_rmsnorm_kernel(float* __restrict__ hidden, const D* __restrict__ delta,
                                   const float* __restrict__ weight, float eps, O* __restrict__ out,
                                   const int32_t* __restrict__ rows, int d) {
  extern __shared__ float row_buf[];  // d floats + 32 scratch
  float* scratch = row_buf + d;
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  float* h = hidden + (size_t)src * d;
  const D* dl = delta ? delta + (size_t)src * d : nullptr;
  float sq = 0.0f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    float x = h[i];
    if (dl) x += to_float(dl[i]);
    row_buf[i] = x;
    sq += x * x;
  }
  const float total = block_sum(sq, scratch);
  const float root = sqrtf(total / (float)d + eps);
  O* o = out + (size_t)r * d;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    const float x = row_buf[i];
    if (!rows && dl) h[i] = x;
    o[i] = from_float<O>((x / root) * weight[i]);
  }
}

// ---------------------------------------------------------------------------------------------
// SiLU(gate) * up over a fused [T, 2*ff] input (gate columns first), output [T, ff]
// ---------------------------------------------------------------------------------------------
template <typename A>
__global__ void silu_mul_kernel(const A* __restrict__ gate_up, A* __restrict__ out, int ff, float clip) {
  const int t = blockIdx.y;
  const A* g = gate_up + (size_t)t * 2 * ff;
  const A* u = g + ff;
  A* o = out + (size_t)t * ff;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < ff; i += gridDim.x * blockDim.x) {
    const float x = to_float(g[i]);
    const float c = fminf(fmaxf(x, -clip), clip);
    const float s = x * (1.0f / (1.0f + expf(-c)));
    o[i] = from_float<A>(s * to_float(u[i]));
  }
}

// ---------------------------------------------------------------------------------------------
// rotary encoding of q and k (in float32, angles from float32 tables built in float64 on the
// host) fused with the write of k and v into the paged cache.
//   qkv      [T, (H + 2*KV) * hd]   q is rotated in place; k, v are read
//   cos/sin  [max_pos, hd/2] or null (no rotation: store only)
//   k_pool / v_pool  [pages, KV, page_size, hd]  of one layer
//   slots    [T]  page * page_size + offset, or -1 to skip the store of a token
// grid (T, H + 2*KV): one block per (token, head); blockDim = hd/2 rounded up to a warp.
// ---------------------------------------------------------------------------------------------
template <typename A, typename C>
__global__ void rope_kv_store_kernel(A* __restrict__ qkv, const int32_t* __restrict__ positions,
                                     const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                     C* __restrict__ k_pool, C* __restrict__ v_pool,
                                     const int32_t* __restrict__ slots, int n_heads, int n_kv, int hd,
                                     int page_size, int store) {
  const int t = blockIdx.x;
  const int head = blockIdx.y;  // [0,H) q heads, [H,H+KV) k heads, [H+KV,H+2KV) v heads
  const int half = hd >> 1;
  A* row = qkv + ((size_t)t * (n_heads + 2 * n_kv) + head) * hd;
  const int pos = positions[t];
  const bool is_q = head < n_heads;
  const bool is_k = !is_q && head < n_heads + n_kv;
  size_t base = 0;
  bool do_store = false;
  if (!is_q && store) {
    const int slot = slots[t];
    if (slot >= 0) {
      const int kvh = is_k ? head - n_heads : head - n_heads - n_kv;
      const int page = slot / page_size, off = slot - page * page_size;
      base = (((size_t)page * n_kv + kvh) * page_size + off) * hd;
      do_store = true;
    }
  }
  if (is_q || is_k) {
    for (int j = threadIdx.x; j < half; j += blockDim.x) {
      float left = to_float(row[j]), right = to_float(row[j + half]);
      float lo = left, hi = right;
      if (cos_t) {
        const float c = cos_t[(size_t)pos * half + j], s = sin_t[(size_t)pos * half + j];
        lo = left * c - right * s;
        hi = right * c + left * s;
      }
      if (is_q) {
        row[j] = from_float<A>(lo);
        row[j + half] = from_float<A>(hi);
      } else if (do_store) {
        k_pool[base + j] = from_float<C>(lo);
        k_pool[base + j + half] = from_float<C>(hi);
      }
    }
  } else if (do_store) {
    for (int j = threadIdx.x; j < hd; j += blockDim.x) v_pool[base + j] = from_float<C>(to_float(row[j]));
  }
}

}  // namespace pkv

using namespace pkv;

PKV_EXPORT int pkv_embedding_gather(const void* table, int table_dtype, const int32_t* ids, float* out,
                                    int n_tokens, int d, int vocab, int* status, void* stream) {
  if (n_tokens <= 0) return 0;
  if (d <= 0 || vocab <= 0) return PKV_ERR_SIZE;
  cudaStream_t s = (cudaStream_t)stream;
  const int threads = d >= 1024 ? 256 : 128;
  if (table_dtype == PKV_F32)
    embedding_gather_kernel<float><<<n_tokens, threads, 0, s>>>((const float*)table, ids, out, d, vocab, status);
  else if (table_dtype == PKV_BF16)
    embedding_gather_kernel<bf16><<<n_tokens, threads, 0, s>>>((const bf16*)table, ids, out, d, vocab, status);
  else
    return PKV_ERR_DTYPE;
  return launch_status();
}

template <typename D, typename O>
static int launch_add_rmsnorm(float* hidden, const void* delta, const float* weight, float eps, void* out,
                              const int32_t* rows, int n_rows, int d, cudaStream_t s) {
  const size_t smem = (size_t)(d + 32) * sizeof(float);
  if (smem > 200 * 1024) return PKV_ERR_LIMIT;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(add_rmsnorm_kernel<D, O>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  const int threads = d >= 2048 ? 512 : (d >= 512 ? 256 : 128);
  add_rmsnorm_kernel<D, O><<<n_rows, threads, smem, s>>>(hidden, (const D*)delta, weight, eps, (O*)out, rows, d);
  return launch_status();
}

PKV_EXPORT int pkv_add_rmsnorm(float* hidden, const void* delta, int delta_dtype, const float* weight, float eps,
                               void* out, int out_dtype, const int32_t* rows, int n_rows, int d, void* stream) {
  if (n_rows <= 0) return 0;
  if (d <= 0) return PKV_ERR_SIZE;
  cudaStream_t s = (cudaStream_t)stream;
  if (!delta) delta_dtype = out_dtype;
  if (delta_dtype == PKV_F32 && out_dtype == PKV_F32)
    return launch_add_rmsnorm<float, float>(hidden, delta, weight, eps, out, rows, n_rows, d, s);
  if (delta_dtype == PKV_BF16 && out_dtype == PKV_BF16)
    return launch_add_rmsnorm<bf16, bf16>(hidden, delta, weight, eps, out, rows, n_rows, d, s);
  if (delta_dtype == PKV_F32 && out_dtype == PKV_BF16)
    return launch_add_rmsnorm<float, bf16>(hidden, delta, weight, eps, out, rows, n_rows, d, s);
  if (delta_dtype == PKV_BF16 && out_dtype == PKV_F32)
    return launch_add_rmsnorm<bf16, float>(hidden, delta, weight, eps, out, rows, n_rows, d, s);
  return PKV_ERR_DTYPE;
}

PKV_EXPORT int pkv_silu_mul(const void* gate_up, void* out, int dtype, int n_tokens, int ff, float clip, void* stream) {
  if (n_tokens <= 0) return 0;
  if (ff <= 0) return PKV_ERR_SIZE;
  cudaStream_t s = (cudaStream_t)stream;
  const int threads = 256;
  int bx = (ff + threads - 1) / threads;
  if (bx > 64) bx = 64;
  // grid.y carries the token axis; split very large batches across launches
  for (int t0 = 0; t0 < n_tokens; t0 += 65535) {
    const int nt = n_tokens - t0 < 65535 ? n_tokens - t0 : 65535;
    dim3 grid(bx, nt);
    if (dtype == PKV_F32)
      silu_mul_kernel<float><<<grid, threads, 0, s>>>((const float*)gate_up + (size_t)t0 * 2 * ff, (float*)out + (size_t)t0 * ff, ff, clip);
    else if (dtype == PKV_BF16)
      silu_mul_kernel<bf16><<<grid, threads, 0, s>>>((const bf16*)gate_up + (size_t)t0 * 2 * ff, (bf16*)out + (size_t)t0 * ff, ff, clip);
    else
      return PKV_ERR_DTYPE;
  }
  return launch_status();
}

PKV_EXPORT int pkv_rope_kv_store(void* qkv, int act_dtype, const int32_t* positions, const float* cos_t,
                                 const float* sin_t, void* k_pool, void* v_pool, int cache_dtype,
                                 const int32_t* slots, int n_tokens, int n_heads, int n_kv, int hd, int page_size,
                                 int store, void* stream) {
  if (n_tokens <= 0) return 0;
  if (n_heads <= 0 || n_kv <= 0 || hd <= 0 || (hd & 1) || page_size <= 0) return PKV_ERR_SIZE;
  if (n_heads + 2 * n_kv > 65535) return PKV_ERR_LIMIT;
  cudaStream_t s = (cudaStream_t)stream;
  int threads = ((hd / 2 + 31) / 32) * 32;
  if (threads > 256) threads = 256;
  dim3 grid(n_tokens, n_heads + 2 * n_kv);
#define PKV_ROPE(A, C) \
  rope_kv_store_kernel<A, C><<<grid, threads, 0, s>>>((A*)qkv, positions, cos_t, sin_t, (C*)k_pool, (C*)v_pool, slots, n_heads, n_kv, hd, page_size, store)
  if (act_dtype == PKV_F32 && cache_dtype == PKV_F32) PKV_ROPE(float, float);
  else if (act_dtype == PKV_BF16 && cache_dtype == PKV_BF16) PKV_ROPE(bf16, bf16);
  else if (act_dtype == PKV_F32 && cache_dtype == PKV_BF16) PKV_ROPE(float, bf16);
  else if (act_dtype == PKV_BF16 && cache_dtype == PKV_F32) PKV_ROPE(bf16, float);
  else return PKV_ERR_DTYPE;
#undef PKV_ROPE
  return launch_status();
}
