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
// With `fed_back` and `fed_back_at`, token t whose fed_back_at[t] >= 0 takes its id from
// fed_back[fed_back_at[t]] instead: the id that the sampler of the step before left on the device,
// so that a decoded token can enter the next step without passing through the host.
// ---------------------------------------------------------------------------------------------
template <typename W>
__global__ void embedding_gather_kernel(const W* __restrict__ table, const int32_t* __restrict__ ids,
                                        float* __restrict__ out, int d, int vocab, int* __restrict__ status,
                                        const int32_t* __restrict__ fed_back, const int32_t* __restrict__ fed_back_at) {
  dependents_may_launch();
  wait_for_prior_kernels();
  const int t = blockIdx.x;
  int id = ids[t];
  if (fed_back_at != nullptr) {
    const int at = fed_back_at[t];
    if (at >= 0) id = fed_back[at];
  }
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
  dependents_may_launch();
  wait_for_prior_kernels();
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

// Where gate and up of output column i sit in an input row. interleave = 0: gate columns
// [0, ff), up columns [ff, 2 ff). interleave = B: blocks of B gate columns followed by the B
// matching up columns (the layout the fused tensor-core product works on).
__device__ __forceinline__ void gate_up_at(int i, int ff, int interleave, int& g, int& u) {
  if (interleave == 0) {
    g = i;
    u = ff + i;
  } else {
    const int b = i / interleave;
    g = b * 2 * interleave + (i - b * interleave);
    u = g + interleave;
  }
}

// The same, for widths that are multiples of 4 and at most 4 * VEC_PER_THREAD * blockDim: every
// thread keeps its part of the row in registers (one pass over memory, 16-byte accesses).
constexpr int NORM_VEC_PER_THREAD = 4;

__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const bf16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
  const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
  const float2 fa = __bfloat1622float2(a), fb = __bfloat1622float2(b);
  return make_float4(fa.x, fa.y, fb.x, fb.y);
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(bf16* p, float4 v) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 raw;
  raw.x = *reinterpret_cast<uint32_t*>(&a);
  raw.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = raw;
}

template <typename D, typename O>
__global__ void add_rmsnorm_vec_kernel(float* __restrict__ hidden, const D* __restrict__ delta,
                                       const float* __restrict__ weight, float eps, O* __restrict__ out,
                                       const int32_t* __restrict__ rows, int d) {
  dependents_may_launch();
  wait_for_prior_kernels();
  __shared__ float scratch[32];
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  float* h = hidden + (size_t)src * d;
  const D* dl = delta ? delta + (size_t)src * d : nullptr;
  const int chunks = d >> 2;
  float4 x[NORM_VEC_PER_THREAD];
  float sq = 0.0f;
#pragma unroll
  for (int i = 0; i < NORM_VEC_PER_THREAD; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    if (c < chunks) {
      float4 v = load4(h + 4 * c);
      if (dl) {
        const float4 e = load4(dl + 4 * c);
        v.x += e.x; v.y += e.y; v.z += e.z; v.w += e.w;
        if (!rows) store4(h + 4 * c, v);
      }
      x[i] = v;
      sq += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
  }
  const float total = block_sum(sq, scratch);
  const float root = sqrtf(total / (float)d + eps);
  O* o = out + (size_t)r * d;
#pragma unroll
  for (int i = 0; i < NORM_VEC_PER_THREAD; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    if (c < chunks) {
      const float4 w = load4(weight + 4 * c);
      store4(o + 4 * c, make_float4((x[i].x / root) * w.x, (x[i].y / root) * w.y, (x[i].z / root) * w.z,
                                    (x[i].w / root) * w.w));
    }
  }
}

// Completes an RMS norm that a matrix-product kernel left in two pieces (the residual epilogues
// of csrc/gemm_small_m.cu and csrc/gemm_stream.cu): `xw` is the stream times the norm's weight,
// `sumsq[part * stride + row]` the sums of squares of the stream per tile of columns.
// out = xw / sqrt(sum / d + eps). One block per row.
__global__ void finish_norm_kernel(const bf16* __restrict__ xw, const float* __restrict__ sumsq, int parts, int stride,
                                   float eps, bf16* __restrict__ out, int d) {
  dependents_may_launch();
  wait_for_prior_kernels();
  __shared__ float inv_root;
  const int row = blockIdx.x;
  if (threadIdx.x < 32) {   // the same order of additions as the product kernel that reads these sums
    float q = 0.0f;
    for (int part = threadIdx.x; part < parts; part += 32) q += sumsq[(size_t)part * stride + row];
    q = warp_sum(q);
    if (threadIdx.x == 0) inv_root = 1.0f / sqrtf(q / (float)d + eps);
  }
  __syncthreads();
  const float r = inv_root;
  for (int c = threadIdx.x; c < d; c += blockDim.x)
    out[(size_t)row * d + c] = __float2bfloat16_rn(__bfloat162float(xw[(size_t)row * d + c]) * r);
}

// ---------------------------------------------------------------------------------------------
// SiLU(gate) * up over a fused [T, 2*ff] input (gate columns first), output [T, ff]
// ---------------------------------------------------------------------------------------------
// ff a multiple of 8 (bfloat16) or 4 (float32): 16-byte accesses, one flat grid over all chunks
template <typename A, int V>
__global__ void silu_mul_vec_kernel(const A* __restrict__ gate_up, A* __restrict__ out, int ff, int in_stride,
                                    int interleave, long long n_chunks, float clip) {
  dependents_may_launch();
  wait_for_prior_kernels();
  const int chunks_per_row = ff / V;
  for (long long c = (long long)blockIdx.x * blockDim.x + threadIdx.x; c < n_chunks; c += (long long)gridDim.x * blockDim.x) {
    const long long t = c / chunks_per_row;
    const int i = (int)(c - t * chunks_per_row) * V;
    int gi, ui;
    gate_up_at(i, ff, interleave, gi, ui);
    const A* g = gate_up + t * in_stride + gi;
    const A* u = gate_up + t * in_stride + ui;
    A* o = out + t * ff + i;
#pragma unroll
    for (int q = 0; q < V; q += 4) {
      const float4 gv = load4(g + q), uv = load4(u + q);
      float4 r;
      r.x = gv.x * (1.0f / (1.0f + expf(-fminf(fmaxf(gv.x, -clip), clip)))) * uv.x;
      r.y = gv.y * (1.0f / (1.0f + expf(-fminf(fmaxf(gv.y, -clip), clip)))) * uv.y;
      r.z = gv.z * (1.0f / (1.0f + expf(-fminf(fmaxf(gv.z, -clip), clip)))) * uv.z;
      r.w = gv.w * (1.0f / (1.0f + expf(-fminf(fmaxf(gv.w, -clip), clip)))) * uv.w;
      store4(o + q, r);
    }
  }
}

template <typename A>
__global__ void silu_mul_kernel(const A* __restrict__ gate_up, A* __restrict__ out, int ff, int in_stride,
                                int interleave, float clip) {
  dependents_may_launch();
  wait_for_prior_kernels();
  const int t = blockIdx.y;
  const A* row = gate_up + (size_t)t * in_stride;
  A* o = out + (size_t)t * ff;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < ff; i += gridDim.x * blockDim.x) {
    int gi, ui;
    gate_up_at(i, ff, interleave, gi, ui);
    const float x = to_float(row[gi]);
    const float c = fminf(fmaxf(x, -clip), clip);
    const float s = x * (1.0f / (1.0f + expf(-c)));
    o[i] = from_float<A>(s * to_float(row[ui]));
  }
}

// ---------------------------------------------------------------------------------------------
// rotary encoding of q and k (in float32, angles from float32 tables built in float64 on the
// host) fused with the write of k and v into the paged cache.
//   qkv      [T, (H + 2*KV) * hd]   q is rotated in place; k, v are read
//   cos/sin  [max_pos, hd/2] or null (no rotation: store only)
//   k_pool / v_pool  [pages, KV, page_size, hd]  of one layer
//   slots    [T]  page * page_size + offset, or -1 to skip the store of a token
// A slot outside the pool (`num_slots`) or a position outside the tables (`max_pos`) is recorded
// in the status word; the store is skipped, the rotation uses position 0.
// grid (T, H + 2*KV): one block per (token, head); blockDim = hd/2 rounded up to a warp.
// ---------------------------------------------------------------------------------------------
template <typename A, typename C>
__global__ void rope_kv_store_kernel(A* __restrict__ qkv, const int32_t* __restrict__ positions,
                                     const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                     C* __restrict__ k_pool, C* __restrict__ v_pool,
                                     const int32_t* __restrict__ slots, int n_heads, int n_kv, int hd,
                                     int page_size, int store, int num_slots, int max_pos, int* __restrict__ status) {
  dependents_may_launch();
  wait_for_prior_kernels();
  const int t = blockIdx.x;
  const int head = blockIdx.y;  // [0,H) q heads, [H,H+KV) k heads, [H+KV,H+2KV) v heads
  const int half = hd >> 1;
  A* row = qkv + ((size_t)t * (n_heads + 2 * n_kv) + head) * hd;
  int pos = positions[t];
  if (cos_t && (pos < 0 || pos >= max_pos)) {
    if (threadIdx.x == 0 && status) atomicExch(status, PKV_STATUS_OUT_OF_RANGE);
    pos = 0;
  }
  const bool is_q = head < n_heads;
  const bool is_k = !is_q && head < n_heads + n_kv;
  size_t base = 0;
  bool do_store = false;
  if (!is_q && store) {
    const int slot = slots[t];
    if (slot >= num_slots || slot < -1) {
      if (threadIdx.x == 0 && status) atomicExch(status, PKV_STATUS_OUT_OF_RANGE);
    } else if (slot >= 0) {
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

// The same for head sizes that are multiples of 8: one block per token, every thread rotates 4
// pairs (left[j..j+3], right[j..j+3]) or copies 4 values of v, with 8- or 16-byte accesses.
template <typename A, typename C>
__global__ void rope_kv_store_vec_kernel(A* __restrict__ qkv, const int32_t* __restrict__ positions,
                                         const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                         C* __restrict__ k_pool, C* __restrict__ v_pool,
                                         const int32_t* __restrict__ slots, int n_heads, int n_kv, int hd,
                                         int page_size, int store, int num_slots, int max_pos,
                                         int* __restrict__ status) {
  dependents_may_launch();
  wait_for_prior_kernels();
  const int t = blockIdx.x;
  const int half = hd >> 1;
  const int quads = half >> 2;                       // groups of 4 pairs per head
  int pos = positions[t];
  int slot = store ? slots[t] : -1;
  if ((cos_t && (pos < 0 || pos >= max_pos)) || slot >= num_slots || slot < -1) {
    if (threadIdx.x == 0 && status) atomicExch(status, PKV_STATUS_OUT_OF_RANGE);
    if (cos_t && (pos < 0 || pos >= max_pos)) pos = 0;
    if (slot >= num_slots || slot < -1) slot = -1;
  }
  const int page = slot >= 0 ? slot / page_size : 0, off = slot >= 0 ? slot - page * page_size : 0;
  A* row = qkv + (size_t)t * (n_heads + 2 * n_kv) * hd;
  const int rot_tasks = (n_heads + n_kv) * quads;
  const int copy_tasks = slot >= 0 ? n_kv * (hd >> 2) : 0;
  for (int task = threadIdx.x; task < rot_tasks + copy_tasks; task += blockDim.x) {
    if (task < rot_tasks) {
      const int head = task / quads, j = (task - head * quads) * 4;
      const bool is_q = head < n_heads;
      if (!is_q && slot < 0) continue;
      A* hp = row + (size_t)head * hd;
      float4 left = load4(hp + j), right = load4(hp + half + j);
      float4 lo = left, hi = right;
      if (cos_t) {
        const float4 c = load4(cos_t + (size_t)pos * half + j), s = load4(sin_t + (size_t)pos * half + j);
        lo = make_float4(left.x * c.x - right.x * s.x, left.y * c.y - right.y * s.y, left.z * c.z - right.z * s.z,
                         left.w * c.w - right.w * s.w);
        hi = make_float4(right.x * c.x + left.x * s.x, right.y * c.y + left.y * s.y, right.z * c.z + left.z * s.z,
                         right.w * c.w + left.w * s.w);
      }
      if (is_q) {
        if (cos_t) { store4(hp + j, lo); store4(hp + half + j, hi); }
      } else {
        C* dst = k_pool + (((size_t)page * n_kv + (head - n_heads)) * page_size + off) * hd;
        store4(dst + j, lo);
        store4(dst + half + j, hi);
      }
    } else {
      const int c = task - rot_tasks;
      const int kvh = c / (hd >> 2), j = (c - kvh * (hd >> 2)) * 4;
      const float4 v = load4(row + (size_t)(n_heads + n_kv + kvh) * hd + j);
      store4(v_pool + (((size_t)page * n_kv + kvh) * page_size + off) * hd + j, v);
    }
  }
}

}  // namespace pkv

using namespace pkv;

PKV_EXPORT int pkv_embedding_gather(const void* table, int table_dtype, const int32_t* ids, float* out,
                                    int n_tokens, int d, int vocab, int* status, const int32_t* fed_back,
                                    const int32_t* fed_back_at, void* stream) {
  if (n_tokens <= 0) return 0;
  if (d <= 0 || vocab <= 0) return PKV_ERR_SIZE;
  cudaStream_t s = (cudaStream_t)stream;
  const int threads = d >= 1024 ? 256 : 128;
  // the first kernel of a step follows a copy from the host, not a kernel: an ordinary launch
  if (table_dtype == PKV_F32)
    return launch_kernel(embedding_gather_kernel<float>, dim3(n_tokens), dim3(threads), 0, s, false, 0,
                         (const float*)table, ids, out, d, vocab, status, fed_back, fed_back_at);
  if (table_dtype == PKV_BF16)
    return launch_kernel(embedding_gather_kernel<bf16>, dim3(n_tokens), dim3(threads), 0, s, false, 0,
                         (const bf16*)table, ids, out, d, vocab, status, fed_back, fed_back_at);
  return PKV_ERR_DTYPE;
}

template <typename D, typename O>
static int launch_add_rmsnorm(float* hidden, const void* delta, const float* weight, float eps, void* out,
                              const int32_t* rows, int n_rows, int d, cudaStream_t s) {
  if (d % 4 == 0 && d <= 4 * NORM_VEC_PER_THREAD * 1024) {
    const int chunks = d / 4;
    int threads = ((chunks + 1) / 2 + 31) / 32 * 32;           // two chunks a thread where that fits
    if (threads < 64) threads = 64;
    if (threads > 1024) threads = 1024;
    return launch_kernel(add_rmsnorm_vec_kernel<D, O>, dim3(n_rows), dim3(threads), 0, s, true, 0,
                         hidden, (const D*)delta, weight, eps, (O*)out, rows, d);
  }
  const size_t smem = (size_t)(d + 32) * sizeof(float);
  if (smem > 200 * 1024) return PKV_ERR_LIMIT;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(add_rmsnorm_kernel<D, O>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  const int threads = d >= 2048 ? 512 : (d >= 512 ? 256 : 128);
  return launch_kernel(add_rmsnorm_kernel<D, O>, dim3(n_rows), dim3(threads), smem, s, true, 0,
                       hidden, (const D*)delta, weight, eps, (O*)out, rows, d);
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

PKV_EXPORT int pkv_finish_norm(const void* xw, const float* sumsq, int parts, int stride, float eps, void* out, int n_rows,
                               int d, void* stream) {
  if (n_rows <= 0) return 0;
  if (d <= 0 || parts <= 0 || n_rows > stride) return PKV_ERR_SIZE;
  return launch_kernel(finish_norm_kernel, dim3(n_rows), dim3(256), 0, (cudaStream_t)stream, true, 0, (const bf16*)xw, sumsq,
                       parts, stride, eps, (bf16*)out, d);
}

PKV_EXPORT int pkv_silu_mul(const void* gate_up, void* out, int dtype, int n_tokens, int ff, int in_stride,
                            int interleave, float clip, void* stream) {
  if (n_tokens <= 0) return 0;
  if (ff <= 0 || interleave < 0 || in_stride < 2 * ff) return PKV_ERR_SIZE;
  cudaStream_t s = (cudaStream_t)stream;
  const int v = dtype == PKV_BF16 ? 8 : 4;
  if ((dtype == PKV_BF16 || dtype == PKV_F32) && ff % v == 0 && in_stride % v == 0 && interleave % v == 0) {
    const long long n_chunks = (long long)n_tokens * (ff / v);
    long long blocks = (n_chunks + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (dtype == PKV_BF16)
      return launch_kernel(silu_mul_vec_kernel<bf16, 8>, dim3((int)blocks), dim3(256), 0, s, true, 0,
                           (const bf16*)gate_up, (bf16*)out, ff, in_stride, interleave, n_chunks, clip);
    return launch_kernel(silu_mul_vec_kernel<float, 4>, dim3((int)blocks), dim3(256), 0, s, true, 0,
                         (const float*)gate_up, (float*)out, ff, in_stride, interleave, n_chunks, clip);
  }
  const int threads = 256;
  int bx = (ff + threads - 1) / threads;
  if (bx > 64) bx = 64;
  // grid.y carries the token axis; split very large batches across launches
  for (int t0 = 0; t0 < n_tokens; t0 += 65535) {
    const int nt = n_tokens - t0 < 65535 ? n_tokens - t0 : 65535;
    dim3 grid(bx, nt);
    int rc;
    if (dtype == PKV_F32)
      rc = launch_kernel(silu_mul_kernel<float>, grid, dim3(threads), 0, s, true, 0,
                         (const float*)gate_up + (size_t)t0 * in_stride, (float*)out + (size_t)t0 * ff, ff, in_stride, interleave, clip);
    else if (dtype == PKV_BF16)
      rc = launch_kernel(silu_mul_kernel<bf16>, grid, dim3(threads), 0, s, true, 0,
                         (const bf16*)gate_up + (size_t)t0 * in_stride, (bf16*)out + (size_t)t0 * ff, ff, in_stride, interleave, clip);
    else
      return PKV_ERR_DTYPE;
    if (rc != 0) return rc;
  }
  return 0;
}

PKV_EXPORT int pkv_rope_kv_store(void* qkv, int act_dtype, const int32_t* positions, const float* cos_t,
                                 const float* sin_t, void* k_pool, void* v_pool, int cache_dtype,
                                 const int32_t* slots, int n_tokens, int n_heads, int n_kv, int hd, int page_size,
                                 int store, int num_slots, int max_pos, int* status, void* stream) {
  if (n_tokens <= 0) return 0;
  if (n_heads <= 0 || n_kv <= 0 || hd <= 0 || (hd & 1) || page_size <= 0) return PKV_ERR_SIZE;
  if ((store && num_slots <= 0) || (cos_t && max_pos <= 0)) return PKV_ERR_SIZE;
  if (n_heads + 2 * n_kv > 65535) return PKV_ERR_LIMIT;
  cudaStream_t s = (cudaStream_t)stream;
  if (hd % 8 == 0) {
    const int tasks = (n_heads + n_kv) * (hd / 8) + n_kv * (hd / 4);
    int vthreads = (tasks + 31) / 32 * 32;
    if (vthreads > 512) vthreads = 512;
#define PKV_ROPE_VEC(A, C)                                                                                   \
  return launch_kernel(rope_kv_store_vec_kernel<A, C>, dim3(n_tokens), dim3(vthreads), 0, s, true, 0, (A*)qkv, \
                       positions, cos_t, sin_t, (C*)k_pool, (C*)v_pool, slots, n_heads, n_kv, hd, page_size, store, num_slots, \
                       max_pos, status)
    if (act_dtype == PKV_F32 && cache_dtype == PKV_F32) PKV_ROPE_VEC(float, float);
    if (act_dtype == PKV_BF16 && cache_dtype == PKV_BF16) PKV_ROPE_VEC(bf16, bf16);
    if (act_dtype == PKV_F32 && cache_dtype == PKV_BF16) PKV_ROPE_VEC(float, bf16);
    if (act_dtype == PKV_BF16 && cache_dtype == PKV_F32) PKV_ROPE_VEC(bf16, float);
#undef PKV_ROPE_VEC
    return PKV_ERR_DTYPE;
  }
  int threads = ((hd / 2 + 31) / 32) * 32;
  if (threads > 256) threads = 256;
  dim3 grid(n_tokens, n_heads + 2 * n_kv);
#define PKV_ROPE(A, C)                                                                                           \
  return launch_kernel(rope_kv_store_kernel<A, C>, grid, dim3(threads), 0, s, true, 0, (A*)qkv, positions, cos_t, \
                       sin_t, (C*)k_pool, (C*)v_pool, slots, n_heads, n_kv, hd, page_size, store, num_slots, max_pos, status)
  if (act_dtype == PKV_F32 && cache_dtype == PKV_F32) PKV_ROPE(float, float);
  if (act_dtype == PKV_BF16 && cache_dtype == PKV_BF16) PKV_ROPE(bf16, bf16);
  if (act_dtype == PKV_F32 && cache_dtype == PKV_BF16) PKV_ROPE(float, bf16);
  if (act_dtype == PKV_BF16 && cache_dtype == PKV_F32) PKV_ROPE(bf16, float);
#undef PKV_ROPE
  return PKV_ERR_DTYPE;
}

// ---------------------------------------------------------------------------------------------
// copy of one cache page (copy-on-write): in both pools, for every layer of a page group, page
// `src` is copied onto page `dst`. A page of one layer is one contiguous run of `page_bytes`
// bytes (a multiple of 4); layers are `layer_stride_bytes` apart. One launch instead of two
// strided copies per pool (reference: src/paged_kv_serving/engine/runner.py:128-133).
// ---------------------------------------------------------------------------------------------
namespace pkv {

template <typename V>
__global__ void copy_page_kernel(uint8_t* __restrict__ k_pool, uint8_t* __restrict__ v_pool, long long layer_stride_bytes,
                                 long long page_bytes, long long src, long long dst) {
  dependents_may_launch();
  wait_for_prior_kernels();
  uint8_t* pool = (blockIdx.y & 1) ? v_pool : k_pool;
  const long long layer = blockIdx.y >> 1;
  const V* from = reinterpret_cast<const V*>(pool + layer * layer_stride_bytes + src * page_bytes);
  V* to = reinterpret_cast<V*>(pool + layer * layer_stride_bytes + dst * page_bytes);
  const long long n = page_bytes / (long long)sizeof(V);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    to[i] = from[i];
}

}  // namespace pkv

PKV_EXPORT int pkv_copy_page(void* k_pool, void* v_pool, int layers, long long layer_stride_bytes, long long page_bytes,
                             long long pages, long long src, long long dst, void* stream) {
  if (layers <= 0 || page_bytes <= 0 || page_bytes % 4 != 0 || layers > 32767) return PKV_ERR_SIZE;
  if (src < 0 || dst < 0 || src >= pages || dst >= pages || src == dst) return PKV_ERR_SIZE;
  if (layer_stride_bytes < pages * page_bytes) return PKV_ERR_SIZE;
  cudaStream_t s = (cudaStream_t)stream;
  const bool wide = page_bytes % 16 == 0 && layer_stride_bytes % 16 == 0 &&
                    (((uintptr_t)k_pool | (uintptr_t)v_pool) & 15) == 0;
  const long long units = page_bytes / (wide ? 16 : 4);
  int bx = (int)((units + 255) / 256);
  if (bx > 32) bx = 32;
  dim3 grid(bx, 2 * layers);
  if (wide)
    return launch_kernel(copy_page_kernel<uint4>, grid, dim3(256), 0, s, true, 0, (uint8_t*)k_pool, (uint8_t*)v_pool,
                         layer_stride_bytes, page_bytes, src, dst);
  return launch_kernel(copy_page_kernel<uint32_t>, grid, dim3(256), 0, s, true, 0, (uint8_t*)k_pool, (uint8_t*)v_pool,
                       layer_stride_bytes, page_bytes, src, dst);
}
