// Paged causal attention, general form: any head size (even, up to 256), any page size, any
// number of heads and key/value groups, float32 or bfloat16 storage, float32 arithmetic.
// It serves the true 32-bit path for prefill and decode alike, and every size the faster
// bfloat16 kernels refuse.
//
// What it computes restates the reference (rouviere-german/paged-kv-serving):
//   src/paged_kv_serving/engine/attention.py:83-121  scores = q.k * scale; a key at a later
//   absolute position than the query is masked; running maximum / sum / accumulator folded tile
//   by tile (online softmax); output acc / sum.
//   src/paged_kv_serving/engine/runner.py:198-212    every entry of a ragged batch attends over
//   its own block table, after the keys and values of the whole batch were written.
// Grouped-query heads (query head h reads key/value head h / (H / KV)) and an optional window
// (keys more than window-1 positions behind the query are masked) generalise it.
//
// Work decomposition: the rows of one (sequence, key/value head) are (query token, head in
// group) pairs, row = token * G + head_in_group. A block of 8 warps takes 8 consecutive rows
// (one warp per row) and walks the keys in tiles of 32 absolute positions, staged once in shared
// memory for all 8 rows. Tiles are aligned to multiples of 32 from position 0 and folded in
// ascending order, and a masked key adds exactly zero, so a row's result does not depend on how
// the batch was cut or on which rows share its block.
#include "common.cuh"

namespace pkv {

constexpr int ATT_WARPS = 8;
constexpr int ATT_TILE = 32;
constexpr int ATT_MAX_ACC = 8;  // head_dim <= 32 * 8

template <typename A, typename C>
__global__ void __launch_bounds__(ATT_WARPS * 32)
paged_attention_generic_kernel(const A* __restrict__ qkv, int q_row_stride, A* __restrict__ out,
                               const C* __restrict__ k_pool, const C* __restrict__ v_pool,
                               const int32_t* __restrict__ block_table, int table_stride,
                               const int32_t* __restrict__ seq_starts, const int32_t* __restrict__ first_pos,
                               const int32_t* __restrict__ work_seq, const int32_t* __restrict__ work_row0,
                               int n_heads, int n_kv, int hd, int page_size, int window, float scale, int num_pages,
                               int* __restrict__ status) {
  extern __shared__ float smem[];
  float* q_s = smem;                              // [ATT_WARPS][hd]
  float* k_s = q_s + ATT_WARPS * hd;              // [ATT_TILE][hd + 1]
  float* v_s = k_s + ATT_TILE * (hd + 1);         // [ATT_TILE][hd]

  const int w = blockIdx.x, kvh = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int s = work_seq[w], row0 = work_row0[w];
  const int tok0 = seq_starts[s];
  const int n_q = seq_starts[s + 1] - tok0;
  const int pos0 = first_pos[s];
  const int group = n_heads / n_kv;
  const int rows_total = n_q * group;

  const int my_row = row0 + warp;
  const bool valid = my_row < rows_total;
  const int q_local = valid ? my_row / group : 0;
  const int head = kvh * group + (valid ? my_row % group : 0);
  const int token = tok0 + q_local;
  const int qpos = pos0 + q_local;

  const int last_row = min(row0 + ATT_WARPS - 1, rows_total - 1);
  const int q_lo = pos0 + row0 / group, q_hi = pos0 + last_row / group;
  const int key_hi = q_hi + 1;                                        // exclusive
  const int key_lo = window > 0 ? max(0, q_lo - window + 1) : 0;      // inclusive
  const int my_lo = window > 0 ? max(0, qpos - window + 1) : 0;

  if (valid) {
    const A* q = qkv + (size_t)token * q_row_stride + (size_t)head * hd;
    for (int d = lane; d < hd; d += 32) q_s[warp * hd + d] = to_float(q[d]);
  }

  float m = -INFINITY, l = 0.0f;
  float acc[ATT_MAX_ACC];
#pragma unroll
  for (int i = 0; i < ATT_MAX_ACC; ++i) acc[i] = 0.0f;

  const int32_t* table = block_table + (size_t)s * table_stride;
  for (int tile = key_lo / ATT_TILE; tile <= (key_hi - 1) / ATT_TILE; ++tile) {
    const int base = tile * ATT_TILE;
    __syncthreads();  // previous tile fully consumed (also orders the q_s writes)
    for (int idx = threadIdx.x; idx < ATT_TILE * hd; idx += ATT_WARPS * 32) {
      const int j = idx / hd, d = idx - j * hd;
      const int pos = base + j;
      float kv = 0.0f, vv = 0.0f;
      if (pos >= key_lo && pos < key_hi) {
        const int page = checked_page(table[pos / page_size], num_pages, status);
        if (page >= 0) {
          const size_t at = (((size_t)page * n_kv + kvh) * page_size + (pos % page_size)) * hd + d;
          kv = to_float(k_pool[at]);
          vv = to_float(v_pool[at]);
        }
      }
      k_s[j * (hd + 1) + d] = kv;
      v_s[j * hd + d] = vv;
    }
    __syncthreads();
    if (!valid || base > qpos || base + ATT_TILE <= my_lo) continue;  // warp-uniform

    const int pos = base + lane;
    float sc = 0.0f;
    const float* qr = q_s + warp * hd;
    const float* kr = k_s + lane * (hd + 1);
    for (int d = 0; d < hd; ++d) sc = fmaf(qr[d], kr[d], sc);
    sc *= scale;
    const bool ok = pos <= qpos && pos >= my_lo;
    sc = ok ? sc : -INFINITY;
    const float tile_max = warp_max(sc);
    if (tile_max == -INFINITY) continue;  // nothing visible in this tile
    const float new_m = fmaxf(m, tile_max);
    const float rescale = expf(m - new_m);       // m = -inf -> 0
    const float p = ok ? expf(sc - new_m) : 0.0f;
    l = l * rescale + warp_sum(p);
#pragma unroll
    for (int i = 0; i < ATT_MAX_ACC; ++i) acc[i] *= rescale;
    for (int j = 0; j < ATT_TILE; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      const float* vr = v_s + j * hd;
#pragma unroll
      for (int i = 0; i < ATT_MAX_ACC; ++i) {
        const int d = lane + 32 * i;
        if (d < hd) acc[i] = fmaf(pj, vr[d], acc[i]);
      }
    }
    m = new_m;
  }

  if (valid) {
    const float denom = l > 0.0f ? l : 1.0f;
    A* o = out + (size_t)token * ((size_t)n_heads * hd) + (size_t)head * hd;
#pragma unroll
    for (int i = 0; i < ATT_MAX_ACC; ++i) {
      const int d = lane + 32 * i;
      if (d < hd) o[d] = from_float<A>(acc[i] / denom);
    }
  }
}

}  // namespace pkv

using namespace pkv;

template <typename A, typename C>
static int launch_generic(const void* qkv, int q_row_stride, void* out, const void* k_pool, const void* v_pool,
                          const int32_t* block_table, int table_stride, const int32_t* seq_starts,
                          const int32_t* first_pos, const int32_t* work_seq, const int32_t* work_row0, int n_work,
                          int n_heads, int n_kv, int hd, int page_size, int window, float scale, int num_pages, int* status,
                          cudaStream_t s) {
  const size_t smem = ((size_t)ATT_WARPS * hd + (size_t)ATT_TILE * (hd + 1) + (size_t)ATT_TILE * hd) * sizeof(float);
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(paged_attention_generic_kernel<A, C>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  dim3 grid(n_work, n_kv);
  paged_attention_generic_kernel<A, C><<<grid, ATT_WARPS * 32, smem, s>>>(
      (const A*)qkv, q_row_stride, (A*)out, (const C*)k_pool, (const C*)v_pool, block_table, table_stride,
      seq_starts, first_pos, work_seq, work_row0, n_heads, n_kv, hd, page_size, window, scale, num_pages, status);
  return launch_status();
}

// Rows per work item, for the host that builds the work list.
PKV_EXPORT int pkv_attention_generic_rows_per_block() { return ATT_WARPS; }

PKV_EXPORT int pkv_paged_attention_generic(const void* qkv, int q_row_stride, void* out, int act_dtype,
                                           const void* k_pool, const void* v_pool, int cache_dtype,
                                           const int32_t* block_table, int table_stride,
                                           const int32_t* seq_starts, const int32_t* first_pos,
                                           const int32_t* work_seq, const int32_t* work_row0, int n_work,
                                           int n_heads, int n_kv, int hd, int page_size, int window, float scale,
                                           int num_pages, int* status, void* stream) {
  if (n_work <= 0) return 0;
  if (n_heads <= 0 || n_kv <= 0 || n_heads % n_kv || hd <= 0 || (hd & 1) || page_size <= 0 || window < 0 || num_pages <= 0)
    return PKV_ERR_SIZE;
  if (hd > 32 * ATT_MAX_ACC || n_kv > 65535) return PKV_ERR_LIMIT;
  cudaStream_t s = (cudaStream_t)stream;
#define PKV_ATT(A, C)                                                                                         \
  return launch_generic<A, C>(qkv, q_row_stride, out, k_pool, v_pool, block_table, table_stride, seq_starts, \
                              first_pos, work_seq, work_row0, n_work, n_heads, n_kv, hd, page_size, window, scale, num_pages, status, s)
  if (act_dtype == PKV_F32 && cache_dtype == PKV_F32) PKV_ATT(float, float);
  if (act_dtype == PKV_BF16 && cache_dtype == PKV_BF16) PKV_ATT(bf16, bf16);
  if (act_dtype == PKV_F32 && cache_dtype == PKV_BF16) PKV_ATT(float, bf16);
  if (act_dtype == PKV_BF16 && cache_dtype == PKV_F32) PKV_ATT(bf16, float);
#undef PKV_ATT
  return PKV_ERR_DTYPE;
}
