// Paged causal attention for bfloat16 on tensor cores: a prefill kernel for long runs of
// queries and a split-KV decode kernel for entries of a few rows, both over block tables.
//
// What they compute restates the reference (rouviere-german/paged-kv-serving):
//   src/paged_kv_serving/engine/attention.py:83-121  scores = q.k * scale, keys after the query's
//   absolute position masked, online softmax folded tile by tile, output acc / sum;
//   src/paged_kv_serving/engine/runner.py:198-212    every entry attends over its own block table.
// Grouped-query heads and an optional window generalise it (see attention_generic.cu, which is
// the float32 twin and takes every size these kernels refuse).
//
// Arithmetic: q, k, v and the probabilities fed to the second product are bfloat16; both
// products accumulate in float32 (mma.sync m16n8k16); scores, maxima, sums, exponentials and the
// output accumulator are float32. Head sizes: multiples of 16 up to 128.
//
// Prefill kernel: one block of 4 warps per (64 query rows of one sequence, query head); each
// warp owns 16 rows; keys are walked in tiles of 64 absolute positions aligned to multiples of 64
// from position 0, double-buffered with cp.async from the pages the block table names.
// Decode kernel: one block per (split of the key range, key/value head, entry); the rows of an
// entry for that head, (query token, head in group) pairs, at most 16, form one MMA row tile that
// all 4 warps share, each warp taking 16 keys of every 64-key tile; warps and then splits are
// merged with the usual (max, sum, accumulator) rule. With more than one split the partial
// results go through scratch memory and a small merge kernel.
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace pkv {

constexpr int AT_BM = 64;       // query rows per prefill block
constexpr int AT_BN = 64;       // keys per tile
constexpr int AT_THREADS = 128;
constexpr int AT_PAD = 8;       // bf16 elements of padding per shared-memory row (16 bytes)
constexpr int DEC_ROWS = 16;    // rows of one decode entry per key/value head
constexpr int PAGE_CACHE = 2048; // block-table entries a block keeps in shared memory

struct AttnParams {
  const bf16* qkv;              // [T, q_row_stride]; queries of head h at column h * HD
  int q_row_stride;
  bf16* out;                    // [T, H * HD]
  const bf16* k_pool;           // [pages, KV, page_size, HD]
  const bf16* v_pool;
  const int32_t* block_table;   // [S, table_stride]
  int table_stride;
  const int32_t* seq_starts;    // [S + 1] first token of each entry in this step
  const int32_t* first_pos;     // [S] absolute position of each entry's first token
  const int32_t* work_a;        // prefill: entry of each work item; decode: entry of each item
  const int32_t* work_b;        // prefill: first query (inside the entry) of each work item
  int n_heads, n_kv, page_size, page_shift, window;   // page_shift: log2(page_size), or -1
  float scale_log2;             // scale * log2(e)
  int num_splits;               // decode only
  int use_cluster;              // decode only: the splits of one (entry, kv head) are one thread-block cluster
  float* part_o;                // decode scratch [T*H, splits, HD]
  float* part_ml;               // decode scratch [T*H, splits, 2]
  int num_pages;                // pages of the pools: table entries are checked against it
  int* status;                  // the device's status word (may be null)
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_u32(smem)), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Load `rows` keys (or values) starting at absolute position `base` into a padded tile.
// Positions outside [lo, hi) and positions whose page was given back are zero-filled.
// The block-table entries of a block's key range, copied to shared memory once: a lookup per
// 16-byte copy from global memory would put a memory latency in front of every copy.
struct PageLookup {
  const int32_t* table;      // the entry's block table in global memory
  const int32_t* cached;     // shared-memory copy of entries [first, first + count), or null
  int first;
  int page_size, page_shift;
  int num_pages;
  int* status;
  __device__ __forceinline__ int entry_of(int pos) const { return page_shift >= 0 ? pos >> page_shift : pos / page_size; }
  __device__ __forceinline__ int page_of(int pos, int& offset) const {
    const int e = entry_of(pos);
    offset = pos - e * page_size;
    return checked_page(cached ? cached[e - first] : table[e], num_pages, status);
  }
};

__device__ __forceinline__ PageLookup make_page_lookup(int32_t* cache, const int32_t* table, int lo, int hi,
                                                       int page_size, int page_shift, int num_pages, int* status) {
  PageLookup look{table, nullptr, 0, page_size, page_shift, num_pages, status};
  if (hi <= lo) return look;
  const int first = look.entry_of(lo), count = look.entry_of(hi - 1) - first + 1;
  if (count <= PAGE_CACHE) {
    for (int i = threadIdx.x; i < count; i += AT_THREADS) cache[i] = table[first + i];
    look.cached = cache;
    look.first = first;
  }
  return look;   // the caller synchronises the block before the first lookup
}

template <int HD>
__device__ __forceinline__ void load_kv_tile(bf16* tile, const bf16* pool, const PageLookup& look, int base, int lo,
                                             int hi, int kvh, int n_kv) {
  constexpr int LD = HD + AT_PAD;
  constexpr int CHUNKS = HD / 8;
  for (int idx = threadIdx.x; idx < AT_BN * CHUNKS; idx += AT_THREADS) {
    const int row = idx / CHUNKS, chunk = idx - row * CHUNKS;
    const int pos = base + row;
    bf16* dst = tile + row * LD + chunk * 8;
    int page = -1, offset = 0;
    if (pos >= lo && pos < hi) page = look.page_of(pos, offset);
    if (page >= 0) {
      const size_t at = (((size_t)page * n_kv + kvh) * look.page_size + offset) * HD + chunk * 8;
      cp_async16(dst, pool + at);
    } else {
      *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// prefill
// ---------------------------------------------------------------------------------------------
template <int HD>
__global__ void __launch_bounds__(AT_THREADS) attention_prefill_kernel(const AttnParams p) {
  constexpr int LD = HD + AT_PAD;
  constexpr int KSTEPS = HD / 16;
  constexpr int DTILES = HD / 8;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* q_s = reinterpret_cast<bf16*>(smem_raw);     // [AT_BM][LD]
  bf16* k_s = q_s + AT_BM * LD;                       // [2][AT_BN][LD]
  bf16* v_s = k_s + 2 * AT_BN * LD;                   // [2][AT_BN][LD]

  const int s = p.work_a[blockIdx.x], q0 = p.work_b[blockIdx.x];
  const int head = blockIdx.y;
  const int kvh = head / (p.n_heads / p.n_kv);
  const int tok0 = p.seq_starts[s];
  const int n_q = p.seq_starts[s + 1] - tok0;
  const int pos0 = p.first_pos[s];
  const int rows_valid = min(AT_BM, n_q - q0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t4 = lane & 3;

  const int qpos_first = pos0 + q0;
  const int key_hi = qpos_first + rows_valid;                                   // exclusive
  const int key_lo = p.window > 0 ? max(0, qpos_first - p.window + 1) : 0;
  const int tile_begin = key_lo / AT_BN, tile_end = (key_hi - 1) / AT_BN;       // inclusive
  __shared__ int32_t page_cache[PAGE_CACHE];
  const PageLookup look = make_page_lookup(page_cache, p.block_table + (size_t)s * p.table_stride, key_lo, key_hi,
                                           p.page_size, p.page_shift, p.num_pages, p.status);

  // queries of this block
  for (int idx = threadIdx.x; idx < AT_BM * (HD / 8); idx += AT_THREADS) {
    const int row = idx / (HD / 8), chunk = idx - row * (HD / 8);
    bf16* dst = q_s + row * LD + chunk * 8;
    if (row < rows_valid)
      cp_async16(dst, p.qkv + (size_t)(tok0 + q0 + row) * p.q_row_stride + (size_t)head * HD + chunk * 8);
    else
      *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
  }
  __syncthreads();   // the page cache is filled
  load_kv_tile<HD>(k_s, p.k_pool, look, tile_begin * AT_BN, key_lo, key_hi, kvh, p.n_kv);
  load_kv_tile<HD>(v_s, p.v_pool, look, tile_begin * AT_BN, key_lo, key_hi, kvh, p.n_kv);
  cp_async_commit();

  // rows of this thread: warp*16 + g and + 8
  const int row_a = warp * 16 + g, row_b = row_a + 8;
  const int qpos_a = qpos_first + row_a, qpos_b = qpos_first + row_b;
  const int warp_qpos_min = qpos_first + warp * 16;
  const int warp_qpos_max = min(qpos_first + warp * 16 + 15, key_hi - 1);
  const bool warp_active = warp * 16 < rows_valid;

  float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.0f, l_b = 0.0f;
  float o[DTILES][4];
#pragma unroll
  for (int i = 0; i < DTILES; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;

  for (int tile = tile_begin; tile <= tile_end; ++tile) {
    const int stage = (tile - tile_begin) & 1;
    const int base = tile * AT_BN;
    if (tile < tile_end) {
      load_kv_tile<HD>(k_s + (stage ^ 1) * AT_BN * LD, p.k_pool, look, base + AT_BN, key_lo, key_hi, kvh, p.n_kv);
      load_kv_tile<HD>(v_s + (stage ^ 1) * AT_BN * LD, p.v_pool, look, base + AT_BN, key_lo, key_hi, kvh, p.n_kv);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const bf16* kt = k_s + stage * AT_BN * LD;
    const bf16* vt = v_s + stage * AT_BN * LD;

    // a warp whose rows all sit before this tile (causal) or after its window has nothing to do
    const bool skip = !warp_active || base > warp_qpos_max ||
                      (p.window > 0 && base + AT_BN - 1 < warp_qpos_min - p.window + 1);
    if (!skip) {
      float sc[AT_BN / 8][4];
#pragma unroll
      for (int j = 0; j < AT_BN / 8; ++j) sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.0f;
#pragma unroll
      for (int kk = 0; kk < KSTEPS; ++kk) {
        uint32_t a[4];
        ldmatrix_x4(a, q_s + (warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * LD + kk * 16 + 8 * (lane >> 4));
#pragma unroll
        for (int jj = 0; jj < AT_BN / 16; ++jj) {
          uint32_t b[4];
          ldmatrix_x4(b, kt + (jj * 16 + (lane & 7) + 8 * (lane >> 4)) * LD + kk * 16 + 8 * ((lane >> 3) & 1));
          mma_bf16(sc[2 * jj], a, b[0], b[1]);
          mma_bf16(sc[2 * jj + 1], a, b[2], b[3]);
        }
      }
      // scale (to the log2 domain) and mask by absolute position
      const bool need_mask = base + AT_BN - 1 > warp_qpos_min ||
                             (p.window > 0 && base < warp_qpos_max - p.window + 1);
      float tmax_a = -INFINITY, tmax_b = -INFINITY;
#pragma unroll
      for (int j = 0; j < AT_BN / 8; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float v = sc[j][e] * p.scale_log2;
          if (need_mask) {
            const int kpos = base + j * 8 + 2 * t4 + (e & 1);
            const int qpos = (e < 2) ? qpos_a : qpos_b;
            const bool ok = kpos <= qpos && (p.window == 0 || kpos > qpos - p.window);
            v = ok ? v : -INFINITY;
          }
          sc[j][e] = v;
          if (e < 2) tmax_a = fmaxf(tmax_a, v); else tmax_b = fmaxf(tmax_b, v);
        }
      }
      tmax_a = fmaxf(tmax_a, __shfl_xor_sync(0xffffffffu, tmax_a, 1));
      tmax_a = fmaxf(tmax_a, __shfl_xor_sync(0xffffffffu, tmax_a, 2));
      tmax_b = fmaxf(tmax_b, __shfl_xor_sync(0xffffffffu, tmax_b, 1));
      tmax_b = fmaxf(tmax_b, __shfl_xor_sync(0xffffffffu, tmax_b, 2));
      const float new_a = fmaxf(m_a, tmax_a), new_b = fmaxf(m_b, tmax_b);
      // a row with nothing visible yet keeps shift 0 so that exp2(-inf - 0) = 0
      const float shift_a = new_a == -INFINITY ? 0.0f : new_a, shift_b = new_b == -INFINITY ? 0.0f : new_b;
      const float resc_a = exp2f(m_a - shift_a), resc_b = exp2f(m_b - shift_b);
      m_a = new_a; m_b = new_b;
      float sum_a = 0.0f, sum_b = 0.0f;
#pragma unroll
      for (int j = 0; j < AT_BN / 8; ++j) {
        sc[j][0] = exp2f(sc[j][0] - shift_a); sc[j][1] = exp2f(sc[j][1] - shift_a);
        sc[j][2] = exp2f(sc[j][2] - shift_b); sc[j][3] = exp2f(sc[j][3] - shift_b);
        sum_a += sc[j][0] + sc[j][1];
        sum_b += sc[j][2] + sc[j][3];
      }
      l_a = l_a * resc_a + sum_a;
      l_b = l_b * resc_b + sum_b;
#pragma unroll
      for (int i = 0; i < DTILES; ++i) { o[i][0] *= resc_a; o[i][1] *= resc_a; o[i][2] *= resc_b; o[i][3] *= resc_b; }
      // O += P V
#pragma unroll
      for (int kk = 0; kk < AT_BN / 16; ++kk) {
        uint32_t a[4];
        a[0] = pack_bf16(sc[2 * kk][0], sc[2 * kk][1]);
        a[1] = pack_bf16(sc[2 * kk][2], sc[2 * kk][3]);
        a[2] = pack_bf16(sc[2 * kk + 1][0], sc[2 * kk + 1][1]);
        a[3] = pack_bf16(sc[2 * kk + 1][2], sc[2 * kk + 1][3]);
#pragma unroll
        for (int dd = 0; dd < DTILES / 2; ++dd) {
          uint32_t b[4];
          ldmatrix_x4_trans(b, vt + (kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * LD + dd * 16 + 8 * (lane >> 4));
          mma_bf16(o[2 * dd], a, b[0], b[1]);
          mma_bf16(o[2 * dd + 1], a, b[2], b[3]);
        }
      }
    }
    __syncthreads();
  }

  // row sums were kept per thread: finish them across the quad, normalise, store
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 1); l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 1); l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
  const float inv_a = l_a > 0.0f ? 1.0f / l_a : 0.0f, inv_b = l_b > 0.0f ? 1.0f / l_b : 0.0f;
  const size_t out_stride = (size_t)p.n_heads * HD;
  if (row_a < rows_valid) {
    bf16* dst = p.out + (size_t)(tok0 + q0 + row_a) * out_stride + (size_t)head * HD;
#pragma unroll
    for (int i = 0; i < DTILES; ++i)
      *reinterpret_cast<uint32_t*>(dst + i * 8 + 2 * t4) = pack_bf16(o[i][0] * inv_a, o[i][1] * inv_a);
  }
  if (row_b < rows_valid) {
    bf16* dst = p.out + (size_t)(tok0 + q0 + row_b) * out_stride + (size_t)head * HD;
#pragma unroll
    for (int i = 0; i < DTILES; ++i)
      *reinterpret_cast<uint32_t*>(dst + i * 8 + 2 * t4) = pack_bf16(o[i][2] * inv_b, o[i][3] * inv_b);
  }
}

// ---------------------------------------------------------------------------------------------
// decode (entries of at most 16 rows per key/value head), split over the key range
// ---------------------------------------------------------------------------------------------
template <int HD>
__global__ void __launch_bounds__(AT_THREADS) attention_decode_kernel(const AttnParams p) {
  wait_for_prior_kernels();
  constexpr int LD = HD + AT_PAD;
  constexpr int KSTEPS = HD / 16;
  constexpr int DTILES = HD / 8;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* q_s = reinterpret_cast<bf16*>(smem_raw);     // [DEC_ROWS][LD]
  bf16* k_s = q_s + DEC_ROWS * LD;                    // [2][AT_BN][LD]
  bf16* v_s = k_s + 2 * AT_BN * LD;                   // [2][AT_BN][LD]
  __shared__ float warp_m[4][DEC_ROWS], warp_l[4][DEC_ROWS];
  __shared__ float part_m[DEC_ROWS], part_l[DEC_ROWS];     // this block's merged state, read by its cluster

  const int split = blockIdx.x, kvh = blockIdx.y, s = p.work_a[blockIdx.z];
  const int group = p.n_heads / p.n_kv;
  const int tok0 = p.seq_starts[s];
  const int n_q = p.seq_starts[s + 1] - tok0;
  const int pos0 = p.first_pos[s];
  const int rows_valid = n_q * group;                  // <= DEC_ROWS by construction of the work list
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t4 = lane & 3;

  const int key_hi = pos0 + n_q;
  const int key_lo = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
  const int tile_first = key_lo / AT_BN, tile_last = (key_hi - 1) / AT_BN;
  const int tiles_per_split = (tile_last - tile_first + p.num_splits) / p.num_splits;
  const int tile_begin = tile_first + split * tiles_per_split;
  const int tile_end = min(tile_last, tile_begin + tiles_per_split - 1);
  __shared__ int32_t page_cache[PAGE_CACHE];
  const PageLookup look = make_page_lookup(page_cache, p.block_table + (size_t)s * p.table_stride,
                                           max(key_lo, tile_begin * AT_BN), min(key_hi, (tile_end + 1) * AT_BN),
                                           p.page_size, p.page_shift, p.num_pages, p.status);

  for (int idx = threadIdx.x; idx < DEC_ROWS * (HD / 8); idx += AT_THREADS) {
    const int row = idx / (HD / 8), chunk = idx - row * (HD / 8);
    bf16* dst = q_s + row * LD + chunk * 8;
    if (row < rows_valid) {
      const int q_local = row / group, head = kvh * group + row % group;
      cp_async16(dst, p.qkv + (size_t)(tok0 + q_local) * p.q_row_stride + (size_t)head * HD + chunk * 8);
    } else {
      *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
    }
  }
  __syncthreads();   // the page cache is filled
  if (tile_begin <= tile_end) {
    load_kv_tile<HD>(k_s, p.k_pool, look, tile_begin * AT_BN, key_lo, key_hi, kvh, p.n_kv);
    load_kv_tile<HD>(v_s, p.v_pool, look, tile_begin * AT_BN, key_lo, key_hi, kvh, p.n_kv);
  }
  cp_async_commit();

  const int row_a = g, row_b = g + 8;
  const int qpos_a = pos0 + row_a / group, qpos_b = pos0 + row_b / group;   // rows beyond rows_valid are never stored
  float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.0f, l_b = 0.0f;
  float o[DTILES][4];
#pragma unroll
  for (int i = 0; i < DTILES; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;

  for (int tile = tile_begin; tile <= tile_end; ++tile) {
    const int stage = (tile - tile_begin) & 1;
    const int base = tile * AT_BN;
    if (tile < tile_end) {
      load_kv_tile<HD>(k_s + (stage ^ 1) * AT_BN * LD, p.k_pool, look, base + AT_BN, key_lo, key_hi, kvh, p.n_kv);
      load_kv_tile<HD>(v_s + (stage ^ 1) * AT_BN * LD, p.v_pool, look, base + AT_BN, key_lo, key_hi, kvh, p.n_kv);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const bf16* kt = k_s + stage * AT_BN * LD + warp * 16 * LD;   // this warp's 16 keys of the tile
    const bf16* vt = v_s + stage * AT_BN * LD + warp * 16 * LD;
    const int wbase = base + warp * 16;
    if (wbase < key_hi && wbase + 15 >= key_lo) {
      float sc[2][4] = {{0.0f, 0.0f, 0.0f, 0.0f}, {0.0f, 0.0f, 0.0f, 0.0f}};
#pragma unroll
      for (int kk = 0; kk < KSTEPS; ++kk) {
        uint32_t a[4], b[4];
        ldmatrix_x4(a, q_s + ((lane & 7) + 8 * ((lane >> 3) & 1)) * LD + kk * 16 + 8 * (lane >> 4));
        ldmatrix_x4(b, kt + ((lane & 7) + 8 * (lane >> 4)) * LD + kk * 16 + 8 * ((lane >> 3) & 1));
        mma_bf16(sc[0], a, b[0], b[1]);
        mma_bf16(sc[1], a, b[2], b[3]);
      }
      float tmax_a = -INFINITY, tmax_b = -INFINITY;
#pragma unroll
      for (int j = 0; j < 2; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int kpos = wbase + j * 8 + 2 * t4 + (e & 1);
          const int qpos = (e < 2) ? qpos_a : qpos_b;
          const bool ok = kpos <= qpos && (p.window == 0 || kpos > qpos - p.window);
          const float v = ok ? sc[j][e] * p.scale_log2 : -INFINITY;
          sc[j][e] = v;
          if (e < 2) tmax_a = fmaxf(tmax_a, v); else tmax_b = fmaxf(tmax_b, v);
        }
      }
      tmax_a = fmaxf(tmax_a, __shfl_xor_sync(0xffffffffu, tmax_a, 1));
      tmax_a = fmaxf(tmax_a, __shfl_xor_sync(0xffffffffu, tmax_a, 2));
      tmax_b = fmaxf(tmax_b, __shfl_xor_sync(0xffffffffu, tmax_b, 1));
      tmax_b = fmaxf(tmax_b, __shfl_xor_sync(0xffffffffu, tmax_b, 2));
      const float new_a = fmaxf(m_a, tmax_a), new_b = fmaxf(m_b, tmax_b);
      const float shift_a = new_a == -INFINITY ? 0.0f : new_a, shift_b = new_b == -INFINITY ? 0.0f : new_b;
      const float resc_a = exp2f(m_a - shift_a), resc_b = exp2f(m_b - shift_b);
      m_a = new_a; m_b = new_b;
      float sum_a = 0.0f, sum_b = 0.0f;
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        sc[j][0] = exp2f(sc[j][0] - shift_a); sc[j][1] = exp2f(sc[j][1] - shift_a);
        sc[j][2] = exp2f(sc[j][2] - shift_b); sc[j][3] = exp2f(sc[j][3] - shift_b);
        sum_a += sc[j][0] + sc[j][1];
        sum_b += sc[j][2] + sc[j][3];
      }
      l_a = l_a * resc_a + sum_a;
      l_b = l_b * resc_b + sum_b;
      uint32_t a[4];
      a[0] = pack_bf16(sc[0][0], sc[0][1]); a[1] = pack_bf16(sc[0][2], sc[0][3]);
      a[2] = pack_bf16(sc[1][0], sc[1][1]); a[3] = pack_bf16(sc[1][2], sc[1][3]);
#pragma unroll
      for (int dd = 0; dd < DTILES / 2; ++dd) {
        uint32_t b[4];
        ldmatrix_x4_trans(b, vt + ((lane & 7) + 8 * ((lane >> 3) & 1)) * LD + dd * 16 + 8 * (lane >> 4));
        o[2 * dd][0] *= resc_a; o[2 * dd][1] *= resc_a; o[2 * dd][2] *= resc_b; o[2 * dd][3] *= resc_b;
        o[2 * dd + 1][0] *= resc_a; o[2 * dd + 1][1] *= resc_a; o[2 * dd + 1][2] *= resc_b; o[2 * dd + 1][3] *= resc_b;
        mma_bf16(o[2 * dd], a, b[0], b[1]);
        mma_bf16(o[2 * dd + 1], a, b[2], b[3]);
      }
    }
    __syncthreads();
  }

  // ---- merge the four warps (each saw a quarter of the keys) ----
  cp_async_wait<0>();   // a split without tiles still has the copy of its queries in flight
  __syncthreads();
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 1); l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 1); l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
  if (t4 == 0) {
    warp_m[warp][row_a] = m_a; warp_m[warp][row_b] = m_b;
    warp_l[warp][row_a] = l_a; warp_l[warp][row_b] = l_b;
  }
  float* o_s = reinterpret_cast<float*>(k_s);          // [4][DEC_ROWS][HD] floats, over the key/value tiles
#pragma unroll
  for (int i = 0; i < DTILES; ++i) {
    float* da = o_s + ((size_t)warp * DEC_ROWS + row_a) * HD + i * 8 + 2 * t4;
    float* db = o_s + ((size_t)warp * DEC_ROWS + row_b) * HD + i * 8 + 2 * t4;
    da[0] = o[i][0]; da[1] = o[i][1];
    db[0] = o[i][2]; db[1] = o[i][3];
  }
  __syncthreads();
  const size_t out_stride = (size_t)p.n_heads * HD;
  for (int idx = threadIdx.x; idx < rows_valid * HD; idx += AT_THREADS) {
    const int row = idx / HD, d = idx - row * HD;
    float m = fmaxf(fmaxf(warp_m[0][row], warp_m[1][row]), fmaxf(warp_m[2][row], warp_m[3][row]));
    float l = 0.0f, acc = 0.0f;
    if (m > -INFINITY) {
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float f = exp2f(warp_m[w][row] - m);     // a warp that saw nothing has m = -inf: factor 0
        l += warp_l[w][row] * f;
        acc += o_s[((size_t)w * DEC_ROWS + row) * HD + d] * f;
      }
    }
    const int q_local = row / group, head = kvh * group + row % group;
    const size_t out_row = (size_t)(tok0 + q_local) * p.n_heads + head;
    if (p.num_splits == 1) {
      p.out[(size_t)(tok0 + q_local) * out_stride + (size_t)head * HD + d] = from_float<bf16>(l > 0.0f ? acc / l : 0.0f);
    } else if (p.use_cluster) {
      reinterpret_cast<float*>(v_s)[row * HD + d] = acc;     // the value tiles are no longer needed
      if (d == 0) {
        part_m[row] = m;
        part_l[row] = l;
      }
    } else {
      p.part_o[(out_row * p.num_splits + split) * HD + d] = acc;
      if (d == 0) {
        p.part_ml[(out_row * p.num_splits + split) * 2] = m;
        p.part_ml[(out_row * p.num_splits + split) * 2 + 1] = l;
      }
    }
  }
  if (p.use_cluster && p.num_splits > 1) {
    // The splits of this (entry, kv head) are the blocks of one cluster: block 0 folds the others'
    // states out of their shared memory (distributed shared memory), no scratch, no second kernel.
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();
    if (split == 0) {
      float* own_o = reinterpret_cast<float*>(v_s);
      // per row: the weight of every split's accumulator, exp2(m_r - M) / L, computed once
      __shared__ float weight[8][DEC_ROWS];
      if (threadIdx.x < rows_valid) {
        const int row = threadIdx.x;
        float mr[8], lr[8];
#pragma unroll
        for (int r = 0; r < 8; ++r) {
          mr[r] = r < p.num_splits ? *cluster.map_shared_rank(&part_m[row], r) : -INFINITY;
          lr[r] = r < p.num_splits ? *cluster.map_shared_rank(&part_l[row], r) : 0.0f;
        }
        float m = -INFINITY;
#pragma unroll
        for (int r = 0; r < 8; ++r) m = fmaxf(m, mr[r]);
        float l = 0.0f;
#pragma unroll
        for (int r = 0; r < 8; ++r) {
          mr[r] = mr[r] > -INFINITY ? exp2f(mr[r] - m) : 0.0f;
          l += lr[r] * mr[r];
        }
        const float inv = l > 0.0f ? 1.0f / l : 0.0f;
#pragma unroll
        for (int r = 0; r < 8; ++r) weight[r][row] = mr[r] * inv;
      }
      __syncthreads();
      for (int idx = threadIdx.x; idx < rows_valid * HD; idx += AT_THREADS) {
        const int row = idx / HD, d = idx - row * HD;
        float part[8];
#pragma unroll
        for (int r = 0; r < 8; ++r) part[r] = r < p.num_splits ? *cluster.map_shared_rank(&own_o[row * HD + d], r) : 0.0f;
        float acc = 0.0f;
#pragma unroll
        for (int r = 0; r < 8; ++r) acc += part[r] * weight[r][row];
        const int q_local = row / group, head = kvh * group + row % group;
        p.out[(size_t)(tok0 + q_local) * out_stride + (size_t)head * HD + d] = from_float<bf16>(acc);
      }
    }
    cluster.sync();     // the others keep their shared memory until block 0 has read it
  }
  dependents_may_launch();   // at the very end: see the note in attention_decode_tma.cu
}

// merge of the splits: one warp per (token, head) output row named by the work list
__global__ void attention_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                       bf16* __restrict__ out, const int32_t* __restrict__ seq_starts,
                                       const int32_t* __restrict__ work_entry, int n_heads, int hd, int num_splits) {
  dependents_may_launch();
  wait_for_prior_kernels();
  const int s = work_entry[blockIdx.y];
  const int tok0 = seq_starts[s], n_q = seq_starts[s + 1] - tok0;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = blockIdx.x * (blockDim.x >> 5) + warp;      // row inside the entry: token * H + head
  if (r >= n_q * n_heads) return;
  const size_t row = (size_t)tok0 * n_heads + r;
  float m = -INFINITY;
  for (int i = 0; i < num_splits; ++i) m = fmaxf(m, part_ml[(row * num_splits + i) * 2]);
  float l = 0.0f;
  for (int i = 0; i < num_splits; ++i) {
    const float mi = part_ml[(row * num_splits + i) * 2];
    if (mi > -INFINITY) l += part_ml[(row * num_splits + i) * 2 + 1] * exp2f(mi - m);
  }
  for (int d = lane; d < hd; d += 32) {
    float acc = 0.0f;
    for (int i = 0; i < num_splits; ++i) {
      const float mi = part_ml[(row * num_splits + i) * 2];
      if (mi > -INFINITY) acc += part_o[(row * num_splits + i) * hd + d] * exp2f(mi - m);
    }
    out[row * hd + d] = from_float<bf16>(l > 0.0f ? acc / l : 0.0f);
  }
}

template <int HD>
static int launch_prefill(const AttnParams& p, int n_work, cudaStream_t s) {
  const size_t smem = (size_t)(AT_BM + 4 * AT_BN) * (HD + AT_PAD) * sizeof(bf16);
  if (smem + (PAGE_CACHE + 256) * sizeof(int32_t) > 48 * 1024) {   // static shared memory counts toward the limit
    cudaError_t e = cudaFuncSetAttribute(attention_prefill_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  attention_prefill_kernel<HD><<<dim3(n_work, p.n_heads), AT_THREADS, smem, s>>>(p);
  return launch_status();
}

template <int HD>
static int launch_decode(const AttnParams& p, int n_work, cudaStream_t s) {
  const size_t smem = (size_t)(DEC_ROWS + 4 * AT_BN) * (HD + AT_PAD) * sizeof(bf16);
  if (smem + (PAGE_CACHE + 256) * sizeof(int32_t) > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(attention_decode_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  const int cluster_x = (p.use_cluster && p.num_splits > 1) ? p.num_splits : 0;
  return launch_kernel(attention_decode_kernel<HD>, dim3(p.num_splits, p.n_kv, n_work), dim3(AT_THREADS), smem, s, true,
                       cluster_x, p);
}

}  // namespace pkv

using namespace pkv;

#define PKV_HD_SWITCH(hd, CALL)          \
  switch (hd) {                          \
    case 16: CALL(16); break;            \
    case 32: CALL(32); break;            \
    case 48: CALL(48); break;            \
    case 64: CALL(64); break;            \
    case 80: CALL(80); break;            \
    case 96: CALL(96); break;            \
    case 112: CALL(112); break;          \
    case 128: CALL(128); break;          \
    default: return PKV_ERR_LIMIT;       \
  }

static int log2_or_minus1(int v) {
  for (int s = 0; s < 31; ++s)
    if ((1 << s) == v) return s;
  return -1;
}

static int check_common(int n_heads, int n_kv, int hd, int page_size, int window, int q_row_stride) {
  if (n_heads <= 0 || n_kv <= 0 || n_heads % n_kv || page_size <= 0 || window < 0) return PKV_ERR_SIZE;
  if (hd % 16 || hd > 128 || hd <= 0) return PKV_ERR_LIMIT;
  if (q_row_stride % 8) return PKV_ERR_ALIGN;          // 16-byte copies of query rows
  if (n_heads > 65535 || n_kv > 65535) return PKV_ERR_LIMIT;
  return 0;
}

// 1 when these kernels take the head size, 0 when the general kernel must be used.
PKV_EXPORT int pkv_attention_bf16_supports(int hd, int q_row_stride) {
  return (hd > 0 && hd % 16 == 0 && hd <= 128 && q_row_stride % 8 == 0) ? 1 : 0;
}

PKV_EXPORT int pkv_attention_bf16_rows(int which) { return which == 0 ? AT_BM : DEC_ROWS; }

// How many decode blocks fit on one SM for this head size (0 when the head size is not taken):
// the host sizes the number of splits so that one wave of blocks covers the work.
template <int HD> static int decode_blocks_per_sm() {
  const size_t smem = (size_t)(DEC_ROWS + 4 * AT_BN) * (HD + AT_PAD) * sizeof(bf16);
  cudaFuncSetAttribute(attention_decode_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  int blocks = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, attention_decode_kernel<HD>, AT_THREADS, smem) != cudaSuccess) return 0;
  return blocks;
}

PKV_EXPORT int pkv_attention_decode_blocks_per_sm(int hd) {
#define CALL(HD) return decode_blocks_per_sm<HD>()
  PKV_HD_SWITCH(hd, CALL)
#undef CALL
  return 0;
}

PKV_EXPORT int pkv_attention_prefill_bf16(const void* qkv, int q_row_stride, void* out, const void* k_pool,
                                          const void* v_pool, const int32_t* block_table, int table_stride,
                                          const int32_t* seq_starts, const int32_t* first_pos,
                                          const int32_t* work_seq, const int32_t* work_q0, int n_work, int n_heads,
                                          int n_kv, int hd, int page_size, int window, float scale, int num_pages,
                                          int* status, void* stream) {
  if (n_work <= 0) return 0;
  const int bad = check_common(n_heads, n_kv, hd, page_size, window, q_row_stride);
  if (bad) return bad;
  if (num_pages <= 0) return PKV_ERR_SIZE;
  AttnParams p{(const bf16*)qkv, q_row_stride, (bf16*)out, (const bf16*)k_pool, (const bf16*)v_pool, block_table,
               table_stride, seq_starts, first_pos, work_seq, work_q0, n_heads, n_kv, page_size, log2_or_minus1(page_size), window,
               scale * 1.4426950408889634f, 1, 0, nullptr, nullptr, num_pages, status};
  cudaStream_t s = (cudaStream_t)stream;
#define CALL(HD) return launch_prefill<HD>(p, n_work, s)
  PKV_HD_SWITCH(hd, CALL)
#undef CALL
  return PKV_ERR_LIMIT;
}

// Floats of scratch the decode kernel needs for `n_rows` (token, head) rows and `num_splits`.
PKV_EXPORT long long pkv_attention_decode_scratch_floats(long long n_rows, int hd, int num_splits) {
  return num_splits <= 1 ? 0 : n_rows * num_splits * (long long)(hd + 2);
}

PKV_EXPORT int pkv_attention_decode_bf16(const void* qkv, int q_row_stride, void* out, const void* k_pool,
                                         const void* v_pool, const int32_t* block_table, int table_stride,
                                         const int32_t* seq_starts, const int32_t* first_pos,
                                         const int32_t* work_seq, int n_work, int max_entry_tokens, int n_heads,
                                         int n_kv, int hd, int page_size, int window, float scale, int num_splits,
                                         float* scratch, long long total_rows, int num_pages, int* status_word,
                                         void* stream) {
  if (n_work <= 0) return 0;
  const int bad = check_common(n_heads, n_kv, hd, page_size, window, q_row_stride);
  if (bad) return bad;
  if (num_pages <= 0) return PKV_ERR_SIZE;
  if (num_splits < 1 || num_splits > 65535 || n_work > 65535) return PKV_ERR_LIMIT;
  if (max_entry_tokens * (n_heads / n_kv) > DEC_ROWS) return PKV_ERR_LIMIT;
  // up to 8 splits (the portable cluster size) merge inside a cluster; more go through scratch
  const int use_cluster = (num_splits > 1 && num_splits <= 8) ? 1 : 0;
  if (num_splits > 1 && !use_cluster && !scratch) return PKV_ERR_SIZE;
  float* part_o = scratch;
  float* part_ml = scratch ? scratch + (size_t)total_rows * num_splits * hd : nullptr;
  AttnParams p{(const bf16*)qkv, q_row_stride, (bf16*)out, (const bf16*)k_pool, (const bf16*)v_pool, block_table,
               table_stride, seq_starts, first_pos, work_seq, nullptr, n_heads, n_kv, page_size, log2_or_minus1(page_size), window,
               scale * 1.4426950408889634f, num_splits, use_cluster, part_o, part_ml, num_pages, status_word};
  cudaStream_t s = (cudaStream_t)stream;
  int status = 0;
#define CALL(HD) status = launch_decode<HD>(p, n_work, s)
  PKV_HD_SWITCH(hd, CALL)
#undef CALL
  if (status || num_splits == 1 || use_cluster) return status;
  const int warps = 4;
  const int rows_max = max_entry_tokens * n_heads;
  return launch_kernel(attention_merge_kernel, dim3((rows_max + warps - 1) / warps, n_work), dim3(warps * 32), 0, s, true, 0,
                       (const float*)part_o, (const float*)part_ml, (bf16*)out, seq_starts, work_seq, n_heads, hd, num_splits);
}
