// Split-KV decode attention fed by TMA: the memory-bound twin of the decode kernel in
// attention_bf16.cu for the common sizes (bfloat16, head size 64 or 128, pages of 8k keys).
//
// What it computes restates the reference (rouviere-german/paged-kv-serving,
// src/paged_kv_serving/engine/attention.py:83-121): scores = q.k * scale, keys after the query's
// absolute position masked, online softmax folded tile by tile, output acc / sum; every entry
// over its own block table (src/paged_kv_serving/engine/runner.py:198-212).
//
// A decode step reads each cached key and value once and does little arithmetic on it, so the
// kernel is built around keeping many bytes in flight per SM. One block per (split of the key
// range, key/value head, entry): two producer warps walk the block table and issue one TMA box per
// page and 64-column panel into a ring of up to six 64-key stages (128-byte swizzle, completion on
// mbarriers); four consumer warps each take 16 keys of every stage with mma.sync (the at most 16
// (query token, head in group) rows of the entry form one MMA row tile), keep their own running
// (maximum, sum, accumulator) and hand the stage back. Warps are merged through shared memory;
// the splits of one entry are the blocks of a thread-block cluster, and the first block merges
// them: the others push their states into its shared memory and leave (or, when the states do
// not fit there, it fetches them out of theirs).
// Every mbarrier wait is bounded; a give-up sets status code 2 and the block leaves in order.
// Build switches for comparisons: -DDT_PRODUCERS=1 (one producer warp), -DDT_NO_PUSH (always
// fetch the other splits' states).
#include <cooperative_groups.h>

#include "attention_decode_common.cuh"

namespace cg = cooperative_groups;

namespace pkv {

#ifndef DT_PRODUCERS
#define DT_PRODUCERS 2
#endif
constexpr int DT_THREADS = 128 + 32 * DT_PRODUCERS;    // four consumer warps and the producer warps
constexpr int DT_TABLE_CACHE = 512;

struct DecTmaParams {
  const bf16* qkv;
  int q_row_stride;
  bf16* out;
  const int32_t* block_table;
  int table_stride;
  const int32_t* seq_starts;
  const int32_t* first_pos;
  const int32_t* work_seq;
  int n_heads, n_kv, page_size, page_shift, window;
  float scale_log2;
  int num_splits;
  int pool_rows;
  int* status;
  int landing_floats;           // room behind the ring for the states the other splits push (0: they are fetched)
};

// Pushing a split's state into the first block of its cluster: a store into that block's shared
// memory which counts its bytes on that block's mbarrier when it has landed.
__device__ __forceinline__ uint32_t in_first_block(uint32_t local_addr) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, 0;" : "=r"(remote) : "r"(local_addr));
  return remote;
}
__device__ __forceinline__ void push_f32(uint32_t remote, float v, uint32_t remote_bar) {
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.f32 [%0], %1, [%2];"
               ::"r"(remote), "f"(v), "r"(remote_bar) : "memory");
}

constexpr int DT_LANDING_FLOATS = 2640;   // in the first block, for the other splits' states (six splits of four rows of 128)

template <int HD, int STAGES>
__global__ void __launch_bounds__(DT_THREADS)
attention_decode_tma_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                            const DecTmaParams p) {
  constexpr int PANELS = HD / 64;
  constexpr uint32_t PANEL_BYTES = DT_BN * 128;                 // 64 keys x 128 bytes
  constexpr uint32_t HALF_BYTES = PANELS * PANEL_BYTES;         // the keys (or the values) of a stage
  constexpr uint32_t STAGE_BYTES = 2 * HALF_BYTES;
  constexpr int KSTEPS = HD / 16;
  constexpr int DTILES = HD / 8;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t full_bar[STAGES], empty_bar[STAGES];
  __shared__ float warp_m[4][DT_ROWS], warp_l[4][DT_ROWS];
  __shared__ float part_m[DT_ROWS], part_l[DT_ROWS];
  __shared__ int32_t table_cache[DT_TABLE_CACHE];
  __shared__ int abort_flag;
  __shared__ __align__(8) uint64_t landing_bar;
  float* landing = reinterpret_cast<float*>(ring + (size_t)STAGES * STAGE_BYTES);   // p.landing_floats, behind the ring

  const int split = blockIdx.x, kvh = blockIdx.y, s = p.work_seq[blockIdx.z];
  const int group = p.n_heads / p.n_kv;
  const int tok0 = p.seq_starts[s];
  const int n_q = p.seq_starts[s + 1] - tok0;
  const int pos0 = p.first_pos[s];
  const int rows_valid = n_q * group;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t4 = lane & 3;

  const int key_hi = pos0 + n_q;
  const int key_lo = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
  const int tile_first = key_lo / DT_BN, tile_last = (key_hi - 1) / DT_BN;
  const int tiles_per_split = (tile_last - tile_first + p.num_splits) / p.num_splits;
  const int tile_begin = tile_first + split * tiles_per_split;
  const int tile_end = min(tile_last, tile_begin + tiles_per_split - 1);
  const int n_tiles = max(0, tile_end - tile_begin + 1);
  const int32_t* table = p.block_table + (size_t)s * p.table_stride;

  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_k)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_v)) : "memory");
    abort_flag = 0;
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(&full_bar[i], DT_PRODUCERS);   // every producer warp announces its own bytes
      mbar_init(&empty_bar[i], 4);          // one arrival per consumer warp
    }
    mbar_init(&landing_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // The splits of an entry are the blocks of one cluster. When their states fit, the other
  // blocks push them into the first block's `landing` (rows x HD sums, then the rows' maxima and
  // weights) and leave; the first block has announced the bytes and waits for them. Otherwise it
  // fetches the states out of the others' shared memory between two cluster barriers.
  const int slot_floats = rows_valid * (HD + 2);
#ifdef DT_NO_PUSH
  const bool push = false;
#else
  const bool push = p.num_splits > 1 && (p.num_splits - 1) * slot_floats <= p.landing_floats;
#endif
  if (push) {
    if (split == 0 && threadIdx.x == 0) mbar_expect_tx(&landing_bar, (uint32_t)((p.num_splits - 1) * slot_floats * 4));
  }
  const int entry_first = n_tiles ? (p.page_shift >= 0 ? (tile_begin * DT_BN) >> p.page_shift : (tile_begin * DT_BN) / p.page_size) : 0;
  const int entry_last = n_tiles ? (p.page_shift >= 0 ? (min(key_hi, (tile_end + 1) * DT_BN) - 1) >> p.page_shift
                                                      : (min(key_hi, (tile_end + 1) * DT_BN) - 1) / p.page_size) : -1;
  const bool table_cached = entry_last - entry_first + 1 <= DT_TABLE_CACHE;
  if (table_cached)
    for (int i = threadIdx.x; i <= entry_last - entry_first; i += DT_THREADS) table_cache[i] = table[entry_first + i];
  __syncthreads();
  // the first block's barrier is ready before anyone pushes: arrive here, wait before pushing
  if (push) asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  // Up to here only the step's index arrays were read, which the host wrote before the step's
  // first kernel. The queries and the newest keys and values come from the kernel before this one.
  wait_for_prior_kernels();
  volatile int* aborted = &abort_flag;

  DecodeState<HD> st;
  st.reset();
  float (&o)[DTILES][4] = st.o;
  float &m_a = st.m_a, &m_b = st.m_b, &l_a = st.l_a, &l_b = st.l_b;

  if (warp >= 4) {
    // ------------------------------------------------------------------------ producers
    // Issuing the boxes of a tile takes a warp about a microsecond at 16 boxes, more than the
    // consumers need for the tile: the producer warps share the boxes.
    const int pw = warp - 4;
    const int pages_per_tile = DT_BN / p.page_size;
    // one box per page and panel, or (two panels) one box per page over both panels
    constexpr int BOX_PANELS = PANELS == 2 ? 2 : 1, BOXES_PER_PAGE = PANELS / BOX_PANELS;
    const int boxes = pages_per_tile * BOXES_PER_PAGE * 2;      // keys and values
    const int my_boxes = (boxes - pw + DT_PRODUCERS - 1) / DT_PRODUCERS;
    const uint32_t my_bytes = (uint32_t)my_boxes * p.page_size * 128 * BOX_PANELS;
    // at most 32 boxes a tile (pages of 8 keys, two panels, keys and values): one box a lane,
    // and what does not change from tile to tile is worked out once
    const int b = pw + lane * DT_PRODUCERS;
    const bool has_box = b < boxes;
    const int which = b / (pages_per_tile * BOXES_PER_PAGE);              // 0: keys, 1: values
    const int rest = b - which * pages_per_tile * BOXES_PER_PAGE;
    const int page_in_tile = rest / BOXES_PER_PAGE, pn = rest - page_in_tile * BOXES_PER_PAGE;
    const int key_in_tile = page_in_tile * p.page_size;
    const uint32_t dst_offset = which * HALF_BYTES +
                                (PANELS == 2 ? (uint32_t)(key_in_tile >> 3) * 2048 : pn * PANEL_BYTES + key_in_tile * 128);
    const CUtensorMap* map = which ? &map_v : &map_k;
    bool ok = true;
    int issued = 0;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int stage = j % STAGES;
      if (lane == 0) {
        if (j >= STAGES && !mbar_wait(&empty_bar[stage], ((j / STAGES) - 1) & 1, aborted)) ok = false;
        if (ok) mbar_expect_tx(&full_bar[stage], my_bytes);
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) break;
      if (has_box) {
        const int pos = (tile_begin + j) * DT_BN + key_in_tile;
        int row = p.pool_rows;                                     // outside the pool: zeros
        if (pos < key_hi && pos + p.page_size > key_lo) {
          const int e = p.page_shift >= 0 ? pos >> p.page_shift : pos / p.page_size;
          const int page = table_cached ? table_cache[e - entry_first] : table[e];
          row = checked_pool_row(page, p.n_kv, kvh, p.page_size, p.pool_rows, p.status);
        }
        if (PANELS == 2) tma_load_4d(ring + (size_t)stage * STAGE_BYTES + dst_offset, map, &full_bar[stage], 0, 0, 0, row >> 3);
        else tma_load_2d(ring + (size_t)stage * STAGE_BYTES + dst_offset, map, &full_bar[stage], 64 * pn, row);
      }
      __syncwarp();
      issued = j + 1;
    }
    if (lane == 0 && *aborted) {
      const long long start = clock64();
      for (int j = max(0, issued - STAGES); j < issued; ++j)
        while (!mbar_try_wait(&full_bar[j % STAGES], (j / STAGES) & 1) && clock64() - start < GM_WAIT_CYCLES) {}
    }
  } else {
    // ------------------------------------------------------------------------ consumers
    // queries of this warp's MMA row tile, straight from global memory into A fragments
    uint32_t qa[KSTEPS][4];
    {
      const int ra = g, rb = g + 8;
      const bf16* pa = nullptr;
      const bf16* pb = nullptr;
      if (ra < rows_valid) pa = p.qkv + (size_t)(tok0 + ra / group) * p.q_row_stride + (size_t)(kvh * group + ra % group) * HD;
      if (rb < rows_valid) pb = p.qkv + (size_t)(tok0 + rb / group) * p.q_row_stride + (size_t)(kvh * group + rb % group) * HD;
#pragma unroll
      for (int kk = 0; kk < KSTEPS; ++kk) {
        qa[kk][0] = pa ? *reinterpret_cast<const uint32_t*>(pa + kk * 16 + 2 * t4) : 0u;
        qa[kk][1] = pb ? *reinterpret_cast<const uint32_t*>(pb + kk * 16 + 2 * t4) : 0u;
        qa[kk][2] = pa ? *reinterpret_cast<const uint32_t*>(pa + kk * 16 + 8 + 2 * t4) : 0u;
        qa[kk][3] = pb ? *reinterpret_cast<const uint32_t*>(pb + kk * 16 + 8 + 2 * t4) : 0u;
      }
    }
    const int row_a = g, row_b = g + 8;
    const int qpos_a = pos0 + row_a / group, qpos_b = pos0 + row_b / group;
    bool ok = true;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int stage = j % STAGES;
      ok = __all_sync(0xffffffffu, mbar_wait(&full_bar[stage], (j / STAGES) & 1, aborted) ? 1 : 0) != 0;
      if (!ok) break;
      const int wbase = (tile_begin + j) * DT_BN + warp * 16;
      decode_tile<HD>(ring + (size_t)stage * STAGE_BYTES, warp, lane, qa, st, wbase, key_lo, key_hi, qpos_a, qpos_b,
                      p.window, p.scale_log2);
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_bar[stage]);     // this warp is done with the stage
    }
  }

  // ---- merge the four consumer warps (each saw a quarter of the keys) ----
  __syncthreads();           // every copy that was waited for has landed; the ring is free
  constexpr int OS = HD + 4;   // row stride of o_s: four floats on, the rows of a warp's store fall into different banks
  float* o_s = reinterpret_cast<float*>(ring);                       // [4][DT_ROWS][OS]
  float* part_o = o_s + 4 * DT_ROWS * OS;                            // [DT_ROWS][HD]
  if (warp < 4) {
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 1); l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 1); l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
    if (t4 == 0) {
      warp_m[warp][g] = m_a; warp_m[warp][g + 8] = m_b;
      warp_l[warp][g] = l_a; warp_l[warp][g + 8] = l_b;
    }
#pragma unroll
    for (int i = 0; i < DTILES; ++i) {
      float* da = o_s + ((size_t)warp * DT_ROWS + g) * OS + i * 8 + 2 * t4;
      float* db = o_s + ((size_t)warp * DT_ROWS + g + 8) * OS + i * 8 + 2 * t4;
      if (g < rows_valid) { da[0] = o[i][0]; da[1] = o[i][1]; }
      if (g + 8 < rows_valid) { db[0] = o[i][2]; db[1] = o[i][3]; }
    }
  }
  __syncthreads();
  if (push) asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");   // passed long ago
  const uint32_t landing_bar_remote = in_first_block(smem_addr(&landing_bar));
  const size_t out_stride = (size_t)p.n_heads * HD;
  for (int idx = threadIdx.x; idx < rows_valid * HD; idx += DT_THREADS) {
    const int row = idx / HD, d = idx - row * HD;
    const float m = fmaxf(fmaxf(warp_m[0][row], warp_m[1][row]), fmaxf(warp_m[2][row], warp_m[3][row]));
    float l = 0.0f, acc = 0.0f;
    if (m > -INFINITY) {
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float f = exp2f(warp_m[w][row] - m);
        l += warp_l[w][row] * f;
        acc += o_s[((size_t)w * DT_ROWS + row) * OS + d] * f;
      }
    }
    if (p.num_splits == 1) {
      const int q_local = row / group, head = kvh * group + row % group;
      p.out[(size_t)(tok0 + q_local) * out_stride + (size_t)head * HD + d] = from_float<bf16>(l > 0.0f ? acc / l : 0.0f);
    } else if (push && split > 0) {
      const uint32_t slot = smem_addr(landing) + (uint32_t)((split - 1) * slot_floats) * 4u;
      push_f32(in_first_block(slot + (uint32_t)(row * HD + d) * 4u), acc, landing_bar_remote);
      if (d == 0) {
        push_f32(in_first_block(slot + (uint32_t)(rows_valid * HD + 2 * row) * 4u), m, landing_bar_remote);
        push_f32(in_first_block(slot + (uint32_t)(rows_valid * HD + 2 * row + 1) * 4u), l, landing_bar_remote);
      }
    } else {
      part_o[row * HD + d] = acc;
      if (d == 0) {
        part_m[row] = m;
        part_l[row] = l;
      }
    }
  }
  __shared__ float weight[8][DT_ROWS];    // per row, the weight of every split's sums: exp2(m_r - M) / L
  if (push && split == 0) {
    __syncthreads();                                   // this block's own state is in part_o, part_m, part_l
    bool landed = mbar_wait(&landing_bar, 0, aborted);  // the others' states have landed
    if (!landed) {
      // given up elsewhere in this block: the others still push, and this block's shared memory
      // must outlive their stores
      const long long start = clock64();
      while (!mbar_try_wait(&landing_bar, 0) && clock64() - start < GM_WAIT_CYCLES) {}
    }
    if (landed) {
      if (threadIdx.x < rows_valid) {
        const int row = threadIdx.x;
        float mr[8], lr[8];
        mr[0] = part_m[row]; lr[0] = part_l[row];
#pragma unroll
        for (int r = 1; r < 8; ++r) {
          const float* ml = landing + (r - 1) * slot_floats + rows_valid * HD + 2 * row;
          mr[r] = r < p.num_splits ? ml[0] : -INFINITY;
          lr[r] = r < p.num_splits ? ml[1] : 0.0f;
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
      for (int idx = threadIdx.x; idx < rows_valid * HD; idx += DT_THREADS) {
        const int row = idx / HD, d = idx - row * HD;
        float acc = part_o[row * HD + d] * weight[0][row];
#pragma unroll
        for (int r = 1; r < 8; ++r)
          if (r < p.num_splits) acc += landing[(r - 1) * slot_floats + row * HD + d] * weight[r][row];
        const int q_local = row / group, head = kvh * group + row % group;
        p.out[(size_t)(tok0 + q_local) * out_stride + (size_t)head * HD + d] = from_float<bf16>(acc);
      }
    }
  } else if (p.num_splits > 1 && !push) {
    // the splits of this (entry, kv head) are the blocks of one cluster: block 0 folds the others'
    // states out of their shared memory
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();
    if (split == 0) {
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
      for (int idx = threadIdx.x; idx < rows_valid * HD; idx += DT_THREADS) {
        const int row = idx / HD, d = idx - row * HD;
        float part[8];
#pragma unroll
        for (int r = 0; r < 8; ++r) part[r] = r < p.num_splits ? *cluster.map_shared_rank(&part_o[row * HD + d], r) : 0.0f;
        float acc = 0.0f;
#pragma unroll
        for (int r = 0; r < 8; ++r) acc += part[r] * weight[r][row];
        const int q_local = row / group, head = kvh * group + row % group;
        p.out[(size_t)(tok0 + q_local) * out_stride + (size_t)head * HD + d] = from_float<bf16>(acc);
      }
    }
    cluster.sync();
  }
  // Only now may the next kernel start: launched while blocks of this kernel were still merging,
  // the product that follows ran 50 us longer; launched here, it gains its launch time.
  dependents_may_launch();
  if (threadIdx.x == 0 && abort_flag) atomicExch(p.status, 2);
}

template <int HD, int STAGES>
static size_t dec_smem() { return (size_t)STAGES * 2 * (HD / 64) * DT_BN * 128 + 1024; }

template <int HD, int STAGES>
static int launch_dec(const CUtensorMap& mk, const CUtensorMap& mv, const DecTmaParams& p, int n_work, cudaStream_t s) {
  const size_t most = dec_smem<HD, STAGES>() + DT_LANDING_FLOATS * sizeof(float);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_decode_tma_kernel<HD, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)most);
    if (e != cudaSuccess) return (int)e;
    // two blocks per SM need nearly all of its memory as shared memory; left to itself the
    // driver may choose a division in which only one fits
    e = cudaFuncSetAttribute(attention_decode_tma_kernel<HD, STAGES>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const size_t smem = dec_smem<HD, STAGES>() + (size_t)p.landing_floats * sizeof(float);
  return launch_kernel(attention_decode_tma_kernel<HD, STAGES>, dim3(p.num_splits, p.n_kv, n_work), dim3(DT_THREADS), smem, s,
                       true, p.num_splits, mk, mv, p);
}

}  // namespace pkv

using namespace pkv;

// 1 when this kernel takes the sizes (else the decode kernel of attention_bf16.cu serves them)
PKV_EXPORT int pkv_attention_decode_tma_supports(int hd, int page_size, int q_row_stride) {
  return ((hd == 64 || hd == 128) && page_size >= 8 && page_size % 8 == 0 && DT_BN % page_size == 0 &&
          q_row_stride % 2 == 0) ? 1 : 0;
}

// Blocks of this kernel that fit on one SM (the host sizes the number of splits with it).
template <int HD, int STAGES> static int dec_blocks_per_sm() {
  int blocks = 0;
  const size_t smem = dec_smem<HD, STAGES>();      // without room for pushed states (one split needs none)
  cudaFuncSetAttribute(attention_decode_tma_kernel<HD, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                       (int)(smem + DT_LANDING_FLOATS * sizeof(float)));
  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, attention_decode_tma_kernel<HD, STAGES>, DT_THREADS, smem);
  return blocks;
}

// Most splits whose states the first block of a cluster can take in its shared memory (the
// faster way to merge them) for entries of `rows` (query token, head in group) rows.
PKV_EXPORT int pkv_attention_decode_tma_pushed_splits(int hd, int rows) {
  return rows > 0 ? 1 + DT_LANDING_FLOATS / (rows * (hd + 2)) : 1;
}

PKV_EXPORT int pkv_attention_decode_tma_blocks_per_sm(int hd, int deep_ring) {
  if (hd == 128) return deep_ring ? dec_blocks_per_sm<128, 6>() : dec_blocks_per_sm<128, 3>();
  if (hd == 64) return deep_ring ? dec_blocks_per_sm<64, 6>() : dec_blocks_per_sm<64, 3>();
  return 0;
}

PKV_EXPORT int pkv_attention_decode_tma(const void* qkv, int q_row_stride, void* out, const void* k_pool,
                                        const void* v_pool, long long n_pages, const int32_t* block_table,
                                        int table_stride, const int32_t* seq_starts, const int32_t* first_pos,
                                        const int32_t* work_seq, int n_work, int max_entry_tokens, int n_heads, int n_kv,
                                        int hd, int page_size, int window, float scale, int num_splits, int deep_ring,
                                        int* status, void* stream) {
  if (n_work <= 0) return 0;
  if (!pkv_attention_decode_tma_supports(hd, page_size, q_row_stride)) return PKV_ERR_LIMIT;
  if (n_heads <= 0 || n_kv <= 0 || n_heads % n_kv || window < 0) return PKV_ERR_SIZE;
  if (num_splits < 1 || num_splits > 8 || n_work > 65535 || n_kv > 65535) return PKV_ERR_LIMIT;
  if (max_entry_tokens * (n_heads / n_kv) > DT_ROWS) return PKV_ERR_LIMIT;
  const long long pool_rows = n_pages * n_kv * page_size;
  if (pool_rows >= (1LL << 31) - page_size) return PKV_ERR_LIMIT;
  if ((uintptr_t)qkv % 4 || (uintptr_t)k_pool % 16 || (uintptr_t)v_pool % 16) return PKV_ERR_ALIGN;
  alignas(64) CUtensorMap map_k, map_v;
  if (!decode_pool_map(k_pool, pool_rows, hd, page_size, &map_k) || !decode_pool_map(v_pool, pool_rows, hd, page_size, &map_v))
    return PKV_ERR_SIZE;
  int shift = -1;
  for (int i = 0; i < 31; ++i)
    if ((1 << i) == page_size) shift = i;
  DecTmaParams p{(const bf16*)qkv, q_row_stride, (bf16*)out, block_table, table_stride, seq_starts, first_pos, work_seq,
                 n_heads, n_kv, page_size, shift, window, scale * 1.4426950408889634f, num_splits, (int)pool_rows, status, 0};
  // room for the pushed states of the largest entry, when that fits beside two blocks per SM
  const int most_floats = (num_splits - 1) * max_entry_tokens * (n_heads / n_kv) * (hd + 2);
  if (num_splits > 1 && most_floats <= DT_LANDING_FLOATS) p.landing_floats = (most_floats + 3) / 4 * 4;
  cudaStream_t s = (cudaStream_t)stream;
  // deep ring: one block per SM with six stages in flight (few blocks, long key ranges);
  // shallow ring: three stages, two blocks per SM, so that one block's start and merge hide
  // behind the other's streaming (many blocks)
  if (hd == 128) return deep_ring ? launch_dec<128, 6>(map_k, map_v, p, n_work, s) : launch_dec<128, 3>(map_k, map_v, p, n_work, s);
  return deep_ring ? launch_dec<64, 6>(map_k, map_v, p, n_work, s) : launch_dec<64, 3>(map_k, map_v, p, n_work, s);
}
