// Decode attention over even shares of the step's work: the (entry, key/value head, 64-key tile)
// units of all decode entries, laid end to end, are cut into as many equal ranges as the GPU
// holds blocks at once, so that every SM streams the same number of keys whatever the batch size
// and however unequal the contexts. One block per (entry, head, split), the other decode kernel,
// leaves SMs idle when its blocks need a second round that is nearly empty (320 blocks on 296
// places); there this kernel is faster (34 against 37 us at 1,100 keys, 83 against 112 us at
// 4,096, 40 heads). Elsewhere it is not: its parts meet in global memory and all its blocks start
// and end together, which costs about 4 us a launch more than a cluster's shared memory.
//
// What it computes restates the reference (rouviere-german/paged-kv-serving,
// src/paged_kv_serving/engine/attention.py:83-121) as attention_decode_tma.cu does, whose stage
// layout, producer warps and tile step it shares. A block's range may begin and end inside an
// (entry, head) pair and cover whole pairs in between. For every run of tiles of one pair (a
// segment) the four consumer warps fold their keys, merge through shared memory (maxima first,
// then rescaled sums added into one accumulator) and either write the output rows (the segment is
// the whole pair) or leave (sums, maximum, weight) in the block's workspace slot and count the
// pair's arrivals: the block that brings the last part adds them up. Nobody waits for anybody.
// Every mbarrier wait is bounded; a give-up sets status code 2 and the block leaves in order.
#include "attention_decode_common.cuh"

namespace pkv {

constexpr int DF_PRODUCERS = 2;
constexpr int DF_CONSUMER_THREADS = 128;
constexpr int DF_THREADS = DF_CONSUMER_THREADS + 32 * DF_PRODUCERS;
constexpr int DF_STAGES = 3;
constexpr int DF_WEIGHT_PARTS = 32;   // parts of a pair whose merge weights are kept in shared memory

struct DecFlatParams {
  const bf16* qkv;
  int q_row_stride;
  bf16* out;
  const int32_t* block_table;
  int table_stride;
  const int32_t* seq_starts;
  const int32_t* first_pos;
  const int32_t* work_seq;
  const int32_t* unit_starts;   // [n_work + 1]: 64-key tiles of the entries before each entry
  int n_work, n_heads, n_kv, page_size, page_shift, window;
  float scale_log2;
  int pool_rows;
  float* workspace;             // [2 * blocks][DT_ROWS * (HD + 2)]: a block's first and last segment
  int* counters;                // [n_work * n_kv]: parts of a pair that have arrived; zero between launches
  int* status;
};

// One entry as the kernel needs it.
struct FlatEntry {
  int s, tok0, n_q, pos0, key_lo, key_hi, tile_first, tiles;
};
__device__ __forceinline__ FlatEntry flat_entry(const DecFlatParams& p, int w) {
  FlatEntry e;
  e.s = p.work_seq[w];
  e.tok0 = p.seq_starts[e.s];
  e.n_q = p.seq_starts[e.s + 1] - e.tok0;
  e.pos0 = p.first_pos[e.s];
  e.key_hi = e.pos0 + e.n_q;
  e.key_lo = p.window > 0 ? max(0, e.pos0 - p.window + 1) : 0;
  e.tile_first = e.key_lo / DT_BN;
  e.tiles = p.unit_starts[w + 1] - p.unit_starts[w];
  return e;
}

// Even ranges: the first `extra` blocks take `share + 1` units.
__device__ __forceinline__ int range_begin(int b, int share, int extra) { return b * share + min(b, extra); }
__device__ __forceinline__ int range_owner(int u, int share, int extra) {
  const int head = extra * (share + 1);
  return u < head ? u / (share + 1) : extra + (u - head) / max(share, 1);
}

template <int HD>
__global__ void __launch_bounds__(DF_THREADS, 2)
attention_decode_flat_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                             const DecFlatParams p) {
  constexpr int STAGES = DF_STAGES;
  constexpr int PANELS = HD / 64;
  constexpr uint32_t PANEL_BYTES = DT_BN * 128;
  constexpr uint32_t HALF_BYTES = PANELS * PANEL_BYTES;
  constexpr uint32_t STAGE_BYTES = 2 * HALF_BYTES;
  constexpr int KSTEPS = HD / 16;
  constexpr int DTILES = HD / 8;
  constexpr int SLOT_FLOATS = DT_ROWS * (HD + 2);
  extern __shared__ uint8_t smem_raw[];
  uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t full_bar[STAGES], empty_bar[STAGES];
  __shared__ float warp_m[4][DT_ROWS];
  __shared__ float row_l[DT_ROWS], row_m[DT_ROWS], row_scale[DT_ROWS];
  __shared__ __align__(16) float acc_s[DT_ROWS * HD];
  __shared__ float part_weight[DF_WEIGHT_PARTS][DT_ROWS];
  __shared__ int abort_flag, first_work, last_part;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t4 = lane & 3;
  const int group = p.n_heads / p.n_kv;
  const int blocks = gridDim.x, b = blockIdx.x;
  const int total = p.n_kv * p.unit_starts[p.n_work];
  const int share = total / blocks, extra = total - share * blocks;
  const int u0 = range_begin(b, share, extra), u1 = range_begin(b + 1, share, extra);

  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_k)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&map_v)) : "memory");
    abort_flag = 0;
    first_work = 0;
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(&full_bar[i], DF_PRODUCERS);   // every producer warp announces its own bytes
      mbar_init(&empty_bar[i], 4);             // one arrival per consumer warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  for (int i = threadIdx.x; i < DT_ROWS * HD; i += DF_THREADS) acc_s[i] = 0.0f;
  if (threadIdx.x < DT_ROWS) row_l[threadIdx.x] = 0.0f;
  __syncthreads();
  // the entry in which this block's range begins
  if (u0 < u1)
    for (int w = threadIdx.x; w < p.n_work; w += DF_THREADS)
      if (p.n_kv * p.unit_starts[w] <= u0 && u0 < p.n_kv * p.unit_starts[w + 1]) first_work = w;
  __syncthreads();
  volatile int* aborted = &abort_flag;

  if (u0 < u1) {
    // every thread walks the same segments: (entry w, head kvh, tiles [t, t + len) of the entry)
    int w = first_work;
    FlatEntry e = flat_entry(p, w);
    const int into = u0 - p.n_kv * p.unit_starts[w];
    int kvh = into / max(e.tiles, 1);
    int t = into - kvh * e.tiles;
    int left = u1 - u0;
    int j = 0;                      // tiles of this block so far: the ring's clock

    if (warp >= 4) {
      // ---------------------------------------------------------------------- producers
      wait_for_prior_kernels();     // the newest keys and values come from the kernel before this one
      const int pw = warp - 4;
      const int pages_per_tile = DT_BN / p.page_size;
      // one box per page and panel, or (two panels) one box per page over both panels
      constexpr int BOX_PANELS = PANELS == 2 ? 2 : 1, BOXES_PER_PAGE = PANELS / BOX_PANELS;
      const int boxes = pages_per_tile * BOXES_PER_PAGE * 2;      // keys and values
      const int my_boxes = (boxes - pw + DF_PRODUCERS - 1) / DF_PRODUCERS;
      const uint32_t my_bytes = (uint32_t)my_boxes * p.page_size * 128 * BOX_PANELS;
      // at most 32 boxes a tile: one a lane; what does not change from tile to tile is worked out once
      const int box = pw + lane * DF_PRODUCERS;
      const bool has_box = box < boxes;
      const int which = box / (pages_per_tile * BOXES_PER_PAGE);  // 0: keys, 1: values
      const int rest = box - which * pages_per_tile * BOXES_PER_PAGE;
      const int page_in_tile = rest / BOXES_PER_PAGE, pn = rest - page_in_tile * BOXES_PER_PAGE;
      const int key_in_tile = page_in_tile * p.page_size;
      const uint32_t dst_offset = which * HALF_BYTES +
                                  (PANELS == 2 ? (uint32_t)(key_in_tile >> 3) * 2048 : pn * PANEL_BYTES + key_in_tile * 128);
      const CUtensorMap* map = which ? &map_v : &map_k;
      bool ok = true;
      while (left > 0 && ok) {
        const int len = min(e.tiles - t, left);
        const int32_t* table = p.block_table + (size_t)e.s * p.table_stride;
        // the pool row of this lane's box in tile tt
        auto row_of = [&](int tt) {
          const int pos = (e.tile_first + tt) * DT_BN + key_in_tile;
          int row = p.pool_rows;                                     // outside the pool: zeros
          if (has_box && pos < e.key_hi && pos + p.page_size > e.key_lo) {
            const int entry = p.page_shift >= 0 ? pos >> p.page_shift : pos / p.page_size;
            const int page = table[entry];
            row = checked_pool_row(page, p.n_kv, kvh, p.page_size, p.pool_rows, p.status);
          }
          return row;
        };
        // looked up four tiles ahead of their use, so that the reads of the table are never waited for
        int rows_ahead[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) rows_ahead[i] = i < len ? row_of(t + i) : 0;
        for (int tt = t; tt < t + len && ok; tt += 4) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            if (tt + i < t + len && ok) {
              const int stage = j % STAGES;
              const int row = rows_ahead[i];
              if (tt + i + 4 < t + len) rows_ahead[i] = row_of(tt + i + 4);
              if (lane == 0) {
                if (j >= STAGES && !mbar_wait(&empty_bar[stage], ((j / STAGES) - 1) & 1, aborted)) ok = false;
                if (ok) mbar_expect_tx(&full_bar[stage], my_bytes);
              }
              ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
              if (ok) {
                if (has_box) {
                  if (PANELS == 2) tma_load_4d(ring + (size_t)stage * STAGE_BYTES + dst_offset, map, &full_bar[stage], 0, 0, 0, row >> 3);
                  else tma_load_2d(ring + (size_t)stage * STAGE_BYTES + dst_offset, map, &full_bar[stage], 64 * pn, row);
                }
                __syncwarp();
                ++j;
              }
            }
          }
        }
        left -= len;
        t = 0;
        if (++kvh == p.n_kv && left > 0) {
          kvh = 0;
          e = flat_entry(p, ++w);
        }
      }
      if (lane == 0 && *aborted) {   // let the copies in flight land before the shared memory is given up
        const long long start = clock64();
        for (int i = max(0, j - STAGES); i < j; ++i)
          while (!mbar_try_wait(&full_bar[i % STAGES], (i / STAGES) & 1) && clock64() - start < GM_WAIT_CYCLES) {}
      }
    } else {
      // ---------------------------------------------------------------------- consumers
      wait_for_prior_kernels();     // the queries come from the kernel before this one
      const int tid = threadIdx.x;  // 0 .. 127
      DecodeState<HD> st;
      bool ok = true;
      int segment = 0;
      const size_t out_stride = (size_t)p.n_heads * HD;
      while (left > 0) {
        const int len = min(e.tiles - t, left);
        const int rows_valid = e.n_q * group;
        // queries of this segment's rows, straight from global memory into A fragments
        uint32_t qa[KSTEPS][4];
        {
          const int ra = g, rb = g + 8;
          const bf16* pa = nullptr;
          const bf16* pb = nullptr;
          if (ra < rows_valid) pa = p.qkv + (size_t)(e.tok0 + ra / group) * p.q_row_stride + (size_t)(kvh * group + ra % group) * HD;
          if (rb < rows_valid) pb = p.qkv + (size_t)(e.tok0 + rb / group) * p.q_row_stride + (size_t)(kvh * group + rb % group) * HD;
#pragma unroll
          for (int kk = 0; kk < KSTEPS; ++kk) {
            qa[kk][0] = pa ? *reinterpret_cast<const uint32_t*>(pa + kk * 16 + 2 * t4) : 0u;
            qa[kk][1] = pb ? *reinterpret_cast<const uint32_t*>(pb + kk * 16 + 2 * t4) : 0u;
            qa[kk][2] = pa ? *reinterpret_cast<const uint32_t*>(pa + kk * 16 + 8 + 2 * t4) : 0u;
            qa[kk][3] = pb ? *reinterpret_cast<const uint32_t*>(pb + kk * 16 + 8 + 2 * t4) : 0u;
          }
        }
        const int qpos_a = e.pos0 + g / group, qpos_b = e.pos0 + (g + 8) / group;
        st.reset();
        for (int tt = t; tt < t + len; ++tt, ++j) {
          if (!ok) continue;          // given up: no more waits, but every barrier below is still kept
          const int stage = j % STAGES;
          ok = __all_sync(0xffffffffu, mbar_wait(&full_bar[stage], (j / STAGES) & 1, aborted) ? 1 : 0) != 0;
          if (!ok) continue;
          decode_tile<HD>(ring + (size_t)stage * STAGE_BYTES, warp, lane, qa, st, (e.tile_first + tt) * DT_BN + warp * 16,
                          e.key_lo, e.key_hi, qpos_a, qpos_b, p.window, p.scale_log2);
          __syncwarp();
          if (lane == 0) mbar_arrive(&empty_bar[stage]);     // this warp is done with the stage
        }

        // ---- the four warps' states into one (each saw a quarter of the keys) ----
        float l_a = st.l_a, l_b = st.l_b;
        l_a += __shfl_xor_sync(0xffffffffu, l_a, 1); l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
        l_b += __shfl_xor_sync(0xffffffffu, l_b, 1); l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
        if (t4 == 0) {
          warp_m[warp][g] = st.m_a;
          warp_m[warp][g + 8] = st.m_b;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        {
          const float max_a = fmaxf(fmaxf(warp_m[0][g], warp_m[1][g]), fmaxf(warp_m[2][g], warp_m[3][g]));
          const float max_b = fmaxf(fmaxf(warp_m[0][g + 8], warp_m[1][g + 8]), fmaxf(warp_m[2][g + 8], warp_m[3][g + 8]));
          const float f_a = st.m_a > -INFINITY ? exp2f(st.m_a - max_a) : 0.0f;
          const float f_b = st.m_b > -INFINITY ? exp2f(st.m_b - max_b) : 0.0f;
          if (g < rows_valid && f_a > 0.0f) {
#pragma unroll
            for (int i = 0; i < DTILES; ++i) {
              atomicAdd(&acc_s[g * HD + i * 8 + 2 * t4], st.o[i][0] * f_a);
              atomicAdd(&acc_s[g * HD + i * 8 + 2 * t4 + 1], st.o[i][1] * f_a);
            }
            if (t4 == 0) atomicAdd(&row_l[g], l_a * f_a);
          }
          if (g + 8 < rows_valid && f_b > 0.0f) {
#pragma unroll
            for (int i = 0; i < DTILES; ++i) {
              atomicAdd(&acc_s[(g + 8) * HD + i * 8 + 2 * t4], st.o[i][2] * f_b);
              atomicAdd(&acc_s[(g + 8) * HD + i * 8 + 2 * t4 + 1], st.o[i][3] * f_b);
            }
            if (t4 == 0) atomicAdd(&row_l[g + 8], l_b * f_b);
          }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");

        // ---- the whole pair: write its rows; a part of it: leave the state for whoever comes last ----
        const bool whole = len == e.tiles;
        const int pair = w * p.n_kv + kvh;
        float* slot = p.workspace + (size_t)(2 * b + (segment ? 1 : 0)) * SLOT_FLOATS;
        for (int idx = tid; idx < rows_valid * HD; idx += DF_CONSUMER_THREADS) {
          const int row = idx / HD, d = idx - row * HD;
          const float acc = acc_s[idx];
          acc_s[idx] = 0.0f;
          const float l = row_l[row];
          if (whole) {
            const int q_local = row / group, head = kvh * group + row % group;
            p.out[(size_t)(e.tok0 + q_local) * out_stride + (size_t)head * HD + d] = from_float<bf16>(l > 0.0f ? acc / l : 0.0f);
          } else {
            __stcg(slot + idx, acc);
            if (d == 0) {
              __stcg(slot + DT_ROWS * HD + row,
                     fmaxf(fmaxf(warp_m[0][row], warp_m[1][row]), fmaxf(warp_m[2][row], warp_m[3][row])));
              __stcg(slot + DT_ROWS * HD + DT_ROWS + row, l);
            }
          }
        }
        if (!whole) __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (tid < DT_ROWS) row_l[tid] = 0.0f;
        if (!whole) {
          // the blocks that hold parts of this pair are neighbours; each part lies in its block's
          // first slot, except that the block in which the pair begins keeps it in its second
          // one when its range began before the pair
          const int pair_begin = p.n_kv * p.unit_starts[w] + kvh * e.tiles;
          const int b_lo = range_owner(pair_begin, share, extra), b_hi = range_owner(pair_begin + e.tiles - 1, share, extra);
          if (tid == 0) {
            const int before = atomicAdd(&p.counters[pair], 1);
            last_part = before == b_hi - b_lo ? 1 : 0;
            if (last_part) p.counters[pair] = 0;            // ready for the next launch
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (last_part) {
            __threadfence();
            const int n_parts = b_hi - b_lo + 1;
            const int lo_slot = 2 * b_lo + (range_begin(b_lo, share, extra) < pair_begin ? 1 : 0);
            auto slot_of = [&](int part) {
              return p.workspace + (size_t)(part == 0 ? lo_slot : 2 * (b_lo + part)) * SLOT_FLOATS;
            };
            // per row the common maximum, the parts' weights exp2(m_part - M) and 1 / L: a warp
            // takes a row, its lanes the parts, so that the reads of all parts are in flight together
            for (int row = warp; row < rows_valid; row += 4) {
              float m = -INFINITY;
              for (int part = lane; part < n_parts; part += 32) m = fmaxf(m, __ldcg(slot_of(part) + DT_ROWS * HD + row));
#pragma unroll
              for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
              float l = 0.0f;
              for (int part = lane; part < n_parts; part += 32) {
                const float pm = __ldcg(slot_of(part) + DT_ROWS * HD + row);
                const float weight = pm > -INFINITY ? exp2f(pm - m) : 0.0f;
                l += __ldcg(slot_of(part) + DT_ROWS * HD + DT_ROWS + row) * weight;
                if (part < DF_WEIGHT_PARTS) part_weight[part][row] = weight;
              }
#pragma unroll
              for (int off = 16; off > 0; off >>= 1) l += __shfl_xor_sync(0xffffffffu, l, off);
              if (lane == 0) {
                row_m[row] = m;
                row_scale[row] = l > 0.0f ? 1.0f / l : 0.0f;
              }
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            for (int idx = 4 * tid; idx < rows_valid * HD; idx += 4 * DF_CONSUMER_THREADS) {
              const int row = idx / HD, d = idx - row * HD;
              float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll 8
              for (int part = 0; part < min(n_parts, DF_WEIGHT_PARTS); ++part) {
                const float4 v = __ldcg(reinterpret_cast<const float4*>(slot_of(part) + idx));
                const float weight = part_weight[part][row];
                acc.x += v.x * weight; acc.y += v.y * weight; acc.z += v.z * weight; acc.w += v.w * weight;
              }
              for (int part = DF_WEIGHT_PARTS; part < n_parts; ++part) {
                const float pm = __ldcg(slot_of(part) + DT_ROWS * HD + row);
                const float weight = pm > -INFINITY ? exp2f(pm - row_m[row]) : 0.0f;
                const float4 v = __ldcg(reinterpret_cast<const float4*>(slot_of(part) + idx));
                acc.x += v.x * weight; acc.y += v.y * weight; acc.z += v.z * weight; acc.w += v.w * weight;
              }
              const int q_local = row / group, head = kvh * group + row % group;
              const float scale = row_scale[row];
              bf16* dst = p.out + (size_t)(e.tok0 + q_local) * out_stride + (size_t)head * HD + d;
              dst[0] = from_float<bf16>(acc.x * scale); dst[1] = from_float<bf16>(acc.y * scale);
              dst[2] = from_float<bf16>(acc.z * scale); dst[3] = from_float<bf16>(acc.w * scale);
            }
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
        }
        ++segment;
        left -= len;
        t = 0;
        if (++kvh == p.n_kv && left > 0) {
          kvh = 0;
          e = flat_entry(p, ++w);
        }
      }
    }
  } else {
    wait_for_prior_kernels();
  }
  __syncthreads();
  dependents_may_launch();
  if (threadIdx.x == 0 && abort_flag) atomicExch(p.status, 2);
}

template <int HD>
static size_t flat_smem() { return (size_t)DF_STAGES * 2 * (HD / 64) * DT_BN * 128 + 1024; }

template <int HD>
static int launch_flat(const CUtensorMap& mk, const CUtensorMap& mv, const DecFlatParams& p, int blocks, cudaStream_t s) {
  const size_t smem = flat_smem<HD>();
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_decode_flat_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    // two blocks per SM need nearly all of its memory as shared memory; left to itself the
    // driver may choose a division in which only one fits
    e = cudaFuncSetAttribute(attention_decode_flat_kernel<HD>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  return launch_kernel(attention_decode_flat_kernel<HD>, dim3(blocks), dim3(DF_THREADS), smem, s, true, 0, mk, mv, p);
}

template <int HD> static int flat_blocks_per_sm() {
  int blocks = 0;
  const size_t smem = flat_smem<HD>();
  cudaFuncSetAttribute(attention_decode_flat_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, attention_decode_flat_kernel<HD>, DF_THREADS, smem);
  return blocks;
}

}  // namespace pkv

using namespace pkv;

// 1 when this kernel takes the sizes (the same as the TMA decode kernel's)
PKV_EXPORT int pkv_attention_decode_flat_supports(int hd, int page_size, int q_row_stride) {
  return ((hd == 64 || hd == 128) && page_size >= 8 && page_size % 8 == 0 && DT_BN % page_size == 0 &&
          q_row_stride % 2 == 0) ? 1 : 0;
}

// Blocks of this kernel that one SM holds (the host launches that many per SM, at most).
PKV_EXPORT int pkv_attention_decode_flat_blocks_per_sm(int hd) {
  if (hd == 128) return flat_blocks_per_sm<128>();
  if (hd == 64) return flat_blocks_per_sm<64>();
  return 0;
}

// Floats of workspace that `blocks` blocks need.
PKV_EXPORT long long pkv_attention_decode_flat_workspace_floats(int hd, int blocks) {
  return 2LL * blocks * DT_ROWS * (hd + 2);
}

PKV_EXPORT int pkv_attention_decode_flat(const void* qkv, int q_row_stride, void* out, const void* k_pool,
                                         const void* v_pool, long long n_pages, const int32_t* block_table,
                                         int table_stride, const int32_t* seq_starts, const int32_t* first_pos,
                                         const int32_t* work_seq, const int32_t* unit_starts, int n_work,
                                         int max_entry_tokens, int n_heads, int n_kv, int hd, int page_size, int window,
                                         float scale, int blocks, void* workspace, long long workspace_floats,
                                         int* counters, long long counters_len, int* status, void* stream) {
  if (n_work <= 0) return 0;
  if (!pkv_attention_decode_flat_supports(hd, page_size, q_row_stride)) return PKV_ERR_LIMIT;
  if (n_heads <= 0 || n_kv <= 0 || n_heads % n_kv || window < 0) return PKV_ERR_SIZE;
  if (blocks < 1 || n_work > (1 << 20)) return PKV_ERR_LIMIT;
  if (max_entry_tokens * (n_heads / n_kv) > DT_ROWS) return PKV_ERR_LIMIT;
  if (workspace_floats < pkv_attention_decode_flat_workspace_floats(hd, blocks) || counters_len < (long long)n_work * n_kv)
    return PKV_ERR_SIZE;
  const long long pool_rows = n_pages * n_kv * page_size;
  if (pool_rows >= (1LL << 31) - page_size) return PKV_ERR_LIMIT;
  if ((uintptr_t)qkv % 4 || (uintptr_t)k_pool % 16 || (uintptr_t)v_pool % 16 || (uintptr_t)workspace % 16) return PKV_ERR_ALIGN;
  alignas(64) CUtensorMap map_k, map_v;
  if (!decode_pool_map(k_pool, pool_rows, hd, page_size, &map_k) || !decode_pool_map(v_pool, pool_rows, hd, page_size, &map_v))
    return PKV_ERR_SIZE;
  int shift = -1;
  for (int i = 0; i < 31; ++i)
    if ((1 << i) == page_size) shift = i;
  DecFlatParams p{(const bf16*)qkv, q_row_stride, (bf16*)out, block_table, table_stride, seq_starts, first_pos, work_seq,
                  unit_starts, n_work, n_heads, n_kv, page_size, shift, window, scale * 1.4426950408889634f,
                  (int)pool_rows, (float*)workspace, counters, status};
  cudaStream_t s = (cudaStream_t)stream;
  return hd == 128 ? launch_flat<128>(map_k, map_v, p, blocks, s) : launch_flat<64>(map_k, map_v, p, blocks, s);
}
