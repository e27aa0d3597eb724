// Paged causal attention for runs of queries (prefill) on the fifth-generation tensor cores.
//
// What it computes restates the reference (rouviere-german/paged-kv-serving):
//   src/paged_kv_serving/engine/attention.py:83-121  scores = q.k * scale, keys after the query's
//   absolute position masked, online softmax folded tile by tile, output acc / sum;
//   src/paged_kv_serving/engine/runner.py:198-212    every entry attends over its own block table.
// Grouped-query heads and an optional window generalise it. attention_bf16.cu (mma.sync) and
// attention_generic.cu (float32) take the sizes this kernel refuses: it wants bfloat16, a head
// size of 64 or 128 and a page size that is a multiple of 8.
//
// One block handles 128 queries of one sequence for one head and walks the keys in tiles of KT
// absolute positions (aligned to multiples of KT from position 0), with six warps. With KT = 64
// (pages of up to 64 keys) a block needs half of an SM's shared memory, registers and tensor
// memory, and two blocks share an SM: one block's softmax runs while the other's products do.
// With KT = 128 (pages of 128 keys) one block fills the SM.
//   warp 0     TMA: the query tile from the fused qkv buffer, then for every key tile the pages
//              the block table names, page by page, into 128-byte-swizzled shared memory (a page
//              that was given back, or that lies past the last key, is fetched from outside the
//              pool and arrives as zeros)
//   warp 1     tcgen05.mma: S = Q.K^T into one of two score buffers in tensor memory, and
//              O += P.V into the output accumulator (V is read in place, as an N-major operand)
//   warps 2-5  softmax, one query row per thread: scores from TMEM, mask by position, running
//              maximum and sum in float32 (log2 domain), probabilities to shared memory as the
//              bfloat16 A operand of the second product; the accumulator in TMEM is rescaled only
//              when a row's maximum grew by more than 2^8 since its last rescale; finally O / sum
// Scores of tile j+1 are computed while the softmax of tile j runs. All hand-overs go through
// mbarriers whose waits are bounded (status code 2 on a give-up, TMEM freed, no hang).
#include "tcgen05.cuh"

namespace pkv {

constexpr int FA_BM = 128;        // queries per block
constexpr int FA_THREADS = 192;
constexpr int FA_TABLE_CACHE = 1024;
constexpr float FA_RESCALE_STEP = 8.0f;   // log2: rescale the accumulator when the maximum grew by 2^8

struct FaParams {
  bf16* out;                     // [T, H * HD]
  const int32_t* block_table;    // [S, table_stride]
  int table_stride;
  const int32_t* seq_starts;
  const int32_t* first_pos;
  const int32_t* work_seq;       // entry of each work item
  const int32_t* work_q0;        // first query (inside the entry) of each work item
  int n_heads, n_kv, page_size, page_shift, window;
  float scale_log2;
  int pool_rows;                 // rows of the key/value maps; a row coordinate >= this reads zeros
  int* status;
};

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// WIDE: a page of keys or values arrives as ONE copy that covers every 64-column panel (the pool
// seen through make_panel_group_map), and a tile lies in shared memory as groups of 8 keys, each
// group panel after panel; otherwise one copy per page and panel, and a tile lies panel after
// panel. With pages of 16 keys the number of copies per tile is what holds this kernel back, and
// the wide form halves it for head size 128.
template <int HD, int KT, bool WIDE>
__global__ void __launch_bounds__(FA_THREADS, KT == 64 ? 2 : 1)
attention_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                         const __grid_constant__ CUtensorMap map_v, const FaParams p) {
  constexpr int FA_BN = KT;                               // keys per tile
  constexpr int PANELS = HD / 64;                         // 64-column panels of a row of Q, K or V
  constexpr uint32_t GROUP_BYTES = PANELS * 1024;         // WIDE: 8 keys, every panel
  constexpr uint32_t PANEL_BYTES = 128 * 128;             // a panel of Q or P: 128 rows of 128 bytes
  constexpr uint32_t Q_BYTES = PANELS * PANEL_BYTES;      // the query tile
  constexpr uint32_t KV_PANEL_BYTES = KT * 128;           // a panel of K or V: KT rows of 128 bytes
  constexpr uint32_t TILE_BYTES = PANELS * KV_PANEL_BYTES;   // a K or V tile
  constexpr int VSTAGES = KT == 64 ? 1 : 2;               // value tiles in flight (one, where two blocks share an SM)
  constexpr uint32_t TMEM_COLS = KT == 64 ? 256 : 512;    // two score buffers of KT columns, then the accumulator
  constexpr uint32_t S_COL = 0, O_COL = 2 * KT;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* q_s = base;
  uint8_t* k_s = q_s + Q_BYTES;                  // [2][TILE_BYTES]
  uint8_t* v_s = k_s + 2 * TILE_BYTES;           // [VSTAGES][TILE_BYTES]
  uint8_t* p_s = v_s + VSTAGES * TILE_BYTES;     // probabilities: 128 rows x KT keys, panels of 64 keys
  __shared__ __align__(8) uint64_t q_full, k_full[2], v_full[2], k_empty[2], v_empty[2], s_full[2], s_empty[2], p_full, pv_done;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  __shared__ int32_t table_cache[FA_TABLE_CACHE];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int item = blockIdx.x / p.n_heads, head = blockIdx.x - item * p.n_heads;
  const int kvh = head / (p.n_heads / p.n_kv);
  const int s = p.work_seq[item], q0 = p.work_q0[item];
  const int tok0 = p.seq_starts[s];
  const int n_q = p.seq_starts[s + 1] - tok0;
  const int pos0 = p.first_pos[s];
  const int rows_valid = min(FA_BM, n_q - q0);
  const int qpos_first = pos0 + q0;
  const int key_hi = qpos_first + rows_valid;                                     // exclusive
  const int key_lo = p.window > 0 ? max(0, qpos_first - p.window + 1) : 0;
  const int tile_begin = key_lo / FA_BN, tile_end = (key_hi - 1) / FA_BN;         // inclusive
  const int n_tiles = tile_end - tile_begin + 1;
  const int32_t* table = p.block_table + (size_t)s * p.table_stride;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(&q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1); mbar_init(&v_full[i], 1);
      mbar_init(&k_empty[i], 1); mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1); mbar_init(&s_empty[i], 4);
    }
    mbar_init(&p_full, 4);
    mbar_init(&pv_done, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // the block-table entries of this block's key range, read once
  const int entry_first = p.page_shift >= 0 ? (tile_begin * FA_BN) >> p.page_shift : (tile_begin * FA_BN) / p.page_size;
  const int entry_last = p.page_shift >= 0 ? (key_hi - 1) >> p.page_shift : (key_hi - 1) / p.page_size;
  const bool table_cached = entry_last - entry_first + 1 <= FA_TABLE_CACHE;
  if (table_cached)
    for (int i = threadIdx.x; i <= entry_last - entry_first; i += FA_THREADS) table_cache[i] = table[entry_first + i];
  if (warp == 1) tmem_alloc(&tmem_slot, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  volatile int* aborted = &abort_flag;

  if (warp == 0) {
    // ------------------------------------------------------------------------ TMA producer
    // Lane 0 waits for a free slot and announces the bytes; then every lane issues one box
    // (one page of one 64-column panel), so the many small copies of a tile start together.
    if (lane == 0) {
      mbar_expect_tx(&q_full, Q_BYTES);
      for (int pn = 0; pn < PANELS; ++pn)
        tma_load_2d(q_s + pn * PANEL_BYTES, &map_q, &q_full, head * HD + 64 * pn, tok0 + q0);
    }
    const int pages_per_tile = FA_BN / p.page_size;
    const int boxes = WIDE ? pages_per_tile : pages_per_tile * PANELS;
    bool ok = true;
    int loaded_k = 0, loaded_v = 0;
    // one tile of keys (which = 0) or values (1): wait for its slot, announce the bytes, one box a lane
    auto load_tile = [&](int which, int j) {
      const int stage = which ? j % VSTAGES : j & 1;
      const int round = which ? j / VSTAGES : j >> 1;
      const int tile_base = (tile_begin + j) * FA_BN;
      uint64_t* empty = which ? &v_empty[stage] : &k_empty[stage];
      uint64_t* full = which ? &v_full[stage] : &k_full[stage];
      if (lane == 0) {
        if (round >= 1 && !mbar_wait(empty, (round - 1) & 1, aborted)) ok = false;
        if (ok) mbar_expect_tx(full, TILE_BYTES);
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) return;
      uint8_t* dst = (which ? v_s : k_s) + stage * TILE_BYTES;
      for (int b = lane; b < boxes; b += 32) {
        const int i = WIDE ? b : b / PANELS, pn = WIDE ? 0 : b - i * PANELS;
        const int pos = tile_base + i * p.page_size;
        int row = p.pool_rows;                               // outside the pool: zeros
        if (pos < key_hi && pos + p.page_size > key_lo) {
          const int e = p.page_shift >= 0 ? pos >> p.page_shift : pos / p.page_size;
          const int page = table_cached ? table_cache[e - entry_first] : table[e];
          row = checked_pool_row(page, p.n_kv, kvh, p.page_size, p.pool_rows, p.status);
        }
        if (WIDE)
          tma_load_4d(dst + (i * p.page_size >> 3) * GROUP_BYTES, which ? &map_v : &map_k, full, 0, 0, 0, row >> 3);
        else
          tma_load_2d(dst + pn * KV_PANEL_BYTES + i * p.page_size * 128, which ? &map_v : &map_k, full, 64 * pn, row);
      }
      __syncwarp();
      if (which) loaded_v = j + 1; else loaded_k = j + 1;
    };
    // the keys of tile j + 1 are asked for before the values of tile j: the next scores are
    // computed while this tile's softmax runs, the values are needed only after it
    load_tile(0, 0);
    for (int j = 0; j < n_tiles && ok; ++j) {
      if (j + 1 < n_tiles) load_tile(0, j + 1);
      if (ok) load_tile(1, j);
    }
    if (lane == 0 && *aborted) {   // let the copies in flight land before the shared memory is given up
      const long long start = clock64();
      while (!mbar_try_wait(&q_full, 0) && clock64() - start < GM_WAIT_CYCLES) {}
      for (int j = max(0, loaded_k - 2); j < loaded_k; ++j)
        while (!mbar_try_wait(&k_full[j & 1], (j >> 1) & 1) && clock64() - start < GM_WAIT_CYCLES) {}
      for (int j = max(0, loaded_v - VSTAGES); j < loaded_v; ++j)
        while (!mbar_try_wait(&v_full[j % VSTAGES], (j / VSTAGES) & 1) && clock64() - start < GM_WAIT_CYCLES) {}
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      // float32 accumulate, bfloat16 operands, M = 128; scores: N = 128, both operands K-major;
      // output: N = HD, A (probabilities) K-major, B (values, [key][dim]) N-major
      const uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(FA_BN >> 3) << 17) | ((uint32_t)(FA_BM >> 4) << 24);
      const uint32_t idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(HD >> 3) << 17) | ((uint32_t)(FA_BM >> 4) << 24);
      auto issue_scores = [&](int j) {
        const int stage = j & 1;
        const uint32_t q_addr = smem_addr(q_s), k_addr = smem_addr(k_s + stage * TILE_BYTES);
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
          const uint64_t k_desc = WIDE ? umma_desc_sbo(k_addr + (ks >> 2) * 1024, GROUP_BYTES)
                                       : umma_desc(k_addr + (ks >> 2) * KV_PANEL_BYTES);
          umma_bf16(tmem_base + S_COL + stage * FA_BN, umma_desc(q_addr + (ks >> 2) * PANEL_BYTES) + 2 * (ks & 3),
                    k_desc + 2 * (ks & 3), idesc_s, ks > 0 ? 1u : 0u);
        }
        umma_commit(&k_empty[stage]);
        umma_commit(&s_full[stage]);
      };
      bool ok = mbar_wait(&q_full, 0, aborted) && mbar_wait(&k_full[0], 0, aborted);
      if (ok) {
        tc_fence_after();
        issue_scores(0);
      }
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (j + 1 < n_tiles) {
          const int next = (j + 1) & 1;
          ok = mbar_wait(&k_full[next], ((j + 1) >> 1) & 1, aborted);
          if (ok && j + 1 >= 2) ok = mbar_wait(&s_empty[next], (((j + 1) >> 1) - 1) & 1, aborted);
          if (!ok) break;
          tc_fence_after();
          issue_scores(j + 1);
        }
        ok = mbar_wait(&p_full, j & 1, aborted) && mbar_wait(&v_full[j % VSTAGES], (j / VSTAGES) & 1, aborted);
        if (!ok) break;
        tc_fence_after();
        const uint32_t p_addr = smem_addr(p_s), v_addr = smem_addr(v_s + (j % VSTAGES) * TILE_BYTES);
#pragma unroll
        for (int ks = 0; ks < FA_BN / 16; ++ks) {
          // 16 keys a step: the next 64 columns of the values KV_PANEL_BYTES (WIDE: 1024) on,
          // the next 8 keys 1024 (WIDE: GROUP_BYTES) on
          const uint64_t v_desc = WIDE ? umma_desc_mn(v_addr + ks * 2 * GROUP_BYTES, 1024, GROUP_BYTES)
                                       : umma_desc_mn(v_addr + ks * 16 * 128, KV_PANEL_BYTES, 1024);
          umma_bf16(tmem_base + O_COL, umma_desc(p_addr + (ks >> 2) * PANEL_BYTES) + 2 * (ks & 3), v_desc, idesc_o,
                    (j > 0 || ks > 0) ? 1u : 0u);
        }
        umma_commit(&v_empty[j % VSTAGES]);
        umma_commit(&pv_done);
      }
    }
  } else {
    // ------------------------------------------------------------------------ softmax and epilogue
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const int qpos = qpos_first + row;
    const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
    float m_ref = -INFINITY, l = 0.0f;
    bool ok = true;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int buf = j & 1;
      const int tile_base = (tile_begin + j) * FA_BN;
      ok = __all_sync(0xffffffffu, mbar_wait(&s_full[buf], (j >> 1) & 1, aborted) ? 1 : 0) != 0;
      if (!ok) break;
      tc_fence_after();
      float sc[FA_BN];
#pragma unroll
      for (int c = 0; c < FA_BN / 32; ++c)
        tmem_load32_nowait(lane_base + S_COL + buf * FA_BN + c * 32, *reinterpret_cast<float(*)[32]>(&sc[c * 32]));
      tmem_load_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_empty[buf]);     // the score buffer may be overwritten

      const bool need_mask = tile_base + FA_BN - 1 > qpos_first || tile_base + FA_BN > key_hi ||
                             (p.window > 0 && tile_base < key_hi - p.window);
      // maximum of the raw scores (the scale is positive, so it can be applied to the maximum)
      float tmax = -INFINITY;
      if (need_mask) {
#pragma unroll
        for (int c = 0; c < FA_BN; ++c) {
          const int kpos = tile_base + c;
          const bool visible = kpos <= qpos && (p.window == 0 || kpos > qpos - p.window);
          sc[c] = visible ? sc[c] : -INFINITY;
          tmax = fmaxf(tmax, sc[c]);
        }
      } else {
        float t0 = -INFINITY, t1 = -INFINITY, t2 = -INFINITY, t3 = -INFINITY;
#pragma unroll
        for (int c = 0; c < FA_BN; c += 4) {
          t0 = fmaxf(t0, sc[c]); t1 = fmaxf(t1, sc[c + 1]); t2 = fmaxf(t2, sc[c + 2]); t3 = fmaxf(t3, sc[c + 3]);
        }
        tmax = fmaxf(fmaxf(t0, t1), fmaxf(t2, t3));
      }
      tmax *= p.scale_log2;
      // the reference maximum moves only when the row's maximum outgrew it by 2^8
      const bool grow = tmax > m_ref + FA_RESCALE_STEP;
      const float m_new = grow ? tmax : m_ref;
      const float alpha = grow ? exp2f(m_ref - m_new) : 1.0f;        // m_ref = -inf gives 0
      const float neg_shift = m_new == -INFINITY ? 0.0f : -m_new;
      float s0 = 0.0f, s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
#pragma unroll
      for (int c = 0; c < FA_BN; c += 4) {
        // p = 2^(score * scale - max): one multiply-add and one ex2 per element; a masked score
        // (-inf) gives exactly 0
        sc[c] = ex2_approx(fmaf(sc[c], p.scale_log2, neg_shift));
        sc[c + 1] = ex2_approx(fmaf(sc[c + 1], p.scale_log2, neg_shift));
        sc[c + 2] = ex2_approx(fmaf(sc[c + 2], p.scale_log2, neg_shift));
        sc[c + 3] = ex2_approx(fmaf(sc[c + 3], p.scale_log2, neg_shift));
        s0 += sc[c]; s1 += sc[c + 1]; s2 += sc[c + 2]; s3 += sc[c + 3];
      }
      const float sum = (s0 + s1) + (s2 + s3);
      l = l * alpha + sum;
      m_ref = m_new;

      if (j > 0) {
        // the previous P.V must be complete: it read the probability buffer and wrote the accumulator
        ok = __all_sync(0xffffffffu, mbar_wait(&pv_done, (j - 1) & 1, aborted) ? 1 : 0) != 0;
        if (!ok) break;
        tc_fence_after();
        if (__any_sync(0xffffffffu, grow ? 1 : 0)) {
#pragma unroll 1
          for (int c = 0; c < HD / 32; ++c) {
            float o[32];
            tmem_load32(lane_base + O_COL + c * 32, o);
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] *= alpha;
            tmem_store32(lane_base + O_COL + c * 32, o);
          }
        }
      }
      // probabilities of this row as the bfloat16 A operand: two panels of 64 keys, rows of 128
      // bytes whose 16-byte chunks are swizzled by the row number
#pragma unroll
      for (int c = 0; c < FA_BN / 8; ++c) {
        uint4 packed;
        uint32_t* w = reinterpret_cast<uint32_t*>(&packed);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          __nv_bfloat162 pair = __floats2bfloat162_rn(sc[c * 8 + 2 * i], sc[c * 8 + 2 * i + 1]);
          w[i] = *reinterpret_cast<uint32_t*>(&pair);
        }
        const int panel = c >> 3, chunk = c & 7;
        *reinterpret_cast<uint4*>(p_s + panel * PANEL_BYTES + row * 128 + ((chunk ^ (row & 7)) << 4)) = packed;
      }
      if (tile_base + FA_BN > key_hi) {
        // slots of the last page past the last key may hold anything (0 x NaN = NaN): clear them
        ok = __all_sync(0xffffffffu, mbar_wait(&v_full[j % VSTAGES], (j / VSTAGES) & 1, aborted) ? 1 : 0) != 0;
        if (!ok) break;
        const int r = key_hi - tile_base + (int)threadIdx.x - 64;     // threads 64..191 take one row each
        if (r < FA_BN)
          for (int pn = 0; pn < PANELS; ++pn) {
            const uint32_t at = WIDE ? (r >> 3) * GROUP_BYTES + pn * 1024 + (r & 7) * 128 : pn * KV_PANEL_BYTES + r * 128;
            uint4* dst = reinterpret_cast<uint4*>(v_s + (j % VSTAGES) * TILE_BYTES + at);
#pragma unroll
            for (int i = 0; i < 8; ++i) dst[i] = make_uint4(0u, 0u, 0u, 0u);
          }
      }
      fence_async_shared();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full);
    }
    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&pv_done, (n_tiles - 1) & 1, aborted) ? 1 : 0) != 0;
    if (ok) {
      tc_fence_after();
      const float inv = l > 0.0f ? 1.0f / l : 0.0f;
      bf16* dst = p.out + (size_t)(tok0 + q0 + row) * ((size_t)p.n_heads * HD) + (size_t)head * HD;
#pragma unroll 1
      for (int c = 0; c < HD / 32; ++c) {
        float o[32];
        tmem_load32(lane_base + O_COL + c * 32, o);
        if (row < rows_valid) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 packed;
            uint32_t* w = reinterpret_cast<uint32_t*>(&packed);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              __nv_bfloat162 pair = __floats2bfloat162_rn(o[i + 2 * k] * inv, o[i + 2 * k + 1] * inv);
              w[k] = *reinterpret_cast<uint32_t*>(&pair);
            }
            *reinterpret_cast<uint4*>(dst + c * 32 + i) = packed;
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
  if (threadIdx.x == 0 && abort_flag) atomicExch(p.status, 2);
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
struct PoolMapKey {
  const void* base;
  long long rows;
  int hd, box, wide;
  CUtensorMap map;
};

// The tensor map of a key or value pool, kept per (pool, sizes, form) and copied to the caller (a
// later lookup may take a table entry's place); false when the driver refuses to encode it.
static bool pool_map(const void* base, long long rows, int hd, int box_rows, int wide, CUtensorMap* out) {
  static PoolMapKey cache[512];
  static int used = 0;
  for (int i = 0; i < used; ++i)
    if (cache[i].base == base && cache[i].rows == rows && cache[i].hd == hd && cache[i].box == box_rows &&
        cache[i].wide == wide) {
      *out = cache[i].map;
      return true;
    }
  static int victim = 0;              // a full table gives up its entries in turn
  PoolMapKey& slot = cache[used < 512 ? used : victim];
  const int rc = wide ? make_panel_group_map(&slot.map, base, rows, hd / 64, box_rows)
                      : make_tile_map(&slot.map, base, rows, hd, hd, box_rows);
  if (rc) {
    slot.base = nullptr;
    return false;
  }
  slot.base = base; slot.rows = rows; slot.hd = hd; slot.box = box_rows; slot.wide = wide;
  if (used < 512) ++used;
  else victim = (victim + 1) % 512;
  *out = slot.map;
  return true;
}

template <int HD, int KT, bool WIDE>
static int launch_fa(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const FaParams& p, int n_work,
                     cudaStream_t s) {
  // the query tile, two key tiles, one or two value tiles, the probabilities, and room to align
  const size_t panels = HD / 64;
  const size_t smem = panels * 128 * 128 + (2 + (KT == 64 ? 1 : 2)) * panels * KT * 128 + (size_t)(KT / 64) * 128 * 128 + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_tcgen05_kernel<HD, KT, WIDE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  attention_tcgen05_kernel<HD, KT, WIDE><<<n_work * p.n_heads, FA_THREADS, smem, s>>>(mq, mk, mv, p);
  return launch_status();
}

}  // namespace pkv

using namespace pkv;

static int g_narrow_boxes = 0;

// 1 when this kernel takes the sizes, 0 when another attention kernel must be used.
PKV_EXPORT int pkv_attention_tcgen05_supports(int hd, int page_size, int q_row_stride) {
  return ((hd == 64 || hd == 128) && page_size >= 8 && page_size % 8 == 0 && 128 % page_size == 0 &&
          q_row_stride % 8 == 0) ? 1 : 0;
}

PKV_EXPORT int pkv_attention_tcgen05_rows() { return FA_BM; }

PKV_EXPORT int pkv_attention_prefill_tcgen05(const void* qkv, int q_row_stride, int n_tokens, void* out,
                                             const void* k_pool, const void* v_pool, long long n_pages,
                                             const int32_t* block_table, int table_stride, const int32_t* seq_starts,
                                             const int32_t* first_pos, const int32_t* work_seq, const int32_t* work_q0,
                                             int n_work, int n_heads, int n_kv, int hd, int page_size, int window,
                                             float scale, int* status, void* stream) {
  if (n_work <= 0) return 0;
  if (!pkv_attention_tcgen05_supports(hd, page_size, q_row_stride)) return PKV_ERR_LIMIT;
  if (n_heads <= 0 || n_kv <= 0 || n_heads % n_kv || window < 0) return PKV_ERR_SIZE;
  const long long pool_rows = n_pages * n_kv * page_size;
  if (pool_rows >= (1LL << 31) - page_size || (long long)n_work * n_heads >= (1LL << 31)) return PKV_ERR_LIMIT;
  if ((uintptr_t)qkv % 16 || (uintptr_t)k_pool % 16 || (uintptr_t)v_pool % 16 || (uintptr_t)out % 16) return PKV_ERR_ALIGN;
  alignas(64) CUtensorMap map_q;
  int r = make_tile_map(&map_q, qkv, n_tokens, q_row_stride, q_row_stride, FA_BM);
  if (r) return r;
  // head size 128: a page in one copy (both 64-column panels) where the driver encodes that map
  int wide = hd == 128 && pool_rows % 8 == 0 && !g_narrow_boxes;
  alignas(64) CUtensorMap map_k, map_v;
  bool mapped = pool_map(k_pool, pool_rows, hd, page_size, wide, &map_k) && pool_map(v_pool, pool_rows, hd, page_size, wide, &map_v);
  if (wide && !mapped) {
    wide = 0;
    mapped = pool_map(k_pool, pool_rows, hd, page_size, 0, &map_k) && pool_map(v_pool, pool_rows, hd, page_size, 0, &map_v);
  }
  if (!mapped) return PKV_ERR_SIZE;
  int shift = -1;
  for (int i = 0; i < 31; ++i)
    if ((1 << i) == page_size) shift = i;
  FaParams p{(bf16*)out, block_table, table_stride, seq_starts, first_pos, work_seq, work_q0, n_heads, n_kv, page_size,
             shift, window, scale * 1.4426950408889634f, (int)pool_rows, status};
  cudaStream_t s = (cudaStream_t)stream;
  // tiles of 64 keys (two blocks to an SM) wherever a page fits one
  if (page_size <= 64) {
    if (hd == 128 && wide) return launch_fa<128, 64, true>(map_q, map_k, map_v, p, n_work, s);
    if (hd == 128) return launch_fa<128, 64, false>(map_q, map_k, map_v, p, n_work, s);
    return launch_fa<64, 64, false>(map_q, map_k, map_v, p, n_work, s);
  }
  if (hd == 128 && wide) return launch_fa<128, 128, true>(map_q, map_k, map_v, p, n_work, s);
  if (hd == 128) return launch_fa<128, 128, false>(map_q, map_k, map_v, p, n_work, s);
  return launch_fa<64, 128, false>(map_q, map_k, map_v, p, n_work, s);
}

// For comparisons and tests: non-zero makes the kernel fetch one copy per page and panel even
// where one copy per page is possible. Returns the previous setting.
PKV_EXPORT int pkv_attention_tcgen05_narrow_boxes(int on) {
  const int before = g_narrow_boxes;
  g_narrow_boxes = on != 0;
  return before;
}
