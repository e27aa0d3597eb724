// Matrix product on the fifth-generation tensor cores of sm_100a, written by hand:
//   D[M, N] = A[M, K] . B[N, K]^T      A, B bfloat16 with K contiguous, accumulation in float32
// Operand tiles are brought into shared memory by TMA (cp.async.bulk.tensor, 128-byte swizzle),
// multiplied by tcgen05.mma issued by one thread, accumulated in tensor memory (TMEM) and read
// back with tcgen05.ld for the epilogue, which is fused with what follows the product in the
// decoder:
//   EPI_BF16      store D as bfloat16                         (QKV, output and down projections)
//   EPI_F32       store D as float32                          (logits of the LM head)
//   EPI_SILU_MUL  B holds gate and up rows interleaved in blocks of 128; the epilogue stores
//                 silu(gate) * up as bfloat16, half as wide   (the SwiGLU feed-forward,
//                 reference formula: src/paged_kv_serving/engine/model.py:49-51, 256-259)
//
// One block per SM walks over 128 x 256 tiles of D with six warps: warp 0 issues the TMA loads
// into a ring of stages, warp 1 allocates TMEM and issues the MMAs (four of K = 16 per 64-wide K
// block), warps 2-5 run the epilogue, each on the 32 TMEM lanes it may address. Two accumulators
// alternate in TMEM, so the epilogue of a tile runs under the MMAs of the next one.
// Ring slots are handed over with mbarriers: TMA completes "full" with its byte count, the MMA
// thread releases "empty" and "accumulator ready" with tcgen05.commit, the epilogue warps hand an
// accumulator back with plain arrivals. No load is multicast; every block fetches its own tiles.
//
// Every wait on an mbarrier is bounded: after about a second without progress a block records
// an error code in the status word, lets its copies in flight land (again bounded), frees its
// TMEM and returns, so a fault in the hand-over can never hang the GPU.
#include "tcgen05.cuh"

namespace pkv {

constexpr int GM_BM = 128;
constexpr int GM_BK = 64;                    // 64 bf16 = 128 bytes = one swizzle row
constexpr int GM_THREADS = 192;
constexpr int GM_UMMA_K = 16;

enum { EPI_BF16 = 0, EPI_F32 = 1, EPI_SILU_MUL = 2 };
enum { GEMM_ERR_TIMEOUT = 2 };

__device__ __forceinline__ float silu_clipped(float x, float clip) {
  const float c = fminf(fmaxf(x, -clip), clip);
  return x * (1.0f / (1.0f + expf(-c)));
}

// Epilogue of one 32-column chunk pair: converts and stores what one thread holds of its row.
template <int EPI>
__device__ __forceinline__ void store_chunk(void* out, int ldo, int row, int col0, int n_valid, const float (&v)[32]) {
  if (EPI == EPI_F32) {
    float* dst = reinterpret_cast<float*>(out) + (size_t)row * ldo + col0;
    if (col0 + 32 <= n_valid) {
#pragma unroll
      for (int i = 0; i < 32; i += 4) *reinterpret_cast<float4*>(dst + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
    } else {
      for (int i = 0; i < 32; ++i)
        if (col0 + i < n_valid) dst[i] = v[i];
    }
  } else {
    bf16* dst = reinterpret_cast<bf16*>(out) + (size_t)row * ldo + col0;
    if (col0 + 32 <= n_valid) {
#pragma unroll
      for (int i = 0; i < 32; i += 8) {
        uint4 packed;
        uint32_t* w = reinterpret_cast<uint32_t*>(&packed);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          __nv_bfloat162 pair = __floats2bfloat162_rn(v[i + 2 * j], v[i + 2 * j + 1]);
          w[j] = *reinterpret_cast<uint32_t*>(&pair);
        }
        *reinterpret_cast<uint4*>(dst + i) = packed;
      }
    } else {
      for (int i = 0; i < 32; ++i)
        if (col0 + i < n_valid) dst[i] = __float2bfloat16_rn(v[i]);
    }
  }
}


// Where tile number `tile` of the walk lies. The row blocks of A are taken in groups of
// `group_m`: within a group row blocks run fastest and every column block of B is visited before
// the next group begins. The blocks in flight then share a few tiles of B (the weights), the
// group's rows of A stay in L2 while B streams past them once per group, and A never has to fit
// L2 as a whole (with all of A as one group, 8,192 rows of width 5,120 are read from memory again
// for every column block, and the product is bound by that).
__device__ __forceinline__ void tile_origin(int tile, int m_tiles, int n_tiles, int group_m, int& m_index, int& n_index) {
  const int per_group = group_m * n_tiles;
  const int group = tile / per_group, within = tile - group * per_group;
  const int first = group * group_m;
  const int rows_here = min(group_m, m_tiles - first);
  n_index = within / rows_here;
  m_index = first + (within - n_index * rows_here);
}

// Persistent: each block walks over output tiles in the order of tile_origin. Two accumulators in
// TMEM alternate, so the epilogue of one tile runs under the MMAs of the next.
template <int BN, int STAGES, int EPI>
__global__ void __launch_bounds__(GM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    void* __restrict__ out, int ldo, int M, int n_valid, int K, int m_tiles, int n_tiles, int group_m,
                    float clip, int* __restrict__ status) {
  constexpr uint32_t A_BYTES = GM_BM * GM_BK * 2;
  constexpr uint32_t B_BYTES = BN * GM_BK * 2;
  constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr uint32_t TMEM_COLS = 2 * BN;           // two accumulators of BN columns (a power of two)
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t full_bar[STAGES], empty_bar[STAGES], acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k_blocks = (K + GM_BK - 1) / GM_BK;
  const int total_tiles = m_tiles * n_tiles;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(&full_bar[i], 1);
      mbar_init(&empty_bar[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&acc_full[i], 1);
      mbar_init(&acc_empty[i], 4);                 // one arrival per epilogue warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(&tmem_slot, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  volatile int* aborted = &abort_flag;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        int m_index, n_index;
        tile_origin(tile, m_tiles, n_tiles, group_m, m_index, n_index);
        const int m0 = m_index * GM_BM, n0 = n_index * BN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int stage = it % STAGES;
          if (it >= STAGES && !mbar_wait(&empty_bar[stage], ((it / STAGES) - 1) & 1, aborted)) { ok = false; break; }
          uint8_t* a_dst = tiles + (size_t)stage * STAGE_BYTES;
          mbar_expect_tx(&full_bar[stage], STAGE_BYTES);
          tma_load_2d(a_dst, &map_a, &full_bar[stage], kb * GM_BK, m0);
          tma_load_2d(a_dst + A_BYTES, &map_b, &full_bar[stage], kb * GM_BK, n0);
        }
      }
      if (*aborted) {
        // let the copies already issued land before the block's shared memory is given up
        for (int j = max(0, it - STAGES); j < it; ++j) {
          const long long start = clock64();
          while (!mbar_try_wait(&full_bar[j % STAGES], (j / STAGES) & 1) && clock64() - start < GM_WAIT_CYCLES) {}
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      // instruction descriptor: float32 accumulator, bfloat16 A and B, both K-major, M = 128, N = BN
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(GM_BM >> 4) << 24);
      int it = 0, local = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++local) {
        const int buf = local & 1;
        if (local >= 2) ok = mbar_wait(&acc_empty[buf], ((local >> 1) - 1) & 1, aborted);   // epilogue drained it
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int stage = it % STAGES;
          ok = mbar_wait(&full_bar[stage], (it / STAGES) & 1, aborted);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_addr = smem_addr(tiles + (size_t)stage * STAGE_BYTES);
          const uint64_t a_desc = umma_desc(a_addr), b_desc = umma_desc(a_addr + A_BYTES);
#pragma unroll
          for (int k = 0; k < GM_BK / GM_UMMA_K; ++k) {
            // advancing 16 elements along K inside the swizzled row: 32 bytes = 2 units of 16 bytes
            umma_bf16(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);          // the slot is free once these MMAs have read it
        }
        if (ok) umma_commit(&acc_full[buf]);       // the accumulator is complete once all MMAs are done
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int quarter = warp & 3;                  // the TMEM lanes this warp may address: 32 * (warp % 4)
    int local = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++local) {
      const int buf = local & 1;
      int m_index, n_index;
      tile_origin(tile, m_tiles, n_tiles, group_m, m_index, n_index);
      const int m0 = m_index * GM_BM, n0 = n_index * BN;
      const int row = m0 + quarter * 32 + lane;
      // every lane waits; the warp goes on only as a whole (tcgen05.ld needs all 32 lanes)
      const bool ready = __all_sync(0xffffffffu, mbar_wait(&acc_full[buf], (local >> 1) & 1, aborted) ? 1 : 0) != 0;
      if (!ready) break;
      tc_fence_after();
      const uint32_t lane_addr = tmem_base + buf * BN + ((uint32_t)(quarter * 32) << 16);
      if (EPI == EPI_SILU_MUL) {
        // columns [0, BN/2) of the tile are gate values, [BN/2, BN) the matching up values
#pragma unroll 1
        for (int c = 0; c < BN / 2; c += 32) {
          float g[32], u[32];
          tmem_load32(lane_addr + c, g);
          tmem_load32(lane_addr + BN / 2 + c, u);
#pragma unroll
          for (int i = 0; i < 32; ++i) g[i] = silu_clipped(g[i], clip) * u[i];
          if (row < M) store_chunk<EPI_BF16>(out, ldo, row, (n0 >> 1) + c, n_valid, g);
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
          float v[32];
          tmem_load32(lane_addr + c, v);
          if (row < M) store_chunk<EPI>(out, ldo, row, n0 + c, n_valid, v);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);   // this warp has read its part of the accumulator
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
  if (threadIdx.x == 0 && abort_flag) atomicExch(status, GEMM_ERR_TIMEOUT);
}

// The same product with pairs of blocks (a cluster of two SMs, tcgen05 cta_group::2): the pair
// computes a 256 x 256 tile, each block holding its 128 rows of A and its 128 of the 256 rows of
// B, so every block moves a third less through its shared memory and the ring is six stages deep.
// Block 0 of the pair issues the MMAs for both (M = 256); the bytes of both blocks' TMA loads are
// counted on block 0's "full" barriers, its commits reach the "empty" and "accumulator ready"
// barriers of both blocks, and the epilogue warps of both hand accumulators back to block 0.
//
// Whole tiles are dealt round-robin while they fill complete waves (so that the pairs in flight
// share a few tiles of B in L2); the tiles of the last, partly filled wave are dealt out stream-K
// fashion instead: their (tile, K block) iterations are cut into equal contiguous shares, one per
// pair, so no SM idles. A share may begin or end inside a tile. The pair whose share holds the first K block of
// a tile owns the tile: if its share ends inside the tile, it adds the partial accumulators that
// the following pairs left in a workspace (in a fixed order, so the result does not depend on
// timing) and runs the epilogue. A pair whose share begins inside a tile computes that part
// first, writes its partial accumulator to the workspace and raises a flag, which the owner
// lowers again; so an owner, at the end of its share, waits only for work done at the start of
// other shares and the pairs never queue up behind one another.
constexpr int PAIR_BN = 256;
constexpr size_t PAIR_SLOT_FLOATS = (size_t)GM_BM * PAIR_BN;       // one block's partial accumulator (one slot per block)

__device__ __forceinline__ int ld_acquire(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// The work of one pair, in order: first its share of the stream-K region (the last `sk_units`
// tiles of the product, cut into equal runs of K blocks), then whole tiles dealt round-robin
// (tile = wave * pairs + pair), so that the pairs in flight share a few tiles of B in L2.
struct PairWork {
  int k_blocks, n_pairs, pair, dp_waves, sk_first_unit;
  long long sk_total;            // K-block iterations in the stream-K region
  long long at, share_end;       // position inside this pair's stream-K share
  int wave;
  __device__ PairWork(int total_units, int k_blocks_, int n_pairs_, int pair_)
      : k_blocks(k_blocks_), n_pairs(n_pairs_), pair(pair_) {
    dp_waves = total_units / n_pairs;
    sk_first_unit = dp_waves * n_pairs;
    sk_total = (long long)(total_units - sk_first_unit) * k_blocks;
    at = sk_total * pair / n_pairs;
    share_end = sk_total * (pair + 1) / n_pairs;
    wave = 0;
  }
  __device__ long long share_begin_of(int q) const { return sk_total * q / n_pairs; }
  // next run of K blocks of one tile; false when the pair is done
  __device__ bool next(int& unit, int& kb0, int& kb1, bool& stream_k, long long& position) {
    if (at < share_end) {
      const int local = (int)(at / k_blocks);
      unit = sk_first_unit + local;
      kb0 = (int)(at - (long long)local * k_blocks);
      kb1 = (int)min((long long)k_blocks, kb0 + (share_end - at));
      stream_k = true;
      position = at;
      at += kb1 - kb0;
      return true;
    }
    if (wave < dp_waves) {
      unit = wave * n_pairs + pair;
      kb0 = 0;
      kb1 = k_blocks;
      stream_k = false;
      position = 0;
      ++wave;
      return true;
    }
    return false;
  }
};

template <int STAGES, int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GM_THREADS, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                         void* __restrict__ out, int ldo, int M, int n_valid, int K, int m_pairs, int n_tiles, float clip,
                         float* __restrict__ workspace, int* __restrict__ flags, int* __restrict__ status) {
  constexpr int BN = PAIR_BN;
  constexpr uint32_t A_BYTES = GM_BM * GM_BK * 2;          // this block's 128 rows of A
  constexpr uint32_t B_BYTES = (BN / 2) * GM_BK * 2;       // this block's half of the B tile
  constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr uint32_t TMEM_COLS = 2 * BN;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t full_bar[STAGES], empty_bar[STAGES], acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();                    // 0: issues the MMAs of the pair
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int k_blocks = (K + GM_BK - 1) / GM_BK;
  const int total_units = m_pairs * n_tiles;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(&full_bar[i], 1);
      mbar_init(&empty_bar[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&acc_full[i], 1);
      mbar_init(&acc_empty[i], 8);                 // four epilogue warps in each block of the pair
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc_pair(&tmem_slot, TMEM_COLS);
  tc_fence_before();
  cluster_sync_all();                              // barriers and TMEM of both blocks are ready
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  volatile int* aborted = &abort_flag;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both blocks)
    if (lane == 0) {
      int it = 0;
      bool ok = true, stream_k;
      int unit, kb0, kb1;
      long long position;
      PairWork work(total_units, k_blocks, n_pairs, pair);
      while (ok && work.next(unit, kb0, kb1, stream_k, position)) {
        const int m0 = (unit % m_pairs) * 2 * GM_BM + (int)rank * GM_BM;
        const int n0 = (unit / m_pairs) * BN + (int)rank * (BN / 2);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int stage = it % STAGES;
          if (it >= STAGES && !mbar_wait(&empty_bar[stage], ((it / STAGES) - 1) & 1, aborted)) { ok = false; break; }
          uint8_t* a_dst = tiles + (size_t)stage * STAGE_BYTES;
          if (rank == 0) mbar_expect_tx(&full_bar[stage], 2 * STAGE_BYTES);     // the bytes of both blocks
          tma_load_2d_pair(a_dst, &map_a, &full_bar[stage], kb * GM_BK, m0);
          tma_load_2d_pair(a_dst + A_BYTES, &map_b, &full_bar[stage], kb * GM_BK, n0);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (block 0 only)
    if (lane == 0 && rank == 0) {
      // float32 accumulator, bfloat16 A and B, both K-major, M = 256 over the pair, N = 256
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)((2 * GM_BM) >> 4) << 24);
      int it = 0, local = 0;
      bool ok = true, stream_k;
      int unit, kb0, kb1;
      long long position;
      PairWork work(total_units, k_blocks, n_pairs, pair);
      for (; ok && work.next(unit, kb0, kb1, stream_k, position); ++local) {
        const int buf = local & 1;
        if (local >= 2) ok = mbar_wait(&acc_empty[buf], ((local >> 1) - 1) & 1, aborted);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int stage = it % STAGES;
          ok = mbar_wait(&full_bar[stage], (it / STAGES) & 1, aborted);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_addr = smem_addr(tiles + (size_t)stage * STAGE_BYTES);
          const uint64_t a_desc = umma_desc(a_addr), b_desc = umma_desc(a_addr + A_BYTES);
#pragma unroll
          for (int k = 0; k < GM_BK / GM_UMMA_K; ++k)
            umma_bf16_pair(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          umma_commit_pair(&empty_bar[stage]);     // frees the slot in both blocks
        }
        if (ok) umma_commit_pair(&acc_full[buf]);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (both blocks)
    const int quarter = warp & 3;
    const int row_in_block = quarter * 32 + lane;
    int local = 0;
    bool ok = true, stream_k;
    int unit, kb0, kb1;
    long long position;
    PairWork work(total_units, k_blocks, n_pairs, pair);
    for (; ok && work.next(unit, kb0, kb1, stream_k, position); ++local) {
      const bool starts_tile = kb0 == 0, ends_tile = kb1 == k_blocks;
      const int buf = local & 1;
      const int m0 = (unit % m_pairs) * 2 * GM_BM + (int)rank * GM_BM, n0 = (unit / m_pairs) * BN;
      const int row = m0 + row_in_block;
      ok = __all_sync(0xffffffffu, mbar_wait(&acc_full[buf], (local >> 1) & 1, aborted) ? 1 : 0) != 0;
      if (!ok) break;
      tc_fence_after();
      const uint32_t lane_addr = tmem_base + buf * BN + ((uint32_t)(quarter * 32) << 16);
      if (!starts_tile) {
        // The share begins inside this tile (its first K blocks belong to the pair before): leave
        // the partial accumulator for that pair. This happens at the start of a share, so the
        // pair that waits for it (at the end of its own share) finds it long done.
        // slot layout [4-column group][row][4]: the 32 lanes of a warp (32 rows) write 512 contiguous bytes
        float4* dst = reinterpret_cast<float4*>(workspace + (size_t)blockIdx.x * PAIR_SLOT_FLOATS) + row_in_block;
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
          float v[32];
          tmem_load32(lane_addr + c, v);
#pragma unroll
          for (int i = 0; i < 32; i += 4) dst[(size_t)((c + i) >> 2) * GM_BM] = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
        }
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");          // all four epilogue warps have written
        if (threadIdx.x == 64) atomicExch(&flags[blockIdx.x], 1);
      } else {
        // This pair began the tile and owns its result. If its share ends inside the tile, the
        // pairs after it computed the remaining K blocks at the start of their shares.
        int helpers = 0;     // pairs (pair, pair + helpers] hold the rest of the tile (some shares may be empty)
        if (!ends_tile) {
          const long long tile_end = (long long)(unit - work.sk_first_unit + 1) * k_blocks;   // in stream-K positions
          while (pair + helpers + 1 < n_pairs && work.share_begin_of(pair + helpers + 1) < tile_end) ++helpers;
          if (threadIdx.x == 64) {
            const long long start = clock64();
            for (int q = pair + 1; q <= pair + helpers && ok; ++q) {
              if (work.share_begin_of(q) == work.share_begin_of(q + 1)) continue;      // an empty share leaves nothing
              const int* flag = &flags[q * 2 + (int)rank];
              while (ld_acquire(flag) == 0) {
                if (*aborted || clock64() - start > GM_WAIT_CYCLES) { *aborted = 1; ok = false; break; }
              }
            }
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
          ok = !*aborted;
          if (!ok) break;
        }
#pragma unroll 1
        for (int c = 0; c < (EPI == EPI_SILU_MUL ? BN / 2 : BN); c += 32) {
          float v[32], u[32];
          tmem_load32(lane_addr + c, v);
          if (EPI == EPI_SILU_MUL) tmem_load32(lane_addr + BN / 2 + c, u);
          for (int q = pair + 1; q <= pair + helpers; ++q) {          // a fixed order: the sum is reproducible
            if (work.share_begin_of(q) == work.share_begin_of(q + 1)) continue;
            const float4* src = reinterpret_cast<const float4*>(workspace + (size_t)(q * 2 + (int)rank) * PAIR_SLOT_FLOATS) + row_in_block;
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
              const float4 a4 = __ldcg(src + (size_t)((c + i) >> 2) * GM_BM);
              v[i] += a4.x; v[i + 1] += a4.y; v[i + 2] += a4.z; v[i + 3] += a4.w;
              if (EPI == EPI_SILU_MUL) {
                const float4 b4 = __ldcg(src + (size_t)((BN / 2 + c + i) >> 2) * GM_BM);
                u[i] += b4.x; u[i + 1] += b4.y; u[i + 2] += b4.z; u[i + 3] += b4.w;
              }
            }
          }
          if (EPI == EPI_SILU_MUL) {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = silu_clipped(v[i], clip) * u[i];
            if (row < M) store_chunk<EPI_BF16>(out, ldo, row, (n0 >> 1) + c, n_valid, v);
          } else {
            if (row < M) store_chunk<EPI>(out, ldo, row, n0 + c, n_valid, v);
          }
        }
        if (helpers) {
          asm volatile("bar.sync 1, 128;" ::: "memory");        // every warp has read the partials
          if (threadIdx.x == 64)
            for (int q = pair + 1; q <= pair + helpers; ++q)
              if (work.share_begin_of(q) != work.share_begin_of(q + 1)) flags[q * 2 + (int)rank] = 0;   // lowered for the next launch
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_remote(&acc_empty[buf], 0);    // to block 0, which issues the MMAs
    }
  }

  tc_fence_before();
  cluster_sync_all();                              // nobody leaves while its peer may still signal it
  if (warp == 1) tmem_dealloc_pair(tmem_base, TMEM_COLS);
  if (threadIdx.x == 0 && abort_flag) atomicExch(status, GEMM_ERR_TIMEOUT);
}

// -----------------------------------------------------------------------------------------------
// host side
// -----------------------------------------------------------------------------------------------
template <int BN, int STAGES, int EPI>
static int launch_gemm(const CUtensorMap& map_a, const CUtensorMap& map_b, void* out, int ldo, int M, int n_tiles_cols,
                       int n_valid, int K, float clip, int* status, cudaStream_t s) {
  const size_t smem = (size_t)STAGES * (GM_BM + BN) * GM_BK * 2 + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, STAGES, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int m_tiles = (M + GM_BM - 1) / GM_BM;
  const long long total = (long long)m_tiles * n_tiles_cols;
  static int sm_count = 0;
  if (!sm_count) {
    int device = 0;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device);
  }
  const int blocks = (int)(total < sm_count ? total : sm_count);
  // as many row blocks of A to a group as hold about 32 MB (a quarter of L2)
  long long group_m = (32LL << 20) / ((long long)GM_BM * K * 2);
  if (group_m < 1) group_m = 1;
  if (group_m > m_tiles) group_m = m_tiles;
  gemm_tcgen05_kernel<BN, STAGES, EPI><<<blocks, GM_THREADS, smem, s>>>(map_a, map_b, out, ldo, M, n_valid, K, m_tiles,
                                                                       n_tiles_cols, (int)group_m, clip, status);
  return launch_status();
}

// Blocks of the pair kernel on this device; its workspace holds one partial-accumulator slot and
// one flag per block.
static int pair_blocks() {
  static int blocks = 0;
  if (!blocks) {
    int device = 0, sms = 0;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    blocks = sms / 2 * 2;
  }
  return blocks;
}

template <int STAGES, int EPI>
static int launch_gemm_pair(const CUtensorMap& map_a, const CUtensorMap& map_b, void* out, int ldo, int M, int n_tiles_cols,
                            int n_valid, int K, float clip, void* workspace, long long workspace_bytes, int* status,
                            cudaStream_t s) {
  const size_t smem = (size_t)STAGES * (GM_BM + 128) * GM_BK * 2 + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_pair_kernel<STAGES, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int m_pairs = (M + 2 * GM_BM - 1) / (2 * GM_BM);
  const int k_blocks = (K + GM_BK - 1) / GM_BK;
  const long long iters = (long long)m_pairs * n_tiles_cols * k_blocks;
  int blocks = pair_blocks();
  if (iters < blocks / 2) blocks = (int)iters * 2;            // never more pairs than iterations
  const size_t flag_bytes = (((size_t)pair_blocks() * sizeof(int)) + 255) / 256 * 256;
  const size_t need = flag_bytes + (size_t)pair_blocks() * PAIR_SLOT_FLOATS * sizeof(float);
  if (!workspace || (size_t)workspace_bytes < need || (uintptr_t)workspace % 16) return PKV_ERR_SIZE;
  int* flags = reinterpret_cast<int*>(workspace);
  float* slots = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(workspace) + flag_bytes);
  gemm_tcgen05_pair_kernel<STAGES, EPI><<<blocks, GM_THREADS, smem, s>>>(map_a, map_b, out, ldo, M, n_valid, K, m_pairs,
                                                                        n_tiles_cols, clip, slots, flags, status);
  return launch_status();
}

}  // namespace pkv

using namespace pkv;

// 1 when this kernel takes the operands (alignment and size rules of TMA), else 0.
PKV_EXPORT int pkv_gemm_tcgen05_supports(long long a_ptr, long long b_ptr, int lda, int ldb, int K) {
  return (a_ptr % 16 == 0 && b_ptr % 16 == 0 && lda % 8 == 0 && ldb % 8 == 0 && K >= 8 && K % 8 == 0) ? 1 : 0;
}

// D = A . B^T with A [M, K] (lda), B [N, K] (ldb), both bfloat16.
//   epilogue 0: out bfloat16 [M, N]; 1: out float32 [M, N];
//   2: B rows interleaved (128 gate rows, 128 up rows, ...), out bfloat16 [M, n_out] = silu(gate) * up.
// `status` is a device int that receives an error code if a block had to give up a wait.
// Bytes of zero-initialised workspace the two-SM kernel wants (partial accumulators and flags
// of its stream-K hand-over). The flags must be zero before the first launch; every launch
// leaves them zero again.
PKV_EXPORT long long pkv_gemm_tcgen05_workspace_bytes() {
  const size_t flag_bytes = (((size_t)pair_blocks() * sizeof(int)) + 255) / 256 * 256;
  return (long long)(flag_bytes + (size_t)pair_blocks() * PAIR_SLOT_FLOATS * sizeof(float));
}

PKV_EXPORT int pkv_gemm_tcgen05(const void* a, int lda, const void* b, int ldb, void* out, int ldo, int M, int N,
                                int K, int epilogue, int n_out, float clip, void* workspace, long long workspace_bytes,
                                int* status, void* stream) {
  if (M <= 0 || N <= 0) return 0;
  if (!pkv_gemm_tcgen05_supports((long long)(uintptr_t)a, (long long)(uintptr_t)b, lda, ldb, K)) return PKV_ERR_ALIGN;
  if (lda < K || ldb < K) return PKV_ERR_SIZE;
  cudaStream_t s = (cudaStream_t)stream;
  alignas(64) CUtensorMap map_a, map_b;
  int r = make_tile_map(&map_a, a, M, K, lda, GM_BM);
  if (r) return r;
  // pairs of blocks (two SMs per tile) pay off once there is more than one 128-row block of A
  const bool use_pairs = workspace != nullptr && M > GM_BM;
  if (epilogue == EPI_SILU_MUL) {
    if (N % 256 || n_out <= 0 || n_out > N / 2 || ldo % 8 || (uintptr_t)out % 16) return PKV_ERR_SIZE;
    r = make_tile_map(&map_b, b, N, K, ldb, use_pairs ? 128 : 256);
    if (r) return r;
    if (use_pairs) return launch_gemm_pair<6, EPI_SILU_MUL>(map_a, map_b, out, ldo, M, N / 256, n_out, K, clip, workspace, workspace_bytes, status, s);
    return launch_gemm<256, 4, EPI_SILU_MUL>(map_a, map_b, out, ldo, M, N / 256, n_out, K, clip, status, s);
  }
  if (epilogue == EPI_BF16) {
    if (ldo % 8 || (uintptr_t)out % 16) return PKV_ERR_ALIGN;
    r = make_tile_map(&map_b, b, N, K, ldb, use_pairs ? 128 : 256);
    if (r) return r;
    if (use_pairs) return launch_gemm_pair<6, EPI_BF16>(map_a, map_b, out, ldo, M, (N + 255) / 256, N, K, clip, workspace, workspace_bytes, status, s);
    return launch_gemm<256, 4, EPI_BF16>(map_a, map_b, out, ldo, M, (N + 255) / 256, N, K, clip, status, s);
  }
  if (epilogue == EPI_F32) {
    if (ldo % 4 || (uintptr_t)out % 16) return PKV_ERR_ALIGN;
    r = make_tile_map(&map_b, b, N, K, ldb, use_pairs ? 128 : 256);
    if (r) return r;
    if (use_pairs) return launch_gemm_pair<6, EPI_F32>(map_a, map_b, out, ldo, M, (N + 255) / 256, N, K, clip, workspace, workspace_bytes, status, s);
    return launch_gemm<256, 4, EPI_F32>(map_a, map_b, out, ldo, M, (N + 255) / 256, N, K, clip, status, s);
  }
  return PKV_ERR_DTYPE;
}
