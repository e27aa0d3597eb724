// Matrix products of decode steps and short portions on the fifth-generation tensor cores:
//   out[M, N] = x[M, K] . w[N, K]^T   for 1 to 128 rows of activations, bfloat16, float32 accumulate.
//
// Such a product reads every weight once and does little arithmetic per byte, so the kernel is
// built around the weight stream, and the weights take the tall side of the MMA:
//
//  * The operands are swapped. A tile of 128 weight rows is the M = 128 operand of tcgen05.mma
//    and the activations its N side (16, 32, 64 or 128 columns, the row count rounded up), so the
//    tensor cores are fully used however few rows a step has. The accumulator [128 weight rows x
//    activation rows] lives in tensor memory; a thread of the epilogue owns one weight row.
//  * Weights arrive by TMA in boxes of 128 (or 256) rows x 64 columns (16 or 32 KB) through a ring
//    of up to eight stages: one copy brings 16 KB, and eight in flight keep an SM's share of the
//    memory bandwidth busy (a ring of such boxes alone streams at the copy rate of the memory).
//    The activations of the same 64 columns ride along in the stage (they come from L2).
//  * One block per SM. The work is (tile of 128 weight rows) x (64-column block of K), laid end to
//    end tile by tile and cut into one even range per block, which may begin and end inside a
//    tile. A tile that several blocks share is settled through a workspace: every block leaves
//    its partial accumulator there, and the block that brings the last part adds the parts in
//    block order (a counter, no waiting). The result therefore depends on the sizes and the
//    weights only, never on timing.
//  * Two accumulators alternate in tensor memory, so the epilogue of one stretch runs under the
//    MMAs of the next. The first weights are requested before `griddepcontrol.wait`.
//
// Where it stands (B200, sizes of an 8-billion-parameter model, 8 to 16 rows): level with the
// mma.sync kernel of gemm_small_m.cu and with cuBLAS on the large products (gate/up 43 to 45 us)
// and behind them on the small ones; the weights alone stream in 35.6 us, and settling the shared
// tiles through global memory at the end of the kernel costs about 4 us. The engine keeps it
// behind a switch (ops/gemm.py: STREAM_ROWS).
//
// Epilogues (the reference's formulas: src/paged_kv_serving/engine/model.py:43-51, 256-264):
//   0  bfloat16 out [M, N]          1  float32 out [M, N]
//   2  silu(gate) * up for gate and up rows interleaved in blocks of 128 (a unit of work is then
//      the 256 rows of a gate block and its up block, two accumulators side by side)
//   3  residual: hidden [M, N] (float32) += product in place; out = hidden * norm_weight in
//      bfloat16; sumsq_out [tiles][stride] receives per 128-column tile and row the sum of squares
//      of the new stream, from which the product that reads `out` completes the RMS norm
// Any epilogue scales its result rows by 1 / sqrt(sum of sumsq_in[.][row] / width + eps) when
// `sumsq_in` is given (the other half of that hand-over).
// Every mbarrier wait is bounded; a give-up sets status code 2 and the block leaves in order.
#include "tcgen05.cuh"

namespace pkv {

constexpr int GS_THREADS = 192;
constexpr int GS_BK = 64;
constexpr int GS_MAX_BLOCKS = 160;
enum { GS_BF16 = 0, GS_F32 = 1, GS_SILU = 2, GS_RESIDUAL = 3 };

struct StreamParams {
  void* out;
  int ld_out, M, N, K, n_out;
  float clip;
  float* partials;     // [blocks][2][cols][128]
  int* counters;       // [tiles], zero between launches
  int tiles, chunks;   // units of 128 (silu: 256) weight rows, 64-column blocks of K
  int share, extra;    // units per block: the first `extra` blocks take share + 1
  float* hidden;
  const float* norm_weight;
  float* sumsq_out;
  int sumsq_out_stride;
  const float* sumsq_in;
  int sumsq_parts, sumsq_in_stride;
  float inv_width, norm_eps;
  int* status;
};

__device__ __forceinline__ float gs_silu(float x, float clip) {
  const float c = fminf(fmaxf(x, -clip), clip);
  return x * (1.0f / (1.0f + expf(-c)));
}

__device__ __forceinline__ void epilogue_barrier() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// NPAD: columns of the MMA (activation rows rounded up); EPI: the epilogue.
template <int NPAD, int EPI, int STAGES>
__global__ void __launch_bounds__(GS_THREADS, 1)
gemm_stream_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, const StreamParams p) {
  constexpr bool SILU = EPI == GS_SILU;
  constexpr int W_ROWS = SILU ? 256 : 128;
  constexpr uint32_t W_BYTES = W_ROWS * 128;
  constexpr uint32_t X_BYTES = NPAD * 128;
  constexpr uint32_t STAGE_BYTES = W_BYTES + X_BYTES;
  constexpr int COLS = SILU ? 2 * NPAD : NPAD;              // accumulator columns in use
  constexpr int BUF_COLS = COLS < 32 ? 32 : COLS;           // columns of one accumulator buffer
  constexpr uint32_t TMEM_COLS = 2 * BUF_COLS;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t full_bar[STAGES], empty_bar[STAGES], acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag, last_flag;
  __shared__ float inv_root_s[128];
  __shared__ float squares[4][EPI == GS_RESIDUAL ? NPAD : 1];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int me = blockIdx.x;
  const int range_begin = me * p.share + min(me, p.extra);
  const int range_end = range_begin + p.share + (me < p.extra ? 1 : 0);

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(&full_bar[i], 1);
      mbar_init(&empty_bar[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&acc_full[i], 1);
      mbar_init(&acc_empty[i], 4);
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
      auto load_w = [&](int j, int u) {
        const int stage = j % STAGES;
        const int tile = u / p.chunks, kb = u - tile * p.chunks;
        mbar_expect_tx(&full_bar[stage], STAGE_BYTES);
        tma_load_2d(ring + (size_t)stage * STAGE_BYTES, &map_w, &full_bar[stage], kb * GS_BK, tile * W_ROWS);
      };
      auto load_x = [&](int j, int u) {
        const int stage = j % STAGES;
        const int tile = u / p.chunks, kb = u - tile * p.chunks;
        tma_load_2d(ring + (size_t)stage * STAGE_BYTES + W_BYTES, &map_x, &full_bar[stage], kb * GS_BK, 0);
      };
      const int n_units = range_end - range_begin;
      const int ahead = min(STAGES, n_units);
      // the weights do not depend on the kernel before this one: their first copies start now;
      // the activations come from that kernel and are asked for once it has finished
      for (int j = 0; j < ahead; ++j) load_w(j, range_begin + j);
      wait_for_prior_kernels();
      for (int j = 0; j < ahead; ++j) load_x(j, range_begin + j);
      int j = ahead;
      bool ok = true;
      for (; j < n_units; ++j) {
        if (!mbar_wait(&empty_bar[j % STAGES], ((j / STAGES) - 1) & 1, aborted)) { ok = false; break; }
        load_w(j, range_begin + j);
        load_x(j, range_begin + j);
      }
      // this block has asked for all its weights: the next kernel may take the places that free up
      dependents_may_launch();
      if (!ok || *aborted) {
        for (int i = max(0, j - STAGES); i < j; ++i) {
          const long long start = clock64();
          while (!mbar_try_wait(&full_bar[i % STAGES], (i / STAGES) & 1) && clock64() - start < GM_WAIT_CYCLES) {}
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(NPAD >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
      int j = 0, local = 0;
      bool ok = true;
      int u = range_begin;
      while (u < range_end && ok) {
        const int tile = u / p.chunks, cb = u - tile * p.chunks;
        const int ce = min(p.chunks, cb + (range_end - u));
        const int buf = local & 1;
        if (local >= 2) ok = mbar_wait(&acc_empty[buf], ((local >> 1) - 1) & 1, aborted);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BUF_COLS;
        for (int kb = cb; kb < ce; ++kb, ++j) {
          const int stage = j % STAGES;
          ok = mbar_wait(&full_bar[stage], (j / STAGES) & 1, aborted);
          if (!ok) break;
          tc_fence_after();
          const uint32_t w_addr = smem_addr(ring + (size_t)stage * STAGE_BYTES);
          const uint64_t w_desc = umma_desc(w_addr), x_desc = umma_desc(w_addr + W_BYTES);
#pragma unroll
          for (int k = 0; k < GS_BK / 16; ++k) {
            const uint32_t acc = (kb > cb || k > 0) ? 1u : 0u;
            umma_bf16(d_tmem, w_desc + 2 * k, x_desc + 2 * k, idesc, acc);
            if (SILU) umma_bf16(d_tmem + NPAD, umma_desc(w_addr + 128 * 128) + 2 * k, x_desc + 2 * k, idesc, acc);
          }
          umma_commit(&empty_bar[stage]);
        }
        if (ok) umma_commit(&acc_full[buf]);
        u += ce - cb;
        ++local;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;                  // weight row inside the tile
    const int et = (warp - 2) * 32 + lane;                // 0..127 among the epilogue threads
    wait_for_prior_kernels();                             // hidden, sumsq_in come from earlier kernels
    const float* inv_root = nullptr;
    if (p.sumsq_in != nullptr) {
      if (et < p.M) {
        float q = 0.0f;
        for (int part = 0; part < p.sumsq_parts; ++part) q += p.sumsq_in[(size_t)part * p.sumsq_in_stride + et];
        inv_root_s[et] = 1.0f / sqrtf(q * p.inv_width + p.norm_eps);
      }
      epilogue_barrier();
      inv_root = inv_root_s;
    }

    // finishes 32 accumulator columns [c0, c0 + 32) of this thread's weight row
    auto finish = [&](int tile, int c0, const float (&a)[32], const float (&b)[32]) {
      const int n = tile * 128 + row;
      if (EPI == GS_SILU) {
        if (n < p.n_out) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int m = c0 + i;
            if (m < p.M) {
              const float scale = inv_root ? inv_root[m] : 1.0f;
              reinterpret_cast<bf16*>(p.out)[(size_t)m * p.ld_out + n] =
                  __float2bfloat16_rn(gs_silu(a[i] * scale, p.clip) * (b[i] * scale));
            }
          }
        }
      } else if (EPI == GS_RESIDUAL) {
        const float w = n < p.N ? p.norm_weight[n] : 0.0f;
        // the stream's old values first, all of them in flight together: read one by one between
        // the stores below (which the compiler must assume to alias them) each would cost a
        // round trip to L2
        float old[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int m = c0 + i;
          old[i] = (i < NPAD && m < p.M && n < p.N) ? __ldcg(p.hidden + (size_t)m * p.ld_out + n) : 0.0f;
        }
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int m = c0 + i;
          float sq = 0.0f;
          if (m < p.M && n < p.N) {
            const size_t at = (size_t)m * p.ld_out + n;
            const float x = old[i] + a[i] * (inv_root ? inv_root[m] : 1.0f);
            p.hidden[at] = x;
            reinterpret_cast<bf16*>(p.out)[at] = __float2bfloat16_rn(x * w);
            sq = x * x;
          }
          if (c0 + i < NPAD) {            // uniform across the warp: every lane takes part in the sum
            sq = warp_sum(sq);
            if (lane == 0) squares[warp - 2][c0 + i] = sq;
          }
        }
      } else {
        if (n < p.N) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int m = c0 + i;
            if (m < p.M) {
              const float v = a[i] * (inv_root ? inv_root[m] : 1.0f);
              if (EPI == GS_F32) reinterpret_cast<float*>(p.out)[(size_t)m * p.ld_out + n] = v;
              else reinterpret_cast<bf16*>(p.out)[(size_t)m * p.ld_out + n] = __float2bfloat16_rn(v);
            }
          }
        }
      }
    };
    auto finish_tile_sums = [&](int tile) {
      if (EPI == GS_RESIDUAL) {
        // the tile's sum of squares per activation row: the four warps' sums in one fixed order
        epilogue_barrier();
        if (et < p.M) p.sumsq_out[(size_t)tile * p.sumsq_out_stride + et] =
            (squares[0][et] + squares[1][et]) + (squares[2][et] + squares[3][et]);
        epilogue_barrier();
      }
    };

    const int big = p.extra * (p.share + 1);
    auto block_of = [&](int u) { return u < big ? u / (p.share + 1) : p.extra + (u - big) / p.share; };
    auto begin_of = [&](int b) { return b * p.share + min(b, p.extra); };

    int local = 0;
    int u = range_begin;
    bool ok = true;
    while (u < range_end && ok) {
      const int tile = u / p.chunks, cb = u - tile * p.chunks;
      const int ce = min(p.chunks, cb + (range_end - u));
      const int buf = local & 1;
      ok = __all_sync(0xffffffffu, mbar_wait(&acc_full[buf], (local >> 1) & 1, aborted) ? 1 : 0) != 0;
      // the four warps go on or give up together: a wait that fails in one of them has set the
      // block's abort flag, and all of them look at it behind the same barrier
      epilogue_barrier();
      if (!ok || *aborted) break;
      tc_fence_after();
      const uint32_t lane_addr = tmem_base + buf * BUF_COLS + ((uint32_t)(quarter * 32) << 16);
      const bool whole = cb == 0 && ce == p.chunks;
      if (whole) {
#pragma unroll 1
        for (int c = 0; c < NPAD; c += 32) {
          float a[32], b[32];
          tmem_load32(lane_addr + c, a);
          if (SILU) {
            if (NPAD >= 32) {
              tmem_load32(lane_addr + NPAD + c, b);
            } else {                   // gate and up columns share one 32-column read
#pragma unroll
              for (int i = 0; i < 32; ++i) b[i] = a[(NPAD + i) & 31];
            }
          }
          if (c + 32 >= NPAD) {        // the last read of this accumulator: hand it back
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);
          }
          finish(tile, c, a, b);
        }
        finish_tile_sums(tile);
      } else {
        // part of a tile: leave it in the workspace; the block that brings the last part adds them
        const int tile_u0 = tile * p.chunks, tile_u1 = tile_u0 + p.chunks;
        const int b_lo = block_of(tile_u0), b_hi = block_of(tile_u1 - 1);
        float* mine = p.partials + ((size_t)me * 2 + (range_begin >= tile_u0 ? 0 : 1)) * (size_t)(COLS * 128);
#pragma unroll 1
        for (int c = 0; c < COLS; c += 32) {
          float a[32];
          tmem_load32(lane_addr + c, a);
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (c + i < COLS) __stcg(mine + (size_t)(c + i) * 128 + row, a[i]);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[buf]);
        __threadfence();
        epilogue_barrier();
        if (et == 0) last_flag = atomicAdd(p.counters + tile, 1) == b_hi - b_lo;
        epilogue_barrier();
        if (last_flag) {
          __threadfence();
#pragma unroll 1
          for (int c = 0; c < NPAD; c += 32) {
            float a[32], b[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) a[i] = b[i] = 0.0f;
            for (int q = b_lo; q <= b_hi; ++q) {
              const float* theirs = p.partials + ((size_t)q * 2 + (begin_of(q) >= tile_u0 ? 0 : 1)) * (size_t)(COLS * 128);
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                if (c + i < NPAD) {
                  a[i] += __ldcg(theirs + (size_t)(c + i) * 128 + row);
                  if (SILU) b[i] += __ldcg(theirs + (size_t)(NPAD + c + i) * 128 + row);
                }
              }
            }
            finish(tile, c, a, b);
          }
          finish_tile_sums(tile);
          if (et == 0) p.counters[tile] = 0;   // ready for the next launch
        }
        epilogue_barrier();                     // last_flag and squares are written again in the next round
      }
      u += ce - cb;
      ++local;
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
struct WeightMapKey {
  const void* base;
  long long rows, cols;
  int box;
  CUtensorMap map;
};

static bool weight_map(const void* base, long long rows, long long cols, int box_rows, CUtensorMap* out) {
  static WeightMapKey cache[1024];
  static int used = 0;
  for (int i = 0; i < used; ++i)
    if (cache[i].base == base && cache[i].rows == rows && cache[i].cols == cols && cache[i].box == box_rows) {
      *out = cache[i].map;
      return true;
    }
  static int victim = 0;              // a full table gives up its entries in turn
  WeightMapKey& slot = cache[used < 1024 ? used : victim];
  if (make_tile_map(&slot.map, base, rows, cols, cols, box_rows)) {
    slot.base = nullptr;
    return false;
  }
  slot.base = base; slot.rows = rows; slot.cols = cols; slot.box = box_rows;
  if (used < 1024) ++used;
  else victim = (victim + 1) % 1024;
  *out = slot.map;
  return true;
}

static int gs_sm_count() {
  static int count[64] = {0};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return 1;
  if (count[device] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || n <= 0) n = 1;
    count[device] = n;
  }
  return count[device];
}

template <int NPAD, int EPI>
static int launch_stream(const CUtensorMap& mw, const CUtensorMap& mx, StreamParams p, int chained, cudaStream_t s) {
  constexpr int W_ROWS = EPI == GS_SILU ? 256 : 128;
  constexpr int STAGE_BYTES = W_ROWS * 128 + NPAD * 128;
  constexpr int STAGES = (200 * 1024) / STAGE_BYTES < 8 ? (200 * 1024) / STAGE_BYTES : 8;
  static_assert(STAGES >= 3, "a ring needs a few stages");
  const size_t smem = (size_t)STAGES * STAGE_BYTES + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_stream_kernel<NPAD, EPI, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const long long units = (long long)p.tiles * p.chunks;
  long long blocks = gs_sm_count() < GS_MAX_BLOCKS ? gs_sm_count() : GS_MAX_BLOCKS;
  if (blocks > units) blocks = units;
  p.share = (int)(units / blocks);
  p.extra = (int)(units % blocks);
  return launch_kernel(gemm_stream_kernel<NPAD, EPI, STAGES>, dim3((unsigned)blocks), dim3(GS_THREADS), smem, s, chained != 0, 0,
                       mw, mx, p);
}

template <int EPI>
static int dispatch_stream(const CUtensorMap& mw, const void* x, int ldx, const StreamParams& p, int chained, cudaStream_t s) {
  const int npad = p.M <= 16 ? 16 : (p.M <= 32 ? 32 : (p.M <= 64 ? 64 : 128));
  alignas(64) CUtensorMap mx;
  const int r = make_tile_map(&mx, x, p.M, p.K, ldx, npad);
  if (r) return r;
  switch (npad) {
    case 16: return launch_stream<16, EPI>(mw, mx, p, chained, s);
    case 32: return launch_stream<32, EPI>(mw, mx, p, chained, s);
    case 64: return launch_stream<64, EPI>(mw, mx, p, chained, s);
    default: return launch_stream<128, EPI>(mw, mx, p, chained, s);
  }
}

}  // namespace pkv

using namespace pkv;

// Bytes of the workspace for products of up to `max_rows` rows (partial accumulators and tile
// counters); it must be zero before its first use and is left zero by every launch.
PKV_EXPORT long long pkv_gemm_stream_workspace_bytes(int max_rows) {
  (void)max_rows;   // one size for every row count: the counters sit behind the largest partials
  return (long long)GS_MAX_BLOCKS * 2 * (2 * 128) * 128 * sizeof(float) + 65536LL * sizeof(int);
}

PKV_EXPORT int pkv_gemm_stream_supports(long long x, long long w, int ldx, int M, int N, int K, int epilogue) {
  if (M < 1 || M > 128 || N < 1 || K < GS_BK || K % GS_BK != 0 || ldx % 8 != 0) return 0;
  if ((x | w) & 15) return 0;
  if (epilogue == GS_SILU && N % 256 != 0) return 0;
  if ((long long)((N + 127) / 128) > 65536) return 0;
  return 1;
}

// out = x . w^T for 1 to 128 rows. `x` is [M, K] with row stride `ldx` (elements), `w` [N, K]
// contiguous, both bfloat16, K a multiple of 64. Epilogues as listed at the top of this file;
// `sumsq_out` is [ceil(N / 128)][sumsq_out_stride], `sumsq_in` [sumsq_parts][sumsq_in_stride].
// `workspace` as sized by pkv_gemm_stream_workspace_bytes(rows >= M). `chained` non-zero launches
// as a programmatic dependent of the kernel before it on the stream.
PKV_EXPORT int pkv_gemm_stream(const void* x, int ldx, const void* w, void* out, int M, int N, int K, int epilogue, int n_out,
                               float clip, int chained, void* workspace, long long workspace_bytes, float* hidden,
                               const float* norm_weight, float* sumsq_out, int sumsq_out_stride, const float* sumsq_in,
                               int sumsq_parts, int sumsq_in_stride, int width, float norm_eps, int* status, void* stream) {
  if (!pkv_gemm_stream_supports((long long)(uintptr_t)x, (long long)(uintptr_t)w, ldx, M, N, K, epilogue)) return PKV_ERR_SIZE;
  if (!workspace || workspace_bytes < pkv_gemm_stream_workspace_bytes(M) || ((uintptr_t)workspace & 15)) return PKV_ERR_SIZE;
  if (!status) return PKV_ERR_SIZE;
  StreamParams p = {};
  p.out = out; p.M = M; p.N = N; p.K = K; p.clip = clip; p.n_out = n_out;
  // the tile counters at a place that does not move with the row count (behind the largest
  // partial accumulators): they must be zero from launch to launch, the partials may hold anything
  p.partials = static_cast<float*>(workspace);
  p.counters = reinterpret_cast<int*>(static_cast<uint8_t*>(workspace) + (size_t)GS_MAX_BLOCKS * 2 * (2 * 128) * 128 * sizeof(float));
  p.chunks = K / GS_BK;
  p.hidden = hidden; p.norm_weight = norm_weight; p.sumsq_out = sumsq_out; p.sumsq_out_stride = sumsq_out_stride;
  p.sumsq_in = sumsq_in; p.sumsq_parts = sumsq_parts; p.sumsq_in_stride = sumsq_in_stride;
  p.inv_width = width > 0 ? 1.0f / (float)width : 0.0f; p.norm_eps = norm_eps;
  p.status = status;
  if (sumsq_in && (sumsq_parts <= 0 || width <= 0 || sumsq_in_stride < M)) return PKV_ERR_SIZE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  alignas(64) CUtensorMap mw;
  if (!weight_map(w, N, K, epilogue == GS_SILU ? 256 : 128, &mw)) return PKV_ERR_SIZE;
  switch (epilogue) {
    case GS_BF16:
    case GS_F32:
      p.tiles = (N + 127) / 128; p.ld_out = N;
      return epilogue == GS_BF16 ? dispatch_stream<GS_BF16>(mw, x, ldx, p, chained, s)
                                 : dispatch_stream<GS_F32>(mw, x, ldx, p, chained, s);
    case GS_SILU:
      if (n_out <= 0 || n_out > N / 2) return PKV_ERR_SIZE;
      p.tiles = N / 256; p.ld_out = n_out;
      return dispatch_stream<GS_SILU>(mw, x, ldx, p, chained, s);
    case GS_RESIDUAL:
      if (!hidden || !norm_weight || !sumsq_out || sumsq_out_stride < M) return PKV_ERR_SIZE;
      p.tiles = (N + 127) / 128; p.ld_out = N;
      return dispatch_stream<GS_RESIDUAL>(mw, x, ldx, p, chained, s);
    default: return PKV_ERR_SIZE;
  }
}
