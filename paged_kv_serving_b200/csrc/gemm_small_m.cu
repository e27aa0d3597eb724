// Matrix products of decode steps: a few rows of activations against a whole weight matrix,
// out[M, N] = x[M, K] . w[N, K]^T in bfloat16 with float32 accumulation, for M up to 32.
//
// Such a product reads every weight once and does almost no arithmetic per byte, so the kernel is
// built around the weight stream.
//
//  * The weight rows are the 16-row side of mma.sync.m16n8k16 and the activations its 8-wide
//    side. A lane loads 16 contiguous bytes of a weight row straight from global memory into
//    registers and uses them as the A fragments of two k-steps; the activations are loaded with
//    the same pattern, so the order of k inside a 32-wide chunk is permuted in the same way on
//    both sides and the dot products are unchanged. There is no shared-memory staging and no
//    barrier in the main loop; two batches of weight loads are in flight per warp, and the
//    activations, which every block reads again, come from L1 after an SM's first blocks.
//  * The work is 16-row tiles x 32-wide chunks of K. A block takes one tile, or, where whole tiles
//    would leave a last wave of blocks nearly empty, an even contiguous range of the work that may
//    begin and end inside a tile. Inside a block the eight warps split each tile's share of K and
//    add their sums through shared memory in warp order. Partial sums of a shared tile go through
//    a workspace, and the block that delivers the last part adds the parts in block order. The
//    result therefore depends on the sizes and the weights only, never on timing or on how many
//    rows the batch has.
//  * The first weights are requested before `griddepcontrol.wait`: launched as a programmatic
//    dependent after a kernel that leaves the SMs mostly idle (a norm over a few rows), the
//    kernel has its first weights on the way while that kernel ends. A block lets the next
//    kernel start only when it has read its own weights.
//
// Epilogues: bfloat16, float32, or silu(gate) * up for gate and up rows interleaved in blocks of
// 128 (the layout of the fused feed-forward weight); the reference's feed-forward is
// src/paged_kv_serving/engine/model.py:258-264.
#include "common.cuh"

namespace {

using pkv::bf16;

constexpr int SMALL_WARPS = 8;
constexpr int SMALL_CHUNK = 32;           // k per chunk: 4 lanes x 8 elements
constexpr int SMALL_MAX_TILES = 65536;    // counters in the workspace
constexpr int SMALL_MAX_BLOCKS = 320;
constexpr int SMALL_SLOT_FLOATS = 8 * 4 * 32;  // largest set of sums of a block
constexpr int EPI_BF16 = 0, EPI_F32 = 1, EPI_SILU_MUL = 2, EPI_RESIDUAL = 3, EPI_ROPE_KV = 4;

__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// weights are read once: past L1, and first to leave L2
__device__ __forceinline__ uint64_t stream_policy() {
  uint64_t policy;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
  return policy;
}
__device__ __forceinline__ uint4 load_stream(const void* p, uint64_t policy) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.v4.u32 {%0,%1,%2,%3}, [%4], %5;"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p), "l"(policy));
  return v;
}

struct SmallParams {
  const bf16* x;
  const bf16* w;
  void* out;
  float* partials;   // [blocks][2][SMALL_SLOT_FLOATS]
  int* counters;     // [tiles], zero between launches
  int M, N, K, ldx, ld_out, n_out;
  int tiles, chunks;  // 16-row tiles (pairs of them with the fused activation), chunks of K per tile
  int share, extra;   // units per block: the first `extra` blocks take share + 1, the others share
  float clip;
  // epilogue 3 (residual): the product is added to the float32 stream in place, the stream times
  // the next norm's weight is stored in bfloat16, and each tile leaves the sum of squares of its
  // 16 columns per row, so that the kernel that reads `xw` can finish the RMS norm by itself
  float* hidden;             // [M, N]
  const float* norm_weight;  // [N]
  float* sumsq_out;          // [tiles][32]
  // any epilogue: rows of the result are scaled by 1 / sqrt(sum of sumsq_in[.][row] / width + eps),
  // which completes an RMS norm whose weight the producer already applied to `x`
  const float* sumsq_in;     // [sumsq_parts][32], or null
  int sumsq_parts;
  float inv_width, norm_eps;
  // epilogue 4 (rotary + cache): `w` is a fused q/k/v projection; queries and keys are rotated by
  // their row's position (half-split pairs), queries go to `out`, keys and values to the paged
  // pools [pages, n_kv, page_size, head_dim] at `slots` (null or -1: nothing is stored)
  const int32_t* positions;  // [M]
  const float* cos_t;        // [positions][head_dim / 2]
  const float* sin_t;
  bf16* k_pool;
  bf16* v_pool;
  const int32_t* slots;      // [M] or null
  int n_heads, n_kv, head_dim, page_size;
  // a slot outside the pools or a position outside the tables is recorded in the status word;
  // the store is then skipped and the rotation uses position 0
  int num_slots, max_pos;
  int* status;
};

template <int RT, int EPI>
__device__ __forceinline__ int tile_first_row(int tile, int r) {
  if (EPI == EPI_SILU_MUL) return (tile >> 3) * 256 + (tile & 7) * 16 + r * 128;  // gate rows, then the up rows
  return (tile * RT + r) * 16;
}

// Stores one value of a finished tile. Sum number `slot` = (r MT + j) 4 + i of lane l is weight
// row first_row(r) + l/4 + 8 (i/2) against activation row 8 j + 2 (l%4) + i%2; with the fused
// activation `s` is the gate sum and `up` the sum of the matching up row. `inv_root` holds the
// row scales (null: none). Returns the square of the new stream value (residual epilogue), else 0.
template <int MT, int RT, int EPI>
__device__ __forceinline__ float store_value(const SmallParams& p, const float* inv_root, int tile, int slot, int l,
                                             float s, float up, float early_a = 0.0f, float early_b = 0.0f) {
  const int i = slot & 3, j = (slot >> 2) % MT, r = slot / (4 * MT);
  const int m = j * 8 + 2 * (l & 3) + (i & 1);
  const int row_in_tile = (l >> 2) + 8 * (i >> 1);
  if (m >= p.M) return 0.0f;
  if (inv_root) {
    s *= inv_root[m];
    up *= inv_root[m];
  }
  if (EPI == EPI_SILU_MUL) {
    const int col = (tile >> 3) * 128 + (tile & 7) * 16 + row_in_tile;
    if (col >= p.n_out) return 0.0f;
    const float clipped = fminf(fmaxf(s, -p.clip), p.clip);
    const float act = s * (1.0f / (1.0f + expf(-clipped)));
    reinterpret_cast<bf16*>(p.out)[(size_t)m * p.ld_out + col] = __float2bfloat16_rn(act * up);
    return 0.0f;
  }
  const int col = tile_first_row<RT, EPI>(tile, r) + row_in_tile;
  if (col >= p.N) return 0.0f;
  const size_t at = (size_t)m * p.ld_out + col;
  if (EPI == EPI_RESIDUAL) {   // early_a, early_b: the stream's value and the norm weight, loaded ahead
    const float x = early_a + s;
    p.hidden[at] = x;
    reinterpret_cast<bf16*>(p.out)[at] = __float2bfloat16_rn(x * early_b);
    return x * x;
  }
  if (EPI == EPI_F32) reinterpret_cast<float*>(p.out)[at] = s;
  else reinterpret_cast<bf16*>(p.out)[at] = __float2bfloat16_rn(s);
  return 0.0f;
}

// Rotary epilogue: `lo` and `hi` are element e = 8 (tile % (head_dim / 16)) + l/4 of a head's first
// half and its partner e + head_dim/2, for activation row 8 j + 2 (l%4) + odd.
template <int MT>
__device__ __forceinline__ void store_rotated(const SmallParams& p, const float* inv_root, int tile, int j, int odd, int l,
                                              float lo, float hi, float c, float sn, int slot) {
  const int m = j * 8 + 2 * (l & 3) + odd;
  if (m >= p.M) return;
  if (inv_root) {
    lo *= inv_root[m];
    hi *= inv_root[m];
  }
  const int per_head = p.head_dim >> 4, head = tile / per_head, half = p.head_dim >> 1;
  const int e = (tile - head * per_head) * 8 + (l >> 2);
  if (head >= p.n_heads + 2 * p.n_kv) return;
  const bool is_v = head >= p.n_heads + p.n_kv;
  if (!is_v && p.cos_t != nullptr) {   // c, sn: loaded ahead for this row's position and element e
    const float a = lo * c - hi * sn, b = hi * c + lo * sn;
    lo = a;
    hi = b;
  }
  if (head < p.n_heads) {
    bf16* q = reinterpret_cast<bf16*>(p.out) + (size_t)m * p.ld_out + (size_t)head * p.head_dim + e;
    q[0] = __float2bfloat16_rn(lo);
    q[half] = __float2bfloat16_rn(hi);
    return;
  }
  if (slot < 0) return;
  const int page = slot / p.page_size, off = slot - page * p.page_size;
  const int kvh = is_v ? head - p.n_heads - p.n_kv : head - p.n_heads;
  bf16* dst = (is_v ? p.v_pool : p.k_pool) + (((size_t)page * p.n_kv + kvh) * p.page_size + off) * p.head_dim + e;
  dst[0] = __float2bfloat16_rn(lo);
  dst[half] = __float2bfloat16_rn(hi);
}

// How many values (or pairs of values) the threads of a block finish per tile.
template <int MT, int RT, int EPI>
struct OUT_COUNT {
  static constexpr int VALUE = (EPI == EPI_SILU_MUL ? MT * 4 : (EPI == EPI_ROPE_KV ? MT * 2 : RT * MT * 4)) * 32;
};

// MT: 8-row groups of activations (M <= 8 MT). RT: 16-row weight tiles per unit of work.
// PER_SM: blocks that share an SM; with three the batches of loads are half as deep.
template <int MT, int RT, int EPI, int PER_SM>
__global__ void __launch_bounds__(SMALL_WARPS * 32, PER_SM) gemm_small_m_kernel(const SmallParams p) {
  constexpr int DEPTH = (PER_SM == 3 ? 2 : 4) / RT;   // chunks per batch of loads
  constexpr int SLOTS = RT * MT * 4;         // sums per lane
  static_assert(SLOTS * 32 <= SMALL_SLOT_FLOATS, "a block's sums fit a workspace slot");
  __shared__ float red[SMALL_WARPS][SLOTS][32];
  __shared__ int is_last;
  __shared__ float inv_root_s[32];
  __shared__ float squares[EPI == EPI_RESIDUAL ? SLOTS * 32 : 1];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  // units of work (tile-major) [range_begin, range_end) of this block; fewer than 2^31 in all
  const int me = blockIdx.x;
  const int range_begin = me * p.share + min(me, p.extra);
  const int range_end = range_begin + p.share + (me < p.extra ? 1 : 0);
  const uint64_t policy = stream_policy();

  const bf16* xp[MT];
#pragma unroll
  for (int j = 0; j < MT; ++j) xp[j] = p.x + (size_t)min(j * 8 + g, p.M - 1) * p.ldx + t * 8;
  const bf16* wp[RT][2];
  auto point_at_tile = [&](int tile) {
#pragma unroll
    for (int r = 0; r < RT; ++r) {
      int row = tile_first_row<RT, EPI>(tile, r) + g, partner = row + 8;
      if (EPI == EPI_ROPE_KV) {
        // a tile holds 8 elements of a head's first half and the 8 they are rotated with, so that
        // one thread ends up with both values of a pair
        const int per_head = p.head_dim >> 4, head = tile / per_head;
        row = head * p.head_dim + (tile - head * per_head) * 8 + g;
        partner = row + (p.head_dim >> 1);
      }
      wp[r][0] = p.w + (size_t)min(row, p.N - 1) * p.K + t * 8;
      wp[r][1] = p.w + (size_t)min(partner, p.N - 1) * p.K + t * 8;
    }
  };
  // the share of one warp in the chunks [cb, ce) of a tile
  auto warp_share = [&](int cb, int ce, int& wb, int& we) {
    const int per = (ce - cb + SMALL_WARPS - 1) / SMALL_WARPS;
    wb = min(ce, cb + warp * per);
    we = min(ce, wb + per);
  };

  float acc[RT][MT][4];
  uint4 wa[2][DEPTH][RT][2];
  auto load_batch = [&](int buf, int c) {
#pragma unroll
    for (int u = 0; u < DEPTH; ++u) {
      const int cc = min(c + u, p.chunks - 1);  // past the share: a valid address, the value is unused
#pragma unroll
      for (int r = 0; r < RT; ++r) {
        wa[buf][u][r][0] = load_stream(wp[r][0] + (size_t)cc * SMALL_CHUNK, policy);
        wa[buf][u][r][1] = load_stream(wp[r][1] + (size_t)cc * SMALL_CHUNK, policy);
      }
    }
  };
  auto use_batch = [&](int buf, int c, int we) {
#pragma unroll
    for (int u = 0; u < DEPTH; ++u) {
      if (c + u < we) {
#pragma unroll
        for (int j = 0; j < MT; ++j) {
          // every block reads all activations; after the first blocks of an SM they come from L1
          const uint4 xv = *reinterpret_cast<const uint4*>(xp[j] + (size_t)(c + u) * SMALL_CHUNK);
#pragma unroll
          for (int r = 0; r < RT; ++r) {
            mma_16816(acc[r][j], wa[buf][u][r][0].x, wa[buf][u][r][1].x, wa[buf][u][r][0].y, wa[buf][u][r][1].y, xv.x, xv.y);
            mma_16816(acc[r][j], wa[buf][u][r][0].z, wa[buf][u][r][1].z, wa[buf][u][r][0].w, wa[buf][u][r][1].w, xv.z, xv.w);
          }
        }
      }
    }
  };

  // first segment of this block's range
  int u0 = range_begin;
  int tile = u0 / p.chunks;
  int cb = u0 - tile * p.chunks;
  int ce = min(p.chunks, cb + (range_end - u0));
  int wb = 0, we = 0;
  if (u0 < range_end) {
    point_at_tile(tile);
    warp_share(cb, ce, wb, we);
    if (wb < we) load_batch(0, wb);
  }
  // the activations come from the kernel before this one; the weights above do not
  pkv::wait_for_prior_kernels();

  const float* inv_root = nullptr;
  if (p.sumsq_in != nullptr) {
    // finish the norm of the rows: the parts are added in one fixed order
    for (int m = warp; m < p.M; m += SMALL_WARPS) {
      float q = 0.0f;
      for (int part = lane; part < p.sumsq_parts; part += 32) q += p.sumsq_in[part * 32 + m];
      q = pkv::warp_sum(q);
      if (lane == 0) inv_root_s[m] = 1.0f / sqrtf(q * p.inv_width + p.norm_eps);
    }
    inv_root = inv_root_s;   // read after the block's next barrier
  }

  // What an epilogue needs besides the sums (the stream's old values and the norm weight; the
  // rotation's cosine, sine and cache slot) is requested when a tile begins, not when it ends.
  constexpr int EARLY = (EPI == EPI_RESIDUAL || EPI == EPI_ROPE_KV) ? (OUT_COUNT<MT, RT, EPI>::VALUE + SMALL_WARPS * 32 - 1) / (SMALL_WARPS * 32) : 1;
  float early_a[EARLY], early_b[EARLY];
  int early_slot[EARLY];

  while (u0 < range_end) {
    if (EPI == EPI_RESIDUAL || EPI == EPI_ROPE_KV) {
#pragma unroll
      for (int it = 0; it < EARLY; ++it) {
        const int idx = threadIdx.x + it * SMALL_WARPS * 32;
        early_a[it] = early_b[it] = 0.0f;
        early_slot[it] = -1;
        if (idx >= OUT_COUNT<MT, RT, EPI>::VALUE) continue;
        const int l = idx & 31;
        if (EPI == EPI_RESIDUAL) {
          const int slot = idx >> 5, i = slot & 3, j = (slot >> 2) % MT;
          const int m = j * 8 + 2 * (l & 3) + (i & 1), col = tile * 16 + (l >> 2) + 8 * (i >> 1);
          if (m < p.M && col < p.N) {
            early_a[it] = p.hidden[(size_t)m * p.ld_out + col];
            early_b[it] = p.norm_weight[col];
          }
        } else {
          const int m = (idx >> 6) * 8 + 2 * (l & 3) + ((idx >> 5) & 1);
          if (m < p.M) {
            const int per_head = p.head_dim >> 4, head = tile / per_head;
            const int e = (tile - head * per_head) * 8 + (l >> 2);
            if (p.cos_t != nullptr && head < p.n_heads + p.n_kv) {
              int position = p.positions[m];
              if (position < 0 || position >= p.max_pos) {
                if (p.status) atomicExch(p.status, PKV_STATUS_OUT_OF_RANGE);
                position = 0;
              }
              const size_t at = (size_t)position * (p.head_dim >> 1) + e;
              early_a[it] = p.cos_t[at];
              early_b[it] = p.sin_t[at];
            }
            if (p.slots != nullptr && head >= p.n_heads) {
              int slot = p.slots[m];
              if (slot >= p.num_slots || slot < -1) {
                if (p.status) atomicExch(p.status, PKV_STATUS_OUT_OF_RANGE);
                slot = -1;
              }
              early_slot[it] = slot;
            }
          }
        }
      }
    }
#pragma unroll
    for (int r = 0; r < RT; ++r)
#pragma unroll
      for (int j = 0; j < MT; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[r][j][i] = 0.0f;
    for (int c = wb; c < we; c += 2 * DEPTH) {
      if (c + DEPTH < we) load_batch(1, c + DEPTH);
      use_batch(0, c, we);
      if (c + 2 * DEPTH < we) load_batch(0, c + 2 * DEPTH);
      if (c + DEPTH < we) use_batch(1, c + DEPTH, we);
    }
    // request the first weights of the next segment before this one is added up
    const int this_tile = tile, this_cb = cb, this_ce = ce;
    u0 += ce - cb;
    if (u0 < range_end) {
      ++tile;
      cb = 0;
      ce = min(p.chunks, range_end - u0);
      point_at_tile(tile);
      warp_share(cb, ce, wb, we);
      if (wb < we) load_batch(0, wb);
    } else {
      // This block has read its weights. Once every block has, the next kernel may take the
      // places that free up and request its own first weights. (Earlier would be no gain: its
      // blocks would sit beside blocks of this kernel that still wait for a place.)
      pkv::dependents_may_launch();
    }

#pragma unroll
    for (int r = 0; r < RT; ++r)
#pragma unroll
      for (int j = 0; j < MT; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) red[warp][(r * MT + j) * 4 + i][lane] = acc[r][j][i];
    __syncthreads();

    // A thread finishes one sum, or two that belong together: gate and up of the fused activation
    // (slots s and s + 4 MT), or a rotary pair (slots 4 j + odd and 4 j + 2 + odd).
    constexpr int OUT_SLOTS = (EPI == EPI_SILU_MUL) ? MT * 4 : (EPI == EPI_ROPE_KV ? MT * 2 : SLOTS);
    auto first_slot = [](int idx) { return EPI == EPI_ROPE_KV ? ((idx >> 6) * 4 + ((idx >> 5) & 1)) : (idx >> 5); };
    constexpr int SECOND = EPI == EPI_SILU_MUL ? MT * 4 : 2;   // distance to the second slot, where there is one
    constexpr bool PAIRED = EPI == EPI_SILU_MUL || EPI == EPI_ROPE_KV;
    auto emit = [&](int idx, int slot, int l, float s, float up) {
      const int it = EARLY > 1 ? idx / (SMALL_WARPS * 32) : 0;
      if (EPI == EPI_ROPE_KV) {
        store_rotated<MT>(p, inv_root, this_tile, slot >> 2, slot & 1, l, s, up, early_a[it], early_b[it], early_slot[it]);
      } else {
        const float q = store_value<MT, RT, EPI>(p, inv_root, this_tile, slot, l, s, up, early_a[it], early_b[it]);
        if (EPI == EPI_RESIDUAL) squares[idx] = q;
      }
    };
    const bool whole = this_cb == 0 && this_ce == p.chunks;
    bool stored = whole;   // whether this block stored the tile (the same for all its threads)
    if (whole) {
      for (int idx = threadIdx.x; idx < OUT_SLOTS * 32; idx += SMALL_WARPS * 32) {
        const int l = idx & 31, slot = first_slot(idx);
        float s = 0.0f, up = 0.0f;
#pragma unroll
        for (int wi = 0; wi < SMALL_WARPS; ++wi) s += red[wi][slot][l];
        if (PAIRED) {
#pragma unroll
          for (int wi = 0; wi < SMALL_WARPS; ++wi) up += red[wi][slot + SECOND][l];
        }
        emit(idx, slot, l, s, up);
      }
    } else {
      // part of a tile: leave it in the workspace; the block that brings the last part adds them.
      const int tile_u0 = this_tile * p.chunks, tile_u1 = tile_u0 + p.chunks;
      const int big = p.extra * (p.share + 1);   // units held by the blocks that take share + 1
      auto block_of = [&](int u) { return u < big ? u / (p.share + 1) : p.extra + (u - big) / p.share; };
      auto begin_of = [&](int b) { return b * p.share + min(b, p.extra); };
      const int b_lo = block_of(tile_u0), b_hi = block_of(tile_u1 - 1);
      float* mine = p.partials + ((size_t)me * 2 + (range_begin >= tile_u0 ? 0 : 1)) * SMALL_SLOT_FLOATS;
      for (int idx = threadIdx.x; idx < SLOTS * 32; idx += SMALL_WARPS * 32) {
        const int l = idx & 31, slot = idx >> 5;
        float s = 0.0f;
#pragma unroll
        for (int wi = 0; wi < SMALL_WARPS; ++wi) s += red[wi][slot][l];
        __stcg(mine + idx, s);
      }
      __threadfence();
      __syncthreads();
      if (threadIdx.x == 0) is_last = atomicAdd(p.counters + this_tile, 1) == b_hi - b_lo;
      __syncthreads();
      stored = is_last != 0;
      if (is_last) {
        __threadfence();
        for (int idx = threadIdx.x; idx < OUT_SLOTS * 32; idx += SMALL_WARPS * 32) {
          const int l = idx & 31, slot = first_slot(idx);
          float s = 0.0f, up = 0.0f;
          for (int q = b_lo; q <= b_hi; ++q) {
            const float* theirs = p.partials + ((size_t)q * 2 + (begin_of(q) >= tile_u0 ? 0 : 1)) * SMALL_SLOT_FLOATS;
            s += __ldcg(theirs + slot * 32 + l);
            if (PAIRED) up += __ldcg(theirs + (slot + SECOND) * 32 + l);
          }
          emit(idx, slot, l, s, up);
        }
        if (threadIdx.x == 0) p.counters[this_tile] = 0;  // ready for the next launch
      }
    }
    if (EPI == EPI_RESIDUAL && stored) {
      // the tile's sum of squares per activation row: its 16 columns in one fixed order
      __syncthreads();
      if (threadIdx.x < p.M) {
        const int m = threadIdx.x, j = m >> 3, t4 = (m & 7) >> 1, odd = m & 1;
        float q = 0.0f;
#pragma unroll
        for (int half = 0; half < 2; ++half)
#pragma unroll
          for (int g8 = 0; g8 < 8; ++g8) q += squares[(j * 4 + half * 2 + odd) * 32 + g8 * 4 + t4];
        p.sumsq_out[this_tile * 32 + m] = q;
      }
    }
    __syncthreads();  // `red`, `is_last` and `squares` are written again in the next round
  }
}

int sm_count() {
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

template <int MT, int RT, int EPI>
int launch_small(SmallParams p, int chained, cudaStream_t stream) {
  // One block per tile is the cheapest arrangement (no tile is shared between blocks), but with a
  // few waves of blocks, two to an SM, the last wave can be nearly empty. Then, and only then,
  // the work is cut into one even range per place instead, at the price of some shared tiles.
  // (Even ranges for every size were timed too: slower inside a step for 1.3 waves, level for 27.)
  const long long places = 2 * sm_count() < SMALL_MAX_BLOCKS ? 2 * sm_count() : SMALL_MAX_BLOCKS;
  long long blocks = p.tiles;
  if (p.tiles > 2 * places) {
    const long long waves = (p.tiles + places - 1) / places;
    if (waves * places * 10 > p.tiles * 11) blocks = places;   // more than a tenth of the places would idle
  }
  const long long units = (long long)p.tiles * p.chunks;
  if (units >= (1ll << 31)) return PKV_ERR_LIMIT;
  p.share = (int)(units / blocks);
  p.extra = (int)(units % blocks);
  if constexpr (MT == 1 && RT == 1) {
    // Between two and three blocks per SM, three blocks of fewer registers share an SM, so that
    // all tiles run at once instead of leaving a small second wave (the fused projection of an
    // 8-billion-parameter model: 384 tiles on 148 SMs).
    if (blocks == p.tiles && p.tiles > places && p.tiles <= 3 * sm_count())
      return pkv::launch_kernel(gemm_small_m_kernel<MT, RT, EPI, 3>, dim3((unsigned)blocks), dim3(SMALL_WARPS * 32), 0,
                                stream, chained != 0, 0, p);
  }
  return pkv::launch_kernel(gemm_small_m_kernel<MT, RT, EPI, 2>, dim3((unsigned)blocks), dim3(SMALL_WARPS * 32), 0, stream,
                            chained != 0, 0, p);
}

template <int EPI>
int dispatch_small(const SmallParams& p, int chained, cudaStream_t stream) {
  constexpr int RT = (EPI == EPI_SILU_MUL) ? 2 : 1;
  if (p.M <= 8) return launch_small<1, RT, EPI>(p, chained, stream);
  if (p.M <= 16) return launch_small<2, RT, EPI>(p, chained, stream);
  if (p.M <= 32) return launch_small<4, RT, EPI>(p, chained, stream);
  return PKV_ERR_LIMIT;
}

}  // namespace

// Largest number of activation rows that `pkv_gemm_small_m` takes with the given epilogue.
PKV_EXPORT int pkv_gemm_small_m_max_rows(int epilogue) { (void)epilogue; return 32; }

// Bytes of the workspace (partial sums and tile counters); it must be zero before its first use
// and is left zero by every launch, so launches on one stream can share it.
PKV_EXPORT long long pkv_gemm_small_m_workspace_bytes() {
  return (long long)SMALL_MAX_BLOCKS * 2 * SMALL_SLOT_FLOATS * sizeof(float) + (long long)SMALL_MAX_TILES * sizeof(int);
}

// out = x . w^T. `x` is [M, K] with row stride `ldx` (elements), `w` [N, K] contiguous, both
// bfloat16. Epilogue 0: bfloat16 out [M, N]; 1: float32 out [M, N]; 2: silu(gate) * up with the
// gate and up rows of `w` interleaved in blocks of 128 (N a multiple of 256), bfloat16 out
// [M, n_out], |gate| clipped to `clip` inside the exponential. K must be a multiple of 32.
// `chained` non-zero launches as a programmatic dependent of the kernel before it on the stream:
// the first weights are requested before that kernel has finished, the activations after.
//
// Epilogue 3 (residual): hidden [M, N] (float32) += product, in place;
// out (bfloat16 [M, N]) = hidden * norm_weight; sumsq_out [ceil(N/16)][32] (float32) receives, per
// 16-column tile and row, the sum of squares of the new stream. A later call that is given that
// array as `sumsq_in` (with `sumsq_parts` = ceil(N/16), `width` = N and `norm_eps`) and `out` as
// its `x` scales its result rows by 1 / sqrt(sum / width + eps): together the residual add, the
// RMS norm and the next product in two launches instead of three.
//
// Epilogue 4 (rotary + cache): `w` is a fused query/key/value projection of n_heads + 2 n_kv heads
// of head_dim (a multiple of 16) columns. Queries and keys are rotated by `positions[row]` with
// the tables cos_t, sin_t [positions][head_dim / 2] (half-split pairs; null tables: no rotation);
// `out` [M, N] receives the queries (its key and value columns are left unwritten); keys and
// values go to the pools [pages, n_kv, page_size, head_dim] at `slots[row]` (null or negative:
// not stored); `num_slots` = pages x page_size and `max_pos` = rows of the tables bound them, and a
// value outside is recorded in `status` (may be null) instead of being used.
PKV_EXPORT int pkv_gemm_small_m(const void* x, const void* w, void* out, int M, int N, int K, int ldx, int epilogue,
                                int n_out, float clip, int chained, void* workspace, long long workspace_bytes,
                                float* hidden, const float* norm_weight, float* sumsq_out, const float* sumsq_in,
                                int sumsq_parts, int width, float norm_eps, const int* positions, const float* cos_t,
                                const float* sin_t, void* k_pool, void* v_pool, const int* slots, int n_heads, int n_kv,
                                int head_dim, int page_size, int num_slots, int max_pos, int* status, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0) return PKV_ERR_SIZE;
  if (K % SMALL_CHUNK != 0 || ldx % 8 != 0) return PKV_ERR_SIZE;
  if (M > pkv_gemm_small_m_max_rows(epilogue)) return PKV_ERR_LIMIT;
  if (((uintptr_t)x | (uintptr_t)w | (uintptr_t)workspace) & 15) return PKV_ERR_ALIGN;
  if (!workspace || workspace_bytes < pkv_gemm_small_m_workspace_bytes()) return PKV_ERR_SIZE;
  SmallParams p;
  p.x = static_cast<const bf16*>(x);
  p.w = static_cast<const bf16*>(w);
  p.out = out;
  p.partials = static_cast<float*>(workspace);
  p.counters = reinterpret_cast<int*>(static_cast<uint8_t*>(workspace) + (size_t)SMALL_MAX_BLOCKS * 2 * SMALL_SLOT_FLOATS * sizeof(float));
  p.M = M; p.N = N; p.K = K; p.ldx = ldx; p.clip = clip;
  p.hidden = hidden; p.norm_weight = norm_weight; p.sumsq_out = sumsq_out;
  p.sumsq_in = sumsq_in; p.sumsq_parts = sumsq_parts; p.norm_eps = norm_eps; p.inv_width = width > 0 ? 1.0f / (float)width : 0.0f;
  if (sumsq_in && (sumsq_parts <= 0 || width <= 0)) return PKV_ERR_SIZE;
  p.positions = positions; p.cos_t = cos_t; p.sin_t = sin_t; p.k_pool = static_cast<bf16*>(k_pool);
  p.v_pool = static_cast<bf16*>(v_pool); p.slots = slots; p.n_heads = n_heads; p.n_kv = n_kv; p.head_dim = head_dim;
  p.page_size = page_size; p.num_slots = num_slots; p.max_pos = max_pos; p.status = status;
  p.chunks = K / SMALL_CHUNK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (epilogue) {
    case EPI_BF16:
    case EPI_F32:
      p.tiles = (N + 15) / 16; p.ld_out = N; p.n_out = N;
      if (p.tiles > SMALL_MAX_TILES) return PKV_ERR_LIMIT;
      return epilogue == EPI_BF16 ? dispatch_small<EPI_BF16>(p, chained, s) : dispatch_small<EPI_F32>(p, chained, s);
    case EPI_ROPE_KV:
      if (head_dim <= 0 || head_dim % 16 != 0 || n_heads <= 0 || n_kv <= 0 || N != (n_heads + 2 * n_kv) * head_dim)
        return PKV_ERR_SIZE;
      if (!positions || (cos_t != nullptr) != (sin_t != nullptr) || page_size <= 0) return PKV_ERR_SIZE;
      if (slots && (!k_pool || !v_pool || num_slots <= 0)) return PKV_ERR_SIZE;
      if (cos_t && max_pos <= 0) return PKV_ERR_SIZE;
      p.tiles = N / 16; p.ld_out = N; p.n_out = N;
      if (p.tiles > SMALL_MAX_TILES) return PKV_ERR_LIMIT;
      return dispatch_small<EPI_ROPE_KV>(p, chained, s);
    case EPI_RESIDUAL:
      if (!hidden || !norm_weight || !sumsq_out) return PKV_ERR_SIZE;
      p.tiles = (N + 15) / 16; p.ld_out = N; p.n_out = N;
      if (p.tiles > SMALL_MAX_TILES) return PKV_ERR_LIMIT;
      return dispatch_small<EPI_RESIDUAL>(p, chained, s);
    case EPI_SILU_MUL:
      if (N % 256 != 0 || n_out <= 0 || n_out > N / 2) return PKV_ERR_SIZE;
      p.tiles = (N / 256) * 8; p.ld_out = n_out; p.n_out = n_out;
      if (p.tiles > SMALL_MAX_TILES) return PKV_ERR_LIMIT;
      return dispatch_small<EPI_SILU_MUL>(p, chained, s);
    default: return PKV_ERR_SIZE;
  }
}
