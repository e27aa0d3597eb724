// What the decode attention kernels share: the fragment helpers, a warp's running softmax state
// and the step that folds 16 keys of a 64-key stage into it.
//
// A stage holds 64 keys and 64 values of one key/value head as TMA left them, the keys first, then
// the values; rows of 128 bytes whose 16-byte chunks are swizzled by the row number (128-byte
// swizzle). Head size 64 (one 64-column panel): 64 rows, one copy per page. Head size 128 (two
// panels): groups of 8 rows, each group panel after panel (8 rows of panel 0, then of panel 1), so
// that one copy brings a whole page (see make_panel_group_map); half as many copies per tile as
// one per page and panel. Consumer warp w takes rows 16 w .. 16 w + 15.
#pragma once

#include "tcgen05.cuh"

namespace pkv {

constexpr int DT_BN = 64;          // keys per stage
constexpr int DT_ROWS = 16;        // rows of an entry per key/value head

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}


// One warp's online-softmax state over the keys it has seen: the MMA row tile's rows g and g + 8
// (maximum, sum, accumulator fragments), in the base-2 domain.
template <int HD>
struct DecodeState {
  float m_a, m_b, l_a, l_b;
  float o[HD / 8][4];
  __device__ __forceinline__ void reset() {
    m_a = m_b = -INFINITY;
    l_a = l_b = 0.0f;
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
  }
};

// Folds keys wbase .. wbase + 15 (rows 16 warp .. of the stage at `stage_smem`) into `st`:
// scores = q.k * scale, keys outside [key_lo, key_hi), after a row's query position or before its
// window masked, shift = new maximum if finite else 0 (the reference's online softmax,
// src/paged_kv_serving/engine/attention.py:100-116).
template <int HD>
__device__ __forceinline__ void decode_tile(uint8_t* stage_smem, int warp, int lane, const uint32_t (&qa)[HD / 16][4],
                                            DecodeState<HD>& st, int wbase, int key_lo, int key_hi, int qpos_a,
                                            int qpos_b, int window, float scale_log2) {
  constexpr int PANELS = HD / 64;
  constexpr uint32_t PANEL_BYTES = DT_BN * 128;
  constexpr uint32_t HALF_BYTES = PANELS * PANEL_BYTES;
  constexpr int KSTEPS = HD / 16;
  constexpr int DTILES = HD / 8;
  // byte offset of 16-byte chunk `chunk` (unswizzled number, 8 per panel) of row `row` in the keys or values
  auto chunk_at = [](int row, int chunk, int swizzled) -> uint32_t {
    const uint32_t in_row = (uint32_t)((swizzled ? ((chunk & 7) ^ (row & 7)) : (chunk & 7)) << 4);
    if (PANELS == 1) return (uint32_t)row * 128 + in_row;
    return (uint32_t)(row >> 3) * (PANELS * 1024) + (uint32_t)(chunk >> 3) * 1024 + (uint32_t)(row & 7) * 128 + in_row;
  };
  const int t4 = lane & 3;
  const uint32_t k_base = smem_addr(stage_smem);
  const uint32_t v_base = k_base + HALF_BYTES;
  float (&o)[DTILES][4] = st.o;
  float &m_a = st.m_a, &m_b = st.m_b, &l_a = st.l_a, &l_b = st.l_b;
  if (wbase < key_hi && wbase + 15 >= key_lo) {
    if (wbase + 16 > key_hi) {
      // slots of the last page past the last key may hold anything (0 x NaN = NaN): clear the
      // value rows this warp will read
      for (int idx = lane; idx < 16 * PANELS * 8; idx += 32) {
        const int r = idx / (PANELS * 8), c = idx - r * (PANELS * 8);
        if (wbase + r >= key_hi)
          *reinterpret_cast<uint4*>(stage_smem + HALF_BYTES + chunk_at(warp * 16 + r, c, 0)) = make_uint4(0u, 0u, 0u, 0u);
      }
      __syncwarp();
    }
    float sc[2][4] = {{0.0f, 0.0f, 0.0f, 0.0f}, {0.0f, 0.0f, 0.0f, 0.0f}};
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk) {
      // keys as the B operand: rows are keys, 16-byte chunks swizzled by the row number
      const int krow = warp * 16 + (lane & 7) + 8 * (lane >> 4);
      const int chunk = kk * 2 + ((lane >> 3) & 1);
      uint32_t b[4];
      ldsm_x4(b, k_base + chunk_at(krow, chunk, 1));
      mma16816(sc[0], qa[kk], b[0], b[1]);
      mma16816(sc[1], qa[kk], b[2], b[3]);
    }
    float tmax_a = -INFINITY, tmax_b = -INFINITY;
#pragma unroll
    for (int jj = 0; jj < 2; ++jj) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int kpos = wbase + jj * 8 + 2 * t4 + (e & 1);
        const int qpos = (e < 2) ? qpos_a : qpos_b;
        const bool visible = kpos <= qpos && (window == 0 || kpos > qpos - window);
        const float v = visible ? sc[jj][e] * scale_log2 : -INFINITY;
        sc[jj][e] = v;
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
    for (int jj = 0; jj < 2; ++jj) {
      sc[jj][0] = exp2f(sc[jj][0] - shift_a); sc[jj][1] = exp2f(sc[jj][1] - shift_a);
      sc[jj][2] = exp2f(sc[jj][2] - shift_b); sc[jj][3] = exp2f(sc[jj][3] - shift_b);
      sum_a += sc[jj][0] + sc[jj][1];
      sum_b += sc[jj][2] + sc[jj][3];
    }
    l_a = l_a * resc_a + sum_a;
    l_b = l_b * resc_b + sum_b;
    uint32_t a[4];
    a[0] = pack2(sc[0][0], sc[0][1]); a[1] = pack2(sc[0][2], sc[0][3]);
    a[2] = pack2(sc[1][0], sc[1][1]); a[3] = pack2(sc[1][2], sc[1][3]);
#pragma unroll
    for (int dd = 0; dd < DTILES / 2; ++dd) {
      // values as the B operand (transposed load): rows are keys, columns dims
      const int vrow = warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1);
      const int chunk = dd * 2 + (lane >> 4);
      uint32_t b[4];
      ldsm_x4_trans(b, v_base + chunk_at(vrow, chunk, 1));
      o[2 * dd][0] *= resc_a; o[2 * dd][1] *= resc_a; o[2 * dd][2] *= resc_b; o[2 * dd][3] *= resc_b;
      o[2 * dd + 1][0] *= resc_a; o[2 * dd + 1][1] *= resc_a; o[2 * dd + 1][2] *= resc_b; o[2 * dd + 1][3] *= resc_b;
      mma16816(o[2 * dd], a, b[0], b[1]);
      mma16816(o[2 * dd + 1], a, b[2], b[3]);
    }
  }
}

// Tensor maps over the page pools, one per (pool, size), copied to the caller (a later lookup may
// take a table entry's place): [rows = pages x kv heads x page size,
// head size], boxes of one page: of its one 64-column panel (head size 64) or of both, group of 8
// rows by group (head size 128). Kept for the life of the library, since a captured graph holds
// them by value and a step asks for the same few again and again.
struct DecMapKey {
  const void* base;
  long long rows;
  int hd, box;
  CUtensorMap map;
};

static bool decode_pool_map(const void* base, long long rows, int hd, int box_rows, CUtensorMap* out) {
  static DecMapKey cache[512];
  static int used = 0;
  for (int i = 0; i < used; ++i)
    if (cache[i].base == base && cache[i].rows == rows && cache[i].hd == hd && cache[i].box == box_rows) {
      *out = cache[i].map;
      return true;
    }
  static int victim = 0;              // a full table gives up its entries in turn
  DecMapKey& slot = cache[used < 512 ? used : victim];
  const int rc = hd == 128 ? make_panel_group_map(&slot.map, base, rows, 2, box_rows)
                           : make_tile_map(&slot.map, base, rows, hd, hd, box_rows);
  if (rc) {
    slot.base = nullptr;
    return false;
  }
  slot.base = base; slot.rows = rows; slot.hd = hd; slot.box = box_rows;
  if (used < 512) ++used;
  else victim = (victim + 1) % 512;
  *out = slot.map;
  return true;
}

}  // namespace pkv
