// Small-batch (decode) path of the WxA16 layer: streaming LUT-dequant matrix products over PACKED indices.
//
// At a few rows per expert the layer is bound by the packed-weight stream, not by arithmetic
// (the reference's small-batch tile class: turboquant_utils/triton_kernels.py:475-510).  Here one launch covers the
// tiles of ALL bit pools; a CTA owns (one tile of <= 32 routed rows) x (128 output columns of gate AND up, or 256
// output columns of down) and walks the 128-wide groups of K:
//   - every thread pulls its weight rows' packed codes of the NEXT group straight from global memory into registers
//     (8 rows of 16*bit consecutive bytes per warp instruction) while the current group is computed;
//   - codes become fp16 codewords in registers: 1- and 2-bit codes by bit spreading + byte permutes against a
//     two-register table, 8-bit uniform codes arithmetically, 4-bit codes through a bank-per-lane shared table;
//   - the weights are the M operand of mma.sync.m16n8k16 (16 weight rows x 8 routed rows per instruction), so a tile
//     of 1..32 routed rows costs 1..4 instructions per 16 weight rows and k-step instead of a padded 128-row tile.
//     A thread's 32 consecutive codes of a row feed 8 k-steps directly: the k order inside a group is permuted the
//     same way for the activation operand (8-byte shared-memory loads), which a dot product does not notice;
//   - per group: total += acc * norm[group, weight row] in fp32 (triton_kernels.py:1430-1473 does it in fp16);
//   - gate_up CTAs finish with SiLU(gate)*up in registers (quantization/wxa16/bit_partitioned_moe.py:925-931).
// The activation tiles (<= 32 rows x 128 fp16 per group) are staged in shared memory with cp.async, two groups deep.
#include "common.cuh"

namespace {

constexpr int kG = DMOQ_GROUP;
constexpr int kThreads = 256;            // 8 warps; warp w owns weight row tiles 2w and 2w+1 of the CTA's 16
constexpr int kRowsMax = 32;             // routed rows per tile (four 8-row MMA column blocks)
constexpr int kXPitch = 272;             // bytes per staged activation row: 128 fp16 + 16 (bank spread)

struct DecPool {
  const uint8_t* idx;      // group-first packed indices (G, N, 16*bit)
  const uint16_t* norm;    // (G, N) fp16, 1/sqrt(128) folded in
  const uint16_t* lut;     // fp16 codebook
  const uint16_t* a_tab;   // gate_up: this pool's rotated activations (rows, hidden) fp16
  int bit, inter, n_members, identity;
};

struct DecArgs {
  DecPool pool[DMOQ_MAX_POOLS];
  int n_pools;
  const DmoqTile* tiles;
  const int32_t* n_tiles;   // [p] tiles of pool p, [8+p] its first tile
  const int32_t* a_row;     // gate_up: table row of each routed row
  const uint16_t* a_rot;    // down: rotated SiLU outputs (routed rows, a_stride) fp16
  int a_stride, hidden, is_down;
  uint16_t* out;            // gate_up: act (routed rows, out_stride) fp16; down: (routed rows, hidden) fp16
  int out_stride;
};

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
  return d;
}
__device__ __forceinline__ void mma_f16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Eight codes, one per 4-bit field of `w`, -> eight fp16 codewords of a table of at most four entries held in two
// registers (entry c = bytes 2c, 2c+1).
__device__ __forceinline__ uint4 expand8_f16(uint32_t w, uint32_t lut0, uint32_t lut1) {
  const uint32_t sl = (w & 0x0F0F0F0Fu) * 34u + 0x10101010u;          // selector bytes of codes 0, 2, 4, 6
  const uint32_t sh = ((w >> 4) & 0x0F0F0F0Fu) * 34u + 0x10101010u;   // ... of codes 1, 3, 5, 7
  uint32_t o[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) o[j] = prmt(lut0, lut1, prmt(sl, sh, (uint32_t)(j | ((4 + j) << 4))));
  return make_uint4(o[0], o[1], o[2], o[3]);
}
// eight 2-bit codes in the low 16 bits -> eight 4-bit fields
__device__ __forceinline__ uint32_t spread2(uint32_t x) {
  x = (x | (x << 8)) & 0x00FF00FFu;
  x = (x | (x << 4)) & 0x0F0F0F0Fu;
  return (x | (x << 2)) & 0x33333333u;
}
// eight 1-bit codes in the low 8 bits -> eight 4-bit fields
__device__ __forceinline__ uint32_t spread1(uint32_t x) {
  x = (x | (x << 12)) & 0x000F000Fu;
  x = (x | (x << 6)) & 0x03030303u;
  return (x | (x << 3)) & 0x11111111u;
}

// The 32 codes a thread holds for one weight row and one group -> 32 fp16 codewords as 16 half2 registers.
template <int BIT>
struct Raw {
  uint32_t w[BIT];   // 32 codes = 4*BIT bytes
};
template <int BIT>
__device__ __forceinline__ Raw<BIT> load_raw(const uint8_t* p) {
  Raw<BIT> r;
  if (BIT == 1) r.w[0] = *reinterpret_cast<const uint32_t*>(p);
  else if (BIT == 2) { const uint2 v = *reinterpret_cast<const uint2*>(p); r.w[0] = v.x; r.w[1] = v.y; }
  else if (BIT == 4) { const uint4 v = *reinterpret_cast<const uint4*>(p); r.w[0] = v.x; r.w[1] = v.y; r.w[2] = v.z; r.w[3] = v.w; }
  else {
    const uint4 v0 = reinterpret_cast<const uint4*>(p)[0], v1 = reinterpret_cast<const uint4*>(p)[1];
    r.w[0] = v0.x; r.w[1] = v0.y; r.w[2] = v0.z; r.w[3] = v0.w; r.w[4] = v1.x; r.w[5] = v1.y; r.w[6] = v1.z; r.w[7] = v1.w;
  }
  return r;
}
template <int BIT>
__device__ __forceinline__ void dequant32(const Raw<BIT>& r, uint32_t (&h)[16], uint32_t lut0, uint32_t lut1, const uint32_t* s_lut,
                                          uint32_t step2) {
  if (BIT == 1 || BIT == 2) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {   // eight codes per step
      uint32_t fields;
      if (BIT == 1) fields = spread1((r.w[0] >> (8 * q)) & 0xFFu);
      else fields = spread2((r.w[q >> 1] >> (16 * (q & 1))) & 0xFFFFu);
      const uint4 v = expand8_f16(fields, lut0, lut1);
      h[4 * q] = v.x; h[4 * q + 1] = v.y; h[4 * q + 2] = v.z; h[4 * q + 3] = v.w;
    }
  } else if (BIT == 4) {            // one table word per code: lane-private bank, entry c at s_lut[c*32 + lane]
#pragma unroll
    for (int q = 0; q < 16; ++q) {
      const uint32_t two = (r.w[q >> 2] >> (8 * (q & 3))) & 0xFFu;
      h[q] = (s_lut[(two & 15u) * 32] & 0xFFFFu) | (s_lut[(two >> 4) * 32] << 16);
    }
  } else {                          // 8-bit uniform codebook: codeword = (index - 128) * step, exact in fp16 arithmetic
#pragma unroll
    for (int q = 0; q < 16; ++q) {
      const uint32_t wv = r.w[q >> 1];
      // bytes b0, b1 -> fp16 pair (1024 + b0, 1024 + b1): 0x6400 | b
      const uint32_t pair = prmt(wv, 0x64646464u, (q & 1) ? 0x4342u : 0x4140u);
      const __half2 v = __hmul2(__hsub2(*reinterpret_cast<const __half2*>(&pair), __float2half2_rn(1152.0f)),
                                *reinterpret_cast<const __half2*>(&step2));
      h[q] = *reinterpret_cast<const uint32_t*>(&v);
    }
  }
}

struct TileCtx {
  DmoqTile tile;
  int n_tb;   // 8-row column blocks in use
};

// One CTA's work for a pool of bit width BIT.
template <int BIT>
__device__ void run_tile(const DecArgs& a, const DecPool& P, const TileCtx& tc, int jb, uint8_t* s_x, uint32_t* s_lut4) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int t4 = lane & 3, rl = lane >> 2;
  const int G = a.is_down ? P.inter / kG : a.hidden / kG;
  const int N = a.is_down ? a.hidden : P.n_members * 2 * P.inter;
  const int gg0 = a.is_down ? tc.tile.rank * G : 0;
  // weight rows of this thread: tile u (0: gate / first 128 columns, 1: up / second 128), rows rl and rl+8
  int n_row[2];
  if (a.is_down) {
    n_row[0] = jb * 256 + (2 * warp) * 16 + rl;
    n_row[1] = jb * 256 + (2 * warp + 1) * 16 + rl;
  } else {
    n_row[0] = tc.tile.rank * 2 * P.inter + jb * 128 + warp * 16 + rl;
    n_row[1] = n_row[0] + P.inter;
  }
  uint32_t lut0 = 0, lut1 = 0, step2 = 0;
  if (BIT <= 2) {
    for (int i = 0; i < (1 << BIT); ++i) {
      const uint32_t e = P.lut[i];
      if (i < 2) lut0 |= e << (16 * i); else lut1 |= e << (16 * (i - 2));
    }
  } else if (BIT == 8) {
    step2 = (uint32_t)P.lut[129] * 0x10001u;
  }
  const uint32_t* my_lut4 = s_lut4 + lane;
  if (BIT == 4) {
    __syncthreads();   // the previous user of the table (none within a CTA today) is done
    for (int i = tid; i < 16 * 32; i += kThreads) s_lut4[i] = P.lut[i >> 5];
  }

  // ---- activation tile staging: rows x 128 fp16 of group g -> s_x[buf]
  const uint16_t* a_base = a.is_down ? a.a_rot : P.a_tab;
  const int a_pitch = a.is_down ? a.a_stride : a.hidden;
  auto stage = [&](int g, int buf) {
    for (int c = tid; c < kRowsMax * 16; c += kThreads) {
      const int r = c >> 4, ch = c & 15;
      const bool ok = r < tc.tile.rows;
      const int src = ok ? (a.is_down ? tc.tile.row0 + r : a.a_row[tc.tile.row0 + r]) : 0;
      cp_async16_zfill(s_x + buf * (kRowsMax * kXPitch) + r * kXPitch + ch * 16,
                       a_base + (size_t)src * a_pitch + g * kG + ch * 8, ok);
    }
    cp_async_commit();
  };
  auto idx_ptr = [&](int g, int u, int hi) {
    return P.idx + ((size_t)(gg0 + g) * N + n_row[u] + 8 * hi) * (16 * BIT) + t4 * (4 * BIT);
  };

  float total[2][4][4];
#pragma unroll
  for (int u = 0; u < 2; ++u)
#pragma unroll
    for (int b = 0; b < 4; ++b)
#pragma unroll
      for (int q = 0; q < 4; ++q) total[u][b][q] = 0.f;

  // Codes and norms of the NEXT group travel in registers while the current group is computed (8-bit codes are 32
  // bytes per row: those are loaded where they are used, the register file has no room for two groups of them).
  constexpr bool kAhead = BIT < 8;
  Raw<BIT> nxt[2][2];
  uint16_t nrm_n[2][2];
#pragma unroll
  for (int u = 0; u < 2; ++u)
#pragma unroll
    for (int hi = 0; hi < 2; ++hi) {
      if (kAhead) nxt[u][hi] = load_raw<BIT>(idx_ptr(0, u, hi));
      nrm_n[u][hi] = P.norm[(size_t)gg0 * N + n_row[u] + 8 * hi];
    }
  stage(0, 0);

  for (int g = 0; g < G; ++g) {
    Raw<BIT> cur[2][2];
    float nrm[2][2];
#pragma unroll
    for (int u = 0; u < 2; ++u)
#pragma unroll
      for (int hi = 0; hi < 2; ++hi) {
        if (kAhead) cur[u][hi] = nxt[u][hi];
        nrm[u][hi] = __half2float(__ushort_as_half(nrm_n[u][hi]));
      }
    if (g + 1 < G) {   // next group's codes, norms and activation tile are on their way during this group's math
#pragma unroll
      for (int u = 0; u < 2; ++u)
#pragma unroll
        for (int hi = 0; hi < 2; ++hi) {
          if (kAhead) nxt[u][hi] = load_raw<BIT>(idx_ptr(g + 1, u, hi));
          nrm_n[u][hi] = P.norm[(size_t)(gg0 + g + 1) * N + n_row[u] + 8 * hi];
        }
      stage(g + 1, (g + 1) & 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();   // group g's activation tile is complete for every thread
    const uint8_t* xs = s_x + (g & 1) * (kRowsMax * kXPitch);

#pragma unroll
    for (int u = 0; u < 2; ++u) {
      float acc[4][4];
#pragma unroll
      for (int b = 0; b < 4; ++b)
#pragma unroll
        for (int q = 0; q < 4; ++q) acc[b][q] = 0.f;
      uint32_t h_lo[16], h_hi[16];   // codewords of rows rl and rl+8: 32 codes each, this thread's k positions 32*t4 ..
      if (kAhead) {
        dequant32<BIT>(cur[u][0], h_lo, lut0, lut1, my_lut4, step2);
        dequant32<BIT>(cur[u][1], h_hi, lut0, lut1, my_lut4, step2);
      } else {
        dequant32<BIT>(load_raw<BIT>(idx_ptr(g, u, 0)), h_lo, lut0, lut1, my_lut4, step2);
        dequant32<BIT>(load_raw<BIT>(idx_ptr(g, u, 1)), h_hi, lut0, lut1, my_lut4, step2);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {   // k-step j covers this thread's codes 4j..4j+3
        const uint32_t af[4] = {h_lo[2 * j], h_hi[2 * j], h_lo[2 * j + 1], h_hi[2 * j + 1]};
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          if (b < tc.n_tb) {
            const uint2 bf = *reinterpret_cast<const uint2*>(xs + (8 * b + rl) * kXPitch + (32 * t4 + 4 * j) * 2);
            mma_f16(acc[b], af, bf.x, bf.y);
          }
        }
      }
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        total[u][b][0] = fmaf(acc[b][0], nrm[u][0], total[u][b][0]);
        total[u][b][1] = fmaf(acc[b][1], nrm[u][0], total[u][b][1]);
        total[u][b][2] = fmaf(acc[b][2], nrm[u][1], total[u][b][2]);
        total[u][b][3] = fmaf(acc[b][3], nrm[u][1], total[u][b][3]);
      }
    }
    __syncthreads();   // every thread is done with this buffer before group g+2 is staged into it
  }

  // ---- outputs: accumulator element q of block b = weight row rl + 8*(q>>1), routed row 8b + 2*t4 + (q&1)
  __half* out = reinterpret_cast<__half*>(a.out);
#pragma unroll
  for (int b = 0; b < 4; ++b)
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int rr = 8 * b + 2 * t4 + (q & 1);
      if (rr >= tc.tile.rows) continue;
      __half* orow = out + (size_t)(tc.tile.row0 + rr) * a.out_stride;
      if (a.is_down) {
#pragma unroll
        for (int u = 0; u < 2; ++u)
          orow[jb * 256 + (2 * warp + u) * 16 + rl + 8 * (q >> 1)] = __float2half_rn(total[u][b][q]);
      } else {
        const float gate = __half2float(__float2half_rn(total[0][b][q]));
        const float up = __half2float(__float2half_rn(total[1][b][q]));
        const float sg = __half2float(__float2half_rn(__fdividef(gate, 1.0f + __expf(-gate))));
        orow[jb * 128 + warp * 16 + rl + 8 * (q >> 1)] = __float2half_rn(__fmul_rn(sg, up));
      }
    }
}

__global__ void __launch_bounds__(kThreads, 2) decode_mm_kernel(DecArgs a) {
  extern __shared__ __align__(16) uint8_t smem[];
  uint8_t* s_x = smem;                                                        // 2 x 32 rows x kXPitch
  uint32_t* s_lut4 = reinterpret_cast<uint32_t*>(smem + 2 * kRowsMax * kXPitch);   // 16 entries x 32 lanes
  const int t = blockIdx.x, jb = blockIdx.y;
  int p = -1;
  for (int q = 0; q < a.n_pools; ++q) {
    const int base = a.n_tiles[DMOQ_MAX_POOLS + q], n = a.n_tiles[q];
    if (t >= base && t < base + n) p = q;
  }
  if (p < 0) return;
  const DecPool& P = a.pool[p];
  if (!a.is_down && jb >= P.inter / 128) return;
  TileCtx tc;
  tc.tile = a.tiles[t];
  if (tc.tile.rows <= 0) return;
  tc.n_tb = (min(tc.tile.rows, kRowsMax) + 7) / 8;
  switch (P.bit) {
    case 1: run_tile<1>(a, P, tc, jb, s_x, s_lut4); break;
    case 2: run_tile<2>(a, P, tc, jb, s_x, s_lut4); break;
    case 4: run_tile<4>(a, P, tc, jb, s_x, s_lut4); break;
    default: run_tile<8>(a, P, tc, jb, s_x, s_lut4); break;
  }
}

int launch_decode(const dmoq_route_t* route, const dmoq_pool_t* pools, int n_pools, int hidden, int is_down,
                  const uint16_t* a_rot, int a_stride, uint16_t* out, int out_stride, cudaStream_t s) {
  DecArgs a{};
  int max_blocks = 0;
  for (int i = 0; i < n_pools; ++i) {
    const dmoq_pool_t& p = pools[i];
    if (p.mode != DMOQ_A16) return DMOQ_EINVAL;
    if (p.inter <= 0 || p.inter % 128 || hidden % 256) return DMOQ_EINVAL;
    if (p.bit == 8 && !p.identity_lut) return DMOQ_EINVAL;   // general 256-entry tables take the tile kernels
    DecPool& d = a.pool[i];
    d.idx = is_down ? p.dn_idx : p.gu_idx;
    d.norm = is_down ? p.dn_norm : p.gu_norm;
    d.lut = static_cast<const uint16_t*>(is_down ? p.dn_lut : p.gu_lut);
    d.a_tab = static_cast<const uint16_t*>(p.act_codes);
    d.bit = p.bit;
    d.inter = p.inter;
    d.n_members = p.n_members;
    d.identity = p.identity_lut;
    if (!d.idx || !d.norm || !d.lut || (!is_down && !d.a_tab)) return DMOQ_EINVAL;
    const int blocks = is_down ? hidden / 256 : p.inter / 128;
    if (blocks > max_blocks) max_blocks = blocks;
  }
  a.n_pools = n_pools;
  a.tiles = reinterpret_cast<const DmoqTile*>(route->tiles);
  a.n_tiles = route->n_tiles;
  a.a_row = route->a_row;
  a.a_rot = a_rot;
  a.a_stride = a_stride;
  a.hidden = hidden;
  a.is_down = is_down;
  a.out = out;
  a.out_stride = out_stride;
  const size_t smem = 2 * kRowsMax * kXPitch + 16 * 32 * sizeof(uint32_t);
  decode_mm_kernel<<<dim3(route->tile_cap, max_blocks), kThreads, smem, s>>>(a);
  return dmoq_launch_status();
}

}  // namespace

// ------------------------------------------------------------------------------------------------ rotations
// Group rotations of the small-batch path, all pools in one launch.  WxA16 rotated activations are plain fp16
// roundings of fp32-accumulated products (turboquant_utils/rotation.py:176; a floating-point stage, no code
// exactness involved), so a small MMA block does it: 32 rows x 128 columns of one group per CTA, the rotation
// matrix read from L2 as the col-major B operand (rot[j][k] is contiguous in k for output column j).
//   gate_up side: rows of x (bf16 or fp16, cast to fp16 first as the reference does) -> every pool's table
//                 (hoisted pools: one row per token; others: the pool's compact rows, sources in pool_src)
//   down side:    rows of the SiLU output of every tile -> a_rot, with the rotation stack of the tile's expert
struct RotPool {
  const uint16_t* rot;     // gate_up: (G_h, 128, 128); down: (n_members * inter/128, 128, 128)
  uint16_t* table;         // gate_up: destination table (rows, hidden)
  int hoisted, cap_rows, inter;
};
struct RotDecArgs {
  RotPool pool[DMOQ_MAX_POOLS];
  int n_pools, is_down, hidden, T;
  const void* x;           // gate_up: (T, hidden)
  int x_is_bf16;
  const int32_t* pool_rows;      // device: rows routed to each pool
  const int32_t* pool_src;       // device: source token of each compact row
  const int32_t* pool_src_base;  // device: first pool_src entry of each pool
  const DmoqTile* tiles;
  const int32_t* n_tiles;
  const uint16_t* act;     // down: (R, act_stride) fp16
  int act_stride;
  uint16_t* a_rot;         // down: (R, a_stride) fp16
  int a_stride;
};

__global__ void __launch_bounds__(128) decode_rotate_kernel(RotDecArgs a) {
  __shared__ __align__(16) uint8_t s_x[kRowsMax * kXPitch];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, t4 = lane & 3, rl = lane >> 2;
  int p, g = blockIdx.y, rows, src_kind;   // src_kind 0: x rows [row0, ..), 1: x rows through pool_src, 2: act rows
  int row0 = 0, src_base = 0;
  const uint16_t* rot;
  uint16_t* dst;
  int dst_pitch, dst_row0, dst_col0;
  if (!a.is_down) {
    p = blockIdx.z;
    const RotPool& P = a.pool[p];
    if (g >= a.hidden / kG) return;
    const int n_rows = P.hoisted ? a.T : min(a.pool_rows[p], P.cap_rows);
    row0 = blockIdx.x * kRowsMax;
    if (row0 >= n_rows) return;
    rows = min(kRowsMax, n_rows - row0);
    src_kind = P.hoisted ? 0 : 1;
    src_base = a.pool_src_base[p];
    rot = P.rot + (size_t)g * kG * kG;
    dst = P.table;
    dst_pitch = a.hidden;
    dst_row0 = row0;
    dst_col0 = g * kG;
  } else {
    const int t = blockIdx.x;
    p = -1;
    for (int q = 0; q < a.n_pools; ++q) {
      const int base = a.n_tiles[DMOQ_MAX_POOLS + q], n = a.n_tiles[q];
      if (t >= base && t < base + n) p = q;
    }
    if (p < 0) return;
    const RotPool& P = a.pool[p];
    const int G = P.inter / kG;
    if (g >= G) return;
    const DmoqTile tile = a.tiles[t];
    if (tile.rows <= 0) return;
    rows = min(tile.rows, kRowsMax);
    row0 = tile.row0;
    src_kind = 2;
    rot = P.rot + (size_t)(tile.rank * G + g) * kG * kG;
    dst = a.a_rot;
    dst_pitch = a.a_stride;
    dst_row0 = row0;
    dst_col0 = g * kG;
  }
  // ---- stage the rows' 128 values of this group as fp16
  for (int c = tid; c < kRowsMax * 16; c += 128) {
    const int r = c >> 4, ch = c & 15;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (r < rows) {
      if (src_kind == 2) {
        v = *reinterpret_cast<const uint4*>(a.act + (size_t)(row0 + r) * a.act_stride + g * kG + ch * 8);
      } else {
        const int src = src_kind == 0 ? row0 + r : a.pool_src[src_base + row0 + r];
        v = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(a.x) + (size_t)src * a.hidden + g * kG + ch * 8);
        if (a.x_is_bf16) {
          uint16_t* u = reinterpret_cast<uint16_t*>(&v);
#pragma unroll
          for (int q = 0; q < 8; ++q) u[q] = __half_as_ushort(__float2half_rn(bf16_bits_to_float(u[q])));
        }
      }
    }
    *reinterpret_cast<uint4*>(s_x + r * kXPitch + ch * 16) = v;
  }
  __syncthreads();
  // ---- warp w: output columns [32w, 32w+32) for both 16-row tiles
  float acc[2][4][4];
#pragma unroll
  for (int m = 0; m < 2; ++m)
#pragma unroll
    for (int n = 0; n < 4; ++n)
#pragma unroll
      for (int q = 0; q < 4; ++q) acc[m][n][q] = 0.f;
#pragma unroll
  for (int ks = 0; ks < 8; ++ks) {
    uint32_t af[2][4];
#pragma unroll
    for (int m = 0; m < 2; ++m) {
      const uint8_t* base = s_x + (16 * m + rl) * kXPitch + (16 * ks + 2 * t4) * 2;
      af[m][0] = *reinterpret_cast<const uint32_t*>(base);
      af[m][1] = *reinterpret_cast<const uint32_t*>(base + 8 * kXPitch);
      af[m][2] = *reinterpret_cast<const uint32_t*>(base + 16);
      af[m][3] = *reinterpret_cast<const uint32_t*>(base + 8 * kXPitch + 16);
    }
#pragma unroll
    for (int n = 0; n < 4; ++n) {
      const uint16_t* col = rot + (size_t)(32 * warp + 8 * n + rl) * kG + 16 * ks + 2 * t4;
      const uint32_t b0 = *reinterpret_cast<const uint32_t*>(col), b1 = *reinterpret_cast<const uint32_t*>(col + 8);
#pragma unroll
      for (int m = 0; m < 2; ++m) mma_f16(acc[m][n], af[m], b0, b1);
    }
  }
#pragma unroll
  for (int m = 0; m < 2; ++m)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int r = 16 * m + rl + 8 * h;
      if (r >= rows) continue;
      uint16_t* orow = dst + (size_t)(dst_row0 + r) * dst_pitch + dst_col0 + 32 * warp + 2 * t4;
#pragma unroll
      for (int n = 0; n < 4; ++n) {
        const __half2 v = __floats2half2_rn(acc[m][n][2 * h], acc[m][n][2 * h + 1]);
        *reinterpret_cast<__half2*>(orow + 8 * n) = v;
      }
    }
}

extern "C" int dmoq_moe_decode_rotate(const dmoq_route_t* route, const dmoq_pool_t* pools_host, int32_t n_pools,
                                      int32_t hidden, const void* x, int32_t x_is_bf16, void* stream) {
  DMOQ_CHECK_ARG(route && pools_host && x && route->pool_rows && route->pool_src && route->pool_src_base);
  DMOQ_CHECK_ARG(n_pools > 0 && n_pools <= DMOQ_MAX_POOLS && hidden > 0 && hidden % kG == 0 && route->T > 0);
  RotDecArgs a{};
  int max_rows = 0;
  for (int i = 0; i < n_pools; ++i) {
    const dmoq_pool_t& p = pools_host[i];
    DMOQ_CHECK_ARG(p.mode == DMOQ_A16 && p.gu_rot && p.act_codes);
    a.pool[i] = RotPool{p.gu_rot, static_cast<uint16_t*>(p.act_codes), p.hoisted, p.act_cap_rows, p.inter};
    const int rows = p.hoisted ? route->T : p.act_cap_rows;
    if (rows > max_rows) max_rows = rows;
  }
  a.n_pools = n_pools;
  a.is_down = 0;
  a.hidden = hidden;
  a.T = route->T;
  a.x = x;
  a.x_is_bf16 = x_is_bf16;
  a.pool_rows = route->pool_rows;
  a.pool_src = route->pool_src;
  a.pool_src_base = route->pool_src_base;
  decode_rotate_kernel<<<dim3(dmoq_ceil_div(max_rows, kRowsMax), hidden / kG, n_pools), 128, 0, static_cast<cudaStream_t>(stream)>>>(a);
  return dmoq_launch_status();
}

extern "C" int dmoq_moe_decode_rotate_down(const dmoq_route_t* route, const dmoq_pool_t* pools_host, int32_t n_pools,
                                           const uint16_t* act, int32_t act_stride, uint16_t* a_rot, int32_t a_stride,
                                           void* stream) {
  DMOQ_CHECK_ARG(route && pools_host && act && a_rot && route->tiles && route->n_tiles && route->tile_m == kRowsMax);
  DMOQ_CHECK_ARG(n_pools > 0 && n_pools <= DMOQ_MAX_POOLS && act_stride % 8 == 0 && a_stride % 8 == 0);
  RotDecArgs a{};
  int max_g = 0;
  for (int i = 0; i < n_pools; ++i) {
    const dmoq_pool_t& p = pools_host[i];
    DMOQ_CHECK_ARG(p.mode == DMOQ_A16 && p.dn_rot && p.inter > 0 && p.inter % kG == 0);
    a.pool[i] = RotPool{p.dn_rot, nullptr, 0, 0, p.inter};
    if (p.inter / kG > max_g) max_g = p.inter / kG;
  }
  a.n_pools = n_pools;
  a.is_down = 1;
  a.tiles = reinterpret_cast<const DmoqTile*>(route->tiles);
  a.n_tiles = route->n_tiles;
  a.act = act;
  a.act_stride = act_stride;
  a.a_rot = a_rot;
  a.a_stride = a_stride;
  decode_rotate_kernel<<<dim3(route->tile_cap, max_g, 1), 128, 0, static_cast<cudaStream_t>(stream)>>>(a);
  return dmoq_launch_status();
}

extern "C" int dmoq_moe_decode_gateup(const dmoq_route_t* route, const dmoq_pool_t* pools_host, int32_t n_pools,
                                      int32_t hidden, uint16_t* act, int32_t act_stride, void* stream) {
  DMOQ_CHECK_ARG(route && pools_host && act && route->tiles && route->n_tiles && route->a_row);
  DMOQ_CHECK_ARG(n_pools > 0 && n_pools <= DMOQ_MAX_POOLS && route->tile_m == kRowsMax && hidden > 0 && act_stride > 0);
  return launch_decode(route, pools_host, n_pools, hidden, 0, nullptr, 0, act, act_stride, static_cast<cudaStream_t>(stream));
}

extern "C" int dmoq_moe_decode_down(const dmoq_route_t* route, const dmoq_pool_t* pools_host, int32_t n_pools,
                                    int32_t hidden, const uint16_t* a_rot, int32_t a_stride, uint16_t* dn, void* stream) {
  DMOQ_CHECK_ARG(route && pools_host && a_rot && dn && route->tiles && route->n_tiles);
  DMOQ_CHECK_ARG(n_pools > 0 && n_pools <= DMOQ_MAX_POOLS && route->tile_m == kRowsMax && hidden > 0 && a_stride % 8 == 0);
  return launch_decode(route, pools_host, n_pools, hidden, 1, a_rot, a_stride, dn, hidden, static_cast<cudaStream_t>(stream));
}
