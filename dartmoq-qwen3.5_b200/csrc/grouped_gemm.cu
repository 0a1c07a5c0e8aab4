// Grouped LUT-dequant GEMM over a bit pool's tile list (all four activation modes).
//
// A tile is 128 routed rows of one expert x 128 output columns.  Per 128-wide
// quantisation group the CTA gathers the activation codes (cp.async), expands
// the packed codebook indices through a byte-indexed lookup table straight
// into a swizzled shared-memory operand tile, runs warp-level tensor-core MMAs
// (s8 -> s32, e4m3 -> f32, f16 -> f32) and folds  (acc * row_scale) * col_norm
// into an fp32 running total in group order, exactly as the reference kernels do
//   turboquant_utils/triton_kernels.py:1375      (A16)
//   turboquant_utils/triton_kernels_a8.py:825    (A8, int32 per group)
//   turboquant_utils/triton_kernels_fp8.py:532   (FP8)
//   turboquant_utils/triton_kernels_fp4.py:587   (FP4, per-32 e8m0 block scales)
// The gate_up tile interleaves gate and up columns so the SiLU*up epilogue
// (quantization/wxa16/bit_partitioned_moe.py:925-931) happens in registers; the
// down tile applies the fp16 -> bf16 -> x routing-weight chain of :960-966.
#include <cstdlib>

#include "common.cuh"

namespace {

constexpr int kBN = 128, kG = DMOQ_GROUP;
constexpr int kThreads = 512;  // 16 warps; 128-row tiles: 4 x 4 warps of 32 x 32, 32-row tiles: 2 x 8 warps of 16 x 16

struct GemmArgs {
  const DmoqTile* tiles;
  const int32_t* n_tiles;
  const int32_t* expert_rank;
  const int32_t* a_row;         // gather map (gate_up) or null (down: own row)
  const float* row_weight;      // sorted routing weights (EPI_WEIGHTED)
  int pool, is_down, inter, hidden, n_members;
  const uint8_t* idx;
  const uint16_t* norm;
  const void* lut;
  int identity_lut, e0;
  const uint8_t* a_codes;
  const uint8_t* a_scales;
  int a_stride;                 // row pitch (elements) of the activation-code table
  void* out;
  int out_stride;
  int32_t* partials;
};

__device__ __constant__ uint16_t kE2M1Half[16] = {0x0000, 0x3800, 0x3C00, 0x3E00, 0x4000, 0x4200, 0x4400, 0x4600,
                                                  0x8000, 0xB800, 0xBC00, 0xBE00, 0xC000, 0xC200, 0xC400, 0xC600};

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

template <int MODE>
struct Mma;
template <>
struct Mma<DMOQ_A8> {
  using Acc = int32_t;
  __device__ static __forceinline__ void run(int32_t (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
};
template <>
struct Mma<DMOQ_FP8> {
  using Acc = float;
  __device__ static __forceinline__ void run(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
};
struct MmaF16 {
  using Acc = float;
  __device__ static __forceinline__ void run(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
};
template <>
struct Mma<DMOQ_A16> : MmaF16 {};
template <>
struct Mma<DMOQ_FP4> : MmaF16 {};

constexpr int kAStages = 3;   // activation operand tiles in flight (copies are issued two groups ahead)

template <int MODE>
struct Traits {
  static constexpr int ES = (MODE == DMOQ_A8 || MODE == DMOQ_FP8) ? 1 : 2;  // operand element bytes in smem
  static constexpr int SG = (MODE == DMOQ_FP4) ? 32 : 128;                  // K elements per scale block
  static constexpr int ROWB = kG * ES;                                      // smem bytes per operand row
  static constexpr int TILEB = kBN * ROWB;                                  // one weight operand tile
};

// swizzled byte offset of 16-byte chunk `c` of row `r`
template <int ROWB>
__device__ __forceinline__ uint32_t swz(int r, int c) {
  return (uint32_t)(r * ROWB + ((c ^ (r & 7)) << 4));
}

template <int MODE, int BIT, int EPI, int BM>
__global__ void __launch_bounds__(kThreads, 1) grouped_gemm_kernel(GemmArgs a) {
  constexpr int kBM = BM;
  constexpr int WN = (BM == 128) ? 4 : 8;          // warps along the columns
  constexpr int MT = (BM == 128) ? 2 : 1;          // 16-row MMA tiles per warp
  constexpr int NT = (BM == 128) ? 4 : 2;          // 8-column MMA tiles per warp
  constexpr int TILEA = BM * Traits<MODE>::ROWB;   // one activation operand tile
  using T = Traits<MODE>;
  using Acc = typename Mma<MODE>::Acc;
  constexpr int ES = T::ES, ROWB = T::ROWB, TILEB = T::TILEB;
  constexpr int EPB = 8 / BIT;          // elements per packed byte
  constexpr int EB = EPB * ES;          // bytes one packed byte expands to
  constexpr int BPG = 16 * BIT;         // packed bytes per row per group
  constexpr int PB = 4 * BIT;           // packed bytes per thread per group (32 elements)
  constexpr int NBLK = kG / T::SG;      // scale blocks per group
  constexpr int KSTEPS_BLK = T::SG * ES / 32;

  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* s_a = smem;                                   // kAStages x TILEA (activation copies run two groups ahead)
  uint8_t* s_b = smem + kAStages * TILEA;                // 2 x TILEB
  float* s_norm = reinterpret_cast<float*>(smem + kAStages * TILEA + 2 * TILEB);   // 2 x 128
  float* s_rs = s_norm + 2 * kBN;                                    // 2 x 128 x 4
  int32_t* s_arow = reinterpret_cast<int32_t*>(s_rs + 2 * kBM * 4);  // 128
  uint8_t* s_blut = reinterpret_cast<uint8_t*>(s_arow + kBM);        // 256 x EB

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int wm = warp / WN, wn = warp % WN;

  // ---- byte -> expanded elements table
  for (int byte = tid; byte < 256; byte += kThreads) {
#pragma unroll
    for (int j = 0; j < EPB; ++j) {
      const int idx = (byte >> (j * BIT)) & ((1 << BIT) - 1);
      if (ES == 1) {
        uint8_t v;
        if (MODE == DMOQ_A8 && a.identity_lut) v = (uint8_t)(int8_t)(idx - 128);
        else v = reinterpret_cast<const uint8_t*>(a.lut)[idx];
        s_blut[byte * EB + j] = v;
      } else {
        uint16_t v;
        if (MODE == DMOQ_FP4) v = kE2M1Half[reinterpret_cast<const uint8_t*>(a.lut)[idx] & 15];
        else v = reinterpret_cast<const uint16_t*>(a.lut)[idx];
        reinterpret_cast<uint16_t*>(s_blut)[byte * EPB + j] = v;
      }
    }
  }

  // the first four 16-bit codewords in two registers (1- and 2-bit codebooks in the 16-bit operand modes)
  uint32_t lut_r0 = 0, lut_r1 = 0;
  if (ES == 2 && BIT <= 2) {
    uint32_t h[4] = {0, 0, 0, 0};
    for (int i = 0; i < (1 << BIT); ++i)
      h[i] = (MODE == DMOQ_FP4) ? kE2M1Half[reinterpret_cast<const uint8_t*>(a.lut)[i] & 15]
                                : reinterpret_cast<const uint16_t*>(a.lut)[i];
    lut_r0 = h[0] | (h[1] << 16);
    lut_r1 = h[2] | (h[3] << 16);
  }

  const int n_tiles = a.n_tiles[a.pool];
  const DmoqTile* tiles = a.tiles + a.n_tiles[DMOQ_MAX_POOLS + a.pool];
  const int NB = a.is_down ? a.hidden / kBN : a.inter / (kBN / 2);
  const int G = a.is_down ? a.inter / kG : a.hidden / kG;   // groups along K for one member
  const int n_total = a.is_down ? a.hidden : a.n_members * 2 * a.inter;
  const int n_work = n_tiles * NB;

  for (int w = blockIdx.x; w < n_work; w += gridDim.x) {
    const DmoqTile tile = tiles[w / NB];
    const int nb = w % NB;
    const int rank = a.expert_rank[tile.expert];
    const int gg0 = a.is_down ? rank * G : 0;
    // weight row of operand-tile row j
    const int seg0 = a.is_down ? nb * kBN : rank * 2 * a.inter + nb * (kBN / 2);
    const int seg1 = a.is_down ? seg0 : seg0 + a.inter;
    auto wrow = [&](int j) { return a.is_down ? seg0 + j : ((j & 1) ? seg1 : seg0) + (j >> 1); };

    __syncthreads();  // previous tile's staging reads are done; table is visible
    if (tid < kBM) {
      int r = tid < tile.rows ? tile.row0 + tid : -1;
      s_arow[tid] = (r < 0) ? -1 : (a.a_row ? a.a_row[r] : r);
    }
    __syncthreads();

    // per-thread dequant / staging coordinates
    const int bj = tid >> 2, bq = tid & 3;
    const int brow = wrow(bj);

    // Everything a thread fetches from global memory for one group and keeps in registers until the group's
    // operand tile is built: packed weight indices, FP4 activation nibbles, the row scale or column norm it
    // stages.  Two groups are in flight (loaded two steps ahead of their use), so the loads have a whole
    // compute step to land; at small row counts this is what the kernel's time is made of.
    struct GroupRegs {
      uint32_t raw_b[PB / 4 > 0 ? PB / 4 : 1];
      uint4 raw_a4;    // FP4 activation nibbles (32 elements)
      uint32_t sc;     // tid < kBM: activation scale bits of row tid; kBM <= tid < kBM + kBN: norm bits of a column
    };

    auto issue_a = [&](int g, int buf) {   // activation codes: asynchronous copies into the operand tile
      if (MODE != DMOQ_FP4) {
        constexpr int CH = ROWB / 16;  // chunks per row
        for (int c = tid; c < kBM * CH; c += kThreads) {
          const int r = c / CH, ch = c % CH;
          const int ar = s_arow[r];
          const uint8_t* src = a.a_codes + ((size_t)(ar < 0 ? 0 : ar) * a.a_stride + (size_t)g * kG) * ES + ch * 16;
          cp_async16_zfill(s_a + buf * TILEA + swz<ROWB>(r, ch), src, ar >= 0);
        }
      }
      cp_async_commit();
    };

    auto load_group = [&](int g, GroupRegs& w) {
      w.raw_a4 = make_uint4(0, 0, 0, 0);
      if (MODE == DMOQ_FP4) {
        const int ar = bj < kBM ? s_arow[bj] : -1;
        if (ar >= 0) w.raw_a4 = *reinterpret_cast<const uint4*>(a.a_codes + (size_t)ar * (a.a_stride / 2) + g * (kG / 2) + bq * 16);
      }
      // packed weight indices for this thread's 32 elements
      const uint8_t* wp = a.idx + ((size_t)(gg0 + g) * n_total + brow) * BPG + bq * PB;
      if (PB == 4) w.raw_b[0] = *reinterpret_cast<const uint32_t*>(wp);
      else if (PB == 8) { uint2 v = *reinterpret_cast<const uint2*>(wp); w.raw_b[0] = v.x; w.raw_b[1] = v.y; }
      else {
#pragma unroll
        for (int q = 0; q < PB / 16; ++q) {
          uint4 v = *reinterpret_cast<const uint4*>(wp + q * 16);
          w.raw_b[q * 4 + 0] = v.x; w.raw_b[q * 4 + 1] = v.y; w.raw_b[q * 4 + 2] = v.z; w.raw_b[q * 4 + 3] = v.w;
        }
      }
      // scales
      w.sc = 0;
      if (tid < kBM) {
        const int ar = s_arow[tid];
        if (ar >= 0) {
          if (MODE == DMOQ_A8 || MODE == DMOQ_FP8)
            w.sc = reinterpret_cast<const uint16_t*>(a.a_scales)[(size_t)ar * (a.a_stride / kG) + g];
          else if (MODE == DMOQ_FP4)
            w.sc = *reinterpret_cast<const uint32_t*>(a.a_scales + (size_t)ar * (a.a_stride / 32) + g * 4);
        }
      } else if (tid < kBM + kBN) {
        w.sc = reinterpret_cast<const uint16_t*>(a.norm)[(size_t)(gg0 + g) * n_total + wrow(tid - kBM)];
      }
    };

    auto expand_to_smem = [&](int buf, int abuf, const GroupRegs& w) {
      // weights: PB packed bytes -> 32 elements -> 2*ES chunks of 16 bytes
      __align__(16) uint8_t ob[32 * ES];
      if (ES == 2 && BIT <= 2) {
        // 16-bit codewords of a 1- or 2-bit codebook fit two registers: look them up with byte permutes instead
        // of the shared-memory table (at small row counts that table's bank conflicts are what the kernel waits on).
        // Codes of one packed byte -> one code per byte -> selector nibbles (2c, 2c+1) -> two codewords per permute.
        uint32_t* ow = reinterpret_cast<uint32_t*>(ob);
#pragma unroll
        for (int i = 0; i < PB; ++i) {
          const uint32_t B = (w.raw_b[i >> 2] >> (8 * (i & 3))) & 255u;
          if (BIT == 2) {
            const uint32_t t = (B | (B << 6) | (B << 12) | (B << 18)) & 0x03030303u;
            const uint32_t sel = t * 34u + 0x10101010u;
            ow[2 * i + 0] = __byte_perm(lut_r0, lut_r1, sel);
            ow[2 * i + 1] = __byte_perm(lut_r0, lut_r1, sel >> 16);
          } else {
            const uint32_t t0 = (B | (B << 7) | (B << 14) | (B << 21)) & 0x01010101u;
            const uint32_t Bh = B >> 4;
            const uint32_t t1 = (Bh | (Bh << 7) | (Bh << 14) | (Bh << 21)) & 0x01010101u;
            const uint32_t s0 = t0 * 34u + 0x10101010u, s1 = t1 * 34u + 0x10101010u;
            ow[4 * i + 0] = __byte_perm(lut_r0, lut_r1, s0);
            ow[4 * i + 1] = __byte_perm(lut_r0, lut_r1, s0 >> 16);
            ow[4 * i + 2] = __byte_perm(lut_r0, lut_r1, s1);
            ow[4 * i + 3] = __byte_perm(lut_r0, lut_r1, s1 >> 16);
          }
        }
      } else
#pragma unroll
      for (int i = 0; i < PB; ++i) {
        const uint32_t byte = (w.raw_b[i >> 2] >> (8 * (i & 3))) & 255u;
        const uint8_t* e = s_blut + byte * EB;
        if (EB >= 4) {
#pragma unroll
          for (int q = 0; q < EB / 4; ++q)
            reinterpret_cast<uint32_t*>(ob)[i * (EB / 4) + q] = reinterpret_cast<const uint32_t*>(e)[q];
        } else if (EB == 2) {
          reinterpret_cast<uint16_t*>(ob)[i] = *reinterpret_cast<const uint16_t*>(e);
        } else {
          ob[i] = *e;
        }
      }
#pragma unroll
      for (int c = 0; c < 2 * ES; ++c)
        *reinterpret_cast<uint4*>(s_b + buf * TILEB + swz<ROWB>(bj, bq * 2 * ES + c)) = reinterpret_cast<const uint4*>(ob)[c];
      if (MODE == DMOQ_FP4 && bj < kBM) {
        __align__(16) uint16_t oa[32];
        const uint32_t words[4] = {w.raw_a4.x, w.raw_a4.y, w.raw_a4.z, w.raw_a4.w};
#pragma unroll
        for (int i = 0; i < 32; ++i) oa[i] = kE2M1Half[(words[i >> 3] >> (4 * (i & 7))) & 15];
#pragma unroll
        for (int c = 0; c < 4; ++c)
          *reinterpret_cast<uint4*>(s_a + abuf * TILEA + swz<ROWB>(bj, bq * 4 + c)) = reinterpret_cast<const uint4*>(oa)[c];
      }
      if (tid < kBM) {
        const bool live = s_arow[tid] >= 0;
        float* rs = s_rs + (buf * kBM + tid) * 4;
        if (MODE == DMOQ_A8 || MODE == DMOQ_FP8) {
          rs[0] = live ? __half2float(__ushort_as_half((uint16_t)w.sc)) : 0.f;
        } else if (MODE == DMOQ_FP4) {
#pragma unroll
          for (int q = 0; q < 4; ++q)
            rs[q] = live ? ldexpf(1.0f, (int)((w.sc >> (8 * q)) & 255) - 127 + a.e0) : 0.f;
        } else {
          rs[0] = 1.f;
        }
      } else if (tid < kBM + kBN) {
        s_norm[buf * kBN + (tid - kBM)] = __half2float(__ushort_as_half((uint16_t)w.sc));
      }
    };


    float total[MT][NT][4];
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
      for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int q = 0; q < 4; ++q) total[i][j][q] = 0.f;

    GroupRegs w_cur, w_next;   // w_next: the group built during this step; w_ahead (below): the one after
    issue_a(0, 0);
    if (G > 1) issue_a(1, 1); else cp_async_commit();   // one commit group per step keeps the wait counts uniform
    load_group(0, w_cur);
    if (G > 1) load_group(1, w_next);
    expand_to_smem(0, 0, w_cur);
    cp_async_wait<1>();   // group 0's activation tile has landed; group 1's may still be in flight
    __syncthreads();

    for (int g = 0; g < G; ++g) {
      const int buf = g & 1;
      const int abuf = g % kAStages;
      GroupRegs w_ahead;
      if (g + 2 < G) {
        issue_a(g + 2, (g + 2) % kAStages);
        load_group(g + 2, w_ahead);
      } else {
        cp_async_commit();
      }

      const uint32_t a_base = smem_u32(s_a + abuf * TILEA);
      const uint32_t b_base = smem_u32(s_b + buf * TILEB);
      const int mat = lane >> 3, rr = lane & 7;
#pragma unroll
      for (int blk = 0; blk < NBLK; ++blk) {
        Acc acc[MT][NT][4];
#pragma unroll
        for (int i = 0; i < MT; ++i)
#pragma unroll
          for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int q = 0; q < 4; ++q) acc[i][j][q] = 0;
#pragma unroll
        for (int ks = 0; ks < KSTEPS_BLK; ++ks) {
          const int kc = (blk * KSTEPS_BLK + ks) * 2;
          uint32_t af[MT][4], bf[NT / 2][4];
#pragma unroll
          for (int mt = 0; mt < MT; ++mt)
            ldmatrix_x4(af[mt], a_base + swz<ROWB>(wm * (MT * 16) + mt * 16 + rr + (mat & 1) * 8, kc + (mat >> 1)));
#pragma unroll
          for (int np = 0; np < NT / 2; ++np)
            ldmatrix_x4(bf[np], b_base + swz<ROWB>(wn * (NT * 8) + np * 16 + rr + (mat >> 1) * 8, kc + (mat & 1)));
#pragma unroll
          for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
              Mma<MODE>::run(acc[mt][nt], af[mt], bf[nt >> 1][(nt & 1) * 2], bf[nt >> 1][(nt & 1) * 2 + 1]);
        }
        // total += (acc * row_scale) * col_norm, unfused, group order
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int r = wm * (MT * 16) + mt * 16 + (lane >> 2) + h * 8;
            const float rs = s_rs[(buf * kBM + r) * 4 + blk];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
              for (int q = 0; q < 2; ++q) {
                const int c = wn * (NT * 8) + nt * 8 + (lane & 3) * 2 + q;
                const float nv = s_norm[buf * kBN + c];
                const float v = __fmul_rn(__fmul_rn((float)acc[mt][nt][h * 2 + q], rs), nv);
                total[mt][nt][h * 2 + q] = __fadd_rn(total[mt][nt][h * 2 + q], v);
                if (MODE == DMOQ_A8 && a.partials != nullptr && r < tile.rows) {
                  const int n_out = a.is_down ? a.hidden : 2 * a.inter;
                  const int n = a.is_down ? nb * kBN + c : (c & 1) * a.inter + nb * (kBN / 2) + (c >> 1);
                  a.partials[((size_t)(tile.row0 + r) * n_out + n) * G + g] = (int32_t)acc[mt][nt][h * 2 + q];
                }
              }
            }
          }
        }
      }

      if (g + 1 < G) expand_to_smem(buf ^ 1, (g + 1) % kAStages, w_next);
      cp_async_wait<1>();   // the next group's activation tile has landed
      __syncthreads();
      if (g + 2 < G) w_next = w_ahead;
    }
    cp_async_wait<0>();

    // ---- epilogue through shared memory (operand buffers are free now)
    if (EPI == DMOQ_EPI_SILU) {
      __half* s_out = reinterpret_cast<__half*>(smem);  // 128 x 64
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int r = wm * (MT * 16) + mt * 16 + (lane >> 2) + h * 8;
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            const float gate = __half2float(__float2half_rn(total[mt][nt][h * 2 + 0]));
            const float up = __half2float(__float2half_rn(total[mt][nt][h * 2 + 1]));
            const float sg = __half2float(__float2half_rn(__fdiv_rn(gate, 1.0f + expf(-gate))));
            s_out[r * 64 + wn * (NT * 4) + nt * 4 + (lane & 3)] = __float2half_rn(__fmul_rn(sg, up));
          }
        }
      __syncthreads();
      __half* out = reinterpret_cast<__half*>(a.out);
      for (int c = tid; c < kBM * 8; c += kThreads) {
        const int r = c >> 3, ch = c & 7;
        if (r < tile.rows)
          *reinterpret_cast<uint4*>(out + (size_t)(tile.row0 + r) * a.out_stride + nb * 64 + ch * 8) =
              *reinterpret_cast<const uint4*>(s_out + r * 64 + ch * 8);
      }
    } else if (EPI == DMOQ_EPI_PLAIN && !a.is_down) {
      // un-fused gate_up output (R, 2*inter) fp16: column j of the tile is gate (even) / up (odd)
      __half* out = reinterpret_cast<__half*>(a.out);
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int r = wm * (MT * 16) + mt * 16 + (lane >> 2) + h * 8;
          if (r >= tile.rows) continue;
#pragma unroll
          for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int q = 0; q < 2; ++q) {
              const int c = wn * (NT * 8) + nt * 8 + (lane & 3) * 2 + q;
              const int n = (c & 1) * a.inter + nb * (kBN / 2) + (c >> 1);
              out[(size_t)(tile.row0 + r) * a.out_stride + n] = __float2half_rn(total[mt][nt][h * 2 + q]);
            }
        }
    } else {
      uint16_t* s_out = reinterpret_cast<uint16_t*>(smem);  // 128 x 128
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int r = wm * (MT * 16) + mt * 16 + (lane >> 2) + h * 8;
          float wgt = 1.f;
          if (EPI == DMOQ_EPI_WEIGHTED) wgt = r < tile.rows ? a.row_weight[tile.row0 + r] : 0.f;
#pragma unroll
          for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int q = 0; q < 2; ++q) {
              const __half h16 = __float2half_rn(total[mt][nt][h * 2 + q]);
              uint16_t bits;
              if (EPI == DMOQ_EPI_WEIGHTED) {
                const __nv_bfloat16 b = __float2bfloat16_rn(__half2float(h16));
                bits = __bfloat16_as_ushort(__float2bfloat16_rn(__fmul_rn(__bfloat162float(b), wgt)));
              } else {
                bits = __half_as_ushort(h16);
              }
              s_out[r * kBN + wn * (NT * 8) + nt * 8 + (lane & 3) * 2 + q] = bits;
            }
        }
      __syncthreads();
      uint16_t* out = reinterpret_cast<uint16_t*>(a.out);
      for (int c = tid; c < kBM * 16; c += kThreads) {
        const int r = c >> 4, ch = c & 15;
        if (r < tile.rows)
          *reinterpret_cast<uint4*>(out + (size_t)(tile.row0 + r) * a.out_stride + nb * kBN + ch * 8) =
              *reinterpret_cast<const uint4*>(s_out + r * kBN + ch * 8);
      }
    }
  }
}

template <int MODE, int BM>
constexpr size_t smem_bytes(int bit) {
  return 2 * (size_t)Traits<MODE>::TILEB + kAStages * (size_t)BM * Traits<MODE>::ROWB + (2 * kBN + 2 * BM * 4) * sizeof(float) +
         BM * sizeof(int32_t) +
         256 * (size_t)(8 / bit) * Traits<MODE>::ES + 128;
}

template <int MODE, int BIT, int EPI, int BM>
int launch(const GemmArgs& a, int work_cap, cudaStream_t s) {
  static DmoqOncePerDevice once;
  bool* configured = once.slot();
  if (configured == nullptr) return DMOQ_EDEVICE;
  const size_t bytes = smem_bytes<MODE, BM>(BIT);
  if (!*configured) {
    if (cudaFuncSetAttribute(grouped_gemm_kernel<MODE, BIT, EPI, BM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes) != cudaSuccess)
      return DMOQ_ELAUNCH;
    *configured = true;
  }
  int grid = dmoq_sm_count();
  if (grid > work_cap) grid = work_cap;
  if (grid < 1) grid = 1;
  grouped_gemm_kernel<MODE, BIT, EPI, BM><<<grid, kThreads, bytes, s>>>(a);
  return dmoq_launch_status();
}

template <int MODE, int BIT, int EPI>
int launch_bm(const GemmArgs& a, int bm, int work_cap, cudaStream_t s) {
  return bm == 128 ? launch<MODE, BIT, EPI, 128>(a, work_cap, s) : launch<MODE, BIT, EPI, 32>(a, work_cap, s);
}

template <int MODE, int BIT>
int launch_epi(const GemmArgs& a, int epi, int bm, int work_cap, cudaStream_t s) {
  switch (epi) {
    case DMOQ_EPI_SILU: return launch_bm<MODE, BIT, DMOQ_EPI_SILU>(a, bm, work_cap, s);
    case DMOQ_EPI_WEIGHTED: return launch_bm<MODE, BIT, DMOQ_EPI_WEIGHTED>(a, bm, work_cap, s);
    case DMOQ_EPI_PLAIN: return launch_bm<MODE, BIT, DMOQ_EPI_PLAIN>(a, bm, work_cap, s);
    default: return DMOQ_EINVAL;
  }
}

template <int MODE>
int launch_bit(const GemmArgs& a, int bit, int epi, int bm, int work_cap, cudaStream_t s) {
  switch (bit) {
    case 1: return launch_epi<MODE, 1>(a, epi, bm, work_cap, s);
    case 2: return launch_epi<MODE, 2>(a, epi, bm, work_cap, s);
    case 4: return launch_epi<MODE, 4>(a, epi, bm, work_cap, s);
    case 8: return launch_epi<MODE, 8>(a, epi, bm, work_cap, s);
    default: return DMOQ_EINVAL;
  }
}

}  // namespace

bool dmoq_tc_supported(const dmoq_pool_t& p, int is_down, int hidden);
int dmoq_grouped_gemm_tc(const dmoq_route_t* route, const dmoq_pool_t& p, int pool_index, int is_down, int epilogue,
                         int hidden, const void* a_codes, const void* a_scales, int a_stride, void* out, int out_stride,
                         int32_t* partials, cudaStream_t s);

bool dmoq_img_supported(const dmoq_pool_t& p, int is_down, int hidden);
int dmoq_grouped_gemm_img(const dmoq_route_t* route, const dmoq_pool_t* pools, int pool_index, int is_down, int epilogue,
                          int hidden, const void* a_codes, const void* a_scales, int a_stride, void* out, int out_stride,
                          int32_t* partials, cudaStream_t s);
int dmoq_grouped_gemm_img_pools(const dmoq_route_t* route, const dmoq_pool_t* pools, const int32_t* pool_ids, int n_ids,
                                int is_down, int epilogue, int hidden, const void* a_codes, const void* a_scales, int a_stride,
                                void* out, int out_stride, int32_t* partials, cudaStream_t s);

// DMOQ_GEMM=mma forces the warp-level MMA kernel for every pool (A/B comparisons); default picks the
// tcgen05 kernel wherever it applies.
static bool use_tc_path() {
  static int cached = -1;
  if (cached < 0) {
    const char* v = getenv("DMOQ_GEMM");
    cached = (v && v[0] == 'm') ? 0 : 1;
  }
  return cached == 1;
}

extern "C" int dmoq_grouped_gemm(const dmoq_route_t* route, const dmoq_pool_t* pools_host, int32_t pool_index,
                                 int32_t is_down, int32_t epilogue, int32_t hidden,
                                 const void* a_codes, const void* a_scales, int32_t a_stride,
                                 void* out, int32_t out_stride, int32_t* partials, void* stream) {
  DMOQ_CHECK_ARG(route && pools_host && a_codes && out);
  DMOQ_CHECK_ARG(pool_index >= 0 && pool_index < route->n_pools);
  DMOQ_CHECK_ARG(route->tile_m == 128 || route->tile_m == 32);
  const dmoq_pool_t& p = pools_host[pool_index];
  DMOQ_CHECK_ARG(p.inter > 0 && p.inter % kG == 0 && hidden > 0 && hidden % kG == 0);
  DMOQ_CHECK_ARG(p.identity_lut || (is_down ? p.dn_lut : p.gu_lut));
  DMOQ_CHECK_ARG(p.mode == DMOQ_A16 || a_scales);
  DMOQ_CHECK_ARG(!(epilogue == DMOQ_EPI_SILU && is_down) && !(epilogue == DMOQ_EPI_WEIGHTED && !is_down));
  DMOQ_CHECK_ARG(out_stride % 8 == 0);
  if (p.bit == 8 && p.mode == DMOQ_FP4) return DMOQ_EINVAL;

  DMOQ_CHECK_ARG((is_down ? p.dn_idx : p.gu_idx) && (is_down ? p.dn_norm : p.gu_norm));
  DMOQ_CHECK_ARG(a_stride >= (is_down ? p.inter : hidden) && a_stride % kG == 0);
  // a pool that comes with a weight image runs on the image-fed tensor-core kernel, which takes whole tiles of the
  // activation-code table: the table must be in routed-row order
  if (route->tile_m == 128 && use_tc_path() && (is_down || route->a_row == nullptr) && dmoq_img_supported(p, is_down, hidden))
    return dmoq_grouped_gemm_img(route, pools_host, pool_index, is_down, epilogue, hidden, a_codes, a_scales, a_stride, out,
                                 out_stride, partials, static_cast<cudaStream_t>(stream));
  if (route->tile_m == 128 && use_tc_path() && dmoq_tc_supported(p, is_down, hidden))
    return dmoq_grouped_gemm_tc(route, p, pool_index, is_down, epilogue, hidden, a_codes, a_scales, a_stride, out,
                                out_stride, partials, static_cast<cudaStream_t>(stream));

  GemmArgs a{};
  a.tiles = reinterpret_cast<const DmoqTile*>(route->tiles);
  a.n_tiles = route->n_tiles;
  a.expert_rank = route->expert_rank;
  a.a_row = is_down ? nullptr : route->a_row;
  a.row_weight = route->sorted_weights;
  a.pool = pool_index;
  a.is_down = is_down;
  a.inter = p.inter;
  a.hidden = hidden;
  a.n_members = p.n_members;
  a.idx = is_down ? p.dn_idx : p.gu_idx;
  a.norm = is_down ? p.dn_norm : p.gu_norm;
  a.lut = is_down ? p.dn_lut : p.gu_lut;
  a.identity_lut = p.identity_lut;
  a.e0 = is_down ? p.dn_e0 : p.gu_e0;
  a.a_codes = static_cast<const uint8_t*>(a_codes);
  a.a_scales = static_cast<const uint8_t*>(a_scales);
  a.a_stride = a_stride;
  DMOQ_CHECK_ARG(a_stride >= (is_down ? p.inter : hidden) && a_stride % kG == 0);
  a.out = out;
  a.out_stride = out_stride;
  a.partials = partials;
  DMOQ_CHECK_ARG(a.idx && a.norm);
  const int nb = is_down ? hidden / kBN : p.inter / (kBN / 2);
  long long cap = (long long)route->tile_cap * nb;
  const int work_cap = cap > (1 << 30) ? (1 << 30) : (int)cap;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (p.mode) {
    case DMOQ_A16: return launch_bit<DMOQ_A16>(a, p.bit, epilogue, route->tile_m, work_cap, s);
    case DMOQ_A8: return launch_bit<DMOQ_A8>(a, p.bit, epilogue, route->tile_m, work_cap, s);
    case DMOQ_FP8: return launch_bit<DMOQ_FP8>(a, p.bit, epilogue, route->tile_m, work_cap, s);
    case DMOQ_FP4: return launch_bit<DMOQ_FP4>(a, p.bit, epilogue, route->tile_m, work_cap, s);
    default: return DMOQ_EINVAL;
  }
}

// The same GEMM for several pools of one activation mode in ONE launch; every listed pool needs its weight image
// and the code table must be in routed-row order.
extern "C" int dmoq_grouped_gemm_pools(const dmoq_route_t* route, const dmoq_pool_t* pools_host, const int32_t* pool_ids,
                                       int32_t n_ids, int32_t is_down, int32_t epilogue, int32_t hidden,
                                       const void* a_codes, const void* a_scales, int32_t a_stride, void* out,
                                       int32_t out_stride, void* stream) {
  DMOQ_CHECK_ARG(route && pools_host && pool_ids && a_codes && out && n_ids >= 1 && n_ids <= DMOQ_MAX_POOLS);
  DMOQ_CHECK_ARG(route->tile_m == 128 && (is_down || route->a_row == nullptr));
  DMOQ_CHECK_ARG(!(epilogue == DMOQ_EPI_SILU && is_down) && !(epilogue == DMOQ_EPI_WEIGHTED && !is_down));
  DMOQ_CHECK_ARG(out_stride % 8 == 0 && hidden > 0 && hidden % kG == 0 && a_stride % kG == 0);
  for (int i = 0; i < n_ids; ++i) {
    DMOQ_CHECK_ARG(pool_ids[i] >= 0 && pool_ids[i] < route->n_pools);
    const dmoq_pool_t& p = pools_host[pool_ids[i]];
    DMOQ_CHECK_ARG(p.mode == DMOQ_A16 || a_scales);
    DMOQ_CHECK_ARG(p.inter > 0 && p.inter % kG == 0 && a_stride >= (is_down ? p.inter : hidden));
  }
  return dmoq_grouped_gemm_img_pools(route, pools_host, pool_ids, n_ids, is_down, epilogue, hidden, a_codes, a_scales, a_stride,
                                     out, out_stride, nullptr, static_cast<cudaStream_t>(stream));
}
