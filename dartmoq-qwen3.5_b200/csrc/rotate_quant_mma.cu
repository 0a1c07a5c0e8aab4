// Group rotation on the tensor cores with an exact fix-up, fused with activation quantisation.
//
// The codes are DEFINED through a sequential fp32 FMA chain over k = 0..127 per rotated value (that is
// what a CPU can reproduce bit for bit).  Computing every value that way costs 128 dependent FMAs; this
// kernel gets the same codes with a few percent of that work:
//   1. all 128x128 rotated values of a row block come from fp16 tensor-core MMAs (fp32 accumulate);
//      they differ from the chain values by at most delta = 2^-16 * |x_row|_2  (the chain's own worst-case
//      rounding bound is 127 * 2^-24 * |x|_2 |p|_2 < 2^-17 |x|_2; the same again is allowed for the MMA);
//   2. the row / block maximum is taken over chain values of every element within 2*delta of the
//      approximate maximum, so the scale is the exact one;
//   3. an element keeps the code of its approximate value only if the whole interval [v-t, v+t]
//      (t = delta / scale) quantises to ONE code; otherwise its chain value is computed and quantised.
// The elements of steps 2 and 3 (about 1 % and 2 % of a block) go through a block-wide queue, so that the
// 256 threads share the chains evenly whichever lanes flagged them.
// Quantisation rules: turboquant_utils/triton_kernels_a8.py:473-484 (int8), triton_kernels_fp8.py:176-187
// (e4m3), triton_kernels_fp4.py:1073-1104 (e2m1 + per-32 e8m0).  The unquantised fp16 output (A16 mode,
// rotation.py:176) is the rounded MMA value: a floating-point output, not a code.
#include "rotq.cuh"

#ifdef DMOQ_ROTQ_PROFILE
__device__ unsigned long long g_rotq_prof[16];
#define RP_T(i)                                                                 \
  do {                                                                          \
    if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) {               \
      const long long now_ = clock64();                                         \
      atomicAdd(&g_rotq_prof[i], (unsigned long long)(now_ - rp_last));         \
      rp_last = now_;                                                           \
    }                                                                           \
  } while (0)
#define RP_START()                                                              \
  do {                                                                          \
    if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) rp_last = clock64(); \
  } while (0)
#else
#define RP_T(i)
#define RP_START()
#endif

namespace {

#ifdef DMOQ_ROTQ_PROFILE
__device__ long long rp_last;
#endif

constexpr int kG = DMOQ_GROUP;
constexpr int kRows = 128;            // rows per block
constexpr int kThreads = 256;         // 8 warps x 16 rows
constexpr int kPitchQ = 144;          // staged code row: 128 one-byte codes + pad (conflict-free 2-byte stores)
constexpr int kPitchH = 272;          // staged fp16 row (A16)
constexpr int kQueueCap = 2048;
constexpr size_t kOff_x16 = 0, kOff_p16 = 32768, kOff_stage = 65536;
constexpr size_t kOff_n2 = kOff_stage + (size_t)kRows * kPitchH;   // |x_row|^2
constexpr size_t kOff_rowmax = kOff_n2 + kRows * 4;                // u32 bits of the exact max |v| per (row, 32-col block)
constexpr size_t kOff_tab = kOff_rowmax + kRows * 16;              // scale (float) or exponent (int) per (row, block)
constexpr size_t kOff_wsum = kOff_tab + kRows * 16;                // per-warp queue counts, one set per phase
constexpr size_t kOff_queue = kOff_wsum + 64;
constexpr size_t kSmem = kOff_queue + (size_t)kQueueCap * 2;       // ~107 KB: two blocks per SM

__device__ __forceinline__ uint32_t swz256(int r, int c) { return (uint32_t)(r * 256 + ((c ^ (r & 7)) << 4)); }

__device__ __forceinline__ void ldsm4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void mma_f16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// A 128 x 128 block of 16-bit values travels in two steps: global memory -> registers (sixteen consecutive lanes
// read the 256 bytes of one row; thread t holds 16 bytes of rows t/16 + 16j), registers -> swizzled fp16 tile.
// The split lets the loads of the NEXT block fly while the current block is finished.
struct XRegs {
  uint4 raw[8];
};
// `row_src(r)` gives the global row or -1 (zero row).
template <typename RowSrc>
__device__ __forceinline__ void load_block(XRegs& xr, const void* base, size_t pitch, size_t col0, RowSrc row_src) {
  const int c = threadIdx.x & 15;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const long long src = row_src((int)(threadIdx.x >> 4) + 16 * j);
    xr.raw[j] = make_uint4(0u, 0u, 0u, 0u);
    if (src >= 0) xr.raw[j] = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(base) + (size_t)src * pitch + col0 + c * 8);
  }
}
__device__ __forceinline__ void store_block(const XRegs& xr, uint8_t* s16, float* s_n2, int is_bf16) {
  const int c = threadIdx.x & 15;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int r = (threadIdx.x >> 4) + 16 * j;
    __align__(16) __half h[8];
    const uint16_t* u = reinterpret_cast<const uint16_t*>(&xr.raw[j]);
    float ss = 0.f;
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      h[q] = is_bf16 ? __float2half_rn(bf16_bits_to_float(u[q])) : __ushort_as_half(u[q]);
      const float f = __half2float(h[q]);
      ss = fmaf(f, f, ss);
    }
    *reinterpret_cast<uint4*>(s16 + swz256(r, c)) = *reinterpret_cast<const uint4*>(h);
    if (s_n2 != nullptr) {
#pragma unroll
      for (int d = 1; d < 16; d <<= 1) ss += __shfl_xor_sync(0xffffffffu, ss, d);
      if (c == 0) s_n2[r] = ss;
    }
  }
}

__device__ __forceinline__ uint32_t code_i8(float v) { return (uint32_t)(uint8_t)(int8_t)fminf(fmaxf(roundf(v), -127.f), 127.f); }
__device__ __forceinline__ uint32_t code_e4m3(float v) { return (uint32_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3); }
__device__ __forceinline__ uint32_t code_e2m1(float y) {
  y = fminf(fmaxf(y, -6.f), 6.f);
  const float a = fabsf(y);
  const uint32_t mag = a < 0.25f ? 0 : a < 0.75f ? 1 : a < 1.25f ? 2 : a < 1.75f ? 3 : a < 2.5f ? 4 : a < 3.5f ? 5 : a < 5.0f ? 6 : 7;
  return mag | (y < 0.f ? 8u : 0u);
}
__device__ __forceinline__ float quad_max(float v) {
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
  return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
}

// ---- exact values: sequential fp32 chains read from the fp16 tiles --------------------------------
struct ChainSrc {
  const uint8_t* row;
  uint32_t sw;
};
__device__ __forceinline__ ChainSrc chain_src(const uint8_t* tile, int r) { return ChainSrc{tile + r * 256, (uint32_t)(r & 7) << 4}; }

__device__ __forceinline__ void chain_step(float& acc, const uint4& xv, const uint4& pv) {
  const __half2* xh = reinterpret_cast<const __half2*>(&xv);
  const __half2* ph = reinterpret_cast<const __half2*>(&pv);
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const float2 xf = __half22float2(xh[q]), pf = __half22float2(ph[q]);
    acc = fmaf(xf.x, pf.x, acc);
    acc = fmaf(xf.y, pf.y, acc);
  }
}
// The loads of chunk c+1 are issued before the eight dependent FMAs of chunk c, so the chain runs at the FMA
// latency instead of waiting on shared memory in every step.
__device__ __forceinline__ float chain1(ChainSrc x, ChainSrc p) {
  float acc = 0.f;
  uint4 xv = *reinterpret_cast<const uint4*>(x.row + x.sw), pv = *reinterpret_cast<const uint4*>(p.row + p.sw);
#pragma unroll
  for (uint32_t c = 0; c < 256; c += 16) {
    uint4 xn = xv, pn = pv;
    if (c + 16 < 256) {
      xn = *reinterpret_cast<const uint4*>(x.row + ((c + 16) ^ x.sw));
      pn = *reinterpret_cast<const uint4*>(p.row + ((c + 16) ^ p.sw));
    }
    chain_step(acc, xv, pv);
    xv = xn;
    pv = pn;
  }
  return acc;
}
// What a thread does with the chain value of queue entry (row, col).
//   PHASE 1: fold |v| into the exact maximum of the entry's (row, 32-column block).
//   PHASE 2: quantise with the row's / block's scale and overwrite the staged approximate code.
template <int MODE, int PHASE>
__device__ __forceinline__ void consume(uint8_t* smem, int ent, float v) {
  const int row = ent >> 8, col = ent & 255;
  const int blk = (MODE == DMOQ_FP4) ? (col >> 5) : 0;
  if (PHASE == 1) {
    atomicMax(reinterpret_cast<uint32_t*>(smem + kOff_rowmax) + row * 4 + blk, __float_as_uint(fabsf(v)));
  } else {
    uint32_t code;
    if (MODE == DMOQ_FP4) {
      code = code_e2m1(ldexpf(v, -reinterpret_cast<const int*>(smem + kOff_tab)[row * 4 + blk]));
    } else {
      const float q = __fdiv_rn(v, reinterpret_cast<const float*>(smem + kOff_tab)[row * 4]);
      code = (MODE == DMOQ_A8) ? code_i8(q) : code_e4m3(q);
    }
    smem[kOff_stage + row * kPitchQ + col] = (uint8_t)code;
  }
}

// Block-wide queue.  mask[h] flags elements of this thread's row (rbase + 8h): bit i = the thread's i-th value of
// that row, column 8*(i/2) + 2*t4 + (i&1).  Every thread of the block must call this (it synchronises).
template <int MODE, int PHASE>
__device__ __forceinline__ void resolve(uint8_t* smem, const uint32_t (&mask)[2], int rbase, int t4) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  int* wsum = reinterpret_cast<int*>(smem + kOff_wsum) + (PHASE - 1) * 8;
  uint16_t* entry = reinterpret_cast<uint16_t*>(smem + kOff_queue);
  const int cnt = __popc(mask[0]) + __popc(mask[1]);
  int incl = cnt;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int n = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= d) incl += n;
  }
  if (lane == 31) wsum[warp] = incl;
  __syncthreads();
  int first = incl - cnt, total = 0;
#pragma unroll
  for (int w = 0; w < 8; ++w) {
    const int n = wsum[w];
    total += n;
    if (w < warp) first += n;
  }
  const uint8_t* x16 = smem + kOff_x16;
  const uint8_t* p16 = smem + kOff_p16;
  for (int q0 = 0; q0 < total; q0 += kQueueCap) {   // one round unless more than kQueueCap elements are flagged
    int rank = first - q0;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      uint32_t m = mask[h];
      while (m) {
        const int i = __ffs(m) - 1;
        m &= m - 1;
        if ((unsigned)rank < (unsigned)kQueueCap)
          entry[rank] = (uint16_t)(((rbase + 8 * h) << 8) | (8 * (i >> 1) + 2 * t4 + (i & 1)));
        ++rank;
      }
    }
    __syncthreads();
    RP_T(8 + (PHASE - 1) * 3);       // scan + enqueue
    const int n = min(kQueueCap, total - q0);
    for (int i = tid; i < n; i += kThreads) {   // one chain at a time: registers stay free for the prefetched block
      const int e0 = entry[i];
      consume<MODE, PHASE>(smem, e0, chain1(chain_src(x16, e0 >> 8), chain_src(p16, e0 & 255)));
    }
    RP_T(9 + (PHASE - 1) * 3);       // this thread's chains
    if (q0 + kQueueCap < total) __syncthreads();   // the queue is refilled
  }
  __syncthreads();
  RP_T(10 + (PHASE - 1) * 3);        // waiting for the slowest warp
}

// One row block: rows [0, rows) of the staged x tile, group g.  `out_row(r)` = destination row.
// `prefetch()` is called once, at the point where the accumulators are dead and only the fix-up chains and the
// copy-out remain: the caller starts the global loads of its next block there.
template <int MODE, typename OutRow, typename Prefetch>
__device__ void rotq_mma_block(const RotArgs& a, uint8_t* smem, int g, int rows, OutRow out_row, Prefetch prefetch) {
  const uint8_t* x16 = smem + kOff_x16;
  const uint8_t* p16 = smem + kOff_p16;
  uint8_t* stage = smem + kOff_stage;
  const float* n2 = reinterpret_cast<const float*>(smem + kOff_n2);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int mat = lane >> 3, rr = lane & 7, t4 = lane & 3;
  const int rbase = warp * 16 + (lane >> 2);

  RP_T(0);   // staging (and whatever preceded this block)
  // ---- approximate rotation on the tensor cores: warp = 16 rows x 128 columns
  float acc[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i)
#pragma unroll
    for (int q = 0; q < 4; ++q) acc[i][q] = 0.f;
  const uint32_t xa = smem_u32(x16), pa = smem_u32(p16);
#pragma unroll
  for (int ks = 0; ks < 8; ++ks) {
    uint32_t af[4];
    ldsm4(af, xa + swz256(warp * 16 + rr + (mat & 1) * 8, 2 * ks + (mat >> 1)));
#pragma unroll
    for (int np = 0; np < 8; ++np) {
      uint32_t bf[4];
      ldsm4(bf, pa + swz256(np * 16 + rr + (mat >> 1) * 8, 2 * ks + (mat & 1)));
      mma_f16(acc[2 * np], af, bf[0], bf[1]);
      mma_f16(acc[2 * np + 1], af, bf[2], bf[3]);
    }
  }

  if (MODE == DMOQ_A16) {
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int nt = 0; nt < 16; ++nt)
        *reinterpret_cast<__half2*>(stage + (rbase + 8 * h) * kPitchH + (8 * nt + 2 * t4) * 2) =
            __floats2half2_rn(acc[nt][2 * h], acc[nt][2 * h + 1]);
    prefetch();
    __syncthreads();
  } else {
    constexpr int NB = (MODE == DMOQ_FP4) ? 4 : 1;      // scale blocks per row of the group
    constexpr int TPB = 16 / NB;                         // n-tiles (8 columns each) per scale block
    float delta[2];
    bool live[2];
    uint32_t mask[2];
    // ---- phase 1: the exact maximum of every row / block
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int r = rbase + 8 * h;
      const float nn = n2[r];
      delta[h] = ldexpf(sqrtf(nn), -16) * 1.01f;
      live[h] = r < rows && nn > 0.f;   // padding rows and all-zero rows never ask for a chain value
      mask[h] = 0;
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        float m = 0.f;
#pragma unroll
        for (int nt = b * TPB; nt < (b + 1) * TPB; ++nt) m = fmaxf(m, fmaxf(fabsf(acc[nt][2 * h]), fabsf(acc[nt][2 * h + 1])));
        m = quad_max(m);
        const float thr = live[h] ? m - 2.f * delta[h] : 3.0e38f;
#pragma unroll
        for (int nt = b * TPB; nt < (b + 1) * TPB; ++nt) {
          mask[h] |= (fabsf(acc[nt][2 * h]) >= thr) ? (1u << (2 * nt)) : 0u;
          mask[h] |= (fabsf(acc[nt][2 * h + 1]) >= thr) ? (2u << (2 * nt)) : 0u;
        }
      }
    }
    RP_T(1);   // MMA + phase-1 flags
    resolve<MODE, 1>(smem, mask, rbase, t4);
    RP_T(2);   // phase-1 chains

    // ---- phase 2: approximate codes for everything, exact ones where the approximation cannot decide
    const uint32_t* rowmax = reinterpret_cast<const uint32_t*>(smem + kOff_rowmax);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int r = rbase + 8 * h;
      uint8_t* srow = stage + r * kPitchQ;
      mask[h] = 0;
      if (MODE == DMOQ_A8 || MODE == DMOQ_FP8) {
        const float amax = __uint_as_float(rowmax[r * 4]);
        const float full = (MODE == DMOQ_A8) ? 127.0f : 448.0f;
        const float tiny = (MODE == DMOQ_A8) ? (float)(1e-8 * 127.0) : (float)(1e-8 * 448.0);
        const float s = (amax < tiny) ? 1e-8f : __fdiv_rn(amax, full);
        const float inv_s = 1.0f / s;
        const float t = delta[h] * inv_s * 1.001f + 3e-5f;   // also covers v*inv_s versus the IEEE quotient v/s
        if (t4 == 0) {
          reinterpret_cast<float*>(smem + kOff_tab)[r * 4] = s;
          if (r < rows)
            reinterpret_cast<__half*>(a.scales)[(size_t)out_row(r) * (a.o_stride / kG) + g] = __float2half_rn(__fmul_rn(s, a.extra_scale));
        }
#pragma unroll
        for (int nt = 0; nt < 16; ++nt) {
          const float q0 = acc[nt][2 * h] * inv_s, q1 = acc[nt][2 * h + 1] * inv_s;
          uint32_t c01;
          if (MODE == DMOQ_A8) {
            // round to nearest even by adding 1.5 * 2^23: the sum's low mantissa byte is the int8 code.  An element
            // that is not flagged is not within t of a half, so this equals the half-away rounding of the definition;
            // |q| < 127.5 always (the row maximum maps to 127), so no clamp is needed.
            const float m0 = q0 + 12582912.0f, m1 = q1 + 12582912.0f;
            const float r0 = m0 - 12582912.0f, r1 = m1 - 12582912.0f;
            mask[h] |= (fabsf(q0 - r0) > 0.5f - t) ? (1u << (2 * nt)) : 0u;
            mask[h] |= (fabsf(q1 - r1) > 0.5f - t) ? (2u << (2 * nt)) : 0u;
            c01 = __byte_perm(__float_as_uint(m0), __float_as_uint(m1), 0x4440);
          } else {
            const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(q0 - t, q1 - t), __NV_SATFINITE, __NV_E4M3);
            const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(q0 + t, q1 + t), __NV_SATFINITE, __NV_E4M3);
            const uint32_t d = lo ^ hi;
            mask[h] |= (d & 0xFFu) ? (1u << (2 * nt)) : 0u;
            mask[h] |= (d & 0xFF00u) ? (2u << (2 * nt)) : 0u;
            c01 = __nv_cvt_float2_to_fp8x2(make_float2(q0, q1), __NV_SATFINITE, __NV_E4M3);
          }
          *reinterpret_cast<uint16_t*>(srow + 8 * nt + 2 * t4) = live[h] ? (uint16_t)c01 : (uint16_t)0;
        }
      } else {
        uint32_t e_bytes = 0;
#pragma unroll
        for (int b = 0; b < NB; ++b) {
          const float amax = fmaxf(__uint_as_float(rowmax[r * 4 + b]), 1e-30f);
          float e = ceilf((float)log2((double)__fdiv_rn(amax, 6.0f)));
          e = fminf(fmaxf(e, -127.f), 127.f);
          const int ei = (int)e;
          e_bytes |= (uint32_t)(ei + 127) << (8 * b);
          if (t4 == 0) reinterpret_cast<int*>(smem + kOff_tab)[r * 4 + b] = ei;
          const float tb = ldexpf(delta[h], -ei) * 1.001f + 1e-6f;
#pragma unroll
          for (int nt = b * TPB; nt < (b + 1) * TPB; ++nt) {
            const float y0 = ldexpf(acc[nt][2 * h], -ei), y1 = ldexpf(acc[nt][2 * h + 1], -ei);
            mask[h] |= (code_e2m1(y0 - tb) != code_e2m1(y0 + tb)) ? (1u << (2 * nt)) : 0u;
            mask[h] |= (code_e2m1(y1 - tb) != code_e2m1(y1 + tb)) ? (2u << (2 * nt)) : 0u;
            const uint32_t c01 = code_e2m1(y0) | (code_e2m1(y1) << 8);
            *reinterpret_cast<uint16_t*>(srow + 8 * nt + 2 * t4) = live[h] ? (uint16_t)c01 : (uint16_t)0;
          }
        }
        if (t4 == 0 && r < rows)
          *reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(a.scales) + (size_t)out_row(r) * (a.o_stride / 32) + g * 4) = e_bytes;
      }
      if (!live[h]) mask[h] = 0;
    }
    RP_T(3);   // phase-2 owner part
    prefetch();
    RP_T(6);   // prefetch issue
    resolve<MODE, 2>(smem, mask, rbase, t4);
    RP_T(4);   // prefetch issue + phase-2 chains
  }

  // ---- coalesced copy-out of the staged tile
  if (MODE == DMOQ_A16) {
    for (int i = tid; i < kRows * 16; i += kThreads) {
      const int r = i >> 4, ch = i & 15;
      if (r < rows)
        *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(a.codes) + ((size_t)out_row(r) * a.o_stride + (size_t)g * kG) * 2 + ch * 16) =
            *reinterpret_cast<const uint4*>(stage + r * kPitchH + ch * 16);
    }
  } else if (MODE == DMOQ_FP4) {   // two staged one-byte codes -> one output byte, even column in the low nibble
    for (int i = tid; i < kRows * 4; i += kThreads) {
      const int r = i >> 2, ch = i & 3;
      if (r < rows) {
        const uint4 lo = *reinterpret_cast<const uint4*>(stage + r * kPitchQ + ch * 32);
        const uint4 hi = *reinterpret_cast<const uint4*>(stage + r * kPitchQ + ch * 32 + 16);
        const uint32_t w[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint32_t a0 = w[2 * j] | (w[2 * j] >> 4), a1 = w[2 * j + 1] | (w[2 * j + 1] >> 4);   // bytes 0 and 2 hold the pairs
          o[j] = (a0 & 0xFFu) | ((a0 >> 8) & 0xFF00u) | ((a1 & 0xFFu) << 16) | ((a1 << 8) & 0xFF000000u);
        }
        *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(a.codes) + (size_t)out_row(r) * (a.o_stride / 2) + (size_t)g * 64 + ch * 16) =
            make_uint4(o[0], o[1], o[2], o[3]);
      }
    }
  } else {
    for (int i = tid; i < kRows * 8; i += kThreads) {
      const int r = i >> 3, ch = i & 7;
      if (r < rows)
        *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(a.codes) + (size_t)out_row(r) * a.o_stride + (size_t)g * kG + ch * 16) =
            *reinterpret_cast<const uint4*>(stage + r * kPitchQ + ch * 16);
    }
  }
  __syncthreads();  // tiles, tables and the staged output are rewritten by the next block
  RP_T(5);   // copy-out
}

// registers -> x tile + row norms + cleared maxima for a row block; ends with a block-wide barrier.
__device__ __forceinline__ void stage_x(const XRegs& xr, const RotArgs& a, uint8_t* smem) {
  store_block(xr, smem + kOff_x16, reinterpret_cast<float*>(smem + kOff_n2), a.src_is_bf16);
  reinterpret_cast<uint2*>(smem + kOff_rowmax)[threadIdx.x] = make_uint2(0u, 0u);
  __syncthreads();
}

__device__ __forceinline__ void stage_rotation(uint8_t* smem, const uint16_t* mat) {
  XRegs pr;
  load_block(pr, mat, kG, 0, [](int r) { return (long long)r; });
  store_block(pr, smem + kOff_p16, nullptr, 0);
}

template <int MODE>
__global__ void __launch_bounds__(kThreads, 2) rotq_mma_rows_kernel(RotArgs a) {
  extern __shared__ __align__(1024) uint8_t smem[];
  const int g = blockIdx.x;
  const int n_rows = a.n_rows_dev ? min(*a.n_rows_dev, a.n_rows) : a.n_rows;
  const int n_blocks = (n_rows + kRows - 1) / kRows;
  if ((int)blockIdx.y >= n_blocks) return;
  RP_START();
  auto load = [&](XRegs& xr, int b) {
    const int row0 = b * kRows, rows = min(kRows, n_rows - row0);
    load_block(xr, a.x, (size_t)a.x_stride, (size_t)g * kG,
               [&](int r) { return r < rows ? (long long)(a.src_row ? a.src_row[row0 + r] : row0 + r) : -1LL; });
  };
  XRegs xr;
  load(xr, blockIdx.y);
  stage_rotation(smem, a.rot + (size_t)g * kG * kG);
  for (int b = blockIdx.y; b < n_blocks; b += gridDim.y) {
    const int row0 = b * kRows, rows = min(kRows, n_rows - row0);
    stage_x(xr, a, smem);
    rotq_mma_block<MODE>(a, smem, g, rows, [&](int r) { return row0 + r; },
                         [&]() { if (b + (int)gridDim.y < n_blocks) load(xr, b + gridDim.y); });
  }
}

template <int MODE>
__global__ void __launch_bounds__(kThreads, 2) rotq_mma_tiles_kernel(RotArgs a) {
  extern __shared__ __align__(1024) uint8_t smem[];
  const int g = blockIdx.x;
  const int n_tiles = a.n_tiles[a.pool];
  const DmoqTile* tiles = a.tiles + a.n_tiles[DMOQ_MAX_POOLS + a.pool];
  auto load = [&](XRegs& xr, const DmoqTile& tile, int r0) {
    const int row0 = tile.row0 + r0, rows = min(kRows, tile.rows - r0);
    load_block(xr, a.x, (size_t)a.x_stride, (size_t)g * kG, [&](int r) { return r < rows ? (long long)(row0 + r) : -1LL; });
  };
  int loaded = -1;
  int t = blockIdx.y;
  if (t >= n_tiles) return;
  RP_START();
  DmoqTile tile = tiles[t];
  int r0 = 0;
  XRegs xr;
  load(xr, tile, 0);
  while (true) {
    const int mat = tile.rank * a.groups_per_member + g;
    if (mat != loaded) {   // every thread left the previous block through its closing barrier
      stage_rotation(smem, a.rot + (size_t)mat * kG * kG);
      loaded = mat;
    }
    const int row0 = tile.row0 + r0, rows = min(kRows, tile.rows - r0);
    // the block after this one: the next 128 rows of the tile, else the first rows of this CTA's next tile
    int t_n = t, r0_n = r0 + kRows;
    DmoqTile tile_n = tile;
    if (r0_n >= tile.rows) {
      t_n = t + gridDim.y;
      r0_n = 0;
    }
    const bool more = t_n < n_tiles;
    if (more && t_n != t) tile_n = tiles[t_n];   // fetched now, used by the prefetch below: no dependent-load stall there
    stage_x(xr, a, smem);
    rotq_mma_block<MODE>(a, smem, g, rows, [&](int r) { return row0 + r; }, [&]() {
      if (more) load(xr, tile_n, r0_n);
    });
    if (!more) break;
    t = t_n;
    r0 = r0_n;
    tile = tile_n;
  }
}

template <int MODE>
int launch_rows(const RotArgs& a, cudaStream_t s) {
  static DmoqOncePerDevice once;
  bool* configured = once.slot();
  if (configured == nullptr) return DMOQ_EDEVICE;
  if (!*configured) {
    if (cudaFuncSetAttribute(rotq_mma_rows_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmem) != cudaSuccess)
      return DMOQ_ELAUNCH;
    *configured = true;
  }
  const int G = a.K / kG;
  const int n_blocks = dmoq_ceil_div(a.n_rows, kRows);
  // two blocks are resident per SM: the grid must not exceed those slots, or the blocks left over run alone
  // after the others have finished their whole share of row blocks
  int gy = (2 * dmoq_sm_count()) / G;
  if (gy > n_blocks) gy = n_blocks;
  if (gy < 1) gy = 1;
  rotq_mma_rows_kernel<MODE><<<dim3(G, gy), kThreads, kSmem, s>>>(a);
  return dmoq_launch_status();
}

template <int MODE>
int launch_tiles(const RotArgs& a, int tile_cap, cudaStream_t s) {
  static DmoqOncePerDevice once;
  bool* configured = once.slot();
  if (configured == nullptr) return DMOQ_EDEVICE;
  if (!*configured) {
    if (cudaFuncSetAttribute(rotq_mma_tiles_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmem) != cudaSuccess)
      return DMOQ_ELAUNCH;
    *configured = true;
  }
  const int G = a.K / kG;
  // two blocks are resident per SM: the grid must not exceed those slots, or the blocks left over run alone
  // after the others have finished their whole share of row blocks
  int gy = (2 * dmoq_sm_count()) / G;
  if (gy > tile_cap) gy = tile_cap;
  if (gy < 1) gy = 1;
  rotq_mma_tiles_kernel<MODE><<<dim3(G, gy), kThreads, kSmem, s>>>(a);
  return dmoq_launch_status();
}

}  // namespace

int dmoq_rotq_mma_rows(int mode, const RotArgs& a, cudaStream_t s) {
  switch (mode) {
    case DMOQ_A16: return launch_rows<DMOQ_A16>(a, s);
    case DMOQ_A8: return launch_rows<DMOQ_A8>(a, s);
    case DMOQ_FP8: return launch_rows<DMOQ_FP8>(a, s);
    case DMOQ_FP4: return launch_rows<DMOQ_FP4>(a, s);
    default: return DMOQ_EINVAL;
  }
}

int dmoq_rotq_mma_tiles(int mode, const RotArgs& a, int tile_cap, cudaStream_t s) {
  switch (mode) {
    case DMOQ_A16: return launch_tiles<DMOQ_A16>(a, tile_cap, s);
    case DMOQ_A8: return launch_tiles<DMOQ_A8>(a, tile_cap, s);
    case DMOQ_FP8: return launch_tiles<DMOQ_FP8>(a, tile_cap, s);
    case DMOQ_FP4: return launch_tiles<DMOQ_FP4>(a, tile_cap, s);
    default: return DMOQ_EINVAL;
  }
}

#ifdef DMOQ_ROTQ_PROFILE
extern "C" int dmoq_rotq_profile(unsigned long long* out16, int reset) {
  if (cudaMemcpyFromSymbol(out16, g_rotq_prof, sizeof(unsigned long long) * 16) != cudaSuccess) return DMOQ_EDEVICE;
  if (reset) {
    unsigned long long z[16] = {0};
    if (cudaMemcpyToSymbol(g_rotq_prof, z, sizeof(z)) != cudaSuccess) return DMOQ_EDEVICE;
  }
  return DMOQ_OK;
}
#endif
