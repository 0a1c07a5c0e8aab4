// Group rotation on the tensor cores with an exact fix-up, fused with activation quantisation.
//
// The codes are DEFINED through a sequential fp32 FMA chain over k = 0..127 per rotated value (that is
// what a CPU can reproduce bit for bit).  Computing every value that way costs 128 dependent FMAs; this
// kernel gets the same codes ~5x cheaper:
//   1. all 128x128 rotated values of a row block come from fp16 tensor-core MMAs (fp32 accumulate);
//      they differ from the chain values by at most delta = 2^-16 * |x_row|_2  (the chain's own worst-case
//      rounding bound is 127 * 2^-24 * |x|_2 |p|_2 < 2^-17 |x|_2; the same again is allowed for the MMA);
//   2. the row / block maximum is taken over chain values of every element within 2*delta of the
//      approximate maximum, so the scale is the exact one;
//   3. an element keeps the code of its approximate value only if the whole interval [v-t, v+t]
//      (t = delta / scale) quantises to ONE code; otherwise its chain value is computed and quantised.
// Quantisation rules: turboquant_utils/triton_kernels_a8.py:473-484 (int8), triton_kernels_fp8.py:176-187
// (e4m3), triton_kernels_fp4.py:1073-1104 (e2m1 + per-32 e8m0).  The unquantised fp16 output (A16 mode,
// rotation.py:176) is the rounded MMA value: a floating-point output, not a code.
#include "rotq.cuh"

namespace {

constexpr int kG = DMOQ_GROUP;
constexpr int kRows = 128;            // rows per block
constexpr int kThreads = 256;         // 8 warps x 16 rows
constexpr int kPitch32 = kG + 4;      // fp32 copies: padded rows, conflict-free 16-byte reads across rows
constexpr size_t kOff_x16 = 0, kOff_p16 = 32768, kOff_x32 = 65536;
constexpr size_t kOff_p32 = kOff_x32 + (size_t)kRows * kPitch32 * 4;
constexpr size_t kOff_n2 = kOff_p32 + (size_t)kG * kPitch32 * 4;
constexpr size_t kOff_queue = kOff_n2 + kRows * 4;                 // 8 warps x 512 x (float result + u16 entry)
constexpr size_t kSmem = kOff_queue + 8 * 512 * 6;

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

// 128 x 128 fp16 matrix (row pitch `pitch` elements in global memory) -> swizzled fp16 tile + padded fp32 copy.
// Thread t stages 64 columns of row t/2.  `row_src(r)` gives the global row or -1 (zero row).
template <typename RowSrc>
__device__ __forceinline__ void stage_matrix(uint8_t* s16, float* s32, float* s_n2, const void* base, int is_bf16,
                                             size_t pitch, size_t col0, RowSrc row_src) {
  const int r = threadIdx.x >> 1, hh = threadIdx.x & 1;
  const long long src = row_src(r);
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    __align__(16) __half h[8];
    if (src >= 0) {
      const uint4 raw = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(base) + (size_t)src * pitch + col0 + hh * 64 + c * 8);
      const uint16_t* u = reinterpret_cast<const uint16_t*>(&raw);
#pragma unroll
      for (int q = 0; q < 8; ++q) h[q] = is_bf16 ? __float2half_rn(bf16_bits_to_float(u[q])) : __ushort_as_half(u[q]);
    } else {
#pragma unroll
      for (int q = 0; q < 8; ++q) h[q] = __ushort_as_half((uint16_t)0);
    }
    *reinterpret_cast<uint4*>(s16 + swz256(r, hh * 8 + c)) = *reinterpret_cast<const uint4*>(h);
    float f[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      f[q] = __half2float(h[q]);
      ss = fmaf(f[q], f[q], ss);
    }
    float* dst = s32 + r * kPitch32 + hh * 64 + c * 8;
    *reinterpret_cast<float4*>(dst) = make_float4(f[0], f[1], f[2], f[3]);
    *reinterpret_cast<float4*>(dst + 4) = make_float4(f[4], f[5], f[6], f[7]);
  }
  if (s_n2 != nullptr) {
    ss += __shfl_xor_sync(0xffffffffu, ss, 1);
    if (hh == 0) s_n2[r] = ss;
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

// ---- warp-cooperative exact values --------------------------------------------------------------
// Few elements need their chain value, and which ones differs from lane to lane.  Letting each lane
// compute its own would make the whole warp walk almost every element (divergence); instead the lanes
// put (row, column) of their flagged elements into a per-warp queue, all 32 lanes then take queue
// entries two at a time, and the owners read the results back.
struct WarpQueue {
  uint16_t* entry;   // kQueueCap x (row << 8 | col)
  float* result;     // kQueueCap
};
constexpr int kQueueCap = 512;   // 32 lanes x 16 elements per pass

// `mask`: flagged elements among this lane's v[i0 .. i0+16) (bit i = element i); row = tile row of the lane.
__device__ __forceinline__ void resolve16(const WarpQueue& q, uint32_t mask, int i0, float (&v)[32], int row, int t4,
                                          const float* x32, const float* p32) {
  const int lane = threadIdx.x & 31;
  const int cnt = __popc(mask);
  int incl = cnt;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int n = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= d) incl += n;
  }
  const int total = __shfl_sync(0xffffffffu, incl, 31);
  if (total == 0) return;
  const int off = incl - cnt;
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    const int i = i0 + j;
    if ((mask >> i) & 1u) {
      const int col = 8 * (i >> 1) + 2 * t4 + (i & 1);
      q.entry[off + __popc(mask & ((1u << i) - 1u))] = (uint16_t)((row << 8) | col);
    }
  }
  __syncwarp();
  for (int base = 0; base < total; base += 64) {
    const int e0 = base + lane, e1 = base + 32 + lane;
    const int ent0 = q.entry[min(e0, total - 1)], ent1 = q.entry[min(e1, total - 1)];
    const float* xa = x32 + (ent0 >> 8) * kPitch32;
    const float* pa = p32 + (ent0 & 255) * kPitch32;
    const float* xb = x32 + (ent1 >> 8) * kPitch32;
    const float* pb = p32 + (ent1 & 255) * kPitch32;
    float a0 = 0.f, a1 = 0.f;   // two independent chains per lane
#pragma unroll 4
    for (int k = 0; k < kG; k += 4) {
      const float4 x0 = *reinterpret_cast<const float4*>(xa + k), p0 = *reinterpret_cast<const float4*>(pa + k);
      const float4 x1 = *reinterpret_cast<const float4*>(xb + k), p1 = *reinterpret_cast<const float4*>(pb + k);
      a0 = fmaf(x0.x, p0.x, a0);
      a1 = fmaf(x1.x, p1.x, a1);
      a0 = fmaf(x0.y, p0.y, a0);
      a1 = fmaf(x1.y, p1.y, a1);
      a0 = fmaf(x0.z, p0.z, a0);
      a1 = fmaf(x1.z, p1.z, a1);
      a0 = fmaf(x0.w, p0.w, a0);
      a1 = fmaf(x1.w, p1.w, a1);
    }
    if (e0 < total) q.result[e0] = a0;
    if (e1 < total) q.result[e1] = a1;
  }
  __syncwarp();
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    const int i = i0 + j;
    if ((mask >> i) & 1u) v[i] = q.result[off + __popc(mask & ((1u << i) - 1u))];
  }
  __syncwarp();
}

// One row block: rows [0, rows) of the staged x tile, group g.  `out_row(r)` = destination row.
template <int MODE, typename OutRow>
__device__ void rotq_mma_block(const RotArgs& a, uint8_t* smem, int g, int rows, OutRow out_row) {
  uint8_t* x16 = smem + kOff_x16;
  const uint8_t* p16 = smem + kOff_p16;
  const float* x32 = reinterpret_cast<const float*>(smem + kOff_x32);
  const float* p32 = reinterpret_cast<const float*>(smem + kOff_p32);
  const float* n2 = reinterpret_cast<const float*>(smem + kOff_n2);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int mat = lane >> 3, rr = lane & 7, t4 = lane & 3;
  WarpQueue wq;
  wq.result = reinterpret_cast<float*>(smem + kOff_queue) + warp * kQueueCap;
  wq.entry = reinterpret_cast<uint16_t*>(smem + kOff_queue + 8 * kQueueCap * 4) + warp * kQueueCap;

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
  __syncthreads();  // every warp is done reading x16: it becomes the output staging tile

  constexpr int ROWB = (MODE == DMOQ_A16) ? 256 : (MODE == DMOQ_FP4) ? 64 : 128;  // staged bytes per row
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = warp * 16 + (lane >> 2) + h * 8;
    float v[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = acc[i >> 1][h * 2 + (i & 1)];
    uint8_t* srow = x16 + r * ROWB;

    if (MODE == DMOQ_A16) {
#pragma unroll
      for (int nt = 0; nt < 16; ++nt)
        *reinterpret_cast<__half2*>(srow + (8 * nt + 2 * t4) * 2) = __floats2half2_rn(v[2 * nt], v[2 * nt + 1]);
      continue;
    }
    const float delta = ldexpf(sqrtf(n2[r]), -16) * 1.01f;
    // padding rows and all-zero rows take part in the warp-wide steps but never ask for a chain value
    const bool live = r < rows && n2[r] > 0.f;

    if (MODE == DMOQ_A8 || MODE == DMOQ_FP8) {
      float m = 0.f;
#pragma unroll
      for (int i = 0; i < 32; ++i) m = fmaxf(m, fabsf(v[i]));
      m = quad_max(m);
      const float thr = live ? m - 2.f * delta : 3.0e38f;
      uint32_t exact = 0;
#pragma unroll
      for (int i = 0; i < 32; ++i) exact |= (fabsf(v[i]) >= thr) ? (1u << i) : 0u;
      resolve16(wq, exact & 0xFFFFu, 0, v, r, t4, x32, p32);
      resolve16(wq, exact & 0xFFFF0000u, 16, v, r, t4, x32, p32);
      float cm = 0.f;
#pragma unroll
      for (int i = 0; i < 32; ++i) cm = ((exact >> i) & 1u) ? fmaxf(cm, fabsf(v[i])) : cm;
      const float amax = quad_max(cm);
      const float full = (MODE == DMOQ_A8) ? 127.0f : 448.0f;
      const float tiny = (MODE == DMOQ_A8) ? (float)(1e-8 * 127.0) : (float)(1e-8 * 448.0);
      const float s = (amax < tiny) ? 1e-8f : __fdiv_rn(amax, full);
      const float inv_s = 1.0f / s;
      const float t = delta * inv_s * 1.001f + 3e-5f;   // also covers v*inv_s versus the IEEE quotient v/s
      uint32_t amb = 0;
      if (live) {
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float q0 = v[i] * inv_s, q1 = v[i + 1] * inv_s;
          if (MODE == DMOQ_A8) {
            amb |= (fabsf(q0 - rintf(q0)) > 0.5f - t) ? (1u << i) : 0u;
            amb |= (fabsf(q1 - rintf(q1)) > 0.5f - t) ? (2u << i) : 0u;
          } else {
            const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(q0 - t, q1 - t), __NV_SATFINITE, __NV_E4M3);
            const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(q0 + t, q1 + t), __NV_SATFINITE, __NV_E4M3);
            const uint32_t d = lo ^ hi;
            amb |= (d & 0xFFu) ? (1u << i) : 0u;
            amb |= (d & 0xFF00u) ? (2u << i) : 0u;
          }
        }
        amb &= ~exact;
      }
      resolve16(wq, amb & 0xFFFFu, 0, v, r, t4, x32, p32);
      resolve16(wq, amb & 0xFFFF0000u, 16, v, r, t4, x32, p32);
      exact |= amb;
      uint32_t c[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        // chain values go through the IEEE quotient exactly as the definition does; for the others the
        // test above guarantees that the approximate quotient rounds to the same code
        const float q = ((exact >> i) & 1u) ? __fdiv_rn(v[i], s) : v[i] * inv_s;
        c[i] = live ? ((MODE == DMOQ_A8) ? code_i8(q) : code_e4m3(q)) : 0u;
      }
#pragma unroll
      for (int nt = 0; nt < 16; ++nt)
        *reinterpret_cast<uint16_t*>(srow + 8 * nt + 2 * t4) = (uint16_t)(c[2 * nt] | (c[2 * nt + 1] << 8));
      if (t4 == 0 && r < rows)
        reinterpret_cast<__half*>(a.scales)[(size_t)out_row(r) * (a.o_stride / kG) + g] = __float2half_rn(__fmul_rn(s, a.extra_scale));
    } else {  // FP4: four 32-column blocks per row, 8 values of each block per thread
      float mb[4], thr[4];
      uint32_t exact = 0;
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        float m = 0.f;
#pragma unroll
        for (int i = 8 * b; i < 8 * b + 8; ++i) m = fmaxf(m, fabsf(v[i]));
        mb[b] = quad_max(m);
        thr[b] = live ? mb[b] - 2.f * delta : 3.0e38f;
#pragma unroll
        for (int i = 8 * b; i < 8 * b + 8; ++i) exact |= (fabsf(v[i]) >= thr[b]) ? (1u << i) : 0u;
      }
      resolve16(wq, exact & 0xFFFFu, 0, v, r, t4, x32, p32);
      resolve16(wq, exact & 0xFFFF0000u, 16, v, r, t4, x32, p32);
      uint32_t e_bytes = 0, amb = 0;
      int ei[4];
      float tb[4];
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        float cm = 0.f;
#pragma unroll
        for (int i = 8 * b; i < 8 * b + 8; ++i) cm = ((exact >> i) & 1u) ? fmaxf(cm, fabsf(v[i])) : cm;
        const float amax = fmaxf(quad_max(cm), 1e-30f);
        float e = ceilf((float)log2((double)__fdiv_rn(amax, 6.0f)));
        e = fminf(fmaxf(e, -127.f), 127.f);
        ei[b] = (int)e;
        e_bytes |= (uint32_t)(ei[b] + 127) << (8 * b);
        tb[b] = ldexpf(delta, -ei[b]) * 1.001f + 1e-6f;
        if (live) {
#pragma unroll
          for (int i = 8 * b; i < 8 * b + 8; ++i) {
            const float y = ldexpf(v[i], -ei[b]);
            amb |= (code_e2m1(y - tb[b]) != code_e2m1(y + tb[b])) ? (1u << i) : 0u;
          }
        }
      }
      amb &= ~exact;
      resolve16(wq, amb & 0xFFFFu, 0, v, r, t4, x32, p32);
      resolve16(wq, amb & 0xFFFF0000u, 16, v, r, t4, x32, p32);
#pragma unroll
      for (int i = 0; i < 32; i += 2) {
        const int b = i >> 3;
        const uint32_t n0 = live ? code_e2m1(ldexpf(v[i], -ei[b])) : 0u;
        const uint32_t n1 = live ? code_e2m1(ldexpf(v[i + 1], -ei[b])) : 0u;
        srow[(8 * (i >> 1) + 2 * t4) >> 1] = (uint8_t)(n0 | (n1 << 4));
      }
      if (t4 == 0 && r < rows)
        *reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(a.scales) + (size_t)out_row(r) * (a.o_stride / 32) + g * 4) = e_bytes;
    }
  }
  __syncthreads();
  // ---- coalesced copy-out of the staged codes
  constexpr int CH = ROWB / 16;
  const size_t row_bytes = (MODE == DMOQ_A16) ? (size_t)a.o_stride * 2 : (MODE == DMOQ_FP4) ? (size_t)a.o_stride / 2 : (size_t)a.o_stride;
  for (int i = tid; i < kRows * CH; i += kThreads) {
    const int r = i / CH, ch = i % CH;
    if (r < rows)
      *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(a.codes) + (size_t)out_row(r) * row_bytes + (size_t)g * ROWB + ch * 16) =
          *reinterpret_cast<const uint4*>(x16 + r * ROWB + ch * 16);
  }
  __syncthreads();  // the staging tile is rewritten by the next block's x
}

__device__ __forceinline__ void stage_rotation(uint8_t* smem, const uint16_t* mat) {
  stage_matrix(smem + kOff_p16, reinterpret_cast<float*>(smem + kOff_p32), nullptr, mat, 0, kG, 0,
               [](int r) { return (long long)r; });
}

template <int MODE>
__global__ void __launch_bounds__(kThreads, 1) rotq_mma_rows_kernel(RotArgs a) {
  extern __shared__ __align__(1024) uint8_t smem[];
  const int g = blockIdx.x;
  const int n_rows = a.n_rows_dev ? min(*a.n_rows_dev, a.n_rows) : a.n_rows;
  const int n_blocks = (n_rows + kRows - 1) / kRows;
  if ((int)blockIdx.y >= n_blocks) return;
  stage_rotation(smem, a.rot + (size_t)g * kG * kG);
  for (int b = blockIdx.y; b < n_blocks; b += gridDim.y) {
    const int row0 = b * kRows, rows = min(kRows, n_rows - row0);
    stage_matrix(smem + kOff_x16, reinterpret_cast<float*>(smem + kOff_x32), reinterpret_cast<float*>(smem + kOff_n2),
                 a.x, a.src_is_bf16, (size_t)a.x_stride, (size_t)g * kG, [&](int r) {
                   return r < rows ? (long long)(a.src_row ? a.src_row[row0 + r] : row0 + r) : -1LL;
                 });
    __syncthreads();
    rotq_mma_block<MODE>(a, smem, g, rows, [&](int r) { return row0 + r; });
  }
}

template <int MODE>
__global__ void __launch_bounds__(kThreads, 1) rotq_mma_tiles_kernel(RotArgs a) {
  extern __shared__ __align__(1024) uint8_t smem[];
  const int g = blockIdx.x;
  const int n_tiles = a.n_tiles[a.pool];
  const DmoqTile* tiles = a.tiles + a.n_tiles[DMOQ_MAX_POOLS + a.pool];
  int loaded = -1;
  for (int t = blockIdx.y; t < n_tiles; t += gridDim.y) {
    const DmoqTile tile = tiles[t];
    const int mat = tile.rank * a.groups_per_member + g;
    if (mat != loaded) {
      stage_rotation(smem, a.rot + (size_t)mat * kG * kG);
      loaded = mat;
    }
    for (int r0 = 0; r0 < tile.rows; r0 += kRows) {
      const int row0 = tile.row0 + r0, rows = min(kRows, tile.rows - r0);
      stage_matrix(smem + kOff_x16, reinterpret_cast<float*>(smem + kOff_x32), reinterpret_cast<float*>(smem + kOff_n2),
                   a.x, a.src_is_bf16, (size_t)a.x_stride, (size_t)g * kG,
                   [&](int r) { return r < rows ? (long long)(row0 + r) : -1LL; });
      __syncthreads();
      rotq_mma_block<MODE>(a, smem, g, rows, [&](int r) { return row0 + r; });
    }
  }
}

template <int MODE>
int launch_rows(const RotArgs& a, cudaStream_t s) {
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(rotq_mma_rows_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmem) != cudaSuccess)
      return DMOQ_ELAUNCH;
    configured = true;
  }
  const int G = a.K / kG;
  const int n_blocks = dmoq_ceil_div(a.n_rows, kRows);
  int gy = dmoq_ceil_div(dmoq_sm_count(), G);
  if (gy > n_blocks) gy = n_blocks;
  if (gy < 1) gy = 1;
  rotq_mma_rows_kernel<MODE><<<dim3(G, gy), kThreads, kSmem, s>>>(a);
  return dmoq_launch_status();
}

template <int MODE>
int launch_tiles(const RotArgs& a, int tile_cap, cudaStream_t s) {
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(rotq_mma_tiles_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmem) != cudaSuccess)
      return DMOQ_ELAUNCH;
    configured = true;
  }
  const int G = a.K / kG;
  int gy = dmoq_ceil_div(dmoq_sm_count(), G);
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
