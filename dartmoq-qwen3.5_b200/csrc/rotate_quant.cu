// Group rotation fused with activation quantisation.
//
// One CTA owns one 128-column group and walks row blocks of 64 rows with the
// group's rotation resident in shared memory.  Each output value is a
// sequential fp32 FMA chain over k = 0..127 (fp16 x fp16 products are exact in
// fp32), so int8 / e4m3 / e2m1 codes and stored scales can be reproduced bit
// for bit on a CPU.  Quantisation rules follow
//   int8       turboquant_utils/triton_kernels_a8.py:429-484
//   e4m3       turboquant_utils/triton_kernels_fp8.py:128-187
//   e2m1+e8m0  turboquant_utils/triton_kernels_fp4.py:1036-1104
// and the unquantised fp16 output stands in for rotation.py:176 (batch_rotate_input).
#include <cstdlib>

#include "common.cuh"
#include "rotq.cuh"

namespace {

constexpr int kG = DMOQ_GROUP;  // 128
constexpr int kRows = 64;       // rows per block
constexpr int kThreads = 128;   // 16 column groups x 8 row groups, 8x8 outputs per thread
constexpr int kPPitch = kG + 4; // padded pitch of the transposed rotation (floats)
constexpr int kXPitch = kRows + 4;


__device__ __forceinline__ void load_rotation(float* s_p, const uint16_t* rot_mat) {
  // s_p[k][j] = P[j][k]
  const __half* p = reinterpret_cast<const __half*>(rot_mat);
  for (int i = threadIdx.x; i < kG * kG / 8; i += kThreads) {
    const int j = i / (kG / 8);
    const int k0 = (i % (kG / 8)) * 8;
    uint4 v = *reinterpret_cast<const uint4*>(p + (size_t)j * kG + k0);
    const __half* h = reinterpret_cast<const __half*>(&v);
#pragma unroll
    for (int q = 0; q < 8; ++q) s_p[(k0 + q) * kPPitch + j] = __half2float(h[q]);
  }
}

__device__ __forceinline__ float2 fma2_rn(float2 a, float2 b, float2 c) {
  float2 d;
  asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tmov.b64 rc, {%6, %7};\n\t"
      "fma.rn.f32x2 rd, ra, rb, rc;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d.x), "=f"(d.y)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
  return d;
}

__device__ __forceinline__ uint8_t e2m1_nibble(float y) {
  float a = fabsf(y);
  uint8_t mag = a < 0.25f ? 0 : a < 0.75f ? 1 : a < 1.25f ? 2 : a < 1.75f ? 3 : a < 2.5f ? 4 : a < 3.5f ? 5 : a < 5.0f ? 6 : 7;
  return mag | (y < 0.f ? 8 : 0);
}

// Rotates + quantises rows [row0, row0+rows) (rows <= 64) of group g.
// out_row(i) = first_out_row + i;  source row = src_row ? src_row[out_row] : out_row.
template <int MODE>
__device__ void rotq_block(const RotArgs& a, const float* s_p, float* s_x, int g, int row0, int rows) {
  const int tid = threadIdx.x;
  // ---- stage x: thread -> (row, 64-column half); s_x[k][row]
  {
    const int r = tid % kRows;
    const int kh = tid / kRows;
    const bool valid = r < rows;
    size_t src = 0;
    if (valid) src = a.src_row ? (size_t)a.src_row[row0 + r] : (size_t)(row0 + r);
    const size_t base = src * (size_t)a.x_stride + (size_t)g * kG + kh * 64;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      float v[8];
      if (valid) {
        uint4 raw = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(a.x) + base + c * 8);
        const uint16_t* u = reinterpret_cast<const uint16_t*>(&raw);
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          if (a.src_is_bf16) {
            v[q] = __half2float(__float2half_rn(bf16_bits_to_float(u[q])));
          } else {
            v[q] = __half2float(__ushort_as_half(u[q]));
          }
        }
      } else {
#pragma unroll
        for (int q = 0; q < 8; ++q) v[q] = 0.f;
      }
#pragma unroll
      for (int q = 0; q < 8; ++q) s_x[(kh * 64 + c * 8 + q) * kXPitch + r] = v[q];
    }
  }
  __syncthreads();

  // ---- 8x8 outputs per thread, sequential in k.  Two neighbouring columns share one packed FMA
  // (fma.rn.f32x2: each half is an ordinary round-to-nearest fma, so every output is still its own chain).
  const int tx = tid % 16, ty = tid / 16;
  float2 acc2[8][4];
#pragma unroll
  for (int r = 0; r < 8; ++r)
#pragma unroll
    for (int c = 0; c < 4; ++c) acc2[r][c] = make_float2(0.f, 0.f);
#pragma unroll 4
  for (int k = 0; k < kG; ++k) {
    const float4 x0 = *reinterpret_cast<const float4*>(&s_x[k * kXPitch + ty * 8]);
    const float4 x1 = *reinterpret_cast<const float4*>(&s_x[k * kXPitch + ty * 8 + 4]);
    const float4 p0 = *reinterpret_cast<const float4*>(&s_p[k * kPPitch + tx * 8]);
    const float4 p1 = *reinterpret_cast<const float4*>(&s_p[k * kPPitch + tx * 8 + 4]);
    const float xv[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
    const float2 pv[4] = {make_float2(p0.x, p0.y), make_float2(p0.z, p0.w), make_float2(p1.x, p1.y), make_float2(p1.z, p1.w)};
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      const float2 xx = make_float2(xv[r], xv[r]);
#pragma unroll
      for (int c = 0; c < 4; ++c) acc2[r][c] = fma2_rn(xx, pv[c], acc2[r][c]);
    }
  }
  float acc[8][8];
#pragma unroll
  for (int r = 0; r < 8; ++r)
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      acc[r][2 * c] = acc2[r][c].x;
      acc[r][2 * c + 1] = acc2[r][c].y;
    }
  __syncthreads();  // s_x may be overwritten by the next block

  const int G = a.o_stride / kG;
#pragma unroll
  for (int r = 0; r < 8; ++r) {
    const int lr = ty * 8 + r;
    const int orow = row0 + lr;
    const bool valid = lr < rows;
    float amax = 0.f;
#pragma unroll
    for (int c = 0; c < 8; ++c) amax = fmaxf(amax, fabsf(acc[r][c]));

    if (MODE == DMOQ_A16) {
      if (valid) {
        __align__(16) __half h[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) h[c] = __float2half_rn(acc[r][c]);
        *reinterpret_cast<uint4*>(reinterpret_cast<__half*>(a.codes) + (size_t)orow * a.o_stride + g * kG + tx * 8) =
            *reinterpret_cast<const uint4*>(h);
      }
    } else if (MODE == DMOQ_A8 || MODE == DMOQ_FP8) {
#pragma unroll
      for (int m = 1; m < 16; m <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
      const float full = (MODE == DMOQ_A8) ? 127.0f : 448.0f;
      const float tiny = (MODE == DMOQ_A8) ? (float)(1e-8 * 127.0) : (float)(1e-8 * 448.0);
      const float s = (amax < tiny) ? 1e-8f : __fdiv_rn(amax, full);
      __align__(8) uint8_t q[8];
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const float v = __fdiv_rn(acc[r][c], s);
        if (MODE == DMOQ_A8) {
          q[c] = (uint8_t)(int8_t)fminf(fmaxf(roundf(v), -127.f), 127.f);
        } else {
          q[c] = (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
        }
      }
      if (valid) {
        *reinterpret_cast<uint2*>(reinterpret_cast<uint8_t*>(a.codes) + (size_t)orow * a.o_stride + g * kG + tx * 8) =
            *reinterpret_cast<const uint2*>(q);
        if (tx == 0)
          reinterpret_cast<__half*>(a.scales)[(size_t)orow * G + g] = __float2half_rn(__fmul_rn(s, a.extra_scale));
      }
    } else {  // FP4: 32-column blocks = 4 threads
#pragma unroll
      for (int m = 1; m < 4; m <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
      amax = fmaxf(amax, 1e-30f);
      // e = ceil(log2(amax/6)) with log2 rounded to fp32 once
      float e = ceilf((float)log2((double)__fdiv_rn(amax, 6.0f)));
      e = fminf(fmaxf(e, -127.f), 127.f);
      uint32_t word = 0;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        float y = ldexpf(acc[r][c], -(int)e);
        y = fminf(fmaxf(y, -6.f), 6.f);
        word |= (uint32_t)e2m1_nibble(y) << (4 * c);
      }
      if (valid) {
        *reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(a.codes) + (size_t)orow * (a.o_stride / 2) + (g * kG + tx * 8) / 2) = word;
        if ((tx & 3) == 0)
          reinterpret_cast<uint8_t*>(a.scales)[(size_t)orow * (a.o_stride / 32) + g * 4 + tx / 4] = (uint8_t)(int)(e + 127.f);
      }
    }
  }
}

template <int MODE>
__global__ void __launch_bounds__(kThreads) rotq_rows_kernel(RotArgs a) {
  extern __shared__ __align__(16) float s_mem[];
  float* s_p = s_mem;
  float* s_x = s_mem + kG * kPPitch;
  const int g = blockIdx.x;
  const int n_rows = a.n_rows_dev ? min(*a.n_rows_dev, a.n_rows) : a.n_rows;
  const int n_blocks = (n_rows + kRows - 1) / kRows;
  if ((int)blockIdx.y >= n_blocks) return;
  load_rotation(s_p, a.rot + (size_t)g * kG * kG);
  __syncthreads();
  for (int b = blockIdx.y; b < n_blocks; b += gridDim.y)
    rotq_block<MODE>(a, s_p, s_x, g, b * kRows, min(kRows, n_rows - b * kRows));
}

template <int MODE>
__global__ void __launch_bounds__(kThreads) rotq_tiles_kernel(RotArgs a) {
  extern __shared__ __align__(16) float s_mem[];
  float* s_p = s_mem;
  float* s_x = s_mem + kG * kPPitch;
  const int g = blockIdx.x;
  const int n_tiles = a.n_tiles[a.pool];
  const DmoqTile* tiles = a.tiles + a.n_tiles[DMOQ_MAX_POOLS + a.pool];
  int loaded = -1;
  for (int t = blockIdx.y; t < n_tiles; t += gridDim.y) {
    const DmoqTile tile = tiles[t];
    const int mat = a.expert_rank[tile.expert] * a.groups_per_member + g;
    if (mat != loaded) {
      __syncthreads();
      load_rotation(s_p, a.rot + (size_t)mat * kG * kG);
      loaded = mat;
      __syncthreads();
    }
    for (int r = 0; r < tile.rows; r += kRows)
      rotq_block<MODE>(a, s_p, s_x, g, tile.row0 + r, min(kRows, tile.rows - r));
  }
}

constexpr size_t kSmemBytes = (size_t)(kG * kPPitch + kG * kXPitch) * sizeof(float);

template <int MODE>
int launch_rows(const RotArgs& a, cudaStream_t s) {
  static DmoqOncePerDevice once;
  bool* configured = once.slot();
  if (configured == nullptr) return DMOQ_EDEVICE;
  if (!*configured) {
    if (cudaFuncSetAttribute(rotq_rows_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes) != cudaSuccess)
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
  rotq_rows_kernel<MODE><<<dim3(G, gy), kThreads, kSmemBytes, s>>>(a);
  return dmoq_launch_status();
}

template <int MODE>
int launch_tiles(const RotArgs& a, int tile_cap, cudaStream_t s) {
  static DmoqOncePerDevice once;
  bool* configured = once.slot();
  if (configured == nullptr) return DMOQ_EDEVICE;
  if (!*configured) {
    if (cudaFuncSetAttribute(rotq_tiles_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes) != cudaSuccess)
      return DMOQ_ELAUNCH;
    *configured = true;
  }
  const int G = a.K / kG;
  // two blocks are resident per SM: the grid must not exceed those slots, or the blocks left over run alone
  // after the others have finished their whole share of row blocks
  int gy = (2 * dmoq_sm_count()) / G;
  if (gy > tile_cap) gy = tile_cap;
  if (gy < 1) gy = 1;
  rotq_tiles_kernel<MODE><<<dim3(G, gy), kThreads, kSmemBytes, s>>>(a);
  return dmoq_launch_status();
}

// The tensor-core kernel with exact fix-up is the default; DMOQ_ROTQ=chain computes every value on the CUDA-core
// FMA chain instead (same codes, for A/B runs).  The unquantised fp16 rotation always uses the tensor cores.
bool use_mma_rotation() {
  static int cached = -1;
  if (cached < 0) {
    const char* v = getenv("DMOQ_ROTQ");
    cached = (v && v[0] == 'c') ? 0 : 1;
  }
  return cached == 1;
}

}  // namespace

int dmoq_sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

extern "C" int dmoq_rotate_quant(int32_t mode, const void* x, int32_t src_is_bf16, int32_t K,
                                 const uint16_t* rot, const int32_t* rot_row_group0,
                                 const int32_t* src_row, int32_t n_rows, const int32_t* n_rows_dev,
                                 float extra_scale, void* codes, void* scales, void* stream) {
  DMOQ_CHECK_ARG(x && rot && codes);
  DMOQ_CHECK_ARG(K > 0 && K % kG == 0 && n_rows >= 0);
  DMOQ_CHECK_ARG(rot_row_group0 == nullptr);  // per-row rotation bases go through dmoq_rotate_quant_down
  DMOQ_CHECK_ARG(mode == DMOQ_A16 || scales);
  if (n_rows == 0) return DMOQ_OK;
  RotArgs a{};
  a.x = x;
  a.src_is_bf16 = src_is_bf16;
  a.K = K;
  a.x_stride = K;
  a.o_stride = K;
  a.rot = rot;
  a.src_row = src_row;
  a.n_rows = n_rows;
  a.n_rows_dev = n_rows_dev;
  a.extra_scale = extra_scale;
  a.codes = codes;
  a.scales = scales;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (mode == DMOQ_A16 || use_mma_rotation()) return dmoq_rotq_mma_rows(mode, a, s);
  switch (mode) {
    case DMOQ_A16: return launch_rows<DMOQ_A16>(a, s);
    case DMOQ_A8: return launch_rows<DMOQ_A8>(a, s);
    case DMOQ_FP8: return launch_rows<DMOQ_FP8>(a, s);
    case DMOQ_FP4: return launch_rows<DMOQ_FP4>(a, s);
    default: return DMOQ_EINVAL;
  }
}

extern "C" int dmoq_rotate_quant_down(const dmoq_route_t* route, const dmoq_pool_t* pools_host, int32_t pool_index,
                                      const uint16_t* act, int32_t act_stride, void* codes, void* scales,
                                      int32_t code_stride, void* stream) {
  DMOQ_CHECK_ARG(route && pools_host && act && codes);
  DMOQ_CHECK_ARG(pool_index >= 0 && pool_index < route->n_pools);
  const dmoq_pool_t& p = pools_host[pool_index];
  DMOQ_CHECK_ARG(p.inter > 0 && p.inter % kG == 0 && p.dn_rot);
  DMOQ_CHECK_ARG(p.mode == DMOQ_A16 || scales);
  RotArgs a{};
  a.x = act;
  a.src_is_bf16 = 0;
  DMOQ_CHECK_ARG(act_stride >= p.inter && act_stride % 8 == 0 && code_stride >= p.inter && code_stride % kG == 0);
  a.K = p.inter;
  a.x_stride = act_stride;
  a.o_stride = code_stride;
  a.rot = p.dn_rot;
  a.extra_scale = p.dn_act_scale;
  a.codes = codes;
  a.scales = scales;
  a.tiles = reinterpret_cast<const DmoqTile*>(route->tiles);
  a.n_tiles = route->n_tiles;
  a.expert_rank = route->expert_rank;
  a.pool = pool_index;
  a.groups_per_member = p.inter / kG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (p.mode == DMOQ_A16 || use_mma_rotation()) return dmoq_rotq_mma_tiles(p.mode, a, route->tile_cap, s);
  switch (p.mode) {
    case DMOQ_A16: return launch_tiles<DMOQ_A16>(a, route->tile_cap, s);
    case DMOQ_A8: return launch_tiles<DMOQ_A8>(a, route->tile_cap, s);
    case DMOQ_FP8: return launch_tiles<DMOQ_FP8>(a, route->tile_cap, s);
    case DMOQ_FP4: return launch_tiles<DMOQ_FP4>(a, route->tile_cap, s);
    default: return DMOQ_EINVAL;
  }
}
