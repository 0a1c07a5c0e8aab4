// Weight images: a pool's packed codebook indices looked up once and written as tensor-core operand rows.
//
//   source   group-first indices (G, N, 16*bit) bytes and norms (G, N) fp16, N = source rows
//            (turboquant_utils/triton_kernels.py:1042 layout)
//   image    A8 / FP8   (G, N, 128) one-byte codewords (int8 table of triton_kernels_a8.py:526, or index-128 for the
//                       uniform 8-bit codebook; e4m3 table of triton_kernels_fp8.py:35)
//            A16        (G, N, 128) fp16 codewords
//            FP4        (ceil(G/2), N, 128 bytes): bytes [0,64) = group 2j, [64,128) = group 2j+1, two e2m1 nibbles per
//                       byte with the even column in the low nibble -- the reference's load-time fold of the codebook
//                       into e2m1 (triton_kernels_fp4.py:80-127), two groups side by side so that one 128-byte
//                       operand row feeds two block-scaled MMAs
//   norms    (G, N) fp32 in image row order
// Image row order: down projections keep the source order.  gate_up images interleave each member's gate and up
// rows in runs of 16 (image rows 32c..32c+15 = gate rows 16c.., 32c+16..32c+31 = up rows 16c..), so that the 32
// accumulator columns one epilogue thread owns hold the gate and the up value of the same 16 outputs.
#include "common.cuh"

namespace {

struct ExpandArgs {
  const uint8_t* idx;      // (G, N, 16*bit)
  const uint16_t* norm;    // (G, N) fp16
  const void* lut;
  int bit, mode, identity;
  int G, N;
  int inter;               // gate_up: rows per member = 2*inter, interleaved; 0 = keep the source order (down)
  void* image;
  float* norm_img;
  float norm_scale;        // the INT8 image norms carry 2^49 (see dmoq.h: the GEMM reads biased sums as denormals)
};

__device__ __forceinline__ int source_row(int n_img, int inter) {
  if (inter == 0) return n_img;
  const int per = 2 * inter;
  const int m = n_img / per, r = n_img % per;
  const int run = r >> 5, within = r & 31;            // 32 image rows = 16 gate + 16 up
  return m * per + (within < 16 ? run * 16 + within : inter + run * 16 + within - 16);
}

template <int BIT>
__global__ void __launch_bounds__(256) expand_kernel(ExpandArgs a) {
  __shared__ uint16_t s_lut[256];
  const int entries = 1 << BIT;
  for (int i = threadIdx.x; i < entries; i += blockDim.x) {
    uint16_t v;
    if (a.mode == DMOQ_A16) v = reinterpret_cast<const uint16_t*>(a.lut)[i];
    else if (a.identity) v = (uint16_t)(uint8_t)(i - 128);
    else v = reinterpret_cast<const uint8_t*>(a.lut)[i];
    s_lut[i] = v;
  }
  __syncthreads();
  constexpr int BPC = 2 * BIT;                         // packed bytes per 16-element chunk
  const long long total = (long long)a.G * a.N * 8;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i & 7);
    const long long gn = i >> 3;
    const int n = (int)(gn % a.N), g = (int)(gn / a.N);
    const int ns = source_row(n, a.inter);
    const uint8_t* src = a.idx + ((size_t)g * a.N + ns) * (16 * BIT) + c * BPC;
    uint32_t raw[BPC / 4 > 0 ? BPC / 4 : 1];
    if (BPC >= 4) {
#pragma unroll
      for (int q = 0; q < BPC / 4; ++q) raw[q] = reinterpret_cast<const uint32_t*>(src)[q];
    } else {
      raw[0] = *reinterpret_cast<const uint16_t*>(src);
    }
    uint16_t cw[16];
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      const int bitpos = k * BIT;
      const uint32_t code = (raw[bitpos >> 5] >> (bitpos & 31)) & (uint32_t)(entries - 1);
      cw[k] = s_lut[code];
    }
    if (a.mode == DMOQ_A16) {
      uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(a.image) + ((size_t)g * a.N + n) * 128 + c * 16);
      uint32_t w[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) w[q] = (uint32_t)cw[2 * q] | ((uint32_t)cw[2 * q + 1] << 16);
      dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
      dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
    } else if (a.mode == DMOQ_FP4) {
      uint32_t w[2] = {0u, 0u};
#pragma unroll
      for (int k = 0; k < 16; ++k) w[k >> 3] |= (uint32_t)(cw[k] & 15u) << (4 * (k & 7));
      uint8_t* dst = reinterpret_cast<uint8_t*>(a.image) + ((size_t)(g >> 1) * a.N + n) * 128 + (g & 1) * 64 + c * 8;
      *reinterpret_cast<uint2*>(dst) = make_uint2(w[0], w[1]);
    } else {
      uint32_t w[4] = {0u, 0u, 0u, 0u};
#pragma unroll
      for (int k = 0; k < 16; ++k) w[k >> 2] |= (uint32_t)(cw[k] & 255u) << (8 * (k & 3));
      uint8_t* dst = reinterpret_cast<uint8_t*>(a.image) + ((size_t)g * a.N + n) * 128 + c * 16;
      *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
    }
    if (c == 0 && a.norm_img != nullptr)
      a.norm_img[(size_t)g * a.N + n] = __half2float(__ushort_as_half(a.norm[(size_t)g * a.N + ns])) * a.norm_scale;
  }
}

}  // namespace

extern "C" size_t dmoq_weight_image_bytes(const dmoq_pool_t* pool, int32_t is_down, int32_t hidden) {
  if (pool == nullptr || pool->inter <= 0 || hidden <= 0 || pool->inter % 128 || hidden % 128) return 0;
  const size_t G = is_down ? (size_t)pool->n_members * pool->inter / 128 : (size_t)hidden / 128;
  const size_t N = is_down ? (size_t)hidden : (size_t)pool->n_members * 2 * pool->inter;
  switch (pool->mode) {
    case DMOQ_A16: return G * N * 256;
    case DMOQ_A8:
    case DMOQ_FP8: return G * N * 128;
    case DMOQ_FP4: return ((G + 1) / 2) * N * 128;
    default: return 0;
  }
}

extern "C" int dmoq_expand_weights(const dmoq_pool_t* pool, int32_t is_down, int32_t hidden, void* image,
                                   float* norm_image, void* stream) {
  DMOQ_CHECK_ARG(pool && image);
  const dmoq_pool_t& p = *pool;
  DMOQ_CHECK_ARG(p.inter > 0 && p.inter % 128 == 0 && hidden > 0 && hidden % 128 == 0 && p.n_members > 0);
  DMOQ_CHECK_ARG(p.bit == 1 || p.bit == 2 || p.bit == 4 || p.bit == 8);
  DMOQ_CHECK_ARG(p.mode >= DMOQ_A16 && p.mode <= DMOQ_FP4);
  ExpandArgs a{};
  a.idx = is_down ? p.dn_idx : p.gu_idx;
  a.norm = is_down ? p.dn_norm : p.gu_norm;
  a.lut = is_down ? p.dn_lut : p.gu_lut;
  a.bit = p.bit;
  a.mode = p.mode;
  a.identity = (p.mode == DMOQ_A8 && p.identity_lut) ? 1 : 0;
  DMOQ_CHECK_ARG(a.idx && (a.norm || norm_image == nullptr) && (a.lut || a.identity));
  DMOQ_CHECK_ARG(!(p.mode == DMOQ_FP4 && p.bit == 8));
  a.G = is_down ? p.n_members * p.inter / 128 : hidden / 128;
  a.N = is_down ? hidden : p.n_members * 2 * p.inter;
  a.inter = is_down ? 0 : p.inter;
  a.image = image;
  a.norm_img = norm_image;
  a.norm_scale = (p.mode == DMOQ_A8) ? DMOQ_A8_NORM_IMAGE_SCALE : 1.0f;
  const long long total = (long long)a.G * a.N * 8;
  long long blocks = (total + 255) / 256;
  const long long cap = 32LL * dmoq_sm_count();
  if (blocks > cap) blocks = cap;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (p.mode == DMOQ_FP4 && (a.G & 1)) {   // the unpaired half of the last image row group must not hold stale bytes
    if (cudaMemsetAsync(static_cast<uint8_t*>(image) + (size_t)(a.G / 2) * a.N * 128, 0, (size_t)a.N * 128, s) != cudaSuccess)
      return DMOQ_ELAUNCH;
  }
  switch (p.bit) {
    case 1: expand_kernel<1><<<(int)blocks, 256, 0, s>>>(a); break;
    case 2: expand_kernel<2><<<(int)blocks, 256, 0, s>>>(a); break;
    case 4: expand_kernel<4><<<(int)blocks, 256, 0, s>>>(a); break;
    default: expand_kernel<8><<<(int)blocks, 256, 0, s>>>(a); break;
  }
  return dmoq_launch_status();
}
