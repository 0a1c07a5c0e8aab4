// Deterministic combine of the routed rows back into token order, the
// group-first relayout kernel, and the small C-ABI utility entry points.
#include "common.cuh"

namespace {

// y[t] = sum over the token's slots (then the shared row) of dn[row], fp32, fixed order.
// Replaces final_hidden_states.index_add_(0, pool_tokens, dn)
// (quantization/wxa16/bit_partitioned_moe.py:966), whose atomic order is not fixed.
// WEIGHTED: dn holds the plain fp16 down-projection outputs and the routing weight is applied here with the
// reference's rounding chain fp16 -> bf16 -> (x weight in fp32) -> bf16 (module :960-965) before the sum.
// Rows are fetched four at a time so that a thread keeps several 16-byte loads in flight.
template <bool WEIGHTED>
__global__ void combine_kernel(const int32_t* __restrict__ row_of, const float* __restrict__ row_weight,
                               const uint16_t* __restrict__ dn, int T, int top_k, int has_shared, int hidden,
                               void* y, int y_is_bf16) {
  const int chunks = hidden / 8;
  const long long total = (long long)T * chunks;
  const int n_src = top_k + (has_shared ? 1 : 0);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(i / chunks), c = (int)(i % chunks);
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int s0 = 0; s0 < n_src; s0 += 4) {
      int row[4];
      uint4 v[4];
      float w[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int s = s0 + k;
        row[k] = -1;
        if (s < n_src) row[k] = (s < top_k) ? row_of[(size_t)t * top_k + s] : row_of[(size_t)T * top_k + t];
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        v[k] = make_uint4(0u, 0u, 0u, 0u);
        w[k] = 0.f;
        if (row[k] >= 0) {
          v[k] = *reinterpret_cast<const uint4*>(dn + (size_t)row[k] * hidden + c * 8);
          if (WEIGHTED) w[k] = row_weight[row[k]];
        }
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        if (row[k] < 0) continue;
        const uint16_t* u = reinterpret_cast<const uint16_t*>(&v[k]);
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          if (WEIGHTED) {
            const float b = __bfloat162float(__float2bfloat16_rn(__half2float(__ushort_as_half(u[q]))));
            acc[q] += __bfloat162float(__float2bfloat16_rn(__fmul_rn(b, w[k])));
          } else {
            acc[q] += bf16_bits_to_float(u[q]);
          }
        }
      }
    }
    __align__(16) uint16_t o[8];
#pragma unroll
    for (int q = 0; q < 8; ++q)
      o[q] = y_is_bf16 ? __bfloat16_as_ushort(__float2bfloat16_rn(acc[q])) : __half_as_ushort(__float2half_rn(acc[q]));
    *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(y) + (size_t)t * hidden + c * 8) =
        *reinterpret_cast<const uint4*>(o);
  }
}

// (N, G*bpg) -> (G, N, bpg), 16-byte granules
__global__ void group_first_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int N, int G, int bpg) {
  const int per_row = bpg / 16;
  const long long total = (long long)N * G * per_row;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int q = (int)(i % per_row);
    const long long ng = i / per_row;
    const int n = (int)(ng % N), g = (int)(ng / N);
    const uint4 v = *reinterpret_cast<const uint4*>(src + ((size_t)n * G + g) * bpg + q * 16);
    *reinterpret_cast<uint4*>(dst + ((size_t)g * N + n) * bpg + q * 16) = v;
  }
}

// every 1- or 2-bit code -> one 4-bit field, low field first; one packed byte per thread and step
template <int BIT>
__global__ void widen_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, long long n_bytes) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n_bytes; i += (long long)gridDim.x * blockDim.x) {
    const uint32_t b = src[i];
    if (BIT == 2) {   // c0 c1 c2 c3 -> bytes (c0 | c1 << 4), (c2 | c3 << 4)
      const uint32_t lo = (b & 3u) | ((b & 0xCu) << 2), hi = ((b >> 4) & 3u) | ((b >> 2) & 0x30u);
      *reinterpret_cast<uint16_t*>(dst + 2 * i) = (uint16_t)(lo | (hi << 8));
    } else {          // eight one-bit codes -> four bytes
      uint32_t w = 0;
#pragma unroll
      for (int k = 0; k < 8; ++k) w |= ((b >> k) & 1u) << (4 * k);
      *reinterpret_cast<uint32_t*>(dst + 4 * i) = w;
    }
  }
}

}  // namespace

extern "C" int dmoq_widen_indices(const uint8_t* packed, int64_t n_bytes, int32_t bit, uint8_t* wide, void* stream) {
  DMOQ_CHECK_ARG(packed && wide && n_bytes >= 0 && (bit == 1 || bit == 2));
  if (n_bytes == 0) return DMOQ_OK;
  long long blocks = (n_bytes + 255) / 256;
  const long long cap = 16LL * dmoq_sm_count();
  if (blocks > cap) blocks = cap;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (bit == 2) widen_kernel<2><<<(int)blocks, 256, 0, s>>>(packed, wide, n_bytes);
  else widen_kernel<1><<<(int)blocks, 256, 0, s>>>(packed, wide, n_bytes);
  return dmoq_launch_status();
}

static int launch_combine(const dmoq_route_t* route, const uint16_t* dn, int32_t hidden, void* y, int32_t y_is_bf16,
                          bool weighted, void* stream) {
  DMOQ_CHECK_ARG(route && dn && y && route->row_of);
  DMOQ_CHECK_ARG(hidden > 0 && hidden % 8 == 0);
  DMOQ_CHECK_ARG(!weighted || route->sorted_weights);
  if (route->T == 0) return DMOQ_OK;
  const long long total = (long long)route->T * (hidden / 8);
  long long blocks = (total + 255) / 256;
  // one block per 256 chunks, far more blocks than resident slots on purpose: blocks then sweep the tokens in order
  // (measured faster than a grid-stride loop over a grid of the resident blocks: 0.33 against 0.36-0.38 ms)
  const long long cap = 1024LL * dmoq_sm_count();
  if (blocks > cap) blocks = cap;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (weighted)
    combine_kernel<true><<<(int)blocks, 256, 0, s>>>(route->row_of, route->sorted_weights, dn, route->T, route->top_k,
                                                     route->has_shared, hidden, y, y_is_bf16);
  else
    combine_kernel<false><<<(int)blocks, 256, 0, s>>>(route->row_of, nullptr, dn, route->T, route->top_k,
                                                      route->has_shared, hidden, y, y_is_bf16);
  return dmoq_launch_status();
}

extern "C" int dmoq_combine(const dmoq_route_t* route, const uint16_t* dn, int32_t hidden,
                            void* y, int32_t y_is_bf16, void* stream) {
  return launch_combine(route, dn, hidden, y, y_is_bf16, false, stream);
}

extern "C" int dmoq_combine_weighted(const dmoq_route_t* route, const uint16_t* dn_f16, int32_t hidden,
                                     void* y, int32_t y_is_bf16, void* stream) {
  return launch_combine(route, dn_f16, hidden, y, y_is_bf16, true, stream);
}

extern "C" int dmoq_convert_group_first(const uint8_t* row_major, int32_t N, int32_t K, int32_t bit,
                                        uint8_t* group_first, void* stream) {
  DMOQ_CHECK_ARG(row_major && group_first);
  DMOQ_CHECK_ARG(bit == 1 || bit == 2 || bit == 4 || bit == 8);
  DMOQ_CHECK_ARG(N > 0 && K > 0 && K % DMOQ_GROUP == 0);
  const int G = K / DMOQ_GROUP, bpg = 16 * bit;
  const long long total = (long long)N * G * (bpg / 16);
  long long blocks = (total + 255) / 256;
  const long long cap = 16LL * dmoq_sm_count();
  if (blocks > cap) blocks = cap;
  group_first_kernel<<<(int)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(row_major, group_first, N, G, bpg);
  return dmoq_launch_status();
}

// Rows of one pool's activation-code table gathered into routed-row order: dst row r = src row a_row[r] for every row
// r of the pool's tiles.  One warp per row, 16-byte chunks; the few scale bytes of a row go along.
__global__ void __launch_bounds__(256) gather_rows_kernel(const DmoqTile* __restrict__ tiles, const int32_t* __restrict__ n_tiles,
                                                          int pool, const int32_t* __restrict__ a_row,
                                                          const uint8_t* __restrict__ src, int src_pitch, int row_bytes,
                                                          uint8_t* __restrict__ dst, int dst_pitch,
                                                          const uint8_t* __restrict__ ssrc, int ssrc_pitch, int scale_bytes,
                                                          uint8_t* __restrict__ sdst, int sdst_pitch) {
  const int n = n_tiles[pool];
  const DmoqTile* mine = tiles + n_tiles[DMOQ_MAX_POOLS + pool];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
  for (int t = blockIdx.x; t < n; t += gridDim.x) {
    const DmoqTile tile = mine[t];
    for (int r = warp; r < tile.rows; r += n_warps) {
      const size_t to = (size_t)(tile.row0 + r), from = (size_t)a_row[tile.row0 + r];
      for (int c = lane * 16; c < row_bytes; c += 512)
        *reinterpret_cast<uint4*>(dst + to * dst_pitch + c) = *reinterpret_cast<const uint4*>(src + from * src_pitch + c);
      if (ssrc != nullptr)
        for (int c = lane * 2; c < scale_bytes; c += 64)
          *reinterpret_cast<uint16_t*>(sdst + to * sdst_pitch + c) = *reinterpret_cast<const uint16_t*>(ssrc + from * ssrc_pitch + c);
    }
  }
}

extern "C" int dmoq_gather_rows(const dmoq_route_t* route, int32_t pool_index, const void* src_codes,
                                int32_t src_pitch_bytes, int32_t row_bytes, void* dst_codes, int32_t dst_pitch_bytes,
                                const void* src_scales, int32_t src_scale_pitch, int32_t scale_bytes, void* dst_scales,
                                int32_t dst_scale_pitch, void* stream) {
  DMOQ_CHECK_ARG(route && src_codes && dst_codes && route->a_row && route->tiles && route->n_tiles);
  DMOQ_CHECK_ARG(pool_index >= 0 && pool_index < route->n_pools);
  DMOQ_CHECK_ARG(row_bytes > 0 && row_bytes % 16 == 0 && src_pitch_bytes % 16 == 0 && dst_pitch_bytes % 16 == 0);
  DMOQ_CHECK_ARG(src_pitch_bytes >= row_bytes && dst_pitch_bytes >= row_bytes);
  DMOQ_CHECK_ARG((src_scales == nullptr) == (dst_scales == nullptr));
  DMOQ_CHECK_ARG(src_scales == nullptr || (scale_bytes > 0 && scale_bytes % 2 == 0 && src_scale_pitch % 2 == 0 && dst_scale_pitch % 2 == 0));
  int blocks = route->tile_cap;
  const int cap = 8 * dmoq_sm_count();
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  gather_rows_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const DmoqTile*>(route->tiles), route->n_tiles, pool_index, route->a_row,
      static_cast<const uint8_t*>(src_codes), src_pitch_bytes, row_bytes, static_cast<uint8_t*>(dst_codes), dst_pitch_bytes,
      static_cast<const uint8_t*>(src_scales), src_scale_pitch, scale_bytes, static_cast<uint8_t*>(dst_scales), dst_scale_pitch);
  return dmoq_launch_status();
}

extern "C" int dmoq_version(void) { return DMOQ_VERSION; }

extern "C" const char* dmoq_strerror(int code) {
  switch (code) {
    case DMOQ_OK: return "ok";
    case DMOQ_EINVAL: return "invalid argument";
    case DMOQ_ELAUNCH: return "CUDA launch or attribute call failed";
    case DMOQ_ESIZE: return "size exceeds a stated maximum or a buffer is too small";
    case DMOQ_EDEVICE: return "no usable CUDA device or device symbol set-up failed";
    default: return "unknown dmoq error";
  }
}
