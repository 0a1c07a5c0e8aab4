// Offline quantiser of the packed format as a device kernel (the reference runs it as torch ops:
// turboquant_utils/quantize.py:350-472).  Per 128-column group and row: L2 norm (>= 1e-8), normalise, rotate by the
// group's orthogonal matrix, scale by sqrt(128), bucket into the codebook's cells (count of cell edges below the
// value, as torch.searchsorted does), pack the indices little-endian within each byte.  The arithmetic is fp32 in a
// fixed order (sequential over the 128 columns), so results are reproducible run to run; against a BLAS-ordered
// evaluation an index can differ only where a rotated value falls within rounding of a cell edge.
#include "common.cuh"

namespace {

constexpr int kG = DMOQ_GROUP;
constexpr int kRows = 64;        // rows per block
constexpr int kThreads = 256;

struct QuantArgs {
  const void* w;            // (N, K) fp32 / fp16 / bf16
  int w_kind;               // 0 fp32, 1 fp16, 2 bf16
  int N, K, bit;
  const float* rot;         // (G, 128, 128) fp32: matrix of group g, used as y = w_normalised @ rot[g]^T
  const float* edges;       // (2^bit - 1) ascending cell edges
  uint8_t* packed;          // (N, K*bit/8)
  uint16_t* norms;          // (N, G) fp16
};

__device__ __forceinline__ float load_w(const QuantArgs& a, size_t i) {
  if (a.w_kind == 0) return reinterpret_cast<const float*>(a.w)[i];
  if (a.w_kind == 1) return __half2float(reinterpret_cast<const __half*>(a.w)[i]);
  return bf16_bits_to_float(reinterpret_cast<const uint16_t*>(a.w)[i]);
}

__global__ void __launch_bounds__(kThreads) quantize_kernel(QuantArgs a) {
  extern __shared__ __align__(16) uint8_t smem[];
  float* s_rot_t = reinterpret_cast<float*>(smem);                 // [k][j] = rot[j][k]
  float* s_w = s_rot_t + kG * kG;                                  // [r][k], normalised
  float* s_edges = s_w + kRows * kG;                               // up to 255
  uint8_t* s_code = reinterpret_cast<uint8_t*>(s_edges + 256);     // [r][j]
  const int g = blockIdx.y, row0 = blockIdx.x * kRows, tid = threadIdx.x;
  const int G = a.K / kG, n_edges = (1 << a.bit) - 1;
  const float* rot = a.rot + (size_t)g * kG * kG;
  for (int i = tid; i < kG * kG; i += kThreads) s_rot_t[(i & 127) * kG + (i >> 7)] = rot[i];
  for (int i = tid; i < n_edges; i += kThreads) s_edges[i] = a.edges[i];
  for (int i = tid; i < kRows * kG; i += kThreads) {
    const int r = i >> 7, k = i & 127;
    s_w[i] = (row0 + r < a.N) ? load_w(a, (size_t)(row0 + r) * a.K + g * kG + k) : 0.f;
  }
  __syncthreads();
  if (tid < kRows) {   // row norms, then normalise in place
    float ss = 0.f;
    for (int k = 0; k < kG; ++k) ss = fmaf(s_w[tid * kG + k], s_w[tid * kG + k], ss);
    const float nrm = fmaxf(sqrtf(ss), 1e-8f);
    if (row0 + tid < a.N) a.norms[(size_t)(row0 + tid) * G + g] = __half_as_ushort(__float2half_rn(nrm));
    for (int k = 0; k < kG; ++k) s_w[tid * kG + k] = __fdiv_rn(s_w[tid * kG + k], nrm);
  }
  __syncthreads();
  const int j = tid & 127, half = tid >> 7;
  const float scale = sqrtf((float)kG);
  for (int r = half * 32; r < half * 32 + 32; ++r) {
    float acc = 0.f;
    for (int k = 0; k < kG; ++k) acc = fmaf(s_w[r * kG + k], s_rot_t[k * kG + j], acc);
    const float y = acc * scale;
    int lo = 0, hi = n_edges;           // first edge >= y  (= number of edges < y)
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (s_edges[mid] < y) lo = mid + 1; else hi = mid;
    }
    s_code[r * kG + j] = (uint8_t)min(lo, n_edges);
  }
  __syncthreads();
  const int per = 8 / a.bit, bytes_per_row = kG / per;
  for (int i = tid; i < kRows * bytes_per_row; i += kThreads) {
    const int r = i / bytes_per_row, bcol = i % bytes_per_row;
    if (row0 + r >= a.N) continue;
    uint32_t v = 0;
    for (int e = 0; e < per; ++e) v |= (uint32_t)s_code[r * kG + bcol * per + e] << (e * a.bit);
    a.packed[(size_t)(row0 + r) * (a.K / per) + g * bytes_per_row + bcol] = (uint8_t)v;
  }
}

}  // namespace

extern "C" int dmoq_quantize_packed(const void* w, int32_t w_kind, int32_t N, int32_t K, int32_t bit, const float* rot,
                                    const float* edges, uint8_t* indices_packed, uint16_t* norms, void* stream) {
  DMOQ_CHECK_ARG(w && rot && edges && indices_packed && norms);
  DMOQ_CHECK_ARG(w_kind >= 0 && w_kind <= 2 && N > 0 && K > 0 && K % kG == 0);
  DMOQ_CHECK_ARG(bit == 1 || bit == 2 || bit == 4 || bit == 8);
  static DmoqOncePerDevice once;
  bool* configured = once.slot();
  if (configured == nullptr) return DMOQ_EDEVICE;
  const size_t smem = (size_t)(kG * kG + kRows * kG + 256) * sizeof(float) + kRows * kG;
  if (!*configured) {
    if (cudaFuncSetAttribute(quantize_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return DMOQ_ELAUNCH;
    *configured = true;
  }
  QuantArgs a{w, w_kind, N, K, bit, rot, edges, indices_packed, norms};
  quantize_kernel<<<dim3(dmoq_ceil_div(N, kRows), K / kG), kThreads, smem, static_cast<cudaStream_t>(stream)>>>(a);
  return dmoq_launch_status();
}
