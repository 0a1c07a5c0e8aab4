// Device-side routing tables: histogram -> scan -> stable counting sort, the
// per-pool tile lists and the activation-table row maps.  No host round trip.
//
// Stands in for argsort + bincount(...).cpu().cumsum() and the Python pool /
// expert_info / block_info builders of the reference
// (quantization/wxa16/bit_partitioned_moe.py:1125-1138, :1014-1057;
//  turboquant_utils/triton_kernels_a8.py:938).
#include "common.cuh"

namespace {

constexpr int kChunk = 1024;  // flat (token, slot) entries per chunk

struct RouteArgs {
  dmoq_route_t r;
  const int64_t* topk_idx;
  const float* topk_w;
  const float* shared_w;
  int32_t* hist;        // (n_chunks, E) chunk histograms, turned into chunk offsets in place
  int32_t* pool_row0;   // (E + has_shared) first activation-table row of each expert inside its pool
  int32_t n_flat;       // T * top_k
  int32_t n_chunks;
};

// --- phase 1: per-chunk histogram ------------------------------------------------------
__device__ void chunk_histogram(const RouteArgs& a, int chunk, int32_t* s_hist) {
  const int E = a.r.E;
  for (int e = threadIdx.x; e < E; e += blockDim.x) s_hist[e] = 0;
  __syncthreads();
  const int lo = chunk * kChunk;
  const int hi = min(lo + kChunk, a.n_flat);
  for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    long long e = a.topk_idx[i];
    if (e >= 0 && e < E) atomicAdd(&s_hist[(int)e], 1);
  }
  __syncthreads();
}

// --- phase 2: scans, pool bookkeeping, tile lists (one block) ---------------------------
__device__ void scan_and_tiles(const RouteArgs& a, int32_t* s_count /* E_tot+1 ints */) {
  const int E = a.r.E;
  const int E_tot = E + a.r.has_shared;
  const int P = a.r.n_pools;
  __shared__ int8_t s_pool[4100];   // pool of each expert, staged once: the serial scan below must not wait on HBM

  // rows per expert; chunk histograms become exclusive chunk offsets
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int run = 0;
    for (int c0 = 0; c0 < a.n_chunks; c0 += 16) {   // sixteen independent loads in flight, then the serial prefix
      int v[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) v[i] = (c0 + i < a.n_chunks) ? a.hist[(size_t)(c0 + i) * E + e] : 0;
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        if (c0 + i < a.n_chunks) a.hist[(size_t)(c0 + i) * E + e] = run;
        run += v[i];
      }
    }
    s_count[e] = run;
  }
  for (int e = threadIdx.x; e < E_tot; e += blockDim.x) {
    const int p = a.r.expert_pool[e];
    s_pool[e] = (int8_t)((p >= 0 && p < P) ? p : -1);
  }
  if (threadIdx.x == 0 && a.r.has_shared) s_count[E] = a.r.T;
  __syncthreads();

  // Prefix sums over the experts by warp 0: every lane owns a contiguous run of experts, sums its run, the
  // warp scans the 1 + 2*pools partial sums with shuffles, then every lane walks its run again with its bases.
  __shared__ int32_t s_slot[4100];   // first tile slot of each expert
  __shared__ int32_t s_row0[4100];   // first row of each expert
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    const int per = (E_tot + 31) / 32;
    const int e0 = min(lane * per, E_tot), e1 = min(e0 + per, E_tot);
    int rows_all = 0, rows_p[DMOQ_MAX_POOLS], tiles_p[DMOQ_MAX_POOLS];
#pragma unroll
    for (int p = 0; p < DMOQ_MAX_POOLS; ++p) rows_p[p] = tiles_p[p] = 0;
    for (int e = e0; e < e1; ++e) {
      const int n = s_count[e], pl = s_pool[e];
      const int nt = (n + a.r.tile_m - 1) / a.r.tile_m;
      rows_all += n;
#pragma unroll
      for (int p = 0; p < DMOQ_MAX_POOLS; ++p) {
        rows_p[p] += (pl == p) ? n : 0;
        tiles_p[p] += (pl == p) ? nt : 0;
      }
    }
    auto excl_scan = [&](int v, int& total) {   // exclusive prefix over the lanes, total in every lane
      int inc = v;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int o = __shfl_up_sync(0xffffffffu, inc, d);
        if (lane >= d) inc += o;
      }
      total = __shfl_sync(0xffffffffu, inc, 31);
      return inc - v;
    };
    int tot_all;
    int run = excl_scan(rows_all, tot_all);
    int prow[DMOQ_MAX_POOLS], pslot[DMOQ_MAX_POOLS], tot_rows[DMOQ_MAX_POOLS], tot_tiles[DMOQ_MAX_POOLS];
#pragma unroll
    for (int p = 0; p < DMOQ_MAX_POOLS; ++p) {
      prow[p] = excl_scan(rows_p[p], tot_rows[p]);
      pslot[p] = excl_scan(tiles_p[p], tot_tiles[p]);
    }
    int tb = 0;   // pool p's tiles start after all tiles of the pools before it
#pragma unroll
    for (int p = 0; p < DMOQ_MAX_POOLS; ++p) {
      pslot[p] += tb;
      if (lane == 0) {
        a.r.pool_rows[p] = tot_rows[p];
        a.r.n_tiles[p] = tot_tiles[p];
        a.r.n_tiles[DMOQ_MAX_POOLS + p] = tb;
      }
      tb += tot_tiles[p];
    }
    for (int e = e0; e < e1; ++e) {
      const int n = s_count[e], pl = s_pool[e];
      const int nt = (n + a.r.tile_m - 1) / a.r.tile_m;
      a.r.expert_rows[e] = run;
      s_row0[e] = run;
      run += n;
      int my_prow = 0, my_slot = 0;
#pragma unroll
      for (int p = 0; p < DMOQ_MAX_POOLS; ++p) {
        if (pl == p) {
          my_prow = prow[p];
          my_slot = pslot[p];
          prow[p] += n;
          pslot[p] += nt;
        }
      }
      a.pool_row0[e] = my_prow;
      s_slot[e] = my_slot;
    }
    if (lane == 31) a.r.expert_rows[E_tot] = tot_all;
  }
  __syncthreads();

  // tile lists: pool p's tiles are contiguous from its base, experts in index order
  for (int e = threadIdx.x; e < E_tot; e += blockDim.x) {
    const int p = s_pool[e];
    if (p < 0) continue;
    const int n = s_count[e];
    if (n == 0) continue;
    int slot = s_slot[e];
    const int row0 = s_row0[e];
    const int rank = a.r.expert_rank[e];
    for (int m = 0; m < n; m += a.r.tile_m, ++slot) {
      if (slot >= a.r.tile_cap) break;
      DmoqTile t{e, row0 + m, min(a.r.tile_m, n - m), rank};
      reinterpret_cast<DmoqTile*>(a.r.tiles)[slot] = t;
    }
  }
}

// --- phase 3: stable placement of one chunk ------------------------------------------------
// The whole block first stages everything the placement reads (the chunk's entries, the chunk offsets,
// the expert row prefix, the pool tables) in shared memory; warp 0 then walks the chunk in order, 32
// entries at a time, so that no step of the serial walk waits on global memory.
struct PlaceSmem {
  int32_t* running;   // E
  int32_t* offset;    // E       chunk offsets of this chunk
  int32_t* rows;      // E + 2   expert row prefix
  int32_t* prow0;     // E + 1   first activation-table row of each expert inside its pool
  int32_t* entry;     // kChunk  expert of each entry (-1 = invalid)
  float* weight;      // kChunk
  int8_t* pool;       // E + 1 (+ padding)
};

__device__ PlaceSmem carve_place_smem(int32_t* base, int E) {
  PlaceSmem m;
  m.running = base;
  m.offset = m.running + E;
  m.rows = m.offset + E;
  m.prow0 = m.rows + E + 2;
  m.entry = m.prow0 + E + 1;
  m.weight = reinterpret_cast<float*>(m.entry + kChunk);
  m.pool = reinterpret_cast<int8_t*>(m.weight + kChunk);
  return m;
}

__host__ __device__ inline size_t place_smem_bytes(int E) {
  return (size_t)(4 * E + 3 + 2 * kChunk) * sizeof(int32_t) + (size_t)E + 8;
}

__device__ void place_chunk(const RouteArgs& a, int chunk, const PlaceSmem& m) {
  const int E = a.r.E;
  const int P = a.r.n_pools;
  const int lo = chunk * kChunk;
  const int hi = min(lo + kChunk, a.n_flat);
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    m.running[e] = 0;
    m.offset[e] = a.hist[(size_t)chunk * E + e];
    m.prow0[e] = a.pool_row0[e];
    const int p = a.r.expert_pool[e];
    m.pool[e] = (int8_t)((p >= 0 && p < P) ? p : -1);
  }
  for (int e = threadIdx.x; e <= E; e += blockDim.x) m.rows[e] = a.r.expert_rows[e];
  for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    const long long e64 = a.topk_idx[i];
    m.entry[i - lo] = (e64 >= 0 && e64 < E) ? (int)e64 : -1;
    m.weight[i - lo] = a.topk_w[i];
  }
  __syncthreads();
  if (threadIdx.x >= 32) return;
  const int lane = threadIdx.x;
  int hoisted[DMOQ_MAX_POOLS], src_base[DMOQ_MAX_POOLS];
#pragma unroll
  for (int p = 0; p < DMOQ_MAX_POOLS; ++p) {
    hoisted[p] = a.r.pool_hoisted[p];
    src_base[p] = a.r.pool_src_base[p];
  }
  for (int base = lo; base < hi; base += 32) {
    const int i = base + lane;
    const int e_in = (i < hi) ? m.entry[i - lo] : -1;
    const bool ok = e_in >= 0;
    const int e = ok ? e_in : -1 - lane;  // invalid lanes get unique keys
    const unsigned peers = __match_any_sync(0xffffffffu, e);
    const int before = __popc(peers & ((1u << lane) - 1));
    int start = 0;
    if (ok) start = m.running[e];
    __syncwarp();
    if (ok && before == 0) m.running[e] = start + __popc(peers);
    __syncwarp();
    if (i < hi) {
      if (!ok) {
        a.r.row_of[i] = -1;
        continue;
      }
      const int within = m.offset[e] + start + before;
      const int pos = m.rows[e] + within;
      const int tok = i / a.r.top_k;
      const int p = m.pool[e];
      a.r.sorted_tokens[pos] = tok;
      a.r.sorted_weights[pos] = m.weight[i - lo];
      if (p < 0) {
        a.r.row_of[i] = -1;  // expert without weights contributes nothing
        a.r.a_row[pos] = 0;
      } else {
        a.r.row_of[i] = pos;
        int hs = 0, sb = 0;
#pragma unroll
        for (int q = 0; q < DMOQ_MAX_POOLS; ++q) {
          if (q == p) {
            hs = hoisted[q];
            sb = src_base[q];
          }
        }
        if (hs) {
          a.r.a_row[pos] = tok;
        } else {
          const int tr = m.prow0[e] + within;
          a.r.a_row[pos] = tr;
          a.r.pool_src[sb + tr] = tok;
        }
      }
    }
  }
}

__device__ void place_shared(const RouteArgs& a, int t0, int t1) {
  const int E = a.r.E;
  const int row0 = a.r.expert_rows[E];
  const int p = a.r.expert_pool[E];
  for (int t = t0 + threadIdx.x; t < t1; t += blockDim.x) {
    const int pos = row0 + t;
    a.r.sorted_tokens[pos] = t;
    a.r.sorted_weights[pos] = a.shared_w ? a.shared_w[t] : 1.0f;
    a.r.row_of[a.n_flat + t] = (p >= 0 && p < a.r.n_pools) ? pos : -1;
    a.r.a_row[pos] = t;
  }
}

__global__ void route_hist_kernel(RouteArgs a) {
  extern __shared__ int32_t s_dyn[];
  chunk_histogram(a, blockIdx.x, s_dyn);
  for (int e = threadIdx.x; e < a.r.E; e += blockDim.x) a.hist[(size_t)blockIdx.x * a.r.E + e] = s_dyn[e];
}

__global__ void __launch_bounds__(1024) route_scan_kernel(RouteArgs a) {
  extern __shared__ int32_t s_dyn[];
  scan_and_tiles(a, s_dyn);
}

__global__ void route_place_kernel(RouteArgs a) {
  extern __shared__ int32_t s_dyn[];
  if ((int)blockIdx.x < a.n_chunks) {
    place_chunk(a, blockIdx.x, carve_place_smem(s_dyn, a.r.E));
  } else if (a.r.has_shared) {
    const int b = blockIdx.x - a.n_chunks;
    place_shared(a, b * kChunk, min((b + 1) * kChunk, a.r.T));
  }
}

// Small problems (one chunk): everything in a single block.
__global__ void __launch_bounds__(1024) route_fused_kernel(RouteArgs a) {
  extern __shared__ int32_t s_dyn[];  // placement tables first, then E+2 counts
  const PlaceSmem m = carve_place_smem(s_dyn, a.r.E);
  int32_t* s_count = s_dyn + (place_smem_bytes(a.r.E) + 3) / 4;
  chunk_histogram(a, 0, m.running);
  for (int e = threadIdx.x; e < a.r.E; e += blockDim.x) a.hist[e] = m.running[e];
  __syncthreads();
  scan_and_tiles(a, s_count);
  __threadfence_block();
  __syncthreads();
  if (a.r.has_shared) place_shared(a, 0, a.r.T);
  place_chunk(a, 0, m);
}

// Shared launch sequence of both routing entry points.
int launch_route(const RouteArgs& a, bool fused, cudaStream_t s) {
  const dmoq_route_t& r = a.r;
  const size_t e_bytes = (size_t)r.E * sizeof(int32_t);
  const size_t place_bytes = place_smem_bytes(r.E) + 16;
  const size_t fused_bytes = place_bytes + e_bytes + 16;
  static DmoqOncePerDevice once;
  bool* configured = once.slot();
  if (configured == nullptr) return DMOQ_EDEVICE;
  if (!*configured) {  // up to 4096 experts: the placement tables can exceed the default 48 KiB
    if (cudaFuncSetAttribute(route_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024) != cudaSuccess ||
        cudaFuncSetAttribute(route_place_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024) != cudaSuccess)
      return DMOQ_ELAUNCH;
    *configured = true;
  }
  if (fused) {
    route_fused_kernel<<<1, 1024, fused_bytes, s>>>(a);
    return dmoq_launch_status();
  }
  route_hist_kernel<<<a.n_chunks, 256, e_bytes, s>>>(a);
  route_scan_kernel<<<1, 1024, e_bytes + 16, s>>>(a);
  const int shared_blocks = r.has_shared ? dmoq_ceil_div(r.T, kChunk) : 0;
  route_place_kernel<<<a.n_chunks + shared_blocks, 128, place_bytes, s>>>(a);
  return dmoq_launch_status();
}

}  // namespace

extern "C" size_t dmoq_route_workspace_bytes(int32_t T, int32_t top_k, int32_t E) {
  if (T < 0 || top_k <= 0 || E <= 0) return 0;
  size_t n_chunks = ((size_t)T * top_k + kChunk - 1) / kChunk;
  if (n_chunks == 0) n_chunks = 1;
  return (n_chunks * (size_t)E + (size_t)E + 1) * sizeof(int32_t);
}

extern "C" int dmoq_route_build(const dmoq_route_t* route, const int64_t* topk_idx, const float* topk_w,
                                const float* shared_w, void* workspace, size_t workspace_bytes,
                                void* stream) {
  DMOQ_CHECK_ARG(route && topk_idx && topk_w && workspace);
  const dmoq_route_t& r = *route;
  DMOQ_CHECK_ARG(r.T >= 0 && r.top_k > 0 && r.E > 0 && r.E <= 4096 && r.tile_m > 0);
  DMOQ_CHECK_ARG(r.n_pools >= 0 && r.n_pools <= DMOQ_MAX_POOLS);
  DMOQ_CHECK_ARG(r.expert_pool && r.expert_rank && r.expert_rows && r.sorted_tokens && r.sorted_weights);
  DMOQ_CHECK_ARG(r.row_of && r.a_row && r.pool_rows && r.pool_src && r.pool_src_base && r.tiles && r.n_tiles);
  DMOQ_CHECK_ARG(r.pool_hoisted);
  if (workspace_bytes < dmoq_route_workspace_bytes(r.T, r.top_k, r.E)) return DMOQ_ESIZE;

  RouteArgs a;
  a.r = r;
  a.topk_idx = topk_idx;
  a.topk_w = topk_w;
  a.shared_w = shared_w;
  a.n_flat = r.T * r.top_k;
  a.n_chunks = dmoq_ceil_div(a.n_flat, kChunk);
  if (a.n_chunks == 0) a.n_chunks = 1;
  a.hist = static_cast<int32_t*>(workspace);
  a.pool_row0 = a.hist + (size_t)a.n_chunks * r.E;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const size_t e_bytes = (size_t)r.E * sizeof(int32_t);

  if (a.n_chunks == 1 && (!r.has_shared || r.T <= 4 * kChunk)) {
    return launch_route(a, true, s);
  }
  return launch_route(a, false, s);
}

// ------------------------------------------------------------------------------------------------
// Routing build for callers that cannot allocate device memory.
//
// Some hosts of this library may not call cudaMalloc at all: code running between
// cudaStreamBeginCapture and cudaStreamEndCapture, real-time serving loops that have frozen their
// memory pools, or plugins whose host framework owns every allocation and hands out none for scratch.
// dmoq_route_build needs a scratch buffer from its caller; this variant brings its own, a fixed
// array in the library's device image.  Every GPU that loads libdmoq.so holds these 4 MiB until the
// process exits.
constexpr size_t kStaticRouteInts = (size_t)1 << 20;
static __device__ __align__(256) int32_t g_route_scratch[kStaticRouteInts];

namespace {
// Device address of g_route_scratch per device ordinal.  In host code the array's name is only a
// handle for the runtime, not an address a kernel could use; the address comes from
// cudaGetSymbolAddress, asked once per device with that device current.
int32_t* g_route_scratch_ptr[64] = {nullptr};

int route_scratch_for_current_device(int32_t** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return DMOQ_EDEVICE;
  if (g_route_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_route_scratch) != cudaSuccess || p == nullptr) return DMOQ_EDEVICE;
    g_route_scratch_ptr[dev] = static_cast<int32_t*>(p);
  }
  *out = g_route_scratch_ptr[dev];
  return DMOQ_OK;
}
}  // namespace

extern "C" size_t dmoq_route_static_max_bytes(void) { return kStaticRouteInts * sizeof(int32_t); }

extern "C" int dmoq_route_build_static(const dmoq_route_t* route, const int64_t* topk_idx, const float* topk_w,
                                       const float* shared_w, void* stream) {
  DMOQ_CHECK_ARG(route && topk_idx && topk_w);
  const dmoq_route_t& r = *route;
  DMOQ_CHECK_ARG(r.T >= 0 && r.top_k > 0 && r.E > 0 && r.E <= 4096 && r.tile_m > 0);
  DMOQ_CHECK_ARG(r.n_pools >= 0 && r.n_pools <= DMOQ_MAX_POOLS);
  DMOQ_CHECK_ARG(r.expert_pool && r.expert_rank && r.expert_rows && r.sorted_tokens && r.sorted_weights);
  DMOQ_CHECK_ARG(r.row_of && r.a_row && r.pool_rows && r.pool_src && r.pool_src_base && r.tiles && r.n_tiles);
  DMOQ_CHECK_ARG(r.pool_hoisted);
  // the same scratch size the allocating variant asks its caller for; larger problems are refused
  const size_t need = dmoq_route_workspace_bytes(r.T, r.top_k, r.E);
  if (need == 0 || need > dmoq_route_static_max_bytes()) return DMOQ_ESIZE;
  int32_t* scratch = nullptr;
  const int rc = route_scratch_for_current_device(&scratch);
  if (rc != DMOQ_OK) return rc;

  RouteArgs a;
  a.r = r;
  a.topk_idx = topk_idx;
  a.topk_w = topk_w;
  a.shared_w = shared_w;
  a.n_flat = r.T * r.top_k;
  a.n_chunks = dmoq_ceil_div(a.n_flat, kChunk);
  if (a.n_chunks == 0) a.n_chunks = 1;
  a.hist = scratch;
  a.pool_row0 = a.hist + (size_t)a.n_chunks * r.E;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (a.n_chunks == 1 && (!r.has_shared || r.T <= 4 * kChunk)) {
    return launch_route(a, true, s);
  }
  return launch_route(a, false, s);
}

// ---------------------------------------------------------------------------------------------------------
// Router selection: fp32 softmax over the experts, the k largest probabilities in descending order (ties: lower
// expert index first), optionally renormalised to sum 1.  One warp per token, NPL logits per lane in registers.
namespace {

// The shared expert's gate for the same token, when asked for: sigmoid(x[t] . w + b) with the roundings of a 16-bit
// Linear followed by a 16-bit sigmoid (quantization/wxa16/bit_partitioned_moe.py:1101-1106): fp32 dot product,
// rounded to the activation type, sigmoid in fp32, rounded again; stored as fp32.
struct SharedGate {
  const uint16_t* x;       // (T, H) bf16 / fp16 rows, 16-byte aligned, H a multiple of 8; NULL = no shared gate
  const uint16_t* w;       // (H) same type
  float bias;
  int H, is_bf16;
  float* out;              // (T)
};

__device__ __forceinline__ float gate_elem(uint16_t bits, int is_bf16) {
  return is_bf16 ? __uint_as_float((uint32_t)bits << 16) : __half2float(__ushort_as_half(bits));
}
__device__ __forceinline__ float gate_round(float v, int is_bf16) {
  return is_bf16 ? __bfloat162float(__float2bfloat16_rn(v)) : __half2float(__float2half_rn(v));
}

template <int NPL>
__global__ void __launch_bounds__(256) router_topk_kernel(const float* __restrict__ logits, int T, int E, int k,
                                                          int renormalize, float* __restrict__ topk_w,
                                                          int64_t* __restrict__ topk_idx, SharedGate sg) {
  const int lane = threadIdx.x & 31;
  const int warps_per_grid = gridDim.x * (blockDim.x >> 5);
  for (int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); t < T; t += warps_per_grid) {
    float v[NPL];
    float m = -INFINITY;
#pragma unroll
    for (int i = 0; i < NPL; ++i) {   // expert e = i * 32 + lane: coalesced reads
      const int e = i * 32 + lane;
      v[i] = e < E ? logits[(size_t)t * E + e] : -INFINITY;
      m = fmaxf(m, v[i]);
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, d));
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
      v[i] = (i * 32 + lane < E) ? expf(v[i] - m) : -1.f;   // probabilities are >= 0; -1 marks padding / taken
      sum += fmaxf(v[i], 0.f);
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, d);
    float my_w = 0.f, top_sum = 0.f;   // lane j keeps the j-th selection
    int my_e = 0;
    for (int j = 0; j < k; ++j) {
      float best = -1.f;
      int best_e = 0x7fffffff;
#pragma unroll
      for (int i = 0; i < NPL; ++i) {
        if (v[i] > best) {   // strict: the lower expert index wins inside a lane
          best = v[i];
          best_e = i * 32 + lane;
        }
      }
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, d);
        const int oe = __shfl_xor_sync(0xffffffffu, best_e, d);
        if (ob > best || (ob == best && oe < best_e)) {
          best = ob;
          best_e = oe;
        }
      }
      const float p = __fdiv_rn(best, sum);
      top_sum += p;
      if (lane == j) {
        my_w = p;
        my_e = best_e;
      }
      if ((best_e & 31) == lane) {
#pragma unroll
        for (int i = 0; i < NPL; ++i)
          if (i == (best_e >> 5)) v[i] = -1.f;
      }
    }
    if (lane < k) {
      topk_w[(size_t)t * k + lane] = renormalize ? __fdiv_rn(my_w, top_sum) : my_w;
      topk_idx[(size_t)t * k + lane] = my_e;
    }
    if (sg.x != nullptr) {
      const uint4* xr = reinterpret_cast<const uint4*>(sg.x + (size_t)t * sg.H);
      const uint4* wr = reinterpret_cast<const uint4*>(sg.w);
      float dot = 0.f;
      for (int c = lane; c < sg.H / 8; c += 32) {
        const uint4 xv = xr[c], wv = wr[c];
        const uint16_t* xe = reinterpret_cast<const uint16_t*>(&xv);
        const uint16_t* we = reinterpret_cast<const uint16_t*>(&wv);
#pragma unroll
        for (int q = 0; q < 8; ++q) dot = fmaf(gate_elem(xe[q], sg.is_bf16), gate_elem(we[q], sg.is_bf16), dot);
      }
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, d);
      if (lane == 0) {
        const float g = gate_round(dot + sg.bias, sg.is_bf16);
        sg.out[t] = gate_round(1.0f / (1.0f + expf(-g)), sg.is_bf16);
      }
    }
  }
}

template <int NPL>
int launch_router(const float* logits, int T, int E, int k, int renorm, float* w, int64_t* idx, const SharedGate& sg, cudaStream_t s) {
  int blocks = dmoq_ceil_div(T, 8);
  const int cap = 16 * dmoq_sm_count();
  if (blocks > cap) blocks = cap;
  router_topk_kernel<NPL><<<blocks, 256, 0, s>>>(logits, T, E, k, renorm, w, idx, sg);
  return dmoq_launch_status();
}

}  // namespace

static int router_dispatch(const float* logits, int T, int E, int top_k, int renormalize, float* topk_w, int64_t* topk_idx,
                    const SharedGate& sg, cudaStream_t s) {
  if (E <= 32) return launch_router<1>(logits, T, E, top_k, renormalize, topk_w, topk_idx, sg, s);
  if (E <= 64) return launch_router<2>(logits, T, E, top_k, renormalize, topk_w, topk_idx, sg, s);
  if (E <= 128) return launch_router<4>(logits, T, E, top_k, renormalize, topk_w, topk_idx, sg, s);
  if (E <= 256) return launch_router<8>(logits, T, E, top_k, renormalize, topk_w, topk_idx, sg, s);
  if (E <= 512) return launch_router<16>(logits, T, E, top_k, renormalize, topk_w, topk_idx, sg, s);
  return launch_router<32>(logits, T, E, top_k, renormalize, topk_w, topk_idx, sg, s);
}

extern "C" int dmoq_router_topk(const float* logits, int32_t T, int32_t E, int32_t top_k, int32_t renormalize,
                                float* topk_w, int64_t* topk_idx, void* stream) {
  DMOQ_CHECK_ARG(logits && topk_w && topk_idx && T >= 0);
  DMOQ_CHECK_ARG(E > 0 && E <= 1024 && top_k > 0 && top_k <= 32 && top_k <= E);
  if (T == 0) return DMOQ_OK;
  return router_dispatch(logits, T, E, top_k, renormalize, topk_w, topk_idx, SharedGate{}, static_cast<cudaStream_t>(stream));
}

extern "C" int dmoq_router_topk_gate(const float* logits, int32_t T, int32_t E, int32_t top_k, int32_t renormalize,
                                     float* topk_w, int64_t* topk_idx, const void* x, int32_t x_is_bf16, int32_t hidden,
                                     const void* gate_w, float gate_bias, float* shared_w, void* stream) {
  DMOQ_CHECK_ARG(logits && topk_w && topk_idx && T >= 0 && x && gate_w && shared_w);
  DMOQ_CHECK_ARG(E > 0 && E <= 1024 && top_k > 0 && top_k <= 32 && top_k <= E);
  DMOQ_CHECK_ARG(hidden > 0 && hidden % 8 == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0 && reinterpret_cast<uintptr_t>(gate_w) % 16 == 0);
  if (T == 0) return DMOQ_OK;
  SharedGate sg{static_cast<const uint16_t*>(x), static_cast<const uint16_t*>(gate_w), gate_bias, hidden, x_is_bf16, shared_w};
  return router_dispatch(logits, T, E, top_k, renormalize, topk_w, topk_idx, sg, static_cast<cudaStream_t>(stream));
}
