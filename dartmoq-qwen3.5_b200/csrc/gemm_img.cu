// Grouped GEMM over "weight images" on the 5th-generation tensor cores (tcgen05 + TMEM), all four activation modes.
//
// A weight image is a pool's weights already looked up in the mode's codeword table and laid out as tensor-core
// operand rows (dmoq_expand_weights): (groups, image rows, 128 columns) of int8 / e4m3 / fp16 codewords, or packed
// e2m1 nibbles with two groups per 128-byte row.  Its tiles need no work in this kernel: one thread brings each
// 128 x 128-byte tile into shared memory with a TMA tensor-map copy (cp.async.bulk.tensor, 128-byte swizzle), so an
// expert that receives many rows pays for the table lookup once per forward (or once at load time) instead of once
// per 128-row tile.  The math is that of the reference's merged kernels:
//   turboquant_utils/triton_kernels.py:1375 (A16), triton_kernels_a8.py:825 (A8, int32 sums per 128-group),
//   triton_kernels_fp8.py:532 (FP8), triton_kernels_fp4.py:587 (FP4: e2m1 x e2m1 with per-32 e8m0 block scales,
//   weights folded to e2m1 at load time, W_FOLDED).
//
// One persistent CTA of 768 threads per SM:
//   warps 0-15   epilogue: warp w drains lanes 32*(w%4).. of columns 32*(w/4).. of the group's accumulator
//                (tcgen05.ld 32x32b: a thread owns one row), folds (acc * row_scale) * col_norm into an fp32 running
//                total, and at the end of a tile writes SiLU*up / plain / weighted rows straight to global memory
//   warp 16      loader: one thread issues, per operand step, the TMA copies of the A tile (128 rows of the sorted
//                activation-code table) and of the B tile, and the bulk copy of the group's column norms
//   warps 16-19  FP4 mode only: store the rows' e8m0 block scales into TMEM (tcgen05.st) for the block-scaled MMA
//   warp 20      one thread issues tcgen05.mma: kind::i8 / f8f6f4 / f16, or kind::mxf4nvf4.block_scale (scale_vec 2X)
//   warps 21-23  idle (setmaxnreg moves their registers to the epilogue)
// Every mbarrier wait is bounded; on a timeout the CTA raises the device status word, stops issuing work and
// falls through to the common teardown, where TMEM is released.
#include <cuda.h>

#include "common.cuh"

// raised when a bounded wait of this file's kernels runs out (read through dmoq_tc_status)
__device__ int g_dmoq_img_status = 0;

// Optional per-role cycle counters (block 0, first warp of each role); compiled in only for tuning builds.
#ifdef DMOQ_IMG_PROFILE
__device__ unsigned long long g_img_prof[32];
#define PROF_DECL long long prof_t0 = 0, prof_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0}
#define PROF_BEGIN() prof_t0 = clock64()
#define PROF_END(i) prof_acc[i] += clock64() - prof_t0
#define PROF_FLUSH(base, cond)                                                        \
  if ((cond) && blockIdx.x == 0 && lane == 0) {                                       \
    for (int i_ = 0; i_ < 8; ++i_) atomicAdd(&g_img_prof[(base) + i_], (unsigned long long)prof_acc[i_]); \
  }
#else
#define PROF_DECL
#define PROF_BEGIN()
#define PROF_END(i)
#define PROF_FLUSH(base, cond)
#endif

namespace {

constexpr int kBM = 128, kG = DMOQ_GROUP;
#ifndef DMOQ_IMG_STAGES
#define DMOQ_IMG_STAGES 4
#endif
constexpr int kStages = DMOQ_IMG_STAGES;   // operand ring depth: one 128-row x 128-byte A tile and one BN-row B tile per stage
constexpr int kEpiWarps = 16;
constexpr int kTileA = kBM * 128;   // bytes of one A operand tile
constexpr uint32_t kSpinLimit = 1u << 26;
constexpr long long kWaitCycles = 2000000000LL;
// INT8 accumulators start from the bit pattern of 1.5*2^23: the int32 sum read back as fp32 is 12582912 + sum
// exactly (|sum| <= 128*127*127 < 2^22), which saves the integer->float conversion.
constexpr uint32_t kMagicBits = 0x4B400000u;
constexpr float kMagicFloat = 12582912.0f;
constexpr int kTmemCols = 512;
constexpr int kSfaCol = 384;        // FP4 (128-column tiles): three accumulators, then the scale-factor columns
constexpr int kSfbCol = kSfaCol + kStages * 2 * 4;

// Tile width and role layout.  BN = 256 (fp16 / INT8 / e4m3 operands): one tcgen05.mma covers 256 columns, so the A
// tile is read from shared memory once per 256 columns and an item's fixed costs are halved; two 256-column
// accumulators fill TMEM; 640 threads (16 epilogue warps, loader warp 16, MMA warp 17).  BN = 128: three
// accumulators + the FP4 scale-factor columns; 768 threads (loader / scale warps 16-19, MMA warp 20).
// setmaxnreg moves registers between warpgroups inside the pool the block got at launch (threads x kRegsLaunch);
// asking for more than the pool holds blocks forever, so the launcher checks the compiled register count.
template <int BN>
struct Cfg {
  static constexpr int kAuxWarps = (BN == 256) ? 4 : 8;                 // warps after the epilogue warps
  static constexpr int kThreads = 32 * (kEpiWarps + kAuxWarps);
  static constexpr int kMmaWarp = (BN == 256) ? kEpiWarps + 1 : kEpiWarps + 4;
  static constexpr int kRegsLaunch = (BN == 256) ? 96 : 80;
  static constexpr int kRegsEpi = (BN == 256) ? 112 : 96;
  static constexpr int kRegsAux = (BN == 256) ? 32 : 40;
  static constexpr int kNormRing = (BN == 256) ? 8 : 16;                // column-norm slots; exceeds the groups in flight
  static constexpr int kTileB = BN * 128;
  static_assert(32 * (kEpiWarps * kRegsEpi + kAuxWarps * kRegsAux) <= kRegsLaunch * kThreads,
                "role register budgets exceed the block's register pool");
};

// One launch covers the tiles of up to DMOQ_MAX_POOLS pools of one activation mode (the kernel never looks at bit
// widths: the images hold codewords).  Per pool: its image (tensor map), norms, sizes and tile list.
struct ImgPool {
  const float* norm_img;      // (groups, n_img) fp32, image row order
  int n_img;                  // image rows per group
  int inter;                  // intermediate size of the pool's members
  int pool;                   // index into the routing tables' per-pool tile lists
};

struct ImgMaps {
  CUtensorMap a;                     // the activation-code table in routed-row order
  CUtensorMap b[DMOQ_MAX_POOLS];     // one weight image per pool of the launch
};

struct ImgArgs {
  const DmoqTile* tiles;
  const int32_t* n_tiles;
  const float* row_weight;
  ImgPool pp[DMOQ_MAX_POOLS];
  int n_pp;
  int is_down, hidden;
  const uint8_t* a_scales;    // A8/FP8: fp16 (rows, K/128); FP4: e8m0 bytes (rows, K/32); row r of the table feeds row r
  int a_stride;               // row pitch of the code table in elements (the codes themselves come through tmap_a)
  void* out;
  int out_stride;
  int32_t* partials;
  uint32_t sfb_word;          // FP4: the weight block scale byte 127+E0 replicated four times
};

// ------------------------------------------------------------------------------------------------ PTX wrappers
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_try_wait_suspend(uint64_t* bar, uint32_t parity, uint32_t ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"(ns)
      : "memory");
  return ok != 0;
}
// Bounded wait (about one second).  Returns false, and raises the abort flag, if the phase never completes; once
// the flag is up every later wait returns at once.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  if (*abort_flag) return false;
  const long long t0 = clock64();
  for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
    if (mbar_try_wait_suspend(bar, parity, 100000u)) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > kWaitCycles) break;
  }
  *abort_flag = 1;
  atomicOr(&g_dmoq_img_status, 1);
  return false;
}
// Time-bounded wait that ignores the abort flag: used at teardown so that no bulk copy is still writing into this
// block's shared memory when it exits.
__device__ __forceinline__ void mbar_wait_quiet(uint64_t* bar, uint32_t parity) {
  const long long t0 = clock64();
  while (!mbar_try_wait_suspend(bar, parity, 100000u)) {
    if (clock64() - t0 > kWaitCycles) break;
  }
}
// 2-D tile of a tensor map -> this block's shared memory; completion counted in bytes on the barrier.  The map lies
// over this GPU's own memory; the inner coordinate x is a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
template <int MODE>
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  if (MODE == DMOQ_A8) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else if (MODE == DMOQ_FP8) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}
// e2m1 x e2m1, one ue8m0 scale per 32 elements of K for each operand, read from TMEM (K = 64 per instruction)
__device__ __forceinline__ void tc_mma_mxf4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::2X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
      : "memory");
}
// accumulator loads: thread t of the warp receives lane base + t, register j = column base + j
// 32 lanes x 8 columns
__device__ __forceinline__ void tc_ld8(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// 32 lanes x 8 columns of one value
__device__ __forceinline__ void tc_st8_fill(uint32_t taddr, uint32_t v) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%1,%1,%1,%1,%1,%1,%1};" ::"r"(taddr), "r"(v) : "memory");
}
// 32 lanes x 4 columns: thread t writes its four values to lane base + t
__device__ __forceinline__ void tc_st4(uint32_t taddr, uint32_t v0, uint32_t v1, uint32_t v2, uint32_t v3) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1,%2,%3,%4};" ::"r"(taddr), "r"(v0), "r"(v1), "r"(v2), "r"(v3)
               : "memory");
}
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }

// K-major, 128-byte swizzle: tile row r is 128 bytes; 16-byte chunk c lives at slot c ^ (r & 7); groups of 8 rows
// are 1024 bytes apart (the descriptor's stride byte offset).  The TMA copy writes the same pattern.
__device__ __forceinline__ uint32_t swz128(int r, int c) { return (uint32_t)(r * 128 + ((c ^ (r & 7)) << 4)); }
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr) {
  return (uint64_t)((smem_addr >> 4) & 0x3FFF) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
         ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}

template <int BN>
struct Smem {
  uint8_t a[kStages][kTileA];              // 1024-byte aligned operand tiles
  uint8_t b[kStages][Cfg<BN>::kTileB];
  float norm[Cfg<BN>::kNormRing][BN];      // column norms of a group, image column order
  uint64_t full[kStages], empty[kStages], acc_full[4], acc_empty[4];
  uint32_t tmem_base;
  int abort_flag;
};

template <int N>
__device__ __forceinline__ void reg_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N>
__device__ __forceinline__ void reg_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }

// Per mode: operand steps per group / groups per operand step (a step = 128 bytes of every operand row).
//   A8, FP8: one step per group.  A16: two steps per group (64 fp16 columns each).
//   FP4: one step carries two groups (64 bytes of packed e2m1 each).
template <int MODE>
struct Shape {
  static constexpr int SPG = (MODE == DMOQ_A16) ? 2 : 1;   // operand steps per group
  static constexpr int GPS = (MODE == DMOQ_FP4) ? 2 : 1;   // groups per operand step
};

template <int MODE, int EPI, int BN>
__global__ void __launch_bounds__(Cfg<BN>::kThreads, 1) gemm_img_kernel(const __grid_constant__ ImgMaps maps,
                                                                        const __grid_constant__ ImgArgs a) {
  using C = Cfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  Smem<BN>& S = *reinterpret_cast<Smem<BN>*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  volatile int* abort_flag = &S.abort_flag;
  constexpr int SPG = Shape<MODE>::SPG, GPS = Shape<MODE>::GPS;
  constexpr int ACC = (BN == 256) ? 2 : (MODE == DMOQ_FP4 ? 3 : 4);   // accumulator buffers in TMEM
  constexpr int NH = BN / 128;                                        // 32-column blocks per epilogue thread
  constexpr int CW = 8;                                               // accumulator columns per TMEM load
  constexpr int NCH = 32 * NH / CW;                                   // loads per group and thread (even)
  constexpr int kMmaWarp = C::kMmaWarp, kNormRing = C::kNormRing;
  static_assert(!(MODE == DMOQ_FP4 && BN != 128), "the FP4 scale-factor columns need 128-column tiles");

  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&S.full[s], MODE == DMOQ_FP4 ? 5 : 1);   // the thread that announces the bulk bytes (+ four scale warps)
      mbar_init(&S.empty[s], 1);
    }
    for (int b = 0; b < 4; ++b) {
      mbar_init(&S.acc_full[b], 1);
      mbar_init(&S.acc_empty[b], kEpiWarps);
    }
    S.abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == kMmaWarp) {  // the MMA warp owns the TMEM allocation
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&S.tmem_base)), "r"(kTmemCols));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = S.tmem_base;
  if (MODE == DMOQ_A8 || MODE == DMOQ_FP4) {
    if (warp < kEpiWarps) {
      const uint32_t t0 = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
      if (MODE == DMOQ_A8) {   // bias every accumulator buffer: this warp's 32 lanes x its columns of each
#pragma unroll
        for (int b = 0; b < ACC; ++b)
#pragma unroll
          for (int q = 0; q < 4 * NH; ++q) tc_st8_fill(t0 + b * BN + (warp >> 2) * (32 * NH) + 8 * q, kMagicBits);
      } else if (warp < 4) {   // the constant weight block scale, for every column and every 32-block of K
        tc_st4(t0 + kSfbCol, a.sfb_word, a.sfb_word, a.sfb_word, a.sfb_word);
      }
      tc_wait_st();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
  }

  // Work items = (tile, column block) pairs of every pool of the launch, pool after pool; CTA b takes items b, b + grid, ...
  // Every role walks the same list, so each computes an item's pool, tile and group count for itself.
  int work_end[DMOQ_MAX_POOLS];       // exclusive prefix of the pools' item counts
  int n_work = 0;
#pragma unroll
  for (int q = 0; q < DMOQ_MAX_POOLS; ++q) {
    if (q < a.n_pp) {
      const int nbq = a.is_down ? a.hidden / BN : a.pp[q].inter / (BN / 2);
      n_work += a.n_tiles[a.pp[q].pool] * nbq;
    }
    work_end[q] = n_work;
  }
  const int stride_w = gridDim.x;
  const int n_items = (int)blockIdx.x < n_work ? (n_work - 1 - (int)blockIdx.x) / stride_w + 1 : 0;
  struct Item {
    DmoqTile tile;
    int q, nb, G;
  };
  auto pool_of_item = [&](int item, int& start) {   // which pool of the launch the CTA's item-th work item belongs to
    const int w = blockIdx.x + item * stride_w;
    int q = 0;
    start = 0;
#pragma unroll
    for (int j = 0; j < DMOQ_MAX_POOLS - 1; ++j)
      if (j + 1 < a.n_pp && w >= work_end[j]) {
        q = j + 1;
        start = work_end[j];
      }
    return q;
  };
  auto groups_of = [&](int q) { return a.is_down ? a.pp[q].inter / kG : a.hidden / kG; };
  auto item_of = [&](int item) {   // item index of this CTA -> pool, tile record, column block (an empty tile past the end)
    Item it_{DmoqTile{0, 0, 0, 0}, 0, 0, 1};
    if (item < n_items) {
      int start;
      const int q = pool_of_item(item, start);
      const int nbq = a.is_down ? a.hidden / BN : a.pp[q].inter / (BN / 2);
      const int local = blockIdx.x + item * stride_w - start;
      it_.q = q;
      it_.nb = local % nbq;
      it_.tile = a.tiles[a.n_tiles[DMOQ_MAX_POOLS + a.pp[q].pool] + local / nbq];
      it_.G = groups_of(q);
    }
    return it_;
  };
  auto steps_of = [&](int G) { return (G * SPG + GPS - 1) / GPS; };

  if (warp < kEpiWarps) {
    // =========================================================================== epilogue warps
    reg_inc<C::kRegsEpi>();
    const int lq = warp & 3, cq = warp >> 2;
    const int row = lq * 32 + lane;                  // tile row of this thread
    const int cbase = cq * (32 * NH);                // first of this thread's 32*NH tile columns
    const uint32_t t_lane = tmem_base + ((uint32_t)(lq * 32) << 16) + cbase;
    const int xs_per_row = a.a_stride / kG;
    uint32_t ia = 0;                                 // groups consumed so far
    uint32_t v[2][8];                                // accumulator chunks: one in the scale math, one in flight
    bool prefetched = false;                         // the upcoming group's first chunk is already on its way
    Item next = item_of(0);
    PROF_DECL;
#ifdef DMOQ_IMG_PROFILE
    const long long prof_start = clock64();
#endif
    for (int item = 0; item < n_items; ++item) {
      const Item cur = next;
      next = item_of(item + 1);
      const DmoqTile tile = cur.tile;
      const int nb = cur.nb, G = cur.G, inter = a.pp[cur.q].inter;
      const bool live = row < tile.rows;
      // row scales: this row's G fp16 values, fetched four at a time (8-byte loads, one block ahead) where the row
      // pitch allows, else one at a time
      const bool has_xs = (MODE == DMOQ_A8 || MODE == DMOQ_FP8);
      const __half* xs_row = reinterpret_cast<const __half*>(a.a_scales) + (size_t)(tile.row0 + (live ? row : 0)) * xs_per_row;
      const bool xs_vec = (xs_per_row & 3) == 0;
      float2 total2[16 * NH];   // pair p = this thread's columns 2p, 2p+1
#pragma unroll
      for (int c = 0; c < 16 * NH; ++c) total2[c] = make_float2(0.f, 0.f);
      uint2 xq = make_uint2(0u, 0u), xq_next = make_uint2(0u, 0u);
      float xs_next = 0.f;
      if (has_xs) {
        if (xs_vec) xq_next = *reinterpret_cast<const uint2*>(xs_row);
        else xs_next = __half2float(xs_row[0]);
      }
      int held = -1;     // accumulator buffer whose release is still owed (its bias stores are in flight)
      auto release = [&]() {
        if (held >= 0) {
          if (MODE == DMOQ_A8) tc_wait_st();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&S.acc_empty[held]);
          held = -1;
        }
      };

      for (int g = 0; g < G; ++g, ++ia) {
        const uint32_t b = ia % ACC, ph = (ia / ACC) & 1;
        const uint32_t slot = ia % kNormRing;
        float xs = 0.f;
        if (has_xs) {
          if (xs_vec) {
            if ((g & 3) == 0) {
              xq = xq_next;
              if (g + 4 < G) xq_next = *reinterpret_cast<const uint2*>(xs_row + g + 4);   // in flight during these groups
            }
            const uint32_t w = (g & 2) ? xq.y : xq.x;
            xs = __half2float(__ushort_as_half((unsigned short)((g & 1) ? (w >> 16) : (w & 0xFFFFu))));
          } else {
            xs = xs_next;
            if (g + 1 < G) xs_next = __half2float(xs_row[g + 1]);
          }
        }
        // The group's norms were bulk-copied before its operand stage completed; the MMA thread saw that completion
        // before it committed acc_full[], so they are visible here.
        if (!prefetched) {
          PROF_BEGIN();
          mbar_wait(&S.acc_full[b], ph, abort_flag);   // on a timeout the flag is up and the data is void
          PROF_END(0);
          tc_fence_after();
          tc_ld8(t_lane + b * BN, v[0]);
        }
        prefetched = false;
        PROF_BEGIN();
        const float2 xs2 = make_float2(xs, xs);
        const float off = (MODE == DMOQ_A8) ? -kMagicFloat * xs : 0.f;
        const float2 off2 = make_float2(off, off);
        // The thread's 32*NH columns in chunks of eight: the load of chunk c+1 (at the end of a group: of the next
        // group's first chunk, if that group is ready) is in flight while chunk c goes through the scale math.
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
          tc_wait_ld();
          // the previous group's buffer goes back to the MMA thread here: its bias stores were issued a whole group
          // ago, so waiting for them costs nothing now
          if (c == 0) release();
          if (c + 1 < NCH) {
            tc_ld8(t_lane + b * BN + CW * (c + 1), v[(c + 1) & 1]);
          } else if (g + 1 < G || item + 1 < n_items) {
            const uint32_t bn_ = (ia + 1) % ACC, phn = ((ia + 1) / ACC) & 1;
            if (mbar_try_wait(&S.acc_full[bn_], phn)) {
              tc_fence_after();
              tc_ld8(t_lane + bn_ * BN, v[(c + 1) & 1]);
              prefetched = true;
            }
          }
          if (MODE == DMOQ_A8) tc_st8_fill(t_lane + b * BN + CW * c, kMagicBits);   // re-arm the bias for the buffer's next use
          const uint32_t(&vc)[8] = v[c & 1];
          const float4* nrm4 = reinterpret_cast<const float4*>(&S.norm[slot][cbase + CW * c]);
#pragma unroll
          for (int q = 0; q < 2; ++q) {
            const float4 n4 = nrm4[q];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const int j = 4 * q + 2 * e;
              const float2 f = make_float2(__uint_as_float(vc[j]), __uint_as_float(vc[j + 1]));
              const float2 n2 = e ? make_float2(n4.z, n4.w) : make_float2(n4.x, n4.y);
              // INT8: (acc_biased - M) * xs in one fma with the exact constant -M*xs; e4m3: acc * xs;
              // fp16 / e2m1 operands: no row scale (the block scales are applied by the MMA)
              const float2 t2 = (MODE == DMOQ_A8 || MODE == DMOQ_FP8) ? fma2(f, xs2, off2) : f;
              total2[(CW * c + j) >> 1] = fma2(t2, n2, total2[(CW * c + j) >> 1]);
            }
          }
          if (BN == 128 && MODE == DMOQ_A8 && a.partials != nullptr && live) {   // parity checks only (128-column tiles)
            const int n_out = a.is_down ? a.hidden : 2 * inter;
#pragma unroll
            for (int j = 0; j < CW; ++j) {
              const int col = CW * c + j;                                        // 0..31
              const int n = a.is_down ? nb * BN + cbase + col
                                      : (col < 16 ? 0 : inter) + nb * (BN / 2) + cq * 16 + (col & 15);
              a.partials[((size_t)(tile.row0 + row) * n_out + n) * G + g] = (int32_t)(vc[j] - kMagicBits);
            }
          }
        }
        PROF_END(2);
        held = (int)b;
      }
      release();   // before the tile's output stores: the MMA thread may run ahead into the next item
      PROF_BEGIN();

      // ---- tile epilogue: a thread owns 32*NH consecutive image columns of its row
#pragma unroll
      for (int h = 0; h < NH; ++h) {
        if (EPI == DMOQ_EPI_SILU) {   // image columns [0,16) of the block = gate, [16,32) = up of 16 consecutive outputs
          uint32_t pk[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            float o[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const float gate = __half2float(__float2half_rn(e ? total2[16 * h + j].y : total2[16 * h + j].x));
              const float up = __half2float(__float2half_rn(e ? total2[16 * h + 8 + j].y : total2[16 * h + 8 + j].x));
              // fast exp and reciprocal (a few fp32 ulps) ahead of the fp16 rounding: a floating-point stage
              const float sg = __half2float(__float2half_rn(__fdividef(gate, 1.0f + __expf(-gate))));
              o[e] = __fmul_rn(sg, up);
            }
            const __half2 h2 = __floats2half2_rn(o[0], o[1]);
            pk[j] = *reinterpret_cast<const uint32_t*>(&h2);
          }
          if (live) {
            uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__half*>(a.out) + (size_t)(tile.row0 + row) * a.out_stride +
                                                  nb * (BN / 2) + (cq * NH + h) * 16);
            dst[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
            dst[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
          }
        } else {
          float wgt = 0.f;
          if (EPI == DMOQ_EPI_WEIGHTED && live) wgt = a.row_weight[tile.row0 + row];
          uint32_t pk[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const __half2 h2 = __floats2half2_rn(total2[16 * h + j].x, total2[16 * h + j].y);   // the fp16 output
            if (EPI == DMOQ_EPI_WEIGHTED) {   // -> bf16, times the routing weight in fp32, -> bf16
              const float2 hf = __half22float2(h2);
              const float2 bf = __bfloat1622float2(__floats2bfloat162_rn(hf.x, hf.y));
              const __nv_bfloat162 o2 = __floats2bfloat162_rn(__fmul_rn(bf.x, wgt), __fmul_rn(bf.y, wgt));
              pk[j] = *reinterpret_cast<const uint32_t*>(&o2);
            } else {
              pk[j] = *reinterpret_cast<const uint32_t*>(&h2);
            }
          }
          if (live) {
            uint16_t* orow = reinterpret_cast<uint16_t*>(a.out) + (size_t)(tile.row0 + row) * a.out_stride;
            if (a.is_down) {
              uint4* dst = reinterpret_cast<uint4*>(orow + nb * BN + cbase + 32 * h);
#pragma unroll
              for (int q = 0; q < 4; ++q) dst[q] = make_uint4(pk[4 * q], pk[4 * q + 1], pk[4 * q + 2], pk[4 * q + 3]);
            } else {   // plain gate_up rows: [gate | up], each inter wide
              uint4* dg = reinterpret_cast<uint4*>(orow + nb * (BN / 2) + (cq * NH + h) * 16);
              uint4* du = reinterpret_cast<uint4*>(orow + inter + nb * (BN / 2) + (cq * NH + h) * 16);
              dg[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
              dg[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
              du[0] = make_uint4(pk[8], pk[9], pk[10], pk[11]);
              du[1] = make_uint4(pk[12], pk[13], pk[14], pk[15]);
            }
          }
        }
      }
      PROF_END(4);
    }
#ifdef DMOQ_IMG_PROFILE
    prof_acc[7] = clock64() - prof_start;
#endif
    PROF_FLUSH(0, warp == 0);
  } else {
    reg_dec<C::kRegsAux>();
    const int pw = warp - kEpiWarps;                  // FP4: 0..3 = TMEM lane quarter of the warp's scale stores
    const bool scale_warp = (MODE == DMOQ_FP4) && pw < 4;
    if (warp == kEpiWarps || scale_warp) {
      // ========================================================================= loader (and FP4 scale) warps
      const bool loader = (warp == kEpiWarps && lane == 0);
      const int sf_per_row = a.a_stride / 32;           // FP4: e8m0 bytes per table row
      uint32_t it = 0, ig = 0;                        // operand steps issued, groups whose norms were requested
      PROF_DECL;
#ifdef DMOQ_IMG_PROFILE
      const long long prof_start = clock64();
#endif
      Item t_next = item_of(0);
      for (int item = 0; item < n_items; ++item) {
        const Item cur = t_next;
        t_next = item_of(item + 1);
        const DmoqTile tile = cur.tile;
        const ImgPool& pp = a.pp[cur.q];
        const int nb = cur.nb, G = cur.G;
        const int gg0 = a.is_down ? tile.rank * G : 0;                       // first image group of this item
        const int img_row0 = a.is_down ? nb * BN : tile.rank * 2 * pp.inter + nb * BN;
        const int steps_per_item = steps_of(G);
        for (int st = 0; st < steps_per_item; ++st, ++it) {
          const int s = it % kStages;
          PROF_BEGIN();
          mbar_wait(&S.empty[s], ((it / kStages) & 1) ^ 1, abort_flag);
          PROF_END(0);
          PROF_BEGIN();
          if (loader) {
            if (!*abort_flag) {
              // A tile: rows [row0, +128) of the sorted code table, 128 bytes of the step; B tile: image rows
              // [img_row0, +BN) of the step's image row group; column norms of the groups the step starts
              const int g_first = (st * GPS) / SPG;
              const int n_groups = (SPG == 2) ? ((st & 1) ? 0 : 1) : min(GPS, G - g_first);
              mbar_arrive_expect_tx(&S.full[s], kTileA + C::kTileB + n_groups * BN * 4);
              int x, y;
              if (MODE == DMOQ_A16) {
                x = (st & 1) * 128;
                y = (gg0 + (st >> 1)) * pp.n_img + img_row0;
              } else if (MODE == DMOQ_FP4) {
                x = 0;
                y = ((gg0 >> 1) + st) * pp.n_img + img_row0;   // two groups per image row group; gg0 is even (checked on the host)
              } else {
                x = 0;
                y = (gg0 + st) * pp.n_img + img_row0;
              }
              tma_load_2d(&S.a[s][0], &maps.a, st * 128, tile.row0, &S.full[s]);
              tma_load_2d(&S.b[s][0], &maps.b[cur.q], x, y, &S.full[s]);
              for (int j = 0; j < n_groups; ++j, ++ig)
                bulk_g2s(&S.norm[ig % kNormRing][0], pp.norm_img + (size_t)(gg0 + g_first + j) * pp.n_img + img_row0, BN * 4, &S.full[s]);
            } else {
              mbar_arrive(&S.full[s]);   // keep the arrival count whole after an abort
            }
          }
          PROF_END(1);
          if (MODE == DMOQ_FP4) {   // the rows' block scales of the step's two groups -> TMEM columns of this stage
            PROF_BEGIN();
#pragma unroll
            for (int j = 0; j < 2; ++j) {
              uint32_t w[4];
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                w[q] = 0x7F7F7F7Fu;
                const int g = st * 2 + j, rr = lane + 32 * q;
                if (rr < tile.rows && g < G)
                  w[q] = *reinterpret_cast<const uint32_t*>(a.a_scales + (size_t)(tile.row0 + rr) * sf_per_row + g * 4);
              }
              tc_st4(tmem_base + ((uint32_t)(pw * 32) << 16) + kSfaCol + (s * 2 + j) * 4, w[0], w[1], w[2], w[3]);
            }
            tc_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&S.full[s]);
            PROF_END(2);
          }
        }
      }
#ifdef DMOQ_IMG_PROFILE
      prof_acc[7] = clock64() - prof_start;
#endif
      PROF_FLUSH(8, warp == kEpiWarps);
      // no bulk copy may still be in flight when the block exits (matters after an abort)
      if (loader)
        for (uint32_t j = (it > (uint32_t)kStages ? it - kStages : 0u); j < it; ++j) mbar_wait_quiet(&S.full[j % kStages], (j / kStages) & 1);
    } else if (warp == kMmaWarp) {
      // ========================================================================= MMA warp
      constexpr uint32_t nm = ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
      constexpr uint32_t idesc_i8 = (2u << 4) | (1u << 7) | (1u << 10) | nm;    // s32 accumulate, signed 8-bit operands
      constexpr uint32_t idesc_f8 = (1u << 4) | nm;                              // f32 accumulate, e4m3 operands
      constexpr uint32_t idesc_f16 = (1u << 4) | nm;                             // f32 accumulate, fp16 operands
      constexpr uint32_t idesc_f4 = (1u << 7) | (1u << 10) | (1u << 23) | nm;    // e2m1 operands, ue8m0 scales, K = 64
      uint32_t it = 0, ia = 0;
      PROF_DECL;
#ifdef DMOQ_IMG_PROFILE
      const long long prof_start = clock64();
#endif
      for (int item = 0; item < n_items; ++item) {
        int start_unused;
        const int G = groups_of(pool_of_item(item, start_unused));
        const int steps_per_item = steps_of(G);
        for (int st = 0; st < steps_per_item; ++st, ++it) {
          const int s = it % kStages;
          PROF_BEGIN();
          bool ok = mbar_wait(&S.full[s], (it / kStages) & 1, abort_flag);
          PROF_END(0);
          PROF_BEGIN();
          const int n_groups = (SPG == 2) ? 1 : min(GPS, G - st * GPS);
          // a group's first MMA needs its accumulator buffer back from the epilogue
          if (SPG == 1 || (st & 1) == 0) {
            for (int j = 0; j < n_groups; ++j) {
              const uint32_t ib = ia + j;
              ok = mbar_wait(&S.acc_empty[ib % ACC], ((ib / ACC) & 1) ^ 1, abort_flag) && ok;
            }
          }
          PROF_END(1);
          PROF_BEGIN();
          tc_fence_after();
          if (lane == 0 && ok) {
            const uint64_t da = make_desc(smem_u32(&S.a[s][0]));
            const uint64_t db = make_desc(smem_u32(&S.b[s][0]));
            if (MODE == DMOQ_FP4) {
              for (int j = 0; j < n_groups; ++j) {
                const uint32_t b = (ia + j) % ACC;
                const uint32_t sfa = tmem_base + kSfaCol + (s * 2 + j) * 4;
#pragma unroll
                for (int k = 0; k < 2; ++k) {   // 64 elements = 32 bytes of K per instruction; scale bytes 2k, 2k+1
                  const uint32_t idesc = idesc_f4 | ((uint32_t)(2 * k) << 4) | ((uint32_t)(2 * k) << 29);
                  tc_mma_mxf4(tmem_base + b * BN, da + 2 * (2 * j + k), db + 2 * (2 * j + k), idesc, sfa, tmem_base + kSfbCol, k > 0);
                }
                tc_commit(&S.acc_full[b]);
              }
              tc_commit(&S.empty[s]);
            } else {
              const uint32_t b = ia % ACC;
              const uint32_t d = tmem_base + b * BN;
#pragma unroll
              for (int k = 0; k < 4; ++k) {  // 32 bytes of K per instruction: +2 in 16-byte units
                if (MODE == DMOQ_A8) tc_mma<DMOQ_A8>(d, da + 2 * k, db + 2 * k, idesc_i8, 1);  // the buffer holds the bias
                else if (MODE == DMOQ_FP8) tc_mma<DMOQ_FP8>(d, da + 2 * k, db + 2 * k, idesc_f8, k > 0);
                else tc_mma<DMOQ_A16>(d, da + 2 * k, db + 2 * k, idesc_f16, ((st & 1) || k > 0) ? 1u : 0u);
              }
              tc_commit(&S.empty[s]);
              if (SPG == 1 || (st & 1)) tc_commit(&S.acc_full[b]);
            }
          }
          if (SPG == 1 || (st & 1)) ia += n_groups;
          __syncwarp();
          PROF_END(2);
        }
      }
#ifdef DMOQ_IMG_PROFILE
      prof_acc[7] = clock64() - prof_start;
#endif
      PROF_FLUSH(16, true);
    }
  }

  // ---- teardown: all roles meet here, then the allocating warp releases TMEM
  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols));
  }
}

// ------------------------------------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
      return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// Tensor map over a byte matrix (a weight image, or the sorted activation-code table): `rows` rows of `row_bytes`
// (a multiple of 16), copied in boxes of 128 bytes x box_rows rows (<= 256); rows past the end read as zero.
int make_image_map(CUtensorMap* map, const void* image, size_t rows, size_t row_bytes, int box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return DMOQ_EDEVICE;
  const cuuint64_t dims[2] = {row_bytes, rows};
  const cuuint64_t strides[1] = {row_bytes};
  const cuuint32_t box[2] = {128, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult rc = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(image), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return rc == CUDA_SUCCESS ? DMOQ_OK : DMOQ_EINVAL;
}

template <int MODE, int EPI, int BN>
int launch(const ImgMaps& maps, const ImgArgs& a, int work_cap, cudaStream_t s) {
  static DmoqOncePerDevice once;
  bool* configured = once.slot();
  if (configured == nullptr) return DMOQ_EDEVICE;
  const int bytes = (int)sizeof(Smem<BN>) + 1024;
  if (!*configured) {
    cudaFuncAttributes fa;
    if (cudaFuncGetAttributes(&fa, gemm_img_kernel<MODE, EPI, BN>) != cudaSuccess) return DMOQ_ELAUNCH;
    if (fa.numRegs != Cfg<BN>::kRegsLaunch) return DMOQ_ELAUNCH;   // the role budgets were sized for this pool
    if (cudaFuncSetAttribute(gemm_img_kernel<MODE, EPI, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess)
      return DMOQ_ELAUNCH;
    *configured = true;
  }
  int grid = dmoq_sm_count();
  if (grid > work_cap) grid = work_cap;
  if (grid < 1) grid = 1;
  gemm_img_kernel<MODE, EPI, BN><<<grid, Cfg<BN>::kThreads, bytes, s>>>(maps, a);
  return dmoq_launch_status();
}

template <int MODE, int BN>
int launch_epi(const ImgMaps& maps, const ImgArgs& a, int epi, int work_cap, cudaStream_t s) {
  switch (epi) {
    case DMOQ_EPI_SILU: return launch<MODE, DMOQ_EPI_SILU, BN>(maps, a, work_cap, s);
    case DMOQ_EPI_WEIGHTED: return launch<MODE, DMOQ_EPI_WEIGHTED, BN>(maps, a, work_cap, s);
    case DMOQ_EPI_PLAIN: return launch<MODE, DMOQ_EPI_PLAIN, BN>(maps, a, work_cap, s);
    default: return DMOQ_EINVAL;
  }
}

}  // namespace

// True when this pool/direction has a weight image the kernel above can run on.
bool dmoq_img_supported(const dmoq_pool_t& p, int is_down, int hidden) {
  const void* img = is_down ? p.dn_img : p.gu_img;
  const float* nimg = is_down ? p.dn_norm_img : p.gu_norm_img;
  if (img == nullptr || nimg == nullptr) return false;
  if (p.inter % 128 != 0 || hidden % 128 != 0) return false;
  if (p.mode == DMOQ_FP4 && (p.inter / 128) % 2 != 0 && is_down && p.n_members > 1) return false;   // image groups pair up
  return true;   // the caller also needs the code table in routed-row order (route->a_row == NULL, or the down side)
}

// One launch over the listed pools (all of one activation mode, each with a weight image for this projection).
int dmoq_grouped_gemm_img_pools(const dmoq_route_t* route, const dmoq_pool_t* pools, const int32_t* pool_ids, int n_ids,
                                int is_down, int epilogue, int hidden, const void* a_codes, const void* a_scales, int a_stride,
                                void* out, int out_stride, int32_t* partials, cudaStream_t s) {
  if (n_ids < 1 || n_ids > DMOQ_MAX_POOLS) return DMOQ_EINVAL;
  const int mode = pools[pool_ids[0]].mode;
  if (mode == DMOQ_FP4 && n_ids != 1) return DMOQ_EINVAL;   // the weight block scale in TMEM is one pool's
  ImgArgs a{};
  ImgMaps maps;
  a.tiles = reinterpret_cast<const DmoqTile*>(route->tiles);
  a.n_tiles = route->n_tiles;
  a.row_weight = route->sorted_weights;
  a.n_pp = n_ids;
  a.is_down = is_down;
  a.hidden = hidden;
  a.a_scales = static_cast<const uint8_t*>(a_scales);
  a.a_stride = a_stride;
  a.out = out;
  a.out_stride = out_stride;
  a.partials = partials;
  // 256-column tiles wherever the shape allows (not FP4: its scale-factor columns share TMEM with the accumulators)
  bool wide = mode != DMOQ_FP4 && partials == nullptr && (is_down ? hidden % 256 == 0 : true);
  for (int i = 0; i < n_ids; ++i) wide = wide && (is_down || pools[pool_ids[i]].inter % 128 == 0);
  const int bn = wide ? 256 : 128;
  long long cap = 0;
  for (int i = 0; i < n_ids; ++i) {
    const dmoq_pool_t& p = pools[pool_ids[i]];
    if (p.mode != mode || !dmoq_img_supported(p, is_down, hidden)) return DMOQ_EINVAL;
    ImgPool& pp = a.pp[i];
    pp.norm_img = is_down ? p.dn_norm_img : p.gu_norm_img;
    pp.n_img = is_down ? hidden : p.n_members * 2 * p.inter;
    pp.inter = p.inter;
    pp.pool = pool_ids[i];
    const int groups = is_down ? p.n_members * p.inter / kG : hidden / kG;
    // image geometry: rows of 128 elements (256 bytes as fp16, 128 bytes otherwise); e2m1 rows hold two groups
    size_t rows, row_bytes;
    if (mode == DMOQ_FP4) {
      rows = (size_t)((groups + 1) / 2) * pp.n_img;
      row_bytes = 128;
      const int e0 = is_down ? p.dn_e0 : p.gu_e0;
      a.sfb_word = 0x01010101u * (uint32_t)((127 + e0) & 0xFF);
    } else {
      rows = (size_t)groups * pp.n_img;
      row_bytes = (mode == DMOQ_A16) ? 256 : 128;
    }
    const int rc = make_image_map(&maps.b[i], is_down ? p.dn_img : p.gu_img, rows, row_bytes, bn);
    if (rc != DMOQ_OK) return rc;
    cap += (long long)route->tile_cap * (is_down ? hidden / bn : p.inter / (bn / 2));
  }
  for (int i = n_ids; i < DMOQ_MAX_POOLS; ++i) maps.b[i] = maps.b[0];
  // the activation-code table: one row per routed row, in routed-row order
  const size_t a_rows = (size_t)route->T * route->top_k + (route->has_shared ? (size_t)route->T : 0);
  const size_t a_pitch = (mode == DMOQ_A16) ? (size_t)a_stride * 2 : (mode == DMOQ_FP4) ? (size_t)a_stride / 2 : (size_t)a_stride;
  const int rc = make_image_map(&maps.a, a_codes, a_rows, a_pitch, 128);
  if (rc != DMOQ_OK) return rc;
  const int work_cap = cap > (1 << 30) ? (1 << 30) : (int)cap;
  switch (mode) {
    case DMOQ_A16: return wide ? launch_epi<DMOQ_A16, 256>(maps, a, epilogue, work_cap, s) : launch_epi<DMOQ_A16, 128>(maps, a, epilogue, work_cap, s);
    case DMOQ_A8: return wide ? launch_epi<DMOQ_A8, 256>(maps, a, epilogue, work_cap, s) : launch_epi<DMOQ_A8, 128>(maps, a, epilogue, work_cap, s);
    case DMOQ_FP8: return wide ? launch_epi<DMOQ_FP8, 256>(maps, a, epilogue, work_cap, s) : launch_epi<DMOQ_FP8, 128>(maps, a, epilogue, work_cap, s);
    case DMOQ_FP4: return launch_epi<DMOQ_FP4, 128>(maps, a, epilogue, work_cap, s);
    default: return DMOQ_EINVAL;
  }
}

int dmoq_grouped_gemm_img(const dmoq_route_t* route, const dmoq_pool_t* pools, int pool_index, int is_down, int epilogue,
                          int hidden, const void* a_codes, const void* a_scales, int a_stride, void* out, int out_stride,
                          int32_t* partials, cudaStream_t s) {
  const int32_t id = pool_index;
  return dmoq_grouped_gemm_img_pools(route, pools, &id, 1, is_down, epilogue, hidden, a_codes, a_scales, a_stride, out,
                                     out_stride, partials, s);
}

#ifdef DMOQ_IMG_PROFILE
extern "C" int dmoq_img_profile(unsigned long long* out32, int reset) {
  if (cudaMemcpyFromSymbol(out32, g_img_prof, sizeof(unsigned long long) * 32) != cudaSuccess) return DMOQ_EDEVICE;
  if (reset) {
    unsigned long long z[32] = {0};
    if (cudaMemcpyToSymbol(g_img_prof, z, sizeof(z)) != cudaSuccess) return DMOQ_EDEVICE;
  }
  return DMOQ_OK;
}
#endif

// Status word of this file's kernels on the current device (0 = no bounded wait ever ran out); synchronises.
int dmoq_img_status(int* out) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_dmoq_img_status, sizeof(int)) != cudaSuccess) return DMOQ_EDEVICE;
  *out = v;
  return DMOQ_OK;
}
