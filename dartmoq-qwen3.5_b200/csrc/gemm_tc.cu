// Grouped LUT-dequant GEMM on the 5th-generation tensor cores (tcgen05 + TMEM), INT8 and e4m3 modes.
//
// One persistent CTA per SM, warp-specialised:
//   warps 0-7   epilogue: drain the per-group accumulator from TMEM (tcgen05.ld), fold
//               (acc * row_scale) * col_norm into an fp32 running total, final SiLU*up or
//               routing-weight epilogue through a padded shared-memory staging tile
//   warps 8-15  producers: gather activation-code rows with cp.async straight into the 128B-swizzled
//               K-major operand tile; look the codebook indices of the raw ring up in registers (byte
//               permutes; 1- and 2-bit codes are stored widened to 4-bit fields for this) and store the
//               codewords into the swizzled B operand tile; they also stage each group's row scales and
//               column norms into a small ring
//   warp 16     one elected thread issues tcgen05.mma (M=128, N=128, K=32 x4 per 128-wide group),
//               tcgen05.commit releases the smem stage and publishes the accumulator
//   warp 17     one thread bulk-copies each group's packed indices into the raw ring
//   warps 18-19 idle (they only give their registers away: setmaxnreg works on whole warpgroups)
// Tile metadata and row indices of the NEXT work item are fetched while the current one runs, so the
// operand pipeline does not drain at item boundaries.
// Four accumulator buffers fill TMEM (4 x 128 columns), so the tensor pipe runs up to three groups ahead
// of the epilogue warps (it keeps going while they write out a finished tile).  Integer group sums are exact (kind::i8, int32), which is
// what turboquant_utils/triton_kernels_a8.py:893-929 computes; kind::f8f6f4 gives the fp32 group sums of
// turboquant_utils/triton_kernels_fp8.py:589-626.
//
// Every wait on an mbarrier is bounded; on a timeout the CTA raises a flag in the device status word,
// stops issuing work, and falls through to the common teardown (TMEM is always released).
#include "common.cuh"

namespace {

constexpr int kBM = 128, kBN = 128, kG = DMOQ_GROUP;
constexpr int kStages = 4;       // operand ring depth (one 128-wide group per stage)
constexpr int kLag = 2;          // producer: stages between issuing the async copies and expanding them
constexpr int kEpiWarps = 8, kProdWarps = 8;
constexpr int kProdThreads = 32 * kProdWarps;
constexpr int kCPT = kBM * 8 / kProdThreads;   // 16-byte operand chunks per producer thread, tile and stage (4)
constexpr int kThreads = 640;     // 5 warpgroups: epilogue x2, producers x2, MMA warp + 3 idle warps
constexpr int kAccBufs = 4;       // accumulator buffers in TMEM
constexpr int kScaleRing = 16;    // per-group scale slots; must exceed kStages + kAccBufs (see the epilogue)
// setmaxnreg moves registers between the warpgroups inside the pool the block got at launch: 640 threads x the
// 96 registers ptxas reports for this kernel.  Asking for more than the pool holds blocks forever, so the
// launch helper refuses to run if the compiled kernel's register count is not kRegsLaunch.
constexpr int kRegsLaunch = 96;
constexpr int kRegsEpi = 168, kRegsProd = 56, kRegsMma = 24;
static_assert(32 * (kEpiWarps * kRegsEpi + kProdWarps * kRegsProd + 4 * kRegsMma) <= kRegsLaunch * kThreads,
              "role register budgets exceed the block's register pool");
static_assert(kThreads == 32 * (kEpiWarps + kProdWarps + 4) && kEpiWarps % 4 == 0 && kProdWarps % 4 == 0, "role layout");
constexpr int kTileB = kBM * kG; // bytes of one int8 / e4m3 operand tile
constexpr int kOutPitch = 272;   // bytes per staged output row (256 + 16: conflict-free 16-byte stores)
constexpr int kRawPad = 64;     // bytes between the gate and the up segment of the raw index tile (bank spread)
constexpr uint32_t kSpinLimit = 1u << 26;
constexpr long long kWaitCycles = 2000000000LL;
// INT8 accumulators start from the bit pattern of 1.5*2^23: the int32 sum read back as fp32 is then
// 12582912 + sum exactly (|sum| <= 128*127*127 < 2^22), which saves the integer->float conversion.
constexpr uint32_t kMagicBits = 0x4B400000u;
constexpr float kMagicFloat = 12582912.0f;

__device__ int g_dmoq_tc_status = 0;

// Optional per-role cycle counters (block 0, first warp of each role); compiled in only for tuning builds.
#ifdef DMOQ_TC_PROFILE
__device__ unsigned long long g_tc_prof[32];
#define PROF_DECL long long prof_t0 = 0, prof_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0}
#define PROF_BEGIN() prof_t0 = clock64()
#define PROF_END(i) prof_acc[i] += clock64() - prof_t0
#define PROF_FLUSH(base, cond)                                                        \
  if ((cond) && blockIdx.x == 0 && lane == 0) {                                       \
    for (int i_ = 0; i_ < 8; ++i_) atomicAdd(&g_tc_prof[(base) + i_], (unsigned long long)prof_acc[i_]); \
  }
#else
#define PROF_DECL
#define PROF_BEGIN()
#define PROF_END(i)
#define PROF_FLUSH(base, cond)
#endif

struct TcArgs {
  const DmoqTile* tiles;
  const int32_t* n_tiles;
  const int32_t* expert_rank;
  const int32_t* a_row;
  const float* row_weight;
  int pool, is_down, inter, hidden, n_members;
  const uint8_t* idx;
  const uint16_t* norm;
  const uint8_t* lut;
  int identity_lut;
  const uint8_t* a_codes;
  const uint16_t* a_scales;
  int a_stride;
  void* out;
  int out_stride;
  int32_t* partials;
};

// ------------------------------------------------------------------------------------------------ PTX wrappers
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
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
// Same, but the hardware may keep the thread suspended for up to `ns` nanoseconds while the phase is pending,
// so a waiting warp does not compete for issue slots and shared-memory bandwidth.
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
// Bounded wait (about one second).  Returns false, and raises the abort flag, if the phase never completes;
// once the flag is up every later wait returns at once.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  if (*abort_flag) return false;
  const long long t0 = clock64();
  for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
    if (mbar_try_wait_suspend(bar, parity, 100000u)) return true;   // <= 0.1 ms per try
    if (*abort_flag) return false;
    if (clock64() - t0 > kWaitCycles) break;
  }
  *abort_flag = 1;
  atomicOr(&g_dmoq_tc_status, 1);
  return false;
}
// One thread announces `bytes` of bulk-copy traffic on the barrier (and arrives on it) ...
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// ... and starts the copies: global -> this block's shared memory, completion counted in bytes on the barrier.
// Both addresses 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
// Time-bounded wait that ignores the abort flag: used at teardown so that no bulk copy is still writing into
// this block's shared memory when it exits.
__device__ __forceinline__ void mbar_wait_quiet(uint64_t* bar, uint32_t parity) {
  const long long t0 = clock64();
  while (!mbar_try_wait_suspend(bar, parity, 100000u)) {
    if (clock64() - t0 > kWaitCycles) break;
  }
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tc_mma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0), "r"(0), "r"(0), "r"(0)
      : "memory");
}
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0), "r"(0), "r"(0), "r"(0)
      : "memory");
}
__device__ __forceinline__ void tc_mma_f8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0), "r"(0), "r"(0), "r"(0)
      : "memory");
}
// 16 lanes x 64 columns: register 4m+2h+e of thread t = lane base + t/4 + 8h, column base + 8m + 2(t%4) + e
__device__ __forceinline__ void tc_ld16x256(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.16x256b.x8.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// 32 lanes x 32 columns of one 32-bit value
__device__ __forceinline__ void tc_st32_fill(uint32_t taddr, uint32_t v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1};"
      ::"r"(taddr), "r"(v)
      : "memory");
}
// 32 lanes x 8 columns: the narrow form keeps only 8 registers busy where the caller is short of them
__device__ __forceinline__ void tc_st8_fill(uint32_t taddr, uint32_t v) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%1,%1,%1,%1,%1,%1,%1};" ::"r"(taddr), "r"(v) : "memory");
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// packed fp32 pairs (each half an IEEE round-to-nearest fma)
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }
__device__ __forceinline__ void bar_sync_epi() { asm volatile("bar.sync 1, %0;" ::"n"(32 * kEpiWarps) : "memory"); }
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
  return d;
}
__device__ __forceinline__ void cp_async_n(void* smem, const void* gmem, int bytes) {
  if (bytes == 16) asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem)), "l"(gmem));
  else if (bytes == 8) asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(smem_u32(smem)), "l"(gmem));
  else asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(smem)), "l"(gmem));
}

// K-major, 128-byte swizzle: tile row r is 128 bytes; 16-byte chunk c lives at slot c ^ (r & 7);
// groups of 8 rows are 1024 bytes apart (the descriptor's stride byte offset).
__device__ __forceinline__ uint32_t swz128(int r, int c) { return (uint32_t)(r * 128 + ((c ^ (r & 7)) << 4)); }
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr) {
  return (uint64_t)((smem_addr >> 4) & 0x3FFF) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
         ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}

// Codeword tables for the in-register expansion: up to 16 one-byte codewords in four registers.
struct Lut {
  uint32_t w[4];
};

// 16 consecutive weights (one 16-byte chunk of the operand row) from their packed indices.
template <int BIT>
__device__ __forceinline__ uint4 expand16(const uint32_t* raw, const Lut& lut, bool identity) {
  uint32_t o[4];
  if (BIT == 8) {  // raw[0..3] = 16 index bytes
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      if (identity) {
        o[q] = raw[q] ^ 0x80808080u;  // index - 128 as int8
      } else {
        o[q] = 0;  // general 256-entry tables take the warp-level MMA path
      }
    }
  } else if (BIT == 4) {  // raw[0..1] = 16 nibbles
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const uint32_t w = raw[h];
      const uint32_t sel = w & 0x77777777u, hi = (w >> 1) & 0x44444444u;
      const uint32_t lo_a = prmt(lut.w[0], lut.w[1], sel), hi_a = prmt(lut.w[2], lut.w[3], sel);
      const uint32_t lo_b = prmt(lut.w[0], lut.w[1], sel >> 16), hi_b = prmt(lut.w[2], lut.w[3], sel >> 16);
      o[2 * h + 0] = prmt(lo_a, hi_a, (hi & 0xFFFFu) | 0x3210u);
      o[2 * h + 1] = prmt(lo_b, hi_b, (hi >> 16) | 0x3210u);
    }
  } else {  // 1- and 2-bit pools arrive widened: raw[0..1] = 16 four-bit fields, each holding one code
    o[0] = prmt(lut.w[0], lut.w[0], raw[0]);        // prmt reads the low four selector nibbles only
    o[1] = prmt(lut.w[0], lut.w[0], raw[0] >> 16);
    o[2] = prmt(lut.w[0], lut.w[0], raw[1]);
    o[3] = prmt(lut.w[0], lut.w[0], raw[1] >> 16);
  }
  return make_uint4(o[0], o[1], o[2], o[3]);
}

// Eight widened codes (one 32-bit word of 4-bit fields) -> eight fp16 codewords (16 bytes) of a codebook with at
// most four entries held in two registers: code c selects bytes (2c, 2c+1).
__device__ __forceinline__ uint4 expand8_f16(uint32_t w, uint32_t lut0, uint32_t lut1) {
  const uint32_t sl = (w & 0x0F0F0F0Fu) * 34u + 0x10101010u;          // selector bytes of codes 0, 2, 4, 6
  const uint32_t sh = ((w >> 4) & 0x0F0F0F0Fu) * 34u + 0x10101010u;   // ... of codes 1, 3, 5, 7
  uint32_t o[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) o[j] = prmt(lut0, lut1, prmt(sl, sh, (uint32_t)(j | ((4 + j) << 4))));
  return make_uint4(o[0], o[1], o[2], o[3]);
}

struct Smem {
  // operand ring, 1024-byte aligned tiles
  uint8_t a[kStages][kTileB];
  uint8_t b[kStages][kTileB];
  uint8_t raw[kStages][kBN * 64 + kRawPad];   // packed indices of one group (<= 64 bytes per row: 4-bit), two segments
  uint8_t out[kBM * kOutPitch];
  float sc_norm[kScaleRing][kBN];   // column norms of a group, tile column order
  float sc_xs[kScaleRing][kBM];     // row scales of a group
  uint64_t full[kStages], empty[kStages], acc_full[kAccBufs], acc_empty[kAccBufs], raw_full[kStages];
  uint32_t tmem_base;
  int abort_flag;
};

template <int N>
__device__ __forceinline__ void reg_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N>
__device__ __forceinline__ void reg_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }

template <int MODE, int BIT, int EPI>
__global__ void __launch_bounds__(kThreads, 1) gemm_tc_kernel(TcArgs a) {
  extern __shared__ uint8_t smem_raw[];
  Smem& S = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  volatile int* abort_flag = &S.abort_flag;
  constexpr int BPG = (BIT <= 2) ? 64 : 16 * BIT;    // index bytes per row per group (1/2-bit codes come widened to 4 bits)
  // fp16 operands: a 128-byte operand row holds 64 columns, so a 128-wide group takes two operand steps
  constexpr int SUB = (MODE == DMOQ_A16) ? 2 : 1;
  constexpr int ES = (MODE == DMOQ_A16) ? 2 : 1;
  constexpr int kMmaWarp = kEpiWarps + kProdWarps;

  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&S.full[s], kProdWarps);
      mbar_init(&S.empty[s], 1);
      mbar_init(&S.raw_full[s], 1);
    }
    for (int b = 0; b < kAccBufs; ++b) {
      mbar_init(&S.acc_full[b], 1);
      mbar_init(&S.acc_empty[b], kEpiWarps);
    }
    S.abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == kMmaWarp) {  // the MMA warp owns the TMEM allocation
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&S.tmem_base)),
                 "r"(kAccBufs * kBN));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = S.tmem_base;
  if (MODE == DMOQ_A8) {
    if (warp < kEpiWarps) {  // bias every accumulator buffer
      const uint32_t t0 = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + (warp >> 2) * 64;
#pragma unroll
      for (int b = 0; b < kAccBufs; ++b) {
        tc_st32_fill(t0 + b * kBN, kMagicBits);
        tc_st32_fill(t0 + b * kBN + 32, kMagicBits);
      }
      tc_wait_st();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
  }

  const int n_tiles = a.n_tiles[a.pool];
  const DmoqTile* tiles = a.tiles + a.n_tiles[DMOQ_MAX_POOLS + a.pool];
  const int NB = a.is_down ? a.hidden / kBN : a.inter / (kBN / 2);
  const int G = a.is_down ? a.inter / kG : a.hidden / kG;
  const int n_total = a.is_down ? a.hidden : a.n_members * 2 * a.inter;
  const int n_work = n_tiles * NB;
  const int stride_w = gridDim.x;
  const int n_items = (int)blockIdx.x < n_work ? (n_work - 1 - (int)blockIdx.x) / stride_w + 1 : 0;
  const DmoqTile kNoTile{0, 0, 0, 0};
  auto tile_of = [&](int item) {   // item index of this CTA -> tile record (clamped past the end)
    const int w = blockIdx.x + item * stride_w;
    return (item < n_items) ? tiles[w / NB] : kNoTile;
  };

  if (warp < kEpiWarps) {
    // =========================================================================== epilogue warps
    // Accumulators are read with the 16x256b shape (the fragment layout of an m16n8 MMA accumulator): thread t of
    // a warp holds, for each of its four rows  quarter*32 + t/4 + 8j  (j = 0..3), the sixteen columns
    // half*64 + 8m + 2(t%4) + {0,1}  (m = 0..7).  A thread therefore needs only 16 column norms per group
    // (8-byte loads shared by the lanes of equal t%4) instead of 64 warp-wide broadcast loads.
    reg_inc<kRegsEpi>();
    const int quarter = warp & 3, half = warp >> 2;
    const int etid = warp * 32 + lane;
    const int t4 = lane & 3;
    const int row_b = quarter * 32 + (lane >> 2);      // rows row_b + 8j
    const int col_b = half * 64 + 2 * t4;              // tile columns col_b + 8m + e
    uint32_t ia = 0;                                  // groups consumed so far
    DmoqTile next = tile_of(0);
    PROF_DECL;
#ifdef DMOQ_TC_PROFILE
    const long long prof_start = clock64();
#endif
    for (int item = 0; item < n_items; ++item) {
      const DmoqTile tile = next;
      next = tile_of(item + 1);                       // in flight while this item is processed
      const int nb = (blockIdx.x + item * stride_w) % NB;

      float2 total2[32];                              // [j][m]: columns (e = 0, 1) of row j, column block m
#pragma unroll
      for (int c = 0; c < 32; ++c) total2[c] = make_float2(0.f, 0.f);

      for (int g = 0; g < G; ++g, ++ia) {
        const uint32_t b = ia % kAccBufs, ph = (ia / kAccBufs) & 1;
        const uint32_t slot = ia % kScaleRing;
        // The group's scales were stored before its producers arrived on full[]; the MMA warp saw that arrival
        // before it committed acc_full[], so they are visible here.  A slot is rewritten kScaleRing groups later and
        // the producers run at most kStages + kAccBufs groups ahead of an unreleased accumulator: still intact.
        PROF_BEGIN();
        mbar_wait(&S.acc_full[b], ph, abort_flag);    // on a timeout the flag is up and the data is void
        PROF_END(1);
        tc_fence_after();
        PROF_BEGIN();
        const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + b * kBN + half * 64;
        uint32_t v0[32], v1[32];                      // rows j = 0,1 and j = 2,3
        tc_ld16x256(taddr, v0);
        tc_ld16x256(taddr + (16u << 16), v1);
        float xs[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) xs[j] = (MODE == DMOQ_A16) ? 1.f : S.sc_xs[slot][row_b + 8 * j];
        float off[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) off[j] = (MODE == DMOQ_A8) ? -kMagicFloat * xs[j] : 0.f;
        const float2* nrm2 = reinterpret_cast<const float2*>(&S.sc_norm[slot][col_b]);
        tc_wait_ld();
        PROF_END(4);
        PROF_BEGIN();
        if (MODE == DMOQ_A8) {   // re-arm the bias for the buffer's next use
#pragma unroll
          for (int q = 0; q < 8; ++q) tc_st8_fill(taddr + 8 * q, kMagicBits);
        }
        PROF_END(5);
        PROF_BEGIN();
#pragma unroll
        for (int m = 0; m < 8; ++m) {
          const float2 n2 = nrm2[4 * m];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint32_t(&v)[32] = (j >> 1) ? v1 : v0;
            const int i = 4 * m + 2 * (j & 1);
            const float2 f = make_float2(__uint_as_float(v[i]), __uint_as_float(v[i + 1]));
            // INT8: (acc_biased - M) * xs in one fma with the exact constant -M*xs (2 x 11 significant bits);
            // e4m3: acc * xs (adding +0 changes nothing: the product is never -0 unless acc is, and then total decides)
            // fp16 operands: no row scale, acc * norm + total
            const float2 t2 = (MODE == DMOQ_A16) ? f : fma2(f, make_float2(xs[j], xs[j]), make_float2(off[j], off[j]));
            total2[j * 8 + m] = fma2(t2, n2, total2[j * 8 + m]);   // (acc*xs)*norm + total, last step fused
          }
        }
        if (MODE == DMOQ_A8 && a.partials != nullptr) {
          const int n_out = a.is_down ? a.hidden : 2 * a.inter;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int row = row_b + 8 * j;
            if (row < tile.rows) {
              const uint32_t(&v)[32] = (j >> 1) ? v1 : v0;
#pragma unroll
              for (int m = 0; m < 8; ++m)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                  const int col = col_b + 8 * m + e;
                  const int n = a.is_down ? nb * kBN + col : (col & 1) * a.inter + nb * (kBN / 2) + (col >> 1);
                  a.partials[((size_t)(tile.row0 + row) * n_out + n) * G + g] = (int32_t)(v[4 * m + 2 * (j & 1) + e] - kMagicBits);
                }
            }
          }
        }
        // release the accumulator buffer only now: the bias stores complete behind the scale math, and with four
        // buffers the tensor pipe does not wait for this one
        if (MODE == DMOQ_A8) tc_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&S.acc_empty[b]);
        PROF_END(6);
      }

      // ---- tile epilogue through the staging tile
      PROF_BEGIN();
      if (EPI == DMOQ_EPI_SILU) {
        bar_sync_epi();  // the previous item's copy-out has finished reading the staging tile
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
          for (int m = 0; m < 8; ++m) {
            const float gate = __half2float(__float2half_rn(total2[j * 8 + m].x));
            const float up = __half2float(__float2half_rn(total2[j * 8 + m].y));
            // fast exp and reciprocal (a few fp32 ulps) ahead of the fp16 rounding: a floating-point stage
            const float sg = __half2float(__float2half_rn(__fdividef(gate, 1.0f + __expf(-gate))));
            *reinterpret_cast<__half*>(&S.out[(row_b + 8 * j) * kOutPitch + (half * 32 + 4 * m + t4) * 2]) =
                __float2half_rn(__fmul_rn(sg, up));
          }
        bar_sync_epi();
        __half* out = reinterpret_cast<__half*>(a.out);
        for (int i = etid; i < kBM * 8; i += 32 * kEpiWarps) {
          const int rr = i >> 3, ch = i & 7;
          if (rr < tile.rows)
            *reinterpret_cast<uint4*>(out + (size_t)(tile.row0 + rr) * a.out_stride + nb * 64 + ch * 8) =
                *reinterpret_cast<const uint4*>(&S.out[rr * kOutPitch + ch * 16]);
        }
      } else if (EPI == DMOQ_EPI_PLAIN && !a.is_down) {
        __half* out = reinterpret_cast<__half*>(a.out);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int row = row_b + 8 * j;
          if (row < tile.rows) {
#pragma unroll
            for (int m = 0; m < 8; ++m) {
              const int oc = nb * (kBN / 2) + half * 32 + 4 * m + t4;   // gate column; the up column is inter further
              out[(size_t)(tile.row0 + row) * a.out_stride + oc] = __float2half_rn(total2[j * 8 + m].x);
              out[(size_t)(tile.row0 + row) * a.out_stride + a.inter + oc] = __float2half_rn(total2[j * 8 + m].y);
            }
          }
        }
      } else {
        bar_sync_epi();
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int row = row_b + 8 * j;
          float wgt = 0.f;
          if (EPI == DMOQ_EPI_WEIGHTED && row < tile.rows) wgt = a.row_weight[tile.row0 + row];
#pragma unroll
          for (int m = 0; m < 8; ++m) {
            uint32_t pk;
            const __half2 h2 = __floats2half2_rn(total2[j * 8 + m].x, total2[j * 8 + m].y);   // the fp16 output
            if (EPI == DMOQ_EPI_WEIGHTED) {   // -> bf16, times the routing weight in fp32, -> bf16
              const float2 hf = __half22float2(h2);
              const float2 bf = __bfloat1622float2(__floats2bfloat162_rn(hf.x, hf.y));
              const __nv_bfloat162 o2 = __floats2bfloat162_rn(__fmul_rn(bf.x, wgt), __fmul_rn(bf.y, wgt));
              pk = *reinterpret_cast<const uint32_t*>(&o2);
            } else {
              pk = *reinterpret_cast<const uint32_t*>(&h2);
            }
            *reinterpret_cast<uint32_t*>(&S.out[row * kOutPitch + (col_b + 8 * m) * 2]) = pk;
          }
        }
        bar_sync_epi();
        uint16_t* out = reinterpret_cast<uint16_t*>(a.out);
        for (int i = etid; i < kBM * 16; i += 32 * kEpiWarps) {
          const int rr = i >> 4, ch = i & 15;
          if (rr < tile.rows)
            *reinterpret_cast<uint4*>(out + (size_t)(tile.row0 + rr) * a.out_stride + nb * kBN + ch * 8) =
                *reinterpret_cast<const uint4*>(&S.out[rr * kOutPitch + ch * 16]);
        }
      }
      PROF_END(2);
    }
#ifdef DMOQ_TC_PROFILE
    prof_acc[3] = clock64() - prof_start;
#endif
    PROF_FLUSH(0, warp == 0);
  } else if (warp < kMmaWarp) {
    // =========================================================================== producer warps
    reg_dec<kRegsProd>();
    const int pt = tid - 32 * kEpiWarps;              // 0..255
    Lut lut;
#pragma unroll
    for (int q = 0; q < 4; ++q) lut.w[q] = 0;
    float lut_step = 0.f;          // fp16 operands, uniform 8-bit codebook: codeword i = (i - 128) * step
    if (MODE == DMOQ_A16 && BIT == 8) lut_step = __half2float(reinterpret_cast<const __half*>(a.lut)[129]);
    if (MODE == DMOQ_A16) {        // up to four fp16 codewords in two registers
      for (int i = 0; i < (1 << BIT) && i < 4; ++i)
        lut.w[i >> 1] |= (uint32_t)reinterpret_cast<const uint16_t*>(a.lut)[i] << (16 * (i & 1));
    } else if (!(BIT == 8)) {
      for (int i = 0; i < (1 << BIT); ++i) lut.w[i >> 2] |= (uint32_t)a.lut[i] << (8 * (i & 3));
    }
    // chunk ownership: kCPT (row, 16-byte chunk) pairs per thread and stage, chosen so that a warp's
    // stores fall on distinct shared-memory bank groups
    auto own_row = [&](int i) { return (pt >> 3) + 32 * i; };
    auto own_chunk = [&](int) { return pt & 7; };
    // Packed indices arrive by bulk copy: gate_up tiles as two 64-row segments (gate rows, then up rows, kRawPad
    // bytes apart), down tiles as one 128-row segment.  Tile row -> byte offset of its BPG index bytes:
    auto raw_off = [&](int row) {
      return a.is_down ? row * BPG : ((row & 1) * (64 * BPG + kRawPad) + (row >> 1) * BPG);
    };
    const int xs_per_row = a.a_stride / kG;
    // threads 0-127 stage the row scale of tile row pt, threads 128-255 the norm of tile column pt - 128
    const bool stages_xs = pt < kBM;
    const int sc_i = pt & (kBM - 1);

    PROF_DECL;
    // the scale value travels in a register from the issue of a group to its publication kLag groups later
    uint16_t sc_q[kLag + 1];
#pragma unroll
    for (int i = 0; i <= kLag; ++i) sc_q[i] = 0;

    auto publish = [&](uint32_t j, int qi) {   // qi: position of group j's scale in the register queue
      const int s = j % kStages;
      if (BIT != 8) {
#ifdef DMOQ_TC_PROFILE
        const long long prof_r0 = clock64();
#endif
        mbar_wait(&S.raw_full[s], (j / kStages) & 1, abort_flag);   // the bulk copy of this group's indices has landed
#ifdef DMOQ_TC_PROFILE
        const long long prof_r1 = clock64();
        prof_acc[5] += prof_r1 - prof_r0;
#endif
#pragma unroll
        for (int i = 0; i < kCPT; ++i) {
          const int row = own_row(i), ch = own_chunk(i);
          if (MODE == DMOQ_A16) {   // eight fp16 codewords per chunk: this step covers half hh of the group's columns
            const uint32_t w = *reinterpret_cast<const uint32_t*>(&S.raw[s][raw_off(row) + (j % SUB) * 32 + ch * 4]);
            *reinterpret_cast<uint4*>(&S.b[s][swz128(row, ch)]) = expand8_f16(w, lut.w[0], lut.w[1]);
          } else {
            const uint2 v = *reinterpret_cast<const uint2*>(&S.raw[s][raw_off(row) + ch * 8]);
            const uint32_t raw[2] = {v.x, v.y};
            *reinterpret_cast<uint4*>(&S.b[s][swz128(row, ch)]) = expand16<BIT>(raw, lut, false);
          }
        }
#ifdef DMOQ_TC_PROFILE
        prof_acc[6] += clock64() - prof_r1;
#endif
      } else if (MODE == DMOQ_A16) {   // uniform 8-bit codebook: codeword = fp16((index - 128) * step), exact in fp32
#pragma unroll
        for (int i = 0; i < kCPT; ++i) {
          const int row = own_row(i), ch = own_chunk(i);
          const uint2 v = *reinterpret_cast<const uint2*>(&S.raw[s][row * 64 + ch * 8]);
          const uint32_t wv[2] = {v.x, v.y};
          uint32_t o[4];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int b0 = (int)((wv[q >> 1] >> (16 * (q & 1))) & 255u) - 128;
            const int b1 = (int)((wv[q >> 1] >> (16 * (q & 1) + 8)) & 255u) - 128;
            const __half2 h2 = __floats2half2_rn(__fmul_rn((float)b0, lut_step), __fmul_rn((float)b1, lut_step));
            o[q] = *reinterpret_cast<const uint32_t*>(&h2);
          }
          *reinterpret_cast<uint4*>(&S.b[s][swz128(row, ch)]) = make_uint4(o[0], o[1], o[2], o[3]);
        }
      } else {
#pragma unroll
        for (int i = 0; i < kCPT; ++i) {
          uint4* p = reinterpret_cast<uint4*>(&S.b[s][swz128(own_row(i), own_chunk(i))]);
          uint4 v = *p;
          uint32_t raw[4] = {v.x, v.y, v.z, v.w};
          *p = expand16<8>(raw, lut, true);
        }
      }
      const uint32_t slot = (j / SUB) % kScaleRing;   // one slot per group (both steps of an fp16 group store the same values)
      uint16_t sc_h = sc_q[0];
#pragma unroll
      for (int i = 1; i <= kLag; ++i) {
        if (qi == i) sc_h = sc_q[i];
      }
      (stages_xs ? S.sc_xs[slot] : S.sc_norm[slot])[sc_i] = __half2float(__ushort_as_half(sc_h));
#ifdef DMOQ_TC_PROFILE
      const long long prof_f0 = clock64();
#endif
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(&S.full[s]);
#ifdef DMOQ_TC_PROFILE
      prof_acc[7] += clock64() - prof_f0;
#endif
    };

    // row bookkeeping of one work item: table rows this thread copies and the row whose scale it stages
    struct Rows {
      int cp[kCPT];
      int own;
    };
    auto rows_of = [&](const DmoqTile& t) {
      Rows rw;
#pragma unroll
      for (int i = 0; i < kCPT; ++i) {
        const int rr = (pt >> 3) + 32 * i;
        rw.cp[i] = rr < t.rows ? (a.a_row ? a.a_row[t.row0 + rr] : t.row0 + rr) : -1;
      }
      rw.own = (stages_xs && sc_i < t.rows) ? (a.a_row ? a.a_row[t.row0 + sc_i] : t.row0 + sc_i) : -1;
      return rw;
    };

    uint32_t it = 0, done = 0;    // operand steps issued / published (SUB steps per group)
#ifdef DMOQ_TC_PROFILE
    const long long prof_start = clock64();
#endif
    DmoqTile t_next = tile_of(0), t_next2 = tile_of(1);
    Rows r_next = rows_of(t_next);
    for (int item = 0; item < n_items; ++item) {
      const DmoqTile tile = t_next;
      const Rows rw = r_next;
      t_next = t_next2;
      t_next2 = tile_of(item + 2);   // two items ahead: its rows are fetched one item ahead without a stall
      r_next = rows_of(t_next);
      const int nb = (blockIdx.x + item * stride_w) % NB;
      const int gg0 = a.is_down ? tile.rank * G : 0;
      const int seg0 = a.is_down ? nb * kBN : tile.rank * 2 * a.inter + nb * (kBN / 2);
      const int seg1 = a.is_down ? seg0 : seg0 + a.inter;
      const int own_n = a.is_down ? seg0 + sc_i : ((sc_i & 1) ? seg1 : seg0) + (sc_i >> 1);
      for (int gs = 0; gs < G * SUB; ++gs, ++it) {
        const int g = gs / SUB, hh = gs % SUB;   // group, and which 128-byte half of its operand rows
        const int s = it % kStages;
        PROF_BEGIN();
        mbar_wait(&S.empty[s], ((it / kStages) & 1) ^ 1, abort_flag);
        PROF_END(0);
        PROF_BEGIN();
#pragma unroll
        for (int i = 0; i < kCPT; ++i) {
          const int rr = (pt >> 3) + 32 * i, ch = pt & 7;
          const uint8_t* src = a.a_codes + ((size_t)(rw.cp[i] < 0 ? 0 : rw.cp[i]) * a.a_stride + (size_t)g * kG) * ES +
                               hh * 128 + ch * 16;
          cp_async16_zfill(&S.a[s][swz128(rr, ch)], src, rw.cp[i] >= 0);
        }
        PROF_END(4);
        if (BIT == 8 && MODE == DMOQ_A16) {   // eight index bytes per fp16 chunk into the raw ring (row pitch 64)
#pragma unroll
          for (int i = 0; i < kCPT; ++i) {
            const int row = own_row(i), ch = own_chunk(i);
            const int n = a.is_down ? seg0 + row : ((row & 1) ? seg1 : seg0) + (row >> 1);
            cp_async_n(&S.raw[s][row * 64 + ch * 8], a.idx + ((size_t)(gg0 + g) * n_total + n) * BPG + hh * 64 + ch * 8, 8);
          }
        } else if (BIT == 8) {   // 8-bit indices go straight into the operand tile (expanded in place)
#pragma unroll
          for (int i = 0; i < kCPT; ++i) {
            const int row = own_row(i), ch = own_chunk(i);
            const int n = a.is_down ? seg0 + row : ((row & 1) ? seg1 : seg0) + (row >> 1);
            cp_async_n(&S.b[s][swz128(row, ch)], a.idx + ((size_t)(gg0 + g) * n_total + n) * BPG + ch * 16, 16);
          }
        }
        cp_async_commit();
        // scale of this group: loaded now, stored when the group is published
#pragma unroll
        for (int i = kLag; i > 0; --i) sc_q[i] = sc_q[i - 1];
        if (stages_xs) sc_q[0] = (MODE != DMOQ_A16 && rw.own >= 0) ? a.a_scales[(size_t)rw.own * xs_per_row + g] : (uint16_t)0;
        else sc_q[0] = a.norm[(size_t)(gg0 + g) * n_total + own_n];
        if (it - done >= (uint32_t)kLag) {
          PROF_BEGIN();
          cp_async_wait<kLag>();
          PROF_END(1);
          PROF_BEGIN();
          publish(done++, kLag);
          PROF_END(2);
        }
      }
    }
    // drain: everything issued must be published so the MMA warp and the epilogue can finish
    while (done < it) {   // the queue is not rotated any more: group j sits at position it-1-j
      const uint32_t pending = it - done - 1;
      if (pending >= 1) cp_async_wait<1>(); else cp_async_wait<0>();
      publish(done, (int)pending);
      ++done;
    }
#ifdef DMOQ_TC_PROFILE
    prof_acc[3] = clock64() - prof_start;
#endif
    PROF_FLUSH(8, warp == kEpiWarps);
  } else {
    reg_dec<kRegsMma>();
    if (warp == kMmaWarp) {
      // ========================================================================= MMA warp
      constexpr uint32_t idesc_i8 = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kBN >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
      constexpr uint32_t idesc_f8 = (1u << 4) | (0u << 7) | (0u << 10) | ((uint32_t)(kBN >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
      constexpr uint32_t idesc_f16 = (1u << 4) | (0u << 7) | (0u << 10) | ((uint32_t)(kBN >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
      const uint32_t total_steps = (uint32_t)n_items * (uint32_t)G * (uint32_t)SUB;
      PROF_DECL;
#ifdef DMOQ_TC_PROFILE
      const long long prof_start = clock64();
#endif
      for (uint32_t it = 0; it < total_steps; ++it) {
        const int s = it % kStages;
        const uint32_t gi = it / SUB, hh = it % SUB;   // group (= accumulator use) and operand step inside it
        const uint32_t b = gi % kAccBufs;
        PROF_BEGIN();
        bool ok = mbar_wait(&S.full[s], (it / kStages) & 1, abort_flag);
        PROF_END(0);
        PROF_BEGIN();
        if (hh == 0) ok = mbar_wait(&S.acc_empty[b], ((gi / kAccBufs) & 1) ^ 1, abort_flag) && ok;
        PROF_END(1);
        tc_fence_after();
        if (lane == 0 && ok) {
          const uint64_t da = make_desc(smem_u32(&S.a[s][0]));
          const uint64_t db = make_desc(smem_u32(&S.b[s][0]));
          const uint32_t d = tmem_base + b * kBN;
#pragma unroll
          for (int k = 0; k < 4; ++k) {  // 32 bytes of K per instruction: +2 in 16-byte units
            if (MODE == DMOQ_A8) tc_mma_i8(d, da + 2 * k, db + 2 * k, idesc_i8, 1);  // buffer holds the bias
            else if (MODE == DMOQ_FP8) tc_mma_f8(d, da + 2 * k, db + 2 * k, idesc_f8, k > 0);
            else tc_mma_f16(d, da + 2 * k, db + 2 * k, idesc_f16, (hh > 0 || k > 0) ? 1u : 0u);
          }
          tc_commit(&S.empty[s]);
          if (hh == SUB - 1) tc_commit(&S.acc_full[b]);
        }
        __syncwarp();
      }
#ifdef DMOQ_TC_PROFILE
      prof_acc[3] = clock64() - prof_start;
#endif
      PROF_FLUSH(16, true);
    } else if (warp == kMmaWarp + 1 && BIT != 8) {
      // ========================================================================= index loader
      // One thread moves each group's packed indices into the raw ring with bulk copies as soon as the stage is
      // free: gate_up tiles as two 64-row segments (gate rows, up rows), down tiles as one 128-row segment.
      if (lane == 0) {
        uint32_t it = 0;
        for (int item = 0; item < n_items; ++item) {
          const DmoqTile tile = tile_of(item);
          const int nb = (blockIdx.x + item * stride_w) % NB;
          const int gg0 = a.is_down ? tile.rank * G : 0;
          const int seg0 = a.is_down ? nb * kBN : tile.rank * 2 * a.inter + nb * (kBN / 2);
          for (int gs = 0; gs < G * SUB; ++gs, ++it) {   // fp16 operands: both steps of a group get the group's indices
            const int g = gs / SUB;
            const int s = it % kStages;
            if (!mbar_wait(&S.empty[s], ((it / kStages) & 1) ^ 1, abort_flag)) break;
            const uint8_t* gsrc = a.idx + ((size_t)(gg0 + g) * n_total + seg0) * BPG;
            mbar_arrive_expect_tx(&S.raw_full[s], kBN * BPG);
            if (a.is_down) {
              bulk_g2s(&S.raw[s][0], gsrc, kBN * BPG, &S.raw_full[s]);
            } else {
              bulk_g2s(&S.raw[s][0], gsrc, 64 * BPG, &S.raw_full[s]);
              bulk_g2s(&S.raw[s][64 * BPG + kRawPad], gsrc + (size_t)a.inter * BPG, 64 * BPG, &S.raw_full[s]);
            }
          }
          if (*abort_flag) break;
        }
        // no bulk copy may still be in flight when the block exits (matters after an abort)
        for (uint32_t j = (it > (uint32_t)kStages ? it - kStages : 0u); j < it; ++j)
          mbar_wait_quiet(&S.raw_full[j % kStages], (j / kStages) & 1);
      }
      __syncwarp();
    }
  }

  // ---- teardown: all roles meet here, then the allocating warp releases TMEM
  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kAccBufs * kBN));
  }
}

template <int MODE, int BIT, int EPI>
int launch(const TcArgs& a, int work_cap, cudaStream_t s) {
  static DmoqOncePerDevice once;
  bool* configured = once.slot();
  if (configured == nullptr) return DMOQ_EDEVICE;
  const int bytes = (int)sizeof(Smem) + 1024;
  if (!*configured) {
    cudaFuncAttributes fa;
    if (cudaFuncGetAttributes(&fa, gemm_tc_kernel<MODE, BIT, EPI>) != cudaSuccess) return DMOQ_ELAUNCH;
    if (fa.numRegs != kRegsLaunch) return DMOQ_ELAUNCH;   // the role budgets were sized for this pool
    if (cudaFuncSetAttribute(gemm_tc_kernel<MODE, BIT, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess)
      return DMOQ_ELAUNCH;
    *configured = true;
  }
  int grid = dmoq_sm_count();
  if (grid > work_cap) grid = work_cap;
  if (grid < 1) grid = 1;
  gemm_tc_kernel<MODE, BIT, EPI><<<grid, kThreads, bytes, s>>>(a);
  return dmoq_launch_status();
}

template <int MODE, int BIT>
int launch_epi(const TcArgs& a, int epi, int work_cap, cudaStream_t s) {
  switch (epi) {
    case DMOQ_EPI_SILU: return launch<MODE, BIT, DMOQ_EPI_SILU>(a, work_cap, s);
    case DMOQ_EPI_WEIGHTED: return launch<MODE, BIT, DMOQ_EPI_WEIGHTED>(a, work_cap, s);
    case DMOQ_EPI_PLAIN: return launch<MODE, BIT, DMOQ_EPI_PLAIN>(a, work_cap, s);
    default: return DMOQ_EINVAL;
  }
}

template <int MODE>
int launch_bit(const TcArgs& a, int bit, int epi, int work_cap, cudaStream_t s) {
  switch (bit) {
    case 1: return launch_epi<MODE, 1>(a, epi, work_cap, s);
    case 2: return launch_epi<MODE, 2>(a, epi, work_cap, s);
    case 4: return launch_epi<MODE, 4>(a, epi, work_cap, s);
    case 8: return launch_epi<MODE, 8>(a, epi, work_cap, s);
    default: return DMOQ_EINVAL;
  }
}

}  // namespace

// True when the tensor-core kernel covers this pool/direction; other cases use the warp-level MMA kernel.
bool dmoq_tc_supported(const dmoq_pool_t& p, int is_down, int hidden) {
  if (p.mode == DMOQ_A16) {   // fp16 operands: codebooks of at most four entries (widened indices), or the uniform 8-bit one
    if (p.bit == 8) return p.identity_lut != 0;
    return p.bit <= 2 && (is_down ? p.dn_idx_wide : p.gu_idx_wide) != nullptr;
  }
  if (p.mode != DMOQ_A8 && p.mode != DMOQ_FP8) return false;
  if (p.bit == 8 && !(p.mode == DMOQ_A8 && p.identity_lut)) return false;
  if (p.bit <= 2 && (is_down ? p.dn_idx_wide : p.gu_idx_wide) == nullptr) return false;   // needs widened indices
  const int G = is_down ? p.inter / kG : hidden / kG;
  return G >= 1;
}

int dmoq_grouped_gemm_tc(const dmoq_route_t* route, const dmoq_pool_t& p, int pool_index, int is_down, int epilogue,
                         int hidden, const void* a_codes, const void* a_scales, int a_stride, void* out, int out_stride,
                         int32_t* partials, cudaStream_t s) {
  TcArgs a{};
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
  a.idx = p.bit <= 2 ? (is_down ? p.dn_idx_wide : p.gu_idx_wide) : (is_down ? p.dn_idx : p.gu_idx);
  a.norm = is_down ? p.dn_norm : p.gu_norm;
  a.lut = static_cast<const uint8_t*>(is_down ? p.dn_lut : p.gu_lut);
  a.identity_lut = p.identity_lut;
  a.a_codes = static_cast<const uint8_t*>(a_codes);
  a.a_scales = static_cast<const uint16_t*>(a_scales);
  a.a_stride = a_stride;
  a.out = out;
  a.out_stride = out_stride;
  a.partials = partials;
  const int nb = is_down ? hidden / kBN : p.inter / (kBN / 2);
  long long cap = (long long)route->tile_cap * nb;
  const int work_cap = cap > (1 << 30) ? (1 << 30) : (int)cap;
  if (p.mode == DMOQ_A8) return launch_bit<DMOQ_A8>(a, p.bit, epilogue, work_cap, s);
  if (p.mode == DMOQ_FP8) return launch_bit<DMOQ_FP8>(a, p.bit, epilogue, work_cap, s);
  switch (p.bit) {   // fp16 operands
    case 1: return launch_epi<DMOQ_A16, 1>(a, epilogue, work_cap, s);
    case 2: return launch_epi<DMOQ_A16, 2>(a, epilogue, work_cap, s);
    case 8: return launch_epi<DMOQ_A16, 8>(a, epilogue, work_cap, s);
    default: return DMOQ_EINVAL;
  }
}

#ifdef DMOQ_TC_PROFILE
extern "C" int dmoq_tc_profile(unsigned long long* out32, int reset) {
  if (cudaMemcpyFromSymbol(out32, g_tc_prof, sizeof(unsigned long long) * 32) != cudaSuccess) return DMOQ_EDEVICE;
  if (reset) {
    unsigned long long z[32] = {0};
    if (cudaMemcpyToSymbol(g_tc_prof, z, sizeof(z)) != cudaSuccess) return DMOQ_EDEVICE;
  }
  return DMOQ_OK;
}
#endif

int dmoq_img_status(int* out);

// Device status word of the tensor-core kernels (both kernel families): 0 = no bounded wait has ever timed out on
// this device.
extern "C" int dmoq_tc_status(int32_t* status_host) {
  if (!status_host) return DMOQ_EINVAL;
  int v = 0, w = 0;
  if (cudaMemcpyFromSymbol(&v, g_dmoq_tc_status, sizeof(int)) != cudaSuccess) return DMOQ_EDEVICE;
  const int rc = dmoq_img_status(&w);
  if (rc != DMOQ_OK) return rc;
  *status_host = v | w;
  return DMOQ_OK;
}
