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
// One persistent CTA per SM (640 threads with 256-column tiles, 768 with 128-column tiles):
//   warps 0-15   epilogue: warp w owns lanes 32*(w%4).. and columns 32*NH*(w/4).. of the group's accumulator and reads
//                them in the 16x256b shape: a thread holds four rows (i, i+8, i+16, i+24 of the lane quarter) and
//                16*NH columns, so a group costs it 16*NH column norms (64-bit shared loads, four addresses per warp)
//                and four row scales; (acc * row_scale) * col_norm goes into fp32 running totals as packed f32x2
//                fused multiply-adds on 64-bit registers; the buffer returns to the MMA thread as soon as its last
//                chunk is in registers.  At the end of a tile the fragments pass through a small swizzled staging
//                block (stmatrix) and leave as full lines: SiLU*up / plain / weighted rows.
//   loader warp  one thread issues, per operand step, the TMA copies of the A tile (128 rows of the routed-order
//                activation-code table) and of the B tile, and the bulk copy of the group's column norms
//   FP4 only     four warps store the rows' e8m0 block scales into TMEM (tcgen05.st) for the block-scaled MMA
//   MMA warp     one thread issues tcgen05.mma: kind::i8 / f8f6f4 / f16, or kind::mxf4nvf4.block_scale (scale_vec 2X);
//                an INT8 group starts with one or two MMAs of constant unsigned tiles (the "bias", see kBias1)
// All shared-memory operands are 32-bit shared-window addresses derived from one base kept opaque to the optimiser.
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
#define PROF_BEGIN2() const long long prof_t1 = clock64()
#define PROF_END2(i) prof_acc[i] += clock64() - prof_t1
#define PROF_FLUSH(base, cond)                                                        \
  if ((cond) && blockIdx.x == 0 && lane == 0) {                                       \
    for (int i_ = 0; i_ < 8; ++i_) atomicAdd(&g_img_prof[(base) + i_], (unsigned long long)prof_acc[i_]); \
  }
#else
#define PROF_DECL
#define PROF_BEGIN()
#define PROF_END(i)
#define PROF_BEGIN2()
#define PROF_END2(i)
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
// INT8 groups start with a "bias" MMA (accumulate off) of two constant unsigned tiles, so every int32 sum lands in
// [0, 2^23): such a bit pattern read as fp32 is the denormal (bias + sum) * 2^-149, exactly, and one fused
// multiply-add removes the bias and applies the row scale: (bias + sum) * 2^-149 * (xs * 2^100) - bias * 2^-49 * xs
// = sum * xs * 2^-49, rounded like sum * xs itself; the norm image carries the other 2^49.  No integer->float
// conversion and no accumulator re-initialisation by the epilogue.  The bias needs few significant bits (its
// product with an 11-bit row scale must be exact in fp32) and must exceed the largest |sum|:
//   one bias MMA  (K = 32):  2 * sum_16(a_j * b_j) = 0x1F8100 = 2064640 >= 128*127*127   (codeword tables clamp to +-127)
//   two bias MMAs (K = 64):  4 * sum_16(a_j * b_j) = 2^21             >= 128*127*128   (identity table: -128 occurs)
// The operand bytes repeat with period 16 along K, so the 128-byte swizzle leaves them where they are, and every
// row is the same, so one 8-row block of 1 KB serves all rows (stride 0 between 8-row groups in the descriptor).
constexpr uint32_t kBias1 = 0x1F8100u, kBias2 = 0x200000u;
constexpr float kXsScale = 1.2676506002282294e30f;           // 2^100
constexpr float kBiasToOff = 1.7763568394002505e-15f;        // 2^-49
__constant__ uint8_t kBiasBytes[4][16] = {
    {253, 229, 255, 255, 255, 255, 255, 255, 255, 255, 255, 255, 255, 255, 255, 255},   // one MMA: A operand
    {254, 252, 255, 255, 255, 255, 255, 255, 255, 255, 255, 255, 255, 255, 255, 255},   // one MMA: B operand
    {151, 151, 151, 151, 151, 151, 151, 151, 151, 151, 151, 151, 151, 151, 3, 255},     // two MMAs: A operand
    {217, 217, 217, 217, 217, 217, 217, 217, 217, 217, 217, 217, 217, 217, 175, 255}};  // two MMAs: B operand
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
  int n_bias;                 // A8: bias MMAs per group (1, or 2 when the pool's weight codes reach -128)
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
  int out_lines;              // the output rows are 16-byte aligned: the down epilogue may store whole lines
  uint32_t sfb_word;          // FP4: the weight block scale byte 127+E0 replicated four times
};

// ------------------------------------------------------------------------------------------------ PTX wrappers
// Every shared-memory operand below is an address in the shared window (32 bits): the kernel derives them all from
// one base it computed once, so no loop recomputes a pointer.
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_try_wait_suspend(uint32_t bar, uint32_t parity, uint32_t ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(ns)
      : "memory");
  return ok != 0;
}
// Bounded wait (about one second).  Returns false, and raises the abort flag, if the phase never completes; once
// the flag is up every later wait returns at once.
__device__ __forceinline__ int abort_get(uint32_t flag) {
  int v;
  asm volatile("ld.volatile.shared.u32 %0, [%1];" : "=r"(v) : "r"(flag) : "memory");
  return v;
}
__device__ __forceinline__ void abort_set(uint32_t flag) {
  asm volatile("st.volatile.shared.u32 [%0], %1;" ::"r"(flag), "r"(1) : "memory");
}
// Bounded wait (about one second).  Returns false, and raises the abort flag, if the phase never completes; once
// the flag is up every later wait returns at once.  A waiting warp shares its scheduler with epilogue warps: it
// probes, sleeps a little where its role can afford the latency, and looks at the abort flag and the clock only
// every 32nd probe.
template <int SLEEP_NS = 0>
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, uint32_t abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  if (abort_get(abort_flag)) return false;
  const long long t0 = clock64();
  for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
    if (mbar_try_wait_suspend(bar, parity, 100000u)) return true;
    if (SLEEP_NS > 0) __nanosleep(SLEEP_NS);
    if ((spin & 31u) == 31u) {
      if (abort_get(abort_flag)) return false;
      if (clock64() - t0 > kWaitCycles) break;
    }
  }
  abort_set(abort_flag);
  atomicOr(&g_dmoq_img_status, 1);
  return false;
}
// Time-bounded wait that ignores the abort flag: used at teardown so that no bulk copy is still writing into this
// block's shared memory when it exits.
__device__ __forceinline__ void mbar_wait_quiet(uint32_t bar, uint32_t parity) {
  const long long t0 = clock64();
  while (!mbar_try_wait_suspend(bar, parity, 100000u)) {
    if (clock64() - t0 > kWaitCycles) break;
  }
}
// 2-D tile of a tensor map -> this block's shared memory; completion counted in bytes on the barrier.  The map lies
// over this GPU's own memory; the inner coordinate x is a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void bulk_g2s(uint32_t smem_dst, const void* gmem_src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_dst), "l"(gmem_src), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
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
// unsigned 8-bit x unsigned 8-bit into the int32 accumulator (the bias MMAs of the INT8 mode)
__device__ __forceinline__ void tc_mma_u8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
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
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// 32 lanes x 4 columns: thread t writes its four values to lane base + t
__device__ __forceinline__ void tc_st4(uint32_t taddr, uint32_t v0, uint32_t v1, uint32_t v2, uint32_t v3) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1,%2,%3,%4};" ::"r"(taddr), "r"(v0), "r"(v1), "r"(v2), "r"(v3)
               : "memory");
}
// 16 lanes x 16 columns: thread t = 4*i + q of the warp receives lane base+i (r0,r1,r4,r5) and lane base+i+8
// (r2,r3,r6,r7) at columns 2q, 2q+1 (r0..r3) and 8+2q, 9+2q (r4..r7); the lane base is the warp's quarter or 16 above it
__device__ __forceinline__ void tc_ld16x16(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.16x256b.x2.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
}
// Four 8x8 matrices of 16-bit values from accumulator-fragment registers (thread t holds row t/4, columns 2(t%4),
// 2(t%4)+1 of each) to shared memory; thread t supplies the address of row t%8 of matrix t/8 (16 bytes per row).
__device__ __forceinline__ void stmatrix_x4(uint32_t addr, uint32_t r0, uint32_t r1, uint32_t r2, uint32_t r3) {
  asm volatile("stmatrix.sync.aligned.m8n8.x4.shared.b16 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(r0), "r"(r1), "r"(r2), "r"(r3)
               : "memory");
}
__device__ __forceinline__ uint4 lds_v4(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
  return v;
}
// Eight output rows of a warp leave as full lines: CH 8x8 matrices of fp16 pairs (w[mi]: this thread's pair of matrix
// mi, accumulator-fragment layout) go through the warp's staging block, 16-byte chunks XOR-swizzled against bank
// conflicts, and come back 16 bytes per thread, so one store instruction covers whole row segments of 16*CH bytes
// instead of eight 16-byte pieces.  Row r of the eight is stored to dst + r * stride if r < rows_left.
template <int CH>
__device__ __forceinline__ void store_rows_staged(uint32_t stage, int lane, const uint32_t (&w)[CH], uint16_t* dst, size_t stride,
                                                  int rows_left) {
  static_assert(CH == 4 || CH == 8, "four or eight 16-byte chunks per staged row");
  const int sr = lane & 7, smi = lane >> 3;                    // stmatrix: this lane addresses row sr of matrix smi
  __syncwarp();                                                // the previous use of the block has been read back
#pragma unroll
  for (int gi = 0; gi < CH / 4; ++gi) {
    const int pc = (4 * gi + smi) ^ ((CH == 8) ? sr : (sr >> 1));
    stmatrix_x4(stage + (uint32_t)(sr * (CH * 16) + pc * 16), w[4 * gi], w[4 * gi + 1], w[4 * gi + 2], w[4 * gi + 3]);
  }
  __syncwarp();
#pragma unroll
  for (int i = 0; i < CH / 4; ++i) {
    const int u = i * 32 + lane, r = u / CH, cl = u % CH;
    const uint4 v4 = lds_v4(stage + (uint32_t)(r * (CH * 16) + ((cl ^ ((CH == 8) ? r : (r >> 1))) * 16)));
    if (r < rows_left) *reinterpret_cast<uint4*>(dst + (size_t)r * stride + cl * 8) = v4;
  }
}
// Pairs of fp32 values live in 64-bit registers from the load to the last fused multiply-add, so that no
// pack / unpack moves stand between the packed instructions.
typedef unsigned long long f32x2_t;
__device__ __forceinline__ f32x2_t lds_x2(uint32_t addr) {
  f32x2_t v;
  asm volatile("ld.shared.b64 %0, [%1];" : "=l"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ f32x2_t pack_x2(uint32_t lo, uint32_t hi) {
  f32x2_t v;
  asm("mov.b64 %0, {%1,%2};" : "=l"(v) : "r"(lo), "r"(hi));
  return v;
}
// the same, kept in program order with the other volatile statements: for registers an asynchronous TMEM load
// fills, which must not be read before the tcgen05.wait::ld that precedes this statement
__device__ __forceinline__ f32x2_t pack_x2_after_wait(uint32_t lo, uint32_t hi) {
  f32x2_t v;
  asm volatile("mov.b64 %0, {%1,%2};" : "=l"(v) : "r"(lo), "r"(hi));
  return v;
}
__device__ __forceinline__ float2 unpack_x2(f32x2_t v) {
  float2 f;
  asm("mov.b64 {%0,%1}, %2;" : "=f"(f.x), "=f"(f.y) : "l"(v));
  return f;
}
__device__ __forceinline__ f32x2_t fma_x2(f32x2_t a, f32x2_t b, f32x2_t c) {
  f32x2_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}

// K-major, 128-byte swizzle: tile row r is 128 bytes; 16-byte chunk c lives at slot c ^ (r & 7); groups of 8 rows
// are 1024 bytes apart (the descriptor's stride byte offset).  The TMA copy writes the same pattern.
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr) {
  return (uint64_t)((smem_addr >> 4) & 0x3FFF) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
         ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}

// the same with stride 0 between 8-row groups: every group of rows reads the one 1 KB block at smem_addr
__device__ __forceinline__ uint64_t make_desc_rows_alias(uint32_t smem_addr) {
  return (uint64_t)((smem_addr >> 4) & 0x3FFF) | ((uint64_t)1 << 16) | ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}

template <int BN>
struct Smem {
  uint8_t a[kStages][kTileA];              // 1024-byte aligned operand tiles
  uint8_t b[kStages][Cfg<BN>::kTileB];
  uint8_t bias[4][1024];                   // A8: constant operand blocks of the bias MMAs (1024-byte aligned)
  float norm[Cfg<BN>::kNormRing][BN];      // column norms of a group, image column order
  uint8_t stage[kEpiWarps][1024];          // per epilogue warp: 8 output rows on their way from fragments to full lines
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
  const int tid = threadIdx.x, lane = tid & 31;
  const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);   // a broadcast value: the compiler keeps what derives from it in uniform registers
  // one base address in the shared window, opaque to the optimiser (it would otherwise recompute the aligned base
  // at every use); every tile, norm slot and barrier is a compile-time offset from it
  uint32_t sb = smem_u32(&S);
  asm volatile("" : "+r"(sb));
  using SM = Smem<BN>;
  const uint32_t abort_flag = sb + (uint32_t)offsetof(SM, abort_flag);
  auto bar_full = [&](uint32_t s_) { return sb + (uint32_t)offsetof(SM, full) + 8u * s_; };
  auto bar_empty = [&](uint32_t s_) { return sb + (uint32_t)offsetof(SM, empty) + 8u * s_; };
  auto bar_acc_full = [&](uint32_t b_) { return sb + (uint32_t)offsetof(SM, acc_full) + 8u * b_; };
  auto bar_acc_empty = [&](uint32_t b_) { return sb + (uint32_t)offsetof(SM, acc_empty) + 8u * b_; };
  auto tile_a = [&](uint32_t s_) { return sb + (uint32_t)offsetof(SM, a) + (uint32_t)kTileA * s_; };
  auto tile_b = [&](uint32_t s_) { return sb + (uint32_t)offsetof(SM, b) + (uint32_t)C::kTileB * s_; };
  auto norm_slot = [&](uint32_t i_) { return sb + (uint32_t)offsetof(SM, norm) + (uint32_t)(BN * 4) * i_; };
  constexpr int SPG = Shape<MODE>::SPG, GPS = Shape<MODE>::GPS;
  constexpr int ACC = (BN == 256) ? 2 : (MODE == DMOQ_FP4 ? 3 : 4);   // accumulator buffers in TMEM
  constexpr int NH = BN / 128;                                        // 32-column blocks per epilogue thread
  constexpr int NCH = 4 * NH;                                         // 16-lane x 16-column accumulator loads per group and warp
  constexpr int kMmaWarp = C::kMmaWarp, kNormRing = C::kNormRing;
  static_assert(!(MODE == DMOQ_FP4 && BN != 128), "the FP4 scale-factor columns need 128-column tiles");

  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar_full(s), MODE == DMOQ_FP4 ? 5 : 1);   // the thread that announces the bulk bytes (+ four scale warps)
      mbar_init(bar_empty(s), 1);
    }
    for (int b = 0; b < 4; ++b) {
      mbar_init(bar_acc_full(b), 1);
      mbar_init(bar_acc_empty(b), kEpiWarps);
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
  const uint32_t tmem_base = __shfl_sync(0xffffffffu, S.tmem_base, 0);
  if (MODE == DMOQ_FP4) {
    if (warp < 4) {   // the constant weight block scale, for every column and every 32-block of K
      tc_st4(tmem_base + ((uint32_t)(warp * 32) << 16) + kSfbCol, a.sfb_word, a.sfb_word, a.sfb_word, a.sfb_word);
      tc_wait_st();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
  }
  if (MODE == DMOQ_A8) {   // the bias operand blocks: 16 bytes repeated, visible to the tensor core's reads after the fence
    for (int i = tid; i < 4 * 1024 / 4; i += C::kThreads) {
      const int t = i >> 8, j = (i & 3) * 4;
      const uint32_t w = (uint32_t)kBiasBytes[t][j] | ((uint32_t)kBiasBytes[t][j + 1] << 8) | ((uint32_t)kBiasBytes[t][j + 2] << 16) |
                         ((uint32_t)kBiasBytes[t][j + 3] << 24);
      reinterpret_cast<uint32_t*>(&S.bias[0][0])[i] = w;
    }
    fence_proxy_async();
    __syncthreads();
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
    // Accumulators come out of TMEM in the 16x256b shape: of a block of 16 lanes x 16 columns thread t = 4*i + q
    // receives rows i and i + 8 at columns 2q, 2q+1, 8+2q, 9+2q.  A thread therefore owns FOUR rows (i, i+8, i+16,
    // i+24 of its warp's lane quarter) and 16*NH of the warp's 32*NH columns, needs only 16*NH column norms per
    // group (64-bit shared loads with four distinct addresses per warp) and four row scales.
    reg_inc<C::kRegsEpi>();
    const int lq = warp & 3, cq = warp >> 2;
    const int li = lane >> 2, qd = lane & 3;
    const int cbase = cq * (32 * NH);                // first of the warp's 32*NH tile columns
    uint32_t t_acc = tmem_base + ((uint32_t)(lq * 32) << 16) + cbase;     // the warp's corner of accumulator 0
    uint32_t norm_u32 = norm_slot(0) + (uint32_t)(cbase + 2 * qd) * 4u;     // this thread's first norm pair of slot 0
    asm volatile("" : "+r"(t_acc), "+r"(norm_u32));                        // kept in registers, not recomputed per use
    const int xs_per_row = a.a_stride / kG;
    const unsigned short* xs_tab = reinterpret_cast<const unsigned short*>(a.a_scales);
    constexpr bool has_xs = (MODE == DMOQ_A8 || MODE == DMOQ_FP8);
    uint32_t ia = 0;                                 // groups consumed so far
    uint32_t v[2][8];                                // accumulator chunks: one in the scale math, one in flight
    PROF_DECL;
#ifdef DMOQ_IMG_PROFILE
    const long long prof_start = clock64();
#endif
    for (int item = 0; item < n_items; ++item) {
      const Item cur = item_of(item);
      const DmoqTile tile = cur.tile;
      const int nb = cur.nb, G = cur.G, inter = a.pp[cur.q].inter;
      const uint32_t bias_int = a.pp[cur.q].n_bias == 2 ? kBias2 : kBias1;
      const float bias_off = (float)bias_int * kBiasToOff;
      // thread row r = 2*h + j: tile row lq*32 + 16*h + 8*j + li
      int xoff[4];                                   // element offset of the row's scales (row 0 of the tile for rows past its end)
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int row = lq * 32 + 8 * r + li;
        xoff[r] = (tile.row0 + (row < tile.rows ? row : 0)) * xs_per_row;
      }
      f32x2_t total2[NCH * 4];   // [chunk c = 2k + h][pair p = j + 2m]: columns 16k + 8m + 2q, +1 of row 2h + j
#pragma unroll
      for (int c = 0; c < NCH * 4; ++c) total2[c] = 0ull;
      uint32_t xraw[4] = {0u, 0u, 0u, 0u};           // the upcoming group's row scales (fp16 bits), one group ahead
      if (has_xs) {
#pragma unroll
        for (int r = 0; r < 4; ++r) xraw[r] = xs_tab[xoff[r]];
      }
      for (int g = 0; g < G; ++g, ++ia) {
        const uint32_t b = ia % ACC, ph = (ia / ACC) & 1;
        const uint32_t nrm = norm_u32 + (ia % kNormRing) * (uint32_t)(BN * 4);
        f32x2_t xs2[4], off2[4];
        if (has_xs) {
#pragma unroll
          for (int r = 0; r < 4; ++r) {
            const float x0 = __half2float(__ushort_as_half((unsigned short)xraw[r]));
            // INT8: the accumulator reads as the denormal (bias + sum) * 2^-149; times xs * 2^100, minus the exact
            // constant bias * 2^-49 * xs, that is sum * xs * 2^-49 in one rounding.  e4m3: acc * xs.
            const float x = (MODE == DMOQ_A8) ? x0 * kXsScale : x0;
            const float o = (MODE == DMOQ_A8) ? -bias_off * x0 : 0.f;
            xs2[r] = pack_x2(__float_as_uint(x), __float_as_uint(x));
            off2[r] = pack_x2(__float_as_uint(o), __float_as_uint(o));
          }
          if (g + 1 < G) {
#pragma unroll
            for (int r = 0; r < 4; ++r) xraw[r] = xs_tab[xoff[r] + g + 1];   // in flight during this group
          }
        }
        // The group's norms were bulk-copied before its operand stage completed; the MMA thread saw that completion
        // before it committed acc_full[], so they are visible here.
        PROF_BEGIN();
        mbar_wait(bar_acc_full(b), ph, abort_flag);   // on a timeout the flag is up and the data is void
        PROF_END(0);
        tc_fence_after();
        tc_ld16x16(t_acc + b * BN, v[0]);
        PROF_BEGIN();
        // Chunks of 16 lanes x 16 columns, c = 2k + h (column block k, lane half h): the load of chunk c+1 is in
        // flight while chunk c goes through the scale math.  The two lane halves of a column block share its norms.
        f32x2_t nr[2];
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
          const int k = c >> 1, h = c & 1;
          if (h == 0) {
            nr[0] = lds_x2(nrm + (uint32_t)(k * 64));
            nr[1] = lds_x2(nrm + (uint32_t)(k * 64 + 32));
          }
          {
            PROF_BEGIN2();
            tc_wait_ld();
            PROF_END2(1);   // a part of the chunk loop's time
          }
          if (c + 1 < NCH) {
            tc_ld16x16(t_acc + (((c + 1) & 1) ? (16u << 16) : 0u) + b * BN + 16 * ((c + 1) >> 1), v[(c + 1) & 1]);
          } else {
            // the group's last chunk is in registers: the buffer goes back to the MMA thread, which gets the time of
            // this chunk's math and of a whole group on the other buffer to refill it
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_acc_empty(b));
          }
          const uint32_t(&vc)[8] = v[c & 1];
#pragma unroll
          for (int p = 0; p < 4; ++p) {   // p = j + 2m
            const int r = 2 * h + (p & 1);
            const f32x2_t f = pack_x2_after_wait(vc[2 * p], vc[2 * p + 1]);
            // fp16 / e2m1 operands: no row scale (the block scales are applied by the MMA)
            const f32x2_t t2 = has_xs ? fma_x2(f, xs2[r], off2[r]) : f;
            total2[c * 4 + p] = fma_x2(t2, nr[p >> 1], total2[c * 4 + p]);
          }
          if (BN == 128 && MODE == DMOQ_A8 && a.partials != nullptr) {   // parity checks only (128-column tiles)
            const int n_out = a.is_down ? a.hidden : 2 * inter;
#pragma unroll
            for (int p = 0; p < 4; ++p) {
              const int row = lq * 32 + 16 * h + 8 * (p & 1) + li;
#pragma unroll
              for (int e = 0; e < 2; ++e) {
                const int col = 16 * k + 8 * (p >> 1) + 2 * qd + e;              // 0..31 within the warp's block
                const int n = a.is_down ? nb * BN + cbase + col
                                        : (col < 16 ? 0 : inter) + nb * (BN / 2) + cq * 16 + (col & 15);
                if (row < tile.rows)
                  a.partials[((size_t)(tile.row0 + row) * n_out + n) * G + g] = (int32_t)(vc[2 * p + e] - bias_int);
              }
            }
          }
        }
        PROF_END(2);
      }
      PROF_BEGIN();

      // ---- tile epilogue: a thread stores pairs of adjacent columns (4 bytes); the four threads of a quad fill 16
      // contiguous bytes of a row, the next pair of the same threads the 16 bytes after them.  One pointer per row,
      // at the thread's first column of the item; every store is that pointer plus a compile-time offset.
      uint16_t* rowp[4];
      bool live[4];
      {
        const int col0 = (EPI != DMOQ_EPI_SILU && a.is_down) ? nb * BN + cbase + 2 * qd : nb * (BN / 2) + cq * NH * 16 + 2 * qd;
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const int row = lq * 32 + 8 * r + li;
          live[r] = row < tile.rows;
          rowp[r] = reinterpret_cast<uint16_t*>(a.out) + (size_t)(tile.row0 + row) * a.out_stride + col0;
        }
      }
      const uint32_t stage = sb + (uint32_t)offsetof(SM, stage) + 1024u * (uint32_t)warp;
      if (EPI == DMOQ_EPI_SILU) {
        // image columns [0,16) of a 32-column block = gate, [16,32) = up of 16 consecutive outputs: chunks 2*h2 and
        // 2*h2 + 1 hold a thread's gate and up values at the same positions
        auto silu_bits = [&](int h2, int h, int p) {
          const float2 gt = unpack_x2(total2[(4 * h2 + h) * 4 + p]), ut = unpack_x2(total2[(4 * h2 + 2 + h) * 4 + p]);
          const __half2 uh = __floats2half2_rn(ut.x, ut.y);                       // fp16 up
          const float2 gf = __half22float2(__floats2half2_rn(gt.x, gt.y));        // fp16 gate, back in fp32
          // fast exp and reciprocal (a few fp32 ulps) ahead of the fp16 rounding: a floating-point stage
          const __half2 sg = __floats2half2_rn(__fdividef(gf.x, 1.0f + __expf(-gf.x)), __fdividef(gf.y, 1.0f + __expf(-gf.y)));
          // fp16(silu * up): the product of two fp16 values is exact in fp32, so one fp16 multiply rounds the same
          const __half2 o2 = __hmul2(sg, uh);
          return *reinterpret_cast<const uint32_t*>(&o2);
        };
        if (NH == 2 && a.out_lines) {   // the warp's 8 rows x 32 outputs per round: matrix mi = 2*h2 + m
          uint16_t* const obase = reinterpret_cast<uint16_t*>(a.out) + (size_t)tile.row0 * a.out_stride + nb * (BN / 2) + cq * NH * 16;
#pragma unroll
          for (int hj = 0; hj < 4; ++hj) {
            const int h = hj >> 1, j = hj & 1, row = lq * 32 + 16 * h + 8 * j;
            uint32_t w[4];
#pragma unroll
            for (int mi = 0; mi < 4; ++mi) w[mi] = silu_bits(mi >> 1, h, j + 2 * (mi & 1));
            store_rows_staged<4>(stage, lane, w, obase + (size_t)row * a.out_stride, a.out_stride, tile.rows - row);
          }
        } else {
#pragma unroll
          for (int h2 = 0; h2 < NH; ++h2)
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
              for (int p = 0; p < 4; ++p) {
                const int r = 2 * h + (p & 1);
                if (live[r]) *reinterpret_cast<uint32_t*>(rowp[r] + h2 * 16 + 8 * (p >> 1)) = silu_bits(h2, h, p);
              }
        }
      } else {
        float wgt[4] = {0.f, 0.f, 0.f, 0.f};
        if (EPI == DMOQ_EPI_WEIGHTED) {
#pragma unroll
          for (int r = 0; r < 4; ++r)
            if (live[r]) wgt[r] = a.row_weight[tile.row0 + lq * 32 + 8 * r + li];
        }
        auto out_bits = [&](int c, int p) {
          const float2 tv = unpack_x2(total2[c * 4 + p]);
          const __half2 hv = __floats2half2_rn(tv.x, tv.y);   // the fp16 output
          uint32_t bits = *reinterpret_cast<const uint32_t*>(&hv);
          if (EPI == DMOQ_EPI_WEIGHTED) {   // -> bf16, times the routing weight in fp32, -> bf16
            const float w = wgt[2 * (c & 1) + (p & 1)];
            const float2 hf = __half22float2(hv);
            const float2 bf = __bfloat1622float2(__floats2bfloat162_rn(hf.x, hf.y));
            const __nv_bfloat162 o2 = __floats2bfloat162_rn(__fmul_rn(bf.x, w), __fmul_rn(bf.y, w));
            bits = *reinterpret_cast<const uint32_t*>(&o2);
          }
          return bits;
        };
        if (a.is_down && a.out_lines) {
          // per round (h, j): the warp's 8 rows x 32*NH columns; matrix mi = 2k + m holds columns 16k + 8m .. +7
          uint16_t* const obase = reinterpret_cast<uint16_t*>(a.out) + (size_t)tile.row0 * a.out_stride + nb * BN + cbase;
#pragma unroll
          for (int hj = 0; hj < 4; ++hj) {
            const int h = hj >> 1, j = hj & 1, row = lq * 32 + 16 * h + 8 * j;
            uint32_t w[4 * NH];
#pragma unroll
            for (int mi = 0; mi < 4 * NH; ++mi) w[mi] = out_bits(2 * (mi >> 1) + h, j + 2 * (mi & 1));
            store_rows_staged<4 * NH>(stage, lane, w, obase + (size_t)row * a.out_stride, a.out_stride, tile.rows - row);
          }
        } else if (a.is_down) {   // tile columns are output columns
#pragma unroll
          for (int c = 0; c < NCH; ++c)
#pragma unroll
            for (int p = 0; p < 4; ++p) {
              const int r = 2 * (c & 1) + (p & 1);
              if (live[r]) *reinterpret_cast<uint32_t*>(rowp[r] + 16 * (c >> 1) + 8 * (p >> 1)) = out_bits(c, p);
            }
        } else {           // plain gate_up rows are [gate | up], each inter wide
#pragma unroll
          for (int c = 0; c < NCH; ++c)
#pragma unroll
            for (int p = 0; p < 4; ++p) {
              const int k = c >> 1, r = 2 * (c & 1) + (p & 1);
              if (live[r]) *reinterpret_cast<uint32_t*>(rowp[r] + ((k & 1) ? inter : 0) + (k >> 1) * 16 + 8 * (p >> 1)) = out_bits(c, p);
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
          mbar_wait<500>(bar_empty(s), ((it / kStages) & 1) ^ 1, abort_flag);
          PROF_END(0);
          PROF_BEGIN();
          if (loader) {
            if (!abort_get(abort_flag)) {
              // A tile: rows [row0, +128) of the sorted code table, 128 bytes of the step; B tile: image rows
              // [img_row0, +BN) of the step's image row group; column norms of the groups the step starts
              const int g_first = (st * GPS) / SPG;
              const int n_groups = (SPG == 2) ? ((st & 1) ? 0 : 1) : min(GPS, G - g_first);
              mbar_arrive_expect_tx(bar_full(s), kTileA + C::kTileB + n_groups * BN * 4);
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
              tma_load_2d(tile_a(s), &maps.a, st * 128, tile.row0, bar_full(s));
              tma_load_2d(tile_b(s), &maps.b[cur.q], x, y, bar_full(s));
              for (int j = 0; j < n_groups; ++j, ++ig)
                bulk_g2s(norm_slot(ig % kNormRing), pp.norm_img + (size_t)(gg0 + g_first + j) * pp.n_img + img_row0, BN * 4, bar_full(s));
            } else {
              mbar_arrive(bar_full(s));   // keep the arrival count whole after an abort
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
            if (lane == 0) mbar_arrive(bar_full(s));
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
        for (uint32_t j = (it > (uint32_t)kStages ? it - kStages : 0u); j < it; ++j) mbar_wait_quiet(bar_full(j % kStages), (j / kStages) & 1);
    } else if (warp == kMmaWarp) {
      // ========================================================================= MMA warp
      constexpr uint32_t nm = ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
      constexpr uint32_t idesc_i8 = (2u << 4) | (1u << 7) | (1u << 10) | nm;    // s32 accumulate, signed 8-bit operands
      constexpr uint32_t idesc_u8 = (2u << 4) | nm;                              // s32 accumulate, unsigned 8-bit operands
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
        const int q_item = pool_of_item(item, start_unused);
        const int G = groups_of(q_item);
        const int n_bias = a.pp[q_item].n_bias;
        const int steps_per_item = steps_of(G);
        for (int st = 0; st < steps_per_item; ++st, ++it) {
          const int s = it % kStages;
          PROF_BEGIN();
          bool ok = mbar_wait<100>(bar_full(s), (it / kStages) & 1, abort_flag);
          PROF_END(0);
          PROF_BEGIN();
          const int n_groups = (SPG == 2) ? 1 : min(GPS, G - st * GPS);
          // a group's first MMA needs its accumulator buffer back from the epilogue
          if (SPG == 1 || (st & 1) == 0) {
            for (int j = 0; j < n_groups; ++j) {
              const uint32_t ib = ia + j;
              ok = mbar_wait<250>(bar_acc_empty(ib % ACC), ((ib / ACC) & 1) ^ 1, abort_flag) && ok;
            }
          }
          PROF_END(1);
          PROF_BEGIN();
          tc_fence_after();
          if (lane == 0 && ok) {
            const uint64_t da = make_desc(tile_a(s));
            const uint64_t db = make_desc(tile_b(s));
            if (MODE == DMOQ_FP4) {
              for (int j = 0; j < n_groups; ++j) {
                const uint32_t b = (ia + j) % ACC;
                const uint32_t sfa = tmem_base + kSfaCol + (s * 2 + j) * 4;
#pragma unroll
                for (int k = 0; k < 2; ++k) {   // 64 elements = 32 bytes of K per instruction; scale bytes 2k, 2k+1
                  const uint32_t idesc = idesc_f4 | ((uint32_t)(2 * k) << 4) | ((uint32_t)(2 * k) << 29);
                  tc_mma_mxf4(tmem_base + b * BN, da + 2 * (2 * j + k), db + 2 * (2 * j + k), idesc, sfa, tmem_base + kSfbCol, k > 0);
                }
                tc_commit(bar_acc_full(b));
              }
              tc_commit(bar_empty(s));
            } else {
              const uint32_t b = ia % ACC;
              const uint32_t d = tmem_base + b * BN;
              if (MODE == DMOQ_A8) {   // the group's sums start from the bias: constant unsigned blocks, accumulate off
                const uint32_t blk = sb + (uint32_t)offsetof(SM, bias) + (n_bias == 2 ? 2048u : 0u);
                const uint64_t ba = make_desc_rows_alias(blk), bb = make_desc_rows_alias(blk + 1024u);
                for (int j = 0; j < n_bias; ++j) tc_mma_u8(d, ba, bb, idesc_u8, j > 0);
              }
#pragma unroll
              for (int k = 0; k < 4; ++k) {  // 32 bytes of K per instruction: +2 in 16-byte units
                if (MODE == DMOQ_A8) tc_mma<DMOQ_A8>(d, da + 2 * k, db + 2 * k, idesc_i8, 1);  // on top of the bias
                else if (MODE == DMOQ_FP8) tc_mma<DMOQ_FP8>(d, da + 2 * k, db + 2 * k, idesc_f8, k > 0);
                else tc_mma<DMOQ_A16>(d, da + 2 * k, db + 2 * k, idesc_f16, ((st & 1) || k > 0) ? 1u : 0u);
              }
              tc_commit(bar_empty(s));
              if (SPG == 1 || (st & 1)) tc_commit(bar_acc_full(b));
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
  a.out_lines = (out_stride % 8 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0) ? 1 : 0;
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
    pp.n_bias = (mode == DMOQ_A8 && p.identity_lut) ? 2 : 1;
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
