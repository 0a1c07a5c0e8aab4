/*
 * dmoq.h - C ABI of libdmoq: the sm_100a kernels behind the mixed-bit
 * codebook-quantized MoE expert layer.
 *
 * The reference project is pure Python and launches Triton kernels through
 * Python wrappers; it has no FFI.  Each entry point below replaces one of
 * those wrappers (or a chain of torch ops around them) and cites it by the
 * file's path inside the reference project.
 *
 * Conventions
 *   - every pointer is a DEVICE pointer unless the name ends in _host
 *   - the caller owns all memory (inputs, outputs, workspaces); nothing here
 *     allocates or frees device memory
 *   - `stream` is a cudaStream_t passed as void*; all work is enqueued on it
 *     and the call returns without synchronising
 *   - return value: DMOQ_OK or a negative DMOQ_E* code; dmoq_strerror() names it
 *   - "rows" are routed (token, expert) pairs sorted by expert; the shared
 *     expert, when present, is expert index E with one row per token
 */
#ifndef DMOQ_H
#define DMOQ_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DMOQ_VERSION 100

enum {
  DMOQ_OK = 0,
  DMOQ_EINVAL = -1,   /* bad argument (null pointer, unsupported size/bit/mode) */
  DMOQ_ELAUNCH = -2,  /* the CUDA runtime refused a launch or an attribute change */
  DMOQ_ESIZE = -3,    /* a size exceeds a stated maximum */
  DMOQ_EDEVICE = -4   /* no usable device / symbol set-up failed */
};

/* activation modes: what the activations are quantised to before the GEMMs */
enum { DMOQ_A16 = 0, DMOQ_A8 = 1, DMOQ_FP8 = 2, DMOQ_FP4 = 3 };

/* GEMM epilogues */
enum {
  DMOQ_EPI_SILU = 0,     /* tile = [gate | up]; store silu(gate)*up as fp16 (I columns)   */
  DMOQ_EPI_WEIGHTED = 1, /* store bf16(bf16(fp16(acc)) * row_weight)  (down projection)   */
  DMOQ_EPI_PLAIN = 2     /* store fp16(acc); gate_up form: (R, 2*inter) = [gate | up]      */
};

/* factor carried by the fp32 norm images of A8 pools (2^49, exact) */
#define DMOQ_A8_NORM_IMAGE_SCALE 562949953421312.0f

#define DMOQ_GROUP 128      /* quantisation group = rotation block, fixed by the format */
#define DMOQ_MAX_POOLS 8

/*
 * One bit pool = all experts stored at the same bit width (plus, optionally,
 * a one-member pool for the shared expert).  Layouts are the reference's
 * "group-first" runtime layout (turboquant_utils/triton_kernels.py:1042):
 *   gu_idx  (G_h, n_members*2*inter, 16*bit) bytes     gu_norm (G_h, n_members*2*inter) fp16
 *   dn_idx  (n_members*inter/128, hidden, 16*bit)      dn_norm (n_members*inter/128, hidden) fp16
 * norms already carry 1/sqrt(128) (and the e2m1 residual in FP4 mode), as the
 * reference prepares them (quantization/wxa16/bit_partitioned_moe.py:203,
 * quantization/wxfp4/bit_partitioned_moe.py:98).
 * Member `rank` owns gu rows [2*inter*rank, 2*inter*(rank+1)) (gate rows first,
 * then up rows) and dn groups [rank*inter/128, (rank+1)*inter/128)
 * (bit_partitioned_moe.py:120-166).
 */
typedef struct dmoq_pool {
  int32_t bit;            /* 1, 2, 4 or 8 */
  int32_t mode;           /* DMOQ_A16/A8/FP8/FP4 for this pool (the FP4 module runs bit 2 as A8) */
  int32_t n_members;
  int32_t inter;          /* intermediate size of every member (multiple of 128) */
  int32_t hoisted;        /* 1: activations of ALL tokens are rotated+quantised once (table row = token) */
  int32_t act_cap_rows;   /* capacity (rows) of this pool's activation-code table */
  const uint8_t* gu_idx;
  const uint16_t* gu_norm;
  const uint8_t* dn_idx;
  const uint16_t* dn_norm;
  const void* gu_lut;     /* 2^bit entries: fp16 (A16), int8 (A8), e4m3 (FP8), e2m1 nibble (FP4); */
  const void* dn_lut;     /* ignored when identity_lut != 0                                          */
  int32_t identity_lut;   /* 8-bit uniform codebook: weight = index-128 (quantization/wxa8/linear.py:64) */
  int32_t gu_e0, dn_e0;   /* FP4: weight block exponent E0 (triton_kernels_fp4.py:74) */
  float gu_act_scale;     /* folded into stored activation scales: cb_step (A8), cb_scale (FP8), else 1 */
  float dn_act_scale;
  const uint16_t* gu_rot; /* (G_h, 128, 128) fp16 rotations, seed 42+bit + g*128            */
  const uint16_t* dn_rot; /* (n_members*inter/128, 128, 128) fp16, seed 42+bit+1000 + j*128 */
  /* per-forward buffers owned by the caller */
  void* act_codes;        /* gate_up-side activation codes, act_cap_rows rows (see dmoq_rotate_quant) */
  void* act_scales;
  /* optional (1- and 2-bit pools): the same indices with every code widened to a 4-bit field,
     (G, N, 64) bytes, made by dmoq_widen_indices.  The tensor-core GEMM looks widened codes up with
     byte permutes instead of spreading bits; when NULL these pools run on the warp-level kernel. */
  const uint8_t* gu_idx_wide;
  const uint8_t* dn_idx_wide;
  /* optional: weight images made by dmoq_expand_weights (codewords already looked up, operand-row layout) with
     their fp32 column norms in image row order.  When present the tensor-core GEMM reads them with TMA tensor-map
     copies instead of expanding indices per tile.  WxFP4 images are the load-time fold of the codebook into e2m1
     (turboquant_utils/triton_kernels_fp4.py:80). */
  const void* gu_img;
  const void* dn_img;
  const float* gu_norm_img;
  const float* dn_norm_img;
} dmoq_pool_t;

/* Routing tables produced by dmoq_route_build; all int32 unless noted. */
typedef struct dmoq_route {
  int32_t T, top_k, E;        /* E routed experts; expert index E is the shared expert when has_shared */
  int32_t has_shared;
  int32_t tile_m;             /* rows per tile in the tile lists */
  int32_t n_pools;
  const int32_t* expert_pool; /* (E+has_shared) static: pool index of each expert, -1 = unused */
  const int32_t* expert_rank; /* (E+has_shared) static: member rank inside its pool           */
  int32_t* expert_rows;       /* (E+has_shared+1) exclusive prefix of rows per expert          */
  int32_t* sorted_tokens;     /* (R) token of each row, R = T*top_k + has_shared*T             */
  float* sorted_weights;      /* (R) routing weight of each row                                */
  int32_t* row_of;            /* (R) row of flat (token, slot) pair; shared rows follow        */
  int32_t* a_row;             /* (R) row of the pool's activation-code table feeding this row;
                                 the GEMMs accept NULL = the table is in routed-row order      */
  int32_t* pool_rows;         /* (DMOQ_MAX_POOLS) rows routed to each pool                     */
  int32_t* pool_src;          /* for non-hoisted pools: token of each compact table row,
                                 pool p's list starts at pool_src_base[p]; size = sum of the
                                 non-hoisted pools' act_cap_rows                               */
  const int32_t* pool_src_base; /* (DMOQ_MAX_POOLS) static: first pool_src entry of each non-hoisted pool */
  int32_t* tiles;             /* (tile_cap, 4): expert, first row, row count, member rank      */
  int32_t* n_tiles;           /* (2*DMOQ_MAX_POOLS) tiles per pool, then each pool's first tile  */
  int32_t tile_cap;
  const int32_t* pool_hoisted;/* (DMOQ_MAX_POOLS) static copy of dmoq_pool_t.hoisted           */
} dmoq_route_t;

int dmoq_version(void);
const char* dmoq_strerror(int code);

/* bytes of scratch dmoq_route_build needs for (T, top_k, E) */
size_t dmoq_route_workspace_bytes(int32_t T, int32_t top_k, int32_t E);

/*
 * Histogram / scan / stable counting sort of the router's top-k choices, the
 * per-pool tile lists and the activation-table row maps, all on the device.
 * Replaces argsort + bincount(...).cpu() + the Python pool/block-info builders
 * (quantization/wxa16/bit_partitioned_moe.py:1125-1138, :1014-1057,
 * turboquant_utils/triton_kernels_a8.py:938).  Rows of one expert are ordered
 * by token index, so the result is deterministic.
 *   topk_idx (T, top_k) int64, topk_w (T, top_k) fp32, shared_w (T) fp32 or NULL
 */
int dmoq_route_build(const dmoq_route_t* route, const int64_t* topk_idx, const float* topk_w,
                     const float* shared_w, void* workspace, size_t workspace_bytes, void* stream);

/*
 * Router selection feeding dmoq_route_build: fp32 softmax of the logits (T, E), the top_k largest
 * probabilities in descending order with their expert indices, renormalised to sum 1 when `renormalize`
 * (the model's router: softmax -> topk [-> normalise]; the module's fallback for gates that return logits is
 * softmax -> topk, quantization/wxa16/bit_partitioned_moe.py:1113-1119).  E <= 1024, top_k <= 32.
 */
int dmoq_router_topk(const float* logits, int32_t T, int32_t E, int32_t top_k, int32_t renormalize,
                     float* topk_w, int64_t* topk_idx, void* stream);

/*
 * The same launch also computes the shared expert's gate of every token,
 *   shared_w[t] = sigmoid(shared_expert_gate(x[t]))      (quantization/wxa16/bit_partitioned_moe.py:1101-1106),
 * with the roundings of a 16-bit Linear(hidden, 1) and a 16-bit sigmoid: fp32 dot product of x[t] (bf16 when
 * x_is_bf16, else fp16; rows of `hidden` elements, 16-byte aligned, hidden a multiple of 8) with gate_w (same type)
 * plus gate_bias, rounded to that type, sigmoid in fp32, rounded again, stored as fp32 (the row weights
 * dmoq_route_build takes for the shared expert).
 */
int dmoq_router_topk_gate(const float* logits, int32_t T, int32_t E, int32_t top_k, int32_t renormalize,
                          float* topk_w, int64_t* topk_idx, const void* x, int32_t x_is_bf16, int32_t hidden,
                          const void* gate_w, float gate_bias, float* shared_w, void* stream);

/*
 * dmoq_route_build for callers that cannot allocate device memory (no counterpart in the reference,
 * whose routing runs as torch ops that allocate freely).  Who needs it: code that runs while a stream
 * is being captured, serving loops that froze their memory pools, host frameworks that own all
 * allocations and grant none for scratch.  The scratch dmoq_route_build takes from its caller lives
 * here in a fixed array inside the library's device image: dmoq_route_static_max_bytes() bytes
 * (4 MiB), held by every GPU that loads the library until the process exits.
 *   - Problems whose dmoq_route_workspace_bytes(T, top_k, E) exceeds that size return DMOQ_ESIZE.
 *   - The first call on each device looks up the array's device address (with that device current);
 *     make that first call outside any stream capture.
 *   - Nothing is allocated or freed, here or in any routine it calls.
 *   - All calls on one GPU share the array.  No word has to start at zero (a call writes every word
 *     before it reads it), but two calls that overlap on the GPU, e.g. on different streams, race.
 * Arguments and results are those of dmoq_route_build without the workspace.
 */
size_t dmoq_route_static_max_bytes(void);
int dmoq_route_build_static(const dmoq_route_t* route, const int64_t* topk_idx, const float* topk_w,
                            const float* shared_w, void* stream);

/*
 * Group rotation fused with activation quantisation
 * (turboquant_utils/triton_kernels_a8.py:429 int8, triton_kernels_fp8.py:128 e4m3,
 *  triton_kernels_fp4.py:1036 e2m1+e8m0; rotation.py:176 for the unquantised A16 case).
 *   x        (n_src_rows, K) bf16 or fp16 (src_is_bf16), K = G*128
 *   rot      rotation stack, fp16; matrix used for (row, group g) is
 *            rot[(rot_row_group0 ? rot_row_group0[row] : 0) + g]
 *   src_row  optional (n_rows) int32: output row i reads x[src_row[i]]; NULL = identity
 *   n_rows_dev optional device int32: actual row count (<= n_rows), read on the device
 *   codes    A16: (n_rows, K) fp16 rotated values;  A8: int8;  FP8: e4m3 bytes;
 *            FP4: (n_rows, K/2) bytes, even k in the low nibble (row-major, not transposed)
 *   scales   A8/FP8: (n_rows, G) fp16 = scale*extra_scale;  FP4: (n_rows, K/32) e8m0 bytes; A16: unused
 * Each output row's accumulation is a sequential fp32 FMA chain over k = 0..127,
 * which makes the integer codes reproducible bit for bit on a CPU.
 */
int dmoq_rotate_quant(int32_t mode, const void* x, int32_t src_is_bf16, int32_t K,
                      const uint16_t* rot, const int32_t* rot_row_group0,
                      const int32_t* src_row, int32_t n_rows, const int32_t* n_rows_dev,
                      float extra_scale, void* codes, void* scales, void* stream);

/*
 * Down-side rotate+quantise of the SiLU output, one rotation stack per expert
 * (quantization/wxa8/bit_partitioned_moe.py:346-358): rows are taken from the
 * tile lists of `route`, the rotation of row r / group g is
 * pool.dn_rot[rank(expert(r))*inter/128 + g].
 *   act (R, act_stride) fp16 -> codes/scales laid out as in dmoq_rotate_quant, rows pitched by
 *   code_stride elements (scales by code_stride/128 resp. code_stride/32)
 */
int dmoq_rotate_quant_down(const dmoq_route_t* route, const dmoq_pool_t* pools_host, int32_t pool_index,
                           const uint16_t* act, int32_t act_stride, void* codes, void* scales,
                           int32_t code_stride, void* stream);

/*
 * Grouped LUT-dequant GEMM over one pool's tile list.
 *   gate_up: out[r, i] = silu(G[r,i]) * U[r,i],  [G|U][r, n] = sum_g norm[g,n] * xs[r,g] * sum_k a[r,g,k]*LUT[idx[g,n,k]]
 *            replaces *_matmul_merged_rows_gf + F.silu*up
 *            (triton_kernels.py:1482, triton_kernels_a8.py:959, triton_kernels_fp8.py:641,
 *             triton_kernels_fp4.py:740; quantization/wxa16/bit_partitioned_moe.py:925-931)
 *   down:    out[r, h] = bf16(bf16(fp16(D[r,h])) * w[r])
 *            replaces *_matmul_merged_in_features_gf + dn.mul_(w)
 *            (triton_kernels.py:1554, triton_kernels_a8.py:1017, triton_kernels_fp8.py:699,
 *             triton_kernels_fp4.py:811; quantization/wxa16/bit_partitioned_moe.py:960-966)
 * `a_codes`/`a_scales` are the pool's activation table (row pitch a_stride elements); rows are gathered through
 * route->a_row (gate_up) or taken at the row's own index (down).
 * `partials` (optional, A8 only): int32 (R, N, G) per-group integer sums for parity checks.
 */
int dmoq_grouped_gemm(const dmoq_route_t* route, const dmoq_pool_t* pools_host, int32_t pool_index,
                      int32_t is_down, int32_t epilogue, int32_t hidden,
                      const void* a_codes, const void* a_scales, int32_t a_stride,
                      void* out, int32_t out_stride, int32_t* partials, void* stream);

/*
 * dmoq_grouped_gemm over several pools of ONE activation mode in a single launch (their tile lists are walked one
 * after the other by the same persistent kernel).  Every listed pool needs its weight image (gu_img / dn_img and the
 * norm image); a_codes / a_scales is one table in routed-row order holding all these pools' rows (route->a_row NULL
 * on the gate_up side).  Small pools then cost no launch of their own.  pool_ids is a HOST array.
 */
int dmoq_grouped_gemm_pools(const dmoq_route_t* route, const dmoq_pool_t* pools_host, const int32_t* pool_ids_host,
                            int32_t n_ids, int32_t is_down, int32_t epilogue, int32_t hidden,
                            const void* a_codes, const void* a_scales, int32_t a_stride,
                            void* out, int32_t out_stride, void* stream);

/*
 * Status word of the tensor-core (tcgen05) GEMM kernels on the current device, copied to the host
 * (synchronises the device).  0 = healthy; bit 0 = a bounded mbarrier wait ran out, the launch that hit
 * it wrote unspecified output.  No reference counterpart: the reference has no device-side waits.
 */
int dmoq_tc_status(int32_t* status_host);

/*
 * Deterministic combine: y[t] = bf16( sum_slots dn[row_of[t*top_k+slot]] (+ dn[shared row of t]) ),
 * accumulated in fp32 in slot order.  Replaces final_hidden_states.index_add_
 * (quantization/wxa16/bit_partitioned_moe.py:966) and the shared-expert add (:1101-1106).
 *   dn (R, hidden) bf16 already multiplied by the routing weight;  y (T, hidden) bf16 or fp16
 */
int dmoq_combine(const dmoq_route_t* route, const uint16_t* dn, int32_t hidden,
                 void* y, int32_t y_is_bf16, void* stream);

/*
 * The same combine over PLAIN fp16 down outputs: the routing weight of each row (route->sorted_weights) is
 * applied here with the reference's rounding chain, y[t] = sum_slots bf16( bf16(fp16 dn[row]) * w[row] ), so
 * the down GEMM can use DMOQ_EPI_PLAIN.  Bit-identical to DMOQ_EPI_WEIGHTED followed by dmoq_combine
 * (quantization/wxa16/bit_partitioned_moe.py:960-967).
 */
int dmoq_combine_weighted(const dmoq_route_t* route, const uint16_t* dn_f16, int32_t hidden,
                          void* y, int32_t y_is_bf16, void* stream);

/*
 * Runtime layout conversion (N, K*bit/8) row-major bytes -> (K/128, N, 16*bit) on the device
 * (turboquant_utils/triton_kernels.py:1042).
 */
int dmoq_convert_group_first(const uint8_t* row_major, int32_t N, int32_t K, int32_t bit,
                             uint8_t* group_first, void* stream);

/*
 * Widen 1- or 2-bit codes to 4-bit fields (low field first): n_bytes packed bytes -> n_bytes*4/bit bytes.
 * A runtime layout of this library (no reference counterpart): group-first indices (G, N, 16*bit) become
 * (G, N, 64) for dmoq_pool_t.gu_idx_wide / dn_idx_wide.
 */
int dmoq_widen_indices(const uint8_t* packed, int64_t n_bytes, int32_t bit, uint8_t* wide, void* stream);

/*
 * Weight image of one pool and one projection (is_down 0: gate_up, 1: down) for dmoq_pool_t.gu_img / dn_img, and its
 * fp32 column norms for gu_norm_img / dn_norm_img (norm_image may be NULL when only the codewords change).  In the A8
 * mode the norm image holds the norms times DMOQ_A8_NORM_IMAGE_SCALE (an exact power of two: the image GEMM reads its
 * biased int32 sums as fp32 denormals and splits the compensating 2^149 between the row scale and the column norm).  Every
 * codebook index is looked up in the pool's mode table once, here, instead of once per 128-row tile in the GEMM:
 *   A8 / FP8 (G, N, 128) bytes, A16 (G, N, 128) fp16, FP4 (ceil(G/2), N, 128) bytes = two groups of packed e2m1 per
 *   row, which is the reference's load-time fold (turboquant_utils/triton_kernels_fp4.py:80-127,
 *   quantization/wxfp4/bit_partitioned_moe.py:98-125); the other modes have no reference counterpart (its kernels
 *   look indices up per tile, triton_kernels_a8.py:893-902).
 * N = n_members*2*inter with each member's gate and up rows interleaved in runs of 16 (gate_up), or hidden (down);
 * G = hidden/128 (gate_up) or n_members*inter/128 (down).  dmoq_weight_image_bytes gives the image size;
 * the norm image holds G*N floats.  Reads pool->{gu,dn}_{idx,norm,lut}, bit, mode, identity_lut, n_members, inter.
 */
/*
 * Small-batch (decode) path of the WxA16 layer: two streaming launches that cover ALL pools of a layer whose routing
 * tables were built with tile_m = 32.  The packed indices are read from global memory as they are stored, looked up in
 * registers and multiplied with warp-level MMAs whose M operand is the weights, so a tile of a few routed rows does not
 * pay for 128.  Same math as dmoq_grouped_gemm in A16 mode (turboquant_utils/triton_kernels.py:1375, small-batch tile
 * class :475-510; SiLU*up of quantization/wxa16/bit_partitioned_moe.py:925-931).
 *   gateup: reads every pool's rotated fp16 activations (pool.act_codes, rows through route->a_row) and writes
 *           act (R, act_stride) fp16 = silu(gate) * up
 *   down:   reads the rotated SiLU outputs a_rot (R, a_stride) fp16 of dmoq_rotate_quant_down and writes plain fp16
 *           rows dn (R, hidden) for dmoq_combine_weighted
 * Pools must be A16 with bit 1, 2, 4, or 8 with the uniform codebook; hidden a multiple of 256.
 */
/* The small-batch path's group rotations, all pools in one launch each (WxA16: rotated values are fp16 roundings of
 * fp32-accumulated products, turboquant_utils/rotation.py:176 -- no activation codes involved):
 *   rotate:      x (T, hidden) bf16/fp16 -> every pool's pool.act_codes table (hoisted pools: row = token; others:
 *                the pool's compact rows through route->pool_src), rotation stack pool.gu_rot
 *   rotate_down: act (R, act_stride) fp16 -> a_rot (R, a_stride) fp16, each tile with its expert's stack from
 *                pool.dn_rot (quantization/wxa16/bit_partitioned_moe.py:934-943) */
int dmoq_moe_decode_rotate(const dmoq_route_t* route, const dmoq_pool_t* pools_host, int32_t n_pools, int32_t hidden,
                           const void* x, int32_t x_is_bf16, void* stream);
int dmoq_moe_decode_rotate_down(const dmoq_route_t* route, const dmoq_pool_t* pools_host, int32_t n_pools,
                                const uint16_t* act, int32_t act_stride, uint16_t* a_rot, int32_t a_stride, void* stream);
int dmoq_moe_decode_gateup(const dmoq_route_t* route, const dmoq_pool_t* pools_host, int32_t n_pools, int32_t hidden,
                           uint16_t* act, int32_t act_stride, void* stream);
int dmoq_moe_decode_down(const dmoq_route_t* route, const dmoq_pool_t* pools_host, int32_t n_pools, int32_t hidden,
                         const uint16_t* a_rot, int32_t a_stride, uint16_t* dn, void* stream);

/*
 * Rows of a pool's activation-code table put into routed-row order: for every row r of the pool's tiles,
 * dst row r = src row route->a_row[r] (row_bytes of codes, scale_bytes of scales; the scale pointers may both be
 * NULL).  After it the pool's GEMM can take whole 128-row tiles of the table with tensor-map copies; it then gets a
 * route whose a_row is NULL (= a row reads the table row of its own index).  Replaces the gather
 * x_pool = hoisted[pool_tokens] of quantization/wxa16/bit_partitioned_moe.py:893-900.
 */
int dmoq_gather_rows(const dmoq_route_t* route, int32_t pool_index, const void* src_codes, int32_t src_pitch_bytes,
                     int32_t row_bytes, void* dst_codes, int32_t dst_pitch_bytes, const void* src_scales,
                     int32_t src_scale_pitch, int32_t scale_bytes, void* dst_scales, int32_t dst_scale_pitch,
                     void* stream);

size_t dmoq_weight_image_bytes(const dmoq_pool_t* pool, int32_t is_down, int32_t hidden);
int dmoq_expand_weights(const dmoq_pool_t* pool, int32_t is_down, int32_t hidden, void* image, float* norm_image,
                        void* stream);

/*
 * Offline quantiser of the packed format (turboquant_utils/quantize.py:350-472, group size 128): per group and row the
 * L2 norm, the rotated normalised row scaled by sqrt(128), its codebook cell (torch.searchsorted over the cell edges),
 * packed little-endian within each byte.
 *   w (N, K) row-major, w_kind 0 fp32 / 1 fp16 / 2 bf16;  rot (K/128, 128, 128) fp32, matrix of group g from seed + g*128
 *   (rotation.py:53);  edges (2^bit - 1) fp32;  indices_packed (N, K*bit/8) u8;  norms (N, K/128) fp16
 * fp32 arithmetic in a fixed order; an index can differ from a BLAS-ordered evaluation only where a value lies within
 * rounding of a cell edge.
 */
int dmoq_quantize_packed(const void* w, int32_t w_kind, int32_t N, int32_t K, int32_t bit, const float* rot,
                         const float* edges, uint8_t* indices_packed, uint16_t* norms, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* DMOQ_H */
