// Arguments shared by the rotate+quantise kernels.
#pragma once
#include "common.cuh"

struct RotArgs {
  const void* x;
  int src_is_bf16;
  int K;                        // columns rotated (multiple of 128)
  int x_stride, o_stride;       // row pitch (elements) of x and of the code table
  const uint16_t* rot;          // fp16 (n_mats, 128, 128)
  const int32_t* src_row;       // optional gather
  int n_rows;
  const int32_t* n_rows_dev;    // optional device-side row count
  float extra_scale;
  void* codes;
  void* scales;
  // tile-driven variant (down side)
  const DmoqTile* tiles;
  const int32_t* n_tiles;       // n_tiles[pool], n_tiles[8+pool] = first tile
  const int32_t* expert_rank;
  int pool;
  int groups_per_member;
};

// tensor-core rotation with exact fix-up (rotate_quant_mma.cu)
int dmoq_rotq_mma_rows(int mode, const RotArgs& a, cudaStream_t s);
int dmoq_rotq_mma_tiles(int mode, const RotArgs& a, int tile_cap, cudaStream_t s);
