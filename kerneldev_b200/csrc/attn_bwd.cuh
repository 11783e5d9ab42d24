// Declarations shared by the backward translation units.
#pragma once
#include "attn_common.cuh"

namespace kd {

struct BwdArgs {
  int B, H, T, NT, NP, Tpad;
  int G;             // heads per CTA
  int d_real;        // head dim of the tensors (a multiple of 16, <= HD); TMA zero-fills the tile columns beyond it
  float scale_log2;  // sm_scale * log2(e)
  float sm_scale;
  const uint32_t* desc;
  const uint32_t* tilebits;   // [B][NT][8][4] class masks of every 128-token tile
  const int32_t* fwd_cnt;
  const uint16_t* fwd_list;
  const int32_t* bwd_cnt;
  const uint16_t* bwd_list;
  const uint8_t* order;   // [B][3][NT]; row 1 = q tiles, row 2 = k tiles, by decreasing list length
  uint32_t* status;
  const void* o;
  int64_t o_sb, o_sh, o_st;
  const void* d_o;
  int64_t do_sb, do_sh, do_st;
  const float* lse;
  float* delta;
  float* dq_acc;     // fp32 (B,H,T,D) dQ accumulation scratch of the fused backward, else null
  void* dq;
  int64_t dq_sb, dq_sh, dq_st;
  void* dk;
  int64_t dk_sb, dk_sh, dk_st;
  void* dv;
  int64_t dv_sb, dv_sh, dv_st;
};

// Fused backward for head dim 64 (attn_bwd_fused.cu): one key-tile-major kernel that forms S and dP once per
// tile, accumulates dK and dV in TMEM and adds its dQ partials to a.dq_acc, then a conversion kernel.
int launch_bwd_fused(const CUtensorMap& tmQ, const CUtensorMap& tmK, const CUtensorMap& tmV, const CUtensorMap& tmDO,
                     const BwdArgs& a, int dtype, dim3 grid, cudaStream_t stream);

}  // namespace kd
