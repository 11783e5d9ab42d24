// Shared host/device declarations of the library: plan view, error reporting, launch entry
// points of the individual translation units.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <limits.h>
#include <stdint.h>

#include "../../include/kd_attention.h"

namespace kd {

// Typed pointers into a plan buffer (see kd_plan_layout for the contents).
struct PlanView {
  int NT, NP, Tpad;
  uint32_t* desc;
  uint32_t* summary;
  uint8_t* cls;
  int32_t* fwd_cnt;
  uint16_t* fwd_list;
  int32_t* bwd_cnt;
  uint16_t* bwd_list;
  uint32_t* tilebits;
  uint8_t* order;
  uint32_t* stats;
  uint32_t* status;
};

inline PlanView make_plan_view(void* plan, const kd_plan_layout& L) {
  char* base = static_cast<char*>(plan);
  PlanView v;
  v.NT = L.NT;
  v.NP = L.NP;
  v.Tpad = L.NT * KD_TILE;
  v.desc = reinterpret_cast<uint32_t*>(base + L.off_desc);
  v.summary = reinterpret_cast<uint32_t*>(base + L.off_summary);
  v.cls = reinterpret_cast<uint8_t*>(base + L.off_cls);
  v.fwd_cnt = reinterpret_cast<int32_t*>(base + L.off_fwd_cnt);
  v.fwd_list = reinterpret_cast<uint16_t*>(base + L.off_fwd_list);
  v.bwd_cnt = reinterpret_cast<int32_t*>(base + L.off_bwd_cnt);
  v.bwd_list = reinterpret_cast<uint16_t*>(base + L.off_bwd_list);
  v.tilebits = reinterpret_cast<uint32_t*>(base + L.off_tilebits);
  v.order = reinterpret_cast<uint8_t*>(base + L.off_order);
  v.stats = reinterpret_cast<uint32_t*>(base + L.off_stats);
  v.status = reinterpret_cast<uint32_t*>(base + L.off_status);
  return v;
}

// records a printf-style message for kd_last_error() and returns `code`
int set_error(int code, const char* fmt, ...);

// 4-D tensor map over a (B,H,T,D) tensor with box (64 elements along D, `box_rows` tokens),
// 128-byte swizzle, zero fill outside the tensor.
int encode_tensor_map(CUtensorMap* out, const kd_tensor& t, int B, int H, int T, int D, int dtype,
                      int box_rows, const char* name);

// 3-D tensor map over a contiguous fp32 (rows, T, D) array with box (32 elements along D, `box_rows` rows of
// one slice), 128-byte swizzle: the target of the fused backward's bulk reductions of dQ tiles.
int encode_tensor_map_f32_rows(CUtensorMap* out, float* base, int slices, int T, int D, int box_rows, const char* name);

int launch_classify(const kd_meta& m, void* plan, cudaStream_t stream);
int launch_mask_dense(const void* plan, int B, int T, uint8_t* out, cudaStream_t stream);
int launch_attn_fwd(const kd_attn_params& p, cudaStream_t stream);
int launch_attn_bwd(const kd_attn_params& p, cudaStream_t stream);
int static_delta_address(size_t rows_needed, float** out);
int launch_hadamard(const kd_tensor& x, const kd_tensor& y, int B, int H, int T, int D, int dtype,
                    const float* signs, int inverse, cudaStream_t stream);

int launch_metadata(const int64_t* tokens, int64_t stride_b, int B, int T, int64_t tok_span, int64_t tok_es,
                    int64_t tok_cls, int64_t tok_maskq, uint8_t* in_span, int64_t* span_id, uint8_t* is_prefix,
                    cudaStream_t stream);

int launch_span_index(const int64_t* tokens, int64_t stride_b, int B, int T, int64_t tok_span, int64_t tok_es,
                      int64_t tok_mask, int32_t* starts, int32_t* ends, int32_t* n_starts, int32_t* n_ends,
                      int32_t* first_mask, cudaStream_t stream);
int launch_span_mean(bool backward, const void* a, int64_t a_sb, int64_t a_st, void* out, int64_t o_sb, int64_t o_st, int B,
                     int T, int C, int S, int dtype, const int32_t* starts, const int32_t* ends, const int32_t* n_starts,
                     const int32_t* n_ends, cudaStream_t stream);

}  // namespace kd
