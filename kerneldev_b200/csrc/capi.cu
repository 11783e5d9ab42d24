// extern "C" surface of libkd_attention.so: argument validation, tensor-map encoding,
// error strings. Declarations and the reference interfaces they replace: include/kd_attention.h.
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include "common.cuh"

namespace kd {

static thread_local char g_last_error[512] = "";

int set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
  return code;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

// The driver entry point is looked up through the runtime, so the library has no link-time
// dependency on libcuda.
static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

int encode_tensor_map(CUtensorMap* out, const kd_tensor& t, int B, int H, int T, int D, int dtype,
                      int box_rows, const char* name) {
  EncodeTiledFn enc = encode_fn();
  if (!enc) return set_error(KD_ERR_DEVICE, "cuTensorMapEncodeTiled is not available from this driver");
  if (t.ptr == nullptr) return set_error(KD_ERR_ARG, "tensor %s is null", name);
  if ((reinterpret_cast<uintptr_t>(t.ptr) & 15u) != 0) return set_error(KD_ERR_ALIGN, "tensor %s: base pointer not 16-byte aligned", name);
  const int64_t sb = t.stride_b * 2, sh = t.stride_h * 2, st = t.stride_t * 2;  // bytes
  if (st <= 0 || (st & 15) || (H > 1 && (sh <= 0 || (sh & 15))) || (B > 1 && (sb <= 0 || (sb & 15))))
    return set_error(KD_ERR_ALIGN, "tensor %s: byte strides (%lld, %lld, %lld) must be positive multiples of 16",
                     name, (long long)sb, (long long)sh, (long long)st);
  // the box is 64 elements wide whatever D is: for D < 64 (or the second box of 64 < D < 128) the elements
  // beyond the tensor are filled with zeros, which leaves every product of the kernels unchanged
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)T, (cuuint64_t)H, (cuuint64_t)B};
  // a stride of a size-1 dimension is never used for addressing but must still be valid
  cuuint64_t strides[3] = {(cuuint64_t)st, (cuuint64_t)(H > 1 ? sh : st * T), (cuuint64_t)(B > 1 ? sb : (H > 1 ? sh * H : st * T))};
  for (int i = 0; i < 3; ++i)
    if (strides[i] & 15) strides[i] = (strides[i] + 15) & ~cuuint64_t(15);
  cuuint32_t box[4] = {64, (cuuint32_t)box_rows, 1, 1};
  cuuint32_t es[4] = {1, 1, 1, 1};
  CUresult r = enc(out, dtype == KD_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
                   t.ptr, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return set_error(KD_ERR_ARG, "cuTensorMapEncodeTiled(%s) failed with CUresult %d", name, (int)r);
  return 0;
}

int encode_tensor_map_f32_rows(CUtensorMap* out, float* base, int slices, int T, int D, int box_rows, const char* name) {
  EncodeTiledFn enc = encode_fn();
  if (!enc) return set_error(KD_ERR_DEVICE, "cuTensorMapEncodeTiled is not available from this driver");
  if (base == nullptr || (reinterpret_cast<uintptr_t>(base) & 15u) != 0) return set_error(KD_ERR_ALIGN, "%s: null or not 16-byte aligned", name);
  cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)T, (cuuint64_t)slices};
  cuuint64_t strides[2] = {(cuuint64_t)D * 4, (cuuint64_t)D * 4 * (cuuint64_t)T};
  cuuint32_t box[3] = {32, (cuuint32_t)box_rows, 1};
  cuuint32_t es[3] = {1, 1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, base, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return set_error(KD_ERR_ARG, "cuTensorMapEncodeTiled(%s) failed with CUresult %d", name, (int)r);
  return 0;
}

static int check_device() {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return set_error(KD_ERR_DEVICE, "cudaGetDevice: %s", cudaGetErrorString(e));
  static thread_local int checked_dev = -1;
  if (checked_dev == dev) return 0;
  int major = 0;
  e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
  if (e != cudaSuccess) return set_error(KD_ERR_DEVICE, "cudaDeviceGetAttribute: %s", cudaGetErrorString(e));
  if (major != 10) return set_error(KD_ERR_DEVICE, "device %d has compute capability %d.x; this library is built for sm_100a only", dev, major);
  checked_dev = dev;
  return 0;
}

static int check_attn(const kd_attn_params* p, bool backward) {
  if (!p) return set_error(KD_ERR_ARG, "params is null");
  if (p->B < 1 || p->H < 1 || p->T < 1) return set_error(KD_ERR_ARG, "bad shape B=%d H=%d T=%d", p->B, p->H, p->T);
  if (p->D < 16 || p->D > 128 || (p->D % 16) != 0) return set_error(KD_ERR_ARG, "head dim %d not supported (a multiple of 16 from 16 to 128)", p->D);
  if (p->dtype != KD_F16 && p->dtype != KD_BF16) return set_error(KD_ERR_ARG, "dtype %d not supported (fp16 or bf16)", p->dtype);
  if (p->T > 128 * KD_TILE) return set_error(KD_ERR_LIMIT, "T=%d exceeds the maximum of %d tokens", p->T, 128 * KD_TILE);
  if (p->H > 65535 || p->B > 65535) return set_error(KD_ERR_LIMIT, "B and H must not exceed 65535");
  if (!(p->sm_scale > 0.f) || !(p->sm_scale < 1e30f)) return set_error(KD_ERR_ARG, "sm_scale must be positive and finite");
  if (p->heads_per_cta < 0) return set_error(KD_ERR_ARG, "heads_per_cta must be 0 (automatic) or positive");
  if (!p->plan) return set_error(KD_ERR_ARG, "plan is null (call kd_classify first)");
  if (!p->lse) return set_error(KD_ERR_ARG, "lse is null");
  if (!p->o.ptr) return set_error(KD_ERR_ARG, "o is null");
  if ((reinterpret_cast<uintptr_t>(p->o.ptr) & 15u) || ((p->o.stride_t * 2) & 15) || ((p->o.stride_h * 2) & 15) || ((p->o.stride_b * 2) & 15))
    return set_error(KD_ERR_ALIGN, "o: pointer and byte strides must be multiples of 16");
  if (backward) {
    if (!p->delta) return set_error(KD_ERR_ARG, "delta scratch is null");
    if (p->bwd_mode != KD_BWD_SPLIT && p->bwd_mode != KD_BWD_FUSED) return set_error(KD_ERR_ARG, "bwd_mode %d unknown", p->bwd_mode);
    if (p->bwd_mode == KD_BWD_FUSED) {
      if (p->D > 64) return set_error(KD_ERR_ARG, "the fused backward (KD_BWD_FUSED) supports head dims up to 64 only, got %d", p->D);
      if (!p->dq_acc || (reinterpret_cast<uintptr_t>(p->dq_acc) & 15u)) return set_error(KD_ERR_ARG, "dq_acc scratch is null or not 16-byte aligned");
    }
    const kd_tensor* outs[3] = {&p->dq, &p->dk, &p->dv};
    for (int i = 0; i < 3; ++i) {
      if (!outs[i]->ptr) return set_error(KD_ERR_ARG, "dq/dk/dv is null");
      if ((reinterpret_cast<uintptr_t>(outs[i]->ptr) & 15u) || ((outs[i]->stride_t * 2) & 15) || ((outs[i]->stride_h * 2) & 15) || ((outs[i]->stride_b * 2) & 15))
        return set_error(KD_ERR_ALIGN, "dq/dk/dv: pointer and byte strides must be multiples of 16");
    }
  }
  return 0;
}

}  // namespace kd

using namespace kd;

extern "C" {

int kd_version(void) { return 1; }

const char* kd_last_error(void) { return g_last_error; }

int kd_plan_layout_get(int32_t B, int32_t T, kd_plan_layout* out) {
  if (!out) return set_error(KD_ERR_ARG, "layout pointer is null");
  if (B < 1 || T < 1) return set_error(KD_ERR_ARG, "bad plan shape B=%d T=%d", B, T);
  if (T > 128 * KD_TILE) return set_error(KD_ERR_LIMIT, "T=%d exceeds the maximum of %d tokens", T, 128 * KD_TILE);
  const size_t NT = (T + KD_TILE - 1) / KD_TILE, NP = (NT + 1) / 2;
  auto up = [](size_t x) { return (x + 255) & ~size_t(255); };
  size_t off = 0;
  out->B = B; out->T = T; out->NT = (int32_t)NT; out->NP = (int32_t)NP;
  out->off_desc = off;     off = up(off + (size_t)B * NT * KD_TILE * 4);
  out->off_summary = off;  off = up(off + (size_t)B * NT * 4 * 4);
  out->off_cls = off;      off = up(off + (size_t)B * NT * NT);
  out->off_fwd_cnt = off;  off = up(off + (size_t)B * NP * 4);
  out->off_fwd_list = off; off = up(off + (size_t)B * NP * NT * 2);
  out->off_bwd_cnt = off;  off = up(off + (size_t)B * NT * 4);
  out->off_bwd_list = off; off = up(off + (size_t)B * NT * NT * 2);
  out->off_tilebits = off; off = up(off + (size_t)B * NT * 8 * 4 * 4);
  out->off_order = off;    off = up(off + (size_t)B * 3 * NT);
  out->off_stats = off;    off = up(off + (size_t)B * 2 * 4);
  out->off_status = off;   off = up(off + 4);
  out->total = off;
  return 0;
}

int kd_classify(const kd_meta* meta, void* plan, void* stream) {
  if (!meta || !plan) return set_error(KD_ERR_ARG, "meta / plan is null");
  if (meta->B < 1 || meta->T < 1) return set_error(KD_ERR_ARG, "bad metadata shape B=%d T=%d", meta->B, meta->T);
  if (meta->B > 65535) return set_error(KD_ERR_LIMIT, "B must not exceed 65535");
  if (reinterpret_cast<uintptr_t>(plan) & 255u) return set_error(KD_ERR_ALIGN, "plan buffer must be 256-byte aligned");
  int rc = check_device();
  if (rc) return rc;
  return launch_classify(*meta, plan, static_cast<cudaStream_t>(stream));
}

int kd_mask_dense(const void* plan, int32_t B, int32_t T, uint8_t* out, void* stream) {
  if (!plan || !out) return set_error(KD_ERR_ARG, "plan / out is null");
  if (B > 65535 || T > 65535) return set_error(KD_ERR_LIMIT, "B and T must not exceed 65535");
  int rc = check_device();
  if (rc) return rc;
  return launch_mask_dense(plan, B, T, out, static_cast<cudaStream_t>(stream));
}

int kd_attn_fwd(const kd_attn_params* p, void* stream) {
  int rc = check_attn(p, false);
  if (rc) return rc;
  if ((rc = check_device()) != 0) return rc;
  return launch_attn_fwd(*p, static_cast<cudaStream_t>(stream));
}

int kd_attn_bwd(const kd_attn_params* p, void* stream) {
  int rc = check_attn(p, true);
  if (rc) return rc;
  if ((rc = check_device()) != 0) return rc;
  return launch_attn_bwd(*p, static_cast<cudaStream_t>(stream));
}

int kd_attn_bwd_static(const kd_attn_params* p, void* stream) {
  if (!p) return set_error(KD_ERR_ARG, "params is null");
  if (p->B < 1 || p->H < 1 || p->T < 1) return set_error(KD_ERR_ARG, "bad shape B=%d H=%d T=%d", p->B, p->H, p->T);
  int rc = check_device();
  if (rc) return rc;
  if ((p->bwd_phases & 3) != 0 && (p->bwd_phases & 3) != 3)
    return set_error(KD_ERR_ARG, "kd_attn_bwd_static runs all backward kernels in one call: bwd_phases must be 0 or 3");
  kd_attn_params q = *p;   // same call as kd_attn_bwd, with the scratch pointed at the library's own array
  float* scratch = nullptr;
  if ((rc = static_delta_address((size_t)p->B * p->H * p->T, &scratch)) != 0) return rc;
  q.delta = scratch;
  q.bwd_mode = KD_BWD_SPLIT;   // the fused backward needs a second, much larger scratch
  if ((rc = check_attn(&q, true)) != 0) return rc;
  return launch_attn_bwd(q, static_cast<cudaStream_t>(stream));
}

int kd_workspace_bytes(int32_t B, int32_t H, int32_t T, int32_t D, size_t* bytes) {
  if (!bytes || B < 1 || H < 1 || T < 1 || D < 1) return set_error(KD_ERR_ARG, "bad workspace query");
  (void)D;
  *bytes = (size_t)B * H * T * sizeof(float);
  return 0;
}

int kd_workspace_bytes_fused(int32_t B, int32_t H, int32_t T, int32_t D, size_t* bytes) {
  if (!bytes || B < 1 || H < 1 || T < 1 || D < 1) return set_error(KD_ERR_ARG, "bad workspace query");
  (void)D;   // rows of the scratch are as wide as the kernel's tile (64 columns) whatever the head dim
  *bytes = (size_t)B * H * T * 64 * sizeof(float);
  return 0;
}

int kd_hadamard(const kd_tensor* x, const kd_tensor* y, int32_t B, int32_t H, int32_t T, int32_t D,
                int32_t dtype, const float* signs, int32_t inverse, void* stream) {
  if (!x || !x->ptr || !y || !y->ptr) return set_error(KD_ERR_ARG, "x / y is null");
  if (B < 1 || H < 1 || T < 1) return set_error(KD_ERR_ARG, "bad shape B=%d H=%d T=%d", B, H, T);
  if (D != 16 && D != 32 && D != 64 && D != 128) return set_error(KD_ERR_ARG, "head dim %d not supported (16, 32, 64 or 128)", D);
  if (dtype != KD_F16 && dtype != KD_BF16) return set_error(KD_ERR_ARG, "dtype %d not supported", dtype);
  if ((reinterpret_cast<uintptr_t>(x->ptr) & 15u) || ((x->stride_t * 2) & 15) || ((x->stride_h * 2) & 15) || ((x->stride_b * 2) & 15))
    return set_error(KD_ERR_ALIGN, "x: pointer and byte strides must be multiples of 16");
  if ((reinterpret_cast<uintptr_t>(y->ptr) & 15u) || ((y->stride_t * 2) & 15) || ((y->stride_h * 2) & 15) || ((y->stride_b * 2) & 15))
    return set_error(KD_ERR_ALIGN, "y: pointer and byte strides must be multiples of 16");
  int rc = check_device();
  if (rc) return rc;
  return launch_hadamard(*x, *y, B, H, T, D, dtype, signs, inverse, static_cast<cudaStream_t>(stream));
}

int kd_metadata_from_tokens(const int64_t* tokens, int64_t stride_b, int32_t B, int32_t T, int64_t tok_span,
                            int64_t tok_es, int64_t tok_cls, int64_t tok_maskq, uint8_t* in_span,
                            int64_t* span_id, uint8_t* is_prefix, void* stream) {
  if (B < 0 || T < 0) return set_error(KD_ERR_ARG, "bad shape B=%d T=%d", B, T);
  if (B == 0 || T == 0) return 0;
  if (!tokens || !in_span || !span_id || !is_prefix) return set_error(KD_ERR_ARG, "tokens / in_span / span_id / is_prefix is null");
  if (stride_b < T) return set_error(KD_ERR_ARG, "stride_b %lld is smaller than T %d", static_cast<long long>(stride_b), T);
  int rc = check_device();
  if (rc) return rc;
  return launch_metadata(tokens, stride_b, B, T, tok_span, tok_es, tok_cls, tok_maskq, in_span, span_id, is_prefix,
                         static_cast<cudaStream_t>(stream));
}

int kd_span_index(const int64_t* tokens, int64_t stride_b, int32_t B, int32_t T, int64_t tok_span, int64_t tok_es,
                  int64_t tok_mask, int32_t* starts, int32_t* ends, int32_t* n_starts, int32_t* n_ends,
                  int32_t* first_mask, void* stream) {
  if (B < 0 || T < 0) return set_error(KD_ERR_ARG, "bad shape B=%d T=%d", B, T);
  if (B == 0 || T == 0) return 0;
  if (!tokens || !starts || !ends || !n_starts || !n_ends || !first_mask) return set_error(KD_ERR_ARG, "null pointer");
  if (stride_b < T) return set_error(KD_ERR_ARG, "stride_b %lld is smaller than T %d", static_cast<long long>(stride_b), T);
  int rc = check_device();
  if (rc) return rc;
  return launch_span_index(tokens, stride_b, B, T, tok_span, tok_es, tok_mask, starts, ends, n_starts, n_ends, first_mask,
                           static_cast<cudaStream_t>(stream));
}

int kd_span_mean(int32_t backward, const void* a, int64_t a_sb, int64_t a_st, void* out, int64_t o_sb, int64_t o_st,
                 int32_t B, int32_t T, int32_t C, int32_t S, int32_t dtype, const int32_t* starts,
                 const int32_t* ends, const int32_t* n_starts, const int32_t* n_ends, void* stream) {
  if (B < 0 || T < 0 || C < 0 || S < 0) return set_error(KD_ERR_ARG, "bad shape B=%d T=%d C=%d S=%d", B, T, C, S);
  if (B == 0 || C == 0 || S == 0) return 0;
  if (!a || !out || !starts || !ends || !n_starts || !n_ends) return set_error(KD_ERR_ARG, "null pointer");
  if (dtype != KD_F16 && dtype != KD_BF16 && dtype != KD_F32) return set_error(KD_ERR_ARG, "dtype %d not supported", dtype);
  int rc = check_device();
  if (rc) return rc;
  return launch_span_mean(backward != 0, a, a_sb, a_st, out, o_sb, o_st, B, T, C, S, dtype, starts, ends, n_starts, n_ends,
                          static_cast<cudaStream_t>(stream));
}

}  // extern "C"
