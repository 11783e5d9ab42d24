// Span means of the cocktail-party head (model.py:258-296): for every row, the j-th [SPAN] token is
// paired with the j-th [ES] token and h_spans[b, j] = mean(x[b, st+1 : ed]) (zero when the pair is
// missing or st + 1 >= ed). The reference finds the markers with .nonzero() and walks the pairs in a
// Python loop over rows and spans; here
//   span_index_kernel   ranks the markers of a row with warp ballots and writes their positions,
//   span_mean_fwd       one CTA per (span, row): column-parallel fp32 sums over the span's tokens,
//   span_mean_bwd       one CTA per (token block, row): grad_x[t] = sum over the spans covering t of
//                       grad_h[j] / len_j  (a gather, so overlapping pairs need no atomics).
// All three are bound by HBM traffic: the forward reads every span token's embedding once.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"

namespace kd {

constexpr int CK_THREADS = 256, CK_WARPS = CK_THREADS / 32;

// positions of the r-th [SPAN] / [ES] of every row (-1 beyond the row's count), the row's [SPAN] count
// and the position of its first [MASK] (-1 if none)
__global__ void __launch_bounds__(CK_THREADS)
span_index_kernel(const int64_t* __restrict__ tokens, int64_t stride_b, int T, int64_t tok_span, int64_t tok_es,
                  int64_t tok_mask, int32_t* __restrict__ starts, int32_t* __restrict__ ends, int32_t* __restrict__ n_starts,
                  int32_t* __restrict__ n_ends, int32_t* __restrict__ first_mask) {
  __shared__ int s_span[CK_WARPS], s_es[CK_WARPS], s_mask[CK_WARPS];
  const int b = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t* x = tokens + (size_t)b * stride_b;
  const int seg = ((T + CK_WARPS * 32 - 1) / (CK_WARPS * 32)) * 32;
  const int t0 = min(warp * seg, T), t1 = min(t0 + seg, T);
  const uint32_t below = (1u << lane) - 1u;
  for (int t = threadIdx.x; t < T; t += CK_THREADS) { starts[(size_t)b * T + t] = -1; ends[(size_t)b * T + t] = -1; }

  int n_span = 0, n_es = 0, fm = T;
  for (int base = t0; base < t1; base += 32) {
    const int t = base + lane;
    const int64_t v = t < t1 ? x[t] : int64_t(-1);
    n_span += __popc(__ballot_sync(0xffffffffu, t < t1 && v == tok_span));
    n_es += __popc(__ballot_sync(0xffffffffu, t < t1 && v == tok_es));
    const uint32_t bm = __ballot_sync(0xffffffffu, t < t1 && v == tok_mask);
    if (bm != 0u && fm == T) fm = base + __ffs(bm) - 1;
  }
  if (lane == 0) { s_span[warp] = n_span; s_es[warp] = n_es; s_mask[warp] = fm; }
  __syncthreads();   // also orders the -1 fill before the position writes below
  int c_span = 0, c_es = 0, tot_span = 0, tot_es = 0, first = T;
  for (int w = 0; w < CK_WARPS; ++w) {
    if (w < warp) { c_span += s_span[w]; c_es += s_es[w]; }
    tot_span += s_span[w]; tot_es += s_es[w];
    first = min(first, s_mask[w]);
  }
  if (threadIdx.x == 0) { n_starts[b] = tot_span; n_ends[b] = tot_es; first_mask[b] = first < T ? first : -1; }
  for (int base = t0; base < t1; base += 32) {
    const int t = base + lane;
    const int64_t v = t < t1 ? x[t] : int64_t(-1);
    const bool is_s = t < t1 && v == tok_span, is_e = t < t1 && v == tok_es;
    const uint32_t bs = __ballot_sync(0xffffffffu, is_s), be = __ballot_sync(0xffffffffu, is_e);
    if (is_s) starts[(size_t)b * T + c_span + __popc(bs & below)] = t;
    if (is_e) ends[(size_t)b * T + c_es + __popc(be & below)] = t;
    c_span += __popc(bs);
    c_es += __popc(be);
  }
}

template <typename E> __device__ __forceinline__ float to_f(E v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename E> __device__ __forceinline__ E from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// the pair j of row b: true when it exists and holds at least one token between its markers
__device__ __forceinline__ bool span_pair(const int32_t* starts, const int32_t* ends, const int32_t* n_starts,
                                          const int32_t* n_ends, int b, int j, int T, int& st, int& ed) {
  if (j >= min(n_starts[b], n_ends[b])) return false;   // zip() of the reference stops at the shorter list
  st = starts[(size_t)b * T + j];
  ed = ends[(size_t)b * T + j];
  return st + 1 < ed;
}

// h[b, j, :] = mean over t in (st, ed) of x[b, t, :]; grid (S, B)
template <typename E>
__global__ void __launch_bounds__(CK_THREADS)
span_mean_fwd_kernel(const E* __restrict__ x, int64_t x_sb, int64_t x_st, int T, int C, const int32_t* __restrict__ starts,
                     const int32_t* __restrict__ ends, const int32_t* __restrict__ n_starts,
                     const int32_t* __restrict__ n_ends, E* __restrict__ h, int S) {
  const int j = blockIdx.x, b = blockIdx.y;
  int st = 0, ed = 0;
  const bool live = span_pair(starts, ends, n_starts, n_ends, b, j, T, st, ed);
  E* out = h + ((size_t)b * S + j) * C;
  const float inv = live ? 1.f / static_cast<float>(ed - st - 1) : 0.f;
  for (int c = threadIdx.x; c < C; c += CK_THREADS) {   // consecutive threads read consecutive columns
    float acc = 0.f;
    if (live) {
      const E* col = x + (size_t)b * x_sb + c;
      for (int t = st + 1; t < ed; ++t) acc += to_f<E>(col[(size_t)t * x_st]);
    }
    out[c] = from_f<E>(acc * inv);
  }
}

// grad_x[b, t, :] = sum_j [st_j < t < ed_j] grad_h[b, j, :] / (ed_j - st_j - 1); grid (ceil(T / 8), B)
template <typename E>
__global__ void __launch_bounds__(CK_THREADS)
span_mean_bwd_kernel(const E* __restrict__ gh, int S, int T, int C, const int32_t* __restrict__ starts,
                     const int32_t* __restrict__ ends, const int32_t* __restrict__ n_starts,
                     const int32_t* __restrict__ n_ends, E* __restrict__ gx, int64_t gx_sb, int64_t gx_st) {
  constexpr int TT = 8;
  const int b = blockIdx.y, tb = blockIdx.x * TT;
  const int n = min(min(n_starts[b], n_ends[b]), S);
  for (int tt = 0; tt < TT; ++tt) {
    const int t = tb + tt;
    if (t >= T) break;
    // pairs that cover t: none for most tokens, one for canonical data (the same for the whole CTA)
    int covers = 0, j0 = 0;
    for (int j = 0; j < n; ++j) {
      const int st = starts[(size_t)b * T + j], ed = ends[(size_t)b * T + j];
      if (st < t && t < ed) { if (covers == 0) j0 = j; ++covers; }
    }
    E* dst = gx + (size_t)b * gx_sb + (size_t)t * gx_st;
    if (covers == 0) {
      for (int c = threadIdx.x; c < C; c += CK_THREADS) dst[c] = from_f<E>(0.f);
    } else {
      for (int c = threadIdx.x; c < C; c += CK_THREADS) {
        float acc = 0.f;
        for (int j = j0; j < n; ++j) {
          const int st = starts[(size_t)b * T + j], ed = ends[(size_t)b * T + j];
          if (st < t && t < ed) acc += to_f<E>(gh[((size_t)b * S + j) * C + c]) / static_cast<float>(ed - st - 1);
          if (covers == 1) break;   // j0 was the only one
        }
        dst[c] = from_f<E>(acc);
      }
    }
  }
}

int launch_span_index(const int64_t* tokens, int64_t stride_b, int B, int T, int64_t tok_span, int64_t tok_es,
                      int64_t tok_mask, int32_t* starts, int32_t* ends, int32_t* n_starts, int32_t* n_ends,
                      int32_t* first_mask, cudaStream_t stream) {
  if (B == 0 || T == 0) return 0;
  span_index_kernel<<<B, CK_THREADS, 0, stream>>>(tokens, stride_b, T, tok_span, tok_es, tok_mask, starts, ends, n_starts,
                                                  n_ends, first_mask);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(KD_ERR_DEVICE, "span_index_kernel launch: %s", cudaGetErrorString(e));
  return 0;
}

template <typename E>
static int span_mean_t(bool backward, const void* a, int64_t a_sb, int64_t a_st, void* out, int64_t o_sb, int64_t o_st, int B,
                       int T, int C, int S, const int32_t* starts, const int32_t* ends, const int32_t* n_starts,
                       const int32_t* n_ends, cudaStream_t stream) {
  if (!backward) {
    span_mean_fwd_kernel<E><<<dim3(S, B), CK_THREADS, 0, stream>>>(static_cast<const E*>(a), a_sb, a_st, T, C, starts, ends,
                                                                   n_starts, n_ends, static_cast<E*>(out), S);
  } else {
    span_mean_bwd_kernel<E><<<dim3((T + 7) / 8, B), CK_THREADS, 0, stream>>>(static_cast<const E*>(a), S, T, C, starts, ends,
                                                                             n_starts, n_ends, static_cast<E*>(out), o_sb, o_st);
  }
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(KD_ERR_DEVICE, "span_mean kernel launch: %s", cudaGetErrorString(e));
  return 0;
}

int launch_span_mean(bool backward, const void* a, int64_t a_sb, int64_t a_st, void* out, int64_t o_sb, int64_t o_st, int B,
                     int T, int C, int S, int dtype, const int32_t* starts, const int32_t* ends, const int32_t* n_starts,
                     const int32_t* n_ends, cudaStream_t stream) {
  if (B == 0 || S == 0 || C == 0 || (backward && T == 0)) return 0;
  if (dtype == KD_F16) return span_mean_t<__half>(backward, a, a_sb, a_st, out, o_sb, o_st, B, T, C, S, starts, ends, n_starts, n_ends, stream);
  if (dtype == KD_BF16) return span_mean_t<__nv_bfloat16>(backward, a, a_sb, a_st, out, o_sb, o_st, B, T, C, S, starts, ends, n_starts, n_ends, stream);
  if (dtype == KD_F32) return span_mean_t<float>(backward, a, a_sb, a_st, out, o_sb, o_st, B, T, C, S, starts, ends, n_starts, n_ends, stream);
  return set_error(KD_ERR_ARG, "dtype %d not supported", dtype);
}

}  // namespace kd
