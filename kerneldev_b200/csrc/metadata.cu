// Metadata from token ids on the device: the three per-token tensors of the hierarchical mask
// (in_span, span_id, is_prefix) for a batch of token rows, as the reference derives them when a
// caller passes token ids only (model.py:203-238):
//   in_span[t]   = (#[SPAN] in x[0..t]) - (#[ES] in x[0..t]) > 0
//   span_id[t]   = #[SPAN] in x[0..t] where in_span, else 0;  -1 at every [MASKQ]
//   is_prefix[t] = t <= position of the first [CLS] (all false without a [CLS])
// The reference does this with two cumulative sums and a host loop that synchronises once per row
// (.nonzero() / .item()). Here one CTA handles a row and each of its warps a contiguous segment of it,
// 32 consecutive tokens per step (coalesced 256-byte loads): the running marker counts inside a step
// come from warp ballots (popc of the ballot below the lane). A first pass counts the markers of each
// segment and finds the first [CLS]; a block-wide scan of the eight segment totals gives every
// segment its starting counts; a second pass writes the outputs (coalesced as well). Integer work,
// bound by HBM traffic (16 bytes read, 10 bytes written per token) and, for small batches, by launch
// latency.
#include "common.cuh"

namespace kd {

constexpr int MD_THREADS = 256, MD_WARPS = MD_THREADS / 32, MD_UNROLL = 4;

__global__ void __launch_bounds__(MD_THREADS)
metadata_kernel(const int64_t* __restrict__ tokens, int64_t stride_b, int T, int64_t tok_span, int64_t tok_es,
                int64_t tok_cls, int64_t tok_maskq, uint8_t* __restrict__ in_span, int64_t* __restrict__ span_id,
                uint8_t* __restrict__ is_prefix) {
  __shared__ int s_span[MD_WARPS], s_es[MD_WARPS], s_cls[MD_WARPS];
  const int b = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t* x = tokens + (size_t)b * stride_b;
  // segment of this warp: a multiple of 32 tokens, so that every step is one aligned 32-token group
  const int seg = ((T + MD_WARPS * 32 - 1) / (MD_WARPS * 32)) * 32;
  const int t0 = min(warp * seg, T), t1 = min(t0 + seg, T);
  const uint32_t upto = 0xFFFFFFFFu >> (31 - lane);   // lanes 0 .. lane

  int n_span = 0, n_es = 0, first_cls = T;
  for (int base = t0; base < t1; base += 32 * MD_UNROLL) {
    int64_t v[MD_UNROLL];   // MD_UNROLL independent loads in flight per lane
#pragma unroll
    for (int u = 0; u < MD_UNROLL; ++u) {
      const int t = base + u * 32 + lane;
      v[u] = t < t1 ? x[t] : int64_t(-1);
    }
#pragma unroll
    for (int u = 0; u < MD_UNROLL; ++u) {
      const bool live = base + u * 32 + lane < t1;
      n_span += __popc(__ballot_sync(0xffffffffu, live && v[u] == tok_span));
      n_es += __popc(__ballot_sync(0xffffffffu, live && v[u] == tok_es));
      const uint32_t bc = __ballot_sync(0xffffffffu, live && v[u] == tok_cls);
      if (bc != 0u && first_cls == T) first_cls = base + u * 32 + __ffs(bc) - 1;
    }
  }
  if (lane == 0) { s_span[warp] = n_span; s_es[warp] = n_es; s_cls[warp] = first_cls; }
  __syncthreads();
  int c_span = 0, c_es = 0, cls = T;   // marker counts before this segment; first [CLS] of the row
  for (int w = 0; w < MD_WARPS; ++w) {
    if (w < warp) { c_span += s_span[w]; c_es += s_es[w]; }
    cls = min(cls, s_cls[w]);
  }

  uint8_t* o_ins = in_span + (size_t)b * T;
  uint8_t* o_pre = is_prefix + (size_t)b * T;
  int64_t* o_sid = span_id + (size_t)b * T;
  for (int base = t0; base < t1; base += 32 * MD_UNROLL) {
    int64_t v[MD_UNROLL];
#pragma unroll
    for (int u = 0; u < MD_UNROLL; ++u) {
      const int t = base + u * 32 + lane;
      v[u] = t < t1 ? x[t] : int64_t(-1);
    }
#pragma unroll
    for (int u = 0; u < MD_UNROLL; ++u) {
      const int t = base + u * 32 + lane;
      const bool live = t < t1;
      const uint32_t bs = __ballot_sync(0xffffffffu, live && v[u] == tok_span);
      const uint32_t be = __ballot_sync(0xffffffffu, live && v[u] == tok_es);
      const int my_span = c_span + __popc(bs & upto), my_es = c_es + __popc(be & upto);   // inclusive counts at t
      c_span += __popc(bs);
      c_es += __popc(be);
      if (live) {
        const bool ins = (my_span - my_es) > 0;
        o_ins[t] = ins ? 1 : 0;
        o_sid[t] = (v[u] == tok_maskq) ? int64_t(-1) : (ins ? int64_t(my_span) : int64_t(0));
        o_pre[t] = (t <= cls && cls < T) ? 1 : 0;
      }
    }
  }
}

int launch_metadata(const int64_t* tokens, int64_t stride_b, int B, int T, int64_t tok_span, int64_t tok_es,
                    int64_t tok_cls, int64_t tok_maskq, uint8_t* in_span, int64_t* span_id, uint8_t* is_prefix,
                    cudaStream_t stream) {
  if (B == 0 || T == 0) return 0;
  metadata_kernel<<<B, MD_THREADS, 0, stream>>>(tokens, stride_b, T, tok_span, tok_es, tok_cls, tok_maskq, in_span,
                                                span_id, is_prefix);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(KD_ERR_DEVICE, "metadata_kernel launch: %s", cudaGetErrorString(e));
  return 0;
}

}  // namespace kd
