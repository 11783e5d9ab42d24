// Plan construction: token descriptors, exact 128x128 tile classification, work lists,
// and the dense-mask materialiser. Integer-only kernels; HBM traffic is a few hundred KB.
#include "common.cuh"
#include "mask_rule.cuh"

namespace kd {

// ---------------------------------------------------------------------------------------
// 1. pack: metadata -> descriptors + per-tile summaries
// ---------------------------------------------------------------------------------------
// summary[b][tile] = { OR of flag bits, AND of flag bits, min span id, max span id } where
// the span id range is taken over the in_span tokens of the tile (sign-extended 24 bit).
__global__ void __launch_bounds__(KD_TILE) pack_kernel(kd_meta m, PlanView pv) {
  const int tile = blockIdx.x, b = blockIdx.y, tid = threadIdx.x;
  const int t = tile * KD_TILE + tid;
  int n_b = m.T;
  if (m.lens != nullptr) n_b = min(m.lens[b], m.T);
  const bool alive = t < n_b;
  uint32_t d = 0;
  if (alive) {
    if (m.rules) {
      const bool ins = m.in_span ? (m.in_span[b * m.in_span_stride_b + t] != 0) : false;
      const bool pre = m.is_prefix ? (m.is_prefix[b * m.is_prefix_stride_b + t] != 0) : false;
      const int64_t sid = m.span_id ? m.span_id[b * m.span_id_stride_b + t] : 0;
      if (sid >= (1 << 23) || sid < -(1 << 23)) atomicOr(pv.status, KD_STATUS_SPAN_RANGE);
      d = pack_token(ins, pre, sid, true);
    } else {
      // no metadata: causal = every token is context; otherwise every token is prefix
      d = pack_plain(m.causal != 0);
    }
  }
  pv.desc[(size_t)b * pv.Tpad + t] = d;
  {
    // 128-bit class masks of the tile: bit t of mask k = descriptor bit k of token t
    // (bits 0..2 = classes as a key, bits 5..7 = classes seen as a query, bit 4 = same-span armed)
    const uint32_t src_bit[8] = {TD_PRE, TD_CTX, TD_INS, TD_PRE << TD_SEES_SHIFT, TD_CTX << TD_SEES_SHIFT,
                                 TD_INS << TD_SEES_SHIFT, TD_SIDPOS, 0u};
    uint32_t* tb = pv.tilebits + ((size_t)b * pv.NT + tile) * 32;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const uint32_t bal = __ballot_sync(0xffffffffu, (d & src_bit[k]) != 0u);
      if ((tid & 31) == 0) tb[k * 4 + (tid >> 5)] = bal;
    }
  }

  uint32_t f_or = d & TD_FLAGS, f_and = d & TD_FLAGS;
  int32_t smin = INT32_MAX, smax = INT32_MIN;
  if (d & TD_INS) {
    const int32_t s = static_cast<int32_t>(d) >> TD_SID_SHIFT;  // arithmetic shift sign-extends
    smin = s;
    smax = s;
  }
  for (int o = 16; o > 0; o >>= 1) {
    f_or |= __shfl_xor_sync(0xffffffffu, f_or, o);
    f_and &= __shfl_xor_sync(0xffffffffu, f_and, o);
    smin = min(smin, __shfl_xor_sync(0xffffffffu, smin, o));
    smax = max(smax, __shfl_xor_sync(0xffffffffu, smax, o));
  }
  __shared__ uint32_t s_or[4], s_and[4];
  __shared__ int32_t s_min[4], s_max[4];
  if ((tid & 31) == 0) {
    s_or[tid >> 5] = f_or;
    s_and[tid >> 5] = f_and;
    s_min[tid >> 5] = smin;
    s_max[tid >> 5] = smax;
  }
  __syncthreads();
  if (tid == 0) {
    uint32_t* out = pv.summary + ((size_t)b * pv.NT + tile) * 4;
    out[0] = s_or[0] | s_or[1] | s_or[2] | s_or[3];
    out[1] = s_and[0] & s_and[1] & s_and[2] & s_and[3];
    out[2] = static_cast<uint32_t>(min(min(s_min[0], s_min[1]), min(s_min[2], s_min[3])));
    out[3] = static_cast<uint32_t>(max(max(s_max[0], s_max[1]), max(s_max[2], s_max[3])));
    if (tile == 0) {
      pv.stats[b * 2 + 0] = 0;
      pv.stats[b * 2 + 1] = 0;
    }
  }
}

// ---------------------------------------------------------------------------------------
// 2. classify: one warp per (b, q_tile, k_tile)
// ---------------------------------------------------------------------------------------
// Tiles whose 128 query tokens share one flag combination and whose 128 key tokens share one
// are decided from the summaries; everything else is decided by evaluating the rule on all
// 128x128 pairs. Both routes give the exact reduction of the dense mask.
__global__ void __launch_bounds__(128) classify_kernel(PlanView pv, int B) {
  __shared__ uint32_t s_k[4][KD_TILE];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long total = (long long)B * pv.NT * pv.NT;
  const long long item = (long long)blockIdx.x * 4 + warp;
  if (item >= total) return;
  const int kt = static_cast<int>(item % pv.NT);
  const int qt = static_cast<int>((item / pv.NT) % pv.NT);
  const int b = static_cast<int>(item / ((long long)pv.NT * pv.NT));

  const uint32_t* sq = pv.summary + ((size_t)b * pv.NT + qt) * 4;
  const uint32_t* sk = pv.summary + ((size_t)b * pv.NT + kt) * 4;
  const uint32_t q_or = sq[0], q_and = sq[1], k_or = sk[0], k_and = sk[1];
  int cls = -1;
  if (q_or == 0u || k_or == 0u) {
    cls = KD_TILE_EMPTY;  // all queries or all keys are beyond the sequence length
  } else if (q_or == q_and && k_or == k_and) {
    // flags only; the span id is handled below
    if (k_or & sees_of_flags(q_or)) {
      cls = KD_TILE_FULL;
    } else if ((k_or & q_or & TD_CTX) != 0u) {
      cls = qt > kt ? KD_TILE_FULL : (qt < kt ? KD_TILE_EMPTY : KD_TILE_PARTIAL);
    } else if ((q_or & TD_SIDPOS) && (k_or & TD_INS)) {
      const int32_t qmin = (int32_t)sq[2], qmax = (int32_t)sq[3];
      const int32_t kmin = (int32_t)sk[2], kmax = (int32_t)sk[3];
      if (qmin == qmax && kmin == kmax) cls = (qmin == kmin) ? KD_TILE_FULL : KD_TILE_EMPTY;
      else if (qmax < kmin || kmax < qmin) cls = KD_TILE_EMPTY;  // disjoint id ranges
    } else {
      cls = KD_TILE_EMPTY;
    }
  }
  if (cls < 0) {
    const uint32_t* dq = pv.desc + (size_t)b * pv.Tpad + (size_t)qt * KD_TILE;
    const uint32_t* dk = pv.desc + (size_t)b * pv.Tpad + (size_t)kt * KD_TILE;
    for (int j = lane; j < KD_TILE; j += 32) s_k[warp][j] = dk[j];
    __syncwarp();
    bool any_on = false, any_off = false;
    for (int r = 0; r < 4; ++r) {
      const int i = qt * KD_TILE + r * 32 + lane;
      const uint32_t qd = dq[r * 32 + lane];
      for (int j = 0; j < KD_TILE; ++j) {
        const bool a = rule_allowed(qd, i, s_k[warp][j], kt * KD_TILE + j);
        any_on |= a;
        any_off |= !a;
      }
      const bool w_on = __any_sync(0xffffffffu, any_on);
      const bool w_off = __any_sync(0xffffffffu, any_off);
      if (w_on && w_off) break;
    }
    const bool w_on = __any_sync(0xffffffffu, any_on);
    const bool w_off = __any_sync(0xffffffffu, any_off);
    cls = w_on ? (w_off ? KD_TILE_PARTIAL : KD_TILE_FULL) : KD_TILE_EMPTY;
  }
  if (lane == 0) {
    pv.cls[((size_t)b * pv.NT + qt) * pv.NT + kt] = static_cast<uint8_t>(cls);
    if (cls == KD_TILE_FULL) atomicAdd(&pv.stats[b * 2 + 0], 1u);
    if (cls == KD_TILE_PARTIAL) atomicAdd(&pv.stats[b * 2 + 1], 1u);
  }
}

// ---------------------------------------------------------------------------------------
// 3. work lists
// ---------------------------------------------------------------------------------------
// forward: per (b, pair p of query tiles 2p, 2p+1) the key tiles that are non-empty for either
// backward: per (b, key tile) the query tiles that are non-empty
// order:    per b, the pairs / query tiles / key tiles sorted by decreasing list length, so that the
//           kernels can schedule the longest work items first
__global__ void __launch_bounds__(128) lists_kernel(PlanView pv) {
  __shared__ int s_cnt[3][128];
  const int b = blockIdx.x;
  for (int w = threadIdx.x; w < pv.NP + 2 * pv.NT; w += blockDim.x) {
    if (w < pv.NP) {
      const int p = w, q0 = 2 * p, q1 = 2 * p + 1;
      uint16_t* list = pv.fwd_list + ((size_t)b * pv.NP + p) * pv.NT;
      int n = 0;
      for (int kt = 0; kt < pv.NT; ++kt) {
        const uint32_t c0 = pv.cls[((size_t)b * pv.NT + q0) * pv.NT + kt];
        const uint32_t c1 = q1 < pv.NT ? pv.cls[((size_t)b * pv.NT + q1) * pv.NT + kt] : KD_TILE_EMPTY;
        if (c0 | c1) list[n++] = static_cast<uint16_t>(kt | (c0 << 8) | (c1 << 10));
      }
      pv.fwd_cnt[b * pv.NP + p] = n;
      s_cnt[0][p] = n;
    } else if (w < pv.NP + pv.NT) {
      const int kt = w - pv.NP;
      uint16_t* list = pv.bwd_list + ((size_t)b * pv.NT + kt) * pv.NT;
      int n = 0;
      for (int qt = 0; qt < pv.NT; ++qt) {
        const uint32_t c = pv.cls[((size_t)b * pv.NT + qt) * pv.NT + kt];
        if (c) list[n++] = static_cast<uint16_t>(qt | (c << 8));
      }
      pv.bwd_cnt[b * pv.NT + kt] = n;
      s_cnt[2][kt] = n;
    } else {
      const int qt = w - pv.NP - pv.NT;
      int n = 0;
      for (int kt = 0; kt < pv.NT; ++kt) n += pv.cls[((size_t)b * pv.NT + qt) * pv.NT + kt] != KD_TILE_EMPTY;
      s_cnt[1][qt] = n;
    }
  }
  __syncthreads();
  for (int w = threadIdx.x; w < 3 * pv.NT; w += blockDim.x) {
    const int kind = w / pv.NT, t = w % pv.NT;
    const int n_items = kind == 0 ? pv.NP : pv.NT;
    if (t >= n_items) continue;
    const int mine = s_cnt[kind][t];
    int rank = 0;
    for (int u = 0; u < n_items; ++u) {
      const int other = s_cnt[kind][u];
      rank += (other > mine) || (other == mine && u < t);
    }
    pv.order[((size_t)b * 3 + kind) * pv.NT + rank] = static_cast<uint8_t>(t);
  }
}

// ---------------------------------------------------------------------------------------
// 4. dense mask materialiser
// ---------------------------------------------------------------------------------------
__global__ void mask_dense_kernel(PlanView pv, int T, uint8_t* out) {
  const int b = blockIdx.z, i = blockIdx.y;
  const uint32_t* d = pv.desc + (size_t)b * pv.Tpad;
  const uint32_t qd = d[i];
  for (int j = blockIdx.x * blockDim.x + threadIdx.x; j < T; j += gridDim.x * blockDim.x)
    out[((size_t)b * T + i) * T + j] = rule_allowed(qd, i, d[j], j) ? 1 : 0;
}

// ---------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------
int launch_classify(const kd_meta& m, void* plan, cudaStream_t stream) {
  kd_plan_layout L;
  if (kd_plan_layout_get(m.B, m.T, &L) != 0) return KD_ERR_ARG;
  PlanView pv = make_plan_view(plan, L);
  cudaError_t e = cudaMemsetAsync(pv.status, 0, sizeof(uint32_t), stream);
  if (e != cudaSuccess) return set_error(KD_ERR_DEVICE, "cudaMemsetAsync(status): %s", cudaGetErrorString(e));
  pack_kernel<<<dim3(L.NT, m.B), KD_TILE, 0, stream>>>(m, pv);
  const long long tiles = (long long)m.B * L.NT * L.NT;
  classify_kernel<<<(unsigned)((tiles + 3) / 4), 128, 0, stream>>>(pv, m.B);
  lists_kernel<<<m.B, 128, 0, stream>>>(pv);
  e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(KD_ERR_DEVICE, "plan kernels: %s", cudaGetErrorString(e));
  return 0;
}

int launch_mask_dense(const void* plan, int B, int T, uint8_t* out, cudaStream_t stream) {
  kd_plan_layout L;
  if (kd_plan_layout_get(B, T, &L) != 0) return KD_ERR_ARG;
  PlanView pv = make_plan_view(const_cast<void*>(plan), L);
  dim3 grid((T + 255) / 256, T, B);
  if (grid.x > 16) grid.x = 16;
  mask_dense_kernel<<<grid, 256, 0, stream>>>(pv, T, out);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(KD_ERR_DEVICE, "mask_dense_kernel: %s", cudaGetErrorString(e));
  return 0;
}

}  // namespace kd
