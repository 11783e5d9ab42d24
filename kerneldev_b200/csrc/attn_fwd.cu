// Forward kernel: O = softmax(mask(Q K^T * scale)) V and base-2 LSE, for sm_100a.
//
// One CTA owns a pair of 128-row query tiles of one (batch, head) and walks the plan's list of
// key tiles that are non-empty for either of them. Roles (warp-specialised, 384 threads):
//   warp 0      TMA producer: Q pair once, then K and V tiles through two rings
//   warp 1      MMA issuer:   S_i = Q_i K^T  (smem x smem -> TMEM),  O_i += P_i V (TMEM x smem)
//   warps 4-7   softmax of query tile 0: TMEM -> registers, rule on PARTIAL tiles, online
//   warps 8-11  softmax of query tile 1  softmax in base 2, P back to TMEM as 16-bit operand
// The two query tiles alternate on the tensor core, so one tile's softmax overlaps the other
// tile's MMAs. EMPTY tiles never appear in the list: they are neither loaded nor multiplied.
//
// Replaces _flash_attn_fwd (original_kernel.py:278-626): same math (scores scaled by
// sm_scale*log2(e), exp2, LSE = m + log2(l)), rows without any visible key give O = 0 and
// LSE = -inf.
#include "attn_common.cuh"

namespace kd {

struct FwdArgs {
  int B, H, T, NT, NP, Tpad;
  float scale_log2;  // sm_scale * log2(e)
  const uint32_t* desc;
  const int32_t* fwd_cnt;
  const uint16_t* fwd_list;
  const uint8_t* order;   // [B][3][NT]; row 0 = pairs sorted by decreasing list length
  unsigned long long* trace;
  uint32_t* status;
  void* o;
  int64_t o_sb, o_sh, o_st;
  float* lse;
};

template <int HD>
struct FwdCfg {
  static constexpr int KBLK = HD / 64;                   // 64-element blocks along D
  static constexpr int TILE_BYTES = KD_TILE * HD * 2;    // one Q / K / V tile
  static constexpr int STAGES = (HD == 64) ? 3 : 2;
  static constexpr int SMEM_Q = 0;
  static constexpr int SMEM_K = SMEM_Q + 2 * TILE_BYTES;
  static constexpr int SMEM_V = SMEM_K + STAGES * TILE_BYTES;
  static constexpr int SMEM_KDESC = SMEM_V + STAGES * TILE_BYTES;  // 8 warps x 128 u32
  static constexpr int SMEM_LIST = SMEM_KDESC + 8 * KD_TILE * 4;     // the pair's work list (<= 128 entries)
  static constexpr int SMEM_TOTAL = SMEM_LIST + 128 * 2;
  static constexpr int SMEM_ALLOC = SMEM_TOTAL + 1024;   // slack for 1024-byte alignment
  // TMEM columns: S0, S1 (128 each, fp32), O0, O1 (HD each); P as 64 columns of packed pairs,
  // in its own region for HD = 64, on top of S for HD = 128 (the tensor pipe runs in order, so
  // S(j+1) is written only after P(j) was consumed by the MMA issued before it).
  static constexpr uint32_t TM_S0 = 0, TM_S1 = 128;
  static constexpr uint32_t TM_O0 = 256, TM_O1 = 256 + HD;
  static constexpr uint32_t TM_P0 = (HD == 64) ? 384 : 0;
  static constexpr uint32_t TM_P1 = (HD == 64) ? 448 : 128;
};

// wait-site codes reported in the status word
enum : uint32_t {
  W_F_QFULL = 0x101, W_F_KEMPTY = 0x102, W_F_VEMPTY = 0x103, W_F_KFULL = 0x104, W_F_VFULL = 0x105,
  W_F_PFULL = 0x106, W_F_SFULL = 0x107, W_F_OFULL = 0x108,
};

template <int HD, bool kBf16>
__global__ void __launch_bounds__(384, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const FwdArgs a) {
  using C = FwdCfg<HD>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sQ = smem_u32(smem + C::SMEM_Q);
  const uint32_t sK = smem_u32(smem + C::SMEM_K);
  const uint32_t sV = smem_u32(smem + C::SMEM_V);
  uint32_t* sKdesc = reinterpret_cast<uint32_t*>(smem + C::SMEM_KDESC);
  uint16_t* sList = reinterpret_cast<uint16_t*>(smem + C::SMEM_LIST);

  __shared__ __align__(8) uint64_t bar_q_full, bar_k_full[C::STAGES], bar_k_empty[C::STAGES],
      bar_v_full[C::STAGES], bar_v_empty[C::STAGES], bar_s_full[2], bar_p_full[2], bar_o_full[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ AbortFlag abortf;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // blockIdx.z walks the pairs from the longest list to the shortest, so the CTAs that take
  // longest are dispatched first
  const int h = blockIdx.x, b = blockIdx.y;
  const int pair = a.order[((size_t)b * 3 + 0) * a.NT + blockIdx.z];
  const int n = a.fwd_cnt[b * a.NP + pair];

  if (tid == 0) {
    abortf.v = 0;
    mbar_init(smem_u32(&bar_q_full), 1);
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(smem_u32(&bar_k_full[s]), 1);
      mbar_init(smem_u32(&bar_k_empty[s]), 1);
      mbar_init(smem_u32(&bar_v_full[s]), 1);
      mbar_init(smem_u32(&bar_v_empty[s]), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&bar_s_full[i]), 1);
      mbar_init(smem_u32(&bar_p_full[i]), 128);
      mbar_init(smem_u32(&bar_o_full[i]), 1);
    }
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_base_s), 512);
    tmem_relinquish();
  }
  if (warp == 2) {
    const uint16_t* list = a.fwd_list + ((size_t)b * a.NP + pair) * a.NT;
    for (int e = lane; e < n; e += 32) sList[e] = list[e];
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tbase = tmem_base_s;
  const uint16_t* list = sList;
  Tracer tr;
  tr.init(a.trace, blockIdx.x == 0 && blockIdx.y == 0 && lane == 0 && (warp == 0 || warp == 1 || warp == 4 || warp == 8),
          blockIdx.z * 4 + (warp == 0 ? 0 : warp == 1 ? 1 : warp == 4 ? 2 : 3));
  tr.ev(1);

  if (warp < 4) {
    reg_dealloc<56>();
    if (warp == 0 && lane == 0 && n > 0) {
      // ------------------------------ TMA producer ------------------------------
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      const int ntile_q = (2 * pair + 1 < a.NT) ? 2 : 1;
      mbar_arrive_expect_tx(smem_u32(&bar_q_full), ntile_q * C::TILE_BYTES);
      for (int t = 0; t < ntile_q; ++t)
        for (int kb = 0; kb < C::KBLK; ++kb)
          tma_load_4d(sQ + t * C::TILE_BYTES + kb * 16384, &tmQ, smem_u32(&bar_q_full), kb * 64,
                      (2 * pair + t) * KD_TILE, h, b);
      bool ok = true;
      int issued = 0;
      for (int e = 0; e < n && ok; ++e) {
        const int s = e % C::STAGES;
        const uint32_t ph = (e / C::STAGES) & 1;
        const int kt = list[e] & 0xFF;
        ok = mbar_wait(smem_u32(&bar_k_empty[s]), ph ^ 1, &abortf, a.status, W_F_KEMPTY);
        if (!ok) break;
        mbar_arrive_expect_tx(smem_u32(&bar_k_full[s]), C::TILE_BYTES);
        for (int kb = 0; kb < C::KBLK; ++kb)
          tma_load_4d(sK + s * C::TILE_BYTES + kb * 16384, &tmK, smem_u32(&bar_k_full[s]), kb * 64,
                      kt * KD_TILE, h, b);
        ok = mbar_wait(smem_u32(&bar_v_empty[s]), ph ^ 1, &abortf, a.status, W_F_VEMPTY);
        if (!ok) {
          // the K load just issued must land before this CTA may exit
          for (int spin = 0; spin < (1 << 20) && !mbar_try_wait(smem_u32(&bar_k_full[s]), ph); ++spin) {}
          break;
        }
        mbar_arrive_expect_tx(smem_u32(&bar_v_full[s]), C::TILE_BYTES);
        for (int kb = 0; kb < C::KBLK; ++kb)
          tma_load_4d(sV + s * C::TILE_BYTES + kb * 16384, &tmV, smem_u32(&bar_v_full[s]), kb * 64,
                      kt * KD_TILE, h, b);
        issued = e + 1;
      }
      if (abortf.v != 0) {
        // unwinding: let every copy already in flight land (bounded) before the CTA exits
        for (int e = max(0, issued - C::STAGES); e < issued; ++e) {
          const int s = e % C::STAGES;
          const uint32_t ph = (e / C::STAGES) & 1;
          for (int spin = 0; spin < (1 << 20) && !mbar_try_wait(smem_u32(&bar_k_full[s]), ph); ++spin) {}
          for (int spin = 0; spin < (1 << 20) && !mbar_try_wait(smem_u32(&bar_v_full[s]), ph); ++spin) {}
        }
        for (int spin = 0; spin < (1 << 20) && !mbar_try_wait(smem_u32(&bar_q_full), 0); ++spin) {}
      }
    } else if (warp == 1 && lane == 0 && n > 0) {
      // ------------------------------ MMA issuer ------------------------------
      const uint32_t idesc_s = make_idesc_f16(kBf16, 0, 0, KD_TILE, KD_TILE);
      const uint32_t idesc_o = make_idesc_f16(kBf16, 0, 1, KD_TILE, HD);
      const uint32_t tS[2] = {tbase + C::TM_S0, tbase + C::TM_S1};
      const uint32_t tO[2] = {tbase + C::TM_O0, tbase + C::TM_O1};
      const uint32_t tP[2] = {tbase + C::TM_P0, tbase + C::TM_P1};
      const uint32_t hi = desc_hi_sw128();
      const uint32_t loQ[2] = {desc_lo_kmajor(sQ), desc_lo_kmajor(sQ + C::TILE_BYTES)};
      const uint32_t loK0 = desc_lo_kmajor(sK), loV0 = desc_lo_mnmajor(sV);
      auto issue_s = [&](int i, int e) {
        const uint32_t kb = loK0 + (e % C::STAGES) * (C::TILE_BYTES >> 4);
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk)
          mma_ss_split(tS[i], loQ[i] + koff_kmajor(kk), kb + koff_kmajor(kk), hi, idesc_s, kk > 0 ? 1u : 0u);
        mma_commit(smem_u32(&bar_s_full[i]));
      };
      auto issue_pv = [&](int i, int e, bool acc) {
        const uint32_t vb = loV0 + (e % C::STAGES) * (C::TILE_BYTES >> 4);
#pragma unroll
        for (int kk = 0; kk < KD_TILE / 16; ++kk)
          mma_ts_split(tO[i], tP[i] + kk * 8, vb + koff_mnmajor(kk), hi, idesc_o, (acc || kk > 0) ? 1u : 0u);
      };
      int last_act[2] = {-1, -1};
      for (int e = 0; e < n; ++e) {
        const uint32_t ent = list[e];
        if ((ent >> 8) & 3) last_act[0] = e;
        if ((ent >> 10) & 3) last_act[1] = e;
      }
      bool ok = mbar_wait(smem_u32(&bar_q_full), 0, &abortf, a.status, W_F_QFULL);
      if (ok) ok = mbar_wait(smem_u32(&bar_k_full[0]), 0, &abortf, a.status, W_F_KFULL);
      if (ok) {
        tc_fence_after_sync();
        const uint32_t ent0 = list[0];
        if ((ent0 >> 8) & 3) issue_s(0, 0);
        if ((ent0 >> 10) & 3) issue_s(1, 0);
        mma_commit(smem_u32(&bar_k_empty[0]));
      }
      bool used[2] = {false, false};
      uint32_t pphase[2] = {0, 0};
      for (int e = 0; e < n && ok; ++e) {
        const uint32_t ent = list[e];
        const uint32_t nxt = (e + 1 < n) ? list[e + 1] : 0u;
        const int s = e % C::STAGES;
        bool v_waited = false, k_waited = false;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          if ((ent >> (8 + 2 * i)) & 3) {
            ok = mbar_wait(smem_u32(&bar_p_full[i]), pphase[i], &abortf, a.status, W_F_PFULL);
            if (!ok) break;
            pphase[i] ^= 1;
            if (!v_waited) {
              ok = mbar_wait(smem_u32(&bar_v_full[s]), (e / C::STAGES) & 1, &abortf, a.status, W_F_VFULL);
              if (!ok) break;
              v_waited = true;
            }
            tr.ev(10 + 2 * i);
            tc_fence_after_sync();
            issue_pv(i, e, used[i]);
            used[i] = true;
            if (e == last_act[i]) mma_commit(smem_u32(&bar_o_full[i]));
          }
          if ((nxt >> (8 + 2 * i)) & 3) {
            if (!k_waited) {
              ok = mbar_wait(smem_u32(&bar_k_full[(e + 1) % C::STAGES]), ((e + 1) / C::STAGES) & 1, &abortf,
                             a.status, W_F_KFULL);
              if (!ok) break;
              k_waited = true;
              tc_fence_after_sync();
            }
            issue_s(i, e + 1);
          }
          tr.ev(11 + 2 * i);
        }
        if (!ok) break;
        mma_commit(smem_u32(&bar_v_empty[s]));
        if (e + 1 < n) mma_commit(smem_u32(&bar_k_empty[(e + 1) % C::STAGES]));
      }
    }
  } else {
    reg_alloc<224>();
    // ------------------------------ softmax warpgroups ------------------------------
    const int i = (warp - 4) >> 2;        // query tile of the pair
    const int wq = warp & 3;              // TMEM lane quadrant of this warp
    const int row = wq * 32 + lane;       // row inside the tile
    const int qtile = 2 * pair + i;
    const int qi = qtile * KD_TILE + row;  // token index of this thread's query
    const bool tile_valid = qtile < a.NT;
    uint32_t* kd_buf = sKdesc + (size_t)(warp - 4) * KD_TILE;   // this warp's copy of a key tile's descriptors
    const uint32_t lane_base = static_cast<uint32_t>(wq * 32) << 16;
    const uint32_t tS = tbase + lane_base + (i == 0 ? C::TM_S0 : C::TM_S1);
    const uint32_t tO = tbase + lane_base + (i == 0 ? C::TM_O0 : C::TM_O1);
    const uint32_t tP = tbase + lane_base + (i == 0 ? C::TM_P0 : C::TM_P1);
    const float c = a.scale_log2;

    const uint32_t qd = tile_valid ? a.desc[(size_t)b * a.Tpad + qi] : 0u;
    float m = -INFINITY, l = 0.f;
    uint32_t sphase = 0;
    int nact = 0;
    bool ok = true;

    // Key descriptors of PARTIAL tiles are fetched one active entry ahead into registers, so their
    // global-memory latency overlaps the previous tile's softmax.
    auto next_active = [&](int from) {
      int e = from;
      while (e < n && ((list[e] >> (8 + 2 * i)) & 3u) == KD_TILE_EMPTY) ++e;
      return e;
    };
    uint32_t kd_pre[4] = {0u, 0u, 0u, 0u};
    auto prefetch_kd = [&](int e) {
      if (e < n && ((list[e] >> (8 + 2 * i)) & 3u) == KD_TILE_PARTIAL) {
        const uint32_t* src = a.desc + (size_t)b * a.Tpad + (size_t)(list[e] & 0xFFu) * KD_TILE;
#pragma unroll
        for (int j = 0; j < 4; ++j) kd_pre[j] = src[j * 32 + lane];
      }
    };
    int e = next_active(0);
    prefetch_kd(e);

    while (e < n) {
      const uint32_t ent = list[e];
      const uint32_t cls = (ent >> (8 + 2 * i)) & 3;
      const int kt = ent & 0xFF;
      tr.ev(20);
      if (cls == KD_TILE_PARTIAL) {
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 4; ++j) kd_buf[j * 32 + lane] = kd_pre[j];
        __syncwarp();
      }
      e = next_active(e + 1);
      prefetch_kd(e);
      tr.ev(21);
      ok = mbar_wait(smem_u32(&bar_s_full[i]), sphase, &abortf, a.status, W_F_SFULL);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      sphase ^= 1;
      tc_fence_after_sync();
      tr.ev(22);

      float s[KD_TILE];
#pragma unroll
      for (int cb = 0; cb < 4; ++cb) {
        uint32_t r[32];
        tmem_ld32(tS + cb * 32, r);
#pragma unroll
        for (int j = 0; j < 32; ++j) s[cb * 32 + j] = __uint_as_float(r[j]);
      }
      tmem_wait_ld();
      tr.ev(23);
      if (cls == KD_TILE_PARTIAL) {
        const int j0 = kt * KD_TILE;
#pragma unroll
        for (int j = 0; j < KD_TILE; j += 4) {
          const uint4 k4 = *reinterpret_cast<const uint4*>(kd_buf + j);
          if (!rule_allowed(qd, qi, k4.x, j0 + j + 0)) s[j + 0] = -INFINITY;
          if (!rule_allowed(qd, qi, k4.y, j0 + j + 1)) s[j + 1] = -INFINITY;
          if (!rule_allowed(qd, qi, k4.z, j0 + j + 2)) s[j + 2] = -INFINITY;
          if (!rule_allowed(qd, qi, k4.w, j0 + j + 3)) s[j + 3] = -INFINITY;
        }
      }
      float mx = s[0];
#pragma unroll
      for (int j = 1; j < KD_TILE; ++j) mx = fmaxf(mx, s[j]);
      // The running maximum is refreshed only when it would grow by more than 2^8 in the
      // exponent; until then the stale value is used consistently for P, l and O, which leaves
      // the normalised result unchanged and skips most O rescales.
      float m_new = m;
      if (m == -INFINITY || (mx - m) * c > 8.0f) m_new = fmaxf(m, mx);
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      const float alpha = (m == -INFINITY) ? 0.f : fast_exp2((m - m_new) * c);
      const bool need_rescale = (nact > 0) && (m_new != m);
      const float neg_mc = -m_use * c;
      float sum = 0.f;
      uint32_t pk[KD_TILE / 2];
#pragma unroll
      for (int j = 0; j < KD_TILE; j += 2) {
        const float p0 = fast_exp2(fmaf(s[j], c, neg_mc));
        const float p1 = fast_exp2(fmaf(s[j + 1], c, neg_mc));
        sum += p0 + p1;
        pk[j / 2] = pack2<kBf16>(p0, p1);
      }
      l = l * alpha + sum;
      m = m_new;
#pragma unroll
      for (int cb = 0; cb < 2; ++cb) {
        uint32_t r[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) r[j] = pk[cb * 32 + j];
        tmem_st32(tP + cb * 32, r);
      }
      if (__any_sync(0xffffffffu, need_rescale)) {
        const float f = need_rescale ? alpha : 1.f;
#pragma unroll
        for (int cb = 0; cb < HD / 32; ++cb) {
          uint32_t r[32];
          tmem_ld32(tO + cb * 32, r);
          tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * f);
          tmem_st32(tO + cb * 32, r);
        }
      }
      tr.ev(24);
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive(smem_u32(&bar_p_full[i]));
      tr.ev(25);
      ++nact;
    }

    // epilogue: normalise, convert, store O and LSE
    if (ok && nact > 0) {
      ok = mbar_wait(smem_u32(&bar_o_full[i]), 0, &abortf, a.status, W_F_OFULL);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok && tile_valid && qi < a.T) {
      a.lse[((size_t)b * a.H + h) * a.T + qi] = (l > 0.f) ? (m * c + log2f(l)) : -INFINITY;
    }
    if (ok) {
      tc_fence_after_sync();
      const float inv_l = (l > 0.f) ? 1.f / l : 0.f;
      uint16_t* orow = reinterpret_cast<uint16_t*>(a.o) + (size_t)b * a.o_sb + (size_t)h * a.o_sh + (size_t)qi * a.o_st;
#pragma unroll
      for (int cb = 0; cb < HD / 32; ++cb) {
        uint32_t r[32];
        if (nact > 0) {
          tmem_ld32(tO + cb * 32, r);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = 0u;
        }
        if (tile_valid && qi < a.T) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            uint4 v;
            v.x = pack2<kBf16>(__uint_as_float(r[j + 0]) * inv_l, __uint_as_float(r[j + 1]) * inv_l);
            v.y = pack2<kBf16>(__uint_as_float(r[j + 2]) * inv_l, __uint_as_float(r[j + 3]) * inv_l);
            v.z = pack2<kBf16>(__uint_as_float(r[j + 4]) * inv_l, __uint_as_float(r[j + 5]) * inv_l);
            v.w = pack2<kBf16>(__uint_as_float(r[j + 6]) * inv_l, __uint_as_float(r[j + 7]) * inv_l);
            *reinterpret_cast<uint4*>(orow + cb * 32 + j) = v;
          }
        }
      }
    }
  }

  tr.ev(31);
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tbase, 512);
}

template <int HD, bool kBf16>
static int launch_fwd_t(const kd_attn_params& p, const kd_plan_layout& L, const PlanView& pv, cudaStream_t stream) {
  using C = FwdCfg<HD>;
  CUtensorMap tmQ, tmK, tmV;
  int rc;
  if ((rc = encode_tensor_map(&tmQ, p.q, p.B, p.H, p.T, p.D, p.dtype, KD_TILE, "q")) != 0) return rc;
  if ((rc = encode_tensor_map(&tmK, p.k, p.B, p.H, p.T, p.D, p.dtype, KD_TILE, "k")) != 0) return rc;
  if ((rc = encode_tensor_map(&tmV, p.v, p.B, p.H, p.T, p.D, p.dtype, KD_TILE, "v")) != 0) return rc;
  FwdArgs a;
  a.B = p.B; a.H = p.H; a.T = p.T; a.NT = L.NT; a.NP = L.NP; a.Tpad = L.NT * KD_TILE;
  a.scale_log2 = p.sm_scale * 1.4426950408889634f;
  a.desc = pv.desc; a.fwd_cnt = pv.fwd_cnt; a.fwd_list = pv.fwd_list; a.status = pv.status;
  a.order = pv.order; a.trace = trace_buffer();
  a.o = p.o.ptr; a.o_sb = p.o.stride_b; a.o_sh = p.o.stride_h; a.o_st = p.o.stride_t;
  a.lse = p.lse;
  auto kern = attn_fwd_kernel<HD, kBf16>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_ALLOC);
  if (e != cudaSuccess) return set_error(KD_ERR_DEVICE, "fwd smem attribute: %s", cudaGetErrorString(e));
  dim3 grid(p.H, p.B, L.NP);
  kern<<<grid, 384, C::SMEM_ALLOC, stream>>>(tmQ, tmK, tmV, a);
  e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(KD_ERR_DEVICE, "attn_fwd_kernel launch: %s", cudaGetErrorString(e));
  return 0;
}

int launch_attn_fwd(const kd_attn_params& p, cudaStream_t stream) {
  kd_plan_layout L;
  if (kd_plan_layout_get(p.B, p.T, &L) != 0) return KD_ERR_ARG;
  PlanView pv = make_plan_view(const_cast<void*>(p.plan), L);
  if (p.D == 64) return p.dtype == KD_BF16 ? launch_fwd_t<64, true>(p, L, pv, stream) : launch_fwd_t<64, false>(p, L, pv, stream);
  if (p.D == 128) return p.dtype == KD_BF16 ? launch_fwd_t<128, true>(p, L, pv, stream) : launch_fwd_t<128, false>(p, L, pv, stream);
  return set_error(KD_ERR_ARG, "head dim %d not supported (64 or 128)", p.D);
}

}  // namespace kd
