// Backward kernels for sm_100a: dQ (query-tile major) and dK/dV (key-tile major).
//
// Both kernels recompute P = exp2(S*scale*log2e - LSE) from Q, K and the saved base-2 LSE and
// form dS = P * (dP - delta), as the reference's two backward workers do
// (_flash_attn_bwd_dq, original_kernel.py:1173-1336; _flash_attn_bwd_dkdv, :1339-1525), but
// walk only the non-empty tiles of the plan and apply the rule only on PARTIAL tiles.
// delta = rowsum(O * dO) (the reference's _flash_attn_bwd_precompute, :629-710) is produced
// by a small bandwidth-bound kernel ahead of the other two.
//
// Shared structure (640 threads): warp 0 = TMA producer, warps 1-3 = MMA issuers, warps 4-19 =
// four compute warpgroups. The backward needs no row reductions, so a 128-column score tile is
// split by columns: a "unit" u = 2*entry + half is one 64-column half, and two warpgroups share a
// unit, 32 columns each, so that sixteen warps (four per scheduler) hide one another's
// tensor-memory, barrier and special-function latencies. A unit owns TMEM buffer u % NBUF
// (64 columns of scores + 64 of dP) and the issuers run NBUF units ahead, so that a warpgroup
// finishing unit u finds its next unit's scores already in TMEM:
//   M1(u): S_u, dP_u  (smem x smem -> TMEM, N = 64)      compute(u): P_u / dS_u -> TMEM (16 bit)
//   M2(u): accumulators += (P_u | dS_u) x smem operand   (A from TMEM);   then M1(u + NBUF)
// Each warpgroup writes its 16 packed columns over the start of the 32 fp32 columns it has just
// read, so the 16-bit operand of a unit sits at columns [0,16) and [32,48) of the buffer.
// The tensor pipe executes in issue order, so M1(u + NBUF) may overwrite the buffer M2(u) read.
// M1 and M2 are issued by different single threads (warps 3 and 2 for M1, warp 1 for M2), so
// that none of them is on the critical path of the other.
#include <algorithm>
#include <mutex>

#include "attn_bwd.cuh"

namespace kd {


template <int HD>
struct BwdCfg {
  static constexpr int KBLK = HD / 64;
  static constexpr int TILE_BYTES = KD_TILE * HD * 2;
  static constexpr int NBUF = (HD == 64) ? 3 : 2;     // score / dP buffers in TMEM
  static constexpr int STAGES = NBUF;                 // ring of (tile, tile) pairs
  static constexpr int NFIX = (HD == 64) ? 2 : 1;     // buffers for the per-head resident tile pair
  static constexpr int SMEM_FIX = 0;                               // NFIX x two resident tiles
  static constexpr int SMEM_RING = SMEM_FIX + NFIX * 2 * TILE_BYTES;  // STAGES x two streamed tiles
  static constexpr int SMEM_STAGE = SMEM_RING + STAGES * 2 * TILE_BYTES;  // per-warp staging
  static constexpr int NSUB = 2;                      // warpgroups that share a 64-column unit
  static constexpr int CPT = 2 / NSUB;                // 32-column chunks per compute thread and unit
  static constexpr int THREADS = 128 + 256 * NSUB;    // four light warps + 2 * NSUB compute warpgroups
  static constexpr int REGS_COMPUTE = KD_REGS_COMPUTE_BWD;
  static constexpr int STAGE_WORDS = 2 * 32 * CPT;                 // per warp (dK/dV kernel): 32*CPT x {lse, delta}
  static constexpr int SMEM_ACT = SMEM_STAGE + 8 * NSUB * STAGE_WORDS * 4;  // compacted entry list
  static constexpr int SMEM_TOTAL = SMEM_ACT + 128 * 2;
  static constexpr int SMEM_ALLOC = SMEM_TOTAL + 1024;
  // TMEM columns
  // buffer j: scores at 128*j, dP at 128*j + 64; accumulators behind the buffers
  static constexpr uint32_t TM_ACC0 = NBUF * 128;        // dQ, or dK
  static constexpr uint32_t TM_ACC1 = NBUF * 128 + HD;   // dV
  static_assert(TM_ACC1 + HD <= 512, "TMEM budget");
  static_assert(SMEM_ALLOC <= 232448, "shared memory budget");
};

enum : uint32_t {
  W_Q_FIXFULL = 0x201, W_Q_RINGEMPTY = 0x202, W_Q_RINGFULL = 0x203, W_Q_PFULL = 0x204, W_Q_SFULL = 0x205,
  W_Q_ACCFULL = 0x206, W_Q_M2ISSUED = 0x207, W_Q_FIXEMPTY = 0x208, W_Q_ACCFREE = 0x209,
  W_K_FIXFULL = 0x301, W_K_RINGEMPTY = 0x302, W_K_RINGFULL = 0x303, W_K_PFULL = 0x304, W_K_SFULL = 0x305,
  W_K_ACCFULL = 0x306, W_K_M2ISSUED = 0x307, W_K_FIXEMPTY = 0x308, W_K_ACCFREE = 0x309,
};

// =========================================================================================
// delta kernel: delta[b, h, t] = sum_d O[b, h, t, d] * dO[b, h, t, d] in fp32 (the reference's
// _flash_attn_bwd_precompute, original_kernel.py:629-710). HD/8 threads share a row, 16 bytes of
// each tensor per thread, so a warp reads whole 128-byte lines; bound by HBM bandwidth. For the fused
// backward it also zeroes the row of the fp32 dQ accumulation scratch (8 floats per thread).
// =========================================================================================
template <int HD, bool kBf16>
__global__ void __launch_bounds__(256) attn_bwd_delta_kernel(const BwdArgs a) {
  constexpr int TPR = HD / 8;   // threads per row
  constexpr int RPB = 256 / TPR;   // rows per block and iteration
  const size_t rows = (size_t)a.B * a.H * a.T;
  const int sub = threadIdx.x % TPR;
  // the loop bound is the same for every thread of the block: the shuffles below need full warps
  for (size_t base = (size_t)blockIdx.x * RPB; base < rows; base += (size_t)gridDim.x * RPB) {
    const size_t r = base + threadIdx.x / TPR;
    const bool live = r < rows;
    float acc = 0.f;
    if (live && sub * 8 < a.d_real) {
      const int t = static_cast<int>(r % a.T);
      const int h = static_cast<int>((r / a.T) % a.H);
      const int b = static_cast<int>(r / ((size_t)a.T * a.H));
      const uint4 ov = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(a.o) + (size_t)b * a.o_sb + (size_t)h * a.o_sh + (size_t)t * a.o_st + sub * 8);
      const uint4 dv = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(a.d_o) + (size_t)b * a.do_sb + (size_t)h * a.do_sh + (size_t)t * a.do_st + sub * 8);
      const uint32_t ow[4] = {ov.x, ov.y, ov.z, ov.w}, dw[4] = {dv.x, dv.y, dv.z, dv.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 x = unpack2<kBf16>(ow[k]), y = unpack2<kBf16>(dw[k]);
        acc = fmaf(x.x, y.x, acc);
        acc = fmaf(x.y, y.y, acc);
      }
    }
#pragma unroll
    for (int d = TPR / 2; d >= 1; d >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, d);
    if (live && sub == 0) a.delta[r] = acc;
    if (live && a.dq_acc != nullptr) {
      float4* z = reinterpret_cast<float4*>(a.dq_acc + r * HD + sub * 8);
      z[0] = make_float4(0.f, 0.f, 0.f, 0.f);
      z[1] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
}

// =========================================================================================
// dQ kernel: one CTA per (b, group of heads, query tile); streams = key halves of the current key
// tile.   M1(i): S_i = Q K_i^T, dP_i = dO V_i^T      M2(i): dQ += dS_i K_i
// The heads of the group are handled one after the other: they share the work list, the barriers
// and the TMEM allocation, and the producer and the issuers run on into the next head while the
// compute warps finish the current one, so the pipeline fill and drain are paid once per CTA.
// =========================================================================================
template <int HD, bool kBf16>
__global__ void __launch_bounds__(BwdCfg<HD>::THREADS, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                   const BwdArgs a) {
  using C = BwdCfg<HD>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sFix = smem_u32(smem + C::SMEM_FIX);    // buffer f: Q at +0, dO at +TILE_BYTES
  const uint32_t sRing = smem_u32(smem + C::SMEM_RING);  // stage s: K at +0, V at +TILE_BYTES
  uint32_t* sStage = reinterpret_cast<uint32_t*>(smem + C::SMEM_STAGE);
  uint16_t* sAct = reinterpret_cast<uint16_t*>(smem + C::SMEM_ACT);

  __shared__ __align__(8) uint64_t bar_fix_full[C::NFIX], bar_fix_empty[C::NFIX], bar_ring_full[C::STAGES],
      bar_ring_empty[C::STAGES], bar_s_full[C::NBUF], bar_p_full[C::NBUF], bar_m2_issued[C::NBUF], bar_acc_full, bar_acc_free;
  __shared__ uint32_t tmem_base_s;
  __shared__ int n_act_s;
  __shared__ AbortFlag abortf;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int h0 = blockIdx.x * a.G, b = blockIdx.y;
  const int nh = min(a.G, a.H - h0);   // this CTA handles heads h0 .. h0 + nh - 1
  const int qt = a.order[((size_t)b * 3 + 1) * a.NT + blockIdx.z];   // longest lists first
  const int pair = qt >> 1, ip = qt & 1;

  if (tid == 0) {
    abortf.v = 0;
    for (int f = 0; f < C::NFIX; ++f) {
      mbar_init(smem_u32(&bar_fix_full[f]), 1);
      mbar_init(smem_u32(&bar_fix_empty[f]), 2);  // both M1 issuers are done with the head's Q and dO
    }
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(smem_u32(&bar_ring_full[s]), 1);
      mbar_init(smem_u32(&bar_ring_empty[s]), 1);
    }
    for (int i = 0; i < C::NBUF; ++i) {
      mbar_init(smem_u32(&bar_s_full[i]), 2);     // one commit from each of the two M1 issuers
      mbar_init(smem_u32(&bar_p_full[i]), 4 * C::NSUB);   // one arrival per warp of the warpgroups that share the unit
      mbar_init(smem_u32(&bar_m2_issued[i]), 1);
    }
    mbar_init(smem_u32(&bar_acc_full), 1);
    mbar_init(smem_u32(&bar_acc_free), 8 * C::NSUB);      // every compute warp has read its part of dQ
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_base_s), 512);
    tmem_relinquish();
  }
  if (warp == 2) {
    // compact the pair's list down to the entries that are non-empty for this query tile
    const int n = a.fwd_cnt[b * a.NP + pair];
    const uint16_t* list = a.fwd_list + ((size_t)b * a.NP + pair) * a.NT;
    int na = 0;
    for (int base = 0; base < n; base += 32) {
      const int e = base + lane;
      const uint32_t ent = e < n ? list[e] : 0u;
      const uint32_t cls = (ent >> (8 + 2 * ip)) & 3u;
      const uint32_t bal = __ballot_sync(0xffffffffu, cls != 0u);
      if (cls != 0u) sAct[na + __popc(bal & ((1u << lane) - 1u))] = static_cast<uint16_t>((ent & 0xFFu) | (cls << 8));
      na += __popc(bal);
    }
    if (lane == 0) n_act_s = na;
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tbase = tmem_base_s;
  const int na = n_act_s;

  if (warp < 4) {
    reg_dealloc<KD_REGS_ISSUE>();
    if (warp == 0 && lane == 0 && na > 0) {
      // ------------------------------ TMA producer ------------------------------
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      tma_prefetch_desc(&tmDO);
      int issued = 0, fix_issued = 0;   // ring entries / resident pairs requested so far, over all heads
      bool ok = true;
      for (int hh = 0; hh < nh && ok; ++hh) {
        const int h = h0 + hh, fb = hh % C::NFIX;
        if (hh >= C::NFIX) {   // the buffer's previous head must have been consumed by both M1 issuers
          ok = mbar_wait(smem_u32(&bar_fix_empty[fb]), (hh / C::NFIX - 1) & 1, &abortf, a.status, W_Q_FIXEMPTY);
          if (!ok) break;
        }
        mbar_arrive_expect_tx(smem_u32(&bar_fix_full[fb]), 2 * C::TILE_BYTES);
        for (int kb = 0; kb < C::KBLK; ++kb) {
          tma_load_4d(sFix + fb * 2 * C::TILE_BYTES + kb * 16384, &tmQ, smem_u32(&bar_fix_full[fb]), kb * 64, qt * KD_TILE, h, b);
          tma_load_4d(sFix + fb * 2 * C::TILE_BYTES + C::TILE_BYTES + kb * 16384, &tmDO, smem_u32(&bar_fix_full[fb]), kb * 64, qt * KD_TILE, h, b);
        }
        fix_issued = hh + 1;
        for (int e = 0; e < na; ++e) {
          const int s = issued % C::STAGES;
          const uint32_t ph = (issued / C::STAGES) & 1;
          const int kt = sAct[e] & 0xFF;
          ok = mbar_wait(smem_u32(&bar_ring_empty[s]), ph ^ 1, &abortf, a.status, W_Q_RINGEMPTY);
          if (!ok) break;
          mbar_arrive_expect_tx(smem_u32(&bar_ring_full[s]), 2 * C::TILE_BYTES);
          const uint32_t dst = sRing + s * 2 * C::TILE_BYTES;
          for (int kb = 0; kb < C::KBLK; ++kb) {
            tma_load_4d(dst + kb * 16384, &tmK, smem_u32(&bar_ring_full[s]), kb * 64, kt * KD_TILE, h, b);
            tma_load_4d(dst + C::TILE_BYTES + kb * 16384, &tmV, smem_u32(&bar_ring_full[s]), kb * 64, kt * KD_TILE, h, b);
          }
          ++issued;
        }
      }
      if (abortf.v != 0) {   // let the copies in flight land before the CTA exits
        for (int e = max(0, issued - C::STAGES); e < issued; ++e)
          for (int spin = 0; spin < (1 << 20) && !mbar_try_wait(smem_u32(&bar_ring_full[e % C::STAGES]), (e / C::STAGES) & 1); ++spin) {}
        for (int f = max(0, fix_issued - C::NFIX); f < fix_issued; ++f)
          for (int spin = 0; spin < (1 << 20) && !mbar_try_wait(smem_u32(&bar_fix_full[f % C::NFIX]), (f / C::NFIX) & 1); ++spin) {}
      }
    } else if ((warp == 3 || warp == 2) && lane == 0 && na > 0) {
      // ------------------------------ M1 issuers: warp 3: S_u = Q K_u^T; warp 2: dP_u = dO V_u^T ------------------------------
      const bool dp_part = (warp == 2);
      const uint32_t idesc_m1 = make_idesc_f16(kBf16, 0, 0, KD_TILE, 64);   // N = 64 keys
      const uint32_t hi = desc_hi_sw128();
      const uint32_t loRingK = desc_lo_kmajor(sRing);
      const int U = 2 * na;
      bool ok = true;
      int buf = 0, round = 0, stage = 0;   // run on across the heads
      uint32_t ring_parity = 0;
      for (int hh = 0; hh < nh && ok; ++hh) {
        const int fb = hh % C::NFIX;
        ok = mbar_wait(smem_u32(&bar_fix_full[fb]), (hh / C::NFIX) & 1, &abortf, a.status, W_Q_FIXFULL);
        if (!ok) break;
        const uint32_t loA = desc_lo_kmajor(sFix + fb * 2 * C::TILE_BYTES + (dp_part ? C::TILE_BYTES : 0));   // dO or Q
        uint64_t adesc[HD / 16];   // A descriptors of the head's k-steps
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) adesc[kk] = desc64(loA + koff_kmajor(kk), hi);
        for (int u = 0; u < U && ok; ++u) {
          const int i = u & 1;
          // operands of the unit, formed ahead of the waits
          // key rows 64i.. of K (scores) or V (dP)
          const uint32_t blo = loRingK + stage * (2 * C::TILE_BYTES >> 4) + i * (64 * 128 >> 4) + (dp_part ? (C::TILE_BYTES >> 4) : 0);
          uint64_t bdesc[HD / 16];
#pragma unroll
          for (int kk = 0; kk < HD / 16; ++kk) bdesc[kk] = desc64(blo + koff_kmajor(kk), hi);
          const uint32_t dst = tbase + buf * 128 + (dp_part ? 64 : 0);
          if (round > 0) {   // buffer free once M2 of its previous unit has been issued
            ok = mbar_wait(smem_u32(&bar_m2_issued[buf]), (round - 1) & 1, &abortf, a.status, W_Q_M2ISSUED);
            if (!ok) break;
          }
          if (i == 0) {      // first unit of a new entry: its K and V tiles must have landed
            ok = mbar_wait(smem_u32(&bar_ring_full[stage]), ring_parity, &abortf, a.status, W_Q_RINGFULL);
            if (!ok) break;
          }
          tc_fence_after_sync();
          mma_ss64<false>(dst, adesc[0], bdesc[0], idesc_m1);
#pragma unroll
          for (int kk = 1; kk < HD / 16; ++kk) mma_ss64<true>(dst, adesc[kk], bdesc[kk], idesc_m1);
          mma_commit(smem_u32(&bar_s_full[buf]));
          if (++buf == C::NBUF) { buf = 0; ++round; }
          if (i == 1 && ++stage == C::STAGES) { stage = 0; ring_parity ^= 1; }
        }
        if (ok) mma_commit(smem_u32(&bar_fix_empty[fb]));   // this issuer's products of the head no longer read Q / dO
      }
    } else if (warp == 1 && lane == 0 && na > 0) {
      // ------------------------------ M2 issuer: dQ += dS_u K_u ------------------------------
      const uint32_t idesc_m2 = make_idesc_f16(kBf16, 0, 1, KD_TILE, HD);   // B = K rows, MN-major
      const uint32_t tAcc = tbase + C::TM_ACC0;
      const uint32_t hi = desc_hi_sw128();
      const uint32_t loRingMN = desc_lo_mnmajor(sRing);
      const int U = 2 * na;
      bool ok = true;
      int buf = 0, stage = 0;
      uint32_t round_parity = 0;
      for (int hh = 0; hh < nh && ok; ++hh) {
        if (hh > 0) {   // the previous head's dQ must have been read out of the accumulator
          ok = mbar_wait(smem_u32(&bar_acc_free), (hh - 1) & 1, &abortf, a.status, W_Q_ACCFREE);
          if (!ok) break;
        }
        for (int u = 0; u < U && ok; ++u) {
          const int i = u & 1;
          // operands of the unit, formed ahead of the wait
          const uint32_t kb = loRingMN + stage * (2 * C::TILE_BYTES >> 4) + i * (64 * 128 >> 4);
          const uint32_t aS = tbase + buf * 128;   // dS_u sits on top of S_u: keys 0-31 at columns [0,16), keys 32-63 at [32,48)
          uint64_t bdesc[4];
          uint32_t aop[4];
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {  // 64 keys of this unit, 16 per MMA
            bdesc[kk] = desc64(kb + koff_mnmajor(kk), hi);
            aop[kk] = aS + (kk >> 1) * 32 + (kk & 1) * 8;
          }
          ok = mbar_wait(smem_u32(&bar_p_full[buf]), round_parity, &abortf, a.status, W_Q_PFULL);
          if (!ok) break;
          tc_fence_after_sync();
          mma_ts64_p(tAcc, aop[0], bdesc[0], idesc_m2, u > 0 ? 1u : 0u);
#pragma unroll
          for (int kk = 1; kk < 4; ++kk) mma_ts64<true>(tAcc, aop[kk], bdesc[kk], idesc_m2);
          if (i == 1) mma_commit(smem_u32(&bar_ring_empty[stage]));
          tc_fence_before_sync();
          mbar_arrive(smem_u32(&bar_m2_issued[buf]));
          if (++buf == C::NBUF) { buf = 0; round_parity ^= 1; }
          if (i == 1 && ++stage == C::STAGES) stage = 0;
        }
        if (ok) mma_commit(smem_u32(&bar_acc_full));
      }
    }
  } else {
    reg_alloc<C::REGS_COMPUTE>();
    // ------------------------------ compute warpgroups ------------------------------
    constexpr int CPT = C::CPT;      // 32-column chunks of a unit this thread handles
    const int g = (warp - 4) >> 2;   // warpgroup
    const int i = g / C::NSUB;       // stream: key half (64 keys) of each key tile
    const int c0 = (g % C::NSUB) * CPT;   // first 32-key chunk of that half handled here
    const int wq = warp & 3;
    const int row = wq * 32 + lane;
    const int qi = qt * KD_TILE + row;
    const bool q_valid = qi < a.T;
    const uint32_t lane_base = static_cast<uint32_t>(wq * 32) << 16;
    const float c = a.scale_log2;
    const uint32_t qd = a.desc[(size_t)b * a.Tpad + qi];
    const int tbw = 2 * i + c0;      // first word of this thread's chunks in the 128-bit class masks of a key tile
    bool ok = true;

    // key descriptors of PARTIAL tiles are fetched one entry ahead into registers
    uint32_t kd_pre[CPT];
    uint32_t tb_pre[3][CPT];   // key-side class masks of the chunks: is_prefix, context, in_span
#pragma unroll
    for (int cc = 0; cc < CPT; ++cc) { kd_pre[cc] = 0u; tb_pre[0][cc] = 0u; tb_pre[1][cc] = 0u; tb_pre[2][cc] = 0u; }
    auto prefetch_kd = [&](uint32_t entry) {
      if ((entry >> 8) == KD_TILE_PARTIAL) {
        const uint32_t ktile = entry & 0xFFu;
        const uint32_t* tbp = a.tilebits + ((size_t)b * a.NT + ktile) * 32;
#pragma unroll
        for (int cc = 0; cc < CPT; ++cc) {
          kd_pre[cc] = a.desc[(size_t)b * a.Tpad + (size_t)ktile * KD_TILE + i * 64 + (c0 + cc) * 32 + lane];
          tb_pre[0][cc] = tbp[4 * TB_PRE + tbw + cc];
          tb_pre[1][cc] = tbp[4 * TB_CTX + tbw + cc];
          tb_pre[2][cc] = tbp[4 * TB_INS + tbw + cc];
        }
      }
    };
    uint32_t ent_next = na > 0 ? sAct[0] : 0u;
    if (na > 0) prefetch_kd(ent_next);
    // per-row scalars of the next head are fetched while the current head is processed
    float nxt_delta = q_valid ? a.delta[((size_t)b * a.H + h0) * a.T + qi] : 0.f;
    float nxt_lse = q_valid ? a.lse[((size_t)b * a.H + h0) * a.T + qi] : 0.f;
    // this stream's next unit, counted over all heads, as (unit / NBUF, unit % NBUF)
    int buf = i % C::NBUF;
    uint32_t rnd = i / C::NBUF;
    const uint32_t sfull0 = smem_u32(&bar_s_full[0]), pfull0 = smem_u32(&bar_p_full[0]);
    const uint32_t tcol = tbase + lane_base + c0 * 32;   // this thread's first chunk inside a buffer

    for (int hh = 0; hh < nh && ok; ++hh) {
      const int h = h0 + hh;
      const float delta = nxt_delta, neg_lse = -nxt_lse;
      if (hh + 1 < nh && q_valid) {
        nxt_delta = a.delta[((size_t)b * a.H + h + 1) * a.T + qi];
        nxt_lse = a.lse[((size_t)b * a.H + h + 1) * a.T + qi];
      }
      for (int e = 0; e < na; ++e) {
        const uint32_t ent = ent_next;
        const uint32_t cls = ent >> 8;
        uint32_t mk[CPT];   // visibility of the chunks' keys for this query row
#pragma unroll
        for (int cc = 0; cc < CPT; ++cc) mk[cc] = 0xFFFFFFFFu;
        if (cls == KD_TILE_PARTIAL) {
          const int j0 = (ent & 0xFF) * KD_TILE + i * 64 + c0 * 32;  // first key handled here
          query_row_mask<CPT>(qd, qi, j0, tb_pre[0], tb_pre[1], tb_pre[2], mk);
          uint32_t any_ins = 0u;
#pragma unroll
          for (int cc = 0; cc < CPT; ++cc) any_ins |= tb_pre[2][cc];
          // "same span": one round per distinct span among the warp's 32 queries; a ballot over the lanes' key descriptors
          // (lane L holds keys L, 32 + L, ... of the chunks) gives the keys of that span, 32 at a time
          const uint32_t my_key = span_key_of_query(qd);
          uint32_t todo = (any_ins != 0u) ? __ballot_sync(0xffffffffu, (qd & TD_SIDPOS) != 0u) : 0u;
          while (todo != 0u) {
            const uint32_t kq = __shfl_sync(0xffffffffu, my_key, __ffs(todo) - 1);
            const bool mine = (my_key == kq);
#pragma unroll
            for (int cc = 0; cc < CPT; ++cc) {
              const uint32_t hit = __ballot_sync(0xffffffffu, span_match_key(kq, kd_pre[cc]) != 0u);
              if (mine) mk[cc] |= hit;
            }
            todo &= ~__ballot_sync(0xffffffffu, mine);
          }
        }
        // the next entry: of this head or, at the end of the list, the first one again for the next head
        if (e + 1 < na || hh + 1 < nh) {
          ent_next = sAct[e + 1 < na ? e + 1 : 0];
          prefetch_kd(ent_next);
        }
        const uint32_t tS = tcol + buf * 128, tP = tS + 64;
        ok = mbar_wait(sfull0 + buf * 8, rnd & 1u, &abortf, a.status, W_Q_SFULL);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after_sync();

#pragma unroll
        for (int cc = 0; cc < CPT; ++cc) {
          uint32_t pk[16];
          uint32_t rs[32], rp[32];
          tmem_ld32(tS + cc * 32, rs);
          tmem_ld32(tP + cc * 32, rp);
          tmem_wait_ld();
          if (cls != KD_TILE_PARTIAL) {   // warp-uniform: the common case carries no mask code at all
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
              const float p0 = fast_exp2(fmaf(__uint_as_float(rs[j]), c, neg_lse));
              const float p1 = fast_exp2(fmaf(__uint_as_float(rs[j + 1]), c, neg_lse));
              pk[j / 2] = pack2<kBf16>(p0 * (__uint_as_float(rp[j]) - delta), p1 * (__uint_as_float(rp[j + 1]) - delta));
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
              float p0 = fast_exp2(fmaf(__uint_as_float(rs[j]), c, neg_lse));
              float p1 = fast_exp2(fmaf(__uint_as_float(rs[j + 1]), c, neg_lse));
              if ((mk[cc] & (1u << j)) == 0u) p0 = 0.f;
              if ((mk[cc] & (2u << j)) == 0u) p1 = 0.f;
              pk[j / 2] = pack2<kBf16>(p0 * (__uint_as_float(rp[j]) - delta), p1 * (__uint_as_float(rp[j + 1]) - delta));
            }
          }
          // dS of the chunk as 16-bit A operand over the start of the scores it was made from (this thread's own row)
          tmem_st16(tS + cc * 32, pk);
        }
        tmem_wait_st();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(pfull0 + buf * 8);
        buf += 2;
        if (buf >= C::NBUF) { buf -= C::NBUF; ++rnd; }
      }
      if (!ok) break;

      // epilogue of this head: warpgroup g stores EC columns of dQ from column g * EC
      if (na > 0) {
        ok = mbar_wait(smem_u32(&bar_acc_full), hh & 1, &abortf, a.status, W_Q_ACCFULL);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
      tc_fence_after_sync();
      constexpr int EC = HD / (2 * C::NSUB);
      constexpr int ECH = EC < 32 ? EC : 32;   // columns per TMEM load
      uint16_t* drow = reinterpret_cast<uint16_t*>(a.dq) + (size_t)b * a.dq_sb + (size_t)h * a.dq_sh + (size_t)qi * a.dq_st + g * EC;
      uint32_t r[EC / ECH][ECH];
      if (na > 0) {
#pragma unroll
        for (int cb = 0; cb < EC / ECH; ++cb) {
          if constexpr (ECH == 16) tmem_ld16(tbase + lane_base + C::TM_ACC0 + g * EC + cb * ECH, r[cb]);
          else tmem_ld32(tbase + lane_base + C::TM_ACC0 + g * EC + cb * ECH, r[cb]);
        }
        tmem_wait_ld();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bar_acc_free));   // the next head's first product may overwrite the accumulator
      } else {
#pragma unroll
        for (int cb = 0; cb < EC / ECH; ++cb)
#pragma unroll
          for (int j = 0; j < ECH; ++j) r[cb][j] = 0u;
      }
      if (q_valid) {
#pragma unroll
        for (int cb = 0; cb < EC / ECH; ++cb) {
          if constexpr (ECH == 16) store_row16_upto<kBf16>(drow + cb * ECH, r[cb], a.sm_scale, g * EC + cb * ECH, a.d_real);
          else store_row32_upto<kBf16>(drow + cb * ECH, r[cb], a.sm_scale, g * EC + cb * ECH, a.d_real);
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tbase, 512);
}

// =========================================================================================
// dK/dV kernel: one CTA per (b, group of heads, key tile); streams = query halves of the current
// query tile.   M1(i): S^T_i = K Q_i^T, dP^T_i = V dO_i^T     M2(i): dV += P^T_i dO_i,  dK += dS^T_i Q_i
// Heads are handled one after the other as in the dQ kernel.
// =========================================================================================
template <int HD, bool kBf16>
__global__ void __launch_bounds__(BwdCfg<HD>::THREADS, 1)
attn_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                     const BwdArgs a) {
  using C = BwdCfg<HD>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sFix = smem_u32(smem + C::SMEM_FIX);    // buffer f: K at +0, V at +TILE_BYTES
  const uint32_t sRing = smem_u32(smem + C::SMEM_RING);  // stage s: Q at +0, dO at +TILE_BYTES
  uint32_t* sStage = reinterpret_cast<uint32_t*>(smem + C::SMEM_STAGE);
  uint16_t* sList = reinterpret_cast<uint16_t*>(smem + C::SMEM_ACT);

  __shared__ __align__(8) uint64_t bar_fix_full[C::NFIX], bar_fix_empty[C::NFIX], bar_ring_full[C::STAGES],
      bar_ring_empty[C::STAGES], bar_s_full[C::NBUF], bar_p_full[C::NBUF], bar_m2_issued[C::NBUF], bar_acc_full, bar_acc_free;
  __shared__ uint32_t tmem_base_s;
  __shared__ AbortFlag abortf;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int h0 = blockIdx.x * a.G, b = blockIdx.y;
  const int nh = min(a.G, a.H - h0);   // this CTA handles heads h0 .. h0 + nh - 1
  const int kt = a.order[((size_t)b * 3 + 2) * a.NT + blockIdx.z];   // longest lists first
  const int n = a.bwd_cnt[b * a.NT + kt];

  if (tid == 0) {
    abortf.v = 0;
    for (int f = 0; f < C::NFIX; ++f) {
      mbar_init(smem_u32(&bar_fix_full[f]), 1);
      mbar_init(smem_u32(&bar_fix_empty[f]), 2);  // both M1 issuers are done with the head's K and V
    }
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(smem_u32(&bar_ring_full[s]), 1);
      mbar_init(smem_u32(&bar_ring_empty[s]), 1);
    }
    for (int i = 0; i < C::NBUF; ++i) {
      mbar_init(smem_u32(&bar_s_full[i]), 2);     // one commit from each of the two M1 issuers
      mbar_init(smem_u32(&bar_p_full[i]), 4 * C::NSUB);   // one arrival per warp of the warpgroups that share the unit
      mbar_init(smem_u32(&bar_m2_issued[i]), 1);
    }
    mbar_init(smem_u32(&bar_acc_full), 1);
    mbar_init(smem_u32(&bar_acc_free), 8 * C::NSUB);      // every compute warp has read its part of dK and dV
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_base_s), 512);
    tmem_relinquish();
  }
  if (warp == 2) {
    const uint16_t* glist = a.bwd_list + ((size_t)b * a.NT + kt) * a.NT;
    for (int e = lane; e < n; e += 32) sList[e] = glist[e];
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tbase = tmem_base_s;
  const uint16_t* list = sList;

  if (warp < 4) {
    reg_dealloc<KD_REGS_ISSUE>();
    if (warp == 0 && lane == 0 && n > 0) {
      // ------------------------------ TMA producer ------------------------------
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      tma_prefetch_desc(&tmDO);
      int issued = 0, fix_issued = 0;   // ring entries / resident pairs requested so far, over all heads
      bool ok = true;
      for (int hh = 0; hh < nh && ok; ++hh) {
        const int h = h0 + hh, fb = hh % C::NFIX;
        if (hh >= C::NFIX) {
          ok = mbar_wait(smem_u32(&bar_fix_empty[fb]), (hh / C::NFIX - 1) & 1, &abortf, a.status, W_K_FIXEMPTY);
          if (!ok) break;
        }
        mbar_arrive_expect_tx(smem_u32(&bar_fix_full[fb]), 2 * C::TILE_BYTES);
        for (int kb = 0; kb < C::KBLK; ++kb) {
          tma_load_4d(sFix + fb * 2 * C::TILE_BYTES + kb * 16384, &tmK, smem_u32(&bar_fix_full[fb]), kb * 64, kt * KD_TILE, h, b);
          tma_load_4d(sFix + fb * 2 * C::TILE_BYTES + C::TILE_BYTES + kb * 16384, &tmV, smem_u32(&bar_fix_full[fb]), kb * 64, kt * KD_TILE, h, b);
        }
        fix_issued = hh + 1;
        for (int e = 0; e < n; ++e) {
          const int s = issued % C::STAGES;
          const uint32_t ph = (issued / C::STAGES) & 1;
          const int qt = list[e] & 0xFF;
          ok = mbar_wait(smem_u32(&bar_ring_empty[s]), ph ^ 1, &abortf, a.status, W_K_RINGEMPTY);
          if (!ok) break;
          mbar_arrive_expect_tx(smem_u32(&bar_ring_full[s]), 2 * C::TILE_BYTES);
          const uint32_t dst = sRing + s * 2 * C::TILE_BYTES;
          for (int kb = 0; kb < C::KBLK; ++kb) {
            tma_load_4d(dst + kb * 16384, &tmQ, smem_u32(&bar_ring_full[s]), kb * 64, qt * KD_TILE, h, b);
            tma_load_4d(dst + C::TILE_BYTES + kb * 16384, &tmDO, smem_u32(&bar_ring_full[s]), kb * 64, qt * KD_TILE, h, b);
          }
          ++issued;
        }
      }
      if (abortf.v != 0) {   // let the copies in flight land before the CTA exits
        for (int e = max(0, issued - C::STAGES); e < issued; ++e)
          for (int spin = 0; spin < (1 << 20) && !mbar_try_wait(smem_u32(&bar_ring_full[e % C::STAGES]), (e / C::STAGES) & 1); ++spin) {}
        for (int f = max(0, fix_issued - C::NFIX); f < fix_issued; ++f)
          for (int spin = 0; spin < (1 << 20) && !mbar_try_wait(smem_u32(&bar_fix_full[f % C::NFIX]), (f / C::NFIX) & 1); ++spin) {}
      }
    } else if ((warp == 3 || warp == 2) && lane == 0 && n > 0) {
      // ------------------------------ M1 issuers: warp 3: S^T_u = K Q_u^T; warp 2: dP^T_u = V dO_u^T ------------------------------
      const bool dp_part = (warp == 2);
      const uint32_t idesc_m1 = make_idesc_f16(kBf16, 0, 0, KD_TILE, 64);   // N = 64 queries
      const uint32_t hi = desc_hi_sw128();
      const uint32_t loRingK = desc_lo_kmajor(sRing);
      const int U = 2 * n;
      bool ok = true;
      int buf = 0, round = 0, stage = 0;   // run on across the heads
      uint32_t ring_parity = 0;
      for (int hh = 0; hh < nh && ok; ++hh) {
        const int fb = hh % C::NFIX;
        ok = mbar_wait(smem_u32(&bar_fix_full[fb]), (hh / C::NFIX) & 1, &abortf, a.status, W_K_FIXFULL);
        if (!ok) break;
        const uint32_t loA = desc_lo_kmajor(sFix + fb * 2 * C::TILE_BYTES + (dp_part ? C::TILE_BYTES : 0));   // V or K
        uint64_t adesc[HD / 16];   // A descriptors of the head's k-steps
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) adesc[kk] = desc64(loA + koff_kmajor(kk), hi);
        for (int u = 0; u < U && ok; ++u) {
          const int i = u & 1;
          // operands of the unit, formed ahead of the waits
          // query rows 64i.. of Q (scores) or dO (dP)
          const uint32_t blo = loRingK + stage * (2 * C::TILE_BYTES >> 4) + i * (64 * 128 >> 4) + (dp_part ? (C::TILE_BYTES >> 4) : 0);
          uint64_t bdesc[HD / 16];
#pragma unroll
          for (int kk = 0; kk < HD / 16; ++kk) bdesc[kk] = desc64(blo + koff_kmajor(kk), hi);
          const uint32_t dst = tbase + buf * 128 + (dp_part ? 64 : 0);
          if (round > 0) {   // buffer free once M2 of its previous unit has been issued
            ok = mbar_wait(smem_u32(&bar_m2_issued[buf]), (round - 1) & 1, &abortf, a.status, W_K_M2ISSUED);
            if (!ok) break;
          }
          if (i == 0) {      // first unit of a new entry: its Q and dO tiles must have landed
            ok = mbar_wait(smem_u32(&bar_ring_full[stage]), ring_parity, &abortf, a.status, W_K_RINGFULL);
            if (!ok) break;
          }
          tc_fence_after_sync();
          mma_ss64<false>(dst, adesc[0], bdesc[0], idesc_m1);
#pragma unroll
          for (int kk = 1; kk < HD / 16; ++kk) mma_ss64<true>(dst, adesc[kk], bdesc[kk], idesc_m1);
          mma_commit(smem_u32(&bar_s_full[buf]));
          if (++buf == C::NBUF) { buf = 0; ++round; }
          if (i == 1 && ++stage == C::STAGES) { stage = 0; ring_parity ^= 1; }
        }
        if (ok) mma_commit(smem_u32(&bar_fix_empty[fb]));   // this issuer's products of the head no longer read K / V
      }
    } else if (warp == 1 && lane == 0 && n > 0) {
      // ------------------------------ M2 issuer: dV += P^T_u dO_u, dK += dS^T_u Q_u ------------------------------
      const uint32_t idesc_m2 = make_idesc_f16(kBf16, 0, 1, KD_TILE, HD);   // B = dO / Q rows, MN-major
      const uint32_t tDK = tbase + C::TM_ACC0, tDV = tbase + C::TM_ACC1;
      const uint32_t hi = desc_hi_sw128();
      const uint32_t loRingMN = desc_lo_mnmajor(sRing);
      const int U = 2 * n;
      bool ok = true;
      int buf = 0, stage = 0;
      uint32_t round_parity = 0;
      for (int hh = 0; hh < nh && ok; ++hh) {
        if (hh > 0) {   // the previous head's dK and dV must have been read out of the accumulators
          ok = mbar_wait(smem_u32(&bar_acc_free), (hh - 1) & 1, &abortf, a.status, W_K_ACCFREE);
          if (!ok) break;
        }
        for (int u = 0; u < U && ok; ++u) {
          const int i = u & 1;
          // operands of the unit, formed ahead of the wait
          const uint32_t qb = loRingMN + stage * (2 * C::TILE_BYTES >> 4) + i * (64 * 128 >> 4);
          const uint32_t dob = qb + (C::TILE_BYTES >> 4);
          const uint32_t aS = tbase + buf * 128;
          // 16-bit operands: queries 0-31 of the unit at columns [0,16) of their buffer half, queries 32-63 at [32,48)
          uint64_t bq[4], bdo[4];
          uint32_t aop[4];
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            bq[kk] = desc64(qb + koff_mnmajor(kk), hi);
            bdo[kk] = desc64(dob + koff_mnmajor(kk), hi);
            aop[kk] = aS + (kk >> 1) * 32 + (kk & 1) * 8;
          }
          ok = mbar_wait(smem_u32(&bar_p_full[buf]), round_parity, &abortf, a.status, W_K_PFULL);
          if (!ok) break;
          tc_fence_after_sync();
          // dV += P^T_u dO_u   (P^T_u on top of S^T_u)
          mma_ts64_p(tDV, aop[0], bdo[0], idesc_m2, u > 0 ? 1u : 0u);
#pragma unroll
          for (int kk = 1; kk < 4; ++kk) mma_ts64<true>(tDV, aop[kk], bdo[kk], idesc_m2);
          // dK += dS^T_u Q_u   (dS^T_u on top of dP^T_u, 64 columns further)
          mma_ts64_p(tDK, aop[0] + 64, bq[0], idesc_m2, u > 0 ? 1u : 0u);
#pragma unroll
          for (int kk = 1; kk < 4; ++kk) mma_ts64<true>(tDK, aop[kk] + 64, bq[kk], idesc_m2);
          if (i == 1) mma_commit(smem_u32(&bar_ring_empty[stage]));
          tc_fence_before_sync();
          mbar_arrive(smem_u32(&bar_m2_issued[buf]));
          if (++buf == C::NBUF) { buf = 0; round_parity ^= 1; }
          if (i == 1 && ++stage == C::STAGES) stage = 0;
        }
        if (ok) mma_commit(smem_u32(&bar_acc_full));
      }
    }
  } else {
    reg_alloc<C::REGS_COMPUTE>();
    // ------------------------------ compute warpgroups ------------------------------
    constexpr int CPT = C::CPT;      // 32-column chunks of a unit this thread handles
    constexpr int QW = 32 * CPT;     // queries of a unit handled by this warp
    const int g = (warp - 4) >> 2;   // warpgroup
    const int i = g / C::NSUB;       // stream: query half (64 queries) of each query tile
    const int c0 = (g % C::NSUB) * CPT;   // first 32-query chunk of that half handled here
    const int wq = warp & 3;
    const int row = wq * 32 + lane;
    const int kj = kt * KD_TILE + row;   // this thread's key
    const bool k_valid = kj < a.T;
    const uint32_t lane_base = static_cast<uint32_t>(wq * 32) << 16;
    uint32_t* st_buf = sStage + (size_t)(warp - 4) * C::STAGE_WORDS;  // [QW lse][QW delta]
    const float c = a.scale_log2;
    const uint32_t kdesc = a.desc[(size_t)b * a.Tpad + kj];
    const int tbw = 2 * i + c0;      // first word of this thread's chunks in the 128-bit class masks of a query tile
    bool ok = true;

    // LSE, delta and the descriptors of the next unit's queries are fetched one unit ahead
    // into registers and handed to the warp through its shared-memory staging buffer
    float pre_lse[CPT], pre_delta[CPT];
    uint32_t pre_desc[CPT];
    // query-side class masks of the next unit: sees-prefix, sees-context, sees-in_span, context, same-span armed
    uint32_t tb_pre[5][CPT];
#pragma unroll
    for (int cc = 0; cc < CPT; ++cc) {
      pre_lse[cc] = 0.f; pre_delta[cc] = 0.f; pre_desc[cc] = 0u;
#pragma unroll
      for (int j = 0; j < 5; ++j) tb_pre[j][cc] = 0u;
    }
    auto prefetch = [&](uint32_t entry, int h) {
      if ((entry >> 8) == KD_TILE_PARTIAL) {
        const uint32_t* tbp = a.tilebits + ((size_t)b * a.NT + (entry & 0xFFu)) * 32;
#pragma unroll
        for (int cc = 0; cc < CPT; ++cc) {
          tb_pre[0][cc] = tbp[4 * TB_SEES_PRE + tbw + cc];
          tb_pre[1][cc] = tbp[4 * TB_SEES_CTX + tbw + cc];
          tb_pre[2][cc] = tbp[4 * TB_SEES_INS + tbw + cc];
          tb_pre[3][cc] = tbp[4 * TB_CTX + tbw + cc];
          tb_pre[4][cc] = tbp[4 * TB_SIDPOS + tbw + cc];
        }
      }
      // a query at or beyond the sequence length reads the last row's scalars: its descriptor is 0,
      // so the tile is PARTIAL and the mask removes it
#pragma unroll
      for (int cc = 0; cc < CPT; ++cc) {
        const int q = (entry & 0xFF) * KD_TILE + i * 64 + (c0 + cc) * 32 + lane;
        const size_t r = ((size_t)b * a.H + h) * a.T + min(q, a.T - 1);
        pre_lse[cc] = a.lse[r];   // negated where it is used: a negation here would wait for the load
        pre_delta[cc] = a.delta[r];
        pre_desc[cc] = a.desc[(size_t)b * a.Tpad + q];
      }
    };
    uint32_t ent_next = n > 0 ? list[0] : 0u;
    if (n > 0) prefetch(ent_next, h0);
    // this stream's next unit, counted over all heads, as (unit / NBUF, unit % NBUF)
    int buf = i % C::NBUF;
    uint32_t rnd = i / C::NBUF;
    const uint32_t sfull0 = smem_u32(&bar_s_full[0]), pfull0 = smem_u32(&bar_p_full[0]);
    const uint32_t tcol = tbase + lane_base + c0 * 32;   // this thread's first chunk inside a buffer

    for (int hh = 0; hh < nh && ok; ++hh) {
      const int h = h0 + hh;
      for (int e = 0; e < n; ++e) {
        const uint32_t ent = ent_next;
        const uint32_t cls = ent >> 8;
        __syncwarp();
#pragma unroll
        for (int cc = 0; cc < CPT; ++cc) {
          st_buf[cc * 32 + lane] = __float_as_uint(pre_lse[cc]);
          st_buf[QW + cc * 32 + lane] = __float_as_uint(pre_delta[cc]);
        }
        __syncwarp();
        uint32_t mk[CPT];   // visibility of this key for the chunks' queries
#pragma unroll
        for (int cc = 0; cc < CPT; ++cc) mk[cc] = 0xFFFFFFFFu;
        if (cls == KD_TILE_PARTIAL) {
          const int i0 = (ent & 0xFF) * KD_TILE + i * 64 + c0 * 32;  // first query handled here
          key_row_mask<CPT>(kdesc, kj, i0, tb_pre[0], tb_pre[1], tb_pre[2], tb_pre[3], mk);
          uint32_t any_armed = 0u;
#pragma unroll
          for (int cc = 0; cc < CPT; ++cc) any_armed |= tb_pre[4][cc];
          // "same span": one round per distinct span among the warp's 32 keys; a ballot over the lanes' query descriptors
          // (lane L holds queries L, 32 + L, ... of the chunks) gives the queries of that span, 32 at a time
          const uint32_t my_key = span_key_of_key(kdesc);
          uint32_t todo = (any_armed != 0u) ? __ballot_sync(0xffffffffu, (kdesc & TD_INS) != 0u) : 0u;
          while (todo != 0u) {
            const uint32_t kk = __shfl_sync(0xffffffffu, my_key, __ffs(todo) - 1);
            const bool mine = (my_key == kk);
#pragma unroll
            for (int cc = 0; cc < CPT; ++cc) {
              const uint32_t hit = __ballot_sync(0xffffffffu, span_match_query(kk, pre_desc[cc]) != 0u);
              if (mine) mk[cc] |= hit;
            }
            todo &= ~__ballot_sync(0xffffffffu, mine);
          }
        }
        // the next entry: of this head or, at the end of the list, the first one again for the next head
        if (e + 1 < n) {
          ent_next = list[e + 1];
          prefetch(ent_next, h);
        } else if (hh + 1 < nh) {
          ent_next = list[0];
          prefetch(ent_next, h + 1);
        }
        const uint32_t tS = tcol + buf * 128, tP = tS + 64;
        ok = mbar_wait(sfull0 + buf * 8, rnd & 1u, &abortf, a.status, W_K_SFULL);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after_sync();

#pragma unroll
        for (int cc = 0; cc < CPT; ++cc) {
          uint32_t pk_p[16], pk_ds[16];
          uint32_t rs[32], rp[32];
          tmem_ld32(tS + cc * 32, rs);
          tmem_ld32(tP + cc * 32, rp);
          tmem_wait_ld();
          if (cls != KD_TILE_PARTIAL) {   // warp-uniform: the common case carries no mask code at all
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              const float4 l4 = *reinterpret_cast<const float4*>(st_buf + cc * 32 + j);        // LSE of 4 queries
              const float4 d4 = *reinterpret_cast<const float4*>(st_buf + QW + cc * 32 + j);   // delta of 4 queries
              const float lw[4] = {l4.x, l4.y, l4.z, l4.w}, dw[4] = {d4.x, d4.y, d4.z, d4.w};
              float pv[4], ds[4];
#pragma unroll
              for (int u2 = 0; u2 < 4; ++u2) pv[u2] = fast_exp2(fmaf(__uint_as_float(rs[j + u2]), c, -lw[u2]));
#pragma unroll
              for (int u2 = 0; u2 < 4; ++u2) ds[u2] = pv[u2] * (__uint_as_float(rp[j + u2]) - dw[u2]);
              pk_p[j / 2] = pack2<kBf16>(pv[0], pv[1]);
              pk_p[j / 2 + 1] = pack2<kBf16>(pv[2], pv[3]);
              pk_ds[j / 2] = pack2<kBf16>(ds[0], ds[1]);
              pk_ds[j / 2 + 1] = pack2<kBf16>(ds[2], ds[3]);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              const float4 l4 = *reinterpret_cast<const float4*>(st_buf + cc * 32 + j);
              const float4 d4 = *reinterpret_cast<const float4*>(st_buf + QW + cc * 32 + j);
              const float lw[4] = {l4.x, l4.y, l4.z, l4.w}, dw[4] = {d4.x, d4.y, d4.z, d4.w};
              float pv[4], ds[4];
#pragma unroll
              for (int u2 = 0; u2 < 4; ++u2) {
                pv[u2] = fast_exp2(fmaf(__uint_as_float(rs[j + u2]), c, -lw[u2]));
                if ((mk[cc] & (1u << (j + u2))) == 0u) pv[u2] = 0.f;
              }
#pragma unroll
              for (int u2 = 0; u2 < 4; ++u2) ds[u2] = pv[u2] * (__uint_as_float(rp[j + u2]) - dw[u2]);
              pk_p[j / 2] = pack2<kBf16>(pv[0], pv[1]);
              pk_p[j / 2 + 1] = pack2<kBf16>(pv[2], pv[3]);
              pk_ds[j / 2] = pack2<kBf16>(ds[0], ds[1]);
              pk_ds[j / 2 + 1] = pack2<kBf16>(ds[2], ds[3]);
            }
          }
          tmem_st16(tS + cc * 32, pk_p);    // P^T of the chunk over the start of the scores it was made from
          tmem_st16(tP + cc * 32, pk_ds);   // dS^T of the chunk over the start of its dP^T
        }
        tmem_wait_st();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(pfull0 + buf * 8);
        buf += 2;
        if (buf >= C::NBUF) { buf -= C::NBUF; ++rnd; }
      }
      if (!ok) break;

      // epilogue of this head: warpgroup g stores EC columns of dK and dV from column g * EC
      if (n > 0) {
        ok = mbar_wait(smem_u32(&bar_acc_full), hh & 1, &abortf, a.status, W_K_ACCFULL);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
      tc_fence_after_sync();
      constexpr int EC = HD / (2 * C::NSUB);
      constexpr int ECH = EC < 32 ? EC : 32;   // columns per TMEM load
      uint16_t* krow = reinterpret_cast<uint16_t*>(a.dk) + (size_t)b * a.dk_sb + (size_t)h * a.dk_sh + (size_t)kj * a.dk_st + g * EC;
      uint16_t* vrow = reinterpret_cast<uint16_t*>(a.dv) + (size_t)b * a.dv_sb + (size_t)h * a.dv_sh + (size_t)kj * a.dv_st + g * EC;
#pragma unroll
      for (int cb = 0; cb < EC / ECH; ++cb) {
        uint32_t rk[ECH], rv[ECH];
        if (n > 0) {
          if constexpr (ECH == 16) {
            tmem_ld16(tbase + lane_base + C::TM_ACC0 + g * EC + cb * ECH, rk);
            tmem_ld16(tbase + lane_base + C::TM_ACC1 + g * EC + cb * ECH, rv);
          } else {
            tmem_ld32(tbase + lane_base + C::TM_ACC0 + g * EC + cb * ECH, rk);
            tmem_ld32(tbase + lane_base + C::TM_ACC1 + g * EC + cb * ECH, rv);
          }
          tmem_wait_ld();
          if (cb == EC / ECH - 1) {
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bar_acc_free));   // the next head's first products may overwrite the accumulators
          }
        } else {
#pragma unroll
          for (int j = 0; j < ECH; ++j) { rk[j] = 0u; rv[j] = 0u; }
        }
        if (k_valid) {
          if constexpr (ECH == 16) {
            store_row16_upto<kBf16>(krow + cb * ECH, rk, a.sm_scale, g * EC + cb * ECH, a.d_real);
            store_row16_upto<kBf16>(vrow + cb * ECH, rv, 1.0f, g * EC + cb * ECH, a.d_real);
          } else {
            store_row32_upto<kBf16>(krow + cb * ECH, rk, a.sm_scale, g * EC + cb * ECH, a.d_real);
            store_row32_upto<kBf16>(vrow + cb * ECH, rv, 1.0f, g * EC + cb * ECH, a.d_real);
          }
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tbase, 512);
}

template <int HD, bool kBf16>
static int launch_bwd_t(const kd_attn_params& p, const kd_plan_layout& L, const PlanView& pv, cudaStream_t stream) {
  using C = BwdCfg<HD>;
  CUtensorMap tmQ, tmK, tmV, tmDO;
  int rc;
  if ((rc = encode_tensor_map(&tmQ, p.q, p.B, p.H, p.T, p.D, p.dtype, KD_TILE, "q")) != 0) return rc;
  if ((rc = encode_tensor_map(&tmK, p.k, p.B, p.H, p.T, p.D, p.dtype, KD_TILE, "k")) != 0) return rc;
  if ((rc = encode_tensor_map(&tmV, p.v, p.B, p.H, p.T, p.D, p.dtype, KD_TILE, "v")) != 0) return rc;
  if ((rc = encode_tensor_map(&tmDO, p.d_o, p.B, p.H, p.T, p.D, p.dtype, KD_TILE, "do")) != 0) return rc;
  BwdArgs a;
  a.B = p.B; a.H = p.H; a.T = p.T; a.NT = L.NT; a.NP = L.NP; a.Tpad = L.NT * KD_TILE;
  a.d_real = p.D;
  a.scale_log2 = p.sm_scale * 1.4426950408889634f;
  a.sm_scale = p.sm_scale;
  a.G = heads_per_cta(p.B, p.H, L.NT, p.heads_per_cta);
  a.desc = pv.desc; a.fwd_cnt = pv.fwd_cnt; a.fwd_list = pv.fwd_list;
  a.bwd_cnt = pv.bwd_cnt; a.bwd_list = pv.bwd_list; a.status = pv.status; a.order = pv.order; a.tilebits = pv.tilebits;
  a.o = p.o.ptr; a.o_sb = p.o.stride_b; a.o_sh = p.o.stride_h; a.o_st = p.o.stride_t;
  a.d_o = p.d_o.ptr; a.do_sb = p.d_o.stride_b; a.do_sh = p.d_o.stride_h; a.do_st = p.d_o.stride_t;
  a.lse = p.lse; a.delta = p.delta;
  const bool fused = (p.bwd_mode == KD_BWD_FUSED);
  a.dq_acc = fused ? p.dq_acc : nullptr;
  a.dq = p.dq.ptr; a.dq_sb = p.dq.stride_b; a.dq_sh = p.dq.stride_h; a.dq_st = p.dq.stride_t;
  a.dk = p.dk.ptr; a.dk_sb = p.dk.stride_b; a.dk_sh = p.dk.stride_h; a.dk_st = p.dk.stride_t;
  a.dv = p.dv.ptr; a.dv_sb = p.dv.stride_b; a.dv_sh = p.dv.stride_h; a.dv_st = p.dv.stride_t;
 
  auto kq = attn_bwd_dq_kernel<HD, kBf16>;
  auto kk = attn_bwd_dkdv_kernel<HD, kBf16>;
  cudaError_t e = cudaFuncSetAttribute(kq, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_ALLOC);
  if (e == cudaSuccess) e = cudaFuncSetAttribute(kk, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_ALLOC);
  if (e != cudaSuccess) return set_error(KD_ERR_DEVICE, "bwd smem attribute: %s", cudaGetErrorString(e));
  dim3 grid((p.H + a.G - 1) / a.G, p.B, L.NT);
  const int phases = (p.bwd_phases & 3) ? (p.bwd_phases & 3) : 3;
  if (phases & 1) {
    const size_t rows = (size_t)p.B * p.H * p.T;
    const int rows_per_block = 256 / (HD / 8);
    const int blocks = static_cast<int>(std::min<size_t>((rows + rows_per_block - 1) / rows_per_block, size_t(148) * 32));
    attn_bwd_delta_kernel<HD, kBf16><<<blocks, 256, 0, stream>>>(a);
    if (!fused) kq<<<grid, C::THREADS, C::SMEM_ALLOC, stream>>>(tmQ, tmK, tmV, tmDO, a);
  }
  if (fused) {
    // bwd_phases 1: the delta kernel alone (it also zeroes dq_acc); 2: the fused kernel and the conversion
    if constexpr (HD == 64) {
      if (phases & 2) return launch_bwd_fused(tmQ, tmK, tmV, tmDO, a, p.dtype, grid, stream);
    }
  } else if (phases & 2) {
    kk<<<grid, C::THREADS, C::SMEM_ALLOC, stream>>>(tmQ, tmK, tmV, tmDO, a);
  }
  e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(KD_ERR_DEVICE, "attn_bwd kernels launch: %s", cudaGetErrorString(e));
  return 0;
}

// ---------------------------------------------------------------------------------------
// Library-owned scratch for kd_attn_bwd_static.
//
// Some hosts may not allocate device memory on the path that calls the backward: an inference or
// training engine that hands every byte of HBM to its own arena at start-up and forbids plugin
// code to call cudaMalloc afterwards, or a caller that is already inside a region where the
// allocator must not run. For them the `delta` scratch of the backward (one float per
// (batch, head, token) row) lives in this fixed array instead of in a caller-supplied buffer.
// Every GPU that loads the library holds the array (4 MiB) until the process exits.
//
// In host code the name of a __device__ array is only a handle; the device address a kernel can
// use is obtained with cudaGetSymbolAddress, once per device, with that device current.
// ---------------------------------------------------------------------------------------
constexpr size_t KD_STATIC_DELTA_ROWS = size_t(1) << 20;   // B*H*T may not exceed this
static __device__ __align__(256) float g_static_delta[KD_STATIC_DELTA_ROWS];

constexpr int KD_MAX_DEVICES = 64;
static float* g_static_delta_addr[KD_MAX_DEVICES] = {};
static std::mutex g_static_delta_mutex;

// Device address of the static scratch on the current device (looked up on first use per device).
int static_delta_address(size_t rows_needed, float** out) {
  if (rows_needed > KD_STATIC_DELTA_ROWS)
    return set_error(KD_ERR_LIMIT, "kd_attn_bwd_static: B*H*T = %zu rows exceed the built-in scratch of %zu rows; "
                     "use kd_attn_bwd with a caller-provided delta buffer", rows_needed, KD_STATIC_DELTA_ROWS);
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return set_error(KD_ERR_DEVICE, "cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= KD_MAX_DEVICES) return set_error(KD_ERR_LIMIT, "device ordinal %d beyond %d", dev, KD_MAX_DEVICES);
  std::lock_guard<std::mutex> lock(g_static_delta_mutex);
  if (g_static_delta_addr[dev] == nullptr) {
    float* ptr = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_static_delta);
    if (e != cudaSuccess || ptr == nullptr)
      return set_error(KD_ERR_DEVICE, "cudaGetSymbolAddress(static delta scratch): %s", cudaGetErrorString(e));
    g_static_delta_addr[dev] = ptr;
  }
  *out = g_static_delta_addr[dev];
  return 0;
}

int launch_attn_bwd(const kd_attn_params& p, cudaStream_t stream) {
  kd_plan_layout L;
  if (kd_plan_layout_get(p.B, p.T, &L) != 0) return KD_ERR_ARG;
  PlanView pv = make_plan_view(const_cast<void*>(p.plan), L);
  if (!p.d_o.ptr) return set_error(KD_ERR_ARG, "d_o is null");
  if (p.D <= 64) return p.dtype == KD_BF16 ? launch_bwd_t<64, true>(p, L, pv, stream) : launch_bwd_t<64, false>(p, L, pv, stream);
  return p.dtype == KD_BF16 ? launch_bwd_t<128, true>(p, L, pv, stream) : launch_bwd_t<128, false>(p, L, pv, stream);
}

}  // namespace kd
