// Fused backward for head dim 64 on sm_100a: dK, dV and dQ from ONE pass over the non-empty tiles.
//
// The two-kernel backward (attn_bwd.cu) follows the reference's split into a dQ worker and a dK/dV
// worker (original_kernel.py:1173-1336, :1339-1525) and so forms S = Q K^T, dP = dO V^T and the
// exponentials twice per tile: 7 matrix products and two exponential passes. This kernel is key-tile
// major like the dK/dV worker and forms them once: per (query tile, key tile)
//     S^T = K Q^T, dP^T = V dO^T                           (smem x smem -> TMEM, in two halves of 64 queries)
//     P^T = exp2(S^T c - LSE), dS^T = P^T (dP^T - delta)   (compute warps; 16-bit results)
//     dV += P^T dO                                         (P^T read from TMEM as the A operand)
//     dK += dS^T Q,  dQ_tile = dS K                        (dS^T written to shared memory once and read by
//                                                           the tensor core K-major for dK, MN-major for dQ)
// 5 products and one exponential pass. dK and dV stay in TMEM for the whole key tile; the dQ partial of
// every tile is added to an fp32 scratch (B,H,T,64) by a TMA bulk reduction (cp.reduce.async.bulk.tensor
// .add, fp32 adds performed in L2 on whole 128-byte lines; the additions of different key tiles arrive in
// no fixed order, so dQ is not bit-reproducible from run to run) and a bandwidth-bound kernel converts
// the scratch to the output dtype afterwards. The delta kernel, which runs first anyway, zeroes the
// scratch. The dQ tile is staged for the reduction in the shared-memory buffer its own dS^T came from,
// which the products have finished reading by then.
//
// Pipeline. P^T has its own TMEM columns and dS^T goes to shared memory, so the S^T / dP^T columns are free
// again as soon as the compute warps have LOADED them. The tile's 128 query columns are two halves with
// their own barriers throughout: warpgroups 0-1 own the first half, 2-3 the second, the S^T / dP^T products
// of a half (N = 64) are issued as soon as that half's columns have been loaded, and dV and dK take a half's
// 64 queries of their inner dimension as soon as that half's P^T / dS^T are written. The two pairs of
// warpgroups therefore run as two pipelines that drift apart in time, and the accumulating products of a
// tile run while the compute warps work on the next one. Every TMEM region is single-buffered (S^T 128 +
// dP^T 128 + P^T 64 + dK 64 + dV 64 + dQ 64 = 512 columns); only dS^T in shared memory is double-buffered.
//
// Heads. A CTA handles several heads of its (batch, key tile) one after the other, and nothing drains between
// them: the ring of Q / dO tiles runs on into the next head; K has two buffers (the next head's K is requested
// a head ahead by the dK / dQ issuer, when the last dQ product of the head before has released the buffer) and
// V one (requested by the S^T / dP^T issuer right after the head's last dP^T product, about a tile before the
// head ends), so the next head's first products are issued while this head's last tile is still in the compute
// warps; dK and dV of the finished head leave through the dQ warps, and only the next head's first
// accumulating products wait for that.
//
// 768 threads: warp 0 producer (lane 0 issues the TMA loads of Q and dO; all lanes copy LSE, delta, token
// descriptors and mask words of the stage's 128 queries to shared memory, so that compute warps find them
// there and issue no global loads); warp 3 issues S^T and dP^T; warp 1 issues dV and warp 2 dK and dQ (24
// products per tile from one thread would make that thread the slowest stage); warps 4-19 are four compute
// warpgroups (32 query columns each, a key row per thread); warps 20-23 move finished dQ tiles from TMEM to
// the scratch and write dK and dV at the end of each head.
#include <algorithm>

#include "attn_bwd.cuh"

namespace kd {

struct FusedCfg {
  static constexpr int HD = 64;
  static constexpr int TILE_BYTES = KD_TILE * HD * 2;
  static constexpr int STAGES = 3;                   // ring of streamed (Q, dO) tile pairs: a stage is held from its TMA load until
                                                     // the tile's dV and dK products have completed, about two tile periods
  // resident tiles of the CTA's key tile: K in two buffers (head hh in buffer hh % 2), V in one. V's last reader in a head
  // is a dP^T product, issued about one tile before the head ends, so the next head's V lands in time without a second
  // buffer; K's last reader is the head's last dQ product, so the next head's K has to be there already.
  static constexpr int SMEM_K = 0;
  static constexpr int SMEM_V = SMEM_K + 2 * TILE_BYTES;
  static constexpr int SMEM_RING = SMEM_V + TILE_BYTES;
  static constexpr int SMEM_DS = SMEM_RING + STAGES * 2 * TILE_BYTES;   // 2 x dS^T of a query tile: two [128 keys][64 queries] blocks
  // per ring stage, beside the tiles: LSE, delta and token descriptor of the stage's 128 queries and the 32 mask words of
  // the query tile, copied there by the producer warp
  static constexpr int SIDE_WORDS = 3 * KD_TILE + 32;
  static constexpr int SMEM_SIDE = SMEM_DS + 2 * 2 * TILE_BYTES;
  static constexpr int SMEM_LIST = SMEM_SIDE + STAGES * SIDE_WORDS * 4;
  static constexpr int SMEM_TOTAL = SMEM_LIST + 128 * 2;
  static constexpr int SMEM_ALLOC = SMEM_TOTAL + 1024;
  static constexpr int THREADS = 768;
  static constexpr uint32_t TM_S = 0, TM_DP = 128, TM_PT = 256, TM_DK = 320, TM_DV = 384, TM_DQ = 448;
  static_assert(TM_DQ + HD <= 512, "TMEM budget");
  static_assert(SMEM_ALLOC <= 232448, "shared memory budget");
  // registers: 80 per thread at launch; light warps release down to 56, the dQ warps to 72, compute warps take 88
  static constexpr int REGS_LIGHT = 56, REGS_DQ = 72, REGS_COMPUTE = 88;
  static constexpr int REGS_LAUNCH = 80;             // per thread at launch: 6 warps per scheduler x 32 x 80 fit its 16384 registers
  static_assert(4 * 32 * REGS_LIGHT + 4 * 32 * REGS_DQ + 16 * 32 * REGS_COMPUTE <= THREADS * REGS_LAUNCH, "register pool");
  static_assert(THREADS == 768, "a 25th warp would put 7 warps on one scheduler and cut the launch count to 72 registers");
};

enum : uint32_t {
  W_U_FIXFULL = 0x401, W_U_RINGEMPTY = 0x402, W_U_RINGFULL = 0x403, W_U_PFULL = 0x404, W_U_SFULL = 0x405,
  W_U_ACCFULL = 0x406, W_U_SPFREE = 0x407, W_U_FIXEMPTY = 0x408, W_U_ACCFREE = 0x409, W_U_DQFULL = 0x40A,
  W_U_DQEMPTY = 0x40B, W_U_DSEMPTY = 0x40C, W_U_PTFREE = 0x40D, W_U_SFULL1 = 0x40E, W_U_SPFREE1 = 0x40F, W_U_VFULL = 0x410,
};

__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
               ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}
__device__ __forceinline__ void st_shared_v4(uint32_t saddr, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(saddr), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}

template <bool kBf16>
__global__ void __launch_bounds__(FusedCfg::THREADS, 1)
attn_bwd_fused_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                      const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                      const __grid_constant__ CUtensorMap tmAcc, const BwdArgs a) {
  using C = FusedCfg;
  constexpr int HD = C::HD;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sK = smem_u32(smem + C::SMEM_K);        // K of head hh at + (hh % 2) TILE_BYTES
  const uint32_t sV = smem_u32(smem + C::SMEM_V);
  const uint32_t sRing = smem_u32(smem + C::SMEM_RING);  // stage s: Q at +0, dO at +TILE_BYTES
  const uint32_t sDS = smem_u32(smem + C::SMEM_DS);      // buffer t: block 0 (queries 0-63) at +0, block 1 at +TILE_BYTES
  uint32_t* sSide = reinterpret_cast<uint32_t*>(smem + C::SMEM_SIDE);
  uint16_t* sList = reinterpret_cast<uint16_t*>(smem + C::SMEM_LIST);

  __shared__ __align__(8) uint64_t bar_k_full[2], bar_k_empty[2], bar_v_full, bar_v_empty, bar_ring_full[C::STAGES],
      bar_ring_empty[C::STAGES], bar_s_full[2], bar_sp_free[2], bar_p_full[2][2], bar_pt_free[2], bar_acc_full, bar_acc_free[2],
      bar_dq_full, bar_dq_empty, bar_ds_empty[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ AbortFlag abortf;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int h0 = blockIdx.x * a.G, b = blockIdx.y;
  const int nh = min(a.G, a.H - h0);   // this CTA handles heads h0 .. h0 + nh - 1
  const int kt = a.order[((size_t)b * 3 + 2) * a.NT + blockIdx.z];   // longest lists first
  const int n = a.bwd_cnt[b * a.NT + kt];

  if (tid == 0) {
    abortf.v = 0;
    for (int f = 0; f < 2; ++f) {
      mbar_init(smem_u32(&bar_k_full[f]), 1);
      mbar_init(smem_u32(&bar_k_empty[f]), 1);   // the head's last dQ product has read K (its S^T products were issued, and so
                                                 // completed, before it: the tensor pipe runs in issue order)
    }
    mbar_init(smem_u32(&bar_v_full), 1);
    mbar_init(smem_u32(&bar_v_empty), 1);        // the head's last dP^T product has read V
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(smem_u32(&bar_ring_full[s]), 2);    // the TMA loads (with their byte count) and the producer warp's own copies
      mbar_init(smem_u32(&bar_ring_empty[s]), 2);   // the dV issuer and the dK / dQ issuer are done with the stage
    }
    // S^T and dP^T are produced and released in two halves of 64 query columns
    mbar_init(smem_u32(&bar_s_full[0]), 1);
    mbar_init(smem_u32(&bar_s_full[1]), 1);
    // the warps of a role arrive once each (lane 0, after a warp-wide sync): hundreds of single-thread arrivals on one
    // barrier would serialise in the shared-memory atomic unit
    // every barrier of a half is used by the two compute warpgroups (8 warps) that own the half
    mbar_init(smem_u32(&bar_sp_free[0]), 8);   // the warps have loaded their S^T and dP^T columns
    mbar_init(smem_u32(&bar_sp_free[1]), 8);
    // P^T of the half is in TMEM and its dS^T block in shared memory. Two barriers per half, used by even and odd tiles: with
    // two dS^T buffers the compute warps may finish two tiles before the dK / dQ issuer has looked at the first, and a parity
    // wait on a single barrier cannot tell "two phases on" from "not yet"
    for (int f = 0; f < 4; ++f) mbar_init(smem_u32(&bar_p_full[f >> 1][f & 1]), 8);
    mbar_init(smem_u32(&bar_pt_free[0]), 1);   // the dV products have read the half's P^T
    mbar_init(smem_u32(&bar_pt_free[1]), 1);
    mbar_init(smem_u32(&bar_dq_full), 1);
    mbar_init(smem_u32(&bar_dq_empty), 4);     // the dQ warps have read the dQ tile out of TMEM
    mbar_init(smem_u32(&bar_ds_empty[0]), 1);  // a dS^T buffer is free: its products and the reduction staged in it are done
    mbar_init(smem_u32(&bar_ds_empty[1]), 1);
    mbar_init(smem_u32(&bar_acc_full), 2);       // both accumulating issuers have committed the head's last products
    mbar_init(smem_u32(&bar_acc_free[0]), 4);  // the dQ warps have read dV out of TMEM
    mbar_init(smem_u32(&bar_acc_free[1]), 4);  // ... and dK
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
    reg_dealloc<C::REGS_LIGHT>();
    if (warp == 0 && n > 0) {
      // ------------------------------ producer warp ------------------------------
      // lane 0 issues the TMA loads; all lanes copy the per-query scalars of the stage (4 queries each) and the tile's
      // mask words (one each) with plain loads, so that the compute warps find everything about a tile in shared memory
      if (lane == 0) {
        tma_prefetch_desc(&tmQ);
        tma_prefetch_desc(&tmK);
        tma_prefetch_desc(&tmV);
        tma_prefetch_desc(&tmDO);
      }
      int issued = 0;   // ring entries requested so far, over all heads
      bool ok = true;
      if (lane == 0) {
        // K and V of the first head and K of the second; later heads' tiles are requested by the issuing threads that see
        // the buffers fall free (the dK / dQ issuer for K, the S^T / dP^T issuer for V)
        mbar_arrive_expect_tx(smem_u32(&bar_k_full[0]), C::TILE_BYTES);
        tma_load_4d(sK, &tmK, smem_u32(&bar_k_full[0]), 0, kt * KD_TILE, h0, b);
        mbar_arrive_expect_tx(smem_u32(&bar_v_full), C::TILE_BYTES);
        tma_load_4d(sV, &tmV, smem_u32(&bar_v_full), 0, kt * KD_TILE, h0, b);
        if (nh > 1) {
          mbar_arrive_expect_tx(smem_u32(&bar_k_full[1]), C::TILE_BYTES);
          tma_load_4d(sK + C::TILE_BYTES, &tmK, smem_u32(&bar_k_full[1]), 0, kt * KD_TILE, h0 + 1, b);
        }
      }
      for (int hh = 0; hh < nh && ok; ++hh) {
        const int h = h0 + hh;
        const float* lse_row = a.lse + ((size_t)b * a.H + h) * a.T;
        const float* delta_row = a.delta + ((size_t)b * a.H + h) * a.T;
        for (int e = 0; e < n; ++e) {
          const int s = issued % C::STAGES;
          const uint32_t ph = (issued / C::STAGES) & 1;
          const int qt = list[e] & 0xFF;
          // the scalars are requested before the wait for the stage: the wait covers their latency
          // (a query at or beyond the sequence length reads the last row's scalars: its descriptor is 0, so the tile is
          // PARTIAL and the mask removes it)
          const int q = qt * KD_TILE + 4 * lane;
          float4 l4, d4;
          l4.x = lse_row[min(q + 0, a.T - 1)]; l4.y = lse_row[min(q + 1, a.T - 1)];
          l4.z = lse_row[min(q + 2, a.T - 1)]; l4.w = lse_row[min(q + 3, a.T - 1)];
          d4.x = delta_row[min(q + 0, a.T - 1)]; d4.y = delta_row[min(q + 1, a.T - 1)];
          d4.z = delta_row[min(q + 2, a.T - 1)]; d4.w = delta_row[min(q + 3, a.T - 1)];
          if (lane == 0) {
            ok = mbar_wait(smem_u32(&bar_ring_empty[s]), ph ^ 1, &abortf, a.status, W_U_RINGEMPTY);
            if (ok) {
              mbar_arrive_expect_tx(smem_u32(&bar_ring_full[s]), 2 * C::TILE_BYTES);
              const uint32_t dst = sRing + s * 2 * C::TILE_BYTES;
              tma_load_4d(dst, &tmQ, smem_u32(&bar_ring_full[s]), 0, qt * KD_TILE, h, b);
              tma_load_4d(dst + C::TILE_BYTES, &tmDO, smem_u32(&bar_ring_full[s]), 0, qt * KD_TILE, h, b);
            }
          }
          ok = __shfl_sync(0xffffffffu, ok, 0);
          if (!ok) break;
          // (descriptors and mask words are fetched after the wait: held across it they would not fit this warp's registers)
          const uint4 c4 = *reinterpret_cast<const uint4*>(a.desc + (size_t)b * a.Tpad + q);   // the descriptor rows are padded to whole tiles
          const uint32_t tbw = a.tilebits[((size_t)b * a.NT + qt) * 32 + lane];
          uint32_t* side = sSide + s * C::SIDE_WORDS;
          *reinterpret_cast<float4*>(side + 4 * lane) = l4;
          *reinterpret_cast<float4*>(side + KD_TILE + 4 * lane) = d4;
          *reinterpret_cast<uint4*>(side + 2 * KD_TILE + 4 * lane) = c4;
          side[3 * KD_TILE + lane] = tbw;
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&bar_ring_full[s]));
          ++issued;
        }
      }
      if (lane == 0 && abortf.v != 0) {   // let the copies in flight land before the CTA exits
        for (int e = max(0, issued - C::STAGES); e < issued; ++e) drain_wait(smem_u32(&bar_ring_full[e % C::STAGES]), (e / C::STAGES) & 1);
        drain_wait(smem_u32(&bar_k_full[0]), 0);
        drain_wait(smem_u32(&bar_v_full), 0);
        if (nh > 1) drain_wait(smem_u32(&bar_k_full[1]), 0);
      }
    } else if (warp == 3 && lane == 0 && n > 0) {
      // ------- M1 issuer: per half of 64 queries, S^T = K Q^T and dP^T = V dO^T into columns 64 half .. 64 half + 63 -------
      const uint32_t idesc_m1 = make_idesc_f16(kBf16, 0, 0, KD_TILE, KD_TILE / 2);
      const uint32_t hi = desc_hi_sw128();
      const uint32_t loRingK = desc_lo_kmajor(sRing);
      bool ok = true;
      int t = 0, stage = 0;   // tiles so far and ring stage, running on across the heads
      uint32_t ring_parity = 0;
      int v_loads = 1;        // V tiles requested so far (the first by the producer)
      for (int hh = 0; hh < nh && ok; ++hh) {
        ok = mbar_wait(smem_u32(&bar_k_full[hh & 1]), (hh >> 1) & 1, &abortf, a.status, W_U_FIXFULL);
        if (!ok) break;
        const uint32_t loK = desc_lo_kmajor(sK + (hh & 1) * C::TILE_BYTES), loV = desc_lo_kmajor(sV);
        bool v_ready = false;
        for (int e = 0; e < n && ok; ++e) {
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            // rows 64 half .. of the stage's Q and dO tiles (128 bytes per row)
            const uint32_t qlo = loRingK + stage * (2 * C::TILE_BYTES >> 4) + half * (C::TILE_BYTES >> 5), dolo = qlo + (C::TILE_BYTES >> 4);
            const uint32_t tS = tbase + C::TM_S + half * 64, tDP = tbase + C::TM_DP + half * 64;
            if (t > 0) {   // the compute warps must have loaded the previous tile's columns of this half
              ok = mbar_wait(smem_u32(&bar_sp_free[half]), (t - 1) & 1, &abortf, a.status, half ? W_U_SPFREE1 : W_U_SPFREE);
              if (!ok) break;
            }
            if (half == 0) {
              ok = mbar_wait(smem_u32(&bar_ring_full[stage]), ring_parity, &abortf, a.status, W_U_RINGFULL);
              if (!ok) break;
            }
            tc_fence_after_sync();
            mma_ss64<false>(tS, desc64(loK, hi), desc64(qlo, hi), idesc_m1);
#pragma unroll
            for (int kk = 1; kk < HD / 16; ++kk) mma_ss64<true>(tS, desc64(loK + koff_kmajor(kk), hi), desc64(qlo + koff_kmajor(kk), hi), idesc_m1);
            if (!v_ready) {   // the head's V is requested late (below), so it is waited for only where it is first needed
              ok = mbar_wait(smem_u32(&bar_v_full), hh & 1, &abortf, a.status, W_U_VFULL);
              if (!ok) break;
              v_ready = true;
            }
            mma_ss64<false>(tDP, desc64(loV, hi), desc64(dolo, hi), idesc_m1);
#pragma unroll
            for (int kk = 1; kk < HD / 16; ++kk) mma_ss64<true>(tDP, desc64(loV + koff_kmajor(kk), hi), desc64(dolo + koff_kmajor(kk), hi), idesc_m1);
            mma_commit(smem_u32(&bar_s_full[half]));
          }
          ++t;
          if (++stage == C::STAGES) { stage = 0; ring_parity ^= 1; }
        }
        if (!ok) break;
        mma_commit(smem_u32(&bar_v_empty));           // the head's dP^T products no longer read V
        if (hh + 1 < nh) {
          // The next head's V goes into the same buffer: this thread waits for its own last products (a few hundred cycles,
          // during which it has nothing else to issue: the next S^T needs columns the compute warps are still reading)
          // and requests the tile.
          ok = mbar_wait(smem_u32(&bar_v_empty), hh & 1, &abortf, a.status, W_U_FIXEMPTY);
          if (!ok) break;
          mbar_arrive_expect_tx(smem_u32(&bar_v_full), C::TILE_BYTES);
          tma_load_4d(sV, &tmV, smem_u32(&bar_v_full), 0, kt * KD_TILE, h0 + hh + 1, b);
          v_loads = hh + 2;
        }
      }
      if (abortf.v != 0 && v_loads > 1) drain_wait(smem_u32(&bar_v_full), (v_loads - 1) & 1);   // let a copy in flight land
    } else if (warp == 1 && lane == 0 && n > 0) {
      // ------- dV issuer: per tile dV += P^T dO (A from TMEM) -------
      const uint32_t idesc_dv = make_idesc_f16(kBf16, 0, 1, KD_TILE, HD);   // B = dO rows, MN-major
      const uint32_t tDV = tbase + C::TM_DV, tPT = tbase + C::TM_PT;
      const uint32_t hi = desc_hi_sw128();
      const uint32_t loRingMN = desc_lo_mnmajor(sRing);
      bool ok = true;
      int t = 0, stage = 0;
      for (int hh = 0; hh < nh && ok; ++hh) {
        if (hh > 0) {   // the previous head's dK and dV must have been read out of the accumulators
          ok = mbar_wait(smem_u32(&bar_acc_free[0]), (hh - 1) & 1, &abortf, a.status, W_U_ACCFREE);
          if (!ok) break;
        }
        for (int e = 0; e < n && ok; ++e) {
          const uint32_t dob = loRingMN + stage * (2 * C::TILE_BYTES >> 4) + (C::TILE_BYTES >> 4);
#pragma unroll
          for (int half = 0; half < 2; ++half) {   // 64 queries of the product's inner dimension at a time
            ok = mbar_wait(smem_u32(&bar_p_full[half][t & 1]), (t >> 1) & 1, &abortf, a.status, W_U_PFULL);
            if (!ok) break;
            tc_fence_after_sync();
#pragma unroll
            for (int kk = 4 * half; kk < 4 * half + 4; ++kk)
              mma_ts_split(tDV, tPT + kk * 8, dob + koff_mnmajor(kk), hi, idesc_dv, (e > 0 || kk > 0) ? 1u : 0u);
            if (half == 0 && t >= 1) {
              // bar_pt_free of tile t also tells the compute warps that the dS^T buffer of tile t + 1 is free, i.e. that the
              // dK / dQ products and the dQ reduction of tile t - 1 are done with it (normally long before this point)
              ok = mbar_wait(smem_u32(&bar_ds_empty[(t + 1) & 1]), ((t - 1) >> 1) & 1, &abortf, a.status, W_U_DSEMPTY);
              if (!ok) break;
            }
            mma_commit(smem_u32(&bar_pt_free[half]));
          }
          if (!ok) break;
          mma_commit(smem_u32(&bar_ring_empty[stage]));   // one of two: dO of the stage is no longer read
          ++t;
          if (++stage == C::STAGES) stage = 0;
        }
        if (ok) mma_commit(smem_u32(&bar_acc_full));
      }
    } else if (warp == 2 && lane == 0 && n > 0) {
      // ------- dK / dQ issuer: per tile dK += dS^T Q and dQ_tile = dS K (A = dS^T from shared memory) -------
      const uint32_t idesc_dk = make_idesc_f16(kBf16, 0, 1, KD_TILE, HD);   // A = dS^T rows (keys) K-major, B = Q rows, MN-major
      const uint32_t idesc_dq = make_idesc_f16(kBf16, 1, 1, KD_TILE, HD);   // A = dS^T read MN-major (M = queries), B = K rows, MN-major
      const uint32_t tDK = tbase + C::TM_DK, tDQ = tbase + C::TM_DQ;
      const uint32_t hi = desc_hi_sw128();
      const uint32_t loRingMN = desc_lo_mnmajor(sRing);
      bool ok = true;
      int t = 0, stage = 0;
      int k_loads = 2;   // K tiles requested so far (the first two by the producer)
      for (int hh = 0; hh < nh && ok; ++hh) {
        const uint32_t loK = desc_lo_mnmajor(sK + (hh & 1) * C::TILE_BYTES);
        ok = mbar_wait(smem_u32(&bar_k_full[hh & 1]), (hh >> 1) & 1, &abortf, a.status, W_U_FIXFULL);
        if (!ok) break;
        if (hh > 0) {
          ok = mbar_wait(smem_u32(&bar_acc_free[1]), (hh - 1) & 1, &abortf, a.status, W_U_ACCFREE);
          if (!ok) break;
        }
        for (int e = 0; e < n && ok; ++e) {
          const int tb = t & 1;
          const uint32_t qb = loRingMN + stage * (2 * C::TILE_BYTES >> 4);
          const uint32_t dsK = desc_lo_kmajor(sDS + tb * (2 * C::TILE_BYTES));     // dS^T as [keys][queries]: K-major A of dK
          const uint32_t dsMN = desc_lo_mnmajor(sDS + tb * (2 * C::TILE_BYTES));   // the same bytes as MN-major A of dQ
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            ok = mbar_wait(smem_u32(&bar_p_full[half][t & 1]), (t >> 1) & 1, &abortf, a.status, W_U_PFULL);
            if (!ok) break;
            tc_fence_after_sync();
#pragma unroll
            for (int kk = 4 * half; kk < 4 * half + 4; ++kk)
              mma_ss_split(tDK, dsK + koff_kmajor(kk), qb + koff_mnmajor(kk), hi, idesc_dk, (e > 0 || kk > 0) ? 1u : 0u);
          }
          if (!ok) break;
          mma_commit(smem_u32(&bar_ring_empty[stage]));   // two of two: Q of the stage is no longer read
          if (t > 0) {   // the dQ warpgroup must have read the previous tile's dQ out of TMEM
            ok = mbar_wait(smem_u32(&bar_dq_empty), (t - 1) & 1, &abortf, a.status, W_U_DQEMPTY);
            if (!ok) break;
            tc_fence_after_sync();
          }
          mma_ss_split(tDQ, dsMN, loK, hi, idesc_dq, 0u);
#pragma unroll
          for (int kk = 1; kk < KD_TILE / 16; ++kk) mma_ss_split(tDQ, dsMN + koff_mnmajor(kk), loK + koff_mnmajor(kk), hi, idesc_dq, 1u);
          mma_commit(smem_u32(&bar_dq_full));   // issued after the dK product by the same thread: it covers both
          ++t;
          if (++stage == C::STAGES) stage = 0;
        }
        if (!ok) break;
        mma_commit(smem_u32(&bar_acc_full));
        mma_commit(smem_u32(&bar_k_empty[hh & 1]));   // the head's dQ products no longer read K
        if (hh + 2 < nh) {
          // The K of the head after next goes into this head's buffer: this thread waits for its own last products (it has
          // nothing to issue before the next tile's dS^T is written) and requests the tile, a whole head ahead of its use.
          ok = mbar_wait(smem_u32(&bar_k_empty[hh & 1]), (hh >> 1) & 1, &abortf, a.status, W_U_FIXEMPTY);
          if (!ok) break;
          mbar_arrive_expect_tx(smem_u32(&bar_k_full[hh & 1]), C::TILE_BYTES);
          tma_load_4d(sK + (hh & 1) * C::TILE_BYTES, &tmK, smem_u32(&bar_k_full[hh & 1]), 0, kt * KD_TILE, h0 + hh + 2, b);
          k_loads = hh + 3;
        }
      }
      // let copies in flight land before the CTA exits: the last two requests of this thread
      if (abortf.v != 0) {
        for (int f = max(2, k_loads - 2); f < k_loads; ++f) drain_wait(smem_u32(&bar_k_full[f & 1]), (f >> 1) & 1);
      }
    }
  } else if (warp < 20) {
    reg_alloc<C::REGS_COMPUTE>();
    // ------------------------------ compute warpgroups ------------------------------
    // warpgroup g handles queries 32 g .. 32 g + 31 of every tile, a key row per thread. Warpgroups 0 and 1 own the first half of
    // the tile's columns, 2 and 3 the second; the halves have their own barriers throughout, so the two pairs of warpgroups run
    // as independent pipelines that drift apart in time: one does arithmetic while the other waits, loads or stores.
    const int g = (warp - 4) >> 2;
    const int half = g >> 1;
    const int wq = warp & 3;
    const int row = wq * 32 + lane;
    const int kj = kt * KD_TILE + row;   // this thread's key
    const uint32_t lane_base = static_cast<uint32_t>(wq * 32) << 16;
    const float c = a.scale_log2;
    const uint32_t kdesc = a.desc[(size_t)b * a.Tpad + kj];
    // this thread's 64 bytes of its key's row in dS^T block g / 2: 16-byte chunks 4 (g % 2) .. + 3, swizzled with the row
    const uint32_t ds_row = static_cast<uint32_t>(half) * C::TILE_BYTES + static_cast<uint32_t>(row) * 128u;
    const uint32_t ds_sw = static_cast<uint32_t>(row & 7);
    bool ok = true;

    int stage = 0;
    int t = 0;   // tiles so far, over all heads
    const uint32_t tS = tbase + lane_base + C::TM_S + g * 32, tP = tbase + lane_base + C::TM_DP + g * 32;
    const uint32_t tPT = tbase + lane_base + C::TM_PT + g * 16;
    const uint32_t b_sfull = smem_u32(&bar_s_full[half]), b_spfree = smem_u32(&bar_sp_free[half]), b_pfull = smem_u32(&bar_p_full[half][0]),
                   b_ptfree = smem_u32(&bar_pt_free[half]);

    for (int hh = 0; hh < nh && ok; ++hh) {
      for (int e = 0; e < n; ++e) {
        const uint32_t ent = list[e];
        const uint32_t cls = ent >> 8;
        // The stage's scalars and mask words were written by the producer warp before its arrival on the stage's barrier;
        // the issuer of S^T waited for that barrier before the products whose completion is awaited here, so no separate
        // wait for the stage is taken.
        ok = mbar_wait(b_sfull, t & 1, &abortf, a.status, half ? W_U_SFULL1 : W_U_SFULL);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t* side = sSide + stage * C::SIDE_WORDS + g * 32;   // this warpgroup's 32 queries
        if (++stage == C::STAGES) stage = 0;
        uint32_t mk = 0xFFFFFFFFu;   // visibility of this key for the 32 queries
        if (cls == KD_TILE_PARTIAL) {
          const uint32_t* tbw = side - g * 32 + 3 * KD_TILE + g;   // word g of every query-side class mask
          const int i0 = (ent & 0xFF) * KD_TILE + g * 32;          // first query handled here
          key_row_mask<1>(kdesc, kj, i0, tbw + 4 * TB_SEES_PRE, tbw + 4 * TB_SEES_CTX, tbw + 4 * TB_SEES_INS, tbw + 4 * TB_CTX, &mk);
          if (tbw[4 * TB_SIDPOS] != 0u) {
            // "same span": lane L holds the descriptor of query number L of this warpgroup; one round per distinct span among
            // the warp's 32 keys, each a ballot over the queries
            const uint32_t qd_lane = side[2 * KD_TILE + lane];
            const uint32_t my_key = span_key_of_key(kdesc);
            uint32_t todo = __ballot_sync(0xffffffffu, (kdesc & TD_INS) != 0u);
            while (todo != 0u) {
              const uint32_t kk = __shfl_sync(0xffffffffu, my_key, __ffs(todo) - 1);
              const uint32_t hit = __ballot_sync(0xffffffffu, span_match_query(kk, qd_lane) != 0u);
              const bool mine = (my_key == kk);
              if (mine) mk |= hit;
              todo &= ~__ballot_sync(0xffffffffu, mine);
            }
          }
        }
        const int tb = t & 1;
        const uint32_t ds_base = sDS + tb * (2 * C::TILE_BYTES) + ds_row;
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {   // 16 queries at a time
          uint32_t pk_p[8], pk_ds[8];
          uint32_t rs[16], rp[16];
          tmem_ld16(tS + hf * 16, rs);
          tmem_ld16(tP + hf * 16, rp);
          tmem_wait_ld();
          if (hf == 1) {   // all of this warp's values are in registers: the next tile's S^T and dP^T may overwrite the half's columns
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(b_spfree);
          }
          const uint32_t mh = mk >> (hf * 16);
#pragma unroll
          for (int j = 0; j < 16; j += 4) {
            const float4 l4 = *reinterpret_cast<const float4*>(side + hf * 16 + j);             // LSE of 4 queries
            const float4 d4 = *reinterpret_cast<const float4*>(side + KD_TILE + hf * 16 + j);   // delta of 4 queries
            const float lw[4] = {l4.x, l4.y, l4.z, l4.w}, dw[4] = {d4.x, d4.y, d4.z, d4.w};
            float pv[4], ds[4];
#pragma unroll
            for (int u2 = 0; u2 < 4; ++u2) pv[u2] = fast_exp2(fmaf(__uint_as_float(rs[j + u2]), c, -lw[u2]));
            if (cls == KD_TILE_PARTIAL) {   // warp-uniform
#pragma unroll
              for (int u2 = 0; u2 < 4; ++u2)
                if ((mh & (1u << (j + u2))) == 0u) pv[u2] = 0.f;
            }
#pragma unroll
            for (int u2 = 0; u2 < 4; ++u2) ds[u2] = pv[u2] * (__uint_as_float(rp[j + u2]) - dw[u2]);
            pk_p[j / 2] = pack2<kBf16>(pv[0], pv[1]);
            pk_p[j / 2 + 1] = pack2<kBf16>(pv[2], pv[3]);
            pk_ds[j / 2] = pack2<kBf16>(ds[0], ds[1]);
            pk_ds[j / 2 + 1] = pack2<kBf16>(ds[2], ds[3]);
          }
          if (hf == 0 && t > 0) {
            // P^T and dS^T may leave the registers once the products that read their previous contents are done: the
            // previous tile's dV, and the dK / dQ / reduction of the tile before that. The dV issuer waits for the latter
            // itself before it signals the former, so one barrier stands for both.
            ok = mbar_wait(b_ptfree, (t - 1) & 1, &abortf, a.status, W_U_PTFREE);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after_sync();
          }
          tmem_st8(tPT + hf * 8, pk_p);
          const uint32_t ch = static_cast<uint32_t>(4 * (g & 1) + 2 * hf);
          st_shared_v4(ds_base + (((ch + 0u) ^ ds_sw) << 4), pk_ds[0], pk_ds[1], pk_ds[2], pk_ds[3]);
          st_shared_v4(ds_base + (((ch + 1u) ^ ds_sw) << 4), pk_ds[4], pk_ds[5], pk_ds[6], pk_ds[7]);
        }
        if (!ok) break;
        fence_proxy_async_smem();   // the dK and dQ products read these shared-memory writes through the async proxy
        tmem_wait_st();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(b_pfull + (t & 1) * 8);
        ++t;
      }
    }
  } else {
    reg_dealloc<C::REGS_DQ>();
    // ------------------------------ dQ warpgroup: TMEM -> shared memory -> bulk reduction into the fp32 scratch ------------------------------
    const int wq = warp & 3;
    const int row = wq * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(wq * 32) << 16;
    const uint32_t st_row = static_cast<uint32_t>(row) * 128u, st_sw = static_cast<uint32_t>(row & 7);
    const bool leader = (warp == 20 && lane == 0);
    if (leader) tma_prefetch_desc(&tmAcc);
    const uint32_t tDQ = tbase + lane_base + C::TM_DQ;
    bool ok = true;
    int t = 0;
    const int kj = kt * KD_TILE + row;   // this thread's key: it also writes that key's rows of dK and dV
    // dK and dV of head number hd leave through these warps as well (a whole 128-byte row per thread): the compute warps
    // go straight on to the next head's tiles, whose S^T / dP^T are already waiting, and the accumulating issuers wait for
    // bar_acc_free before they overwrite the accumulators.
    auto write_out = [&](int hd) -> bool {
      if (n > 0) {
        ok = mbar_wait(smem_u32(&bar_acc_full), hd & 1, &abortf, a.status, W_U_ACCFULL);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) return false;
        tc_fence_after_sync();
      }
      const int h = h0 + hd;
      uint16_t* krow = reinterpret_cast<uint16_t*>(a.dk) + (size_t)b * a.dk_sb + (size_t)h * a.dk_sh + (size_t)kj * a.dk_st;
      uint16_t* vrow = reinterpret_cast<uint16_t*>(a.dv) + (size_t)b * a.dv_sb + (size_t)h * a.dv_sh + (size_t)kj * a.dv_st;
#pragma unroll
      for (int part = 0; part < 4; ++part) {   // dV columns 0-31, 32-63, then dK: the next head's first dV product is the
                                               // one the compute warps wait for, so dV is released first
        uint32_t r[32];
        const bool is_k = part >= 2;
        if (n > 0) {
          tmem_ld32(tbase + lane_base + (is_k ? C::TM_DK : C::TM_DV) + (part & 1) * 32, r);
          tmem_wait_ld();
          if (part & 1) {   // the accumulator is in registers: the next head's first product may overwrite it
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bar_acc_free[is_k ? 1 : 0]));
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = 0u;
        }
        if (kj < a.T) store_row32_upto<kBf16>((is_k ? krow : vrow) + (part & 1) * 32, r, is_k ? a.sm_scale : 1.0f, (part & 1) * 32, a.d_real);
      }
      return true;
    };
    for (int hh = 0; hh < nh && ok; ++hh) {
      const int bh = b * a.H + h0 + hh;
      if (n == 0) write_out(hh);
      for (int e = 0; e < n; ++e) {
        const int tb = t & 1;
        const int q0 = (list[e] & 0xFF) * KD_TILE;
        ok = mbar_wait(smem_u32(&bar_dq_full), t & 1, &abortf, a.status, W_U_DQFULL);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after_sync();
        // The dQ product was the last reader of this tile's dS^T buffer (the dK product was issued before it by the same
        // thread): its 32 KB now stage the dQ tile as two [128 rows][32 floats] boxes in the 128-byte-swizzled layout the
        // tensor map expects.
        const uint32_t stage = sDS + tb * (2 * C::TILE_BYTES);
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          uint32_t r[32];
          tmem_ld32(tDQ + hf * 32, r);
          tmem_wait_ld();
          if (hf == 1) {
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bar_dq_empty));   // the next tile's dQ product may overwrite the TMEM columns
          }
#pragma unroll
          for (int cch = 0; cch < 8; ++cch)
            st_shared_v4(stage + hf * C::TILE_BYTES + st_row + ((static_cast<uint32_t>(cch) ^ st_sw) << 4), r[4 * cch], r[4 * cch + 1],
                         r[4 * cch + 2], r[4 * cch + 3]);
        }
        fence_proxy_async_smem();
        named_bar_sync(1, 128);
        if (leader) {
          tma_reduce_add_3d(&tmAcc, stage, 0, q0, bh);
          tma_reduce_add_3d(&tmAcc, stage + C::TILE_BYTES, 32, q0, bh);
          bulk_commit_group();
        }
        // after the head's last tile its dK and dV are complete (their last products were issued before the dQ product
        // this warpgroup has just consumed): they are written while the bulk reduction reads the staged tile
        if (e == n - 1 && !write_out(hh)) break;
        if (leader) {
          bulk_wait_group_read0();
          mbar_arrive(smem_u32(&bar_ds_empty[tb]));    // compute warps may write the tile after next's dS^T here
        }
        ++t;
      }
    }
    if (leader) bulk_wait_group0();
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tbase, 512);
}

// dq[b, h, t, :] = dq_acc[b, h, t, :] * sm_scale in the output dtype; 8 threads per row, 32 bytes in and 16 out each
template <bool kBf16>
__global__ void __launch_bounds__(256) attn_bwd_dq_convert_kernel(const BwdArgs a) {
  constexpr int HD = FusedCfg::HD, TPR = HD / 8;
  const size_t rows = (size_t)a.B * a.H * a.T;
  const int sub = threadIdx.x % TPR;
  for (size_t r = (size_t)blockIdx.x * (256 / TPR) + threadIdx.x / TPR; r < rows; r += (size_t)gridDim.x * (256 / TPR)) {
    const int t = static_cast<int>(r % a.T);
    const int h = static_cast<int>((r / a.T) % a.H);
    const int b = static_cast<int>(r / ((size_t)a.T * a.H));
    if (sub * 8 >= a.d_real) continue;
    const float4* src = reinterpret_cast<const float4*>(a.dq_acc + r * HD + sub * 8);
    const float4 x = src[0], y = src[1];
    uint4 v;
    v.x = pack2<kBf16>(x.x * a.sm_scale, x.y * a.sm_scale);
    v.y = pack2<kBf16>(x.z * a.sm_scale, x.w * a.sm_scale);
    v.z = pack2<kBf16>(y.x * a.sm_scale, y.y * a.sm_scale);
    v.w = pack2<kBf16>(y.z * a.sm_scale, y.w * a.sm_scale);
    *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(a.dq) + (size_t)b * a.dq_sb + (size_t)h * a.dq_sh + (size_t)t * a.dq_st + sub * 8) = v;
  }
}

template <bool kBf16>
static int launch_fused_t(const CUtensorMap& tmQ, const CUtensorMap& tmK, const CUtensorMap& tmV, const CUtensorMap& tmDO,
                          const BwdArgs& a, dim3 grid, cudaStream_t stream) {
  using C = FusedCfg;
  CUtensorMap tmAcc;
  int rc = encode_tensor_map_f32_rows(&tmAcc, a.dq_acc, a.B * a.H, a.T, C::HD, KD_TILE, "dq_acc");
  if (rc != 0) return rc;
  auto kern = attn_bwd_fused_kernel<kBf16>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_ALLOC);
  if (e != cudaSuccess) return set_error(KD_ERR_DEVICE, "fused bwd smem attribute: %s", cudaGetErrorString(e));
  // The warps re-divide the registers the CTA was launched with; a request beyond that pool would block for ever,
  // so a build whose per-thread count is below the one the division assumes is refused here.
  static int launch_regs = 0;
  if (launch_regs == 0) {
    cudaFuncAttributes fa;
    e = cudaFuncGetAttributes(&fa, kern);
    if (e != cudaSuccess) return set_error(KD_ERR_DEVICE, "fused bwd attributes: %s", cudaGetErrorString(e));
    launch_regs = fa.numRegs;
  }
  if (launch_regs < C::REGS_LAUNCH) return set_error(KD_ERR_DEVICE, "fused bwd was built with %d registers per thread, needs %d", launch_regs, C::REGS_LAUNCH);
  kern<<<grid, C::THREADS, C::SMEM_ALLOC, stream>>>(tmQ, tmK, tmV, tmDO, tmAcc, a);
  const size_t rows = (size_t)a.B * a.H * a.T;
  const int blocks = static_cast<int>(std::min<size_t>((rows + 31) / 32, size_t(148) * 32));
  attn_bwd_dq_convert_kernel<kBf16><<<blocks, 256, 0, stream>>>(a);
  e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(KD_ERR_DEVICE, "fused bwd kernels launch: %s", cudaGetErrorString(e));
  return 0;
}

int launch_bwd_fused(const CUtensorMap& tmQ, const CUtensorMap& tmK, const CUtensorMap& tmV, const CUtensorMap& tmDO,
                     const BwdArgs& a, int dtype, dim3 grid, cudaStream_t stream) {
  return dtype == KD_BF16 ? launch_fused_t<true>(tmQ, tmK, tmV, tmDO, a, grid, stream)
                          : launch_fused_t<false>(tmQ, tmK, tmV, tmDO, a, grid, stream);
}

}  // namespace kd
