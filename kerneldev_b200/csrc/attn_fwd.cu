// Forward kernel: O = softmax(mask(Q K^T * scale)) V and base-2 LSE, for sm_100a.
//
// One CTA owns a pair of 128-row query tiles of one (batch, head) and walks the plan's list of
// key tiles that are non-empty for either of them. Roles (warp-specialised, 384 threads):
//   warp 0      TMA producer: Q pair once, then K and V tiles through two rings
//   warp 1      P V issuer:   O_i += P V    (TMEM x smem -> TMEM)
//   warp 3      S issuer:     S = Q_i K^T   (smem x smem -> TMEM)
//   warp 2      builds the unit list and the issuers' per-unit commands in shared memory at start-up
//   warps 4-7   softmax of query tile 0: TMEM -> registers, rule on PARTIAL tiles, online
//   warps 8-11  softmax of query tile 1  softmax in base 2, P back to TMEM as 16-bit operand
//
// A "unit" is one (key tile, query tile) product that is not EMPTY. Units are numbered in list
// order; unit u computes its scores into TMEM buffer u % NBUF (128 fp32 columns), and P (64
// columns of packed pairs) is written over the same buffer. The S issuer runs NBUF units ahead of
// the P V issuer:   S(u + NBUF) is issued as soon as P(u) V has been issued,
// so a softmax warpgroup that finishes unit u finds the scores of its next unit already in
// TMEM, and the tensor core works on other units while it computes. The tensor pipe executes
// in issue order, which is what allows S(u + NBUF) to overwrite the buffer P(u) was read from.
// The two issuers are single threads that share their schedulers with the softmax warps, so
// everything they need per unit is precomputed into one 16-byte command each.
// EMPTY tiles never appear in the list: they are neither loaded nor multiplied.
//
// Replaces _flash_attn_fwd (original_kernel.py:278-626): same math (scores scaled by
// sm_scale*log2(e), exp2, LSE = m + log2(l)); rows without any visible key give O = 0 and
// LSE = -inf.
#include "attn_common.cuh"
#ifdef KD_TEST_DROP_LOAD
#include <stdlib.h>
#endif

namespace kd {

struct FwdArgs {
  int B, H, T, NT, NP, Tpad;
  int G;             // heads handled one after the other by a CTA (they share the pair's work list)
  int d_real;        // head dim of the tensors (a multiple of 16, <= HD); TMA zero-fills the tile columns beyond it
  float scale_log2;  // sm_scale * log2(e)
  const uint32_t* desc;
  const uint32_t* tilebits;   // [B][NT][8][4] class masks of every 128-token tile
  const int32_t* fwd_cnt;
  const uint16_t* fwd_list;
  const uint8_t* order;   // [B][3][NT]; row 0 = pairs sorted by decreasing list length
  uint32_t* status;
  void* o;
  int64_t o_sb, o_sh, o_st;
  float* lse;
#ifdef KD_TEST_DROP_LOAD
  int test_drop_load;   // wait time-out test build: the producer of CTA (0,0,0) leaves out its first K tile load
#endif
};

template <int HD>
struct FwdCfg {
  static constexpr int KBLK = HD / 64;                   // 64-element blocks along D
  static constexpr int TILE_BYTES = KD_TILE * HD * 2;    // one Q / K / V tile
  static constexpr int NBUF = (HD == 64) ? 3 : 2;        // score buffers in TMEM
  static constexpr int KST = NBUF;                       // K ring stages
  static constexpr int VST = (HD == 64) ? 3 : 2;         // V ring stages
  static constexpr int NQ = (HD == 64) ? 2 : 1;          // Q pair buffers: the next head's Q loads while this head computes
  static constexpr int SMEM_Q = 0;
  static constexpr int SMEM_K = SMEM_Q + NQ * 2 * TILE_BYTES;
  static constexpr int SMEM_V = SMEM_K + KST * TILE_BYTES;
  static constexpr int SMEM_LIST = SMEM_V + VST * TILE_BYTES;      // the pair's work list (<= 128 entries)
  static constexpr int SMEM_UNITS = SMEM_LIST + 128 * 2;           // unit list (<= 256 units)
  static constexpr int SMEM_CMD = SMEM_UNITS + 256 * 2;            // 256 x {S command, P V command} (uint4 each)
  static constexpr int SMEM_WCMD = SMEM_CMD + 256 * 2 * 16;        // 2 x 256 softmax commands (u32 each)
  static constexpr int SMEM_TOTAL = SMEM_WCMD + 2 * 256 * 4;
  static constexpr int SMEM_ALLOC = SMEM_TOTAL + 1024;   // slack for 1024-byte alignment
  static constexpr int CW = KD_TILE;                     // score columns per softmax thread: a whole row
  static constexpr int THREADS = 384;                    // four light warps + one softmax warpgroup per query tile
  static constexpr int REGS_COMPUTE = KD_REGS_COMPUTE;
  // TMEM columns: NBUF score buffers of 128, then O0 and O1 (HD each)
  static constexpr uint32_t TM_O0 = NBUF * 128, TM_O1 = NBUF * 128 + HD;
  static_assert(TM_O1 + HD <= 512, "TMEM budget");
  static_assert(SMEM_ALLOC <= 232448, "shared memory budget");
};

// unit descriptor: entry index (7 bits) | query tile of the pair << 7 | tile class << 8
__device__ __forceinline__ int unit_entry(uint32_t u) { return u & 0x7F; }
__device__ __forceinline__ int unit_tile(uint32_t u) { return (u >> 7) & 1; }
__device__ __forceinline__ uint32_t unit_class(uint32_t u) { return (u >> 8) & 3; }

// command flags (word z of a command)
constexpr uint32_t CMD_WAIT = 8u, CMD_RELEASE = 16u, CMD_ACC = 32u, CMD_TILE1 = 64u;
// softmax command of a warpgroup's k-th unit: key tile | class << 8 | (unit index mod NBUF) << 10
__device__ __forceinline__ int wcmd_kt(uint32_t c) { return c & 0xFF; }
__device__ __forceinline__ uint32_t wcmd_class(uint32_t c) { return (c >> 8) & 3; }
__device__ __forceinline__ int wcmd_buf(uint32_t c) { return (c >> 10) & 3; }

// wait-site codes reported in the status word
enum : uint32_t {
  W_F_QFULL = 0x101, W_F_KEMPTY = 0x102, W_F_VEMPTY = 0x103, W_F_KFULL = 0x104, W_F_VFULL = 0x105,
  W_F_PFULL = 0x106, W_F_SFULL = 0x107, W_F_PVDONE = 0x108, W_F_PVISSUED = 0x109, W_F_QEMPTY = 0x10A, W_F_OFREE = 0x10B,
};

template <int HD, bool kBf16>
__global__ void __launch_bounds__(FwdCfg<HD>::THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const FwdArgs a) {
  using C = FwdCfg<HD>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sQ = smem_u32(smem + C::SMEM_Q);
  const uint32_t sK = smem_u32(smem + C::SMEM_K);
  const uint32_t sV = smem_u32(smem + C::SMEM_V);
  uint16_t* sList = reinterpret_cast<uint16_t*>(smem + C::SMEM_LIST);
  uint16_t* sUnits = reinterpret_cast<uint16_t*>(smem + C::SMEM_UNITS);
  uint4* sCmd = reinterpret_cast<uint4*>(smem + C::SMEM_CMD);   // [u][0] = S command, [u][1] = P V command
  uint32_t* sWcmd = reinterpret_cast<uint32_t*>(smem + C::SMEM_WCMD);   // [tile][k]

  __shared__ __align__(8) uint64_t bar_q_full[C::NQ], bar_q_empty[C::NQ], bar_k_full[C::KST], bar_k_empty[C::KST],
      bar_v_full[C::VST], bar_v_empty[C::VST], bar_s_full[2 * C::NBUF], bar_p_full[C::NBUF], bar_pv_issued[C::NBUF],
      bar_pv_done[2], bar_o_free[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ int n_units_s, n_own_s[2];
  __shared__ AbortFlag abortf;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // blockIdx.z walks the pairs from the longest list to the shortest, so the CTAs that take
  // longest are dispatched first
  const int h0 = blockIdx.x * a.G, b = blockIdx.y;
  const int nh = min(a.G, a.H - h0);   // this CTA handles heads h0 .. h0 + nh - 1, one after the other
  const int pair = a.order[((size_t)b * 3 + 0) * a.NT + blockIdx.z];
  const int n = a.fwd_cnt[b * a.NP + pair];

  if (tid == 0) {
    abortf.v = 0;
    for (int s = 0; s < C::NQ; ++s) {
      mbar_init(smem_u32(&bar_q_full[s]), 1);
      mbar_init(smem_u32(&bar_q_empty[s]), 1);
    }
    for (int s = 0; s < C::KST; ++s) {
      mbar_init(smem_u32(&bar_k_full[s]), 1);
      mbar_init(smem_u32(&bar_k_empty[s]), 1);
    }
    for (int s = 0; s < C::VST; ++s) {
      mbar_init(smem_u32(&bar_v_full[s]), 1);
      mbar_init(smem_u32(&bar_v_empty[s]), 1);
    }
    for (int s = 0; s < C::NBUF; ++s) {
      // one "scores ready" barrier per (buffer, query tile): each softmax warpgroup then sees every
      // phase of the barriers it waits on, which is what makes a parity wait sound
      mbar_init(smem_u32(&bar_s_full[2 * s]), 1);
      mbar_init(smem_u32(&bar_s_full[2 * s + 1]), 1);
      mbar_init(smem_u32(&bar_p_full[s]), 4);   // one arrival per softmax warp (lane 0, after a warp-wide sync)
      mbar_init(smem_u32(&bar_pv_issued[s]), 1);
    }
    mbar_init(smem_u32(&bar_pv_done[0]), 1);
    mbar_init(smem_u32(&bar_pv_done[1]), 1);
    mbar_init(smem_u32(&bar_o_free[0]), 4);
    mbar_init(smem_u32(&bar_o_free[1]), 4);
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&tmem_base_s), 512);
    tmem_relinquish();
  }
  if (warp == 2) {
    // stage the pair's list and expand it into units (one per non-empty (key tile, query tile))
    const uint16_t* glist = a.fwd_list + ((size_t)b * a.NP + pair) * a.NT;
    int nu = 0;
    for (int base = 0; base < n; base += 32) {
      const int e = base + lane;
      const uint32_t ent = e < n ? glist[e] : 0u;
      if (e < n) sList[e] = static_cast<uint16_t>(ent);
      const uint32_t c0 = (ent >> 8) & 3u, c1 = (ent >> 10) & 3u;
      const int cnt = (c0 != 0u) + (c1 != 0u);
      int incl = cnt;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
      }
      int pos = nu + incl - cnt;
      if (c0) sUnits[pos++] = static_cast<uint16_t>(e | (0 << 7) | (c0 << 8));
      if (c1) sUnits[pos++] = static_cast<uint16_t>(e | (1 << 7) | (c1 << 8));
      nu += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) n_units_s = nu;
    __syncwarp();
    // per-unit commands for the two issuers and for the softmax warpgroups
    const uint32_t loQ0 = desc_lo_kmajor(sQ), loK0 = desc_lo_kmajor(sK), loV0 = desc_lo_mnmajor(sV);
    int cnt_key[2 * C::NBUF];   // units seen so far per (buffer, tile)
#pragma unroll
    for (int j = 0; j < 2 * C::NBUF; ++j) cnt_key[j] = 0;
    const uint32_t lt_mask = (1u << lane) - 1u;
    for (int base = 0; base < nu; base += 32) {
      const int u = base + lane;
      const bool valid = u < nu;
      const uint32_t un = valid ? sUnits[u] : 0u;
      const int e = unit_entry(un), i = unit_tile(un), buf = u % C::NBUF, key = 2 * buf + i;
      // rank of this unit among the units of its query tile (counts still exclude this chunk)
      int rank_tile = 0;
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        const uint32_t bal = __ballot_sync(0xffffffffu, valid && i == t);
        int before = 0;
#pragma unroll
        for (int j = 0; j < C::NBUF; ++j) before += cnt_key[2 * j + t];
        if (i == t) rank_tile = before + __popc(bal & lt_mask);
      }
      // rank among the units that share its (buffer, tile) barrier; then add this chunk to the counts
      int rank_key = 0;
#pragma unroll
      for (int j = 0; j < 2 * C::NBUF; ++j) {
        const uint32_t bal = __ballot_sync(0xffffffffu, valid && key == j);
        if (key == j) rank_key = cnt_key[j] + __popc(bal & lt_mask);
        cnt_key[j] += __popc(bal);
      }
      if (valid) {
        const bool first_of_entry = (u == 0) || unit_entry(sUnits[u - 1]) != e;
        const bool last_of_entry = (u + 1 >= nu) || unit_entry(sUnits[u + 1]) != e;
        uint4 cs, cp;
        // ring stages and barrier parities run on across heads, so the issuers keep them in counters;
        // the commands carry what is the same for every head
        cs.x = loQ0 + i * (C::TILE_BYTES >> 4);
        cs.y = loK0;
        cs.z = (first_of_entry ? CMD_WAIT : 0u) | (last_of_entry ? CMD_RELEASE : 0u) | (i ? CMD_TILE1 : 0u);
        cs.w = 0u;
        cp.x = 0u;
        cp.y = loV0;
        cp.z = (first_of_entry ? CMD_WAIT : 0u) | (last_of_entry ? CMD_RELEASE : 0u) | (rank_tile == 0 ? 0u : CMD_ACC) |
               (i ? CMD_TILE1 : 0u);
        cp.w = 0u;
        sCmd[2 * u] = cs;
        sCmd[2 * u + 1] = cp;
        sWcmd[i * 256 + rank_tile] = (sList[e] & 0xFFu) | (unit_class(un) << 8) | (static_cast<uint32_t>(buf) << 10);
        (void)rank_key;
      }
    }
    if (lane == 0) {
      int t0 = 0, t1 = 0;
#pragma unroll
      for (int j = 0; j < C::NBUF; ++j) { t0 += cnt_key[2 * j]; t1 += cnt_key[2 * j + 1]; }
      n_own_s[0] = t0;
      n_own_s[1] = t1;
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tbase = tmem_base_s;
  const int U = n_units_s;

  if (warp < 4) {
    reg_dealloc<KD_REGS_ISSUE>();
    if (warp == 0 && lane == 0 && n > 0) {
      // ------------------------------ TMA producer ------------------------------
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      const int ntile_q = (2 * pair + 1 < a.NT) ? 2 : 1;
      bool ok = true;
      auto load_q = [&](int hh) -> bool {   // Q pair of head h0 + hh into buffer hh % NQ
        const int qb = hh % C::NQ, qround = hh / C::NQ;
        if (qround > 0 && !mbar_wait(smem_u32(&bar_q_empty[qb]), (qround - 1) & 1, &abortf, a.status, W_F_QEMPTY)) return false;
        mbar_arrive_expect_tx(smem_u32(&bar_q_full[qb]), ntile_q * C::TILE_BYTES);
        for (int t = 0; t < ntile_q; ++t)
          for (int kb = 0; kb < C::KBLK; ++kb)
            tma_load_4d(sQ + (qb * 2 + t) * C::TILE_BYTES + kb * 16384, &tmQ, smem_u32(&bar_q_full[qb]), kb * 64,
                        (2 * pair + t) * KD_TILE, h0 + hh, b);
        return true;
      };
      int k_cnt = 0, v_cnt = 0, q_loaded = 0;   // tiles issued so far, over all heads
      int k_dropped = -1;                       // index of a K tile that was never requested (test builds only)
      ok = load_q(0);
      q_loaded = 1;
      for (int hh = 0; hh < nh && ok; ++hh) {
        if (C::NQ > 1 && hh + 1 < nh) {       // next head's Q lands while this head runs
          ok = load_q(hh + 1);
          q_loaded = hh + 2;
          if (!ok) break;
        }
        for (int e = 0; e < n && ok; ++e) {
          const int kt = sList[e] & 0xFF;
#ifdef KD_TEST_DROP_LOAD
          // Test build only: this one K tile is never requested (no copy, no expected bytes), so the S issuer's
          // bounded wait for it runs out and the CTA has to unwind. Nothing is left in flight for the stage.
          if (a.test_drop_load && hh == 0 && e == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) {
            k_dropped = k_cnt++;
          } else
#endif
          {
            const int s = k_cnt % C::KST;
            ok = mbar_wait(smem_u32(&bar_k_empty[s]), ((k_cnt / C::KST) & 1) ^ 1, &abortf, a.status, W_F_KEMPTY);
            if (!ok) break;
            mbar_arrive_expect_tx(smem_u32(&bar_k_full[s]), C::TILE_BYTES);
            for (int kb = 0; kb < C::KBLK; ++kb)
              tma_load_4d(sK + s * C::TILE_BYTES + kb * 16384, &tmK, smem_u32(&bar_k_full[s]), kb * 64, kt * KD_TILE, h0 + hh, b);
            ++k_cnt;
          }
          {
            const int s = v_cnt % C::VST;
            ok = mbar_wait(smem_u32(&bar_v_empty[s]), ((v_cnt / C::VST) & 1) ^ 1, &abortf, a.status, W_F_VEMPTY);
            if (!ok) break;
            mbar_arrive_expect_tx(smem_u32(&bar_v_full[s]), C::TILE_BYTES);
            for (int kb = 0; kb < C::KBLK; ++kb)
              tma_load_4d(sV + s * C::TILE_BYTES + kb * 16384, &tmV, smem_u32(&bar_v_full[s]), kb * 64, kt * KD_TILE, h0 + hh, b);
            ++v_cnt;
          }
        }
        if (C::NQ == 1 && hh + 1 < nh && ok) {
          ok = load_q(hh + 1);
          q_loaded = hh + 2;
        }
      }
      if (abortf.v != 0) {
        // unwinding: let every copy already in flight land (bounded) before the CTA exits
        for (int e = max(0, k_cnt - C::KST); e < k_cnt; ++e)
          if (e != k_dropped) drain_wait(smem_u32(&bar_k_full[e % C::KST]), (e / C::KST) & 1);
        for (int e = max(0, v_cnt - C::VST); e < v_cnt; ++e) drain_wait(smem_u32(&bar_v_full[e % C::VST]), (e / C::VST) & 1);
        for (int hh = max(0, q_loaded - C::NQ); hh < q_loaded; ++hh) drain_wait(smem_u32(&bar_q_full[hh % C::NQ]), (hh / C::NQ) & 1);
      }
    } else if (warp == 3 && lane == 0 && U > 0) {
      // ------------------------------ S issuer ------------------------------
      const uint32_t idesc_s = make_idesc_f16(kBf16, 0, 0, KD_TILE, KD_TILE);
      const uint32_t hi = desc_hi_sw128();
      bool ok = true;
      int buf = 0, round = 0;      // the g-th unit over all heads uses buffer g % NBUF in round g / NBUF
      int kstage = 0;
      uint32_t kparity = 0;
      for (int hh = 0; hh < nh && ok; ++hh) {
        const int qb = hh % C::NQ;
        ok = mbar_wait(smem_u32(&bar_q_full[qb]), (hh / C::NQ) & 1, &abortf, a.status, W_F_QFULL);
        const uint32_t q_off = qb * (2 * C::TILE_BYTES >> 4);
        for (int u = 0; u < U && ok; ++u) {
          const uint4 c = sCmd[2 * u];
          // operands of the unit, formed ahead of the waits
          const uint32_t d = tbase + buf * 128;
          const uint32_t qlo = c.x + q_off, klo = c.y + kstage * (C::TILE_BYTES >> 4);
          uint64_t qdesc[HD / 16], kdesc[HD / 16];
#pragma unroll
          for (int kk = 0; kk < HD / 16; ++kk) {
            qdesc[kk] = desc64(qlo + koff_kmajor(kk), hi);
            kdesc[kk] = desc64(klo + koff_kmajor(kk), hi);
          }
          if (round > 0) {
            // the buffer is free once P V of the unit that used it in the previous round has been issued
            ok = mbar_wait(smem_u32(&bar_pv_issued[buf]), (round - 1) & 1, &abortf, a.status, W_F_PVISSUED);
            if (!ok) break;
          }
          if (c.z & CMD_WAIT) {
            ok = mbar_wait(smem_u32(&bar_k_full[kstage]), kparity, &abortf, a.status, W_F_KFULL);
            if (!ok) break;
          }
          tc_fence_after_sync();
          mma_ss64<false>(d, qdesc[0], kdesc[0], idesc_s);
#pragma unroll
          for (int kk = 1; kk < HD / 16; ++kk) mma_ss64<true>(d, qdesc[kk], kdesc[kk], idesc_s);
          mma_commit(smem_u32(&bar_s_full[2 * buf + ((c.z & CMD_TILE1) ? 1 : 0)]));
          if (c.z & CMD_RELEASE) {
            mma_commit(smem_u32(&bar_k_empty[kstage]));
            if (++kstage == C::KST) { kstage = 0; kparity ^= 1; }
          }
          if (++buf == C::NBUF) {
            buf = 0;
            ++round;
          }
        }
        if (ok) mma_commit(smem_u32(&bar_q_empty[qb]));   // Q of this head is no longer read once the MMAs above are done
      }
    } else if (warp == 1 && lane == 0 && U > 0) {
      // ------------------------------ P V issuer ------------------------------
      const uint32_t idesc_o = make_idesc_f16(kBf16, 0, 1, KD_TILE, HD);
      const uint32_t hi = desc_hi_sw128();
      bool ok = true;
      int buf = 0, vstage = 0;
      uint32_t round_parity = 0, vparity = 0;
      for (int hh = 0; hh < nh && ok; ++hh) {
        for (int u = 0; u < U && ok; ++u) {
          const uint4 c = sCmd[2 * u + 1];
          // operands of the unit, formed ahead of the waits
          const uint32_t vlo = c.y + vstage * (C::TILE_BYTES >> 4);
          const uint32_t aP = tbase + buf * 128;
          uint64_t vdesc[KD_TILE / 16];
          uint32_t pop[KD_TILE / 16];
#pragma unroll
          for (int kk = 0; kk < KD_TILE / 16; ++kk) {
            vdesc[kk] = desc64(vlo + koff_mnmajor(kk), hi);
            pop[kk] = aP + kk * 8;   // P of 16 keys = 8 packed columns at the start of the score buffer
          }
          ok = mbar_wait(smem_u32(&bar_p_full[buf]), round_parity, &abortf, a.status, W_F_PFULL);
          if (!ok) break;
          if (c.z & CMD_WAIT) {
            ok = mbar_wait(smem_u32(&bar_v_full[vstage]), vparity, &abortf, a.status, W_F_VFULL);
            if (!ok) break;
          }
          const uint32_t i = (c.z & CMD_TILE1) ? 1u : 0u;
          const uint32_t acc0 = (c.z & CMD_ACC) ? 1u : 0u;
          if (acc0 == 0u && hh > 0) {
            // first product of this query tile for a new head overwrites O_i: the softmax warpgroup must
            // have read the previous head's result out of it
            ok = mbar_wait(smem_u32(&bar_o_free[i]), (hh - 1) & 1, &abortf, a.status, W_F_OFREE);
            if (!ok) break;
          }
          tc_fence_after_sync();
          const uint32_t dO = tbase + C::TM_O0 + i * HD;
          mma_ts64_p(dO, pop[0], vdesc[0], idesc_o, acc0);
#pragma unroll
          for (int kk = 1; kk < KD_TILE / 16; ++kk) mma_ts64<true>(dO, pop[kk], vdesc[kk], idesc_o);
          mma_commit(smem_u32(&bar_pv_done[i]));
          if (c.z & CMD_RELEASE) {
            mma_commit(smem_u32(&bar_v_empty[vstage]));
            if (++vstage == C::VST) { vstage = 0; vparity ^= 1; }
          }
          // hand the buffer back to the S issuer, ordered after the MMAs above
          tc_fence_before_sync();
          mbar_arrive(smem_u32(&bar_pv_issued[buf]));
          if (++buf == C::NBUF) {
            buf = 0;
            round_parity ^= 1;
          }
        }
      }
    }
  } else {
    reg_alloc<C::REGS_COMPUTE>();
    // ------------------------------ softmax warpgroups ------------------------------
    // One warpgroup per query tile; each thread owns one row of 128 scores.
    constexpr int CW = C::CW, NW = CW / 32;
    const int i = (warp - 4) >> 2;        // warpgroup = query tile of the pair
    const int wq = warp & 3;              // TMEM lane quadrant of this warp
    const int row = wq * 32 + lane;       // row inside the tile
    const int qtile = 2 * pair + i;
    const int qi = qtile * KD_TILE + row;  // token index of this thread's query
    const bool tile_valid = qtile < a.NT;
    const uint32_t lane_base = static_cast<uint32_t>(wq * 32) << 16;
    const uint32_t tO = tbase + lane_base + (i == 0 ? C::TM_O0 : C::TM_O1);   // this thread's row of O
    const float c = a.scale_log2;

    const uint32_t qd = tile_valid ? a.desc[(size_t)b * a.Tpad + qi] : 0u;
    bool ok = true;

    // Key descriptors (lane L holds keys L, 32 + L, ...) and class masks of PARTIAL tiles are fetched one unit ahead
    // into registers, so their global-memory latency overlaps the previous tile's softmax.
    const int n_own = n_own_s[i];
    const uint32_t* wcmd = sWcmd + i * 256;
    uint32_t kd_pre[NW];
    uint32_t tb_pre[3][NW];   // key-side class masks of this thread's columns: is_prefix, context, in_span
#pragma unroll
    for (int w = 0; w < NW; ++w) { kd_pre[w] = 0u; tb_pre[0][w] = 0u; tb_pre[1][w] = 0u; tb_pre[2][w] = 0u; }
    auto prefetch_kd = [&](uint32_t cmd) {
      if (wcmd_class(cmd) == KD_TILE_PARTIAL) {
        const uint32_t* src = a.desc + (size_t)b * a.Tpad + (size_t)wcmd_kt(cmd) * KD_TILE;
        const uint4* tbp = reinterpret_cast<const uint4*>(a.tilebits + ((size_t)b * a.NT + wcmd_kt(cmd)) * 32);
#pragma unroll
        for (int w = 0; w < NW; ++w) kd_pre[w] = src[w * 32 + lane];
        static_assert(NW == 4, "a class mask of a tile is four words: one 16-byte load each");
        constexpr int cls3[3] = {TB_PRE, TB_CTX, TB_INS};
#pragma unroll
        for (int k3 = 0; k3 < 3; ++k3) {
          const uint4 m4 = tbp[cls3[k3]];
          tb_pre[k3][0] = m4.x; tb_pre[k3][1] = m4.y; tb_pre[k3][2] = m4.z; tb_pre[k3][3] = m4.w;
        }
      }
    };
    uint32_t cmd_next = n_own > 0 ? wcmd[0] : 0u;
    if (n_own > 0) prefetch_kd(cmd_next);
    // state that runs on across the heads of this CTA
    int buf_off = 0;            // (units of the heads done so far) mod NBUF: rotation of the buffers
    uint32_t sfull_par = 0;     // bit j: parity of the next phase of this tile's score barrier on buffer j
    int pv_seen = 0;            // P V products of this query tile issued so far (phases of bar_pv_done[i])

    for (int hh = 0; hh < nh && ok; ++hh) {
    const int h = h0 + hh;
    float m = -INFINITY, l = 0.f;
    int nact = 0;
    for (int k = 0; k < n_own; ++k) {
      const uint32_t cmd = cmd_next;
      const uint32_t cls = wcmd_class(cmd);
      const int kt = wcmd_kt(cmd);
      int buf = wcmd_buf(cmd) + buf_off;
      if (buf >= C::NBUF) buf -= C::NBUF;
      const uint32_t tS = tbase + lane_base + buf * 128;
      ok = mbar_wait(smem_u32(&bar_s_full[2 * buf + i]), (sfull_par >> buf) & 1u, &abortf, a.status, W_F_SFULL);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      sfull_par ^= 1u << buf;
      tc_fence_after_sync();

      float sc[CW];
#pragma unroll
      for (int cb = 0; cb < NW; ++cb) {
        uint32_t r[32];
        tmem_ld32(tS + cb * 32, r);
#pragma unroll
        for (int j = 0; j < 32; ++j) sc[cb * 32 + j] = __uint_as_float(r[j]);
      }
      tmem_wait_ld();
      if (cls == KD_TILE_PARTIAL) {
        // The row's visibility mask comes from the tile's class masks with a few word-wide
        // operations; only the "same span" term needs the individual key descriptors.
        const int j0 = kt * KD_TILE;
        uint32_t mk[NW];
        query_row_mask<NW>(qd, qi, j0, tb_pre[0], tb_pre[1], tb_pre[2], mk);
        uint32_t any_ins = 0u;
#pragma unroll
        for (int w = 0; w < NW; ++w) any_ins |= tb_pre[2][w];
        // "same span": one round per distinct span among the warp's 32 queries; a ballot over the lanes' key descriptors
        // gives the keys of that span, 32 at a time
        const uint32_t my_key = span_key_of_query(qd);
        uint32_t todo = (any_ins != 0u) ? __ballot_sync(0xffffffffu, (qd & TD_SIDPOS) != 0u) : 0u;
        while (todo != 0u) {
          const uint32_t kq = __shfl_sync(0xffffffffu, my_key, __ffs(todo) - 1);
          const bool mine = (my_key == kq);
#pragma unroll
          for (int w = 0; w < NW; ++w) {
            const uint32_t hit = __ballot_sync(0xffffffffu, span_match_key(kq, kd_pre[w]) != 0u);
            if (mine) mk[w] |= hit;
          }
          todo &= ~__ballot_sync(0xffffffffu, mine);
        }
#pragma unroll
        for (int w = 0; w < NW; ++w) {
          if (__all_sync(0xffffffffu, mk[w] == 0xFFFFFFFFu)) continue;   // all 32 keys visible to all 32 queries
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if ((mk[w] & (1u << j)) == 0u) sc[w * 32 + j] = -INFINITY;
        }
      }
      if (k + 1 < n_own || hh + 1 < nh) {   // the next head walks the same list again
        cmd_next = wcmd[k + 1 < n_own ? k + 1 : 0];
        prefetch_kd(cmd_next);
      }
      // four independent chains for the row maximum and for the row sum: a single chain of
      // dependent operations would be latency-bound
      float mx4[4] = {sc[0], sc[1], sc[2], sc[3]};
#pragma unroll
      for (int j = 4; j + 8 <= CW; j += 8) {   // three-input maximum: two new scores per instruction
        mx4[0] = fmax3(mx4[0], sc[j + 0], sc[j + 4]);
        mx4[1] = fmax3(mx4[1], sc[j + 1], sc[j + 5]);
        mx4[2] = fmax3(mx4[2], sc[j + 2], sc[j + 6]);
        mx4[3] = fmax3(mx4[3], sc[j + 3], sc[j + 7]);
      }
#pragma unroll
      for (int k4 = 0; k4 < 4; ++k4) mx4[k4] = fmaxf(mx4[k4], sc[CW - 4 + k4]);
      float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      // The running maximum is refreshed only when it would grow by more than 2^8 in the
      // exponent; until then the stale value is used consistently for P, l and O, which leaves
      // the normalised result unchanged and skips most O rescales.
      float m_new = m;
      if (m == -INFINITY || (mx - m) * c > 8.0f) m_new = fmaxf(m, mx);
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      const float alpha = (m == -INFINITY) ? 0.f : fast_exp2((m - m_new) * c);
      const bool need_rescale = (nact > 0) && (m_new != m);
      const float neg_mc = -m_use * c;
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
      uint32_t pk[CW / 2];
#pragma unroll
      for (int j = 0; j < CW; j += 4) {
        const float p0 = fast_exp2(fmaf(sc[j], c, neg_mc));
        const float p1 = fast_exp2(fmaf(sc[j + 1], c, neg_mc));
        const float p2 = fast_exp2(fmaf(sc[j + 2], c, neg_mc));
        const float p3 = fast_exp2(fmaf(sc[j + 3], c, neg_mc));
        sum4[0] += p0;
        sum4[1] += p1;
        sum4[2] += p2;
        sum4[3] += p3;
        pk[j / 2] = pack2<kBf16>(p0, p1);
        pk[j / 2 + 1] = pack2<kBf16>(p2, p3);
      }
      const float sum = (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
      l = l * alpha + sum;
      m = m_new;
#pragma unroll
      for (int cb = 0; cb < CW / 64; ++cb) {
        uint32_t r[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) r[j] = pk[cb * 32 + j];
        tmem_st32(tS + cb * 32, r);   // P over the start of this thread's own score columns
      }
      if (nact > 0) {
        // O_i may be touched only after the previous P V product of this query tile has completed;
        // the wait is taken for every unit so that no phase of the barrier goes unobserved
        ok = mbar_wait(smem_u32(&bar_pv_done[i]), (pv_seen - 1) & 1, &abortf, a.status, W_F_PVDONE);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
      if (__any_sync(0xffffffffu, need_rescale)) {
        tc_fence_after_sync();
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
      tmem_wait_st();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bar_p_full[buf]));
      ++nact;
      ++pv_seen;
    }
    if (!ok) break;
    buf_off += U % C::NBUF;
    if (buf_off >= C::NBUF) buf_off -= C::NBUF;

    // epilogue of this head: normalise, convert, store this thread's share of O, and LSE
    if (nact > 0) {
      ok = mbar_wait(smem_u32(&bar_pv_done[i]), (pv_seen - 1) & 1, &abortf, a.status, W_F_PVDONE);
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
        if (cb == HD / 32 - 1 && nact > 0) {
          // this thread's share of O_i has been read out: the next head's first product may overwrite it
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&bar_o_free[i]));
        }
        if (tile_valid && qi < a.T) store_row32_upto<kBf16>(orow + cb * 32, r, inv_l, cb * 32, a.d_real);
      }
    }
    }  // heads
  }

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
  a.d_real = p.D;
  a.scale_log2 = p.sm_scale * 1.4426950408889634f;
  a.G = heads_per_cta(p.B, p.H, L.NP, p.heads_per_cta, 3, 4);
  a.desc = pv.desc; a.fwd_cnt = pv.fwd_cnt; a.fwd_list = pv.fwd_list; a.status = pv.status;
  a.order = pv.order; a.tilebits = pv.tilebits;
  a.o = p.o.ptr; a.o_sb = p.o.stride_b; a.o_sh = p.o.stride_h; a.o_st = p.o.stride_t;
  a.lse = p.lse;
#ifdef KD_TEST_DROP_LOAD
  const char* drop = getenv("KD_TEST_DROP_LOAD");
  a.test_drop_load = (drop != nullptr && atoi(drop) != 0) ? 1 : 0;
#endif
  auto kern = attn_fwd_kernel<HD, kBf16>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_ALLOC);
  if (e != cudaSuccess) return set_error(KD_ERR_DEVICE, "fwd smem attribute: %s", cudaGetErrorString(e));
  dim3 grid((p.H + a.G - 1) / a.G, p.B, L.NP);
  kern<<<grid, C::THREADS, C::SMEM_ALLOC, stream>>>(tmQ, tmK, tmV, a);
  e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(KD_ERR_DEVICE, "attn_fwd_kernel launch: %s", cudaGetErrorString(e));
  return 0;
}

int launch_attn_fwd(const kd_attn_params& p, cudaStream_t stream) {
  kd_plan_layout L;
  if (kd_plan_layout_get(p.B, p.T, &L) != 0) return KD_ERR_ARG;
  PlanView pv = make_plan_view(const_cast<void*>(p.plan), L);
  // head dims below the tile width run on the next wider instantiation: TMA zero-fills the missing columns
  if (p.D <= 64) return p.dtype == KD_BF16 ? launch_fwd_t<64, true>(p, L, pv, stream) : launch_fwd_t<64, false>(p, L, pv, stream);
  return p.dtype == KD_BF16 ? launch_fwd_t<128, true>(p, L, pv, stream) : launch_fwd_t<128, false>(p, L, pv, stream);
}

}  // namespace kd
