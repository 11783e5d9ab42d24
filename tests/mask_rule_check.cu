// Host-side check of the bit-parallel form of the visibility rule (mask_rule.cuh) against its
// per-element form, on random descriptors that include overlapping flags and arbitrary span ids.
// Built and run by tests/test_host_logic.py (host code only; no GPU needed).
#include <cstdio>
#include <cstdint>
#include <cstdlib>
#include "../kerneldev_b200/csrc/mask_rule.cuh"

using namespace kd;

static uint32_t rng_state = 12345u;
static uint32_t rnd() { rng_state = rng_state * 1664525u + 1013904223u; return rng_state >> 8; }

static void class_masks(const uint32_t* d, int n, uint32_t bit, uint32_t* out) {
  for (int w = 0; w < n / 32; ++w) {
    out[w] = 0;
    for (int t = 0; t < 32; ++t) if (d[w * 32 + t] & bit) out[w] |= 1u << t;
  }
}

int main() {
  long long bad = 0, checked = 0;
  for (int trial = 0; trial < 200; ++trial) {
    uint32_t q[128], k[128];
    const int mode = trial % 4;
    for (int t = 0; t < 128; ++t) {
      for (int side = 0; side < 2; ++side) {
        bool ins = (rnd() % 100) < 35, pre = (rnd() % 100) < 25;
        long long sid = (long long)(rnd() % 6) - 1;              // -1 .. 4
        bool alive = (rnd() % 100) < 92;
        if (mode == 1) { ins = t >= 40 && t < 100; pre = t < 10; sid = ins ? 1 + t / 30 : (t == 100 ? -1 : 0); }  // canonical-like runs
        if (mode == 2) { ins = true; pre = false; sid = 1 + (t / 16); }                                           // all spans
        (side ? k : q)[t] = pack_token(ins, pre, sid, alive);
      }
    }
    const int i_base = (int)(rnd() % 4) * 128, j_base = (int)(rnd() % 4) * 128;
    uint32_t kp[4], kc[4], ki[4], qsp[4], qsc[4], qsi[4], qc[4];
    class_masks(k, 128, TD_PRE, kp); class_masks(k, 128, TD_CTX, kc); class_masks(k, 128, TD_INS, ki);
    class_masks(q, 128, TD_PRE << TD_SEES_SHIFT, qsp); class_masks(q, 128, TD_CTX << TD_SEES_SHIFT, qsc);
    class_masks(q, 128, TD_INS << TD_SEES_SHIFT, qsi); class_masks(q, 128, TD_CTX, qc);
    // query rows against 128 keys
    for (int r = 0; r < 128; ++r) {
      uint32_t m[4];
      query_row_mask<4>(q[r], i_base + r, j_base, kp, kc, ki, m);
      for (int j = 0; j < 128; ++j) {
        bool got = ((m[j >> 5] >> (j & 31)) & 1u) || same_span(q[r], k[j]);
        bad += (span_match_key(span_key_of_query(q[r]), k[j]) != 0u) != same_span(q[r], k[j]);
        bad += (span_match_query(span_key_of_key(k[j]), q[r]) != 0u) != same_span(q[r], k[j]);
        bool ref = rule_allowed(q[r], i_base + r, k[j], j_base + j);
        bad += got != ref; ++checked;
      }
    }
    // key rows against two 64-query halves
    for (int r = 0; r < 128; ++r)
      for (int half = 0; half < 2; ++half) {
        uint32_t m[2];
        key_row_mask<2>(k[r], j_base + r, i_base + 64 * half, qsp + 2 * half, qsc + 2 * half, qsi + 2 * half, qc + 2 * half, m);
        for (int t = 0; t < 64; ++t) {
          const int qi = 64 * half + t;
          bool got = ((m[t >> 5] >> (t & 31)) & 1u) || same_span(q[qi], k[r]);
          bool ref = rule_allowed(q[qi], i_base + qi, k[r], j_base + r);
          bad += got != ref; ++checked;
        }
      }
  }
  printf("checked=%lld bad=%lld\n", checked, bad);
  return bad == 0 ? 0 : 1;
}
