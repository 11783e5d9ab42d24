// Packed per-token descriptors and the 4-section visibility rule.
//
// The rule is the boolean function evaluated per element by the reference forward kernel
// (original_kernel.py:480-517) and, transposed, by its backward workers (:1289-1328,
// :1475-1514). It is restated here on a packed 32-bit descriptor so that one 32-bit load per
// token carries everything the rule needs, for the token as a query and as a key.
#pragma once
#include <stdint.h>

namespace kd {

// descriptor bits
constexpr uint32_t TD_PRE = 1u << 0;     // is_prefix
constexpr uint32_t TD_CTX = 1u << 1;     // context: !in_span & !is_prefix & span_id != -1
constexpr uint32_t TD_INS = 1u << 2;     // in_span
constexpr uint32_t TD_MQ = 1u << 3;      // span_id == -1  ([MASKQ])
constexpr uint32_t TD_SIDPOS = 1u << 4;  // in_span && span_id > 0 (same-span rule armed)
constexpr uint32_t TD_FLAGS = 0x1Fu;
// bits [5,8): as a QUERY, the key classes (PRE / CTX / INS, shifted up by 5) this token sees
// regardless of position and span id
constexpr int TD_SEES_SHIFT = 5;
constexpr int TD_SID_SHIFT = 8;          // span id, low 24 bits, in bits [8,32)
// A token at or beyond the sequence length (lens[b] or T) has descriptor 0: it sees nothing
// and nothing sees it, which is the length mask of original_kernel.py:517.

// key classes a query with these flag bits sees unconditionally
__host__ __device__ __forceinline__ uint32_t sees_of_flags(uint32_t f) {
  uint32_t u = 0;
  if (f & (TD_PRE | TD_CTX | TD_MQ)) u |= TD_PRE;  // prefix<->prefix, context->prefix, MASKQ->prefix
  if (f & TD_INS) u |= TD_CTX;                     // span -> every context key (not causal)
  if (f & TD_MQ) u |= TD_INS;                      // MASKQ -> every span token
  return u;
}

__host__ __device__ __forceinline__ uint32_t pack_token(bool in_span, bool is_prefix, int64_t span_id,
                                                        bool alive) {
  if (!alive) return 0u;
  const bool mq = (span_id == -1);
  uint32_t d = 0;
  if (is_prefix) d |= TD_PRE;
  if (!in_span && !is_prefix && !mq) d |= TD_CTX;
  if (in_span) d |= TD_INS;
  if (mq) d |= TD_MQ;
  if (in_span && span_id > 0) d |= TD_SIDPOS;
  d |= sees_of_flags(d) << TD_SEES_SHIFT;
  d |= (static_cast<uint32_t>(static_cast<int32_t>(span_id)) & 0xFFFFFFu) << TD_SID_SHIFT;
  return d;
}

// descriptor of a token when no metadata is given: causal -> context, otherwise prefix
__host__ __device__ __forceinline__ uint32_t pack_plain(bool causal) {
  const uint32_t f = causal ? TD_CTX : TD_PRE;
  return f | (sees_of_flags(f) << TD_SEES_SHIFT);
}

// allowed(i, j): query index i with descriptor qd, key index j with descriptor kdesc
__host__ __device__ __forceinline__ bool rule_allowed(uint32_t qd, int i, uint32_t kdesc, int j) {
  const bool a = ((qd >> TD_SEES_SHIFT) & kdesc & 7u) != 0u;
  const bool c = ((qd & kdesc & TD_CTX) != 0u) && (i >= j);
  const bool s = ((qd & TD_SIDPOS) != 0u) && ((kdesc & TD_INS) != 0u) && (((qd ^ kdesc) >> TD_SID_SHIFT) == 0u);
  return a || c || s;
}

// ---------------------------------------------------------------------------------------
// Bit-parallel form of the rule for one row against a run of W*32 tokens of the other side.
// The plan stores, per 128-token tile, eight 128-bit masks (index = TB_*); a row combines a few of
// them with word-wide logic instead of evaluating the rule per element.
// ---------------------------------------------------------------------------------------
constexpr int TB_PRE = 0, TB_CTX = 1, TB_INS = 2, TB_SEES_PRE = 3, TB_SEES_CTX = 4, TB_SEES_INS = 5, TB_SIDPOS = 6;

// mask with the lowest n bits set, n clamped to [0, 32]
__host__ __device__ __forceinline__ uint32_t low_bits(int n) {
  return n <= 0 ? 0u : (n >= 32 ? 0xFFFFFFFFu : ((1u << n) - 1u));
}

// Query row with descriptor qd at index i against W words of key-side masks (PRE, CTX, INS) of the
// keys j0 .. j0 + 32 W - 1: every term of the rule except "same span".
template <int W>
__host__ __device__ __forceinline__ void query_row_mask(uint32_t qd, int i, int j0, const uint32_t* k_pre,
                                                        const uint32_t* k_ctx, const uint32_t* k_ins, uint32_t* m) {
  const uint32_t sees = qd >> TD_SEES_SHIFT;
  const uint32_t s_pre = (sees & TD_PRE) ? 0xFFFFFFFFu : 0u, s_ctx = (sees & TD_CTX) ? 0xFFFFFFFFu : 0u,
                 s_ins = (sees & TD_INS) ? 0xFFFFFFFFu : 0u, q_ctx = (qd & TD_CTX) ? 0xFFFFFFFFu : 0u;
#pragma unroll
  for (int w = 0; w < W; ++w) {
    const uint32_t causal = low_bits(i - j0 - 32 * w + 1);   // keys j <= i
    m[w] = (k_pre[w] & s_pre) | (k_ctx[w] & (s_ctx | (q_ctx & causal))) | (k_ins[w] & s_ins);
  }
}

// Key row with descriptor kd at index j against W words of query-side masks of the queries
// i0 .. i0 + 32 W - 1: every term of the rule except "same span".
template <int W>
__host__ __device__ __forceinline__ void key_row_mask(uint32_t kdesc, int j, int i0, const uint32_t* q_sees_pre,
                                                      const uint32_t* q_sees_ctx, const uint32_t* q_sees_ins,
                                                      const uint32_t* q_ctx, uint32_t* m) {
  const uint32_t is_pre = (kdesc & TD_PRE) ? 0xFFFFFFFFu : 0u, is_ctx = (kdesc & TD_CTX) ? 0xFFFFFFFFu : 0u,
                 is_ins = (kdesc & TD_INS) ? 0xFFFFFFFFu : 0u;
#pragma unroll
  for (int w = 0; w < W; ++w) {
    const uint32_t causal = ~low_bits(j - i0 - 32 * w);      // queries i >= j
    m[w] = (q_sees_pre[w] & is_pre) | (is_ctx & (q_sees_ctx[w] | (q_ctx[w] & causal))) | (q_sees_ins[w] & is_ins);
  }
}

// "same span" term for one pair of descriptors
__host__ __device__ __forceinline__ bool same_span(uint32_t qd, uint32_t kdesc) {
  return ((qd & TD_SIDPOS) != 0u) && ((kdesc & TD_INS) != 0u) && (((qd ^ kdesc) >> TD_SID_SHIFT) == 0u);
}

// Branch-free form for inner loops: the row side is folded once into a match key (span id bits
// plus the in_span flag, or a value no descriptor can produce when the rule is not armed); each
// token of the other side then costs one AND and one compare.
constexpr uint32_t TD_SPAN_KEY_BITS = 0xFFFFFF00u | TD_INS;
// key of a QUERY row matched against KEY descriptors: key needs in_span and the same id
__host__ __device__ __forceinline__ uint32_t span_key_of_query(uint32_t qd) {
  return (qd & TD_SIDPOS) ? ((qd & 0xFFFFFF00u) | TD_INS) : 0x00000001u;   // bit 0 is outside TD_SPAN_KEY_BITS: never matches
}
__host__ __device__ __forceinline__ uint32_t span_match_key(uint32_t key, uint32_t kdesc) {
  return ((kdesc & TD_SPAN_KEY_BITS) == key) ? 1u : 0u;
}
// key of a KEY row matched against QUERY descriptors: query needs the rule armed and the same id
constexpr uint32_t TD_SPAN_QUERY_BITS = 0xFFFFFF00u | TD_SIDPOS;
__host__ __device__ __forceinline__ uint32_t span_key_of_key(uint32_t kdesc) {
  return (kdesc & TD_INS) ? ((kdesc & 0xFFFFFF00u) | TD_SIDPOS) : 0x00000001u;
}
__host__ __device__ __forceinline__ uint32_t span_match_query(uint32_t key, uint32_t qd) {
  return ((qd & TD_SPAN_QUERY_BITS) == key) ? 1u : 0u;
}

}  // namespace kd
