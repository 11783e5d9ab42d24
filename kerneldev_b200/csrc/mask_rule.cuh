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

}  // namespace kd
