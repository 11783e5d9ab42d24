/*
 * kd_attention.h -- C ABI of libkd_attention.so: hierarchical-mask flash attention
 * (forward + backward) for NVIDIA B200 (sm_100a).
 *
 * This library replaces the GPU side of KernelDev's attention operator
 * (original_kernel.py in the reference project). Each entry point below names the
 * reference interface it stands in for (file:line inside the reference project).
 *
 * Conventions
 *  - Every pointer inside the parameter structs is a DEVICE pointer owned by the caller.
 *    The library allocates no device memory. The state it keeps between calls is a per-thread
 *    last-error string and, for kd_attn_bwd_static only, a fixed scratch array on every GPU
 *    together with its cached device address.
 *  - All entry points enqueue work on the given CUDA stream and return immediately:
 *    0 = enqueued, negative = rejected on the host before any launch (see kd_last_error()).
 *  - Device-side problems (a bounded wait that ran out, an unsupported span_id value) are
 *    reported through the 32-bit status word at plan offset `off_status`; it stays 0 on success.
 *  - Tensors are (B, H, T, D) with arbitrary element strides for b, h and t and unit stride
 *    along D; base pointers and the byte strides must be multiples of 16.
 *  - dtype: KD_F16 or KD_BF16; D: a multiple of 16 from 16 to 128 (the reference accepts 16, 32, 64, 128 and
 *    256, original_kernel.py:1720). Head dims below 64 run on the 64-wide kernels and those from 80 to 112 on
 *    the 128-wide ones: TMA fills the missing tile columns with zeros, which changes no product.
 */
#ifndef KD_ATTENTION_H_
#define KD_ATTENTION_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define KD_F16 0
#define KD_BF16 1
#define KD_F32 2   /* kd_span_mean only */

#define KD_TILE 128 /* mask classification and kernel tile edge (tokens) */

/* tile classes stored in the plan (one byte per (b, q_tile, k_tile)) */
#define KD_TILE_EMPTY 0   /* no (q,k) pair allowed: skipped without loading */
#define KD_TILE_FULL 1    /* every pair allowed: no per-element rule */
#define KD_TILE_PARTIAL 2 /* mixed: 4-section rule evaluated per element */

/* kd_attn_params.bwd_mode */
#define KD_BWD_SPLIT 0
#define KD_BWD_FUSED 1

/* error codes (negative return values) */
#define KD_ERR_ARG (-1)     /* bad shape / dtype / null pointer */
#define KD_ERR_ALIGN (-2)   /* pointer or stride not 16-byte aligned */
#define KD_ERR_DEVICE (-3)  /* not an sm_100 device, or CUDA runtime error */
#define KD_ERR_LIMIT (-4)   /* size beyond a stated maximum */

/* bits of the device status word */
#define KD_STATUS_TIMEOUT 0x10000000u  /* | code of the wait that gave up */
#define KD_STATUS_SPAN_RANGE 0x20000000u /* a span_id does not fit in 24 signed bits */

/* Per-token metadata of one batch, as produced by the reference's collate function
 * (data_builder.py:603-653) and consumed by _flash_attn_fwd (original_kernel.py:332-347,
 * :460-478). Any of the three metadata pointers may be NULL ("not given"). */
typedef struct kd_meta {
  int32_t B, T;
  const uint8_t* in_span;   /* (B,T) bool as bytes, token stride 1 */
  const int64_t* span_id;   /* (B,T) int64 */
  const uint8_t* is_prefix; /* (B,T) bool as bytes */
  const int32_t* lens;      /* (B,) int32 or NULL: keys/queries >= lens[b] are masked */
  int64_t in_span_stride_b, span_id_stride_b, is_prefix_stride_b; /* elements */
  int32_t causal;     /* used only when rules == 0 (original_kernel.py:512-515) */
  int32_t rules;      /* 1 when any of attention_mask/in_span/span_id/is_prefix was given
                         (the negation of FAST_PATH_NO_RULES, original_kernel.py:422) */
} kd_meta;

/* Byte offsets of the pieces of a plan inside the caller's plan buffer. */
typedef struct kd_plan_layout {
  int32_t B, T, NT, NP;  /* NT = ceil(T/128) tiles, NP = ceil(NT/2) query tile pairs */
  size_t off_desc;       /* uint32 [B][NT*128]   packed token descriptors */
  size_t off_summary;    /* uint32 [B][NT][4]    per-tile flag OR / AND, min / max span id */
  size_t off_cls;        /* uint8  [B][NT][NT]   tile class, index [b][q_tile][k_tile] */
  size_t off_fwd_cnt;    /* int32  [B][NP]       entries in the forward list of a q tile pair */
  size_t off_fwd_list;   /* uint16 [B][NP][NT]   k_tile | class(q tile 2p) << 8 | class(2p+1) << 10 */
  size_t off_bwd_cnt;    /* int32  [B][NT]       entries in the backward list of a k tile */
  size_t off_bwd_list;   /* uint16 [B][NT][NT]   q_tile | class << 8 */
  size_t off_tilebits;   /* uint32 [B][NT][8][4] 128-bit masks over the tokens of a tile: 0 is_prefix, 1 context,
                                                 2 in_span, 3..5 "as a query sees prefix / context / in_span keys
                                                 regardless of position", 6 same-span rule armed, 7 unused */
  size_t off_order;      /* uint8  [B][3][NT]    tiles sorted by decreasing work: [0] forward q tile
                                                 pairs, [1] dQ q tiles, [2] dK/dV k tiles */
  size_t off_stats;      /* uint32 [B][2]        number of FULL and of PARTIAL tiles */
  size_t off_status;     /* uint32               device status word (0 = ok) */
  size_t total;          /* bytes the caller must provide (256-byte aligned base) */
} kd_plan_layout;

typedef struct kd_tensor {
  void* ptr;
  int64_t stride_b, stride_h, stride_t; /* in elements; stride along D is 1 */
} kd_tensor;

typedef struct kd_attn_params {
  int32_t B, H, T, D;
  int32_t dtype;     /* KD_F16 / KD_BF16 */
  float sm_scale;    /* multiplies QK^T (original_kernel.py:415) */
  kd_tensor q, k, v; /* inputs */
  kd_tensor o;       /* forward: output; backward: input */
  kd_tensor d_o;     /* backward input dO */
  kd_tensor dq, dk, dv; /* backward outputs */
  float* lse;        /* (B,H,T) contiguous, base-2 log-sum-exp: m + log2(l)
                        (original_kernel.py:603-604); forward output, backward input */
  float* delta;      /* (B,H,T) contiguous fp32 scratch of the backward: rowsum(O * dO)
                        (kd_workspace_bytes gives its size) */
  const void* plan;  /* filled by kd_classify for the same (B,T) */
  int32_t bwd_phases; /* kd_attn_bwd only. 0 or 3: all kernels; 1: the delta kernel and the dQ
                         kernel; 2: the dK/dV kernel alone (reads delta of an earlier pass 1).
                         Lets a caller time the two large kernels separately. */
  int32_t bwd_mode;   /* kd_attn_bwd only. KD_BWD_SPLIT (0): a dQ kernel and a dK/dV kernel as in the reference
                         (original_kernel.py:1173-1336, :1339-1525), results bit-reproducible. KD_BWD_FUSED (1),
                         D = 64 only: one kernel forms S and dP once per tile and adds its dQ partials to dq_acc
                         with fp32 atomics (dQ then differs in the last bits from run to run). With
                         KD_BWD_FUSED, bwd_phases 1 runs the delta kernel alone and 2 the fused kernel. */
  float* dq_acc;      /* KD_BWD_FUSED: (B,H,T,D) contiguous fp32 scratch (kd_workspace_bytes_fused gives its
                         size); the library zeroes it itself. Ignored otherwise. */
  int32_t heads_per_cta; /* 0: chosen by the library from the grid size. n >= 1: every CTA handles n heads
                         one after the other (they share the plan's work list); a tuning and test knob. */
} kd_attn_params;

/* Size and layout of a plan for B sequences of T tokens. */
int kd_plan_layout_get(int32_t B, int32_t T, kd_plan_layout* out);

/* Packs the metadata into token descriptors, classifies every 128x128 tile as
 * EMPTY / FULL / PARTIAL from the exact rule (original_kernel.py:480-517) and builds the
 * per-tile work lists. Replaces the loop-bound choice at original_kernel.py:350-360, which
 * only ever skips tiles above the causal diagonal. */
int kd_classify(const kd_meta* meta, void* plan, void* stream);

/* Writes the dense mask (B,T,T) as bytes from the plan's descriptors: the debug output
 * the reference produces with return_attention_mask=True (original_kernel.py:520-545). */
int kd_mask_dense(const void* plan, int32_t B, int32_t T, uint8_t* out, void* stream);

/* Forward: O and base-2 LSE. Replaces flash_attention::forward
 * (attention_forward_adapter, original_kernel.py:1697-1778) and the kernel it launches,
 * _flash_attn_fwd (original_kernel.py:278-626). */
int kd_attn_fwd(const kd_attn_params* p, void* stream);

/* Backward: dQ, dK, dV. Replaces flash_attention::backward (attention_backward_adapter,
 * original_kernel.py:1806-1898): _flash_attn_bwd_precompute (:629-710) and _flash_attn_bwd
 * with its dQ and dK/dV workers (:713-838, :1173-1525). */
int kd_attn_bwd(const kd_attn_params* p, void* stream);

/* kd_attn_bwd without any caller-provided scratch. This entry point has no counterpart in the
 * reference. It is for hosts that are not allowed to allocate device memory where they call the
 * backward -- an engine that reserves all of HBM for its own arena at start-up and bans cudaMalloc
 * in plugin code, or a caller already inside a region where the allocator must not run. The
 * `delta` field of the params is ignored: the kernels use a fixed 4 MiB array inside the library
 * (every GPU that loads the library holds it until the process exits), so B*H*T must not exceed
 * 1,048,576 rows; larger problems are rejected with KD_ERR_LIMIT. The call allocates nothing.
 *  - The first call on each device looks up the array's device address (one cudaGetSymbolAddress,
 *    with that device current); make that first call before starting any stream capture.
 *  - All calls share the one array. Nothing in it has to start at zero (the delta kernel rewrites
 *    every row before the dQ and dK/dV kernels read it), but two calls that overlap on the GPU --
 *    different streams, or different host threads -- race on it. Serialise them.
 *  - bwd_phases must be 0 or 3: a dK/dV-only pass (2) would read whatever the previous call, perhaps
 *    of another problem, left in the array, so it is rejected with KD_ERR_ARG.
 *  - Inputs, outputs and results are exactly those of kd_attn_bwd. */
int kd_attn_bwd_static(const kd_attn_params* p, void* stream);

/* Bytes of the scratch buffer `delta` that kd_attn_bwd needs. */
int kd_workspace_bytes(int32_t B, int32_t H, int32_t T, int32_t D, size_t* bytes);

/* Bytes of the scratch buffer `dq_acc` that kd_attn_bwd needs with bwd_mode KD_BWD_FUSED (no counterpart in
 * the reference, which accumulates dQ in registers of its query-tile-major worker). */
int kd_workspace_bytes_fused(int32_t B, int32_t H, int32_t T, int32_t D, size_t* bytes);

/* Incoherent-processing transform over the last dimension, the "hadamard_transform" /
 * "generate_hadamard_signs" utilities the reference names in README.md:68-77 without shipping
 * code for them. signs is (H,D) of +-1 (or NULL for all +1).
 *   inverse = 0:  y = WHT(x * signs[h]) / sqrt(D)      (applied to Q and K)
 *   inverse = 1:  y = WHT(x) / sqrt(D) * signs[h]      (its transpose, applied to dQ and dK)
 * WHT is the Walsh-Hadamard transform in natural (Sylvester) order. y may alias x. */
int kd_hadamard(const kd_tensor* x, const kd_tensor* y, int32_t B, int32_t H, int32_t T, int32_t D,
                int32_t dtype, const float* signs, int32_t inverse, void* stream);

/* Per-token mask metadata from token ids, on the device (replaces the fallback of
 * GPTModel.forward, model.py:203-238: two cumulative sums plus a host loop with one .nonzero() /
 * .item() synchronisation per row).
 *   tokens     int64 (B,T), unit stride along T, stride_b elements between rows
 *   tok_*      ids of [SPAN], [ES], [CLS] and [MASKQ] (data_builder.py:44-51)
 *   in_span    uint8 (B,T) contiguous out: (#[SPAN] - #[ES] in tokens[b, 0..t]) > 0
 *   span_id    int64 (B,T) contiguous out: #[SPAN] in tokens[b, 0..t] where in_span, else 0; -1 at [MASKQ]
 *   is_prefix  uint8 (B,T) contiguous out: t <= index of the first [CLS] of the row (none: all 0)
 * The outputs are what kd_classify takes (bool tensors are one byte per element). */
int kd_metadata_from_tokens(const int64_t* tokens, int64_t stride_b, int32_t B, int32_t T, int64_t tok_span,
                            int64_t tok_es, int64_t tok_cls, int64_t tok_maskq, uint8_t* in_span,
                            int64_t* span_id, uint8_t* is_prefix, void* stream);

/* Span means of the cocktail-party head (model.py:258-296). kd_span_index ranks the [SPAN] and [ES]
 * markers of every row: starts / ends are int32 (B,T) with the position of the r-th marker of the
 * row at [b][r] and -1 beyond its count; n_starts / n_ends (B) are the counts and first_mask (B) the
 * position of the row's first [MASK] token or -1 (replaces the .nonzero() / torch.unique calls of
 * model.py:265-277). */
int kd_span_index(const int64_t* tokens, int64_t stride_b, int32_t B, int32_t T, int64_t tok_span, int64_t tok_es,
                  int64_t tok_mask, int32_t* starts, int32_t* ends, int32_t* n_starts, int32_t* n_ends,
                  int32_t* first_mask, void* stream);

/* backward = 0: h[b, j, :] = mean(x[b, st_j + 1 : ed_j, :]) for the pairs j < min(n_starts, n_ends) of row b
 * with st_j + 1 < ed_j, zero otherwise (the Python double loop of model.py:287-293);
 *   a = x (B,T,C) with element strides a_sb, a_st and unit stride along C; out = h (B,S,C) contiguous.
 * backward = 1: its gradient, grad_x[b, t, :] = sum over the pairs covering t of grad_h[b, j, :] / (ed_j - st_j - 1);
 *   a = grad_h (B,S,C) contiguous; out = grad_x (B,T,C) with element strides o_sb, o_st.
 * dtype KD_F16 / KD_BF16 / KD_F32 (sums in fp32). S is the padded span count of h (the reference uses the
 * largest n_starts of the batch). */
int kd_span_mean(int32_t backward, const void* a, int64_t a_sb, int64_t a_st, void* out, int64_t o_sb, int64_t o_st,
                 int32_t B, int32_t T, int32_t C, int32_t S, int32_t dtype, const int32_t* starts,
                 const int32_t* ends, const int32_t* n_starts, const int32_t* n_ends, void* stream);

/* Message for the last negative return value on this host thread. */
const char* kd_last_error(void);

int kd_version(void);

#ifdef __cplusplus
}
#endif
#endif /* KD_ATTENTION_H_ */
