// Device helpers shared by the forward and backward attention kernels: pre-split shared-memory
// descriptors (so the single MMA-issuing thread spends two integer adds per MMA, not a 64-bit
// descriptor build), work-list staging, 16-bit row stores.
#pragma once
#include "common.cuh"
#include "mask_rule.cuh"
#include "sm100_prims.cuh"

// Register split between the four light warps (producer, MMA issuer, list builder, idle) and the
// eight compute warps: 4*32*ISSUE + 8*32*COMPUTE must not exceed 65536.
#ifndef KD_REGS_ISSUE
#define KD_REGS_ISSUE 56
#endif
#ifndef KD_REGS_COMPUTE
#define KD_REGS_COMPUTE 224
#endif
// The backward kernels run sixteen compute warps (640 threads, 96 registers each at launch):
// 4*32*(96 - ISSUE) released registers cover 16*32*(COMPUTE_BWD - 96).
#ifndef KD_REGS_COMPUTE_BWD
#define KD_REGS_COMPUTE_BWD 104
#endif

namespace kd {

// High words of the two descriptor kinds used here (layout, version, stride byte offset 1024);
// the low word carries the start address and the leading byte offset.
__device__ __forceinline__ uint32_t desc_hi_sw128() {
  return static_cast<uint32_t>(make_smem_desc(0, 0, 1024, KD_LAYOUT_SW128) >> 32);
}
// low word of a K-major tile descriptor at k-step 0 (leading byte offset field = 1)
__device__ __forceinline__ uint32_t desc_lo_kmajor(uint32_t saddr) { return ((saddr >> 4) & 0x3FFFu) | (1u << 16); }
// low word of an MN-major tile descriptor whose 64-wide MN blocks are 16 KB apart
__device__ __forceinline__ uint32_t desc_lo_mnmajor(uint32_t saddr) { return ((saddr >> 4) & 0x3FFFu) | (1024u << 16); }
// offset (in 16-byte units) of k-step kk inside a K-major tile built from [rows][64] blocks 16 KB apart
__device__ __forceinline__ constexpr uint32_t koff_kmajor(int kk) { return static_cast<uint32_t>((kk / 4) * 1024 + (kk % 4) * 2); }
// offset (16-byte units) of k-step kk (16 rows of 128 bytes) inside an MN-major tile
__device__ __forceinline__ constexpr uint32_t koff_mnmajor(int kk) { return static_cast<uint32_t>(kk * 128); }

__device__ __forceinline__ void mma_ss_split(uint32_t d_tmem, uint32_t alo, uint32_t blo, uint32_t hi,
                                             uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      ".reg .b64 da, db;\n"
      "mov.b64 da, {%1, %3};\n"
      "mov.b64 db, {%2, %3};\n"
      "setp.ne.b32 p, %5, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n"
      "}\n"
      ::"r"(d_tmem), "r"(alo), "r"(blo), "r"(hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
// MMA forms whose shared-memory descriptors are complete 64-bit values. The issuing thread forms
// them BEFORE it waits for the barriers of a unit, so that once the barriers have fired the MMAs go
// out back to back with no address arithmetic between them: that thread shares its scheduler with
// busy compute warps, and every dependent instruction in its path costs it 10-20 cycles.
__device__ __forceinline__ uint64_t desc64(uint32_t lo, uint32_t hi) { return (static_cast<uint64_t>(hi) << 32) | lo; }
// maximum of three floats in one instruction (sm_100)
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

template <bool kAccumulate>
__device__ __forceinline__ void mma_ss64(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "n"(kAccumulate ? 1 : 0)
      : "memory");
}
template <bool kAccumulate>
__device__ __forceinline__ void mma_ts64(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
      "}\n"
      ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "n"(kAccumulate ? 1 : 0)
      : "memory");
}
// accumulate flag known only at run time (first product into an accumulator)
__device__ __forceinline__ void mma_ts64_p(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
      "}\n"
      ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_ts_split(uint32_t d_tmem, uint32_t a_tmem, uint32_t blo, uint32_t hi,
                                             uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      ".reg .b64 db;\n"
      "mov.b64 db, {%2, %3};\n"
      "setp.ne.b32 p, %5, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n"
      "}\n"
      ::"r"(d_tmem), "r"(a_tmem), "r"(blo), "r"(hi), "r"(idesc), "r"(accumulate)
      : "memory");
}

// stores 32 fp32 accumulator values (scaled) as 16-bit elements to a row in global memory
template <bool kBf16>
__device__ __forceinline__ void store_row32(uint16_t* dst, const uint32_t (&r)[32], float f) {
#pragma unroll
  for (int j = 0; j < 32; j += 8) {
    uint4 v;
    v.x = pack2<kBf16>(__uint_as_float(r[j + 0]) * f, __uint_as_float(r[j + 1]) * f);
    v.y = pack2<kBf16>(__uint_as_float(r[j + 2]) * f, __uint_as_float(r[j + 3]) * f);
    v.z = pack2<kBf16>(__uint_as_float(r[j + 4]) * f, __uint_as_float(r[j + 5]) * f);
    v.w = pack2<kBf16>(__uint_as_float(r[j + 6]) * f, __uint_as_float(r[j + 7]) * f);
    *reinterpret_cast<uint4*>(dst + j) = v;
  }
}

template <bool kBf16>
__device__ __forceinline__ void store_row16(uint16_t* dst, const uint32_t (&r)[16], float f) {
#pragma unroll
  for (int j = 0; j < 16; j += 8) {
    uint4 v;
    v.x = pack2<kBf16>(__uint_as_float(r[j + 0]) * f, __uint_as_float(r[j + 1]) * f);
    v.y = pack2<kBf16>(__uint_as_float(r[j + 2]) * f, __uint_as_float(r[j + 3]) * f);
    v.z = pack2<kBf16>(__uint_as_float(r[j + 4]) * f, __uint_as_float(r[j + 5]) * f);
    v.w = pack2<kBf16>(__uint_as_float(r[j + 6]) * f, __uint_as_float(r[j + 7]) * f);
    *reinterpret_cast<uint4*>(dst + j) = v;
  }
}

// 32 (or 16) accumulator columns starting at column `col` of a row whose real width is d_real (a multiple
// of 16): the columns at or beyond d_real belong to the zero-filled part of a tile and are not stored.
template <bool kBf16>
__device__ __forceinline__ void store_row32_upto(uint16_t* dst, const uint32_t (&r)[32], float f, int col, int d_real) {
  if (col + 32 <= d_real) {
    store_row32<kBf16>(dst, r, f);
  } else if (col < d_real) {   // 16 columns left
#pragma unroll
    for (int j = 0; j < 16; j += 8) {
      uint4 v;
      v.x = pack2<kBf16>(__uint_as_float(r[j + 0]) * f, __uint_as_float(r[j + 1]) * f);
      v.y = pack2<kBf16>(__uint_as_float(r[j + 2]) * f, __uint_as_float(r[j + 3]) * f);
      v.z = pack2<kBf16>(__uint_as_float(r[j + 4]) * f, __uint_as_float(r[j + 5]) * f);
      v.w = pack2<kBf16>(__uint_as_float(r[j + 6]) * f, __uint_as_float(r[j + 7]) * f);
      *reinterpret_cast<uint4*>(dst + j) = v;
    }
  }
}
template <bool kBf16>
__device__ __forceinline__ void store_row16_upto(uint16_t* dst, const uint32_t (&r)[16], float f, int col, int d_real) {
  if (col < d_real) store_row16<kBf16>(dst, r, f);
}

// Heads a CTA handles one after the other (they share the plan's work list, so the list staging,
// the TMEM allocation and the pipeline fill are paid once): as many as keeps about per_sm CTAs per SM,
// at most g_max (the longest-first dispatch order keeps the SMs balanced with that few). Measured
// best over batches 4-16 of config 2 and configs 1 and 3: backward 6 per SM, up to 8 heads; forward (a
// CTA already holds two query tiles) 3 per SM, up to 4. Fewer CTAs than that lose more to imbalance
// between sequences of different section lengths than the shared pipeline fill saves.
inline int heads_per_cta(int B, int H, int items_per_batch, int forced, int per_sm = 6, int g_max = 8) {
  if (forced >= 1) return forced < H ? forced : H;
  static int sm_count = 0;
  if (sm_count == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sm_count <= 0)
      sm_count = 148;
  }
  const long long ctas = (long long)B * H * items_per_batch;
  long long g = ctas / ((long long)sm_count * per_sm);
  if (g < 1) g = 1;
  if (g > g_max) g = g_max;
  if (g > H) g = H;
  return static_cast<int>(g);
}

// bounded wait used while unwinding after an abort: lets a TMA copy that is already in flight land
__device__ __forceinline__ void drain_wait(uint32_t bar, uint32_t parity) {
  for (int spin = 0; spin < (1 << 20) && !mbar_try_wait(bar, parity); ++spin) {
  }
}

}  // namespace kd
