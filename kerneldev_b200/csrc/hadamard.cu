// Incoherent-processing pre-pass: per-head sign flip and normalised Walsh-Hadamard transform
// over the head dimension. HBM-bound: reads and writes each element once; the butterflies run
// in registers (in-thread stages for the low index bits, warp shuffles for the high ones).
#include <algorithm>

#include "common.cuh"
#include "sm100_prims.cuh"

namespace kd {

// TPR = min(4, HD/8) threads share a token row; thread `sub` holds the 16-byte chunks sub, sub + TPR, ... of the
// row (CH = HD/8/TPR chunks of 8 elements), so that a warp-wide load covers 64 contiguous bytes per row.
// Element index = 8 * (sub + TPR * i) + k: index bits 0-2 (k) and the bits of i are butterflied in registers,
// the bits of `sub` with warp shuffles (two stages at most). Rows are walked with a grid-stride loop; bound by
// HBM bandwidth (2 * rows * HD * 2 bytes per call).
template <int HD, bool kBf16>
__global__ void __launch_bounds__(256) hadamard_kernel(const uint16_t* x, int64_t x_sb, int64_t x_sh, int64_t x_st,
                                                       uint16_t* y, int64_t y_sb, int64_t y_sh, int64_t y_st,
                                                       int B, int H, int T, const float* signs, int inverse) {
  constexpr int TPR = (HD / 8 < 4) ? HD / 8 : 4;   // threads per row
  constexpr int CH = HD / 8 / TPR;                 // chunks per thread
  constexpr int RPB = 256 / TPR;                   // rows per block and iteration
  const int sub = threadIdx.x % TPR;
  const long long rows = (long long)B * H * T;
  const float norm = rsqrtf(static_cast<float>(HD));
  // the loop bound is the same for every thread of a warp: the shuffles below need all lanes
  for (long long base = (long long)blockIdx.x * RPB; base < rows; base += (long long)gridDim.x * RPB) {
    const long long row = base + threadIdx.x / TPR;
    const bool live = row < rows;
    const long long rr = live ? row : rows - 1;
    const int t = static_cast<int>(rr % T);
    const int h = static_cast<int>((rr / T) % H);
    const int b = static_cast<int>(rr / ((long long)T * H));
    const uint16_t* src = x + (size_t)b * x_sb + (size_t)h * x_sh + (size_t)t * x_st;
    uint16_t* dst = y + (size_t)b * y_sb + (size_t)h * y_sh + (size_t)t * y_st;
    const float* sg = signs ? signs + h * HD : nullptr;
    uint4 in[CH];
#pragma unroll
    for (int i = 0; i < CH; ++i) in[i] = *reinterpret_cast<const uint4*>(src + (sub + TPR * i) * 8);
    float v[CH][8];
#pragma unroll
    for (int i = 0; i < CH; ++i) {
      const uint32_t w[4] = {in[i].x, in[i].y, in[i].z, in[i].w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = unpack2<kBf16>(w[k]);
        v[i][2 * k] = f.x; v[i][2 * k + 1] = f.y;
      }
      if (sg != nullptr && !inverse) {
        const float4 s0 = *reinterpret_cast<const float4*>(sg + (sub + TPR * i) * 8);
        const float4 s1 = *reinterpret_cast<const float4*>(sg + (sub + TPR * i) * 8 + 4);
        v[i][0] *= s0.x; v[i][1] *= s0.y; v[i][2] *= s0.z; v[i][3] *= s0.w;
        v[i][4] *= s1.x; v[i][5] *= s1.y; v[i][6] *= s1.z; v[i][7] *= s1.w;
      }
    }
    // index bits 0-2: inside a chunk
#pragma unroll
    for (int i = 0; i < CH; ++i) {
#pragma unroll
      for (int s = 1; s < 8; s <<= 1) {
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          if ((k & s) == 0) {
            const float a0 = v[i][k], a1 = v[i][k | s];
            v[i][k] = a0 + a1;
            v[i][k | s] = a0 - a1;
          }
        }
      }
    }
    // the bits of `sub`: across the threads of the row
#pragma unroll
    for (int s = 1; s < TPR; s <<= 1) {
#pragma unroll
      for (int i = 0; i < CH; ++i) {
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const float other = __shfl_xor_sync(0xffffffffu, v[i][k], s);
          v[i][k] = (sub & s) ? (other - v[i][k]) : (v[i][k] + other);
        }
      }
    }
    // the bits of the chunk counter i: between this thread's chunks
#pragma unroll
    for (int s = 1; s < CH; s <<= 1) {
#pragma unroll
      for (int i = 0; i < CH; ++i) {
        if ((i & s) == 0) {
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const float a0 = v[i][k], a1 = v[i | s][k];
            v[i][k] = a0 + a1;
            v[i | s][k] = a0 - a1;
          }
        }
      }
    }
#pragma unroll
    for (int i = 0; i < CH; ++i) {
      float f[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) f[k] = v[i][k] * norm;
      if (sg != nullptr && inverse) {
        const float4 s0 = *reinterpret_cast<const float4*>(sg + (sub + TPR * i) * 8);
        const float4 s1 = *reinterpret_cast<const float4*>(sg + (sub + TPR * i) * 8 + 4);
        f[0] *= s0.x; f[1] *= s0.y; f[2] *= s0.z; f[3] *= s0.w; f[4] *= s1.x; f[5] *= s1.y; f[6] *= s1.z; f[7] *= s1.w;
      }
      if (live) {
        uint4 out;
        out.x = pack2<kBf16>(f[0], f[1]);
        out.y = pack2<kBf16>(f[2], f[3]);
        out.z = pack2<kBf16>(f[4], f[5]);
        out.w = pack2<kBf16>(f[6], f[7]);
        *reinterpret_cast<uint4*>(dst + (sub + TPR * i) * 8) = out;
      }
    }
  }
}

int launch_hadamard(const kd_tensor& x, const kd_tensor& y, int B, int H, int T, int D, int dtype,
                    const float* signs, int inverse, cudaStream_t stream) {
  const long long rows = (long long)B * H * T;
  const int rows_per_block = 256 / (D / 8 < 4 ? D / 8 : 4);
  const unsigned blocks = static_cast<unsigned>(std::min<long long>((rows + rows_per_block - 1) / rows_per_block, 148LL * 32));
  const uint16_t* xp = static_cast<const uint16_t*>(x.ptr);
  uint16_t* yp = static_cast<uint16_t*>(y.ptr);
#define KD_LAUNCH_H(HD, BF)                                                                             \
  hadamard_kernel<HD, BF><<<blocks, 256, 0, stream>>>(xp, x.stride_b, x.stride_h, x.stride_t, yp,       \
                                                      y.stride_b, y.stride_h, y.stride_t, B, H, T, signs, inverse)
  if (D == 16 && dtype == KD_BF16) KD_LAUNCH_H(16, true);
  else if (D == 16) KD_LAUNCH_H(16, false);
  else if (D == 32 && dtype == KD_BF16) KD_LAUNCH_H(32, true);
  else if (D == 32) KD_LAUNCH_H(32, false);
  else if (D == 64 && dtype == KD_BF16) KD_LAUNCH_H(64, true);
  else if (D == 64) KD_LAUNCH_H(64, false);
  else if (D == 128 && dtype == KD_BF16) KD_LAUNCH_H(128, true);
  else KD_LAUNCH_H(128, false);
#undef KD_LAUNCH_H
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(KD_ERR_DEVICE, "hadamard_kernel launch: %s", cudaGetErrorString(e));
  return 0;
}

}  // namespace kd
