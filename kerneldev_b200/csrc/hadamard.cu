// Incoherent-processing pre-pass: per-head sign flip and normalised Walsh-Hadamard transform
// over the head dimension. HBM-bound: reads and writes each element once; the butterflies run
// in registers (in-thread stages for the low index bits, warp shuffles for the high ones).
#include <algorithm>

#include "common.cuh"
#include "sm100_prims.cuh"

namespace kd {

// HD/8 threads share a token row: thread t of the group holds elements [8t, 8t+8) (one 16-byte load and store,
// so a warp moves whole 128-byte lines). Index bits 0-2 are butterflied in registers, the bits above them
// with warp shuffles inside the group. Rows are walked with a grid-stride loop; bound by HBM bandwidth
// (2 * rows * HD * 2 bytes per call).
template <int HD, bool kBf16>
__global__ void __launch_bounds__(256) hadamard_kernel(const uint16_t* x, int64_t x_sb, int64_t x_sh, int64_t x_st,
                                                       uint16_t* y, int64_t y_sb, int64_t y_sh, int64_t y_st,
                                                       int B, int H, int T, const float* signs, int inverse) {
  constexpr int TPR = HD / 8;          // threads per row: 4, 8 or 16
  constexpr int RPB = 256 / TPR;       // rows per block and iteration
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
    const uint4 in = *reinterpret_cast<const uint4*>(x + (size_t)b * x_sb + (size_t)h * x_sh + (size_t)t * x_st + sub * 8);
    float v[8], sg[8];
    {
      const uint32_t w[4] = {in.x, in.y, in.z, in.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = unpack2<kBf16>(w[k]);
        v[2 * k] = f.x; v[2 * k + 1] = f.y;
      }
    }
    if (signs) {
      const float4 s0 = *reinterpret_cast<const float4*>(signs + h * HD + sub * 8);
      const float4 s1 = *reinterpret_cast<const float4*>(signs + h * HD + sub * 8 + 4);
      sg[0] = s0.x; sg[1] = s0.y; sg[2] = s0.z; sg[3] = s0.w; sg[4] = s1.x; sg[5] = s1.y; sg[6] = s1.z; sg[7] = s1.w;
    } else {
#pragma unroll
      for (int k = 0; k < 8; ++k) sg[k] = 1.f;
    }
    if (!inverse) {
#pragma unroll
      for (int k = 0; k < 8; ++k) v[k] *= sg[k];
    }
    // in-thread butterflies: index bits 0, 1, 2
#pragma unroll
    for (int s = 1; s < 8; s <<= 1) {
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        if ((k & s) == 0) {
          const float a0 = v[k], a1 = v[k | s];
          v[k] = a0 + a1;
          v[k | s] = a0 - a1;
        }
      }
    }
    // butterflies across the threads of the row: index bits 3 and above = bits of `sub`
#pragma unroll
    for (int s = 1; s < TPR; s <<= 1) {
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float other = __shfl_xor_sync(0xffffffffu, v[k], s);
        v[k] = (sub & s) ? (other - v[k]) : (v[k] + other);
      }
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) v[k] *= inverse ? norm * sg[k] : norm;
    if (live) {
      uint4 out;
      out.x = pack2<kBf16>(v[0], v[1]);
      out.y = pack2<kBf16>(v[2], v[3]);
      out.z = pack2<kBf16>(v[4], v[5]);
      out.w = pack2<kBf16>(v[6], v[7]);
      *reinterpret_cast<uint4*>(y + (size_t)b * y_sb + (size_t)h * y_sh + (size_t)t * y_st + sub * 8) = out;
    }
  }
}

int launch_hadamard(const kd_tensor& x, const kd_tensor& y, int B, int H, int T, int D, int dtype,
                    const float* signs, int inverse, cudaStream_t stream) {
  const long long rows = (long long)B * H * T;
  const int rows_per_block = 256 / (D / 8);
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
