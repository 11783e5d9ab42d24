// Incoherent-processing pre-pass: per-head sign flip and normalised Walsh-Hadamard transform
// over the head dimension. HBM-bound: reads and writes each element once; the butterflies run
// in registers (in-thread stages for the low index bits, warp shuffles for the high ones).
#include "common.cuh"
#include "sm100_prims.cuh"

namespace kd {

// One warp per token row: lane l holds elements [l*E, (l+1)*E), E = D / 32.
template <int HD, bool kBf16>
__global__ void __launch_bounds__(256) hadamard_kernel(const uint16_t* x, int64_t x_sb, int64_t x_sh, int64_t x_st,
                                                       uint16_t* y, int64_t y_sb, int64_t y_sh, int64_t y_st,
                                                       int B, int H, int T, const float* signs, int inverse) {
  constexpr int E = HD / 32;  // 2 or 4 elements per lane
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= (long long)B * H * T) return;
  const int t = static_cast<int>(row % T);
  const int h = static_cast<int>((row / T) % H);
  const int b = static_cast<int>(row / ((long long)T * H));
  const uint16_t* src = x + (size_t)b * x_sb + (size_t)h * x_sh + (size_t)t * x_st + lane * E;
  uint16_t* dst = y + (size_t)b * y_sb + (size_t)h * y_sh + (size_t)t * y_st + lane * E;

  float v[E];
  if constexpr (E == 2) {
    const float2 f = unpack2<kBf16>(*reinterpret_cast<const uint32_t*>(src));
    v[0] = f.x; v[1] = f.y;
  } else {
    const uint2 w = *reinterpret_cast<const uint2*>(src);
    const float2 f0 = unpack2<kBf16>(w.x), f1 = unpack2<kBf16>(w.y);
    v[0] = f0.x; v[1] = f0.y; v[2] = f1.x; v[3] = f1.y;
  }
  float sg[E];
#pragma unroll
  for (int k = 0; k < E; ++k) sg[k] = signs ? signs[h * HD + lane * E + k] : 1.f;
  if (!inverse) {
#pragma unroll
    for (int k = 0; k < E; ++k) v[k] *= sg[k];
  }
  // in-thread butterflies (index bits below log2(E))
#pragma unroll
  for (int s = 1; s < E; s <<= 1) {
#pragma unroll
    for (int k = 0; k < E; ++k) {
      if ((k & s) == 0) {
        const float a0 = v[k], a1 = v[k | s];
        v[k] = a0 + a1;
        v[k | s] = a0 - a1;
      }
    }
  }
  // cross-lane butterflies (index bits log2(E) and above = lane bits)
#pragma unroll
  for (int s = 1; s < 32; s <<= 1) {
#pragma unroll
    for (int k = 0; k < E; ++k) {
      const float other = __shfl_xor_sync(0xffffffffu, v[k], s);
      v[k] = (lane & s) ? (other - v[k]) : (v[k] + other);
    }
  }
  const float norm = (HD == 64) ? 0.125f : 0.08838834764831845f;  // 1 / sqrt(D)
#pragma unroll
  for (int k = 0; k < E; ++k) v[k] *= inverse ? norm * sg[k] : norm;
  if constexpr (E == 2) {
    *reinterpret_cast<uint32_t*>(dst) = pack2<kBf16>(v[0], v[1]);
  } else {
    uint2 w;
    w.x = pack2<kBf16>(v[0], v[1]);
    w.y = pack2<kBf16>(v[2], v[3]);
    *reinterpret_cast<uint2*>(dst) = w;
  }
}

int launch_hadamard(const kd_tensor& x, const kd_tensor& y, int B, int H, int T, int D, int dtype,
                    const float* signs, int inverse, cudaStream_t stream) {
  const long long rows = (long long)B * H * T;
  const unsigned blocks = static_cast<unsigned>((rows + 7) / 8);
  const uint16_t* xp = static_cast<const uint16_t*>(x.ptr);
  uint16_t* yp = static_cast<uint16_t*>(y.ptr);
#define KD_LAUNCH_H(HD, BF)                                                                             \
  hadamard_kernel<HD, BF><<<blocks, 256, 0, stream>>>(xp, x.stride_b, x.stride_h, x.stride_t, yp,       \
                                                      y.stride_b, y.stride_h, y.stride_t, B, H, T, signs, inverse)
  if (D == 64 && dtype == KD_BF16) KD_LAUNCH_H(64, true);
  else if (D == 64) KD_LAUNCH_H(64, false);
  else if (D == 128 && dtype == KD_BF16) KD_LAUNCH_H(128, true);
  else KD_LAUNCH_H(128, false);
#undef KD_LAUNCH_H
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(KD_ERR_DEVICE, "hadamard_kernel launch: %s", cudaGetErrorString(e));
  return 0;
}

}  // namespace kd
