// Group-64 asymmetric INT4 quantiser and packer in one kernel: FP16 / FP32 weights in, packed
// words + FP32 scales + INT32 zero points out, in the reference layout.
//
// Restates the reference's quantize_int4 + pack_int4 (lowbitlinear/quantization.py:33-86 and
// :112-141) with the arithmetic of its CPU path, operation for operation, so the results are
// bit-identical to the reference run on CPU tensors:
//   lo = min(min(group), 0)      hi = max(max(group), 0)
//   scale = (hi - lo) / 15       IEEE division; 1 when the quotient is not positive
//   zero  = clamp(rint(-lo / scale), 0, 15)
//   q     = clamp(rint(w / scale + zero), 0, 15)      division, then a separate addition
// (round half to even, no fused multiply-add, no reciprocal).  One warp owns one group of one
// row: a lane holds two neighbouring weights, min / max go through shuffles, two levels make a
// byte and four lanes' bytes make a word.  Columns past K pack as level 0, as the reference pads.
#include "kernels.h"

namespace lbl {
namespace {

constexpr int kWarpsPerCta = 8;

template <typename T>
__device__ __forceinline__ float to_float(T v);
template <>
__device__ __forceinline__ float to_float<float>(float v) {
  return v;
}
template <>
__device__ __forceinline__ float to_float<__half>(__half v) {
  return __half2float(v);
}

template <typename T>
__global__ void __launch_bounds__(kWarpsPerCta * 32)
    w4_quantize_pack_kernel(const T* __restrict__ weight, uint32_t* __restrict__ packed,
                            float* __restrict__ scales, int32_t* __restrict__ zeros, int64_t N,
                            int64_t K) {
  const int lane = threadIdx.x & 31;
  const int64_t groups = (K + 63) / 64;
  const int64_t words = (K + 7) / 8;
  const int64_t item = static_cast<int64_t>(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5);
  if (item >= N * groups) return;
  const int64_t row = item / groups;
  const int64_t group = item - row * groups;
  const int64_t k0 = group * 64 + 2 * lane;

  const bool in0 = k0 < K;
  const bool in1 = k0 + 1 < K;
  const T* src = weight + row * K + k0;
  const float w0 = in0 ? to_float<T>(src[0]) : 0.0f;
  const float w1 = in1 ? to_float<T>(src[1]) : 0.0f;

  // Zeros for the missing columns leave a minimum clamped to <= 0 and a maximum clamped to >= 0
  // unchanged.
  float lo = fminf(fminf(w0, w1), 0.0f);
  float hi = fmaxf(fmaxf(w0, w1), 0.0f);
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) {
    lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, offset));
    hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, offset));
  }
  const float raw = __fdiv_rn(__fsub_rn(hi, lo), 15.0f);
  const float scale = raw > 0.0f ? raw : 1.0f;
  const float zero_f = fminf(fmaxf(rintf(__fdiv_rn(-lo, scale)), 0.0f), 15.0f);
  const float q0 = fminf(fmaxf(rintf(__fadd_rn(__fdiv_rn(w0, scale), zero_f)), 0.0f), 15.0f);
  const float q1 = fminf(fmaxf(rintf(__fadd_rn(__fdiv_rn(w1, scale), zero_f)), 0.0f), 15.0f);
  const uint32_t level0 = in0 ? static_cast<uint32_t>(q0) : 0u;
  const uint32_t level1 = in1 ? static_cast<uint32_t>(q1) : 0u;

  // byte = two levels, low nibble first; word = the bytes of four neighbouring lanes.
  const uint32_t byte = level0 | (level1 << 4);
  uint32_t word = byte;
  word |= __shfl_down_sync(0xffffffffu, byte, 1) << 8;
  word |= __shfl_down_sync(0xffffffffu, byte, 2) << 16;
  word |= __shfl_down_sync(0xffffffffu, byte, 3) << 24;
  const int64_t word_index = group * 8 + (lane >> 2);
  if ((lane & 3) == 0 && word_index < words) packed[row * words + word_index] = word;
  if (lane == 0) {
    scales[row * groups + group] = scale;
    zeros[row * groups + group] = static_cast<int32_t>(zero_f);
  }
}

}  // namespace

cudaError_t launch_quantize(const void* weight, bool weight_is_fp32, int64_t N, int64_t K,
                            uint32_t* packed, float* scales, int32_t* zeros, cudaStream_t stream) {
  const int64_t groups = (K + 63) / 64;
  const int64_t items = N * groups;
  const int64_t blocks = (items + kWarpsPerCta - 1) / kWarpsPerCta;
  if (blocks <= 0 || blocks > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
  const dim3 grid(static_cast<unsigned>(blocks));
  if (weight_is_fp32) {
    w4_quantize_pack_kernel<float><<<grid, kWarpsPerCta * 32, 0, stream>>>(
        static_cast<const float*>(weight), packed, scales, zeros, N, K);
  } else {
    w4_quantize_pack_kernel<__half><<<grid, kWarpsPerCta * 32, 0, stream>>>(
        static_cast<const __half*>(weight), packed, scales, zeros, N, K);
  }
  return cudaGetLastError();
}

}  // namespace lbl
