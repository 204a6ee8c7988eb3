// Masked any-shape W4A16 kernel: the correctness floor that serves every M, N, K >= 1,
// including K that is not a multiple of 8 or 64 and N, M tails.
//
// One warp owns one output row n and up to kBatch rows of X.  Lanes stride over the packed
// words of the row; every word is read once, its scale and zero point once, and each of its
// (up to) eight columns is dequantised in FP32 as (q - zero) * scale -- optionally rounded to
// FP16, the operand policy of the reference GEMM (csrc/cute_w4a16_gemm.cu:160-162) -- and
// multiplied into FP32 accumulators.  A shuffle tree finishes the row
// (the reduction of csrc/w4a16_gemv_warp_vec.cu:97-103).
#include "common.cuh"
#include "kernels.h"

namespace lbl {
namespace {

constexpr int kWarpsPerCta = 4;
constexpr int kBatch = 8;

template <bool kRoundWeights>
__global__ void __launch_bounds__(kWarpsPerCta * 32)
    w4a16_generic_kernel(const __half* __restrict__ x, const uint32_t* __restrict__ packed,
                         const float* __restrict__ scales, const int32_t* __restrict__ zeros,
                         __half* __restrict__ y, int64_t M, int64_t N, int64_t K) {
  const int lane = threadIdx.x & 31;
  const int64_t n = static_cast<int64_t>(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5);
  const int64_t m0 = static_cast<int64_t>(blockIdx.y) * kBatch;
  if (n >= N) return;

  const int64_t words = (K + 7) / 8;
  const int64_t groups = (K + 63) / 64;
  const int batch = static_cast<int>(M - m0 < kBatch ? M - m0 : kBatch);

  float acc[kBatch];
#pragma unroll
  for (int i = 0; i < kBatch; ++i) acc[i] = 0.0f;

  for (int64_t word = lane; word < words; word += 32) {
    const uint32_t bits = packed[n * words + word];
    const int64_t meta = n * groups + (word >> 3);
    const float scale = scales[meta];
    const int zero = zeros[meta];
    const int64_t k_base = word * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int64_t k = k_base + j;
      if (k < K) {
        const int q = static_cast<int>((bits >> (4 * j)) & 0xFu);
        float w = static_cast<float>(q - zero) * scale;
        if (kRoundWeights) w = __half2float(__float2half_rn(w));
#pragma unroll
        for (int i = 0; i < kBatch; ++i) {
          if (i < batch) acc[i] = fmaf(__half2float(x[(m0 + i) * K + k]), w, acc[i]);
        }
      }
    }
  }

#pragma unroll
  for (int i = 0; i < kBatch; ++i) {
    float v = acc[i];
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) v += __shfl_xor_sync(0xffffffffu, v, offset);
    if (lane == 0 && i < batch) y[(m0 + i) * N + n] = __float2half_rn(v);
  }
}

}  // namespace

cudaError_t launch_generic(const Problem& p, bool round_weights_to_fp16, cudaStream_t stream) {
  const int64_t row_blocks = (p.N + kWarpsPerCta - 1) / kWarpsPerCta;
  const int64_t batch_blocks = (p.M + kBatch - 1) / kBatch;
  if (row_blocks > 0x7fffffffLL || batch_blocks > 65535) return cudaErrorInvalidConfiguration;
  const dim3 grid(static_cast<unsigned>(row_blocks), static_cast<unsigned>(batch_blocks));
  if (round_weights_to_fp16) {
    w4a16_generic_kernel<true><<<grid, kWarpsPerCta * 32, 0, stream>>>(
        p.x, p.packed, p.scales, p.zeros, p.y, p.M, p.N, p.K);
  } else {
    w4a16_generic_kernel<false><<<grid, kWarpsPerCta * 32, 0, stream>>>(
        p.x, p.packed, p.scales, p.zeros, p.y, p.M, p.N, p.K);
  }
  return cudaGetLastError();
}

}  // namespace lbl
