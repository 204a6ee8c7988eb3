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
// (round half to even, no fused multiply-add, no reciprocal).  Sixteen lanes own one group of
// one row: a lane holds four neighbouring weights, min / max go through shuffles, a lane's four
// levels make half a word and two lanes make a word.  Columns past K pack as level 0, as the
// reference pads.
#include "kernels.h"

namespace lbl {
namespace {

constexpr int kWarpsPerCta = 8;

// Four neighbouring weights of one row as floats; columns at or past `limit` read as 0.
template <typename T>
__device__ __forceinline__ void load4(const T* row, int64_t k0, int64_t limit, bool vector_ok,
                                      float (&w)[4]);

template <>
__device__ __forceinline__ void load4<__half>(const __half* row, int64_t k0, int64_t limit,
                                              bool vector_ok, float (&w)[4]) {
  if (vector_ok && k0 + 4 <= limit) {
    const uint2 raw = *reinterpret_cast<const uint2*>(row + k0);
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
    const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
    w[0] = a.x, w[1] = a.y, w[2] = b.x, w[3] = b.y;
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) w[i] = (k0 + i < limit) ? __half2float(row[k0 + i]) : 0.0f;
  }
}

template <>
__device__ __forceinline__ void load4<float>(const float* row, int64_t k0, int64_t limit,
                                             bool vector_ok, float (&w)[4]) {
  if (vector_ok && k0 + 4 <= limit) {
    const float4 raw = *reinterpret_cast<const float4*>(row + k0);
    w[0] = raw.x, w[1] = raw.y, w[2] = raw.z, w[3] = raw.w;
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) w[i] = (k0 + i < limit) ? row[k0 + i] : 0.0f;
  }
}

// A warp owns two neighbouring groups of one row (16 lanes each, four weights per lane).
template <typename T>
__global__ void __launch_bounds__(kWarpsPerCta * 32)
    w4_quantize_pack_kernel(const T* __restrict__ weight, uint32_t* __restrict__ packed,
                            float* __restrict__ scales, int32_t* __restrict__ zeros, int64_t N,
                            int64_t K, bool vector_ok) {
  const int lane = threadIdx.x & 31;
  const int64_t groups = (K + 63) / 64;
  const int64_t pairs = (groups + 1) / 2;
  const int64_t words = (K + 7) / 8;
  const int64_t total = N * pairs;
  const int64_t item = static_cast<int64_t>(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5);
  if (item >= total) return;
  int64_t row, pair;
  if (total <= 0xffffffffLL) {  // the usual case: one 32-bit division instead of a 64-bit one
    const uint32_t r = static_cast<uint32_t>(item) / static_cast<uint32_t>(pairs);
    row = r;
    pair = static_cast<uint32_t>(item) - r * static_cast<uint32_t>(pairs);
  } else {
    row = item / pairs;
    pair = item - row * pairs;
  }
  const int sub = lane & 15;
  const int64_t group = pair * 2 + (lane >> 4);
  const bool group_ok = group < groups;
  const int64_t k0 = group * 64 + 4 * sub;

  float w[4];
  load4<T>(weight + row * K, k0, group_ok ? K : 0, vector_ok, w);

  // Zeros for the missing columns leave a minimum clamped to <= 0 and a maximum clamped to >= 0
  // unchanged.
  float lo = fminf(fminf(fminf(w[0], w[1]), fminf(w[2], w[3])), 0.0f);
  float hi = fmaxf(fmaxf(fmaxf(w[0], w[1]), fmaxf(w[2], w[3])), 0.0f);
#pragma unroll
  for (int offset = 8; offset > 0; offset >>= 1) {  // stays inside each half of the warp
    lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, offset));
    hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, offset));
  }
  const float raw = __fdiv_rn(__fsub_rn(hi, lo), 15.0f);
  const float scale = raw > 0.0f ? raw : 1.0f;
  const float zero_f = fminf(fmaxf(rintf(__fdiv_rn(-lo, scale)), 0.0f), 15.0f);

  // Two levels make a byte (low nibble first), a lane's four levels make half a word.
  uint32_t half_word = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float q = fminf(fmaxf(rintf(__fadd_rn(__fdiv_rn(w[i], scale), zero_f)), 0.0f), 15.0f);
    const uint32_t level = (k0 + i < K) ? static_cast<uint32_t>(q) : 0u;
    half_word |= level << (4 * i);
  }
  const uint32_t word = half_word | (__shfl_down_sync(0xffffffffu, half_word, 1) << 16);
  const int64_t word_index = group * 8 + (sub >> 1);
  if (group_ok && (sub & 1) == 0 && word_index < words) packed[row * words + word_index] = word;
  if (group_ok && sub == 0) {
    scales[row * groups + group] = scale;
    zeros[row * groups + group] = static_cast<int32_t>(zero_f);
  }
}

// ---------------------------------------------------------------------------------------------
// Dequantiser: packed words -> dense weights, w = float(q - zero) * scale in FP32
// (lowbitlinear/quantization.py:88-110 after :143-171), stored as FP32 or rounded once to FP16
// (what the reference benchmark's pre-dequantised baseline holds, bench_w4a16.py:37-43).
// A thread expands one word into eight neighbouring weights; HBM-bound on its own stores.
// ---------------------------------------------------------------------------------------------
template <typename Out>
__global__ void __launch_bounds__(256)
    w4_dequantize_kernel(const uint32_t* __restrict__ packed, const float* __restrict__ scales,
                         const int32_t* __restrict__ zeros, Out* __restrict__ out, int64_t N,
                         int64_t K, bool vector_ok) {
  const int64_t words = (K + 7) / 8;
  const int64_t groups = (K + 63) / 64;
  const int64_t word = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t row = blockIdx.y;
  if (word >= words) return;
  const uint32_t bits = packed[row * words + word];
  const float scale = scales[row * groups + (word >> 3)];
  const int zero = zeros[row * groups + (word >> 3)];
  float w[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    w[i] = __fmul_rn(static_cast<float>(static_cast<int>((bits >> (4 * i)) & 15u) - zero), scale);
  }
  Out* dst = out + row * K + word * 8;
  if (vector_ok) {  // K % 8 == 0 and an aligned base: every thread owns 16 or 32 aligned bytes
    if constexpr (sizeof(Out) == 2) {
      uint4 v;
      __half2 h;
      h = __floats2half2_rn(w[0], w[1]), v.x = *reinterpret_cast<uint32_t*>(&h);
      h = __floats2half2_rn(w[2], w[3]), v.y = *reinterpret_cast<uint32_t*>(&h);
      h = __floats2half2_rn(w[4], w[5]), v.z = *reinterpret_cast<uint32_t*>(&h);
      h = __floats2half2_rn(w[6], w[7]), v.w = *reinterpret_cast<uint32_t*>(&h);
      *reinterpret_cast<uint4*>(dst) = v;
    } else {
      reinterpret_cast<float4*>(dst)[0] = make_float4(w[0], w[1], w[2], w[3]);
      reinterpret_cast<float4*>(dst)[1] = make_float4(w[4], w[5], w[6], w[7]);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (word * 8 + i < K) {
        if constexpr (sizeof(Out) == 2) {
          dst[i] = __float2half_rn(w[i]);
        } else {
          dst[i] = w[i];
        }
      }
    }
  }
}

}  // namespace

cudaError_t launch_quantize(const void* weight, bool weight_is_fp32, int64_t N, int64_t K,
                            uint32_t* packed, float* scales, int32_t* zeros, cudaStream_t stream) {
  const int64_t groups = (K + 63) / 64;
  const int64_t items = N * ((groups + 1) / 2);
  const int64_t blocks = (items + kWarpsPerCta - 1) / kWarpsPerCta;
  if (blocks <= 0 || blocks > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
  const dim3 grid(static_cast<unsigned>(blocks));
  // 8- or 16-byte loads need every row to start on such a boundary.
  const size_t vector_bytes = weight_is_fp32 ? 16 : 8;
  const bool vector_ok = K % 4 == 0 && reinterpret_cast<uintptr_t>(weight) % vector_bytes == 0;
  if (weight_is_fp32) {
    w4_quantize_pack_kernel<float><<<grid, kWarpsPerCta * 32, 0, stream>>>(
        static_cast<const float*>(weight), packed, scales, zeros, N, K, vector_ok);
  } else {
    w4_quantize_pack_kernel<__half><<<grid, kWarpsPerCta * 32, 0, stream>>>(
        static_cast<const __half*>(weight), packed, scales, zeros, N, K, vector_ok);
  }
  return cudaGetLastError();
}

cudaError_t launch_dequantize(const uint32_t* packed, const float* scales, const int32_t* zeros,
                              void* out, bool out_is_fp32, int64_t N, int64_t K,
                              cudaStream_t stream) {
  const int64_t words = (K + 7) / 8;
  const int64_t groups = (K + 63) / 64;
  const int64_t blocks_x = (words + 255) / 256;
  if (N <= 0 || blocks_x > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
  const bool vector_ok = K % 8 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0;
  constexpr int64_t kRowsPerLaunch = 65535;  // limit of the grid's y extent
  for (int64_t r0 = 0; r0 < N; r0 += kRowsPerLaunch) {
    const int64_t rows = N - r0 < kRowsPerLaunch ? N - r0 : kRowsPerLaunch;
    const dim3 grid(static_cast<unsigned>(blocks_x), static_cast<unsigned>(rows));
    if (out_is_fp32) {
      w4_dequantize_kernel<float><<<grid, 256, 0, stream>>>(
          packed + r0 * words, scales + r0 * groups, zeros + r0 * groups,
          static_cast<float*>(out) + r0 * K, rows, K, vector_ok);
    } else {
      w4_dequantize_kernel<__half><<<grid, 256, 0, stream>>>(
          packed + r0 * words, scales + r0 * groups, zeros + r0 * groups,
          static_cast<__half*>(out) + r0 * K, rows, K, vector_ok);
    }
    const cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) return err;
  }
  return cudaSuccess;
}

}  // namespace lbl
