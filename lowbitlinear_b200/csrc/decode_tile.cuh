// Device code shared by the decode GEMV kernels (M <= 2): the single-problem kernel in
// gemv_decode.cu and the grouped kernel in gemv_grouped.cu.  CTA roles, the shared-memory header,
// the activation operand and the arithmetic of one pipeline stage are the same in both; what
// differs is how a CTA finds its work.
#pragma once

#include "common.cuh"

#include <type_traits>

namespace lbl {
namespace decode {

constexpr int kRows = 16;
constexpr int kConsumerWarps = 8;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kProducerWarp = kConsumerWarps;     // one lane issues the copies
constexpr int kReducerWarp = kConsumerWarps + 1;  // adds the consumers' parts of each unit, writes y
constexpr int kThreads = kConsumerThreads + 64;
constexpr int kMaxSlots = 8;
constexpr int kHeaderBytes = 384;
constexpr int kRedBuffers = 8;  // unit results wait here for their reduction; see the unit loop

struct Header {
  uint64_t full[kMaxSlots];
  uint64_t empty[kMaxSlots];
  uint64_t red_full[kRedBuffers];   // all eight warps have deposited their part of a unit
  uint64_t red_empty[kRedBuffers];  // the reducer has read the buffer
  int abort_flag;
  int ticket;
  int pad[2];
  uint4 zeros[4];  // B operand of the lanes that feed no activation column
};
static_assert(sizeof(Header) <= kHeaderBytes, "header does not fit");

// Shared-memory loads by 32-bit address (volatile: they stay behind the barrier wait).
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(addr));
  return v;
}
// The same with a compile-time byte offset, which the load instruction carries itself (no address
// arithmetic per load).
template <int kOffset>
__device__ __forceinline__ uint4 lds128_at(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4+%5];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(addr), "n"(kOffset));
  return v;
}
template <int kOffset>
__device__ __forceinline__ float lds_f32_at(uint32_t addr) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1+%2];" : "=f"(v) : "r"(addr), "n"(kOffset));
  return v;
}
template <int kOffset>
__device__ __forceinline__ int lds_s32_at(uint32_t addr) {
  int v;
  asm volatile("ld.shared.s32 %0, [%1+%2];" : "=r"(v) : "r"(addr), "n"(kOffset));
  return v;
}
__device__ __forceinline__ float lds_f32(uint32_t addr) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ int lds_s32(uint32_t addr) {
  int v;
  asm volatile("ld.shared.s32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}

__device__ __forceinline__ uint32_t pack_half2(__half lo, __half hi) {
  return static_cast<uint32_t>(__half_as_ushort(lo)) |
         (static_cast<uint32_t>(__half_as_ushort(hi)) << 16);
}

// Activation operand of one K segment.  Word w of row m (columns 8w..8w+7) becomes the 16 bytes
//   (x0, x4) (x1, x5)/16 (x2, x6) (x3, x7)/16
// in the order the nibble extraction delivers the weights (odd nibbles carry a factor 16), at
// xf[m * words + w]; sx[group * 2 + m] is the FP32 sum of the group's 64 activations divided by
// kNibbleUnit.
__device__ __forceinline__ void build_activation_operand(const __half* x, int M, int K, int kseg,
                                                      int k_begin, uint4* xf, float* sx, int tid) {
  const int groups = kseg / 64;
  const int words_seg = kseg / 8;
  if (M < 2) {
    for (int i = tid; i < groups; i += kConsumerThreads) sx[2 * i + 1] = 0.0f;
  }
  const __half sixteenth = __float2half_rn(0.0625f);
  const int total = M * words_seg;  // multiple of 32, so a warp is never split by `idx < total`
  // The raw activations go straight to their place in shared memory with asynchronous 16-byte
  // copies, all issued before any is waited for: the operand costs one trip to the L2 however
  // long K is (register loads would be kept apart by the shuffles below, one trip per pass).
  // Each thread then rewrites, in place, the words it copied itself.
  for (int idx = tid; idx < total; idx += kConsumerThreads) {
    const int m = idx / words_seg;
    const int wd = idx - m * words_seg;
    const __half* src = x + static_cast<size_t>(m) * K + k_begin + wd * 8;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr(&xf[idx])), "l"(src)
                 : "memory");
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  for (int idx = tid; idx < total; idx += kConsumerThreads) {
    const int m = idx / words_seg;
    const int wd = idx - m * words_seg;
    const uint4 raw = xf[idx];
    const __half2 v01 = *reinterpret_cast<const __half2*>(&raw.x);
    const __half2 v23 = *reinterpret_cast<const __half2*>(&raw.y);
    const __half2 v45 = *reinterpret_cast<const __half2*>(&raw.z);
    const __half2 v67 = *reinterpret_cast<const __half2*>(&raw.w);
    const __half x0 = __low2half(v01), x1 = __high2half(v01);
    const __half x2 = __low2half(v23), x3 = __high2half(v23);
    const __half x4 = __low2half(v45), x5 = __high2half(v45);
    const __half x6 = __low2half(v67), x7 = __high2half(v67);
    float sum = ((__half2float(x0) + __half2float(x1)) + (__half2float(x2) + __half2float(x3))) +
                ((__half2float(x4) + __half2float(x5)) + (__half2float(x6) + __half2float(x7)));
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    sum += __shfl_xor_sync(0xffffffffu, sum, 4);
    uint4 out;
    out.x = pack_half2(x0, x4);
    out.y = pack_half2(__hmul(x1, sixteenth), __hmul(x5, sixteenth));
    out.z = pack_half2(x2, x6);
    out.w = pack_half2(__hmul(x3, sixteenth), __hmul(x7, sixteenth));
    xf[idx] = out;
    if ((wd & 7) == 0) sx[(wd >> 3) * 2 + m] = sum * (1.0f / kNibbleUnit);  // exact: a power of two
  }
}

// Arithmetic of one pipeline stage for one consumer warp, after the stage's `full` barrier has
// been passed: `slot_base` is the 32-bit shared address of the ring slot, `st` the stage's index
// within the unit (it selects the activations), `xf_addr` / `sx_base` this lane's base addresses
// into the activation operand and the per-group activation sums.  Adds into acc_a (row g) and
// acc_b (row g + 8).
__device__ __forceinline__ void consume_stage(uint32_t slot_base, int packed_pitch, int meta_pitch,
                                              int stage_k, int st, uint32_t xf_addr, uint32_t sx_base,
                                              int warp, int g, int t, int group_parity, bool feeds_b,
                                              uint4 (&xb)[4], float& acc_a, float& acc_b) {
  const int macro_per_stage = stage_k / 128;
  const int scales_block = kRows * packed_pitch;
  const float zero4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  // 32-bit shared-memory addresses of this lane's operands for macro tile `warp`; macro tile
  // warp + 8 u lies at a fixed distance from it.
  const uint32_t base = slot_base;
  const uint32_t wa_addr = base + g * packed_pitch + t * 16 + warp * 64;
  const uint32_t wb_addr = wa_addr + 8 * packed_pitch;
  const uint32_t meta_a = base + scales_block + g * meta_pitch + (2 * warp + group_parity) * 4;
  const uint32_t meta_b = meta_a + 8 * meta_pitch;
  const uint32_t zero_delta = static_cast<uint32_t>(kRows * meta_pitch);  // scales -> zero points
  const uint32_t xb_addr = xf_addr + static_cast<uint32_t>(st * (stage_k / 8) + warp * 16) * 16;
  const uint32_t sx_addr = sx_base + static_cast<uint32_t>(st * (stage_k / 64) + 2 * warp) * 8;

  const uint32_t zmeta_a = meta_a + zero_delta;
  const uint32_t zmeta_b = meta_b + zero_delta;
  // Arithmetic of one macro tile (16 rows x 128 columns) once its operands are in registers.
  auto consume = [&](const uint4& wa, const uint4& wb, float scale_a, float scale_b, float zero_a,
                     float zero_b, float sum_x) {
    const uint32_t words_a[4] = {wa.x, wa.y, wa.z, wa.w};
    const uint32_t words_b[4] = {wb.x, wb.y, wb.z, wb.w};
    // One chain of eight MMAs: the nibble extraction of the next word is independent of it
    // and the other warps of the scheduler fill the rest of the latency.
    float d[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint32_t qa[4], qb[4];
      nibbles_as_subnormal_half2(words_a[i], qa);
      nibbles_as_subnormal_half2(words_b[i], qb);
      const uint32_t a0[4] = {qa[0], qb[0], qa[1], qb[1]};
      const uint32_t a1[4] = {qa[2], qb[2], qa[3], qb[3]};
      if (i == 0) {
        mma_m16n8k16(d, a0, xb[i].x, xb[i].y, zero4);
      } else {
        mma_m16n8k16(d, a0, xb[i].x, xb[i].y, d);
      }
      mma_m16n8k16(d, a1, xb[i].z, xb[i].w, d);
    }
    // acc += scale * unit * (sum q x - zero * sum x / unit): the MMA result carries the factor
    // 1 / kNibbleUnit of the nibble encoding, and sx holds sum x already divided by it.
    const float qx_a = d[0] + d[1];
    const float qx_b = d[2] + d[3];
    acc_a = fmaf(scale_a * kNibbleUnit, fmaf(-zero_a, sum_x, qx_a), acc_a);
    acc_b = fmaf(scale_b * kNibbleUnit, fmaf(-zero_b, sum_x, qx_b), acc_b);
  };
  // Macro tile `warp + 8 u` of the stage; with u known at compile time every load is
  // base register + immediate.
  auto macro_tile_at = [&](auto u_const) {
    constexpr int u = decltype(u_const)::value;
    const uint4 wa = lds128_at<u * 512>(wa_addr);
    const uint4 wb = lds128_at<u * 512>(wb_addr);
    if (feeds_b) {
      xb[0] = lds128_at<u * 2048>(xb_addr);
      xb[1] = lds128_at<u * 2048 + 16>(xb_addr);
      xb[2] = lds128_at<u * 2048 + 32>(xb_addr);
      xb[3] = lds128_at<u * 2048 + 48>(xb_addr);
    }
    const float scale_a = lds_f32_at<u * 64>(meta_a);
    const float scale_b = lds_f32_at<u * 64>(meta_b);
    const float zero_a = static_cast<float>(lds_s32_at<u * 64>(zmeta_a));
    const float zero_b = static_cast<float>(lds_s32_at<u * 64>(zmeta_b));
    const float sum_x = lds_f32_at<u * 128>(sx_addr);
    consume(wa, wb, scale_a, scale_b, zero_a, zero_b, sum_x);
  };
  auto macro_tile = [&](int u) {
    const uint4 wa = lds128(wa_addr + u * 512);
    const uint4 wb = lds128(wb_addr + u * 512);
    if (feeds_b) {
#pragma unroll
      for (int i = 0; i < 4; ++i) xb[i] = lds128(xb_addr + u * 2048 + i * 16);
    }
    const float scale_a = lds_f32(meta_a + u * 64);
    const float scale_b = lds_f32(meta_b + u * 64);
    const float zero_a = static_cast<float>(lds_s32(zmeta_a + u * 64));
    const float zero_b = static_cast<float>(lds_s32(zmeta_b + u * 64));
    const float sum_x = lds_f32(sx_addr + u * 128);
    consume(wa, wb, scale_a, scale_b, zero_a, zero_b, sum_x);
  };
  if (macro_per_stage == 16) {  // stage of 2048 columns: two macro tiles per warp
    macro_tile_at(std::integral_constant<int, 0>{});
    macro_tile_at(std::integral_constant<int, 1>{});
  } else if (macro_per_stage == 8) {
    macro_tile_at(std::integral_constant<int, 0>{});
  } else {
    for (int u = 0; warp + 8 * u < macro_per_stage; ++u) macro_tile(u);
  }
}

}  // namespace decode
}  // namespace lbl
