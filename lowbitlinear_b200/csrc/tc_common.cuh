// tcgen05 / TMEM wrappers and the exact dequantisation shared by the tensor-core kernels
// (gemm_tc.cu, gemm_tc_small.cu).
#pragma once

#include "common.cuh"

namespace lbl {
namespace {

// ---- tcgen05 / TMA wrappers -------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_addr(smem_result)),
               "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void fence_async_proxy() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
// Arrives once on `bar` when every MMA issued so far by this thread has finished.
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_addr(bar))
               : "memory");
}
__device__ __forceinline__ void mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                        uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes (64 FP16) with the
// 128-byte swizzle: 8-row atoms of 1024 bytes follow each other (stride byte offset 1024), the
// leading byte offset is unused for swizzled K-major tiles (encoded 1), version 1 (sm_100),
// layout type 2 (SWIZZLE_128B).  Addresses and offsets are in 16-byte units.
__device__ __forceinline__ uint64_t smem_desc_k_major_sw128(uint32_t byte_addr) {
  const uint32_t lo = ((byte_addr >> 4) & 0x3FFFu) | (1u << 16);
  const uint32_t hi = (1024u >> 4) | (1u << 14) | (2u << 29);
  return (static_cast<uint64_t>(hi) << 32) | lo;
}

// Instruction descriptor, kind::f16: D = F32 (bits 4-5 = 1), A = B = F16 (0), both K-major (0),
// N / 8 at bits 17-22, M / 16 at bits 24-28.
__host__ __device__ constexpr uint32_t instr_desc_f16(uint32_t m, uint32_t n) {
  return (1u << 4) | ((n / 8) << 17) | ((m / 16) << 24);
}

__device__ __forceinline__ void tmem_load_32cols(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
        "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
        "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]),
        "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
        "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_load_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ---- dequantisation of one packed word into eight FP16 weights in column order ----------------
// A nibble masked in place and OR-ed into the mantissa of 2^23 is the float 2^23 + 16^i q (i = its
// position in the 16-bit half of the word), with one LOP3 and no shift; subtracting 2^23 + 16^i z
// leaves 16^i (q - z) exactly, and the product with 16^-i scale has exactly the bits of
// float(q - z) * scale, since both factors only moved by a power of two.  It is rounded to FP32 and
// then once to FP16, as the reference does.  Additions and multiplications are packed pairs.
struct GroupConstants {
  float2 neg_c01, neg_c23;  // -(2^23 + 16^i zero), i = 0..3
  float2 s01, s23;          // 16^-i scale
};

__device__ __forceinline__ GroupConstants group_constants(float scale, int zero) {
  const float z = static_cast<float>(zero);
  GroupConstants g;
  g.neg_c01 = make_float2(-(8388608.0f + z), -(8388608.0f + 16.0f * z));
  g.neg_c23 = make_float2(-(8388608.0f + 256.0f * z), -(8388608.0f + 4096.0f * z));
  g.s01 = make_float2(scale, scale * 0.0625f);
  g.s23 = make_float2(scale * 0.00390625f, scale * 0.000244140625f);
  return g;
}

__device__ __forceinline__ uint32_t two_weights(uint32_t bits, uint32_t mask_a, uint32_t mask_b,
                                                float2 neg_c, float2 s) {
  const float2 f = make_float2(__uint_as_float((bits & mask_a) | 0x4B000000u),
                               __uint_as_float((bits & mask_b) | 0x4B000000u));
  const float2 w = __fmul2_rn(__fadd2_rn(f, neg_c), s);
  const __half2 h = __floats2half2_rn(w.x, w.y);
  return *reinterpret_cast<const uint32_t*>(&h);
}

__device__ __forceinline__ uint4 dequant_word(uint32_t word, const GroupConstants& g) {
  const uint32_t hi = word >> 16;
  uint4 out;
  out.x = two_weights(word, 0x000Fu, 0x00F0u, g.neg_c01, g.s01);
  out.y = two_weights(word, 0x0F00u, 0xF000u, g.neg_c23, g.s23);
  out.z = two_weights(hi, 0x000Fu, 0x00F0u, g.neg_c01, g.s01);
  out.w = two_weights(hi, 0x0F00u, 0xF000u, g.neg_c23, g.s23);
  return out;
}

// ---- the dequantisation worker shared by the tensor-core kernels ------------------------------
// Two or four threads own one weight row of the K-major, 128-byte-swizzled tile.  A thread keeps
// its packed words of two super blocks (256 columns: four groups) and the row's metadata in
// registers, one super block being consumed while the next is in flight.
// Registers that hold a thread's share of one super block (256 columns: four groups) of its row:
// kWords packed words of each of the four k-blocks, and the row's metadata.
template <int kWords>
struct RowPrefetch {
  uint32_t words[4][kWords];
  float4 scale;
  int4 zero;
};

// Walks super blocks [sb_begin, sb_end) of weight row `n`.  kThreadsPerRow (2 or 4) threads own one
// weight row of the K-major, 128-byte-swizzled tile, 32 or 16 columns of every k-block each.  For
// its j-th k-block (one group) a thread waits until ring stage j % kStages is free, writes its
// dequantised weights into the stage's tile at `tiles + stage * kStageBytes`, fences the async
// proxy and arrives (one arrival per warp) on full[stage].  `worker` is the thread's index among
// the dequantisation threads (row = worker / kThreadsPerRow); `status_code` is reported if a wait
// on `empty` expires.  With `full_cluster_base` != 0 the arrival goes to that shared::cluster
// address + 8 * stage instead (the barrier of the first CTA of a pair), with release semantics at
// cluster scope.
template <int kStages, int kStageBytes, int kThreadsPerRow = 2>
__device__ __forceinline__ void dequantise_rows(const uint32_t* packed, const float* scales,
                                                const int32_t* zeros, int K, size_t n0, int worker,
                                                int sb_begin, int sb_end, uint8_t* tiles,
                                                uint64_t* full, uint64_t* empty,
                                                volatile int* abort_flag, int* status, int status_code,
                                                uint32_t full_cluster_base = 0) {
  static_assert(kThreadsPerRow == 2 || kThreadsPerRow == 4, "two or four threads per weight row");
  constexpr int kWords = 8 / kThreadsPerRow;  // packed words per thread and k-block
  const int lane = threadIdx.x & 31;
  const int row = worker / kThreadsPerRow;
  const int part = worker % kThreadsPerRow;
  const size_t n = n0 + row;
  const uint32_t* packed_row = packed + n * (K / 8) + part * kWords;
  const float* scale_row = scales + n * (K / 64);
  const int32_t* zero_row = zeros + n * (K / 64);
  const uint32_t row_offset = (row >> 3) * 1024 + (row & 7) * 128;
  const uint32_t swz = row & 7;

  auto prefetch = [&](RowPrefetch<kWords>& buf, int super_block) {
#ifdef LBL_TC_SKIP_DEQUANT
    return;
#endif
    const uint32_t* src = packed_row + super_block * 32;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if constexpr (kWords == 4) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(src + j * 8));
        buf.words[j][0] = v.x, buf.words[j][1] = v.y, buf.words[j][2] = v.z, buf.words[j][3] = v.w;
      } else {
        const uint2 v = __ldg(reinterpret_cast<const uint2*>(src + j * 8));
        buf.words[j][0] = v.x, buf.words[j][1] = v.y;
      }
    }
    buf.scale = __ldg(reinterpret_cast<const float4*>(scale_row + super_block * 4));
    buf.zero = __ldg(reinterpret_cast<const int4*>(zero_row + super_block * 4));
  };
  // `sb` counts this CTA's super blocks from 0; the data come from super block sb_begin + sb.
  auto run_super_block = [&](const RowPrefetch<kWords>& cur, int sb) {
    const float sc[4] = {cur.scale.x, cur.scale.y, cur.scale.z, cur.scale.w};
    const int zp[4] = {cur.zero.x, cur.zero.y, cur.zero.z, cur.zero.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int kb = sb * 4 + j;
      const int s = kb % kStages;
      const int round = kb / kStages;
      if (round > 0) mbar_wait_bounded(&empty[s], (round - 1) & 1, abort_flag, status, status_code);
#ifndef LBL_TC_SKIP_DEQUANT  // ablation switch: the warps only hand the stages on
      const GroupConstants group = group_constants(sc[j], zp[j]);
      uint8_t* dst = tiles + s * kStageBytes + row_offset;
#pragma unroll
      for (int c = 0; c < kWords; ++c) {
#ifdef LBL_TC_NO_ARITHMETIC  // ablation switch: loads and stores, no arithmetic
        const uint4 out = make_uint4(cur.words[j][c], cur.words[j][c] >> 4, __float_as_uint(group.s01.x),
                                     __float_as_uint(group.neg_c01.x));
#else
        const uint4 out = dequant_word(cur.words[j][c], group);
#endif
        *reinterpret_cast<uint4*>(dst + ((static_cast<uint32_t>(part * kWords + c) ^ swz) << 4)) = out;
      }
#endif
      fence_async_proxy();  // generic-proxy writes -> visible to the tensor core's reads
      __syncwarp();
      if (lane == 0) {
        if (full_cluster_base != 0) {
          asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(
                           full_cluster_base + 8u * static_cast<uint32_t>(s))
                       : "memory");
        } else {
          mbar_arrive(&full[s]);
        }
      }
    }
  };

  const int super_blocks = sb_end - sb_begin;
  RowPrefetch<kWords> buf[2];
  prefetch(buf[0], sb_begin);
  for (int sb = 0; sb < super_blocks; sb += 2) {
    if (sb + 1 < super_blocks) prefetch(buf[1], sb_begin + sb + 1);
    run_super_block(buf[0], sb);
    if (sb + 1 < super_blocks) {
      if (sb + 2 < super_blocks) prefetch(buf[0], sb_begin + sb + 2);
      run_super_block(buf[1], sb + 1);
    }
  }
}

}  // namespace
}  // namespace lbl
