// Prefill W4A16 GEMM for sm_100a: TMA + in-kernel dequantisation + tcgen05 MMA with FP32
// accumulators in tensor memory.
//
//   Y[M,N] = fp16( X[M,K] . W^T ),   W[n,k] = fp16( float(q[n,k] - zero[n,k/64]) * scale[n,k/64] )
//
// The FP32 product rounded once to FP16 is the operand policy of the reference GEMM
// (csrc/cute_w4a16_gemm.cu:150-165) and is reproduced bit for bit.
//
// One CTA computes a 256 x 256 output tile as two 128 x 256 accumulators that fill the SM's
// 512 TMEM columns, walking K in blocks of 64 (one quantisation group) through a 3-stage ring:
//
//   warp 0      one thread issues a 2-D TMA load of the X block (256 rows x 64 columns, 128-byte
//               swizzle) per stage.
//   warps 2-9   thread r owns weight row n0 + r.  It prefetches 128 bytes of packed words and the
//               matching 4 scales / zero points straight from the reference layout into registers
//               (256 columns of K at a time), dequantises one group per stage and writes the 64
//               FP16 values as one 128-byte row of the K-major, 128-byte-swizzled B tile, then
//               fences the async proxy and arrives on the stage's barrier.
//   warp 1      one thread waits for both halves of a stage and issues 4 (K=16) x 2 (accumulator)
//               tcgen05.mma instructions, M=128, N=256; tcgen05.commit releases the stage.
//   warps 2-9   after the last commit: tcgen05.ld of the accumulators (each warp its 32-lane
//               quarter), FP32 -> FP16, 16-byte stores to Y with the M tail masked.
//
// Each weight is dequantised once per 256 rows of X, which keeps the CUDA-core work (about 3.6
// instructions per weight for the exact policy) under the tensor-core time of the tile.
// Every wait on an mbarrier is bounded; a timeout sets the device status word and the CTA drains.
// Shapes: N % 256 == 0 and K % 256 == 0; any M >= 1.  No cluster launch, no multicast.
#include "common.cuh"
#include "kernels.h"
#include "tensor_map.h"

namespace lbl {
namespace {

constexpr int kBM = 256;
constexpr int kBN = 256;
constexpr int kBK = 64;
constexpr int kStages = 3;
constexpr int kStageBytesA = kBM * kBK * 2;
constexpr int kStageBytesB = kBN * kBK * 2;
constexpr int kDequantWarps = 8;
constexpr int kThreads = 32 * (2 + kDequantWarps);
constexpr int kTmemCols = 512;
constexpr int kBarrierBytes = 256;
constexpr int kSmemBytes = kStages * (kStageBytesA + kStageBytesB) + kBarrierBytes + 1024;

struct Barriers {
  uint64_t a_full[kStages];
  uint64_t b_full[kStages];
  uint64_t empty[kStages];
  uint64_t acc_full;
  uint32_t tmem_base;
  int abort_flag;
};
static_assert(sizeof(Barriers) <= kBarrierBytes, "barrier block too large");

struct GemmParams {
  const uint32_t* packed;
  const float* scales;
  const int32_t* zeros;
  __half* y;
  int M, N, K;
  int m_tiles;
  int* status;
};

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
constexpr uint32_t kInstrDesc = (1u << 4) | ((kBN / 8) << 17) | ((128u / 16) << 24);

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

struct RowPrefetch {
  uint4 words[8];  // 32 packed words = 256 columns
  float4 scale;    // 4 groups
  int4 zero;
};

__device__ __forceinline__ void prefetch_row(RowPrefetch& buf, const uint32_t* packed_row,
                                             const float* scale_row, const int32_t* zero_row,
                                             int super_block) {
  const uint4* src = reinterpret_cast<const uint4*>(packed_row + super_block * 32);
#pragma unroll
  for (int i = 0; i < 8; ++i) buf.words[i] = __ldg(src + i);
  buf.scale = __ldg(reinterpret_cast<const float4*>(scale_row + super_block * 4));
  buf.zero = __ldg(reinterpret_cast<const int4*>(zero_row + super_block * 4));
}

__global__ void __launch_bounds__(kThreads, 1)
    w4a16_gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_x, const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  // The swizzled tiles need 1024-byte alignment.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + kStages * kStageBytesA;
  Barriers* bars = reinterpret_cast<Barriers*>(smem + kStages * (kStageBytesA + kStageBytesB));
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_tile = blockIdx.x / p.m_tiles;
  const int m_tile = blockIdx.x - n_tile * p.m_tiles;
  const int m0 = m_tile * kBM;
  const int n0 = n_tile * kBN;
  const int k_blocks = p.K / kBK;
  const int halves = (p.M - m0 > 128) ? 2 : 1;  // accumulators in use

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&bars->a_full[s], 1);
      mbar_init(&bars->b_full[s], kDequantWarps);
      mbar_init(&bars->empty[s], 1);
    }
    mbar_init(&bars->acc_full, 1);
    bars->abort_flag = 0;
    mbar_init_fence();
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&bars->tmem_base);

  if (warp == 0) {
    // ------------------------------- TMA producer (X blocks) ---------------------------------
    if (lane == 0) {
      for (int kb = 0; kb < k_blocks; ++kb) {
        const int s = kb % kStages;
        const int round = kb / kStages;
        if (round > 0) {
          mbar_wait_bounded(&bars->empty[s], (round - 1) & 1, abort_flag, p.status,
                            kStatusGemmWait + 1);
        }
        if (*abort_flag) break;
        mbar_arrive_expect_tx(&bars->a_full[s], kStageBytesA);
        tma_load_2d(smem_a + s * kStageBytesA, &tmap_x, kb * kBK, m0, &bars->a_full[s]);
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer ------------------------------------------------
    if (lane == 0) {
      for (int kb = 0; kb < k_blocks; ++kb) {
        const int s = kb % kStages;
        const int round = kb / kStages;
        mbar_wait_bounded(&bars->a_full[s], round & 1, abort_flag, p.status, kStatusGemmWait + 2);
        mbar_wait_bounded(&bars->b_full[s], round & 1, abort_flag, p.status, kStatusGemmWait + 3);
        if (*abort_flag) break;
        tc_fence_after_sync();
        const uint32_t a_addr = smem_addr(smem_a + s * kStageBytesA);
        const uint32_t b_addr = smem_addr(smem_b + s * kStageBytesB);
#pragma unroll
        for (int kk = 0; kk < kBK / 16; ++kk) {
          const uint64_t b_desc = smem_desc_k_major_sw128(b_addr + kk * 32);
          for (int h = 0; h < halves; ++h) {
            const uint64_t a_desc = smem_desc_k_major_sw128(a_addr + h * (128 * 128) + kk * 32);
            mma_f16(tmem_base + h * kBN, a_desc, b_desc, kInstrDesc, (kb | kk) != 0 ? 1u : 0u);
          }
        }
        mma_commit(&bars->empty[s]);  // frees the stage once these MMAs have read it
      }
      if (!*abort_flag) mma_commit(&bars->acc_full);
    }
  } else {
    // ------------------------------- dequantisation warps --------------------------------------
    const int row = (warp - 2) * 32 + lane;  // row of the B tile, 0..255
    const size_t n = static_cast<size_t>(n0 + row);
    const uint32_t* packed_row = p.packed + n * (p.K / 8);
    const float* scale_row = p.scales + n * (p.K / 64);
    const int32_t* zero_row = p.zeros + n * (p.K / 64);
    const uint32_t row_offset = (row >> 3) * 1024 + (row & 7) * 128;
    const uint32_t swz = row & 7;
    const int super_blocks = p.K / 256;

    RowPrefetch buf[2];
    prefetch_row(buf[0], packed_row, scale_row, zero_row, 0);

    auto run_super_block = [&](const RowPrefetch& cur, int sb) {
      const float sc[4] = {cur.scale.x, cur.scale.y, cur.scale.z, cur.scale.w};
      const int zp[4] = {cur.zero.x, cur.zero.y, cur.zero.z, cur.zero.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int kb = sb * 4 + j;
        const int s = kb % kStages;
        const int round = kb / kStages;
        if (round > 0) {
          mbar_wait_bounded(&bars->empty[s], (round - 1) & 1, abort_flag, p.status,
                            kStatusGemmWait + 4);
        }
        const GroupConstants group = group_constants(sc[j], zp[j]);
        uint8_t* dst = smem_b + s * kStageBytesB + row_offset;
        const uint4 wa = cur.words[2 * j];
        const uint4 wb = cur.words[2 * j + 1];
        const uint32_t w[8] = {wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w};
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint4 out = dequant_word(w[c], group);
          *reinterpret_cast<uint4*>(dst + ((static_cast<uint32_t>(c) ^ swz) << 4)) = out;
        }
        fence_async_proxy();  // generic-proxy writes -> visible to the tensor core's reads
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->b_full[s]);
      }
    };

    for (int sb = 0; sb < super_blocks; sb += 2) {
      if (sb + 1 < super_blocks) prefetch_row(buf[1], packed_row, scale_row, zero_row, sb + 1);
      run_super_block(buf[0], sb);
      if (sb + 1 < super_blocks) {
        if (sb + 2 < super_blocks) prefetch_row(buf[0], packed_row, scale_row, zero_row, sb + 2);
        run_super_block(buf[1], sb + 1);
      }
    }

    // ------------------------------- epilogue ---------------------------------------------------
    const bool ok = mbar_wait_bounded(&bars->acc_full, 0, abort_flag, p.status, kStatusGemmWait + 5);
    tc_fence_after_sync();
    const int quarter = warp & 3;        // TMEM lanes this warp may read
    const int h = (warp - 2) >> 2;       // accumulator handled by this warp
    if (ok && h < halves) {
      const int m = m0 + h * 128 + quarter * 32 + lane;
      __half* out_row = p.y + static_cast<size_t>(m < p.M ? m : 0) * p.N + n0;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + h * kBN;
      for (int c0 = 0; c0 < kBN; c0 += 32) {
        uint32_t v[32];
        tmem_load_32cols(taddr + c0, v);
        tmem_load_wait();
        if (m < p.M) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 o;
            __half2 h0 = __floats2half2_rn(__uint_as_float(v[8 * i + 0]), __uint_as_float(v[8 * i + 1]));
            __half2 h1 = __floats2half2_rn(__uint_as_float(v[8 * i + 2]), __uint_as_float(v[8 * i + 3]));
            __half2 h2 = __floats2half2_rn(__uint_as_float(v[8 * i + 4]), __uint_as_float(v[8 * i + 5]));
            __half2 h3 = __floats2half2_rn(__uint_as_float(v[8 * i + 6]), __uint_as_float(v[8 * i + 7]));
            o.x = *reinterpret_cast<uint32_t*>(&h0);
            o.y = *reinterpret_cast<uint32_t*>(&h1);
            o.z = *reinterpret_cast<uint32_t*>(&h2);
            o.w = *reinterpret_cast<uint32_t*>(&h3);
            *reinterpret_cast<uint4*>(out_row + c0 + 8 * i) = o;
          }
        }
      }
    }
  }

  if (*abort_flag) {
    // Give copies that are still in flight time to land before the shared memory is released.
    const long long start = clock64();
    while (clock64() - start < 200000) {
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace

bool gemm_tc_supports(int64_t M, int64_t N, int64_t K) {
  return M >= 1 && N >= kBN && N % kBN == 0 && K >= 256 && K % 256 == 0 && M <= (1 << 24) &&
         N <= (1 << 24) && K <= (1 << 24) && (N / kBN) * ((M + kBM - 1) / kBM) <= 0x7fffffffLL;
}

cudaError_t launch_gemm_tc(const Problem& p, int* status_word, cudaStream_t stream) {
  CUtensorMap tmap;
  const uint64_t dims[2] = {static_cast<uint64_t>(p.K), static_cast<uint64_t>(p.M)};
  const uint64_t strides[1] = {static_cast<uint64_t>(p.K) * sizeof(__half)};
  const uint32_t box[2] = {kBK, kBM};
  if (!encode_tensor_map(&tmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, p.x, dims, strides, box,
                         CU_TENSOR_MAP_SWIZZLE_128B)) {
    return cudaErrorInvalidValue;
  }

  static bool configured[64] = {};
  int device = 0;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess) return err;
  if (device < 0 || device >= 64 || !configured[device]) {
    err = cudaFuncSetAttribute(w4a16_gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               kSmemBytes);
    if (err != cudaSuccess) return err;
    if (device >= 0 && device < 64) configured[device] = true;
  }

  GemmParams gp;
  gp.packed = p.packed;
  gp.scales = p.scales;
  gp.zeros = p.zeros;
  gp.y = p.y;
  gp.M = static_cast<int>(p.M);
  gp.N = static_cast<int>(p.N);
  gp.K = static_cast<int>(p.K);
  gp.m_tiles = static_cast<int>((p.M + kBM - 1) / kBM);
  gp.status = status_word;
  const unsigned grid = static_cast<unsigned>((p.N / kBN) * gp.m_tiles);
  w4a16_gemm_tc_kernel<<<grid, kThreads, kSmemBytes, stream>>>(tmap, gp);
  return cudaGetLastError();
}

}  // namespace lbl
