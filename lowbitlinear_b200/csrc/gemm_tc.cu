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
//   warps 2-17  two threads own weight row n0 + r, half a group each.  A thread prefetches its 64
//               bytes of packed words and the row's 4 scales / zero points straight from the
//               reference layout into registers (256 columns of K at a time), dequantises its 32
//               weights of one group per stage into the row's 128 bytes of the K-major,
//               128-byte-swizzled B tile, then fences the async proxy and arrives on the stage's
//               barrier.  (Sixteen warps instead of eight: +6 % at M = 2048; the dequantisation
//               is latency-bound, not throughput-bound.)
//   warp 1      one thread waits for both halves of a stage and issues 4 (K=16) x 2 (accumulator)
//               tcgen05.mma instructions, M=128, N=256; tcgen05.commit releases the stage.
//   warps 2-17  after the last commit: tcgen05.ld of the accumulators (each warp a 32-lane
//               quarter of one accumulator and half of its columns), FP32 -> FP16, 16-byte stores
//               to Y with the M tail masked.
//
// Each weight is dequantised once per 256 rows of X (about 2.6 instructions per weight for the
// exact policy).
// Every wait on an mbarrier is bounded; a timeout sets the device status word and the CTA drains.
// With programmatic dependent launch the set-up and the weights of the first stages overlap the
// previous kernel in the stream; the X loads and the outputs wait for it -- unless the caller
// declares the call independent of that kernel (LBL_FLAG_INDEPENDENT), in which case nothing waits
// and this kernel's CTAs fill the SMs that the last, partial wave of the previous one leaves idle.
// Shapes: N % 256 == 0 and K % 256 == 0; any M >= 1.  No cluster launch, no multicast.
#include "kernels.h"
#include "tc_common.cuh"
#include "tensor_map.h"

namespace lbl {
namespace {

constexpr int kBM = 256;
constexpr int kBN = 256;
constexpr int kBK = 64;
constexpr int kStages = 3;
constexpr int kStageBytesA = kBM * kBK * 2;
constexpr int kStageBytesB = kBN * kBK * 2;
constexpr int kDequantWarps = 16;  // two threads per weight row, half a group each
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
  int wait_previous;  // programmatic dependent launch: wait for the previous kernel before touching X and Y
  int* status;
};

constexpr uint32_t kInstrDesc = instr_desc_f16(128, kBN);

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
  // Programmatic dependent launch (no-ops without it): the next kernel in the stream may set itself
  // up while this one runs; in this one only the activations and the outputs depend on the kernel
  // before, so the weights are fetched and dequantised without waiting.
  pdl_allow_next_kernel();

  if (warp == 0) {
    // ------------------------------- TMA producer (X blocks) ---------------------------------
    if (lane == 0) {
      if (p.wait_previous) pdl_wait_for_previous_kernel();
      for (int kb = 0; kb < k_blocks; ++kb) {
        const int s = kb % kStages;
        const int round = kb / kStages;
        if (round > 0) {
          mbar_wait_bounded(&bars->empty[s], (round - 1) & 1, abort_flag, p.status,
                            kStatusGemmWait + 1);
        }
        if (*abort_flag) break;
#ifdef LBL_TC_SKIP_TMA  // ablation switch
        mbar_arrive(&bars->a_full[s]);
#else
        mbar_arrive_expect_tx(&bars->a_full[s], kStageBytesA);
        tma_load_2d(smem_a + s * kStageBytesA, &tmap_x, kb * kBK, m0, &bars->a_full[s]);
#endif
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
#ifndef LBL_TC_SKIP_MMA  // ablation switch
            mma_f16(tmem_base + h * kBN, a_desc, b_desc, kInstrDesc, (kb | kk) != 0 ? 1u : 0u);
#endif
          }
        }
        mma_commit(&bars->empty[s]);  // frees the stage once these MMAs have read it
      }
      if (!*abort_flag) mma_commit(&bars->acc_full);
    }
  } else {
    // ------------------------------- dequantisation warps --------------------------------------
    dequantise_rows<kStages, kStageBytesB>(p.packed, p.scales, p.zeros, p.K, static_cast<size_t>(n0),
                                           (warp - 2) * 32 + lane, 0, p.K / 256, smem_b, bars->b_full,
                                           bars->empty, abort_flag, p.status, kStatusGemmWait + 4);

    // ------------------------------- epilogue ---------------------------------------------------
    const bool ok = mbar_wait_bounded(&bars->acc_full, 0, abort_flag, p.status, kStatusGemmWait + 5);
    tc_fence_after_sync();
    if (p.wait_previous) pdl_wait_for_previous_kernel();  // before the first write to Y
    const int quarter = warp & 3;        // TMEM lanes this warp may read
    const int h = ((warp - 2) >> 2) & 1;  // accumulator handled by this warp
    const int column_half = (warp - 2) >> 3;  // two warps share a quarter of an accumulator
    if (ok && h < halves) {
      const int m = m0 + h * 128 + quarter * 32 + lane;
      __half* out_row = p.y + static_cast<size_t>(m < p.M ? m : 0) * p.N + n0;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + h * kBN;
      for (int c0 = column_half * (kBN / 2); c0 < (column_half + 1) * (kBN / 2); c0 += 32) {
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

cudaError_t launch_gemm_tc(const Problem& p, int* status_word, cudaStream_t stream, bool pdl, bool independent) {
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
  gp.wait_previous = independent ? 0 : 1;
  const unsigned grid = static_cast<unsigned>((p.N / kBN) * gp.m_tiles);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, w4a16_gemm_tc_kernel, tmap, gp);
}

}  // namespace lbl
