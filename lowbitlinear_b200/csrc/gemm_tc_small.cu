// W4A16 GEMM for a few rows of activations (M <= 128) on sm_100a: the weights take the M side of
// the tcgen05 MMA.
//
//   Y[M,N] = fp16( X[M,K] . W^T ),   W[n,k] = fp16( float(q[n,k] - zero[n,k/64]) * scale[n,k/64] )
//
// (the operand policy of the reference GEMM, csrc/cute_w4a16_gemm.cu:150-165, bit for bit, as in
// gemm_tc.cu).  With 16 to 128 rows of X the 256 x 256 tiles of gemm_tc.cu leave most of the tensor
// core and most SMs idle and every CTA dequantises 256 rows of weights over the whole of K.  Here
// a CTA owns 128 weight rows and a slice of K and computes the transposed tile
//
//   D[128 weight rows, BT tokens] = W_tile[128, K slice] . X[BT, K slice]^T,   BT = M rounded up to 16
//
// with two or four accumulators of BT columns in tensor memory (the MMAs of a k-block alternate
// between them, the epilogue adds them); two CTAs share an SM.  K is cut into slices (whole super
// blocks of 256 columns) until the waves of two CTAs per SM are about full; slices of one row block
// meet as FP32 partial tiles in the scratch, and the CTA that draws the block's last ticket adds
// them in slice order and writes FP16 (same protocol as the split-K GEMV: bit-reproducible).
//
//   warp 0      one thread issues the 2-D TMA load of the X block (BT rows x 64 columns, 128-byte
//               swizzle, rows past M zero-filled) per stage.
//   warps 2-9   two threads per weight row: registers <- packed words and metadata of 256 columns
//               at a time, half a group each dequantised per stage into the row's 128 bytes of the
//               K-major, swizzled A tile (exact policy, tc_common.cuh).
//   warp 1      one thread issues 4 tcgen05.mma (M = 128, N = BT, K = 16) per stage.
//   warps 2-9   epilogue: tcgen05.ld of the accumulator, lane = weight row, so that for each token
//               a warp stores 32 neighbouring outputs.
//
// With programmatic dependent launch the weights are fetched and dequantised before the previous
// kernel in the stream has finished; the X loads, the outputs and the scratch wait for it.
// Every wait on an mbarrier is bounded.  Shapes: N % 128 == 0, K % 256 == 0, 1 <= M <= 128.
// No cluster launch, no multicast.
#include "kernels.h"
#include "tc_common.cuh"
#include "tensor_map.h"

#include <cstdlib>

namespace lbl {
namespace {

constexpr int kRowsW = 128;  // weight rows per CTA = M of the MMA
constexpr int kBK = 64;
constexpr int kStages = 3;
constexpr int kMaxTokens = 128;
constexpr int kStageBytesW = kRowsW * kBK * 2;      // 16 KB
constexpr int kStageBytesX = kMaxTokens * kBK * 2;  // 16 KB (BT * 128 bytes are used)
constexpr int kDequantWarps = 8;  // two threads per weight row, half a group each
constexpr int kThreads = 32 * (2 + kDequantWarps);
constexpr int kTmemCols = 256;  // accumulators of BT columns each; two CTAs share the 512 of an SM
constexpr int kBarrierBytes = 256;
constexpr int kSmemBytes = kStages * (kStageBytesW + kStageBytesX) + kBarrierBytes + 1024;
constexpr int kStatusSmallWait = 300;
constexpr int kMaxSlices = 8;  // the final addition keeps one 16-byte load per slice in flight

struct Barriers {
  uint64_t x_full[kStages];
  uint64_t w_full[kStages];
  uint64_t empty[kStages];
  uint64_t acc_full;
  uint32_t tmem_base;
  int abort_flag;
  int ticket;
};
static_assert(sizeof(Barriers) <= kBarrierBytes, "barrier block too large");

struct SmallParams {
  const uint32_t* packed;
  const float* scales;
  const int32_t* zeros;
  __half* y;
  int M, N, K;
  int tokens;    // BT: M rounded up to a multiple of 16
  int n_blocks;  // N / 128
  int slices;    // pieces of K per row block
  float* partials;  // [n_block][slice][M][128] FP32 when slices > 1
  int* tickets;     // one per row block
  int* status;
};

__global__ void __launch_bounds__(kThreads, 2)
    w4a16_gemm_tc_small_kernel(const __grid_constant__ CUtensorMap tmap_x, const SmallParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* smem_w = smem;
  uint8_t* smem_x = smem + kStages * kStageBytesW;
  Barriers* bars = reinterpret_cast<Barriers*>(smem + kStages * (kStageBytesW + kStageBytesX));
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // Slices of one row block are neighbours in the grid, so that they run at about the same time.
  const int n_block = blockIdx.x / p.slices;
  const int slice = blockIdx.x - n_block * p.slices;
  const int n0 = n_block * kRowsW;
  const int sb_total = p.K / 256;
  const int sb_begin = slice * sb_total / p.slices;
  const int sb_end = (slice + 1) * sb_total / p.slices;
  const int kb_begin = sb_begin * 4;
  const int k_blocks = (sb_end - sb_begin) * 4;
  const uint32_t idesc = instr_desc_f16(kRowsW, static_cast<uint32_t>(p.tokens));
  // The four MMAs of a k-block go to different accumulators where the tensor memory has room for
  // them: MMAs on one accumulator run one after the other, and with so few columns each of them
  // is nearly all latency.  The epilogue adds the accumulators.
  const int accumulators = p.tokens <= 64 ? 4 : 2;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&bars->x_full[s], 1);
      mbar_init(&bars->w_full[s], kDequantWarps);
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
  // Programmatic dependent launch (no-ops without it): the next kernel in the stream may start
  // as soon as it finds room; in this one only the activations, the outputs and the scratch
  // depend on the kernel before, so the weights are fetched and dequantised without waiting.
  pdl_allow_next_kernel();

  if (warp == 0) {
    // ------------------------------- TMA producer (X blocks) ---------------------------------
    if (lane == 0) {
      pdl_wait_for_previous_kernel();
      for (int kb = 0; kb < k_blocks; ++kb) {
        const int s = kb % kStages;
        const int round = kb / kStages;
        if (round > 0) {
          mbar_wait_bounded(&bars->empty[s], (round - 1) & 1, abort_flag, p.status, kStatusSmallWait + 1);
        }
        if (*abort_flag) break;
        mbar_arrive_expect_tx(&bars->x_full[s], static_cast<uint32_t>(p.tokens) * kBK * 2);
        tma_load_2d(smem_x + s * kStageBytesX, &tmap_x, (kb_begin + kb) * kBK, 0, &bars->x_full[s]);
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer ------------------------------------------------
    if (lane == 0) {
      for (int kb = 0; kb < k_blocks; ++kb) {
        const int s = kb % kStages;
        const int round = kb / kStages;
        mbar_wait_bounded(&bars->x_full[s], round & 1, abort_flag, p.status, kStatusSmallWait + 2);
        mbar_wait_bounded(&bars->w_full[s], round & 1, abort_flag, p.status, kStatusSmallWait + 3);
        if (*abort_flag) break;
        tc_fence_after_sync();
        const uint32_t w_addr = smem_addr(smem_w + s * kStageBytesW);
        const uint32_t x_addr = smem_addr(smem_x + s * kStageBytesX);
#pragma unroll
        for (int kk = 0; kk < kBK / 16; ++kk) {
          const int acc = kk & (accumulators - 1);
          mma_f16(tmem_base + static_cast<uint32_t>(acc * p.tokens),
                  smem_desc_k_major_sw128(w_addr + kk * 32), smem_desc_k_major_sw128(x_addr + kk * 32),
                  idesc, (kb > 0 || kk >= accumulators) ? 1u : 0u);
        }
        mma_commit(&bars->empty[s]);  // frees the stage once these MMAs have read it
      }
      if (!*abort_flag) mma_commit(&bars->acc_full);
    }
  } else {
    // ------------------------------- dequantisation warps --------------------------------------
    dequantise_rows<kStages, kStageBytesW>(p.packed, p.scales, p.zeros, p.K, static_cast<size_t>(n0),
                                           (warp - 2) * 32 + lane, sb_begin, sb_end, smem_w,
                                           bars->w_full, bars->empty, abort_flag, p.status,
                                           kStatusSmallWait + 4);

    // ------------------------------- epilogue ---------------------------------------------------
    const bool ok = mbar_wait_bounded(&bars->acc_full, 0, abort_flag, p.status, kStatusSmallWait + 5);
    tc_fence_after_sync();
    pdl_wait_for_previous_kernel();  // before the first write to Y or the scratch
    const int quarter = warp & 3;         // TMEM lanes this warp may read
    const int r = quarter * 32 + lane;    // weight row of the tile = TMEM lane
    const int pair = (warp - 2) >> 2;     // two warps share a quarter: even / odd 32-token chunks
    const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    // 32 token columns starting at c0, summed over the accumulators in a fixed order.  (A chunk may
    // reach past BT into the next accumulator's columns; those values belong to tokens >= M and
    // are never stored.)
    auto load_sum = [&](int c0, uint32_t (&v)[32]) {
      tmem_load_32cols(taddr + c0, v);
      tmem_load_wait();
      for (int a = 1; a < accumulators; ++a) {
        uint32_t w[32];
        tmem_load_32cols(taddr + a * p.tokens + c0, w);
        tmem_load_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) + __uint_as_float(w[i]));
      }
    };
    if (p.slices == 1) {
      if (ok) {
        __half* out = p.y + n0 + r;
        for (int c0 = 32 * pair; c0 < p.tokens; c0 += 64) {
          uint32_t v[32];
          load_sum(c0, v);
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int t = c0 + i;
            if (t < p.M) out[static_cast<size_t>(t) * p.N] = __float2half_rn(__uint_as_float(v[i]));
          }
        }
      }
    } else {
      // One slice of K: FP32 partial tile [token][weight row] to the scratch, then the ticket.
      float* block_partials = p.partials + static_cast<size_t>(n_block) * p.slices * p.M * kRowsW;
      if (ok) {
        float* dst = block_partials + static_cast<size_t>(slice) * p.M * kRowsW + r;
        for (int c0 = 32 * pair; c0 < p.tokens; c0 += 64) {
          uint32_t v[32];
          load_sum(c0, v);
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int t = c0 + i;
            if (t < p.M) dst[static_cast<size_t>(t) * kRowsW] = __uint_as_float(v[i]);
          }
        }
      }
      __threadfence();
      named_barrier(1, kDequantWarps * 32);
      if (threadIdx.x == 64) bars->ticket = atomicAdd(&p.tickets[n_block], 1);
      named_barrier(1, kDequantWarps * 32);
      if (bars->ticket == p.slices - 1) {
        __threadfence();
        // Last slice of this row block to arrive: add the partial tiles in slice order.  A thread
        // takes four neighbouring weight rows of one token at a time and has the loads of all
        // slices in flight together (16 bytes each); a warp covers the 128 rows of a token.
        const int quad = lane * 4;
        const int first_token = warp - 2;
        for (int t = first_token; t < p.M; t += kDequantWarps) {
          float4 part[kMaxSlices];
#pragma unroll
          for (int s = 0; s < kMaxSlices; ++s) {
            if (s < p.slices) {
              part[s] = __ldcg(reinterpret_cast<const float4*>(
                  block_partials + (static_cast<size_t>(s) * p.M + t) * kRowsW + quad));
            }
          }
          float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
          for (int s = 0; s < kMaxSlices; ++s) {
            if (s < p.slices) {
              v.x += part[s].x, v.y += part[s].y, v.z += part[s].z, v.w += part[s].w;
            }
          }
          const __half2 lo = __floats2half2_rn(v.x, v.y);
          const __half2 hi = __floats2half2_rn(v.z, v.w);
          uint2 o;
          o.x = *reinterpret_cast<const uint32_t*>(&lo);
          o.y = *reinterpret_cast<const uint32_t*>(&hi);
          *reinterpret_cast<uint2*>(p.y + static_cast<size_t>(t) * p.N + n0 + quad) = o;
        }
        if (threadIdx.x == 64) p.tickets[n_block] = 0;
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

// Slices of K per row block.  Two CTAs fit an SM, so the grid runs in waves of 2 * sm_count CTAs:
// among 1..kMaxSlices (at least two super blocks of K per slice) take the smallest count whose
// last wave is at least 90 % full, else the count with the fullest waves.
int small_slices(int64_t N, int64_t K, int sm_count) {
  const int64_t n_blocks = N / kRowsW;
  int64_t most = K / 256 / 2;
  if (most > kMaxSlices) most = kMaxSlices;
  if (most < 1) most = 1;
  const int64_t wave = 2 * static_cast<int64_t>(sm_count > 0 ? sm_count : 148);
  int best = 1;
  double best_fill = 0.0;
  for (int64_t s = 1; s <= most; ++s) {
    const int64_t ctas = n_blocks * s;
    const int64_t waves = (ctas + wave - 1) / wave;
    const double fill = static_cast<double>(ctas) / static_cast<double>(waves * wave);
    if (fill >= 0.9) return static_cast<int>(s);
    if (fill > best_fill) best_fill = fill, best = static_cast<int>(s);
  }
  return best;
}

}  // namespace

bool gemm_tc_small_supports(int64_t M, int64_t N, int64_t K) {
  return M >= 1 && M <= kMaxTokens && N >= kRowsW && N % kRowsW == 0 && K >= 256 && K % 256 == 0 &&
         N <= (1 << 24) && K <= (1 << 24);
}

size_t gemm_tc_small_workspace_bytes(int64_t M, int64_t N, int64_t K, int sm_count) {
  if (!gemm_tc_small_supports(M, N, K)) return 0;
  const int slices = small_slices(N, K, sm_count);
  if (slices == 1 || N / kRowsW > static_cast<int64_t>(kSkinnyTicketBytes / sizeof(int))) return 0;
  return kSkinnyTicketBytes + static_cast<size_t>(N / kRowsW) * slices * M * kRowsW * sizeof(float);
}

cudaError_t launch_gemm_tc_small(const Problem& p, int* status_word, cudaStream_t stream, void* workspace,
                                 size_t workspace_bytes, int sm_count, bool pdl) {
  const int tokens = static_cast<int>((p.M + 15) / 16 * 16);
  CUtensorMap tmap;
  const uint64_t dims[2] = {static_cast<uint64_t>(p.K), static_cast<uint64_t>(p.M)};
  const uint64_t strides[1] = {static_cast<uint64_t>(p.K) * sizeof(__half)};
  const uint32_t box[2] = {kBK, static_cast<uint32_t>(tokens)};
  if (!encode_tensor_map(&tmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, p.x, dims, strides, box,
                         CU_TENSOR_MAP_SWIZZLE_128B)) {
    return cudaErrorInvalidValue;
  }

  static bool configured[64] = {};
  int device = 0;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess) return err;
  if (device < 0 || device >= 64 || !configured[device]) {
    err = cudaFuncSetAttribute(w4a16_gemm_tc_small_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               kSmemBytes);
    if (err != cudaSuccess) return err;
    if (device >= 0 && device < 64) configured[device] = true;
  }

  SmallParams sp;
  sp.packed = p.packed;
  sp.scales = p.scales;
  sp.zeros = p.zeros;
  sp.y = p.y;
  sp.M = static_cast<int>(p.M);
  sp.N = static_cast<int>(p.N);
  sp.K = static_cast<int>(p.K);
  sp.tokens = tokens;
  sp.n_blocks = static_cast<int>(p.N / kRowsW);
  sp.slices = 1;
  sp.partials = nullptr;
  sp.tickets = nullptr;
  sp.status = status_word;
  // Slicing K needs the scratch (tickets + FP32 partial tiles); without it, one CTA per row block.
  const size_t need = gemm_tc_small_workspace_bytes(p.M, p.N, p.K, sm_count);
  if (need > 0 && workspace != nullptr && workspace_bytes >= need) {
    sp.slices = small_slices(p.N, p.K, sm_count);
    sp.tickets = static_cast<int*>(workspace);
    sp.partials = reinterpret_cast<float*>(static_cast<char*>(workspace) + kSkinnyTicketBytes);
  }
  const unsigned grid = static_cast<unsigned>(sp.n_blocks) * static_cast<unsigned>(sp.slices);
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
  return cudaLaunchKernelEx(&cfg, w4a16_gemm_tc_small_kernel, tmap, sp);
}

}  // namespace lbl
