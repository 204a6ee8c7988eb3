// Prefill W4A16 GEMM for sm_100a on pairs of SMs: TMA + in-kernel dequantisation + tcgen05 MMA
// across two CTAs (cta_group::2), FP32 accumulators in tensor memory.
//
//   Y[M,N] = fp16( X[M,K] . W^T ),   W[n,k] = fp16( float(q[n,k] - zero[n,k/64]) * scale[n,k/64] )
//
// Same operand policy (csrc/cute_w4a16_gemm.cu:150-165 of the reference, bit for bit) and the same
// roles as gemm_tc.cu.  What changes is who dequantises what.  Ablations of that kernel show two
// costs of equal size that overlap badly: the tensor pipe (a tcgen05.mma of M = 128, K = 16 takes
// about 200 cycles) and the exact dequantisation of the 256 weight rows of every 256 x 256 tile
// (0.75 us per 64-column block, as long as the block's eight MMAs).  Here two CTAs of a cluster
// share a 512 (tokens) x 256 (weight rows) tile and ONE dequantised copy of its weights:
//
//   * each CTA dequantises only 128 of the 256 weight rows of a k-block (half the work per flop)
//     into its shared memory; tcgen05.mma.cta_group::2 reads the B operand from both CTAs, 128
//     rows from each (N = 256);
//   * each CTA loads the X blocks of ITS 256 token rows (two groups of 128) and holds their
//     accumulators: M = 256 of a pair MMA is 128 token rows per CTA, two pair MMAs per 16 columns
//     of K (one per token group), 512 columns of tensor memory per CTA as before;
//   * per k-block a CTA holds 32 KB of X and 16 KB of weights, in two rings of four stages each
//     (gemm_tc.cu has room for three).
//
// Synchronisation across the pair: each CTA tracks its own copies and warps on its own barriers;
// one thread of the second CTA reports each finished k-block to the first CTA with a single remote
// arrival (shared::cluster address), one thread of the first CTA issues the MMAs, and
// tcgen05.commit in its cluster-wide form releases a stage (and announces the finished
// accumulators) in both CTAs.  Each CTA issues its own copies, each with one destination.  Every
// wait on an mbarrier is bounded; the pair meets at a cluster barrier before it releases tensor
// memory.  Shapes: N % 256 == 0 and K % 256 == 0; any M >= 1.
#include "kernels.h"
#include "tc_common.cuh"
#include "tensor_map.h"

namespace lbl {
namespace {

constexpr int kTokensGroup = 128;  // token rows of one accumulator = its lanes
constexpr int kTokensCta = 256;    // two groups per CTA
constexpr int kTokensPair = 512;
constexpr int kRowsCta = 128;      // weight rows a CTA dequantises: its half of the pair's 256
constexpr int kNPair = 256;        // weight rows (output columns) of a pair's tile
constexpr int kBK = 64;
#ifndef LBL_PAIR_STAGES_A
#define LBL_PAIR_STAGES_A 4
#endif
#ifndef LBL_PAIR_STAGES_B
#define LBL_PAIR_STAGES_B 4
#endif
// Two rings, X blocks (32 KB a stage) and dequantised weights (16 KB a stage), each with its own
// barriers so that their depths can differ.  Measured at M = 2048 on Gate/Up: 4 + 4 stages 457 us,
// 3 + 6 stages 473, 2 + 8 stages 466: the depth of the weight ring is not what bounds the kernel.
constexpr int kStagesA = LBL_PAIR_STAGES_A;
constexpr int kStagesB = LBL_PAIR_STAGES_B;
constexpr int kStageBytesA = kTokensCta * kBK * 2;  // 32 KB: two 16 KB groups
constexpr int kStageBytesB = kRowsCta * kBK * 2;    // 16 KB
#ifndef LBL_PAIR_THREADS_PER_ROW
#define LBL_PAIR_THREADS_PER_ROW 2
#endif
constexpr int kThreadsPerRow = LBL_PAIR_THREADS_PER_ROW;  // 2 or 4 (four measured 2 % slower)
constexpr int kDequantWarps = kRowsCta * kThreadsPerRow / 32;
constexpr int kThreads = 32 * (2 + kDequantWarps);
constexpr int kTmemCols = 512;
constexpr int kBarrierBytes = 256;
constexpr int kSmemBytes = kStagesA * kStageBytesA + kStagesB * kStageBytesB + kBarrierBytes + 1024;
constexpr int kStatusPairWait = 500;
// The epilogue stages the CTA's FP16 tile (256 token rows x 256 columns) in the rings' memory;
// 16 bytes of padding per row keep the lanes' 16-byte stores on different banks.
constexpr int kOutPitch = kNPair * 2 + 16;
static_assert(kTokensCta * kOutPitch <= kStagesA * kStageBytesA + kStagesB * kStageBytesB, "tile does not fit the rings");

constexpr int kRelaySlots = 4;
constexpr int kMaxScatterRanks = 8;
struct Barriers {
  uint64_t a_full[kStagesA];   // this CTA's X blocks have landed
  uint64_t a_empty[kStagesA];  // the MMAs have read the X stage (cluster-wide commit)
  uint64_t b_full[kStagesB];   // this CTA's warps have dequantised their rows
  uint64_t b_empty[kStagesB];  // the MMAs have read the weight stage (cluster-wide commit)
  uint64_t peer_ready[kRelaySlots];  // first CTA's: the second CTA's k-block is complete
  uint64_t acc_full;         // each CTA's own
  uint32_t tmem_base;
  int abort_flag;
};
static_assert(sizeof(Barriers) <= kBarrierBytes, "barrier block too large");

struct PairParams {
  const uint32_t* packed;
  const float* scales;
  const int32_t* zeros;
  __half* y;
  int M, N, K;
  int m_tiles;  // ceil(M / 512)
  int wait_previous;  // programmatic dependent launch: wait for the previous kernel before touching X and Y
  int* status;
  // Tensor-parallel K split: instead of y, the tile goes to the rank that owns its columns --
  // scatter[o] is this rank's slot [M, owner_cols] in the exchange buffer of rank o (peer memory
  // for o != this rank), written with plain 16-byte stores over NVLink as each tile finishes.
  __half* scatter[kMaxScatterRanks];
  int owner_cols;  // 0: no scatter
};

constexpr uint32_t kInstrDescPair = instr_desc_f16(256, 256);

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of `addr` (a shared::cta address of this CTA) in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(addr), "r"(rank));
  return out;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_result, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(smem_result)),
               "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void mma_f16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on the barrier at this shared-memory offset in both CTAs of the pair once every MMA
// issued so far has finished.
__device__ __forceinline__ void mma_commit_pair(uint64_t* bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
          smem_addr(bar)),
      "h"(static_cast<uint16_t>(3))
      : "memory");
}
// Bounded wait with acquire semantics at cluster scope (the other CTA's arrivals order its writes).
__device__ __forceinline__ bool mbar_wait_cluster_bounded(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                                          int* status_word, int status_code) {
  const long long start = clock64();
  while (true) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(smem_addr(bar)), "r"(parity)
        : "memory");
    if (done) return true;
    if (*abort_flag) return false;
    if (clock64() - start > kWaitLimitCycles) {
      *abort_flag = 1;
      atomicCAS(status_word, 0, status_code);
      return false;
    }
  }
}

__global__ void __launch_bounds__(kThreads, 1)
    w4a16_gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap tmap_x, const PairParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + kStagesA * kStageBytesA;
  Barriers* bars = reinterpret_cast<Barriers*>(smem + kStagesA * kStageBytesA + kStagesB * kStageBytesB);
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0: issues the MMAs and owns the full barriers
  const int pair = blockIdx.x >> 1;
  const int n_pair = pair / p.m_tiles;
  const int m_tile = pair - n_pair * p.m_tiles;
  // Token group g of this CTA is rows m0 + g * 256 .. + 128: the pair MMA g spans 256 consecutive
  // tokens, 128 from each CTA.
  const int m0 = m_tile * kTokensPair + static_cast<int>(rank) * kTokensGroup;
  const int n0 = n_pair * kNPair;
  const int k_blocks = p.K / kBK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStagesA; ++s) {
      mbar_init(&bars->a_full[s], 1);
      mbar_init(&bars->a_empty[s], 1);
    }
    for (int s = 0; s < kStagesB; ++s) {
      mbar_init(&bars->b_full[s], kDequantWarps);
      mbar_init(&bars->b_empty[s], 1);
    }
    for (int s = 0; s < kRelaySlots; ++s) mbar_init(&bars->peer_ready[s], 1);
    mbar_init(&bars->acc_full, 1);
    bars->abort_flag = 0;
    mbar_init_fence();
  }
  if (warp == 1) {
    tmem_alloc_pair(&bars->tmem_base, kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  // Both CTAs' barriers exist and both allocations are done before anybody signals across.
  cluster_sync_all();
  tc_fence_after_sync();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&bars->tmem_base);
  const uint32_t peer_ready_leader = map_to_cta(smem_addr(&bars->peer_ready[0]), 0);
  // Programmatic dependent launch (no-ops without it): the next kernel in the stream may start as
  // soon as every CTA of this one is running.  Weights never depend on the previous kernel; X and Y
  // wait for it unless the caller has declared this call independent of it, and then this kernel's
  // pairs fill the SMs that the previous kernel's last, partial wave leaves idle.
  pdl_allow_next_kernel();

  if (warp == 0) {
    // ------------------------------- TMA producer (this CTA's X rows) ---------------------------
    if (lane == 0) {
      if (p.wait_previous) pdl_wait_for_previous_kernel();
      for (int kb = 0; kb < k_blocks; ++kb) {
        const int s = kb % kStagesA;
        const int round = kb / kStagesA;
        if (round > 0) {
          mbar_wait_bounded(&bars->a_empty[s], (round - 1) & 1, abort_flag, p.status, kStatusPairWait + 1);
        }
        if (*abort_flag) break;
#ifdef LBL_TC_SKIP_TMA  // ablation switch: the stage is handed on without its copies
        mbar_arrive(&bars->a_full[s]);
#else
        mbar_arrive_expect_tx(&bars->a_full[s], kStageBytesA);
        for (int g = 0; g < 2; ++g) {
          tma_load_2d(smem_a + s * kStageBytesA + g * (kStageBytesA / 2), &tmap_x, kb * kBK, m0 + g * 256,
                      &bars->a_full[s]);
        }
#endif
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer (first CTA) / relay (second CTA) ----------------
    // All signalling across the pair goes through one thread per CTA: the second CTA's thread waits
    // for its own copies and warps and makes ONE remote arrival per k-block (eight remote arrivals
    // and a remote completion per copy were measured at 0.8 us per k-block with nothing else running).
    if (lane == 0 && rank == 1) {
      for (int kb = 0; kb < k_blocks; ++kb) {
        const int s = kb % kStagesA;
        const int sb = kb % kStagesB;
        mbar_wait_bounded(&bars->a_full[s], (kb / kStagesA) & 1, abort_flag, p.status, kStatusPairWait + 6);
        mbar_wait_bounded(&bars->b_full[sb], (kb / kStagesB) & 1, abort_flag, p.status, kStatusPairWait + 7);
        if (*abort_flag) break;
        asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(
                         peer_ready_leader + 8u * static_cast<uint32_t>(kb % kRelaySlots))
                     : "memory");
      }
    }
    if (lane == 0 && rank == 0) {
      for (int kb = 0; kb < k_blocks; ++kb) {
        const int s = kb % kStagesA;
        const int sb = kb % kStagesB;
        mbar_wait_bounded(&bars->a_full[s], (kb / kStagesA) & 1, abort_flag, p.status, kStatusPairWait + 2);
        mbar_wait_bounded(&bars->b_full[sb], (kb / kStagesB) & 1, abort_flag, p.status, kStatusPairWait + 3);
        mbar_wait_cluster_bounded(&bars->peer_ready[kb % kRelaySlots], (kb / kRelaySlots) & 1, abort_flag, p.status,
                                  kStatusPairWait + 8);
        if (*abort_flag) break;
        tc_fence_after_sync();
        const uint32_t a_addr = smem_addr(smem_a + s * kStageBytesA);
        const uint32_t b_addr = smem_addr(smem_b + sb * kStageBytesB);
#pragma unroll
        for (int kk = 0; kk < kBK / 16; ++kk) {
          const uint64_t b_desc = smem_desc_k_major_sw128(b_addr + kk * 32);
#pragma unroll
          for (int g = 0; g < 2; ++g) {
            const uint64_t a_desc = smem_desc_k_major_sw128(a_addr + g * (kStageBytesA / 2) + kk * 32);
#ifndef LBL_TC_SKIP_MMA  // ablation switch
            mma_f16_pair(tmem_base + g * 256, a_desc, b_desc, kInstrDescPair, (kb | kk) != 0 ? 1u : 0u);
#endif
          }
        }
        mma_commit_pair(&bars->a_empty[s]);   // frees the X stage in both CTAs
        mma_commit_pair(&bars->b_empty[sb]);  // and the weight stage
      }
      if (!*abort_flag) mma_commit_pair(&bars->acc_full);
    }
  } else {
    // ------------------------------- dequantisation warps --------------------------------------
    // This CTA's half of the pair's 256 weight rows: B columns rank * 128 .. + 128 of every MMA.
    dequantise_rows<kStagesB, kStageBytesB, kThreadsPerRow>(p.packed, p.scales, p.zeros, p.K,
                                           static_cast<size_t>(n0) + rank * 128, (warp - 2) * 32 + lane, 0,
                                           p.K / 256, smem_b, bars->b_full, bars->b_empty, abort_flag, p.status,
                                           kStatusPairWait + 4);

    // ------------------------------- epilogue ---------------------------------------------------
    const bool ok = mbar_wait_bounded(&bars->acc_full, 0, abort_flag, p.status, kStatusPairWait + 5);
    tc_fence_after_sync();
    if (p.wait_previous) pdl_wait_for_previous_kernel();  // before the first write to Y
    const int quarter = warp & 3;               // TMEM lanes this warp may read
    const int g = ((warp - 2) >> 2) & 1;        // token group (accumulator) handled by this warp
    const int column_part = (warp - 2) >> 3;    // with sixteen warps two share a quarter of an accumulator
    constexpr int kColumnParts = kDequantWarps / 8;
    constexpr int kColsWarp = kNPair / kColumnParts;
    if (ok) {
      // The accumulators are complete, so every stage of both rings has been read: the rings' shared
      // memory now stages the FP16 tile, and rows leave it as whole 512-byte runs (a lane of the
      // accumulator is a token row: written straight from registers, a warp's store would touch 32
      // rows with 16 bytes each -- tolerable in local memory, very slow as NVLink packets).
      const int row_cta = g * kTokensGroup + quarter * 32;  // first of this warp's 32 rows within the CTA's 256
      uint8_t* stage = smem_a;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + g * 256;
      const uint32_t my_row = smem_addr(stage + (row_cta + lane) * kOutPitch);
      for (int c0 = column_part * kColsWarp; c0 < (column_part + 1) * kColsWarp; c0 += 32) {
        uint32_t v[32];
        tmem_load_32cols(taddr + c0, v);
        tmem_load_wait();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          __half2 h0 = __floats2half2_rn(__uint_as_float(v[8 * i + 0]), __uint_as_float(v[8 * i + 1]));
          __half2 h1 = __floats2half2_rn(__uint_as_float(v[8 * i + 2]), __uint_as_float(v[8 * i + 3]));
          __half2 h2 = __floats2half2_rn(__uint_as_float(v[8 * i + 4]), __uint_as_float(v[8 * i + 5]));
          __half2 h3 = __floats2half2_rn(__uint_as_float(v[8 * i + 6]), __uint_as_float(v[8 * i + 7]));
          asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(my_row + (c0 + 8 * i) * 2),
                       "r"(*reinterpret_cast<uint32_t*>(&h0)), "r"(*reinterpret_cast<uint32_t*>(&h1)),
                       "r"(*reinterpret_cast<uint32_t*>(&h2)), "r"(*reinterpret_cast<uint32_t*>(&h3))
                       : "memory");
        }
      }
      __syncwarp();
      // Destination of the tile: y, or this rank's slot at the rank that owns the columns.
      __half* out;
      size_t pitch;
      if (p.owner_cols == 0) {
        out = p.y + n0;
        pitch = static_cast<size_t>(p.N);
      } else {
        const int owner = n0 / p.owner_cols;
        out = p.scatter[owner] + (n0 - owner * p.owner_cols);
        pitch = static_cast<size_t>(p.owner_cols);
      }
      constexpr int kLanesPerRow = kColsWarp / 8;       // 16-byte pieces of a row's part
      constexpr int kRowsPerStep = 32 / kLanesPerRow;
      const int piece = lane % kLanesPerRow;
      const int sub_row = lane / kLanesPerRow;
      const int col = column_part * kColsWarp + piece * 8;
#pragma unroll 4
      for (int r = sub_row; r < 32; r += kRowsPerStep) {
        const int m = m0 + g * 256 + quarter * 32 + r;
        const uint4 piece_value = *reinterpret_cast<const uint4*>(stage + (row_cta + r) * kOutPitch + col * 2);
        if (m < p.M) *reinterpret_cast<uint4*>(out + static_cast<size_t>(m) * pitch + col) = piece_value;
      }
      // Tiles sent to a peer are ordered before whatever this GPU tells that peer afterwards by the
      // end of the kernel: the exchange's first flag is raised by a later launch (a fence here would
      // hold the SM until every store has been acknowledged across NVLink).
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
  // Neither CTA may leave (or free tensor memory) while the other could still signal it.
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

}  // namespace

bool gemm_tc_pair_supports(int64_t M, int64_t N, int64_t K) {
  return M >= 1 && N >= kNPair && N % kNPair == 0 && K >= 256 && K % 256 == 0 && M <= (1 << 24) &&
         N <= (1 << 24) && K <= (1 << 24) &&
         (N / kNPair) * ((M + kTokensPair - 1) / kTokensPair) <= 0x3fffffffLL;
}

cudaError_t launch_gemm_tc_pair(const Problem& p, int* status_word, cudaStream_t stream, bool pdl, bool independent,
                                const PairScatter* scatter) {
  if (scatter != nullptr) {
    if (scatter->world < 2 || scatter->world > kMaxScatterRanks || p.N % scatter->world != 0 ||
        (p.N / scatter->world) % kNPair != 0) {
      return cudaErrorInvalidValue;
    }
  }
  CUtensorMap tmap;
  const uint64_t dims[2] = {static_cast<uint64_t>(p.K), static_cast<uint64_t>(p.M)};
  const uint64_t strides[1] = {static_cast<uint64_t>(p.K) * sizeof(__half)};
  const uint32_t box[2] = {kBK, kTokensGroup};
  if (!encode_tensor_map(&tmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, p.x, dims, strides, box,
                         CU_TENSOR_MAP_SWIZZLE_128B)) {
    return cudaErrorInvalidValue;
  }
  static bool configured[64] = {};
  int device = 0;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess) return err;
  if (device < 0 || device >= 64 || !configured[device]) {
    err = cudaFuncSetAttribute(w4a16_gemm_tc_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (err != cudaSuccess) return err;
    if (device >= 0 && device < 64) configured[device] = true;
  }
  PairParams pp;
  pp.packed = p.packed;
  pp.scales = p.scales;
  pp.zeros = p.zeros;
  pp.y = p.y;
  pp.M = static_cast<int>(p.M);
  pp.N = static_cast<int>(p.N);
  pp.K = static_cast<int>(p.K);
  pp.m_tiles = static_cast<int>((p.M + kTokensPair - 1) / kTokensPair);
  pp.status = status_word;
  pp.wait_previous = independent ? 0 : 1;
  pp.owner_cols = 0;
  for (int r = 0; r < kMaxScatterRanks; ++r) pp.scatter[r] = nullptr;
  if (scatter != nullptr) {
    pp.owner_cols = static_cast<int>(p.N / scatter->world);
    for (int r = 0; r < scatter->world; ++r) pp.scatter[r] = scatter->slot[r];
  }
  const unsigned pairs = static_cast<unsigned>((p.N / kNPair) * pp.m_tiles);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, w4a16_gemm_tc_pair_kernel, tmap, pp);
}

}  // namespace lbl
