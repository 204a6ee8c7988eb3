// All-reduce of FP32 partial sums over NVLink peer memory, for the K-split linears of a
// tensor-parallel group (one process per GPU, same node).
//
// Every rank owns an exchange buffer that its peers have mapped through CUDA IPC: a control
// block, one flag line per source rank, and two FP32 vectors selected by the parity of an epoch
// counter.  The kernel that runs before this one (the grouped GEMV) has left this rank's partial
// sums in the vector of the coming epoch.  This kernel then
//   1. tells every peer that the vector is complete (one release store per peer, into the peer's
//      buffer, so that everybody polls its own memory),
//   2. waits -- bounded -- until every peer has said the same,
//   3. adds the ranks' vectors in rank order with vector loads over NVLink (each rank reads all
//      of them, so all ranks compute the same bits: FP32 sums, one rounding to FP16), and
//   4. advances the epoch.
// Plain peer loads and stores only: no multimem, no multicast, no NCCL.  Two vectors suffice: a
// rank can start writing epoch e + 1 only after its own all-reduce of epoch e, which waited for
// every peer's flag of epoch e, which a peer raises only after it has finished reading epoch e - 1.
// If a peer's flag does not arrive in time the outputs are filled with NaN and the device status
// word is set; nothing stale is ever summed.
#include "common.cuh"
#include "kernels.h"

namespace lbl {
namespace {

constexpr int kReduceThreads = 256;
constexpr int kMaxPeers = 8;
constexpr int kStatusPeerWait = 110;  // a peer's flag did not arrive in time

struct ReduceParams {
  unsigned char* peers[kMaxPeers];
  const ReduceSegment* segments;
  int rank, world, capacity_n;
  int ctas_total;
  int* status;
};

__device__ __forceinline__ void store_release_sys(unsigned int* ptr, unsigned int value) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(ptr), "r"(value) : "memory");
}
__device__ __forceinline__ unsigned int load_acquire_sys(const unsigned int* ptr) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(ptr) : "memory");
  return v;
}
__device__ __forceinline__ float4 load_relaxed_sys_v4(const float* ptr) {
  float4 v;
  // volatile keeps it behind the flag wait; no memory clobber, so the loads of all ranks are in
  // flight together.
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(ptr));
  return v;
}

// grid = (CTAs per segment, segments).
__global__ void __launch_bounds__(kReduceThreads) peer_allreduce_kernel(const ReduceParams p) {
  __shared__ int timed_out;
  const int tid = threadIdx.x;
  pdl_allow_next_kernel();
  // This GPU's partial sums come from the previous kernel in the stream.
  pdl_wait_for_previous_kernel();
  unsigned char* own = p.peers[p.rank];
  int* done = reinterpret_cast<int*>(own + kPeerDoneOffset);
  volatile unsigned int* epoch_word = reinterpret_cast<volatile unsigned int*>(own + kPeerEpochOffset);
  const unsigned int epoch = *epoch_word + 1;
  if (tid == 0) timed_out = 0;
  __syncthreads();
  if (tid < p.world && tid != p.rank) {
    if (blockIdx.x == 0 && blockIdx.y == 0) {
      __threadfence_system();
      store_release_sys(reinterpret_cast<unsigned int*>(p.peers[tid] + kPeerFlagsOffset + p.rank * 128), epoch);
    }
    const unsigned int* mine = reinterpret_cast<const unsigned int*>(own + kPeerFlagsOffset + tid * 128);
    const long long start = clock64();
    while (static_cast<int>(load_acquire_sys(mine) - epoch) < 0) {
      if (clock64() - start > kWaitLimitCycles) {
        atomicCAS(p.status, 0, kStatusPeerWait);
        timed_out = 1;
        break;
      }
      __nanosleep(100);
    }
  }
  __syncthreads();

  const ReduceSegment seg = p.segments[blockIdx.y];
  const size_t vec = static_cast<size_t>(epoch & 1) * p.capacity_n + seg.offset;
  if (timed_out) {
    for (int n = blockIdx.x * kReduceThreads + tid; n < seg.count; n += gridDim.x * kReduceThreads) {
      seg.dst[n] = __ushort_as_half(0x7E00);
    }
  } else {
    for (int n = (blockIdx.x * kReduceThreads + tid) * 4; n < seg.count; n += gridDim.x * kReduceThreads * 4) {
      float4 part[kMaxPeers];
#pragma unroll
      for (int r = 0; r < kMaxPeers; ++r) {
        if (r < p.world) {
          part[r] = load_relaxed_sys_v4(reinterpret_cast<const float*>(p.peers[r] + kPeerBufferHeaderBytes) + vec + n);
        }
      }
      float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
      for (int r = 0; r < kMaxPeers; ++r) {
        if (r < p.world) {
          v.x += part[r].x;
          v.y += part[r].y;
          v.z += part[r].z;
          v.w += part[r].w;
        }
      }
      const __half2 lo = __floats2half2_rn(v.x, v.y);
      const __half2 hi = __floats2half2_rn(v.z, v.w);
      uint2 out;
      out.x = *reinterpret_cast<const uint32_t*>(&lo);
      out.y = *reinterpret_cast<const uint32_t*>(&hi);
      *reinterpret_cast<uint2*>(seg.dst + n) = out;
    }
  }
  // The last CTA to finish opens the next epoch.
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    if (atomicAdd(done, 1) == p.ctas_total - 1) {
      *done = 0;
      *epoch_word = epoch;
      __threadfence();
    }
  }
}

}  // namespace

cudaError_t launch_peer_allreduce(const PeerReduceLaunch& launch, bool pdl, cudaStream_t stream) {
  const PeerReduce& ex = launch.exchange;
  if (ex.world < 2 || ex.world > kMaxPeers || ex.rank < 0 || ex.rank >= ex.world || launch.segment_count < 1) {
    return cudaErrorInvalidValue;
  }
  ReduceParams kp;
  for (int r = 0; r < kMaxPeers; ++r) {
    kp.peers[r] = r < ex.world ? static_cast<unsigned char*>(ex.buffers[r]) : nullptr;
  }
  kp.segments = launch.segments;
  kp.rank = ex.rank;
  kp.world = ex.world;
  kp.capacity_n = ex.capacity_n;
  kp.status = launch.status;
  int per_segment = (launch.longest / 4 + kReduceThreads - 1) / kReduceThreads;
  // About one wave of CTAs is plenty: the vectors are small and the loads are latency-bound.
  const int cap = (296 + launch.segment_count - 1) / launch.segment_count;
  if (per_segment > cap) per_segment = cap;
  if (per_segment < 1) per_segment = 1;
  kp.ctas_total = per_segment * launch.segment_count;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(per_segment), static_cast<unsigned>(launch.segment_count));
  cfg.blockDim = dim3(kReduceThreads);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, peer_allreduce_kernel, kp);
}

}  // namespace lbl
