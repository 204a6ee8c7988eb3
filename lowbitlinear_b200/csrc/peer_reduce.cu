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
#ifdef LBL_TRACE_EXCHANGE
  const unsigned long long entered = global_timer_ns();
#endif
  // This GPU's partial sums come from the previous kernel in the stream.
  pdl_wait_for_previous_kernel();
  unsigned char* own = p.peers[p.rank];
  int* done = reinterpret_cast<int*>(own + kPeerDoneOffset);
  volatile unsigned int* epoch_word = reinterpret_cast<volatile unsigned int*>(own + kPeerEpochOffset);
  const unsigned int epoch = *epoch_word + 1;
#ifdef LBL_TRACE_EXCHANGE  // measurement build: time stamps in the control block, see gemv_grouped.cu
  unsigned long long* trace = reinterpret_cast<unsigned long long*>(own + 1536) + ((epoch - 1) % 8) * 8;
  const bool first_block = blockIdx.x == 0 && blockIdx.y == 0 && tid == 0;
  if (first_block) trace[2] = entered, trace[3] = global_timer_ns();
#endif
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
#ifdef LBL_TRACE_EXCHANGE
  if (first_block) trace[4] = global_timer_ns();
#endif

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
#ifdef LBL_TRACE_EXCHANGE
    atomicMax(trace + 5, global_timer_ns());
#endif
    __threadfence();
    if (atomicAdd(done, 1) == p.ctas_total - 1) {
      *done = 0;
      *epoch_word = epoch;
      __threadfence();
#ifdef LBL_TRACE_EXCHANGE
      trace[6] = global_timer_ns();
#endif
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Two-shot all-reduce of a K-split GEMM output [M, N] (large M).  Rank o owns the columns
// [o N / world, (o + 1) N / world).  The GEMM's epilogue (gemm_tc2.cu) has already written every
// rank's partial tile of those columns into rank o's exchange buffer, tile by tile while the GEMM
// ran: slot r of the buffer = rank r's partial [M, owner_cols], FP16.  What is left:
//   kernel 1 (reduce): tell every peer "my GEMM is complete" and wait for the same from them; add
//     the `world` slots of the own columns in rank order (FP32 sums, one rounding to FP16); write
//     the sums to y and to the `result` block of the own buffer; the last CTA tells every peer
//     "my columns are reduced";
//   kernel 2 (gather): wait for that message from every peer and copy their result blocks into y
//     with vector loads over NVLink; the last CTA advances the epoch by two.
// Every rank ends with the same bits in y.  A buffer serves one all-reduce at a time: the next
// GEMM that scatters into it must be ordered after this rank's gather kernel (same stream, or an
// event).  That suffices across ranks too: a peer raises its second flag only after it has read
// its slots, and rewrites its result block only after every rank's next first flag, which a rank
// raises after its own gather.
struct SliceParams {
  unsigned char* peers[kMaxPeers];
  __half* y;
  int rank, world;
  int M, N, owner_cols;
  int ctas_total;
  int* status;
};

__device__ __forceinline__ uint4 load_relaxed_sys_u4(const void* ptr) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(ptr));
  return v;
}

// Threads 0 .. world-1 (except `rank`) each wait, bounded, for flags[src] >= epoch in the own buffer.
__device__ __forceinline__ void wait_for_peers(unsigned char* own, int rank, int world, unsigned int epoch,
                                               int* status, int* timed_out) {
  const int tid = threadIdx.x;
  if (tid < world && tid != rank) {
    const unsigned int* mine = reinterpret_cast<const unsigned int*>(own + kPeerFlagsOffset + tid * 128);
    const long long start = clock64();
    while (static_cast<int>(load_acquire_sys(mine) - epoch) < 0) {
      if (clock64() - start > kWaitLimitCycles) {
        atomicCAS(status, 0, kStatusPeerWait);
        *timed_out = 1;
        break;
      }
      __nanosleep(100);
    }
  }
}

__device__ __forceinline__ void accumulate_half8(float (&acc)[8], const uint4& v) {
  const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __half22float2(h[i]);
    acc[2 * i] += f.x;
    acc[2 * i + 1] += f.y;
  }
}

__global__ void __launch_bounds__(kReduceThreads) peer_slice_reduce_kernel(const SliceParams p) {
  __shared__ int timed_out;
  const int tid = threadIdx.x;
  unsigned char* own = p.peers[p.rank];
  int* done = reinterpret_cast<int*>(own + kPeerDoneOffset);
  const unsigned int epoch = *reinterpret_cast<volatile unsigned int*>(own + kPeerEpochOffset) + 1;
  if (tid == 0) timed_out = 0;
  __syncthreads();
  // This kernel is launched without programmatic dependent launch: the GEMM before it in the
  // stream is complete, its tiles are in the owners' buffers.
  if (blockIdx.x == 0 && tid < p.world && tid != p.rank) {
    __threadfence_system();
    store_release_sys(reinterpret_cast<unsigned int*>(p.peers[tid] + kPeerFlagsOffset + p.rank * 128), epoch);
  }
  wait_for_peers(own, p.rank, p.world, epoch, p.status, &timed_out);
  __syncthreads();

  const size_t slice_bytes = static_cast<size_t>(p.M) * p.owner_cols * sizeof(__half);
  const unsigned char* slots = own + kPeerBufferHeaderBytes;
  unsigned char* result = own + kPeerBufferHeaderBytes + static_cast<size_t>(p.world) * slice_bytes;
  const int chunks_per_row = p.owner_cols / 8;
  const long long chunks = static_cast<long long>(p.M) * chunks_per_row;
  const bool failed = timed_out != 0;
  for (long long c = static_cast<long long>(blockIdx.x) * kReduceThreads + tid; c < chunks;
       c += static_cast<long long>(gridDim.x) * kReduceThreads) {
    uint4 out;
    if (failed) {
      out = make_uint4(0x7E007E00u, 0x7E007E00u, 0x7E007E00u, 0x7E007E00u);
    } else {
      uint4 part[kMaxPeers];
#pragma unroll
      for (int r = 0; r < kMaxPeers; ++r) {
        if (r < p.world) part[r] = load_relaxed_sys_u4(slots + r * slice_bytes + c * 16);
      }
      float acc[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
      for (int r = 0; r < kMaxPeers; ++r) {
        if (r < p.world) accumulate_half8(acc, part[r]);
      }
      __half2 h[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(acc[2 * i], acc[2 * i + 1]);
      out = *reinterpret_cast<const uint4*>(h);
    }
    *reinterpret_cast<uint4*>(result + c * 16) = out;
    const long long row = c / chunks_per_row;
    const int col = static_cast<int>(c - row * chunks_per_row) * 8;
    *reinterpret_cast<uint4*>(p.y + row * p.N + p.rank * p.owner_cols + col) = out;
  }
  __syncthreads();
  if (tid == 0) {
    __threadfence_system();
    if (atomicAdd(done, 1) == p.ctas_total - 1) {
      *done = 0;
      __threadfence_system();
      for (int r = 0; r < p.world; ++r) {
        if (r != p.rank) {
          store_release_sys(reinterpret_cast<unsigned int*>(p.peers[r] + kPeerFlagsOffset + p.rank * 128), epoch + 1);
        }
      }
    }
  }
}

__global__ void __launch_bounds__(kReduceThreads) peer_slice_gather_kernel(const SliceParams p) {
  __shared__ int timed_out;
  const int tid = threadIdx.x;
  // Kernels that follow in the stream and use programmatic dependent launch may start now.
  pdl_allow_next_kernel();
  unsigned char* own = p.peers[p.rank];
  int* done = reinterpret_cast<int*>(own + kPeerDoneOffset);
  volatile unsigned int* epoch_word = reinterpret_cast<volatile unsigned int*>(own + kPeerEpochOffset);
  const unsigned int epoch = *epoch_word + 2;
  if (tid == 0) timed_out = 0;
  __syncthreads();
  wait_for_peers(own, p.rank, p.world, epoch, p.status, &timed_out);
  __syncthreads();

  const size_t slice_bytes = static_cast<size_t>(p.M) * p.owner_cols * sizeof(__half);
  const size_t result_offset = kPeerBufferHeaderBytes + static_cast<size_t>(p.world) * slice_bytes;
  const int chunks_per_row = p.owner_cols / 8;
  const long long chunks = static_cast<long long>(p.M) * chunks_per_row;
  const bool failed = timed_out != 0;
  constexpr int kInFlight = 4;
  const long long stride = static_cast<long long>(gridDim.x) * kReduceThreads;
  for (int step = 1; step < p.world; ++step) {
    const int r = (p.rank + step) % p.world;  // every rank starts at another peer
    const unsigned char* src = p.peers[r] + result_offset;
    for (long long c0 = static_cast<long long>(blockIdx.x) * kReduceThreads + tid; c0 < chunks; c0 += stride * kInFlight) {
      uint4 v[kInFlight];
#pragma unroll
      for (int i = 0; i < kInFlight; ++i) {
        const long long c = c0 + i * stride;
        if (c < chunks) {
          v[i] = failed ? make_uint4(0x7E007E00u, 0x7E007E00u, 0x7E007E00u, 0x7E007E00u)
                        : load_relaxed_sys_u4(src + c * 16);
        }
      }
#pragma unroll
      for (int i = 0; i < kInFlight; ++i) {
        const long long c = c0 + i * stride;
        if (c < chunks) {
          const long long row = c / chunks_per_row;
          const int col = static_cast<int>(c - row * chunks_per_row) * 8;
          *reinterpret_cast<uint4*>(p.y + row * p.N + r * p.owner_cols + col) = v[i];
        }
      }
    }
  }
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

size_t peer_gemm_buffer_bytes(int64_t M, int64_t N, int world) {
  if (M <= 0 || N <= 0 || world < 1) return 0;
  // world slots of [M, N / world] plus the result block of the same size, FP16.
  return kPeerBufferHeaderBytes + static_cast<size_t>(M) * N * sizeof(__half) +
         static_cast<size_t>(M) * (N / world) * sizeof(__half);
}

cudaError_t launch_peer_slice_allreduce(const PeerReduce& ex, __half* y, int64_t M, int64_t N, int sm_count,
                                        int* status, cudaStream_t stream) {
  if (ex.world < 2 || ex.world > kMaxPeers || ex.rank < 0 || ex.rank >= ex.world || M < 1 || N % (8 * ex.world) != 0) {
    return cudaErrorInvalidValue;
  }
  SliceParams kp;
  for (int r = 0; r < kMaxPeers; ++r) {
    kp.peers[r] = r < ex.world ? static_cast<unsigned char*>(ex.buffers[r]) : nullptr;
  }
  kp.y = y;
  kp.rank = ex.rank;
  kp.world = ex.world;
  kp.M = static_cast<int>(M);
  kp.N = static_cast<int>(N);
  kp.owner_cols = static_cast<int>(N / ex.world);
  kp.status = status;
  const long long chunks = static_cast<long long>(M) * (kp.owner_cols / 8);
  long long ctas = (chunks + kReduceThreads - 1) / kReduceThreads;
  const long long cap = 4LL * (sm_count > 0 ? sm_count : 148);
  if (ctas > cap) ctas = cap;
  if (ctas < 1) ctas = 1;
  kp.ctas_total = static_cast<int>(ctas);
  peer_slice_reduce_kernel<<<static_cast<unsigned>(ctas), kReduceThreads, 0, stream>>>(kp);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return err;
  peer_slice_gather_kernel<<<static_cast<unsigned>(ctas), kReduceThreads, 0, stream>>>(kp);
  return cudaGetLastError();
}

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
