// Decode GEMV (M <= 2): the instruction-lean form of the streaming kernel in skinny.cu.
//
// Same data movement as skinny.cu -- persistent CTAs, one producer warp, a ring of stages filled
// by three tiled TMA copies each (packed words, scales, zero points of 16 rows; evict-first in the
// L2), optional split-K with an ordered reduction -- plus a reducer warp that adds the eight
// consumer warps' unit results and writes them out, so the consumers never wait for one another
// or for global memory.  The warp MMA is used differently.  With at most two rows of
// activations, six of the eight B columns of an m16n8k16 MMA would be idle.  Here they separate
// the four lanes of a quad instead: column n of B holds the activations of the k-slots owned by
// lane n of the quad and zeros elsewhere, so one MMA yields, per weight row, four partial sums
// that belong to four different 32-column pieces of K.  Each lane can therefore read 16 bytes
// (32 weights) of its row with a single shared-memory load, and eight MMAs consume 16 rows by
// 128 columns (two quantisation groups) with
//     2 loads of weights, 40 integer instructions of nibble extraction, 8 MMAs in one chain,
//     4 predicated loads of activations and about 15 instructions of FP32 scale / zero point,
// roughly a third of the instructions per weight of the general kernel.  Columns 4-7 carry the
// second activation row when M = 2.
//
// Numerics are those of skinny.cu: raw levels q as exact FP16 subnormals, FP32 accumulation,
//     acc += scale * (sum_k q x - zero * sum_k x)   per group, in FP32.
#include "decode_tile.cuh"

#include "kernels.h"
#include "tensor_map.h"

namespace lbl {
namespace {

using namespace decode;

constexpr int kMaxPeers = 8;

struct DecodeParams {
  const __half* x;
  __half* y;
  float* partials;
  int* tickets;
  int* status;
  int M, N, K;
  int kseg, nsplit, stage_k, stages_per_unit, slots;
  int row_tiles, units;
  int packed_pitch, meta_pitch, slot_bytes;
  int sx_offset, red_offset, xf_offset, ring_offset;
  // Fused K-split all-reduce over peer memory (world == 0: off).  peers[r] is rank r's exchange
  // buffer as mapped into this process; peers[rank] is this GPU's own.
  int rank, world, capacity_n;
  unsigned char* peers[kMaxPeers];
};

// Layout of an exchange buffer (see lbl_peer_buffer_* in the C ABI).
constexpr int kPeerDataOffset = 2048;    // two FP32 vectors of capacity_n (epoch parity)
constexpr int kStatusPeerWait = 110;     // status code: a peer's flag did not arrive in time
struct PeerControl {
  int done;            // CTAs of the running kernel that have finished their units
  unsigned int epoch;  // number of all-reduces this GPU has completed
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
  // volatile keeps it behind the flag wait; no memory clobber, so independent loads can be issued
  // back to back before their values are used.
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(ptr));
  return v;
}
__device__ __forceinline__ float load_relaxed_sys(const float* ptr) {
  float v;
  asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(v) : "l"(ptr) : "memory");
  return v;
}

// The CTA's work list, walked in the same order by the producer, the consumers and the reducer:
// units a grid apart, unit = K segment `ks` of row tile `rt` (ks-major).  Coordinates advance by
// counting; there is no division in the loops.
struct UnitCursor {
  int unit, next_ks, next_rt;
  int ks, rt;  // the current unit, valid after next()

  __device__ __forceinline__ UnitCursor() : unit(blockIdx.x), next_ks(0), next_rt(blockIdx.x) {}

  __device__ __forceinline__ bool next(const DecodeParams& p) {
    if (unit >= p.units) return false;
    while (next_rt >= p.row_tiles) next_rt -= p.row_tiles, ++next_ks;
    ks = next_ks, rt = next_rt;
    unit += gridDim.x, next_rt += gridDim.x;
    return true;
  }
};

__global__ void __launch_bounds__(kThreads, 2)
    w4a16_gemv_decode_kernel(const __grid_constant__ CUtensorMap tmap_w,
                             const __grid_constant__ CUtensorMap tmap_s,
                             const __grid_constant__ CUtensorMap tmap_z, const DecodeParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  Header* hdr = reinterpret_cast<Header*>(smem);
  float* sx = reinterpret_cast<float*>(smem + p.sx_offset);
  float* red = reinterpret_cast<float*>(smem + p.red_offset);
  uint4* xf = reinterpret_cast<uint4*>(smem + p.xf_offset);
  uint8_t* ring = smem + p.ring_offset;
  volatile int* abort_flag = &hdr->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.slots; ++s) {
      mbar_init(&hdr->full[s], 1);
      mbar_init(&hdr->empty[s], kConsumerWarps);
    }
    for (int b = 0; b < kRedBuffers; ++b) {
      mbar_init(&hdr->red_full[b], kConsumerWarps);
      mbar_init(&hdr->red_empty[b], 1);
    }
    hdr->abort_flag = 0;
    hdr->ticket = 0;
    for (int i = 0; i < 4; ++i) hdr->zeros[i] = make_uint4(0u, 0u, 0u, 0u);
    mbar_init_fence();
  }
  __syncthreads();
  // The next kernel in the stream may start filling its own ring as soon as it finds room.
  pdl_allow_next_kernel();

  const int scales_block = kRows * p.packed_pitch;
  const int zeros_block = scales_block + kRows * p.meta_pitch;

  if (warp == kProducerWarp) {
    // ------------------------------- producer ------------------------------------------------
    if (lane == 0) {
      // Slot and round of the ring advance by counting (no division in the loop); the unit's
      // K segment and row tile likewise.  (Prefetching the stages behind the ring into the L2
      // while the consumers wait for their activations was measured and lost: the prefetches
      // compete with the loads the consumers are waiting for.)
      const uint64_t stream_once = l2_evict_first_policy();
      int slot = 0, round = 0;
      auto load_stage = [&](int stage_index, int n0) {
        if (round > 0) {
          mbar_wait_bounded(&hdr->empty[slot], (round - 1) & 1, abort_flag, p.status,
                            kStatusSkinnyEmptyWait);
        }
        // The tensor maps view every row as [K / stage_k][stage_k (+ padding)]; padding and
        // rows past N are zero-filled by the copy engine and cost no traffic.
        uint8_t* base = ring + static_cast<size_t>(slot) * p.slot_bytes;
        mbar_arrive_expect_tx(&hdr->full[slot], static_cast<uint32_t>(p.slot_bytes));
        tma_load_3d_hint(base, &tmap_w, 0, stage_index, n0, &hdr->full[slot], stream_once);
        tma_load_3d_hint(base + scales_block, &tmap_s, 0, stage_index, n0, &hdr->full[slot], stream_once);
        tma_load_3d_hint(base + zeros_block, &tmap_z, 0, stage_index, n0, &hdr->full[slot], stream_once);
        if (++slot == p.slots) slot = 0, ++round;
      };
      UnitCursor cur;
      while (cur.next(p)) {
        for (int st = 0; st < p.stages_per_unit; ++st) {
          if (*abort_flag) return;
          load_stage(cur.ks * p.stages_per_unit + st, cur.rt * kRows);
        }
      }
    }
    return;
  }

  if (warp == kReducerWarp) {
    // ------------------------------- reducer -------------------------------------------------
    // Adds the eight consumer warps' parts of each unit in a fixed order (lane = activation row
    // * 16 + weight row) and writes the result -- or, with split-K, runs the ticket protocol:
    // partial sums to the scratch, and the CTA that draws a row tile's last ticket adds them in
    // split order.  The global round trips of that protocol happen here, off the consumers' path.
    pdl_wait_for_previous_kernel();
    // With the fused all-reduce this GPU's FP32 result goes to its exchange buffer (the vector
    // of the next epoch's parity) instead of y.
    float* exchange_out = nullptr;
    if (p.world > 0) {
      const PeerControl* own = reinterpret_cast<const PeerControl*>(p.peers[p.rank]);
      const unsigned int next_epoch = *reinterpret_cast<const volatile unsigned int*>(&own->epoch) + 1;
      exchange_out = reinterpret_cast<float*>(p.peers[p.rank] + kPeerDataOffset) +
                     static_cast<size_t>(next_epoch & 1) * p.capacity_n;
    }
    const int row = lane & 15;
    const int col = lane >> 4;
    UnitCursor cur;
    for (int j = 0; cur.next(p); ++j) {
      const int n0 = cur.rt * kRows;
      const int buffer = j & (kRedBuffers - 1);
      mbar_wait_bounded(&hdr->red_full[buffer], (j / kRedBuffers) & 1, abort_flag, p.status,
                        kStatusSkinnyFullWait);
      const float* parts = red + buffer * kConsumerWarps * (kRows * 4);
      float v = 0.0f;
#pragma unroll
      for (int w = 0; w < kConsumerWarps; ++w) {
        v += parts[w * (kRows * 4) + row * 4 + 2 * col] + parts[w * (kRows * 4) + row * 4 + 2 * col + 1];
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&hdr->red_empty[buffer]);
      const bool valid = col < p.M && n0 + row < p.N;
      bool last = true;
      if (p.nsplit > 1) {
        if (valid) p.partials[(static_cast<size_t>(cur.ks) * p.M + col) * p.N + n0 + row] = v;
        __threadfence();
        __syncwarp();
        int ticket = 0;
        if (lane == 0) ticket = atomicAdd(&p.tickets[cur.rt], 1);
        ticket = __shfl_sync(0xffffffffu, ticket, 0);
        last = ticket == p.nsplit - 1;
        if (last) {
          __threadfence();
          if (valid) {
            v = 0.0f;
            for (int s = 0; s < p.nsplit; ++s) {
              v += __ldcg(&p.partials[(static_cast<size_t>(s) * p.M + col) * p.N + n0 + row]);
            }
          }
          if (lane == 0) p.tickets[cur.rt] = 0;
        }
      }
      if (last && valid) {
        if (exchange_out != nullptr) {
          exchange_out[n0 + row] = v;
        } else {
          p.y[static_cast<size_t>(col) * p.N + n0 + row] = __float2half_rn(v);
        }
      }
    }
    // The all-reduce may only count this CTA as done once its results are out.
    if (p.world > 0) {
      __threadfence();
      named_barrier(2, kConsumerThreads + 32);
    }
    return;
  }

  // --------------------------------- consumers -----------------------------------------------
  const int tid = threadIdx.x;  // 0..255
  const int g = lane >> 2;
  const int t = lane & 3;
  // B operand: column n = g of this lane carries activation row n / 4 for the k-slots of quad
  // lane n % 4, so only lanes with g % 4 == t hold activations; the others hold zeros.
  const int feed_row = g >> 2;
  const bool feeds_b = ((g & 3) == t) && (feed_row < p.M);
  // D result: this lane's columns 2t, 2t+1 are the two halves of group (t & 1) of the macro
  // tile, for activation row t / 2.
  const int out_row = t >> 1;
  const int group_parity = t & 1;
  const int words_seg = p.kseg / 8;
  const uint32_t ring_addr = smem_addr(ring);
  const uint32_t sx_base = smem_addr(sx) + static_cast<uint32_t>(group_parity * 2 + out_row) * 4;
  const uint32_t xf_addr = smem_addr(xf) + static_cast<uint32_t>(feed_row * words_seg + t * 4) * 16;
  // Lanes that feed no activation column never load: their B registers stay zero for good.
  uint4 xb[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) xb[i] = make_uint4(0u, 0u, 0u, 0u);

  // Fused all-reduce: the last CTA of this GPU to finish combines the ranks (after the loop).
  PeerControl* ctrl = nullptr;
  unsigned int epoch = 0;

  int slot = 0, parity = 0;  // ring position, advanced by counting
  int seq = 0;               // units this CTA has computed
  const int rotation_step = (p.stage_k / 128) & 7;
  int current_ks = -1;
  UnitCursor cur;
  while (cur.next(p)) {
    const int ks = cur.ks;

    if (ks != current_ks) {
      // Activations are the only input the previous kernel may have produced.
      if (current_ks < 0) {
        pdl_wait_for_previous_kernel();
        if (p.world > 0) {
          ctrl = reinterpret_cast<PeerControl*>(p.peers[p.rank]);
          epoch = *reinterpret_cast<volatile unsigned int*>(&ctrl->epoch) + 1;
        }
      }
      // A later segment (split-K with several segments per CTA): every warp must be done with
      // the old operand before it is overwritten.
      if (current_ks >= 0) named_barrier(1, kConsumerThreads);
      build_activation_operand(p.x, p.M, p.K, p.kseg, ks * p.kseg, xf, sx, tid);
      named_barrier(1, kConsumerThreads);
      current_ks = ks;
    }

    float acc_a = 0.0f;  // row n0 + g
    float acc_b = 0.0f;  // row n0 + g + 8
    for (int st = 0; st < p.stages_per_unit; ++st) {
      mbar_wait_bounded(&hdr->full[slot], parity, abort_flag, p.status, kStatusSkinnyFullWait);

      // Stages whose macro tiles are not a multiple of the eight warps (K = 1536: twelve) would
      // give four warps twice the work: the warps take the tiles in rotation, as a function of the
      // row tile and the stage alone (the grouped kernel uses the same one: same bits).
      const int vwarp = (warp - (cur.rt * p.stages_per_unit + st) * rotation_step) & 7;
      consume_stage(ring_addr + static_cast<uint32_t>(slot * p.slot_bytes), p.packed_pitch, p.meta_pitch,
                    p.stage_k, st, xf_addr, sx_base, vwarp, g, t, group_parity, feeds_b, xb, acc_a, acc_b);
      __syncwarp();
      if (lane == 0) mbar_arrive(&hdr->empty[slot]);
      if (++slot == p.slots) slot = 0, parity ^= 1;
    }

    // ---- deposit this warp's part of the unit in one of kRedBuffers buffers; the reducer warp
    // adds the eight parts when all have arrived.  No consumer waits for another here, so the warps
    // of a CTA never run in lockstep; a buffer is written again only after the reducer has read it.
    {
      const int buffer = seq & (kRedBuffers - 1);
      if (seq >= kRedBuffers) {
        mbar_wait_bounded(&hdr->red_empty[buffer], ((seq / kRedBuffers) - 1) & 1, abort_flag, p.status,
                          kStatusSkinnyEmptyWait);
      }
      float* mine = red + (buffer * kConsumerWarps + warp) * (kRows * 4);
      mine[g * 4 + t] = acc_a;
      mine[(g + 8) * 4 + t] = acc_b;
      __syncwarp();
      if (lane == 0) mbar_arrive(&hdr->red_full[buffer]);
    }
    ++seq;
  }

  if (p.world == 0) return;
  // ---- fused all-reduce: the last CTA of this GPU tells its peers, waits for theirs, and adds the
  // ranks' vectors in rank order (so every rank computes the same bits) ---------------------------
  if (ctrl == nullptr) {  // a CTA without units still has to be counted
    pdl_wait_for_previous_kernel();
    ctrl = reinterpret_cast<PeerControl*>(p.peers[p.rank]);
    epoch = *reinterpret_cast<volatile unsigned int*>(&ctrl->epoch) + 1;
  }
  // The reducer warp joins once this CTA's results are in the exchange buffer.
  named_barrier(2, kConsumerThreads + 32);
  __threadfence();
  named_barrier(1, kConsumerThreads);
  if (tid == 0) hdr->ticket = atomicAdd(&ctrl->done, 1);
  named_barrier(1, kConsumerThreads);
  if (hdr->ticket != static_cast<int>(gridDim.x) - 1) return;
  __threadfence();
  if (tid < p.world && tid != p.rank) {
    // Publish: this GPU's vector for `epoch` is complete.  The flag lives in the peer's buffer, so
    // that every GPU polls its own memory.
    __threadfence_system();
    store_release_sys(reinterpret_cast<unsigned int*>(p.peers[tid] + kPeerFlagsOffset + p.rank * 128), epoch);
    const unsigned int* mine =
        reinterpret_cast<const unsigned int*>(p.peers[p.rank] + kPeerFlagsOffset + tid * 128);
    const long long start = clock64();
    while (static_cast<int>(load_acquire_sys(mine) - epoch) < 0) {
      if (clock64() - start > kWaitLimitCycles) {  // bounded: report, never sum stale vectors
        atomicCAS(p.status, 0, kStatusPeerWait);
        *abort_flag = 1;
        break;
      }
    }
  }
  named_barrier(1, kConsumerThreads);
  if (*abort_flag) {
    // A peer never reported: the sum would mix this step's vectors with stale ones.  The output is
    // filled with NaN instead, so that the failure shows in the data as well as in the status word.
    for (int n = tid; n < p.N; n += kConsumerThreads) p.y[n] = __ushort_as_half(0x7E00);
    if (tid == 0) {
      ctrl->done = 0;
      *reinterpret_cast<volatile unsigned int*>(&ctrl->epoch) = epoch;
    }
    return;
  }
  const size_t vec = static_cast<size_t>(epoch & 1) * p.capacity_n;
  // The loads of two chunks from all ranks are issued before any is used: one NVLink round trip
  // per pair of chunks instead of one per load.
  const int n4 = p.N & ~3;
  for (int n = tid * 4; n < n4; n += kConsumerThreads * 8) {
    const int n_next = n + kConsumerThreads * 4;
    float4 part[2][kMaxPeers];
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      const int nc = c == 0 ? n : n_next;
#pragma unroll
      for (int r = 0; r < kMaxPeers; ++r) {
        if (r < p.world && nc < n4) {
          part[c][r] = load_relaxed_sys_v4(reinterpret_cast<const float*>(p.peers[r] + kPeerDataOffset) + vec + nc);
        }
      }
    }
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      const int nc = c == 0 ? n : n_next;
      if (nc >= n4) continue;
      float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
      for (int r = 0; r < kMaxPeers; ++r) {
        if (r < p.world) {
          v.x += part[c][r].x;
          v.y += part[c][r].y;
          v.z += part[c][r].z;
          v.w += part[c][r].w;
        }
      }
      __half2 lo = __floats2half2_rn(v.x, v.y);
      __half2 hi = __floats2half2_rn(v.z, v.w);
      uint2 out;
      out.x = *reinterpret_cast<uint32_t*>(&lo);
      out.y = *reinterpret_cast<uint32_t*>(&hi);
      *reinterpret_cast<uint2*>(p.y + nc) = out;
    }
  }
  for (int n = n4 + tid; n < p.N; n += kConsumerThreads) {
    float v = 0.0f;
    for (int r = 0; r < p.world; ++r) {
      v += load_relaxed_sys(reinterpret_cast<const float*>(p.peers[r] + kPeerDataOffset) + vec + n);
    }
    p.y[n] = __float2half_rn(v);
  }
  if (tid == 0) {
    ctrl->done = 0;
    *reinterpret_cast<volatile unsigned int*>(&ctrl->epoch) = epoch;
  }
}

}  // namespace

cudaError_t launch_gemv_decode(const Problem& p, const SkinnyPlan& plan, float* partials,
                               int* tickets, int* status_word, bool pdl, cudaStream_t stream,
                               const PeerReduce* reduce) {
  static_assert(kPeerDataOffset == static_cast<int>(kPeerBufferHeaderBytes), "layout mismatch");
  DecodeParams kp;
  kp.rank = 0;
  kp.world = 0;
  kp.capacity_n = 0;
  for (int i = 0; i < kMaxPeers; ++i) kp.peers[i] = nullptr;
  if (reduce != nullptr) {
    if (p.M != 1 || reduce->world < 1 || reduce->world > kMaxPeers || reduce->rank < 0 ||
        reduce->rank >= reduce->world || p.N > reduce->capacity_n) {
      return cudaErrorInvalidValue;
    }
    kp.rank = reduce->rank;
    kp.world = reduce->world;
    kp.capacity_n = reduce->capacity_n;
    for (int i = 0; i < reduce->world; ++i) kp.peers[i] = static_cast<unsigned char*>(reduce->buffers[i]);
  }
  kp.x = p.x;
  kp.y = p.y;
  kp.partials = partials;
  kp.tickets = tickets;
  kp.status = status_word;
  kp.M = static_cast<int>(p.M);
  kp.N = static_cast<int>(p.N);
  kp.K = static_cast<int>(p.K);
  kp.kseg = plan.kseg;
  kp.nsplit = plan.nsplit;
  kp.stage_k = plan.stage_k;
  kp.stages_per_unit = plan.kseg / plan.stage_k;
  kp.slots = plan.slots;
  kp.row_tiles = plan.row_tiles;
  kp.units = plan.row_tiles * plan.nsplit;
  kp.packed_pitch = plan.packed_pitch;
  kp.meta_pitch = plan.meta_pitch;
  kp.slot_bytes = plan.slot_bytes;
  kp.sx_offset = plan.sx_offset;
  kp.red_offset = plan.red_offset;
  kp.xf_offset = plan.xf_offset;
  kp.ring_offset = plan.ring_offset;
  CUtensorMap maps[3];
  if (!skinny_encode_maps(p, plan, maps)) return cudaErrorInvalidValue;

  // The opt-in to large dynamic shared memory is per device; repeating it is harmless.
  static bool configured[64] = {};
  int device = 0;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess) return err;
  if (device < 0 || device >= 64 || !configured[device]) {
    err = cudaFuncSetAttribute(w4a16_gemv_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               216 * 1024);
    if (err != cudaSuccess) return err;
    if (device >= 0 && device < 64) configured[device] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(plan.grid));
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = static_cast<size_t>(plan.smem_bytes);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, w4a16_gemv_decode_kernel, maps[0], maps[1], maps[2], kp);
}

}  // namespace lbl
