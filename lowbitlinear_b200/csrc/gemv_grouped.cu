// Grouped decode GEMV: one persistent launch over a list of independent W4A16 problems (M <= 2).
//
// A decode step of a model is a few hundred small GEMVs; launched one by one, each pays a few
// microseconds of fixed cost (grid start, cold pipeline, activations to every CTA, a partial last
// round of row tiles) that at these sizes rivals the time the weights need to cross the memory
// bus.  Here the problems of a step are described once, on the host, as a plan in device memory:
// per problem the three tensor maps over the reference layout, pointers and sizes; per CTA a list
// of segments, a segment being a run of consecutive 16-row tiles of one problem.  The plan cuts
// the stream of all problems' pipeline stages into one contiguous share per CTA, so a CTA starts its pipeline
// once, builds an activation operand once or twice, and streams its share at the copy rate; there
// is no tail of idle CTAs between problems and no split-K (small-N problems are simply short
// shares of the stream).
//
// CTA roles, pipeline and arithmetic are those of gemv_decode.cu (decode_tile.cuh): a producer
// lane issues three tiled TMA copies per stage, eight consumer warps run the warp MMAs on raw
// nibbles, a reducer warp adds the warps' parts and writes the outputs.  The problems of a group
// must not depend on each other: their activations are all read, and their outputs all written,
// by the one launch, in no particular order.
#include "decode_tile.cuh"

#include "kernels.h"
#include "tensor_map.h"

#include <algorithm>
#include <cstddef>
#include <cstring>
#include <vector>

namespace lbl {
namespace {

using namespace decode;

// One problem of the group as the kernel reads it (device memory, written once by the host).
struct alignas(128) GroupProblem {
  CUtensorMap w, s, z;  // packed words, scales, zero points (see skinny_encode_maps)
  const __half* x;      // [M, K]
  __half* y;            // [M, N] FP16, or
  float* y32;           // [M, N] FP32 when not null (partial sums of a K-split shard)
  int M, N, K;
  int stage_k, stages_per_unit, packed_pitch, meta_pitch, slot_bytes;
  int row_tiles;
  int pad[17];
};
static_assert(sizeof(GroupProblem) == 512, "descriptor layout");
static_assert(offsetof(GroupProblem, s) % 64 == 0 && offsetof(GroupProblem, z) % 64 == 0, "tensor map alignment");

// A run of consecutive row tiles of one problem; a CTA owns a contiguous range of segments.
struct GroupSegment {
  int problem, rt_begin, rt_count, pad;
};

struct GroupParams {
  const GroupProblem* problems;
  const GroupSegment* segments;
  const int* first_segment;  // [grid + 1]
  int* status;
  // Tensor-parallel groups: FP32 partial sums go to this GPU's exchange buffer, into the vector
  // of the next epoch's parity (see peer_reduce.cu).  Null / 0 otherwise.
  const unsigned int* epoch_word;
  int parity_stride;  // floats between the two vectors
  int slots, slot_stride;
  int sx_offset, red_offset, xf_offset, ring_offset;
};

__device__ __forceinline__ GroupSegment load_segment(const GroupSegment* ptr) {
  const int4 v = __ldg(reinterpret_cast<const int4*>(ptr));
  GroupSegment s;
  s.problem = v.x, s.rt_begin = v.y, s.rt_count = v.z, s.pad = v.w;
  return s;
}

__global__ void __launch_bounds__(kThreads, 2) w4a16_gemv_grouped_kernel(const GroupParams p) {
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
  pdl_allow_next_kernel();
#ifdef LBL_TRACE_EXCHANGE  // measurement build: time stamps in the exchange buffer's control block
  unsigned long long* trace = nullptr;
  if (p.epoch_word != nullptr) {
    const unsigned int e = *reinterpret_cast<const volatile unsigned int*>(p.epoch_word);
    trace = reinterpret_cast<unsigned long long*>(reinterpret_cast<unsigned char*>(const_cast<unsigned int*>(p.epoch_word)) - 4 + 1536) + (e % 8) * 8;
    if (blockIdx.x == 0 && threadIdx.x == 0) trace[0] = global_timer_ns();
  }
#endif

  const int seg_begin = __ldg(&p.first_segment[blockIdx.x]);
  const int seg_end = __ldg(&p.first_segment[blockIdx.x + 1]);

  if (warp == kProducerWarp) {
    // ------------------------------- producer ------------------------------------------------
    if (lane == 0) {
      const uint64_t stream_once = l2_evict_first_policy();
      int slot = 0, round = 0;
      for (int seg = seg_begin; seg < seg_end; ++seg) {
        const GroupSegment sg = load_segment(&p.segments[seg]);
        const GroupProblem* pr = &p.problems[sg.problem];
        const int stages_per_unit = __ldg(&pr->stages_per_unit);
        const int packed_pitch = __ldg(&pr->packed_pitch);
        const int meta_pitch = __ldg(&pr->meta_pitch);
        const uint32_t slot_bytes = static_cast<uint32_t>(__ldg(&pr->slot_bytes));
        const int scales_block = kRows * packed_pitch;
        const int zeros_block = scales_block + kRows * meta_pitch;
        for (int rt = sg.rt_begin; rt < sg.rt_begin + sg.rt_count; ++rt) {
          const int n0 = rt * kRows;
          for (int st = 0; st < stages_per_unit; ++st) {
            if (*abort_flag) return;
            if (round > 0) {
              mbar_wait_bounded(&hdr->empty[slot], (round - 1) & 1, abort_flag, p.status,
                                kStatusSkinnyEmptyWait);
            }
            uint8_t* base = ring + static_cast<size_t>(slot) * p.slot_stride;
            mbar_arrive_expect_tx(&hdr->full[slot], slot_bytes);
            tma_load_3d_hint(base, &pr->w, 0, st, n0, &hdr->full[slot], stream_once);
            tma_load_3d_hint(base + scales_block, &pr->s, 0, st, n0, &hdr->full[slot], stream_once);
            tma_load_3d_hint(base + zeros_block, &pr->z, 0, st, n0, &hdr->full[slot], stream_once);
            if (++slot == p.slots) slot = 0, ++round;
          }
        }
      }
    }
    return;
  }

  if (warp == kReducerWarp) {
    // ------------------------------- reducer -------------------------------------------------
    pdl_wait_for_previous_kernel();
    size_t parity_offset = 0;
    if (p.epoch_word != nullptr) {
      const unsigned int next_epoch = *reinterpret_cast<const volatile unsigned int*>(p.epoch_word) + 1;
      parity_offset = static_cast<size_t>(next_epoch & 1) * p.parity_stride;
    }
    const int row = lane & 15;
    const int col = lane >> 4;
    int j = 0;
    for (int seg = seg_begin; seg < seg_end; ++seg) {
      const GroupSegment sg = load_segment(&p.segments[seg]);
      const GroupProblem* pr = &p.problems[sg.problem];
      const int M = __ldg(&pr->M);
      const int N = __ldg(&pr->N);
      __half* y = pr->y;
      float* y32 = pr->y32 == nullptr ? nullptr : pr->y32 + parity_offset;
      for (int rt = sg.rt_begin; rt < sg.rt_begin + sg.rt_count; ++rt, ++j) {
        const int n0 = rt * kRows;
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
        if (col < M && n0 + row < N) {
          if (y32 != nullptr) {
            y32[static_cast<size_t>(col) * N + n0 + row] = v;
          } else {
            y[static_cast<size_t>(col) * N + n0 + row] = __float2half_rn(v);
          }
        }
      }
    }
#ifdef LBL_TRACE_EXCHANGE
    if (trace != nullptr && lane == 0) atomicMax(trace + 1, global_timer_ns());
#endif
    return;
  }

  // --------------------------------- consumers -----------------------------------------------
  const int tid = threadIdx.x;  // 0..255
  const int g = lane >> 2;
  const int t = lane & 3;
  const int feed_row = g >> 2;
  const int out_row = t >> 1;
  const int group_parity = t & 1;
  const uint32_t ring_addr = smem_addr(ring);
  const uint32_t sx_base = smem_addr(sx) + static_cast<uint32_t>(group_parity * 2 + out_row) * 4;
  uint4 xb[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) xb[i] = make_uint4(0u, 0u, 0u, 0u);

  int slot = 0, parity = 0;  // ring position, advanced by counting
  int seq = 0;               // units this CTA has computed
  int current_problem = -1;
  int rotation_step = 0;  // see the stage loop
  // Geometry of the current problem.
  int stages_per_unit = 0, packed_pitch = 0, meta_pitch = 0, stage_k = 0;
  bool feeds_b = false;
  uint32_t xf_addr = 0;
  for (int seg = seg_begin; seg < seg_end; ++seg) {
    const GroupSegment sg = load_segment(&p.segments[seg]);
    if (sg.problem != current_problem) {
      const GroupProblem* pr = &p.problems[sg.problem];
      // Activations are the only input the previous kernel in the stream may have produced.
      if (current_problem < 0) {
        pdl_wait_for_previous_kernel();
      } else {
        named_barrier(1, kConsumerThreads);  // every warp is done with the old operand
      }
      const int M = __ldg(&pr->M);
      const int K = __ldg(&pr->K);
      stages_per_unit = __ldg(&pr->stages_per_unit);
      packed_pitch = __ldg(&pr->packed_pitch);
      meta_pitch = __ldg(&pr->meta_pitch);
      stage_k = __ldg(&pr->stage_k);
      rotation_step = (stage_k / 128) & 7;
      build_activation_operand(pr->x, M, K, K, 0, xf, sx, tid);
      named_barrier(1, kConsumerThreads);
      // B operand: column n = g of this lane carries activation row n / 4 for the k-slots of quad
      // lane n % 4, so only lanes with g % 4 == t hold activations; the others keep zeros.
      const bool fed_before = feeds_b;
      feeds_b = ((g & 3) == t) && (feed_row < M);
      if (fed_before && !feeds_b) {
#pragma unroll
        for (int i = 0; i < 4; ++i) xb[i] = make_uint4(0u, 0u, 0u, 0u);
      }
      xf_addr = smem_addr(xf) + static_cast<uint32_t>(feed_row * (K / 8) + t * 4) * 16;
      current_problem = sg.problem;
    }

    for (int rt = sg.rt_begin; rt < sg.rt_begin + sg.rt_count; ++rt) {
      float acc_a = 0.0f;  // row n0 + g
      float acc_b = 0.0f;  // row n0 + g + 8
      for (int st = 0; st < stages_per_unit; ++st) {
        mbar_wait_bounded(&hdr->full[slot], parity, abort_flag, p.status, kStatusSkinnyFullWait);
        // A stage whose 128-column macro tiles are not a multiple of the eight warps (K = 1536 or
        // 3072: twelve) would give four warps twice the work of the others; the warps take the
        // tiles in rotation from stage to stage instead, so the leftover moves round.  The warps run
        // asynchronously (the reducer collects their parts), so balance over a few stages is enough.
        // The rotation is a function of the row tile and the stage alone, so that every kernel
        // that computes this unit adds its parts in the same order (same bits).
        const int vwarp = (warp - (rt * stages_per_unit + st) * rotation_step) & 7;
        consume_stage(ring_addr + static_cast<uint32_t>(slot * p.slot_stride), packed_pitch, meta_pitch,
                      stage_k, st, xf_addr, sx_base, vwarp, g, t, group_parity, feeds_b, xb, acc_a, acc_b);
        __syncwarp();
        if (lane == 0) mbar_arrive(&hdr->empty[slot]);
        if (++slot == p.slots) slot = 0, parity ^= 1;
      }
      // Deposit this warp's part of the unit; the reducer warp adds the eight parts.
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
      ++seq;
    }
  }
}

constexpr int kSmemBudgetTwoCtas = 110 * 1024;

}  // namespace

// Host side of a group: the launch geometry plus the device memory that holds the plan.
struct GroupPlan {
  int device = 0;
  int count = 0;
  int grid = 0;
  int smem_bytes = 0;
  void* device_memory = nullptr;  // problems, segments, first_segment in one allocation
  GroupParams params{};
  int64_t algorithmic_bytes = 0;
  bool has_reduce = false;
  PeerReduceLaunch reduce{};
};

cudaError_t group_plan_create(const GroupProblemDesc* descs, int count, int sm_count, int* status_word,
                              const PeerReduce* exchange, GroupPlan** out, const char** why) {
  *out = nullptr;
  *why = "";
  if (count <= 0) {
    *why = "a group needs at least one problem";
    return cudaErrorInvalidValue;
  }
  std::vector<GroupProblem> problems(static_cast<size_t>(count));
  int max_slot = 0, max_xf = 0, max_sx = 0;
  int64_t total_cost = 0, bytes = 0, reduce_elems = 0;
  std::vector<ReduceSegment> reduce_segments;
  for (int i = 0; i < count; ++i) {
    const GroupProblemDesc& d = descs[i];
    SkinnyPlan plan;
    if (d.M < 1 || d.M > 2 || !skinny_make_plan(d.M, d.N, d.K, /*want_split=*/0, sm_count, &plan) ||
        !plan.columns || plan.nsplit != 1) {
      *why = "grouped GEMV serves M <= 2, K % 256 == 0 and M * K <= 32768";
      return cudaErrorInvalidValue;
    }
    Problem prob;
    prob.x = static_cast<const __half*>(d.x);
    prob.packed = reinterpret_cast<const uint32_t*>(d.packed);
    prob.scales = d.scales;
    prob.zeros = d.zeros;
    prob.y = static_cast<__half*>(d.y);
    prob.M = d.M, prob.N = d.N, prob.K = d.K;
    CUtensorMap maps[3];
    if (!skinny_encode_maps(prob, plan, maps)) {
      *why = "the driver rejected a tensor map";
      return cudaErrorInvalidValue;
    }
    GroupProblem& g = problems[static_cast<size_t>(i)];
    std::memset(&g, 0, sizeof(g));
    g.w = maps[0], g.s = maps[1], g.z = maps[2];
    g.x = prob.x;
    g.y = prob.y;
    g.y32 = nullptr;
    if (d.reduce && exchange != nullptr && exchange->world > 1) {
      // Partial sums of a K-split shard: FP32 into the exchange buffer, summed over the ranks and
      // rounded to FP16 into y by the all-reduce kernel that follows.
      const int64_t elems = d.M * d.N;
      if (elems % 4 != 0 || reduce_elems + elems > exchange->capacity_n) {
        *why = "the reduced outputs do not fit the exchange buffers (or M * N is not a multiple of 4)";
        return cudaErrorInvalidValue;
      }
      g.y32 = reinterpret_cast<float*>(static_cast<unsigned char*>(exchange->buffers[exchange->rank]) +
                                       kPeerBufferHeaderBytes) + reduce_elems;
      reduce_segments.push_back(ReduceSegment{prob.y, static_cast<int>(reduce_elems), static_cast<int>(elems)});
      reduce_elems += elems;
    }
    g.M = static_cast<int>(d.M), g.N = static_cast<int>(d.N), g.K = static_cast<int>(d.K);
    g.stage_k = plan.stage_k;
    g.stages_per_unit = plan.kseg / plan.stage_k;
    g.packed_pitch = plan.packed_pitch;
    g.meta_pitch = plan.meta_pitch;
    g.slot_bytes = plan.slot_bytes;
    g.row_tiles = plan.row_tiles;
    max_slot = std::max(max_slot, plan.slot_bytes);
    max_xf = std::max(max_xf, (g.M * g.K * 2 + 127) / 128 * 128);
    max_sx = std::max(max_sx, ((g.K / 64) * 2 * 4 + 127) / 128 * 128);
    total_cost += static_cast<int64_t>(g.row_tiles) * g.stages_per_unit;
    bytes += d.N * d.K / 2 + 8 * d.N * (d.K / 64) + 2 * d.M * d.K + 2 * d.M * d.N;
  }
  const int red_bytes = kRedBuffers * kConsumerWarps * kRows * 4 * 4;
  const int fixed = kHeaderBytes + max_sx + red_bytes + max_xf;
  int slots = (kSmemBudgetTwoCtas - fixed) / max_slot;
  slots = std::min(slots, 6);
  if (slots < 2) {
    *why = "the activations of the largest problem leave no room for the copy ring";
    return cudaErrorInvalidValue;
  }
  const int grid = 2 * sm_count;

  // Cut the stream of units into `grid` contiguous shares of equal cost.  The cost of a unit is its
  // number of pipeline stages, not its bytes: a CTA keeps a fixed number of stages in flight, so
  // under a saturated memory system it retires stages at the same rate whatever their width, and
  // shares with equal stage counts end together (measured on K-split shards with K = 3072 next to
  // K = 4096: balancing by bytes left the CTAs with the narrower stages a third behind).
  std::vector<GroupSegment> segments;
  std::vector<int> first(static_cast<size_t>(grid) + 1, 0);
  {
    int prob = 0, rt = 0;
    int64_t done = 0;
    for (int c = 0; c < grid; ++c) {
      first[static_cast<size_t>(c)] = static_cast<int>(segments.size());
      const int64_t target = total_cost * (c + 1) / grid;
      while (prob < count && (done < target || c == grid - 1)) {
        const GroupProblem& g = problems[static_cast<size_t>(prob)];
        const int left = g.row_tiles - rt;
        const int64_t unit_cost = g.stages_per_unit;
        // Units of this problem that fit below the target (at least one, so that shares advance).
        int64_t take = (target - done + unit_cost - 1) / unit_cost;
        if (c == grid - 1 || take > left) take = left;
        if (take < 1) take = 1;
        segments.push_back(GroupSegment{prob, rt, static_cast<int>(take), 0});
        done += take * unit_cost;
        rt += static_cast<int>(take);
        if (rt == g.row_tiles) ++prob, rt = 0;
      }
    }
    first[static_cast<size_t>(grid)] = static_cast<int>(segments.size());
  }

  const size_t problems_bytes = problems.size() * sizeof(GroupProblem);
  const size_t segments_bytes = (segments.size() * sizeof(GroupSegment) + 127) / 128 * 128;
  const size_t first_bytes = (first.size() * sizeof(int) + 127) / 128 * 128;
  const size_t reduce_bytes = reduce_segments.size() * sizeof(ReduceSegment);
  void* memory = nullptr;
  cudaError_t err = cudaMalloc(&memory, problems_bytes + segments_bytes + first_bytes + reduce_bytes + 16);
  if (err != cudaSuccess) return err;
  char* base = static_cast<char*>(memory);
  err = cudaMemcpy(base, problems.data(), problems_bytes, cudaMemcpyHostToDevice);
  if (err == cudaSuccess && !segments.empty()) {
    err = cudaMemcpy(base + problems_bytes, segments.data(), segments.size() * sizeof(GroupSegment),
                     cudaMemcpyHostToDevice);
  }
  if (err == cudaSuccess) {
    err = cudaMemcpy(base + problems_bytes + segments_bytes, first.data(), first.size() * sizeof(int),
                     cudaMemcpyHostToDevice);
  }
  if (err == cudaSuccess && reduce_bytes > 0) {
    err = cudaMemcpy(base + problems_bytes + segments_bytes + first_bytes, reduce_segments.data(), reduce_bytes,
                     cudaMemcpyHostToDevice);
  }
  if (err == cudaSuccess) {
    err = cudaFuncSetAttribute(w4a16_gemv_grouped_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               216 * 1024);
  }
  if (err != cudaSuccess) {
    cudaFree(memory);
    return err;
  }
  GroupPlan* plan = new GroupPlan;
  cudaGetDevice(&plan->device);
  plan->count = count;
  plan->grid = grid;
  plan->smem_bytes = fixed + slots * max_slot;
  plan->device_memory = memory;
  plan->algorithmic_bytes = bytes;
  plan->params.problems = reinterpret_cast<const GroupProblem*>(base);
  plan->params.segments = reinterpret_cast<const GroupSegment*>(base + problems_bytes);
  plan->params.first_segment = reinterpret_cast<const int*>(base + problems_bytes + segments_bytes);
  plan->params.status = status_word;
  plan->params.slots = slots;
  plan->params.slot_stride = max_slot;
  plan->params.sx_offset = kHeaderBytes;
  plan->params.red_offset = kHeaderBytes + max_sx;
  plan->params.xf_offset = plan->params.red_offset + red_bytes;
  plan->params.ring_offset = plan->params.xf_offset + max_xf;
  plan->params.epoch_word = nullptr;
  plan->params.parity_stride = 0;
  if (!reduce_segments.empty()) {
    unsigned char* own = static_cast<unsigned char*>(exchange->buffers[exchange->rank]);
    plan->params.epoch_word = reinterpret_cast<const unsigned int*>(own + kPeerEpochOffset);
    plan->params.parity_stride = exchange->capacity_n;
    plan->has_reduce = true;
    plan->reduce.exchange = *exchange;
    plan->reduce.segments = reinterpret_cast<const ReduceSegment*>(base + problems_bytes + segments_bytes + first_bytes);
    plan->reduce.segment_count = static_cast<int>(reduce_segments.size());
    int longest = 0;
    for (const ReduceSegment& r : reduce_segments) longest = std::max(longest, r.count);
    plan->reduce.longest = longest;
    plan->reduce.status = status_word;
  }
  *out = plan;
  return cudaSuccess;
}

void group_plan_destroy(GroupPlan* plan) {
  if (plan == nullptr) return;
  cudaFree(plan->device_memory);
  delete plan;
}

int group_plan_device(const GroupPlan* plan) { return plan->device; }
int group_plan_count(const GroupPlan* plan) { return plan->count; }
int64_t group_plan_bytes(const GroupPlan* plan) { return plan->algorithmic_bytes; }

cudaError_t launch_gemv_grouped(const GroupPlan* plan, bool pdl, cudaStream_t stream) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(plan->grid));
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = static_cast<size_t>(plan->smem_bytes);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  const cudaError_t err = cudaLaunchKernelEx(&cfg, w4a16_gemv_grouped_kernel, plan->params);
  if (err != cudaSuccess || !plan->has_reduce) return err;
  return launch_peer_allreduce(plan->reduce, pdl, stream);
}

}  // namespace lbl
