// Host-side interface between the C ABI (api.cu) and the kernel translation units.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

struct CUtensorMap_st;  // driver API tensor map (cuda.h)

namespace lbl {

// One W4A16 problem in the reference layout.  Pointers are device pointers.
struct Problem {
  const __half* x;         // [M, K]
  const uint32_t* packed;  // [N, ceil(K/8)]
  const float* scales;     // [N, ceil(K/64)]
  const int32_t* zeros;    // [N, ceil(K/64)]
  __half* y;               // [M, N]
  int64_t M, N, K;
};

// ----- masked any-shape kernel (generic.cu) ----------------------------------------------------
cudaError_t launch_generic(const Problem& p, bool round_weights_to_fp16, cudaStream_t stream);

// ----- quantiser + packer (quantize.cu) --------------------------------------------------------
// weight [N, K] FP16 or FP32 -> packed [N, ceil(K/8)], scales / zeros [N, ceil(K/64)].
cudaError_t launch_quantize(const void* weight, bool weight_is_fp32, int64_t N, int64_t K,
                            uint32_t* packed, float* scales, int32_t* zeros, cudaStream_t stream);

// packed [N, ceil(K/8)] + scales / zeros -> dense weight [N, K], FP16 or FP32.
cudaError_t launch_dequantize(const uint32_t* packed, const float* scales, const int32_t* zeros,
                              void* out, bool out_is_fp32, int64_t N, int64_t K,
                              cudaStream_t stream);

// ----- streaming skinny kernel, optional split-K (skinny.cu) -----------------------------------
struct SkinnyPlan {
  int kseg;         // columns of K handled by one unit; divides K; multiple of 256
  int nsplit;       // K / kseg
  int stage_k;      // columns of K per pipeline stage; divides kseg; multiple of 256
  int slots;        // depth of the shared-memory ring
  int grid;         // persistent CTAs
  int smem_bytes;   // dynamic shared memory per CTA
  int row_tiles;    // ceil(N / 16)
  bool columns;     // M <= 2: the decode form (gemv_decode.cu) runs instead of the general one
  int packed_pad;   // bytes of padding per packed row in shared memory
  int packed_pitch, meta_pitch, slot_bytes;           // shared-memory layout of one ring slot
  int sx_offset, red_offset, xf_offset, ring_offset;  // regions of the CTA's shared memory
  size_t partial_bytes;  // split-K partial sums (0 when nsplit == 1)
  size_t ticket_bytes;   // arrival counters (0 when nsplit == 1, else kSkinnyTicketBytes)
};

constexpr int kSkinnyMaxM = 32;
// Largest activation operand (M * kseg * 2 bytes) the streaming kernel keeps in shared memory; a
// longer K is cut into segments that meet in scratch memory.
constexpr int kSkinnyOperandBytes = 128 * 1024;
// Split-K scratch layout: a fixed region of arrival counters (one int per 16-row tile) at the
// start, partial sums behind it.  The counter region never moves, whatever the problem, so a
// buffer that was zeroed once stays valid for every later call: counters are left at zero by
// each kernel and partial sums need no initial value.
constexpr size_t kSkinnyTicketBytes = 64 * 1024;
constexpr int kSkinnyMaxSplitRowTiles = static_cast<int>(kSkinnyTicketBytes / sizeof(int));

// True when the skinny kernel can serve the shape (M <= 32, K a multiple of 256).
bool skinny_supports(int64_t M, int64_t N, int64_t K);
// Fills `plan` for the shape; `want_split` < 0 lets the heuristic decide, 0 forbids split-K,
// > 0 asks for at least that many splits where the shape allows it.
bool skinny_make_plan(int64_t M, int64_t N, int64_t K, int want_split, int sm_count,
                      SkinnyPlan* plan);
bool skinny_encode_maps(const Problem& p, const SkinnyPlan& plan, ::CUtensorMap_st* maps);
// Fused K-split all-reduce of the decode GEMV: exchange buffers of all ranks as mapped into this
// process (buffers[rank] is this GPU's own), each holding two FP32 vectors of capacity_n.
struct PeerReduce {
  int rank, world, capacity_n;
  void* buffers[8];
};
constexpr size_t kPeerBufferHeaderBytes = 2048;
cudaError_t launch_gemv_decode(const Problem& p, const SkinnyPlan& plan, float* partials,
                               int* tickets, int* status_word, bool pdl, cudaStream_t stream,
                               const PeerReduce* reduce = nullptr);
cudaError_t launch_skinny(const Problem& p, const SkinnyPlan& plan, float* partials, int* tickets,
                          int* status_word, bool pdl, cudaStream_t stream);

// ----- all-reduce of FP32 vectors over peer memory (peer_reduce.cu) -----------------------------
// Layout of an exchange buffer: a control block (CTAs done, epoch), one flag line per source
// rank, then two FP32 vectors of capacity_n selected by the parity of the epoch.
constexpr size_t kPeerDoneOffset = 0;
constexpr size_t kPeerEpochOffset = 4;
constexpr size_t kPeerFlagsOffset = 128;  // world flags, one 128-byte line each: flags[src] = epoch
// One reduced output: `count` FP32 partial sums at `offset` floats into the vector -> dst FP16.
struct ReduceSegment {
  __half* dst;
  int offset;
  int count;
};
struct PeerReduceLaunch {
  PeerReduce exchange;
  const ReduceSegment* segments;  // device memory
  int segment_count;
  int longest;                    // largest count of any segment
  int* status;
};
// Sums every segment over the ranks (in rank order, FP32) and writes FP16 to its dst on this GPU.
// Every rank must launch it, after the kernel that wrote its own partial sums, on a stream of
// its own device.  Advances the exchange's epoch.
cudaError_t launch_peer_allreduce(const PeerReduceLaunch& launch, bool pdl, cudaStream_t stream);

// Two-shot all-reduce of a K-split GEMM output [M, N] whose partial tiles the GEMM has scattered
// to the owners of their columns (launch_gemm_tc_pair with PairScatter).  Layout of such an
// exchange buffer: the control block as above, `world` slots of [M, N / world] FP16 (slot r =
// rank r's partial of the owner's columns), then the owner's reduced block [M, N / world].
size_t peer_gemm_buffer_bytes(int64_t M, int64_t N, int world);
// Two launches on `stream` (no programmatic dependent launch: they start when the stream's
// earlier work, the scattering GEMM included, is complete): reduce the own columns, then gather
// the peers' columns; y [M, N] ends up identical on all ranks.  Advances the exchange's epoch by 2.
cudaError_t launch_peer_slice_allreduce(const PeerReduce& exchange, __half* y, int64_t M, int64_t N, int sm_count,
                                        int* status, cudaStream_t stream);

// ----- grouped decode GEMV (gemv_grouped.cu) ---------------------------------------------------
struct GroupProblemDesc {
  const void* x;
  const int32_t* packed;
  const float* scales;
  const int32_t* zeros;
  void* y;
  int64_t M, N, K;
  bool reduce;  // K-split shard: y receives the sum over the ranks of the exchange
};
struct GroupPlan;
// Builds the plan (tensor maps, per-CTA work lists) in device memory of the current device.
// Synchronous (cudaMalloc + cudaMemcpy).  `why` receives a reason when the shapes are refused.
cudaError_t group_plan_create(const GroupProblemDesc* descs, int count, int sm_count, int* status_word,
                              const PeerReduce* exchange, GroupPlan** out, const char** why);
void group_plan_destroy(GroupPlan* plan);
int group_plan_device(const GroupPlan* plan);
int group_plan_count(const GroupPlan* plan);
int64_t group_plan_bytes(const GroupPlan* plan);
cudaError_t launch_gemv_grouped(const GroupPlan* plan, bool pdl, cudaStream_t stream);

// ----- TMA + tcgen05 GEMM (gemm_tc.cu) ---------------------------------------------------------
bool gemm_tc_supports(int64_t M, int64_t N, int64_t K);
// `independent`: with `pdl`, do not wait for the previous kernel in the stream at all.
cudaError_t launch_gemm_tc(const Problem& p, int* status_word, cudaStream_t stream, bool pdl, bool independent);

// ----- tcgen05 GEMM for M <= 128, weights on the M side of the MMA (gemm_tc_small.cu) ----------
bool gemm_tc_small_supports(int64_t M, int64_t N, int64_t K);
// Scratch that lets K be cut into slices (0: the shape needs none).  Layout: the fixed region of
// arrival counters, then FP32 partial tiles.  Optional: without it one CTA walks the whole of K.
size_t gemm_tc_small_workspace_bytes(int64_t M, int64_t N, int64_t K, int sm_count);
cudaError_t launch_gemm_tc_small(const Problem& p, int* status_word, cudaStream_t stream, void* workspace,
                                 size_t workspace_bytes, int sm_count, bool pdl);


// ----- TMA + tcgen05 GEMM on pairs of CTAs, cta_group::2 (gemm_tc2.cu) ---------------------------
bool gemm_tc_pair_supports(int64_t M, int64_t N, int64_t K);
// With `scatter` the output does not go to p.y: the tile of columns [o N / world, (o + 1) N / world)
// is written to slot[o], row pitch N / world (this rank's slot in the exchange buffer of rank o).
struct PairScatter {
  __half* slot[8];
  int world;
};
cudaError_t launch_gemm_tc_pair(const Problem& p, int* status_word, cudaStream_t stream, bool pdl, bool independent,
                                const PairScatter* scatter = nullptr);

// ----- tcgen05 GEMM with the weights passed through tensor memory (gemm_wt.cu) ------------------
bool gemm_wt_supports(int64_t M, int64_t N, int64_t K);
// Scratch that lets K be cut into slices when there are few tokens and few row blocks (0: none).
size_t gemm_wt_workspace_bytes(int64_t M, int64_t N, int64_t K, int sm_count);
cudaError_t launch_gemm_wt(const Problem& p, int* status_word, cudaStream_t stream, void* workspace,
                           size_t workspace_bytes, int sm_count, bool pdl);

}  // namespace lbl
