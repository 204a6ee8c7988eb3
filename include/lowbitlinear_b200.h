/*
 * lowbitlinear_b200 -- C ABI of the B200 (sm_100a) W4A16 linear kernels.
 *
 * Computes  Y[M,N] = fp16( X[M,K] . dequant(W)[N,K]^T )  for weights stored as group-64
 * asymmetric INT4:
 *   packed_w  int32 [N, ceil(K/8)]   eight unsigned nibbles per word, low nibble first
 *   scales    float [N, ceil(K/64)]
 *   zeros     int32 [N, ceil(K/64)]  zero points in 0..15
 *   w[n,k] = (q[n,k] - zeros[n,k/64]) * scales[n,k/64]
 * X and Y are IEEE binary16, row-major and dense.  All pointers are device pointers on
 * `device`; nothing is retained after a call returns; no call synchronises the host.
 *
 * Every function returns LBL_OK (0) or a negative code and then leaves a message that
 * lbl_last_error() returns to the same host thread.
 *
 * The entry points replace the two launchers of the reference extension
 * (NanjinLin/LowBitLinear):
 *   lbl_w4a16_gemv  <-  w4a16_gemv_warp_vec_launcher   csrc/w4a16_gemv_warp_vec.cu:111-195
 *   lbl_w4a16_gemm  <-  cute_w4a16_gemm_launcher       csrc/cute_w4a16_gemm.cu:190-248
 * Tensor allocation, dtype/shape/contiguity checks and exception text stay with the host
 * binding, as TORCH_CHECK does for the reference.
 */
#ifndef LOWBITLINEAR_B200_H_
#define LOWBITLINEAR_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LBL_OK 0
#define LBL_ERR_INVALID (-1)     /* null pointer, bad size or misaligned buffer            */
#define LBL_ERR_CUDA (-2)        /* a CUDA runtime call or the launch itself failed         */
#define LBL_ERR_WORKSPACE (-3)   /* workspace missing or smaller than lbl_w4a16_workspace_bytes */
#define LBL_ERR_UNSUPPORTED (-4) /* forced path cannot serve this shape                     */
#define LBL_ERR_DEVICE_WAIT (-5) /* a bounded device-side wait expired (see lbl_device_status) */

/* Kernel paths.  LBL_PATH_AUTO lets the size-based dispatcher choose. */
#define LBL_PATH_AUTO 0
#define LBL_PATH_GENERIC 1      /* masked any-shape kernel (plain loads, FP32 FMA)          */
#define LBL_PATH_GEMV 2         /* streaming skinny kernel, M <= 32, one pass over K        */
#define LBL_PATH_GEMV_SPLITK 3  /* same kernel, K split across CTAs, ordered reduction      */
#define LBL_PATH_GEMM_TC 4      /* TMA + tcgen05 tensor-core GEMM, FP32 accumulators in TMEM */
#define LBL_PATH_GEMM_TC_SMALL 5 /* tcgen05 GEMM for M <= 128: weights on the M side of the MMA,
                                    K cut into slices (uses the scratch when there is one)   */

#define LBL_PATH_GEMM_WT 6       /* tcgen05 GEMM, weights dequantised in registers and handed to the
                                    MMA through tensor memory (any M; K sliced when M is small)  */

#define LBL_PATH_GEMM_TC_PAIR 7 /* the tcgen05 GEMM on pairs of CTAs (cta_group::2): a 512 x 256 tile per
                                    pair that shares one dequantised copy of the weights            */

/* Flags. */
#define LBL_FLAG_PDL 1u            /* programmatic dependent launch: weights are prefetched
                                      before the previous kernel in the stream has finished.
                                      Only set it when that kernel does not write the weights. */
#define LBL_FLAG_ROUND_WEIGHTS 2u  /* round each dequantised weight to FP16 before the multiply (the
                                      reference GEMM's operand policy, csrc/cute_w4a16_gemm.cu:160-162)
                                      also where the dispatcher would pick a streaming kernel, which
                                      keeps the FP32 scale: the any-shape operator then runs a
                                      tensor-core or the masked kernel instead (slower where it matters:
                                      M <= 8, and M <= 16 on shapes with N >= 16384)  */

#define LBL_FLAG_INDEPENDENT 4u    /* with LBL_FLAG_PDL: this call reads nothing that the previous kernel
                                      in the stream writes and writes nothing that it reads or writes,
                                      so it need not wait for it at all; its CTAs then start on the SMs
                                      that the previous kernel's last, partial wave leaves idle.  Honoured
                                      by the large tensor-core GEMMs (LBL_PATH_GEMM_TC, _TC_PAIR), which
                                      use no scratch; every other path keeps waiting.               */

/* Library version: major * 10000 + minor * 100 + patch. */
int lbl_version(void);

/* Message of the last failing call made by the calling thread ("" if none). */
const char* lbl_last_error(void);

/* Path the dispatcher takes for this problem.  `op` is 0 for the M = 1 operator
 * (FP32 dequantisation) and 1 for the any-shape operator. */
int lbl_w4a16_select_path(int64_t M, int64_t N, int64_t K, int op);

/* Bytes of scratch the given path (or LBL_PATH_AUTO) wants for this problem; 0 if none.
 * Split-K GEMV requires it (LBL_ERR_WORKSPACE otherwise); LBL_PATH_GEMM_TC_SMALL uses it to cut K
 * into slices and runs one CTA per 128 output columns without it.
 * The scratch starts with a fixed 64 KiB region of arrival counters (one per 16-row tile or
 * 128-column block), followed by the FP32 partial sums.  The buffer must be zero before the first call that
 * uses it (lbl_w4a16_workspace_init); every call leaves the counters zero again and the
 * counter region never moves, so one buffer can be reused by successive calls, of any
 * shape, on the same stream.  Calls that overlap on the GPU need separate buffers. */
size_t lbl_w4a16_workspace_bytes(int64_t M, int64_t N, int64_t K, int path);

/* Zero a scratch buffer on `stream` (asynchronous). */
int lbl_w4a16_workspace_init(void* workspace, size_t workspace_bytes, int device, void* stream);

/* y[1,N] = fp16( x[1,K] . dequant(W)^T ), FP32 dequantisation and accumulation.
 * Requires group_size == 64, K > 0, K % 64 == 0, N > 0, x 16-byte aligned -- the contract of
 * the reference's w4a16_gemv_warp_vec_launcher (csrc/w4a16_gemv_warp_vec.cu:111-195). */
int lbl_w4a16_gemv(const void* x, const int32_t* packed_w, const float* scales,
                   const int32_t* zeros, void* y, int64_t N, int64_t K, int group_size,
                   void* workspace, size_t workspace_bytes, unsigned flags, int device,
                   void* stream);

/* Y[M,N] for any M, N, K >= 0 (empty outputs are a no-op; K == 0 writes zeros) -- the
 * contract of the reference's cute_w4a16_gemm_launcher (csrc/cute_w4a16_gemm.cu:190-248). */
int lbl_w4a16_gemm(const void* X, const int32_t* packed_w, const float* scales,
                   const int32_t* zeros, void* Y, int64_t M, int64_t N, int64_t K,
                   void* workspace, size_t workspace_bytes, unsigned flags, int device,
                   void* stream);

/* The dispatcher itself: `path` forces a kernel (LBL_ERR_UNSUPPORTED if it cannot serve the
 * shape) or is LBL_PATH_AUTO; `op` selects the numeric policy as in lbl_w4a16_select_path;
 * `path_taken`, when not null, receives the path that ran.  The reference has no counterpart:
 * its choice is made in Python (lowbitlinear/linear.py:100-121). */
int lbl_w4a16_linear(const void* X, const int32_t* packed_w, const float* scales,
                     const int32_t* zeros, void* Y, int64_t M, int64_t N, int64_t K, int op,
                     int path, void* workspace, size_t workspace_bytes, unsigned flags,
                     int device, void* stream, int* path_taken);

/* The M = 1 GEMV for callers that have no way to allocate device memory: a plugin that is
 * handed nothing but input and output pointers by its host application, code that runs where
 * cudaMalloc is not allowed (it synchronises the whole device, and is illegal while a stream
 * is being captured), or a process whose memory budget was fixed up front.  (No counterpart in
 * the reference; its launchers allocate through torch.)
 *
 * It is lbl_w4a16_gemv with K split across CTAs, but the split-K scratch (arrival counters and
 * FP32 partial sums) is a fixed array of lbl_w4a16_gemv_noalloc_scratch_bytes() = 1 MiB inside
 * the library image: every GPU that loads the library holds that megabyte until the process
 * ends, and the call itself performs no cudaMalloc, cudaFree or any other allocation.
 *  - Limit: 64 KiB + nsplit * N * 4 bytes must fit (for example N = 4096 with K = 12288, or
 *    N = 24576 with K = 4096).  Larger problems are rejected with LBL_ERR_WORKSPACE and a
 *    message; use lbl_w4a16_gemv with your own workspace for those.
 *  - The first call on each device looks up the array's device address and clears its counters
 *    on `stream`; make that first call outside any stream capture.
 *  - All calls on a device share the one array, which keeps what the last call left in it (the
 *    kernel puts its counters back to zero before it ends).  Two calls that overlap on the GPU,
 *    for instance from different streams, race on it; serialise them.
 * Same argument contract as lbl_w4a16_gemv otherwise (K % 256 == 0, 16-byte aligned tensors). */
size_t lbl_w4a16_gemv_noalloc_scratch_bytes(void);
int lbl_w4a16_gemv_noalloc(const void* x, const int32_t* packed_w, const float* scales,
                           const int32_t* zeros, void* y, int64_t N, int64_t K, int group_size,
                           unsigned flags, int device, void* stream);

/* ---- Row-parallel (K-split) GEMV with the all-reduce fused into the kernel -----------------
 * The reference has no multi-GPU code; this is the tensor-parallel form of its Down projection.
 * Every rank (one process per GPU, same node) owns an exchange buffer created with
 * lbl_peer_buffer_create, exports its 64-byte IPC handle, and opens the handles of its peers.
 * lbl_w4a16_gemv_allreduce computes this rank's partial y over its K slice, leaves the FP32
 * vector in its own buffer, raises a flag in every peer's buffer, waits (bounded, about 2 s)
 * for the peers' flags, and adds the ranks' vectors in rank order over NVLink peer loads:
 * every rank ends with the same FP16 y[1, N].  All ranks must make the same sequence of calls.
 * buffers[r] is rank r's buffer as mapped in this process (buffers[rank] = own buffer),
 * buffer_capacity_n the max_n all buffers were sized for.  Buffers are double-buffered by
 * call parity, so calls may follow each other without a host synchronisation. */
size_t lbl_peer_buffer_bytes(int64_t max_n);
int lbl_peer_buffer_create(size_t bytes, int device, void** buffer);
int lbl_peer_buffer_export(const void* buffer, void* handle64);
/* Diagnostics: copies `bytes` at `offset` of the buffer's 2 KiB control block to the host
 * (synchronous).  Bytes 1536..2047 hold eight records of eight 64-bit %globaltimer stamps when the
 * library was built with -D LBL_TRACE_EXCHANGE (start and end of the grouped GEMV; entry, end of
 * the wait for the GEMV, flags complete, sums complete and epoch update of the all-reduce kernel);
 * zeros otherwise. */
int lbl_peer_buffer_peek(const void* buffer, size_t offset, void* host_dst, size_t bytes, int device);
int lbl_peer_buffer_open(const void* handle64, int device, void** buffer);
int lbl_peer_buffer_close(void* buffer, int device);
int lbl_peer_buffer_destroy(void* buffer, int device);
int lbl_w4a16_gemv_allreduce(const void* x, const int32_t* packed_w, const float* scales,
                             const int32_t* zeros, void* y, int64_t N, int64_t K, int group_size,
                             int rank, int world, void* const* buffers, int64_t buffer_capacity_n,
                             void* workspace, size_t workspace_bytes, unsigned flags, int device,
                             void* stream);

/* ---- K-split GEMM with the all-reduce fused into it (large M, tensor parallel) ----------------
 * The reference has no multi-GPU path; this is the large-M counterpart of
 * lbl_w4a16_gemv_allreduce.  Rank r holds columns [r K / world, (r + 1) K / world) of the weight
 * (x, packed_w, scales, zeros are the rank's shard; K is the shard's K).  Rank o owns the output
 * columns [o N / world, (o + 1) N / world).
 *   lbl_w4a16_gemm_scatter            the tcgen05 GEMM on CTA pairs; each finished 512 x 256 tile of
 *                                     partial outputs is stored, FP16, straight into the exchange
 *                                     buffer of the rank that owns its columns (NVLink peer stores
 *                                     from the epilogue, tile by tile while the GEMM runs).
 *   lbl_peer_gemm_allreduce_finish    two launches: (1) flags to and from every peer, then each
 *                                     rank adds the `world` partials of its own columns in rank
 *                                     order (FP32 sums, one rounding to FP16) into y and into its
 *                                     result block; (2) flags again, then each rank copies the
 *                                     peers' result blocks into y with vector loads over NVLink.
 *                                     Every rank ends with the same bits in y[M, N].
 *   lbl_w4a16_gemm_allreduce          both, on one stream.
 * Exchange buffers: lbl_peer_buffer_create(lbl_peer_gemm_buffer_bytes(M, N, world)), exported and
 * opened like the decode buffers; buffers[r] is rank r's buffer as mapped here, buffer_bytes the
 * size all of them have.  One all-reduce per set of buffers at a time: the next scatter into them
 * must be ordered after this rank's finish (same stream, or an event when finish runs on a side
 * stream so that other GEMMs overlap it).  All ranks make the same sequence of calls.  Needs
 * N % (256 * world) == 0 and K % 256 == 0; LBL_FLAG_PDL / LBL_FLAG_INDEPENDENT apply to the GEMM
 * launch.  Waits for peers are bounded (about 2 s): on expiry y is filled with NaN and
 * lbl_device_status reports 110. */
size_t lbl_peer_gemm_buffer_bytes(int64_t M, int64_t N, int world);
int lbl_w4a16_gemm_scatter(const void* x, const int32_t* packed_w, const float* scales,
                           const int32_t* zeros, int64_t M, int64_t N, int64_t K, int rank, int world,
                           void* const* buffers, size_t buffer_bytes, unsigned flags, int device,
                           void* stream);
int lbl_peer_gemm_allreduce_finish(void* y, int64_t M, int64_t N, int rank, int world,
                                   void* const* buffers, size_t buffer_bytes, int device,
                                   void* stream);
int lbl_w4a16_gemm_allreduce(const void* x, const int32_t* packed_w, const float* scales,
                             const int32_t* zeros, void* y, int64_t M, int64_t N, int64_t K, int rank,
                             int world, void* const* buffers, size_t buffer_bytes, unsigned flags,
                             int device, void* stream);

/* ---- Grouped decode GEMV: many independent problems, one launch ------------------------------
 * The reference launches one kernel per linear (csrc/w4a16_gemv_warp_vec.cu:171-187); at decode
 * sizes the fixed cost of a launch rivals the time its weights need to cross the memory bus.  A
 * group describes a list of problems with M <= 2 once -- lbl_w4a16_group_create builds their
 * tensor maps and cuts the byte stream of all weights into one contiguous share per persistent
 * CTA, in device memory it allocates (a synchronous set-up call) -- and lbl_w4a16_group_run then
 * computes all of them in ONE launch on `stream`, reading x and writing y of every problem as
 * given at creation (static buffers, which is also what CUDA-graph capture wants).
 *  - The problems must be independent: no problem's x may be another problem's y.
 *  - Per problem: 1 <= M <= 2, K % 256 == 0, M * K <= 32768, all tensors 16-byte aligned;
 *    FP32-scale numerics of lbl_w4a16_gemv.
 *  - Tensor parallel: create the group on every rank with that rank's shards, pass the exchange
 *    buffers of all ranks (lbl_peer_buffer_*) and set `reduce` on the K-split problems; run then
 *    launches a second kernel that sums those problems' FP32 partial outputs over the ranks with
 *    plain peer loads over NVLink (bounded wait for the peers; NaN outputs and a non-zero
 *    lbl_device_status if a peer never shows up) and writes the same FP16 y on every rank.  All
 *    ranks must run their groups the same number of times.  With world == 1 pass rank 0,
 *    world 1, buffers NULL.
 * A group may be run any number of times, also inside a stream capture; destroy it after the
 * last run has finished. */
typedef struct lbl_w4a16_problem {
  const void* x;            /* [M, K] FP16 */
  const int32_t* packed_w;  /* [N, K/8] */
  const float* scales;      /* [N, K/64] */
  const int32_t* zeros;     /* [N, K/64] */
  void* y;                  /* [M, N] FP16 */
  int64_t M, N, K;
  int32_t reduce;           /* 1: K-split shard, y = sum over the ranks (needs the exchange) */
  int32_t reserved;
} lbl_w4a16_problem;
typedef struct lbl_w4a16_group lbl_w4a16_group;
int lbl_w4a16_group_create(const lbl_w4a16_problem* problems, int count, int rank, int world,
                           void* const* buffers, int64_t buffer_capacity_n, int device,
                           lbl_w4a16_group** group);
int lbl_w4a16_group_run(lbl_w4a16_group* group, unsigned flags, void* stream);
/* Sum over the problems of N K / 2 + 8 N K / 64 + 2 M K + 2 M N (what a benchmark divides by). */
int64_t lbl_w4a16_group_algorithmic_bytes(const lbl_w4a16_group* group);
int lbl_w4a16_group_destroy(lbl_w4a16_group* group);

/* ---- Quantiser -----------------------------------------------------------------------------
 * Replaces QuantizedLinear.from_float's quantize_int4 + pack_int4 pair
 * (lowbitlinear/linear.py:55-76, lowbitlinear/quantization.py:33-86 and :112-141) for weights
 * that are already on the GPU: one kernel reads weight [N, K] (FP16, or FP32 when
 * weight_is_fp32 != 0; row-major contiguous) and writes packed_w [N, ceil(K/8)],
 * scales [N, ceil(K/64)] and zeros [N, ceil(K/64)].  The arithmetic is the reference's CPU
 * arithmetic (IEEE FP32 division, round half to even, no fused multiply-add), so all three
 * outputs are bit-identical to the reference run on CPU tensors; columns past K pack as level 0.
 * group_size must be 64 (LBL_ERR_UNSUPPORTED otherwise); any N >= 0 and K >= 1. */
int lbl_w4a16_quantize(const void* weight, int weight_is_fp32, int64_t N, int64_t K,
                       int group_size, int32_t* packed_w, float* scales, int32_t* zeros,
                       int device, void* stream);

/* The inverse for weights on the GPU: unpack_int4 + dequantize_int4
 * (lowbitlinear/quantization.py:143-171 and :88-110) in one kernel.  Writes weight [N, K] =
 * float(q - zero) * scale, as FP32 (weight_is_fp32 != 0, bit-identical to the reference) or
 * rounded once to FP16 (the dense matrix the reference benchmark's pre-dequantised baseline
 * multiplies, benchmarks/bench_w4a16.py:37-43).  group_size must be 64. */
int lbl_w4a16_dequantize(const int32_t* packed_w, const float* scales, const int32_t* zeros,
                         void* weight, int weight_is_fp32, int64_t N, int64_t K, int group_size,
                         int device, void* stream);

/* Reads (and clears) the device-side status word of `device`: 0, or a code left by a
 * kernel whose bounded wait on a barrier expired.  Synchronises the device. */
int lbl_device_status(int device, int* status);

#ifdef __cplusplus
}
#endif

#endif /* LOWBITLINEAR_B200_H_ */
