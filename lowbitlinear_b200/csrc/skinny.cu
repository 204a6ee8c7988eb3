// Streaming W4A16 kernel for skinny activations (M <= 32): the decode GEMV and its split-K form.
//
// The kernel is HBM-bound: 0.625 bytes per weight (packed nibble + its share of scale and zero
// point) against 2 M flops.  Its job is to keep enough bytes in flight and to spend as few issue
// slots per weight as possible.
//
// Data movement.  A persistent CTA walks a list of units; a unit is 16 weight rows by `kseg`
// columns.  One producer warp streams the unit through a ring of shared-memory slots with three
// tiled TMA copies per slot (cp.async.bulk.tensor, completion counted on an mbarrier): 16 rows
// of packed words plus the matching scale and zero-point rows, each read straight from the
// reference layout ([N, K/8] words, [N, K/64] metadata).  The copy box is wider than the
// tensor's inner extent, so the rows land with a zero-filled pad whose pitch keeps the fragment
// loads below bank-conflict free at no cost in traffic.  Weight copies never depend on
// the previous kernel in the stream, so with programmatic dependent launch they start while that
// kernel is still draining; only the activation read waits for it.
//
// Arithmetic.  Eight consumer warps share a slot by quantisation group.  For one group (16 rows
// by 64 columns) a warp loads 8 bytes per lane and row, turns each word into four half2 values
// with one shift and four ANDs (nibbles become FP16 subnormals, see common.cuh), and issues four
// m16n8k16 warp MMAs whose A operand is the raw levels q and whose B operand is the activation
// block; FP32 accumulation.  The group's scale and zero point are applied once, in FP32:
//     acc += scale * (sum_k q x  -  zero * sum_k x)
// with the per-group activation sums computed once per CTA.  (q - zero) is never formed and the
// scale is never rounded to FP16.
//
// Reduction.  The warps' partial rows are added in a fixed order through shared memory.  With
// split-K, every unit writes FP32 partials to scratch and takes a ticket for its row tile; the
// CTA that draws the last ticket adds the partials in split order and writes FP16, then puts the
// ticket counter back to zero.  Results are bit-reproducible from run to run.
#include "common.cuh"
#include "kernels.h"
#include "tensor_map.h"

#include <algorithm>
#include <type_traits>

namespace lbl {
namespace {

constexpr int kRows = 16;
constexpr int kConsumerWarps = 8;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kThreads = kConsumerThreads + 32;
constexpr int kMaxSlots = 8;
constexpr int kHeaderBytes = 384;
constexpr int kMaxStageK = 2048;
// Activation operand kept in shared memory.  Up to 64 KB two CTAs share an SM; a larger operand
// leaves room for one, which still beats cutting K (Down at M = 4: 18 against 24 us; Gate/Up at
// M = 16: 40 against 82 us).
constexpr int kXfBudgetBytes = kSkinnyOperandBytes;
constexpr int kSmemBudgetTwoCtas = 110 * 1024;
constexpr int kSmemBudgetOneCta = 200 * 1024;

struct KernelParams {
  const __half* x;
  __half* y;
  float* partials;
  int* tickets;
  int* status;
  int M, N, K;
  int kseg, nsplit, stage_k, stages_per_unit, slots;
  int row_tiles, units;
  int packed_pitch;  // bytes between rows of a slot's packed block
  int meta_pitch;    // bytes between rows of a slot's scale / zero block
  int slot_bytes;
  int sx_offset, red_offset, xf_offset, ring_offset;  // shared-memory layout
};

struct Header {
  uint64_t full[kMaxSlots];
  uint64_t empty[kMaxSlots];
  int abort_flag;
  int ticket;
};
static_assert(sizeof(Header) <= kHeaderBytes, "header does not fit");

__device__ __forceinline__ uint32_t pack_half2(__half lo, __half hi) {
  return static_cast<uint32_t>(__half_as_ushort(lo)) |
         (static_cast<uint32_t>(__half_as_ushort(hi)) << 16);
}

// Builds, for the K segment starting at column `k_begin`, the MMA B operand of every
// (group, step) and the per-group activation sums.  Runs on the 256 consumer threads.
//
// Column layout inside a group: lane t of a quad owns words 2t and 2t+1 (columns 16t..16t+15).
// Word half h and nibble pair p give MMA step s = 2h + p, whose four k-slots in this lane are
//   b0 = (x[c + 0], x[c + 4])          c = 64 G + 16 t + 8 h + 2 p
//   b1 = (x[c + 1], x[c + 5]) / 16     (the odd nibbles carry a factor 16, see common.cuh)
template <int NT>
__device__ __forceinline__ void build_activation_operand(const KernelParams& p, int k_begin,
                                                         uint2* xf, float* sx, int tid) {
  constexpr int MC = 8 * NT;
  const int groups = p.kseg / 64;
  const int words_seg = p.kseg / 8;
  for (int i = tid; i < groups * MC; i += kConsumerThreads) {
    if (i % MC >= p.M) sx[i] = 0.0f;
  }
  const __half sixteenth = __float2half_rn(0.0625f);
  const int total = p.M * words_seg;  // multiple of 32: whole warps stay together below
  // The loads of a batch are issued before the first one is used: one trip to the L2 per batch
  // instead of one per pass (the shuffles would otherwise keep each pass's load behind the
  // arithmetic of the pass before).
  constexpr int kBatch = 4;
  for (int first = 0; first < total; first += kBatch * kConsumerThreads) {
    uint4 raw[kBatch];
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      const int idx = first + j * kConsumerThreads + tid;
      if (idx < total) {
        const int m = idx / words_seg;
        const int wd = idx - m * words_seg;
        raw[j] = __ldcg(reinterpret_cast<const uint4*>(p.x + static_cast<size_t>(m) * p.K + k_begin + wd * 8));
      }
    }
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      const int idx = first + j * kConsumerThreads + tid;
      if (idx >= total) break;
      const int m = idx / words_seg;
      const int wd = idx - m * words_seg;
      const __half2 v01 = *reinterpret_cast<const __half2*>(&raw[j].x);
      const __half2 v23 = *reinterpret_cast<const __half2*>(&raw[j].y);
      const __half2 v45 = *reinterpret_cast<const __half2*>(&raw[j].z);
      const __half2 v67 = *reinterpret_cast<const __half2*>(&raw[j].w);
      const __half x0 = __low2half(v01), x1 = __high2half(v01);
      const __half x2 = __low2half(v23), x3 = __high2half(v23);
      const __half x4 = __low2half(v45), x5 = __high2half(v45);
      const __half x6 = __low2half(v67), x7 = __high2half(v67);
      float sum = ((__half2float(x0) + __half2float(x1)) + (__half2float(x2) + __half2float(x3))) +
                  ((__half2float(x4) + __half2float(x5)) + (__half2float(x6) + __half2float(x7)));
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      sum += __shfl_xor_sync(0xffffffffu, sum, 4);
      const int group = wd >> 3;
      const int wq = wd & 7;
      const int t = wq >> 1;
      const int h = wq & 1;
      uint2 step0, step1;
      step0.x = pack_half2(x0, x4);
      step0.y = pack_half2(__hmul(x1, sixteenth), __hmul(x5, sixteenth));
      step1.x = pack_half2(x2, x6);
      step1.y = pack_half2(__hmul(x3, sixteenth), __hmul(x7, sixteenth));
      xf[((group * 4 + 2 * h) * p.M + m) * 4 + t] = step0;
      xf[((group * 4 + 2 * h + 1) * p.M + m) * 4 + t] = step1;
      if (wq == 0) sx[group * MC + m] = sum;
    }
  }
}

template <int NT>
__global__ void __launch_bounds__(kThreads, (NT <= 2 ? 2 : 1))
    w4a16_skinny_kernel(const __grid_constant__ CUtensorMap tmap_w,
                        const __grid_constant__ CUtensorMap tmap_s,
                        const __grid_constant__ CUtensorMap tmap_z, const KernelParams p) {
  constexpr int MC = 8 * NT;
  extern __shared__ __align__(128) uint8_t smem[];
  Header* hdr = reinterpret_cast<Header*>(smem);
  float* sx = reinterpret_cast<float*>(smem + p.sx_offset);
  float* red = reinterpret_cast<float*>(smem + p.red_offset);
  uint2* xf = reinterpret_cast<uint2*>(smem + p.xf_offset);
  uint8_t* ring = smem + p.ring_offset;
  volatile int* abort_flag = &hdr->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.slots; ++s) {
      mbar_init(&hdr->full[s], 1);
      mbar_init(&hdr->empty[s], kConsumerWarps);
    }
    hdr->abort_flag = 0;
    hdr->ticket = 0;
    mbar_init_fence();
  }
  __syncthreads();
  // The next kernel in the stream may start filling its own ring as soon as it finds room.
  pdl_allow_next_kernel();

  const int zeros_block = kRows * p.packed_pitch + kRows * p.meta_pitch;

  if (warp == kConsumerWarps) {
    // ------------------------------- producer ------------------------------------------------
    // Weights are read once per call: first in line for eviction from the L2.
    const uint64_t stream_once = l2_evict_first_policy();
    int slot = 0, round = 0;  // ring position, advanced by counting
    for (int unit = blockIdx.x; unit < p.units; unit += gridDim.x) {
      const int ks = unit / p.row_tiles;
      const int rt = unit - ks * p.row_tiles;
      const int n0 = rt * kRows;
      for (int st = 0; st < p.stages_per_unit; ++st) {
        if (round > 0) {
          mbar_wait_bounded(&hdr->empty[slot], (round - 1) & 1, abort_flag, p.status,
                            kStatusSkinnyEmptyWait);
        }
        if (*abort_flag) break;
        // Stage index along K: the tensor maps view every row as [K / stage_k][stage_k].
        const int stage_index = ks * p.stages_per_unit + st;
        if (lane == 0) {
          // Three tiled copies per stage; each box is 16 rows by (stage columns + padding), the
          // padding lies outside the tensor's inner extent and is zero-filled without traffic,
          // as are rows past N.  A box always counts its full size on the barrier.
          uint8_t* base = ring + static_cast<size_t>(slot) * p.slot_bytes;
          mbar_arrive_expect_tx(&hdr->full[slot], static_cast<uint32_t>(p.slot_bytes));
          tma_load_3d_hint(base, &tmap_w, 0, stage_index, n0, &hdr->full[slot], stream_once);
          tma_load_3d_hint(base + kRows * p.packed_pitch, &tmap_s, 0, stage_index, n0, &hdr->full[slot],
                           stream_once);
          tma_load_3d_hint(base + zeros_block, &tmap_z, 0, stage_index, n0, &hdr->full[slot], stream_once);
        }
        if (++slot == p.slots) slot = 0, ++round;
      }
      if (*abort_flag) break;
    }
    return;
  }

  // --------------------------------- consumers -----------------------------------------------
  const int tid = threadIdx.x;  // 0..255
  const int g = lane >> 2;
  const int t = lane & 3;
  const int groups_per_stage = p.stage_k / 64;
  const float zero4[4] = {0.0f, 0.0f, 0.0f, 0.0f};

  int slot = 0, parity = 0;  // ring position, advanced by counting
  int current_ks = -1;
  for (int unit = blockIdx.x; unit < p.units; unit += gridDim.x) {
    const int ks = unit / p.row_tiles;
    const int rt = unit - ks * p.row_tiles;
    const int n0 = rt * kRows;

    if (ks != current_ks) {
      // Activations are the only input the previous kernel may have produced.
      if (current_ks < 0) pdl_wait_for_previous_kernel();
      build_activation_operand<NT>(p, ks * p.kseg, xf, sx, tid);
      named_barrier(1, kConsumerThreads);
      current_ks = ks;
    }

    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[nt][i] = 0.0f;
    }

    for (int st = 0; st < p.stages_per_unit; ++st) {
      mbar_wait_bounded(&hdr->full[slot], parity, abort_flag, p.status, kStatusSkinnyFullWait);

      const uint8_t* base = ring + static_cast<size_t>(slot) * p.slot_bytes;
      const uint8_t* row_a = base + g * p.packed_pitch + t * 8;
      const uint8_t* row_b = row_a + 8 * p.packed_pitch;
      const float* sc_a = reinterpret_cast<const float*>(base + kRows * p.packed_pitch + g * p.meta_pitch);
      const float* sc_b = reinterpret_cast<const float*>(base + kRows * p.packed_pitch + (g + 8) * p.meta_pitch);
      const int* zp_a = reinterpret_cast<const int*>(base + zeros_block + g * p.meta_pitch);
      const int* zp_b = reinterpret_cast<const int*>(base + zeros_block + (g + 8) * p.meta_pitch);

      // U groups are processed together and every group runs two MMA chains (steps 0-1 and
      // steps 2-3), so that 2 U independent tensor-core instructions are in flight per warp.
      auto run_groups = [&](auto u_tag, int G0) {
        constexpr int U = decltype(u_tag)::value;
        uint2 wa[U], wb[U];
        float scale_a[U], scale_b[U], zero_a[U], zero_b[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int G = G0 + u * kConsumerWarps;
          wa[u] = *reinterpret_cast<const uint2*>(row_a + G * 32);
          wb[u] = *reinterpret_cast<const uint2*>(row_b + G * 32);
          scale_a[u] = sc_a[G];
          scale_b[u] = sc_b[G];
          zero_a[u] = static_cast<float>(zp_a[G]);
          zero_b[u] = static_cast<float>(zp_b[G]);
        }
        uint32_t ha[U][8], hb[U][8];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          uint32_t q[4];
          nibbles_as_subnormal_half2(wa[u].x, q);
          ha[u][0] = q[0]; ha[u][1] = q[1]; ha[u][2] = q[2]; ha[u][3] = q[3];
          nibbles_as_subnormal_half2(wa[u].y, q);
          ha[u][4] = q[0]; ha[u][5] = q[1]; ha[u][6] = q[2]; ha[u][7] = q[3];
          nibbles_as_subnormal_half2(wb[u].x, q);
          hb[u][0] = q[0]; hb[u][1] = q[1]; hb[u][2] = q[2]; hb[u][3] = q[3];
          nibbles_as_subnormal_half2(wb[u].y, q);
          hb[u][4] = q[0]; hb[u][5] = q[1]; hb[u][6] = q[2]; hb[u][7] = q[3];
        }
        float d[U][2][NT][4];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            const int s = 2 * c + j;  // chain c covers steps 2c and 2c + 1
#pragma unroll
            for (int u = 0; u < U; ++u) {
              const int group_in_seg = st * groups_per_stage + G0 + u * kConsumerWarps;
              const uint2* xf_step = xf + (static_cast<size_t>(group_in_seg) * 4 + s) * p.M * 4 + t;
              const uint32_t a[4] = {ha[u][2 * s], hb[u][2 * s], ha[u][2 * s + 1], hb[u][2 * s + 1]};
#pragma unroll
              for (int nt = 0; nt < NT; ++nt) {
                const int n = nt * 8 + g;
                uint2 b = make_uint2(0u, 0u);
                if (n < p.M) b = xf_step[n * 4];
                if (j == 0) {
                  mma_m16n8k16(d[u][c][nt], a, b.x, b.y, zero4);
                } else {
                  mma_m16n8k16(d[u][c][nt], a, b.x, b.y, d[u][c][nt]);
                }
              }
            }
          }
        }
        // acc += scale * (sum q x) - (scale * zero) * (sum x); the MMA result carries the
        // factor 1 / kNibbleUnit of the nibble encoding.
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int group_in_seg = st * groups_per_stage + G0 + u * kConsumerWarps;
          const float fa = scale_a[u] * kNibbleUnit;
          const float fb = scale_b[u] * kNibbleUnit;
          const float ca = -(scale_a[u] * zero_a[u]);
          const float cb = -(scale_b[u] * zero_b[u]);
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            const float2 sums =
                *reinterpret_cast<const float2*>(sx + group_in_seg * MC + nt * 8 + 2 * t);
            acc[nt][0] = fmaf(fa, d[u][0][nt][0] + d[u][1][nt][0], acc[nt][0]);
            acc[nt][1] = fmaf(fa, d[u][0][nt][1] + d[u][1][nt][1], acc[nt][1]);
            acc[nt][2] = fmaf(fb, d[u][0][nt][2] + d[u][1][nt][2], acc[nt][2]);
            acc[nt][3] = fmaf(fb, d[u][0][nt][3] + d[u][1][nt][3], acc[nt][3]);
            acc[nt][0] = fmaf(ca, sums.x, acc[nt][0]);
            acc[nt][1] = fmaf(ca, sums.y, acc[nt][1]);
            acc[nt][2] = fmaf(cb, sums.x, acc[nt][2]);
            acc[nt][3] = fmaf(cb, sums.y, acc[nt][3]);
          }
        }
      };
      constexpr int kUnroll = NT == 1 ? 2 : 1;
      int G = warp;
      for (; G + (kUnroll - 1) * kConsumerWarps < groups_per_stage; G += kUnroll * kConsumerWarps) {
        run_groups(std::integral_constant<int, kUnroll>{}, G);
      }
      for (; G < groups_per_stage; G += kConsumerWarps) {
        run_groups(std::integral_constant<int, 1>{}, G);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&hdr->empty[slot]);
      if (++slot == p.slots) slot = 0, parity ^= 1;
    }

    // ---- cross-warp reduction of the unit, fixed order ---------------------------------------
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      float* r0 = red + (warp * kRows + g) * MC + nt * 8 + 2 * t;
      float* r1 = red + (warp * kRows + g + 8) * MC + nt * 8 + 2 * t;
      r0[0] = acc[nt][0];
      r0[1] = acc[nt][1];
      r1[0] = acc[nt][2];
      r1[1] = acc[nt][3];
    }
    named_barrier(1, kConsumerThreads);
    for (int o = tid; o < kRows * MC; o += kConsumerThreads) {
      const int col = o / kRows;
      const int row = o - col * kRows;
      float v = 0.0f;
#pragma unroll
      for (int w = 0; w < kConsumerWarps; ++w) v += red[(w * kRows + row) * MC + col];
      if (col < p.M && n0 + row < p.N) {
        if (p.nsplit == 1) {
          p.y[static_cast<size_t>(col) * p.N + n0 + row] = __float2half_rn(v);
        } else {
          p.partials[(static_cast<size_t>(ks) * p.M + col) * p.N + n0 + row] = v;
        }
      }
    }
    if (p.nsplit > 1) {
      __threadfence();
      named_barrier(1, kConsumerThreads);
      if (tid == 0) hdr->ticket = atomicAdd(&p.tickets[rt], 1);
      named_barrier(1, kConsumerThreads);
      if (hdr->ticket == p.nsplit - 1) {
        __threadfence();
        for (int o = tid; o < kRows * MC; o += kConsumerThreads) {
          const int col = o / kRows;
          const int row = o - col * kRows;
          if (col < p.M && n0 + row < p.N) {
            float v = 0.0f;
            for (int s = 0; s < p.nsplit; ++s) {
              v += __ldcg(&p.partials[(static_cast<size_t>(s) * p.M + col) * p.N + n0 + row]);
            }
            p.y[static_cast<size_t>(col) * p.N + n0 + row] = __float2half_rn(v);
          }
        }
        if (tid == 0) p.tickets[rt] = 0;
      }
    }
    named_barrier(1, kConsumerThreads);
  }
}

template <int NT>
cudaError_t launch_nt(const CUtensorMap (&maps)[3], const KernelParams& kp, const SkinnyPlan& plan,
                      bool pdl, cudaStream_t stream) {
  // The opt-in to large dynamic shared memory is per device and per kernel; repeating it is
  // harmless, so a racy "done" flag is enough.
  static bool configured[64] = {};
  int device = 0;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess) return err;
  if (device < 0 || device >= 64 || !configured[device]) {
    err = cudaFuncSetAttribute(w4a16_skinny_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               kSmemBudgetOneCta + 16 * 1024);
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
  return cudaLaunchKernelEx(&cfg, w4a16_skinny_kernel<NT>, maps[0], maps[1], maps[2], kp);
}

}  // namespace

bool skinny_supports(int64_t M, int64_t N, int64_t K) {
  return M >= 1 && M <= kSkinnyMaxM && N >= 1 && K >= 256 && K % 256 == 0 &&
         N <= 0x7fffffffLL - kRows && K <= (1 << 24) && M * N <= 0x7fffffffLL;
}

bool skinny_make_plan(int64_t M, int64_t N, int64_t K, int want_split, int sm_count,
                      SkinnyPlan* plan) {
  if (!skinny_supports(M, N, K)) return false;
  const int m = static_cast<int>(M);
  const int k = static_cast<int>(K);
  const int nt = m <= 8 ? 1 : (m <= 16 ? 2 : 4);
  const int mc = 8 * nt;
  const int row_tiles = static_cast<int>((N + kRows - 1) / kRows);
  const int chunks = k / 256;

  // Candidate splits: every divisor d of K / 256 gives kseg = K / d.
  const int kseg_cap = std::max(256, (kXfBudgetBytes / (2 * m)) / 256 * 256);
  const int target_units = sm_count;  // split K only when the row tiles cannot fill the SMs
  const int forced = want_split > 0 ? want_split : 0;
  int nsplit = 0;
  for (int d = 1; d <= chunks; ++d) {
    if (chunks % d != 0) continue;
    const int kseg = k / d;
    if (kseg > kseg_cap) continue;
    if (d > 1 && row_tiles > kSkinnyMaxSplitRowTiles) break;  // counters would not fit
    nsplit = d;
    if (forced > 0) {
      if (d >= forced) break;
      continue;
    }
    if (want_split == 0) break;                                      // no more than necessary
    if (static_cast<int64_t>(row_tiles) * d >= target_units) break;  // enough units
    if (kseg <= 1024) break;                                         // pieces would get too small
  }
  if (nsplit == 0) return false;
  const int kseg = k / nsplit;

  int stage_k = 256;
  for (int c = kMaxStageK / 256; c >= 1; --c) {
    if (kseg % (256 * c) == 0) {
      stage_k = 256 * c;
      break;
    }
  }

  // The decode form (M <= 2) reads 16 bytes per lane and needs a row pitch of 64 mod 128 bytes;
  // the general form reads 8 bytes per lane and needs 32 mod 128.
  const bool columns = m <= 2;
  const int packed_pad = columns ? 64 : 32;
  const int packed_pitch = stage_k / 2 + packed_pad;
  const int meta_pitch = stage_k / 16 + 16;
  const int slot_bytes = kRows * packed_pitch + 2 * kRows * meta_pitch;
  auto round128 = [](int v) { return (v + 127) / 128 * 128; };
  const int sx_bytes = round128(columns ? (kseg / 64) * 2 * 4 : (kseg / 64) * mc * 4);
  // Decode form: eight buffers of unit results (see gemv_decode.cu), general form: one.
  const int red_bytes = round128(columns ? 8 * kConsumerWarps * kRows * 4 * 4 : kConsumerWarps * kRows * mc * 4);
  const int xf_bytes = round128(m * kseg * 2);
  const int fixed = kHeaderBytes + sx_bytes + red_bytes + xf_bytes;

  int budget = kSmemBudgetTwoCtas;
  int per_sm = 2;
  if (fixed + 2 * slot_bytes > budget) {
    budget = kSmemBudgetOneCta;
    per_sm = 1;
  }
  int slots = (budget - fixed) / slot_bytes;
  slots = std::min(slots, columns ? 6 : kMaxSlots);
  if (slots < 2) return false;

  const int64_t units = static_cast<int64_t>(row_tiles) * nsplit;
  plan->kseg = kseg;
  plan->nsplit = nsplit;
  plan->stage_k = stage_k;
  plan->slots = slots;
  plan->grid = static_cast<int>(std::min<int64_t>(units, static_cast<int64_t>(per_sm) * sm_count));
  plan->smem_bytes = fixed + slots * slot_bytes;
  plan->row_tiles = row_tiles;
  plan->columns = columns;
  plan->packed_pad = packed_pad;
  plan->packed_pitch = packed_pitch;
  plan->meta_pitch = meta_pitch;
  plan->slot_bytes = slot_bytes;
  plan->sx_offset = kHeaderBytes;
  plan->red_offset = plan->sx_offset + sx_bytes;
  plan->xf_offset = plan->red_offset + red_bytes;
  plan->ring_offset = plan->xf_offset + xf_bytes;
  plan->partial_bytes = nsplit > 1 ? static_cast<size_t>(nsplit) * M * N * sizeof(float) : 0;
  plan->ticket_bytes = nsplit > 1 ? kSkinnyTicketBytes : 0;
  return units <= 0x7fffffffLL;
}

// Tensor maps over the reference layout.  Each row is viewed as [K / stage_k][stage_k]; a box
// takes 16 rows of one stage plus a few elements of padding per row.  The padding is outside the
// inner extent, so it is zero-filled and costs no traffic, and it gives the rows in shared memory
// the pitch that keeps the fragment loads free of bank conflicts.
static bool encode_maps_uncached(const Problem& p, const SkinnyPlan& plan, CUtensorMap* maps) {
  const uint64_t stages_in_row = static_cast<uint64_t>(p.K / plan.stage_k);
  const uint64_t n_rows = static_cast<uint64_t>(p.N);
  {
    const uint64_t dims[3] = {static_cast<uint64_t>(plan.stage_k / 16), stages_in_row, n_rows};
    const uint64_t strides[2] = {static_cast<uint64_t>(plan.stage_k / 2),
                                 static_cast<uint64_t>(p.K / 2)};
    const uint32_t box[3] = {static_cast<uint32_t>(plan.stage_k / 16 + plan.packed_pad / 8), 1, kRows};
    if (!encode_tensor_map(&maps[0], CU_TENSOR_MAP_DATA_TYPE_UINT64, 3, p.packed, dims, strides, box,
                           CU_TENSOR_MAP_SWIZZLE_NONE)) {
      return false;
    }
  }
  const uint64_t dims[3] = {static_cast<uint64_t>(plan.stage_k / 64), stages_in_row, n_rows};
  const uint64_t strides[2] = {static_cast<uint64_t>(plan.stage_k / 16),
                               static_cast<uint64_t>(p.K / 16)};
  const uint32_t box[3] = {static_cast<uint32_t>(plan.stage_k / 64 + 4), 1, kRows};
  return encode_tensor_map(&maps[1], CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, p.scales, dims, strides, box,
                           CU_TENSOR_MAP_SWIZZLE_NONE) &&
         encode_tensor_map(&maps[2], CU_TENSOR_MAP_DATA_TYPE_INT32, 3, p.zeros, dims, strides, box,
                           CU_TENSOR_MAP_SWIZZLE_NONE);
}

// A tensor map is a pure function of the addresses, the shape and the box, and inference calls
// the same few linears over and over: the last maps of each host thread are kept and reused,
// which saves three driver calls per launch.
bool skinny_encode_maps(const Problem& p, const SkinnyPlan& plan, CUtensorMap* maps) {
  struct Entry {
    const void* packed = nullptr;
    const void* scales = nullptr;
    const void* zeros = nullptr;
    int64_t N = 0, K = 0;
    int stage_k = 0, packed_pad = 0;
    CUtensorMap maps[3];
  };
  constexpr int kEntries = 64;
  thread_local Entry cache[kEntries];
  const uintptr_t mix = reinterpret_cast<uintptr_t>(p.packed) >> 8;
  Entry& e = cache[(mix ^ (mix >> 6) ^ (mix >> 12)) % kEntries];
  const bool hit = e.packed == p.packed && e.scales == p.scales && e.zeros == p.zeros &&
                   e.N == p.N && e.K == p.K && e.stage_k == plan.stage_k &&
                   e.packed_pad == plan.packed_pad;
  if (!hit) {
    if (!encode_maps_uncached(p, plan, e.maps)) {
      e.packed = nullptr;
      return false;
    }
    e.packed = p.packed, e.scales = p.scales, e.zeros = p.zeros;
    e.N = p.N, e.K = p.K, e.stage_k = plan.stage_k, e.packed_pad = plan.packed_pad;
  }
  for (int i = 0; i < 3; ++i) maps[i] = e.maps[i];
  return true;
}

cudaError_t launch_skinny(const Problem& p, const SkinnyPlan& plan, float* partials, int* tickets,
                          int* status_word, bool pdl, cudaStream_t stream) {
  if (plan.columns) return launch_gemv_decode(p, plan, partials, tickets, status_word, pdl, stream);
  const int m = static_cast<int>(p.M);
  const int nt = m <= 8 ? 1 : (m <= 16 ? 2 : 4);
  KernelParams kp;
  kp.x = p.x;
  kp.y = p.y;
  kp.partials = partials;
  kp.tickets = tickets;
  kp.status = status_word;
  kp.M = m;
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
  switch (nt) {
    case 1:
      return launch_nt<1>(maps, kp, plan, pdl, stream);
    case 2:
      return launch_nt<2>(maps, kp, plan, pdl, stream);
    default:
      return launch_nt<4>(maps, kp, plan, pdl, stream);
  }
}

}  // namespace lbl
