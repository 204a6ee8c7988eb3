// C ABI of the library (declared in include/lowbitlinear_b200.h): argument checks, the
// size-based dispatcher, scratch layout and the per-device status word.
#include "../../include/lowbitlinear_b200.h"

#include "kernels.h"

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

namespace {

constexpr int kVersion = 100;  // 0.1.0
constexpr int kMaxDevices = 64;

thread_local char g_error[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list args;
  va_start(args, fmt);
  std::vsnprintf(g_error, sizeof(g_error), fmt, args);
  va_end(args);
  return code;
}

int fail_cuda(cudaError_t err, const char* what) {
  return fail(LBL_ERR_CUDA, "%s: %s", what, cudaGetErrorString(err));
}

// One status word per device; kernels with bounded waits report through it.
__device__ int g_device_status = 0;

struct DeviceInfo {
  bool ready = false;
  int sm_count = 0;
  int* status_word = nullptr;
};
DeviceInfo g_devices[kMaxDevices];
std::mutex g_devices_mutex;

// Makes `device` current for the scope and restores the previous one.
class DeviceScope {
 public:
  explicit DeviceScope(int device) {
    ok_ = cudaGetDevice(&previous_) == cudaSuccess;
    if (ok_ && previous_ != device) {
      ok_ = cudaSetDevice(device) == cudaSuccess;
      switched_ = ok_;
    }
  }
  ~DeviceScope() {
    if (switched_) cudaSetDevice(previous_);
  }
  bool ok() const { return ok_; }

 private:
  int previous_ = 0;
  bool ok_ = false;
  bool switched_ = false;
};

// Requires `device` to be current.
int device_info(int device, DeviceInfo* out) {
  if (device < 0 || device >= kMaxDevices) return fail(LBL_ERR_INVALID, "device %d out of range", device);
  std::lock_guard<std::mutex> lock(g_devices_mutex);
  DeviceInfo& info = g_devices[device];
  if (!info.ready) {
    cudaError_t err = cudaDeviceGetAttribute(&info.sm_count, cudaDevAttrMultiProcessorCount, device);
    if (err != cudaSuccess) return fail_cuda(err, "cudaDeviceGetAttribute");
    int major = 0;
    err = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device);
    if (err != cudaSuccess) return fail_cuda(err, "cudaDeviceGetAttribute");
    if (major != 10) {
      return fail(LBL_ERR_UNSUPPORTED, "device %d has compute capability %d.x; this library is built for sm_100a only", device, major);
    }
    void* ptr = nullptr;
    err = cudaGetSymbolAddress(&ptr, g_device_status);
    if (err != cudaSuccess) return fail_cuda(err, "cudaGetSymbolAddress");
    info.status_word = static_cast<int*>(ptr);
    info.ready = true;
  }
  *out = info;
  return LBL_OK;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// The one runtime knob: LBL_FORCE_PATH=<path code> makes every dispatcher call without an explicit
// path take that kernel (crossover measurements).  Read once, when the library is first used.
int forced_path_from_env() {
  static const int forced = [] {
    const char* v = std::getenv("LBL_FORCE_PATH");
    return (v == nullptr || *v == '\0') ? LBL_PATH_AUTO : std::atoi(v);
  }();
  return forced;
}

// Crossover thresholds (measured on B200).  From kTcSmallMinM rows of activations on, shapes the
// small-M tensor-core GEMM can serve go to it instead of the streaming kernel; from kTcMinM on
// the large tensor-core GEMM takes what the small one cannot.
constexpr int kTcMinM = 17;
constexpr int kTcSmallMinM = 9;

int select_path(int64_t M, int64_t N, int64_t K, int op, int sm_count) {
  (void)op;
  if (M <= 0 || N <= 0 || K <= 0) return LBL_PATH_GENERIC;
  const bool skinny_ok = lbl::skinny_supports(M, N, K);
  const bool tc_ok = lbl::gemm_tc_supports(M, N, K);
  // Measured crossover (B200): the streaming kernels win up to M = 16; from M = 9 the
  // tensor-core GEMM already wins when N is large enough to fill the SMs with 256-wide tiles.
  // Measured (B200): with 9..128 rows of activations the small-M tensor-core GEMM wins wherever
  // the 256-wide tiles of the large one cannot fill the SMs (N < 16384), and up to M = 32 beyond.
  const bool wide = N >= 16384;
  // On a wide shape the streaming kernel still wins at 9..16 rows when the whole activation operand
  // fits its shared memory (Gate/Up, M = 16: 40 us against 55 and 62 for the tensor-core GEMMs).
  const bool stream_wide = wide && M <= 16 && skinny_ok && M * K * 2 <= lbl::kSkinnyOperandBytes;
  if (M >= kTcSmallMinM && lbl::gemm_tc_small_supports(M, N, K) && (!wide || M <= 32 || !tc_ok) && !stream_wide) {
    return LBL_PATH_GEMM_TC_SMALL;
  }
  // A long K whose activations do not fit the streaming kernel's operand budget is split along K
  // there (ordered fix-up); from six rows on the small tensor-core GEMM is faster (Down, M = 8:
  // 29 against 34 us).
  if (M >= 6 && M * K * 2 > lbl::kSkinnyOperandBytes && !wide && lbl::gemm_tc_small_supports(M, N, K)) {
    return LBL_PATH_GEMM_TC_SMALL;
  }
  // More than 128 rows of activations on a shape whose 256 x 256 tiles would leave most SMs idle
  // (less than half a wave: small N, a tensor-parallel shard): the tensor-memory GEMM cuts K into
  // slices until the SMs are busy.  Also the only tensor-core kernel for N % 256 == 128.
  if (M > 128 && lbl::gemm_wt_supports(M, N, K)) {
    const int64_t tc_ctas = (N / 256) * ((M + 255) / 256);
    // Measured (B200): it wins below a third of a wave, and up to half a wave when K is long
    // enough for eight slices.
    if (!tc_ok || 3 * tc_ctas <= sm_count || (2 * tc_ctas <= sm_count && K >= 8192)) return LBL_PATH_GEMM_WT;
  }
  // Pairs of CTAs that share one dequantised copy of the weights run a k-block in 0.83 of the time
  // of single CTAs (measured, M = 384 .. 8192 on the benchmark shapes), but their tile holds 512
  // tokens instead of 256: whichever needs fewer (weighted) waves of the SMs wins.
  if (tc_ok && M > 128 && lbl::gemm_tc_pair_supports(M, N, K)) {
    const int64_t pair_slots = sm_count >= 2 ? sm_count / 2 : 1;
    const int64_t pairs = (N / 256) * ((M + 511) / 512);
    const int64_t tc_ctas = (N / 256) * ((M + 255) / 256);
    const int64_t waves_pair = (pairs + pair_slots - 1) / pair_slots;
    const int64_t waves_tc = (tc_ctas + sm_count - 1) / sm_count;
    if (10 * waves_pair <= 12 * waves_tc) return LBL_PATH_GEMM_TC_PAIR;
  }
  if (tc_ok && (M >= kTcMinM || (wide && M >= 9 && !stream_wide) || !skinny_ok)) return LBL_PATH_GEMM_TC;
  if (skinny_ok) {
    lbl::SkinnyPlan plan;
    if (lbl::skinny_make_plan(M, N, K, -1, sm_count, &plan)) {
      return plan.nsplit > 1 ? LBL_PATH_GEMV_SPLITK : LBL_PATH_GEMV;
    }
  }
  return LBL_PATH_GENERIC;
}

int run_linear(const void* X, const int32_t* packed_w, const float* scales, const int32_t* zeros,
               void* Y, int64_t M, int64_t N, int64_t K, int op, int path, void* workspace,
               size_t workspace_bytes, unsigned flags, int device, void* stream, int* path_taken) {
  if (M < 0 || N < 0 || K < 0) return fail(LBL_ERR_INVALID, "negative dimension (M=%lld N=%lld K=%lld)", (long long)M, (long long)N, (long long)K);
  if (path_taken != nullptr) *path_taken = LBL_PATH_AUTO;
  if (M == 0 || N == 0) return LBL_OK;  // empty output
  // Every path that touches the scratch does so with 16-byte vector accesses and 4-byte atomics.
  if (workspace != nullptr && workspace_bytes > 0 && !aligned16(workspace)) {
    return fail(LBL_ERR_INVALID, "workspace must be 16-byte aligned");
  }
  if (Y == nullptr) return fail(LBL_ERR_INVALID, "Y is null");
  cudaStream_t cu_stream = static_cast<cudaStream_t>(stream);

  DeviceScope scope(device);
  if (!scope.ok()) return fail(LBL_ERR_CUDA, "cannot make device %d current", device);
  DeviceInfo info;
  const int rc = device_info(device, &info);
  if (rc != LBL_OK) return rc;

  if (K == 0) {
    const cudaError_t err = cudaMemsetAsync(Y, 0, static_cast<size_t>(M) * N * sizeof(__half), cu_stream);
    if (err != cudaSuccess) return fail_cuda(err, "cudaMemsetAsync");
    return LBL_OK;
  }
  if (X == nullptr || packed_w == nullptr || scales == nullptr || zeros == nullptr) {
    return fail(LBL_ERR_INVALID, "null tensor pointer");
  }

  lbl::Problem prob;
  prob.x = static_cast<const __half*>(X);
  prob.packed = reinterpret_cast<const uint32_t*>(packed_w);
  prob.scales = scales;
  prob.zeros = zeros;
  prob.y = static_cast<__half*>(Y);
  prob.M = M;
  prob.N = N;
  prob.K = K;

  const bool forced = path != LBL_PATH_AUTO;
  if (!forced) {
    path = forced_path_from_env();
    if (path == LBL_PATH_AUTO) path = select_path(M, N, K, op, info.sm_count);
  }
  // The reference GEMM's operand policy on request: the streaming kernels keep the FP32 scale, so
  // the any-shape operator is sent to a kernel that rounds each dequantised weight to FP16.
  if (!forced && op == 1 && (flags & LBL_FLAG_ROUND_WEIGHTS) != 0 &&
      (path == LBL_PATH_GEMV || path == LBL_PATH_GEMV_SPLITK)) {
    if (lbl::gemm_tc_small_supports(M, N, K)) {
      path = LBL_PATH_GEMM_TC_SMALL;
    } else if (lbl::gemm_wt_supports(M, N, K)) {
      path = LBL_PATH_GEMM_WT;
    } else if (lbl::gemm_tc_supports(M, N, K)) {
      path = LBL_PATH_GEMM_TC;
    } else {
      path = LBL_PATH_GENERIC;
    }
  }
  // Calls declared independent of their neighbours overlap in time: the CTAs of the next call fill
  // the SMs this one leaves idle, so a tile count far below a wave is no loss, and the paired
  // kernel (no scratch, never waits) beats cutting K into slices (scratch, waits for its neighbours).
  if (!forced && path == LBL_PATH_GEMM_WT && (flags & LBL_FLAG_PDL) != 0 && (flags & LBL_FLAG_INDEPENDENT) != 0 &&
      M >= 384 && lbl::gemm_tc_pair_supports(M, N, K)) {
    path = LBL_PATH_GEMM_TC_PAIR;
  }
  // The fast kernels use 16-byte vector accesses and bulk copies on every operand.
  const bool all_aligned = aligned16(X) && aligned16(packed_w) && aligned16(scales) &&
                           aligned16(zeros) && aligned16(Y);
  if (!all_aligned && path != LBL_PATH_GENERIC) {
    if (forced) return fail(LBL_ERR_UNSUPPORTED, "forced path %d needs 16-byte aligned tensors", path);
    path = LBL_PATH_GENERIC;
  }

  cudaError_t err = cudaSuccess;
  switch (path) {
    case LBL_PATH_GENERIC: {
      const bool round_weights = (flags & LBL_FLAG_ROUND_WEIGHTS) != 0 || op == 1;
      err = lbl::launch_generic(prob, round_weights, cu_stream);
      break;
    }
    case LBL_PATH_GEMV:
    case LBL_PATH_GEMV_SPLITK: {
      lbl::SkinnyPlan plan;
      const int want = forced ? (path == LBL_PATH_GEMV ? 0 : 2) : -1;
      if (!lbl::skinny_make_plan(M, N, K, want, info.sm_count, &plan)) {
        return fail(LBL_ERR_UNSUPPORTED, "streaming kernel cannot serve M=%lld N=%lld K=%lld (needs M <= 32, K %% 256 == 0)", (long long)M, (long long)N, (long long)K);
      }
      float* partials = nullptr;
      int* tickets = nullptr;
      if (plan.nsplit > 1) {
        const size_t need = plan.partial_bytes + plan.ticket_bytes;
        if (workspace == nullptr || workspace_bytes < need) {
          return fail(LBL_ERR_WORKSPACE, "split-K needs %zu bytes of scratch, got %zu", need, workspace_bytes);
        }
        tickets = static_cast<int*>(workspace);
        partials = reinterpret_cast<float*>(static_cast<char*>(workspace) + plan.ticket_bytes);
      }
      path = plan.nsplit > 1 ? LBL_PATH_GEMV_SPLITK : LBL_PATH_GEMV;
      err = lbl::launch_skinny(prob, plan, partials, tickets, info.status_word,
                               (flags & LBL_FLAG_PDL) != 0, cu_stream);
      break;
    }
    case LBL_PATH_GEMM_TC: {
      if (!lbl::gemm_tc_supports(M, N, K)) {
        return fail(LBL_ERR_UNSUPPORTED, "tensor-core GEMM cannot serve M=%lld N=%lld K=%lld (needs N %% 256 == 0, K %% 256 == 0)", (long long)M, (long long)N, (long long)K);
      }
      err = lbl::launch_gemm_tc(prob, info.status_word, cu_stream, (flags & LBL_FLAG_PDL) != 0,
                                (flags & LBL_FLAG_INDEPENDENT) != 0);
      break;
    }
    case LBL_PATH_GEMM_TC_SMALL: {
      if (!lbl::gemm_tc_small_supports(M, N, K)) {
        return fail(LBL_ERR_UNSUPPORTED, "small-M tensor-core GEMM cannot serve M=%lld N=%lld K=%lld (needs M <= 128, N %% 128 == 0, K %% 256 == 0)", (long long)M, (long long)N, (long long)K);
      }
      err = lbl::launch_gemm_tc_small(prob, info.status_word, cu_stream, workspace, workspace_bytes,
                                      info.sm_count, (flags & LBL_FLAG_PDL) != 0);
      break;
    }
    case LBL_PATH_GEMM_TC_PAIR: {
      if (!lbl::gemm_tc_pair_supports(M, N, K)) {
        return fail(LBL_ERR_UNSUPPORTED, "paired tensor-core GEMM cannot serve M=%lld N=%lld K=%lld (needs N %% 256 == 0, K %% 256 == 0)", (long long)M, (long long)N, (long long)K);
      }
      err = lbl::launch_gemm_tc_pair(prob, info.status_word, cu_stream, (flags & LBL_FLAG_PDL) != 0,
                                     (flags & LBL_FLAG_INDEPENDENT) != 0);
      break;
    }
    case LBL_PATH_GEMM_WT: {
      if (!lbl::gemm_wt_supports(M, N, K)) {
        return fail(LBL_ERR_UNSUPPORTED, "tensor-memory GEMM cannot serve M=%lld N=%lld K=%lld (needs N %% 128 == 0, K %% 256 == 0)", (long long)M, (long long)N, (long long)K);
      }
      err = lbl::launch_gemm_wt(prob, info.status_word, cu_stream, workspace, workspace_bytes, info.sm_count,
                                (flags & LBL_FLAG_PDL) != 0);
      break;
    }
    default:
      return fail(LBL_ERR_INVALID, "unknown path %d", path);
  }
  if (err != cudaSuccess) return fail_cuda(err, "kernel launch");
  if (path_taken != nullptr) *path_taken = path;
  return LBL_OK;
}

int sm_count_or_default(int device_hint) {
  int device = device_hint;
  if (device < 0 && cudaGetDevice(&device) != cudaSuccess) return 148;
  int sms = 0;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0) {
    cudaGetLastError();
    return 148;  // B200
  }
  return sms;
}

}  // namespace

extern "C" {

int lbl_version(void) { return kVersion; }

const char* lbl_last_error(void) { return g_error; }

int lbl_w4a16_select_path(int64_t M, int64_t N, int64_t K, int op) {
  const int forced = forced_path_from_env();
  if (forced != LBL_PATH_AUTO) return forced;
  return select_path(M, N, K, op, sm_count_or_default(-1));
}

size_t lbl_w4a16_workspace_bytes(int64_t M, int64_t N, int64_t K, int path) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  const int sms = sm_count_or_default(-1);
  if (path == LBL_PATH_AUTO) {
    path = forced_path_from_env();
    if (path == LBL_PATH_AUTO) path = select_path(M, N, K, 0, sms);
  }
  if (path == LBL_PATH_GEMM_TC_SMALL) return lbl::gemm_tc_small_workspace_bytes(M, N, K, sms);
  if (path == LBL_PATH_GEMM_WT) return lbl::gemm_wt_workspace_bytes(M, N, K, sms);
  if (path != LBL_PATH_GEMV && path != LBL_PATH_GEMV_SPLITK) return 0;
  lbl::SkinnyPlan plan;
  const int want = path == LBL_PATH_GEMV_SPLITK ? 2 : -1;
  if (!lbl::skinny_make_plan(M, N, K, want, sms, &plan)) return 0;
  // The AUTO plan may split less than a forced split-K plan; report the larger need.
  size_t need = plan.partial_bytes + plan.ticket_bytes;
  lbl::SkinnyPlan auto_plan;
  if (lbl::skinny_make_plan(M, N, K, -1, sms, &auto_plan)) {
    const size_t other = auto_plan.partial_bytes + auto_plan.ticket_bytes;
    if (other > need) need = other;
  }
  return need;
}

int lbl_w4a16_workspace_init(void* workspace, size_t workspace_bytes, int device, void* stream) {
  if (workspace_bytes == 0) return LBL_OK;
  if (workspace == nullptr) return fail(LBL_ERR_INVALID, "workspace is null");
  DeviceScope scope(device);
  if (!scope.ok()) return fail(LBL_ERR_CUDA, "cannot make device %d current", device);
  const cudaError_t err = cudaMemsetAsync(workspace, 0, workspace_bytes, static_cast<cudaStream_t>(stream));
  if (err != cudaSuccess) return fail_cuda(err, "cudaMemsetAsync");
  return LBL_OK;
}

int lbl_w4a16_gemv(const void* x, const int32_t* packed_w, const float* scales,
                   const int32_t* zeros, void* y, int64_t N, int64_t K, int group_size,
                   void* workspace, size_t workspace_bytes, unsigned flags, int device,
                   void* stream) {
  if (group_size != 64 || K <= 0 || K % 64 != 0) {
    return fail(LBL_ERR_INVALID, "Expected group_size=64 and K divisible by 64 (group_size=%d K=%lld)", group_size, (long long)K);
  }
  if (N <= 0 || N > 0x7fffffffLL || K > 0x7fffffffLL) return fail(LBL_ERR_INVALID, "Invalid N or K");
  if ((reinterpret_cast<uintptr_t>(x) & 15u) != 0) return fail(LBL_ERR_INVALID, "x must be 16-byte aligned");
  return run_linear(x, packed_w, scales, zeros, y, 1, N, K, 0, LBL_PATH_AUTO, workspace,
                    workspace_bytes, flags, device, stream, nullptr);
}

int lbl_w4a16_gemm(const void* X, const int32_t* packed_w, const float* scales,
                   const int32_t* zeros, void* Y, int64_t M, int64_t N, int64_t K,
                   void* workspace, size_t workspace_bytes, unsigned flags, int device,
                   void* stream) {
  return run_linear(X, packed_w, scales, zeros, Y, M, N, K, 1, LBL_PATH_AUTO, workspace,
                    workspace_bytes, flags, device, stream, nullptr);
}

int lbl_w4a16_linear(const void* X, const int32_t* packed_w, const float* scales,
                     const int32_t* zeros, void* Y, int64_t M, int64_t N, int64_t K, int op,
                     int path, void* workspace, size_t workspace_bytes, unsigned flags,
                     int device, void* stream, int* path_taken) {
  if (op != 0 && op != 1) return fail(LBL_ERR_INVALID, "op must be 0 or 1");
  return run_linear(X, packed_w, scales, zeros, Y, M, N, K, op, path, workspace, workspace_bytes,
                    flags, device, stream, path_taken);
}

int lbl_w4a16_quantize(const void* weight, int weight_is_fp32, int64_t N, int64_t K,
                       int group_size, int32_t* packed_w, float* scales, int32_t* zeros,
                       int device, void* stream) {
  if (group_size != 64) {
    return fail(LBL_ERR_UNSUPPORTED, "the device quantiser supports group_size=64 only (got %d)", group_size);
  }
  if (N < 0 || K <= 0) return fail(LBL_ERR_INVALID, "Invalid N or K (N=%lld K=%lld)", (long long)N, (long long)K);
  if (N == 0) return LBL_OK;
  if (weight == nullptr || packed_w == nullptr || scales == nullptr || zeros == nullptr) {
    return fail(LBL_ERR_INVALID, "null tensor pointer");
  }
  DeviceScope scope(device);
  if (!scope.ok()) return fail(LBL_ERR_CUDA, "cannot make device %d current", device);
  const cudaError_t err =
      lbl::launch_quantize(weight, weight_is_fp32 != 0, N, K, reinterpret_cast<uint32_t*>(packed_w),
                           scales, zeros, static_cast<cudaStream_t>(stream));
  if (err != cudaSuccess) return fail_cuda(err, "quantise launch");
  return LBL_OK;
}

int lbl_w4a16_dequantize(const int32_t* packed_w, const float* scales, const int32_t* zeros,
                         void* weight, int weight_is_fp32, int64_t N, int64_t K, int group_size,
                         int device, void* stream) {
  if (group_size != 64) {
    return fail(LBL_ERR_UNSUPPORTED, "the device dequantiser supports group_size=64 only (got %d)", group_size);
  }
  if (N < 0 || K <= 0) return fail(LBL_ERR_INVALID, "Invalid N or K (N=%lld K=%lld)", (long long)N, (long long)K);
  if (N == 0) return LBL_OK;
  if (weight == nullptr || packed_w == nullptr || scales == nullptr || zeros == nullptr) {
    return fail(LBL_ERR_INVALID, "null tensor pointer");
  }
  DeviceScope scope(device);
  if (!scope.ok()) return fail(LBL_ERR_CUDA, "cannot make device %d current", device);
  const cudaError_t err = lbl::launch_dequantize(reinterpret_cast<const uint32_t*>(packed_w), scales,
                                                 zeros, weight, weight_is_fp32 != 0, N, K,
                                                 static_cast<cudaStream_t>(stream));
  if (err != cudaSuccess) return fail_cuda(err, "dequantise launch");
  return LBL_OK;
}

int lbl_device_status(int device, int* status) {
  if (status == nullptr) return fail(LBL_ERR_INVALID, "status is null");
  DeviceScope scope(device);
  if (!scope.ok()) return fail(LBL_ERR_CUDA, "cannot make device %d current", device);
  DeviceInfo info;
  const int rc = device_info(device, &info);
  if (rc != LBL_OK) return rc;
  cudaError_t err = cudaDeviceSynchronize();
  if (err != cudaSuccess) return fail_cuda(err, "cudaDeviceSynchronize");
  err = cudaMemcpy(status, info.status_word, sizeof(int), cudaMemcpyDeviceToHost);
  if (err != cudaSuccess) return fail_cuda(err, "cudaMemcpy");
  if (*status != 0) {
    const int zero = 0;
    err = cudaMemcpy(info.status_word, &zero, sizeof(int), cudaMemcpyHostToDevice);
    if (err != cudaSuccess) return fail_cuda(err, "cudaMemcpy");
  }
  return LBL_OK;
}

// ---------------------------------------------------------------------------------------------
// GEMV for callers that cannot allocate device memory.
//
// Split-K needs scratch (arrival counters and FP32 partial sums).  Here it lives in a fixed
// array that is part of the library image, so the caller provides inputs and outputs only.
// Every GPU that loads the library carries these bytes until the process exits.
// ---------------------------------------------------------------------------------------------
}  // extern "C"

namespace {

constexpr size_t kStaticScratchBytes = 1u << 20;  // 64 KiB of counters + 960 KiB of partial sums
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// In host code `g_static_scratch` is only a handle for the runtime; the device address has to be
// asked for, once per device and with that device current.
void* g_static_scratch_address[kMaxDevices] = {};
std::mutex g_static_scratch_mutex;

// Requires `device` to be current.  The first call per device also clears the counters.
int static_scratch(int device, cudaStream_t stream, void** out) {
  std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
  if (g_static_scratch_address[device] == nullptr) {
    void* ptr = nullptr;
    cudaError_t err = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (err != cudaSuccess) return fail_cuda(err, "cudaGetSymbolAddress(static scratch)");
    err = cudaMemsetAsync(ptr, 0, lbl::kSkinnyTicketBytes, stream);
    if (err != cudaSuccess) return fail_cuda(err, "cudaMemsetAsync(static scratch)");
    g_static_scratch_address[device] = ptr;
  }
  *out = g_static_scratch_address[device];
  return LBL_OK;
}

}  // namespace

extern "C" {

size_t lbl_w4a16_gemv_noalloc_scratch_bytes(void) { return kStaticScratchBytes; }

int lbl_w4a16_gemv_noalloc(const void* x, const int32_t* packed_w, const float* scales,
                           const int32_t* zeros, void* y, int64_t N, int64_t K, int group_size,
                           unsigned flags, int device, void* stream) {
  if (group_size != 64 || K <= 0 || K % 64 != 0) {
    return fail(LBL_ERR_INVALID, "Expected group_size=64 and K divisible by 64 (group_size=%d K=%lld)", group_size, (long long)K);
  }
  if (N <= 0 || N > 0x7fffffffLL || K > 0x7fffffffLL) return fail(LBL_ERR_INVALID, "Invalid N or K");
  if (x == nullptr || packed_w == nullptr || scales == nullptr || zeros == nullptr || y == nullptr) {
    return fail(LBL_ERR_INVALID, "null tensor pointer");
  }
  if (!aligned16(x) || !aligned16(packed_w) || !aligned16(scales) || !aligned16(zeros) || !aligned16(y)) {
    return fail(LBL_ERR_INVALID, "all tensors must be 16-byte aligned");
  }
  cudaStream_t cu_stream = static_cast<cudaStream_t>(stream);
  DeviceScope scope(device);
  if (!scope.ok()) return fail(LBL_ERR_CUDA, "cannot make device %d current", device);
  DeviceInfo info;
  int rc = device_info(device, &info);
  if (rc != LBL_OK) return rc;

  lbl::SkinnyPlan plan;
  if (!lbl::skinny_make_plan(1, N, K, /*want_split=*/2, info.sm_count, &plan)) {
    return fail(LBL_ERR_UNSUPPORTED, "the streaming kernel needs K %% 256 == 0 (K=%lld)", (long long)K);
  }
  const size_t need = plan.partial_bytes + plan.ticket_bytes;
  if (need > kStaticScratchBytes) {
    return fail(LBL_ERR_WORKSPACE, "N=%lld K=%lld needs %zu bytes of split-K scratch; the built-in scratch holds %zu. Use lbl_w4a16_gemv with a caller-provided workspace", (long long)N, (long long)K, need, kStaticScratchBytes);
  }
  void* scratch = nullptr;
  rc = static_scratch(device, cu_stream, &scratch);
  if (rc != LBL_OK) return rc;

  lbl::Problem prob;
  prob.x = static_cast<const __half*>(x);
  prob.packed = reinterpret_cast<const uint32_t*>(packed_w);
  prob.scales = scales;
  prob.zeros = zeros;
  prob.y = static_cast<__half*>(y);
  prob.M = 1;
  prob.N = N;
  prob.K = K;
  int* tickets = plan.nsplit > 1 ? static_cast<int*>(scratch) : nullptr;
  float* partials = plan.nsplit > 1
                        ? reinterpret_cast<float*>(static_cast<char*>(scratch) + plan.ticket_bytes)
                        : nullptr;
  const cudaError_t err = lbl::launch_skinny(prob, plan, partials, tickets, info.status_word,
                                             (flags & LBL_FLAG_PDL) != 0, cu_stream);
  if (err != cudaSuccess) return fail_cuda(err, "kernel launch");
  return LBL_OK;
}

// ---------------------------------------------------------------------------------------------
// Row-parallel (K-split) GEMV with the all-reduce fused into the kernel.
//
// Each rank owns an exchange buffer that its peers map through CUDA IPC.  A rank's kernel leaves
// its FP32 result vector in its own buffer, the last CTA raises a flag in every peer's buffer,
// waits (bounded) for the peers' flags in its own, and adds the vectors of all ranks in rank
// order, reading the peers' memory with plain loads over NVLink.  No NCCL call, no multicast.
// ---------------------------------------------------------------------------------------------
size_t lbl_peer_buffer_bytes(int64_t max_n) {
  if (max_n <= 0) return 0;
  return lbl::kPeerBufferHeaderBytes + 2 * static_cast<size_t>(max_n) * sizeof(float);
}

int lbl_peer_buffer_create(size_t bytes, int device, void** buffer) {
  if (buffer == nullptr || bytes < lbl::kPeerBufferHeaderBytes) return fail(LBL_ERR_INVALID, "bad peer buffer request");
  DeviceScope scope(device);
  if (!scope.ok()) return fail(LBL_ERR_CUDA, "cannot make device %d current", device);
  void* ptr = nullptr;
  cudaError_t err = cudaMalloc(&ptr, bytes);
  if (err != cudaSuccess) return fail_cuda(err, "cudaMalloc(peer buffer)");
  err = cudaMemset(ptr, 0, bytes);
  if (err != cudaSuccess) {
    cudaFree(ptr);
    return fail_cuda(err, "cudaMemset(peer buffer)");
  }
  *buffer = ptr;
  return LBL_OK;
}

int lbl_peer_buffer_peek(const void* buffer, size_t offset, void* host_dst, size_t bytes, int device) {
  if (buffer == nullptr || host_dst == nullptr || offset + bytes > lbl::kPeerBufferHeaderBytes) {
    return fail(LBL_ERR_INVALID, "peek reads the %zu-byte control block only", lbl::kPeerBufferHeaderBytes);
  }
  DeviceScope scope(device);
  if (!scope.ok()) return fail(LBL_ERR_CUDA, "cannot make device %d current", device);
  const cudaError_t err = cudaMemcpy(host_dst, static_cast<const unsigned char*>(buffer) + offset, bytes, cudaMemcpyDeviceToHost);
  if (err != cudaSuccess) return fail_cuda(err, "cudaMemcpy(control block)");
  return LBL_OK;
}

int lbl_peer_buffer_export(const void* buffer, void* handle64) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  if (buffer == nullptr || handle64 == nullptr) return fail(LBL_ERR_INVALID, "null argument");
  cudaIpcMemHandle_t handle;
  const cudaError_t err = cudaIpcGetMemHandle(&handle, const_cast<void*>(buffer));
  if (err != cudaSuccess) return fail_cuda(err, "cudaIpcGetMemHandle");
  std::memcpy(handle64, &handle, sizeof(handle));
  return LBL_OK;
}

int lbl_peer_buffer_open(const void* handle64, int device, void** buffer) {
  if (buffer == nullptr || handle64 == nullptr) return fail(LBL_ERR_INVALID, "null argument");
  DeviceScope scope(device);
  if (!scope.ok()) return fail(LBL_ERR_CUDA, "cannot make device %d current", device);
  cudaIpcMemHandle_t handle;
  std::memcpy(&handle, handle64, sizeof(handle));
  void* ptr = nullptr;
  const cudaError_t err = cudaIpcOpenMemHandle(&ptr, handle, cudaIpcMemLazyEnablePeerAccess);
  if (err != cudaSuccess) return fail_cuda(err, "cudaIpcOpenMemHandle");
  *buffer = ptr;
  return LBL_OK;
}

int lbl_peer_buffer_close(void* buffer, int device) {
  if (buffer == nullptr) return LBL_OK;
  DeviceScope scope(device);
  if (!scope.ok()) return fail(LBL_ERR_CUDA, "cannot make device %d current", device);
  const cudaError_t err = cudaIpcCloseMemHandle(buffer);
  if (err != cudaSuccess) return fail_cuda(err, "cudaIpcCloseMemHandle");
  return LBL_OK;
}

int lbl_peer_buffer_destroy(void* buffer, int device) {
  if (buffer == nullptr) return LBL_OK;
  DeviceScope scope(device);
  if (!scope.ok()) return fail(LBL_ERR_CUDA, "cannot make device %d current", device);
  const cudaError_t err = cudaFree(buffer);
  if (err != cudaSuccess) return fail_cuda(err, "cudaFree(peer buffer)");
  return LBL_OK;
}

int lbl_w4a16_gemv_allreduce(const void* x, const int32_t* packed_w, const float* scales,
                             const int32_t* zeros, void* y, int64_t N, int64_t K, int group_size,
                             int rank, int world, void* const* buffers, int64_t buffer_capacity_n,
                             void* workspace, size_t workspace_bytes, unsigned flags, int device,
                             void* stream) {
  if (group_size != 64 || K <= 0 || K % 256 != 0) {
    return fail(LBL_ERR_UNSUPPORTED, "the fused all-reduce GEMV needs group_size=64 and K %% 256 == 0 (K=%lld)", (long long)K);
  }
  if (N <= 0 || N > 0x7fffffffLL || N > buffer_capacity_n) return fail(LBL_ERR_INVALID, "N=%lld does not fit the exchange buffers (capacity %lld)", (long long)N, (long long)buffer_capacity_n);
  if (buffer_capacity_n % 4 != 0) return fail(LBL_ERR_INVALID, "buffer_capacity_n must be a multiple of 4");
  if (world < 1 || world > 8 || rank < 0 || rank >= world || buffers == nullptr) return fail(LBL_ERR_INVALID, "bad rank/world/buffers");
  if (x == nullptr || packed_w == nullptr || scales == nullptr || zeros == nullptr || y == nullptr) return fail(LBL_ERR_INVALID, "null tensor pointer");
  if (!aligned16(x) || !aligned16(packed_w) || !aligned16(scales) || !aligned16(zeros) || !aligned16(y)) return fail(LBL_ERR_INVALID, "all tensors must be 16-byte aligned");
  for (int r = 0; r < world; ++r) {
    if (buffers[r] == nullptr) return fail(LBL_ERR_INVALID, "exchange buffer of rank %d is null", r);
  }
  if (workspace != nullptr && workspace_bytes > 0 && !aligned16(workspace)) {
    return fail(LBL_ERR_INVALID, "workspace must be 16-byte aligned");
  }
  cudaStream_t cu_stream = static_cast<cudaStream_t>(stream);
  DeviceScope scope(device);
  if (!scope.ok()) return fail(LBL_ERR_CUDA, "cannot make device %d current", device);
  DeviceInfo info;
  const int rc = device_info(device, &info);
  if (rc != LBL_OK) return rc;

  lbl::SkinnyPlan plan;
  if (!lbl::skinny_make_plan(1, N, K, -1, info.sm_count, &plan) || !plan.columns) {
    return fail(LBL_ERR_UNSUPPORTED, "no decode plan for N=%lld K=%lld", (long long)N, (long long)K);
  }
  float* partials = nullptr;
  int* tickets = nullptr;
  if (plan.nsplit > 1) {
    const size_t need = plan.partial_bytes + plan.ticket_bytes;
    if (workspace == nullptr || workspace_bytes < need) return fail(LBL_ERR_WORKSPACE, "split-K needs %zu bytes of scratch, got %zu", need, workspace_bytes);
    tickets = static_cast<int*>(workspace);
    partials = reinterpret_cast<float*>(static_cast<char*>(workspace) + plan.ticket_bytes);
  }
  lbl::Problem prob;
  prob.x = static_cast<const __half*>(x);
  prob.packed = reinterpret_cast<const uint32_t*>(packed_w);
  prob.scales = scales;
  prob.zeros = zeros;
  prob.y = static_cast<__half*>(y);
  prob.M = 1;
  prob.N = N;
  prob.K = K;
  lbl::PeerReduce reduce;
  reduce.rank = rank;
  reduce.world = world;
  reduce.capacity_n = static_cast<int>(buffer_capacity_n);
  for (int r = 0; r < 8; ++r) reduce.buffers[r] = r < world ? buffers[r] : nullptr;
  const cudaError_t err = lbl::launch_gemv_decode(prob, plan, partials, tickets, info.status_word,
                                                  (flags & LBL_FLAG_PDL) != 0, cu_stream, &reduce);
  if (err != cudaSuccess) return fail_cuda(err, "kernel launch");
  return LBL_OK;
}

// ---------------------------------------------------------------------------------------------
// K-split GEMM with a two-shot all-reduce over peer memory (large M).
// ---------------------------------------------------------------------------------------------
size_t lbl_peer_gemm_buffer_bytes(int64_t M, int64_t N, int world) {
  if (M <= 0 || N <= 0 || world < 1 || world > 8 || N % world != 0) return 0;
  return lbl::peer_gemm_buffer_bytes(M, N, world);
}

static int check_gemm_exchange(int64_t M, int64_t N, int rank, int world, void* const* buffers, size_t buffer_bytes) {
  if (world < 2 || world > 8 || rank < 0 || rank >= world || buffers == nullptr) return fail(LBL_ERR_INVALID, "bad rank/world/buffers");
  if (M <= 0 || N <= 0 || M > 0x7fffffffLL || N > 0x7fffffffLL) return fail(LBL_ERR_INVALID, "bad shape M=%lld N=%lld", (long long)M, (long long)N);
  if (N % (256 * world) != 0) {
    return fail(LBL_ERR_UNSUPPORTED, "the GEMM all-reduce needs N %% (256 * world) == 0 (N=%lld, world=%d)", (long long)N, world);
  }
  const size_t need = lbl::peer_gemm_buffer_bytes(M, N, world);
  if (buffer_bytes < need) return fail(LBL_ERR_WORKSPACE, "exchange buffers hold %zu bytes, M=%lld N=%lld needs %zu", buffer_bytes, (long long)M, (long long)N, need);
  for (int r = 0; r < world; ++r) {
    if (buffers[r] == nullptr || !aligned16(buffers[r])) return fail(LBL_ERR_INVALID, "exchange buffer of rank %d is null or misaligned", r);
  }
  return LBL_OK;
}

int lbl_w4a16_gemm_scatter(const void* x, const int32_t* packed_w, const float* scales, const int32_t* zeros,
                           int64_t M, int64_t N, int64_t K, int rank, int world, void* const* buffers,
                           size_t buffer_bytes, unsigned flags, int device, void* stream) {
  int rc = check_gemm_exchange(M, N, rank, world, buffers, buffer_bytes);
  if (rc != LBL_OK) return rc;
  if (!lbl::gemm_tc_pair_supports(M, N, K)) {
    return fail(LBL_ERR_UNSUPPORTED, "the scattering GEMM needs N %% 256 == 0 and K %% 256 == 0 (N=%lld K=%lld)", (long long)N, (long long)K);
  }
  if (x == nullptr || packed_w == nullptr || scales == nullptr || zeros == nullptr) return fail(LBL_ERR_INVALID, "null tensor pointer");
  if (!aligned16(x) || !aligned16(packed_w) || !aligned16(scales) || !aligned16(zeros)) return fail(LBL_ERR_INVALID, "all tensors must be 16-byte aligned");
  DeviceScope scope(device);
  if (!scope.ok()) return fail(LBL_ERR_CUDA, "cannot make device %d current", device);
  DeviceInfo info;
  rc = device_info(device, &info);
  if (rc != LBL_OK) return rc;
  lbl::Problem prob;
  prob.x = static_cast<const __half*>(x);
  prob.packed = reinterpret_cast<const uint32_t*>(packed_w);
  prob.scales = scales;
  prob.zeros = zeros;
  prob.y = nullptr;
  prob.M = M;
  prob.N = N;
  prob.K = K;
  lbl::PairScatter scatter;
  scatter.world = world;
  const size_t slice_bytes = static_cast<size_t>(M) * (N / world) * sizeof(__half);
  for (int r = 0; r < 8; ++r) {
    scatter.slot[r] = r < world ? reinterpret_cast<__half*>(static_cast<unsigned char*>(buffers[r]) + lbl::kPeerBufferHeaderBytes + rank * slice_bytes) : nullptr;
  }
  const bool pdl = (flags & LBL_FLAG_PDL) != 0;
  const cudaError_t err = lbl::launch_gemm_tc_pair(prob, info.status_word, static_cast<cudaStream_t>(stream), pdl,
                                                   pdl && (flags & LBL_FLAG_INDEPENDENT) != 0, &scatter);
  if (err != cudaSuccess) return fail_cuda(err, "kernel launch");
  return LBL_OK;
}

int lbl_peer_gemm_allreduce_finish(void* y, int64_t M, int64_t N, int rank, int world, void* const* buffers,
                                   size_t buffer_bytes, int device, void* stream) {
  const int rc0 = check_gemm_exchange(M, N, rank, world, buffers, buffer_bytes);
  if (rc0 != LBL_OK) return rc0;
  if (y == nullptr || !aligned16(y)) return fail(LBL_ERR_INVALID, "y is null or not 16-byte aligned");
  DeviceScope scope(device);
  if (!scope.ok()) return fail(LBL_ERR_CUDA, "cannot make device %d current", device);
  DeviceInfo info;
  const int rc = device_info(device, &info);
  if (rc != LBL_OK) return rc;
  lbl::PeerReduce exchange;
  exchange.rank = rank;
  exchange.world = world;
  exchange.capacity_n = 0;
  for (int r = 0; r < 8; ++r) exchange.buffers[r] = r < world ? buffers[r] : nullptr;
  const cudaError_t err = lbl::launch_peer_slice_allreduce(exchange, static_cast<__half*>(y), M, N, info.sm_count,
                                                           info.status_word, static_cast<cudaStream_t>(stream));
  if (err != cudaSuccess) return fail_cuda(err, "kernel launch");
  return LBL_OK;
}

int lbl_w4a16_gemm_allreduce(const void* x, const int32_t* packed_w, const float* scales, const int32_t* zeros,
                             void* y, int64_t M, int64_t N, int64_t K, int rank, int world, void* const* buffers,
                             size_t buffer_bytes, unsigned flags, int device, void* stream) {
  const int rc = lbl_w4a16_gemm_scatter(x, packed_w, scales, zeros, M, N, K, rank, world, buffers, buffer_bytes, flags,
                                        device, stream);
  if (rc != LBL_OK) return rc;
  return lbl_peer_gemm_allreduce_finish(y, M, N, rank, world, buffers, buffer_bytes, device, stream);
}

// ---------------------------------------------------------------------------------------------
// Grouped decode GEMV: a list of independent problems in one persistent launch.
// ---------------------------------------------------------------------------------------------
struct lbl_w4a16_group {
  lbl::GroupPlan* plan;
};

int lbl_w4a16_group_create(const lbl_w4a16_problem* problems, int count, int rank, int world,
                           void* const* buffers, int64_t buffer_capacity_n, int device,
                           lbl_w4a16_group** group) {
  if (group == nullptr) return fail(LBL_ERR_INVALID, "group is null");
  *group = nullptr;
  if (problems == nullptr || count <= 0) return fail(LBL_ERR_INVALID, "a group needs at least one problem");
  if (world < 1 || world > 8 || rank < 0 || rank >= world) return fail(LBL_ERR_INVALID, "bad rank/world");
  lbl::PeerReduce exchange;
  exchange.rank = rank;
  exchange.world = world;
  exchange.capacity_n = 0;
  for (int r = 0; r < 8; ++r) exchange.buffers[r] = nullptr;
  bool any_reduce = false;
  std::vector<lbl::GroupProblemDesc> descs(static_cast<size_t>(count));
  for (int i = 0; i < count; ++i) {
    const lbl_w4a16_problem& q = problems[i];
    if (q.x == nullptr || q.packed_w == nullptr || q.scales == nullptr || q.zeros == nullptr || q.y == nullptr) {
      return fail(LBL_ERR_INVALID, "problem %d: null tensor pointer", i);
    }
    if (!aligned16(q.x) || !aligned16(q.packed_w) || !aligned16(q.scales) || !aligned16(q.zeros) || !aligned16(q.y)) {
      return fail(LBL_ERR_INVALID, "problem %d: all tensors must be 16-byte aligned", i);
    }
    if (q.M < 1 || q.M > 2 || q.N < 1 || q.K < 256 || q.K % 256 != 0 || q.N > 0x7fffffffLL - 16 || q.M * q.K > 32768) {
      return fail(LBL_ERR_UNSUPPORTED, "problem %d: the grouped GEMV serves 1 <= M <= 2, K %% 256 == 0, M * K <= 32768 (M=%lld N=%lld K=%lld)", i, (long long)q.M, (long long)q.N, (long long)q.K);
    }
    lbl::GroupProblemDesc& d = descs[static_cast<size_t>(i)];
    d.x = q.x, d.packed = q.packed_w, d.scales = q.scales, d.zeros = q.zeros, d.y = q.y;
    d.M = q.M, d.N = q.N, d.K = q.K;
    d.reduce = q.reduce != 0 && world > 1;
    any_reduce = any_reduce || d.reduce;
  }
  if (any_reduce) {
    if (buffers == nullptr || buffer_capacity_n <= 0 || buffer_capacity_n % 4 != 0 || buffer_capacity_n > 0x7fffffffLL) {
      return fail(LBL_ERR_INVALID, "problems with reduce=1 need the exchange buffers of all ranks");
    }
    for (int r = 0; r < world; ++r) {
      if (buffers[r] == nullptr) return fail(LBL_ERR_INVALID, "exchange buffer of rank %d is null", r);
      exchange.buffers[r] = buffers[r];
    }
    exchange.capacity_n = static_cast<int>(buffer_capacity_n);
  }
  DeviceScope scope(device);
  if (!scope.ok()) return fail(LBL_ERR_CUDA, "cannot make device %d current", device);
  DeviceInfo info;
  const int rc = device_info(device, &info);
  if (rc != LBL_OK) return rc;
  lbl::GroupPlan* plan = nullptr;
  const char* why = "";
  const cudaError_t err = lbl::group_plan_create(descs.data(), count, info.sm_count, info.status_word,
                                                 any_reduce ? &exchange : nullptr, &plan, &why);
  if (err != cudaSuccess) {
    if (why != nullptr && *why != '\0') return fail(LBL_ERR_UNSUPPORTED, "%s", why);
    return fail_cuda(err, "group plan");
  }
  *group = new lbl_w4a16_group{plan};
  return LBL_OK;
}

int lbl_w4a16_group_run(lbl_w4a16_group* group, unsigned flags, void* stream) {
  if (group == nullptr || group->plan == nullptr) return fail(LBL_ERR_INVALID, "group is null");
  DeviceScope scope(lbl::group_plan_device(group->plan));
  if (!scope.ok()) return fail(LBL_ERR_CUDA, "cannot make the group's device current");
  const cudaError_t err = lbl::launch_gemv_grouped(group->plan, (flags & LBL_FLAG_PDL) != 0,
                                                   static_cast<cudaStream_t>(stream));
  if (err != cudaSuccess) return fail_cuda(err, "kernel launch");
  return LBL_OK;
}

int64_t lbl_w4a16_group_algorithmic_bytes(const lbl_w4a16_group* group) {
  if (group == nullptr || group->plan == nullptr) return 0;
  return lbl::group_plan_bytes(group->plan);
}

int lbl_w4a16_group_destroy(lbl_w4a16_group* group) {
  if (group == nullptr) return LBL_OK;
  if (group->plan != nullptr) {
    DeviceScope scope(lbl::group_plan_device(group->plan));
    lbl::group_plan_destroy(group->plan);
  }
  delete group;
  return LBL_OK;
}

}  // extern "C"
