// gnb200_bwd_static_scratch: the backward pass for callers that cannot hand the library a scratch
// buffer because they are not allowed to allocate device memory at all.
//
// Who that is: code that runs where cudaMalloc / cudaFree (or a framework allocator that may fall
// through to them) is off limits - an inference runtime whose plugins get their input and output
// buffers from the host application and a fixed memory budget decided at start-up, a real-time
// loop that must not take the driver's allocation lock, a step that is being recorded into a
// stream capture, or a foreign-function binding that only ever sees the tensors it was given.
// gnb200_bwd needs up to a few MB of scratch from its caller; this variant brings its own: a
// fixed array in the library's device data segment.
//
// What that costs and what to watch for:
//   * GNB200_STATIC_SCRATCH_BYTES (4 MiB) of device memory are held on every GPU that loads the
//     library, from load until the process exits, whether or not this entry point is ever used.
//   * Problems whose backward plan needs more scratch than that are refused with
//     GNB200_ERR_WORKSPACE and a message that states both sizes; nothing is launched.
//   * The first call on a device looks up the device address of the array (cudaGetSymbolAddress,
//     once per device, with that device current).  Make that first call outside any stream
//     capture; later calls only enqueue kernels.
//   * All calls on a device share the one array.  Two calls whose kernels can overlap on the GPU
//     (different streams, no ordering between them) would overwrite each other's partial sums:
//     order them.  The array keeps whatever the last call left in it; no call depends on that,
//     because every scratch word a call reads is written earlier in the same call, so nothing
//     has to be cleared in between.
//   * No cudaMalloc, cudaFree or other allocating routine is called, here or below.
#include <mutex>

#include "../../include/gnb200.h"
#include "gn_kernels.h"

namespace gnb200 {
int report_error(int code, const char* fmt, ...);  // gn_capi.cu: fills gnb200_last_error()
}

namespace {

// The scratch itself.  In host code the name `g_static_scratch` is only a handle for the runtime
// (its host-side shadow), never a device address: a kernel must be given the pointer obtained
// from cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_static_scratch[GNB200_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
std::mutex g_addr_mutex;
void* g_scratch_addr[kMaxDevices] = {};

// Device address of the array on the current device (looked up once per device).
cudaError_t static_scratch_address(void** out) {
  int dev = -1;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return err;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(g_addr_mutex);
  if (g_scratch_addr[dev] == nullptr) {
    void* ptr = nullptr;
    err = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (err != cudaSuccess) return err;
    g_scratch_addr[dev] = ptr;
  }
  *out = g_scratch_addr[dev];
  return cudaSuccess;
}

bool is_aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

extern "C" int gnb200_bwd_static_scratch(const void* dy, const void* x, const void* gamma, const void* beta,
                                         const float* mean, const float* rstd, int64_t N, int64_t R, int64_t C,
                                         int64_t G, int act, int dtype, void* dx, float* dgamma_dbeta_f32,
                                         void* dgamma, void* dbeta, void* stream) {
  if (dtype != GNB200_F32 && dtype != GNB200_F16 && dtype != GNB200_BF16)
    return gnb200::report_error(GNB200_ERR_INVALID_ARGUMENT, "gnb200_bwd_static_scratch: unknown dtype code %d", dtype);
  if (act < GNB200_ACT_IDENTITY || act > GNB200_ACT_GELU_TANH)
    return gnb200::report_error(GNB200_ERR_INVALID_ARGUMENT, "gnb200_bwd_static_scratch: unknown activation code %d", act);
  if (N < 1 || R < 1 || C < 1 || G < 1 || C % G != 0)
    return gnb200::report_error(GNB200_ERR_INVALID_ARGUMENT,
                                "gnb200_bwd_static_scratch: need positive N, R, C, G with C divisible by G "
                                "(got N=%lld R=%lld C=%lld G=%lld)",
                                (long long)N, (long long)R, (long long)C, (long long)G);
  if (!dy || !x || !gamma || !beta || !mean || !rstd || !dx || !dgamma_dbeta_f32)
    return gnb200::report_error(GNB200_ERR_INVALID_ARGUMENT, "gnb200_bwd_static_scratch: null tensor pointer");
  if (gnb200::wait_gave_up_on_current_device())
    return gnb200::report_error(GNB200_ERR_EXCHANGE_TIMEOUT,
                                "gnb200_bwd_static_scratch: a kernel of an earlier call on this device gave up waiting "
                                "for its peers; see gnb200_wait_timeouts() / gnb200_clear_wait_timeouts()");
  gnb200::Plan plan;
  const bool al = is_aligned16(x) && is_aligned16(dy) && is_aligned16(dx) && is_aligned16(gamma) && is_aligned16(beta);
  if (!gnb200::make_plan(N, R, C, G, dtype, 1, al, &plan))
    return gnb200::report_error(GNB200_ERR_UNSUPPORTED,
                                "gnb200_bwd_static_scratch: shape N=%lld R=%lld C=%lld G=%lld is outside the supported "
                                "index range",
                                (long long)N, (long long)R, (long long)C, (long long)G);
  if (plan.ws_bytes > (size_t)GNB200_STATIC_SCRATCH_BYTES)
    return gnb200::report_error(GNB200_ERR_WORKSPACE,
                                "gnb200_bwd_static_scratch: this problem needs %zu bytes of scratch but the built-in "
                                "array holds %zu; use gnb200_bwd with a caller-provided workspace",
                                plan.ws_bytes, (size_t)GNB200_STATIC_SCRATCH_BYTES);
  void* scratch = nullptr;
  cudaError_t err = static_scratch_address(&scratch);
  if (err != cudaSuccess)
    return gnb200::report_error(GNB200_ERR_CUDA, "gnb200_bwd_static_scratch: cannot resolve the scratch array: %s",
                                cudaGetErrorString(err));
  gnb200::BwdCall call = {dy, x, gamma, beta, mean, rstd, dx, dgamma_dbeta_f32, dgamma, dbeta, scratch, act, dtype};
  err = gnb200::launch_backward(call, plan, reinterpret_cast<cudaStream_t>(stream));
  if (err != cudaSuccess)
    return gnb200::report_error(GNB200_ERR_CUDA, "gnb200_bwd_static_scratch: CUDA error: %s", cudaGetErrorString(err));
  return GNB200_OK;
}
