// extern "C" entry points of libgnb200.so (declared in include/gnb200.h).
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <mutex>

#include "../../include/gnb200.h"
#include "gn_kernels.h"

namespace {

thread_local char g_last_error[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
  return code;
}

}  // namespace

namespace gnb200 {
__device__ unsigned int g_wait_timeouts = 0;

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_wait_mu;
unsigned int* g_counter_addr[kMaxDevices] = {};
// One word per device in mapped pinned host memory: a kernel whose bounded wait gave up sets its
// device's word, and the entry points read it on the host without synchronising.
volatile unsigned int* g_host_mirror = nullptr;
unsigned int* g_mirror_dev_addr[kMaxDevices] = {};
}  // namespace

cudaError_t wait_limit_for_device(WaitLimit* out) {
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return err;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(g_wait_mu);
  if (!g_host_mirror) {
    void* h = nullptr;
    err = cudaHostAlloc(&h, kMaxDevices * sizeof(unsigned int), cudaHostAllocMapped | cudaHostAllocPortable);
    if (err != cudaSuccess) return err;
    memset(h, 0, kMaxDevices * sizeof(unsigned int));
    g_host_mirror = static_cast<volatile unsigned int*>(h);
  }
  if (!g_counter_addr[dev]) {
    void* p = nullptr;
    err = cudaGetSymbolAddress(&p, g_wait_timeouts);
    if (err != cudaSuccess) return err;
    void* m = nullptr;
    err = cudaHostGetDevicePointer(&m, const_cast<unsigned int*>(g_host_mirror) + dev, 0);
    if (err != cudaSuccess) return err;
    g_counter_addr[dev] = static_cast<unsigned int*>(p);
    g_mirror_dev_addr[dev] = static_cast<unsigned int*>(m);
  }
  out->timeouts = g_counter_addr[dev];
  out->host_mirror = g_mirror_dev_addr[dev];
  out->clocks = 2000000000LL;  // about a second
  out->polls = 1u << 16;
  // GNB200_WAIT_CLOCKS: a shorter limit for bring-up of new kernels
  if (const char* v = getenv("GNB200_WAIT_CLOCKS")) {
    const long long c = atoll(v);
    if (c > 0) {
      out->clocks = c;
      out->polls = 256;
    }
  }
  return cudaSuccess;
}

// Non-zero once a kernel on the current device has recorded a wait that gave up (no synchronisation:
// the kernel stores to mapped host memory).
bool wait_gave_up_on_current_device() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return false;
  const volatile unsigned int* m = g_host_mirror;
  return m != nullptr && m[dev] != 0;
}

void clear_wait_mirror_on_current_device() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return;
  if (g_host_mirror) g_host_mirror[dev] = 0;
}

// Same thread-local text as fail(), for entry points that live in other translation units.
int report_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
  return code;
}
}  // namespace gnb200

namespace {

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int check_common(int64_t N, int64_t R, int64_t C, int64_t G, int act, int dtype) {
  if (dtype != GNB200_F32 && dtype != GNB200_F16 && dtype != GNB200_BF16)
    return fail(GNB200_ERR_INVALID_ARGUMENT, "gnb200: unknown dtype code %d (0=f32, 1=f16, 2=bf16)", dtype);
  if (act < GNB200_ACT_IDENTITY || act > GNB200_ACT_GELU_TANH)
    return fail(GNB200_ERR_INVALID_ARGUMENT, "gnb200: unknown activation code %d (valid: 0..4)", act);
  if (N < 1 || R < 1 || C < 1 || G < 1)
    return fail(GNB200_ERR_INVALID_ARGUMENT, "gnb200: N, R, C, G must be positive (got N=%lld R=%lld C=%lld G=%lld)",
                (long long)N, (long long)R, (long long)C, (long long)G);
  if (C % G != 0)
    return fail(GNB200_ERR_INVALID_ARGUMENT, "gnb200: num_channels %lld is not divisible by num_groups %lld",
                (long long)C, (long long)G);
  if (gnb200::wait_gave_up_on_current_device())
    return fail(GNB200_ERR_EXCHANGE_TIMEOUT,
                "gnb200: a kernel of an earlier call on this device gave up waiting for its peers; every result "
                "since the last check is invalid (NaN where the wait was needed). gnb200_wait_timeouts() gives the "
                "count, gnb200_clear_wait_timeouts() re-arms the library");
  return GNB200_OK;
}

}  // namespace

extern "C" {

int gnb200_version(void) { return 100; }

const char* gnb200_last_error(void) { return g_last_error; }

int gnb200_act_code(const char* name) {
  if (!name) return -1;
  if (!strcmp(name, "identity")) return GNB200_ACT_IDENTITY;
  if (!strcmp(name, "relu")) return GNB200_ACT_RELU;
  if (!strcmp(name, "silu") || !strcmp(name, "swish")) return GNB200_ACT_SILU;
  if (!strcmp(name, "gelu")) return GNB200_ACT_GELU;
  if (!strcmp(name, "gelu_tanh")) return GNB200_ACT_GELU_TANH;
  return -1;
}

size_t gnb200_fwd_workspace_bytes(int64_t N, int64_t R, int64_t C, int64_t G, int dtype) {
  return gnb200::plan_workspace_bytes(N, R, C, G, dtype, 0);
}

size_t gnb200_bwd_workspace_bytes(int64_t N, int64_t R, int64_t C, int64_t G, int dtype) {
  return gnb200::plan_workspace_bytes(N, R, C, G, dtype, 1);
}

int gnb200_fwd(const void* x, const void* gamma, const void* beta, int64_t N, int64_t R, int64_t C, int64_t G,
               double eps, int act, int dtype, void* y, float* mean, float* rstd, void* workspace,
               size_t workspace_bytes, void* stream) {
  int rc = check_common(N, R, C, G, act, dtype);
  if (rc != GNB200_OK) return rc;
  if (!x || !gamma || !beta || !y || !mean || !rstd)
    return fail(GNB200_ERR_INVALID_ARGUMENT, "gnb200_fwd: null tensor pointer");
  gnb200::Plan plan;
  // the vector kernels read x, y, gamma and beta with 16-byte accesses: all four must be aligned
  const bool al = aligned16(x) && aligned16(y) && aligned16(gamma) && aligned16(beta);
  if (!gnb200::make_plan(N, R, C, G, dtype, 0, al, &plan))
    return fail(GNB200_ERR_UNSUPPORTED, "gnb200_fwd: shape N=%lld R=%lld C=%lld G=%lld is outside the supported index range",
                (long long)N, (long long)R, (long long)C, (long long)G);
  if (plan.ws_bytes > 0 && (!workspace || workspace_bytes < plan.ws_bytes || !aligned16(workspace)))
    return fail(GNB200_ERR_WORKSPACE, "gnb200_fwd: needs a 16-byte aligned workspace of %zu bytes, got %zu at %p",
                plan.ws_bytes, workspace_bytes, workspace);
  gnb200::FwdCall call = {x, gamma, beta, y, mean, rstd, workspace, (float)eps, act, dtype};
  const cudaError_t err = gnb200::launch_forward(call, plan, reinterpret_cast<cudaStream_t>(stream));
  if (err != cudaSuccess) {
    (void)cudaGetLastError();  // a failed runtime call must not be reported again by a later, healthy call
    return fail(GNB200_ERR_CUDA, "gnb200_fwd: CUDA error: %s", cudaGetErrorString(err));
  }
  return GNB200_OK;
}

// Fills *px from the caller's table of exchange buffers; `who` names the entry point in messages.
static int make_peer_exchange(const void* const* peer_bufs, int rank, int world, int64_t C, bool collect, const char* who,
                              gnb200::PeerExchange* px) {
  if (world < 1 || world > gnb200::kMaxPeers || rank < 0 || rank >= world)
    return fail(GNB200_ERR_INVALID_ARGUMENT, "%s: rank %d of %d ranks (1 .. %d ranks supported)", who, rank, world,
                gnb200::kMaxPeers);
  if (C < 1 || C > (1 << 24)) return fail(GNB200_ERR_INVALID_ARGUMENT, "%s: C = %lld", who, (long long)C);
  *px = gnb200::PeerExchange{};
  px->world = world;
  px->rank = rank;
  px->C = (int)C;
  px->nblk = (int)((C + gnb200::kPeerBlock - 1) / gnb200::kPeerBlock);
  px->collect = collect ? 1 : 0;
  if (world == 1) return GNB200_OK;
  if (!peer_bufs) return fail(GNB200_ERR_INVALID_ARGUMENT, "%s: null table of exchange buffers", who);
  for (int q = 0; q < world; ++q) {
    if (!peer_bufs[q] || !aligned16(peer_bufs[q]))
      return fail(GNB200_ERR_INVALID_ARGUMENT, "%s: exchange buffer of rank %d is null or not 16-byte aligned (%p)", who, q,
                  peer_bufs[q]);
    px->base[q] = static_cast<char*>(const_cast<void*>(peer_bufs[q]));
  }
  const cudaError_t err = gnb200::wait_limit_for_device(&px->wait);
  if (err != cudaSuccess) {
    (void)cudaGetLastError();
    return fail(GNB200_ERR_CUDA, "%s: CUDA error: %s", who, cudaGetErrorString(err));
  }
  return GNB200_OK;
}

static int bwd_impl(const char* who, const void* dy, const void* x, const void* gamma, const void* beta, const float* mean,
                    const float* rstd, int64_t N, int64_t R, int64_t C, int64_t G, int act, int dtype, void* dx,
                    float* dgamma_dbeta_f32, void* dgamma, void* dbeta, void* workspace, size_t workspace_bytes,
                    const gnb200::PeerExchange* px, void* stream) {
  int rc = check_common(N, R, C, G, act, dtype);
  if (rc != GNB200_OK) return rc;
  if (!dy || !x || !gamma || !beta || !mean || !rstd || !dx || !dgamma_dbeta_f32)
    return fail(GNB200_ERR_INVALID_ARGUMENT, "%s: null tensor pointer", who);
  gnb200::Plan plan;
  const bool al = aligned16(x) && aligned16(dy) && aligned16(dx) && aligned16(gamma) && aligned16(beta);
  if (!gnb200::make_plan(N, R, C, G, dtype, 1, al, &plan))
    return fail(GNB200_ERR_UNSUPPORTED, "%s: shape N=%lld R=%lld C=%lld G=%lld is outside the supported index range", who,
                (long long)N, (long long)R, (long long)C, (long long)G);
  if (plan.ws_bytes > 0 && (!workspace || workspace_bytes < plan.ws_bytes || !aligned16(workspace)))
    return fail(GNB200_ERR_WORKSPACE, "%s: needs a 16-byte aligned workspace of %zu bytes, got %zu at %p", who,
                plan.ws_bytes, workspace_bytes, workspace);
  gnb200::BwdCall call = {dy, x, gamma, beta, mean, rstd, dx, dgamma_dbeta_f32, dgamma, dbeta, workspace, act, dtype};
  call.peer = px;
  const cudaError_t err = gnb200::launch_backward(call, plan, reinterpret_cast<cudaStream_t>(stream));
  if (err != cudaSuccess) {
    (void)cudaGetLastError();
    return fail(GNB200_ERR_CUDA, "%s: CUDA error: %s", who, cudaGetErrorString(err));
  }
  return GNB200_OK;
}

int gnb200_bwd(const void* dy, const void* x, const void* gamma, const void* beta, const float* mean,
               const float* rstd, int64_t N, int64_t R, int64_t C, int64_t G, int act, int dtype, void* dx,
               float* dgamma_dbeta_f32, void* dgamma, void* dbeta, void* workspace, size_t workspace_bytes,
               void* stream) {
  return bwd_impl("gnb200_bwd", dy, x, gamma, beta, mean, rstd, N, R, C, G, act, dtype, dx, dgamma_dbeta_f32, dgamma, dbeta,
                  workspace, workspace_bytes, nullptr, stream);
}

size_t gnb200_peer_exchange_bytes(int64_t C, int world) {
  if (C < 1 || C > (1 << 24) || world < 1 || world > gnb200::kMaxPeers) return 0;
  return gnb200::peer_exchange_bytes(world, (int)C);
}

int gnb200_bwd_peer(const void* dy, const void* x, const void* gamma, const void* beta, const float* mean,
                    const float* rstd, int64_t N, int64_t R, int64_t C, int64_t G, int act, int dtype, void* dx,
                    float* dgamma_dbeta_f32, void* dgamma, void* dbeta, void* workspace, size_t workspace_bytes,
                    const void* const* peer_bufs, int rank, int world, void* stream) {
  gnb200::PeerExchange px;
  const int rc = make_peer_exchange(peer_bufs, rank, world, C, true, "gnb200_bwd_peer", &px);
  if (rc != GNB200_OK) return rc;
  return bwd_impl("gnb200_bwd_peer", dy, x, gamma, beta, mean, rstd, N, R, C, G, act, dtype, dx, dgamma_dbeta_f32, dgamma,
                  dbeta, workspace, workspace_bytes, &px, stream);
}

int gnb200_bwd_peer_push(const void* dy, const void* x, const void* gamma, const void* beta, const float* mean,
                         const float* rstd, int64_t N, int64_t R, int64_t C, int64_t G, int act, int dtype, void* dx,
                         float* dgamma_dbeta_f32, void* workspace, size_t workspace_bytes, const void* const* peer_bufs,
                         int rank, int world, void* stream) {
  gnb200::PeerExchange px;
  const int rc = make_peer_exchange(peer_bufs, rank, world, C, false, "gnb200_bwd_peer_push", &px);
  if (rc != GNB200_OK) return rc;
  return bwd_impl("gnb200_bwd_peer_push", dy, x, gamma, beta, mean, rstd, N, R, C, G, act, dtype, dx, dgamma_dbeta_f32,
                  nullptr, nullptr, workspace, workspace_bytes, &px, stream);
}

// push and / or collect on a gradient buffer, as a kernel of its own
static int exchange_impl(const char* who, float* dgamma_dbeta_f32, void* dgamma, void* dbeta, int64_t C, int dtype,
                         const void* const* peer_bufs, int rank, int world, bool push, bool collect, void* stream) {
  if (dtype < GNB200_F32 || dtype > GNB200_BF16) return fail(GNB200_ERR_INVALID_ARGUMENT, "%s: unknown dtype code %d", who, dtype);
  if (!dgamma_dbeta_f32) return fail(GNB200_ERR_INVALID_ARGUMENT, "%s: null gradient buffer", who);
  if (gnb200::wait_gave_up_on_current_device())
    return fail(GNB200_ERR_EXCHANGE_TIMEOUT, "%s: an earlier bounded wait on this device gave up", who);
  gnb200::PeerExchange px;
  const int rc = make_peer_exchange(peer_bufs, rank, world, C, collect, who, &px);
  if (rc != GNB200_OK) return rc;
  gnb200::BwdCall call = {};
  call.dparam_f32 = dgamma_dbeta_f32;
  call.dgamma = dgamma;
  call.dbeta = dbeta;
  call.dtype = dtype;
  call.peer = &px;
  const cudaError_t err = gnb200::launch_param_exchange(call, (int)C, reinterpret_cast<cudaStream_t>(stream), false, push, collect);
  if (err != cudaSuccess) {
    (void)cudaGetLastError();
    return fail(GNB200_ERR_CUDA, "%s: CUDA error: %s", who, cudaGetErrorString(err));
  }
  return GNB200_OK;
}

int gnb200_peer_collect(float* dgamma_dbeta_f32, void* dgamma, void* dbeta, int64_t C, int dtype,
                        const void* const* peer_bufs, int rank, int world, void* stream) {
  return exchange_impl("gnb200_peer_collect", dgamma_dbeta_f32, dgamma, dbeta, C, dtype, peer_bufs, rank, world, false, true,
                       stream);
}

int gnb200_allreduce_param_grads(float* dgamma_dbeta_f32, void* dgamma, void* dbeta, int64_t C, int dtype,
                                 const void* const* peer_bufs, int rank, int world, void* stream) {
  return exchange_impl("gnb200_allreduce_param_grads", dgamma_dbeta_f32, dgamma, dbeta, C, dtype, peer_bufs, rank, world,
                       true, true, stream);
}

size_t gnb200_fwd_nchw_workspace_bytes(int64_t N, int64_t R, int64_t C, int64_t G, int dtype) {
  return gnb200::nchw_workspace_bytes(N, R, C, G, dtype, 0);
}

size_t gnb200_bwd_nchw_workspace_bytes(int64_t N, int64_t R, int64_t C, int64_t G, int dtype) {
  return gnb200::nchw_workspace_bytes(N, R, C, G, dtype, 1);
}

int gnb200_fwd_nchw(const void* x, const void* gamma, const void* beta, int64_t N, int64_t R, int64_t C, int64_t G,
                    double eps, int act, int dtype, void* y, float* mean, float* rstd, void* workspace,
                    size_t workspace_bytes, void* stream) {
  int rc = check_common(N, R, C, G, act, dtype);
  if (rc != GNB200_OK) return rc;
  if (!x || !gamma || !beta || !y || !mean || !rstd)
    return fail(GNB200_ERR_INVALID_ARGUMENT, "gnb200_fwd_nchw: null tensor pointer");
  if (!gnb200::nchw_shape_supported(N, R, C, G))
    return fail(GNB200_ERR_UNSUPPORTED, "gnb200_fwd_nchw: shape N=%lld R=%lld C=%lld G=%lld is outside the supported index range",
                (long long)N, (long long)R, (long long)C, (long long)G);
  const size_t need = gnb200::nchw_workspace_bytes(N, R, C, G, dtype, 0);
  if (!workspace || workspace_bytes < need || !aligned16(workspace))
    return fail(GNB200_ERR_WORKSPACE, "gnb200_fwd_nchw: needs a 16-byte aligned workspace of %zu bytes, got %zu at %p", need,
                workspace_bytes, workspace);
  gnb200::FwdCall call = {x, gamma, beta, y, mean, rstd, workspace, (float)eps, act, dtype};
  const cudaError_t err = gnb200::launch_forward_nchw(call, N, R, C, G, reinterpret_cast<cudaStream_t>(stream));
  if (err != cudaSuccess) {
    (void)cudaGetLastError();
    return fail(GNB200_ERR_CUDA, "gnb200_fwd_nchw: CUDA error: %s", cudaGetErrorString(err));
  }
  return GNB200_OK;
}

int gnb200_bwd_nchw(const void* dy, const void* x, const void* gamma, const void* beta, const float* mean,
                    const float* rstd, int64_t N, int64_t R, int64_t C, int64_t G, int act, int dtype, void* dx,
                    float* dgamma_dbeta_f32, void* dgamma, void* dbeta, void* workspace, size_t workspace_bytes,
                    void* stream) {
  int rc = check_common(N, R, C, G, act, dtype);
  if (rc != GNB200_OK) return rc;
  if (!dy || !x || !gamma || !beta || !mean || !rstd || !dx || !dgamma_dbeta_f32)
    return fail(GNB200_ERR_INVALID_ARGUMENT, "gnb200_bwd_nchw: null tensor pointer");
  if (!gnb200::nchw_shape_supported(N, R, C, G))
    return fail(GNB200_ERR_UNSUPPORTED, "gnb200_bwd_nchw: shape N=%lld R=%lld C=%lld G=%lld is outside the supported index range",
                (long long)N, (long long)R, (long long)C, (long long)G);
  const size_t need = gnb200::nchw_workspace_bytes(N, R, C, G, dtype, 1);
  if (!workspace || workspace_bytes < need || !aligned16(workspace))
    return fail(GNB200_ERR_WORKSPACE, "gnb200_bwd_nchw: needs a 16-byte aligned workspace of %zu bytes, got %zu at %p", need,
                workspace_bytes, workspace);
  gnb200::BwdCall call = {dy, x, gamma, beta, mean, rstd, dx, dgamma_dbeta_f32, dgamma, dbeta, workspace, act, dtype};
  const cudaError_t err = gnb200::launch_backward_nchw(call, N, R, C, G, reinterpret_cast<cudaStream_t>(stream));
  if (err != cudaSuccess) {
    (void)cudaGetLastError();
    return fail(GNB200_ERR_CUDA, "gnb200_bwd_nchw: CUDA error: %s", cudaGetErrorString(err));
  }
  return GNB200_OK;
}

static int check_f64(int64_t N, int64_t R, int64_t C, int64_t G, int act, int layout, const char* who) {
  if (act < GNB200_ACT_IDENTITY || act > GNB200_ACT_GELU_TANH)
    return fail(GNB200_ERR_INVALID_ARGUMENT, "%s: unknown activation code %d (valid: 0..4)", who, act);
  if (layout != GNB200_LAYOUT_NHWC && layout != GNB200_LAYOUT_NCHW)
    return fail(GNB200_ERR_INVALID_ARGUMENT, "%s: unknown layout code %d (0 = NHWC, 1 = NCHW)", who, layout);
  if (N < 1 || R < 1 || C < 1 || G < 1 || C % G != 0)
    return fail(GNB200_ERR_INVALID_ARGUMENT, "%s: need positive N, R, C, G with C divisible by G (got N=%lld R=%lld C=%lld G=%lld)",
                who, (long long)N, (long long)R, (long long)C, (long long)G);
  if (N * G > 0x7fffffffLL || (double)N * (double)R * (double)C > 9.0e15)
    return fail(GNB200_ERR_UNSUPPORTED, "%s: shape is outside the supported index range", who);
  return GNB200_OK;
}

size_t gnb200_bwd_f64_workspace_bytes(int64_t N, int64_t R, int64_t C, int64_t G) {
  (void)R;
  (void)G;
  return N > 0 && C > 0 ? (size_t)N * (size_t)C * 2 * sizeof(double) : 0;
}

int gnb200_fwd_f64(const double* x, const double* gamma, const double* beta, int64_t N, int64_t R, int64_t C,
                   int64_t G, double eps, int act, int layout, double* y, double* mean, double* rstd, void* stream) {
  int rc = check_f64(N, R, C, G, act, layout, "gnb200_fwd_f64");
  if (rc != GNB200_OK) return rc;
  if (!x || !gamma || !beta || !y || !mean || !rstd)
    return fail(GNB200_ERR_INVALID_ARGUMENT, "gnb200_fwd_f64: null tensor pointer");
  const cudaError_t err = gnb200::launch_forward_f64(x, gamma, beta, N, R, C, G, eps, act, layout == GNB200_LAYOUT_NHWC, y,
                                                     mean, rstd, reinterpret_cast<cudaStream_t>(stream));
  if (err != cudaSuccess) {
    (void)cudaGetLastError();
    return fail(GNB200_ERR_CUDA, "gnb200_fwd_f64: CUDA error: %s", cudaGetErrorString(err));
  }
  return GNB200_OK;
}

int gnb200_bwd_f64(const double* dy, const double* x, const double* gamma, const double* beta, const double* mean,
                   const double* rstd, int64_t N, int64_t R, int64_t C, int64_t G, int act, int layout, double* dx,
                   double* dgamma, double* dbeta, void* workspace, size_t workspace_bytes, void* stream) {
  int rc = check_f64(N, R, C, G, act, layout, "gnb200_bwd_f64");
  if (rc != GNB200_OK) return rc;
  if (!dy || !x || !gamma || !beta || !mean || !rstd || !dx || !dgamma || !dbeta)
    return fail(GNB200_ERR_INVALID_ARGUMENT, "gnb200_bwd_f64: null tensor pointer");
  const size_t need = gnb200_bwd_f64_workspace_bytes(N, R, C, G);
  if (!workspace || workspace_bytes < need || !aligned16(workspace))
    return fail(GNB200_ERR_WORKSPACE, "gnb200_bwd_f64: needs a 16-byte aligned workspace of %zu bytes, got %zu at %p", need,
                workspace_bytes, workspace);
  const cudaError_t err =
      gnb200::launch_backward_f64(dy, x, gamma, beta, mean, rstd, N, R, C, G, act, layout == GNB200_LAYOUT_NHWC, dx, dgamma,
                                  dbeta, static_cast<double*>(workspace), reinterpret_cast<cudaStream_t>(stream));
  if (err != cudaSuccess) {
    (void)cudaGetLastError();
    return fail(GNB200_ERR_CUDA, "gnb200_bwd_f64: CUDA error: %s", cudaGetErrorString(err));
  }
  return GNB200_OK;
}

int gnb200_describe_plan(int64_t N, int64_t R, int64_t C, int64_t G, int dtype, int direction, char* buf,
                         int buf_len) {
  gnb200::Plan p;
  char text[512];
  if (C < 1 || G < 1 || !gnb200::make_plan(N, R, C, G, dtype, direction, true, &p)) {
    snprintf(text, sizeof(text), "unsupported");
  } else {
    const gnb200::Geom& g = p.geom;
    if (p.wave) {
      const gnb200::WaveGeom& w = p.wgeom;
      snprintf(text, sizeof(text),
               "%s wave ve=%d cw=%d ncb=%d ty=%d threads=%d rows=%d chunks=%d k=1 persist=1 grid=%lld smem=%zu ws=%zu "
               "launches=%d waves=%d ipw=%d box=%dx%d stages=%d teams=%d",
               direction == 0 ? "fwd" : "bwd", p.ve, w.CW, w.ncb, w.TY, p.threads, w.rows_per_chunk, w.chunks, p.grid,
               p.smem_bytes, p.ws_bytes, p.launches, w.waves, w.ipw, w.CW, w.BR, w.stages, w.teams);
    } else
    snprintf(text, sizeof(text),
             "%s %s ve=%d cw=%d ncb=%d ty=%d threads=%d rows=%d chunks=%d k=%d persist=%d grid=%lld smem=%zu ws=%zu launches=%d",
             direction == 0 ? "fwd" : "bwd", p.fused ? "fused" : "twopass", p.ve, g.CW, g.ncb, g.TY, p.threads,
             g.rows_per_cta, g.chunks, g.k, g.persist, p.grid, p.smem_bytes, p.ws_bytes, p.launches);
  }
  const int need = (int)strlen(text) + 1;
  if (buf && buf_len > 0) {
    strncpy(buf, text, (size_t)buf_len - 1);
    buf[buf_len - 1] = '\0';
  }
  return need;
}

void gnb200_debug_set_trace(void* device_buffer, size_t bytes) { gnb200::debug_set_trace(device_buffer, bytes); }

int gnb200_clear_wait_timeouts(void) {
  const unsigned int zero = 0;
  const cudaError_t err = cudaMemcpyToSymbol(gnb200::g_wait_timeouts, &zero, sizeof(zero));
  if (err != cudaSuccess) return fail(GNB200_ERR_CUDA, "gnb200_clear_wait_timeouts: CUDA error: %s", cudaGetErrorString(err));
  gnb200::clear_wait_mirror_on_current_device();
  return GNB200_OK;
}

int gnb200_selftest_exchange_timeout(const void* x, const void* gamma, const void* beta, int64_t N, int64_t R,
                                     int64_t C, int64_t G, double eps, int act, int dtype, void* y, float* mean,
                                     float* rstd, void* stream) {
  int rc = check_common(N, R, C, G, act, dtype);
  if (rc != GNB200_OK) return rc;
  if (!x || !gamma || !beta || !y || !mean || !rstd)
    return fail(GNB200_ERR_INVALID_ARGUMENT, "gnb200_selftest_exchange_timeout: null tensor pointer");
  gnb200::Plan plan;
  const bool al = aligned16(x) && aligned16(y) && aligned16(gamma) && aligned16(beta);
  if (!gnb200::make_plan(N, R, C, G, dtype, 0, al, &plan) || !plan.fused || plan.geom.k < 2)
    return fail(GNB200_ERR_UNSUPPORTED,
                "gnb200_selftest_exchange_timeout: the problem must take the fused forward plan with a cluster of at "
                "least two CTAs");
  gnb200::FwdCall call = {x, gamma, beta, y, mean, rstd, nullptr, (float)eps, act, dtype};
  call.test_skip_push_rank = 1;
  call.test_wait_clocks = 2000000;  // about a millisecond
  const cudaError_t err = gnb200::launch_forward(call, plan, reinterpret_cast<cudaStream_t>(stream));
  if (err == cudaErrorInvalidConfiguration)
    return fail(GNB200_ERR_UNSUPPORTED,
                "gnb200_selftest_exchange_timeout: the problem has more (sample, column block) slabs than clusters are "
                "resident; use a smaller batch");
  if (err != cudaSuccess) return fail(GNB200_ERR_CUDA, "gnb200_selftest_exchange_timeout: CUDA error: %s", cudaGetErrorString(err));
  return GNB200_OK;
}

long long gnb200_wait_timeouts(void) {
  unsigned int v = 0;
  const cudaError_t err = cudaMemcpyFromSymbol(&v, gnb200::g_wait_timeouts, sizeof(v));
  if (err != cudaSuccess) return fail(GNB200_ERR_CUDA, "gnb200_wait_timeouts: CUDA error: %s", cudaGetErrorString(err));
  return (long long)v;
}

int gnb200_launch_count(int64_t N, int64_t R, int64_t C, int64_t G, int dtype, int direction) {
  gnb200::Plan p;
  if (C < 1 || G < 1 || !gnb200::make_plan(N, R, C, G, dtype, direction, true, &p)) return -1;
  return p.launches;
}

}  // extern "C"
