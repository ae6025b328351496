// extern "C" entry points of libgnb200.so (declared in include/gnb200.h).
#include <stdarg.h>
#include <stdio.h>
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

cudaError_t wait_timeout_counter(unsigned int** counter) {
  constexpr int kMaxDevices = 64;
  static std::mutex mu;
  static unsigned int* addr[kMaxDevices] = {};
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return err;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(mu);
  if (!addr[dev]) {
    void* p = nullptr;
    err = cudaGetSymbolAddress(&p, g_wait_timeouts);
    if (err != cudaSuccess) return err;
    addr[dev] = static_cast<unsigned int*>(p);
  }
  *counter = addr[dev];
  return cudaSuccess;
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
  const bool al = aligned16(x) && aligned16(y);
  if (!gnb200::make_plan(N, R, C, G, dtype, 0, al, &plan))
    return fail(GNB200_ERR_UNSUPPORTED, "gnb200_fwd: shape N=%lld R=%lld C=%lld G=%lld is outside the supported index range",
                (long long)N, (long long)R, (long long)C, (long long)G);
  if (plan.ws_bytes > 0 && (!workspace || workspace_bytes < plan.ws_bytes || !aligned16(workspace)))
    return fail(GNB200_ERR_WORKSPACE, "gnb200_fwd: needs a 16-byte aligned workspace of %zu bytes, got %zu at %p",
                plan.ws_bytes, workspace_bytes, workspace);
  gnb200::FwdCall call = {x, gamma, beta, y, mean, rstd, workspace, (float)eps, act, dtype};
  const cudaError_t err = gnb200::launch_forward(call, plan, reinterpret_cast<cudaStream_t>(stream));
  if (err != cudaSuccess) return fail(GNB200_ERR_CUDA, "gnb200_fwd: CUDA error: %s", cudaGetErrorString(err));
  return GNB200_OK;
}

int gnb200_bwd(const void* dy, const void* x, const void* gamma, const void* beta, const float* mean,
               const float* rstd, int64_t N, int64_t R, int64_t C, int64_t G, int act, int dtype, void* dx,
               float* dgamma_dbeta_f32, void* dgamma, void* dbeta, void* workspace, size_t workspace_bytes,
               void* stream) {
  int rc = check_common(N, R, C, G, act, dtype);
  if (rc != GNB200_OK) return rc;
  if (!dy || !x || !gamma || !beta || !mean || !rstd || !dx || !dgamma_dbeta_f32)
    return fail(GNB200_ERR_INVALID_ARGUMENT, "gnb200_bwd: null tensor pointer");
  gnb200::Plan plan;
  const bool al = aligned16(x) && aligned16(dy) && aligned16(dx);
  if (!gnb200::make_plan(N, R, C, G, dtype, 1, al, &plan))
    return fail(GNB200_ERR_UNSUPPORTED, "gnb200_bwd: shape N=%lld R=%lld C=%lld G=%lld is outside the supported index range",
                (long long)N, (long long)R, (long long)C, (long long)G);
  if (plan.ws_bytes > 0 && (!workspace || workspace_bytes < plan.ws_bytes || !aligned16(workspace)))
    return fail(GNB200_ERR_WORKSPACE, "gnb200_bwd: needs a 16-byte aligned workspace of %zu bytes, got %zu at %p",
                plan.ws_bytes, workspace_bytes, workspace);
  gnb200::BwdCall call = {dy, x, gamma, beta, mean, rstd, dx, dgamma_dbeta_f32, dgamma, dbeta, workspace, act, dtype};
  const cudaError_t err = gnb200::launch_backward(call, plan, reinterpret_cast<cudaStream_t>(stream));
  if (err != cudaSuccess) return fail(GNB200_ERR_CUDA, "gnb200_bwd: CUDA error: %s", cudaGetErrorString(err));
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
