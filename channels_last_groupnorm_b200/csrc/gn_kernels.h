// Host-side declarations shared by the planner, the launchers and the C ABI.
#pragma once
#include <stddef.h>
#include <stdint.h>

#include "gn_common.cuh"
#include "gn_peer.cuh"

namespace gnb200 {

// A launch plan for one direction of one problem.
struct Plan {
  bool fused;         // true: one cluster kernel holds the slab on chip; false: a multi-pass path
  bool wave;          // multi-pass as one persistent cooperative kernel (gn_wave.cu, geometry in wgeom)
  int ve;             // elements per thread-vector (16 bytes worth, or 1)
  int threads;        // CTA size
  long long grid;     // CTAs of the streaming kernels
  size_t smem_bytes;  // dynamic shared memory of the first streaming kernel
  size_t ws_bytes;    // scratch bytes this plan needs
  int launches;       // kernels enqueued per call
  bool chain;         // kernels after the first are launched as programmatic dependents of their predecessor
  Geom geom;
  WaveGeom wgeom;
};

struct FwdCall {
  const void* x;
  const void* gamma;
  const void* beta;
  void* y;
  float* mean;
  float* rstd;
  void* workspace;
  float eps;
  int act;
  int dtype;
  // exchange self-test only (gnb200_selftest_exchange_timeout): the cluster rank that withholds
  // its pushes (-1: none) and the give-up limit of the waits in SM clocks (0: the default)
  int test_skip_push_rank = -1;
  long long test_wait_clocks = 0;
};

struct BwdCall {
  const void* dy;
  const void* x;
  const void* gamma;
  const void* beta;
  const float* mean;
  const float* rstd;
  void* dx;
  float* dparam_f32;  // [dgamma | dbeta], 2*C floats
  void* dgamma;       // optional, tensor dtype
  void* dbeta;        // optional, tensor dtype
  void* workspace;
  int act;
  int dtype;
  // optional: the parameter gradients are summed over the ranks of one node inside the kernel that
  // produces them (gn_peer.cuh); null or world <= 1: the gradients of this rank only
  const PeerExchange* peer = nullptr;
};

// direction: 0 forward, 1 backward.  `aligned16`: every tensor pointer is 16-byte aligned.
// Returns false (and leaves *plan untouched) if the shape cannot be indexed.
bool make_plan(int64_t N, int64_t R, int64_t C, int64_t G, int dtype, int direction, bool aligned16, Plan* plan);

// Largest scratch requirement over the plans the library may pick for this problem.
size_t plan_workspace_bytes(int64_t N, int64_t R, int64_t C, int64_t G, int dtype, int direction);

// Raises a kernel's dynamic shared-memory limit (and allows a non-portable cluster size) once per
// device and kernel; later calls with a request that is already covered cost one map lookup.
cudaError_t ensure_kernel_attributes(const void* func, size_t smem_bytes, bool nonportable_cluster);

// Number of clusters of `cfg` (cluster dimension, block size and dynamic shared memory set) that
// can be resident on the current device at once (>= 1), cached per device, kernel and shape.
cudaError_t resident_clusters(const void* func, const cudaLaunchConfig_t* cfg, int* clusters);

// Limits and give-up record of the kernels' bounded waits on the current device (device counter,
// mapped host word, default limits).  The first call in a process allocates the host words.
cudaError_t wait_limit_for_device(WaitLimit* out);
// True once a kernel on the current device has recorded a wait that gave up; no synchronisation.
bool wait_gave_up_on_current_device();
void clear_wait_mirror_on_current_device();

// wave plan (gn_wave.cu)
void debug_set_trace(void* ptr, size_t bytes);
size_t wave_workspace_bytes(const WaveGeom& g, int direction);
cudaError_t launch_forward_wave(const FwdCall& c, const Plan& p, cudaStream_t stream);
cudaError_t launch_backward_wave(const BwdCall& c, const Plan& p, cudaStream_t stream);
// dgamma / dbeta from `rows` rows of per-channel (S1, S2) pairs (gn_bwd.cu)
// `chained`: as a programmatic dependent of the kernel before it in the stream
cudaError_t launch_param_grads(const BwdCall& c, const float* sums, int rows, int C, cudaStream_t stream,
                               bool chained = false);
// Exchange of a finished [dgamma | dbeta] buffer over the ranks of c.peer (gn_bwd.cu): `push` posts the
// buffer's values, `collect` replaces them (and the typed copies) by the sums over the ranks
cudaError_t launch_param_exchange(const BwdCall& c, int C, cudaStream_t stream, bool chained, bool push, bool collect);
// GNB200_CHAIN != 0 (the default): the kernels of a multi-kernel call are launched as programmatic
// dependents of their predecessors
bool chain_enabled();

// channels-first tensors (gn_nchw.cu)
bool nchw_shape_supported(int64_t N, int64_t R, int64_t C, int64_t G);
size_t nchw_workspace_bytes(int64_t N, int64_t R, int64_t C, int64_t G, int dtype, int direction);
int nchw_launch_count(int direction);
cudaError_t launch_forward_nchw(const FwdCall& c, int64_t N, int64_t R, int64_t C, int64_t G, cudaStream_t stream);
cudaError_t launch_backward_nchw(const BwdCall& c, int64_t N, int64_t R, int64_t C, int64_t G, cudaStream_t stream);
// double precision, either layout (gn_f64.cu); `sums` holds 2 * N * C doubles
cudaError_t launch_forward_f64(const double* x, const double* gamma, const double* beta, long long N, long long R,
                               long long C, long long G, double eps, int act, bool nhwc, double* y, double* mean,
                               double* rstd, cudaStream_t stream);
cudaError_t launch_backward_f64(const double* dy, const double* x, const double* gamma, const double* beta,
                                const double* mean, const double* rstd, long long N, long long R, long long C,
                                long long G, int act, bool nhwc, double* dx, double* dgamma, double* dbeta,
                                double* sums, cudaStream_t stream);

// Launches `kern`; with `chained` as a programmatic dependent of the previous kernel in `stream`
// (the kernel must call grid_dep_wait() before it touches anything that kernel wrote).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_chained(void (*kern)(KArgs...), unsigned grid, dim3 block, size_t smem, cudaStream_t stream,
                                  bool chained, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = chained ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

cudaError_t launch_forward(const FwdCall& c, const Plan& p, cudaStream_t stream);
cudaError_t launch_backward(const BwdCall& c, const Plan& p, cudaStream_t stream);

}  // namespace gnb200
