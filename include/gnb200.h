/*
 * gnb200 — channels-last (NHWC) GroupNorm + fused activation for NVIDIA B200 (sm_100a).
 *
 * C ABI of libgnb200.so.  Plain pointers and sizes only: no torch / ATen types cross this
 * boundary, so the library can be bound from C, C++, ctypes, cgo, JNI ...
 *
 * What each entry point stands in for in the reference project
 * (latentCall145/channels-last-groupnorm, paths relative to that project):
 *
 *   gnb200_fwd              <- run_gn_fwd_kernels<T>   src/gnnhwc/csrc/gn_kernel.h:11-24
 *                                                      (body: src/gnnhwc/csrc/gn_kernel.cu:439-531)
 *   gnb200_bwd              <- run_gn_bwd_kernels<T>   src/gnnhwc/csrc/gn_kernel.h:26-41
 *                                                      (body: src/gnnhwc/csrc/gn_kernel.cu:932-1055)
 *   gnb200_*_workspace_bytes<- the CUDACachingAllocator::raw_alloc sizes computed inside the two
 *                              launchers (gn_kernel.cu:461, 954, 973-974, 998-1001); here the caller
 *                              owns the scratch buffer instead
 *   gnb200_act_code         <- the activation_to_code table   src/gnnhwc/custom_gn.py:52-59
 *
 * Tensor layout (identical to the reference's (N, R, C) view, custom_gn.cpp:24,66-67):
 *   x, y, dy, dx : N * R * C elements, NHWC-contiguous (channel is the fastest dimension,
 *                  R = product of the spatial extents)
 *   gamma, beta  : C elements, same dtype as x
 *   mean, rstd   : N * G floats (always fp32; the reference stores them in the tensor dtype)
 *
 * Every pointer is a device pointer on the current CUDA device.  All work is enqueued on
 * `stream` and nothing synchronises with the host.  No entry point below allocates device
 * memory: scratch comes from the caller (`workspace`) or, for gnb200_bwd_static_scratch, from a
 * fixed array inside the library.
 *
 * The first call of a kernel variant on a device raises its shared-memory limit, asks the
 * driver how many thread-block clusters fit the device and resolves the address of a diagnostic
 * counter (all cached afterwards): make one call per problem before a stream capture.
 */
#ifndef GNB200_H_
#define GNB200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* element types of x / y / dy / dx / gamma / beta */
enum { GNB200_F32 = 0, GNB200_F16 = 1, GNB200_BF16 = 2 };

/* fused activation; same numbering as the reference (src/gnnhwc/custom_gn.py:52-59) */
enum {
  GNB200_ACT_IDENTITY = 0,
  GNB200_ACT_RELU = 1,
  GNB200_ACT_SILU = 2, /* alias "swish" */
  GNB200_ACT_GELU = 3, /* erf form */
  GNB200_ACT_GELU_TANH = 4
};

/* status codes: 0 = success, negative = failure (gnb200_last_error() has the text) */
enum {
  GNB200_OK = 0,
  GNB200_ERR_INVALID_ARGUMENT = -1, /* null pointer, bad dtype/activation, C % G != 0, sizes <= 0 ... */
  GNB200_ERR_WORKSPACE = -2,        /* workspace missing or smaller than gnb200_*_workspace_bytes() */
  GNB200_ERR_CUDA = -3,             /* a CUDA runtime call or kernel launch failed */
  GNB200_ERR_UNSUPPORTED = -4,      /* shape outside the supported index range */
  GNB200_ERR_EXCHANGE_TIMEOUT = -5  /* a kernel of an EARLIER call on this device gave up a bounded wait: every
                                       result since the last check is invalid; see gnb200_wait_timeouts() */
};

/* Library version, e.g. 100 = 0.1.0 */
int gnb200_version(void);

/* Text of the last failure on the calling thread ("" if none). Never NULL. */
const char* gnb200_last_error(void);

/* "identity" | "relu" | "silu" | "swish" | "gelu" | "gelu_tanh" -> code, or -1 if unknown. */
int gnb200_act_code(const char* name);

/* Scratch bytes that gnb200_fwd / gnb200_bwd need for this problem (0 is possible). */
size_t gnb200_fwd_workspace_bytes(int64_t N, int64_t R, int64_t C, int64_t G, int dtype);
size_t gnb200_bwd_workspace_bytes(int64_t N, int64_t R, int64_t C, int64_t G, int dtype);

/*
 * Forward:  y = act(gamma * (x - mean) * rstd + beta), statistics per (sample, group) over the
 * R * (C/G) elements of the slab, biased variance, rstd = 1/sqrt(var + eps).
 * Writes y (N*R*C), mean and rstd (N*G floats each).  `workspace` may be NULL when
 * gnb200_fwd_workspace_bytes() is 0.  `stream` is a cudaStream_t (NULL = default stream).
 */
int gnb200_fwd(const void* x, const void* gamma, const void* beta,
               int64_t N, int64_t R, int64_t C, int64_t G, double eps, int act, int dtype,
               void* y, float* mean, float* rstd,
               void* workspace, size_t workspace_bytes, void* stream);

/*
 * Backward.  Reads dy, x, gamma, beta and the mean/rstd written by gnb200_fwd.
 * Writes dx (N*R*C) and the parameter gradients:
 *   dgamma_dbeta_f32 : 2*C floats, [dgamma | dbeta] packed, summed over this call's N samples in
 *                      a fixed order (no atomics).  Required.  This is the buffer a data-parallel
 *                      caller all-reduces across ranks.
 *   dgamma, dbeta    : C elements each in the tensor dtype (what the reference returns,
 *                      custom_gn.cpp:70-71).  Either may be NULL to skip the cast.
 */
int gnb200_bwd(const void* dy, const void* x, const void* gamma, const void* beta,
               const float* mean, const float* rstd,
               int64_t N, int64_t R, int64_t C, int64_t G, int act, int dtype,
               void* dx, float* dgamma_dbeta_f32, void* dgamma, void* dbeta,
               void* workspace, size_t workspace_bytes, void* stream);

/*
 * Channels-first (NCHW) tensors: x, y, dy, dx are N * C * R elements with the pixel index fastest,
 * everything else as for gnb200_fwd / gnb200_bwd (same argument lists, same results, same status
 * codes; mean / rstd from gnb200_fwd_nchw feed gnb200_bwd_nchw).  The workspace is always needed
 * (sizes from the two queries below).  These replace the branch of the reference's module that hands
 * inputs whose channel stride is not 1 to torch's group_norm + activation
 * (src/gnnhwc/custom_gn.py:75-79): native kernels, no permute, no call into torch.
 */
size_t gnb200_fwd_nchw_workspace_bytes(int64_t N, int64_t R, int64_t C, int64_t G, int dtype);
size_t gnb200_bwd_nchw_workspace_bytes(int64_t N, int64_t R, int64_t C, int64_t G, int dtype);
int gnb200_fwd_nchw(const void* x, const void* gamma, const void* beta,
                    int64_t N, int64_t R, int64_t C, int64_t G, double eps, int act, int dtype,
                    void* y, float* mean, float* rstd,
                    void* workspace, size_t workspace_bytes, void* stream);
int gnb200_bwd_nchw(const void* dy, const void* x, const void* gamma, const void* beta,
                    const float* mean, const float* rstd,
                    int64_t N, int64_t R, int64_t C, int64_t G, int act, int dtype,
                    void* dx, float* dgamma_dbeta_f32, void* dgamma, void* dbeta,
                    void* workspace, size_t workspace_bytes, void* stream);

/*
 * Double precision, either layout.  The reference instantiates its launchers for double too
 * (src/gnnhwc/csrc/custom_gn.cpp:29-33, gn_kernel.cu:533-536, 1057-1060).  Tensors, parameters,
 * statistics and parameter gradients are all double here; gnb200_bwd_f64 needs a workspace of
 * gnb200_bwd_f64_workspace_bytes() bytes (2 * N * C doubles).  A compatibility path (one CTA per
 * (sample, group) slab), not a tuned one.  layout: GNB200_LAYOUT_NHWC or GNB200_LAYOUT_NCHW.
 */
enum { GNB200_LAYOUT_NHWC = 0, GNB200_LAYOUT_NCHW = 1 };
size_t gnb200_bwd_f64_workspace_bytes(int64_t N, int64_t R, int64_t C, int64_t G);
int gnb200_fwd_f64(const double* x, const double* gamma, const double* beta,
                   int64_t N, int64_t R, int64_t C, int64_t G, double eps, int act, int layout,
                   double* y, double* mean, double* rstd, void* stream);
int gnb200_bwd_f64(const double* dy, const double* x, const double* gamma, const double* beta,
                   const double* mean, const double* rstd,
                   int64_t N, int64_t R, int64_t C, int64_t G, int act, int layout,
                   double* dx, double* dgamma, double* dbeta,
                   void* workspace, size_t workspace_bytes, void* stream);

/*
 * Backward for callers that must not allocate device memory and therefore cannot supply the
 * `workspace` of gnb200_bwd: plugins of an inference runtime that owns all buffers, real-time
 * loops that may not touch the allocator, code inside a stream capture, thin FFI bindings that
 * only see the tensors they were handed.  Same arguments and results as gnb200_bwd without
 * `workspace` / `workspace_bytes`; the scratch is a fixed GNB200_STATIC_SCRATCH_BYTES array inside
 * the library (held on every GPU that loads the library until the process exits).
 * This entry point has no counterpart in the reference, whose launcher always allocates
 * (src/gnnhwc/csrc/gn_kernel.cu:954-1001).
 *   - A problem whose plan needs more scratch than the array returns GNB200_ERR_WORKSPACE
 *     (gnb200_last_error() states both sizes); nothing is launched.
 *   - The first call on a device resolves the array's device address; make it before any stream
 *     capture.  It never calls cudaMalloc / cudaFree or any allocating routine.
 *   - All calls on a device share the array: calls whose kernels may overlap on the GPU race and
 *     must be ordered by the caller.  Nothing needs clearing between calls.
 */
#define GNB200_STATIC_SCRATCH_BYTES (4u << 20)
int gnb200_bwd_static_scratch(const void* dy, const void* x, const void* gamma, const void* beta,
                              const float* mean, const float* rstd,
                              int64_t N, int64_t R, int64_t C, int64_t G, int act, int dtype,
                              void* dx, float* dgamma_dbeta_f32, void* dgamma, void* dbeta, void* stream);

/*
 * Data-parallel ranks on the GPUs of one node (the batch is split over the ranks; statistics are per
 * sample, so only dgamma / dbeta need the other ranks).  The sum over the ranks is done by the
 * library's own kernels over peer-mapped memory - no library collective, no multicast object:
 *   push     inside the kernel that produces [dgamma | dbeta], every rank stores its 2 * C floats
 *            into its slot of EVERY rank's exchange buffer (plain stores through peer-mapped pointers,
 *            NVLink), each value in one 8-byte store together with the number of the push;
 *   collect  a rank waits until all ranks' values with the expected number stand in its OWN buffer, adds
 *            them in rank order (all ranks get the same bits) and notes that the slots have been read,
 *            which its next push passes on to the peers and which frees the slots for the push after next.
 * gnb200_bwd_peer       = gnb200_bwd + push + collect in one call: dgamma_dbeta_f32 / dgamma / dbeta
 *                         hold the sums over the ranks (one NVLink round trip inside the call).
 * gnb200_bwd_peer_push  = gnb200_bwd + push: dgamma_dbeta_f32 holds this rank's own sums and the call
 *                         waits for nobody; gnb200_peer_collect, any time later on the same stream or
 *                         one ordered after it (typically before the optimizer step, when every
 *                         contribution has long arrived), writes the sums over the ranks.  At most two
 *                         pushes may be outstanding (pushed, not yet collected) per buffer set.
 * gnb200_allreduce_param_grads = push + collect on a finished buffer, in place (for the channels-first
 *                         entry points, or for gradients accumulated over several calls).
 * The reference has no multi-GPU code; these entry points have no counterpart there (they stand
 * where a framework would call an all-reduce after run_gn_bwd_kernels,
 * src/gnnhwc/csrc/gn_kernel.h:26-41).
 *   peer_bufs : host array of `world` device pointers; peer_bufs[q] is rank q's exchange buffer as
 *               mapped into THIS process (peer_bufs[rank] is this rank's own buffer).  Every buffer
 *               has gnb200_peer_exchange_bytes(C, world) bytes, is 16-byte aligned, was zeroed once
 *               before its first use and belongs to one (C, world) pair.  How the buffers are
 *               allocated and mapped (symmetric memory, CUDA IPC, cuMem) is the caller's business.
 *   dgamma, dbeta : optional typed copies (C elements of `dtype`) of the summed buffer.
 *   Every rank must make the same sequence of pushes and collects on a buffer set.  Waits for other
 *   ranks are bounded like every wait of the library (about a second): a rank that waits longer gets
 *   NaN gradients and GNB200_ERR_EXCHANGE_TIMEOUT from the next call on (see gnb200_wait_timeouts
 *   below).  With push and collect apart the ranks need not be in step during the backward pass;
 *   with gnb200_bwd_peer they must be within that second of each other.
 *   world == 1: no exchange (gnb200_bwd; collect leaves the buffer as it is).  1 <= world <= 16.
 */
size_t gnb200_peer_exchange_bytes(int64_t C, int world);
int gnb200_bwd_peer(const void* dy, const void* x, const void* gamma, const void* beta,
                    const float* mean, const float* rstd,
                    int64_t N, int64_t R, int64_t C, int64_t G, int act, int dtype,
                    void* dx, float* dgamma_dbeta_f32, void* dgamma, void* dbeta,
                    void* workspace, size_t workspace_bytes,
                    const void* const* peer_bufs, int rank, int world, void* stream);
int gnb200_bwd_peer_push(const void* dy, const void* x, const void* gamma, const void* beta,
                         const float* mean, const float* rstd,
                         int64_t N, int64_t R, int64_t C, int64_t G, int act, int dtype,
                         void* dx, float* dgamma_dbeta_f32,
                         void* workspace, size_t workspace_bytes,
                         const void* const* peer_bufs, int rank, int world, void* stream);
int gnb200_peer_collect(float* dgamma_dbeta_f32, void* dgamma, void* dbeta, int64_t C, int dtype,
                        const void* const* peer_bufs, int rank, int world, void* stream);
int gnb200_allreduce_param_grads(float* dgamma_dbeta_f32, void* dgamma, void* dbeta, int64_t C, int dtype,
                                 const void* const* peer_bufs, int rank, int world, void* stream);

/*
 * Describes the launch plan chosen for a problem ("fwd fused k=4 cw=64 ..."), for logs, tests
 * and benchmarks.  Writes at most buf_len bytes including the terminating NUL; returns the
 * number of bytes the full text needs.  direction: 0 = forward, 1 = backward.
 */
int gnb200_describe_plan(int64_t N, int64_t R, int64_t C, int64_t G, int dtype, int direction,
                         char* buf, int buf_len);

/*
 * Diagnostics.  The kernels wait for one another in a few places (the CTAs of a cluster exchange
 * statistics through shared-memory mailboxes; the persistent multi-pass kernels wait for the CTA
 * that merges a slab's partial sums).  Every such wait is bounded (about a second of SM clocks
 * and tens of thousands of polls): a wait that gives up is counted, the statistics or
 * coefficients it was waiting for become NaN - so y, mean, rstd or dx of the affected slabs are
 * NaN, never plausible-looking numbers - and the kernel runs to its end instead of hanging the
 * GPU.  The kernel also sets a word of mapped host memory, which gnb200_fwd / gnb200_bwd /
 * gnb200_bwd_static_scratch read without synchronising: from the next call on they launch nothing and
 * return GNB200_ERR_EXCHANGE_TIMEOUT until gnb200_clear_wait_timeouts() is called.
 * No counterpart in the reference (its kernels never wait for one another).
 *
 * gnb200_wait_timeouts        number of waits that gave up on the current device since the library
 *                             was loaded or cleared (0 in any healthy run; negative = error).
 *                             Synchronises with the device.
 * gnb200_clear_wait_timeouts  resets the count and re-arms the entry points.  Synchronises.
 */
long long gnb200_wait_timeouts(void);
int gnb200_clear_wait_timeouts(void);

/*
 * Self-test of the give-up path, for test suites only.  Runs the fused forward plan on the given
 * problem with a wait limit of about a millisecond while cluster rank 1 of every cluster withholds
 * its contribution to the exchange (decided on the host; nothing faults, traps or hangs: every CTA
 * pushes before it waits, every wait runs out, every CTA exits).  Afterwards y, mean and rstd are
 * NaN, gnb200_wait_timeouts() is positive and the other entry points return
 * GNB200_ERR_EXCHANGE_TIMEOUT until gnb200_clear_wait_timeouts().  The problem must take the fused
 * forward plan with a cluster of at least two CTAs and have no more (sample, column block) slabs
 * than clusters are resident at once (GNB200_ERR_UNSUPPORTED otherwise).
 * No counterpart in the reference.
 */
int gnb200_selftest_exchange_timeout(const void* x, const void* gamma, const void* beta,
                                     int64_t N, int64_t R, int64_t C, int64_t G, double eps, int act, int dtype,
                                     void* y, float* mean, float* rstd, void* stream);

/*
 * Tuning aid.  While a device buffer is registered here, the forward kernel of the wave plan (the
 * persistent kernel used for slabs that do not fit a cluster) stores the GPU's nanosecond timer at a
 * few points of every pass of every CTA: buffer[(cta * steps + step) * 4 + k], steps = 2 * waves, k =
 * 0 start of the step, 1 end of streaming (pass A) / statistics known (pass B), 2 partials delivered
 * (A) / output written (B), 3 slab merged and published (A).  NULL switches it off (the default).
 * Not thread-safe; no counterpart in the reference.
 */
void gnb200_debug_set_trace(void* device_buffer, size_t bytes);

/* Number of kernel launches gnb200_fwd / gnb200_bwd enqueue for this problem. */
int gnb200_launch_count(int64_t N, int64_t R, int64_t C, int64_t G, int dtype, int direction);

#ifdef __cplusplus
}
#endif
#endif /* GNB200_H_ */
