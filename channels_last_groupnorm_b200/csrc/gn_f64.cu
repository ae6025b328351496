// Double-precision GroupNorm (+activation), forward and backward, for NHWC and NCHW tensors.
//
// The reference instantiates its launchers for double as well (src/gnnhwc/csrc/custom_gn.cpp:29-33,
// gn_kernel.cu:533-536, 1057-1060) and its own test inputs are fp64 (test/check_outputs.py:161-185).
// fp64 is a compatibility path here, not a tuned one: one CTA per (sample, group) slab, statistics
// by two sweeps (sum, then squared deviations about the mean), every sum in double and in a fixed
// order.  Statistics, parameter gradients and scratch are double as well.
//
// Element (n, c, r):  NHWC  x[(n * R + r) * C + c]      NCHW  x[(n * C + c) * R + r]
#include "../../include/gnb200.h"
#include "gn_kernels.h"

namespace gnb200 {

namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ double act_fwd_d(int act, double v) {
  switch (act) {
    case kActIdentity: return v;
    case kActRelu: return v > 0.0 ? v : 0.0;
    case kActSilu: return v / (1.0 + exp(-v));
    case kActGelu: return 0.5 * v * (1.0 + erf(v * 0.70710678118654752440));
    default: {
      const double kBeta = 0.79788456080286535588;  // sqrt(2 / pi)
      return 0.5 * v * (1.0 + tanh(kBeta * (v + 0.044715 * v * v * v)));
    }
  }
}
// d act(v) / dv, the formulas of gn_kernel.cu:62-106 of the reference in double
__device__ __forceinline__ double act_grad_d(int act, double v) {
  switch (act) {
    case kActIdentity: return 1.0;
    case kActRelu: return v > 0.0 ? 1.0 : 0.0;
    case kActSilu: {
      const double s = 1.0 / (1.0 + exp(-v));
      return s * (1.0 + v * (1.0 - s));
    }
    case kActGelu: {
      const double cdf = 0.5 * (1.0 + erf(v * 0.70710678118654752440));
      const double pdf = exp(-0.5 * v * v) * 0.39894228040143267794;
      return cdf + v * pdf;
    }
    default: {
      const double kBeta = 0.79788456080286535588;
      const double t = tanh(kBeta * (v + 0.044715 * v * v * v));
      const double dinner = kBeta * (1.0 + 3.0 * 0.044715 * v * v);
      return 0.5 * (1.0 + t) + 0.5 * v * (1.0 - t * t) * dinner;
    }
  }
}

// CTA-wide sum in a fixed order (warp trees, then the warp results in warp order); every thread gets it
__device__ __forceinline__ double block_sum_d(double v, double* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int d = 16; d >= 1; d >>= 1) v += __shfl_down_sync(0xffffffffu, v, d);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  double t = 0.0;
  for (int w = 0; w < kThreads / 32; ++w) t += scratch[w];
  return t;
}

// Walks the D * R elements of slab (n, g) in memory order: i -> (channel, address)
struct Slab {
  const long long R, C, D;
  const long long base_c;  // first channel of the group
  const long long n;
  const bool nhwc;
  __device__ __forceinline__ long long count() const { return D * R; }
  __device__ __forceinline__ void at(long long i, long long& c, long long& addr) const {
    if (nhwc) {
      const long long r = i / D;
      c = base_c + (i - r * D);
      addr = (n * R + r) * C + c;
    } else {
      const long long cl = i / R;
      c = base_c + cl;
      addr = (n * C + c) * R + (i - cl * R);
    }
  }
};

__global__ void __launch_bounds__(kThreads)
    gn_f64_fwd_kernel(const double* __restrict__ x, const double* __restrict__ gamma, const double* __restrict__ beta,
                      double* __restrict__ y, double* __restrict__ mean_out, double* __restrict__ rstd_out, long long R,
                      long long C, long long G, double eps, int act, bool nhwc) {
  __shared__ double scratch[kThreads / 32];
  const long long n = blockIdx.x / G, grp = blockIdx.x - n * G, D = C / G;
  const Slab sl = {R, C, D, grp * D, n, nhwc};
  const long long m = sl.count();
  double s = 0.0;
  for (long long i = threadIdx.x; i < m; i += kThreads) {
    long long c, a;
    sl.at(i, c, a);
    s += x[a];
  }
  const double mu = block_sum_d(s, scratch) / (double)m;
  double q = 0.0;
  for (long long i = threadIdx.x; i < m; i += kThreads) {
    long long c, a;
    sl.at(i, c, a);
    const double d = x[a] - mu;
    q = fma(d, d, q);
  }
  const double rs = 1.0 / sqrt(block_sum_d(q, scratch) / (double)m + eps);
  if (threadIdx.x == 0) {
    mean_out[blockIdx.x] = mu;
    rstd_out[blockIdx.x] = rs;
  }
  for (long long i = threadIdx.x; i < m; i += kThreads) {
    long long c, a;
    sl.at(i, c, a);
    y[a] = act_fwd_d(act, fma((x[a] - mu) * rs, gamma[c], beta[c]));
  }
}

// sums[(n * C + c) * 2 + {0, 1}] = S1, S2 of (n, c);  dx of the slab
__global__ void __launch_bounds__(kThreads)
    gn_f64_bwd_kernel(const double* __restrict__ dy, const double* __restrict__ x, const double* __restrict__ gamma,
                      const double* __restrict__ beta, const double* __restrict__ mean_in,
                      const double* __restrict__ rstd_in, double* __restrict__ dx, double* __restrict__ sums,
                      long long R, long long C, long long G, int act, bool nhwc) {
  __shared__ double scratch[kThreads / 32];
  const long long n = blockIdx.x / G, grp = blockIdx.x - n * G, D = C / G;
  const double mu = mean_in[blockIdx.x], rs = rstd_in[blockIdx.x];
  // per-channel sums, one channel at a time (threads stride over the pixels), and the group sums
  double A = 0.0, B = 0.0;
  for (long long cl = 0; cl < D; ++cl) {
    const long long c = grp * D + cl;
    const double ga = gamma[c], be = beta[c];
    double s1 = 0.0, s2 = 0.0;
    for (long long r = threadIdx.x; r < R; r += kThreads) {
      const long long a = nhwc ? (n * R + r) * C + c : (n * C + c) * R + r;
      const double xh = (x[a] - mu) * rs;
      const double dyh = dy[a] * act_grad_d(act, fma(xh, ga, be));
      s1 += dyh;
      s2 = fma(dyh, xh, s2);
    }
    s1 = block_sum_d(s1, scratch);
    s2 = block_sum_d(s2, scratch);
    if (threadIdx.x == 0) {
      sums[(n * C + c) * 2] = s1;
      sums[(n * C + c) * 2 + 1] = s2;
    }
    A = fma(ga, s1, A);
    B = fma(ga, s2, B);
  }
  const double inv_m = 1.0 / ((double)D * (double)R);
  A *= inv_m;
  B *= inv_m;
  const Slab sl = {R, C, D, grp * D, n, nhwc};
  const long long m = sl.count();
  for (long long i = threadIdx.x; i < m; i += kThreads) {
    long long c, a;
    sl.at(i, c, a);
    const double ga = gamma[c];
    const double xh = (x[a] - mu) * rs;
    const double dyh = dy[a] * act_grad_d(act, fma(xh, ga, beta[c]));
    dx[a] = rs * (ga * dyh - A - xh * B);
  }
}

// dgamma_c = sum_n S2[n, c], dbeta_c = sum_n S1[n, c], samples in ascending order
__global__ void __launch_bounds__(kThreads)
    gn_f64_param_kernel(const double* __restrict__ sums, long long N, long long C, double* __restrict__ dgamma,
                        double* __restrict__ dbeta) {
  const long long c = (long long)blockIdx.x * kThreads + threadIdx.x;
  if (c >= C) return;
  double t1 = 0.0, t2 = 0.0;
  for (long long n = 0; n < N; ++n) {
    t1 += sums[(n * C + c) * 2];
    t2 += sums[(n * C + c) * 2 + 1];
  }
  dgamma[c] = t2;
  dbeta[c] = t1;
}

}  // namespace

cudaError_t launch_forward_f64(const double* x, const double* gamma, const double* beta, long long N, long long R,
                               long long C, long long G, double eps, int act, bool nhwc, double* y, double* mean,
                               double* rstd, cudaStream_t stream) {
  gn_f64_fwd_kernel<<<(unsigned)(N * G), kThreads, 0, stream>>>(x, gamma, beta, y, mean, rstd, R, C, G, eps, act, nhwc);
  return cudaGetLastError();
}

cudaError_t launch_backward_f64(const double* dy, const double* x, const double* gamma, const double* beta,
                                const double* mean, const double* rstd, long long N, long long R, long long C,
                                long long G, int act, bool nhwc, double* dx, double* dgamma, double* dbeta,
                                double* sums, cudaStream_t stream) {
  gn_f64_bwd_kernel<<<(unsigned)(N * G), kThreads, 0, stream>>>(dy, x, gamma, beta, mean, rstd, dx, sums, R, C, G, act,
                                                               nhwc);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return err;
  gn_f64_param_kernel<<<(unsigned)((C + kThreads - 1) / kThreads), kThreads, 0, stream>>>(sums, N, C, dgamma, dbeta);
  return cudaGetLastError();
}

}  // namespace gnb200
