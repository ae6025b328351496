/*
 * TEST INFRASTRUCTURE ONLY - never linked into, imported by or shipped with the product library.
 *
 * Plain-C, double-precision restatement of the channels-last GroupNorm (+activation) algorithm of
 * latentCall145/channels-last-groupnorm.  Each function names the reference code it follows
 * (paths relative to that project).  Used as the checker by tests/, by the smoke run and by the
 * CPU-baseline leg of the benchmark.
 *
 * Parity pin: the reference has no CPU implementation and no golden vectors of its own
 * (its tests compare against torch on the GPU).  This oracle is therefore pinned three ways by
 * tests/test_oracle.py: against torch.nn.functional.group_norm + activation in fp64 (autograd
 * for the gradients), against outputs of the unmodified reference extension recorded on a B200
 * (tests/golden/, produced by tests/golden/make_golden.py), and against finite differences.
 *
 * Layout: x, dy, y, dx are N*R*C doubles, NHWC (channel fastest); gamma, beta: C; mean, rstd: N*G.
 */
#include <math.h>
#include <stddef.h>
#include <stdlib.h>

typedef struct {
  double mean, m2, nf;
} welford_t;

/* Welford.h:33-47  WelfordOps::reduce - add one sample */
static welford_t welford_reduce(welford_t acc, double data) {
  welford_t r;
  r.nf = acc.nf + 1.0;
  double delta = data - acc.mean;
  r.mean = acc.mean + delta / r.nf;
  r.m2 = acc.m2 + delta * (data - r.mean);
  return r;
}

/* Welford.h:48-66  WelfordOps::combine - merge two partial results (Chan et al.) */
static welford_t welford_combine(welford_t a, welford_t b) {
  if (a.nf == 0) return b;
  if (b.nf == 0) return a;
  welford_t r;
  double delta = b.mean - a.mean;
  r.nf = a.nf + b.nf;
  double nb_over_n = b.nf / r.nf;
  r.mean = a.mean + delta * nb_over_n;
  r.m2 = a.m2 + b.m2 + delta * delta * a.nf * nb_over_n;
  return r;
}

/* gn_kernel.cu:121-128  closest_factor - largest divisor of n that is <= sqrt(n) */
static long closest_factor(long n) {
  long f = 1;
  for (long i = 1; i * i <= n; ++i)
    if (n % i == 0) f = i;
  return f;
}

/* gn_kernel.cu:62-87  activations; codes as in custom_gn.py:52-59 */
static double act_fn(int act, double x) {
  switch (act) {
    case 1: return x > 0 ? x : 0.0;
    case 2: return x / (1.0 + exp(-x));
    case 3: return x * 0.5 * (1.0 + erf(x * M_SQRT1_2));
    case 4: {
      const double kBeta = M_SQRT2 * M_2_SQRTPI * 0.5, kKappa = 0.044715;
      return 0.5 * x * (1.0 + tanh(kBeta * (x + kKappa * x * x * x)));
    }
    default: return x;
  }
}

/* gn_kernel.cu:63-106  derivatives of the activations */
static double act_grad(int act, double x) {
  switch (act) {
    case 1: return x > 0 ? 1.0 : 0.0;
    case 2: {
      const double s = 1.0 / (1.0 + exp(-x));
      return s * (1.0 + x * (1.0 - s));
    }
    case 3: {
      const double kBeta = M_2_SQRTPI * M_SQRT1_2 * 0.5;
      const double cdf = 0.5 * (1.0 + erf(x * M_SQRT1_2));
      const double pdf = exp(-0.5 * x * x) * kBeta;
      return cdf + x * pdf;
    }
    case 4: {
      const double kBeta = M_SQRT2 * M_2_SQRTPI * 0.5, kKappa = 0.044715;
      const double x_sq = x * x, inner = kBeta * (x + kKappa * x_sq * x), t = tanh(inner);
      const double left = 0.5 * x, right = 1.0 + t;
      return 0.5 * right + left * (1.0 - t * t) * kBeta * (1.0 + 3.0 * kKappa * x_sq);
    }
    default: return 1.0;
  }
}

/*
 * Forward.  Statistics follow the reference's two stages: compute_stats_pt1 (gn_kernel.cu:132-224)
 * reduces each of H' rows of W' pixels of a group with Welford, compute_stats_pt2 (226-292)
 * combines the H' partials and projects to mean and rstd = rsqrt(var + eps) with biased variance
 * (Welford.h:67-72, correction 0; gn_kernel.cu:290-291).  scale_shift_kernel (305-412) then
 * applies y = act(x * a + b) with a = rstd * gamma, b = beta - mean * a (gn_kernel.cu:350-351).
 */
void gn_oracle_fwd(const double* x, const double* gamma, const double* beta, long N, long R, long C, long G,
                   double eps, int act, double* y, double* mean, double* rstd) {
  const long D = C / G;
  const long Hp = closest_factor(R), Wp = R / Hp;
  for (long n = 0; n < N; ++n) {
    for (long g = 0; g < G; ++g) {
      welford_t total = {0, 0, 0};
      for (long h = 0; h < Hp; ++h) {
        welford_t row = {0, 0, 0};
        for (long w = 0; w < Wp; ++w) {
          const double* px = x + ((n * R + h * Wp + w) * C + g * D);
          for (long d = 0; d < D; ++d) row = welford_reduce(row, px[d]);
        }
        total = welford_combine(total, row);
      }
      const double var = total.m2 / total.nf;
      const double mu = total.mean, rs = 1.0 / sqrt(var + eps);
      mean[n * G + g] = mu;
      rstd[n * G + g] = rs;
      for (long r = 0; r < R; ++r) {
        const double* px = x + ((n * R + r) * C + g * D);
        double* py = y + ((n * R + r) * C + g * D);
        for (long d = 0; d < D; ++d) {
          const double a = rs * gamma[g * D + d];
          const double b = beta[g * D + d] - mu * a;
          py[d] = act_fn(act, px[d] * a + b);
        }
      }
    }
  }
}

/*
 * Backward, in the reference's own formulation:
 *   width_reduce + height_reduce (gn_kernel.cu:557-693): per (n, c)
 *       xdy_sum = sum_r dy * act'(x*a+b) * x,   dy_sum = sum_r dy * act'(x*a+b)     (613-618)
 *   compute_dweight_dbias (695-728):
 *       dweight_c = sum_n (xdy_sum - mean * dy_sum) * rstd,   dbias_c = sum_n dy_sum   (723-727)
 *   compute_bwd_scale_biases (730-801): per (n, g) with s = 1 / (D * R)
 *       c1 = (mean * sum_c gamma dy_sum - sum_c gamma xdy_sum) * s * rstd^3
 *       c2 = -mean * c1 - sum_c gamma dy_sum * s * rstd                                  (797-800)
 *   dx_elem_kernel (803-905):  dx = a * dy * act'(x*a+b) + c1 * x + c2                   (868-872)
 * dgamma and dbeta are overwritten (no accumulation into the caller's buffers).
 */
void gn_oracle_bwd(const double* dy, const double* x, const double* gamma, const double* beta, const double* mean,
                   const double* rstd, long N, long R, long C, long G, int act, double* dx, double* dgamma,
                   double* dbeta) {
  const long D = C / G;
  double* xdy_sum = (double*)calloc((size_t)(N * C), sizeof(double));
  double* dy_sum = (double*)calloc((size_t)(N * C), sizeof(double));
  for (long n = 0; n < N; ++n) {
    for (long g = 0; g < G; ++g) {
      const double mu = mean[n * G + g], rs = rstd[n * G + g];
      for (long d = 0; d < D; ++d) {
        const long c = g * D + d;
        const double a = rs * gamma[c], b = beta[c] - mu * a;
        double s_xdy = 0, s_dy = 0;
        for (long r = 0; r < R; ++r) {
          const long i = (n * R + r) * C + c;
          const double dyh = dy[i] * act_grad(act, x[i] * a + b);
          s_xdy += dyh * x[i];
          s_dy += dyh;
        }
        xdy_sum[n * C + c] = s_xdy;
        dy_sum[n * C + c] = s_dy;
      }
      double xdy_gamma = 0, dy_gamma = 0;
      for (long d = 0; d < D; ++d) {
        const long c = g * D + d;
        xdy_gamma += gamma[c] * xdy_sum[n * C + c];
        dy_gamma += gamma[c] * dy_sum[n * C + c];
      }
      const double s = 1.0 / (double)(D * R);
      const double c1 = (mu * dy_gamma - xdy_gamma) * s * rs * rs * rs;
      const double c2 = -mu * c1 - dy_gamma * s * rs;
      for (long r = 0; r < R; ++r) {
        for (long d = 0; d < D; ++d) {
          const long c = g * D + d;
          const long i = (n * R + r) * C + c;
          const double a = rs * gamma[c], b = beta[c] - mu * a;
          dx[i] = a * dy[i] * act_grad(act, x[i] * a + b) + c1 * x[i] + c2;
        }
      }
    }
  }
  for (long c = 0; c < C; ++c) {
    const long g = c / D;
    double s1 = 0, s2 = 0;
    for (long n = 0; n < N; ++n) {
      s1 += (xdy_sum[n * C + c] - mean[n * G + g] * dy_sum[n * C + c]) * rstd[n * G + g];
      s2 += dy_sum[n * C + c];
    }
    dgamma[c] = s1;
    dbeta[c] = s2;
  }
  free(xdy_sum);
  free(dy_sum);
}
