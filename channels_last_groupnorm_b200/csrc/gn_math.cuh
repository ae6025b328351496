// Per-thread arithmetic shared by the forward / backward kernels of every launch plan: running
// moments, affine coefficients, and one row of the backward sums.
#pragma once
#include "gn_common.cuh"

namespace gnb200 {

template <int VE>
__device__ __forceinline__ void welford_step(const float (&f)[VE], float (&mean)[VE], float (&m2)[VE], float& cnt) {
  cnt += 1.0f;
  const float inv = __fdividef(1.0f, cnt);
#pragma unroll
  for (int e = 0; e < VE; ++e) {
    const float d = f[e] - mean[e];
    mean[e] = fmaf(d, inv, mean[e]);
    m2[e] = fmaf(d, f[e] - mean[e], m2[e]);
  }
}

// 16-bit tensors accumulate shifted sums instead: with K a value of the thread's own data (its
// first row),  s += x - K,  q += (x - K)^2;  the subtraction converts the 16-bit element on the fly
// (mixed-precision sub), three instructions per element and no division in the loop.  Because K is
// one of the samples, (K - mean)^2 <= M2, so q <= (n + 1) M2 and the cancellation in
// M2 = q - s^2 / n costs at most (n + 1) ulp of the thread's M2 - n is the thread's row count, a
// few hundred at most - where sums of raw squares would lose mean^2 / var.
template <typename T, int VE, int KN>
__device__ __forceinline__ void shifted_step(const uint4& w, const float (&K)[KN], float (&s)[VE], float (&q)[VE]) {
  static_assert(sizeof(T) == 2 && VE == 8, "16-bit elements, 16-byte vectors");
  const uint32_t r[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    uint16_t lo, hi;
    split_halves(r[e], lo, hi);
    const float d0 = mixed_sub<T>(lo, K[KN == 1 ? 0 : 2 * e]);
    const float d1 = mixed_sub<T>(hi, K[KN == 1 ? 0 : 2 * e + 1]);
    s[2 * e] += d0;
    s[2 * e + 1] += d1;
    q[2 * e] = fmaf(d0, d0, q[2 * e]);
    q[2 * e + 1] = fmaf(d1, d1, q[2 * e + 1]);
  }
}

// (s, q) about K over `rows` rows  ->  per-lane (mean, M2); s and q are overwritten.
template <int VE, int KN>
__device__ __forceinline__ void shifted_finish(const float (&K)[KN], int rows, float (&mean)[VE], float (&m2)[VE],
                                               float& cnt) {
  cnt = (float)rows;
  const float inv = rows > 0 ? 1.0f / cnt : 0.f;
#pragma unroll
  for (int e = 0; e < VE; ++e) {
    const float s = mean[e], q = m2[e];
    const float ds = s * inv;
    mean[e] = K[KN == 1 ? 0 : e] + ds;
    m2[e] = fmaxf(fmaf(-s, ds, q), 0.f);
  }
}

// Per-lane affine coefficients  a = rstd * gamma,  b = beta - mean * a  for the thread's channels.
// `stat_mean` / `stat_rstd` are indexed by group relative to g_base.  UNI: all VE channels of the
// thread belong to one group, so the statistics are looked up once.
template <typename T, int VE, bool UNI>
__device__ __forceinline__ void lane_affine(const T* gamma, const T* beta, const float* stat_mean,
                                            const float* stat_rstd, int g_base, int c_first, const FastDiv div_D,
                                            float (&a)[VE], float (&b)[VE]) {
  float ga[VE], be[VE];
  load_params<T, VE>(gamma, c_first, ga);
  load_params<T, VE>(beta, c_first, be);
  if constexpr (UNI) {
    const int s = div_D.div(c_first) - g_base;
    const float mu = stat_mean[s], rs = stat_rstd[s];
#pragma unroll
    for (int e = 0; e < VE; ++e) {
      a[e] = rs * ga[e];
      b[e] = fmaf(-mu, a[e], be[e]);
    }
  } else {
#pragma unroll
    for (int e = 0; e < VE; ++e) {
      const int s = div_D.div(c_first + e) - g_base;
      a[e] = stat_rstd[s] * ga[e];
      b[e] = fmaf(-stat_mean[s], a[e], be[e]);
    }
  }
}

// The same from parameter vectors fetched earlier (raw 16-byte loads issued before phase 1 so that
// their latency is off the critical path between the statistics and the output pass).
template <typename T, int VE, bool UNI>
__device__ __forceinline__ void lane_affine_raw(const uint4& ga_raw, const uint4& be_raw, const float* stat_mean,
                                                const float* stat_rstd, int g_base, int c_first, const FastDiv div_D,
                                                float (&a)[VE], float (&b)[VE]) {
  static_assert(sizeof(T) * VE == 16, "16-byte vectors only");
  float ga[VE], be[VE];
  unpack16<T, VE>(ga_raw, ga);
  unpack16<T, VE>(be_raw, be);
  if constexpr (UNI) {
    const int s = div_D.div(c_first) - g_base;
    const float mu = stat_mean[s], rs = stat_rstd[s];
#pragma unroll
    for (int e = 0; e < VE; ++e) {
      a[e] = rs * ga[e];
      b[e] = fmaf(-mu, a[e], be[e]);
    }
  } else {
#pragma unroll
    for (int e = 0; e < VE; ++e) {
      const int s = div_D.div(c_first + e) - g_base;
      a[e] = stat_rstd[s] * ga[e];
      b[e] = fmaf(-stat_mean[s], a[e], be[e]);
    }
  }
}

template <typename T, int VE>
struct BwdLane {
  float r[VE];    // rstd of the lane's group
  float nmr[VE];  // -mean * rstd
  float ga[VE];   // gamma
  float be[VE];   // beta
};

// UNI: all VE channels of the thread belong to one group (one statistics lookup; the compiler
// then keeps a single register for each of r / nmr).
template <typename T, int VE, bool UNI>
__device__ __forceinline__ void lane_setup(const T* gamma, const T* beta, const float* mean_n, const float* rstd_n,
                                           int c_first, const FastDiv div_D, BwdLane<T, VE>& L) {
  load_params<T, VE>(gamma, c_first, L.ga);
  load_params<T, VE>(beta, c_first, L.be);
  if constexpr (UNI) {
    const int grp = div_D.div(c_first);
    const float rs = rstd_n[grp];
    const float nm = -mean_n[grp] * rs;
#pragma unroll
    for (int e = 0; e < VE; ++e) {
      L.r[e] = rs;
      L.nmr[e] = nm;
    }
  } else {
#pragma unroll
    for (int e = 0; e < VE; ++e) {
      const int grp = div_D.div(c_first + e);
      const float rs = rstd_n[grp];
      L.r[e] = rs;
      L.nmr[e] = -mean_n[grp] * rs;
    }
  }
}

// One row of phase 1: dyh = dy * act'(yh) for the thread's VE channels, sums updated.
template <typename T, int VE, int ACT>
__device__ __forceinline__ void bwd_row_sums(const float (&fx)[VE], float (&fd)[VE], const BwdLane<T, VE>& L,
                                             float (&s1)[VE], float (&s2)[VE]) {
  float xh[VE], yh[VE], gr[VE];
#pragma unroll
  for (int e = 0; e < VE; ++e) {
    xh[e] = fmaf(fx[e], L.r[e], L.nmr[e]);
    yh[e] = fmaf(xh[e], L.ga[e], L.be[e]);
  }
  act_grad_vec<T, VE, ACT>(yh, gr);
#pragma unroll
  for (int e = 0; e < VE; ++e) {
    fd[e] *= gr[e];
    s1[e] += fd[e];
    s2[e] = fmaf(fd[e], xh[e], s2[e]);
  }
}

// 16-bit tensors, fused path: yh straight from x (a = rstd * gamma, b = beta - mean * a) and S2
// accumulated against the raw x; the caller converts it with S2 = rstd * (S2raw - mean * S1).  One
// FMA per element less; the conversion's rounding (relative 1e-7 * |mean| * rstd) is far below a
// 16-bit result.
// It works on the packed 16-bit values: dyh = dy * act'(yh) is formed two channels at a time in the tensor's own 16-bit format - which is
// the format it is parked in anyway - and enters the fp32 sums through mixed-precision add / fma,
// so dy is never unpacked and dyh never packed.  act' is evaluated in f16x2; for bf16 tensors it
// is rounded to bf16 before the product.  Returns the packed dyh.
template <typename T, int ACT>
__device__ __forceinline__ uint4 bwd_row_sums_packed(const uint4& xw, const uint4& dw, const float (&a)[8],
                                                     const float (&b)[8], float (&s1)[8], float (&s2)[8]) {
  static_assert(sizeof(T) == 2, "16-bit tensors only");
  const uint32_t xr[4] = {xw.x, xw.y, xw.z, xw.w}, dr[4] = {dw.x, dw.y, dw.z, dw.w};
  uint32_t out[4];
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    uint16_t x0, x1;
    split_halves(xr[p], x0, x1);
    uint32_t dyh = dr[p];
    if constexpr (ACT != kActIdentity) {
      const float yh0 = fmaf(mixed_add<T>(x0, -0.0f), a[2 * p], b[2 * p]);
      const float yh1 = fmaf(mixed_add<T>(x1, -0.0f), a[2 * p + 1], b[2 * p + 1]);
      const __half2 g = act_grad_h2<ACT>(f32x2_to_h2_sat(yh0, yh1));
      if constexpr (std::is_same<T, __half>::value) {
        const __half2 r = __hmul2(*reinterpret_cast<const __half2*>(&dr[p]), g);
        dyh = *reinterpret_cast<const uint32_t*>(&r);
      } else {
        const float2 gf = __half22float2(g);
        const __nv_bfloat162 gb = __floats2bfloat162_rn(gf.x, gf.y);
        const __nv_bfloat162 r = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&dr[p]), gb);
        dyh = *reinterpret_cast<const uint32_t*>(&r);
      }
    }
    uint16_t d0, d1;
    split_halves(dyh, d0, d1);
    s1[2 * p] = mixed_add<T>(d0, s1[2 * p]);
    s1[2 * p + 1] = mixed_add<T>(d1, s1[2 * p + 1]);
    s2[2 * p] = mixed_fma<T>(d0, x0, s2[2 * p]);
    s2[2 * p + 1] = mixed_fma<T>(d1, x1, s2[2 * p + 1]);
    out[p] = dyh;
  }
  return make_uint4(out[0], out[1], out[2], out[3]);
}

}  // namespace gnb200
