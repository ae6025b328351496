// GroupNorm (+activation) for channels-first (NCHW) tensors, forward and backward, sm_100a.
//
// The reference sends inputs whose channel stride is not 1 to torch's group_norm followed by the
// activation (src/gnnhwc/custom_gn.py:75-79); there is no permute here and no call into torch: in
// NCHW storage the slab of (sample n, group g) is one contiguous run of D * R elements, and the R
// pixels of a channel are contiguous inside it, so the statistics are plain contiguous reductions
// and gamma / beta are per-run scalars.
//
//   forward   stats kernel (partial moments per slab chunk) -> apply kernel (merges the slab's
//             partials in a fixed order, then y = act(x a_c + b_c))
//   backward  reduce kernel (one warp per piece of a channel row: S1, S2) -> finalize kernel
//             (per-channel sums, group sums A, B) -> parameter-gradient kernel -> dx kernel
//
// Vectors are 16 bytes when R is a multiple of the vector width and the pointers are aligned (every
// channel row then starts on a 16-byte boundary), single elements otherwise.  Sums are fp32, formed in
// an order fixed by the launch geometry: no atomics, bit-identical reruns.
#include "gn_kernels.h"
#include "gn_math.cuh"

namespace gnb200 {

namespace {

constexpr int kThreads = 256;
constexpr int kUnroll = 4;

struct NchwGeom {
  int N, C, G, D;
  long long R;
  long long slab_vecs;   // vectors per (n, g) slab: D * R / VE
  long long chunk_vecs;  // forward: vectors per CTA chunk
  int chunks;            // forward: chunks per slab
  long long row_vecs;    // backward: vectors per channel row: R / VE
  long long piece_vecs;  // backward: vectors per warp piece
  int ppr;               // backward: pieces per channel row
  FastDiv div_R;         // element offset inside a slab -> channel (R < 2^31)
};

template <typename T, int VE>
__device__ __forceinline__ void load_vec(const T* p, float (&f)[VE]) {
  if constexpr (sizeof(T) * VE == 16) {
    unpack16<T, VE>(ldg128(p), f);
  } else {
#pragma unroll
    for (int e = 0; e < VE; ++e) f[e] = load_param<T>(p, e);
  }
}
template <typename T, int VE>
__device__ __forceinline__ void store_vec(T* p, const float (&f)[VE]) {
  if constexpr (sizeof(T) * VE == 16) {
    stg128(p, pack16<T, VE>(f));
  } else {
#pragma unroll
    for (int e = 0; e < VE; ++e) p[e] = store_param<T>(f[e]);
  }
}

// ------------------------------------------------------------------------------------------------
// forward 1: partial moments of chunk `chunk` of slab `slab` -> part[slab * chunks + chunk] = (mean, M2, n, -)
// ------------------------------------------------------------------------------------------------
template <typename T, int VE>
__global__ void __launch_bounds__(kThreads)
    gn_nchw_stats_kernel(const T* __restrict__ x, float4* __restrict__ part, const NchwGeom g) {
  __shared__ float scratch[kThreads / 32];
  grid_dep_launch_dependents();  // the apply kernel may take its place; it waits for this grid's partials
  const long long slab = blockIdx.x / g.chunks;
  const int chunk = (int)(blockIdx.x - slab * g.chunks);
  const long long v0 = (long long)chunk * g.chunk_vecs;
  const long long v1 = min(g.slab_vecs, v0 + g.chunk_vecs);
  const T* base = x + slab * g.slab_vecs * VE;
  // per-thread Welford over the lanes of its vectors (one count for all lanes)
  float mean[VE], m2[VE], cnt = 0.f;
#pragma unroll
  for (int e = 0; e < VE; ++e) mean[e] = 0.f, m2[e] = 0.f;
  long long v = v0 + threadIdx.x;
  for (; v + (kUnroll - 1) * kThreads < v1; v += kUnroll * kThreads) {
    float f[kUnroll][VE];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) load_vec<T, VE>(base + (v + u * kThreads) * VE, f[u]);
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) welford_step<VE>(f[u], mean, m2, cnt);
  }
  for (; v < v1; v += kThreads) {
    float f[VE];
    load_vec<T, VE>(base + v * VE, f);
    welford_step<VE>(f, mean, m2, cnt);
  }
  // lanes -> thread, then threads -> CTA: mean first, squared deviations about it second
  float tsum = 0.f;
#pragma unroll
  for (int e = 0; e < VE; ++e) tsum += mean[e];
  const float n_cta = block_sum(cnt * (float)VE, scratch);
  const float mu = block_sum(cnt * tsum, scratch) / n_cta;
  float dev = 0.f;
#pragma unroll
  for (int e = 0; e < VE; ++e) {
    const float d = mean[e] - mu;
    dev += fmaf(cnt * d, d, m2[e]);
  }
  const float M2 = block_sum(dev, scratch);
  if (threadIdx.x == 0) part[blockIdx.x] = make_float4(mu, M2, n_cta, 0.f);
}

// Fixed-order merge of the `chunks` partials of a slab by one warp (sums about the first chunk's
// mean, so that nothing cancels for a large |mean|).  Every lane returns the result.
__device__ __forceinline__ void merge_partials(const float4* __restrict__ p, int chunks, float eps, float& mu, float& rs) {
  const int lane = threadIdx.x & 31;
  const float K0 = p[0].x;
  float an = 0.f, ad = 0.f, aq = 0.f;
  for (int i = lane; i < chunks; i += 32) {
    const float4 v = p[i];
    const float d = v.x - K0;
    an += v.z;
    ad = fmaf(v.z, d, ad);
    aq += fmaf(v.z * d, d, v.y);
  }
#pragma unroll
  for (int b = 16; b >= 1; b >>= 1) {
    an += __shfl_xor_sync(0xffffffffu, an, b);
    ad += __shfl_xor_sync(0xffffffffu, ad, b);
    aq += __shfl_xor_sync(0xffffffffu, aq, b);
  }
  const float dm = ad / an;
  mu = K0 + dm;
  rs = rsqrtf(fmaxf(fmaf(-ad, dm, aq) / an, 0.f) + eps);
}

// ------------------------------------------------------------------------------------------------
// forward 2: statistics of the slab, then y = act(x * a_c + b_c) over the chunk
// ------------------------------------------------------------------------------------------------
template <typename T, int VE, int ACT>
__global__ void __launch_bounds__(kThreads)
    gn_nchw_apply_kernel(const T* __restrict__ x, const T* __restrict__ gamma, const T* __restrict__ beta,
                         const float4* __restrict__ part, T* __restrict__ y, float* __restrict__ mean_out,
                         float* __restrict__ rstd_out, float eps, const NchwGeom g) {
  constexpr bool FAST = sizeof(T) == 2;
  __shared__ float s_stat[2];
  const long long slab = blockIdx.x / g.chunks;
  const int chunk = (int)(blockIdx.x - slab * g.chunks);
  grid_dep_wait();  // the statistics kernel's partials
  if (threadIdx.x < 32) {
    float mu, rs;
    merge_partials(part + slab * g.chunks, g.chunks, eps, mu, rs);
    if (threadIdx.x == 0) {
      s_stat[0] = mu;
      s_stat[1] = rs;
      if (chunk == 0) {
        mean_out[slab] = mu;
        rstd_out[slab] = rs;
      }
    }
  }
  __syncthreads();
  const float mu = s_stat[0], rs = s_stat[1];
  const int c_base = (int)(slab % g.G) * g.D;
  const long long v0 = (long long)chunk * g.chunk_vecs;
  const long long v1 = min(g.slab_vecs, v0 + g.chunk_vecs);
  const T* xs = x + slab * g.slab_vecs * VE;
  T* ys = y + slab * g.slab_vecs * VE;
  auto one = [&](long long v, const float (&f)[VE]) {
    // VE > 1: the vector lies inside one channel row (R is a multiple of VE)
    const int c = c_base + g.div_R.div((int)(v * VE));
    const float a = rs * load_param<T>(gamma, c);
    const float b = fmaf(-mu, a, load_param<T>(beta, c));
    float o[VE];
#pragma unroll
    for (int e = 0; e < VE; ++e) o[e] = fmaf(f[e], a, b);
    if constexpr (sizeof(T) * VE == 16) {
      stg128(ys + v * VE, act_pack16<T, VE, ACT>(o));
    } else {
#pragma unroll
      for (int e = 0; e < VE; ++e) ys[v * VE + e] = store_param<T>(act_fwd<ACT, FAST>(o[e]));
    }
  };
  long long v = v0 + threadIdx.x;
  for (; v + (kUnroll - 1) * kThreads < v1; v += kUnroll * kThreads) {
    float f[kUnroll][VE];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) load_vec<T, VE>(xs + (v + u * kThreads) * VE, f[u]);
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) one(v + u * kThreads, f[u]);
  }
  for (; v < v1; v += kThreads) {
    float f[VE];
    load_vec<T, VE>(xs + v * VE, f);
    one(v, f);
  }
}

// ------------------------------------------------------------------------------------------------
// backward 1: one warp per piece of a channel row:  tp[(n * C + c) * ppr + j] = (S1, S2)
// ------------------------------------------------------------------------------------------------
template <typename T, int VE, int ACT>
__global__ void __launch_bounds__(kThreads)
    gn_nchw_reduce_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ gamma,
                          const T* __restrict__ beta, const float* __restrict__ mean_in,
                          const float* __restrict__ rstd_in, float2* __restrict__ tp, long long pieces,
                          const NchwGeom g) {
  grid_dep_launch_dependents();  // the kernels after this one wait for this grid before they read its sums
  const int lane = threadIdx.x & 31;
  const long long piece = (long long)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
  if (piece >= pieces) return;
  const long long row = piece / g.ppr;  // n * C + c
  const int j = (int)(piece - row * g.ppr);
  const int n = (int)(row / g.C), c = (int)(row - (long long)n * g.C);
  const int grp = c / g.D;
  const float rs = rstd_in[(size_t)n * g.G + grp];
  const float nmr = -mean_in[(size_t)n * g.G + grp] * rs;
  const float ga = load_param<T>(gamma, c), be = load_param<T>(beta, c);
  const long long v0 = (long long)j * g.piece_vecs;
  const long long v1 = min(g.row_vecs, v0 + g.piece_vecs);
  const T* xs = x + row * g.R;
  const T* ds = dy + row * g.R;
  float s1 = 0.f, s2 = 0.f;
  auto one = [&](const float (&fx)[VE], const float (&fd)[VE]) {
    float xh[VE], yh[VE], gr[VE];
#pragma unroll
    for (int e = 0; e < VE; ++e) {
      xh[e] = fmaf(fx[e], rs, nmr);
      yh[e] = fmaf(xh[e], ga, be);
    }
    act_grad_vec<T, VE, ACT>(yh, gr);
#pragma unroll
    for (int e = 0; e < VE; ++e) {
      const float dyh = fd[e] * gr[e];
      s1 += dyh;
      s2 = fmaf(dyh, xh[e], s2);
    }
  };
  long long v = v0 + lane;
  for (; v + (kUnroll - 1) * 32 < v1; v += kUnroll * 32) {
    float fx[kUnroll][VE], fd[kUnroll][VE];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      load_vec<T, VE>(xs + (v + u * 32) * VE, fx[u]);
      load_vec<T, VE>(ds + (v + u * 32) * VE, fd[u]);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) one(fx[u], fd[u]);
  }
  for (; v < v1; v += 32) {
    float fx[VE], fd[VE];
    load_vec<T, VE>(xs + v * VE, fx);
    load_vec<T, VE>(ds + v * VE, fd);
    one(fx, fd);
  }
#pragma unroll
  for (int b = 16; b >= 1; b >>= 1) {
    s1 += __shfl_xor_sync(0xffffffffu, s1, b);
    s2 += __shfl_xor_sync(0xffffffffu, s2, b);
  }
  if (lane == 0) tp[piece] = make_float2(s1, s2);
}

// backward 2: one CTA per (n, g): channel sums over the pieces (ascending) -> sums[n * C + c], and
// the gamma-weighted group sums -> coef[(n * G + g) * 2] = A, B
template <typename T>
__global__ void __launch_bounds__(128)
    gn_nchw_finalize_kernel(const float2* __restrict__ tp, const T* __restrict__ gamma, float2* __restrict__ sums,
                            float* __restrict__ coef, const NchwGeom g) {
  __shared__ float scratch[4];
  grid_dep_launch_dependents();
  grid_dep_wait();  // the reduce kernel's sums
  const int n = blockIdx.x / g.G, grp = blockIdx.x - n * g.G;
  float w1 = 0.f, w2 = 0.f;
  for (int cl = threadIdx.x; cl < g.D; cl += 128) {
    const int c = grp * g.D + cl;
    const float2* p = tp + ((size_t)n * g.C + c) * g.ppr;
    float t1 = 0.f, t2 = 0.f;
    for (int j = 0; j < g.ppr; ++j) {
      t1 += p[j].x;
      t2 += p[j].y;
    }
    sums[(size_t)n * g.C + c] = make_float2(t1, t2);
    const float ga = load_param<T>(gamma, c);
    w1 = fmaf(ga, t1, w1);
    w2 = fmaf(ga, t2, w2);
  }
  w1 = block_sum(w1, scratch);
  w2 = block_sum(w2, scratch);
  if (threadIdx.x == 0) {
    const float inv_m = 1.0f / ((float)g.D * (float)g.R);
    coef[(size_t)blockIdx.x * 2] = w1 * inv_m;
    coef[(size_t)blockIdx.x * 2 + 1] = w2 * inv_m;
  }
}

// backward 4: dx = rstd * (gamma_c * dyh - A - xh * B), one warp per piece as in the reduce kernel
template <typename T, int VE, int ACT>
__global__ void __launch_bounds__(kThreads)
    gn_nchw_dx_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ gamma,
                      const T* __restrict__ beta, const float* __restrict__ mean_in, const float* __restrict__ rstd_in,
                      const float* __restrict__ coef, T* __restrict__ dx, long long pieces, const NchwGeom g) {
  const int lane = threadIdx.x & 31;
  const long long piece = (long long)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
  if (piece >= pieces) return;
  const long long row = piece / g.ppr;
  const int j = (int)(piece - row * g.ppr);
  const int n = (int)(row / g.C), c = (int)(row - (long long)n * g.C);
  const int grp = c / g.D;
  const float rs = rstd_in[(size_t)n * g.G + grp];
  const float nmr = -mean_in[(size_t)n * g.G + grp] * rs;
  const float ga = load_param<T>(gamma, c), be = load_param<T>(beta, c);
  const float ag = rs * ga;
  grid_dep_wait();  // the finalize kernel's coefficients (everything above is the caller's)
  const float nb = -rs * coef[((size_t)n * g.G + grp) * 2 + 1];
  const float na = -rs * coef[((size_t)n * g.G + grp) * 2];
  const long long v0 = (long long)j * g.piece_vecs;
  const long long v1 = min(g.row_vecs, v0 + g.piece_vecs);
  const T* xs = x + row * g.R;
  const T* ds = dy + row * g.R;
  T* os = dx + row * g.R;
  auto one = [&](long long v, const float (&fx)[VE], const float (&fd)[VE]) {
    float xh[VE], yh[VE], gr[VE], o[VE];
#pragma unroll
    for (int e = 0; e < VE; ++e) {
      xh[e] = fmaf(fx[e], rs, nmr);
      yh[e] = fmaf(xh[e], ga, be);
    }
    act_grad_vec<T, VE, ACT>(yh, gr);
#pragma unroll
    for (int e = 0; e < VE; ++e) o[e] = fmaf(ag, fd[e] * gr[e], fmaf(nb, xh[e], na));
    store_vec<T, VE>(os + v * VE, o);
  };
  long long v = v0 + lane;
  for (; v + (kUnroll - 1) * 32 < v1; v += kUnroll * 32) {
    float fx[kUnroll][VE], fd[kUnroll][VE];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      load_vec<T, VE>(xs + (v + u * 32) * VE, fx[u]);
      load_vec<T, VE>(ds + (v + u * 32) * VE, fd[u]);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) one(v + u * 32, fx[u], fd[u]);
  }
  for (; v < v1; v += 32) {
    float fx[VE], fd[VE];
    load_vec<T, VE>(xs + v * VE, fx);
    load_vec<T, VE>(ds + v * VE, fd);
    one(v, fx, fd);
  }
}

// ------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------
constexpr int kSmCount = 148;

// n / d for 0 <= n < 2^31 (same construction as the NHWC planner's)
FastDiv fast_div(long long d) {
  FastDiv f;
  if (d < 1) d = 1;
  uint32_t s = 0;
  while ((1ull << s) < (unsigned long long)d) ++s;
  f.mul = (uint32_t)(((1ull << 32) * ((1ull << s) - (unsigned long long)d)) / (unsigned long long)d + 1);
  f.shr = s;
  return f;
}

NchwGeom make_geom(long long N, long long R, long long C, long long G, int ve) {
  NchwGeom g = {};
  g.N = (int)N, g.C = (int)C, g.G = (int)G, g.D = (int)(C / G), g.R = R;
  g.slab_vecs = (long long)g.D * R / ve;
  g.row_vecs = R / ve;
  g.div_R = fast_div(R);
  // forward: about four CTAs per SM, at least 2048 vectors (32 KB) per chunk
  const long long slabs = N * G;
  long long chunks = (4LL * kSmCount + slabs - 1) / slabs;
  const long long max_chunks = (g.slab_vecs + 2047) / 2048;
  if (chunks > max_chunks) chunks = max_chunks;
  if (chunks < 1) chunks = 1;
  if (chunks > 1024) chunks = 1024;
  g.chunk_vecs = (g.slab_vecs + chunks - 1) / chunks;
  g.chunks = (int)((g.slab_vecs + g.chunk_vecs - 1) / g.chunk_vecs);
  // backward: one warp per piece of a channel row; about 16 warps per SM, 128 .. 2048 vectors per piece
  const long long rows = N * C;
  long long ppr = (16LL * kSmCount + rows - 1) / rows;
  const long long max_ppr = (g.row_vecs + 127) / 128;
  if (ppr > max_ppr) ppr = max_ppr;
  if (ppr < 1) ppr = 1;
  long long piece = (g.row_vecs + ppr - 1) / ppr;
  if (piece > 2048) piece = 2048;
  piece = (piece + 31) / 32 * 32;
  g.piece_vecs = piece;
  g.ppr = (int)((g.row_vecs + piece - 1) / piece);
  return g;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

struct BwdScratch {
  size_t tp, sums, coef, total;
};
BwdScratch bwd_scratch(const NchwGeom& g) {
  BwdScratch s;
  s.tp = 0;
  s.sums = (size_t)g.N * g.C * g.ppr * sizeof(float2);
  s.coef = s.sums + (size_t)g.N * g.C * sizeof(float2);
  s.total = (s.coef + (size_t)g.N * g.G * 2 * sizeof(float) + 15) & ~(size_t)15;
  return s;
}

template <typename T, int VE, int ACT>
cudaError_t fwd_t(const FwdCall& c, const NchwGeom& g, cudaStream_t stream) {
  float4* part = static_cast<float4*>(c.workspace);
  const unsigned grid = (unsigned)((long long)g.N * g.G * g.chunks);
  gn_nchw_stats_kernel<T, VE><<<grid, kThreads, 0, stream>>>((const T*)c.x, part, g);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return err;
  return launch_chained(gn_nchw_apply_kernel<T, VE, ACT>, grid, dim3(kThreads), 0, stream, chain_enabled(), (const T*)c.x,
                        (const T*)c.gamma, (const T*)c.beta, part, (T*)c.y, c.mean, c.rstd, c.eps, g);
}

template <typename T, int VE, int ACT>
cudaError_t bwd_t(const BwdCall& c, const NchwGeom& g, cudaStream_t stream) {
  const BwdScratch s = bwd_scratch(g);
  char* ws = static_cast<char*>(c.workspace);
  float2* tp = reinterpret_cast<float2*>(ws + s.tp);
  float2* sums = reinterpret_cast<float2*>(ws + s.sums);
  float* coef = reinterpret_cast<float*>(ws + s.coef);
  const long long pieces = (long long)g.N * g.C * g.ppr;
  const unsigned grid = (unsigned)((pieces + kThreads / 32 - 1) / (kThreads / 32));
  gn_nchw_reduce_kernel<T, VE, ACT><<<grid, kThreads, 0, stream>>>((const T*)c.dy, (const T*)c.x, (const T*)c.gamma,
                                                                   (const T*)c.beta, c.mean, c.rstd, tp, pieces, g);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) return err;
  const bool chain = chain_enabled();
  err = launch_chained(gn_nchw_finalize_kernel<T>, (unsigned)(g.N * g.G), dim3(128), 0, stream, chain, tp, (const T*)c.gamma,
                       sums, coef, g);
  if (err != cudaSuccess) return err;
  err = launch_param_grads(c, reinterpret_cast<const float*>(sums), g.N, g.C, stream, chain);
  if (err != cudaSuccess) return err;
  return launch_chained(gn_nchw_dx_kernel<T, VE, ACT>, grid, dim3(kThreads), 0, stream, chain, (const T*)c.dy, (const T*)c.x,
                        (const T*)c.gamma, (const T*)c.beta, c.mean, c.rstd, coef, (T*)c.dx, pieces, g);
}

template <typename T, int VE>
cudaError_t fwd_act(const FwdCall& c, const NchwGeom& g, cudaStream_t stream) {
  switch (c.act) {
    case kActIdentity: return fwd_t<T, VE, kActIdentity>(c, g, stream);
    case kActRelu: return fwd_t<T, VE, kActRelu>(c, g, stream);
    case kActSilu: return fwd_t<T, VE, kActSilu>(c, g, stream);
    case kActGelu: return fwd_t<T, VE, kActGelu>(c, g, stream);
    default: return fwd_t<T, VE, kActGeluTanh>(c, g, stream);
  }
}
template <typename T, int VE>
cudaError_t bwd_act(const BwdCall& c, const NchwGeom& g, cudaStream_t stream) {
  switch (c.act) {
    case kActIdentity: return bwd_t<T, VE, kActIdentity>(c, g, stream);
    case kActRelu: return bwd_t<T, VE, kActRelu>(c, g, stream);
    case kActSilu: return bwd_t<T, VE, kActSilu>(c, g, stream);
    case kActGelu: return bwd_t<T, VE, kActGelu>(c, g, stream);
    default: return bwd_t<T, VE, kActGeluTanh>(c, g, stream);
  }
}

int vector_width(long long R, int dtype, bool aligned) {
  const int vfull = dtype == 0 ? 4 : 8;
  return (aligned && R % vfull == 0) ? vfull : 1;
}

}  // namespace

bool nchw_shape_supported(int64_t N, int64_t R, int64_t C, int64_t G) {
  if (N < 1 || R < 1 || C < 1 || G < 1 || C % G != 0) return false;
  if (R > 0x7fffffffLL || C > (1 << 24) || N * G > 0x7fffffffLL || N * C > 0x7fffffffLL) return false;
  if ((C / G) * R > 0x7fffffffLL) return false;  // offsets inside a slab are 32-bit
  return (double)N * (double)R * (double)C <= 9.0e15;
}

size_t nchw_workspace_bytes(int64_t N, int64_t R, int64_t C, int64_t G, int dtype, int direction) {
  if (!nchw_shape_supported(N, R, C, G)) return 0;
  size_t best = 0;
  for (int aligned = 0; aligned < 2; ++aligned) {
    const NchwGeom g = make_geom(N, R, C, G, vector_width(R, dtype, aligned != 0));
    const size_t need = direction == 0 ? (((size_t)g.N * g.G * g.chunks * sizeof(float4) + 15) & ~(size_t)15)
                                       : bwd_scratch(g).total;
    if (need > best) best = need;
  }
  return best;
}

int nchw_launch_count(int direction) { return direction == 0 ? 2 : 4; }

cudaError_t launch_forward_nchw(const FwdCall& c, int64_t N, int64_t R, int64_t C, int64_t G, cudaStream_t stream) {
  const bool al = aligned16(c.x) && aligned16(c.y);
  const int ve = vector_width(R, c.dtype, al);
  const NchwGeom g = make_geom(N, R, C, G, ve);
  switch (c.dtype) {
    case 0: return ve == 1 ? fwd_act<float, 1>(c, g, stream) : fwd_act<float, 4>(c, g, stream);
    case 1: return ve == 1 ? fwd_act<__half, 1>(c, g, stream) : fwd_act<__half, 8>(c, g, stream);
    default: return ve == 1 ? fwd_act<__nv_bfloat16, 1>(c, g, stream) : fwd_act<__nv_bfloat16, 8>(c, g, stream);
  }
}

cudaError_t launch_backward_nchw(const BwdCall& c, int64_t N, int64_t R, int64_t C, int64_t G, cudaStream_t stream) {
  const bool al = aligned16(c.x) && aligned16(c.dy) && aligned16(c.dx);
  const int ve = vector_width(R, c.dtype, al);
  const NchwGeom g = make_geom(N, R, C, G, ve);
  switch (c.dtype) {
    case 0: return ve == 1 ? bwd_act<float, 1>(c, g, stream) : bwd_act<float, 4>(c, g, stream);
    case 1: return ve == 1 ? bwd_act<__half, 1>(c, g, stream) : bwd_act<__half, 8>(c, g, stream);
    default: return ve == 1 ? bwd_act<__nv_bfloat16, 1>(c, g, stream) : bwd_act<__nv_bfloat16, 8>(c, g, stream);
  }
}

}  // namespace gnb200
