// Backward GroupNorm (+activation) kernels for NHWC tensors, sm_100a.
//
// With  xh = (x - mean) * rstd,  yh = gamma * xh + beta,  dyh = dy * act'(yh)  the
// per-(sample, channel) sums are
//     S1[n,c] = sum_r dyh          S2[n,c] = sum_r dyh * xh
// and  dbeta_c = sum_n S1,  dgamma_c = sum_n S2,
//      A[n,g] = sum_{c in g} gamma_c S1 / (D R),   B[n,g] = sum_{c in g} gamma_c S2 / (D R),
//      dx = rstd * (gamma_c * dyh - A - xh * B).
// This is the reference's formula (src/gnnhwc/csrc/gn_kernel.cu:613-618, 723-727, 786-800,
// 868-872) rewritten in terms of xh so that no large terms cancel when |mean| >> 1/rstd.
//
//  fused   one launch + a tiny parameter-gradient kernel.  A cluster of k CTAs owns one (sample,
//          column block) slab: it reads x and dy once from HBM, reduces S1/S2, keeps dyh in shared
//          memory, exchanges the group sums by pushing them into its peers' shared memory
//          (st.async + mbarrier, no cluster barrier) and writes dx from the dyh tile and x, which
//          it reads a second time from L2 a few microseconds after the first read (the slab share
//          of all resident CTAs is a few tens of MB, far below L2).
//          HBM traffic: x and dy read once, dx written once.
//  two-pass  reduce kernel (per-tile channel sums to scratch) -> finalize (fixed-order sums, A, B)
//          -> parameter-gradient kernel -> apply kernel (reverse tile order for L2 reuse).
//
// Every sum is formed in an order fixed by the launch geometry: no atomics, bit-identical reruns.
#include <stdlib.h>

#include "gn_kernels.h"
#include "gn_math.cuh"

namespace gnb200 {

constexpr int kRingDepth = 4;  // rows in flight per thread in the multi-kernel reduce kernel

// Phase 1 of the multi-kernel path: S1, S2 over the thread's rows.  16-byte vectors of x and dy
// travel through two shared-memory rings with cp.async (kRingDepth rows per thread in flight,
// no registers held); slot s of the thread lives at ring + s * ring_stride.
template <typename T, int VE, int ACT>
__device__ __forceinline__ void stream_bwd_sums(const T* __restrict__ gx, const T* __restrict__ gd,
                                                size_t gstep_elems, int iters, uint32_t ring_x, uint32_t ring_d,
                                                uint32_t ring_stride, const BwdLane<T, VE>& L, float (&s1)[VE],
                                                float (&s2)[VE]) {
  if constexpr (sizeof(T) * VE == 16) {
    constexpr bool kRaw = sizeof(T) == 2;  // 16-bit tensors: packed arithmetic, S2 against the raw x
    float a[VE], b[VE];
#pragma unroll
    for (int e = 0; e < VE; ++e) {
      a[e] = L.r[e] * L.ga[e];
      b[e] = fmaf(L.nmr[e], L.ga[e], L.be[e]);
    }
#pragma unroll
    for (int d = 0; d < kRingDepth; ++d) {
      if (d < iters) {
        cp_async16(ring_x + d * ring_stride, gx);
        cp_async16(ring_d + d * ring_stride, gd);
        gx += gstep_elems;
        gd += gstep_elems;
      }
      cp_async_commit();
    }
    for (int i = 0; i < iters; ++i) {
      cp_async_wait<kRingDepth - 1>();
      const uint32_t off = (i & (kRingDepth - 1)) * ring_stride;
      const uint4 xw = lds128(ring_x + off), dw = lds128(ring_d + off);
      if (i + kRingDepth < iters) {
        cp_async16(ring_x + off, gx);
        cp_async16(ring_d + off, gd);
        gx += gstep_elems;
        gd += gstep_elems;
      }
      cp_async_commit();
      if constexpr (kRaw) {
        bwd_row_sums_packed<T, ACT>(xw, dw, a, b, s1, s2);
      } else {
        float fx[VE], fd[VE];
        unpack16<T, VE>(xw, fx);
        unpack16<T, VE>(dw, fd);
        bwd_row_sums<T, VE, ACT>(fx, fd, L, s1, s2);
      }
    }
    if constexpr (kRaw) {  // S2 = sum dyh * xh = rstd * (sum dyh * x - mean * sum dyh)
#pragma unroll
      for (int e = 0; e < VE; ++e) s2[e] = fmaf(L.r[e], s2[e], L.nmr[e] * s1[e]);
    }
  } else {
    for (int i = 0; i < iters; ++i) {
      float fx[VE], fd[VE];
#pragma unroll
      for (int e = 0; e < VE; ++e) {
        fx[e] = load_param<T>(gx, e);
        fd[e] = load_param<T>(gd, e);
      }
      gx += gstep_elems;
      gd += gstep_elems;
      bwd_row_sums<T, VE, ACT>(fx, fd, L, s1, s2);
    }
  }
}

constexpr int kXRing = 4;  // x rows in flight per thread in the fused backward kernel

// Phase 1 of the fused path.  dy rows are copied straight into the shared-memory tile, x rows go
// through a kXRing-deep shared-memory ring (cp.async, one commit group per row, kXRing rows in
// flight per thread).  dyh = dy * act'(yh) is accumulated into the channel sums and written back
// over the dy tile, rounded to T, so that phase 2 does not evaluate the activation derivative
// again.  (For 16-bit T this rounds dyh once more than a recompute would: half a unit in the last
// place of T on one term of dx.)  x is not kept on chip: phase 2 reads it again from L2.
// State of the copy pipeline between its start (tile_fill_start) and the loop that consumes it.
template <typename T>
struct BwdPipe {
  const T* gx;
  const T* gd;
  uint32_t wd;
  int dy_issued;
};

// Starts the copies of phase 1.  dy needs no ring - every row has its own tile slot - so it runs
// kXRing rows ahead of x: commit group j holds x row j and dy row j + kXRing, after a first group
// with dy rows 0 .. kXRing - 1.  Called before the thread fetches its parameters and statistics,
// so that their latency overlaps the first rows' instead of preceding it.
template <typename T, int VE>
__device__ __forceinline__ BwdPipe<T> tile_fill_start(const T* __restrict__ gx, const T* __restrict__ gd,
                                                      size_t gstep_elems, uint32_t ring, uint32_t ring_stride,
                                                      uint32_t sd, uint32_t sstep_bytes, int iters) {
  BwdPipe<T> p = {gx, gd, sd, 0};
  if constexpr (sizeof(T) * VE == 16) {
#pragma unroll
    for (int d = 0; d < kXRing; ++d) {
      if (d < iters) {
        cp_async16(p.wd, p.gd);
        p.gd += gstep_elems;
        p.wd += sstep_bytes;
        ++p.dy_issued;
      }
    }
    cp_async_commit();
#pragma unroll
    for (int d = 0; d < kXRing; ++d) {
      if (d < iters) {
        cp_async16(ring + d * ring_stride, p.gx);
        p.gx += gstep_elems;
      }
      if (p.dy_issued < iters) {
        cp_async16(p.wd, p.gd);
        p.gd += gstep_elems;
        p.wd += sstep_bytes;
        ++p.dy_issued;
      }
      cp_async_commit();
    }
  }
  return p;
}

template <typename T, int VE, int ACT>
__device__ __forceinline__ void tile_fill_bwd_sums(BwdPipe<T> pipe, size_t gstep_elems, uint32_t ring,
                                                   uint32_t ring_stride, uint32_t sd, uint32_t sstep_bytes, int iters,
                                                   const BwdLane<T, VE>& L, float (&s1)[VE], float (&s2)[VE]) {
  const T* gx = pipe.gx;
  const T* gd = pipe.gd;
  if constexpr (sizeof(T) * VE == 16) {
    constexpr bool kRaw = sizeof(T) == 2;
    float a[VE], b[VE];
#pragma unroll
    for (int e = 0; e < VE; ++e) {
      a[e] = L.r[e] * L.ga[e];
      b[e] = fmaf(L.nmr[e], L.ga[e], L.be[e]);
    }
    uint32_t wd = pipe.wd;
    int dy_issued = pipe.dy_issued;
    uint32_t rd = sd;
    for (int i = 0; i < iters; ++i) {
      cp_async_wait<kXRing - 1>();
      const uint32_t slot = ring + (i & (kXRing - 1)) * ring_stride;
      const uint4 xw = lds128(slot), dw = lds128(rd);
      if (i + kXRing < iters) {
        cp_async16(slot, gx);
        gx += gstep_elems;
      }
      if (dy_issued < iters) {
        cp_async16(wd, gd);
        gd += gstep_elems;
        wd += sstep_bytes;
        ++dy_issued;
      }
      cp_async_commit();
      if constexpr (kRaw) {
        const uint4 dyh = bwd_row_sums_packed<T, ACT>(xw, dw, a, b, s1, s2);
        if constexpr (ACT != kActIdentity) sts128(rd, dyh);  // identity: dyh is dy, already in place
      } else {
        float fx[VE], fd[VE];
        unpack16<T, VE>(xw, fx);
        unpack16<T, VE>(dw, fd);
        bwd_row_sums<T, VE, ACT>(fx, fd, L, s1, s2);
        sts128(rd, pack16<T, VE>(fd));
      }
      rd += sstep_bytes;
    }
    if constexpr (kRaw) {  // S2 = sum dyh * xh = rstd * (sum dyh * x - mean * sum dyh)
#pragma unroll
      for (int e = 0; e < VE; ++e) s2[e] = fmaf(L.r[e], s2[e], L.nmr[e] * s1[e]);
    }
  } else {
    T* wd = reinterpret_cast<T*>(__cvta_shared_to_generic(sd));
    for (int i = 0; i < iters; ++i) {
      float fx[VE], fd[VE];
#pragma unroll
      for (int e = 0; e < VE; ++e) {
        fx[e] = load_param<T>(gx, e);
        fd[e] = load_param<T>(gd, e);
      }
      bwd_row_sums<T, VE, ACT>(fx, fd, L, s1, s2);
#pragma unroll
      for (int e = 0; e < VE; ++e) wd[e] = store_param<T>(fd[e]);
      gx += gstep_elems;
      gd += gstep_elems;
      wd += sstep_bytes / sizeof(T);
    }
  }
}

// Starts the ring of phase 2: the thread's first kXRing x rows, one commit group each.
template <typename T, int VE>
__device__ __forceinline__ void tile_bwd_dx_start(const T* __restrict__ gx, size_t gstep_elems, uint32_t ring,
                                                  uint32_t ring_stride, int iters) {
  if constexpr (sizeof(T) * VE == 16) {
#pragma unroll
    for (int d = 0; d < kXRing; ++d) {
      if (d < iters) {
        cp_async16(ring + d * ring_stride, gx);
        gx += gstep_elems;
      }
      cp_async_commit();
    }
  }
}

// Phase 2 of the fused path: dx = ag * dyh + (nb * xh + na); dyh from the shared-memory tile, x
// a second time from global memory (an L2 hit: it was read microseconds earlier) through the same
// ring.  ag = rstd * gamma, nb = -rstd * B, na = -rstd * A per lane.
template <typename T, int VE>
__device__ __forceinline__ void tile_bwd_dx(const T* __restrict__ gx, uint32_t ring, uint32_t ring_stride,
                                            uint32_t sd, uint32_t sstep_bytes, T* __restrict__ gdst,
                                            size_t gstep_elems, int iters, const BwdLane<T, VE>& L,
                                            const float (&A)[VE], const float (&B)[VE]) {
  float ag[VE], nb[VE], na[VE];
#pragma unroll
  for (int e = 0; e < VE; ++e) {
    ag[e] = L.r[e] * L.ga[e];
    nb[e] = -L.r[e] * B[e];
    na[e] = -L.r[e] * A[e];
  }
  if constexpr (sizeof(T) * VE == 16) {
    // 16-bit results: fold xh = r x + nmr into the coefficients (nb xh + na = c1 x + c2); the
    // extra rounding is far below the 16-bit result.  fp32 keeps the xh form.
    constexpr bool kFold = sizeof(T) == 2;
    float c1[VE], c2[VE];
#pragma unroll
    for (int e = 0; e < VE; ++e) {
      c1[e] = nb[e] * L.r[e];
      c2[e] = fmaf(nb[e], L.nmr[e], na[e]);
    }
    T* gp = gdst;
    gx += (size_t)min(iters, kXRing) * gstep_elems;  // tile_bwd_dx_start has issued these rows
    for (int i = 0; i < iters; ++i) {
      cp_async_wait<kXRing - 1>();
      const uint32_t slot = ring + (i & (kXRing - 1)) * ring_stride;
      float fx[VE], fd[VE];
      unpack16<T, VE>(lds128(slot), fx);
      unpack16<T, VE>(lds128(sd), fd);
      sd += sstep_bytes;
      if (i + kXRing < iters) {
        cp_async16(slot, gx);
        gx += gstep_elems;
      }
      cp_async_commit();
#pragma unroll
      for (int e = 0; e < VE; ++e) {
        if constexpr (kFold) {
          fx[e] = fmaf(ag[e], fd[e], fmaf(c1[e], fx[e], c2[e]));
        } else {
          const float xh = fmaf(fx[e], L.r[e], L.nmr[e]);
          fx[e] = fmaf(ag[e], fd[e], fmaf(nb[e], xh, na[e]));
        }
      }
      stg128(gp, pack16<T, VE>(fx));
      gp += gstep_elems;
    }
  } else {
    const T* pd = reinterpret_cast<const T*>(__cvta_shared_to_generic(sd));
    T* gp = gdst;
    for (int i = 0; i < iters; ++i) {
#pragma unroll
      for (int e = 0; e < VE; ++e) {
        const float xh = fmaf(load_param<T>(gx, e), L.r[e], L.nmr[e]);
        gp[e] = store_param<T>(fmaf(ag[e], load_param<T>(pd, e), fmaf(nb[e], xh, na[e])));
      }
      gx += gstep_elems;
      pd += sstep_bytes / sizeof(T);
      gp += gstep_elems;
    }
  }
}

// Phase 2, global to global (multi-kernel path): dx = ag * dyh + (nb * xh + na) with per-lane
// ag = rstd * gamma, nb = -rstd * B, na = -rstd * A.
//   kStashed = true : `dys` holds dyh already (fused path);  false: dys holds dy, act' is recomputed.
template <typename T, int VE, int ACT, bool kStashed>
__device__ __forceinline__ void stream_bwd_dx(const Pack<T, VE>* xs, const Pack<T, VE>* dys, size_t src_stride_vec,
                                              Pack<T, VE>* __restrict__ dst, size_t dst_stride_vec, int nrows, int ty,
                                              int TY, const BwdLane<T, VE>& L, const float (&A)[VE],
                                              const float (&B)[VE]) {
  constexpr int U = 4;
  float ag[VE], nb[VE], na[VE];
#pragma unroll
  for (int e = 0; e < VE; ++e) {
    ag[e] = L.r[e] * L.ga[e];
    nb[e] = -L.r[e] * B[e];
    na[e] = -L.r[e] * A[e];
  }
  const size_t sstep = (size_t)TY * src_stride_vec, dstep = (size_t)TY * dst_stride_vec;
  const Pack<T, VE>* px = xs + (size_t)ty * src_stride_vec;
  const Pack<T, VE>* pd = dys + (size_t)ty * src_stride_vec;
  Pack<T, VE>* po = dst + (size_t)ty * dst_stride_vec;
  int left = ty < nrows ? (nrows - ty + TY - 1) / TY : 0;
  while (left > 0) {
    const int nb_rows = left < U ? left : U;
    Pack<T, VE> vx[U], vd[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (u < nb_rows) {
        vx[u] = *px;
        vd[u] = *pd;
        px += sstep;
        pd += sstep;
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (u < nb_rows) {
        float fx[VE], fd[VE];
        unpack<T, VE>(vx[u], fx);
        unpack<T, VE>(vd[u], fd);
        float xh[VE], yh[VE], gr[VE];
#pragma unroll
        for (int e = 0; e < VE; ++e) {
          xh[e] = fmaf(fx[e], L.r[e], L.nmr[e]);
          yh[e] = fmaf(xh[e], L.ga[e], L.be[e]);
        }
        if constexpr (!kStashed) act_grad_vec<T, VE, ACT>(yh, gr);
#pragma unroll
        for (int e = 0; e < VE; ++e) {
          const float dyh = kStashed ? fd[e] : fd[e] * gr[e];
          fx[e] = fmaf(ag[e], dyh, fmaf(nb[e], xh[e], na[e]));
        }
        st_stream(po, pack<T, VE>(fx));
        po += dstep;
      }
    }
    left -= nb_rows;
  }
}

// ------------------------------------------------------------------------------------------------
// fused kernel.  grid.x = N * ncb * k, cluster (k,1,1).
// dynamic smem: [dyh tile][x ring kXRing*threads*16 B][red][generic reductions only: part 2*max(threads,CW), chan 2*CW]
//               [group partials 2*slots][coef 2*slots][inbox 4*k*slots][mbarrier]
// scratch out : sums[((n * k + rank) * C + c) * 2 + {0,1}] = S1, S2 over this CTA's rows
// ------------------------------------------------------------------------------------------------
// MAXT: CTA size class.  128-thread launches are compiled for five CTAs per SM (<= 96 registers).
// SHUF: the shuffle reductions (Geom::shuf) are compiled in instead of the generic ones.
template <typename T, int VE, int ACT, bool UNI, int MAXT, bool SHUF>
__global__ void __launch_bounds__(MAXT, MAXT == 128 ? 5 : 1)
    gn_bwd_fused_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ gamma,
                        const T* __restrict__ beta, const float* __restrict__ mean_in,
                        const float* __restrict__ rstd_in, T* __restrict__ dx, float* __restrict__ sums, const Geom g) {
  extern __shared__ uint4 smem_raw[];
  using P = Pack<T, VE>;
  const unsigned k = cluster_nctarank(), rank = cluster_ctarank();
  const int item = blockIdx.x / k;  // k is a power of two
  const int n = g.div_ncb.div(item), cb = item - n * g.ncb;
  const int c0 = cb * g.CW;
  const int r0 = min((int)rank * g.rows_per_cta, g.R);
  const int nrows = min(g.rows_per_cta, g.R - r0);

  const size_t tile_bytes = ((size_t)g.rows_per_cta * g.CV * sizeof(P) + 15) & ~(size_t)15;
  const size_t ring_bytes = sizeof(P) == 16 ? (size_t)kXRing * blockDim.x * 16 : 0;
  P* tile_dy = reinterpret_cast<P*>(smem_raw);
  const uint32_t ring = smem_addr(reinterpret_cast<char*>(smem_raw) + tile_bytes) + threadIdx.x * 16;
  const uint32_t ring_stride = blockDim.x * 16;
  float* red = reinterpret_cast<float*>(reinterpret_cast<char*>(smem_raw) + tile_bytes + ring_bytes);
  constexpr bool shuf = SHUF;
  float* part = red + g.red_floats;                      // generic reductions only
  float* chan = part + 2 * max((int)blockDim.x, g.CW);  // generic reductions only
  float* spart = shuf ? part : chan + 2 * g.CW;  // generic reductions: [2*s] = sum gamma S1, [2*s+1] = sum gamma S2 of this CTA
  float* coef = spart + 2 * g.slots;             // A[s], B[slots + s]
  // inbox of the exchange: entry (q, s) = the group sums (gamma S1, gamma S2, -, -) of rank q's
  // rows, 16-byte aligned, followed by its mbarrier
  float* inbox = coef + 2 * g.slots;
  inbox += (4 - ((reinterpret_cast<uintptr_t>(inbox) >> 2) & 3)) & 3;
  uint64_t* mbar = reinterpret_cast<uint64_t*>(inbox + 4 * k * g.slots);

  const int tid = threadIdx.x;
  const int ty = g.div_CV.div(tid), tx = tid - ty * g.CV;
  const bool streaming = (ty < g.TY) && (c0 + tx * VE < g.C);
  const size_t base = ((size_t)n * g.R + r0 + ty) * g.C + c0 + (size_t)tx * VE;
  const int iters = (streaming && ty < nrows) ? (nrows - ty + g.TY - 1) / g.TY : 0;
  const uint32_t sd = smem_addr(tile_dy + ty * g.CV + tx);
  const uint32_t sstep = (uint32_t)(g.TY * g.CV * sizeof(P));
  const size_t gstep = (size_t)g.TY * g.C;

  BwdLane<T, VE> L;
  float s1[VE], s2[VE];
#pragma unroll
  for (int e = 0; e < VE; ++e) s1[e] = 0.f, s2[e] = 0.f;
  BwdPipe<T> pipe = {x + base, dy + base, sd, 0};
  if (streaming) pipe = tile_fill_start<T, VE>(x + base, dy + base, gstep, ring, ring_stride, sd, sstep, iters);
  // The inbox barrier: one arrival (thread 0, which also announces the bytes) per use, one use
  // per launch.  Every CTA of the cluster must have initialised its barrier before a peer pushes
  // to it: the cluster barrier that guarantees this is entered here and left after phase 1.
  if (tid == 0) {
    mbar_init(mbar, 1);
    fence_mbar_init_cluster();
    mbar_arrive_expect_tx(mbar, k * g.slots * 16);
  }
  cluster_arrive_relaxed();
  if (streaming) {
    lane_setup<T, VE, UNI>(gamma, beta, mean_in + (size_t)n * g.G, rstd_in + (size_t)n * g.G, c0 + tx * VE, g.div_D, L);
    tile_fill_bwd_sums<T, VE, ACT>(pipe, gstep, ring, ring_stride, sd, sstep, iters, L, s1, s2);
    // the first x rows of phase 2 (L2 hits) travel while the cluster exchanges its sums
    tile_bwd_dx_start<T, VE>(x + base, gstep, ring, ring_stride, iters);
  }

  cluster_wait();  // the peers' inbox barriers exist (every CTA arrived long ago)
  int g_lo, n_slots;
  cb_groups(g, c0, g_lo, n_slots);
  const int c_valid = min(g.CW, g.C - c0);
  if constexpr (shuf) {
    // gamma-weighted group sums straight from registers: xor-butterflies + one pass over the warps
    float a1 = 0.f, a2 = 0.f;
    if (streaming) {
#pragma unroll
      for (int e = 0; e < VE; ++e) {
        a1 = fmaf(L.ga[e], s1[e], a1);
        a2 = fmaf(L.ga[e], s2[e], a2);
      }
    }
    const float t1 = cta_slot_sum_shuf(g, a1, tx, red);
    const float t2 = cta_slot_sum_shuf(g, a2, tx, red + g.wsum_stride);
    if (tid < g.CV && (tid & ((1 << g.tps_shift) - 1)) == 0) {
      const int s = tid >> g.tps_shift;
      for (unsigned q = 0; q < k; ++q) st_async_f32x4(inbox + 4 * (rank * g.slots + s), mbar, q, t1, t2, 0.f, 0.f);
    }
  } else {
    cta_channel_sums<VE>(g, s1, s2, tx, ty, c0, red, part, chan);
    // gamma-weighted group sums of this CTA's rows: one warp per group, fixed lane order
    const int warp = tid >> 5, lane = tid & 31, nwarps = (blockDim.x + 31) >> 5;
    for (int s = warp; s < n_slots; s += nwarps) {
      const int lo = max((g_lo + s) * g.D, c0) - c0;
      const int hi = min((g_lo + s + 1) * g.D, c0 + c_valid) - c0;
      float a1 = 0.f, a2 = 0.f;
      for (int c = lo + lane; c < hi; c += 32) {
        const float ga = load_param<T>(gamma, c0 + c);
        a1 = fmaf(ga, chan[c], a1);
        a2 = fmaf(ga, chan[g.CW + c], a2);
      }
      a1 = warp_sum(a1);
      a2 = warp_sum(a2);
      if (lane == 0) {
        spart[2 * s] = a1;
        spart[2 * s + 1] = a2;
      }
    }
  }
  if constexpr (!shuf) {
    __syncthreads();
    for (int s = tid; s < g.slots; s += blockDim.x) {
      const bool live = s < n_slots;
      const float a1 = live ? spart[2 * s] : 0.f, a2 = live ? spart[2 * s + 1] : 0.f;
      for (unsigned q = 0; q < k; ++q) st_async_f32x4(inbox + 4 * (rank * g.slots + s), mbar, q, a1, a2, 0.f, 0.f);
    }
  }
  // Channel sums of this CTA's rows go to scratch (summed over samples and cluster ranks by the
  // parameter-gradient kernel).  On the shuffle path this work overlaps the wait for the peers.
  {
    float2* out = reinterpret_cast<float2*>(sums) + (((size_t)n * k + rank) * g.C + c0);
    if constexpr (shuf) {
      cta_channel_sums_shuf<VE>(g, s1, s2, tx, red + g.wpart_off, out, c_valid);
    } else {
      for (int c = tid; c < c_valid; c += blockDim.x) out[c] = make_float2(chan[c], chan[g.CW + c]);
    }
  }
  // every CTA of the cluster pushed its group sums into every inbox: no cluster barrier, no fence
  // a wait that gives up yields NaN coefficients: the failure shows in dx (the channel sums in
  // scratch, hence dgamma / dbeta, come from this CTA's own rows and stay valid)
  const bool ok = mbar_wait_bounded(mbar, 0, g.wait);
  const float inv_m = ok ? 1.0f / ((float)g.D * (float)g.R) : __int_as_float(0x7fc00000);
  for (int s = tid; s < n_slots; s += blockDim.x) {
    float a1 = 0.f, a2 = 0.f;
    for (unsigned q = 0; q < k; ++q) {
      const float4 v = *reinterpret_cast<const float4*>(inbox + 4 * (q * g.slots + s));
      a1 += v.x;
      a2 += v.y;
    }
    coef[s] = a1 * inv_m;
    coef[g.slots + s] = a2 * inv_m;
  }
  __syncthreads();

  // the parameter-gradient kernel may be placed now; it waits for this grid before it reads the sums
  grid_dep_launch_dependents();
  if (streaming) {
    float A[VE], B[VE];
    if constexpr (UNI) {
      const int s = g.div_D.div(c0 + tx * VE) - g_lo;
      const float a0 = coef[s], b0 = coef[g.slots + s];
#pragma unroll
      for (int e = 0; e < VE; ++e) A[e] = a0, B[e] = b0;
    } else {
#pragma unroll
      for (int e = 0; e < VE; ++e) {
        const int s = g.div_D.div(c0 + tx * VE + e) - g_lo;
        A[e] = coef[s];
        B[e] = coef[g.slots + s];
      }
    }
    tile_bwd_dx<T, VE>(x + base, ring, ring_stride, sd, sstep, dx + base, gstep, iters, L, A, B);
  }
  // No exit barrier: nothing reaches into this CTA's shared memory once its wait has completed.
}

// ------------------------------------------------------------------------------------------------
// parameter gradients:  dbeta_c = sum_n S1[n,c],  dgamma_c = sum_n S2[n,c]  over the N rows of `sums`
// (one per sample, or per sample and cluster rank; ascending per lane,
// then the row lanes in order).  block (32, row lanes), grid ceil(C / 32).
// ------------------------------------------------------------------------------------------------
// PEER: the exchange over the ranks is compiled in.  (Its table of peer pointers is indexed at run
// time: the descriptor is a __grid_constant__ so that it is read in place, and single-GPU launches
// take the instantiation without it - a by-value copy into every thread's local memory cost 2 us.)
// LANES row lanes: 32, or 8 for the PEER instantiation when there are few rows to add - its CTAs are
// programmatic dependents of the backward kernel, and 256 threads with the exchange's registers find room
// on an SM as soon as one CTA of that kernel has left, where 1024 threads need the SM all but empty.
template <typename T, bool PEER, int LANES>
__global__ void __launch_bounds__(32 * LANES)
    gn_bwd_param_kernel(const float* __restrict__ sums, int N, int C, float* __restrict__ dparam_f32,
                        T* __restrict__ dgamma, T* __restrict__ dbeta, const __grid_constant__ PeerExchange px) {
  constexpr int kLanes = LANES;  // row lanes: block (32 channels, kLanes row lanes)
  __shared__ float sm1[kLanes][33], sm2[kLanes][33];
  grid_dep_launch_dependents();
  PeerPush pp = {};
  if constexpr (PEER) {  // the bookkeeping of the exchange does not depend on the kernel before
    if (threadIdx.y == 0) pp = peer_push_begin(px, blockIdx.x);
  }
  grid_dep_wait();  // the sums of the kernel before
  const int c = blockIdx.x * 32 + threadIdx.x;
  float a1 = 0.f, a2 = 0.f;
  if (c < C) {
#pragma unroll 4
    for (int n = threadIdx.y; n < N; n += kLanes) {
      const float2 v = reinterpret_cast<const float2*>(sums)[(size_t)n * C + c];
      a1 += v.x;
      a2 += v.y;
    }
  }
  sm1[threadIdx.y][threadIdx.x] = a1;
  sm2[threadIdx.y][threadIdx.x] = a2;
  __syncthreads();
  if (threadIdx.y == 0) {  // one full warp: lane = channel of the block
    float t1 = 0.f, t2 = 0.f;
#pragma unroll
    for (int j = 0; j < kLanes; ++j) {
      t1 += sm1[j][threadIdx.x];
      t2 += sm2[j][threadIdx.x];
    }
    // data-parallel ranks of one node: post this rank's sums into every rank's exchange buffer and,
    // unless the caller collects later, wait for the others' and add them up in rank order
    if constexpr (PEER) {
      const bool pushed = peer_push_block(px, blockIdx.x, c < C, t2, t1, pp);
      if (px.collect) peer_collect_block<(LANES <= 8 ? 8 : 4)>(px, blockIdx.x, c < C, t2, t1);
      else if (!pushed) t1 = t2 = __int_as_float(0x7fc00000);
    }
    if (c < C) {
      dparam_f32[c] = t2;      // dgamma
      dparam_f32[C + c] = t1;  // dbeta
      if (dgamma) dgamma[c] = store_param<T>(t2);
      if (dbeta) dbeta[c] = store_param<T>(t1);
    }
  }
}

// The exchange without the sums, on a [dgamma | dbeta] buffer of this rank: block (32), grid
// ceil(C / 32).  push: post the buffer's values; collect: replace them by the sums over the ranks.
template <typename T>
__global__ void __launch_bounds__(32)
    gn_param_exchange_kernel(int C, float* __restrict__ dparam_f32, T* __restrict__ dgamma, T* __restrict__ dbeta,
                             bool push, bool collect, const __grid_constant__ PeerExchange px) {
  PeerPush pp = {};
  if (push) pp = peer_push_begin(px, blockIdx.x);
  grid_dep_wait();  // the kernel that wrote dparam_f32
  const int c = blockIdx.x * 32 + threadIdx.x;
  float dg = 0.f, db = 0.f;
  if (push && c < C) {
    dg = dparam_f32[c];
    db = dparam_f32[C + c];
  }
  bool ok = true;
  if (push) ok = peer_push_block(px, blockIdx.x, c < C, dg, db, pp);
  if (collect) peer_collect_block<8>(px, blockIdx.x, c < C, dg, db);
  if (!collect && !ok) dg = db = __int_as_float(0x7fc00000);
  if (c < C && (collect || !ok)) {
    dparam_f32[c] = dg;
    dparam_f32[C + c] = db;
    if (dgamma) dgamma[c] = store_param<T>(dg);
    if (dbeta) dbeta[c] = store_param<T>(db);
  }
}

// ------------------------------------------------------------------------------------------------
// two-pass, kernel 1: per-tile channel sums.  grid.x = N * chunks * ncb.
// scratch: tpart[((n * chunks + chunk) * C + c) * 2 + {0,1}]
// ------------------------------------------------------------------------------------------------
template <typename T, int VE, int ACT, bool UNI>
__global__ void __launch_bounds__(kMaxThreads)
    gn_bwd_reduce_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ gamma,
                         const T* __restrict__ beta, const float* __restrict__ mean_in,
                         const float* __restrict__ rstd_in, float* __restrict__ tpart, const Geom g) {
  extern __shared__ uint4 smem_raw[];
  using P = Pack<T, VE>;
  // [ring x][ring dy] (kRingDepth * blockDim vectors each) [red][part][chan]
  const size_t ring_bytes = sizeof(T) * VE == 16 ? (size_t)kRingDepth * blockDim.x * 16 : 0;
  float* red = reinterpret_cast<float*>(reinterpret_cast<char*>(smem_raw) + 2 * ring_bytes);
  float* part = red + g.red_floats;
  float* chan = part + 2 * max((int)blockDim.x, g.CW);
  grid_dep_launch_dependents();  // the kernels after this one wait for this grid before they read its sums
  const int tile_id = blockIdx.x;
  const int t1 = g.div_ncb.div(tile_id), cb = tile_id - t1 * g.ncb;
  const int n = g.div_chunks.div(t1), chunk = t1 - n * g.chunks;
  const int c0 = cb * g.CW;
  const int r0 = chunk * g.rows_per_cta;
  const int nrows = min(g.rows_per_cta, g.R - r0);
  const int tid = threadIdx.x;
  const int ty = g.div_CV.div(tid), tx = tid - ty * g.CV;
  const bool streaming = (ty < g.TY) && (c0 + tx * VE < g.C);
  const size_t base = ((size_t)n * g.R + r0 + ty) * g.C + c0 + (size_t)tx * VE;
  const int iters = (streaming && ty < nrows) ? (nrows - ty + g.TY - 1) / g.TY : 0;

  BwdLane<T, VE> L;
  float s1[VE], s2[VE];
#pragma unroll
  for (int e = 0; e < VE; ++e) s1[e] = 0.f, s2[e] = 0.f;
  if (streaming) {
    lane_setup<T, VE, UNI>(gamma, beta, mean_in + (size_t)n * g.G, rstd_in + (size_t)n * g.G, c0 + tx * VE, g.div_D, L);
    const uint32_t ring = smem_addr(smem_raw) + tid * 16;
    stream_bwd_sums<T, VE, ACT>(x + base, dy + base, (size_t)g.TY * g.C, iters, ring, ring + (uint32_t)ring_bytes,
                                blockDim.x * 16, L, s1, s2);
  }
  cta_channel_sums<VE>(g, s1, s2, tx, ty, c0, red, part, chan);
  const int c_valid = min(g.CW, g.C - c0);
  float2* out = reinterpret_cast<float2*>(tpart) + ((size_t)n * g.chunks + chunk) * g.C + c0;
  for (int c = tid; c < c_valid; c += blockDim.x) out[c] = make_float2(chan[c], chan[g.CW + c]);
}

// two-pass, kernel 2: one CTA of 256 threads per (n, group).  The group's channels are taken in
// blocks of W (a power of two <= 32 covering D); thread t owns channel t % W of the block and the
// tiles t / W, t / W + 256 / W, ... (fixed); the lanes of a warp that hold the same channel are combined
// by an xor butterfly and the eight warps in warp order.  Writes S1, S2 per channel of the sample and
// the group's A, B.
template <typename T>
__global__ void __launch_bounds__(256)
    gn_bwd_finalize_kernel(const float* __restrict__ tpart, const T* __restrict__ gamma, float* __restrict__ sums,
                           float* __restrict__ coef, const Geom g) {
  __shared__ float sm1[8][32], sm2[8][32];
  __shared__ float scratch[8];
  grid_dep_launch_dependents();
  grid_dep_wait();  // the reduce kernel's channel sums
  const int n = blockIdx.x / g.G, grp = blockIdx.x - n * g.G;
  int sh = 0;
  while ((1 << sh) < g.D && sh < 5) ++sh;
  const int W = 1 << sh, J = 256 >> sh;
  const int lx = threadIdx.x & (W - 1), ly = threadIdx.x >> sh;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float w1 = 0.f, w2 = 0.f;  // gamma-weighted sums held by the first W threads
  for (int cbase = 0; cbase < g.D; cbase += W) {
    const int cin = cbase + lx;
    const bool valid = cin < g.D;
    const int c = grp * g.D + cin;
    float a1 = 0.f, a2 = 0.f;
    if (valid) {
#pragma unroll 8
      for (int chunk = ly; chunk < g.chunks; chunk += J) {
        const float2 v = reinterpret_cast<const float2*>(tpart)[((size_t)n * g.chunks + chunk) * g.C + c];
        a1 += v.x;
        a2 += v.y;
      }
    }
    // lanes of a warp that hold the same channel (equal lane mod W), then the eight warps in order
    for (int b = W; b < 32; b <<= 1) {
      a1 += __shfl_xor_sync(0xffffffffu, a1, b);
      a2 += __shfl_xor_sync(0xffffffffu, a2, b);
    }
    if (lane < W) {
      sm1[warp][lane] = a1;
      sm2[warp][lane] = a2;
    }
    __syncthreads();
    if (threadIdx.x < W && valid) {
      float t1 = 0.f, t2 = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) {
        t1 += sm1[w][threadIdx.x];
        t2 += sm2[w][threadIdx.x];
      }
      reinterpret_cast<float2*>(sums)[(size_t)n * g.C + c] = make_float2(t1, t2);
      const float ga = load_param<T>(gamma, c);
      w1 = fmaf(ga, t1, w1);
      w2 = fmaf(ga, t2, w2);
    }
    __syncthreads();
  }
  w1 = block_sum(w1, scratch);
  w2 = block_sum(w2, scratch);
  if (threadIdx.x == 0) {
    const float inv_m = 1.0f / ((float)g.D * (float)g.R);
    coef[((size_t)n * g.G + grp) * 2] = w1 * inv_m;
    coef[((size_t)n * g.G + grp) * 2 + 1] = w2 * inv_m;
  }
}

// two-pass, kernel 4: dx.  Reverse tile order relative to the reduce kernel.
template <typename T, int VE, int ACT, bool UNI>
__global__ void __launch_bounds__(kMaxThreads)
    gn_bwd_apply_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ gamma,
                        const T* __restrict__ beta, const float* __restrict__ mean_in,
                        const float* __restrict__ rstd_in, const float* __restrict__ coef, T* __restrict__ dx,
                        const Geom g) {
  using P = Pack<T, VE>;
  const int tile_id = gridDim.x - 1 - blockIdx.x;
  const int t1 = g.div_ncb.div(tile_id), cb = tile_id - t1 * g.ncb;
  const int n = g.div_chunks.div(t1), chunk = t1 - n * g.chunks;
  const int c0 = cb * g.CW;
  const int r0 = chunk * g.rows_per_cta;
  const int nrows = min(g.rows_per_cta, g.R - r0);
  const int tid = threadIdx.x;
  const int ty = g.div_CV.div(tid), tx = tid - ty * g.CV;
  if (ty >= g.TY || c0 + tx * VE >= g.C) return;
  BwdLane<T, VE> L;
  lane_setup<T, VE, UNI>(gamma, beta, mean_in + (size_t)n * g.G, rstd_in + (size_t)n * g.G, c0 + tx * VE, g.div_D, L);
  grid_dep_wait();  // the finalize kernel's coefficients (the parameters above are the caller's)
  float A[VE], B[VE];
  if constexpr (UNI) {
    const int grp = g.div_D.div(c0 + tx * VE);
    const float a0 = coef[((size_t)n * g.G + grp) * 2], b0 = coef[((size_t)n * g.G + grp) * 2 + 1];
#pragma unroll
    for (int e = 0; e < VE; ++e) A[e] = a0, B[e] = b0;
  } else {
#pragma unroll
    for (int e = 0; e < VE; ++e) {
      const int grp = g.div_D.div(c0 + tx * VE + e);
      A[e] = coef[((size_t)n * g.G + grp) * 2];
      B[e] = coef[((size_t)n * g.G + grp) * 2 + 1];
    }
  }
  const size_t base = ((size_t)n * g.R + r0) * g.C + c0 + (size_t)tx * VE;
  const size_t rs = (size_t)g.C / VE;
  stream_bwd_dx<T, VE, ACT, false>(reinterpret_cast<const P*>(x + base), reinterpret_cast<const P*>(dy + base), rs,
                                   reinterpret_cast<P*>(dx + base), rs, nrows, ty, g.TY, L, A, B);
}

// ------------------------------------------------------------------------------------------------
// host-side launchers
// ------------------------------------------------------------------------------------------------
template <typename T>
static cudaError_t launch_param(const BwdCall& c, const float* sums, int rows, const Geom& g, cudaStream_t stream,
                                bool chained) {
  const dim3 block(32, 32, 1);
  const unsigned blocks = (unsigned)((g.C + 31) / 32);
  if (c.peer && c.peer->world > 1) {
    // (the order in which the samples' sums are added depends on the lane count, which depends only on the
    // row count: the ranks of a group have equal batches, so every rank adds in the same order)
    const char* forced = getenv("GNB200_PEER_LANES");  // experiments: 8 or 32
    const int few = forced && *forced ? atoi(forced) : (rows < 128 ? 8 : 32);
    if (few == 8)
      return launch_chained(gn_bwd_param_kernel<T, true, 8>, blocks, dim3(32, 8, 1), 0, stream, chained, sums, rows, g.C,
                            c.dparam_f32, (T*)c.dgamma, (T*)c.dbeta, *c.peer);
    return launch_chained(gn_bwd_param_kernel<T, true, 32>, blocks, block, 0, stream, chained, sums, rows, g.C, c.dparam_f32,
                          (T*)c.dgamma, (T*)c.dbeta, *c.peer);
  }
  return launch_chained(gn_bwd_param_kernel<T, false, 32>, blocks, block, 0, stream, chained, sums, rows, g.C, c.dparam_f32,
                        (T*)c.dgamma, (T*)c.dbeta, PeerExchange{});
}

template <typename T>
static cudaError_t launch_exchange(const BwdCall& c, int C, cudaStream_t stream, bool chained, bool push, bool collect) {
  return launch_chained(gn_param_exchange_kernel<T>, (unsigned)((C + 31) / 32), dim3(32), 0, stream, chained, C,
                        c.dparam_f32, (T*)c.dgamma, (T*)c.dbeta, push, collect, *c.peer);
}

template <typename T, int VE, int ACT, bool UNI>
static cudaError_t launch_bwd_u(const BwdCall& c, const Plan& p, cudaStream_t stream) {
  Geom g = p.geom;
  if (p.fused) {
    float* sums = reinterpret_cast<float*>(c.workspace);
    cudaError_t werr = wait_limit_for_device(&g.wait);
    if (werr != cudaSuccess) return werr;
    g.skip_push_rank = -1;
    constexpr bool kCanShuf = UNI && VE >= 4;
    auto kern = p.threads <= 128 ? gn_bwd_fused_kernel<T, VE, ACT, UNI, 128, false>
                                 : gn_bwd_fused_kernel<T, VE, ACT, UNI, kMaxThreads, false>;
    if constexpr (kCanShuf) {
      if (g.shuf)
        kern = p.threads <= 128 ? gn_bwd_fused_kernel<T, VE, ACT, UNI, 128, true>
                                : gn_bwd_fused_kernel<T, VE, ACT, UNI, kMaxThreads, true>;
    }
    cudaError_t err = ensure_kernel_attributes((const void*)kern, p.smem_bytes, g.k > 8);
    if (err != cudaSuccess) return err;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)p.grid, 1, 1);
    cfg.blockDim = dim3((unsigned)p.threads, 1, 1);
    cfg.dynamicSmemBytes = p.smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)g.k;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    err = cudaLaunchKernelEx(&cfg, kern, (const T*)c.dy, (const T*)c.x, (const T*)c.gamma, (const T*)c.beta, c.mean,
                             c.rstd, (T*)c.dx, sums, g);
    if (err != cudaSuccess) return err;
    return launch_param<T>(c, sums, g.N * g.k, g, stream, p.chain);
  }
  // two-pass scratch: [tile partials N*chunks*C*2][sums N*C*2][coef N*G*2]
  float* tpart = reinterpret_cast<float*>(c.workspace);
  float* sums = tpart + (size_t)g.N * g.chunks * g.C * 2;
  float* coef = sums + (size_t)g.N * g.C * 2;
  cudaError_t err = ensure_kernel_attributes((const void*)gn_bwd_reduce_kernel<T, VE, ACT, UNI>, p.smem_bytes, false);
  if (err != cudaSuccess) return err;
  gn_bwd_reduce_kernel<T, VE, ACT, UNI><<<(unsigned)p.grid, p.threads, p.smem_bytes, stream>>>(
      (const T*)c.dy, (const T*)c.x, (const T*)c.gamma, (const T*)c.beta, c.mean, c.rstd, tpart, g);
  err = cudaGetLastError();
  if (err != cudaSuccess) return err;
  err = launch_chained(gn_bwd_finalize_kernel<T>, (unsigned)(g.N * g.G), dim3(256), 0, stream, p.chain, tpart,
                       (const T*)c.gamma, sums, coef, g);
  if (err != cudaSuccess) return err;
  err = launch_param<T>(c, sums, g.N, g, stream, p.chain);
  if (err != cudaSuccess) return err;
  return launch_chained(gn_bwd_apply_kernel<T, VE, ACT, UNI>, (unsigned)p.grid, dim3((unsigned)p.threads), 0, stream, p.chain,
                        (const T*)c.dy, (const T*)c.x, (const T*)c.gamma, (const T*)c.beta, c.mean, c.rstd, coef, (T*)c.dx, g);
}

template <typename T, int VE, int ACT>
static cudaError_t launch_bwd_t(const BwdCall& c, const Plan& p, cudaStream_t stream) {
  const bool uni = VE == 1 || p.geom.D % VE == 0;
  if (uni) return launch_bwd_u<T, VE, ACT, true>(c, p, stream);
  if constexpr (VE > 1) return launch_bwd_u<T, VE, ACT, false>(c, p, stream);
  return cudaErrorInvalidValue;
}

template <typename T, int VE>
static cudaError_t launch_bwd_act(const BwdCall& c, const Plan& p, cudaStream_t stream) {
  switch (c.act) {
    case kActIdentity: return launch_bwd_t<T, VE, kActIdentity>(c, p, stream);
    case kActRelu: return launch_bwd_t<T, VE, kActRelu>(c, p, stream);
    case kActSilu: return launch_bwd_t<T, VE, kActSilu>(c, p, stream);
    case kActGelu: return launch_bwd_t<T, VE, kActGelu>(c, p, stream);
    default: return launch_bwd_t<T, VE, kActGeluTanh>(c, p, stream);
  }
}

template <typename T>
static cudaError_t launch_bwd_ve(const BwdCall& c, const Plan& p, cudaStream_t stream) {
  constexpr int VFULL = 16 / sizeof(T);
  return p.ve == 1 ? launch_bwd_act<T, 1>(c, p, stream) : launch_bwd_act<T, VFULL>(c, p, stream);
}

cudaError_t launch_param_grads(const BwdCall& c, const float* sums, int rows, int C, cudaStream_t stream, bool chained) {
  Geom g = {};
  g.C = C;
  switch (c.dtype) {
    case 0: return launch_param<float>(c, sums, rows, g, stream, chained);
    case 1: return launch_param<__half>(c, sums, rows, g, stream, chained);
    default: return launch_param<__nv_bfloat16>(c, sums, rows, g, stream, chained);
  }
}

cudaError_t launch_param_exchange(const BwdCall& c, int C, cudaStream_t stream, bool chained, bool push, bool collect) {
  if (!c.peer || c.peer->world <= 1) return cudaSuccess;
  switch (c.dtype) {
    case 0: return launch_exchange<float>(c, C, stream, chained, push, collect);
    case 1: return launch_exchange<__half>(c, C, stream, chained, push, collect);
    default: return launch_exchange<__nv_bfloat16>(c, C, stream, chained, push, collect);
  }
}

cudaError_t launch_backward(const BwdCall& c, const Plan& p, cudaStream_t stream) {
  if (p.wave) {
    // the wave kernel finishes dgamma / dbeta itself; the exchange over the ranks follows it
    const cudaError_t err = launch_backward_wave(c, p, stream);
    if (err != cudaSuccess) return err;
    return launch_param_exchange(c, p.wgeom.C, stream, false, true, c.peer && c.peer->collect);
  }
  switch (c.dtype) {
    case 0: return launch_bwd_ve<float>(c, p, stream);
    case 1: return launch_bwd_ve<__half>(c, p, stream);
    default: return launch_bwd_ve<__nv_bfloat16>(c, p, stream);
  }
}

}  // namespace gnb200
