// Forward GroupNorm (+activation) kernels for NHWC tensors, sm_100a.
//
// Two launch plans (chosen by the host planner in gn_plan.cu):
//
//  fused   one launch of persistent thread-block clusters.  A cluster of k CTAs works through
//          (sample, column block) slabs; each CTA copies its rows from HBM once (16-byte cp.async
//          along C) into shared memory while accumulating moments, the k partial moments are
//          pushed into the peers' shared memory (st.async + mbarrier), and the tile is normalised,
//          scaled, shifted, activated and written from shared memory while its slots are refilled
//          with the rows of the cluster's next slab.  HBM traffic: one read + one write of the tensor.
//
//  two-pass  for slabs that do not fit a cluster's shared memory: stats kernel (partial moments
//          per CTA to scratch) -> finalize kernel (fixed-order merge -> mean, rstd) -> apply
//          kernel, which walks the tensor in the opposite order so the part of x read last is
//          re-read from L2.
//
// The reference computes the same quantities with compute_stats_pt1 / compute_stats_pt2 /
// scale_shift_kernel (src/gnnhwc/csrc/gn_kernel.cu:132-224, 226-292, 305-412).
#include "gn_kernels.h"
#include "gn_math.cuh"

namespace gnb200 {

constexpr int kRingDepth = 4;  // rows in flight per thread in the multi-kernel streaming kernels

// Per-thread running moments over the rows this thread owns (rows ty, ty + TY, ...) in the
// multi-kernel path.  16-byte vectors go through a shared-memory ring with cp.async: kRingDepth
// rows per thread are in flight without holding registers; slot s of the thread lives at
// ring + s * ring_stride.  Other vector widths use plain loads.
template <typename T, int VE, bool UNI>
__device__ __forceinline__ void stream_moments(const T* __restrict__ gsrc, size_t gstep_elems, int iters,
                                               uint32_t ring, uint32_t ring_stride, float (&mean)[VE],
                                               float (&m2)[VE], float& cnt) {
  if constexpr (sizeof(T) * VE == 16) {
    const T* gp = gsrc;
#pragma unroll
    for (int d = 0; d < kRingDepth; ++d) {
      if (d < iters) {
        cp_async16(ring + d * ring_stride, gp);
        gp += gstep_elems;
      }
      cp_async_commit();
    }
    constexpr bool kShifted = sizeof(T) == 2;
    constexpr int KN = UNI ? 1 : VE;
    float K[KN];
    if constexpr (kShifted) {
      cp_async_wait<kRingDepth - 1>();  // row 0 has landed; its values are the shift
#pragma unroll
      for (int e = 0; e < KN; ++e) K[e] = 0.f;
      if (iters > 0) {
        float f0[VE];
        unpack16<T, VE>(lds128(ring), f0);
#pragma unroll
        for (int e = 0; e < KN; ++e) K[e] = f0[e];
      }
    }
    for (int i = 0; i < iters; ++i) {
      cp_async_wait<kRingDepth - 1>();
      const uint32_t slot = ring + (i & (kRingDepth - 1)) * ring_stride;
      const uint4 w = lds128(slot);
      if (i + kRingDepth < iters) {
        cp_async16(slot, gp);
        gp += gstep_elems;
      }
      cp_async_commit();
      if constexpr (kShifted) {
        shifted_step<T, VE, KN>(w, K, mean, m2);
      } else {
        float f[VE];
        unpack16<T, VE>(w, f);
        welford_step<VE>(f, mean, m2, cnt);
      }
    }
    if constexpr (kShifted) shifted_finish<VE, KN>(K, iters, mean, m2, cnt);
  } else {
    const T* gp = gsrc;
    for (int i = 0; i < iters; ++i) {
      float f[VE];
#pragma unroll
      for (int e = 0; e < VE; ++e) f[e] = load_param<T>(gp, e);
      gp += gstep_elems;
      welford_step<VE>(f, mean, m2, cnt);
    }
  }
}

constexpr int kFirstRows = 8;  // rows per thread copied ahead at the start of a CTA's first item

// Fused path: `iters` of the thread's rows (ty, ty + TY, ...) of its column vector are copied into
// the shared-memory tile with cp.async, one commit group per row.
// Every thread reads back only what it copied itself, so no block barrier is needed.
template <typename T, int VE>
__device__ __forceinline__ void tile_issue(const T* __restrict__ gsrc, size_t gstep_elems, uint32_t stile,
                                           uint32_t sstep_bytes, int iters) {
  if constexpr (sizeof(T) * VE == 16) {
#pragma unroll 4
    for (int i = 0; i < iters; ++i) {
      cp_async16(stile, gsrc);
      cp_async_commit();
      stile += sstep_bytes;
      gsrc += gstep_elems;
    }
  } else {
    T* sp = reinterpret_cast<T*>(__cvta_shared_to_generic(stile));
    for (int i = 0; i < iters; ++i) {
#pragma unroll
      for (int e = 0; e < VE; ++e) sp[e] = gsrc[e];
      gsrc += gstep_elems;
      sp += sstep_bytes / sizeof(T);
    }
  }
}

// Fused path, phase 1: moments of the thread's rows in the tile, consumed as they land.  The rows
// were copied by cp.async, one commit group per row in row order, and on entry no younger group of
// the thread is in flight: row j may be read once at most iters - 1 - j groups are pending.
// `feed`: only the first kLag rows have been issued so far (a CTA's first item); the others are
// issued here, one per consumed row, from gfeed (row kLag of the thread) onwards - copying every
// row at once at kernel start, when all CTAs do the same, floods the memory system.
template <typename T, int VE, bool UNI>
__device__ __forceinline__ void tile_moments(uint32_t stile, uint32_t sstep_bytes, int iters, float (&mean)[VE],
                                             float (&m2)[VE], float& cnt, bool feed, const T* __restrict__ gfeed,
                                             size_t gstep_elems) {
  if constexpr (sizeof(T) * VE == 16) {
    constexpr int kLag = kFirstRows;  // rows that may be in flight behind the one being consumed
    constexpr bool kShifted = sizeof(T) == 2;
    constexpr int KN = UNI ? 1 : VE;
    float K[KN];
    uint32_t rp = stile;
    auto consume = [&]() {
      const uint4 w = lds128(rp);
      rp += sstep_bytes;
      if constexpr (kShifted) {
        shifted_step<T, VE, KN>(w, K, mean, m2);
      } else {
        float f[VE];
        unpack16<T, VE>(w, f);
        welford_step<VE>(f, mean, m2, cnt);
      }
    };
    if constexpr (kShifted) {  // the shift: the values of row 0
#pragma unroll
      for (int e = 0; e < KN; ++e) K[e] = 0.f;
      if (iters > 0) {
        cp_async_wait_dyn8(min(iters, kLag) - 1);
        float f0[VE];
        unpack16<T, VE>(lds128(stile), f0);
#pragma unroll
        for (int e = 0; e < KN; ++e) K[e] = f0[e];
      }
    }
    int i = 0;
    uint32_t wp = stile + kLag * sstep_bytes;
#pragma unroll 2
    for (; i < iters - kLag; ++i) {
      cp_async_wait<kLag - 1>();
      consume();
      if (feed) {
        cp_async16(wp, gfeed);
        cp_async_commit();
        wp += sstep_bytes;
        gfeed += gstep_elems;
      }
    }
    const int rem = iters - i;  // <= kLag rows left: row (iters - 1 - t) needs at most t pending groups
#define GNB200_TAIL_ROW(t) \
  if (rem > t) {           \
    cp_async_wait<t>();    \
    consume();             \
  }
    GNB200_TAIL_ROW(7)
    GNB200_TAIL_ROW(6)
    GNB200_TAIL_ROW(5)
    GNB200_TAIL_ROW(4)
    GNB200_TAIL_ROW(3)
    GNB200_TAIL_ROW(2)
    GNB200_TAIL_ROW(1)
    GNB200_TAIL_ROW(0)
#undef GNB200_TAIL_ROW
    static_assert(kLag == 8, "the tail above is written out for eight rows");
    if constexpr (kShifted) shifted_finish<VE, KN>(K, iters, mean, m2, cnt);
  } else {
    const T* sp = reinterpret_cast<const T*>(__cvta_shared_to_generic(stile));
    for (int i = 0; i < iters; ++i) {
      float f[VE];
#pragma unroll
      for (int e = 0; e < VE; ++e) f[e] = load_param<T>(sp, e);
      sp += sstep_bytes / sizeof(T);
      welford_step<VE>(f, mean, m2, cnt);
    }
  }
}

// Fused path, phase 2: y = act(x * a + b) from the tile to global memory.  With `refill` set, each
// tile slot is refilled with the same row of the cluster's next item (`gnext`) as soon as it has
// been read - one cp.async commit group per row - so the next item streams in while this one
// streams out and the tile never sits half empty.
template <typename T, int VE, int ACT>
__device__ __forceinline__ void tile_apply(uint32_t stile, uint32_t sstep_bytes, T* __restrict__ gdst,
                                           size_t gstep_elems, int iters, const float (&a)[VE], const float (&b)[VE],
                                           bool refill, const T* __restrict__ gnext) {
  constexpr bool FAST = sizeof(T) == 2;
  if constexpr (sizeof(T) * VE == 16) {
    uint32_t sp = stile;
    T* gp = gdst;
#pragma unroll 2
    for (int i = 0; i < iters; ++i) {
      float f[VE];
      unpack16<T, VE>(lds128(sp), f);
      if (refill) {
        cp_async16(sp, gnext);
        cp_async_commit();
        gnext += gstep_elems;
      }
      sp += sstep_bytes;
#pragma unroll
      for (int e = 0; e < VE; ++e) f[e] = fmaf(f[e], a[e], b[e]);
      stg128(gp, act_pack16<T, VE, ACT>(f));
      gp += gstep_elems;
    }
  } else {
    T* sp = reinterpret_cast<T*>(__cvta_shared_to_generic(stile));
    T* gp = gdst;
    for (int i = 0; i < iters; ++i) {
#pragma unroll
      for (int e = 0; e < VE; ++e) {
        gp[e] = store_param<T>(act_fwd<ACT, FAST>(fmaf(load_param<T>(sp, e), a[e], b[e])));
        if (refill) sp[e] = gnext[e];
      }
      if (refill) gnext += gstep_elems;
      sp += sstep_bytes / sizeof(T);
      gp += gstep_elems;
    }
  }
}

// y = act(x * a + b) over the rows this thread owns, global to global (multi-kernel path).
template <typename T, int VE, int ACT>
__device__ __forceinline__ void stream_apply(const Pack<T, VE>* __restrict__ src, size_t src_stride_vec,
                                             Pack<T, VE>* __restrict__ dst, size_t dst_stride_vec, int nrows, int ty,
                                             int TY, const float (&a)[VE], const float (&b)[VE]) {
  constexpr bool FAST = sizeof(T) == 2;
  constexpr int U = 4;
  const size_t sstep = (size_t)TY * src_stride_vec, dstep = (size_t)TY * dst_stride_vec;
  const Pack<T, VE>* sp = src + (size_t)ty * src_stride_vec;
  Pack<T, VE>* dp = dst + (size_t)ty * dst_stride_vec;
  int left = ty < nrows ? (nrows - ty + TY - 1) / TY : 0;
  for (; left >= U; left -= U) {
    Pack<T, VE> v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      v[u] = ld_stream(sp);
      sp += sstep;
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      float f[VE];
      unpack<T, VE>(v[u], f);
      if constexpr (sizeof(T) * VE == 16) {
#pragma unroll
        for (int e = 0; e < VE; ++e) f[e] = fmaf(f[e], a[e], b[e]);
        stg128(dp, act_pack16<T, VE, ACT>(f));
      } else {
#pragma unroll
        for (int e = 0; e < VE; ++e) f[e] = act_fwd<ACT, FAST>(fmaf(f[e], a[e], b[e]));
        st_stream(dp, pack<T, VE>(f));
      }
      dp += dstep;
    }
  }
  for (; left > 0; --left) {
    float f[VE];
    unpack<T, VE>(ld_stream(sp), f);
    sp += sstep;
#pragma unroll
    for (int e = 0; e < VE; ++e) f[e] = act_fwd<ACT, FAST>(fmaf(f[e], a[e], b[e]));
    st_stream(dp, pack<T, VE>(f));
    dp += dstep;
  }
}

// CTA-local moments of every group slot of the column block from the per-thread Welford states:
// first the slot means (sum of cnt * mean / n), then the squared deviations around them.
//   slot[s]            = local mean      slot[slots + s] = local M2      slot[2 * slots + s] = local count
// scratch: red (TY * CW floats), tmp (slots floats).
template <int VE, bool UNI>
__device__ __forceinline__ void cta_slot_moments(const Geom& g, const float (&mean)[VE], const float (&m2)[VE],
                                                 float cnt, int tx, int ty, int c0, int nrows, int g_lo, int n_slots,
                                                 float* red, float* tmp, float* slot) {
  constexpr int NV = UNI ? 1 : VE;
  float val[NV];
  if constexpr (UNI) {
    float sm = 0.f;
#pragma unroll
    for (int e = 0; e < VE; ++e) sm += mean[e];
    val[0] = cnt * sm;
  } else {
#pragma unroll
    for (int e = 0; e < VE; ++e) val[e] = cnt * mean[e];
  }
  cta_group_sum<VE, NV>(g, val, tx, ty, c0, g_lo, n_slots, red, tmp);
  const int c_end = min(c0 + g.CW, g.C);
  for (int s = threadIdx.x; s < n_slots; s += blockDim.x) {
    const int w = min((g_lo + s + 1) * g.D, c_end) - max((g_lo + s) * g.D, c0);
    const float n_loc = (float)nrows * (float)w;
    slot[s] = n_loc > 0.f ? tmp[s] / n_loc : 0.f;
    slot[2 * g.slots + s] = n_loc;
  }
  __syncthreads();
  if constexpr (UNI) {
    const float lm = slot[g.div_D.div(min(c0 + tx * VE, g.C - 1)) - g_lo];
    float acc = 0.f, dev = 0.f;
#pragma unroll
    for (int e = 0; e < VE; ++e) {
      const float d = mean[e] - lm;
      dev = fmaf(d, d, dev);
      acc += m2[e];
    }
    val[0] = fmaf(cnt, dev, acc);
  } else {
#pragma unroll
    for (int e = 0; e < VE; ++e) {
      const int c = min(c0 + tx * VE + e, g.C - 1);
      const float d = mean[e] - slot[g.div_D.div(c) - g_lo];
      val[e] = fmaf(cnt * d, d, m2[e]);
    }
  }
  cta_group_sum<VE, NV>(g, val, tx, ty, c0, g_lo, n_slots, red, slot + g.slots);
}

// ------------------------------------------------------------------------------------------------
// fused one-pass kernel.  cluster = (k,1,1); an item is one (sample, column block) slab and each
// CTA of the cluster owns rows_per_cta of its rows.  The grid holds the clusters that are resident
// at once (or one per item if there are fewer items); cluster c works on items c, c + n_clusters,
// ...  While a CTA writes the y rows of one item it refills the tile, row by row, with the x rows
// of its next item, so DRAM reads and writes overlap and the exchange of statistics of one item
// is the only time a CTA does not move data.  The exchange itself needs no cluster barrier: every
// CTA pushes its (mean, M2, count) into the inboxes of all CTAs of the cluster (st.async) and
// waits on its own mbarrier for the k contributions; inboxes alternate between two copies, and a
// copy is pushed to again only by peers that have seen this CTA's contribution to the next item.
// dynamic smem: [tile rows_per_cta * CV packs][red][tmp slots][slot 3*slots][stat 2*slots]
//               [2 inboxes of k*slots entries of 4 floats][2 mbarriers][dead flag]
// ------------------------------------------------------------------------------------------------
// MAXT: CTA size class.  128-thread launches are compiled for six CTAs per SM (<= 80 registers).
template <typename T, int VE, int ACT, bool UNI, int MAXT>
__global__ void __launch_bounds__(MAXT, MAXT == 128 ? 6 : 2)
    gn_fwd_fused_kernel(const T* __restrict__ x, const T* __restrict__ gamma, const T* __restrict__ beta,
                        T* __restrict__ y, float* __restrict__ mean_out, float* __restrict__ rstd_out, float eps,
                        const Geom g) {
  extern __shared__ uint4 smem_raw[];
  using P = Pack<T, VE>;
  constexpr bool kVec = sizeof(T) * VE == 16;
  const unsigned k = cluster_nctarank(), rank = cluster_ctarank();
  const int n_items = g.N * g.ncb;
  const int n_clusters = (int)(gridDim.x / k);  // k is a power of two
  const int r0 = min((int)rank * g.rows_per_cta, g.R);
  const int nrows = min(g.rows_per_cta, g.R - r0);

  const size_t tile_bytes = ((size_t)g.rows_per_cta * g.CV * sizeof(P) + 15) & ~(size_t)15;
  float* red = reinterpret_cast<float*>(reinterpret_cast<char*>(smem_raw) + tile_bytes);
  float* tmp = red + g.red_floats;
  float* slot = tmp + g.slots;       // generic reductions: local mean | local M2 | local count
  float* stat = slot + 3 * g.slots;  // mean[slots], rstd[slots]
  // push exchange: two inboxes of k * slots entries (mean, M2, count, -), 16-byte aligned, and
  // their mbarriers
  float* inbox2 = stat + 2 * g.slots;
  inbox2 += (4 - ((reinterpret_cast<uintptr_t>(inbox2) >> 2) & 3)) & 3;
  uint64_t* mbar2 = reinterpret_cast<uint64_t*>(inbox2 + 2 * 4 * k * g.slots);

  const int tid = threadIdx.x;
  const int ty = g.div_CV.div(tid), tx = tid - ty * g.CV;
  // the fused plans use column blocks that divide C, so a thread's column is valid for every item
  const bool streaming = (ty < g.TY) && (tx * VE < g.CW);
  const int iters = (streaming && ty < nrows) ? (nrows - ty + g.TY - 1) / g.TY : 0;
  const uint32_t stile = smem_addr(reinterpret_cast<P*>(smem_raw) + ty * g.CV + tx);
  const uint32_t sstep = (uint32_t)(g.TY * g.CV * sizeof(P));
  const size_t gstep = (size_t)g.TY * g.C;
  const size_t row_off = ((size_t)r0 + ty) * g.C + (size_t)tx * VE;

  // Inbox barriers: one arrival (thread 0, which also announces the bytes) per use.  Every CTA of
  // the cluster must have initialised them before a peer pushes to them: the cluster barrier that
  // guarantees this is entered here and left just before this CTA's first push.
  // Set by thread 0 when its wait for an exchange gave up.  From then on the CTA is `dead`: it
  // keeps pushing its contributions (its peers' waits must end) but no longer arrives or waits on
  // its own barriers, whose phase may never complete - arriving again on such a barrier is
  // undefined - and it writes NaN statistics, so every output of its remaining items is NaN.
  volatile unsigned int& s_dead = *reinterpret_cast<volatile unsigned int*>(mbar2 + 2);
  if (threadIdx.x == 0) {
    s_dead = 0;
    mbar_init(mbar2, 1);
    mbar_init(mbar2 + 1, 1);
    fence_mbar_init_cluster();
  }
  cluster_arrive_relaxed();
  int item = (int)(blockIdx.x / k);
  unsigned parity = 0, uses = 0;
  if (item < n_items) {
    const int n = g.div_ncb.div(item), cb = item - n * g.ncb;
    tile_issue<T, VE>(x + (size_t)n * g.R * g.C + cb * g.CW + row_off, gstep, stile, sstep,
                      kVec ? min(iters, kFirstRows) : iters);
  }
  bool first = true;
  for (; item < n_items; item += n_clusters, parity ^= 1u) {
    const int n = g.div_ncb.div(item), cb = item - n * g.ncb;
    const int c0 = cb * g.CW;
    const size_t base = (size_t)n * g.R * g.C + c0 + row_off;
    uint4 ga_raw = make_uint4(0, 0, 0, 0), be_raw = make_uint4(0, 0, 0, 0);
    if constexpr (kVec) {
      if (streaming) {
        ga_raw = *reinterpret_cast<const uint4*>(gamma + c0 + tx * VE);
        be_raw = *reinterpret_cast<const uint4*>(beta + c0 + tx * VE);
      }
    }
    float* inbox = inbox2 + parity * 4 * k * g.slots;
    uint64_t* mbar = mbar2 + parity;
    // (thread 0 stored s_dead before the block barrier that ends the previous item)
    const bool dead = !first && s_dead != 0;
    if (tid == 0) {
      // a dead CTA only balances the bytes its peers go on delivering, so that the barrier's
      // transaction count stays bounded
      if (!dead)
        mbar_arrive_expect_tx(mbar, k * g.slots * 16);
      else
        mbar_expect_tx(mbar, k * g.slots * 16);
    }
    const bool pushing = (int)rank != g.skip_push_rank;
    float mean[VE], m2[VE], cnt = 0.f;
#pragma unroll
    for (int e = 0; e < VE; ++e) mean[e] = 0.f, m2[e] = 0.f;
    tile_moments<T, VE, UNI>(stile, sstep, iters, mean, m2, cnt, first, x + base + (size_t)kFirstRows * gstep, gstep);
    if (first) cluster_wait();  // the peers' inbox barriers exist (every CTA arrived long ago)
    first = false;
    int g_lo, n_slots;
    cb_groups(g, c0, g_lo, n_slots);
    if (UNI && g.shuf) {
      // shuffle reductions: red doubles as the two warp-sum buffers
      float sm = 0.f;
#pragma unroll
      for (int e = 0; e < VE; ++e) sm += mean[e];
      const float n_loc = (float)nrows * (float)g.D;
      const float tot = cta_slot_sum_shuf(g, cnt * sm, tx, red);
      const float lm = n_loc > 0.f ? tot / n_loc : 0.f;
      float acc = 0.f, dev = 0.f;
#pragma unroll
      for (int e = 0; e < VE; ++e) {
        const float d = mean[e] - lm;
        dev = fmaf(d, d, dev);
        acc += m2[e];
      }
      const float m2loc = cta_slot_sum_shuf(g, fmaf(cnt, dev, acc), tx, red + g.wsum_stride);
      if (pushing && tid < g.CV && (tid & ((1 << g.tps_shift) - 1)) == 0) {
        const int s = tid >> g.tps_shift;
        for (unsigned q = 0; q < k; ++q) st_async_f32x4(inbox + 4 * (rank * g.slots + s), mbar, q, lm, m2loc, n_loc, 0.f);
      }
    } else {
      cta_slot_moments<VE, UNI>(g, mean, m2, cnt, tx, ty, c0, nrows, g_lo, n_slots, red, tmp, slot);
      __syncthreads();
      for (int s = tid; pushing && s < g.slots; s += blockDim.x) {
        const bool live = s < n_slots;
        const float a = live ? slot[s] : 0.f, b = live ? slot[g.slots + s] : 0.f, c = live ? slot[2 * g.slots + s] : 0.f;
        for (unsigned q = 0; q < k; ++q) st_async_f32x4(inbox + 4 * (rank * g.slots + s), mbar, q, a, b, c, 0.f);
      }
    }
    {
      // Every CTA of the cluster pushed (mean, M2, count) of each slot into every inbox.  Combine them
      // in rank order (every CTA gets bit-identical statistics):
      //   mean = sum n_q mean_q / sum n_q,  M2 = sum M2_q + n_q (mean_q - mean)^2
      // A wait that gives up (or a dead CTA) yields NaN statistics: the failure is visible in y,
      // mean and rstd, and the entry points report it from the next call on.
      const bool ok = !dead && mbar_wait_bounded(mbar, (uses >> 1) & 1u, g.wait);
      ++uses;
      if (tid == 0 && !ok) s_dead = 1;
      for (int s = tid; s < n_slots; s += blockDim.x) {
        float wsum = 0.f, ntot = 0.f;
        for (unsigned q = 0; q < k; ++q) {
          const float4 v = *reinterpret_cast<const float4*>(inbox + 4 * (q * g.slots + s));
          wsum = fmaf(v.z, v.x, wsum);
          ntot += v.z;
        }
        const float mu = ok ? wsum / ntot : __int_as_float(0x7fc00000);
        float m2tot = 0.f;
        for (unsigned q = 0; q < k; ++q) {
          const float4 v = *reinterpret_cast<const float4*>(inbox + 4 * (q * g.slots + s));
          const float d = v.x - mu;
          m2tot += fmaf(v.z * d, d, v.y);
        }
        const float rs = ok ? rsqrtf(fmaxf(m2tot / ntot, 0.f) + eps) : __int_as_float(0x7fc00000);
        stat[s] = mu;
        stat[g.slots + s] = rs;
        if (rank == 0) {
          mean_out[(size_t)n * g.G + g_lo + s] = mu;
          rstd_out[(size_t)n * g.G + g_lo + s] = rs;
        }
      }
      __syncthreads();
    }

    if (streaming) {
      float a[VE], b[VE];
      if constexpr (kVec)
        lane_affine_raw<T, VE, UNI>(ga_raw, be_raw, stat, stat + g.slots, g_lo, c0 + tx * VE, g.div_D, a, b);
      else
        lane_affine<T, VE, UNI>(gamma, beta, stat, stat + g.slots, g_lo, c0 + tx * VE, g.div_D, a, b);
      // the cluster's next item, whose rows take over the tile slots as they are read
      const int nxt = item + n_clusters;
      const bool refill = nxt < n_items;
      const int n2 = refill ? g.div_ncb.div(nxt) : 0, cb2 = nxt - n2 * g.ncb;
      tile_apply<T, VE, ACT>(stile, sstep, y + base, gstep, iters, a, b, refill,
                             x + (size_t)n2 * g.R * g.C + (refill ? cb2 * g.CW : 0) + row_off);
    }
    // No barrier here: the next item's reductions write red / tmp / slot before their first
    // barrier, none of which is read by the output pass, and `stat` is rewritten only after it.
  }
  // No exit barrier: nothing reaches into this CTA's shared memory after the wait of its last item.
}

// ------------------------------------------------------------------------------------------------
// two-pass, kernel 1: CTA-local moments per tile.  grid.x = N * chunks * ncb.
// scratch layout: wpart[(((n * chunks + chunk) * ncb + cb) * slots + s) * 3] = {mean, M2, count}
// ------------------------------------------------------------------------------------------------
template <typename T, int VE, bool UNI>
__global__ void __launch_bounds__(kMaxThreads)
    gn_fwd_stats_kernel(const T* __restrict__ x, float* __restrict__ wpart, const Geom g) {
  extern __shared__ uint4 smem_raw[];
  using P = Pack<T, VE>;
  // [ring: kRingDepth * blockDim vectors][red][tmp][slot]
  const size_t ring_bytes = sizeof(T) * VE == 16 ? (size_t)kRingDepth * blockDim.x * 16 : 0;
  float* red = reinterpret_cast<float*>(reinterpret_cast<char*>(smem_raw) + ring_bytes);
  float* tmp = red + g.red_floats;
  float* slot = tmp + g.slots;

  // the finalize and apply kernels may take their places on the SMs now; they wait for this grid
  // before they read its partials
  grid_dep_launch_dependents();
  const int tile_id = blockIdx.x;
  const int t1 = g.div_ncb.div(tile_id), cb = tile_id - t1 * g.ncb;
  const int n = g.div_chunks.div(t1), chunk = t1 - n * g.chunks;
  const int c0 = cb * g.CW;
  const int r0 = chunk * g.rows_per_cta;
  const int nrows = min(g.rows_per_cta, g.R - r0);
  const int tid = threadIdx.x;
  const int ty = g.div_CV.div(tid), tx = tid - ty * g.CV;
  const bool streaming = (ty < g.TY) && (c0 + tx * VE < g.C);

  float mean[VE], m2[VE], cnt = 0.f;
#pragma unroll
  for (int e = 0; e < VE; ++e) mean[e] = 0.f, m2[e] = 0.f;
  const size_t base = ((size_t)n * g.R + r0 + ty) * g.C + c0 + (size_t)tx * VE;
  const int iters = (streaming && ty < nrows) ? (nrows - ty + g.TY - 1) / g.TY : 0;
  stream_moments<T, VE, UNI>(x + base, (size_t)g.TY * g.C, iters, smem_addr(smem_raw) + tid * 16, blockDim.x * 16, mean, m2,
                        cnt);
  int g_lo, n_slots;
  cb_groups(g, c0, g_lo, n_slots);
  cta_slot_moments<VE, UNI>(g, mean, m2, cnt, tx, ty, c0, nrows, g_lo, n_slots, red, tmp, slot);
  float* out = wpart + (size_t)tile_id * g.slots * 3;
  for (int s = tid; s < n_slots; s += blockDim.x) {
    out[3 * s + 0] = slot[s];
    out[3 * s + 1] = slot[g.slots + s];
    out[3 * s + 2] = slot[2 * g.slots + s];
  }
}

// two-pass, kernel 2: one CTA per (n, group) merges all partials that cover the group in ONE sweep:
// sums about the first partial's mean (nothing cancels for a large |mean|), every thread's loads in
// flight at once, one block reduction of the three sums (warp butterflies, then the warps in order) -
// a fixed order, so the result is reproducible.
__global__ void __launch_bounds__(256)
    gn_fwd_finalize_kernel(const float* __restrict__ wpart, float* __restrict__ mean_out,
                           float* __restrict__ rstd_out, float eps, const Geom g) {
  __shared__ float red[8][3];
  grid_dep_launch_dependents();
  grid_dep_wait();  // the statistics kernel's partials
  const int n = blockIdx.x / g.G, grp = blockIdx.x - n * g.G;
  const int cb_lo = (grp * g.D) / g.CW, cb_hi = ((grp + 1) * g.D - 1) / g.CW;
  const int ncov = cb_hi - cb_lo + 1;
  const int total = ncov * g.chunks;
  auto partial = [&](int i) {
    const int chunk = i / ncov, cb = cb_lo + (i - chunk * ncov);
    const int s = grp - (cb * g.CW) / g.D;
    return wpart + ((((size_t)n * g.chunks + chunk) * g.ncb + cb) * g.slots + s) * 3;
  };
  const float K0 = partial(0)[0];  // the same word for every thread: one broadcast load
  float an = 0.f, ad = 0.f, aq = 0.f;
#pragma unroll 4
  for (int i = threadIdx.x; i < total; i += 256) {
    const float* p = partial(i);
    const float d = p[0] - K0, c = p[2];
    an += c;
    ad = fmaf(c, d, ad);
    aq += fmaf(c * d, d, p[1]);
  }
#pragma unroll
  for (int b = 16; b >= 1; b >>= 1) {
    an += __shfl_xor_sync(0xffffffffu, an, b);
    ad += __shfl_xor_sync(0xffffffffu, ad, b);
    aq += __shfl_xor_sync(0xffffffffu, aq, b);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) red[warp][0] = an, red[warp][1] = ad, red[warp][2] = aq;
  __syncthreads();
  if (threadIdx.x == 0) {
    an = ad = aq = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) an += red[w][0], ad += red[w][1], aq += red[w][2];
    const float dm = ad / an;
    mean_out[blockIdx.x] = K0 + dm;
    rstd_out[blockIdx.x] = rsqrtf(fmaxf(fmaf(-ad, dm, aq) / an, 0.f) + eps);
  }
}

// two-pass, kernel 3: normalise + affine + activation.  Tiles are visited in the reverse order of
// kernel 1 (tile_id = last - blockIdx.x), so the most recently read part of x is re-read first.
template <typename T, int VE, int ACT, bool UNI>
__global__ void __launch_bounds__(kMaxThreads)
    gn_fwd_apply_kernel(const T* __restrict__ x, const T* __restrict__ gamma, const T* __restrict__ beta,
                        const float* __restrict__ mean_in, const float* __restrict__ rstd_in, T* __restrict__ y,
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
  grid_dep_wait();  // the finalize kernel's statistics
  float a[VE], b[VE];
  lane_affine<T, VE, UNI>(gamma, beta, mean_in + (size_t)n * g.G, rstd_in + (size_t)n * g.G, 0, c0 + tx * VE, g.div_D, a, b);
  const size_t base = ((size_t)n * g.R + r0) * g.C + c0 + (size_t)tx * VE;
  const size_t rs = (size_t)g.C / VE;
  stream_apply<T, VE, ACT>(reinterpret_cast<const P*>(x + base), rs, reinterpret_cast<P*>(y + base), rs, nrows, ty, g.TY,
                           a, b);
}

// ------------------------------------------------------------------------------------------------
// host-side launchers
// ------------------------------------------------------------------------------------------------
template <typename T, int VE, int ACT, bool UNI>
static cudaError_t launch_fused(const FwdCall& c, const Plan& p, cudaStream_t stream) {
  auto kern = p.threads <= 128 ? gn_fwd_fused_kernel<T, VE, ACT, UNI, 128> : gn_fwd_fused_kernel<T, VE, ACT, UNI, kMaxThreads>;
  cudaError_t err = ensure_kernel_attributes((const void*)kern, p.smem_bytes, p.geom.k > 8);
  if (err != cudaSuccess) return err;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)p.grid, 1, 1);
  cfg.blockDim = dim3((unsigned)p.threads, 1, 1);
  cfg.dynamicSmemBytes = p.smem_bytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)p.geom.k;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (p.geom.persist) {  // as many clusters as are resident at once
    int clusters = 0;
    err = resident_clusters((const void*)kern, &cfg, &clusters);
    if (err != cudaSuccess) return err;
    const long long items = (long long)p.geom.N * p.geom.ncb;
    if (clusters > items) clusters = (int)items;
    cfg.gridDim.x = (unsigned)clusters * (unsigned)p.geom.k;
  }
  Geom g = p.geom;
  err = wait_limit_for_device(&g.wait);
  if (err != cudaSuccess) return err;
  g.skip_push_rank = c.test_skip_push_rank;
  if (c.test_wait_clocks > 0) {
    g.wait.clocks = c.test_wait_clocks;
    g.wait.polls = 64;
  }
  // the exchange self-test wants one item per cluster, so that no barrier is used twice
  if (c.test_skip_push_rank >= 0 && (long long)g.N * g.ncb * g.k > (long long)cfg.gridDim.x) return cudaErrorInvalidConfiguration;
  return cudaLaunchKernelEx(&cfg, kern, (const T*)c.x, (const T*)c.gamma, (const T*)c.beta, (T*)c.y, c.mean, c.rstd,
                            c.eps, g);
}

template <typename T, int VE, int ACT, bool UNI>
static cudaError_t launch_two_pass(const FwdCall& c, const Plan& p, cudaStream_t stream) {
  float* wpart = reinterpret_cast<float*>(c.workspace);
  cudaError_t err = ensure_kernel_attributes((const void*)gn_fwd_stats_kernel<T, VE, UNI>, p.smem_bytes, false);
  if (err != cudaSuccess) return err;
  gn_fwd_stats_kernel<T, VE, UNI><<<(unsigned)p.grid, p.threads, p.smem_bytes, stream>>>((const T*)c.x, wpart, p.geom);
  err = cudaGetLastError();
  if (err != cudaSuccess) return err;
  err = launch_chained(gn_fwd_finalize_kernel, (unsigned)(p.geom.N * p.geom.G), dim3(256), 0, stream, p.chain, wpart, c.mean,
                       c.rstd, c.eps, p.geom);
  if (err != cudaSuccess) return err;
  return launch_chained(gn_fwd_apply_kernel<T, VE, ACT, UNI>, (unsigned)p.grid, dim3((unsigned)p.threads), 0, stream, p.chain,
                        (const T*)c.x, (const T*)c.gamma, (const T*)c.beta, c.mean, c.rstd, (T*)c.y, p.geom);
}

template <typename T, int VE, int ACT>
static cudaError_t launch_fwd_t(const FwdCall& c, const Plan& p, cudaStream_t stream) {
  // uniform: every thread-vector lies inside one group (always true for single-element vectors)
  const bool uni = VE == 1 || p.geom.D % VE == 0;
  if (uni) return p.fused ? launch_fused<T, VE, ACT, true>(c, p, stream) : launch_two_pass<T, VE, ACT, true>(c, p, stream);
  if constexpr (VE > 1)
    return p.fused ? launch_fused<T, VE, ACT, false>(c, p, stream) : launch_two_pass<T, VE, ACT, false>(c, p, stream);
  return cudaErrorInvalidValue;
}

template <typename T, int VE>
static cudaError_t launch_fwd_act(const FwdCall& c, const Plan& p, cudaStream_t stream) {
  switch (c.act) {
    case kActIdentity: return launch_fwd_t<T, VE, kActIdentity>(c, p, stream);
    case kActRelu: return launch_fwd_t<T, VE, kActRelu>(c, p, stream);
    case kActSilu: return launch_fwd_t<T, VE, kActSilu>(c, p, stream);
    case kActGelu: return launch_fwd_t<T, VE, kActGelu>(c, p, stream);
    default: return launch_fwd_t<T, VE, kActGeluTanh>(c, p, stream);
  }
}

template <typename T>
static cudaError_t launch_fwd_ve(const FwdCall& c, const Plan& p, cudaStream_t stream) {
  constexpr int VFULL = 16 / sizeof(T);
  return p.ve == 1 ? launch_fwd_act<T, 1>(c, p, stream) : launch_fwd_act<T, VFULL>(c, p, stream);
}

cudaError_t launch_forward(const FwdCall& c, const Plan& p, cudaStream_t stream) {
  if (p.wave) return launch_forward_wave(c, p, stream);
  switch (c.dtype) {
    case 0: return launch_fwd_ve<float>(c, p, stream);
    case 1: return launch_fwd_ve<__half>(c, p, stream);
    default: return launch_fwd_ve<__nv_bfloat16>(c, p, stream);
  }
}

}  // namespace gnb200
