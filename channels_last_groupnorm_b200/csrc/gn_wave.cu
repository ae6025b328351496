// "Wave" launch plan for slabs that do not fit a thread-block cluster: forward and backward
// GroupNorm (+activation) for NHWC tensors as ONE persistent cooperative kernel each, sm_100a.
//
// The multi-kernel plan it replaces (and the reference's compute_stats_pt1 / pt2 / scale_shift and
// width_reduce / height_reduce / compute_bwd_scale_biases / dx_elem chains,
// src/gnnhwc/csrc/gn_kernel.cu:439-531, 932-1055) reads the tensor once for the statistics and a
// second time for the output pass; when the tensor is larger than L2 the second read comes from
// HBM again.  Here the tensor is cut into waves - ranges of (sample, column block) slabs of a few
// tens of MB - and each wave is taken through both passes before the next one is touched, so the
// second pass finds its rows in L2:
//
//   for every wave:   pass A  every CTA streams its row chunk of the wave's slabs and writes partial
//                             sums to scratch; the CTA that delivers a slab's last partial merges
//                             them (fixed order, no atomics on values) and raises the slab's flag
//                     pass B  every CTA waits (bounded) for its slab's flag, then streams the same
//                             rows again - L2 hits - and writes y / dx with streaming stores
//
// All CTAs of the grid are resident (cooperative launch), so a CTA may wait for a flag that
// another CTA raises.  Rows travel by TMA: one producer warp issues 2-D tiled bulk copies
// (cp.async.bulk.tensor, box = column block x rows) into a ring of shared-memory stages, each
// completing on an mbarrier; the consumer warps read a stage into registers, hand the stage back
// through a second mbarrier and do the arithmetic.  No thread computes a global load address.
#include <cuda.h>

#include <map>
#include <mutex>

#include "gn_kernels.h"
#include "gn_math.cuh"

namespace gnb200 {

unsigned long long* debug_trace_buffer(size_t need);

namespace {

// ------------------------------------------------------------------------------------------------
// device helpers
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const CUtensorMap* tm, int c, int row, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(smem_dst),
      "l"(tm), "r"(c), "r"(row), "r"(smem_addr(bar))
      : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
// A consumer warp hands a stage back to the producer only after it has USED the vectors it read from
// the stage.  The shared-memory loads are merely issued when the warp moves on; signalling the stage
// as free right after them let the producer's next TMA copy into the stage (fast when the rows come from
// L2) now and then overtake a load that was still queued, and a warp computed one stage's rows from
// pieces of a later stage.  So the arrival follows the arithmetic in program order - instructions
// issue in order and the arithmetic cannot issue before its operands have arrived - and pin_regs keeps
// the compiler from moving that arithmetic behind the arrival (the output stores of pass B are
// volatile asm statements and stay in front of it by themselves).
template <int N>
__device__ __forceinline__ void pin_regs(float (&a)[N]) {
#pragma unroll
  for (int e = 0; e < N; ++e) asm volatile("" : "+f"(a[e]));
}
__device__ __forceinline__ void release_stage(uint64_t* empty_bar, int lane) {
  __syncwarp();
  if (lane == 0) mbar_arrive(empty_bar);
}
// Block barrier of the consumer warps only (the producer warp never joins it).  The call sites
// follow code in which single lanes of a warp act alone (lane 0 stores a partial, thread 0 counts a
// delivery), so the warp is brought together first and the barrier is the form that counts threads
// and does not require a converged warp: an aligned bar.sync executed by a warp whose lanes had
// not yet reconverged let the barrier open before every warp had arrived.
__device__ __forceinline__ void consumer_sync(int consumers) {
  __syncwarp();
  asm volatile("barrier.sync 1, %0;" ::"r"(consumers) : "memory");
}
__device__ __forceinline__ float warp_sum_all(float v) {
#pragma unroll
  for (int b = 16; b >= 1; b >>= 1) v += __shfl_xor_sync(0xffffffffu, v, b);
  return v;
}
// streaming 16-byte store: the line is marked evict-first, so results do not push the rows that
// pass B still has to read out of L2
__device__ __forceinline__ void stg128_stream(void* p, const uint4 v) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_u32(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// counter + 1 with release and acquire semantics in one round trip: the writes this CTA made before
// its block barrier are released, and if the returned value tells that every other CTA has
// incremented, their writes are acquired.  Returns the value before the increment.
__device__ __forceinline__ unsigned int atom_inc_acq_rel(unsigned int* p) {
  unsigned int v;
  asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_inc_release(unsigned int* p) {
  asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(p) : "memory");
}
// A pair of floats published as ONE 64-bit word, which is its own flag: the scratch words start as
// all ones (cudaMemsetAsync with 0xFF; no result of the kernels has that bit pattern - their NaN is
// 0x7fc00000), the merging CTA stores the pair with one 8-byte store, and a reader that sees
// anything but all ones has both values.  No fence and no second round trip for the data.
constexpr unsigned long long kUnset = 0xFFFFFFFFFFFFFFFFull;
__device__ __forceinline__ void publish_pair(unsigned long long* word, float a, float b) {
  const unsigned long long v = ((unsigned long long)__float_as_uint(b) << 32) | __float_as_uint(a);
  asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(word), "l"(v) : "memory");
}
// Waits (bounded like mbar_wait_bounded) for a published pair; false if the wait gave up.
__device__ __forceinline__ bool wait_pair(const unsigned long long* word, const WaitLimit& lim, float& a, float& b) {
  unsigned long long v;
  asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(word) : "memory");
  if (v == kUnset) {
    const long long t0 = clock64();
    unsigned int polls = 0;
    for (;;) {
      asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(word) : "memory");
      if (v != kUnset) break;
      if (++polls > lim.polls && clock64() - t0 > lim.clocks) {
        wait_gave_up(lim);
        return false;
      }
      __nanosleep(32);
    }
  }
  a = __uint_as_float((unsigned int)(v & 0xffffffffu));
  b = __uint_as_float((unsigned int)(v >> 32));
  return true;
}

#define kNaN __int_as_float(0x7fc00000)

// Optional timeline for tuning (WaveGeom::trace, set with gnb200_debug_set_trace): thread 0 of every CTA
// stores the global nanosecond timer at a few points of every step: trace[(cta * steps + step) * 4 + k].
__device__ __forceinline__ void trace_mark(const WaveGeom& g, int step, int k) {
  if (g.trace != nullptr && threadIdx.x == 0) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    g.trace[((size_t)blockIdx.x * (2 * g.waves) + step) * 4 + k] = t;  // (a team uses the first 2 * its waves steps)
  }
}

// mbarrier waits of the wave kernels.  `gave_up` is the CTA's shared flag: the first wait that runs
// out sets it (and poisons the results, see the callers); from then on no wait of this CTA spends
// its limit again, so a broken run ends after about one limit instead of one limit per stage.
// producer (a single thread):
__device__ __forceinline__ void producer_wait(uint64_t* bar, unsigned parity, volatile int* gave_up, const WaitLimit& lim) {
  if (mbar_try_wait(bar, parity)) return;
  if (*gave_up != 0) return;
  if (!mbar_wait_bounded(bar, parity, lim)) *gave_up = 1;
}
// consumers (whole warps): if the phase is not complete yet, lane 0 alone polls - 256 polling threads
// would take issue slots from the CTAs that share the SM - and afterwards every lane observes the
// completed phase with one more try_wait of its own, which is what makes the TMA's writes visible
// to it.
__device__ __forceinline__ void consumer_wait(uint64_t* bar, unsigned parity, volatile int* gave_up, const WaitLimit& lim) {
  if (__all_sync(0xffffffffu, mbar_try_wait(bar, parity))) return;
  if ((threadIdx.x & 31) == 0 && *gave_up == 0) {
    if (!mbar_wait_bounded(bar, parity, lim)) *gave_up = 1;
  }
  __syncwarp();
  (void)mbar_try_wait(bar, parity);
}

// One unit of work: the rows [r0, r1) of one (sample, column block) slab.
struct Unit {
  int item, n, c0, chunk, r0, r1;
};
// Unit u (0 <= u < units of the wave) of wave `wave`: chunk-major, so that CTAs with neighbouring
// indices work on the same rows of neighbouring column blocks.
__device__ __forceinline__ Unit decode_unit(const WaveGeom& g, int wave, int u) {
  const int item0 = wave * g.ipw;
  const int n_it = min(g.ipw, g.items - item0);
  Unit t;
  t.chunk = u / n_it;
  t.item = item0 + (u - t.chunk * n_it);
  t.n = g.div_ncb.div(t.item);
  t.c0 = (t.item - t.n * g.ncb) * g.CW;
  t.r0 = t.chunk * g.rows_per_chunk;
  t.r1 = min(g.R, t.r0 + g.rows_per_chunk);
  return t;
}
__device__ __forceinline__ int wave_units(const WaveGeom& g, int wave) {
  return min(g.ipw, g.items - wave * g.ipw) * g.chunks;
}

// Teams.  The CTAs are dealt to `teams` teams (team = blockIdx % teams); team t takes the waves t,
// t + teams, ... through their passes on its own, so the teams drift apart in time: while one team
// waits for its slabs to be merged or writes results, another reads the next wave from HBM.  Up to
// `teams` waves share L2.  Within a team the order of the steps is A0 B0 A1 B1 ... or, overlapped
// (WaveGeom::overlap), A0 A1 B0 A2 B1 ... B(last) with the team's own waves.
struct Team {
  int id, cta, ctas, waves, steps;
};
__device__ __forceinline__ Team my_team(const WaveGeom& g) {
  Team t;
  t.id = (int)(blockIdx.x % (unsigned)g.teams);
  t.cta = (int)(blockIdx.x / (unsigned)g.teams);
  t.ctas = (int)(gridDim.x / (unsigned)g.teams);
  t.waves = t.id < g.waves ? (g.waves - t.id + g.teams - 1) / g.teams : 0;
  t.steps = 2 * t.waves;
  return t;
}
__device__ __forceinline__ void schedule(const WaveGeom& g, const Team& tm, int step, int& pass, int& wave) {
  int w;
  if (!g.overlap) {
    w = step >> 1;
    pass = step & 1;
  } else if (step == 0) {
    pass = 0, w = 0;
  } else if (step == tm.steps - 1) {
    pass = 1, w = tm.waves - 1;
  } else if (step & 1) {
    pass = 0, w = (step + 1) >> 1;
  } else {
    pass = 1, w = (step >> 1) - 1;
  }
  wave = tm.id + w * g.teams;
}

// Ring position shared by the producer and the consumers: stage index and the parity of its use.
struct Ring {
  int s;
  unsigned ph;
  __device__ __forceinline__ void next(int stages) {
    if (++s == stages) {
      s = 0;
      ph ^= 1u;
    }
  }
};

// The producer: lane 0 of the last warp.  Walks through exactly the stage sequence the consumers
// expect - the schedule above, and in every step this CTA's units in order - and keeps up to
// `stages` boxes in flight.  NT = tensors per stage (1: x; 2: x and dy).
template <int NT>
__device__ __forceinline__ void produce(const WaveGeom& g, const CUtensorMap* tm_a, const CUtensorMap* tm_b,
                                        uint32_t stage0, uint64_t* full, uint64_t* empty, volatile int* gave_up) {
  Ring ring = {0, 0};
  bool wrapped = false;
  const uint32_t box_bytes = (uint32_t)g.box_bytes;
  const Team tm = my_team(g);
  for (int step = 0; step < tm.steps; ++step) {
    int pass, wave;
    schedule(g, tm, step, pass, wave);
    const int units = wave_units(g, wave);
    for (int u = tm.cta; u < units; u += tm.ctas) {
      const Unit t = decode_unit(g, wave, u);
      for (int r = t.r0; r < t.r1; r += g.BR) {
        // the consumers have emptied this stage (its previous use has the opposite parity)
        if (wrapped) producer_wait(&empty[ring.s], ring.ph ^ 1u, gave_up, g.wait);
        mbar_arrive_expect_tx(&full[ring.s], NT * box_bytes);
        const uint32_t dst = stage0 + (uint32_t)ring.s * NT * (uint32_t)g.stage_bytes;
        tma_load_2d(dst, tm_a, t.c0, t.n * g.R + r, &full[ring.s]);
        if (NT == 2) tma_load_2d(dst + (uint32_t)g.stage_bytes, tm_b, t.c0, t.n * g.R + r, &full[ring.s]);
        ring.next(g.stages);
        if (ring.s == 0) wrapped = true;
      }
    }
  }
}

// Shared-memory carve-up (dynamic): [stages * NT boxes, 1024-byte aligned][full, empty mbarriers]
// [flags][reduction scratch floats].
struct Smem {
  uint32_t stage0;
  uint64_t* full;
  uint64_t* empty;
  volatile int* flags;  // [0] this CTA delivered the slab's last partial  [1] a wait gave up
  float* red;
};
template <int NT>
__device__ __forceinline__ Smem carve(const WaveGeom& g, unsigned char* base) {
  const uintptr_t p = (reinterpret_cast<uintptr_t>(base) + 1023) & ~(uintptr_t)1023;
  Smem s;
  s.stage0 = smem_addr(reinterpret_cast<void*>(p));
  unsigned char* q = reinterpret_cast<unsigned char*>(p) + (size_t)g.stages * NT * g.stage_bytes;
  s.full = reinterpret_cast<uint64_t*>(q);
  s.empty = s.full + g.stages;
  s.flags = reinterpret_cast<volatile int*>(s.empty + g.stages);
  s.red = reinterpret_cast<float*>(const_cast<int*>(s.flags) + 4);
  return s;
}

// mbarrier set-up by thread 0, then a block barrier of all warps (the only one the producer joins)
__device__ __forceinline__ void init_ring(const WaveGeom& g, const Smem& sm) {
  if (threadIdx.x == 0) {
    for (int s = 0; s < g.stages; ++s) {
      mbar_init(&sm.full[s], 1);
      mbar_init(&sm.empty[s], (unsigned)(g.consumers / 32));
    }
    sm.flags[0] = 0;
    sm.flags[1] = 0;
    fence_mbar_init_cluster();
  }
  __syncthreads();
}

// The unit's partials have been stored (by any of the consumer threads).  After a block barrier
// thread 0 counts the unit as delivered (counters start at all ones, like every scratch word that is
// cleared).  Returns true (to every consumer thread) if this CTA delivered the slab's last unit and
// has to merge the slab; all other units' partials are then visible to it.  Two consumer barriers.
__device__ __forceinline__ bool deliver(const WaveGeom& g, const Smem& sm, unsigned int* count, int item) {
  consumer_sync(g.consumers);
  if (threadIdx.x == 0) sm.flags[0] = (atom_inc_acq_rel(&count[item]) + 1u) == (unsigned)(g.chunks - 1) ? 1 : 0;
  consumer_sync(g.consumers);
  return sm.flags[0] != 0;
}

constexpr int kMergeUnroll = 8;  // partials a lane has in flight while a slab is merged

// ------------------------------------------------------------------------------------------------
// forward
// scratch: part[(item * chunks + chunk) * slots + s] = (mean, M2, count, -) of the unit's rows
// ------------------------------------------------------------------------------------------------
template <typename T, int ACT, bool UNI, int KR>
__global__ void __launch_bounds__(kWaveThreads, 3)
    gn_fwd_wave_kernel(const __grid_constant__ CUtensorMap tm_x, const T* __restrict__ gamma,
                       const T* __restrict__ beta, T* __restrict__ y, float* mean_out, float* rstd_out, float eps,
                       float4* part, unsigned int* count, unsigned long long* stat_words, const WaveGeom g) {
  constexpr int VE = 16 / sizeof(T);
  constexpr bool kShifted = sizeof(T) == 2;
  constexpr int KN = UNI ? 1 : VE;
  extern __shared__ unsigned char smem_raw[];
  const Smem sm = carve<1>(g, smem_raw);
  init_ring(g, sm);
  const int tid = threadIdx.x;
  if (tid >= g.consumers) {
    if (tid == g.consumers) produce<1>(g, &tm_x, &tm_x, sm.stage0, sm.full, sm.empty, &sm.flags[1]);
    return;
  }
  const int ty = g.div_CV.div(tid), tx = tid - ty * g.CV;
  const bool streaming = ty < g.TY;
  const int lane = tid & 31, warp = tid >> 5, nwarps = g.consumers >> 5;
  const uint32_t my_off = streaming ? (uint32_t)(ty * g.CV + tx) * 16u : 0u;  // idle threads read vector 0
  const uint32_t row_step = (uint32_t)(g.TY * g.CV) * 16u;  // bytes between a thread's rows in a stage
  float* red_mean = sm.red;
  float* red_m2 = red_mean + g.consumers * VE;
  float* red_cnt = red_m2 + g.consumers * VE;
  float* stat = red_cnt + g.consumers;  // mean[slots], rstd[slots]
  Ring ring = {0, 0};

  const Team tm = my_team(g);
  for (int step = 0; step < tm.steps; ++step) {
    int pass, wave;
    schedule(g, tm, step, pass, wave);
    const int units = wave_units(g, wave);
    trace_mark(g, step, 0);
    if (pass == 0) {
      // ---------------- pass A: partial moments ----------------
      for (int u = tm.cta; u < units; u += tm.ctas) {
        const Unit t = decode_unit(g, wave, u);
        float mean[VE], m2[VE], cnt = 0.f, K[KN];
#pragma unroll
        for (int e = 0; e < VE; ++e) mean[e] = 0.f, m2[e] = 0.f;
#pragma unroll
        for (int e = 0; e < KN; ++e) K[e] = 0.f;
        int rows_done = 0;
        for (int r = t.r0; r < t.r1; r += g.BR) {
          consumer_wait(&sm.full[ring.s], ring.ph, &sm.flags[1], g.wait);
          const uint32_t base = sm.stage0 + (uint32_t)ring.s * g.stage_bytes + my_off;
          uint4 w[KR];
#pragma unroll
          for (int j = 0; j < KR; ++j) w[j] = lds128(base + j * row_step);
          if (streaming) {
#pragma unroll
            for (int j = 0; j < KR; ++j) {
              if (r + ty + j * g.TY < t.r1) {
                if constexpr (kShifted) {
                  if (rows_done == 0) {  // the shift: the values of the thread's first row
                    float f0[VE];
                    unpack16<T, VE>(w[j], f0);
#pragma unroll
                    for (int e = 0; e < KN; ++e) K[e] = f0[e];
                  }
                  shifted_step<T, VE, KN>(w[j], K, mean, m2);
                } else {
                  float f[VE];
                  unpack16<T, VE>(w[j], f);
                  welford_step<VE>(f, mean, m2, cnt);
                }
                ++rows_done;
              }
            }
          }
          pin_regs(mean);
          pin_regs(m2);
          release_stage(&sm.empty[ring.s], lane);
          ring.next(g.stages);
        }
        trace_mark(g, step, 1);
        if constexpr (kShifted) shifted_finish<VE, KN>(K, rows_done, mean, m2, cnt);
        // CTA reduction: every thread parks its per-lane moments; one warp per group slot merges
        // them in a fixed order (mean first, then the squared deviations about it)
#pragma unroll
        for (int e = 0; e < VE; ++e) {
          red_mean[tid * VE + e] = mean[e];
          red_m2[tid * VE + e] = m2[e];
        }
        red_cnt[tid] = streaming ? cnt : 0.f;
        consumer_sync(g.consumers);
        for (int s = warp; s < g.slots; s += nwarps) {
          const int total = g.TY * g.D;
          float an = 0.f, am = 0.f;
          for (int i = lane; i < total; i += 32) {
            const int jy = g.div_D.div(i), c = s * g.D + (i - jy * g.D);
            const int th = jy * g.CV + c / VE;
            const float n_i = red_cnt[th];
            an += n_i;
            am = fmaf(n_i, red_mean[th * VE + (c % VE)], am);
          }
          an = warp_sum_all(an);
          am = warp_sum_all(am);
          const float mu = an > 0.f ? am / an : 0.f;
          float a2 = 0.f;
          for (int i = lane; i < total; i += 32) {
            const int jy = g.div_D.div(i), c = s * g.D + (i - jy * g.D);
            const int th = jy * g.CV + c / VE;
            const float d = red_mean[th * VE + (c % VE)] - mu;
            a2 += fmaf(red_cnt[th] * d, d, red_m2[th * VE + (c % VE)]);
          }
          a2 = warp_sum_all(a2);
          if (lane == 0) part[((size_t)t.item * g.chunks + t.chunk) * g.slots + s] = make_float4(mu, a2, an, 0.f);
        }
        const bool last_unit = deliver(g, sm, count, t.item);
        trace_mark(g, step, 2);
        if (last_unit) {
          // This CTA brought the slab's last partial: merge all of them and publish mean / rstd.
          // One warp per group slot; a lane keeps kMergeUnroll loads in flight; sums are taken about
          // the first chunk's mean, so that nothing cancels when |mean| is large.
          const int g_lo = g.div_D.div(t.c0);
          const float4* row0 = part + (size_t)t.item * g.chunks * g.slots;
          for (int s = warp; s < g.slots; s += nwarps) {
            float K0 = 0.f, an = 0.f, ad = 0.f, aq = 0.f;
            for (int base = lane; base < g.chunks + lane; base += 32 * kMergeUnroll) {
              float4 v[kMergeUnroll];
#pragma unroll
              for (int q = 0; q < kMergeUnroll; ++q) {
                const int ch = base + 32 * q;
                v[q] = ch < g.chunks ? __ldcg(&row0[(size_t)ch * g.slots + s]) : make_float4(0.f, 0.f, 0.f, 0.f);
              }
              if (base == lane) K0 = __shfl_sync(0xffffffffu, v[0].x, 0);  // chunk 0's mean, loaded by lane 0
#pragma unroll
              for (int q = 0; q < kMergeUnroll; ++q) {
                const float d = v[q].x - K0;
                an += v[q].z;
                ad = fmaf(v[q].z, d, ad);
                aq += fmaf(v[q].z * d, d, v[q].y);
              }
            }
            an = warp_sum_all(an);
            ad = warp_sum_all(ad);
            aq = warp_sum_all(aq);
            if (lane == 0) {
              const bool bad = sm.flags[1] != 0;
              const float dm = ad / an;
              const float var = fmaxf(fmaf(-ad, dm, aq) / an, 0.f);
              const float mu = bad ? kNaN : K0 + dm, rs = bad ? kNaN : rsqrtf(var + eps);
              publish_pair(&stat_words[(size_t)t.item * g.slots + s], mu, rs);  // what pass B waits for
              mean_out[(size_t)t.n * g.G + g_lo + s] = mu;
              rstd_out[(size_t)t.n * g.G + g_lo + s] = rs;
            }
          }
        }
        trace_mark(g, step, 3);
      }
    } else {
      // ---------------- pass B: normalise, scale, shift, activate ----------------
      for (int u = tm.cta; u < units; u += tm.ctas) {
        const Unit t = decode_unit(g, wave, u);
        const int g_lo = g.div_D.div(t.c0);
        for (int s = tid; s < g.slots; s += g.consumers) {
          float mu = kNaN, rs = kNaN;  // a wait that gave up poisons what depends on it
          if (sm.flags[1] != 0 || !wait_pair(&stat_words[(size_t)t.item * g.slots + s], g.wait, mu, rs)) {
            sm.flags[1] = 1;
            mu = rs = kNaN;
          }
          stat[s] = mu;
          stat[g.slots + s] = rs;
        }
        consumer_sync(g.consumers);
        trace_mark(g, step, 1);
        float a[VE], b[VE];
        if (streaming) lane_affine<T, VE, UNI>(gamma, beta, stat, stat + g.slots, g_lo, t.c0 + tx * VE, g.div_D, a, b);
        T* yrow = y + ((size_t)t.n * g.R + t.r0 + ty) * g.C + t.c0 + tx * VE;
        const size_t ystep = (size_t)g.TY * g.C;
        for (int r = t.r0; r < t.r1; r += g.BR) {
          consumer_wait(&sm.full[ring.s], ring.ph, &sm.flags[1], g.wait);
          const uint32_t base = sm.stage0 + (uint32_t)ring.s * g.stage_bytes + my_off;
          uint4 w[KR];
#pragma unroll
          for (int j = 0; j < KR; ++j) w[j] = lds128(base + j * row_step);
          if (streaming) {
#pragma unroll
            for (int j = 0; j < KR; ++j) {
              if (r + ty + j * g.TY < t.r1) {
                float f[VE];
                unpack16<T, VE>(w[j], f);
#pragma unroll
                for (int e = 0; e < VE; ++e) f[e] = fmaf(f[e], a[e], b[e]);
                stg128_stream(yrow + (size_t)j * ystep, act_pack16<T, VE, ACT>(f));
              }
            }
          }
          release_stage(&sm.empty[ring.s], lane);
          ring.next(g.stages);
          yrow += (size_t)KR * ystep;
        }
        trace_mark(g, step, 2);
        consumer_sync(g.consumers);  // `stat` is rewritten by the next unit
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------
// backward
// scratch: tpart[(n * chunks + chunk) * C + c] = (S1, S2) of channel c over the rows of chunk `chunk`
//          gpart[(item * chunks + chunk) * slots + s] = gamma-weighted sums of the unit's group slot s
//          coef_words[item * slots + s] = (A, B) of group slot s as one 64-bit word, all ones until the slab's last chunk is merged
// Only the small group sums are on the path between the passes; the channel sums are added up - for
// dgamma / dbeta - by all CTAs together when they have finished their last unit.
// ------------------------------------------------------------------------------------------------
// dx of one 16-byte vector of a 16-bit tensor: dyh = dy * act'(x a + b) with act' in packed half
// precision, dx = ag * dyh + c1 * x + c2.
template <typename T, int ACT>
__device__ __forceinline__ uint4 bwd_dx_packed(const uint4& xw, const uint4& dw, const float (&a)[8],
                                               const float (&b)[8], const float (&ag)[8], const float (&c1)[8],
                                               const float (&c2)[8]) {
  static_assert(sizeof(T) == 2, "16-bit tensors only");
  float fx[8], fd[8], o[8];
  unpack16<T, 8>(xw, fx);
  unpack16<T, 8>(dw, fd);
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    float g0 = 1.f, g1 = 1.f;
    if constexpr (ACT != kActIdentity) {
      const float yh0 = fmaf(fx[2 * p], a[2 * p], b[2 * p]);
      const float yh1 = fmaf(fx[2 * p + 1], a[2 * p + 1], b[2 * p + 1]);
      const float2 gf = __half22float2(act_grad_h2<ACT>(f32x2_to_h2_sat(yh0, yh1)));
      g0 = gf.x;
      g1 = gf.y;
    }
    o[2 * p] = fmaf(ag[2 * p], fd[2 * p] * g0, fmaf(c1[2 * p], fx[2 * p], c2[2 * p]));
    o[2 * p + 1] = fmaf(ag[2 * p + 1], fd[2 * p + 1] * g1, fmaf(c1[2 * p + 1], fx[2 * p + 1], c2[2 * p + 1]));
  }
  return pack16<T, 8>(o);
}

template <typename T, int ACT, bool UNI, int KR>
__global__ void __launch_bounds__(kWaveThreads, 2)
    gn_bwd_wave_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_dy,
                       const T* __restrict__ gamma, const T* __restrict__ beta, const float* __restrict__ mean_in,
                       const float* __restrict__ rstd_in, T* __restrict__ dx, float2* tpart, float2* gpart,
                       unsigned long long* coef_words, unsigned int* count, unsigned int* done,
                       float* __restrict__ dparam_f32,
                       T* __restrict__ dgamma, T* __restrict__ dbeta, const WaveGeom g) {
  constexpr int VE = 16 / sizeof(T);
  constexpr bool kRaw = sizeof(T) == 2;  // 16-bit tensors: packed arithmetic, S2 against the raw x
  extern __shared__ unsigned char smem_raw[];
  const Smem sm = carve<2>(g, smem_raw);
  init_ring(g, sm);
  const int tid = threadIdx.x;
  if (tid >= g.consumers) {
    if (tid == g.consumers) produce<2>(g, &tm_x, &tm_dy, sm.stage0, sm.full, sm.empty, &sm.flags[1]);
    return;
  }
  const int ty = g.div_CV.div(tid), tx = tid - ty * g.CV;
  const bool streaming = ty < g.TY;
  const int lane = tid & 31, warp = tid >> 5, nwarps = g.consumers >> 5;
  const uint32_t my_off = streaming ? (uint32_t)(ty * g.CV + tx) * 16u : 0u;
  const uint32_t row_step = (uint32_t)(g.TY * g.CV) * 16u;
  float* red1 = sm.red;
  float* red2 = red1 + g.consumers * VE;
  float* schan = red2 + g.consumers * VE;  // S1[CW], S2[CW] of the unit
  float* scoef = schan + 2 * g.CW;         // A[slots], B[slots]
  Ring ring = {0, 0};
  const float inv_m = 1.0f / ((float)g.D * (float)g.R);

  const Team tm = my_team(g);
  for (int step = 0; step < tm.steps; ++step) {
    int pass, wave;
    schedule(g, tm, step, pass, wave);
    const int units = wave_units(g, wave);
    if (pass == 0) {
      // ---------------- pass A: per-channel sums of dyh and dyh * xh ----------------
      for (int u = tm.cta; u < units; u += tm.ctas) {
        const Unit t = decode_unit(g, wave, u);
        BwdLane<T, VE> L;
        float a[VE], b[VE], s1[VE], s2[VE];
#pragma unroll
        for (int e = 0; e < VE; ++e) s1[e] = 0.f, s2[e] = 0.f, a[e] = 0.f, b[e] = 0.f;
        if (streaming) {
          lane_setup<T, VE, UNI>(gamma, beta, mean_in + (size_t)t.n * g.G, rstd_in + (size_t)t.n * g.G,
                                 t.c0 + tx * VE, g.div_D, L);
#pragma unroll
          for (int e = 0; e < VE; ++e) {
            a[e] = L.r[e] * L.ga[e];
            b[e] = fmaf(L.nmr[e], L.ga[e], L.be[e]);
          }
        }
        for (int r = t.r0; r < t.r1; r += g.BR) {
          consumer_wait(&sm.full[ring.s], ring.ph, &sm.flags[1], g.wait);
          const uint32_t base = sm.stage0 + (uint32_t)ring.s * 2u * g.stage_bytes + my_off;
          uint4 xw[KR], dw[KR];
#pragma unroll
          for (int j = 0; j < KR; ++j) {
            xw[j] = lds128(base + j * row_step);
            dw[j] = lds128(base + g.stage_bytes + j * row_step);
          }
          if (streaming) {
#pragma unroll
            for (int j = 0; j < KR; ++j) {
              if (r + ty + j * g.TY < t.r1) {
                if constexpr (kRaw) {
                  bwd_row_sums_packed<T, ACT>(xw[j], dw[j], a, b, s1, s2);
                } else {
                  float fx[VE], fd[VE];
                  unpack16<T, VE>(xw[j], fx);
                  unpack16<T, VE>(dw[j], fd);
                  bwd_row_sums<T, VE, ACT>(fx, fd, L, s1, s2);
                }
              }
            }
          }
          pin_regs(s1);
          pin_regs(s2);
          release_stage(&sm.empty[ring.s], lane);
          ring.next(g.stages);
        }
        if constexpr (kRaw) {  // S2 = sum dyh * xh = rstd * (sum dyh * x - mean * sum dyh)
          if (streaming) {
#pragma unroll
            for (int e = 0; e < VE; ++e) s2[e] = fmaf(L.r[e], s2[e], L.nmr[e] * s1[e]);
          }
        }
#pragma unroll
        for (int e = 0; e < VE; ++e) {
          red1[tid * VE + e] = s1[e];
          red2[tid * VE + e] = s2[e];
        }
        consumer_sync(g.consumers);
        for (int c = tid; c < g.CW; c += g.consumers) {  // channel sums over the row lanes, fixed order
          float t1 = 0.f, t2 = 0.f;
          const int v = c / VE, e = c % VE;
          for (int jy = 0; jy < g.TY; ++jy) {
            t1 += red1[(jy * g.CV + v) * VE + e];
            t2 += red2[(jy * g.CV + v) * VE + e];
          }
          schan[c] = t1;
          schan[g.CW + c] = t2;
          tpart[((size_t)t.n * g.chunks + t.chunk) * g.C + t.c0 + c] = make_float2(t1, t2);
        }
        consumer_sync(g.consumers);
        for (int s = warp; s < g.slots; s += nwarps) {  // gamma-weighted group sums of the unit
          float w1 = 0.f, w2 = 0.f;
          for (int c = s * g.D + lane; c < (s + 1) * g.D; c += 32) {
            const float ga = load_param<T>(gamma, t.c0 + c);
            w1 = fmaf(ga, schan[c], w1);
            w2 = fmaf(ga, schan[g.CW + c], w2);
          }
          w1 = warp_sum_all(w1);
          w2 = warp_sum_all(w2);
          if (lane == 0) gpart[((size_t)t.item * g.chunks + t.chunk) * g.slots + s] = make_float2(w1, w2);
        }
        if (deliver(g, sm, count, t.item)) {
          // merge the slab's group sums (one warp per slot, kMergeUnroll loads in flight per lane)
          const float2* row0 = gpart + (size_t)t.item * g.chunks * g.slots;
          for (int s = warp; s < g.slots; s += nwarps) {
            float w1 = 0.f, w2 = 0.f;
            for (int base = lane; base < g.chunks; base += 32 * kMergeUnroll) {
              float2 v[kMergeUnroll];
#pragma unroll
              for (int q = 0; q < kMergeUnroll; ++q) {
                const int ch = base + 32 * q;
                v[q] = ch < g.chunks ? __ldcg(&row0[(size_t)ch * g.slots + s]) : make_float2(0.f, 0.f);
              }
#pragma unroll
              for (int q = 0; q < kMergeUnroll; ++q) w1 += v[q].x, w2 += v[q].y;
            }
            w1 = warp_sum_all(w1);
            w2 = warp_sum_all(w2);
            if (lane == 0) {
              const bool bad = sm.flags[1] != 0;
              publish_pair(&coef_words[(size_t)t.item * g.slots + s], bad ? kNaN : w1 * inv_m, bad ? kNaN : w2 * inv_m);
            }
          }
          // every unit of the slab has delivered its channel sums: one more slab whose part of tpart is complete
          if (tid == 0) red_inc_release(done);
        }
      }
    } else {
      // ---------------- pass B: dx ----------------
      for (int u = tm.cta; u < units; u += tm.ctas) {
        const Unit t = decode_unit(g, wave, u);
        const int g_lo = g.div_D.div(t.c0);
        for (int s = tid; s < g.slots; s += g.consumers) {
          float A = kNaN, B = kNaN;
          if (sm.flags[1] != 0 || !wait_pair(&coef_words[(size_t)t.item * g.slots + s], g.wait, A, B)) {
            sm.flags[1] = 1;
            A = B = kNaN;
          }
          scoef[s] = A;
          scoef[g.slots + s] = B;
        }
        consumer_sync(g.consumers);
        BwdLane<T, VE> L;
        float a[VE], b[VE], ag[VE], c1[VE], c2[VE];
#pragma unroll
        for (int e = 0; e < VE; ++e) a[e] = b[e] = ag[e] = c1[e] = c2[e] = 0.f;
        if (streaming) {
          lane_setup<T, VE, UNI>(gamma, beta, mean_in + (size_t)t.n * g.G, rstd_in + (size_t)t.n * g.G,
                                 t.c0 + tx * VE, g.div_D, L);
#pragma unroll
          for (int e = 0; e < VE; ++e) {
            const int s = g.div_D.div(t.c0 + tx * VE + (UNI ? 0 : e)) - g_lo;
            const float A = scoef[s], B = scoef[g.slots + s];
            a[e] = L.r[e] * L.ga[e];
            b[e] = fmaf(L.nmr[e], L.ga[e], L.be[e]);
            ag[e] = a[e];
            // dx = ag dyh - r (A + xh B) with xh = r x + nmr:  c1 x + c2 (16-bit) or nb xh + na (fp32)
            const float nb = -L.r[e] * B, na = -L.r[e] * A;
            if constexpr (kRaw) {
              c1[e] = nb * L.r[e];
              c2[e] = fmaf(nb, L.nmr[e], na);
            } else {
              c1[e] = nb;
              c2[e] = na;
            }
          }
        }
        T* orow = dx + ((size_t)t.n * g.R + t.r0 + ty) * g.C + t.c0 + tx * VE;
        const size_t ostep = (size_t)g.TY * g.C;
        for (int r = t.r0; r < t.r1; r += g.BR) {
          consumer_wait(&sm.full[ring.s], ring.ph, &sm.flags[1], g.wait);
          const uint32_t base = sm.stage0 + (uint32_t)ring.s * 2u * g.stage_bytes + my_off;
          uint4 xw[KR], dw[KR];
#pragma unroll
          for (int j = 0; j < KR; ++j) {
            xw[j] = lds128(base + j * row_step);
            dw[j] = lds128(base + g.stage_bytes + j * row_step);
          }
          if (streaming) {
#pragma unroll
            for (int j = 0; j < KR; ++j) {
              if (r + ty + j * g.TY < t.r1) {
                if constexpr (kRaw) {
                  stg128_stream(orow + (size_t)j * ostep, bwd_dx_packed<T, ACT>(xw[j], dw[j], a, b, ag, c1, c2));
                } else {
                  float fx[VE], fd[VE], xh[VE], yh[VE], gr[VE];
                  unpack16<T, VE>(xw[j], fx);
                  unpack16<T, VE>(dw[j], fd);
#pragma unroll
                  for (int e = 0; e < VE; ++e) {
                    xh[e] = fmaf(fx[e], L.r[e], L.nmr[e]);
                    yh[e] = fmaf(xh[e], L.ga[e], L.be[e]);
                  }
                  act_grad_vec<T, VE, ACT>(yh, gr);
#pragma unroll
                  for (int e = 0; e < VE; ++e) fx[e] = fmaf(ag[e], fd[e] * gr[e], fmaf(c1[e], xh[e], c2[e]));
                  stg128_stream(orow + (size_t)j * ostep, pack16<T, VE>(fx));
                }
              }
            }
          }
          release_stage(&sm.empty[ring.s], lane);
          ring.next(g.stages);
          orow += (size_t)KR * ostep;
        }
        consumer_sync(g.consumers);  // `scoef` is rewritten by the next unit
      }
    }
  }
  // ---------------- tail: dgamma / dbeta ----------------
  // Every slab of the call has been merged once `done` equals the number of slabs; all channel sums
  // in tpart are then visible.  The grid's warps share the channels; a warp adds up the N * chunks
  // rows of its channel in a fixed order (lane-strided, then the butterfly).
  if (tid == 0 && sm.flags[1] == 0) {
    const long long t0 = clock64();
    unsigned int polls = 0;
    while (ld_acquire_u32(done) + 1u < (unsigned)g.items) {  // the counter starts at all ones
      if (++polls > g.wait.polls && clock64() - t0 > g.wait.clocks) {
        wait_gave_up(g.wait);
        sm.flags[1] = 1;
        break;
      }
      __nanosleep(40);
    }
  }
  consumer_sync(g.consumers);
  const bool bad = sm.flags[1] != 0;
  const int rows = g.N * g.chunks;
  for (int c = blockIdx.x * nwarps + warp; c < g.C; c += gridDim.x * nwarps) {
    float t1 = 0.f, t2 = 0.f;
    for (int base = lane; base < rows; base += 32 * kMergeUnroll) {
      float2 v[kMergeUnroll];
#pragma unroll
      for (int q = 0; q < kMergeUnroll; ++q) {
        const int row = base + 32 * q;
        v[q] = row < rows ? __ldcg(&tpart[(size_t)row * g.C + c]) : make_float2(0.f, 0.f);
      }
#pragma unroll
      for (int q = 0; q < kMergeUnroll; ++q) t1 += v[q].x, t2 += v[q].y;
    }
    t1 = warp_sum_all(t1);
    t2 = warp_sum_all(t2);
    if (lane == 0) {
      if (bad) t1 = t2 = kNaN;
      dparam_f32[c] = t2;        // dgamma
      dparam_f32[g.C + c] = t1;  // dbeta
      if (dgamma) dgamma[c] = store_param<T>(t2);
      if (dbeta) dbeta[c] = store_param<T>(t1);
    }
  }
}

}  // namespace

namespace {

// ------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled through the runtime's driver entry-point lookup (the library does not link
// libcuda directly)
cudaError_t encode_fn(EncodeTiledFn* out) {
  static std::mutex mu;
  static EncodeTiledFn fn = nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t err = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
    if (err != cudaSuccess) return err;
    if (q != cudaDriverEntryPointSuccess || !p) return cudaErrorNotSupported;
    fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  *out = fn;
  return cudaSuccess;
}

// 2-D map of an NHWC tensor seen as (N * R) rows of C elements; box = CW x BR.
cudaError_t make_tensor_map(CUtensorMap* tm, const void* base, int dtype, const WaveGeom& g) {
  EncodeTiledFn enc = nullptr;
  cudaError_t err = encode_fn(&enc);
  if (err != cudaSuccess) return err;
  const size_t es = dtype == 0 ? 4 : 2;
  const CUtensorMapDataType dt = dtype == 0   ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                 : dtype == 1 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                              : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const cuuint64_t dims[2] = {(cuuint64_t)g.C, (cuuint64_t)g.N * (cuuint64_t)g.R};
  const cuuint64_t strides[1] = {(cuuint64_t)g.C * es};
  const cuuint32_t box[2] = {(cuuint32_t)g.CW, (cuuint32_t)g.BR};
  const cuuint32_t estr[2] = {1, 1};
  // no promotion of the L2 fetch size beyond the row segment: a wave reads 64-byte segments of
  // 256-byte rows and must not drag the neighbouring column blocks into L2
  const CUtensorMapL2promotion promo =
      (size_t)g.CW * es >= 256 ? CU_TENSOR_MAP_L2_PROMOTION_L2_256B
      : (size_t)g.CW * es >= 128 ? CU_TENSOR_MAP_L2_PROMOTION_L2_128B
      : (size_t)g.CW * es >= 64 ? CU_TENSOR_MAP_L2_PROMOTION_L2_64B
                                : CU_TENSOR_MAP_L2_PROMOTION_NONE;
  const CUresult rc = enc(tm, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_NONE, promo, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return rc == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

// the cooperative grid of the plan must be resident at once
cudaError_t check_resident(const void* func, int threads, size_t smem, long long grid) {
  struct Key {
    int dev;
    const void* func;
    size_t smem;
    bool operator<(const Key& o) const {
      if (dev != o.dev) return dev < o.dev;
      if (func != o.func) return func < o.func;
      return smem < o.smem;
    }
  };
  static std::mutex mu;
  static std::map<Key, long long> cache;
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return err;
  std::lock_guard<std::mutex> lock(mu);
  const Key key = {dev, func, smem};
  auto it = cache.find(key);
  if (it == cache.end()) {
    int per_sm = 0, sms = 0;
    err = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, func, threads, smem);
    if (err != cudaSuccess) return err;
    err = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (err != cudaSuccess) return err;
    it = cache.emplace(key, (long long)per_sm * sms).first;
  }
  return grid <= it->second ? cudaSuccess : cudaErrorCooperativeLaunchTooLarge;
}

template <typename Kern, typename... Args>
cudaError_t launch_cooperative(Kern kern, const Plan& p, cudaStream_t stream, Args... args) {
  cudaError_t err = ensure_kernel_attributes((const void*)kern, p.smem_bytes, false);
  if (err != cudaSuccess) return err;
  err = check_resident((const void*)kern, p.threads, p.smem_bytes, p.grid);
  if (err != cudaSuccess) return err;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)p.grid, 1, 1);
  cfg.blockDim = dim3((unsigned)p.threads, 1, 1);
  cfg.dynamicSmemBytes = p.smem_bytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, args...);
}

// scratch layout of the wave plans (offsets in bytes from a 16-byte aligned base); everything from
// `clear` to `total` is set to all ones before the launch
struct FwdScratch {
  size_t part, clear, words, count, total;
};
FwdScratch fwd_scratch(const WaveGeom& g) {
  FwdScratch s;
  s.part = 0;
  s.clear = (size_t)g.items * g.chunks * g.slots * sizeof(float4);
  s.words = s.clear;
  s.count = s.words + (size_t)g.items * g.slots * 8;
  s.total = (s.count + (size_t)g.items * 4 + 15) & ~(size_t)15;
  return s;
}
struct BwdScratch {
  size_t tpart, gpart, clear, words, count, done, total;
};
BwdScratch bwd_scratch(const WaveGeom& g) {
  BwdScratch s;
  s.tpart = 0;
  s.gpart = (size_t)g.N * g.chunks * g.C * sizeof(float2);
  s.clear = s.gpart + (size_t)g.items * g.chunks * g.slots * sizeof(float2);
  s.words = s.clear;
  s.count = s.words + (size_t)g.items * g.slots * 8;
  s.done = s.count + (size_t)g.items * 4;
  s.total = (s.done + 4 + 15) & ~(size_t)15;
  return s;
}

template <typename T, int ACT, bool UNI>
cudaError_t launch_fwd_wave_t(const FwdCall& c, const Plan& p, cudaStream_t stream) {
  WaveGeom g = p.wgeom;
  cudaError_t err = wait_limit_for_device(&g.wait);
  if (err != cudaSuccess) return err;
  g.trace = debug_trace_buffer((size_t)p.grid * 2 * g.waves * 4 * sizeof(unsigned long long));
  CUtensorMap tm;
  err = make_tensor_map(&tm, c.x, c.dtype, g);
  if (err != cudaSuccess) return err;
  const FwdScratch s = fwd_scratch(g);
  char* ws = static_cast<char*>(c.workspace);
  err = cudaMemsetAsync(ws + s.clear, 0xFF, s.total - s.clear, stream);  // statistics words and arrival counters
  if (err != cudaSuccess) return err;
  auto args = [&](auto kern) {
    return launch_cooperative(kern, p, stream, tm, (const T*)c.gamma, (const T*)c.beta, (T*)c.y, c.mean, c.rstd, c.eps,
                              reinterpret_cast<float4*>(ws + s.part), reinterpret_cast<unsigned int*>(ws + s.count),
                              reinterpret_cast<unsigned long long*>(ws + s.words), g);
  };
  return g.KR == 2 ? args(gn_fwd_wave_kernel<T, ACT, UNI, 2>) : args(gn_fwd_wave_kernel<T, ACT, UNI, 4>);
}

template <typename T, int ACT, bool UNI>
cudaError_t launch_bwd_wave_t(const BwdCall& c, const Plan& p, cudaStream_t stream) {
  WaveGeom g = p.wgeom;
  cudaError_t err = wait_limit_for_device(&g.wait);
  if (err != cudaSuccess) return err;
  CUtensorMap tm_x, tm_dy;
  err = make_tensor_map(&tm_x, c.x, c.dtype, g);
  if (err != cudaSuccess) return err;
  err = make_tensor_map(&tm_dy, c.dy, c.dtype, g);
  if (err != cudaSuccess) return err;
  const BwdScratch s = bwd_scratch(g);
  char* ws = static_cast<char*>(c.workspace);
  err = cudaMemsetAsync(ws + s.clear, 0xFF, s.total - s.clear, stream);
  if (err != cudaSuccess) return err;
  auto args = [&](auto kern) {
    return launch_cooperative(kern, p, stream, tm_x, tm_dy, (const T*)c.gamma, (const T*)c.beta, c.mean, c.rstd,
                              (T*)c.dx, reinterpret_cast<float2*>(ws + s.tpart), reinterpret_cast<float2*>(ws + s.gpart),
                              reinterpret_cast<unsigned long long*>(ws + s.words),
                              reinterpret_cast<unsigned int*>(ws + s.count), reinterpret_cast<unsigned int*>(ws + s.done),
                              c.dparam_f32, (T*)c.dgamma, (T*)c.dbeta, g);
  };
  return g.KR == 2 ? args(gn_bwd_wave_kernel<T, ACT, UNI, 2>) : args(gn_bwd_wave_kernel<T, ACT, UNI, 4>);
}

template <typename T, int ACT>
cudaError_t launch_fwd_wave_u(const FwdCall& c, const Plan& p, cudaStream_t stream) {
  constexpr int VE = 16 / sizeof(T);
  return p.wgeom.D % VE == 0 ? launch_fwd_wave_t<T, ACT, true>(c, p, stream) : launch_fwd_wave_t<T, ACT, false>(c, p, stream);
}
template <typename T, int ACT>
cudaError_t launch_bwd_wave_u(const BwdCall& c, const Plan& p, cudaStream_t stream) {
  constexpr int VE = 16 / sizeof(T);
  return p.wgeom.D % VE == 0 ? launch_bwd_wave_t<T, ACT, true>(c, p, stream) : launch_bwd_wave_t<T, ACT, false>(c, p, stream);
}
template <typename T>
cudaError_t launch_fwd_wave_a(const FwdCall& c, const Plan& p, cudaStream_t stream) {
  switch (c.act) {
    case kActIdentity: return launch_fwd_wave_u<T, kActIdentity>(c, p, stream);
    case kActRelu: return launch_fwd_wave_u<T, kActRelu>(c, p, stream);
    case kActSilu: return launch_fwd_wave_u<T, kActSilu>(c, p, stream);
    case kActGelu: return launch_fwd_wave_u<T, kActGelu>(c, p, stream);
    default: return launch_fwd_wave_u<T, kActGeluTanh>(c, p, stream);
  }
}
template <typename T>
cudaError_t launch_bwd_wave_a(const BwdCall& c, const Plan& p, cudaStream_t stream) {
  switch (c.act) {
    case kActIdentity: return launch_bwd_wave_u<T, kActIdentity>(c, p, stream);
    case kActRelu: return launch_bwd_wave_u<T, kActRelu>(c, p, stream);
    case kActSilu: return launch_bwd_wave_u<T, kActSilu>(c, p, stream);
    case kActGelu: return launch_bwd_wave_u<T, kActGelu>(c, p, stream);
    default: return launch_bwd_wave_u<T, kActGeluTanh>(c, p, stream);
  }
}

}  // namespace

namespace {
unsigned long long* g_trace_ptr = nullptr;
size_t g_trace_bytes = 0;
}  // namespace
void debug_set_trace(void* ptr, size_t bytes) {
  g_trace_ptr = static_cast<unsigned long long*>(ptr);
  g_trace_bytes = bytes;
}
unsigned long long* debug_trace_buffer(size_t need) { return (g_trace_ptr && g_trace_bytes >= need) ? g_trace_ptr : nullptr; }

size_t wave_workspace_bytes(const WaveGeom& g, int direction) {
  return direction == 0 ? fwd_scratch(g).total : bwd_scratch(g).total;
}

cudaError_t launch_forward_wave(const FwdCall& c, const Plan& p, cudaStream_t stream) {
  switch (c.dtype) {
    case 0: return launch_fwd_wave_a<float>(c, p, stream);
    case 1: return launch_fwd_wave_a<__half>(c, p, stream);
    default: return launch_fwd_wave_a<__nv_bfloat16>(c, p, stream);
  }
}

cudaError_t launch_backward_wave(const BwdCall& c, const Plan& p, cudaStream_t stream) {
  switch (c.dtype) {
    case 0: return launch_bwd_wave_a<float>(c, p, stream);
    case 1: return launch_bwd_wave_a<__half>(c, p, stream);
    default: return launch_bwd_wave_a<__nv_bfloat16>(c, p, stream);
  }
}

}  // namespace gnb200
