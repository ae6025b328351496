// Host-side launch planner: picks vector width, column-block width, CTA shape, cluster size and
// the fused / multi-kernel path for one problem.  Plays the role of the reference's
// calc_block_params / closest_factor heuristics (src/gnnhwc/csrc/gn_kernel.cu:37-60, 121-128),
// but is organised around B200 resources: 148 SMs, <= 227 KB shared memory per CTA, clusters of
// up to 8 (16 non-portable) CTAs.
//
// Environment overrides (for experiments and benchmarks only):
//   GNB200_FORCE_PATH = fused | twopass     GNB200_CW = channels per column block
//   GNB200_K = cluster size                 GNB200_THREADS = target CTA size
//   GNB200_TILE_KB = shared-memory tile budget per CTA (fused path)
//   GNB200_ROWS = rows per CTA tile (multi-kernel path)
#include <stdlib.h>
#include <string.h>

#include <map>
#include <mutex>
#include <utility>

#include "gn_kernels.h"

namespace gnb200 {

namespace {

constexpr int kSmCount = 148;
constexpr size_t kSmemMaxOptin = 227 * 1024;

long long gcd_ll(long long a, long long b) {
  while (b) {
    long long t = a % b;
    a = b;
    b = t;
  }
  return a;
}

int env_int(const char* name, int fallback) {
  const char* v = getenv(name);
  if (!v || !*v) return fallback;
  return atoi(v);
}

int round_up(int v, int m) { return (v + m - 1) / m * m; }

// n / d == (umulhi(n, mul) + n) >> shr for 0 <= n < 2^31 (round-up method, 33-bit multiplier)
FastDiv make_fast_div(int d) {
  FastDiv f;
  if (d < 1) d = 1;
  uint32_t s = 0;
  while ((1ull << s) < (unsigned long long)d) ++s;
  const unsigned long long m = ((1ull << 32) * ((1ull << s) - (unsigned long long)d)) / (unsigned long long)d + 1;
  f.mul = (uint32_t)m;
  f.shr = s;
  return f;
}

// shared-memory floats of the CTA reductions (layouts in gn_fwd.cu / gn_bwd.cu)
// forward `red` scratch: the per-row-lane values of the generic reduction, or two warp-sum buffers
// of the shuffle reduction, or the gathered slot arrays of up to 16 cluster peers
int round_up4(int v) { return (v + 3) & ~3; }
// warp-sum buffer of the shuffle reductions: one float per (warp, group slot)
int wsum_stride_floats(int threads, int CV, int tps_shift) { return round_up4(((threads + 31) / 32) * (CV >> tps_shift)); }

size_t fwd_red_floats(int CW, int CV, int TY, int slots, int threads, bool shuf, int tps_shift) {
  if (shuf) {  // two warp-sum buffers, overlaid later by the gathered slot arrays of the peers
    const int a = 2 * wsum_stride_floats(threads, CV, tps_shift), b = 16 * 3 * slots;
    return (size_t)round_up4(a > b ? a : b);
  }
  size_t r = (size_t)TY * CW;
  if (r < 1024) r = 1024;
  if (r < (size_t)16 * 3 * slots) r = (size_t)16 * 3 * slots;
  return r;
}
// red, tmp, two slot arrays, stat, and for the push exchange two inboxes of k * slots entries of
// four floats plus alignment slack and two mbarriers
size_t fwd_fold_floats(int CW, int CV, int TY, int slots, int threads, bool shuf, int tps_shift, int k) {
  // (+ 12: up to 3 floats of alignment slack, two 8-byte mbarriers, the dead flag and its padding)
  return fwd_red_floats(CW, CV, TY, slots, threads, shuf, tps_shift) + (size_t)9 * slots + 8 + (size_t)2 * 4 * k * slots + 12;
}
// backward scratch of the CTA reductions.
// Generic reductions: red = the per-row-lane channel sums (2 * TY * CW floats), then part and chan.
// Shuffle reductions (fused kernel only): red = [two warp-sum buffers of wsum_stride floats,
// overlaid later by the gathered group sums of up to 16 cluster peers][per-warp channel sums
// nwarps * 2 * CW from wpart_off]; part and chan are not used.
int bwd_wpart_off(int threads, int CV, int tps_shift, int slots) {
  (void)slots;
  return round_up4(2 * wsum_stride_floats(threads, CV, tps_shift));
}
size_t bwd_red_floats(int CW, int CV, int TY, int slots, int threads, bool shuf, int tps_shift) {
  if (shuf) return (size_t)bwd_wpart_off(threads, CV, tps_shift, slots) + (size_t)((threads + 31) / 32) * 2 * CW;
  size_t r = (size_t)2 * TY * CW;
  if (r < 1024) r = 1024;
  if (r < (size_t)16 * 2 * slots) r = (size_t)16 * 2 * slots;
  return r;
}
// k: cluster size (inbox of the exchange: k * slots entries of four floats, alignment slack, mbarrier)
size_t bwd_fold_floats(int CW, int CV, int TY, int slots, int threads, bool shuf, int tps_shift, int k) {
  const size_t lanes = shuf ? 0 : (size_t)2 * (threads > CW ? threads : CW) + (size_t)2 * CW;  // part, chan
  return bwd_red_floats(CW, CV, TY, slots, threads, shuf, tps_shift) + lanes + (size_t)4 * slots + 8 + (size_t)4 * k * slots + 8;
}

bool is_pow2(int v) { return v > 0 && (v & (v - 1)) == 0; }

// Shuffle reductions of the fused kernels: every 16-byte vector lies in one group, and CV and the
// threads per group row (D / ve) are powers of two with CV <= 32.
bool shuffle_geometry(int D, int ve, int CV, int* tps_shift) {
  *tps_shift = 0;
  if (ve < 4 || D % ve != 0) return false;
  const int tps = D / ve;
  if (!(is_pow2(CV) && CV <= 32 && is_pow2(tps) && tps <= CV) || getenv("GNB200_NO_SHUF") != nullptr) return false;
  while ((1 << *tps_shift) < tps) ++*tps_shift;
  return true;
}

// `fused`: the plan is for the fused kernels (the multi-kernel path never uses shuffle reductions)
void fill_divisors(Geom* g, int ve, int direction, int threads, bool fused) {
  g->shuf = 0;
  g->tps_shift = 0;
  g->skip_push_rank = -1;
  int tps_shift = 0;
  if (fused && shuffle_geometry(g->D, ve, g->CV, &tps_shift)) {
    g->shuf = 1;
    g->tps_shift = tps_shift;
  }
  g->wsum_stride = g->shuf ? wsum_stride_floats(threads, g->CV, tps_shift) : 0;
  g->wpart_off = (direction == 1 && g->shuf) ? bwd_wpart_off(threads, g->CV, tps_shift, g->slots) : 0;
  g->red_floats = (int)(direction == 0 ? fwd_red_floats(g->CW, g->CV, g->TY, g->slots, threads, g->shuf != 0, tps_shift)
                                       : bwd_red_floats(g->CW, g->CV, g->TY, g->slots, threads, g->shuf != 0, tps_shift));
  g->div_D = make_fast_div(g->D);
  g->div_CV = make_fast_div(g->CV);
  g->div_CW = make_fast_div(g->CW);
  g->div_ncb = make_fast_div(g->ncb);
  g->div_chunks = make_fast_div(g->chunks);
}

struct Shape {
  int N, R, C, G, D, s, ve;
  int direction;
};

// thread layout for a column block of CV vectors: TY row lanes, CTA size rounded to a warp
void thread_layout(int CV, int rows_per_cta, int target_threads, int* TY, int* threads) {
  int ty = target_threads / CV;
  if (ty < 1) ty = 1;
  if (ty > rows_per_cta) ty = rows_per_cta;
  if (ty < 1) ty = 1;
  *TY = ty;
  *threads = round_up(CV * ty, 32);
}

// One fused candidate: column block of `cw` channels split over a cluster of `k` CTAs.
// Returns false if the tile does not fit; otherwise fills *out and a heuristic score
// (higher is better): SMs kept busy x row-segment efficiency x co-residency.
bool plan_fused_candidate(const Shape& sh, int cw, int k, int target_threads, Plan* out, double* score) {
  const int ve = sh.ve, s = sh.s;
  const int ncb = sh.C / cw;
  const int CV = cw / ve;
  const int slots = cw / sh.D;
  const int rows = (sh.R + k - 1) / k;
  if (k > 1 && (long long)rows * (k - 1) >= sh.R) return false;  // a CTA of the cluster would be idle
  int TY, threads;
  thread_layout(CV, rows, target_threads, &TY, &threads);
  // larger CTAs only pay when every thread still owns >= 16 rows (per-thread set-up is amortised)
  if (target_threads > 128 && env_int("GNB200_THREADS", 0) == 0 && rows / TY < 16) return false;
  // forward: the x tile.  backward: the dy * act' tile plus a 4-row cp.async ring for x
  const size_t ring = (sh.direction == 1 && ve > 1) ? (size_t)4 * threads * 16 : 0;
  const size_t tile = (((size_t)rows * CV * ve * s + 15) & ~(size_t)15) + ring;
  int tps_shift = 0;
  const bool shuf = shuffle_geometry(sh.D, ve, CV, &tps_shift);
  const size_t fold = (sh.direction == 0 ? fwd_fold_floats(cw, CV, TY, slots, threads, shuf, tps_shift, k)
                                         : bwd_fold_floats(cw, CV, TY, slots, threads, shuf, tps_shift, k)) * 4;
  if (tile + fold > kSmemMaxOptin - 1024) return false;

  Plan p = {};
  p.fused = true;
  p.wave = false;
  p.ve = ve;
  p.threads = threads;
  p.grid = (long long)sh.N * ncb * k;
  p.smem_bytes = tile + fold;
  p.ws_bytes = sh.direction == 0 ? 0 : (size_t)sh.N * k * sh.C * 2 * sizeof(float);  // channel sums per cluster rank
  p.launches = sh.direction == 0 ? 1 : 2;
  p.geom = Geom{sh.N, sh.R, sh.C, sh.G, sh.D, cw, CV, TY, ncb, rows, k, slots, k};
  // forward: launch only the clusters that are resident at once; each loops over its items
  p.geom.persist = (sh.direction == 0 && env_int("GNB200_PERSIST", 1) != 0) ? 1 : 0;
  fill_divisors(&p.geom, ve, sh.direction, threads, true);
  if (p.grid > 0x7fffffffLL) return false;

  // Heuristic fitted to measurements on B200 (bf16 / fp16, N x 256 x 64 x 64 and similar):
  // the kernels are bound by instruction issue and latency rather than DRAM, so co-resident CTAs
  // per SM matter most, then rows per thread (per-thread set-up is amortised over them), then the
  // contiguous row segment (64 B is nearly as good as 128 B; 32 B wastes DRAM sectors).
  const long long seg = (long long)cw * s;
  // 32-byte segments waste DRAM bursts on large tensors; a tensor that fits L2 shares the bursts
  // between the CTAs of neighbouring column blocks
  const bool small_tensor = (double)sh.N * sh.R * sh.C * s <= 32.0 * 1024 * 1024;
  const double seg_eff = seg >= 128 ? 1.0 : seg >= 64 ? 0.95 : seg >= 32 ? (small_tensor ? 0.85 : 0.5) : 0.3;
  const double sms = (double)(p.grid < kSmCount ? p.grid : kSmCount);
  int per_sm = (int)(kSmemMaxOptin / (tile + fold + 1024));
  const int by_threads = 2048 / threads;
  if (per_sm > by_threads) per_sm = by_threads;
  const long long per_sm_by_grid = (p.grid + kSmCount - 1) / kSmCount;  // a small grid leaves SMs half empty
  if (per_sm > per_sm_by_grid) per_sm = (int)per_sm_by_grid;
  // resident warps per SM hide latency: ~24 are enough, 4 are far too few
  const int warps = per_sm * (threads / 32);
  const double occ_w = warps >= 24 ? 1.0 : warps >= 16 ? 0.93 : warps >= 12 ? 0.86 : warps >= 8 ? 0.72 : warps >= 4 ? 0.5 : 0.3;
  // ... and several CTAs per SM interleave their load / reduce / store phases
  const double occ_c = per_sm >= 6 ? 1.0 : per_sm >= 4 ? 0.96 : per_sm == 3 ? 0.92 : per_sm == 2 ? 0.85 : 0.7;
  const double occ = occ_w * occ_c;
  const int rpt = rows / TY;
  const double rpt_eff = rpt >= 16 ? 1.0 : rpt >= 8 ? 0.93 : rpt >= 4 ? 0.85 : 0.75;
  const double sync_eff = 1.0 - 0.004 * k;  // mild preference for smaller clusters
  *score = sms * seg_eff * occ * rpt_eff * sync_eff;
  *out = p;
  return true;
}

bool plan_fused(const Shape& sh, Plan* out) {
  const int ve = sh.ve;
  const long long U = (long long)sh.D / gcd_ll(sh.D, ve) * ve;  // lcm(D, ve): whole groups, whole vectors
  if (U > sh.C || sh.C % U != 0) return false;
  const int units = (int)(sh.C / U);
  const int force_cw = env_int("GNB200_CW", 0);
  const int force_k = env_int("GNB200_K", 0);
  const int force_threads = env_int("GNB200_THREADS", 0);
  const int k_max = force_k == 16 ? 16 : 8;  // 16 needs the non-portable cluster size: opt-in only
  bool found = false;
  double best = -1.0;
  for (int m = 1; m <= units; ++m) {
    if (units % m) continue;
    const long long w = U * m;
    if (w / ve > kMaxThreads) break;
    if (force_cw > 0 && w != force_cw) continue;
    for (int k = 1; k <= k_max; k *= 2) {
      if (force_k > 0 && k != force_k) continue;
      for (int threads = 128; threads <= 512; threads *= 2) {
        if (force_threads > 0 && threads != 128) continue;
        Plan cand;
        double score;
        if (!plan_fused_candidate(sh, (int)w, k, force_threads > 0 ? force_threads : threads, &cand, &score)) continue;
        if (score > best * 1.0001) {
          best = score;
          *out = cand;
          found = true;
        }
      }
    }
  }
  return found;
}

bool plan_two_pass(const Shape& sh, Plan* out) {
  const int ve = sh.ve, s = sh.s;
  const int target_threads = env_int("GNB200_THREADS", 256);
  int cw = sh.C;
  if (cw / ve > 256) cw = 256 * ve;  // last column block may be ragged
  const int force_cw = env_int("GNB200_CW", 0);
  if (force_cw > 0 && force_cw % ve == 0 && force_cw / ve <= kMaxThreads && force_cw <= sh.C) cw = force_cw;
  const int ncb = (sh.C + cw - 1) / cw;
  const int CV = cw / ve;
  int slots = (cw - 1) / sh.D + 2;
  if (slots > sh.G) slots = sh.G;

  // rows per CTA tile: large tiles amortise the per-thread set-up and the per-CTA reduction; about
  // four tiles per SM measured best for the reduce and apply kernels (up to 512 KB of x per tile),
  // and at least two tiles per SM when the problem allows
  const long long row_bytes = (long long)cw * s;
  long long tile_target = (long long)sh.N * sh.R * sh.C * s / (4LL * kSmCount);
  if (tile_target < 64 * 1024) tile_target = 64 * 1024;
  if (tile_target > 512 * 1024) tile_target = 512 * 1024;
  long long rows = (tile_target + row_bytes - 1) / row_bytes;
  if (rows > sh.R) rows = sh.R;
  const long long want_tiles = 2LL * kSmCount;
  long long chunks = (sh.R + rows - 1) / rows;
  if ((long long)sh.N * ncb * chunks < want_tiles) {
    long long need = (want_tiles + (long long)sh.N * ncb - 1) / ((long long)sh.N * ncb);
    long long min_rows = 2LL * (target_threads / CV > 0 ? target_threads / CV : 1);
    long long r2 = (sh.R + need - 1) / need;
    if (r2 < min_rows) r2 = min_rows;
    if (r2 < rows) rows = r2;
  }
  const int force_rows = env_int("GNB200_ROWS", 0);
  if (force_rows > 0) rows = force_rows;
  if (rows > sh.R) rows = sh.R;
  if (rows < 1) rows = 1;
  chunks = (sh.R + rows - 1) / rows;
  int TY, threads;
  thread_layout(CV, (int)rows, target_threads, &TY, &threads);

  Plan p = {};
  p.fused = false;
  p.wave = false;
  p.ve = ve;
  p.threads = threads;
  p.grid = (long long)sh.N * chunks * ncb;
  if (p.grid > 0x7fffffffLL) return false;
  // shared-memory rings of the streaming kernels: 4 rows x 16 bytes per thread (x; x and dy) - kRingDepth
  const size_t ring = ve > 1 ? (size_t)4 * threads * 16 : 0;
  if (sh.direction == 0) {
    p.smem_bytes = ring + fwd_fold_floats(cw, CV, TY, slots, threads, false, 0, 1) * 4;
    p.ws_bytes = (size_t)p.grid * slots * 3 * sizeof(float);
    p.launches = 3;
  } else {
    p.smem_bytes = 2 * ring + bwd_fold_floats(cw, CV, TY, slots, threads, false, 0, 1) * 4;
    p.ws_bytes = ((size_t)sh.N * chunks * sh.C * 2 + (size_t)sh.N * sh.C * 2 + (size_t)sh.N * sh.G * 2) * sizeof(float);
    p.launches = 4;
  }
  p.geom = Geom{sh.N, sh.R, sh.C, sh.G, sh.D, cw, CV, TY, ncb, (int)rows, (int)chunks, slots, 1};
  p.geom.persist = 0;
  fill_divisors(&p.geom, ve, sh.direction, threads, false);
  *out = p;
  return true;
}

// Wave plan (gn_wave.cu): one persistent cooperative kernel per direction.  Column blocks are whole
// groups and whole 16-byte vectors, at most 256 elements wide (the TMA box limit), and as wide as the
// L2 budget of a wave allows: a wave - `ipw` (sample, column block) slabs - is read twice, and the
// second read should hit L2.  GNB200_WAVE_MB overrides the budget, GNB200_WAVE_CW the width,
// GNB200_WAVE_TEAMS / _OVERLAP the number of teams and the order of the passes,
// GNB200_WAVE_STAGES / _KR / _PER_SM / _GRID the ring depth, rows per thread and stage, CTAs per SM and
// an upper bound of the grid.
bool plan_wave(const Shape& sh, Plan* out) {
  const int ve = sh.ve, s = sh.s;
  if (ve == 1) return false;  // TMA needs 16-byte aligned rows and bases
  const long long U = (long long)sh.D / gcd_ll(sh.D, ve) * ve;
  if (U > 256 || sh.C % U != 0) return false;
  if ((long long)sh.N * sh.R > 0x7fffffffLL) return false;
  const int tensors = sh.direction == 0 ? 1 : 2;  // tensors a wave keeps in L2 between its passes
  int teams_req = env_int("GNB200_WAVE_TEAMS", 2);
  if (teams_req < 1) teams_req = 1;
  if (teams_req > 3) teams_req = 3;
  // L2 budget of one wave: `teams` waves are in flight at once
  // (defaults from sweeps over the 1024-px VAE-decoder shapes on B200: two teams, overlapped order, 96 MB
  // forward / 144 MB backward in flight - somewhat more than L2 holds measured best)
  double budget = (double)env_int("GNB200_WAVE_MB", sh.direction == 0 ? 96 : 144) * 1024.0 * 1024.0 / teams_req;
  // ... and, backward, at least four waves, so that the teams' passes interleave (512@256^2: 69 us with four
  // waves of 33 MB, 79 us with two of 67 MB), as long as that does not shorten the row segments below 128 bytes
  // (the forward kernel measured better with two waves: 49 against 54 us)
  if (sh.direction == 1 && env_int("GNB200_WAVE_MB", 0) == 0) {
    const double quarter = (double)sh.N * sh.R * sh.C * s * tensors / 4.0;
    const double seg128 = (double)sh.R * 128.0 * tensors;  // a slab with 128-byte row segments
    if (quarter < budget && quarter >= seg128) budget = quarter;
  }
  const int units = (int)(sh.C / U);
  int cw = 0, cw_min64 = 0, cw_fit = 0, cw_first = 0;
  for (int m = 1; m <= units; ++m) {
    if (units % m) continue;
    const long long w = U * m;
    if (w > 256) break;
    if (!cw_first) cw_first = (int)w;
    if (!cw_min64 && w * s >= 64) cw_min64 = (int)w;
    if ((double)sh.R * w * s * tensors <= budget) cw_fit = (int)w;
  }
  cw = cw_fit;
  if (cw_min64 && cw < cw_min64) cw = cw_min64;  // rather a wave above the budget than short row segments
  if (!cw) cw = cw_first;
  const int force_cw = env_int("GNB200_WAVE_CW", 0);
  if (force_cw > 0 && force_cw % U == 0 && sh.C % force_cw == 0 && force_cw <= 256) cw = force_cw;

  WaveGeom g = {};
  g.N = sh.N, g.R = sh.R, g.C = sh.C, g.G = sh.G, g.D = sh.D;
  g.CW = cw;
  g.CV = cw / ve;
  g.ncb = sh.C / cw;
  g.slots = cw / sh.D;
  g.consumers = kWaveConsumers;
  g.KR = env_int("GNB200_WAVE_KR", sh.direction == 0 ? 4 : 2) == 2 ? 2 : 4;
  g.TY = g.consumers / g.CV;
  if (g.TY > 256 / g.KR) g.TY = 256 / g.KR;
  g.BR = g.KR * g.TY;
  g.box_bytes = g.BR * g.CW * s;
  g.stage_bytes = (g.box_bytes + 127) & ~127;
  g.stages = env_int("GNB200_WAVE_STAGES", sh.direction == 0 ? 3 : 4);
  if (g.stages < 2) g.stages = 2;
  if (g.stages > 8) g.stages = 8;
  const size_t red_floats = sh.direction == 0 ? (size_t)2 * g.consumers * ve + g.consumers + 2 * g.slots
                                              : (size_t)2 * g.consumers * ve + 2 * g.CW + 2 * g.slots;
  size_t smem = 0;
  for (;; --g.stages) {
    smem = 1024 + (size_t)g.stages * tensors * g.stage_bytes + (size_t)2 * g.stages * 8 + 16 + red_floats * 4 + 16 +
           (size_t)env_int("GNB200_WAVE_PAD", 0);
    if (smem <= kSmemMaxOptin - 1024 || g.stages == 2) break;
  }
  if (smem > kSmemMaxOptin - 1024) return false;
  int per_sm = (int)(kSmemMaxOptin / (smem + 1024));
  const int cap = sh.direction == 0 ? 3 : 2;  // the kernels' __launch_bounds__
  if (per_sm > cap) per_sm = cap;
  const int force_per_sm = env_int("GNB200_WAVE_PER_SM", 0);
  if (force_per_sm > 0 && force_per_sm < per_sm) per_sm = force_per_sm;
  long long grid = (long long)kSmCount * per_sm;

  g.items = sh.N * g.ncb;
  const double item_bytes = (double)sh.R * cw * s * tensors;
  g.teams = teams_req > per_sm ? per_sm : teams_req;
  long long ipw = (long long)(budget / item_bytes);
  if (ipw < 1) ipw = 1;
  if (ipw > g.items) ipw = g.items;
  g.waves = (int)((g.items + ipw - 1) / ipw);
  g.ipw = (g.items + g.waves - 1) / g.waves;
  g.waves = (g.items + g.ipw - 1) / g.ipw;
  if (g.teams > g.waves) g.teams = g.waves;
  const long long tgrid = grid / g.teams;  // CTAs of one team: they share a wave's units
  long long want_chunks = (tgrid + g.ipw - 1) / g.ipw;
  long long rows = (sh.R + want_chunks - 1) / want_chunks;
  rows = (rows + g.BR - 1) / g.BR * g.BR;
  g.rows_per_chunk = (int)rows;
  g.chunks = (int)((sh.R + rows - 1) / rows);
  grid = tgrid * g.teams;
  if ((long long)g.ipw * g.chunks < tgrid) grid = (long long)g.ipw * g.chunks * g.teams;
  const int force_grid = env_int("GNB200_WAVE_GRID", 0);  // tests: fewer CTAs than units, several units per CTA
  if (force_grid > 0 && force_grid < grid) grid = force_grid < g.teams ? g.teams : force_grid / g.teams * g.teams;
  g.overlap = env_int("GNB200_WAVE_OVERLAP", 1) != 0 ? 1 : 0;
  g.div_D = make_fast_div(sh.D);
  g.div_CV = make_fast_div(g.CV);
  g.div_ncb = make_fast_div(g.ncb);

  Plan p = {};
  p.fused = false;
  p.wave = true;
  p.ve = ve;
  p.threads = kWaveThreads;
  p.grid = grid;
  p.smem_bytes = smem;
  p.ws_bytes = wave_workspace_bytes(g, sh.direction);
  p.launches = 1;
  p.wgeom = g;
  // the fields of `geom` that descriptions and tests read
  p.geom = Geom{sh.N, sh.R, sh.C, sh.G, sh.D, cw, g.CV, g.TY, g.ncb, g.rows_per_chunk, g.chunks, g.slots, 1};
  *out = p;
  return true;
}

}  // namespace

static bool make_plan_inner(int64_t N, int64_t R, int64_t C, int64_t G, int dtype, int direction, bool aligned16, Plan* plan);

bool make_plan(int64_t N, int64_t R, int64_t C, int64_t G, int dtype, int direction, bool aligned16, Plan* plan) {
  if (!make_plan_inner(N, R, C, G, dtype, direction, aligned16, plan)) return false;
  // GNB200_CHAIN = 0: every kernel of a call waits for the whole previous kernel (plain stream order)
  plan->chain = chain_enabled();
  return true;
}

bool chain_enabled() { return env_int("GNB200_CHAIN", 1) != 0; }

static bool make_plan_inner(int64_t N, int64_t R, int64_t C, int64_t G, int dtype, int direction, bool aligned16, Plan* plan) {
  if (N < 1 || R < 1 || C < 1 || G < 1 || C % G != 0) return false;
  if (N > 0x7fffffffLL || R > 0x7fffffffLL || C > (1 << 24) || (long long)N * G > 0x7fffffffLL) return false;
  if ((double)N * (double)R * (double)C > 9.0e15) return false;
  Shape sh;
  sh.N = (int)N;
  sh.R = (int)R;
  sh.C = (int)C;
  sh.G = (int)G;
  sh.D = (int)(C / G);
  sh.s = dtype == 0 ? 4 : 2;
  const int vfull = 16 / sh.s;
  sh.ve = (aligned16 && C % vfull == 0) ? vfull : 1;
  sh.direction = direction;
  // GNB200_FORCE_PATH = twopass: the multi-kernel plan; wave: the wave plan where the shape allows it
  const char* force = getenv("GNB200_FORCE_PATH");
  const bool twopass_only = force && !strcmp(force, "twopass");
  const bool skip_fused = twopass_only || (force && !strcmp(force, "wave"));
  if (!skip_fused && plan_fused(sh, plan)) return true;
  if (force && !strcmp(force, "wave")) {
    if (plan_wave(sh, plan)) return true;
  } else if (!twopass_only && sh.direction == 1) {
    // Measured on B200 (1024-px VAE-decoder shapes, fp16 SiLU): the wave plan beats the multi-kernel plan
    // in the backward direction when its row segments are at least 128 bytes (512@256^2: 70 vs 82 us,
    // 256@512^2: 130 vs 141 us) and loses with 64-byte segments (128@1024^2: 255 vs 243 us) and in the
    // forward direction (49 vs 44, 85 vs 78, 182 vs 148 us), where it saves the third pass over the tensor
    // but pays more for its waves' synchronisation than that pass costs.
    Plan w;
    if (plan_wave(sh, &w) && (long long)w.wgeom.CW * sh.s >= 128) {
      *plan = w;
      return true;
    }
  }
  return plan_two_pass(sh, plan);
}

cudaError_t ensure_kernel_attributes(const void* func, size_t smem_bytes, bool nonportable_cluster) {
  static std::mutex mu;
  static std::map<std::pair<int, const void*>, std::pair<size_t, bool>> done;
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return err;
  std::lock_guard<std::mutex> lock(mu);
  auto& st = done[std::make_pair(dev, func)];
  if (smem_bytes > 48 * 1024 && smem_bytes > st.first) {
    // the opt-in limit covers the kernel's static shared memory too
    cudaFuncAttributes fa;
    err = cudaFuncGetAttributes(&fa, func);
    if (err != cudaSuccess) return err;
    const size_t room = kSmemMaxOptin - fa.sharedSizeBytes;
    err = cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)room);
    if (err != cudaSuccess) return err;
    st.first = room;
  }
  if (nonportable_cluster && !st.second) {
    err = cudaFuncSetAttribute(func, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    if (err != cudaSuccess) return err;
    st.second = true;
  }
  return cudaSuccess;
}

cudaError_t resident_clusters(const void* func, const cudaLaunchConfig_t* cfg, int* clusters) {
  struct Key {
    int dev;
    const void* func;
    unsigned threads, k;
    size_t smem;
    bool operator<(const Key& o) const {
      if (dev != o.dev) return dev < o.dev;
      if (func != o.func) return func < o.func;
      if (threads != o.threads) return threads < o.threads;
      if (k != o.k) return k < o.k;
      return smem < o.smem;
    }
  };
  static std::mutex mu;
  static std::map<Key, int> cache;
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return err;
  unsigned k = 1;
  for (unsigned i = 0; i < cfg->numAttrs; ++i)
    if (cfg->attrs[i].id == cudaLaunchAttributeClusterDimension) k = cfg->attrs[i].val.clusterDim.x;
  const Key key = {dev, func, cfg->blockDim.x, k, cfg->dynamicSmemBytes};
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it == cache.end()) {
    // the query wants a grid that is a multiple of the cluster size; the answer does not depend on it
    cudaLaunchConfig_t q = *cfg;
    q.gridDim = dim3(k, 1, 1);
    int n = 0;
    err = cudaOccupancyMaxActiveClusters(&n, func, &q);
    if (err != cudaSuccess) return err;
    if (n < 1) n = 1;
    it = cache.emplace(key, n).first;
  }
  *clusters = it->second;
  return cudaSuccess;
}

size_t plan_workspace_bytes(int64_t N, int64_t R, int64_t C, int64_t G, int dtype, int direction) {
  size_t best = 0;
  for (int aligned = 0; aligned < 2; ++aligned) {
    Plan p;
    if (make_plan(N, R, C, G, dtype, direction, aligned != 0, &p) && p.ws_bytes > best) best = p.ws_bytes;
  }
  return best;
}

}  // namespace gnb200
