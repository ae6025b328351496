// All-reduce of the packed fp32 [dgamma | dbeta] buffer over the GPUs of one node, done by the
// library's own kernels over peer-mapped memory: no library collective, no multicast object.
//
//   push     every rank stores its 2 * C floats into its slot of EVERY rank's exchange buffer (plain
//            stores through peer-mapped pointers, NVLink), each stamped with the number of the push.
//            This happens inside the kernel that produces the gradients and waits for nobody (but
//            see "slot reuse" below).
//   collect  a rank waits - bounded - until the values of all ranks with the expected number stand in
//            its OWN buffer, adds them in rank order (so every rank gets the same bits) and
//            acknowledges.  It can run right after the push in the same kernel (one call, one NVLink
//            crossing of latency) or as a kernel of its own much later, e.g. before the optimizer
//            step, when every contribution has long arrived and the ranks need not be in step during
//            the backward pass.
//
// The reference has no multi-GPU code; this replaces the NCCL all-reduce of the data-parallel
// extension (2 KB for C = 256: pure latency).
//
// Exchange buffer of one rank (same layout on every rank; `world` ranks, nblk = ceil(C / 32) blocks):
//   uint2    slot[2][world][2 * C]    slot[p][q][i] = (bits of rank q's float i, number of the push), parity p
//   unsigned ack[world][nblk]         ack[q][b] = number of the last call whose block b rank q has collected
//   unsigned pushed[nblk]             this rank's push counter per block        (the last four arrays are
//   unsigned collected[nblk]          this rank's collect counter per block      never written by peers)
//   unsigned done[nblk]               number of the last collect that has finished reading its slots
//   unsigned acked[nblk]              number of the last collect this rank has acknowledged to the peers
// The buffer must be zero before the first call.  Pushes and collects are numbered per block, 1, 2, ...
// Every value travels with the number of its push in ONE 8-byte store, which arrives whole: a reader that
// sees the number sees the value, so neither side needs a fence or a separate flag on the way in (the
// scheme of low-latency collectives).  Slot reuse: push s overwrites the slots of push s - 2, so it first
// waits (bounded; in practice never) until every rank has acknowledged collect s - 2.  A collect only
// notes locally (release, GPU scope) that it has read its slots; the word goes to the peers at the
// start of the rank's NEXT push as a plain store - a system-scope release at the end of
// the collect would wait about 2 us for this kernel's own stores to the peers to be confirmed, on the
// critical path of every call.  The loads being acknowledged belong to an earlier kernel, or precede a
// GPU-scope acquire of `done` in program order: they have returned their values before the store issues.
// (A collect that is never followed by a push needs no acknowledgement.)  Every rank must make the same
// sequence of pushes and collects; a buffer set serves 2^32 - 1 of them (the numbers are 32-bit and 0 means "never written").
#pragma once
#include "gn_common.cuh"

namespace gnb200 {

constexpr int kMaxPeers = 16;
constexpr int kPeerBlock = 32;  // channels per exchange block (one warp)

struct PeerExchange {
  int world;  // <= 1: no exchange
  int rank;
  int C;
  int nblk;
  int collect;            // 1: the pushing kernel also collects (all-reduce in one call); 0: push only
  char* base[kMaxPeers];  // exchange buffer of rank q as mapped into this GPU's address space
  WaitLimit wait;
};

__host__ __device__ inline size_t peer_slot_words(int world, int C) { return (size_t)2 * world * 2 * C; }  // 8 bytes each
__host__ __device__ inline size_t peer_exchange_bytes(int world, int C) {
  const int nblk = (C + kPeerBlock - 1) / kPeerBlock;
  const size_t words = (size_t)world * nblk + 4 * (size_t)nblk;
  return (peer_slot_words(world, C) * 8 + words * sizeof(unsigned) + 255) & ~(size_t)255;
}

// Word arrays of the exchange buffer at `base`
struct PeerWords {
  unsigned *ack, *pushed, *collected, *done, *acked;
};
__device__ __forceinline__ PeerWords peer_words(char* base, int world, int C, int nblk) {
  PeerWords w;
  w.ack = reinterpret_cast<unsigned*>(base + peer_slot_words(world, C) * 8);
  w.pushed = w.ack + (size_t)world * nblk;
  w.collected = w.pushed + nblk;
  w.done = w.collected + nblk;
  w.acked = w.done + nblk;
  return w;
}

__device__ __forceinline__ void st_release_sys_u32(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_relaxed_sys_u32(unsigned* p, unsigned v) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_release_gpu_u32(unsigned* p, unsigned v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_gpu_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_relaxed_sys_v2(uint2* p, unsigned a, unsigned b) {
  asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(a), "r"(b) : "memory");
}
__device__ __forceinline__ uint2 ld_relaxed_sys_v2(const uint2* p) {
  uint2 v;
  asm volatile("ld.relaxed.sys.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
  return v;
}

// Lanes q < world poll word[q * stride] until it has reached `want` (numbers only grow; the
// comparison tolerates wrap-around).  Returns false in every lane if any wait gave up.
__device__ __forceinline__ bool peer_wait_words(const unsigned* word, size_t stride, unsigned want, int world,
                                                const WaitLimit& lim) {
  const int lane = threadIdx.x & 31;
  bool ok = true;
  if (lane < world) {
    const unsigned* f = word + (size_t)lane * stride;
    if ((int)(ld_acquire_sys_u32(f) - want) < 0) {
      const long long t0 = clock64();
      unsigned polls = 0;
      while ((int)(ld_acquire_sys_u32(f) - want) < 0) {
        if (++polls > lim.polls && clock64() - t0 > lim.clocks) {
          ok = false;
          break;
        }
        __nanosleep(32);
      }
    }
  }
  ok = __all_sync(0xffffffffu, ok);
  if (!ok && lane == 0) wait_gave_up(lim);
  return ok;
}

// First half of a push, by one full warp: numbers the push, passes this rank's acknowledgement on and
// looks once whether the slots are free.  It touches nothing but the exchange buffers, so a kernel
// calls it before it waits for the values it is going to push.
struct PeerPush {
  unsigned seq;
  bool ready;  // every rank has acknowledged push seq - 2
};
__device__ __forceinline__ PeerPush peer_push_begin(const PeerExchange& px, int blk) {
  const int lane = threadIdx.x & 31;
  const int world = px.world, C = px.C, nblk = px.nblk;
  const PeerWords mine = peer_words(px.base[px.rank], world, C, nblk);
  unsigned seq = 0, fin = 0, ack = 0;
  if (lane == 0) {
    seq = mine.pushed[blk] + 1;
    fin = ld_acquire_gpu_u32(mine.done + blk);  // collects that have read their slots (possibly on another stream)
    ack = mine.acked[blk];
    mine.pushed[blk] = seq;
    mine.acked[blk] = fin;
  }
  seq = __shfl_sync(0xffffffffu, seq, 0);
  fin = __shfl_sync(0xffffffffu, fin, 0);
  ack = __shfl_sync(0xffffffffu, ack, 0);
  // first, which of the peers' slots this rank has finished reading (before any wait: every rank may be
  // waiting for exactly this word)
  if (fin != ack && lane < world) {
    const PeerWords theirs = peer_words(px.base[lane], world, C, nblk);
    st_relaxed_sys_u32(theirs.ack + (size_t)px.rank * nblk + blk, fin);
  }
  // the slots of push seq - 2 are free once every rank has collected it
  bool free_now = true;
  if (seq > 2 && lane < world) free_now = (int)(ld_acquire_sys_u32(mine.ack + (size_t)lane * nblk + blk) - (seq - 2)) >= 0;
  PeerPush pp;
  pp.seq = seq;
  pp.ready = __all_sync(0xffffffffu, free_now);
  return pp;
}

// Second half: lane l holds (dg, db) of channel blk * 32 + l (`valid`: the channel exists).  Returns
// false if the wait for the slots to become free gave up (nothing is stored then: the peers' collect
// of this call will give up too, and report it).
__device__ __forceinline__ bool peer_push_block(const PeerExchange& px, int blk, bool valid, float dg, float db,
                                                const PeerPush& pp) {
  const int lane = threadIdx.x & 31;
  const int world = px.world, C = px.C, nblk = px.nblk;
  const PeerWords mine = peer_words(px.base[px.rank], world, C, nblk);
  const unsigned seq = pp.seq, par = seq & 1u;
  if (!pp.ready && !peer_wait_words(mine.ack + blk, (size_t)nblk, seq - 2, world, px.wait)) return false;
  const int c = blk * kPeerBlock + lane;
  if (valid) {
    for (int q = 0; q < world; ++q) {  // my slot [par][rank] in every rank's buffer (my own included)
      uint2* slot = reinterpret_cast<uint2*>(px.base[q]) + ((size_t)par * world + px.rank) * 2 * C;
      st_relaxed_sys_v2(slot + c, __float_as_uint(dg), seq);
      st_relaxed_sys_v2(slot + C + c, __float_as_uint(db), seq);
    }
  }
  return true;
}

// Collect of one block by one full warp: dg, db become the sums over all ranks (NaN after a wait
// that gave up), in rank order.  kBatch: ranks whose values are requested together (independent
// loads; 16 registers per 4 ranks).
template <int kBatch = 4>
__device__ __forceinline__ void peer_collect_block(const PeerExchange& px, int blk, bool valid, float& dg, float& db) {
  const int lane = threadIdx.x & 31;
  const int world = px.world, C = px.C, nblk = px.nblk;
  const PeerWords mine = peer_words(px.base[px.rank], world, C, nblk);
  unsigned seq = 0;
  if (lane == 0) {
    seq = mine.collected[blk] + 1;
    mine.collected[blk] = seq;
  }
  seq = __shfl_sync(0xffffffffu, seq, 0);
  const unsigned par = seq & 1u;
  const int c = blk * kPeerBlock + lane;
  const uint2* slots = reinterpret_cast<const uint2*>(px.base[px.rank]) + (size_t)par * world * 2 * C;
  float sg = 0.f, sb = 0.f;
  bool ok = true;
  if (valid) {
    const long long t0 = clock64();
    unsigned polls = 0;
    for (int q0 = 0; q0 < world && ok; q0 += kBatch) {
      uint2 vg[kBatch], vb[kBatch];
#pragma unroll
      for (int j = 0; j < kBatch; ++j) {
        if (q0 + j < world) {
          const uint2* pg = slots + (size_t)(q0 + j) * 2 * C + c;
          vg[j] = ld_relaxed_sys_v2(pg);
          vb[j] = ld_relaxed_sys_v2(pg + C);
        }
      }
#pragma unroll
      for (int j = 0; j < kBatch; ++j) {  // rank order: the same bits on every rank
        if (q0 + j < world && ok) {
          const uint2* pg = slots + (size_t)(q0 + j) * 2 * C + c;
          while (vg[j].y != seq || vb[j].y != seq) {  // each value arrives together with its number
            if (++polls > px.wait.polls && clock64() - t0 > px.wait.clocks) {
              ok = false;
              break;
            }
            __nanosleep(32);
            vg[j] = ld_relaxed_sys_v2(pg);
            vb[j] = ld_relaxed_sys_v2(pg + C);
          }
          sg += __uint_as_float(vg[j].x);
          sb += __uint_as_float(vb[j].x);
        }
      }
    }
  }
  ok = __all_sync(0xffffffffu, ok);
  if (!ok) {
    if (lane == 0) wait_gave_up(px.wait);
    sg = sb = __int_as_float(0x7fc00000);
  }
  dg = sg;
  db = sb;
  // Note that the slots have been read (also after a give-up, so that the peers' pushes are not held
  // up): the loads above come before the barrier in every lane's program order, the release after it.
  // This rank's next push passes the number on to the peers.
  __syncwarp();
  if (lane == 0) st_release_gpu_u32(mine.done + blk, seq);
}

}  // namespace gnb200
