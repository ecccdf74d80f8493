// Exchange of output slices between the GPUs of a tensor-parallel group, done inside the producing
// and consuming kernels over peer-mapped memory (plain NVLink stores, local loads; no multicast,
// no fences, no separate flags).
//
// Protocol ("stamped words"). Every 32-bit word that crosses GPUs travels as an 8-byte pair
// {word, stamp}, written with ONE 8-byte store, so a reader that sees the expected stamp also sees
// the word that was written with it. A decode step has a fixed list of exchange points numbered
// seq = 0, 1, ...; the stamp of exchange point seq in step `epoch` is epoch * kPeerMaxSeq + seq + 1
// (never 0, the value of a fresh buffer), where epoch is a device counter that every rank advances
// once per step, so a replayed CUDA graph needs no host-side argument changes. A producer stores its
// slice as stamped pairs into the destination buffer of every rank, its own included; a consumer
// re-reads the pairs it needs from its own buffer (bypassing L1) until every stamp matches.
//
// A destination buffer may be reused by a later exchange point only if every rank must have
// consumed the earlier contents before any rank can reach the later producer; the decode step's
// order of exchange points guarantees that (each rank needs every other rank's slice at each point).
//
// Every poll loop is bounded by a wall-clock deadline; on expiry the kernel records kErrPeerWait
// and carries on with what it has (the step's result is then wrong and the host sees the error
// code), and once an error is recorded later waits give up at once.
#pragma once
#include "fq_common.cuh"

namespace fq {

constexpr int kPeerMaxWorld = 8;
constexpr int kPeerMaxSeq = 1024;

struct PeerCtx {
  int world, rank;
  int wait_seq;            // exchange point whose data this kernel consumes, or -1
  int push_seq;            // exchange point this kernel produces, or -1
  const uint32_t* epoch;   // local step counter
  unsigned long long wait_ns;  // deadline of every poll loop (FUELQ_OPT_PEER_WAIT_MS)
};

__device__ __forceinline__ uint32_t peer_stamp(const PeerCtx& c, int seq) {
  return *reinterpret_cast<const volatile uint32_t*>(c.epoch) * (uint32_t)kPeerMaxSeq + (uint32_t)seq + 1u;
}

__device__ __forceinline__ void st_pair(uint2* p, uint32_t word, uint32_t stamp) {
  asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(word), "r"(stamp) : "memory");
}
__device__ __forceinline__ uint2 ld_pair(const uint2* p) {
  uint2 v;
  asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}
// two adjacent pairs (16-byte aligned); each 8-byte half is consistent on its own
__device__ __forceinline__ uint4 ld_pair2(const uint2* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

__device__ __forceinline__ unsigned long long peer_now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Bounded retry bookkeeping for one thread's poll loop.
struct PeerPoll {
  unsigned long long t0 = 0, limit_ns;
  uint32_t i = 0;
  __device__ __forceinline__ explicit PeerPoll(unsigned long long limit) : limit_ns(limit) {}
  // call after a failed attempt; false = give up (error recorded or already present)
  __device__ __forceinline__ bool again() {
    if (i == 0) t0 = peer_now_ns();
    ++i;
    if (*reinterpret_cast<volatile int*>(&g_fq_dev_error) != 0) return false;
    if (i > 16) __nanosleep(i < 256 ? 64 : 512);
    if ((i & 63u) == 0u && peer_now_ns() - t0 > limit_ns) {
      record_dev_error(kErrPeerWait);
      return false;
    }
    return true;
  }
};

// All loads of an attempt are issued before any stamp is looked at, so an attempt costs one memory round
// trip; the stamps are checked with plain ALU operations (no short-circuit) for the same reason.
//
// NA + NB words (both even, sources 16-byte aligned) from two places of stamped buffers, polling until all
// stamps match.
template <int NA, int NB>
__device__ __forceinline__ void peer_load_words2(const uint2* srca, const uint2* srcb, uint32_t want, uint32_t (&outa)[NA],
                                                 uint32_t (&outb)[NB == 0 ? 2 : NB], unsigned long long limit_ns) {
  static_assert(NA % 2 == 0 && NB % 2 == 0, "pairs are read two at a time");
  PeerPoll poll(limit_ns);
  for (;;) {
    uint4 va[NA / 2], vb[NB == 0 ? 1 : NB / 2];
#pragma unroll
    for (int j = 0; j < NA / 2; ++j) va[j] = ld_pair2(srca + 2 * j);
#pragma unroll
    for (int j = 0; j < NB / 2; ++j) vb[j] = ld_pair2(srcb + 2 * j);
    uint32_t bad = 0;
#pragma unroll
    for (int j = 0; j < NA / 2; ++j) {
      outa[2 * j] = va[j].x, outa[2 * j + 1] = va[j].z;
      bad |= (va[j].y ^ want) | (va[j].w ^ want);
    }
#pragma unroll
    for (int j = 0; j < NB / 2; ++j) {
      outb[2 * j] = vb[j].x, outb[2 * j + 1] = vb[j].z;
      bad |= (vb[j].y ^ want) | (vb[j].w ^ want);
    }
    if (bad == 0 || !poll.again()) return;
  }
}
template <int NW>
__device__ __forceinline__ void peer_load_words(const uint2* src, uint32_t want, uint32_t (&out)[NW], unsigned long long limit_ns) {
  uint32_t none[2];
  peer_load_words2<NW, 0>(src, src, want, out, none, limit_ns);
}

}  // namespace fq
