// Device-side pieces shared by the two sparse exchange kernels (K2: gTop-k tree,
// K2t: Top-k all-gather): the per-rank descriptor, peer pushes with flags, the
// direct-address merge of two sparse sets, and the residual put-back.
//
// Merging without sorting: each rank owns an int32 table `map` of d entries.
// To join set A (n_a entries) with set B, A first writes map[A[i].idx] = i; an
// entry (j, v) of B is shared iff p = map[j] satisfies p < n_a && A[p].idx == j.
// The second test makes stale table contents harmless, so the table is never
// cleared.
#pragma once
#include "select_common.cuh"
#include "host_api.h"

namespace gtk {

// Layout of the symmetric (peer-visible) region of one rank, identical on all
// ranks.  Two parities (epoch & 1) so that a fast sender of call e+1 never
// overwrites what a slow reader of call e still needs.
//   slots : [2][kMaxRounds][kcap] pairs   receive slot of each tree round
//   ag    : [2][kMaxPeers][kcap] pairs    all-gather slots, one per source rank (K2t only)
//   gout  : [2][kcap] pairs               the global top-k set
//   flags : [2][kFlagsPerParity] u64      (epoch << 32) | count
constexpr int kFlagBcast = kMaxRounds;             // flag index of the broadcast
constexpr int kFlagAg0 = kMaxRounds + 1;           // first all-gather flag (one per source)
constexpr int kFlagsPerParity = kMaxRounds + 1 + kMaxPeers;

struct K2Rank {
  const Pair* sel;        // local selection written by K1
  const K1State* st;      // st->n_sel = number of local pairs
  Pair* work[2];          // [kcap_work] ping-pong merge buffers
  int32_t* map;           // [d] direct-address table
  float* resid;           // [d] residual
  Pair* slots;            // local symmetric buffers
  Pair* ag;
  Pair* gout;
  uint64_t* flags;
  Ctrl* ctrl;             // TWO control blocks.  K2 uses block (call & 1) and cleans the other one itself;
                          // K2t uses block 0, cleared by the host before every launch
  unsigned int* n_global; // kResWords device words: result of the last call, see kRes* below
  unsigned int* epoch;    // device word: call counter (starts at 1); the kernel reads it at entry and
                          // adds one after its last barrier, so a replayed CUDA graph needs no new argument
  Pair* peer_slots[kMaxPeers];
  Pair* peer_ag[kMaxPeers];
  Pair* peer_gout[kMaxPeers];
  uint64_t* peer_flags[kMaxPeers];
};

// Result words of an exchange (K2Rank::n_global).  kResCount is what the consumer (K3) reads: the
// number of pairs in gout[parity], 0 after a failed call.  The other three are written once, by
// the first failing call, and never cleared by a kernel: while kResStatus is non-zero every later
// call returns at once with an empty result.
constexpr int kResCount = 0;
constexpr int kResStatus = 1;
constexpr int kResWhere = 2;
constexpr int kResEpoch = 3;
constexpr int kResWords = 4;

struct ExchangeShared {
  SelectShared sel;
  unsigned int payload;
  int ok;
};

__device__ __forceinline__ size_t slot_off(unsigned int parity, unsigned int round,
                                           unsigned int kcap) {
  return ((size_t)parity * kMaxRounds + round) * kcap;
}
__device__ __forceinline__ size_t ag_off(unsigned int parity, unsigned int src, unsigned int kcap) {
  return ((size_t)parity * kMaxPeers + src) * kcap;
}
__device__ __forceinline__ size_t flag_off(unsigned int parity, unsigned int which) {
  return (size_t)parity * kFlagsPerParity + which;
}

// All CTAs of the rank copy n pairs to dst (peer or local memory).  The caller
// then calls cta_fence_peer_stores(), passes the rank barrier, and one thread
// publishes the data with release_flag().
__device__ __forceinline__ void push_pairs(Pair* dst, const Pair* src, unsigned int n,
                                           unsigned int cta, unsigned int nct) {
  const unsigned int stride = nct * kSelThreads;
  for (unsigned int i = cta * kSelThreads + threadIdx.x; i < n; i += stride)
    st_pair(&dst[i], ld_pair_cg(&src[i]));
}

// Called by all threads of a CTA of a multi-CTA rank after its last store into peer memory of a phase
// and before the rank's barrier: one thread issues a system-scope fence on behalf of the CTA (the
// __syncthreads orders the other threads' stores before it).  By the PTX memory model the flag's own
// st.release.sys, issued after the rank's barrier, already covers these stores (the barrier is a
// morally strong synchronisation and release is cumulative); the fence makes each SM wait for the
// acknowledgement of its own NVLink stores instead of leaving that to one SM's release on behalf of
// all, which is the form library collectives use (one fencing thread per CTA that stored).  A rank
// served by a single CTA needs no extra fence: the thread that raises the flag sits in the CTA that
// stored.  Cost: 2-3 us per sending phase.
__device__ __forceinline__ void cta_fence_peer_stores(bool single_cta) {
  if (single_cta) return;
  __syncthreads();
  if (threadIdx.x == 0) __threadfence_system();
}

// Publish: st.release.sys orders every store that happens-before it (this
// thread's own and, through the preceding barrier, every other thread's).
__device__ __forceinline__ void release_flag(uint64_t* flag, uint32_t epoch, uint32_t count) {
  st_release_sys_u64(flag, ((uint64_t)epoch << 32) | (uint64_t)count);
}

// One thread per CTA waits for the flag, the CTA learns the count.
__device__ __forceinline__ bool cta_wait_flag(ExchangeShared& sh, const uint64_t* flag,
                                              uint32_t epoch, Ctrl* ctrl, uint64_t limit_ns,
                                              uint32_t where, unsigned int* count) {
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t payload = 0;
    sh.ok = wait_flag(flag, epoch, ctrl, limit_ns, where, &payload) ? 1 : 0;
    sh.payload = payload;
  }
  __syncthreads();
  *count = sh.payload;
  return sh.ok != 0;
}

// A <- copy of src, and map[idx] = position.
__device__ __forceinline__ void copy_and_map(Pair* A, const Pair* src, unsigned int n, int32_t* map,
                                             unsigned int d, unsigned int cta, unsigned int nct,
                                             Ctrl* ctrl) {
  const unsigned int stride = nct * kSelThreads;
  for (unsigned int i = cta * kSelThreads + threadIdx.x; i < n; i += stride) {
    const Pair e = ld_pair_cg(&src[i]);
    st_pair(&A[i], e);
    if ((unsigned int)e.idx < d) map[e.idx] = (int32_t)i;
    else record_error(ctrl, ST_BOUNDS, 300);
  }
}

__device__ __forceinline__ void build_map(const Pair* A, unsigned int n, int32_t* map,
                                          unsigned int d, unsigned int cta, unsigned int nct,
                                          Ctrl* ctrl) {
  const unsigned int stride = nct * kSelThreads;
  for (unsigned int i = cta * kSelThreads + threadIdx.x; i < n; i += stride) {
    const Pair e = ld_pair_cg(&A[i]);
    if ((unsigned int)e.idx < d) map[e.idx] = (int32_t)i;
    else record_error(ctrl, ST_BOUNDS, 301);
  }
}

// Shared indices: A[p].val += B[j].val and B[j] is marked dead (idx = -1).
// B lives in local memory.  Indices are unique inside A and inside B, so every
// A[p] is touched by at most one thread.
__device__ __forceinline__ void probe_merge(Pair* A, unsigned int n_a, Pair* B, unsigned int n_b,
                                            const int32_t* map, unsigned int d, unsigned int cta,
                                            unsigned int nct, Ctrl* ctrl) {
  const unsigned int stride = nct * kSelThreads;
  for (unsigned int j = cta * kSelThreads + threadIdx.x; j < n_b; j += stride) {
    const Pair e = ld_pair_cg(&B[j]);
    if ((unsigned int)e.idx >= d) {
      record_error(ctrl, ST_BOUNDS, 302);
      B[j].idx = -1;
      continue;
    }
    const unsigned int p = (unsigned int)__ldcg(&map[e.idx]);
    if (p < n_a) {
      const Pair a = ld_pair_cg(&A[p]);
      if (a.idx == e.idx) {
        A[p].val = a.val + e.val;
        B[j].idx = -1;
      }
    }
  }
}

// Residual put-back (compression.py:66-75 in the reference): every locally
// selected entry whose index is not in the global set returns to the residual.
// Requires map[] built over G.
__device__ __forceinline__ void put_back(const Pair* sel, unsigned int n_sel, const Pair* G,
                                         unsigned int n_g, const int32_t* map, float* resid,
                                         unsigned int d, unsigned int cta, unsigned int nct) {
  const unsigned int stride = nct * kSelThreads;
  for (unsigned int i = cta * kSelThreads + threadIdx.x; i < n_sel; i += stride) {
    const Pair e = sel[i];
    if ((unsigned int)e.idx >= d) continue;
    const unsigned int p = (unsigned int)__ldcg(&map[e.idx]);
    bool in_global = false;
    if (p < n_g) in_global = ld_pair_cg(&G[p]).idx == e.idx;
    if (!in_global) resid[e.idx] += e.val;
  }
}

}  // namespace gtk
