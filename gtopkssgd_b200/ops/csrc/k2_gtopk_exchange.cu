// K2: the gTop-k recursive-doubling exchange as one persistent kernel.
//
// Semantics of gtopk_sparse_allreduce in the reference (allreducer.py:71-163):
// log2(P) rounds; in round r rank i + 2^r sends its k pairs to rank i for every
// i = 0 (mod 2^(r+1)); the receiver sums values on shared indices and keeps the k
// largest magnitudes of the union; rank 0 ends with the global set and
// broadcasts it; every rank returns "selected locally but not globally" values
// to its residual (compression.py:66-75).
//
// Here every transfer is a plain NVLink peer store into the partner's receive
// slot followed by a release store of an epoch-stamped flag in the partner's
// memory; a receiver polls only its own memory.  No MPI, no NCCL, no host
// staging, no per-round barrier between ranks.
//
// One launch serves gridDim.y ranks: 1 in production (one process per GPU), P
// when all ranks are emulated on one GPU for testing, in which case the launch
// is cooperative so that all CTAs are co-resident and the flag waits make
// progress.  gridDim.x CTAs serve each rank and meet in RankBarrier.
//
// A merged set is compacted straight to where the next phase reads it: into the
// partner's receive slot when this rank sends in the next round, into every
// rank's global-set buffer after the last round (rank 0), into the local work
// buffer otherwise.  So only round 0 has a separate push, and there is no
// separate broadcast copy.
//
// No host-side clearing: the rank owns two control blocks; call e uses block
// (e & 1) and zeroes the other one for call e + 1 once its own work is done.
//
// Failure: any wait that runs out, any capacity or bounds error makes the call
// publish an EMPTY global set (n_global = 0, so the consumer applies nothing) and
// a sticky status in the result words; the call counter is not advanced and every
// later call returns at once with an empty set until the host has rebuilt the
// exchange.
#include <cstddef>
#include "exchange_common.cuh"

namespace gtk {

// kK2Cache = union entries each thread keeps in registers across the phases of a round (template
// parameter of the kernel: 4 by default, 8 when a 16-CTA cluster serves up to 64 K union entries).

constexpr int kK2Pred = 3;  // second-digit histograms are built on the fly for this many predicted first digits

struct K2Shared {
  ExchangeShared ex;
  unsigned int hist0[kHistBins];  // this CTA's share of the first-digit histogram, built on the fly
  unsigned int hist1[kK2Pred][1024];  // second digit of the entries whose first digit is pred, pred+1, pred+2
  unsigned int cursor;            // single-CTA ranks: output cursor and tie tickets of the current round
  unsigned int tie;               // live here instead of in global memory (two round trips less per round)
};

__device__ __forceinline__ void hist0_clear(K2Shared& sh) {
  for (int i = threadIdx.x; i < kHistBins; i += kSelThreads) sh.hist0[i] = 0u;
  for (int i = threadIdx.x; i < kK2Pred * 1024; i += kSelThreads) (&sh.hist1[0][0])[i] = 0u;
  __syncthreads();
}
// Global home of the second-digit histogram of predicted first digit pred + off, inside one round's set.
__device__ __forceinline__ unsigned int* pred_row(unsigned int (*set)[kHistBins], unsigned int off) {
  return off < 2u ? set[1] + off * 1024u : set[2];
}
// Adds this CTA's (possibly "negative", i.e. wrapped) partial counts to a round's global histograms
// (first digit, and second digit for the predicted first digits) and zeroes the shared copies.
__device__ __forceinline__ void hist0_flush(K2Shared& sh, unsigned int (*set)[kHistBins]) {
  __syncthreads();
  for (int i = threadIdx.x; i < kHistBins; i += kSelThreads) {
    const unsigned int c = sh.hist0[i];
    if (c) atomicAdd(&set[0][i], c);
    sh.hist0[i] = 0u;
  }
  for (int i = threadIdx.x; i < kK2Pred * 1024; i += kSelThreads) {
    const unsigned int c = sh.hist1[i >> 10][i & 1023];
    if (c) atomicAdd(&pred_row(set, (unsigned int)i >> 10)[i & 1023], c);
    sh.hist1[i >> 10][i & 1023] = 0u;
  }
  __syncthreads();
}

template <int kK2Cache>
__global__ void __launch_bounds__(kSelThreads, 1)
k2_gtopk_exchange(const K2Rank* __restrict__ ranks, unsigned int rank_base, unsigned int P,
                  unsigned int k, unsigned int kcap, unsigned int d, unsigned long long limit_ns,
                  int use_cluster) {
  __shared__ K2Shared sh;
  SelectShared& ss = sh.ex.sel;
  const K2Rank& R = ranks[blockIdx.y];
  const unsigned int epoch = __ldcg(R.epoch);  // every CTA reads it before its first barrier
  const unsigned int me = rank_base + blockIdx.y;
  const unsigned int cta = blockIdx.x, nct = gridDim.x;
  const unsigned int parity = epoch & 1u;
  const unsigned int stride = nct * kSelThreads;
  const unsigned int lane0 = cta * kSelThreads + threadIdx.x;  // union index of this thread's trip 0
  const bool single = nct == 1;  // the whole rank is this CTA: histograms never leave shared memory
  Ctrl* ctrl = R.ctrl + parity;
  int32_t* const map = R.map;
  RankBarrier bar{ctrl, nct, 0u, limit_ns, nullptr, use_cluster != 0};
  // Leaves an empty result and the sticky status behind; called by every CTA that gives up.
  auto fail = [&]() {
    if (threadIdx.x == 0) {
      atomicExch(&R.n_global[kResCount], 0u);
      unsigned int st = ld_relaxed_gpu_u32(&ctrl->status);
      if (st == 0u) st = ST_TIMEOUT_BARRIER;  // left because another CTA of the rank did
      if (atomicCAS(&R.n_global[kResStatus], 0u, st) == 0u) {
        R.n_global[kResWhere] = ld_relaxed_gpu_u32(&ctrl->where);
        R.n_global[kResEpoch] = epoch;
      }
    }
  };
  if (__ldcg(&R.n_global[kResStatus]) != 0u) {  // an earlier call failed: nothing is exchanged any more
    if (cta == 0 && threadIdx.x == 0) R.n_global[kResCount] = 0u;
    return;
  }

  unsigned int n_sel = R.st->n_sel;
  if (n_sel > kcap) n_sel = kcap;
  const Pair* cur = R.sel;  // current set of this rank
  unsigned int n_cur = n_sel;
  int cur_buf = -1;         // -1: cur is the read-only selection of K1; else index of the work buffer

  unsigned int rounds = 0;
  while ((1u << rounds) < P) ++rounds;
  hist0_clear(sh);
  trace_stamp(ctrl, 0);
  // Every live entry of a round's union is counted once by its first radix digit and, if that digit is
  // pred0, pred0 + 1 or pred0 + 2, by its second digit as well (delta = 1 adds, 0xffffffff removes).  The
  // union's k-th magnitude is at least this rank's own, and for heavy-tailed gradients about one first
  // digit (a factor 2^(1/8)) above it, so the re-select usually finds both digits without a sweep.
  unsigned int pred0 = mag_key(R.st->kth_mag) >> 20;  // round 0: first digit of K1's k-th magnitude
  auto tally = [&](float v, unsigned int delta) {
    const uint32_t key = mag_key(v);
    const unsigned int fd = key >> 20;
    atomicAdd(&sh.hist0[fd], delta);
    const unsigned int off = fd - pred0;  // wraps for fd < pred0
    if (off < (unsigned int)kK2Pred) atomicAdd(&sh.hist1[off][(key >> 10) & 1023u], delta);
  };

  for (unsigned int r = 0; r < rounds; ++r) {
    const unsigned int bit = 1u << r;
    const unsigned int low = me & (2u * bit - 1u);
    if (low == bit) {
      // ---- sender: push the current set into the partner's slot, raise its flag
      const unsigned int partner = me - bit;
      Pair* dst = R.peer_slots[partner] + slot_off(parity, r, kcap);
      push_pairs(dst, cur, n_cur, cta, nct);
      cta_fence_peer_stores(single);
      if (!bar.sync(200 + r)) { fail(); return; }
      trace_stamp(ctrl, 1 + 8 * r + 6);
      if (cta == 0 && threadIdx.x == 0)
        release_flag(R.peer_flags[partner] + flag_off(parity, r), epoch, n_cur);
      trace_stamp(ctrl, 1 + 8 * r + 7);
      break;
    }
    if (low != 0u) break;  // already left the tree

    // ---- receiver.  A = current set in a writable work buffer, with map[] and the first-digit
    // histogram describing it (built here in round 0, by the previous compaction afterwards).
    Pair* A;
    const bool copied = cur_buf < 0;
    if (copied) {
      A = R.work[0];
      for (unsigned int i = lane0; i < n_cur; i += stride) {
        const Pair e = ld_pair_cg(&cur[i]);
        st_pair(&A[i], e);
        if ((unsigned int)e.idx < d) map[e.idx] = (int32_t)i;
        else record_error(ctrl, ST_BOUNDS, 300);
        tally(e.val, 1u);
      }
      cur_buf = 0;
    } else {
      A = R.work[cur_buf];
    }
    unsigned int n_b = 0;
    trace_stamp(ctrl, 1 + 8 * r + 0);
    if (!cta_wait_flag(sh.ex, R.flags + flag_off(parity, r), epoch, ctrl, limit_ns, 210 + r, &n_b)) {
      fail();
      return;
    }
    trace_stamp(ctrl, 1 + 8 * r + 1);
    if (n_b > kcap) {
      record_error(ctrl, ST_CAPACITY, 220 + r);
      n_b = kcap;
    }
    Pair* B = R.slots + slot_off(parity, r, kcap);
    const unsigned int n_a = n_cur;
    const unsigned int n_u = n_a + n_b;
    const unsigned int trips = (n_u + stride - 1) / stride;
    // A and map must be complete: after the copy above that needs a barrier, after a previous
    // round its closing barrier already gave it
    if (copied && !bar.sync(230 + r)) { fail(); return; }
    trace_stamp(ctrl, 1 + 8 * r + 2);

    // ---- probe: every thread joins its own B entries against A (sum on shared indices) and
    // keeps them in registers; three dependent loads, issued level by level.
    Pair c[kK2Cache];
    unsigned int pm[kK2Cache];
    auto join = [&](Pair& e, unsigned int p, unsigned int j) {
      bool matched = false;
      if (p < n_a) {
        const Pair a = ld_pair_cg(&A[p]);
        if (a.idx == e.idx) {
          const float nv = a.val + e.val;
          A[p].val = nv;  // A[p] belongs to another thread's sweep: goes through memory
          tally(a.val, 0xffffffffu);
          tally(nv, 1u);
          B[j].idx = -1;
          e.idx = -1;
          matched = true;
        }
      }
      if (!matched) tally(e.val, 1u);
    };
#pragma unroll
    for (int t = 0; t < kK2Cache; ++t) {
      const unsigned int i = (unsigned int)t * stride + lane0;
      c[t].idx = -1;
      c[t].val = 0.f;
      if ((unsigned int)t < trips && i >= n_a && i < n_u) c[t] = ld_pair_cg(&B[i - n_a]);
    }
#pragma unroll
    for (int t = 0; t < kK2Cache; ++t) {
      pm[t] = 0xffffffffu;
      if (c[t].idx >= 0) {
        if ((unsigned int)c[t].idx < d) {
          pm[t] = (unsigned int)__ldcg(&map[c[t].idx]);
        } else {
          record_error(ctrl, ST_BOUNDS, 302);
          B[(unsigned int)t * stride + lane0 - n_a].idx = -1;
          c[t].idx = -1;
        }
      }
    }
#pragma unroll
    for (int t = 0; t < kK2Cache; ++t)
      if (c[t].idx >= 0) join(c[t], pm[t], (unsigned int)t * stride + lane0 - n_a);
    for (unsigned int t = kK2Cache; t < trips; ++t) {  // entries beyond the register cache
      const unsigned int i = t * stride + lane0;
      if (i >= n_a && i < n_u) {
        Pair e = ld_pair_cg(&B[i - n_a]);
        if ((unsigned int)e.idx >= d) {
          record_error(ctrl, ST_BOUNDS, 302);
          B[i - n_a].idx = -1;
        } else {
          join(e, (unsigned int)__ldcg(&map[e.idx]), i - n_a);
        }
      }
    }
    if (!single) hist0_flush(sh, ctrl->hist[r]);
    if (!bar.sync(240 + r)) { fail(); return; }  // sums and the on-the-fly histograms complete
    trace_stamp(ctrl, 1 + 8 * r + 3);

    // ---- every thread now loads its A entries (with the merged values) next to its B entries
#pragma unroll
    for (int t = 0; t < kK2Cache; ++t) {
      const unsigned int i = (unsigned int)t * stride + lane0;
      if ((unsigned int)t < trips && i < n_a) c[t] = ld_pair_cg(&A[i]);
    }
    auto entry = [&](unsigned int t) -> Pair {  // entry of trip t >= kK2Cache, from memory
      const unsigned int i = t * stride + lane0;
      Pair e;
      e.idx = -1;
      e.val = 0.f;
      if (i < n_u) e = ld_pair_cg(i < n_a ? &A[i] : &B[i - n_a]);
      return e;
    };

    // ---- re-select: the first digit is known from the histogram built on the fly
    Threshold th;
    th.select_all = false;
    th.key = 0u;
    th.quota = 0u;
    find_digit_in<kHistBins>(ss, single ? sh.hist0 : ctrl->hist[r][0], k, single);
    const bool all = ss.res_total <= k;
    uint32_t prefix = ss.res_digit;
    unsigned int k_rem = ss.res_krem;
    __syncthreads();
    const unsigned int first_digit = prefix;
    const unsigned int pred_off = first_digit - pred0;  // wraps when the threshold digit is below the prediction
    const bool predicted = !all && pred_off < (unsigned int)kK2Pred;
    if (predicted) {
      // second digit: counted on the fly, no sweep and no barrier
      find_digit_in<1024>(ss, single ? sh.hist1[pred_off] : pred_row(ctrl->hist[r], pred_off), k_rem, single);
      prefix = (prefix << 10) | ss.res_digit;
      k_rem = ss.res_krem;
      __syncthreads();
    }
    if (single) hist0_clear(sh);  // from here on the shared histograms collect the next round's digits
    pred0 = all ? 0u : first_digit;  // the next union's threshold is at least this one
    if (all) {
      th.select_all = true;
    } else {
      if (!predicted) {
        // pass 1: bits 19..10 of the entries whose first digit is the threshold digit
        smem_hist_clear(ss);
#pragma unroll
        for (int t = 0; t < kK2Cache; ++t)
          if (c[t].idx >= 0 && (mag_key(c[t].val) >> 20) == prefix)
            atomicAdd(&ss.hist[(mag_key(c[t].val) >> 10) & 1023u], 1u);
        for (unsigned int t = kK2Cache; t < trips; ++t) {
          const Pair e = entry(t);
          if (e.idx >= 0 && (mag_key(e.val) >> 20) == prefix)
            atomicAdd(&ss.hist[(mag_key(e.val) >> 10) & 1023u], 1u);
        }
        if (!single) smem_hist_flush(ss, ctrl->hist[r][2] + 1024, 1024);
        if (!bar.sync(250 + 10 * r)) { fail(); return; }
        find_digit<1024>(ss, ctrl->hist[r][2] + 1024, k_rem, single);
        prefix = (prefix << 10) | ss.res_digit;
        k_rem = ss.res_krem;
        __syncthreads();
      }
      // pass 2: bits 9..0
      smem_hist_clear(ss);
#pragma unroll
      for (int t = 0; t < kK2Cache; ++t)
        if (c[t].idx >= 0 && (mag_key(c[t].val) >> 10) == prefix)
          atomicAdd(&ss.hist[mag_key(c[t].val) & 1023u], 1u);
      for (unsigned int t = kK2Cache; t < trips; ++t) {
        const Pair e = entry(t);
        if (e.idx >= 0 && (mag_key(e.val) >> 10) == prefix) atomicAdd(&ss.hist[mag_key(e.val) & 1023u], 1u);
      }
      if (!single) smem_hist_flush(ss, ctrl->hist[r][3], 1024);
      if (!bar.sync(251 + 10 * r)) { fail(); return; }
      find_digit<1024>(ss, ctrl->hist[r][3], k_rem, single);
      th.key = (prefix << 10) | ss.res_digit;
      th.quota = ss.res_krem;
      __syncthreads();
    }
    trace_stamp(ctrl, 1 + 8 * r + 4);

    // ---- compaction of the winners to where the next phase reads them
    const bool last = r + 1 == rounds;                                  // then me == 0
    const bool send_next = !last && (me & (4u * bit - 1u)) == 2u * bit;  // sender of round r + 1
    const bool keep = !last && !send_next;                              // receiver again in round r + 1
    Pair* OUT;
    if (last) OUT = R.gout + (size_t)parity * kcap;
    else if (send_next) OUT = R.peer_slots[me - 2u * bit] + slot_off(parity, r + 1, kcap);
    else OUT = R.work[cur_buf ^ 1];
    // keep: the table and (below) the first-digit histogram of the next round are built on the way;
    // last: the table over the global set serves the residual put-back, and every peer gets its copy
    auto on_placed = [&](Pair e, unsigned int pos) {
      if (send_next) return;
      map[e.idx] = (int32_t)pos;
      if (last)
        for (unsigned int q = 1; q < P; ++q) st_pair(R.peer_gout[q] + (size_t)parity * kcap + pos, e);
    };
    unsigned int* const cursor = single ? &sh.cursor : &ctrl->cursor[r];
    unsigned int* const tie = single ? &sh.tie : &ctrl->tie[r];
    if (single && threadIdx.x == 0) {
      sh.cursor = 0u;
      sh.tie = 0u;
    }
    StagedAppender app{&ss, OUT, cursor, kcap, ctrl};
    app.begin();  // (a __syncthreads: the two words above are visible)
    auto consider = [&](const Pair& e) {
      if (e.idx >= 0 && passes_threshold(mag_key(e.val), th, tie)) {
        app.put(e);
        if (keep) tally(e.val, 1u);
      }
    };
#pragma unroll
    for (int t = 0; t < kK2Cache; ++t) {
      if ((unsigned int)t < trips) {
        consider(c[t]);
        app.end_tile(on_placed);
      }
    }
    for (unsigned int t = kK2Cache; t < trips; ++t) {
      consider(entry(t));
      app.end_tile(on_placed);
    }
    app.flush(on_placed);
    if (!single && keep) hist0_flush(sh, ctrl->hist[r + 1]);
    if (!keep) cta_fence_peer_stores(single);  // the winners went into other GPUs' memory
    if (!bar.sync(290 + r)) { fail(); return; }  // OUT and its cursor complete
    trace_stamp(ctrl, 1 + 8 * r + 5);
    n_cur = single ? sh.cursor : __ldcg(&ctrl->cursor[r]);
    if (n_cur > kcap) n_cur = kcap;
    if (send_next) {
      if (cta == 0 && threadIdx.x == 0)
        release_flag(R.peer_flags[me - 2u * bit] + flag_off(parity, r + 1), epoch, n_cur);
      trace_stamp(ctrl, 1 + 8 * (r + 1) + 7);
      break;  // left the tree
    }
    if (last) break;
    cur_buf ^= 1;
    cur = R.work[cur_buf];
  }

  // ---- the global set: rank 0 has just written it into every rank's buffer and only raises the
  // flags; the others wait for theirs and build the table over it
  Pair* G = R.gout + (size_t)parity * kcap;
  unsigned int n_g = 0;
  if (me == 0u) {
    n_g = n_cur;
    if (cta == 0 && threadIdx.x < P && threadIdx.x > 0)  // one releasing thread per destination
      release_flag(R.peer_flags[threadIdx.x] + flag_off(parity, kFlagBcast), epoch, n_cur);
    trace_stamp(ctrl, 40);
    trace_stamp(ctrl, 41);
  } else {
    if (!cta_wait_flag(sh.ex, R.flags + flag_off(parity, kFlagBcast), epoch, ctrl, limit_ns, 410, &n_g)) {
      fail();
      return;
    }
    if (n_g > kcap) {
      record_error(ctrl, ST_CAPACITY, 411);
      n_g = kcap;
    }
    trace_stamp(ctrl, 40);
    build_map(G, n_g, map, d, cta, nct, ctrl);
    if (!bar.sync(420)) { fail(); return; }
    trace_stamp(ctrl, 41);
  }
  // ---- residual put-back of S_local \ S_global
  put_back(R.sel, n_sel, G, n_g, map, R.resid, d, cta, nct);
  trace_stamp(ctrl, 42);
  // ---- the other control block, for the next call (nobody waits for this rank any more)
  {
    uint4* other = reinterpret_cast<uint4*>(R.ctrl + (parity ^ 1u));
    const size_t nvec16 = (offsetof(Ctrl, hist) + (size_t)(rounds + 1) * sizeof(((Ctrl*)0)->hist[0])) / 16;
    for (size_t i = lane0; i < nvec16; i += stride) other[i] = make_uint4(0u, 0u, 0u, 0u);
  }
  if (!bar.sync(430)) { fail(); return; }  // every CTA is past its last use of the call counter
  if (cta == 0 && threadIdx.x == 0) {
    if (aborted(ctrl)) {  // a bounds or capacity error that no wait noticed
      fail();
    } else {
      R.n_global[kResCount] = n_g;
      *R.epoch = epoch + 1u;
    }
  }
}

}  // namespace gtk

using namespace gtk;

extern "C" unsigned long long gtk_k2rank_bytes(void) { return sizeof(K2Rank); }

// Symmetric-region geometry, in bytes, for a given kcap: offsets of slots, ag,
// gout and flags, and the total size.  out[0..4] = {slots, ag, gout, flags, total}.
extern "C" void gtk_symm_layout(unsigned int kcap, int with_allgather, unsigned long long* out) {
  unsigned long long off = 0;
  out[0] = off;
  off += 2ull * kMaxRounds * kcap * sizeof(Pair);
  out[1] = off;
  if (with_allgather) off += 2ull * kMaxPeers * kcap * sizeof(Pair);
  out[2] = off;
  off += 2ull * kcap * sizeof(Pair);
  off = (off + 255ull) & ~255ull;
  out[3] = off;
  off += 2ull * kFlagsPerParity * sizeof(uint64_t);
  off = (off + 255ull) & ~255ull;
  out[4] = off;
}

// Fill one K2Rank descriptor on the host (the caller copies it to the device).
extern "C" int gtk_k2rank_fill(void* desc_host, const void* sel, const void* st, void* work0,
                               void* work1, void* map, void* resid, void* symm_local, void* ctrl,
                               void* n_global, void* epoch_word, unsigned int kcap,
                               int with_allgather, unsigned int P, void* const* symm_peers) {
  if (P > (unsigned int)kMaxPeers) return GTK_ERR_ARG;
  unsigned long long lay[5];
  gtk_symm_layout(kcap, with_allgather, lay);
  K2Rank* r = (K2Rank*)desc_host;
  r->sel = (const Pair*)sel;
  r->st = (const K1State*)st;
  r->work[0] = (Pair*)work0;
  r->work[1] = (Pair*)work1;
  r->map = (int32_t*)map;
  r->resid = (float*)resid;
  char* base = (char*)symm_local;
  r->slots = (Pair*)(base + lay[0]);
  r->ag = (Pair*)(base + lay[1]);
  r->gout = (Pair*)(base + lay[2]);
  r->flags = (uint64_t*)(base + lay[3]);
  r->ctrl = (Ctrl*)ctrl;
  r->n_global = (unsigned int*)n_global;
  r->epoch = (unsigned int*)epoch_word;
  for (unsigned int q = 0; q < (unsigned int)kMaxPeers; ++q) {
    char* pb = q < P ? (char*)symm_peers[q] : nullptr;
    r->peer_slots[q] = pb ? (Pair*)(pb + lay[0]) : nullptr;
    r->peer_ag[q] = pb ? (Pair*)(pb + lay[1]) : nullptr;
    r->peer_gout[q] = pb ? (Pair*)(pb + lay[2]) : nullptr;
    r->peer_flags[q] = pb ? (uint64_t*)(pb + lay[3]) : nullptr;
  }
  return GTK_OK;
}

using K2Kernel = void (*)(const K2Rank*, unsigned int, unsigned int, unsigned int, unsigned int, unsigned int,
                          unsigned long long, int);

// Register-cache depth for a launch: 8 entries per thread when a cluster's threads would otherwise
// have to re-read part of the union from memory in every phase, 4 otherwise.
static int k2_cache_depth(unsigned int k, unsigned int nctas, int cluster) {
  const unsigned long long per_thread4 = 4ull * nctas * kSelThreads;
  return (cluster && 2ull * k > per_thread4) ? 8 : 4;
}
static K2Kernel k2_kernel(int depth) { return depth == 8 ? k2_gtopk_exchange<8> : k2_gtopk_exchange<4>; }

static int k2_max_coresident(int depth) {
  static int cached[2] = {0, 0};  // the occupancy query costs microseconds; the answer never changes
  int& c = cached[depth == 8];
  if (c) return c;
  const DeviceInfo* di = gtk_device_info();
  if (!di) return 0;
  int occ = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, (const void*)k2_kernel(depth), kSelThreads, 0) !=
      cudaSuccess)
    return 0;
  c = occ * di->sms;
  return c;
}

// Largest cluster (CTAs of one rank joined by the hardware barrier) that `nranks` ranks can hold
// co-resident on this device; 0 if clusters cannot be used.  Cached per (nranks, nctas).
static bool k2_cluster_fits(unsigned int nranks, unsigned int nctas) {
  static int cache[kMaxPeers + 1][17] = {};  // 0 unknown, 1 yes, 2 no
  if (nctas < 2 || nctas > 16 || (nctas & (nctas - 1)) || nranks > (unsigned int)kMaxPeers) return false;
  int& c = cache[nranks][nctas];
  if (c) return c == 1;
  c = 2;
  const DeviceInfo* di = gtk_device_info();
  if (!di || !di->cluster) return false;
  for (int depth : {4, 8}) {
    if (nctas > 8 && cudaFuncSetAttribute((const void*)k2_kernel(depth),
                                          cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess) {
      cudaGetLastError();
      return false;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(nctas, nranks);
    cfg.blockDim = dim3(kSelThreads);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = nctas;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int nclusters = 0;
    if (cudaOccupancyMaxActiveClusters(&nclusters, (const void*)k2_kernel(depth), &cfg) != cudaSuccess) {
      cudaGetLastError();
      return false;
    }
    if (nclusters < (int)nranks) return false;
  }
  c = 1;
  return true;
}

// ranks_dev: device array of nranks_in_launch K2Rank descriptors (1 in production).  Nothing is
// cleared here: the kernel alternates between the two control blocks of each rank.
// use_cluster: 1 = join the CTAs of a rank into one thread-block cluster (hardware barrier) when
// nctas is 2, 4, 8 or 16 and the device can hold the clusters; 0 = software barrier.
extern "C" int gtk_k2_exchange(const void* ranks_dev, unsigned int nranks, unsigned int rank_base,
                               unsigned int P, unsigned int k, unsigned int kcap, unsigned int d,
                               unsigned int nctas, unsigned long long limit_ns, int use_cluster,
                               void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (P < 2 || (P & (P - 1)) != 0 || P > (unsigned int)kMaxPeers) return GTK_ERR_ARG;
  if (k == 0 || k > kcap || nranks == 0 || nctas == 0) return GTK_ERR_ARG;
  const K2Rank* ranks = (const K2Rank*)ranks_dev;
  int cluster = (use_cluster && k2_cluster_fits(nranks, nctas)) ? 1 : 0;
  const int depth = k2_cache_depth(k, nctas, cluster);
  const K2Kernel fn = k2_kernel(depth);
  if ((int)(nranks * nctas) > k2_max_coresident(depth)) return GTK_ERR_ARG;
  void* args[] = {&ranks, &rank_base, &P, &k, &kcap, &d, &limit_ns, &cluster};
  cudaError_t e;
  if (cluster) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(nctas, nranks);
    cfg.blockDim = dim3(kSelThreads);
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = nctas;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeCooperative;  // several emulated ranks wait on one another
    attr[1].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = nranks > 1 ? 2 : 1;  // one cluster is co-scheduled by the hardware anyway
    e = cudaLaunchKernelExC(&cfg, (const void*)fn, args);
  } else if (nranks * nctas == 1) {
    // one CTA waits on nobody of its own launch: a plain launch
    fn<<<dim3(1, 1), dim3(kSelThreads), 0, stream>>>(ranks, rank_base, P, k, kcap, d, limit_ns, 0);
    e = cudaGetLastError();
  } else {
    e = cudaLaunchCooperativeKernel((void*)fn, dim3(nctas, nranks), dim3(kSelThreads), args, 0, stream);
  }
  gtk_count_launch(1);
  if (e != cudaSuccess) return GTK_ERR_CUDA;
  return GTK_OK;
}
