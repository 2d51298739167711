// Multi-CTA exact top-k-by-magnitude selection (3-pass radix select: 11+10+10
// bits of the |value| bit pattern) and unordered compaction, shared by the
// candidate select of K1, the dense fallback of K1 and the per-round re-select
// of K2.  All CTAs of a rank run the same sequence and meet in RankBarrier.
#pragma once
#include "common.cuh"

namespace gtk {

constexpr int kSelThreads = 512;
constexpr int kStageCap = 2048;  // pairs staged in shared memory before one global cursor bump

struct SelectShared {
  unsigned int hist[kHistBins];
  unsigned int warp_tot[kSelThreads / 32];
  unsigned int res_digit;
  unsigned int res_krem;
  unsigned int res_total;
  unsigned int res_equal;
  unsigned int stage_n;
  unsigned int stage_base;
  Pair stage[kStageCap];
};

struct Threshold {
  uint32_t key;        // bit pattern of the k-th largest magnitude
  uint32_t quota;      // how many entries equal to key are still selected
  bool select_all;     // fewer live entries than k: everything is selected
};

__device__ __forceinline__ void smem_hist_clear(SelectShared& s) {
  for (int i = threadIdx.x; i < kHistBins; i += kSelThreads) s.hist[i] = 0u;
  __syncthreads();
}

__device__ __forceinline__ void smem_hist_flush(SelectShared& s, unsigned int* ghist, int nbins) {
  __syncthreads();
  for (int i = threadIdx.x; i < nbins; i += kSelThreads) {
    const unsigned int c = s.hist[i];
    if (c) atomicAdd(&ghist[i], c);
  }
}

// Every CTA scans the (complete) global histogram from the top bin downwards and
// finds the digit D with count(bins > D) < k_rem <= count(bins >= D).
// Results are left in shared memory: res_digit, res_krem (k_rem minus the count
// above D), res_total (all entries), res_equal (count in bin D).
// counts: the histogram to scan; in_smem says whether it is a shared-memory
// array of this CTA (single-CTA ranks never touch a global copy) or a global one.
template <int NBINS>
__device__ __forceinline__ void find_digit_in(SelectShared& s, const unsigned int* counts,
                                              unsigned int k_rem, bool in_smem) {
  constexpr int BPT = NBINS / kSelThreads;
  static_assert(BPT >= 1, "bins per thread");
  const int t = threadIdx.x;
  unsigned int c[BPT];
  unsigned int mine = 0;
#pragma unroll
  for (int j = 0; j < BPT; ++j) {
    c[j] = in_smem ? counts[t * BPT + j] : __ldcg(&counts[t * BPT + j]);
    mine += c[j];
  }
  // inclusive suffix sum over threads (higher thread = higher bins)
  unsigned int suf = mine;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned int v = __shfl_down_sync(0xffffffffu, suf, o);
    if ((int)lane_id() + o < 32) suf += v;
  }
  const int w = t >> 5;
  if (lane_id() == 0) s.warp_tot[w] = suf;
  if (t == 0) { s.res_digit = 0u; s.res_krem = 0u; s.res_equal = 0u; }
  __syncthreads();
  unsigned int above_warps = 0, total = 0;
#pragma unroll
  for (int i = 0; i < kSelThreads / 32; ++i) {
    const unsigned int v = s.warp_tot[i];
    total += v;
    if (i > w) above_warps += v;
  }
  const unsigned int above = above_warps + (suf - mine);  // entries in bins above this thread's
  if (t == 0) s.res_total = total;
  if (above < k_rem && k_rem <= above + mine) {
    unsigned int a = above;
#pragma unroll
    for (int j = BPT - 1; j >= 0; --j) {
      if (a < k_rem && k_rem <= a + c[j]) {
        s.res_digit = (unsigned int)(t * BPT + j);
        s.res_krem = k_rem - a;
        s.res_equal = c[j];
      }
      a += c[j];
    }
  }
  __syncthreads();
}

template <int NBINS>
__device__ __forceinline__ void find_digit(SelectShared& s, const unsigned int* ghist,
                                           unsigned int k_rem, bool local) {
  find_digit_in<NBINS>(s, local ? s.hist : ghist, k_rem, local);
}

// Radix select of the k-th largest magnitude over `n` logical entries, where
// key_at(i) returns the 31-bit magnitude key of entry i, or 0xffffffff for a dead
// entry.  hist points to three zeroed global histograms [3][kHistBins].
// have_pass0: hist[0] already holds the complete first-digit histogram of the
// entries (an earlier phase built it), so the first sweep is skipped.
// pre1 / pre1_lo / pre1_n: complete second-digit histograms (1024 bins each) of
// the entries whose first digit is pre1_lo, pre1_lo + 1, ..., pre1_lo + pre1_n - 1;
// if the threshold's first digit is one of them the second sweep is skipped too.
// Returns false on abort.
template <typename KeyAt>
__device__ __forceinline__ bool radix_select_kth(SelectShared& s, RankBarrier& bar, unsigned int cta,
                                                 unsigned int nctas, unsigned int n, unsigned int k,
                                                 unsigned int (*hist)[kHistBins], KeyAt key_at,
                                                 Threshold* out, uint32_t where,
                                                 bool have_pass0 = false,
                                                 unsigned int (*pre1)[kHistBins] = nullptr,
                                                 unsigned int pre1_lo = 0u, unsigned int pre1_n = 0u) {
  const unsigned int stride = nctas * kSelThreads;
  uint32_t prefix = 0;
  unsigned int k_rem = k;
  const bool local = nctas == 1;
  // pass 0: bits 30..20
  if (!have_pass0) {
    smem_hist_clear(s);
    for (unsigned int i = cta * kSelThreads + threadIdx.x; i < n; i += stride) {
      const uint32_t key = key_at(i);
      if (key != 0xffffffffu) atomicAdd(&s.hist[key >> 20], 1u);
    }
    if (!local) smem_hist_flush(s, hist[0], kHistBins);
    if (!bar.sync(where + 0)) return false;
  }
  find_digit<kHistBins>(s, hist[0], k_rem, local && !have_pass0);
  if (s.res_total <= k) {  // not more live entries than k: keep them all
    out->key = 0u;
    out->quota = 0u;
    out->select_all = true;
    __syncthreads();
    return true;
  }
  prefix = s.res_digit;
  k_rem = s.res_krem;
  __syncthreads();
  // pass 1: bits 19..10
  const unsigned int pre_off = prefix - pre1_lo;  // wraps when prefix < pre1_lo
  if (pre1 != nullptr && pre_off < pre1_n) {
    find_digit<1024>(s, pre1[pre_off], k_rem, false);  // built earlier: no sweep, no barrier
  } else {
    smem_hist_clear(s);
    for (unsigned int i = cta * kSelThreads + threadIdx.x; i < n; i += stride) {
      const uint32_t key = key_at(i);
      if (key != 0xffffffffu && (key >> 20) == prefix) atomicAdd(&s.hist[(key >> 10) & 1023u], 1u);
    }
    if (!local) smem_hist_flush(s, hist[1], 1024);
    if (!bar.sync(where + 1)) return false;
    find_digit<1024>(s, hist[1], k_rem, local);
  }
  prefix = (prefix << 10) | s.res_digit;
  k_rem = s.res_krem;
  __syncthreads();
  // pass 2: bits 9..0
  smem_hist_clear(s);
  for (unsigned int i = cta * kSelThreads + threadIdx.x; i < n; i += stride) {
    const uint32_t key = key_at(i);
    if (key != 0xffffffffu && (key >> 10) == prefix) atomicAdd(&s.hist[key & 1023u], 1u);
  }
  if (!local) smem_hist_flush(s, hist[2], 1024);
  if (!bar.sync(where + 2)) return false;
  find_digit<1024>(s, hist[2], k_rem, local);
  out->key = (prefix << 10) | s.res_digit;
  out->quota = s.res_krem;
  out->select_all = false;
  __syncthreads();
  return true;
}

// CTA-wide staged append.  Call put() from any thread, then end_tile() from all
// threads once per loop trip (at most kSelThreads puts between two end_tile calls).
struct StagedAppender {
  SelectShared* s;
  Pair* out;             // may be peer memory
  unsigned int* cursor;  // global cursor (local memory)
  unsigned int cap;
  Ctrl* ctrl;

  __device__ __forceinline__ void begin() {
    if (threadIdx.x == 0) s->stage_n = 0u;
    __syncthreads();
  }
  __device__ __forceinline__ void put(Pair p) {
    const unsigned int pos = atomicAdd(&s->stage_n, 1u);
    s->stage[pos] = p;
  }
  template <typename OnPlaced>
  __device__ __forceinline__ void flush(OnPlaced on_placed) {
    __syncthreads();
    const unsigned int n = s->stage_n;
    if (n) {
      if (threadIdx.x == 0) s->stage_base = atomicAdd(cursor, n);
      __syncthreads();
      const unsigned int base = s->stage_base;
      for (unsigned int i = threadIdx.x; i < n; i += kSelThreads) {
        const unsigned int pos = base + i;
        if (pos < cap) {
          st_pair(&out[pos], s->stage[i]);
          on_placed(s->stage[i], pos);
        } else {
          record_error(ctrl, ST_CAPACITY, 900);
        }
      }
      __syncthreads();
      if (threadIdx.x == 0) s->stage_n = 0u;
    }
    __syncthreads();
  }
  template <typename OnPlaced>
  __device__ __forceinline__ void end_tile(OnPlaced on_placed) {
    __syncthreads();
    if (s->stage_n > (unsigned int)(kStageCap - kSelThreads)) flush(on_placed);
  }
};

// Decide one entry against the threshold.  Entries equal to the threshold take a
// ticket; the first `quota` tickets are selected.
__device__ __forceinline__ bool passes_threshold(uint32_t key, const Threshold& th,
                                                 unsigned int* tie_counter) {
  if (th.select_all) return true;
  if (key > th.key) return true;
  if (key == th.key) return atomicAdd(tie_counter, 1u) < th.quota;
  return false;
}

}  // namespace gtk
