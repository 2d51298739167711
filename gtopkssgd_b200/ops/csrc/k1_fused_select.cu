// K1: fused residual add + magnitude top-k selection + residual write-back,
// one cooperative kernel.
//
// Replaces the op sequence of the reference's TopKCompressor.compress
// (compression.py:32-57: add_, abs, topk, gather, mask fill/scatter, mul, sub_)
// and the gather of the selected values (allreducer.py:543).
//
// Phase 1 (all CTAs)  one streaming pass over g and r (read 8d bytes, write 4d):
//     acc = g*scale + r; entries with |acc| >= tau become candidates (appended to
//     a bounded list, r <- 0, first radix digit counted), all others r <- acc.
//     tau is a device-resident prediction from the previous call.
//     Non-finite entries (+-Inf, NaN) count as the largest magnitudes on both paths,
//     NaN above Inf, as torch.topk(|acc|) ranks them: they are selected, never left
//     in the residual.
// grid barrier
// Phase 2  normal mode (k <= C <= cap candidates): the first C/1024 CTAs run the
//     remaining two radix passes over the candidates, compact the k winners,
//     return the rejected candidates to r and re-predict tau from the measured
//     tail slope; the other CTAs leave.
//     exact mode (C < k or the list overflowed; always on the first call, when
//     tau is +inf): all CTAs restore r = acc from the stored candidates, then run
//     a 3-pass radix select over all d entries of r and one collect pass.
// The dense sparsified gradient of the reference is never materialised; the
// output is k (int32 index, fp32 value) pairs in no particular order.
//
// No host-side clearing: the caller provides two control blocks; call i uses
// block (i & 1) and zeroes the other one for call i + 1 (i is K1State::n_calls,
// read on the device, so the launch can be replayed from a CUDA graph).
#include <atomic>
#include <cstddef>
#include "select_common.cuh"
#include "host_api.h"

namespace gtk {

constexpr int kK1Threads = kSelThreads;    // 512
constexpr int kK1Vec = 4;                  // float4 loads of g and of r in flight per thread
constexpr int kWarpStage = 128;            // pairs staged per warp
constexpr int kWarpFlushAt = kWarpStage - 32;
// From this many float4 per array on (48 M elements) the stream pass hands work out dynamically; below
// it the static split is faster (measured: +3.6 % at 138 M and +1.5 % at 64 M, but -4 % at 25.6 M).
constexpr long long kDynamicMinVec = 12ll * 1000 * 1000;

constexpr int kPredDigits = 3;  // second-digit histograms are kept for the predicted first digit and its neighbours
struct StreamShared {
  Pair wstage[kK1Threads / 32][kWarpStage];  // per-warp candidate staging
  unsigned int hist[kHistBins];              // first radix digit of this CTA's candidates
  unsigned int hist1[kPredDigits][1024];     // second digit of the candidates whose first digit is pred-1, pred, pred+1
};
constexpr size_t kK1SmemBytes =
    sizeof(StreamShared) > sizeof(SelectShared) ? sizeof(StreamShared) : sizeof(SelectShared);
// bytes of a control block that K1 dirties: header, trace, three histogram sets
// (set 0: candidate select, set 1: exact mode, set 2: second-digit histograms built by the stream pass)
constexpr size_t kK1ClearBytes = offsetof(Ctrl, hist) + 3 * sizeof(((Ctrl*)0)->hist[0]);

__device__ __forceinline__ void warp_flush(Pair* wbuf, unsigned int& wcnt, Pair* cand,
                                           unsigned int cap, unsigned int* counter, float* r) {
  __syncwarp();
  unsigned int base = 0;
  if (lane_id() == 0) base = atomicAdd(counter, wcnt);
  base = __shfl_sync(0xffffffffu, base, 0);
  for (unsigned int i = lane_id(); i < wcnt; i += 32) {
    const Pair p = wbuf[i];
    if (base + i < cap) {
      st_pair(&cand[base + i], p);
    } else {
      r[p.idx] = p.val;  // list is full: the entry stays in the residual
    }
  }
  wcnt = 0;
  __syncwarp();
}

// Counts one candidate: its first radix digit always, its second digit when the
// first one is within one of `pred` (the first digit of the previous call's k-th
// magnitude), so that the candidate select can usually skip its first sweep.
__device__ __forceinline__ void count_candidate(StreamShared& ss, float a, unsigned int pred) {
  const uint32_t key = mag_key(a);
  const unsigned int fd = key >> 20;
  atomicAdd(&ss.hist[fd], 1u);
  const unsigned int off = fd - pred + 1u;  // wraps for fd < pred - 1: then off >= kPredDigits
  if (off < (unsigned int)kPredDigits) atomicAdd(&ss.hist1[off][(key >> 10) & 1023u], 1u);
}

// One tile of the stream pass: kK1Vec float4 of g and of r per thread, STRIDE
// float4 apart (the CTA's 512 threads or one warp's 32 lanes work side by side).
template <int STRIDE>
__device__ __forceinline__ void stream_tile(long long v0, long long nvec, long long head,
                                            const float4* __restrict__ g4, float4* __restrict__ r4,
                                            float scale, float tau, unsigned int pred, StreamShared& ss,
                                            Pair* wbuf,
                                            unsigned int& wcnt, Pair* __restrict__ cand, unsigned int cap,
                                            unsigned int* counter, float* __restrict__ r) {
  // Candidates are decided on the bit pattern of |acc|, which orders like the magnitude for finite
  // values and puts +-Inf and NaN on top: a non-finite entry is a candidate on this path exactly as it
  // is the largest key on the exact path (torch.topk(|acc|) in compression.py:43 also ranks NaN first).
  const uint32_t tau_key = __float_as_uint(tau);
  float4 gv[kK1Vec], rv[kK1Vec];
#pragma unroll
  for (int u = 0; u < kK1Vec; ++u) {
    const long long v = v0 + (long long)u * STRIDE;
    if (v < nvec) {
      gv[u] = __ldcs(&g4[v]);
      rv[u] = r4[v];
    } else {
      gv[u] = make_float4(0.f, 0.f, 0.f, 0.f);
      rv[u] = gv[u];
    }
  }
#pragma unroll
  for (int u = 0; u < kK1Vec; ++u) {
    const long long v = v0 + (long long)u * STRIDE;
    const bool inb = v < nvec;
    float a[4];
    a[0] = fmaf(gv[u].x, scale, rv[u].x);
    a[1] = fmaf(gv[u].y, scale, rv[u].y);
    a[2] = fmaf(gv[u].z, scale, rv[u].z);
    a[3] = fmaf(gv[u].w, scale, rv[u].w);
    bool c[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) c[e] = inb && (mag_key(a[e]) >= tau_key);
    if (inb) {
      float4 o;
      o.x = c[0] ? 0.f : a[0];
      o.y = c[1] ? 0.f : a[1];
      o.z = c[2] ? 0.f : a[2];
      o.w = c[3] ? 0.f : a[3];
      r4[v] = o;
    }
    const unsigned int any = __ballot_sync(0xffffffffu, c[0] | c[1] | c[2] | c[3]);
    if (any) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const unsigned int m = __ballot_sync(0xffffffffu, c[e]);
        if (m) {
          if (c[e]) {
            Pair p;
            p.idx = (int32_t)(head + (v << 2) + e);
            p.val = a[e];
            wbuf[wcnt + __popc(m & lanemask_lt())] = p;
            count_candidate(ss, a[e], pred);
          }
          wcnt += __popc(m);
          if (wcnt > (unsigned int)kWarpFlushAt) warp_flush(wbuf, wcnt, cand, cap, counter, r);
        }
      }
    }
  }
}

__device__ __forceinline__ void stream_phase(StreamShared& ss, const float* __restrict__ g,
                                             float* __restrict__ r, float scale, float tau,
                                             Pair* __restrict__ cand, unsigned int cap, Ctrl* ctrl,
                                             long long d, unsigned int pred) {
  for (int i = threadIdx.x; i < kHistBins; i += kK1Threads) ss.hist[i] = 0u;
  for (int i = threadIdx.x; i < kPredDigits * 1024; i += kK1Threads) (&ss.hist1[0][0])[i] = 0u;
  __syncthreads();
  Pair* wbuf = ss.wstage[threadIdx.x >> 5];
  unsigned int wcnt = 0;
  unsigned int* counter = &ctrl->n_out;

  // Leading scalars up to the first 16-byte boundary (g and r share the offset).
  const unsigned int mis = (unsigned int)((reinterpret_cast<uintptr_t>(r) >> 2) & 3u);
  long long head = mis ? (4 - mis) : 0;
  if (head > d) head = d;
  const long long nvec = (d - head) >> 2;
  const long long tail0 = head + (nvec << 2);
  const float4* g4 = reinterpret_cast<const float4*>(g + head);
  float4* r4 = reinterpret_cast<float4*>(r + head);

  constexpr long long kTileVec = (long long)kK1Threads * kK1Vec;
  constexpr long long kWarpTileVec = 32ll * kK1Vec;
  if (nvec < kDynamicMinVec) {
    // Static split: CTA b takes tiles b, b + grid, ...; every load instruction of the CTA covers 8 KB.
    // (One contiguous, equally sized range per CTA was tried: its ragged last tile costs almost a full
    // tile's latency in every CTA, and the call got 3 % slower at d = 25.6 M.)
    const long long ntiles = (nvec + kTileVec - 1) / kTileVec;
    for (long long tile = blockIdx.x; tile < ntiles; tile += gridDim.x)
      stream_tile<kK1Threads>(tile * kTileVec + threadIdx.x, nvec, head, g4, r4, scale, tau, pred, ss, wbuf, wcnt,
                              cand, cap, counter, r);
  } else {
    // Large vectors: SMs do not all see the same memory bandwidth, and with the static split the grid
    // barrier waited up to 13 us (d = 64 M) for the slowest CTA.  Here work is handed out per warp in
    // chunks of kChunkTiles warp-tiles (32 lanes x kK1Vec float4): the first chunk of a warp is fixed,
    // further chunks come from a ticket counter that is read one chunk ahead, so the atomic's latency
    // hides behind the loads.
    constexpr long long kChunkTiles = 4;
    const long long nchunks = (nvec + kWarpTileVec * kChunkTiles - 1) / (kWarpTileVec * kChunkTiles);
    const unsigned int nwarps_grid = gridDim.x * (kK1Threads / 32);
    unsigned int* ticket = &ctrl->scratch[1];
    long long chunk = (long long)blockIdx.x * (kK1Threads / 32) + (threadIdx.x >> 5);
    while (chunk < nchunks) {
      unsigned int nxt = 0;
      if (lane_id() == 0) nxt = atomicAdd(ticket, 1u);  // consumed after this chunk
      for (long long wt = 0; wt < kChunkTiles; ++wt) {
        const long long base = (chunk * kChunkTiles + wt) * kWarpTileVec;
        if (base >= nvec) break;  // warp-uniform
        stream_tile<32>(base + lane_id(), nvec, head, g4, r4, scale, tau, pred, ss, wbuf, wcnt, cand, cap, counter,
                        r);
      }
      nxt = __shfl_sync(0xffffffffu, nxt, 0);
      chunk = (long long)nwarps_grid + nxt;
    }
  }
  // Scalar head and tail (at most 3 + 3 entries), one warp of CTA 0.
  const uint32_t tau_key = __float_as_uint(tau);
  if (blockIdx.x == 0 && threadIdx.x < 32) {
    const long long nscalar = head + (d - tail0);
    for (long long base = 0; base < nscalar; base += 32) {
      const long long j = base + lane_id();
      bool c = false;
      float a = 0.f;
      long long i = 0;
      if (j < nscalar) {
        i = j < head ? j : tail0 + (j - head);
        a = fmaf(g[i], scale, r[i]);
        c = mag_key(a) >= tau_key;
        r[i] = c ? 0.f : a;
      }
      const unsigned int m = __ballot_sync(0xffffffffu, c);
      if (m) {
        if (c) {
          Pair p;
          p.idx = (int32_t)i;
          p.val = a;
          wbuf[wcnt + __popc(m & lanemask_lt())] = p;
          count_candidate(ss, a, pred);
        }
        wcnt += __popc(m);
        if (wcnt > (unsigned int)kWarpFlushAt) warp_flush(wbuf, wcnt, cand, cap, counter, r);
      }
    }
  }
  if (wcnt) warp_flush(wbuf, wcnt, cand, cap, counter, r);
  // publish this CTA's part of the first-pass histogram
  __syncthreads();
  for (int i = threadIdx.x; i < kHistBins; i += kK1Threads) {
    const unsigned int c = ss.hist[i];
    if (c) atomicAdd(&ctrl->hist[0][0][i], c);
  }
  for (int i = threadIdx.x; i < kPredDigits * 1024; i += kK1Threads) {
    const unsigned int c = ss.hist1[i >> 10][i & 1023];
    if (c) atomicAdd(&ctrl->hist[2][i >> 10][i & 1023], c);
  }
}

// Re-predict tau so that the next stream pass yields about target_ratio * k
// candidates, assuming a power-law tail count(t) = k * (t / t_k)^(-alpha) whose
// exponent is measured from (C candidates at tau_used, k entries at t_k).
__device__ __forceinline__ float predict_tau(float t_k, float tau_used, unsigned int C,
                                             unsigned int k, float target_ratio) {
  float alpha = 8.0f;
  const float ratio = (float)C / (float)(k ? k : 1u);
  if (tau_used > 0.f && tau_used < t_k * 0.999f && ratio > 1.05f && isfinite(tau_used)) {
    alpha = logf(ratio) / logf(t_k / tau_used);
    alpha = fminf(fmaxf(alpha, 2.0f), 64.0f);
  }
  const float next = t_k * expf(-logf(target_ratio) / alpha);
  return next > 0.f ? next : 0.f;
}

__global__ void __launch_bounds__(kK1Threads, 2)
k1_fused(const float* __restrict__ g, float* __restrict__ r, const float* __restrict__ g_scale,
         long long d, Pair* __restrict__ cand, unsigned int cap, Pair* __restrict__ sel,
         unsigned int k, K1State* st, Ctrl* ctrl_pair, float target_ratio,
         unsigned long long limit_ns) {
  __shared__ __align__(16) unsigned char smem_raw[kK1SmemBytes];
  // Every CTA reads the call parity before the grid barrier; it is advanced after it.
  const unsigned int calls = st->n_calls;
  Ctrl* ctrl = ctrl_pair + (calls & 1u);
  {  // prepare the other control block for the next call
    uint4* other = reinterpret_cast<uint4*>(ctrl_pair + ((calls & 1u) ^ 1u));
    const size_t nvec16 = kK1ClearBytes / 16;
    for (size_t i = (size_t)blockIdx.x * kK1Threads + threadIdx.x; i < nvec16;
         i += (size_t)gridDim.x * kK1Threads)
      other[i] = make_uint4(0u, 0u, 0u, 0u);
  }
  const float tau_used = st->tau;
  const float scale = g_scale ? *g_scale : 1.0f;
  trace_stamp(ctrl, 0);
  const unsigned int pred = mag_key(st->kth_mag) >> 20;  // first digit of the previous call's k-th magnitude
  stream_phase(*reinterpret_cast<StreamShared*>(smem_raw), g, r, scale, tau_used, cand, cap, ctrl, d, pred);

  trace_stamp(ctrl, 1);  // CTA 0 finished its share of the stream
  RankBarrier bar_all{ctrl, gridDim.x, 0u, limit_ns};
  if (!bar_all.sync(90)) return;
  trace_stamp(ctrl, 2);  // every CTA did
  if (blockIdx.x == 0 && threadIdx.x == 0) st->n_calls = calls + 1u;

  SelectShared& s = *reinterpret_cast<SelectShared*>(smem_raw);
  const unsigned int count = __ldcg(&ctrl->n_out);
  const unsigned int C = count < cap ? count : cap;
  const bool exact_mode = (count > cap) || (C < k);
  Threshold th;
  auto none = [](Pair, unsigned int) {};

  if (!exact_mode) {
    unsigned int nct = (C + 1023u) / 1024u;  // one or two candidates per thread and pass
    if (nct < 1u) nct = 1u;
    if (nct > gridDim.x) nct = gridDim.x;
    if (blockIdx.x >= nct) return;
    RankBarrier bar{ctrl, nct, 0u, limit_ns, &ctrl->scratch[0]};
    auto key_at = [&](unsigned int i) -> uint32_t { return mag_key(ld_pair_cg(&cand[i]).val); };
    if (!radix_select_kth(s, bar, blockIdx.x, nct, C, k, ctrl->hist[0], key_at, &th, 100, true, ctrl->hist[2],
                          pred - 1u, kPredDigits))
      return;
    trace_stamp(ctrl, 3);  // k-th magnitude known
    StagedAppender app{&s, sel, &ctrl->cursor[0], k, ctrl};
    app.begin();
    const unsigned int stride = nct * kSelThreads;
    const unsigned int trips = (C + stride - 1) / stride;
    for (unsigned int t = 0; t < trips; ++t) {
      const unsigned int i = t * stride + blockIdx.x * kSelThreads + threadIdx.x;
      if (i < C) {
        const Pair e = ld_pair_cg(&cand[i]);
        if (passes_threshold(mag_key(e.val), th, &ctrl->tie[0])) {
          app.put(e);
        } else {
          r[e.idx] = e.val;
        }
      }
      app.end_tile(none);
    }
    app.flush(none);
    trace_stamp(ctrl, 4);  // CTA 0 compacted its share
    if (blockIdx.x == 0 && threadIdx.x == 0) {
      const float t_k = __uint_as_float(th.key);
      st->n_sel = k;
      st->n_cand = count;
      st->fallback = 0u;
      st->kth_mag = t_k;
      st->tau = predict_tau(t_k, tau_used, C, k, target_ratio);
    }
    return;
  }

  // Exact mode: every CTA of the grid takes part.
  const unsigned int nct = gridDim.x;
  const unsigned int stride = nct * kSelThreads;
  for (unsigned int i = blockIdx.x * kSelThreads + threadIdx.x; i < C; i += stride) {
    const Pair e = ld_pair_cg(&cand[i]);
    r[e.idx] = e.val;
  }
  if (!bar_all.sync(110)) return;
  const unsigned int n = (unsigned int)d;
  auto key_at = [&](unsigned int i) -> uint32_t { return mag_key(__ldcg(&r[i])); };
  if (!radix_select_kth(s, bar_all, blockIdx.x, nct, n, k, ctrl->hist[1], key_at, &th, 120)) return;
  StagedAppender app{&s, sel, &ctrl->cursor[1], k, ctrl};
  app.begin();
  const unsigned int trips = (n + stride - 1) / stride;
  for (unsigned int t = 0; t < trips; ++t) {
    const unsigned int i = t * stride + blockIdx.x * kSelThreads + threadIdx.x;
    if (i < n) {
      const float v = __ldcg(&r[i]);
      if (passes_threshold(mag_key(v), th, &ctrl->tie[1])) {
        Pair e;
        e.idx = (int32_t)i;
        e.val = v;
        app.put(e);
        r[i] = 0.f;
      }
    }
    app.end_tile(none);
  }
  app.flush(none);
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    const float t_k = th.select_all ? 0.f : __uint_as_float(th.key);
    st->n_sel = th.select_all ? s.res_total : k;
    st->n_cand = count;
    st->fallback = 1u;
    st->n_fallbacks += 1u;
    st->kth_mag = t_k;
    st->tau = predict_tau(t_k, 0.f, 0u, k, target_ratio);
  }
  trace_stamp(ctrl, 5);  // exact mode: CTA 0 collected its share
}

}  // namespace gtk

using namespace gtk;

extern "C" unsigned long long gtk_ctrl_bytes(void) { return sizeof(Ctrl); }

namespace {
// Co-resident CTAs of k1_fused on the current device (cached).
int k1_max_grid() {
  static std::atomic<int> cached[64];  // per device: GPUs of one process need not be alike
  const DeviceInfo* di = gtk_device_info();
  if (!di || di->device < 0 || di->device >= 64) return 0;
  const int have = cached[di->device].load(std::memory_order_relaxed);
  if (have) return have;
  int occ = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, k1_fused, kK1Threads, 0) != cudaSuccess ||
      occ < 1)
    return 0;
  if (occ > 2) occ = 2;
  cached[di->device].store(di->sms * occ, std::memory_order_relaxed);
  return di->sms * occ;
}

int k1_launch(const float* g, float* r, const float* g_scale, long long d, unsigned int k,
              Pair* cand, unsigned int cap, Pair* sel, K1State* st, Ctrl* ctrl_pair,
              float target_ratio, unsigned long long limit_ns, cudaStream_t stream) {
  const int max_grid = k1_max_grid();
  if (max_grid < 1) return GTK_ERR_CUDA;
  const long long tile = (long long)kK1Threads * kK1Vec;
  const long long ntiles = ((d / 4) + tile - 1) / tile;
  long long want = (cap + 1023u) / 1024u;  // CTAs the candidate select can use
  if (ntiles > want) want = ntiles;
  int grid = want < max_grid ? (int)(want > 0 ? want : 1) : max_grid;
  void* args[] = {&g, &r, &g_scale, &d, &cand, &cap, &sel, &k, &st, &ctrl_pair, &target_ratio, &limit_ns};
  const cudaError_t e = cudaLaunchCooperativeKernel((void*)k1_fused, dim3(grid), dim3(kK1Threads),
                                                    args, 0, stream);
  gtk_count_launch(1);
  return e == cudaSuccess ? GTK_OK : GTK_ERR_CUDA;
}
}  // namespace

// ctrl: TWO consecutive control blocks (2 * gtk_ctrl_bytes()), zero when first used.
extern "C" int gtk_k1_select(const float* g, float* r, const float* g_scale, long long d,
                             unsigned int k, void* cand, unsigned int cap, void* sel, void* state,
                             void* ctrl, float target_ratio, unsigned long long limit_ns,
                             void* stream_) {
  if (d <= 0 || d >= (1ll << 31) || k == 0 || k > cap) return GTK_ERR_ARG;
  // g and r must share their offset inside a 16-byte line (same flat layout)
  if ((reinterpret_cast<uintptr_t>(g) & 15u) != (reinterpret_cast<uintptr_t>(r) & 15u) ||
      (reinterpret_cast<uintptr_t>(r) & 3u) != 0u)
    return GTK_ERR_ARG;
  return k1_launch(g, r, g_scale, d, k, (Pair*)cand, cap, (Pair*)sel, (K1State*)state, (Ctrl*)ctrl,
                   target_ratio, limit_ns, (cudaStream_t)stream_);
}

// ---------------------------------------------------------------------------
// Allocation-free variant (declared and documented in k1_select_noalloc.h).
// The scratch that gtk_k1_select takes from its caller lives here in a static
// device array; the kernel is the one above, unchanged.
// ---------------------------------------------------------------------------
#include <mutex>
#include "k1_select_noalloc.h"

namespace {

constexpr unsigned int kNoAllocMaxK = 16384u;
constexpr unsigned int kNoAllocCap = 131072u;                         // candidate pairs (8 x max k)
constexpr size_t kNoAllocCtrlOff = 0;                                  // two control blocks
constexpr size_t kNoAllocStateOff = (2 * sizeof(Ctrl) + 255) / 256 * 256;
constexpr size_t kNoAllocCandOff = kNoAllocStateOff + 256;
constexpr size_t kNoAllocBytes = kNoAllocCandOff + (size_t)kNoAllocCap * sizeof(Pair);

// In host code this name is only a handle for cudaGetSymbolAddress, never an address.
// Static device storage starts zeroed, which is what the control blocks need on first use.
static __device__ __align__(256) unsigned char g_k1_noalloc_scratch[kNoAllocBytes];

// Forget the predicted threshold.  The call counter is left alone: it decides which
// control block is clean.
__global__ void k1_noalloc_reset_state(K1State* st) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    st->tau = __int_as_float(0x7f800000);  // +inf: the next call takes the exact path
    st->n_sel = 0u;
    st->n_cand = 0u;
    st->fallback = 0u;
    st->kth_mag = 0.f;
  }
}

__global__ void k1_noalloc_publish_count(const K1State* st, unsigned int* n_sel_out) {
  if (threadIdx.x == 0 && blockIdx.x == 0) *n_sel_out = st->n_sel;
}

struct NoAllocDevice {
  unsigned char* base = nullptr;  // device address of g_k1_noalloc_scratch on this device
};
std::mutex g_noalloc_mu;
NoAllocDevice g_noalloc_dev[64];

}  // namespace

extern "C" unsigned int gtk_k1_noalloc_max_k(void) { return kNoAllocMaxK; }
extern "C" unsigned long long gtk_k1_noalloc_scratch_bytes(void) { return kNoAllocBytes; }

extern "C" int gtk_k1_select_noalloc(const float* g, float* r, long long d, unsigned int k,
                                     void* sel_out, unsigned int* n_sel_out, int reset_threshold,
                                     void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (k > kNoAllocMaxK) return GTK_ERR_TOO_LARGE;
  if (d <= 0 || d >= (1ll << 31) || k == 0 || !g || !r || !sel_out) return GTK_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(g) & 15u) != (reinterpret_cast<uintptr_t>(r) & 15u) ||
      (reinterpret_cast<uintptr_t>(r) & 3u) != 0u)
    return GTK_ERR_ARG;
  // pairs are stored with one 8-byte access, the count with a 4-byte one
  if ((reinterpret_cast<uintptr_t>(sel_out) & 7u) != 0u ||
      (n_sel_out && (reinterpret_cast<uintptr_t>(n_sel_out) & 3u) != 0u))
    return GTK_ERR_ARG;
  const DeviceInfo* di = gtk_device_info();
  if (!di || di->device < 0 || di->device >= 64) return GTK_ERR_CUDA;
  NoAllocDevice dev;
  bool first = false;
  {
    std::lock_guard<std::mutex> lk(g_noalloc_mu);
    NoAllocDevice& slot = g_noalloc_dev[di->device];
    if (!slot.base) {
      // once per device, with that device current
      void* p = nullptr;
      if (cudaGetSymbolAddress(&p, g_k1_noalloc_scratch) != cudaSuccess || !p) return GTK_ERR_CUDA;
      slot.base = static_cast<unsigned char*>(p);
      first = true;
    }
    dev = slot;
  }
  Ctrl* ctrl_pair = reinterpret_cast<Ctrl*>(dev.base + kNoAllocCtrlOff);
  K1State* st = reinterpret_cast<K1State*>(dev.base + kNoAllocStateOff);
  Pair* cand = reinterpret_cast<Pair*>(dev.base + kNoAllocCandOff);
  if (first || reset_threshold) {
    k1_noalloc_reset_state<<<1, 32, 0, stream>>>(st);
    gtk_count_launch(1);
  }
  // What must start at zero -- the control block of this call -- was cleared by the previous call
  // (or is still in its initial zero state); the candidate list is overwritten before it is read.
  const int code = k1_launch(g, r, nullptr, d, k, cand, kNoAllocCap, static_cast<Pair*>(sel_out), st,
                             ctrl_pair, 3.0f, 2000000000ull, stream);
  if (code != GTK_OK) return code;
  if (n_sel_out) {
    k1_noalloc_publish_count<<<1, 32, 0, stream>>>(st, n_sel_out);
    gtk_count_launch(1);
  }
  return cudaGetLastError() == cudaSuccess ? GTK_OK : GTK_ERR_CUDA;
}

// Status of the shared scratch on the current device: out_status_where[0] = status code of the first
// failure recorded in either control block (0: none; the codes of gtk::Status), [1] = its code
// location.  With reset != 0 both control blocks and the threshold state are cleared afterwards, which
// is what brings the entry point back after a failed call (a barrier that ran into its limit leaves
// its control block marked aborted).  Copies 16 bytes to the host and waits for `stream` only; no
// allocation.  Returns GTK_ERR_ARG before the first gtk_k1_select_noalloc call on this device.
extern "C" int gtk_k1_noalloc_status(unsigned int* out_status_where, int reset, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  const DeviceInfo* di = gtk_device_info();
  if (!di || di->device < 0 || di->device >= 64) return GTK_ERR_CUDA;
  NoAllocDevice dev;
  {
    std::lock_guard<std::mutex> lk(g_noalloc_mu);
    dev = g_noalloc_dev[di->device];
  }
  if (!dev.base) return GTK_ERR_ARG;
  Ctrl* ctrl_pair = reinterpret_cast<Ctrl*>(dev.base + kNoAllocCtrlOff);
  unsigned int words[2][2] = {{0u, 0u}, {0u, 0u}};
  for (int b = 0; b < 2; ++b)
    if (cudaMemcpyAsync(words[b], &ctrl_pair[b].status, 2 * sizeof(unsigned int), cudaMemcpyDeviceToHost,
                        stream) != cudaSuccess)
      return GTK_ERR_CUDA;
  if (reset) {
    if (cudaMemsetAsync(ctrl_pair, 0, 2 * sizeof(Ctrl), stream) != cudaSuccess) return GTK_ERR_CUDA;
    k1_noalloc_reset_state<<<1, 32, 0, stream>>>(reinterpret_cast<K1State*>(dev.base + kNoAllocStateOff));
    gtk_count_launch(1);
  }
  if (cudaStreamSynchronize(stream) != cudaSuccess) return GTK_ERR_CUDA;
  const int b = words[0][0] ? 0 : 1;
  if (out_status_where) {
    out_status_where[0] = words[b][0];
    out_status_where[1] = words[b][1];
  }
  return GTK_OK;
}
