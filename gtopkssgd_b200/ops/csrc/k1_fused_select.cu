// K1: fused residual add + magnitude top-k selection + residual write-back.
//
// Replaces the op sequence of the reference's TopKCompressor.compress
// (compression.py:32-57: add_, abs, topk, gather, mask fill/scatter, mul, sub_)
// and the gather of the selected values (allreducer.py:543).
//
// Two launches:
//   k1_stream  one streaming pass over g and r (read 8d bytes, write 4d bytes):
//              acc = g*scale + r; entries with |acc| >= tau become candidates
//              (appended to a bounded list, r <- 0), all others r <- acc.
//              tau is a device-resident prediction from the previous call.
//   k1_finish  cooperative kernel.  Normal mode: exact radix select of the k
//              largest magnitudes among the C candidates (k <= C <= cap),
//              rejected candidates go back into r, tau is re-predicted from the
//              measured tail slope.  Exact mode (C < k or the list overflowed;
//              always on the first call, when tau is +inf): restore r = acc from
//              the stored candidates, then a 3-pass radix select over all d
//              entries of r and one collect pass.
// The dense sparsified gradient of the reference is never materialised; the
// output is k (int32 index, fp32 value) pairs in no particular order.
#include <cstddef>
#include "select_common.cuh"
#include "host_api.h"

namespace gtk {

constexpr int kK1Threads = 512;
constexpr int kK1Vec = 4;                  // float4 loads of g and of r in flight per thread
constexpr int kWarpStage = 128;            // pairs staged per warp
constexpr int kWarpFlushAt = kWarpStage - 32;

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

__global__ void __launch_bounds__(kK1Threads, 2)
k1_stream(const float* __restrict__ g, float* __restrict__ r, const float* __restrict__ g_scale,
          const K1State* __restrict__ st, Pair* __restrict__ cand, unsigned int cap, Ctrl* ctrl,
          long long d) {
  __shared__ Pair wstage[kK1Threads / 32][kWarpStage];
  __shared__ unsigned int shist[kHistBins];  // first radix digit of every candidate of this CTA
  for (int i = threadIdx.x; i < kHistBins; i += kK1Threads) shist[i] = 0u;
  __syncthreads();
  Pair* wbuf = wstage[threadIdx.x >> 5];
  unsigned int wcnt = 0;
  const float tau = st->tau;
  const float scale = g_scale ? *g_scale : 1.0f;
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
  const long long ntiles = (nvec + kTileVec - 1) / kTileVec;
  for (long long tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
    const long long v0 = tile * kTileVec + threadIdx.x;
    float4 gv[kK1Vec], rv[kK1Vec];
#pragma unroll
    for (int u = 0; u < kK1Vec; ++u) {
      const long long v = v0 + (long long)u * kK1Threads;
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
      const long long v = v0 + (long long)u * kK1Threads;
      const bool inb = v < nvec;
      float a[4];
      a[0] = fmaf(gv[u].x, scale, rv[u].x);
      a[1] = fmaf(gv[u].y, scale, rv[u].y);
      a[2] = fmaf(gv[u].z, scale, rv[u].z);
      a[3] = fmaf(gv[u].w, scale, rv[u].w);
      bool c[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) c[e] = inb && (fabsf(a[e]) >= tau);
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
              atomicAdd(&shist[mag_key(a[e]) >> 20], 1u);
            }
            wcnt += __popc(m);
            if (wcnt > (unsigned int)kWarpFlushAt) warp_flush(wbuf, wcnt, cand, cap, counter, r);
          }
        }
      }
    }
  }
  // Scalar head and tail (at most 3 + 3 entries), one warp of CTA 0.
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
        c = fabsf(a) >= tau;
        r[i] = c ? 0.f : a;
      }
      const unsigned int m = __ballot_sync(0xffffffffu, c);
      if (m) {
        if (c) {
          Pair p;
          p.idx = (int32_t)i;
          p.val = a;
          wbuf[wcnt + __popc(m & lanemask_lt())] = p;
          atomicAdd(&shist[mag_key(a) >> 20], 1u);
        }
        wcnt += __popc(m);
        if (wcnt > (unsigned int)kWarpFlushAt) warp_flush(wbuf, wcnt, cand, cap, counter, r);
      }
    }
  }
  if (wcnt) warp_flush(wbuf, wcnt, cand, cap, counter, r);
  // publish this CTA's part of the first-pass histogram (k1_finish starts from it)
  __syncthreads();
  for (int i = threadIdx.x; i < kHistBins; i += kK1Threads) {
    const unsigned int c = shist[i];
    if (c) atomicAdd(&ctrl->hist[0][0][i], c);
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

__global__ void __launch_bounds__(kSelThreads)
k1_finish(float* __restrict__ r, long long d, Pair* __restrict__ cand, unsigned int cap,
          Pair* __restrict__ sel, unsigned int k, K1State* st, Ctrl* ctrl, float target_ratio,
          unsigned long long limit_ns) {
  __shared__ SelectShared s;
  const unsigned int count = ctrl->n_out;
  const unsigned int C = count < cap ? count : cap;
  const bool exact_mode = (count > cap) || (C < k);
  Threshold th;
  auto none = [](Pair, unsigned int) {};

  if (!exact_mode) {
    unsigned int nct = (C + 1023u) / 1024u;  // one or two candidates per thread and pass
    if (nct < 1u) nct = 1u;
    if (nct > gridDim.x) nct = gridDim.x;
    if (blockIdx.x >= nct) return;
    RankBarrier bar{ctrl, nct, 0u, limit_ns};
    auto key_at = [&](unsigned int i) -> uint32_t { return mag_key(cand[i].val); };
    if (!radix_select_kth(s, bar, blockIdx.x, nct, C, k, ctrl->hist[0], key_at, &th, 100, true))
      return;
    StagedAppender app{&s, sel, &ctrl->cursor[0], k, ctrl};
    app.begin();
    const unsigned int stride = nct * kSelThreads;
    const unsigned int trips = (C + stride - 1) / stride;
    for (unsigned int t = 0; t < trips; ++t) {
      const unsigned int i = t * stride + blockIdx.x * kSelThreads + threadIdx.x;
      if (i < C) {
        const Pair e = cand[i];
        if (passes_threshold(mag_key(e.val), th, &ctrl->tie[0])) {
          app.put(e);
        } else {
          r[e.idx] = e.val;
        }
      }
      app.end_tile(none);
    }
    app.flush(none);
    if (blockIdx.x == 0 && threadIdx.x == 0) {
      const float t_k = __uint_as_float(th.key);
      const float tau_used = st->tau;
      st->n_sel = k;
      st->n_cand = count;
      st->fallback = 0u;
      st->n_calls += 1u;
      st->kth_mag = t_k;
      st->tau = predict_tau(t_k, tau_used, C, k, target_ratio);
    }
    return;
  }

  // Exact mode: every CTA of the grid takes part.
  const unsigned int nct = gridDim.x;
  RankBarrier bar{ctrl, nct, 0u, limit_ns};
  const unsigned int stride = nct * kSelThreads;
  for (unsigned int i = blockIdx.x * kSelThreads + threadIdx.x; i < C; i += stride) {
    const Pair e = cand[i];
    r[e.idx] = e.val;
  }
  if (!bar.sync(110)) return;
  const unsigned int n = (unsigned int)d;
  auto key_at = [&](unsigned int i) -> uint32_t { return mag_key(__ldcg(&r[i])); };
  if (!radix_select_kth(s, bar, blockIdx.x, nct, n, k, ctrl->hist[1], key_at, &th, 120)) return;
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
    st->n_calls += 1u;
    st->kth_mag = t_k;
    st->tau = predict_tau(t_k, 0.f, 0u, k, target_ratio);
  }
}

}  // namespace gtk

using namespace gtk;

extern "C" unsigned long long gtk_ctrl_bytes(void) { return sizeof(Ctrl); }

extern "C" int gtk_k1_select(const float* g, float* r, const float* g_scale, long long d,
                             unsigned int k, void* cand, unsigned int cap, void* sel, void* state,
                             void* ctrl, float target_ratio, unsigned long long limit_ns,
                             void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (d <= 0 || d >= (1ll << 31) || k == 0 || k > cap) return GTK_ERR_ARG;
  // g and r must share their offset inside a 16-byte line (same flat layout)
  if ((reinterpret_cast<uintptr_t>(g) & 15u) != (reinterpret_cast<uintptr_t>(r) & 15u) ||
      (reinterpret_cast<uintptr_t>(r) & 3u) != 0u)
    return GTK_ERR_ARG;
  const DeviceInfo* di = gtk_device_info();
  if (!di) return GTK_ERR_CUDA;
  // header + trace + the two histogram sets K1 can touch
  const size_t clear_bytes = offsetof(Ctrl, hist) + 2 * sizeof(((Ctrl*)0)->hist[0]);
  cudaError_t e = cudaMemsetAsync(ctrl, 0, clear_bytes, stream);
  if (e != cudaSuccess) return GTK_ERR_CUDA;
  const long long nvec = d / 4;
  const long long tile = (long long)kK1Threads * kK1Vec;
  long long ntiles = (nvec + tile - 1) / tile;
  int grid = di->sms * 2;
  if (ntiles < grid) grid = ntiles > 0 ? (int)ntiles : 1;
  k1_stream<<<grid, kK1Threads, 0, stream>>>(g, r, g_scale, (const K1State*)state, (Pair*)cand, cap,
                                             (Ctrl*)ctrl, d);
  gtk_count_launch(1);
  static int finish_grid = 0;
  if (!finish_grid) {
    int occ = 0;
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, k1_finish, kSelThreads, 0);
    if (occ < 1) return GTK_ERR_CUDA;
    if (occ > 2) occ = 2;
    finish_grid = di->sms * occ;
  }
  float* r_ = r;
  Pair* cand_ = (Pair*)cand;
  Pair* sel_ = (Pair*)sel;
  K1State* st_ = (K1State*)state;
  Ctrl* ctrl_ = (Ctrl*)ctrl;
  void* args[] = {&r_, &d, &cand_, &cap, &sel_, &k, &st_, &ctrl_, &target_ratio, &limit_ns};
  e = cudaLaunchCooperativeKernel((void*)k1_finish, dim3(finish_grid), dim3(kSelThreads), args, 0,
                                  stream);
  gtk_count_launch(1);
  if (e != cudaSuccess) return GTK_ERR_CUDA;
  return cudaGetLastError() == cudaSuccess ? GTK_OK : GTK_ERR_CUDA;
}

// ---------------------------------------------------------------------------
// Allocation-free variant (declared and documented in k1_select_noalloc.h).
// The scratch that gtk_k1_select takes from its caller lives here in a static
// device array; the kernels are the ones above, unchanged.
// ---------------------------------------------------------------------------
#include <mutex>
#include "k1_select_noalloc.h"

namespace {

constexpr unsigned int kNoAllocMaxK = 16384u;
constexpr unsigned int kNoAllocCap = 131072u;                         // candidate pairs (8 x max k)
constexpr size_t kNoAllocCtrlOff = 0;
constexpr size_t kNoAllocStateOff = (sizeof(Ctrl) + 255) / 256 * 256;
constexpr size_t kNoAllocCandOff = kNoAllocStateOff + 256;
constexpr size_t kNoAllocBytes = kNoAllocCandOff + (size_t)kNoAllocCap * sizeof(Pair);

// In host code this name is only a handle for cudaGetSymbolAddress, never an address.
static __device__ __align__(256) unsigned char g_k1_noalloc_scratch[kNoAllocBytes];

__global__ void k1_noalloc_reset_state(K1State* st) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    st->tau = __int_as_float(0x7f800000);  // +inf: the next call takes the exact path
    st->n_sel = 0u;
    st->n_cand = 0u;
    st->fallback = 0u;
    st->n_fallbacks = 0u;
    st->n_calls = 0u;
    st->kth_mag = 0.f;
    st->reserved = 0u;
  }
}

__global__ void k1_noalloc_publish_count(const K1State* st, unsigned int* n_sel_out) {
  if (threadIdx.x == 0 && blockIdx.x == 0) *n_sel_out = st->n_sel;
}

struct NoAllocDevice {
  unsigned char* base = nullptr;  // device address of g_k1_noalloc_scratch on this device
  int finish_grid = 0;
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
      int occ = 0;
      if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, k1_finish, kSelThreads, 0) !=
              cudaSuccess || occ < 1)
        return GTK_ERR_CUDA;
      slot.finish_grid = di->sms * (occ > 2 ? 2 : occ);
      slot.base = static_cast<unsigned char*>(p);
      first = true;
    }
    dev = slot;
  }
  Ctrl* ctrl = reinterpret_cast<Ctrl*>(dev.base + kNoAllocCtrlOff);
  K1State* st = reinterpret_cast<K1State*>(dev.base + kNoAllocStateOff);
  Pair* cand = reinterpret_cast<Pair*>(dev.base + kNoAllocCandOff);
  unsigned int cap = kNoAllocCap;
  if (first || reset_threshold) {
    k1_noalloc_reset_state<<<1, 32, 0, stream>>>(st);
    gtk_count_launch(1);
  }
  // the control block must start at zero; everything else in the scratch is overwritten before use
  if (cudaMemsetAsync(ctrl, 0, sizeof(Ctrl), stream) != cudaSuccess) return GTK_ERR_CUDA;
  const long long nvec = d / 4;
  const long long tile = (long long)kK1Threads * kK1Vec;
  const long long ntiles = (nvec + tile - 1) / tile;
  int grid = di->sms * 2;
  if (ntiles < grid) grid = ntiles > 0 ? (int)ntiles : 1;
  k1_stream<<<grid, kK1Threads, 0, stream>>>(g, r, nullptr, st, cand, cap, ctrl, d);
  gtk_count_launch(1);
  Pair* sel = static_cast<Pair*>(sel_out);
  float target_ratio = 3.0f;
  unsigned long long limit_ns = 2000000000ull;
  void* args[] = {&r, &d, &cand, &cap, &sel, &k, &st, &ctrl, &target_ratio, &limit_ns};
  if (cudaLaunchCooperativeKernel((void*)k1_finish, dim3(dev.finish_grid), dim3(kSelThreads), args,
                                  0, stream) != cudaSuccess)
    return GTK_ERR_CUDA;
  gtk_count_launch(1);
  if (n_sel_out) {
    k1_noalloc_publish_count<<<1, 32, 0, stream>>>(st, n_sel_out);
    gtk_count_launch(1);
  }
  return cudaGetLastError() == cudaSuccess ? GTK_OK : GTK_ERR_CUDA;
}
