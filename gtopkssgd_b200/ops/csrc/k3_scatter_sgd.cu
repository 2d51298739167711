// K3: sparse scatter + averaging + weight decay + momentum/nesterov SGD over the
// flat parameter and momentum buffers.
//
// Replaces, in the reference: fill_(0) + scatter of the global values + "/= P"
// (allreducer.py:458-475) and the per-parameter SGD loop of
// distributed_optimizer.py:105-143 (d_p += wd*p; buf = m*buf + d_p, first step
// buf = d_p; nesterov d_p += m*buf; p -= lr*d_p), three launches per tensor.
//
// The update is split so that the dense gradient is never built:
//   dense part   g = wd*p (+ coef*scale*g_dense in dense mode);
//                buf = m*buf + f*g;  p -= lr*(nesterov ? g + m*buf : buf)
//                -- independent of the exchange, so it may run while K2 is in flight.
//   sparse part  for each global pair (j, v): s = coef*scale*v, sb = f*s;
//                buf[j] += sb;  p[j] -= lr*(nesterov ? s + m*sb : sb)
// where f = 1 on the first step and 1 - dampening afterwards.  Both parts add up
// to the reference's update because it is affine in the gradient.
#include "common.cuh"
#include "host_api.h"

namespace gtk {

constexpr int kK3Threads = 512;

// Sparse inputs may live in a two-parity buffer written by the exchange kernel:
// the segment base is pairs + ((*parity_word - 1) & 1) * parity_stride, where
// parity_word is the exchange's call counter after the call (nullptr: no offset).
__device__ __forceinline__ const Pair* parity_base(const Pair* pairs, const unsigned int* parity_word,
                                                   unsigned int parity_stride) {
  if (!parity_word) return pairs;
  return pairs + (size_t)((*parity_word - 1u) & 1u) * parity_stride;
}

struct SgdHyper {
  const float* lr_ptr;  // device-resident learning rate (read when non-null; lets a captured graph follow a schedule)
  float lr;
  float momentum;
  float dampening;
  float weight_decay;
  int nesterov;
  int first_step;
};

template <bool HAS_G, bool HAS_BUF>
__global__ void __launch_bounds__(kK3Threads, 2)
k3_dense(float* __restrict__ p, float* __restrict__ buf, const float* __restrict__ g,
         const float* __restrict__ coef_ptr, float scale, long long d, SgdHyper h) {
  if (h.lr_ptr) h.lr = *h.lr_ptr;
  const float coef = (HAS_G && coef_ptr) ? (*coef_ptr) * scale : scale;
  const float f = h.first_step ? 1.0f : 1.0f - h.dampening;
  const float m = h.momentum;
  auto upd = [&](float& pj, float& bj, float gj) {
    float gr = h.weight_decay * pj;
    if (HAS_G) gr = fmaf(gj, coef, gr);
    float step = gr;
    if (HAS_BUF) {
      bj = fmaf(m, bj, f * gr);
      step = h.nesterov ? fmaf(m, bj, gr) : bj;
    }
    pj = fmaf(-h.lr, step, pj);
  };
  const unsigned int mis = (unsigned int)((reinterpret_cast<uintptr_t>(p) >> 2) & 3u);
  long long head = mis ? (4 - mis) : 0;
  if (head > d) head = d;
  const long long nvec = (d - head) >> 2;
  const long long tail0 = head + (nvec << 2);
  float4* p4 = reinterpret_cast<float4*>(p + head);
  float4* b4 = reinterpret_cast<float4*>(buf + head);
  const float4* g4 = reinterpret_cast<const float4*>(g + head);
  const long long stride = (long long)gridDim.x * kK3Threads;
  for (long long v = (long long)blockIdx.x * kK3Threads + threadIdx.x; v < nvec; v += 2 * stride) {
    const long long v1 = v + stride;
    const bool two = v1 < nvec;
    float4 pa = p4[v], pb = two ? p4[v1] : make_float4(0, 0, 0, 0);
    float4 ba = make_float4(0, 0, 0, 0), bb = ba, ga = ba, gb = ba;
    if (HAS_BUF) { ba = b4[v]; if (two) bb = b4[v1]; }
    if (HAS_G) { ga = __ldcs(&g4[v]); if (two) gb = __ldcs(&g4[v1]); }
    upd(pa.x, ba.x, ga.x); upd(pa.y, ba.y, ga.y); upd(pa.z, ba.z, ga.z); upd(pa.w, ba.w, ga.w);
    p4[v] = pa;
    if (HAS_BUF) b4[v] = ba;
    if (two) {
      upd(pb.x, bb.x, gb.x); upd(pb.y, bb.y, gb.y); upd(pb.z, bb.z, gb.z); upd(pb.w, bb.w, gb.w);
      p4[v1] = pb;
      if (HAS_BUF) b4[v1] = bb;
    }
  }
  if (blockIdx.x == 0) {
    const long long nscalar = head + (d - tail0);
    for (long long j = threadIdx.x; j < nscalar; j += kK3Threads) {
      const long long i = j < head ? j : tail0 + (j - head);
      float pj = p[i], bj = HAS_BUF ? buf[i] : 0.f, gj = HAS_G ? g[i] : 0.f;
      upd(pj, bj, gj);
      p[i] = pj;
      if (HAS_BUF) buf[i] = bj;
    }
  }
}

// Sparse part.  `pairs` holds nseg segments of seg_stride pairs; segment s has
// counts[s] live pairs.  use_atomics: indices may repeat across segments.
__global__ void __launch_bounds__(256)
k3_sparse(float* __restrict__ p, float* __restrict__ buf, const Pair* __restrict__ pairs,
          const unsigned int* __restrict__ counts, unsigned int nseg, unsigned int seg_stride,
          const float* __restrict__ coef_ptr, float scale, unsigned int d, SgdHyper h,
          int use_atomics, unsigned int* __restrict__ bad_index_count,
          const unsigned int* __restrict__ parity_word, unsigned int parity_stride) {
  if (h.lr_ptr) h.lr = *h.lr_ptr;
  pairs = parity_base(pairs, parity_word, parity_stride);
  const float coef = coef_ptr ? (*coef_ptr) * scale : scale;
  const float f = h.first_step ? 1.0f : 1.0f - h.dampening;
  const bool has_buf = buf != nullptr && h.momentum != 0.f;
  const unsigned int stride = gridDim.x * blockDim.x;
  for (unsigned int s = 0; s < nseg; ++s) {
    unsigned int n = counts[s];
    if (n > seg_stride) n = seg_stride;
    const Pair* seg = pairs + (size_t)s * seg_stride;
    for (unsigned int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
      const Pair e = seg[i];
      if ((unsigned int)e.idx >= d) {
        atomicAdd(bad_index_count, 1u);
        continue;
      }
      const float sv = e.val * coef;
      float step = sv;
      if (has_buf) {
        const float sb = f * sv;
        if (use_atomics) atomicAdd(&buf[e.idx], sb);
        else buf[e.idx] += sb;
        step = h.nesterov ? fmaf(h.momentum, sb, sv) : sb;
      }
      if (use_atomics) atomicAdd(&p[e.idx], -h.lr * step);
      else p[e.idx] = fmaf(-h.lr, step, p[e.idx]);
    }
  }
}

// Optional: build the dense averaged gradient (for callers that want to look at
// p.grad after synchronize()).  g must have been zeroed by the caller.
__global__ void __launch_bounds__(256)
k3_scatter_dense(float* __restrict__ g, const Pair* __restrict__ pairs,
                 const unsigned int* __restrict__ counts, unsigned int nseg,
                 unsigned int seg_stride, float scale, unsigned int d, int use_atomics,
                 const unsigned int* __restrict__ parity_word, unsigned int parity_stride) {
  pairs = parity_base(pairs, parity_word, parity_stride);
  const unsigned int stride = gridDim.x * blockDim.x;
  for (unsigned int s = 0; s < nseg; ++s) {
    unsigned int n = counts[s];
    if (n > seg_stride) n = seg_stride;
    const Pair* seg = pairs + (size_t)s * seg_stride;
    for (unsigned int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
      const Pair e = seg[i];
      if ((unsigned int)e.idx >= d) continue;
      if (use_atomics) atomicAdd(&g[e.idx], e.val * scale);
      else g[e.idx] = e.val * scale;
    }
  }
}

// Momentum correction (distributed_optimizer.py:81-88 in the reference, off by default there): the
// velocity, not the raw gradient, is what gets sparsified.  v = m*v + g; g = v, over a whole merged
// group in one pass (the reference does it per parameter tensor inside the gradient hook).
__global__ void __launch_bounds__(kK3Threads, 2)
k3_momentum_correct(float* __restrict__ v, float* __restrict__ g, float m, long long d) {
  const unsigned int mis = (unsigned int)((reinterpret_cast<uintptr_t>(g) >> 2) & 3u);
  long long head = mis ? (4 - mis) : 0;
  if (head > d) head = d;
  const long long nvec = (d - head) >> 2;
  const long long tail0 = head + (nvec << 2);
  float4* v4 = reinterpret_cast<float4*>(v + head);
  float4* g4 = reinterpret_cast<float4*>(g + head);
  const long long stride = (long long)gridDim.x * kK3Threads;
  for (long long i = (long long)blockIdx.x * kK3Threads + threadIdx.x; i < nvec; i += stride) {
    float4 a = v4[i];
    const float4 b = g4[i];
    a.x = fmaf(m, a.x, b.x); a.y = fmaf(m, a.y, b.y); a.z = fmaf(m, a.z, b.z); a.w = fmaf(m, a.w, b.w);
    v4[i] = a;
    g4[i] = a;
  }
  if (blockIdx.x == 0) {
    const long long nscalar = head + (d - tail0);
    for (long long j = threadIdx.x; j < nscalar; j += kK3Threads) {
      const long long i = j < head ? j : tail0 + (j - head);
      const float a = fmaf(m, v[i], g[i]);
      v[i] = a;
      g[i] = a;
    }
  }
}

}  // namespace gtk

using namespace gtk;

static int dense_grid(long long d) {
  const DeviceInfo* di = gtk_device_info();
  const int sms = di ? di->sms : 148;
  long long need = (d / 4 + 2ll * kK3Threads - 1) / (2ll * kK3Threads);
  long long grid = (long long)sms * 2;
  if (need < grid) grid = need > 0 ? need : 1;
  return (int)grid;
}

extern "C" int gtk_k3_dense(float* p, float* buf, const float* g, const float* coef, float scale,
                            long long d, float lr, const float* lr_ptr, float momentum, float dampening,
                            float weight_decay, int nesterov, int first_step, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (d <= 0) return GTK_ERR_ARG;
  const bool has_buf = momentum != 0.f && buf != nullptr;
  const bool has_g = g != nullptr;
  if (!has_g && !has_buf && weight_decay == 0.f) return GTK_OK;  // nothing to do
  const uintptr_t a = reinterpret_cast<uintptr_t>(p) & 15u;
  if ((has_buf && (reinterpret_cast<uintptr_t>(buf) & 15u) != a) ||
      (has_g && (reinterpret_cast<uintptr_t>(g) & 15u) != a))
    return GTK_ERR_ARG;
  SgdHyper h{lr_ptr, lr, momentum, dampening, weight_decay, nesterov, first_step};
  const int grid = dense_grid(d);
  if (has_g && has_buf) k3_dense<true, true><<<grid, kK3Threads, 0, stream>>>(p, buf, g, coef, scale, d, h);
  else if (has_g) k3_dense<true, false><<<grid, kK3Threads, 0, stream>>>(p, p, g, coef, scale, d, h);
  else if (has_buf) k3_dense<false, true><<<grid, kK3Threads, 0, stream>>>(p, buf, p, coef, scale, d, h);
  else k3_dense<false, false><<<grid, kK3Threads, 0, stream>>>(p, p, p, coef, scale, d, h);
  gtk_count_launch(1);
  return cudaGetLastError() == cudaSuccess ? GTK_OK : GTK_ERR_CUDA;
}

extern "C" int gtk_k3_sparse(float* p, float* buf, const void* pairs, const unsigned int* counts,
                             unsigned int nseg, unsigned int seg_stride, const float* coef,
                             float scale, unsigned int d, float lr, const float* lr_ptr, float momentum,
                             float dampening, float weight_decay, int nesterov, int first_step,
                             int use_atomics, unsigned int* bad_index_count,
                             const unsigned int* parity_word, unsigned int parity_stride,
                             void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (nseg == 0 || seg_stride == 0) return GTK_ERR_ARG;
  SgdHyper h{lr_ptr, lr, momentum, dampening, weight_decay, nesterov, first_step};
  unsigned int blocks = (seg_stride + 255u) / 256u;
  if (blocks > 1184u) blocks = 1184u;
  k3_sparse<<<blocks, 256, 0, stream>>>(p, buf, (const Pair*)pairs, counts, nseg, seg_stride, coef,
                                        scale, d, h, use_atomics, bad_index_count, parity_word,
                                        parity_stride);
  gtk_count_launch(1);
  return cudaGetLastError() == cudaSuccess ? GTK_OK : GTK_ERR_CUDA;
}

extern "C" int gtk_k3_scatter_dense(float* g, const void* pairs, const unsigned int* counts,
                                    unsigned int nseg, unsigned int seg_stride, float scale,
                                    long long d, int use_atomics, const unsigned int* parity_word,
                                    unsigned int parity_stride, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (cudaMemsetAsync(g, 0, (size_t)d * sizeof(float), stream) != cudaSuccess) return GTK_ERR_CUDA;
  unsigned int blocks = (seg_stride + 255u) / 256u;
  if (blocks > 1184u) blocks = 1184u;
  k3_scatter_dense<<<blocks, 256, 0, stream>>>(g, (const Pair*)pairs, counts, nseg, seg_stride,
                                               scale, (unsigned int)d, use_atomics, parity_word,
                                               parity_stride);
  gtk_count_launch(1);
  return cudaGetLastError() == cudaSuccess ? GTK_OK : GTK_ERR_CUDA;
}

extern "C" int gtk_k3_momentum_correct(float* v, float* g, float momentum, long long d, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (d <= 0 || !v || !g) return GTK_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(v) & 15u) != (reinterpret_cast<uintptr_t>(g) & 15u)) return GTK_ERR_ARG;
  k3_momentum_correct<<<dense_grid(d), kK3Threads, 0, stream>>>(v, g, momentum, d);
  gtk_count_launch(1);
  return cudaGetLastError() == cudaSuccess ? GTK_OK : GTK_ERR_CUDA;
}
