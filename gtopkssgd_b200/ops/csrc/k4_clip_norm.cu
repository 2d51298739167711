// K4: gradient-norm clipping without a host round trip.
//
// Replaces the reference's norm().item() + mul_ before compression
// (allreducer.py:531-538) and torch.nn.utils.clip_grad_norm_ on the reduced
// gradients (gtopk_trainer.py:81-86).  The squared norm is accumulated on the
// device (dense vector or sparse pairs, several calls may add into the same
// accumulator), a one-thread kernel turns it into
//     coef = min(1, max_norm / (scale * sqrt(sumsq) + 1e-6))
// and the consumers (K1 stream pass, K3) read coef from device memory.
#include "common.cuh"
#include "host_api.h"

namespace gtk {

struct ClipState {
  double sumsq;   // accumulator, cleared by finalize
  float norm;     // last norm (after scale)
  float coef;     // last clip coefficient
};

constexpr int kK4Threads = 512;

__device__ __forceinline__ void block_accumulate(double local, double* acc) {
  __shared__ double wsum[kK4Threads / 32];
  local = warp_sum(local);
  if (lane_id() == 0) wsum[threadIdx.x >> 5] = local;
  __syncthreads();
  if (threadIdx.x < 32) {
    double v = threadIdx.x < kK4Threads / 32 ? wsum[threadIdx.x] : 0.0;
    v = warp_sum(v);
    if (threadIdx.x == 0 && v != 0.0) atomicAdd(acc, v);
  }
}

__global__ void __launch_bounds__(kK4Threads)
k4_sumsq_dense(const float* __restrict__ x, long long d, ClipState* st) {
  const unsigned int mis = (unsigned int)((reinterpret_cast<uintptr_t>(x) >> 2) & 3u);
  long long head = mis ? (4 - mis) : 0;
  if (head > d) head = d;
  const long long nvec = (d - head) >> 2;
  const long long tail0 = head + (nvec << 2);
  const float4* x4 = reinterpret_cast<const float4*>(x + head);
  const long long stride = (long long)gridDim.x * kK4Threads;
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  double total = 0.0;
  int since = 0;
  for (long long v = (long long)blockIdx.x * kK4Threads + threadIdx.x; v < nvec; v += 4 * stride) {
    float4 a = x4[v];
    float4 b = v + stride < nvec ? x4[v + stride] : make_float4(0, 0, 0, 0);
    float4 c = v + 2 * stride < nvec ? x4[v + 2 * stride] : make_float4(0, 0, 0, 0);
    float4 e = v + 3 * stride < nvec ? x4[v + 3 * stride] : make_float4(0, 0, 0, 0);
    s0 += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
    s1 += b.x * b.x + b.y * b.y + b.z * b.z + b.w * b.w;
    s2 += c.x * c.x + c.y * c.y + c.z * c.z + c.w * c.w;
    s3 += e.x * e.x + e.y * e.y + e.z * e.z + e.w * e.w;
    if (++since == 64) {  // fold into double now and then to bound the fp32 error
      total += (double)s0 + (double)s1 + (double)s2 + (double)s3;
      s0 = s1 = s2 = s3 = 0.f;
      since = 0;
    }
  }
  total += (double)s0 + (double)s1 + (double)s2 + (double)s3;
  if (blockIdx.x == 0) {
    const long long nscalar = head + (d - tail0);
    for (long long j = threadIdx.x; j < nscalar; j += kK4Threads) {
      const long long i = j < head ? j : tail0 + (j - head);
      total += (double)x[i] * (double)x[i];
    }
  }
  block_accumulate(total, &st->sumsq);
}

__global__ void __launch_bounds__(kK4Threads)
k4_sumsq_pairs(const Pair* __restrict__ pairs, const unsigned int* __restrict__ counts,
               unsigned int nseg, unsigned int seg_stride, ClipState* st,
               const unsigned int* __restrict__ parity_word, unsigned int parity_stride) {
  if (parity_word) pairs += (size_t)((*parity_word - 1u) & 1u) * parity_stride;
  double total = 0.0;
  const unsigned int stride = gridDim.x * kK4Threads;
  for (unsigned int s = 0; s < nseg; ++s) {
    unsigned int n = counts[s];
    if (n > seg_stride) n = seg_stride;
    const Pair* seg = pairs + (size_t)s * seg_stride;
    for (unsigned int i = blockIdx.x * kK4Threads + threadIdx.x; i < n; i += stride) {
      const float v = seg[i].val;
      total += (double)v * (double)v;
    }
  }
  block_accumulate(total, &st->sumsq);
}

__global__ void k4_finalize(ClipState* st, float scale, float max_norm, float* coef_out) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    const float norm = scale * (float)sqrt(st->sumsq);
    float coef = max_norm / (norm + 1e-6f);
    if (!(coef < 1.0f)) coef = 1.0f;
    st->norm = norm;
    st->coef = coef;
    st->sumsq = 0.0;
    if (coef_out) *coef_out = coef;
  }
}

}  // namespace gtk

using namespace gtk;

extern "C" unsigned long long gtk_clipstate_bytes(void) { return sizeof(ClipState); }

extern "C" int gtk_k4_sumsq_dense(const float* x, long long d, void* state, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (d <= 0) return GTK_ERR_ARG;
  const DeviceInfo* di = gtk_device_info();
  const int sms = di ? di->sms : 148;
  long long need = (d / 4 + 4ll * kK4Threads - 1) / (4ll * kK4Threads);
  long long grid = (long long)sms * 4;
  if (need < grid) grid = need > 0 ? need : 1;
  k4_sumsq_dense<<<(int)grid, kK4Threads, 0, stream>>>(x, d, (ClipState*)state);
  gtk_count_launch(1);
  return cudaGetLastError() == cudaSuccess ? GTK_OK : GTK_ERR_CUDA;
}

extern "C" int gtk_k4_sumsq_pairs(const void* pairs, const unsigned int* counts, unsigned int nseg,
                                  unsigned int seg_stride, void* state,
                                  const unsigned int* parity_word, unsigned int parity_stride,
                                  void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (nseg == 0 || seg_stride == 0) return GTK_ERR_ARG;
  unsigned int blocks = (seg_stride + kK4Threads - 1) / kK4Threads;
  if (blocks > 592u) blocks = 592u;
  k4_sumsq_pairs<<<blocks, kK4Threads, 0, stream>>>((const Pair*)pairs, counts, nseg, seg_stride,
                                                    (ClipState*)state, parity_word, parity_stride);
  gtk_count_launch(1);
  return cudaGetLastError() == cudaSuccess ? GTK_OK : GTK_ERR_CUDA;
}

extern "C" int gtk_k4_finalize(void* state, float scale, float max_norm, float* coef_out,
                               void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  k4_finalize<<<1, 32, 0, stream>>>((ClipState*)state, scale, max_norm, coef_out);
  gtk_count_launch(1);
  return cudaGetLastError() == cudaSuccess ? GTK_OK : GTK_ERR_CUDA;
}
