// K2t: Top-k all-gather exchange ('topk') and its re-selecting variant ('topk2').
//
// 'topk'  (allreducer.py:29-64 + 461-466 in the reference): every rank ends
//         with all P selections; the dense result is the sum of the P sparse
//         vectors, nothing returns to the residual.  Here each rank pushes its k
//         pairs into slot[rank] of every peer with NVLink peer stores and one
//         flag per source; the consumer (K3, atomic mode) applies the P segments.
// 'topk2' (allreducer.py:467-473): the summed vector is re-sparsified to its k
//         largest magnitudes, and locally selected entries that did not survive
//         return to the residual.  Here the P lists are merged in rank order
//         (same arithmetic on every rank, so all ranks get the same set) with
//         the direct-address table, then radix-selected.
#include "exchange_common.cuh"

namespace gtk {

__global__ void __launch_bounds__(kSelThreads)
k2t_topk_allgather(const K2Rank* __restrict__ ranks, unsigned int rank_base, unsigned int P,
                   unsigned int k, unsigned int kcap, unsigned int work_cap, unsigned int d,
                   int reselect, unsigned int* __restrict__ seg_counts_all,
                   unsigned long long limit_ns) {
  __shared__ ExchangeShared sh;
  const K2Rank& R = ranks[blockIdx.y];
  const unsigned int epoch = __ldcg(R.epoch);
  const unsigned int me = rank_base + blockIdx.y;
  const unsigned int cta = blockIdx.x, nct = gridDim.x;
  const unsigned int parity = epoch & 1u;
  Ctrl* ctrl = R.ctrl;
  RankBarrier bar{ctrl, nct, 0u, limit_ns};
  unsigned int* seg_counts = seg_counts_all + (size_t)blockIdx.y * kMaxPeers;

  // A call that gives up leaves EMPTY results (no segment, no global pair: the consumer applies
  // nothing) and a sticky status; later calls return at once until the host rebuilds the exchange.
  auto fail = [&]() {
    if (threadIdx.x == 0) {
      atomicExch(&R.n_global[kResCount], 0u);
      if (cta == 0)
        for (unsigned int q = 0; q < (unsigned int)kMaxPeers; ++q) seg_counts[q] = 0u;
      unsigned int st = ld_relaxed_gpu_u32(&ctrl->status);
      if (st == 0u) st = ST_TIMEOUT_BARRIER;
      if (atomicCAS(&R.n_global[kResStatus], 0u, st) == 0u) {
        R.n_global[kResWhere] = ld_relaxed_gpu_u32(&ctrl->where);
        R.n_global[kResEpoch] = epoch;
      }
    }
  };
  if (__ldcg(&R.n_global[kResStatus]) != 0u) {
    if (cta == 0 && threadIdx.x < (unsigned int)kMaxPeers) seg_counts[threadIdx.x] = 0u;
    if (cta == 0 && threadIdx.x == 0) R.n_global[kResCount] = 0u;
    return;
  }

  unsigned int n_sel = R.st->n_sel;
  if (n_sel > kcap) n_sel = kcap;

  // push my selection into slot[me] of every rank (my own included)
  for (unsigned int q = 0; q < P; ++q) {
    Pair* dst = (q == me ? R.ag : R.peer_ag[q]) + ag_off(parity, me, kcap);
    push_pairs(dst, R.sel, n_sel, cta, nct);
  }
  cta_fence_peer_stores(nct == 1);
  if (!bar.sync(500)) { fail(); return; }
  if (cta == 0 && threadIdx.x < P && threadIdx.x != me)  // one releasing thread per destination
    release_flag(R.peer_flags[threadIdx.x] + flag_off(parity, kFlagAg0 + me), epoch, n_sel);
  // wait for every source
  unsigned int counts[kMaxPeers];
  for (unsigned int q = 0; q < P; ++q) {
    unsigned int c = n_sel;
    if (q != me) {
      if (!cta_wait_flag(sh, R.flags + flag_off(parity, kFlagAg0 + q), epoch, ctrl, limit_ns,
                         510 + q, &c)) {
        fail();
        return;
      }
      if (c > kcap) {
        record_error(ctrl, ST_CAPACITY, 530 + q);
        c = kcap;
      }
    }
    counts[q] = c;
  }
  if (cta == 0 && threadIdx.x < P) seg_counts[threadIdx.x] = counts[threadIdx.x];
  if (!reselect) {
    if (!bar.sync(535)) { fail(); return; }  // every CTA has read the epoch word
    if (cta == 0 && threadIdx.x == 0) {
      if (aborted(ctrl)) fail();
      else *R.epoch = epoch + 1u;
    }
    return;
  }

  // ---- topk2: merge the P lists in rank order, then keep the k largest sums
  Pair* A = R.work[0];
  const Pair* L0 = R.ag + ag_off(parity, 0, kcap);
  copy_and_map(A, L0, counts[0], R.map, d, cta, nct, ctrl);
  unsigned int n_a = counts[0];
  if (cta == 0 && threadIdx.x == 0) ctrl->n_live = n_a;
  if (!bar.sync(540)) { fail(); return; }
  const unsigned int stride = nct * kSelThreads;
  for (unsigned int q = 1; q < P; ++q) {
    const Pair* B = R.ag + ag_off(parity, q, kcap);
    const unsigned int n_b = counts[q];
    const unsigned int trips = (n_b + stride - 1) / stride;
    for (unsigned int t = 0; t < trips; ++t) {
      const unsigned int j = t * stride + cta * kSelThreads + threadIdx.x;
      bool append = false;
      Pair e;
      e.idx = -1;
      e.val = 0.f;
      if (j < n_b) {
        e = ld_pair_cg(&B[j]);
        if ((unsigned int)e.idx >= d) {
          record_error(ctrl, ST_BOUNDS, 550);
        } else {
          append = true;
          const unsigned int p = (unsigned int)__ldcg(&R.map[e.idx]);
          if (p < n_a) {
            const Pair a = ld_pair_cg(&A[p]);
            if (a.idx == e.idx) {
              A[p].val = a.val + e.val;
              append = false;
            }
          }
        }
      }
      const unsigned int m = __ballot_sync(0xffffffffu, append);
      if (m) {
        unsigned int base = 0;
        if (lane_id() == (unsigned int)(__ffs(m) - 1)) base = atomicAdd(&ctrl->n_live, __popc(m));
        base = __shfl_sync(0xffffffffu, base, __ffs(m) - 1);
        if (append) {
          const unsigned int pos = base + __popc(m & lanemask_lt());
          if (pos < work_cap) {
            st_pair(&A[pos], e);
            R.map[e.idx] = (int32_t)pos;
          } else {
            record_error(ctrl, ST_CAPACITY, 551);
          }
        }
      }
    }
    if (!bar.sync(560 + q)) { fail(); return; }
    n_a = __ldcg(&ctrl->n_live);
    if (n_a > work_cap) n_a = work_cap;
  }
  auto key_at = [&](unsigned int i) -> uint32_t { return mag_key(ld_pair_cg(&A[i]).val); };
  Threshold th;
  if (!radix_select_kth(sh.sel, bar, cta, nct, n_a, k, ctrl->hist[0], key_at, &th, 580)) { fail(); return; }
  Pair* G = R.gout + (size_t)parity * kcap;
  int32_t* map = R.map;
  auto on_placed = [&](Pair e, unsigned int pos) { map[e.idx] = (int32_t)pos; };
  StagedAppender app{&sh.sel, G, &ctrl->cursor[0], kcap, ctrl};
  app.begin();
  const unsigned int trips = (n_a + stride - 1) / stride;
  for (unsigned int t = 0; t < trips; ++t) {
    const unsigned int i = t * stride + cta * kSelThreads + threadIdx.x;
    if (i < n_a) {
      const Pair e = ld_pair_cg(&A[i]);
      if (passes_threshold(mag_key(e.val), th, &ctrl->tie[0])) app.put(e);
    }
    app.end_tile(on_placed);
  }
  app.flush(on_placed);
  if (!bar.sync(590)) { fail(); return; }
  unsigned int n_g = __ldcg(&ctrl->cursor[0]);
  if (n_g > kcap) n_g = kcap;
  put_back(R.sel, n_sel, G, n_g, R.map, R.resid, d, cta, nct);
  if (!bar.sync(595)) { fail(); return; }
  if (cta == 0 && threadIdx.x == 0) {
    if (aborted(ctrl)) {
      fail();
    } else {
      R.n_global[kResCount] = n_g;
      *R.epoch = epoch + 1u;
    }
  }
}

}  // namespace gtk

using namespace gtk;

extern "C" int gtk_k2t_allgather(const void* ranks_dev, void* const* ctrl_dev, unsigned int nranks,
                                 unsigned int rank_base, unsigned int P, unsigned int k,
                                 unsigned int kcap, unsigned int work_cap, unsigned int d,
                                 int reselect, void* seg_counts,
                                 unsigned int nctas, unsigned long long limit_ns, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  if (P < 2 || P > (unsigned int)kMaxPeers) return GTK_ERR_ARG;
  if (k == 0 || k > kcap || nranks == 0 || nctas == 0) return GTK_ERR_ARG;
  const DeviceInfo* di = gtk_device_info();
  if (!di) return GTK_ERR_CUDA;
  static int occ = 0;
  if (!occ && cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, (const void*)k2t_topk_allgather,
                                                            kSelThreads, 0) != cudaSuccess)
    return GTK_ERR_CUDA;
  if ((int)(nranks * nctas) > occ * di->sms) return GTK_ERR_ARG;
  for (unsigned int i = 0; i < nranks; ++i)
    if (cudaMemsetAsync(ctrl_dev[i], 0, sizeof(Ctrl), stream) != cudaSuccess) return GTK_ERR_CUDA;
  const K2Rank* ranks = (const K2Rank*)ranks_dev;
  unsigned int* segc = (unsigned int*)seg_counts;
  void* args[] = {&ranks, &rank_base, &P, &k, &kcap, &work_cap, &d, &reselect, &segc, &limit_ns};
  cudaError_t e = cudaLaunchCooperativeKernel((void*)k2t_topk_allgather, dim3(nctas, nranks),
                                              dim3(kSelThreads), args, 0, stream);
  gtk_count_launch(1);
  return e == cudaSuccess ? GTK_OK : GTK_ERR_CUDA;
}
