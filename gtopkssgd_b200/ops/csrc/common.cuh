// Shared device-side building blocks for the gTop-k kernels (sm_100a).
//
// Everything that waits (flag waits, grid barriers) is bounded: after a time
// limit read from %globaltimer the waiter records an error status, raises the
// rank-wide abort word so that every other waiter of the same rank leaves too,
// and the kernel returns normally.  Nothing here traps or spins forever.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace gtk {

// One sparse gradient entry on the wire and in every work buffer: 8 bytes.
struct __align__(8) Pair {
  int32_t idx;
  float val;
};

// Status codes written to Ctrl::status (first error wins).
enum Status : uint32_t {
  ST_OK = 0,
  ST_TIMEOUT_FLAG = 1,     // a peer never raised its flag within the limit
  ST_TIMEOUT_BARRIER = 2,  // a CTA of this rank never reached the barrier
  ST_CAPACITY = 3,         // a list grew beyond its buffer
  ST_BOUNDS = 4,           // an index outside [0, d) was seen and skipped
};

constexpr int kHistBins = 2048;   // 11-bit first radix digit
constexpr int kMaxRounds = 4;     // log2(16) recursive-doubling rounds
constexpr int kMaxPeers = 16;
constexpr int kTraceSlots = 64;

// Per-rank control block.  The host clears it (one async memset) before every
// launch that uses it, so every counter starts at zero.
struct Ctrl {
  unsigned int bar;         // grid-barrier arrival counter
  unsigned int abort;       // non-zero: every wait returns at once
  unsigned int status;      // Status of the first failure
  unsigned int where;       // code location of the first failure
  unsigned int n_out;       // output cursor of the current compaction
  unsigned int n_tie;       // tickets handed to entries equal to the threshold
  unsigned int n_live;      // live entries of the current union
  unsigned int scratch[9];
  unsigned int cursor[kMaxRounds + 2];        // one output cursor per round
  unsigned int tie[kMaxRounds + 2];           // one tie counter per round
  unsigned int live[kMaxRounds + 2];
  unsigned int pad[64 - 16 - 3 * (kMaxRounds + 2)];
  unsigned long long trace[kTraceSlots];      // %globaltimer stamps of CTA 0 at phase boundaries
  // Radix histograms, one set of four rows per tree round (K2) or per use (K1: sets 0-2, rows 0-2).
  // K2 rows: 0 = first digit; 1 and 2[0..1023] = second digit of the entries whose first digit is one
  // of three predicted ones (1024 bins each); 2[1024..] = second digit counted by a sweep when the
  // prediction missed; 3 = third digit.
  unsigned int hist[kMaxRounds + 2][4][kHistBins];
};

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

struct Ctrl;
__device__ __forceinline__ void trace_stamp(Ctrl* c, int slot);

__device__ __forceinline__ uint64_t ld_acquire_sys_u64(const uint64_t* p) {
  uint64_t v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys_u64(uint64_t* p, uint64_t v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_gpu_u32(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned int ld_relaxed_gpu_u32(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_gpu_add(unsigned int* p, unsigned int v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Phase stamp for the device-side trace: thread 0 of the rank's CTA 0 only.
__device__ __forceinline__ void trace_stamp(Ctrl* c, int slot) {
  if (blockIdx.x == 0 && threadIdx.x == 0 && slot < kTraceSlots) c->trace[slot] = globaltimer_ns();
}

// Pair <-> 64-bit word, so that a pair always moves with one 8-byte access.
__device__ __forceinline__ unsigned long long pair_bits(Pair p) {
  return (unsigned long long)(uint32_t)p.idx | ((unsigned long long)__float_as_uint(p.val) << 32);
}
__device__ __forceinline__ Pair bits_pair(unsigned long long b) {
  Pair p;
  p.idx = (int32_t)(uint32_t)(b & 0xffffffffull);
  p.val = __uint_as_float((uint32_t)(b >> 32));
  return p;
}
// L1-bypassing load: data another GPU (or another CTA) wrote during this launch.
__device__ __forceinline__ Pair ld_pair_cg(const Pair* p) {
  return bits_pair(__ldcg(reinterpret_cast<const unsigned long long*>(p)));
}
__device__ __forceinline__ void st_pair(Pair* p, Pair v) {
  *reinterpret_cast<unsigned long long*>(p) = pair_bits(v);
}
// Magnitude key: the bit pattern of |v| orders like |v| for every finite value.
__device__ __forceinline__ uint32_t mag_key(float v) { return __float_as_uint(v) & 0x7fffffffu; }

__device__ __forceinline__ void record_error(Ctrl* c, uint32_t status, uint32_t where) {
  if (atomicCAS(&c->status, 0u, status) == 0u) c->where = where;
  atomicExch(&c->abort, 1u);
  __threadfence();
}

__device__ __forceinline__ bool aborted(const Ctrl* c) {
  return ld_relaxed_gpu_u32(&c->abort) != 0u;
}

// Barrier over the `nctas` CTAs that serve one rank.  `gen` is a per-thread
// running count of barriers passed (identical in all threads of all CTAs of the
// rank).  Returns false if the rank aborted or the limit ran out.
struct RankBarrier {
  Ctrl* ctrl;
  unsigned int nctas;
  unsigned int gen;
  uint64_t limit_ns;
  unsigned int* counter = nullptr;  // arrival counter; nullptr: ctrl->bar
  bool cluster = false;             // the rank's CTAs form one thread-block cluster: hardware barrier

  __device__ __forceinline__ bool sync(uint32_t where) {
    __shared__ int ok_s;
    unsigned int* const arrivals = counter ? counter : &ctrl->bar;
    if (nctas == 1) {  // a single CTA learns of its own failures through its shared flags
      __syncthreads();
      return true;
    }
    if (cluster) {
      // Cluster-scope release/acquire: global and shared writes made before the barrier by any
      // CTA of the cluster are visible to all of them after it.  The hardware barrier waits only
      // for threads that have not exited, so a CTA that gave up on a flag wait does not block it.
      asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
      asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
      return true;
    }
    gen += 1;
    __syncthreads();
    if (threadIdx.x == 0) {
      int ok = 1;
      __threadfence();
      red_release_gpu_add(arrivals, 1u);
      const unsigned int target = gen * nctas;
      const uint64_t t0 = globaltimer_ns();
      unsigned int spins = 0;
      while (ld_acquire_gpu_u32(arrivals) < target) {
        if (aborted(ctrl)) { ok = 0; break; }
        if ((++spins & 63u) == 0u && globaltimer_ns() - t0 > limit_ns) {
          record_error(ctrl, ST_TIMEOUT_BARRIER, where);
          ok = 0;
          break;
        }
      }
      if (ok && aborted(ctrl)) ok = 0;
      ok_s = ok;
    }
    __syncthreads();
    const bool ok = ok_s != 0;
    __syncthreads();
    return ok;
  }
};

// Bounded wait until the flag word carries `epoch` in its upper half.  Called by
// one thread.  Returns the flag's lower half (a count) through *payload.
__device__ __forceinline__ bool wait_flag(const uint64_t* flag, uint32_t epoch, Ctrl* ctrl,
                                          uint64_t limit_ns, uint32_t where, uint32_t* payload) {
  const uint64_t t0 = globaltimer_ns();
  unsigned int spins = 0;
  for (;;) {
    const uint64_t v = ld_acquire_sys_u64(flag);
    if ((uint32_t)(v >> 32) == epoch) {
      *payload = (uint32_t)(v & 0xffffffffull);
      return true;
    }
    if (aborted(ctrl)) return false;
    if ((++spins & 31u) == 0u) {
      if (globaltimer_ns() - t0 > limit_ns) {
        record_error(ctrl, ST_TIMEOUT_FLAG, where);
        return false;
      }
      __nanosleep(40);
    }
  }
}

// Warp-level helpers ---------------------------------------------------------
__device__ __forceinline__ unsigned int lane_id() { return threadIdx.x & 31u; }
__device__ __forceinline__ unsigned int lanemask_lt() {
  unsigned int m;
  asm("mov.u32 %0, %%lanemask_lt;" : "=r"(m));
  return m;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

}  // namespace gtk
