// gtk_k1_select_noalloc: the fused residual-add + top-k select of K1 for
// callers that are not allowed to allocate device memory.
//
// This entry point has no counterpart in the reference (which has no native
// code at all); it exists for embedders of this library.
//
// Who needs it.  cudaMalloc / cudaFree are heavyweight calls: they synchronise
// the whole device, and they fail when some other component (a framework's
// caching allocator, a second process) already owns the memory.  A host
// application that runs this library under a fixed, pre-planned memory budget,
// or a latency-critical loop that cannot afford an implicit device-wide
// synchronisation, therefore cannot use an interface that makes it allocate
// the candidate list and control block the regular entry point
// (gtk_k1_select) expects from its caller.
//
// What it does.  Same operation and same result as gtk_k1_select:
//     acc = g + r;  sel_out <- the k largest-magnitude (int32 idx, fp32 acc) pairs;
//     r <- acc off the selection, 0 on it;  g is not modified.
// The scratch memory (control block, threshold-prediction state, candidate
// list; about 1.5 MB) lives in a file-scope static __device__ array inside the
// library, so every GPU that loads the library holds that array until the
// process exits.  The caller passes only inputs and outputs.  No call to
// cudaMalloc, cudaFree or any allocating library routine is made.
//
// Limits and rules.
//  * k <= gtk_k1_noalloc_max_k() (16384); larger k is refused with
//    GTK_ERR_TOO_LARGE and nothing is enqueued.  1 <= d < 2^31.  g and r must be
//    4-byte aligned and share their offset within a 16-byte line; sel_out must be
//    8-byte aligned and n_sel_out 4-byte aligned (GTK_ERR_ARG otherwise: a pair is
//    stored with one 8-byte access).
//  * Device-side failures (the grid barrier running into its 2 s limit) are not
//    visible in the outputs.  gtk_k1_noalloc_status reads the status words out of
//    the scratch and, on request, clears the scratch so that the next call starts
//    clean; call it whenever the result matters more than the time of one stream
//    synchronisation.
//  * All calls on one device share the one scratch array.  Two calls that overlap
//    on the GPU (different streams without ordering, or several host threads)
//    race on it: order them on one stream or with events.
//  * The array keeps the previous call's contents.  What has to start at zero is
//    the control block of a call: the array holds two of them, every call clears
//    the one the next call will use, and static device storage starts zeroed.
//    The predicted threshold is deliberately kept (it only steers speed, never
//    the result) and is forgotten when reset_threshold != 0.
//  * The first call on each device resolves the device address of the scratch
//    array (cudaGetSymbolAddress) and initialises the threshold state.  Make that
//    first call before any stream capture begins.
#pragma once
#include "host_api.h"

#ifdef __cplusplus
extern "C" {
#endif

#define GTK_ERR_TOO_LARGE (-4)

// Largest k the static scratch can serve.
unsigned int gtk_k1_noalloc_max_k(void);
// Bytes of the static scratch array (held per GPU for the life of the process).
unsigned long long gtk_k1_noalloc_scratch_bytes(void);

// g, r: device pointers to d floats.  sel_out: device buffer of at least k pairs
// (8 bytes each).  n_sel_out: optional device word receiving the number of
// pairs written (k, or fewer when d < k).  Enqueues on `stream` and returns.
int gtk_k1_select_noalloc(const float* g, float* r, long long d, unsigned int k, void* sel_out,
                          unsigned int* n_sel_out, int reset_threshold, void* stream);

// out_status_where: two host words, [0] = status of the first recorded failure
// (0 none, 2 = barrier limit, 3 = list capacity), [1] = its code location.
// reset != 0 also clears both control blocks and the predicted threshold.
// Waits for `stream`; allocates nothing.
int gtk_k1_noalloc_status(unsigned int* out_status_where, int reset, void* stream);

#ifdef __cplusplus
}
#endif
