// C ABI of libgtopk_b200.so.  Every entry point takes raw device pointers and a
// CUDA stream handle, enqueues work on that stream and returns without
// synchronising.  Return value: GTK_OK or a negative GTK_ERR_* code.
// Device-side failures (a wait that ran out, a full list) are reported through
// the status word of the control block, which the caller reads when it wants to.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  GTK_OK = 0,
  GTK_ERR_ARG = -1,
  GTK_ERR_CUDA = -2,
  GTK_ERR_UNSUPPORTED = -3,
};

// Persistent per-group selection state (device memory, 32 bytes).
typedef struct K1State {
  float tau;                 // candidate threshold of the next stream pass (+inf: none yet)
  unsigned int n_sel;        // pairs written by the last select
  unsigned int n_cand;       // candidates seen by the last stream pass (may exceed the list size)
  unsigned int fallback;     // 1 if the last call took the exact dense path
  unsigned int n_fallbacks;  // running count of exact dense passes
  unsigned int n_calls;      // running count of calls
  float kth_mag;             // exact k-th magnitude of the last call
  unsigned int reserved;
} K1State;

typedef struct DeviceInfo {
  int device;
  int sms;
  int coop;
  int cluster;
} DeviceInfo;

const DeviceInfo* gtk_device_info(void);
void gtk_count_launch(int n);
long long gtk_launch_count(void);
void gtk_reset_launch_count(void);
unsigned long long gtk_ctrl_bytes(void);
unsigned long long gtk_k1state_bytes(void);
const char* gtk_last_cuda_error(void);

int gtk_k1_select(const float* g, float* r, const float* g_scale, long long d, unsigned int k,
                  void* cand, unsigned int cap, void* sel, void* state, void* ctrl,
                  float target_ratio, unsigned long long limit_ns, void* stream);

#ifdef __cplusplus
}
#endif
