// Process-wide count of kernels launched by this library (bench.py reports it as
// `gpu_launches`). Relaxed atomics: it is bookkeeping, not synchronisation.
#pragma once
#ifdef __cplusplus
extern "C" {
#endif
void cocclkCountLaunches(long n);
long cocclkLaunchCount(void);
#ifdef __cplusplus
}
#endif
