/* Test-only entry points of libletheprobe.so (built from tests/native/probe.cu by
 * lethe_b200._build.build_probe()).  They are not part of the GDN interface in include/lethe_gdn.h and
 * have no counterpart in the reference project. */
#ifndef LETHE_PROBE_H_
#define LETHE_PROBE_H_

#ifdef __cplusplus
extern "C" {
#endif

/* One tcgen05 product D[128 x N] = (+/-) A * B on one CTA (optionally twice, accumulating), with the
 * operand orientation (a_mn / b_mn: contracted along tile rows) and the tile-fill method (0 threads,
 * 1 tensor-map loads, 2 bulk copies of host-swizzled images) chosen by the caller. */
int lethe_probe_umma(const void* A, const void* B, float* D, int* status, int a_mn, int b_mn, int N,
                     int kc, int fill, int a_neg, int twice, void* cuda_stream);

/* One CTA waits on a barrier that nothing completes, with a limit of `limit_cycles` clock cycles
 * (1e3 .. 2e8).  Expected outcome: *status == 101 (the wait site), trace[0] == 1 (abort flag raised),
 * trace[1] ~ limit_cycles / 1024, trace[2] ~ 0 (the second wait fell through), kernel returned. */
int lethe_probe_starved_wait(int* status, long long limit_cycles, int* trace, void* cuda_stream);

#ifdef __cplusplus
}
#endif
#endif
