/* cxxattn diagnostics: measurement and self-test hooks of libcxxattn.so.  Nothing here is needed to
 * use the attention entry points of cxxattn.h; tests and the benchmark call these.  None has a
 * counterpart in the reference, which has no timing hooks and aborts on its one run-time check
 * (src/TwoStage/two_stage_cuda_kernels.cu:316-321). */
#ifndef CXXATTN_DIAG_H_
#define CXXATTN_DIAG_H_

#include "cxxattn.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Two cudaEvent_t handles that later cxxattn_mha_bwd calls (dtype BF16) of the calling thread
 * record on their stream right before and right after the main backward kernel, so that its
 * duration can be read without the pre- and post-pass.  NULL, NULL switches it off. */
void cxxattn_set_timing_events(void* start_event, void* stop_event);

/* One-tile check of the tcgen05 operand conventions (bf16 device buffers, float result):
 *   mode 0: D[128x128] = A[128x64] B[128x64]^T;  mode 1: D[128x64] = A[128x128] B[128x64];
 *   mode 2: D[128x64]  = A[128x128]^T B[128x64]. */
int cxxattn_selftest_umma(int mode, const void* A, const void* B, float* D, cxxattn_stream_t stream);

/* Shows that a bounded device-side wait ends by itself: launches ONE CTA whose threads wait, with the
 * same wait routine as the attention kernels but a limit of `limit_ns` nanoseconds (1000 .. 2e9), on
 * a barrier that nothing ever arrives on.  The wait gives up, the CTA records wait site 990 in the
 * status word, frees its tensor memory and returns; the following cxxattn_sync_status() therefore
 * reports CXXATTN_ERR_TIMEOUT, and launches after it are unaffected.  Nothing traps or spins. */
int cxxattn_selftest_wait_limit(uint64_t limit_ns, cxxattn_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* CXXATTN_DIAG_H_ */
