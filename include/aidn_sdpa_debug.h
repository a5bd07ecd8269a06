/*
 * aidn_sdpa_debug.h — test and development hook of libaidotnet_sdpa_sm100.  Not part of the drop-in surface: nothing in
 * the reference binds it and a production caller never needs it.  No counterpart in the reference.
 */
#ifndef AIDN_SDPA_DEBUG_H_
#define AIDN_SDPA_DEBUG_H_

#include "aidn_sdpa.h"

#ifdef __cplusplus
extern "C" {
#endif

/* mode 0: off.
 * mode 3: the TMA producers of the tcgen05 kernels of this handle (prefill, backward, projection GEMM) withhold their
 *         loads and every bounded device-side wait gives up after 20 ms instead of 2 s, so that a test can watch
 *         aidn_sdpa_poll report AIDN_ETIMEOUT and the next launch succeed — without any fault on the device.  `buf`
 *         is ignored.
 * modes 1, 2 and 4 exist only in development builds of the library (compiled with -DAIDN_PREFILL_TRACE=1): value tap,
 *         per-work-item timeline and per-step clock stamps of the prefill kernel, written to `buf`.  The shipped build
 *         ignores them. */
AIDN_API int aidn_sdpa_debug_set(aidn_sdpa_t h, float* buf, int mode);

#ifdef __cplusplus
}
#endif
#endif /* AIDN_SDPA_DEBUG_H_ */
