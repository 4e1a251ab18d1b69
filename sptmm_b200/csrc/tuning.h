/*
 * tuning.h -- extra entry points of the TUNING build of the library (build.py --tuning, which
 * compiles with -DSPTMM_TUNING into libsptmm_tuning.so).  That build records kernel timelines and
 * lets environment variables override launch constants; the product library has neither.
 */
#ifndef SPTMM_TUNING_H
#define SPTMM_TUNING_H

#include "../../include/sptmm.h"

#ifdef __cplusplus
extern "C" {
#endif

/* While `dev_ptr` (64 x uint64 of device memory) is set, the per-call kernel's first CTAs record
 * %globaltimer at entry, after the wait on the previous kernel, after staging X, after the gather
 * loop and at exit.  NULL switches it off. */
int sptmm_set_trace_buffer(void *dev_ptr);

/* Timestamps of a sequence run (layout: see k_seq); NULL = off. */
int sptmm_seq_set_trace(sptmm_seq *seq, void *dev_ptr);

#ifdef __cplusplus
}
#endif
#endif
