/* gpu_common.h -- shared state of the C host layer above the sm_100a launchers: the stream
 * every launch uses and the last error text of the int-returning entry points. */
#ifndef FLUKE_SRC_GPU_COMMON_H
#define FLUKE_SRC_GPU_COMMON_H

#include <stdio.h>
#include <stdlib.h>

#include "../fluke_b200/csrc/fluke_sm100.h"

/* Stream passed to every launcher (NULL = legacy default stream). */
void *fluke_host_stream(void);

/* Records `code` (a cudaError_t as int) as the last error and returns it unchanged. */
int fluke_host_note_error(int code);

/* Post-launch check of the void entry points: a non-zero launcher result prints the CUDA
 * error with its location and exits, like checkKernel() in the reference
 * (src/cuda_utils.h:5-23). */
#define FLUKE_CHECK_LAUNCH(call)                                                              \
    {                                                                                         \
        int fluke_rc_ = (call);                                                               \
        if (fluke_rc_ != 0) {                                                                 \
            fprintf(stderr, "CUDA error: %s \n in file: %s, line number: %d\n",               \
                    fluke_sm100_error_string(fluke_rc_), __FILE__, __LINE__);                 \
            exit(1);                                                                          \
        }                                                                                     \
    }

#endif
