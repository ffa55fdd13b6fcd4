/* error.h -- internal check macros of the host code. Same behaviour as the reference's
 * src/error.h:43-81: print a located message to stderr, then exit(EXIT_FAILURE). */
#ifndef FLUKE_SRC_ERROR_H
#define FLUKE_SRC_ERROR_H

#include <errno.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <fluke/fluke_error.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FLUKE_DIE_IF_(cond, ...)          \
    {                                     \
        if (cond) {                       \
            FLUKE_ERROR(__VA_ARGS__)      \
            exit(EXIT_FAILURE);           \
        }                                 \
    }

#define MALLOC_ERROR()  FLUKE_ERROR("Failed to allocate memory: %s", strerror(errno))
#define MALLOC_CHK(ret) FLUKE_DIE_IF_((ret) == NULL, "Failed to allocate memory: %s", strerror(errno))
#define F_CHK(ret, file) FLUKE_DIE_IF_((ret) == NULL, "Could not to open file %s: %s", file, strerror(errno))
#define NULL_CHK(ret)   FLUKE_DIE_IF_((ret) == NULL, "NULL returned: %s.", strerror(errno))
#define NEG_CHK(ret)    FLUKE_DIE_IF_((ret) < 0, "Negative value returned: %s.", strerror(errno))

#define ASSERT(ret)                                                                   \
    {                                                                                 \
        if ((ret) == 0) {                                                             \
            fprintf(stderr, FLUKE_ERROR_PREFIX "Assertion failed." FLUKE_NO_COLOUR    \
                            " At %s:%d\nExiting.\n",                                  \
                    __func__, __FILE__, __LINE__ - 1);                                \
            exit(EXIT_FAILURE);                                                       \
        }                                                                             \
    }

#ifdef __cplusplus
}
#endif

#endif
