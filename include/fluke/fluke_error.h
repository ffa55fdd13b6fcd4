/* fluke_error.h -- log-level control and stderr logging macros of the fluke C ABI.
 *
 * Interface-compatible with the reference header include/fluke/fluke_error.h:41-106
 * (enum values, accessor names and macro names are part of the ABI that slorado
 * compiles against); the default level is FLUKE_LOG_VERB as in the reference
 * (src/error.c:33).
 */
#ifndef FLUKE_ERROR_H
#define FLUKE_ERROR_H

#include <stdio.h>
#include <string.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Verbosity of what the library prints to stderr; each level includes the ones above it. */
enum fluke_log_level_opt {
    FLUKE_LOG_OFF,  /* silent                      */
    FLUKE_LOG_ERR,  /* errors                      */
    FLUKE_LOG_WARN, /* + warnings                  */
    FLUKE_LOG_INFO, /* + information               */
    FLUKE_LOG_VERB, /* + verbose notes (default)   */
    FLUKE_LOG_DBUG, /* + debugging                 */
    FLUKE_LOG_TRAC  /* + tracing                   */
};

enum fluke_log_level_opt get_fluke_log_level();
void set_fluke_log_level(enum fluke_log_level_opt level);

#define fluke_log_level get_fluke_log_level()

#define FLUKE_DEBUG_PREFIX   "[FLUKE_DEBUG] %s: "
#define FLUKE_VERBOSE_PREFIX "[FLUKE_INFO] %s: "
#define FLUKE_INFO_PREFIX    "[%s::FLUKE_INFO]\033[1;34m "
#define FLUKE_WARNING_PREFIX "[%s::FLUKE_WARNING]\033[1;33m "
#define FLUKE_ERROR_PREFIX   "[%s::FLUKE_ERROR]\033[1;31m "
#define FLUKE_NO_COLOUR      "\033[0m"

/* Message with a trailing source location, printed when the level is at least `lvl`. */
#define FLUKE_LOG_AT_(lvl, prefix, tail, msg, ...)                                   \
    {                                                                                \
        if (fluke_log_level >= (lvl)) {                                              \
            fprintf(stderr, prefix msg tail " At %s:%d\n", __func__, __VA_ARGS__,    \
                    __FILE__, __LINE__ - 1);                                         \
        }                                                                            \
    }

/* Message without a source location. */
#define FLUKE_LOG_PLAIN_(lvl, prefix, tail, msg, ...)                                \
    {                                                                                \
        if (fluke_log_level >= (lvl)) {                                              \
            fprintf(stderr, prefix msg tail "\n", __func__, __VA_ARGS__);            \
        }                                                                            \
    }

#define FLUKE_LOG_TRACE(msg, ...) FLUKE_LOG_AT_(FLUKE_LOG_TRAC, FLUKE_DEBUG_PREFIX, "", msg, __VA_ARGS__)
#define FLUKE_LOG_DEBUG(msg, ...) FLUKE_LOG_AT_(FLUKE_LOG_DBUG, FLUKE_DEBUG_PREFIX, "", msg, __VA_ARGS__)
#define FLUKE_VERBOSE(msg, ...)   FLUKE_LOG_PLAIN_(FLUKE_LOG_VERB, FLUKE_VERBOSE_PREFIX, "", msg, __VA_ARGS__)
#define FLUKE_INFO(msg, ...)      FLUKE_LOG_PLAIN_(FLUKE_LOG_INFO, FLUKE_INFO_PREFIX, FLUKE_NO_COLOUR, msg, __VA_ARGS__)
#define FLUKE_WARNING(msg, ...)   FLUKE_LOG_AT_(FLUKE_LOG_WARN, FLUKE_WARNING_PREFIX, FLUKE_NO_COLOUR, msg, __VA_ARGS__)
#define FLUKE_ERROR(msg, ...)     FLUKE_LOG_AT_(FLUKE_LOG_ERR, FLUKE_ERROR_PREFIX, FLUKE_NO_COLOUR, msg, __VA_ARGS__)

#ifdef __cplusplus
}
#endif

#endif /* FLUKE_ERROR_H */
