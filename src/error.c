/* error.c -- process-wide log level (reference: src/error.c:33-41; default VERB). */
#include <fluke/fluke_error.h>

static enum fluke_log_level_opt g_level = FLUKE_LOG_VERB;

enum fluke_log_level_opt get_fluke_log_level() { return g_level; }

void set_fluke_log_level(enum fluke_log_level_opt level) { g_level = level; }
