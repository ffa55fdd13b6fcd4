/* misc.c -- host helpers (reference: src/misc.c:48-127). */
#include "misc.h"
#include "error.h"

#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/resource.h>
#include <sys/time.h>

static double tv_seconds(struct timeval tv) { return (double)tv.tv_sec + 1e-6 * (double)tv.tv_usec; }

double fluke_realtime(void) {
    struct timeval now;
    gettimeofday(&now, NULL);
    return tv_seconds(now);
}

double fluke_cputime(void) {
    struct rusage ru;
    getrusage(RUSAGE_SELF, &ru);
    return tv_seconds(ru.ru_utime) + tv_seconds(ru.ru_stime);
}

long fluke_peakrss(void) {
    struct rusage ru;
    getrusage(RUSAGE_SELF, &ru);
#ifdef __APPLE__
    return ru.ru_maxrss;
#else
    return ru.ru_maxrss * 1024L;
#endif
}

void fluke_print_size(const char *name, uint64_t bytes) {
    static const char *unit[] = {"B", "KiB", "MiB", "GiB", "TiB"};
    double v = (double)bytes;
    int u = 0;
    while (v >= 1024.0 && u < 4) { v /= 1024.0; ++u; }
    fprintf(stderr, "[%s] %s : %.1f %s\n", __func__, name, v, unit[u]);
}

int64_t fluke_mm_parse_num(const char *str) {
    char *end = NULL;
    double v = strtod(str, &end);
    switch (*end) {
        case 'g': case 'G': v *= 1e9; break;
        case 'm': case 'M': v *= 1e6; break;
        case 'k': case 'K': v *= 1e3; break;
        default: break;
    }
    return (int64_t)(v + .499);
}

void fluke_yes_or_no(uint64_t *flag_a, uint64_t flag, const char *opt_name, const char *arg,
                     int yes_to_set) {
    int yes = (strcmp(arg, "yes") == 0 || strcmp(arg, "y") == 0);
    int no = (strcmp(arg, "no") == 0 || strcmp(arg, "n") == 0);
    if (!yes && !no) {
        FLUKE_WARNING("option '--%s' only accepts 'yes' or 'no'.", opt_name);
        return;
    }
    if ((yes && yes_to_set) || (no && !yes_to_set)) *flag_a |= flag;
    else *flag_a &= ~flag;
}
