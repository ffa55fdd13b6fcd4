/* misc.h -- small host helpers exported from the library, same names as the reference's
 * src/misc.h:20-32 (wall/CPU time, peak RSS, size printing, number parsing). */
#ifndef FLUKE_SRC_MISC_H
#define FLUKE_SRC_MISC_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

double fluke_realtime(void);   /* wall clock, seconds            */
double fluke_cputime(void);    /* user+system CPU time, seconds  */
long fluke_peakrss(void);      /* peak resident set size, bytes  */
void fluke_print_size(const char *name, uint64_t bytes);
int64_t fluke_mm_parse_num(const char *str);   /* "4k", "2M", "1g" -> integer */
void fluke_yes_or_no(uint64_t *flag_a, uint64_t flag, const char *opt_name, const char *arg,
                     int yes_to_set);

#ifdef __cplusplus
}
#endif

#endif
