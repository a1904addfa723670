/* Linux stand-in for the two macOS timing calls that the reference's
 * langtax/q8_gemv.c uses, so that file compiles unmodified with gcc.
 * Timing only: it does not touch the arithmetic the golden checksum pins. */
#ifndef ORC_SHIM_MACH_TIME_H
#define ORC_SHIM_MACH_TIME_H
#include <stdint.h>
#include <time.h>
typedef struct { uint32_t numer, denom; } mach_timebase_info_data_t;
static inline int mach_timebase_info(mach_timebase_info_data_t* tb) { tb->numer = 1; tb->denom = 1; return 0; }
static inline uint64_t mach_absolute_time(void) {
  struct timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return (uint64_t)ts.tv_sec * 1000000000ull + (uint64_t)ts.tv_nsec;
}
#endif
