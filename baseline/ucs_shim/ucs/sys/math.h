#ifndef UCS_SHIM_MATH_H_
#define UCS_SHIM_MATH_H_
#include "compiler_def.h"
#define ucs_min(a, b) ((a) < (b) ? (a) : (b))
#define ucs_max(a, b) ((a) > (b) ? (a) : (b))
#define ucs_for_each_bit(index, map) \
    for ((index) = __builtin_ctzl(map); (index) < 64 && ((map) >> (index)); (index) += 1 + __builtin_ctzl(((map) >> (index) >> 1) | (1ul << 62)))
#endif
