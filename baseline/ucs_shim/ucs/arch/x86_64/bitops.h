#ifndef UCS_SHIM_BITOPS_H_
#define UCS_SHIM_BITOPS_H_
#include <stdint.h>
static inline unsigned ucs_ilog2_u32(uint32_t n) { return 31 - (unsigned)__builtin_clz(n); }
static inline unsigned ucs_ilog2_u64(uint64_t n) { return 63 - (unsigned)__builtin_clzl(n); }
static inline unsigned __ucs_ilog2_u32(uint32_t n) { return ucs_ilog2_u32(n); }
static inline unsigned __ucs_ilog2_u64(uint64_t n) { return ucs_ilog2_u64(n); }
#endif
