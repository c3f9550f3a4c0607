#ifndef UCS_SHIM_ATOMIC_H_
#define UCS_SHIM_ATOMIC_H_
#include <stdint.h>
static inline void     ucs_atomic_add32(volatile uint32_t *p, uint32_t v) { __atomic_fetch_add(p, v, __ATOMIC_SEQ_CST); }
static inline void     ucs_atomic_sub32(volatile uint32_t *p, uint32_t v) { __atomic_fetch_sub(p, v, __ATOMIC_SEQ_CST); }
static inline uint32_t ucs_atomic_cswap32(volatile uint32_t *p, uint32_t cmp, uint32_t swap)
{
    __atomic_compare_exchange_n(p, &cmp, swap, 0, __ATOMIC_SEQ_CST, __ATOMIC_SEQ_CST);
    return cmp;
}
#endif
