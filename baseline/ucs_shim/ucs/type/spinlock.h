#ifndef UCS_SHIM_SPINLOCK_H_
#define UCS_SHIM_SPINLOCK_H_
#include <pthread.h>
#include "status.h"
typedef struct ucs_spinlock { pthread_spinlock_t lock; } ucs_spinlock_t;
static inline ucs_status_t ucs_spinlock_init(ucs_spinlock_t *l, int flags) { (void)flags; pthread_spin_init(&l->lock, 0); return UCS_OK; }
static inline void ucs_spinlock_destroy(ucs_spinlock_t *l) { pthread_spin_destroy(&l->lock); }
static inline void ucs_spin_lock(ucs_spinlock_t *l) { pthread_spin_lock(&l->lock); }
static inline void ucs_spin_unlock(ucs_spinlock_t *l) { pthread_spin_unlock(&l->lock); }
#endif
