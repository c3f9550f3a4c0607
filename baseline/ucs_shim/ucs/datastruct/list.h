#ifndef UCS_SHIM_LIST_H_
#define UCS_SHIM_LIST_H_
#include "../sys/compiler_def.h"
typedef struct ucs_list_link { struct ucs_list_link *prev, *next; } ucs_list_link_t;
static inline void ucs_list_head_init(ucs_list_link_t *h) { h->prev = h->next = h; }
static inline int  ucs_list_is_empty(ucs_list_link_t *h) { return h->next == h; }
static inline void ucs_list_add_tail(ucs_list_link_t *h, ucs_list_link_t *e)
{
    e->prev = h->prev; e->next = h; h->prev->next = e; h->prev = e;
}
static inline void ucs_list_del(ucs_list_link_t *e) { e->prev->next = e->next; e->next->prev = e->prev; }
static inline ucs_list_link_t *ucs_list_extract_head_(ucs_list_link_t *h) { ucs_list_link_t *e = h->next; ucs_list_del(e); return e; }
#define ucs_list_extract_head(head, type, member) ucs_container_of(ucs_list_extract_head_(head), type, member)
#define ucs_list_for_each_safe(elem, tmp, head, member)                                              \
    for (elem = ucs_container_of((head)->next, __typeof__(*elem), member),                           \
        tmp  = ucs_container_of(elem->member.next, __typeof__(*elem), member);                       \
         &elem->member != (head);                                                                    \
         elem = tmp, tmp = ucs_container_of(tmp->member.next, __typeof__(*tmp), member))
#endif
