/* Minimal stand-in for the UCS headers the reference (openucx/xccl) includes. It exists only so
 * that the reference's unmodified core, utilities and NCCL team can be compiled on a machine
 * without UCX for the baseline arm of bench.py. Written from the public UCS API names; it is not
 * UCX code and is not ABI-compatible with it. */
#ifndef UCS_SHIM_COMPILER_DEF_H_
#define UCS_SHIM_COMPILER_DEF_H_
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
#define BEGIN_C_DECLS extern "C" {
#define END_C_DECLS }
#else
#define BEGIN_C_DECLS
#define END_C_DECLS
#endif
#define UCS_BIT(i) (1ul << (i))
#define UCS_MASK(i) (UCS_BIT(i) - 1)
#define ucs_offsetof(type, member) offsetof(type, member)
#define ucs_container_of(ptr, type, member) ((type *)((char *)(ptr) - offsetof(type, member)))
#define ucs_derived_of(ptr, type) ((type *)(ptr))
#define ucs_likely(x) __builtin_expect(!!(x), 1)
#define ucs_unlikely(x) __builtin_expect(!!(x), 0)
#define UCS_F_CTOR __attribute__((constructor))
#define UCS_F_DTOR __attribute__((destructor))
#define UCS_V_UNUSED __attribute__((unused))
#define ucs_static_array_size(a) (sizeof(a) / sizeof((a)[0]))
#endif
