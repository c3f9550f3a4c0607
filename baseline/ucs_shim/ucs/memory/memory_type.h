#ifndef UCS_SHIM_MEMORY_TYPE_H_
#define UCS_SHIM_MEMORY_TYPE_H_
typedef enum ucs_memory_type {
    UCS_MEMORY_TYPE_HOST, UCS_MEMORY_TYPE_CUDA, UCS_MEMORY_TYPE_CUDA_MANAGED, UCS_MEMORY_TYPE_ROCM,
    UCS_MEMORY_TYPE_ROCM_MANAGED, UCS_MEMORY_TYPE_LAST
} ucs_memory_type_t;
extern const char *ucs_memory_type_names[];
#endif
