#ifndef UCS_SHIM_CONFIG_TYPES_H_
#define UCS_SHIM_CONFIG_TYPES_H_
#include "../sys/compiler_def.h"
typedef enum {
    UCS_LOG_LEVEL_FATAL, UCS_LOG_LEVEL_ERROR, UCS_LOG_LEVEL_WARN, UCS_LOG_LEVEL_DIAG, UCS_LOG_LEVEL_INFO,
    UCS_LOG_LEVEL_DEBUG, UCS_LOG_LEVEL_TRACE, UCS_LOG_LEVEL_TRACE_REQ, UCS_LOG_LEVEL_TRACE_DATA,
    UCS_LOG_LEVEL_TRACE_ASYNC, UCS_LOG_LEVEL_TRACE_FUNC, UCS_LOG_LEVEL_TRACE_POLL, UCS_LOG_LEVEL_LAST
} ucs_log_level_t;
typedef struct ucs_log_component_config { ucs_log_level_t log_level; char name[16]; } ucs_log_component_config_t;
typedef enum {
    UCS_CONFIG_PRINT_CONFIG = UCS_BIT(0), UCS_CONFIG_PRINT_HEADER = UCS_BIT(1), UCS_CONFIG_PRINT_DOC = UCS_BIT(2),
    UCS_CONFIG_PRINT_HIDDEN = UCS_BIT(3)
} ucs_config_print_flags_t;
typedef struct { char **names; unsigned count; unsigned pad; } ucs_config_names_array_t;
#endif
