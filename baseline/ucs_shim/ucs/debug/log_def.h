#ifndef UCS_SHIM_LOG_DEF_H_
#define UCS_SHIM_LOG_DEF_H_
#include "../config/types.h"
BEGIN_C_DECLS
void ucs_shim_log(const char *file, int line, int level, const ucs_log_component_config_t *comp, const char *fmt, ...)
    __attribute__((format(printf, 5, 6)));
END_C_DECLS
#define ucs_log_component(_level, _comp, _fmt, ...)                                                   \
    do {                                                                                              \
        if ((int)(_level) <= (int)(_comp)->log_level)                                                 \
            ucs_shim_log(__FILE__, __LINE__, (int)(_level), (_comp), _fmt, ##__VA_ARGS__);             \
    } while (0)
#endif
