#ifndef UCS_SHIM_CONFIG_PARSER_H_
#define UCS_SHIM_CONFIG_PARSER_H_
#include <stdio.h>
#include "types.h"
#include "../type/status.h"
#include "../datastruct/list.h"
#include "../sys/preprocessor.h"
BEGIN_C_DECLS
enum { UCS_SHIM_T_STRING = 1, UCS_SHIM_T_INT, UCS_SHIM_T_UINT, UCS_SHIM_T_BOOL, UCS_SHIM_T_MEMUNITS, UCS_SHIM_T_LOG_COMP,
       UCS_SHIM_T_TABLE, UCS_SHIM_T_TERNARY, UCS_SHIM_T_DOUBLE, UCS_SHIM_T_STRING_ARRAY };
typedef struct ucs_config_parser { int kind; const void *arg; } ucs_config_parser_t;
typedef struct ucs_config_field {
    const char *name; const char *dfl_value; const char *doc; size_t offset; ucs_config_parser_t parser;
} ucs_config_field_t;
#define UCS_CONFIG_TYPE_STRING   {UCS_SHIM_T_STRING, NULL}
#define UCS_CONFIG_TYPE_INT      {UCS_SHIM_T_INT, NULL}
#define UCS_CONFIG_TYPE_UINT     {UCS_SHIM_T_UINT, NULL}
#define UCS_CONFIG_TYPE_BOOL     {UCS_SHIM_T_BOOL, NULL}
#define UCS_CONFIG_TYPE_TERNARY  {UCS_SHIM_T_TERNARY, NULL}
#define UCS_CONFIG_TYPE_DOUBLE   {UCS_SHIM_T_DOUBLE, NULL}
#define UCS_CONFIG_TYPE_MEMUNITS {UCS_SHIM_T_MEMUNITS, NULL}
#define UCS_CONFIG_TYPE_LOG_COMP {UCS_SHIM_T_LOG_COMP, NULL}
#define UCS_CONFIG_TYPE_STRING_ARRAY {UCS_SHIM_T_STRING_ARRAY, NULL}
#define UCS_CONFIG_TYPE_TABLE(t) {UCS_SHIM_T_TABLE, t}
typedef struct ucs_config_global_list_entry {
    const char *name; const char *prefix; ucs_config_field_t *table; size_t size; ucs_list_link_t list;
} ucs_config_global_list_entry_t;
#define UCS_CONFIG_REGISTER_TABLE(_fields, _name, _prefix, _type, _list) /* no global listing in the shim */
ucs_status_t ucs_config_parser_fill_opts(void *opts, ucs_config_field_t *fields, const char *env_prefix,
                                         const char *table_prefix, int ignore_errors);
ucs_status_t ucs_config_parser_set_value(void *opts, ucs_config_field_t *fields, const char *name, const char *value);
void         ucs_config_parser_release_opts(void *opts, ucs_config_field_t *fields);
void         ucs_config_parser_print_opts(FILE *stream, const char *title, const void *opts, ucs_config_field_t *fields,
                                          const char *table_prefix, const char *prefix, ucs_config_print_flags_t flags);
void         ucs_config_parser_warn_unused_env_vars_once(const char *env_prefix);
END_C_DECLS
#endif
