/* Implementation of the UCS stand-in declared under baseline/ucs_shim/ucs/. See
 * ucs/sys/compiler_def.h for what it is and is not. */
#include <ctype.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <strings.h>
#include <unistd.h>

#include <ucs/config/parser.h>
#include <ucs/debug/log_def.h>
#include <ucs/memory/memory_type.h>

const char *ucs_memory_type_names[] = {"host", "cuda", "cuda-managed", "rocm", "rocm-managed", "unknown"};
ucs_list_link_t ucs_config_global_list = {&ucs_config_global_list, &ucs_config_global_list};

static const char *const level_names[] = {"FATAL", "ERROR", "WARN", "DIAG", "INFO", "DEBUG", "TRACE", "REQ",
                                          "DATA", "ASYNC", "FUNC", "POLL"};

void ucs_shim_log(const char *file, int line, int level, const ucs_log_component_config_t *comp, const char *fmt, ...)
{
    char    msg[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(msg, sizeof(msg), fmt, ap);
    va_end(ap);
    const char *base = strrchr(file, '/');
    fprintf(stderr, "[%d] %-5s %s %s:%d %s\n", (int)getpid(), level_names[level < 12 ? level : 11], comp->name,
            base ? base + 1 : file, line, msg);
}

static int parse_level(const char *v)
{
    for (int i = 0; i < 12; i++) {
        if (strcasecmp(v, level_names[i]) == 0) return i;
    }
    if (strcasecmp(v, "trace_req") == 0) return UCS_LOG_LEVEL_TRACE_REQ;
    return isdigit((unsigned char)v[0]) ? atoi(v) : -1;
}

static long long parse_mem(const char *v, int *ok)
{
    char     *end = NULL;
    double    d   = strtod(v, &end);
    long long m   = 1;
    *ok           = end != v;
    if (strcasecmp(v, "inf") == 0) { *ok = 1; return (long long)-1; }
    switch (tolower((unsigned char)*end)) {
    case 'k': m = 1ll << 10; break;
    case 'm': m = 1ll << 20; break;
    case 'g': m = 1ll << 30; break;
    default: break;
    }
    return (long long)(d * (double)m);
}

static int set_field(void *opts, const ucs_config_field_t *f, const char *v)
{
    char *p = (char *)opts + f->offset;
    int   ok = 1;
    switch (f->parser.kind) {
    case UCS_SHIM_T_STRING: free(*(char **)p); *(char **)p = strdup(v); return 1;
    case UCS_SHIM_T_INT: *(int *)p = atoi(v); return 1;
    case UCS_SHIM_T_UINT: *(unsigned *)p = (unsigned)strtoul(v, NULL, 10); return 1;
    case UCS_SHIM_T_DOUBLE: *(double *)p = strtod(v, NULL); return 1;
    case UCS_SHIM_T_BOOL:
    case UCS_SHIM_T_TERNARY:
        if (!strcasecmp(v, "y") || !strcasecmp(v, "yes") || !strcmp(v, "1") || !strcasecmp(v, "on")) { *(int *)p = 1; return 1; }
        if (!strcasecmp(v, "n") || !strcasecmp(v, "no") || !strcmp(v, "0") || !strcasecmp(v, "off")) { *(int *)p = 0; return 1; }
        if (f->parser.kind == UCS_SHIM_T_TERNARY && !strcasecmp(v, "try")) { *(int *)p = 2; return 1; }
        return 0;
    case UCS_SHIM_T_MEMUNITS: *(size_t *)p = (size_t)parse_mem(v, &ok); return ok;
    case UCS_SHIM_T_LOG_COMP: {
        int lvl = parse_level(v);
        if (lvl < 0) return 0;
        ((ucs_log_component_config_t *)p)->log_level = (ucs_log_level_t)lvl;
        return 1;
    }
    default: return 0;
    }
}

static void init_string_fields(void *opts, const ucs_config_field_t *fields)
{
    for (const ucs_config_field_t *f = fields; f->name != NULL; f++) {
        if (f->parser.kind == UCS_SHIM_T_TABLE) {
            init_string_fields((char *)opts + f->offset, (const ucs_config_field_t *)f->parser.arg);
        } else if (f->parser.kind == UCS_SHIM_T_STRING) {
            *(char **)((char *)opts + f->offset) = NULL;
        }
    }
}

static ucs_status_t fill(void *opts, const ucs_config_field_t *fields, const char *env_prefix, const char *table_prefix)
{
    for (const ucs_config_field_t *f = fields; f->name != NULL; f++) {
        if (f->parser.kind == UCS_SHIM_T_TABLE) {
            ucs_status_t st = fill((char *)opts + f->offset, (const ucs_config_field_t *)f->parser.arg, env_prefix, table_prefix);
            if (st != UCS_OK) return st;
            continue;
        }
        char        var[256];
        const char *v = NULL;
        /* <env_prefix><table_prefix><NAME>; when env_prefix carries a user prefix ("P_XCCL_"), the plain
         * "XCCL_" spelling is tried as a fallback, as UCS does with sub-prefixes */
        snprintf(var, sizeof(var), "%s%s%s", env_prefix ? env_prefix : "", table_prefix ? table_prefix : "", f->name);
        v = getenv(var);
        if (v == NULL && env_prefix != NULL) {
            const char *x = strstr(env_prefix, "XCCL_");
            if (x != NULL && x != env_prefix) {
                snprintf(var, sizeof(var), "%s%s%s", x, table_prefix ? table_prefix : "", f->name);
                v = getenv(var);
            }
        }
        if (!set_field(opts, f, v != NULL ? v : f->dfl_value)) {
            if (v == NULL || !set_field(opts, f, f->dfl_value)) return UCS_ERR_INVALID_PARAM;
        }
    }
    return UCS_OK;
}

ucs_status_t ucs_config_parser_fill_opts(void *opts, ucs_config_field_t *fields, const char *env_prefix,
                                         const char *table_prefix, int ignore_errors)
{
    (void)ignore_errors;
    init_string_fields(opts, fields);
    return fill(opts, fields, env_prefix, table_prefix);
}

ucs_status_t ucs_config_parser_set_value(void *opts, ucs_config_field_t *fields, const char *name, const char *value)
{
    for (const ucs_config_field_t *f = fields; f->name != NULL; f++) {
        if (f->parser.kind == UCS_SHIM_T_TABLE) {
            if (ucs_config_parser_set_value((char *)opts + f->offset, (ucs_config_field_t *)f->parser.arg, name, value) == UCS_OK) return UCS_OK;
        } else if (strcmp(f->name, name) == 0) {
            return set_field(opts, f, value) ? UCS_OK : UCS_ERR_INVALID_PARAM;
        }
    }
    return UCS_ERR_NO_ELEM;
}

void ucs_config_parser_release_opts(void *opts, ucs_config_field_t *fields)
{
    for (const ucs_config_field_t *f = fields; f->name != NULL; f++) {
        if (f->parser.kind == UCS_SHIM_T_TABLE) {
            ucs_config_parser_release_opts((char *)opts + f->offset, (ucs_config_field_t *)f->parser.arg);
        } else if (f->parser.kind == UCS_SHIM_T_STRING) {
            free(*(char **)((char *)opts + f->offset));
            *(char **)((char *)opts + f->offset) = NULL;
        }
    }
}

void ucs_config_parser_print_opts(FILE *stream, const char *title, const void *opts, ucs_config_field_t *fields,
                                  const char *table_prefix, const char *prefix, ucs_config_print_flags_t flags)
{
    (void)opts; (void)flags;
    fprintf(stream, "# %s\n", title ? title : "");
    for (const ucs_config_field_t *f = fields; f->name != NULL; f++) {
        if (f->parser.kind != UCS_SHIM_T_TABLE) fprintf(stream, "%s%s%s (default %s)\n", prefix ? prefix : "", table_prefix ? table_prefix : "", f->name, f->dfl_value);
    }
}

void ucs_config_parser_warn_unused_env_vars_once(const char *env_prefix) { (void)env_prefix; }
