/* Checks of the public C API that need no team: header inlines (datatype sizes, endpoint ranges, team-library names),
 * status strings, configuration read / modify / print, team-library list and attributes, and the capability filter
 * of xccl_lib_init. Prints "api surface ok" and exits 0, or names the first failed check and exits 1.
 * Reference for the behaviour checked: src/api/xccl.h:246-310 (ranges), :391-407 and :478-502 (datatypes),
 * src/api/xccl_tls.h:27-69 (names), src/core/xccl_lib.c:27-42 (capability filter), src/core/xccl_query.c:12-80. */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <xccl/xccl.h>

#define CHECK(cond)                                                             \
    do {                                                                        \
        if (!(cond)) {                                                          \
            fprintf(stderr, "failed at line %d: %s\n", __LINE__, #cond);        \
            return 1;                                                           \
        }                                                                       \
    } while (0)

static int times_three(int rank, void *ctx) { return rank * 3 + *(int *)ctx; }

static int has_tl(const xccl_tl_id_t *ids, unsigned n, xccl_tl_id_t want)
{
    unsigned i;
    for (i = 0; i < n; i++) {
        if (ids[i] == want) return 1;
    }
    return 0;
}

int main(void)
{
    /* datatypes */
    CHECK(xccl_dt_size(XCCL_DT_INT8) == 1 && xccl_dt_size(XCCL_DT_UINT8) == 1);
    CHECK(xccl_dt_size(XCCL_DT_INT16) == 2 && xccl_dt_size(XCCL_DT_UINT16) == 2 && xccl_dt_size(XCCL_DT_FLOAT16) == 2);
    CHECK(xccl_dt_size(XCCL_DT_BFLOAT16) == 2);
    CHECK(xccl_dt_size(XCCL_DT_INT32) == 4 && xccl_dt_size(XCCL_DT_UINT32) == 4 && xccl_dt_size(XCCL_DT_FLOAT32) == 4);
    CHECK(xccl_dt_size(XCCL_DT_INT64) == 8 && xccl_dt_size(XCCL_DT_UINT64) == 8 && xccl_dt_size(XCCL_DT_FLOAT64) == 8);
    CHECK(xccl_dt_size(XCCL_DT_INT128) == 16 && xccl_dt_size(XCCL_DT_UINT128) == 16);
    CHECK(xccl_dt_size(XCCL_DT_UNSUPPORTED) == 0);

    /* endpoint ranges */
    {
        int             map[4] = {7, 5, 3, 1}, base = 2;
        xccl_ep_range_t r;
        memset(&r, 0, sizeof(r));
        r.type = XCCL_EP_RANGE_FULL;
        CHECK(xccl_range_to_rank(r, 5) == 5);
        r.type           = XCCL_EP_RANGE_STRIDED;
        r.strided.start  = 4;
        r.strided.stride = 3;
        CHECK(xccl_range_to_rank(r, 0) == 4 && xccl_range_to_rank(r, 2) == 10);
        r.type    = XCCL_EP_RANGE_MAP;
        r.map.map = map;
        CHECK(xccl_range_to_rank(r, 0) == 7 && xccl_range_to_rank(r, 3) == 1);
        r.type      = XCCL_EP_RANGE_CB;
        r.cb.cb     = times_three;
        r.cb.cb_ctx = &base;
        CHECK(xccl_range_to_rank(r, 4) == 14);
        r.type = XCCL_EP_RANGE_UNDEFINED;
        CHECK(xccl_range_to_rank(r, 1) == -1);
    }

    /* team-library names: same values as the reference, NVLINK added behind them */
    CHECK(XCCL_TL_UCX == 1 && XCCL_TL_HIER == 2 && XCCL_TL_SHARP == 4 && XCCL_TL_HMC == 8 && XCCL_TL_SHMSEG == 16);
    CHECK(XCCL_TL_MRAIL == 32 && XCCL_TL_NCCL == 64 && XCCL_TL_MPOD == 128 && XCCL_TL_NVLINK == 256);
    CHECK(strcmp(xccl_tl_str(XCCL_TL_UCX), "ucx") == 0 && strcmp(xccl_tl_str(XCCL_TL_NVLINK), "nvlink") == 0);
    CHECK(xccl_tl_str((xccl_tl_id_t)3) == NULL);
    CHECK(xccl_tls_str_to_bitmap("ucx,nccl") == (xccl_tl_id_t)(XCCL_TL_UCX | XCCL_TL_NCCL));
    CHECK(xccl_tls_str_to_bitmap("hier") == XCCL_TL_HIER);
    CHECK(xccl_tls_str_to_bitmap("nothing") == XCCL_TL_NULL && xccl_tls_str_to_bitmap(NULL) == XCCL_TL_NULL);
    CHECK((XCCL_TL_ALL & XCCL_TL_NVLINK) && (XCCL_TL_ALL & XCCL_TL_UCX));

    /* status codes and strings */
    CHECK(XCCL_OK == 0 && XCCL_INPROGRESS == 1 && XCCL_ERR_LAST == -100);
    CHECK(xccl_status_str(XCCL_OK) != NULL && xccl_status_str(XCCL_ERR_UNSUPPORTED) != NULL);
    CHECK(strcmp(xccl_status_str(XCCL_OK), xccl_status_str(XCCL_ERR_NO_MEMORY)) != 0);
    CHECK(xccl_status_str((xccl_status_t)-77) != NULL);

    /* library configuration: read with a caller prefix, print, release */
    {
        xccl_lib_config_t *cfg = NULL;
        char               buf[65536];
        FILE              *f;
        size_t             n;
        setenv("MYAPP_XCCL_LOG_LEVEL", "debug", 1);
        CHECK(xccl_lib_config_read("MYAPP", NULL, &cfg) == XCCL_OK && cfg != NULL);
        f = tmpfile();
        CHECK(f != NULL);
        xccl_lib_config_print(cfg, f, "library", (xccl_config_print_flags_t)(XCCL_CONFIG_PRINT_CONFIG | XCCL_CONFIG_PRINT_DOC |
                                                                           XCCL_CONFIG_PRINT_HEADER));
        rewind(f);
        n      = fread(buf, 1, sizeof(buf) - 1, f);
        buf[n] = '\0';
        fclose(f);
        CHECK(strstr(buf, "LOG_LEVEL") != NULL && strstr(buf, "debug") != NULL);
        CHECK(strstr(buf, "TEAM_LIB_PATH") != NULL && strstr(buf, "LF_TASKS_QUEUE_SIZE") != NULL);
        xccl_lib_config_release(cfg);
        unsetenv("MYAPP_XCCL_LOG_LEVEL");
    }

    /* capability filter, team-library list and attributes, context configuration */
    {
        xccl_lib_params_t lp;
        xccl_lib_h        lib = NULL, lib_get = NULL;
        xccl_tl_id_t     *ids = NULL, one;
        unsigned          n   = 0;
        int               have_sharp;
        xccl_tl_attr_t    attr;
        xccl_context_config_t *cc = NULL;

        memset(&lp, 0, sizeof(lp));
        lp.field_mask = XCCL_LIB_PARAM_FIELD_COLL_TYPES;
        lp.coll_types = XCCL_COLL_CAP_ALLREDUCE | XCCL_COLL_CAP_BARRIER;
        CHECK(xccl_lib_init(&lp, NULL, &lib) == XCCL_OK);
        CHECK(xccl_get_tl_list(lib, &ids, &n) == XCCL_OK && n >= 2);
        CHECK(has_tl(ids, n, XCCL_TL_UCX) && has_tl(ids, n, XCCL_TL_HIER));
        CHECK(!has_tl(ids, n, XCCL_TL_SHMSEG)); /* serves FANOUT_GET only */
        have_sharp = has_tl(ids, n, XCCL_TL_SHARP);   /* opens only where there is a CUDA device */
        xccl_free_tl_list(ids);

        /* only the shared-segment team implements FANOUT_GET */
        memset(&lp, 0, sizeof(lp));
        lp.field_mask = XCCL_LIB_PARAM_FIELD_COLL_TYPES;
        lp.coll_types = XCCL_COLL_CAP_FANOUT_GET;
        CHECK(xccl_lib_init(&lp, NULL, &lib_get) == XCCL_OK);
        CHECK(xccl_get_tl_list(lib_get, &ids, &n) == XCCL_OK && n == 1 && ids[0] == XCCL_TL_SHMSEG);
        xccl_free_tl_list(ids);
        xccl_lib_cleanup(lib_get);

        memset(&attr, 0, sizeof(attr));
        attr.field_mask = XCCL_TL_ATTR_FIELD_CONTEXT_CREATE_MODE;
        one             = XCCL_TL_UCX;
        CHECK(xccl_tl_query(lib, &one, &attr) == XCCL_OK);
        CHECK(attr.context_create_mode == XCCL_TEAM_LIB_CONTEXT_CREATE_MODE_LOCAL);
        one = XCCL_TL_SHARP;
        if (have_sharp) {
            CHECK(xccl_tl_query(lib, &one, &attr) == XCCL_OK);
            CHECK(attr.context_create_mode == XCCL_TEAM_LIB_CONTEXT_CREATE_MODE_GLOBAL);
        } else {
            CHECK(xccl_tl_query(lib, &one, &attr) == XCCL_ERR_NO_ELEM);
        }
        one = (xccl_tl_id_t)(XCCL_TL_UCX | XCCL_TL_HIER); /* one team library at a time */
        CHECK(xccl_tl_query(lib, &one, &attr) != XCCL_OK);

        /* per-team-library options: environment, then modify; unknown names and bad values are refused */
        setenv("XCCL_TEAM_UCX_ALLREDUCE_KN_RADIX", "3", 1);
        CHECK(xccl_context_config_read(lib, NULL, NULL, &cc) == XCCL_OK && cc != NULL);
        one = XCCL_TL_UCX;
        CHECK(xccl_context_config_modify(&one, cc, "ALLREDUCE_KN_RADIX", "5") == XCCL_OK);
        CHECK(xccl_context_config_modify(&one, cc, "NO_SUCH_OPTION", "1") != XCCL_OK);
        CHECK(xccl_context_config_modify(&one, cc, "ALLREDUCE_KN_RADIX", "many") != XCCL_OK);
        one = XCCL_TL_HIER;
        CHECK(xccl_context_config_modify(&one, cc, "BCAST_PIPELINE_THRESH", "64k") == XCCL_OK);
        CHECK(xccl_context_config_modify(&one, cc, "BCAST_PIPELINE_THRESH", "inf") == XCCL_OK);
        CHECK(xccl_context_config_modify(&one, cc, "BCAST_PIPELINE_THRESH", "12 parsecs") != XCCL_OK);
        CHECK(xccl_context_config_modify(&one, cc, "ENABLE_SHMSEG", "y") == XCCL_OK);
        CHECK(xccl_context_config_modify(&one, cc, "ENABLE_SHMSEG", "off") == XCCL_OK);
        CHECK(xccl_context_config_modify(&one, cc, "ENABLE_SHMSEG", "perhaps") != XCCL_OK);
        CHECK(xccl_context_config_modify(&one, cc, "BCAST_PIPELINE_DEPTH", "-3") != XCCL_OK);   /* unsigned */
        one = XCCL_TL_MPOD;   /* no such team library in this config when it was filtered out, or no such option */
        CHECK(xccl_context_config_modify(&one, cc, "NO_SUCH_OPTION", "1") != XCCL_OK);
        xccl_context_config_release(cc);
        unsetenv("XCCL_TEAM_UCX_ALLREDUCE_KN_RADIX");
        xccl_lib_cleanup(lib);
    }
    printf("api surface ok\n");
    return 0;
}
