// A minimal out-of-tree team library, built by tests/test_plugin_teardown.py into xccl_team_lib_demo.so and
// found through XCCL_TEAM_LIB_PATH. It serves nothing; it records its life cycle (constructed, opened, closed,
// unloaded) in the file named by XCCL_DEMO_PLUGIN_LOG so that the test can check the library's teardown.
#include <cstdio>
#include <cstdlib>

#include "core/core.h"

namespace {

void note(const char *what)
{
    const char *path = std::getenv("XCCL_DEMO_PLUGIN_LOG");
    if (path == nullptr) return;
    if (FILE *f = std::fopen(path, "a")) {
        std::fprintf(f, "%s\n", what);
        std::fclose(f);
    }
}

class DemoLib final : public xccl::TeamLib {
public:
    DemoLib() : TeamLib((xccl_tl_id_t)XCCL_BIT(12), 1) { note("constructed"); }
    ~DemoLib() override { note("unloaded"); }
    xccl_status_t open() override
    {
        note("opened");
        return XCCL_OK;
    }
    void close() override { note("closed"); }
    xccl_status_t context_create(xccl_lib *, const xccl_context_params_t &, const xccl::OptTable &, xccl::TlContext **) override
    {
        return XCCL_ERR_UNSUPPORTED;
    }
};

DemoLib g_demo;

}  // namespace

extern "C" xccl::TeamLib *xccl_team_lib_create(void) { return &g_demo; }
