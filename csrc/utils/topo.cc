#include "topo.h"

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <sched.h>
#include <set>
#include <sstream>

namespace xccl {

uint64_t str_hash_djb2(const char *s)
{
    uint64_t h = 5381;
    for (; *s != '\0'; s++) {
        h = h * 33 + (unsigned char)*s;
    }
    return h;
}

std::vector<int> parse_cpu_list(const std::string &s)
{
    std::vector<int>  out;
    std::stringstream ss(s);
    std::string       tok;
    while (std::getline(ss, tok, ',')) {
        if (tok.empty()) continue;
        int    a = 0, b = 0;
        size_t dash = tok.find('-');
        if (dash == std::string::npos) {
            a = b = std::atoi(tok.c_str());
        } else {
            a = std::atoi(tok.substr(0, dash).c_str());
            b = std::atoi(tok.substr(dash + 1).c_str());
        }
        for (int c = a; c <= b; c++) out.push_back(c);
    }
    return out;
}

static int package_of_cpu(int cpu)
{
    char path[128];
    std::snprintf(path, sizeof(path), "/sys/devices/system/cpu/cpu%d/topology/physical_package_id", cpu);
    std::ifstream in(path);
    int           id = -1;
    if (in) in >> id;
    return id;
}

int bound_socket_id()
{
    const char *fake = std::getenv("XCCL_FAKE_SOCKET_ID");
    if (fake != nullptr) {
        return std::atoi(fake);
    }
    std::ifstream poss("/sys/devices/system/cpu/possible");
    std::string   line;
    if (!poss || !std::getline(poss, line)) {
        return -1;
    }
    std::vector<int> cpus = parse_cpu_list(line);
    cpu_set_t        mask;
    CPU_ZERO(&mask);
    if (sched_getaffinity(0, sizeof(mask), &mask) != 0) {
        return -1;
    }
    std::set<int> all_pkgs, my_pkgs;
    for (int c : cpus) {
        int pkg = package_of_cpu(c);
        if (pkg < 0) continue;
        all_pkgs.insert(pkg);
        if (c < CPU_SETSIZE && CPU_ISSET(c, &mask)) my_pkgs.insert(pkg);
    }
    if (my_pkgs.size() != 1) {
        return -1;
    }
    // physical package ids may be sparse: report the position among the sorted ids
    return (int)std::distance(all_pkgs.begin(), all_pkgs.find(*my_pkgs.begin()));
}

std::string join_names(const std::vector<std::string> &names)
{
    std::string out;
    for (size_t i = 0; i < names.size(); i++) {
        if (i != 0) out += ",";
        out += names[i];
    }
    return out;
}

}  // namespace xccl
