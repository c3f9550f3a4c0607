// Process placement facts used by the hierarchy layer: host-name hash and bound CPU socket.
// Reference: src/utils/socketid.c:31-210, src/utils/utils.h:29-62.
#pragma once
#include <cstdint>
#include <string>
#include <vector>

namespace xccl {

uint64_t str_hash_djb2(const char *s);

// Logical index (0..n_sockets-1) of the CPU package this process is bound to, or -1 when its
// affinity mask covers more than one package (or cannot be read). XCCL_FAKE_SOCKET_ID
// overrides the answer, so that multi-socket layouts can be tested on any machine.
int bound_socket_id();

// "0-3,8,10-11" -> {0,1,2,3,8,10,11}
std::vector<int> parse_cpu_list(const std::string &s);

// Joins names with commas: {"a","b"} -> "a,b"
std::string join_names(const std::vector<std::string> &names);

}  // namespace xccl
