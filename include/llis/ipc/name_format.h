// Names of the per-server and per-client IPC objects (reference: src/ipc/name_format.cpp:7-17).
#pragma once

#include <llis/ipc/defs.h>

#include <string>

namespace llis {
namespace ipc {

inline std::string s2c_socket_name(const std::string& server_name, ClientId client_id) {
    return "llis-socket-s2c-" + server_name + "-" + std::to_string(client_id);
}
inline std::string s2c_channel_name(const std::string& server_name, ClientId client_id) {
    return "s2c:" + server_name + ":" + std::to_string(client_id);
}
inline std::string c2s_channel_name(const std::string& server_name) { return "c2s:" + server_name; }

}  // namespace ipc
}  // namespace llis
