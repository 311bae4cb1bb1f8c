// Process-boundary front-end of a server: the c2s message loop of llis_server
// (reference: src/server/server.cpp:29-167, src/server/registered_job.cpp:26-59,95-105).
#pragma once

#include <llis/ipc/shm_channel.h>
#include <llis/ipc/unix_datagram_socket.h>

#include <chrono>
#include <deque>
#include <memory>
#include <string>
#include <vector>

#include "server.h"

namespace llis {
namespace server {

class IpcServer {
  public:
    static constexpr size_t c2s_channel_size = 1024;   // include/llis/server/server.h:15
    static constexpr size_t s2c_channel_size = 4096;   // :22

    IpcServer(std::string name, const pb_server_config& cfg);
    ~IpcServer();
    // One iteration of the serve loop: at most one client message, then ring records.
    // Returns false once EXIT_CMD was received.
    bool step();
    void serve() { while (step()) {} }
    pb_server* core() { return core_.get(); }

  private:
    struct ClientConnection {
        ipc::ShmChannel s2c_channel;
        ipc::UnixDatagramSocket s2c_socket;   // sender addressed to the client's socket
        bool in_use = false;
        bool gone = false;              // its socket vanished: the process has exited
        unsigned pending_wakeups = 0;   // datagrams that did not fit the client's receive queue yet
        std::deque<void*> pending_done; // completions that did not fit its ring yet (a client that is not draining)
        std::chrono::steady_clock::time_point stalled_since{};   // when pending_done became non-empty
    };
    void complete(ClientConnection& c, void* remote_ptr);
    void retry_completions();
    void wake(ClientConnection& c);
    void retry_wakeups();
    struct RegisteredJob {
        ClientId client_id = 0;
        std::string shm_name;
        int shm_fd = -1;
        size_t pool_bytes = 0;
        std::vector<void*> mapped;            // pool chunks, in the order the client grew the pool
        std::vector<size_t> mapped_bytes;
    };
    void handle_c2s();
    void handle_register_client();
    void handle_register_job();
    void handle_launch_job();
    void handle_grow_pool();

    std::string name_;
    std::unique_ptr<pb_server> core_;
    ipc::ShmChannel c2s_channel_;
    ipc::UnixDatagramSocket s2c_socket_;
    std::vector<std::unique_ptr<ClientConnection>> clients_;
    std::vector<RegisteredJob> jobs_;     // index = job_ref_id = type id in the core server
    bool running_ = true;
};

}  // namespace server
}  // namespace llis
