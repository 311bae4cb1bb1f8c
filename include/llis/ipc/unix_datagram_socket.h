// Abstract-namespace unix datagram socket: the server's "job started" (pre-notify) signal to a
// client.  Same addressing as the reference (src/ipc/unix_datagram_socket.cpp:53-84): sun_path[0] = 0
// followed by the name.
#pragma once

#include <sys/socket.h>
#include <sys/types.h>
#include <sys/un.h>

#include <string>

namespace llis {
namespace ipc {

class UnixDatagramSocket {
  public:
    UnixDatagramSocket();
    explicit UnixDatagramSocket(const std::string& name);
    ~UnixDatagramSocket();
    UnixDatagramSocket(const UnixDatagramSocket&) = delete;
    UnixDatagramSocket& operator=(const UnixDatagramSocket&) = delete;
    UnixDatagramSocket(UnixDatagramSocket&& o) noexcept { *this = std::move(o); }
    UnixDatagramSocket& operator=(UnixDatagramSocket&& o) noexcept;

    void bind(const std::string& name);
    // A sender on this socket addressed to `name` (does not own the descriptor).
    UnixDatagramSocket connect(const std::string& name);
    ssize_t write(const void* buf, size_t count);
    // Non-blocking send that reports instead of throwing: bytes sent, or -errno (-EAGAIN / -ENOBUFS when
    // the receiver's queue is full, -ECONNREFUSED / -ENOENT when nobody is bound to the name any more).
    // Not in the reference, whose server blocks in sendto(); a blocked server and a client blocked on a
    // full request ring would wait for each other.
    ssize_t try_write(const void* buf, size_t count);
    ssize_t read(void* buf, size_t count);
    // As read(), but gives up after timeout_ms (returns 0).
    ssize_t read_timeout(void* buf, size_t count, int timeout_ms);

  private:
    explicit UnixDatagramSocket(int fd) : socket_(fd), is_owner_(false) {}
    int socket_ = -1;
    bool is_owner_ = false;
    sockaddr_un remote_addr_{};
};

}  // namespace ipc
}  // namespace llis
