// Byte-stream ring in POSIX shared memory between client and server processes.
//
// Wire-compatible with the reference's ShmChannelBase<false> (include/llis/ipc/shm_channel.h:11-130,
// include/llis/ipc/shm_channel_impl.h:35-120, src/ipc/shm_channel.cu:52-127): object name
// "llis:channel:<name>", header = { size_t size; size_t read_pos; size_t write_pos; lock byte },
// ring bytes right behind it, one byte always left free, positions published after each copy,
// an optional spin lock for several writers.  Host only: the GPU-writable variant of the reference
// is not on the serving hot path (its only user is a test kernel).
#pragma once

#include <atomic>
#include <cstddef>
#include <cstdint>
#include <string>

namespace llis {
namespace ipc {

class ShmChannel {
  public:
    ShmChannel() = default;
    // size > 0 creates the object (and its ring of `size` bytes); size == 0 attaches to an existing one.
    explicit ShmChannel(const std::string& name, size_t size = 0) { connect(name, size); }
    // Anonymous (same-process) ring.
    explicit ShmChannel(size_t size) { connect("", size); }
    ~ShmChannel() { disconnect(); }
    ShmChannel(const ShmChannel&) = delete;
    ShmChannel& operator=(const ShmChannel&) = delete;
    ShmChannel(ShmChannel&& o) noexcept { *this = std::move(o); }
    ShmChannel& operator=(ShmChannel&& o) noexcept;

    void connect(const std::string& name, size_t size = 0);
    // Second endpoint on the same mapping (other direction / other thread); does not own the mapping.
    void connect(ShmChannel* other);
    void disconnect();
    bool is_connected() const { return shm_ != nullptr; }
    size_t capacity() const { return size_; }

    // Blocking; max_spins > 0 bounds every internal wait and makes the call return false when it runs out.
    bool read(void* buf, size_t size, uint64_t max_spins = 0);
    bool write(const void* buf, size_t size, uint64_t max_spins = 0);
    bool can_read();
    // Bytes a write() could place right now without waiting for the reader.
    size_t writable_bytes();

    template <typename T> void read(T* v) { read(static_cast<void*>(v), sizeof(T)); }
    template <typename T> void write(T v) { write(static_cast<const void*>(&v), sizeof(T)); }
    void read(std::string* s) {
        size_t len = 0;
        read(&len);
        s->resize(len);
        if (len) read(&(*s)[0], len);
    }
    void write(const std::string& s) {
        write(s.size());
        if (!s.empty()) write(s.data(), s.size());
    }
    void write(const char* s) { write(std::string(s)); }

    void acquire_writer_lock();
    void release_writer_lock();

  private:
    struct Header;
    int fd_ = -1;
    char* shm_ = nullptr;
    char* ring_ = nullptr;
    size_t size_ = 0, total_size_ = 0;
    bool owner_ = false, created_ = false;
    std::string shm_name_;
    size_t cached_read_ = 0, cached_write_ = 0;
    std::atomic<size_t>* read_pos_ = nullptr;
    std::atomic<size_t>* write_pos_ = nullptr;
    std::atomic_flag* lock_ = nullptr;
};

using ShmChannelCpuReader = ShmChannel;
using ShmChannelCpuWriter = ShmChannel;

}  // namespace ipc
}  // namespace llis
