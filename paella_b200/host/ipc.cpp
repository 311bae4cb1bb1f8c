// Client<->server IPC: shared-memory byte ring and abstract unix datagram socket.
#include <cerrno>
#include <llis/ipc/shm_channel.h>
#include <llis/ipc/unix_datagram_socket.h>

#include <fcntl.h>
#include <poll.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstring>
#include <stdexcept>

namespace llis {
namespace ipc {

namespace {
[[noreturn]] void fail(const std::string& what) { throw std::runtime_error(what + ": " + strerror(errno)); }
constexpr size_t kReadPosOff = sizeof(size_t);
constexpr size_t kWritePosOff = 2 * sizeof(size_t);
constexpr size_t kLockOff = 3 * sizeof(size_t);
constexpr size_t kRingOff = kLockOff + sizeof(std::atomic_flag);
static_assert(sizeof(std::atomic<size_t>) == sizeof(size_t), "positions must be plain words in shared memory");
}  // namespace

ShmChannel& ShmChannel::operator=(ShmChannel&& o) noexcept {
    if (this != &o) {
        disconnect();
        fd_ = o.fd_; shm_ = o.shm_; ring_ = o.ring_; size_ = o.size_; total_size_ = o.total_size_;
        owner_ = o.owner_; created_ = o.created_; shm_name_ = std::move(o.shm_name_);
        cached_read_ = o.cached_read_; cached_write_ = o.cached_write_;
        read_pos_ = o.read_pos_; write_pos_ = o.write_pos_; lock_ = o.lock_;
        o.shm_ = nullptr; o.fd_ = -1; o.owner_ = false;
    }
    return *this;
}

void ShmChannel::connect(const std::string& name, size_t size) {
    disconnect();
    created_ = name.empty() || size > 0;
    if (!name.empty()) {
        shm_name_ = "llis:channel:" + name;
        fd_ = shm_open(shm_name_.c_str(), created_ ? (O_CREAT | O_RDWR) : O_RDWR, 0600);
        if (fd_ < 0) fail("shm_open(" + shm_name_ + ")");
        if (created_) {
            size_ = size;
        } else {
            void* hdr = mmap(nullptr, sizeof(size_t), PROT_READ, MAP_SHARED, fd_, 0);
            if (hdr == MAP_FAILED) fail("mmap(channel header)");
            size_ = *static_cast<size_t*>(hdr);
            munmap(hdr, sizeof(size_t));
        }
    } else {
        shm_name_.clear();
        size_ = size;
    }
    if (size_ < 2) throw std::runtime_error("shm channel needs a ring of at least 2 bytes");
    total_size_ = kRingOff + size_;
    void* p;
    if (!name.empty()) {
        if (created_ && ftruncate(fd_, (off_t)total_size_) != 0) fail("ftruncate(channel)");
        p = mmap(nullptr, total_size_, PROT_READ | PROT_WRITE, MAP_SHARED, fd_, 0);
    } else {
        p = mmap(nullptr, total_size_, PROT_READ | PROT_WRITE, MAP_SHARED | MAP_ANONYMOUS, -1, 0);
    }
    if (p == MAP_FAILED) fail("mmap(channel)");
    shm_ = static_cast<char*>(p);
    owner_ = true;
    ring_ = shm_ + kRingOff;
    read_pos_ = reinterpret_cast<std::atomic<size_t>*>(shm_ + kReadPosOff);
    write_pos_ = reinterpret_cast<std::atomic<size_t>*>(shm_ + kWritePosOff);
    lock_ = reinterpret_cast<std::atomic_flag*>(shm_ + kLockOff);
    if (created_) {
        *reinterpret_cast<size_t*>(shm_) = size_;
        read_pos_->store(0, std::memory_order_release);
        write_pos_->store(0, std::memory_order_release);
        lock_->clear(std::memory_order_release);
        cached_read_ = cached_write_ = 0;
    } else {
        cached_read_ = read_pos_->load(std::memory_order_acquire);
        cached_write_ = write_pos_->load(std::memory_order_acquire);
    }
}

void ShmChannel::connect(ShmChannel* o) {
    disconnect();
    fd_ = -1; shm_ = o->shm_; ring_ = o->ring_; size_ = o->size_; total_size_ = o->total_size_;
    owner_ = false; created_ = false; shm_name_.clear();
    read_pos_ = o->read_pos_; write_pos_ = o->write_pos_; lock_ = o->lock_;
    cached_read_ = read_pos_->load(std::memory_order_acquire);
    cached_write_ = write_pos_->load(std::memory_order_acquire);
}

void ShmChannel::disconnect() {
    if (shm_ && owner_) {
        munmap(shm_, total_size_);
        if (fd_ >= 0) close(fd_);
        if (created_ && !shm_name_.empty()) shm_unlink(shm_name_.c_str());
    }
    shm_ = nullptr;
    fd_ = -1;
    owner_ = false;
}

bool ShmChannel::read(void* buf, size_t size, uint64_t max_spins) {
    char* out = static_cast<char*>(buf);
    while (size > 0) {
        uint64_t spins = 0;
        while ((cached_write_ = write_pos_->load(std::memory_order_acquire)) == cached_read_) {
            if (max_spins && ++spins > max_spins) return false;
        }
        const size_t end = cached_write_ < cached_read_ ? size_ : cached_write_;
        const size_t n = size < end - cached_read_ ? size : end - cached_read_;
        memcpy(out, ring_ + cached_read_, n);
        out += n;
        size -= n;
        cached_read_ += n;
        if (cached_read_ == size_) cached_read_ = 0;
        read_pos_->store(cached_read_, std::memory_order_release);
    }
    return true;
}

bool ShmChannel::write(const void* buf, size_t size, uint64_t max_spins) {
    const char* in = static_cast<const char*>(buf);
    while (size > 0) {
        uint64_t spins = 0;
        while ((cached_write_ + 1) % size_ == (cached_read_ = read_pos_->load(std::memory_order_acquire))) {
            if (max_spins && ++spins > max_spins) return false;
        }
        size_t room;
        if (cached_read_ <= cached_write_) room = size_ - cached_write_ - (cached_read_ == 0 ? 1 : 0);
        else room = cached_read_ - cached_write_ - 1;
        const size_t n = size < room ? size : room;
        memcpy(ring_ + cached_write_, in, n);
        in += n;
        size -= n;
        cached_write_ += n;
        if (cached_write_ == size_) cached_write_ = 0;
        write_pos_->store(cached_write_, std::memory_order_release);
    }
    return true;
}

bool ShmChannel::can_read() {
    if (cached_write_ != cached_read_) return true;
    return write_pos_->load(std::memory_order_acquire) != cached_read_;
}

size_t ShmChannel::writable_bytes() {
    cached_read_ = read_pos_->load(std::memory_order_acquire);
    const size_t used = cached_write_ >= cached_read_ ? cached_write_ - cached_read_ : size_ - cached_read_ + cached_write_;
    return size_ - 1 - used;        // one byte always stays free
}

void ShmChannel::acquire_writer_lock() {
    while (lock_->test_and_set(std::memory_order_acquire)) {}
    // another writer may have moved the shared position since this endpoint last wrote
    cached_write_ = write_pos_->load(std::memory_order_acquire);
}
void ShmChannel::release_writer_lock() { lock_->clear(std::memory_order_release); }

// ---------------------------------------------------------------------------------------------
UnixDatagramSocket::UnixDatagramSocket() {
    socket_ = socket(AF_UNIX, SOCK_DGRAM, 0);
    if (socket_ < 0) fail("socket(AF_UNIX, SOCK_DGRAM)");
    is_owner_ = true;
}
UnixDatagramSocket::UnixDatagramSocket(const std::string& name) : UnixDatagramSocket() { bind(name); }
UnixDatagramSocket::~UnixDatagramSocket() {
    if (is_owner_ && socket_ >= 0) close(socket_);
}
UnixDatagramSocket& UnixDatagramSocket::operator=(UnixDatagramSocket&& o) noexcept {
    if (this != &o) {
        if (is_owner_ && socket_ >= 0) close(socket_);
        socket_ = o.socket_; is_owner_ = o.is_owner_; remote_addr_ = o.remote_addr_;
        o.socket_ = -1; o.is_owner_ = false;
    }
    return *this;
}
static void abstract_addr(sockaddr_un* a, const std::string& name) {
    memset(a, 0, sizeof(*a));
    a->sun_family = AF_UNIX;
    strncpy(a->sun_path + 1, name.c_str(), sizeof(a->sun_path) - 2);
}
void UnixDatagramSocket::bind(const std::string& name) {
    sockaddr_un a;
    abstract_addr(&a, name);
    if (::bind(socket_, reinterpret_cast<const sockaddr*>(&a), sizeof(a)) != 0) fail("bind(" + name + ")");
}
UnixDatagramSocket UnixDatagramSocket::connect(const std::string& name) {
    UnixDatagramSocket res(socket_);
    abstract_addr(&res.remote_addr_, name);
    return res;
}
ssize_t UnixDatagramSocket::write(const void* buf, size_t count) {
    const ssize_t n = sendto(socket_, buf, count, 0, reinterpret_cast<const sockaddr*>(&remote_addr_), sizeof(remote_addr_));
    if (n < 0) fail("sendto");
    return n;
}
ssize_t UnixDatagramSocket::try_write(const void* buf, size_t count) {
    const ssize_t n = sendto(socket_, buf, count, MSG_DONTWAIT | MSG_NOSIGNAL, reinterpret_cast<const sockaddr*>(&remote_addr_), sizeof(remote_addr_));
    return n >= 0 ? n : -(ssize_t)errno;
}
ssize_t UnixDatagramSocket::read(void* buf, size_t count) {
    const ssize_t n = ::read(socket_, buf, count);
    if (n < 0) fail("read(datagram)");
    return n;
}
ssize_t UnixDatagramSocket::read_timeout(void* buf, size_t count, int timeout_ms) {
    pollfd p{socket_, POLLIN, 0};
    const int r = poll(&p, 1, timeout_ms);
    if (r < 0) fail("poll(datagram)");
    if (r == 0) return 0;
    return read(buf, count);
}

}  // namespace ipc
}  // namespace llis
