#include "ipc_server.h"

#include <cuda_runtime.h>
#include <fcntl.h>
#include <llis/ipc/defs.h>
#include <llis/ipc/name_format.h>
#include <sys/mman.h>
#include <unistd.h>

#include <cerrno>
#include <cstdio>
#include <cstring>
#include <stdexcept>

namespace llis {
namespace server {

IpcServer::IpcServer(std::string name, const pb_server_config& cfg) : name_(std::move(name)) {
    core_ = std::make_unique<pb_server>();
    if (core_->init(cfg) != PB_OK) throw std::runtime_error(pb_last_error());
    c2s_channel_.connect(ipc::c2s_channel_name(name_), c2s_channel_size);
    core_->on_job_starts = [this](job::Job* job) { wake(*clients_[job->get_client_id()]); };
    core_->on_job_ends = [this](job::Job* job) { complete(*clients_[job->get_client_id()], job->get_remote_ptr()); };
}

// Completion entry for one job on its client's ring.  Never waits: a client that is alive but not
// draining (or one that died with nothing left to wake) would otherwise stall the one server thread, and
// with it every other client.  What does not fit is kept, in order, and retried from step(); a client whose
// ring stays full for kStallLimit is treated as gone.
void IpcServer::complete(ClientConnection& c, void* remote_ptr) {
    if (c.gone) return;             // nobody reads that ring any more
    if (c.pending_done.empty() && c.s2c_channel.writable_bytes() >= sizeof(remote_ptr)) {
        c.s2c_channel.write(remote_ptr);
        return;
    }
    if (c.pending_done.empty()) c.stalled_since = std::chrono::steady_clock::now();
    c.pending_done.push_back(remote_ptr);
}

void IpcServer::retry_completions() {
    constexpr auto kStallLimit = std::chrono::seconds(10);
    for (auto& cp : clients_) {
        ClientConnection& c = *cp;
        while (!c.gone && !c.pending_done.empty() && c.s2c_channel.writable_bytes() >= sizeof(void*)) {
            c.s2c_channel.write(c.pending_done.front());
            c.pending_done.pop_front();
            c.stalled_since = std::chrono::steady_clock::now();
        }
        if (!c.gone && !c.pending_done.empty() && std::chrono::steady_clock::now() - c.stalled_since > kStallLimit) {
            fprintf(stderr, "llis_server: a client has not read its completions for 10 s; dropping it\n");
            c.gone = true;
            c.pending_done.clear();
            c.pending_wakeups = 0;
        }
    }
}

// One wake-up datagram per finishing job.  The client's receive queue is short (net.unix.max_dgram_qlen,
// typically 10): a send that does not fit is kept and retried from step(), never waited for - a server
// blocked in sendto() and a client blocked writing the full request ring would deadlock.
void IpcServer::wake(ClientConnection& c) {
    if (c.gone) return;
    if (c.pending_wakeups > 0) { ++c.pending_wakeups; return; }     // keep the order simple: queue behind the backlog
    const bool msg = true;
    const ssize_t n = c.s2c_socket.try_write(&msg, sizeof(msg));
    if (n >= 0) return;
    if (n == -EAGAIN || n == -EWOULDBLOCK || n == -ENOBUFS) { ++c.pending_wakeups; return; }
    size_t id = 0;
    while (id < clients_.size() && clients_[id].get() != &c) ++id;
    fprintf(stderr, "llis_server: client %zu is gone (%s); dropping its notifications\n", id, strerror((int)-n));
    c.gone = true;
}

void IpcServer::retry_wakeups() {
    for (auto& cp : clients_) {
        ClientConnection& c = *cp;
        while (!c.gone && c.pending_wakeups > 0) {
            const bool msg = true;
            const ssize_t n = c.s2c_socket.try_write(&msg, sizeof(msg));
            if (n >= 0) { --c.pending_wakeups; continue; }
            if (n == -EAGAIN || n == -EWOULDBLOCK || n == -ENOBUFS) break;
            c.gone = true;
            c.pending_wakeups = 0;
        }
    }
}

IpcServer::~IpcServer() {
    for (RegisteredJob& j : jobs_) {
        for (void* p : j.mapped) cudaHostUnregister(p);
        if (j.shm_fd >= 0) close(j.shm_fd);
    }
}

bool IpcServer::step() {
    // drain what the clients have queued (bounded, so that notifications are still polled in between)
    for (int i = 0; i < 32 && running_ && c2s_channel_.can_read(); ++i) handle_c2s();
    if (core_->step(64) < 0) throw std::runtime_error(pb_last_error());
    retry_completions();
    retry_wakeups();
    return running_;
}

void IpcServer::handle_c2s() {
    MsgType type;
    c2s_channel_.read(&type);
    switch (type) {
        case MsgType::REGISTER_CLIENT: handle_register_client(); break;
        case MsgType::REGISTER_JOB: handle_register_job(); break;
        case MsgType::LAUNCH_JOB: handle_launch_job(); break;
        case MsgType::GROW_POOL: handle_grow_pool(); break;
        case MsgType::CUDA_PROFILER_START:
        case MsgType::CUDA_PROFILER_STOP:
            break;   // accepted and ignored
        case MsgType::PROFILER_CMD: {
            ProfilerMsgType cmd;
            c2s_channel_.read(&cmd);
            std::string path;
            if (cmd == ProfilerMsgType::SAVE) c2s_channel_.read(&path);
            if (core_->profiler_cmd((uint32_t)cmd, path.c_str()) != PB_OK) fprintf(stderr, "llis_server: profiler command %u: %s\n", (unsigned)cmd, pb_last_error());
            break;
        }
        case MsgType::EXIT_CMD: running_ = false; break;
    }
}

void IpcServer::handle_register_client() {
    ClientId tmp_id;
    c2s_channel_.read(&tmp_id);
    ipc::ShmChannel tmp(ipc::s2c_channel_name(name_, tmp_id));          // the client's temporary ring
    ClientId id = (ClientId)clients_.size();
    for (ClientId i = 0; i < clients_.size(); ++i)
        if (!clients_[i]->in_use) { id = i; break; }
    if (id == clients_.size()) clients_.push_back(std::make_unique<ClientConnection>());
    ClientConnection& c = *clients_[id];
    c.in_use = true;
    c.s2c_channel.connect(ipc::s2c_channel_name(name_, id), s2c_channel_size);
    c.s2c_socket = s2c_socket_.connect(ipc::s2c_socket_name(name_, id));
    tmp.write(id);
}

void IpcServer::handle_register_job() {
    ClientId client_id;
    std::string path, shm_name;
    c2s_channel_.read(&client_id);
    c2s_channel_.read(&path);
    c2s_channel_.read(&shm_name);
    uint32_t type_id = 0;
    if (core_->register_job(path.c_str(), &type_id) != PB_OK) throw std::runtime_error(pb_last_error());
    if (jobs_.size() <= type_id) jobs_.resize(type_id + 1);
    RegisteredJob& j = jobs_[type_id];
    j.client_id = client_id;
    j.shm_name = shm_name;
    j.shm_fd = shm_open(shm_name.c_str(), O_RDWR, 0600);
    if (j.shm_fd < 0) throw std::runtime_error("cannot open the client's request pool " + shm_name);
    clients_[client_id]->s2c_channel.write((JobRefId)type_id);
}

void IpcServer::handle_grow_pool() {
    JobRefId id;
    size_t num_new_bytes;
    c2s_channel_.read(&id);
    c2s_channel_.read(&num_new_bytes);
    if (id >= jobs_.size() || jobs_[id].shm_fd < 0 || num_new_bytes == 0) {
        fprintf(stderr, "llis_server: GROW_POOL for unknown job %u (or of 0 bytes) ignored\n", id);
        return;
    }
    RegisteredJob& j = jobs_[id];
    void* p = mmap(nullptr, num_new_bytes, PROT_READ | PROT_WRITE, MAP_SHARED, j.shm_fd, (off_t)j.pool_bytes);
    if (p == MAP_FAILED) throw std::runtime_error("mmap of the client's request pool failed");
    if (mlock(p, num_new_bytes) != 0) fprintf(stderr, "llis_server: mlock of %zu pool bytes failed (continuing)\n", num_new_bytes);
    // Pinned and mapped: kernels read requests and write results in place.
    const cudaError_t e = cudaHostRegister(p, num_new_bytes, cudaHostRegisterMapped | cudaHostRegisterPortable);
    if (e != cudaSuccess) throw std::runtime_error(std::string("cudaHostRegister(request pool): ") + cudaGetErrorString(e));
    j.pool_bytes += num_new_bytes;
    j.mapped.push_back(p);
    j.mapped_bytes.push_back(num_new_bytes);
}

void IpcServer::handle_launch_job() {
    JobRefId id;
    int chunk;
    size_t offset;
    void* remote_ptr;
    c2s_channel_.read(&id);
    c2s_channel_.read(&chunk);
    c2s_channel_.read(&offset);
    c2s_channel_.read(&remote_ptr);
    // A malformed message must not take the server down for every other client: check what it names.
    if (id >= jobs_.size() || jobs_[id].shm_fd < 0) {
        fprintf(stderr, "llis_server: LAUNCH_JOB names unknown job %u; ignored (no client to answer)\n", id);
        return;
    }
    RegisteredJob& j = jobs_[id];
    int rc = PB_OK;
    const size_t slot_bytes = core_->types[id]->slot_bytes;
    if (chunk < 0 || (size_t)chunk >= j.mapped.size() || slot_bytes > j.mapped_bytes[(size_t)chunk] ||
        offset > j.mapped_bytes[(size_t)chunk] - slot_bytes) {
        fprintf(stderr, "llis_server: LAUNCH_JOB of job %u names chunk %d offset %zu outside its request pool\n", id, chunk, offset);
        rc = PB_ERR_INVALID;
    } else {
        void* io = static_cast<char*>(j.mapped[(size_t)chunk]) + offset;
        rc = core_->launch(id, io, (uint64_t)(uintptr_t)remote_ptr, j.client_id);
        if (rc != PB_OK) fprintf(stderr, "llis_server: launch of job type %u failed: %s\n", id, pb_last_error());
    }
    if (rc != PB_OK && j.client_id < clients_.size() && clients_[j.client_id]->in_use) {
        // The job never reached the scheduler, so no completion would ever come and the client's wait() would
        // block for good: answer now with what a finished job sends (wake-up datagram, then its pointer).
        ClientConnection& c = *clients_[j.client_id];
        wake(c);
        complete(c, remote_ptr);
    }
}

}  // namespace server
}  // namespace llis
