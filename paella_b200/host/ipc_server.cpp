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
    core_->on_job_ends = [this](job::Job* job) {
        ClientConnection& c = *clients_[job->get_client_id()];
        if (c.gone) return;             // nobody reads that ring any more
        void* remote = job->get_remote_ptr();
        c.s2c_channel.write(remote);
    };
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
    RegisteredJob& j = jobs_.at(id);
    void* p = mmap(nullptr, num_new_bytes, PROT_READ | PROT_WRITE, MAP_SHARED, j.shm_fd, (off_t)j.pool_bytes);
    if (p == MAP_FAILED) throw std::runtime_error("mmap of the client's request pool failed");
    if (mlock(p, num_new_bytes) != 0) fprintf(stderr, "llis_server: mlock of %zu pool bytes failed (continuing)\n", num_new_bytes);
    // Pinned and mapped: kernels read requests and write results in place.
    const cudaError_t e = cudaHostRegister(p, num_new_bytes, cudaHostRegisterMapped | cudaHostRegisterPortable);
    if (e != cudaSuccess) throw std::runtime_error(std::string("cudaHostRegister(request pool): ") + cudaGetErrorString(e));
    j.pool_bytes += num_new_bytes;
    j.mapped.push_back(p);
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
    RegisteredJob& j = jobs_.at(id);
    void* io = static_cast<char*>(j.mapped.at((size_t)chunk)) + offset;
    const int rc = core_->launch(id, io, (uint64_t)(uintptr_t)remote_ptr, j.client_id);
    if (rc != PB_OK) fprintf(stderr, "llis_server: launch of job type %u failed: %s\n", id, pb_last_error());
}

}  // namespace server
}  // namespace llis
