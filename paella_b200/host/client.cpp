#include <llis/client/client.h>
#include <llis/ipc/defs.h>
#include <llis/ipc/name_format.h>

#include <dlfcn.h>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <random>
#include <stdexcept>

namespace llis {
namespace client {

namespace {
constexpr size_t kPoolChunkBytes = 30638080;   // fixed chunk of the reference (src/client/job_ref.cpp:74)
}

// ---- JobInstanceRef -------------------------------------------------------------------------
void* JobInstanceRef::get_output_ptr() {
    // the job's own offset (input size rounded up to 8); the reference adds the raw input size, which
    // is the same for every served model because their input sizes are multiples of 8
    return static_cast<char*>(io_shm_entry_.ptr) + job_ref_->get_job()->get_output_offset();
}

void JobInstanceRef::launch() {
    ipc::ShmChannel* c2s = job_ref_->get_client()->get_c2s_channel();
    c2s->acquire_writer_lock();
    c2s->write(MsgType::LAUNCH_JOB);
    c2s->write(job_ref_->get_job_ref_id());
    c2s->write(io_shm_entry_.id);
    c2s->write(io_shm_entry_.offset);
    c2s->write(this);
    c2s->release_writer_lock();
}

void JobInstanceRef::release() { job_ref_->release_io_shm_entry(io_shm_entry_); }
JobRefId JobInstanceRef::get_job_ref_id() const { return job_ref_->get_job_ref_id(); }

// ---- JobRef -----------------------------------------------------------------------------------
JobRef::JobRef(job::Job* job, Client* client, std::string model_path) : job_(job), client_(client), model_path_(std::move(model_path)) {
    pinned_mem_size_ = job_->get_pinned_mem_size();
    shm_name_ = "llis:shm:" + std::to_string(client_->get_client_id()) + ":" + std::to_string((intptr_t)this);
    shm_fd_ = shm_open(shm_name_.c_str(), O_CREAT | O_RDWR, 0600);
    if (shm_fd_ < 0) throw std::runtime_error("shm_open(" + shm_name_ + ") failed");
    register_job();
    grow_pool(2);
}

void JobRef::register_job() {
    ipc::ShmChannel* c2s = client_->get_c2s_channel();
    c2s->acquire_writer_lock();
    c2s->write(MsgType::REGISTER_JOB);
    c2s->write(client_->get_client_id());
    c2s->write(model_path_);
    c2s->write(shm_name_);
    c2s->release_writer_lock();
    client_->get_s2c_channel()->read(&job_ref_id_);
}

JobInstanceRef* JobRef::create_instance() {
    if (pinned_mem_free_list_.empty()) grow_pool(pool_size_);
    const IoShmEntry e = pinned_mem_free_list_.back();
    pinned_mem_free_list_.pop_back();
    return client_->add_job_instance_ref(JobInstanceRef(this, e));
}

void JobRef::grow_pool(size_t) {
    const size_t num_new_bytes = kPoolChunkBytes;
    const size_t num_new_entries = num_new_bytes / pinned_mem_size_;
    const size_t old_bytes = pool_size_in_bytes_;
    pool_size_ += num_new_entries;
    pool_size_in_bytes_ += num_new_bytes;
    if (ftruncate(shm_fd_, (off_t)pool_size_in_bytes_) != 0) throw std::runtime_error("ftruncate(request pool) failed");
    void* p = mmap(nullptr, num_new_bytes, PROT_READ | PROT_WRITE, MAP_SHARED, shm_fd_, (off_t)old_bytes);
    if (p == MAP_FAILED) throw std::runtime_error("mmap(request pool) failed");
    pinned_mem_list_.push_back(p);
    for (size_t i = 0; i < num_new_entries; ++i) {
        IoShmEntry e;
        e.id = (int)pinned_mem_list_.size() - 1;
        e.offset = i * pinned_mem_size_;
        e.ptr = static_cast<char*>(p) + e.offset;
        pinned_mem_free_list_.push_back(e);
    }
    ipc::ShmChannel* c2s = client_->get_c2s_channel();
    c2s->acquire_writer_lock();
    c2s->write(MsgType::GROW_POOL);
    c2s->write(job_ref_id_);
    c2s->write(num_new_bytes);
    c2s->release_writer_lock();
}

// ---- Client -----------------------------------------------------------------------------------
Client::Client(std::string server_name) : server_name_(std::move(server_name)), c2s_channel_(ipc::c2s_channel_name(server_name_)) {
    std::random_device rnd;
    client_id_ = rnd();
    // temporary ring named after a random id; the server answers on it with the permanent id
    s2c_channel_.connect(ipc::s2c_channel_name(server_name_, client_id_), 8);
    c2s_channel_.acquire_writer_lock();
    c2s_channel_.write(MsgType::REGISTER_CLIENT);
    c2s_channel_.write(client_id_);
    c2s_channel_.release_writer_lock();
    s2c_channel_.read(&client_id_);
    s2c_channel_.disconnect();
    s2c_channel_.connect(ipc::s2c_channel_name(server_name_, client_id_));
    s2c_socket_.bind(ipc::s2c_socket_name(server_name_, client_id_));
}

Client::~Client() = default;

JobRef* Client::register_job(const std::string& path) {
    void* handle = dlopen(path.c_str(), RTLD_NOW);
    if (!handle) throw std::runtime_error(std::string("cannot load job definition: ") + dlerror());
    typedef job::Job* (*init_job_t)();
    init_job_t init_job = (init_job_t)dlsym(handle, "init_job");
    if (!init_job) throw std::runtime_error(path + " exports no init_job");
    job_refs_.push_back(std::make_unique<JobRef>(init_job(), this, path));
    return job_refs_.back().get();
}

JobInstanceRef* Client::add_job_instance_ref(JobInstanceRef ref) {
    std::lock_guard<std::mutex> lk(mtx_);
    if (unused_job_instance_refs_.empty()) {
        ref.set_id((JobInstanceRefId)job_instance_refs_.size());
        job_instance_refs_.push_back(std::make_unique<JobInstanceRef>(ref));
        return job_instance_refs_.back().get();
    }
    const JobInstanceRefId id = unused_job_instance_refs_.back();
    unused_job_instance_refs_.pop_back();
    ref.set_id(id);
    *job_instance_refs_[id] = ref;
    return job_instance_refs_[id].get();
}

void Client::release_job_instance_ref(JobInstanceRef* ref) {
    std::lock_guard<std::mutex> lk(mtx_);
    unused_job_instance_refs_.push_back(ref->get_id());
}

// One wake-up datagram and one ring entry per finished job (src/client/client.cpp:103-131 of the
// reference: read the datagram, then the entry).  The datagram is only a hint - it is sent when the
// job's last stage STARTS, and a server may deliver it late when this socket's short queue is full -
// so an entry that is already in the ring is taken at once and the datagram it "owes" is swallowed
// when it turns up.  Datagrams and entries stay paired one to one.
JobInstanceRef* Client::wait() {
    for (;;) {
        JobInstanceRef* r = wait_timeout(1000);
        if (r) return r;
    }
}

JobInstanceRef* Client::wait_timeout(int timeout_ms) {
    for (;;) {
        if (s2c_channel_.can_read()) {
            JobInstanceRef* res = nullptr;
            s2c_channel_.read(&res);
            ++entries_ahead_;
            return res;
        }
        bool flag;
        if (s2c_socket_.read_timeout(&flag, sizeof(flag), timeout_ms) <= 0) return nullptr;
        if (entries_ahead_ > 0) { --entries_ahead_; continue; }      // pays for an entry taken earlier
        JobInstanceRef* res = nullptr;                                // its entry follows shortly
        s2c_channel_.read(&res);
        return res;
    }
}

void Client::kill_server() {
    c2s_channel_.acquire_writer_lock();
    c2s_channel_.write(MsgType::EXIT_CMD);
    c2s_channel_.release_writer_lock();
}

void Client::profiler_cmd(ProfilerMsgType cmd, const std::string& path) {
    c2s_channel_.acquire_writer_lock();
    c2s_channel_.write(MsgType::PROFILER_CMD);
    c2s_channel_.write(cmd);
    if (cmd == ProfilerMsgType::SAVE) c2s_channel_.write(path);
    c2s_channel_.release_writer_lock();
}

}  // namespace client
}  // namespace llis
