// Client library: talks to a llis_server over the c2s / s2c shared-memory rings and the start-notify
// datagram socket.  Same classes, methods and wire messages as the reference's client
// (src/client/client.cpp, src/client/job_ref.cpp, src/client/job_instance_ref.cpp):
//   REGISTER_CLIENT {tmp id}                      -> permanent id on the temporary s2c ring
//   REGISTER_JOB    {client id, plugin path, shm name} -> job_ref_id on s2c
//   GROW_POOL       {job_ref_id, bytes}           (pool chunks of 30 638 080 bytes, job_ref.cpp:70-101)
//   LAUNCH_JOB      {job_ref_id, chunk id (int), offset (size_t), JobInstanceRef*}
//   completion: one byte on the datagram socket when the job's pre-notify stage is dispatched,
//   then the JobInstanceRef* on s2c when the job ends (client.cpp:118-128).
#pragma once

#include <llis/ipc/shm_channel.h>
#include <llis/ipc/unix_datagram_socket.h>
#include <llis/job/job.h>

#include <memory>
#include <mutex>
#include <string>
#include <vector>

namespace llis {
namespace client {

class Client;
class JobRef;

struct IoShmEntry {
    int id = 0;            // which pool chunk
    size_t offset = 0;     // byte offset inside the chunk
    void* ptr = nullptr;   // client-side address
};

class JobInstanceRef {
  public:
    JobInstanceRef(JobRef* job_ref, IoShmEntry entry) : job_ref_(job_ref), io_shm_entry_(entry) {}
    void launch();
    void release();
    void* get_input_ptr() { return io_shm_entry_.ptr; }
    void* get_output_ptr();
    void set_id(JobInstanceRefId id) { id_ = id; }
    JobInstanceRefId get_id() const { return id_; }
    JobRefId get_job_ref_id() const;
    JobRef* get_job_ref() const { return job_ref_; }
    void set_start_time(double t) { start_time_ = t; }
    double get_start_time() const { return start_time_; }

  private:
    JobRef* job_ref_;
    IoShmEntry io_shm_entry_;
    JobInstanceRefId id_ = 0;
    double start_time_ = 0;
};

class JobRef {
  public:
    JobRef(job::Job* job, Client* client, std::string model_path);
    JobRef(const JobRef&) = delete;
    JobRef& operator=(const JobRef&) = delete;
    JobInstanceRef* create_instance();
    void release_io_shm_entry(IoShmEntry e) { pinned_mem_free_list_.push_back(e); }
    JobRefId get_job_ref_id() const { return job_ref_id_; }
    job::Job* get_job() const { return job_; }
    Client* get_client() const { return client_; }
    size_t pool_entries() const { return pool_size_; }

  private:
    void register_job();
    void grow_pool(size_t least_num_new_entries);
    job::Job* job_;
    Client* client_;
    std::string model_path_;
    std::string shm_name_;
    int shm_fd_ = -1;
    size_t pinned_mem_size_ = 0;
    size_t pool_size_ = 0, pool_size_in_bytes_ = 0;
    std::vector<void*> pinned_mem_list_;
    std::vector<IoShmEntry> pinned_mem_free_list_;
    JobRefId job_ref_id_ = 0;
};

class Client {
  public:
    explicit Client(std::string server_name);
    ~Client();
    Client(const Client&) = delete;
    Client& operator=(const Client&) = delete;

    // dlopens the plugin for its I/O sizes and registers it with the server.
    JobRef* register_job(const std::string& path);
    // Blocks for the next finished job: start datagram first, then the pointer on s2c.
    JobInstanceRef* wait();
    // As wait(), but returns NULL when nothing finished within timeout_ms.
    JobInstanceRef* wait_timeout(int timeout_ms);
    void kill_server();
    // PROFILER_CMD + sub-command (src/client/profiler_client.cpp of the reference: set/unset_record_job_events,
    // set/unset_record_run_next_times, ..., save(path)); `path` travels only with ProfilerMsgType::SAVE.
    void profiler_cmd(ProfilerMsgType cmd, const std::string& path = std::string());

    ClientId get_client_id() const { return client_id_; }
    ipc::ShmChannel* get_c2s_channel() { return &c2s_channel_; }
    ipc::ShmChannel* get_s2c_channel() { return &s2c_channel_; }
    JobInstanceRef* add_job_instance_ref(JobInstanceRef ref);
    void release_job_instance_ref(JobInstanceRef* ref);

  private:
    std::string server_name_;
    ipc::ShmChannel c2s_channel_;
    ipc::ShmChannel s2c_channel_;
    ipc::UnixDatagramSocket s2c_socket_;
    size_t entries_ahead_ = 0;   // ring entries consumed before their wake-up datagram arrived
    ClientId client_id_ = 0;
    std::mutex mtx_;
    std::vector<std::unique_ptr<JobInstanceRef>> job_instance_refs_;
    std::vector<JobInstanceRefId> unused_job_instance_refs_;
    std::vector<std::unique_ptr<JobRef>> job_refs_;
};

}  // namespace client
}  // namespace llis
