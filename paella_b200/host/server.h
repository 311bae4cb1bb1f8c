// One serving instance: ring + stream/notifier pools + scheduler + job registry,
// with an in-process client endpoint (launch / poll_done).
//
// Plays the part of the reference's Server (src/server/server.cpp:29-35 serve loop,
// :43-80 message dispatch, :120-167 launch and completion messages) and of
// RegisteredJob's plugin loading (src/server/registered_job.cpp:26-59).  One object per
// GPU; every method must be called from the thread that created it.
#pragma once

#include <llis/ipc/shm_primitive_channel.h>
#include <llis/job/finished_block_notifier.h>
#include <llis/server/scheduler.h>

#include <chrono>
#include <functional>
#include <memory>
#include <string>
#include <vector>

#include "paella_b200.h"
#include "registry.h"

struct pb_server final : public llis::server::SchedulerHost {
    struct Done {
        uint64_t cookie;
        int32_t error;
    };

    pb_server() = default;
    ~pb_server() override;
    int init(const pb_server_config& cfg);
    int register_job(const char* path, uint32_t* id_out);
    int launch(uint32_t job_ref_id, void* io_ptr, uint64_t cookie, llis::ClientId client_id = 0);
    int step(int max_records);

    // SchedulerHost
    double now_us() override {
        return std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now().time_since_epoch()).count();
    }
    void after_mem_stage(llis::job::Job* job) override;
    void update_job_stage_length(llis::job::Job* job, unsigned stage, double len) override { type_of(job).update_stage_length(stage, len); }
    bool has_job_stage_resource(llis::job::Job* job, unsigned stage) override { return type_of(job).has_stage_resource(stage); }
    void set_job_stage_resource(llis::job::Job* job, unsigned stage, float res) override { type_of(job).set_stage_resource(stage, res); }
    double get_job_remaining_rl(llis::job::Job* job, unsigned from) override { return type_of(job).remaining_rl(from); }
    const std::vector<double>& get_job_stage_lengths(llis::job::Job* job) override { return type_of(job).stage_lengths; }
    const std::vector<float>& get_job_stage_resources(llis::job::Job* job) override { return type_of(job).stage_resources; }
    void notify_job_starts(llis::job::Job* job) override {
        ++num_pre_notified;
        if (on_job_starts) on_job_starts(job);
    }
    void notify_job_ends(llis::job::Job* job) override {
        if (on_job_ends) on_job_ends(job);
        else done.push_back(Done{(uint64_t)(uintptr_t)job->get_remote_ptr(), job->has_error()});
    }
    void release_job_instance(llis::job::Job* job) override { type_of(job).give_back(job); }
    void on_dispatch(llis::job::Job*, bool is_mem, bool, unsigned, unsigned) override {
        if (is_mem) ++num_mem_stages; else ++num_kernels;
    }

    llis::server::JobType& type_of(llis::job::Job* job) { return *types[job->get_registered_job_id()]; }

    // Set by the IPC front-end: completion goes to the client's rings instead of the `done` list.
    std::function<void(llis::job::Job*)> on_job_starts, on_job_ends;
    pb_server_config cfg{};
    int device = 0;
    llis::ipc::Gpu2SchedChannel channel;
    std::vector<cudaStream_t> streams;
    llis::job::FinishedBlockNotifier* notifiers_raw = nullptr;
    std::unique_ptr<llis::server::Scheduler> scheduler;
    std::vector<std::unique_ptr<llis::server::JobType>> types;
    std::vector<Done> done;
    uint64_t num_pre_notified = 0, num_kernels = 0, num_mem_stages = 0, num_records = 0;
    int last_error = 0;
};
