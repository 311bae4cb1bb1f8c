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
#include <unordered_map>
#include <utility>
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
    void update_job_stage_length(llis::job::Job* job, unsigned stage, double len) override {
        type_of(job).update_stage_length(stage, len);
        if (job_events_flag) record_job_event(job, kKernelFinished, now_us());
    }
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
        if (job_events_flag) finish_job_events(job);
        if (on_job_ends) on_job_ends(job);
        else done.push_back(Done{(uint64_t)(uintptr_t)job->get_remote_ptr(), job->has_error()});
    }
    void release_job_instance(llis::job::Job* job) override { type_of(job).give_back(job); }
    void on_dispatch(llis::job::Job* job, bool is_mem, bool, unsigned, unsigned) override {
        if (is_mem) ++num_mem_stages; else ++num_kernels;
        if (job_events_flag) record_job_event(job, kKernelSchedStart, now_us());
    }
    void on_stage_submitted(llis::job::Job* job, double start_us, double end_us) override {
        if (job_events_flag) { record_job_event(job, kKernelSubmitStart, start_us); record_job_event(job, kKernelSubmitEnd, end_us); }
        if (run_next_times_flag) run_next_times.push_back(RunNext{start_us, end_us, job->get_cur_num_blocks()});
    }

    // ---- job-event timeline (the reference's Profiler: include/llis/server/profiler.h:15-23, event codes on
    // the wire of its output file; src/server/profiler.cpp:113-121 writes one line per job, "code time_us" pairs)
    enum JobEvent { kJobSubmitted = 0, kKernelSchedStart = 1, kKernelSchedAbort = 2, kKernelSubmitStart = 3, kKernelSubmitEnd = 4,
                    kKernelFinished = 5, kJobFinished = 6 };
    struct RunNext { double start_us, end_us; unsigned num_blocks; };
    void record_job_event(llis::job::Job* job, JobEvent e, double t_us) { events_cur[job].emplace_back((int)e, t_us); }
    void finish_job_events(llis::job::Job* job);
    // One profiler sub-command (llis::ProfilerMsgType value); `path` only for SAVE.  Returns PB_OK or an error code.
    int profiler_cmd(uint32_t msg_type, const char* path);
    int profiler_save(const std::string& path);
    bool job_events_flag = false, run_next_times_flag = false;
    std::unordered_map<llis::job::Job*, std::vector<std::pair<int, double>>> events_cur;
    std::vector<std::vector<std::pair<int, double>>> events_all;
    std::vector<RunNext> run_next_times;
    std::string profile_prefix;      // PB_PROFILE_PREFIX: record from the start, save when the server goes away

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
    double last_watchdog_us = 0;
    uint64_t num_watchdog = 0;          // requests the stage watchdog gave up
};
