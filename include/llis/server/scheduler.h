// Scheduler interface and the services a scheduler needs from its server.
//
// Scheduler mirrors the reference's include/llis/server/scheduler.h:18-31
// (handle_new_job + try_handle_block_start_finish); SchedulerHost gathers the Server
// methods the reference's schedulers call (include/llis/server/server.h:24-71:
// update_job_stage_length, has/set_job_stage_resource, get_job_remaining_rl,
// get_job_stage_lengths/resources, notify_job_starts/ends, release_job_instance), plus
// the clock and the pools, so the same scheduler object runs against a live GPU or
// against a recorded trace.
#pragma once

#include <chrono>
#include <memory>
#include <string>
#include <vector>

#include <llis/job/instrument_info.h>
#include <llis/job/job.h>
#include <llis/server/sm_resources.h>

namespace llis {
namespace server {

class SchedulerHost {
  public:
    virtual ~SchedulerHost() = default;
    virtual double now_us() = 0;
    // Called right after run_next() of a copy stage: must make a kMemDone record for the
    // job appear once the copy has completed (live server: a one-block marker kernel
    // queued behind the copy on the job's stream).
    virtual void after_mem_stage(job::Job* job) = 0;
    virtual void update_job_stage_length(job::Job* job, unsigned stage, double len_us) = 0;
    virtual bool has_job_stage_resource(job::Job* job, unsigned stage) = 0;
    virtual void set_job_stage_resource(job::Job* job, unsigned stage, float res) = 0;
    virtual double get_job_remaining_rl(job::Job* job, unsigned from_stage) = 0;
    virtual const std::vector<double>& get_job_stage_lengths(job::Job* job) = 0;
    virtual const std::vector<float>& get_job_stage_resources(job::Job* job) = 0;
    virtual void notify_job_starts(job::Job* job) = 0;
    virtual void notify_job_ends(job::Job* job) = 0;
    virtual void release_job_instance(job::Job* job) = 0;
    // Observation hook: host time around a stage's run_next() (profiler: KERNEL_SUBMIT_START / _END).
    virtual void on_stage_submitted(job::Job* job, double start_us, double end_us) { (void)job; (void)start_us; (void)end_us; }
    // Observation hook: one call per dispatched stage (decision log for replay parity).
    virtual void on_dispatch(job::Job* job, bool is_mem, bool unfit, unsigned stream_slot, unsigned notifier_slot) {
        (void)job; (void)is_mem; (void)unfit; (void)stream_slot; (void)notifier_slot;
    }
};

struct SchedulerConfig {
    unsigned num_streams = 500;
    unsigned extra_kernels = 2;       // over-subscribed ("unfit") kernels allowed in flight
    double unfairness_threshold = 1e6;
    unsigned sched_sleep = 0;
    unsigned max_gang = 1;            // jobs of one type the scheduler may dispatch as one launch per stage (1 = never)
    // Stage watchdog (0 = off, the reference: a kernel that never reports its last block wedges the server,
    // src/server/server.cpp:29-35 has no timeout).  A stage in flight for longer than
    // max(watchdog_factor x the type's learned length of that stage, watchdog_floor_us) is given up:
    // the job (and its gang) ends with PB_ERR_TIMEOUT, its occupancy is released, and its job id, stream and
    // notifier are retired for good, because the kernel may still be running and report later.
    double watchdog_factor = 0;
    double watchdog_floor_us = 100000;
    SmTotals totals;
};

class Scheduler {
  public:
    virtual ~Scheduler() = default;
    virtual void handle_new_job(job::Job* job) = 0;
    // Consumes one notification record (block start, block end or copy done).
    virtual void handle_record(const job::InstrumentInfo& info) = 0;
    // Deferred scheduling (off by default = the reference's behaviour: the dispatch loop runs inside every
    // handle_new_job / handle_record that may have made a stage runnable).  When on, those calls only update
    // the queue and the occupancy model, and the dispatch loop runs once per flush(): the server calls it after
    // each batch of client messages and ring records.  Fewer passes over the queue per request, and requests
    // that arrive together are queued together, which is what lets a gang form.
    virtual void set_deferred(bool on) { (void)on; }
    virtual void flush() {}
    // Gives up stages that have been in flight for too long (see SchedulerConfig::watchdog_factor); returns how
    // many jobs were failed.  The server calls it about once a millisecond.
    virtual unsigned check_watchdog(double now_us) { (void)now_us; return 0; }
    virtual unsigned num_jobs() const = 0;
    virtual uint64_t num_decisions() const = 0;
    virtual const char* name() const = 0;

    // Stream / notifier pools are handed over by the server (slot i <-> element i).
    virtual void set_pools(const std::vector<cudaStream_t>& streams, const std::vector<job::FinishedBlockNotifier*>& notifiers) = 0;

    // Records the scheduler made up itself: when a plugin's run_next() fails (error flag set, nothing
    // was enqueued) no notification will ever come from the GPU, so the scheduler queues the records
    // that close the stage and the server feeds them back through handle_record().  The job then
    // runs (and fails) through its remaining stages and ends with its error reported to the client.
    bool take_synthetic(std::vector<job::InstrumentInfo>* out) {
        if (synthetic_.empty()) return false;
        out->swap(synthetic_);
        synthetic_.clear();
        return true;
    }

    static std::unique_ptr<Scheduler> create(const std::string& name, const SchedulerConfig& cfg, SchedulerHost* host);

    // Host time spent inside plugins' run_next() so far (CUDA launch calls), nanoseconds.
    uint64_t run_next_ns() const { return run_next_ns_; }

  protected:
    void run_stage(job::Job* job, SchedulerHost* host) {
        const auto t0 = std::chrono::steady_clock::now();
        job->run_next();
        const auto t1 = std::chrono::steady_clock::now();
        run_next_ns_ += (uint64_t)std::chrono::duration_cast<std::chrono::nanoseconds>(t1 - t0).count();
        host->on_stage_submitted(job, std::chrono::duration<double, std::micro>(t0.time_since_epoch()).count(),
                                 std::chrono::duration<double, std::micro>(t1.time_since_epoch()).count());
    }
    uint64_t run_next_ns_ = 0;

    // Closes the stage a failed run_next() left open (see take_synthetic).
    void close_failed_stage(job::Job* job, bool is_mem) {
        job::InstrumentInfo r{};
        r.job_id = job->get_id();
        r.status = 1;
        if (is_mem) {
            r.is_start = job::InstrumentInfo::kMemDone;
            r.num = 1;
            synthetic_.push_back(r);
            return;
        }
        for (int kind = 0; kind < 2; ++kind) {
            unsigned left = job->get_cur_num_blocks();
            while (left > 0) {
                const unsigned n = left > 255 ? 255 : left;
                r.is_start = kind == 0 ? job::InstrumentInfo::kStart : job::InstrumentInfo::kEnd;
                r.num = (uint8_t)n;
                synthetic_.push_back(r);
                left -= n;
            }
        }
    }
    std::vector<job::InstrumentInfo> synthetic_;
};

}  // namespace server
}  // namespace llis
