// The kernel-granularity scheduler ("full3"): SRPT-like priority = minus the remaining
// sum of stage_length x stage_resource, a deficit-counter fairness override between job
// types, a whole-GPU occupancy check with a bounded number of over-subscribed kernels.
//
// Decision-for-decision equivalent to the reference's SchedulerFull3
// (src/server/scheduler_full3.cpp:123-459): handle_block_start :123-144,
// handle_block_finish :146-222, handle_mem_finish :224-270, handle_new_job :272-313,
// schedule_job :315-452, calculate_priority :454-459.  Pools are LIFO as there
// (:391-397,206-207,262), ids are recycled LIFO (:280-287).
//
// What changed for this machine: copy-stage completions arrive as kMemDone records in the
// same ring as block notifications instead of a driver callback thread and a second ring;
// the occupancy totals are those of the device in use (148 SMs on B200) and include tensor
// memory; time comes from the host interface so a trace replays exactly.
//
// Gangs (SchedulerConfig::max_gang > 1; off by default, and off in every replay): when the job
// about to be dispatched is at its first stage and its plugin can run several jobs per launch,
// the queued jobs of the same type that have not started either - at most max_gang - 1 and at
// most the plugin's capacity - are taken out of the queue with it and follow it for the rest
// of their life: each stage of the leader is ONE dispatch (one stream, one notifier, one set
// of records) that serves every member, and when the leader ends all members end.  Nothing
// waits for a gang to fill: only jobs that are already queued at dispatch time join.
#include <llis/job/context.h>
#include <llis/server/job_queue.h>
#include <llis/server/scheduler.h>

#include <algorithm>
#include <cstdio>

namespace llis {
namespace server {

namespace {

class SchedulerFull3 final : public Scheduler {
  public:
    SchedulerFull3(const SchedulerConfig& cfg, SchedulerHost* host)
        : host_(host), cfg_(cfg), job_queue_(cfg.unfairness_threshold), gpu_resources_(cfg.totals),
          max_num_outstanding_kernels_(cfg.extra_kernels) {}

    const char* name() const override { return "full3"; }
    void set_deferred(bool on) override {
        deferred_ = on;
        if (!on) flush();
    }
    void flush() override {
        if (!dirty_) return;
        dirty_ = false;
        dispatch_loop();
    }
    unsigned num_jobs() const override { return num_jobs_; }
    uint64_t num_decisions() const override { return num_decisions_; }

    void set_pools(const std::vector<cudaStream_t>& streams, const std::vector<job::FinishedBlockNotifier*>& notifiers) override {
        all_streams_ = streams;
        all_notifiers_ = notifiers;
        free_streams_.clear();
        free_notifiers_.clear();
        for (unsigned i = 0; i < streams.size(); ++i) free_streams_.push_back(i);
        for (unsigned i = 0; i < notifiers.size(); ++i) free_notifiers_.push_back(i);
        job_stream_slot_.clear();
        job_notifier_slot_.clear();
    }

    void handle_new_job(job::Job* job) override {
        if (!job->has_next()) {
            // nothing to run: the client still gets its start and end messages (the reference releases such a
            // job silently, scheduler_full3.cpp:274-278, and its client waits for ever)
            host_->notify_job_starts(job);
            host_->notify_job_ends(job);
            host_->release_job_instance(job);
            return;
        }
        JobId id;
        if (unused_job_id_.empty()) {
            id = (JobId)jobs_.size();
            jobs_.push_back(job);
            job_stream_slot_.push_back(0);
            job_notifier_slot_.push_back(0);
            followers_.emplace_back();
        } else {
            id = unused_job_id_.back();
            unused_job_id_.pop_back();
            jobs_[id] = job;
        }
        job->set_id(id);
        const unsigned next = (unsigned)(job->get_cur_stage() + 1);
        if (!host_->has_job_stage_resource(job, next)) host_->set_job_stage_resource(job, next, 1);
        job->set_stage_lengths_resources(host_->get_job_remaining_rl(job, 0), host_->get_job_stage_lengths(job),
                                         host_->get_job_stage_resources(job));
        job->set_priority(calculate_priority(job));
        job_queue_.push(job);
        ++num_jobs_;
        schedule_job();
    }

    void handle_record(const job::InstrumentInfo& info) override {
        if (info.job_id >= jobs_.size() || jobs_[info.job_id] == nullptr) {
            ++num_stray_records_;
            return;
        }
        if (info.is_start == job::InstrumentInfo::kStart) handle_block_start(info);
        else if (info.is_start == job::InstrumentInfo::kEnd) handle_block_finish(info);
        else handle_mem_finish(info);
    }

  private:
    void handle_block_start(const job::InstrumentInfo& info) {
        job::Job* job = jobs_[info.job_id];
        if (!job->mark_block_start(info.num)) {
            if (job->is_unfit()) {
                job->unset_unfit();
                --num_outstanding_kernels_;
                schedule_job();
            }
        }
    }

    // Common tail of a finished stage: learn its length, re-queue or finish the job.
    void stage_finished(job::Job* job) {
        const double length = host_->now_us() - job->get_stage_start_time_us();
        host_->update_job_stage_length(job, (unsigned)job->get_cur_stage(), length);
        if (job->has_next()) {
            const unsigned next = (unsigned)(job->get_cur_stage() + 1);
            if (!host_->has_job_stage_resource(job, next)) host_->set_job_stage_resource(job, next, 1);
            job->set_priority(calculate_priority(job));
            job_queue_.push(job);
        } else {
            host_->notify_job_ends(job);
            --num_jobs_;
            // the members of its gang end with it (and share its failure, if any)
            for (job::Job* f : followers_[job->get_id()]) {
                if (job->has_error()) f->set_error(job->has_error());
                host_->notify_job_ends(f);
                --num_jobs_;
            }
        }
    }

    void handle_block_finish(const job::InstrumentInfo& info) {
        job::Job* job = jobs_[info.job_id];
        job->mark_block_finish(info.num);
        const bool stage_done = !job->is_running();
        if (stage_done) {
            stage_finished(job);
            if (job->is_unfit()) {   // start records may still be in flight when the last end arrives
                job->unset_unfit();
                --num_outstanding_kernels_;
            }
            free_streams_.push_back(job_stream_slot_[info.job_id]);
            free_notifiers_.push_back(job_notifier_slot_[info.job_id]);
        }
        gpu_resources_.release(job, info.num);
        if (stage_done && !job->has_next()) retire(job);
        schedule_job();
    }

    void handle_mem_finish(const job::InstrumentInfo& info) {
        job::Job* job = jobs_[info.job_id];
        job->unset_running();
        stage_finished(job);
        free_streams_.push_back(job_stream_slot_[info.job_id]);
        if (!job->has_next()) retire(job);
        schedule_job();
    }

    // Fails every stage that has been in flight longer than its limit.  The GPU may still be running it, so
    // nothing of the dispatch is reused: the job id stays unknown to handle_record (late records count as stray),
    // the stream and the notifier do not go back to their pools.
    unsigned check_watchdog(double now_us) override {
        if (cfg_.watchdog_factor <= 0) return 0;
        unsigned failed = 0;
        for (JobId id = 0; id < jobs_.size(); ++id) {
            job::Job* job = jobs_[id];
            if (!job || !job->is_running()) continue;
            const std::vector<double>& lens = host_->get_job_stage_lengths(job);
            const size_t st = (size_t)job->get_cur_stage();
            const double learned = st < lens.size() ? lens[st] : 0.0;
            const double limit = std::max(cfg_.watchdog_factor * learned, cfg_.watchdog_floor_us);
            if (now_us - job->get_stage_start_time_us() <= limit) continue;
            job->set_error(-5 /* PB_ERR_TIMEOUT */);
            const bool was_mem = job->is_mem_stage_in_flight();
            if (!was_mem) gpu_resources_.release(job, job->running_blocks());
            job->unset_running();
            if (job->is_unfit()) { job->unset_unfit(); --num_outstanding_kernels_; }
            host_->notify_job_ends(job);
            --num_jobs_;
            for (job::Job* f : followers_[id]) {
                f->set_error(-5);
                host_->notify_job_ends(f);
                --num_jobs_;
                jobs_[f->get_id()] = nullptr;      // followers never had a dispatch of their own: their ids can be reused
                unused_job_id_.push_back(f->get_id());
                host_->release_job_instance(f);
            }
            followers_[id].clear();
            jobs_[id] = nullptr;                   // quarantined: not pushed to unused_job_id_
            host_->release_job_instance(job);
            ++num_watchdog_;
            ++failed;
        }
        if (failed) schedule_job();
        return failed;
    }

    void retire(job::Job* job) {
        const JobId id = job->get_id();
        for (job::Job* f : followers_[id]) retire(f);
        followers_[id].clear();
        unused_job_id_.push_back(id);
        jobs_[id] = nullptr;
        host_->release_job_instance(job);
    }

    // Takes the queued, not yet started jobs of the leader's type out of the queue as its followers.
    void form_gang(job::Job* leader) {
        std::vector<job::Job*>& fol = followers_[leader->get_id()];
        const unsigned want = std::min(cfg_.max_gang, leader->get_gang_capacity());
        const JobRefId type = leader->get_registered_job_id();
        while (fol.size() + 1 < want) {
            job::Job* f = job_queue_.pop_of_type_if(type, [](const job::Job* j) { return j->get_cur_stage() == -1 && !j->is_mem(); });
            if (!f) break;
            f->set_started();
            fol.push_back(f);
        }
        if (!fol.empty()) {
            leader->apply_gang_size((unsigned)fol.size() + 1);
            ++num_gangs_;
            num_gang_members_ += fol.size() + 1;
        }
    }

    void schedule_job() {
        if (deferred_) { dirty_ = true; return; }
        dispatch_loop();
    }

    void dispatch_loop() {
        if (free_streams_.empty() || job_queue_.empty()) return;
        do {
            job::Job* job = job_queue_.top();
            if (cfg_.sched_sleep > 0) {
                for (volatile unsigned i = 0; i < cfg_.sched_sleep; ++i) {}
            }
            const bool is_mem = job->is_mem();
            if (!is_mem && free_notifiers_.empty()) break;      // cannot happen while every kernel reports each block once
            bool unfit = false;
            if (!is_mem && !gpu_resources_.job_fits(job)) {
                // A stage larger than the whole GPU (a gang's, or with no over-subscription allowed) never fits: with
                // nothing in flight waiting cannot help, so it goes as an over-subscribed stage (the reference would
                // wait for ever, scheduler_full3.cpp:380-392).
                if (num_outstanding_kernels_ >= (int)max_num_outstanding_kernels_ && !gpu_resources_.idle()) break;
                ++num_outstanding_kernels_;
                job->set_unfit();
                unfit = true;
            }
            job_queue_.pop();
            if (cfg_.max_gang > 1 && !is_mem && job->get_cur_stage() == -1 && job->get_gang_capacity() > 1) form_gang(job);
            if (!job->has_started()) job->set_started();

            const unsigned sslot = free_streams_.back();
            free_streams_.pop_back();
            job_stream_slot_[job->get_id()] = sslot;
            job->set_running(all_streams_[sslot], host_->now_us());
            unsigned nslot = 0;
            if (!is_mem) {
                nslot = free_notifiers_.back();
                free_notifiers_.pop_back();
                job_notifier_slot_[job->get_id()] = nslot;
                job->set_finished_block_notifier(all_notifiers_[nslot]);
                gpu_resources_.acquire(job, (int)job->get_cur_num_blocks());
            }
            const std::vector<job::Job*>& gang = followers_[job->get_id()];
            if (job->is_pre_notify()) {
                host_->notify_job_starts(job);
                for (job::Job* f : gang) host_->notify_job_starts(f);
            }
            ++num_decisions_;
            host_->on_dispatch(job, is_mem, unfit, sslot, nslot);

            job::Context::set_gang(gang.data(), (unsigned)gang.size());
            run_stage(job, host_);
            job::Context::set_gang(nullptr, 0);
            if (!job->has_error() && is_mem) host_->after_mem_stage(job);     // may fail too (the marker kernel's launch)
            if (job->has_error()) close_failed_stage(job, is_mem);
            if (free_streams_.empty()) break;
        } while (!job_queue_.empty());
    }

    // Priority = -(remaining length x resource); the stage about to be queued is then
    // taken out of the remainder (scheduler_full3.cpp:454-459).
    static double calculate_priority(job::Job* job) {
        const double rl = job->get_cur_rl();
        job->dec_cur_rl();
        return -rl;
    }

    SchedulerHost* host_;
    SchedulerConfig cfg_;
    JobQueue job_queue_;
    SmResources gpu_resources_;
    std::vector<cudaStream_t> all_streams_;
    std::vector<job::FinishedBlockNotifier*> all_notifiers_;
    std::vector<unsigned> free_streams_, free_notifiers_;
    std::vector<unsigned> job_stream_slot_, job_notifier_slot_;   // by JobId
    std::vector<job::Job*> jobs_;                                 // by JobId
    std::vector<std::vector<job::Job*>> followers_;               // by JobId of the leader: the other members of its gang
    uint64_t num_gangs_ = 0, num_gang_members_ = 0;
    bool deferred_ = false, dirty_ = false;
    uint64_t num_watchdog_ = 0;
    std::vector<JobId> unused_job_id_;
    unsigned num_jobs_ = 0;
    uint64_t num_decisions_ = 0;
    uint64_t num_stray_records_ = 0;
    int num_outstanding_kernels_ = 0;
    unsigned max_num_outstanding_kernels_ = 2;
};

}  // namespace

std::unique_ptr<Scheduler> make_scheduler_full3(const SchedulerConfig& cfg, SchedulerHost* host) {
    return std::unique_ptr<Scheduler>(new SchedulerFull3(cfg, host));
}

}  // namespace server
}  // namespace llis
