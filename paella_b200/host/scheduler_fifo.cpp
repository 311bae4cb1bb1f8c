// Ablation schedulers.
//  "fifo"  : job by job - every stage of the head job is enqueued at once on one stream and
//            the job's end is detected by counting block-end and copy-done records
//            (reference: src/server/scheduler_fifo.cpp:83-124,197-255).  With one stream this
//            is the single-stream baseline, with many the job-by-job multi-stream one.
//  "fifo2" : kernel by kernel in arrival order, no occupancy check
//            (reference: include/llis/server/scheduler_fifo2.h:33-38,62 - a min-heap on the
//            job's unique id; src/server/scheduler_fifo2.cpp).
#include <llis/server/scheduler.h>

#include <algorithm>
#include <deque>
#include <queue>

#include "registry.h"

namespace llis {
namespace server {

namespace {

using job::InstrumentInfo;
using job::Job;

class PoolsBase : public Scheduler {
  public:
    PoolsBase(const SchedulerConfig& cfg, SchedulerHost* host) : host_(host), cfg_(cfg) {}
    unsigned num_jobs() const override { return num_jobs_; }
    uint64_t num_decisions() const override { return num_decisions_; }
    void set_pools(const std::vector<cudaStream_t>& streams, const std::vector<job::FinishedBlockNotifier*>& notifiers) override {
        all_streams_ = streams;
        all_notifiers_ = notifiers;
        free_streams_.clear();
        free_notifiers_.clear();
        for (unsigned i = 0; i < streams.size(); ++i) free_streams_.push_back(i);
        for (unsigned i = 0; i < notifiers.size(); ++i) free_notifiers_.push_back(i);
    }

  protected:
    JobId admit(Job* job) {
        JobId id;
        if (unused_job_id_.empty()) {
            id = (JobId)jobs_.size();
            jobs_.push_back(job);
            stream_slot_.push_back(0);
            notifier_slot_.push_back(0);
            remaining_.push_back(0);
            pre_notify_left_.push_back(0);
            pre_notify_sent_.push_back(false);
        } else {
            id = unused_job_id_.back();
            unused_job_id_.pop_back();
            jobs_[id] = job;
            remaining_[id] = 0;
            pre_notify_left_[id] = 0;
            pre_notify_sent_[id] = false;
        }
        job->set_id(id);
        ++num_jobs_;
        return id;
    }
    void retire(Job* job) {
        const JobId id = job->get_id();
        unused_job_id_.push_back(id);
        jobs_[id] = nullptr;
        host_->release_job_instance(job);
        --num_jobs_;
    }
    Job* lookup(const InstrumentInfo& info) { return info.job_id < jobs_.size() ? jobs_[info.job_id] : nullptr; }

    SchedulerHost* host_;
    SchedulerConfig cfg_;
    std::vector<cudaStream_t> all_streams_;
    std::vector<job::FinishedBlockNotifier*> all_notifiers_;
    std::vector<unsigned> free_streams_, free_notifiers_;
    std::vector<unsigned> stream_slot_, notifier_slot_;
    std::vector<Job*> jobs_;
    std::vector<JobId> unused_job_id_;
    std::vector<long> remaining_, pre_notify_left_;
    std::vector<bool> pre_notify_sent_;
    unsigned num_jobs_ = 0;
    uint64_t num_decisions_ = 0;
};

class SchedulerFifo final : public PoolsBase {
  public:
    using PoolsBase::PoolsBase;
    const char* name() const override { return "fifo"; }

    void handle_new_job(Job* job) override {
        if (!job->has_next()) { host_->notify_job_starts(job); host_->notify_job_ends(job); host_->release_job_instance(job); return; }
        admit(job);
        queue_.push_back(job);
        schedule_job();
    }

    void handle_record(const InstrumentInfo& info) override {
        Job* job = lookup(info);
        if (!job || info.is_start == InstrumentInfo::kStart) return;
        const JobId id = info.job_id;
        const long n = info.is_start == InstrumentInfo::kEnd ? (long)info.num : 1;
        remaining_[id] -= n;
        pre_notify_left_[id] -= n;
        if (pre_notify_left_[id] <= 0 && !pre_notify_sent_[id]) {
            host_->notify_job_starts(job);
            pre_notify_sent_[id] = true;
        }
        if (remaining_[id] == 0) {
            host_->notify_job_ends(job);
            free_streams_.push_back(stream_slot_[id]);
            free_notifiers_.push_back(notifier_slot_[id]);
            retire(job);
        }
        schedule_job();
    }

  private:
    void schedule_job() {
        while (!free_streams_.empty() && !queue_.empty()) {
            Job* job = queue_.front();
            queue_.pop_front();
            const JobId id = job->get_id();
            job->set_started();
            const unsigned ss = free_streams_.back();
            free_streams_.pop_back();
            const unsigned ns = free_notifiers_.back();
            free_notifiers_.pop_back();
            stream_slot_[id] = ss;
            notifier_slot_[id] = ns;
            bool saw_pre_notify = false;
            while (job->has_next()) {
                const bool is_mem = job->is_mem();
                const long n = is_mem ? 1 : (long)job->get_num_blocks();
                remaining_[id] += n;
                if (!saw_pre_notify) {
                    pre_notify_left_[id] += n;
                    if (job->is_pre_notify()) saw_pre_notify = true;
                }
                job->set_running(all_streams_[ss], host_->now_us());
                job->set_finished_block_notifier(all_notifiers_[ns]);
                ++num_decisions_;
                host_->on_dispatch(job, is_mem, false, ss, ns);
                run_stage(job, host_);
                if (!job->has_error() && is_mem) host_->after_mem_stage(job);
                if (job->has_error()) close_failed_stage(job, is_mem);
            }
        }
    }
    std::deque<Job*> queue_;
};

class SchedulerFifo2 final : public PoolsBase {
  public:
    using PoolsBase::PoolsBase;
    const char* name() const override { return "fifo2"; }

    void handle_new_job(Job* job) override {
        if (!job->has_next()) { host_->notify_job_starts(job); host_->notify_job_ends(job); host_->release_job_instance(job); return; }
        admit(job);
        heap_.push(job);
        schedule_job();
    }

    void handle_record(const InstrumentInfo& info) override {
        Job* job = lookup(info);
        if (!job || info.is_start == InstrumentInfo::kStart) return;
        if (info.is_start == InstrumentInfo::kEnd) {
            job->mark_block_finish(info.num);
            if (job->is_running()) return;
            free_notifiers_.push_back(notifier_slot_[info.job_id]);
        } else {
            job->unset_running();
        }
        free_streams_.push_back(stream_slot_[info.job_id]);
        if (job->has_next()) {
            heap_.push(job);
        } else {
            host_->notify_job_ends(job);
            retire(job);
        }
        schedule_job();
    }

  private:
    struct Later {
        bool operator()(const Job* a, const Job* b) const { return a->get_unique_id() > b->get_unique_id(); }
    };
    void schedule_job() {
        while (!free_streams_.empty() && !heap_.empty()) {
            Job* job = heap_.top();
            heap_.pop();
            const JobId id = job->get_id();
            const bool is_mem = job->is_mem();
            if (!job->has_started()) job->set_started();
            const unsigned ss = free_streams_.back();
            free_streams_.pop_back();
            stream_slot_[id] = ss;
            job->set_running(all_streams_[ss], host_->now_us());
            unsigned ns = 0;
            if (!is_mem) {
                ns = free_notifiers_.back();
                free_notifiers_.pop_back();
                notifier_slot_[id] = ns;
                job->set_finished_block_notifier(all_notifiers_[ns]);
            }
            if (job->is_pre_notify()) host_->notify_job_starts(job);
            ++num_decisions_;
            host_->on_dispatch(job, is_mem, false, ss, ns);
            run_stage(job, host_);
            if (!job->has_error() && is_mem) host_->after_mem_stage(job);
            if (job->has_error()) close_failed_stage(job, is_mem);
        }
    }
    std::priority_queue<Job*, std::vector<Job*>, Later> heap_;
};

}  // namespace

std::unique_ptr<Scheduler> make_scheduler_fifo(const SchedulerConfig& cfg, SchedulerHost* host) {
    return std::unique_ptr<Scheduler>(new SchedulerFifo(cfg, host));
}
std::unique_ptr<Scheduler> make_scheduler_fifo2(const SchedulerConfig& cfg, SchedulerHost* host) {
    return std::unique_ptr<Scheduler>(new SchedulerFifo2(cfg, host));
}

}  // namespace server
}  // namespace llis
