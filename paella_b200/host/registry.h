// Job types known to a server: plugin entry point, instance pool and the learned
// per-stage lengths.  Restates the bookkeeping of the reference's RegisteredJob
// (src/server/registered_job.cpp:61-93 instance pool, :112-137 stage-length EWMA
// (old + new) / 2, :139-182 resources and remaining length x resource).
#pragma once

#include <llis/job/job.h>
#include <llis/server/scheduler.h>

#include <functional>
#include <memory>
#include <string>
#include <vector>

namespace llis {
namespace server {

struct JobType {
    JobRefId id = 0;
    std::string path;
    void* dl_handle = nullptr;
    std::function<job::Job*()> make;          // init_job of the plugin (or a fake in replay)
    std::vector<job::Job*> unused;            // LIFO pool of idle instances
    std::vector<job::Job*> all;               // every instance ever made (never destroyed, as in the reference)
    std::vector<double> stage_lengths;
    std::vector<float> stage_resources;
    size_t in_bytes = 0, out_bytes = 0, slot_bytes = 0;

    void update_stage_length(unsigned stage, double len) {
        if (stage_lengths.size() > stage) stage_lengths[stage] = (stage_lengths[stage] + len) / 2;
        else stage_lengths.push_back(len);
    }
    bool has_stage_resource(unsigned stage) const { return stage_resources.size() > stage; }
    void set_stage_resource(unsigned stage, float res) {
        if (stage_resources.size() <= stage) stage_resources.push_back(res);
    }
    double remaining_rl(unsigned from) const {
        double sum = 0;
        for (unsigned i = from; i < stage_lengths.size(); ++i) sum += stage_lengths[i] * (i < stage_resources.size() ? stage_resources[i] : 0.f);
        return sum;
    }
    // Takes an idle instance or makes one; `fresh` tells the caller to run full_init.
    job::Job* take(bool* fresh) {
        if (unused.empty()) {
            job::Job* j = make();
            if (j) all.push_back(j);
            *fresh = true;
            return j;
        }
        job::Job* j = unused.back();
        unused.pop_back();
        *fresh = false;
        return j;
    }
    void give_back(job::Job* j) { unused.push_back(j); }
};

std::unique_ptr<Scheduler> make_scheduler_full3(const SchedulerConfig& cfg, SchedulerHost* host);
std::unique_ptr<Scheduler> make_scheduler_fifo(const SchedulerConfig& cfg, SchedulerHost* host);
std::unique_ptr<Scheduler> make_scheduler_fifo2(const SchedulerConfig& cfg, SchedulerHost* host);

}  // namespace server
}  // namespace llis
