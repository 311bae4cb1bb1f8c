// Scheduler replay: drives the product scheduler with a recorded event trace, fake
// streams/notifiers and table-driven jobs, and returns its decision log.  No GPU involved.
#include <llis/job/context.h>
#include <llis/server/scheduler.h>

#include <cstring>
#include <memory>
#include <vector>

#include "../csrc/pb_common.h"
#include "registry.h"

using llis::job::InstrumentInfo;
using llis::job::Job;

namespace {

// A job whose stages come from a table: follows the adapters' protocol (resources of stage
// k+1 are declared before run_next() of stage k returns; init() leaves stage 0 declared).
class TableJob final : public Job {
  public:
    explicit TableJob(const pb_replay_type* t) : t_(t) {}
    size_t get_input_size() override { return 8; }
    size_t get_output_size() override { return 8; }
    size_t get_param_size() override { return 4; }
    void full_init(void* io) override { init(io); }
    void init(void*) override { next_ = 0; declare(); }
    void run_next() override { ++next_; declare(); }
    bool has_next() const override { return next_ < t_->num_stages; }

  private:
    void declare() {
        if (next_ >= t_->num_stages) return;
        if (t_->stage_is_mem[next_]) set_is_mem(); else unset_is_mem();
        if (t_->stage_pre_notify[next_]) set_pre_notify();
        set_num_blocks(t_->stage_blocks[next_]);
        set_num_threads_per_block(t_->stage_threads[next_]);
        set_smem_size_per_block(t_->stage_smem[next_]);
        set_num_registers_per_thread(t_->stage_regs[next_]);
    }
    const pb_replay_type* t_;
    uint32_t next_ = 0;
};

struct ReplayHost final : public llis::server::SchedulerHost {
    std::vector<std::unique_ptr<llis::server::JobType>> types;
    std::vector<std::unique_ptr<TableJob>> owned;
    double now = 0;
    uint32_t event_index = 0;
    pb_replay_decision* log = nullptr;
    uint32_t max_log = 0, n_log = 0, n_finished = 0;

    llis::server::JobType& type_of(Job* j) { return *types[j->get_registered_job_id()]; }
    double now_us() override { return now; }
    void after_mem_stage(Job*) override {}
    void update_job_stage_length(Job* j, unsigned s, double l) override { type_of(j).update_stage_length(s, l); }
    bool has_job_stage_resource(Job* j, unsigned s) override { return type_of(j).has_stage_resource(s); }
    void set_job_stage_resource(Job* j, unsigned s, float r) override { type_of(j).set_stage_resource(s, r); }
    double get_job_remaining_rl(Job* j, unsigned f) override { return type_of(j).remaining_rl(f); }
    const std::vector<double>& get_job_stage_lengths(Job* j) override { return type_of(j).stage_lengths; }
    const std::vector<float>& get_job_stage_resources(Job* j) override { return type_of(j).stage_resources; }
    void notify_job_starts(Job*) override {}
    void notify_job_ends(Job*) override { ++n_finished; }
    void release_job_instance(Job* j) override { type_of(j).give_back(j); }
    void on_dispatch(Job* j, bool is_mem, bool unfit, unsigned ss, unsigned ns) override {
        if (n_log < max_log) {
            pb_replay_decision& d = log[n_log];
            d.event_index = event_index;
            d.job_id = j->get_id();
            d.type = j->get_registered_job_id();
            d.stage = (uint32_t)j->get_cur_stage();
            d.is_mem = is_mem;
            d.unfit = unfit;
            d.stream_slot = ss;
            d.notifier_slot = is_mem ? 0xFFFFFFFFu : ns;
            d.priority = j->get_priority();
        }
        ++n_log;
    }
};

}  // namespace

extern "C" int pb_sched_replay(const pb_replay_config* cfg, const pb_replay_type* types, uint32_t num_types,
                               const pb_replay_event* events, uint32_t num_events, pb_replay_decision* decisions,
                               uint32_t max_decisions, uint32_t* num_decisions_out, uint32_t* num_finished_out) {
    PB_REQUIRE(cfg && types && events && num_decisions_out, "pb_sched_replay: NULL argument");
    ReplayHost host;
    host.log = decisions;
    host.max_log = decisions ? max_decisions : 0;
    for (uint32_t i = 0; i < num_types; ++i) {
        auto t = std::make_unique<llis::server::JobType>();
        t->id = i;
        const pb_replay_type* rt = &types[i];
        ReplayHost* hp = &host;
        t->make = [rt, hp]() -> Job* {
            hp->owned.push_back(std::make_unique<TableJob>(rt));
            return hp->owned.back().get();
        };
        host.types.push_back(std::move(t));
    }
    llis::server::SchedulerConfig sc;
    sc.num_streams = cfg->num_streams;
    sc.extra_kernels = cfg->extra_kernels;
    sc.unfairness_threshold = cfg->unfairness_threshold;
    sc.totals.regs = cfg->total_regs;
    sc.totals.smem = cfg->total_smem;
    sc.totals.threads = cfg->total_threads;
    sc.totals.blocks = cfg->total_blocks;
    sc.totals.tmem_cols = 1 << 30;
    auto sched = llis::server::Scheduler::create("full3", sc, &host);
    std::vector<cudaStream_t> streams(cfg->num_streams);
    std::vector<llis::job::FinishedBlockNotifier*> nfs(cfg->num_streams);
    for (uint32_t i = 0; i < cfg->num_streams; ++i) {
        streams[i] = (cudaStream_t)(uintptr_t)(i + 1);
        nfs[i] = (llis::job::FinishedBlockNotifier*)(uintptr_t)(i + 1);
    }
    sched->set_pools(streams, nfs);
    for (uint32_t e = 0; e < num_events; ++e) {
        const pb_replay_event& ev = events[e];
        host.now = ev.time_us;
        host.event_index = e;
        if (ev.kind == 0) {
            PB_REQUIRE(ev.a < num_types, "replay event %u: unknown job type %u", e, ev.a);
            llis::server::JobType& t = *host.types[ev.a];
            bool fresh = false;
            Job* j = t.take(&fresh);
            if (fresh) { j->set_client_details(0, t.id); j->full_init(nullptr); }
            else { j->reset_internal(); j->init(nullptr); }
            sched->handle_new_job(j);
        } else {
            InstrumentInfo info{};
            info.is_start = ev.kind == 1 ? InstrumentInfo::kStart : (ev.kind == 2 ? InstrumentInfo::kEnd : InstrumentInfo::kMemDone);
            info.job_id = ev.a;
            info.num = (uint8_t)ev.b;
            sched->handle_record(info);
        }
    }
    *num_decisions_out = host.n_log;
    if (num_finished_out) *num_finished_out = host.n_finished;
    return PB_OK;
}
