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
    // gang_capacity > 1: the job can lead a gang; a gang of n declares n times the blocks of one job.
    // stage_fails (may be NULL): run_next() of a marked stage enqueues nothing and raises the error flag.
    TableJob(const pb_replay_type* t, unsigned gang_capacity = 1, const uint8_t* stage_fails = nullptr)
        : t_(t), cap_(gang_capacity < 1 ? 1 : gang_capacity), fails_(stage_fails), row_(cap_) {}
    size_t get_input_size() override { return 8; }
    size_t get_output_size() override { return 8; }
    size_t get_param_size() override { return 4; }
    void full_init(void* io) override { init(io); }
    void init(void*) override { next_ = 0; gang_n_ = 1; declare(); }
    void run_next() override {
        unsigned nf = 0;
        llis::job::Context::get_gang(&nf);
        gang_n_ = 1 + nf;
        if (fails_ && fails_[next_]) set_error(PB_ERR_CUDA);
        ++next_;
        declare();
    }
    bool has_next() const override { return next_ < t_->num_stages; }
    unsigned gang_size() const { return gang_n_; }

  private:
    void declare() {
        if (next_ >= t_->num_stages) return;
        if (t_->stage_is_mem[next_]) set_is_mem(); else unset_is_mem();
        if (t_->stage_pre_notify[next_]) set_pre_notify();
        for (unsigned n = 1; n <= cap_; ++n) {
            llis::job::StageDecl& d = row_[n - 1];
            d.num_blocks = t_->stage_blocks[next_] * n;
            d.num_threads_per_block = t_->stage_threads[next_];
            d.smem_size_per_block = t_->stage_smem[next_];
            d.num_registers_per_thread = t_->stage_regs[next_];
        }
        set_next_stage(row_[gang_n_ - 1]);
        set_gang_decls(cap_ > 1 && !t_->stage_is_mem[next_] ? row_.data() : nullptr, cap_);
    }
    const pb_replay_type* t_;
    unsigned cap_;
    const uint8_t* fails_;
    std::vector<llis::job::StageDecl> row_;
    unsigned gang_n_ = 1;
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


// ---- interactive simulation ---------------------------------------------------------------------
// The same scheduler object, fake pools and table-driven jobs, driven call by call: the caller plays the
// GPU (it turns the dispatches it is told about into start / end / copy-done records, or withholds them)
// and the clients.  Used by the CPU tests of what a recorded trace cannot express: gangs, deferred
// dispatch, failing plugins and the stage watchdog.
struct pb_sched_sim final : public llis::server::SchedulerHost {
    std::vector<std::unique_ptr<llis::server::JobType>> types;
    std::vector<std::unique_ptr<TableJob>> owned;
    std::unique_ptr<llis::server::Scheduler> sched;
    std::vector<pb_sim_decision> decisions;
    std::vector<std::pair<uint64_t, int32_t>> finished;
    double now = 0;
    unsigned gang_capacity = 1;
    std::vector<const uint8_t*> fails;

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
    void notify_job_ends(Job* j) override { finished.emplace_back((uint64_t)(uintptr_t)j->get_remote_ptr(), (int32_t)j->has_error()); }
    void release_job_instance(Job* j) override { type_of(j).give_back(j); }
    void on_dispatch(Job* j, bool is_mem, bool unfit, unsigned, unsigned) override {
        pb_sim_decision d;
        d.job_id = j->get_id();
        d.type = j->get_registered_job_id();
        d.stage = (uint32_t)j->get_cur_stage();
        d.is_mem = is_mem;
        d.unfit = unfit;
        d.num_blocks = j->get_cur_num_blocks();
        unsigned nf = 0;
        llis::job::Context::get_gang(&nf);
        d.gang_size = 1;                       // filled in after run_next (the gang is listed only around it)
        d.failed = 0;
        d.cookie = (uint64_t)(uintptr_t)j->get_remote_ptr();
        decisions.push_back(d);
    }
    void on_stage_submitted(Job* j, double, double) override {
        if (decisions.empty()) return;
        decisions.back().gang_size = static_cast<TableJob*>(j)->gang_size();
        decisions.back().failed = j->has_error() ? 1u : 0u;      // nothing was enqueued: the GPU will send no record
    }
    void drain_synthetic() {
        std::vector<InstrumentInfo> made_up;
        while (sched->take_synthetic(&made_up))
            for (const InstrumentInfo& r : made_up) sched->handle_record(r);
    }
};

extern "C" {

int pb_sched_sim_create(const pb_sim_config* cfg, const pb_replay_type* types, uint32_t num_types, const uint8_t* const* stage_fails,
                        pb_sched_sim** out) {
    PB_REQUIRE(cfg && types && out && num_types >= 1, "pb_sched_sim_create: NULL argument");
    pb_sched_sim* sim = new pb_sched_sim();
    sim->gang_capacity = cfg->gang_capacity ? cfg->gang_capacity : 1;
    for (uint32_t i = 0; i < num_types; ++i) {
        auto t = std::make_unique<llis::server::JobType>();
        t->id = i;
        const pb_replay_type* rt = &types[i];
        const uint8_t* f = stage_fails ? stage_fails[i] : nullptr;
        t->make = [rt, f, sim]() -> Job* {
            sim->owned.push_back(std::make_unique<TableJob>(rt, sim->gang_capacity, f));
            return sim->owned.back().get();
        };
        sim->types.push_back(std::move(t));
    }
    llis::server::SchedulerConfig sc;
    sc.num_streams = cfg->base.num_streams;
    sc.extra_kernels = cfg->base.extra_kernels;
    sc.unfairness_threshold = cfg->base.unfairness_threshold;
    sc.totals.regs = cfg->base.total_regs;
    sc.totals.smem = cfg->base.total_smem;
    sc.totals.threads = cfg->base.total_threads;
    sc.totals.blocks = cfg->base.total_blocks;
    sc.totals.tmem_cols = 1 << 30;
    sc.max_gang = cfg->max_gang ? cfg->max_gang : 1;
    sc.watchdog_factor = cfg->watchdog_factor;
    if (cfg->watchdog_floor_us > 0) sc.watchdog_floor_us = cfg->watchdog_floor_us;
    sim->sched = llis::server::Scheduler::create(cfg->scheduler ? cfg->scheduler : "full3", sc, sim);
    if (!sim->sched) { delete sim; pb::set_error("pb_sched_sim_create: unknown scheduler"); return PB_ERR_INVALID; }
    std::vector<cudaStream_t> streams(sc.num_streams);
    std::vector<llis::job::FinishedBlockNotifier*> nfs(sc.num_streams);
    for (uint32_t i = 0; i < sc.num_streams; ++i) {
        streams[i] = (cudaStream_t)(uintptr_t)(i + 1);
        nfs[i] = (llis::job::FinishedBlockNotifier*)(uintptr_t)(i + 1);
    }
    sim->sched->set_pools(streams, nfs);
    sim->sched->set_deferred(cfg->deferred != 0 || sc.max_gang > 1);
    *out = sim;
    return PB_OK;
}

void pb_sched_sim_destroy(pb_sched_sim* sim) { delete sim; }

int pb_sched_sim_new_job(pb_sched_sim* sim, uint32_t type, double now_us, uint64_t cookie) {
    PB_REQUIRE(sim && type < sim->types.size(), "pb_sched_sim_new_job: unknown job type %u", type);
    sim->now = now_us;
    llis::server::JobType& t = *sim->types[type];
    bool fresh = false;
    Job* j = t.take(&fresh);
    j->set_remote_ptr((void*)(uintptr_t)cookie);
    if (fresh) { j->set_client_details(0, t.id); j->full_init(nullptr); }
    else { j->reset_internal(); j->init(nullptr); }
    sim->sched->handle_new_job(j);
    sim->drain_synthetic();
    return PB_OK;
}

int pb_sched_sim_record(pb_sched_sim* sim, uint32_t kind, uint32_t job_id, uint32_t num, double now_us) {
    PB_REQUIRE(sim && kind >= 1 && kind <= 3, "pb_sched_sim_record: kind %u outside 1..3", kind);
    sim->now = now_us;
    InstrumentInfo info{};
    info.is_start = kind == 1 ? InstrumentInfo::kStart : (kind == 2 ? InstrumentInfo::kEnd : InstrumentInfo::kMemDone);
    info.job_id = job_id;
    info.num = (uint8_t)num;
    sim->sched->handle_record(info);
    sim->drain_synthetic();
    return PB_OK;
}

int pb_sched_sim_flush(pb_sched_sim* sim, double now_us) {
    PB_REQUIRE(sim != nullptr, "pb_sched_sim_flush: NULL simulation");
    sim->now = now_us;
    sim->sched->flush();
    sim->drain_synthetic();
    sim->sched->flush();
    const unsigned failed = sim->sched->check_watchdog(now_us);
    sim->sched->flush();
    return (int)failed;
}

int pb_sched_sim_take_decisions(pb_sched_sim* sim, pb_sim_decision* out, int max) {
    if (!sim || !out) return PB_ERR_INVALID;
    int n = 0;
    while (n < max && n < (int)sim->decisions.size()) { out[n] = sim->decisions[(size_t)n]; ++n; }
    sim->decisions.erase(sim->decisions.begin(), sim->decisions.begin() + n);
    return n;
}

int pb_sched_sim_take_finished(pb_sched_sim* sim, uint64_t* cookies, int32_t* errors, int max) {
    if (!sim || !cookies) return PB_ERR_INVALID;
    int n = 0;
    while (n < max && n < (int)sim->finished.size()) {
        cookies[n] = sim->finished[(size_t)n].first;
        if (errors) errors[n] = sim->finished[(size_t)n].second;
        ++n;
    }
    sim->finished.erase(sim->finished.begin(), sim->finished.begin() + n);
    return n;
}

uint32_t pb_sched_sim_jobs_in_flight(const pb_sched_sim* sim) { return sim ? sim->sched->num_jobs() : 0; }

}  // extern "C"
