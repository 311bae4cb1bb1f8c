#include "server.h"

#include <llis/ipc/defs.h>

#include <cuda_runtime.h>
#include <dlfcn.h>
#include <llis/job/context.h>

#include <cstring>

#include "../csrc/pb_common.h"

using llis::job::Context;
using llis::job::InstrumentInfo;
using llis::job::Job;

pb_server::~pb_server() {
    cudaSetDevice(device);
    cudaDeviceSynchronize();
    if (!profile_prefix.empty()) profiler_save(profile_prefix);
    // plugins that can give back what their instances of this server hold on the device
    for (auto& t : types) {
        if (!t->dl_handle) continue;
        typedef void (*release_t)(void*);
        if (release_t fn = (release_t)dlsym(t->dl_handle, "pb_plugin_release")) fn(this);
    }
    for (cudaStream_t s : streams) cudaStreamDestroy(s);
    if (notifiers_raw) llis::job::FinishedBlockNotifier::free_array(notifiers_raw);
    // Plugin instances are never destroyed (their class has no virtual destructor in the
    // plugin ABI); device memory they hold goes away with the context.
}

void pb_server::finish_job_events(Job* job) {
    auto it = events_cur.find(job);
    if (it == events_cur.end()) return;
    it->second.emplace_back((int)kJobFinished, now_us());
    events_all.push_back(std::move(it->second));
    events_cur.erase(it);
}

int pb_server::profiler_cmd(uint32_t msg_type, const char* path) {
    switch ((llis::ProfilerMsgType)msg_type) {
        case llis::ProfilerMsgType::SET_RECORD_JOB_EVENTS: job_events_flag = true; return PB_OK;
        case llis::ProfilerMsgType::UNSET_RECORD_JOB_EVENTS: job_events_flag = false; return PB_OK;
        case llis::ProfilerMsgType::SET_RECORD_RUN_NEXT_TIMES: run_next_times_flag = true; return PB_OK;
        case llis::ProfilerMsgType::UNSET_RECORD_RUN_NEXT_TIMES: run_next_times_flag = false; return PB_OK;
        case llis::ProfilerMsgType::SAVE:
            PB_REQUIRE(path != nullptr && path[0], "profiler SAVE needs a path prefix");
            return profiler_save(path);
        default:
            // kernel info, per-block execution times, block placement and resource events: accepted, nothing recorded
            return msg_type <= (uint32_t)llis::ProfilerMsgType::SAVE ? PB_OK : PB_ERR_INVALID;
    }
}

// Files and line formats of src/server/profiler.cpp:101-121: "<prefix>_run_next_times.txt" with
// "start_us end_us duration_us num_blocks", "<prefix>_job_events.txt" with one line per finished job.
int pb_server::profiler_save(const std::string& path) {
    FILE* fp = fopen((path + "_run_next_times.txt").c_str(), "w");
    if (!fp) { pb::set_error("cannot write %s_run_next_times.txt", path.c_str()); return PB_ERR_IO; }
    for (const RunNext& r : run_next_times) fprintf(fp, "%f %f %f %u\n", r.start_us, r.end_us, r.end_us - r.start_us, r.num_blocks);
    fclose(fp);
    fp = fopen((path + "_job_events.txt").c_str(), "w");
    if (!fp) { pb::set_error("cannot write %s_job_events.txt", path.c_str()); return PB_ERR_IO; }
    for (const auto& job : events_all) {
        for (const auto& ev : job) fprintf(fp, "%u %f ", (unsigned)ev.first, ev.second);
        fprintf(fp, "\n");
    }
    fclose(fp);
    return PB_OK;
}

int pb_server::init(const pb_server_config& c) {
    cfg = c;
    device = c.device;
    if (const char* pp = getenv("PB_PROFILE_PREFIX")) {
        if (pp[0]) { profile_prefix = pp; job_events_flag = run_next_times_flag = true; }
    }
    PB_CUDA(cudaSetDevice(device));
    Context::set_device(device);
    llis::server::SchedulerConfig sc;
    sc.num_streams = c.num_streams ? c.num_streams : 500;
    sc.extra_kernels = c.extra_kernels;
    sc.unfairness_threshold = c.unfairness_threshold;
    sc.sched_sleep = c.sched_sleep;
    sc.watchdog_factor = c.watchdog_factor;
    if (c.watchdog_floor_ms > 0) sc.watchdog_floor_us = 1000.0 * c.watchdog_floor_ms;
    sc.max_gang = c.max_gang > 1 ? (c.max_gang < PB_MAX_GANG ? c.max_gang : PB_MAX_GANG) : 1;
    int rc = llis::server::SmResources::query_device(device, &sc.totals);
    if (rc != PB_OK) return rc;
    try {
        channel.connect(c.ring_capacity ? c.ring_capacity : (1ull << 20), device);
        notifiers_raw = llis::job::FinishedBlockNotifier::create_array(sc.num_streams, &channel);
    } catch (const std::exception& e) {
        pb::set_error("%s", e.what());
        return PB_ERR_CUDA;
    }
    Context::set_gpu2sched_channel(&channel);
    streams.resize(sc.num_streams);
    std::vector<llis::job::FinishedBlockNotifier*> nfs(sc.num_streams);
    for (unsigned i = 0; i < sc.num_streams; ++i) {
        PB_CUDA(cudaStreamCreateWithFlags(&streams[i], cudaStreamNonBlocking));
        nfs[i] = notifiers_raw + i;
    }
    scheduler = llis::server::Scheduler::create(c.scheduler ? c.scheduler : "full3", sc, this);
    PB_REQUIRE(scheduler != nullptr, "unknown scheduler '%s'", c.scheduler ? c.scheduler : "");
    scheduler->set_pools(streams, nfs);
    scheduler->set_deferred(c.deferred_schedule != 0 || sc.max_gang > 1);
    return PB_OK;
}

int pb_server::register_job(const char* path, uint32_t* id_out) {
    void* h = dlopen(path, RTLD_LAZY | RTLD_GLOBAL);
    if (!h) { pb::set_error("dlopen(%s): %s", path, dlerror()); return PB_ERR_IO; }
    typedef Job* (*init_job_t)();
    init_job_t fn = (init_job_t)dlsym(h, "init_job");
    if (!fn) { pb::set_error("%s exports no init_job", path); return PB_ERR_IO; }
    auto t = std::make_unique<llis::server::JobType>();
    t->id = (llis::JobRefId)types.size();
    t->path = path;
    t->dl_handle = h;
    t->make = [fn]() { return fn(); };
    Job* probe = fn();
    PB_REQUIRE(probe != nullptr, "%s: init_job returned NULL", path);
    t->in_bytes = probe->get_input_size();
    t->out_bytes = probe->get_output_size();
    t->slot_bytes = probe->get_pinned_mem_size();
    *id_out = t->id;
    types.push_back(std::move(t));
    return PB_OK;
}

int pb_server::launch(uint32_t job_ref_id, void* io_ptr, uint64_t cookie, llis::ClientId client_id) {
    PB_REQUIRE(job_ref_id < types.size(), "launch: unknown job type %u", job_ref_id);
    llis::server::JobType& t = *types[job_ref_id];
    bool fresh = false;
    Job* job = t.take(&fresh);
    PB_REQUIRE(job != nullptr, "launch: plugin could not create an instance");
    Context::set_device(device);
    Context::set_device_resident(cfg.device_resident != 0);
    Context::set_max_gang(cfg.max_gang > 1 ? cfg.max_gang : 1);
    Context::set_owner(this);
    job->set_remote_ptr((void*)(uintptr_t)cookie);
    if (fresh) {
        job->set_client_details(client_id, t.id);
        Context::set_current_job(job);
        job->full_init(io_ptr);
    } else {
        job->reset_internal();
        Context::set_current_job(job);
        job->init(io_ptr);
    }
    if (job->has_error()) {
        pb::set_error("job type %u failed to initialise: %s", job_ref_id, pb_last_error());
        t.give_back(job);
        return job->has_error();
    }
    if (job_events_flag) record_job_event(job, kJobSubmitted, now_us());
    scheduler->handle_new_job(job);
    return PB_OK;
}

void pb_server::after_mem_stage(Job* job) {
    const int rc = pb_launch_mem_done(job->get_cuda_stream(), job->get_id(), notifiers_raw);
    if (rc != PB_OK) job->set_error(rc);
}

int pb_server::step(int max_records) {
    uint64_t recs[64];
    int handled = 0;
    std::vector<InstrumentInfo> made_up;
    if (cfg.watchdog_factor > 0) {
        const double t = now_us();
        if (t - last_watchdog_us > 1000.0) { last_watchdog_us = t; num_watchdog += scheduler->check_watchdog(t); }
    }
    scheduler->flush();          // requests admitted since the last step
    while (scheduler->take_synthetic(&made_up)) {
        for (const InstrumentInfo& r : made_up) scheduler->handle_record(r);
        scheduler->flush();
    }
    while (handled < max_records) {
        const int want = max_records - handled < 64 ? max_records - handled : 64;
        const int n = pb_ring_poll(channel.handle(), recs, want);
        if (n < 0) { last_error = n; return n; }
        for (int i = 0; i < n; ++i) scheduler->handle_record(InstrumentInfo::unpack(recs[i]));
        scheduler->flush();
        handled += n;
        num_records += (uint64_t)n;
        if (n < want) break;
    }
    return handled;
}

namespace llis {
namespace server {

int SmResources::query_device(int device, SmTotals* out) {
    cudaDeviceProp prop;
    PB_CUDA(cudaGetDeviceProperties(&prop, device));
    out->num_sms = prop.multiProcessorCount;
    out->regs = prop.regsPerMultiprocessor * prop.multiProcessorCount;
    out->smem = (int)prop.sharedMemPerMultiprocessor * prop.multiProcessorCount;
    out->threads = prop.maxThreadsPerMultiProcessor * prop.multiProcessorCount;
    out->blocks = prop.maxBlocksPerMultiProcessor * prop.multiProcessorCount;
    out->tmem_cols = prop.major >= 10 ? 512 * prop.multiProcessorCount : 0;
    return PB_OK;
}

double SmResources::occupancy() const {
    const double a = 1. - (double)left_.threads / (double)max_.threads;
    const double b = 1. - (double)left_.smem / (double)max_.smem;
    const double c = 1. - (double)left_.regs / (double)max_.regs;
    return a > b ? (a > c ? a : c) : (b > c ? b : c);
}

}  // namespace server
}  // namespace llis

extern "C" {

void pb_server_config_default(pb_server_config* cfg) {
    memset(cfg, 0, sizeof(*cfg));
    cfg->num_streams = 500;
    cfg->extra_kernels = 2;
    cfg->unfairness_threshold = 1e6f;
    cfg->ring_capacity = 1ull << 20;
    cfg->scheduler = "full3";
    cfg->max_gang = 1;
}

int pb_server_create(const pb_server_config* cfg, pb_server** out) {
    PB_REQUIRE(cfg && out, "pb_server_create: NULL argument");
    pb_server* s = new pb_server();
    const int rc = s->init(*cfg);
    if (rc != PB_OK) { delete s; return rc; }
    *out = s;
    return PB_OK;
}

void pb_server_destroy(pb_server* s) { delete s; }

int pb_server_register_job(pb_server* s, const char* plugin_path, uint32_t* id_out) {
    PB_REQUIRE(s && plugin_path && id_out, "pb_server_register_job: NULL argument");
    return s->register_job(plugin_path, id_out);
}

int pb_server_job_io_bytes(pb_server* s, uint32_t id, size_t* in_bytes, size_t* out_bytes, size_t* slot_bytes) {
    PB_REQUIRE(s && id < s->types.size(), "pb_server_job_io_bytes: unknown job type");
    if (in_bytes) *in_bytes = s->types[id]->in_bytes;
    if (out_bytes) *out_bytes = s->types[id]->out_bytes;
    if (slot_bytes) *slot_bytes = s->types[id]->slot_bytes;
    return PB_OK;
}

int pb_server_launch(pb_server* s, uint32_t id, void* io_ptr, uint64_t cookie) {
    PB_REQUIRE(s && io_ptr, "pb_server_launch: NULL argument");
    return s->launch(id, io_ptr, cookie);
}

int pb_server_step(pb_server* s, int max_records) { return s ? s->step(max_records) : PB_ERR_INVALID; }

int pb_server_poll_done(pb_server* s, uint64_t* cookies, int32_t* errors, int max) {
    if (!s) return PB_ERR_INVALID;
    int n = 0;
    while (n < max && n < (int)s->done.size()) {
        cookies[n] = s->done[n].cookie;
        if (errors) errors[n] = s->done[n].error;
        ++n;
    }
    s->done.erase(s->done.begin(), s->done.begin() + n);
    return n;
}

uint64_t pb_server_num_decisions(const pb_server* s) { return s ? s->scheduler->num_decisions() : 0; }
uint32_t pb_server_jobs_in_flight(const pb_server* s) { return s ? s->scheduler->num_jobs() : 0; }

int pb_server_profiler_cmd(pb_server* s, uint32_t cmd, const char* path) {
    PB_REQUIRE(s != nullptr, "pb_server_profiler_cmd: NULL server");
    return s->profiler_cmd(cmd, path);
}

}  // extern "C"
