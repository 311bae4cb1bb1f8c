// Load generator and request router over one server per GPU.
//
// Workload semantics are those of the reference's load generator (app/client.cpp):
// job type = lower_bound over cumulative proportions of a uniform float (:161-165),
// inter-arrival times exponential or lognormal with mu = ln(mean) - sigma^2/2 (:128-136),
// std::mt19937(seed), a total outstanding cap (:151-154) and per-type instance caps with
// late launch of "due" jobs (:167-175), latency = completion - SCHEDULED arrival (:74,177),
// one warm-up launch per instance before timing (:426-446), percentiles sorted[n*q]
// (:192-212).
//
// Scale-out: the path has no cross-GPU exchange, so the router deals requests of one global
// arrival stream round-robin to independent per-GPU replicas (server + pools + weights); each
// replica is driven by one host thread that both submits its due requests and runs the
// server's poll/dispatch loop, so no queue or lock sits between "client" and scheduler.
#include <cuda_runtime.h>
#include <llis/job/context.h>
#include <pthread.h>
#include <sched.h>

#include <algorithm>
#include <atomic>
#include <chrono>
#include <cmath>
#include <cstring>
#include <deque>
#include <random>
#include <thread>
#include <vector>

#include "../csrc/pb_common.h"
#include "server.h"

namespace {

using Clock = std::chrono::steady_clock;

double us_since(Clock::time_point t0) { return std::chrono::duration<double, std::micro>(Clock::now() - t0).count(); }

struct Request {
    double arrival_us;   // scheduled arrival relative to the common start
    int type;
    bool measured;
};

struct Slot {
    void* io = nullptr;
    int type = 0;
    bool measured = false;      // a measured request has completed in this slot
};

struct GpuResult {
    std::vector<double> lat[PB_MAX_JOB_TYPES];
    double first_arrival_us = 0, last_done_us = 0;
    double event_ms = 0;   // CUDA-event time around the measured phase (device clock)
    uint64_t measured = 0, kernels = 0, records = 0, decisions = 0, h2d = 0, d2h = 0;
    double host_launch_us = 0, host_busy_us = 0, host_idle_us = 0;
    int errors = 0;
    uint32_t samples = 0;
    uint64_t sample_bytes = 0;
    int rc = PB_OK;
    char err[256] = "";
};

pb_latency_stats stats_of(std::vector<double>& v) {
    pb_latency_stats s;
    memset(&s, 0, sizeof(s));
    s.count = v.size();
    if (v.empty()) return s;
    std::sort(v.begin(), v.end());
    double mean = 0, sq = 0;
    for (double x : v) { mean += x / (double)v.size(); sq += x * x / (double)v.size(); }
    s.mean_us = mean;
    s.sd_us = v.size() > 1 ? std::sqrt(std::max(0.0, (sq - mean * mean) * ((double)v.size() / ((double)v.size() - 1)))) : 0;
    s.p50_us = v[v.size() / 2];
    s.p90_us = v[(size_t)(v.size() * 0.90)];
    s.p95_us = v[(size_t)(v.size() * 0.95)];
    s.p99_us = v[(size_t)(v.size() * 0.99)];
    s.max_us = v.back();
    return s;
}

// The router: one global, seeded arrival stream (warm-up requests, then measured ones; each phase
// starts at t = 0) dealt round-robin to the replicas.  Pure host code.
std::vector<std::vector<Request>> plan_requests(const pb_loadgen_config* cfg) {
    const int G = cfg->num_gpus;
    std::vector<float> cum(cfg->num_types);
    float acc = 0;
    for (int t = 0; t < cfg->num_types; ++t) { acc += cfg->proportions[t]; cum[t] = acc; }
    std::mt19937 gen(cfg->seed);
    std::uniform_real_distribution<float> d_type(0, 1);
    const bool open_loop = cfg->mean_interarrival_us > 0;
    const double mean_global = open_loop ? cfg->mean_interarrival_us / G : 1.0;
    std::exponential_distribution<> d_exp(1. / mean_global);
    const double mu = std::log(mean_global) - cfg->lognormal_sigma * cfg->lognormal_sigma / 2;
    std::lognormal_distribution<> d_ln(mu, cfg->lognormal_sigma > 0 ? cfg->lognormal_sigma : 1.0);
    std::vector<std::vector<Request>> reqs(G);
    for (int phase = 0; phase < 2; ++phase) {
        const uint64_t n = (uint64_t)(phase == 0 ? cfg->warmup_jobs : cfg->num_jobs) * G;
        double t_next = 0;
        for (uint64_t i = 0; i < n; ++i) {
            Request r;
            r.arrival_us = t_next;
            int ty = (int)(std::lower_bound(cum.begin(), cum.end(), d_type(gen)) - cum.begin());
            r.type = ty >= cfg->num_types ? cfg->num_types - 1 : ty;
            r.measured = phase == 1;
            reqs[i % G].push_back(r);
            if (open_loop) t_next += cfg->lognormal_sigma > 0 ? d_ln(gen) : d_exp(gen);
        }
    }
    return reqs;
}

// One replica: owns a server on `device` and plays its share of the request stream.
void run_replica(const pb_loadgen_config* cfg, int gpu_index, const std::vector<Request>* reqs, std::atomic<int>* ready,
                 std::atomic<int>* go, std::atomic<int>* phase2_ready, GpuResult* out) {
    const int device = cfg->devices[gpu_index];
    // This thread submits, polls the ring and makes every CUDA launch call of its GPU: keep it on one core
    // (the reference pins its server loop with taskset, sosp23_artifact/gen_data_fig11_paella.sh:63), and
    // allocate the request slots after that so that their pages are first touched from there.
    if (cfg->cpu_of_replica[gpu_index] >= 0) {
        cpu_set_t set;
        CPU_ZERO(&set);
        CPU_SET(cfg->cpu_of_replica[gpu_index], &set);
        if (pthread_setaffinity_np(pthread_self(), sizeof(set), &set) != 0)
            fprintf(stderr, "paella_b200: could not pin replica %d to cpu %d (continuing unpinned)\n", gpu_index, cfg->cpu_of_replica[gpu_index]);
    }
    auto fail = [&](int rc) {
        out->rc = rc;
        snprintf(out->err, sizeof(out->err), "%s", pb_last_error());
        ready->fetch_add(1);
        phase2_ready->fetch_add(1);   // never leave the other replicas waiting
    };
    pb_server_config sc = cfg->server;
    sc.device = device;
    sc.device_resident = cfg->device_resident;
    pb_server* srv = nullptr;
    int rc = pb_server_create(&sc, &srv);
    if (rc != PB_OK) return fail(rc);

    const int nt = cfg->num_types;
    std::vector<uint32_t> type_id(nt);
    std::vector<size_t> in_b(nt), out_b(nt), slot_b(nt);
    std::vector<std::vector<int>> free_slots(nt);
    std::vector<Slot> slots;
    std::vector<void*> pinned;
    std::mt19937 fill_rng(cfg->seed + 977u * (unsigned)gpu_index);
    std::normal_distribution<float> nd(0.f, 1.f);
    std::uniform_real_distribution<float> ud(0.f, 1.f);
    for (int t = 0; t < nt; ++t) {
        rc = pb_server_register_job(srv, cfg->plugin_paths[t], &type_id[t]);
        if (rc != PB_OK) { pb_server_destroy(srv); return fail(rc); }
        pb_server_job_io_bytes(srv, type_id[t], &in_b[t], &out_b[t], &slot_b[t]);
        const unsigned n = cfg->max_outstanding[t] ? cfg->max_outstanding[t] : 1;
        void* base = nullptr;
        if (cudaHostAlloc(&base, slot_b[t] * n, cudaHostAllocDefault) != cudaSuccess) {
            pb::set_error("cudaHostAlloc of %zu bytes of request slots failed", slot_b[t] * n);
            pb_server_destroy(srv);
            return fail(PB_ERR_CUDA);
        }
        pinned.push_back(base);
        for (unsigned i = 0; i < n; ++i) {
            Slot s;
            s.io = (char*)base + slot_b[t] * i;
            s.type = t;
            float* f = (float*)s.io;
            for (size_t k = 0; k < in_b[t] / 4; ++k) f[k] = cfg->input_uniform[t] ? ud(fill_rng) : nd(fill_rng);
            free_slots[t].push_back((int)slots.size());
            slots.push_back(s);
        }
    }

    // cookie = slot index << 32 | request index (or 0xffffffff for warm-up launches)
    std::vector<uint64_t> cookies(256);
    std::vector<int32_t> errs(256);
    int last_step_records = 0;
    auto drain = [&](auto&& on_done) -> int {
        const int st = pb_server_step(srv, 256);
        if (st < 0) return st;
        last_step_records = st;
        int n;
        while ((n = pb_server_poll_done(srv, cookies.data(), errs.data(), 256)) > 0)
            for (int i = 0; i < n; ++i) on_done(cookies[i], errs[i]);
        return PB_OK;
    };

    // ---- one launch per instance, un-timed: runs full_init (weights, buffers) ----
    {
        size_t outstanding = 0;
        for (size_t i = 0; i < slots.size(); ++i) {
            rc = pb_server_launch(srv, type_id[slots[i].type], slots[i].io, ((uint64_t)i << 32) | 0xffffffffu);
            if (rc != PB_OK) { pb_server_destroy(srv); return fail(rc); }
            ++outstanding;
        }
        const Clock::time_point w0 = Clock::now();
        while (outstanding > 0) {
            rc = drain([&](uint64_t, int32_t e) { --outstanding; if (e) ++out->errors; });
            if (rc != PB_OK) { pb_server_destroy(srv); return fail(rc); }
            if (us_since(w0) > 120e6) { pb::set_error("warm-up launches did not finish within 120 s"); pb_server_destroy(srv); return fail(PB_ERR_TIMEOUT); }
        }
    }

    ready->fetch_add(1);
    while (go->load(std::memory_order_acquire) == 0) std::this_thread::yield();

    const bool closed_loop = cfg->mean_interarrival_us <= 0;
    const unsigned cap = cfg->concurrency ? cfg->concurrency : 1u << 30;
    std::vector<double> submit_us(reqs->size(), 0.0);
    bool have_first = false;
    int loop_rc = PB_OK;

    // Plays requests [lo, hi) to completion; arrival times are relative to `start`.
    auto play = [&](size_t lo, size_t hi, Clock::time_point start) {
        std::vector<std::deque<uint32_t>> due(nt);
        size_t next_req = lo, done_reqs = 0, outstanding = 0;
        auto launch_req = [&](uint32_t ri) -> int {
            const Request& r = (*reqs)[ri];
            const int slot = free_slots[r.type].back();
            free_slots[r.type].pop_back();
            if (closed_loop) submit_us[ri] = us_since(start);
            if (r.measured && !cfg->device_resident) { out->h2d += in_b[r.type]; out->d2h += out_b[r.type]; }
            return pb_server_launch(srv, type_id[r.type], slots[slot].io, ((uint64_t)slot << 32) | ri);
        };
        const Clock::time_point run0 = Clock::now();
        Clock::time_point it0 = run0;
        while (done_reqs < hi - lo && loop_rc == PB_OK) {
            const size_t next_before = next_req;
            while (next_req < hi && outstanding < cap) {
                const Request& r = (*reqs)[next_req];
                if (!closed_loop && us_since(start) < r.arrival_us) break;
                ++outstanding;
                if (free_slots[r.type].empty()) due[r.type].push_back((uint32_t)next_req);
                else loop_rc = launch_req((uint32_t)next_req);
                ++next_req;
                if (loop_rc != PB_OK) break;
            }
            if (loop_rc != PB_OK) break;
            const int drc = drain([&](uint64_t cookie, int32_t e) {
                const uint32_t ri = (uint32_t)(cookie & 0xffffffffu);
                const int slot = (int)(cookie >> 32);
                const Request& r = (*reqs)[ri];
                const double now = us_since(start);
                if (e) ++out->errors;
                if (r.measured) {
                    const double t_arr = closed_loop ? submit_us[ri] : r.arrival_us;
                    out->lat[r.type].push_back(now - t_arr);
                    if (!have_first || t_arr < out->first_arrival_us) { out->first_arrival_us = t_arr; have_first = true; }
                    out->last_done_us = std::max(out->last_done_us, now);
                    ++out->measured;
                    slots[(size_t)slot].measured = true;
                }
                free_slots[r.type].push_back(slot);
                --outstanding;
                ++done_reqs;
                if (!due[r.type].empty()) {
                    const uint32_t q = due[r.type].front();
                    due[r.type].pop_front();
                    const int lrc = launch_req(q);
                    if (lrc != PB_OK && loop_rc == PB_OK) loop_rc = lrc;
                }
            });
            if (drc != PB_OK && loop_rc == PB_OK) loop_rc = drc;
            // an iteration that neither submitted nor saw a notification is waiting for the GPU
            const Clock::time_point it1 = Clock::now();
            const double it_us = std::chrono::duration<double, std::micro>(it1 - it0).count();
            if (next_req == next_before && last_step_records == 0) out->host_idle_us += it_us;
            else out->host_busy_us += it_us;
            it0 = it1;
            if (us_since(run0) > 600e6) { pb::set_error("load run exceeded 600 s"); loop_rc = PB_ERR_TIMEOUT; }
        }
    };

    // ---- un-timed warm-up requests, fully drained ----
    size_t n_warm = 0;
    while (n_warm < reqs->size() && !(*reqs)[n_warm].measured) ++n_warm;
    play(0, n_warm, Clock::now());
    cudaDeviceSynchronize();

    // ---- measured requests: all replicas start together; CUDA events bracket the phase ----
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    cudaEventCreate(&ev0);
    cudaEventCreate(&ev1);
    phase2_ready->fetch_add(1);
    while (phase2_ready->load(std::memory_order_acquire) < cfg->num_gpus) std::this_thread::yield();
    const uint64_t kernels0 = srv->num_kernels, records0 = srv->num_records, decisions0 = srv->scheduler->num_decisions();
    const uint64_t launch_ns0 = srv->scheduler->run_next_ns();
    out->host_idle_us = out->host_busy_us = 0;
    cudaEventRecord(ev0, 0);
    play(n_warm, reqs->size(), Clock::now());
    cudaDeviceSynchronize();
    cudaEventRecord(ev1, 0);
    cudaEventSynchronize(ev1);
    float ms = 0;
    if (cudaEventElapsedTime(&ms, ev0, ev1) == cudaSuccess) out->event_ms = ms;
    cudaEventDestroy(ev0);
    cudaEventDestroy(ev1);

    out->kernels = srv->num_kernels - kernels0;
    out->host_launch_us = (double)(srv->scheduler->run_next_ns() - launch_ns0) * 1e-3;
    out->records = srv->num_records - records0;
    out->decisions = srv->scheduler->num_decisions() - decisions0;
    if (loop_rc != PB_OK) {
        out->rc = loop_rc;
        snprintf(out->err, sizeof(out->err), "%s", pb_last_error());
    }
    // Samples for an output check by the caller: replica 0 copies out, per job type, the first slots in which a
    // measured request completed - the slot's input and the result the serving path left beside it.
    if (gpu_index == 0 && cfg->sample_buf && cfg->samples_per_type > 0 && !cfg->device_resident) {
        char* dst = static_cast<char*>(cfg->sample_buf);
        uint64_t used = 0;
        std::vector<uint32_t> taken(nt, 0);
        for (size_t i = 0; i < slots.size(); ++i) {
            const Slot& sl = slots[i];
            const int t = sl.type;
            if (!sl.measured || taken[t] >= cfg->samples_per_type) continue;
            const uint64_t in_pad = (in_b[t] + 7) / 8 * 8, out_pad = (out_b[t] + 7) / 8 * 8;
            const uint64_t need = 24 + in_pad + out_pad;
            if (used + need > cfg->sample_buf_bytes) break;
            const uint32_t hdr32[2] = {(uint32_t)t, (uint32_t)i};
            const uint64_t hdr64[2] = {(uint64_t)in_b[t], (uint64_t)out_b[t]};
            memcpy(dst + used, hdr32, 8);
            memcpy(dst + used + 8, hdr64, 16);
            memcpy(dst + used + 24, sl.io, in_b[t]);
            memcpy(dst + used + 24 + in_pad, (const char*)sl.io + in_pad, out_b[t]);
            used += need;
            ++taken[t];
            ++out->samples;
        }
        out->sample_bytes = used;
    }
    pb_server_destroy(srv);
    for (void* p : pinned) cudaFreeHost(p);
}

}  // namespace

extern "C" {

void pb_loadgen_config_default(pb_loadgen_config* cfg) {
    memset(cfg, 0, sizeof(*cfg));
    cfg->num_gpus = 1;
    for (int i = 0; i < PB_MAX_GPUS; ++i) cfg->devices[i] = i;
    cfg->concurrency = 64;
    cfg->mean_interarrival_us = 0;
    cfg->num_jobs = 1000;
    cfg->warmup_jobs = 100;
    cfg->seed = 1;
    for (int i = 0; i < PB_MAX_GPUS; ++i) cfg->cpu_of_replica[i] = -1;
    pb_server_config_default(&cfg->server);
}

int pb_loadgen_run(const pb_loadgen_config* cfg, pb_loadgen_result* out) {
    PB_REQUIRE(cfg && out, "pb_loadgen_run: NULL argument");
    PB_REQUIRE(cfg->num_gpus >= 1 && cfg->num_gpus <= PB_MAX_GPUS, "pb_loadgen_run: num_gpus %d out of range", cfg->num_gpus);
    PB_REQUIRE(cfg->num_types >= 1 && cfg->num_types <= PB_MAX_JOB_TYPES, "pb_loadgen_run: num_types %d out of range", cfg->num_types);
    memset(out, 0, sizeof(*out));
    const int G = cfg->num_gpus;
    std::vector<std::vector<Request>> reqs = plan_requests(cfg);

    std::vector<GpuResult> res(G);
    std::atomic<int> ready(0), go(0), phase2(0);
    std::vector<std::thread> th;
    for (int g = 0; g < G; ++g) th.emplace_back(run_replica, cfg, g, &reqs[g], &ready, &go, &phase2, &res[g]);
    while (ready.load() < G) std::this_thread::yield();
    go.store(1, std::memory_order_release);
    for (auto& t : th) t.join();

    int rc = PB_OK;
    std::vector<double> all;
    std::vector<std::vector<double>> per_type(cfg->num_types);
    double first = 1e300, last = 0;
    uint64_t measured = 0;
    for (int g = 0; g < G; ++g) {
        if (res[g].rc != PB_OK && rc == PB_OK) { rc = res[g].rc; pb::set_error("replica %d: %s", g, res[g].err); }
        for (int t = 0; t < cfg->num_types; ++t) {
            per_type[t].insert(per_type[t].end(), res[g].lat[t].begin(), res[g].lat[t].end());
            all.insert(all.end(), res[g].lat[t].begin(), res[g].lat[t].end());
        }
        if (res[g].measured) {
            first = std::min(first, res[g].first_arrival_us);
            last = std::max(last, res[g].last_done_us);
            out->per_gpu_rps[g] = res[g].measured / ((res[g].last_done_us - res[g].first_arrival_us) * 1e-6);
        }
        measured += res[g].measured;
        out->kernels_launched += res[g].kernels;
        out->host_launch_us += res[g].host_launch_us;
        out->host_sched_us += res[g].host_busy_us - res[g].host_launch_us;
        out->host_idle_us += res[g].host_idle_us;
        out->records_consumed += res[g].records;
        out->decisions += res[g].decisions;
        out->h2d_bytes += res[g].h2d;
        out->d2h_bytes += res[g].d2h;
        out->errors += res[g].errors;
        out->samples += res[g].samples;
        out->sample_bytes += res[g].sample_bytes;
        out->elapsed_event_ms = std::max(out->elapsed_event_ms, res[g].event_ms);
    }
    if (rc != PB_OK) return rc;
    out->elapsed_us = measured ? last - first : 0;
    out->throughput_rps = out->elapsed_us > 0 ? measured / (out->elapsed_us * 1e-6) : 0;
    out->all = stats_of(all);
    for (int t = 0; t < cfg->num_types; ++t) out->per_type[t] = stats_of(per_type[t]);
    return PB_OK;
}

int pb_loadgen_plan(const pb_loadgen_config* cfg, int replica, uint32_t* types, double* arrivals_us, uint8_t* measured,
                    uint32_t max, uint32_t* n_out) {
    PB_REQUIRE(cfg && n_out, "pb_loadgen_plan: NULL argument");
    PB_REQUIRE(cfg->num_gpus >= 1 && cfg->num_gpus <= PB_MAX_GPUS && replica >= 0 && replica < cfg->num_gpus,
               "pb_loadgen_plan: replica %d of %d", replica, cfg->num_gpus);
    PB_REQUIRE(cfg->num_types >= 1 && cfg->num_types <= PB_MAX_JOB_TYPES, "pb_loadgen_plan: num_types %d out of range", cfg->num_types);
    const std::vector<Request> r = plan_requests(cfg)[replica];
    *n_out = (uint32_t)r.size();
    for (uint32_t i = 0; i < r.size() && i < max; ++i) {
        if (types) types[i] = (uint32_t)r[i].type;
        if (arrivals_us) arrivals_us[i] = r[i].arrival_us;
        if (measured) measured[i] = r[i].measured ? 1 : 0;
    }
    return PB_OK;
}

}  // extern "C"
