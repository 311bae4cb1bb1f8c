// llis_app_client: open-loop load generator over the client library.  Options and positional job
// triples of the reference (app/client.cpp:246-405):
//   --server_name S --iat MEAN_US [--ln_sigma SIGMA] --concurrency N --num_jobs N
//   [--start_record_num N] --seed N --prefix PATH   <job.so> <proportion> <max_outstanding> ...
// Arrivals exponential (lognormal with --ln_sigma), job type by cumulative proportions, latency =
// completion - scheduled arrival, stats mean,p50,p90,p95,p99,max,sd with sorted[n*q] (:192-212).
// Writes <prefix>.txt: "iat,num_jobs,elapsed_us" followed by the seven stats overall and per model.
#include <llis/client/client.h>

#include <algorithm>
#include <atomic>
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <deque>
#include <random>
#include <string>
#include <thread>
#include <vector>

using Clock = std::chrono::steady_clock;
using llis::client::JobInstanceRef;

static void stats(FILE* fp, std::vector<double> v) {
    if (v.empty()) { fprintf(fp, ",0,0,0,0,0,0,0"); return; }
    std::sort(v.begin(), v.end());
    double mean = 0, sq = 0;
    for (double x : v) { mean += x / v.size(); sq += x * x / v.size(); }
    const double sd = v.size() > 1 ? std::sqrt(std::max(0.0, (sq - mean * mean) * ((double)v.size() / (v.size() - 1)))) : 0;
    fprintf(fp, ",%f,%f,%f,%f,%f,%f,%f", mean, v[v.size() / 2], v[(size_t)(v.size() * 0.90)], v[(size_t)(v.size() * 0.95)],
            v[(size_t)(v.size() * 0.99)], v.back(), sd);
}

int main(int argc, char** argv) {
    std::string server_name, prefix = "llis_app_client";
    double iat = -1, sigma = 0;
    unsigned concurrency = 64, num_jobs = 1000, start_record = 0, seed = 1;
    int i = 1;
    for (; i < argc && strncmp(argv[i], "--", 2) == 0; i += 2) {
        const std::string a = argv[i];
        const char* v = i + 1 < argc ? argv[i + 1] : "";
        if (a == "--server_name") server_name = v;
        else if (a == "--iat") iat = atof(v);
        else if (a == "--ln_sigma") sigma = atof(v);
        else if (a == "--concurrency") concurrency = (unsigned)atoi(v);
        else if (a == "--num_jobs") num_jobs = (unsigned)atoi(v);
        else if (a == "--start_record_num") start_record = (unsigned)atoi(v);
        else if (a == "--seed") seed = (unsigned)atoi(v);
        else if (a == "--prefix") prefix = v;
        else { fprintf(stderr, "unknown option %s\n", a.c_str()); return 2; }
    }
    if (server_name.empty() || iat <= 0 || (argc - i) < 3 || (argc - i) % 3 != 0) {
        fprintf(stderr, "usage: llis_app_client --server_name S --iat US [--ln_sigma X] [--concurrency N] [--num_jobs N] [--start_record_num N] "
                        "[--seed N] [--prefix P] <job.so> <proportion> <max_outstanding> ...\n");
        return 2;
    }
    llis::client::Client client(server_name);
    struct Type { llis::client::JobRef* ref; float prop; unsigned cap; std::vector<JobInstanceRef*> idle; std::deque<double> due; std::vector<double> lat; };
    std::vector<Type> types;
    std::vector<float> cum;
    float acc = 0;
    for (; i + 2 < argc + 0; i += 3) {
        Type t{};
        t.ref = client.register_job(argv[i]);
        t.prop = (float)atof(argv[i + 1]);
        t.cap = (unsigned)atoi(argv[i + 2]);
        for (unsigned k = 0; k < t.cap; ++k) t.idle.push_back(t.ref->create_instance());
        acc += t.prop;
        cum.push_back(acc);
        types.push_back(std::move(t));
    }
    auto type_of = [&](JobInstanceRef* r) -> Type& {
        for (Type& t : types) if (t.ref == r->get_job_ref()) return t;
        return types[0];
    };
    // one warm-up launch per instance (app/client.cpp:426-446)
    {
        size_t n = 0;
        for (Type& t : types) for (JobInstanceRef* r : t.idle) { r->launch(); ++n; }
        while (n > 0) { client.wait(); --n; }
    }
    std::mt19937 gen(seed);
    std::exponential_distribution<> d_exp(1. / iat);
    std::lognormal_distribution<> d_ln(std::log(iat) - sigma * sigma / 2, sigma > 0 ? sigma : 1.0);
    std::uniform_real_distribution<float> d_type(0, 1);

    std::atomic<unsigned> outstanding(0), finished(0);
    std::vector<double> all_lat;
    const Clock::time_point t0 = Clock::now();
    auto now_us = [&] { return std::chrono::duration<double, std::micro>(Clock::now() - t0).count(); };
    unsigned submitted = 0, recorded_from = start_record;
    double next_submit = 0, last_done = 0;
    // Single thread: submit what is due, then collect completions without blocking.
    while (finished.load() < num_jobs) {
        if (submitted < num_jobs && now_us() >= next_submit && outstanding.load() < concurrency) {
            const unsigned ty = (unsigned)(std::lower_bound(cum.begin(), cum.end(), d_type(gen)) - cum.begin());
            Type& t = types[std::min<size_t>(ty, types.size() - 1)];
            if (t.idle.empty()) {
                t.due.push_back(next_submit);
            } else {
                JobInstanceRef* r = t.idle.back();
                t.idle.pop_back();
                r->set_start_time(next_submit);
                r->launch();
            }
            ++outstanding;
            ++submitted;
            next_submit += sigma > 0 ? d_ln(gen) : d_exp(gen);
        }
        JobInstanceRef* r = client.wait_timeout(0);
        if (!r) continue;
        const double now = now_us();
        Type& t = type_of(r);
        const unsigned idx = finished.fetch_add(1);
        if (idx >= recorded_from) { t.lat.push_back(now - r->get_start_time()); all_lat.push_back(now - r->get_start_time()); }
        last_done = now;
        --outstanding;
        if (!t.due.empty()) {
            r->set_start_time(t.due.front());
            t.due.pop_front();
            r->launch();
        } else {
            t.idle.push_back(r);
        }
    }
    FILE* fp = fopen((prefix + ".txt").c_str(), "w");
    if (!fp) fp = stdout;
    fprintf(fp, "%f,%u,%f", iat, num_jobs, last_done);
    stats(fp, all_lat);
    for (Type& t : types) stats(fp, t.lat);
    fprintf(fp, "\n");
    if (fp != stdout) fclose(fp);
    printf("jobs %u elapsed_us %.0f throughput_rps %.1f\n", num_jobs, last_done, num_jobs / (last_done * 1e-6));
    return 0;
}
