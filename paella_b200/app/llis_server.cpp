// llis_server: one serving process for one GPU.  Flags of the reference (src/server/server.cpp:204-226)
// plus --gpu: --name <server name> --sched {full3,fifo,fifo2} --num_streams N --extra_kernels N
// --unfair X --sched_sleep N --gpu I.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>

#include "../host/ipc_server.h"

int main(int argc, char** argv) {
    pb_server_config cfg;
    pb_server_config_default(&cfg);
    std::string name, sched = "full3";
    for (int i = 1; i < argc; ++i) {
        std::string a = argv[i];
        std::string val;
        const size_t eq = a.find('=');
        if (eq != std::string::npos) { val = a.substr(eq + 1); a = a.substr(0, eq); }
        else if (a != "--help" && i + 1 < argc) val = argv[++i];
        if (a == "--help") {
            printf("llis_server --name NAME [--sched full3|fifo|fifo2] [--num_streams 500] [--extra_kernels 2] [--unfair 1e6] "
                   "[--sched_sleep 0] [--gpu 0] [--gang 1] [--deferred 0]\n");
            return 1;
        }
        else if (a == "--name") name = val;
        else if (a == "--sched") sched = val;
        else if (a == "--num_streams") cfg.num_streams = (uint32_t)atoi(val.c_str());
        else if (a == "--extra_kernels") cfg.extra_kernels = (uint32_t)atoi(val.c_str());
        else if (a == "--unfair") cfg.unfairness_threshold = (float)atof(val.c_str());
        else if (a == "--sched_sleep") cfg.sched_sleep = (uint32_t)atoi(val.c_str());
        else if (a == "--gpu") cfg.device = atoi(val.c_str());
        else if (a == "--gang") cfg.max_gang = (uint32_t)atoi(val.c_str());
        else if (a == "--deferred") cfg.deferred_schedule = (uint32_t)atoi(val.c_str());
        else { fprintf(stderr, "llis_server: unknown option %s\n", a.c_str()); return 2; }
    }
    if (name.empty()) { fprintf(stderr, "llis_server: --name is required\n"); return 2; }
    cfg.scheduler = sched.c_str();
    try {
        llis::server::IpcServer server(name, cfg);
        fprintf(stderr, "llis_server '%s' on GPU %d, scheduler %s\n", name.c_str(), cfg.device, sched.c_str());
        server.serve();
    } catch (const std::exception& e) {
        fprintf(stderr, "llis_server: %s\n", e.what());
        return 1;
    }
    return 0;
}
