// 10 kernels per job (jobs/dummy_short/dummy_short.cu:43-62), each block busy for 10 us.
#include "synthetic_jobs.h"
extern "C" __attribute__((visibility("default"))) llis::job::Job* init_job() {
    return new pbjobs::SpinJob((unsigned)pbjobs::env_ul("PB_DUMMY_SHORT_KERNELS", 10), pbjobs::env_ul("PB_DUMMY_SHORT_NS", 10000), "PB_DUMMY_SHORT_BLOCKS");
}
