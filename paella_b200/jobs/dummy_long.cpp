// 50 kernels per job in the reference (jobs/dummy_long); here each block is busy for 1 ms.
#include "synthetic_jobs.h"
extern "C" __attribute__((visibility("default"))) llis::job::Job* init_job() {
    return new pbjobs::SpinJob((unsigned)pbjobs::env_ul("PB_DUMMY_LONG_KERNELS", 10), pbjobs::env_ul("PB_DUMMY_LONG_NS", 1000000), "PB_DUMMY_LONG_BLOCKS");
}
