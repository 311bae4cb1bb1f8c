#include "synthetic_jobs.h"
extern "C" __attribute__((visibility("default"))) llis::job::Job* init_job() { return new pbjobs::VecAddJob(); }
