// Inception-v3 adapter.  The benchmark configuration serves it at 299x299; the reference
// compiles its copy at 224x224 (jobs/tvm_inception_v3/tvm_inception_v3.cpp:12).
#include "model_job.h"
PB_DEFINE_MODEL_JOB("inception_v3", 299 * 299 * 3, 1000)
