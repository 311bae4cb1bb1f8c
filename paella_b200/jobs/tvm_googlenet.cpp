// googlenet adapter; I/O sizes as jobs/tvm_googlenet/tvm_googlenet.cpp (224*224*3 floats in, 1000 out).
#include "model_job.h"
PB_DEFINE_MODEL_JOB("googlenet", 224 * 224 * 3, 1000)
