// DenseNet-121 adapter; I/O sizes as jobs/tvm_densenet121/tvm_densenet121.cpp (224*224*3 floats in, 1000 out).
#include "model_job.h"
PB_DEFINE_MODEL_JOB("densenet121", 224 * 224 * 3, 1000)
