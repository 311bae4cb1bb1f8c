// squeezenet1_1 adapter; I/O sizes as jobs/tvm_squeezenet1_1/tvm_squeezenet1_1.cpp (224*224*3 floats in, 1000 out).
#include "model_job.h"
PB_DEFINE_MODEL_JOB("squeezenet1_1", 224 * 224 * 3, 1000)
