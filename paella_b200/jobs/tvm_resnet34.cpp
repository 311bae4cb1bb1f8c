// ResNet-34 adapter; I/O sizes as jobs/tvm_resnet34/tvm_resnet34.cpp (224*224*3 floats in, 1000 out).
#include "model_job.h"
PB_DEFINE_MODEL_JOB("resnet34", 224 * 224 * 3, 1000)
