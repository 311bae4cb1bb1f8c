// ResNet-18 adapter; I/O sizes as jobs/tvm_resnet18/tvm_resnet18.cpp (224*224*3 floats in, 1000 out).
#include "model_job.h"
PB_DEFINE_MODEL_JOB("resnet18", 224 * 224 * 3, 1000)
