// ResNet-50 adapter; I/O sizes as jobs/tvm_resnet50/tvm_resnet50.cpp (224*224*3 floats in, 1000 out).
#include "model_job.h"
PB_DEFINE_MODEL_JOB("resnet50", 224 * 224 * 3, 1000)
