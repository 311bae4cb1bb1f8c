// MobileNetV2 adapter; I/O sizes as jobs/tvm_mobilenet/tvm_mobilenet.cpp (224*224*3 floats in, 1000 out).
#include "model_job.h"
PB_DEFINE_MODEL_JOB("mobilenet", 224 * 224 * 3, 1000)
