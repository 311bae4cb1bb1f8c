// ArcFace ResNet-100 adapter; I/O sizes as jobs/tvm_arcfaceresnet100/tvm_arcfaceresnet100.cpp
// (112*112*3 floats in, a 512-float embedding out).
#include "model_job.h"
PB_DEFINE_MODEL_JOB("arcfaceresnet100", 112 * 112 * 3, 512)
