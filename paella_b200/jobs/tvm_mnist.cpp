// MNIST CNN adapter; I/O sizes as jobs/tvm_mnist/tvm_mnist.cpp:12-18 (28*28 floats in, 10 out).
#include "model_job.h"
PB_DEFINE_MODEL_JOB("mnist", 28 * 28, 10)
