// 320x240 face detector adapter.  Input as jobs/tvm_ultraface320/tvm_ultraface320.cpp:10-12 (240*320*3 floats).
// The reference's adapter returns the graph's first output only, 4420 x 2 scores (:14-16); here the boxes follow
// them in the same output block: [4420 x 2 scores | 4420 x 4 corner-form boxes].  A client that reads 4420*2
// floats at the output offset sees the same tensor as with the reference.
#include "model_job.h"
PB_DEFINE_MODEL_JOB("ultraface320", 240 * 320 * 3, 4420 * 6)
