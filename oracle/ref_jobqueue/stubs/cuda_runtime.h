#pragma once
typedef struct CUstream_st* cudaStream_t;
