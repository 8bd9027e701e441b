// Single translation unit of libptwm_b200.so: the kernels live in headers, so
// decode and encode hosts are compiled together.
#include "ptwm_b200.cu"
#include "encoder.cu"
#include "noalloc.cu"
