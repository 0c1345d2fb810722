// placeholder until the tcgen05 attention kernels land
#include "include/gv_kernels.h"
#include "include/gv_ptx.cuh"
GV_DEFINE_ERROR_READER(gv_read_error_attn)
