// placeholder until the peer-memory kernels land
#include "include/gv_kernels.h"
#include "include/gv_ptx.cuh"
GV_DEFINE_ERROR_READER(gv_read_error_comm)
