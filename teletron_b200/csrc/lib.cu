// Library-wide host helpers: version and last-CUDA-error bookkeeping.
#include "common.cuh"
#include "teletron_b200.h"

#include <string.h>

static char g_last_error[256] = "";

int tt_record_cuda(cudaError_t e) {
    strncpy(g_last_error, cudaGetErrorString(e), sizeof(g_last_error) - 1);
    return TT_ERR_CUDA;
}

extern "C" const char* tt_last_cuda_error() { return g_last_error; }
extern "C" int tt_version() { return 1; }
