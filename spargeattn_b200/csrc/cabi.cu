// Status strings and ABI version of the C interface declared in include/sparge_b200.h.
#include "common.cuh"

extern "C" const char* sparge_strerror(int status) {
  switch (status) {
    case SPARGE_OK: return "ok";
    case SPARGE_ERR_INVALID_ARG: return "invalid argument (head_dim must be 64 or 128, dtype code 0/1, sizes positive)";
    case SPARGE_ERR_NULL: return "a required pointer is NULL";
    case SPARGE_ERR_CUDA: return "a CUDA call failed";
    case SPARGE_ERR_TOO_LARGE: return "a size exceeds what the kernel supports";
    case SPARGE_ERR_UNSUPPORTED: return "not implemented in this build";
    default: return "unknown status";
  }
}

extern "C" int sparge_abi_version(void) { return 1; }
