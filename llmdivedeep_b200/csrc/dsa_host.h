// Host-side helpers shared by the .cu files: error reporting and launch checks.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/dsa_b200.h"

namespace dsa {

// Records a message for dsa_last_error_string() and returns `code`.
int set_error(int code, const char* fmt, ...);
// cudaGetLastError() after a launch; no synchronisation.
int check_launch(const char* what);
// Multiprocessor count of the current device (cached per device).
int sm_count();

}  // namespace dsa
