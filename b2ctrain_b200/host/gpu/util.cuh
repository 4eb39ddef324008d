// Forwarding header: a caller written against the reference tree includes "gpu/util.cuh" for DevBuf, CUDA_CHECK and the tile constants (src/gpu/util.cuh);
// with this folder on the include path it gets the same names from the B200 host mirror.
#pragma once
#include "../b2c_api.h"
