// Forwarding header: a caller written against the reference tree includes "gpu/optim.h" for OptimParams and optimizer_step (src/gpu/optim.h);
// with this folder on the include path it gets the same names from the B200 host mirror.
#pragma once
#include "../b2c_api.h"
