// Forwarding header: a caller written against the reference tree includes "gpu/refine.h" for RefineState and its
// parameter structs (src/gpu/refine.h); with this folder on the include path it gets them from the B200 host mirror.
#pragma once
#include "../refine.h"
