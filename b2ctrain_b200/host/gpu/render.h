// Forwarding header: a caller written against the reference tree includes "gpu/render.h" for CameraGPU, RenderParams, RenderCtx and the forward / backward operators (src/gpu/render.h);
// with this folder on the include path it gets the same names from the B200 host mirror.
#pragma once
#include "../b2c_api.h"
