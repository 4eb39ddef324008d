// Forwarding header: a caller written against the reference tree includes "dataset/camera.h" for Camera (src/dataset/camera.h);
// with this folder on the include path it gets the same names from the B200 host mirror.
#pragma once
#include "../b2c_api.h"
