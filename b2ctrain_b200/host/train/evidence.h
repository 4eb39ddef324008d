// Forwarding header: a caller written against the reference tree includes "train/evidence.h" for compute_evidence and
// the two downloads (src/train/evidence.h); with this folder on the include path it gets them from the B200 host mirror.
#pragma once
#include "../evidence.h"
