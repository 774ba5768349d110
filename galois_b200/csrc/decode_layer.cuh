// Internal interface of the persistent decode-layer kernel (decode_layer.cu).
#pragma once
#include "common.cuh"

#include <math.h>

// Sets the kernel's shared-memory limit on the current device.
int gb_decode_init(galois_b200_ctx* ctx);
