// Internal interface of the general Q4_0 mat-mul kernel (mul_mat_q4_0.cu).
#pragma once
#include "common.cuh"

// General path: any K % 32 == 0, any row / batch strides, dims 2/3 broadcast.
int gb_mmv_q4_0_direct(galois_b200_ctx* ctx, const void* w, const galois_dim* wd, const gb_q8_soa& xq,
                       const galois_dim* xd, float* dst, const galois_dim* dd);
