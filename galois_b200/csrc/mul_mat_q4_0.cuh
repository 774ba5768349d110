// Internal interface of the small-batch Q4_0 mat-mul kernels (mul_mat_q4_0.cu).
#pragma once
#include "common.cuh"

// Sets the shared-memory limit of every bulk-kernel instance on the current device.
int gb_mmv_bulk_init(galois_b200_ctx* ctx);
// True when the bulk-copy GEMV can take this problem (2-D, contiguous weights,
// K % 256 == 0, 16-byte aligned base, batch <= 8).
bool gb_mmv_bulk_supported(const galois_b200_ctx* ctx, const void* w, const galois_dim* wd, const galois_dim* xd,
                           const galois_dim* dd);
int gb_mmv_q4_0_bulk(galois_b200_ctx* ctx, const void* w, const galois_dim* wd, const gb_q8_soa& xq,
                     const galois_dim* xd, float* dst, const galois_dim* dd);
// General path: any K % 32 == 0, any row / batch strides.
int gb_mmv_q4_0_direct(galois_b200_ctx* ctx, const void* w, const galois_dim* wd, const gb_q8_soa& xq,
                       const galois_dim* xd, float* dst, const galois_dim* dd);
