// Internal interface of the activation quantiser (quantize.cu).
#pragma once
#include "common.cuh"

// Bytes of scratch the structure-of-arrays Q8_0 form of `nrows` rows of `k` floats needs.
size_t gb_q8_soa_bytes(int64_t k, int64_t nrows);
// Quantises every row of x (f32 {K, ne1, ne2, ne3}, nb[0] == 1) into `scratch`
// (rows numbered i11 + i12*ne11 + i13*ne12*ne11, as in src/op.rs:1405-1420) and
// fills `out` with the two array pointers.
int gb_quantize_q8_soa(galois_b200_ctx* ctx, const float* x, const galois_dim* xd, void* scratch, gb_q8_soa* out);
