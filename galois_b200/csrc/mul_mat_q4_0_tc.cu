// Large-batch (prefill) Q4_0 x Q8_0 mat-mul on the tcgen05 int8 tensor-core path.
#include "mul_mat_q4_0_tc.cuh"

int gb_mm_tc_init(galois_b200_ctx*) { return 0; }
bool gb_mm_tc_supported(const galois_b200_ctx*, const void*, const galois_dim*, const galois_dim*, const galois_dim*) {
    return false;
}
size_t gb_mm_tc_scratch_bytes(const galois_dim*, const galois_dim*) { return 0; }
int gb_mm_q4_0_tc(galois_b200_ctx* ctx, const void*, const galois_dim*, const gb_q8_soa&, const galois_dim*, float*,
                  const galois_dim*, void*) {
    return gb_fail(ctx, GALOIS_B200_E_LAYOUT, "mul_mat_q4_0: tensor-core variant not available");
}
