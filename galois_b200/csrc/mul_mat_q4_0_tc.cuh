// Internal interface of the large-batch (prefill) Q4_0 mat-mul on the
// tcgen05 int8 tensor-core path (mul_mat_q4_0_tc.cu).
#pragma once
#include "common.cuh"

// Batches at least this large take the tensor-core path when it supports the shape.
#define GB_TC_MIN_BATCH 9

int gb_mm_tc_init(galois_b200_ctx* ctx);
// 2-D contiguous weights with K % 256 == 0 and a 16-byte aligned base; 16-byte aligned activations.
bool gb_mm_tc_supported(const galois_b200_ctx* ctx, const void* w, const galois_dim* wd, const float* x, const galois_dim* xd,
                        const galois_dim* dd);
// Scratch for the quantised activations in the tensor-core operand layout.
size_t gb_mm_tc_scratch_bytes(const galois_dim* wd, const galois_dim* xd);
// Quantises x into `scratch` and runs the GEMM (two launches).
int gb_mm_q4_0_tc(galois_b200_ctx* ctx, const void* w, const galois_dim* wd, const float* x, const galois_dim* xd, float* dst,
                  const galois_dim* dd, void* scratch);
// Test hook: the same two launches on ONE 128 x 64 tile (N <= 128, B <= 64); the epilogue also stores
// every per-block integer sum it scales: out[(block * 128 + row) * 64 + column], int32.
int gb_mm_q4_0_tc_block_isums(galois_b200_ctx* ctx, const void* w, const galois_dim* wd, const float* x, const galois_dim* xd, float* dst,
                              const galois_dim* dd, void* scratch, int32_t* out);

// One-time repack of a weight for the tensor-core GEMM (the upload step, src/cuda.rs:231-239 of galois): a
// copy of w with the nibbles as unsigned bytes in UMMA operand order and f32 block scales, kept in the
// context under w's device address until released.  Calling it again for the same address refreshes the copy.
int gb_mm_tc_prepare(galois_b200_ctx* ctx, const void* w, const galois_dim* wd);
int gb_mm_tc_release(galois_b200_ctx* ctx, const void* w);
int gb_mm_tc_release_range(galois_b200_ctx* ctx, const void* lo, const void* hi);
void gb_mm_tc_release_all(galois_b200_ctx* ctx);
bool gb_mm_tc_prepared(galois_b200_ctx* ctx, const void* w, const galois_dim* wd);
int gb_mm_tp_bn(const galois_b200_ctx* ctx, int64_t N, int64_t B);
// The GEMM on the prepared copy (quantiser + GEMM, two launches; same scratch as gb_mm_q4_0_tc).
int gb_mm_q4_0_tp(galois_b200_ctx* ctx, const void* w, const galois_dim* wd, const float* x, const galois_dim* xd, float* dst,
                  const galois_dim* dd, void* scratch);
