// Internal interface of the streaming decode GEMV (gemv_q4_0.cu).
#pragma once
#include "common.cuh"
#include "gather.cuh"

// Sets the shared-memory limit of every kernel instance on the current device.
int gb_gemv_init(galois_b200_ctx* ctx);
// True when the streaming GEMV can take this problem: 2-D contiguous weights with 16-byte
// aligned rows (K % 256 == 0), one activation row, 16-byte aligned f32 activations.
bool gb_gemv_supported(const galois_b200_ctx* ctx, const void* w, const galois_dim* wd, const float* x, const galois_dim* xd,
                       const galois_dim* dd);
// One launch: quantises x inside the kernel and runs the GEMV (cluster launch, with programmatic
// dependent launch when the context allows it).  Needs no scratch memory.
int gb_gemv_q4_0(galois_b200_ctx* ctx, const void* w, const galois_dim* wd, const float* x, const galois_dim* xd, float* dst,
                 const galois_dim* dd);
// The same launch for one band of a row-sharded mat-mul: `dst` points at the band's first row
// inside this rank's full result (gather->P.nranks == 0: not sharded).  Each result also goes to
// every peer's inbox and the kernel's tail receives the peers' bands (protocol of gather.cuh).
// `extra` (optional): a residual `res` of the shape of dst (row stride res_nb1): dst = res + mat-mul
// result, the sum rounded once as Add::f rounds it; and, for one activation row, an op pair applied
// to the row before it is quantised (pro_kind 1: rms_norm with `pro_eps` then mul by the gain row
// `pro_aux`; 2: silu then mul by `pro_aux`, laid out like x), rounded as the separate ops round.
struct gb_gemv_extra {
    const float* res;
    int64_t res_nb1;
    int pro_kind;
    const float* pro_aux;
    float pro_eps;
    int epi_kind;  // 1: weight rows 2i / 2i + 1 are gate_i / up_i and dst row i = silu(gate_i . x) * (up_i . x) (dst has N / 2 rows)
};
// gb_gemv_q4_0_gather with epi_kind != 0 on a shape whose row pairs do not share a warp: nothing was launched.
constexpr int GB_GEMV_NO_PAIR_EPILOGUE = 1;
int gb_gemv_q4_0_gather(galois_b200_ctx* ctx, const void* w, const galois_dim* wd, const float* x, const galois_dim* xd, float* dst,
                        const galois_dim* dd, const gb_gather_args* gather, const gb_gemv_extra* extra);
// True when the GEMV was built with the 128-thread CTAs the in-kernel rms_norm needs.
bool gb_gemv_has_prologue();
// Test hook: per-block integer sums as the GEMV's dp4a sequence forms them (nb even, w 4-byte aligned;
// xq in the 34-byte Q8_0 format).
int gb_gemv_block_isums(galois_b200_ctx* ctx, const void* w, const void* xq, int64_t nb, int32_t* out);
// How the one-row GEMV deals the K / 32 blocks of a weight row to the lanes of a warp (segment of `seg`
// block pairs per lane, `split`: several rows per pass, `npass` passes with the activations hoisted into
// registers; npass == 0: not hoisted).  False when the GEMV does not take rows of K elements at all.
bool gb_gemv_row_plan(const galois_b200_ctx* ctx, int64_t K, int* seg, int* split, int* npass);
