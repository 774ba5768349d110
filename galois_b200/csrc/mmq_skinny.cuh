// Internal interface of the skinny (2..192 activation rows) Q4_0 mat-mul on mma.sync (mmq_skinny.cu).
#pragma once
#include "common.cuh"
#include "gather.cuh"

// 16 activation rows per pass over the weights; up to 12 passes before the tcgen05 GEMM takes over
// (4096 x 4096: 28 us at 64 rows against 57 us there; the two meet near 200 rows).
constexpr int GB_SKINNY_MAX_BATCH = 192;
// The automatic choice uses this kernel from this many activation rows on (below it: the dp4a GEMV).
constexpr int GB_SKINNY_MIN_BATCH = 2;

// Sets the shared-memory limit of the kernel instances on the current device.
int gb_mmq_skinny_init(galois_b200_ctx* ctx);
// True for 2-D contiguous weights with K % 256 == 0 and a 16-byte aligned base, batch <= 192,
// 16-byte aligned f32 activations.
bool gb_mmq_skinny_supported(const galois_b200_ctx* ctx, const void* w, const galois_dim* wd, const float* x, const galois_dim* xd,
                             const galois_dim* dd);
// Bytes of scratch the two launches share (the quantised activations in fragment order).
size_t gb_mmq_skinny_scratch_bytes(const galois_dim* wd, const galois_dim* xd);
// Two launches per 16 activation rows: the fragment-order Q8_0 quantiser, then the mat-mul.
// `gather` (optional): the call computes one band of a row-sharded mat-mul; `dst` points at the
// band's first row inside this rank's full result, every result also goes to the peers' inboxes and
// each pass's tail receives the peers' rows (protocol of gather.cuh).
int gb_mmq_skinny(galois_b200_ctx* ctx, const void* w, const galois_dim* wd, const float* x, const galois_dim* xd, float* dst,
                  const galois_dim* dd, void* scratch, const gb_gather_args* gather = nullptr);
// Test hook: per-block integer sums as the kernel's mma.sync + magic-number conversion forms them
// (xq in the 34-byte Q8_0 format).
int gb_mmq_skinny_block_isums(galois_b200_ctx* ctx, const void* w, const void* xq, int64_t nb, int32_t* out);
