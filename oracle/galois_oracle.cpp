// galois_oracle.cpp — CPU restatement of the galois (crate `wwml`) CPU ops that
// define the numerics of the Q4_0 mat-mul / attention-chain path.
//
// THIS IS TEST INFRASTRUCTURE, NOT PRODUCT CODE.  It is the checker the GPU
// kernels are compared against and the CPU baseline the bench times.  Nothing
// in the shipped library may call into it.
//
// PARITY UNPINNED: the reference's own tests hold no numeric assertion, golden
// vector or fixture for any function restated here (its tests only print), and
// the reference (nightly Rust + crates.io dependencies) cannot be compiled in
// this image.  The restatement is pinned only by (a) the reference's source,
// followed line by line and cited below, (b) agreement between its AVX2 path
// and its scalar path, and (c) hand-computed vectors held in tests/golden/.
//
// Third-party arithmetic the reference relies on and how it is restated:
//   * crate `half` 2.3.1 f32<->f16 (IEEE round-to-nearest-even)  -> F16C
//     `_cvtss_sh(x, _MM_FROUND_TO_NEAREST_INT)` / `_cvtsh_ss`, cross-checked by
//     a bit-level software conversion (orc_f32_to_f16_soft).
//   * Rust std f32::{exp,sin,cos,powf,sqrt,round,max,abs} -> glibc libm
//     expf/sinf/cosf/powf/sqrtf/roundf/fmaxf/fabsf.
//   * nightly core::simd f32x32::reduce_sum -> ordered left-to-right sum
//     (simd_reduce_add_ordered).
//   * rayon: scheduling only; restated with std::thread.
//
// Build: g++ -O3 -mavx -mavx2 -mfma -mf16c -ffp-contract=off -pthread -shared -fPIC
// (-ffp-contract=off because rustc never contracts a*b+c on its own).
//
// All `file:line` citations are paths inside the galois repository.

#include <immintrin.h>
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <thread>
#include <vector>

extern "C" {

// Layout descriptor: mirrors `Dim { n_dims, shape, stride }` (src/shape.rs:29-34).
// ggml order: index 0 is the fastest dimension; strides are counted in
// elements, in *blocks* for quantised types (src/shape.rs:422-430).
typedef struct {
    int32_t n_dims;
    int64_t ne[4];
    int64_t nb[4];
} orc_dim;

// src/ggml_quants.rs:140-145  #[repr(C)] BlockQ4_0 { d: f16, qs: [u8; 16] }
typedef struct {
    uint16_t d;
    uint8_t qs[16];
} orc_block_q4_0;
// src/ggml_quants.rs:721-726  #[repr(C)] BlockQ8_0 { d: f16, qs: [i8; 32] }
typedef struct {
    uint16_t d;
    int8_t qs[32];
} orc_block_q8_0;

// BlockQ6K (src/ggml_quants.rs:484-491) and BlockQ8K (:676-682), QK_K = 256
#pragma pack(push, 1)
struct orc_block_q6k {
    uint8_t ql[128];   // low 4 bits
    uint8_t qh[64];    // high 2 bits
    int8_t scales[16]; // one per 16 elements
    uint16_t d;        // f16 super-block scale
};
#pragma pack(pop)
struct orc_block_q8k {
    float d;
    int8_t qs[256];
    int16_t bsums[16];
};
static_assert(sizeof(orc_block_q6k) == 210, "Q6K block is 210 bytes");
static_assert(sizeof(orc_block_q8k) == 292, "Q8K block is 292 bytes");
static_assert(sizeof(orc_block_q4_0) == 18, "Q4_0 block is 18 bytes");
static_assert(sizeof(orc_block_q8_0) == 34, "Q8_0 block is 34 bytes");

// ---------------------------------------------------------------- f16 helpers
static inline uint16_t f32_to_f16(float x) {
    return (uint16_t)_cvtss_sh(x, _MM_FROUND_TO_NEAREST_INT | _MM_FROUND_NO_EXC);
}
static inline float f16_to_f32(uint16_t h) { return _cvtsh_ss(h); }

uint16_t orc_f32_to_f16(float x) { return f32_to_f16(x); }
float orc_f16_to_f32(uint16_t h) { return f16_to_f32(h); }

// Bit-level IEEE-754 binary32 -> binary16, round to nearest even.  Independent
// of F16C; used only to cross-check the intrinsic.
uint16_t orc_f32_to_f16_soft(float x) {
    uint32_t u;
    memcpy(&u, &x, 4);
    uint32_t sign = (u >> 16) & 0x8000u;
    uint32_t em = u & 0x7fffffffu;
    if (em >= 0x7f800000u) {  // inf / nan
        return (uint16_t)(sign | 0x7c00u | ((em > 0x7f800000u) ? (0x0200u | ((em >> 13) & 0x3ffu)) : 0));
    }
    if (em >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u);  // rounds to inf
    if (em < 0x33000001u) return (uint16_t)sign;               // rounds to zero
    int32_t exp = (int32_t)(em >> 23) - 127;
    uint32_t man = (em & 0x7fffffu) | 0x800000u;
    int shift;
    uint32_t base;
    if (exp < -14) {  // subnormal half
        shift = 13 + (-14 - exp);
        base = 0;
    } else {
        shift = 13;
        base = (uint32_t)(exp + 15) << 10;
        man &= 0x7fffffu;
    }
    uint32_t q = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1);
    uint32_t half = 1u << (shift - 1);
    if (rem > half || (rem == half && (q & 1))) q++;
    return (uint16_t)(sign | (base + q));
}

void orc_f32_to_f16_row(const float* x, uint16_t* y, int64_t n) {
    for (int64_t i = 0; i < n; i++) y[i] = f32_to_f16(x[i]);
}
void orc_f16_to_f32_row(const uint16_t* x, float* y, int64_t n) {
    for (int64_t i = 0; i < n; i++) y[i] = f16_to_f32(x[i]);
}

// ------------------------------------------------------------------ RNG
// Synthetic-data generator shared by every test and bench: splitmix64 counter
// stream -> Box-Muller in f64 -> f32.  Not part of the reference (it has no
// data generator); deterministic across machines.
static inline uint64_t splitmix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}
static void fill_normal_range(float* dst, int64_t n, uint64_t base, float mean, float stddev, int64_t i0, int64_t i1) {
    const double two_pi = 6.283185307179586476925286766559;
    for (int64_t i = i0; i < i1; i += 2) {
        uint64_t a = splitmix64(base + (uint64_t)i);
        uint64_t b = splitmix64(base + (uint64_t)i + 1);
        double u1 = ((double)(a >> 11) + 1.0) * (1.0 / 9007199254740992.0);  // (0,1]
        double u2 = (double)(b >> 11) * (1.0 / 9007199254740992.0);          // [0,1)
        double r = sqrt(-2.0 * log(u1));
        dst[i] = (float)((double)mean + (double)stddev * r * cos(two_pi * u2));
        if (i + 1 < n) dst[i + 1] = (float)((double)mean + (double)stddev * r * sin(two_pi * u2));
    }
}
// Element i depends only on (seed, i), so the range is split over threads freely.
void orc_fill_normal(float* dst, int64_t n, uint64_t seed, float mean, float stddev) {
    const uint64_t base = splitmix64(seed ^ 0xD6E8FEB86659FD93ull);
    int nt = (int)std::min<int64_t>(std::max(1u, std::thread::hardware_concurrency()), 16);
    if (n < (1 << 16)) nt = 1;
    const int64_t per = (((n + nt - 1) / nt) + 1) & ~(int64_t)1;  // even chunk starts
    std::vector<std::thread> pool;
    for (int t = 1; t < nt; t++) {
        const int64_t i0 = std::min<int64_t>(n, per * t), i1 = std::min<int64_t>(n, per * (t + 1));
        if (i0 < i1) pool.emplace_back(fill_normal_range, dst, n, base, mean, stddev, i0, i1);
    }
    fill_normal_range(dst, n, base, mean, stddev, 0, std::min<int64_t>(n, per));
    for (auto& th : pool) th.join();
}

// ------------------------------------------------------------------ Q4_0
// The reference has NO Q4_0 quantiser (`<BlockQ4_0 as QuantType>::from_f32` is
// `todo!()`, src/ggml_quants.rs:198-200); weights reach it as raw bytes.  This
// is the scheme the block format's decode `(q-8)*d` (src/ggml_quants.rs:209-228)
// presupposes: the element of largest magnitude, with its sign, maps to -8.
// Parity never depends on it: oracle and GPU consume the same quantised bytes.
void orc_quantize_row_q4_0(const float* x, void* vy, int64_t k) {
    orc_block_q4_0* y = (orc_block_q4_0*)vy;
    const int64_t nb = k / 32;
    for (int64_t i = 0; i < nb; i++) {
        float amax = 0.0f, mx = 0.0f;
        for (int j = 0; j < 32; j++) {
            float v = x[i * 32 + j];
            if (amax < fabsf(v)) {
                amax = fabsf(v);
                mx = v;
            }
        }
        const float d = mx / -8.0f;
        const float id = d != 0.0f ? 1.0f / d : 0.0f;
        y[i].d = f32_to_f16(d);
        for (int j = 0; j < 16; j++) {
            const float x0 = x[i * 32 + j] * id;
            const float x1 = x[i * 32 + 16 + j] * id;
            int q0 = (int)(x0 + 8.5f);
            int q1 = (int)(x1 + 8.5f);
            q0 = q0 < 0 ? 0 : (q0 > 15 ? 15 : q0);
            q1 = q1 < 0 ? 0 : (q1 > 15 ? 15 : q1);
            y[i].qs[j] = (uint8_t)(q0 | (q1 << 4));
        }
    }
}

// src/ggml_quants.rs:209-228  <BlockQ4_0 as QuantType>::to_f32
void orc_dequantize_row_q4_0(const void* vx, float* dst, int64_t k) {
    const orc_block_q4_0* src = (const orc_block_q4_0*)vx;
    const int64_t nb = k / 32;
    for (int64_t i = 0; i < nb; i++) {
        const float d = f16_to_f32(src[i].d);
        for (int j = 0; j < 16; j++) {
            const uint8_t vi = src[i].qs[j];
            const int8_t vi0 = (int8_t)(vi & 0x0F);
            const int8_t vi1 = (int8_t)(vi >> 4);
            dst[i * 32 + j] = (float)(vi0 - 8) * d;
            dst[i * 32 + j + 16] = (float)(vi1 - 8) * d;
        }
    }
}

// ------------------------------------------------------------------ Q8_0
// src/ggml_quants.rs:736-764  <BlockQ8_0 as QuantType>::from_f32
// ("quantize_row_q8_0").  amax via f32::max/abs, d = amax / 127,
// id = 1/d (from the UNROUNDED f32 d), q = f32::round(x*id) as i8
// (round half away from zero; `as i8` saturates but |x*id| <= 127 always).
void orc_quantize_row_q8_0(const float* x, void* vy, int64_t k) {
    orc_block_q8_0* y = (orc_block_q8_0*)vy;
    const int64_t nb = k / 32;
    for (int64_t i = 0; i < nb; i++) {
        float amax = 0.0f;
        const float* xs = x + i * 32;
        for (int j = 0; j < 32; j++) amax = fmaxf(amax, fabsf(xs[j]));
        const float d = amax / 127.0f;
        const float id = d != 0.0f ? 1.0f / d : 0.0f;
        y[i].d = f32_to_f16(d);
        for (int j = 0; j < 32; j++) {
            float r = roundf(xs[j] * id);
            // Rust `as i8` saturates and maps NaN to 0.
            int v = (r != r) ? 0 : (r > 127.0f ? 127 : (r < -128.0f ? -128 : (int)r));
            y[i].qs[j] = (int8_t)v;
        }
    }
}

// ------------------------------------------------------------ Q4_0 . Q8_0 dot
// src/ggml_quants.rs:55-60   sum_i16_pairs_float
static inline __m256 sum_i16_pairs_float(__m256i x) {
    const __m256i ones = _mm256_set1_epi16(1);
    const __m256i summed_pairs = _mm256_madd_epi16(ones, x);
    return _mm256_cvtepi32_ps(summed_pairs);
}
// src/ggml_quants.rs:62-66   mul_sum_us8_pairs_float
static inline __m256 mul_sum_us8_pairs_float(__m256i ax, __m256i sy) {
    const __m256i dot = _mm256_maddubs_epi16(ax, sy);
    return sum_i16_pairs_float(dot);
}
// src/ggml_quants.rs:68-75   hsum_float_8
static inline float hsum_float_8(__m256 x) {
    __m128 res = _mm256_extractf128_ps(x, 1);
    res = _mm_add_ps(res, _mm256_castps256_ps128(x));
    res = _mm_add_ps(res, _mm_movehl_ps(res, res));
    res = _mm_add_ss(res, _mm_movehdup_ps(res));
    return _mm_cvtss_f32(res);
}
// src/ggml_quants.rs:77-83   bytes_from_nibbles_32
static inline __m256i bytes_from_nibbles_32(const uint8_t* rsi) {
    const __m128i tmp = _mm_loadu_si128((const __m128i*)rsi);
    const __m256i bytes = _mm256_insertf128_si256(_mm256_castsi128_si256(tmp), _mm_srli_epi16(tmp, 4), 1);
    const __m256i low_mask = _mm256_set1_epi8(0xF);
    return _mm256_and_si256(low_mask, bytes);
}
// src/ggml_quants.rs:85-90   mul_sum_i8_pairs_float
static inline __m256 mul_sum_i8_pairs_float(__m256i x, __m256i y) {
    const __m256i ax = _mm256_sign_epi8(x, x);
    const __m256i sy = _mm256_sign_epi8(y, x);
    return mul_sum_us8_pairs_float(ax, sy);
}

// src/ggml_quants.rs:156-172   BlockQ4_0::vec_dot_q8_0   (cfg target_feature="avx")
float orc_vec_dot_q4_0_q8_0_avx(const void* vx, const void* vy, int64_t nb) {
    const orc_block_q4_0* x = (const orc_block_q4_0*)vx;
    const orc_block_q8_0* y = (const orc_block_q8_0*)vy;
    __m256 acc = _mm256_setzero_ps();
    for (int64_t i = 0; i < nb; i++) {
        const __m256 d = _mm256_set1_ps(f16_to_f32(x[i].d) * f16_to_f32(y[i].d));
        __m256i bx = bytes_from_nibbles_32(x[i].qs);
        const __m256i off = _mm256_set1_epi8(8);
        bx = _mm256_sub_epi8(bx, off);
        const __m256i by = _mm256_loadu_si256((const __m256i*)y[i].qs);
        const __m256 q = mul_sum_i8_pairs_float(bx, by);
        acc = _mm256_fmadd_ps(d, q, acc);
    }
    return hsum_float_8(acc);
}

// src/ggml_quants.rs:174-191   BlockQ4_0::vec_dot_unopt   (no AVX)
float orc_vec_dot_q4_0_q8_0_scalar(const void* vx, const void* vy, int64_t nb) {
    const orc_block_q4_0* xs = (const orc_block_q4_0*)vx;
    const orc_block_q8_0* ys = (const orc_block_q8_0*)vy;
    float sumf = 0.0f;
    for (int64_t i = 0; i < nb; i++) {
        int32_t sum_i = 0;
        for (int j = 0; j < 16; j++) {
            const int32_t v0 = (int32_t)(xs[i].qs[j] & 0x0F) - 8;
            const int32_t v1 = (int32_t)(xs[i].qs[j] >> 4) - 8;
            sum_i += v0 * (int32_t)ys[i].qs[j] + v1 * (int32_t)ys[i].qs[j + 16];
        }
        sumf += (float)sum_i * f16_to_f32(xs[i].d) * f16_to_f32(ys[i].d);
    }
    return sumf;
}

// Per-block integer sums  sum_j (q4_j - 8) * q8_j  (the quantity that must be
// bit-exact on the GPU).  `via_avx` != 0 derives them from the AVX path's eight
// exact lane sums (src/ggml_quants.rs:163-168), else from the scalar loop
// (src/ggml_quants.rs:180-186).
void orc_block_isums_q4_0_q8_0(const void* vx, const void* vy, int64_t nb, int32_t* out, int via_avx) {
    const orc_block_q4_0* x = (const orc_block_q4_0*)vx;
    const orc_block_q8_0* y = (const orc_block_q8_0*)vy;
    for (int64_t i = 0; i < nb; i++) {
        if (via_avx) {
            __m256i bx = bytes_from_nibbles_32(x[i].qs);
            bx = _mm256_sub_epi8(bx, _mm256_set1_epi8(8));
            const __m256i by = _mm256_loadu_si256((const __m256i*)y[i].qs);
            const __m256 q = mul_sum_i8_pairs_float(bx, by);
            float lanes[8];
            _mm256_storeu_ps(lanes, q);
            int32_t s = 0;
            for (int l = 0; l < 8; l++) s += (int32_t)lanes[l];
            out[i] = s;
        } else {
            int32_t sum_i = 0;
            for (int j = 0; j < 16; j++) {
                const int32_t v0 = (int32_t)(x[i].qs[j] & 0x0F) - 8;
                const int32_t v1 = (int32_t)(x[i].qs[j] >> 4) - 8;
                sum_i += v0 * (int32_t)y[i].qs[j] + v1 * (int32_t)y[i].qs[j + 16];
            }
            out[i] = sum_i;
        }
    }
}

// ------------------------------------------------------------------ f16 dot
// src/op.rs:137-196  vec_dot_f16 (cfg target_feature="avx2"): four 8-lane f32
// accumulators, separate mul and add, ((s0+s1)+(s2+s3)), 128-bit halves,
// movehl, movehdup, scalar tail.
static float vec_dot_f16_avx2(const uint16_t* x, const uint16_t* y, int64_t k) {
    const int64_t n32 = k & ~(int64_t)31;
    __m256 sum0 = _mm256_setzero_ps(), sum1 = _mm256_setzero_ps();
    __m256 sum2 = _mm256_setzero_ps(), sum3 = _mm256_setzero_ps();
    for (int64_t i = 0; i < n32; i += 32) {
        const __m256 x0 = _mm256_cvtph_ps(_mm_loadu_si128((const __m128i*)(x + i + 0)));
        const __m256 x1 = _mm256_cvtph_ps(_mm_loadu_si128((const __m128i*)(x + i + 8)));
        const __m256 x2 = _mm256_cvtph_ps(_mm_loadu_si128((const __m128i*)(x + i + 16)));
        const __m256 x3 = _mm256_cvtph_ps(_mm_loadu_si128((const __m128i*)(x + i + 24)));
        const __m256 y0 = _mm256_cvtph_ps(_mm_loadu_si128((const __m128i*)(y + i + 0)));
        const __m256 y1 = _mm256_cvtph_ps(_mm_loadu_si128((const __m128i*)(y + i + 8)));
        const __m256 y2 = _mm256_cvtph_ps(_mm_loadu_si128((const __m128i*)(y + i + 16)));
        const __m256 y3 = _mm256_cvtph_ps(_mm_loadu_si128((const __m128i*)(y + i + 24)));
        sum0 = _mm256_add_ps(_mm256_mul_ps(x0, y0), sum0);
        sum1 = _mm256_add_ps(_mm256_mul_ps(x1, y1), sum1);
        sum2 = _mm256_add_ps(_mm256_mul_ps(x2, y2), sum2);
        sum3 = _mm256_add_ps(_mm256_mul_ps(x3, y3), sum3);
    }
    const __m256 sum01 = _mm256_add_ps(sum0, sum1);
    const __m256 sum23 = _mm256_add_ps(sum2, sum3);
    const __m256 sum0123 = _mm256_add_ps(sum01, sum23);
    const __m128 r4 = _mm_add_ps(_mm256_castps256_ps128(sum0123), _mm256_extractf128_ps(sum0123, 1));
    const __m128 r2 = _mm_add_ps(r4, _mm_movehl_ps(r4, r4));
    const __m128 r1 = _mm_add_ss(r2, _mm_movehdup_ps(r2));
    float sumf = _mm_cvtss_f32(r1);
    for (int64_t i = n32; i < k; i++) sumf += f16_to_f32(x[i]) * f16_to_f32(y[i]);
    return sumf;
}
// src/op.rs:128-135  vec_dot_f16 without avx2
static float vec_dot_f16_scalar(const uint16_t* x, const uint16_t* y, int64_t k) {
    float res = 0.0f;
    for (int64_t i = 0; i < k; i++) res += f16_to_f32(x[i]) * f16_to_f32(y[i]);
    return res;
}
float orc_vec_dot_f16(const uint16_t* x, const uint16_t* y, int64_t k, int use_avx) {
    return use_avx ? vec_dot_f16_avx2(x, y, k) : vec_dot_f16_scalar(x, y, k);
}

// ------------------------------------------------------------------ Q6K . Q8K
// <BlockQ8K as QuantType>::from_f32 (src/ggml_quants.rs:687-719): per 256 elements, `max` = the first element
// of largest magnitude WITH its sign, iscale = -128 / max, q = min(round(iscale * x), 127) as i8 (a
// saturating cast), bsums = sums of 16 quants, d = 1 / iscale; an all-zero block has d = 0.
void orc_quantize_row_q8k(const float* x, void* vy, int64_t k) {
    orc_block_q8k* y = (orc_block_q8k*)vy;
    for (int64_t i = 0; i < k / 256; i++) {
        const float* xs = x + i * 256;
        float max = 0.0f, amax = 0.0f;
        for (int j = 0; j < 256; j++)
            if (amax < fabsf(xs[j])) amax = fabsf(xs[j]), max = xs[j];
        if (amax == 0.0f) {
            y[i].d = 0.0f;
            memset(y[i].qs, 0, 256);
            // (the reference leaves bsums as they were; a fresh Vec is zeroed)
            memset(y[i].bsums, 0, sizeof(y[i].bsums));
            continue;
        }
        const float iscale = -128.0f / max;
        for (int j = 0; j < 256; j++) {
            const float v = fminf(roundf(iscale * xs[j]), 127.0f);
            y[i].qs[j] = (int8_t)std::max(-128.0f, v);  // `as i8` saturates
        }
        for (int j = 0; j < 16; j++) {
            int sum = 0;
            for (int ii = 0; ii < 16; ii++) sum += y[i].qs[j * 16 + ii];
            y[i].bsums[j] = (int16_t)sum;
        }
        y[i].d = 1.0f / iscale;
    }
}

// The 6-bit quant (0..63) of element e of a super-block, as BlockQ6K::from_f32 packs it
// (src/ggml_quants.rs:543-560): within each half of 128, element l + 32 m (m = 0..3) has its low nibble in
// ql[l + 32 (m & 1)] (low half of the byte for m < 2, high half otherwise) and its top two bits in bits
// 2m .. 2m + 1 of qh[l].
static inline int q6k_quant(const orc_block_q6k& b, int e) {
    const int half = e / 128, r = e % 128, m = r / 32, l = r % 32;
    const uint8_t lo = b.ql[half * 64 + l + 32 * (m & 1)];
    const int nib = m < 2 ? (lo & 0xF) : (lo >> 4);
    const int top = (b.qh[half * 32 + l] >> (2 * m)) & 3;
    return nib | (top << 4);
}

// Element e is d * scales[e / 16] * (q - 32): the decode BlockQ6K::vec_dot presupposes (the reference's
// to_f32 is an empty body, src/ggml_quants.rs:566).
void orc_dequantize_row_q6k(const void* vx, float* dst, int64_t k) {
    const orc_block_q6k* x = (const orc_block_q6k*)vx;
    for (int64_t i = 0; i < k / 256; i++) {
        const float d = f16_to_f32(x[i].d);
        for (int e = 0; e < 256; e++) dst[i * 256 + e] = d * (float)x[i].scales[e / 16] * (float)(q6k_quant(x[i], e) - 32);
    }
}

// A Q6K quantiser for synthetic weights (NOT the reference's make_qx_quants search, src/ggml_quants.rs:235-330,
// 496-563: parity of the mat-mul does not depend on how the bytes were chosen, both sides consume the same
// ones).  Sub-block scale = amax / 31, super-block d = largest sub-block scale / 127.
void orc_quantize_row_q6k(const float* x, void* vy, int64_t k) {
    orc_block_q6k* y = (orc_block_q6k*)vy;
    for (int64_t i = 0; i < k / 256; i++) {
        const float* xs = x + i * 256;
        float sub[16], smax = 0.0f;
        for (int s = 0; s < 16; s++) {
            float a = 0.0f;
            for (int j = 0; j < 16; j++) a = fmaxf(a, fabsf(xs[16 * s + j]));
            sub[s] = a / 31.0f;
            smax = fmaxf(smax, sub[s]);
        }
        memset(&y[i], 0, sizeof(y[i]));
        const float d = smax / 127.0f;
        y[i].d = f32_to_f16(d);
        const float dq = f16_to_f32(y[i].d);
        uint8_t L[256];
        for (int s = 0; s < 16; s++) {
            int sc = dq > 0.0f ? (int)roundf(sub[s] / dq) : 0;
            sc = std::min(127, std::max(sc, dq > 0.0f && sub[s] > 0.0f ? 1 : 0));
            y[i].scales[s] = (int8_t)sc;
            const float step = dq * (float)sc;
            for (int j = 0; j < 16; j++) {
                int q = step > 0.0f ? (int)roundf(xs[16 * s + j] / step) : 0;
                L[16 * s + j] = (uint8_t)(std::min(31, std::max(-32, q)) + 32);
            }
        }
        for (int half = 0; half < 2; half++)
            for (int l = 0; l < 32; l++) {
                const uint8_t* q = L + 128 * half;
                y[i].ql[64 * half + l] = (q[l] & 0xF) | ((q[l + 64] & 0xF) << 4);
                y[i].ql[64 * half + l + 32] = (q[l + 32] & 0xF) | ((q[l + 96] & 0xF) << 4);
                y[i].qh[32 * half + l] = (q[l] >> 4) | ((q[l + 32] >> 4) << 2) | ((q[l + 64] >> 4) << 4) | ((q[l + 96] >> 4) << 6);
            }
    }
}

// BlockQ6K::vec_dot (src/ggml_quants.rs:568-665), AVX2, intrinsic for intrinsic.  get_scale_shuffle(i)
// (:44-53) is row i of a table whose row i holds byte 2i eight times, then byte 2i + 1 eight times.
static inline __m128i q6k_scale_shuffle(int i) {
    return _mm_set_epi8(2 * i + 1, 2 * i + 1, 2 * i + 1, 2 * i + 1, 2 * i + 1, 2 * i + 1, 2 * i + 1, 2 * i + 1, 2 * i, 2 * i, 2 * i, 2 * i,
                        2 * i, 2 * i, 2 * i, 2 * i);
}
float orc_vec_dot_q6k_q8k_avx(const void* vx, const void* vy, int64_t nb) {
    const orc_block_q6k* xs = (const orc_block_q6k*)vx;
    const orc_block_q8k* ys = (const orc_block_q8k*)vy;
    const __m256i m4 = _mm256_set1_epi8(0xF), m2 = _mm256_set1_epi8(3), m32s = _mm256_set1_epi8(32);
    __m256 acc = _mm256_setzero_ps();
    for (int64_t i = 0; i < nb; i++) {
        const float d = ys[i].d * f16_to_f32(xs[i].d);
        const uint8_t* q4 = xs[i].ql;
        const uint8_t* qh = xs[i].qh;
        const int8_t* q8 = ys[i].qs;
        const __m128i scales = _mm_loadu_si128((const __m128i*)xs[i].scales);
        __m256i sumi = _mm256_setzero_si256();
        for (int j = 0; j < 2; j++) {
            const int is = j * 4;
            const __m128i scale_0 = _mm_shuffle_epi8(scales, q6k_scale_shuffle(is));
            const __m128i scale_1 = _mm_shuffle_epi8(scales, q6k_scale_shuffle(is + 1));
            const __m128i scale_2 = _mm_shuffle_epi8(scales, q6k_scale_shuffle(is + 2));
            const __m128i scale_3 = _mm_shuffle_epi8(scales, q6k_scale_shuffle(is + 3));
            const __m256i q4bits1 = _mm256_loadu_si256((const __m256i*)q4);
            q4 += 32;
            const __m256i q4bits2 = _mm256_loadu_si256((const __m256i*)q4);
            q4 += 32;
            const __m256i q4bits_h = _mm256_loadu_si256((const __m256i*)qh);
            qh += 32;
            const __m256i q4h_0 = _mm256_slli_epi16(_mm256_and_si256(q4bits_h, m2), 4);
            const __m256i q4h_1 = _mm256_slli_epi16(_mm256_and_si256(_mm256_srli_epi16(q4bits_h, 2), m2), 4);
            const __m256i q4h_2 = _mm256_slli_epi16(_mm256_and_si256(_mm256_srli_epi16(q4bits_h, 4), m2), 4);
            const __m256i q4h_3 = _mm256_slli_epi16(_mm256_and_si256(_mm256_srli_epi16(q4bits_h, 6), m2), 4);
            const __m256i q4_0 = _mm256_or_si256(_mm256_and_si256(q4bits1, m4), q4h_0);
            const __m256i q4_1 = _mm256_or_si256(_mm256_and_si256(q4bits2, m4), q4h_1);
            const __m256i q4_2 = _mm256_or_si256(_mm256_and_si256(_mm256_srli_epi16(q4bits1, 4), m4), q4h_2);
            const __m256i q4_3 = _mm256_or_si256(_mm256_and_si256(_mm256_srli_epi16(q4bits2, 4), m4), q4h_3);
            const __m256i q8_0 = _mm256_loadu_si256((const __m256i*)q8);
            const __m256i q8_1 = _mm256_loadu_si256((const __m256i*)(q8 + 32));
            const __m256i q8_2 = _mm256_loadu_si256((const __m256i*)(q8 + 64));
            const __m256i q8_3 = _mm256_loadu_si256((const __m256i*)(q8 + 96));
            q8 += 128;
            const __m256i q8s_0 = _mm256_maddubs_epi16(m32s, q8_0), q8s_1 = _mm256_maddubs_epi16(m32s, q8_1);
            const __m256i q8s_2 = _mm256_maddubs_epi16(m32s, q8_2), q8s_3 = _mm256_maddubs_epi16(m32s, q8_3);
            __m256i p16_0 = _mm256_maddubs_epi16(q4_0, q8_0), p16_1 = _mm256_maddubs_epi16(q4_1, q8_1);
            __m256i p16_2 = _mm256_maddubs_epi16(q4_2, q8_2), p16_3 = _mm256_maddubs_epi16(q4_3, q8_3);
            p16_0 = _mm256_sub_epi16(p16_0, q8s_0), p16_1 = _mm256_sub_epi16(p16_1, q8s_1);
            p16_2 = _mm256_sub_epi16(p16_2, q8s_2), p16_3 = _mm256_sub_epi16(p16_3, q8s_3);
            p16_0 = _mm256_madd_epi16(_mm256_cvtepi8_epi16(scale_0), p16_0);
            p16_1 = _mm256_madd_epi16(_mm256_cvtepi8_epi16(scale_1), p16_1);
            p16_2 = _mm256_madd_epi16(_mm256_cvtepi8_epi16(scale_2), p16_2);
            p16_3 = _mm256_madd_epi16(_mm256_cvtepi8_epi16(scale_3), p16_3);
            sumi = _mm256_add_epi32(sumi, _mm256_add_epi32(p16_0, p16_1));
            sumi = _mm256_add_epi32(sumi, _mm256_add_epi32(p16_2, p16_3));
        }
        acc = _mm256_fmadd_ps(_mm256_broadcast_ss(&d), _mm256_cvtepi32_ps(sumi), acc);
    }
    return hsum_float_8(acc);
}

// Per super-block: sum over its 16 sub-blocks of scale * sum (q - 32) * q8, in plain integer arithmetic
// (what the eight i32 lanes of `sumi` above add up to), and with via_avx != 0 the lanes themselves summed.
void orc_block_isums_q6k_q8k(const void* vx, const void* vy, int64_t nb, int32_t* out, int via_avx) {
    const orc_block_q6k* xs = (const orc_block_q6k*)vx;
    const orc_block_q8k* ys = (const orc_block_q8k*)vy;
    for (int64_t i = 0; i < nb; i++) {
        if (!via_avx) {
            int32_t t = 0;
            for (int e = 0; e < 256; e++) t += (int32_t)xs[i].scales[e / 16] * (q6k_quant(xs[i], e) - 32) * (int32_t)ys[i].qs[e];
            out[i] = t;
        } else {
            // run the vector code on this block alone with both scales forced to 1: acc lanes = float(sumi lanes)
            orc_block_q6k x1 = xs[i];
            orc_block_q8k y1 = ys[i];
            x1.d = f32_to_f16(1.0f);
            y1.d = 1.0f;
            // the lanes are exact integers below 2^24 for these magnitudes, and so is their float sum here
            out[i] = (int32_t)orc_vec_dot_q6k_q8k_avx(&x1, &y1, 1);
        }
    }
}

// ------------------------------------------------------------------ mat-mul
// src/op.rs:1383-1598  MatMul::f_q_f32_f32<T>, generic over the weight block
// type T (BlockQ4_0 -> VecDotType BlockQ8_0, block 32; f16 -> VecDotType f16,
// block 1: src/ggml_quants.rs:113-135).
//   1. quantise every activation row to VecDotType, serially (:1398-1420)
//   2. nth = 4 fixed tasks (:1438), split over src0 rows if nr0 > nr1 else over
//      src1 rows (:1491-1492), 16x16 tiling (:1477-1478, :1513-1516)
//   3. dst[i1*nb1 + i2*nb2 + i3*nb3 + ir0] = vec_dot(src0 row, quantised src1 row)
// with src0 broadcast over dims 2/3: i02 = i12 / r2, i03 = i13 / r3 (:1482-1483).
// kind: 0 = Q4_0 weights, 1 = F16 weights, 2 = Q6K weights (VecDotType BlockQ8K, block 256).  use_avx selects
// the vec_dot flavour.
// nth is the task count (4 in the reference); returns 0 or a negative code when
// an assertion of the reference would fire.
static int mul_mat_driver(int kind, const void* w, const orc_dim* wd, const float* x, const orc_dim* xd,
                          float* dst, const orc_dim* dd, int nth, int use_avx) {
    const int64_t ne00 = wd->ne[0], ne01 = wd->ne[1], ne02 = wd->ne[2], ne03 = wd->ne[3];
    const int64_t ne10 = xd->ne[0], ne11 = xd->ne[1], ne12 = xd->ne[2], ne13 = xd->ne[3];
    const int64_t ne0 = dd->ne[0], ne1 = dd->ne[1], ne2 = dd->ne[2], ne3 = dd->ne[3];
    const int64_t nb00 = wd->nb[0], nb01 = wd->nb[1], nb02 = wd->nb[2], nb03 = wd->nb[3];
    const int64_t nb10 = xd->nb[0], nb11 = xd->nb[1], nb12 = xd->nb[2], nb13 = xd->nb[3];
    const int64_t nb0 = dd->nb[0], nb1 = dd->nb[1], nb2 = dd->nb[2], nb3 = dd->nb[3];
    const int64_t block_size = kind == 0 ? 32 : (kind == 2 ? 256 : 1);
    if (ne00 != ne10) return -1;
    if (ne10 % block_size != 0) return -1;                                  // from_f32 panics
    if (!(ne0 == ne01 && ne1 == ne11 && ne2 == ne12 && ne3 == ne13)) return -2;  // :1422-1425
    if (!(nb00 == 1 && nb10 == 1)) return -3;                               // :1428-1429
    if (!(nb0 == 1 && nb0 <= nb1 && nb1 <= nb2 && nb2 <= nb3)) return -4;   // :1432-1435
    if (ne02 == 0 || ne03 == 0 || ne12 % ne02 != 0 || ne13 % ne03 != 0) return -5;  // :1473-1474

    const int64_t row_size = ne10 / block_size;  // VecDotType elements per activation row
    const size_t vd_bytes = kind == 0 ? sizeof(orc_block_q8_0) : (kind == 2 ? sizeof(orc_block_q8k) : sizeof(uint16_t));
    const size_t w_bytes = kind == 0 ? sizeof(orc_block_q4_0) : (kind == 2 ? sizeof(orc_block_q6k) : sizeof(uint16_t));
    std::vector<uint8_t> quant_list((size_t)(ne11 * ne12 * ne13 * row_size) * vd_bytes);
    {
        int64_t idx = 0;
        for (int64_t i13 = 0; i13 < ne13; i13++)
            for (int64_t i12 = 0; i12 < ne12; i12++)
                for (int64_t i11 = 0; i11 < ne11; i11++) {
                    const float* src = x + i13 * nb13 + i12 * nb12 + i11 * nb11;
                    uint8_t* q = quant_list.data() + (size_t)idx * vd_bytes;
                    if (kind == 0)
                        orc_quantize_row_q8_0(src, q, ne10);
                    else if (kind == 2)
                        orc_quantize_row_q8k(src, q, ne10);
                    else
                        orc_f32_to_f16_row(src, (uint16_t*)q, ne10);  // src/ggml_quants.rs:117-122
                    idx += row_size;
                }
    }
    const int64_t blck_0 = 16, blck_1 = 16;
    const int64_t r2 = ne12 / ne02, r3 = ne13 / ne03;
    const int64_t nr0 = ne01, nr1 = ne11 * ne12 * ne13;
    const uint8_t* wbytes = (const uint8_t*)w;

    auto task = [&](int ith) {
        const int64_t nth0 = nr0 > nr1 ? nth : 1;
        const int64_t nth1 = nr0 > nr1 ? 1 : nth;
        const int64_t ith0 = ith % nth0, ith1 = ith / nth0;
        const int64_t dr0 = (nr0 + nth0 - 1) / nth0, dr1 = (nr1 + nth1 - 1) / nth1;
        const int64_t ir010 = dr0 * ith0, ir011 = std::min(ir010 + dr0, nr0);
        const int64_t ir110 = dr1 * ith1, ir111 = std::min(ir110 + dr1, nr1);
        for (int64_t iir1 = ir110; iir1 < ir111; iir1 += blck_1)
            for (int64_t iir0 = ir010; iir0 < ir011; iir0 += blck_0)
                for (int64_t ir1 = iir1; ir1 < std::min(iir1 + blck_1, ir111); ir1++) {
                    const int64_t i13 = ir1 / (ne12 * ne11);
                    const int64_t i12 = (ir1 - i13 * ne12 * ne11) / ne11;
                    const int64_t i11 = ir1 - i13 * ne12 * ne11 - i12 * ne11;
                    const int64_t i03 = i13 / r3, i02 = i12 / r2;
                    const uint8_t* src0 = wbytes + (size_t)(i02 * nb02 + i03 * nb03) * w_bytes;
                    const uint8_t* src1 =
                        quant_list.data() + (size_t)((i11 + i12 * ne11 + i13 * ne12 * ne11) * row_size) * vd_bytes;
                    float* d = dst + i11 * nb1 + i12 * nb2 + i13 * nb3;
                    for (int64_t ir0 = iir0; ir0 < std::min(iir0 + blck_0, ir011); ir0++) {
                        const uint8_t* wrow = src0 + (size_t)(ir0 * nb01) * w_bytes;
                        float v;
                        if (kind == 0)
                            v = use_avx ? orc_vec_dot_q4_0_q8_0_avx(wrow, src1, ne00 / 32)
                                        : orc_vec_dot_q4_0_q8_0_scalar(wrow, src1, ne00 / 32);
                        else if (kind == 2)
                            v = orc_vec_dot_q6k_q8k_avx(wrow, src1, ne00 / 256);  // the reference has no scalar Q6K dot
                        else
                            v = orc_vec_dot_f16((const uint16_t*)wrow, (const uint16_t*)src1, ne00, use_avx);
                        d[ir0] = v;
                    }
                }
    };
    if (nth <= 1) {
        task(0);
    } else {
        std::vector<std::thread> pool;
        for (int t = 1; t < nth; t++) pool.emplace_back(task, t);
        task(0);
        for (auto& t : pool) t.join();
    }
    return 0;
}

int orc_mul_mat_q4_0_f32(const void* w, const orc_dim* wd, const float* x, const orc_dim* xd, float* dst,
                         const orc_dim* dd, int nth, int use_avx) {
    return mul_mat_driver(0, w, wd, x, xd, dst, dd, nth, use_avx);
}
// (Q6K, F32, F32) arm of Map2::map (src/op.rs:3454-3456)
int orc_mul_mat_q6k_f32(const void* w, const orc_dim* wd, const float* x, const orc_dim* xd, float* dst,
                        const orc_dim* dd, int nth, int use_avx) {
    return mul_mat_driver(2, w, wd, x, xd, dst, dd, nth, use_avx);
}
int orc_mul_mat_f16_f32(const void* w, const orc_dim* wd, const float* x, const orc_dim* xd, float* dst,
                        const orc_dim* dd, int nth, int use_avx) {
    return mul_mat_driver(1, w, wd, x, xd, dst, dd, nth, use_avx);
}

// ------------------------------------------------------------- f32 row math
// src/lib.rs:551-562  f32::vec_scale  (f32x32 lanes then scalar tail: each
// element is one f32 multiply either way)
static void vec_scale(int64_t n, float* y, float v) {
    for (int64_t i = 0; i < n; i++) y[i] *= v;
}

// src/lib.rs:594-604  f32::rms_norm ; src/lib.rs:536-540 reduce_sum ;
// row loop src/op.rs:1263-1314.  Only the first ne00 & !31 elements enter the
// sum of squares; each 32-chunk is squared and summed left to right, chunk
// sums are then added sequentially (Iterator::sum from 0.0).
int orc_rms_norm_f32(const float* x, const orc_dim* xd, float* y, const orc_dim* yd, float eps) {
    const int64_t ne00 = xd->ne[0], ne01 = xd->ne[1], ne02 = xd->ne[2], ne03 = xd->ne[3];
    for (int64_t i03 = 0; i03 < ne03; i03++)
        for (int64_t i02 = 0; i02 < ne02; i02++)
            for (int64_t i01 = 0; i01 < ne01; i01++) {
                const float* xr = x + i01 * xd->nb[1] + i02 * xd->nb[2] + i03 * xd->nb[3];
                float* yr = y + i01 * yd->nb[1] + i02 * yd->nb[2] + i03 * yd->nb[3];
                const int64_t n32 = ne00 & ~(int64_t)31;
                float mean = 0.0f;
                for (int64_t c = 0; c < n32; c += 32) {
                    float s = -0.0f;  // simd_reduce_add_ordered(v, -0.)
                    for (int j = 0; j < 32; j++) {
                        const float v = xr[c + j] * xr[c + j];
                        s += v;
                    }
                    mean += s;
                }
                mean /= (float)ne00;
                if (yr != xr) memmove(yr, xr, (size_t)ne00 * sizeof(float));
                const float scale = 1.0f / sqrtf(mean + eps);
                vec_scale(ne00, yr, scale);
            }
    return 0;
}

// src/op.rs:2649-2756  RopeCustom::f_x_y_x  (mode 0 only: neox / glm are todo!())
// theta_scale = powf(freq_base, -2/n_dims) (:2697); per row theta = freq_scale*p
// (:2717); per adjacent pair: cos, sin, zeta, THEN theta *= theta_scale (:2734).
// Note the pair loop runs over all of ne0, not only n_dims (:2721).
int orc_rope_f32(const float* x, const orc_dim* xd, const int32_t* pos, const orc_dim* pd, float* y,
                 const orc_dim* yd, int n_dims, int mode, int n_ctx, float freq_base, float freq_scale,
                 float xpos_base, int xpos_down) {
    (void)pd;
    (void)n_ctx;
    const int64_t ne0 = yd->ne[0], ne1 = yd->ne[1], ne2 = yd->ne[2], ne3 = yd->ne[3];
    if (xd->nb[0] != 1) return -3;                    // :2673
    if (!(n_dims <= ne0 && n_dims % 2 == 0)) return -2;  // :2680-2681
    if (mode & 4) return -6;                          // glm: todo!()
    if (mode & 2) return -6;                          // neox: todo!()
    const float theta_scale = powf(freq_base, -2.0f / (float)n_dims);
    for (int64_t i3 = 0; i3 < ne3; i3++)
        for (int64_t i2 = 0; i2 < ne2; i2++) {
            const float p = (float)pos[i2];
            for (int64_t i1 = 0; i1 < ne1; i1++) {
                float theta = freq_scale * p;
                for (int64_t i0 = 0; i0 < ne0; i0 += 2) {
                    const float cos_theta = cosf(theta);
                    const float sin_theta = sinf(theta);
                    float zeta = xpos_base != 0.0f
                                     ? powf(((float)i0 + 0.4f * (float)ne0) / (1.4f * (float)ne0), p / xpos_base)
                                     : 1.0f;
                    if (xpos_down) zeta = 1.0f / zeta;
                    theta *= theta_scale;
                    const float* src = x + i3 * xd->nb[3] + i2 * xd->nb[2] + i1 * xd->nb[1] + i0 * xd->nb[0];
                    float* d = y + i3 * yd->nb[3] + i2 * yd->nb[2] + i1 * yd->nb[1] + i0 * yd->nb[0];
                    const float x0 = src[0], x1 = src[1];
                    d[0] = x0 * cos_theta * zeta - x1 * sin_theta * zeta;
                    d[1] = x0 * sin_theta * zeta + x1 * cos_theta * zeta;
                }
            }
        }
    return 0;
}

// f16 look-up tables: src/op.rs:227-252 (init_silu_cache, init_exp_cache) with
// compute_silu src/op.rs:88-90.  Entry i = f16( f( f32(f16::from_bits(i)) ) ).
static uint16_t g_exp_lut[65536];
static uint16_t g_silu_lut[65536];
static bool g_lut_ready = false;
static void init_luts() {
    if (g_lut_ready) return;
    for (uint32_t i = 0; i < 65536; i++) {
        const float v = f16_to_f32((uint16_t)i);
        g_exp_lut[i] = f32_to_f16(expf(v));
        g_silu_lut[i] = f32_to_f16(v / (1.0f + expf(-v)));
    }
    g_lut_ready = true;
}
const uint16_t* orc_exp_f16_table(void) {
    init_luts();
    return g_exp_lut;
}
const uint16_t* orc_silu_f16_table(void) {
    init_luts();
    return g_silu_lut;
}

// src/lib.rs:564-592  f32::softmax ; row loop src/op.rs:2917-2977.
// max over the row; -inf inputs give 0; otherwise the argument (x - max) is
// rounded to f16, looked up in the f16 exp table, widened to f32; sequential
// f32 sum; scale by 1/sum.  Returns -7 where the reference asserts sum > 0.
static int softmax_row(int64_t nc, float* dp, const float* sp) {
    init_luts();
    float mx = -INFINITY;
    for (int64_t i = 0; i < nc; i++) mx = fmaxf(mx, sp[i]);
    float sum = 0.0f;
    for (int64_t i = 0; i < nc; i++) {
        if (sp[i] == -INFINITY) {
            dp[i] = 0.0f;
        } else {
            const uint16_t s = f32_to_f16(sp[i] - mx);
            const float val = f16_to_f32(g_exp_lut[s]);
            sum += val;
            dp[i] = val;
        }
    }
    if (!(sum > 0.0f)) return -7;
    sum = 1.0f / sum;
    vec_scale(nc, dp, sum);
    return 0;
}
int orc_soft_max_f32(const float* x, const orc_dim* xd, float* y, const orc_dim* yd) {
    const int64_t nc = xd->ne[0];
    const int64_t nr = xd->ne[1] * xd->ne[2] * xd->ne[3];
    for (int64_t i1 = 0; i1 < nr; i1++) {
        int rc = softmax_row(nc, y + i1 * yd->nb[1], x + i1 * xd->nb[1]);
        if (rc) return rc;
    }
    return 0;
}

// Fused variant with no single counterpart in the reference: equals
// galois_scale (src/op.rs:3258-3279, Scale::f :2369-2409) by `scale`, then
// "set column c > pos[token] to -inf" (the reference has no mask op; its
// softmax maps -inf to 0, src/lib.rs:574-575), then galois_soft_max.
// Rows are [ne0 = columns][ne1 = heads][ne2 = tokens]; pos may be NULL.
int orc_soft_max_ext_f32(const float* x, const orc_dim* xd, float* y, const orc_dim* yd, float scale,
                         const int32_t* pos) {
    const int64_t nc = xd->ne[0];
    std::vector<float> tmp((size_t)nc);
    for (int64_t i3 = 0; i3 < xd->ne[3]; i3++)
        for (int64_t i2 = 0; i2 < xd->ne[2]; i2++)
            for (int64_t i1 = 0; i1 < xd->ne[1]; i1++) {
                const float* sp = x + i1 * xd->nb[1] + i2 * xd->nb[2] + i3 * xd->nb[3];
                float* dp = y + i1 * yd->nb[1] + i2 * yd->nb[2] + i3 * yd->nb[3];
                for (int64_t c = 0; c < nc; c++) {
                    float v = sp[c] * scale;
                    if (pos && c > (int64_t)pos[i2]) v = -INFINITY;
                    tmp[(size_t)c] = v;
                }
                int rc = softmax_row(nc, dp, tmp.data());
                if (rc) return rc;
            }
    return 0;
}

// src/op.rs:2843-2868 Silu::f ; src/lib.rs:543-549 f32::vec_silu (f16 LUT both ways)
int orc_silu_f32(const float* x, const orc_dim* xd, float* y, const orc_dim* yd) {
    init_luts();
    const int64_t nc = xd->ne[0];
    const int64_t nr = xd->ne[1] * xd->ne[2] * xd->ne[3];
    for (int64_t i1 = 0; i1 < nr; i1++)
        for (int64_t i = 0; i < nc; i++)
            y[i1 * yd->nb[1] + i] = f16_to_f32(g_silu_lut[f32_to_f16(x[i1 * xd->nb[1] + i])]);
    return 0;
}

// src/op.rs:318-464 Add::f and src/op.rs:466-611 Mul::f with
// src/lib.rs:606-659 vec_add / vec_mul: dst row ir (dst treated as contiguous
// chunks of ne00, :364-366) = src0 row (op) src1 row, src1 broadcast by modulo
// on dims 1..3 (:371-373).  is_mul: 0 add, 1 mul.
static int add_mul(int is_mul, const float* a, const orc_dim* ad, const float* b, const orc_dim* bd, float* dst,
                   const orc_dim* dd) {
    const int64_t ne00 = ad->ne[0], ne01 = ad->ne[1], ne02 = ad->ne[2], ne03 = ad->ne[3];
    const int64_t ne11 = bd->ne[1], ne12 = bd->ne[2], ne13 = bd->ne[3];
    for (int i = 0; i < 4; i++)
        if (ad->ne[i] != dd->ne[i]) return -2;
    if (!(ad->nb[0] == 1 && dd->nb[0] == 1 && bd->nb[0] == 1)) return -3;
    if (bd->ne[0] < ne00) return -2;  // slice src1[..ne00] would panic
    const int64_t nr = ne01 * ne02 * ne03;
    for (int64_t ir = 0; ir < nr; ir++) {
        const int64_t i03 = ir / (ne02 * ne01);
        const int64_t i02 = (ir - i03 * ne02 * ne01) / ne01;
        const int64_t i01 = ir - i03 * ne02 * ne01 - i02 * ne01;
        const int64_t i13 = i03 % ne13, i12 = i02 % ne12, i11 = i01 % ne11;
        const float* s0 = a + i03 * ad->nb[3] + i02 * ad->nb[2] + i01 * ad->nb[1];
        const float* s1 = b + i13 * bd->nb[3] + i12 * bd->nb[2] + i11 * bd->nb[1];
        float* d = dst + ir * ne00;
        for (int64_t i = 0; i < ne00; i++) d[i] = is_mul ? s0[i] * s1[i] : s0[i] + s1[i];
    }
    return 0;
}
int orc_add_f32(const float* a, const orc_dim* ad, const float* b, const orc_dim* bd, float* dst,
                const orc_dim* dd) {
    return add_mul(0, a, ad, b, bd, dst, dd);
}
int orc_mul_f32(const float* a, const orc_dim* ad, const float* b, const orc_dim* bd, float* dst,
                const orc_dim* dd) {
    return add_mul(1, a, ad, b, bd, dst, dd);
}

// src/op.rs:2369-2409 Scale::f : contiguous src/dst, scalar operand.
int orc_scale_f32(const float* x, const orc_dim* xd, float s, float* y, const orc_dim* yd) {
    const int64_t nc = xd->ne[0];
    const int64_t nr = xd->ne[1] * xd->ne[2] * xd->ne[3];
    for (int64_t i1 = 0; i1 < nr; i1++) {
        float* d = y + i1 * yd->nb[1];
        const float* sp = x + i1 * xd->nb[1];
        if (d != sp) memmove(d, sp, (size_t)nc * sizeof(float));
        vec_scale(nc, d, s);
    }
    return 0;
}

// src/op.rs:1984-2090 Cpy::f_x_y (f32 -> f16, RNE via Y::from_x) and
// src/op.rs:1928-1978 Cpy::f (f32 -> f32).  Source is walked in ggml order
// (i03,i02,i01,i00); the destination is filled in its own ggml order, i.e. the
// k-th source element lands on the k-th logical destination element, which for
// a non-contiguous destination is at i10*nb0 + i11*nb1 + i12*nb2 + i13*nb3.
// to_f16: 0 -> f32 destination, 1 -> f16 destination.
int orc_cpy_f32(const float* x, const orc_dim* xd, void* y, const orc_dim* yd, int to_f16) {
    const int64_t ne00 = xd->ne[0], ne01 = xd->ne[1], ne02 = xd->ne[2], ne03 = xd->ne[3];
    const int64_t ne0 = yd->ne[0], ne1 = yd->ne[1], ne2 = yd->ne[2];
    const int64_t total = ne00 * ne01 * ne02 * ne03;
    if (total != yd->ne[0] * yd->ne[1] * yd->ne[2] * yd->ne[3]) return -2;
    int64_t k = 0;
    for (int64_t i03 = 0; i03 < ne03; i03++)
        for (int64_t i02 = 0; i02 < ne02; i02++)
            for (int64_t i01 = 0; i01 < ne01; i01++)
                for (int64_t i00 = 0; i00 < ne00; i00++, k++) {
                    const float v = x[i00 * xd->nb[0] + i01 * xd->nb[1] + i02 * xd->nb[2] + i03 * xd->nb[3]];
                    const int64_t i10 = k % ne0, i11 = (k / ne0) % ne1, i12 = (k / (ne0 * ne1)) % ne2,
                                  i13 = k / (ne0 * ne1 * ne2);
                    const int64_t o = i10 * yd->nb[0] + i11 * yd->nb[1] + i12 * yd->nb[2] + i13 * yd->nb[3];
                    if (to_f16)
                        ((uint16_t*)y)[o] = f32_to_f16(v);
                    else
                        ((float*)y)[o] = v;
                }
    return 0;
}

int orc_has_avx2(void) { return __builtin_cpu_supports("avx2") && __builtin_cpu_supports("fma") && __builtin_cpu_supports("f16c"); }

}  // extern "C"
