// CPU oracle for the quantized-matmul hot path.  TEST INFRASTRUCTURE ONLY:
// nothing under this directory is part of the shipped library, and the shipped
// library never links, loads or calls it.  It is the checker the parity tests
// hold the CUDA kernels to, and the CPU baseline the benchmark times.
//
// Every function restates, in plain C++ and in the reference's own operation
// order, one function of antonellof/frink v0.63.0.  The citation beside each
// function is the file:line (path inside that project) it follows.  The
// reference is Rust and cannot be compiled where this was written, so the
// restatement is pinned instead by the reference's own golden vectors and
// known-answer tests (tests/golden/, tests/test_oracle_goldens.py).
//
// Build: g++ -O2 -std=c++17 -ffp-contract=off (contraction OFF is load-bearing:
// the reference is Rust, which never fuses a*b+c; where the reference spells
// `mul_add` this file spells fmaf()).
#include <cmath>
#include <cstdint>
#include <cstring>
#include <algorithm>
#include <functional>
#include <thread>
#include <vector>
#if defined(__AVX2__) && defined(__FMA__) && defined(__F16C__)
#include <immintrin.h>
#define FKO_AVX2 1
#else
#define FKO_AVX2 0
#endif

#define FKO_API extern "C" __attribute__((visibility("default")))

namespace {

// ---------------------------------------------------------------- f16 <-> f32
// IEEE binary16, round to nearest even: the `half` crate's semantics, and
// crates/frink-cuda/src/dp4a_twin.rs:34-61 (f32_to_f16_bits).
inline float f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {
            int e = -1;
            do { e++; man <<= 1; } while ((man & 0x400u) == 0);
            man &= 0x3FFu;
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float f;
    std::memcpy(&f, &bits, 4);
    return f;
}

inline uint16_t f32_to_f16(float f) {
    uint32_t u;
    std::memcpy(&u, &f, 4);
    uint32_t sign = (u >> 16) & 0x8000u;
    uint32_t ax = u & 0x7FFFFFFFu;
    uint32_t h;
    if (ax >= 0x7F800000u) {
        h = sign | 0x7C00u | (ax > 0x7F800000u ? 0x0200u : 0u);
    } else if (ax >= 0x477FF000u) {
        h = sign | 0x7C00u;
    } else if (ax < 0x38800000u) {
        if (ax < 0x33000000u) {
            h = sign;
        } else {
            uint32_t m = (ax & 0x7FFFFFu) | 0x800000u;
            uint32_t shift = 126u - (ax >> 23);
            uint32_t k = m >> shift;
            uint32_t rem = m & ((1u << shift) - 1u);
            uint32_t half = 1u << (shift - 1u);
            if (rem > half || (rem == half && (k & 1u))) k++;
            h = sign | k;
        }
    } else {
        uint32_t r = ax - 0x38000000u;
        h = sign | ((r + 0x0FFFu + ((r >> 13) & 1u)) >> 13);
    }
    return (uint16_t)h;
}

inline float f16_at(const uint8_t* p) { return f16_to_f32((uint16_t)(p[0] | (p[1] << 8))); }
inline int32_t i32_at(const uint8_t* p) {
    uint32_t v = (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24);
    return (int32_t)v;
}
inline float f32_from_bits(uint32_t b) { float f; std::memcpy(&f, &b, 4); return f; }

constexpr int Q4K_BYTES = 144, Q5K_BYTES = 176, Q6K_BYTES = 210, Q80_BYTES = 34, MX4_BYTES = 17, Q81_BYTES = 36;

// crates/frink-quant/src/lib.rs:321-330 (q4_k_scale_min)
inline void q4k_scale_min(int j, const uint8_t* s, uint8_t* sc, uint8_t* m) {
    if (j < 4) {
        *sc = s[j] & 63;
        *m = s[j + 4] & 63;
    } else {
        *sc = (uint8_t)((s[j + 4] & 0x0F) | ((s[j - 4] >> 6) << 4));
        *m = (uint8_t)((s[j + 4] >> 4) | ((s[j] >> 6) << 4));
    }
}

// crates/frink-quant/src/lib.rs:4947-4949 (KVALUES_MXFP4) and :4960-4966 (e8m0_scale)
const float KV_MXFP4[16] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f,
                            -0.0f, -0.5f, -1.0f, -1.5f, -2.0f, -3.0f, -4.0f, -6.0f};
inline float e8m0_scale(uint8_t e) { return e == 0 ? f32_from_bits(0x00400000u) : f32_from_bits((uint32_t)e << 23); }
// crates/frink-quant/src/legacy_q8.rs:149 (KVALUES_MXFP4_X2) and :154-160 (e8m0_to_fp32_half)
const int8_t KV_MXFP4_X2[16] = {0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12};
inline float e8m0_half(uint8_t e) { return e < 2 ? f32_from_bits(0x00200000u << e) : f32_from_bits((uint32_t)(e - 1) << 23); }

// ------------------------------------------------------------ block decoding
// One block of `kind` into its f32 values.  Q4_K lib.rs:334-364, Q6_K
// lib.rs:519-552, Q8_0 lib.rs:271-286, GGUF MXFP4 lib.rs:5576-5582.
void decode_q4_k(const uint8_t* b, float* y) {
    float d = f16_at(b), dmin = f16_at(b + 2);
    const uint8_t* scales = b + 4;
    const uint8_t* qs = b + 16;
    int is = 0, q_off = 0, o = 0;
    for (int it = 0; it < 4; it++) {
        uint8_t sc1, m1, sc2, m2;
        q4k_scale_min(is, scales, &sc1, &m1);
        q4k_scale_min(is + 1, scales, &sc2, &m2);
        float d1 = d * (float)sc1, min1 = dmin * (float)m1;
        float d2 = d * (float)sc2, min2 = dmin * (float)m2;
        for (int l = 0; l < 32; l++) y[o++] = d1 * (float)(qs[q_off + l] & 0x0F) - min1;
        for (int l = 0; l < 32; l++) y[o++] = d2 * (float)(qs[q_off + l] >> 4) - min2;
        q_off += 32;
        is += 2;
    }
}

// The 256 five-bit codes (0..31) of one Q5_K block, in element order: the low four bits as Q4_K's nibbles, the fifth
// from qh, whose 32 bytes serve all four 64-element groups at bit positions 2g (low nibbles) and 2g + 1 (high).
// crates/frink-quant/src/lib.rs:424-460.
void q5k_codes(const uint8_t* b, uint8_t* q) {
    const uint8_t* qh = b + 16;
    const uint8_t* qs = b + 48;
    for (int g = 0; g < 4; g++)
        for (int l = 0; l < 32; l++) {
            q[64 * g + l] = (uint8_t)((qs[32 * g + l] & 0x0F) + (((qh[l] >> (2 * g)) & 1) << 4));
            q[64 * g + 32 + l] = (uint8_t)((qs[32 * g + l] >> 4) + (((qh[l] >> (2 * g + 1)) & 1) << 4));
        }
}

void decode_q5_k(const uint8_t* b, float* y) {
    uint8_t q[256];
    q5k_codes(b, q);
    float d = f16_at(b), dmin = f16_at(b + 2);
    for (int j = 0; j < 8; j++) {
        uint8_t sc, m;
        q4k_scale_min(j, b + 4, &sc, &m);
        float dj = d * (float)sc, mj = dmin * (float)m;
        for (int l = 0; l < 32; l++) y[32 * j + l] = dj * (float)q[32 * j + l] - mj;
    }
}

// The 256 signed 6-bit codes (-32..31) of one Q6_K block, in element order.
void q6k_codes(const uint8_t* b, int8_t* q) {
    for (int half = 0; half < 2; half++) {
        const uint8_t* ql = b + half * 64;
        const uint8_t* qh = b + 128 + half * 32;
        int8_t* y = q + half * 128;
        for (int l = 0; l < 32; l++) {
            y[l] = (int8_t)((ql[l] & 0x0F) | ((qh[l] & 3) << 4)) - 32;
            y[l + 32] = (int8_t)((ql[l + 32] & 0x0F) | (((qh[l] >> 2) & 3) << 4)) - 32;
            y[l + 64] = (int8_t)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
            y[l + 96] = (int8_t)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
        }
    }
}

void decode_q6_k(const uint8_t* b, float* y) {
    int8_t q[256];
    q6k_codes(b, q);
    float d = f16_at(b + 208);
    for (int half = 0; half < 2; half++) {
        const int8_t* sc = (const int8_t*)(b + 192 + half * 8);
        for (int l = 0; l < 32; l++) {
            int is = l / 16;
            int o = half * 128 + l;
            y[o] = d * (float)sc[is] * (float)q[o];
            y[o + 32] = d * (float)sc[is + 2] * (float)q[o + 32];
            y[o + 64] = d * (float)sc[is + 4] * (float)q[o + 64];
            y[o + 96] = d * (float)sc[is + 6] * (float)q[o + 96];
        }
    }
}

void decode_q8_0(const uint8_t* b, float* y) {
    float scale = f16_at(b);
    for (int i = 0; i < 32; i++) y[i] = (float)(int8_t)b[2 + i] * scale;
}

void decode_mxfp4(const uint8_t* b, float* y) {
    float d = e8m0_scale(b[0]);
    for (int j = 0; j < 16; j++) {
        y[j] = d * KV_MXFP4[b[1 + j] & 0x0F];
        y[j + 16] = d * KV_MXFP4[b[1 + j] >> 4];
    }
}

// BF16: the upper half of an f32 (crates/frink-quant/src/lib.rs:232-250); a "block" is one value.
void decode_bf16(const uint8_t* b, float* y) { y[0] = f32_from_bits((uint32_t)(b[0] | (b[1] << 8)) << 16); }

struct KindInfo { int block_bytes, block_elems; void (*decode)(const uint8_t*, float*); };
// ggml type tags: Q8_0 = 8, Q4_K = 12, Q5_K = 13, Q6_K = 14, MXFP4 = 39.
bool kind_info(int kind, KindInfo* k) {
    switch (kind) {
        case 12: *k = {Q4K_BYTES, 256, decode_q4_k}; return true;
        case 13: *k = {Q5K_BYTES, 256, decode_q5_k}; return true;
        case 14: *k = {Q6K_BYTES, 256, decode_q6_k}; return true;
        case 8: *k = {Q80_BYTES, 32, decode_q8_0}; return true;
        case 39: *k = {MX4_BYTES, 32, decode_mxfp4}; return true;
        case 30: *k = {2, 1, decode_bf16}; return true;
    }
    return false;
}

// ------------------------------------------------- L0: fused f32 dots, scalar
// crates/frink-quant/src/lib.rs:386-415
float dot_q4_k_f32_scalar(const uint8_t* row, int nblk, const float* x) {
    float acc = 0.0f;
    int base = 0;
    for (int b = 0; b < nblk; b++) {
        const uint8_t* blk = row + (size_t)b * Q4K_BYTES;
        float d = f16_at(blk), dmin = f16_at(blk + 2);
        const uint8_t* scales = blk + 4;
        const uint8_t* qs = blk + 16;
        int is = 0, q_off = 0;
        for (int it = 0; it < 4; it++) {
            uint8_t sc1, m1, sc2, m2;
            q4k_scale_min(is, scales, &sc1, &m1);
            q4k_scale_min(is + 1, scales, &sc2, &m2);
            float d1 = d * (float)sc1, min1 = dmin * (float)m1;
            float d2 = d * (float)sc2, min2 = dmin * (float)m2;
            for (int l = 0; l < 32; l++) acc += (d1 * (float)(qs[q_off + l] & 0x0F) - min1) * x[base + l];
            for (int l = 0; l < 32; l++) acc += (d2 * (float)(qs[q_off + l] >> 4) - min2) * x[base + 32 + l];
            q_off += 32;
            base += 64;
            is += 2;
        }
    }
    return acc;
}

// crates/frink-quant/src/lib.rs:481-515: the dequantized value times x, accumulated in element order
float dot_q5_k_f32_scalar(const uint8_t* row, int nblk, const float* x) {
    float acc = 0.0f;
    uint8_t q[256];
    for (int b = 0; b < nblk; b++) {
        const uint8_t* blk = row + (size_t)b * Q5K_BYTES;
        q5k_codes(blk, q);
        float d = f16_at(blk), dmin = f16_at(blk + 2);
        for (int j = 0; j < 8; j++) {
            uint8_t sc, m;
            q4k_scale_min(j, blk + 4, &sc, &m);
            float dj = d * (float)sc, mj = dmin * (float)m;
            for (int l = 0; l < 32; l++) acc += (dj * (float)q[32 * j + l] - mj) * x[b * 256 + 32 * j + l];
        }
    }
    return acc;
}

// crates/frink-quant/src/lib.rs:574-605
float dot_q6_k_f32_scalar(const uint8_t* row, int nblk, const float* x) {
    float acc = 0.0f;
    int x_base = 0;
    for (int b = 0; b < nblk; b++) {
        const uint8_t* blk = row + (size_t)b * Q6K_BYTES;
        float d = f16_at(blk + 208);
        for (int half = 0; half < 2; half++) {
            const uint8_t* ql = blk + half * 64;
            const uint8_t* qh = blk + 128 + half * 32;
            const int8_t* sc = (const int8_t*)(blk + 192 + half * 8);
            const float* xh = x + x_base;
            for (int l = 0; l < 32; l++) {
                int is = l / 16;
                int8_t q1 = (int8_t)((ql[l] & 0x0F) | ((qh[l] & 3) << 4)) - 32;
                int8_t q2 = (int8_t)((ql[l + 32] & 0x0F) | (((qh[l] >> 2) & 3) << 4)) - 32;
                int8_t q3 = (int8_t)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
                int8_t q4 = (int8_t)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
                acc += d * (float)sc[is] * (float)q1 * xh[l];
                acc += d * (float)sc[is + 2] * (float)q2 * xh[l + 32];
                acc += d * (float)sc[is + 4] * (float)q3 * xh[l + 64];
                acc += d * (float)sc[is + 6] * (float)q4 * xh[l + 96];
            }
            x_base += 128;
        }
    }
    return acc;
}

// crates/frink-quant/src/lib.rs:663-686
float dot_q8_0_f32_scalar(const uint8_t* row, int nblk, const float* x) {
    float acc = 0.0f;
    for (int b = 0; b < nblk; b++) {
        const uint8_t* blk = row + (size_t)b * Q80_BYTES;
        float scale = f16_at(blk);
        float block_acc = 0.0f;
        for (int i = 0; i < 32; i++) block_acc += (float)(int8_t)blk[2 + i] * x[b * 32 + i];
        acc += block_acc * scale;
    }
    return acc;
}

// crates/frink-quant/src/lib.rs:5421-5447 with the walk at :5576-5582
float dot_mxfp4_f32_scalar(const uint8_t* row, int nblk, const float* x) {
    float acc = 0.0f;
    for (int b = 0; b < nblk; b++) {
        const uint8_t* blk = row + (size_t)b * MX4_BYTES;
        float d = e8m0_scale(blk[0]);
        for (int j = 0; j < 16; j++) {
            acc += d * KV_MXFP4[blk[1 + j] & 0x0F] * x[b * 32 + j];
            acc += d * KV_MXFP4[blk[1 + j] >> 4] * x[b * 32 + j + 16];
        }
    }
    return acc;
}

float dot_f32_scalar(int kind, const uint8_t* row, int nblk, const float* x) {
    switch (kind) {
        case 12: return dot_q4_k_f32_scalar(row, nblk, x);
        case 13: return dot_q5_k_f32_scalar(row, nblk, x);
        case 14: return dot_q6_k_f32_scalar(row, nblk, x);
        case 8: return dot_q8_0_f32_scalar(row, nblk, x);
        case 39: return dot_mxfp4_f32_scalar(row, nblk, x);
    }
    return NAN;
}

#if FKO_AVX2
// The x86 production decode kernel for Q4_K: the AVX2+FMA form of the fused
// dot (crates/frink-quant/src/lib.rs:1412; dispatched at :370-384).  Eight
// lanes of f32, nibbles widened through epi32, one FMA per 8 weights:
// value = (d*sc)*nib - dmin*m, accumulated as fma(value, x, acc).
inline float hsum256(__m256 v) {
    __m128 lo = _mm256_castps256_ps128(v), hi = _mm256_extractf128_ps(v, 1);
    lo = _mm_add_ps(lo, hi);
    lo = _mm_hadd_ps(lo, lo);
    lo = _mm_hadd_ps(lo, lo);
    return _mm_cvtss_f32(lo);
}
float dot_q4_k_f32_avx2(const uint8_t* row, int nblk, const float* x) {
    __m256 acc = _mm256_setzero_ps();
    const __m128i mask = _mm_set1_epi8(0x0F);
    int base = 0;
    for (int b = 0; b < nblk; b++) {
        const uint8_t* blk = row + (size_t)b * Q4K_BYTES;
        float d = f16_at(blk), dmin = f16_at(blk + 2);
        const uint8_t* scales = blk + 4;
        const uint8_t* qs = blk + 16;
        for (int it = 0; it < 4; it++) {
            uint8_t sc1, m1, sc2, m2;
            q4k_scale_min(2 * it, scales, &sc1, &m1);
            q4k_scale_min(2 * it + 1, scales, &sc2, &m2);
            __m256 d1 = _mm256_set1_ps(d * (float)sc1), n1 = _mm256_set1_ps(dmin * (float)m1);
            __m256 d2 = _mm256_set1_ps(d * (float)sc2), n2 = _mm256_set1_ps(dmin * (float)m2);
            for (int l = 0; l < 32; l += 8) {
                __m128i raw = _mm_loadl_epi64((const __m128i*)(qs + 32 * it + l));
                __m128i lo8 = _mm_and_si128(raw, mask);
                __m128i hi8 = _mm_and_si128(_mm_srli_epi16(raw, 4), mask);
                __m256 lo = _mm256_cvtepi32_ps(_mm256_cvtepu8_epi32(lo8));
                __m256 hi = _mm256_cvtepi32_ps(_mm256_cvtepu8_epi32(hi8));
                __m256 w1 = _mm256_fmsub_ps(d1, lo, n1);
                __m256 w2 = _mm256_fmsub_ps(d2, hi, n2);
                acc = _mm256_fmadd_ps(w1, _mm256_loadu_ps(x + base + l), acc);
                acc = _mm256_fmadd_ps(w2, _mm256_loadu_ps(x + base + 32 + l), acc);
            }
            base += 64;
        }
    }
    return hsum256(acc);
}
#endif

// f64 dequantize-then-dot: the "exact" reference the fp32 tolerance is taken
// against (crates/frink-cuda/src/dp4a_twin.rs:402-440 uses the same shape).
double dot_dequant_f64(int kind, const uint8_t* row, int nblk, const float* x) {
    KindInfo k;
    if (!kind_info(kind, &k)) return NAN;
    float w[256];
    double acc = 0.0;
    for (int b = 0; b < nblk; b++) {
        k.decode(row + (size_t)b * k.block_bytes, w);
        for (int i = 0; i < k.block_elems; i++) acc += (double)w[i] * (double)x[(size_t)b * k.block_elems + i];
    }
    return acc;
}

// -------------------------------------------- CPU activation quantizers (L2)
// crates/frink-quant/src/act_quant.rs:69-104 (quantize_activations_q8_k)
inline float round_ties_even(float v) { return std::nearbyintf(v); }  // default FE_TONEAREST
void quantize_q8_k(const float* x, int n, int8_t* q, float* d, int16_t* bsums) {
    int nb = n / 256;
    std::memset(q, 0, (size_t)n);
    for (int b = 0; b < nb; b++) {
        const float* c = x + (size_t)b * 256;
        d[b] = 0.0f;
        for (int i = 0; i < 16; i++) bsums[b * 16 + i] = 0;
        float amax = 0.0f;
        for (int i = 0; i < 256; i++) amax = std::fmax(amax, std::fabs(c[i]));
        if (amax == 0.0f) continue;
        float iscale = 127.0f / amax;
        for (int i = 0; i < 256; i++) {
            float r = round_ties_even(iscale * c[i]);
            r = std::fmin(std::fmax(r, -127.0f), 127.0f);
            q[(size_t)b * 256 + i] = (int8_t)r;
        }
        d[b] = 1.0f / iscale;
        for (int g = 0; g < 16; g++) {
            int s = 0;
            for (int i = 0; i < 16; i++) s += q[(size_t)b * 256 + g * 16 + i];
            bsums[b * 16 + g] = (int16_t)s;
        }
    }
}

// crates/frink-quant/src/act_quant.rs:157-189 (quantize_q8_0_as); form 0 = NEON,
// 1 = AVX (what an x86 host with AVX runs), 2 = scalar.
void quantize_q8_0_act(const float* x, int n, int form, int8_t* q, float* d) {
    int nb = n / 32;
    for (int b = 0; b < nb; b++) {
        const float* c = x + (size_t)b * 32;
        float amax = 0.0f;
        for (int i = 0; i < 32; i++) amax = std::fmax(amax, std::fabs(c[i]));
        float scale = amax / 127.0f;
        float inv = 0.0f;
        if (form == 1) { if (amax != 0.0f) inv = 127.0f / amax; }
        else { if (scale != 0.0f) inv = 1.0f / scale; }
        d[b] = f16_to_f32(f32_to_f16(scale));
        for (int i = 0; i < 32; i++) {
            float scaled = c[i] * inv;
            float r = (form == 2) ? std::roundf(scaled) : round_ties_even(scaled);
            r = std::fmin(std::fmax(r, -127.0f), 127.0f);
            q[(size_t)b * 32 + i] = (int8_t)r;
        }
    }
}

// ------------------------------------------------- L2: CPU integer vec_dots
// crates/frink-quant/src/lib.rs:822-869
float dot_q4_k_q8k(const uint8_t* row, int nblk, const int8_t* aq, const float* ad, const int16_t* bs) {
    float acc = 0.0f;
    for (int b = 0; b < nblk; b++) {
        const uint8_t* blk = row + (size_t)b * Q4K_BYTES;
        float d = f16_at(blk), dmin = f16_at(blk + 2);
        const uint8_t* scales = blk + 4;
        const uint8_t* qs = blk + 16;
        float da = ad[b];
        const int8_t* q8 = aq + (size_t)b * 256;
        const int16_t* bsums = bs + b * 16;
        int sum_min = 0;
        for (int i = 0; i < 8; i++) {
            uint8_t sc, m;
            q4k_scale_min(i, scales, &sc, &m);
            sum_min += (int)m * ((int)bsums[2 * i] + (int)bsums[2 * i + 1]);
        }
        acc -= dmin * da * (float)sum_min;
        int q_off = 0, base = 0, is = 0;
        for (int it = 0; it < 4; it++) {
            uint8_t sc1, sc2, m;
            q4k_scale_min(is, scales, &sc1, &m);
            q4k_scale_min(is + 1, scales, &sc2, &m);
            int isum1 = 0, isum2 = 0;
            for (int l = 0; l < 32; l++) isum1 += (int)(qs[q_off + l] & 0x0F) * (int)q8[base + l];
            for (int l = 0; l < 32; l++) isum2 += (int)(qs[q_off + l] >> 4) * (int)q8[base + 32 + l];
            acc += d * da * ((float)sc1 * (float)isum1 + (float)sc2 * (float)isum2);
            q_off += 32;
            base += 64;
            is += 2;
        }
    }
    return acc;
}

// crates/frink-quant/src/lib.rs:886-939
float dot_q5_k_q8k(const uint8_t* row, int nblk, const int8_t* aq, const float* ad, const int16_t* bs) {
    float acc = 0.0f;
    uint8_t q[256];
    for (int b = 0; b < nblk; b++) {
        const uint8_t* blk = row + (size_t)b * Q5K_BYTES;
        q5k_codes(blk, q);
        float d = f16_at(blk), dmin = f16_at(blk + 2);
        float da = ad[b];
        const int8_t* q8 = aq + (size_t)b * 256;
        const int16_t* bsums = bs + b * 16;
        int sum_min = 0;
        for (int i = 0; i < 8; i++) {
            uint8_t sc, m;
            q4k_scale_min(i, blk + 4, &sc, &m);
            sum_min += (int)m * ((int)bsums[2 * i] + (int)bsums[2 * i + 1]);
        }
        acc -= dmin * da * (float)sum_min;
        for (int it = 0; it < 4; it++) {
            uint8_t sc1, sc2, m;
            q4k_scale_min(2 * it, blk + 4, &sc1, &m);
            q4k_scale_min(2 * it + 1, blk + 4, &sc2, &m);
            int isum1 = 0, isum2 = 0;
            for (int l = 0; l < 32; l++) isum1 += (int)q[64 * it + l] * (int)q8[64 * it + l];
            for (int l = 0; l < 32; l++) isum2 += (int)q[64 * it + 32 + l] * (int)q8[64 * it + 32 + l];
            acc += d * da * ((float)sc1 * (float)isum1 + (float)sc2 * (float)isum2);
        }
    }
    return acc;
}

// crates/frink-quant/src/lib.rs:1069-1110
float dot_q6_k_q8k(const uint8_t* row, int nblk, const int8_t* aq, const float* ad) {
    float acc = 0.0f;
    int8_t q[256];
    for (int b = 0; b < nblk; b++) {
        const uint8_t* blk = row + (size_t)b * Q6K_BYTES;
        float d = f16_at(blk + 208);
        float da = ad[b];
        const int8_t* q8 = aq + (size_t)b * 256;
        q6k_codes(blk, q);
        int isum = 0;
        for (int half = 0; half < 2; half++) {
            const int8_t* sc = (const int8_t*)(blk + 192 + half * 8);
            for (int l = 0; l < 32; l++) {
                int is = l / 16;
                int o = half * 128 + l;
                isum += (int)sc[is] * (int)q[o] * (int)q8[o];
                isum += (int)sc[is + 2] * (int)q[o + 32] * (int)q8[o + 32];
                isum += (int)sc[is + 4] * (int)q[o + 64] * (int)q8[o + 64];
                isum += (int)sc[is + 6] * (int)q[o + 96] * (int)q8[o + 96];
            }
        }
        acc += d * da * (float)isum;
    }
    return acc;
}

// crates/frink-quant/src/lib.rs:711-733
float dot_q8_0_q8(const uint8_t* row, int nblk, const int8_t* aq, const float* ad) {
    float acc = 0.0f;
    for (int b = 0; b < nblk; b++) {
        const uint8_t* blk = row + (size_t)b * Q80_BYTES;
        float dw = f16_at(blk);
        int isum = 0;
        for (int i = 0; i < 32; i++) isum += (int)(int8_t)blk[2 + i] * (int)aq[(size_t)b * 32 + i];
        acc += dw * ad[b] * (float)isum;
    }
    return acc;
}

// crates/frink-quant/src/legacy_q8.rs:168-184 with the Mxfp4 block at :134-147
float dot_mxfp4_q8(const uint8_t* row, int nblk, const int8_t* aq, const float* ad) {
    float acc = 0.0f;
    for (int b = 0; b < nblk; b++) {
        const uint8_t* blk = row + (size_t)b * MX4_BYTES;
        const int8_t* y = aq + (size_t)b * 32;
        int isum = 0;
        // decode order j, j+16; the sum walks elements 0..31 in order
        int8_t w[32];
        for (int j = 0; j < 16; j++) {
            w[j] = KV_MXFP4_X2[blk[1 + j] & 0xF];
            w[j + 16] = KV_MXFP4_X2[blk[1 + j] >> 4];
        }
        for (int i = 0; i < 32; i++) isum += (int)w[i] * (int)y[i];
        float block_acc = e8m0_half(blk[0]) * (float)isum;
        acc += ad[b] * block_acc;
    }
    return acc;
}

// ------------------------------------------- L1: the q8_1 decode quantizer
// crates/frink-cuda/src/dp4a_twin.rs:78-108 (quantize_q8_1): per 32 values,
// amax and the f32 sum through the xor butterfly, d = amax/127 stored as f16,
// q = roundf(x / d) with the unrounded f32 d.
void butterfly32(float* lanes, bool is_max) {
    static const int offs[5] = {16, 8, 4, 2, 1};
    for (int oi = 0; oi < 5; oi++) {
        float prev[32];
        std::memcpy(prev, lanes, sizeof(prev));
        for (int l = 0; l < 32; l++) {
            float a = prev[l], b = prev[l ^ offs[oi]];
            lanes[l] = is_max ? std::fmax(a, b) : a + b;
        }
    }
}

void quantize_q8_1(const float* x, int n, uint8_t* out) {
    int nb = n / 32;
    for (int b = 0; b < nb; b++) {
        const float* blk = x + (size_t)b * 32;
        uint8_t* o = out + (size_t)b * Q81_BYTES;
        float a[32], v[32];
        for (int l = 0; l < 32; l++) { a[l] = std::fabs(blk[l]); v[l] = blk[l]; }
        butterfly32(a, true);
        butterfly32(v, false);
        float amax = a[0], sum = v[0];
        float d = amax / 127.0f;
        uint16_t dh = f32_to_f16(d), sh = f32_to_f16(sum);
        o[0] = dh & 0xFF; o[1] = dh >> 8; o[2] = sh & 0xFF; o[3] = sh >> 8;
        for (int l = 0; l < 32; l++) {
            int q = (amax == 0.0f) ? 0 : (int)std::roundf(blk[l] / d);
            o[4 + l] = (uint8_t)(int8_t)q;
        }
    }
}

// crates/frink-cuda/src/dp4a_twin.rs:113-130 (q8_1_dequant / q8_1_round)
void q8_1_dequant(const uint8_t* y, int nb, float* out) {
    for (int b = 0; b < nb; b++) {
        const uint8_t* blk = y + (size_t)b * Q81_BYTES;
        float d = f16_at(blk);
        for (int i = 0; i < 32; i++) out[(size_t)b * 32 + i] = (float)(int8_t)blk[4 + i] * d;
    }
}

// crates/frink-cuda/src/dp4a_twin.rs:133-139 (dp4a)
inline int32_t dp4a(int32_t a, int32_t b, int32_t c) {
    for (int i = 0; i < 4; i++) {
        int8_t ab = (int8_t)((uint32_t)a >> (8 * i));
        int8_t bb = (int8_t)((uint32_t)b >> (8 * i));
        c = (int32_t)((uint32_t)c + (uint32_t)((int32_t)ab * (int32_t)bb));
    }
    return c;
}

// crates/frink-cuda/src/dp4a_twin.rs:142-166 (vec_dot_q4_k)
float vec_dot_q4_k(const uint8_t* blk, const uint8_t* y, int iqs) {
    int bq8_offset = 2 * ((iqs / 2) / 4);
    int r = (iqs / 2) % 4;
    int q4 = 16 + 16 * bq8_offset + 4 * r;
    int32_t v0 = i32_at(blk + q4), v1 = i32_at(blk + q4 + 16);
    const uint8_t* scales = blk + 4;
    float sumf_d = 0.0f, sumf_m = 0.0f;
    for (int i = 0; i < 2; i++) {
        uint8_t sc, m;
        q4k_scale_min(bq8_offset + i, scales, &sc, &m);
        const uint8_t* b8 = y + (size_t)(bq8_offset + i) * Q81_BYTES;
        float d8 = f16_at(b8);
        int32_t u0 = i32_at(b8 + 4 + 4 * r), u1 = i32_at(b8 + 4 + 16 + 4 * r);
        int32_t v0i = (v0 >> (4 * i)) & 0x0F0F0F0F, v1i = (v1 >> (4 * i)) & 0x0F0F0F0F;
        int32_t dot1 = dp4a(v1i, u1, dp4a(v0i, u0, 0));
        int32_t dot2 = dp4a(0x01010101, u1, dp4a(0x01010101, u0, 0));
        sumf_d += d8 * (float)(dot1 * (int32_t)sc);
        sumf_m += d8 * (float)(dot2 * (int32_t)m);
    }
    return f16_at(blk) * sumf_d - f16_at(blk + 2) * sumf_m;
}

// crates/frink-cuda/src/dp4a_twin.rs:170-194 (vec_dot_q6_k)
float vec_dot_q6_k(const uint8_t* blk, const uint8_t* y, int iqs) {
    int bq8_offset = 4 * (iqs / 16) + (iqs % 16) / 8;
    int scale_offset = 8 * (iqs / 16) + (iqs % 16) / 4;
    int vh_shift = 2 * ((iqs % 16) / 8);
    uint32_t vl[2], vh[2];
    for (int j = 0; j < 2; j++) {
        vl[j] = (uint32_t)i32_at(blk + 4 * (iqs + j));
        vh[j] = (uint32_t)i32_at(blk + 128 + 4 * (8 * (iqs / 16) + iqs % 8 + j)) >> vh_shift;
    }
    float sumf = 0.0f;
    for (int i = 0; i < 2; i++) {
        const uint8_t* b8 = y + (size_t)(bq8_offset + 2 * i) * Q81_BYTES;
        int32_t sc = (int32_t)(int8_t)blk[192 + scale_offset + 4 * i];
        int32_t sumi = 0;
        for (int j = 0; j < 2; j++) {
            int32_t u = i32_at(b8 + 4 + 4 * (iqs % 8 + j));
            int32_t vil = (int32_t)((vl[j] >> (4 * i)) & 0x0F0F0F0Fu);
            int32_t vih = (int32_t)(((vh[j] >> (4 * i)) << 4) & 0x30303030u);
            sumi = dp4a(vil | vih, u, sumi);
            sumi = dp4a((int32_t)0xE0E0E0E0u, u, sumi);
        }
        sumf += f16_at(b8) * (float)(sumi * sc);
    }
    return f16_at(blk + 208) * sumf;
}

// crates/frink-cuda/src/dp4a_twin.rs:198-208 (vec_dot_q8_0)
float vec_dot_q8_0(const uint8_t* blk, const uint8_t* y, int iqs) {
    int32_t sumi = 0;
    for (int i = 0; i < 2; i++) sumi = dp4a(i32_at(blk + 2 + 4 * (iqs + i)), i32_at(y + 4 + 4 * (iqs + i)), sumi);
    return f16_at(blk) * f16_at(y) * (float)sumi;
}

// crates/frink-cuda/src/dp4a_twin.rs:216-231 (vec_dot_mxfp4)
float vec_dot_mxfp4(const uint8_t* blk, const uint8_t* y, int iqs) {
    int32_t sumi = 0;
    for (int l = 0; l < 2; l++) {
        const uint8_t* codes = blk + 1 + 4 * (iqs + l);
        uint32_t lo = 0, hi = 0;
        for (int b = 0; b < 4; b++) {
            lo |= (uint32_t)(uint8_t)KV_MXFP4_X2[codes[b] & 15] << (8 * b);
            hi |= (uint32_t)(uint8_t)KV_MXFP4_X2[codes[b] >> 4] << (8 * b);
        }
        sumi = dp4a((int32_t)lo, i32_at(y + 4 + 4 * (iqs + l)), sumi);
        sumi = dp4a((int32_t)hi, i32_at(y + 4 + 4 * (iqs + l + 4)), sumi);
    }
    float d = e8m0_scale(blk[0]) * 0.5f * f16_at(y);
    return d * (float)sumi;
}

struct Dp4aKind { int qk, qi, vdr, block_bytes; float (*dot)(const uint8_t*, const uint8_t*, int); };
// crates/frink-cuda/src/matvec_kinds/dp4a.rs:201-242 (DP4A table)
bool dp4a_kind(int kind, Dp4aKind* k) {
    switch (kind) {
        case 12: *k = {256, 32, 2, Q4K_BYTES, vec_dot_q4_k}; return true;
        case 14: *k = {256, 32, 2, Q6K_BYTES, vec_dot_q6_k}; return true;
        case 8: *k = {32, 8, 2, Q80_BYTES, vec_dot_q8_0}; return true;
        case 39: *k = {32, 4, 2, MX4_BYTES, vec_dot_mxfp4}; return true;
    }
    return false;
}

// crates/frink-cuda/src/dp4a_twin.rs:247-292 (thread_blocks, dp4a_matvec_row)
// and crates/frink-cuda/src/coalesced_twin.rs:44-53 (warp_sum).
float dp4a_matvec_row(const Dp4aKind& k, const uint8_t* row, const uint8_t* y, int n_blocks, int nwarps) {
    int tpb = k.qi / k.vdr;
    int q8pb = k.qk / 32;
    float lanes[32];
    for (int lane = 0; lane < 32; lane++) {
        float s = 0.0f;
        for (int w = 0; w < nwarps; w++) {
            int tid = 32 * w + lane;
            int iqs = k.vdr * (tid % tpb);
            float acc = 0.0f;
            for (int b = tid / tpb; b < n_blocks; b += 32 * nwarps / tpb) {
                acc += k.dot(row + (size_t)b * k.block_bytes, y + (size_t)b * q8pb * Q81_BYTES, iqs);
            }
            if (w == 0) s = acc; else s += acc;
        }
        lanes[lane] = s;
    }
    for (int s = 16; s > 0; s >>= 1)
        for (int l = 0; l < s; l++) lanes[l] += lanes[l + s];
    return lanes[0];
}

// Per-run exact integer dots of one weight row against q8_1 activations: the
// integers every dp4a word-dot above is a partial sum of.  A "run" is 32
// activations (one q8_1 block) for Q4_K, Q5_K, Q8_0 and MXFP4 and 16 for Q6_K (its
// scale granularity).  Q4_K: sum nib*q8.  Q5_K: sum (nib + 16 bit)*q8.  Q6_K: sum (q6-32)*q8.  Q8_0: sum
// qw*q8.  MXFP4: sum kvalue_x2*q8.
void row_isums(int kind, const uint8_t* row, int nblk, const uint8_t* y, int32_t* out) {
    if (kind == 12) {
        for (int b = 0; b < nblk; b++) {
            const uint8_t* qs = row + (size_t)b * Q4K_BYTES + 16;
            for (int j = 0; j < 8; j++) {
                const uint8_t* q8 = y + (size_t)(b * 8 + j) * Q81_BYTES + 4;
                int s = 0;
                for (int l = 0; l < 32; l++) {
                    int nib = (j & 1) ? (qs[(j / 2) * 32 + l] >> 4) : (qs[(j / 2) * 32 + l] & 0x0F);
                    s += nib * (int)(int8_t)q8[l];
                }
                out[b * 8 + j] = s;
            }
        }
    } else if (kind == 13) {
        uint8_t q[256];
        for (int b = 0; b < nblk; b++) {
            q5k_codes(row + (size_t)b * Q5K_BYTES, q);
            for (int j = 0; j < 8; j++) {
                const uint8_t* q8 = y + (size_t)(b * 8 + j) * Q81_BYTES + 4;
                int s = 0;
                for (int l = 0; l < 32; l++) s += (int)q[32 * j + l] * (int)(int8_t)q8[l];
                out[b * 8 + j] = s;
            }
        }
    } else if (kind == 14) {
        int8_t q[256];
        for (int b = 0; b < nblk; b++) {
            q6k_codes(row + (size_t)b * Q6K_BYTES, q);
            for (int g = 0; g < 16; g++) {
                const uint8_t* q8 = y + (size_t)(b * 8 + g / 2) * Q81_BYTES + 4 + (g & 1) * 16;
                int s = 0;
                for (int l = 0; l < 16; l++) s += (int)q[g * 16 + l] * (int)(int8_t)q8[l];
                out[b * 16 + g] = s;
            }
        }
    } else if (kind == 8) {
        for (int b = 0; b < nblk; b++) {
            const uint8_t* blk = row + (size_t)b * Q80_BYTES;
            const uint8_t* q8 = y + (size_t)b * Q81_BYTES + 4;
            int s = 0;
            for (int l = 0; l < 32; l++) s += (int)(int8_t)blk[2 + l] * (int)(int8_t)q8[l];
            out[b] = s;
        }
    } else if (kind == 39) {
        for (int b = 0; b < nblk; b++) {
            const uint8_t* blk = row + (size_t)b * MX4_BYTES;
            const uint8_t* q8 = y + (size_t)b * Q81_BYTES + 4;
            int s = 0;
            for (int j = 0; j < 16; j++) {
                s += (int)KV_MXFP4_X2[blk[1 + j] & 0xF] * (int)(int8_t)q8[j];
                s += (int)KV_MXFP4_X2[blk[1 + j] >> 4] * (int)(int8_t)q8[j + 16];
            }
            out[b] = s;
        }
    }
}

// ------------------------------------------------------------------ encoders
// crates/frink-quant/src/encode.rs:91-108 (encode_block_q8_0)
void encode_block_q8_0(const float* blk, uint8_t* out) {
    float amax = 0.0f;
    for (int i = 0; i < 32; i++) {
        float av = std::fabs(blk[i]);
        amax = amax > av ? amax : av;
    }
    float d = amax / 127.0f;
    float id = d != 0.0f ? 1.0f / d : 0.0f;
    uint16_t dh = f32_to_f16(d);
    out[0] = dh & 0xFF;
    out[1] = dh >> 8;
    for (int i = 0; i < 32; i++) {
        float r = std::roundf(blk[i] * id);
        r = std::fmin(std::fmax(r, -128.0f), 127.0f);  // Rust `as i8` saturates
        out[2 + i] = (uint8_t)(int8_t)r;
    }
}

// crates/frink-quant/src/encode/fit.rs:92-96 (nearest_int)
inline int nearest_int(float fval) {
    float val = fval + 12582912.0f;
    int32_t i;
    std::memcpy(&i, &val, 4);
    return (i & 0x007fffff) - 0x00400000;
}
inline int clampi(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }

// crates/frink-quant/src/encode/fit.rs:111-206 (make_qkx2_quants)
void make_qkx2_quants(int n, const float* x, const float* weights, uint8_t* l, uint8_t* laux, int nmax,
                      float rmin, float rdelta, int nstep, bool use_mad, float* out_scale, float* out_min) {
    float min = x[0], max = x[0];
    float sum_w = weights[0];
    float sum_x = sum_w * x[0];
    for (int i = 1; i < n; i++) {
        if (x[i] < min) min = x[i];
        if (x[i] > max) max = x[i];
        float w = weights[i];
        sum_w += w;
        sum_x = fmaf(w, x[i], sum_x);
    }
    if (min > 0.0f) min = 0.0f;
    if (max == min) {
        for (int i = 0; i < n; i++) l[i] = 0;
        *out_scale = 0.0f;
        *out_min = -min;
        return;
    }
    float iscale = (float)nmax / (max - min);
    float scale = 1.0f / iscale;
    float best_error = 0.0f;
    for (int i = 0; i < n; i++) {
        int li = clampi(nearest_int(iscale * (x[i] - min)), 0, nmax);
        l[i] = (uint8_t)li;
        float diff = fmaf(scale, (float)l[i], min) - x[i];
        diff = use_mad ? std::fabs(diff) : diff * diff;
        best_error = fmaf(weights[i], diff, best_error);
    }
    if (nstep < 1) {
        *out_scale = scale;
        *out_min = -min;
        return;
    }
    for (int is = 0; is <= nstep; is++) {
        iscale = (rmin + rdelta * (float)is + (float)nmax) / (max - min);
        float sum_l = 0.0f, sum_l2 = 0.0f, sum_xl = 0.0f;
        for (int i = 0; i < n; i++) {
            int li = clampi(nearest_int(iscale * (x[i] - min)), 0, nmax);
            laux[i] = (uint8_t)li;
            float w = weights[i];
            sum_l = fmaf(w, (float)li, sum_l);
            sum_l2 = fmaf(w * (float)li, (float)li, sum_l2);
            sum_xl = fmaf(w * (float)li, x[i], sum_xl);
        }
        float det = fmaf(sum_w, sum_l2, -(sum_l * sum_l));
        if (det > 0.0f) {
            float this_scale = fmaf(sum_w, sum_xl, -(sum_x * sum_l)) / det;
            float this_min = fmaf(sum_l2, sum_x, -(sum_l * sum_xl)) / det;
            if (this_min > 0.0f) {
                this_min = 0.0f;
                this_scale = sum_xl / sum_l2;
            }
            float cur_error = 0.0f;
            for (int i = 0; i < n; i++) {
                float diff = fmaf(this_scale, (float)laux[i], this_min) - x[i];
                diff = use_mad ? std::fabs(diff) : diff * diff;
                cur_error = fmaf(weights[i], diff, cur_error);
            }
            if (cur_error < best_error) {
                for (int i = 0; i < n; i++) l[i] = laux[i];
                best_error = cur_error;
                scale = this_scale;
                min = this_min;
            }
        }
    }
    *out_scale = scale;
    *out_min = -min;
}

// crates/frink-quant/src/encode/fit.rs:243-323 (make_qx_quants), plain path
// (no importance matrix): weight by rmse_type, :225-236 (qx_weight).
inline float qx_weight(const float* x, int rmse_type, int i) {
    switch (rmse_type) {
        case 1: return x[i] * x[i];
        case 2: return 1.0f;
        case 3: return std::fabs(x[i]);
        default: return std::sqrt(std::fabs(x[i]));
    }
}
float make_qx_quants(int n, const float* x, int8_t* l, int nmax, int rmse_type) {
    float max = 0.0f, amax = 0.0f;
    for (int i = 0; i < n; i++) {
        float ax = std::fabs(x[i]);
        if (ax > amax) { amax = ax; max = x[i]; }
    }
    if (amax < 1e-15f) {
        for (int i = 0; i < n; i++) l[i] = 0;
        return 0.0f;
    }
    float iscale = -(float)nmax / max;
    if (rmse_type == 0) {
        for (int i = 0; i < n; i++) {
            int li = nearest_int(iscale * x[i]);
            l[i] = (int8_t)(nmax + clampi(li, -nmax, nmax - 1));
        }
        return 1.0f / iscale;
    }
    bool return_early = false;
    if (rmse_type < 0) { rmse_type = -rmse_type; return_early = true; }
    float sumlx = 0.0f, suml2 = 0.0f;
    for (int i = 0; i < n; i++) {
        int li = clampi(nearest_int(iscale * x[i]), -nmax, nmax - 1);
        l[i] = (int8_t)(li + nmax);
        float w = qx_weight(x, rmse_type, i);
        sumlx = fmaf(w * x[i], (float)li, sumlx);
        suml2 = fmaf(w * (float)li, (float)li, suml2);
    }
    float scale = suml2 != 0.0f ? sumlx / suml2 : 0.0f;
    if (return_early) return suml2 > 0.0f ? 0.5f * (scale + 1.0f / iscale) : 1.0f / iscale;
    float best = scale * sumlx;
    for (int is = -9; is <= 9; is++) {
        if (is == 0) continue;
        iscale = -((float)nmax + 0.1f * (float)is) / max;
        sumlx = 0.0f;
        suml2 = 0.0f;
        for (int i = 0; i < n; i++) {
            int li = clampi(nearest_int(iscale * x[i]), -nmax, nmax - 1);
            float w = qx_weight(x, rmse_type, i);
            sumlx = fmaf(w * x[i], (float)li, sumlx);
            suml2 = fmaf(w * (float)li, (float)li, suml2);
        }
        if (suml2 > 0.0f && sumlx * sumlx > best * suml2) {
            for (int i = 0; i < n; i++) {
                int li = nearest_int(iscale * x[i]);
                l[i] = (int8_t)(nmax + clampi(li, -nmax, nmax - 1));
            }
            scale = sumlx / suml2;
            best = scale * sumlx;
        }
    }
    return scale;
}

// crates/frink-quant/src/encode/fit.rs:576-592 (pack_scale_min)
inline void pack_scale_min(uint8_t* packed, int j, uint8_t ls, uint8_t lm) {
    if (j < 4) {
        packed[j] = ls;
        packed[j + 4] = lm;
    } else {
        packed[j + 4] = (uint8_t)((ls & 0xF) | ((lm & 0xF) << 4));
        packed[j - 4] |= (uint8_t)((ls >> 4) << 6);
        packed[j] |= (uint8_t)((lm >> 4) << 6);
    }
}

// crates/frink-quant/src/encode/fit.rs:416-566 (fit_qk_super_block, plain path): the three-stage fit Q4_K and Q5_K share
// -- per sub-block scale / min search over the kind's candidate grid, 6-bit packing of the eight scales and mins against
// their maxima, and the requantization of every code against the packed (rounded) scales.
struct QkFit { int nmax; float rmin, rdelta; int nstep; };
void fit_qk_super_block(const float* block, const QkFit& f, uint8_t* l, uint8_t* packed, uint16_t* dh_out, uint16_t* dmh_out) {
    uint8_t laux[32];
    float weights[32], mins[8], scales[8];
    float max_scale = 0.0f, max_min = 0.0f;
    std::memset(l, 0, 256);
    for (int j = 0; j < 8; j++) {
        const float* xs = block + 32 * j;
        // fit.rs:327-336 (qk_sub_block_weights): not fused in the reference
        float sum_x2 = 0.0f;
        for (int i = 0; i < 32; i++) sum_x2 += xs[i] * xs[i];
        float av_x = std::sqrt(sum_x2 / 32.0f);
        for (int i = 0; i < 32; i++) weights[i] = av_x + std::fabs(xs[i]);
        float scale, min;
        make_qkx2_quants(32, xs, weights, l + 32 * j, laux, f.nmax, f.rmin, f.rdelta, f.nstep, false, &scale, &min);
        scales[j] = scale;
        mins[j] = min;
        if (scale > max_scale) max_scale = scale;
        if (min > max_min) max_min = min;
    }
    std::memset(packed, 0, 12);
    float inv_scale = max_scale > 0.0f ? 63.0f / max_scale : 0.0f;
    float inv_min = max_min > 0.0f ? 63.0f / max_min : 0.0f;
    for (int j = 0; j < 8; j++) {
        uint8_t ls = (uint8_t)nearest_int(inv_scale * scales[j]);  // narrow first, then clamp
        uint8_t lm = (uint8_t)nearest_int(inv_min * mins[j]);
        if (ls > 63) ls = 63;
        if (lm > 63) lm = 63;
        pack_scale_min(packed, j, ls, lm);
    }
    uint16_t dh = f32_to_f16(max_scale / 63.0f), dmh = f32_to_f16(max_min / 63.0f);
    float d = f16_to_f32(dh), dmin = f16_to_f32(dmh);
    for (int j = 0; j < 8; j++) {
        uint8_t sc, m;
        q4k_scale_min(j, packed, &sc, &m);
        float dj = d * (float)sc;
        if (dj == 0.0f) continue;
        float dm = dmin * (float)m;
        for (int ii = 0; ii < 32; ii++) {
            int idx = 32 * j + ii;
            l[idx] = (uint8_t)clampi(nearest_int((block[idx] + dm) / dj), 0, f.nmax);
        }
    }
    *dh_out = dh;
    *dmh_out = dmh;
}

// crates/frink-quant/src/encode/q4_k.rs:83-102 (encode_block_q4_k): the Q4_K grid (-1.0, 0.1, 20), nmax 15.
void encode_block_q4_k(const float* block, uint8_t* out) {
    uint8_t l[256], packed[12];
    uint16_t dh, dmh;
    fit_qk_super_block(block, QkFit{15, -1.0f, 0.1f, 20}, l, packed, &dh, &dmh);
    out[0] = dh & 0xFF; out[1] = dh >> 8; out[2] = dmh & 0xFF; out[3] = dmh >> 8;
    std::memcpy(out + 4, packed, 12);
    int o = 16;
    for (int j = 0; j < 256; j += 64)
        for (int i = 0; i < 32; i++) out[o++] = (uint8_t)(l[j + i] | (l[j + i + 32] << 4));
}

// crates/frink-quant/src/encode/q5_k.rs:9-62 (encode_block_q5_k): the grid (-0.5, 0.1, 15), nmax 31; the fifth bit of every
// code goes to qh (bit 2g for the low-nibble half of 64-element group g, 2g + 1 for the high), the low four stay nibbles.
void encode_block_q5_k(const float* block, uint8_t* out) {
    uint8_t l[256], packed[12];
    uint16_t dh, dmh;
    fit_qk_super_block(block, QkFit{31, -0.5f, 0.1f, 15}, l, packed, &dh, &dmh);
    out[0] = dh & 0xFF; out[1] = dh >> 8; out[2] = dmh & 0xFF; out[3] = dmh >> 8;
    std::memcpy(out + 4, packed, 12);
    uint8_t* qh = out + 16;
    uint8_t* ql = out + 48;
    std::memset(qh, 0, 32);
    for (int g = 0; g < 4; g++)
        for (int j = 0; j < 32; j++) {
            uint8_t l1 = l[64 * g + j], l2 = l[64 * g + 32 + j];
            if (l1 > 15) { l1 -= 16; qh[j] |= (uint8_t)(1u << (2 * g)); }
            if (l2 > 15) { l2 -= 16; qh[j] |= (uint8_t)(2u << (2 * g)); }
            ql[32 * g + j] = (uint8_t)(l1 | (l2 << 4));
        }
}

// crates/frink-quant/src/encode/q6_k.rs:72-175 (encode_block_q6_k, plain path)
void encode_block_q6_k(const float* block, uint8_t* out) {
    int8_t l[256] = {0};
    float scales[16];
    float max_scale = 0.0f, max_abs_scale = 0.0f;
    for (int ib = 0; ib < 16; ib++) {
        float scale = make_qx_quants(16, block + 16 * ib, l + 16 * ib, 32, 1);
        scales[ib] = scale;
        float abs_scale = std::fabs(scale);
        if (abs_scale > max_abs_scale) { max_abs_scale = abs_scale; max_scale = scale; }
    }
    if (max_abs_scale < 1e-15f) {
        std::memset(out, 0, Q6K_BYTES);
        return;
    }
    float iscale = -128.0f / max_scale;
    uint16_t dh = f32_to_f16(1.0f / iscale);
    float d = f16_to_f32(dh);
    int8_t qscales[16];
    for (int ib = 0; ib < 16; ib++) {
        int v = nearest_int(iscale * scales[ib]);
        if (v > 127) v = 127;
        qscales[ib] = (int8_t)v;  // wraps below -128 as the C does
    }
    for (int j = 0; j < 16; j++) {
        float dj = d * (float)qscales[j];
        if (dj == 0.0f) continue;
        for (int ii = 0; ii < 16; ii++) {
            int idx = 16 * j + ii;
            l[idx] = (int8_t)(clampi(nearest_int(block[idx] / dj), -32, 31) + 32);
        }
    }
    uint8_t* ql = out;
    uint8_t* qh = out + 128;
    for (int half = 0; half < 2; half++) {
        int j = half * 128, qlo = half * 64, qho = half * 32;
        for (int i = 0; i < 32; i++) {
            uint8_t q1 = (uint8_t)(l[j + i] & 0xF), q2 = (uint8_t)(l[j + i + 32] & 0xF);
            uint8_t q3 = (uint8_t)(l[j + i + 64] & 0xF), q4 = (uint8_t)(l[j + i + 96] & 0xF);
            ql[qlo + i] = (uint8_t)(q1 | (q3 << 4));
            ql[qlo + i + 32] = (uint8_t)(q2 | (q4 << 4));
            qh[qho + i] = (uint8_t)(((uint8_t)(l[j + i] >> 4)) | (((uint8_t)(l[j + i + 32] >> 4)) << 2) |
                                    (((uint8_t)(l[j + i + 64] >> 4)) << 4) | (((uint8_t)(l[j + i + 96] >> 4)) << 6));
        }
    }
    for (int i = 0; i < 16; i++) out[192 + i] = (uint8_t)qscales[i];
    out[208] = dh & 0xFF;
    out[209] = dh >> 8;
}

// crates/frink-models/tests/common/quant_encode.rs:103-131 (mxfp4_row): the
// reference has no production MXFP4 writer; this is its test encoder.
void encode_block_mxfp4(const float* block, uint8_t* out) {
    float amax = 0.0f;
    for (int i = 0; i < 32; i++) amax = std::fmax(amax, std::fabs(block[i]));
    int e = 1;
    if (amax != 0.0f) e = clampi((int)std::ceil(std::log2(amax / 6.0f)) + 127, 1, 254);
    float d = f32_from_bits((uint32_t)e << 23);
    auto code = [&](float v) {
        int best = 0;
        float bd = std::fabs(KV_MXFP4[0] * d - v);
        for (int c = 1; c < 16; c++) {
            float dc = std::fabs(KV_MXFP4[c] * d - v);
            if (dc < bd) { bd = dc; best = c; }  // first minimum wins
        }
        return (uint8_t)best;
    };
    out[0] = (uint8_t)e;
    for (int j = 0; j < 16; j++) out[1 + j] = (uint8_t)(code(block[j]) | (code(block[j + 16]) << 4));
}

// ------------------------------------------------------------------ routing
// crates/frink-moe/src/lib.rs:567-589 (route_top_k_softmax, modes 0 and 1) and
// :1012-1031 (route_top_k_softmax_weight, mode 2).  The reference's host sort
// is unstable; ties follow the device kernel's documented rule, lower id first
// (crates/frink-cuda/src/prefill/kernels.rs:178-267).
void route_top_k(const float* logits, const float* bias, int n, int k, int mode, int* ids, float* w) {
    std::vector<float> v(n);
    for (int e = 0; e < n; e++) v[e] = logits[e] + (bias ? bias[e] : 0.0f);
    // Selection is by (biased) logit, as the device kernel selects; softmax is
    // monotonic, so this is the host's order by probability with the tie rule
    // made explicit (two logits that round to one probability stay ordered).
    std::vector<int> idx(n);
    for (int e = 0; e < n; e++) idx[e] = e;
    std::stable_sort(idx.begin(), idx.end(), [&](int a, int b) { return v[a] > v[b]; });
    int kk = std::min(k, n);
    if (mode == 2) {
        float mx = -INFINITY;
        for (int s = 0; s < kk; s++) mx = std::fmax(mx, v[idx[s]]);
        float es = 0.0f;
        std::vector<float> ex(kk);
        for (int s = 0; s < kk; s++) { ex[s] = std::exp(v[idx[s]] - mx); es += ex[s]; }
        for (int s = 0; s < kk; s++) { ids[s] = idx[s]; w[s] = es > 0.0f ? ex[s] / es : ex[s]; }
        return;
    }
    float mx = -INFINITY, sum = 0.0f;
    for (int e = 0; e < n; e++) mx = std::fmax(mx, v[e]);
    std::vector<float> exps(n);
    for (int e = 0; e < n; e++) exps[e] = std::exp(v[e] - mx);
    for (int e = 0; e < n; e++) sum += exps[e];
    float ts = 0.0f;
    for (int s = 0; s < kk; s++) { ids[s] = idx[s]; w[s] = exps[idx[s]] / sum; ts += w[s]; }
    if (mode == 1) for (int s = 0; s < kk; s++) w[s] /= ts;
}

// Row-parallel split, contiguous chunks, as crates/frink-core/src/par.rs
// (items_mut) hands a matrix's rows to its workers.
void run_rows(int rows, int nthreads, const std::function<void(int, int)>& body) {
    if (nthreads <= 1 || rows < 2 * nthreads) { body(0, rows); return; }
    std::vector<std::thread> th;
    int per = (rows + nthreads - 1) / nthreads;
    for (int t = 0; t < nthreads; t++) {
        int lo = t * per, hi = std::min(rows, lo + per);
        if (lo >= hi) break;
        th.emplace_back([=, &body] { body(lo, hi); });
    }
    for (auto& t : th) t.join();
}
}  // namespace

// ================================================================= C exports
FKO_API int fko_has_avx2(void) { return FKO_AVX2; }
FKO_API float fko_f16_to_f32(uint16_t h) { return f16_to_f32(h); }
FKO_API uint16_t fko_f32_to_f16(float f) { return f32_to_f16(f); }

FKO_API int fko_block_bytes(int kind) { KindInfo k; return kind_info(kind, &k) ? k.block_bytes : -1; }
FKO_API int fko_block_elems(int kind) { KindInfo k; return kind_info(kind, &k) ? k.block_elems : -1; }

// `nbytes` of blocks of `kind` into f32; returns elements written or -1.
FKO_API long fko_dequant(int kind, const uint8_t* src, long nbytes, float* out) {
    KindInfo k;
    if (!kind_info(kind, &k) || nbytes % k.block_bytes != 0) return -1;
    long nb = nbytes / k.block_bytes;
    for (long b = 0; b < nb; b++) k.decode(src + b * k.block_bytes, out + b * k.block_elems);
    return nb * k.block_elems;
}

FKO_API float fko_dot_f32_scalar(int kind, const uint8_t* row, int nblk, const float* x) {
    return dot_f32_scalar(kind, row, nblk, x);
}
FKO_API double fko_dot_dequant_f64(int kind, const uint8_t* row, int nblk, const float* x) {
    return dot_dequant_f64(kind, row, nblk, x);
}

FKO_API void fko_quantize_q8_k(const float* x, int n, int8_t* q, float* d, int16_t* bsums) { quantize_q8_k(x, n, q, d, bsums); }
FKO_API void fko_quantize_q8_0_act(const float* x, int n, int form, int8_t* q, float* d) { quantize_q8_0_act(x, n, form, q, d); }
FKO_API void fko_quantize_q8_1(const float* x, int n, uint8_t* out) { quantize_q8_1(x, n, out); }
FKO_API void fko_q8_1_dequant(const uint8_t* y, int nb, float* out) { q8_1_dequant(y, nb, out); }

// L2 integer dot of one row.  K-quants take Q8_K activations (q, d, bsums);
// Q8_0 and MXFP4 take Q8_0-form activations (q, d; bsums ignored).
// The exact integers of dot_q4_k_q8_scalar (crates/frink-quant/src/lib.rs:822-869) per super-block:
// out[2 b] = sum over the four trips of sc1 * isum1 + sc2 * isum2, out[2 b + 1] = sum_min.
FKO_API void fko_row_isums_q4k_q8k(const uint8_t* row, int nblk, const int8_t* aq, const int16_t* bs, int32_t* out) {
    for (int b = 0; b < nblk; b++) {
        const uint8_t* blk = row + (size_t)b * Q4K_BYTES;
        const uint8_t* scales = blk + 4;
        const uint8_t* qs = blk + 16;
        const int8_t* q8 = aq + (size_t)b * 256;
        const int16_t* bsums = bs + b * 16;
        int sum_min = 0;
        for (int i = 0; i < 8; i++) {
            uint8_t sc, m;
            q4k_scale_min(i, scales, &sc, &m);
            sum_min += (int)m * ((int)bsums[2 * i] + (int)bsums[2 * i + 1]);
        }
        long long S = 0;
        int q_off = 0, base = 0, is = 0;
        for (int it = 0; it < 4; it++) {
            uint8_t sc1, sc2, m;
            q4k_scale_min(is, scales, &sc1, &m);
            q4k_scale_min(is + 1, scales, &sc2, &m);
            int isum1 = 0, isum2 = 0;
            for (int l = 0; l < 32; l++) isum1 += (int)(qs[q_off + l] & 0x0F) * (int)q8[base + l];
            for (int l = 0; l < 32; l++) isum2 += (int)(qs[q_off + l] >> 4) * (int)q8[base + 32 + l];
            S += (long long)sc1 * isum1 + (long long)sc2 * isum2;
            q_off += 32;
            base += 64;
            is += 2;
        }
        out[2 * b] = (int32_t)S;
        out[2 * b + 1] = sum_min;
    }
}

FKO_API float fko_dot_q8(int kind, const uint8_t* row, int nblk, const int8_t* q, const float* d, const int16_t* bsums) {
    switch (kind) {
        case 12: return dot_q4_k_q8k(row, nblk, q, d, bsums);
        case 13: return dot_q5_k_q8k(row, nblk, q, d, bsums);
        case 14: return dot_q6_k_q8k(row, nblk, q, d);
        case 8: return dot_q8_0_q8(row, nblk, q, d);
        case 39: return dot_mxfp4_q8(row, nblk, q, d);
    }
    return NAN;
}

FKO_API float fko_dp4a_row(int kind, const uint8_t* row, const uint8_t* y, int n_blocks, int nwarps) {
    Dp4aKind k;
    if (!dp4a_kind(kind, &k)) return NAN;
    return dp4a_matvec_row(k, row, y, n_blocks, nwarps);
}
FKO_API int fko_runs_per_block(int kind) { return kind == 12 || kind == 13 ? 8 : kind == 14 ? 16 : 1; }
FKO_API void fko_row_isums(int kind, const uint8_t* row, int nblk, const uint8_t* y, int32_t* out) { row_isums(kind, row, nblk, y, out); }

// Encode `n` f32 (a whole number of blocks) as `kind`; returns bytes written or -1.
FKO_API long fko_encode(int kind, const float* src, long n, uint8_t* out) {
    KindInfo k;
    if (!kind_info(kind, &k) || n % k.block_elems != 0) return -1;
    long nb = n / k.block_elems;
    for (long b = 0; b < nb; b++) {
        const float* s = src + b * k.block_elems;
        uint8_t* o = out + b * k.block_bytes;
        switch (kind) {
            case 12: encode_block_q4_k(s, o); break;
            case 13: encode_block_q5_k(s, o); break;
            case 14: encode_block_q6_k(s, o); break;
            case 8: encode_block_q8_0(s, o); break;
            case 39: encode_block_mxfp4(s, o); break;
            case 30: {   // round to nearest even on the upper half (test data; the reference only reads this format)
                uint32_t u;
                std::memcpy(&u, s, 4);
                u += 0x7FFFu + ((u >> 16) & 1u);
                o[0] = (uint8_t)(u >> 16);
                o[1] = (uint8_t)(u >> 24);
                break;
            }
        }
    }
    return nb * k.block_bytes;
}
// The same, split over `nthreads` host threads (rows are independent).
FKO_API long fko_encode_mt(int kind, const float* src, long n, uint8_t* out, int nthreads) {
    KindInfo k;
    if (!kind_info(kind, &k) || n % k.block_elems != 0) return -1;
    long nb = n / k.block_elems;
    run_rows((int)nb, nthreads, [&](int lo, int hi) {
        fko_encode(kind, src + (long)lo * k.block_elems, (long)(hi - lo) * k.block_elems, out + (long)lo * k.block_bytes);
    });
    return nb * k.block_bytes;
}
FKO_API int fko_nearest_int(float v) { return nearest_int(v); }

// y[b][r] = dot(W[r], x[b]) with the reference's x86 decode path: the fused
// f32 dot per row (crates/frink-core/src/weight_matrix.rs:1234-1262), rows split
// over threads.  simd != 0 takes the AVX2 form where this build has one (Q4_K).
FKO_API int fko_matvec_f32(int kind, const uint8_t* w, int rows, int cols, const float* x, int batch, float* y,
                           int nthreads, int simd) {
    KindInfo k;
    if (!kind_info(kind, &k) || cols % k.block_elems != 0) return -1;
    int nblk = cols / k.block_elems;
    size_t row_bytes = (size_t)nblk * k.block_bytes;
    run_rows(rows, nthreads, [&](int lo, int hi) {
        for (int b = 0; b < batch; b++)
            for (int r = lo; r < hi; r++) {
                const uint8_t* row = w + (size_t)r * row_bytes;
                const float* xb = x + (size_t)b * cols;
#if FKO_AVX2
                if (simd && kind == 12) { y[(size_t)b * rows + r] = dot_q4_k_f32_avx2(row, nblk, xb); continue; }
#endif
                y[(size_t)b * rows + r] = dot_f32_scalar(kind, row, nblk, xb);
            }
    });
    return 0;
}

// out[t][r] with the reference's CPU batched path (crates/frink-core/src/
// weight_matrix.rs:2348-2423, :3038, :3256): activations quantized once per
// token (Q8_K for the K-quants, Q8_0 AVX form for Q8_0/MXFP4), then integer
// row dots, non-repacked.
FKO_API int fko_matmul_q8(int kind, const uint8_t* w, int rows, int cols, const float* x, int batch, float* out, int nthreads) {
    KindInfo k;
    if (!kind_info(kind, &k) || cols % 256 != 0 && (kind == 12 || kind == 13 || kind == 14)) return -1;
    if (cols % k.block_elems != 0) return -1;
    int nblk = cols / k.block_elems;
    size_t row_bytes = (size_t)nblk * k.block_bytes;
    bool kq = (kind == 12 || kind == 13 || kind == 14);
    std::vector<int8_t> q((size_t)batch * cols);
    std::vector<float> d((size_t)batch * (kq ? cols / 256 : cols / 32));
    std::vector<int16_t> bs(kq ? (size_t)batch * cols / 16 : 1);
    for (int t = 0; t < batch; t++) {
        if (kq) quantize_q8_k(x + (size_t)t * cols, cols, q.data() + (size_t)t * cols, d.data() + (size_t)t * (cols / 256), bs.data() + (size_t)t * (cols / 16));
        else quantize_q8_0_act(x + (size_t)t * cols, cols, 1, q.data() + (size_t)t * cols, d.data() + (size_t)t * (cols / 32));
    }
    run_rows(rows, nthreads, [&](int lo, int hi) {
        for (int r = lo; r < hi; r++) {
            const uint8_t* row = w + (size_t)r * row_bytes;
            for (int t = 0; t < batch; t++) {
                const int8_t* qt = q.data() + (size_t)t * cols;
                const float* dt = d.data() + (size_t)t * (kq ? cols / 256 : cols / 32);
                const int16_t* bt = kq ? bs.data() + (size_t)t * (cols / 16) : nullptr;
                out[(size_t)t * rows + r] = fko_dot_q8(kind, row, nblk, qt, dt, bt);
            }
        }
    });
    return 0;
}

// Reference for the fp32 tolerance: f64 dequantize-then-dot of every row.
FKO_API int fko_matmul_f64(int kind, const uint8_t* w, int rows, int cols, const float* x, int batch, double* out, int nthreads) {
    KindInfo k;
    if (!kind_info(kind, &k) || cols % k.block_elems != 0) return -1;
    int nblk = cols / k.block_elems;
    size_t row_bytes = (size_t)nblk * k.block_bytes;
    run_rows(rows, nthreads, [&](int lo, int hi) {
        std::vector<float> wrow(cols);
        for (int r = lo; r < hi; r++) {
            const uint8_t* row = w + (size_t)r * row_bytes;
            for (int b = 0; b < nblk; b++) k.decode(row + (size_t)b * k.block_bytes, wrow.data() + (size_t)b * k.block_elems);
            for (int t = 0; t < batch; t++) {
                const float* xt = x + (size_t)t * cols;
                double acc = 0.0;
                for (int i = 0; i < cols; i++) acc += (double)wrow[i] * (double)xt[i];
                out[(size_t)t * rows + r] = acc;
            }
        }
    });
    return 0;
}

FKO_API void fko_route_top_k(const float* logits, const float* bias, int n, int k, int mode, int batch, int* ids, float* w) {
    for (int t = 0; t < batch; t++) route_top_k(logits + (size_t)t * n, bias, n, k, mode, ids + (size_t)t * k, w + (size_t)t * k);
}

// crates/frink-core/src/matmul.rs:634,647 (silu) and the SwiGLU combine
// act(gate) * up (crates/frink-moe/src/glu_act.rs:216).
FKO_API void fko_silu_mul(const float* gate, const float* up, int n, float* out) {
    for (int i = 0; i < n; i++) {
        float g = gate[i];
        out[i] = (g / (1.0f + std::exp(-g))) * up[i];
    }
}
// crates/frink-moe/src/lib.rs:988-999 (swiglu_oai)
FKO_API void fko_swiglu_oai(const float* gate, const float* up, int n, float alpha, float limit, float* out) {
    for (int i = 0; i < n; i++) {
        float x = std::fmin(gate[i], limit);
        float y = std::fmin(std::fmax(up[i], -limit), limit);
        float out_glu = x / (1.0f + std::exp(alpha * -x));
        out[i] = out_glu * (y + 1.0f);
    }
}
// crates/frink-moe/src/lib.rs:1246-1263 (combine_expert_outputs, routed part):
// from zero, in routing order, out += expert * weight.
FKO_API void fko_combine(const float* ys, const float* w, int k, int n, float* out) {
    for (int i = 0; i < n; i++) out[i] = 0.0f;
    for (int j = 0; j < k; j++)
        for (int i = 0; i < n; i++) out[i] += ys[(size_t)j * n + i] * w[j];
}
