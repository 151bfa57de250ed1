/*
 * ztq_oracle.c -- CPU restatement of ztensor's weight-quantized matrix-vector path.
 *
 * TEST INFRASTRUCTURE ONLY: the parity checker and the timed CPU baseline.
 * See ztq_oracle.h for the pinning status.  Citations are file:line inside
 * zerfoo/ztensor.  Compile with -ffp-contract=off: every `a*b + c` below that
 * is written as two statements must stay two roundings.
 */
#include "ztq_oracle.h"

#include <math.h>
#include <pthread.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

#if defined(__AVX2__) && defined(__FMA__)
#include <immintrin.h>
#endif

/* ------------------------------------------------------------------ */
/* binary16                                                            */
/* ------------------------------------------------------------------ */

static inline uint32_t f32_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float bits_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

/* float32 -> binary16, round to nearest even, gradual underflow, overflow to
 * infinity, NaN kept quiet.  Stands in for float16.FromFloat32 of
 * zerfoo/float16 v0.2.0 (call sites: tensor/quantized.go:63,
 * tensor/quantized_gptq.go:85-86, tensor/fp16_storage.go:32). */
uint16_t zo_f32_to_f16(float v) {
    uint32_t x = f32_bits(v);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t absx = x & 0x7fffffffu;
    if (absx >= 0x7f800000u) {                       /* Inf / NaN */
        if (absx > 0x7f800000u) return (uint16_t)(sign | 0x7e00u);
        return (uint16_t)(sign | 0x7c00u);
    }
    if (absx >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u); /* >= 65520 rounds to Inf */
    if (absx < 0x33000001u) return (uint16_t)sign;              /* <= 2^-25 rounds to 0  */
    int32_t e = (int32_t)(absx >> 23) - 127;
    uint32_t m = (absx & 0x7fffffu) | 0x800000u;                /* 24-bit significand */
    uint32_t shift;
    uint32_t hexp;
    if (e < -14) { shift = (uint32_t)(13 + (-14 - e)); hexp = 0; }  /* subnormal half */
    else         { shift = 13; hexp = (uint32_t)(e + 15); }
    uint32_t q = m >> shift;
    uint32_t rem = m & ((1u << shift) - 1u);
    uint32_t half = 1u << (shift - 1);
    if (rem > half || (rem == half && (q & 1u))) q++;
    uint32_t h;
    if (hexp == 0) h = q;                      /* q may carry into exponent 1: correct */
    else           h = ((hexp - 1u) << 10) + q; /* q includes the hidden bit (1<<10)    */
    return (uint16_t)(sign | h);
}

/* binary16 -> float32 (float16.ToFloat32): exact for every input. */
float zo_f16_to_f32(uint16_t h) {
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t frac = h & 0x3ffu;
    if (exp == 0) {
        if (frac == 0) return bits_f32(sign);
        float f = (float)frac * (1.0f / 16777216.0f); /* frac * 2^-24, exact */
        return sign ? -f : f;
    }
    if (exp == 31) return bits_f32(sign | 0x7f800000u | (frac << 13));
    return bits_f32(sign | ((exp + 112u) << 23) | (frac << 13));
}

/* internal/xblas/q4dot.go:54-78: subnormals decoded, Inf/NaN -> 0. */
float zo_xblas_f16_bits_to_f32(uint16_t bits) {
    uint32_t sign = ((uint32_t)bits >> 15) & 1u;
    uint32_t exp = ((uint32_t)bits >> 10) & 0x1fu;
    uint32_t frac = (uint32_t)bits & 0x3ffu;
    if (exp == 0) {
        if (frac == 0) return 0.0f;
        float f = (float)frac / 1024.0f;
        f *= 1.0f / 16384.0f;
        if (sign == 1) f = -f;
        return f;
    }
    if (exp == 31) return 0.0f;
    uint32_t e = exp - 15u + 127u;
    return bits_f32((sign << 31) | (e << 23) | (frac << 13));
}

void zo_f16_from_f32(const float* src, int64_t n, uint16_t* dst) {
    for (int64_t i = 0; i < n; i++) dst[i] = zo_f32_to_f16(src[i]);
}

void zo_f16_slice(const uint16_t* src, int64_t n, float* dst) {
    for (int64_t i = 0; i < n; i++) dst[i] = zo_f16_to_f32(src[i]);
}

/* Go helpers ---------------------------------------------------------- */

static inline int clamp_int(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }

/* int(math.Round(float64(v))): round half away from zero. */
static inline int go_round_to_int(float v) { return (int)round((double)v); }

static inline uint16_t rd16(const uint8_t* p) { return (uint16_t)(p[0] | ((uint16_t)p[1] << 8)); }
static inline void wr16(uint8_t* p, uint16_t v) { p[0] = (uint8_t)(v & 0xff); p[1] = (uint8_t)(v >> 8); }

/* ------------------------------------------------------------------ */
/* Q4_0                                                                */
/* ------------------------------------------------------------------ */

int64_t zo_q4_num_blocks(int64_t n) { return (n + 31) / 32; }

/* tensor/quantized.go:37-91 */
void zo_quantize_q4(const float* src, int64_t n, uint8_t* blocks) {
    int64_t nb = zo_q4_num_blocks(n);
    for (int64_t bi = 0; bi < nb; bi++) {
        int64_t off = bi * 32;
        float absmax = 0.0f;
        for (int j = 0; j < 32; j++) {
            float v = (off + j < n) ? src[off + j] : 0.0f;
            float av = (float)fabs((double)v);
            if (av > absmax) absmax = av;
        }
        float scale = 0.0f;
        if (absmax > 0) scale = absmax / 7.0f;
        uint8_t* blk = blocks + bi * 18;
        wr16(blk, zo_f32_to_f16(scale));
        float inv = 0.0f;
        if (scale > 0) inv = 1.0f / scale;           /* the f32 scale, not the fp16 one (:68-71) */
        for (int j = 0; j < 16; j++) {
            float v0 = (off + j < n) ? src[off + j] : 0.0f;
            float v1 = (off + j + 16 < n) ? src[off + j + 16] : 0.0f;
            float p0 = v0 * inv, p1 = v1 * inv;
            int q0 = clamp_int(go_round_to_int(p0), -8, 7);
            int q1 = clamp_int(go_round_to_int(p1), -8, 7);
            blk[2 + j] = (uint8_t)((uint8_t)(q0 + 8) | (uint8_t)((uint8_t)(q1 + 8) << 4));
        }
    }
}

/* tensor/quantized.go:96-114 */
void zo_dequantize_q4(const uint8_t* blocks, int64_t n, float* dst) {
    int64_t nb = zo_q4_num_blocks(n);
    for (int64_t bi = 0; bi < nb; bi++) {
        const uint8_t* blk = blocks + bi * 18;
        float scale = zo_f16_to_f32(rd16(blk));
        int64_t off = bi * 32;
        for (int j = 0; j < 16; j++) {
            uint8_t packed = blk[2 + j];
            int q0 = (int)(packed & 0x0f) - 8;
            int q1 = (int)(packed >> 4) - 8;
            if (off + j < n) dst[off + j] = (float)q0 * scale;
            if (off + j + 16 < n) dst[off + j + 16] = (float)q1 * scale;
        }
    }
}

/* tensor/quantized.go:196-199 */
int64_t zo_q4_gpu_data_offset(int64_t total_blocks) {
    return (total_blocks * 2 + 15) & ~(int64_t)15;
}

/* tensor/quantized.go:158-187: [scales][pad to 16][16-byte data blocks] */
void zo_q4_raw_bytes_gpu(const uint8_t* blocks, int64_t nb, uint8_t* out) {
    int64_t doff = zo_q4_gpu_data_offset(nb);
    memset(out, 0, (size_t)(doff + nb * 16));
    for (int64_t i = 0; i < nb; i++) {
        out[i * 2] = blocks[i * 18];
        out[i * 2 + 1] = blocks[i * 18 + 1];
        memcpy(out + doff + i * 16, blocks + i * 18 + 2, 16);
    }
}

/* ------------------------------------------------------------------ */
/* Q8_0                                                                */
/* ------------------------------------------------------------------ */

/* tensor/quantized.go:301-341 */
void zo_quantize_q8(const float* src, int64_t n, uint8_t* blocks) {
    int64_t nb = (n + 31) / 32;
    for (int64_t bi = 0; bi < nb; bi++) {
        int64_t off = bi * 32;
        float absmax = 0.0f;
        for (int j = 0; j < 32; j++) {
            float v = (off + j < n) ? src[off + j] : 0.0f;
            float av = (float)fabs((double)v);
            if (av > absmax) absmax = av;
        }
        float scale = 0.0f;
        if (absmax > 0) scale = absmax / 127.0f;
        uint8_t* blk = blocks + bi * 36;
        memcpy(blk, &scale, 4);                       /* little-endian f32 (:427-438) */
        float inv = 0.0f;
        if (scale > 0) inv = 1.0f / scale;
        for (int j = 0; j < 32; j++) {
            float v = (off + j < n) ? src[off + j] : 0.0f;
            float p = v * inv;
            blk[4 + j] = (uint8_t)(int8_t)clamp_int(go_round_to_int(p), -128, 127);
        }
    }
}

/* tensor/quantized.go:344-355 */
void zo_dequantize_q8(const uint8_t* blocks, int64_t n, float* dst) {
    int64_t nb = (n + 31) / 32;
    for (int64_t bi = 0; bi < nb; bi++) {
        const uint8_t* blk = blocks + bi * 36;
        float scale;
        memcpy(&scale, blk, 4);
        int64_t off = bi * 32;
        for (int j = 0; j < 32; j++) {
            if (off + j >= n) break;
            dst[off + j] = (float)(int8_t)blk[4 + j] * scale;
        }
    }
}

/* ------------------------------------------------------------------ */
/* IQ4_NL                                                              */
/* ------------------------------------------------------------------ */

/* tensor/iq4_storage.go:28-33 */
static const float kIQ4NLTable[16] = {
    -1.0f, -0.6961928f, -0.5250730f, -0.3947555f,
    -0.2831612f, -0.1790887f, -0.0805542f, 0.0f,
    0.0805542f, 0.1790887f, 0.2831612f, 0.3947555f,
    0.5250730f, 0.6961928f, 1.0f, 1.3312578f,
};

void zo_iq4nl_table(float out[16]) { memcpy(out, kIQ4NLTable, sizeof(kIQ4NLTable)); }

/* tensor/iq4_storage.go:36-46 (one block) and :75-89 (storage, partial tail) */
void zo_dequantize_iq4nl(const uint8_t* raw, int64_t n, float* dst) {
    int64_t nb = (n + 31) / 32;
    for (int64_t bi = 0; bi < nb; bi++) {
        const uint8_t* blk = raw + bi * 18;
        float d = zo_f16_to_f32(rd16(blk));
        float tmp[32];
        for (int i = 0; i < 16; i++) {
            uint8_t lo = blk[2 + i] & 0x0f;
            uint8_t hi = blk[2 + i] >> 4;
            tmp[2 * i] = d * kIQ4NLTable[lo];
            tmp[2 * i + 1] = d * kIQ4NLTable[hi];
        }
        int64_t off = bi * 32;
        int64_t rem = n - off;
        if (rem > 32) rem = 32;
        memcpy(dst + off, tmp, (size_t)rem * sizeof(float));
    }
}

/* ------------------------------------------------------------------ */
/* ternary                                                             */
/* ------------------------------------------------------------------ */

/* tensor/ternary_storage.go:29-62: encoded = val+1 at bits 2*(i%4) of byte i/4 */
void zo_ternary_pack(const int8_t* vals, int64_t n, uint8_t* data) {
    memset(data, 0, (size_t)((n + 3) / 4));
    for (int64_t i = 0; i < n; i++) {
        uint8_t enc = (uint8_t)(vals[i] + 1);
        unsigned sh = (unsigned)(i % 4) * 2u;
        data[i / 4] = (uint8_t)((data[i / 4] & ~(0x03u << sh)) | ((enc & 0x03u) << sh));
    }
}

/* tensor/ternary_storage.go:39-47 */
int8_t zo_ternary_get(const uint8_t* data, int64_t i) {
    unsigned sh = (unsigned)(i % 4) * 2u;
    return (int8_t)((int8_t)((data[i / 4] >> sh) & 0x03u) - 1);
}

/* compute/ternary_gemv.go:12-77.  The byte-aligned fast path multiplies by a
 * 256x4 table of float32(int8(bits)-1) (so the unused code 3 decodes to +2
 * there, :70-76) and adds four products per byte in order; the other path adds
 * or subtracts x[j] per element. */
void zo_ternary_gemv(const uint8_t* raw, const float* x, int rows, int cols, float* y) {
    static float lut[256][4];
    static int lut_ready = 0;
    if (!lut_ready) {
        for (int b = 0; b < 256; b++)
            for (int k = 0; k < 4; k++)
                lut[b][k] = (float)((int8_t)((b >> (k * 2)) & 0x03) - 1);
        lut_ready = 1;
    }
    for (int i = 0; i < rows; i++) {
        float sum = 0.0f;
        int64_t base = (int64_t)i * cols;
        int j = 0;
        int64_t byte_start = base / 4;
        unsigned start_shift = (unsigned)(base % 4) * 2u;
        if (start_shift == 0) {
            int full = cols / 4;
            for (int bi = 0; bi < full; bi++) {
                const float* l = lut[raw[byte_start + bi]];
                float p;
                p = l[0] * x[j];     sum = sum + p;
                p = l[1] * x[j + 1]; sum = sum + p;
                p = l[2] * x[j + 2]; sum = sum + p;
                p = l[3] * x[j + 3]; sum = sum + p;
                j += 4;
            }
        }
        for (; j < cols; j++) {
            int64_t idx = base + j;
            unsigned bits = (raw[idx / 4] >> ((unsigned)(idx % 4) * 2u)) & 0x03u;
            if (bits == 0) sum -= x[j];
            else if (bits == 2) sum += x[j];
        }
        y[i] = sum;
    }
}

/* ------------------------------------------------------------------ */
/* GPTQ (4-bit) and AWQ                                                */
/* ------------------------------------------------------------------ */

int64_t zo_gptq4_data_bytes(int64_t n, int group) {
    int64_t ng = (n + group - 1) / group, total = 0;
    for (int64_t gi = 0; gi < ng; gi++) {
        int64_t cnt = n - gi * group; if (cnt > group) cnt = group;
        total += (cnt + 1) / 2;
    }
    return total;
}

int64_t zo_awq_data_bytes(int64_t n, int group) {
    int64_t ng = (n + group - 1) / group, total = 0;
    for (int64_t gi = 0; gi < ng; gi++) {
        int64_t cnt = n - gi * group; if (cnt > group) cnt = group;
        total += 4 * ((cnt + 7) / 8);
    }
    return total;
}

/* Shared min/max -> scale, zero (quantized_gptq.go:60-86, quantized_awq.go:60-83). */
static void group_scale_zero(const float* g, int64_t cnt, int maxval, uint16_t* s16, uint16_t* z16) {
    float mn = g[0], mx = g[0];
    for (int64_t j = 1; j < cnt; j++) {
        if (g[j] < mn) mn = g[j];
        if (g[j] > mx) mx = g[j];
    }
    float scale = 0.0f;
    float range = mx - mn;
    if (range > 0) scale = range / (float)maxval;
    float zero = 0.0f;
    if (scale > 0) zero = -mn / scale;
    *s16 = zo_f32_to_f16(scale);
    *z16 = zo_f32_to_f16(zero);
}

/* tensor/quantized_gptq.go:45-130, bits == 4 */
void zo_quantize_gptq4(const float* src, int64_t n, int group,
                       uint8_t* data, uint16_t* scales, uint16_t* zeros) {
    int64_t ng = (n + group - 1) / group;
    int64_t doff = 0;
    for (int64_t gi = 0; gi < ng; gi++) {
        int64_t off = gi * group;
        int64_t cnt = n - off; if (cnt > group) cnt = group;
        const float* g = src + off;
        group_scale_zero(g, cnt, 15, &scales[gi], &zeros[gi]);
        float sf = zo_f16_to_f32(scales[gi]);
        float zf = zo_f16_to_f32(zeros[gi]);
        float inv = 0.0f;
        if (sf > 0) inv = 1.0f / sf;
        int64_t plen = (cnt + 1) / 2;
        uint8_t* packed = data + doff;
        memset(packed, 0, (size_t)plen);
        for (int64_t j = 0; j < cnt; j++) {
            float p = g[j] * inv;
            float t = p + zf;
            int q = clamp_int(go_round_to_int(t), 0, 15);
            if ((j & 1) == 0) packed[j / 2] = (uint8_t)(q & 0xf);
            else packed[j / 2] |= (uint8_t)((q & 0xf) << 4);
        }
        doff += plen;
    }
}

/* tensor/quantized_gptq.go:134-163 */
void zo_dequantize_gptq4(const uint8_t* data, const uint16_t* scales, const uint16_t* zeros,
                         int64_t n, int group, float* dst) {
    int64_t ng = (n + group - 1) / group;
    int64_t doff = 0;
    for (int64_t gi = 0; gi < ng; gi++) {
        float scale = zo_f16_to_f32(scales[gi]);
        float zero = zo_f16_to_f32(zeros[gi]);
        int64_t off = gi * group;
        int64_t cnt = n - off; if (cnt > group) cnt = group;
        const uint8_t* packed = data + doff;
        for (int64_t j = 0; j < cnt; j++) {
            int q = (j & 1) ? (packed[j / 2] >> 4) : (packed[j / 2] & 0xf);
            float d = (float)q - zero;
            dst[off + j] = d * scale;
        }
        doff += (cnt + 1) / 2;
    }
}

/* tensor/quantized_awq.go:44-114: q = int(v*inv + zero + 0.5), truncating */
void zo_quantize_awq(const float* src, int64_t n, int group,
                     uint8_t* data, uint16_t* scales, uint16_t* zeros) {
    int64_t ng = (n + group - 1) / group;
    int64_t doff = 0;
    for (int64_t gi = 0; gi < ng; gi++) {
        int64_t off = gi * group;
        int64_t cnt = n - off; if (cnt > group) cnt = group;
        const float* g = src + off;
        group_scale_zero(g, cnt, 15, &scales[gi], &zeros[gi]);
        float sf = zo_f16_to_f32(scales[gi]);
        float zf = zo_f16_to_f32(zeros[gi]);
        float inv = 0.0f;
        if (sf > 0) inv = 1.0f / sf;
        int64_t words = (cnt + 7) / 8;
        uint8_t* packed = data + doff;
        memset(packed, 0, (size_t)words * 4);
        for (int64_t j = 0; j < cnt; j++) {
            float p = g[j] * inv;
            float t = p + zf;
            float u = t + 0.5f;
            int q = clamp_int((int)u, 0, 15);
            /* nibble j%8 of little-endian word j/8 == nibble j%2 of byte j/2 */
            int64_t byte = (j / 8) * 4 + (j % 8) / 2;
            packed[byte] |= (uint8_t)((q & 0xf) << (4 * (j & 1)));
        }
        doff += words * 4;
    }
}

/* tensor/quantized_awq.go:118-136 */
void zo_dequantize_awq(const uint8_t* data, const uint16_t* scales, const uint16_t* zeros,
                       int64_t n, int group, float* dst) {
    int64_t ng = (n + group - 1) / group;
    int64_t doff = 0;
    for (int64_t gi = 0; gi < ng; gi++) {
        float scale = zo_f16_to_f32(scales[gi]);
        float zero = zo_f16_to_f32(zeros[gi]);
        int64_t off = gi * group;
        int64_t cnt = n - off; if (cnt > group) cnt = group;
        const uint8_t* packed = data + doff;
        for (int64_t j = 0; j < cnt; j++) {
            int64_t byte = (j / 8) * 4 + (j % 8) / 2;
            int q = (packed[byte] >> (4 * (j & 1))) & 0xf;
            float d = (float)q - zero;
            dst[off + j] = d * scale;
        }
        doff += 4 * ((cnt + 7) / 8);
    }
}

/* ------------------------------------------------------------------ */
/* internal/xblas                                                      */
/* ------------------------------------------------------------------ */

/* sgemmAccRow, internal/xblas/gemm_simd_amd64.s:9-75: c[j] += a*b[j].
 * Lanes handled in 16/8/4-wide chunks use VFMADD231PS (one rounding); the
 * last n%4 elements use MULSS then ADDSS (two roundings). */
static void sgemm_acc_row(float* c, const float* b, float a, int n) {
    int j = 0;
#if defined(__AVX2__) && defined(__FMA__)
    __m256 va = _mm256_set1_ps(a);
    for (; n - j >= 16; j += 16) {
        __m256 c0 = _mm256_loadu_ps(c + j), c1 = _mm256_loadu_ps(c + j + 8);
        c0 = _mm256_fmadd_ps(va, _mm256_loadu_ps(b + j), c0);
        c1 = _mm256_fmadd_ps(va, _mm256_loadu_ps(b + j + 8), c1);
        _mm256_storeu_ps(c + j, c0);
        _mm256_storeu_ps(c + j + 8, c1);
    }
    if (n - j >= 8) {
        __m256 c0 = _mm256_fmadd_ps(va, _mm256_loadu_ps(b + j), _mm256_loadu_ps(c + j));
        _mm256_storeu_ps(c + j, c0);
        j += 8;
    }
    if (n - j >= 4) {
        __m128 c0 = _mm_fmadd_ps(_mm256_castps256_ps128(va), _mm_loadu_ps(b + j), _mm_loadu_ps(c + j));
        _mm_storeu_ps(c + j, c0);
        j += 4;
    }
#else
    int nv = n & ~3;
    for (; j < nv; j++) c[j] = fmaf(a, b[j], c[j]);
#endif
    for (; j < n; j++) {
        float t = b[j] * a;
        c[j] = t + c[j];
    }
}

/* SgemmSimd, internal/xblas/gemm_simd_amd64.go:16-36 */
void zo_sgemm_simd(int m, int n, int k, const float* a, const float* b, float* c) {
    if (m == 0 || n == 0 || k == 0) return;
    for (int p0 = 0; p0 < k; p0 += 256) {
        int p1 = p0 + 256 < k ? p0 + 256 : k;
        for (int i = 0; i < m; i++) {
            float* crow = c + (int64_t)i * n;
            for (int p = p0; p < p1; p++) {
                float av = a[(int64_t)i * k + p];
                if (av != 0) sgemm_acc_row(crow, b + (int64_t)p * n, av, n);
            }
        }
    }
}

/* GemmQ4F32Fused, internal/xblas/gemm_quant.go:37-74 with dequantQ4Block :637-644.
 * k must be a multiple of 32 (the reference's fallback for other k calls
 * itself and never returns; nothing is computed for such k here). */
void zo_gemm_q4_f32_fused(int m, int n, int k, const uint8_t* a, const float* b, float* c) {
    if (k % 32 != 0) return;
    int bpr = k / 32;
    for (int64_t i = 0; i < (int64_t)m * n; i++) c[i] = 0.0f;
    float buf[32];
    for (int i = 0; i < m; i++) {
        float* crow = c + (int64_t)i * n;
        for (int bi = 0; bi < bpr; bi++) {
            const uint8_t* blk = a + ((int64_t)i * bpr + bi) * 18;
            float scale = zo_f16_to_f32(rd16(blk));     /* BlockScaleF32, quantized.go:215-217 */
            if (scale == 0) continue;
            for (int p = 0; p < 16; p++) {
                uint8_t bv = blk[2 + p];
                buf[p] = (float)((int)(bv & 0x0f) - 8) * scale;
                buf[p + 16] = (float)((int)(bv >> 4) - 8) * scale;
            }
            int kbase = bi * 32;
            for (int p = 0; p < 32; p++) {
                float av = buf[p];
                if (av != 0) sgemm_acc_row(crow, b + (int64_t)(kbase + p) * n, av, n);
            }
        }
    }
}

/* q4DotRowScalar + q4DotBlockScalar, internal/xblas/q4dot.go:10-52 */
static float q4_dot_row(const uint8_t* base, const float* x, int nblocks) {
    float total = 0.0f;
    for (int bi = 0; bi < nblocks; bi++) {
        const uint8_t* blk = base + (int64_t)bi * 18;
        float scale = zo_xblas_f16_bits_to_f32(rd16(blk));
        const float* xs = x + (int64_t)bi * 32;
        float sum = 0.0f;
        for (int p = 0; p < 16; p++) {
            uint8_t bv = blk[2 + p];
            float lo = (float)((int)(bv & 0x0f) - 8);
            float hi = (float)((int)(bv >> 4) - 8);
            float t = lo * xs[p];
            sum = sum + t;
            t = hi * xs[p + 16];
            sum = sum + t;
        }
        float bs = sum * scale;
        total = total + bs;
    }
    return total;
}

int zo_num_cpu(void) {
    long n = sysconf(_SC_NPROCESSORS_ONLN);
    return n > 0 ? (int)n : 1;
}

/* internal/xblas/gemm_quant.go:99-105 */
int zo_nt_threads(int n, int k, int ncpu) {
    if (ncpu <= 0) ncpu = zo_num_cpu();
    if ((int64_t)n * k < 256 * 256) return 1;
    int c = ncpu < n / 4 ? ncpu : n / 4;
    return c > 1 ? c : 1;
}

typedef struct {
    int kind;            /* 4 or 8 */
    int j0, j1, bpr;
    const float* a;
    const uint8_t* b;
    float* c;
} nt_task;

static void q8_rows(const nt_task* t) {
    float buf[32];
    for (int j = t->j0; j < t->j1; j++) {
        float sum = 0.0f;
        for (int bi = 0; bi < t->bpr; bi++) {
            const uint8_t* blk = t->b + ((int64_t)j * t->bpr + bi) * 36;
            float scale;
            memcpy(&scale, blk, 4);
            for (int p = 0; p < 32; p++) buf[p] = (float)(int8_t)blk[4 + p] * scale; /* DequantizeBlock, quantized.go:358-363 */
            const float* as = t->a + (int64_t)bi * 32;
            for (int p = 0; p < 32; p++) {
                float pr = as[p] * buf[p];
                sum = sum + pr;
            }
        }
        t->c[j] = sum;
    }
}

static void* nt_worker(void* arg) {
    const nt_task* t = (const nt_task*)arg;
    if (t->kind == 4) {
        for (int j = t->j0; j < t->j1; j++)
            t->c[j] = q4_dot_row(t->b + (int64_t)j * t->bpr * 18, t->a, t->bpr);
    } else {
        q8_rows(t);
    }
    return NULL;
}

/* Row-chunked fan-out of the m==1 NT paths (gemm_quant.go:122-157, 209-264). */
static void nt_parallel(int kind, int n, const float* a, const uint8_t* b, float* c, int bpr, int ncores) {
    int chunk = (n + ncores - 1) / ncores;
    pthread_t* th = (pthread_t*)malloc(sizeof(pthread_t) * (size_t)ncores);
    nt_task* tk = (nt_task*)malloc(sizeof(nt_task) * (size_t)ncores);
    int used = 0;
    for (int t = 0; t < ncores; t++) {
        int j0 = t * chunk;
        if (j0 >= n) break;
        int j1 = j0 + chunk < n ? j0 + chunk : n;
        tk[used] = (nt_task){kind, j0, j1, bpr, a, b, c};
        used++;
    }
    for (int t = 1; t < used; t++) pthread_create(&th[t], NULL, nt_worker, &tk[t]);
    if (used > 0) nt_worker(&tk[0]);
    for (int t = 1; t < used; t++) pthread_join(th[t], NULL);
    free(th);
    free(tk);
}

/* GemmF32Q4NT, internal/xblas/gemm_quant.go:81-120 (k % 32 == 0 only) */
void zo_gemm_f32_q4_nt(int m, int n, int k, const float* a, const uint8_t* b, float* c, int ncpu) {
    if (k % 32 != 0) return;
    int bpr = k / 32;
    if (m == 1) {
        int nc = zo_nt_threads(n, k, ncpu);
        if (nc > 1) { nt_parallel(4, n, a, b, c, bpr, nc); return; }
    }
    for (int i = 0; i < m; i++)
        for (int j = 0; j < n; j++)
            c[(int64_t)i * n + j] = q4_dot_row(b + (int64_t)j * bpr * 18, a + (int64_t)i * k, bpr);
}

/* GemmQ8F32, internal/xblas/gemm_quant.go:24-28 */
void zo_gemm_q8_f32(int m, int n, int k, const uint8_t* a, const float* b, float* c) {
    int64_t len = (int64_t)m * k;
    float* af = (float*)malloc(sizeof(float) * (size_t)len);
    zo_dequantize_q8(a, len, af);
    zo_sgemm_simd(m, n, k, af, b, c);
    free(af);
}

/* GemmF32Q8NT, internal/xblas/gemm_quant.go:163-207 (k % 32 == 0 only) */
void zo_gemm_f32_q8_nt(int m, int n, int k, const float* a, const uint8_t* b, float* c, int ncpu) {
    if (k % 32 != 0) return;
    int bpr = k / 32;
    if (m == 1) {
        int nc = zo_nt_threads(n, k, ncpu);
        if (nc > 1) { nt_parallel(8, n, a, b, c, bpr, nc); return; }
    }
    for (int i = 0; i < m; i++) {
        nt_task t = {8, 0, n, bpr, a + (int64_t)i * k, b, c + (int64_t)i * n};
        q8_rows(&t);
    }
}

/* internal/cuda/kernels/fused_add_rmsnorm.cu:13-50, one row of length D: the block of `block` threads (the power
 * of two the launcher picks, :67-69) sums squares per thread over a strided range (:30-35), reduces them with a
 * halving tree (:39-44) and scales by rsqrt(mean + eps) (:47).  residual may be NULL (then sum = input). */
void zo_fused_add_rmsnorm(const float* input, const float* residual, const float* weight, float* normed_out,
                          float* sum_out, float eps, int D) {
    int block = 1;
    while (block < D && block < 256) block <<= 1;
    float sdata[256];
    for (int t = 0; t < block; t++) {
        float local_sq = 0.0f;
        for (int i = t; i < D; i += block) {
            float v = residual ? input[i] + residual[i] : input[i];
            sum_out[i] = v;
            float sq = v * v;
            local_sq = local_sq + sq;
        }
        sdata[t] = local_sq;
    }
    for (int s = block / 2; s > 0; s >>= 1)
        for (int t = 0; t < s; t++) sdata[t] = sdata[t] + sdata[t + s];
    float mean = sdata[0] / (float)D;
    float scale = 1.0f / sqrtf(mean + eps);
    for (int i = 0; i < D; i++) {
        float a = sum_out[i] * scale;
        normed_out[i] = a * weight[i];
    }
}

/* internal/cuda/kernels/fused_swiglu.cu:10-21 */
void zo_fused_swiglu(const float* w1, const float* w3, float* out, int n) {
    for (int i = 0; i < n; i++) {
        float x = w1[i];
        float gate = 1.0f / (1.0f + expf(-x));
        float a = x * gate;
        out[i] = a * w3[i];
    }
}

/* ======================================================================== Q4_K
 * tensor/quantized_kquant.go.  A super-block: fp16 d, fp16 dmin, 12 bytes of 6-bit scales and mins of the eight
 * 32-weight sub-blocks, 128 bytes of nibbles; per 64 weights 32 bytes, low nibbles = the first 32, high = the next 32. */
void zo_q4k_scales_mins(const uint8_t* block, uint8_t* scales, uint8_t* mins) {       /* :34-49 */
    const uint8_t* sc = block + 4;
    for (int i = 0; i < 4; i++) {
        scales[i] = sc[i] & 63;
        mins[i] = sc[4 + i] & 63;
    }
    for (int i = 0; i < 4; i++) {
        scales[4 + i] = (uint8_t)((sc[8 + i] & 0x0F) | ((sc[i] >> 6) << 4));
        mins[4 + i] = (uint8_t)((sc[8 + i] >> 4) | ((sc[4 + i] >> 6) << 4));
    }
}

static void q4k_dequant_block(const uint8_t* raw, float* dst) {                        /* DequantizeQ4K, :54-78 */
    float d = zo_f16_to_f32(rd16(raw));
    float dmin = zo_f16_to_f32(rd16(raw + 2));
    uint8_t scales[8], mins[8];
    zo_q4k_scales_mins(raw, scales, mins);
    const uint8_t* q = raw + 16;
    for (int g = 0; g < 4; g++) {
        float sc0 = d * (float)scales[2 * g], mn0 = dmin * (float)mins[2 * g];
        float sc1 = d * (float)scales[2 * g + 1], mn1 = dmin * (float)mins[2 * g + 1];
        for (int l = 0; l < 32; l++) {
            uint8_t b = q[g * 32 + l];
            float t0 = sc0 * (float)(b & 0x0F);
            float t1 = sc1 * (float)(b >> 4);
            dst[g * 64 + l] = t0 - mn0;
            dst[g * 64 + l + 32] = t1 - mn1;
        }
    }
}

static void q4k_dequant_sub(const uint8_t* raw, int sub, float* dst) {                 /* DequantizeSubBlock, :82-104 */
    float d = zo_f16_to_f32(rd16(raw));
    float dmin = zo_f16_to_f32(rd16(raw + 2));
    uint8_t scales[8], mins[8];
    zo_q4k_scales_mins(raw, scales, mins);
    float sc = d * (float)scales[sub], mn = dmin * (float)mins[sub];
    const uint8_t* q = raw + 16 + (sub / 2) * 32;
    for (int l = 0; l < 32; l++) {
        float t = sc * (float)((sub & 1) ? (q[l] >> 4) : (q[l] & 0x0F));
        dst[l] = t - mn;
    }
}

void zo_dequantize_q4k(const uint8_t* raw, int64_t n, float* dst) {                    /* :263-277: whole blocks, then a clipped tail */
    int64_t nb = (n + 255) / 256;
    float tmp[256];
    for (int64_t bi = 0; bi < nb; bi++) {
        int64_t off = bi * 256;
        if (off + 256 <= n) q4k_dequant_block(raw + bi * 144, dst + off);
        else {
            q4k_dequant_block(raw + bi * 144, tmp);
            for (int64_t i = 0; off + i < n; i++) dst[off + i] = tmp[i];
        }
    }
}

void zo_quantize_q4k(const float* src, int64_t n, uint8_t* raw) {                      /* QuantizeQ4K, :108-233 */
    int64_t nb = (n + 255) / 256;
    for (int64_t bi = 0; bi < nb; bi++) {
        float values[256];
        for (int i = 0; i < 256; i++) values[i] = (bi * 256 + i < n) ? src[bi * 256 + i] : 0.0f;
        float sub_scale[8], sub_min[8];
        for (int sb = 0; sb < 8; sb++) {
            float mn = values[sb * 32], mx = values[sb * 32];
            for (int j = 1; j < 32; j++) {
                float v = values[sb * 32 + j];
                if (v < mn) mn = v;
                if (v > mx) mx = v;
            }
            if (mn > 0) mn = 0;
            float range = mx - mn;
            sub_scale[sb] = range / 15.0f;
            sub_min[sb] = -mn;
        }
        float max_scale = 0, max_min = 0;
        for (int sb = 0; sb < 8; sb++) {
            if (sub_scale[sb] > max_scale) max_scale = sub_scale[sb];
            if (sub_min[sb] > max_min) max_min = sub_min[sb];
        }
        float d = max_scale / 63.0f, dmin = max_min / 63.0f;
        uint8_t sq[8] = {0}, mq[8] = {0};
        for (int sb = 0; sb < 8; sb++) {
            if (d > 0) {
                float r = sub_scale[sb] / d;
                int v = (int)((double)r + 0.5);
                if (v > 63) v = 63;
                sq[sb] = (uint8_t)v;
            }
            if (dmin > 0) {
                float r = sub_min[sb] / dmin;
                int v = (int)((double)r + 0.5);
                if (v > 63) v = 63;
                mq[sb] = (uint8_t)v;
            }
        }
        uint8_t* blk = raw + bi * 144;
        uint16_t d16 = zo_f32_to_f16(d), dmin16 = zo_f32_to_f16(dmin);
        wr16(blk, d16);
        wr16(blk + 2, dmin16);
        for (int i = 0; i < 4; i++) {
            blk[4 + i] = (uint8_t)((sq[i] & 63) | ((sq[4 + i] >> 4) << 6));
            blk[8 + i] = (uint8_t)((mq[i] & 63) | ((mq[4 + i] >> 4) << 6));
        }
        for (int i = 0; i < 4; i++) blk[12 + i] = (uint8_t)((sq[4 + i] & 0x0F) | ((mq[4 + i] & 0x0F) << 4));
        float drt = zo_f16_to_f32(d16), dminrt = zo_f16_to_f32(dmin16);
        for (int g = 0; g < 4; g++) {
            float sc0 = drt * (float)sq[2 * g], mn0 = dminrt * (float)mq[2 * g];
            float sc1 = drt * (float)sq[2 * g + 1], mn1 = dminrt * (float)mq[2 * g + 1];
            float inv0 = sc0 > 0 ? 1.0f / sc0 : 0.0f, inv1 = sc1 > 0 ? 1.0f / sc1 : 0.0f;
            for (int l = 0; l < 32; l++) {
                float a0 = values[g * 64 + l] + mn0, a1 = values[g * 64 + l + 32] + mn1;
                float p0 = a0 * inv0, p1 = a1 * inv1;
                int q0 = (int)((double)p0 + 0.5), q1 = (int)((double)p1 + 0.5);
                if (q0 < 0) q0 = 0; else if (q0 > 15) q0 = 15;
                if (q1 < 0) q1 = 0; else if (q1 > 15) q1 = 15;
                blk[16 + g * 32 + l] = (uint8_t)(q0 | (q1 << 4));
            }
        }
    }
}

void zo_gemm_q4k_f32(int m, int n, int k, const uint8_t* a, const float* b, float* c) {   /* gemm_q4k.go:15-50 */
    if (k % 256 != 0) return;
    int spr = k / 256;
    for (int64_t i = 0; i < (int64_t)m * n; i++) c[i] = 0.0f;
    float buf[32];
    for (int i = 0; i < m; i++) {
        float* crow = c + (int64_t)i * n;
        for (int sbi = 0; sbi < spr; sbi++) {
            const uint8_t* blk = a + ((int64_t)i * spr + sbi) * 144;
            for (int sub = 0; sub < 8; sub++) {
                int kbase = sbi * 256 + sub * 32;
                q4k_dequant_sub(blk, sub, buf);
                for (int p = 0; p < 32; p++) {
                    float av = buf[p];
                    if (av != 0) sgemm_acc_row(crow, b + (int64_t)(kbase + p) * n, av, n);
                }
            }
        }
    }
}

static float q4k_dot_row(const uint8_t* base, const float* x, int spr) {                /* gemm_q4k.go:86-98: one running sum */
    float sum = 0.0f;
    float buf[32];
    for (int sbi = 0; sbi < spr; sbi++) {
        for (int sub = 0; sub < 8; sub++) {
            q4k_dequant_sub(base + (int64_t)sbi * 144, sub, buf);
            const float* xs = x + sbi * 256 + sub * 32;
            for (int p = 0; p < 32; p++) {
                float pr = xs[p] * buf[p];
                sum = sum + pr;
            }
        }
    }
    return sum;
}

typedef struct { int j0, j1, spr; const float* a; const uint8_t* b; float* c; } q4k_task;
static void* q4k_worker(void* arg) {
    const q4k_task* t = (const q4k_task*)arg;
    for (int j = t->j0; j < t->j1; j++) t->c[j] = q4k_dot_row(t->b + (int64_t)j * t->spr * 144, t->a, t->spr);
    return NULL;
}

void zo_gemm_f32_q4k_nt(int m, int n, int k, const float* a, const uint8_t* b, float* c, int ncpu) {   /* gemm_q4k.go:54-140 */
    if (k % 256 != 0) return;
    int spr = k / 256;
    if (m == 1) {
        int nc = zo_nt_threads(n, k, ncpu);          /* same threshold and min(cores, n/4) rule as the Q4_0 path (:76-83) */
        if (nc > 1) {
            int chunk = (n + nc - 1) / nc;
            pthread_t* th = (pthread_t*)malloc(sizeof(pthread_t) * (size_t)nc);
            q4k_task* tk = (q4k_task*)malloc(sizeof(q4k_task) * (size_t)nc);
            int used = 0;
            for (int t = 0; t < nc; t++) {
                int j0 = t * chunk;
                if (j0 >= n) break;
                int j1 = j0 + chunk < n ? j0 + chunk : n;
                tk[used++] = (q4k_task){j0, j1, spr, a, b, c};
            }
            for (int t = 1; t < used; t++) pthread_create(&th[t], NULL, q4k_worker, &tk[t]);
            if (used > 0) q4k_worker(&tk[0]);
            for (int t = 1; t < used; t++) pthread_join(th[t], NULL);
            free(th);
            free(tk);
            return;
        }
    }
    for (int i = 0; i < m; i++)
        for (int j = 0; j < n; j++)
            c[(int64_t)i * n + j] = q4k_dot_row(b + (int64_t)j * spr * 144, a + (int64_t)i * k, spr);
}

/* ======================================================================== Q5_K
 * tensor/quantized_kquant.go:489-552.  Header and scale region as Q4_K; 128 bytes ql (low nibbles = first 32 of a
 * group of 64, high nibbles = next 32), 32 bytes qh: bit 2g of qh[l] is the fifth bit of element l of group g's
 * first half, bit 2g+1 of its second half. */
static void q5k_dequant_block(const uint8_t* raw, float* dst) {                        /* DequantizeQ5K, :511-552 */
    float d = zo_f16_to_f32(rd16(raw));
    float dmin = zo_f16_to_f32(rd16(raw + 2));
    uint8_t scales[8], mins[8];
    zo_q4k_scales_mins(raw, scales, mins);
    const uint8_t* ql = raw + 16;
    const uint8_t* qh = raw + 144;
    uint8_t u1 = 1, u2 = 2;
    for (int g = 0; g < 4; g++) {
        float sc0 = d * (float)scales[2 * g], mn0 = dmin * (float)mins[2 * g];
        float sc1 = d * (float)scales[2 * g + 1], mn1 = dmin * (float)mins[2 * g + 1];
        for (int l = 0; l < 32; l++) {
            uint8_t q = ql[g * 32 + l], hb = qh[l];
            uint8_t h0 = (hb & u1) ? 16 : 0, h1 = (hb & u2) ? 16 : 0;
            float t0 = sc0 * (float)((q & 0x0F) | h0);
            float t1 = sc1 * (float)((q >> 4) | h1);
            dst[g * 64 + l] = t0 - mn0;
            dst[g * 64 + l + 32] = t1 - mn1;
        }
        u1 = (uint8_t)(u1 << 2);
        u2 = (uint8_t)(u2 << 2);
    }
}

void zo_dequantize_q5k(const uint8_t* raw, int64_t n, float* dst) {                    /* :579-596 */
    int64_t nb = (n + 255) / 256;
    float tmp[256];
    for (int64_t bi = 0; bi < nb; bi++) {
        int64_t off = bi * 256;
        if (off + 256 <= n) q5k_dequant_block(raw + bi * 176, dst + off);
        else {
            q5k_dequant_block(raw + bi * 176, tmp);
            for (int64_t i = 0; off + i < n; i++) dst[off + i] = tmp[i];
        }
    }
}

/* Test-data generator (the reference only reads Q5_K): the Q4_K quantizer's recipe with 31 levels.  Parity is
 * on the bytes this writes, whatever their quality. */
void zo_make_q5k_blocks(const float* src, int64_t n, uint8_t* raw) {
    int64_t nb = (n + 255) / 256;
    for (int64_t bi = 0; bi < nb; bi++) {
        float values[256];
        for (int i = 0; i < 256; i++) values[i] = (bi * 256 + i < n) ? src[bi * 256 + i] : 0.0f;
        float sub_scale[8], sub_min[8], max_scale = 0, max_min = 0;
        for (int sb = 0; sb < 8; sb++) {
            float mn = values[sb * 32], mx = values[sb * 32];
            for (int j = 1; j < 32; j++) {
                float v = values[sb * 32 + j];
                if (v < mn) mn = v;
                if (v > mx) mx = v;
            }
            if (mn > 0) mn = 0;
            sub_scale[sb] = (mx - mn) / 31.0f;
            sub_min[sb] = -mn;
            if (sub_scale[sb] > max_scale) max_scale = sub_scale[sb];
            if (sub_min[sb] > max_min) max_min = sub_min[sb];
        }
        float d = max_scale / 63.0f, dmin = max_min / 63.0f;
        uint8_t sq[8] = {0}, mq[8] = {0};
        for (int sb = 0; sb < 8; sb++) {
            if (d > 0) { int v = (int)((double)(sub_scale[sb] / d) + 0.5); sq[sb] = (uint8_t)(v > 63 ? 63 : v); }
            if (dmin > 0) { int v = (int)((double)(sub_min[sb] / dmin) + 0.5); mq[sb] = (uint8_t)(v > 63 ? 63 : v); }
        }
        uint8_t* blk = raw + bi * 176;
        for (int i = 0; i < 176; i++) blk[i] = 0;
        uint16_t d16 = zo_f32_to_f16(d), dmin16 = zo_f32_to_f16(dmin);
        wr16(blk, d16);
        wr16(blk + 2, dmin16);
        for (int i = 0; i < 4; i++) {
            blk[4 + i] = (uint8_t)((sq[i] & 63) | ((sq[4 + i] >> 4) << 6));
            blk[8 + i] = (uint8_t)((mq[i] & 63) | ((mq[4 + i] >> 4) << 6));
            blk[12 + i] = (uint8_t)((sq[4 + i] & 0x0F) | ((mq[4 + i] & 0x0F) << 4));
        }
        float drt = zo_f16_to_f32(d16), dminrt = zo_f16_to_f32(dmin16);
        for (int g = 0; g < 4; g++) {
            float sc0 = drt * (float)sq[2 * g], mn0 = dminrt * (float)mq[2 * g];
            float sc1 = drt * (float)sq[2 * g + 1], mn1 = dminrt * (float)mq[2 * g + 1];
            float inv0 = sc0 > 0 ? 1.0f / sc0 : 0.0f, inv1 = sc1 > 0 ? 1.0f / sc1 : 0.0f;
            for (int l = 0; l < 32; l++) {
                int q0 = (int)((double)((values[g * 64 + l] + mn0) * inv0) + 0.5);
                int q1 = (int)((double)((values[g * 64 + l + 32] + mn1) * inv1) + 0.5);
                if (q0 < 0) q0 = 0; else if (q0 > 31) q0 = 31;
                if (q1 < 0) q1 = 0; else if (q1 > 31) q1 = 31;
                blk[16 + g * 32 + l] = (uint8_t)((q0 & 15) | ((q1 & 15) << 4));
                if (q0 & 16) blk[144 + l] |= (uint8_t)(1u << (2 * g));
                if (q1 & 16) blk[144 + l] |= (uint8_t)(1u << (2 * g + 1));
            }
        }
    }
}

static float q5k_dot_row(const uint8_t* base, const float* x, int bpr) {               /* gemm_quant.go:303-313: one running sum */
    float sum = 0.0f, buf[256];
    for (int bi = 0; bi < bpr; bi++) {
        q5k_dequant_block(base + (int64_t)bi * 176, buf);
        const float* xs = x + bi * 256;
        for (int p = 0; p < 256; p++) {
            float pr = xs[p] * buf[p];
            sum = sum + pr;
        }
    }
    return sum;
}

typedef struct { int j0, j1, bpr; const float* a; const uint8_t* b; float* c; } q5k_task;
static void* q5k_worker(void* arg) {
    const q5k_task* t = (const q5k_task*)arg;
    for (int j = t->j0; j < t->j1; j++) t->c[j] = q5k_dot_row(t->b + (int64_t)j * t->bpr * 176, t->a, t->bpr);
    return NULL;
}

void zo_gemm_f32_q5k_nt(int m, int n, int k, const float* a, const uint8_t* b, float* c, int ncpu) {   /* gemm_quant.go:273-360 */
    if (k % 256 != 0) return;
    int bpr = k / 256;
    if (m == 1) {
        int nc = zo_nt_threads(n, k, ncpu);          /* q5kGemvParallelThreshold == 256 * 256, min(cores, n / 4) (:266-298) */
        if (nc > 1) {
            int chunk = (n + nc - 1) / nc;
            pthread_t* th = (pthread_t*)malloc(sizeof(pthread_t) * (size_t)nc);
            q5k_task* tk = (q5k_task*)malloc(sizeof(q5k_task) * (size_t)nc);
            int used = 0;
            for (int t = 0; t < nc; t++) {
                int j0 = t * chunk;
                if (j0 >= n) break;
                int j1 = j0 + chunk < n ? j0 + chunk : n;
                tk[used++] = (q5k_task){j0, j1, bpr, a, b, c};
            }
            for (int t = 1; t < used; t++) pthread_create(&th[t], NULL, q5k_worker, &tk[t]);
            if (used > 0) q5k_worker(&tk[0]);
            for (int t = 1; t < used; t++) pthread_join(th[t], NULL);
            free(th);
            free(tk);
            return;
        }
    }
    for (int i = 0; i < m; i++)
        for (int j = 0; j < n; j++)
            c[(int64_t)i * n + j] = q5k_dot_row(b + (int64_t)j * bpr * 176, a + (int64_t)i * k, bpr);
}

/* ======================================================================== Q6_K
 * tensor/quantized_kquant.go:335-382.  ql[128] low nibbles, qh[64] high two bits, int8 scales[16] (one per 16
 * weights), fp16 d.  Per half of 128: byte ql[l] / ql[32+l] and qh[l] carry elements l, 32+l, 64+l, 96+l. */
static void q6k_dequant_block(const uint8_t* raw, float* dst) {                        /* DequantizeQ6K, :355-382 */
    const uint8_t* ql = raw;
    const uint8_t* qh = raw + 128;
    const int8_t* sc = (const int8_t*)(raw + 192);
    float d = zo_f16_to_f32(rd16(raw + 208));
    for (int half = 0; half < 2; half++) {
        const uint8_t* l4 = ql + half * 64;
        const uint8_t* h2 = qh + half * 32;
        const int8_t* s8 = sc + half * 8;
        float* out = dst + half * 128;
        for (int l = 0; l < 32; l++) {
            int is = l / 16;
            int q1 = (int)(int8_t)((l4[l] & 0x0F) | ((h2[l] & 3) << 4)) - 32;
            int q2 = (int)(int8_t)((l4[32 + l] & 0x0F) | (((h2[l] >> 2) & 3) << 4)) - 32;
            int q3 = (int)(int8_t)((l4[l] >> 4) | (((h2[l] >> 4) & 3) << 4)) - 32;
            int q4 = (int)(int8_t)((l4[32 + l] >> 4) | (((h2[l] >> 6) & 3) << 4)) - 32;
            float t;
            t = d * (float)s8[is + 0]; out[l] = t * (float)q1;
            t = d * (float)s8[is + 2]; out[32 + l] = t * (float)q2;
            t = d * (float)s8[is + 4]; out[64 + l] = t * (float)q3;
            t = d * (float)s8[is + 6]; out[96 + l] = t * (float)q4;
        }
    }
}

void zo_dequantize_q6k(const uint8_t* raw, int64_t n, float* dst) {                    /* :411-428 */
    int64_t nb = (n + 255) / 256;
    float tmp[256];
    for (int64_t bi = 0; bi < nb; bi++) {
        int64_t off = bi * 256;
        if (off + 256 <= n) q6k_dequant_block(raw + bi * 210, dst + off);
        else {
            q6k_dequant_block(raw + bi * 210, tmp);
            for (int64_t i = 0; off + i < n; i++) dst[off + i] = tmp[i];
        }
    }
}

/* Test-data generator (the reference only reads Q6_K): d = absmax / (31 * 127), int8 scale per 16 weights,
 * 6-bit codes round(v / (d * scale)) + 32 -- the recipe of the reference's own test builder.  Parity is on the
 * bytes this writes. */
void zo_make_q6k_blocks(const float* src, int64_t n, uint8_t* raw) {
    int64_t nb = (n + 255) / 256;
    for (int64_t bi = 0; bi < nb; bi++) {
        float values[256];
        uint8_t* blk = raw + bi * 210;
        for (int i = 0; i < 210; i++) blk[i] = 0;
        float absmax = 0;
        for (int i = 0; i < 256; i++) {
            values[i] = (bi * 256 + i < n) ? src[bi * 256 + i] : 0.0f;
            float av = fabsf(values[i]);
            if (av > absmax) absmax = av;
        }
        float d = absmax / (31.0f * 127.0f);
        if (d == 0) continue;
        uint16_t d16 = zo_f32_to_f16(d);
        float drt = zo_f16_to_f32(d16);
        if (drt == 0) continue;
        int8_t sub[16];
        for (int sb = 0; sb < 16; sb++) {
            float mx = 0;
            for (int j = 0; j < 16; j++) { float av = fabsf(values[sb * 16 + j]); if (av > mx) mx = av; }
            float s = mx / (drt * 31.0f);
            if (s > 127) s = 127;
            sub[sb] = (int8_t)(int)((double)s + 0.5);
            blk[192 + sb] = (uint8_t)sub[sb];
        }
        int q[256];
        for (int pos = 0; pos < 256; pos++) {
            float s = drt * (float)sub[pos / 16];
            int v = 32;
            if (s > 0) {
                double r = (double)(values[pos] / s);
                v = (int)(r < 0 ? r - 0.5 : r + 0.5) + 32;
                if (v < 0) v = 0; else if (v > 63) v = 63;
            }
            q[pos] = v;
        }
        for (int half = 0; half < 2; half++)
            for (int l = 0; l < 32; l++) {
                int q1 = q[half * 128 + l], q2 = q[half * 128 + 32 + l], q3 = q[half * 128 + 64 + l], q4 = q[half * 128 + 96 + l];
                blk[half * 64 + l] = (uint8_t)((q1 & 0x0F) | ((q3 & 0x0F) << 4));
                blk[half * 64 + 32 + l] = (uint8_t)((q2 & 0x0F) | ((q4 & 0x0F) << 4));
                blk[128 + half * 32 + l] = (uint8_t)(((q1 >> 4) & 3) | (((q2 >> 4) & 3) << 2) | (((q3 >> 4) & 3) << 4) | (((q4 >> 4) & 3) << 6));
            }
        wr16(blk + 208, d16);
    }
}

static float q6k_dot_row(const uint8_t* base, const float* x, int bpr) {               /* gemm_quant.go:413-425: one running sum */
    float sum = 0.0f, buf[256];
    for (int bi = 0; bi < bpr; bi++) {
        q6k_dequant_block(base + (int64_t)bi * 210, buf);
        const float* xs = x + bi * 256;
        for (int p = 0; p < 256; p++) {
            float pr = xs[p] * buf[p];
            sum = sum + pr;
        }
    }
    return sum;
}

typedef struct { int j0, j1, bpr; const float* a; const uint8_t* b; float* c; } q6k_task;
static void* q6k_worker(void* arg) {
    const q6k_task* t = (const q6k_task*)arg;
    for (int j = t->j0; j < t->j1; j++) t->c[j] = q6k_dot_row(t->b + (int64_t)j * t->bpr * 210, t->a, t->bpr);
    return NULL;
}

void zo_gemm_f32_q6k_nt(int m, int n, int k, const float* a, const uint8_t* b, float* c, int ncpu) {   /* gemm_quant.go:384-470 */
    if (k % 256 != 0) return;
    int bpr = k / 256;
    if (m == 1) {
        int nc = zo_nt_threads(n, k, ncpu);          /* q6kGemvParallelThreshold == 256 * 256, min(cores, n / 4) */
        if (nc > 1) {
            int chunk = (n + nc - 1) / nc;
            pthread_t* th = (pthread_t*)malloc(sizeof(pthread_t) * (size_t)nc);
            q6k_task* tk = (q6k_task*)malloc(sizeof(q6k_task) * (size_t)nc);
            int used = 0;
            for (int t = 0; t < nc; t++) {
                int j0 = t * chunk;
                if (j0 >= n) break;
                int j1 = j0 + chunk < n ? j0 + chunk : n;
                tk[used++] = (q6k_task){j0, j1, bpr, a, b, c};
            }
            for (int t = 1; t < used; t++) pthread_create(&th[t], NULL, q6k_worker, &tk[t]);
            if (used > 0) q6k_worker(&tk[0]);
            for (int t = 1; t < used; t++) pthread_join(th[t], NULL);
            free(th);
            free(tk);
            return;
        }
    }
    for (int i = 0; i < m; i++)
        for (int j = 0; j < n; j++)
            c[(int64_t)i * n + j] = q6k_dot_row(b + (int64_t)j * bpr * 210, a + (int64_t)i * k, bpr);
}
