// formats.cuh -- device-side quantizers, dequantizers and residency repacks.
//
// The quantizers reproduce the reference's CPU quantizers bit for bit
// (tensor/quantized.go:37-91, 301-341; tensor/quantized_gptq.go:45-130;
// tensor/quantized_awq.go:44-114): every float32 operation is an explicit
// round-to-nearest intrinsic so nothing is contracted into an FMA, rounding to
// integer is half-away-from-zero (GPTQ, Q4_0, Q8_0) or add-0.5-and-truncate (AWQ).
#pragma once

#include "gemv_stream.cuh"

namespace ztq {

__device__ __forceinline__ int clampi(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }

// ---------------------------------------------------------------- repacks
__global__ void repack_blocks18_kernel(const uint8_t* __restrict__ aos, uint8_t* __restrict__ sep, long long nb,
                                       long long data_off) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;   // one thread per 2 source bytes
    const long long blk = i / 9;
    const int part = (int)(i - blk * 9);
    if (blk >= nb) return;
    const uint16_t v = *reinterpret_cast<const uint16_t*>(aos + blk * 18 + part * 2);   // 18-byte blocks are 2-aligned
    if (part == 0) *reinterpret_cast<uint16_t*>(sep + blk * 2) = v;
    else *reinterpret_cast<uint16_t*>(sep + data_off + blk * 16 + (part - 1) * 2) = v;
}

__global__ void pack_w4g_meta_kernel(const uint16_t* __restrict__ scales, const uint16_t* __restrict__ zeros,
                                     uint32_t* __restrict__ meta, long long ng) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < ng) meta[i] = (uint32_t)scales[i] | ((uint32_t)zeros[i] << 16);
}

// flat 2-bit codes (element e at bits 2*(e%4) of byte e/4) -> rows padded to whole bytes
__global__ void repack_ternary_rows_kernel(const uint8_t* __restrict__ flat, uint8_t* __restrict__ rows, int M, int K) {
    const int rb = (K + 3) / 4;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)M * rb) return;
    const int m = (int)(i / rb), c = (int)(i - (long long)m * rb);
    uint32_t out = 0;
#pragma unroll
    for (int t = 0; t < 4; ++t) {
        const int k = c * 4 + t;
        if (k < K) {
            const long long e = (long long)m * K + k;
            out |= ((flat[e >> 2] >> (2 * (int)(e & 3))) & 3u) << (2 * t);
        } else {
            out |= 1u << (2 * t);      // padding decodes to 0
        }
    }
    rows[i] = (uint8_t)out;
}

// ---------------------------------------------------------------- quantizers
// Q4_0 and Q8_0: eight lanes per 32-value block, four consecutive values each.
template <int BITS>
__global__ void quantize_block32_kernel(const float* __restrict__ src, uint8_t* __restrict__ out, long long nb,
                                        long long data_off) {
    const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long blk = t >> 3;
    const int l = (int)(t & 7);
    const bool live = blk < nb;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (live) v = *reinterpret_cast<const float4*>(src + blk * 32 + l * 4);
    float am = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
    const float qmax = BITS == 4 ? 7.0f : 127.0f;
    float scale = 0.f, inv = 0.f;
    if (am > 0.f) { scale = __fdiv_rn(am, qmax); }
    if (scale > 0.f) inv = __fdiv_rn(1.0f, scale);
    const int lo = BITS == 4 ? -8 : -128, hi = BITS == 4 ? 7 : 127;
    const int q0 = clampi((int)roundf(__fmul_rn(v.x, inv)), lo, hi);
    const int q1 = clampi((int)roundf(__fmul_rn(v.y, inv)), lo, hi);
    const int q2 = clampi((int)roundf(__fmul_rn(v.z, inv)), lo, hi);
    const int q3 = clampi((int)roundf(__fmul_rn(v.w, inv)), lo, hi);
    if (BITS == 8) {
        if (!live) return;
        uint8_t* b = out + blk * 36;
        if (l == 0) *reinterpret_cast<float*>(b) = scale;
        *reinterpret_cast<uint32_t*>(b + 4 + l * 4) =
            (uint32_t)(uint8_t)q0 | ((uint32_t)(uint8_t)q1 << 8) | ((uint32_t)(uint8_t)q2 << 16) | ((uint32_t)(uint8_t)q3 << 24);
    } else {
        // element j pairs with element j+16: lanes 0-3 take their high nibbles from lanes 4-7
        const uint32_t mine = (uint32_t)(q0 + 8) | ((uint32_t)(q1 + 8) << 8) | ((uint32_t)(q2 + 8) << 16) | ((uint32_t)(q3 + 8) << 24);
        const uint32_t other = __shfl_down_sync(0xffffffffu, mine, 4);
        if (!live) return;
        if (l == 0) *reinterpret_cast<__half*>(out + blk * 2) = __float2half_rn(scale);
        if (l < 4) *reinterpret_cast<uint32_t*>(out + data_off + blk * 16 + l * 4) = mine | (other << 4);
    }
}

// GPTQ-4 / AWQ: one warp per group of 128 consecutive values (group == 128),
// or one thread per group for other group sizes (generic, slower).
__device__ __forceinline__ int w4g_code(float v, float inv, float zf, int awq) {
    const float t = __fadd_rn(__fmul_rn(v, inv), zf);
    const int q = awq ? (int)__fadd_rn(t, 0.5f) : (int)roundf(t);
    return clampi(q, 0, 15);
}

__global__ void quantize_w4g128_kernel(const float* __restrict__ src, uint8_t* __restrict__ qdata,
                                       uint32_t* __restrict__ meta, long long ng, int awq) {
    const long long g = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (g >= ng) return;                                 // whole warps leave together
    const float4 v = *reinterpret_cast<const float4*>(src + g * 128 + lane * 4);
    float mn = fminf(fminf(v.x, v.y), fminf(v.z, v.w));
    float mx = fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    }
    float scale = 0.f, zero = 0.f;
    const float range = __fsub_rn(mx, mn);
    if (range > 0.f) scale = __fdiv_rn(range, 15.0f);
    if (scale > 0.f) zero = __fdiv_rn(-mn, scale);
    const __half s16 = __float2half_rn(scale), z16 = __float2half_rn(zero);
    const float sf = __half2float(s16), zf = __half2float(z16);
    float inv = 0.f;
    if (sf > 0.f) inv = __fdiv_rn(1.0f, sf);
    const int q0 = w4g_code(v.x, inv, zf, awq), q1 = w4g_code(v.y, inv, zf, awq);
    const int q2 = w4g_code(v.z, inv, zf, awq), q3 = w4g_code(v.w, inv, zf, awq);
    *reinterpret_cast<uint16_t*>(qdata + g * 64 + lane * 2) = (uint16_t)(q0 | (q1 << 4) | (q2 << 8) | (q3 << 12));
    if (lane == 0) meta[g] = (uint32_t)__half_as_ushort(s16) | ((uint32_t)__half_as_ushort(z16) << 16);
}

__global__ void quantize_w4g_generic_kernel(const float* __restrict__ src, uint8_t* __restrict__ qdata,
                                            uint32_t* __restrict__ meta, long long ng, int group, int awq) {
    const long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (g >= ng) return;
    const float* s = src + g * group;
    float mn = s[0], mx = s[0];
    for (int j = 1; j < group; ++j) { mn = fminf(mn, s[j]); mx = fmaxf(mx, s[j]); }
    float scale = 0.f, zero = 0.f;
    const float range = __fsub_rn(mx, mn);
    if (range > 0.f) scale = __fdiv_rn(range, 15.0f);
    if (scale > 0.f) zero = __fdiv_rn(-mn, scale);
    const __half s16 = __float2half_rn(scale), z16 = __float2half_rn(zero);
    const float sf = __half2float(s16), zf = __half2float(z16);
    float inv = 0.f;
    if (sf > 0.f) inv = __fdiv_rn(1.0f, sf);
    uint8_t* d = qdata + g * (group / 2);
    for (int j = 0; j < group; j += 2)
        d[j >> 1] = (uint8_t)(w4g_code(s[j], inv, zf, awq) | (w4g_code(s[j + 1], inv, zf, awq) << 4));
    meta[g] = (uint32_t)__half_as_ushort(s16) | ((uint32_t)__half_as_ushort(z16) << 16);
}

// ---------------------------------------------------------------- dequantize
// One thread per element; same expression as the storages' Dequantize().
__global__ void dequantize_kernel(int fmt, const uint8_t* __restrict__ w, const uint8_t* __restrict__ meta,
                                  float* __restrict__ dst, long long n, int aux) {
    const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= n) return;
    float out;
    if (fmt == F_Q4_0) {
        const long long blk = e >> 5;
        const int j = (int)(e & 31);
        const uint8_t byte = w[blk * 16 + (j & 15)];
        const int q = (j < 16 ? (byte & 0xf) : (byte >> 4)) - 8;
        out = __fmul_rn((float)q, h2f(reinterpret_cast<const uint16_t*>(meta)[blk]));
    } else if (fmt == F_IQ4NL) {
        const long long blk = e >> 5;
        const int j = (int)(e & 31);
        const uint8_t byte = w[blk * 16 + (j >> 1)];
        const int q = (j & 1) ? (byte >> 4) : (byte & 0xf);
        out = __fmul_rn(h2f(reinterpret_cast<const uint16_t*>(meta)[blk]), c_iq4nl[q]);
    } else if (fmt == F_W4G) {
        const long long g = e / aux;
        const uint8_t byte = w[e >> 1];
        const int q = (e & 1) ? (byte >> 4) : (byte & 0xf);
        const uint32_t m = reinterpret_cast<const uint32_t*>(meta)[g];
        out = __fmul_rn(__fsub_rn((float)q, h2f((uint16_t)(m >> 16))), h2f((uint16_t)(m & 0xffff)));
    } else if (fmt == F_Q8_0) {
        const long long blk = e >> 5;
        const int j = (int)(e & 31);
        const uint8_t* b = w + blk * 36;
        out = __fmul_rn((float)(int8_t)b[4 + j], *reinterpret_cast<const float*>(b));
    } else {  // ternary, row-aligned, aux = K
        const int rb = (aux + 3) / 4;
        const long long m = e / aux;
        const int k = (int)(e - m * aux);
        out = (float)(int)((w[m * rb + (k >> 2)] >> (2 * (k & 3))) & 3u) - 1.0f;
    }
    dst[e] = out;
}

// Q4_K super-blocks of 144 bytes {16 header bytes, 128 nibble bytes} -> all headers, then (16-byte aligned) all
// nibble bytes: the split tensor.Q4Storage.RawBytesGPU makes for Q4_0, so that rows of codes and rows of headers
// are contiguous and every 16-byte load is aligned.  One thread per 16 bytes.
__global__ void repack_blocks144_kernel(const uint8_t* __restrict__ aos, uint8_t* __restrict__ sep, long long nblocks,
                                        long long data_off) {
    const long long total = nblocks * 9;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long b = i / 9;
        const int part = (int)(i - b * 9);
        const uint8_t* src = aos + b * 144 + part * 16;
        uint4 v;
        memcpy(&v, src, 16);                                  // 144-byte blocks are 16-byte aligned when aos is
        uint8_t* dst = part == 0 ? sep + b * 16 : sep + data_off + b * 128 + (part - 1) * 16;
        *reinterpret_cast<uint4*>(dst) = v;
    }
}

// Q5_K super-blocks of 176 bytes {16 header, 128 ql, 32 qh} -> per super-block 48 bytes {header, qh}, then
// (16-byte aligned) the 128 ql bytes of every super-block.  One thread per 16 bytes.
__global__ void repack_blocks176_kernel(const uint8_t* __restrict__ aos, uint8_t* __restrict__ sep, long long nblocks,
                                        long long data_off) {
    const long long total = nblocks * 11;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long b = i / 11;
        const int part = (int)(i - b * 11);                   // 0 header, 1..8 ql, 9..10 qh
        uint4 v;
        memcpy(&v, aos + b * 176 + part * 16, 16);
        uint8_t* dst = part == 0 ? sep + b * 48 : part <= 8 ? sep + data_off + b * 128 + (part - 1) * 16 : sep + b * 48 + 16 + (part - 9) * 16;
        *reinterpret_cast<uint4*>(dst) = v;
    }
}

// Q6_K super-blocks of 210 bytes {128 ql, 64 qh, 16 scales, fp16 d} (not 16-byte aligned) -> per super-block 96
// side bytes {qh, scales, d, 14 zero bytes}, then (16-byte aligned) the 128 ql bytes of every super-block.
// One thread per 16 output bytes, source read byte by byte.
__global__ void repack_blocks210_kernel(const uint8_t* __restrict__ aos, uint8_t* __restrict__ sep, long long nblocks,
                                        long long data_off) {
    const long long total = nblocks * 14;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long b = i / 14;
        const int part = (int)(i - b * 14);                   // 0..7 ql, 8..11 qh, 12 scales, 13 d
        const uint8_t* src = aos + b * 210 + (part < 8 ? part * 16 : part < 12 ? 128 + (part - 8) * 16 : part == 12 ? 192 : 208);
        const int nbytes = part == 13 ? 2 : 16;
        uint8_t v[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = j < nbytes ? src[j] : (uint8_t)0;
        uint8_t* dst = part < 8 ? sep + data_off + b * 128 + part * 16 : sep + b * 96 + (part - 8) * 16;
        uint4 o;
        memcpy(&o, v, 16);
        *reinterpret_cast<uint4*>(dst) = o;
    }
}

// Rows of two matrices of the same shape, interleaved: out row 2i = a row i, out row 2i+1 = b row i
// (row_bytes a multiple of 16).  Used to lay gate and up projections out as (gate_i, up_i) pairs.
__global__ void interleave_rows_kernel(const uint4* __restrict__ a, const uint4* __restrict__ b, uint4* __restrict__ out,
                                       long long rows, int vec_per_row) {
    const long long total = rows * vec_per_row;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / vec_per_row;
        const int c = (int)(i - r * vec_per_row);
        out[(2 * r) * vec_per_row + c] = a[i];
        out[(2 * r + 1) * vec_per_row + c] = b[i];
    }
}

// y[M, N] = x[M, K] * w[K, N], w float32 row-major: the product compute.MatMulW4A16 forms when the 4-bit weights sit
// on the B side (compute/w4a16.go:107-119): the dequantized slice is a literal [K, N] matrix and CPUEngine.MatMul runs
// SgemmSimd over it (internal/xblas/gemm_simd_amd64.go:16-36): c[i, :] += a[i, p] * b[p, :] with p ascending, one
// fused multiply-add per element in the columns the 4-lane groups cover and an unfused multiply then add in the
// last n % 4 columns.  One thread per output keeps exactly that order.  A correctness path (the reference's own
// test of this layout is 2 x 32 x 3), not a tuned one.
__global__ void matmul_wkn_kernel(const void* __restrict__ x, const float* __restrict__ w, float* __restrict__ y, int M, int K, int N,
                                  int x_f32) {
    grid_dep_launch();
    grid_dep_wait();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)M * N) return;
    const int m = (int)(idx / N), n = (int)(idx - (long long)m * N);
    const bool fused = n < (N & ~3);
    float acc = 0.f;
    for (int p = 0; p < K; ++p) {
        const float a = x_f32 ? reinterpret_cast<const float*>(x)[(size_t)m * K + p]
                              : __half2float(reinterpret_cast<const __half*>(x)[(size_t)m * K + p]);
        const float b = w[(size_t)p * N + n];
        acc = fused ? __fmaf_rn(a, b, acc) : __fadd_rn(acc, __fmul_rn(a, b));
    }
    y[idx] = acc;
}

}  // namespace ztq
