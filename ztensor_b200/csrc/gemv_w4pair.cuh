// gemv_w4pair.cuh -- batch-1 GEMV for the 4-bit formats with a linear code
// (Q4_0 and GPTQ/AWQ group-128), 64 weights per lane per row.
//
// Same pipeline as gemv_stream.cuh (producer thread + 1-D bulk copies into a
// ring of stages, teams of warps spanning K, fixed-order reductions), with the
// per-row overhead of a lane (scale decode, integer-to-float, address math,
// reduction) amortised over two 16-byte chunks instead of one:
//   - lane `m` of a team owns the chunk pair (2m, 2m+1) of every row; the two
//     128-bit shared loads are issued so that each one is bank-conflict free
//     (lanes 0-3 of every octet read their even chunk first, lanes 4-7 their
//     odd chunk), and the lane's activation planes are stored in that same
//     order, so nothing is swapped at run time;
//   - the activation vector is converted to integer planes once per CTA, in
//     shared memory, by all consumer threads together;
//   - the 64 activations of a lane share one block exponent (|X| < 2^21, so
//     that sum(code * X) over 64 codes fits an int32): the integer dot product
//     of the pair is exact, converted to float once, and scaled once (W4G: one
//     {scale, zero} pair covers both chunks; Q4_0: one scale per chunk).
#pragma once

#include "gemv_stream.cuh"

namespace ztq {

template <int FMT> struct PairX {
    uint32_t w[3][16];   // plane, then 8 words of the first-loaded chunk and 8 of the second
    float inv;           // 2^-s of the shared block exponent
    float c0, c1;        // Q4_0: -8 * sum(x) of the first / second chunk; W4G: c0 = sum(x) of both
};

// Eight consecutive elements of a [K] vector of fp16 or fp32.
__device__ __forceinline__ void load8(const void* base, bool f32, long long stride, int u, float (&v)[8]) {
    if (stride == 1 && (reinterpret_cast<uintptr_t>(base) & 15) == 0) {
        if (f32) {
            const float4 a = reinterpret_cast<const float4*>(base)[2 * u], b = reinterpret_cast<const float4*>(base)[2 * u + 1];
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
        } else {
            const uint4 q = reinterpret_cast<const uint4*>(base)[u];
            const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const __half2 h = *reinterpret_cast<const __half2*>(&w[j]);
                v[2 * j] = __low2float(h);
                v[2 * j + 1] = __high2float(h);
            }
        }
        return;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const long long idx = (long long)(u * 8 + i) * stride;
        v[i] = f32 ? reinterpret_cast<const float*>(base)[idx] : __half2float(reinterpret_cast<const __half*>(base)[idx]);
    }
}

// Where word `wi` (0..7) of 32-activation chunk `chunk` of a plane lives in shared memory.  A lane of the row loop
// owns the chunk pair (2m, 2m+1) and reads its 64 bytes per plane as four 16-byte pieces, in the order
// {first-loaded chunk: words 0-3, words 4-7; second-loaded chunk: words 0-3, words 4-7} (lanes 4-7 of every
// octet load their odd chunk first).  A plane is therefore stored piece-major: piece j of lane-slot m at
// j * slots * 16 + m * 16 bytes, so that each of the four loads of a warp reads 32 consecutive 16-byte units --
// no bank conflicts.  (Chunk-major storage put the lanes of a load 64 bytes apart: a four-way conflict on every
// one of the twelve loads, about a microsecond per launch.)
__device__ __forceinline__ uint32_t* xs_word(uint8_t* plane, int slots, int chunk, int wi) {
    const int m = chunk >> 1, e = chunk & 1, first = (m >> 2) & 1;
    const int piece = (e == first ? 0 : 2) + (wi >> 2);
    return reinterpret_cast<uint32_t*>(plane) + ((size_t)piece * slots + m) * 4 + (wi & 3);
}

// One unit (eight consecutive activations v, largest magnitude am) -> fixed point -> planes in shared memory.
// All 32 lanes of a warp call this together (shuffles).
template <int FMT>
__device__ __forceinline__ void convert_unit(const GemvParams& p, uint8_t* xs, float* xmeta, int u, const float (&v)[8], float am) {
    float sm = ((v[0] + v[1]) + (v[2] + v[3])) + ((v[4] + v[5]) + (v[6] + v[7]));
    am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 1));
    am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 2));
    am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 4));
    sm += __shfl_xor_sync(0xffffffffu, sm, 1);
    sm += __shfl_xor_sync(0xffffffffu, sm, 2);            // sum of this thread's 32-chunk
    const float other = __shfl_xor_sync(0xffffffffu, sm, 4);
    const uint32_t e = __float_as_uint(am) >> 23;
    const uint32_t eb = am > 0.f ? e : 127u;
    constexpr int top = 20;                               // |X| <= 2^21
    const float scale = __uint_as_float((uint32_t)(127 + top + 127 - (int)eb) << 23);
    uint32_t X[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) X[i] = __float_as_uint(fmaf(v[i], scale, 12582912.0f));
    const int chunk = u >> 2, j = u & 3;
    // Q4_0 consumes the activations in natural order (words 2j, 2j+1 of the chunk); the sequential
    // formats consume even elements (words 0..3) and odd elements (words 4..7) separately.
    uint32_t wa[3], wb[3];
    if (FMT == F_Q4_0 || FMT == F_Q4K || FMT == F_Q5K || FMT == F_Q6K) { transpose3(X[0], X[1], X[2], X[3], wa); transpose3(X[4], X[5], X[6], X[7], wb); }
    else { transpose3(X[0], X[2], X[4], X[6], wa); transpose3(X[1], X[3], X[5], X[7], wb); }
    wa[2] = fix_top_plane(wa[2]);
    wb[2] = fix_top_plane(wb[2]);
    const int slots = p.K >> 6;
#pragma unroll
    for (int pl = 0; pl < 3; ++pl) {
        uint8_t* plane = xs + (size_t)pl * p.K;
        if (FMT == F_Q6K) {
            // Q6_K: per half of 128 weights, bytes ql[l] (l < 32) carry elements l (low nibble) and 64 + l (high),
            // bytes ql[32 + l] elements 32 + l and 96 + l.  A lane's pair of chunks is 32 consecutive ql bytes:
            // pair pi of the super-block = half 2 (pi / 2), second 32 bytes if pi odd.
            const int eb = (u * 8) & 255, r = eb & 127, stream = r >> 5, l = r & 31;
            const int pair = (u >> 5) * 4 + (eb >> 7) * 2 + (stream & 1);
            *reinterpret_cast<uint2*>(xs_word(plane, slots, pair * 2 + (l >> 4), (stream >> 1) * 4 + ((l & 15) >> 2))) = make_uint2(wa[pl], wb[pl]);
        } else if (FMT == F_Q4K || FMT == F_Q5K) {
            // Q4_K / Q5_K: the 32 bytes of a 64-weight group carry elements 0-31 in their low nibbles and 32-63 in their
            // high nibbles; data chunk h (16 bytes) therefore meets elements 16h .. 16h+15 (words 0-3) and
            // 32 + 16h .. (words 4-7).  e = first element of this unit inside its group of 64.
            const int e = (u & 7) * 8;
            *reinterpret_cast<uint2*>(xs_word(plane, slots, (u >> 3) * 2 + ((e >> 4) & 1), (e >> 5) * 4 + ((e & 15) >> 2))) = make_uint2(wa[pl], wb[pl]);
        } else if (FMT == F_Q4_0) {
            *reinterpret_cast<uint2*>(xs_word(plane, slots, chunk, 2 * j)) = make_uint2(wa[pl], wb[pl]);
        } else {
            *xs_word(plane, slots, chunk, j) = wa[pl];
            *xs_word(plane, slots, chunk, 4 + j) = wb[pl];
        }
    }
    if ((u & 7) == 0) {               // first thread of the slot: its chunk is the even one
        float4 m;
        m.x = __uint_as_float((uint32_t)((int)eb - top) << 23);
        if (FMT == F_Q4_0) { m.y = -8.0f * sm; m.z = -8.0f * other; }
        else if (FMT == F_Q4K || FMT == F_Q5K) { m.y = sm; m.z = other; }     // sums of the two sub-blocks of 32
        else { m.y = sm + other; m.z = 0.f; }
        m.w = 0.f;
        reinterpret_cast<float4*>(xmeta)[u >> 3] = m;
    }
}

// Cooperative conversion of the activation vector into shared memory, once per
// CTA: each consumer thread converts units of 8 consecutive activations; the 8
// threads of a 64-activation slot agree on the block exponent with shuffles.
//   xs    [3][K] bytes, per 32-chunk eight words in the order chunk_dot consumes them
//   xmeta [K/64][4] floats: {2^-s, c0, c1, unused}
template <int FMT>
__device__ __forceinline__ void convert_x_cta(const GemvParams& p, uint8_t* xs, float* xmeta, int ctid, int CT) {
    const int units = p.K >> 3;                               // a multiple of 32: whole warps loop together
    const bool fast = !p.x_f32 && p.xs_k == 1 && ((reinterpret_cast<uintptr_t>(p.x) & 15) == 0);
    for (int u = ctid; u < units; u += CT) {
        float v[8];
        float am = 0.f;
        if (fast) {
            const uint4 q = reinterpret_cast<const uint4*>(p.x)[u];
            const uint32_t w[4] = {q.x, q.y, q.z, q.w};
            __half2 hm = __habs2(*reinterpret_cast<const __half2*>(&w[0]));
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const __half2 h = *reinterpret_cast<const __half2*>(&w[j]);
                if (j) hm = __hmax2(hm, __habs2(h));           // largest magnitude on the packed halves
                v[2 * j] = __low2float(h);
                v[2 * j + 1] = __high2float(h);
            }
            am = fmaxf(__low2float(hm), __high2float(hm));
        } else {
            load8(p.x, p.x_f32 != 0, p.xs_k, u, v);
#pragma unroll
            for (int i = 0; i < 8; ++i) am = fmaxf(am, fabsf(v[i]));
        }
        convert_unit<FMT>(p, xs, xmeta, u, v, am);
    }
}

// The same with RMSNorm folded in (fused_add_rmsnorm.cu:13-50 of the reference):
//   v = x + residual;  scale = rsqrt(mean(v^2) + eps);  activation = (v * scale) * weight.
// Every CTA needs the whole vector anyway, so every CTA computes the mean itself (K <= 32768 values): 512
// threads, lane tree, then warps in order (fixed).  The first CTA also writes v (the updated residual stream)
// when asked.  Up to 16 values and gains per thread stay in registers between the two phases (K <= 8192);
// longer vectors are read a second time (from L1 / L2).  `red`: 32 floats of shared memory, free at this point.
template <int FMT>
__device__ __forceinline__ void convert_x_cta_rmsnorm(const GemvParams& p, uint8_t* xs, float* xmeta, float* red, int ctid, int CT) {
    constexpr int UMAX = 2;
    const int units = p.K >> 3;
    const bool f32 = p.x_f32 != 0;
    const bool inreg = units <= UMAX * CT;
    float v[UMAX][8], g[UMAX][8];
    auto load_v = [&](int u, float (&dst)[8]) {
        load8(p.x, f32, p.xs_k, u, dst);
        if (p.fz.residual) {
            float r[8];
            load8(p.fz.residual, f32, 1, u, r);
#pragma unroll
            for (int i = 0; i < 8; ++i) dst[i] += r[i];
        }
    };
    auto load_g = [&](int u, float (&dst)[8]) {
        const float4 g0 = reinterpret_cast<const float4*>(p.fz.norm_weight)[2 * u];
        const float4 g1 = reinterpret_cast<const float4*>(p.fz.norm_weight)[2 * u + 1];
        dst[0] = g0.x; dst[1] = g0.y; dst[2] = g0.z; dst[3] = g0.w; dst[4] = g1.x; dst[5] = g1.y; dst[6] = g1.z; dst[7] = g1.w;
    };
    auto store_sum = [&](int u, const float (&src)[8]) {
        if (!p.fz.sum_out || blockIdx.x != 0) return;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if (f32) reinterpret_cast<float*>(p.fz.sum_out)[u * 8 + i] = src[i];
            else reinterpret_cast<__half*>(p.fz.sum_out)[u * 8 + i] = __float2half_rn(src[i]);
        }
    };
    float sq = 0.f;
    if (inreg) {
#pragma unroll
        for (int j = 0; j < UMAX; ++j) {
            const int u = ctid + j * CT;
            if (u < units) {
                load_v(u, v[j]);
                load_g(u, g[j]);
            }
        }
#pragma unroll
        for (int j = 0; j < UMAX; ++j) {
            const int u = ctid + j * CT;
            if (u < units) {
                store_sum(u, v[j]);
#pragma unroll
                for (int i = 0; i < 8; ++i) sq = fmaf(v[j][i], v[j][i], sq);
            }
        }
    } else {
        for (int u = ctid; u < units; u += CT) {
            load_v(u, v[0]);
            store_sum(u, v[0]);
#pragma unroll
            for (int i = 0; i < 8; ++i) sq = fmaf(v[0][i], v[0][i], sq);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
    if ((ctid & 31) == 0) red[ctid >> 5] = sq;
    bar_sync(1, CT);
    float tot = 0.f;
    for (int w = 0; w < CT / 32; ++w) tot += red[w];
    const float nscale = rsqrtf(tot / (float)p.K + p.fz.eps);
    auto finish = [&](int u, float (&vv)[8], const float (&gg)[8]) {
        float am = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            vv[i] = (vv[i] * nscale) * gg[i];                 // the reference's order of products
            am = fmaxf(am, fabsf(vv[i]));
        }
        convert_unit<FMT>(p, xs, xmeta, u, vv, am);
    };
    if (inreg) {
#pragma unroll
        for (int j = 0; j < UMAX; ++j) {
            const int u = ctid + j * CT;
            if (u < units) finish(u, v[j], g[j]);
        }
    } else {
        for (int u = ctid; u < units; u += CT) {
            load_v(u, v[0]);
            load_g(u, g[0]);
            finish(u, v[0], g[0]);
        }
    }
    // `red` (the partial-sum scratch) is written again only after the barrier that follows the conversion
}

// Registers of one lane: the planes of its two chunks in load order.
template <int FMT>
__device__ __forceinline__ void load_pair_x(const uint8_t* xs, const float* xmeta, int K, int m, int first, bool live,
                                            PairX<FMT>& px) {
    if (!live) {
#pragma unroll
        for (int pl = 0; pl < 3; ++pl)
#pragma unroll
            for (int i = 0; i < 16; ++i) px.w[pl][i] = 0;
        px.inv = px.c0 = px.c1 = 0.f;
        return;
    }
    (void)first;                                          // the piece-major layout already stores the pieces in load order
    const int slots = K >> 6;
#pragma unroll
    for (int pl = 0; pl < 3; ++pl) {
        const uint4* src = reinterpret_cast<const uint4*>(xs + (size_t)pl * K) + m;
        const uint4 a0 = src[0], a1 = src[slots], b0 = src[2 * slots], b1 = src[3 * slots];
        px.w[pl][0] = a0.x; px.w[pl][1] = a0.y; px.w[pl][2] = a0.z; px.w[pl][3] = a0.w;
        px.w[pl][4] = a1.x; px.w[pl][5] = a1.y; px.w[pl][6] = a1.z; px.w[pl][7] = a1.w;
        px.w[pl][8] = b0.x; px.w[pl][9] = b0.y; px.w[pl][10] = b0.z; px.w[pl][11] = b0.w;
        px.w[pl][12] = b1.x; px.w[pl][13] = b1.y; px.w[pl][14] = b1.z; px.w[pl][15] = b1.w;
    }
    if (FMT == F_Q6K) {
        // low-nibble codes meet activations of the 64-block 2 (pair / 2) of the super-block, high-nibble codes the
        // next one: two block exponents, no sums needed (the codes are made signed)
        const int blk = (m >> 2) * 4 + ((m & 3) >> 1) * 2;
        px.inv = reinterpret_cast<const float4*>(xmeta)[blk].x;
        px.c0 = reinterpret_cast<const float4*>(xmeta)[blk + 1].x;
        px.c1 = 0.f;
        return;
    }
    const float4 mt = reinterpret_cast<const float4*>(xmeta)[m];
    px.inv = mt.x;
    if (FMT == F_Q4_0) { px.c0 = first ? mt.z : mt.y; px.c1 = first ? mt.y : mt.z; }
    else if (FMT == F_Q4K || FMT == F_Q5K) { px.c0 = mt.y; px.c1 = mt.z; }    // by sub-block, whichever chunk is loaded first
    else { px.c0 = mt.y; px.c1 = 0.f; }
}

// Exact integer dot of one 16-byte chunk (32 codes) with eight activation words per plane.
__device__ __forceinline__ void chunk_dot(const uint4 q, const uint32_t (&xw)[3][16], int h, int& s0, int& s1, int& s2) {
    const uint32_t qw[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int m = 0; m < 4; ++m) {
        const uint32_t lo = qw[m] & 0x0f0f0f0fu;
        const uint32_t hi = (qw[m] >> 4) & 0x0f0f0f0fu;
        s0 = dp4a_uu(lo, xw[0][h * 8 + m], s0);
        s1 = dp4a_uu(lo, xw[1][h * 8 + m], s1);
        s2 = dp4a_us(lo, xw[2][h * 8 + m], s2);
        s0 = dp4a_uu(hi, xw[0][h * 8 + 4 + m], s0);
        s1 = dp4a_uu(hi, xw[1][h * 8 + 4 + m], s1);
        s2 = dp4a_us(hi, xw[2][h * 8 + 4 + m], s2);
    }
}

// The same with the low-nibble and high-nibble sums kept apart (Q4_K: they belong to different sub-blocks).
__device__ __forceinline__ void chunk_dot2(const uint4 q, const uint32_t (&xw)[3][16], int h, int (&lo3)[3], int (&hi3)[3]) {
    const uint32_t qw[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int m = 0; m < 4; ++m) {
        const uint32_t lo = qw[m] & 0x0f0f0f0fu;
        const uint32_t hi = (qw[m] >> 4) & 0x0f0f0f0fu;
        lo3[0] = dp4a_uu(lo, xw[0][h * 8 + m], lo3[0]);
        lo3[1] = dp4a_uu(lo, xw[1][h * 8 + m], lo3[1]);
        lo3[2] = dp4a_us(lo, xw[2][h * 8 + m], lo3[2]);
        hi3[0] = dp4a_uu(hi, xw[0][h * 8 + 4 + m], hi3[0]);
        hi3[1] = dp4a_uu(hi, xw[1][h * 8 + 4 + m], hi3[1]);
        hi3[2] = dp4a_us(hi, xw[2][h * 8 + 4 + m], hi3[2]);
    }
}

// Q5_K: the fifth bit of the sixteen low-nibble codes of a chunk is bit `bit` of the matching sixteen qh bytes, of
// the high-nibble codes bit `bit + 1`.
__device__ __forceinline__ void chunk_dot2_q5(const uint4 q, const uint4 qh, uint32_t bit, const uint32_t (&xw)[3][16], int h,
                                              int (&lo3)[3], int (&hi3)[3]) {
    const uint32_t qw[4] = {q.x, q.y, q.z, q.w};
    const uint32_t hw[4] = {qh.x, qh.y, qh.z, qh.w};
#pragma unroll
    for (int m = 0; m < 4; ++m) {
        const uint32_t hb = hw[m] >> bit;
        const uint32_t lo = (qw[m] & 0x0f0f0f0fu) | ((hb & 0x01010101u) << 4);
        const uint32_t hi = ((qw[m] >> 4) & 0x0f0f0f0fu) | ((hb & 0x02020202u) << 3);
        lo3[0] = dp4a_uu(lo, xw[0][h * 8 + m], lo3[0]);
        lo3[1] = dp4a_uu(lo, xw[1][h * 8 + m], lo3[1]);
        lo3[2] = dp4a_us(lo, xw[2][h * 8 + m], lo3[2]);
        hi3[0] = dp4a_uu(hi, xw[0][h * 8 + 4 + m], hi3[0]);
        hi3[1] = dp4a_uu(hi, xw[1][h * 8 + 4 + m], hi3[1]);
        hi3[2] = dp4a_us(hi, xw[2][h * 8 + 4 + m], hi3[2]);
    }
}

// Q6_K: 6-bit codes = nibble | two bits of the matching qh byte (bit position `slo` for the low nibbles, `shi` for the
// high ones), made signed (code - 32) with three word-wide operations; the low-nibble sixteen and the high-nibble
// sixteen are sub-blocks of their own.
__device__ __forceinline__ void chunk_dot2_q6(const uint4 q, const uint4 qh, uint32_t slo, uint32_t shi,
                                              const uint32_t (&xw)[3][16], int h, int (&lo3)[3], int (&hi3)[3]) {
    const uint32_t qw[4] = {q.x, q.y, q.z, q.w};
    const uint32_t hw[4] = {qh.x, qh.y, qh.z, qh.w};
#pragma unroll
    for (int m = 0; m < 4; ++m) {
        uint32_t lo = (qw[m] & 0x0f0f0f0fu) | (((hw[m] >> slo) & 0x03030303u) << 4);
        uint32_t hi = ((qw[m] >> 4) & 0x0f0f0f0fu) | (((hw[m] >> shi) & 0x03030303u) << 4);
        lo = ((lo | 0x80808080u) - 0x20202020u) ^ 0x80808080u;        // bytes 0..63 -> signed bytes -32..31
        hi = ((hi | 0x80808080u) - 0x20202020u) ^ 0x80808080u;
        lo3[0] = dp4a_su(lo, xw[0][h * 8 + m], lo3[0]);
        lo3[1] = dp4a_su(lo, xw[1][h * 8 + m], lo3[1]);
        lo3[2] = dp4a_ss(lo, xw[2][h * 8 + m], lo3[2]);
        hi3[0] = dp4a_su(hi, xw[0][h * 8 + 4 + m], hi3[0]);
        hi3[1] = dp4a_su(hi, xw[1][h * 8 + 4 + m], hi3[1]);
        hi3[2] = dp4a_ss(hi, xw[2][h * 8 + 4 + m], hi3[2]);
    }
}

template <int FMT>
__device__ __forceinline__ float pair_row(const uint8_t* srow, const uint8_t* smeta_row, uint32_t off_first,
                                          uint32_t off_second, uint32_t meta_first, uint32_t meta_second,
                                          const PairX<FMT>& px) {
    const uint4 qa = *reinterpret_cast<const uint4*>(srow + off_first);
    const uint4 qb = *reinterpret_cast<const uint4*>(srow + off_second);
    if (FMT == F_Q6K) {
        // side bytes of the super-block (meta_first): 64 bytes qh, 16 int8 scales, fp16 d.  meta_second = pair of the
        // super-block (0..3): half = pair / 2, second 32 ql bytes if odd; chunk c = 16-byte chunk inside the pair.
        const uint8_t* side = smeta_row + meta_first;
        const uint32_t half = meta_second >> 1, odd = meta_second & 1u;
        const uint32_t ca = (off_first >> 4) & 1u, cb = (off_second >> 4) & 1u;
        const uint4 ha = *reinterpret_cast<const uint4*>(side + half * 32u + ca * 16u);
        const uint4 hb = *reinterpret_cast<const uint4*>(side + half * 32u + cb * 16u);
        int la[3] = {0, 0, 0}, ua[3] = {0, 0, 0}, lb[3] = {0, 0, 0}, ub[3] = {0, 0, 0};
        chunk_dot2_q6(qa, ha, 2u * odd, 4u + 2u * odd, px.w, 0, la, ua);
        chunk_dot2_q6(qb, hb, 2u * odd, 4u + 2u * odd, px.w, 1, lb, ub);
        const int8_t* sc = reinterpret_cast<const int8_t*>(side + 64) + half * 8u + odd * 2u;   // + c: low; + 4 + c: high
        const float d = h2f(*reinterpret_cast<const uint16_t*>(side + 80));
        const float fla = (float)((la[2] * 256 + la[1]) * 256 + la[0]), fua = (float)((ua[2] * 256 + ua[1]) * 256 + ua[0]);
        const float flb = (float)((lb[2] * 256 + lb[1]) * 256 + lb[0]), fub = (float)((ub[2] * 256 + ub[1]) * 256 + ub[0]);
        const float lo = fmaf((float)sc[ca], fla, (float)sc[cb] * flb);
        const float hi = fmaf((float)sc[4 + ca], fua, (float)sc[4 + cb] * fub);
        return d * fmaf(lo, px.inv, hi * px.c0);
    }
    if (FMT == F_Q4K || FMT == F_Q5K) {
        // header of the super-block (meta_first = its offset): fp16 d, fp16 dmin, 12 bytes of 6-bit scales / mins
        // (decodeQ4KScalesMins, tensor/quantized_kquant.go:34-49); meta_second = group of 64 inside it (0..3),
        // whose sub-blocks are 2g (low nibbles) and 2g+1 (high nibbles)
        const uint4 hd = *reinterpret_cast<const uint4*>(smeta_row + meta_first);
        int lo3[3] = {0, 0, 0}, hi3[3] = {0, 0, 0};
        if (FMT == F_Q5K) {
            // side data of a super-block: 16 header bytes, then the 32 qh bytes; the data chunk at row offset o
            // (o / 16 odd or even) goes with qh bytes 16 (o / 16 & 1) .. +15
            const uint4 ha = *reinterpret_cast<const uint4*>(smeta_row + meta_first + 16 + (off_first & 16u));
            const uint4 hb = *reinterpret_cast<const uint4*>(smeta_row + meta_first + 16 + (off_second & 16u));
            chunk_dot2_q5(qa, ha, 2u * meta_second, px.w, 0, lo3, hi3);
            chunk_dot2_q5(qb, hb, 2u * meta_second, px.w, 1, lo3, hi3);
        } else {
            chunk_dot2(qa, px.w, 0, lo3, hi3);
            chunk_dot2(qb, px.w, 1, lo3, hi3);
        }
        const float dl = (float)((lo3[2] * 256 + lo3[1]) * 256 + lo3[0]);
        const float dh = (float)((hi3[2] * 256 + hi3[1]) * 256 + hi3[0]);
        const float d = h2f((uint16_t)(hd.x & 0xffff)), dmin = h2f((uint16_t)(hd.x >> 16));
        // Sub-blocks 0..3: six low bits of bytes 0-3 (scales) / 4-7 (mins); sub-blocks 4..7: a nibble of bytes
        // 8-11 plus the two high bits of bytes 0-3 / 4-7.  Which case applies depends on the lane only
        // (g = its group of 64), so the selectors below are loop-invariant and nothing diverges.
        const uint32_t g = meta_second;
        const bool upper = g >= 2;
        const uint32_t sh = 16u * (g & 1u);                // the group's two sub-blocks sit in adjacent bytes
        const uint32_t low_mask = upper ? 0x0F0Fu : 0x3F3Fu;
        const uint32_t s2 = ((upper ? hd.w : hd.y) >> sh) & low_mask;                  // two scales' low bits
        const uint32_t m2 = ((upper ? (hd.w >> 4) : hd.z) >> sh) & low_mask;           // two mins' low bits
        const uint32_t hs = upper ? ((hd.y >> (sh + 6)) & 0x0303u) << 4 : 0u;          // their high bits (upper half)
        const uint32_t hm = upper ? ((hd.z >> (sh + 6)) & 0x0303u) << 4 : 0u;
        const uint32_t sc = s2 | hs, mn = m2 | hm;
        const uint32_t sc0 = sc & 0xffu, sc1 = sc >> 8, mn0 = mn & 0xffu, mn1 = mn >> 8;
        // sum_k (d sc q - dmin mn) x = d sc (sum q x) - dmin mn (sum x); d * sc is exact in fp32
        const float a0 = (d * (float)sc0) * (dl * px.inv) - (dmin * (float)mn0) * px.c0;
        const float a1 = (d * (float)sc1) * (dh * px.inv) - (dmin * (float)mn1) * px.c1;
        return a0 + a1;
    }
    if (FMT == F_W4G) {
        const __half2 sz = *reinterpret_cast<const __half2*>(smeta_row + meta_first);
        int s0 = 0, s1 = 0, s2 = 0;
        chunk_dot(qa, px.w, 0, s0, s1, s2);
        chunk_dot(qb, px.w, 1, s0, s1, s2);
        const float d = (float)((s2 * 256 + s1) * 256 + s0);
        const float s = __low2float(sz), z = __high2float(sz);
        return s * fmaf(d, px.inv, -z * px.c0);
    } else {
        const float sa = h2f(*reinterpret_cast<const uint16_t*>(smeta_row + meta_first));
        const float sb = h2f(*reinterpret_cast<const uint16_t*>(smeta_row + meta_second));
        int a0 = 0, a1 = 0, a2 = 0, b0 = 0, b1 = 0, b2 = 0;
        chunk_dot(qa, px.w, 0, a0, a1, a2);
        chunk_dot(qb, px.w, 1, b0, b1, b2);
        const float da = (float)((a2 * 256 + a1) * 256 + a0);
        const float db = (float)((b2 * 256 + b1) * 256 + b0);
        return fmaf(sa, fmaf(da, px.inv, px.c0), sb * fmaf(db, px.inv, px.c1));
    }
}

// FUSED: the RMSNorm / SwiGLU hooks of FuseParams are compiled in (a separate instantiation, so that the plain
// kernel pays nothing for them: a few hundred cycles per launch matter on matrices of a few MB).
template <int FMT, int RT, bool FUSED = false, bool AR = false>
__global__ void __launch_bounds__(544, 1) gemv_w4pair_kernel(const GemvParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    const int CW = p.T * p.WPT;
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + p.bar_off);
    const int S_all = p.S + p.Sx;                                // the last Sx stages overlay xs / xmeta (free after the prologue)
    uint64_t* empty = full + S_all;
    uint64_t* xdone = empty + S_all;                             // every consumer warp has its activations in registers
    unsigned* ar_word = reinterpret_cast<unsigned*>(xdone + 1);  // all-reduce sequence number of this launch
    volatile unsigned* abort_word = ar_word + 1;                 // raised by a warp that gave up on a wait
    float* part = reinterpret_cast<float*>(smem + p.part_off);   // [P rows][WPT]
    uint8_t* xs = smem + p.x_off;                                // [3][K] activation planes
    float* xmeta = reinterpret_cast<float*>(xs + 3 * (size_t)p.K);   // [K/64][4]

    if (tid == 0) {
        for (int s = 0; s < S_all; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], CW); }
        mbar_init(xdone, CW);
        *abort_word = 0;
        mbar_fence_init();
    }
    __syncthreads();
    grid_dep_launch();

    // contiguous rows per CTA; with the SwiGLU epilogue whole (gate, up) pairs
    const int unit = (FUSED && p.fz.swiglu) ? 2 : 1;
    const int r_begin = unit * (int)(((long long)(p.N / unit) * blockIdx.x) / gridDim.x);
    const int r_end = unit * (int)(((long long)(p.N / unit) * (blockIdx.x + 1)) / gridDim.x);
    const int n_tiles = (r_end - r_begin + p.R - 1) / p.R;

    if (warp == CW) {
        if (lane == 0) {
            const uint64_t pol = l2_evict_first_policy();
            for (int it = 0; it < n_tiles; ++it) {
                const int s = it % S_all;
                if (it >= S_all && !mbar_wait(&empty[s], ((it / S_all) - 1) & 1)) { report_error(ZTQ_ERR_EMPTY_WAIT); break; }
                if (it == p.S && !mbar_wait(xdone, 0)) { report_error(ZTQ_ERR_EMPTY_WAIT); break; }   // first overlay stage
                const int row0 = r_begin + it * p.R;
                const int rows = min(p.R, r_end - row0);
                uint8_t* dst = smem + (size_t)s * p.stage_stride;
                const uint32_t bd = (uint32_t)rows * p.row_bytes;
                const uint32_t bm = (uint32_t)rows * p.meta_row_bytes;
                mbar_expect_tx(&full[s], bd + bm);
                bulk_g2s_hint(dst, p.w + (size_t)row0 * p.row_bytes, bd, &full[s], pol);
                bulk_g2s_hint(dst + (size_t)p.R * p.row_bytes, p.meta + (size_t)row0 * p.meta_row_bytes, bm, &full[s], pol);
            }
        }
        return;
    }

    const int team = warp / p.WPT;
    const int wit = warp - team * p.WPT;
    const int m = wit * 32 + lane;                    // chunk pair of this lane
    const bool live = m < p.slots;                    // slots = K / 64
    const int first = ((lane >> 2) & 1);              // lanes 4-7 of an octet read their odd chunk first
    const uint32_t off_first = (uint32_t)(2 * m + first) * 16u;
    const uint32_t off_second = (uint32_t)(2 * m + 1 - first) * 16u;
    const uint32_t meta_first = FMT == F_Q6K ? (uint32_t)(m >> 2) * 96u : FMT == F_Q5K ? (uint32_t)(m >> 2) * 48u : FMT == F_Q4K ? (uint32_t)(m >> 2) * 16u
                              : FMT == F_W4G ? (uint32_t)(m >> 1) * 4u : (uint32_t)(2 * m + first) * 2u;
    const uint32_t meta_second = (FMT == F_Q4K || FMT == F_Q5K || FMT == F_Q6K) ? (uint32_t)(m & 3)
                               : FMT == F_W4G ? meta_first : (uint32_t)(2 * m + 1 - first) * 2u;
    const int ctid = warp * 32 + lane;
    const int CT = CW * 32;
    const uint32_t team_off = (uint32_t)team * p.row_bytes, team_moff = (uint32_t)team * p.meta_row_bytes;
    const uint32_t step = (uint32_t)p.T * p.row_bytes, mstep = (uint32_t)p.T * p.meta_row_bytes;
    const uint32_t meta_base = (uint32_t)p.R * p.row_bytes;

    PairX<FMT> px;
    grid_dep_wait();                                  // x may be the previous kernel's output
    if (FUSED && p.fz.norm_weight) convert_x_cta_rmsnorm<FMT>(p, xs, xmeta, part, ctid, CT);
    else convert_x_cta<FMT>(p, xs, xmeta, ctid, CT);
    bar_sync(1, CT);
    load_pair_x<FMT>(xs, xmeta, p.K, m, first, live, px);

    __syncwarp();
    if (lane == 0) mbar_arrive(xdone);                // this warp no longer reads xs / xmeta

    const unsigned seq = ar_begin<AR>(p, ar_word, ctid, CT);
    const int tiles_per_pass = p.P / p.R;
    for (int t0 = 0; t0 < n_tiles; t0 += tiles_per_pass) {
        const int t1 = min(n_tiles, t0 + tiles_per_pass);
        for (int it = t0; it < t1; ++it) {
            const int s = it % S_all;
            // a warp that gives up raises the abort word and goes on to the barrier, where all warps leave together
            if (!mbar_wait(&full[s], (it / S_all) & 1)) { report_error(ZTQ_ERR_FULL_WAIT); *abort_word = 1; break; }
            const int rows = min(p.R, r_end - (r_begin + it * p.R));
            const uint8_t* sdata = smem + (uint32_t)s * p.stage_stride + team_off;
            const uint8_t* smeta = smem + (uint32_t)s * p.stage_stride + meta_base + team_moff;
            float acc[RT];
#pragma unroll
            for (int rr = 0; rr < RT; ++rr) acc[rr] = 0.f;
            if (live) {
                if (rows == p.R) {
#pragma unroll
                    for (int rr = 0; rr < RT; ++rr)
                        acc[rr] = pair_row<FMT>(sdata + rr * step, smeta + rr * mstep, off_first, off_second, meta_first,
                                                meta_second, px);
                } else {
#pragma unroll
                    for (int rr = 0; rr < RT; ++rr)
                        if (team + rr * p.T < rows)
                            acc[rr] = pair_row<FMT>(sdata + rr * step, smeta + rr * mstep, off_first, off_second,
                                                    meta_first, meta_second, px);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);

            const float tot = warp_sum_v<RT>(acc, lane);
            if ((lane & (32 / RT - 1)) == 0) {
                const int rr = lane / (32 / RT);
                const int lr = (it - t0) * p.R + team + rr * p.T;
                part[lr * p.WPT + wit] = tot;
            }
        }
        bar_sync(1, CT);
        if (*abort_word) break;                       // the same value in every warp
        const int prow0 = r_begin + t0 * p.R;
        const int prows = min(r_end, r_begin + t1 * p.R) - prow0;
        finish_pass<1, false, FUSED, AR>(p, part, prow0, prows, ctid, CT, seq, t0 / tiles_per_pass);
        if (t1 < n_tiles) bar_sync(1, CT);
    }
    ar_end<AR>(p, seq, ctid == 0);
}

}  // namespace ztq
