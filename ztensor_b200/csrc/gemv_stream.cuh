// gemv_stream.cuh -- batch-1/2 dequant-GEMV for every packed format, sm_100a.
//
// y[b, n] = sum_k dequant(W[n, k]) * x[b, k]          (W row-major [N, K], packed)
//
// One persistent CTA per (SM, slot): a producer thread streams whole weight
// rows into a ring of shared-memory stages with 1-D bulk async copies (TMA
// engine, mbarrier completion, no multicast); consumer warps are organised in
// teams.  A team spans K: thread t of a team owns the same 32 (ternary: 64)
// consecutive k of every row, so its activations live in registers for the
// whole kernel, already multiplied by the power of two that undoes the bit
// position its nibble is decoded at.  A nibble becomes a float with one LOP3
// (OR into the mantissa of 2^23) and one packed subtract; products accumulate
// in fp32 pairs (fma.rn.f32x2).  Row sums are reduced with a fixed butterfly,
// then across the warps of the team in warp order: results repeat bit for bit
// from run to run and do not depend on the grid size.
#pragma once

#include "ztq_common.cuh"

namespace ztq {

enum Fmt : int { F_Q4_0 = 0, F_IQ4NL = 1, F_W4G = 2, F_Q8_0 = 3, F_TERN = 4 };

struct GemvParams {
    const uint8_t* w;        // packed rows, row_bytes each
    const uint8_t* meta;     // per-row side data (scales / scale+zero), meta_row_bytes each; may be null
    const __half* row_scale; // ternary: optional fp16 scale per output row
    const void* x;           // activations, fp16 or fp32
    void* y;                 // outputs, fp16 or fp32
    long long xs_b, xs_k;    // element strides of x
    long long ys_b, ys_n;    // element strides of y
    int x_f32, y_f32;
    int N, K;
    int row_bytes, meta_row_bytes;
    int R;                   // rows per stage
    int S;                   // stages
    int stage_stride;        // bytes between stages
    int T;                   // teams per CTA
    int WPT;                 // warps per team
    int slots;               // K / slot width
    int part_off;            // smem offset of the partial-sum scratch
    int bar_off;             // smem offset of the mbarriers
};

template <int FMT> struct FmtTraits;
template <> struct FmtTraits<F_Q4_0>  { static constexpr int SLOT_W = 32, SLOT_B = 16, META_B = 2; };
template <> struct FmtTraits<F_IQ4NL> { static constexpr int SLOT_W = 32, SLOT_B = 16, META_B = 2; };
template <> struct FmtTraits<F_W4G>   { static constexpr int SLOT_W = 32, SLOT_B = 16, META_B = 1; };  // 4 B per 128
template <> struct FmtTraits<F_Q8_0>  { static constexpr int SLOT_W = 32, SLOT_B = 36, META_B = 0; };
template <> struct FmtTraits<F_TERN>  { static constexpr int SLOT_W = 64, SLOT_B = 16, META_B = 0; };

// IQ4_NL reconstruction points (tensor/iq4_storage.go:28-33 of the reference).
__constant__ float c_iq4nl[16] = {
    -1.0f, -0.6961928f, -0.5250730f, -0.3947555f, -0.2831612f, -0.1790887f, -0.0805542f, 0.0f,
    0.0805542f, 0.1790887f, 0.2831612f, 0.3947555f, 0.5250730f, 0.6961928f, 1.0f, 1.3312578f,
};

// ---- which k of its slot register i of a thread multiplies, and at which
// ---- mantissa bit the matching code is decoded (x is pre-scaled by 2^-p).
template <int FMT> __device__ __forceinline__ constexpr int reg_k(int i) {
    if (FMT == F_Q4_0) {            // byte j: low nibble = element j, high nibble = element j+16
        int m = i >> 3, j = i & 7;
        return (j & 1) ? 16 + 4 * m + (j >> 1) : 4 * m + (j >> 1);
    }
    return i;                       // sequential formats
}
template <int FMT> __device__ __forceinline__ constexpr int reg_p(int i) {
    if (FMT == F_Q4_0 || FMT == F_W4G) { int j = i & 7; return j < 5 ? 4 * j : 4 * j - 12; }
    if (FMT == F_TERN) { int t = i & 15; return t < 8 ? 2 * t : 2 * (t - 8); }
    return 0;
}

__device__ __forceinline__ float magic(uint32_t bits) { return __uint_as_float(0x4B000000u | bits); }

// Sum of code * x over one 32-bit word of eight nibbles; xr already carries 2^-p.
__device__ __forceinline__ void dot_word4(uint32_t w, const float* xr, f2& acc) {
    const f2 neg = {-8388608.0f, -8388608.0f};
    const uint32_t h = w >> 12;
    f2 v;
    v = fadd2(f2{magic(w & 0x0000000fu), magic(w & 0x000000f0u)}, neg); acc = ffma2(v, f2{xr[0], xr[1]}, acc);
    v = fadd2(f2{magic(w & 0x00000f00u), magic(w & 0x0000f000u)}, neg); acc = ffma2(v, f2{xr[2], xr[3]}, acc);
    v = fadd2(f2{magic(w & 0x000f0000u), magic(h & 0x00000f00u)}, neg); acc = ffma2(v, f2{xr[4], xr[5]}, acc);
    v = fadd2(f2{magic(h & 0x0000f000u), magic(h & 0x000f0000u)}, neg); acc = ffma2(v, f2{xr[6], xr[7]}, acc);
}

// Sixteen 2-bit codes per word.
__device__ __forceinline__ void dot_word2(uint32_t w, const float* xr, f2& acc) {
    const f2 neg = {-8388608.0f, -8388608.0f};
    const uint32_t h = w >> 16;
    f2 v;
#pragma unroll
    for (int t = 0; t < 8; t += 2) {
        v = fadd2(f2{magic(w & (3u << (2 * t))), magic(w & (3u << (2 * t + 2)))}, neg);
        acc = ffma2(v, f2{xr[t], xr[t + 1]}, acc);
    }
#pragma unroll
    for (int t = 0; t < 8; t += 2) {
        v = fadd2(f2{magic(h & (3u << (2 * t))), magic(h & (3u << (2 * t + 2)))}, neg);
        acc = ffma2(v, f2{xr[8 + t], xr[9 + t]}, acc);
    }
}

// Four int8 per word: flip the sign bit, drop each byte into the mantissa of
// 2^23, subtract 2^23 + 128.
__device__ __forceinline__ void dot_word8(uint32_t w, const float* xr, f2& acc) {
    const f2 neg = {-8388736.0f, -8388736.0f};
    const uint32_t u = w ^ 0x80808080u;
    f2 v;
    v = fadd2(f2{__uint_as_float(__byte_perm(u, 0x4B000000u, 0x7540)),
                 __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7541))}, neg);
    acc = ffma2(v, f2{xr[0], xr[1]}, acc);
    v = fadd2(f2{__uint_as_float(__byte_perm(u, 0x4B000000u, 0x7542)),
                 __uint_as_float(__byte_perm(u, 0x4B000000u, 0x7543))}, neg);
    acc = ffma2(v, f2{xr[2], xr[3]}, acc);
}

// One slot of one row against BC activation vectors.  Returns the slot's
// contribution to y, scale applied.
//   lut: per-lane copy of the IQ4_NL table in shared memory (entry e of lane l
//   at lut[e * 32 + l]), unused by the other formats.
template <int FMT, int BC>
__device__ __forceinline__ void slot_dot(const uint8_t* sdata, const uint8_t* smeta, int slot,
                                         const float (&xr)[BC][FmtTraits<FMT>::SLOT_W], const float (&sx)[BC],
                                         const float* lut, float (&out)[BC]) {
    if (FMT == F_Q8_0) {
        const uint32_t* blk = reinterpret_cast<const uint32_t*>(sdata + slot * 36);
        const float scale = __uint_as_float(blk[0]);
        f2 acc[BC];
#pragma unroll
        for (int b = 0; b < BC; ++b) acc[b] = f2{0.f, 0.f};
#pragma unroll
        for (int d = 0; d < 8; ++d) {
            const uint32_t w = blk[1 + d];
#pragma unroll
            for (int b = 0; b < BC; ++b) dot_word8(w, &xr[b][4 * d], acc[b]);
        }
#pragma unroll
        for (int b = 0; b < BC; ++b) out[b] = scale * (acc[b].x + acc[b].y);
        return;
    }
    const uint4 q = *reinterpret_cast<const uint4*>(sdata + slot * 16);
    const uint32_t qw[4] = {q.x, q.y, q.z, q.w};
    if (FMT == F_IQ4NL) {
        const float d = h2f(*reinterpret_cast<const uint16_t*>(smeta + slot * 2));
        float acc[BC];
#pragma unroll
        for (int b = 0; b < BC; ++b) acc[b] = 0.f;
#pragma unroll
        for (int m = 0; m < 4; ++m) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const uint32_t off = (j < 2) ? ((qw[m] << (7 - 4 * j)) & 0x780u) : ((qw[m] >> (4 * j - 7)) & 0x780u);
                const float t = *reinterpret_cast<const float*>(reinterpret_cast<const uint8_t*>(lut) + off);
#pragma unroll
                for (int b = 0; b < BC; ++b) acc[b] = fmaf(t, xr[b][8 * m + j], acc[b]);
            }
        }
#pragma unroll
        for (int b = 0; b < BC; ++b) out[b] = d * acc[b];
        return;
    }
    f2 acc[BC];
#pragma unroll
    for (int b = 0; b < BC; ++b) acc[b] = f2{0.f, 0.f};
    if (FMT == F_TERN) {
#pragma unroll
        for (int m = 0; m < 4; ++m)
#pragma unroll
            for (int b = 0; b < BC; ++b) dot_word2(qw[m], &xr[b][16 * m], acc[b]);
#pragma unroll
        for (int b = 0; b < BC; ++b) out[b] = (acc[b].x + acc[b].y) - sx[b];   // sum (c-1) x
        return;
    }
#pragma unroll
    for (int m = 0; m < 4; ++m)
#pragma unroll
        for (int b = 0; b < BC; ++b) dot_word4(qw[m], &xr[b][8 * m], acc[b]);
    if (FMT == F_Q4_0) {
        const float s = h2f(*reinterpret_cast<const uint16_t*>(smeta + slot * 2));
#pragma unroll
        for (int b = 0; b < BC; ++b) out[b] = s * ((acc[b].x + acc[b].y) - 8.0f * sx[b]);
    } else {  // F_W4G: (q - z) * s with one {scale, zero} pair per 128 weights
        const __half2 sz = *reinterpret_cast<const __half2*>(smeta + (slot >> 2) * 4);
        const float s = __low2float(sz), z = __high2float(sz);
#pragma unroll
        for (int b = 0; b < BC; ++b) out[b] = s * ((acc[b].x + acc[b].y) - z * sx[b]);
    }
}

// Values to reduce per thread = RT rows x BC batches (2 or 4).  After the call
// lane L holds the warp total of value index ((L>>4)&1) [V=2] or
// ((L>>4)&1)*2 + ((L>>3)&1) [V=4].
template <int V> __device__ __forceinline__ float warp_sum_v(const float (&v)[V], int lane) {
    if (V == 1) return warp_sum(v[0]);
    if (V == 2) return warp_sum2(v[0], v[1], lane);
    const bool h16 = (lane & 16) != 0;
    float k0 = h16 ? v[2] : v[0], k1 = h16 ? v[3] : v[1];
    const float s0 = h16 ? v[0] : v[2], s1 = h16 ? v[1] : v[3];
    k0 += __shfl_xor_sync(0xffffffffu, s0, 16);
    k1 += __shfl_xor_sync(0xffffffffu, s1, 16);
    const bool h8 = (lane & 8) != 0;
    float keep = h8 ? k1 : k0;
    const float send = h8 ? k0 : k1;
    keep += __shfl_xor_sync(0xffffffffu, send, 8);
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) keep += __shfl_xor_sync(0xffffffffu, keep, o);
    return keep;
}

constexpr int kRT = 2;   // rows per team per stage

template <int FMT, int BC, int SPT>
__global__ void __launch_bounds__(544, 1) gemv_stream_kernel(const GemvParams p) {
    using TR = FmtTraits<FMT>;
    constexpr int XN = TR::SLOT_W;
    constexpr int V = kRT * BC;
    extern __shared__ __align__(128) uint8_t smem[];

    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    const int CW = p.T * p.WPT;                       // consumer warps
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + p.bar_off);
    uint64_t* empty = full + p.S;
    float* part = reinterpret_cast<float*>(smem + p.part_off);   // [2][T][V][WPT]
    float* lut = part + 2 * p.T * V * p.WPT;                     // IQ4_NL only: [16][32]

    if (tid == 0) {
        for (int s = 0; s < p.S; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], CW); }
        mbar_fence_init();
    }
    if (FMT == F_IQ4NL) for (int i = tid; i < 512; i += blockDim.x) lut[i] = c_iq4nl[i >> 5];
    __syncthreads();
    grid_dep_launch();

    // contiguous row range of this CTA
    const int r_begin = (int)(((long long)p.N * blockIdx.x) / gridDim.x);
    const int r_end = (int)(((long long)p.N * (blockIdx.x + 1)) / gridDim.x);
    const int n_tiles = (r_end - r_begin + p.R - 1) / p.R;

    if (warp == CW) {
        // ------------------------------------------------ producer
        if (lane == 0) {
            const uint64_t pol = l2_evict_first_policy();
            for (int it = 0; it < n_tiles; ++it) {
                const int s = it % p.S;
                if (it >= p.S && !mbar_wait(&empty[s], ((it / p.S) - 1) & 1)) { report_error(ZTQ_ERR_EMPTY_WAIT); break; }
                const int row0 = r_begin + it * p.R;
                const int rows = min(p.R, r_end - row0);
                uint8_t* dst = smem + (size_t)s * p.stage_stride;
                const uint32_t bd = (uint32_t)rows * p.row_bytes;
                const uint32_t bm = (uint32_t)rows * p.meta_row_bytes;
                mbar_expect_tx(&full[s], bd + bm);
                bulk_g2s_hint(dst, p.w + (size_t)row0 * p.row_bytes, bd, &full[s], pol);
                if (bm) bulk_g2s_hint(dst + (size_t)p.R * p.row_bytes, p.meta + (size_t)row0 * p.meta_row_bytes, bm,
                                      &full[s], pol);
            }
        }
        return;
    }

    // ---------------------------------------------------- consumers
    const int team = warp / p.WPT;
    const int wit = warp - team * p.WPT;            // warp in team
    const int tit = wit * 32 + lane;                // thread in team
    const int G = p.WPT * 32;

    // activations of this thread's slots -> registers (scaled by 2^-p)
    float xr[SPT][BC][XN];
    float sx[SPT][BC];
    grid_dep_wait();                                // x may come from the previous kernel
#pragma unroll
    for (int sp = 0; sp < SPT; ++sp) {
        const int slot = tit + sp * G;
        const bool live = slot < p.slots;
#pragma unroll
        for (int b = 0; b < BC; ++b) {
            float s = 0.f;
#pragma unroll
            for (int i = 0; i < XN; ++i) {
                float v = 0.f;
                if (live) {
                    const long long idx = (long long)b * p.xs_b + (long long)(slot * XN + reg_k<FMT>(i)) * p.xs_k;
                    v = p.x_f32 ? reinterpret_cast<const float*>(p.x)[idx]
                                : __half2float(reinterpret_cast<const __half*>(p.x)[idx]);
                }
                s += v;
                xr[sp][b][i] = v * __uint_as_float((uint32_t)(127 - reg_p<FMT>(i)) << 23);
            }
            sx[sp][b] = s;
        }
    }

    for (int it = 0; it < n_tiles; ++it) {
        const int s = it % p.S;
        if (!mbar_wait(&full[s], (it / p.S) & 1)) { report_error(ZTQ_ERR_FULL_WAIT); break; }
        const int row0 = r_begin + it * p.R;
        const int rows = min(p.R, r_end - row0);
        const uint8_t* sdata = smem + (size_t)s * p.stage_stride;
        const uint8_t* smeta = sdata + (size_t)p.R * p.row_bytes;

        float acc[V];
#pragma unroll
        for (int v = 0; v < V; ++v) acc[v] = 0.f;
#pragma unroll
        for (int rr = 0; rr < kRT; ++rr) {
            const int r = team + rr * p.T;
            if (r < rows) {
#pragma unroll
                for (int sp = 0; sp < SPT; ++sp) {
                    const int slot = tit + sp * G;
                    if (slot < p.slots) {
                        float o[BC];
                        slot_dot<FMT, BC>(sdata + (size_t)r * p.row_bytes, smeta + (size_t)r * p.meta_row_bytes, slot,
                                          xr[sp], sx[sp], lut + lane, o);
#pragma unroll
                        for (int b = 0; b < BC; ++b) acc[rr * BC + b] += o[b];
                    }
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);       // stage may be refilled

        const float tot = warp_sum_v<V>(acc, lane);
        float* pp = part + ((size_t)((it & 1) * p.T + team) * V) * p.WPT;
        if ((lane & (V == 4 ? 7 : 15)) == 0) {
            const int vi = (V == 4) ? (lane >> 3) : (lane >> 4);
            pp[vi * p.WPT + wit] = tot;
        }
        if (p.WPT > 1) bar_sync(1 + team, G); else __syncwarp();
        if (tit < V) {
            float sum = 0.f;
            for (int w = 0; w < p.WPT; ++w) sum += pp[tit * p.WPT + w];   // warp order: fixed
            const int rr = tit / BC, b = tit - rr * BC;
            const int r = team + rr * p.T;
            if (r < rows) {
                const int n = row0 + r;
                if (FMT == F_TERN && p.row_scale) sum *= __half2float(p.row_scale[n]);
                const long long yi = (long long)b * p.ys_b + (long long)n * p.ys_n;
                if (p.y_f32) reinterpret_cast<float*>(p.y)[yi] = sum;
                else reinterpret_cast<__half*>(p.y)[yi] = __float2half_rn(sum);
            }
        }
    }
}

// ---------------------------------------------------------------------------
// Plain kernel for shapes the streaming kernel does not take (K not a multiple
// of the alignment the bulk copies need, or very long rows): one warp per
// row, direct 128-bit loads, the same dequantisation identities, lanes reduced
// with the same butterfly.
// ---------------------------------------------------------------------------
template <int FMT>
__global__ void __launch_bounds__(256) gemv_plain_kernel(const GemvParams p, int batch) {
    using TR = FmtTraits<FMT>;
    constexpr int XN = TR::SLOT_W;
    grid_dep_launch();
    grid_dep_wait();
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= p.N) return;
    const uint8_t* wrow = p.w + (size_t)row * p.row_bytes;
    const uint8_t* mrow = p.meta ? p.meta + (size_t)row * p.meta_row_bytes : nullptr;
    for (int b = 0; b < batch; ++b) {
        float acc = 0.f;
        for (int slot = lane; slot < p.slots; slot += 32) {
            float xv[XN];
            float sx = 0.f;
#pragma unroll
            for (int i = 0; i < XN; ++i) {
                const long long idx = (long long)b * p.xs_b + (long long)(slot * XN + i) * p.xs_k;
                xv[i] = p.x_f32 ? reinterpret_cast<const float*>(p.x)[idx]
                                : __half2float(reinterpret_cast<const __half*>(p.x)[idx]);
                sx += xv[i];
            }
            float d = 0.f;
            if (FMT == F_Q8_0) {
                const uint32_t* blk = reinterpret_cast<const uint32_t*>(wrow + (size_t)slot * 36);
                const float scale = __uint_as_float(blk[0]);
#pragma unroll
                for (int w = 0; w < 8; ++w) {
                    const uint32_t u = blk[1 + w];
#pragma unroll
                    for (int i = 0; i < 4; ++i) d = fmaf((float)(int8_t)((u >> (8 * i)) & 0xff), xv[4 * w + i], d);
                }
                d *= scale;
            } else if (FMT == F_TERN) {
                const uint4 q = *reinterpret_cast<const uint4*>(wrow + (size_t)slot * 16);
                const uint32_t qw[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                for (int m = 0; m < 4; ++m)
#pragma unroll
                    for (int t = 0; t < 16; ++t) {
                        const uint32_t c = (qw[m] >> (2 * t)) & 3u;
                        if (c == 2u) d += xv[16 * m + t];
                        else if (c == 0u) d -= xv[16 * m + t];
                    }
            } else {
                const uint4 q = *reinterpret_cast<const uint4*>(wrow + (size_t)slot * 16);
                const uint32_t qw[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                for (int m = 0; m < 4; ++m)
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const uint32_t nib = (qw[m] >> (4 * j)) & 0xfu;
                        const int i = 8 * m + j;
                        if (FMT == F_IQ4NL) d = fmaf(c_iq4nl[nib], xv[i], d);
                        else d = fmaf((float)nib, xv[reg_k<FMT>(i)], d);
                    }
                if (FMT == F_Q4_0) d = h2f(*reinterpret_cast<const uint16_t*>(mrow + slot * 2)) * (d - 8.0f * sx);
                else if (FMT == F_IQ4NL) d = h2f(*reinterpret_cast<const uint16_t*>(mrow + slot * 2)) * d;
                else {
                    const __half2 sz = *reinterpret_cast<const __half2*>(mrow + (slot >> 2) * 4);
                    d = __low2float(sz) * (d - __high2float(sz) * sx);
                }
            }
            acc += d;
        }
        acc = warp_sum(acc);
        if (lane == 0) {
            if (FMT == F_TERN && p.row_scale) acc *= __half2float(p.row_scale[row]);
            const long long yi = (long long)b * p.ys_b + (long long)row * p.ys_n;
            if (p.y_f32) reinterpret_cast<float*>(p.y)[yi] = acc;
            else reinterpret_cast<__half*>(p.y)[yi] = __float2half_rn(acc);
        }
    }
}

}  // namespace ztq
