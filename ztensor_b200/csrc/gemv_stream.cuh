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

enum Fmt : int { F_Q4_0 = 0, F_IQ4NL = 1, F_W4G = 2, F_Q8_0 = 3, F_TERN = 4, F_Q4K = 5, F_Q5K = 6, F_Q6K = 7 };   // the K-quants: chunk-pair kernel only

constexpr int kMaxRanks = 8;

// All-reduce fused into a row-parallel GEMV (one process per GPU, peers mapped
// with CUDA IPC).  Each rank owns
//   slots  [2][world][slot_stride] cells of 8 bytes {fp32 partial, tag}, double-buffered by launch parity
//   state  [2] unsigned                 {launch sequence, CTAs finished} of this rank
// and holds the peers' `slots` addresses.  world == 0: no all-reduce.
struct ArParams {
    int world, rank;
    int slot_stride;
    uint2* slots[kMaxRanks];
    unsigned* state;
};

// Element-wise work of the steps either side of a projection, folded into the GEMV (chunk-pair kernel only).
struct FuseParams {
    const void* residual;      // [K], same type as x: x + residual is what gets normalised (null: x alone)
    const float* norm_weight;  // [K] float32 gains of the RMSNorm; null = no normalisation
    void* sum_out;             // [K], same type as x: x + residual, written by the first CTA (null: not wanted)
    float eps;
    int swiglu;                // rows are (gate_i, up_i) pairs: y[i] = silu(gate_i) * up_i, N / 2 outputs
};

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
    int Sx;                  // chunk-pair kernel: further stages that reuse the activation planes' shared memory once every
                             // warp holds its activations in registers
    int stage_stride;        // bytes between stages
    int T;                   // teams per CTA
    int WPT;                 // warps per team
    int slots;               // K / slot width
    int P;                   // rows per pass (multiple of R): partial sums of a pass live in smem
    int part_off;            // smem offset of the partial-sum scratch
    int bar_off;             // smem offset of the mbarriers
    int x_off;               // smem offset of the converted activations (chunk-pair kernel)
    int gshift;              // W4G: log2(group / 32): 32-weight slot s belongs to group s >> gshift
    // split-K: the grid is `splits` groups of CTAs; group g handles columns [g K, (g+1) K) of rows that are
    // w_stride / meta_stride bytes apart, reads x from element g K on and writes y at element g N.
    int splits;              // 0 or 1: no split
    int w_stride, meta_stride;
    ArParams ar;             // fused all-reduce of the outputs (row-parallel shards)
    FuseParams fz;           // fused RMSNorm on x / SwiGLU on y (all zero: off)
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
                                         const float* lut, float (&out)[BC], int gshift = 2) {
    if (FMT == F_Q8_0) {
        const uint32_t* blk = reinterpret_cast<const uint32_t*>(sdata + slot * 36);
        const float scale = __uint_as_float(blk[0]);
        f2 acc[BC][2];                       // two independent chains per vector
#pragma unroll
        for (int b = 0; b < BC; ++b) acc[b][0] = acc[b][1] = f2{0.f, 0.f};
#pragma unroll
        for (int d = 0; d < 8; ++d) {
            const uint32_t w = blk[1 + d];
#pragma unroll
            for (int b = 0; b < BC; ++b) dot_word8(w, &xr[b][4 * d], acc[b][d & 1]);
        }
#pragma unroll
        for (int b = 0; b < BC; ++b) out[b] = scale * ((acc[b][0].x + acc[b][0].y) + (acc[b][1].x + acc[b][1].y));
        return;
    }
    const uint4 q = *reinterpret_cast<const uint4*>(sdata + slot * 16);
    const uint32_t qw[4] = {q.x, q.y, q.z, q.w};
    if (FMT == F_IQ4NL) {
        const float d = h2f(*reinterpret_cast<const uint16_t*>(smeta + slot * 2));
        float acc[BC][2];
#pragma unroll
        for (int b = 0; b < BC; ++b) acc[b][0] = acc[b][1] = 0.f;
#pragma unroll
        for (int m = 0; m < 4; ++m) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const uint32_t off = (j < 2) ? ((qw[m] << (7 - 4 * j)) & 0x780u) : ((qw[m] >> (4 * j - 7)) & 0x780u);
                const float t = *reinterpret_cast<const float*>(reinterpret_cast<const uint8_t*>(lut) + off);
#pragma unroll
                for (int b = 0; b < BC; ++b) acc[b][j & 1] = fmaf(t, xr[b][8 * m + j], acc[b][j & 1]);
            }
        }
#pragma unroll
        for (int b = 0; b < BC; ++b) out[b] = d * (acc[b][0] + acc[b][1]);
        return;
    }
    f2 acc2[BC][2];                          // two independent chains per vector
#pragma unroll
    for (int b = 0; b < BC; ++b) acc2[b][0] = acc2[b][1] = f2{0.f, 0.f};
    if (FMT == F_TERN) {
#pragma unroll
        for (int m = 0; m < 4; ++m)
#pragma unroll
            for (int b = 0; b < BC; ++b) dot_word2(qw[m], &xr[b][16 * m], acc2[b][m & 1]);
#pragma unroll
        for (int b = 0; b < BC; ++b)
            out[b] = ((acc2[b][0].x + acc2[b][0].y) + (acc2[b][1].x + acc2[b][1].y)) - sx[b];   // sum (c-1) x
        return;
    }
#pragma unroll
    for (int m = 0; m < 4; ++m)
#pragma unroll
        for (int b = 0; b < BC; ++b) dot_word4(qw[m], &xr[b][8 * m], acc2[b][m & 1]);
    f2 acc[BC];
#pragma unroll
    for (int b = 0; b < BC; ++b) acc[b] = f2{acc2[b][0].x + acc2[b][1].x, acc2[b][0].y + acc2[b][1].y};
    if (FMT == F_Q4_0) {
        const float s = h2f(*reinterpret_cast<const uint16_t*>(smeta + slot * 2));
#pragma unroll
        for (int b = 0; b < BC; ++b) out[b] = s * ((acc[b].x + acc[b].y) - 8.0f * sx[b]);
    } else {  // F_W4G: (q - z) * s with one {scale, zero} pair per 128 weights
        const __half2 sz = *reinterpret_cast<const __half2*>(smeta + (slot >> gshift) * 4);
        const float s = __low2float(sz), z = __high2float(sz);
#pragma unroll
        for (int b = 0; b < BC; ++b) out[b] = s * ((acc[b].x + acc[b].y) - z * sx[b]);
    }
}

// ---------------------------------------------------------------------------
// Final phase of a pass: the per-warp partial sums of rows [row0, row0 + rows)
// are in shared memory (part[(lr * BC + b) * WPT + w]); add them in warp order
// and write y.  With an all-reduce attached the sum is first pushed as fp32 to
// slot (parity, my rank) of EVERY rank, then a sequence flag is published to
// every rank, the CTA waits (bounded) until every rank has published the same
// sequence number for this CTA index, and the final value is the sum of the
// local slots in rank order, identical bit for bit on all ranks.  All ranks run
// the same launch sequence with the same grid, so CTA c of launch s on rank a
// pairs with CTA c of launch s on rank b; `seq` is read from device memory after
// the grid dependency wait, so a replayed CUDA graph counts launches correctly.
// ---------------------------------------------------------------------------
// yoff: element offset of this K-split's partial outputs (0 without a split)
__device__ __forceinline__ void store_y(const GemvParams& p, int b, int n, float v, long long yoff = 0) {
    const long long yi = (long long)b * p.ys_b + (long long)n * p.ys_n + yoff;
    if (p.y_f32) reinterpret_cast<float*>(p.y)[yi] = v;
    else reinterpret_cast<__half*>(p.y)[yi] = __float2half_rn(v);
}

// AR: the all-reduce over the ranks of a row-parallel shard is compiled in (separate instantiations: its cells and polls
// cost every kernel registers, and a spill costs a trip to L2 when shared memory takes nearly all of the L1).
template <int BC, bool TERN, bool FUSED = false, bool AR = false>
__device__ __forceinline__ void finish_pass(const GemvParams& p, const float* part, int row0, int rows, int ctid, int CT,
                                            unsigned seq, int pass_idx, long long yoff = 0) {
    if (FUSED && !AR && BC == 1 && p.fz.swiglu) {
        // rows (2j, 2j+1) = (gate_j, up_j): silu(gate) * up, the formula of fused_swiglu.cu:10-21 of the reference
        for (int j = ctid; j < rows / 2; j += CT) {
            float g = 0.f, u = 0.f;
            for (int w = 0; w < p.WPT; ++w) { g += part[(size_t)(2 * j) * p.WPT + w]; u += part[(size_t)(2 * j + 1) * p.WPT + w]; }
            const float sig = 1.0f / (1.0f + expf(-g));
            store_y(p, 0, row0 / 2 + j, g * sig * u);
        }
        return;
    }
    if constexpr (!AR) {
        for (int i = ctid; i < rows * BC; i += CT) {
            float sum = 0.f;
            for (int w = 0; w < p.WPT; ++w) sum += part[(size_t)i * p.WPT + w];     // warp order: fixed
            const int lr = i / BC, b = i - lr * BC;
            if (TERN && p.row_scale) sum *= __half2float(p.row_scale[row0 + lr]);
            store_y(p, b, row0 + lr, sum, yoff);
        }
        return;
    } else {
    // Every output row travels as one 8-byte cell {fp32 partial, tag}: a single store per peer,
    // no flags and no fences.  The thread that produced a row pushes it to every rank, then
    // polls (bounded) its own rank's cells of that row until each carries this launch's tag and
    // adds them in rank order.  Cells are double-buffered by launch parity: a peer can be at
    // most one all-reduce ahead, so it never overwrites a cell that is still being waited for.
    // The tag is the launch sequence number (+1: zero-initialised cells carry 0).  A row belongs to exactly one
    // pass of one CTA, so its cell is written once per launch and the pass index adds nothing; the full 32 bits of
    // the sequence are kept, and a cell of this parity was last written two launches ago, so a wrap of the counter
    // cannot make a stale cell look current.
    (void)pass_idx;
    const unsigned tag = seq + 1u;
    const size_t par_off = (size_t)(seq & 1u) * p.ar.world * p.ar.slot_stride;
    for (int i = ctid; i < rows * BC; i += CT) {
        float sum = 0.f;
        for (int w = 0; w < p.WPT; ++w) sum += part[(size_t)i * p.WPT + w];     // warp order: fixed
        const int lr = i / BC, b = i - lr * BC;
        const size_t idx = (size_t)b * p.N + (row0 + lr);
        const size_t mine = par_off + (size_t)p.ar.rank * p.ar.slot_stride + idx;
        for (int r = 0; r < p.ar.world; ++r) st_cell_sys(p.ar.slots[r] + mine, __float_as_uint(sum), tag);
    }
    for (int i = ctid; i < rows * BC; i += CT) {
        const int lr = i / BC, b = i - lr * BC;
        const size_t idx = (size_t)b * p.N + (row0 + lr);
        const uint2* src = p.ar.slots[p.ar.rank] + par_off + idx;
        // All ranks' cells are requested before any is looked at, and on every further round all that are still
        // missing are requested together: the round trips to L2 overlap instead of following one another (waiting for
        // rank 0's cell, then finding rank 1's copy stale and fetching it again, and so on, cost one round trip per
        // peer: about 3 us at eight ranks).
        uint2 v[kMaxRanks];
#pragma unroll
        for (int r = 0; r < kMaxRanks; ++r)
            if (r < p.ar.world) v[r] = ld_cell_sys(src + (size_t)r * p.ar.slot_stride);
        bool ok = true;
        for (uint32_t it = 0;; ++it) {
            bool all = true;
#pragma unroll
            for (int r = 0; r < kMaxRanks; ++r)
                if (r < p.ar.world && v[r].y != tag) all = false;
            if (all) break;
            if (it >= (1u << 21)) { ok = false; break; }                    // about a second: give up, flag, return
            __nanosleep(20);
#pragma unroll
            for (int r = 0; r < kMaxRanks; ++r)
                if (r < p.ar.world && v[r].y != tag) v[r] = ld_cell_sys(src + (size_t)r * p.ar.slot_stride);
        }
        float tot = 0.f;
#pragma unroll
        for (int r = 0; r < kMaxRanks; ++r)
            if (r < p.ar.world) tot += __uint_as_float(v[r].x);             // rank order: fixed
        if (!ok) report_error(ZTQ_ERR_FLAG_WAIT);
        store_y(p, b, row0 + lr, tot);
    }
    }                                                           // AR
}

// Launch sequence number of this rank's all-reduce kernels: read after the grid
// dependency wait; the last CTA to finish advances it for the next launch.
// One thread reads the word; the others get it through shared memory.
template <bool AR>
__device__ __forceinline__ unsigned ar_begin(const GemvParams& p, unsigned* smem_word, int ctid, int CT) {
    if (!AR) return 0;
    // `state` is only ever touched by this rank's own kernels, and the previous kernel is
    // complete (grid dependency wait): a plain load sees its last value.
    if (ctid == 0) *smem_word = *reinterpret_cast<volatile unsigned*>(p.ar.state);
    bar_sync(1, CT);
    return *smem_word;
}
template <bool AR>
__device__ __forceinline__ void ar_end(const GemvParams& p, unsigned seq, bool leader) {
    if (!AR || !leader) return;
    __threadfence();
    const unsigned done = atomicAdd(p.ar.state + 1, 1u) + 1u;
    if (done == gridDim.x) {                       // last CTA: local state for this rank's next launch
        p.ar.state[1] = 0;
        p.ar.state[0] = seq + 1u;
    }
}

// ===========================================================================
// Integer inner loop.
//
// The activations of a slot are turned, once per kernel, into block-fixed-point:
// X_k = x_k * 2^s rounded to an integer with s chosen so that |X_k| <= 2^21
// (fp16 inputs within a factor 2^10 of the slot's largest magnitude are
// represented exactly, smaller ones to 2^-22 of that magnitude), and split into
// int8 planes X = p2 * 65536 + p1 * 256 + p0 (p2 signed, p1 and p0 unsigned).  The codes of
// a row are masked into bytes (one LOP3 per four codes) and multiplied with
// dp4a: the dot product of a slot is an exact integer.  Scales, zero points and
// the sum over slots are fp32.
// ===========================================================================
template <int NP, int XN> struct XInt {
    uint32_t w[NP][XN / 4];   // plane p, word j = four activations in the order the codes are consumed
    float inv;                // 2^-s
    float sxf;                // sum of the slot's activations (for the -8 / -zero / -1 offsets)
};

// order in which dp4a consumes the activations of a slot
template <int FMT> __device__ __forceinline__ constexpr int int_k(int i) {
    if (FMT == F_W4G || FMT == F_IQ4NL) {     // byte b: low nibble = element 2b, high = 2b+1
        // words 0..3: even elements of byte-words 0..3, words 4..7: odd elements
        int wd = i >> 2, j = i & 3;
        return wd < 4 ? 8 * wd + 2 * j : 8 * (wd - 4) + 2 * j + 1;
    }
    if (FMT == F_TERN) {                      // word m, shift t: codes 16m + t + 4j
        int wd = i >> 2, j = i & 3;
        int m = wd >> 2, t = wd & 3;
        return 16 * m + t + 4 * j;
    }
    return i;                                 // Q4_0 (low nibbles = first 16, high = last 16) and Q8_0
}

__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c) {   // unsigned a, signed b
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ int dp4a_uu(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.u32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ int dp4a_ss(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ int dp4a_su(uint32_t a, uint32_t b, int c) {   // signed a, unsigned b
    int d;
    asm("dp4a.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// byte `pl` of four integers -> one word (a in the low byte)
__device__ __forceinline__ uint32_t pack_plane(uint32_t a, uint32_t b, uint32_t c, uint32_t d, int pl) {
    const uint32_t ab = __byte_perm(a, b, 0x0040 + 0x0011 * pl);
    const uint32_t cd = __byte_perm(c, d, 0x0040 + 0x0011 * pl);
    return __byte_perm(ab, cd, 0x5410);
}
// bytes 0, 1, 2 of four integers -> three words (seven byte permutes)
__device__ __forceinline__ void transpose3(uint32_t a, uint32_t b, uint32_t c, uint32_t d, uint32_t (&out)[3]) {
    const uint32_t ab = __byte_perm(a, b, 0x5140), cd = __byte_perm(c, d, 0x5140);   // {a0 b0 a1 b1}, {c0 d0 c1 d1}
    out[0] = __byte_perm(ab, cd, 0x5410);
    out[1] = __byte_perm(ab, cd, 0x7632);
    out[2] = __byte_perm(__byte_perm(a, b, 0x0062), __byte_perm(c, d, 0x0062), 0x5410);
}
// The integers come from the mantissa of (x * 2^s + 1.5 * 2^23): their low 24
// bits are X + 2^22.  Planes 0 and 1 are the low bytes of X as they stand; the
// top byte is 0x40 + (X >> 16) and becomes the signed byte (X >> 16) with three
// word-wide operations (no borrow can cross a byte: every byte is in [0x20, 0x5f]).
__device__ __forceinline__ uint32_t fix_top_plane(uint32_t w) {
    return ((w | 0x80808080u) - 0x40404040u) ^ 0x80808080u;
}

template <int FMT, int NP, int XN>
__device__ __forceinline__ void make_xint(const float (&raw)[XN], XInt<NP, XN>& xi) {
    static_assert(NP == 3, "three planes");
    float am = 0.f, s = 0.f;
#pragma unroll
    for (int i = 0; i < XN; ++i) { am = fmaxf(am, fabsf(raw[i])); s += raw[i]; }
    xi.sxf = s;
    // s = 20 - floor(log2(am)): |X| <= 2^21 (a float32 activation just below a power of two may round up to
    // it), so that sum(code * X) over a slot fits an int32 for 4-bit and 2-bit codes (64 * 15 * 2^21 < 2^31)
    // and X + 2^22 stays inside the mantissa
    const int top = 20;
    const uint32_t e = __float_as_uint(am) >> 23;             // biased exponent (am >= 0)
    const uint32_t eb = am > 0.f ? e : 127u;
    const float scale = __uint_as_float((uint32_t)(127 + top + 127 - (int)eb) << 23);
    xi.inv = __uint_as_float((uint32_t)((int)eb - top) << 23);
    // x * 2^s + 1.5 * 2^23: one FMA rounds to the nearest integer (ties to even, like cvt.rni) and leaves
    // X + 2^22 in the low 24 bits -- no conversion instruction (those run at a quarter of the FMA rate)
    uint32_t X[XN];
#pragma unroll
    for (int i = 0; i < XN; ++i) X[i] = __float_as_uint(fmaf(raw[i], scale, 12582912.0f));
#pragma unroll
    for (int j = 0; j < XN / 4; ++j) {
        uint32_t pl[3];
        transpose3(X[int_k<FMT>(4 * j)], X[int_k<FMT>(4 * j + 1)], X[int_k<FMT>(4 * j + 2)], X[int_k<FMT>(4 * j + 3)], pl);
        xi.w[0][j] = pl[0];
        xi.w[1][j] = pl[1];
        xi.w[2][j] = fix_top_plane(pl[2]);
    }
}

// (sum over the slot of code * X) as a float: planes combined high to low.
// EXACT_INT: the total fits an int32 (4-bit and 2-bit codes), combine in integers
// and convert once; otherwise (int8 weights) combine in fp32.
template <int NP, bool EXACT_INT> __device__ __forceinline__ float combine_planes(const int (&S)[NP]) {
    if (EXACT_INT) {
        if (NP == 3) return (float)((S[2] * 256 + S[1]) * 256 + S[0]);
        return (float)(S[1] * 256 + S[0]);
    }
    if (NP == 3) return fmaf(fmaf((float)S[2], 256.0f, (float)S[1]), 256.0f, (float)S[0]);
    return fmaf((float)S[1], 256.0f, (float)S[0]);
}

template <int FMT, int BC, int NP>
__device__ __forceinline__ void slot_dot_int(const uint8_t* sdata, const uint8_t* smeta, int slot,
                                             const XInt<NP, FmtTraits<FMT>::SLOT_W> (&xi)[BC], float (&out)[BC],
                                             int gshift = 2) {
    int S[BC][NP];
#pragma unroll
    for (int b = 0; b < BC; ++b)
#pragma unroll
        for (int pl = 0; pl < NP; ++pl) S[b][pl] = 0;

    if (FMT == F_Q8_0) {
        const uint32_t* blk = reinterpret_cast<const uint32_t*>(sdata + slot * 36);
        const float scale = __uint_as_float(blk[0]);
#pragma unroll
        for (int d = 0; d < 8; ++d) {
            const uint32_t w = blk[1 + d];
#pragma unroll
            for (int b = 0; b < BC; ++b) {
#pragma unroll
                for (int pl = 0; pl < NP - 1; ++pl) S[b][pl] = dp4a_su(w, xi[b].w[pl][d], S[b][pl]);
                S[b][NP - 1] = dp4a_ss(w, xi[b].w[NP - 1][d], S[b][NP - 1]);
            }
        }
#pragma unroll
        for (int b = 0; b < BC; ++b) out[b] = (scale * xi[b].inv) * combine_planes<NP, false>(S[b]);
        return;
    }
    const uint4 q = *reinterpret_cast<const uint4*>(sdata + slot * 16);
    const uint32_t qw[4] = {q.x, q.y, q.z, q.w};
    if (FMT == F_TERN) {
#pragma unroll
        for (int m = 0; m < 4; ++m) {
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                const uint32_t c = (qw[m] >> (2 * t)) & 0x03030303u;
#pragma unroll
                for (int b = 0; b < BC; ++b) {
#pragma unroll
                    for (int pl = 0; pl < NP - 1; ++pl) S[b][pl] = dp4a_uu(c, xi[b].w[pl][4 * m + t], S[b][pl]);
                    S[b][NP - 1] = dp4a_us(c, xi[b].w[NP - 1][4 * m + t], S[b][NP - 1]);
                }
            }
        }
#pragma unroll
        for (int b = 0; b < BC; ++b) out[b] = fmaf(combine_planes<NP, true>(S[b]), xi[b].inv, -xi[b].sxf);   // sum (c-1) x
        return;
    }
#pragma unroll
    for (int m = 0; m < 4; ++m) {
        const uint32_t lo = qw[m] & 0x0f0f0f0fu;
        const uint32_t hi = (qw[m] >> 4) & 0x0f0f0f0fu;
#pragma unroll
        for (int b = 0; b < BC; ++b) {
#pragma unroll
            for (int pl = 0; pl < NP - 1; ++pl) {
                S[b][pl] = dp4a_uu(lo, xi[b].w[pl][m], S[b][pl]);
                S[b][pl] = dp4a_uu(hi, xi[b].w[pl][4 + m], S[b][pl]);
            }
            S[b][NP - 1] = dp4a_us(lo, xi[b].w[NP - 1][m], S[b][NP - 1]);
            S[b][NP - 1] = dp4a_us(hi, xi[b].w[NP - 1][4 + m], S[b][NP - 1]);
        }
    }
    if (FMT == F_Q4_0) {
        const float s = h2f(*reinterpret_cast<const uint16_t*>(smeta + slot * 2));
#pragma unroll
        for (int b = 0; b < BC; ++b) out[b] = s * fmaf(combine_planes<NP, true>(S[b]), xi[b].inv, -8.0f * xi[b].sxf);
    } else {  // F_W4G
        const __half2 sz = *reinterpret_cast<const __half2*>(smeta + (slot >> gshift) * 4);
        const float s = __low2float(sz), z = __high2float(sz);
#pragma unroll
        for (int b = 0; b < BC; ++b) out[b] = s * fmaf(combine_planes<NP, true>(S[b]), xi[b].inv, -z * xi[b].sxf);
    }
}

// Transposed butterfly over V = 2, 4 or 8 per-lane values: each halving step
// exchanges half of the values with the partner lane, so V values cost about
// V + 5 - log2(V) shuffles instead of 5 V.  Afterwards lane L holds the warp
// total of value index L / (32 / V) (all lanes of that group hold it).  The
// association order depends only on lane ids: results repeat bit for bit.
template <int V> __device__ __forceinline__ float warp_sum_v(float (&v)[V], int lane) {
    int o = 16;
#pragma unroll
    for (int n = V; n > 1; n >>= 1, o >>= 1) {
        const bool up = (lane & o) != 0;
#pragma unroll
        for (int i = 0; i < n / 2; ++i) {
            const float keep = up ? v[i + n / 2] : v[i];
            const float send = up ? v[i] : v[i + n / 2];
            v[i] = keep + __shfl_xor_sync(0xffffffffu, send, o);
        }
    }
#pragma unroll
    for (; o > 0; o >>= 1) v[0] += __shfl_xor_sync(0xffffffffu, v[0], o);
    return v[0];
}

// Activations of one slot -> registers, permuted to the order the codes are
// decoded in and multiplied by 2^-p.  Fast path: contiguous fp16, 16-byte aligned.
// xoff: element offset of this K-split's activations (0 without a split)
template <int XN>
__device__ __forceinline__ void load_x_raw(const GemvParams& p, int b, int slot, bool live, float (&raw)[XN], long long xoff = 0) {
    const bool fast = !p.x_f32 && p.xs_k == 1;
    if (fast) {
        const __half* base = reinterpret_cast<const __half*>(p.x) + (long long)b * p.xs_b + (long long)slot * XN + xoff;
        if (live && (reinterpret_cast<uintptr_t>(base) & 15) == 0) {
#pragma unroll
            for (int v = 0; v < XN / 8; ++v) {
                const uint4 q = reinterpret_cast<const uint4*>(base)[v];
                const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const __half2 h = *reinterpret_cast<const __half2*>(&w[j]);
                    raw[v * 8 + 2 * j] = __low2float(h);
                    raw[v * 8 + 2 * j + 1] = __high2float(h);
                }
            }
        } else {
#pragma unroll
            for (int i = 0; i < XN; ++i) raw[i] = live ? __half2float(base[i]) : 0.f;
        }
    } else {
#pragma unroll
        for (int i = 0; i < XN; ++i) {
            float v = 0.f;
            if (live) {
                const long long idx = (long long)b * p.xs_b + (long long)(slot * XN + i) * p.xs_k + xoff;
                v = p.x_f32 ? reinterpret_cast<const float*>(p.x)[idx]
                            : __half2float(reinterpret_cast<const __half*>(p.x)[idx]);
            }
            raw[i] = v;
        }
    }
}

template <int FMT, int XN>
__device__ __forceinline__ void load_x_slot(const GemvParams& p, int b, int slot, bool live, float (&xr)[XN], float& sx,
                                            long long xoff = 0) {
    float raw[XN];
    load_x_raw<XN>(p, b, slot, live, raw, xoff);
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < XN; ++i) s += raw[i];
    sx = s;
#pragma unroll
    for (int i = 0; i < XN; ++i) xr[i] = raw[reg_k<FMT>(i)] * __uint_as_float((uint32_t)(127 - reg_p<FMT>(i)) << 23);
}

// BIG = 17-warp CTA owning a whole SM (long rows); otherwise 9 warps and half
// an SM, so that the next GEMV in the stream (programmatic dependent launch)
// is resident and prefetching its weights while this one computes.
// FP = decode codes to fp32 in registers (magic-number LOP3) instead of the
// integer inner loop; IQ4_NL (a float table) always takes the fp32 path.
template <int FMT, int BC, int SPT, int RT, bool BIG, bool FP, bool AR = false>
__global__ void __launch_bounds__(BIG ? 544 : 288, BIG ? 1 : 2) gemv_stream_kernel(const GemvParams p) {
    using TR = FmtTraits<FMT>;
    constexpr int XN = TR::SLOT_W;
    constexpr int V = RT * BC;
    constexpr int NP = 3;
    extern __shared__ __align__(128) uint8_t smem[];

    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    const int CW = p.T * p.WPT;                       // consumer warps
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + p.bar_off);
    uint64_t* empty = full + p.S;
    float* part = reinterpret_cast<float*>(smem + p.part_off);   // [P rows][BC][WPT]
    float* lut = part + p.P * BC * p.WPT;                        // IQ4_NL only: [16][32]

    // two words behind the barriers: the all-reduce sequence number of this launch, and the CTA's abort word
    unsigned* ar_word = reinterpret_cast<unsigned*>(empty + p.S);
    volatile unsigned* abort_word = ar_word + 1;
    if (tid == 0) {
        for (int s = 0; s < p.S; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], CW); }
        *abort_word = 0;
        mbar_fence_init();
    }
    if (FMT == F_IQ4NL) for (int i = tid; i < 512; i += blockDim.x) lut[i] = c_iq4nl[i >> 5];
    __syncthreads();
    grid_dep_launch();

    // contiguous row range of this CTA (within its K-split, if any)
    int cta = blockIdx.x, nctas = gridDim.x, split = 0;
    if (p.splits > 1) {
        nctas = gridDim.x / p.splits;
        split = blockIdx.x / nctas;
        cta = blockIdx.x - split * nctas;
    }
    const int r_begin = (int)(((long long)p.N * cta) / nctas);
    const int r_end = (int)(((long long)p.N * (cta + 1)) / nctas);
    const int n_tiles = (r_end - r_begin + p.R - 1) / p.R;

    if (warp == CW) {
        // ------------------------------------------------ producer (weights never depend on the previous kernel)
        if (lane == 0) {
            const uint64_t pol = l2_evict_first_policy();
            const bool strided = p.splits > 1;
            const uint8_t* wbase = p.w + (strided ? (size_t)split * p.row_bytes : 0);
            const uint8_t* mbase = p.meta + (strided ? (size_t)split * p.meta_row_bytes : 0);
            for (int it = 0; it < n_tiles; ++it) {
                const int s = it % p.S;
                if (it >= p.S && !mbar_wait(&empty[s], ((it / p.S) - 1) & 1)) { report_error(ZTQ_ERR_EMPTY_WAIT); break; }
                const int row0 = r_begin + it * p.R;
                const int rows = min(p.R, r_end - row0);
                uint8_t* dst = smem + (size_t)s * p.stage_stride;
                const uint32_t bd = (uint32_t)rows * p.row_bytes;
                const uint32_t bm = (uint32_t)rows * p.meta_row_bytes;
                mbar_expect_tx(&full[s], bd + bm);
                if (!strided) {
                    bulk_g2s_hint(dst, wbase + (size_t)row0 * p.row_bytes, bd, &full[s], pol);
                    if (bm) bulk_g2s_hint(dst + (size_t)p.R * p.row_bytes, mbase + (size_t)row0 * p.meta_row_bytes, bm,
                                          &full[s], pol);
                } else {                     // one copy per row: the K-slices of consecutive rows are not adjacent
                    for (int r = 0; r < rows; ++r) {
                        bulk_g2s_hint(dst + (size_t)r * p.row_bytes, wbase + (size_t)(row0 + r) * p.w_stride, p.row_bytes,
                                      &full[s], pol);
                        if (bm) bulk_g2s_hint(dst + (size_t)p.R * p.row_bytes + (size_t)r * p.meta_row_bytes,
                                              mbase + (size_t)(row0 + r) * p.meta_stride, p.meta_row_bytes, &full[s], pol);
                    }
                }
            }
        }
        return;
    }

    // ---------------------------------------------------- consumers
    const int team = warp / p.WPT;
    const int wit = warp - team * p.WPT;            // warp in team
    const int tit = wit * 32 + lane;                // thread in team
    const int G = p.WPT * 32;
    const int ctid = warp * 32 + lane;              // consumer thread id
    const int CT = CW * 32;

    float xr[FP ? SPT : 1][FP ? BC : 1][FP ? XN : 1];
    float sx[FP ? SPT : 1][FP ? BC : 1];
    XInt<NP, XN> xi[FP ? 1 : SPT][FP ? 1 : BC];
    // this split's view of x and y, as element offsets (a modified copy of the parameter block would live in local
    // memory: 280 bytes per thread behind an L1 that the shared-memory carve-out leaves almost nothing of)
    const long long xoff = p.splits > 1 ? (long long)split * p.K * p.xs_k : 0;
    const long long yoff = p.splits > 1 ? (long long)split * p.N : 0;
    grid_dep_wait();                                // x may be the previous kernel's output
#pragma unroll
    for (int sp = 0; sp < SPT; ++sp) {
        const int slot = tit + sp * G;
#pragma unroll
        for (int b = 0; b < BC; ++b) {
            if constexpr (FP) {
                load_x_slot<FMT, XN>(p, b, slot, slot < p.slots, xr[sp][b], sx[sp][b], xoff);
            } else {
                float raw[XN];
                load_x_raw<XN>(p, b, slot, slot < p.slots, raw, xoff);
                make_xint<FMT, NP, XN>(raw, xi[sp][b]);
            }
        }
    }

    const unsigned seq = ar_begin<AR>(p, ar_word, ctid, CT);
    const int tiles_per_pass = p.P / p.R;
    for (int t0 = 0; t0 < n_tiles; t0 += tiles_per_pass) {
        const int t1 = min(n_tiles, t0 + tiles_per_pass);
        for (int it = t0; it < t1; ++it) {
            const int s = it % p.S;
            // a warp that gives up raises the CTA's abort word and still goes to the barrier below, where every
            // consumer warp reads the word and leaves together: nobody is left waiting at a barrier for a warp
            // that has gone
            if (!mbar_wait(&full[s], (it / p.S) & 1)) { report_error(ZTQ_ERR_FULL_WAIT); *abort_word = 1; break; }
            const int row0 = r_begin + it * p.R;
            const int rows = min(p.R, r_end - row0);
            const uint8_t* sdata = smem + (size_t)s * p.stage_stride;
            const uint8_t* smeta = sdata + (size_t)p.R * p.row_bytes;

            float acc[V];
#pragma unroll
            for (int v = 0; v < V; ++v) acc[v] = 0.f;
#pragma unroll
            for (int sp = 0; sp < SPT; ++sp) {
                const int slot = tit + sp * G;
                if (slot < p.slots) {
#pragma unroll
                    for (int rr = 0; rr < RT; ++rr) {
                        const int r = team + rr * p.T;
                        if (r < rows) {
                            float o[BC];
                            if constexpr (FP)
                                slot_dot<FMT, BC>(sdata + (size_t)r * p.row_bytes, smeta + (size_t)r * p.meta_row_bytes,
                                                  slot, xr[sp], sx[sp], lut + lane, o, p.gshift);
                            else
                                slot_dot_int<FMT, BC, NP>(sdata + (size_t)r * p.row_bytes,
                                                          smeta + (size_t)r * p.meta_row_bytes, slot, xi[sp], o, p.gshift);
#pragma unroll
                            for (int b = 0; b < BC; ++b) acc[rr * BC + b] += o[b];
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);       // stage may be refilled

            const float tot = warp_sum_v<V>(acc, lane);
            if ((lane & (32 / V - 1)) == 0) {
                const int vi = lane / (32 / V);
                const int rr = vi / BC, b = vi - rr * BC;
                const int lr = (it - t0) * p.R + team + rr * p.T;     // row inside this pass
                part[((size_t)lr * BC + b) * p.WPT + wit] = tot;
            }
        }
        // every row of the pass has its per-warp partial sums in shared memory
        bar_sync(1, CT);
        if (*abort_word) break;                         // the same value in every warp: all leave here
        const int prow0 = r_begin + t0 * p.R;
        const int prows = min(r_end, r_begin + t1 * p.R) - prow0;
        finish_pass<BC, FMT == F_TERN, false, AR>(p, part, prow0, prows, ctid, CT, seq, t0 / tiles_per_pass, yoff);
        if (t1 < n_tiles) bar_sync(1, CT);
    }
    ar_end<AR>(p, seq, ctid == 0);
}

// Second pass of split-K: y[n] = sum over splits of partial[split][n], in split order (fixed), then the
// output conversion.  One thread per output.
__global__ void splitk_reduce_kernel(const float* __restrict__ partial, void* __restrict__ y, int N, int splits, int y_f32) {
    grid_dep_launch();
    grid_dep_wait();
    const int n = blockIdx.x * blockDim.x + threadIdx.x;
    if (n >= N) return;
    float s = 0.f;
    for (int i = 0; i < splits; ++i) s += partial[(size_t)i * N + n];
    if (y_f32) reinterpret_cast<float*>(y)[n] = s;
    else reinterpret_cast<__half*>(y)[n] = __float2half_rn(s);
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
                    const __half2 sz = *reinterpret_cast<const __half2*>(mrow + (slot >> p.gshift) * 4);
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
