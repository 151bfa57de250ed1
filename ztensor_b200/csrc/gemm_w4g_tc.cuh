// gemm_w4g_tc.cuh -- W4A16 skinny GEMM on the 5th-generation tensor cores (tcgen05 + TMEM), sm_100a.
//
//   y[b, n] = sum_k (q[n,k] - z[n,g]) * s[n,g] * x[b,k]       16 <= padded batch <= 32, group g = k / 128
//
// The weights are the M operand (tiles of 128 rows), the activations the N operand (batch padded to 16 or
// 32).  For every group of 128 k the integer codes q (0..15, exact in fp16) and the fp16 activations are
// multiplied on the tensor cores into a TMEM accumulator of their own (fp32, fresh per group), because scale
// and zero point change with the group:
//   y[b, n] += s[n,g] * (D_g[n,b] - z[n,g] * sum_{k in g} x[b,k]).
// A tiles and accumulators are rings of four in tensor memory, activation blocks a ring of eight in shared
// memory, so decode, MMA and epilogue of neighbouring groups overlap.
// Nothing is rounded before the tensor core sees it (codes and fp16 activations are exact operands; products
// of a 4-bit and an 11-bit significand are exact in the fp32 accumulator).
//
// Roles inside a CTA of 27 warps (one CTA per SM, persistent over row tiles).  Every role is a chain of
// dependent instructions per step, so what bounds a step is the longest chain, not the instruction count:
//   warps 0-7    epilogue: tcgen05.ld of two groups' accumulators (lane = row, half of the columns per warp),
//                scale / zero, running sums
//   warps 8-23   decode, two sets of eight warps on alternating groups: nibbles (staged by TMA) -> fp16 codes ->
//                A operand written straight into TENSOR MEMORY (tcgen05.st, lane = row, one 32-bit column = two
//                k), so the expanded weights never cross shared memory: an fp16 A tile is 4x the packed bytes
//                and a shared-memory round trip of it costs more bandwidth than the SM has at HBM speed
//   warp 24      weight producer: 2-D tiled copies (cp.async.bulk.tensor.2d, no multicast) of 128 rows x 128
//                bytes (two groups) with the 128-byte swizzle, so that the decode warps read them conflict-free
//   warp 25      MMA issuer: one elected thread, 4 x tcgen05.mma kind::i8 (M=128, N=48|96, K=32) or 8 x kind::f16
//                (N=16|32, K=16) per group, one tcgen05.commit
//   warp 26      activation producer: one bulk copy of a prepared block per group
// The activations are prepared once per call by tc_prepare_x_kernel: per group of 128 k one block of the
// workspace holds the B tile in the UMMA canonical K-major layout without swizzle (core matrices of 8 rows x 16
// bytes, k permuted like the codes) followed by sum_k x[b, k] of the group; the producer fetches a block with one
// bulk copy per group, so no warp of the main kernel touches x.
// The eight k of one 32-bit word of nibbles are decoded in the order (k0,k4,k1,k5,k2,k6,k3,k7); the B tile
// permutes the activations the same way, which leaves every dot product unchanged.
// Every wait is bounded; on a give-up the kernel records an error, releases its TMEM columns and returns.
#pragma once

#include <cuda.h>

#include "gemv_stream.cuh"

namespace ztq {

struct TcParams {
    const uint32_t* meta;     // half2 {scale, zero} per (row, group), row-major [N][K/128]
    const uint8_t* xprep;     // workspace: per group {B tile, sums} as written by tc_prepare_x_kernel
    void* y;                  // [batch][N] fp16 or fp32
    int y_f32;
    int N, K, batch;
    int nmma;                 // 16 or 32: batch padded to the MMA N extent
    int G;                    // K / 128
    // K split: a row tile's K range is cut into S slices of Gs = G / S groups, one work item each, so that
    // matrices with few row tiles still fill the SMs.  Every slice writes fp32 partial sums; the epilogue warp
    // that arrives last at the tile's counter adds the slices in slice order (fixed) and stores y.
    int S, Gs;
    float* partial;           // [S][nmma][N] (S > 1)
    unsigned* counters;       // [row tiles][8 epilogue warps], zero between launches
    // Row-parallel shard (ar.world >= 2, AR instantiations only): the warp that holds a tile's final sums pushes them
    // as {value, tag} cells to every rank (the protocol of finish_pass in gemv_stream.cuh: same slots, same launch
    // sequence word, so GEMV and tensor-core launches of one rank can alternate) and goes on with its next item; the
    // cells of all ranks are collected, added in rank order and stored after the CTA's last item.
    ArParams ar;
};

constexpr int kTcStages = 6;                       // raw nibble stages (two groups each)
constexpr int kTcDone = 16;                        // ring of MMA-completion barriers (>= every consumer's lag)
constexpr int kTcTailSlots = 4, kTcTailGroups = 8; // ring of per-column float blocks, eight groups per slot
constexpr int kTcBuf = 4;                          // depth of the A-tile and accumulator rings (TMEM), one scale per group
// Formats with a scale per 32 weights (Q4_0): each of a group's four MMAs (K = 32 = one block) gets an accumulator of
// its own, so a ring slot holds four times the accumulator columns and the rings are two deep.
__host__ __device__ constexpr int tc_bufs(int gb) { return gb == 4 ? 2 : 4; }
// depth of the ring of B tiles in shared memory (a power of two <= kTcDone): about 96 KB
__host__ __device__ constexpr int tc_bring(int tile_bytes) { return tile_bytes > 6144 ? 8 : 16; }
constexpr int kTcRawBytes = 128 * 128;             // two groups of one tile: 128 rows x 128 bytes (128-byte swizzle)
// Q8_0 (W8): the raw stage holds the 36-byte blocks themselves, 128 rows x 144 bytes per group, two groups per stage;
// three stages (108 KB), a B ring of eight tiles, and a ring of the blocks' float scales for the epilogue
constexpr int kTcStagesW8 = 3, kTcRawBytesW8 = 2 * 128 * 144, kTcBRingW8 = 8;
constexpr int kTcScaleRing = 4;                    // groups whose scales are kept: twice the accumulator ring
constexpr int kTcScaleBytes = kTcScaleRing * 128 * 16;
__host__ __device__ constexpr int tc_stages(bool w8) { return w8 ? kTcStagesW8 : kTcStages; }
__host__ __device__ constexpr int tc_raw_bytes(bool w8) { return w8 ? kTcRawBytesW8 : kTcRawBytes; }
constexpr int kTcRawWarp = 24, kTcMmaWarp = 25, kTcBWarp = 26;
constexpr int kTcThreads = 27 * 32;
constexpr int kTcArPend = 48;                      // tiles an epilogue warp may leave waiting for their peers' cells
constexpr int kTcArSmem = 8 * kTcArPend * 2 + 16;  // the lists of those tiles, after the barriers

// ---- tcgen05 / TMA wrappers -------------------------------------------------
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
            smem_u32(dst)),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
    return pred != 0;
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void proxy_fence_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// A operand in tensor memory (lane = row, column = two consecutive k), B from shared memory.
__device__ __forceinline__ void tc_mma_f16_ta(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
        "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Same for 8-bit integers: A unsigned (the codes), B signed (activation digits), int32 accumulator, K = 32.
__device__ __forceinline__ void tc_mma_i8_ta(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
        "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// sixteen consecutive 32-bit columns of this thread's lane
__device__ __forceinline__ void tc_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
// Shared-memory matrix descriptor, K-major, no swizzle: core matrices of 8 rows x 16 bytes stored as 128
// contiguous bytes; lbo = bytes between core matrices adjacent along K, sbo = along M/N.
__device__ __forceinline__ uint64_t tc_smem_desc(const void* ptr, uint32_t lbo, uint32_t sbo) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_u32(ptr) & 0x3FFFFu) >> 4);
    d |= (uint64_t)((lbo >> 4) & 0x3FFFu) << 16;
    d |= (uint64_t)((sbo >> 4) & 0x3FFFu) << 32;
    d |= (uint64_t)1 << 46;                          // descriptor version of sm_100
    return d;                                        // base offset 0, swizzle mode 0 (none)
}
// Instruction descriptor of kind::f16: fp32 accumulator, fp16 A and B, both K-major, M=128, N=n.
__device__ __forceinline__ uint32_t tc_idesc_f16(int n) {
    return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}
// Instruction descriptor of kind::i8: int32 accumulator, unsigned 8-bit A, signed 8-bit B, both K-major, M=128, N=n.
__device__ __forceinline__ uint32_t tc_idesc_i8(int n) {
    return (2u << 4) | (0u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}
// eight consecutive 32-bit columns of this thread's lane; the caller waits (tc_wait_ld) before using them
__device__ __forceinline__ void tc_ld8_nowait(uint32_t taddr, int (&r)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr));
}
__device__ __forceinline__ void tc_ld4_nowait(uint32_t taddr, int (&r)[4]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(taddr));
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void tc_ld_row(uint32_t taddr, float (&v)[N]);
template <>
__device__ __forceinline__ void tc_ld_row<16>(uint32_t taddr, float (&v)[16]) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
template <>
__device__ __forceinline__ void tc_ld_row<32>(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// Eight nibbles of a word -> eight fp16 integers in the order (k0,k4,k1,k5,k2,k6,k3,k7).
__device__ __forceinline__ uint4 decode_word_f16(uint32_t w) {
    const __half2 bias_lo = __halves2half2(__ushort_as_half(0xE400), __ushort_as_half(0xE400));   // -1024
    const __half2 sixteenth = __halves2half2(__ushort_as_half(0x2C00), __ushort_as_half(0x2C00)); // 1/16
    const __half2 bias_hi = __halves2half2(__ushort_as_half(0xD400), __ushort_as_half(0xD400));   // -64
    const uint32_t h = w >> 8;
    uint32_t a = (w & 0x000f000fu) | 0x64006400u;     // 1024 + (k0, k4)
    uint32_t b = (w & 0x00f000f0u) | 0x64006400u;     // 1024 + 16 (k1, k5)
    uint32_t c = (h & 0x000f000fu) | 0x64006400u;     // 1024 + (k2, k6)
    uint32_t d = (h & 0x00f000f0u) | 0x64006400u;     // 1024 + 16 (k3, k7)
    __half2 ha = __hadd2(*reinterpret_cast<__half2*>(&a), bias_lo);
    __half2 hb = __hfma2(*reinterpret_cast<__half2*>(&b), sixteenth, bias_hi);
    __half2 hc = __hadd2(*reinterpret_cast<__half2*>(&c), bias_lo);
    __half2 hd = __hfma2(*reinterpret_cast<__half2*>(&d), sixteenth, bias_hi);
    uint4 o;
    o.x = *reinterpret_cast<uint32_t*>(&ha);
    o.y = *reinterpret_cast<uint32_t*>(&hb);
    o.z = *reinterpret_cast<uint32_t*>(&hc);
    o.w = *reinterpret_cast<uint32_t*>(&hd);
    return o;
}

// Workspace: G B tiles, then G blocks of per-column floats (fp16 operands: sum_k x; integer operands: {c, sum_k X}).
// N extent of an integer MMA: three digit planes of nb columns, rounded up to the multiple of 16 that M = 128 wants
__host__ __device__ constexpr int tc_nmma_i8(int nb) { return (3 * nb + 15) & ~15; }
__host__ __device__ constexpr int tc_tile_bytes(int nb, bool i8) { return i8 ? tc_nmma_i8(nb) * 128 : nb * 256; }
__host__ __device__ constexpr int tc_tail_bytes(int nb, bool i8, int gb = 1) { return gb == 4 ? nb * 32 : i8 ? nb * 8 : nb * 4; }

// Integer variant of the preparation.  Per (column b, group g) the 128 activations become 21-bit fixed point
//   X[k] = rint(x[k] * 2^(19-e)),  2^e <= max|x| < 2^(e+1)        (|X| < 2^20; exact for all but elements below 2^-19 max)
// split into balanced base-256 digits X = p0 + 256 p1 + 65536 p2, each an int8.  The B tile has 3 nb rows
// (row = plane * nb + b) of 128 bytes in the order the decode warps emit the codes: per word of eight nibbles
// (k0,k2,k4,k6,k1,k3,k5,k7).  Behind the tile: per column {c = 2^(e-19), float(sum_k X[k])}.
// One block per group, eight threads per column (16 k each).
__global__ void tc_prepare_x_i8_kernel(const __half* __restrict__ x, uint8_t* __restrict__ ws, int K, int batch, int nb,
                                       unsigned* counters, int n_counters) {
    grid_dep_launch();
    grid_dep_wait();
    const int g = blockIdx.x;
    if (g == 0) for (int i = threadIdx.x; i < n_counters; i += blockDim.x) counters[i] = 0;
    uint8_t* blk = ws + (size_t)g * tc_tile_bytes(nb, true);
    float2* tail = reinterpret_cast<float2*>(ws + (size_t)gridDim.x * tc_tile_bytes(nb, true) + (size_t)g * tc_tail_bytes(nb, true));
    const int b = threadIdx.x >> 3, ki = threadIdx.x & 7;         // blockDim.x == 8 nb
    float v[16];
    if (b < batch) {
        const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)b * K + (size_t)g * 128 + ki * 16);
        const uint4 q0 = src[0], q1 = src[1];
        const uint32_t w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
            v[2 * i] = f.x; v[2 * i + 1] = f.y;
        }
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = 0.f;
    }
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const int e = amax > 0.f ? (int)(__float_as_uint(amax) >> 23) - 127 : 19;
    const float scale = __uint_as_float((uint32_t)(19 - e + 127) << 23);
    int X[16], sum = 0;
#pragma unroll
    for (int i = 0; i < 16; ++i) { X[i] = __float2int_rn(v[i] * scale); sum += X[i]; }
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    // digits; byte j of the 16-byte row <- element perm[j] of this thread's sixteen
    uint32_t pl[3][4];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        const int wd = j >> 3, pos = j & 7;
        const int src = wd * 8 + (pos < 4 ? 2 * pos : 2 * (pos - 4) + 1);
        const int X0 = X[src];
        const int p0 = (int)(int8_t)(X0 & 0xff);
        const int X1 = (X0 - p0) >> 8;
        const int p1 = (int)(int8_t)(X1 & 0xff);
        const int p2 = (X1 - p1) >> 8;
        const int sh = (j & 3) * 8;
        if ((j & 3) == 0) pl[0][j >> 2] = pl[1][j >> 2] = pl[2][j >> 2] = 0;
        pl[0][j >> 2] |= (uint32_t)(p0 & 0xff) << sh;
        pl[1][j >> 2] |= (uint32_t)(p1 & 0xff) << sh;
        pl[2][j >> 2] |= (uint32_t)(p2 & 0xff) << sh;
    }
    const int n8 = tc_nmma_i8(nb) / 8;                        // rows beyond 3 nb (nb = 8) stay unwritten: their columns are never read
#pragma unroll
    for (int pn = 0; pn < 3; ++pn) {
        const int n = pn * nb + b;
        *reinterpret_cast<uint4*>(blk + (size_t)(ki * n8 + (n >> 3)) * 128 + (n & 7) * 16) =
            make_uint4(pl[pn][0], pl[pn][1], pl[pn][2], pl[pn][3]);
    }
    if (ki == 0) {
        const float c = b < batch ? __uint_as_float((uint32_t)(e - 19 + 127) << 23) : 0.f;
        tail[b] = make_float2(c, (float)sum);
    }
}


// The same for Q4_0 weights (blocks of 32 with their own scale; byte j of a block = elements j and j + 16).  The
// four MMAs of a group are the four blocks; the decode warps emit a block's codes as (e0-3, e16-19, e4-7, e20-23 |
// e8-11, e24-27, e12-15, e28-31), and the B tile lists the activations in that order: 16-byte chunk 2j of a row
// holds elements {0-3, 16-19, 4-7, 20-23} of block j, chunk 2j+1 elements {8-11, 24-27, 12-15, 28-31}.  Behind the
// tile, per column: {c = 2^(e-19), float(sum X) of block 0, 1, 2, 3, 0, 0, 0} -- the -8 offset of the codes needs
// the sums block by block.  One exponent per (column, group of 128), as above.
__global__ void tc_prepare_x_i8_q4_0_kernel(const __half* __restrict__ x, uint8_t* __restrict__ ws, int K, int batch, int nb,
                                            unsigned* counters, int n_counters) {
    grid_dep_launch();
    grid_dep_wait();
    const int g = blockIdx.x;
    if (g == 0) for (int i = threadIdx.x; i < n_counters; i += blockDim.x) counters[i] = 0;
    uint8_t* blk = ws + (size_t)g * tc_tile_bytes(nb, true);
    float* tail = reinterpret_cast<float*>(ws + (size_t)gridDim.x * tc_tile_bytes(nb, true) + (size_t)g * tc_tail_bytes(nb, true, 4));
    const int b = threadIdx.x >> 3, ki = threadIdx.x & 7;         // blockDim.x == 8 nb; ki: 16-byte chunk of the row
    const int j = ki >> 1, half = ki & 1;                         // block of the group, which eight of its first / last sixteen
    float v[16];
    if (b < batch) {
        const __half* src = x + (size_t)b * K + (size_t)g * 128 + j * 32 + half * 8;
        const uint4 q0 = *reinterpret_cast<const uint4*>(src), q1 = *reinterpret_cast<const uint4*>(src + 16);
        const uint32_t w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
            v[2 * i] = f.x; v[2 * i + 1] = f.y;                   // v[0..7] = elements 8 half + 0..7, v[8..15] = 16 + 8 half + 0..7
        }
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = 0.f;
    }
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const int e = amax > 0.f ? (int)(__float_as_uint(amax) >> 23) - 127 : 19;
    const float scale = __uint_as_float((uint32_t)(19 - e + 127) << 23);
    int X[16], sum = 0;
#pragma unroll
    for (int i = 0; i < 16; ++i) { X[i] = __float2int_rn(v[i] * scale); sum += X[i]; }
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);                  // both halves of the block
    // byte t of the chunk <- element perm[t]: (v0-3, v8-11, v4-7, v12-15)
    uint32_t pl[3][4];
#pragma unroll
    for (int t = 0; t < 16; ++t) {
        const int src = (t & 3) + ((t >> 2) & 1) * 8 + (t >> 3) * 4;
        const int X0 = X[src];
        const int p0 = (int)(int8_t)(X0 & 0xff);
        const int X1 = (X0 - p0) >> 8;
        const int p1 = (int)(int8_t)(X1 & 0xff);
        const int p2 = (X1 - p1) >> 8;
        const int sh = (t & 3) * 8;
        if ((t & 3) == 0) pl[0][t >> 2] = pl[1][t >> 2] = pl[2][t >> 2] = 0;
        pl[0][t >> 2] |= (uint32_t)(p0 & 0xff) << sh;
        pl[1][t >> 2] |= (uint32_t)(p1 & 0xff) << sh;
        pl[2][t >> 2] |= (uint32_t)(p2 & 0xff) << sh;
    }
    const int n8 = tc_nmma_i8(nb) / 8;
#pragma unroll
    for (int pn = 0; pn < 3; ++pn) {
        const int n = pn * nb + b;
        *reinterpret_cast<uint4*>(blk + (size_t)(ki * n8 + (n >> 3)) * 128 + (n & 7) * 16) =
            make_uint4(pl[pn][0], pl[pn][1], pl[pn][2], pl[pn][3]);
    }
    float* tb = tail + b * 8;
    if (ki == 0) {
        tb[0] = b < batch ? __uint_as_float((uint32_t)(e - 19 + 127) << 23) : 0.f;
        tb[5] = tb[6] = tb[7] = 0.f;
    }
    if (half == 0) tb[1 + j] = (float)sum;
}

// The same for Q8_0 weights (blocks of 32 int8 in natural order, no zero point).  The codes reach +-127, so the fixed
// point is two bits shorter, |X| < 2^18 (exact for elements within 2^-7 of the group's largest, 2^-19 of it otherwise):
// a block's sum of 32 products then stays below 2^31.  Chunk ki of a B-tile row = elements 16 ki .. 16 ki + 15 of the
// group.  Behind the tile, per column: {c = 2^(e-17), 0, ...} in the 32-byte records of the Q4_0 variant.
__global__ void tc_prepare_x_i8_q8_0_kernel(const __half* __restrict__ x, uint8_t* __restrict__ ws, int K, int batch, int nb,
                                            unsigned* counters, int n_counters) {
    grid_dep_launch();
    grid_dep_wait();
    const int g = blockIdx.x;
    if (g == 0) for (int i = threadIdx.x; i < n_counters; i += blockDim.x) counters[i] = 0;
    uint8_t* blk = ws + (size_t)g * tc_tile_bytes(nb, true);
    float* tail = reinterpret_cast<float*>(ws + (size_t)gridDim.x * tc_tile_bytes(nb, true) + (size_t)g * tc_tail_bytes(nb, true, 4));
    const int b = threadIdx.x >> 3, ki = threadIdx.x & 7;         // blockDim.x == 8 nb
    float v[16];
    if (b < batch) {
        const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)b * K + (size_t)g * 128 + ki * 16);
        const uint4 q0 = src[0], q1 = src[1];
        const uint32_t w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
            v[2 * i] = f.x; v[2 * i + 1] = f.y;
        }
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = 0.f;
    }
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const int e = amax > 0.f ? (int)(__float_as_uint(amax) >> 23) - 127 : 17;
    const float scale = __uint_as_float((uint32_t)(17 - e + 127) << 23);
    uint32_t pl[3][4];
#pragma unroll
    for (int t = 0; t < 16; ++t) {
        const int X0 = __float2int_rn(v[t] * scale);
        const int p0 = (int)(int8_t)(X0 & 0xff);
        const int X1 = (X0 - p0) >> 8;
        const int p1 = (int)(int8_t)(X1 & 0xff);
        const int p2 = (X1 - p1) >> 8;
        const int sh = (t & 3) * 8;
        if ((t & 3) == 0) pl[0][t >> 2] = pl[1][t >> 2] = pl[2][t >> 2] = 0;
        pl[0][t >> 2] |= (uint32_t)(p0 & 0xff) << sh;
        pl[1][t >> 2] |= (uint32_t)(p1 & 0xff) << sh;
        pl[2][t >> 2] |= (uint32_t)(p2 & 0xff) << sh;
    }
    const int n8 = tc_nmma_i8(nb) / 8;
#pragma unroll
    for (int pn = 0; pn < 3; ++pn) {
        const int n = pn * nb + b;
        *reinterpret_cast<uint4*>(blk + (size_t)(ki * n8 + (n >> 3)) * 128 + (n & 7) * 16) =
            make_uint4(pl[pn][0], pl[pn][1], pl[pn][2], pl[pn][3]);
    }
    tail[b * 8 + ki] = (ki == 0 && b < batch) ? __uint_as_float((uint32_t)(e - 17 + 127) << 23) : 0.f;
}

// One block per group of 128 k: x[b, g*128 .. +127] -> B tile (core matrix (ki, b/8) at (ki * nmma/8 + b/8) * 128,
// row b%8 at 16 bytes, the eight k of a row in the order (k0,k4,k1,k5,k2,k6,k3,k7)) and the group's sums.
__global__ void tc_prepare_x_kernel(const __half* __restrict__ x, uint8_t* __restrict__ ws, int K, int batch, int nmma,
                                    unsigned* counters, int n_counters) {
    grid_dep_launch();
    grid_dep_wait();
    const int g = blockIdx.x;
    if (g == 0) for (int i = threadIdx.x; i < n_counters; i += blockDim.x) counters[i] = 0;
    uint8_t* blk = ws + (size_t)g * tc_tile_bytes(nmma, false);
    float* tail = reinterpret_cast<float*>(ws + (size_t)gridDim.x * tc_tile_bytes(nmma, false) + (size_t)g * tc_tail_bytes(nmma, false));
    for (int item = threadIdx.x; item < nmma * 16; item += blockDim.x) {
        const int ki = item % 16, b = item / 16;                  // consecutive threads: consecutive 16-byte pieces of a row
        uint4 q = make_uint4(0, 0, 0, 0);
        if (b < batch) q = *reinterpret_cast<const uint4*>(x + (size_t)b * K + (size_t)g * 128 + ki * 8);
        uint4 o;
        o.x = __byte_perm(q.x, q.z, 0x5410);
        o.y = __byte_perm(q.x, q.z, 0x7632);
        o.z = __byte_perm(q.y, q.w, 0x5410);
        o.w = __byte_perm(q.y, q.w, 0x7632);
        *reinterpret_cast<uint4*>(blk + (size_t)(ki * (nmma / 8) + (b >> 3)) * 128 + (b & 7) * 16) = o;
    }
    for (int b = threadIdx.x; b < nmma; b += blockDim.x) {        // sums in k order: fixed
        float s = 0.f;
        if (b < batch) {
            const __half* src = x + (size_t)b * K + (size_t)g * 128;
            for (int k = 0; k < 128; ++k) s += __half2float(src[k]);
        }
        tail[b] = s;
    }
}

// All-reduce, second half: wait (bounded) until every rank's cells of output row `rw`, columns col0 .. col0 + CW - 1,
// carry this launch's tag, add them in rank order, store.  Not inlined: it runs once per tile after the CTA's
// last item and must not cost the epilogue loop registers.
template <int CW>
__device__ __noinline__ void tc_ar_collect(const TcParams& p, int rw, int col0, unsigned seq) {
    if (rw >= p.N) return;
    const unsigned tag = seq + 1u;
    const uint2* mine = p.ar.slots[p.ar.rank] + (size_t)(seq & 1u) * p.ar.world * p.ar.slot_stride;
    const int world = p.ar.world, stride = p.ar.slot_stride;
    bool ok = true;
    // two columns per round: their sixteen cells are in flight together (a round is a trip to L2)
    for (int b = 0; b < CW && col0 + b < p.batch && ok; b += 2) {
        const bool two = col0 + b + 1 < p.batch;
        const size_t yi = (size_t)(col0 + b) * p.N + rw;
        const uint2* src0 = mine + yi;
        const uint2* src1 = two ? src0 + p.N : src0;
        uint2 v0[kMaxRanks], v1[kMaxRanks];
#pragma unroll
        for (int r = 0; r < kMaxRanks; ++r)
            if (r < world) { v0[r] = ld_cell_sys(src0 + (size_t)r * stride); v1[r] = ld_cell_sys(src1 + (size_t)r * stride); }
        for (uint32_t n = 0;; ++n) {                                        // missing cells are fetched again together
            bool all = true;
#pragma unroll
            for (int r = 0; r < kMaxRanks; ++r)
                if (r < world && (v0[r].y != tag || v1[r].y != tag)) all = false;
            if (all) break;
            if (n >= (1u << 21)) { ok = false; break; }                     // about a second: give up, flag, return
            __nanosleep(20);
#pragma unroll
            for (int r = 0; r < kMaxRanks; ++r) {
                if (r < world && v0[r].y != tag) v0[r] = ld_cell_sys(src0 + (size_t)r * stride);
                if (r < world && v1[r].y != tag) v1[r] = ld_cell_sys(src1 + (size_t)r * stride);
            }
        }
        float t0 = 0.f, t1 = 0.f;
#pragma unroll
        for (int r = 0; r < kMaxRanks; ++r)
            if (r < world) { t0 += __uint_as_float(v0[r].x); t1 += __uint_as_float(v1[r].x); }   // rank order: fixed
        if (ok) {
            if (p.y_f32) {
                reinterpret_cast<float*>(p.y)[yi] = t0;
                if (two) reinterpret_cast<float*>(p.y)[yi + p.N] = t1;
            } else {
                reinterpret_cast<__half*>(p.y)[yi] = __float2half_rn(t0);
                if (two) reinterpret_cast<__half*>(p.y)[yi + p.N] = __float2half_rn(t1);
            }
        }
    }
    if (!ok) report_error(ZTQ_ERR_FLAG_WAIT);
}
// NB: batch columns (8, 16 or 32; 8 only with integer operands).  I8: integer operands (codes x activation digits, exact int32 sums) instead of
// fp16 operands.  An MMA of 128 rows costs the tensor pipe about the same whatever its N, so what counts is k per
// MMA: 32 for 8-bit operands, 16 for fp16.
// SPLIT: the K range of a row tile is cut into p.S > 1 slices (separate instantiation: the unsplit kernel keeps
// its registers).
// GB: scale blocks per group of 128 k: 1 = GPTQ / AWQ group 128 (p.meta: half2 {scale, zero} per group), 4 = Q4_0
// (p.meta: fp16 scale per block of 32, zero point 8; integer operands, NB <= 16).
// AR: the all-reduce over the ranks of a row-parallel shard in the epilogue (p.ar).
// W8: Q8_0 weights (GB == 4): the stages hold raw 36-byte blocks {float scale, 32 int8}; "decoding" is picking the
// code words out of a row's bytes (signed A operand), the scales go to the epilogue through a ring in shared memory,
// there is no zero point.
template <int NB, bool I8, bool SPLIT, int GB = 1, bool AR = false, bool W8 = false>
__global__ void __launch_bounds__(kTcThreads, 1) gemm_w4g_tc_kernel(const __grid_constant__ CUtensorMap wmap, const __grid_constant__ TcParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int NMMA = I8 ? tc_nmma_i8(NB) : NB;                // N extent of an MMA = accumulator columns of a group
    constexpr int ACOLS = I8 ? 32 : 64;                           // TMEM columns of an A tile (128 k)
    constexpr int NSTEP = I8 ? 4 : 8;                             // MMAs per group
    constexpr int B_BYTES = tc_tile_bytes(NB, I8);                // B tile of one group
    constexpr int B_STRIDE = B_BYTES;
    constexpr int T_BYTES = tc_tail_bytes(NB, I8, GB);            // per-column floats of one group
    constexpr int kTcBRing = W8 ? kTcBRingW8 : tc_bring(B_BYTES);
    constexpr int kTcStages = tc_stages(W8);                      // (shadow the file-scope constants: per format)
    constexpr int kTcRawBytes = tc_raw_bytes(W8);
    static_assert(!W8 || (GB == 4 && I8 && !AR), "Q8_0: a scale per block, integer operands");
    constexpr int KB = tc_bufs(GB);                               // depth of the A-tile and accumulator rings
    constexpr int DCOLS = GB * NMMA;                              // accumulator columns of one ring slot
    constexpr int TMEM_COLS = 512;                                // accumulators: KB x DCOLS, A tiles: KB x ACOLS
    static_assert(GB == 1 || (GB == 4 && I8 && NB <= 16), "a scale per 32 weights: integer operands, at most 16 columns");
    static_assert(KB * (DCOLS + ACOLS) <= TMEM_COLS, "TMEM budget");
    static_assert(kTcBRing <= kTcDone && B_BYTES % 128 == 0, "ring depth");
    constexpr int A_COL0 = KB * DCOLS;                            // first column of the A ring
    uint8_t* raw = smem;                                          // [stages][128 rows][128 B], 128-byte swizzle
    uint8_t* bbuf = raw + kTcStages * kTcRawBytes;                // [kTcBRing] B tiles
    uint8_t* tbuf = bbuf + kTcBRing * B_STRIDE;                   // [kTcTailSlots][kTcTailGroups] per-column floats
    float4* sring = reinterpret_cast<float4*>(tbuf + kTcTailSlots * kTcTailGroups * T_BYTES);   // [kTcScaleRing][128 rows] (W8)
    uint64_t* bars = reinterpret_cast<uint64_t*>(tbuf + kTcTailSlots * kTcTailGroups * T_BYTES + (W8 ? kTcScaleBytes : 0));
    uint64_t* raw_full = bars;                 // [kTcStages]    TMA bytes landed
    uint64_t* raw_empty = raw_full + kTcStages; //               16 decode warps done with the stage
    uint64_t* b_full = raw_empty + kTcStages;  // [kTcBRing]     bulk copy landed
    uint64_t* t_full = b_full + kTcBRing;      // [kTcTailSlots] bulk copy landed
    uint64_t* t_free = t_full + kTcTailSlots;  //                8 epilogue warps are done with the slot
    uint64_t* a_full = t_free + kTcTailSlots;  // [kTcBuf]       8 decode warps have stored the A tile
    uint64_t* d_empty = a_full + kTcBuf;       //                8 epilogue warps have read the accumulator
    uint64_t* mma_done = d_empty + kTcBuf;     // [kTcDone]      tcgen05.commit of step it on [it % kTcDone]: its A tile and
                                               //                B tile are free again, its accumulator is complete
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(mma_done + kTcDone);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);
    unsigned* ar_seq = tmem_holder + 2;                                        // this launch's sequence number (AR)
    uint16_t* ar_pend = reinterpret_cast<uint16_t*>(tmem_holder + 4);          // [8 warps][kTcArPend] tiles pushed, not yet collected

    // warp index through a shuffle: the compiler then knows it is the same in every lane, keeps the role loops'
    // addresses, descriptors and counters in uniform registers and feeds tcgen05 instructions from there
    const int tid = threadIdx.x, warp = __shfl_sync(0xffffffffu, tid >> 5, 0), lane = tid & 31;
    if (tid == 0) {
        for (int s = 0; s < kTcStages; ++s) { mbar_init(&raw_full[s], 1); mbar_init(&raw_empty[s], 16); }
        for (int i = 0; i < kTcBRing; ++i) mbar_init(&b_full[i], 1);
        for (int i = 0; i < kTcTailSlots; ++i) { mbar_init(&t_full[i], 1); mbar_init(&t_free[i], 8); }
        for (int i = 0; i < kTcBuf; ++i) { mbar_init(&a_full[i], 8); mbar_init(&d_empty[i], 8); }
        for (int i = 0; i < kTcDone; ++i) mbar_init(&mma_done[i], 1);
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == kTcMmaWarp) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_holder)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // The grid dependency (the activation-preparation kernel in front of this one, and whatever produced its input) is
    // waited for only by the roles that read or write what depends on it: the activation producer and the epilogue.
    // The weight producer starts at once, so the weights stream in while the preparation kernel still runs.
    grid_dep_launch();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_holder;

    const int S_ = SPLIT ? p.S : 1, Gs_ = SPLIT ? p.Gs : p.G;   // constants of the unsplit instantiation
    // work item w = (row tile w / S, K slice w % S); this CTA takes items blockIdx.x, blockIdx.x + gridDim.x, ...
    const int n_items = ((p.N + 127) / 128) * S_;
    const int my_items = (n_items - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
    const int total = my_items * Gs_;                             // steps of this CTA; even (Gs % 4 == 0)

    if (warp == kTcRawWarp) {
        // ---------------------------------------------------------------- weights: one TMA box (two groups) per stage
        if (lane == 0) {
            int w = blockIdx.x, gp = 0, s = 0, round = 0;          // gp: pair of groups inside the item
            const int pairs = total >> 1, ipairs = Gs_ >> 1;
            int tile = w / S_, gp0 = (w - tile * S_) * ipairs;
            for (int pr = 0; pr < pairs; ++pr) {
                if (round > 0 && !mbar_wait(&raw_empty[s], (round - 1) & 1)) { report_error(ZTQ_ERR_EMPTY_WAIT); *abort_flag = 1; break; }
                mbar_expect_tx(&raw_full[s], kTcRawBytes);
                if (W8) {                                          // one box of 144 bytes x 128 rows per group
                    tma_load_2d(raw + (size_t)s * kTcRawBytes, &wmap, (gp0 + gp) * 288, tile * 128, &raw_full[s]);
                    tma_load_2d(raw + (size_t)s * kTcRawBytes + kTcRawBytes / 2, &wmap, (gp0 + gp) * 288 + 144, tile * 128, &raw_full[s]);
                } else
                tma_load_2d(raw + (size_t)s * kTcRawBytes, &wmap, (gp0 + gp) * 128, tile * 128, &raw_full[s]);
                if (++gp == ipairs) { gp = 0; w += gridDim.x; tile = w / S_; gp0 = (w - tile * S_) * ipairs; }
                if (++s == kTcStages) { s = 0; ++round; }
            }
        }
    } else if (warp == kTcBWarp) {
        // ---------------------------------------------------------------- activations: one prepared block per group
        grid_dep_wait();
        if (lane == 0) {
            const uint8_t* tails = p.xprep + (size_t)p.G * B_BYTES;
            int w = blockIdx.x, l = 0, ts = 0, tround = 0;         // l: group inside the item
            int g = (w % S_) * Gs_;
            for (int it = 0; it < total; ++it) {
                if ((l & (kTcTailGroups - 1)) == 0) {              // the per-column floats of the next eight groups
                    if (tround > 0 && !mbar_wait(&t_free[ts], (tround - 1) & 1)) { report_error(ZTQ_ERR_EMPTY_WAIT); *abort_flag = 1; break; }
                    const int ng = Gs_ - l < kTcTailGroups ? Gs_ - l : kTcTailGroups;
                    mbar_expect_tx(&t_full[ts], (uint32_t)(ng * T_BYTES));
                    bulk_g2s(tbuf + (size_t)ts * kTcTailGroups * T_BYTES, tails + (size_t)g * T_BYTES, (uint32_t)(ng * T_BYTES), &t_full[ts]);
                    if (++ts == kTcTailSlots) { ts = 0; ++tround; }
                }
                const int bb = it & (kTcBRing - 1), j = it - kTcBRing;     // the slot's previous user: step j
                if (j >= 0 && !mbar_wait(&mma_done[j & (kTcDone - 1)], (j / kTcDone) & 1)) { report_error(ZTQ_ERR_EMPTY_WAIT); *abort_flag = 1; break; }
                mbar_expect_tx(&b_full[bb], B_BYTES);
                bulk_g2s(bbuf + (size_t)bb * B_STRIDE, p.xprep + (size_t)g * B_BYTES, B_BYTES, &b_full[bb]);
                ++g;
                if (++l == Gs_) { l = 0; w += gridDim.x; g = (w % S_) * Gs_; }
            }
        }
    } else if (warp == kTcMmaWarp) {
        // ---------------------------------------------------------------- MMA issuer (one thread; descriptors are
        // built once, a step only adds offsets to their low words)
        // all lanes run the loop and the waits; one elected lane issues
        {
            const bool leader = elect_one();
            const uint32_t idesc = I8 ? (tc_idesc_i8(NMMA) | (W8 ? (1u << 7) : 0u)) : tc_idesc_f16(NMMA);   // W8: signed A
            // B tile, K-major without swizzle: LBO (K direction) = (NMMA/8) core matrices, SBO (N direction) = 128 bytes
            const uint32_t desc_lo0 = ((smem_u32(bbuf) & 0x3FFFFu) >> 4) | ((uint32_t)(((NMMA / 8) * 128) >> 4) << 16);
            const uint32_t desc_hi = (128u >> 4) | (1u << 14);     // SBO, descriptor version of sm_100 (bit 46)
            for (int it = 0; it < total; ++it) {
                const int ab = it & (KB - 1), bb = it & (kTcBRing - 1);
                const uint32_t ph = (it / KB) & 1;
                if (!mbar_wait(&a_full[ab], ph) || !mbar_wait(&b_full[bb], (it / kTcBRing) & 1) ||
                    (it >= KB && !mbar_wait(&d_empty[ab], ph ^ 1))) { if (leader) { report_error(ZTQ_ERR_TMEM_WAIT); *abort_flag = 1; } break; }
                tc_fence_after();
                const uint32_t lo = desc_lo0 + (uint32_t)bb * (B_STRIDE >> 4);
                const uint32_t a_t = tmem_base + A_COL0 + (uint32_t)ab * ACOLS;
                const uint32_t d_t = tmem_base + (uint32_t)ab * DCOLS;
                if (leader) {
#pragma unroll
                    for (int j = 0; j < NSTEP; ++j) {              // k-step j: 8 columns of A (16 or 32 k), core columns 2j, 2j+1 of B
                        uint64_t bd;
                        asm("mov.b64 %0, {%1, %2};" : "=l"(bd) : "r"(lo + (uint32_t)j * (2 * (NMMA / 8) * 128 >> 4)), "r"(desc_hi));
                        if (GB == 4) tc_mma_i8_ta(d_t + (uint32_t)j * NMMA, a_t + 8 * j, bd, idesc, 0);   // one block of 32: its own accumulator
                        else if (I8) tc_mma_i8_ta(d_t, a_t + 8 * j, bd, idesc, j > 0);
                        else tc_mma_f16_ta(d_t, a_t + 8 * j, bd, idesc, j > 0);
                    }
                    tc_commit(&mma_done[it & (kTcDone - 1)]);      // fires when the MMAs above are done
                }
                __syncwarp();
            }
        }
    } else if (warp >= 8 && warp < 24) {
        // ---------------------------------------------------------------- decode: two sets of 8 warps -> A tiles in TMEM
        // Set 0 (warps 8-15) takes the even steps, set 1 (warps 16-23) the odd ones: a step's chain of dependent
        // instructions is longer than the step may last, so two steps are always in flight.  Warp w may touch TMEM
        // lanes 32 (w % 4) .. +31: it decodes those rows; within a set the first four warps take the first 64 k of
        // the group (columns 0-31 of the A tile), the last four the other 64 k (columns 32-63).
        const int idx = warp - 8, qtr = warp & 3, kh = (idx >> 2) & 1, set = idx >> 3;
        const int r = qtr * 32 + lane;
        const uint32_t swz = (uint32_t)(r & 7);
        const uint32_t c0 = (uint32_t)(set * 4 + kh * 2);          // first 16-byte chunk of this warp's 64 k within the row
        const uint32_t off0 = ((c0 ^ swz) << 4), off1 = (((c0 + 1) ^ swz) << 4);   // 128-byte swizzle of the TMA
        const uint32_t a_lane = tmem_base + ((uint32_t)(qtr * 32) << 16) + A_COL0 + kh * (ACOLS / 2);
        int s = 0, rph = 0;                                        // raw stage of the pair of groups, its phase
        for (int it = set; it < total; it += 2) {
            const int ab = it & (KB - 1), j = it - KB;             // the A slot's previous user: step j
            if (!mbar_wait(&raw_full[s], rph) ||
                (j >= 0 && !mbar_wait(&mma_done[j & (kTcDone - 1)], (j / kTcDone) & 1))) { report_error(ZTQ_ERR_FULL_WAIT); *abort_flag = 1; break; }
            tc_fence_after();
            const uint32_t a_t = a_lane + (uint32_t)ab * ACOLS;
            if constexpr (W8) {
                // this warp's half of the row: blocks 2 kh, 2 kh + 1 = 72 bytes {scale, 8 code words} x 2, 8-byte aligned
                // four 16-byte loads and one of 8 bytes (rows are 144 bytes apart: 16-byte loads of 8 lanes cover all banks
                // once; 8-byte loads alone would collide two by two)
                const uint8_t* rp = raw + (size_t)s * kTcRawBytes + (size_t)set * (kTcRawBytes / 2) + r * 144 + kh * 72;
                uint32_t wds[18];
                if (kh == 0) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const uint4 v = reinterpret_cast<const uint4*>(rp)[i];
                        wds[4 * i] = v.x; wds[4 * i + 1] = v.y; wds[4 * i + 2] = v.z; wds[4 * i + 3] = v.w;
                    }
                    const uint2 t = *reinterpret_cast<const uint2*>(rp + 64);
                    wds[16] = t.x; wds[17] = t.y;
                } else {
                    const uint2 t = *reinterpret_cast<const uint2*>(rp);
                    wds[0] = t.x; wds[1] = t.y;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const uint4 v = reinterpret_cast<const uint4*>(rp + 8)[i];
                        wds[2 + 4 * i] = v.x; wds[3 + 4 * i] = v.y; wds[4 + 4 * i] = v.z; wds[5 + 4 * i] = v.w;
                    }
                }
                const uint32_t cols[16] = {wds[1], wds[2], wds[3], wds[4], wds[5], wds[6], wds[7], wds[8],
                                           wds[10], wds[11], wds[12], wds[13], wds[14], wds[15], wds[16], wds[17]};
                tc_st16(a_t, cols);
                // the two scales for the epilogue (slot it mod 4: free again once the accumulator slot of step it - 4
                // has been read, which the MMA of step it - 2 waited for)
                float2* sp = reinterpret_cast<float2*>(&sring[(size_t)(it & (kTcScaleRing - 1)) * 128 + r]) + kh;
                *sp = make_float2(__uint_as_float(wds[0]), __uint_as_float(wds[9]));
                __syncwarp();
                if (lane == 0) mbar_arrive(&raw_empty[s]);
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&a_full[ab]);
                if (++s == kTcStages) { s = 0; rph ^= 1; }
                continue;
            }
            const uint8_t* rs = raw + (size_t)s * kTcRawBytes + r * 128;
            const uint4 q0 = *reinterpret_cast<const uint4*>(rs + off0);
            const uint4 q1 = *reinterpret_cast<const uint4*>(rs + off1);
            if (I8) {
                // a word of eight nibbles -> two columns of four uint8 codes: (k0,k2,k4,k6) and (k1,k3,k5,k7)
                const uint32_t w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
                uint32_t cols[16];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    cols[2 * i] = w[i] & 0x0f0f0f0fu;
                    cols[2 * i + 1] = (w[i] >> 4) & 0x0f0f0f0fu;
                }
                tc_st16(a_t, cols);
            } else {
                {
                    const uint4 w0 = decode_word_f16(q0.x), w1 = decode_word_f16(q0.y), w2 = decode_word_f16(q0.z), w3 = decode_word_f16(q0.w);
                    const uint32_t cols[16] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w, w2.x, w2.y, w2.z, w2.w, w3.x, w3.y, w3.z, w3.w};
                    tc_st16(a_t, cols);
                }
                {
                    const uint4 w0 = decode_word_f16(q1.x), w1 = decode_word_f16(q1.y), w2 = decode_word_f16(q1.z), w3 = decode_word_f16(q1.w);
                    const uint32_t cols[16] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w, w2.x, w2.y, w2.z, w2.w, w3.x, w3.y, w3.z, w3.w};
                    tc_st16(a_t + 16, cols);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&raw_empty[s]);             // the nibbles are in registers
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&a_full[ab]);
            if (++s == kTcStages) { s = 0; rph ^= 1; }
        }
    } else if (warp < 8) {
        // ---------------------------------------------------------------- epilogue: lane = row of the tile; warps w
        // and w + 4 share the rows 32 (w % 4) .. +31 and take half of the batch columns each; two groups per turn
        constexpr int CW = NB / 2;                                 // columns of this warp
        grid_dep_wait();                                           // counters, partial sums, y and the all-reduce state
        // the sequence word is only ever written by this rank's own kernels, and the previous one is complete
        const unsigned ar_seq_v = AR ? *reinterpret_cast<volatile unsigned*>(p.ar.state) : 0u;
        if (AR && tid == 0) *ar_seq = ar_seq_v;                    // for the update after the last item
        const int qtr = warp & 3, col0 = (warp >> 2) * CW;
        const int row_in_tile = qtr * 32 + lane;
        float acc[CW];
        uint4 mq[2], nq[2];                                        // {scale, zero} of eight groups: in use, prefetched
        int w = blockIdx.x, l = 0, ts = 0, tph = 0;                // l: group inside the item
        int tile = w / S_, slice = w - tile * S_;
        int g = slice * Gs_;
        int row = tile * 128 + row_in_tile;
        auto load_meta = [&](int rw, int g0, uint4 (&dst)[2]) {
            dst[0] = dst[1] = make_uint4(0, 0, 0, 0);
            if (rw < p.N) {
                const uint4* mp = reinterpret_cast<const uint4*>(p.meta + (size_t)rw * p.G + g0);
                dst[0] = __ldg(mp);
                if (g0 + 4 < p.G) dst[1] = __ldg(mp + 1);
            }
        };
        // a scale per block of 32 (GB == 4): p.meta is the fp16 scale array [N][K / 32]; one 16-byte load brings the
        // eight scales of a turn's two groups, fetched one turn ahead
        auto load_sc = [&](int rw, int g0) -> uint4 {
            if (rw >= p.N) return make_uint4(0, 0, 0, 0);
            return __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(p.meta) + ((size_t)rw * p.G + g0) * 4));
        };
        uint4 sc_next = make_uint4(0, 0, 0, 0);
        if (total > 0) {
            if (GB == 4 && !W8) sc_next = load_sc(row, g);
            else if (GB == 1) load_meta(row, g, nq);
        }
        const uint32_t d_lane = tmem_base + ((uint32_t)(qtr * 32) << 16) + col0;
        auto store_y = [&](int rw, int b, float v) {
            const size_t yi = (size_t)(col0 + b) * p.N + rw;
            if (p.y_f32) reinterpret_cast<float*>(p.y)[yi] = v;
            else reinterpret_cast<__half*>(p.y)[yi] = __float2half_rn(v);
        };
        int n_pend = 0;                                            // all-reduce: tiles pushed, not yet collected
        for (int it = 0; it < total; it += 2) {                    // groups g, g + 1 (total and G are even)
            const int db = it & (KB - 1);
            if (l == 0) {
#pragma unroll
                for (int b = 0; b < CW; ++b) acc[b] = 0.f;
            }
            uint4 sc_cur = sc_next;
            if (GB == 4 && !W8) {
                if (l + 2 < Gs_) sc_next = load_sc(row, g + 2);
                else if (it + 2 < total) {                         // first turn of this CTA's next item
                    const int wn = w + (int)gridDim.x, tn = wn / S_;
                    sc_next = load_sc(tn * 128 + row_in_tile, (wn - tn * S_) * Gs_);
                }
            }
            if (GB == 1 && (l & 7) == 0) {                         // take the prefetched block, fetch the one after
                mq[0] = nq[0]; mq[1] = nq[1];
                if (l + 8 < Gs_) load_meta(row, g + 8, nq);
                else if (it + 8 < total) {                         // first block of this CTA's next item
                    const int wn = w + (int)gridDim.x, tn = wn / S_;
                    load_meta(tn * 128 + row_in_tile, (wn - tn * S_) * Gs_, nq);
                }
            }
            const uint4 mv = ((l >> 2) & 1) ? mq[1] : mq[0];
            const uint32_t m0 = (l & 2) ? mv.z : mv.x, m1 = (l & 2) ? mv.w : mv.y;
            const float s[2] = {h2f((uint16_t)(m0 & 0xffff)), h2f((uint16_t)(m1 & 0xffff))};
            const float nz[2] = {-h2f((uint16_t)(m0 >> 16)), -h2f((uint16_t)(m1 >> 16))};
            // MMAs complete in order: the later group's commit covers both
            if (((l & (kTcTailGroups - 1)) == 0 && !mbar_wait(&t_full[ts], tph)) ||
                !mbar_wait(&mma_done[(it + 1) & (kTcDone - 1)], ((it + 1) / kTcDone) & 1)) {
                report_error(ZTQ_ERR_TMEM_WAIT); *abort_flag = 1; break;
            }
            tc_fence_after();
            const uint8_t* tail0 = tbuf + (size_t)(ts * kTcTailGroups + (l & (kTcTailGroups - 1))) * T_BYTES;
            if constexpr (GB == 4) {
                // Q4_0: block j of group u has its own accumulator (columns j NMMA ..) and its own scale:
                //   y += (s_uj c_b) (S_ujb - 8 sumX_ujb)
                const uint32_t scw[4] = {sc_cur.x, sc_cur.y, sc_cur.z, sc_cur.w};
#pragma unroll
                for (int h = 0; h < CW / 4; ++h) {
#pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        const float* tb = reinterpret_cast<const float*>(tail0 + (size_t)u * T_BYTES) + (col0 + h * 4) * 8;
#pragma unroll
                        for (int jp = 0; jp < 2; ++jp) {           // two blocks per round of tensor-memory loads
                            int d[2][3][4];
#pragma unroll
                            for (int jj = 0; jj < 2; ++jj)
#pragma unroll
                                for (int pn = 0; pn < 3; ++pn)
                                    tc_ld4_nowait(d_lane + (uint32_t)(db + u) * DCOLS + (uint32_t)(2 * jp + jj) * NMMA + pn * NB + h * 4, d[jj][pn]);
                            tc_wait_ld();
                            float sj[2];
                            if constexpr (W8) {
                                const float2 sv = reinterpret_cast<const float2*>(&sring[(size_t)((it + u) & (kTcScaleRing - 1)) * 128 + row_in_tile])[jp];
                                sj[0] = sv.x; sj[1] = sv.y;
                            } else {
                                const uint32_t sw = scw[2 * u + jp];
                                sj[0] = h2f((uint16_t)(sw & 0xffff)); sj[1] = h2f((uint16_t)(sw >> 16));
                            }
#pragma unroll
                            for (int jj = 0; jj < 2; ++jj)
#pragma unroll
                                for (int c = 0; c < 4; ++c) {
                                    const float S = __int2float_rn((d[jj][2][c] * 256 + d[jj][1][c]) * 256 + d[jj][0][c]);
                                    if (W8) acc[h * 4 + c] = fmaf(sj[jj] * tb[c * 8], S, acc[h * 4 + c]);      // symmetric codes: no offset
                                    else acc[h * 4 + c] = fmaf(sj[jj] * tb[c * 8], fmaf(-8.0f, tb[c * 8 + 1 + 2 * jp + jj], S), acc[h * 4 + c]);
                                }
                        }
                    }
                }
            } else {
#pragma unroll
            for (int h = 0; h < CW / 4; ++h) {                     // four columns of both groups at a time
                if (I8) {
                    // per column b: S = sum_k q X = D0 + 256 D1 + 65536 D2 (|S| < 2^31), then
                    //   y += (s c_b) (S - z sum_k X),   c_b the power of two that undoes the fixed-point scale
                    int d[2][3][4];
#pragma unroll
                    for (int u = 0; u < 2; ++u)
#pragma unroll
                        for (int pn = 0; pn < 3; ++pn) tc_ld4_nowait(d_lane + (uint32_t)(db + u) * DCOLS + pn * NB + h * 4, d[u][pn]);
                    tc_wait_ld();
#pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        const float4* cs4 = reinterpret_cast<const float4*>(tail0 + (size_t)u * T_BYTES) + (col0 + h * 4) / 2;
#pragma unroll
                        for (int j2 = 0; j2 < 2; ++j2) {
                            const float4 cs = cs4[j2];             // {c, sumX} of two columns
                            const int ja = 2 * j2, jb = 2 * j2 + 1;
                            const float Sa = __int2float_rn((d[u][2][ja] * 256 + d[u][1][ja]) * 256 + d[u][0][ja]);
                            const float Sb = __int2float_rn((d[u][2][jb] * 256 + d[u][1][jb]) * 256 + d[u][0][jb]);
                            acc[h * 4 + ja] = fmaf(s[u] * cs.x, fmaf(nz[u], cs.y, Sa), acc[h * 4 + ja]);
                            acc[h * 4 + jb] = fmaf(s[u] * cs.z, fmaf(nz[u], cs.w, Sb), acc[h * 4 + jb]);
                        }
                    }
                } else {
                    int d[2][4];
#pragma unroll
                    for (int u = 0; u < 2; ++u) tc_ld4_nowait(d_lane + (uint32_t)(db + u) * DCOLS + h * 4, d[u]);
                    tc_wait_ld();
#pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        const float4 sv = reinterpret_cast<const float4*>(tail0 + (size_t)u * T_BYTES)[(col0 + h * 4) / 4];
                        acc[h * 4 + 0] = fmaf(s[u], fmaf(nz[u], sv.x, __int_as_float(d[u][0])), acc[h * 4 + 0]);
                        acc[h * 4 + 1] = fmaf(s[u], fmaf(nz[u], sv.y, __int_as_float(d[u][1])), acc[h * 4 + 1]);
                        acc[h * 4 + 2] = fmaf(s[u], fmaf(nz[u], sv.z, __int_as_float(d[u][2])), acc[h * 4 + 2]);
                        acc[h * 4 + 3] = fmaf(s[u], fmaf(nz[u], sv.w, __int_as_float(d[u][3])), acc[h * 4 + 3]);
                    }
                }
            }
            }                                                      // GB == 1
            tc_fence_before();
            __syncwarp();
            g += 2;
            l += 2;
            const bool slot_done = (l & (kTcTailGroups - 1)) == 0 || l == Gs_;
            if (lane == 0) {
                mbar_arrive(&d_empty[db]); mbar_arrive(&d_empty[db + 1]);
                if (slot_done) mbar_arrive(&t_free[ts]);
            }
            if (slot_done && ++ts == kTcTailSlots) { ts = 0; tph ^= 1; }
            if (l == Gs_) {                                       // the item is complete
                bool store = true;
                if (SPLIT) {
                    // this slice's partial sums, then the tile's counter: the last of the S slices adds them all
                    if (row < p.N) {
#pragma unroll
                        for (int b = 0; b < CW; ++b) p.partial[((size_t)slice * NB + col0 + b) * p.N + row] = acc[b];
                    }
                    __threadfence();
                    __syncwarp();
                    unsigned seen = 0;
                    if (lane == 0) seen = atomicAdd(&p.counters[tile * 8 + warp], 1u);
                    seen = __shfl_sync(0xffffffffu, seen, 0);
                    store = seen == (unsigned)(S_ - 1);
                    if (store) {
                        __threadfence();
                        if (lane == 0) p.counters[tile * 8 + warp] = 0;          // ready for the next launch
                        if (row < p.N) {
#pragma unroll
                            for (int b = 0; b < CW; ++b) acc[b] = 0.f;
                            for (int sl = 0; sl < S_; ++sl) {                 // slice order: fixed; CW loads in flight
                                float v[CW];
#pragma unroll
                                for (int b = 0; b < CW; ++b) v[b] = __ldcg(&p.partial[((size_t)sl * NB + col0 + b) * p.N + row]);
#pragma unroll
                                for (int b = 0; b < CW; ++b) acc[b] += v[b];
                            }
                        }
                    }
                }
                if (AR && store) {
                    if (row < p.N) {
                        const unsigned seq = ar_seq_v;
                        const size_t base = ((size_t)(seq & 1u) * p.ar.world + p.ar.rank) * p.ar.slot_stride + row;
#pragma unroll
                        for (int b = 0; b < CW; ++b) {
                            if (col0 + b < p.batch) {
                                const size_t mine = base + (size_t)(col0 + b) * p.N;
                                for (int r = 0; r < p.ar.world; ++r) st_cell_sys(p.ar.slots[r] + mine, __float_as_uint(acc[b]), seq + 1u);
                            }
                        }
                    }
                    // collected after the CTA's last item: the peers' cells arrive while it works on the next ones
                    // (the launcher refuses shapes that give a CTA more than kTcArPend items)
                    if (n_pend < kTcArPend) {
                        if (lane == 0) ar_pend[warp * kTcArPend + n_pend] = (uint16_t)tile;
                        ++n_pend;
                    }
                } else if (store && row < p.N) {
#pragma unroll
                    for (int b = 0; b < CW; ++b)
                        if (col0 + b < p.batch) store_y(row, b, acc[b]);
                }
                l = 0;
                w += gridDim.x;
                tile = w / S_;
                slice = w - tile * S_;
                g = slice * Gs_;
                row = tile * 128 + row_in_tile;
            }
        }
        if (AR && !*abort_flag) {
            __syncwarp();
            for (int i = 0; i < n_pend; ++i) tc_ar_collect<CW>(p, (int)ar_pend[warp * kTcArPend + i] * 128 + row_in_tile, col0, ar_seq_v);
        }
    }
    // ---- teardown: everybody meets, then the allocating warp returns the TMEM columns
    tc_fence_before();
    __syncthreads();
    if (warp == kTcMmaWarp) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
    if (AR && tid == 0) {                           // the last CTA to finish advances the sequence for the next launch
        __threadfence();
        const unsigned done = atomicAdd(p.ar.state + 1, 1u) + 1u;
        if (done == gridDim.x) {
            p.ar.state[1] = 0;
            p.ar.state[0] = *ar_seq + 1u;
        }
    }
}

}  // namespace ztq
