// gemm_w4g_tc.cuh -- W4A16 skinny GEMM on the 5th-generation tensor cores (tcgen05 + TMEM), sm_100a.
//
//   y[b, n] = sum_k (q[n,k] - z[n,g]) * s[n,g] * x[b,k]       16 <= padded batch <= 32, group g = k / 128
//
// The weights are the M operand (tiles of 128 rows), the activations the N operand (batch padded to 16 or
// 32).  For every group of 128 k the integer codes q (0..15, exact in fp16) and the fp16 activations are
// multiplied on the tensor cores into a TMEM accumulator of their own (fp32, fresh per group), because scale
// and zero point change with the group:
//   y[b, n] += s[n,g] * (D_g[n,b] - z[n,g] * sum_{k in g} x[b,k]).
// A tiles, B tiles and accumulators are rings of three, so decode, MMA and epilogue of neighbouring groups overlap.
// Nothing is rounded before the tensor core sees it (codes and fp16 activations are exact operands; products
// of a 4-bit and an 11-bit significand are exact in the fp32 accumulator).
//
// Roles inside a CTA of 16 warps (one CTA per SM, persistent over row tiles):
//   warps 0-3    epilogue: tcgen05.ld of the group's accumulator (lane = row), scale / zero, running sums
//   warps 4-11   decode: nibbles (staged by TMA) -> fp16 codes -> A tile in shared memory, UMMA canonical
//                K-major layout without swizzle (core matrices of 8 rows x 16 bytes)
//   warp 12      TMA producer: 2-D tiled copies (cp.async.bulk.tensor.2d, no multicast) of 128 rows x 128 bytes
//                (two groups) with the 128-byte swizzle, so that the decode warps read them conflict-free
//   warp 13      MMA issuer: one thread, 8 x tcgen05.mma (M=128, N=16|32, K=16) per group, tcgen05.commit
//   warps 14-15  activation stager: x[b, group] -> B tile in shared memory (same layout family)
// The eight k of one 32-bit word of nibbles are decoded in the order (k0,k4,k1,k5,k2,k6,k3,k7); the B tile
// permutes the activations the same way, which leaves every dot product unchanged.
// Every wait is bounded; on a give-up the kernel records an error, releases its TMEM columns and returns.
#pragma once

#include <cuda.h>

#include "gemv_stream.cuh"

namespace ztq {

struct TcParams {
    const uint32_t* meta;     // half2 {scale, zero} per (row, group), row-major [N][K/128]
    const __half* x;          // [batch][K] fp16
    void* y;                  // [batch][N] fp16 or fp32
    int y_f32;
    int N, K, batch;
    int nmma;                 // 16 or 32: batch padded to the MMA N extent
    int G;                    // K / 128
};

constexpr int kTcStages = 4;                       // raw nibble stages (two groups each)
constexpr int kTcBuf = 3;                          // depth of the A-tile, B-tile and accumulator rings
constexpr int kTcSxRing = 8;                       // ring of per-group activation sums (> 2 * kTcBuf steps ahead)
constexpr int kTcRawBytes = 128 * 128;             // two groups of one tile: 128 rows x 128 bytes (128-byte swizzle)
constexpr int kTcABytes = 128 * 128 * 2;           // fp16 codes of one group of one tile
constexpr int kTcThreads = 16 * 32;

// ---- tcgen05 / TMA wrappers -------------------------------------------------
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
            smem_u32(dst)),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
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

template <int NMMA>
__global__ void __launch_bounds__(kTcThreads, 1) gemm_w4g_tc_kernel(const __grid_constant__ CUtensorMap wmap, const TcParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int B_BYTES = NMMA * 128 * 2;                       // one group of activations
    constexpr int PARTS = 64 / NMMA;                              // stager threads per batch column
    constexpr int TMEM_COLS = kTcBuf * NMMA <= 32 ? 32 : (kTcBuf * NMMA <= 64 ? 64 : 128);
    uint8_t* raw = smem;                                          // [stages][128 rows][128 B], 128-byte swizzle
    uint8_t* abuf = raw + kTcStages * kTcRawBytes;                // [kTcBuf][A tile]
    uint8_t* bbuf = abuf + kTcBuf * kTcABytes;                    // [kTcBuf][B tile]
    float* sxp = reinterpret_cast<float*>(bbuf + kTcBuf * B_BYTES);   // [kTcSxRing][PARTS][NMMA] partial sums of x
    uint64_t* bars = reinterpret_cast<uint64_t*>(sxp + kTcSxRing * PARTS * NMMA);
    uint64_t* raw_full = bars;                 // [stages]
    uint64_t* raw_empty = raw_full + kTcStages;
    uint64_t* a_full = raw_empty + kTcStages;  // [kTcBuf] each
    uint64_t* a_empty = a_full + kTcBuf;
    uint64_t* b_full = a_empty + kTcBuf;
    uint64_t* b_empty = b_full + kTcBuf;
    uint64_t* d_full = b_empty + kTcBuf;
    uint64_t* d_empty = d_full + kTcBuf;
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(d_empty + kTcBuf);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int s = 0; s < kTcStages; ++s) { mbar_init(&raw_full[s], 1); mbar_init(&raw_empty[s], 8); }
        for (int i = 0; i < kTcBuf; ++i) {
            mbar_init(&a_full[i], 8); mbar_init(&a_empty[i], 1);
            mbar_init(&b_full[i], 2); mbar_init(&b_empty[i], 1);
            mbar_init(&d_full[i], 1); mbar_init(&d_empty[i], 4);
        }
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 13) {                                              // TMEM: two accumulators of NMMA columns
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_holder)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    grid_dep_launch();
    grid_dep_wait();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_holder;

    const int n_tiles = (p.N + 127) / 128;
    const int my_tiles = (n_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
    const int total = my_tiles * p.G;                              // (tile, group) steps of this CTA

    if (warp == 12) {
        // ---------------------------------------------------------------- TMA producer (one stage = two groups)
        if (lane == 0) {
            const int pairs = total / 2;
            for (int it = 0; it < pairs; ++it) {
                const int s = it % kTcStages;
                if (it >= kTcStages && !mbar_wait(&raw_empty[s], ((it / kTcStages) - 1) & 1)) { report_error(ZTQ_ERR_EMPTY_WAIT); *abort_flag = 1; break; }
                const int tile = blockIdx.x + (it / (p.G / 2)) * gridDim.x, gp = it % (p.G / 2);
                mbar_expect_tx(&raw_full[s], kTcRawBytes);
                tma_load_2d(raw + (size_t)s * kTcRawBytes, &wmap, gp * 128, tile * 128, &raw_full[s]);
            }
        }
    } else if (warp == 13) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            const uint32_t idesc = tc_idesc_f16(NMMA);
            for (int it = 0; it < total; ++it) {
                const int ab = it % kTcBuf;
                const uint32_t ph = (it / kTcBuf) & 1;
                if (!mbar_wait(&a_full[ab], ph) || !mbar_wait(&b_full[ab], ph) ||
                    (it >= kTcBuf && !mbar_wait(&d_empty[ab], ph ^ 1))) { report_error(ZTQ_ERR_TMEM_WAIT); *abort_flag = 1; break; }
                tc_fence_after();
                const uint8_t* A = abuf + (size_t)ab * kTcABytes;
                const uint8_t* Bt = bbuf + (size_t)ab * B_BYTES;
#pragma unroll
                for (int j = 0; j < 8; ++j) {                      // k-step j: core-matrix columns 2j and 2j+1
                    const uint64_t ad = tc_smem_desc(A + (size_t)j * 2 * 2048, 2048, 128);
                    const uint64_t bd = tc_smem_desc(Bt + (size_t)j * 2 * (NMMA / 8) * 128, (NMMA / 8) * 128, 128);
                    tc_mma_f16(tmem_base + (uint32_t)ab * NMMA, ad, bd, idesc, j > 0);
                }
                tc_commit(&a_empty[ab]);                           // each commit fires when the MMAs above are done
                tc_commit(&b_empty[ab]);
                tc_commit(&d_full[ab]);
            }
        }
    } else if (warp >= 14) {
        // ---------------------------------------------------------------- activation stager (64 threads)
        // The 16-byte pieces of the next group are fetched into registers while the current one is stored.
        const int st = tid - 14 * 32;
        constexpr int ITEMS = NMMA * 16 / 64;                      // (batch row, core column) pieces per thread
        uint4 pre[ITEMS];
        auto fetch = [&](int g) {
#pragma unroll
            for (int i = 0; i < ITEMS; ++i) {
                const int item = st + i * 64;
                const int b = item % NMMA, ki = item / NMMA;
                pre[i] = make_uint4(0, 0, 0, 0);
                if (b < p.batch) pre[i] = __ldg(reinterpret_cast<const uint4*>(p.x + (size_t)b * p.K + (size_t)g * 128 + ki * 8));
            }
        };
        if (total > 0) fetch(0);
        for (int it = 0; it < total; ++it) {
            const int bb = it % kTcBuf;
            if (it >= kTcBuf && !mbar_wait(&b_empty[bb], ((it / kTcBuf) - 1) & 1)) { report_error(ZTQ_ERR_EMPTY_WAIT); *abort_flag = 1; break; }
            uint8_t* Bt = bbuf + (size_t)bb * B_BYTES;
            float psum = 0.f;                                      // this thread's share of sum_k x[b, k] over the group
#pragma unroll
            for (int i = 0; i < ITEMS; ++i) {
                const int item = st + i * 64;
                const int b = item % NMMA, ki = item / NMMA;
                const uint4 q = pre[i];
                {
                    const uint32_t w4[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const __half2 h = *reinterpret_cast<const __half2*>(&w4[j]);
                        psum += __low2float(h);
                        psum += __high2float(h);
                    }
                }
                uint4 o;                                           // (k0..k7) -> (k0,k4,k1,k5,k2,k6,k3,k7)
                o.x = __byte_perm(q.x, q.z, 0x5410);
                o.y = __byte_perm(q.x, q.z, 0x7632);
                o.z = __byte_perm(q.y, q.w, 0x5410);
                o.w = __byte_perm(q.y, q.w, 0x7632);
                *reinterpret_cast<uint4*>(Bt + (size_t)(ki * (NMMA / 8) + (b >> 3)) * 128 + (b & 7) * 16) = o;
            }
            // every item of a thread has the same batch column: st % NMMA; the columns's PARTS partial sums are
            // added by the epilogue in a fixed order
            sxp[((it % kTcSxRing) * PARTS + st / NMMA) * NMMA + (st % NMMA)] = psum;
            proxy_fence_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(&b_full[bb]);
            if (it + 1 < total) fetch((it + 1) % p.G);
        }
    } else if (warp >= 4) {
        // ---------------------------------------------------------------- decode: 8 warps, (row block, chunk)
        const int dw = warp - 4;                                   // two (row block, 16-byte chunk) items per warp
        for (int it = 0; it < total; ++it) {
            const int pr = it >> 1, half = it & 1;                 // raw stage of this pair of groups, which half
            const int s = pr % kTcStages, ab = it % kTcBuf;
            if ((half == 0 && !mbar_wait(&raw_full[s], (pr / kTcStages) & 1)) ||
                (it >= kTcBuf && !mbar_wait(&a_empty[ab], ((it / kTcBuf) - 1) & 1))) { report_error(ZTQ_ERR_FULL_WAIT); *abort_flag = 1; break; }
            const uint8_t* rs = raw + (size_t)s * kTcRawBytes;
            uint8_t* A = abuf + (size_t)ab * kTcABytes;
#pragma unroll
            for (int q2 = 0; q2 < 2; ++q2) {
                const int item = dw * 2 + q2;                      // 0..15
                const int c = item & 3, r = (item >> 2) * 32 + lane;
                // 128-byte swizzle of the TMA: 16-byte chunk j of row r sits at chunk j ^ (r & 7)
                const uint4 q = *reinterpret_cast<const uint4*>(rs + r * 128 + (((half * 4 + c) ^ (r & 7)) << 4));
                const uint32_t qw[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                for (int j = 0; j < 4; ++j)                        // word j = eight k = core column 4c + j
                    *reinterpret_cast<uint4*>(A + (size_t)((4 * c + j) * 16 + (r >> 3)) * 128 + (r & 7) * 16) =
                        decode_word_f16(qw[j]);
            }
            proxy_fence_async();                                   // generic-proxy stores -> visible to the tensor core
            __syncwarp();
            if (lane == 0) {
                if (half == 1) mbar_arrive(&raw_empty[s]);
                mbar_arrive(&a_full[ab]);
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue: lane = row of the tile
        const int row_in_tile = warp * 32 + lane;
        float acc[NMMA];
        uint4 mq[2];
        for (int it = 0; it < total; ++it) {
            const int tile = blockIdx.x + (it / p.G) * gridDim.x, g = it % p.G, db = it % kTcBuf;
            const int row = tile * 128 + row_in_tile;
            if (g == 0) {
#pragma unroll
                for (int b = 0; b < NMMA; ++b) acc[b] = 0.f;
            }
            if ((g & 7) == 0) {                                    // eight groups of {scale, zero} per 32-byte load
                mq[0] = mq[1] = make_uint4(0, 0, 0, 0);
                if (row < p.N) {
                    const uint4* mp = reinterpret_cast<const uint4*>(p.meta + (size_t)row * p.G + g);
                    mq[0] = __ldg(mp);
                    if (g + 4 < p.G) mq[1] = __ldg(mp + 1);
                }
            }
            const uint4 mv = ((g >> 2) & 1) ? mq[1] : mq[0];
            const uint32_t m = (g & 3) == 0 ? mv.x : (g & 3) == 1 ? mv.y : (g & 3) == 2 ? mv.z : mv.w;
            if (!mbar_wait(&d_full[db], (it / kTcBuf) & 1)) { report_error(ZTQ_ERR_TMEM_WAIT); *abort_flag = 1; break; }
            tc_fence_after();
            float d[NMMA];
            tc_ld_row<NMMA>(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)db * NMMA, d);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&d_empty[db]);
            const float s = h2f((uint16_t)(m & 0xffff)), z = h2f((uint16_t)(m >> 16));
            const float* sx = sxp + (size_t)(it % kTcSxRing) * PARTS * NMMA;
#pragma unroll
            for (int b = 0; b < NMMA; ++b) {
                float sb = sx[b];
#pragma unroll
                for (int pt = 1; pt < PARTS; ++pt) sb += sx[pt * NMMA + b];
                acc[b] = fmaf(s, fmaf(-z, sb, d[b]), acc[b]);
            }
            if (g == p.G - 1 && row < p.N) {
#pragma unroll
                for (int b = 0; b < NMMA; ++b) {
                    if (b < p.batch) {
                        const size_t yi = (size_t)b * p.N + row;
                        if (p.y_f32) reinterpret_cast<float*>(p.y)[yi] = acc[b];
                        else reinterpret_cast<__half*>(p.y)[yi] = __float2half_rn(acc[b]);
                    }
                }
            }
        }
    }
    // ---- teardown: everybody meets, then the allocating warp returns the TMEM columns
    tc_fence_before();
    __syncthreads();
    if (warp == 13) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

}  // namespace ztq
