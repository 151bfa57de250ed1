// ztq_common.cuh -- device primitives shared by the sm_100a kernels.
//
// mbarrier + 1-D bulk async copy (TMA engine, no tensor map, never multicast),
// bounded waits, packed fp32x2 arithmetic, warp reductions with a fixed order.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ztq {

// Device-side error word.  A kernel that gives up on a bounded wait stores a
// non-zero code here and returns; the host reads it with ztq_device_error().
// 0 = no error.
enum : int {
    ZTQ_ERR_NONE = 0,
    ZTQ_ERR_FULL_WAIT = 1,    // consumer gave up waiting for a weight tile
    ZTQ_ERR_EMPTY_WAIT = 2,   // producer gave up waiting for a free stage
    ZTQ_ERR_TMEM_WAIT = 3,    // epilogue gave up waiting for the tensor pipe
    ZTQ_ERR_FLAG_WAIT = 4,    // all-reduce gave up waiting for a peer's flag
};

__device__ int g_ztq_error = 0;   // the library is a single translation unit

__device__ __forceinline__ void report_error(int code) { atomicCAS(&g_ztq_error, 0, code); }

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: every try_wait already sleeps up to a hardware time limit, so
// kSpinLimit tries is seconds, not microseconds.  Returns false on give-up.
constexpr uint32_t kSpinLimit = 1u << 22;
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    for (uint32_t i = 0; i < kSpinLimit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}

// ---------------------------------------------------------------- bulk copy
// global -> shared, completion counted in bytes on `bar`.  Both addresses must
// be 16-byte aligned and `bytes` a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
            smem_u32(dst_smem)),
        "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}
// Same with an L2 eviction-priority hint (weights are read once).
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ void bulk_g2s_hint(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar,
                                              uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::
            "r"(smem_u32(dst_smem)),
        "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
        : "memory");
}

// ---------------------------------------------------------------- PDL
// Programmatic dependent launch: `grid_dep_wait` blocks until the kernels this
// one depends on have completed and flushed; `grid_dep_launch` lets the next
// kernel in the stream start its prologue.  Both are no-ops without the
// launch attribute.
__device__ __forceinline__ void grid_dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_dep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---------------------------------------------------------------- named barrier
__device__ __forceinline__ void bar_sync(int id, int nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// ---------------------------------------------------------------- fp32x2
// Packed pair arithmetic (one issue slot for two fp32 lanes on sm_100).
struct f2 {
    float x, y;
};
__device__ __forceinline__ f2 ffma2(f2 a, f2 b, f2 c) {
    f2 d;
    asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\t"
        "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tmov.b64 rc, {%6, %7};\n\t"
        "fma.rn.f32x2 rd, ra, rb, rc;\n\t"
        "mov.b64 {%0, %1}, rd;\n\t}"
        : "=f"(d.x), "=f"(d.y)
        : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
    return d;
}
__device__ __forceinline__ f2 fadd2(f2 a, f2 b) {
    f2 d;
    asm("{\n\t.reg .b64 ra, rb, rd;\n\t"
        "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
        "add.rn.f32x2 rd, ra, rb;\n\t"
        "mov.b64 {%0, %1}, rd;\n\t}"
        : "=f"(d.x), "=f"(d.y)
        : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
    return d;
}

// ---------------------------------------------------------------- reductions
// Butterfly sum over the 32 lanes; every lane ends with the same value and the
// association order is fixed by the lane ids, so results repeat run to run.
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Reduce two per-lane values at once: after the first exchange lanes 0-15 own
// value a and lanes 16-31 own value b.  Result: lanes 0-15 return sum(a),
// lanes 16-31 return sum(b).
__device__ __forceinline__ float warp_sum2(float a, float b, int lane) {
    const bool hi = (lane & 16) != 0;
    float keep = hi ? b : a;
    float send = hi ? a : b;
    keep += __shfl_xor_sync(0xffffffffu, send, 16);
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) keep += __shfl_xor_sync(0xffffffffu, keep, o);
    return keep;
}

// ---------------------------------------------------------------- system-scope flags (peer GPUs)
__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// 8-byte {value, tag} cells: one store and one load move value and tag together,
// so a receiver that sees the expected tag also sees the value, without fences.
__device__ __forceinline__ void st_cell_sys(uint2* p, uint32_t value_bits, uint32_t tag) {
    asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(value_bits), "r"(tag) : "memory");
}
__device__ __forceinline__ uint2 ld_cell_sys(const uint2* p) {
    uint2 v;
    asm volatile("ld.relaxed.sys.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ float h2f(uint16_t bits) { return __half2float(__ushort_as_half(bits)); }

}  // namespace ztq
