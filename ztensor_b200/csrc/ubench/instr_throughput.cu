// instr_throughput.cu -- thread-instructions per clock per SM of the instructions the GEMV inner loops are built from.
// Build: nvcc -O3 -std=c++17 -gencode arch=compute_100a,code=sm_100a -o instr_throughput instr_throughput.cu
// Each kernel runs 8 independent dependency chains per thread, 1024 threads per SM; the loop overhead (about 3
// instructions per 8) is included, so full-rate pipes read a little below their nominal width.
#include <cstdio>
#include <cstdint>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#define ITERS 4096
#define CHK(x) do{cudaError_t e=(x); if(e){printf("err %s line %d\n", cudaGetErrorString(e), __LINE__); return 1;}}while(0)

template<int OP> __global__ void k(unsigned long long* out, uint32_t seed, float* sink) {
    uint32_t a[8]; float f[8]; 
    for (int i=0;i<8;i++){ a[i]=seed*(i+1)+threadIdx.x; f[i]=(float)(a[i]&255); }
    unsigned long long fa[4];
    for (int i=0;i<4;i++) fa[i] = ((unsigned long long)__float_as_uint(1.0f+i)<<32) | __float_as_uint(0.5f+i);
    unsigned long long fb = ((unsigned long long)__float_as_uint(1.0001f)<<32) | __float_as_uint(0.9999f);
    __syncthreads();
    long long t0 = clock64();
    #pragma unroll 1
    for (int it=0; it<ITERS; ++it) {
        #pragma unroll
        for (int i=0;i<8;i++) {
            if (OP==0) asm volatile("lop3.b32 %0, %0, %1, 0x4B000000, 0xEA;" : "+r"(a[i]) : "r"(seed));
            if (OP==1) asm volatile("shf.r.wrap.b32 %0, %0, %0, 3;" : "+r"(a[i]));
            if (OP==2) asm volatile("mad.lo.u32 %0, %0, %1, %1;" : "+r"(a[i]) : "r"(seed));
            if (OP==3) asm volatile("fma.rn.f32 %0, %0, %1, %1;" : "+f"(f[i]) : "f"(1.0001f));
            if (OP==4) asm volatile("fma.rn.f32x2 %0, %0, %1, %1;" : "+l"(fa[i&3]) : "l"(fb));
            if (OP==5) asm volatile("add.rn.f32x2 %0, %0, %1;" : "+l"(fa[i&3]) : "l"(fb));
            if (OP==6) asm volatile("fma.rn.f16x2 %0, %0, %1, %1;" : "+r"(a[i]) : "r"(0x3c003c00u));
            if (OP==7) asm volatile("dp4a.u32.s32 %0, %1, %2, %0;" : "+r"(a[i]) : "r"(seed), "r"(0x01020304u));
            if (OP==8) asm volatile("prmt.b32 %0, %0, %1, 0x7540;" : "+r"(a[i]) : "r"(0x4B000000u));
            if (OP==9) { asm volatile("{.reg .b16 h; mov.b32 {h,_}, %1; cvt.f32.f16 %0, h;}" : "=f"(f[i]) : "r"(a[i])); a[i] += __float_as_uint(f[i]); }
            if (OP==10) asm volatile("{.reg .b16 h,g; mov.b32 {h,g}, %1; fma.rn.f32.f16 %0, h, g, %0;}" : "+f"(f[i]) : "r"(0x3c003c01u));
            if (OP==11) asm volatile("mad.wide.u32 %0, %1, %2, %0;" : "+l"(fa[i&3]) : "r"(a[i]), "r"(65536u));
            if (OP==12) asm volatile("mul.hi.u32 %0, %0, %1;" : "+r"(a[i]) : "r"(0x00100001u));
            if (OP==13) { // mix: 1 lop3 + 0.5 fadd2 + 0.5 ffma2 per weight (8 weights)
                asm volatile("lop3.b32 %0, %0, %1, 0x4B000000, 0xEA;" : "+r"(a[i]) : "r"(seed));
                if (i&1) { asm volatile("add.rn.f32x2 %0, %0, %1;" : "+l"(fa[(i>>1)&3]) : "l"(fb));
                           asm volatile("fma.rn.f32x2 %0, %0, %1, %1;" : "+l"(fa[(i>>1)&3]) : "l"(fb)); }
            }
            if (OP==14) { // mix: lop3 + ffma2 (0.5)
                asm volatile("lop3.b32 %0, %0, %1, 0x4B000000, 0xEA;" : "+r"(a[i]) : "r"(seed));
                if (i&1) asm volatile("fma.rn.f32x2 %0, %0, %1, %1;" : "+l"(fa[(i>>1)&3]) : "l"(fb));
            }
            if (OP==15) { // mix lop3 + fma (scalar)
                asm volatile("lop3.b32 %0, %0, %1, 0x4B000000, 0xEA;" : "+r"(a[i]) : "r"(seed));
                asm volatile("fma.rn.f32 %0, %0, %1, %1;" : "+f"(f[i]) : "f"(1.0001f));
            }
            if (OP==16) { // mix: 3 alu + 4 dp4a per 8 weights (int path) ~ per i: do once per 8
                if (i<3) asm volatile("lop3.b32 %0, %0, %1, 0x0f0f0f0f, 0xEA;" : "+r"(a[i]) : "r"(seed));
                if (i>=4) asm volatile("dp4a.u32.s32 %0, %1, %2, %0;" : "+r"(a[i]) : "r"(a[i-4]), "r"(0x01020304u));
            }
            if (OP==17) { // mix: imad shift + lop3 + ffma2
                asm volatile("mad.lo.u32 %0, %0, %1, %1;" : "+r"(a[i]) : "r"(seed));
                asm volatile("lop3.b32 %0, %0, %1, 0x4B000000, 0xEA;" : "+r"(a[i]) : "r"(seed));
                if (i&1) asm volatile("fma.rn.f32x2 %0, %0, %1, %1;" : "+l"(fa[(i>>1)&3]) : "l"(fb));
            }
            if (OP==18) { // hfma2 + lop3
                asm volatile("lop3.b32 %0, %0, %1, 0x64006400, 0xEA;" : "+r"(a[i]) : "r"(seed));
                asm volatile("fma.rn.f16x2 %0, %0, %1, %1;" : "+r"(a[(i+1)&7]) : "r"(0x3c003c00u));
            }
        }
    }
    long long t1 = clock64();
    uint32_t acc=0; float facc=0; for(int i=0;i<8;i++){acc+=a[i]; facc+=f[i];} for(int i=0;i<4;i++) acc += (uint32_t)(fa[i]>>32) + (uint32_t)fa[i];
    if (acc==0x12345678 && facc==1.5f) sink[0]=facc;
    if (threadIdx.x==0) out[blockIdx.x] = (unsigned long long)(t1-t0);
}

template<int OP> int run(const char* name, double instr_per_inner, int sms) {
    unsigned long long* d; float* s; CHK(cudaMalloc(&d, sizeof(unsigned long long)*sms*4)); CHK(cudaMalloc(&s, 16));
    for (int threads : {256, 1024}) {
        int blocks = sms * (threads==256 ? 4 : 1);  // 1024 threads / SM
        k<OP><<<blocks, threads>>>(d, 12345u, s); CHK(cudaDeviceSynchronize());
        k<OP><<<blocks, threads>>>(d, 12345u, s); CHK(cudaDeviceSynchronize());
        unsigned long long h[1024]; CHK(cudaMemcpy(h, d, sizeof(unsigned long long)*blocks, cudaMemcpyDeviceToHost));
        double mx=0; for(int i=0;i<blocks;i++) mx = h[i]>mx?h[i]:mx;
        double per_sm_threads = 1024.0;
        double ipc = per_sm_threads * ITERS * instr_per_inner / mx;
        printf("%-28s threads/blk=%4d  thread-instr/clk/SM = %7.1f  (warp-instr/clk/SM %.2f)\n", name, threads, ipc, ipc/32);
    }
    cudaFree(d); cudaFree(s); return 0;
}

int main() {
    int sms; cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, 0);
    int clk; cudaDeviceGetAttribute(&clk, cudaDevAttrClockRate, 0); printf("SMs %d clockRate %d kHz\n", sms, clk);
    run<0>("lop3", 8, sms); run<1>("shf", 8, sms); run<2>("imad.lo", 8, sms); run<3>("ffma", 8, sms);
    run<4>("ffma2 (f32x2)", 8, sms); run<5>("fadd2 (f32x2)", 8, sms); run<6>("hfma2", 8, sms); run<7>("dp4a", 8, sms);
    run<8>("prmt", 8, sms); run<9>("cvt.f32.f16 (+iadd)", 16, sms); run<10>("fma.f32.f16 mixed", 8, sms);
    run<11>("mad.wide.u32", 8, sms); run<12>("mul.hi.u32", 8, sms);
    run<13>("mix lop3+.5fadd2+.5ffma2", 16, sms); run<14>("mix lop3+.5ffma2", 12, sms); run<15>("mix lop3+ffma", 16, sms);
    run<16>("mix int: 3lop3+4dp4a", 7, sms); run<17>("mix imad+lop3+.5ffma2", 20, sms); run<18>("mix lop3+hfma2", 16, sms);
    return 0;
}
