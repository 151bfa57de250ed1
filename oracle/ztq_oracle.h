/*
 * ztq_oracle.h -- CPU restatement of ztensor's weight-quantized matrix-vector path.
 *
 * TEST INFRASTRUCTURE ONLY.  This library is the checker the CUDA kernels are
 * compared against and the timed CPU baseline.  Nothing in the shipped GPU path
 * links, imports or calls it.
 *
 * Every function cites the file:line of zerfoo/ztensor it follows.  The Go
 * original cannot be compiled where this was written (no Go toolchain), so the
 * arithmetic is restated in C, operation for operation: float32 everywhere,
 * multiply and add kept as two roundings where the Go compiler emits two
 * (GOAMD64=v1 never fuses), fused where the reference's AVX2 assembly fuses.
 * Build with -ffp-contract=off.
 *
 * Parity pin: the known-answer vectors of the reference's own tests
 * (compute/ternary_gemv_test.go, the tensor/ storage tests, compute/w4a16_test.go,
 * internal/xblas/gemm_quant_test.go) are replayed against this library.
 * One piece is unpinned: zerfoo/float16 v0.2.0 (go.mod:6) is not vendored in
 * the reference tree, so its float32->float16 rounding is ASSUMED to be IEEE
 * round-to-nearest-even with gradual underflow.  That only affects scales,
 * zero points and activations that the test harness *generates*; the GPU and
 * this oracle always consume the same packed bytes.
 */
#ifndef ZTQ_ORACLE_H
#define ZTQ_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- binary16 <-> binary32 (zerfoo/float16 FromFloat32 / ToFloat32) ---- */
uint16_t zo_f32_to_f16(float v);
float    zo_f16_to_f32(uint16_t h);
/* xblas' own decoder: Inf/NaN -> 0 (internal/xblas/q4dot.go:54-78). */
float    zo_xblas_f16_bits_to_f32(uint16_t h);
void     zo_f16_from_f32(const float* src, int64_t n, uint16_t* dst);   /* tensor/fp16_storage.go:24-37 */
void     zo_f16_slice(const uint16_t* src, int64_t n, float* dst);      /* tensor/fp16_storage.go:53-63 */

/* ---- Q4_0: 18-byte blocks {fp16 scale, 16 packed bytes} (tensor/quantized.go:17-20) ---- */
int64_t zo_q4_num_blocks(int64_t n);
void    zo_quantize_q4(const float* src, int64_t n, uint8_t* blocks18);            /* :37-91  */
void    zo_dequantize_q4(const uint8_t* blocks18, int64_t n, float* dst);          /* :96-114 */
int64_t zo_q4_gpu_data_offset(int64_t total_blocks);                               /* :196-199 */
void    zo_q4_raw_bytes_gpu(const uint8_t* blocks18, int64_t n_blocks, uint8_t* out); /* :158-187 */

/* ---- Q8_0: 36-byte blocks {f32 scale, 32 x int8} (tensor/quantized.go:283-286) ---- */
void zo_quantize_q8(const float* src, int64_t n, uint8_t* blocks36);               /* :301-341 */
void zo_dequantize_q8(const uint8_t* blocks36, int64_t n, float* dst);             /* :344-355 */

/* ---- IQ4_NL: 18-byte blocks, 16-entry float32 table (tensor/iq4_storage.go:28-46) ---- */
void zo_iq4nl_table(float out[16]);
void zo_dequantize_iq4nl(const uint8_t* raw18, int64_t n, float* dst);             /* :36-46, :75-89 */

/* ---- ternary: 2 bits per value, flat across rows (tensor/ternary_storage.go) ---- */
void   zo_ternary_pack(const int8_t* vals, int64_t n, uint8_t* data);              /* :29-62 */
int8_t zo_ternary_get(const uint8_t* data, int64_t i);                             /* :39-47 */
void   zo_ternary_gemv(const uint8_t* data, const float* x, int rows, int cols, float* y); /* compute/ternary_gemv.go:12-77 */
/* ---- Q4_K (tensor/quantized_kquant.go): super-blocks of 256 weights in 144 bytes ---- */
void   zo_quantize_q4k(const float* src, int64_t n, uint8_t* raw);                    /* QuantizeQ4K, :108-233 */
void   zo_dequantize_q4k(const uint8_t* raw, int64_t n, float* dst);                  /* Q4KStorage.Dequantize / DequantizeQ4K, :54-78, :263-277 */
void   zo_q4k_scales_mins(const uint8_t* block, uint8_t* scales8, uint8_t* mins8);    /* decodeQ4KScalesMins, :34-49 */
void   zo_gemm_q4k_f32(int m, int n, int k, const uint8_t* a, const float* b, float* c);             /* xblas.GemmQ4KF32, gemm_q4k.go:15-50 (k % 256 == 0) */
void   zo_gemm_f32_q4k_nt(int m, int n, int k, const float* a, const uint8_t* b, float* c, int ncpu); /* xblas.GemmF32Q4KNT, gemm_q4k.go:54-140 */

/* ---- Q5_K (tensor/quantized_kquant.go:489-621): Q4_K plus one high bit per weight, 176 bytes per 256 ---- */
void   zo_dequantize_q5k(const uint8_t* raw, int64_t n, float* dst);                  /* DequantizeQ5K :511-552, Q5KStorage.Dequantize :579-596 */
void   zo_make_q5k_blocks(const float* src, int64_t n, uint8_t* raw);                 /* harness: the reference has no Q5_K quantizer */
void   zo_gemm_f32_q5k_nt(int m, int n, int k, const float* a, const uint8_t* b, float* c, int ncpu); /* xblas.GemmF32Q5KNT, gemm_quant.go:273-360 */

/* ---- Q6_K (tensor/quantized_kquant.go:335-483): 6-bit codes, int8 scale per 16 weights, 210 bytes per 256 ---- */
void   zo_dequantize_q6k(const uint8_t* raw, int64_t n, float* dst);                  /* DequantizeQ6K :355-382, Q6KStorage.Dequantize :411-428 */
void   zo_make_q6k_blocks(const float* src, int64_t n, uint8_t* raw);                 /* harness: the reference has no Q6_K quantizer */
void   zo_gemm_f32_q6k_nt(int m, int n, int k, const float* a, const uint8_t* b, float* c, int ncpu); /* xblas.GemmF32Q6KNT, gemm_quant.go:384-470 */

/* The element-wise steps either side of a projection (restated from the reference's device code, which is the
 * only float32 statement of them on this path): */
void   zo_fused_add_rmsnorm(const float* input, const float* residual, const float* weight, float* normed_out,
                            float* sum_out, float eps, int D);     /* internal/cuda/kernels/fused_add_rmsnorm.cu:13-50, one row */
void   zo_fused_swiglu(const float* w1, const float* w3, float* out, int n);   /* internal/cuda/kernels/fused_swiglu.cu:10-21 */

/* ---- GPTQ (4-bit) and AWQ: per-group fp16 scale + fp16 zero point ----
 * data: groups concatenated, (count+1)/2 bytes per GPTQ group, 4*((count+7)/8)
 * bytes per AWQ group (little-endian uint32 words, 8 nibbles each).           */
int64_t zo_gptq4_data_bytes(int64_t n, int group);
int64_t zo_awq_data_bytes(int64_t n, int group);
void zo_quantize_gptq4(const float* src, int64_t n, int group,
                       uint8_t* data, uint16_t* scales, uint16_t* zeros);          /* tensor/quantized_gptq.go:45-130 */
void zo_dequantize_gptq4(const uint8_t* data, const uint16_t* scales, const uint16_t* zeros,
                         int64_t n, int group, float* dst);                        /* :134-163 */
void zo_quantize_awq(const float* src, int64_t n, int group,
                     uint8_t* data, uint16_t* scales, uint16_t* zeros);            /* tensor/quantized_awq.go:44-114 */
void zo_dequantize_awq(const uint8_t* data, const uint16_t* scales, const uint16_t* zeros,
                       int64_t n, int group, float* dst);                          /* :118-136 */

/* ---- internal/xblas ---- */
/* C += A*B, row-major, K tiled by 256, skips a==0 (gemm_simd_amd64.go:16-36 + .s:9-75). */
void zo_sgemm_simd(int m, int n, int k, const float* a, const float* b, float* c);
/* A-side Q4: zero C, per block dequant, axpy per nonzero value (gemm_quant.go:37-74,637-644). */
void zo_gemm_q4_f32_fused(int m, int n, int k, const uint8_t* a_blocks18, const float* b, float* c);
/* B-side Q4 [N,K]: c[i,j] = q4DotRow (gemm_quant.go:81-157, q4dot.go:10-52). ncpu<=0: use online CPUs. */
void zo_gemm_f32_q4_nt(int m, int n, int k, const float* a, const uint8_t* b_blocks18, float* c, int ncpu);
/* A-side Q8: full dequant then sgemm (gemm_quant.go:24-28). */
void zo_gemm_q8_f32(int m, int n, int k, const uint8_t* a_blocks36, const float* b, float* c);
/* B-side Q8 [N,K] (gemm_quant.go:163-264). */
void zo_gemm_f32_q8_nt(int m, int n, int k, const float* a, const uint8_t* b_blocks36, float* c, int ncpu);

/* Number of worker threads the reference would use for the m==1 NT paths
 * (gemm_quant.go:99-105): min(NumCPU, n/4) when n*k >= 65536, else 1. */
int zo_nt_threads(int n, int k, int ncpu);
int zo_num_cpu(void);

#ifdef __cplusplus
}
#endif
#endif /* ZTQ_ORACLE_H */
