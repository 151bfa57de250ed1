/*
 * ztq.h -- C ABI of libztq_sm100a.so: B200 (sm_100a) weight-quantized GEMV kernels
 * behind ztensor's kernel-library calling convention.
 *
 * Conventions (the ones ztensor's zero-CGo binding layer relies on,
 * internal/cuda/purego.go:237 `Ccall(fn, args ...uintptr)`):
 *   - every argument is an integer-class machine word (pointers, int, cudaStream_t);
 *   - the return value is a cudaError_t, 0 = success;
 *   - all pointers are DEVICE pointers owned by the caller; a launcher allocates
 *     nothing, keeps nothing, never synchronises and never reads device memory,
 *     so it can be recorded into a CUDA graph;
 *   - launches are asynchronous on `stream` (NULL = legacy default stream);
 *   - argument errors are reported as cudaErrorInvalidValue before any launch.
 *     There is no CPU fallback: the caller decides what to do with an error.
 *
 * Packed-weight layouts on the device ("residency layouts"):
 *   Q4_0     separated, exactly Q4Storage.RawBytesGPU (tensor/quantized.go:158-187):
 *            [fp16 scale x nBlocks][pad to 16 B][16 data bytes x nBlocks]
 *   IQ4_NL   the same separated layout (built from the 18-byte blocks by
 *            ztq_repack_blocks18)
 *   Q8_0     Q8Storage.RawBytes (tensor/quantized.go:427-438): 36-byte blocks
 *            {f32 scale, 32 x int8}, unchanged
 *   W4G      GPTQ 4-bit / AWQ, one layout for both (their packed bytes are
 *            identical): [data: K/2 bytes per row] + [half2 {scale, zero} per group]
 *   ternary  TernaryStorage bytes with every row starting on a byte
 *            (ceil(K/4) bytes per row; identical to RawBytes when K % 4 == 0),
 *            the layout internal/cuda/kernels/ternary_gemv.cu:21-29 expects
 */
#ifndef ZTQ_H
#define ZTQ_H

#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* flags for the ztq_gemv_* entry points */
#define ZTQ_X_F32   1   /* activations are float32 (default: fp16)            */
#define ZTQ_Y_F32   2   /* outputs are float32 (default: fp16, round-nearest)  */
#define ZTQ_X_KB    4   /* activations laid out [K, batch] (default [batch,K]) */
#define ZTQ_Y_NB    8   /* outputs laid out [N, batch] (default [batch, N])    */
#define ZTQ_NO_PDL 16   /* launch without the programmatic-dependent-launch attribute.  With it (the default) a kernel
                           starts fetching the packed WEIGHTS before it waits for the preceding kernel of the stream;
                           activations, workspaces and outputs are ordered after that kernel.  Kernels of this
                           library that write weight layouts never release their dependents early, so sequences of
                           ztq calls are safe; a caller whose own kernel writes weights and triggers its dependents
                           early (griddepcontrol.launch_dependents) directly in front of a ztq launch passes this flag. */
#define ZTQ_PLAIN  32   /* force the plain (non-streaming) kernel              */
#define ZTQ_FP32_DECODE 64 /* decode codes to fp32 in registers instead of the exact integer block dot */

/* ---- drop-in replacements: same names, arguments and meaning as the
 * ---- reference's launchers ------------------------------------------------ */

/* Replaces internal/cuda/kernels/gemm_q4.h:29-33 (gemm_q4.cu:163-201).
 * C[M,N] = dequant(A_q4[M,K]) * B[K,N]; A in the separated layout, data region
 * at byte `data_offset`; B, C float32 row-major.  K % 32 must be 0. */
cudaError_t gemm_q4_f32(const void* A_q4, const float* B, float* C, int M, int K, int N, int data_offset,
                        cudaStream_t stream);

/* Replaces internal/cuda/kernels/gemm_q8.h (gemm_q8.cu:156-182): A is M*K/32
 * 36-byte Q8_0 blocks. */
cudaError_t gemm_q8_f32(const void* A_q8, const float* B, float* C, int M, int K, int N, cudaStream_t stream);

/* Replaces internal/cuda/kernels/ternary_gemv.h:33-37 (ternary_gemv.cu:85-99):
 * y[m] = sum_k decode(W[m,k]) * x[k], W row-aligned 2-bit codes, x, y float32. */
cudaError_t ternary_gemv_f32(const void* W_ternary, const float* x, float* y, int M, int K, cudaStream_t stream);

/* ---- fp16-activation entry points (the W4A16 path and its siblings).
 * y[b, n] = sum_k dequant(W[n, k]) * x[b, k], 1 <= batch.  These are what
 * GPUEngine.MatMul's B-weight branches (compute/gpu_engine.go:2127-2204 for Q4,
 * :2617-2686 for Q8) and a GPUEngine.MatMulW4A16 (the optional interface of
 * compute/w4a16.go:139-143) bind instead of transposing around gemm_q4_f32. */
cudaError_t ztq_gemv_q4_0(const void* w_sep, int data_offset, const void* x, void* y, int N, int K, int batch,
                          int flags, cudaStream_t stream);
cudaError_t ztq_gemv_iq4nl(const void* w_sep, int data_offset, const void* x, void* y, int N, int K, int batch,
                           int flags, cudaStream_t stream);
cudaError_t ztq_gemv_q8_0(const void* w_blocks36, const void* x, void* y, int N, int K, int batch, int flags,
                          cudaStream_t stream);
/* GPTQ 4-bit / AWQ: qdata = N*K/2 bytes, meta = half2 {scale, zero} per group,
 * groups of `group` consecutive k inside a row (a power of two >= 32 dividing K;
 * 128 is the tuned case). */
cudaError_t ztq_gemv_w4g(const void* qdata, const void* meta, const void* x, void* y, int N, int K, int group,
                         int batch, int flags, cudaStream_t stream);
/* Three or more activation rows (any batch >= 1 is accepted): the same product as ztq_gemv_w4g, group 128, fp16
 * activations [batch, K], outputs [batch, N], computed as a skinny GEMM on the tcgen05 tensor cores with TMEM
 * accumulators (weights as the M operand, batch padded to 8, 16 or 32 as the N operand, 32 activation vectors per
 * pass over the weights).  Default operands: the 4-bit codes and the activations as three int8 digit planes of a
 * 21-bit block fixed point (exact integer group sums); ZTQ_FP32_DECODE: fp16 operands, nothing rounded.
 * This is the batched form of the W4A16 entry a GPUEngine.MatMulW4A16 (compute/w4a16.go:139-143) binds when
 * m >= 3; the reference has no tensor-core path for quantized weights (its batch path is the naive 16x16 tile
 * kernel of gemm_q4.cu:119-159).  `workspace` (>= ztq_gemm_w4g_tc_workspace_bytes(N, K, batch), 256-byte aligned,
 * caller-owned, overwritten) receives the activations rearranged into tensor-core tiles by a small first kernel.
 * K % 512 == 0.  Flags: ZTQ_Y_F32, ZTQ_NO_PDL, ZTQ_FP32_DECODE. */
size_t ztq_gemm_w4g_tc_workspace_bytes(int N, int K, int batch);
cudaError_t ztq_gemm_w4g_tc(const void* qdata, const void* meta, const void* x, void* y, int N, int K, int group, int batch,
                            void* workspace, size_t workspace_bytes, int flags, cudaStream_t stream);
/* The same for Q4_0 weights (a scale per block of 32, zero point 8): the batched form of ztq_gemv_q4_0, which the
 * B-weight branch of GPUEngine.MatMul binds from three activation rows on, where the reference transposes, runs its
 * 16x16 tile kernel and transposes back (compute/gpu_engine.go:2166-2203, gemm_q4.cu:119-159).  Each of a group's
 * four tensor-core steps (32 k = one block) keeps an accumulator of its own and the epilogue applies the block
 * scales; 16 activation vectors per pass over the weights.  w_sep / data_offset as for ztq_gemv_q4_0
 * (data_offset > 0), fp16 activations [batch, K], outputs [batch, N]; K % 512 == 0.  Flags: ZTQ_Y_F32, ZTQ_NO_PDL. */
size_t ztq_gemm_q4_0_tc_workspace_bytes(int N, int K, int batch);
cudaError_t ztq_gemm_q4_0_tc(const void* w_sep, int data_offset, const void* x, void* y, int N, int K, int batch, void* workspace,
                             size_t workspace_bytes, int flags, cudaStream_t stream);

/* Q8_0 with 3 or more activation rows, on the storage's own bytes (Q8Storage.RawBytes: 36-byte blocks {float32 scale,
 * 32 int8}, 16-byte aligned base): the same tensor-core kernel with the int8 codes as the signed operand, the scales
 * taken from the blocks as they stream through shared memory, activations as 18-bit block fixed point (a block's 32
 * products with codes up to +-127 stay inside int32).  K % 512 == 0, fp16 activations [batch, K], y [batch, N] fp16
 * (or fp32 with ZTQ_Y_F32); replaces the tile kernel of gemm_q8.cu:113-152 for batches. */
size_t ztq_gemm_q8_0_tc_workspace_bytes(int N, int K, int batch);
cudaError_t ztq_gemm_q8_0_tc(const void* blocks36, const void* x, void* y, int N, int K, int batch, void* workspace,
                             size_t workspace_bytes, int flags, cudaStream_t stream);
/* Ternary with an optional fp16 scale per output row (row_scale may be NULL). */
cudaError_t ztq_gemv_ternary(const void* w_rows, const void* row_scale, const void* x, void* y, int N, int K,
                             int batch, int flags, cudaStream_t stream);

/* ---- split-K for narrow outputs (few rows, long K), batch 1.  The K axis is cut into `splits`
 * (2..64) equal slices handled by separate groups of CTAs; each writes fp32 partial sums of all N rows
 * to `workspace` (>= ztq_splitk_workspace_bytes(N, splits), 16-byte aligned, caller-owned, contents
 * overwritten), and a second kernel adds the slices in slice order: deterministic, no atomics.
 * Completes the "split-K with a deterministic second-pass reduction" the reference's kernels lack
 * (gemm_q4.cu:163-191 launches ceil(M/16) blocks whatever K is).  K/splits must be a multiple of
 * 256 (Q4_0) or of 4*group (W4G).  Activations are one contiguous vector [K], outputs [N].
 * Flags: ZTQ_X_F32, ZTQ_Y_F32, ZTQ_NO_PDL, ZTQ_FP32_DECODE; any other flag (the layout flags ZTQ_X_KB /
 * ZTQ_Y_NB, ZTQ_PLAIN) returns cudaErrorInvalidValue. */
size_t ztq_splitk_workspace_bytes(int N, int splits);
cudaError_t ztq_gemv_w4g_splitk(const void* qdata, const void* meta, const void* x, void* y, int N, int K, int group,
                                int splits, void* workspace, size_t workspace_bytes, int flags, cudaStream_t stream);
cudaError_t ztq_gemv_q4_0_splitk(const void* w_sep, int data_offset, const void* x, void* y, int N, int K, int splits,
                                 void* workspace, size_t workspace_bytes, int flags, cudaStream_t stream);

/* Split-K GEMV for callers that must not allocate.  No counterpart in the reference.
 *
 * Who needs it: an engine that hands out every device buffer from an arena it sized at start-up and
 * treats a cudaMalloc after that point as a bug, or a caller that is already recording a CUDA graph,
 * where allocating is not allowed.  Such a caller has nowhere to get the split-K workspace from, so
 * this variant brings its own: the fp32 partial sums go into a fixed array inside the library
 * (ZTQ_STATIC_SCRATCH_BYTES, resident on every GPU that loads the library until the process ends).
 * The call allocates nothing and frees nothing; inputs and the output are still the caller's.
 *
 * Limits and rules:
 *   - N * splits * 4 bytes must not exceed ZTQ_STATIC_SCRATCH_BYTES, otherwise cudaErrorInvalidValue
 *     is returned and nothing is launched (use ztq_gemv_w4g_splitk with your own workspace instead);
 *   - the first call on each device looks up the array's device address (the device must be
 *     current); make that first call before starting any stream capture on that device.  A first
 *     call made on a capturing stream returns cudaErrorStreamCaptureUnsupported and leaves no trace:
 *     a later call outside capture does the set-up;
 *   - all calls share the one array and it keeps whatever the last call left in it.  Nothing in it
 *     has to start at zero: every call overwrites the N * splits partial sums it later reads.  Two
 *     calls whose kernels can overlap on the GPU (different streams, no dependency) race on the array:
 *     keep calls to this entry point ordered on one stream or otherwise serialised.
 * Arguments and results are those of ztq_gemv_w4g_splitk. */
#define ZTQ_STATIC_SCRATCH_BYTES (1 << 20)
cudaError_t ztq_gemv_w4g_splitk_static(const void* qdata, const void* meta, const void* x, void* y, int N, int K,
                                       int group, int splits, int flags, cudaStream_t stream);

/* ---- tensor-parallel row shards: GEMV with the all-reduce of its outputs fused in.
 * No counterpart in the reference (its all-reduce, internal/nccl/nccl_purego.go:267-285,
 * has no caller); this is the shard path of a row-parallel
 * projection.  Every rank (one process per GPU) calls the same sequence of
 * *_allreduce launchers with the same shapes.  The kernel pushes every fp32
 * partial output as an 8-byte {value, tag} cell into every rank's slot buffer
 * with one plain peer store (no multicast, no fences), then waits a bounded time
 * until its own rank's cells of that row carry the tag of this launch and adds
 * them in rank order, so y is the full sum and is bit-identical on all ranks.
 * If a peer never arrives the kernel gives up, sets the device error word
 * (ztq_device_error() == 4) and returns; the context stays usable.
 * The all-reduce exists in the integer-arithmetic kernels only: ZTQ_FP32_DECODE and ZTQ_PLAIN are refused
 * (cudaErrorInvalidValue) by the *_allreduce entry points. */
typedef struct ZtqAllReduce {
    int world, rank;      /* 2..8 ranks */
    int slot_stride;      /* cells per (parity, rank) slot: >= batch * N of the largest reduced output */
    int reserved;
    void* slots[8];       /* slots[r]: rank r's slot buffer as mapped in THIS process:
                             2 * world * slot_stride cells of 8 bytes, zero-initialised */
    void* state;          /* this rank's {launch sequence, finished CTAs}: 2 unsigned, zero-initialised */
} ZtqAllReduce;

cudaError_t ztq_gemv_w4g_allreduce(const void* qdata, const void* meta, const void* x, void* y, int N, int K, int group,
                                   int batch, int flags, const ZtqAllReduce* ar, cudaStream_t stream);
/* The same for 3 or more activation rows: ztq_gemm_w4g_tc with the all-reduce in its epilogue.  The warp that holds
 * a row tile's final sums pushes them as cells and goes on with its next tile; the peers' cells are collected after
 * the CTA's last tile.  Integer operands only (ZTQ_FP32_DECODE is refused); passes of 16 activation rows, each one
 * launch of the sequence every rank counts; slot_stride >= min(batch, 16) * N.  GEMV and tensor-core launchers of
 * one ZtqAllReduce may alternate freely as long as every rank issues the same sequence. */
cudaError_t ztq_gemm_w4g_tc_allreduce(const void* qdata, const void* meta, const void* x, void* y, int N, int K, int group,
                                      int batch, void* workspace, size_t workspace_bytes, int flags, const ZtqAllReduce* ar,
                                      cudaStream_t stream);
cudaError_t ztq_gemv_q4_0_allreduce(const void* w_sep, int data_offset, const void* x, void* y, int N, int K, int batch,
                                    int flags, const ZtqAllReduce* ar, cudaStream_t stream);

/* ---- Q4_K (tensor/quantized_kquant.go: super-blocks of 256 weights in 144 bytes) --------------------
 * y[b, n] = sum_k dequant(W[n, k]) * x[b, k], the product xblas.GemmF32Q4KNT / GemmQ4KF32 compute on the CPU engine
 * (internal/xblas/gemm_q4k.go:15-140) and gemv_q4k_f32 on the reference's GPU path (compute/gpu_engine.go:2209-2330).
 * w_sep is the separated device layout made by ztq_repack_blocks144: the 16 header bytes {fp16 d, fp16 dmin, 12
 * bytes of 6-bit scales and mins} of every super-block, then at data_offset = 16 * nblocks the 128 nibble bytes of
 * every super-block.  K % 256 == 0 and K >= 2048; batch <= 8 (one pass over the weights per row).
 * Flags: ZTQ_X_F32, ZTQ_Y_F32, ZTQ_NO_PDL. */
cudaError_t ztq_gemv_q4k(const void* w_sep, long long data_offset, const void* x, void* y, int N, int K, int batch, int flags,
                         cudaStream_t stream);
/* RawBytes() of a Q4KStorage (144-byte super-blocks, 16-byte aligned) -> the separated layout above. */
cudaError_t ztq_repack_blocks144(const void* aos, void* sep, long long nblocks, cudaStream_t stream);
/* Q5_K (tensor/quantized_kquant.go:489-621; CPU product xblas.GemmF32Q5KNT, internal/xblas/gemm_quant.go:273-360;
 * the reference's GPU path is gemv_q5k_f32): as Q4_K with a fifth bit per weight.  Separated layout made by
 * ztq_repack_blocks176: per super-block 48 side bytes {16 header bytes, the 32 qh bytes}, then at data_offset =
 * 48 * nblocks the 128 low-nibble bytes of every super-block.  Same limits and flags as ztq_gemv_q4k. */
cudaError_t ztq_gemv_q5k(const void* w_sep, long long data_offset, const void* x, void* y, int N, int K, int batch, int flags,
                         cudaStream_t stream);
cudaError_t ztq_repack_blocks176(const void* aos, void* sep, long long nblocks, cudaStream_t stream);
/* Q6_K (tensor/quantized_kquant.go:335-483; CPU product xblas.GemmF32Q6KNT, internal/xblas/gemm_quant.go:384-470;
 * the reference's GPU path is gemv_q6k_f32): 6-bit codes, one int8 scale per 16 weights, one fp16 d per 256.
 * Separated layout made by ztq_repack_blocks210 (the 210-byte source blocks need no alignment): per super-block 96
 * side bytes {64 bytes qh, 16 scales, fp16 d, 14 zero bytes}, then at data_offset = 96 * nblocks the 128 ql bytes
 * of every super-block.  Same limits and flags as ztq_gemv_q4k. */
cudaError_t ztq_gemv_q6k(const void* w_sep, long long data_offset, const void* x, void* y, int N, int K, int batch, int flags,
                         cudaStream_t stream);
cudaError_t ztq_repack_blocks210(const void* aos, void* sep, long long nblocks, cudaStream_t stream);

/* ---- the steps either side of a projection, folded into the GEMV (batch 1) ---------------------
 * The reference runs RMSNorm and SwiGLU as kernels of their own around MatMul
 * (internal/cuda/kernels/fused_add_rmsnorm.cu:13-50, fused_swiglu.cu:10-21).  Here, for W4A16 weights (group
 * 128, K >= 2048, K % 256 == 0):
 *   norm_weight != NULL:  the GEMV reads  v = x + residual  (residual may be NULL), normalises it on the way
 *                         in, activation[k] = v[k] * rsqrt(mean(v^2) + eps) * norm_weight[k], and writes v to
 *                         sum_out when that is not NULL (sum_out must not alias x or residual: other CTAs
 *                         still read them).  x, residual, sum_out share x's element type (fp16, or fp32 with
 *                         ZTQ_X_F32); norm_weight is float32, 16-byte aligned; eps travels as its bit pattern.
 *   swiglu != 0:          rows of the matrix are (gate_i, up_i) pairs (ztq_interleave_rows lays them out so);
 *                         y has N / 2 entries, y[i] = gate_i * sigmoid(gate_i) * up_i.
 * Flags: ZTQ_X_F32, ZTQ_Y_F32, ZTQ_NO_PDL. */
typedef struct ZtqGemvFusion {
    const void* residual;
    const void* norm_weight;
    void* sum_out;
    unsigned int eps_bits;
    int swiglu;
} ZtqGemvFusion;
cudaError_t ztq_gemv_w4g_fused(const void* qdata, const void* meta, const void* x, void* y, int N, int K, int group, int flags,
                               const ZtqGemvFusion* fz, cudaStream_t stream);
/* out row 2i = a row i, out row 2i+1 = b row i; rows of row_bytes bytes (a multiple of 16), 16-byte aligned
 * pointers.  Applied to the packed codes and to the {scale, zero} rows of a gate and an up projection it gives
 * the pair layout the SwiGLU epilogue wants (tensor.MergeQ4Storage, tensor/quantized.go:227, concatenates instead). */
cudaError_t ztq_interleave_rows(const void* a, const void* b, void* out, long long rows, int row_bytes, cudaStream_t stream);

/* Set-up helpers for the buffers above (not for the hot path: they allocate
 * and map memory).  ztq_symm_alloc returns zeroed device memory that can be
 * exported; the 64-byte handle travels to the peer processes by any host
 * channel; ztq_ipc_open maps a peer's buffer and enables peer access. */
cudaError_t ztq_symm_alloc(void** ptr, size_t bytes);
cudaError_t ztq_symm_free(void* ptr);
/* Zeroes a buffer of ztq_symm_alloc and waits for the device.  Used to bring the ranks back in step after a
 * launch that gave up on a peer (ztq_device_error() == 4): all ranks stop launching, meet on the host, zero
 * their slot buffer and state words, meet again, and carry on from sequence number 0. */
cudaError_t ztq_symm_zero(void* ptr, size_t bytes);
cudaError_t ztq_ipc_export(void* ptr, void* handle64);
cudaError_t ztq_ipc_open(const void* handle64, void** ptr);
cudaError_t ztq_ipc_close(void* ptr);

/* ---- residency: repack and quantize on the device -------------------------
 * One-off helpers for UploadWeights (compute/gpu_engine.go:778-1058). */

/* 18-byte AoS blocks (Q4Storage.RawBytes / IQ4NLStorage.RawBytes) -> separated layout. */
cudaError_t ztq_repack_blocks18(const void* aos, void* sep, long long n_blocks, cudaStream_t stream);
/* GPTQ/AWQ group scales and zeros (two fp16 arrays) -> interleaved half2 meta. */
cudaError_t ztq_pack_w4g_meta(const void* scales, const void* zeros, void* meta, long long n_groups,
                              cudaStream_t stream);
/* Flat TernaryStorage bytes -> row-aligned rows (a copy when K % 4 == 0). */
cudaError_t ztq_repack_ternary_rows(const void* flat, void* rows, int M, int K, cudaStream_t stream);

/* float32 -> packed, bit-identical to tensor.QuantizeQ4 / QuantizeQ8 /
 * QuantizeGPTQ(.,group,4) / QuantizeAWQ (n multiple of 32 / group). */
cudaError_t ztq_quantize_q4_0(const float* src, void* sep, long long n, cudaStream_t stream);
cudaError_t ztq_quantize_q8_0(const float* src, void* blocks36, long long n, cudaStream_t stream);
cudaError_t ztq_quantize_w4g(const float* src, void* qdata, void* meta, long long n, int group, int awq_rounding,
                             cudaStream_t stream);

/* packed -> float32, bit-identical to the storages' Dequantize(). fmt: 0 Q4_0,
 * 1 IQ4_NL, 2 W4G, 3 Q8_0, 4 ternary (row-aligned, aux = K). */
cudaError_t ztq_dequantize(int fmt, const void* w, const void* meta_or_null, float* dst, long long n, int aux,
                           cudaStream_t stream);

/* y[M, N] = x[M, K] * w[K, N] with w float32 row-major, as ztq_dequantize leaves the Slice() of a 4-bit storage:
 * the product of compute.MatMulW4A16 when the weights are the B operand (compute/w4a16.go:107-119), where the
 * dequantized slice is multiplied as a literal [K, N] matrix by CPUEngine.MatMul -> SgemmSimd
 * (internal/xblas/gemm_simd_amd64.go:16-36).  Summation over k ascending, fused multiply-add except in the last
 * N % 4 columns (multiply, then add), which is the order of that routine.  x: fp16, or float32 with ZTQ_X_F32.
 * A correctness path for that operand layout, not a tuned kernel.  Flags: ZTQ_X_F32, ZTQ_NO_PDL. */
cudaError_t ztq_matmul_wkn_f32(const void* x, const float* w_kn, float* y, int M, int K, int N, int flags, cudaStream_t stream);

/* ---- probes ---------------------------------------------------------------- */
/* The launch plan the first launch of a call with these arguments gets on a device of `sms` SMs (host
 * arithmetic only, no device needed).  fmt: 0 Q4_0, 1 IQ4_NL, 2 W4G, 3 Q8_0, 4 ternary, 5 Q4_K, 6 Q5_K, 7 Q6_K
 * (the ztq_gemv_* entry points), 8 ztq_gemm_w4g_tc.  out[12]:
 *   GEMV    {kernel: 0 plain / 1 streaming / 2 chunk-pair, activation rows per launch, rows per team per stage,
 *            rows per stage, stages, overlay stages, rows per pass, grid, tiles of the busiest CTA, passes of
 *            the busiest CTA, warps per team, teams}
 *   tensor  {3, padded columns, K slices, groups per slice, row tiles, work items, grid, items of the busiest
 *            CTA, 0, 0, 0, 0}
 * Returns 0, or 1 for arguments no entry point accepts.  Tests use it to state which code path a shape runs. */
int ztq_describe_plan(int fmt, int N, int K, int group, int batch, int sms, int* out);
int ztq_check_sm100(void);          /* 1 when the current device is compute capability 10.x */
/* Launches a kernel that does nothing, with the grid, block size, dynamic shared memory and (unless ZTQ_NO_PDL)
 * the programmatic-dependent-launch attribute of a GEMV launch.  A stream of these measures the floor of a
 * dependent launch on the device at hand: the part of a small GEMV's time that no kernel change can remove. */
cudaError_t ztq_probe_launch(int grid, int threads, int smem_bytes, int flags, cudaStream_t stream);
int ztq_abi_version(void);
/* Reads and clears the device-side error word (0 = none; see ztq_common.cuh).
 * Synchronises the device: a diagnostic call, not for the hot path. */
int ztq_device_error(void);

#ifdef __cplusplus
}
#endif
#endif /* ZTQ_H */
