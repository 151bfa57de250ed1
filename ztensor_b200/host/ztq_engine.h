// ztq_engine.h -- host-side mirror (C++) of the parts of ztensor's Go API that
// reach the quantized GEMV path, written above the C-ABI of include/ztq.h.
//
// Names, argument meaning and error behaviour follow the reference so that the
// Go maintainer can read this as the change to make there:
//   tensor.Q4Storage / Q8Storage / IQ4NLStorage / GPTQStorage / AWQStorage /
//   TernaryStorage / Float16Storage          (tensor/*.go)
//   compute.GPUEngine.UploadWeights / MatMul (compute/gpu_engine.go:778, :1409)
//   compute.TryW4A16MatMul / W4A16MatMuler   (compute/w4a16.go:139-168)
//   compute.TernaryGEMVGPU                   (compute/ternary_gemv_gpu.go:18)
// Differences, all deliberate: there is NO CPU fallback (an error is returned
// where the reference would silently call the CPU engine), packed weights stay
// packed on the device for every format (the reference re-uploads IQ4_NL / GPTQ /
// AWQ / ternary as float32), and TernaryStorage gained a device pointer.
#pragma once

#include <atomic>
#include <cstddef>
#include <cstdint>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

namespace ztq {

// Go-style error value: empty message == nil.
struct Error {
    std::string msg;
    bool ok() const { return msg.empty(); }
    static Error None() { return {}; }
};

enum class Kind { CPU, GPU, Float16, Q4, Q8, IQ4NL, GPTQ, AWQ, Ternary, Q4K, Q5K, Q6K };

// tensor.Storage[float32] (tensor/storage.go:11-21), reduced to what the path needs.
class Storage {
  public:
    virtual ~Storage();
    virtual Kind kind() const = 0;
    virtual size_t Len() const = 0;
    // SetGPUPtr / GPUPtr (e.g. tensor/quantized.go:202-212): device copy of the residency
    // layout; the storage owns it once set through the engine.
    void SetGPUPtr(void* ptr, size_t bytes, int device) { gpu_ptr_ = ptr; gpu_bytes_ = bytes; gpu_dev_ = device; }
    void* GPUPtr() const { return gpu_ptr_; }
    size_t GPUByteSize() const { return gpu_bytes_; }
    int GPUDevice() const { return gpu_dev_; }
    bool owns_gpu = false;

  protected:
    void* gpu_ptr_ = nullptr;
    size_t gpu_bytes_ = 0;
    int gpu_dev_ = -1;
};

// tensor.CPUStorage[float32]
class CPUStorage : public Storage {
  public:
    explicit CPUStorage(std::vector<float> v) : data(std::move(v)) {}
    Kind kind() const override { return Kind::CPU; }
    size_t Len() const override { return data.size(); }
    std::vector<float> data;
};

// gpuapi.MemPool + gpuapi.EpochMemPool (internal/gpuapi/mempool.go:9-24 and :26-50): device buffers are cached by
// size class and handed out again, so a warmed-up engine allocates nothing from the driver; Reset() reclaims
// every allocation wholesale (arena use) and advances the epoch, and a Free that carries an older epoch is
// dropped -- by then the bytes belong to somebody else.
class DevicePool {
  public:
    explicit DevicePool(int device) : device_(device) {}
    ~DevicePool();
    // A buffer of at least `bytes` bytes (256-byte aligned).  no_driver_alloc: fail instead of calling cudaMalloc
    // (what an allocation during stream capture must do).
    Error Alloc(size_t bytes, void** ptr, bool no_driver_alloc = false);
    void Free(void* ptr, size_t bytes);
    void FreeAtEpoch(void* ptr, size_t bytes, uint64_t epoch);
    uint64_t Epoch() const { return epoch_.load(); }
    void Reset();
    Error Drain();                                        // cached buffers back to the driver
    void Stats(int* allocations, size_t* total_bytes) const;
    long long DriverAllocs() const { return driver_allocs_.load(); }   // cudaMalloc calls so far

  private:
    static size_t size_class(size_t bytes);
    int device_;
    mutable std::mutex mu_;
    std::map<size_t, std::vector<void*>> free_;           // size class -> cached pointers
    std::map<void*, size_t> all_;                         // every buffer this pool got from the driver
    std::atomic<uint64_t> epoch_{0};
    std::atomic<long long> driver_allocs_{0};
};

// tensor.GPUStorage (tensor/gpu_storage.go:25-46): a device buffer of float32 (or fp16) elements.  Ownership
// follows the reference: a storage made from a pool (NewGPUStorageFromPool, :136-170) carries a reference count
// shared with its views (View(), :512-529); Free() gives up this holder's reference and only the last one returns
// the buffer -- to the pool at the epoch it was taken in (FreeAtEpoch), or to the driver when there is no pool.
// A storage that merely wraps a caller's pointer (owned == false, no pool) never frees anything.
class GPUStorage : public Storage {
  public:
    GPUStorage(void* ptr, size_t len, bool f16, int device, bool owned);
    ~GPUStorage() override;                               // Free()
    Kind kind() const override { return Kind::GPU; }
    size_t Len() const override { return len; }
    static std::shared_ptr<GPUStorage> FromPool(void* ptr, size_t len, bool f16, int device, DevicePool* pool, size_t alloc_bytes);
    // A view of `length` elements starting `offset_elems` in: shares the buffer and the reference count.
    std::shared_ptr<GPUStorage> View(size_t offset_elems, size_t length);
    void Free();
    int RefCount() const { return refcount_ ? refcount_->load() : (GPUPtr() ? 1 : 0); }
    bool IsView() const { return view_; }
    size_t len;
    bool f16;

  private:
    DevicePool* pool_ = nullptr;
    std::shared_ptr<std::atomic<int>> refcount_;
    void* base_ = nullptr;                                // start of the allocation (views point inside it)
    size_t alloc_bytes_ = 0;
    uint64_t pool_epoch_ = 0;
    bool view_ = false;
};

// tensor.Float16Storage (tensor/fp16_storage.go:14-22): little-endian binary16 bytes.
class Float16Storage : public Storage {
  public:
    Kind kind() const override { return Kind::Float16; }
    size_t Len() const override { return len; }
    std::vector<uint8_t> data;
    size_t len = 0;
};
std::shared_ptr<Float16Storage> NewFloat16StorageFromRaw(const uint8_t* raw, size_t num_elems);
std::shared_ptr<Float16Storage> NewFloat16StorageFromF32(const float* src, size_t n);   // round-to-nearest-even

// tensor.Q4Storage (tensor/quantized.go:23-34): 18-byte blocks {fp16 scale, 16 bytes}.
class Q4Storage : public Storage {
  public:
    Kind kind() const override { return Kind::Q4; }
    size_t Len() const override { return len; }
    size_t NumBlocks() const { return (len + 31) / 32; }
    const std::vector<uint8_t>& RawBytes() const { return blocks; }
    std::vector<uint8_t> RawBytesGPU() const;           // separated layout, tensor/quantized.go:158-187
    std::vector<uint8_t> blocks;
    size_t len = 0;
};
size_t Q4GPUDataOffset(size_t total_blocks);             // tensor/quantized.go:196-199
Error NewQ4StorageFromRaw(const uint8_t* raw, size_t raw_len, long long num_elements, std::shared_ptr<Q4Storage>* out);

// tensor.Q8Storage (tensor/quantized.go:283-298): 36-byte blocks {f32 scale, 32 x int8}.
class Q8Storage : public Storage {
  public:
    Kind kind() const override { return Kind::Q8; }
    size_t Len() const override { return len; }
    size_t NumBlocks() const { return (len + 31) / 32; }
    const std::vector<uint8_t>& RawBytes() const { return blocks; }
    std::vector<uint8_t> blocks;
    size_t len = 0;
};
Error NewQ8StorageFromBlocks(const float* scales, const int8_t* quants, size_t n_scales, long long num_elements,
                             std::shared_ptr<Q8Storage>* out);

// tensor.IQ4NLStorage (tensor/iq4_storage.go:49-72)
class IQ4NLStorage : public Storage {
  public:
    Kind kind() const override { return Kind::IQ4NL; }
    size_t Len() const override { return len; }
    size_t NumBlocks() const { return (len + 31) / 32; }
    const std::vector<uint8_t>& RawBytes() const { return raw; }
    std::vector<uint8_t> raw;
    size_t len = 0;
};
Error NewIQ4NLStorageFromRaw(const uint8_t* raw, size_t raw_len, long long num_elements, std::shared_ptr<IQ4NLStorage>* out);

// tensor.Q4KStorage (tensor/quantized_kquant.go:236-260): super-blocks of 256 weights in 144 bytes.
class Q4KStorage : public Storage {
  public:
    Kind kind() const override { return Kind::Q4K; }
    size_t Len() const override { return len; }
    size_t NumBlocks() const { return (len + 255) / 256; }
    const std::vector<uint8_t>& RawBytes() const { return raw; }
    std::vector<uint8_t> raw;
    size_t len = 0;
};
Error NewQ4KStorageFromRaw(const uint8_t* raw, size_t raw_len, long long num_elements, std::shared_ptr<Q4KStorage>* out);

// tensor.Q5KStorage (tensor/quantized_kquant.go:554-577): super-blocks of 256 weights in 176 bytes.
class Q5KStorage : public Storage {
  public:
    Kind kind() const override { return Kind::Q5K; }
    size_t Len() const override { return len; }
    size_t NumBlocks() const { return (len + 255) / 256; }
    const std::vector<uint8_t>& RawBytes() const { return raw; }
    std::vector<uint8_t> raw;
    size_t len = 0;
};
Error NewQ5KStorageFromRaw(const uint8_t* raw, size_t raw_len, long long num_elements, std::shared_ptr<Q5KStorage>* out);

// tensor.Q6KStorage (tensor/quantized_kquant.go:385-409): super-blocks of 256 weights in 210 bytes.
class Q6KStorage : public Storage {
  public:
    Kind kind() const override { return Kind::Q6K; }
    size_t Len() const override { return len; }
    size_t NumBlocks() const { return (len + 255) / 256; }
    const std::vector<uint8_t>& RawBytes() const { return raw; }
    std::vector<uint8_t> raw;
    size_t len = 0;
};
Error NewQ6KStorageFromRaw(const uint8_t* raw, size_t raw_len, long long num_elements, std::shared_ptr<Q6KStorage>* out);

// tensor.GPTQStorage (bits == 4) and tensor.AWQStorage: per-group fp16 scale and zero point.
class GroupQuantStorage : public Storage {
  public:
    explicit GroupQuantStorage(bool awq) : awq(awq) {}
    Kind kind() const override { return awq ? Kind::AWQ : Kind::GPTQ; }
    size_t Len() const override { return len; }
    size_t NumGroups() const { return (len + group_size - 1) / group_size; }
    int GroupSize() const { return group_size; }
    int Bits() const { return 4; }
    bool awq;
    std::vector<uint8_t> data;       // packed nibbles, groups concatenated (AWQ words are little-endian: same bytes)
    std::vector<uint16_t> scales, zeros;
    size_t len = 0;
    int group_size = 128;
    size_t gpu_meta_off = 0;         // byte offset of the half2 {scale, zero} array inside the device copy
};
// A GPTQ / AWQ weight that already lives on the device in the residency layout ([nibbles][pad to 256][meta]): the
// storage adopts the pointer without owning it (weights quantized on the device, or mapped by somebody else).
std::shared_ptr<GroupQuantStorage> NewGroupQuantStorageOnDevice(void* dev, size_t dev_bytes, size_t meta_off, long long num_elements,
                                                                int group_size, bool awq, int device);
Error NewGPTQStorageFromRaw(const uint8_t* data, size_t data_len, const uint16_t* scales, size_t n_scales,
                            const uint16_t* zeros, size_t n_zeros, long long num_elements, int group_size, int bits,
                            std::shared_ptr<GroupQuantStorage>* out);
Error NewAWQStorageFromRaw(const uint32_t* data, size_t n_words, const uint16_t* scales, size_t n_scales,
                           const uint16_t* zeros, size_t n_zeros, long long num_elements, int group_size,
                           std::shared_ptr<GroupQuantStorage>* out);

// tensor.TernaryStorage (tensor/ternary_storage.go): 2 bits per value, flat.
class TernaryStorage : public Storage {
  public:
    Kind kind() const override { return Kind::Ternary; }
    size_t Len() const override { return len; }
    const std::vector<uint8_t>& RawBytes() const { return data; }
    int Get(size_t i) const { return (int)((data[i / 4] >> ((i % 4) * 2)) & 3) - 1; }
    std::vector<uint8_t> data;
    size_t len = 0;
    // per-output-row fp16 scale (not in the reference; the benchmark's ternary configuration)
    std::vector<uint16_t> row_scale;
    void* gpu_row_scale = nullptr;
};
Error NewTernaryStorageFrom(const int8_t* values, size_t n, std::shared_ptr<TernaryStorage>* out);

// tensor.TensorNumeric[float32]: a shape and a storage.
struct Tensor {
    std::vector<int> shape;
    std::shared_ptr<Storage> storage;
};

// compute.GPUEngine[float32], the quantized-MatMul part.
class GPUEngine {
  public:
    static Error New(int device_id, std::unique_ptr<GPUEngine>* out);      // NewGPUEngine
    ~GPUEngine();

    // Quantize float32 on the device with the library's quantizers (bit-identical to
    // tensor.QuantizeQ4 / QuantizeQ8 / QuantizeGPTQ(.,group,4) / QuantizeAWQ) and return host storages.
    Error QuantizeQ4(const float* src, size_t n, std::shared_ptr<Q4Storage>* out);
    Error QuantizeQ8(const float* src, size_t n, std::shared_ptr<Q8Storage>* out);
    Error QuantizeGPTQ(const float* src, size_t n, int group_size, int bits, std::shared_ptr<GroupQuantStorage>* out);
    Error QuantizeAWQ(const float* src, size_t n, int group_size, std::shared_ptr<GroupQuantStorage>* out);

    // UploadWeights (compute/gpu_engine.go:778): packed residency for EVERY quantized format.
    Error UploadWeights(const std::vector<Tensor*>& tensors);

    // MatMul (compute/gpu_engine.go:1409): c = a @ b for 2-D operands (leading batch dimensions of the
    // activation operand are flattened).  One operand must be a quantized weight: on A it is [N, K] and b is
    // the activations [K, batch]; on B it is the "virtual transpose" (logical [K, N], stored [N, K]) and a is
    // [batch, K].  The result is a float32 GPUStorage tensor, or is written into dst's storage when given.
    Error MatMul(const Tensor& a, const Tensor& b, Tensor* result, Tensor* dst = nullptr);

    // W4A16MatMuler (compute/w4a16.go:139-143): 4-bit weights x Float16Storage activations.  Operand layout as in
    // compute.MatMulW4A16 (w4a16.go:71-119), which dequantizes the weights and multiplies the two matrices as they
    // are: weights on A are [N, K] (rows of K weights: the GEMV kernels); weights on B are a LITERAL row-major
    // [K, N] matrix -- no virtual transpose, unlike Engine.MatMul's quantized-B case -- and are multiplied by a
    // dequantize + dense kernel pair in the reference's order of summation.
    Error MatMulW4A16(const Tensor& a, const Tensor& b, Tensor* result, Tensor* dst = nullptr);

    // A device-resident activation tensor (fp16 or float32) from the engine's pool, and a host -> device copy into
    // it on the engine's stream (GPUStorage.CopyFromHostAsync, tensor/gpu_storage.go:455-466).
    Error NewDeviceTensor(const std::vector<int>& shape, bool f16, Tensor* out);
    Error CopyFromHost(const Tensor& t, const void* host, size_t bytes);
    Error CopyToHost(const Tensor& t, void* host, size_t bytes);     // asynchronous on the engine's stream

    // CUDA-graph capture of a run of engine calls (compute/gpu_engine.go:1179-1259).  While capturing, nothing
    // synchronises and the pool may only hand out cached buffers (run the same calls once before capturing).
    Error BeginCapture();
    Error EndCapture(void** graph_exec);
    Error ReplayGraph(void* graph_exec);
    Error DestroyGraph(void* graph_exec);
    bool CaptureActive() const { return capturing_; }

    // Copy a result tensor to the host (result.Data() in the reference).
    Error ToHost(const Tensor& t, std::vector<float>* out);
    Error Sync();
    DevicePool* Pool() { return pool_.get(); }
    void* Stream() const { return stream_; }
    int DeviceID() const { return device_; }
    // number of kernel launches issued by this engine (tests assert the GPU path ran)
    long long launches = 0;

  private:
    GPUEngine() = default;
    Error upload_one(Storage* s, int rows, int cols);
    Error quant_gemv(const Storage& w, int n, int k, const Tensor& act, bool act_is_kb, int batch, Tensor* result,
                     Tensor* dst, const std::vector<int>& out_shape);
    Error activation_ptr(const Tensor& act, size_t elems, const void** ptr, bool* f32, void** staged, size_t* staged_bytes);
    Error w4a16_b_literal(const Tensor& a, const Tensor& b, Tensor* result, Tensor* dst);
    int device_ = 0;
    void* stream_ = nullptr;
    std::unique_ptr<DevicePool> pool_;
    bool capturing_ = false;
};

// compute.TryW4A16MatMul (compute/w4a16.go:148-168): matched == false when the pair is not W4A16.
Error TryW4A16MatMul(GPUEngine& eng, const Tensor& a, const Tensor& b, Tensor* result, bool* matched, Tensor* dst = nullptr);
bool IsW4A16(const Tensor& a, const Tensor& b);                         // compute/w4a16.go:196-199
std::string QuantFormat(const Storage& s);                              // compute/w4a16.go:180-192

// compute.TernaryGEMVGPU (compute/ternary_gemv_gpu.go:18): y[i] = sum_j w[i,j] x[j].  The weights are
// uploaded once (cached on the storage), not per call; errors are returned, never hidden by a CPU path.
Error TernaryGEMVGPU(GPUEngine& eng, TernaryStorage& weights, const float* x, int rows, int cols, std::vector<float>* y);

}  // namespace ztq
