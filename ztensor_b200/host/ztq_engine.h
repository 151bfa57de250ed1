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

#include <cstddef>
#include <cstdint>
#include <map>
#include <memory>
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

// tensor.GPUStorage (tensor/gpu_storage.go:25-46): a device buffer of float32 (or fp16) elements.
class GPUStorage : public Storage {
  public:
    GPUStorage(void* ptr, size_t len, bool f16, int device, bool owned);
    ~GPUStorage() override;
    Kind kind() const override { return Kind::GPU; }
    size_t Len() const override { return len; }
    size_t len;
    bool f16;
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
};
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

    // W4A16MatMuler (compute/w4a16.go:139-143): 4-bit weights x Float16Storage activations.
    Error MatMulW4A16(const Tensor& a, const Tensor& b, Tensor* result, Tensor* dst = nullptr);

    // Copy a result tensor to the host (result.Data() in the reference).
    Error ToHost(const Tensor& t, std::vector<float>* out);
    Error Sync();
    void* Stream() const { return stream_; }
    int DeviceID() const { return device_; }
    // number of kernel launches issued by this engine (tests assert the GPU path ran)
    long long launches = 0;

  private:
    GPUEngine() = default;
    Error upload_one(Storage* s, int rows, int cols);
    Error quant_gemv(const Storage& w, int n, int k, const Tensor& act, bool act_is_kb, int batch, Tensor* result,
                     Tensor* dst, const std::vector<int>& out_shape);
    Error activation_ptr(const Tensor& act, size_t elems, const void** ptr, bool* f32, void** to_free);
    int device_ = 0;
    void* stream_ = nullptr;
};

// compute.TryW4A16MatMul (compute/w4a16.go:148-168): matched == false when the pair is not W4A16.
Error TryW4A16MatMul(GPUEngine& eng, const Tensor& a, const Tensor& b, Tensor* result, bool* matched, Tensor* dst = nullptr);
bool IsW4A16(const Tensor& a, const Tensor& b);                         // compute/w4a16.go:196-199
std::string QuantFormat(const Storage& s);                              // compute/w4a16.go:180-192

// compute.TernaryGEMVGPU (compute/ternary_gemv_gpu.go:18): y[i] = sum_j w[i,j] x[j].  The weights are
// uploaded once (cached on the storage), not per call; errors are returned, never hidden by a CPU path.
Error TernaryGEMVGPU(GPUEngine& eng, TernaryStorage& weights, const float* x, int rows, int cols, std::vector<float>* y);

}  // namespace ztq
