// ztq_engine.cc -- see ztq_engine.h.  Everything numeric happens on the device
// through the C-ABI of include/ztq.h; this file is shapes, dispatch, residency
// and error text.
#include "ztq_engine.h"

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>

#include "../../include/ztq.h"

namespace ztq {

namespace {

std::string fmt_shape(const std::vector<int>& s) {
    std::string o = "[";
    for (size_t i = 0; i < s.size(); ++i) o += (i ? " " : "") + std::to_string(s[i]);
    return o + "]";
}

Error cuda_err(cudaError_t e, const char* what) {
    if (e == cudaSuccess) return Error::None();
    char buf[160];
    snprintf(buf, sizeof(buf), "%s failed (cuda error %d)", what, (int)e);
    return Error{buf};
}

// internal/cuda/kernels/elementwise_purego.go:11-16
Error kernel_err(cudaError_t e, const char* name) {
    if (e == cudaSuccess) return Error::None();
    char buf[160];
    snprintf(buf, sizeof(buf), "%s kernel failed (cuda error %d)", name, (int)e);
    return Error{buf};
}

bool is_quant(Kind k) { return k == Kind::Q4 || k == Kind::Q8 || k == Kind::IQ4NL || k == Kind::GPTQ || k == Kind::AWQ || k == Kind::Ternary || k == Kind::Q4K || k == Kind::Q5K || k == Kind::Q6K; }
bool is_w4(Kind k) { return k == Kind::Q4 || k == Kind::GPTQ || k == Kind::AWQ; }
size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

}  // namespace

Storage::~Storage() {
    if (owns_gpu && gpu_ptr_) cudaFree(gpu_ptr_);
}

// ---------------------------------------------------------------------------- device pool
DevicePool::~DevicePool() { Drain(); }

size_t DevicePool::size_class(size_t bytes) {
    size_t c = 256;
    while (c < bytes) c <<= 1;
    return c;
}

Error DevicePool::Alloc(size_t bytes, void** ptr, bool no_driver_alloc) {
    const size_t c = size_class(bytes ? bytes : 1);
    {
        std::lock_guard<std::mutex> lk(mu_);
        auto it = free_.find(c);
        if (it != free_.end() && !it->second.empty()) {
            *ptr = it->second.back();
            it->second.pop_back();
            return Error::None();
        }
    }
    if (no_driver_alloc)
        return Error{"GPU pool: no cached buffer of " + std::to_string(c) + " bytes during stream capture (run the same calls once before capturing)"};
    cudaSetDevice(device_);
    void* p = nullptr;
    Error e = cuda_err(cudaMalloc(&p, c), "cudaMalloc");
    if (!e.ok()) return e;
    driver_allocs_.fetch_add(1);
    std::lock_guard<std::mutex> lk(mu_);
    all_[p] = c;
    *ptr = p;
    return Error::None();
}

void DevicePool::Free(void* ptr, size_t bytes) {
    if (!ptr) return;
    std::lock_guard<std::mutex> lk(mu_);
    auto it = all_.find(ptr);
    if (it == all_.end()) return;                             // not one of ours
    (void)bytes;
    free_[it->second].push_back(ptr);
}

void DevicePool::FreeAtEpoch(void* ptr, size_t bytes, uint64_t epoch) {
    if (epoch != epoch_.load()) return;                       // reclaimed by a Reset() since: the bytes are somebody else's now
    Free(ptr, bytes);
}

void DevicePool::Reset() {
    std::lock_guard<std::mutex> lk(mu_);
    epoch_.fetch_add(1);
    free_.clear();
    for (auto& kv : all_) free_[kv.second].push_back(kv.first);   // everything is available again
}

Error DevicePool::Drain() {
    std::lock_guard<std::mutex> lk(mu_);
    cudaError_t first = cudaSuccess;
    for (auto& kv : free_)
        for (void* p : kv.second) {
            cudaError_t e = cudaFree(p);
            if (e != cudaSuccess && first == cudaSuccess) first = e;
            all_.erase(p);
        }
    free_.clear();
    return cuda_err(first, "cudaFree");
}

void DevicePool::Stats(int* allocations, size_t* total_bytes) const {
    std::lock_guard<std::mutex> lk(mu_);
    int n = 0;
    size_t b = 0;
    for (auto& kv : free_) { n += (int)kv.second.size(); b += kv.first * kv.second.size(); }
    if (allocations) *allocations = n;
    if (total_bytes) *total_bytes = b;
}

// ---------------------------------------------------------------------------- GPUStorage
GPUStorage::GPUStorage(void* ptr, size_t n, bool half, int device, bool owned) : len(n), f16(half) {
    SetGPUPtr(ptr, n * (half ? 2 : 4), device);
    owns_gpu = false;                                         // ownership goes through the reference count, not the base class
    base_ = ptr;
    alloc_bytes_ = n * (half ? 2 : 4);
    if (owned) {                                              // owned outside a pool: counted, freed to the driver by the last holder
        refcount_ = std::make_shared<std::atomic<int>>(1);
    } else {
        view_ = true;                                         // a caller's pointer: never freed here
    }
}

std::shared_ptr<GPUStorage> GPUStorage::FromPool(void* ptr, size_t n, bool half, int device, DevicePool* pool, size_t alloc_bytes) {
    auto g = std::make_shared<GPUStorage>(ptr, n, half, device, true);
    g->pool_ = pool;
    g->alloc_bytes_ = alloc_bytes;
    g->pool_epoch_ = pool ? pool->Epoch() : 0;
    return g;
}

std::shared_ptr<GPUStorage> GPUStorage::View(size_t offset_elems, size_t length) {
    if (!GPUPtr() || offset_elems + length > len) return nullptr;
    uint8_t* p = static_cast<uint8_t*>(GPUPtr()) + offset_elems * (f16 ? 2 : 4);
    auto v = std::make_shared<GPUStorage>(p, length, f16, GPUDevice(), false);
    v->base_ = base_;
    v->alloc_bytes_ = alloc_bytes_;
    v->pool_ = pool_;
    v->pool_epoch_ = pool_epoch_;
    if (refcount_) {                                          // shares ownership with the parent
        v->refcount_ = refcount_;
        refcount_->fetch_add(1);
        v->view_ = false;
    }
    return v;
}

void GPUStorage::Free() {
    if (!GPUPtr()) return;
    void* base = base_;
    SetGPUPtr(nullptr, 0, GPUDevice());
    len = 0;
    if (!refcount_) return;                                   // non-owning view of a caller's pointer
    if (refcount_->fetch_sub(1) > 1) return;                  // somebody else still holds the buffer
    if (pool_) pool_->FreeAtEpoch(base, alloc_bytes_, pool_epoch_);
    else cudaFree(base);
}

GPUStorage::~GPUStorage() { Free(); }

// ---------------------------------------------------------------------------- constructors
std::shared_ptr<Float16Storage> NewFloat16StorageFromRaw(const uint8_t* raw, size_t num_elems) {
    auto s = std::make_shared<Float16Storage>();
    s->data.assign(raw, raw + num_elems * 2);
    s->len = num_elems;
    return s;
}

std::shared_ptr<Float16Storage> NewFloat16StorageFromF32(const float* src, size_t n) {
    auto s = std::make_shared<Float16Storage>();
    s->data.resize(n * 2);
    s->len = n;
    for (size_t i = 0; i < n; ++i) {
        const __half h = __float2half_rn(src[i]);             // IEEE round-to-nearest-even, host path of cuda_fp16.h
        uint16_t bits;
        memcpy(&bits, &h, 2);
        s->data[2 * i] = (uint8_t)(bits & 0xff);
        s->data[2 * i + 1] = (uint8_t)(bits >> 8);
    }
    return s;
}

size_t Q4GPUDataOffset(size_t total_blocks) { return (total_blocks * 2 + 15) & ~(size_t)15; }

std::vector<uint8_t> Q4Storage::RawBytesGPU() const {
    const size_t nb = NumBlocks(), off = Q4GPUDataOffset(nb);
    std::vector<uint8_t> out(off + nb * 16, 0);
    for (size_t i = 0; i < nb; ++i) {
        out[2 * i] = blocks[18 * i];
        out[2 * i + 1] = blocks[18 * i + 1];
        memcpy(&out[off + 16 * i], &blocks[18 * i + 2], 16);
    }
    return out;
}

// tensor/quantized.go:247-268
Error NewQ4StorageFromRaw(const uint8_t* raw, size_t raw_len, long long n, std::shared_ptr<Q4Storage>* out) {
    if (n <= 0) return Error{"numElements must be positive, got " + std::to_string(n)};
    const size_t nb = ((size_t)n + 31) / 32;
    if (raw_len < nb * 18)
        return Error{"Q4_0 raw data too short: need " + std::to_string(nb * 18) + " bytes for " + std::to_string(nb) +
                     " blocks, got " + std::to_string(raw_len)};
    auto s = std::make_shared<Q4Storage>();
    s->blocks.assign(raw, raw + nb * 18);
    s->len = (size_t)n;
    *out = s;
    return Error::None();
}

// tensor/quantized.go:455-480
Error NewQ8StorageFromBlocks(const float* scales, const int8_t* quants, size_t n_scales, long long n,
                             std::shared_ptr<Q8Storage>* out) {
    if (n <= 0) return Error{"numElements must be positive, got " + std::to_string(n)};
    const size_t nb = ((size_t)n + 31) / 32;
    if (n_scales != nb) return Error{"expected " + std::to_string(nb) + " scales, got " + std::to_string(n_scales)};
    auto s = std::make_shared<Q8Storage>();
    s->blocks.resize(nb * 36);
    for (size_t i = 0; i < nb; ++i) {
        memcpy(&s->blocks[36 * i], &scales[i], 4);
        memcpy(&s->blocks[36 * i + 4], &quants[32 * i], 32);
    }
    s->len = (size_t)n;
    *out = s;
    return Error::None();
}

// tensor/iq4_storage.go:61-72
Error NewIQ4NLStorageFromRaw(const uint8_t* raw, size_t raw_len, long long n, std::shared_ptr<IQ4NLStorage>* out) {
    if (n <= 0) return Error{"numElements must be positive, got " + std::to_string(n)};
    const size_t nb = ((size_t)n + 31) / 32, need = nb * 18;
    if (raw_len < need)
        return Error{"IQ4_NL raw data too short: need " + std::to_string(need) + " bytes for " + std::to_string(nb) +
                     " blocks, got " + std::to_string(raw_len)};
    auto s = std::make_shared<IQ4NLStorage>();
    s->raw.assign(raw, raw + need);
    s->len = (size_t)n;
    *out = s;
    return Error::None();
}

// tensor/quantized_kquant.go:248-260
Error NewQ4KStorageFromRaw(const uint8_t* raw, size_t raw_len, long long n, std::shared_ptr<Q4KStorage>* out) {
    if (n <= 0) return Error{"numElements must be positive, got " + std::to_string(n)};
    const size_t nb = ((size_t)n + 255) / 256, need = nb * 144;
    if (raw_len < need)
        return Error{"Q4_K raw data too short: need " + std::to_string(need) + " bytes for " + std::to_string(nb) +
                     " blocks, got " + std::to_string(raw_len)};
    auto s = std::make_shared<Q4KStorage>();
    s->raw.assign(raw, raw + need);
    s->len = (size_t)n;
    *out = s;
    return Error::None();
}

// tensor/quantized_kquant.go:564-577
Error NewQ5KStorageFromRaw(const uint8_t* raw, size_t raw_len, long long n, std::shared_ptr<Q5KStorage>* out) {
    if (n <= 0) return Error{"numElements must be positive, got " + std::to_string(n)};
    const size_t nb = ((size_t)n + 255) / 256, need = nb * 176;
    if (raw_len < need)
        return Error{"Q5_K raw data too short: need " + std::to_string(need) + " bytes for " + std::to_string(nb) +
                     " blocks, got " + std::to_string(raw_len)};
    auto s = std::make_shared<Q5KStorage>();
    s->raw.assign(raw, raw + need);
    s->len = (size_t)n;
    *out = s;
    return Error::None();
}

// tensor/quantized_kquant.go:397-409
Error NewQ6KStorageFromRaw(const uint8_t* raw, size_t raw_len, long long n, std::shared_ptr<Q6KStorage>* out) {
    if (n <= 0) return Error{"numElements must be positive, got " + std::to_string(n)};
    const size_t nb = ((size_t)n + 255) / 256, need = nb * 210;
    if (raw_len < need)
        return Error{"Q6_K raw data too short: need " + std::to_string(need) + " bytes for " + std::to_string(nb) +
                     " blocks, got " + std::to_string(raw_len)};
    auto s = std::make_shared<Q6KStorage>();
    s->raw.assign(raw, raw + need);
    s->len = (size_t)n;
    *out = s;
    return Error::None();
}

// tensor/quantized_gptq.go:217-277 (4-bit only here)
Error NewGPTQStorageFromRaw(const uint8_t* data, size_t data_len, const uint16_t* scales, size_t n_scales,
                            const uint16_t* zeros, size_t n_zeros, long long n, int group_size, int bits,
                            std::shared_ptr<GroupQuantStorage>* out) {
    if (n <= 0) return Error{"numElements must be positive, got " + std::to_string(n)};
    if (bits != 4 && bits != 8) return Error{"bits must be 4 or 8, got " + std::to_string(bits)};
    if (bits != 4) return Error{"GPTQ 8-bit is outside the 4-bit GEMV path"};
    if (group_size <= 0) return Error{"groupSize must be positive, got " + std::to_string(group_size)};
    const size_t ng = ((size_t)n + group_size - 1) / group_size;
    if (n_scales != ng) return Error{"expected " + std::to_string(ng) + " scales for " + std::to_string(ng) + " groups, got " + std::to_string(n_scales)};
    if (n_zeros != ng) return Error{"expected " + std::to_string(ng) + " zeros for " + std::to_string(ng) + " groups, got " + std::to_string(n_zeros)};
    size_t total = 0;
    for (size_t g = 0; g < ng; ++g) {
        size_t cnt = (size_t)n - g * group_size;
        if (cnt > (size_t)group_size) cnt = group_size;
        total += (cnt + 1) / 2;
    }
    if (data_len < total) return Error{"GPTQ data too short: need " + std::to_string(total) + " bytes, got " + std::to_string(data_len)};
    auto s = std::make_shared<GroupQuantStorage>(false);
    s->data.assign(data, data + total);
    s->scales.assign(scales, scales + ng);
    s->zeros.assign(zeros, zeros + ng);
    s->len = (size_t)n;
    s->group_size = group_size;
    *out = s;
    return Error::None();
}

// tensor/quantized_awq.go:186-237
Error NewAWQStorageFromRaw(const uint32_t* data, size_t n_words, const uint16_t* scales, size_t n_scales,
                           const uint16_t* zeros, size_t n_zeros, long long n, int group_size,
                           std::shared_ptr<GroupQuantStorage>* out) {
    if (n <= 0) return Error{"numElements must be positive, got " + std::to_string(n)};
    if (group_size <= 0) return Error{"groupSize must be positive, got " + std::to_string(group_size)};
    const size_t ng = ((size_t)n + group_size - 1) / group_size;
    if (n_scales != ng) return Error{"expected " + std::to_string(ng) + " scales for " + std::to_string(ng) + " groups, got " + std::to_string(n_scales)};
    if (n_zeros != ng) return Error{"expected " + std::to_string(ng) + " zeros for " + std::to_string(ng) + " groups, got " + std::to_string(n_zeros)};
    size_t total = 0;
    for (size_t g = 0; g < ng; ++g) {
        size_t cnt = (size_t)n - g * group_size;
        if (cnt > (size_t)group_size) cnt = group_size;
        total += (cnt + 7) / 8;
    }
    if (n_words < total) return Error{"AWQ data too short: need " + std::to_string(total) + " uint32s, got " + std::to_string(n_words)};
    auto s = std::make_shared<GroupQuantStorage>(true);
    s->data.resize(total * 4);
    memcpy(s->data.data(), data, total * 4);                  // little-endian words: nibble j%8 of word j/8 == nibble j%2 of byte j/2
    s->scales.assign(scales, scales + ng);
    s->zeros.assign(zeros, zeros + ng);
    s->len = (size_t)n;
    s->group_size = group_size;
    *out = s;
    return Error::None();
}

// tensor/ternary_storage.go:27-62 (a panic there is an error here)
Error NewTernaryStorageFrom(const int8_t* values, size_t n, std::shared_ptr<TernaryStorage>* out) {
    auto s = std::make_shared<TernaryStorage>();
    s->data.assign((n + 3) / 4, 0);
    s->len = n;
    for (size_t i = 0; i < n; ++i) {
        if (values[i] < -1 || values[i] > 1) return Error{"tensor: TernaryStorage value must be -1, 0, or 1"};
        s->data[i / 4] |= (uint8_t)((values[i] + 1) << ((i % 4) * 2));
    }
    *out = s;
    return Error::None();
}

// ---------------------------------------------------------------------------- engine
Error GPUEngine::New(int device_id, std::unique_ptr<GPUEngine>* out) {
    int count = 0;
    Error e = cuda_err(cudaGetDeviceCount(&count), "cudaGetDeviceCount");
    if (!e.ok()) return e;
    if (device_id < 0 || device_id >= count) return Error{"invalid device id " + std::to_string(device_id)};
    if ((e = cuda_err(cudaSetDevice(device_id), "cudaSetDevice")), !e.ok()) return e;
    if (!ztq_check_sm100()) return Error{"GPUEngine: device is not compute capability 10.x; the kernel library is sm_100a only"};
    std::unique_ptr<GPUEngine> g(new GPUEngine());
    g->device_ = device_id;
    cudaStream_t s;
    if ((e = cuda_err(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking), "cudaStreamCreate")), !e.ok()) return e;
    g->stream_ = s;
    g->pool_ = std::make_unique<DevicePool>(device_id);
    *out = std::move(g);
    return Error::None();
}

GPUEngine::~GPUEngine() {
    if (stream_) {
        cudaStreamSynchronize((cudaStream_t)stream_);
        cudaStreamDestroy((cudaStream_t)stream_);
    }
    // storages that outlive the engine keep their device pointers: the pool is released, not destroyed under them
    if (pool_) { pool_->Drain(); (void)pool_.release(); }
}

// ---------------------------------------------------------------------------- capture, device tensors
Error GPUEngine::BeginCapture() {
    if (capturing_) return Error{"BeginCapture: a capture is already active"};
    cudaSetDevice(device_);
    Error e = cuda_err(cudaStreamBeginCapture((cudaStream_t)stream_, cudaStreamCaptureModeThreadLocal), "cudaStreamBeginCapture");
    if (e.ok()) capturing_ = true;
    return e;
}

Error GPUEngine::EndCapture(void** graph_exec) {
    if (!capturing_) return Error{"EndCapture: no capture is active"};
    capturing_ = false;
    cudaGraph_t g = nullptr;
    Error e = cuda_err(cudaStreamEndCapture((cudaStream_t)stream_, &g), "cudaStreamEndCapture");
    if (!e.ok()) return e;
    cudaGraphExec_t ge = nullptr;
    e = cuda_err(cudaGraphInstantiate(&ge, g, 0), "cudaGraphInstantiate");
    cudaGraphDestroy(g);
    if (!e.ok()) return e;
    *graph_exec = ge;
    return Error::None();
}

Error GPUEngine::ReplayGraph(void* graph_exec) {
    if (!graph_exec) return Error{"ReplayGraph: nil graph"};
    return cuda_err(cudaGraphLaunch((cudaGraphExec_t)graph_exec, (cudaStream_t)stream_), "cudaGraphLaunch");
}

Error GPUEngine::DestroyGraph(void* graph_exec) {
    if (!graph_exec) return Error::None();
    return cuda_err(cudaGraphExecDestroy((cudaGraphExec_t)graph_exec), "cudaGraphExecDestroy");
}

Error GPUEngine::NewDeviceTensor(const std::vector<int>& shape, bool f16, Tensor* out) {
    size_t n = 1;
    for (int d : shape) {
        if (d <= 0) return Error{"NewDeviceTensor: dimensions must be positive"};
        n *= (size_t)d;
    }
    const size_t bytes = n * (f16 ? 2 : 4);
    void* p = nullptr;
    Error e = pool_->Alloc(bytes, &p, capturing_);
    if (!e.ok()) return e;
    out->shape = shape;
    out->storage = GPUStorage::FromPool(p, n, f16, device_, pool_.get(), bytes);
    return Error::None();
}

Error GPUEngine::CopyFromHost(const Tensor& t, const void* host, size_t bytes) {
    if (!t.storage || t.storage->kind() != Kind::GPU || !t.storage->GPUPtr()) return Error{"CopyFromHost: not a device tensor"};
    if (bytes > t.storage->GPUByteSize()) return Error{"CopyFromHost: more bytes than the tensor holds"};
    return cuda_err(cudaMemcpyAsync(t.storage->GPUPtr(), host, bytes, cudaMemcpyHostToDevice, (cudaStream_t)stream_), "cudaMemcpy H2D");
}

Error GPUEngine::CopyToHost(const Tensor& t, void* host, size_t bytes) {
    if (!t.storage || t.storage->kind() != Kind::GPU || !t.storage->GPUPtr()) return Error{"CopyToHost: not a device tensor"};
    if (bytes > t.storage->GPUByteSize()) return Error{"CopyToHost: more bytes than the tensor holds"};
    return cuda_err(cudaMemcpyAsync(host, t.storage->GPUPtr(), bytes, cudaMemcpyDeviceToHost, (cudaStream_t)stream_), "cudaMemcpy D2H");
}

Error GPUEngine::Sync() { return cuda_err(cudaStreamSynchronize((cudaStream_t)stream_), "cudaStreamSynchronize"); }

namespace {
struct DevBuf {                       // scoped device allocation
    void* p = nullptr;
    ~DevBuf() { if (p) cudaFree(p); }
    Error alloc(size_t n) { return cuda_err(cudaMalloc(&p, n ? n : 1), "cudaMalloc"); }
};
}  // namespace

Error GPUEngine::QuantizeQ4(const float* src, size_t n, std::shared_ptr<Q4Storage>* out) {
    if (n == 0 || n % 32) return Error{"QuantizeQ4: the device quantizer takes a multiple of 32 elements, got " + std::to_string(n)};
    cudaSetDevice(device_);
    auto st = (cudaStream_t)stream_;
    const size_t nb = n / 32, off = Q4GPUDataOffset(nb);
    DevBuf dsrc, dsep;
    Error e;
    if (!(e = dsrc.alloc(n * 4)).ok() || !(e = dsep.alloc(off + nb * 16)).ok()) return e;
    if (!(e = cuda_err(cudaMemcpyAsync(dsrc.p, src, n * 4, cudaMemcpyHostToDevice, st), "cudaMemcpy H2D")).ok()) return e;
    if (!(e = kernel_err(ztq_quantize_q4_0((const float*)dsrc.p, dsep.p, (long long)n, st), "ztq_quantize_q4_0")).ok()) return e;
    ++launches;
    std::vector<uint8_t> sep(off + nb * 16);
    if (!(e = cuda_err(cudaMemcpyAsync(sep.data(), dsep.p, sep.size(), cudaMemcpyDeviceToHost, st), "cudaMemcpy D2H")).ok()) return e;
    if (!(e = Sync()).ok()) return e;
    auto s = std::make_shared<Q4Storage>();
    s->blocks.resize(nb * 18);
    s->len = n;
    for (size_t i = 0; i < nb; ++i) {
        s->blocks[18 * i] = sep[2 * i];
        s->blocks[18 * i + 1] = sep[2 * i + 1];
        memcpy(&s->blocks[18 * i + 2], &sep[off + 16 * i], 16);
    }
    *out = s;
    return Error::None();
}

Error GPUEngine::QuantizeQ8(const float* src, size_t n, std::shared_ptr<Q8Storage>* out) {
    if (n == 0 || n % 32) return Error{"QuantizeQ8: the device quantizer takes a multiple of 32 elements, got " + std::to_string(n)};
    cudaSetDevice(device_);
    auto st = (cudaStream_t)stream_;
    DevBuf dsrc, dq;
    Error e;
    if (!(e = dsrc.alloc(n * 4)).ok() || !(e = dq.alloc(n / 32 * 36)).ok()) return e;
    if (!(e = cuda_err(cudaMemcpyAsync(dsrc.p, src, n * 4, cudaMemcpyHostToDevice, st), "cudaMemcpy H2D")).ok()) return e;
    if (!(e = kernel_err(ztq_quantize_q8_0((const float*)dsrc.p, dq.p, (long long)n, st), "ztq_quantize_q8_0")).ok()) return e;
    ++launches;
    auto s = std::make_shared<Q8Storage>();
    s->blocks.resize(n / 32 * 36);
    s->len = n;
    if (!(e = cuda_err(cudaMemcpyAsync(s->blocks.data(), dq.p, s->blocks.size(), cudaMemcpyDeviceToHost, st), "cudaMemcpy D2H")).ok()) return e;
    if (!(e = Sync()).ok()) return e;
    *out = s;
    return Error::None();
}

static Error quantize_group(GPUEngine& g, void* stream, int device, const float* src, size_t n, int group, bool awq,
                            std::shared_ptr<GroupQuantStorage>* out) {
    if (group <= 0 || group % 2 || n == 0 || n % group)
        return Error{"group quantizer: the element count must be a positive multiple of an even group size"};
    cudaSetDevice(device);
    auto st = (cudaStream_t)stream;
    const size_t ng = n / group;
    DevBuf dsrc, dq, dm;
    Error e;
    if (!(e = dsrc.alloc(n * 4)).ok() || !(e = dq.alloc(n / 2)).ok() || !(e = dm.alloc(ng * 4)).ok()) return e;
    if (!(e = cuda_err(cudaMemcpyAsync(dsrc.p, src, n * 4, cudaMemcpyHostToDevice, st), "cudaMemcpy H2D")).ok()) return e;
    if (!(e = kernel_err(ztq_quantize_w4g((const float*)dsrc.p, dq.p, dm.p, (long long)n, group, awq ? 1 : 0, st), "ztq_quantize_w4g")).ok()) return e;
    ++g.launches;
    auto s = std::make_shared<GroupQuantStorage>(awq);
    s->data.resize(n / 2);
    s->len = n;
    s->group_size = group;
    std::vector<uint32_t> meta(ng);
    if (!(e = cuda_err(cudaMemcpyAsync(s->data.data(), dq.p, n / 2, cudaMemcpyDeviceToHost, st), "cudaMemcpy D2H")).ok()) return e;
    if (!(e = cuda_err(cudaMemcpyAsync(meta.data(), dm.p, ng * 4, cudaMemcpyDeviceToHost, st), "cudaMemcpy D2H")).ok()) return e;
    if (!(e = g.Sync()).ok()) return e;
    s->scales.resize(ng);
    s->zeros.resize(ng);
    for (size_t i = 0; i < ng; ++i) {
        s->scales[i] = (uint16_t)(meta[i] & 0xffff);
        s->zeros[i] = (uint16_t)(meta[i] >> 16);
    }
    *out = s;
    return Error::None();
}

Error GPUEngine::QuantizeGPTQ(const float* src, size_t n, int group_size, int bits, std::shared_ptr<GroupQuantStorage>* out) {
    if (bits != 4) return Error{"QuantizeGPTQ: only the 4-bit path is implemented"};
    return quantize_group(*this, stream_, device_, src, n, group_size, false, out);
}
Error GPUEngine::QuantizeAWQ(const float* src, size_t n, int group_size, std::shared_ptr<GroupQuantStorage>* out) {
    return quantize_group(*this, stream_, device_, src, n, group_size, true, out);
}

// Residency layouts on the device (the GPUPtr of each storage):
//   Q4 / IQ4NL   separated layout (RawBytesGPU); data region at Q4GPUDataOffset(NumBlocks)
//   Q8           RawBytes
//   GPTQ / AWQ   [nibbles: Len/2 bytes][pad to 256][half2 {scale, zero} per group]
//   Ternary      rows x ceil(cols/4) bytes, every row byte aligned
//   Float16      raw little-endian binary16
Error GPUEngine::upload_one(Storage* s, int rows, int cols) {
    if (s->GPUPtr()) return Error::None();
    cudaSetDevice(device_);
    auto st = (cudaStream_t)stream_;
    Error e;
    void* dev = nullptr;
    size_t bytes = 0;
    switch (s->kind()) {
        case Kind::Q4K:
        case Kind::Q5K:
        case Kind::Q6K: {                                      // 144 / 176 / 210-byte super-blocks -> side bytes, then nibbles
            const bool q5 = s->kind() == Kind::Q5K, q6 = s->kind() == Kind::Q6K;
            const auto& aos = q6 ? static_cast<Q6KStorage*>(s)->raw : q5 ? static_cast<Q5KStorage*>(s)->raw : static_cast<Q4KStorage*>(s)->raw;
            const size_t nb = (s->Len() + 255) / 256;
            if (s->Len() % 256) return Error{"UploadWeights: K-quant tensors must hold whole super-blocks of 256"};
            bytes = nb * (q6 ? 224 : q5 ? 176 : 144);
            DevBuf tmp;
            if (!(e = tmp.alloc(aos.size())).ok()) return e;
            if (!(e = cuda_err(cudaMalloc(&dev, bytes), "cudaMalloc")).ok()) return e;
            if (!(e = cuda_err(cudaMemcpyAsync(tmp.p, aos.data(), aos.size(), cudaMemcpyHostToDevice, st), "cudaMemcpy H2D")).ok()) return e;
            if (!(e = q6 ? kernel_err(ztq_repack_blocks210(tmp.p, dev, (long long)nb, st), "ztq_repack_blocks210")
                      : q5 ? kernel_err(ztq_repack_blocks176(tmp.p, dev, (long long)nb, st), "ztq_repack_blocks176")
                         : kernel_err(ztq_repack_blocks144(tmp.p, dev, (long long)nb, st), "ztq_repack_blocks144")).ok()) return e;
            ++launches;
            if (!(e = Sync()).ok()) return e;
            break;
        }
        case Kind::Q4:
        case Kind::IQ4NL: {
            const auto& aos = s->kind() == Kind::Q4 ? static_cast<Q4Storage*>(s)->blocks : static_cast<IQ4NLStorage*>(s)->raw;
            const size_t nb = (s->Len() + 31) / 32;
            bytes = Q4GPUDataOffset(nb) + nb * 16;
            DevBuf tmp;
            if (!(e = tmp.alloc(aos.size())).ok()) return e;
            if (!(e = cuda_err(cudaMalloc(&dev, bytes), "cudaMalloc")).ok()) return e;
            cudaMemsetAsync(dev, 0, bytes, st);
            if (!(e = cuda_err(cudaMemcpyAsync(tmp.p, aos.data(), aos.size(), cudaMemcpyHostToDevice, st), "cudaMemcpy H2D")).ok()) return e;
            if (!(e = kernel_err(ztq_repack_blocks18(tmp.p, dev, (long long)nb, st), "ztq_repack_blocks18")).ok()) return e;
            ++launches;
            if (!(e = Sync()).ok()) return e;
            break;
        }
        case Kind::Q8: {
            auto* q = static_cast<Q8Storage*>(s);
            bytes = q->blocks.size();
            if (!(e = cuda_err(cudaMalloc(&dev, bytes), "cudaMalloc")).ok()) return e;
            if (!(e = cuda_err(cudaMemcpyAsync(dev, q->blocks.data(), bytes, cudaMemcpyHostToDevice, st), "cudaMemcpy H2D")).ok()) return e;
            if (!(e = Sync()).ok()) return e;
            break;
        }
        case Kind::GPTQ:
        case Kind::AWQ: {
            auto* q = static_cast<GroupQuantStorage*>(s);
            if (q->len % q->group_size) return Error{"UploadWeights: GPTQ/AWQ length must be a multiple of the group size"};
            const size_t ng = q->NumGroups(), moff = align256(q->data.size());
            q->gpu_meta_off = moff;
            bytes = moff + ng * 4;
            DevBuf ts, tz;
            if (!(e = ts.alloc(ng * 2)).ok() || !(e = tz.alloc(ng * 2)).ok()) return e;
            if (!(e = cuda_err(cudaMalloc(&dev, bytes), "cudaMalloc")).ok()) return e;
            cudaMemcpyAsync(dev, q->data.data(), q->data.size(), cudaMemcpyHostToDevice, st);
            cudaMemcpyAsync(ts.p, q->scales.data(), ng * 2, cudaMemcpyHostToDevice, st);
            cudaMemcpyAsync(tz.p, q->zeros.data(), ng * 2, cudaMemcpyHostToDevice, st);
            if (!(e = kernel_err(ztq_pack_w4g_meta(ts.p, tz.p, (uint8_t*)dev + moff, (long long)ng, st), "ztq_pack_w4g_meta")).ok()) return e;
            ++launches;
            if (!(e = Sync()).ok()) return e;
            break;
        }
        case Kind::Ternary: {
            auto* t = static_cast<TernaryStorage*>(s);
            if (rows <= 0 || cols <= 0 || (size_t)rows * cols != t->len)
                return Error{"UploadWeights: ternary weights need a 2-D shape matching their length"};
            bytes = (size_t)rows * ((cols + 3) / 4);
            DevBuf flat;
            if (!(e = flat.alloc(t->data.size())).ok()) return e;
            if (!(e = cuda_err(cudaMalloc(&dev, bytes), "cudaMalloc")).ok()) return e;
            cudaMemcpyAsync(flat.p, t->data.data(), t->data.size(), cudaMemcpyHostToDevice, st);
            if (!(e = kernel_err(ztq_repack_ternary_rows(flat.p, dev, rows, cols, st), "ztq_repack_ternary_rows")).ok()) return e;
            ++launches;
            if (!t->row_scale.empty()) {
                if (t->row_scale.size() != (size_t)rows) return Error{"UploadWeights: one row scale per output row expected"};
                if (!(e = cuda_err(cudaMalloc(&t->gpu_row_scale, rows * 2), "cudaMalloc")).ok()) return e;
                cudaMemcpyAsync(t->gpu_row_scale, t->row_scale.data(), rows * 2, cudaMemcpyHostToDevice, st);
            }
            if (!(e = Sync()).ok()) return e;
            break;
        }
        case Kind::Float16: {
            auto* f = static_cast<Float16Storage*>(s);
            bytes = f->data.size();
            if (!(e = cuda_err(cudaMalloc(&dev, bytes ? bytes : 1), "cudaMalloc")).ok()) return e;
            if (!(e = cuda_err(cudaMemcpyAsync(dev, f->data.data(), bytes, cudaMemcpyHostToDevice, st), "cudaMemcpy H2D")).ok()) return e;
            if (!(e = Sync()).ok()) return e;
            break;
        }
        default:
            return Error::None();                              // float32 tensors: nothing to pack
    }
    s->SetGPUPtr(dev, bytes, device_);
    s->owns_gpu = true;
    return Error::None();
}

std::shared_ptr<GroupQuantStorage> NewGroupQuantStorageOnDevice(void* dev, size_t dev_bytes, size_t meta_off, long long n, int group_size,
                                                                bool awq, int device) {
    if (!dev || n <= 0 || group_size <= 0 || n % group_size || meta_off < (size_t)n / 2 || (meta_off & 15) ||
        dev_bytes < meta_off + (size_t)(n / group_size) * 4)
        return nullptr;
    auto s = std::make_shared<GroupQuantStorage>(awq);
    s->len = (size_t)n;
    s->group_size = group_size;
    s->gpu_meta_off = meta_off;
    s->SetGPUPtr(dev, dev_bytes, device);
    s->owns_gpu = false;
    return s;
}

Error GPUEngine::UploadWeights(const std::vector<Tensor*>& tensors) {
    for (Tensor* t : tensors) {
        if (!t || !t->storage) return Error{"UploadWeights: nil tensor"};
        const int rows = t->shape.size() == 2 ? t->shape[0] : 0, cols = t->shape.size() == 2 ? t->shape[1] : 0;
        Error e = upload_one(t->storage.get(), rows, cols);
        if (!e.ok()) return e;
    }
    return Error::None();
}

// Device pointer of the activation operand (getDevicePtr, compute/gpu_kernels.go:126): resident storages are
// used in place; host storages are staged through a pool buffer for this op (returned in `staged`; the caller
// gives it back to the pool once its kernel is enqueued -- the stream orders the reuse).
Error GPUEngine::activation_ptr(const Tensor& act, size_t elems, const void** ptr, bool* f32, void** staged, size_t* staged_bytes) {
    *staged = nullptr;
    *staged_bytes = 0;
    Storage* s = act.storage.get();
    if (s->Len() < elems) return Error{"activation storage is shorter than its shape"};
    auto st = (cudaStream_t)stream_;
    const void* host = nullptr;
    switch (s->kind()) {
        case Kind::GPU: {
            auto* g = static_cast<GPUStorage*>(s);
            if (!g->GPUPtr()) return Error{"MatMul: the activation storage has been freed"};
            *ptr = g->GPUPtr();
            *f32 = !g->f16;
            return Error::None();
        }
        case Kind::Float16: {
            auto* f = static_cast<Float16Storage*>(s);
            *f32 = false;
            if (f->GPUPtr()) { *ptr = f->GPUPtr(); return Error::None(); }
            host = f->data.data();
            *staged_bytes = elems * 2;
            break;
        }
        case Kind::CPU:
            *f32 = true;
            host = static_cast<CPUStorage*>(s)->data.data();
            *staged_bytes = elems * 4;
            break;
        default:
            return Error{"MatMul: the activation operand must be float32, Float16Storage or GPUStorage"};
    }
    if (capturing_) return Error{"MatMul: host activations cannot be staged during stream capture (make them device tensors first)"};
    Error e = pool_->Alloc(*staged_bytes, staged);
    if (!e.ok()) return e;
    *ptr = *staged;
    // pageable host memory: the copy is staged by the driver before the call returns, the host vector may change after it
    return cuda_err(cudaMemcpyAsync(*staged, host, *staged_bytes, cudaMemcpyHostToDevice, st), "cudaMemcpy H2D");
}

// One quantized GEMV / skinny GEMM: everything is enqueued on the engine's stream and the call returns without
// waiting (compute/gpu_engine_matmul.go:89-100: output from the pool, no synchronisation), unless the caller asked
// for the result in host memory (a CPUStorage dst), which needs the copy to be complete.
Error GPUEngine::quant_gemv(const Storage& w_const, int n, int k, const Tensor& act, bool act_is_kb, int batch,
                            Tensor* result, Tensor* dst, const std::vector<int>& out_shape) {
    Storage& w = const_cast<Storage&>(w_const);
    if ((size_t)n * k != w.Len())
        return Error{"MatMul: weight storage holds " + std::to_string(w.Len()) + " elements, shape needs " + std::to_string((size_t)n * k)};
    cudaSetDevice(device_);
    auto st = (cudaStream_t)stream_;
    Error e;
    if (!w.GPUPtr()) {
        if (capturing_) return Error{"MatMul: weights must be uploaded (UploadWeights) before stream capture"};
        if (!(e = upload_one(&w, n, k)).ok()) return e;        // no-op when UploadWeights ran
    }
    const void* xptr = nullptr;
    bool xf32 = false;
    void* xstaged = nullptr;
    size_t xstaged_bytes = 0;
    if (!(e = activation_ptr(act, (size_t)batch * k, &xptr, &xf32, &xstaged, &xstaged_bytes)).ok()) {
        pool_->Free(xstaged, xstaged_bytes);
        return e;
    }

    // output: dst's own device buffer when it has one of the right size, else a buffer from the pool
    const size_t out_elems = (size_t)n * batch;
    void* yptr = nullptr;
    bool y_pooled = false;
    GPUStorage* dst_gpu = nullptr;
    auto give_back = [&]() {
        pool_->Free(xstaged, xstaged_bytes);
        if (y_pooled) pool_->Free(yptr, out_elems * 4);
    };
    if (dst && dst->storage && dst->storage->kind() == Kind::GPU) {
        dst_gpu = static_cast<GPUStorage*>(dst->storage.get());
        if (dst_gpu->f16 || dst_gpu->Len() != out_elems || !dst_gpu->GPUPtr()) { give_back(); return Error{"MatMul: dst storage does not match the result size"}; }
        yptr = dst_gpu->GPUPtr();
    } else {
        if (dst && dst->storage && (dst->storage->kind() != Kind::CPU || dst->storage->Len() != out_elems)) {
            give_back();
            return Error{"MatMul: dst storage does not match the result size"};
        }
        if (!(e = pool_->Alloc(out_elems * 4, &yptr, capturing_)).ok()) { give_back(); return e; }
        y_pooled = true;
    }
    int flags = ZTQ_Y_F32 | (xf32 ? ZTQ_X_F32 : 0) | (act_is_kb ? (ZTQ_X_KB | ZTQ_Y_NB) : 0);
    cudaError_t ce = cudaSuccess;
    const char* name = "";
    const uint8_t* wp = (const uint8_t*)w.GPUPtr();
    void* tc_ws = nullptr;
    size_t tc_ws_bytes = 0;
    switch (w.kind()) {
        case Kind::Q4:
            // three or more fp16 activation rows: the tensor-core kernel (the reference transposes around its tile
            // kernel here, compute/gpu_engine.go:2166-2203)
            if (batch >= 3 && !xf32 && !act_is_kb && k % 512 == 0 && w.Len() % 32 == 0) {
                tc_ws_bytes = ztq_gemm_q4_0_tc_workspace_bytes(n, k, batch);
                if (!(e = pool_->Alloc(tc_ws_bytes, &tc_ws, capturing_)).ok()) { give_back(); return e; }
                name = "ztq_gemm_q4_0_tc";
                ce = ztq_gemm_q4_0_tc(wp, (int)Q4GPUDataOffset(w.Len() / 32), xptr, yptr, n, k, batch, tc_ws, tc_ws_bytes, ZTQ_Y_F32, st);
                pool_->Free(tc_ws, tc_ws_bytes);
                break;
            }
            name = "ztq_gemv_q4_0";
            ce = ztq_gemv_q4_0(wp, (int)Q4GPUDataOffset((w.Len() + 31) / 32), xptr, yptr, n, k, batch, flags, st);
            break;
        case Kind::IQ4NL:
            name = "ztq_gemv_iq4nl";
            ce = ztq_gemv_iq4nl(wp, (int)Q4GPUDataOffset((w.Len() + 31) / 32), xptr, yptr, n, k, batch, flags, st);
            break;
        case Kind::Q4K:
        case Kind::Q5K:
        case Kind::Q6K: {                                      // Q5_K / Q6_K: B side only in the reference (cpu_engine.go:2475-2489)
            if (act_is_kb && batch > 1) {
                give_back();
                return Error{std::string("MatMul: ") + (w.kind() == Kind::Q4K ? "Q4_K" : w.kind() == Kind::Q5K ? "Q5_K" : "Q6_K") +
                             " weights on the A side take one activation column"};
            }
            const int side = w.kind() == Kind::Q4K ? 16 : w.kind() == Kind::Q5K ? 48 : 96;
            const long long off = (long long)((w.Len() + 255) / 256) * side;
            const int kf = ZTQ_Y_F32 | (xf32 ? ZTQ_X_F32 : 0);
            if (w.kind() == Kind::Q4K) { name = "ztq_gemv_q4k"; ce = ztq_gemv_q4k(wp, off, xptr, yptr, n, k, batch, kf, st); }
            else if (w.kind() == Kind::Q5K) { name = "ztq_gemv_q5k"; ce = ztq_gemv_q5k(wp, off, xptr, yptr, n, k, batch, kf, st); }
            else { name = "ztq_gemv_q6k"; ce = ztq_gemv_q6k(wp, off, xptr, yptr, n, k, batch, kf, st); }
            break;
        }
        case Kind::Q8:
            // three or more fp16 activation rows: the tensor-core kernel on the same 36-byte blocks (the reference
            // runs its tile kernel here, internal/cuda/kernels/gemm_q8.cu:113-152)
            if (batch >= 3 && !xf32 && !act_is_kb && k % 512 == 0 && w.Len() % 32 == 0) {
                tc_ws_bytes = ztq_gemm_q8_0_tc_workspace_bytes(n, k, batch);
                if (!(e = pool_->Alloc(tc_ws_bytes, &tc_ws, capturing_)).ok()) { give_back(); return e; }
                name = "ztq_gemm_q8_0_tc";
                ce = ztq_gemm_q8_0_tc(wp, xptr, yptr, n, k, batch, tc_ws, tc_ws_bytes, ZTQ_Y_F32, st);
                pool_->Free(tc_ws, tc_ws_bytes);
                break;
            }
            name = "ztq_gemv_q8_0";
            ce = ztq_gemv_q8_0(wp, xptr, yptr, n, k, batch, flags, st);
            break;
        case Kind::GPTQ:
        case Kind::AWQ: {
            auto& q = static_cast<GroupQuantStorage&>(w);
            // three or more fp16 activation rows: the tensor-core kernel (one pass over the weights per 32 rows,
            // the GEMV makes one per 2 rows); its workspace comes from the pool and goes back once the launch is
            // enqueued (the stream orders the reuse)
            if (batch >= 3 && !xf32 && !act_is_kb && q.group_size == 128 && k % 512 == 0) {
                tc_ws_bytes = ztq_gemm_w4g_tc_workspace_bytes(n, k, batch);
                if (!(e = pool_->Alloc(tc_ws_bytes, &tc_ws, capturing_)).ok()) { give_back(); return e; }
                name = "ztq_gemm_w4g_tc";
                ce = ztq_gemm_w4g_tc(wp, wp + q.gpu_meta_off, xptr, yptr, n, k, q.group_size, batch, tc_ws, tc_ws_bytes,
                                     ZTQ_Y_F32, st);
                pool_->Free(tc_ws, tc_ws_bytes);
                break;
            }
            name = "ztq_gemv_w4g";
            ce = ztq_gemv_w4g(wp, wp + q.gpu_meta_off, xptr, yptr, n, k, q.group_size, batch, flags, st);
            break;
        }
        case Kind::Ternary: {
            auto& t = static_cast<TernaryStorage&>(w);
            if (k % 64 == 0) {
                name = "ztq_gemv_ternary";
                ce = ztq_gemv_ternary(wp, t.gpu_row_scale, xptr, yptr, n, k, batch, flags, st);
            } else if (batch == 1 && xf32 && !t.gpu_row_scale) {
                name = "ternary_gemv_f32";
                ce = ternary_gemv_f32(wp, (const float*)xptr, (float*)yptr, n, k, st);
            } else {
                give_back();
                return Error{"MatMul: ternary rows that are not a multiple of 64 wide take one float32 vector and no row scale"};
            }
            break;
        }
        default:
            give_back();
            return Error{"MatMul: unsupported weight storage"};
    }
    ++launches;
    if (!(e = kernel_err(ce, name)).ok()) { give_back(); return e; }   // no CPU fallback: the caller decides
    pool_->Free(xstaged, xstaged_bytes);                               // staged activations: reusable in stream order
    xstaged = nullptr;

    if (dst && dst->storage && dst->storage->kind() == Kind::CPU) {    // the result is wanted in host memory: copy and wait
        if (capturing_) { give_back(); return Error{"MatMul: a host dst cannot be filled during stream capture"}; }
        auto* c = static_cast<CPUStorage*>(dst->storage.get());
        e = cuda_err(cudaMemcpyAsync(c->data.data(), yptr, out_elems * 4, cudaMemcpyDeviceToHost, st), "cudaMemcpy D2H");
        if (e.ok()) e = Sync();
        give_back();
        if (!e.ok()) return e;
        dst->shape = out_shape;
        if (result) *result = *dst;
        return Error::None();
    }
    if (dst_gpu) {
        dst->shape = out_shape;
        if (result) *result = *dst;
        return Error::None();
    }
    if (result) {
        result->shape = out_shape;
        result->storage = GPUStorage::FromPool(yptr, out_elems, false, device_, pool_.get(), out_elems * 4);
    } else {
        pool_->Free(yptr, out_elems * 4);
    }
    return Error::None();
}

Error GPUEngine::MatMul(const Tensor& a, const Tensor& b, Tensor* result, Tensor* dst) {
    if (!a.storage || !b.storage) return Error{"input tensors cannot be nil"};
    if (a.shape.size() < 2 || b.shape.size() < 2) return Error{"tensors must have at least 2 dimensions"};
    const int ak = a.shape.back(), bk = b.shape[b.shape.size() - 2];
    if (ak != bk)
        return Error{"invalid shapes for matrix multiplication: a.Shape()=" + fmt_shape(a.shape) + ", b.Shape()=" +
                     fmt_shape(b.shape) + " (inner dimensions " + std::to_string(ak) + " != " + std::to_string(bk) + ")"};
    const Kind ka = a.storage->kind(), kb = b.storage->kind();
    if (is_quant(ka)) {
        // weights on A: [N, K] @ [K, batch] -> [N, batch]
        if (a.shape.size() != 2 || b.shape.size() != 2) return Error{"MatMul: a quantized A operand takes 2-D operands"};
        const int n = a.shape[0], k = a.shape[1], batch = b.shape[1];
        return quant_gemv(*a.storage, n, k, b, true, batch, result, dst, {n, batch});
    }
    if (is_quant(kb)) {
        // weights on B behind a virtual transpose: logical [K, N], stored [N, K]; a is [..., K]
        if (b.shape.size() != 2) return Error{"MatMul: a quantized B operand must be 2-D"};
        const int k = b.shape[0], n = b.shape[1];
        long long batch = 1;
        for (size_t i = 0; i + 1 < a.shape.size(); ++i) batch *= a.shape[i];
        std::vector<int> out_shape(a.shape.begin(), a.shape.end() - 1);
        out_shape.push_back(n);
        return quant_gemv(*b.storage, n, k, a, false, (int)batch, result, dst, out_shape);
    }
    return Error{"MatMul: neither operand is a quantized weight; the dense float32 path is not part of this engine"};
}

// ---------------------------------------------------------------------------- W4A16
std::string QuantFormat(const Storage& s) {
    switch (s.kind()) {
        case Kind::Q4: return "Q4_0";
        case Kind::GPTQ: return "GPTQ_4";
        case Kind::AWQ: return "AWQ";
        default: return "";
    }
}

bool IsW4A16(const Tensor& a, const Tensor& b) {
    if (!a.storage || !b.storage) return false;
    return (is_w4(a.storage->kind()) && b.storage->kind() == Kind::Float16) ||
           (is_w4(b.storage->kind()) && a.storage->kind() == Kind::Float16);
}

Error GPUEngine::MatMulW4A16(const Tensor& a, const Tensor& b, Tensor* result, Tensor* dst) {
    if (!IsW4A16(a, b)) return Error{"MatMulW4A16: inputs are not W4A16 — need 4-bit weights and FP16 activations"};
    if (is_w4(a.storage->kind())) return MatMul(a, b, result, dst);       // weights on A: [N, K] x [K, batch]
    return w4a16_b_literal(a, b, result, dst);                            // weights on B: a literal [K, N] matrix
}

// compute.MatMulW4A16 with the weights as the B operand (compute/w4a16.go:107-119): w4.Slice() becomes a plain
// float32 tensor of b's shape [K, N] and CPUEngine.MatMul multiplies act [M, K] by it.  Here: dequantize on the
// device (bit-identical to Slice()) into a pool buffer, then the dense kernel that keeps SgemmSimd's order.
Error GPUEngine::w4a16_b_literal(const Tensor& a, const Tensor& b, Tensor* result, Tensor* dst) {
    if (a.shape.size() != 2 || b.shape.size() != 2) return Error{"MatMulW4A16: 2-D operands expected"};
    const int m = a.shape[0], k = a.shape[1], kb = b.shape[0], n = b.shape[1];
    if (k != kb)
        return Error{"invalid shapes for matrix multiplication: a.Shape()=" + fmt_shape(a.shape) + ", b.Shape()=" + fmt_shape(b.shape) +
                     " (inner dimensions " + std::to_string(k) + " != " + std::to_string(kb) + ")"};
    Storage& w = *b.storage;
    if ((size_t)k * n != w.Len()) return Error{"MatMulW4A16: weight storage does not match its shape"};
    if (capturing_ && !w.GPUPtr()) return Error{"MatMulW4A16: weights must be uploaded before stream capture"};
    cudaSetDevice(device_);
    auto st = (cudaStream_t)stream_;
    Error e = upload_one(&w, k, n);
    if (!e.ok()) return e;
    const void* xptr = nullptr;
    bool xf32 = false;
    void* xstaged = nullptr;
    size_t xstaged_bytes = 0;
    if (!(e = activation_ptr(a, (size_t)m * k, &xptr, &xf32, &xstaged, &xstaged_bytes)).ok()) { pool_->Free(xstaged, xstaged_bytes); return e; }
    const size_t welems = (size_t)k * n, out_elems = (size_t)m * n;
    void* wf = nullptr;
    void* yptr = nullptr;
    auto give_back = [&]() { pool_->Free(xstaged, xstaged_bytes); pool_->Free(wf, welems * 4); pool_->Free(yptr, out_elems * 4); };
    if (!(e = pool_->Alloc(welems * 4, &wf, capturing_)).ok() || !(e = pool_->Alloc(out_elems * 4, &yptr, capturing_)).ok()) { give_back(); return e; }
    const uint8_t* wp = (const uint8_t*)w.GPUPtr();
    cudaError_t ce;
    if (w.kind() == Kind::Q4) {
        if (w.Len() % 32) { give_back(); return Error{"MatMulW4A16: Q4_0 weights must hold whole blocks of 32"}; }
        ce = ztq_dequantize(0, wp, nullptr, (float*)wf, (long long)welems, (int)Q4GPUDataOffset(w.Len() / 32), st);
    } else {
        auto& q = static_cast<GroupQuantStorage&>(w);
        ce = ztq_dequantize(2, wp, wp + q.gpu_meta_off, (float*)wf, (long long)welems, q.group_size, st);
    }
    ++launches;
    if (!(e = kernel_err(ce, "ztq_dequantize")).ok()) { give_back(); return e; }
    ce = ztq_matmul_wkn_f32(xptr, (const float*)wf, (float*)yptr, m, k, n, xf32 ? ZTQ_X_F32 : 0, st);
    ++launches;
    if (!(e = kernel_err(ce, "ztq_matmul_wkn_f32")).ok()) { give_back(); return e; }
    pool_->Free(xstaged, xstaged_bytes);
    pool_->Free(wf, welems * 4);
    xstaged = wf = nullptr;
    const std::vector<int> out_shape{m, n};
    if (dst && dst->storage) {
        if (dst->storage->Len() != out_elems) { give_back(); return Error{"MatMul: dst storage does not match the result size"}; }
        if (dst->storage->kind() == Kind::CPU && !capturing_) {
            auto* c = static_cast<CPUStorage*>(dst->storage.get());
            e = cuda_err(cudaMemcpyAsync(c->data.data(), yptr, out_elems * 4, cudaMemcpyDeviceToHost, st), "cudaMemcpy D2H");
            if (e.ok()) e = Sync();
        } else if (dst->storage->kind() == Kind::GPU && !static_cast<GPUStorage*>(dst->storage.get())->f16 && dst->storage->GPUPtr()) {
            // dst keeps its own buffer (compute/gpu_kernels.go:248-272): copy the result into it
            e = cuda_err(cudaMemcpyAsync(dst->storage->GPUPtr(), yptr, out_elems * 4, cudaMemcpyDeviceToDevice, st), "cudaMemcpy D2D");
        } else {
            e = Error{"MatMul: dst storage does not match the result size"};
        }
        pool_->Free(yptr, out_elems * 4);
        yptr = nullptr;
        if (!e.ok()) return e;
        dst->shape = out_shape;
        if (result) *result = *dst;
        return Error::None();
    }
    if (result) {
        result->shape = out_shape;
        result->storage = GPUStorage::FromPool(yptr, out_elems, false, device_, pool_.get(), out_elems * 4);
    } else {
        pool_->Free(yptr, out_elems * 4);
    }
    return Error::None();
}

Error TryW4A16MatMul(GPUEngine& eng, const Tensor& a, const Tensor& b, Tensor* result, bool* matched, Tensor* dst) {
    *matched = IsW4A16(a, b);
    if (!*matched) return Error::None();
    return eng.MatMulW4A16(a, b, result, dst);
}

Error GPUEngine::ToHost(const Tensor& t, std::vector<float>* out) {
    if (!t.storage) return Error{"nil tensor"};
    if (t.storage->kind() == Kind::CPU) { *out = static_cast<CPUStorage*>(t.storage.get())->data; return Error::None(); }
    if (t.storage->kind() != Kind::GPU) return Error{"ToHost: not a float32 result tensor"};
    auto* g = static_cast<GPUStorage*>(t.storage.get());
    if (g->f16) return Error{"ToHost: fp16 device tensors are not results of this engine"};
    out->resize(g->Len());
    Error e = cuda_err(cudaMemcpyAsync(out->data(), g->GPUPtr(), g->Len() * 4, cudaMemcpyDeviceToHost, (cudaStream_t)stream_), "cudaMemcpy D2H");
    return e.ok() ? Sync() : e;
}

// ---------------------------------------------------------------------------- ternary free function
Error TernaryGEMVGPU(GPUEngine& eng, TernaryStorage& weights, const float* x, int rows, int cols, std::vector<float>* y) {
    if (rows <= 0 || cols <= 0 || (size_t)rows * cols != weights.Len())
        return Error{"TernaryGEMVGPU: rows*cols does not match the weight count"};
    Tensor w{{rows, cols}, std::shared_ptr<Storage>(&weights, [](Storage*) {})};
    Tensor xt{{cols, 1}, std::make_shared<CPUStorage>(std::vector<float>(x, x + cols))};
    Tensor out{{rows, 1}, std::make_shared<CPUStorage>(std::vector<float>((size_t)rows))};
    Error e = eng.MatMul(w, xt, nullptr, &out);
    if (!e.ok()) return e;
    *y = static_cast<CPUStorage*>(out.storage.get())->data;
    return Error::None();
}

}  // namespace ztq
