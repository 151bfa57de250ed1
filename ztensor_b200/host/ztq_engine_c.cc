// ztq_engine_c.cc -- flat C entry points over ztq::GPUEngine so that the parity
// tests (ctypes) and foreign bindings can drive the engine-level API.  Handles
// are opaque pointers; functions that can fail return 0 on success and copy the
// error text into `err`.
#include <cstring>

#include "ztq_engine.h"

using namespace ztq;

namespace {
int fail(const Error& e, char* err, int cap) {
    if (e.ok()) return 0;
    if (err && cap > 0) { strncpy(err, e.msg.c_str(), cap - 1); err[cap - 1] = 0; }
    return 1;
}
Tensor* mk(std::shared_ptr<Storage> s, const int* shape, int rank) {
    auto* t = new Tensor();
    t->shape.assign(shape, shape + rank);
    t->storage = std::move(s);
    return t;
}
}  // namespace

extern "C" {

void* zt_engine_new(int device, char* err, int cap) {
    std::unique_ptr<GPUEngine> g;
    if (fail(GPUEngine::New(device, &g), err, cap)) return nullptr;
    return g.release();
}
void zt_engine_free(void* e) { delete static_cast<GPUEngine*>(e); }
long long zt_engine_launches(void* e) { return static_cast<GPUEngine*>(e)->launches; }

void zt_tensor_free(void* t) { delete static_cast<Tensor*>(t); }
int zt_tensor_kind(void* t) { return (int)static_cast<Tensor*>(t)->storage->kind(); }
int zt_tensor_resident(void* t) { return static_cast<Tensor*>(t)->storage->GPUPtr() != nullptr; }
int zt_tensor_shape(void* t, int* shape, int cap) {
    auto& s = static_cast<Tensor*>(t)->shape;
    for (int i = 0; i < (int)s.size() && i < cap; ++i) shape[i] = s[i];
    return (int)s.size();
}

void* zt_tensor_cpu(const float* data, const int* shape, int rank) {
    size_t n = 1;
    for (int i = 0; i < rank; ++i) n *= shape[i];
    return mk(std::make_shared<CPUStorage>(std::vector<float>(data, data + n)), shape, rank);
}
void* zt_tensor_f16_raw(const uint8_t* raw, const int* shape, int rank) {
    size_t n = 1;
    for (int i = 0; i < rank; ++i) n *= shape[i];
    return mk(NewFloat16StorageFromRaw(raw, n), shape, rank);
}
void* zt_tensor_f16_from_f32(const float* src, const int* shape, int rank) {
    size_t n = 1;
    for (int i = 0; i < rank; ++i) n *= shape[i];
    return mk(NewFloat16StorageFromF32(src, n), shape, rank);
}
void* zt_tensor_q4_raw(const uint8_t* raw, long long raw_len, long long n, const int* shape, int rank, char* err, int cap) {
    std::shared_ptr<Q4Storage> s;
    if (fail(NewQ4StorageFromRaw(raw, (size_t)raw_len, n, &s), err, cap)) return nullptr;
    return mk(s, shape, rank);
}
void* zt_tensor_q8_blocks(const float* scales, const int8_t* quants, long long n_scales, long long n, const int* shape,
                          int rank, char* err, int cap) {
    std::shared_ptr<Q8Storage> s;
    if (fail(NewQ8StorageFromBlocks(scales, quants, (size_t)n_scales, n, &s), err, cap)) return nullptr;
    return mk(s, shape, rank);
}
void* zt_tensor_iq4nl_raw(const uint8_t* raw, long long raw_len, long long n, const int* shape, int rank, char* err, int cap) {
    std::shared_ptr<IQ4NLStorage> s;
    if (fail(NewIQ4NLStorageFromRaw(raw, (size_t)raw_len, n, &s), err, cap)) return nullptr;
    return mk(s, shape, rank);
}
void* zt_tensor_q4k_raw(const uint8_t* raw, long long raw_len, long long n, const int* shape, int rank, char* err, int cap) {
    std::shared_ptr<Q4KStorage> s;
    if (fail(NewQ4KStorageFromRaw(raw, (size_t)raw_len, n, &s), err, cap)) return nullptr;
    return mk(s, shape, rank);
}
void* zt_tensor_q5k_raw(const uint8_t* raw, long long raw_len, long long n, const int* shape, int rank, char* err, int cap) {
    std::shared_ptr<Q5KStorage> s;
    if (fail(NewQ5KStorageFromRaw(raw, (size_t)raw_len, n, &s), err, cap)) return nullptr;
    return mk(s, shape, rank);
}
void* zt_tensor_q6k_raw(const uint8_t* raw, long long raw_len, long long n, const int* shape, int rank, char* err, int cap) {
    std::shared_ptr<Q6KStorage> s;
    if (fail(NewQ6KStorageFromRaw(raw, (size_t)raw_len, n, &s), err, cap)) return nullptr;
    return mk(s, shape, rank);
}
void* zt_tensor_gptq_raw(const uint8_t* data, long long data_len, const uint16_t* scales, const uint16_t* zeros,
                         long long n_groups, long long n, int group, int bits, const int* shape, int rank, char* err, int cap) {
    std::shared_ptr<GroupQuantStorage> s;
    if (fail(NewGPTQStorageFromRaw(data, (size_t)data_len, scales, (size_t)n_groups, zeros, (size_t)n_groups, n, group, bits, &s), err, cap))
        return nullptr;
    return mk(s, shape, rank);
}
void* zt_tensor_awq_raw(const uint32_t* words, long long n_words, const uint16_t* scales, const uint16_t* zeros,
                        long long n_groups, long long n, int group, const int* shape, int rank, char* err, int cap) {
    std::shared_ptr<GroupQuantStorage> s;
    if (fail(NewAWQStorageFromRaw(words, (size_t)n_words, scales, (size_t)n_groups, zeros, (size_t)n_groups, n, group, &s), err, cap))
        return nullptr;
    return mk(s, shape, rank);
}
void* zt_tensor_ternary(const int8_t* values, long long n, const uint16_t* row_scale, long long n_scale, const int* shape,
                        int rank, char* err, int cap) {
    std::shared_ptr<TernaryStorage> s;
    if (fail(NewTernaryStorageFrom(values, (size_t)n, &s), err, cap)) return nullptr;
    if (row_scale && n_scale > 0) s->row_scale.assign(row_scale, row_scale + n_scale);
    return mk(s, shape, rank);
}

// kind: 3 Q4, 4 Q8, 6 GPTQ, 7 AWQ (values of ztq::Kind)
void* zt_quantize(void* eng, int kind, const float* src, long long n, int group, const int* shape, int rank, char* err, int cap) {
    auto* g = static_cast<GPUEngine*>(eng);
    if (kind == (int)Kind::Q4) {
        std::shared_ptr<Q4Storage> s;
        if (fail(g->QuantizeQ4(src, (size_t)n, &s), err, cap)) return nullptr;
        return mk(s, shape, rank);
    }
    if (kind == (int)Kind::Q8) {
        std::shared_ptr<Q8Storage> s;
        if (fail(g->QuantizeQ8(src, (size_t)n, &s), err, cap)) return nullptr;
        return mk(s, shape, rank);
    }
    if (kind == (int)Kind::GPTQ || kind == (int)Kind::AWQ) {
        std::shared_ptr<GroupQuantStorage> s;
        Error e = kind == (int)Kind::GPTQ ? g->QuantizeGPTQ(src, (size_t)n, group, 4, &s) : g->QuantizeAWQ(src, (size_t)n, group, &s);
        if (fail(e, err, cap)) return nullptr;
        return mk(s, shape, rank);
    }
    fail(Error{"zt_quantize: unknown kind"}, err, cap);
    return nullptr;
}

// Packed bytes of a storage: which = 0 main bytes (blocks / data / raw), 1 scales, 2 zeros.  Returns the size.
long long zt_tensor_bytes(void* t, int which, uint8_t* out, long long cap) {
    Storage* s = static_cast<Tensor*>(t)->storage.get();
    const uint8_t* p = nullptr;
    size_t n = 0;
    switch (s->kind()) {
        case Kind::Q4: p = static_cast<Q4Storage*>(s)->blocks.data(); n = static_cast<Q4Storage*>(s)->blocks.size(); break;
        case Kind::Q8: p = static_cast<Q8Storage*>(s)->blocks.data(); n = static_cast<Q8Storage*>(s)->blocks.size(); break;
        case Kind::IQ4NL: p = static_cast<IQ4NLStorage*>(s)->raw.data(); n = static_cast<IQ4NLStorage*>(s)->raw.size(); break;
        case Kind::Q4K: p = static_cast<Q4KStorage*>(s)->raw.data(); n = static_cast<Q4KStorage*>(s)->raw.size(); break;
        case Kind::Q5K: p = static_cast<Q5KStorage*>(s)->raw.data(); n = static_cast<Q5KStorage*>(s)->raw.size(); break;
        case Kind::Q6K: p = static_cast<Q6KStorage*>(s)->raw.data(); n = static_cast<Q6KStorage*>(s)->raw.size(); break;
        case Kind::Ternary: p = static_cast<TernaryStorage*>(s)->data.data(); n = static_cast<TernaryStorage*>(s)->data.size(); break;
        case Kind::Float16: p = static_cast<Float16Storage*>(s)->data.data(); n = static_cast<Float16Storage*>(s)->data.size(); break;
        case Kind::GPTQ:
        case Kind::AWQ: {
            auto* q = static_cast<GroupQuantStorage*>(s);
            if (which == 0) { p = q->data.data(); n = q->data.size(); }
            else if (which == 1) { p = (const uint8_t*)q->scales.data(); n = q->scales.size() * 2; }
            else { p = (const uint8_t*)q->zeros.data(); n = q->zeros.size() * 2; }
            break;
        }
        default: return -1;
    }
    if (out && (long long)n <= cap) memcpy(out, p, n);
    return (long long)n;
}

int zt_upload_weights(void* eng, void** tensors, int n, char* err, int cap) {
    std::vector<Tensor*> v;
    for (int i = 0; i < n; ++i) v.push_back(static_cast<Tensor*>(tensors[i]));
    return fail(static_cast<GPUEngine*>(eng)->UploadWeights(v), err, cap);
}

// mode 0: Engine.MatMul, 1: MatMulW4A16, 2: TryW4A16MatMul (sets *matched).  The result is copied to out_host.
int zt_matmul(void* eng, void* a, void* b, void* dst, int mode, float* out_host, long long out_cap, int* out_shape,
              int* out_rank, int* matched, char* err, int cap) {
    auto* g = static_cast<GPUEngine*>(eng);
    Tensor res;
    Error e;
    bool m = true;
    Tensor* d = static_cast<Tensor*>(dst);
    if (mode == 0) e = g->MatMul(*static_cast<Tensor*>(a), *static_cast<Tensor*>(b), &res, d);
    else if (mode == 1) e = g->MatMulW4A16(*static_cast<Tensor*>(a), *static_cast<Tensor*>(b), &res, d);
    else e = TryW4A16MatMul(*g, *static_cast<Tensor*>(a), *static_cast<Tensor*>(b), &res, &m, d);
    if (matched) *matched = m ? 1 : 0;
    if (fail(e, err, cap)) return 1;
    if (!m) return 0;
    std::vector<float> host;
    if (fail(g->ToHost(res, &host), err, cap)) return 1;
    if ((long long)host.size() > out_cap) return fail(Error{"zt_matmul: output buffer too small"}, err, cap);
    memcpy(out_host, host.data(), host.size() * 4);
    *out_rank = (int)res.shape.size();
    for (size_t i = 0; i < res.shape.size(); ++i) out_shape[i] = res.shape[i];
    return 0;
}

// ---- device-resident tensors, asynchronous MatMul, capture, pool (the parts of the engine a decode loop uses)
void* zt_device_tensor(void* eng, const int* shape, int rank, int f16, char* err, int cap) {
    auto* t = new Tensor();
    if (fail(static_cast<GPUEngine*>(eng)->NewDeviceTensor(std::vector<int>(shape, shape + rank), f16 != 0, t), err, cap)) { delete t; return nullptr; }
    return t;
}
void* zt_tensor_w4g_device(void* dev, long long dev_bytes, long long meta_off, long long n, int group, int awq, int device,
                           const int* shape, int rank, char* err, int cap) {
    auto s = NewGroupQuantStorageOnDevice(dev, (size_t)dev_bytes, (size_t)meta_off, n, group, awq != 0, device);
    if (!s) { fail(Error{"zt_tensor_w4g_device: pointer, sizes or offsets do not describe a resident GPTQ/AWQ weight"}, err, cap); return nullptr; }
    return mk(s, shape, rank);
}
int zt_copy_from_host(void* eng, void* t, const void* host, long long bytes, char* err, int cap) {
    return fail(static_cast<GPUEngine*>(eng)->CopyFromHost(*static_cast<Tensor*>(t), host, (size_t)bytes), err, cap);
}
int zt_copy_to_host(void* eng, void* t, void* host, long long bytes, char* err, int cap) {
    return fail(static_cast<GPUEngine*>(eng)->CopyToHost(*static_cast<Tensor*>(t), host, (size_t)bytes), err, cap);
}
int zt_engine_sync(void* eng, char* err, int cap) { return fail(static_cast<GPUEngine*>(eng)->Sync(), err, cap); }
void* zt_engine_stream(void* eng) { return static_cast<GPUEngine*>(eng)->Stream(); }
unsigned long long zt_tensor_device_ptr(void* t) { return (unsigned long long)static_cast<Tensor*>(t)->storage->GPUPtr(); }

// mode as zt_matmul; nothing is copied and nothing waits: the result tensor (a new handle, or null when !matched)
// lives on the device.
void* zt_matmul_async(void* eng, void* a, void* b, void* dst, int mode, int* matched, char* err, int cap) {
    auto* g = static_cast<GPUEngine*>(eng);
    auto* res = new Tensor();
    Error e;
    bool m = true;
    Tensor* d = static_cast<Tensor*>(dst);
    if (mode == 0) e = g->MatMul(*static_cast<Tensor*>(a), *static_cast<Tensor*>(b), res, d);
    else if (mode == 1) e = g->MatMulW4A16(*static_cast<Tensor*>(a), *static_cast<Tensor*>(b), res, d);
    else e = TryW4A16MatMul(*g, *static_cast<Tensor*>(a), *static_cast<Tensor*>(b), res, &m, d);
    if (matched) *matched = m ? 1 : 0;
    if (fail(e, err, cap) || !m) { delete res; return nullptr; }
    return res;
}
int zt_tensor_to_host(void* eng, void* t, float* out, long long cap_elems, char* err, int cap) {
    std::vector<float> host;
    if (fail(static_cast<GPUEngine*>(eng)->ToHost(*static_cast<Tensor*>(t), &host), err, cap)) return 1;
    if ((long long)host.size() > cap_elems) return fail(Error{"zt_tensor_to_host: output buffer too small"}, err, cap);
    memcpy(out, host.data(), host.size() * 4);
    return 0;
}

int zt_begin_capture(void* eng, char* err, int cap) { return fail(static_cast<GPUEngine*>(eng)->BeginCapture(), err, cap); }
void* zt_end_capture(void* eng, char* err, int cap) {
    void* ge = nullptr;
    if (fail(static_cast<GPUEngine*>(eng)->EndCapture(&ge), err, cap)) return nullptr;
    return ge;
}
int zt_replay_graph(void* eng, void* graph, char* err, int cap) { return fail(static_cast<GPUEngine*>(eng)->ReplayGraph(graph), err, cap); }
int zt_destroy_graph(void* eng, void* graph, char* err, int cap) { return fail(static_cast<GPUEngine*>(eng)->DestroyGraph(graph), err, cap); }

long long zt_pool_driver_allocs(void* eng) { return static_cast<GPUEngine*>(eng)->Pool()->DriverAllocs(); }
long long zt_pool_epoch(void* eng) { return (long long)static_cast<GPUEngine*>(eng)->Pool()->Epoch(); }
void zt_pool_reset(void* eng) { static_cast<GPUEngine*>(eng)->Pool()->Reset(); }
int zt_pool_cached(void* eng, long long* bytes) {
    int n = 0;
    size_t b = 0;
    static_cast<GPUEngine*>(eng)->Pool()->Stats(&n, &b);
    if (bytes) *bytes = (long long)b;
    return n;
}

// GPUStorage ownership (tensor/gpu_storage.go): views share the reference count, the last Free returns the buffer
void* zt_tensor_view(void* t, long long offset_elems, long long len, const int* shape, int rank, char* err, int cap) {
    auto* src = static_cast<Tensor*>(t);
    if (!src->storage || src->storage->kind() != Kind::GPU) { fail(Error{"zt_tensor_view: not a device tensor"}, err, cap); return nullptr; }
    auto v = static_cast<GPUStorage*>(src->storage.get())->View((size_t)offset_elems, (size_t)len);
    if (!v) { fail(Error{"zt_tensor_view: range outside the storage"}, err, cap); return nullptr; }
    return mk(v, shape, rank);
}
int zt_tensor_refcount(void* t) {
    auto* s = static_cast<Tensor*>(t)->storage.get();
    return s && s->kind() == Kind::GPU ? static_cast<GPUStorage*>(s)->RefCount() : -1;
}
void zt_tensor_free_storage(void* t) {
    auto* s = static_cast<Tensor*>(t)->storage.get();
    if (s && s->kind() == Kind::GPU) static_cast<GPUStorage*>(s)->Free();
}

int zt_ternary_gemv_gpu(void* eng, void* w, const float* x, int rows, int cols, float* y, char* err, int cap) {
    auto* t = static_cast<Tensor*>(w);
    if (t->storage->kind() != Kind::Ternary) return fail(Error{"zt_ternary_gemv_gpu: not a ternary tensor"}, err, cap);
    std::vector<float> out;
    if (fail(TernaryGEMVGPU(*static_cast<GPUEngine*>(eng), *static_cast<TernaryStorage*>(t->storage.get()), x, rows, cols, &out), err, cap))
        return 1;
    memcpy(y, out.data(), out.size() * 4);
    return 0;
}

}  // extern "C"
