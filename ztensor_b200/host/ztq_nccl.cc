// ztq_nccl.cc -- see ztq_nccl.h.
#include "ztq_nccl.h"

#include <dlfcn.h>

#include <cstdlib>
#include <cstring>
#include <mutex>

namespace ztq {
namespace nccl {

namespace {

struct IdByValue { char internal[kUniqueIDBytes]; };                 // layout of ncclUniqueId (nccl.h)

struct Lib {
    void* handle = nullptr;
    int (*getUniqueId)(IdByValue*) = nullptr;
    int (*commInitRank)(void**, int, IdByValue, int) = nullptr;      // the id travels by value
    int (*commDestroy)(void*) = nullptr;
    int (*commGetAsyncError)(void*, int*) = nullptr;
    int (*allReduce)(const void*, void*, size_t, int, int, void*, void*) = nullptr;
    int (*broadcast)(const void*, void*, size_t, int, int, void*, void*) = nullptr;
    int (*groupStart)() = nullptr;
    int (*groupEnd)() = nullptr;
    const char* (*getErrorString)(int) = nullptr;
};

Lib g_lib;
std::mutex g_mu;
bool g_loaded = false;
std::string g_load_err = "nccl: not loaded";

template <typename F>
bool sym(void* h, const char* name, F* out, std::string* err) {
    void* p = dlsym(h, name);
    if (!p) { *err = std::string("nccl: dlsym ") + name + " failed"; return false; }
    *out = reinterpret_cast<F>(p);
    return true;
}

}  // namespace

Error Load(const char* path) {
    std::lock_guard<std::mutex> lk(g_mu);
    if (g_loaded) return Error::None();
    const char* env = std::getenv("ZTQ_NCCL_LIB");
    const char* candidates[4] = {path, env, "libnccl.so.2", "libnccl.so"};
    void* h = nullptr;
    std::string last = "no candidate path";
    for (const char* c : candidates) {
        if (!c || !*c) continue;
        h = dlopen(c, RTLD_LAZY | RTLD_GLOBAL);
        if (h) break;
        const char* e = dlerror();
        last = e ? e : "dlopen failed";
    }
    if (!h) { g_load_err = "nccl: dlopen failed: " + last; return Error{g_load_err}; }
    Lib l;
    l.handle = h;
    std::string err;
    if (!sym(h, "ncclGetUniqueId", &l.getUniqueId, &err) || !sym(h, "ncclCommInitRank", &l.commInitRank, &err) ||
        !sym(h, "ncclCommDestroy", &l.commDestroy, &err) || !sym(h, "ncclCommGetAsyncError", &l.commGetAsyncError, &err) ||
        !sym(h, "ncclAllReduce", &l.allReduce, &err) || !sym(h, "ncclBroadcast", &l.broadcast, &err) ||
        !sym(h, "ncclGroupStart", &l.groupStart, &err) || !sym(h, "ncclGroupEnd", &l.groupEnd, &err) ||
        !sym(h, "ncclGetErrorString", &l.getErrorString, &err)) {
        g_load_err = err;
        return Error{err};
    }
    g_lib = l;
    g_loaded = true;
    return Error::None();
}

bool Available() { return Load().ok(); }

std::string ErrorString(int rc) {
    if (g_loaded && g_lib.getErrorString) {
        const char* s = g_lib.getErrorString(rc);
        if (s) return s;
    }
    return "ncclResult=" + std::to_string(rc);
}

namespace {
Error need_lib() {
    Error e = Load();
    return e;
}
Error rc_err(int rc, const std::string& what) {
    if (rc == 0) return Error::None();
    return Error{what + " failed: " + ErrorString(rc)};
}
}  // namespace

Error GetUniqueID(UniqueID* out) {
    Error e = need_lib();
    if (!e.ok()) return e;
    IdByValue id;
    std::memset(&id, 0, sizeof(id));
    e = rc_err(g_lib.getUniqueId(&id), "ncclGetUniqueId");
    if (e.ok()) std::memcpy(out->id, id.internal, kUniqueIDBytes);
    return e;
}

Error UniqueIDFromBytes(const void* bytes, size_t n, UniqueID* out) {
    if (n != (size_t)kUniqueIDBytes) return Error{"UniqueIDFromBytes: expected 128 bytes, got " + std::to_string(n)};
    std::memcpy(out->id, bytes, kUniqueIDBytes);
    return Error::None();
}

Error Comm::InitRank(const UniqueID& uid, int n_ranks, int rank, std::unique_ptr<Comm>* out) {
    Error e = need_lib();
    if (!e.ok()) return e;
    if (n_ranks <= 0 || rank < 0 || rank >= n_ranks) return Error{"nccl InitRank: rank outside [0, nRanks)"};
    IdByValue id;
    std::memcpy(id.internal, uid.id, kUniqueIDBytes);
    void* comm = nullptr;
    e = rc_err(g_lib.commInitRank(&comm, n_ranks, id, rank),
               "ncclCommInitRank(nRanks=" + std::to_string(n_ranks) + ", rank=" + std::to_string(rank) + ")");
    if (!e.ok()) return e;
    std::unique_ptr<Comm> c(new Comm());
    c->comm_ = comm;
    c->rank_ = rank;
    c->n_ranks_ = n_ranks;
    *out = std::move(c);
    return Error::None();
}

Comm::~Comm() { Destroy(); }

Error Comm::Destroy() {
    if (!comm_) return Error::None();
    void* c = comm_;
    comm_ = nullptr;
    return rc_err(g_lib.commDestroy(c), "ncclCommDestroy");
}

Error Comm::AllReduce(const void* send, void* recv, size_t count, DataType dtype, ReduceOp op, void* stream) {
    if (!comm_) return Error{"nccl AllReduce: communicator destroyed"};
    return rc_err(g_lib.allReduce(send, recv, count, (int)dtype, (int)op, comm_, stream), "ncclAllReduce");
}

Error Comm::Broadcast(const void* send, void* recv, size_t count, DataType dtype, int root, void* stream) {
    if (!comm_) return Error{"nccl Broadcast: communicator destroyed"};
    return rc_err(g_lib.broadcast(send, recv, count, (int)dtype, root, comm_, stream), "ncclBroadcast");
}

Error Comm::GetAsyncError(int* result) {
    if (!comm_) return Error{"nccl GetAsyncError: communicator destroyed"};
    return rc_err(g_lib.commGetAsyncError(comm_, result), "ncclCommGetAsyncError");
}

Error GroupStart() {
    Error e = need_lib();
    return e.ok() ? rc_err(g_lib.groupStart(), "ncclGroupStart") : e;
}
Error GroupEnd() {
    Error e = need_lib();
    return e.ok() ? rc_err(g_lib.groupEnd(), "ncclGroupEnd") : e;
}

}  // namespace nccl
}  // namespace ztq

// ---- flat C entry points: every argument an integer-class word, 0 = success, error text copied into `err` ----
using namespace ztq;
namespace {
int nfail(const Error& e, char* err, int cap) {
    if (e.ok()) return 0;
    if (err && cap > 0) { strncpy(err, e.msg.c_str(), cap - 1); err[cap - 1] = 0; }
    return 1;
}
}  // namespace

extern "C" {
int zt_nccl_load(const char* path, char* err, int cap) { return nfail(nccl::Load(path), err, cap); }
int zt_nccl_get_unique_id(void* out128, char* err, int cap) {
    nccl::UniqueID id;
    if (nfail(nccl::GetUniqueID(&id), err, cap)) return 1;
    memcpy(out128, id.id, nccl::kUniqueIDBytes);
    return 0;
}
// The x86-64 trampoline: the 128-byte id by pointer, passed on by value in compiled code.
void* zt_nccl_comm_init_rank(const void* uid128, int n_ranks, int rank, char* err, int cap) {
    nccl::UniqueID id;
    if (nfail(nccl::UniqueIDFromBytes(uid128, nccl::kUniqueIDBytes, &id), err, cap)) return nullptr;
    std::unique_ptr<nccl::Comm> c;
    if (nfail(nccl::Comm::InitRank(id, n_ranks, rank, &c), err, cap)) return nullptr;
    return c.release();
}
int zt_nccl_all_reduce(void* comm, const void* send, void* recv, long long count, int dtype, int op, void* stream, char* err, int cap) {
    return nfail(static_cast<nccl::Comm*>(comm)->AllReduce(send, recv, (size_t)count, (nccl::DataType)dtype, (nccl::ReduceOp)op, stream), err, cap);
}
int zt_nccl_broadcast(void* comm, const void* send, void* recv, long long count, int dtype, int root, void* stream, char* err, int cap) {
    return nfail(static_cast<nccl::Comm*>(comm)->Broadcast(send, recv, (size_t)count, (nccl::DataType)dtype, root, stream), err, cap);
}
int zt_nccl_comm_destroy(void* comm, char* err, int cap) {
    auto* c = static_cast<nccl::Comm*>(comm);
    const int rc = nfail(c->Destroy(), err, cap);
    delete c;
    return rc;
}
int zt_nccl_error_string(int rc, char* out, int cap) {
    const std::string s = nccl::ErrorString(rc);
    if (out && cap > 0) { strncpy(out, s.c_str(), cap - 1); out[cap - 1] = 0; }
    return (int)s.size();
}
}  // extern "C"
