// ztq_nccl.h -- host-side binding of libnccl.so.2, loaded at run time with dlopen: the C++ mirror of the
// reference's zero-CGo binding (internal/nccl/nccl_purego.go), with the two things the tensor-parallel shard
// path needs that the reference lacks: the 16-bit element types (ncclFloat16 / ncclBfloat16 are missing from its
// DataType, nccl_purego.go:52-59) and an ncclCommInitRank that can be reached with integer-class arguments only.
//
// ncclCommInitRank takes the 128-byte ncclUniqueId BY VALUE.  On AArch64 a caller may pass a pointer instead
// (the reference relies on that, nccl_purego.go:225-247); on System V x86-64 the aggregate travels on the
// stack, which a register-only foreign call (cuda.Ccall) cannot do.  zt_nccl_comm_init_rank below takes the id
// by pointer and makes the by-value call in compiled code: it is the trampoline a pure-Go caller on
// linux/amd64 binds instead of ncclCommInitRank itself.
#pragma once

#include <cstddef>
#include <memory>
#include <string>

#include "ztq_engine.h"

namespace ztq {
namespace nccl {

constexpr int kUniqueIDBytes = 128;

// ncclDataType_t (stable ABI of NCCL 2.x)
enum class DataType : int { Int8 = 0, Uint8 = 1, Int32 = 2, Uint32 = 3, Int64 = 4, Uint64 = 5, Float16 = 6, Float32 = 7, Float64 = 8, Bfloat16 = 9 };
// ncclRedOp_t
enum class ReduceOp : int { Sum = 0, Prod = 1, Max = 2, Min = 3, Avg = 4 };

// Load libnccl (candidates: `path` when given, $ZTQ_NCCL_LIB, libnccl.so.2, libnccl.so).  Idempotent.
Error Load(const char* path = nullptr);
bool Available();
std::string ErrorString(int nccl_result);

struct UniqueID {
    unsigned char id[kUniqueIDBytes];
};
Error GetUniqueID(UniqueID* out);                                   // one rank calls this and sends the bytes to the others
Error UniqueIDFromBytes(const void* bytes, size_t n, UniqueID* out);

class Comm {
  public:
    // The CUDA device of this rank must be current.  All ranks call with the same id and nRanks.
    static Error InitRank(const UniqueID& uid, int n_ranks, int rank, std::unique_ptr<Comm>* out);
    ~Comm();
    // In-place when send == recv.  count in elements.  Asynchronous on `stream` (a cudaStream_t); can be captured.
    Error AllReduce(const void* send, void* recv, size_t count, DataType dtype, ReduceOp op, void* stream);
    Error Broadcast(const void* send, void* recv, size_t count, DataType dtype, int root, void* stream);
    Error GetAsyncError(int* nccl_result);
    Error Destroy();
    int Rank() const { return rank_; }
    int Size() const { return n_ranks_; }

  private:
    Comm() = default;
    void* comm_ = nullptr;
    int rank_ = 0, n_ranks_ = 0;
};

Error GroupStart();
Error GroupEnd();

}  // namespace nccl
}  // namespace ztq
