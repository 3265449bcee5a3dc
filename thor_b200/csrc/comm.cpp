// The one collective the path needs: an in-place fp32 allreduce of per-GPU partials (full reductions,
// LayerNorm dgamma / dbeta) over NCCL, for hosts that are not Python.  NCCL is loaded at run time with
// dlopen -- the library links no communication code and single-GPU users never touch it.  The reference
// has no multi-GPU path; there is nothing it replaces.
#include <dlfcn.h>

#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>

#include "common.cuh"

namespace {

struct NcclId {
    char bytes[128];  // ncclUniqueId (NCCL_UNIQUE_ID_BYTES)
};
using NcclComm = void*;

struct NcclApi {
    void* handle = nullptr;
    int (*GetUniqueId)(NcclId*) = nullptr;
    int (*CommInitRank)(NcclComm*, int, NcclId, int) = nullptr;
    int (*AllReduce)(const void*, void*, size_t, int, int, NcclComm, cudaStream_t) = nullptr;
    int (*CommDestroy)(NcclComm) = nullptr;
    int (*GroupStart)() = nullptr;
    int (*GroupEnd)() = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
    std::string error;
};

NcclApi& nccl() {
    static NcclApi api;
    static std::once_flag once;
    std::call_once(once, [] {
        std::string tried;
        const char* env = getenv("THOR_B200_NCCL_LIB");
        for (const char* name : {env, "libnccl.so.2", "libnccl.so"}) {
            if (!name || !*name) continue;
            api.handle = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
            if (api.handle) break;
            tried += std::string(name) + " ";
        }
        if (!api.handle) {
            api.error = "NCCL not found (tried " + tried + "): set THOR_B200_NCCL_LIB";
            return;
        }
        auto sym = [&](const char* n) { return dlsym(api.handle, n); };
        api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(sym("ncclGetUniqueId"));
        api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(sym("ncclCommInitRank"));
        api.AllReduce = reinterpret_cast<decltype(api.AllReduce)>(sym("ncclAllReduce"));
        api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(sym("ncclCommDestroy"));
        api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(sym("ncclGetErrorString"));
        api.GroupStart = reinterpret_cast<decltype(api.GroupStart)>(sym("ncclGroupStart"));
        api.GroupEnd = reinterpret_cast<decltype(api.GroupEnd)>(sym("ncclGroupEnd"));
        if (!api.GetUniqueId || !api.CommInitRank || !api.AllReduce || !api.CommDestroy || !api.GetErrorString || !api.GroupStart || !api.GroupEnd) api.error = "NCCL library lacks a required symbol";
    });
    return api;
}

// Minima and maxima cross the ranks as 32-bit integer keys whose signed order is the float order, with every NaN mapped
// to the key that wins (the largest key for a maximum, the smallest for a minimum): the rule of the reduction seam --
// a NaN in any shard is the result -- which NCCL's own floating-point min / max do not promise.  Decoding needs no flag:
// the winning keys are themselves NaN bit patterns.
__global__ void encodeOrderedKeys(float* values, uint64_t n, int nan_wins_high) {
    const uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float v = values[i];
    const int b = __float_as_int(v);
    int key = b >= 0 ? b : (b ^ 0x7fffffff);
    if (v != v) key = nan_wins_high ? 0x7fffffff : static_cast<int>(0x80000000u);
    reinterpret_cast<int*>(values)[i] = key;
}
__global__ void decodeOrderedKeys(float* values, uint64_t n) {
    const uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int key = reinterpret_cast<const int*>(values)[i];
    values[i] = __int_as_float(key >= 0 ? key : (key ^ 0x7fffffff));
}

int ncclFail(const char* what, int rc) { return tb::fail(THOR_B200_CUDA_ERROR, "%s failed: %s", what, nccl().GetErrorString(rc)); }

}  // namespace

struct thor_b200_comm {
    NcclComm comm = nullptr;
    int nranks = 0, rank = 0;
};

extern "C" {

int thor_b200_comm_unique_id(void* out_id_128_bytes) {
    using namespace tb;
    TB_REQUIRE(out_id_128_bytes != nullptr, "comm_unique_id: null output");
    NcclApi& api = nccl();
    if (!api.error.empty()) return fail(THOR_B200_UNSUPPORTED, "comm_unique_id: %s", api.error.c_str());
    NcclId id;
    if (int rc = api.GetUniqueId(&id)) return ncclFail("ncclGetUniqueId", rc);
    memcpy(out_id_128_bytes, id.bytes, sizeof(id.bytes));
    return THOR_B200_OK;
}

int thor_b200_comm_init(int nranks, int rank, const void* unique_id_128_bytes, thor_b200_comm** out_comm) {
    using namespace tb;
    TB_REQUIRE(out_comm != nullptr && unique_id_128_bytes != nullptr, "comm_init: null argument");
    *out_comm = nullptr;
    TB_REQUIRE(nranks >= 1 && rank >= 0 && rank < nranks, "comm_init: rank %d of %d is out of range", rank, nranks);
    NcclApi& api = nccl();
    if (!api.error.empty()) return fail(THOR_B200_UNSUPPORTED, "comm_init: %s", api.error.c_str());
    NcclId id;
    memcpy(id.bytes, unique_id_128_bytes, sizeof(id.bytes));
    auto c = new thor_b200_comm();
    c->nranks = nranks;
    c->rank = rank;
    if (int rc = api.CommInitRank(&c->comm, nranks, id, rank)) {
        delete c;
        return ncclFail("ncclCommInitRank", rc);
    }
    *out_comm = c;
    return THOR_B200_OK;
}

int thor_b200_comm_allreduce_f32(thor_b200_comm* comm, void* buffer, uint64_t count, int op, void* stream) {
    using namespace tb;
    TB_REQUIRE(comm != nullptr && comm->comm != nullptr, "comm_allreduce_f32: null communicator");
    TB_REQUIRE(buffer != nullptr || count == 0, "comm_allreduce_f32: null buffer");
    TB_REQUIRE(op >= 0 && op <= 2, "comm_allreduce_f32: op must be 0 (sum), 1 (max) or 2 (min)");
    if (count == 0) return THOR_B200_OK;
    constexpr int kFloat32 = 7;                 // ncclFloat32
    const int red = op == 0 ? 0 : (op == 1 ? 2 : 3);  // ncclSum, ncclMax, ncclMin
    if (int rc = nccl().AllReduce(buffer, buffer, static_cast<size_t>(count), kFloat32, red, comm->comm, static_cast<cudaStream_t>(stream)))
        return ncclFail("ncclAllReduce", rc);
    return THOR_B200_OK;
}

int thor_b200_comm_allreduce_stats_f32(thor_b200_comm* comm, void* sums, uint64_t n_sums, void* maxima, uint64_t n_maxima, void* minima, uint64_t n_minima,
                                       void* stream_v) {
    using namespace tb;
    TB_REQUIRE(comm != nullptr && comm->comm != nullptr, "comm_allreduce_stats_f32: null communicator");
    TB_REQUIRE((sums != nullptr || n_sums == 0) && (maxima != nullptr || n_maxima == 0) && (minima != nullptr || n_minima == 0),
               "comm_allreduce_stats_f32: a buffer with a non-zero count is null");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    NcclApi& api = nccl();
    constexpr int kInt32 = 2, kFloat32 = 7, kSum = 0, kMax = 2, kMin = 3;  // ncclInt32, ncclFloat32, ncclSum, ncclMax, ncclMin
    auto blocks = [](uint64_t n) { return static_cast<unsigned>((n + 255) / 256); };
    if (n_maxima) encodeOrderedKeys<<<blocks(n_maxima), 256, 0, stream>>>(static_cast<float*>(maxima), n_maxima, 1);
    if (n_minima) encodeOrderedKeys<<<blocks(n_minima), 256, 0, stream>>>(static_cast<float*>(minima), n_minima, 0);
    TB_CUDA(cudaGetLastError());
    // one group: NCCL launches the (up to three) small collectives together
    if (int rc = api.GroupStart()) return ncclFail("ncclGroupStart", rc);
    int rc = 0;
    if (n_sums) rc = api.AllReduce(sums, sums, static_cast<size_t>(n_sums), kFloat32, kSum, comm->comm, stream);
    if (!rc && n_maxima) rc = api.AllReduce(maxima, maxima, static_cast<size_t>(n_maxima), kInt32, kMax, comm->comm, stream);
    if (!rc && n_minima) rc = api.AllReduce(minima, minima, static_cast<size_t>(n_minima), kInt32, kMin, comm->comm, stream);
    const int end = api.GroupEnd();
    if (rc) return ncclFail("ncclAllReduce", rc);
    if (end) return ncclFail("ncclGroupEnd", end);
    if (n_maxima) decodeOrderedKeys<<<blocks(n_maxima), 256, 0, stream>>>(static_cast<float*>(maxima), n_maxima);
    if (n_minima) decodeOrderedKeys<<<blocks(n_minima), 256, 0, stream>>>(static_cast<float*>(minima), n_minima);
    TB_CUDA(cudaGetLastError());
    countLaunch((n_maxima ? 2 : 0) + (n_minima ? 2 : 0));
    return THOR_B200_OK;
}

// ---- overlapped combine ---------------------------------------------------------------------------
// A step of a row-sharded job ends with small fp32 partials (two or three statistics, or a [2, cols] block of column
// sums) that have to be combined across the ranks while the NEXT step's kernel already runs.  The combiner owns a
// high-priority side stream and one (ready, done) event pair per slot; the caller double-buffers its partials over the
// slots.  Everything is stream-ordered: no call blocks the host.
struct thor_b200_combiner {
    thor_b200_comm* comm = nullptr;
    cudaStream_t side = nullptr;
    int slots = 0;
    cudaEvent_t ready[8] = {}, done[8] = {};
    bool used[8] = {};
};

int thor_b200_combiner_create(thor_b200_comm* comm, int slots, thor_b200_combiner** out) {
    using namespace tb;
    TB_REQUIRE(comm != nullptr && out != nullptr, "combiner_create: null argument");
    TB_REQUIRE(slots >= 1 && slots <= 8, "combiner_create: between 1 and 8 slots");
    *out = nullptr;
    auto c = new thor_b200_combiner();
    c->comm = comm;
    c->slots = slots;
    int least = 0, greatest = 0;
    cudaError_t e = cudaDeviceGetStreamPriorityRange(&least, &greatest);
    if (e == cudaSuccess) e = cudaStreamCreateWithPriority(&c->side, cudaStreamNonBlocking, greatest);
    for (int i = 0; i < slots && e == cudaSuccess; ++i) {
        e = cudaEventCreateWithFlags(&c->ready[i], cudaEventDisableTiming);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&c->done[i], cudaEventDisableTiming);
    }
    if (e != cudaSuccess) {
        thor_b200_combiner_destroy(c);
        return fail(THOR_B200_CUDA_ERROR, "combiner_create: %s", cudaGetErrorString(e));
    }
    *out = c;
    return THOR_B200_OK;
}

int thor_b200_combiner_wait(thor_b200_combiner* c, int slot, void* stream) {
    using namespace tb;
    TB_REQUIRE(c != nullptr && slot >= 0 && slot < c->slots, "combiner_wait: bad combiner or slot");
    if (c->used[slot]) TB_CUDA(cudaStreamWaitEvent(static_cast<cudaStream_t>(stream), c->done[slot], 0));
    return THOR_B200_OK;
}

int thor_b200_combiner_submit(thor_b200_combiner* c, int slot, void* producer_stream, void* sums, uint64_t n_sums, void* maxima, uint64_t n_maxima,
                              void* minima, uint64_t n_minima, void* rounded_sums, int rounded_dtype) {
    using namespace tb;
    TB_REQUIRE(c != nullptr && slot >= 0 && slot < c->slots, "combiner_submit: bad combiner or slot");
    TB_REQUIRE(rounded_sums == nullptr || (sums != nullptr && n_sums > 0), "combiner_submit: rounded_sums needs sums");
    TB_CUDA(cudaEventRecord(c->ready[slot], static_cast<cudaStream_t>(producer_stream)));
    TB_CUDA(cudaStreamWaitEvent(c->side, c->ready[slot], 0));
    if (int st = thor_b200_comm_allreduce_stats_f32(c->comm, sums, n_sums, maxima, n_maxima, minima, n_minima, c->side)) return st;
    if (rounded_sums != nullptr)
        if (int st = thor_b200_cast_launch(sums, rounded_sums, THOR_B200_FP32, rounded_dtype, static_cast<int64_t>(n_sums), c->side)) return st;
    TB_CUDA(cudaEventRecord(c->done[slot], c->side));
    c->used[slot] = true;
    return THOR_B200_OK;
}

int thor_b200_combiner_drain(thor_b200_combiner* c, void* stream) {
    using namespace tb;
    TB_REQUIRE(c != nullptr, "combiner_drain: null combiner");
    for (int i = 0; i < c->slots; ++i)
        if (c->used[i]) TB_CUDA(cudaStreamWaitEvent(static_cast<cudaStream_t>(stream), c->done[i], 0));
    return THOR_B200_OK;
}

void* thor_b200_combiner_stream(thor_b200_combiner* c) { return c ? c->side : nullptr; }

void thor_b200_combiner_destroy(thor_b200_combiner* c) {
    if (!c) return;
    for (int i = 0; i < 8; ++i) {
        if (c->ready[i]) cudaEventDestroy(c->ready[i]);
        if (c->done[i]) cudaEventDestroy(c->done[i]);
    }
    if (c->side) cudaStreamDestroy(c->side);
    delete c;
}

void thor_b200_comm_destroy(thor_b200_comm* comm) {
    if (!comm) return;
    if (comm->comm) nccl().CommDestroy(comm->comm);
    delete comm;
}

}  // extern "C"
