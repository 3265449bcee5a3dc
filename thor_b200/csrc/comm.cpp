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
        if (!api.GetUniqueId || !api.CommInitRank || !api.AllReduce || !api.CommDestroy || !api.GetErrorString) api.error = "NCCL library lacks a required symbol";
    });
    return api;
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

void thor_b200_comm_destroy(thor_b200_comm* comm) {
    if (!comm) return;
    if (comm->comm) nccl().CommDestroy(comm->comm);
    delete comm;
}

}  // extern "C"
