// Multi-GPU groups behind the C ABI: one process per GPU, NCCL over NVLink / NVSwitch.
//
// The reference has no multi-GPU execution yet: its engine refuses tensor-parallel
// topologies (src/architecture/deepseek_v4/runtime/v4_model_host.hpp:94-100) and plans a C++
// TensorParallelGroup (plans-and-docs/execution/active/MULTI_GPU_EXECUTION_PLAN.md:189-235).
// This file is that layer for the routed-expert path, so that a C++ host drives expert and
// tensor parallelism through the same library as the kernels:
//
//   expert parallel   dispatch  = all-gather of the ranks' activation rows;
//                     exchange  = the partial output rows go to the ranks that own the tokens
//                                 (grouped send/recv, an equal-split all-to-all);
//                     combine   = aeon_b200_ep_combine adds the received slices in rank order.
//   tensor parallel   tp_reduce = reduce-scatter (fp32 sum) of the partial outputs.
//   pipeline          pp_send / pp_recv = the stage hand-off, a byte copy like the reference's
//                     handoff_residual (src/architecture/deepseek_v4/runtime/v4_graph.hpp:454-513).
//
// NCCL is looked up with dlopen when the first group is created: the library has no
// link-time dependence on it and single-GPU users never load it. A process that already
// holds a libnccl.so.2 (PyTorch ships one) gets that same copy.
#include "common.cuh"

#include <dlfcn.h>

#include <cstring>
#include <mutex>

namespace aeon_b200 {

namespace {

// The few NCCL declarations used, restated so that building needs no NCCL headers. The
// values are NCCL's public ABI (nccl.h): ncclUniqueId is 128 opaque bytes, ncclSuccess 0,
// ncclFloat32 7, ncclUint8 1, ncclSum 0.
struct NcclUniqueId { char internal[128]; };
using NcclComm = void*;
constexpr int kNcclSuccess = 0;
constexpr int kNcclUint8 = 1;
constexpr int kNcclFloat32 = 7;
constexpr int kNcclSum = 0;

struct NcclApi {
    int (*GetUniqueId)(NcclUniqueId*);
    int (*CommInitRank)(NcclComm*, int, NcclUniqueId, int);
    int (*CommDestroy)(NcclComm);
    int (*CommAbort)(NcclComm);
    int (*AllGather)(const void*, void*, size_t, int, NcclComm, cudaStream_t);
    int (*ReduceScatter)(const void*, void*, size_t, int, int, NcclComm, cudaStream_t);
    int (*Send)(const void*, size_t, int, int, NcclComm, cudaStream_t);
    int (*Recv)(void*, size_t, int, int, NcclComm, cudaStream_t);
    int (*GroupStart)();
    int (*GroupEnd)();
    const char* (*GetErrorString)(int);
    int (*GetVersion)(int*);
};

const NcclApi& nccl() {
    static NcclApi api{};
    static std::once_flag once;
    static std::string failure;
    std::call_once(once, [] {
        void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (!h) {
            failure = std::string("NCCL is not available: ") + dlerror();
            return;
        }
        auto sym = [&](const char* name) -> void* {
            void* p = dlsym(h, name);
            if (!p && failure.empty()) failure = std::string("NCCL symbol missing: ") + name;
            return p;
        };
        api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(sym("ncclGetUniqueId"));
        api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(sym("ncclCommInitRank"));
        api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(sym("ncclCommDestroy"));
        api.CommAbort = reinterpret_cast<decltype(api.CommAbort)>(sym("ncclCommAbort"));
        api.AllGather = reinterpret_cast<decltype(api.AllGather)>(sym("ncclAllGather"));
        api.ReduceScatter = reinterpret_cast<decltype(api.ReduceScatter)>(sym("ncclReduceScatter"));
        api.Send = reinterpret_cast<decltype(api.Send)>(sym("ncclSend"));
        api.Recv = reinterpret_cast<decltype(api.Recv)>(sym("ncclRecv"));
        api.GroupStart = reinterpret_cast<decltype(api.GroupStart)>(sym("ncclGroupStart"));
        api.GroupEnd = reinterpret_cast<decltype(api.GroupEnd)>(sym("ncclGroupEnd"));
        api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(sym("ncclGetErrorString"));
        api.GetVersion = reinterpret_cast<decltype(api.GetVersion)>(sym("ncclGetVersion"));
    });
    if (!failure.empty()) throw StatusError(AEON_B200_ERR_UNSUPPORTED, failure);
    return api;
}

void nccl_check(int rc, const char* what) {
    if (rc != kNcclSuccess)
        throw StatusError(AEON_B200_ERR_CUDA, std::string(what) + ": " + nccl().GetErrorString(rc));
}

struct DeviceScope {
    int previous{-1};
    explicit DeviceScope(int device) {
        AEON_CUDA_CHECK(cudaGetDevice(&previous));
        if (previous != device) AEON_CUDA_CHECK(cudaSetDevice(device));
        else previous = -1;
    }
    ~DeviceScope() {
        if (previous >= 0) (void)cudaSetDevice(previous);
    }
};

}  // namespace

}  // namespace aeon_b200

struct aeon_b200_group {
    int rank, world, device;
    aeon_b200::NcclComm comm;
};

using namespace aeon_b200;

extern "C" {

int aeon_b200_group_unique_id(void* id_host) {
    return guarded([&] {
        require(id_host != nullptr, "aeon_b200_group_unique_id: null pointer");
        static_assert(sizeof(NcclUniqueId) == AEON_B200_GROUP_ID_BYTES, "id size");
        NcclUniqueId id;
        nccl_check(nccl().GetUniqueId(&id), "ncclGetUniqueId");
        std::memcpy(id_host, &id, sizeof(id));
    });
}

int aeon_b200_group_create(const void* id_host, int rank, int world, int device,
                           aeon_b200_group** out_host) {
    return guarded([&] {
        require(id_host && out_host, "aeon_b200_group_create: null pointer");
        require(world >= 1 && rank >= 0 && rank < world, "aeon_b200_group_create: rank must be in [0, world)");
        DeviceScope scope(device);
        NcclUniqueId id;
        std::memcpy(&id, id_host, sizeof(id));
        NcclComm comm = nullptr;
        nccl_check(nccl().CommInitRank(&comm, world, id, rank), "ncclCommInitRank");
        aeon_b200_group* g = new aeon_b200_group{rank, world, device, comm};
        *out_host = g;
    });
}

int aeon_b200_group_destroy(aeon_b200_group* group) {
    return guarded([&] {
        if (!group) return;
        DeviceScope scope(group->device);
        // every collective of this rank has been enqueued by now; let them finish first
        AEON_CUDA_CHECK(cudaDeviceSynchronize());
        nccl_check(nccl().CommDestroy(group->comm), "ncclCommDestroy");
        delete group;
    });
}

int aeon_b200_group_rank(const aeon_b200_group* group) { return group ? group->rank : -1; }
int aeon_b200_group_world(const aeon_b200_group* group) { return group ? group->world : 0; }

int aeon_b200_ep_dispatch(aeon_b200_group* group, const void* x_local, int tokens_local,
                          int64_t row_bytes, void* x_all, void* stream) {
    return guarded([&] {
        require(group && x_local && x_all, "aeon_b200_ep_dispatch: null pointer");
        require(tokens_local > 0 && row_bytes > 0, "aeon_b200_ep_dispatch: empty rows");
        DeviceScope scope(group->device);
        nccl_check(nccl().AllGather(x_local, x_all, static_cast<size_t>(tokens_local) * row_bytes, kNcclUint8,
                                    group->comm, static_cast<cudaStream_t>(stream)),
                   "ncclAllGather");
    });
}

int aeon_b200_ep_dispatch_routed(aeon_b200_group* group, const void* x_local, int tokens_local,
                                 int64_t row_bytes, void* x_all, const int32_t* ids_local,
                                 const float* weights_local, int top_k, int32_t* ids_all,
                                 float* weights_all, void* stream) {
    return guarded([&] {
        require(group && x_local && x_all && ids_local && weights_local && ids_all && weights_all,
                "aeon_b200_ep_dispatch_routed: null pointer");
        require(tokens_local > 0 && row_bytes > 0 && top_k > 0, "aeon_b200_ep_dispatch_routed: empty rows");
        DeviceScope scope(group->device);
        cudaStream_t s = static_cast<cudaStream_t>(stream);
        const size_t draws = static_cast<size_t>(tokens_local) * top_k;
        // one grouped call: the three gathers go out as a single launch
        nccl_check(nccl().GroupStart(), "ncclGroupStart");
        nccl_check(nccl().AllGather(x_local, x_all, static_cast<size_t>(tokens_local) * row_bytes, kNcclUint8,
                                    group->comm, s), "ncclAllGather");
        nccl_check(nccl().AllGather(ids_local, ids_all, draws * sizeof(int32_t), kNcclUint8, group->comm, s),
                   "ncclAllGather");
        nccl_check(nccl().AllGather(weights_local, weights_all, draws * sizeof(float), kNcclUint8, group->comm, s),
                   "ncclAllGather");
        nccl_check(nccl().GroupEnd(), "ncclGroupEnd");
    });
}

int aeon_b200_ep_exchange(aeon_b200_group* group, const float* partial, int tokens_local, int hidden,
                          float* recv, void* stream) {
    return guarded([&] {
        require(group && partial && recv, "aeon_b200_ep_exchange: null pointer");
        require(tokens_local > 0 && hidden > 0, "aeon_b200_ep_exchange: empty rows");
        DeviceScope scope(group->device);
        const size_t count = static_cast<size_t>(tokens_local) * hidden;
        cudaStream_t s = static_cast<cudaStream_t>(stream);
        nccl_check(nccl().GroupStart(), "ncclGroupStart");
        for (int r = 0; r < group->world; ++r) {
            nccl_check(nccl().Send(partial + r * count, count, kNcclFloat32, r, group->comm, s), "ncclSend");
            nccl_check(nccl().Recv(recv + r * count, count, kNcclFloat32, r, group->comm, s), "ncclRecv");
        }
        nccl_check(nccl().GroupEnd(), "ncclGroupEnd");
    });
}

int aeon_b200_tp_reduce(aeon_b200_group* group, const float* partial, int tokens_local, int hidden,
                        float* out_local, void* stream) {
    return guarded([&] {
        require(group && partial && out_local, "aeon_b200_tp_reduce: null pointer");
        require(tokens_local > 0 && hidden > 0, "aeon_b200_tp_reduce: empty rows");
        DeviceScope scope(group->device);
        nccl_check(nccl().ReduceScatter(partial, out_local, static_cast<size_t>(tokens_local) * hidden,
                                        kNcclFloat32, kNcclSum, group->comm, static_cast<cudaStream_t>(stream)),
                   "ncclReduceScatter");
    });
}

int aeon_b200_pp_send(aeon_b200_group* group, const void* rows, uint64_t bytes, int peer, void* stream) {
    return guarded([&] {
        require(group && rows, "aeon_b200_pp_send: null pointer");
        require(peer >= 0 && peer < group->world && peer != group->rank, "aeon_b200_pp_send: bad peer rank");
        DeviceScope scope(group->device);
        nccl_check(nccl().Send(rows, bytes, kNcclUint8, peer, group->comm, static_cast<cudaStream_t>(stream)),
                   "ncclSend");
    });
}

int aeon_b200_pp_recv(aeon_b200_group* group, void* rows, uint64_t bytes, int peer, void* stream) {
    return guarded([&] {
        require(group && rows, "aeon_b200_pp_recv: null pointer");
        require(peer >= 0 && peer < group->world && peer != group->rank, "aeon_b200_pp_recv: bad peer rank");
        DeviceScope scope(group->device);
        nccl_check(nccl().Recv(rows, bytes, kNcclUint8, peer, group->comm, static_cast<cudaStream_t>(stream)),
                   "ncclRecv");
    });
}

}  // extern "C"
