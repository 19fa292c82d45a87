// Device, stream, event and pinned-memory entry points of the C ABI: what a C++ host needs
// around the kernels without including the CUDA runtime itself. They carry the reference's
// explicit-device rule (src/platform/device.hpp:24-90: the device is an index the caller
// supplies, never a heuristic; a bad index is a named error), its four traffic-class streams
// (src/infrastructure/device_streams.hpp:32-74: non-blocking, all or none), best-effort peer
// access enabled from the accessing device (src/infrastructure/parallel/peer_access.hpp:29-50)
// and the pinned staging + event ordering of its tiered expert supply
// (src/infrastructure/expert/transport/tiered_expert_supply.hpp).
#include "common.cuh"

#include <cstring>

using namespace aeon_b200;

extern "C" {

int aeon_b200_device_count(int* count_host) {
    return guarded([&] {
        require(count_host != nullptr, "aeon_b200_device_count: null pointer");
        AEON_CUDA_CHECK(cudaGetDeviceCount(count_host));
    });
}

int aeon_b200_device_current(int* device_host) {
    return guarded([&] {
        require(device_host != nullptr, "aeon_b200_device_current: null pointer");
        AEON_CUDA_CHECK(cudaGetDevice(device_host));
    });
}

int aeon_b200_device_select(int index) {
    return guarded([&] {
        int count = 0;
        AEON_CUDA_CHECK(cudaGetDeviceCount(&count));
        if (count <= 0) throw StatusError(AEON_B200_ERR_CUDA, "select_device: no CUDA devices are visible");
        if (index < 0 || index >= count)
            throw StatusError(AEON_B200_ERR_OUT_OF_RANGE,
                              "select_device: device index " + std::to_string(index) + " is out of range for " +
                                  std::to_string(count) + " visible devices");
        AEON_CUDA_CHECK(cudaSetDevice(index));
    });
}

int aeon_b200_device_describe(int index, char* name_host, int name_bytes, int* pci_bus_host,
                              int* sm_count_host, uint64_t* memory_bytes_host) {
    return guarded([&] {
        cudaDeviceProp props{};
        AEON_CUDA_CHECK(cudaGetDeviceProperties(&props, index));
        if (name_host != nullptr && name_bytes > 0) {
            std::strncpy(name_host, props.name, static_cast<size_t>(name_bytes) - 1);
            name_host[name_bytes - 1] = '\0';
        }
        if (pci_bus_host) *pci_bus_host = props.pciBusID;
        if (sm_count_host) *sm_count_host = props.multiProcessorCount;
        if (memory_bytes_host) *memory_bytes_host = props.totalGlobalMem;
    });
}

int aeon_b200_device_enable_peer_access(int accessor, int peer, int* enabled_host) {
    return guarded([&] {
        if (enabled_host) *enabled_host = 0;
        if (accessor == peer) return;
        int can = 0;
        if (cudaDeviceCanAccessPeer(&can, accessor, peer) != cudaSuccess || can == 0) {
            (void)cudaGetLastError();
            return;                        // best effort: the copy still works through the host
        }
        int previous = -1;
        AEON_CUDA_CHECK(cudaGetDevice(&previous));
        AEON_CUDA_CHECK(cudaSetDevice(accessor));
        const cudaError_t e = cudaDeviceEnablePeerAccess(peer, 0);
        (void)cudaGetLastError();          // already enabled and declined are both non-fatal
        (void)cudaSetDevice(previous);
        if (enabled_host) *enabled_host = (e == cudaSuccess || e == cudaErrorPeerAccessAlreadyEnabled) ? 1 : 0;
    });
}

int aeon_b200_stream_create(void** stream_host) {
    return guarded([&] {
        require(stream_host != nullptr, "aeon_b200_stream_create: null pointer");
        cudaStream_t s = nullptr;
        AEON_CUDA_CHECK(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
        *stream_host = s;
    });
}

int aeon_b200_stream_destroy(void* stream) {
    return guarded([&] {
        if (stream) AEON_CUDA_CHECK(cudaStreamDestroy(static_cast<cudaStream_t>(stream)));
    });
}

int aeon_b200_stream_synchronize(void* stream) {
    return guarded([&] { AEON_CUDA_CHECK(cudaStreamSynchronize(static_cast<cudaStream_t>(stream))); });
}

int aeon_b200_event_create(void** event_host) {
    return guarded([&] {
        require(event_host != nullptr, "aeon_b200_event_create: null pointer");
        cudaEvent_t e = nullptr;
        AEON_CUDA_CHECK(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        *event_host = e;
    });
}

int aeon_b200_event_destroy(void* event) {
    return guarded([&] {
        if (event) AEON_CUDA_CHECK(cudaEventDestroy(static_cast<cudaEvent_t>(event)));
    });
}

int aeon_b200_event_record(void* event, void* stream) {
    return guarded([&] {
        require(event != nullptr, "aeon_b200_event_record: null event");
        AEON_CUDA_CHECK(cudaEventRecord(static_cast<cudaEvent_t>(event), static_cast<cudaStream_t>(stream)));
    });
}

int aeon_b200_event_synchronize(void* event) {
    return guarded([&] {
        require(event != nullptr, "aeon_b200_event_synchronize: null event");
        AEON_CUDA_CHECK(cudaEventSynchronize(static_cast<cudaEvent_t>(event)));
    });
}

int aeon_b200_stream_wait_event(void* stream, void* event) {
    return guarded([&] {
        require(event != nullptr, "aeon_b200_stream_wait_event: null event");
        AEON_CUDA_CHECK(cudaStreamWaitEvent(static_cast<cudaStream_t>(stream), static_cast<cudaEvent_t>(event), 0));
    });
}

int aeon_b200_host_alloc_pinned(uint64_t bytes, void** out_host) {
    return guarded([&] {
        require(out_host != nullptr && bytes > 0, "aeon_b200_host_alloc_pinned: null pointer or zero size");
        void* p = nullptr;
        AEON_CUDA_CHECK(cudaHostAlloc(&p, bytes, cudaHostAllocDefault));
        *out_host = p;
    });
}

int aeon_b200_host_free_pinned(void* pinned) {
    return guarded([&] {
        if (pinned) AEON_CUDA_CHECK(cudaFreeHost(pinned));
    });
}

int aeon_b200_copy_to_device_async(void* dst_device, const void* src_host, uint64_t bytes, void* stream) {
    return guarded([&] {
        require(dst_device && src_host, "aeon_b200_copy_to_device_async: null pointer");
        AEON_CUDA_CHECK(cudaMemcpyAsync(dst_device, src_host, bytes, cudaMemcpyHostToDevice,
                                        static_cast<cudaStream_t>(stream)));
    });
}

int aeon_b200_copy_to_host_async(void* dst_host, const void* src_device, uint64_t bytes, void* stream) {
    return guarded([&] {
        require(dst_host && src_device, "aeon_b200_copy_to_host_async: null pointer");
        AEON_CUDA_CHECK(cudaMemcpyAsync(dst_host, src_device, bytes, cudaMemcpyDeviceToHost,
                                        static_cast<cudaStream_t>(stream)));
    });
}

int aeon_b200_device_alloc(uint64_t bytes, int device, void** out_host) {
    return guarded([&] {
        require(out_host != nullptr && bytes > 0, "aeon_b200_device_alloc: null pointer or zero size");
        int previous = -1;
        AEON_CUDA_CHECK(cudaGetDevice(&previous));
        AEON_CUDA_CHECK(cudaSetDevice(device));
        void* p = nullptr;
        const cudaError_t e = cudaMalloc(&p, bytes);
        (void)cudaSetDevice(previous);
        AEON_CUDA_CHECK(e);
        *out_host = p;
    });
}

int aeon_b200_device_free(void* device_ptr) {
    return guarded([&] {
        if (device_ptr) AEON_CUDA_CHECK(cudaFree(device_ptr));
    });
}

}  // extern "C"
