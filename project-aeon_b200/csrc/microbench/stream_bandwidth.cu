// Microbenchmark behind one design decision of the decode kernels: the packed int4 weights go
// from HBM straight into registers (128-bit streaming loads, several per lane in flight) and
// never through a shared-memory ring fed by bulk copies. It times, on the whole GPU and over a
// 4 GB buffer (far larger than L2),
//   bulk   one producer warp per CTA issuing untiled bulk copies (cp.async.bulk + mbarrier) of
//          `copy` bytes from `copies` separate streams into a ring of `stages` stages, eight
//          consumer warps reading `work` 16-byte vectors per stage from shared memory, and
//   ldg    every warp reading 512 bytes per instruction with U loads per lane in flight,
// and prints GB/s for each configuration. Build and run (B200):
//   make -C project-aeon_b200/csrc microbench && project-aeon_b200/build/stream_bandwidth
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <vector>

#include "../ptx.cuh"

using namespace aeon_b200;

__global__ void __launch_bounds__(288, 1)
bulk_ring_kernel(const uint8_t* src, size_t per_cta, int copy, int copies, int stages, int work,
                 unsigned* sink, int* error) {
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t base = ptx::smem_u32(smem);
    const uint32_t full = base, empty = base + 64, data = base + 128;
    const int stage_bytes = copy * copies;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int s = 0; s < stages; ++s) {
            ptx::mbar_init(full + 8 * s, 1);
            ptx::mbar_init(empty + 8 * s, 8);
        }
        ptx::fence_barrier_init();
    }
    __syncthreads();
    const uint8_t* mine = src + static_cast<size_t>(blockIdx.x) * per_cta;
    const int rounds = static_cast<int>(per_cta / stage_bytes);
    if (warp == 8) {                                   // producer
        const uint64_t policy = ptx::policy_evict_first();
        for (int n = 0; n < rounds; ++n) {
            const int s = n % stages;
            const uint32_t parity = (n / stages) & 1;
            if (lane == 0) {
                (void)ptx::mbar_wait(empty + 8 * s, parity ^ 1, error);     // bounded
                ptx::mbar_arrive_expect_tx(full + 8 * s, stage_bytes);
            }
            __syncwarp();
            for (int c = lane; c < copies; c += 32)
                ptx::bulk_g2s(data + s * stage_bytes + c * copy,
                              mine + static_cast<size_t>(n) * stage_bytes + static_cast<size_t>(c) * copy, copy,
                              full + 8 * s, policy);
        }
        return;
    }
    unsigned acc = 0;                                  // consumers
    for (int n = 0; n < rounds; ++n) {
        const int s = n % stages;
        const uint32_t parity = (n / stages) & 1;
        (void)ptx::mbar_wait(full + 8 * s, parity, error);
        __syncwarp();
        for (int i = 0; i < work; ++i) {
            const uint4 v = ptx::lds128(data + s * stage_bytes + ((tid + i * 256) * 16) % stage_bytes);
            acc += v.x ^ v.y ^ v.z ^ v.w;
        }
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(empty + 8 * s);
    }
    if (acc == 0x12345) sink[0] = acc;
}

template <int U>
__global__ void __launch_bounds__(512, 1)
register_stream_kernel(const uint4* src, size_t vectors_per_cta, unsigned* sink) {
    const uint4* mine = src + static_cast<size_t>(blockIdx.x) * vectors_per_cta;
    unsigned acc = 0;
    const size_t stride = blockDim.x;
    for (size_t i = threadIdx.x; i + (U - 1) * stride < vectors_per_cta; i += U * stride) {
        uint4 v[U];
#pragma unroll
        for (int u = 0; u < U; ++u)
            asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                         : "=r"(v[u].x), "=r"(v[u].y), "=r"(v[u].z), "=r"(v[u].w)
                         : "l"(mine + i + u * stride));
#pragma unroll
        for (int u = 0; u < U; ++u) acc += v[u].x ^ v[u].y ^ v[u].z ^ v[u].w;
    }
    if (acc == 0x12345) sink[0] = acc;
}

#define CHECK(x)                                                                      \
    do {                                                                              \
        cudaError_t e_ = (x);                                                         \
        if (e_ != cudaSuccess) {                                                      \
            std::printf("CUDA error %s at line %d\n", cudaGetErrorString(e_), __LINE__); \
            return 2;                                                                 \
        }                                                                             \
    } while (0)

template <int U>
static int time_register_stream(const uint8_t* buf, size_t vectors_per_cta, int ctas, int threads, unsigned* sink,
                                cudaEvent_t a, cudaEvent_t b) {
    for (int rep = 0; rep < 2; ++rep) {
        CHECK(cudaEventRecord(a));
        register_stream_kernel<U><<<ctas, threads>>>(reinterpret_cast<const uint4*>(buf), vectors_per_cta, sink);
        CHECK(cudaEventRecord(b));
        CHECK(cudaEventSynchronize(b));
    }
    float ms = 0.f;
    CHECK(cudaEventElapsedTime(&ms, a, b));
    std::printf("ldg   loads/lane in flight=%2d  ctas=%3d threads=%3d  in flight/SM=%7d B : %7.1f GB/s\n", U, ctas,
                threads, U * 16 * threads * (ctas / 148), vectors_per_cta * 16.0 * ctas / ms / 1e6);
    return 0;
}

int main() {
    const size_t total = static_cast<size_t>(4) << 30;
    uint8_t* buf = nullptr;
    unsigned* sink = nullptr;
    int* error = nullptr;
    CHECK(cudaMalloc(&buf, total));
    CHECK(cudaMemset(buf, 1, total));
    CHECK(cudaMalloc(&sink, 4));
    CHECK(cudaMalloc(&error, 4));
    CHECK(cudaMemset(error, 0, 4));
    int sms = 0;
    CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, 0));
    cudaEvent_t a, b;
    CHECK(cudaEventCreate(&a));
    CHECK(cudaEventCreate(&b));
    CHECK(cudaFuncSetAttribute(bulk_ring_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    struct Config { int copy, copies, stages, work; };
    const std::vector<Config> configs = {
        {512, 32, 4, 4},  {1024, 16, 4, 4}, {2048, 8, 2, 4},  {2048, 8, 4, 4},  {2048, 8, 8, 4},  {2048, 16, 4, 8},
        {4096, 4, 4, 4},  {4096, 8, 4, 8},  {8192, 2, 4, 4},  {8192, 4, 4, 8},  {16384, 1, 4, 4}, {16384, 2, 4, 8},
        {16384, 2, 6, 8}, {32768, 1, 4, 8}, {32768, 1, 6, 8},
    };
    for (const Config& c : configs) {
        const int stage_bytes = c.copy * c.copies;
        const size_t per_cta = (total / sms) / stage_bytes * stage_bytes;
        const size_t smem = 128 + static_cast<size_t>(stage_bytes) * c.stages;
        if (smem > 200 * 1024) continue;
        for (int rep = 0; rep < 2; ++rep) {
            CHECK(cudaEventRecord(a));
            bulk_ring_kernel<<<sms, 288, smem>>>(buf, per_cta, c.copy, c.copies, c.stages, c.work, sink, error);
            CHECK(cudaEventRecord(b));
            CHECK(cudaEventSynchronize(b));
        }
        float ms = 0.f;
        CHECK(cudaEventElapsedTime(&ms, a, b));
        std::printf("bulk  copy=%5d B x%2d  stages=%d  smem reads/stage=%2d  in flight/SM=%7zu B : %7.1f GB/s\n", c.copy,
                    c.copies, c.stages, c.work, static_cast<size_t>(stage_bytes) * c.stages, per_cta * sms / ms / 1e6);
    }
    const size_t vectors_per_cta = total / 16 / sms;
    if (time_register_stream<4>(buf, vectors_per_cta, sms, 512, sink, a, b)) return 2;
    if (time_register_stream<8>(buf, vectors_per_cta, sms, 512, sink, a, b)) return 2;
    if (time_register_stream<8>(buf, vectors_per_cta / 2, sms * 2, 256, sink, a, b)) return 2;
    if (time_register_stream<16>(buf, vectors_per_cta, sms, 256, sink, a, b)) return 2;
    int flag = 0;
    CHECK(cudaMemcpy(&flag, error, 4, cudaMemcpyDeviceToHost));
    std::printf("wait time-outs: %d\n", flag);
    return flag == 0 ? 0 : 1;
}
