// Microbenchmark: what one tcgen05.mma (kind::f16, cta_group::1, M = 128, K = 16, both operands
// in 128-byte-swizzled shared memory, fp32 accumulator in TMEM) costs on this GPU as a function of
// N, with nothing else running on the SM. One CTA per SM; one thread issues `iters` rounds of four
// MMAs (one 64-wide k-block, as the grouped GEMM does) over `stages` operand tiles that are never
// rewritten (their contents are whatever shared memory holds: only the timing matters). Two forms:
//   issue    all MMAs back to back, one commit at the end;
//   commit   one commit per k-block, as in the pipelined kernel (nobody waits on them but the end).
// and the A operand either in shared memory (a descriptor) or in tensor memory (128 lanes x 8
// packed columns per MMA). Prints cycles per MMA and the fraction of the nominal rate (4096 MACs per cycle per SM).
//   make -C project-aeon_b200/csrc microbench && project-aeon_b200/build/mma_rate
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>

#include "../ptx.cuh"
#include "../tc5.cuh"

using namespace aeon_b200;

constexpr int kStages = 4;
constexpr int kStageA = 128 * 64 * 2;     // 16 KB
constexpr int kStageB = 256 * 64 * 2;     // 32 KB

__global__ void __launch_bounds__(128, 1)
mma_rate_kernel(int n, int iters, int commit_each, int halves, int a_in_tmem, long long* cycles, int* error) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem0 = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem0 - ptx::smem_u32(smem_raw));
    const uint32_t a_smem = smem0;
    const uint32_t b_smem = smem0 + kStages * kStageA;
    const uint32_t bar = b_smem + kStages * kStageB;          // [0]: per-k-block commits, [8]: final
    const uint32_t slot = bar + 32;
    volatile uint32_t* slot_gen = reinterpret_cast<volatile uint32_t*>(smem_gen + (slot - smem0));
    const int tid = threadIdx.x, warp = tid >> 5;
    // finite fp16 operands
    for (int i = tid; i < (kStages * (kStageA + kStageB)) / 4; i += blockDim.x)
        reinterpret_cast<uint32_t*>(smem_gen)[i] = 0x3C003C00u;
    if (tid == 0) {
        ptx::mbar_init(bar, 1);
        ptx::mbar_init(bar + 8, 1);
        ptx::fence_barrier_init();
    }
    if (warp == 0) {
        tc5::tmem_alloc(slot, 512);
        tc5::tmem_relinquish();
    }
    ptx::fence_proxy_async();
    tc5::fence_before_sync();
    __syncthreads();
    tc5::fence_after_sync();
    const uint32_t tmem = *slot_gen;
    if (tid == 0) {
        const uint32_t idesc = tc5::idesc_f16(128, static_cast<uint32_t>(n));
        const uint64_t a0 = tc5::smem_desc_sw128(a_smem), b0 = tc5::smem_desc_sw128(b_smem);
        const long long start = clock64();
        for (int it = 0; it < iters; ++it) {
#pragma unroll
            for (int s = 0; s < kStages; ++s) {
                for (int h = 0; h < halves; ++h) {
                    if (a_in_tmem) {
                        // A operand: 128 lanes x 8 columns per MMA (16 fp16 = 8 packed columns), kept in
                        // the columns above the accumulator (N <= 128 in this mode)
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk)
                            tc5::mma_f16_ts(tmem + h * 128, tmem + 256 + (s * 4 + kk) * 8,
                                            b0 + ((s * kStageB + kk * 32) >> 4), idesc, 1u);
                    } else {
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk)
                            tc5::mma_f16_ss(tmem + h * 256, a0 + ((s * kStageA + kk * 32) >> 4),
                                            b0 + ((s * kStageB + kk * 32) >> 4), idesc, 1u);
                    }
                }
                if (commit_each) tc5::commit(bar);
            }
        }
        tc5::commit(bar + 8);
        const bool ok = ptx::mbar_wait(bar + 8, 0, error);        // bounded
        const long long stop = clock64();
        if (!ok) atomicExch(error, 1);
        if (blockIdx.x == 0) cycles[0] = stop - start;
    }
    tc5::fence_before_sync();
    __syncthreads();
    if (warp == 0) {
        tc5::fence_after_sync();
        tc5::tmem_dealloc(tmem, 512);
    }
}

#define CHECK(x)                                                                         \
    do {                                                                                 \
        cudaError_t e_ = (x);                                                            \
        if (e_ != cudaSuccess) {                                                         \
            std::printf("CUDA error %s at line %d\n", cudaGetErrorString(e_), __LINE__); \
            return 2;                                                                    \
        }                                                                                \
    } while (0)

int main() {
    long long* d_cycles = nullptr;
    int* d_error = nullptr;
    CHECK(cudaMalloc(&d_cycles, 8));
    CHECK(cudaMalloc(&d_error, 4));
    CHECK(cudaMemset(d_error, 0, 4));
    int sms = 0;
    CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, 0));
    const int smem = 1024 + kStages * (kStageA + kStageB) + 256;
    CHECK(cudaFuncSetAttribute(mma_rate_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    const int iters = 2000;                    // x 4 k-blocks x 4 MMAs
    for (int a_in_tmem = 0; a_in_tmem <= 1; ++a_in_tmem)
    for (int halves = 1; halves <= 2; ++halves)
        for (int commit_each = 0; commit_each <= 1; ++commit_each)
            for (int n : {32, 64, 96, 128, 192, 256}) {
                if (a_in_tmem && n > 128) continue;      // the A columns sit above a 2 x 128-column accumulator
                long long cycles = 0;
                for (int rep = 0; rep < 2; ++rep) {
                    mma_rate_kernel<<<sms, 128, smem>>>(n, iters, commit_each, halves, a_in_tmem, d_cycles, d_error);
                    CHECK(cudaGetLastError());
                    CHECK(cudaDeviceSynchronize());
                }
                CHECK(cudaMemcpy(&cycles, d_cycles, 8, cudaMemcpyDeviceToHost));
                const double mmas = static_cast<double>(iters) * kStages * 4 * halves;
                const double per_mma = cycles / mmas;
                const double ideal = 128.0 * n * 16 / 4096.0;
                std::printf("A in %s  %s  accumulators=%d  N=%3d : %7.1f cycles per MMA  (nominal %5.1f, %.2f of nominal rate)\n",
                            a_in_tmem ? "tensor memory" : "shared memory", commit_each ? "commit per k-block" : "issue only        ", halves, n, per_mma, ideal,
                            ideal / per_mma);
            }
    int flag = 0;
    CHECK(cudaMemcpy(&flag, d_error, 4, cudaMemcpyDeviceToHost));
    std::printf("wait time-outs: %d\n", flag);
    return flag == 0 ? 0 : 1;
}
