// Shared expert at decode batch sizes: a dense 16-bit FFN with the same clamped SwiGLU,
// written into the fp32 accumulator as its initial value.
//
// Stands in for run_layer_body_moe_shared_expert[_batch]
// (src/architecture/deepseek_v4/layer/v4_layer_body_moe.hpp:216-256;
//  src/architecture/deepseek_v4/layer/v4_layer_body_batch.hpp:863-917), which runs three
// gemv_fp16_vec8_kernel launches and v4_swiglu_clamp_kernel
// (src/architecture/deepseek_v4/kernels/v4_swiglu_clamp.hpp:18-34).
//
// Both phases stream the row-major weights once with 128-bit loads straight into MMA
// operand registers (weight rows are the M operand, tokens the N operand; the four lanes of
// a row read 64 contiguous bytes). A CTA owns 16 weight rows (of W1 and W3 together in
// phase 1) and a group of 8, 16 or 32 tokens, and splits K over its warps; the partial sums
// meet in shared memory. Every token group streams the weights again (from L2 after the first),
// so larger batches use the 32-token form: 8 warps x 4 MMA N tiles, which halves that traffic
// against the 16-token form at the same shared-memory footprint.
// Products of two 16-bit floats are exact in the fp32 accumulator. The fp32 hidden vector
// is handed to phase 2 as three 16-bit pieces (hi + mid + lo), so no precision is lost
// between the phases.
#include "common.cuh"
#include "ptx.cuh"

namespace aeon_b200 {

namespace {

// Above this many tokens the tensor-core form (shared_expert_tc.cu) takes over. Its time is
// nearly flat in the token count (both operands arrive by TMA; it is bound by streaming the 88 MB
// of weights), while the kernels here stream the weights once per group of up to 32 tokens.
// Measured on B200, microseconds per call: these kernels 31 / 38 / 67 / 76 / 94 at 8 / 16 / 17 /
// 32 / 64 tokens, the tensor-core form 49 / 52 / 54 at 65 / 96 / 128.
constexpr int kTensorCoreFrom = 16;

// Instances <warps, N tiles>: <16, 1> up to 8 tokens, <16, 2> up to 16, <8, 4> beyond
// (32 tokens per CTA pass). The reduction buffer stays within 32 KB of static shared memory.

template <bool kBf16>
__device__ __forceinline__ void mma16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                      uint32_t a3, uint32_t b0, uint32_t b1) {
    if constexpr (kBf16) ptx::mma_bf16(d, a0, a1, a2, a3, b0, b1);
    else ptx::mma_f16(d, a0, a1, a2, a3, b0, b1);
}

template <bool kBf16>
__device__ __forceinline__ uint16_t narrow(float v) {
    if constexpr (kBf16) return __bfloat16_as_ushort(__float2bfloat16_rn(v));
    else return __half_as_ushort(__float2half_rn(v));
}

template <bool kBf16>
__device__ __forceinline__ float widen(uint16_t v) {
    if constexpr (kBf16) return __bfloat162float(__ushort_as_bfloat16(v));
    else return __half2float(__ushort_as_half(v));
}

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// Phase 1: hidden[t, r] = swiglu(W1[r,:] . x[t,:], W3[r,:] . x[t,:]) as three 16-bit pieces.
template <bool kBf16, int kWarps, int kNT>
__global__ void __launch_bounds__(kWarps * 32)
shared_gate_up_kernel(const uint16_t* __restrict__ w1, const uint16_t* __restrict__ w3,
                      const uint16_t* __restrict__ x, int64_t x_stride, int tokens, int H, int I,
                      float limit, uint16_t* __restrict__ hid_hi, uint16_t* __restrict__ hid_mid,
                      uint16_t* __restrict__ hid_lo) {
    __shared__ float red[kWarps][2][kNT][128];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int row0 = blockIdx.x * 16;
    const int tok0 = blockIdx.y * (kNT * 8);
    const int kspan = H / kWarps;
    const int kbeg = warp * kspan;

    float acc[2][kNT][4];
#pragma unroll
    for (int m = 0; m < 2; ++m)
#pragma unroll
        for (int n = 0; n < kNT; ++n)
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[m][n][c] = 0.f;

    const uint16_t* w1a = w1 + static_cast<size_t>(row0 + g) * H;
    const uint16_t* w1b = w1 + static_cast<size_t>(row0 + g + 8) * H;
    const uint16_t* w3a = w3 + static_cast<size_t>(row0 + g) * H;
    const uint16_t* w3b = w3 + static_cast<size_t>(row0 + g + 8) * H;

#pragma unroll 2
    for (int k = kbeg; k < kbeg + kspan; k += 32) {
        const int kk = k + 8 * t;
        const uint4 a1 = ldg_stream(w1a + kk), b1 = ldg_stream(w1b + kk);
        const uint4 a3 = ldg_stream(w3a + kk), b3 = ldg_stream(w3b + kk);
#pragma unroll
        for (int n = 0; n < kNT; ++n) {
            const int token = tok0 + n * 8 + g;
            uint4 xv = make_uint4(0, 0, 0, 0);
            if (token < tokens)
                xv = __ldg(reinterpret_cast<const uint4*>(x + static_cast<size_t>(token) * x_stride + kk));
            mma16<kBf16>(acc[0][n], a1.x, b1.x, a1.y, b1.y, xv.x, xv.y);
            mma16<kBf16>(acc[0][n], a1.z, b1.z, a1.w, b1.w, xv.z, xv.w);
            mma16<kBf16>(acc[1][n], a3.x, b3.x, a3.y, b3.y, xv.x, xv.y);
            mma16<kBf16>(acc[1][n], a3.z, b3.z, a3.w, b3.w, xv.z, xv.w);
        }
    }
#pragma unroll
    for (int m = 0; m < 2; ++m)
#pragma unroll
        for (int n = 0; n < kNT; ++n)
            *reinterpret_cast<float4*>(&red[warp][m][n][lane * 4]) =
                make_float4(acc[m][n][0], acc[m][n][1], acc[m][n][2], acc[m][n][3]);
    __syncthreads();
    for (int o = threadIdx.x; o < kNT * 128; o += kWarps * 32) {
        const int n = o >> 7, idx = o & 127;
        float gate = 0.f, up = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
            gate += red[w][0][n][idx];
            up += red[w][1][n][idx];
        }
        const int lo = idx >> 2, c = idx & 3;
        const int go = lo >> 2, to = lo & 3;
        const int token = tok0 + n * 8 + 2 * to + (c & 1);
        const int row = row0 + go + 8 * (c >> 1);
        if (token < tokens) {
            gate = fminf(gate, limit);
            up = fminf(fmaxf(up, -limit), limit);
            const float h = (gate / (1.0f + expf(-gate))) * up;
            const uint16_t hi = narrow<kBf16>(h);
            const float r1 = h - widen<kBf16>(hi);
            const uint16_t mid = narrow<kBf16>(r1);
            const uint16_t low = narrow<kBf16>(r1 - widen<kBf16>(mid));
            const size_t at = static_cast<size_t>(token) * I + row;
            hid_hi[at] = hi;
            hid_mid[at] = mid;
            hid_lo[at] = low;
        }
    }
}

// Phase 2: out[t, r] = W2[r,:] . hidden[t,:]  (written, not added).
template <bool kBf16, int kWarps, int kNT>
__global__ void __launch_bounds__(kWarps * 32)
shared_down_kernel(const uint16_t* __restrict__ w2, const uint16_t* __restrict__ hid_hi,
                   const uint16_t* __restrict__ hid_mid, const uint16_t* __restrict__ hid_lo,
                   int tokens, int H, int I, float* __restrict__ out, int64_t out_stride) {
    __shared__ float red[kWarps][kNT][128];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int row0 = blockIdx.x * 16;
    const int tok0 = blockIdx.y * (kNT * 8);
    const int kspan = I / kWarps;
    const int kbeg = warp * kspan;

    float acc[kNT][4];
#pragma unroll
    for (int n = 0; n < kNT; ++n)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[n][c] = 0.f;

    const uint16_t* wa = w2 + static_cast<size_t>(row0 + g) * I;
    const uint16_t* wb = w2 + static_cast<size_t>(row0 + g + 8) * I;
#pragma unroll 2
    for (int k = kbeg; k < kbeg + kspan; k += 32) {
        const int kk = k + 8 * t;
        const uint4 a = ldg_stream(wa + kk), b = ldg_stream(wb + kk);
#pragma unroll
        for (int n = 0; n < kNT; ++n) {
            const int token = tok0 + n * 8 + g;
            // Loads are predicated per lane; the MMAs run on the whole warp.
            uint4 h0 = make_uint4(0, 0, 0, 0), h1 = h0, h2 = h0;
            if (token < tokens) {
                const size_t at = static_cast<size_t>(token) * I + kk;
                h0 = __ldg(reinterpret_cast<const uint4*>(hid_hi + at));
                h1 = __ldg(reinterpret_cast<const uint4*>(hid_mid + at));
                h2 = __ldg(reinterpret_cast<const uint4*>(hid_lo + at));
            }
            mma16<kBf16>(acc[n], a.x, b.x, a.y, b.y, h0.x, h0.y);
            mma16<kBf16>(acc[n], a.z, b.z, a.w, b.w, h0.z, h0.w);
            mma16<kBf16>(acc[n], a.x, b.x, a.y, b.y, h1.x, h1.y);
            mma16<kBf16>(acc[n], a.z, b.z, a.w, b.w, h1.z, h1.w);
            mma16<kBf16>(acc[n], a.x, b.x, a.y, b.y, h2.x, h2.y);
            mma16<kBf16>(acc[n], a.z, b.z, a.w, b.w, h2.z, h2.w);
        }
    }
#pragma unroll
    for (int n = 0; n < kNT; ++n)
        *reinterpret_cast<float4*>(&red[warp][n][lane * 4]) =
            make_float4(acc[n][0], acc[n][1], acc[n][2], acc[n][3]);
    __syncthreads();
    for (int o = threadIdx.x; o < kNT * 128; o += kWarps * 32) {
        const int n = o >> 7, idx = o & 127;
        float sum = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) sum += red[w][n][idx];
        const int lo = idx >> 2, c = idx & 3;
        const int go = lo >> 2, to = lo & 3;
        const int token = tok0 + n * 8 + 2 * to + (c & 1);
        const int row = row0 + go + 8 * (c >> 1);
        if (token < tokens) out[static_cast<size_t>(token) * out_stride + row] = sum;
    }
}

template <bool kBf16, int kWarps, int kNT>
void launch_shared_instance(aeon_b200_ctx* ctx, const void* w1, const void* w3, const void* w2,
                            const void* x, int64_t x_stride, int tokens, float* moe_accum,
                            int64_t accum_stride, cudaStream_t stream) {
    const aeon_b200_moe_config& cfg = ctx->cfg;
    const int groups = (tokens + kNT * 8 - 1) / (kNT * 8);
    uint16_t* hi = reinterpret_cast<uint16_t*>(ctx->d_sh_hi);
    uint16_t* mid = reinterpret_cast<uint16_t*>(ctx->d_sh_mid);
    uint16_t* lo = reinterpret_cast<uint16_t*>(ctx->d_sh_lo);
    const dim3 grid1(cfg.intermediate / 16, groups), grid2(cfg.hidden / 16, groups);
    shared_gate_up_kernel<kBf16, kWarps, kNT><<<grid1, kWarps * 32, 0, stream>>>(
        static_cast<const uint16_t*>(w1), static_cast<const uint16_t*>(w3), static_cast<const uint16_t*>(x),
        x_stride, tokens, cfg.hidden, cfg.intermediate, cfg.swiglu_limit, hi, mid, lo);
    AEON_CUDA_CHECK(cudaGetLastError());
    shared_down_kernel<kBf16, kWarps, kNT><<<grid2, kWarps * 32, 0, stream>>>(
        static_cast<const uint16_t*>(w2), hi, mid, lo, tokens, cfg.hidden, cfg.intermediate, moe_accum,
        accum_stride);
    AEON_CUDA_CHECK(cudaGetLastError());
}

template <bool kBf16>
void launch_shared_dtype(aeon_b200_ctx* ctx, const void* w1, const void* w3, const void* w2,
                         const void* x, int64_t x_stride, int tokens, float* moe_accum,
                         int64_t accum_stride, cudaStream_t stream) {
    if (tokens <= 8)
        launch_shared_instance<kBf16, 16, 1>(ctx, w1, w3, w2, x, x_stride, tokens, moe_accum, accum_stride, stream);
    else if (tokens <= 16)
        launch_shared_instance<kBf16, 16, 2>(ctx, w1, w3, w2, x, x_stride, tokens, moe_accum, accum_stride, stream);
    else
        launch_shared_instance<kBf16, 8, 4>(ctx, w1, w3, w2, x, x_stride, tokens, moe_accum, accum_stride, stream);
}

}  // namespace

void launch_shared_expert(aeon_b200_ctx* ctx, const void* w1, const void* w3, const void* w2,
                          const void* x, int64_t x_stride, int tokens, float* moe_accum,
                          int64_t accum_stride, cudaStream_t stream) {
    const aeon_b200_moe_config& cfg = ctx->cfg;
    require(w1 && w3 && w2 && x && moe_accum, "aeon_b200_shared_expert: null pointer argument");
    require(tokens > 0 && tokens <= ctx->max_tokens,
            "aeon_b200_shared_expert: tokens must be in [1, max_tokens of the context]");
    require(x_stride >= cfg.hidden && x_stride % 8 == 0 && accum_stride >= cfg.hidden,
            "aeon_b200_shared_expert: bad row stride");
    require(cfg.hidden % 512 == 0 && cfg.intermediate % 512 == 0,
            "aeon_b200_shared_expert: hidden and intermediate must be multiples of 512");
    if (tokens > kTensorCoreFrom && shared_expert_tc_supports(cfg, accum_stride)) {
        // a dense contraction from here on: tensor-core form
        launch_shared_expert_tc(ctx, w1, w3, w2, x, x_stride, tokens, moe_accum, accum_stride, stream);
        return;
    }
    if (cfg.act_dtype == AEON_B200_BF16)
        launch_shared_dtype<true>(ctx, w1, w3, w2, x, x_stride, tokens, moe_accum, accum_stride, stream);
    else
        launch_shared_dtype<false>(ctx, w1, w3, w2, x, x_stride, tokens, moe_accum, accum_stride, stream);
    ctx->launches += 2;
}

}  // namespace aeon_b200
