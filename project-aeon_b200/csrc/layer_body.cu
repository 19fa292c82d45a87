// The steps of a layer either side of the MoE FFN: the hyper-connection pre-mix of the four
// residual streams with the FFN RMSNorm (front), and the post expansion back to four streams.
//
// Stands in for the FFN half of the reference's layer body around the expert path:
//   front: hc_project_kernel + hc_sinkhorn_normalize_kernel + hc_pre_combine_kernel
//          (src/architecture/deepseek_v4/kernels/hc_sinkhorn.hpp:22-257) and the FFN RMSNorm,
//          as issued per token by src/architecture/deepseek_v4/layer/v4_layer_body_attention.hpp:95-150;
//   post:  hc_post_kernel (hc_sinkhorn.hpp:259-290), issued by run_layer_body_moe_post
//          (src/architecture/deepseek_v4/layer/v4_layer_body_moe.hpp:258-283).
// The arithmetic follows the reference's fp64 statement of it
// (src/architecture/deepseek_v4/reference/dsv4_oracle.hpp:489-631): mixes over the flattened
// residual with the RMS folded into the projection output, sigmoid gates (only the pre gate
// carries the eps), softmax over the comb's output axis, then alternating normalisations with
// the eps in every denominator; comb[i][j] contracts incoming stream i into outgoing stream j.
//
// The front is one kernel, one CTA per token: it keeps the pre-combined row in registers
// between the combine and the norm, so the 16-bit rounding the reference applies between its
// two kernels disappears; the mix coefficients stay on the device for the post kernel.
#include "common.cuh"

namespace aeon_b200 {

namespace {

constexpr int kHc = 4;                       // residual streams
constexpr int kMixes = kHc * (kHc + 2);      // 4 pre + 4 post + 16 comb logits
constexpr int kThreads = 256;
constexpr int kMaxVecPerThread = 4;          // 8-column vectors of the hidden row per thread: H <= 8192

template <bool kBf16>
__device__ __forceinline__ void widen8(const uint4& v, float (&out)[8]) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        if constexpr (kBf16) {
            out[2 * i] = __uint_as_float(w[i] << 16);
            out[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
        } else {
            const __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
            out[2 * i] = __low2float(h);
            out[2 * i + 1] = __high2float(h);
        }
    }
}

template <bool kBf16>
__device__ __forceinline__ uint4 narrow8(const float (&v)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        if constexpr (kBf16) {
            const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
            w[i] = *reinterpret_cast<const uint32_t*>(&h);
        } else {
            const __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
            w[i] = *reinterpret_cast<const uint32_t*>(&h);
        }
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}

// Sum over the CTA in a fixed order: butterfly inside each warp, then warp 0..7 in order.
__device__ __forceinline__ float block_sum(float v, float* scratch /*[8]*/) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, off);
    __syncthreads();                        // scratch may still be read from an earlier use
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
    __syncthreads();
    float total = 0.f;
#pragma unroll
    for (int w = 0; w < kThreads / 32; ++w) total += scratch[w];
    return total;
}

struct FrontParams {
    const uint16_t* res_mid;     // [tokens, 4, H]
    const float* hc_fn;          // [24, 4 H]
    const float* hc_base;        // [24]
    const float* hc_scale;       // [3]
    const uint16_t* norm_weight; // [H]
    int H;
    float rms_eps, pre_eps, sinkhorn_eps, post_mult, norm_eps;
    int sinkhorn_iters;
    uint16_t* ffn_norm;          // [tokens, out_stride]
    int64_t out_stride;
    float* pre_mix;              // [tokens, 4]
    float* post_mix;             // [tokens, 4]
    float* comb;                 // [tokens, 16]
};

template <bool kBf16>
__global__ void __launch_bounds__(kThreads) hc_ffn_front_kernel(const FrontParams p) {
    __shared__ float s_part[kThreads / 32][kMixes + 1];
    __shared__ float s_mix[kMixes + 1];
    __shared__ float s_pre[kHc];
    __shared__ float s_red[kThreads / 32];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int token = blockIdx.x;
    const int H = p.H;
    const int flat_vecs = kHc * H / 8;
    const uint4* res = reinterpret_cast<const uint4*>(p.res_mid + static_cast<size_t>(token) * kHc * H);

    // ---- mixes: 24 dot products of the flattened residual with the rows of hc_fn, and its sum of squares
    float acc[kMixes + 1];
#pragma unroll
    for (int m = 0; m <= kMixes; ++m) acc[m] = 0.f;
    for (int v = tid; v < flat_vecs; v += kThreads) {
        float r[8];
        widen8<kBf16>(__ldg(res + v), r);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[kMixes] = fmaf(r[i], r[i], acc[kMixes]);
#pragma unroll
        for (int m = 0; m < kMixes; ++m) {
            const float4* f = reinterpret_cast<const float4*>(p.hc_fn + static_cast<size_t>(m) * kHc * H) + 2 * v;
            const float4 a = __ldg(f), b = __ldg(f + 1);
            float s = acc[m];
            s = fmaf(r[0], a.x, s); s = fmaf(r[1], a.y, s); s = fmaf(r[2], a.z, s); s = fmaf(r[3], a.w, s);
            s = fmaf(r[4], b.x, s); s = fmaf(r[5], b.y, s); s = fmaf(r[6], b.z, s); s = fmaf(r[7], b.w, s);
            acc[m] = s;
        }
    }
#pragma unroll
    for (int m = 0; m <= kMixes; ++m) {
        float v = acc[m];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, off);
        if (lane == 0) s_part[warp][m] = v;
    }
    __syncthreads();
    if (tid <= kMixes) {
        float total = 0.f;
#pragma unroll
        for (int w = 0; w < kThreads / 32; ++w) total += s_part[w][tid];
        s_mix[tid] = total;
    }
    __syncthreads();

    // ---- gates and the Sinkhorn comb: lane l < 16 of warp 0 owns comb[i = l / 4][j = l % 4]
    if (warp == 0) {
        const float inv_rms = rsqrtf(s_mix[kMixes] / static_cast<float>(kHc * H) + p.rms_eps);
        const float s0 = p.hc_scale[0], s1 = p.hc_scale[1], s2 = p.hc_scale[2];
        if (lane < kHc) {
            const float pre = 1.0f / (1.0f + expf(-(s_mix[lane] * inv_rms * s0 + p.hc_base[lane]))) + p.pre_eps;
            const float post = 1.0f / (1.0f + expf(-(s_mix[kHc + lane] * inv_rms * s1 + p.hc_base[kHc + lane]))) *
                               p.post_mult;
            s_pre[lane] = pre;
            p.pre_mix[static_cast<size_t>(token) * kHc + lane] = pre;
            p.post_mix[static_cast<size_t>(token) * kHc + lane] = post;
        }
        const int cell = lane & 15;         // lanes 16-31 mirror 0-15 so the shuffles stay full-warp
        float c = s_mix[2 * kHc + cell] * inv_rms * s2 + p.hc_base[2 * kHc + cell];
        // softmax over j (lanes that differ in bits 0-1)
        float mx = fmaxf(c, __shfl_xor_sync(0xFFFFFFFFu, c, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 2));
        c = expf(c - mx);
        float sum = c + __shfl_xor_sync(0xFFFFFFFFu, c, 1);
        sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 2);
        c = c / sum + p.sinkhorn_eps;
        auto over_i = [&]() {               // contraction axis: lanes that differ in bits 2-3
            float col = c + __shfl_xor_sync(0xFFFFFFFFu, c, 4);
            col += __shfl_xor_sync(0xFFFFFFFFu, col, 8);
            c *= 1.0f / (col + p.sinkhorn_eps);
        };
        auto over_j = [&]() {
            float row = c + __shfl_xor_sync(0xFFFFFFFFu, c, 1);
            row += __shfl_xor_sync(0xFFFFFFFFu, row, 2);
            c *= 1.0f / (row + p.sinkhorn_eps);
        };
        over_i();
        for (int it = 0; it < p.sinkhorn_iters - 1; ++it) {
            over_j();
            over_i();
        }
        if (lane < 16) p.comb[static_cast<size_t>(token) * 16 + lane] = c;
    }
    __syncthreads();

    // ---- pre-combine, RMSNorm, 16-bit store; the combined row stays in registers
    const float p0 = s_pre[0], p1 = s_pre[1], p2 = s_pre[2], p3 = s_pre[3];
    const int row_vecs = H / 8;
    float pre[kMaxVecPerThread][8];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < kMaxVecPerThread; ++k) {
        const int v = tid + k * kThreads;
        if (v < row_vecs) {
            float a[8], b[8], c[8], d[8];
            widen8<kBf16>(__ldg(res + v), a);
            widen8<kBf16>(__ldg(res + row_vecs + v), b);
            widen8<kBf16>(__ldg(res + 2 * row_vecs + v), c);
            widen8<kBf16>(__ldg(res + 3 * row_vecs + v), d);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float x = fmaf(p3, d[i], fmaf(p2, c[i], fmaf(p1, b[i], p0 * a[i])));
                pre[k][i] = x;
                ss = fmaf(x, x, ss);
            }
        }
    }
    const float total = block_sum(ss, s_red);
    const float inv = rsqrtf(total / static_cast<float>(H) + p.norm_eps);
    uint16_t* out = p.ffn_norm + static_cast<size_t>(token) * p.out_stride;
#pragma unroll
    for (int k = 0; k < kMaxVecPerThread; ++k) {
        const int v = tid + k * kThreads;
        if (v < row_vecs) {
            float w[8], y[8];
            widen8<kBf16>(__ldg(reinterpret_cast<const uint4*>(p.norm_weight) + v), w);
#pragma unroll
            for (int i = 0; i < 8; ++i) y[i] = pre[k][i] * inv * w[i];
            reinterpret_cast<uint4*>(out)[v] = narrow8<kBf16>(y);
        }
    }
}

// res_out[t][j][h] = post[t][j] * layer_out[t][h] + sum_i comb[t][i][j] * res_mid[t][i][h]
template <bool kBf16>
__global__ void __launch_bounds__(kThreads)
hc_post_kernel(const float* __restrict__ layer_out, int64_t layer_stride, const uint16_t* __restrict__ res_mid,
               const float* __restrict__ post_mix, const float* __restrict__ comb, int H,
               uint16_t* __restrict__ res_out) {
    __shared__ float s_post[kHc];
    __shared__ float s_comb[kHc * kHc];
    const int token = blockIdx.y;
    if (threadIdx.x < kHc) s_post[threadIdx.x] = post_mix[static_cast<size_t>(token) * kHc + threadIdx.x];
    if (threadIdx.x < kHc * kHc) s_comb[threadIdx.x] = comb[static_cast<size_t>(token) * 16 + threadIdx.x];
    __syncthreads();
    const int row_vecs = H / 8;
    const int v = blockIdx.x * kThreads + threadIdx.x;
    if (v >= row_vecs) return;
    const uint4* res = reinterpret_cast<const uint4*>(res_mid + static_cast<size_t>(token) * kHc * H);
    const float4* lo = reinterpret_cast<const float4*>(layer_out + static_cast<size_t>(token) * layer_stride) + 2 * v;
    const float4 la = lo[0], lb = lo[1];
    const float l[8] = {la.x, la.y, la.z, la.w, lb.x, lb.y, lb.z, lb.w};
    float r[kHc][8];
#pragma unroll
    for (int i = 0; i < kHc; ++i) widen8<kBf16>(__ldg(res + i * row_vecs + v), r[i]);
    uint4* out = reinterpret_cast<uint4*>(res_out + static_cast<size_t>(token) * kHc * H);
#pragma unroll
    for (int j = 0; j < kHc; ++j) {
        float y[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            float acc = s_post[j] * l[e];
#pragma unroll
            for (int i = 0; i < kHc; ++i) acc = fmaf(s_comb[i * kHc + j], r[i][e], acc);
            y[e] = acc;
        }
        out[j * row_vecs + v] = narrow8<kBf16>(y);
    }
}

}  // namespace

void launch_hc_ffn_front(aeon_b200_ctx* ctx, const void* res_mid, const float* hc_fn, const float* hc_base,
                         const float* hc_scale3, const void* norm_weight, int tokens,
                         const aeon_b200_hc_params& hp, void* ffn_norm, int64_t out_stride, float* pre_mix,
                         float* post_mix, float* comb, cudaStream_t stream) {
    const aeon_b200_moe_config& cfg = ctx->cfg;
    require(res_mid && hc_fn && hc_base && hc_scale3 && norm_weight && ffn_norm && pre_mix && post_mix && comb,
            "aeon_b200_hc_ffn_front: null pointer argument");
    require(tokens > 0, "aeon_b200_hc_ffn_front: tokens must be positive");
    require(cfg.hidden % 8 == 0 && cfg.hidden <= 8 * kThreads * kMaxVecPerThread,
            "aeon_b200_hc_ffn_front: hidden must be a multiple of 8, at most 8192");
    require(out_stride >= cfg.hidden && out_stride % 8 == 0, "aeon_b200_hc_ffn_front: bad row stride");
    require(hp.sinkhorn_iters >= 1 && hp.sinkhorn_iters <= 1000, "aeon_b200_hc_ffn_front: sinkhorn_iters out of range");
    FrontParams p{};
    p.res_mid = static_cast<const uint16_t*>(res_mid);
    p.hc_fn = hc_fn;
    p.hc_base = hc_base;
    p.hc_scale = hc_scale3;
    p.norm_weight = static_cast<const uint16_t*>(norm_weight);
    p.H = cfg.hidden;
    p.rms_eps = hp.rms_eps;
    p.pre_eps = hp.pre_eps;
    p.sinkhorn_eps = hp.sinkhorn_eps;
    p.post_mult = hp.post_mult;
    p.norm_eps = hp.norm_eps;
    p.sinkhorn_iters = hp.sinkhorn_iters;
    p.ffn_norm = static_cast<uint16_t*>(ffn_norm);
    p.out_stride = out_stride;
    p.pre_mix = pre_mix;
    p.post_mix = post_mix;
    p.comb = comb;
    if (cfg.act_dtype == AEON_B200_BF16) hc_ffn_front_kernel<true><<<tokens, kThreads, 0, stream>>>(p);
    else hc_ffn_front_kernel<false><<<tokens, kThreads, 0, stream>>>(p);
    AEON_CUDA_CHECK(cudaGetLastError());
    ctx->launches += 1;
}

void launch_hc_post(aeon_b200_ctx* ctx, const float* layer_out, int64_t layer_stride, const void* res_mid,
                    const float* post_mix, const float* comb, int tokens, void* res_out, cudaStream_t stream) {
    const aeon_b200_moe_config& cfg = ctx->cfg;
    require(layer_out && res_mid && post_mix && comb && res_out, "aeon_b200_hc_post: null pointer argument");
    require(tokens > 0 && tokens <= 65535, "aeon_b200_hc_post: tokens must be in [1, 65535]");
    require(cfg.hidden % 8 == 0 && layer_stride >= cfg.hidden && layer_stride % 4 == 0,
            "aeon_b200_hc_post: hidden must be a multiple of 8 and the row stride a multiple of 4");
    const dim3 grid((cfg.hidden / 8 + kThreads - 1) / kThreads, tokens);
    if (cfg.act_dtype == AEON_B200_BF16)
        hc_post_kernel<true><<<grid, kThreads, 0, stream>>>(layer_out, layer_stride, static_cast<const uint16_t*>(res_mid),
                                                            post_mix, comb, cfg.hidden, static_cast<uint16_t*>(res_out));
    else
        hc_post_kernel<false><<<grid, kThreads, 0, stream>>>(layer_out, layer_stride, static_cast<const uint16_t*>(res_mid),
                                                             post_mix, comb, cfg.hidden, static_cast<uint16_t*>(res_out));
    AEON_CUDA_CHECK(cudaGetLastError());
    ctx->launches += 1;
}

}  // namespace aeon_b200
