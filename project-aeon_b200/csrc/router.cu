// Router: gate projection, score, top-k, renormalise, scale.
//
// Stands in for dispatch_router (src/architecture/deepseek_v4/layer/v4_layer_body_moe.hpp:124-159)
// = gemv_fp16_vec8_kernel (src/platform/ops/gemv.hpp:72-110) + v4_half_to_float_n_kernel +
// moe_router_kernel (src/architecture/deepseek_v4/kernels/moe_router.hpp:104-189).
//
// The logits are fp32 with a *defined* summation order so a CPU can reproduce them bit for
// bit and the selected ids can be checked exactly rather than up to near-ties: 32 partial
// sums, partial l taking in ascending k the elements whose 8-wide vector index (k / 8) is
// congruent to l modulo 32 (one fused multiply-add each; products of two 16-bit floats are
// exact in fp32), then a butterfly over lane distances 16, 8, 4, 2, 1. The reference rounds
// its logits to fp16 between the projection and the selection; that rounding is dropped.
//
// Selection: descending key, ties to the lower index (moe_router.hpp:154-169). With a bias
// the key is score + bias, as in the reference; without one the key is the logit itself,
// which orders identically (both score functions are strictly increasing) and does not
// depend on the device's exp/log rounding. Stored weights are the unbiased scores of the
// selected experts, divided by their sum when renormalising, then scaled.
#include "common.cuh"
#include "ptx.cuh"

#include <mutex>

namespace aeon_b200 {

namespace {

constexpr int kLogitWarps = 2;      // experts per CTA (many small CTAs: the kernel is latency-bound)
constexpr int kLogitTokens = 4;     // tokens per CTA

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

// One warp per expert, kTok tokens per CTA pass. A lane walks its vectors (lane, lane + 32, ...)
// in ascending order in batches of kLogitBatch: the batch's gate vectors are all loaded
// before the first is used, then each token's activation vectors likewise, so a warp keeps
// kLogitBatch 16-byte loads in flight instead of one (there is no branch between a load and the
// next: a token index past the end is clamped to the last token and its result dropped).
// The order of the fused multiply-adds into each accumulator is the defined one.
constexpr int kLogitBatch = 8;

template <bool kBf16, int kTok>
__global__ void __launch_bounds__(kLogitWarps * 32)
router_logits_kernel(const uint16_t* __restrict__ x, int64_t x_stride,
                     const uint16_t* __restrict__ gate, int tokens, int experts, int hidden,
                     float* __restrict__ logits) {
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int e = blockIdx.x * kLogitWarps + warp;
    const int t0 = blockIdx.y * kTok;
    if (e >= experts) return;

    float acc[kTok];
#pragma unroll
    for (int j = 0; j < kTok; ++j) acc[j] = 0.f;

    const uint4* grow = reinterpret_cast<const uint4*>(gate + static_cast<size_t>(e) * hidden);
    const int vectors = hidden / 8;      // a multiple of 32: a batch slot is live for the whole warp or not at all
    for (int v0 = lane; v0 < vectors; v0 += 32 * kLogitBatch) {
        uint4 gq[kLogitBatch];
#pragma unroll
        for (int u = 0; u < kLogitBatch; ++u) {
            const int v = v0 + 32 * u;
            gq[u] = v < vectors ? __ldg(grow + v) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int j = 0; j < kTok; ++j) {
            const uint4* xrow = reinterpret_cast<const uint4*>(
                x + static_cast<size_t>(min(t0 + j, tokens - 1)) * x_stride);
            uint4 xq[kLogitBatch];
#pragma unroll
            for (int u = 0; u < kLogitBatch; ++u) {
                const int v = v0 + 32 * u;
                xq[u] = v < vectors ? __ldg(xrow + v) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int u = 0; u < kLogitBatch; ++u) {
                if (v0 + 32 * u < vectors) {
                    float gv[8], xv[8];
                    widen8<kBf16>(gq[u], gv);
                    widen8<kBf16>(xq[u], xv);
#pragma unroll
                    for (int i = 0; i < 8; ++i) acc[j] = fmaf(gv[i], xv[i], acc[j]);
                }
            }
        }
    }
#pragma unroll
    for (int j = 0; j < kTok; ++j) {
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) acc[j] += __shfl_xor_sync(0xFFFFFFFFu, acc[j], off);
        if (lane == 0 && t0 + j < tokens) logits[static_cast<size_t>(t0 + j) * experts + e] = acc[j];
    }
}

// The same logits for batches of 16 tokens and more, tiled: a CTA of four warps owns 16 experts x
// 8 tokens, a warp 4 experts x 8 tokens, so a gate vector is used for eight tokens and an
// activation vector for sixteen experts (the per-expert kernel above re-reads 1.25 rows per
// logit, this one 0.19: at batch 128 that is 590 MB against 90 MB through L2, and that kernel
// was bound by exactly that traffic). The operands of a step (one 16-byte vector per lane and
// row: 24 rows, 12 KB) come through a four-stage shared-memory ring filled with cp.async three
// steps ahead, so no warp waits on a global load: with the loads straight into registers, one
// step ahead, the kernel spent 1 us per step on the L2 round trip against 0.25 us of arithmetic.
// Every logit is still the defined sum: lane l adds its vectors l, l + 32, ... in ascending
// order, element by element, one fused multiply-add each, then the butterfly -- the results are
// bit-identical to the kernel above.
constexpr int kTileExperts = 4;     // per warp
constexpr int kTileTokens = 8;      // per CTA (and per warp); 4 for batches that would leave SMs idle
constexpr int kTileWarps = 4;
constexpr int kTileStages = 4;

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(ptx::smem_u32(smem_dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int kPending>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(kPending) : "memory");
}

template <bool kBf16, int kTileTokens>
__global__ void __launch_bounds__(kTileWarps * 32)
router_logits_tile_kernel(const uint16_t* __restrict__ x, int64_t x_stride,
                          const uint16_t* __restrict__ gate, int tokens, int experts, int hidden,
                          float* __restrict__ logits) {
    static_assert(kTileTokens % kTileWarps == 0, "every warp copies the same number of token rows");
    constexpr int kTileRows = kTileWarps * kTileExperts + kTileTokens;   // operand rows per step
    constexpr int kCopyTokens = kTileTokens / kTileWarps;                // token rows a warp copies
    // [stage][row][lane]: rows 0..15 the CTA's gate rows (4 per warp), then its token rows
    __shared__ uint4 ring[kTileStages][kTileRows][32];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int e0 = (blockIdx.x * kTileWarps + warp) * kTileExperts;
    const int t0 = blockIdx.y * kTileTokens;

    float acc[kTileExperts][kTileTokens];
#pragma unroll
    for (int a = 0; a < kTileExperts; ++a)
#pragma unroll
        for (int j = 0; j < kTileTokens; ++j) acc[a][j] = 0.f;

    // The rows this thread copies every step: its warp's four gate rows and its share of the token
    // rows. Rows past the end are clamped to the last one and their results dropped.
    const uint4* src[kTileExperts + kCopyTokens];
#pragma unroll
    for (int a = 0; a < kTileExperts; ++a)
        src[a] = reinterpret_cast<const uint4*>(gate + static_cast<size_t>(min(e0 + a, experts - 1)) * hidden) + lane;
#pragma unroll
    for (int q = 0; q < kCopyTokens; ++q)
        src[kTileExperts + q] = reinterpret_cast<const uint4*>(
                                    x + static_cast<size_t>(min(t0 + kCopyTokens * warp + q, tokens - 1)) * x_stride) + lane;
    auto issue = [&](int step) {
        uint4(*st)[32] = ring[step % kTileStages];
#pragma unroll
        for (int a = 0; a < kTileExperts; ++a) cp_async16(&st[warp * kTileExperts + a][lane], src[a] + step * 32);
#pragma unroll
        for (int q = 0; q < kCopyTokens; ++q)
            cp_async16(&st[kTileWarps * kTileExperts + kCopyTokens * warp + q][lane], src[kTileExperts + q] + step * 32);
    };

    const int steps = hidden / 256;       // 32 lanes x 8 elements per step; hidden is a multiple of 256 here
#pragma unroll
    for (int s = 0; s < kTileStages - 1; ++s) {
        if (s < steps) issue(s);
        cp_async_commit();
    }
    for (int step = 0; step < steps; ++step) {
        cp_async_wait<kTileStages - 2>();     // this thread's copies of `step` have landed
        __syncthreads();                      // ... and everyone's; everyone is also done with step - 1
        if (step + kTileStages - 1 < steps) issue(step + kTileStages - 1);      // into the stage step - 1 used
        cp_async_commit();
        const uint4(*st)[32] = ring[step % kTileStages];
        float gv[kTileExperts][8];
#pragma unroll
        for (int a = 0; a < kTileExperts; ++a) widen8<kBf16>(st[warp * kTileExperts + a][lane], gv[a]);
#pragma unroll
        for (int j = 0; j < kTileTokens; ++j) {
            float xv[8];
            widen8<kBf16>(st[kTileWarps * kTileExperts + j][lane], xv);
#pragma unroll
            for (int a = 0; a < kTileExperts; ++a)
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[a][j] = fmaf(gv[a][i], xv[i], acc[a][j]);
        }
    }
#pragma unroll
    for (int a = 0; a < kTileExperts; ++a)
#pragma unroll
        for (int j = 0; j < kTileTokens; ++j) {
            float sum = acc[a][j];
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, off);
            if (lane == 0 && e0 + a < experts && t0 + j < tokens)
                logits[static_cast<size_t>(t0 + j) * experts + e0 + a] = sum;
        }
}

__device__ __forceinline__ float score_of(float logit, int score_fn) {
    if (score_fn == AEON_B200_SCORE_SIGMOID) return 1.0f / (1.0f + expf(-logit));
    // sqrt(softplus), softplus with the threshold of 20 the reference model uses.
    return logit > 20.0f ? sqrtf(logit) : sqrtf(log1pf(expf(logit)));
}

constexpr int kSelectWarps = 4;

__global__ void __launch_bounds__(kSelectWarps * 32)
router_select_kernel(const float* __restrict__ logits, const float* __restrict__ bias,
                     const int64_t* __restrict__ hash_table, const int32_t* __restrict__ token_ids,
                     int tokens, int experts, int top_k, int score_fn, int renormalize,
                     float scaling, float* __restrict__ out_weights, int32_t* __restrict__ out_ids,
                     int32_t* __restrict__ error) {
    extern __shared__ float keys[];   // [kSelectWarps][experts]
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int token = blockIdx.x * kSelectWarps + warp;
    if (token >= tokens) return;
    const float* row = logits + static_cast<size_t>(token) * experts;
    float* key = keys + warp * experts;
    float* w_out = out_weights + static_cast<size_t>(token) * top_k;
    int32_t* id_out = out_ids + static_cast<size_t>(token) * top_k;

    float my_weight = 0.f;   // lane k keeps the k-th selected score
    int my_id = -1;

    if (hash_table != nullptr && token_ids != nullptr) {
        if (lane < top_k) {
            my_id = static_cast<int32_t>(hash_table[static_cast<size_t>(token_ids[token]) * top_k + lane]);
            // a table entry outside [0, experts) is reported and never used as an index
            if (my_id < 0 || my_id >= experts) {
                if (error != nullptr) atomicCAS(error, kErrNone, kErrIdOutOfRange);
                my_weight = 0.f;
            } else {
                my_weight = score_of(row[my_id], score_fn);
            }
        }
    } else {
        for (int e = lane; e < experts; e += 32)
            key[e] = (bias != nullptr) ? score_of(row[e], score_fn) + bias[e] : row[e];
        __syncwarp();
        for (int k = 0; k < top_k; ++k) {
            float best = -INFINITY;
            int best_e = 0x7FFFFFFF;
            for (int e = lane; e < experts; e += 32) {
                const float v = key[e];
                if (v > best) { best = v; best_e = e; }   // ascending e: first maximum wins
            }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) {
                const float ov = __shfl_xor_sync(0xFFFFFFFFu, best, off);
                const int oe = __shfl_xor_sync(0xFFFFFFFFu, best_e, off);
                if (ov > best || (ov == best && oe < best_e)) { best = ov; best_e = oe; }
            }
            if (best_e == 0x7FFFFFFF) best_e = 0;   // every key was NaN or -inf
            if (lane == k) {
                my_id = best_e;
                my_weight = score_of(row[best_e], score_fn);
            }
            if (lane == (best_e & 31)) key[best_e] = -INFINITY;
            __syncwarp();
            // a key of -inf can be re-selected only when fewer than top_k finite keys exist
        }
    }

    float sum = (lane < top_k) ? my_weight : 0.f;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, off);
    if (lane < top_k) {
        float w = my_weight;
        // moe_router.hpp:176-186 divides by (sum + 1e-20f): scores that all underflow give
        // weights of 0, not NaN
        if (renormalize) w = w / (sum + 1e-20f);
        w *= scaling;
        w_out[lane] = w;
        id_out[lane] = my_id;
    }
}

template <bool kBf16>
void launch_logits_dtype(const aeon_b200_moe_config& cfg, const void* x, int64_t x_stride, const void* gate,
                         int tokens, float* logits, cudaStream_t stream) {
    const int expert_ctas = (cfg.experts + kLogitWarps - 1) / kLogitWarps;
    const uint16_t* xs = static_cast<const uint16_t*>(x);
    const uint16_t* gs = static_cast<const uint16_t*>(gate);
    if (tokens >= 2 * kTileTokens && cfg.hidden % 256 == 0) {
        const int expert_groups = (cfg.experts + kTileWarps * kTileExperts - 1) / (kTileWarps * kTileExperts);
        // a CTA's time is the length of its K loop whatever the batch: when 8-token tiles would leave
        // more than half of the SMs without a CTA, 4-token tiles halve each CTA's work instead
        if (expert_groups * ((tokens + kTileTokens - 1) / kTileTokens) * 2 <= 148) {
            const dim3 grid(expert_groups, (tokens + 3) / 4);
            router_logits_tile_kernel<kBf16, 4><<<grid, kTileWarps * 32, 0, stream>>>(xs, x_stride, gs, tokens,
                                                                                   cfg.experts, cfg.hidden, logits);
        } else {
            const dim3 grid(expert_groups, (tokens + kTileTokens - 1) / kTileTokens);
            router_logits_tile_kernel<kBf16, kTileTokens><<<grid, kTileWarps * 32, 0, stream>>>(
                xs, x_stride, gs, tokens, cfg.experts, cfg.hidden, logits);
        }
    } else if (tokens < kLogitTokens) {
        // one token per CTA pass: no clamped duplicates at the smallest batches
        router_logits_kernel<kBf16, 1><<<dim3(expert_ctas, tokens), kLogitWarps * 32, 0, stream>>>(
            xs, x_stride, gs, tokens, cfg.experts, cfg.hidden, logits);
    } else {
        router_logits_kernel<kBf16, kLogitTokens>
            <<<dim3(expert_ctas, (tokens + kLogitTokens - 1) / kLogitTokens), kLogitWarps * 32, 0, stream>>>(
                xs, x_stride, gs, tokens, cfg.experts, cfg.hidden, logits);
    }
    AEON_CUDA_CHECK(cudaGetLastError());
}

void launch_logits(const aeon_b200_moe_config& cfg, const void* x, int64_t x_stride, const void* gate,
                   int tokens, float* logits, cudaStream_t stream) {
    if (cfg.act_dtype == AEON_B200_BF16) launch_logits_dtype<true>(cfg, x, x_stride, gate, tokens, logits, stream);
    else launch_logits_dtype<false>(cfg, x, x_stride, gate, tokens, logits, stream);
}

}  // namespace

void launch_router(aeon_b200_ctx* ctx, const void* x, int64_t x_stride, const void* gate,
                   const float* bias, const int64_t* hash_table, const int32_t* token_ids,
                   int tokens, float* topk_weights, int32_t* topk_ids, float* logits_out,
                   cudaStream_t stream) {
    const aeon_b200_moe_config& cfg = ctx->cfg;
    require(x && gate && topk_weights && topk_ids, "aeon_b200_router_topk: null pointer argument");
    require(tokens > 0, "aeon_b200_router_topk: tokens must be positive");
    require(logits_out != nullptr || tokens <= ctx->max_tokens,
            "aeon_b200_router_topk: tokens exceed the context's max_tokens and no logits buffer was given");
    require(x_stride >= cfg.hidden && x_stride % 8 == 0,
            "aeon_b200_router_topk: x_stride must be >= hidden and a multiple of 8");
    require(aligned16(x) && aligned16(gate),
            "aeon_b200_router_topk: x and gate must be 16-byte aligned (128-bit loads)");
    require(cfg.top_k <= 32, "aeon_b200_router_topk: top_k above 32 is not supported");
    float* logits = logits_out != nullptr ? logits_out : ctx->d_logits;

    launch_logits(cfg, x, x_stride, gate, tokens, logits, stream);
    const size_t smem = static_cast<size_t>(kSelectWarps) * cfg.experts * sizeof(float);
    router_select_kernel<<<(tokens + kSelectWarps - 1) / kSelectWarps, kSelectWarps * 32, smem, stream>>>(
        logits, bias, hash_table, token_ids, tokens, cfg.experts, cfg.top_k, cfg.score_fn,
        cfg.renormalize, cfg.routed_scaling, topk_weights, topk_ids, ctx->d_error);
    AEON_CUDA_CHECK(cudaGetLastError());
    ctx->launches += 2;
}

// ---------------------------------------------------------------------------------------
// Router entry point for callers that must not allocate device memory.
//
// Some callers cannot call cudaMalloc where they need the router: code that works under a
// fixed memory budget that a context's scratch was never part of, or a plugin host that
// forbids allocation after start-up. aeon_b200_router_topk needs a context, and creating a context allocates. This
// variant needs none: its only scratch, the fp32 logits [tokens, experts], lives in the
// file-scope device array below, which every GPU that loads this library holds until the
// process exits (kNoAllocMaxTokens * kNoAllocMaxExperts * 4 bytes = 256 KiB).
//
// In host code the array's name is only a host-side handle, not a device address, so the
// device address is looked up once per device with cudaGetSymbolAddress (with that device
// current) and handed to the kernels as an ordinary pointer.
constexpr int kNoAllocMaxTokens = 64;
constexpr int kNoAllocMaxExperts = 1024;
static __device__ __align__(256) float g_noalloc_logits[kNoAllocMaxTokens * kNoAllocMaxExperts];

constexpr int kNoAllocMaxDevices = 64;
static float* g_noalloc_logits_ptr[kNoAllocMaxDevices] = {};
static std::mutex g_noalloc_mutex;

static float* noalloc_scratch_for_current_device() {
    int device = -1;
    AEON_CUDA_CHECK(cudaGetDevice(&device));
    if (device < 0 || device >= kNoAllocMaxDevices)
        throw StatusError(AEON_B200_ERR_UNSUPPORTED,
                          "aeon_b200_router_topk_noalloc: device index above 63");
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    if (g_noalloc_logits_ptr[device] == nullptr) {
        float* ptr = nullptr;
        AEON_CUDA_CHECK(cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_noalloc_logits));
        g_noalloc_logits_ptr[device] = ptr;
    }
    return g_noalloc_logits_ptr[device];
}

void launch_router_noalloc(const aeon_b200_moe_config& cfg, const void* x, int64_t x_stride,
                           const void* gate, const float* bias, int tokens, float* topk_weights,
                           int32_t* topk_ids, cudaStream_t stream) {
    validate_config(cfg);
    require(x && gate && topk_weights && topk_ids,
            "aeon_b200_router_topk_noalloc: null pointer argument");
    require(tokens > 0, "aeon_b200_router_topk_noalloc: tokens must be positive");
    if (tokens > kNoAllocMaxTokens || cfg.experts > kNoAllocMaxExperts)
        throw StatusError(AEON_B200_ERR_INVALID_ARGUMENT,
                          "aeon_b200_router_topk_noalloc: at most 64 tokens and 1024 experts fit the "
                          "built-in scratch; use aeon_b200_router_topk with a context beyond that");
    require(x_stride >= cfg.hidden && x_stride % 8 == 0,
            "aeon_b200_router_topk_noalloc: x_stride must be >= hidden and a multiple of 8");
    require(aligned16(x) && aligned16(gate),
            "aeon_b200_router_topk_noalloc: x and gate must be 16-byte aligned (128-bit loads)");
    float* logits = noalloc_scratch_for_current_device();

    launch_logits(cfg, x, x_stride, gate, tokens, logits, stream);
    const size_t smem = static_cast<size_t>(kSelectWarps) * cfg.experts * sizeof(float);
    router_select_kernel<<<(tokens + kSelectWarps - 1) / kSelectWarps, kSelectWarps * 32, smem, stream>>>(
        logits, bias, nullptr, nullptr, tokens, cfg.experts, cfg.top_k, cfg.score_fn, cfg.renormalize,
        cfg.routed_scaling, topk_weights, topk_ids, nullptr);
    AEON_CUDA_CHECK(cudaGetLastError());
}

}  // namespace aeon_b200
