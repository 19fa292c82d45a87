// Shared expert at larger batches: its two dense projections as tcgen05 GEMMs.
//
// Stands in for the batched shared expert of the reference,
// run_layer_body_moe_shared_expert_batch (src/architecture/deepseek_v4/layer/v4_layer_body_batch.hpp:863-917:
// three project_dense calls, src/architecture/deepseek_v4/layer/v4_dense_projection.hpp:21-36, and
// v4_swiglu_clamp_kernel). At larger batches the work is a dense contraction (128 tokens: 11.3
// GFLOP against 88 MB of weights), so it runs on the tensor cores with the pipeline of the grouped
// expert GEMM (prefill.cu): weight rows are the MMA M dimension (128 per tile), tokens the N
// dimension (16..256), K in blocks of 64, fp32 accumulators in tensor memory.
//
//   warps 0-3   epilogue: tcgen05.ld, store the tile's fp32 partial sums;
//   warp 4      one thread issues the tiled TMA loads of both operands (no multicast): the dense
//               16-bit weights are MMA-ready as they lie in memory, so a 128-row x 64-column box
//               lands in the 128-byte-swizzled K-major tile without passing through registers
//               (a first version copied them with eight warps of 128-bit loads and stores and was
//               bound by those warps, 58 us for the two projections against 14 us of HBM time);
//   warp 5      MMA issue and commits; owns the tensor-memory allocation.
//
// The projections are small in M x N (32 and 56 row blocks for one token tile), so K is split
// over up to four CTAs per tile to occupy the SMs; every split writes its partial tile to a
// scratch buffer and a small finishing kernel adds the splits in a fixed order (bit-reproducible,
// no atomics), applies the clamped SwiGLU after the first projection and writes the result.
//
// Numerics: products of two 16-bit floats are exact in the fp32 accumulator. The fp32 hidden
// vector enters the second projection as three 16-bit planes (hi + mid + lo) that are summed by
// running the K loop over the planes, so nothing is rounded between the projections.
#include "common.cuh"
#include "ptx.cuh"
#include "tc5.cuh"
#include "tensor_map.cuh"

#include <algorithm>

namespace aeon_b200 {

namespace {

constexpr int kTileM = 128;
constexpr int kTileK = 64;
constexpr int kMaxN = 256;
constexpr int kStages = 4;
constexpr int kEpilogueWarps = 4;
constexpr int kTmaWarp = kEpilogueWarps, kMmaWarp = kEpilogueWarps + 1;
constexpr int kPrefetch = 4;         // K-splits are whole multiples of this many k-blocks
constexpr int kThreads = (kEpilogueWarps + 2) * 32;
constexpr int kStageA = kTileM * kTileK * 2;          // 16 KB
constexpr int kStageB = kMaxN * kTileK * 2;           // 32 KB
constexpr int kSmemBytes = 1024 /*align*/ + kStages * (kStageA + kStageB) + 256 /*barriers*/;
constexpr int kTmemCols = 512;

struct DenseParams {
    const uint16_t* wa;   // first projection: W1 [I, K]; second: W2 [H, K]
    const uint16_t* wb;   // first projection: W3 [I, K]; second: unused
    int K;                // columns of the weight matrices
    int rows;             // columns of the partial buffer: 2 I (gate | up) or H
    int half_rows;        // I for the first projection: the up value of hidden column j is column I + j
    int tokens;
    int planes;           // activation planes the K loop runs over: 1 (x) or 3 (hidden hi, mid, lo)
    int splits;           // K-splits per tile
    float* partial;       // [splits][tokens][rows]
    int32_t* error;
};

__device__ __forceinline__ void flag_error(int32_t* error, int code) { atomicCAS(error, kErrNone, code); }


// item -> (token tile, row block, split); the split runs fastest
struct Item {
    int tt, rb, sp;
};
__device__ __forceinline__ Item decode_item(int item, int row_blocks, int splits) {
    Item it;
    it.sp = item % splits;
    const int t = item / splits;
    it.rb = t % row_blocks;
    it.tt = t / row_blocks;
    return it;
}

// kGateUp: row block rb < I / 128 is rows rb*128 .. of W1 (wmap_a), the others rows of W3 (wmap_b),
// so the partial buffer's columns are [gate I | up I]; else row block rb is rows rb*128 .. of W2.
// map0..2: the activation planes.
template <bool kGateUp, bool kBf16>
__global__ void __launch_bounds__(kThreads, 1)
shared_dense_gemm_kernel(const DenseParams p, const __grid_constant__ CUtensorMap map0,
                         const __grid_constant__ CUtensorMap map1, const __grid_constant__ CUtensorMap map2,
                         const __grid_constant__ CUtensorMap wmap_a, const __grid_constant__ CUtensorMap wmap_b) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem0 = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem0 - ptx::smem_u32(smem_raw));
    const uint32_t a_smem = smem0;
    const uint32_t b_smem = smem0 + kStages * kStageA;
    const uint32_t bar0 = b_smem + kStages * kStageB;
    const uint32_t full_bar = bar0;                    // kStages
    const uint32_t empty_bar = bar0 + 8 * kStages;     // kStages
    const uint32_t acc_full = bar0 + 16 * kStages;     // 2
    const uint32_t acc_empty = acc_full + 16;          // 2
    const uint32_t tmem_slot = acc_empty + 16;         // 4 B
    volatile uint32_t* tmem_slot_gen =
        reinterpret_cast<volatile uint32_t*>(smem_gen + (tmem_slot - smem0));

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;

    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) {
            ptx::mbar_init(full_bar + 8 * s, 1);             // the TMA thread's arrive with the byte count
            ptx::mbar_init(empty_bar + 8 * s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            ptx::mbar_init(acc_full + 8 * b, 1);
            ptx::mbar_init(acc_empty + 8 * b, kEpilogueWarps);
        }
        ptx::fence_barrier_init();
    }
    if (warp == kMmaWarp) {
        tc5::tmem_alloc(tmem_slot, kTmemCols);
        tc5::tmem_relinquish();
    }
    tc5::fence_before_sync();
    __syncthreads();
    tc5::fence_after_sync();
    const uint32_t tmem_base = *tmem_slot_gen;

    const int row_blocks = p.rows / kTileM;
    const int token_tiles = (p.tokens + kMaxN - 1) / kMaxN;
    const int kb_plane = p.K / kTileK;                       // k-blocks of one activation plane
    const int kb_split = p.planes * kb_plane / p.splits;     // k-blocks of one item
    const int total_items = token_tiles * row_blocks * p.splits;

    if (warp == kTmaWarp) {
        // ------------------------------ TMA: both operands ---------------------------------------
        if (lane == 0) {
            uint32_t n = 0;
            for (int item = blockIdx.x; item < total_items; item += gridDim.x) {
                const Item it = decode_item(item, row_blocks, p.splits);
                const int tok0 = it.tt * kMaxN;
                const int ntok = min(kMaxN, p.tokens - tok0);
                const int boxes = (ntok + 63) / 64;
                const CUtensorMap* wmap = &wmap_a;
                int wrow = it.rb * kTileM;
                if constexpr (kGateUp) {
                    if (wrow >= p.half_rows) {
                        wmap = &wmap_b;
                        wrow -= p.half_rows;
                    }
                }
                for (int k = 0; k < kb_split; ++k, ++n) {
                    const int kg = it.sp * kb_split + k;
                    const int plane = kg / kb_plane;
                    const int kb = kg - plane * kb_plane;
                    const CUtensorMap* map = plane == 0 ? &map0 : (plane == 1 ? &map1 : &map2);
                    const int s = n % kStages;
                    const uint32_t parity = (n / kStages) & 1;
                    if (!ptx::mbar_wait(empty_bar + 8 * s, parity ^ 1, p.error)) flag_error(p.error, kErrWaitTimeout);
                    ptx::mbar_arrive_expect_tx(full_bar + 8 * s, boxes * 64 * kTileK * 2 + kStageA);
                    tc5::tma_load_2d(a_smem + s * kStageA, wmap, kb * kTileK, wrow, full_bar + 8 * s);
                    for (int b = 0; b < boxes; ++b)
                        tc5::tma_load_2d(b_smem + s * kStageB + b * (64 * kTileK * 2), map, kb * kTileK,
                                         tok0 + b * 64, full_bar + 8 * s);
                }
            }
        }
    } else if (warp == kMmaWarp) {
        // ------------------------------ MMA issue ---------------------------------------------
        if (lane == 0) {
            uint32_t n = 0, count = 0;
            for (int item = blockIdx.x; item < total_items; item += gridDim.x, ++count) {
                const Item it = decode_item(item, row_blocks, p.splits);
                const int ntok = min(kMaxN, p.tokens - it.tt * kMaxN);
                const uint32_t n_mma = static_cast<uint32_t>((ntok + 15) & ~15);
                const uint32_t idesc = tc5::idesc_16bit(kTileM, n_mma, kBf16);
                const uint32_t buf = count & 1;
                if (!ptx::mbar_wait(acc_empty + 8 * buf, ((count >> 1) & 1) ^ 1, p.error))
                    flag_error(p.error, kErrWaitTimeout);
                tc5::fence_after_sync();
                const uint32_t d_tmem = tmem_base + buf * kMaxN;
                for (int k = 0; k < kb_split; ++k, ++n) {
                    const int s = n % kStages;
                    const uint32_t parity = (n / kStages) & 1;
                    if (!ptx::mbar_wait(full_bar + 8 * s, parity, p.error)) flag_error(p.error, kErrWaitTimeout);
                    tc5::fence_after_sync();
                    const uint32_t a_addr = a_smem + s * kStageA;
                    const uint32_t b_addr = b_smem + s * kStageB;
#pragma unroll
                    for (int kk = 0; kk < kTileK / 16; ++kk) {
                        tc5::mma_f16_ss(d_tmem, tc5::smem_desc_sw128(a_addr + kk * 32),
                                        tc5::smem_desc_sw128(b_addr + kk * 32), idesc,
                                        (k > 0 || kk > 0) ? 1u : 0u);
                    }
                    tc5::commit(empty_bar + 8 * s);      // stage free when these MMAs are done
                }
                tc5::commit(acc_full + 8 * buf);         // accumulator complete
            }
        }
    } else {
        // ------------------------------ epilogue: fp32 partial tile ------------------------------
        const int quad = warp;                              // TMEM lanes 32*quad .. +31
        const int r = quad * 32 + lane;                     // tile row of this thread
        uint32_t count = 0;
        for (int item = blockIdx.x; item < total_items; item += gridDim.x, ++count) {
            const Item it = decode_item(item, row_blocks, p.splits);
            const int tok0 = it.tt * kMaxN;
            const int ntok = min(kMaxN, p.tokens - tok0);
            const int col = it.rb * kTileM + r;
            float* out = p.partial + (static_cast<size_t>(it.sp) * p.tokens + tok0) * p.rows + col;
            const uint32_t buf = count & 1;
            if (!ptx::mbar_wait(acc_full + 8 * buf, (count >> 1) & 1, p.error)) flag_error(p.error, kErrWaitTimeout);
            tc5::fence_after_sync();
            const uint32_t taddr = tmem_base + ((static_cast<uint32_t>(quad) * 32u) << 16) + buf * kMaxN;
            for (int c0 = 0; c0 < ntok; c0 += 32) {
                uint32_t v[32];
                tc5::ld_32x32(taddr + c0, v);
                tc5::ld_wait();
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    if (c0 + j < ntok) out[static_cast<size_t>(c0 + j) * p.rows] = __uint_as_float(v[j]);
            }
            tc5::fence_before_sync();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(acc_empty + 8 * buf);
        }
    }

    tc5::fence_before_sync();
    __syncthreads();
    if (warp == kMmaWarp) {
        tc5::fence_after_sync();
        tc5::tmem_dealloc(tmem_base, kTmemCols);
    }
}

template <bool kBf16>
__device__ __forceinline__ uint16_t narrow16(float v) {
    if constexpr (kBf16) return __bfloat16_as_ushort(__float2bfloat16_rn(v));
    else return __half_as_ushort(__float2half_rn(v));
}

template <bool kBf16>
__device__ __forceinline__ float widen16(uint16_t v) {
    if constexpr (kBf16) return __bfloat162float(__ushort_as_bfloat16(v));
    else return __half2float(__ushort_as_half(v));
}

// hidden[t, j] = swiglu(sum_s P[s][t][j], sum_s P[s][t][I + j]) as three 16-bit planes.
template <bool kBf16>
__global__ void shared_swiglu_finish_kernel(const float* __restrict__ partial, int splits, int tokens, int I,
                                            float limit, uint16_t* __restrict__ hid_hi,
                                            uint16_t* __restrict__ hid_mid, uint16_t* __restrict__ hid_lo) {
    const int64_t total = static_cast<int64_t>(tokens) * I;
    const size_t plane = static_cast<size_t>(tokens) * 2 * I;
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int t = static_cast<int>(i / I);
        const int j = static_cast<int>(i - static_cast<int64_t>(t) * I);
        const float* base = partial + static_cast<size_t>(t) * 2 * I + j;
        float gate = 0.f, up = 0.f;
        for (int s = 0; s < splits; ++s) {
            gate += base[s * plane];
            up += base[s * plane + I];
        }
        gate = fminf(gate, limit);
        up = fminf(fmaxf(up, -limit), limit);
        const float h = (gate / (1.0f + expf(-gate))) * up;
        const uint16_t hi = narrow16<kBf16>(h);
        const float r1 = h - widen16<kBf16>(hi);
        const uint16_t mid = narrow16<kBf16>(r1);
        const uint16_t low = narrow16<kBf16>(r1 - widen16<kBf16>(mid));
        hid_hi[i] = hi;
        hid_mid[i] = mid;
        hid_lo[i] = low;
    }
}

// out[t, r] = sum_s P[s][t][r]  (written, not added)
__global__ void shared_down_finish_kernel(const float* __restrict__ partial, int splits, int tokens, int H,
                                          float* __restrict__ out, int64_t out_stride) {
    const int vec_per_row = H / 4;
    const int64_t total = static_cast<int64_t>(tokens) * vec_per_row;
    const size_t plane = static_cast<size_t>(tokens) * vec_per_row;
    const float4* src = reinterpret_cast<const float4*>(partial);
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int t = static_cast<int>(i / vec_per_row);
        const int v = static_cast<int>(i - static_cast<int64_t>(t) * vec_per_row);
        float4 a = src[i];
        for (int s = 1; s < splits; ++s) {
            const float4 b = src[s * plane + i];
            a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
        }
        reinterpret_cast<float4*>(out + t * out_stride)[v] = a;
    }
}

struct SharedTcScratch {
    float* partial{nullptr};
    size_t floats{0};
};

// K-splits so that tiles x splits comes close to the SM count without exceeding it; every
// split must be a whole number of prefetch rounds.
int choose_splits(int tiles, int k_blocks, int sm_count) {
    int s = 1;
    while (s < 4 && tiles * s * 2 <= sm_count && k_blocks % (s * 2 * kPrefetch) == 0) s *= 2;
    return s;
}

template <bool kBf16>
void run(aeon_b200_ctx* ctx, const void* w1, const void* w3, const void* w2, const void* x, int64_t x_stride,
         int tokens, float* moe_accum, int64_t accum_stride, cudaStream_t stream) {
    const aeon_b200_moe_config& cfg = ctx->cfg;
    const int H = cfg.hidden, I = cfg.intermediate;
    const int token_tiles = (tokens + kMaxN - 1) / kMaxN;
    const int splits1 = choose_splits(token_tiles * (2 * I / kTileM), H / kTileK, ctx->sm_count);
    const int splits2 = choose_splits(token_tiles * (H / kTileM), 3 * (I / kTileK), ctx->sm_count);
    const size_t need = std::max(static_cast<size_t>(splits1) * tokens * 2 * I,
                                 static_cast<size_t>(splits2) * tokens * H);
    SharedTcScratch* s = static_cast<SharedTcScratch*>(ctx->shared_tc);
    if (s == nullptr) {
        s = new SharedTcScratch();
        ctx->shared_tc = s;
    }
    if (s->floats < need) {
        ctx_device_free(ctx, s->partial);
        s->partial = nullptr;
        s->floats = 0;
        s->partial = static_cast<float*>(ctx_device_alloc(ctx, need * sizeof(float), "shared expert split-K partials"));
        s->floats = need;
    }
    uint16_t* hi = reinterpret_cast<uint16_t*>(ctx->d_sh_hi);
    uint16_t* mid = reinterpret_cast<uint16_t*>(ctx->d_sh_mid);
    uint16_t* lo = reinterpret_cast<uint16_t*>(ctx->d_sh_lo);

    const CUtensorMap x_map = make_rowmajor16_map(x, tokens, H, x_stride);
    const CUtensorMap hi_map = make_rowmajor16_map(hi, tokens, I, I);
    const CUtensorMap mid_map = make_rowmajor16_map(mid, tokens, I, I);
    const CUtensorMap lo_map = make_rowmajor16_map(lo, tokens, I, I);
    // the dense weights, one 128-row box per k-block
    const CUtensorMap w1_map = make_rowmajor16_map(w1, I, H, H, kTileM);
    const CUtensorMap w3_map = make_rowmajor16_map(w3, I, H, H, kTileM);
    const CUtensorMap w2_map = make_rowmajor16_map(w2, H, I, I, kTileM);

    auto gemm1 = shared_dense_gemm_kernel<true, kBf16>;
    auto gemm2 = shared_dense_gemm_kernel<false, kBf16>;
    AEON_CUDA_CHECK(cudaFuncSetAttribute(gemm1, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
    AEON_CUDA_CHECK(cudaFuncSetAttribute(gemm2, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));

    DenseParams p{};
    p.wa = static_cast<const uint16_t*>(w1);
    p.wb = static_cast<const uint16_t*>(w3);
    p.K = H;
    p.rows = 2 * I;
    p.half_rows = I;
    p.tokens = tokens;
    p.planes = 1;
    p.splits = splits1;
    p.partial = s->partial;
    p.error = ctx->d_error;
    const int items1 = token_tiles * (2 * I / kTileM) * splits1;
    gemm1<<<std::min(items1, ctx->sm_count), kThreads, kSmemBytes, stream>>>(p, x_map, x_map, x_map, w1_map, w3_map);
    AEON_CUDA_CHECK(cudaGetLastError());
    {
        const int64_t total = static_cast<int64_t>(tokens) * I;
        const int blocks = static_cast<int>(std::min<int64_t>((total + 255) / 256, 8 * ctx->sm_count));
        shared_swiglu_finish_kernel<kBf16><<<blocks, 256, 0, stream>>>(s->partial, splits1, tokens, I,
                                                                       cfg.swiglu_limit, hi, mid, lo);
        AEON_CUDA_CHECK(cudaGetLastError());
    }
    p.wa = static_cast<const uint16_t*>(w2);
    p.wb = nullptr;
    p.K = I;
    p.rows = H;
    p.half_rows = 0;
    p.planes = 3;
    p.splits = splits2;
    const int items2 = token_tiles * (H / kTileM) * splits2;
    gemm2<<<std::min(items2, ctx->sm_count), kThreads, kSmemBytes, stream>>>(p, hi_map, mid_map, lo_map, w2_map, w2_map);
    AEON_CUDA_CHECK(cudaGetLastError());
    {
        const int64_t total = static_cast<int64_t>(tokens) * H / 4;
        const int blocks = static_cast<int>(std::min<int64_t>((total + 255) / 256, 8 * ctx->sm_count));
        shared_down_finish_kernel<<<blocks, 256, 0, stream>>>(s->partial, splits2, tokens, H, moe_accum,
                                                              accum_stride);
        AEON_CUDA_CHECK(cudaGetLastError());
    }
}

}  // namespace

void free_shared_tc_scratch(aeon_b200_ctx* ctx) {
    SharedTcScratch* s = static_cast<SharedTcScratch*>(ctx->shared_tc);
    if (!s) return;
    ctx_device_free(ctx, s->partial);
    delete s;
    ctx->shared_tc = nullptr;
}

bool shared_expert_tc_supports(const aeon_b200_moe_config& cfg, int64_t accum_stride) {
    // whole 128-row tiles, whole prefetch rounds per K-split, 16-byte output rows
    return cfg.hidden % 256 == 0 && cfg.intermediate % 256 == 0 && accum_stride % 4 == 0;
}

void launch_shared_expert_tc(aeon_b200_ctx* ctx, const void* w1, const void* w3, const void* w2,
                             const void* x, int64_t x_stride, int tokens, float* moe_accum,
                             int64_t accum_stride, cudaStream_t stream) {
    // One token tile (up to 256 tokens) per pass. The split-K partial sums and the hidden planes
    // are sized for one tile (the context's scratch holds max_tokens rows, and a tile is what
    // the 512 TMEM columns of a CTA accumulate), so a larger batch runs tile by tile; stream
    // order keeps the passes apart and the 88 MB of dense weights stay L2-resident between them.
    const uint16_t* xs = static_cast<const uint16_t*>(x);
    for (int t0 = 0; t0 < tokens; t0 += kMaxN) {
        const int n = std::min(kMaxN, tokens - t0);
        const void* xc = xs + static_cast<size_t>(t0) * x_stride;
        float* oc = moe_accum + static_cast<size_t>(t0) * accum_stride;
        if (ctx->cfg.act_dtype == AEON_B200_BF16)
            run<true>(ctx, w1, w3, w2, xc, x_stride, n, oc, accum_stride, stream);
        else
            run<false>(ctx, w1, w3, w2, xc, x_stride, n, oc, accum_stride, stream);
        ctx->launches += 4;
    }
}

}  // namespace aeon_b200
