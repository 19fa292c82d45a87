// Counting sort of the (token, slot) draws by expert id, plus the decode work list.
//
// Stands in for the reference's three permutation kernels
// (src/platform/ops/expert_permutation.hpp:50-128): histogram + exclusive scan ->
// expert_offsets[E+1]; deterministic placement in ascending draw order -> token_indices,
// draw_indices; weights gathered by position. The reference places with one thread per
// expert walking every draw (O(E * draws)); here each warp owns a contiguous chunk of
// draws, counts it with warp match/ballot, and a per-(warp, expert) running base makes the
// placement order-exact without any atomics, so the result is a pure function of the ids.
#include "common.cuh"

#include <algorithm>

namespace aeon_b200 {

namespace {

constexpr int kPermThreads = 1024;

__device__ __forceinline__ int block_exclusive_scan(int value, int* warp_sums, int* total) {
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    int inclusive = value;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const int v = __shfl_up_sync(0xFFFFFFFFu, inclusive, off);
        if (lane >= off) inclusive += v;
    }
    if (lane == 31) warp_sums[warp] = inclusive;
    __syncthreads();
    if (warp == 0) {
        int s = warp_sums[lane];
        int inc = s;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const int v = __shfl_up_sync(0xFFFFFFFFu, inc, off);
            if (lane >= off) inc += v;
        }
        warp_sums[lane] = inc - s;
        if (lane == 31) *total = inc;
    }
    __syncthreads();
    const int result = warp_sums[warp] + inclusive - value;
    __syncthreads();
    return result;
}

__global__ void __launch_bounds__(kPermThreads, 1)
expert_permutation_kernel(const int32_t* __restrict__ ids, int draws, int slots, int experts,
                          int walk_warps, int32_t* __restrict__ offsets,
                          int32_t* __restrict__ token_idx, int32_t* __restrict__ draw_idx,
                          const float* __restrict__ weights, float* __restrict__ wpos,
                          const int32_t* __restrict__ slot_of, WorkEntry* __restrict__ entries,
                          int32_t* __restrict__ counts, int skip_absent, int pool_slots, int entries_cap,
                          int32_t* __restrict__ error) {
    extern __shared__ int hist[];   // [walk_warps][experts]
    __shared__ int warp_sums[32];
    __shared__ int scan_total;

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;

    for (int i = tid; i < walk_warps * experts; i += kPermThreads) hist[i] = 0;
    __syncthreads();

    // Chunk of draws per walking warp, a multiple of 32 so a warp step never straddles.
    const int chunk = ((draws + walk_warps - 1) / walk_warps + 31) & ~31;
    const int begin = warp * chunk;
    const int end = min(begin + chunk, draws);
    const unsigned lt_mask = (1u << lane) - 1u;

    if (warp < walk_warps) {
        for (int d0 = begin; d0 < end; d0 += 32) {
            const int d = d0 + lane;
            int e = (d < end) ? ids[d] : -1;
            const bool valid = (e >= 0 && e < experts);
            const int key = valid ? e : -1 - lane;
            const unsigned peers = __match_any_sync(0xFFFFFFFFu, key);
            if (valid && (peers & lt_mask) == 0) hist[warp * experts + e] += __popc(peers);
            __syncwarp();
        }
    }
    __syncthreads();

    // Per-expert totals, exclusive scan, and per-(warp, expert) starting positions.
    int total = 0;
    if (tid < experts)
        for (int w = 0; w < walk_warps; ++w) total += hist[w * experts + tid];
    const int offset = block_exclusive_scan(tid < experts ? total : 0, warp_sums, &scan_total);
    const int placed = scan_total;
    if (tid < experts) {
        offsets[tid] = offset;
        int run = offset;
        for (int w = 0; w < walk_warps; ++w) {
            const int c = hist[w * experts + tid];
            hist[w * experts + tid] = run;
            run += c;
        }
    }
    if (tid == 0) offsets[experts] = placed;
    __syncthreads();

    if (warp < walk_warps) {
        for (int d0 = begin; d0 < end; d0 += 32) {
            const int d = d0 + lane;
            int e = (d < end) ? ids[d] : -1;
            const bool valid = (e >= 0 && e < experts);
            const int key = valid ? e : -1 - lane;
            const unsigned peers = __match_any_sync(0xFFFFFFFFu, key);
            if (valid) {
                const int pos = hist[warp * experts + e] + __popc(peers & lt_mask);
                if (index_ok(pos, draws, error)) {
                    token_idx[pos] = d / slots;
                    draw_idx[pos] = d;
                    if (weights != nullptr) wpos[pos] = weights[d];
                }
            }
            __syncwarp();
            if (valid && (peers & lt_mask) == 0) hist[warp * experts + e] += __popc(peers);
            __syncwarp();
        }
    }

    // Decode work list: one entry per (expert, group of up to 8 of its positions).
    if (entries != nullptr) {
        int my_slot = (tid < experts) ? (slot_of != nullptr ? slot_of[tid] : tid) : -1;
        // a slot at or above the declared pool size is reported and its expert treated as absent:
        // it must never become an address
        if (pool_slots > 0 && my_slot >= pool_slots) {
            if (error != nullptr) atomicCAS(error, kErrNone, kErrIdOutOfRange);
            my_slot = -1;
        }
        // An expert without a pool slot gets no entry when absent experts are skipped
        // (expert-parallel slice); otherwise it keeps its entries and the kernels flag it.
        const bool listed = tid < experts && !(skip_absent && my_slot < 0);
        const int chunks = listed ? (total + 7) / 8 : 0;
        const int ebase = block_exclusive_scan(chunks, warp_sums, &scan_total);
        const int n_entries = scan_total;
        const int distinct = block_exclusive_scan((listed && total > 0) ? 1 : 0, warp_sums,
                                                  &scan_total);
        (void)distinct;
        if (listed) {
            const int slot = my_slot;
            for (int c = 0; c < chunks; ++c) {
                WorkEntry w;
                w.expert = tid;
                w.pos0 = offset + 8 * c;
                w.ntok = min(8, total - 8 * c);
                w.slot = slot;
                if (index_ok(ebase + c, entries_cap, error)) entries[ebase + c] = w;
            }
        }
        if (tid == 0) {
            counts[0] = n_entries;
            counts[1] = scan_total;
            counts[2] = placed;
        }
    }
}

}  // namespace

void launch_permutation(aeon_b200_ctx* ctx, const int32_t* topk_ids, int tokens, int slots,
                        int experts, int32_t* expert_offsets, int32_t* token_indices,
                        int32_t* draw_indices, const float* weights, float* weights_by_position,
                        const int32_t* slot_of_expert, WorkEntry* entries, int32_t* counts,
                        bool skip_absent, cudaStream_t stream) {
    // the work list holds at most one entry per expert plus one per eight draws (rounded up per expert)
    const int entries_cap = experts + tokens * slots / 8 + 1;
    require(tokens >= 0 && slots > 0, "aeon_b200_expert_permutation: bad token or slot count");
    // An empty chunk is legal (the reference's permutation gate runs T = 0): only the
    // offsets are written then, so the per-draw arrays may be absent.
    require(expert_offsets != nullptr &&
                (tokens == 0 || (topk_ids && token_indices && draw_indices)),
            "aeon_b200_expert_permutation: null pointer argument");
    require(experts > 0 && experts <= kPermThreads,
            "aeon_b200_expert_permutation: experts must be in [1, 1024]");
    require(weights == nullptr || weights_by_position != nullptr || tokens == 0,
            "aeon_b200_expert_permutation: weights given without weights_by_position");
    const int draws = tokens * slots;
    int walk_warps = std::min(32, std::max(1, (40 * 1024) / (experts * 4)));
    walk_warps = std::min(walk_warps, std::max(1, (draws + 31) / 32));
    const size_t smem = static_cast<size_t>(walk_warps) * experts * sizeof(int);
    expert_permutation_kernel<<<1, kPermThreads, smem, stream>>>(
        topk_ids, draws, slots, experts, walk_warps, expert_offsets, token_indices, draw_indices,
        weights, weights_by_position, slot_of_expert, entries, counts, skip_absent ? 1 : 0, ctx->pool_slots,
        entries_cap, ctx->d_error);
    AEON_CUDA_CHECK(cudaGetLastError());
    ctx->launches += 1;
}

}  // namespace aeon_b200
