// Decode path of the routed-expert MoE FFN for sm_100a.
//
//   kernel A  (moe_w13_swiglu_kernel): per (expert, row tile) streams the int4 W1 and W3
//             rows and their fp16 group scales through a bulk-copy (TMA engine) /
//             mbarrier pipeline, unpacks nibbles in registers, multiplies them with the
//             expert's tokens on the warp MMA, applies the group scales in fp32, and
//             writes the clamped SwiGLU as an fp16 (hi, lo) pair.
//   kernel B  (moe_w2_accum_kernel): the same streaming for W2 over the (hi, lo) hidden,
//             writes weight * (W2 h) per draw, and the last CTA to finish an output row
//             tile adds the per-draw slices to the fp32 accumulator in slot order.
//
// Stands in for aeon_moe_fused_gate_up_kernel
// (src/backend/swizzled_w4a16/kernels/aeon_moe_fused_w13.hpp:27-111),
// aeon_moe_fused_w2_contrib_kernel (src/backend/swizzled_w4a16/kernels/aeon_moe_fused_w2.hpp:199-229)
// and moe_accumulate_fixed_order_kernel (src/platform/ops/moe_accumulate.hpp:73-92) of the
// reference. Differences that matter numerically: int4 values enter the MMA as exact
// fp16 integers and the fp16 group scale multiplies the fp32 group sum, so dequantisation
// is exact; the hidden vector is carried as hi + lo fp16 (about 22 bits) instead of one
// fp16; the output accumulator is fp32.
//
// Work decomposition. The draws of a call are sorted by expert (permutation.cu). A work
// entry is up to 8 consecutive positions of one expert; an item is (entry, row tile).
// CTAs are persistent and take items round-robin. Inside a CTA, warp 8 is the producer
// (one lane issues bulk copies), warps 0-7 consume: every pipeline stage covers 1024
// columns and consumer warp w owns columns [128w, 128w+128) of it, so the eight warps
// hold K-split partial sums that are added through shared memory at the end of an item.
//
// MMA mapping. The weight rows are the M operand (16 per MMA tile), the tokens the N
// operand (8), so lane (g = lane/4, t = lane%4) holds weight rows g and g+8 and token g.
// A lane reads one 16-byte atom (32 consecutive columns of one row) per row; the four
// lanes of a row cover the 128 columns of one scale group, and eight MMAs consume them.
// Which column lands in which MMA k-slot is irrelevant as long as the activation operand
// uses the same assignment, which is why the activations (and the hidden vector) are
// stored in a permuted column order: within each 128, column 32t + 8i + r sits at
// 32i + 8t + r, making the four lanes' 16-byte reads contiguous.
#include "common.cuh"
#include "ptx.cuh"

#include <algorithm>

namespace aeon_b200 {

namespace {

constexpr int kConsumerWarps = 8;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kThreads = kConsumerThreads + 32;
constexpr int kStageK = 1024;       // columns per pipeline stage
constexpr int kTokTile = 8;         // tokens per work entry (one MMA N tile)
constexpr int kPad = 64;            // bytes; shifts alternate rows by half the banks

struct DecodeParams {
    const uint8_t* pool;
    uint64_t payload_bytes;
    MatrixGeom w1, w2, w3;
    int H, I, top_k, tokens;
    const __half* xperm;
    const WorkEntry* entries;
    const int32_t* counts;
    const int32_t* token_idx;
    const int32_t* draw_idx;
    const float* wpos;
    const int32_t* topk_ids;
    const int32_t* slot_of;
    int skip_absent;
    int experts;
    __half* hid_hi;
    __half* hid_lo;
    float* contrib;
    int32_t* tile_done;
    float* accum;
    int64_t accum_stride;
    float limit;
    int32_t* error;
};

template <int G>
__device__ __forceinline__ int perm_col(int k) {
    if constexpr (G == 128) {
        const int r = k & 127;
        return (k & ~127) + ((r >> 3) & 3) * 32 + (r >> 5) * 8 + (r & 7);
    } else {
        return k;
    }
}

// ----- shared-memory geometry -------------------------------------------------------
template <int G, int MT>
struct GeomA {
    static constexpr int kBlocks = 4 * MT;                    // row-blocks (4 rows) per matrix
    static constexpr int kSeg = 4 * 512 + kPad;               // one row-block, one stage
    static constexpr int kScaleSeg = (G == 128) ? 64 : 256;   // scale bytes per row-block per stage
    static constexpr int kActRow = kStageK * 2 + kPad;
    static constexpr int kWeightBytes = 2 * kBlocks * kSeg;
    static constexpr int kScaleBytes = 2 * kBlocks * kScaleSeg;
    static constexpr int kActBytes = kTokTile * kActRow;
    static constexpr int kStageBytes = kWeightBytes + kScaleBytes + kActBytes;
    static constexpr int kRedBytes = kConsumerWarps * 2 * MT * 128 * 4;
    static constexpr int kStages = (MT == 1) ? 4 : 3;
    static constexpr int kSmem = 128 + kStages * kStageBytes + kRedBytes;
};

template <int G, int MT>
struct GeomB {
    static constexpr int kBlocks = 2 * MT;                    // row-blocks (8 rows)
    static constexpr int kSeg = 8 * 512;
    static constexpr int kScaleSeg = (G == 128) ? 128 : 512;
    static constexpr int kActRow = 2 * kStageK * 2 + kPad;    // hi then lo
    static constexpr int kWeightBytes = kBlocks * kSeg;
    static constexpr int kScaleBytes = kBlocks * kScaleSeg;
    static constexpr int kActBytes = kTokTile * kActRow;
    static constexpr int kStageBytes = kWeightBytes + kScaleBytes + kActBytes;
    static constexpr int kRedBytes = kConsumerWarps * MT * 128 * 4;
    static constexpr int kStages = 3;
    static constexpr int kSmem = 128 + kStages * kStageBytes + kRedBytes;
};

__device__ __forceinline__ void flag_error(int32_t* error, int code) {
    atomicCAS(error, kErrNone, code);
}

// ----- kernel A: W1/W3 dual product + clamped SwiGLU -----------------------------------
template <int G, int MT>
__global__ void __launch_bounds__(kThreads, 1)
moe_w13_swiglu_kernel(const DecodeParams p) {
    using S = GeomA<G, MT>;
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t smem_base = ptx::smem_u32(smem);
    const uint32_t full_bar = smem_base;                 // S::kStages x 8 B
    const uint32_t empty_bar = smem_base + 64;           // S::kStages x 8 B
    const uint32_t stage_base = smem_base + 128;
    float* red = reinterpret_cast<float*>(smem + 128 + S::kStages * S::kStageBytes);

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;

    if (tid == 0) {
        for (int s = 0; s < S::kStages; ++s) {
            ptx::mbar_init(full_bar + 8 * s, 1);
            ptx::mbar_init(empty_bar + 8 * s, kConsumerWarps);
        }
        ptx::fence_barrier_init();
    }
    __syncthreads();

    const int entries = p.counts[0];
    const int tiles = p.I / (16 * MT);
    const int total_items = entries * tiles;
    const int stages_per_item = p.H / kStageK;

    if (warp == kConsumerWarps) {
        // ---------------- producer ----------------
        if (lane != 0) return;
        const uint64_t stream_policy = ptx::policy_evict_first();
        const uint64_t keep_policy = ptx::policy_evict_last();
        uint32_t n = 0;
        for (int item = blockIdx.x; item < total_items; item += gridDim.x) {
            const int m = item / tiles;
            const int rt = item - m * tiles;
            const WorkEntry e = p.entries[m];
            if (e.slot < 0) flag_error(p.error, kErrExpertAbsent);
            const uint8_t* payload = p.pool + static_cast<uint64_t>(e.slot < 0 ? 0 : e.slot) * p.payload_bytes;
            const int block0 = rt * S::kBlocks;
            for (int ks = 0; ks < stages_per_item; ++ks, ++n) {
                const int s = n % S::kStages;
                const uint32_t parity = (n / S::kStages) & 1;
                if (!ptx::mbar_wait(empty_bar + 8 * s, parity ^ 1, p.error)) flag_error(p.error, kErrWaitTimeout);
                const uint32_t bar = full_bar + 8 * s;
                const uint32_t bytes = 2 * S::kBlocks * (2048 + S::kScaleSeg) + e.ntok * 2048;
                ptx::mbar_arrive_expect_tx(bar, bytes);
                const uint32_t sw = stage_base + s * S::kStageBytes;
                const uint32_t ss = sw + S::kWeightBytes;
                const uint32_t sa = ss + S::kScaleBytes;
#pragma unroll
                for (int mat = 0; mat < 2; ++mat) {
                    const MatrixGeom& g = mat == 0 ? p.w1 : p.w3;
                    const uint8_t* packed = payload + g.packed_offset;
                    const uint8_t* scales = payload + g.scale_offset;
                    for (int b = 0; b < S::kBlocks; ++b) {
                        ptx::bulk_g2s(sw + (mat * S::kBlocks + b) * S::kSeg,
                                      packed + static_cast<size_t>(block0 + b) * g.block_bytes + ks * 2048,
                                      2048, bar, stream_policy);
                        ptx::bulk_g2s(ss + (mat * S::kBlocks + b) * S::kScaleSeg,
                                      scales + static_cast<size_t>(block0 + b) * g.block_scale_bytes +
                                          ks * S::kScaleSeg,
                                      S::kScaleSeg, bar, stream_policy);
                    }
                }
                for (int tok = 0; tok < e.ntok; ++tok) {
                    const int token = p.token_idx[e.pos0 + tok];
                    ptx::bulk_g2s(sa + tok * S::kActRow,
                                  p.xperm + static_cast<size_t>(token) * p.H + ks * kStageK,
                                  2048, bar, keep_policy);
                }
            }
        }
        return;
    }

    // ---------------- consumers ----------------
    const int g = lane >> 2;
    const int t = lane & 3;
    const int ii = warp >> 1;     // 256-column iteration inside the stage
    const int hh = warp & 1;      // which 128-column half of it
    const int rib = g >> 1;       // row inside its 4-row block
    uint32_t n = 0;
    for (int item = blockIdx.x; item < total_items; item += gridDim.x) {
        const int m = item / tiles;
        const int rt = item - m * tiles;
        const WorkEntry e = p.entries[m];

        float acc[MT][2][4];
#pragma unroll
        for (int a = 0; a < MT; ++a)
#pragma unroll
            for (int b = 0; b < 2; ++b)
#pragma unroll
                for (int c = 0; c < 4; ++c) acc[a][b][c] = 0.f;

        for (int ks = 0; ks < stages_per_item; ++ks, ++n) {
            const int s = n % S::kStages;
            const uint32_t parity = (n / S::kStages) & 1;
            if (!ptx::mbar_wait(full_bar + 8 * s, parity, p.error)) flag_error(p.error, kErrWaitTimeout);
            __syncwarp();
            const uint32_t sw = stage_base + s * S::kStageBytes;
            const uint32_t ss = sw + S::kWeightBytes;
            const uint32_t sa = ss + S::kScaleBytes + g * S::kActRow;

            if constexpr (G == 128) {
                uint4 bfrag[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    bfrag[i] = (g < e.ntok) ? ptx::lds128(sa + (warp * 128 + i * 32 + t * 8) * 2)
                                            : make_uint4(0, 0, 0, 0);
                }
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
                    for (int mat = 0; mat < 2; ++mat) {
                        const int blk0 = mat * S::kBlocks + mt * 4 + (g & 1);
                        const int blk1 = blk0 + 2;
                        const uint32_t in_seg = ii * 512 + (rib * 8 + hh * 4 + t) * 16;
                        const uint4 qa = ptx::lds128(sw + blk0 * S::kSeg + in_seg);
                        const uint4 qb = ptx::lds128(sw + blk1 * S::kSeg + in_seg);
                        const uint32_t sc_off = ii * 16 + (rib * 2 + hh) * 2;
                        const float sca = ptx::lds_half_as_float(ss + blk0 * S::kScaleSeg + sc_off);
                        const float scb = ptx::lds_half_as_float(ss + blk1 * S::kScaleSeg + sc_off);
                        float tmp[4] = {0.f, 0.f, 0.f, 0.f};
                        const uint32_t wa[4] = {qa.x, qa.y, qa.z, qa.w};
                        const uint32_t wb[4] = {qb.x, qb.y, qb.z, qb.w};
                        const uint32_t bx[4] = {bfrag[0].x, bfrag[1].x, bfrag[2].x, bfrag[3].x};
                        const uint32_t by[4] = {bfrag[0].y, bfrag[1].y, bfrag[2].y, bfrag[3].y};
                        const uint32_t bz[4] = {bfrag[0].z, bfrag[1].z, bfrag[2].z, bfrag[3].z};
                        const uint32_t bw[4] = {bfrag[0].w, bfrag[1].w, bfrag[2].w, bfrag[3].w};
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            uint32_t pa[4], pb[4];
                            ptx::unpack_word(wa[i], pa);
                            ptx::unpack_word(wb[i], pb);
                            ptx::mma_f16(tmp, pa[0], pb[0], pa[1], pb[1], bx[i], by[i]);
                            ptx::mma_f16(tmp, pa[2], pb[2], pa[3], pb[3], bz[i], bw[i]);
                        }
                        acc[mt][mat][0] = fmaf(sca, tmp[0], acc[mt][mat][0]);
                        acc[mt][mat][1] = fmaf(sca, tmp[1], acc[mt][mat][1]);
                        acc[mt][mat][2] = fmaf(scb, tmp[2], acc[mt][mat][2]);
                        acc[mt][mat][3] = fmaf(scb, tmp[3], acc[mt][mat][3]);
                    }
                }
            } else {
                // group 32: the four lanes of a row share one atom (word t each), and the
                // scale applies after every two MMAs.
#pragma unroll
                for (int a = 0; a < 4; ++a) {
                    const int slice = hh * 4 + a;
                    const uint4 bf = (g < e.ntok) ? ptx::lds128(sa + (warp * 128 + a * 32 + t * 8) * 2)
                                                  : make_uint4(0, 0, 0, 0);
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
                        for (int mat = 0; mat < 2; ++mat) {
                            const int blk0 = mat * S::kBlocks + mt * 4 + (g & 1);
                            const int blk1 = blk0 + 2;
                            const uint32_t atom = ii * 512 + (rib * 8 + slice) * 16;
                            const uint32_t wa = ptx::lds32(sw + blk0 * S::kSeg + atom + t * 4);
                            const uint32_t wb = ptx::lds32(sw + blk1 * S::kSeg + atom + t * 4);
                            const uint32_t sc_off = ii * 64 + (rib * 8 + slice) * 2;
                            const float sca = ptx::lds_half_as_float(ss + blk0 * S::kScaleSeg + sc_off);
                            const float scb = ptx::lds_half_as_float(ss + blk1 * S::kScaleSeg + sc_off);
                            float tmp[4] = {0.f, 0.f, 0.f, 0.f};
                            uint32_t pa[4], pb[4];
                            ptx::unpack_word(wa, pa);
                            ptx::unpack_word(wb, pb);
                            ptx::mma_f16(tmp, pa[0], pb[0], pa[1], pb[1], bf.x, bf.y);
                            ptx::mma_f16(tmp, pa[2], pb[2], pa[3], pb[3], bf.z, bf.w);
                            acc[mt][mat][0] = fmaf(sca, tmp[0], acc[mt][mat][0]);
                            acc[mt][mat][1] = fmaf(sca, tmp[1], acc[mt][mat][1]);
                            acc[mt][mat][2] = fmaf(scb, tmp[2], acc[mt][mat][2]);
                            acc[mt][mat][3] = fmaf(scb, tmp[3], acc[mt][mat][3]);
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(empty_bar + 8 * s);
        }

        // K-split partials -> shared, fixed-order sum, SwiGLU, hi/lo store.
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int mat = 0; mat < 2; ++mat)
                *reinterpret_cast<float4*>(&red[((warp * 2 + mat) * MT + mt) * 128 + lane * 4]) =
                    make_float4(acc[mt][mat][0], acc[mt][mat][1], acc[mt][mat][2], acc[mt][mat][3]);
        ptx::named_bar_sync(1, kConsumerThreads);
        for (int o = tid; o < MT * 128; o += kConsumerThreads) {
            const int mt = o >> 7;
            const int idx = o & 127;
            float gate = 0.f, up = 0.f;
#pragma unroll
            for (int w = 0; w < kConsumerWarps; ++w) {
                gate += red[((w * 2 + 0) * MT + mt) * 128 + idx];
                up += red[((w * 2 + 1) * MT + mt) * 128 + idx];
            }
            const int lo = idx >> 2, c = idx & 3;
            const int go = lo >> 2, to = lo & 3;
            const int token = 2 * to + (c & 1);
            const int row_in_tile = (mt * 4 + (c >> 1) * 2 + (go & 1)) * 4 + (go >> 1);
            if (token < e.ntok) {
                gate = fminf(gate, p.limit);
                up = fminf(fmaxf(up, -p.limit), p.limit);
                const float h = (gate / (1.0f + expf(-gate))) * up;
                const __half hi = __float2half_rn(h);
                const __half lo16 = __float2half_rn(h - __half2float(hi));
                const int col = rt * (16 * MT) + row_in_tile;
                const size_t at = static_cast<size_t>(e.pos0 + token) * p.I + perm_col<G>(col);
                p.hid_hi[at] = hi;
                p.hid_lo[at] = lo16;
            }
        }
        ptx::named_bar_sync(1, kConsumerThreads);
    }
}

// ----- kernel B: W2 product, per-draw weighted slices, slot-order accumulate ------------
template <int G, int MT>
__global__ void __launch_bounds__(kThreads, 1)
moe_w2_accum_kernel(const DecodeParams p) {
    using S = GeomB<G, MT>;
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t smem_base = ptx::smem_u32(smem);
    const uint32_t full_bar = smem_base;
    const uint32_t empty_bar = smem_base + 64;
    const uint32_t stage_base = smem_base + 128;
    float* red = reinterpret_cast<float*>(smem + 128 + S::kStages * S::kStageBytes);
    __shared__ int s_last;

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;

    if (tid == 0) {
        for (int s = 0; s < S::kStages; ++s) {
            ptx::mbar_init(full_bar + 8 * s, 1);
            ptx::mbar_init(empty_bar + 8 * s, kConsumerWarps);
        }
        ptx::fence_barrier_init();
    }
    __syncthreads();

    const int entries = p.counts[0];
    constexpr int kRows = 16 * MT;
    const int tiles = p.H / kRows;
    const int total_items = entries * tiles;
    const int stages_per_item = p.I / kStageK;

    if (warp == kConsumerWarps) {
        if (lane != 0) return;
        const uint64_t stream_policy = ptx::policy_evict_first();
        const uint64_t keep_policy = ptx::policy_evict_last();
        uint32_t n = 0;
        for (int item = blockIdx.x; item < total_items; item += gridDim.x) {
            const int m = item / tiles;
            const int rt = item - m * tiles;
            const WorkEntry e = p.entries[m];
            const uint8_t* payload = p.pool + static_cast<uint64_t>(e.slot < 0 ? 0 : e.slot) * p.payload_bytes;
            const uint8_t* packed = payload + p.w2.packed_offset;
            const uint8_t* scales = payload + p.w2.scale_offset;
            const int block0 = rt * S::kBlocks;
            for (int ks = 0; ks < stages_per_item; ++ks, ++n) {
                const int s = n % S::kStages;
                const uint32_t parity = (n / S::kStages) & 1;
                if (!ptx::mbar_wait(empty_bar + 8 * s, parity ^ 1, p.error)) flag_error(p.error, kErrWaitTimeout);
                const uint32_t bar = full_bar + 8 * s;
                const uint32_t bytes = S::kBlocks * (S::kSeg + S::kScaleSeg) + e.ntok * 4096;
                ptx::mbar_arrive_expect_tx(bar, bytes);
                const uint32_t sw = stage_base + s * S::kStageBytes;
                const uint32_t ss = sw + S::kWeightBytes;
                const uint32_t sa = ss + S::kScaleBytes;
                for (int b = 0; b < S::kBlocks; ++b) {
                    ptx::bulk_g2s(sw + b * S::kSeg,
                                  packed + static_cast<size_t>(block0 + b) * p.w2.block_bytes + ks * S::kSeg,
                                  S::kSeg, bar, stream_policy);
                    ptx::bulk_g2s(ss + b * S::kScaleSeg,
                                  scales + static_cast<size_t>(block0 + b) * p.w2.block_scale_bytes +
                                      ks * S::kScaleSeg,
                                  S::kScaleSeg, bar, stream_policy);
                }
                for (int tok = 0; tok < e.ntok; ++tok) {
                    const size_t at = static_cast<size_t>(e.pos0 + tok) * p.I + ks * kStageK;
                    ptx::bulk_g2s(sa + tok * S::kActRow, p.hid_hi + at, 2048, bar, keep_policy);
                    ptx::bulk_g2s(sa + tok * S::kActRow + 2048, p.hid_lo + at, 2048, bar, keep_policy);
                }
            }
        }
        return;
    }

    const int g = lane >> 2;
    const int t = lane & 3;
    uint32_t n = 0;
    for (int item = blockIdx.x; item < total_items; item += gridDim.x) {
        const int m = item / tiles;
        const int rt = item - m * tiles;
        const WorkEntry e = p.entries[m];

        float acc[MT][4];
#pragma unroll
        for (int a = 0; a < MT; ++a)
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[a][c] = 0.f;

        for (int ks = 0; ks < stages_per_item; ++ks, ++n) {
            const int s = n % S::kStages;
            const uint32_t parity = (n / S::kStages) & 1;
            if (!ptx::mbar_wait(full_bar + 8 * s, parity, p.error)) flag_error(p.error, kErrWaitTimeout);
            __syncwarp();
            const uint32_t sw = stage_base + s * S::kStageBytes;
            const uint32_t ss = sw + S::kWeightBytes;
            const uint32_t sa = ss + S::kScaleBytes + g * S::kActRow;

            if constexpr (G == 128) {
                uint4 bhi[4], blo[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const uint32_t off = (warp * 128 + i * 32 + t * 8) * 2;
                    bhi[i] = (g < e.ntok) ? ptx::lds128(sa + off) : make_uint4(0, 0, 0, 0);
                    blo[i] = (g < e.ntok) ? ptx::lds128(sa + 2048 + off) : make_uint4(0, 0, 0, 0);
                }
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    const int blk0 = 2 * mt, blk1 = 2 * mt + 1;
                    const uint32_t in_seg = warp * 512 + (g * 4 + t) * 16;
                    const uint4 qa = ptx::lds128(sw + blk0 * S::kSeg + in_seg);
                    const uint4 qb = ptx::lds128(sw + blk1 * S::kSeg + in_seg);
                    const uint32_t sc_off = warp * 16 + g * 2;
                    const float sca = ptx::lds_half_as_float(ss + blk0 * S::kScaleSeg + sc_off);
                    const float scb = ptx::lds_half_as_float(ss + blk1 * S::kScaleSeg + sc_off);
                    float tmp[4] = {0.f, 0.f, 0.f, 0.f};
                    const uint32_t wa[4] = {qa.x, qa.y, qa.z, qa.w};
                    const uint32_t wb[4] = {qb.x, qb.y, qb.z, qb.w};
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        uint32_t pa[4], pb[4];
                        ptx::unpack_word(wa[i], pa);
                        ptx::unpack_word(wb[i], pb);
                        ptx::mma_f16(tmp, pa[0], pb[0], pa[1], pb[1], bhi[i].x, bhi[i].y);
                        ptx::mma_f16(tmp, pa[0], pb[0], pa[1], pb[1], blo[i].x, blo[i].y);
                        ptx::mma_f16(tmp, pa[2], pb[2], pa[3], pb[3], bhi[i].z, bhi[i].w);
                        ptx::mma_f16(tmp, pa[2], pb[2], pa[3], pb[3], blo[i].z, blo[i].w);
                    }
                    acc[mt][0] = fmaf(sca, tmp[0], acc[mt][0]);
                    acc[mt][1] = fmaf(sca, tmp[1], acc[mt][1]);
                    acc[mt][2] = fmaf(scb, tmp[2], acc[mt][2]);
                    acc[mt][3] = fmaf(scb, tmp[3], acc[mt][3]);
                }
            } else {
#pragma unroll
                for (int a = 0; a < 4; ++a) {
                    const uint32_t off = (warp * 128 + a * 32 + t * 8) * 2;
                    const uint4 bh = (g < e.ntok) ? ptx::lds128(sa + off) : make_uint4(0, 0, 0, 0);
                    const uint4 bl = (g < e.ntok) ? ptx::lds128(sa + 2048 + off) : make_uint4(0, 0, 0, 0);
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        const int blk0 = 2 * mt, blk1 = 2 * mt + 1;
                        const uint32_t atom = warp * 512 + (g * 4 + a) * 16;
                        const uint32_t wa = ptx::lds32(sw + blk0 * S::kSeg + atom + t * 4);
                        const uint32_t wb = ptx::lds32(sw + blk1 * S::kSeg + atom + t * 4);
                        const uint32_t sc_off = warp * 64 + (g * 4 + a) * 2;
                        const float sca = ptx::lds_half_as_float(ss + blk0 * S::kScaleSeg + sc_off);
                        const float scb = ptx::lds_half_as_float(ss + blk1 * S::kScaleSeg + sc_off);
                        float tmp[4] = {0.f, 0.f, 0.f, 0.f};
                        uint32_t pa[4], pb[4];
                        ptx::unpack_word(wa, pa);
                        ptx::unpack_word(wb, pb);
                        ptx::mma_f16(tmp, pa[0], pb[0], pa[1], pb[1], bh.x, bh.y);
                        ptx::mma_f16(tmp, pa[0], pb[0], pa[1], pb[1], bl.x, bl.y);
                        ptx::mma_f16(tmp, pa[2], pb[2], pa[3], pb[3], bh.z, bh.w);
                        ptx::mma_f16(tmp, pa[2], pb[2], pa[3], pb[3], bl.z, bl.w);
                        acc[mt][0] = fmaf(sca, tmp[0], acc[mt][0]);
                        acc[mt][1] = fmaf(sca, tmp[1], acc[mt][1]);
                        acc[mt][2] = fmaf(scb, tmp[2], acc[mt][2]);
                        acc[mt][3] = fmaf(scb, tmp[3], acc[mt][3]);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(empty_bar + 8 * s);
        }

#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
            *reinterpret_cast<float4*>(&red[(warp * MT + mt) * 128 + lane * 4]) =
                make_float4(acc[mt][0], acc[mt][1], acc[mt][2], acc[mt][3]);
        ptx::named_bar_sync(1, kConsumerThreads);
        for (int o = tid; o < MT * 128; o += kConsumerThreads) {
            const int mt = o >> 7;
            const int idx = o & 127;
            float sum = 0.f;
#pragma unroll
            for (int w = 0; w < kConsumerWarps; ++w) sum += red[(w * MT + mt) * 128 + idx];
            const int lo = idx >> 2, c = idx & 3;
            const int go = lo >> 2, to = lo & 3;
            const int token = 2 * to + (c & 1);
            const int row = rt * kRows + mt * 16 + go + 8 * (c >> 1);
            if (token < e.ntok) {
                const int pos = e.pos0 + token;
                const int draw = p.draw_idx[pos];
                p.contrib[static_cast<size_t>(draw) * p.H + row] = p.wpos[pos] * sum;
            }
        }
        __threadfence();
        ptx::named_bar_sync(1, kConsumerThreads);
        if (tid == 0) {
            const int prev = atomicAdd(&p.tile_done[rt], 1);
            s_last = (prev == entries - 1);
        }
        ptx::named_bar_sync(1, kConsumerThreads);
        if (s_last) {
            // Every entry's slice of this row tile is in memory: add the draws of each
            // token to the accumulator in slot order (one rounding chain, fixed order).
            __threadfence();
            for (int o = tid; o < p.tokens * kRows; o += kConsumerThreads) {
                const int token = o / kRows;
                const int row = rt * kRows + (o - token * kRows);
                float a = p.accum[static_cast<size_t>(token) * p.accum_stride + row];
                for (int slot = 0; slot < p.top_k; ++slot) {
                    const int draw = token * p.top_k + slot;
                    const int id = p.topk_ids[draw];
                    if (id >= 0 && id < p.experts && !(p.skip_absent && p.slot_of[id] < 0))
                        a += __ldcg(&p.contrib[static_cast<size_t>(draw) * p.H + row]);
                }
                p.accum[static_cast<size_t>(token) * p.accum_stride + row] = a;
            }
        }
    }
}

// ----- activation staging: 16-bit -> fp16 in the kernels' column order -------------------
template <int G>
__global__ void stage_activations_kernel(const void* __restrict__ x, int64_t x_stride, int dtype,
                                         int tokens, int H, __half* __restrict__ out) {
    const int64_t total = static_cast<int64_t>(tokens) * H;
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int token = static_cast<int>(i / H);
        const int k = static_cast<int>(i - static_cast<int64_t>(token) * H);
        float v;
        if (dtype == AEON_B200_BF16) {
            v = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(x)[token * x_stride + k]);
        } else {
            v = __half2float(reinterpret_cast<const __half*>(x)[token * x_stride + k]);
        }
        out[static_cast<size_t>(token) * H + perm_col<G>(k)] = __float2half_rn(v);
    }
}

template <int G, int MTA, int MTB>
void launch_decode_kernels(aeon_b200_ctx* ctx, const DecodeParams& p, cudaStream_t stream) {
    using SA = GeomA<G, MTA>;
    using SB = GeomB<G, MTB>;
    static bool configured = false;
    if (!configured) {
        AEON_CUDA_CHECK(cudaFuncSetAttribute(moe_w13_swiglu_kernel<G, MTA>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, SA::kSmem));
        AEON_CUDA_CHECK(cudaFuncSetAttribute(moe_w2_accum_kernel<G, MTB>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, SB::kSmem));
        configured = true;
    }
    cudaEvent_t* ev = nullptr;
    if (ctx->timing_enabled) {
        std::vector<cudaEvent_t>& pool = *ctx->timing_events;
        if (ctx->timing_used + 3 > pool.size()) {
            const size_t old = pool.size();
            pool.resize(old + 96);
            for (size_t i = old; i < pool.size(); ++i) AEON_CUDA_CHECK(cudaEventCreate(&pool[i]));
        }
        ev = &pool[ctx->timing_used];
        ctx->timing_used += 3;
        AEON_CUDA_CHECK(cudaEventRecord(ev[0], stream));
    }
    moe_w13_swiglu_kernel<G, MTA><<<ctx->sm_count, kThreads, SA::kSmem, stream>>>(p);
    AEON_CUDA_CHECK(cudaGetLastError());
    if (ev) AEON_CUDA_CHECK(cudaEventRecord(ev[1], stream));
    moe_w2_accum_kernel<G, MTB><<<ctx->sm_count, kThreads, SB::kSmem, stream>>>(p);
    AEON_CUDA_CHECK(cudaGetLastError());
    if (ev) AEON_CUDA_CHECK(cudaEventRecord(ev[2], stream));
    ctx->launches += 2;
}

__global__ void ep_combine_kernel(float* __restrict__ out, int64_t out_stride,
                                  const float* __restrict__ partials, int ranks, int tokens,
                                  int hidden) {
    const int64_t total = static_cast<int64_t>(tokens) * hidden / 4;
    const int64_t plane = static_cast<int64_t>(tokens) * hidden / 4;
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t token = (i * 4) / hidden;
        const int64_t col = (i * 4) - token * hidden;
        float4* dst = reinterpret_cast<float4*>(out + token * out_stride + col);
        float4 a = *dst;
        for (int r = 0; r < ranks; ++r) {
            const float4 v = reinterpret_cast<const float4*>(partials)[r * plane + i];
            a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w;
        }
        *dst = a;
    }
}

}  // namespace

void launch_ep_combine(float* out, int64_t out_stride, const float* partials, int ranks,
                       int tokens, int hidden, cudaStream_t stream) {
    require(out && partials, "aeon_b200_ep_combine: null pointer argument");
    require(ranks > 0 && tokens > 0 && hidden > 0 && hidden % 4 == 0 && out_stride % 4 == 0,
            "aeon_b200_ep_combine: hidden and out_stride must be multiples of 4");
    const int64_t total = static_cast<int64_t>(tokens) * hidden / 4;
    const int blocks = static_cast<int>(std::min<int64_t>((total + 255) / 256, 2048));
    ep_combine_kernel<<<blocks, 256, 0, stream>>>(out, out_stride, partials, ranks, tokens, hidden);
    AEON_CUDA_CHECK(cudaGetLastError());
}

void launch_moe_decode(aeon_b200_ctx* ctx, const void* pool_base, const int32_t* slot_of_expert,
                       const void* x, int64_t x_stride, const int32_t* topk_ids,
                       const float* topk_weights, int tokens, float* moe_accum,
                       int64_t accum_stride, uint32_t flags, cudaStream_t stream) {
    const aeon_b200_moe_config& cfg = ctx->cfg;
    require(pool_base && slot_of_expert && x && topk_ids && topk_weights && moe_accum,
            "aeon_b200_moe_decode: null pointer argument");
    require(tokens > 0 && tokens <= ctx->max_tokens,
            "aeon_b200_moe_decode: tokens must be in [1, max_tokens of the context]");
    require(x_stride >= cfg.hidden && accum_stride >= cfg.hidden,
            "aeon_b200_moe_decode: row strides must be at least the hidden width");

    // 1. activations -> fp16 in kernel column order
    const int64_t total = static_cast<int64_t>(tokens) * cfg.hidden;
    const int blocks = static_cast<int>(std::min<int64_t>((total + 255) / 256, 4 * ctx->sm_count));
    if (cfg.group_size == 128) {
        stage_activations_kernel<128><<<blocks, 256, 0, stream>>>(x, x_stride, cfg.act_dtype, tokens,
                                                                  cfg.hidden, ctx->d_xperm);
    } else {
        stage_activations_kernel<32><<<blocks, 256, 0, stream>>>(x, x_stride, cfg.act_dtype, tokens,
                                                                 cfg.hidden, ctx->d_xperm);
    }
    AEON_CUDA_CHECK(cudaGetLastError());
    ctx->launches += 1;

    // 2. draws sorted by expert + work list
    launch_permutation(ctx, topk_ids, tokens, cfg.top_k, cfg.experts, ctx->d_offsets,
                       ctx->d_token_idx, ctx->d_draw_idx, topk_weights, ctx->d_wpos,
                       slot_of_expert, ctx->d_entries, ctx->d_counts,
                       (flags & AEON_B200_DECODE_SKIP_ABSENT) != 0, stream);

    // 3. the two streaming kernels
    DecodeParams p{};
    p.pool = static_cast<const uint8_t*>(pool_base);
    p.payload_bytes = ctx->geom.payload_bytes;
    p.w1 = ctx->geom.w1;
    p.w2 = ctx->geom.w2;
    p.w3 = ctx->geom.w3;
    p.H = cfg.hidden;
    p.I = cfg.intermediate;
    p.top_k = cfg.top_k;
    p.tokens = tokens;
    p.xperm = ctx->d_xperm;
    p.entries = ctx->d_entries;
    p.counts = ctx->d_counts;
    p.token_idx = ctx->d_token_idx;
    p.draw_idx = ctx->d_draw_idx;
    p.wpos = ctx->d_wpos;
    p.topk_ids = topk_ids;
    p.slot_of = slot_of_expert;
    p.skip_absent = (flags & AEON_B200_DECODE_SKIP_ABSENT) ? 1 : 0;
    p.experts = cfg.experts;
    p.hid_hi = ctx->d_hidden_hi;
    p.hid_lo = ctx->d_hidden_lo;
    p.contrib = ctx->d_contrib;
    p.tile_done = ctx->d_tile_done;
    p.accum = moe_accum;
    p.accum_stride = accum_stride;
    p.limit = cfg.swiglu_limit;
    p.error = ctx->d_error;

    if (cfg.group_size == 128) {
        launch_decode_kernels<128, 1, 2>(ctx, p, stream);
    } else {
        launch_decode_kernels<32, 1, 2>(ctx, p, stream);
    }
}

}  // namespace aeon_b200
