// Prefill path: per-expert grouped GEMMs on the tcgen05 tensor cores of sm_100a.
//
// Stands in for the reference's grouped expert pair and its scheduler:
// moe_grouped_gate_up_kernel / moe_grouped_down_kernel
// (src/platform/rdna3/moe_grouped_ffn.hpp:77-288), the dequantising feed
// (src/backend/swizzled_w4a16/kernels/swizzled_w4a16_feed.hpp:52-92) and
// run_moe_grouped_expert_batch (src/architecture/deepseek_v4/moe/moe_grouped_batch.hpp:55-147).
// The reference batches experts eight at a time from the host after a device-to-host copy of
// the offsets; here the tile list is built on the device and one persistent launch per GEMM
// walks it, so there is no host round trip and no per-launch expert limit.
//
// Shape of one tile. The weight rows are the MMA M dimension, the expert's tokens the N
// dimension (16..128, so ragged token counts cost little), K runs in blocks of 64. A CTA tile is
// 256 weight rows: two 128-row MMAs per k-step that share one activation tile in shared memory,
//     D_h[128 weight rows, N tokens] += Wq_h[128, 64] * X[N, 64]^T   h = 0, 1   (tcgen05.mma kind::f16)
// so every activation byte that comes up from L2 feeds 256 weight rows. (With 128-row CTA tiles
// each k-block pulled 16 KB of activations for 1 M MACs and the kernel sat at the L2-to-SM
// bandwidth and TMA latency of that stream, not at the tensor pipe: doubling the dequantising
// warps changed nothing.) The fp32 accumulators live in tensor memory: two buffers of two
// 128-column halves, so the epilogue of one tile overlaps the main loop of the next.
//
// Warp roles of a CTA (480 threads):
//   warps 0-3   epilogue: tcgen05.ld their TMEM lane quadrant of both halves, finish (SwiGLU /
//               routing weight), store;
//   warps 4-11  dequantise: one thread per weight row of the 256-row tile. Per k-block a thread
//               loads its row's two packed atoms (32 bytes, four k-blocks ahead) and the scale,
//               converts the 64 int4 values to fp16(q * scale) in registers and writes the row's
//               128 bytes into the 128-byte-swizzled K-major operand tile in shared memory. The
//               loop is unrolled over the ring so stage indices, parities' positions and every
//               address offset are compile-time constants: profiling the first form (two
//               threads per row, run-time stage arithmetic) showed the kernel bound by issued
//               instructions -- 3,000 warp instructions per k-block, of which the conversion
//               itself needs about 900 -- not by the tensor pipe, HBM, L2 or shared memory
//               (leaving out the stores, the conversion arithmetic, the activation loads or
//               even the MMAs each changed the time by less than 15 %);
//   warp 12     one thread issues the tiled TMA loads of the activation operand (no multicast);
//   warps 13-14 one thread each issues the MMAs and the commits of one 128-row half; warp 13
//               owns the TMEM allocation.
// A 4-stage ring of (weight tile, activation tile) pairs connects them through mbarriers.
// Every wait is bounded; a wait that runs out sets the context's error flag, after which all
// waits fall through and the kernel ends (TMEM is always freed).
//
// Numerics. MMA operands are fp16: the weight operand is fp16(q * scale) (one rounding of the
// exact product), activations are the 16-bit inputs converted to fp16, the hidden vector is
// rounded to fp16 between the two GEMMs, accumulation is fp32. The parity oracle applies the
// same three roundings (the method of the reference's own grouped gate,
// tests/test_v4_grouped_wmma_oracle.cpp:63-73,219-228).
//
// GEMM 1 puts W1 in the first 128-row half of a CTA tile and the same rows of W3 in the second:
// the gate and the up value of a hidden element sit in the same TMEM lane of the two accumulator
// halves, so one epilogue thread reads both and no lane is idle or shuffling.
#include "common.cuh"
#include "ptx.cuh"
#include "tc5.cuh"
#include "tensor_map.cuh"

#include <algorithm>
#include <type_traits>

namespace aeon_b200 {

namespace {

constexpr int kHalfM = 128;         // weight rows per MMA (the TMEM lanes)
constexpr int kHalves = 2;          // MMAs per k-step that share the activation tile
constexpr int kTileM = kHalfM * kHalves;   // weight rows per CTA tile
constexpr int kTileK = 64;          // K per pipeline stage (one 128-byte swizzled row)
constexpr int kMaxN = 128;          // tokens per tile
constexpr int kStages = 4;
constexpr int kEpilogueWarps = 4;
constexpr int kDequantWarps = kTileM / 32;            // one thread per weight row of the tile
constexpr int kPrefetch = 4;         // k-blocks of packed weights a dequantising thread keeps in flight
constexpr int kTmaWarp = kEpilogueWarps + kDequantWarps;
constexpr int kMmaWarp0 = kTmaWarp + 1;       // one MMA-issuing warp per 128-row half
constexpr int kThreads = (kMmaWarp0 + kHalves) * 32;
constexpr int kHalfA = kHalfM * kTileK * 2;           // 16 KB: one half's operand tile
constexpr int kStageA = kHalves * kHalfA;             // 32 KB
constexpr int kStageB = kMaxN * kTileK * 2;           // 16 KB
constexpr int kSmemBytes = 1024 /*align*/ + kStages * (kStageA + kStageB) + 256 /*barriers*/;
constexpr int kTmemCols = 512;

struct PrefillTile {
    int slot;      // pool slot of the expert
    int pos0;      // first position (expert-sorted order)
    int ntok;      // tokens of this tile (<= kMaxN)
    int pad;
};

struct PrefillParams {
    const uint8_t* pool;
    uint64_t payload_bytes;
    MatrixGeom w1, w2, w3;
    int group;
    int H, I;
    const PrefillTile* tiles;
    const int32_t* n_tiles;
    const int32_t* draw_idx;
    const float* wpos;
    __half* hidden;       // [positions, I] fp16
    float* contrib;       // [draws, H] fp32
    float limit;
    int32_t* error;
    // extents for the bounds-checked build
    int draws_cap;        // rows of hidden / contrib, entries of draw_idx / wpos
    int tiles_cap;        // tiles
};

__device__ __forceinline__ void flag_error(int32_t* error, int code) { atomicCAS(error, kErrNone, code); }

__device__ __forceinline__ uint4 ldg128(const uint8_t* p) {
    uint4 v;
    asm("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}

// One packed word (8 columns) -> 8 fp16 values fp16((nibble - 8) * scale) in column order.
__device__ __forceinline__ uint4 dequant_word(uint32_t w, uint32_t scale2) {
    uint32_t p[4];
    ptx::unpack_word(w, p);     // exact integers nibble - 8 as fp16 pairs
    return make_uint4(hmul2_u32(p[0], scale2), hmul2_u32(p[1], scale2), hmul2_u32(p[2], scale2),
                      hmul2_u32(p[3], scale2));
}

// kGateUp: GEMM 1 (W1/W3 interleaved rows, K = hidden, SwiGLU epilogue -> hidden fp16)
// else:    GEMM 2 (W2 rows, K = intermediate, routing-weight epilogue -> contrib fp32)
template <bool kGateUp, int G>
__global__ void __launch_bounds__(kThreads, 1)
moe_grouped_gemm_kernel(const PrefillParams p, const __grid_constant__ CUtensorMap act_map) {
    extern __shared__ uint8_t smem_raw[];
    // the swizzled operand tiles need 1024-byte alignment
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
            ptx::mbar_init(full_bar + 8 * s, kDequantWarps + 1);
            ptx::mbar_init(empty_bar + 8 * s, kHalves);      // one commit per MMA-issuing thread
        }
        for (int b = 0; b < 2; ++b) {
            ptx::mbar_init(acc_full + 8 * b, kHalves);
            ptx::mbar_init(acc_empty + 8 * b, kEpilogueWarps);
        }
        ptx::fence_barrier_init();
    }
    if (warp == kMmaWarp0) {
        tc5::tmem_alloc(tmem_slot, kTmemCols);
        tc5::tmem_relinquish();
    }
    tc5::fence_before_sync();
    __syncthreads();
    tc5::fence_after_sync();
    const uint32_t tmem_base = *tmem_slot_gen;

    const int K = kGateUp ? p.H : p.I;
    const int row_blocks = kGateUp ? p.I / kHalfM : p.H / kTileM;
    const int kblocks = K / kTileK;
    const int n_tiles = index_ok(*p.n_tiles, p.tiles_cap + 1, p.error) ? *p.n_tiles : 0;
    const int total_items = n_tiles * row_blocks;

    if (warp == kTmaWarp) {
        // ------------------------------ TMA: activation operand ------------------------------
        if (lane == 0) {
            const int rounds = kblocks / kStages;
            uint32_t phase = 0;
            for (int item = blockIdx.x; item < total_items; item += gridDim.x) {
                const PrefillTile tile = p.tiles[item / row_blocks];
                const bool two_boxes = tile.ntok > 64;                  // a box is 64 token rows
                const uint32_t bytes = (two_boxes ? 2 : 1) * 64 * kTileK * 2;
                for (int j = 0; j < rounds; ++j) {
#pragma unroll
                    for (int i = 0; i < kStages; ++i) {
                        const int k0 = (j * kStages + i) * kTileK;
                        if (!ptx::mbar_wait(empty_bar + 8 * i, phase ^ 1, p.error)) flag_error(p.error, kErrWaitTimeout);
                        ptx::mbar_arrive_expect_tx(full_bar + 8 * i, bytes);
                        tc5::tma_load_2d(b_smem + i * kStageB, &act_map, k0, tile.pos0, full_bar + 8 * i);
                        if (two_boxes)
                            tc5::tma_load_2d(b_smem + i * kStageB + 64 * kTileK * 2, &act_map, k0, tile.pos0 + 64,
                                             full_bar + 8 * i);
                    }
                    phase ^= 1;
                }
            }
        }
    } else if (warp >= kMmaWarp0) {
        // ------------------------------ MMA issue ---------------------------------------------
        // One thread per 128-row half, each with its own accumulator columns. A single thread
        // issuing both halves was the kernel's limit: per k-block it ran eight MMAs plus sixteen
        // descriptor constructions and the ring arithmetic as one serial instruction stream,
        // about 1,100 cycles against 320 of tensor time. Here the round over the ring is unrolled,
        // so a descriptor is the base descriptor plus a constant, and each thread issues four MMAs.
        const int h = warp - kMmaWarp0;
        if (lane == 0) {
            const uint64_t a_desc0 = tc5::smem_desc_sw128(a_smem + h * kHalfA);
            const uint64_t b_desc0 = tc5::smem_desc_sw128(b_smem);
            const int rounds = kblocks / kStages;
            uint32_t phase = 0, it = 0;
            for (int item = blockIdx.x; item < total_items; item += gridDim.x, ++it) {
                const PrefillTile tile = p.tiles[item / row_blocks];
                const uint32_t n_mma = static_cast<uint32_t>((tile.ntok + 15) & ~15);
                const uint32_t idesc = tc5::idesc_f16(kHalfM, n_mma);
                const uint32_t buf = it & 1;
                if (!ptx::mbar_wait(acc_empty + 8 * buf, ((it >> 1) & 1) ^ 1, p.error))
                    flag_error(p.error, kErrWaitTimeout);
                tc5::fence_after_sync();
                const uint32_t d_tmem = tmem_base + buf * (kHalves * kMaxN) + h * kMaxN;
                for (int j = 0; j < rounds; ++j) {
#pragma unroll
                    for (int i = 0; i < kStages; ++i) {
                        if (!ptx::mbar_wait(full_bar + 8 * i, phase, p.error)) flag_error(p.error, kErrWaitTimeout);
                        tc5::fence_after_sync();
#pragma unroll
                        for (int kk = 0; kk < kTileK / 16; ++kk) {
                            // the start-address field counts 16-byte units: adding a byte offset >> 4 moves the tile
                            tc5::mma_f16_ss(d_tmem, a_desc0 + ((i * kStageA + kk * 32) >> 4),
                                            b_desc0 + ((i * kStageB + kk * 32) >> 4), idesc,
                                            (i == 0 && kk == 0) ? (j != 0 ? 1u : 0u) : 1u);
                        }
                        tc5::commit(empty_bar + 8 * i);      // this half is done with the stage
                    }
                    phase ^= 1;
                }
                tc5::commit(acc_full + 8 * buf);             // this half's accumulator is complete
            }
        }
    } else if (warp >= kEpilogueWarps) {
        // ------------------------------ dequantise the weight operand ------------------------
        // Thread (mh, r) owns row r of 128-row half mh for the whole item. Round j covers the four
        // k-blocks 4j .. 4j+3, which are exactly the four ring stages in order (an item starts on a
        // multiple of four k-blocks), so inside the unrolled round the stage, the shared-memory
        // address and the load offsets are constants and only the phase bit changes per round.
        const int d = tid - kEpilogueWarps * 32;
        const int mh = d / kHalfM;
        const int r = d - mh * kHalfM;
        // chunk c (16 bytes, 8 columns) of the row goes to position c ^ (r & 7) of its 128-byte line
        uint8_t* const row_dst = smem_gen + mh * kHalfA + (r >> 3) * 1024 + (r & 7) * 128;
        const uint32_t swz = static_cast<uint32_t>(r & 7) << 4;
        // The swizzle configuration is fixed per matrix kind (validated with the config):
        // W1/W3 rows come 4 to a 512-byte line with 8 atoms each, W2 rows 8 with 4 atoms.
        constexpr int RPW = kGateUp ? 4 : 8, LPR = kGateUp ? 8 : 4;
        constexpr int apg = G / 32;                    // atoms per scale group
        constexpr int kScaleLineBytes = 32 / apg * 2;  // scale bytes per 512-byte line
        constexpr int kRoundBytes = (8 / LPR) * 512;   // packed bytes a row advances per round (8 atoms)
        constexpr int kRoundScaleBytes = (8 / LPR) * kScaleLineBytes;
        uint32_t phase = 0;                            // parity of the ring pass the next round fills
        for (int item = blockIdx.x; item < total_items; item += gridDim.x) {
            const int ti = item / row_blocks;
            const int rb = item - ti * row_blocks;
            const PrefillTile tile = p.tiles[ti];
            const uint8_t* payload = p.pool + static_cast<uint64_t>(tile.slot < 0 ? 0 : tile.slot) * p.payload_bytes;
            const MatrixGeom* gm;
            int row;
            if constexpr (kGateUp) {
                gm = mh ? &p.w3 : &p.w1;               // first half: gate rows, second half: up rows
                row = rb * kHalfM + r;
            } else {
                gm = &p.w2;
                row = rb * kTileM + mh * kHalfM + r;
            }
            const int blk = row / RPW, rib = row - blk * RPW;
            // atom a of the row (32 columns): line a / LPR, position rib * LPR + a % LPR; k-block kb is
            // the atom pair (2 kb, 2 kb + 1), adjacent in its line
            const uint8_t* packed = payload + gm->packed_offset + static_cast<size_t>(blk) * gm->block_bytes +
                                    (rib * LPR) * 16;
            const uint8_t* scales = payload + gm->scale_offset + static_cast<size_t>(blk) * gm->block_scale_bytes +
                                    rib * (LPR / apg) * 2;
            // k-block i of a round: its 32 packed bytes and its scale(s), as offsets from the round's base
            auto fetch = [&](const uint8_t* pk, const uint8_t* sc, int i, uint4& q0, uint4& q1, uint32_t& s2) {
                const int a = 2 * i;                                   // first atom of the k-block within the round
                const int off = (a / LPR) * 512 + (a % LPR) * 16;
                q0 = ldg128(pk + off);
                q1 = ldg128(pk + off + 16);
                // raw loads only: any arithmetic on the values here would wait for them
                const int soff = (a / LPR) * kScaleLineBytes + ((a % LPR) / apg) * 2;
                if constexpr (apg == 1) s2 = __ldg(reinterpret_cast<const uint32_t*>(sc + soff));      // two atoms, two scales
                else s2 = __ldg(reinterpret_cast<const uint16_t*>(sc + soff));                         // one scale for both
            };
            uint4 qa[kStages], qb[kStages];
            uint32_t sbuf[kStages];
#pragma unroll
            for (int i = 0; i < kStages; ++i) fetch(packed, scales, i, qa[i], qb[i], sbuf[i]);
            const int rounds = kblocks / kStages;
            for (int j = 0; j < rounds; ++j) {
                const bool more = j + 1 < rounds;
                packed += kRoundBytes;
                scales += kRoundScaleBytes;
#pragma unroll
                for (int i = 0; i < kStages; ++i) {
                    const uint4 q0 = qa[i], q1 = qb[i];
                    const uint32_t sraw = sbuf[i];
                    if (more) fetch(packed, scales, i, qa[i], qb[i], sbuf[i]);
                    uint32_t s2a, s2b;                              // the scale in both halves of a word
                    if constexpr (apg == 1) {
                        s2a = (sraw & 0xFFFFu) * 0x10001u;
                        s2b = (sraw >> 16) * 0x10001u;
                    } else {
                        s2a = s2b = sraw * 0x10001u;
                    }
                    if (!ptx::mbar_wait(empty_bar + 8 * i, phase ^ 1, p.error)) flag_error(p.error, kErrWaitTimeout);
                    uint8_t* dst = row_dst + i * kStageA;
                    *reinterpret_cast<uint4*>(dst + ((0u << 4) ^ swz)) = dequant_word(q0.x, s2a);
                    *reinterpret_cast<uint4*>(dst + ((1u << 4) ^ swz)) = dequant_word(q0.y, s2a);
                    *reinterpret_cast<uint4*>(dst + ((2u << 4) ^ swz)) = dequant_word(q0.z, s2a);
                    *reinterpret_cast<uint4*>(dst + ((3u << 4) ^ swz)) = dequant_word(q0.w, s2a);
                    *reinterpret_cast<uint4*>(dst + ((4u << 4) ^ swz)) = dequant_word(q1.x, s2b);
                    *reinterpret_cast<uint4*>(dst + ((5u << 4) ^ swz)) = dequant_word(q1.y, s2b);
                    *reinterpret_cast<uint4*>(dst + ((6u << 4) ^ swz)) = dequant_word(q1.z, s2b);
                    *reinterpret_cast<uint4*>(dst + ((7u << 4) ^ swz)) = dequant_word(q1.w, s2b);
                    // generic-proxy writes must be visible to the tensor core (async proxy)
                    ptx::fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(full_bar + 8 * i);
                }
                phase ^= 1;
            }
        }
    } else {
        // ------------------------------ epilogue -------------------------------------------------
        const int quad = warp;                              // TMEM lanes 32*quad .. +31
        uint32_t it = 0;
        for (int item = blockIdx.x; item < total_items; item += gridDim.x, ++it) {
            const int ti = item / row_blocks;
            const int rb = item - ti * row_blocks;
            const PrefillTile tile = p.tiles[ti];
            // GEMM 2: the tile's draw rows and routing weights do not depend on the accumulators, so they
            // are fetched before the wait: lane j holds position 32 c + j of chunk c
            int my_draw[kMaxN / 32];
            float my_w[kMaxN / 32];
            if constexpr (!kGateUp) {
#pragma unroll
                for (int c = 0; c < kMaxN / 32; ++c) {
                    const int my_pos = tile.pos0 + c * 32 + lane;
                    const bool have = c * 32 + lane < tile.ntok && index_ok(my_pos, p.draws_cap, p.error);
                    my_draw[c] = have ? p.draw_idx[my_pos] : -1;
                    my_w[c] = have ? p.wpos[my_pos] : 0.f;
                    if (have && !index_ok(my_draw[c], p.draws_cap, p.error)) my_draw[c] = -1;
                }
            }
            const uint32_t buf = it & 1;
            if (!ptx::mbar_wait(acc_full + 8 * buf, (it >> 1) & 1, p.error)) flag_error(p.error, kErrWaitTimeout);
            tc5::fence_after_sync();
            const uint32_t tlane = tmem_base + ((static_cast<uint32_t>(quad) * 32u) << 16) + buf * (kHalves * kMaxN);
            if constexpr (kGateUp) {
                // lane L of the first half holds the gate of hidden column rb*128 + L, the same lane of
                // the second half its up value: one thread finishes the element. The hidden vector is
                // rounded to fp16 right after, so the fast exponential and division cost nothing visible.
                const int hcol = rb * kHalfM + quad * 32 + lane;
                for (int c0 = 0; c0 < tile.ntok; c0 += 16) {
                    uint32_t gv[16], uv[16];
                    tc5::ld_32x16(tlane + c0, gv);
                    tc5::ld_32x16(tlane + kMaxN + c0, uv);
                    tc5::ld_wait();
                    __half* out = p.hidden + static_cast<size_t>(tile.pos0 + c0) * p.I + hcol;
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        if (c0 + j < tile.ntok && index_ok(tile.pos0 + c0 + j, p.draws_cap, p.error)) {
                            const float gate = fminf(__uint_as_float(gv[j]), p.limit);
                            const float up = fminf(fmaxf(__uint_as_float(uv[j]), -p.limit), p.limit);
                            const float hv = __fdividef(gate, 1.0f + __expf(-gate)) * up;
                            out[static_cast<size_t>(j) * p.I] = __float2half_rn(hv);
                        }
                    }
                }
            } else {
                for (int h = 0; h < kHalves; ++h) {
                    const int row = rb * kTileM + h * kHalfM + quad * 32 + lane;
#pragma unroll
                    for (int c = 0; c < kMaxN / 32; ++c) {
                        if (c * 32 >= tile.ntok) break;
                        uint32_t v[32];
                        tc5::ld_32x32(tlane + h * kMaxN + c * 32, v);
                        tc5::ld_wait();
                        // every lane takes the chunk's draws and weights by shuffle instead of 2 x 32 dependent loads
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const int draw = __shfl_sync(0xFFFFFFFFu, my_draw[c], j);
                            const float wj = __shfl_sync(0xFFFFFFFFu, my_w[c], j);
                            if (draw >= 0) p.contrib[static_cast<size_t>(draw) * p.H + row] = wj * __uint_as_float(v[j]);
                        }
                    }
                }
            }
            tc5::fence_before_sync();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(acc_empty + 8 * buf);
        }
    }

    tc5::fence_before_sync();
    __syncthreads();
    if (warp == kMmaWarp0) {
        tc5::fence_after_sync();
        tc5::tmem_dealloc(tmem_base, kTmemCols);
    }
}

// Activation rows gathered into expert-sorted order as fp16: xg[pos, :] = fp16(x[token_idx[pos], :]).
__global__ void gather_activations_kernel(const void* __restrict__ x, int64_t x_stride, int dtype,
                                          const int32_t* __restrict__ token_idx,
                                          const int32_t* __restrict__ counts, int H,
                                          __half* __restrict__ xg, int tokens, int draws_cap,
                                          int32_t* __restrict__ error) {
    const int placed = index_ok(counts[2], draws_cap + 1, error) ? counts[2] : 0;
    const int vec_per_row = H / 8;
    const int64_t total = static_cast<int64_t>(placed) * vec_per_row;
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int pos = static_cast<int>(i / vec_per_row);
        const int v = static_cast<int>(i - static_cast<int64_t>(pos) * vec_per_row);
        const int token = token_idx[pos];
        if (!index_ok(token, tokens, error)) continue;      // a token index outside the batch: reported, row left as it is
        const uint4 in = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(x) + token * x_stride)[v];
        uint4 out = in;
        if (dtype == AEON_B200_BF16) {
            const uint32_t w[4] = {in.x, in.y, in.z, in.w};
            uint32_t o[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float lo = __uint_as_float(w[k] << 16), hi = __uint_as_float(w[k] & 0xFFFF0000u);
                const __half2 h = __floats2half2_rn(lo, hi);
                o[k] = *reinterpret_cast<const uint32_t*>(&h);
            }
            out = make_uint4(o[0], o[1], o[2], o[3]);
        }
        reinterpret_cast<uint4*>(xg + static_cast<size_t>(pos) * H)[v] = out;
    }
}

// Tile list: every expert's positions in runs of at most kMaxN. One CTA; experts <= 1024.
__global__ void build_tiles_kernel(const int32_t* __restrict__ offsets, const int32_t* __restrict__ slot_of,
                                   int experts, int skip_absent, PrefillTile* __restrict__ tiles,
                                   int32_t* __restrict__ n_tiles, int32_t* __restrict__ error, int pool_slots,
                                   int tiles_cap) {
    __shared__ int base[1025];
    const int e = threadIdx.x;
    int count = 0, slot = -1;
    if (e < experts) {
        count = offsets[e + 1] - offsets[e];
        slot = slot_of ? slot_of[e] : e;
        if (pool_slots > 0 && slot >= pool_slots) {          // never an address: reported, treated as absent
            atomicCAS(error, kErrNone, kErrIdOutOfRange);
            slot = -1;
            count = 0;
        }
        if (slot < 0 && count > 0) {
            if (skip_absent) count = 0;
            else atomicCAS(error, kErrNone, kErrExpertAbsent);
        }
    }
    const int mine = (count + kMaxN - 1) / kMaxN;
    base[e] = mine;
    __syncthreads();
    if (e == 0) {
        int run = 0;
        for (int i = 0; i < experts; ++i) { const int c = base[i]; base[i] = run; run += c; }
        base[experts] = run;
        *n_tiles = run;
    }
    __syncthreads();
    if (e < experts) {
        for (int c = 0; c < mine; ++c) {
            PrefillTile t;
            t.slot = slot;
            t.pos0 = offsets[e] + c * kMaxN;
            t.ntok = min(kMaxN, count - c * kMaxN);
            t.pad = e;
            if (index_ok(base[e] + c, tiles_cap, error)) tiles[base[e] + c] = t;
        }
    }
}

__global__ void moe_accumulate_prefill_kernel(float* __restrict__ accum, int64_t accum_stride,
                                              const float* __restrict__ contrib,
                                              const int32_t* __restrict__ ids,
                                              const int32_t* __restrict__ slot_of, int skip_absent,
                                              int overwrite, int experts, int tokens, int top_k, int H, int pool_slots) {
    const int vec_per_row = H / 4;
    const int64_t total = static_cast<int64_t>(tokens) * vec_per_row;
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int token = static_cast<int>(i / vec_per_row);
        const int v = static_cast<int>(i - static_cast<int64_t>(token) * vec_per_row);
        float4* dst = reinterpret_cast<float4*>(accum + token * accum_stride) + v;
        float4 a = overwrite ? make_float4(0.f, 0.f, 0.f, 0.f) : *dst;
        for (int slot = 0; slot < top_k; ++slot) {
            const int draw = token * top_k + slot;
            const int id = ids[draw];
            // absent: no slot, or a slot beyond the declared pool (reported by the work-list kernel)
            if (id >= 0 && id < experts &&
                !(skip_absent && (slot_of[id] < 0 || (pool_slots > 0 && slot_of[id] >= pool_slots)))) {
                const float4 c = reinterpret_cast<const float4*>(contrib + static_cast<size_t>(draw) * H)[v];
                a.x += c.x; a.y += c.y; a.z += c.z; a.w += c.w;
            }
        }
        *dst = a;
    }
}

}  // namespace

struct PrefillScratch {
    int max_tokens{0};
    __half* xg{nullptr};
    __half* hidden{nullptr};
    float* contrib{nullptr};
    int32_t *offsets{nullptr}, *token_idx{nullptr}, *draw_idx{nullptr}, *counts{nullptr}, *n_tiles{nullptr};
    float* wpos{nullptr};
    PrefillTile* tiles{nullptr};
    WorkEntry* entries{nullptr};
    CUtensorMap x_map, h_map;
    uint64_t bytes{0};
};

void free_prefill_scratch(aeon_b200_ctx* ctx) {
    PrefillScratch* s = static_cast<PrefillScratch*>(ctx->prefill);
    if (!s) return;
    void* bufs[] = {s->xg, s->hidden, s->contrib, s->offsets, s->token_idx, s->draw_idx, s->counts,
                    s->n_tiles, s->wpos, s->tiles, s->entries};
    for (void* b : bufs) ctx_device_free(ctx, b);
    delete s;
    ctx->prefill = nullptr;
}

static PrefillScratch* ensure_scratch(aeon_b200_ctx* ctx, int tokens) {
    PrefillScratch* s = static_cast<PrefillScratch*>(ctx->prefill);
    if (s && s->max_tokens >= tokens) return s;
    free_prefill_scratch(ctx);
    s = new PrefillScratch();
    ctx->prefill = s;
    const aeon_b200_moe_config& cfg = ctx->cfg;
    const size_t draws = static_cast<size_t>(tokens) * cfg.top_k;
    auto alloc = [&](auto*& ptr, size_t count) {
        using Ptr = std::remove_reference_t<decltype(ptr)>;
        ptr = static_cast<Ptr>(ctx_device_alloc(ctx, count * sizeof(*ptr), "prefill scratch"));
        s->bytes += count * sizeof(*ptr);
    };
    // 64 spare rows so a TMA box that starts inside the last tile stays inside the allocation
    alloc(s->xg, (draws + 64) * cfg.hidden);
    alloc(s->hidden, (draws + 64) * cfg.intermediate);
    alloc(s->contrib, draws * cfg.hidden);
    alloc(s->offsets, cfg.experts + 1);
    alloc(s->token_idx, draws);
    alloc(s->draw_idx, draws);
    alloc(s->wpos, draws);
    alloc(s->counts, 4);
    alloc(s->n_tiles, 1);
    alloc(s->tiles, cfg.experts + draws / kMaxN + 1);
    alloc(s->entries, cfg.experts + draws / 8 + 1);
    AEON_CUDA_CHECK(cudaMemset(s->xg, 0, (draws + 64) * cfg.hidden * sizeof(__half)));
    AEON_CUDA_CHECK(cudaMemset(s->hidden, 0, (draws + 64) * cfg.intermediate * sizeof(__half)));
    s->x_map = make_rowmajor16_map(s->xg, draws + 64, cfg.hidden, cfg.hidden);
    s->h_map = make_rowmajor16_map(s->hidden, draws + 64, cfg.intermediate, cfg.intermediate);
    s->max_tokens = tokens;
    return s;
}

void launch_moe_prefill(aeon_b200_ctx* ctx, const void* pool_base, const int32_t* slot_of_expert,
                        const void* x, int64_t x_stride, const int32_t* topk_ids,
                        const float* topk_weights, int tokens, float* moe_accum, int64_t accum_stride,
                        uint32_t flags, cudaStream_t stream) {
    const aeon_b200_moe_config& cfg = ctx->cfg;
    require(pool_base && slot_of_expert && x && topk_ids && topk_weights && moe_accum,
            "aeon_b200_moe_prefill: null pointer argument");
    require(tokens > 0 && tokens <= 65536, "aeon_b200_moe_prefill: tokens must be in [1, 65536]");
    require(x_stride >= cfg.hidden && x_stride % 8 == 0 && accum_stride >= cfg.hidden && accum_stride % 4 == 0,
            "aeon_b200_moe_prefill: bad row stride");
    require(aligned16(x) && aligned16(moe_accum),
            "aeon_b200_moe_prefill: x and moe_accum must be 16-byte aligned (128-bit accesses)");
    require(cfg.hidden % (kTileK * kPrefetch) == 0 && cfg.intermediate % (kTileK * kPrefetch) == 0,
            "aeon_b200_moe_prefill: hidden and intermediate must be multiples of 256");
    PrefillScratch* s = ensure_scratch(ctx, tokens);
    const bool skip = (flags & AEON_B200_DECODE_SKIP_ABSENT) != 0;

    launch_permutation(ctx, topk_ids, tokens, cfg.top_k, cfg.experts, s->offsets, s->token_idx, s->draw_idx,
                       topk_weights, s->wpos, slot_of_expert, s->entries, s->counts, skip, stream);
    const int tiles_cap = cfg.experts + tokens * cfg.top_k / kMaxN + 1;
    build_tiles_kernel<<<1, 1024, 0, stream>>>(s->offsets, slot_of_expert, cfg.experts, skip ? 1 : 0, s->tiles,
                                               s->n_tiles, ctx->d_error, ctx->pool_slots, tiles_cap);
    AEON_CUDA_CHECK(cudaGetLastError());
    gather_activations_kernel<<<4 * ctx->sm_count, 256, 0, stream>>>(
        x, x_stride, cfg.act_dtype, s->token_idx, s->counts, cfg.hidden, s->xg, tokens, tokens * cfg.top_k, ctx->d_error);
    AEON_CUDA_CHECK(cudaGetLastError());

    PrefillParams p{};
    p.pool = static_cast<const uint8_t*>(pool_base);
    p.payload_bytes = ctx->geom.payload_bytes;
    p.w1 = ctx->geom.w1;
    p.w2 = ctx->geom.w2;
    p.w3 = ctx->geom.w3;
    p.group = cfg.group_size;
    p.H = cfg.hidden;
    p.I = cfg.intermediate;
    p.tiles = s->tiles;
    p.n_tiles = s->n_tiles;
    p.draw_idx = s->draw_idx;
    p.wpos = s->wpos;
    p.hidden = s->hidden;
    p.contrib = s->contrib;
    p.limit = cfg.swiglu_limit;
    p.error = ctx->d_error;
    p.draws_cap = tokens * cfg.top_k;
    p.tiles_cap = tiles_cap;


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
    auto launch = [&](auto kernel, const CUtensorMap& map) {
        AEON_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
        kernel<<<ctx->sm_count, kThreads, kSmemBytes, stream>>>(p, map);
        AEON_CUDA_CHECK(cudaGetLastError());
    };
    if (cfg.group_size == 128) launch(moe_grouped_gemm_kernel<true, 128>, s->x_map);
    else launch(moe_grouped_gemm_kernel<true, 32>, s->x_map);
    if (ev) AEON_CUDA_CHECK(cudaEventRecord(ev[1], stream));
    if (cfg.group_size == 128) launch(moe_grouped_gemm_kernel<false, 128>, s->h_map);
    else launch(moe_grouped_gemm_kernel<false, 32>, s->h_map);
    if (ev) AEON_CUDA_CHECK(cudaEventRecord(ev[2], stream));

    const int64_t vecs = static_cast<int64_t>(tokens) * cfg.hidden / 4;
    const int blocks = static_cast<int>(std::min<int64_t>((vecs + 255) / 256, 8 * ctx->sm_count));
    moe_accumulate_prefill_kernel<<<blocks, 256, 0, stream>>>(moe_accum, accum_stride, s->contrib, topk_ids,
                                                              slot_of_expert, skip ? 1 : 0,
                                                              (flags & AEON_B200_DECODE_OVERWRITE) ? 1 : 0,
                                                              cfg.experts, tokens, cfg.top_k, cfg.hidden,
                                                              ctx->pool_slots);
    AEON_CUDA_CHECK(cudaGetLastError());
    ctx->launches += 6;
}

}  // namespace aeon_b200
