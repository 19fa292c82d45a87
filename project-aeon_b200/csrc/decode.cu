// Decode path of the routed-expert MoE FFN for sm_100a.
//
//   kernel A  (moe_w13_swiglu_kernel): per (expert, 16-row tile) streams the int4 W1 and W3
//             rows with 128-bit coalesced loads straight into MMA operand registers, unpacks
//             the nibbles there, multiplies them with the expert's tokens on the warp MMA,
//             applies the fp16 group scales in fp32, and writes the clamped SwiGLU as an fp16
//             (hi, lo) pair.
//   kernel B  (moe_w2_contrib_kernel): the same streaming for W2 over the (hi, lo) hidden;
//             writes weight * (W2 h) per draw, one writer per element.
//   kernel C  (moe_accumulate_kernel): adds the per-draw slices of every token to the fp32
//             accumulator in slot order.
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
// entry is up to 8 consecutive positions of one expert; an item is (entry, row tile). Each
// CTA owns a contiguous range of items, so consecutive items mostly share their entry: the
// entry's activation rows (fp16, up to 8 tokens x K) are brought into shared memory once by
// bulk copies (TMA engine) and reused by every row tile, and the item's group scales are
// bulk-copied one item ahead. The weights themselves never touch shared memory: the warps of
// a CTA split K in 128-column chunks, each lane loads its 16-byte atoms with streaming
// 128-bit loads and keeps the next item's atoms in flight in registers while it computes
// (measured on B200: this form sustains 6.5-6.8 TB/s, where 2 KB bulk copies through a
// 64 KB shared-memory ring stop near 4.1 TB/s).
//
// MMA mapping. The weight rows are the M operand (16 per MMA tile), the tokens the N
// operand (8), so lane (g = lane/4, t = lane%4) holds weight rows g and g+8 and token g.
// A lane reads one 16-byte atom (32 consecutive columns of one row) per row; the four
// lanes of a row cover the 128 columns of one scale group, and eight MMAs consume them.
// Which column lands in which MMA k-slot is irrelevant as long as the activation operand
// uses the same assignment, which is why the activations (and the hidden vector) are
// stored in a permuted column order: within each 128, column 32t + 8i + r sits at
// 32i + 8t + r, making the four lanes' 16-byte shared-memory reads contiguous.
#include "common.cuh"
#include "ptx.cuh"

#include <algorithm>

namespace aeon_b200 {

namespace {

constexpr int kTokTile = 8;         // tokens per work entry (one MMA N tile)
constexpr int kPad = 64;            // bytes; shifts alternate activation rows by half the banks
constexpr int kSmemEntries = 384;   // work entries cached in shared memory
constexpr int kSmemDraws = 1024;    // draw-indexed values cached in shared memory

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
    int overwrite;
    int experts;
    __half* hid_hi;
    __half* hid_lo;
    float* contrib;
    float* accum;
    int64_t accum_stride;
    float limit;
    int32_t* error;
    // extents of the buffers above, for the bounds-checked build
    long long hidden_elems;    // hid_hi / hid_lo
    long long contrib_elems;   // contrib
    int draws_cap;             // rows of hid_* / contrib, entries of token_idx / draw_idx / wpos
    int entries_cap;           // entries
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

__device__ __forceinline__ void flag_error(int32_t* error, int code) {
    atomicCAS(error, kErrNone, code);
}

// Streaming loads: read-only path, no L1 allocation (every weight byte is used once).
__device__ __forceinline__ uint4 ldg_stream128(const uint8_t* p) {
    uint4 v;
    asm("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
        : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
        : "l"(p));
    return v;
}

__device__ __forceinline__ uint32_t ldg_stream32(const uint8_t* p) {
    uint32_t v;
    asm("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}

// Registers holding one 128-column chunk of a lane's two rows (rows g and g+8) for kMats
// matrices: one 16-byte atom per (matrix, row) at group 128; at group 32 the four lanes of
// a row share each atom and a lane keeps only its own 32-bit word of the four atoms.
template <int G, int kMats>
struct ChunkRegs {
    static constexpr int kWords = (G == 128) ? 4 : 4;
    uint32_t w[kMats][2][kWords];   // [matrix][row half][word or atom]
};

template <int G, int kMats>
__device__ __forceinline__ void load_chunk(ChunkRegs<G, kMats>& r, const uint8_t* const (&base)[kMats][2],
                                           uint32_t chunk_off) {
#pragma unroll
    for (int m = 0; m < kMats; ++m)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            if constexpr (G == 128) {
                const uint4 v = ldg_stream128(base[m][h] + chunk_off);
                r.w[m][h][0] = v.x; r.w[m][h][1] = v.y; r.w[m][h][2] = v.z; r.w[m][h][3] = v.w;
            } else {
#pragma unroll
                for (int a = 0; a < 4; ++a) r.w[m][h][a] = ldg_stream32(base[m][h] + chunk_off + a * 16);
            }
        }
}

// Per-(token, scale group) sums of the activation tile, the zero-point term of
// ptx::fold_group. `rows` activation rows of `groups` scale groups of G fp16 values each sit
// in shared memory `row_stride` bytes apart (a second plane, the lo part of the hidden vector,
// `plane_stride` bytes after the first when planes == 2). Output xs[(grp * planes + plane) * 8
// + row] as fp32; rows >= valid_rows get 0. Warps take (plane, row, group) triples round
// robin; every sum is a fixed lane pattern plus a butterfly, so it is reproducible. kHiScaled:
// the columns that meet the high-nibble plane (bit 1 of the column index) are stored divided by
// 16 (row-streaming kernels) and enter the sum multiplied back.
template <int G, bool kHiScaled = false>
__device__ __forceinline__ void group_sums(uint32_t act_smem, int row_stride, int plane_stride,
                                           int planes, int valid_rows, int groups, float* xs,
                                           int warp, int warps, int lane) {
    const int total = planes * kTokTile * groups;
    for (int idx = warp; idx < total; idx += warps) {
        const int grp = idx % groups;
        const int row = (idx / groups) % kTokTile;
        const int plane = idx / (groups * kTokTile);
        float v = 0.f;
        if (row < valid_rows) {
            const uint32_t at = act_smem + row * row_stride + plane * plane_stride + grp * (G * 2);
            if constexpr (G == 128) {
                const uint2 q = ptx::lds64(at + lane * 8);
                const __half2 a = *reinterpret_cast<const __half2*>(&q.x);
                const __half2 b = *reinterpret_cast<const __half2*>(&q.y);
                // a lane's four positions are columns 0,1,2,3 or 4,5,6,7 modulo 8: the second pair is
                // the scaled one either way
                v = (__low2float(a) + __high2float(a)) +
                    (kHiScaled ? 16.0f : 1.0f) * (__low2float(b) + __high2float(b));
            } else {
                v = __half2float(__ushort_as_half(static_cast<unsigned short>(ptx::lds16(at + lane * 2))));
            }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, off);
        }
        if (lane == 0) xs[(grp * planes + plane) * kTokTile + row] = v;
    }
}

// ----- kernel A: W1/W3 dual product + clamped SwiGLU -----------------------------------
// One 16-row tile per item; the CTA's KW warps split K, NCH chunks of 128 columns each
// (KW * NCH * 128 == hidden), chunk j of warp w being chunk j * KW + w so that the warps
// of a CTA read neighbouring 64-byte runs at the same time.
template <int G, int KW, int NCH>
struct GeomA {
    static constexpr int kThreads = KW * 32;
    static constexpr int kHidden = KW * NCH * 128;
    static constexpr int kActRow = kHidden * 2 + kPad;
    static constexpr int kActBytes = kTokTile * kActRow;
    static constexpr int kBlockScaleBytes = (kHidden / 256) * ((G == 128) ? 16 : 64);
    static constexpr int kScaleBuf = 2 * 4 * kBlockScaleBytes;       // 2 matrices x 4 row-blocks
    static constexpr int kRedBuf = KW * 2 * 128 * 4;
    static constexpr int kGroups = kHidden / G;
    static constexpr int kXsBytes = kGroups * kTokTile * 4;
    static constexpr int kBarBytes = 64;
    static constexpr int kSmem = kBarBytes + kActBytes + 2 * kScaleBuf + 2 * kRedBuf + kXsBytes;
};

template <int G, int KW, int NCH>
__global__ void __launch_bounds__(KW * 32, 1)
moe_w13_swiglu_kernel(const DecodeParams p) {
    using S = GeomA<G, KW, NCH>;
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t smem_base = ptx::smem_u32(smem);
    const uint32_t act_bar = smem_base;                  // 8 B
    const uint32_t scale_bar = smem_base + 16;           // 2 x 8 B
    const uint32_t act_smem = smem_base + S::kBarBytes;
    const uint32_t scale_smem = act_smem + S::kActBytes;
    float* red = reinterpret_cast<float*>(smem + S::kBarBytes + S::kActBytes + 2 * S::kScaleBuf);
    float* xs = red + 2 * (S::kRedBuf / 4);
    const uint32_t xs_smem = scale_smem + 2 * S::kScaleBuf + 2 * S::kRedBuf;
    __shared__ WorkEntry s_entries[kSmemEntries];
    __shared__ int32_t s_token_idx[kSmemDraws];

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const int g = lane >> 2;
    const int t = lane & 3;

    const int entries = index_ok(p.counts[0], p.entries_cap + 1, p.error) ? p.counts[0] : 0;
    const int placed = p.counts[2];
    const int tiles = p.I / 16;
    const int total_items = entries * tiles;
    // contiguous, balanced item range of this CTA
    const int lo = static_cast<int>(static_cast<int64_t>(total_items) * blockIdx.x / gridDim.x);
    const int hi = static_cast<int>(static_cast<int64_t>(total_items) * (blockIdx.x + 1) / gridDim.x);
    if (lo >= hi) return;

    if (tid == 0) {
        ptx::mbar_init(act_bar, 1);
        ptx::mbar_init(scale_bar, 1);
        ptx::mbar_init(scale_bar + 8, 1);
        ptx::fence_barrier_init();
    }
    const bool cached_entries = entries <= kSmemEntries;
    const bool cached_draws = placed <= kSmemDraws;
    if (cached_entries) {
        const int m_lo = lo / tiles, m_hi = (hi - 1) / tiles;
        for (int i = m_lo + tid; i <= m_hi; i += S::kThreads) s_entries[i] = p.entries[i];
    }
    if (cached_draws)
        for (int i = tid; i < placed; i += S::kThreads) s_token_idx[i] = p.token_idx[i];
    __syncthreads();
    const WorkEntry* ent = cached_entries ? s_entries : p.entries;
    const int32_t* token_idx = cached_draws ? s_token_idx : p.token_idx;

    // Lane-constant byte offsets of its two rows inside a 16-row tile (4 row-blocks of 4).
    uint32_t lane_off[2], lane_sc[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int r = g + 8 * h;
        const int blk = r >> 2, rib = r & 3;
        if constexpr (G == 128) {
            lane_off[h] = blk * p.w1.block_bytes + (rib * 8 + t) * 16;
            lane_sc[h] = blk * S::kBlockScaleBytes + rib * 4;
        } else {
            lane_off[h] = blk * p.w1.block_bytes + rib * 128 + t * 4;
            lane_sc[h] = blk * S::kBlockScaleBytes + rib * 16;
        }
    }
    // chunk c -> byte offset inside a row-block: iteration (256 columns) c/2, half c%2
    auto chunk_off = [](int c) -> uint32_t { return (c >> 1) * 512 + (c & 1) * 64; };

    const uint64_t stream_policy = ptx::policy_evict_first();
    const uint64_t keep_policy = ptx::policy_evict_last();

    auto item_bases = [&](int it, const uint8_t* (&base)[2][2], const uint8_t*& scales1,
                          const uint8_t*& scales3, WorkEntry& e, int& m, int& rt) {
        m = it / tiles;
        rt = it - m * tiles;
        e = ent[m];
        const uint8_t* payload = p.pool + static_cast<uint64_t>(e.slot < 0 ? 0 : e.slot) * p.payload_bytes;
        const uint8_t* w1 = payload + p.w1.packed_offset + static_cast<size_t>(rt) * 4 * p.w1.block_bytes;
        const uint8_t* w3 = payload + p.w3.packed_offset + static_cast<size_t>(rt) * 4 * p.w3.block_bytes;
        base[0][0] = w1 + lane_off[0]; base[0][1] = w1 + lane_off[1];
        base[1][0] = w3 + lane_off[0]; base[1][1] = w3 + lane_off[1];
        scales1 = payload + p.w1.scale_offset + static_cast<size_t>(rt) * 4 * S::kBlockScaleBytes;
        scales3 = payload + p.w3.scale_offset + static_cast<size_t>(rt) * 4 * S::kBlockScaleBytes;
    };
    auto issue_scales = [&](const uint8_t* s1, const uint8_t* s3, int buf) {
        // one thread: the item's scales are two contiguous runs (4 row-blocks per matrix)
        const uint32_t bar = scale_bar + 8 * buf;
        ptx::mbar_arrive_expect_tx(bar, S::kScaleBuf);
        const uint32_t dst = scale_smem + buf * S::kScaleBuf;
        ptx::bulk_g2s(dst, s1, 4 * S::kBlockScaleBytes, bar, stream_policy);
        ptx::bulk_g2s(dst + 4 * S::kBlockScaleBytes, s3, 4 * S::kBlockScaleBytes, bar, stream_policy);
    };

    // ---- prologue: first item's scales and weights in flight ----
    ChunkRegs<G, 2> wbuf[NCH];
    const uint8_t* base[2][2];
    const uint8_t *sc1, *sc3;
    WorkEntry e;
    int m, rt;
    item_bases(lo, base, sc1, sc3, e, m, rt);
    if (e.slot < 0 && tid == 0) flag_error(p.error, kErrExpertAbsent);
    if (tid == 0) issue_scales(sc1, sc3, 0);
#pragma unroll
    for (int j = 0; j < NCH; ++j) load_chunk<G, 2>(wbuf[j], base, chunk_off(j * KW + warp));

    int cur_entry = -1;
    uint32_t act_phase = 0;
    for (int it = lo, idx = 0; it < hi; ++it, ++idx) {
        // ---- the entry's activation rows, when the entry changes ----
        if (m != cur_entry) {
            if (warp == 0) {
                if (lane == 0) ptx::mbar_arrive_expect_tx(act_bar, e.ntok * S::kHidden * 2);
                __syncwarp();
                if (lane < e.ntok) {
                    // a token index outside the batch is reported and row 0 copied in its place
                    const int raw = index_ok(e.pos0 + lane, p.draws_cap, p.error) ? token_idx[e.pos0 + lane] : 0;
                    const int token = index_ok(raw, p.tokens, p.error) ? raw : 0;
                    ptx::bulk_g2s(act_smem + lane * S::kActRow,
                                  p.xperm + static_cast<size_t>(token) * S::kHidden, S::kHidden * 2,
                                  act_bar, keep_policy);
                }
            }
            if (!ptx::mbar_wait(act_bar, act_phase & 1, p.error)) flag_error(p.error, kErrWaitTimeout);
            ++act_phase;
            cur_entry = m;
            __syncwarp();
            group_sums<G>(act_smem, S::kActRow, 0, 1, e.ntok, S::kGroups, xs, warp, KW, lane);
            __syncthreads();
        }
        const WorkEntry cur = e;
        const int cur_rt = rt;

        // ---- next item: scales by bulk copy, weight addresses for the register refill ----
        const bool has_next = it + 1 < hi;
        const uint8_t* nbase[2][2] = {{base[0][0], base[0][1]}, {base[1][0], base[1][1]}};
        if (has_next) {
            item_bases(it + 1, nbase, sc1, sc3, e, m, rt);
            if (tid == 0) {
                if (e.slot < 0) flag_error(p.error, kErrExpertAbsent);
                issue_scales(sc1, sc3, (idx + 1) & 1);
            }
        }
        if (!ptx::mbar_wait(scale_bar + 8 * (idx & 1), (idx >> 1) & 1, p.error))
            flag_error(p.error, kErrWaitTimeout);
        __syncwarp();
        const uint32_t sc_smem = scale_smem + (idx & 1) * S::kScaleBuf;
        const uint32_t a_row = act_smem + g * S::kActRow;

        float acc[2][4];
#pragma unroll
        for (int a = 0; a < 2; ++a)
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[a][c] = 0.f;

#pragma unroll
        for (int j = 0; j < NCH; ++j) {
            const int c = j * KW + warp;
            if constexpr (G == 128) {
                uint4 bfrag[4];
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    bfrag[i] = (g < cur.ntok) ? ptx::lds128(a_row + (c * 128 + i * 32 + t * 8) * 2)
                                              : make_uint4(0, 0, 0, 0);
                const float2 xsum = ptx::lds_f2(xs_smem + (c * kTokTile + 2 * t) * 4);
#pragma unroll
                for (int mat = 0; mat < 2; ++mat) {
                    const uint32_t sc_at = sc_smem + mat * 4 * S::kBlockScaleBytes + (c >> 1) * 16 + (c & 1) * 2;
                    const float sca = ptx::lds_half_as_float(sc_at + lane_sc[0]);
                    const float scb = ptx::lds_half_as_float(sc_at + lane_sc[1]);
                    float tlo[4] = {0.f, 0.f, 0.f, 0.f};
                    float thi[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        ptx::mma_word(tlo, thi, wbuf[j].w[mat][0][i], wbuf[j].w[mat][1][i], bfrag[i]);
                    ptx::fold_group(acc[mat], tlo, thi, sca, scb, xsum);
                }
            } else {
                // group 32: atom a of the chunk is one scale group; the lane holds word t of it
#pragma unroll
                for (int a = 0; a < 4; ++a) {
                    const uint4 bf = (g < cur.ntok) ? ptx::lds128(a_row + (c * 128 + a * 32 + t * 8) * 2)
                                                    : make_uint4(0, 0, 0, 0);
                    const float2 xsum = ptx::lds_f2(xs_smem + ((c * 4 + a) * kTokTile + 2 * t) * 4);
#pragma unroll
                    for (int mat = 0; mat < 2; ++mat) {
                        const uint32_t sc_at = sc_smem + mat * 4 * S::kBlockScaleBytes + (c >> 1) * 64 +
                                               ((c & 1) * 4 + a) * 2;
                        const float sca = ptx::lds_half_as_float(sc_at + lane_sc[0]);
                        const float scb = ptx::lds_half_as_float(sc_at + lane_sc[1]);
                        float tlo[4] = {0.f, 0.f, 0.f, 0.f};
                        float thi[4] = {0.f, 0.f, 0.f, 0.f};
                        ptx::mma_word(tlo, thi, wbuf[j].w[mat][0][a], wbuf[j].w[mat][1][a], bf);
                        ptx::fold_group(acc[mat], tlo, thi, sca, scb, xsum);
                    }
                }
            }
            // this chunk's registers are free: put the next item's chunk in flight
            if (has_next) load_chunk<G, 2>(wbuf[j], nbase, chunk_off(c));
        }
        if (has_next) {
#pragma unroll
            for (int a = 0; a < 2; ++a)
#pragma unroll
                for (int h = 0; h < 2; ++h) base[a][h] = nbase[a][h];
        }

        // K-split partials -> shared (double-buffered: one barrier per item), fixed-order
        // sum, SwiGLU, hi/lo store.
        float* rbuf = red + (idx & 1) * (S::kRedBuf / 4);
#pragma unroll
        for (int mat = 0; mat < 2; ++mat)
            *reinterpret_cast<float4*>(&rbuf[(warp * 2 + mat) * 128 + lane * 4]) =
                make_float4(acc[mat][0], acc[mat][1], acc[mat][2], acc[mat][3]);
        __syncthreads();
        if (tid < 128) {
            float gate = 0.f, up = 0.f;
#pragma unroll
            for (int w = 0; w < KW; ++w) {
                gate += rbuf[(w * 2 + 0) * 128 + tid];
                up += rbuf[(w * 2 + 1) * 128 + tid];
            }
            const int lo4 = tid >> 2, c = tid & 3;
            const int go = lo4 >> 2, to = lo4 & 3;
            const int token = 2 * to + (c & 1);
            const int row = go + 8 * (c >> 1);
            if (token < cur.ntok) {
                gate = fminf(gate, p.limit);
                up = fminf(fmaxf(up, -p.limit), p.limit);
                const float hval = (gate / (1.0f + expf(-gate))) * up;
                const __half hi16 = __float2half_rn(hval);
                const __half lo16 = __float2half_rn(hval - __half2float(hi16));
                const size_t at = static_cast<size_t>(cur.pos0 + token) * p.I + perm_col<G>(cur_rt * 16 + row);
                if (index_ok(static_cast<long long>(at), p.hidden_elems, p.error)) {
                    p.hid_hi[at] = hi16;
                    p.hid_lo[at] = lo16;
                }
            }
        }
    }
}

// ----- kernel B: W2 product, per-draw weighted slices -------------------------------------
// MW workers of KW warps per CTA; a worker owns MT 16-row tiles of the CTA's MW*MT*16-row
// item and splits K = intermediate over its warps (KW * NCH * 128 == intermediate). The MT
// tiles of a worker share every activation fragment read from shared memory. Workers share
// the entry's hidden rows and nothing else (own scale buffers, own named barrier), so they
// only meet when the entry changes. P items of weights are kept in flight per lane.
template <int G, int MW, int MT, int KW, int NCH, int P>
struct GeomB {
    static constexpr int kThreads = MW * KW * 32;
    static constexpr int kInter = KW * NCH * 128;
    static constexpr int kItemRows = MW * MT * 16;
    static constexpr int kActRow = 2 * kInter * 2 + kPad;            // hi then lo
    static constexpr int kActBytes = kTokTile * kActRow;
    static constexpr int kBlockScaleBytes = (kInter / 128) * ((G == 128) ? 16 : 64);
    static constexpr int kScaleBuf = 2 * MT * kBlockScaleBytes;       // a worker's row-blocks
    static constexpr int kRedBuf = KW * MT * 128 * 4;
    static constexpr int kGroups = kInter / G;
    static constexpr int kXsBytes = kGroups * 2 * kTokTile * 4;       // [group][hi|lo][token]
    static constexpr int kBarBytes = 128;
    static constexpr int kSmem = kBarBytes + kActBytes + MW * 2 * kScaleBuf + MW * 2 * kRedBuf + kXsBytes;
};

template <int G, int MW, int MT, int KW, int NCH, int P>
__global__ void __launch_bounds__(MW * KW * 32, 1)
moe_w2_contrib_kernel(const DecodeParams p) {
    using S = GeomB<G, MW, MT, KW, NCH, P>;
    static_assert(MW <= 4, "barrier slots");
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t smem_base = ptx::smem_u32(smem);
    const uint32_t act_bar = smem_base;                  // 8 B
    const uint32_t scale_bar0 = smem_base + 16;          // MW x 2 x 8 B
    const uint32_t act_smem = smem_base + S::kBarBytes;
    const uint32_t scale_smem0 = act_smem + S::kActBytes;
    float* red0 = reinterpret_cast<float*>(smem + S::kBarBytes + S::kActBytes + MW * 2 * S::kScaleBuf);
    float* xs = red0 + MW * 2 * (S::kRedBuf / 4);
    const uint32_t xs_smem = scale_smem0 + MW * 2 * S::kScaleBuf + MW * 2 * S::kRedBuf;
    __shared__ WorkEntry s_entries[kSmemEntries];
    __shared__ int32_t s_draw_idx[kSmemDraws];
    __shared__ float s_wpos[kSmemDraws];

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const int wk = warp / KW;          // worker
    const int kw = warp % KW;          // K-split index inside the worker
    const int wtid = tid - wk * KW * 32;
    const int g = lane >> 2;
    const int t = lane & 3;

    const int entries = index_ok(p.counts[0], p.entries_cap + 1, p.error) ? p.counts[0] : 0;
    const int placed = p.counts[2];
    const int tiles = p.H / S::kItemRows;
    const int total_items = entries * tiles;
    const int lo = static_cast<int>(static_cast<int64_t>(total_items) * blockIdx.x / gridDim.x);
    const int hi = static_cast<int>(static_cast<int64_t>(total_items) * (blockIdx.x + 1) / gridDim.x);
    if (lo >= hi) return;

    if (tid == 0) {
        ptx::mbar_init(act_bar, 1);
        for (int i = 0; i < MW * 2; ++i) ptx::mbar_init(scale_bar0 + 8 * i, 1);
        ptx::fence_barrier_init();
    }
    const bool cached_entries = entries <= kSmemEntries;
    const bool cached_draws = placed <= kSmemDraws;
    if (cached_entries) {
        const int m_lo = lo / tiles, m_hi = (hi - 1) / tiles;
        for (int i = m_lo + tid; i <= m_hi; i += S::kThreads) s_entries[i] = p.entries[i];
    }
    if (cached_draws)
        for (int i = tid; i < placed; i += S::kThreads) {
            s_draw_idx[i] = p.draw_idx[i];
            s_wpos[i] = p.wpos[i];
        }
    __syncthreads();
    const WorkEntry* ent = cached_entries ? s_entries : p.entries;
    const int32_t* draw_idx = cached_draws ? s_draw_idx : p.draw_idx;
    const float* wpos = cached_draws ? s_wpos : p.wpos;

    const uint32_t scale_bar = scale_bar0 + wk * 16;
    const uint32_t scale_smem = scale_smem0 + wk * 2 * S::kScaleBuf;
    float* red = red0 + wk * 2 * (S::kRedBuf / 4);

    // W2 row-blocks hold 8 rows: rows g of a tile are its first block, rows g+8 the second,
    // and a warp's 32 lanes read one contiguous 512-byte line per block.
    uint32_t lane_off[MT][2], lane_sc[MT][2];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int blk = mt * 2 + h;
            if constexpr (G == 128) {
                lane_off[mt][h] = blk * p.w2.block_bytes + (g * 4 + t) * 16;
                lane_sc[mt][h] = blk * S::kBlockScaleBytes + g * 2;
            } else {
                lane_off[mt][h] = blk * p.w2.block_bytes + g * 64 + t * 4;
                lane_sc[mt][h] = blk * S::kBlockScaleBytes + g * 8;
            }
        }
    const uint64_t stream_policy = ptx::policy_evict_first();
    const uint64_t keep_policy = ptx::policy_evict_last();

    // (entry index, row tile) of an item; items advance one row tile at a time
    auto locate = [&](int it, int& m, int& rt) { m = it / tiles; rt = it - m * tiles; };
    auto weights_of = [&](int m, int rt) -> const uint8_t* {
        const WorkEntry e = ent[m];
        return p.pool + static_cast<uint64_t>(e.slot < 0 ? 0 : e.slot) * p.payload_bytes;
    };
    auto set_bases = [&](const uint8_t* payload, int rt, const uint8_t* (&base)[MT][2]) {
        const size_t block0 = static_cast<size_t>(rt * MW + wk) * 2 * MT;
        const uint8_t* w = payload + p.w2.packed_offset + block0 * p.w2.block_bytes;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            base[mt][0] = w + lane_off[mt][0];
            base[mt][1] = w + lane_off[mt][1];
        }
    };
    auto issue_scales = [&](const uint8_t* payload, int rt, int buf) {
        const size_t block0 = static_cast<size_t>(rt * MW + wk) * 2 * MT;
        const uint32_t bar = scale_bar + 8 * buf;
        ptx::mbar_arrive_expect_tx(bar, S::kScaleBuf);
        ptx::bulk_g2s(scale_smem + buf * S::kScaleBuf,
                      payload + p.w2.scale_offset + block0 * S::kBlockScaleBytes, S::kScaleBuf, bar,
                      stream_policy);
    };

    // ---- prologue: P items of weights in flight, first item's scales ----
    ChunkRegs<G, MT> wbuf[P][NCH];
#pragma unroll
    for (int q = 0; q < P; ++q) {
        if (lo + q < hi) {
            int m, rt;
            locate(lo + q, m, rt);
            const uint8_t* payload = weights_of(m, rt);
            const uint8_t* b[MT][2];
            set_bases(payload, rt, b);
            if (q == 0 && wtid == 0) issue_scales(payload, rt, 0);
#pragma unroll
            for (int j = 0; j < NCH; ++j) load_chunk<G, MT>(wbuf[q][j], b, (j * KW + kw) * 512);
        }
    }

    int cur_entry = -1;
    uint32_t act_phase = 0;
    for (int base_it = lo; base_it < hi; base_it += P) {
#pragma unroll
        for (int q = 0; q < P; ++q) {
            const int it = base_it + q;
            if (it >= hi) break;
            const int idx = it - lo;
            int m, rt;
            locate(it, m, rt);
            const WorkEntry e = ent[m];

            if (m != cur_entry) {
                // every worker must be done with the previous entry's rows
                __syncthreads();
                if (warp == 0) {
                    if (lane == 0) ptx::mbar_arrive_expect_tx(act_bar, e.ntok * S::kInter * 4);
                    __syncwarp();
                    if (lane < 2 * e.ntok) {
                        const int tok = lane >> 1, part = lane & 1;
                        const int pos = index_ok(e.pos0 + tok, p.draws_cap, p.error) ? e.pos0 + tok : 0;
                        const __half* src = (part == 0 ? p.hid_hi : p.hid_lo) + static_cast<size_t>(pos) * S::kInter;
                        ptx::bulk_g2s(act_smem + tok * S::kActRow + part * S::kInter * 2, src,
                                      S::kInter * 2, act_bar, keep_policy);
                    }
                }
                if (!ptx::mbar_wait(act_bar, act_phase & 1, p.error)) flag_error(p.error, kErrWaitTimeout);
                ++act_phase;
                cur_entry = m;
                __syncwarp();
                group_sums<G>(act_smem, S::kActRow, S::kInter * 2, 2, e.ntok, S::kGroups, xs, warp,
                              MW * KW, lane);
                __syncthreads();
            }

            // next item's scales (one thread of this worker); addresses of the item P ahead
            if (it + 1 < hi && wtid == 0) {
                int nm, nrt;
                locate(it + 1, nm, nrt);
                issue_scales(weights_of(nm, nrt), nrt, (idx + 1) & 1);
            }
            const bool refill = it + P < hi;
            const uint8_t* nbase[MT][2];
            {
                int nm = m, nrt = rt;
                if (refill) locate(it + P, nm, nrt);
                set_bases(weights_of(nm, nrt), nrt, nbase);
            }
            if (!ptx::mbar_wait(scale_bar + 8 * (idx & 1), (idx >> 1) & 1, p.error))
                flag_error(p.error, kErrWaitTimeout);
            __syncwarp();
            const uint32_t sc_smem = scale_smem + (idx & 1) * S::kScaleBuf;

            // Up to four tokens: the hi and lo parts ride in one MMA as eight token columns
            // (columns 0-3 hi of tokens 0-3, columns 4-7 lo), halving the MMA count; the two
            // column halves are added after the K-split sum. More tokens: one pass per part.
            const bool packed = e.ntok <= 4;
            float acc[MT][4];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int c = 0; c < 4; ++c) acc[mt][c] = 0.f;
#pragma unroll
            for (int j = 0; j < NCH; ++j) {
                const int c = j * KW + kw;
                const int passes = packed ? 1 : 2;
                for (int part = 0; part < passes; ++part) {
                    const int tok = packed ? (g & 3) : g;
                    const int my_part = packed ? (g >> 2) : part;
                    const bool live = tok < e.ntok;
                    const uint32_t b_row = act_smem + tok * S::kActRow + my_part * (S::kInter * 2);
                    // xs columns of this lane's accumulators: tokens 2t, 2t+1 of the pass
                    const uint32_t xs_col = packed ? ((t >> 1) * kTokTile + 2 * (t & 1))
                                                   : (part * kTokTile + 2 * t);
                    if constexpr (G == 128) {
                        uint4 bf[4];
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            bf[i] = live ? ptx::lds128(b_row + (c * 128 + i * 32 + t * 8) * 2)
                                         : make_uint4(0, 0, 0, 0);
                        const float2 xsum = ptx::lds_f2(xs_smem + (c * 2 * kTokTile + xs_col) * 4);
#pragma unroll
                        for (int mt = 0; mt < MT; ++mt) {
                            const float sca = ptx::lds_half_as_float(sc_smem + c * 16 + lane_sc[mt][0]);
                            const float scb = ptx::lds_half_as_float(sc_smem + c * 16 + lane_sc[mt][1]);
                            float tlo[4] = {0.f, 0.f, 0.f, 0.f};
                            float thi[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                            for (int i = 0; i < 4; ++i)
                                ptx::mma_word(tlo, thi, wbuf[q][j].w[mt][0][i], wbuf[q][j].w[mt][1][i], bf[i]);
                            ptx::fold_group(acc[mt], tlo, thi, sca, scb, xsum);
                        }
                    } else {
#pragma unroll
                        for (int a = 0; a < 4; ++a) {
                            const uint4 bf = live ? ptx::lds128(b_row + (c * 128 + a * 32 + t * 8) * 2)
                                                  : make_uint4(0, 0, 0, 0);
                            const float2 xsum =
                                ptx::lds_f2(xs_smem + ((c * 4 + a) * 2 * kTokTile + xs_col) * 4);
#pragma unroll
                            for (int mt = 0; mt < MT; ++mt) {
                                const float sca =
                                    ptx::lds_half_as_float(sc_smem + c * 64 + a * 2 + lane_sc[mt][0]);
                                const float scb =
                                    ptx::lds_half_as_float(sc_smem + c * 64 + a * 2 + lane_sc[mt][1]);
                                float tlo[4] = {0.f, 0.f, 0.f, 0.f};
                                float thi[4] = {0.f, 0.f, 0.f, 0.f};
                                ptx::mma_word(tlo, thi, wbuf[q][j].w[mt][0][a], wbuf[q][j].w[mt][1][a], bf);
                                ptx::fold_group(acc[mt], tlo, thi, sca, scb, xsum);
                            }
                        }
                    }
                }
                if (refill) load_chunk<G, MT>(wbuf[q][j], nbase, c * 512);
            }

            float* rbuf = red + (idx & 1) * (S::kRedBuf / 4);
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
                *reinterpret_cast<float4*>(&rbuf[(kw * MT + mt) * 128 + lane * 4]) =
                    make_float4(acc[mt][0], acc[mt][1], acc[mt][2], acc[mt][3]);
            ptx::named_bar_sync(1 + wk, KW * 32);
            for (int o = wtid; o < MT * 128; o += KW * 32) {
                const int mt = o >> 7, idx128 = o & 127;
                const int lo4 = idx128 >> 2, c = idx128 & 3;
                const int go = lo4 >> 2, to = lo4 & 3;
                float sum = 0.f;
#pragma unroll
                for (int w = 0; w < KW; ++w) sum += rbuf[(w * MT + mt) * 128 + idx128];
                if (packed) {
                    // columns 2to+(c&1) (hi) and the same + 4 (lo) are two lanes apart: +8 floats
                    float lo_part = 0.f;
                    if (to < 2) {
#pragma unroll
                        for (int w = 0; w < KW; ++w) lo_part += rbuf[(w * MT + mt) * 128 + idx128 + 8];
                    }
                    sum += lo_part;
                }
                const int token = (packed && to >= 2) ? kTokTile : 2 * to + (c & 1);
                const int row = ((rt * MW + wk) * MT + mt) * 16 + go + 8 * (c >> 1);
                if (token < e.ntok) {
                    const int pos = e.pos0 + token;
                    if (index_ok(pos, p.draws_cap, p.error)) {
                        const int draw = draw_idx[pos];
                        if (index_ok(draw, p.draws_cap, p.error))
                            p.contrib[static_cast<size_t>(draw) * p.H + row] = wpos[pos] * sum;
                    }
                }
            }
        }
    }
}

// =========================================================================================
// Row-streaming forms of kernels A and B (group 128).
//
// Each warp owns whole weight rows: one 16-row tile of W1 and W3 (kernel A) or MT 16-row tiles
// of W2 (kernel B) over the full K, with the accumulators in its registers from the first
// column to the last. No K-split, so no cross-warp reduction, no per-tile barrier and no
// scale staging: the warps of a CTA run independently and only meet when the CTA moves to
// another work entry, whose activation rows they share in shared memory. A warp keeps D
// "steps" of its rows' packed words and scales in flight in a register ring (a step is the
// 512-byte line of each of its row-blocks: 256 columns for W1/W3, 128 for W2) and refills a
// ring slot as soon as it has consumed it, across tile boundaries, so the loads never drain.
//
// Scheduling unit: W consecutive tiles of one entry, one per warp. A CTA owns a contiguous,
// balanced range of units; all its warps walk the same units, so an entry change is uniform
// across the CTA and is the only place with a CTA-wide barrier.
// =========================================================================================

__device__ __forceinline__ WorkEntry ldg_entry(const WorkEntry* p) {
    const int4 v = __ldg(reinterpret_cast<const int4*>(p));
    WorkEntry e;
    e.expert = v.x; e.pos0 = v.y; e.ntok = v.z; e.slot = v.w;
    return e;
}

__device__ __forceinline__ uint32_t ldg_stream16(const uint8_t* p) {
    uint16_t v;
    asm("ld.global.nc.L1::no_allocate.u16 %0, [%1];" : "=h"(v) : "l"(p));
    return v;
}

__device__ __forceinline__ float half_bits_to_float(uint32_t bits16) {
    return __half2float(__ushort_as_half(static_cast<unsigned short>(bits16)));
}

template <int W, int D, int NSTEP>
struct GeomRowsA {
    static constexpr int kThreads = W * 32;
    static constexpr int kHidden = NSTEP * 256;
    static constexpr int kActRow = kHidden * 2 + kPad;
    static constexpr int kActBytes = kTokTile * kActRow;
    static constexpr int kGroups = kHidden / 128;
    static constexpr int kBlockScaleBytes = NSTEP * 16;          // per 4-row block
    static constexpr int kXsBytes = kGroups * kTokTile * 4;
    static constexpr int kBarBytes = 64;
    static constexpr int kSmem = kBarBytes + kActBytes + kXsBytes;
    static_assert(NSTEP % D == 0, "the ring depth must divide the steps of a tile");
};

// One ring slot of kernel A: a step (256 columns) of rows g and g+8 of W1 and W3.
struct RingA {
    uint4 w[2][2][2];        // [matrix][row half][chunk of the step]
    uint32_t sc[2][2];       // [matrix][row half]: the two chunks' fp16 scales
};

template <int W, int D, int NSTEP>
__global__ void __launch_bounds__(W * 32, 1)
moe_w13_rows_kernel(const DecodeParams p) {
    using S = GeomRowsA<W, D, NSTEP>;
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t smem_base = ptx::smem_u32(smem);
    const uint32_t act_bar = smem_base;
    const uint32_t act_smem = smem_base + S::kBarBytes;
    const uint32_t xs_smem = act_smem + S::kActBytes;
    float* xs = reinterpret_cast<float*>(smem + S::kBarBytes + S::kActBytes);

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const int g = lane >> 2;
    const int t = lane & 3;

    const int entries = index_ok(p.counts[0], p.entries_cap + 1, p.error) ? p.counts[0] : 0;
    const int tiles = p.I / 16;                       // 16-row tiles per entry
    const int upe = (tiles + W - 1) / W;              // units per entry
    const int total_units = entries * upe;
    const int lo = static_cast<int>(static_cast<int64_t>(total_units) * blockIdx.x / gridDim.x);
    const int hi = static_cast<int>(static_cast<int64_t>(total_units) * (blockIdx.x + 1) / gridDim.x);
    if (lo >= hi) return;

    if (tid == 0) {
        ptx::mbar_init(act_bar, 1);
        ptx::fence_barrier_init();
    }
    __syncthreads();

    // Lane-constant offsets of its two rows inside a 16-row tile (4 row-blocks of 4 rows).
    uint32_t lane_off[2], lane_sc[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int r = g + 8 * h;
        const int blk = r >> 2, rib = r & 3;
        lane_off[h] = blk * p.w1.block_bytes + (rib * 8 + t) * 16;
        lane_sc[h] = blk * S::kBlockScaleBytes + rib * 4;
    }
    const uint64_t keep_policy = ptx::policy_evict_last();

    // A unit -> this warp's tile: the entry, the row tile, and the four stream bases.
    struct Tile {
        const uint8_t* wp[2];     // packed W1 / W3 of the tile
        const uint8_t* sp[2];     // scales  W1 / W3 of the tile
        WorkEntry e;
        int m, rt;
        bool active;
    };
    auto locate = [&](int u, Tile& x) {
        x.m = u / upe;
        x.rt = (u - x.m * upe) * W + warp;
        x.active = x.rt < tiles;
        x.e = ldg_entry(p.entries + x.m);
        const uint8_t* payload = p.pool + static_cast<uint64_t>(x.e.slot < 0 ? 0 : x.e.slot) * p.payload_bytes;
        const size_t rt = static_cast<size_t>(x.active ? x.rt : 0);
        x.wp[0] = payload + p.w1.packed_offset + rt * 4 * p.w1.block_bytes;
        x.wp[1] = payload + p.w3.packed_offset + rt * 4 * p.w3.block_bytes;
        x.sp[0] = payload + p.w1.scale_offset + rt * 4 * S::kBlockScaleBytes;
        x.sp[1] = payload + p.w3.scale_offset + rt * 4 * S::kBlockScaleBytes;
    };
    auto load_step = [&](RingA& r, const Tile& x, int step) {
#pragma unroll
        for (int mat = 0; mat < 2; ++mat)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint8_t* src = x.wp[mat] + lane_off[h] + step * 512;
                r.w[mat][h][0] = ldg_stream128(src);
                r.w[mat][h][1] = ldg_stream128(src + 64);
                r.sc[mat][h] = ldg_stream32(x.sp[mat] + lane_sc[h] + step * 16);
            }
    };

    Tile cur, nxt;
    locate(lo, cur);
    if (cur.e.slot < 0 && tid == 0) flag_error(p.error, kErrExpertAbsent);
    RingA ring[D];
    if (cur.active) {
#pragma unroll
        for (int d = 0; d < D; ++d) load_step(ring[d], cur, d);
    }

    int cur_entry = -1;
    uint32_t act_phase = 0;
    const uint32_t a_row = act_smem + g * S::kActRow;
    for (int u = lo; u < hi; ++u) {
        const bool has_next = u + 1 < hi;
        nxt = cur;
        if (has_next) {
            locate(u + 1, nxt);
            if (nxt.e.slot < 0 && tid == 0) flag_error(p.error, kErrExpertAbsent);
        }
        // ---- the entry's activation rows, when the CTA moves to another entry ----
        if (cur.m != cur_entry) {
            __syncthreads();                 // every warp is done with the previous rows
            if (warp == 0) {
                if (lane == 0) ptx::mbar_arrive_expect_tx(act_bar, cur.e.ntok * S::kHidden * 2);
                __syncwarp();
                if (lane < cur.e.ntok) {
                    // a token index outside the batch is reported and row 0 copied in its place
                    const int raw = index_ok(cur.e.pos0 + lane, p.draws_cap, p.error) ? __ldg(p.token_idx + cur.e.pos0 + lane) : 0;
                    const int token = index_ok(raw, p.tokens, p.error) ? raw : 0;
                    ptx::bulk_g2s(act_smem + lane * S::kActRow,
                                  p.xperm + static_cast<size_t>(token) * S::kHidden, S::kHidden * 2,
                                  act_bar, keep_policy);
                }
            }
            if (!ptx::mbar_wait(act_bar, act_phase & 1, p.error)) flag_error(p.error, kErrWaitTimeout);
            ++act_phase;
            cur_entry = cur.m;
            __syncwarp();
            group_sums<128, true>(act_smem, S::kActRow, 0, 1, cur.e.ntok, S::kGroups, xs, warp, W, lane);
            __syncthreads();
        }

        float acc[2][4];
#pragma unroll
        for (int a = 0; a < 2; ++a)
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[a][c] = 0.f;

        if (cur.active) {
#pragma unroll 1
            for (int s0 = 0; s0 < NSTEP; s0 += D) {
                const bool last = s0 + D >= NSTEP;
#pragma unroll
                for (int d = 0; d < D; ++d) {
                    const int s = s0 + d;
#pragma unroll
                    for (int cc = 0; cc < 2; ++cc) {
                        const int c = 2 * s + cc;
                        // Rows of tokens past the entry's count hold stale bytes: an MMA column
                        // only feeds its own output column, and those columns are never stored.
                        uint4 bf[4];
#pragma unroll
                        for (int i = 0; i < 4; ++i) bf[i] = ptx::lds128(a_row + (c * 128 + i * 32 + t * 8) * 2);
                        float2 xs8 = ptx::lds_f2(xs_smem + (c * kTokTile + 2 * t) * 4);
                        xs8.x *= -8.0f;
                        xs8.y *= -8.0f;
#pragma unroll
                        for (int mat = 0; mat < 2; ++mat) {
                            const uint32_t s0bits = ring[d].sc[mat][0], s1bits = ring[d].sc[mat][1];
                            const float sca = cc ? ptx::half_hi_as_float(s0bits) : ptx::half_lo_as_float(s0bits);
                            const float scb = cc ? ptx::half_hi_as_float(s1bits) : ptx::half_lo_as_float(s1bits);
                            const uint4 wa = ring[d].w[mat][0][cc], wb = ring[d].w[mat][1][cc];
                            float T[4];
                            ptx::mma_planes<true>(T, ptx::word_planes(wa.x, wb.x), bf[0]);
                            ptx::mma_planes<false>(T, ptx::word_planes(wa.y, wb.y), bf[1]);
                            ptx::mma_planes<false>(T, ptx::word_planes(wa.z, wb.z), bf[2]);
                            ptx::mma_planes<false>(T, ptx::word_planes(wa.w, wb.w), bf[3]);
                            ptx::fold_single(acc[mat], T, sca, scb, xs8);
                        }
                    }
                    // the slot is free: this tile's step s + D, or the next tile's step d
                    if (!last) load_step(ring[d], cur, s + D);
                    else if (has_next && nxt.active) load_step(ring[d], nxt, d);
                }
            }
            // clamped SwiGLU and the (hi, lo) store: gate and up of an element sit in one lane
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int token = 2 * t + (j & 1);
                const int row = g + 8 * (j >> 1);
                if (token < cur.e.ntok) {
                    const float gate = fminf(acc[0][j], p.limit);
                    const float up = fminf(fmaxf(acc[1][j], -p.limit), p.limit);
                    const float hval = (gate / (1.0f + expf(-gate))) * up;
                    __half hi16 = __float2half_rn(hval);
                    __half lo16 = __float2half_rn(hval - __half2float(hi16));
                    if (g & 2) {   // hidden columns that meet kernel B's high-nibble plane: stored / 16
                        hi16 = __hmul(hi16, __float2half_rn(0.0625f));
                        lo16 = __hmul(lo16, __float2half_rn(0.0625f));
                    }
                    const size_t at = static_cast<size_t>(cur.e.pos0 + token) * p.I + perm_col<128>(cur.rt * 16 + row);
                    if (index_ok(static_cast<long long>(at), p.hidden_elems, p.error)) {
                        p.hid_hi[at] = hi16;
                        p.hid_lo[at] = lo16;
                    }
                }
            }
        } else if (has_next && nxt.active) {
            // an idle warp of a partly filled unit still starts its next tile's stream
#pragma unroll
            for (int d = 0; d < D; ++d) load_step(ring[d], nxt, d);
        }
        cur = nxt;
    }
}

template <int W, int MT, int D, int NCHUNK>
struct GeomRowsB {
    static constexpr int kThreads = W * 32;
    static constexpr int kInter = NCHUNK * 128;
    static constexpr int kActRow = 2 * kInter * 2 + kPad;           // hi then lo
    static constexpr int kActBytes = kTokTile * kActRow;
    static constexpr int kGroups = NCHUNK;
    static constexpr int kBlockScaleBytes = NCHUNK * 16;           // per 8-row block
    static constexpr int kXsBytes = kGroups * 2 * kTokTile * 4;    // [group][hi|lo][token]
    static constexpr int kBarBytes = 64;
    static constexpr int kSmem = kBarBytes + kActBytes + kXsBytes;
    static constexpr int kItemRows = MT * 16;
    static_assert(NCHUNK % D == 0, "the ring depth must divide the chunks of a tile");
};

// One ring slot of kernel B: a chunk (128 columns) of rows g and g+8 of MT tiles of W2.
template <int MT>
struct RingB {
    uint4 w[MT][2];
    uint32_t sc[MT][2];
};

template <int W, int MT, int D, int NCHUNK>
__global__ void __launch_bounds__(W * 32, 1)
moe_w2_rows_kernel(const DecodeParams p) {
    using S = GeomRowsB<W, MT, D, NCHUNK>;
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t smem_base = ptx::smem_u32(smem);
    const uint32_t act_bar = smem_base;
    const uint32_t act_smem = smem_base + S::kBarBytes;
    const uint32_t xs_smem = act_smem + S::kActBytes;
    float* xs = reinterpret_cast<float*>(smem + S::kBarBytes + S::kActBytes);

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const int g = lane >> 2;
    const int t = lane & 3;

    const int entries = index_ok(p.counts[0], p.entries_cap + 1, p.error) ? p.counts[0] : 0;
    const int items = p.H / S::kItemRows;             // MT-tile items per entry
    const int upe = (items + W - 1) / W;
    const int total_units = entries * upe;
    const int lo = static_cast<int>(static_cast<int64_t>(total_units) * blockIdx.x / gridDim.x);
    const int hi = static_cast<int>(static_cast<int64_t>(total_units) * (blockIdx.x + 1) / gridDim.x);
    if (lo >= hi) return;

    if (tid == 0) {
        ptx::mbar_init(act_bar, 1);
        ptx::fence_barrier_init();
    }
    __syncthreads();

    // W2 row-blocks hold 8 rows: rows g of a tile are its first block, rows g+8 the second; a
    // warp's 32 lanes read one contiguous 512-byte line per block and chunk.
    const uint32_t lane_off = (g * 4 + t) * 16;
    const uint32_t lane_sc = g * 2;
    const uint64_t keep_policy = ptx::policy_evict_last();

    struct Tile {
        const uint8_t* wp;        // packed rows of the item (2 * MT row-blocks)
        const uint8_t* sp;        // their scales
        WorkEntry e;
        int m, it;
        bool active;
    };
    auto locate = [&](int u, Tile& x) {
        x.m = u / upe;
        x.it = (u - x.m * upe) * W + warp;
        x.active = x.it < items;
        x.e = ldg_entry(p.entries + x.m);
        const uint8_t* payload = p.pool + static_cast<uint64_t>(x.e.slot < 0 ? 0 : x.e.slot) * p.payload_bytes;
        const size_t block0 = static_cast<size_t>(x.active ? x.it : 0) * 2 * MT;
        x.wp = payload + p.w2.packed_offset + block0 * p.w2.block_bytes;
        x.sp = payload + p.w2.scale_offset + block0 * S::kBlockScaleBytes;
    };
    auto load_chunk_b = [&](RingB<MT>& r, const Tile& x, int c) {
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int blk = mt * 2 + h;
                r.w[mt][h] = ldg_stream128(x.wp + static_cast<size_t>(blk) * p.w2.block_bytes + lane_off + c * 512);
                r.sc[mt][h] = ldg_stream16(x.sp + blk * S::kBlockScaleBytes + lane_sc + c * 16);
            }
    };

    Tile cur, nxt;
    locate(lo, cur);
    if (cur.e.slot < 0 && tid == 0) flag_error(p.error, kErrExpertAbsent);
    RingB<MT> ring[D];
    if (cur.active) {
#pragma unroll
        for (int d = 0; d < D; ++d) load_chunk_b(ring[d], cur, d);
    }

    int cur_entry = -1;
    uint32_t act_phase = 0;
    int my_draw[2] = {0, 0};
    float my_weight[2] = {0.f, 0.f};
    for (int u = lo; u < hi; ++u) {
        const bool has_next = u + 1 < hi;
        nxt = cur;
        if (has_next) {
            locate(u + 1, nxt);
            if (nxt.e.slot < 0 && tid == 0) flag_error(p.error, kErrExpertAbsent);
        }
        if (cur.m != cur_entry) {
            __syncthreads();
            if (warp == 0) {
                if (lane == 0) ptx::mbar_arrive_expect_tx(act_bar, cur.e.ntok * S::kInter * 4);
                __syncwarp();
                if (lane < 2 * cur.e.ntok) {
                    const int tok = lane >> 1, part = lane & 1;
                    const int pos = index_ok(cur.e.pos0 + tok, p.draws_cap, p.error) ? cur.e.pos0 + tok : 0;
                    const __half* src = (part == 0 ? p.hid_hi : p.hid_lo) + static_cast<size_t>(pos) * S::kInter;
                    ptx::bulk_g2s(act_smem + tok * S::kActRow + part * S::kInter * 2, src, S::kInter * 2,
                                  act_bar, keep_policy);
                }
            }
            if (!ptx::mbar_wait(act_bar, act_phase & 1, p.error)) flag_error(p.error, kErrWaitTimeout);
            ++act_phase;
            cur_entry = cur.m;
            __syncwarp();
            group_sums<128, true>(act_smem, S::kActRow, S::kInter * 2, 2, cur.e.ntok, S::kGroups, xs, warp, W, lane);
            __syncthreads();
            // the two tokens this lane stores for: draw rows and routing weights, once per entry
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int token = 2 * t + j;
                const bool live = token < cur.e.ntok && index_ok(cur.e.pos0 + token, p.draws_cap, p.error);
                my_draw[j] = live ? __ldg(p.draw_idx + cur.e.pos0 + token) : -1;
                my_weight[j] = live ? __ldg(p.wpos + cur.e.pos0 + token) : 0.f;
                // a draw index outside the scratch is reported; the lane then stores nothing for it
                if (live && !index_ok(my_draw[j], p.draws_cap, p.error)) my_draw[j] = -1;
            }
        }

        // Up to four tokens: hi and lo ride in one MMA as eight token columns (0-3 hi of tokens
        // 0-3, 4-7 lo) and the two halves are added in the epilogue. More tokens: one pass per part.
        const bool packed = cur.e.ntok <= 4;
        float acc[MT][4];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[mt][c] = 0.f;

        if (cur.active) {
            const int tok = packed ? (g & 3) : g;
            const uint32_t b_tok = act_smem + tok * S::kActRow;
#pragma unroll 1
            for (int c0 = 0; c0 < NCHUNK; c0 += D) {
                const bool last = c0 + D >= NCHUNK;
#pragma unroll
                for (int d = 0; d < D; ++d) {
                    const int c = c0 + d;
                    // Packed: one pass over eight columns (hi of tokens 0-3, lo of tokens 0-3). Otherwise
                    // the hi and the lo part of the eight tokens are two passes that share the masked
                    // weight planes and add into the same accumulator (same token columns).
                    const uint32_t b_first = b_tok + (packed ? (g >> 2) : 0) * (S::kInter * 2) + (c * 128 + t * 8) * 2;
                    const uint32_t xs_at = xs_smem + (c * 2 * kTokTile + (packed ? ((t >> 1) * kTokTile + 2 * (t & 1)) : 2 * t)) * 4;
                    float2 xs8 = ptx::lds_f2(xs_at);
                    if (!packed) {
                        const float2 lo_sum = ptx::lds_f2(xs_at + kTokTile * 4);
                        xs8.x += lo_sum.x;
                        xs8.y += lo_sum.y;
                    }
                    xs8.x *= -8.0f;
                    xs8.y *= -8.0f;
                    float T[MT][4], Tb[MT][4];     // the lo pass keeps its own chain: twice the MMAs in flight
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const uint4 bf_a = ptx::lds128(b_first + i * 64);
                        uint4 bf_b = make_uint4(0, 0, 0, 0);
                        if (!packed) bf_b = ptx::lds128(b_first + S::kInter * 2 + i * 64);
#pragma unroll
                        for (int mt = 0; mt < MT; ++mt) {
                            const uint4 wa = ring[d].w[mt][0], wb = ring[d].w[mt][1];
                            const uint32_t wai = i == 0 ? wa.x : i == 1 ? wa.y : i == 2 ? wa.z : wa.w;
                            const uint32_t wbi = i == 0 ? wb.x : i == 1 ? wb.y : i == 2 ? wb.z : wb.w;
                            const ptx::WordPlanes planes = ptx::word_planes(wai, wbi);
                            if (i == 0) ptx::mma_planes<true>(T[mt], planes, bf_a);
                            else ptx::mma_planes<false>(T[mt], planes, bf_a);
                            if (!packed) {
                                if (i == 0) ptx::mma_planes<true>(Tb[mt], planes, bf_b);
                                else ptx::mma_planes<false>(Tb[mt], planes, bf_b);
                            }
                        }
                    }
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        if (!packed) {
#pragma unroll
                            for (int q = 0; q < 4; ++q) T[mt][q] += Tb[mt][q];
                        }
                        ptx::fold_single(acc[mt], T[mt], half_bits_to_float(ring[d].sc[mt][0]),
                                         half_bits_to_float(ring[d].sc[mt][1]), xs8);
                    }
                    if (!last) load_chunk_b(ring[d], cur, c + D);
                    else if (has_next && nxt.active) load_chunk_b(ring[d], nxt, d);
                }
            }
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float v = acc[mt][j];
                    if (packed) v += __shfl_xor_sync(0xFFFFFFFFu, v, 2);   // lo half sits two lanes on
                    const int token = 2 * t + (j & 1);
                    const bool mine = packed ? (t < 2) : true;
                    const int row = (cur.it * MT + mt) * 16 + g + 8 * (j >> 1);
                    if (mine && token < cur.e.ntok && my_draw[j & 1] >= 0)
                        p.contrib[static_cast<size_t>(my_draw[j & 1]) * p.H + row] = my_weight[j & 1] * v;
                }
        } else if (has_next && nxt.active) {
#pragma unroll
            for (int d = 0; d < D; ++d) load_chunk_b(ring[d], nxt, d);
        }
        cur = nxt;
    }
}

// ----- kernel C: slot-order accumulate -------------------------------------------------------
// accum[t, :] += sum over slot 0..k-1, in that order, of contrib[t*k + slot, :] (fp32). The
// fixed order and the single writer per element of kernel B make the whole routed path
// bit-reproducible. Draws whose expert id is out of range, or absent when absent experts are
// skipped, contribute nothing.
__global__ void moe_accumulate_kernel(float* __restrict__ accum, int64_t accum_stride,
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

// ----- activation staging: 16-bit -> fp16 in the kernels' column order -------------------
template <int G>
__global__ void stage_activations_kernel(const void* __restrict__ x, int64_t x_stride, int dtype,
                                         int tokens, int H, __half* __restrict__ out, long long out_elems,
                                         int32_t* __restrict__ error) {
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
        __half h = __float2half_rn(v);
        // group 128 (row-streaming kernels): columns that meet the high-nibble plane are stored / 16
        if (G == 128 && (k & 2)) h = __hmul(h, __float2half_rn(0.0625f));
        const size_t at = static_cast<size_t>(token) * H + perm_col<G>(k);
        if (index_ok(static_cast<long long>(at), out_elems, error)) out[at] = h;
    }
}

template <class KernelA, class KernelB>
void launch_pair(aeon_b200_ctx* ctx, const DecodeParams& p, KernelA ka, int threads_a, int smem_a,
                 KernelB kb, int threads_b, int smem_b, int ctas_per_sm_b, cudaStream_t stream) {
    AEON_CUDA_CHECK(cudaFuncSetAttribute(ka, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_a));
    AEON_CUDA_CHECK(cudaFuncSetAttribute(kb, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_b));
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
    ka<<<ctx->sm_count, threads_a, smem_a, stream>>>(p);
    AEON_CUDA_CHECK(cudaGetLastError());
    if (ev) AEON_CUDA_CHECK(cudaEventRecord(ev[1], stream));
    kb<<<ctx->sm_count * ctas_per_sm_b, threads_b, smem_b, stream>>>(p);
    AEON_CUDA_CHECK(cudaGetLastError());
    if (ev) AEON_CUDA_CHECK(cudaEventRecord(ev[2], stream));
    ctx->launches += 2;
    if (p.accum != nullptr) {
        const int64_t vecs = static_cast<int64_t>(p.tokens) * p.H / 4;
        const int blocks = static_cast<int>(std::min<int64_t>((vecs + 255) / 256, 4 * ctx->sm_count));
        moe_accumulate_kernel<<<blocks, 256, 0, stream>>>(p.accum, p.accum_stride, p.contrib, p.topk_ids,
                                                          p.slot_of, p.skip_absent, p.overwrite, p.experts,
                                                          p.tokens, p.top_k, p.H, ctx->pool_slots);
        AEON_CUDA_CHECK(cudaGetLastError());
        ctx->launches += 1;
    }
}

template <int G, int KWA, int NCHA, int MWB = 2, int MTB = 2, int KWB = 8, int NCHB = 2, int PB = 1>
void launch_decode_kernels(aeon_b200_ctx* ctx, const DecodeParams& p, cudaStream_t stream) {
    using SA = GeomA<G, KWA, NCHA>;
    // intermediate = 2048: two workers of eight warps, two 16-row tiles per worker, two chunks
    // per warp (64-row items). Measured alternatives, all slower on B200: four K-warps x four
    // chunks with two CTAs per SM (spills under the 128-register cap, 2.0 TB/s), one worker of
    // four tiles (2.8 TB/s), one worker with two items in flight (2.8 TB/s); this one 3.1 TB/s.
    using SB = GeomB<G, MWB, MTB, KWB, NCHB, PB>;
    if (p.I != SB::kInter || p.H != SA::kHidden)
        throw StatusError(AEON_B200_ERR_UNSUPPORTED,
                          "aeon_b200_moe_decode: no kernel instance for this hidden/intermediate size");
    launch_pair(ctx, p, moe_w13_swiglu_kernel<G, KWA, NCHA>, SA::kThreads, SA::kSmem,
                moe_w2_contrib_kernel<G, MWB, MTB, KWB, NCHB, PB>, SB::kThreads, SB::kSmem, 1, stream);
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
    require(ranks > 0 && tokens > 0 && hidden > 0 && hidden % 4 == 0 && out_stride % 4 == 0 &&
                aligned16(out) && aligned16(partials),
            "aeon_b200_ep_combine: hidden and out_stride must be multiples of 4, pointers 16-byte aligned");
    const int64_t total = static_cast<int64_t>(tokens) * hidden / 4;
    const int blocks = static_cast<int>(std::min<int64_t>((total + 255) / 256, 2048));
    ep_combine_kernel<<<blocks, 256, 0, stream>>>(out, out_stride, partials, ranks, tokens, hidden);
    AEON_CUDA_CHECK(cudaGetLastError());
}

void launch_moe_accumulate(aeon_b200_ctx* ctx, const int32_t* slot_of_expert, const int32_t* topk_ids,
                           int tokens, float* moe_accum, int64_t accum_stride, uint32_t flags,
                           cudaStream_t stream) {
    const aeon_b200_moe_config& cfg = ctx->cfg;
    require(slot_of_expert && topk_ids && moe_accum, "aeon_b200_moe_accumulate: null pointer argument");
    require(tokens > 0 && tokens <= ctx->max_tokens,
            "aeon_b200_moe_accumulate: tokens must be in [1, max_tokens of the context]");
    require(accum_stride >= cfg.hidden && accum_stride % 4 == 0 && aligned16(moe_accum),
            "aeon_b200_moe_accumulate: moe_accum must be 16-byte aligned, accum_stride >= hidden and a "
            "multiple of 4");
    const int64_t vecs = static_cast<int64_t>(tokens) * cfg.hidden / 4;
    const int blocks = static_cast<int>(std::min<int64_t>((vecs + 255) / 256, 4 * ctx->sm_count));
    moe_accumulate_kernel<<<blocks, 256, 0, stream>>>(
        moe_accum, accum_stride, ctx->d_contrib, topk_ids, slot_of_expert,
        (flags & AEON_B200_DECODE_SKIP_ABSENT) ? 1 : 0, (flags & AEON_B200_DECODE_OVERWRITE) ? 1 : 0,
        cfg.experts, tokens, cfg.top_k, cfg.hidden, ctx->pool_slots);
    AEON_CUDA_CHECK(cudaGetLastError());
    ctx->launches += 1;
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
    require(accum_stride % 4 == 0 && aligned16(moe_accum),
            "aeon_b200_moe_decode: moe_accum must be 16-byte aligned and accum_stride a multiple of 4 "
            "(the accumulate uses 128-bit accesses)");

    // 1. draws sorted by expert + work list, on the context's own stream: it needs the routing only
    //    and runs beside the staging of the activations (two short, latency-bound kernels). Under
    //    stream capture the two events become graph edges.
    AEON_CUDA_CHECK(cudaEventRecord(ctx->aux_fork, stream));
    AEON_CUDA_CHECK(cudaStreamWaitEvent(ctx->aux_stream, ctx->aux_fork, 0));
    launch_permutation(ctx, topk_ids, tokens, cfg.top_k, cfg.experts, ctx->d_offsets,
                       ctx->d_token_idx, ctx->d_draw_idx, topk_weights, ctx->d_wpos,
                       slot_of_expert, ctx->d_entries, ctx->d_counts,
                       (flags & AEON_B200_DECODE_SKIP_ABSENT) != 0, ctx->aux_stream);
    AEON_CUDA_CHECK(cudaEventRecord(ctx->aux_join, ctx->aux_stream));

    // 2. activations -> fp16 in kernel column order
    const int64_t total = static_cast<int64_t>(tokens) * cfg.hidden;
    const int blocks = static_cast<int>(std::min<int64_t>((total + 255) / 256, 4 * ctx->sm_count));
    if (cfg.group_size == 128) {
        stage_activations_kernel<128><<<blocks, 256, 0, stream>>>(
            x, x_stride, cfg.act_dtype, tokens, cfg.hidden, ctx->d_xperm,
            static_cast<long long>(ctx->max_tokens) * cfg.hidden, ctx->d_error);
    } else {
        stage_activations_kernel<32><<<blocks, 256, 0, stream>>>(
            x, x_stride, cfg.act_dtype, tokens, cfg.hidden, ctx->d_xperm,
            static_cast<long long>(ctx->max_tokens) * cfg.hidden, ctx->d_error);
    }
    AEON_CUDA_CHECK(cudaGetLastError());
    ctx->launches += 1;

    AEON_CUDA_CHECK(cudaStreamWaitEvent(stream, ctx->aux_join, 0));

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
    p.overwrite = (flags & AEON_B200_DECODE_OVERWRITE) ? 1 : 0;
    p.experts = cfg.experts;
    p.hid_hi = ctx->d_hidden_hi;
    p.hid_lo = ctx->d_hidden_lo;
    p.contrib = ctx->d_contrib;
    p.accum = (flags & AEON_B200_DECODE_DEFER_ACCUMULATE) ? nullptr : moe_accum;
    p.accum_stride = accum_stride;
    p.limit = cfg.swiglu_limit;
    p.error = ctx->d_error;
    p.draws_cap = ctx->max_tokens * cfg.top_k;
    p.hidden_elems = static_cast<long long>(p.draws_cap) * cfg.intermediate;
    p.contrib_elems = static_cast<long long>(p.draws_cap) * cfg.hidden;
    p.entries_cap = cfg.experts + p.draws_cap / 8 + 1;

    // Kernel instances: K-warps x chunks-per-warp x 128 columns = hidden.
    // Group 128: the row-streaming kernels. Kernel A: eight warps (two per scheduler, no register
    // cap in the way) with a four-step ring, 128 KB of weights in flight per SM; kernel B: sixteen
    // warps of two tiles each with a two-chunk ring. Both chosen by timing the alternatives on
    // B200 (8/12/16 warps x ring depths 1..8), alone and beside the shared expert's kernels. Group
    // 32 (the reference model's own shape) keeps the K-split kernels.
    if (cfg.group_size == 128 && cfg.intermediate == 2048 && (cfg.hidden == 7168 || cfg.hidden == 4096)) {
        using SB = GeomRowsB<16, 2, 2, 16>;
        if (cfg.hidden == 7168) {
            using SA = GeomRowsA<8, 4, 28>;
            launch_pair(ctx, p, moe_w13_rows_kernel<8, 4, 28>, SA::kThreads, SA::kSmem,
                        moe_w2_rows_kernel<16, 2, 2, 16>, SB::kThreads, SB::kSmem, 1, stream);
        } else {
            using SA = GeomRowsA<8, 4, 16>;
            launch_pair(ctx, p, moe_w13_rows_kernel<8, 4, 16>, SA::kThreads, SA::kSmem,
                        moe_w2_rows_kernel<16, 2, 2, 16>, SB::kThreads, SB::kSmem, 1, stream);
        }
    } else if (cfg.group_size == 32 && cfg.hidden == 4096) {
        launch_decode_kernels<32, 16, 2>(ctx, p, stream);
    } else if (cfg.group_size == 32 && cfg.hidden == 7168) {
        launch_decode_kernels<32, 14, 4>(ctx, p, stream);
    } else {
        throw StatusError(AEON_B200_ERR_UNSUPPORTED,
                          "aeon_b200_moe_decode: supported hidden sizes are 4096 and 7168 "
                          "(intermediate 2048)");
    }
}

}  // namespace aeon_b200
