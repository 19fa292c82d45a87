// Shard-aware expert payloads (host only): the "expert v3" layout of the reference's
// multi-GPU plan (plans-and-docs/execution/active/MULTI_GPU_EXECUTION_PLAN.md:151-181), which
// the reference itself has not built (its writer, scripts/convert_safetensors_to_aeon.py:46-187,
// and its loader, src/infrastructure/artifact/aeon_loader.hpp:345-405, stop at v2).
//
// A v3 payload is `shards` complete payloads back to back. Shard s holds the slice
// [s * I/shards, (s+1) * I/shards) of the expert's intermediate dimension: those rows of W1
// and W3 and those columns of W2, cut from the checkpoint (source) layout and swizzled as
// matrices of their own, in the region order and 4 KiB alignment of a whole payload
// (the shard rule of tests/test_expert_shard_equivalence.cpp:286-340 and
// tests/test_w2_shard_equivalence.cpp:92-112). A tensor-parallel rank of degree tp reads the
// shards/tp consecutive shards that start at rank * shards/tp: one contiguous, 4 KiB-aligned
// byte range, disjoint from every other rank's, the ranges together covering the payload.
// shards == 1 is the v2 payload, byte for byte.
#include "common.cuh"

#include <cstring>
#include <vector>

namespace aeon_b200 {
namespace {

struct ShardPlan {
    aeon_b200_moe_config whole, unit;   // the expert and one shard of it
    ExpertGeom whole_geom, unit_geom;
    int shards, Is;
};

ShardPlan make_plan(const aeon_b200_moe_config* cfg, int shards, const char* who) {
    require(cfg != nullptr, who);
    require(shards > 0 && cfg->intermediate % shards == 0, "expert shards: shard count must divide the intermediate size");
    ShardPlan p{};
    p.whole = *cfg;
    p.unit = *cfg;
    p.unit.intermediate = cfg->intermediate / shards;
    p.whole_geom = make_geom(p.whole);     // validates (multiples of 256 included)
    p.unit_geom = make_geom(p.unit);
    p.shards = shards;
    p.Is = p.unit.intermediate;
    return p;
}

struct SourceConst {
    const uint32_t *w1p, *w2p, *w3p;
    const uint16_t *w1s, *w2s, *w3s;
};
struct SourceMut {
    uint32_t *w1p, *w2p, *w3p;
    uint16_t *w1s, *w2s, *w3s;
};

// One payload of `geom` (intermediate = rows_i) <-> source tensors whose intermediate dimension
// is `src_i` wide, of which the payload covers [first, first + rows_i).
void payload_from_source(const aeon_b200_moe_config& c, const ExpertGeom& geom, int rows_i, int src_i,
                         int first, const SourceConst& src, uint8_t* payload) {
    const int H = c.hidden, G = c.group_size;
    std::memset(payload, 0, geom.payload_bytes);
    auto packed = [&](const MatrixGeom& m) { return reinterpret_cast<uint32_t*>(payload + m.packed_offset); };
    auto scales = [&](const MatrixGeom& m) { return reinterpret_cast<uint16_t*>(payload + m.scale_offset); };
    // W1 / W3: rows of the source are contiguous
    const size_t row_words = H / 8, row_scales = H / G;
    relayout_w4a16(src.w1p + first * row_words, src.w1s + first * row_scales, packed(geom.w1), scales(geom.w1),
                   rows_i, H, c.w13_rpw, c.w13_lpr, G, true);
    relayout_w4a16(src.w3p + first * row_words, src.w3s + first * row_scales, packed(geom.w3), scales(geom.w3),
                   rows_i, H, c.w13_rpw, c.w13_lpr, G, true);
    // W2: a column range of every row
    std::vector<uint32_t> cut_p(static_cast<size_t>(H) * rows_i / 8);
    std::vector<uint16_t> cut_s(static_cast<size_t>(H) * rows_i / G);
    for (int r = 0; r < H; ++r) {
        std::memcpy(&cut_p[static_cast<size_t>(r) * rows_i / 8],
                    src.w2p + static_cast<size_t>(r) * src_i / 8 + first / 8, rows_i / 8 * sizeof(uint32_t));
        std::memcpy(&cut_s[static_cast<size_t>(r) * rows_i / G],
                    src.w2s + static_cast<size_t>(r) * src_i / G + first / G, rows_i / G * sizeof(uint16_t));
    }
    relayout_w4a16(cut_p.data(), cut_s.data(), packed(geom.w2), scales(geom.w2), H, rows_i, c.w2_rpw, c.w2_lpr,
                   G, true);
}

void source_from_payload(const aeon_b200_moe_config& c, const ExpertGeom& geom, int rows_i, int dst_i,
                         int first, const uint8_t* payload, const SourceMut& dst) {
    const int H = c.hidden, G = c.group_size;
    auto packed = [&](const MatrixGeom& m) { return reinterpret_cast<const uint32_t*>(payload + m.packed_offset); };
    auto scales = [&](const MatrixGeom& m) { return reinterpret_cast<const uint16_t*>(payload + m.scale_offset); };
    const size_t row_words = H / 8, row_scales = H / G;
    relayout_w4a16(packed(geom.w1), scales(geom.w1), dst.w1p + first * row_words, dst.w1s + first * row_scales,
                   rows_i, H, c.w13_rpw, c.w13_lpr, G, false);
    relayout_w4a16(packed(geom.w3), scales(geom.w3), dst.w3p + first * row_words, dst.w3s + first * row_scales,
                   rows_i, H, c.w13_rpw, c.w13_lpr, G, false);
    std::vector<uint32_t> cut_p(static_cast<size_t>(H) * rows_i / 8);
    std::vector<uint16_t> cut_s(static_cast<size_t>(H) * rows_i / G);
    relayout_w4a16(packed(geom.w2), scales(geom.w2), cut_p.data(), cut_s.data(), H, rows_i, c.w2_rpw, c.w2_lpr,
                   G, false);
    for (int r = 0; r < H; ++r) {
        std::memcpy(dst.w2p + static_cast<size_t>(r) * dst_i / 8 + first / 8,
                    &cut_p[static_cast<size_t>(r) * rows_i / 8], rows_i / 8 * sizeof(uint32_t));
        std::memcpy(dst.w2s + static_cast<size_t>(r) * dst_i / G + first / G,
                    &cut_s[static_cast<size_t>(r) * rows_i / G], rows_i / G * sizeof(uint16_t));
    }
}

}  // namespace
}  // namespace aeon_b200

using namespace aeon_b200;

extern "C" {

int aeon_b200_expert_shard_bytes(const aeon_b200_moe_config* cfg, int shards, uint64_t* shard_bytes) {
    return guarded([&] {
        require(shard_bytes != nullptr, "aeon_b200_expert_shard_bytes: null argument");
        const ShardPlan p = make_plan(cfg, shards, "aeon_b200_expert_shard_bytes: null config");
        *shard_bytes = p.unit_geom.payload_bytes;
    });
}

int aeon_b200_pack_expert_shards(const aeon_b200_moe_config* cfg, int shards, const uint32_t* w1p,
                                 const uint16_t* w1s, const uint32_t* w2p, const uint16_t* w2s,
                                 const uint32_t* w3p, const uint16_t* w3s, uint8_t* payload) {
    return guarded([&] {
        require(w1p && w1s && w2p && w2s && w3p && w3s && payload, "aeon_b200_pack_expert_shards: null pointer argument");
        const ShardPlan p = make_plan(cfg, shards, "aeon_b200_pack_expert_shards: null config");
        const SourceConst src{w1p, w2p, w3p, w1s, w2s, w3s};
        for (int s = 0; s < shards; ++s)
            payload_from_source(p.unit, p.unit_geom, p.Is, p.whole.intermediate, s * p.Is, src,
                                payload + static_cast<uint64_t>(s) * p.unit_geom.payload_bytes);
    });
}

int aeon_b200_unpack_expert_shards(const aeon_b200_moe_config* cfg, int shards, const uint8_t* payload,
                                   uint32_t* w1p, uint16_t* w1s, uint32_t* w2p, uint16_t* w2s,
                                   uint32_t* w3p, uint16_t* w3s) {
    return guarded([&] {
        require(w1p && w1s && w2p && w2s && w3p && w3s && payload, "aeon_b200_unpack_expert_shards: null pointer argument");
        const ShardPlan p = make_plan(cfg, shards, "aeon_b200_unpack_expert_shards: null config");
        const SourceMut dst{w1p, w2p, w3p, w1s, w2s, w3s};
        for (int s = 0; s < shards; ++s)
            source_from_payload(p.unit, p.unit_geom, p.Is, p.whole.intermediate, s * p.Is,
                                payload + static_cast<uint64_t>(s) * p.unit_geom.payload_bytes, dst);
    });
}

int aeon_b200_expert_rank_slice(const aeon_b200_moe_config* cfg, int shards, int tp, int rank,
                                uint64_t* offset, uint64_t* length) {
    return guarded([&] {
        require(offset && length, "aeon_b200_expert_rank_slice: null argument");
        const ShardPlan p = make_plan(cfg, shards, "aeon_b200_expert_rank_slice: null config");
        if (tp <= 0 || shards % tp != 0)
            throw StatusError(AEON_B200_ERR_INVALID_ARGUMENT,
                              "aeon_b200_expert_rank_slice: tensor_parallel=" + std::to_string(tp) +
                                  " does not divide the artifact's max tensor-parallel degree " +
                                  std::to_string(shards));
        if (rank < 0 || rank >= tp)
            throw StatusError(AEON_B200_ERR_OUT_OF_RANGE, "aeon_b200_expert_rank_slice: rank out of range");
        const uint64_t per_rank = static_cast<uint64_t>(shards / tp) * p.unit_geom.payload_bytes;
        *offset = static_cast<uint64_t>(rank) * per_rank;
        *length = per_rank;
    });
}

int aeon_b200_merge_expert_shards(const aeon_b200_moe_config* cfg, int shards, const uint8_t* slice,
                                  uint8_t* payload) {
    return guarded([&] {
        require(slice && payload, "aeon_b200_merge_expert_shards: null pointer argument");
        // `cfg` describes the slice as a whole (intermediate = shards * shard width)
        const ShardPlan p = make_plan(cfg, shards, "aeon_b200_merge_expert_shards: null config");
        if (shards == 1) {
            std::memcpy(payload, slice, p.whole_geom.payload_bytes);
            return;
        }
        const size_t H = p.whole.hidden, I = p.whole.intermediate, G = p.whole.group_size;
        std::vector<uint32_t> w1p(I * H / 8), w2p(H * I / 8), w3p(I * H / 8);
        std::vector<uint16_t> w1s(I * H / G), w2s(H * I / G), w3s(I * H / G);
        const SourceMut mid{w1p.data(), w2p.data(), w3p.data(), w1s.data(), w2s.data(), w3s.data()};
        for (int s = 0; s < shards; ++s)
            source_from_payload(p.unit, p.unit_geom, p.Is, p.whole.intermediate, s * p.Is,
                                slice + static_cast<uint64_t>(s) * p.unit_geom.payload_bytes, mid);
        const SourceConst src{w1p.data(), w2p.data(), w3p.data(), w1s.data(), w2s.data(), w3s.data()};
        payload_from_source(p.whole, p.whole_geom, p.whole.intermediate, p.whole.intermediate, 0, src, payload);
    });
}

}  // extern "C"
