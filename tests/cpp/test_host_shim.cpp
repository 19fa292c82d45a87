// Host-only checks of the C++ layer (no GPU): the topology resolver and id parser against
// the cases of the reference's tests/test_parallel_topology.cpp:83-256 (stage-major mapping,
// 43-layer splits, refusals, parser), the registry's reservation / lease / eviction state
// machine with the invariant audit after every step
// (tests/test_expert_registry_warm_state.cpp), the expert container round trip
// (index header + entries, the loader contract of aeon_loader.hpp:345-405), the shard-aware
// version 3 of it with rank slices, and the dense container behind AeonModelLoader.
#include "aeon_b200_host.hpp"

#include <sstream>

#include <cstdio>
#include <cstdlib>
#include <functional>

using namespace aeon::core;

static int g_fail = 0;
static void check(const char* label, bool ok) {
    std::printf("  %-70s %s\n", label, ok ? "PASS" : "FAIL");
    if (!ok) ++g_fail;
}
template <class E>
static bool throws(const std::function<void()>& f, const char* needle = nullptr) {
    try { f(); } catch (const E& e) { return needle == nullptr || std::string(e.what()).find(needle) != std::string::npos; }
    catch (...) { return false; }
    return false;
}

int main(int argc, char** argv) {
    const std::string tmp = argc > 1 ? argv[1] : "/tmp";
    std::printf("[host shim]\n");
    // ---- topology ----
    {
        ParallelTopologyConfig c; c.tensor_parallel = 2; c.pipeline_parallel = 2; c.device_ids = {3, 1, 0, 2};
        const ParallelTopology t = ParallelTopology::resolve(c, 4, 8, 43);
        check("stage-major device mapping", t.device(0, 0) == 3 && t.device(0, 1) == 1 && t.device(1, 0) == 0 && t.device(1, 1) == 2);
        check("43 layers over 2 stages: 22 + 21", t.stage_layers(0).count == 22 && t.stage_layers(1).first == 22 && t.stage_layers(1).count == 21);
        check("stage_of", t.stage_of(0) == 0 && t.stage_of(21) == 0 && t.stage_of(22) == 1 && t.stage_of(42) == 1);
    }
    for (uint32_t pp : {1u, 2u, 3u, 4u}) {
        ParallelTopologyConfig c; c.pipeline_parallel = pp;
        const ParallelTopology t = ParallelTopology::resolve(c, 8, 1, 43);
        uint32_t total = 0, prev_end = 0; bool contiguous = true, front_heavy = true;
        for (uint32_t s = 0; s < pp; ++s) {
            contiguous &= t.stage_layers(s).first == prev_end;
            prev_end = t.stage_layers(s).end(); total += t.stage_layers(s).count;
            if (s) front_heavy &= t.stage_layers(s).count <= t.stage_layers(s - 1).count;
        }
        check("43-layer split is contiguous, complete, remainder first", contiguous && total == 43 && front_heavy);
    }
    {
        ParallelTopologyConfig c;
        check("default topology is single device", ParallelTopology::resolve(c, 1, 1, 43).is_single_device());
        c.tensor_parallel = 0;
        check("refuses degree 0", throws<std::invalid_argument>([&] { ParallelTopology::resolve(c, 8, 8, 43); }, "at least 1"));
        c.tensor_parallel = 3;
        check("refuses tp not dividing the artifact degree", throws<std::invalid_argument>([&] { ParallelTopology::resolve(c, 8, 8, 43); }, "does not divide"));
        c.tensor_parallel = 1; c.pipeline_parallel = 44;
        check("refuses pp above the layer count", throws<std::invalid_argument>([&] { ParallelTopology::resolve(c, 64, 1, 43); }, "exceeds"));
        c.pipeline_parallel = 2; c.device_ids = {0};
        check("refuses a short id list", throws<std::invalid_argument>([&] { ParallelTopology::resolve(c, 8, 1, 43); }, "entries"));
        c.device_ids = {0, 9};
        check("refuses an id beyond the visible devices", throws<std::invalid_argument>([&] { ParallelTopology::resolve(c, 8, 1, 43); }, "out of range"));
        c.device_ids = {1, 1};
        check("refuses a repeated id", throws<std::invalid_argument>([&] { ParallelTopology::resolve(c, 8, 1, 43); }, "more than once"));
        c.device_ids.clear(); c.pipeline_parallel = 1;
        check("refuses zero layers", throws<std::invalid_argument>([&] { ParallelTopology::resolve(c, 8, 1, 0); }, "no layers"));
        check("refuses artifact degree 0", throws<std::invalid_argument>([&] { ParallelTopology::resolve(c, 8, 0, 43); }));
        c.expert_parallel = 2; c.tensor_parallel = 2;
        check("refuses ep and tp together", throws<std::invalid_argument>([&] { ParallelTopology::resolve(c, 8, 8, 43); }, "share the ranks"));
    }
    {
        ParallelTopologyConfig c; c.expert_parallel = 8;
        const ParallelTopology t = ParallelTopology::resolve(c, 8, 1, 8);
        const ExpertShardDescriptor d = t.rank_slice(3, 256, 2048);
        check("expert-parallel slice: rank 3 of 8 owns experts 96..127", d.first_expert == 96 && d.expert_count == 32 && d.owns_expert(127) && !d.owns_expert(128) && d.intermediate_count == 2048);
        check("expert count must divide", throws<std::invalid_argument>([&] { t.rank_slice(0, 250, 2048); }));
        ParallelTopologyConfig c2; c2.tensor_parallel = 4;
        const ParallelTopology t2 = ParallelTopology::resolve(c2, 8, 8, 8);
        const ExpertShardDescriptor d2 = t2.rank_slice(2, 256, 2048);
        check("tensor-parallel slice: rank 2 of 4 owns intermediate 1024..1535", d2.first_intermediate == 1024 && d2.intermediate_count == 512 && d2.expert_count == 256);
    }
    {
        check("parser: plain list", parse_device_ids("0,1,3") == std::vector<int>({0, 1, 3}));
        check("parser: blanks ignored", parse_device_ids(" 2 ,\t5") == std::vector<int>({2, 5}));
        check("parser: empty text is the default", parse_device_ids("").empty());
        check("parser: doubled comma refused", throws<std::invalid_argument>([] { parse_device_ids("0,,1"); }, "empty entry"));
        check("parser: trailing comma refused", throws<std::invalid_argument>([] { parse_device_ids("0,1,"); }, "empty entry"));
        check("parser: non-numeric refused", throws<std::invalid_argument>([] { parse_device_ids("0,x"); }, "invalid device id"));
        check("parser: negative refused", throws<std::invalid_argument>([] { parse_device_ids("-1"); }, "non-negative"));
    }
    // ---- registry ----
    {
        ExpertRegistry reg(2, 8, 6);       // 16 experts, 6 slots: forces evictions
        bool ok = reg.invariants_hold() && reg.free_vram_slot_count() == 6;
        std::vector<ExpertRequestReservation> rs;
        for (uint32_t e = 0; e < 6; ++e) {
            rs.push_back(reg.reserve_request(0, e));
            ok &= rs.back().kind == ExpertRequestKind::COLD_MISS && rs.back().lease_acquired && reg.invariants_hold();
        }
        ok &= reg.free_vram_slot_count() == 0 && reg.pending_transfer_count() == 6 && !reg.expert_resident(0, 0);
        for (auto& r : rs) { reg.complete_request(r.operation_id); ok &= reg.invariants_hold(); }
        ok &= reg.expert_resident(0, 0) && reg.pending_transfer_count() == 0;
        check("cold misses take free slots, publish on completion", ok);

        const ExpertRequestReservation hit = reg.reserve_request(0, 2);
        check("resident expert: hot hit on its own slot with a lease", hit.kind == ExpertRequestKind::HOT_HIT && hit.vram_slot == rs[2].vram_slot && reg.lease_count(hit.global_expert_id) == 2);
        check("every slot leased: a new expert cannot be placed", throws<std::runtime_error>([&] { reg.reserve_request(1, 0); }, "no reclaimable"));
        for (auto& r : rs) reg.release_lease(r.global_expert_id);
        reg.release_lease(hit.global_expert_id);
        check("double release is a protocol error", throws<std::logic_error>([&] { reg.release_lease(hit.global_expert_id); }));
        // LRU: expert 2 was touched last, expert 0 is the coldest
        const ExpertRequestReservation miss = reg.reserve_request(1, 0);
        check("eviction takes the least recently used unleased expert", miss.kind == ExpertRequestKind::COLD_MISS && miss.evicted_global_id == 0 && miss.vram_slot == rs[0].vram_slot && !reg.expert_resident(0, 0) && reg.invariants_hold());
        const ExpertRequestReservation again = reg.reserve_request(1, 0);
        check("second request while the upload is pending", again.kind == ExpertRequestKind::PENDING && again.vram_slot == miss.vram_slot);
        reg.fail_request(miss.operation_id);
        check("failed upload rolls back: slot free again, audit clean", reg.free_vram_slot_count() == 1 && !reg.expert_resident(1, 0) && reg.invariants_hold());
        check("ids out of range", throws<std::out_of_range>([&] { reg.get_global_id(2, 0); }) && throws<std::out_of_range>([&] { reg.get_global_id(0, 8); }));
        const std::vector<int32_t> table = reg.layer_slot_table(0);
        check("layer slot table: absent experts are -1", table.size() == 8 && table[0] == -1 && table[1] == rs[1].vram_slot && table[7] == -1);

        ExpertRegistry full(2, 8, 16);
        full.populate_all_hot();
        bool all = full.invariants_hold();
        for (uint32_t l = 0; l < 2; ++l)
            for (uint32_t e = 0; e < 8; ++e) all &= full.reserve_request(l, e).kind == ExpertRequestKind::HOT_HIT;
        check("full residency: every request is a hot hit", all && full.cold_misses == 0 && full.hot_hits == 16 && full.invariants_hold());
    }
    // ---- expert container ----
    {
        const uint64_t bytes = 8192;
        std::vector<std::vector<uint8_t>> payloads(6, std::vector<uint8_t>(bytes));
        std::vector<const uint8_t*> ptrs;
        for (size_t i = 0; i < payloads.size(); ++i) {
            for (size_t j = 0; j < bytes; ++j) payloads[i][j] = static_cast<uint8_t>((i * 131 + j * 7) & 0xFF);
            ptrs.push_back(payloads[i].data());
        }
        const std::string idx = tmp + "/aeon_test.index", exp = tmp + "/aeon_test.experts";
        AeonExpertContainer::write(idx, exp, 2, 2, 3, bytes, ptrs);
        AeonExpertContainer c;
        c.open(idx, exp, 2, bytes);
        bool ok = c.format().num_layers == 2 && c.format().experts_per_layer == 3 && c.format().payload_bytes == bytes;
        for (uint32_t l = 0; l < 2; ++l)
            for (uint32_t e = 0; e < 3; ++e)
                ok &= std::memcmp(c.get_expert_data(l, e), payloads[l * 3 + e].data(), bytes) == 0 &&
                      c.get_expert_location(l, e).offset == (l * 3 + e) * bytes;
        check("container round trip: payloads byte-identical, offsets sector-aligned", ok);
        check("container: expert id out of range", throws<std::out_of_range>([&] { c.get_expert_data(2, 0); }));
        AeonExpertContainer bad;
        check("container: version mismatch refused", throws<std::runtime_error>([&] { bad.open(idx, exp, 3, bytes); }, "version"));
        check("container: payload size mismatch refused", throws<std::runtime_error>([&] { bad.open(idx, exp, 2, 4096); }, "payload size"));
        { std::ofstream t(idx, std::ios::binary | std::ios::trunc); t.write("AEON_EXPERTS", 12); }
        check("container: truncated index refused", throws<std::runtime_error>([&] { bad.open(idx, exp, 2, bytes); }, "too small"));
        { std::ofstream t(idx, std::ios::binary | std::ios::trunc); std::vector<char> z(64, 0); t.write(z.data(), 64); }
        check("container: bad magic refused", throws<std::runtime_error>([&] { bad.open(idx, exp, 2, bytes); }, "magic"));
        std::remove(idx.c_str()); std::remove(exp.c_str());
    }
    // ---- registry under random traffic against a shadow model ----
    {
        const uint32_t layers = 3, experts = 16, slots = 10;
        ExpertRegistry reg(layers, experts, slots);
        struct Shadow { int slot{-1}; bool published{false}; uint32_t leases{0}; uint64_t op{0}; };
        std::vector<Shadow> shadow(layers * experts);
        uint64_t state = 0x2545F4914F6CDD1Dull;
        auto rnd = [&](uint32_t n) { state ^= state << 13; state ^= state >> 7; state ^= state << 17; return static_cast<uint32_t>(state % n); };
        bool ok = true;
        uint64_t refusals = 0, evictions = 0;
        for (int step = 0; step < 20000 && ok; ++step) {
            const uint32_t gid = rnd(layers * experts);
            Shadow& sh = shadow[gid];
            switch (rnd(4)) {
                case 0: {   // request
                    try {
                        const ExpertRequestReservation r = reg.reserve_request(gid / experts, gid % experts);
                        if (sh.slot >= 0 && sh.published) ok &= r.kind == ExpertRequestKind::HOT_HIT && r.vram_slot == sh.slot;
                        else if (sh.slot >= 0) ok &= r.kind == ExpertRequestKind::PENDING && r.operation_id == sh.op;
                        else {
                            ok &= r.kind == ExpertRequestKind::COLD_MISS && r.vram_slot >= 0;
                            if (r.evicted_global_id >= 0) {
                                Shadow& v = shadow[r.evicted_global_id];
                                ok &= v.published && v.leases == 0 && v.slot == r.vram_slot;   // only idle residents lose slots
                                v = Shadow{};
                                ++evictions;
                            }
                            for (const Shadow& other : shadow) ok &= other.slot != r.vram_slot;      // the slot was really free
                            sh.slot = r.vram_slot; sh.published = false; sh.op = r.operation_id;
                        }
                        ++sh.leases;
                    } catch (const std::runtime_error&) {
                        // legal only when no slot is free and every published resident is leased
                        bool reclaimable = reg.free_vram_slot_count() > 0;
                        for (const Shadow& o : shadow) reclaimable |= o.published && o.leases == 0;
                        ok &= !reclaimable && sh.slot < 0;
                        ++refusals;
                    }
                    break;
                }
                case 1:     // an upload finishes
                    if (sh.slot >= 0 && !sh.published) { reg.complete_request(sh.op); sh.published = true; sh.op = 0; }
                    break;
                case 2: {   // a lease is returned: the next leased expert at or after the drawn id
                    uint32_t g = gid;
                    for (uint32_t i = 0; i < layers * experts && shadow[g].leases == 0; ++i) g = (g + 1) % (layers * experts);
                    if (shadow[g].leases > 0) { reg.release_lease(g); --shadow[g].leases; }
                    else ok &= throws<std::logic_error>([&] { reg.release_lease(gid); });
                    break;
                }
                case 3:     // an upload fails (rare)
                    if (sh.slot >= 0 && !sh.published && rnd(4) == 0) { reg.fail_request(sh.op); sh = Shadow{}; }
                    break;
            }
            ok &= reg.invariants_hold();
            if (step % 97 == 0)
                for (uint32_t g = 0; g < layers * experts; ++g)
                    ok &= reg.slot_of(g / experts, g % experts) == ((shadow[g].published) ? shadow[g].slot : -1) &&
                          reg.lease_count(g) == shadow[g].leases;
        }
        check("20000 random requests / completions / releases / failures agree with a shadow model", ok);
        std::printf("  (evictions %llu, refusals %llu)\n", static_cast<unsigned long long>(evictions),
                    static_cast<unsigned long long>(refusals));
        check("the traffic exercised evictions and full-pool refusals", evictions > 100 && refusals > 0);
    }
    // ---- shard-aware (version 3) expert container, dense container, loader ----
    {
        aeon_b200_moe_config cfg = moe_config_preset("baseline");
        cfg.hidden = 256; cfg.intermediate = 2048; cfg.experts = 32; cfg.top_k = 4;
        const uint32_t D = 8, layers = 1;
        const size_t H = cfg.hidden, I = cfg.intermediate, G = cfg.group_size;
        struct Source { std::vector<uint32_t> w1p, w2p, w3p; std::vector<uint16_t> w1s, w2s, w3s; };
        auto make_source = [&](uint32_t seed) {
            Source s;
            uint64_t state = 0x9E3779B97F4A7C15ull * (seed + 1);
            auto next = [&] { state ^= state << 13; state ^= state >> 7; state ^= state << 17; return state; };
            s.w1p.resize(I * H / 8); s.w3p.resize(I * H / 8); s.w2p.resize(H * I / 8);
            s.w1s.resize(I * H / G); s.w3s.resize(I * H / G); s.w2s.resize(H * I / G);
            for (auto* v : {&s.w1p, &s.w2p, &s.w3p}) for (auto& w : *v) w = static_cast<uint32_t>(next());
            for (auto* v : {&s.w1s, &s.w2s, &s.w3s}) for (auto& w : *v) w = static_cast<uint16_t>(0x2000 + next() % 0x800);
            return s;
        };
        const ExpertFormatDescriptor f3 = make_swizzled_expert_format(cfg, layers, D);
        check("v3 format: 8 shards, shard_bytes x 8 = payload, version 3",
              f3.version == 3 && f3.shard_count == D && f3.shard_bytes * D == f3.payload_bytes);
        std::vector<std::vector<uint8_t>> payloads(cfg.experts, std::vector<uint8_t>(f3.payload_bytes));
        std::vector<const uint8_t*> ptrs;
        for (int e = 0; e < cfg.experts; ++e) {
            const Source s = make_source(e);
            check_status(aeon_b200_pack_expert_shards(&cfg, D, s.w1p.data(), s.w1s.data(), s.w2p.data(), s.w2s.data(),
                                                      s.w3p.data(), s.w3s.data(), payloads[e].data()));
            ptrs.push_back(payloads[e].data());
        }
        const std::string dir = tmp;
        const std::string idx = dir + "/model_experts_swizzled.index", exp = dir + "/model_experts_swizzled.aeon";
        AeonExpertContainer::write(idx, exp, 3, layers, cfg.experts, f3.payload_bytes, ptrs, D);
        AeonExpertContainer c;
        c.open(idx, exp, 0, 0);
        check("v3 container: header fields read back", c.format().version == 3 && c.format().shard_count == D &&
                                                          c.format().shard_bytes == f3.shard_bytes);
        bool tiles = true;
        for (uint32_t tp : {1u, 2u, 4u, 8u}) {
            const auto whole = c.get_expert_location(0, 5);
            uint64_t cursor = whole.offset;
            for (uint32_t r = 0; r < tp; ++r) {
                const auto sl = c.rank_slice(0, 5, tp, r);
                tiles &= sl.offset == cursor && sl.offset % 4096 == 0 && sl.length == whole.length / tp;
                cursor += sl.length;
            }
            tiles &= cursor == whole.offset + whole.length;
        }
        check("rank slices: contiguous, sector-aligned, disjoint, cover the payload", tiles);
        check("rank_slice: tp that does not divide the shard count refused",
              throws<std::invalid_argument>([&] { c.rank_slice(0, 5, 3, 0); }, "does not divide"));
        check("rank_slice: rank out of range", throws<std::out_of_range>([&] { c.rank_slice(0, 5, 2, 2); }));
        {
            // rank 1 of tp 2: its merged payload equals the payload packed from its half of the source
            const Source s = make_source(5);
            aeon_b200_moe_config half = cfg; half.intermediate = cfg.intermediate / 2;
            const size_t Ih = half.intermediate;
            Source h;
            h.w1p.assign(s.w1p.begin() + Ih * H / 8, s.w1p.end()); h.w1s.assign(s.w1s.begin() + Ih * H / G, s.w1s.end());
            h.w3p.assign(s.w3p.begin() + Ih * H / 8, s.w3p.end()); h.w3s.assign(s.w3s.begin() + Ih * H / G, s.w3s.end());
            for (size_t r = 0; r < H; ++r) {
                h.w2p.insert(h.w2p.end(), s.w2p.begin() + r * I / 8 + Ih / 8, s.w2p.begin() + (r + 1) * I / 8);
                h.w2s.insert(h.w2s.end(), s.w2s.begin() + r * I / G + Ih / G, s.w2s.begin() + (r + 1) * I / G);
            }
            aeon_b200_expert_layout lay{};
            check_status(aeon_b200_expert_layout_of(&half, &lay));
            std::vector<uint8_t> direct(lay.payload_bytes);
            check_status(aeon_b200_pack_expert_shards(&half, 1, h.w1p.data(), h.w1s.data(), h.w2p.data(), h.w2s.data(),
                                                      h.w3p.data(), h.w3s.data(), direct.data()));
            check("read_rank_payload(tp 2, rank 1) = payload packed from that half of the source",
                  c.read_rank_payload(cfg, 0, 5, 2, 1) == direct);
        }
        AeonExpertContainer v2only;
        check("v3 index refused when version 2 is demanded",
              throws<std::runtime_error>([&] { v2only.open(idx, exp, 2, 0); }, "version"));
        check("write: shards need version 3",
              throws<std::invalid_argument>([&] { AeonExpertContainer::write(idx + ".x", exp + ".x", 2, layers, cfg.experts, f3.payload_bytes, ptrs, D); }));
        std::remove((idx + ".x").c_str()); std::remove((exp + ".x").c_str());

        // dense container written by hand: header, JSON directory, 4 KiB-aligned payload
        const std::string dense_path = dir + "/model_dense.aeon";
        std::vector<uint16_t> gate(static_cast<size_t>(cfg.experts) * H);
        for (size_t i = 0; i < gate.size(); ++i) gate[i] = static_cast<uint16_t>(i * 7 + 1);
        std::vector<float> bias(cfg.experts);
        for (size_t i = 0; i < bias.size(); ++i) bias[i] = 0.25f * static_cast<float>(i);
        auto write_dense = [&](const std::string& directory, uint32_t version, uint32_t count) {
            std::ofstream out(dense_path, std::ios::binary | std::ios::trunc);
            const uint64_t dir_len = directory.size();
            out.write("AEON_DENSE\0\0", 12);
            out.write(reinterpret_cast<const char*>(&version), 4);
            out.write(reinterpret_cast<const char*>(&count), 4);
            out.write(reinterpret_cast<const char*>(&dir_len), 8);
            out.write(directory.data(), static_cast<std::streamsize>(directory.size()));
            const size_t pre = 28 + directory.size();
            std::vector<char> pad((4096 - pre % 4096) % 4096, 0);
            out.write(pad.data(), static_cast<std::streamsize>(pad.size()));
            out.write(reinterpret_cast<const char*>(gate.data()), static_cast<std::streamsize>(gate.size() * 2));
            out.write(reinterpret_cast<const char*>(bias.data()), static_cast<std::streamsize>(bias.size() * 4));
        };
        const std::string directory =
            "[\n  {\"name\": \"layers.0.ffn.gate.weight\", \"offset\": 0, \"size\": " + std::to_string(gate.size() * 2) +
            ", \"dtype\": \"BF16\", \"shape\": [" + std::to_string(cfg.experts) + ", " + std::to_string(H) + "]},\n"
            "  {\"name\": \"layers.0.ffn.gate.bias\", \"offset\": " + std::to_string(gate.size() * 2) +
            ", \"size\": " + std::to_string(bias.size() * 4) + ", \"dtype\": \"F32\", \"shape\": [" +
            std::to_string(cfg.experts) + "]}\n]";
        write_dense(directory, 1, 2);
        AeonModelLoader loader;
        loader.open_model(dir);
        const LoadedTensor& g = loader.get_tensor("layers.0.ffn.gate.weight");
        const LoadedTensor& b = loader.get_tensor("layers.0.ffn.gate.bias");
        check("loader: dense tensors by name (bytes, dtype, shape)",
              g.byte_size == static_cast<int64_t>(gate.size() * 2) && g.dtype == "BF16" && g.shape.size() == 2 &&
                  g.shape[0] == cfg.experts && std::memcmp(g.data, gate.data(), gate.size() * 2) == 0 &&
                  b.dtype == "F32" && std::memcmp(b.data, bias.data(), bias.size() * 4) == 0 &&
                  (reinterpret_cast<uintptr_t>(g.data) - reinterpret_cast<uintptr_t>(loader.dense().get_tensor("layers.0.ffn.gate.weight").data)) == 0);
        check("loader: experts, max tensor-parallel degree and rank slices through one object",
              loader.max_tensor_parallel() == D && loader.expert_format().payload_bytes == f3.payload_bytes &&
                  std::memcmp(loader.get_expert_data(0, 31), payloads[31].data(), f3.payload_bytes) == 0 &&
                  loader.rank_slice(0, 31, 8, 7).offset == loader.get_expert_location(0, 31).offset + 7 * f3.shard_bytes);
        check("loader: missing tensor", !loader.has_tensor("layers.0.ffn.gate.tid2eid") &&
                                             throws<std::runtime_error>([&] { loader.get_tensor("layers.0.ffn.gate.tid2eid"); }, "Missing"));
        AeonDenseContainer bad;
        write_dense(directory, 2, 2);
        check("dense: version mismatch refused", throws<std::runtime_error>([&] { bad.open(dense_path); }, "version"));
        write_dense(directory, 1, 3);
        check("dense: count mismatch refused", throws<std::runtime_error>([&] { bad.open(dense_path); }, "count"));
        write_dense("[{\"name\": \"a\", \"offset\": 0, \"size\": 99999999, \"dtype\": \"U8\", \"shape\": [1]}]", 1, 1);
        check("dense: range beyond the payload refused", throws<std::runtime_error>([&] { bad.open(dense_path); }, "exceeds payload"));
        write_dense("[{\"name\": \"a\", \"offset\": 0, \"size\": 8, \"dtype\": \"U8\"}]", 1, 1);
        check("dense: entry without a shape refused", throws<std::runtime_error>([&] { bad.open(dense_path); }, "Malformed"));
        write_dense(directory + "x", 1, 2);
        check("dense: text after the directory refused", throws<std::runtime_error>([&] { bad.open(dense_path); }, "Malformed"));
        {
            // damaged directories: every outcome is either a clean open or a runtime_error
            uint64_t state = 0x9E3779B97F4A7C15ull;
            auto rnd = [&](uint32_t n) { state ^= state << 13; state ^= state >> 7; state ^= state << 17; return static_cast<uint32_t>(state % n); };
            bool contained = true;
            int opened = 0, refused = 0;
            for (int trial = 0; trial < 400 && contained; ++trial) {
                std::string d = directory;
                const int edits = 1 + static_cast<int>(rnd(3));
                for (int e = 0; e < edits; ++e) {
                    const size_t at = rnd(static_cast<uint32_t>(d.size()));
                    switch (rnd(3)) {
                        case 0: d[at] = static_cast<char>(32 + rnd(95)); break;
                        case 1: d.erase(at, 1 + rnd(4)); break;
                        default: d.insert(at, 1, "[]{}\",:-0123456789"[rnd(19)]); break;
                    }
                    if (d.empty()) d = "[";
                }
                write_dense(d, 1, 2);
                try { bad.open(dense_path); ++opened; }
                catch (const std::runtime_error&) { ++refused; }
                catch (...) { contained = false; }
            }
            std::printf("  (damaged directories: %d opened, %d refused)\n", opened, refused);
            check("dense: 400 damaged directories are opened or refused, nothing else", contained && refused > 100);
        }
        std::remove(idx.c_str()); std::remove(exp.c_str()); std::remove(dense_path.c_str());
    }
    // ---- a model directory written by the Python converter (argv[2]), read by this loader ----
    if (argc > 2) {
        const std::string model_dir = argv[2];
        std::ifstream expect_file(model_dir + "/expected.txt");
        uint64_t shard_count = 0, payload_bytes = 0, expert_hash = 0, gate_hash = 0, slice_offset = 0;
        expect_file >> shard_count >> payload_bytes >> expert_hash >> gate_hash >> slice_offset;
        auto fnv = [](const uint8_t* p, size_t n) {
            uint64_t h = 0xcbf29ce484222325ull;
            for (size_t i = 0; i < n; ++i) { h ^= p[i]; h *= 0x100000001b3ull; }
            return h;
        };
        AeonModelLoader loader;
        loader.open_model(model_dir);
        check("python-written artifact: header fields", loader.max_tensor_parallel() == shard_count &&
                                                          loader.expert_format().payload_bytes == payload_bytes);
        check("python-written artifact: expert (0,3) bytes", fnv(loader.get_expert_data(0, 3), payload_bytes) == expert_hash);
        const LoadedTensor& g = loader.get_tensor("layers.0.ffn.gate.weight");
        check("python-written artifact: gate tensor bytes", fnv(g.data, static_cast<size_t>(g.byte_size)) == gate_hash);
        check("python-written artifact: rank slice (tp 2, rank 1) offset", loader.rank_slice(0, 3, 2, 1).offset == slice_offset);

        // the directory carries a manifest: the loader went through it (backend resolved and
        // checked against the artifact first, loaded identity against the manifest last)
        const std::string manifest_path = model_dir + "/model_manifest.json";
        const AeonModelManifest manifest = AeonModelManifest::load_from_json(manifest_path);
        check("manifest: identity, backend, catalog and shard degree",
              manifest.weight_backend == "swizzled_w4a16" && !manifest.model_family.empty() &&
                  !manifest.architecture.empty() && manifest.num_layers == 1 && manifest.experts_per_layer == 32 &&
                  manifest.max_tensor_parallel == shard_count &&
                  manifest.artifact.expected_expert_payload_bytes == payload_bytes &&
                  manifest.dense_file_bytes == loader.dense().file_size());
        std::ifstream in(manifest_path);
        std::stringstream whole;
        whole << in.rdbuf();
        const std::string good = whole.str();
        auto with = [&](const std::string& from, const std::string& to) {
            std::string text = good;
            const size_t at = text.find(from);
            if (at == std::string::npos) return false;
            text.replace(at, from.size(), to);
            std::ofstream(manifest_path, std::ios::trunc) << text;
            return true;
        };
        AeonModelLoader refused;
        check("manifest: an unknown weight backend is refused before any file is opened",
              with("\"weight_backend\": \"swizzled_w4a16\"", "\"weight_backend\": \"dense_fp8\"") &&
                  throws<std::invalid_argument>([&] { refused.open_model(model_dir); }, "weight backend"));
        check("manifest: a payload size the artifact does not have is refused",
              with("\"expert_payload_bytes\": " + std::to_string(payload_bytes),
                   "\"expert_payload_bytes\": " + std::to_string(payload_bytes + 4096)) &&
                  throws<std::runtime_error>([&] { refused.open_model(model_dir); }));
        check("manifest: a dense size that is not the file's is refused",
              with("\"dense_file_bytes\": " + std::to_string(manifest.dense_file_bytes),
                   "\"dense_file_bytes\": " + std::to_string(manifest.dense_file_bytes + 1)) &&
                  throws<std::runtime_error>([&] { refused.open_model(model_dir); }, "dense file size"));
        check("manifest: a missing key is refused",
              with("\"model_family\"", "\"model_clan\"") &&
                  throws<std::invalid_argument>([&] { refused.open_model(model_dir); }, "model_family"));
        std::ofstream(manifest_path, std::ios::trunc) << good;
        refused.open_model(model_dir);
        check("manifest: restored, the directory opens again", refused.max_tensor_parallel() == shard_count);
    }
    // ---- backend registry ----
    {
        const aeon_b200_moe_config ref = moe_config_preset("ref_dsv4");
        const ExpertFormatDescriptor f = make_swizzled_expert_format(ref, 43);
        const ExpertBackendDescriptor& by_name = ExpertBackendRegistry::resolve("swizzled_w4a16");
        check("backend registry: by name, by kind, with a format",
              by_name.supports_fused_moe_experts && &ExpertBackendRegistry::resolve(ExpertFormatKind::SWIZZLED_W4A16) == &by_name &&
                  &ExpertBackendRegistry::resolve("swizzled_w4a16", f) == &by_name && &ExpertBackendRegistry::resolve(f) == &by_name);
        check("backend registry: unknown name refused",
              throws<std::invalid_argument>([] { ExpertBackendRegistry::resolve("gguf_q4"); }, "unsupported weight backend"));
        check("backend registry: unknown format kind refused",
              throws<std::invalid_argument>([] { ExpertBackendRegistry::resolve(ExpertFormatKind::OPAQUE); }, "no backend"));
        const ExpertBackendDescriptor bound = ExpertBackendRegistry::for_config(ref);
        ExpertFormatDescriptor other = f;
        other.payload_bytes += 4096;
        check("backend bound to a layer shape refuses an artifact of another payload size",
              bound.payload_bytes == 14155776u && throws<std::runtime_error>([&] { bound.validate_format(other); }, "incompatible"));
        ExpertFormatDescriptor old_version = f;
        old_version.version = 1;
        check("backend refuses a format version it does not read",
              throws<std::runtime_error>([&] { by_name.validate_format(old_version); }, "incompatible"));
    }
    // ---- format / presets through the C ABI ----
    {
        const aeon_b200_moe_config ref = moe_config_preset("ref_dsv4");
        const ExpertFormatDescriptor f = make_swizzled_expert_format(ref, 43);
        check("reference preset payload = 14,155,776 bytes", f.payload_bytes == 14155776u && f.total_experts() == 43u * 256u);
        check("unknown preset -> invalid_argument", throws<std::invalid_argument>([] { moe_config_preset("x"); }));
        ExpertFormatDescriptor z = f; z.payload_bytes = 100;
        check("payload must be sector-aligned", throws<std::invalid_argument>([&] { z.validate_payload(); }));
    }
    std::printf("[host shim] %s (%d failures)\n", g_fail == 0 ? "ALL PASS" : "FAILED", g_fail);
    return g_fail == 0 ? 0 : 1;
}
