// Host-only checks of the C++ layer (no GPU): the topology resolver and id parser against
// the cases of the reference's tests/test_parallel_topology.cpp:83-256 (stage-major mapping,
// 43-layer splits, refusals, parser), the registry's reservation / lease / eviction state
// machine with the invariant audit after every step
// (tests/test_expert_registry_warm_state.cpp), and the expert container round trip
// (index header + entries, the loader contract of aeon_loader.hpp:345-405).
#include "aeon_b200_host.hpp"

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
