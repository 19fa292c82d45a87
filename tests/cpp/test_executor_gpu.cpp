// GPU check of the C++ executor (needs a B200): V4TieredExpertExecutor over a pool smaller
// than the catalog (8 slots for 32 experts, so misses, uploads and evictions all happen) must
// give results bit-identical to the direct C-ABI call on a fully resident pool — the shape of
// the reference's tests/test_v4_expert_executor.cpp:12-75 (tiered executor vs direct-payload
// executor, 8-slot pool to force the drain path, wrong-expert probe must differ). The token
// loop is the reference layer body's own sequence (src/architecture/deepseek_v4/layer/
// v4_layer_body_moe.hpp:160-192,285-312): router ids read back to the host, on_routing_ready,
// shared expert (here: a cleared accumulator), accumulate_routed(layer, pos, x, weights, accum),
// on_routed_consumed. The same is then run with the miss uploads on their own stream
// (DeviceContext / DeviceStreams) and must still be bit-identical.
#include "aeon_b200_host.hpp"

#include <cuda_runtime.h>

#include <cstdio>
#include <functional>
#include <random>

using namespace aeon::core;

static int g_fail = 0;
static void check(const char* label, bool ok) {
    std::printf("  %-74s %s\n", label, ok ? "PASS" : "FAIL");
    if (!ok) ++g_fail;
}
template <class E>
static bool throws(const std::function<void()>& f) {
    try { f(); } catch (const E&) { return true; } catch (...) { return false; }
    return false;
}
#define CUDA_OK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { std::printf("CUDA error %s at %d\n", cudaGetErrorString(e_), __LINE__); return 2; } } while (0)

static uint16_t f2h(float f) {          // small positive normal floats only
    uint32_t u; std::memcpy(&u, &f, 4);
    const uint32_t e = ((u >> 23) & 0xFF) - 127 + 15, m = (u >> 13) & 0x3FF;
    return static_cast<uint16_t>((e << 10) | m);
}

int main(int argc, char** argv) {
    const std::string tmp = argc > 1 ? argv[1] : "/tmp";
    std::printf("[executor on GPU]\n");
    aeon_b200_moe_config cfg = moe_config_preset("ref_dsv4");
    cfg.experts = 32;
    const int E = cfg.experts, K = cfg.top_k, H = cfg.hidden;
    const ExpertFormatDescriptor format = make_swizzled_expert_format(cfg, 1);
    aeon_b200_expert_layout lay{};
    check_status(aeon_b200_expert_layout_of(&cfg, &lay));

    // synthetic payloads (random nibbles, scales 2^-8 * (1 + i % 29) as the reference's fixtures)
    std::vector<std::vector<uint8_t>> payloads(E, std::vector<uint8_t>(format.payload_bytes, 0));
    std::mt19937 rng(12345);
    for (int e = 0; e < E; ++e) {
        uint32_t* w = reinterpret_cast<uint32_t*>(payloads[e].data());
        for (size_t i = 0; i < format.payload_bytes / 4; ++i) w[i] = rng();
        const uint64_t scale_regions[3][2] = {{lay.w1_scale_offset, lay.w13_scale_bytes},
                                              {lay.w2_scale_offset, lay.w2_scale_bytes},
                                              {lay.w3_scale_offset, lay.w13_scale_bytes}};
        for (auto& reg : scale_regions) {
            uint16_t* s = reinterpret_cast<uint16_t*>(payloads[e].data() + reg[0]);
            for (size_t i = 0; i < reg[1] / 2; ++i) s[i] = f2h(std::ldexp(1.0f + static_cast<float>((i + e) % 29), -12));
        }
    }
    std::vector<const uint8_t*> ptrs;
    for (auto& p : payloads) ptrs.push_back(p.data());
    const std::string idx = tmp + "/exec.index", exp = tmp + "/exec.experts";
    AeonExpertContainer::write(idx, exp, 2, 1, E, format.payload_bytes, ptrs);
    AeonExpertContainer container;
    container.open(idx, exp, 2, format.payload_bytes);

    select_device(0, false);
    check("a device index that is not there is a named error",
          throws<std::runtime_error>([&] { select_device(4096, false); }));
    enable_peer_access({0}, false);                   // one device: nothing to enable, nothing to refuse
    DeviceContext device_context = DeviceContext::create(0);
    check("a device context carries four distinct streams",
          device_context.streams.compute && device_context.streams.sdma && device_context.streams.sdma_cold &&
              device_context.streams.demotion && device_context.streams.compute != device_context.streams.sdma_cold);
    cudaStream_t stream;
    CUDA_OK(cudaStreamCreate(&stream));
    UnifiedVRAMExpertPool small_pool(8, cfg, format), full_pool(E, cfg, format);
    for (int e = 0; e < E; ++e) full_pool.upload_from_host_expert(e, payloads[e].data(), stream);
    ExpertRegistry registry(1, E, 8);
    V4TieredExpertExecutor exec(cfg, 0, 8, small_pool, registry, &container, stream);

    // direct path: its own context, identity slot table
    aeon_b200_ctx* direct = nullptr;
    check_status(aeon_b200_ctx_create(&cfg, 0, 8, &direct));
    std::vector<int32_t> identity(E);
    for (int e = 0; e < E; ++e) identity[e] = e;
    int32_t* d_identity; CUDA_OK(cudaMalloc(&d_identity, E * 4));
    CUDA_OK(cudaMemcpy(d_identity, identity.data(), E * 4, cudaMemcpyHostToDevice));

    const int T = 3;
    std::vector<uint16_t> x(T * H);
    for (auto& v : x) v = f2h(0.25f + static_cast<float>(rng() % 1000) / 500.0f) | ((rng() & 1) << 15);
    std::vector<int32_t> ids = {0, 1, 2, 3, 4, 5,   4, 5, 6, 7, 8, 9,   31, 30, 9, 8, 1, 0};
    std::vector<float> w(T * K);
    for (auto& v : w) v = 0.05f + static_cast<float>(rng() % 100) / 400.0f;
    uint16_t* d_x; int32_t* d_ids; float *d_w, *d_a, *d_b;
    CUDA_OK(cudaMalloc(&d_x, x.size() * 2)); CUDA_OK(cudaMalloc(&d_ids, ids.size() * 4));
    CUDA_OK(cudaMalloc(&d_w, w.size() * 4)); CUDA_OK(cudaMalloc(&d_a, T * H * 4)); CUDA_OK(cudaMalloc(&d_b, T * H * 4));
    CUDA_OK(cudaMemcpy(d_x, x.data(), x.size() * 2, cudaMemcpyHostToDevice));
    CUDA_OK(cudaMemcpy(d_ids, ids.data(), ids.size() * 4, cudaMemcpyHostToDevice));
    CUDA_OK(cudaMemcpy(d_w, w.data(), w.size() * 4, cudaMemcpyHostToDevice));
    std::vector<float> a(T * H), b(T * H);
    auto fetch = [&](float* d, std::vector<float>& h) {
        cudaStreamSynchronize(stream);
        cudaMemcpy(h.data(), d, h.size() * 4, cudaMemcpyDeviceToHost);
    };

    check("accumulate before any dispatch is a protocol error",
          throws<std::logic_error>([&] { exec.accumulate_routed(0, 0, d_x, d_ids, d_w, d_a); }));
    check("a short id list is refused",
          throws<std::invalid_argument>([&] { exec.on_routing_ready(0, 0, {1, 2, 3}, {1.f, 1.f, 1.f}); }));

    // token by token through the tiered executor (misses -> uploads, then evictions)
    bool identical = true;
    for (int t = 0; t < T; ++t) {
        std::vector<int32_t> row(ids.begin() + t * K, ids.begin() + (t + 1) * K);
        std::vector<float> wrow(w.begin() + t * K, w.begin() + (t + 1) * K);
        exec.on_routing_ready(0, t, row, wrow);
        CUDA_OK(cudaMemsetAsync(d_a + t * H, 0, H * 4, stream));
        exec.accumulate_routed(0, t, d_x + t * H, d_w + t * K, d_a + t * H);     // ids: the announced ones
        exec.on_routed_consumed(0, t);
        exec.check_device();
        exec.release_leases();       // token boundary
        identical &= registry.invariants_hold();
    }
    CUDA_OK(cudaMemsetAsync(d_b, 0, T * H * 4, stream));
    check_status(aeon_b200_moe_decode(direct, full_pool.d_experts, d_identity, d_x, H, d_ids, d_w, T, d_b, H, 0, stream));
    check_status(aeon_b200_ctx_check(direct, stream));
    fetch(d_a, a); fetch(d_b, b);
    // the per-token calls sum one token each; the direct call sums three tokens per expert
    // tile, but every output element is one token's own fixed-order sum: bytes must agree
    identical &= std::memcmp(a.data(), b.data(), a.size() * 4) == 0;
    bool nonzero = false;
    for (float v : b) nonzero |= (v != 0.0f);
    check("tiered executor (8-slot pool) == direct call (resident pool), bit for bit", identical && nonzero);
    check("the small pool really evicted", registry.evictions >= 4 && registry.cold_misses >= 12 && registry.hot_hits >= 2);
    check("leases are back to zero at the token boundary", exec.outstanding_leases() == 0);

    // the same tokens with the miss uploads on their own stream, through pinned staging
    {
        ExpertRegistry async_registry(1, E, 8);
        UnifiedVRAMExpertPool async_pool(8, cfg, format);
        V4TieredExpertExecutor async_exec(cfg, 0, 8, async_pool, async_registry, &container, device_context.streams);
        cudaStream_t cs = static_cast<cudaStream_t>(device_context.streams.compute);
        CUDA_OK(cudaStreamSynchronize(stream));
        bool ok = true;
        for (int round = 0; round < 2; ++round)           // second round: slots evicted in the first come back
            for (int t = 0; t < T; ++t) {
                std::vector<int32_t> row(ids.begin() + t * K, ids.begin() + (t + 1) * K);
                std::vector<float> wrow(w.begin() + t * K, w.begin() + (t + 1) * K);
                async_exec.on_routing_ready(0, t, row, wrow);
                CUDA_OK(cudaMemsetAsync(d_a + t * H, 0, H * 4, cs));
                async_exec.accumulate_routed(0, t, d_x + t * H, d_w + t * K, d_a + t * H);
                async_exec.on_routed_consumed(0, t);
                async_exec.release_leases();
                ok &= async_registry.invariants_hold();
            }
        async_exec.check_device();
        CUDA_OK(cudaStreamSynchronize(cs));
        CUDA_OK(cudaMemcpy(a.data(), d_a, a.size() * 4, cudaMemcpyDeviceToHost));
        check("asynchronous supply (upload stream + pinned staging) == direct call, bit for bit",
              ok && std::memcmp(a.data(), b.data(), a.size() * 4) == 0);
        check("it uploaded through the staging ring more often than the ring is long",
              async_exec.uploads() > V4TieredExpertExecutor::kStagingBuffers && async_registry.evictions >= 4);
    }

    // chunk-wide dispatch: the layer's union is requested once
    registry.init(1, E, 16);
    UnifiedVRAMExpertPool mid_pool(16, cfg, format);
    V4TieredExpertExecutor batch_exec(cfg, 0, 8, mid_pool, registry, &container, stream);
    std::vector<std::vector<int32_t>> bids;
    std::vector<std::vector<float>> bw;
    for (int t = 0; t < T; ++t) {
        bids.emplace_back(ids.begin() + t * K, ids.begin() + (t + 1) * K);
        bw.emplace_back(w.begin() + t * K, w.begin() + (t + 1) * K);
    }
    batch_exec.on_routing_ready_batch(0, 10, bids, bw);
    CUDA_OK(cudaMemsetAsync(d_a, 0, T * H * 4, stream));
    batch_exec.accumulate_routed_batch(0, 10, T, d_x, H, d_ids, K, d_w, K, d_a, H);
    batch_exec.check_device();
    fetch(d_a, a);
    check("chunk-wide dispatch == direct call, bit for bit", std::memcmp(a.data(), b.data(), a.size() * 4) == 0);
    CUDA_OK(cudaMemsetAsync(d_a, 0, T * H * 4, stream));
    batch_exec.accumulate_routed_batch(0, 10, T, d_x, H, nullptr, 0, d_w, K, d_a, H);   // the announced ids
    batch_exec.check_device();
    fetch(d_a, a);
    check("chunk-wide consume with the announced ids == direct call, bit for bit",
          std::memcmp(a.data(), b.data(), a.size() * 4) == 0);
    {
        // the seam's default bodies: an executor that only implements the per-token form
        struct PerToken final : V4RoutedExpertExecutor {
            V4TieredExpertExecutor& inner;
            int calls{0};
            explicit PerToken(V4TieredExpertExecutor& e) : inner(e) {}
            void accumulate_routed(uint32_t layer, uint32_t pos, const act16* x, const float* weights,
                                   float* accum) override {
                ++calls;
                inner.accumulate_routed(layer, pos, x, weights, accum);
            }
        } per_token(batch_exec);
        CUDA_OK(cudaMemsetAsync(d_a, 0, T * H * 4, stream));
        V4RoutedExpertExecutor& seam = per_token;
        seam.accumulate_routed_batch(0, 10, T, d_x, H, nullptr, 0, d_w, K, d_a, H);
        batch_exec.check_device();
        fetch(d_a, a);
        check("the default chunk body is the per-token sequence", per_token.calls == T &&
                                                                      std::memcmp(a.data(), b.data(), a.size() * 4) == 0);
    }
    check("the chunk issued one deduplicated set (18 draws -> 12 distinct experts)",
          batch_exec.batch_draws() == 18 && batch_exec.batch_distinct() == 12 && batch_exec.last_dispatch_tokens() == 3);
    check("a mismatched batch consume is a protocol error",
          throws<std::logic_error>([&] { batch_exec.accumulate_routed_batch(0, 11, T, d_x, H, d_ids, K, d_w, K, d_a, H); }));
    batch_exec.release_leases();

    // wrong-expert probe: one different id must change the result
    std::vector<int32_t> wrong = ids;
    wrong[0] = 17;
    CUDA_OK(cudaMemcpy(d_ids, wrong.data(), wrong.size() * 4, cudaMemcpyHostToDevice));
    CUDA_OK(cudaMemsetAsync(d_a, 0, T * H * 4, stream));
    check_status(aeon_b200_moe_decode(direct, full_pool.d_experts, d_identity, d_x, H, d_ids, d_w, T, d_a, H, 0, stream));
    fetch(d_a, a);
    check("wrong-expert probe goes red", std::memcmp(a.data(), b.data(), H * 4) != 0 &&
                                             std::memcmp(a.data() + H, b.data() + H, 2 * H * 4) == 0);

    device_context.destroy();
    aeon_b200_ctx_destroy(direct);
    std::remove(idx.c_str()); std::remove(exp.c_str());
    std::printf("[executor on GPU] %s (%d failures)\n", g_fail == 0 ? "ALL PASS" : "FAILED", g_fail);
    return g_fail == 0 ? 0 : 1;
}
