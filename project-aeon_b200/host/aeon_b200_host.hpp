// C++ host layer over the C ABI (include/aeon_b200.h), keeping the reference's class and
// function names for the routed-expert path so engine code compiles against it with
// hipStream_t -> cudaStream_t as the only type change. Header-only; link libaeon_b200.so.
//
//   ParallelTopologyConfig / LayerRange / parse_device_ids / ParallelTopology
//                               src/infrastructure/parallel/parallel_topology.hpp:34-211
//   ExpertShardDescriptor       the shard-aware fields the reference only plans
//                               (plans-and-docs/.../MULTI_GPU_EXECUTION_PLAN.md:151-181) and its
//                               shard-equivalence tests exercise
//                               (tests/test_expert_shard_equivalence.cpp:286-340)
//   ExpertFormatDescriptor      src/infrastructure/expert/storage/expert_format.hpp:10-60
//   UnifiedVRAMExpertPool       src/backend/swizzled_w4a16/core/vram_expert_pool.hpp:22-82 over
//                               src/infrastructure/expert/storage/expert_payload_pool.hpp:16-131
//   ExpertRegistry              src/infrastructure/expert/residency/expert_registry.hpp:26-1064
//                               (the HBM-resident subset: hot hits, cold misses into free or
//                               least-recently-used unleased slots, leases, invariant audit)
//   AeonModelLoader             src/infrastructure/artifact/aeon_loader.hpp:41-166: AeonExpertContainer
//                               (the expert index + payload file, :145-166,318-441, in version 2
//                               and in the planned shard-aware version 3 with rank_slice) and
//                               AeonDenseContainer (the dense file, :243-316,441-479)
//   V4RoutedExpertExecutor      src/architecture/deepseek_v4/layer/v4_layer_body_moe.hpp:32-112
//   V4TieredExpertExecutor      src/architecture/deepseek_v4/moe/v4_expert_executor.hpp:178-634
//   dispatch_router             src/architecture/deepseek_v4/layer/v4_layer_body_moe.hpp:124-159
//   dispatch_expert_permutation src/platform/ops/expert_permutation.hpp:130-175
//   select_device / DeviceScope src/platform/device.hpp:29-90
//   DeviceStreams               src/infrastructure/device_streams.hpp:32-74
//   DeviceContext               src/infrastructure/parallel/device_context.hpp:23-49
//   enable_peer_access          src/infrastructure/parallel/peer_access.hpp:29-50
//   ExpertBackendRegistry       src/infrastructure/backend_registry/expert_backend.hpp:14-79
//   AeonModelManifest           src/infrastructure/artifact/model_manifest.hpp:102-209
//   ParallelGroup               the communicator the reference plans as TensorParallelGroup
//                               (plans-and-docs/execution/active/MULTI_GPU_EXECUTION_PLAN.md:189-235)
#pragma once

#include "aeon_b200.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <array>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <functional>
#include <iostream>
#include <list>
#include <sstream>
#include <stdexcept>
#include <string>
#include <string_view>
#include <unordered_map>
#include <vector>

namespace aeon::core {

// ---------------------------------------------------------------------------------------------
// Status -> the exception kinds the reference throws (shape/argument: invalid_argument;
// protocol: logic_error; ids: out_of_range; device: runtime_error, as CHECK_HIP does,
// src/infrastructure/hip_check.hpp:20-27).
// ---------------------------------------------------------------------------------------------
inline void check_status(int status) {
    if (status == AEON_B200_OK) return;
    const std::string what = aeon_b200_last_error();
    switch (status) {
        case AEON_B200_ERR_INVALID_ARGUMENT: throw std::invalid_argument(what);
        case AEON_B200_ERR_LOGIC: throw std::logic_error(what);
        case AEON_B200_ERR_OUT_OF_RANGE: throw std::out_of_range(what);
        default: throw std::runtime_error(what);
    }
}

inline aeon_b200_moe_config moe_config_preset(const char* name) {
    aeon_b200_moe_config cfg{};
    check_status(aeon_b200_config_preset(name, &cfg));
    return cfg;
}

// ---------------------------------------------------------------------------------------------
// Devices and streams. The device is an index the caller supplies, never a heuristic; a device
// that is not there is a named error (src/platform/device.hpp:24-61).
// ---------------------------------------------------------------------------------------------
inline int select_device(int index, bool verbose = true) {
    const int status = aeon_b200_device_select(index);
    if (status != AEON_B200_OK) throw std::runtime_error(aeon_b200_last_error());
    if (verbose) {
        char name[128] = {0};
        int pci_bus = 0;
        if (aeon_b200_device_describe(index, name, sizeof(name), &pci_bus, nullptr, nullptr) == AEON_B200_OK)
            std::cout << "[Aeon Device] Using GPU [" << index << "]: " << name << " (PCI Bus 0x" << std::hex << pci_bus
                      << std::dec << ")" << std::endl;
    }
    return index;
}

// Sets a device for a region and restores the previous one on exit, so a per-rank object (a
// stream set, a pool) is built under its own device without leaking that choice.
class DeviceScope {
public:
    explicit DeviceScope(int index) {
        if (aeon_b200_device_current(&previous_) != AEON_B200_OK) previous_ = 0;
        if (aeon_b200_device_select(index) != AEON_B200_OK)
            throw std::runtime_error(std::string("DeviceScope: ") + aeon_b200_last_error());
    }
    ~DeviceScope() { (void)aeon_b200_device_select(previous_); }
    DeviceScope(const DeviceScope&) = delete;
    DeviceScope& operator=(const DeviceScope&) = delete;

private:
    int previous_{0};
};

// The four streams of a device, split by traffic class (compute: every kernel, and where
// per-transfer events are awaited; sdma: warm-tier uploads; sdma_cold: cold-tier uploads;
// demotion: eviction downloads). Non-blocking; all four or none.
struct DeviceStreams {
    void* compute{nullptr};
    void* sdma{nullptr};
    void* sdma_cold{nullptr};
    void* demotion{nullptr};

    static DeviceStreams create() {
        DeviceStreams streams;
        try {
            streams.compute = create_one("compute");
            streams.sdma = create_one("sdma");
            streams.sdma_cold = create_one("sdma_cold");
            streams.demotion = create_one("demotion");
        } catch (...) {
            streams.destroy();
            throw;
        }
        return streams;
    }
    void destroy() noexcept {
        for (void** stream : {&compute, &sdma, &sdma_cold, &demotion}) {
            if (*stream != nullptr) {
                (void)aeon_b200_stream_destroy(*stream);
                *stream = nullptr;
            }
        }
    }

private:
    static void* create_one(const char* identity) {
        void* stream = nullptr;
        if (aeon_b200_stream_create(&stream) != AEON_B200_OK)
            throw std::runtime_error(std::string("DeviceStreams: stream create(") + identity + "): " +
                                     aeon_b200_last_error());
        return stream;
    }
};

// A device and the four streams that belong to it, created under its own DeviceScope.
struct DeviceContext {
    int device{-1};
    DeviceStreams streams;

    static DeviceContext create(int device) {
        DeviceContext context;
        context.device = device;
        {
            DeviceScope scope(device);
            context.streams = DeviceStreams::create();
        }
        return context;
    }
    void destroy() noexcept {
        streams.destroy();
        device = -1;
    }
};

// Peer access for every ordered pair of `devices` where the hardware allows it, enabled from the
// accessing device. Best effort, never a refusal: a copy between devices works without it.
inline void enable_peer_access(const std::vector<int>& devices, bool verbose = false) {
    for (int accessor : devices)
        for (int peer : devices) {
            if (accessor == peer) continue;
            int enabled = 0;
            (void)aeon_b200_device_enable_peer_access(accessor, peer, &enabled);
            if (!enabled && verbose)
                std::printf("[Peer] device %d cannot access device %d directly\n", accessor, peer);
        }
}

// ---------------------------------------------------------------------------------------------
// Parallel topology (pure host).
// ---------------------------------------------------------------------------------------------
struct ParallelTopologyConfig {
    std::vector<int> device_ids;       // stage-major; empty = 0 .. tp*pp-1
    uint32_t tensor_parallel{1};
    uint32_t pipeline_parallel{1};
    uint32_t expert_parallel{1};       // new: ranks the routed experts are split over
};

struct LayerRange {
    uint32_t first{0};
    uint32_t count{0};
    uint32_t end() const noexcept { return first + count; }
    bool contains(uint32_t layer) const noexcept { return layer >= first && layer < end(); }
};

// "0,1,3" -> {0,1,3}. Empty text = empty list (use the default). Blanks around an entry are
// ignored; an empty or non-numeric or negative entry is refused, naming the offending text.
inline std::vector<int> parse_device_ids(std::string_view text) {
    std::vector<int> ids;
    if (text.empty()) return ids;
    size_t start = 0;
    for (;;) {
        size_t comma = text.find(',', start);
        if (comma == std::string_view::npos) comma = text.size();
        std::string_view entry = text.substr(start, comma - start);
        while (!entry.empty() && (entry.front() == ' ' || entry.front() == '\t')) entry.remove_prefix(1);
        while (!entry.empty() && (entry.back() == ' ' || entry.back() == '\t')) entry.remove_suffix(1);
        if (entry.empty())
            throw std::invalid_argument("device id list has an empty entry: \"" + std::string(text) + "\"");
        if (entry.front() == '-' && entry.size() > 1 &&
            std::all_of(entry.begin() + 1, entry.end(), [](char c) { return c >= '0' && c <= '9'; }))
            throw std::invalid_argument("device id must be non-negative: \"" + std::string(entry) + "\"");
        long value = 0;
        for (char ch : entry) {
            if (ch < '0' || ch > '9')
                throw std::invalid_argument("invalid device id: \"" + std::string(entry) + "\"");
            value = value * 10 + (ch - '0');
            if (value > (1 << 20))
                throw std::invalid_argument("invalid device id: \"" + std::string(entry) + "\"");
        }
        ids.push_back(static_cast<int>(value));
        if (comma == text.size()) break;
        start = comma + 1;
    }
    return ids;
}

// Which experts / which slice of the intermediate dimension one rank owns.
struct ExpertShardDescriptor {
    uint32_t rank{0};
    uint32_t shard_count{1};
    uint32_t first_expert{0}, expert_count{0};          // expert parallel: contiguous block
    uint32_t first_intermediate{0}, intermediate_count{0};  // W2-intermediate tensor parallel
    bool owns_expert(uint32_t e) const noexcept { return e >= first_expert && e < first_expert + expert_count; }
};

class ParallelTopology {
public:
    static ParallelTopology resolve(const ParallelTopologyConfig& config, int visible_devices,
                                    uint32_t artifact_max_tp, uint32_t num_layers) {
        const uint32_t tp = config.tensor_parallel, pp = config.pipeline_parallel;
        const uint32_t ep = config.expert_parallel;
        const auto n = [](auto v) { return std::to_string(v); };
        const size_t rank_count = static_cast<size_t>(tp) * ep * pp;
        std::vector<int> ids = config.device_ids;
        if (ids.empty())
            for (size_t i = 0; i < rank_count; ++i) ids.push_back(static_cast<int>(i));
        // The refusals. Their order and their texts are the contract shared with the reference
        // (src/infrastructure/parallel/parallel_topology.hpp:114-164); the first rule that is
        // broken is the one reported, and a later rule may rely on the earlier ones holding.
        struct Rule {
            std::function<bool()> broken;
            std::function<std::string()> message;
        };
        const Rule rules[] = {
            {[&] { return tp == 0 || pp == 0 || ep == 0; },
             [&] {
                 return "tensor, pipeline and expert degrees must be at least 1 (tensor_parallel=" + n(tp) +
                        ", pipeline_parallel=" + n(pp) + ", expert_parallel=" + n(ep) + ")";
             }},
            {[&] { return num_layers == 0; }, [&] { return std::string("the model has no layers"); }},
            {[&] { return artifact_max_tp == 0; },
             [&] { return std::string("the artifact's max tensor-parallel degree is 0"); }},
            {[&] { return artifact_max_tp % tp != 0; },
             [&] {
                 return "tensor_parallel=" + n(tp) + " does not divide the artifact's max tensor-parallel degree " +
                        n(artifact_max_tp);
             }},
            {[&] { return pp > num_layers; },
             [&] { return "pipeline_parallel=" + n(pp) + " exceeds the " + n(num_layers) + " model layers"; }},
            {[&] { return ep > 1 && tp > 1; },
             [&] {
                 return std::string("expert_parallel and tensor_parallel share the ranks of a stage; set one of "
                                    "them to 1");
             }},
            {[&] { return ids.size() != rank_count; },
             [&] { return "device_ids has " + n(ids.size()) + " entries but tp * ep * pp = " + n(rank_count); }},
        };
        for (const Rule& rule : rules)
            if (rule.broken()) throw std::invalid_argument("parallel topology: " + rule.message());
        for (size_t i = 0; i < ids.size(); ++i) {
            if (ids[i] < 0 || ids[i] >= visible_devices)
                throw std::invalid_argument("parallel topology: device id " + n(ids[i]) + " is out of range for " +
                                            n(visible_devices) + " visible devices");
            if (std::find(ids.begin(), ids.begin() + i, ids[i]) != ids.begin() + i)
                throw std::invalid_argument("parallel topology: device id " + n(ids[i]) + " is listed more than once");
        }
        ParallelTopology topo;
        topo.tp_ = tp;
        topo.pp_ = pp;
        topo.ep_ = ep;
        topo.device_ids_ = std::move(ids);
        // contiguous ranges, remainder to the earliest stages
        const uint32_t base = num_layers / pp, remainder = num_layers % pp;
        uint32_t first = 0;
        for (uint32_t stage = 0; stage < pp; ++stage) {
            const uint32_t count = base + (stage < remainder ? 1u : 0u);
            topo.stages_.push_back(LayerRange{first, count});
            first += count;
        }
        return topo;
    }

    uint32_t tp() const noexcept { return tp_; }
    uint32_t pp() const noexcept { return pp_; }
    uint32_t ep() const noexcept { return ep_; }
    uint32_t ranks_per_stage() const noexcept { return tp_ * ep_; }
    // stage-major: device_ids[stage * ranks_per_stage + rank]
    int device(uint32_t stage, uint32_t rank) const noexcept {
        return device_ids_[static_cast<size_t>(stage) * ranks_per_stage() + rank];
    }
    LayerRange stage_layers(uint32_t stage) const noexcept { return stages_[stage]; }
    uint32_t stage_of(uint32_t layer) const noexcept {
        uint32_t stage = 0;
        while (stage + 1 < stages_.size() && stages_[stage].end() <= layer) ++stage;
        return stage;
    }
    bool is_single_device() const noexcept { return tp_ == 1 && pp_ == 1 && ep_ == 1; }
    const std::vector<int>& device_ids() const noexcept { return device_ids_; }

    // The slice of a layer's routed experts that rank `rank` of a stage holds: a contiguous
    // block of experts under expert parallelism, a contiguous block of the intermediate
    // dimension (W1/W3 rows, W2 columns) under tensor parallelism.
    ExpertShardDescriptor rank_slice(uint32_t rank, uint32_t experts, uint32_t intermediate) const {
        if (rank >= ranks_per_stage()) throw std::out_of_range("parallel topology: rank out of range");
        if (experts % ep_ != 0)
            throw std::invalid_argument("parallel topology: expert_parallel=" + std::to_string(ep_) +
                                        " does not divide the " + std::to_string(experts) + " experts");
        if (intermediate % (tp_ * 128) != 0)
            throw std::invalid_argument("parallel topology: every tensor-parallel shard of the intermediate "
                                        "dimension must be a multiple of 128 columns");
        ExpertShardDescriptor d;
        d.rank = rank;
        d.shard_count = ranks_per_stage();
        const uint32_t er = ep_ > 1 ? rank : 0, tr = tp_ > 1 ? rank : 0;
        d.expert_count = experts / ep_;
        d.first_expert = er * d.expert_count;
        d.intermediate_count = intermediate / tp_;
        d.first_intermediate = tr * d.intermediate_count;
        return d;
    }

private:
    uint32_t tp_{1}, pp_{1}, ep_{1};
    std::vector<int> device_ids_;
    std::vector<LayerRange> stages_;
};

// ---------------------------------------------------------------------------------------------
// Expert payload format and pool.
// ---------------------------------------------------------------------------------------------
enum class ExpertFormatKind : uint32_t { OPAQUE = 0, SWIZZLED_W4A16 = 1, UNKNOWN = 0xFFFFFFFFu };

struct ExpertFormatDescriptor {
    ExpertFormatKind kind{ExpertFormatKind::SWIZZLED_W4A16};
    uint32_t version{2};
    uint32_t sector_size{4096};
    uint32_t num_layers{0};
    uint32_t experts_per_layer{0};
    size_t payload_bytes{0};
    // Shard-aware payloads (version 3): shard_count self-contained shards of the intermediate
    // dimension, shard-major. Version 2 means {1, payload_bytes}; shard_bytes 0 is read as that.
    uint32_t shard_count{1};
    size_t shard_bytes{0};

    uint64_t total_experts() const noexcept { return static_cast<uint64_t>(num_layers) * experts_per_layer; }
    size_t bytes_per_shard() const noexcept { return shard_bytes != 0 ? shard_bytes : payload_bytes; }
    void validate_payload() const {
        if (payload_bytes == 0 || sector_size == 0 || payload_bytes % sector_size != 0)
            throw std::invalid_argument("ExpertFormatDescriptor: payload must be a positive multiple of the sector size");
        if (shard_count == 0 || static_cast<uint64_t>(shard_count) * bytes_per_shard() != payload_bytes)
            throw std::invalid_argument("ExpertFormatDescriptor: shard_count x shard_bytes must equal the payload size");
        if (bytes_per_shard() % sector_size != 0)
            throw std::invalid_argument("ExpertFormatDescriptor: shard_bytes must be a multiple of the sector size");
    }
    void validate_catalog() const {
        validate_payload();
        if (num_layers == 0 || experts_per_layer == 0)
            throw std::invalid_argument("ExpertFormatDescriptor: empty expert catalog");
    }
};

inline ExpertFormatDescriptor make_swizzled_expert_format(const aeon_b200_moe_config& cfg, uint32_t layers,
                                                          uint32_t shard_count = 1) {
    uint64_t shard_bytes = 0;
    check_status(aeon_b200_expert_shard_bytes(&cfg, static_cast<int>(shard_count), &shard_bytes));
    ExpertFormatDescriptor f;
    f.kind = ExpertFormatKind::SWIZZLED_W4A16;
    f.version = shard_count > 1 ? 3 : 2;
    f.num_layers = layers;
    f.experts_per_layer = static_cast<uint32_t>(cfg.experts);
    f.payload_bytes = static_cast<size_t>(shard_bytes) * shard_count;
    f.shard_count = shard_count;
    f.shard_bytes = static_cast<size_t>(shard_bytes);
    return f;
}

// Which weight backend executes which expert format (expert_backend.hpp:14-79). One backend
// here, the swizzled W4A16 one; its payload size follows the layer shape instead of being one
// compile-time constant, so a descriptor is made for a configuration and validates the size an
// artifact declares against it.
struct ExpertBackendDescriptor {
    std::string_view name;
    ExpertFormatKind format_kind{ExpertFormatKind::UNKNOWN};
    uint32_t artifact_version_min{0}, artifact_version_max{0};
    size_t payload_bytes{0};                 // 0: any size (no configuration bound to the descriptor)
    bool supports_fused_moe_experts{false};

    void validate_format(const ExpertFormatDescriptor& format) const {
        if (format.kind != format_kind || format.version < artifact_version_min ||
            format.version > artifact_version_max || (payload_bytes != 0 && format.payload_bytes != payload_bytes))
            throw std::runtime_error("Expert backend '" + std::string(name) +
                                     "' is incompatible with the loaded expert artifact");
    }
};

class ExpertBackendRegistry {
public:
    static const ExpertBackendDescriptor& resolve(std::string_view name) {
        if (name == "swizzled_w4a16") return swizzled_w4a16();
        throw std::invalid_argument("ExpertBackendRegistry: unsupported weight backend '" + std::string(name) + "'");
    }
    static const ExpertBackendDescriptor& resolve(ExpertFormatKind kind) {
        if (kind == ExpertFormatKind::SWIZZLED_W4A16) return swizzled_w4a16();
        throw std::invalid_argument("ExpertBackendRegistry: no backend is registered for the requested expert format");
    }
    static const ExpertBackendDescriptor& resolve(std::string_view name, const ExpertFormatDescriptor& format) {
        const ExpertBackendDescriptor& backend = resolve(name);
        backend.validate_format(format);
        return backend;
    }
    static const ExpertBackendDescriptor& resolve(const ExpertFormatDescriptor& format) {
        const ExpertBackendDescriptor& backend = resolve(format.kind);
        backend.validate_format(format);
        return backend;
    }
    // The backend bound to one layer shape: its payload size is the swizzled layout's.
    static ExpertBackendDescriptor for_config(const aeon_b200_moe_config& cfg) {
        ExpertBackendDescriptor d = swizzled_w4a16();
        aeon_b200_expert_layout layout{};
        check_status(aeon_b200_expert_layout_of(&cfg, &layout));
        d.payload_bytes = static_cast<size_t>(layout.payload_bytes);
        return d;
    }

private:
    static const ExpertBackendDescriptor& swizzled_w4a16() {
        // version 2: the reference's container; version 3: the shard-aware one
        static const ExpertBackendDescriptor descriptor{"swizzled_w4a16", ExpertFormatKind::SWIZZLED_W4A16, 2, 3, 0, true};
        return descriptor;
    }
};

// One device slab of slots x payload_bytes; a slot is a byte-identical expert payload.
class UnifiedVRAMExpertPool {
public:
    uint32_t num_slots{0};
    uint8_t* d_experts{nullptr};

    UnifiedVRAMExpertPool() = default;
    UnifiedVRAMExpertPool(uint32_t slots, const aeon_b200_moe_config& cfg, ExpertFormatDescriptor format,
                          int device = 0)
        : cfg_(cfg), format_(format), device_(device) {
        format_.validate_payload();
        check_status(aeon_b200_expert_layout_of(&cfg_, &layout_));
        if (format_.kind == ExpertFormatKind::SWIZZLED_W4A16 && format_.payload_bytes != layout_.payload_bytes)
            throw std::invalid_argument("UnifiedVRAMExpertPool: payload size does not match the swizzled layout");
        if (slots == 0) return;
        void* base = nullptr;
        check_status(aeon_b200_pool_create(format_.payload_bytes, slots, device, &base));
        d_experts = static_cast<uint8_t*>(base);
        num_slots = slots;
    }
    ~UnifiedVRAMExpertPool() { release(); }
    UnifiedVRAMExpertPool(const UnifiedVRAMExpertPool&) = delete;
    UnifiedVRAMExpertPool& operator=(const UnifiedVRAMExpertPool&) = delete;
    UnifiedVRAMExpertPool(UnifiedVRAMExpertPool&& o) noexcept { take(std::move(o)); }
    UnifiedVRAMExpertPool& operator=(UnifiedVRAMExpertPool&& o) noexcept {
        if (this != &o) { release(); take(std::move(o)); }
        return *this;
    }

    const ExpertFormatDescriptor& format() const noexcept { return format_; }
    uint8_t* get_slot_base(uint32_t slot) const {
        if (d_experts == nullptr || slot >= num_slots)
            throw std::runtime_error("ExpertPayloadPool: Invalid slot index " + std::to_string(slot));
        return d_experts + static_cast<size_t>(slot) * format_.payload_bytes;
    }
    void upload_from_host_expert(uint32_t slot, const uint8_t* host_payload, void* stream = nullptr) {
        if (slot >= num_slots || host_payload == nullptr)
            throw std::runtime_error("ExpertPayloadPool: Invalid upload source or slot index");
        check_status(aeon_b200_pool_upload(d_experts, format_.payload_bytes, slot, host_payload, stream));
    }
    // Typed views; only a swizzled-format pool has them (the reference's format guard).
    const uint32_t* get_w1_packed(uint32_t s) const { return view<uint32_t>(s, layout_.w1_packed_offset); }
    const uint16_t* get_w1_scale(uint32_t s) const { return view<uint16_t>(s, layout_.w1_scale_offset); }
    const uint32_t* get_w2_packed(uint32_t s) const { return view<uint32_t>(s, layout_.w2_packed_offset); }
    const uint16_t* get_w2_scale(uint32_t s) const { return view<uint16_t>(s, layout_.w2_scale_offset); }
    const uint32_t* get_w3_packed(uint32_t s) const { return view<uint32_t>(s, layout_.w3_packed_offset); }
    const uint16_t* get_w3_scale(uint32_t s) const { return view<uint16_t>(s, layout_.w3_scale_offset); }

private:
    template <class T>
    const T* view(uint32_t slot, uint64_t offset) const {
        if (format_.kind != ExpertFormatKind::SWIZZLED_W4A16)
            throw std::logic_error("UnifiedVRAMExpertPool: swizzled views requested from a pool of another format");
        return reinterpret_cast<const T*>(get_slot_base(slot) + offset);
    }
    void release() noexcept {
        if (d_experts) (void)aeon_b200_pool_destroy(d_experts, device_);
        d_experts = nullptr;
        num_slots = 0;
    }
    void take(UnifiedVRAMExpertPool&& o) noexcept {
        num_slots = o.num_slots; d_experts = o.d_experts; cfg_ = o.cfg_; format_ = o.format_;
        layout_ = o.layout_; device_ = o.device_;
        o.d_experts = nullptr; o.num_slots = 0;
    }
    aeon_b200_moe_config cfg_{};
    ExpertFormatDescriptor format_{};
    aeon_b200_expert_layout layout_{};
    int device_{0};
};

// ---------------------------------------------------------------------------------------------
// Registry: which expert of which layer sits in which pool slot. Host integers only.
// ---------------------------------------------------------------------------------------------
enum class ExpertTier : uint8_t { HOT_VRAM = 0, WARM_HOST = 1, COLD_NVME = 2 };
enum class ExpertRequestKind : uint8_t { HOT_HIT = 0, WARM_PROMOTION = 1, COLD_MISS = 2, PENDING = 3, COLD_STAGED = 4 };

struct ExpertRequestReservation {
    ExpertRequestKind kind{ExpertRequestKind::COLD_MISS};
    ExpertTier source_tier{ExpertTier::COLD_NVME};
    uint32_t global_expert_id{0};
    uint64_t operation_id{0};
    int32_t vram_slot{-1};
    bool lease_acquired{false};
    int32_t evicted_global_id{-1};     // the expert that lost the slot, if any
};

class ExpertRegistry {
public:
    uint32_t num_layers{0};
    uint32_t experts_per_layer{0};
    uint32_t vram_capacity{0};

    ExpertRegistry() = default;
    ExpertRegistry(uint32_t layers, uint32_t experts, uint32_t slots) { init(layers, experts, slots); }

    void init(uint32_t layers, uint32_t experts, uint32_t slots) {
        if (layers == 0 || experts == 0) throw std::invalid_argument("ExpertRegistry: empty catalog");
        num_layers = layers;
        experts_per_layer = experts;
        vram_capacity = slots;
        entries_.assign(static_cast<size_t>(layers) * experts, Entry{});
        free_slots_.clear();
        for (uint32_t s = slots; s > 0; --s) free_slots_.push_back(static_cast<int32_t>(s - 1));
        lru_.clear();
        pending_.clear();
        next_operation_ = 1;
        hot_hits = cold_misses = evictions = 0;
    }

    uint32_t get_global_id(uint32_t layer, uint32_t expert) const {
        if (layer >= num_layers || expert >= experts_per_layer)
            throw std::out_of_range("ExpertRegistry: layer or expert id out of range");
        return layer * experts_per_layer + expert;
    }

    // Mark every expert resident in slot order (the full-residency start state).
    void populate_all_hot() {
        if (vram_capacity < entries_.size())
            throw std::invalid_argument("ExpertRegistry: the pool is smaller than the catalog");
        for (uint32_t gid = 0; gid < entries_.size(); ++gid) {
            if (entries_[gid].slot >= 0) continue;
            entries_[gid].slot = free_slots_.back();
            free_slots_.pop_back();
            entries_[gid].published = true;
            lru_.push_front(gid);
            entries_[gid].lru_it = lru_.begin();
            entries_[gid].in_lru = true;
        }
    }

    // A request for (layer, expert) with a lease. Resident: HOT_HIT. Otherwise a slot is taken
    // from the free list, or from the least recently used resident expert that holds no lease
    // and has no operation pending; the caller uploads the payload and calls complete_request.
    ExpertRequestReservation reserve_request(uint32_t layer, uint32_t expert) {
        const uint32_t gid = get_global_id(layer, expert);
        Entry& e = entries_[gid];
        ExpertRequestReservation r;
        r.global_expert_id = gid;
        if (e.slot >= 0 && e.published) {
            ++hot_hits;
            touch(gid);
            ++e.lease_count;
            r.kind = ExpertRequestKind::HOT_HIT;
            r.source_tier = ExpertTier::HOT_VRAM;
            r.vram_slot = e.slot;
            r.lease_acquired = true;
            return r;
        }
        if (e.slot >= 0 && !e.published) {      // an upload for it is already in flight
            ++e.lease_count;
            r.kind = ExpertRequestKind::PENDING;
            r.vram_slot = e.slot;
            r.operation_id = e.operation_id;
            r.lease_acquired = true;
            return r;
        }
        int32_t slot = -1;
        if (!free_slots_.empty()) {
            slot = free_slots_.back();
            free_slots_.pop_back();
        } else {
            for (auto it = lru_.rbegin(); it != lru_.rend(); ++it) {
                Entry& victim = entries_[*it];
                if (victim.lease_count == 0 && victim.published) {
                    slot = victim.slot;
                    r.evicted_global_id = static_cast<int32_t>(*it);
                    victim.slot = -1;
                    victim.published = false;
                    victim.in_lru = false;
                    lru_.erase(victim.lru_it);
                    ++evictions;
                    break;
                }
            }
        }
        if (slot < 0) throw std::runtime_error("ExpertRegistry: no reclaimable Hot VRAM slot");
        ++cold_misses;
        e.slot = slot;
        e.published = false;
        e.operation_id = next_operation_++;
        ++e.lease_count;
        pending_[e.operation_id] = gid;
        r.kind = ExpertRequestKind::COLD_MISS;
        r.vram_slot = slot;
        r.operation_id = e.operation_id;
        r.lease_acquired = true;
        return r;
    }

    void complete_request(uint64_t operation_id) {
        auto it = pending_.find(operation_id);
        if (it == pending_.end()) throw std::logic_error("ExpertRegistry: unknown operation id");
        Entry& e = entries_[it->second];
        e.published = true;
        e.operation_id = 0;
        lru_.push_front(it->second);
        e.lru_it = lru_.begin();
        e.in_lru = true;
        pending_.erase(it);
    }

    // Roll a failed upload back: the slot returns to the free list, leases on it are dropped.
    void fail_request(uint64_t operation_id) {
        auto it = pending_.find(operation_id);
        if (it == pending_.end()) throw std::logic_error("ExpertRegistry: unknown operation id");
        Entry& e = entries_[it->second];
        free_slots_.push_back(e.slot);
        e = Entry{};
        pending_.erase(it);
    }

    void release_lease(uint32_t gid) {
        if (gid >= entries_.size()) throw std::out_of_range("ExpertRegistry: global id out of range");
        if (entries_[gid].lease_count == 0) throw std::logic_error("ExpertRegistry: lease released twice");
        --entries_[gid].lease_count;
    }

    bool expert_resident(uint32_t layer, uint32_t expert) const {
        const Entry& e = entries_[get_global_id(layer, expert)];
        return e.slot >= 0 && e.published;
    }
    int32_t slot_of(uint32_t layer, uint32_t expert) const {
        const Entry& e = entries_[get_global_id(layer, expert)];
        return (e.slot >= 0 && e.published) ? e.slot : -1;
    }
    uint32_t lease_count(uint32_t gid) const { return entries_.at(gid).lease_count; }
    size_t free_vram_slot_count() const noexcept { return free_slots_.size(); }
    uint64_t pending_transfer_count() const noexcept { return pending_.size(); }

    // slot table of one layer as the kernels want it: expert -> slot, -1 when absent
    std::vector<int32_t> layer_slot_table(uint32_t layer) const {
        std::vector<int32_t> table(experts_per_layer, -1);
        for (uint32_t e = 0; e < experts_per_layer; ++e) table[e] = slot_of(layer, e);
        return table;
    }

    // Audit: every slot is owned at most once, free + owned = capacity, the LRU list holds
    // exactly the published residents, pending operations point at unpublished owners.
    bool invariants_hold() const noexcept {
        std::vector<int> owner(vram_capacity, 0);
        size_t owned = 0, published = 0;
        for (const Entry& e : entries_) {
            if (e.slot < 0) {
                if (e.published || e.in_lru) return false;
                continue;
            }
            if (static_cast<uint32_t>(e.slot) >= vram_capacity || owner[e.slot]++) return false;
            ++owned;
            if (e.published) ++published;
            if (e.published != e.in_lru) return false;
        }
        for (int32_t s : free_slots_)
            if (s < 0 || static_cast<uint32_t>(s) >= vram_capacity || owner[s]++) return false;
        if (owned + free_slots_.size() != vram_capacity) return false;
        if (lru_.size() != published) return false;
        for (const auto& kv : pending_)
            if (kv.second >= entries_.size() || entries_[kv.second].published) return false;
        return true;
    }

    uint64_t hot_hits{0}, cold_misses{0}, evictions{0};

private:
    struct Entry {
        int32_t slot{-1};
        bool published{false};
        bool in_lru{false};
        uint32_t lease_count{0};
        uint64_t operation_id{0};
        std::list<uint32_t>::iterator lru_it{};
    };
    void touch(uint32_t gid) {
        Entry& e = entries_[gid];
        if (e.in_lru) lru_.erase(e.lru_it);
        lru_.push_front(gid);
        e.lru_it = lru_.begin();
        e.in_lru = true;
    }
    std::vector<Entry> entries_;
    std::vector<int32_t> free_slots_;
    std::list<uint32_t> lru_;
    std::unordered_map<uint64_t, uint32_t> pending_;
    uint64_t next_operation_{1};
};

class ExpertLeaseHolder {
public:
    virtual ~ExpertLeaseHolder() = default;
    virtual void release_leases() = 0;
    virtual size_t outstanding_leases() const noexcept = 0;
};

// ---------------------------------------------------------------------------------------------
// Read-only memory mapping of a file (the loader maps both containers, aeon_loader.hpp:243-270).
// ---------------------------------------------------------------------------------------------
class MappedFile {
public:
    MappedFile() = default;
    MappedFile(const MappedFile&) = delete;
    MappedFile& operator=(const MappedFile&) = delete;
    ~MappedFile() { close(); }

    void open(const std::string& path, const char* what) {
        close();
        fd_ = ::open(path.c_str(), O_RDONLY);
        if (fd_ < 0) throw std::runtime_error(std::string("AeonModelLoader: Failed to open ") + what + ": " + path);
        struct stat st;
        if (::fstat(fd_, &st) != 0) {
            close();
            throw std::runtime_error(std::string("AeonModelLoader: Failed to stat ") + what + ": " + path);
        }
        size_ = static_cast<size_t>(st.st_size);
        if (size_ != 0) {
            void* m = ::mmap(nullptr, size_, PROT_READ, MAP_SHARED, fd_, 0);
            if (m == MAP_FAILED) {
                close();
                throw std::runtime_error(std::string("AeonModelLoader: Failed to mmap ") + what + ": " + path);
            }
            base_ = static_cast<const uint8_t*>(m);
        }
    }
    void close() noexcept {
        if (base_) ::munmap(const_cast<uint8_t*>(base_), size_);
        if (fd_ >= 0) ::close(fd_);
        base_ = nullptr; size_ = 0; fd_ = -1;
    }
    const uint8_t* data() const noexcept { return base_; }
    size_t size() const noexcept { return size_; }

private:
    int fd_{-1};
    const uint8_t* base_{nullptr};
    size_t size_{0};
};

// ---------------------------------------------------------------------------------------------
// Expert container: `.index` = magic "AEON_EXPERTS", u32 version, u32 layers, u32 experts per
// layer, u64 payload bytes (version 2: 32 bytes), then for version 3 u32 shard count, u32 zero,
// u64 shard bytes (48 bytes), then (u64 offset, u64 length) per expert; payloads in a second,
// memory-mapped file. Version 3 is the shard-aware layout the reference plans
// (plans-and-docs/execution/active/MULTI_GPU_EXECUTION_PLAN.md:151-181).
// ---------------------------------------------------------------------------------------------
class AeonExpertContainer {
public:
    struct Location { uint64_t offset; uint64_t length; };

    // expected_version 0 accepts 2 and 3; expected_payload_bytes 0 accepts any size.
    void open(const std::string& index_path, const std::string& experts_path, uint32_t expected_version,
              size_t expected_payload_bytes) {
        std::ifstream idx(index_path, std::ios::binary);
        if (!idx) throw std::runtime_error("AeonModelLoader: Failed to open expert index: " + index_path);
        std::vector<uint8_t> buf((std::istreambuf_iterator<char>(idx)), std::istreambuf_iterator<char>());
        if (buf.size() < 32) throw std::runtime_error("AeonModelLoader: Expert index too small for header!");
        if (std::memcmp(buf.data(), "AEON_EXPERTS", 12) != 0)
            throw std::runtime_error("AeonModelLoader: Invalid expert index magic!");
        uint32_t version, layers, experts;
        uint64_t expert_bytes;
        std::memcpy(&version, buf.data() + 12, 4);
        std::memcpy(&layers, buf.data() + 16, 4);
        std::memcpy(&experts, buf.data() + 20, 4);
        std::memcpy(&expert_bytes, buf.data() + 24, 8);
        if (expected_version != 0 ? version != expected_version : (version != 2 && version != 3))
            throw std::runtime_error("AeonModelLoader: Unexpected expert index version " + std::to_string(version) +
                                     ", expected " + (expected_version ? std::to_string(expected_version) : "2 or 3"));
        if (expected_payload_bytes != 0 && expert_bytes != expected_payload_bytes)
            throw std::runtime_error("AeonModelLoader: Expert payload size does not match the artifact specification");
        size_t head = 32;
        uint32_t shard_count = 1;
        uint64_t shard_bytes = expert_bytes;
        if (version == 3) {
            if (buf.size() < 48) throw std::runtime_error("AeonModelLoader: Expert index too small for header!");
            std::memcpy(&shard_count, buf.data() + 32, 4);
            std::memcpy(&shard_bytes, buf.data() + 40, 8);
            head = 48;
        }
        ExpertFormatDescriptor f;
        f.kind = ExpertFormatKind::SWIZZLED_W4A16;
        f.version = version;
        f.num_layers = layers;
        f.experts_per_layer = experts;
        f.payload_bytes = static_cast<size_t>(expert_bytes);
        f.shard_count = shard_count;
        f.shard_bytes = static_cast<size_t>(shard_bytes);
        try {
            f.validate_catalog();
        } catch (const std::invalid_argument& e) {
            throw std::runtime_error(std::string("AeonModelLoader: ") + e.what());
        }
        const uint64_t total = f.total_experts();
        if (buf.size() < head + total * 16) throw std::runtime_error("AeonModelLoader: Expert index has incomplete entries!");
        std::vector<Location> locations(total);
        for (uint64_t i = 0; i < total; ++i) {
            uint64_t off, len;
            std::memcpy(&off, buf.data() + head + i * 16, 8);
            std::memcpy(&len, buf.data() + head + i * 16 + 8, 8);
            if (len != expert_bytes || off % f.sector_size != 0)
                throw std::runtime_error("AeonModelLoader: Expert index contains an invalid payload entry");
            locations[i] = Location{off, len};
        }
        file_.open(experts_path, "experts file");
        for (const Location& l : locations)
            if (l.offset + l.length > file_.size()) {
                file_.close();
                throw std::runtime_error("AeonModelLoader: Expert payload lies outside the experts file");
            }
        format_ = f;
        locations_ = std::move(locations);
    }

    const ExpertFormatDescriptor& format() const noexcept { return format_; }
    void close() noexcept {
        locations_.clear();
        format_ = ExpertFormatDescriptor{};
        file_.close();
    }
    Location get_expert_location(uint32_t layer, uint32_t expert) const { return locations_.at(index_of(layer, expert)); }
    const uint8_t* get_expert_data(uint32_t layer, uint32_t expert) const {
        return file_.data() + locations_.at(index_of(layer, expert)).offset;
    }

    // What rank `rank` of a tensor-parallel group of degree `tp` reads of one expert: one
    // contiguous, sector-aligned range, offset + rank * (shards / tp) * shard_bytes, payload / tp
    // long. tp must divide the artifact's shard count (its maximum tensor-parallel degree).
    Location rank_slice(uint32_t layer, uint32_t expert, uint32_t tp, uint32_t rank) const {
        const Location whole = get_expert_location(layer, expert);
        if (tp == 0 || format_.shard_count % tp != 0)
            throw std::invalid_argument("AeonModelLoader: tensor_parallel=" + std::to_string(tp) +
                                        " does not divide the artifact's max tensor-parallel degree " +
                                        std::to_string(format_.shard_count));
        if (rank >= tp) throw std::out_of_range("AeonModelLoader: tensor-parallel rank out of range");
        const uint64_t per_rank = static_cast<uint64_t>(format_.shard_count / tp) * format_.bytes_per_shard();
        return Location{whole.offset + rank * per_rank, per_rank};
    }

    // The payload rank `rank` uploads into its pool: its slice with the slice's shards merged
    // into one swizzled payload of width cfg.intermediate / tp. `cfg` describes the whole expert.
    std::vector<uint8_t> read_rank_payload(const aeon_b200_moe_config& cfg, uint32_t layer, uint32_t expert,
                                           uint32_t tp, uint32_t rank) const {
        const Location slice = rank_slice(layer, expert, tp, rank);
        aeon_b200_moe_config rank_cfg = cfg;
        rank_cfg.intermediate = cfg.intermediate / static_cast<int32_t>(tp);
        aeon_b200_expert_layout lay{};
        check_status(aeon_b200_expert_layout_of(&rank_cfg, &lay));
        std::vector<uint8_t> out(lay.payload_bytes);
        check_status(aeon_b200_merge_expert_shards(&rank_cfg, static_cast<int>(format_.shard_count / tp),
                                                   file_.data() + slice.offset, out.data()));
        return out;
    }

    // Writer used by tools and tests: payloads in (layer, expert) order, sector-aligned.
    // shard_count > 1 writes the version-3 header (the payloads must already be shard-major,
    // aeon_b200_pack_expert_shards).
    static void write(const std::string& index_path, const std::string& experts_path, uint32_t version,
                      uint32_t layers, uint32_t experts, uint64_t expert_bytes,
                      const std::vector<const uint8_t*>& payloads, uint32_t shard_count = 1) {
        if (payloads.size() != static_cast<size_t>(layers) * experts)
            throw std::invalid_argument("AeonExpertContainer::write: payload count does not match the catalog");
        if (shard_count == 0 || expert_bytes % shard_count != 0 || (version < 3 && shard_count != 1))
            throw std::invalid_argument("AeonExpertContainer::write: shard count does not fit the version or the payload size");
        std::ofstream idx(index_path, std::ios::binary), exp(experts_path, std::ios::binary);
        if (!idx || !exp) throw std::runtime_error("AeonExpertContainer::write: cannot create the output files");
        idx.write("AEON_EXPERTS", 12);
        idx.write(reinterpret_cast<const char*>(&version), 4);
        idx.write(reinterpret_cast<const char*>(&layers), 4);
        idx.write(reinterpret_cast<const char*>(&experts), 4);
        idx.write(reinterpret_cast<const char*>(&expert_bytes), 8);
        if (version >= 3) {
            const uint32_t zero = 0;
            const uint64_t shard_bytes = expert_bytes / shard_count;
            idx.write(reinterpret_cast<const char*>(&shard_count), 4);
            idx.write(reinterpret_cast<const char*>(&zero), 4);
            idx.write(reinterpret_cast<const char*>(&shard_bytes), 8);
        }
        uint64_t offset = 0;
        for (const uint8_t* payload : payloads) {
            idx.write(reinterpret_cast<const char*>(&offset), 8);
            idx.write(reinterpret_cast<const char*>(&expert_bytes), 8);
            exp.write(reinterpret_cast<const char*>(payload), static_cast<std::streamsize>(expert_bytes));
            offset += expert_bytes;
        }
    }

private:
    size_t index_of(uint32_t layer, uint32_t expert) const {
        if (layer >= format_.num_layers || expert >= format_.experts_per_layer)
            throw std::out_of_range("AeonModelLoader: expert id out of range");
        return static_cast<size_t>(layer) * format_.experts_per_layer + expert;
    }
    ExpertFormatDescriptor format_{};
    std::vector<Location> locations_;
    MappedFile file_;
};

// ---------------------------------------------------------------------------------------------
// Dense container: "AEON_DENSE\0\0", u32 version, u32 tensor count, u64 directory length, a
// JSON directory [{name, offset, size, dtype, shape}], tensor bytes from the next 4 KiB
// boundary (src/infrastructure/artifact/aeon_loader.hpp:243-316,441-479). The router gate and
// the shared expert of every layer live here
// (src/architecture/deepseek_v4/spec/v4_dense_weight_binding.hpp:123-137).
// ---------------------------------------------------------------------------------------------
struct LoadedTensor {
    const uint8_t* data{nullptr};
    int64_t byte_size{0};
    std::string dtype;
    std::vector<int64_t> shape;
};

namespace detail {

// The few JSON forms the directory uses: an array of flat objects whose values are strings,
// integers or arrays of integers. Anything else is refused.
class DirectoryParser {
public:
    explicit DirectoryParser(const std::string& text) : s_(text) {}

    template <class F>   // F(name, offset, size, dtype, shape)
    size_t parse(F&& emit) {
        size_t count = 0;
        skip();
        expect('[');
        skip();
        if (peek() == ']') { ++i_; end(); return 0; }
        for (;;) {
            std::string name, dtype;
            int64_t offset = -1, size = -1;
            std::vector<int64_t> shape;
            bool has_name = false, has_dtype = false, has_offset = false, has_size = false, has_shape = false;
            skip();
            expect('{');
            for (;;) {
                skip();
                const std::string key = string();
                skip();
                expect(':');
                skip();
                if (key == "name") { name = string(); has_name = true; }
                else if (key == "dtype") { dtype = string(); has_dtype = true; }
                else if (key == "offset") { offset = integer(); has_offset = true; }
                else if (key == "size") { size = integer(); has_size = true; }
                else if (key == "shape") {
                    expect('[');
                    skip();
                    if (peek() == ']') ++i_;
                    else
                        for (;;) {
                            skip();
                            shape.push_back(integer());
                            skip();
                            if (peek() == ',') { ++i_; continue; }
                            expect(']');
                            break;
                        }
                    has_shape = true;
                } else {
                    fail("unknown key \"" + key + "\"");
                }
                skip();
                if (peek() == ',') { ++i_; continue; }
                expect('}');
                break;
            }
            if (!(has_name && has_dtype && has_offset && has_size && has_shape)) fail("entry lacks a field");
            emit(name, offset, size, dtype, shape);
            ++count;
            skip();
            if (peek() == ',') { ++i_; continue; }
            expect(']');
            break;
        }
        end();
        return count;
    }

private:
    void end() { skip(); if (i_ != s_.size()) fail("text after the directory"); }
    [[noreturn]] void fail(const std::string& why) const {
        throw std::runtime_error("AeonModelLoader: Malformed dense directory (" + why + " at byte " + std::to_string(i_) + ")");
    }
    char peek() const { return i_ < s_.size() ? s_[i_] : '\0'; }
    void skip() { while (i_ < s_.size() && (s_[i_] == ' ' || s_[i_] == '\n' || s_[i_] == '\t' || s_[i_] == '\r')) ++i_; }
    void expect(char c) { if (peek() != c) fail(std::string("expected '") + c + "'"); ++i_; }
    std::string string() {
        expect('"');
        std::string out;
        while (i_ < s_.size() && s_[i_] != '"') {
            if (s_[i_] == '\\') {
                if (i_ + 1 >= s_.size()) fail("dangling escape");
                const char e = s_[i_ + 1];
                if (e == '"' || e == '\\' || e == '/') out.push_back(e);
                else fail("unsupported escape");
                i_ += 2;
            } else {
                out.push_back(s_[i_++]);
            }
        }
        expect('"');
        return out;
    }
    int64_t integer() {
        const size_t start = i_;
        bool negative = false;
        if (peek() == '-') { negative = true; ++i_; }
        if (peek() < '0' || peek() > '9') fail("expected an integer");
        int64_t v = 0;
        while (peek() >= '0' && peek() <= '9') {
            if (v > (INT64_MAX - 9) / 10) fail("integer too large");
            v = v * 10 + (s_[i_++] - '0');
        }
        if (peek() == '.' || peek() == 'e' || peek() == 'E') { i_ = start; fail("expected an integer"); }
        return negative ? -v : v;
    }
    const std::string& s_;
    size_t i_{0};
};

}  // namespace detail

class AeonDenseContainer {
public:
    void open(const std::string& path, uint32_t expected_version = 1) {
        file_.open(path, "dense file");
        tensors_.clear();
        if (file_.size() < 28) throw std::runtime_error("AeonModelLoader: Dense file too small for header: " + path);
        if (std::memcmp(file_.data(), "AEON_DENSE\0\0", 12) != 0)
            throw std::runtime_error("AeonModelLoader: Invalid dense magic in " + path);
        uint32_t version, count;
        uint64_t dir_len;
        std::memcpy(&version, file_.data() + 12, 4);
        std::memcpy(&count, file_.data() + 16, 4);
        std::memcpy(&dir_len, file_.data() + 20, 8);
        if (version != expected_version)
            throw std::runtime_error("AeonModelLoader: Unexpected dense format version " + std::to_string(version) +
                                     ", expected " + std::to_string(expected_version));
        if (dir_len > file_.size() - 28) throw std::runtime_error("AeonModelLoader: Directory length exceeds file size!");
        const std::string dir(reinterpret_cast<const char*>(file_.data() + 28), static_cast<size_t>(dir_len));
        size_t start = 28 + static_cast<size_t>(dir_len);
        start += (4096 - start % 4096) % 4096;
        if (start > file_.size()) throw std::runtime_error("AeonModelLoader: Dense payload starts beyond file size");
        const uint64_t room = file_.size() - start;
        const uint8_t* base = file_.data() + start;
        detail::DirectoryParser parser(dir);
        const size_t parsed = parser.parse([&](const std::string& name, int64_t offset, int64_t size,
                                               const std::string& dtype, const std::vector<int64_t>& shape) {
            if (offset < 0 || size < 0) throw std::runtime_error("AeonModelLoader: Dense directory contains a negative range");
            if (static_cast<uint64_t>(offset) > room || static_cast<uint64_t>(size) > room - static_cast<uint64_t>(offset))
                throw std::runtime_error("AeonModelLoader: Dense tensor range exceeds payload");
            for (int64_t d : shape)
                if (d < 0) throw std::runtime_error("AeonModelLoader: Dense tensor shape is negative");
            LoadedTensor t;
            t.data = base + offset;
            t.byte_size = size;
            t.dtype = dtype;
            t.shape = shape;
            if (!tensors_.emplace(name, std::move(t)).second)
                throw std::runtime_error("AeonModelLoader: Duplicate dense tensor: " + name);
        });
        if (parsed != count) throw std::runtime_error("AeonModelLoader: Dense directory count does not match its header");
    }

    bool has_tensor(const std::string& name) const { return tensors_.count(name) != 0; }
    const LoadedTensor& get_tensor(const std::string& name) const {
        const auto it = tensors_.find(name);
        if (it == tensors_.end()) throw std::runtime_error("AeonModelLoader: Missing dense tensor: " + name);
        return it->second;
    }
    size_t tensor_count() const noexcept { return tensors_.size(); }
    size_t file_size() const noexcept { return file_.size(); }
    void close() noexcept {
        tensors_.clear();
        file_.close();
    }

private:
    MappedFile file_;
    std::unordered_map<std::string, LoadedTensor> tensors_;
};

// What a model directory declares about itself (model_manifest.json; the reference's
// AeonModelManifest, src/infrastructure/artifact/model_manifest.hpp:102-209): identity, the weight
// backend, the three file names, format versions and sizes. Keys are unique in the file, so
// each is found by name wherever it sits (the "artifact" object is flattened). Version 1 is the
// reference's manifest; version 2 adds the shard fields of the shard-aware container.
struct AeonArtifactSpec {
    std::string dense_filename{"model_dense.aeon"};
    std::string experts_filename{"model_experts_swizzled.aeon"};
    std::string index_filename{"model_experts_swizzled.index"};
    uint32_t expected_dense_version{1};
    ExpertFormatKind expert_format_kind{ExpertFormatKind::SWIZZLED_W4A16};
    uint32_t expected_expert_version{0};           // 0: version 2 or 3
    uint32_t expert_sector_size{4096};
    size_t expected_expert_payload_bytes{0};       // 0: any
};

struct AeonModelManifest {
    uint32_t manifest_version{0};
    std::string model_family, architecture, weight_backend;
    AeonArtifactSpec artifact{};
    size_t dense_file_bytes{0};
    uint32_t num_layers{0}, experts_per_layer{0};
    uint32_t max_tensor_parallel{1};

    static AeonModelManifest load_from_json(const std::string& manifest_path) {
        std::ifstream file(manifest_path);
        if (!file.is_open()) throw std::runtime_error("AeonModelManifest: failed to open manifest: " + manifest_path);
        std::stringstream buffer;
        buffer << file.rdbuf();
        const std::string text = buffer.str();
        AeonModelManifest m;
        m.manifest_version = static_cast<uint32_t>(number(text, "manifest_version"));
        m.model_family = string(text, "model_family");
        m.architecture = string(text, "architecture");
        m.weight_backend = string(text, "weight_backend");
        m.artifact.dense_filename = string(text, "dense_filename");
        m.artifact.experts_filename = string(text, "experts_filename");
        m.artifact.index_filename = string(text, "index_filename");
        m.artifact.expected_dense_version = static_cast<uint32_t>(number(text, "dense_format_version"));
        const std::string format = string(text, "expert_format");
        m.artifact.expert_format_kind =
            format == "swizzled_w4a16" ? ExpertFormatKind::SWIZZLED_W4A16 : ExpertFormatKind::UNKNOWN;
        m.artifact.expected_expert_version = static_cast<uint32_t>(number(text, "expert_format_version"));
        m.artifact.expert_sector_size = static_cast<uint32_t>(number(text, "expert_sector_size"));
        m.artifact.expected_expert_payload_bytes = static_cast<size_t>(number(text, "expert_payload_bytes"));
        m.dense_file_bytes = static_cast<size_t>(number(text, "dense_file_bytes"));
        m.num_layers = static_cast<uint32_t>(number(text, "num_layers"));
        m.experts_per_layer = static_cast<uint32_t>(number(text, "experts_per_layer"));
        if (has_key(text, "max_tensor_parallel"))
            m.max_tensor_parallel = static_cast<uint32_t>(number(text, "max_tensor_parallel"));
        m.validate();
        return m;
    }

    void validate() const {
        if (manifest_version != 1 && manifest_version != 2)
            throw std::invalid_argument("AeonModelManifest: unsupported manifest version " + std::to_string(manifest_version));
        if (model_family.empty() || architecture.empty() || weight_backend.empty())
            throw std::invalid_argument("AeonModelManifest: model identity is incomplete");
        const uint32_t sector = artifact.expert_sector_size;
        if (artifact.dense_filename.empty() || artifact.experts_filename.empty() || artifact.index_filename.empty() ||
            artifact.expected_dense_version == 0 || artifact.expert_format_kind == ExpertFormatKind::UNKNOWN ||
            artifact.expected_expert_version == 0 || sector == 0 || (sector & (sector - 1)) != 0 ||
            artifact.expected_expert_payload_bytes == 0)
            throw std::invalid_argument("AeonModelManifest: artifact identity is incomplete");
        if (weight_backend != ExpertBackendRegistry::resolve(artifact.expert_format_kind).name)
            throw std::invalid_argument("AeonModelManifest: weight backend does not match expert format kind");
        if (dense_file_bytes == 0 || num_layers == 0 || experts_per_layer == 0)
            throw std::invalid_argument("AeonModelManifest: dense size and catalog dimensions must be non-zero");
        if (artifact.expected_expert_payload_bytes % sector != 0)
            throw std::invalid_argument("AeonModelManifest: expert payload is not a multiple of the sector size");
    }

    void validate_loaded(const ExpertFormatDescriptor& loaded, size_t loaded_dense_file_bytes) const {
        validate();
        if (loaded_dense_file_bytes != dense_file_bytes)
            throw std::runtime_error("AeonModelManifest: dense file size does not match the manifest");
        if (loaded.kind != artifact.expert_format_kind || loaded.version != artifact.expected_expert_version ||
            loaded.sector_size != artifact.expert_sector_size ||
            loaded.payload_bytes != artifact.expected_expert_payload_bytes || loaded.num_layers != num_layers ||
            loaded.experts_per_layer != experts_per_layer || loaded.shard_count != max_tensor_parallel)
            throw std::runtime_error("AeonModelManifest: loaded artifact identity does not match the manifest");
    }

private:
    static size_t value_start(const std::string& text, const std::string& key) {
        const std::string quoted = "\"" + key + "\"";
        size_t at = text.find(quoted);
        if (at == std::string::npos) throw std::invalid_argument("AeonModelManifest: missing key '" + key + "'");
        at = text.find(':', at + quoted.size());
        if (at == std::string::npos) throw std::invalid_argument("AeonModelManifest: key '" + key + "' has no value");
        ++at;
        while (at < text.size() && (text[at] == ' ' || text[at] == '\t' || text[at] == '\n' || text[at] == '\r')) ++at;
        return at;
    }
    static bool has_key(const std::string& text, const std::string& key) {
        return text.find("\"" + key + "\"") != std::string::npos;
    }
    static uint64_t number(const std::string& text, const std::string& key) {
        size_t at = value_start(text, key);
        if (at >= text.size() || text[at] < '0' || text[at] > '9')
            throw std::invalid_argument("AeonModelManifest: key '" + key + "' is not an unsigned number");
        uint64_t value = 0;
        for (; at < text.size() && text[at] >= '0' && text[at] <= '9'; ++at) value = value * 10 + (text[at] - '0');
        return value;
    }
    static std::string string(const std::string& text, const std::string& key) {
        size_t at = value_start(text, key);
        if (at >= text.size() || text[at] != '"')
            throw std::invalid_argument("AeonModelManifest: key '" + key + "' is not a string");
        const size_t end = text.find('"', at + 1);
        if (end == std::string::npos) throw std::invalid_argument("AeonModelManifest: key '" + key + "' is not a string");
        return text.substr(at + 1, end - at - 1);
    }
};

// The reference's loader surface for this path (src/infrastructure/artifact/aeon_loader.hpp:
// 41-166): one model directory, dense tensors by name, experts by (layer, expert), plus the
// planned rank_slice. A directory with a manifest is opened through it: the backend the manifest
// names is resolved and checked against the artifact first, the files after, and the loaded
// identity against the manifest last (aeon_loader.hpp:43-78).
class AeonModelLoader {
public:
    using Artifact = AeonArtifactSpec;

    void open_model(const std::string& model_dir) {
        const std::string manifest_path = model_dir + "/model_manifest.json";
        std::ifstream probe(manifest_path);
        if (probe.is_open()) {
            probe.close();
            open_model(model_dir, AeonModelManifest::load_from_json(manifest_path));
            return;
        }
        open_model(model_dir, Artifact{});
    }
    void open_model(const std::string& model_dir, const Artifact& artifact) {
        const uint32_t sector = artifact.expert_sector_size;
        if (artifact.dense_filename.empty() || artifact.experts_filename.empty() || artifact.index_filename.empty() ||
            artifact.expected_dense_version == 0 || sector == 0 || (sector & (sector - 1)) != 0)
            throw std::invalid_argument("AeonModelLoader: artifact specification is incomplete");
        dense_.open(model_dir + "/" + artifact.dense_filename, artifact.expected_dense_version);
        experts_.open(model_dir + "/" + artifact.index_filename, model_dir + "/" + artifact.experts_filename,
                      artifact.expected_expert_version, artifact.expected_expert_payload_bytes);
        model_dir_ = model_dir;
    }
    void open_model(const std::string& model_dir, const AeonModelManifest& manifest) {
        manifest.validate();
        const ExpertBackendDescriptor& backend = ExpertBackendRegistry::resolve(manifest.weight_backend);
        if (backend.format_kind != manifest.artifact.expert_format_kind)
            throw std::invalid_argument("AeonModelLoader: manifest backend does not match its artifact format");
        open_model(model_dir, manifest.artifact);
        try {
            backend.validate_format(experts_.format());
            manifest.validate_loaded(experts_.format(), dense_.file_size());
        } catch (...) {
            dense_.close();
            experts_.close();
            model_dir_.clear();
            throw;
        }
    }

    const std::string& model_dir() const noexcept { return model_dir_; }
    bool has_tensor(const std::string& name) const { return dense_.has_tensor(name); }
    const LoadedTensor& get_tensor(const std::string& name) const { return dense_.get_tensor(name); }
    const ExpertFormatDescriptor& expert_format() const noexcept { return experts_.format(); }
    uint32_t max_tensor_parallel() const noexcept { return experts_.format().shard_count; }
    AeonExpertContainer::Location get_expert_location(uint32_t layer, uint32_t expert) const {
        return experts_.get_expert_location(layer, expert);
    }
    const uint8_t* get_expert_data(uint32_t layer, uint32_t expert) const { return experts_.get_expert_data(layer, expert); }
    AeonExpertContainer::Location rank_slice(uint32_t layer, uint32_t expert, uint32_t tp, uint32_t rank) const {
        return experts_.rank_slice(layer, expert, tp, rank);
    }
    const AeonExpertContainer& experts() const noexcept { return experts_; }
    const AeonDenseContainer& dense() const noexcept { return dense_; }

private:
    std::string model_dir_;
    AeonDenseContainer dense_;
    AeonExpertContainer experts_;
};

// ---------------------------------------------------------------------------------------------
// Device dispatch helpers with the reference's names.
// ---------------------------------------------------------------------------------------------
inline void dispatch_router(aeon_b200_ctx* ctx, const void* activation, int activation_stride, const void* gate_weight,
                            const float* gate_bias, const int64_t* tid2eid, const int32_t* device_token_ids,
                            float* topk_weights, int32_t* topk_indices, int count, void* stream) {
    check_status(aeon_b200_router_topk(ctx, activation, activation_stride, gate_weight, gate_bias, tid2eid,
                                       device_token_ids, count, topk_weights, topk_indices, nullptr, stream));
}

inline void dispatch_expert_permutation(aeon_b200_ctx* ctx, const int* topk_indices, int token_count, int slots,
                                        int expert_count, int* expert_offsets, int* token_indices,
                                        int* draw_indices, const float* weights, float* weights_by_position,
                                        void* stream) {
    check_status(aeon_b200_expert_permutation(ctx, topk_indices, token_count, slots, expert_count, expert_offsets,
                                              token_indices, draw_indices, weights, weights_by_position, stream));
}

// ---------------------------------------------------------------------------------------------
// The executor seam and its B200 implementation.
// ---------------------------------------------------------------------------------------------
// 16-bit activation element (fp16 or bf16 bits, as the configuration's act_dtype says): the
// reference's `half`. The accumulator is fp32 here where the reference's is fp16; that and
// hipStream_t -> a stream handle are the only type differences of the seam
// (src/architecture/deepseek_v4/layer/v4_layer_body_moe.hpp:32-112).
using act16 = uint16_t;

class V4RoutedExpertExecutor {
public:
    virtual ~V4RoutedExpertExecutor() = default;
    virtual void on_routing_ready(uint32_t layer_id, uint32_t position, const std::vector<int32_t>& ids,
                                  const std::vector<float>& weights) {
        (void)layer_id; (void)position; (void)ids; (void)weights;
    }
    // A layer-wide dispatch; the default is the per-token sequence.
    virtual void on_routing_ready_batch(uint32_t layer_id, uint32_t first_position,
                                        const std::vector<std::vector<int32_t>>& ids,
                                        const std::vector<std::vector<float>>& weights) {
        for (size_t i = 0; i < ids.size(); ++i)
            on_routing_ready(layer_id, first_position + static_cast<uint32_t>(i), ids[i], weights[i]);
    }
    // moe_accum += sum_k w_k * W2_k * clamped_swiglu(W1_k x, W3_k x); it holds the shared expert's
    // output on entry. The routed ids are the ones the matching on_routing_ready announced.
    virtual void accumulate_routed(uint32_t layer_id, uint32_t position, const act16* expert_input,
                                   const float* expert_weights, float* moe_accum) = 0;
    // The chunk-wide form; the default is the per-token sequence, so token_count == 1 reproduces
    // accumulate_routed.
    virtual void accumulate_routed_batch(uint32_t layer_id, uint32_t first_position, uint32_t token_count,
                                         const act16* batch_input, int input_stride, const int* batch_ids,
                                         int ids_stride, const float* batch_weights, int weights_stride,
                                         float* batch_output, int output_stride) {
        (void)batch_ids; (void)ids_stride;
        for (uint32_t token = 0; token < token_count; ++token)
            accumulate_routed(layer_id, first_position + token, batch_input + static_cast<size_t>(token) * input_stride,
                              batch_weights + static_cast<size_t>(token) * weights_stride,
                              batch_output + static_cast<size_t>(token) * output_stride);
    }
    virtual void on_routed_consumed(uint32_t layer_id, uint32_t position) { (void)layer_id; (void)position; }
};

// Borrows pool, registry and (optionally) the expert container; owns its context, the device
// copies of the layer's slot table and routed ids, and the staging of the miss path. HBM-first:
// with every expert resident each request is a hot hit and nothing is copied. Otherwise the
// layer's misses are deduplicated, then submitted together: each payload goes from the
// memory-mapped container through one of a ring of pinned staging buffers to its pool slot on the
// cold-upload stream, ordered after the compute work that may still read the evicted expert,
// and the compute stream waits on one event for the whole set -- the shape of the reference's
// tiered supply (src/architecture/deepseek_v4/moe/v4_expert_supply.hpp:202-258,
// src/infrastructure/expert/transport/tiered_expert_supply.hpp) without its host-RAM warm tier
// and NVMe reader. Decode-sized chunks go to the streaming kernels, larger ones to the grouped
// tcgen05 path.
class V4TieredExpertExecutor final : public V4RoutedExpertExecutor, public ExpertLeaseHolder {
public:
    static constexpr uint32_t kDecodeChunk = 128;
    static constexpr uint32_t kStagingBuffers = 4;

    // Every stream-ordered operation on one caller-supplied stream (uploads included).
    V4TieredExpertExecutor(const aeon_b200_moe_config& cfg, int device, uint32_t max_chunk,
                           UnifiedVRAMExpertPool& pool, ExpertRegistry& registry,
                           const AeonExpertContainer* container, void* compute_stream, uint32_t first_layer = 0)
        : cfg_(cfg), pool_(pool), registry_(registry), container_(container), stream_(compute_stream),
          upload_stream_(nullptr), first_layer_(first_layer) {
        init(device, max_chunk);
    }
    // Kernels on streams.compute, miss uploads on streams.sdma_cold (asynchronous supply).
    V4TieredExpertExecutor(const aeon_b200_moe_config& cfg, int device, uint32_t max_chunk,
                           UnifiedVRAMExpertPool& pool, ExpertRegistry& registry,
                           const AeonExpertContainer* container, const DeviceStreams& streams,
                           uint32_t first_layer = 0)
        : cfg_(cfg), pool_(pool), registry_(registry), container_(container), stream_(streams.compute),
          upload_stream_(streams.sdma_cold), first_layer_(first_layer) {
        init(device, max_chunk);
    }
    ~V4TieredExpertExecutor() override {
        if (ctx_) (void)aeon_b200_ctx_destroy(ctx_);
        if (d_slot_table_) (void)aeon_b200_device_free(d_slot_table_);
        if (d_ids_) (void)aeon_b200_device_free(d_ids_);
        for (Staging& st : staging_) {
            if (st.pinned) (void)aeon_b200_host_free_pinned(st.pinned);
            if (st.done) (void)aeon_b200_event_destroy(st.done);
        }
        if (compute_mark_) (void)aeon_b200_event_destroy(compute_mark_);
        if (uploads_done_) (void)aeon_b200_event_destroy(uploads_done_);
    }

    void on_routing_ready(uint32_t layer_id, uint32_t position, const std::vector<int32_t>& ids,
                          const std::vector<float>& weights) override {
        (void)weights;
        if (ids.size() != static_cast<size_t>(cfg_.top_k))
            throw std::invalid_argument("V4TieredExpertExecutor: expected " + std::to_string(cfg_.top_k) +
                                        " routed experts, got " + std::to_string(ids.size()));
        begin_dispatch(layer_id, position, 1);
        for (int32_t id : ids) request(layer_id, id);
        submit_transfers();
        publish_slot_table(layer_id);
        publish_ids(ids.data(), ids.size());
        batch_draws_ += ids.size();
    }

    void on_routing_ready_batch(uint32_t layer_id, uint32_t first_position,
                                const std::vector<std::vector<int32_t>>& ids,
                                const std::vector<std::vector<float>>& weights) override {
        (void)weights;
        if (ids.empty())
            throw std::invalid_argument("V4TieredExpertExecutor: a layer-wide dispatch needs at least one token");
        if (ids.size() > max_chunk_)
            throw std::invalid_argument("V4TieredExpertExecutor: the dispatch exceeds the executor's chunk size");
        begin_dispatch(layer_id, first_position, static_cast<uint32_t>(ids.size()));
        std::vector<uint8_t> seen(registry_.experts_per_layer, 0);
        flat_ids_.clear();
        for (const auto& row : ids) {
            if (row.size() != static_cast<size_t>(cfg_.top_k))
                throw std::invalid_argument("V4TieredExpertExecutor: every token needs top_k routed experts");
            for (int32_t id : row) {
                if (id < 0 || static_cast<uint32_t>(id) >= registry_.experts_per_layer)
                    throw std::out_of_range("V4TieredExpertExecutor: routed expert id out of range");
                if (!seen[id]) { seen[id] = 1; request(layer_id, id); }   // the layer's union, once
                flat_ids_.push_back(id);
                ++batch_draws_;
            }
        }
        submit_transfers();
        publish_slot_table(layer_id);
        publish_ids(flat_ids_.data(), flat_ids_.size());
    }

    void accumulate_routed(uint32_t layer_id, uint32_t position, const act16* expert_input,
                           const float* expert_weights, float* moe_accum) override {
        accumulate_routed(layer_id, position, expert_input,
                          d_ids_ + static_cast<size_t>(checked_row(layer_id, position)) * cfg_.top_k, expert_weights,
                          moe_accum);
    }
    // The same with the token's routed ids already on the device (no host round trip of the routing).
    void accumulate_routed(uint32_t layer_id, uint32_t position, const act16* expert_input, const int* expert_ids_device,
                           const float* expert_weights, float* moe_accum) {
        (void)checked_row(layer_id, position);
        check_status(aeon_b200_moe_decode(ctx_, pool_.d_experts, d_slot_table_, expert_input, cfg_.hidden,
                                          expert_ids_device, expert_weights, 1, moe_accum, cfg_.hidden, 0, stream_));
    }

    // batch_ids: the chunk's ids on the device, [token, top_k]; nullptr uses the ids the matching
    // on_routing_ready_batch announced.
    void accumulate_routed_batch(uint32_t layer_id, uint32_t first_position, uint32_t token_count,
                                 const act16* batch_input, int input_stride, const int* batch_ids, int ids_stride,
                                 const float* batch_weights, int weights_stride, float* batch_output,
                                 int output_stride) override {
        if (token_count == 0) return;
        if (!dispatched_ || current_layer_ != layer_id || first_position != first_position_ ||
            token_count != token_count_)
            throw std::logic_error("V4TieredExpertExecutor: accumulate_routed_batch without a matching batch dispatch");
        if ((batch_ids != nullptr && ids_stride != cfg_.top_k) || weights_stride != cfg_.top_k)
            throw std::invalid_argument("V4TieredExpertExecutor: batch ids and weights must be [token, top_k]");
        const int* ids = batch_ids != nullptr ? batch_ids : d_ids_;
        if (token_count <= kDecodeChunk) {
            check_status(aeon_b200_moe_decode(ctx_, pool_.d_experts, d_slot_table_, batch_input, input_stride, ids,
                                              batch_weights, static_cast<int>(token_count), batch_output,
                                              output_stride, 0, stream_));
        } else {
            check_status(aeon_b200_moe_prefill(ctx_, pool_.d_experts, d_slot_table_, batch_input, input_stride, ids,
                                               batch_weights, static_cast<int>(token_count), batch_output,
                                               output_stride, 0, stream_));
        }
    }

    void release_leases() override {
        for (uint32_t gid : leases_) registry_.release_lease(gid);
        leases_.clear();
    }
    size_t outstanding_leases() const noexcept override { return leases_.size(); }
    uint64_t batch_draws() const noexcept { return batch_draws_; }
    uint64_t batch_distinct() const noexcept { return batch_distinct_; }
    uint64_t uploads() const noexcept { return uploads_; }
    uint32_t last_dispatch_tokens() const noexcept { return token_count_; }
    aeon_b200_ctx* context() const noexcept { return ctx_; }
    void check_device() { check_status(aeon_b200_ctx_check(ctx_, stream_)); }

private:
    struct Staging {
        void* pinned{nullptr};
        void* done{nullptr};      // recorded after the buffer's last upload
        bool in_flight{false};
    };
    struct Miss {
        uint32_t slot, local_layer, expert;
        uint64_t operation_id;
    };

    void init(int device, uint32_t max_chunk) {
        if (registry_.vram_capacity == 0)
            throw std::invalid_argument("V4TieredExpertExecutor: the VRAM expert pool has no slots");
        if (registry_.experts_per_layer != static_cast<uint32_t>(cfg_.experts))
            throw std::invalid_argument("V4TieredExpertExecutor: registry and config disagree on the expert count");
        if (max_chunk == 0) throw std::invalid_argument("V4TieredExpertExecutor: the chunk size must be positive");
        device_ = device;
        max_chunk_ = max_chunk;
        check_status(aeon_b200_ctx_create(&cfg_, device, static_cast<int>(std::min(max_chunk, kDecodeChunk)), &ctx_));
        void* raw = nullptr;
        check_status(aeon_b200_device_alloc(static_cast<uint64_t>(cfg_.experts) * sizeof(int32_t), device, &raw));
        d_slot_table_ = static_cast<int32_t*>(raw);
        check_status(aeon_b200_device_alloc(static_cast<uint64_t>(max_chunk) * cfg_.top_k * sizeof(int32_t), device, &raw));
        d_ids_ = static_cast<int32_t*>(raw);
        if (upload_stream_ != nullptr) {
            DeviceScope scope(device);
            for (Staging& st : staging_) {
                check_status(aeon_b200_host_alloc_pinned(pool_.format().payload_bytes, &st.pinned));
                check_status(aeon_b200_event_create(&st.done));
            }
            check_status(aeon_b200_event_create(&compute_mark_));
            check_status(aeon_b200_event_create(&uploads_done_));
        }
    }
    void begin_dispatch(uint32_t layer_id, uint32_t first_position, uint32_t tokens) {
        if (layer_id < first_layer_ || layer_id - first_layer_ >= registry_.num_layers)
            throw std::out_of_range("V4TieredExpertExecutor: layer outside this stage");
        current_layer_ = layer_id;
        first_position_ = first_position;
        token_count_ = tokens;
        dispatched_ = true;
        misses_.clear();
    }
    uint32_t checked_row(uint32_t layer_id, uint32_t position) const {
        if (!dispatched_ || current_layer_ != layer_id)
            throw std::logic_error("V4TieredExpertExecutor: accumulate_routed without a matching on_routing_ready");
        if (position < first_position_ || position - first_position_ >= token_count_)
            throw std::out_of_range("V4TieredExpertExecutor: token index past the batch's token count");
        return position - first_position_;
    }
    void request(uint32_t layer_id, int32_t expert) {
        if (expert < 0 || static_cast<uint32_t>(expert) >= registry_.experts_per_layer)
            throw std::out_of_range("V4TieredExpertExecutor: routed expert id out of range");
        const uint32_t local = layer_id - first_layer_;
        ExpertRequestReservation r = registry_.reserve_request(local, static_cast<uint32_t>(expert));
        leases_.push_back(r.global_expert_id);
        ++batch_distinct_;
        if (r.kind == ExpertRequestKind::COLD_MISS) {
            if (container_ == nullptr) {
                registry_.fail_request(r.operation_id);
                leases_.pop_back();
                throw std::logic_error("V4TieredExpertExecutor: a routed expert is not resident and no container was given");
            }
            misses_.push_back(Miss{static_cast<uint32_t>(r.vram_slot), local, static_cast<uint32_t>(expert), r.operation_id});
        }
    }
    // The dispatch's misses, together. Without an upload stream: stream-ordered copies on the compute
    // stream. With one: pinned staging ring -> pool slot on the upload stream, which first waits for
    // the compute work enqueued so far (it may still read an expert this dispatch evicts); the
    // compute stream then waits for the whole set.
    void submit_transfers() {
        if (misses_.empty()) return;
        const size_t bytes = pool_.format().payload_bytes;
        if (upload_stream_ == nullptr) {
            for (const Miss& m : misses_) {
                pool_.upload_from_host_expert(m.slot, container_->get_expert_data(m.local_layer, m.expert), stream_);
                registry_.complete_request(m.operation_id);
            }
        } else {
            check_status(aeon_b200_event_record(compute_mark_, stream_));
            check_status(aeon_b200_stream_wait_event(upload_stream_, compute_mark_));
            for (const Miss& m : misses_) {
                Staging& st = staging_[next_staging_];
                next_staging_ = (next_staging_ + 1) % kStagingBuffers;
                if (st.in_flight) check_status(aeon_b200_event_synchronize(st.done));   // its last upload has left
                std::memcpy(st.pinned, container_->get_expert_data(m.local_layer, m.expert), bytes);
                check_status(aeon_b200_copy_to_device_async(pool_.get_slot_base(m.slot), st.pinned, bytes, upload_stream_));
                check_status(aeon_b200_event_record(st.done, upload_stream_));
                st.in_flight = true;
            }
            check_status(aeon_b200_event_record(uploads_done_, upload_stream_));
            check_status(aeon_b200_stream_wait_event(stream_, uploads_done_));
            for (const Miss& m : misses_) registry_.complete_request(m.operation_id);
        }
        uploads_ += misses_.size();
        misses_.clear();
    }
    void publish_slot_table(uint32_t layer_id) {
        host_table_ = registry_.layer_slot_table(layer_id - first_layer_);
        // stream-ordered copy from pageable memory (staged before the call returns): the kernels
        // that follow on the same stream read the new table
        check_status(aeon_b200_copy_to_device_async(d_slot_table_, host_table_.data(),
                                                    host_table_.size() * sizeof(int32_t), stream_));
    }
    void publish_ids(const int32_t* ids, size_t count) {
        check_status(aeon_b200_copy_to_device_async(d_ids_, ids, count * sizeof(int32_t), stream_));
    }

    aeon_b200_moe_config cfg_;
    UnifiedVRAMExpertPool& pool_;
    ExpertRegistry& registry_;
    const AeonExpertContainer* container_;
    void* stream_;
    void* upload_stream_;
    uint32_t first_layer_;
    aeon_b200_ctx* ctx_{nullptr};
    int32_t* d_slot_table_{nullptr};
    int32_t* d_ids_{nullptr};
    int device_{0};
    uint32_t max_chunk_{0};
    Staging staging_[kStagingBuffers];
    uint32_t next_staging_{0};
    void* compute_mark_{nullptr};
    void* uploads_done_{nullptr};
    std::vector<Miss> misses_;
    std::vector<int32_t> host_table_, flat_ids_;
    std::vector<uint32_t> leases_;
    uint32_t current_layer_{0}, first_position_{0}, token_count_{0};
    bool dispatched_{false};
    uint64_t batch_draws_{0}, batch_distinct_{0}, uploads_{0};
};

// ---------------------------------------------------------------------------------------------
// One rank's membership of a multi-GPU group: the communicator the reference plans as
// TensorParallelGroup (MULTI_GPU_EXECUTION_PLAN.md:189-235), over the library's NCCL entry points.
// One rank calls unique_id(), the bytes travel by any host channel, every rank constructs its
// member with them (a collective call).
// ---------------------------------------------------------------------------------------------
class ParallelGroup {
public:
    using UniqueId = std::array<uint8_t, AEON_B200_GROUP_ID_BYTES>;

    static UniqueId unique_id() {
        UniqueId id{};
        check_status(aeon_b200_group_unique_id(id.data()));
        return id;
    }
    ParallelGroup(const UniqueId& id, int rank, int world, int device) {
        check_status(aeon_b200_group_create(id.data(), rank, world, device, &group_));
    }
    ~ParallelGroup() {
        if (group_) (void)aeon_b200_group_destroy(group_);
    }
    ParallelGroup(const ParallelGroup&) = delete;
    ParallelGroup& operator=(const ParallelGroup&) = delete;

    int rank() const noexcept { return aeon_b200_group_rank(group_); }
    int world() const noexcept { return aeon_b200_group_world(group_); }

    // expert parallel: every rank's activation rows to every rank, rank order
    void dispatch(const act16* x_local, int tokens_local, int hidden, act16* x_all, void* stream) {
        check_status(aeon_b200_ep_dispatch(group_, x_local, tokens_local, static_cast<int64_t>(hidden) * 2, x_all, stream));
    }
    // the same with the routing every rank computed for its own tokens (one grouped call)
    void dispatch_routed(const act16* x_local, int tokens_local, int hidden, act16* x_all, const int32_t* ids_local,
                         const float* weights_local, int top_k, int32_t* ids_all, float* weights_all, void* stream) {
        check_status(aeon_b200_ep_dispatch_routed(group_, x_local, tokens_local, static_cast<int64_t>(hidden) * 2, x_all,
                                                  ids_local, weights_local, top_k, ids_all, weights_all, stream));
    }
    // expert parallel: partial rows to the ranks that own the tokens, then add in rank order
    void exchange(const float* partial, int tokens_local, int hidden, float* recv, void* stream) {
        check_status(aeon_b200_ep_exchange(group_, partial, tokens_local, hidden, recv, stream));
    }
    void combine(float* out, int64_t out_stride, const float* recv, int tokens_local, int hidden, void* stream) {
        check_status(aeon_b200_ep_combine(out, out_stride, recv, world(), tokens_local, hidden, stream));
    }
    // tensor parallel: sum of the partial outputs, each rank keeps its tokens' rows
    void reduce(const float* partial, int tokens_local, int hidden, float* out_local, void* stream) {
        check_status(aeon_b200_tp_reduce(group_, partial, tokens_local, hidden, out_local, stream));
    }
    // pipeline: the stage hand-off
    void send(const void* rows, uint64_t bytes, int peer, void* stream) {
        check_status(aeon_b200_pp_send(group_, rows, bytes, peer, stream));
    }
    void recv(void* rows, uint64_t bytes, int peer, void* stream) {
        check_status(aeon_b200_pp_recv(group_, rows, bytes, peer, stream));
    }
    aeon_b200_group* handle() const noexcept { return group_; }

private:
    aeon_b200_group* group_{nullptr};
};

}  // namespace aeon::core
