// extern "C" surface of libaeon_b200.so: configuration, geometry, host swizzle, context,
// pool, and the entry points that forward to the kernel launchers.
#include "common.cuh"

#include <cstring>
#include <vector>

namespace aeon_b200 {

namespace {
thread_local std::string g_last_error;
}

void set_last_error(const std::string& message) { g_last_error = message; }

void validate_config(const aeon_b200_moe_config& c) {
    require(c.hidden > 0 && c.intermediate > 0, "config: hidden and intermediate must be positive");
    // 256 = four 64-column k-blocks of the grouped path; a tensor-parallel shard of the
    // intermediate dimension (2048 / 8 = 256) is a legal "expert" of its own. The decode
    // kernels additionally need one of their compiled (hidden, intermediate) instances.
    require(c.hidden % 256 == 0 && c.intermediate % 256 == 0,
            "config: hidden and intermediate must be multiples of 256");
    require(c.experts > 0 && c.experts <= 1024 && c.experts % 32 == 0,
            "config: experts must be a multiple of 32 in [32, 1024]");
    require(c.top_k > 0 && c.top_k <= 32 && c.top_k <= c.experts, "config: top_k must be in [1, 32]");
    require(c.group_size == 32 || c.group_size == 128, "config: group_size must be 32 or 128");
    require(c.act_dtype == AEON_B200_F16 || c.act_dtype == AEON_B200_BF16, "config: unknown act_dtype");
    require(c.score_fn == AEON_B200_SCORE_SQRT_SOFTPLUS || c.score_fn == AEON_B200_SCORE_SIGMOID,
            "config: unknown score_fn");
    require(c.swiglu_limit > 0.f, "config: swiglu_limit must be positive");
    // The decode kernels are written for the reference's swizzle configurations
    // (W1/W3: 4 rows x 8 lanes, W2: 8 rows x 4 lanes per 512-byte wave line).
    require(c.w13_rpw == 4 && c.w13_lpr == 8 && c.w2_rpw == 8 && c.w2_lpr == 4,
            "config: swizzle must be rpw/lpr = 4/8 for W1,W3 and 8/4 for W2");
}

static MatrixGeom matrix_geom(int rows, int cols, int rpw, int lpr, int group) {
    MatrixGeom m{};
    m.rows = rows;
    m.cols = cols;
    m.rpw = rpw;
    m.lpr = lpr;
    m.iters = (cols / 32) / lpr;
    m.block_bytes = m.iters * 512;
    m.block_scale_bytes = m.iters * 32 / (group / 32) * 2;
    return m;
}

ExpertGeom make_geom(const aeon_b200_moe_config& c) {
    validate_config(c);
    ExpertGeom g{};
    g.group = c.group_size;
    g.w1 = matrix_geom(c.intermediate, c.hidden, c.w13_rpw, c.w13_lpr, c.group_size);
    g.w3 = g.w1;
    g.w2 = matrix_geom(c.hidden, c.intermediate, c.w2_rpw, c.w2_lpr, c.group_size);
    uint64_t cursor = 0;
    auto place = [&](MatrixGeom& m) {
        const uint64_t weights = static_cast<uint64_t>(m.rows) * m.cols;
        m.packed_offset = cursor;
        cursor = (cursor + weights / 2 + 4095) / 4096 * 4096;
        m.scale_offset = cursor;
        cursor = (cursor + weights / c.group_size * 2 + 4095) / 4096 * 4096;
    };
    place(g.w1);
    place(g.w2);
    place(g.w3);
    g.payload_bytes = cursor;
    return g;
}

namespace {

void check_swizzle_args(int N, int K, int rpw, int lpr, int group) {
    // Same rules as validate_w4a16_swizzle
    // (src/backend/swizzled_w4a16/kernels/aeon_w4a16_swizzle.hpp:36-43) plus the group rule.
    require(rpw > 0 && lpr > 0 && rpw * lpr == 32, "swizzle: rpw * lpr must be 32");
    require(N > 0 && K > 0 && N % rpw == 0 && K % 32 == 0 && (K / 32) % lpr == 0,
            "swizzle: N must divide by rpw and K/32 by lpr");
    require(group >= 32 && group % 32 == 0 && lpr % (group / 32) == 0,
            "swizzle: group must be a multiple of 32 whose atoms fit one row's lanes");
}

inline uint32_t permute_word(uint32_t source) {
    // destination nibble p holds source nibble {0,2,4,6,1,3,5,7}[p]
    uint32_t out = 0;
    for (int p = 0; p < 8; ++p) {
        const int from = (p < 4) ? 2 * p : 2 * (p - 4) + 1;
        out |= ((source >> (4 * from)) & 0xFu) << (4 * p);
    }
    return out;
}

inline uint32_t unpermute_word(uint32_t source) {
    uint32_t out = 0;
    for (int p = 0; p < 8; ++p) {
        const int to = (p < 4) ? 2 * p : 2 * (p - 4) + 1;
        out |= ((source >> (4 * p)) & 0xFu) << (4 * to);
    }
    return out;
}

}  // namespace

// Walks every 16-byte atom once; `forward` copies checkpoint order -> swizzled order.
void relayout_w4a16(const uint32_t* src_packed, const uint16_t* src_scale, uint32_t* dst_packed,
              uint16_t* dst_scale, int N, int K, int rpw, int lpr, int group, bool forward) {
    const int atoms_per_row = K / 32;
    const int iters = atoms_per_row / lpr;
    const int apg = group / 32;
    const int groups_per_row = K / group;
    for (int row = 0; row < N; ++row) {
        const size_t block = static_cast<size_t>(row / rpw);
        const int rib = row % rpw;
        for (int a = 0; a < atoms_per_row; ++a) {
            const size_t atom = (block * iters + a / lpr) * 32 + static_cast<size_t>(rib) * lpr + a % lpr;
            const size_t linear = static_cast<size_t>(row) * atoms_per_row + a;
            for (int w = 0; w < 4; ++w) {
                if (forward) dst_packed[atom * 4 + w] = permute_word(src_packed[linear * 4 + w]);
                else dst_packed[linear * 4 + w] = unpermute_word(src_packed[atom * 4 + w]);
            }
            if (a % apg == 0) {
                const size_t swz = atom / apg;
                const size_t lin = static_cast<size_t>(row) * groups_per_row + a / apg;
                if (forward) dst_scale[swz] = src_scale[lin];
                else dst_scale[lin] = src_scale[swz];
            }
        }
    }
}

namespace {

template <class T>
T* device_alloc(aeon_b200_ctx* ctx, size_t count, uint64_t& total, const char* name) {
    total += count * sizeof(T);
    return static_cast<T*>(ctx_device_alloc(ctx, count * sizeof(T), name));
}

cudaStream_t as_stream(void* s) { return static_cast<cudaStream_t>(s); }

struct DeviceGuard {
    int previous{-1};
    explicit DeviceGuard(int device) {
        AEON_CUDA_CHECK(cudaGetDevice(&previous));
        if (previous != device) AEON_CUDA_CHECK(cudaSetDevice(device));
        else previous = -1;
    }
    ~DeviceGuard() {
        if (previous >= 0) (void)cudaSetDevice(previous);
    }
};

}  // namespace

void* ctx_device_alloc(aeon_b200_ctx* ctx, size_t bytes, const char* name) {
    void* p = nullptr;
    AEON_CUDA_CHECK(cudaMalloc(&p, bytes + (kBoundsChecked ? kGuardBytes : 0)));
    if (kBoundsChecked) {
        uint8_t* guard = static_cast<uint8_t*>(p) + bytes;
        const cudaError_t e = cudaMemset(guard, kGuardPattern, kGuardBytes);
        if (e != cudaSuccess) {
            (void)cudaFree(p);
            AEON_CUDA_CHECK(e);
        }
        if (ctx->guards == nullptr) ctx->guards = new std::vector<ScratchGuard>();
        ctx->guards->push_back(ScratchGuard{p, guard, name});
    }
    return p;
}

void ctx_device_free(aeon_b200_ctx* ctx, void* base) noexcept {
    if (base == nullptr) return;
    if (ctx->guards != nullptr)
        for (size_t i = 0; i < ctx->guards->size(); ++i)
            if ((*ctx->guards)[i].base == base) {
                ctx->guards->erase(ctx->guards->begin() + static_cast<std::ptrdiff_t>(i));
                break;
            }
    (void)cudaFree(base);
}

namespace {

void free_ctx_buffers(aeon_b200_ctx* c) {
    void* bufs[] = {c->d_xperm, c->d_logits, c->d_offsets, c->d_token_idx, c->d_draw_idx, c->d_wpos,
                    c->d_entries, c->d_counts, c->d_hidden_hi, c->d_hidden_lo, c->d_contrib,
                    c->d_error, c->d_sh_hi, c->d_sh_mid, c->d_sh_lo};
    for (void* b : bufs) ctx_device_free(c, b);
    free_prefill_scratch(c);
    free_shared_tc_scratch(c);
    if (c->timing_events) {
        for (cudaEvent_t e : *c->timing_events) (void)cudaEventDestroy(e);
        delete c->timing_events;
        c->timing_events = nullptr;
    }
    delete c->guards;
    c->guards = nullptr;
    if (c->aux_fork) (void)cudaEventDestroy(c->aux_fork);
    if (c->aux_join) (void)cudaEventDestroy(c->aux_join);
    if (c->aux_stream) (void)cudaStreamDestroy(c->aux_stream);
    c->aux_fork = c->aux_join = nullptr;
    c->aux_stream = nullptr;
}

}  // namespace
}  // namespace aeon_b200

using namespace aeon_b200;

extern "C" {

const char* aeon_b200_last_error(void) { return g_last_error.c_str(); }
const char* aeon_b200_version(void) { return "aeon_b200 0.1 (sm_100a)"; }

int aeon_b200_config_preset(const char* name, aeon_b200_moe_config* out) {
    return guarded([&] {
        require(name && out, "aeon_b200_config_preset: null argument");
        aeon_b200_moe_config c{};
        c.w13_rpw = 4; c.w13_lpr = 8; c.w2_rpw = 8; c.w2_lpr = 4;
        c.swiglu_limit = 10.0f;
        c.renormalize = 1;
        c.experts = 256;
        c.intermediate = 2048;
        if (std::strcmp(name, "ref_dsv4") == 0) {
            c.hidden = 4096; c.top_k = 6; c.group_size = 32; c.act_dtype = AEON_B200_F16;
            c.score_fn = AEON_B200_SCORE_SQRT_SOFTPLUS; c.routed_scaling = 1.5f;
        } else if (std::strcmp(name, "baseline") == 0) {
            c.hidden = 7168; c.top_k = 8; c.group_size = 128; c.act_dtype = AEON_B200_BF16;
            c.score_fn = AEON_B200_SCORE_SIGMOID; c.routed_scaling = 1.0f;
        } else {
            throw StatusError(AEON_B200_ERR_INVALID_ARGUMENT,
                              std::string("aeon_b200_config_preset: unknown preset '") + name + "'");
        }
        *out = c;
    });
}

int aeon_b200_config_validate(const aeon_b200_moe_config* cfg) {
    return guarded([&] {
        require(cfg != nullptr, "aeon_b200_config_validate: null config");
        validate_config(*cfg);
    });
}

int aeon_b200_expert_layout_of(const aeon_b200_moe_config* cfg, aeon_b200_expert_layout* out) {
    return guarded([&] {
        require(cfg && out, "aeon_b200_expert_layout_of: null argument");
        const ExpertGeom g = make_geom(*cfg);
        out->payload_bytes = g.payload_bytes;
        out->w1_packed_offset = g.w1.packed_offset;
        out->w1_scale_offset = g.w1.scale_offset;
        out->w2_packed_offset = g.w2.packed_offset;
        out->w2_scale_offset = g.w2.scale_offset;
        out->w3_packed_offset = g.w3.packed_offset;
        out->w3_scale_offset = g.w3.scale_offset;
        const uint64_t w13 = static_cast<uint64_t>(cfg->hidden) * cfg->intermediate;
        out->w13_packed_bytes = w13 / 2;
        out->w13_scale_bytes = w13 / cfg->group_size * 2;
        out->w2_packed_bytes = w13 / 2;
        out->w2_scale_bytes = w13 / cfg->group_size * 2;
    });
}

int aeon_b200_swizzle_w4a16(const uint32_t* sp, const uint16_t* ss, uint32_t* dp, uint16_t* ds, int N,
                            int K, int rpw, int lpr, int group) {
    return guarded([&] {
        require(sp && ss && dp && ds, "aeon_b200_swizzle_w4a16: null pointer argument");
        check_swizzle_args(N, K, rpw, lpr, group);
        relayout_w4a16(sp, ss, dp, ds, N, K, rpw, lpr, group, true);
    });
}

int aeon_b200_unswizzle_w4a16(const uint32_t* sp, const uint16_t* ss, uint32_t* dp, uint16_t* ds, int N,
                              int K, int rpw, int lpr, int group) {
    return guarded([&] {
        require(sp && ss && dp && ds, "aeon_b200_unswizzle_w4a16: null pointer argument");
        check_swizzle_args(N, K, rpw, lpr, group);
        relayout_w4a16(sp, ss, dp, ds, N, K, rpw, lpr, group, false);
    });
}

int aeon_b200_ctx_create(const aeon_b200_moe_config* cfg, int device, int max_tokens,
                         aeon_b200_ctx** out) {
    return guarded([&] {
        require(cfg && out, "aeon_b200_ctx_create: null argument");
        require(max_tokens > 0 && max_tokens <= 4096, "aeon_b200_ctx_create: max_tokens must be in [1, 4096]");
        validate_config(*cfg);
        int count = 0;
        AEON_CUDA_CHECK(cudaGetDeviceCount(&count));
        require(device >= 0 && device < count, "aeon_b200_ctx_create: device index out of range");
        cudaDeviceProp prop{};
        AEON_CUDA_CHECK(cudaGetDeviceProperties(&prop, device));
        if (prop.major != 10) {
            throw StatusError(AEON_B200_ERR_UNSUPPORTED,
                              "aeon_b200_ctx_create: this library contains sm_100a code only and the "
                              "device is not compute capability 10.x");
        }
        DeviceGuard guard(device);
        aeon_b200_ctx* c = new aeon_b200_ctx();
        std::memset(c, 0, sizeof(*c));
        c->cfg = *cfg;
        c->geom = make_geom(*cfg);
        c->device = device;
        c->sm_count = prop.multiProcessorCount;
        c->max_tokens = max_tokens;
        c->timing_events = new std::vector<cudaEvent_t>();
        try {
            const size_t T = static_cast<size_t>(max_tokens);
            const size_t draws = T * cfg->top_k;
            uint64_t total = 0;
            c->d_xperm = device_alloc<__half>(c, T * cfg->hidden, total, "xperm");
            c->d_logits = device_alloc<float>(c, T * cfg->experts, total, "logits");
            c->d_offsets = device_alloc<int32_t>(c, cfg->experts + 1, total, "offsets");
            c->d_token_idx = device_alloc<int32_t>(c, draws, total, "token_idx");
            c->d_draw_idx = device_alloc<int32_t>(c, draws, total, "draw_idx");
            c->d_wpos = device_alloc<float>(c, draws, total, "wpos");
            c->d_entries = device_alloc<WorkEntry>(c, cfg->experts + draws / 8 + 1, total, "entries");
            c->d_counts = device_alloc<int32_t>(c, 4, total, "counts");
            c->d_hidden_hi = device_alloc<__half>(c, draws * cfg->intermediate, total, "hidden_hi");
            c->d_hidden_lo = device_alloc<__half>(c, draws * cfg->intermediate, total, "hidden_lo");
            c->d_contrib = device_alloc<float>(c, draws * cfg->hidden, total, "contrib");
            c->d_error = device_alloc<int32_t>(c, 1, total, "error");
            c->d_sh_hi = device_alloc<__half>(c, T * cfg->intermediate, total, "sh_hi");
            c->d_sh_mid = device_alloc<__half>(c, T * cfg->intermediate, total, "sh_mid");
            c->d_sh_lo = device_alloc<__half>(c, T * cfg->intermediate, total, "sh_lo");
            AEON_CUDA_CHECK(cudaMemset(c->d_error, 0, sizeof(int32_t)));
            AEON_CUDA_CHECK(cudaMemset(c->d_counts, 0, 4 * sizeof(int32_t)));
            AEON_CUDA_CHECK(cudaStreamCreateWithFlags(&c->aux_stream, cudaStreamNonBlocking));
            AEON_CUDA_CHECK(cudaEventCreateWithFlags(&c->aux_fork, cudaEventDisableTiming));
            AEON_CUDA_CHECK(cudaEventCreateWithFlags(&c->aux_join, cudaEventDisableTiming));
            c->scratch_bytes = total;
        } catch (...) {
            free_ctx_buffers(c);
            delete c;
            throw;
        }
        *out = c;
    });
}

int aeon_b200_ctx_destroy(aeon_b200_ctx* ctx) {
    return guarded([&] {
        if (!ctx) return;
        DeviceGuard guard(ctx->device);
        free_ctx_buffers(ctx);
        delete ctx;
    });
}

uint64_t aeon_b200_ctx_scratch_bytes(const aeon_b200_ctx* ctx) { return ctx ? ctx->scratch_bytes : 0; }
uint64_t aeon_b200_ctx_launches(const aeon_b200_ctx* ctx) { return ctx ? ctx->launches : 0; }

int aeon_b200_ctx_check(aeon_b200_ctx* ctx, void* stream) {
    return guarded([&] {
        require(ctx != nullptr, "aeon_b200_ctx_check: null context");
        DeviceGuard guard(ctx->device);
        AEON_CUDA_CHECK(cudaStreamSynchronize(as_stream(stream)));
        int32_t flag = 0;
        AEON_CUDA_CHECK(cudaMemcpy(&flag, ctx->d_error, sizeof(flag), cudaMemcpyDeviceToHost));
        if (flag != kErrNone) {
            AEON_CUDA_CHECK(cudaMemset(ctx->d_error, 0, sizeof(int32_t)));
            switch (flag) {
                case kErrWaitTimeout:
                    throw StatusError(AEON_B200_ERR_TIMEOUT, "device: a bounded pipeline wait ran out");
                case kErrExpertAbsent:
                    throw StatusError(AEON_B200_ERR_LOGIC,
                                      "device: a routed expert has no pool slot (slot_of_expert < 0)");
                case kErrBounds:
                    throw StatusError(AEON_B200_ERR_OUT_OF_RANGE,
                                      "device: an index left its buffer (bounds-checked build; the access was skipped)");
                default:
                    throw StatusError(AEON_B200_ERR_OUT_OF_RANGE,
                                      "device: an expert id, a hash-table entry or a pool slot is out of range");
            }
        }
        if (kBoundsChecked && ctx->guards != nullptr) {
            uint8_t host[kGuardBytes];
            for (const ScratchGuard& guard : *ctx->guards) {
                AEON_CUDA_CHECK(cudaMemcpy(host, guard.guard, kGuardBytes, cudaMemcpyDeviceToHost));
                for (size_t i = 0; i < kGuardBytes; ++i)
                    if (host[i] != kGuardPattern)
                        throw StatusError(AEON_B200_ERR_OUT_OF_RANGE,
                                          std::string("device: the guard region behind scratch buffer '") + guard.name +
                                              "' was overwritten at byte " + std::to_string(i));
            }
        }
    });
}

int aeon_b200_ctx_set_pool_slots(aeon_b200_ctx* ctx, int slots) {
    return guarded([&] {
        require(ctx != nullptr && slots >= 0, "aeon_b200_ctx_set_pool_slots: null context or negative slot count");
        ctx->pool_slots = slots;
    });
}

int aeon_b200_bounds_checked(void) { return kBoundsChecked ? 1 : 0; }

int aeon_b200_ctx_set_timing(aeon_b200_ctx* ctx, int enabled) {
    return guarded([&] {
        require(ctx != nullptr, "aeon_b200_ctx_set_timing: null context");
        ctx->timing_enabled = enabled ? 1 : 0;
    });
}

int aeon_b200_ctx_kernel_times(aeon_b200_ctx* ctx, void* stream, double* total_ms, int64_t* launches) {
    return guarded([&] {
        require(ctx && total_ms && launches, "aeon_b200_ctx_kernel_times: null argument");
        DeviceGuard guard(ctx->device);
        AEON_CUDA_CHECK(cudaStreamSynchronize(as_stream(stream)));
        std::vector<cudaEvent_t>& pool = *ctx->timing_events;
        for (size_t i = 0; i + 2 < ctx->timing_used; i += 3) {
            float a = 0.f, b = 0.f;
            AEON_CUDA_CHECK(cudaEventElapsedTime(&a, pool[i], pool[i + 1]));
            AEON_CUDA_CHECK(cudaEventElapsedTime(&b, pool[i + 1], pool[i + 2]));
            ctx->timing_ms[0] += a;
            ctx->timing_ms[1] += b;
            ctx->timing_launches[0] += 1;
            ctx->timing_launches[1] += 1;
        }
        ctx->timing_used = 0;
        for (int k = 0; k < 2; ++k) {
            total_ms[k] = ctx->timing_ms[k];
            launches[k] = ctx->timing_launches[k];
            ctx->timing_ms[k] = 0.0;
            ctx->timing_launches[k] = 0;
        }
    });
}

int aeon_b200_ctx_last_stats(aeon_b200_ctx* ctx, void* stream, int32_t* distinct, int32_t* entries) {
    return guarded([&] {
        require(ctx != nullptr, "aeon_b200_ctx_last_stats: null context");
        DeviceGuard guard(ctx->device);
        AEON_CUDA_CHECK(cudaStreamSynchronize(as_stream(stream)));
        int32_t counts[4] = {0, 0, 0, 0};
        AEON_CUDA_CHECK(cudaMemcpy(counts, ctx->d_counts, sizeof(counts), cudaMemcpyDeviceToHost));
        if (entries) *entries = counts[0];
        if (distinct) *distinct = counts[1];
    });
}

int aeon_b200_pool_create(uint64_t payload_bytes, uint32_t slots, int device, void** out) {
    return guarded([&] {
        require(out != nullptr, "aeon_b200_pool_create: null output");
        require(payload_bytes > 0 && payload_bytes % 4096 == 0,
                "aeon_b200_pool_create: payload_bytes must be a positive multiple of 4096");
        require(slots > 0, "aeon_b200_pool_create: the pool needs at least one slot");
        DeviceGuard guard(device);
        void* p = nullptr;
        AEON_CUDA_CHECK(cudaMalloc(&p, payload_bytes * slots));
        *out = p;
    });
}

int aeon_b200_pool_destroy(void* base, int device) {
    return guarded([&] {
        if (!base) return;
        DeviceGuard guard(device);
        AEON_CUDA_CHECK(cudaFree(base));
    });
}

int aeon_b200_pool_upload(void* base, uint64_t payload_bytes, uint32_t slot, const void* payload_host,
                          void* stream) {
    return guarded([&] {
        require(base && payload_host, "aeon_b200_pool_upload: null pointer argument");
        AEON_CUDA_CHECK(cudaMemcpyAsync(static_cast<uint8_t*>(base) + payload_bytes * slot, payload_host,
                                        payload_bytes, cudaMemcpyHostToDevice, as_stream(stream)));
    });
}

int aeon_b200_router_topk(aeon_b200_ctx* ctx, const void* x, int64_t x_stride, const void* gate,
                          const float* bias, const int64_t* hash_table, const int32_t* token_ids,
                          int tokens, float* topk_weights, int32_t* topk_ids, float* logits_out,
                          void* stream) {
    return guarded([&] {
        require(ctx != nullptr, "aeon_b200_router_topk: null context");
        DeviceGuard guard(ctx->device);
        launch_router(ctx, x, x_stride, gate, bias, hash_table, token_ids, tokens, topk_weights,
                      topk_ids, logits_out, as_stream(stream));
    });
}

int aeon_b200_router_topk_noalloc(const aeon_b200_moe_config* cfg, const void* x, int64_t x_stride,
                                  const void* gate, const float* bias, int tokens,
                                  float* topk_weights, int32_t* topk_ids, void* stream) {
    return guarded([&] {
        require(cfg != nullptr, "aeon_b200_router_topk_noalloc: null config");
        launch_router_noalloc(*cfg, x, x_stride, gate, bias, tokens, topk_weights, topk_ids,
                              as_stream(stream));
    });
}

int aeon_b200_expert_permutation(aeon_b200_ctx* ctx, const int32_t* topk_ids, int tokens, int slots,
                                 int experts, int32_t* expert_offsets, int32_t* token_indices,
                                 int32_t* draw_indices, const float* weights,
                                 float* weights_by_position, void* stream) {
    return guarded([&] {
        require(ctx != nullptr, "aeon_b200_expert_permutation: null context");
        DeviceGuard guard(ctx->device);
        launch_permutation(ctx, topk_ids, tokens, slots, experts, expert_offsets, token_indices,
                           draw_indices, weights, weights_by_position, nullptr, nullptr, nullptr,
                           false, as_stream(stream));
    });
}

int aeon_b200_shared_expert(aeon_b200_ctx* ctx, const void* w1, const void* w3, const void* w2,
                            const void* x, int64_t x_stride, int tokens, float* moe_accum,
                            int64_t accum_stride, void* stream) {
    return guarded([&] {
        require(ctx != nullptr, "aeon_b200_shared_expert: null context");
        DeviceGuard guard(ctx->device);
        launch_shared_expert(ctx, w1, w3, w2, x, x_stride, tokens, moe_accum, accum_stride,
                             as_stream(stream));
    });
}

int aeon_b200_moe_decode(aeon_b200_ctx* ctx, const void* pool_base, const int32_t* slot_of_expert,
                         const void* x, int64_t x_stride, const int32_t* topk_ids,
                         const float* topk_weights, int tokens, float* moe_accum,
                         int64_t accum_stride, uint32_t flags, void* stream) {
    return guarded([&] {
        require(ctx != nullptr, "aeon_b200_moe_decode: null context");
        DeviceGuard guard(ctx->device);
        launch_moe_decode(ctx, pool_base, slot_of_expert, x, x_stride, topk_ids, topk_weights, tokens,
                          moe_accum, accum_stride, flags, as_stream(stream));
    });
}

int aeon_b200_moe_accumulate(aeon_b200_ctx* ctx, const int32_t* slot_of_expert, const int32_t* topk_ids,
                             int tokens, float* moe_accum, int64_t accum_stride, uint32_t flags,
                             void* stream) {
    return guarded([&] {
        require(ctx != nullptr, "aeon_b200_moe_accumulate: null context");
        DeviceGuard guard(ctx->device);
        launch_moe_accumulate(ctx, slot_of_expert, topk_ids, tokens, moe_accum, accum_stride, flags,
                              as_stream(stream));
    });
}

int aeon_b200_moe_prefill(aeon_b200_ctx* ctx, const void* pool_base, const int32_t* slot_of_expert,
                          const void* x, int64_t x_stride, const int32_t* topk_ids,
                          const float* topk_weights, int tokens, float* moe_accum,
                          int64_t accum_stride, uint32_t flags, void* stream) {
    return guarded([&] {
        require(ctx != nullptr, "aeon_b200_moe_prefill: null context");
        DeviceGuard guard(ctx->device);
        launch_moe_prefill(ctx, pool_base, slot_of_expert, x, x_stride, topk_ids, topk_weights, tokens,
                           moe_accum, accum_stride, flags, as_stream(stream));
    });
}

int aeon_b200_hc_params_default(aeon_b200_hc_params* out) {
    return guarded([&] {
        require(out != nullptr, "aeon_b200_hc_params_default: null argument");
        // src/architecture/deepseek_v4/reference/dsv4_oracle.hpp:489-495; spec/config.hpp:66-70
        *out = aeon_b200_hc_params{1e-6f, 1e-6f, 1e-6f, 2.0f, 1e-6f, 20};
    });
}

int aeon_b200_hc_ffn_front(aeon_b200_ctx* ctx, const void* res_mid, const float* hc_fn, const float* hc_base,
                           const float* hc_scale3, const void* norm_weight, int tokens,
                           const aeon_b200_hc_params* params, void* ffn_norm_out, int64_t out_stride,
                           float* pre_mix_out, float* post_mix_out, float* comb_out, void* stream) {
    return guarded([&] {
        require(ctx != nullptr && params != nullptr, "aeon_b200_hc_ffn_front: null context or parameters");
        DeviceGuard guard(ctx->device);
        launch_hc_ffn_front(ctx, res_mid, hc_fn, hc_base, hc_scale3, norm_weight, tokens, *params, ffn_norm_out,
                            out_stride, pre_mix_out, post_mix_out, comb_out, as_stream(stream));
    });
}

int aeon_b200_hc_post(aeon_b200_ctx* ctx, const float* moe_out, int64_t moe_stride, const void* res_mid,
                      const float* post_mix, const float* comb, int tokens, void* res_out, void* stream) {
    return guarded([&] {
        require(ctx != nullptr, "aeon_b200_hc_post: null context");
        DeviceGuard guard(ctx->device);
        launch_hc_post(ctx, moe_out, moe_stride, res_mid, post_mix, comb, tokens, res_out, as_stream(stream));
    });
}

int aeon_b200_ep_combine(float* out, int64_t out_stride, const float* partials, int ranks, int tokens,
                         int hidden, void* stream) {
    return guarded([&] {
        launch_ep_combine(out, out_stride, partials, ranks, tokens, hidden, as_stream(stream));
    });
}

int aeon_b200_synth_fill_experts(const aeon_b200_moe_config* cfg, void* pool_base, uint32_t first_slot,
                                 uint32_t count, uint64_t seed, uint32_t layer, uint32_t first_expert,
                                 const uint16_t* scale_table, uint32_t table_n, void* stream) {
    return guarded([&] {
        require(cfg != nullptr, "aeon_b200_synth_fill_experts: null config");
        launch_synth_experts(*cfg, pool_base, first_slot, count, seed, layer, first_expert, scale_table,
                             table_n, as_stream(stream));
    });
}

int aeon_b200_synth_fill_dense16(void* out, uint64_t count, uint64_t seed, uint32_t layer,
                                 uint32_t stream_id, const uint16_t* magnitude_table, uint32_t table_n,
                                 void* stream) {
    return guarded([&] {
        launch_synth_dense16(out, count, seed, layer, stream_id, magnitude_table, table_n,
                             as_stream(stream));
    });
}

}  // extern "C"
