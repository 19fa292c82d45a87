// Internal declarations shared by the translation units of libaeon_b200.so.
#pragma once

#include "aeon_b200.h"

#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <stdexcept>
#include <string>
#include <vector>

namespace aeon_b200 {

// ---------------------------------------------------------------------------
// Error plumbing: C++ exceptions inside, status codes at the ABI.
// ---------------------------------------------------------------------------
struct StatusError : std::runtime_error {
    int status;
    StatusError(int s, const std::string& what) : std::runtime_error(what), status(s) {}
};

void set_last_error(const std::string& message);

#define AEON_CUDA_CHECK(expr)                                                              \
    do {                                                                                   \
        cudaError_t _e = (expr);                                                           \
        if (_e != cudaSuccess) {                                                           \
            throw ::aeon_b200::StatusError(                                                \
                AEON_B200_ERR_CUDA, std::string(#expr) + ": " + cudaGetErrorString(_e) +  \
                                        " (" __FILE__ ":" + std::to_string(__LINE__) + ")"); \
        }                                                                                  \
    } while (0)

inline void require(bool ok, const char* message) {
    if (!ok) throw StatusError(AEON_B200_ERR_INVALID_ARGUMENT, message);
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <class F>
int guarded(F&& f) noexcept {
    try {
        f();
        return AEON_B200_OK;
    } catch (const StatusError& e) {
        set_last_error(e.what());
        return e.status;
    } catch (const std::exception& e) {
        set_last_error(e.what());
        return AEON_B200_ERR_CUDA;
    }
}

// ---------------------------------------------------------------------------
// Geometry of one swizzled matrix (device-visible POD).
// ---------------------------------------------------------------------------
struct MatrixGeom {
    uint64_t packed_offset;   // bytes from payload start
    uint64_t scale_offset;
    int rows, cols, rpw, lpr;
    int iters;                // (cols / 32) / lpr
    int block_bytes;          // packed bytes of one row-block: iters * 512
    int block_scale_bytes;    // scale bytes of one row-block: iters * 32 / (group/32) * 2
};

struct ExpertGeom {
    MatrixGeom w1, w2, w3;
    uint64_t payload_bytes;
    int group;
};

ExpertGeom make_geom(const aeon_b200_moe_config& cfg);
void validate_config(const aeon_b200_moe_config& cfg);
// Host re-layout of one matrix between checkpoint order and swizzled order (capi.cu).
void relayout_w4a16(const uint32_t* src_packed, const uint16_t* src_scale, uint32_t* dst_packed,
                    uint16_t* dst_scale, int N, int K, int rpw, int lpr, int group, bool forward);

// Device error flag values (ctx->d_error).
enum : int {
    kErrNone = 0,
    kErrWaitTimeout = 1,      // an mbarrier wait ran out of iterations
    kErrExpertAbsent = 2,     // slot_of_expert[e] < 0 for a routed expert
    kErrIdOutOfRange = 3,     // an expert id, a table entry or a pool slot outside its range
    kErrBounds = 4            // bounds-checked build: an index left its buffer (the access was skipped)
};

// ---------------------------------------------------------------------------
// Bounds-checked build: make EXTRA_NVCCFLAGS=-DAEON_B200_BOUNDS=1. Every index the kernels
// derive from run-time data (gathers through token / draw / slot lists, stores into scratch and
// output buffers) is checked against the extent of its buffer; a violation sets the context's
// error flag and the access is skipped -- nothing traps, so the context stays usable and
// aeon_b200_ctx_check reports AEON_B200_ERR_OUT_OF_RANGE. The context's scratch buffers also get
// a guard region behind them whose pattern aeon_b200_ctx_check verifies. In the normal build
// index_ok is the constant true and the guards are not allocated. This is the substitute for a
// memory checker where none can be run.
// ---------------------------------------------------------------------------
#ifdef AEON_B200_BOUNDS
constexpr bool kBoundsChecked = true;
__device__ __forceinline__ bool index_ok(long long index, long long extent, int32_t* error) {
    if (index >= 0 && index < extent) return true;
    if (error != nullptr) atomicCAS(error, kErrNone, kErrBounds);
    return false;
}
#else
constexpr bool kBoundsChecked = false;
__device__ __forceinline__ constexpr bool index_ok(long long, long long, int32_t*) { return true; }
#endif
constexpr size_t kGuardBytes = 256;
constexpr uint8_t kGuardPattern = 0xC5;

// One entry of the decode work list: the tokens [pos0, pos0+ntok) of the
// expert-sorted draw order all belong to `expert`, whose payload is pool slot `slot`.
struct WorkEntry {
    int expert, pos0, ntok, slot;
};

struct ScratchGuard {
    const void* base;         // the buffer
    const uint8_t* guard;     // kGuardBytes of kGuardPattern right behind it
    const char* name;
};

}  // namespace aeon_b200

struct aeon_b200_ctx {
    aeon_b200_moe_config cfg;
    aeon_b200::ExpertGeom geom;
    int device;
    int sm_count;
    int max_tokens;
    uint64_t scratch_bytes;
    uint64_t launches;

    // --- device scratch ---
    __half* d_xperm;        // [max_tokens, H] fp16 activations in the kernels' K order
    float* d_logits;        // [max_tokens, E]
    int32_t* d_offsets;     // [E + 1]
    int32_t* d_token_idx;   // [max_tokens * k]
    int32_t* d_draw_idx;    // [max_tokens * k]
    float* d_wpos;          // [max_tokens * k]
    aeon_b200::WorkEntry* d_entries;  // [E + max_tokens * k / 8 + 1]
    int32_t* d_counts;      // [0] = entries, [1] = distinct experts, [2] = draws placed
    __half* d_hidden_hi;    // [max_tokens * k, I]
    __half* d_hidden_lo;    // [max_tokens * k, I]
    float* d_contrib;       // [max_tokens * k, H]
    int32_t* d_error;       // device error flag
    // optional per-kernel timing (events recorded on the caller's stream)
    int pool_slots;         // slots of the expert pool the calls will be given (0: not declared)
    // bounds-checked build: guard regions behind the scratch buffers
    std::vector<aeon_b200::ScratchGuard>* guards;
    int timing_enabled;
    std::vector<cudaEvent_t>* timing_events;   // triples: before A, between A and B, after B
    size_t timing_used;
    double timing_ms[2];
    int64_t timing_launches[2];

    // prefill (grouped GEMM) scratch, allocated on first use and grown on demand
    void* prefill;

    // shared expert scratch
    __half* d_sh_hi;        // [max_tokens, I] (hi/mid/lo split of the fp32 hidden)
    __half* d_sh_mid;
    __half* d_sh_lo;
    void* shared_tc;        // split-K partial sums of the tensor-core form, allocated on first use

    // the permutation of a decode call runs beside the activation staging on this stream
    cudaStream_t aux_stream;
    cudaEvent_t aux_fork, aux_join;
};

namespace aeon_b200 {

// Launchers (one per translation unit).
void launch_router(aeon_b200_ctx* ctx, const void* x, int64_t x_stride, const void* gate,
                   const float* bias, const int64_t* hash_table, const int32_t* token_ids,
                   int tokens, float* topk_weights, int32_t* topk_ids, float* logits_out,
                   cudaStream_t stream);
void launch_router_noalloc(const aeon_b200_moe_config& cfg, const void* x, int64_t x_stride,
                           const void* gate, const float* bias, int tokens, float* topk_weights,
                           int32_t* topk_ids, cudaStream_t stream);
void launch_permutation(aeon_b200_ctx* ctx, const int32_t* topk_ids, int tokens, int slots,
                        int experts, int32_t* expert_offsets, int32_t* token_indices,
                        int32_t* draw_indices, const float* weights, float* weights_by_position,
                        const int32_t* slot_of_expert, WorkEntry* entries, int32_t* counts,
                        bool skip_absent, cudaStream_t stream);
void launch_moe_decode(aeon_b200_ctx* ctx, const void* pool_base, const int32_t* slot_of_expert,
                       const void* x, int64_t x_stride, const int32_t* topk_ids,
                       const float* topk_weights, int tokens, float* moe_accum,
                       int64_t accum_stride, uint32_t flags, cudaStream_t stream);
void launch_moe_accumulate(aeon_b200_ctx* ctx, const int32_t* slot_of_expert, const int32_t* topk_ids,
                           int tokens, float* moe_accum, int64_t accum_stride, uint32_t flags,
                           cudaStream_t stream);
void launch_moe_prefill(aeon_b200_ctx* ctx, const void* pool_base, const int32_t* slot_of_expert,
                        const void* x, int64_t x_stride, const int32_t* topk_ids,
                        const float* topk_weights, int tokens, float* moe_accum, int64_t accum_stride,
                        uint32_t flags, cudaStream_t stream);
void free_prefill_scratch(aeon_b200_ctx* ctx);
// cudaMalloc of `bytes` for a context; the bounds-checked build appends a guard region, fills it
// with the guard pattern and registers it under `name` for aeon_b200_ctx_check.
void* ctx_device_alloc(aeon_b200_ctx* ctx, size_t bytes, const char* name);
void ctx_device_free(aeon_b200_ctx* ctx, void* base) noexcept;
void launch_ep_combine(float* out, int64_t out_stride, const float* partials, int ranks,
                       int tokens, int hidden, cudaStream_t stream);
void launch_shared_expert(aeon_b200_ctx* ctx, const void* w1, const void* w3, const void* w2,
                          const void* x, int64_t x_stride, int tokens, float* moe_accum,
                          int64_t accum_stride, cudaStream_t stream);
// tensor-core form of the shared expert (shared_expert_tc.cu), used at larger batches
bool shared_expert_tc_supports(const aeon_b200_moe_config& cfg, int64_t accum_stride);
void launch_shared_expert_tc(aeon_b200_ctx* ctx, const void* w1, const void* w3, const void* w2,
                             const void* x, int64_t x_stride, int tokens, float* moe_accum,
                             int64_t accum_stride, cudaStream_t stream);
void free_shared_tc_scratch(aeon_b200_ctx* ctx);
void launch_hc_ffn_front(aeon_b200_ctx* ctx, const void* res_mid, const float* hc_fn, const float* hc_base,
                         const float* hc_scale3, const void* norm_weight, int tokens,
                         const aeon_b200_hc_params& hp, void* ffn_norm, int64_t out_stride, float* pre_mix,
                         float* post_mix, float* comb, cudaStream_t stream);
void launch_hc_post(aeon_b200_ctx* ctx, const float* layer_out, int64_t layer_stride, const void* res_mid,
                    const float* post_mix, const float* comb, int tokens, void* res_out, cudaStream_t stream);
void launch_synth_experts(const aeon_b200_moe_config& cfg, void* pool_base, uint32_t first_slot,
                          uint32_t count, uint64_t seed, uint32_t layer, uint32_t first_expert,
                          const uint16_t* scale_table, uint32_t table_n, cudaStream_t stream);
void launch_synth_dense16(void* out, uint64_t count, uint64_t seed, uint32_t layer,
                          uint32_t stream_id, const uint16_t* table, uint32_t table_n,
                          cudaStream_t stream);

}  // namespace aeon_b200
