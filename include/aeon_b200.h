/*
 * aeon_b200 — C ABI of the B200-native routed-expert MoE FFN path.
 *
 * The reference project (marcoLapiello/project-aeon) has no C ABI for this path:
 * its kernels are header-only HIP templates included straight into the engine
 * (src/architecture/deepseek_v4/moe/v4_expert_executor.hpp:50-61). Each entry
 * point below therefore cites the reference *source-level* interface it stands
 * in for; the C++ shim in project-aeon_b200/host/ restores the reference class
 * and function names on top of these calls.
 *
 * Conventions
 *  - Every function returns an aeon_b200_status; 0 is success. The message for
 *    the last failure on the calling thread is aeon_b200_last_error().
 *  - Pointers are DEVICE pointers unless the parameter name ends in `_host`.
 *  - `stream` is a cudaStream_t passed as void* (NULL = the default stream).
 *  - Strides are in elements of the pointed-to type.
 *  - 16-bit tensors (activations, gate matrix, shared-expert weights) are raw
 *    IEEE fp16 or bfloat16 bit patterns, selected by aeon_b200_moe_config.act_dtype.
 *  - There is no CPU fallback anywhere: a call on a machine without a usable
 *    sm_100 device returns AEON_B200_ERR_CUDA.
 */
#ifndef AEON_B200_H
#define AEON_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum aeon_b200_status {
    AEON_B200_OK = 0,
    AEON_B200_ERR_INVALID_ARGUMENT = 1, /* shape / argument violation (std::invalid_argument in the reference) */
    AEON_B200_ERR_LOGIC = 2,            /* protocol violation (std::logic_error) */
    AEON_B200_ERR_CUDA = 3,             /* device error (std::runtime_error from CHECK_HIP, src/infrastructure/hip_check.hpp:20-27) */
    AEON_B200_ERR_OUT_OF_RANGE = 4,     /* id out of range (std::out_of_range) */
    AEON_B200_ERR_TIMEOUT = 5,          /* a bounded device-side wait ran out */
    AEON_B200_ERR_UNSUPPORTED = 6
} aeon_b200_status;

enum { AEON_B200_F16 = 0, AEON_B200_BF16 = 1 };
enum { AEON_B200_SCORE_SQRT_SOFTPLUS = 0, AEON_B200_SCORE_SIGMOID = 1 };

/*
 * Shape and model choices of one MoE layer. Replaces the constants the
 * reference hard-codes: V4RoutedExpertScratch::kExperts/kHidden/kIntermediate
 * (src/architecture/deepseek_v4/moe/v4_expert_executor.hpp:96-101), the router
 * scalars (src/architecture/deepseek_v4/spec/config.hpp:54-62) and the swizzle
 * configurations kCfgW13 / kCfgW2
 * (src/backend/swizzled_w4a16/kernels/aeon_w4a16_swizzle.hpp:14-15).
 */
typedef struct aeon_b200_moe_config {
    int32_t hidden;         /* H: model width; K of W1/W3, N of W2 */
    int32_t intermediate;   /* I: expert width; N of W1/W3, K of W2 */
    int32_t experts;        /* routed experts per layer */
    int32_t top_k;          /* routed experts per token */
    int32_t group_size;     /* columns sharing one fp16 scale: 32 or 128 */
    int32_t act_dtype;      /* AEON_B200_F16 / AEON_B200_BF16 */
    int32_t score_fn;       /* AEON_B200_SCORE_* */
    int32_t renormalize;    /* divide the selected scores by their sum */
    float routed_scaling;   /* multiplies the (renormalised) weights */
    float swiglu_limit;     /* clamp of the SwiGLU: gate <= L, |up| <= L */
    int32_t w13_rpw, w13_lpr; /* swizzle rows-per-wave / lanes-per-row of W1 and W3 */
    int32_t w2_rpw, w2_lpr;   /* same for W2 */
} aeon_b200_moe_config;

/* Byte geometry of one expert payload: W1 packed, W1 scales, W2 packed, W2
 * scales, W3 packed, W3 scales, each region on a 4 KiB boundary. Replaces the
 * constants of src/backend/swizzled_w4a16/core/swizzled_expert_format.hpp:11-30. */
typedef struct aeon_b200_expert_layout {
    uint64_t payload_bytes;
    uint64_t w1_packed_offset, w1_scale_offset;
    uint64_t w2_packed_offset, w2_scale_offset;
    uint64_t w3_packed_offset, w3_scale_offset;
    uint64_t w13_packed_bytes, w13_scale_bytes;
    uint64_t w2_packed_bytes, w2_scale_bytes;
} aeon_b200_expert_layout;

typedef struct aeon_b200_ctx aeon_b200_ctx;

const char* aeon_b200_last_error(void);
const char* aeon_b200_version(void);

/* Named presets: "ref_dsv4" (the reference model's shapes: H 4096, I 2048, 256
 * experts, top-6, group 32, fp16, sqrt-softplus x1.5) and "baseline" (H 7168,
 * I 2048, 256 experts, top-8, group 128, bf16, sigmoid renormalised to 1). */
int aeon_b200_config_preset(const char* name, aeon_b200_moe_config* out_host);
int aeon_b200_config_validate(const aeon_b200_moe_config* cfg_host);
int aeon_b200_expert_layout_of(const aeon_b200_moe_config* cfg_host,
                               aeon_b200_expert_layout* out_host);

/* Host re-layout between checkpoint order (row-major [N, K/8] words of eight
 * nibbles, scales [N, K/group]) and the swizzled order the kernels read.
 * Replaces swizzle_w4a16 / unswizzle_w4a16
 * (src/backend/swizzled_w4a16/kernels/aeon_w4a16_swizzle.hpp:46-129). */
int aeon_b200_swizzle_w4a16(const uint32_t* src_packed_host, const uint16_t* src_scale_host,
                            uint32_t* dst_packed_host, uint16_t* dst_scale_host,
                            int N, int K, int rpw, int lpr, int group);
int aeon_b200_unswizzle_w4a16(const uint32_t* src_packed_host, const uint16_t* src_scale_host,
                              uint32_t* dst_packed_host, uint16_t* dst_scale_host,
                              int N, int K, int rpw, int lpr, int group);

/*
 * Shard-aware expert payloads (host only). The reference plans this layout as
 * "expert v3" (plans-and-docs/execution/active/MULTI_GPU_EXECUTION_PLAN.md:151-181)
 * but ships only v2 (writer scripts/convert_safetensors_to_aeon.py:46-187, loader
 * src/infrastructure/artifact/aeon_loader.hpp:345-405). A payload of `shards`
 * shards is `shards` complete payloads back to back; shard s holds the slice
 * [s*I/shards, (s+1)*I/shards) of the intermediate dimension (rows of W1/W3,
 * columns of W2, cut from the checkpoint layout and swizzled on their own: the
 * rule of tests/test_expert_shard_equivalence.cpp:286-340). shards == 1 is the
 * v2 payload. `cfg_host` always describes the whole expert (or, for merge, the
 * whole slice); source tensors are row-major W1/W3 [I, H/8] words + [I, H/group]
 * scales and W2 [H, I/8] + [H, I/group].
 */
int aeon_b200_expert_shard_bytes(const aeon_b200_moe_config* cfg_host, int shards,
                                 uint64_t* shard_bytes_host);
int aeon_b200_pack_expert_shards(const aeon_b200_moe_config* cfg_host, int shards,
                                 const uint32_t* w1_packed_host, const uint16_t* w1_scale_host,
                                 const uint32_t* w2_packed_host, const uint16_t* w2_scale_host,
                                 const uint32_t* w3_packed_host, const uint16_t* w3_scale_host,
                                 uint8_t* payload_host);
int aeon_b200_unpack_expert_shards(const aeon_b200_moe_config* cfg_host, int shards,
                                   const uint8_t* payload_host,
                                   uint32_t* w1_packed_host, uint16_t* w1_scale_host,
                                   uint32_t* w2_packed_host, uint16_t* w2_scale_host,
                                   uint32_t* w3_packed_host, uint16_t* w3_scale_host);
/* Byte range, inside a payload of `shards` shards, that rank `rank` of a
 * tensor-parallel group of degree `tp` reads: offset = rank * (shards/tp) *
 * shard_bytes, length = payload_bytes / tp (the planned AeonModelLoader::rank_slice).
 * tp must divide shards (invalid_argument otherwise); rank in [0, tp). */
int aeon_b200_expert_rank_slice(const aeon_b200_moe_config* cfg_host, int shards, int tp, int rank,
                                uint64_t* offset_host, uint64_t* length_host);
/* A rank slice of `shards` shards -> one payload of intermediate width
 * cfg_host->intermediate (= shards * shard width), the form the kernels read.
 * Done once at load time, so the kernels carry no shard arithmetic. */
int aeon_b200_merge_expert_shards(const aeon_b200_moe_config* cfg_host, int shards,
                                  const uint8_t* slice_host, uint8_t* payload_host);

/* A context owns the device scratch of the path for up to `max_tokens` tokens
 * per call. Replaces V4RoutedExpertScratch
 * (src/architecture/deepseek_v4/moe/v4_expert_executor.hpp:95-173). */
int aeon_b200_ctx_create(const aeon_b200_moe_config* cfg_host, int device, int max_tokens,
                         aeon_b200_ctx** out_host);
int aeon_b200_ctx_destroy(aeon_b200_ctx* ctx);
uint64_t aeon_b200_ctx_scratch_bytes(const aeon_b200_ctx* ctx);
/* Synchronises `stream` and reports a device-side error flag (a bounded wait
 * that ran out, an id out of range) as a status. */
int aeon_b200_ctx_check(aeon_b200_ctx* ctx, void* stream);
/* Kernel launches issued by this context since creation (the benchmark's count). */
uint64_t aeon_b200_ctx_launches(const aeon_b200_ctx* ctx);
/* Declares how many slots the expert pool given to this context's calls has. From then on a
 * slot_of_expert entry at or above it is reported (aeon_b200_ctx_check: OUT_OF_RANGE) and its
 * expert treated as absent, instead of being used as an address. 0 withdraws the declaration.
 * The reference bounds its slot by construction (ExpertPayloadPool::get_slot_base throws,
 * src/infrastructure/expert/storage/expert_payload_pool.hpp:70-78); here the table lives on the
 * device, so the check does too. */
int aeon_b200_ctx_set_pool_slots(aeon_b200_ctx* ctx, int slots);
/* 1 when the library was built with -DAEON_B200_BOUNDS=1: every run-time-derived index in the
 * kernels is checked against its buffer and skipped when outside (the error flag is set), and
 * aeon_b200_ctx_check also verifies guard regions behind the context's scratch buffers. The
 * stand-in for a memory checker; the reference relies on its own host-side checks
 * (src/infrastructure/hip_check.hpp:20-27). */
int aeon_b200_bounds_checked(void);

/* Expert payload pool: one device slab of slots x payload_bytes, a slot being a
 * byte-identical expert payload. Replaces ExpertPayloadPool
 * (src/infrastructure/expert/storage/expert_payload_pool.hpp:16-131). */
int aeon_b200_pool_create(uint64_t payload_bytes, uint32_t slots, int device, void** out_base_host);
int aeon_b200_pool_destroy(void* base, int device);
int aeon_b200_pool_upload(void* base, uint64_t payload_bytes, uint32_t slot,
                          const void* payload_host, void* stream);

/* Router: gate projection + score + top-k + renormalise + scale, one call.
 * Replaces dispatch_router
 * (src/architecture/deepseek_v4/layer/v4_layer_body_moe.hpp:124-159), i.e.
 * gemv_fp16_vec8_kernel + v4_half_to_float_n_kernel + moe_router_kernel
 * (src/architecture/deepseek_v4/kernels/moe_router.hpp:104-189).
 * x[tokens, x_stride] and gate[experts, hidden] are 16-bit (act_dtype);
 * bias[experts] fp32 may be NULL. hash_table[vocab, top_k] (int64) + token_ids
 * select the table-lookup branch when both are non-NULL. Outputs: ids in
 * descending selection order, ties to the lower index; logits_out[tokens,
 * experts] fp32 is optional. */
int aeon_b200_router_topk(aeon_b200_ctx* ctx, const void* x, int64_t x_stride, const void* gate,
                          const float* bias, const int64_t* hash_table, const int32_t* token_ids,
                          int tokens, float* topk_weights, int32_t* topk_ids, float* logits_out,
                          void* stream);

/* The same router for callers that cannot allocate device memory: code that works under a
 * fixed memory budget, or runs in a host that forbids allocation after start-up. It takes no context (creating one allocates) and makes no cudaMalloc, cudaFree
 * or other allocating call: its logits scratch is a 256 KiB array built into the library,
 * which every GPU that loads the library holds until the process exits. Limits: tokens <=
 * 64 and experts <= 1024; larger sizes return AEON_B200_ERR_INVALID_ARGUMENT. The table
 * (hash) branch is not offered. It runs on the current device; the first call on each
 * device looks up the scratch's device address, so make that first call outside any stream
 * capture. All calls on a device share the one scratch (it holds the last call's logits;
 * nothing in it needs clearing): calls that overlap on the GPU, e.g. on two streams, race.
 * This entry point has no counterpart in the reference. */
int aeon_b200_router_topk_noalloc(const aeon_b200_moe_config* cfg_host, const void* x,
                                  int64_t x_stride, const void* gate, const float* bias, int tokens,
                                  float* topk_weights, int32_t* topk_ids, void* stream);

/* Counting sort of the (token, slot) draws by expert. Replaces
 * dispatch_expert_permutation (src/platform/ops/expert_permutation.hpp:44-175):
 * expert_offsets[experts+1], token_indices[draws], draw_indices[draws] and,
 * when `weights` is non-NULL, weights_by_position[draws]. Ascending expert
 * order, ascending draw order inside an expert; ids outside [0, experts) are
 * dropped. */
int aeon_b200_expert_permutation(aeon_b200_ctx* ctx, const int32_t* topk_ids, int tokens,
                                 int slots, int experts, int32_t* expert_offsets,
                                 int32_t* token_indices, int32_t* draw_indices,
                                 const float* weights, float* weights_by_position, void* stream);

/* Shared expert: dense 16-bit FFN with the same clamped SwiGLU, WRITTEN into
 * moe_accum (fp32) as the accumulator's initial value. Replaces
 * run_layer_body_moe_shared_expert[_batch]
 * (src/architecture/deepseek_v4/layer/v4_layer_body_moe.hpp:216-256,
 *  src/architecture/deepseek_v4/layer/v4_layer_body_batch.hpp:863-917).
 * w1, w3: [I, H]; w2: [H, I]; row-major, act_dtype. Up to 16 tokens the weights
 * are streamed through warp MMAs; above, the two projections run as split-K
 * tcgen05 GEMMs, whose partial-sum scratch is allocated by the first such call
 * on a context (make that call outside any stream capture). */
int aeon_b200_shared_expert(aeon_b200_ctx* ctx, const void* w1, const void* w3, const void* w2,
                            const void* x, int64_t x_stride, int tokens, float* moe_accum,
                            int64_t accum_stride, void* stream);

/* Decode path: for every token, moe_accum[t,:] += sum over its top_k slots, in
 * slot order, of weight * W2_e * clamped_swiglu(W1_e x, W3_e x); fp32 in and out.
 * Replaces V4TieredExpertExecutor::accumulate_routed / accumulate_routed_batch
 * (src/architecture/deepseek_v4/moe/v4_expert_executor.hpp:298-370,379-461), i.e.
 * aeon_moe_fused_gate_up_kernel, aeon_moe_fused_w2_contrib_kernel and
 * moe_accumulate_fixed_order_kernel. `pool_base` is the expert pool slab;
 * slot_of_expert[experts] maps a routed expert id to its slot (-1: absent, which
 * raises the context's error flag, unless AEON_B200_DECODE_SKIP_ABSENT is set in `flags`:
 * then draws of absent experts contribute nothing, which is the expert-parallel case
 * where this GPU holds a slice of the experts and moe_accum is a partial sum). Each
 * distinct expert's weights are read once per call. tokens <= the context's max_tokens. */
enum {
    AEON_B200_DECODE_SKIP_ABSENT = 1,
    /* Stop after the per-draw slices are written; the caller finishes with
     * aeon_b200_moe_accumulate. Lets the shared expert (which produces moe_accum's initial
     * value) run on another stream while the routed experts stream their weights. */
    AEON_B200_DECODE_DEFER_ACCUMULATE = 2,
    /* moe_accum[t,:] = the routed sum instead of += : the accumulator's previous contents are
     * neither read nor needed (rows whose draws are all skipped become 0). Saves the caller a
     * zero fill when moe_accum is a per-rank partial sum (expert or tensor parallel). */
    AEON_B200_DECODE_OVERWRITE = 4
};
int aeon_b200_moe_decode(aeon_b200_ctx* ctx, const void* pool_base, const int32_t* slot_of_expert,
                         const void* x, int64_t x_stride, const int32_t* topk_ids,
                         const float* topk_weights, int tokens, float* moe_accum,
                         int64_t accum_stride, uint32_t flags, void* stream);

/* Second half of a deferred decode call: moe_accum[t,:] += the slot-order sum of the per-draw
 * slices the last aeon_b200_moe_decode(..., AEON_B200_DECODE_DEFER_ACCUMULATE) of this context
 * left in its scratch. Same ids / slot table / flags as that call. Replaces
 * moe_accumulate_fixed_order_kernel (src/platform/ops/moe_accumulate.hpp:73-92). */
int aeon_b200_moe_accumulate(aeon_b200_ctx* ctx, const int32_t* slot_of_expert, const int32_t* topk_ids,
                             int tokens, float* moe_accum, int64_t accum_stride, uint32_t flags,
                             void* stream);

/* Prefill path: the same contract as aeon_b200_moe_decode (moe_accum[t,:] += routed sum in
 * slot order, fp32) for chunks of many tokens, computed as per-expert grouped GEMMs on the
 * tcgen05 tensor cores: int4 weights are dequantised to fp16 into shared memory, the expert's
 * tokens (gathered in expert order) are the other operand, accumulation is fp32 in tensor
 * memory. Replaces V4TieredExpertExecutor::accumulate_routed_batch's grouped branch
 * (src/architecture/deepseek_v4/moe/v4_expert_executor.hpp:379-461), run_moe_grouped_expert_batch
 * (src/architecture/deepseek_v4/moe/moe_grouped_batch.hpp:55-147) and the kernels
 * moe_grouped_gate_up_kernel / moe_grouped_down_kernel
 * (src/platform/rdna3/moe_grouped_ffn.hpp:77-288). MMA operands are fp16 (weights rounded once
 * from q*scale, the hidden vector rounded to fp16 between the two GEMMs). Scratch for the
 * chunk is allocated on the first call and grown when a larger chunk arrives (the reference's
 * allocate_chunk_scratch, v4_expert_executor.hpp:127-153). tokens <= 65536. */
int aeon_b200_moe_prefill(aeon_b200_ctx* ctx, const void* pool_base, const int32_t* slot_of_expert,
                          const void* x, int64_t x_stride, const int32_t* topk_ids,
                          const float* topk_weights, int tokens, float* moe_accum,
                          int64_t accum_stride, uint32_t flags, void* stream);

/*
 * The steps of a layer either side of the MoE FFN (the caller of the path,
 * src/architecture/deepseek_v4/layer/v4_layer_body_moe.hpp:204-312): the
 * hyper-connection pre-mix of the four residual streams fused with the FFN
 * RMSNorm, and the post expansion back to four streams. Replace
 * hc_project_kernel + hc_sinkhorn_normalize_kernel + hc_pre_combine_kernel +
 * the FFN norm, and hc_post_kernel
 * (src/architecture/deepseek_v4/kernels/hc_sinkhorn.hpp:22-290). With these the
 * activation the router and the experts read, the routing and the mix
 * coefficients all stay on the device from residual in to residual out.
 *
 * res_mid / res_out: [tokens, 4, hidden] 16-bit (act_dtype), contiguous.
 * hc_fn fp32 [24, 4*hidden], hc_base fp32 [24], hc_scale3 fp32 [3] (device).
 * norm_weight [hidden] 16-bit. Outputs of the front: ffn_norm_out [tokens,
 * out_stride] 16-bit, pre/post_mix_out fp32 [tokens, 4], comb_out fp32
 * [tokens, 16] with comb[i*4 + j] contracting stream i into stream j.
 * moe_out: the fp32 accumulator of the path (shared expert + routed experts).
 */
typedef struct aeon_b200_hc_params {
    float rms_eps;         /* RMS of the flattened residual in the mixes */
    float pre_eps;         /* added to the pre gate only */
    float sinkhorn_eps;    /* in every Sinkhorn denominator and after the softmax */
    float post_mult;       /* multiplies the post gate (2 in the reference model) */
    float norm_eps;        /* FFN RMSNorm */
    int32_t sinkhorn_iters;
} aeon_b200_hc_params;
int aeon_b200_hc_params_default(aeon_b200_hc_params* out_host);
int aeon_b200_hc_ffn_front(aeon_b200_ctx* ctx, const void* res_mid, const float* hc_fn,
                           const float* hc_base, const float* hc_scale3, const void* norm_weight,
                           int tokens, const aeon_b200_hc_params* params_host, void* ffn_norm_out,
                           int64_t out_stride, float* pre_mix_out, float* post_mix_out,
                           float* comb_out, void* stream);
int aeon_b200_hc_post(aeon_b200_ctx* ctx, const float* moe_out, int64_t moe_stride,
                      const void* res_mid, const float* post_mix, const float* comb, int tokens,
                      void* res_out, void* stream);

/* Expert-parallel combine: out[t, :] += sum over r = 0..ranks-1, in rank order, of
 * partials[r, t, :] (fp32; partials is [ranks, tokens, hidden] dense, as an equal-split
 * all-to-all delivers it). The fixed order makes the result independent of arrival order.
 * The reference has no expert parallelism (it is deferred:
 * plans-and-docs/specs-and-requirements/multi-gpu/MULTI_GPU_REQUIREMENTS.md:103); the
 * order rule follows its fixed-slot-order accumulate
 * (src/platform/ops/moe_accumulate.hpp:73-92). */
int aeon_b200_ep_combine(float* out, int64_t out_stride, const float* partials, int ranks,
                         int tokens, int hidden, void* stream);

/* ---- devices, streams, events, pinned memory --------------------------------------------------
 * What a C++ host needs around the kernels without including the CUDA runtime. Replaces the
 * reference's direct runtime calls in select_device / DeviceScope (src/platform/device.hpp:29-90),
 * DeviceStreams (src/infrastructure/device_streams.hpp:32-74), enable_peer_access
 * (src/infrastructure/parallel/peer_access.hpp:29-50) and the pinned staging and event ordering of
 * its tiered expert supply (src/infrastructure/expert/transport/tiered_expert_supply.hpp).
 * aeon_b200_device_select validates the index against the visible devices and makes it current
 * (OUT_OF_RANGE for a bad index: a caller that asked for a device that is not there wants to
 * know). Streams are non-blocking and belong to the device current at creation. Peer access is
 * best effort and never an error: enabled_host tells whether the pair is enabled afterwards. */
int aeon_b200_device_count(int* count_host);
int aeon_b200_device_current(int* device_host);
int aeon_b200_device_select(int index);
int aeon_b200_device_describe(int index, char* name_host, int name_bytes, int* pci_bus_host,
                              int* sm_count_host, uint64_t* memory_bytes_host);
int aeon_b200_device_enable_peer_access(int accessor, int peer, int* enabled_host);
int aeon_b200_device_alloc(uint64_t bytes, int device, void** out_host);
int aeon_b200_device_free(void* device_ptr);
int aeon_b200_stream_create(void** stream_host);
int aeon_b200_stream_destroy(void* stream);
int aeon_b200_stream_synchronize(void* stream);
int aeon_b200_stream_wait_event(void* stream, void* event);
int aeon_b200_event_create(void** event_host);
int aeon_b200_event_destroy(void* event);
int aeon_b200_event_record(void* event, void* stream);
int aeon_b200_event_synchronize(void* event);
int aeon_b200_host_alloc_pinned(uint64_t bytes, void** out_host);
int aeon_b200_host_free_pinned(void* pinned);
int aeon_b200_copy_to_device_async(void* dst_device, const void* src_host, uint64_t bytes, void* stream);
int aeon_b200_copy_to_host_async(void* dst_host, const void* src_device, uint64_t bytes, void* stream);

/* ---- multi-GPU groups (one process per GPU, NCCL over NVLink / NVSwitch) -------------------
 * The reference engine refuses tensor-parallel topologies today
 * (src/architecture/deepseek_v4/runtime/v4_model_host.hpp:94-100) and plans a C++
 * TensorParallelGroup with an NCCL-style communicator
 * (plans-and-docs/execution/active/MULTI_GPU_EXECUTION_PLAN.md:189-235); these entry points are
 * that layer for the routed-expert path. One rank creates an id, hands the 128 bytes to the
 * others by any host channel, and every rank creates its group with it (a collective call).
 * NCCL is loaded on first use; a library build without NCCL present still serves one GPU. */
#define AEON_B200_GROUP_ID_BYTES 128
typedef struct aeon_b200_group aeon_b200_group;
int aeon_b200_group_unique_id(void* id_host);
int aeon_b200_group_create(const void* id_host, int rank, int world, int device,
                           aeon_b200_group** out_host);
int aeon_b200_group_destroy(aeon_b200_group* group);
int aeon_b200_group_rank(const aeon_b200_group* group);
int aeon_b200_group_world(const aeon_b200_group* group);

/* Expert-parallel dispatch: every rank contributes its tokens_local activation rows of
 * row_bytes bytes each and receives all ranks' rows in rank order, x_all[world * tokens_local]
 * (an all-gather; at decode sizes a padded all-to-all would move the same bytes). */
int aeon_b200_ep_dispatch(aeon_b200_group* group, const void* x_local, int tokens_local,
                          int64_t row_bytes, void* x_all, void* stream);
/* The dispatch for ranks that route their own tokens: besides the activation rows, every rank
 * contributes the routing of its tokens_local tokens (ids_local / weights_local [tokens_local,
 * top_k], from aeon_b200_router_topk on x_local) and receives the whole batch's routing in rank
 * order. The router is a per-token function, so the gathered routing equals, bit for bit, what a
 * router run on x_all returns; each rank computes 1 / world of it instead of all of it. The three
 * gathers are one grouped NCCL call. */
int aeon_b200_ep_dispatch_routed(aeon_b200_group* group, const void* x_local, int tokens_local,
                                 int64_t row_bytes, void* x_all, const int32_t* ids_local,
                                 const float* weights_local, int top_k, int32_t* ids_all,
                                 float* weights_all, void* stream);
/* Expert-parallel exchange: partial[world * tokens_local, hidden] holds this rank's partial
 * output rows for every token of the batch; rows [r * tokens_local, (r+1) * tokens_local) go to
 * rank r, whose recv[s, :, :] receives the slice computed by rank s (an equal-split all-to-all).
 * aeon_b200_ep_combine then adds the `world` slices in rank order. */
int aeon_b200_ep_exchange(aeon_b200_group* group, const float* partial, int tokens_local, int hidden,
                          float* recv, void* stream);
/* Tensor-parallel reduce: partial[world * tokens_local, hidden] fp32 partial outputs (each rank
 * holds a slice of every expert's intermediate dimension) are summed over the ranks and rank r
 * keeps rows [r * tokens_local, (r+1) * tokens_local) in out_local (a reduce-scatter). The W2
 * split this finishes is the one tests/test_w2_shard_equivalence.cpp:138-296 shows exact. */
int aeon_b200_tp_reduce(aeon_b200_group* group, const float* partial, int tokens_local, int hidden,
                        float* out_local, void* stream);
/* Pipeline-stage hand-off of `bytes` bytes to / from rank `peer`: a byte copy, like
 * handoff_residual (src/architecture/deepseek_v4/runtime/v4_graph.hpp:454-513). */
int aeon_b200_pp_send(aeon_b200_group* group, const void* rows, uint64_t bytes, int peer, void* stream);
int aeon_b200_pp_recv(aeon_b200_group* group, void* rows, uint64_t bytes, int peer, void* stream);

/* ---- expert-parallel combine fused with the accumulate, over peer memory ---------------------
 * The one-kernel form of "accumulate, exchange, combine": every rank owns a receive buffer
 * [world, tokens_local_max, hidden] fp32 that its peers map through CUDA IPC (created
 * collectively over a group; at most 8 ranks of one box). aeon_b200_moe_accumulate_push is the
 * second half of a deferred decode call (like aeon_b200_moe_accumulate) for an expert-parallel
 * rank: it sums, per token of the whole batch and in slot order, the per-draw slices of the
 * experts resident here and stores each row straight into the receive buffer of the rank that
 * owns the token (plain peer stores over NVLink), then raises that owner's flag for this rank.
 * aeon_b200_ep_peer_combine waits, with a bound, for the `world` flags of the call and adds the
 * slices to out[tokens_local, :] in rank order. A flag that does not arrive within the budget
 * (default 2 s) is reported by aeon_b200_ctx_check as TIMEOUT; the peer object is then out of
 * step and must be destroyed. Calls must alternate push / combine, once each per layer on every
 * rank, with the layer's dispatch (aeon_b200_ep_dispatch, aeon_b200_ep_dispatch_routed or
 * aeon_b200_ep_peer_dispatch) between one layer's combine and the next layer's push: waiting for
 * every rank's dispatch is what keeps a fast rank from overwriting rows a slow owner still reads. No counterpart in the reference (no expert parallelism there); the
 * summation order follows src/platform/ops/moe_accumulate.hpp:73-92. */
typedef struct aeon_b200_ep_peer aeon_b200_ep_peer;
int aeon_b200_ep_peer_create(aeon_b200_group* group, int device, int tokens_local_max, int hidden,
                             aeon_b200_ep_peer** out_host);
/* The dispatch in the same form: stores this rank's tokens_local activation rows (16-bit
 * elements, dense, 16-byte aligned) and the routing it computed for them (ids_local /
 * weights_local [tokens_local, top_k]) into every rank's gather buffers, raises one flag per
 * rank, and waits (bounded, as the combine does) for all ranks' rows. Returns this rank's gather
 * buffers, valid once the call's work on `stream` is done: x_all[world * tokens_local, hidden],
 * ids_all / weights_all[world * tokens_local, top_k], in rank order -- what
 * aeon_b200_ep_dispatch_routed delivers, without a collective. The buffers belong to the peer
 * object and are overwritten by the next dispatch. */
int aeon_b200_ep_peer_dispatch(aeon_b200_ctx* ctx, aeon_b200_ep_peer* peer, const void* x_local,
                               int tokens_local, const int32_t* ids_local, const float* weights_local,
                               void** x_all, int32_t** ids_all, float** weights_all, void* stream);
int aeon_b200_ep_peer_destroy(aeon_b200_ep_peer* peer);
int aeon_b200_ep_peer_set_wait_budget(aeon_b200_ep_peer* peer, double milliseconds);
int aeon_b200_moe_accumulate_push(aeon_b200_ctx* ctx, aeon_b200_ep_peer* peer, const int32_t* slot_of_expert,
                                  const int32_t* topk_ids, int tokens_local, void* stream);
int aeon_b200_ep_peer_combine(aeon_b200_ctx* ctx, aeon_b200_ep_peer* peer, float* out, int64_t out_stride,
                              int tokens_local, void* stream);

/* Statistics of the last decode/prefill call of this context (host values read
 * back after a synchronise): distinct experts touched and work-list entries. */
int aeon_b200_ctx_last_stats(aeon_b200_ctx* ctx, void* stream, int32_t* distinct_experts_host,
                             int32_t* entries_host);

/* Per-kernel device timing. When enabled, the decode path brackets its two streaming
 * kernels with CUDA events on the caller's stream; aeon_b200_ctx_kernel_times synchronises
 * the stream, adds up the elapsed times since the last call and returns, for kernel
 * 0 (W1/W3 + SwiGLU) and 1 (W2 + accumulate), the total milliseconds and launch counts.
 * No counterpart in the reference, which times regions with its PhaseProfiler
 * (src/infrastructure/profiling/phase_profiler.hpp:41-110). */
int aeon_b200_ctx_set_timing(aeon_b200_ctx* ctx, int enabled);
int aeon_b200_ctx_kernel_times(aeon_b200_ctx* ctx, void* stream, double* total_ms_host2,
                               int64_t* launches_host2);

/* Counter-based synthetic tensors, bit-identical to the CPU test oracle's
 * generators, so benchmark pools are filled on the device. Expert payloads:
 * nibbles uniform in 0..15 (q = nibble - 8), scales drawn from `scale_table`
 * (fp16 bit patterns, table_n a power of two). Dense tensors: magnitude from
 * the table, sign from the draw. These have no counterpart in the reference,
 * whose tests build payloads on the host
 * (tests/test_w2_shard_equivalence.cpp:80-87). */
int aeon_b200_synth_fill_experts(const aeon_b200_moe_config* cfg_host, void* pool_base,
                                 uint32_t first_slot, uint32_t count, uint64_t seed,
                                 uint32_t layer, uint32_t first_expert,
                                 const uint16_t* scale_table, uint32_t table_n, void* stream);
int aeon_b200_synth_fill_dense16(void* out, uint64_t count, uint64_t seed, uint32_t layer,
                                 uint32_t stream_id, const uint16_t* magnitude_table,
                                 uint32_t table_n, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* AEON_B200_H */
