// The engine-side executor shown in INTEGRATION.md, verbatim: it must compile against the host
// header with `override` on both accumulate members, i.e. the seam has the reference's signatures
// (src/architecture/deepseek_v4/layer/v4_layer_body_moe.hpp:32-112). Compile-only check.
#include "aeon_b200_host.hpp"
class B200RoutedExpertExecutor final : public aeon::core::V4RoutedExpertExecutor {
public:
    B200RoutedExpertExecutor(const aeon_b200_moe_config& cfg, int device, int max_chunk,
                             const void* pool_base, const int32_t* slot_of_expert_dev, void* compute)
        : cfg_(cfg), pool_(pool_base), slots_(slot_of_expert_dev), stream_(compute) {
        aeon::core::check_status(aeon_b200_ctx_create(&cfg, device, max_chunk, &ctx_));
    }
    ~B200RoutedExpertExecutor() override { aeon_b200_ctx_destroy(ctx_); }

    void accumulate_routed(uint32_t layer, uint32_t pos, const aeon::core::act16* x,
                           const float* weights, float* moe_accum) override {
        accumulate_routed_batch(layer, pos, 1, x, cfg_.hidden, ids_dev_, cfg_.top_k, weights, cfg_.top_k,
                                moe_accum, cfg_.hidden);
    }
    void accumulate_routed_batch(uint32_t, uint32_t, uint32_t tokens, const aeon::core::act16* x, int x_stride,
                                 const int* ids, int, const float* weights, int,
                                 float* moe_accum, int out_stride) override {
        aeon::core::check_status(aeon_b200_moe_decode(ctx_, pool_, slots_, x, x_stride, ids, weights,
                                                      static_cast<int>(tokens), moe_accum, out_stride, 0, stream_));
    }
    void set_device_ids(const int* ids_dev) { ids_dev_ = ids_dev; }
private:
    aeon_b200_moe_config cfg_;
    aeon_b200_ctx* ctx_{};
    const void* pool_;
    const int32_t* slots_;
    const int* ids_dev_{};
    void* stream_;
};
int main() { return 0; }
