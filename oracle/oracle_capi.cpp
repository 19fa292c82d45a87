// TEST INFRASTRUCTURE — NOT A PRODUCT PATH.
// C entry points over aeon_oracle.hpp so the parity tests and the benchmark's
// CPU-baseline leg can call the CPU oracle through ctypes. Nothing in the CUDA
// library links or loads this file.
#include "aeon_oracle.hpp"

#include <cstdio>
#include <string>

#ifdef _OPENMP
#include <omp.h>
#endif

using namespace aeon_oracle;

namespace {
thread_local std::string g_error;

struct LayoutArgs {
    int hidden, intermediate, group, w13_rpw, w13_lpr, w2_rpw, w2_lpr;
};

ExpertLayout layout_of(const LayoutArgs* a) {
    return make_expert_layout(a->hidden, a->intermediate, a->group, a->w13_rpw, a->w13_lpr,
                              a->w2_rpw, a->w2_lpr);
}

const MatrixLayout& matrix_of(const ExpertLayout& L, int kind) {
    switch (kind) {
        case 0: return L.w1;
        case 1: return L.w2;
        case 2: return L.w3;
    }
    throw std::invalid_argument("aeon_oracle: matrix kind must be 0 (W1), 1 (W2) or 2 (W3)");
}

template <class F>
int guarded(F&& f) {
    try {
        f();
        return 0;
    } catch (const std::exception& e) {
        g_error = e.what();
        return 1;
    }
}
}  // namespace

extern "C" {

const char* ao_last_error() { return g_error.c_str(); }

int ao_threads() {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

// Sets the thread count of the parallel loops (a launcher may have exported
// OMP_NUM_THREADS=1 before this library was loaded). Returns the count now in force.
int ao_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
    return omp_get_max_threads();
#else
    (void)n;
    return 1;
#endif
}

// out[0]=payload_bytes; then per matrix (W1, W2, W3): packed_offset, scale_offset,
// rows, columns, rpw, lpr, iterations  (7 values each) -> 22 values.
int ao_layout(const LayoutArgs* a, uint64_t* out) {
    return guarded([&] {
        const ExpertLayout L = layout_of(a);
        out[0] = L.payload_bytes;
        const MatrixLayout* mats[3] = {&L.w1, &L.w2, &L.w3};
        for (int m = 0; m < 3; ++m) {
            uint64_t* o = out + 1 + 7 * m;
            o[0] = mats[m]->packed_offset;
            o[1] = mats[m]->scale_offset;
            o[2] = static_cast<uint64_t>(mats[m]->rows);
            o[3] = static_cast<uint64_t>(mats[m]->columns);
            o[4] = static_cast<uint64_t>(mats[m]->rows_per_wave);
            o[5] = static_cast<uint64_t>(mats[m]->lanes_per_row);
            o[6] = static_cast<uint64_t>(mats[m]->iterations());
        }
    });
}

int ao_swizzled_address(const LayoutArgs* a, int kind, int row, int column, uint64_t* out3) {
    return guarded([&] {
        const ExpertLayout L = layout_of(a);
        const SwizzledAddress s = swizzled_address(matrix_of(L, kind), row, column);
        out3[0] = s.scale_slot;
        out3[1] = s.packed_word;
        out3[2] = static_cast<uint64_t>(s.nibble);
    });
}

int ao_rng_fill(uint64_t seed, double scale, uint64_t n, double* out) {
    return guarded([&] {
        Rng rng(seed);
        for (uint64_t i = 0; i < n; ++i) out[i] = rng.symmetric(scale);
    });
}

int ao_rng_u64(uint64_t seed, uint64_t n, uint64_t* out) {
    return guarded([&] {
        Rng rng(seed);
        for (uint64_t i = 0; i < n; ++i) out[i] = rng.next_u64();
    });
}

int ao_half_bits_to_double(const uint16_t* bits, uint64_t n, double* out) {
    return guarded([&] { for (uint64_t i = 0; i < n; ++i) out[i] = half_bits_to_double(bits[i]); });
}

int ao_double_to_half_bits(const double* v, uint64_t n, uint16_t* out) {
    return guarded([&] { for (uint64_t i = 0; i < n; ++i) out[i] = double_to_half_bits(v[i]); });
}

int ao_synth_expert_payload(const LayoutArgs* a, uint8_t* payload, uint64_t seed, uint32_t layer,
                            uint32_t expert, const uint16_t* table, uint32_t table_n) {
    return guarded([&] {
        synth_expert_payload(payload, layout_of(a), seed, layer, expert, table, table_n);
    });
}

int ao_synth_dense16(uint16_t* out, uint64_t count, uint64_t seed, uint32_t layer,
                     uint32_t stream, const uint16_t* table, uint32_t table_n) {
    return guarded([&] { synth_dense16(out, count, seed, layer, stream, table, table_n); });
}

// mode: 0 = default decode, 1 = unsigned zero point (wrong), 2 = unpermuted nibbles (wrong)
int ao_decode_matrix(const LayoutArgs* a, int kind, const uint8_t* payload, int mode,
                     double* out) {
    return guarded([&] {
        const ExpertLayout L = layout_of(a);
        SwizzledDecodeOptions opt;
        opt.signed_zero_point = (mode != 1);
        opt.permute_nibbles = (mode != 2);
        const std::vector<double> w = swizzled_decode(payload, matrix_of(L, kind), opt);
        std::memcpy(out, w.data(), w.size() * sizeof(double));
    });
}

int ao_encode_matrix(const LayoutArgs* a, int kind, uint8_t* payload, const double* w) {
    return guarded([&] {
        const ExpertLayout L = layout_of(a);
        const MatrixLayout& m = matrix_of(L, kind);
        swizzled_encode(payload, m, std::vector<double>(w, w + m.weight_count()));
    });
}

int ao_swizzle_from_source(const LayoutArgs* a, int kind, const uint32_t* src_packed,
                           const uint16_t* src_scale, uint8_t* payload) {
    return guarded([&] {
        const ExpertLayout L = layout_of(a);
        swizzle_from_source(src_packed, src_scale, payload, matrix_of(L, kind));
    });
}

// logits[T, E] in fp64 from 16-bit gate and activations (dtype 0 = fp16, 1 = bf16).
int ao_router_logits_f64(const uint16_t* gate, int gate_dtype, int experts, int hidden,
                         const uint16_t* x, int x_dtype, int tokens, int x_stride, double* out) {
    return guarded([&] {
        for (int t = 0; t < tokens; ++t) {
            std::vector<double> xv(static_cast<size_t>(hidden));
            for (int i = 0; i < hidden; ++i)
                xv[i] = bits16_to_double(x[static_cast<size_t>(t) * x_stride + i],
                                         static_cast<Dtype16>(x_dtype));
            const std::vector<double> l = router_logits(gate, static_cast<Dtype16>(gate_dtype),
                                                        experts, hidden, xv);
            std::memcpy(out + static_cast<size_t>(t) * experts, l.data(),
                        sizeof(double) * experts);
        }
    });
}

int ao_router_logits_f32_ordered(const uint16_t* gate, int gate_dtype, int experts, int hidden,
                                 const uint16_t* x, int x_dtype, int tokens, int x_stride,
                                 float* out) {
    return guarded([&] {
#ifdef _OPENMP
#pragma omp parallel for schedule(static) collapse(2)
#endif
        for (int t = 0; t < tokens; ++t)
            for (int e = 0; e < experts; ++e)
                out[static_cast<size_t>(t) * experts + e] = router_logit_f32_ordered(
                    gate + static_cast<size_t>(e) * hidden, static_cast<Dtype16>(gate_dtype),
                    x + static_cast<size_t>(t) * x_stride, static_cast<Dtype16>(x_dtype), hidden);
    });
}

// Selection from fp64 logits. bias may be null. Outputs ids[T,k], weights[T,k], margin[T].
int ao_router_topk(const double* logits, const double* bias, int tokens, int experts, int top_k,
                   double scaling, int score_fn, int renormalize, int bias_before_score,
                   int32_t* ids, double* weights, double* margin) {
    return guarded([&] {
        std::vector<double> b;
        if (bias) b.assign(bias, bias + experts);
        for (int t = 0; t < tokens; ++t) {
            const std::vector<double> l(logits + static_cast<size_t>(t) * experts,
                                        logits + static_cast<size_t>(t + 1) * experts);
            const RouterSelection s = router_topk(l, b, top_k, scaling,
                                                  static_cast<ScoreFn>(score_fn),
                                                  renormalize != 0, bias_before_score != 0);
            for (int k = 0; k < top_k; ++k) {
                ids[static_cast<size_t>(t) * top_k + k] = s.ids[k];
                weights[static_cast<size_t>(t) * top_k + k] = s.weights[k];
            }
            if (margin) margin[t] = s.min_margin;
        }
    });
}

int ao_router_hash(const double* logits, int experts, const int64_t* table_row, int top_k,
                   double scaling, int score_fn, int32_t* ids, double* weights) {
    return guarded([&] {
        const std::vector<double> l(logits, logits + experts);
        const RouterSelection s = router_hash(l, std::vector<int64_t>(table_row, table_row + top_k),
                                              scaling, static_cast<ScoreFn>(score_fn));
        for (int k = 0; k < top_k; ++k) { ids[k] = s.ids[k]; weights[k] = s.weights[k]; }
    });
}

int ao_topk_indices(const double* scores, int n, int k, int32_t* out) {
    return guarded([&] {
        const std::vector<int32_t> r = topk_indices(std::vector<double>(scores, scores + n), k);
        for (size_t i = 0; i < r.size(); ++i) out[i] = r[i];
    });
}

double ao_clamped_swiglu(double gate, double up, double limit, int mode) {
    return clamped_swiglu(gate, up, limit, static_cast<ClampMode>(mode));
}

// One routed expert on one activation vector. hidden_out (size I), gate_out/up_out
// (size I) are optional.
int ao_expert_ffn(const LayoutArgs* a, const uint8_t* payload, const double* x, double limit,
                  int clamp_mode, double* out, double* hidden_out, double* gate_out,
                  double* up_out) {
    return guarded([&] {
        const ExpertLayout L = layout_of(a);
        const size_t H = static_cast<size_t>(a->hidden), I = static_cast<size_t>(a->intermediate);
        const DecodedExpertWeights d = decode_expert_weights(payload, L);
        const std::vector<double> xv(x, x + H);
        ExpertGateUp pre;
        const std::vector<double> h = expert_hidden_decoded(
            d.w1, d.w3, I, H, xv, limit, static_cast<ClampMode>(clamp_mode), &pre);
        const std::vector<double> y = matvec(H, I, h,
            [&](size_t o, size_t i) { return d.w2[o * I + i]; });
        std::memcpy(out, y.data(), H * sizeof(double));
        if (hidden_out) std::memcpy(hidden_out, h.data(), I * sizeof(double));
        if (gate_out) std::memcpy(gate_out, pre.gate.data(), I * sizeof(double));
        if (up_out) std::memcpy(up_out, pre.up.data(), I * sizeof(double));
    });
}

// The same expert on `tokens` activation vectors (decode once, reuse), x[T,H] -> out[T,H].
int ao_expert_ffn_batch(const LayoutArgs* a, const uint8_t* payload, const double* x, int tokens,
                        double limit, double* out) {
    return guarded([&] {
        const ExpertLayout L = layout_of(a);
        const size_t H = static_cast<size_t>(a->hidden), I = static_cast<size_t>(a->intermediate);
        const DecodedExpertWeights d = decode_expert_weights(payload, L);
        for (int t = 0; t < tokens; ++t) {
            const std::vector<double> xv(x + t * H, x + (t + 1) * H);
            const std::vector<double> y = expert_ffn_decoded(d, I, H, xv, limit);
            std::memcpy(out + t * H, y.data(), H * sizeof(double));
        }
    });
}

int ao_dense_ffn(const uint16_t* w1, const uint16_t* w3, const uint16_t* w2, int dtype,
                 int intermediate, int hidden, const double* x, double limit, double* out) {
    return guarded([&] {
        const size_t H = static_cast<size_t>(hidden), I = static_cast<size_t>(intermediate);
        const Dtype16 dt = static_cast<Dtype16>(dtype);
        std::vector<double> a(I * H), b(I * H), c(H * I);
        for (size_t i = 0; i < I * H; ++i) {
            a[i] = bits16_to_double(w1[i], dt);
            b[i] = bits16_to_double(w3[i], dt);
            c[i] = bits16_to_double(w2[i], dt);
        }
        const std::vector<double> y = dense_ffn(I, H, std::vector<double>(x, x + H), a, b, c, limit);
        std::memcpy(out, y.data(), H * sizeof(double));
    });
}

// routed_sum (slot order) + shared. expert_out[k, H], weights[k], shared[H] (nullable).
int ao_moe_combine(const double* expert_out, const double* weights, int k, int hidden,
                   const double* shared, double* out) {
    return guarded([&] {
        std::vector<std::vector<double>> eo(static_cast<size_t>(k));
        for (int i = 0; i < k; ++i)
            eo[i].assign(expert_out + static_cast<size_t>(i) * hidden,
                         expert_out + static_cast<size_t>(i + 1) * hidden);
        std::vector<double> sh;
        if (shared) sh.assign(shared, shared + hidden);
        const std::vector<double> y =
            moe_combine(eo, std::vector<double>(weights, weights + k), sh);
        std::memcpy(out, y.data(), sizeof(double) * hidden);
    });
}

// One whole MoE layer on one token, the timed unit of the CPU baseline:
// router logits -> top-k -> k routed experts (payloads generated by the caller)
// -> shared expert -> combine. payloads[k] are the selected experts' payloads in
// slot order. Returns the layer output in out[H].
int ao_moe_layer_token(const LayoutArgs* a, const uint8_t* const* payloads, const double* weights,
                       int top_k, const uint16_t* sw1, const uint16_t* sw3, const uint16_t* sw2,
                       int shared_dtype, const double* x, double limit, double* out) {
    return guarded([&] {
        const ExpertLayout L = layout_of(a);
        const size_t H = static_cast<size_t>(a->hidden), I = static_cast<size_t>(a->intermediate);
        const std::vector<double> xv(x, x + H);
        std::vector<std::vector<double>> eo;
        for (int k = 0; k < top_k; ++k) eo.push_back(expert_ffn(payloads[k], L, xv, limit));
        std::vector<double> sh;
        if (sw1) {
            const Dtype16 dt = static_cast<Dtype16>(shared_dtype);
            std::vector<double> p(I * H), q(I * H), r(H * I);
            for (size_t i = 0; i < I * H; ++i) {
                p[i] = bits16_to_double(sw1[i], dt);
                q[i] = bits16_to_double(sw3[i], dt);
                r[i] = bits16_to_double(sw2[i], dt);
            }
            sh = dense_ffn(I, H, xv, p, q, r, limit);
        }
        const std::vector<double> y =
            moe_combine(eo, std::vector<double>(weights, weights + top_k), sh);
        std::memcpy(out, y.data(), sizeof(double) * H);
    });
}

// stats[0..3] = max_abs, max_rel, rms_abs, rel_l2
int ao_compare(const double* want, const double* got, uint64_t n, double rel_floor, double* stats) {
    return guarded([&] {
        const ErrorStats s = compare(std::vector<double>(want, want + n),
                                     std::vector<double>(got, got + n), rel_floor);
        stats[0] = s.max_abs;
        stats[1] = s.max_rel;
        stats[2] = s.rms_abs;
        stats[3] = s.rel_l2;
    });
}

// FNV-1a over a byte range (fixture checksums).
uint64_t ao_fnv1a(const uint8_t* data, uint64_t bytes) {
    uint64_t h = 0xCBF29CE484222325ull;
    for (uint64_t i = 0; i < bytes; ++i) { h ^= data[i]; h *= 0x100000001B3ull; }
    return h;
}

// dense_ffn on fp64 weights (row-major [I,H], [I,H], [H,I]).
int ao_dense_ffn_f64(const double* w1, const double* w3, const double* w2, int intermediate,
                     int hidden, const double* x, double limit, double* out) {
    return guarded([&] {
        const size_t H = static_cast<size_t>(hidden), I = static_cast<size_t>(intermediate);
        const std::vector<double> y = dense_ffn(
            I, H, std::vector<double>(x, x + H), std::vector<double>(w1, w1 + I * H),
            std::vector<double>(w3, w3 + I * H), std::vector<double>(w2, w2 + H * I), limit);
        std::memcpy(out, y.data(), H * sizeof(double));
    });
}

// Front of the FFN half of a layer: residual streams [hc, hidden] -> mix coefficients and
// the normalised FFN input. mixes_out [hc*(hc+2)], pre_out / post_out [hc], comb_out [hc*hc],
// ffn_pre_out / ffn_norm_out [hidden]; norm_weight may be null (weightless RMSNorm).
int ao_ffn_front(const double* res_mid, int hidden, int hc, const float* hc_fn, const float* hc_base,
                 const float* hc_scale3, const double* norm_weight, double norm_eps, double* mixes_out,
                 double* pre_out, double* post_out, double* comb_out, double* ffn_pre_out,
                 double* ffn_norm_out) {
    return guarded([&] {
        const size_t H = static_cast<size_t>(hidden), S = static_cast<size_t>(hc);
        const std::vector<double> res(res_mid, res_mid + S * H);
        const std::vector<double> w = norm_weight ? std::vector<double>(norm_weight, norm_weight + H)
                                                  : std::vector<double>(H, 1.0);
        const FfnFront f = ffn_front(res, H, hc_fn, hc_base, hc_scale3, w, norm_eps, HcParams{});
        std::memcpy(mixes_out, f.hc.mixes.data(), f.hc.mixes.size() * sizeof(double));
        std::memcpy(pre_out, f.hc.pre_mix.data(), S * sizeof(double));
        std::memcpy(post_out, f.hc.post_mix.data(), S * sizeof(double));
        std::memcpy(comb_out, f.hc.comb.data(), S * S * sizeof(double));
        std::memcpy(ffn_pre_out, f.ffn_pre.data(), H * sizeof(double));
        std::memcpy(ffn_norm_out, f.ffn_norm.data(), H * sizeof(double));
    });
}

// out[hc, hidden] = post expansion of the layer output back to the residual streams.
int ao_hc_post(const double* layer_out, const double* residual, const double* post_mix, const double* comb,
               int hidden, int hc, int transpose_comb, double* out) {
    return guarded([&] {
        const size_t H = static_cast<size_t>(hidden), S = static_cast<size_t>(hc);
        const std::vector<double> y = hc_post(std::vector<double>(layer_out, layer_out + H),
                                              std::vector<double>(residual, residual + S * H),
                                              std::vector<double>(post_mix, post_mix + S),
                                              std::vector<double>(comb, comb + S * S), H, transpose_comb != 0);
        std::memcpy(out, y.data(), S * H * sizeof(double));
    });
}

}  // extern "C"
