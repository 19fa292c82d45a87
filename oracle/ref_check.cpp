// TEST INFRASTRUCTURE — NOT A PRODUCT PATH.
//
// Pins the CPU restatement (aeon_oracle.hpp) against the UNMODIFIED reference
// headers, compiled from where they lie (see oracle/Makefile: the include path
// points into the reference tree; no reference source is copied). At the
// reference's own shapes every restated function must agree bit-for-bit with the
// function it follows. With `--golden <path>` it also writes the reference's own
// outputs for a set of seeded cases to a JSON fixture, so the restatement can be
// re-checked on machines where the reference tree is absent.
//
// Reference headers used:
//   src/architecture/deepseek_v4/reference/dsv4_oracle.hpp   (fp64 host oracle)
//   src/backend/swizzled_w4a16/kernels/aeon_w4a16_swizzle.hpp (host swizzle)
#include "architecture/deepseek_v4/reference/dsv4_oracle.hpp"
#include "backend/swizzled_w4a16/kernels/aeon_w4a16_swizzle.hpp"

#include "aeon_oracle.hpp"

#include <cinttypes>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

namespace ref = aeon::reference;
namespace ao = aeon_oracle;

namespace {

int g_failures = 0;

void check(const char* label, bool ok) {
    std::printf("  %-64s %s\n", label, ok ? "PASS" : "FAIL");
    if (!ok) ++g_failures;
}

bool bit_equal(const std::vector<double>& a, const std::vector<double>& b) {
    return a.size() == b.size() &&
           (a.empty() || std::memcmp(a.data(), b.data(), a.size() * sizeof(double)) == 0);
}

uint64_t fnv1a(const void* data, size_t bytes) {
    const uint8_t* p = static_cast<const uint8_t*>(data);
    uint64_t h = 0xCBF29CE484222325ull;
    for (size_t i = 0; i < bytes; ++i) { h ^= p[i]; h *= 0x100000001B3ull; }
    return h;
}

void json_doubles(FILE* f, const char* key, const std::vector<double>& v, bool last = false) {
    // Hex-float keeps every bit; Python's float.fromhex reads it back exactly.
    std::fprintf(f, "  \"%s\": [", key);
    for (size_t i = 0; i < v.size(); ++i) std::fprintf(f, "%s\"%a\"", i ? ", " : "", v[i]);
    std::fprintf(f, "]%s\n", last ? "" : ",");
}

void json_ints(FILE* f, const char* key, const std::vector<int32_t>& v) {
    std::fprintf(f, "  \"%s\": [", key);
    for (size_t i = 0; i < v.size(); ++i) std::fprintf(f, "%s%d", i ? ", " : "", v[i]);
    std::fprintf(f, "],\n");
}

ao::MatrixLayout layout_for(ref::SwizzledKind kind, const ao::ExpertLayout& L) {
    switch (kind) {
        case ref::SwizzledKind::W1: return L.w1;
        case ref::SwizzledKind::W2: return L.w2;
        case ref::SwizzledKind::W3: return L.w3;
    }
    return L.w1;
}

}  // namespace

int main(int argc, char** argv) {
    const char* golden_path = nullptr;
    for (int i = 1; i + 1 < argc; ++i)
        if (std::string(argv[i]) == "--golden") golden_path = argv[i + 1];

    std::printf("[ref_check] restatement vs unmodified reference headers (reference shapes)\n");

    // --- Rng -----------------------------------------------------------------
    {
        ref::Rng a(0x0E7E1217ull);
        ao::Rng b(0x0E7E1217ull);
        bool same = true;
        for (int i = 0; i < 100000; ++i) same &= (a.next_u64() == b.next_u64());
        ref::Rng c(0), d0(0x1207E8C0ull);
        ao::Rng e(0), d1(0x1207E8C0ull);
        for (int i = 0; i < 1000; ++i) {
            same &= (c.symmetric(4.0) == e.symmetric(4.0));
            same &= (d0.uniform01() == d1.uniform01());
        }
        check("Rng: SplitMix64 stream, uniform01, symmetric", same);
    }

    // --- fp16 widening over every bit pattern --------------------------------
    {
        bool same = true;
        for (uint32_t bits = 0; bits < 65536; ++bits) {
            const double a = ref::half_bits_to_double(static_cast<uint16_t>(bits));
            const double b = ao::half_bits_to_double(static_cast<uint16_t>(bits));
            same &= (std::memcmp(&a, &b, sizeof(a)) == 0) || (std::isnan(a) && std::isnan(b));
            if (!std::isnan(a) && !std::isinf(a)) {
                same &= (ao::double_to_half_bits(a) == static_cast<uint16_t>(bits)) ||
                        (a == 0.0);   // +-0 keep their sign; checked separately
            }
        }
        same &= ao::double_to_half_bits(0.0) == 0 && ao::double_to_half_bits(-0.0) == 0x8000;
        for (int e = -20; e <= 20; ++e)
            same &= ref::half_bits_of_power_of_two(e) == ao::half_bits_of_power_of_two(e);
        check("half_bits_to_double (65536 patterns) + exact inverse", same);
    }

    const ao::ExpertLayout L = ao::make_expert_layout(4096, 2048, 32);
    check("payload geometry = 14,155,776 B and the reference region offsets",
          L.payload_bytes == 14155776u &&
          L.w1.packed_offset == ref::swizzled_shape(ref::SwizzledKind::W1).packed_offset &&
          L.w1.scale_offset == ref::swizzled_shape(ref::SwizzledKind::W1).scale_offset &&
          L.w2.packed_offset == ref::swizzled_shape(ref::SwizzledKind::W2).packed_offset &&
          L.w2.scale_offset == ref::swizzled_shape(ref::SwizzledKind::W2).scale_offset &&
          L.w3.packed_offset == ref::swizzled_shape(ref::SwizzledKind::W3).packed_offset &&
          L.w3.scale_offset == ref::swizzled_shape(ref::SwizzledKind::W3).scale_offset);

    // --- swizzled_address, every element of every matrix ----------------------
    {
        bool same = true;
        const ref::SwizzledKind kinds[3] = {ref::SwizzledKind::W1, ref::SwizzledKind::W2,
                                            ref::SwizzledKind::W3};
        for (ref::SwizzledKind kind : kinds) {
            const ref::SwizzledShape shape = ref::swizzled_shape(kind);
            const ao::MatrixLayout m = layout_for(kind, L);
            for (int row = 0; row < shape.rows; row += 3)
                for (int col = 0; col < shape.columns; ++col) {
                    const ref::SwizzledAddress a = ref::swizzled_address(shape, row, col);
                    const ao::SwizzledAddress b = ao::swizzled_address(m, row, col);
                    same &= a.storage_slot == b.scale_slot && a.packed_word == b.packed_word &&
                            a.nibble == b.nibble;
                }
        }
        check("swizzled_address for W1/W2/W3 (every third row, every column)", same);
    }

    // --- encode / decode / expert FFN on the reference's own fixture ----------
    // Same seed and draw order as tests/test_v4_expert_oracle.cpp:116-130.
    ref::Rng gen(0x0E7E1217ull);
    std::vector<double> src_w1(2048 * 4096), src_w3(2048 * 4096), src_w2(4096 * 2048);
    for (double& v : src_w1) v = gen.symmetric(0.06);
    for (double& v : src_w3) v = gen.symmetric(0.06);
    for (double& v : src_w2) v = gen.symmetric(0.06);
    std::vector<uint8_t> payload_ref(L.payload_bytes, 0), payload_ao(L.payload_bytes, 0);
    ref::swizzled_encode(payload_ref.data(), ref::SwizzledKind::W1, src_w1);
    ref::swizzled_encode(payload_ref.data(), ref::SwizzledKind::W3, src_w3);
    ref::swizzled_encode(payload_ref.data(), ref::SwizzledKind::W2, src_w2);
    ao::swizzled_encode(payload_ao.data(), L.w1, src_w1);
    ao::swizzled_encode(payload_ao.data(), L.w3, src_w3);
    ao::swizzled_encode(payload_ao.data(), L.w2, src_w2);
    check("swizzled_encode: payload bytes identical", payload_ref == payload_ao);

    const std::vector<double> dec_ref = ref::swizzled_decode(payload_ref.data(), ref::SwizzledKind::W2);
    check("swizzled_decode W2: bit-identical",
          bit_equal(dec_ref, ao::swizzled_decode(payload_ref.data(), L.w2)));
    check("swizzled_decode W1: bit-identical",
          bit_equal(ref::swizzled_decode(payload_ref.data(), ref::SwizzledKind::W1),
                    ao::swizzled_decode(payload_ref.data(), L.w1)));
    {
        ref::SwizzledDecodeOptions ro; ro.signed_zero_point = false;
        ao::SwizzledDecodeOptions oo; oo.signed_zero_point = false;
        bool same = bit_equal(ref::swizzled_decode(payload_ref.data(), ref::SwizzledKind::W3, ro),
                              ao::swizzled_decode(payload_ref.data(), L.w3, oo));
        ref::SwizzledDecodeOptions rp; rp.permute_nibbles = false;
        ao::SwizzledDecodeOptions op; op.permute_nibbles = false;
        same &= bit_equal(ref::swizzled_decode(payload_ref.data(), ref::SwizzledKind::W3, rp),
                          ao::swizzled_decode(payload_ref.data(), L.w3, op));
        check("swizzled_decode wrong-variant controls: bit-identical", same);
    }

    // Host swizzle of a source-layout matrix (the loader-side transform).
    {
        // Source words from the reference tests' formula
        // (tests/test_w2_shard_equivalence.cpp:80-87).
        auto make_source_word = [](size_t i, int seed) {
            uint32_t w = 0;
            for (int n = 0; n < 8; ++n) w |= static_cast<uint32_t>((i * 3 + n * 5 + seed) % 16) << (4 * n);
            return w;
        };
        const int N = 4096, K = 2048;
        std::vector<uint32_t> sp(static_cast<size_t>(N) * K / 8), dp(sp.size());
        std::vector<uint16_t> ss(static_cast<size_t>(N) * K / 32), ds(ss.size());
        for (size_t i = 0; i < sp.size(); ++i) sp[i] = make_source_word(i, 7);
        for (size_t i = 0; i < ss.size(); ++i)
            ss[i] = ao::double_to_half_bits(std::ldexp(1.0 + static_cast<double>((i + 7) % 29), -8));
        aeon::swizzle_w4a16<uint16_t>(sp.data(), ss.data(), dp.data(), ds.data(), N, K, aeon::kCfgW2);
        std::vector<uint8_t> pay(L.payload_bytes, 0);
        ao::swizzle_from_source(sp.data(), ss.data(), pay.data(), L.w2);
        const bool same =
            std::memcmp(pay.data() + L.w2.packed_offset, dp.data(), dp.size() * 4) == 0 &&
            std::memcmp(pay.data() + L.w2.scale_offset, ds.data(), ds.size() * 2) == 0;
        check("swizzle_from_source == reference swizzle_w4a16 (W2 shape)", same);
    }

    ref::Rng agen(0xAC7100ull);
    std::vector<double> activation(4096);
    for (double& v : activation) v = agen.symmetric(1.0);
    const std::vector<double> ffn_ref = ref::expert_ffn(payload_ref.data(), activation);
    const std::vector<double> ffn_ao = ao::expert_ffn(payload_ref.data(), L, activation);
    check("expert_ffn (decode + W1/W3 + clamped SwiGLU + W2): bit-identical",
          bit_equal(ffn_ref, ffn_ao));
    {
        std::vector<double> big = activation;
        for (double& v : big) v *= 8.0;   // drives gate/up past the clamp
        bool same = bit_equal(ref::expert_ffn(payload_ref.data(), big),
                              ao::expert_ffn(payload_ref.data(), L, big));
        same &= bit_equal(ref::expert_ffn(payload_ref.data(), big, 10.0, ref::ClampMode::Symmetric),
                          ao::expert_ffn(payload_ref.data(), L, big, 10.0, ao::ClampMode::Symmetric));
        check("expert_ffn at 8x activations, asymmetric and symmetric clamp", same);
    }

    // --- clamped SwiGLU probes (tests/test_v4_expert_oracle.cpp:302) ---------
    std::vector<double> swiglu_out;
    {
        const double probes[8] = {-40, -12, -5, 0, 5, 12, 40, 3};
        bool same = true;
        for (double g : probes)
            for (double u : probes)
                for (int mode = 0; mode < 3; ++mode) {
                    const double a = ref::clamped_swiglu(g, u, 10.0, static_cast<ref::ClampMode>(mode));
                    const double b = ao::clamped_swiglu(g, u, 10.0, static_cast<ao::ClampMode>(mode));
                    same &= std::memcmp(&a, &b, sizeof(a)) == 0;
                    if (mode == 0) swiglu_out.push_back(a);
                }
        check("clamped_swiglu probes x 3 clamp modes", same);
    }

    // --- router --------------------------------------------------------------
    // Seed and ranges of tests/test_v4_router_oracle.cpp:179,226-228.
    ref::Rng rgen(0x1207E8C0ull);
    std::vector<double> logits(256), bias(256);
    for (double& x : logits) x = static_cast<double>(static_cast<float>(rgen.symmetric(4.0)));
    for (double& b : bias) b = static_cast<double>(static_cast<float>(rgen.symmetric(0.5)));
    const ref::RouterSelection rsel = ref::router_topk(logits, bias, 6, 1.5);
    const ao::RouterSelection asel = ao::router_topk(logits, bias, 6, 1.5);
    check("router_topk (sqrt-softplus, bias, top-6, x1.5): ids + weights",
          rsel.ids == asel.ids && bit_equal(rsel.weights, asel.weights));
    {
        const ref::RouterSelection r0 = ref::router_topk(logits, {}, 6, 1.5);
        const ao::RouterSelection a0 = ao::router_topk(logits, {}, 6, 1.5);
        const ref::RouterSelection r1 = ref::router_topk(logits, bias, 6, 1.5, true);
        const ao::RouterSelection a1 = ao::router_topk(logits, bias, 6, 1.5,
                                                       ao::ScoreFn::SqrtSoftplus, true, true);
        check("router_topk without bias, and the bias-before-softplus control",
              r0.ids == a0.ids && bit_equal(r0.weights, a0.weights) && r1.ids == a1.ids &&
                  bit_equal(r1.weights, a1.weights));
    }
    std::vector<int32_t> tie_ids;
    {
        std::vector<double> tied(256, 0.0);
        tied[7] = tied[70] = tied[180] = tied[255] = 3.0;
        const ref::RouterSelection r = ref::router_topk(tied, {}, 6, 1.5);
        const ao::RouterSelection a = ao::router_topk(tied, {}, 6, 1.5);
        tie_ids = r.ids;
        check("four-way tie resolves to the lowest indices (7, 70, 180, 255, 0, 1)",
              r.ids == a.ids && r.ids[0] == 7 && r.ids[1] == 70 && r.ids[2] == 180 &&
                  r.ids[3] == 255 && r.ids[4] == 0 && r.ids[5] == 1);
    }
    std::vector<int32_t> hash_ids;
    std::vector<double> hash_w;
    {
        const std::vector<int64_t> row = {200, 3, 77, 150, 9, 31};
        const ref::RouterSelection r = ref::router_hash(logits, row, 1.5);
        const ao::RouterSelection a = ao::router_hash(logits, row, 1.5);
        hash_ids = r.ids;
        hash_w = r.weights;
        check("router_hash: ids in table order + weights", r.ids == a.ids &&
                                                              bit_equal(r.weights, a.weights));
    }

    // --- dense FFN (shared expert), small shape -------------------------------
    std::vector<double> dense_out;
    {
        ref::Rng dgen(0x5A4ED00ull);
        const size_t I = 96, H = 160;
        std::vector<double> x = dgen.vector_filled(H, 1.0), w1 = dgen.vector_filled(I * H, 0.3),
                            w3 = dgen.vector_filled(I * H, 0.3), w2 = dgen.vector_filled(H * I, 0.3);
        dense_out = ref::dense_ffn(I, H, x, w1, w3, w2);
        ao::Rng dgen2(0x5A4ED00ull);
        std::vector<double> x2 = dgen2.vector_filled(H, 1.0), v1 = dgen2.vector_filled(I * H, 0.3),
                            v3 = dgen2.vector_filled(I * H, 0.3), v2 = dgen2.vector_filled(H * I, 0.3);
        check("dense_ffn (shared expert): bit-identical",
              bit_equal(dense_out, ao::dense_ffn(I, H, x2, v1, v3, v2)));
    }

    // --- compare() -------------------------------------------------------------
    {
        std::vector<double> noisy = ffn_ref;
        for (size_t i = 0; i < noisy.size(); i += 5) noisy[i] *= 1.0 + 1e-4;
        const ref::ErrorStats a = ref::compare(ffn_ref, noisy);
        const ao::ErrorStats b = ao::compare(ffn_ref, noisy);
        check("compare(): max_abs / max_rel / rms identical",
              a.max_abs == b.max_abs && a.max_rel == b.max_rel && a.rms_abs == b.rms_abs &&
                  a.max_abs_index == b.max_abs_index);
    }

    // --- hyper-connection pre-mix, FFN RMSNorm, post expansion (the caller of the path) ---
    std::vector<double> hc_golden_front, hc_golden_post;
    {
        const size_t hidden = 192, hc = 4, n_mix = hc * (hc + 2);
        ref::Rng g(0x4C0FFEEull);
        const std::vector<double> res_mid = g.vector_filled(hc * hidden, 1.5);
        std::vector<float> fn(n_mix * hc * hidden), base(n_mix), scale(3);
        for (float& v : fn) v = static_cast<float>(g.symmetric(0.05));
        for (float& v : base) v = static_cast<float>(g.symmetric(0.5));
        for (float& v : scale) v = static_cast<float>(0.5 + g.uniform01());
        const std::vector<double> norm_w = g.vector_filled(hidden, 1.0);
        const std::vector<double> layer_out = g.vector_filled(hidden, 2.0);
        ref::HcParams rp;
        const std::vector<double> mixes_ref = ref::hc_mixes(
            res_mid, n_mix, [&](size_t m, size_t k) { return static_cast<double>(fn[m * hc * hidden + k]); },
            hc * hidden, rp.rms_eps);
        ref::HcPreResult rh;
        ref::hc_sinkhorn(mixes_ref, std::vector<double>(scale.begin(), scale.end()),
                         std::vector<double>(base.begin(), base.end()), hc, rp, rh);
        const std::vector<double> pre_ref = ref::hc_pre_combine(res_mid, rh.pre_mix, hidden);
        const std::vector<double> norm_ref = ref::rmsnorm(pre_ref, norm_w, 1e-6);
        const std::vector<double> post_ref = ref::hc_post(layer_out, res_mid, rh.post_mix, rh.comb, hidden);
        const std::vector<double> post_t_ref = ref::hc_post(layer_out, res_mid, rh.post_mix, rh.comb, hidden, true);

        ao::HcParams ap;
        const ao::FfnFront front = ao::ffn_front(res_mid, hidden, fn.data(), base.data(), scale.data(), norm_w, 1e-6, ap);
        check("hc_mixes + hc_sinkhorn (pre, post, comb): bit-identical",
              bit_equal(front.hc.mixes, mixes_ref) && bit_equal(front.hc.pre_mix, rh.pre_mix) &&
                  bit_equal(front.hc.post_mix, rh.post_mix) && bit_equal(front.hc.comb, rh.comb));
        check("hc_pre_combine + rmsnorm (FFN input): bit-identical",
              bit_equal(front.ffn_pre, pre_ref) && bit_equal(front.ffn_norm, norm_ref));
        check("rmsnorm_unit: bit-identical", bit_equal(ao::rmsnorm_unit(pre_ref, 1e-6), ref::rmsnorm_unit(pre_ref, 1e-6)));
        const std::vector<double> post_ao = ao::hc_post(layer_out, res_mid, front.hc.post_mix, front.hc.comb, hidden);
        check("hc_post and its transposed-comb control: bit-identical",
              bit_equal(post_ao, post_ref) &&
                  bit_equal(ao::hc_post(layer_out, res_mid, front.hc.post_mix, front.hc.comb, hidden, true), post_t_ref));
        // the control is a different answer, so the comb convention is pinned by the above
        check("transposed comb differs from the correct reading by > 1e-2",
              ref::compare(post_ref, post_t_ref).max_abs > 1e-2);
        // comb is doubly stochastic up to the eps terms
        bool stochastic = true;
        for (size_t i = 0; i < hc; ++i) {
            double row = 0.0, col = 0.0;
            for (size_t j = 0; j < hc; ++j) { row += rh.comb[i * hc + j]; col += rh.comb[j * hc + i]; }
            stochastic = stochastic && std::fabs(row - 1.0) < 1e-4 && std::fabs(col - 1.0) < 1e-4;
        }
        check("comb rows and columns sum to 1 within 1e-4", stochastic);
        hc_golden_front = front.hc.pre_mix;
        hc_golden_front.insert(hc_golden_front.end(), rh.post_mix.begin(), rh.post_mix.end());
        hc_golden_front.insert(hc_golden_front.end(), rh.comb.begin(), rh.comb.end());
        hc_golden_front.insert(hc_golden_front.end(), norm_ref.begin(), norm_ref.begin() + 16);
        hc_golden_post.assign(post_ref.begin(), post_ref.begin() + 16);
        hc_golden_post.insert(hc_golden_post.end(), post_ref.end() - 16, post_ref.end());
    }

    if (golden_path != nullptr) {
        FILE* f = std::fopen(golden_path, "w");
        if (!f) { std::perror("golden"); return 2; }
        std::fprintf(f, "{\n");
        std::fprintf(f, "  \"generator\": \"oracle/ref_check.cpp --golden, values produced by the reference's own functions\",\n");
        std::fprintf(f, "  \"expert_seed\": \"0x0E7E1217\", \"activation_seed\": \"0xAC7100\", \"router_seed\": \"0x1207E8C0\", \"dense_seed\": \"0x5A4ED00\",\n");
        std::fprintf(f, "  \"payload_fnv1a\": \"%016" PRIx64 "\",\n", fnv1a(payload_ref.data(), payload_ref.size()));
        std::fprintf(f, "  \"decoded_w2_fnv1a\": \"%016" PRIx64 "\",\n", fnv1a(dec_ref.data(), dec_ref.size() * sizeof(double)));
        std::fprintf(f, "  \"expert_ffn_fnv1a\": \"%016" PRIx64 "\",\n", fnv1a(ffn_ref.data(), ffn_ref.size() * sizeof(double)));
        json_doubles(f, "expert_ffn_first64", std::vector<double>(ffn_ref.begin(), ffn_ref.begin() + 64));
        json_ints(f, "router_ids", rsel.ids);
        json_doubles(f, "router_weights", rsel.weights);
        json_ints(f, "tie_ids", tie_ids);
        json_ints(f, "hash_ids", hash_ids);
        json_doubles(f, "hash_weights", hash_w);
        json_doubles(f, "swiglu_probe_grid", swiglu_out);
        json_doubles(f, "dense_ffn", dense_out);
        std::fprintf(f, "  \"hc_seed\": \"0x4C0FFEE\",\n");
        json_doubles(f, "hc_pre_post_comb_norm16", hc_golden_front);
        json_doubles(f, "hc_post_first16_last16", hc_golden_post, true);
        std::fprintf(f, "}\n");
        std::fclose(f);
        std::printf("  golden fixture written to %s\n", golden_path);
    }

    std::printf("[ref_check] %s (%d failure%s)\n", g_failures == 0 ? "ALL PASS" : "FAILED",
                g_failures, g_failures == 1 ? "" : "s");
    return g_failures == 0 ? 0 : 1;
}
