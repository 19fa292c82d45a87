// Thin inline-PTX wrappers used by the sm_100a kernels: shared-memory barriers
// (mbarrier), bulk asynchronous copies (the TMA engine's untiled form), the
// warp-level 16x8x16 MMA, and the int4 -> fp16 register unpack.
#pragma once

#include <cuda_fp16.h>
#include <cstdint>

namespace aeon_b200 {
namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}

__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async;" ::: "memory");
}

// Shared-memory-only form: orders this thread's shared-memory writes before later
// async-proxy reads (tensor core, TMA) without waiting on its global loads in flight.
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait. Returns false when the iteration budget ran out, or at once when
// `error_flag` is already set: after the first failure every later wait of the launch falls
// through, so the kernel keeps its barrier structure (nobody is left alone at a bar.sync)
// and ends quickly. The caller records the failure in the flag.
constexpr uint32_t kWaitBudget = 1u << 21;

__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity,
                                          const volatile int32_t* error_flag) {
    for (uint32_t i = 0; i < kWaitBudget; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 255u) == 255u && *error_flag != 0) return false;
    }
    return false;
}

__device__ __forceinline__ uint64_t policy_evict_first() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}

__device__ __forceinline__ uint64_t policy_evict_last() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
    return p;
}

// Untiled bulk copy global -> shared, completion counted in bytes on `bar`.
// Both addresses 16-byte aligned, `bytes` a multiple of 16.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes,
                                         uint32_t bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
        "[%0], [%1], %2, [%3], %4;" ::"r"(dst), "l"(src), "r"(bytes), "r"(bar), "l"(policy)
        : "memory");
}

__device__ __forceinline__ void named_bar_sync(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "r"(addr));
    return v;
}

__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}

__device__ __forceinline__ float lds_half_as_float(uint32_t addr) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
    return __half2float(__ushort_as_half(v));
}

// D += A(16x16, row) * B(16x8, col), fp16 operands, fp32 accumulate.
__device__ __forceinline__ void mma_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                        uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int kLut>
__device__ __forceinline__ uint32_t lop3(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, %4;" : "=r"(r) : "r"(a), "r"(b), "r"(c), "n"(kLut));
    return r;
}

__device__ __forceinline__ uint32_t hsub2_u32(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("sub.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}

__device__ __forceinline__ uint32_t hfma2_u32(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t r;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
    return r;
}

// One swizzled 32-bit word holds eight consecutive columns of a row, nibble
// position p = column 2p (p < 4) or column 2(p-4)+1 (p >= 4), so the 16-bit
// halves of (word >> 4p) & 0x000F000F are the column pair (2p, 2p+1). OR-ing
// 0x6400 into a half gives the fp16 number 1024 + nibble (or 1024 + 16*nibble
// for the nibble one position up), from which the signed value nibble - 8 is
// one exact half2 operation away. Output: pairs[p] = fp16x2 (q(2p), q(2p+1)).
__device__ __forceinline__ void unpack_word(uint32_t w, uint32_t (&pairs)[4]) {
    constexpr uint32_t kMagic = 0x64006400u;      // 1024.0 | 1024.0
    constexpr uint32_t k1032 = 0x64086408u;       // 1032.0
    constexpr uint32_t kSixteenth = 0x2C002C00u;  // 1/16
    constexpr uint32_t kMinus72 = 0xD480D480u;    // -72.0
    constexpr int kAndOr = (0xF0 & 0xCC) | 0xAA;  // (a & b) | c
    const uint32_t w8 = w >> 8;
    const uint32_t p0 = lop3<kAndOr>(w, 0x000F000Fu, kMagic);
    const uint32_t p1 = lop3<kAndOr>(w, 0x00F000F0u, kMagic);
    const uint32_t p2 = lop3<kAndOr>(w8, 0x000F000Fu, kMagic);
    const uint32_t p3 = lop3<kAndOr>(w8, 0x00F000F0u, kMagic);
    pairs[0] = hsub2_u32(p0, k1032);
    pairs[1] = hfma2_u32(p1, kSixteenth, kMinus72);
    pairs[2] = hsub2_u32(p2, k1032);
    pairs[3] = hfma2_u32(p3, kSixteenth, kMinus72);
}

// Cheaper form used by the streaming kernels. The masked bits of a swizzled word are
// already valid fp16 numbers: (w & 0x000F000F) read as two fp16 values is the pair of
// SUBNORMALS nibble * 2^-24, and (w & 0x00F000F0) is nibble * 2^-20. The tensor core takes
// fp16 subnormals at full precision, so the unsigned nibbles can go into the MMA as they are
// (one AND per column pair, no subtract); the power-of-two factor and the zero point are
// applied once per scale group in fp32:
//     sum_k (u_k - 8) x_k  =  2^24 * (T_lo + T_hi / 16)  -  8 * sum_k x_k
// where T_lo / T_hi accumulate the low-plane / high-plane products (they need separate
// accumulators because their factors differ) and sum_k x_k is a per-(token, group) constant.
// One word (8 columns of rows g and g+8) costs two MMAs: the low plane holds columns
// {0,1} and {4,5} of the word, the high plane {2,3} and {6,7}; `b` holds the token's
// activations for the 8 columns as (x,y,z,w) = column pairs (0,1),(2,3),(4,5),(6,7).
__device__ __forceinline__ void mma_word(float (&tlo)[4], float (&thi)[4], uint32_t wa, uint32_t wb,
                                         const uint4& b) {
    const uint32_t wa8 = wa >> 8, wb8 = wb >> 8;
    mma_f16(tlo, wa & 0x000F000Fu, wb & 0x000F000Fu, wa8 & 0x000F000Fu, wb8 & 0x000F000Fu, b.x, b.z);
    mma_f16(thi, wa & 0x00F000F0u, wb & 0x00F000F0u, wa8 & 0x00F000F0u, wb8 & 0x00F000F0u, b.y, b.w);
}

// acc += scale * (2^24 * (tlo + thi/16) - 8 * xsum): rows g (sa) and g+8 (sb), token
// columns 2t (xs.x) and 2t+1 (xs.y).
__device__ __forceinline__ void fold_group(float (&acc)[4], const float (&tlo)[4],
                                           const float (&thi)[4], float sa, float sb, float2 xs) {
    const float sa24 = sa * 16777216.0f, sb24 = sb * 16777216.0f;
    const float sa8 = -8.0f * sa, sb8 = -8.0f * sb;
    acc[0] = fmaf(sa24, fmaf(thi[0], 0.0625f, tlo[0]), fmaf(sa8, xs.x, acc[0]));
    acc[1] = fmaf(sa24, fmaf(thi[1], 0.0625f, tlo[1]), fmaf(sa8, xs.y, acc[1]));
    acc[2] = fmaf(sb24, fmaf(thi[2], 0.0625f, tlo[2]), fmaf(sb8, xs.x, acc[2]));
    acc[3] = fmaf(sb24, fmaf(thi[3], 0.0625f, tlo[3]), fmaf(sb8, xs.y, acc[3]));
}

// ---- single-accumulator form (row-streaming kernels) -------------------------------------------
// When the activations of the columns that meet the high-nibble plane (columns 2, 3, 6, 7 of
// every 8: bit 1 of the column index) are stored divided by 16 -- exact in fp16 above the
// subnormal range, within 2^-25 absolute below it -- both planes carry the factor 2^-24 and can
// share one accumulator:
//     sum_k (u_k - 8) x_k  =  2^24 * T  -  8 * sum_k x_k
// which halves the accumulator registers and drops the plane-merging multiply-add.

// D = A * B with a zero addend (the first MMA of a chain: no accumulator to clear beforehand).
__device__ __forceinline__ void mma_f16_first(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                              uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
}

// The two nibble planes of a word pair (rows g and g+8) as MMA A fragments.
struct WordPlanes {
    uint32_t lo[4], hi[4];
};

__device__ __forceinline__ WordPlanes word_planes(uint32_t wa, uint32_t wb) {
    const uint32_t wa8 = wa >> 8, wb8 = wb >> 8;
    WordPlanes p;
    p.lo[0] = wa & 0x000F000Fu; p.lo[1] = wb & 0x000F000Fu; p.lo[2] = wa8 & 0x000F000Fu; p.lo[3] = wb8 & 0x000F000Fu;
    p.hi[0] = wa & 0x00F000F0u; p.hi[1] = wb & 0x00F000F0u; p.hi[2] = wa8 & 0x00F000F0u; p.hi[3] = wb8 & 0x00F000F0u;
    return p;
}

// T (+)= planes * b: b = the token's activations for the word's 8 columns as column pairs
// (0,1),(2,3),(4,5),(6,7), pairs (2,3) and (6,7) pre-divided by 16. kFirst starts the chain.
template <bool kFirst>
__device__ __forceinline__ void mma_planes(float (&T)[4], const WordPlanes& p, const uint4& b) {
    if constexpr (kFirst) mma_f16_first(T, p.lo[0], p.lo[1], p.lo[2], p.lo[3], b.x, b.z);
    else mma_f16(T, p.lo[0], p.lo[1], p.lo[2], p.lo[3], b.x, b.z);
    mma_f16(T, p.hi[0], p.hi[1], p.hi[2], p.hi[3], b.y, b.w);
}

// acc += scale * (2^24 * T + xs8) with xs8 = -8 * (token, group) activation sum: rows g (sa)
// and g+8 (sb), token columns 2t (xs8.x) and 2t+1 (xs8.y).
__device__ __forceinline__ void fold_single(float (&acc)[4], const float (&T)[4], float sa, float sb, float2 xs8) {
    acc[0] = fmaf(sa, fmaf(T[0], 16777216.0f, xs8.x), acc[0]);
    acc[1] = fmaf(sa, fmaf(T[1], 16777216.0f, xs8.y), acc[1]);
    acc[2] = fmaf(sb, fmaf(T[2], 16777216.0f, xs8.x), acc[2]);
    acc[3] = fmaf(sb, fmaf(T[3], 16777216.0f, xs8.y), acc[3]);
}

// The two fp16 halves of a 32-bit word as fp32.
__device__ __forceinline__ float half_lo_as_float(uint32_t bits) {
    return __low2float(*reinterpret_cast<const __half2*>(&bits));
}
__device__ __forceinline__ float half_hi_as_float(uint32_t bits) {
    return __high2float(*reinterpret_cast<const __half2*>(&bits));
}

__device__ __forceinline__ float2 lds_f2(uint32_t addr) {
    float2 v;
    asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(addr));
    return v;
}

__device__ __forceinline__ uint2 lds64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}

__device__ __forceinline__ uint32_t lds16(uint32_t addr) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
    return v;
}

}  // namespace ptx
}  // namespace aeon_b200
