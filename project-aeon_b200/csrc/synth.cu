// Counter-based synthetic tensors, generated on the device so that benchmark pools
// (several GB per layer) never cross the bus. A value is a pure function of
// (seed, layer, expert, stream, index):
//   packed word i = low 32 bits of mix(key ^ (i+1) * GOLDEN)        -> eight uniform nibbles
//   scale j       = table[mix(key' ^ (j+1) * GOLDEN) & (n-1)]        -> fp16 bit pattern
//   dense value i = table[r & (n-1)] | sign(r >> 31)
// with mix = the SplitMix64 finaliser. The test oracle evaluates the same functions on the
// CPU, so device pools and oracle payloads are byte-identical by construction.
#include "common.cuh"

#include <algorithm>

namespace aeon_b200 {

namespace {

constexpr uint64_t kGolden = 0x9E3779B97F4A7C15ull;

__host__ __device__ __forceinline__ uint64_t mix64(uint64_t z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

__host__ __device__ __forceinline__ uint64_t synth_key(uint64_t seed, uint32_t layer,
                                                       uint32_t expert, uint32_t stream) {
    uint64_t k = mix64(seed + kGolden);
    k = mix64(k ^ (static_cast<uint64_t>(layer) + 1) * 0xD1B54A32D192ED03ull);
    k = mix64(k ^ (static_cast<uint64_t>(expert) + 1) * 0x8CB92BA72F3D8DD7ull);
    k = mix64(k ^ (static_cast<uint64_t>(stream) + 1) * 0xA0761D6478BD642Full);
    return k;
}

__device__ __forceinline__ uint32_t synth_u32(uint64_t key, uint64_t index) {
    return static_cast<uint32_t>(mix64(key ^ ((index + 1) * kGolden)));
}

struct SynthRegion {
    uint64_t offset;   // bytes from payload start
    uint64_t count;    // u32 words (packed) or u16 scales
};

struct SynthParams {
    uint8_t* pool;
    uint64_t payload_bytes;
    uint32_t first_slot, count, layer, first_expert;
    uint64_t seed;
    SynthRegion packed[3];
    SynthRegion scales[3];
    const uint16_t* table;
    uint32_t table_mask;
};

// grid.y = expert index within the call, grid.z = region (0..5), grid.x strides the region.
__global__ void synth_experts_kernel(const SynthParams p) {
    const uint32_t ei = blockIdx.y;
    const uint32_t region = blockIdx.z;
    const uint32_t m = region >> 1;
    uint8_t* payload = p.pool + static_cast<uint64_t>(p.first_slot + ei) * p.payload_bytes;
    const uint64_t key = synth_key(p.seed, p.layer, p.first_expert + ei, region);
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    if ((region & 1) == 0) {
        uint4* out = reinterpret_cast<uint4*>(payload + p.packed[m].offset);
        const uint64_t vecs = p.packed[m].count / 4;
        for (uint64_t v = blockIdx.x * static_cast<uint64_t>(blockDim.x) + threadIdx.x; v < vecs; v += stride) {
            uint4 w;
            w.x = synth_u32(key, 4 * v + 0);
            w.y = synth_u32(key, 4 * v + 1);
            w.z = synth_u32(key, 4 * v + 2);
            w.w = synth_u32(key, 4 * v + 3);
            out[v] = w;
        }
    } else {
        uint16_t* out = reinterpret_cast<uint16_t*>(payload + p.scales[m].offset);
        for (uint64_t j = blockIdx.x * static_cast<uint64_t>(blockDim.x) + threadIdx.x; j < p.scales[m].count; j += stride)
            out[j] = p.table[synth_u32(key, j) & p.table_mask];
    }
}

__global__ void synth_dense16_kernel(uint16_t* out, uint64_t count, uint64_t key,
                                     const uint16_t* table, uint32_t mask) {
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    for (uint64_t i = blockIdx.x * static_cast<uint64_t>(blockDim.x) + threadIdx.x; i < count; i += stride) {
        const uint32_t r = synth_u32(key, i);
        out[i] = static_cast<uint16_t>(table[r & mask] | ((r >> 31) << 15));
    }
}

}  // namespace

void launch_synth_experts(const aeon_b200_moe_config& cfg, void* pool_base, uint32_t first_slot,
                          uint32_t count, uint64_t seed, uint32_t layer, uint32_t first_expert,
                          const uint16_t* scale_table, uint32_t table_n, cudaStream_t stream) {
    require(pool_base && scale_table, "aeon_b200_synth_fill_experts: null pointer argument");
    require(table_n > 0 && (table_n & (table_n - 1)) == 0,
            "aeon_b200_synth_fill_experts: table_n must be a power of two");
    if (count == 0) return;
    const ExpertGeom g = make_geom(cfg);
    SynthParams p{};
    p.pool = static_cast<uint8_t*>(pool_base);
    p.payload_bytes = g.payload_bytes;
    p.first_slot = first_slot;
    p.count = count;
    p.layer = layer;
    p.first_expert = first_expert;
    p.seed = seed;
    const MatrixGeom* mats[3] = {&g.w1, &g.w2, &g.w3};
    for (int m = 0; m < 3; ++m) {
        const uint64_t weights = static_cast<uint64_t>(mats[m]->rows) * mats[m]->cols;
        p.packed[m] = {mats[m]->packed_offset, weights / 8};
        p.scales[m] = {mats[m]->scale_offset, weights / static_cast<uint64_t>(g.group)};
    }
    p.table = scale_table;
    p.table_mask = table_n - 1;
    // grid.y is limited to 65535 experts per launch.
    for (uint32_t done = 0; done < count; done += 32768) {
        SynthParams q = p;
        q.first_slot = first_slot + done;
        q.first_expert = first_expert + done;
        const uint32_t n = std::min<uint32_t>(32768, count - done);
        synth_experts_kernel<<<dim3(64, n, 6), 256, 0, stream>>>(q);
        AEON_CUDA_CHECK(cudaGetLastError());
    }
}

void launch_synth_dense16(void* out, uint64_t count, uint64_t seed, uint32_t layer,
                          uint32_t stream_id, const uint16_t* table, uint32_t table_n,
                          cudaStream_t stream) {
    require(out && table, "aeon_b200_synth_fill_dense16: null pointer argument");
    require(table_n > 0 && (table_n & (table_n - 1)) == 0,
            "aeon_b200_synth_fill_dense16: table_n must be a power of two");
    if (count == 0) return;
    const uint64_t key = synth_key(seed, layer, 0xFFFFu, stream_id);
    const int blocks = static_cast<int>(std::min<uint64_t>((count + 255) / 256, 4096));
    synth_dense16_kernel<<<blocks, 256, 0, stream>>>(static_cast<uint16_t*>(out), count, key, table,
                                                     table_n - 1);
    AEON_CUDA_CHECK(cudaGetLastError());
}

}  // namespace aeon_b200
