// Expert-parallel combine fused with the slot-order accumulate, over peer memory.
//
// In the collective form of the expert-parallel layer a rank first sums its resident experts'
// per-draw slices into a local fp32 partial [tokens, H] (kernel C), then an all-to-all moves the
// rows to the ranks that own the tokens, then a third kernel adds the received slices. Here
// kernel C writes each finished row straight into its owner's receive buffer with plain 128-bit
// peer stores over NVLink, and raises one flag per (owner, source rank) when the owner's rows are
// complete; the owner's combine kernel waits for the `world` flags of the call and adds the
// slices in rank order. No collective, no local partial, one kernel fewer, and the transfer of a
// row overlaps the summation of the next.
//
// Memory: every rank allocates one receive buffer [world, tokens_local_max, H] fp32 and one flag
// line with cudaMalloc, exports both with CUDA IPC, and maps its peers' (the 64-byte handles
// travel through the group's own all-gather). Only plain loads and stores touch peer memory: no
// multicast, no multimem, no TMA.
//
// Ordering. Writer: row stores, __threadfence_system(), then the last block to finish an owner's
// rows stores the flag (release, system scope). Reader: acquire load of the flag at system scope,
// then the rows. The flag value is the call's epoch, kept in device memory and advanced by the
// kernels themselves, so a captured CUDA graph replays correctly and no flag is ever reset.
// Reuse of the single receive buffer is safe because every layer starts with the dispatch
// all-gather: a rank cannot leave layer l+1's gather before every rank has entered it, i.e.
// before every owner's combine of layer l has finished reading.
//
// The dispatch has the same form (aeon_b200_ep_peer_dispatch): every rank stores its activation
// rows and the routing it computed for them into each peer's gather buffer and raises one flag per
// peer; the kernel's last block then waits for the `world` flags of its own buffer. At decode
// sizes (a few hundred KB per rank) this replaces a collective whose cost is its latency. The
// reuse argument carries over without a collective in the loop: a rank reaches layer l+1's
// dispatch only after its combine of layer l saw every rank's flag, and a rank raises that flag
// for an owner only after it has finished reading that owner's rows of layer l's gather buffers;
// a rank pushes partial rows of layer l+1 only after every rank's dispatch flag of layer l+1,
// which each rank raises after its own combine of layer l has finished reading (stream order).
//
// Every wait is bounded: when a flag does not arrive within the budget (a peer that died or never
// launched) the combine kernel records kErrWaitTimeout in the context's error flag, adds what it
// has and returns; aeon_b200_ctx_check reports AEON_B200_ERR_TIMEOUT and the context stays usable.
//
// The reference has no expert parallelism (deferred:
// plans-and-docs/specs-and-requirements/multi-gpu/MULTI_GPU_REQUIREMENTS.md:103); the summation
// order follows its fixed-slot-order accumulate (src/platform/ops/moe_accumulate.hpp:73-92).
#include "common.cuh"

#include <algorithm>
#include <cstring>

struct aeon_b200_group;
extern "C" int aeon_b200_group_rank(const aeon_b200_group* group);
extern "C" int aeon_b200_group_world(const aeon_b200_group* group);
extern "C" int aeon_b200_ep_dispatch(aeon_b200_group* group, const void* x_local, int tokens_local,
                                     int64_t row_bytes, void* x_all, void* stream);

namespace aeon_b200 {
namespace {

constexpr int kMaxRanks = 8;
constexpr int kFlagStride = 32;           // uint32 per flag: one 128-byte line each

constexpr int kMaxTopK = 32;

struct PeerView {                         // device-visible, passed by value
    float* recv[kMaxRanks];               // rank r's receive buffer [world, tl_max, H] as mapped here
    uint32_t* flags[kMaxRanks];           // rank r's flag lines [world] as mapped here
    uint8_t* gather[kMaxRanks];           // rank r's gather block (layout: GatherLayout) as mapped here
    int rank, world, tl_max, hidden;
};

// One rank's gather block: activation rows (16-bit elements), routing ids and weights of the whole
// batch in rank order, and the dispatch flags, each part 256-byte aligned.
struct GatherLayout {
    size_t x_off, ids_off, weights_off, flags_off, bytes;
};

inline GatherLayout gather_layout(int world, int tl_max, int hidden) {
    auto up = [](size_t v) { return (v + 255) & ~static_cast<size_t>(255); };
    GatherLayout g{};
    const size_t tokens = static_cast<size_t>(world) * tl_max;
    g.x_off = 0;
    g.ids_off = up(tokens * hidden * 2);
    g.weights_off = g.ids_off + up(tokens * kMaxTopK * 4);
    g.flags_off = g.weights_off + up(tokens * kMaxTopK * 4);
    g.bytes = g.flags_off + kMaxRanks * kFlagStride * 4;
    return g;
}

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Dispatch over peer memory. grid = world * blocks_per_peer; block (q, b) copies this rank's rows
// (and block (q, 0) its routing) into rank q's gather block at this rank's place, then the last
// block for q raises q's flag for this rank; the last block of the grid waits, bounded, for the
// `world` flags of this rank's own block. state[0] = epoch of the last completed call,
// state[1] = blocks finished, state[2 + q] = blocks finished for peer q.
__global__ void ep_dispatch_push_wait_kernel(PeerView view, GatherLayout lay, const uint4* __restrict__ x_local,
                                             const int32_t* __restrict__ ids_local,
                                             const float* __restrict__ weights_local, int tl, int row_vecs,
                                             int top_k, uint32_t* __restrict__ state, int blocks_per_peer,
                                             long long wait_cycles, int32_t* __restrict__ error) {
    const int q = blockIdx.x / blocks_per_peer;
    const int b = blockIdx.x - q * blocks_per_peer;
    const uint32_t epoch = state[0] + 1;
    uint8_t* block = view.gather[q];
    const int64_t vecs = static_cast<int64_t>(tl) * row_vecs;
    uint4* x_dst = reinterpret_cast<uint4*>(block + lay.x_off) + static_cast<int64_t>(view.rank) * vecs;
    for (int64_t i = static_cast<int64_t>(b) * blockDim.x + threadIdx.x; i < vecs;
         i += static_cast<int64_t>(blocks_per_peer) * blockDim.x)
        x_dst[i] = __ldg(x_local + i);                                        // local or peer store
    if (b == 0) {
        const int draws = tl * top_k;
        int32_t* ids_dst = reinterpret_cast<int32_t*>(block + lay.ids_off) + view.rank * draws;
        float* w_dst = reinterpret_cast<float*>(block + lay.weights_off) + view.rank * draws;
        for (int i = threadIdx.x; i < draws; i += blockDim.x) {
            ids_dst[i] = ids_local[i];
            w_dst[i] = weights_local[i];
        }
    }
    __threadfence_system();
    __syncthreads();
    __shared__ int last_of_grid;
    if (threadIdx.x == 0) {
        if (atomicAdd(&state[2 + q], 1u) == static_cast<uint32_t>(blocks_per_peer - 1)) {
            state[2 + q] = 0;
            __threadfence_system();
            st_release_sys(reinterpret_cast<uint32_t*>(block + lay.flags_off) + view.rank * kFlagStride, epoch);
        }
        last_of_grid = atomicAdd(&state[1], 1u) == gridDim.x - 1;
    }
    __syncthreads();
    if (!last_of_grid) return;
    // every flag this rank owes is out (or will be, by blocks that need nothing from this one):
    // wait for the rows of the others
    if (threadIdx.x < view.world) {
        const uint32_t* flag = reinterpret_cast<const uint32_t*>(view.gather[view.rank] + lay.flags_off) +
                               threadIdx.x * kFlagStride;
        const long long start = clock64();
        bool ok = false;
        for (;;) {
            if (static_cast<int32_t>(ld_acquire_sys(flag) - epoch) >= 0) { ok = true; break; }
            if (clock64() - start > wait_cycles) break;
            if (error != nullptr && *reinterpret_cast<volatile int32_t*>(error) != 0) break;
            __nanosleep(100);
        }
        if (!ok && error != nullptr) atomicCAS(error, kErrNone, kErrWaitTimeout);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        state[1] = 0;
        __threadfence();
        state[0] = epoch;
    }
}

// Kernel C with the owners' receive buffers as destination. grid = world * blocks_per_owner;
// block (o, b) sums the rows of owner o's tokens [o * tl, (o+1) * tl). state[0] = epoch of the
// last completed call, state[1] = blocks finished in this call, state[2 + o] = blocks finished
// for owner o.
__global__ void ep_accumulate_push_kernel(PeerView view, const float* __restrict__ contrib,
                                          const int32_t* __restrict__ ids, const int32_t* __restrict__ slot_of,
                                          int experts, int tl, int top_k, int pool_slots,
                                          uint32_t* __restrict__ state, int blocks_per_owner) {
    const int H = view.hidden;
    const int owner = blockIdx.x / blocks_per_owner;
    const int b = blockIdx.x - owner * blocks_per_owner;
    const uint32_t epoch = state[0] + 1;
    const int vec_per_row = H / 4;
    const int64_t total = static_cast<int64_t>(tl) * vec_per_row;
    float4* dst_base = reinterpret_cast<float4*>(view.recv[owner]) +
                       static_cast<int64_t>(view.rank) * view.tl_max * vec_per_row;
    for (int64_t i = static_cast<int64_t>(b) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<int64_t>(blocks_per_owner) * blockDim.x) {
        const int t_local = static_cast<int>(i / vec_per_row);
        const int v = static_cast<int>(i - static_cast<int64_t>(t_local) * vec_per_row);
        const int token = owner * tl + t_local;
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int slot = 0; slot < top_k; ++slot) {
            const int draw = token * top_k + slot;
            const int id = ids[draw];
            if (id >= 0 && id < experts) {
                const int s = slot_of[id];
                if (s >= 0 && !(pool_slots > 0 && s >= pool_slots)) {          // resident here
                    const float4 c = reinterpret_cast<const float4*>(contrib + static_cast<size_t>(draw) * H)[v];
                    a.x += c.x; a.y += c.y; a.z += c.z; a.w += c.w;
                }
            }
        }
        dst_base[static_cast<int64_t>(t_local) * vec_per_row + v] = a;      // local or peer store
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        if (atomicAdd(&state[2 + owner], 1u) == static_cast<uint32_t>(blocks_per_owner - 1)) {
            state[2 + owner] = 0;
            __threadfence_system();
            st_release_sys(view.flags[owner] + view.rank * kFlagStride, epoch);   // owner's rows are there
        }
        if (atomicAdd(&state[1], 1u) == gridDim.x - 1) {
            state[1] = 0;
            __threadfence();
            state[0] = epoch;                                                     // the call is over
        }
    }
}

// out[t, :] += sum_r recv[r, t, :] in rank order, after the `world` flags of this call arrived.
// state[0] = epoch of the last completed call, state[1] = blocks finished.
__global__ void ep_combine_wait_kernel(PeerView view, float* __restrict__ out, int64_t out_stride, int tl,
                                       uint32_t* __restrict__ state, long long wait_cycles,
                                       int32_t* __restrict__ error) {
    const int H = view.hidden;
    const uint32_t epoch = state[0] + 1;
    __shared__ int arrived;
    if (threadIdx.x == 0) arrived = 1;
    __syncthreads();
    if (threadIdx.x < view.world) {
        const uint32_t* flag = view.flags[view.rank] + threadIdx.x * kFlagStride;
        const long long start = clock64();
        bool ok = false;
        // the flag only ever grows: a value at or past this call's epoch means the rows are there
        for (;;) {
            if (static_cast<int32_t>(ld_acquire_sys(flag) - epoch) >= 0) { ok = true; break; }
            if (clock64() - start > wait_cycles) break;
            if (error != nullptr && *reinterpret_cast<volatile int32_t*>(error) != 0) break;
            __nanosleep(200);
        }
        if (!ok) {
            arrived = 0;
            if (error != nullptr) atomicCAS(error, kErrNone, kErrWaitTimeout);
        }
    }
    __syncthreads();
    const bool complete = arrived != 0;
    const int vec_per_row = H / 4;
    const int64_t total = static_cast<int64_t>(tl) * vec_per_row;
    const int64_t plane = static_cast<int64_t>(view.tl_max) * vec_per_row;
    const float4* recv = reinterpret_cast<const float4*>(view.recv[view.rank]);
    if (complete) {
        for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
             i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
            const int t = static_cast<int>(i / vec_per_row);
            const int v = static_cast<int>(i - static_cast<int64_t>(t) * vec_per_row);
            float4* dst = reinterpret_cast<float4*>(out + t * out_stride) + v;
            float4 a = *dst;
            for (int r = 0; r < view.world; ++r) {
                // L2 reads: these rows were written by other GPUs, which this SM's L1 does not see
                const float4 c = __ldcg(recv + r * plane + i);
                a.x += c.x; a.y += c.y; a.z += c.z; a.w += c.w;
            }
            *dst = a;
        }
    }
    __syncthreads();
    if (threadIdx.x == 0 && atomicAdd(&state[1], 1u) == gridDim.x - 1) {
        state[1] = 0;
        __threadfence();
        state[0] = epoch;
    }
}

}  // namespace
}  // namespace aeon_b200

using namespace aeon_b200;

struct aeon_b200_ep_peer {
    aeon_b200_group* group;
    int rank, world, device, tl_max, hidden;
    float* recv_local;
    uint32_t* flags_local;
    uint8_t* gather_local;       // this rank's gather block (GatherLayout)
    GatherLayout gather;
    uint32_t* push_state;        // [2 + kMaxRanks]
    uint32_t* wait_state;        // [2]
    uint32_t* dispatch_state;    // [2 + kMaxRanks]
    void* mapped[3 * kMaxRanks]; // peers' buffers opened through IPC (closed at destroy)
    PeerView view;
    double wait_budget_ms;
    int clock_khz;
};

extern "C" {

int aeon_b200_ep_peer_create(aeon_b200_group* group, int device, int tokens_local_max, int hidden,
                             aeon_b200_ep_peer** out_host) {
    return guarded([&] {
        require(group && out_host, "aeon_b200_ep_peer_create: null pointer");
        require(tokens_local_max > 0 && hidden > 0 && hidden % 4 == 0,
                "aeon_b200_ep_peer_create: tokens_local_max must be positive and hidden a multiple of 4");
        const int world = aeon_b200_group_world(group), rank = aeon_b200_group_rank(group);
        require(world >= 1 && world <= kMaxRanks, "aeon_b200_ep_peer_create: at most 8 ranks share peer buffers");
        int previous = -1;
        AEON_CUDA_CHECK(cudaGetDevice(&previous));
        AEON_CUDA_CHECK(cudaSetDevice(device));
        aeon_b200_ep_peer* p = new aeon_b200_ep_peer();
        std::memset(p, 0, sizeof(*p));
        p->group = group; p->rank = rank; p->world = world; p->device = device;
        p->tl_max = tokens_local_max; p->hidden = hidden;
        p->wait_budget_ms = 2000.0;
        try {
            const size_t recv_bytes = static_cast<size_t>(world) * tokens_local_max * hidden * sizeof(float);
            AEON_CUDA_CHECK(cudaMalloc(reinterpret_cast<void**>(&p->recv_local), recv_bytes));
            AEON_CUDA_CHECK(cudaMalloc(reinterpret_cast<void**>(&p->flags_local), kMaxRanks * kFlagStride * 4));
            p->gather = gather_layout(world, tokens_local_max, hidden);
            AEON_CUDA_CHECK(cudaMalloc(reinterpret_cast<void**>(&p->gather_local), p->gather.bytes));
            AEON_CUDA_CHECK(cudaMemset(p->gather_local, 0, p->gather.bytes));
            AEON_CUDA_CHECK(cudaMalloc(reinterpret_cast<void**>(&p->dispatch_state), (2 + kMaxRanks) * 4));
            AEON_CUDA_CHECK(cudaMemset(p->dispatch_state, 0, (2 + kMaxRanks) * 4));
            AEON_CUDA_CHECK(cudaMalloc(reinterpret_cast<void**>(&p->push_state), (2 + kMaxRanks) * 4));
            AEON_CUDA_CHECK(cudaMalloc(reinterpret_cast<void**>(&p->wait_state), 2 * 4));
            AEON_CUDA_CHECK(cudaMemset(p->flags_local, 0, kMaxRanks * kFlagStride * 4));
            AEON_CUDA_CHECK(cudaMemset(p->push_state, 0, (2 + kMaxRanks) * 4));
            AEON_CUDA_CHECK(cudaMemset(p->wait_state, 0, 2 * 4));
            AEON_CUDA_CHECK(cudaDeviceGetAttribute(&p->clock_khz, cudaDevAttrClockRate, device));

            // exchange the IPC handles through the group's own all-gather
            struct Handles { cudaIpcMemHandle_t recv, flags, gather; };
            Handles mine{};
            if (world > 1) {
                AEON_CUDA_CHECK(cudaIpcGetMemHandle(&mine.recv, p->recv_local));
                AEON_CUDA_CHECK(cudaIpcGetMemHandle(&mine.flags, p->flags_local));
                AEON_CUDA_CHECK(cudaIpcGetMemHandle(&mine.gather, p->gather_local));
            }
            std::vector<Handles> all(world);
            all[rank] = mine;
            if (world > 1) {
                Handles *d_mine = nullptr, *d_all = nullptr;
                AEON_CUDA_CHECK(cudaMalloc(reinterpret_cast<void**>(&d_mine), sizeof(Handles)));
                AEON_CUDA_CHECK(cudaMalloc(reinterpret_cast<void**>(&d_all), sizeof(Handles) * world));
                AEON_CUDA_CHECK(cudaMemcpy(d_mine, &mine, sizeof(Handles), cudaMemcpyHostToDevice));
                const int rc = aeon_b200_ep_dispatch(group, d_mine, 1, sizeof(Handles), d_all, nullptr);
                cudaError_t e = cudaDeviceSynchronize();
                if (rc == AEON_B200_OK && e == cudaSuccess)
                    e = cudaMemcpy(all.data(), d_all, sizeof(Handles) * world, cudaMemcpyDeviceToHost);
                (void)cudaFree(d_mine);
                (void)cudaFree(d_all);
                if (rc != AEON_B200_OK) throw StatusError(rc, aeon_b200_last_error());
                AEON_CUDA_CHECK(e);
            }
            p->view.rank = rank; p->view.world = world; p->view.tl_max = tokens_local_max; p->view.hidden = hidden;
            for (int r = 0; r < world; ++r) {
                if (r == rank) {
                    p->view.recv[r] = p->recv_local;
                    p->view.flags[r] = p->flags_local;
                    p->view.gather[r] = p->gather_local;
                    continue;
                }
                void *recv = nullptr, *flags = nullptr, *gather = nullptr;
                AEON_CUDA_CHECK(cudaIpcOpenMemHandle(&recv, all[r].recv, cudaIpcMemLazyEnablePeerAccess));
                p->mapped[2 * r] = recv;
                AEON_CUDA_CHECK(cudaIpcOpenMemHandle(&flags, all[r].flags, cudaIpcMemLazyEnablePeerAccess));
                p->mapped[2 * r + 1] = flags;
                AEON_CUDA_CHECK(cudaIpcOpenMemHandle(&gather, all[r].gather, cudaIpcMemLazyEnablePeerAccess));
                p->mapped[2 * kMaxRanks + r] = gather;
                p->view.recv[r] = static_cast<float*>(recv);
                p->view.flags[r] = static_cast<uint32_t*>(flags);
                p->view.gather[r] = static_cast<uint8_t*>(gather);
            }
        } catch (...) {
            for (void* m : p->mapped)
                if (m) (void)cudaIpcCloseMemHandle(m);
            (void)cudaFree(p->recv_local); (void)cudaFree(p->flags_local); (void)cudaFree(p->gather_local);
            (void)cudaFree(p->push_state); (void)cudaFree(p->wait_state); (void)cudaFree(p->dispatch_state);
            delete p;
            (void)cudaSetDevice(previous);
            throw;
        }
        (void)cudaSetDevice(previous);
        *out_host = p;
    });
}

int aeon_b200_ep_peer_destroy(aeon_b200_ep_peer* peer) {
    return guarded([&] {
        if (!peer) return;
        int previous = -1;
        AEON_CUDA_CHECK(cudaGetDevice(&previous));
        AEON_CUDA_CHECK(cudaSetDevice(peer->device));
        (void)cudaDeviceSynchronize();
        for (void* m : peer->mapped)
            if (m) (void)cudaIpcCloseMemHandle(m);
        (void)cudaFree(peer->recv_local); (void)cudaFree(peer->flags_local); (void)cudaFree(peer->gather_local);
        (void)cudaFree(peer->push_state); (void)cudaFree(peer->wait_state); (void)cudaFree(peer->dispatch_state);
        delete peer;
        (void)cudaSetDevice(previous);
    });
}

int aeon_b200_ep_peer_set_wait_budget(aeon_b200_ep_peer* peer, double milliseconds) {
    return guarded([&] {
        require(peer != nullptr && milliseconds > 0.0 && milliseconds <= 60000.0,
                "aeon_b200_ep_peer_set_wait_budget: the budget must be in (0, 60000] ms");
        peer->wait_budget_ms = milliseconds;
    });
}

int aeon_b200_ep_peer_dispatch(aeon_b200_ctx* ctx, aeon_b200_ep_peer* peer, const void* x_local,
                               int tokens_local, const int32_t* ids_local, const float* weights_local,
                               void** x_all, int32_t** ids_all, float** weights_all, void* stream) {
    return guarded([&] {
        require(ctx && peer && x_local && ids_local && weights_local && x_all && ids_all && weights_all,
                "aeon_b200_ep_peer_dispatch: null pointer argument");
        require(ctx->device == peer->device && ctx->cfg.hidden == peer->hidden,
                "aeon_b200_ep_peer_dispatch: context and peer buffers disagree on device or hidden width");
        require(tokens_local > 0 && tokens_local <= peer->tl_max,
                "aeon_b200_ep_peer_dispatch: tokens_local outside the peer buffers");
        require(ctx->cfg.top_k <= kMaxTopK, "aeon_b200_ep_peer_dispatch: top_k above 32 is not supported");
        require(aligned16(x_local) && peer->hidden % 8 == 0,
                "aeon_b200_ep_peer_dispatch: x_local must be 16-byte aligned dense rows (128-bit copies)");
        const int row_vecs = peer->hidden * 2 / 16;
        const int64_t vecs = static_cast<int64_t>(tokens_local) * row_vecs;
        const int per_peer = static_cast<int>(std::max<int64_t>(
            1, std::min<int64_t>((vecs + 255) / 256, ctx->sm_count / peer->world)));
        const long long cycles = static_cast<long long>(peer->wait_budget_ms * peer->clock_khz);
        ep_dispatch_push_wait_kernel<<<peer->world * per_peer, 256, 0, static_cast<cudaStream_t>(stream)>>>(
            peer->view, peer->gather, static_cast<const uint4*>(x_local), ids_local, weights_local, tokens_local,
            row_vecs, ctx->cfg.top_k, peer->dispatch_state, per_peer, cycles, ctx->d_error);
        AEON_CUDA_CHECK(cudaGetLastError());
        ctx->launches += 1;
        *x_all = peer->gather_local + peer->gather.x_off;
        *ids_all = reinterpret_cast<int32_t*>(peer->gather_local + peer->gather.ids_off);
        *weights_all = reinterpret_cast<float*>(peer->gather_local + peer->gather.weights_off);
    });
}

int aeon_b200_moe_accumulate_push(aeon_b200_ctx* ctx, aeon_b200_ep_peer* peer, const int32_t* slot_of_expert,
                                  const int32_t* topk_ids, int tokens_local, void* stream) {
    return guarded([&] {
        require(ctx && peer && slot_of_expert && topk_ids, "aeon_b200_moe_accumulate_push: null pointer argument");
        require(ctx->device == peer->device && ctx->cfg.hidden == peer->hidden,
                "aeon_b200_moe_accumulate_push: context and peer buffers disagree on device or hidden width");
        require(tokens_local > 0 && tokens_local <= peer->tl_max &&
                    tokens_local * peer->world <= ctx->max_tokens,
                "aeon_b200_moe_accumulate_push: tokens_local outside the peer buffers or the context");
        const aeon_b200_moe_config& cfg = ctx->cfg;
        const int64_t vecs = static_cast<int64_t>(tokens_local) * cfg.hidden / 4;
        const int per_owner = static_cast<int>(std::max<int64_t>(
            1, std::min<int64_t>((vecs + 255) / 256, 4 * ctx->sm_count / peer->world)));
        ep_accumulate_push_kernel<<<peer->world * per_owner, 256, 0, static_cast<cudaStream_t>(stream)>>>(
            peer->view, ctx->d_contrib, topk_ids, slot_of_expert, cfg.experts, tokens_local, cfg.top_k,
            ctx->pool_slots, peer->push_state, per_owner);
        AEON_CUDA_CHECK(cudaGetLastError());
        ctx->launches += 1;
    });
}

int aeon_b200_ep_peer_combine(aeon_b200_ctx* ctx, aeon_b200_ep_peer* peer, float* out, int64_t out_stride,
                              int tokens_local, void* stream) {
    return guarded([&] {
        require(ctx && peer && out, "aeon_b200_ep_peer_combine: null pointer argument");
        require(ctx->device == peer->device, "aeon_b200_ep_peer_combine: context and peer buffers are on different devices");
        require(tokens_local > 0 && tokens_local <= peer->tl_max, "aeon_b200_ep_peer_combine: tokens_local outside the peer buffers");
        require(out_stride >= peer->hidden && out_stride % 4 == 0 && aligned16(out),
                "aeon_b200_ep_peer_combine: out must be 16-byte aligned, out_stride >= hidden and a multiple of 4");
        const int64_t vecs = static_cast<int64_t>(tokens_local) * peer->hidden / 4;
        const int blocks = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>((vecs + 255) / 256, 2 * ctx->sm_count)));
        const long long cycles = static_cast<long long>(peer->wait_budget_ms * peer->clock_khz);
        ep_combine_wait_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
            peer->view, out, out_stride, tokens_local, peer->wait_state, cycles, ctx->d_error);
        AEON_CUDA_CHECK(cudaGetLastError());
        ctx->launches += 1;
    });
}

}  // extern "C"
