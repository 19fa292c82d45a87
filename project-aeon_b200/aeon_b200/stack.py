"""A stack of MoE layers on one GPU or expert-parallel over the GPUs of one box.

This is the call a user of the library makes for a batch of decode tokens:

    model = MoeStack(cfg, layers=8, max_tokens=128, seed=0, rank=r, world=R, dist=dist)
    model.forward(x, out)        # x[layers, tokens_local, H] 16-bit, out fp32

Per layer: router top-k -> shared expert (the accumulator's initial value) -> routed
experts. Weights are synthetic (see synth.py); a real model uploads payloads into the pools.

Expert parallelism (world > 1). Expert e lives on rank e // (E / world); gate and shared
expert are replicated; every rank owns tokens_local = tokens / world tokens.
  shared    the shared expert of the rank's own tokens runs on a side stream beside everything
            up to the combine, whose initial value it produces.
  routing   every rank routes its own tokens. The router is a per-token function, so the
            gathered routing is bit-identical to a router run on the whole batch.
  dispatch  rows and routing of every rank to every rank: a grouped all-gather
            (Group.ep_dispatch_routed) or, with peer_combine, plain stores into every rank's
            gather buffers and a bounded wait for the others' (PeerCombine.dispatch). At decode
            batch sizes a padded equal-split all-to-all would move exactly the same bytes.
  compute   each rank runs only its resident experts over the whole batch (absent experts are
            skipped).
  combine   collective form: the partial rows are written (no zero fill), an equal-split
            all-to-all moves them to their owners, the owners add the `world` slices in rank
            order. Peer form: the accumulate stores each finished row straight into its owner's
            receive buffer and the owner waits for `world` flags, then adds in rank order. Either
            way the summation order is fixed, independent of arrival.
"""
from __future__ import annotations

import numpy as np

import aeon_b200
from aeon_b200 import synth


def _torch_bits(bits: np.ndarray, dtype: int, device):
    import torch
    t = torch.from_numpy(bits.view(np.int16).copy()).to(device)
    return t.view(torch.bfloat16 if dtype == aeon_b200.BF16 else torch.float16)


def ep_dispatch_and_route(ops, dist, x_local, x_all, routing_all=None, group=None):
    """Dispatch and routing of one expert-parallel layer. Without `routing_all` every rank gathers
    the batch and runs the router on all of it (replicated, identical inputs). With routing_all =
    (ids_all, weights_all) every rank routes its own tokens and the routing is gathered with the
    rows: the router is a per-token function, so the result is the same bit for bit, and each
    rank does 1 / world of the router's work. `dist.ep_dispatch_routed` (the library's group) does
    the three gathers as one call; a plain torch.distributed module does them one by one."""
    scope = {} if group is None else {"group": group}
    if routing_all is None:
        dist.all_gather_into_tensor(x_all, x_local, **scope)
        return ops.router(x_all)
    ids_all, weights_all = routing_all
    weights_local, ids_local = ops.router(x_local)
    fused = getattr(dist, "ep_dispatch_routed", None)
    if fused is not None:
        fused(x_local, x_all, ids_local, weights_local, ids_all, weights_all)
    else:
        dist.all_gather_into_tensor(x_all, x_local, **scope)
        dist.all_gather_into_tensor(ids_all, ids_local.contiguous(), **scope)
        dist.all_gather_into_tensor(weights_all, weights_local.contiguous(), **scope)
    return weights_all, ids_all


def ep_layer_forward_peer(ops, dist, world, x_local, out_local, x_all, group=None, routing_all=None):
    """The same layer with the combine fused into the accumulate over peer memory: after the
    dispatch and the routing, `ops.routed_push` runs the resident experts and
    stores each finished partial row straight into the receive buffer of the rank that owns the
    token; `ops.combine_peer` waits for every rank's rows and adds them in rank order. One
    collective per layer instead of two, no local partial, no exchange kernel."""
    ops.shared(x_local, out_local)        # needs the rank's own rows only: may run beside all that follows
    if getattr(ops, "peer_dispatch", False):
        # the dispatch over peer memory too: route the rank's own tokens, store rows and routing into
        # every rank's gather buffers, wait for the others' (no collective in the layer)
        weights_local, ids_local = ops.router(x_local)
        x_all, ids, weights = ops.dispatch_peer(x_local, ids_local, weights_local)
    else:
        weights, ids = ep_dispatch_and_route(ops, dist, x_local, x_all, routing_all, group)
    ops.routed_push(x_all, ids, weights, out_local, x_local.shape[0])
    ops.combine_peer(out_local)
    return weights, ids


def ep_layer_forward(ops, dist, world, x_local, out_local, x_all, partial, recv, group=None, routing_all=None):
    """One expert-parallel MoE layer on this rank (the protocol of the module docstring).

    `ops` supplies the compute: router(x) -> (weights, ids); shared(x, out) writes the shared
    expert into out; routed(x, ids, weights, out, skip_absent, overwrite) adds the resident
    experts' contributions to out, or writes them over it when overwrite is set; combine(out, recv) adds recv[r] for r = 0..world-1 in that order. The
    collectives are `dist`'s (NCCL on GPUs; gloo in the CPU tests of the protocol).
    Returns the (replicated) routing of the whole batch."""
    scope = {} if group is None else {"group": group}          # the ranks of one pipeline stage
    ops.shared(x_local, out_local)        # needs the rank's own rows only: may run beside all that follows
    weights, ids = ep_dispatch_and_route(ops, dist, x_local, x_all, routing_all, group)
    ops.routed(x_all, ids, weights, partial, skip_absent=True, overwrite=True)   # writes, needs no zero fill
    if not recv.is_contiguous():
        raise ValueError("the receive buffer must be a dense [world, tokens_local, hidden] block")
    dist.all_to_all_single(recv.view(-1, recv.shape[-1]), partial, **scope)   # combine: rows to owners
    ops.combine(out_local, recv)
    return weights, ids


class StageTopology:
    """One process per GPU, `world` ranks as `pp` pipeline stages of world / pp ranks each
    (expert- or tensor-parallel inside a stage). Stage-major like the reference's topology
    (src/infrastructure/parallel/parallel_topology.hpp:166-199): global rank = stage *
    ranks_per_stage + rank_in_stage; layers split contiguously, remainder to the earliest stages.
    The peer of a rank in the next stage is the rank with the same index inside that stage, so a
    hand-off moves each rank's own token rows and nothing else."""

    def __init__(self, world: int, pp: int, layers: int):
        if pp < 1 or world < 1 or world % pp:
            raise ValueError(f"pipeline_parallel={pp} does not divide the {world} ranks")
        if pp > layers:
            raise ValueError(f"pipeline_parallel={pp} exceeds the {layers} model layers")
        self.world, self.pp, self.layers = world, pp, layers
        self.ranks_per_stage = world // pp
        base, rem = divmod(layers, pp)
        self._ranges, first = [], 0
        for stage in range(pp):
            count = base + (1 if stage < rem else 0)
            self._ranges.append(range(first, first + count))
            first += count

    def stage_of_rank(self, rank: int) -> int:
        return rank // self.ranks_per_stage

    def rank_in_stage(self, rank: int) -> int:
        return rank % self.ranks_per_stage

    def stage_ranks(self, stage: int):
        return list(range(stage * self.ranks_per_stage, (stage + 1) * self.ranks_per_stage))

    def stage_layers(self, stage: int) -> range:
        return self._ranges[stage]

    def stage_of_layer(self, layer: int) -> int:
        for stage, r in enumerate(self._ranges):
            if layer in r:
                return stage
        raise IndexError("layer out of range")

    def peer(self, rank: int, stage: int) -> int:
        return stage * self.ranks_per_stage + self.rank_in_stage(rank)


def pipeline_forward(topo: StageTopology, dist, rank: int, carry, run_layers):
    """One pass of a pipelined stack on this rank: receive the carried rows from the previous
    stage (a byte copy, as the reference's stage hand-off is,
    src/architecture/deepseek_v4/runtime/v4_graph.hpp:454-513, so the pipelined result equals the
    single-stage one bit for bit), run this stage's layers with `run_layers(carry, layers)`, and
    send the result on. Returns the carry on the last stage, None elsewhere. The point-to-point
    calls are `dist`'s (NCCL send/recv between the GPUs; gloo in the CPU tests)."""
    stage = topo.stage_of_rank(rank)
    if stage > 0:
        dist.recv(carry, src=topo.peer(rank, stage - 1))
    carry = run_layers(carry, topo.stage_layers(stage))
    if stage + 1 < topo.pp:
        dist.send(carry, dst=topo.peer(rank, stage + 1))
        return None
    return carry


def tp_layer_forward(ops, dist, world, x, out_local, partial):
    """One MoE layer with the experts' intermediate dimension split over `world` ranks
    (W1/W3 rows and W2 columns [r*I/world, (r+1)*I/world) on rank r, each shard swizzled as a
    matrix of its own; the reference shows this split exact on one GPU in
    tests/test_expert_shard_equivalence.cpp and tests/test_w2_shard_equivalence.cpp).

    Every rank holds all tokens `x` and all experts' shards: the router runs replicated, the
    rank computes its shard's contribution for every token into the fp32 `partial`
    [tokens, H], a reduce-scatter (sum) over NCCL hands each rank the finished rows of its
    tokens_local = tokens / world tokens, and the shared expert (replicated weights) of those
    rows is added by their owner. `ops.routed` must run with the shard's configuration
    (intermediate / world). The cross-rank sum order is the collective's, so results are
    compared with a tolerance and required to be identical run to run at a fixed world size."""
    tokens = x.shape[0]
    tl = tokens // world
    rank = dist.get_rank()
    weights, ids = ops.router(x)
    ops.routed(x, ids, weights, partial, skip_absent=False, overwrite=True)
    routed_local = out_local.new_empty(out_local.shape)
    dist.reduce_scatter_tensor(routed_local, partial)
    ops.shared(x[rank * tl:(rank + 1) * tl], out_local)
    out_local += routed_local
    return weights, ids


def layer_body_moe(ctx, w, hc, res_mid, prefill: bool = False):
    """The FFN half of a layer around the path, all on the device: residual streams
    res_mid [T, 4, H] 16-bit -> pre-mix + FFN RMSNorm -> router -> shared expert -> routed
    experts -> post expansion -> res_out [T, 4, H]. Stands in for
    run_layer_body_moe_router + run_layer_body_moe_and_post
    (src/architecture/deepseek_v4/layer/v4_layer_body_moe.hpp:124-312) with the routing kept on
    the device (the reference copies it to the host per token, :188-192).

    `w` carries gate / shared / pool / slot_of (MoeLayerWeights); `hc` is a dict with the
    layer's hc_ffn_fn [24, 4H] fp32, hc_ffn_base [24], hc_ffn_scale [3] and ffn_norm weight [H].
    Returns (res_out, ffn_norm, weights, ids, moe_out)."""
    import torch
    ffn_norm, _pre, post, comb = ctx.hc_ffn_front(res_mid, hc["fn"], hc["base"], hc["scale"], hc["norm"])
    T, H = ffn_norm.shape
    moe_out = torch.empty(T, H, dtype=torch.float32, device=ffn_norm.device)
    ctx.shared_expert(w.shared[0], w.shared[1], w.shared[2], ffn_norm, moe_out)
    weights, ids = ctx.router_topk(ffn_norm, w.gate, bias=getattr(w, "gate_bias", None))
    if prefill:
        ctx.moe_prefill(w.pool.base, w.slot_of, ffn_norm, ids, weights, moe_out)
    else:
        ctx.moe_decode(w.pool.base, w.slot_of, ffn_norm, ids, weights, moe_out)
    res_out = ctx.hc_post(moe_out, res_mid, post, comb)
    return res_out, ffn_norm, weights, ids, moe_out


class _DeviceOps:
    """The library's kernels behind the four calls ep_layer_forward needs."""

    def __init__(self, ctx, w, side=None):
        self.ctx, self.w = ctx, w
        # side = (stream, fork event, join event): the shared expert then runs on that stream,
        # and the combine, the first reader of what it wrote, waits for it
        self.side = side

    def router(self, x):
        return self.ctx.router_topk(x, self.w.gate)

    def shared(self, x, out):
        if self.side is None:
            self.ctx.shared_expert(self.w.shared[0], self.w.shared[1], self.w.shared[2], x, out)
            return
        import torch
        stream, fork, join = self.side
        fork.record(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            stream.wait_event(fork)
            self.ctx.shared_expert(self.w.shared[0], self.w.shared[1], self.w.shared[2], x, out)
            join.record(stream)

    def _join_shared(self):
        if self.side is not None:
            import torch
            torch.cuda.current_stream().wait_event(self.side[2])

    def routed(self, x, ids, weights, out, skip_absent, overwrite=False):
        self.ctx.moe_decode(self.w.pool.base, self.w.slot_of, x, ids, weights, out,
                            skip_absent=skip_absent, overwrite=overwrite)

    def combine(self, out, recv):
        self._join_shared()
        aeon_b200.ep_combine(out, recv)

    # -- the peer-memory form of the combine (and of the dispatch) -----------------------------------
    peer = None
    peer_dispatch = False

    def dispatch_peer(self, x_local, ids_local, weights_local):
        return self.peer.dispatch(self.ctx, x_local, ids_local, weights_local)

    def routed_push(self, x, ids, weights, scratch_out, tokens_local):
        self.ctx.moe_decode(self.w.pool.base, self.w.slot_of, x, ids, weights, scratch_out,
                            skip_absent=True, defer_accumulate=True)
        self.peer.push(self.ctx, self.w.slot_of, ids, tokens_local)

    def combine_peer(self, out):
        self._join_shared()
        self.peer.combine(self.ctx, out)


class MoeLayerWeights:
    """Device-resident weights of one layer for one rank's expert slice."""

    def __init__(self, cfg, layer: int, seed: int, device: int, first_expert: int, count: int,
                 tables):
        import torch
        dev = f"cuda:{device}"
        scale_table, dense_table = tables
        self.pool = aeon_b200.ExpertPool(cfg, count, device)
        self.pool.fill_synthetic(0, count, seed, layer, first_expert, scale_table)
        slot_of = np.full(cfg.experts, -1, dtype=np.int32)
        slot_of[first_expert:first_expert + count] = np.arange(count, dtype=np.int32)
        self.slot_of = torch.from_numpy(slot_of).to(dev)
        rng = np.random.default_rng([seed, layer, 0x6A7E])
        self.gate_bits = synth.normal_bits(rng, (cfg.experts, cfg.hidden), 0.01, cfg.act_dtype)
        self.gate = _torch_bits(self.gate_bits, cfg.act_dtype, dev)
        n = cfg.hidden * cfg.intermediate
        self.shared = []
        for stream_id in range(3):
            t = torch.empty(n, dtype=torch.int16, device=dev)
            aeon_b200.synth_fill_dense16(t, seed, layer, stream_id, dense_table)
            self.shared.append(t)


class LoadedLayer:
    """One layer's weights for the path, read from a model directory (the dense and the expert
    container, aeon_b200.artifact) onto a device: gate (+ bias or hash table), shared expert,
    the hyper-connection / norm tensors of the FFN half, and this rank's experts in a pool.
    Takes the place of the per-layer uploads of
    src/architecture/deepseek_v4/spec/v4_dense_weight_binding.hpp:86-137 and of the expert
    supply's initial fill. `tp` > 1 loads the rank's slice of every expert through
    rank_slice (the pool's configuration then has intermediate / tp); `experts` limits the
    resident set (default: all)."""

    def __init__(self, cfg, model_dir: str, layer: int, device: int = 0, experts=None, tp: int = 1,
                 tp_rank: int = 0):
        import os
        import torch
        from aeon_b200 import artifact
        dev = f"cuda:{device}"
        self.cfg = cfg
        self.cfg_rank = cfg.copy(intermediate=cfg.intermediate // tp)
        dense = artifact.DenseContainer(os.path.join(model_dir, artifact.DENSE_FILENAME))
        art = artifact.ExpertArtifact(model_dir)
        names = artifact.moe_layer_tensor_names(layer)
        prefix = f"layers.{layer}."

        def bits16(name):
            want = "BF16" if cfg.act_dtype == aeon_b200.BF16 else "F16"
            if dense.dtype_of(name) != want:
                raise aeon_b200.AeonError(1, f"{name} is {dense.dtype_of(name)}, the configuration wants {want}")
            raw = np.asarray(dense.raw(name)).view(np.uint16)
            return raw, _torch_bits(raw, cfg.act_dtype, dev)

        def f32(name):
            return torch.from_numpy(np.asarray(dense.raw(name)).view(np.float32).copy()).to(dev)

        self.gate_bits, self.gate = bits16(names["gate"])
        self.gate_bits = self.gate_bits.reshape(cfg.experts, cfg.hidden)
        self.gate = self.gate.reshape(cfg.experts, cfg.hidden)
        self.gate_bias = f32(names["gate_bias"]) if dense.has_tensor(names["gate_bias"]) else None
        self.shared_bits, self.shared = [], []
        for key in ("shared_w1", "shared_w3", "shared_w2"):
            b, t = bits16(names[key])
            self.shared_bits.append(b)
            self.shared.append(t.view(torch.int16))
        self.hc = None
        if dense.has_tensor(prefix + "hc_ffn_fn"):
            norm_bits, norm = bits16(prefix + "ffn_norm.weight")
            self.hc = dict(fn=f32(prefix + "hc_ffn_fn").reshape(24, 4 * cfg.hidden), base=f32(prefix + "hc_ffn_base"),
                           scale=f32(prefix + "hc_ffn_scale"), norm=norm, norm_bits=norm_bits)
        resident = list(range(cfg.experts)) if experts is None else list(experts)
        self.pool = aeon_b200.ExpertPool(self.cfg_rank, len(resident), device)
        slot_of = np.full(cfg.experts, -1, dtype=np.int32)
        for slot, e in enumerate(resident):
            self.pool.upload(slot, art.rank_payload(cfg, layer, e, tp, tp_rank))
            slot_of[e] = slot
        self.slot_of = torch.from_numpy(slot_of).to(dev)
        self.artifact = art


class MoeStack:
    def __init__(self, cfg, layers: int, max_tokens: int, seed: int = 0, device: int = 0,
                 rank: int = 0, world: int = 1, dist=None, peer_combine: bool = False):
        import torch
        if world > 1 and (cfg.experts % world or max_tokens % world):
            raise aeon_b200.AeonError(1, "experts and tokens must divide by the number of ranks")
        self.cfg, self.layers, self.world, self.rank, self.dist = cfg, layers, world, rank, dist
        self.device = device
        self.max_tokens = max_tokens
        dev = f"cuda:{device}"
        scale_np = synth.half_normal_table(0.02, 1e-4, 4096, dtype=aeon_b200.F16)
        dense_np = synth.half_normal_table(0.02, 0.0, 4096, dtype=cfg.act_dtype)
        tables = (torch.from_numpy(scale_np.view(np.int16).copy()).to(dev),
                  torch.from_numpy(dense_np.view(np.int16).copy()).to(dev))
        self.scale_table_np, self.dense_table_np = scale_np, dense_np
        per_rank = cfg.experts // world
        self.first_expert = rank * per_rank
        self.weights = [MoeLayerWeights(cfg, l, seed, device, self.first_expert, per_rank, tables)
                        for l in range(layers)]
        self.ctx = aeon_b200.Context(cfg, device, max_tokens)
        self._stats = [dict(distinct=0, draws=0, tokens=0) for _ in range(layers)]
        self.group = None
        self.peer = None
        # with peer_combine: the dispatch over peer memory as well (False: the grouped NCCL gather)
        self.peer_dispatch = True
        if world > 1:
            H = cfg.hidden
            # the data-path collectives run on the library's own communicator (C ABI); `dist` only
            # carries the 128-byte id to the other ranks
            self.group = aeon_b200.Group.from_process_group(dist, device)
            self.x_all = torch.empty(max_tokens, H, dtype=self.weights[0].gate.dtype, device=dev)
            self.partial = torch.empty(max_tokens, H, dtype=torch.float32, device=dev)
            # every rank routes its own tokens; the routing of the batch is gathered with the rows
            self.ids_all = torch.empty(max_tokens, cfg.top_k, dtype=torch.int32, device=dev)
            self.weights_all = torch.empty(max_tokens, cfg.top_k, dtype=torch.float32, device=dev)
            self.recv = torch.empty(world, max_tokens // world, H, dtype=torch.float32, device=dev)
            # peer_combine: the combine fused with the accumulate over CUDA-IPC mapped buffers
            self.peer = aeon_b200.PeerCombine(self.group, device, max_tokens // world, H) if peer_combine else None
        self._extra_launches = 0
        # False: the shared expert runs on the caller's stream ahead of the router, so that no
        # other kernel is resident while the routed kernels run (used to time them alone)
        self.overlap_shared = True
        self._side = torch.cuda.Stream(device=dev)
        self._fork = torch.cuda.Event()
        self._join = torch.cuda.Event()
        self._graphs = {}          # (x pointer, out pointer) -> (graph, launches per replay)
        torch.cuda.synchronize(device)

    # -- bookkeeping ----------------------------------------------------------------------
    @property
    def launches(self) -> int:
        return self.ctx.launches + self._extra_launches

    def set_timing(self, enabled: bool) -> None:
        self.ctx.set_timing(enabled)

    def kernel_times(self):
        return self.ctx.kernel_times()

    def routing_stats(self):
        """Per layer: distinct resident experts touched, draws served here, tokens seen."""
        return self._stats

    # -- the step -------------------------------------------------------------------------
    def forward(self, x, out, collect_stats: bool = False):
        """x[layers, tokens_local, H] 16-bit -> out[layers, tokens_local, H] fp32."""
        captured = None if collect_stats else self._graphs.get((x.data_ptr(), out.data_ptr()))
        if captured is not None:
            captured[0].replay()
            self._extra_launches += captured[1]
            return
        for l in range(self.layers):
            self.forward_layer(l, x[l], out[l], collect_stats)

    def capture(self, x, out):
        """Records one step over the fixed buffers x / out as a CUDA graph; later forward(x, out)
        calls with the same buffers replay it (one launch for the whole stack, no per-kernel
        launch gaps). The step must have run once already (lazy allocations happen there).
        Several buffer pairs may be captured (double-buffered callers replay them in turn)."""
        import torch
        before = self.launches
        graph = torch.cuda.CUDAGraph()
        torch.cuda.synchronize()
        with torch.cuda.graph(graph):
            for l in range(self.layers):
                self.forward_layer(l, x[l], out[l])
        self._graphs[(x.data_ptr(), out.data_ptr())] = (graph, self.launches - before)

    def close(self):
        """Releases the captured step and leaves the multi-GPU group (a collective call)."""
        self.release_graph()
        if self.peer is not None:
            self.peer.close()
            self.peer = None
        if self.group is not None:
            self.group.close()
            self.group = None

    def release_graph(self):
        """Drops the captured step. A graph that holds NCCL nodes keeps references into the
        communicator (NCCL frees a captured plan only when its graph is destroyed), so the
        process group must not be torn down while the graph is alive."""
        if self._graphs:
            import torch
            torch.cuda.synchronize()
            for graph, _ in self._graphs.values():
                graph.reset()
            self._graphs = {}
            torch.cuda.synchronize()

    def forward_layer(self, l: int, x, out, collect_stats: bool = False, return_routing: bool = False):
        w = self.weights[l]
        ctx = self.ctx
        ops = _DeviceOps(ctx, w, (self._side, self._fork, self._join)
                         if self.world > 1 and self.overlap_shared else None)
        if self.world == 1 and not self.overlap_shared:
            ops.shared(x, out)
            weights, ids = ops.router(x)
            ctx.moe_decode(w.pool.base, w.slot_of, x, ids, weights, out, defer_accumulate=True)
            ctx.moe_accumulate(w.slot_of, ids, out)
            tokens_seen = x.shape[0]
        elif self.world == 1:
            # The shared expert (88 MB of dense weights, no dependence on the routing) runs on
            # a side stream while the main stream does router -> permutation -> routed experts;
            # the two meet at the slot-order accumulate, whose initial value it produces.
            import torch
            main = torch.cuda.current_stream()
            self._fork.record(main)
            with torch.cuda.stream(self._side):
                self._side.wait_event(self._fork)
                ops.shared(x, out)
                self._join.record(self._side)
            weights, ids = ops.router(x)
            ctx.moe_decode(w.pool.base, w.slot_of, x, ids, weights, out, defer_accumulate=True)
            main.wait_event(self._join)
            ctx.moe_accumulate(w.slot_of, ids, out)
            tokens_seen = x.shape[0]
        else:
            tl = x.shape[0]
            tokens_seen = tl * self.world
            routing_all = (self.ids_all[:tokens_seen], self.weights_all[:tokens_seen])
            if self.peer is not None:
                ops.peer = self.peer
                ops.peer_dispatch = self.peer_dispatch
                weights, ids = ep_layer_forward_peer(ops, self.group, self.world, x, out, self.x_all[:tokens_seen],
                                                     routing_all=routing_all)
                self._extra_launches += 1
                if collect_stats:
                    distinct, _ = ctx.last_stats()
                    flat = ids.flatten()
                    local = ((flat >= self.first_expert) &
                             (flat < self.first_expert + self.cfg.experts // self.world)).sum().item()
                    self._stats[l] = dict(distinct=distinct, draws=int(local), tokens=tokens_seen)
                return (weights.clone(), ids.clone()) if return_routing else None    # the gather buffers are reused
            weights, ids = ep_layer_forward(ops, self.group, self.world, x, out,
                                            self.x_all[:tokens_seen], self.partial[:tokens_seen],
                                            self.recv.view(-1)[:tokens_seen * x.shape[1]]
                                            .view(self.world, tl, x.shape[1]), routing_all=routing_all)
            self._extra_launches += 2
        if collect_stats:
            distinct, _ = ctx.last_stats()
            flat = ids.flatten()
            local = ((flat >= self.first_expert) &
                     (flat < self.first_expert + self.cfg.experts // self.world)).sum().item()
            self._stats[l] = dict(distinct=distinct, draws=int(local), tokens=tokens_seen)
        if return_routing:
            return (weights.clone(), ids.clone()) if self.world > 1 else (weights, ids)

    # -- configuration-1 sweep: one layer at batch 1/8/32/128, rotating over the layers so
    #    consecutive iterations stream different weights (a batch-1 step touches ~180 MB,
    #    the order of the L2 capacity) ----------------------------------------------------
    def batch_sweep(self, batches, x, out, peak_gbs: float, iters: int = 20):
        import torch
        cfg = self.cfg
        lay = aeon_b200.expert_layout(cfg)
        expert_bytes = 2 * (lay.w13_packed_bytes + lay.w13_scale_bytes) + lay.w2_packed_bytes + lay.w2_scale_bytes
        results = []
        for b in batches:
            if b > x.shape[1]:
                continue
            distinct = []
            for l in range(self.layers):          # warm-up pass, also collects the routing stats
                self.forward_layer(l, x[l, :b], out[l, :b], collect_stats=True)
                distinct.append(self._stats[l]["distinct"])
            torch.cuda.synchronize()
            total_iters = max(iters, self.layers)
            # per-kernel device times: eager launches with the library's events around the kernels
            self.ctx.set_timing(True)
            for i in range(total_iters):
                l = i % self.layers
                self.forward_layer(l, x[l, :b], out[l, :b])
            (ms_a, n_a), (ms_b, n_b) = self.ctx.kernel_times()
            self.ctx.set_timing(False)
            # the layer time: one pass over the layers replayed as a CUDA graph, so the figure is the
            # device's and not the host's launch rate (at batch 1 a layer is ten launches of 3-40 us)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for l in range(self.layers):
                    self.forward_layer(l, x[l, :b], out[l, :b])
            replays = max(1, total_iters // self.layers)
            graph.replay()
            torch.cuda.synchronize()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for _ in range(replays):
                graph.replay()
            end.record()
            torch.cuda.synchronize()
            us_layer = start.elapsed_time(end) * 1e3 / (replays * self.layers)
            graph.reset()
            mean_d = float(np.mean(distinct))
            routed_bytes = mean_d * expert_bytes
            kernel_us = (ms_a + ms_b) * 1e3 / max(n_a, 1)
            results.append({
                "batch": b, "us_per_layer": us_layer, "tokens_per_s_per_layer": b / (us_layer * 1e-6),
                "distinct_experts": mean_d, "routed_weight_bytes": routed_bytes,
                "routed_kernels_us": kernel_us,
                "routed_kernels_gbs": routed_bytes / (kernel_us * 1e-6) / 1e9,
                "routed_kernels_frac_of_peak": routed_bytes / (kernel_us * 1e-6) / 1e9 / peak_gbs,
                "layer_gbs_incl_router_shared": (routed_bytes + cfg.experts * cfg.hidden * 2 +
                                                 3 * cfg.hidden * cfg.intermediate * 2) / (us_layer * 1e-6) / 1e9,
            })
        return results
