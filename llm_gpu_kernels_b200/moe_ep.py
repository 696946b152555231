"""Expert-parallel MoE layer over the ranks of one node.

The reference is single-GPU and has nothing here; this is the natural sharding
of its path: experts are independent, so rank ``r`` of ``G`` owns experts
``[r*E/G, (r+1)*E/G)`` (their weights only) and its own slice of the tokens.
One forward on every rank:

 1. router + ranked dispatch of the local tokens over ALL experts. The
    dispatch sorts routes by expert, and experts are contiguous per rank, so
    ``grouped_input`` already is the send buffer, split by destination rank.
 2. all-gather of the per-expert counts (G*E int32), one host read of the
    split sizes, then the all-to-all-v of the routed rows (BF16, NCCL over
    NVLink) straight into the input buffer of the local expert plan.
 3. the local experts run the ordinary fixed-route path (top-1, weight 1) on
    the received rows; a device scalar tells the kernels how many rows of the
    fixed-capacity buffers are real this forward.
 4. all-to-all-v of the results back, straight into ``down_output`` of the
    token-owning plan, and its weighted combine in slot order.

No kernel touches another GPU's memory; rows always land in a local buffer
first. The exchange logic is device-agnostic (``backend`` supplies the compute
stages), which is how the two-rank CPU tests drive it over gloo.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist

from .moe import _prepare
from .moe_full_policy import token_tile_for

STATUS_EP_OVERFLOW = 8


def expert_range(rank: int, world: int, experts: int):
    """Contiguous block of experts owned by ``rank``."""
    if experts % world:
        raise ValueError("experts must divide evenly over the ranks")
    per = experts // world
    return rank * per, (rank + 1) * per


def split_sizes(counts_by_peer: torch.Tensor):
    """Rows per peer from a ``[G, E/G]`` count matrix (host list)."""
    return [int(v) for v in counts_by_peer.sum(dim=1).tolist()]


def received_expert_ids(recv_counts: torch.Tensor, total: int):
    """Local expert id of every received row.

    Peer ``s`` sends its rows sorted by expert, ``recv_counts[s, e]`` of them for
    local expert ``e``; the receive buffer is the concatenation over peers.
    """
    peers, local = recv_counts.shape
    pattern = torch.arange(local, dtype=torch.int32, device=recv_counts.device).repeat(peers)
    return torch.repeat_interleave(pattern, recv_counts.reshape(-1).long(), output_size=total)


class CudaBackend:
    """The compute stages on one GPU: a route-only plan for the local tokens and a
    fixed-route plan (top-1, capacity rows) over the local experts."""

    def __init__(self, x, gate_up_local, down_local, ids, routing_weights, *, experts, router_weight, capacity,
                 global_routes, gate_up_scales=None, down_scales=None):
        device = x.device
        hidden = x.shape[1]
        local_experts = gate_up_local.shape[0]
        self.token_plan = _prepare(x, None, None, ids, routing_weights, router_weight=router_weight,
                                   route_only_experts=experts)
        self.recv_x = torch.zeros((capacity, hidden), dtype=torch.bfloat16, device=device)
        self.recv_ids = torch.zeros((capacity, 1), dtype=torch.int32, device=device)
        self.recv_rw = torch.ones((capacity, 1), dtype=torch.float32, device=device)
        self.valid = torch.zeros((1,), dtype=torch.int32, device=device)
        inter = down_local.shape[2] * (8 if down_scales is not None else 1)
        tensor_tiles = hidden % 8 == 0 and inter % 8 == 0 and hidden >= 64 and inter >= 64
        # tile from the global load per expert, not from the (worst-case) capacity
        tile = token_tile_for(global_routes, experts, 1) if tensor_tiles else 0
        self.expert_plan = _prepare(self.recv_x, gate_up_local, down_local, self.recv_ids, self.recv_rw,
                                    token_tile=tile, valid_routes=self.valid,
                                    gate_up_scales=gate_up_scales, down_scales=down_scales)
        self.local_experts = local_experts

    # token-owning side
    def route_and_dispatch(self):
        self.token_plan.route()
        self.token_plan.dispatch()
        return self.token_plan.counts

    @property
    def send_rows(self):
        return self.token_plan.grouped_input

    @property
    def return_rows(self):
        return self.token_plan.down_output

    def combine(self):
        self.token_plan.combine()
        return self.token_plan.output

    # expert-owning side
    @property
    def recv_rows(self):
        return self.recv_x

    def set_received(self, expert_ids, total):
        self.recv_ids[:total, 0].copy_(expert_ids)
        self.valid.fill_(total)

    def expert_forward(self):
        return self.expert_plan.run()

    def status(self):
        return int(self.token_plan.status.item()) | int(self.expert_plan.status.item())


@dataclass
class ExpertParallelStats:
    sent: list
    received: list

    @property
    def rows_received(self):
        return sum(self.received)


class ExpertParallelMoE:
    """Prepared expert-parallel layer; ``run()`` returns this rank's ``[T_local, H]`` output."""

    def __init__(self, backend, *, experts, group=None, capacity):
        self.backend = backend
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.experts = experts
        self.local_experts = experts // self.world
        self.capacity = capacity
        self.stats = None
        self.status_flags = 0

    def _exchange_rows(self, recv, send, recv_splits, send_splits):
        # BF16 rows travel as raw bytes (a dtype every backend moves)
        dist.all_to_all_single(recv.view(torch.uint8), send.view(torch.uint8), recv_splits, send_splits,
                               group=self.group)

    def run(self):
        be = self.backend
        counts = be.route_and_dispatch()                                    # [E] int32, local routes per expert
        # every rank learns the whole [G, E] count matrix (G*E int32), so all ranks take the same
        # decision on a capacity overflow without another collective
        all_counts = torch.empty((self.world * self.experts,), dtype=counts.dtype, device=counts.device)
        dist.all_gather_into_tensor(all_counts, counts.contiguous().view(-1), group=self.group)
        by_owner = all_counts.view(self.world, self.world, self.local_experts)       # [source, owner, expert]
        send_counts = by_owner[self.rank]                                             # [owner, E/G]
        recv_counts = by_owner[:, self.rank].contiguous()                             # [source, E/G]
        per_owner = by_owner.sum(dim=(0, 2)).tolist()                                 # the one host read
        send_splits, recv_splits = split_sizes(send_counts), split_sizes(recv_counts)
        n_send, n_recv = sum(send_splits), sum(recv_splits)
        self.stats = ExpertParallelStats(send_splits, recv_splits)
        if max(per_owner) > self.capacity:
            n_recv = int(max(per_owner))
            self.status_flags |= STATUS_EP_OVERFLOW
            raise RuntimeError(f"expert-parallel receive capacity exceeded: {n_recv} rows > {self.capacity} "
                               f"(status {STATUS_EP_OVERFLOW})")
        self._exchange_rows(be.recv_rows[:n_recv], be.send_rows[:n_send], recv_splits, send_splits)
        be.set_received(received_expert_ids(recv_counts, n_recv), n_recv)
        result = be.expert_forward()                                        # [capacity, H], received order
        self._exchange_rows(be.return_rows[:n_send], result[:n_recv], send_splits, recv_splits)
        return be.combine()

    def check_inputs(self):
        flags = self.backend.status() | self.status_flags
        if flags:
            raise ValueError(f"invalid runtime MoE inputs: GPU status={flags} "
                             "(1=IDs, 2=nonfinite weights, 4=kernel wait timeout, 8=EP capacity)")


def prepare_ep_moe(x, gate_up_local, down_local, ids, routing_weights, *, experts, router_weight=None, group=None,
                   capacity=None, gate_up_scales=None, down_scales=None):
    """Prepare the expert-parallel layer on this rank.

    ``x`` [T_local,H] are this rank's tokens; ``gate_up_local`` / ``down_local`` hold only the
    experts of :func:`expert_range`; ``ids`` / ``routing_weights`` [T_local,K] are inputs (global expert
    ids) or, with ``router_weight`` [E,H], outputs. ``capacity`` = rows this rank can receive
    (default: every route of every rank, assuming equal token counts).
    """
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    lo, hi = expert_range(rank, world, experts)
    if gate_up_local.shape[0] != hi - lo or down_local.shape[0] != hi - lo:
        raise ValueError(f"rank {rank} must hold experts [{lo},{hi})")
    routes = ids.numel()
    capacity = capacity if capacity is not None else max(1, routes * world)
    backend = CudaBackend(x, gate_up_local, down_local, ids, routing_weights, experts=experts,
                          router_weight=router_weight, capacity=capacity, global_routes=max(1, routes * world),
                          gate_up_scales=gate_up_scales, down_scales=down_scales)
    return ExpertParallelMoE(backend, experts=experts, group=group, capacity=capacity)


# ------------------------------------------------------------------------------------------------
# Peer-memory mode: rows cross NVLink by plain stores from the dispatch / return kernels
# (csrc/ep.cu). No NCCL call and no host read inside run(): the whole forward is a fixed sequence
# of kernel launches on the current stream.

class _DeviceBytes:
    """Exposes a raw device allocation to torch through the CUDA array interface."""

    def __init__(self, ptr, nbytes):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False),
                                         "version": 3, "strides": None}


class PeerBuffers:
    """One peer-visible allocation per name on every rank; ``ptrs[name][g]`` is rank g's buffer as mapped here."""

    def __init__(self, sizes: dict, group=None):
        import ctypes
        from . import _native
        self._native, self._ctypes = _native, ctypes
        self.lib = _native.load()
        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.local, self.ptrs, self._imported = {}, {}, []
        handles = {}
        for name, nbytes in sizes.items():
            ptr = ctypes.c_void_p()
            _native.check(self.lib.b200moe_peer_alloc(max(256, int(nbytes)), ctypes.byref(ptr)))
            self.local[name] = ptr.value
            handle = ctypes.create_string_buffer(64)
            if self.world > 1:
                _native.check(self.lib.b200moe_peer_export(ptr, handle))
            handles[name] = handle.raw
        everyone = [None] * self.world
        if self.world > 1:
            dist.all_gather_object(everyone, handles, group=group)
        for name in sizes:
            row = []
            for g in range(self.world):
                if g == self.rank:
                    row.append(self.local[name])
                else:
                    ptr = ctypes.c_void_p()
                    _native.check(self.lib.b200moe_peer_import(everyone[g][name], ctypes.byref(ptr)))
                    self._imported.append(ptr.value)
                    row.append(ptr.value)
            self.ptrs[name] = row
        if self.world > 1:
            dist.barrier(group=group)

    def tensor(self, name, nbytes, device):
        return torch.as_tensor(_DeviceBytes(self.local[name], nbytes), device=device)

    def close(self):
        if self.lib is None:
            return
        torch.cuda.synchronize()
        if self.world > 1:
            dist.barrier(group=self.group)  # nobody may still be writing into a buffer about to go away
        for ptr in self._imported:
            self.lib.b200moe_peer_close(self._ctypes.c_void_p(ptr))
        for ptr in self.local.values():
            self.lib.b200moe_peer_free(self._ctypes.c_void_p(ptr))
        self.lib = None


class PeerExpertParallelMoE:
    """Expert-parallel layer whose exchange runs inside the kernels over peer memory."""

    def __init__(self, x, gate_up_local, down_local, ids, routing_weights, *, experts, router_weight=None,
                 group=None, capacity=None, gate_up_scales=None, down_scales=None):
        import ctypes
        from . import _native
        from .moe import _prepare_expert_side
        self._native = _native
        self.lib = _native.load()
        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if self.world > _native.EP_MAX_RANKS:
            raise ValueError("peer-memory expert parallelism covers the GPUs of one node (at most 8 ranks)")
        lo, hi = expert_range(self.rank, self.world, experts)
        if gate_up_local.shape[0] != hi - lo or down_local.shape[0] != hi - lo:
            raise ValueError(f"rank {self.rank} must hold experts [{lo},{hi})")
        device = x.device
        tokens, hidden = x.shape
        topk = ids.shape[1]
        routes = tokens * topk
        self.capacity = capacity if capacity is not None else max(1, routes * self.world)
        row_bytes = hidden * 2
        sizes = {"recv": self.capacity * row_bytes, "ret": max(1, routes) * row_bytes,
                 "counts": self.world * experts * 4, "flags": 256, "dest": self.capacity * 4}
        with torch.cuda.device(device):
            self.buffers = PeerBuffers(sizes, group)
        recv = self.buffers.tensor("recv", sizes["recv"], device).view(torch.bfloat16).view(self.capacity, hidden)
        ret = self.buffers.tensor("ret", max(1, routes) * row_bytes, device).view(torch.bfloat16)[:routes * hidden]
        ret = ret.view(routes, hidden)
        self.token_plan = _prepare(x, None, None, ids, routing_weights, router_weight=router_weight,
                                   route_only_experts=experts, copy_rows=False, workspace={"down_output": ret},
                                   warm=False)
        inter = down_local.shape[2] * (8 if down_scales is not None else 1)
        tensor_tiles = hidden % 8 == 0 and inter % 8 == 0 and hidden >= 64 and inter >= 64
        tile = token_tile_for(max(1, routes * self.world), experts, 1) if tensor_tiles else 0
        dest = self.buffers.tensor("dest", self.capacity * 4, device).view(torch.int32)
        self.return_bases = torch.tensor(self.buffers.ptrs["ret"] + [0] * (_native.EP_MAX_RANKS - self.world),
                                         dtype=torch.int64, device=device)
        self.expert_plan = _prepare_expert_side(gate_up_local, down_local, recv, token_tile=tile,
                                                gate_up_scales=gate_up_scales, down_scales=down_scales,
                                                row_dest=dest, return_bases=self.return_bases)
        self.expert_rows = torch.zeros((1,), dtype=torch.int32, device=device)
        self.tables = torch.zeros((int(self.lib.b200moe_ep_table_ints(self.world, experts)),), dtype=torch.int32,
                                  device=device)
        tp, ep = self.token_plan, self.expert_plan
        ptr = lambda t: ctypes.c_void_p(t.data_ptr())
        args = _native.EpArgs(rank=self.rank, world=self.world, experts=experts, topk=topk, hidden=hidden,
                              tokens=tokens, capacity=self.capacity, token_tile=ep.token_tile,
                              ids_are_int64=int(ids.dtype == torch.int64),
                              x=ptr(x), ids=ptr(ids), ranks=ptr(tp.ranks), counts=ptr(tp.counts),
                              expert_counts=ptr(ep.counts), expert_offsets=ptr(ep.offsets), expert_tasks=ptr(ep.tasks),
                              expert_rows=ptr(self.expert_rows), expert_output=ptr(ep.down_output),
                              tables=ptr(self.tables), status=ptr(tp.status),
                              expert_chain=ctypes.c_void_p(ep.chain[0]), expert_chain_words=ep.chain[1],
                              expert_status=ptr(ep.status), mapping=ptr(tp.mapping),
                              fused_return=int(ep.fused_return))
        for field, name in (("recv_rows_peers", "recv"), ("return_rows_peers", "ret"),
                            ("all_counts_peers", "counts"), ("flags_peers", "flags"), ("row_dest_peers", "dest")):
            array = getattr(args, field)
            for g in range(self.world):
                array[g] = self.buffers.ptrs[name][g]
        self.args = args
        self._device = device
        self.stats = None
        self.run()  # warm-up forward, as every prepare entry point does

    def run(self):
        check, lib, args = self._native.check, self.lib, ctypes_byref(self.args)
        tp, ep = self.token_plan, self.expert_plan
        stream = torch.cuda.current_stream(self._device).cuda_stream
        tp.route()
        tp.dispatch()
        check(lib.b200moe_ep_exchange_counts(args, stream))
        check(lib.b200moe_ep_send_rows(args, stream))
        # gate/up + SwiGLU and down over the received rows, as one forward of the expert plan: the two kernels are
        # chained through the completion counters that the count exchange zeroed, and (BF16 tensor-core schedule)
        # the down projection stores every result row straight into its token owner's buffer over NVLink
        check(ep._forward(ep._plan, stream))
        check(lib.b200moe_ep_return_rows(args, stream))   # fused return: only the closing barrier
        tp.combine()
        return tp.output

    @property
    def rows_received(self):
        return int(self.expert_rows.item())

    def check_inputs(self):
        flags = int(self.token_plan.status.item()) | int(self.expert_plan.status.item())
        if flags:
            raise ValueError(f"invalid runtime MoE inputs: GPU status={flags} "
                             "(1=IDs, 2=nonfinite weights, 4=kernel wait timeout, 8=EP capacity)")

    def close(self):
        self.buffers.close()


def ctypes_byref(obj):
    import ctypes
    return ctypes.byref(obj)


def prepare_peer_ep_moe(x, gate_up_local, down_local, ids, routing_weights, *, experts, router_weight=None,
                        group=None, capacity=None, gate_up_scales=None, down_scales=None):
    """Expert-parallel layer with the exchange fused into the dispatch / return kernels over NVLink
    peer memory. Same arguments as :func:`prepare_ep_moe`. Call ``close()`` before the process group goes away."""
    return PeerExpertParallelMoE(x, gate_up_local, down_local, ids, routing_weights, experts=experts,
                                 router_weight=router_weight, group=group, capacity=capacity,
                                 gate_up_scales=gate_up_scales, down_scales=down_scales)
