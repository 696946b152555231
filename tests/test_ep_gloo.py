"""Expert-parallel exchange logic on two CPU ranks over gloo (no GPU).

The compute stages are played by the CPU oracle; what is under test is the
host side of llm_gpu_kernels_b200.moe_ep: expert ownership, split sizes, the
order of rows on the wire, the ids rebuilt on the receiving side and the way
back. Two ranks together must reproduce the single-process oracle."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import moe_oracle as O
from tests.util import make_inputs


class OracleBackend:
    def __init__(self, x, gate_up_local, down_local, ids, rw, experts, capacity):
        self.x, self.gu, self.dn, self.ids, self.rw, self.experts = x, gate_up_local, down_local, ids, rw, experts
        self.recv = torch.zeros(capacity, x.shape[1], dtype=torch.bfloat16)
        self.ret = torch.zeros(ids.numel(), x.shape[1], dtype=torch.bfloat16)

    def route_and_dispatch(self):
        counts, _, _, self.mapping = O.dispatch_oracle(self.ids, self.experts)
        self.grouped = O.grouped_input_oracle(self.x, self.mapping, self.ids.shape[1])
        return counts

    send_rows = property(lambda self: self.grouped)
    return_rows = property(lambda self: self.ret)
    recv_rows = property(lambda self: self.recv)

    def set_received(self, expert_ids, total):
        self.recv_ids, self.total = expert_ids.long(), total

    def expert_forward(self):
        out = torch.zeros_like(self.recv)
        if self.total:
            rows = self.recv[:self.total]
            y = O.moe_oracle(rows, self.gu, self.dn, self.recv_ids[:, None], torch.ones(self.total, 1))
            out[:self.total] = y.bfloat16()
        return out

    def combine(self):
        k = self.ids.shape[1]
        picked = self.ret[self.mapping.long()].float().reshape(-1, k, self.ret.shape[1])
        return (picked * self.rw[:, :, None]).sum(1)

    def status(self):
        return 0


def _worker(rank, world, port, result):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from llm_gpu_kernels_b200.moe_ep import ExpertParallelMoE, expert_range
        experts, topk, hidden, inter, t_local = 8, 2, 32, 16, 11
        x, gu, dn, ids, rw = make_inputs(t_local * world, experts, topk, hidden, inter, seed=3, pattern="hot",
                                         id_dtype=torch.int64, signed=True)
        lo, hi = expert_range(rank, world, experts)
        mine = slice(rank * t_local, (rank + 1) * t_local)
        backend = OracleBackend(x[mine], gu[lo:hi], dn[lo:hi], ids[mine], rw[mine], experts, t_local * topk * world)
        ep = ExpertParallelMoE(backend, experts=experts, capacity=t_local * topk * world)
        out = ep.run()
        ref = O.moe_oracle(x, gu, dn, ids, rw)[mine]
        m = O.error_metrics(out, ref)
        assert m["relative_rms"] < 5e-3, m
        # every route of every rank arrived at its owner exactly once
        received = torch.tensor([ep.stats.rows_received])
        dist.all_reduce(received)
        assert int(received) == ids.numel()
        owned = ((ids >= lo) & (ids < hi)).sum().item()
        assert ep.stats.rows_received == owned
        ep.check_inputs()
        # capacity overflow is reported, not silently truncated
        small = ExpertParallelMoE(backend, experts=experts, capacity=1)
        with pytest.raises(RuntimeError, match="capacity"):
            small.run()
        result[rank] = m["relative_rms"]
    finally:
        dist.destroy_process_group()


def test_two_ranks_reproduce_single_process_oracle():
    world = 2
    manager = mp.Manager()
    result = manager.dict()
    mp.spawn(_worker, args=(world, 29731, result), nprocs=world, join=True)
    assert len(result) == world


def test_helpers():
    from llm_gpu_kernels_b200.moe_ep import expert_range, received_expert_ids, split_sizes
    assert expert_range(3, 4, 128) == (96, 128)
    with pytest.raises(ValueError):
        expert_range(0, 3, 128)
    counts = torch.tensor([[2, 0, 1], [0, 3, 0]], dtype=torch.int32)
    assert split_sizes(counts) == [3, 3]
    assert received_expert_ids(counts, 6).tolist() == [0, 0, 2, 1, 1, 1]
