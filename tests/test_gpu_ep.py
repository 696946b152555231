"""Expert-parallel path on GPUs: NCCL all-to-all between ranks, each rank running the CUDA
plans. One-rank case runs in-process on any B200; the two-rank case needs two GPUs."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import moe_oracle as O
from tests.util import make_inputs, seeded_layer

pytestmark = pytest.mark.gpu


def _run_rank(rank, world, port, shape, result):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from llm_gpu_kernels_b200.moe_ep import expert_range, prepare_ep_moe
        from llm_gpu_kernels_b200.moe_ranked import prepare_ranked_moe_launcher
        t_local, experts, topk, hidden, inter, use_router = shape
        wr, gate_up, down, x = seeded_layer(5, t_local * world, hidden, inter, experts, wscale=0.05)
        _, _, _, ids_all, rw_all = make_inputs(t_local * world, experts, topk, 8, 8, seed=6, pattern="hot")
        lo, hi = expert_range(rank, world, experts)
        mine = slice(rank * t_local, (rank + 1) * t_local)
        ids = ids_all[mine].contiguous().to(dev)
        rw = rw_all[mine].contiguous().to(dev)
        ep = prepare_ep_moe(x[mine].contiguous().to(dev), gate_up[lo:hi].contiguous().to(dev),
                            down[lo:hi].contiguous().to(dev), ids, rw, experts=experts,
                            router_weight=wr.to(dev) if use_router else None)
        for _ in range(2):
            out = ep.run()
        torch.cuda.synchronize()
        ep.check_inputs()
        # parity 1: against the FP32 oracle on the routes this rank used
        ref = O.moe_oracle(x[mine], gate_up, down, ids.cpu(), rw.cpu())
        m = O.error_metrics(out.float().cpu(), ref)
        assert m["relative_rms"] <= 5e-3 and m["normalized_max"] <= 8e-3, m
        # parity 2: bit-identical to the single-GPU plan on the same tokens, routes and tile schedule
        expert_plan = ep.backend.expert_plan
        pinned = dict(token_tile=expert_plan.token_tile, down_tiles=expert_plan.down_tiles) if expert_plan.schedule == "tcgen05" else {}
        single = prepare_ranked_moe_launcher(x[mine].contiguous().to(dev), gate_up.to(dev), down.to(dev),
                                             ids.clone(), rw.clone(), **pinned)
        assert torch.equal(single.run(), out)
        # parity 3: the counts of all ranks add up to the global histogram, bit-exact
        total = ep.backend.token_plan.counts.clone()
        dist.all_reduce(total)
        gathered = [torch.empty_like(ids) for _ in range(world)]
        dist.all_gather(gathered, ids)
        expect = torch.bincount(torch.cat(gathered).reshape(-1).long().cpu(), minlength=experts)
        assert torch.equal(total.cpu().long(), expect)
        # peer-memory mode: the exchange runs inside the kernels over NVLink; same bits, no host read
        from llm_gpu_kernels_b200.moe_ep import prepare_peer_ep_moe
        ids2, rw2 = ids.clone(), rw.clone()
        peer = prepare_peer_ep_moe(x[mine].contiguous().to(dev), gate_up[lo:hi].contiguous().to(dev),
                                   down[lo:hi].contiguous().to(dev), ids2, rw2, experts=experts,
                                   router_weight=wr.to(dev) if use_router else None)
        try:
            for _ in range(3):
                out2 = peer.run()
            torch.cuda.synchronize()
            peer.check_inputs()
            assert torch.equal(ids2, ids) and torch.equal(out2, out)
            assert peer.rows_received == ep.stats.rows_received
            # new routes in place (all to the last expert: one rank receives everything), then back
            if not use_router:
                keep = ids2.clone()
                ids2.fill_(experts - 1)
                out3 = peer.run()
                torch.cuda.synchronize()
                peer.check_inputs()
                ref3 = O.moe_oracle(x[mine], gate_up, down, ids2.cpu(), rw2.cpu())
                m3 = O.error_metrics(out3.float().cpu(), ref3)
                assert m3["relative_rms"] <= 5e-3, m3
                assert peer.rows_received == (t_local * topk * world if rank == world - 1 else 0)
                ids2.copy_(keep)
                assert torch.equal(peer.run(), out)
        finally:
            peer.close()
        result[rank] = (m["relative_rms"], ep.stats.rows_received)
    finally:
        dist.destroy_process_group()


SHAPES = [(96, 16, 4, 256, 128, False), (50, 8, 2, 128, 64, True), (33, 4, 2, 72, 40, True)]


@pytest.mark.parametrize("shape", SHAPES)
def test_one_rank_expert_parallel(shape):
    result = mp.Manager().dict()
    mp.spawn(_run_rank, args=(1, 29741, shape, result), nprocs=1, join=True)
    assert result[0][1] == shape[0] * shape[2]


# the last shape: one expert per rank with 4096 rows each, i.e. token tile 256 on the expert side (one MMA issuer,
# rows returned from the down epilogue without a second partial sum)
@pytest.mark.parametrize("shape", [(96, 16, 4, 256, 128, True), (1024, 128, 8, 2048, 768, True),
                                   (2048, 2, 2, 512, 1024, True)])
def test_two_rank_expert_parallel(shape):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    result = mp.Manager().dict()
    mp.spawn(_run_rank, args=(2, 29743, shape, result), nprocs=2, join=True)
    assert sum(v[1] for v in result.values()) == 2 * shape[0] * shape[2]


def _run_overflow(rank, world, port, result):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from llm_gpu_kernels_b200.moe_ep import expert_range, prepare_peer_ep_moe
        t_local, experts, topk, hidden, inter = 40, 8, 2, 128, 64
        x, gate_up, down, ids_all, rw_all = make_inputs(t_local * world, experts, topk, hidden, inter, seed=12,
                                                        pattern="balanced", wscale=0.1)
        lo, hi = expert_range(rank, world, experts)
        mine = slice(rank * t_local, (rank + 1) * t_local)
        ids, rw = ids_all[mine].contiguous().to(dev), rw_all[mine].contiguous().to(dev)
        capacity = 100                      # balanced routes: 80 rows per rank fit; everything to one expert does not
        peer = prepare_peer_ep_moe(x[mine].contiguous().to(dev), gate_up[lo:hi].contiguous().to(dev),
                                   down[lo:hi].contiguous().to(dev), ids, rw, experts=experts, capacity=capacity)
        try:
            out = peer.run().clone()
            torch.cuda.synchronize()
            peer.check_inputs()
            ref = O.moe_oracle(x[mine], gate_up, down, ids.cpu(), rw.cpu())
            assert O.error_metrics(out.float().cpu(), ref)["relative_rms"] <= 5e-3
            keep = ids.clone()
            ids.fill_(experts - 1)          # 160 rows for the last rank: more than its receive buffer holds
            peer.run()
            torch.cuda.synchronize()
            status = int(peer.token_plan.status.item())
            with pytest.raises(ValueError, match="status=8"):
                peer.check_inputs()
            ids.copy_(keep)                 # the next forward restarts the status words on both plans
            assert torch.equal(peer.run(), out)
            peer.check_inputs()
            result[rank] = status
        finally:
            peer.close()
    finally:
        dist.destroy_process_group()


def test_two_rank_receive_overflow_is_flagged_on_every_rank():
    """Every rank sees the same count matrix, so the rank whose own rows all fit must raise status 8 too (it
    would otherwise combine rows the overflowing owner never produced)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    result = mp.Manager().dict()
    mp.spawn(_run_overflow, args=(2, 29747, result), nprocs=2, join=True)
    assert dict(result) == {0: 8, 1: 8}


def test_absent_peer_is_reported_not_waited_for():
    """A rank whose peer never arrives: the count exchange's barrier gives up after its 1 s bound, raises status
    bit 4 (a bounded wait ran out) and returns; the context stays usable. The "peer" is a second set of local
    buffers that nothing ever writes - no second process, no second kernel."""
    import ctypes
    import time
    from llm_gpu_kernels_b200 import _native
    from llm_gpu_kernels_b200.moe_ranked import prepare_ranked_moe_launcher
    lib = _native.load()
    dev = torch.device("cuda:0")
    experts, topk, hidden, tokens, capacity = 8, 2, 128, 16, 64
    i32 = lambda n: torch.zeros(n, dtype=torch.int32, device=dev)
    bf16 = lambda *s: torch.zeros(*s, dtype=torch.bfloat16, device=dev)
    ptr = lambda t: ctypes.c_void_p(t.data_ptr())
    x, ids, ranks, counts, status = bf16(tokens, hidden), i32(tokens * topk), i32(tokens * topk), i32(experts), i32(1)
    keep = dict(ec=i32(experts), eo=i32(experts), et=i32(experts + 1), er=i32(1), out=bf16(capacity, hidden),
                tables=i32(int(lib.b200moe_ep_table_ints(2, experts))))
    peers = {name: [make() for _ in range(2)] for name, make in (
        ("recv_rows_peers", lambda: bf16(capacity, hidden)), ("return_rows_peers", lambda: bf16(tokens * topk, hidden)),
        ("all_counts_peers", lambda: i32(2 * experts)), ("flags_peers", lambda: i32(64)))}
    args = _native.EpArgs(rank=0, world=2, experts=experts, topk=topk, hidden=hidden, tokens=tokens,
                          capacity=capacity, token_tile=16, ids_are_int64=0, x=ptr(x), ids=ptr(ids), ranks=ptr(ranks),
                          counts=ptr(counts), expert_counts=ptr(keep["ec"]), expert_offsets=ptr(keep["eo"]),
                          expert_tasks=ptr(keep["et"]), expert_rows=ptr(keep["er"]), expert_output=ptr(keep["out"]),
                          tables=ptr(keep["tables"]), status=ptr(status))
    for field, buffers in peers.items():
        for g in range(2):
            getattr(args, field)[g] = buffers[g].data_ptr()
    stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    torch.cuda.synchronize()
    start = time.time()
    _native.check(lib.b200moe_ep_exchange_counts(ctypes.byref(args), stream))
    torch.cuda.synchronize()
    waited = time.time() - start
    assert int(status) & 4, "the barrier must report that its wait ran out"
    assert 0.5 < waited < 10.0, waited
    # the context is intact: an ordinary layer still runs and checks out
    layer = make_inputs(20, 4, 2, 128, 64, seed=2, wscale=0.1, device=dev)
    prepared = prepare_ranked_moe_launcher(*layer)
    prepared.run()
    prepared.check_inputs()
