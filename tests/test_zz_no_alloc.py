"""The dispatch entry point that allocates nothing (``b200moe_dispatch_static``).

Some hosts cannot call cudaMalloc once they are running: a serving process
whose framework owns all GPU memory, a real-time control loop, a plug-in that
is handed only its input and output buffers. For them the library keeps the
scratch of the dispatch kernels in a fixed device array of its own, good for
up to 65536 routes. These tests call that entry point through the C ABI and
compare it, bit for bit (the tolerance of every dispatch test here), with the
regular ``b200moe_dispatch`` that works on a caller-allocated workspace, and with
the CPU dispatch oracle.
Collected last on purpose: a run that stops at the first failure has then
already run every other test.
"""
import ctypes

import pytest
import torch

from llm_gpu_kernels_b200 import _native
from oracle import moe_oracle as O
from tests.util import make_inputs


def _args(tokens, experts, topk, hidden, ids_are_int64, token_tile, **ptrs):
    fields = {k: ctypes.c_void_p(v.data_ptr()) if v is not None else None for k, v in ptrs.items()}
    return _native.DispatchArgs(tokens=tokens, experts=experts, topk=topk, hidden=hidden,
                                ids_are_int64=ids_are_int64, token_tile=token_tile, **fields)


def test_static_dispatch_refuses_sizes_beyond_its_scratch():
    """Validation happens before the device is touched, so this needs no GPU."""
    lib = _native.load()
    too_many = _native.DispatchArgs(tokens=8193, experts=128, topk=8, hidden=2048, token_tile=16)
    assert 8193 * 8 > _native.STATIC_DISPATCH_MAX_ROUTES
    assert lib.b200moe_dispatch_static(ctypes.byref(too_many), None) == _native.ERR_INVALID
    assert "65536" in _native.last_error()
    for bad in (dict(experts=257), dict(topk=33), dict(hidden=0), dict(token_tile=0)):
        fields = dict(tokens=4, experts=8, topk=2, hidden=64, token_tile=16)
        fields.update(bad)
        assert lib.b200moe_dispatch_static(ctypes.byref(_native.DispatchArgs(**fields)), None) == _native.ERR_INVALID
    # misaligned pointers are refused on the host too (never dereferenced: the check comes before any launch)
    names = ("x", "ids", "routing_weights", "counts", "offsets", "cursors", "tasks", "ranks", "mapping",
             "grouped_input", "status")
    good = {name: 0x10000 + 0x1000 * i for i, name in enumerate(names)}
    for name, skew, int64 in (("counts", 2, 0), ("routing_weights", 1, 0), ("ids", 4, 1), ("ids", 2, 0), ("x", 1, 0),
                              ("status", 2, 0), ("mapping", 3, 0)):
        ptrs = dict(good)
        ptrs[name] += skew
        bad = _native.DispatchArgs(tokens=4, experts=8, topk=2, hidden=64, ids_are_int64=int64, token_tile=16, **ptrs)
        assert lib.b200moe_dispatch_static(ctypes.byref(bad), None) == _native.ERR_INVALID, name
        assert "misaligned" in _native.last_error()


@pytest.mark.gpu
@pytest.mark.parametrize("tokens,experts,topk,hidden,id_dtype", [
    (2500, 64, 8, 64, torch.int32),     # 20000 routes: 157 partitions of the counting kernel
    (193, 128, 8, 256, torch.int64),    # a size the regular entry point serves with its one-block path
])
def test_static_dispatch_matches_regular_dispatch_twice(tokens, experts, topk, hidden, id_dtype):
    from llm_gpu_kernels_b200.moe import prepare_moe
    assert torch.cuda.is_available()
    dev = torch.device("cuda:0")
    lib = _native.load()
    x, gate_up, down, ids, rw = make_inputs(tokens, experts, topk, hidden, 64, seed=5, id_dtype=id_dtype,
                                            device=dev, wscale=0.1)
    regular = prepare_moe(x, gate_up, down, ids, rw, keep_grouped_input=True)
    routes = tokens * topk
    i32 = lambda n: torch.full((n,), -12345, dtype=torch.int32, device=dev)
    out = dict(counts=i32(experts), offsets=i32(experts), cursors=i32(experts), tasks=i32(experts + 1),
               ranks=i32(routes), mapping=i32(routes),
               grouped_input=torch.zeros(routes, hidden, dtype=torch.bfloat16, device=dev), status=i32(1))
    args = _args(tokens, experts, topk, hidden, int(id_dtype == torch.int64), regular.token_tile,
                 x=x, ids=ids, routing_weights=rw, **out)
    stream = torch.cuda.current_stream(dev).cuda_stream
    # two calls in a row on one stream; the second sees new routes, one bad id and one NaN weight
    for call in range(2):
        if call == 1:
            fresh = make_inputs(tokens, experts, topk, hidden, 64, seed=6, id_dtype=id_dtype, pattern="hot")
            ids.copy_(fresh[3])
            ids[1, 0] = experts
            rw[2, 1] = float("nan")
        regular.dispatch()
        _native.check(lib.b200moe_dispatch_static(ctypes.byref(args), stream))
        torch.cuda.synchronize(dev)
        for name, mine in out.items():
            theirs = getattr(regular, name)
            if name == "grouped_input":
                rows = regular.mapping[regular.mapping >= 0].long()
                assert torch.equal(mine[rows], theirs[rows]), f"call {call}: grouped_input"
            else:
                assert torch.equal(mine, theirs), f"call {call}: {name}"
        assert int(out["status"].item()) == (0 if call == 0 else 3)
        # and against the CPU oracle directly (an invalid id has rank / mapping -1 there as well)
        counts, offsets, ranks, mapping = O.dispatch_oracle(ids.cpu(), experts)
        for name, want in (("counts", counts), ("offsets", offsets), ("ranks", ranks), ("mapping", mapping)):
            assert torch.equal(out[name].cpu(), want), f"call {call}: {name} against the oracle"
        valid = mapping >= 0
        gathered = out["grouped_input"].cpu()[mapping[valid].long()]
        assert torch.equal(gathered, x.cpu().repeat_interleave(topk, 0)[valid]), f"call {call}: rows against the oracle"
