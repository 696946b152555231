"""Host-side logic and the C-ABI surface; nothing here needs a GPU."""
import ctypes
import re
from pathlib import Path

import pytest
import torch

from llm_gpu_kernels_b200 import _native, moe_full_policy
from llm_gpu_kernels_b200.gemm import GemmConfig
from llm_gpu_kernels_b200.moe import prepare_moe

ROOT = Path(__file__).resolve().parents[1]


def declared_symbols():
    text = "\n".join(p.read_text() for p in (ROOT / "include").glob("*.h"))
    return sorted(set(re.findall(r"\b(b200moe_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _native.load()
    names = declared_symbols()
    assert len(names) >= 12
    for name in names:
        assert hasattr(lib, name), f"{name} declared in include/ but not exported"
    assert set(names) >= set(_native.EXPORTS)
    assert lib.b200moe_abi_version() == _native.ABI_VERSION


def make_plan(**kw):
    lib = _native.load()
    fields = dict(tokens=17, experts=128, topk=8, hidden=2048, intermediate=768)
    fields.update(kw)
    shape = _native.Shape(**fields)
    handle = ctypes.c_void_p()
    code = lib.b200moe_plan_create(ctypes.byref(shape), ctypes.byref(handle))
    return lib, code, handle


def test_plan_create_and_workspace_sizes():
    lib, code, handle = make_plan()
    assert code == 0
    ws = _native.Workspace()
    assert lib.b200moe_plan_workspace(handle, ctypes.byref(ws)) == 0
    r = 17 * 8
    assert ws.output == 17 * 2048 * 2 and ws.mapping == r * 4 and ws.ranks == r * 4
    assert ws.grouped_input == r * 2048 * 2 and ws.activated == r * 768 * 2 and ws.down_output == r * 2048 * 2
    assert ws.tasks == 129 * 4 and ws.status == 4
    assert ws.schedule == _native.SCHEDULE_TCGEN05 and ws.token_tile == 16 and ws.launches == 5
    lib.b200moe_plan_destroy(handle)


@pytest.mark.parametrize("tokens,expect", [(17, 16), (193, 32), (1024, 128), (8192, 128), (16384, 256)])
def test_token_tile_is_shape_only(tokens, expect):
    lib, code, handle = make_plan(tokens=tokens)
    ws = _native.Workspace()
    lib.b200moe_plan_workspace(handle, ctypes.byref(ws))
    assert ws.token_tile == expect == moe_full_policy.token_tile_for(tokens, 128, 8)
    lib.b200moe_plan_destroy(handle)


@pytest.mark.parametrize("kw", [dict(experts=0), dict(experts=257), dict(topk=0), dict(topk=33), dict(hidden=0),
                                dict(intermediate=0), dict(tokens=-1), dict(tokens=2**20, topk=32),
                                dict(token_tile=48), dict(schedule=9)])
def test_plan_create_rejects(kw):
    lib, code, _ = make_plan(**kw)
    assert code == _native.ERR_INVALID
    assert _native.last_error()
    with pytest.raises(ValueError):
        _native.check(code)


def resolved(**kw):
    lib, code, handle = make_plan(**kw)
    assert code == 0, _native.last_error()
    ws = _native.Workspace()
    assert lib.b200moe_plan_workspace(handle, ctypes.byref(ws)) == 0
    out = {name: getattr(ws, name) for name, _ in _native.Workspace._fields_ if name != "reserved"}
    lib.b200moe_plan_destroy(handle)
    return out


def test_gather_rule_is_shape_only():
    """fused_gather = 1 gathers while experts average at most three 128-row tiles (routes <= 384 x experts); 2 always;
    0 never. A gathering plan has no grouped_input and a source_rows table instead."""
    for tokens, expect in ((17, 1), (1024, 1), (6144, 1), (6145, 0), (8192, 0)):
        ws = resolved(tokens=tokens, fused_gather=1)
        assert ws["gathers"] == expect, tokens
        assert ws["grouped_input"] == (0 if expect else tokens * 8 * 2048 * 2)
        assert ws["source_rows"] == (tokens * 8 * 4 if expect else 0)
    assert resolved(tokens=8192, fused_gather=2)["gathers"] == 1
    assert resolved(tokens=1024, fused_gather=0)["gathers"] == 0
    assert resolved(tokens=1024)["gathers"] == 0                      # the C default of the field is 0
    assert make_plan(fused_gather=3)[1] == _native.ERR_INVALID


def test_down_schedule_resolution():
    """down_tiles: 0 resolves to pair tiles up to token tile 128 and to one 128-channel tile at 256; 3 (wide) needs
    token tile 128; W4 and generic plans report 0."""
    assert resolved(tokens=17)["down_tiles"] == 1 and resolved(tokens=8192)["down_tiles"] == 1
    assert resolved(tokens=16384)["token_tile"] == 256 and resolved(tokens=16384)["down_tiles"] == 2
    assert resolved(tokens=1024, down_tiles=2)["down_tiles"] == 2
    assert resolved(tokens=1024, down_tiles=3)["down_tiles"] == 3
    assert resolved(tokens=17, token_tile=128, down_tiles=3)["down_tiles"] == 3
    assert make_plan(tokens=17, down_tiles=3)[1] == _native.ERR_INVALID          # token tile 16
    assert make_plan(tokens=16384, down_tiles=3)[1] == _native.ERR_INVALID       # token tile 256
    assert make_plan(down_tiles=4)[1] == _native.ERR_INVALID
    assert resolved(down_format=_native.WEIGHTS_W4G128, gate_up_format=_native.WEIGHTS_W4G128)["down_tiles"] == 0
    assert resolved(hidden=67, intermediate=33, experts=3, topk=2, tokens=9)["down_tiles"] == 0


@pytest.mark.parametrize("tokens,launches", [(17, 5), (256, 5), (257, 5), (1024, 5), (2048, 5), (2049, 7), (8192, 7)])
def test_launches_per_forward(tokens, launches):
    """Router + dispatch + gate/up + down + combine: the dispatch is one kernel up to 16384 routes (a cluster of 1, 2,
    4 or 8 blocks) when no rows are copied, three kernels above."""
    assert resolved(tokens=tokens, use_router=1, fused_gather=1)["launches"] == launches


def test_odd_shapes_take_the_generic_schedule():
    lib, code, handle = make_plan(hidden=67, intermediate=33, experts=3, topk=2, tokens=9)
    assert code == 0
    ws = _native.Workspace()
    lib.b200moe_plan_workspace(handle, ctypes.byref(ws))
    assert ws.schedule == _native.SCHEDULE_GENERIC and ws.token_tile == 32
    lib.b200moe_plan_destroy(handle)
    _, code, _ = make_plan(hidden=67, intermediate=33, schedule=_native.SCHEDULE_TCGEN05)
    assert code == _native.ERR_UNSUPPORTED


def test_forward_before_bind_is_a_state_error():
    lib, code, handle = make_plan()
    assert lib.b200moe_forward(handle, None) == _native.ERR_STATE
    assert "bind" in _native.last_error()
    lib.b200moe_plan_destroy(handle)


def test_gemm_config_validation():
    assert GemmConfig().block_m == 32
    for bad in (dict(block_m=8), dict(block_n=48), dict(warps=2), dict(stages=5)):
        with pytest.raises(ValueError):
            GemmConfig(**bad)


def test_policy_is_shape_only():
    cfg, bucket = moe_full_policy.select(17, 128, 8, 2048, 768)
    assert (cfg.block_m, bucket) == (16, "small")
    assert moe_full_policy.select(1024, 128, 8, 2048, 768)[1] == "medium"
    assert moe_full_policy.select(4096, 128, 8, 2048, 768) == (GemmConfig(block_m=128), "large")
    assert moe_full_policy.select(0, 128, 8, 2048, 768)[1] == "small"
    with pytest.raises(ValueError):
        moe_full_policy.select(-1, 128, 8, 2048, 768)


def test_prepare_rejects_host_tensors_without_touching_a_gpu():
    x = torch.zeros(4, 64, dtype=torch.bfloat16)
    gu = torch.zeros(2, 128, 64, dtype=torch.bfloat16)
    dn = torch.zeros(2, 64, 64, dtype=torch.bfloat16)
    ids = torch.zeros(4, 2, dtype=torch.int32)
    rw = torch.zeros(4, 2)
    with pytest.raises(ValueError, match="contiguous CUDA BF16"):
        prepare_moe(x, gu, dn, ids, rw)
