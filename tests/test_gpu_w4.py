"""W4A16 parity on a B200: packed int4 weights (reference W4G128 v1 format) through the CUDA path,
against the FP32 oracle evaluated on the dequantised weights. Tolerance: relative RMS 1e-2."""
import pytest
import torch

from llm_gpu_kernels_b200.moe_weight_layout import repack_gate_up
from llm_gpu_kernels_b200.moe_weight_quant import dequantize_gate_up_reference, quantize_down, quantize_gate_up
from oracle import moe_oracle as O
from tests.util import make_inputs, seeded_layer

pytestmark = pytest.mark.gpu
REL_RMS_W4 = 1e-2


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available()
    return torch.device("cuda:0")


def check(out, x, gate_up_deq, down_deq, ids, rw):
    m = O.error_metrics(out.float().cpu(), O.moe_oracle(x, gate_up_deq, down_deq, ids.cpu(), rw.cpu()))
    assert m["finite"] and m["relative_rms"] <= REL_RMS_W4 and m["normalized_max"] <= REL_RMS_W4, m
    return m


@pytest.mark.parametrize("tile", [0, 16, 64])
def test_down_dequant_is_bit_exact(dev, tile):
    """One-hot activation rows make the down GEMM print the dequantised operand itself:
    down_output[row, c] must equal bf16_rn(q * scale) of weight [expert, c, k] exactly. Tile 16 is the
    weight-streaming kernel (dequantisation in registers), 64 the tensor-memory operand, the default (128) the
    shared-memory operand."""
    from llm_gpu_kernels_b200.gemm import GemmConfig
    from llm_gpu_kernels_b200.moe_w4_cuda import prepare_w4_moe
    e, h, i, t, k = 3, 256, 256, 64, 2
    x, gate_up, down, ids, rw = make_inputs(t, e, k, h, i, seed=1, wscale=0.05)
    pg, pd = quantize_gate_up(gate_up), quantize_down(down)
    p = prepare_w4_moe(x.to(dev), pg.to(dev), None, ids.to(dev), rw.to(dev), packed_down=pd.to(dev),
                       down_config=GemmConfig(block_m=tile) if tile else None)
    assert p.base.token_tile == (tile or 128)
    base = p.base
    rows = t * k
    hot = torch.arange(rows) * 7 % i
    act = torch.zeros(rows, i, dtype=torch.bfloat16)
    act[torch.arange(rows), hot] = 1.0
    base.activated.copy_(act)
    base.down_project()
    torch.cuda.synchronize()
    deq = dequantize_gate_up_reference(pd)                      # [E, H, I]
    offsets = base.offsets.cpu().tolist() + [rows]
    got = base.down_output.cpu()
    for expert in range(e):
        for row in range(offsets[expert], offsets[expert + 1]):
            assert torch.equal(got[row], deq[expert, :, hot[row]]), (expert, row)


@pytest.mark.parametrize("t,e,k,h,i,both,tile", [
    (40, 8, 2, 256, 128, False, 0), (40, 8, 2, 256, 128, True, 0), (130, 4, 4, 128, 384, True, 64),
    (300, 2, 1, 384, 256, True, 256), (9, 16, 8, 512, 128, False, 16),
    # the weight-streaming kernel (tile 16): many token tiles per expert, K of one half stage (128) and of one and
    # a half stages (384), 256-channel down tiles with a ragged upper half (H = 128, 384), I not a multiple of 16
    (40, 8, 2, 256, 128, True, 16), (130, 4, 4, 128, 384, True, 16), (33, 4, 2, 384, 256, True, 16),
    (20, 3, 1, 128, 72, False, 16), (5, 32, 4, 2048, 768, True, 16), (64, 2, 2, 1024, 128, True, 16),
])
def test_w4_small_shapes(dev, t, e, k, h, i, both, tile):
    from llm_gpu_kernels_b200.gemm import GemmConfig
    from llm_gpu_kernels_b200.moe_w4_cuda import prepare_w4_moe
    x, gate_up, down, ids, rw = make_inputs(t, e, k, h, i, seed=50 + t, wscale=0.05, signed=True)
    pg = quantize_gate_up(gate_up)
    pd = quantize_down(down) if both else None
    cfg = GemmConfig(block_m=tile) if tile else None
    p = prepare_w4_moe(x.to(dev), pg.to(dev), None if both else down.to(dev), ids.to(dev), rw.to(dev),
                       packed_down=pd.to(dev) if both else None, down_config=cfg)
    out = p.run()
    torch.cuda.synchronize()
    p.check_inputs()
    check(out, x, dequantize_gate_up_reference(pg), dequantize_gate_up_reference(pd) if both else down, ids, rw)
    assert torch.equal(p.run(), out)
    assert p.base.gathers == (p.base.token_tile <= 16)
    if p.base.gathers:   # the materialised dispatch gives the same bits
        kept = prepare_w4_moe(x.to(dev), pg.to(dev), None if both else down.to(dev), ids.to(dev), rw.to(dev),
                              packed_down=pd.to(dev) if both else None, down_config=cfg, keep_grouped_input=True)
        assert not kept.base.gathers and torch.equal(kept.run(), out)


@pytest.fixture(scope="module")
def qwen_w4():
    wr, gate_up, down, _ = seeded_layer(0, 1, 2048, 768, 128)
    pg, pd = quantize_gate_up(gate_up), quantize_down(down)
    return wr, pg, pd, dequantize_gate_up_reference(pg), dequantize_gate_up_reference(pd), down


@pytest.mark.parametrize("tokens", [17, 193, 1024])
def test_qwen_shape_w4(dev, qwen_w4, tokens):
    """benchmark configuration 3: Qwen3-30B-A3B layer shape, gate/up and down both W4G128, router on."""
    from llm_gpu_kernels_b200.moe_w4_cuda import prepare_w4_moe
    wr, pg, pd, gate_up_deq, down_deq, _ = qwen_w4
    x = torch.randn(tokens, 2048, generator=torch.Generator().manual_seed(tokens)).bfloat16()
    ids = torch.zeros(tokens, 8, dtype=torch.int32, device=dev)
    rw = torch.zeros(tokens, 8, dtype=torch.float32, device=dev)
    p = prepare_w4_moe(x.to(dev), pg.to(dev), None, ids, rw, packed_down=pd.to(dev), router_weight=wr.to(dev))
    out = p.run()
    torch.cuda.synchronize()
    p.check_inputs()
    _, _, probs = O.router_oracle(x, wr, 8)
    ok, msg = O.router_agrees(ids.cpu(), rw.cpu(), probs, 8)
    assert ok, msg
    m = check(out, x, gate_up_deq, down_deq, ids, rw)
    print(f"W4 T={tokens} rel_rms={m['relative_rms']:.2e}")


def test_reference_configuration_gate_up_only_and_layout_entry(dev, qwen_w4):
    """The reference packs gate/up only (down BF16); its re-laid-out pack must give the same bits."""
    from llm_gpu_kernels_b200.moe_w4_cuda import prepare_w4_moe
    from llm_gpu_kernels_b200.moe_w4_layout_cuda import prepare_w4_layout_moe
    wr, pg, pd, gate_up_deq, _, down = qwen_w4
    x, _, _, ids, rw = make_inputs(193, 128, 8, 2048, 8, seed=9, pattern="hot")
    args = (x.to(dev),)
    a = prepare_w4_moe(x.to(dev), pg.to(dev), down.to(dev), ids.to(dev), rw.to(dev))
    out = a.run().clone()
    check(out, x, gate_up_deq, down, ids, rw)
    b = prepare_w4_layout_moe(x.to(dev), repack_gate_up(pg).to(dev), down.to(dev), ids.to(dev), rw.to(dev))
    assert torch.equal(b.run(), out)
    assert a.names == ("dispatch", "gate_up_swiglu", "down", "combine")


def test_w4_rejections(dev):
    from llm_gpu_kernels_b200.moe_w4_cuda import prepare_w4_moe
    x, gate_up, down, ids, rw = make_inputs(4, 2, 1, 128, 128, seed=2)
    pg = quantize_gate_up(gate_up)
    with pytest.raises(ValueError):
        prepare_w4_moe(x.to(dev), pg, down.to(dev), ids.to(dev), rw.to(dev))          # pack still on the host
    with pytest.raises(ValueError):
        prepare_w4_moe(x.to(dev), "packed", down.to(dev), ids.to(dev), rw.to(dev))
    with pytest.raises(ValueError):
        prepare_w4_moe(x.to(dev), pg.to(dev), down.to(dev), ids.to(dev), rw.to(dev), packed_down=pg.to(dev))
