"""Regenerates the golden fixtures in this directory from the reference project.

Run in a container that has the reference checkout (it is NOT needed to run the
tests; the tests only read the committed ``*.pt`` / ``*.json`` files):

    python tests/golden/make_golden.py /path/to/reference

It imports the reference's own Python functions - ``moe_reference``
(src/llm_gpu_kernels/reference.py:17), ``quantize_gate_up`` /
``dequantize_gate_up_reference`` (moe_weight_quant.py:35,55),
``repack_gate_up`` / ``restore_v1_layout`` (moe_weight_layout.py:81,130),
``validate_dispatch`` (moe_benchmark.py:139), ``error`` (benchmark.py:28),
``write_real_moe_trace`` / ``validate_real_moe_trace`` (moe_real_trace.py:267,448) -
runs them on seeded CPU inputs, and stores inputs (small cases) or input
digests (large cases) together with the reference's outputs.
"""
import hashlib
import json
import sys
from pathlib import Path
from types import SimpleNamespace

import torch

HERE = Path(__file__).resolve().parent


def digest(t):
    t = t.detach().cpu().contiguous()
    h = hashlib.sha256(str((str(t.dtype), tuple(t.shape))).encode())
    h.update(t.view(torch.uint8).numpy().tobytes())
    return h.hexdigest()


def seeded_layer(seed, tokens, hidden, inter, experts, wscale):
    """Draw order: router weight, gate_up, down, x; FP32 draws cast to BF16."""
    g = torch.Generator().manual_seed(seed)
    wr = (wscale * torch.randn(experts, hidden, generator=g)).bfloat16()
    gu = (wscale * torch.randn(experts, 2 * inter, hidden, generator=g)).bfloat16()
    dn = (wscale * torch.randn(experts, hidden, inter, generator=g)).bfloat16()
    x = torch.randn(tokens, hidden, generator=g).bfloat16()
    return wr, gu, dn, x


def router_formula(x, wr, topk):
    # scripts/capture_qwen3_moe_layer0.py:583-586 applied to FP32 logits
    w = torch.softmax(x.float() @ wr.float().T, dim=1, dtype=torch.float32)
    w, ids = torch.topk(w, topk, dim=-1)
    return ids.to(torch.int32), (w / w.sum(dim=-1, keepdim=True)).float()


def main(ref_root):
    sys.path.insert(0, str(Path(ref_root) / "src"))
    from llm_gpu_kernels.reference import moe_reference
    from llm_gpu_kernels.benchmark import error
    from llm_gpu_kernels.moe_benchmark import validate_dispatch, make_ids
    from llm_gpu_kernels.moe_weight_quant import quantize_gate_up, dequantize_gate_up_reference
    from llm_gpu_kernels.moe_weight_layout import repack_gate_up, restore_v1_layout
    torch.set_num_threads(8)
    meta = {"torch": torch.__version__}

    # 1. mini case, everything stored: duplicate ids, signed weights, int64 ids
    g = torch.Generator().manual_seed(1234)
    x = torch.randn(9, 64, generator=g).bfloat16()
    gu = torch.randn(4, 64, 64, generator=g).bfloat16()
    dn = torch.randn(4, 64, 32, generator=g).bfloat16()
    ids = make_ids(9, 4, 2, "duplicate", g)
    ids[3] = torch.tensor([1, 1])
    rw = torch.rand(9, 2, generator=g) * 2 - 1
    torch.save({"x": x, "gate_up": gu, "down": dn, "ids": ids, "rw": rw,
                "out": moe_reference(x, gu, dn, ids, rw)}, HERE / "mini_fixed_route.pt")

    # 2. the reference's own three-token hand case (benchmark.py:152-157)
    g = torch.Generator().manual_seed(7)
    x = torch.randn(3, 8, generator=g).bfloat16()
    gu = torch.randn(3, 10, 8, generator=g).bfloat16()
    dn = torch.randn(3, 8, 5, generator=g).bfloat16()
    ids = torch.tensor([[0, 0], [2, 1], [1, 2]])
    rw = torch.tensor([[0.3, 0.7], [0.1, 0.9], [0.8, 0.2]])
    oracle = torch.zeros(3, 8)
    for token in range(3):
        for slot in range(2):
            e = int(ids[token, slot])
            a, b = (gu[e].float() @ x[token].float()).chunk(2)
            oracle[token] += rw[token, slot] * (dn[e].float() @ (torch.nn.functional.silu(a) * b))
    ref = moe_reference(x, gu, dn, ids, rw)
    assert error(ref, oracle)["passed"]
    torch.save({"x": x, "gate_up": gu, "down": dn, "ids": ids, "rw": rw, "out": ref,
                "per_route": oracle}, HERE / "three_token.pt")

    # 3. tiny layer, seed 0 (T=64,H=256,I=128,E=8,K=2): router formula + moe_reference
    wr, gu, dn, x = seeded_layer(0, 64, 256, 128, 8, 0.02)
    ids, rw = router_formula(x, wr, 2)
    out = moe_reference(x, gu, dn, ids, rw)
    torch.save({"ids": ids, "rw": rw, "out": out,
                "digests": {"router_weight": digest(wr), "gate_up": digest(gu), "down": digest(dn),
                            "x": digest(x)}}, HERE / "tiny_layer_seed0.pt")

    # 4. dispatch: the stable canonical order passes the reference validator
    from oracle.moe_oracle import dispatch_oracle, grouped_input_oracle
    g = torch.Generator().manual_seed(5)
    cases = []
    for (t, e, k, pattern) in ((33, 16, 4, "random"), (19, 3, 2, "duplicate"), (7, 8, 8, "all_hot"),
                               (193, 128, 8, "hot")):
        ids = make_ids(t, e, k, pattern, g)
        xs = torch.randn(t, 32, generator=g).bfloat16()
        counts, offsets, ranks, mapping = dispatch_oracle(ids, e)
        fake = SimpleNamespace(counts=counts, offsets=offsets, mapping=mapping,
                               grouped_input=grouped_input_oracle(xs, mapping, k))
        checks = validate_dispatch(fake, xs, ids)
        assert checks["passed"], checks
        cases.append({"ids": ids, "experts": e, "counts": counts, "offsets": offsets, "ranks": ranks,
                      "mapping": mapping})
    torch.save(cases, HERE / "dispatch_cases.pt")

    # 5. W4G128: reference quantiser on a seeded (128,1536,2048) weight -> digests + a slice
    g = torch.Generator().manual_seed(22)
    w = torch.empty(128, 1536, 2048, dtype=torch.bfloat16)
    for e in range(128):
        w[e] = (0.02 * torch.randn(1536, 2048, generator=g)).bfloat16()
    w[5, 17, 256:384] = 0  # an all-zero group: scale must be 1
    packed = quantize_gate_up(w)
    deq = dequantize_gate_up_reference(packed)
    rep = repack_gate_up(packed)
    back = restore_v1_layout(rep)
    assert torch.equal(back.words, packed.words) and torch.equal(back.scales, packed.scales)
    meta["w4"] = {"seed": 22, "source_sha256": digest(w), "words_sha256": digest(packed.words),
                  "scales_sha256": digest(packed.scales), "dequant_sha256": digest(deq),
                  "v2_words_sha256": digest(rep.words), "v2_scales_sha256": digest(rep.scales),
                  "format_error": packed.metadata["weight_format_error"]}
    torch.save({"words": packed.words[5, 16:20].clone(), "scales": packed.scales[5, 16:20].clone(),
                "source": w[5, 16:20].clone(), "dequant": deq[5, 16:20].clone()}, HERE / "w4_slice.pt")
    # 6. real-trace bundle: a 6-token trace written by the REFERENCE's writer (committed: manifest + trace
    #    tensors; the 1.8 GB weight bundle it references is the seeded layer, regenerated by the tests), and the
    #    reverse direction: a bundle written by this package's writer passes the reference's validator.
    import shutil
    import tempfile
    from llm_gpu_kernels import moe_real_trace as ref_trace
    from llm_gpu_kernels_b200 import moe_real_trace as our_trace
    g = torch.Generator().manual_seed(0)
    wr = (0.02 * torch.randn(128, 2048, generator=g)).bfloat16()
    gu = torch.empty(128, 1536, 2048, dtype=torch.bfloat16)
    dn = torch.empty(128, 2048, 768, dtype=torch.bfloat16)
    for e in range(128):
        gu[e] = (0.02 * torch.randn(1536, 2048, generator=g)).bfloat16()
    for e in range(128):
        dn[e] = (0.02 * torch.randn(2048, 768, generator=g)).bfloat16()
    x = torch.randn(6, 2048, generator=torch.Generator().manual_seed(31)).bfloat16()
    ids, rw = router_formula(x, wr, 8)
    rw = rw.bfloat16().float()      # the captured model's convention (capture script :587-588)
    out_dir = HERE / "ref_trace"
    shutil.rmtree(out_dir, ignore_errors=True)
    with tempfile.TemporaryDirectory() as tmp:
        tmp = Path(tmp)
        torch.save({"gate_up": gu, "down": dn}, tmp / "weights.pt")
        weight_sha = ref_trace.sha256_file(tmp / "weights.pt")
        ref = {name: {"path": "weights.pt", "tensor_name": name, "shape": list(t.shape), "dtype": "bfloat16",
                      "sha256": weight_sha, "source_manifest_sha256": "0" * 64}
               for name, t in (("gate_up", gu), ("down", dn))}
        ref_trace.write_real_moe_trace(tmp / "trace.json", "trace.pt", x=x, expert_ids=ids, route_weights=rw,
                                       provenance={"generator": "tests/golden/make_golden.py", "tokens": 6,
                                                   "weights": "seeded_layer(seed 0), N(0, 0.02)"}, weights=ref)
        ref_trace.validate_real_moe_trace(tmp / "trace.json")                 # the reference accepts its own bundle
        ours = our_trace.validate_real_moe_trace(tmp / "trace.json", load_weights=True)   # and so does this package
        assert torch.equal(ours.tensors["x"], x) and torch.equal(ours.weights["down"], dn)
        out_dir.mkdir()
        shutil.copy(tmp / "trace.json", out_dir / "trace.json")
        shutil.copy(tmp / "trace.pt", out_dir / "trace.pt")
        # the other direction
        manifest = our_trace.write_real_moe_trace(tmp / "ours", x, ids, rw, gu, dn, provenance={"writer": "b200"})
        accepted = ref_trace.validate_real_moe_trace(manifest, load_weights=True)
        assert torch.equal(accepted.tensors["expert_ids"], ids)
        meta["real_trace"] = {"weights_file_sha256": weight_sha, "gate_up_tensor_sha256": our_trace.tensor_sha256(gu),
                              "down_tensor_sha256": our_trace.tensor_sha256(dn),
                              "oracle_out_sha256": digest(moe_reference(x, gu, dn, ids, rw)),
                              "our_writer_accepted_by_reference_validator": True}
        torch.save({"out": moe_reference(x, gu, dn, ids, rw)}, out_dir / "reference_output.pt")
    (HERE / "golden_meta.json").write_text(json.dumps(meta, indent=1))
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    sys.path.insert(0, str(HERE.parents[1]))
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <path to a checkout of the reference project>")
    main(sys.argv[1])
