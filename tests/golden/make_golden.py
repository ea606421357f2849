"""Generate ``reference_vectors.pt`` by EXECUTING the reference's own Python definitions on the CPU.

Run in a checkout that has the reference mounted:

    python tests/golden/make_golden.py /path/to/prime-flash-moe

The reference modules cannot be imported as they are (``test/test.py`` runs a CUDA sweep at import
time, ``test/test_mxfp8.py`` and ``prime_moe/__init__.py`` import the compiled extension), so the
function definitions are lifted out of the source files with ``ast`` and executed unchanged in a
namespace that provides ``torch``. Nothing from the reference is copied into this repository: only
the inputs fed to those functions and the outputs they returned are stored.

Functions executed (path inside the reference : name):
  test/test.py                : moe_naive_from_topk, moe_align_block_size_simple
  test/test_mxfp8.py          : _shared_exponent, quantize_mx, dequantize_mx, moe_naive_from_topk
  prime_moe/__init__.py       : pack_scales_blocked
"""
from __future__ import annotations

import ast
import os
import sys
from pathlib import Path

import torch


def lift(path: Path, names, extra_globals=None):
    tree = ast.parse(path.read_text())
    ns = {"torch": torch}
    ns.update(extra_globals or {})
    wanted = set(names)
    for node in tree.body:
        if isinstance(node, ast.FunctionDef) and node.name in wanted:
            node.decorator_list = []
            exec(compile(ast.Module([node], []), str(path), "exec"), ns)
        elif isinstance(node, ast.Assign) and all(isinstance(t, ast.Name) for t in node.targets):
            if {t.id for t in node.targets} & {"BLOCK", "E4M3_MAX", "E4M3_EMAX"}:
                exec(compile(ast.Module([node], []), str(path), "exec"), ns)
    missing = wanted - set(ns)
    assert not missing, f"{path}: {missing} not found"
    return ns


def main(ref_root: str) -> None:
    ref = Path(ref_root)
    t1 = lift(ref / "test" / "test.py", ["moe_naive_from_topk", "moe_align_block_size_simple"])
    init = lift(ref / "prime_moe" / "__init__.py", ["pack_scales_blocked"])
    t2 = lift(ref / "test" / "test_mxfp8.py",
              ["_shared_exponent", "quantize_mx", "dequantize_mx", "moe_naive_from_topk"],
              {"BLOCK": init["BLOCK"]})
    g = torch.Generator().manual_seed(20261125)
    out = {"about": "outputs of the reference's Python definitions executed on CPU; see make_golden.py",
           "torch": torch.__version__}

    # ---- routing tables (test/test.py:81-120) ----
    align = []
    for (T, E, k) in [(1, 8, 2), (8, 8, 4), (33, 5, 3), (256, 8, 4), (200, 37, 9), (130, 257, 9)]:
        ids = torch.stack([torch.randperm(E, generator=g)[:k] if k <= E else torch.randint(0, E, (k,), generator=g)
                           for _ in range(T)]).to(torch.int32)
        if E == 37:  # the reference's sweeps force the last expert and allow duplicates (test/test.py:155-156)
            ids = torch.randint(0, E - 1, (T, k), generator=g, dtype=torch.int32)
            ids[:, -1] = E - 1
        s, e, n = t1["moe_align_block_size_simple"](ids, 128, E)
        align.append({"topk_ids": ids, "num_experts": E, "block_m": 128, "sorted_token_ids": s, "expert_ids": e,
                      "num_tokens_post_padded": n})
    out["align"] = align

    # ---- MX quantiser (test/test_mxfp8.py:21-47) ----
    quant = []
    base = torch.randn(24, 128, generator=g)
    cases = {
        "normal": base,
        "small": base * 1e-3,
        "large": base * 3e4,
        "tiny": base * 1e-38,
        "mixed_blocks": base * torch.logspace(-6, 6, 24).unsqueeze(1),
        "with_zero_block": torch.cat([torch.zeros(2, 128), base[:2]]),
        "exact_pow2": torch.full((2, 64), 256.0),
        "near_e4m3_max": torch.tensor([[447.9, 448.0, 449.0, 463.9, 464.0, 480.0, 511.9, 512.0] * 4]),
        "bf16_input": base.to(torch.bfloat16),
    }
    for name, t in cases.items():
        q, s = t2["quantize_mx"](t)
        quant.append({"name": name, "input": t, "q": q.view(torch.uint8), "scales": s.view(torch.uint8),
                      "dequant": t2["dequantize_mx"](q, s)})
    out["quant"] = quant

    # ---- blocked scale layout (prime_moe/__init__.py:106-115) ----
    packs = []
    for shape in [(128, 4), (256, 8), (2, 128, 16), (3, 384, 4)]:
        u = torch.randint(0, 255, shape, generator=g, dtype=torch.uint8)
        packs.append({"scales": u, "packed": init["pack_scales_blocked"](u.view(torch.float8_e8m0fnu)).view(torch.uint8)})
    out["pack"] = packs

    # ---- MoE reference, bf16 (test/test.py:13-48), inputs as in test/test.py:149-157 ----
    moe = []
    for (T, K, E, N, k) in [(16, 128, 3, 256, 2), (40, 256, 5, 256, 3)]:
        x = (torch.randn(T, K, generator=g) * 0.05).to(torch.bfloat16)
        w1 = (torch.randn(E, N, K, generator=g) * 0.05).to(torch.bfloat16)
        w2 = (torch.randn(E, K, N // 2, generator=g) * 0.05).to(torch.bfloat16)
        ids = torch.randint(0, E - 1, (T, k), generator=g, dtype=torch.int32)
        ids[:, -1] = E - 1
        wts = torch.softmax(torch.randn(T, k, generator=g), dim=-1)
        moe.append({"x": x, "w1": w1, "w2": w2, "topk_ids": ids, "topk_weights": wts,
                    "out": t1["moe_naive_from_topk"](x, w1, w2, ids, wts)})
    out["moe_bf16"] = moe

    # ---- MoE reference, mxfp8 (test/test_mxfp8.py:50-77) on dequantised inputs ----
    moe8 = []
    for (T, K, E, N, k) in [(16, 256, 3, 256, 2)]:
        x = (torch.randn(T, K, generator=g) * 0.05).to(torch.bfloat16)
        w1 = (torch.randn(E, N, K, generator=g) * 0.05).to(torch.bfloat16)
        w2 = (torch.randn(E, K, N // 2, generator=g) * 0.05).to(torch.bfloat16)
        xq, xs = t2["quantize_mx"](x)
        w1q, w1s = t2["quantize_mx"](w1)
        w2q, w2s = t2["quantize_mx"](w2)
        ids = torch.randint(0, E - 1, (T, k), generator=g, dtype=torch.int32)
        ids[:, -1] = E - 1
        wts = torch.softmax(torch.randn(T, k, generator=g), dim=-1)
        ref = t2["moe_naive_from_topk"](t2["dequantize_mx"](xq, xs).to(torch.bfloat16),
                                        t2["dequantize_mx"](w1q, w1s).to(torch.bfloat16),
                                        t2["dequantize_mx"](w2q, w2s).to(torch.bfloat16), ids, wts)
        moe8.append({"x_q": xq.view(torch.uint8), "x_scales": xs.view(torch.uint8), "w1_q": w1q.view(torch.uint8),
                     "w1_scales": w1s.view(torch.uint8), "w2_q": w2q.view(torch.uint8),
                     "w2_scales": w2s.view(torch.uint8), "topk_ids": ids, "topk_weights": wts, "out": ref})
    out["moe_mxfp8"] = moe8

    dst = Path(__file__).resolve().parent / "reference_vectors.pt"
    torch.save(out, dst)
    print(f"wrote {dst} ({dst.stat().st_size / 1024:.0f} KiB)")


if __name__ == "__main__":
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("PMOE_REFERENCE_ROOT")
    if not root:
        sys.exit("usage: python tests/golden/make_golden.py /path/to/prime-flash-moe   (or set PMOE_REFERENCE_ROOT)")
    main(root)
