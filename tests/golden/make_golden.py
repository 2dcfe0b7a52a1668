"""Generate the golden fixtures of tests/golden/ by EXECUTING the reference.

Run where the reference checkout (read-only) is available and name it in
$RTX_REFERENCE:

    RTX_REFERENCE=<reference checkout> python tests/golden/make_golden.py

What it executes (nothing is copied into this repository):
  * rtx.autotune.legacy._torch_mxfp8_reference (rtx/autotune/legacy.py:783-806),
    imported from the reference package;
  * the reference tests' own restatements `_reference_to_mx` / `_reference_linear`
    (tests/test_mxfp8_fwd.py:12-47) and `_reference` (tests/test_mxfp8_quant.py:25-46),
    exec'd from the test files' text because importing those modules needs an SM120 GPU stack.

Outputs: mxfp8_golden.npz (small arrays: inputs as BF16 bit patterns, payload
codes, scale codes, BF16 output bits) and mxfp8_golden.json (SHA-256 digests of
larger cases whose inputs are regenerated from the recorded seeds).

The reference holds no NVFP4 golden bytes and pins NVFP4 only against TorchAO
(not installed), so there is no NVFP4 fixture.
"""
from __future__ import annotations

import hashlib
import json
import os
import sys

import numpy as np
import torch

REF = os.environ.get("RTX_REFERENCE")
if not REF or not os.path.isdir(REF):
    raise SystemExit("set RTX_REFERENCE to the reference checkout")
HERE = os.path.dirname(os.path.abspath(__file__))


def _exec_defs(path: str, start: str, stop: str) -> dict:
    src = open(path).read()
    ns = {"torch": torch}
    exec("from __future__ import annotations\n" + src[src.index(start):src.index(stop)], ns)
    return ns


def bits(t: torch.Tensor) -> np.ndarray:
    if t.dtype == torch.bfloat16:
        return t.contiguous().view(torch.int16).numpy().view(np.uint16)
    return t.contiguous().view(torch.uint8).numpy()


def digest(t: torch.Tensor) -> str:
    return hashlib.sha256(bits(t).tobytes()).hexdigest()


def main() -> None:
    sys.path.insert(0, REF)
    from rtx.autotune.legacy import _torch_mxfp8_reference

    fwd = _exec_defs(os.path.join(REF, "tests/test_mxfp8_fwd.py"), "def _reference_to_mx", "class MXFP8ConfigTests")
    qnt = _exec_defs(os.path.join(REF, "tests/test_mxfp8_quant.py"), "def _reference(", "class MXFP8QuantConfigTests")
    to_mx, ref_linear, ref_quant = fwd["_reference_to_mx"], fwd["_reference_linear"], qnt["_reference"]

    arrays: dict[str, np.ndarray] = {}
    manifest: dict[str, dict] = {}

    # known answer: tests/test_mxfp8_quant.py:186-220
    src = torch.zeros(1, 32)
    src[0, 0] = 480
    for rounding in ("floor", "infinity"):
        q, s = ref_quant(src.bfloat16(), scale_rounding=rounding)
        arrays[f"ka480_{rounding}_q"] = bits(q)
        arrays[f"ka480_{rounding}_s"] = bits(s)

    # quantizer cases: seed 1701 128x256 (tests/test_mxfp8_quant.py:151-184), ragged extras
    for name, seed, shape in [("q1701", 1701, (128, 256)), ("q1703", 1703, (64, 256)), ("qrag", 7, (9, 127)),
                              ("qtiny", 8, (3, 1)), ("q33", 9, (5, 33))]:
        torch.manual_seed(seed)
        x = torch.randn(*shape).bfloat16()
        for rounding in ("infinity", "floor"):
            q, s = to_mx(x, scale_rounding=rounding)
            arrays[f"{name}_{rounding}_q"] = bits(q)
            arrays[f"{name}_{rounding}_s"] = bits(s)
        arrays[f"{name}_x"] = bits(x)
        manifest[name] = {"seed": seed, "shape": list(shape), "draw": "torch.manual_seed(seed); randn(shape).bfloat16()"}

    # special values: zeros, NaN, inf, tiny, huge
    x = torch.zeros(8, 64)
    x[1, 3] = float("nan")
    x[2, 40] = float("inf")
    x[3, :] = 1e-30
    x[4, :] = 3e38
    x[5, 0] = -448.0
    x[6, 33] = 2.0 ** -20
    x[7, :32] = torch.linspace(-500, 500, 32)
    x = x.bfloat16()
    for rounding in ("infinity", "floor"):
        q, s = to_mx(x, scale_rounding=rounding)
        arrays[f"special_{rounding}_q"] = bits(q)
        arrays[f"special_{rounding}_s"] = bits(s)
    arrays["special_x"] = bits(x)

    # forward outputs: tests/test_mxfp8_fwd.py:359-380 (seed 123, x = randn*0.5)
    for (m, n, k) in [(128, 128, 128), (37, 70, 128), (5, 129, 256), (3, 5, 1), (7, 11, 17), (9, 131, 127)]:
        torch.manual_seed(123)
        x = (torch.randn(m, k) * 0.5).bfloat16()
        w = (torch.randn(n, k) * 0.5).bfloat16()
        y = ref_linear(x, w)
        key = f"fwd_{m}_{n}_{k}"
        arrays[key + "_y"] = bits(y)
        manifest[key] = {"seed": 123, "m": m, "n": n, "k": k,
                         "draw": "torch.manual_seed(123); x=(randn(m,k)*0.5).bfloat16(); w=(randn(n,k)*0.5).bfloat16()"}

    # 257x385x256 seed 321 (tests/test_mxfp8_fwd.py:394-478): digest only
    torch.manual_seed(321)
    x = (torch.randn(257, 256) * 0.5).bfloat16()
    w = (torch.randn(385, 256) * 0.5).bfloat16()
    manifest["fwd_257_385_256"] = {"seed": 321, "m": 257, "n": 385, "k": 256, "sha256_y": digest(ref_linear(x, w)),
                                   "draw": "torch.manual_seed(321); x=(randn(257,256)*0.5).bfloat16(); w=(randn(385,256)*0.5).bfloat16()"}

    # benchmark configuration 1 through the reference's own legacy function: digest + corner
    gen = torch.Generator().manual_seed(0)
    x = torch.randn(256, 1024, generator=gen).bfloat16()
    w = (torch.randn(1024, 1024, generator=gen) / 32.0).bfloat16()
    y = _torch_mxfp8_reference(x, w)
    manifest["config1"] = {"seed": 0, "m": 256, "n": 1024, "k": 1024, "sha256_y": digest(y),
                           "draw": "g=Generator().manual_seed(0); x=randn(256,1024,generator=g).bfloat16(); w=(randn(1024,1024,generator=g)/32).bfloat16()"}
    arrays["config1_y_corner"] = bits(y[:16, :16].contiguous())

    np.savez_compressed(os.path.join(HERE, "mxfp8_golden.npz"), **arrays)
    with open(os.path.join(HERE, "mxfp8_golden.json"), "w") as f:
        json.dump(manifest, f, indent=1, sort_keys=True)
    print("wrote", len(arrays), "arrays,", len(manifest), "manifest entries")


if __name__ == "__main__":
    main()
