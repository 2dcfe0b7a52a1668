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

NVFP4: the reference holds no golden payload bytes and pins payloads only against
TorchAO (not installed), so there is no NVFP4 payload fixture.  Its OUTER scale
is pure PyTorch, though: `_current_tensor_scale` / `_outer_tensor_scale`
(rtx/fp4.py:343-365) are exec'd from the file's text and evaluated on every
non-negative BF16 magnitude (zero, subnormals, infinity) and NaN, for both modes
-> nvfp4_outer_scale.npz.  The same sweep records where the integer exponent
rule of the reference's kernels (rtx/kernels/nvfp4_quant.py:117-143) differs
from the PyTorch `exp2(ceil(log2(t)))` form: on BF16 magnitudes (count stored in
nvfp4_outer_scale.json, expected 0) and on FP32 probes one ulp either side of
2688 * 2^e (listed there input by input).
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


def integer_power2_rule(amax: np.ndarray) -> np.ndarray:
    """The exponent-bump rule of rtx/kernels/nvfp4_quant.py:117-143 on FP32 amax values, with the
    quotient formed by division as rtx/fp4.py:361 does (bit patterns of the scale)."""
    with np.errstate(invalid="ignore", over="ignore"):
        t = np.maximum((amax / np.float32(2688.0)).astype(np.float32), np.float32(2.0 ** -126))
    b = t.view(np.uint32)
    e = b & np.uint32(0x7F800000)
    e = np.where((b & np.uint32(0x007FFFFF)) != 0, e + np.uint32(1 << 23), e).astype(np.uint32)
    return np.where(amax > 0, e, np.float32(1.0).view(np.uint32)).astype(np.uint32)


def nvfp4_outer_scale_fixture() -> None:
    fp4 = _exec_defs(os.path.join(REF, "rtx/fp4.py"), "def _current_tensor_scale", "def _delayed_amax_state")
    outer = fp4["_outer_tensor_scale"]

    def run(values: np.ndarray, mode: str) -> np.ndarray:
        out = np.empty(len(values), dtype=np.uint32)
        for i, v in enumerate(values):
            out[i] = outer(torch.from_numpy(np.array([[v]], dtype=np.float32)), mode).view(torch.int32).item() & 0xFFFFFFFF
        return out

    # every non-negative BF16 bit pattern up to +inf, then one NaN
    bf16_bits = np.concatenate([np.arange(0, 0x7F81, dtype=np.uint32), np.array([0x7FC0], dtype=np.uint32)])
    amax = (bf16_bits << 16).astype(np.uint32).view(np.float32)
    exact = run(amax, "exact")
    power2 = run(amax, "power2")
    finite = np.isfinite(amax)
    rule = integer_power2_rule(amax)
    bf16_disagree = [int(b) for b in bf16_bits[finite][rule[finite] != power2[finite]]]

    # FP32 probes that no BF16 tensor produces: one ulp either side of 2688 * 2^e (quotient next to a power of two)
    probes = []
    for e in range(-120, 110, 1):
        c = np.float32(2688.0 * 2.0 ** e) if -149 <= e + 11 <= 127 else None
        if c is None or not np.isfinite(c) or c == 0:
            continue
        probes += [np.nextafter(c, np.float32(0)), c, np.nextafter(c, np.float32(np.inf))]
    probes = np.array(probes, dtype=np.float32)
    probe_ref = run(probes, "power2")
    probe_rule = integer_power2_rule(probes)
    listed = [{"amax_bits": int(a.view(np.uint32)), "amax": float(a), "reference_scale_bits": int(r),
               "integer_rule_scale_bits": int(g)}
              for a, r, g in zip(probes, probe_ref, probe_rule) if r != g]
    np.savez_compressed(os.path.join(HERE, "nvfp4_outer_scale.npz"), bf16_bits=bf16_bits.astype(np.uint16),
                        exact_scale_bits=exact, power2_scale_bits=power2, fp32_probe_bits=probes.view(np.uint32),
                        fp32_probe_power2_scale_bits=probe_ref)
    with open(os.path.join(HERE, "nvfp4_outer_scale.json"), "w") as f:
        json.dump({"source": "rtx/fp4.py:343-365 exec'd on CPU (torch %s)" % torch.__version__,
                   "bf16_magnitudes": int(len(bf16_bits)),
                   "bf16_inputs_where_integer_rule_differs": bf16_disagree,
                   "fp32_probes": int(len(probes)),
                   "fp32_probes_where_integer_rule_differs": listed}, f, indent=1)
    print("nvfp4 outer scale:", len(bf16_bits), "BF16 magnitudes,", len(bf16_disagree), "disagree;",
          len(probes), "FP32 probes,", len(listed), "disagree")


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

    nvfp4_outer_scale_fixture()

    np.savez_compressed(os.path.join(HERE, "mxfp8_golden.npz"), **arrays)
    with open(os.path.join(HERE, "mxfp8_golden.json"), "w") as f:
        json.dump(manifest, f, indent=1, sort_keys=True)
    print("wrote", len(arrays), "arrays,", len(manifest), "manifest entries")


if __name__ == "__main__":
    main()
