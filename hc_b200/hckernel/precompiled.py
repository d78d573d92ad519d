"""Bodies that are compiled ahead of time into straight-line kernels.

The reference compiles every kernel body when it is first called
(python/hckernel/dispatcher.py:81-137 hands the source to the MLIR pipeline).
Here nothing is compiled at run time: an element-wise or row body is recorded,
translated into a program for the accumulator machine (``elementwise.py``) and
interpreted by ``csrc/kernels/map_elements.cu`` / ``row_program.cu``.  The
interpreter spends several instructions on decoding and operand selection for
every arithmetic one, which is what bounds it on long bodies.

This module is the ahead-of-time half: the bodies listed below - the row and
element-wise bodies that recur (centring, normalising, softmax and its
relatives (the plain softmax body has a kernel of its own, ``softmax_rows.cu``),
scale-and-shift, rectifiers, distances, a Horner polynomial) - are
translated here, at build time, and written to
``csrc/kernels/fused_programs.h`` as constant programs.  ``row_fused.cu`` and
``map_fused.cu`` instantiate one kernel per program in which every operation
and operand is known to the compiler, so the program becomes straight-line
code with the same operations in the same order (no contraction into fused
multiply-adds), bit for bit the interpreter's results.  At run time
``hcRowProgram`` / ``hcMapElements`` compare the program they are given with
the table and launch the precompiled kernel on a match; any other body runs
on the interpreter as before.  Constants are operands, not part of the match:
``a * 2.0 - b`` and ``a * 0.5 - b`` are the same program.

    python -m hc_b200.hckernel.precompiled            # rewrite the header
    python -m hc_b200.hckernel.precompiled --check    # exit 1 if it is stale

Adding a body to the lists below and rebuilding is all it takes to precompile
another one.
"""

from __future__ import annotations

import sys
from pathlib import Path

import numpy as np

HEADER = Path(__file__).resolve().parent.parent / "csrc" / "kernels" / "fused_programs.h"


# ---- row bodies: fn(tiles of whole rows) -> rows ---------------------------------------
def centre(t):
    return t - t.mean(axis=1, keepdims=True)


def l2_normalise(t):
    return t / np.sqrt((t * t).sum(axis=1, keepdims=True))


def log_softmax(t):
    shifted = t - t.max(axis=1, keepdims=True)
    return shifted - np.log(np.exp(shifted).sum(axis=1, keepdims=True))


def softmax_temperature(t):
    e = np.exp((t - t.max(axis=1, keepdims=True)) * 0.5)
    return e / e.sum(axis=1, keepdims=True)


def scaled_difference(a, b):
    return (a - b) / np.maximum(np.abs(a).max(axis=1, keepdims=True), 1.0)


def standardise(t):
    d = t - t.mean(axis=1, keepdims=True)
    return d / np.sqrt((d * d).mean(axis=1, keepdims=True) + 1e-5)


def rms_normalise(t):
    return t / np.sqrt((t * t).mean(axis=1, keepdims=True) + 1e-6)


def max_normalise(t):
    return t / np.abs(t).max(axis=1, keepdims=True)


def sum_normalise(t):
    return t / t.sum(axis=1, keepdims=True)


ROW_BODIES = [
    ("centre", centre, 1),
    ("l2_normalise", l2_normalise, 1),
    ("log_softmax", log_softmax, 1),
    ("softmax_temperature", softmax_temperature, 1),
    ("scaled_difference", scaled_difference, 2),
    ("standardise", standardise, 1),
    ("rms_normalise", rms_normalise, 1),
    ("max_normalise", max_normalise, 1),
    ("sum_normalise", sum_normalise, 1),
]

# ---- element-wise bodies: fn(tiles) -> tile ----------------------------------------------
MAP_BODIES = [
    ("relu_axpby", lambda a, b: np.maximum(a * 2.0 - b, 0.0), 2),
    ("axpby", lambda a, b: a * 2.0 + b * 3.0, 2),
    ("axpy", lambda a, b: a * 2.0 + b, 2),
    ("scale_shift", lambda a: a * 2.0 + 1.0, 1),
    ("scale", lambda a: a * 2.0, 1),
    ("relu", lambda a: np.maximum(a, 0.0), 1),
    ("clamp", lambda a: np.minimum(np.maximum(a, 0.0), 1.0), 1),
    ("square_plus", lambda a: a * a + 1.0, 1),
    ("gauss", lambda a: np.exp(-(a * a)), 1),
    ("poly4", lambda a: (((a * 0.5 + 1.0) * a + 2.0) * a - 3.0) * a + 0.25, 1),
    ("add", lambda a, b: a + b, 2),
    ("sub", lambda a, b: a - b, 2),
    ("mul", lambda a, b: a * b, 2),
    ("div", lambda a, b: a / b, 2),
    ("abs_difference", lambda a, b: np.abs(a - b), 2),
    ("squared_difference", lambda a, b: (a - b) * (a - b), 2),
    ("hypot", lambda a, b: np.sqrt(a * a + b * b), 2),
    ("mixed", lambda a, b: (a + b) / (np.sqrt(np.abs(a)) + 1.5) - np.minimum(a, b) * (-b), 2),
    ("three_inputs", lambda a, b, c: (a - b) * (b - c) / (c * c + 1.0), 3),
    ("multiply_add", lambda a, b, c: a * b + c, 3),
]


class _Array:
    def __init__(self, shape, dtype="float32"):
        self.shape, self.dtype = tuple(shape), dtype


def translate():
    """``(row programs, map programs)``: lists of ``(name, inputs, code)`` with the
    instruction words the front door produces for each body.  The words do not
    depend on the shape or on the element type (float32 and float64 are checked
    to agree)."""
    from ..workloads import make_elementwise, make_rowwise

    rows, maps = [], []
    for name, fn, count in ROW_BODIES:
        codes = []
        for dtype in ("float32", "float64"):
            arrays = tuple(_Array((64, 256), dtype) for _ in range(count + 1))
            plan = make_rowwise(fn, count).plan_for(arrays + (8,))
            if plan.family != "row_program":
                raise RuntimeError(f"{name}: recorded as {plan.family}, not as a row program")
            codes.append(tuple(int(c) for c in plan.roles["code"]))
        if codes[0] != codes[1]:
            raise RuntimeError(f"{name}: float32 and float64 programs differ")
        rows.append((name, count, codes[0]))
    for name, fn, count in MAP_BODIES:
        codes = []
        for dtype in ("float32", "float64"):
            arrays = tuple(_Array((64, 256), dtype) for _ in range(count + 1))
            plan = make_elementwise(fn, count, 2, (4, 64)).plan_for(arrays)
            if plan.family != "map_elements":
                raise RuntimeError(f"{name}: recorded as {plan.family}, not as an element-wise body")
            codes.append(tuple(int(c) for c in plan.roles["code"]))
        if codes[0] != codes[1]:
            raise RuntimeError(f"{name}: float32 and float64 programs differ")
        maps.append((name, count, codes[0]))
    for group in (rows, maps):
        seen = {}
        for name, count, code in group:
            if (count, code) in seen:
                raise RuntimeError(f"{name} and {seen[(count, code)]} are the same program")
            seen[(count, code)] = name
    return rows, maps


def render() -> str:
    rows, maps = translate()
    out = [
        "// Programs compiled ahead of time into straight-line kernels (row_fused.cu,",
        "// map_fused.cu) and matched at run time by hcRowProgram / hcMapElements.",
        "// Written by `python -m hc_b200.hckernel.precompiled` from the bodies listed in",
        "// hc_b200/hckernel/precompiled.py: edit that list, not this file.",
        "#pragma once",
        "",
        "#include <stdint.h>",
        "",
        "namespace hcfused {",
    ]
    for kind, group in (("row", rows), ("map", maps)):
        for name, count, code in group:
            words = ", ".join(f"0x{c:x}u" for c in code)
            out += [
                f"struct {kind}_{name} {{",
                f"  static constexpr int nin = {count}, n = {len(code)};",
                f"  static constexpr uint32_t code[{len(code)}] = {{{words}}};",
                "};",
            ]
    out += ["} // namespace hcfused", ""]
    for kind, group in (("ROW", rows), ("MAP", maps)):
        out.append(f"#define HC_FUSED_{kind}_LIST(X) \\")
        out += [f"  X({name}) \\" for name, _, _ in group[:-1]]
        out.append(f"  X({group[-1][0]})")
        out.append("")
    return "\n".join(out)


def main(argv):
    text = render()
    if "--check" in argv:
        if not HEADER.exists() or HEADER.read_text() != text:
            print(f"{HEADER} is stale: run `python -m hc_b200.hckernel.precompiled`")
            return 1
        return 0
    HEADER.write_text(text)
    print(f"wrote {HEADER}")
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))
