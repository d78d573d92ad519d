"""Run-time specialisation, the part that needs no GPU: hcSpecialiseCompile
turns a program for the accumulator machine into an sm_100a image with NVRTC
(the kernel templates are embedded in the library as text), gives the same image
for the same program, keeps images in the directory of HC_B200_KERNEL_CACHE, and
refuses what the straight-line kernels do not cover (row programs on integers
or with the later operators)."""

import os
import subprocess
import sys

import pytest

from hc_b200 import capi
from hc_b200.hckernel import elementwise as ew


def _program(code, nin):
    p = capi.HcMapProgram()
    p.nInputs, p.nInstr = nin, len(code)
    for i, word in enumerate(code):
        p.code[i] = word
    return p


# max(in0 * c0, in1) + c1, then exp: not one of the bodies compiled ahead of time.
MAP_CODE = [ew.LOAD | (1 << 8), ew.MUL | (9 << 8), ew.ADD | (0 << 8), ew.MAX | (8 << 8), ew.EXP]
# log-softmax's words with a square root at the end.
ROW_CODE = [0x0, 0x12, 0x0, 0x1402, 0xb, 0x111, 0x1580, 0x90, 0x293, 0x0, 0x1402, 0x1602, ew.SQRT]


@pytest.mark.parametrize("dtype", [capi.HC_F32, capi.HC_F64])
@pytest.mark.parametrize("row,code,nin", [(False, MAP_CODE, 2), (True, ROW_CODE, 1),
                                          (False, [ew.LOAD | (16 << 8), ew.ADD | (17 << 8)], 0),
                                          (False, [ew.LOAD, ew.ADD | (1 << 8), ew.ADD | (2 << 8),
                                                   ew.MUL | (3 << 8)], 4)])
def test_programs_compile_to_device_images(row, code, nin, dtype):
    image, tag = capi.specialise_compile(_program(code, nin), row_program=row, dtype=dtype)
    assert image[:4] == b"\x7fELF" and len(image) > 4096
    assert tag.startswith("j") and len(tag) == 17
    kind = "row" if row else "map"
    suffix = "f64_v1" if dtype == capi.HC_F64 else "f32_v1"
    assert f"hc_{kind}_fused_{tag}_{suffix}".encode() in image  # the kernel's name in the image
    other = "f32_v1" if dtype == capi.HC_F64 else "f64_v1"
    assert f"hc_{kind}_fused_{tag}_{other}".encode() not in image  # one element type per image
    again, tag2 = capi.specialise_compile(_program(code, nin), row_program=row, dtype=dtype)
    assert tag2 == tag and len(again) == len(image)


def test_constants_are_not_part_of_the_key():
    a, b = _program(MAP_CODE, 2), _program(MAP_CODE, 2)
    a.consts[0], b.consts[0] = 2.0, -3.5
    assert capi.specialise_compile(a)[1] == capi.specialise_compile(b)[1]
    c = _program(MAP_CODE[:-1] + [ew.LOG], 2)
    assert capi.specialise_compile(c)[1] != capi.specialise_compile(a)[1]


def test_the_later_operators_and_integer_tiles():
    """Element-wise programs compile with the whole operator table and on integer
    tiles; row programs take the operations up to `set` on floats only."""
    later = [ew.LOAD, ew.FLOORDIV | (1 << 8), ew.SAVE0, ew.LOAD, ew.LT | (1 << 8),
             ew.ADD | (4 << 8)]
    image, tag = capi.specialise_compile(_program(later, 2))
    assert f"hc_map_fused_{tag}_f32_v4".encode() in image
    for dtype, name in ((capi.HC_I32, "i32_v4"), (capi.HC_I64, "i64_v2")):
        ints = [ew.LOAD, ew.SHL | (8 << 8), ew.XOR | (1 << 8), ew.MOD | (9 << 8), ew.INV]
        image, tag = capi.specialise_compile(_program(ints, 2), dtype=dtype)
        assert f"hc_map_fused_{tag}_{name}".encode() in image
    with pytest.raises(RuntimeError, match="row programs of the operations up to `set`"):
        capi.specialise_compile(_program([ew.LOAD, ew.FLOORDIV | (8 << 8)], 1), row_program=True)
    with pytest.raises(RuntimeError, match="row programs of the operations up to `set`"):
        capi.specialise_compile(_program(ROW_CODE, 1), row_program=True, dtype=capi.HC_I32)
    with pytest.raises(RuntimeError, match="element-wise programs on float32"):
        capi.specialise_compile(_program(MAP_CODE, 2), dtype=capi.HC_BF16)


def test_images_are_kept_in_the_cache_directory(tmp_path):
    """In a process of its own: the directory is read from the environment."""
    script = (
        "import time\n"
        "from hc_b200 import capi\n"
        "p = capi.HcMapProgram(); code = %r\n"
        "p.nInputs, p.nInstr = 2, len(code)\n"
        "for i, w in enumerate(code): p.code[i] = w\n"
        "first = capi.specialise_compile(p)\n"
        "t = time.perf_counter(); second = capi.specialise_compile(p); dt = time.perf_counter() - t\n"
        "assert first == second\n"
        "print(len(first[0]), dt)\n" % (MAP_CODE,)
    )
    env = dict(os.environ, HC_B200_KERNEL_CACHE=str(tmp_path))
    env["PYTHONPATH"] = os.pathsep.join([os.path.dirname(os.path.dirname(__file__)),
                                         env.get("PYTHONPATH", "")])
    out = subprocess.run([sys.executable, "-c", script], env=env, capture_output=True, text=True,
                         timeout=300)
    assert out.returncode == 0, out.stderr
    size, seconds = out.stdout.split()
    files = list(tmp_path.glob("hc-map-*.cubin"))
    assert len(files) == 1 and files[0].stat().st_size == int(size)
    assert float(seconds) < 0.05  # read back, not compiled again
