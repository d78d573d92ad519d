"""Record host-side behaviour of the reference's runtime libraries as JSON.

Needs ``oracle/_ref`` (built by ``oracle/build_ref.py`` from the reference's
own sources, against a driver stand-in that has no devices).  Stores:

* the exported ``ol*`` symbols of both libraries,
* ``olSuggestBlockSize`` results over a grid of global sizes,
* the error texts for malformed device descriptions.

Run: ``python tests/golden/make_abi_golden.py``
"""

import ctypes as C
import itertools
import json
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
REPO = HERE.parent.parent
sys.path.insert(0, str(REPO))

from oracle import build_ref  # noqa: E402

CB = C.CFUNCTYPE(None, C.c_void_p, C.c_int, C.c_char_p)


def exports(path):
    out = subprocess.run(["nm", "-D", "--defined-only", str(path)], capture_output=True, text=True,
                         check=True).stdout
    return sorted(line.split()[-1] for line in out.splitlines() if " T " in line)


def main():
    ref = build_ref.build()
    if ref is None:
        raise SystemExit("reference tree not available")
    backend = C.CDLL(str(ref / "libhc-cuda-runtime.so"))
    loader = C.CDLL(str(ref / "libhc-gpu-runtime-loader.so"))
    data = {"backend_exports": exports(ref / "libhc-cuda-runtime.so"),
            "loader_exports": exports(ref / "libhc-gpu-runtime-loader.so")}

    fn = backend.olSuggestBlockSize
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p, C.POINTER(C.c_size_t), C.POINTER(C.c_size_t), C.c_size_t]
    sizes = [0, 1, 2, 3, 7, 16, 27, 31, 32, 33, 64, 100, 128, 255, 256, 512, 513, 813, 1000,
             1023, 1024, 1025, 4096, 100000]
    table = []
    for nd in (1, 2, 3):
        for combo in itertools.product(sizes, repeat=nd):
            if nd == 3 and sum(1 for c in combo if c in (7, 27, 31, 33, 100, 255, 513, 1000, 1023)) > 1:
                continue  # keep the file small
            g = (C.c_size_t * 3)(*combo)
            b = (C.c_size_t * 3)(9, 9, 9)
            rc = fn(None, g, b, nd)
            table.append([list(combo), rc, list(b)[:nd]])
    for nd in (0, 4):
        g = (C.c_size_t * 4)(8, 8, 8, 8)
        b = (C.c_size_t * 4)(9, 9, 9, 9)
        table.append([[8] * nd, fn(None, g, b, nd), []])
    data["suggest_block_size"] = table

    def errors(lib, desc):
        seen = []
        cb = CB(lambda ctx, sev, text: seen.append([sev, text.decode()]))
        lib.olCreateDevice.restype = C.c_void_p
        lib.olCreateDevice.argtypes = [C.c_char_p, CB, C.c_void_p]
        handle = lib.olCreateDevice(desc.encode(), cb, None)
        return {"handle_is_null": not handle, "messages": seen}

    data["backend_errors"] = {d: errors(backend, d) for d in
                              ["cuda:x", "hip:0", "cuda", "", "cuda:", "cuda:0"]}
    data["loader_errors"] = {d: errors(loader, d) for d in ["nocolon", "foo:0", ""]}
    (HERE / "reference_abi.json").write_text(json.dumps(data, indent=0))
    print("wrote", HERE / "reference_abi.json", len(table), "block-size cases")
    print(json.dumps(data["backend_errors"], indent=1))
    print(json.dumps(data["loader_errors"], indent=1))


if __name__ == "__main__":
    main()
