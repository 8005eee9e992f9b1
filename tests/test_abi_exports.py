"""The C-ABI library loads and exports every function include/bdfp4.h declares (no GPU needed),
and its host-side argument checks refuse bad calls before anything is launched."""

import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def lib():
    import bdfp4

    if not bdfp4.LIB_PATH.exists():
        import importlib.util

        spec = importlib.util.spec_from_file_location("bdfp4_build", ROOT / "bitdecoding-fp4_b200" / "build.py")
        module = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(module)
        module.build_library()
    return bdfp4.library()


def declared_functions():
    header = (ROOT / "include" / "bdfp4.h").read_text()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    return sorted(set(re.findall(r"\b(bdfp4_[a-z0-9_]+)\s*\(", header)))


def test_every_declared_symbol_is_exported(lib):
    import bdfp4

    names = declared_functions()
    assert names, "no declarations found in include/bdfp4.h"
    assert set(names) == set(bdfp4.EXPORTS)
    for name in names:
        assert getattr(lib, name) is not None


def test_version_and_status_strings(lib):
    import bdfp4

    assert lib.bdfp4_version() >= 100
    assert lib.bdfp4_status_string(bdfp4.OK) == b"ok"
    assert b"contract" in lib.bdfp4_status_string(bdfp4.E_ARG)


def test_argument_errors_are_refused_on_the_host(lib):
    """Null structs and impossible geometries return BDFP4_E_ARG; nothing touches the GPU."""
    import bdfp4

    assert lib.bdfp4_kv_write(None, None) == bdfp4.E_ARG
    assert lib.bdfp4_quantize_query(None, None) == bdfp4.E_ARG
    assert lib.bdfp4_decode(None, None) == bdfp4.E_ARG
    assert lib.bdfp4_combine(None, None, 1, 1, 1, None, 128, None) == bdfp4.E_ARG
    args = bdfp4.DecodeArgs()
    args.rows, args.heads_q, args.heads_kv = 1, 7, 2  # heads_q not a multiple of heads_kv
    assert lib.bdfp4_decode(ctypes.byref(args), None) == bdfp4.E_ARG
    q = bdfp4.QuantizeQueryArgs()
    q.rows, q.heads_q, q.heads_kv, q.scale_mode = 1, 8, 2, 9  # unknown scale mode
    assert lib.bdfp4_quantize_query(ctypes.byref(q), None) == bdfp4.E_ARG
    with pytest.raises(bdfp4.KernelError):
        bdfp4.check("bdfp4_decode", bdfp4.E_ARG)


def test_struct_sizes_match_the_header(lib):
    """ctypes mirrors of the argument structs have the sizes the C compiler gives them."""
    import subprocess
    import tempfile

    import bdfp4

    source = '#include <stdio.h>\n#include "bdfp4.h"\nint main(void){printf("%zu %zu %zu %zu %zu\\n", ' \
             "sizeof(bdfp4_kv_write_args), sizeof(bdfp4_quantize_query_args), sizeof(bdfp4_decode_args), " \
             "sizeof(bdfp4_mla_decode_args), sizeof(bdfp4_exchange_args));return 0;}\n"
    with tempfile.TemporaryDirectory() as tmp:
        src = Path(tmp) / "sizes.c"
        src.write_text(source)
        exe = Path(tmp) / "sizes"
        subprocess.run(["gcc", "-I", str(ROOT / "include"), str(src), "-o", str(exe)], check=True)
        sizes = [int(x) for x in subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout.split()]
    assert sizes == [ctypes.sizeof(bdfp4.KvWriteArgs), ctypes.sizeof(bdfp4.QuantizeQueryArgs),
                     ctypes.sizeof(bdfp4.DecodeArgs), ctypes.sizeof(bdfp4.MlaDecodeArgs),
                     ctypes.sizeof(bdfp4.ExchangeArgs)]


def test_exchange_region_size_and_argument_checks(lib):
    """The exchange region holds two sets of one 132-float record and one flag word per (source rank,
    row, head); a world outside 1..8, a step of zero and missing pointers are refused on the host."""
    import bdfp4

    assert bdfp4.exchange_bytes(4, 1, 32) == 2 * 4 * 32 * (132 * 4 + 4)
    assert lib.bdfp4_exchange_bytes(9, 1, 32) == 0 and lib.bdfp4_exchange_bytes(0, 1, 32) == 0
    with pytest.raises(ValueError):
        bdfp4.exchange_bytes(9, 1, 32)
    assert lib.bdfp4_exchange_merge(None, None) == bdfp4.E_ARG
    a = bdfp4.ExchangeArgs()
    a.rows, a.heads_q, a.world, a.rank, a.parts, a.step = 1, 8, 2, 0, 1, 1
    assert lib.bdfp4_exchange_merge(ctypes.byref(a), None) == bdfp4.E_ARG  # no partials, no regions, no output
    assert lib.bdfp4_peer_alloc(0, None, None) == bdfp4.E_ARG
    assert lib.bdfp4_peer_open(None, None) == bdfp4.E_ARG
