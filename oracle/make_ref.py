"""Recipe for ``oracle/_ref``: the reference's own CPU model of the path, made importable.

    python oracle/make_ref.py [--reference <checkout of OpenBitSys/BitDecoding-FP4>]

TEST INFRASTRUCTURE. OpenBitSys/BitDecoding-FP4 is pure Python; the CPU model of its quantizers and
of its decode-order attention is ``src/nvfp4_decode_kernel/reference.py`` with its two small
dependencies ``p_scale.py`` and ``scale_mode.py`` (torch only). This script places those three files,
unmodified, under ``oracle/_ref/nvfp4_decode_kernel_ref/`` (listed in ``.gitignore``: they are never
committed) so that ``bench.py --impl reference`` and its ``cpu_baseline`` leg can time the reference
itself where the reference tree is not mounted. Nothing in the product imports it.
"""

from __future__ import annotations

import argparse
import shutil
from pathlib import Path

FILES = ("reference.py", "p_scale.py", "scale_mode.py")
TARGET = Path(__file__).resolve().parent / "_ref" / "nvfp4_decode_kernel_ref"


def make(reference_root: str = "/root/reference") -> Path | None:
    """Returns the package directory, or None when the reference tree is not there."""
    source = Path(reference_root) / "src" / "nvfp4_decode_kernel"
    if not all((source / name).exists() for name in FILES):
        return None
    TARGET.mkdir(parents=True, exist_ok=True)
    for name in FILES:
        shutil.copyfile(source / name, TARGET / name)
    (TARGET / "__init__.py").write_text("")
    return TARGET


if __name__ == "__main__":
    parser = argparse.ArgumentParser()
    parser.add_argument("--reference", default="/root/reference")
    made = make(parser.parse_args().reference)
    print(made if made else "reference tree not found; oracle/_ref not made")
