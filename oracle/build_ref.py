"""Place the reference project's own host implementation of the path under ``oracle/_ref/``.

TEST / BENCHMARK INFRASTRUCTURE, NOT PRODUCT. The reference is pure Python; the one file that holds its
CPU path for this hot path, ``gdn2/reference.py`` (``recurrent_gdn2``, ``chunk_gdn2_torch``), depends on
torch alone. This recipe copies that file, unmodified, from a checkout of the reference into
``oracle/_ref/gdn2_reference.py`` and writes its SHA-256 beside it. ``oracle/_ref/`` is a build output: it
is git-ignored (no reference source enters this repository's history) and travels with the built kernel
library to the machine that runs the benchmark, where no checkout of the reference exists.

Used by ``bench.py`` (``--impl reference`` and the ``cpu_baseline`` leg, ``kind: "reference"``) and by
``tests/test_oracle.py`` to cross-check the oracle restatement against the reference itself.

    python oracle/build_ref.py [--reference /path/to/GDT2_TileLang]
"""

from __future__ import annotations

import argparse
import hashlib
import pathlib
import shutil

HERE = pathlib.Path(__file__).resolve().parent
OUT = HERE / "_ref"
DEFAULT_REFERENCE = pathlib.Path("/root/reference")


def build_ref(reference: pathlib.Path = DEFAULT_REFERENCE) -> pathlib.Path | None:
    """Copy ``<reference>/gdn2/reference.py`` to ``oracle/_ref/gdn2_reference.py``. Returns the new path, or
    ``None`` when no checkout is present (the prebuilt copy, if any, is left as it is)."""
    src = pathlib.Path(reference) / "gdn2" / "reference.py"
    if not src.exists():
        return None
    OUT.mkdir(exist_ok=True)
    dst = OUT / "gdn2_reference.py"
    shutil.copyfile(src, dst)
    (OUT / "gdn2_reference.sha256").write_text(hashlib.sha256(dst.read_bytes()).hexdigest() + "  gdn2/reference.py\n")
    return dst


def load_ref():
    """The vendored module, or ``None`` when ``oracle/_ref`` has not been built."""
    path = OUT / "gdn2_reference.py"
    if not path.exists():
        return None
    import importlib.util

    spec = importlib.util.spec_from_file_location("gdn2_reference_vendored", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=str(DEFAULT_REFERENCE))
    out = build_ref(pathlib.Path(ap.parse_args().reference))
    print(out if out else "no reference checkout found; nothing built")
