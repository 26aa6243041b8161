"""Builds ``oracle/_ref/``: the reference project's own Python modules, compiled to bytecode.

The reference (RishiShah99/lethe) is pure Python on the CPU side of this path, so "building" it means
byte-compiling its sources where they lie.  Only compiled ``.pyc`` files are written, into the
git-ignored ``oracle/_ref/lethe/`` tree (sourceless imports: ``x.pyc`` sits where ``x.py`` would);
no reference source is copied.  The tree travels with the checkout to a machine that has no copy
of the reference, where the tests and the benchmark's CPU arm import ``lethe.*`` from it:

  * ``lethe.kernels.references.*``      the token-serial and chunkwise references (fp32 / fp64)
  * ``lethe.kernels.cute.gdn2_assemble`` the backward assembly with its ``k1_fn`` / ``k2_fn`` hooks
  * ``lethe.kernels.cute.gdn2_family``   the family wrappers (KDA, GLA, LA, SSD)
  * ``lethe.kernels.ops.gdn_layer``      the autograd op
  * ``lethe.verifier.*``                 the contract gates and the op harness

This is test infrastructure.  Nothing in the ``lethe_b200`` package imports it.

Usage:  python oracle/make_ref.py [/path/to/reference]        (default /root/reference)
"""

from __future__ import annotations

import os
import py_compile
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
SUBTREES = ("lethe",)          # everything under src/lethe (a few hundred KB of bytecode)


def build(reference_root: str = "/root/reference", quiet: bool = False) -> str | None:
    src_root = os.path.join(reference_root, "src")
    if not os.path.isdir(os.path.join(src_root, "lethe")):
        if not quiet:
            print(f"make_ref: no reference at {reference_root}; keeping {OUT} as it is", file=sys.stderr)
        return OUT if os.path.isdir(os.path.join(OUT, "lethe")) else None
    tmp = OUT + ".tmp"
    shutil.rmtree(tmp, ignore_errors=True)
    n = 0
    for sub in SUBTREES:
        for dirpath, _dirs, files in os.walk(os.path.join(src_root, sub)):
            rel = os.path.relpath(dirpath, src_root)
            for f in files:
                if not f.endswith(".py"):
                    continue
                dst = os.path.join(tmp, rel, f[:-3] + ".pyc")
                os.makedirs(os.path.dirname(dst), exist_ok=True)
                # dfile: the path tracebacks show; UNCHECKED_HASH: valid without the source file
                py_compile.compile(os.path.join(dirpath, f), cfile=dst, dfile=os.path.join("reference", "src", rel, f),
                                   doraise=True, invalidation_mode=py_compile.PycInvalidationMode.UNCHECKED_HASH)
                n += 1
    with open(os.path.join(tmp, "BUILT_FROM"), "w") as fh:
        fh.write(f"byte-compiled from {src_root} by oracle/make_ref.py with Python {sys.version.split()[0]}; {n} modules\n")
    shutil.rmtree(OUT, ignore_errors=True)
    os.replace(tmp, OUT)
    if not quiet:
        print(f"make_ref: {n} modules -> {OUT}")
    return OUT


def path() -> str | None:
    """``oracle/_ref`` if it holds the compiled reference, else None."""
    return OUT if os.path.isfile(os.path.join(OUT, "lethe", "__init__.pyc")) else None


def import_reference():
    """Put ``oracle/_ref`` on ``sys.path`` and return the imported ``lethe`` package, or None when the
    compiled reference is absent."""
    p = path()
    if p is None:
        return None
    if p not in sys.path:
        sys.path.insert(0, p)
    import lethe  # noqa: PLC0415

    return lethe


if __name__ == "__main__":
    build(sys.argv[1] if len(sys.argv) > 1 else "/root/reference")
