"""Builds ``oracle/_ref/``: the reference project's own Python modules, compiled to bytecode.

The reference (RishiShah99/lethe) is pure Python on the CPU side of this path, so "building" it means
byte-compiling its sources where they lie.  Only compiled code objects are written, into the
git-ignored ``oracle/_ref/lethe/`` tree (``x.lbc`` where ``x.py`` would sit: the content of a ``.pyc``
under a name that file-synchronisation tools do not filter out as a cache file); no reference source is
copied.  ``import_reference()`` installs a small import hook that loads ``lethe.*`` from those files.  The tree travels with the checkout to a machine that has no copy
of the reference, where the tests and the benchmark's CPU arm import ``lethe.*`` from it:

  * ``lethe.kernels.references.*``      the token-serial and chunkwise references (fp32 / fp64)
  * ``lethe.kernels.cute.gdn2_assemble`` the backward assembly with its ``k1_fn`` / ``k2_fn`` hooks
  * ``lethe.kernels.cute.gdn2_family``   the family wrappers (KDA, GLA, LA, SSD)
  * ``lethe.kernels.ops.gdn_layer``      the autograd op
  * ``lethe.verifier.*``                 the contract gates and the op harness

This is test infrastructure.  Nothing in the ``lethe_b200`` package imports it.

Usage:  python oracle/make_ref.py [path of the reference checkout]      (default: ``REFERENCE_ROOT`` below,
or the environment variable ``LETHE_REFERENCE_ROOT``)
"""

from __future__ import annotations

import importlib.abc
import importlib.util
import marshal
import os
import py_compile
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
SUBTREES = ("lethe",)          # everything under src/lethe (a few hundred KB of bytecode)
EXT = ".lbc"                   # a .pyc by content: 16-byte header, then the marshalled code object
REFERENCE_ROOT = os.environ.get("LETHE_REFERENCE_ROOT", "/root/reference")


def build(reference_root: str = REFERENCE_ROOT, quiet: bool = False) -> str | None:
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
                dst = os.path.join(tmp, rel, f[:-3] + EXT)
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
    return OUT if os.path.isfile(os.path.join(OUT, "lethe", "__init__" + EXT)) else None


class _RefImporter(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    """Finds and loads ``lethe`` and its submodules from the ``.lbc`` files under ``oracle/_ref``."""

    def __init__(self, root: str):
        self.root = root

    def _file(self, fullname: str):
        rel = os.path.join(self.root, *fullname.split("."))
        if os.path.isfile(os.path.join(rel, "__init__" + EXT)):
            return os.path.join(rel, "__init__" + EXT), True
        if os.path.isfile(rel + EXT):
            return rel + EXT, False
        return None, False

    def find_spec(self, fullname, path=None, target=None):
        if fullname != "lethe" and not fullname.startswith("lethe."):
            return None
        file, is_pkg = self._file(fullname)
        if file is None:
            return None
        spec = importlib.util.spec_from_loader(fullname, self, origin=file, is_package=is_pkg)
        if is_pkg:
            spec.submodule_search_locations = [os.path.dirname(file)]
        return spec

    def create_module(self, spec):
        return None

    def exec_module(self, module):
        file, _ = self._file(module.__name__)
        with open(file, "rb") as fh:
            data = fh.read()
        module.__file__ = file
        exec(marshal.loads(data[16:]), module.__dict__)        # noqa: S102  (our own build product)


def import_reference():
    """Install the import hook for ``oracle/_ref`` and return the imported ``lethe`` package, or None when
    the compiled reference is absent."""
    p = path()
    if p is None:
        return None
    if not any(isinstance(f, _RefImporter) for f in sys.meta_path):
        sys.meta_path.insert(0, _RefImporter(p))
    import lethe  # noqa: PLC0415

    return lethe


if __name__ == "__main__":
    build(sys.argv[1] if len(sys.argv) > 1 else REFERENCE_ROOT)
