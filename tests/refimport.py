"""Test helper: the reference project's own modules, imported from ``oracle/_ref`` (bytecode compiled
from the reference checkout by ``oracle/make_ref.py``; it travels with the repository to machines that
have no copy of the reference).  Tests that need it skip when it is absent."""

import pytest

from oracle import make_ref


def reference():
    """The imported ``lethe`` package of the reference, or skip."""
    pkg = make_ref.import_reference()
    if pkg is None:
        pytest.skip("oracle/_ref is absent: run `python oracle/make_ref.py` where the reference checkout is")
    return pkg
