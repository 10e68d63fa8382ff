"""Drop-in names of the reference package.

The directory beside this file holds a package called ``i6_native_ops`` whose ``fbw`` and
``fast_viterbi`` sub-packages re-export this library's modules under the reference's import paths
(``i6_native_ops/fbw/__init__.py``, ``i6_native_ops/fast_viterbi/__init__.py``).  Code written against
the reference -- its own ``test/fbw.py`` and ``test/fast_viterbi.py`` included -- then runs unchanged:

    PYTHONPATH=$(python -c 'import i6_native_ops_b200.compat as c; print(c.path())') python -m unittest test/fbw.py

or, inside a program, ``i6_native_ops_b200.compat.install()`` before the first ``import i6_native_ops``.
Only the two automaton ops are provided; the reference's transducer losses are not part of this library.
"""
import os
import sys


def path() -> str:
    """Directory to put on ``sys.path`` / ``PYTHONPATH``."""
    return os.path.dirname(os.path.abspath(__file__))


def install() -> None:
    """Make ``import i6_native_ops.fbw`` / ``import i6_native_ops.fast_viterbi`` resolve to this library."""
    if path() not in sys.path:
        sys.path.insert(0, path())
