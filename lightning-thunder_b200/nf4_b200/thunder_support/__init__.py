"""Bring-up of Thunder where its optional dependencies are missing.

`bootstrap()` makes `import thunder` work: it looks for Thunder on sys.path, then in
`baseline/_ref` (a `pip install --target` of the reference), and puts small pure-Python
stand-ins for `optree`, `looseversion`, `lightning_utilities` and `opt_einsum` on sys.path when
the real packages are absent.  Real `optree` is a C extension and therefore opaque to Thunder's
bytecode interpreter; the stand-in is Python, so its entry points are registered as opaque
lookasides after import (same idiom as thunder/tests/test_networks.py:262-267).
"""

from __future__ import annotations

import importlib.util
import os
import sys

_HERE = os.path.dirname(os.path.abspath(__file__))
_SHIMS = os.path.join(_HERE, "shims")
_REPO = os.path.dirname(os.path.dirname(os.path.dirname(_HERE)))
_done = False


def thunder_available() -> bool:
    try:
        bootstrap()
        return True
    except ImportError:
        return False


def bootstrap():
    """Imports thunder (adding fallbacks to sys.path as needed) and returns the module."""
    global _done
    if _done:
        import thunder

        return thunder
    if importlib.util.find_spec("thunder") is None:
        ref = os.path.join(_REPO, "baseline", "_ref")
        if os.path.isdir(os.path.join(ref, "thunder")):
            sys.path.append(ref)
        else:
            raise ImportError("thunder is not importable and baseline/_ref/thunder does not exist")
    shimmed = []
    for name in ("optree", "looseversion", "lightning_utilities", "opt_einsum"):
        if importlib.util.find_spec(name) is None:
            if _SHIMS not in sys.path:
                sys.path.append(_SHIMS)
            shimmed.append(name)
    import thunder

    if "optree" in shimmed:
        import optree
        from thunder.core.interpreter import interpreter_needs_wrap
        from thunder.core.jit_ext import register_general_jit_lookaside

        for fn in (optree.tree_flatten, optree.tree_unflatten, optree.tree_map, optree.tree_iter, optree.tree_leaves):
            register_general_jit_lookaside(fn)(interpreter_needs_wrap(fn))
    _done = True
    return thunder
