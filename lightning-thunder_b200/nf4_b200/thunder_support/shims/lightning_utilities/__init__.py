"""Stand-in for the parts of `lightning_utilities` Thunder imports."""

import importlib
import operator

from .core.imports import package_available  # noqa: F401


def compare_version(package: str, op, version: str, use_base_version: bool = False) -> bool:
    from looseversion import LooseVersion

    try:
        mod = importlib.import_module(package)
    except Exception:
        return False
    v = getattr(mod, "__version__", None)
    if v is None:
        return False
    v = str(v)
    if use_base_version:
        v = v.split("+")[0]
    return op(LooseVersion(v), LooseVersion(version))
