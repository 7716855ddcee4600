"""Stand-in for the `looseversion` package: LooseVersion with ordering on mixed int/str parts."""

import re


class LooseVersion:
    _component = re.compile(r"(\d+|[a-z]+|\.)", re.I)

    def __init__(self, vstring=None):
        self.vstring = str(vstring) if vstring is not None else ""
        parts = [p for p in self._component.split(self.vstring) if p and p != "."]
        self.version = [int(p) if p.isdigit() else p for p in parts]

    def _cmp(self, other):
        if isinstance(other, str):
            other = LooseVersion(other)
        a, b = self.version, other.version
        for x, y in zip(a, b):
            if type(x) is type(y):
                if x != y:
                    return -1 if x < y else 1
            else:   # numbers sort after strings ("1.0rc1" < "1.0.1")
                return 1 if isinstance(x, int) else -1
        return (len(a) > len(b)) - (len(a) < len(b))

    def __eq__(self, o): return self._cmp(o) == 0
    def __lt__(self, o): return self._cmp(o) < 0
    def __le__(self, o): return self._cmp(o) <= 0
    def __gt__(self, o): return self._cmp(o) > 0
    def __ge__(self, o): return self._cmp(o) >= 0
    def __repr__(self): return f"LooseVersion('{self.vstring}')"
    def __str__(self): return self.vstring
    def __hash__(self): return hash(tuple(self.version))
