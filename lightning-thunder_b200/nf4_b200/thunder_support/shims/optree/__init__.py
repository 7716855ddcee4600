"""Minimal pure-Python stand-in for the `optree` package, covering what Thunder's
thunder/core/pytree.py uses: register_pytree_node, tree_flatten, tree_unflatten, tree_map,
tree_iter with `none_is_leaf` and a namespace registry.  Used only when the real (C++) optree is
not installed; Thunder is otherwise run unmodified."""

from __future__ import annotations

from collections import OrderedDict, defaultdict, deque

__version__ = "0.0-shim"

_registry: dict = {}        # (namespace, type) -> (flatten, unflatten)


def register_pytree_node(cls, flatten_func, unflatten_func, *, namespace=""):
    _registry[(namespace, cls)] = (flatten_func, unflatten_func)
    return cls


def _lookup(t, namespace):
    r = _registry.get((namespace, t))
    if r is None and namespace != "":
        r = _registry.get(("", t))
    return r


def _is_namedtuple(x):
    return isinstance(x, tuple) and hasattr(type(x), "_fields") and hasattr(x, "_asdict")


class PyTreeSpec:
    """kind: 'leaf' | 'none' | 'tuple' | 'list' | 'dict' | 'odict' | 'ddict' | 'ntuple' | 'deque' | 'custom'."""

    __slots__ = ("kind", "meta", "children", "num_leaves", "type", "unflatten_func", "none_is_leaf", "namespace")

    def __init__(self, kind, meta, children, type_=None, unflatten_func=None, none_is_leaf=False, namespace=""):
        self.kind, self.meta, self.children = kind, meta, children
        self.type, self.unflatten_func = type_, unflatten_func
        self.none_is_leaf, self.namespace = none_is_leaf, namespace
        self.num_leaves = 1 if kind == "leaf" else sum(c.num_leaves for c in children)

    @property
    def num_children(self):
        return len(self.children)

    def _build(self, it):
        k = self.kind
        if k == "leaf":
            return next(it)
        kids = [c._build(it) for c in self.children]
        if k == "none":
            return None
        if k == "tuple":
            return tuple(kids)
        if k == "list":
            return kids
        if k == "dict":
            return dict(zip(self.meta, kids))
        if k == "odict":
            return OrderedDict(zip(self.meta, kids))
        if k == "ddict":
            factory, keys = self.meta
            return defaultdict(factory, zip(keys, kids))
        if k == "ntuple":
            return self.type(*kids)
        if k == "deque":
            return deque(kids, maxlen=self.meta)
        return self.unflatten_func(self.meta, kids)

    def unflatten(self, leaves):
        leaves = list(leaves)
        if len(leaves) != self.num_leaves:
            raise ValueError(f"treespec expects {self.num_leaves} leaves, got {len(leaves)}")
        return self._build(iter(leaves))

    def __eq__(self, other):
        return (isinstance(other, PyTreeSpec) and self.kind == other.kind and self.type == other.type
                and self.meta == other.meta and self.children == other.children)

    def __hash__(self):
        return hash((self.kind, self.num_leaves, len(self.children)))

    def __repr__(self):
        return f"PyTreeSpec({self.kind}, leaves={self.num_leaves})"


def _sorted_keys(d):
    try:
        return sorted(d)
    except TypeError:
        return list(d)


def _flatten(x, leaves, none_is_leaf, namespace):
    t = type(x)
    if x is None:
        if none_is_leaf:
            leaves.append(x)
            return PyTreeSpec("leaf", None, (), none_is_leaf=none_is_leaf, namespace=namespace)
        return PyTreeSpec("none", None, (), none_is_leaf=none_is_leaf, namespace=namespace)
    reg = _lookup(t, namespace)
    if reg is not None:
        out = reg[0](x)
        children, meta = out[0], out[1]
        # a flatten function may itself return (leaves, spec) of a nested flatten
        if isinstance(meta, PyTreeSpec) and len(out) == 2:
            kids = [_flatten(c, leaves, none_is_leaf, namespace) for c in children]
            return PyTreeSpec("custom", meta, tuple(kids), t, reg[1], none_is_leaf, namespace)
        kids = [_flatten(c, leaves, none_is_leaf, namespace) for c in children]
        return PyTreeSpec("custom", meta, tuple(kids), t, reg[1], none_is_leaf, namespace)
    if t is tuple:
        return PyTreeSpec("tuple", None, tuple(_flatten(c, leaves, none_is_leaf, namespace) for c in x), t)
    if t is list:
        return PyTreeSpec("list", None, tuple(_flatten(c, leaves, none_is_leaf, namespace) for c in x), t)
    if t is dict:
        keys = _sorted_keys(x)
        return PyTreeSpec("dict", keys, tuple(_flatten(x[k], leaves, none_is_leaf, namespace) for k in keys), t)
    if t is OrderedDict:
        keys = list(x)
        return PyTreeSpec("odict", keys, tuple(_flatten(x[k], leaves, none_is_leaf, namespace) for k in keys), t)
    if t is defaultdict:
        keys = _sorted_keys(x)
        return PyTreeSpec("ddict", (x.default_factory, keys),
                          tuple(_flatten(x[k], leaves, none_is_leaf, namespace) for k in keys), t)
    if t is deque:
        return PyTreeSpec("deque", x.maxlen, tuple(_flatten(c, leaves, none_is_leaf, namespace) for c in x), t)
    if _is_namedtuple(x):
        return PyTreeSpec("ntuple", None, tuple(_flatten(c, leaves, none_is_leaf, namespace) for c in x), t)
    leaves.append(x)
    return PyTreeSpec("leaf", None, (), none_is_leaf=none_is_leaf, namespace=namespace)


def tree_flatten(tree, is_leaf=None, *, none_is_leaf=False, namespace=""):
    leaves: list = []
    spec = _flatten(tree, leaves, none_is_leaf, namespace)
    return leaves, spec


def tree_unflatten(treespec, leaves):
    return treespec.unflatten(leaves)


def tree_leaves(tree, is_leaf=None, *, none_is_leaf=False, namespace=""):
    return tree_flatten(tree, none_is_leaf=none_is_leaf, namespace=namespace)[0]


def tree_iter(tree, is_leaf=None, *, none_is_leaf=False, namespace=""):
    return iter(tree_leaves(tree, none_is_leaf=none_is_leaf, namespace=namespace))


def tree_structure(tree, is_leaf=None, *, none_is_leaf=False, namespace=""):
    return tree_flatten(tree, none_is_leaf=none_is_leaf, namespace=namespace)[1]


def tree_map(func, tree, *rests, is_leaf=None, none_is_leaf=False, namespace=""):
    leaves, spec = tree_flatten(tree, none_is_leaf=none_is_leaf, namespace=namespace)
    others = [tree_flatten(r, none_is_leaf=none_is_leaf, namespace=namespace)[0] for r in rests]
    return spec.unflatten([func(*xs) for xs in zip(leaves, *others)])


treespec_leaf = lambda none_is_leaf=False, namespace="": PyTreeSpec("leaf", None, ())
