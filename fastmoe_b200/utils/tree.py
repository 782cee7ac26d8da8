r"""
Minimal pytree helpers.

The reference depends on the external ``dm-tree`` package for
``tree.map_structure`` / ``tree.flatten`` (``fmoe/layers.py:4,59,63,77``).  MoE inputs
and outputs may be a tensor, a list/tuple or a dict of tensors; nothing more is needed,
so the dependency is replaced by this module.  Dict leaves are visited in sorted-key
order, like ``dm-tree`` does.
"""
from collections import OrderedDict


def _is_namedtuple(x):
    return isinstance(x, tuple) and hasattr(x, "_fields")


def flatten(structure):
    r"""Leaves of ``structure`` in deterministic order."""
    out = []

    def visit(node):
        if isinstance(node, dict):
            for key in sorted(node.keys()):
                visit(node[key])
        elif isinstance(node, (list, tuple)):
            for item in node:
                visit(item)
        else:
            out.append(node)

    visit(structure)
    return out


def map_structure(fn, *structures):
    r"""Apply ``fn`` leaf-wise over one or more structures of identical shape."""
    first = structures[0]
    if isinstance(first, dict):
        keys = sorted(first.keys())
        mapped = [(k, map_structure(fn, *[s[k] for s in structures])) for k in keys]
        if isinstance(first, OrderedDict):
            return OrderedDict((k, dict(mapped)[k]) for k in first.keys())
        lookup = dict(mapped)
        return type(first)((k, lookup[k]) for k in first.keys())
    if _is_namedtuple(first):
        return type(first)(*[map_structure(fn, *items) for items in zip(*structures)])
    if isinstance(first, (list, tuple)):
        return type(first)(map_structure(fn, *items) for items in zip(*structures))
    return fn(*structures)


def first_leaf(structure):
    return flatten(structure)[0]
