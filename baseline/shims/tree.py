"""Stand-in for the `dm-tree` package on the reference's import path.

The unmodified reference does `import tree` (fmoe/layers.py:4) and uses only
`tree.map_structure` and `tree.flatten`; dm-tree is not installed on this box and cannot be
fetched.  This file is used by the reference arm of the benchmark only.
"""


def flatten(structure):
    if isinstance(structure, dict):
        out = []
        for key in sorted(structure):
            out.extend(flatten(structure[key]))
        return out
    if isinstance(structure, (list, tuple)):
        out = []
        for item in structure:
            out.extend(flatten(item))
        return out
    return [structure]


def map_structure(func, *structures):
    first = structures[0]
    if isinstance(first, dict):
        return type(first)((k, map_structure(func, *[s[k] for s in structures])) for k in first)
    if isinstance(first, (list, tuple)):
        return type(first)(map_structure(func, *items) for items in zip(*structures))
    return func(*structures)
