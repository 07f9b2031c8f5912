"""Minimal pytree helpers (lists, tuples, namedtuples, dicts, None).

The reference walks nested containers of specs and arrays with `jax.tree`
(e.g. jax_tpu_embedding/sparsecore/lib/nn/embedding.py:56-64,681-686).  JAX is not a
dependency here, so the same traversal order is implemented directly: dict keys
are visited in sorted order, None is an empty subtree, everything else is a leaf.
"""

from __future__ import annotations

from typing import Any, Callable


def _is_namedtuple(x) -> bool:
  return isinstance(x, tuple) and hasattr(x, "_fields")


def _children(x):
  """Returns (keys, children) for a container node, or None for a leaf."""
  if x is None:
    return (), ()
  if isinstance(x, dict):
    keys = sorted(x.keys())
    return tuple(keys), tuple(x[k] for k in keys)
  if isinstance(x, (list, tuple)):
    return tuple(range(len(x))), tuple(x)
  return None


def _rebuild(proto, children):
  if proto is None:
    return None
  if isinstance(proto, dict):
    return type(proto)(zip(sorted(proto.keys()), children)) if type(proto) is not dict else dict(
        zip(sorted(proto.keys()), children))
  if _is_namedtuple(proto):
    return type(proto)(*children)
  return type(proto)(children)


def leaves_with_path(tree, is_leaf: Callable[[Any], bool] | None = None, _path=()):
  if is_leaf is not None and is_leaf(tree):
    return [(_path, tree)]
  node = _children(tree)
  if node is None:
    return [(_path, tree)]
  out = []
  for k, c in zip(*node):
    out.extend(leaves_with_path(c, is_leaf, _path + (k,)))
  return out


def leaves(tree, is_leaf=None):
  return [v for _, v in leaves_with_path(tree, is_leaf)]


def structure(tree, is_leaf=None):
  """A hashable description of the container structure (leaves become '*')."""
  if is_leaf is not None and is_leaf(tree):
    return "*"
  node = _children(tree)
  if node is None:
    return "*"
  keys, kids = node
  return (type(tree).__name__, tuple((k, structure(c, is_leaf)) for k, c in zip(keys, kids)))


def flatten(tree, is_leaf=None):
  return leaves(tree, is_leaf), tree


def unflatten(proto, new_leaves, is_leaf=None):
  it = iter(new_leaves)

  def go(t):
    if is_leaf is not None and is_leaf(t):
      return next(it)
    node = _children(t)
    if node is None:
      return next(it)
    return _rebuild(t, [go(c) for c in node[1]])

  return go(proto)


def tree_map(fn, tree, *rest, is_leaf=None):
  def go(t, others):
    if is_leaf is not None and is_leaf(t):
      return fn(t, *others)
    node = _children(t)
    if node is None:
      return fn(t, *others)
    keys, kids = node
    other_kids = []
    for o in others:
      onode = _children(o)
      if onode is None or onode[0] != keys:
        raise ValueError("tree_map: structures do not match")
      other_kids.append(onode[1])
    return _rebuild(t, [go(c, [ok[i] for ok in other_kids]) for i, c in enumerate(kids)])

  return go(tree, list(rest))


def assert_same_structure(a, b, a_name="a", b_name="b"):
  """ValueError unless both trees have identical leaf paths (embedding.py:56-64)."""
  a_paths = [p for p, _ in leaves_with_path(a)]
  b_paths = [p for p, _ in leaves_with_path(b)]
  if a_paths != b_paths:
    raise ValueError(
        f"Pytree structures of {a_name} and {b_name} do not match.\n"
        f"{a_name}: {structure(a)}\n{b_name}: {structure(b)}")
