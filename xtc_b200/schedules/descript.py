"""Declarative schedules ("descript") on top of the Scheduler interface.

The reference describes a loop nest as an ordered mapping from loop
declarations to annotations and turns it into scheduler calls
(``schedules/descript.py:36-58,512-542``; grammar ``schedules/parsing.py:
110-283``).  This module accepts the same specifications, so a script written
for the reference runs with the import changed:

    descript_scheduler(scheduler=sch, node_name="C", abstract_dims=["I", "J", "K"],
                       spec={"K": {}, "I": {}, "J": {},
                             "I#2": {"unroll": True}, "J#16": {"vectorize": True}})

Declarations, in loop order from the outside in:

* ``"A"``           the loop over axis A itself;
* ``"A#n"``         a tile of axis A of n iterations (the k-th tile of A is named ``A<k>``);
* ``"A[x:y]"``      the iterations x..y of A as a nest of their own, the value being a
                    nested specification; ``"A[:z:]"`` = the next z iterations.  Segments
                    must follow one another and cover the axis when its size is known.

Annotations: ``unroll`` (True = the whole loop, or a factor), ``vectorize``,
``parallelize``, ``buffer`` (memory type or "default"), ``pack`` ((input, memory
type, pad)).  Sizes may be names looked up in ``sample``.  What is not carried
over: symbolic constraints between unbound parameters (the reference hands those
to its sampling strategies); a name without a value in ``sample`` is an error.
"""

from __future__ import annotations

import re
from typing import Any, Mapping

__all__ = ["descript_scheduler", "ScheduleParseError", "ScheduleInterpretError"]

_SPLIT = re.compile(r"^(.*)\[(-?\w*)?:(-?\w*)?\]$")
_SPLIT_SIZE = re.compile(r"^(.*)\[:(\w*):\]$")
_ANNOTATIONS = ("unroll", "vectorize", "parallelize", "buffer", "pack", "partial", "full")


class ScheduleParseError(ValueError):
    pass


class ScheduleInterpretError(ValueError):
    pass


def _value(text: Any, sample: Mapping[str, int], what: str) -> int:
    """An integer literal, or a parameter name bound by ``sample``."""
    if isinstance(text, bool):
        raise ScheduleParseError(f"{what}: expected an integer, got {text!r}")
    if isinstance(text, int):
        return text
    s = str(text)
    if re.fullmatch(r"-?\d+", s):
        return int(s)
    if s in sample:
        return int(sample[s])
    raise ScheduleInterpretError(f"{what}: parameter {s!r} has no value in the sample")


class _Nest:
    """What one root (the node, or one split segment) records before it is applied."""

    def __init__(self, root: str, dims: list[str]) -> None:
        self.root = root
        self.splits: dict[str, dict[str, int]] = {}
        self.tiles: dict[str, dict[str, int]] = {d: {} for d in dims}
        self.interchange: list[str] = []
        self.vectorize: list[str] = []
        self.parallelize: list[str] = []
        self.unroll: dict[str, int] = {}
        self.buffer_at: dict[str, str | None] = {}
        self.pack_at: dict[str, tuple[int, str | None, bool]] = {}
        self.children: list[_Nest] = []


class _Interpreter:
    def __init__(self, dims: list[str], dim_sizes: Mapping[str, int], matrices: list[str],
                 sample: Mapping[str, int]) -> None:
        self.dims = dims
        self.dim_sizes = dict(dim_sizes)
        self.matrices = matrices
        self.sample = sample

    def check_axis(self, axis: str) -> None:
        if axis not in self.dims:
            raise ScheduleInterpretError(
                f"Axis {axis} is not a defined axis (defined axis: {self.dims}).")

    def nest(self, spec: Mapping[str, Any], root: str, head: list[str],
             extents: dict[str, int | None]) -> _Nest:
        node = _Nest(root, self.dims)
        node.interchange = list(head)
        sizes: dict[str, int | None] = dict(extents)   # loop name -> iterations, where known
        cut: dict[str, int | None] = {a: 0 for a in self.dims}  # where the last segment ended
        current = ""
        for decl, value in spec.items():
            if value is None:
                value = {}
            if not isinstance(value, Mapping):
                raise ScheduleParseError(f"`{decl}`: expected a mapping of annotations, got {value!r}")
            if ":" in decl:
                self.split(decl, value, node, cut, extents)
                continue
            if "#" in decl:
                parts = decl.split("#")
                if len(parts) != 2:
                    raise ScheduleParseError(f"`{decl}`: invalid tile syntax, expected 'axis#size'")
                axis = parts[0]
                self.check_axis(axis)
                size = _value(parts[1], self.sample, f"`{decl}`")
                if size <= 0:
                    raise ScheduleInterpretError(f"`{decl}`: tile sizes should be strictly positive.")
                current = f"{axis}{len(node.tiles[axis])}"
                node.tiles[axis][current] = size
                sizes[current] = size
                node.interchange.append(current)
            else:
                if decl in self.matrices:
                    self.annotate(value, decl, current, sizes, node)
                    continue
                self.check_axis(decl)
                if decl in node.interchange:
                    raise ScheduleInterpretError(f"Axis {decl} is scheduled twice (or more).")
                current = decl
                node.interchange.append(decl)
            self.annotate(value, decl, current, sizes, node)
        for axis, at in cut.items():
            if at not in (0, None) and extents.get(axis) not in (None, at):
                raise ScheduleInterpretError(f"Splitting of {axis} unachieved (stops at {at}).")
        return node

    def split(self, decl: str, body: Mapping[str, Any], node: _Nest, cut: dict[str, int | None],
              extents: dict[str, int | None]) -> None:
        m = _SPLIT.match(decl)
        size = None
        if m:
            axis, lo, hi = m.group(1), m.group(2) or None, m.group(3) or None
        else:
            m = _SPLIT_SIZE.match(decl)
            if not m:
                raise ScheduleParseError(f"`{decl}`: invalid split syntax")
            axis, lo, hi, size = m.group(1), None, None, m.group(2) or None
        self.check_axis(axis)
        prev = cut[axis]
        if prev is None:
            raise ScheduleInterpretError(f"{decl}: {axis} already covered.")
        extent = extents.get(axis)
        if size is not None:
            start = prev
            end: int | None = start + _value(size, self.sample, f"`{decl}`")
        else:
            start = prev if lo is None else _value(lo, self.sample, f"`{decl}`")
            end = extent if hi is None else _value(hi, self.sample, f"`{decl}`")
            if start > prev:
                raise ScheduleInterpretError(
                    f"{decl}: splitting doesn't fully cover {axis} (jumps from {prev} to {start}).")
            if start < prev:
                raise ScheduleInterpretError(
                    f"{decl}: the segment begins at {start} but the previous one ends at {prev}.")
            if end is not None and start >= end:
                raise ScheduleInterpretError(
                    f"{decl}: the ending point should be greater than the starting point.")
        if extent is not None and end is not None and end > extent:
            raise ScheduleInterpretError(f"{decl}: the segment ends at {end}, past the {extent} iterations of {axis}.")
        cut[axis] = None if (hi is None and size is None) else end
        name = f"{axis}[{len(node.splits.setdefault(axis, {}))}]"
        node.splits[axis][name] = start
        node.interchange.append(name)
        inner = dict(extents)
        inner[axis] = None if end is None else end - start
        node.children.append(self.nest(body, f"{node.root}/{name}", [axis], inner))

    def annotate(self, value: Mapping[str, Any], decl: str, loop: str,
                 sizes: Mapping[str, int | None], node: _Nest) -> None:
        for key in value:
            if key not in _ANNOTATIONS:
                raise ScheduleParseError(f"Unknown annotation on {decl}: {key}")
        if "partial" in value and "full" in value:
            raise ScheduleParseError(f"{decl} has both annotations full and partial")
        if "unroll" in value and value["unroll"] is not False:
            param = value["unroll"]
            if param is True or param is None:
                if sizes.get(loop) is None:
                    raise ScheduleInterpretError(
                        f"{loop}'s size being unknown, an unroll factor is needed.")
                factor = sizes[loop]
            elif isinstance(param, (int, str)):
                factor = _value(param, self.sample, f'`{{"unroll" = {param}}}`')
                if factor <= 0:
                    raise ScheduleInterpretError(
                        f'`{{"unroll" = {param}}}`: unroll parameter should be strictly positive.')
            else:
                raise ScheduleParseError(
                    f'`{{"unroll" = {param}}}`: unroll parameter should be True, False, or a string or integer.')
            node.unroll[loop] = int(factor)
        for key, noun, target in (("vectorize", "vectorization", node.vectorize),
                                  ("parallelize", "parallelization", node.parallelize)):
            if key in value:
                param = True if value[key] is None else value[key]
                if isinstance(param, str):
                    param = bool(_value(param, self.sample, f'`{{"{key}" = {param}}}`'))
                if not isinstance(param, bool):
                    raise ScheduleParseError(
                        f'`{{"{key}" = {param}}}`: {noun} parameter should be True, False or a string.')
                if param:
                    target.append(loop)
        if "buffer" in value:
            param = value["buffer"]
            if not isinstance(param, str):
                raise ScheduleParseError(
                    f'`{{"buffer" = {param}}}`: buffer parameter should be a string (mtype).')
            node.buffer_at[loop] = None if param == "default" else param
        if "pack" in value:
            param = value["pack"]
            if param is None:
                param = (decl, None, False)
            if not isinstance(param, (list, tuple)) or len(param) != 3:
                raise ScheduleParseError(
                    f'`{{"pack" = {param}}}` on {decl}: pack parameter should be a tuple (input_idx, mtype, pad).')
            which, mtype, pad = param
            mtype = None if mtype == "default" else mtype
            if isinstance(which, str) and which in self.matrices:
                idx = self.matrices.index(which)
                if idx == len(self.matrices) - 1:   # the last matrix is the output: a write buffer
                    node.buffer_at[loop] = mtype
                    return
                which = idx
            node.pack_at[loop] = (_value(which, self.sample, f"`pack` on {decl}"), mtype, bool(pad))


def _apply(node: _Nest, scheduler: Any) -> None:
    """The call sequence of the reference's ``_apply_node`` (schedules/descript.py:519-542)."""
    root = node.root
    for dim, segments in node.splits.items():
        scheduler.split(dim, segments, root=root)
    for dim, tiles in node.tiles.items():
        scheduler.tile(dim, tiles, root=root)
    scheduler.interchange(node.interchange, root=root)
    scheduler.vectorize(node.vectorize, root=root)
    scheduler.parallelize(node.parallelize, root=root)
    scheduler.unroll(node.unroll, root=root)
    for axis, mtype in node.buffer_at.items():
        scheduler.buffer_at(axis, mtype=mtype, root=root)
    for axis, (idx, mtype, pad) in node.pack_at.items():
        scheduler.pack_at(axis, idx, mtype=mtype, pad=pad, root=root)
    for child in node.children:
        _apply(child, scheduler)


def descript_scheduler(scheduler: Any, node_name: str, abstract_dims: list[str],
                       spec: Mapping[str, Any] | str,
                       abstract_dim_sizes: Mapping[str, int] | None = None,
                       abstract_matrix: list[str] | None = None,
                       sample: Mapping[str, int] | None = None) -> None:
    """Apply a declarative schedule to ``scheduler`` (same signature as the reference's
    ``descript_scheduler``, schedules/descript.py:36-58).  ``spec`` is a mapping or its
    YAML text; key order is loop order."""
    if isinstance(spec, str):
        import yaml

        spec = yaml.safe_load(spec)
    if not isinstance(spec, Mapping):
        raise ScheduleParseError("the specification must be a mapping from declarations to annotations")
    spec = dict(spec)
    spec.pop("constraints", None)  # constraints between unbound parameters: nothing left to check
    sizes = dict(abstract_dim_sizes or {})
    interp = _Interpreter(list(abstract_dims), sizes, list(abstract_matrix or []), dict(sample or {}))
    extents: dict[str, int | None] = {d: sizes.get(d) for d in abstract_dims}
    nest = interp.nest(spec, node_name, [], extents)
    target = scheduler
    if callable(getattr(type(scheduler), "node", None)):  # several nodes: address the named one
        try:
            target = scheduler.node(node_name)
        except KeyError:
            target = scheduler
    target.set_dims(list(abstract_dims))
    _apply(nest, target)
