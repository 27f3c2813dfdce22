"""Metadata filters compiled to the 64-bit row / query masks of the GPU search.

The reference filters candidates *before* distances (``Indexes/IVFIndex.swift:163-165``) by evaluating a
``SearchFilter`` on every stored vector's JSON metadata, one task per vector
(``Core/FilterEvaluator.swift:375-437``).  The GPU search instead keeps a 64-bit mask per row and takes a mask per
query: row r is eligible for query q iff ``row_mask[r] & query_mask[q] != 0``.  This module is the bridge:

* the filter types mirror ``SearchFilter`` (``Core/Protocols.swift:493-541``): ``MetadataFilter`` (key, operation,
  value), ``VectorFilter`` (dimension range, magnitude, sparsity), ``CompositeFilter`` (and / or / not);
* ``FilterBitmaskCompiler.register`` gives a filter one of the 64 bits;
* ``row_masks`` evaluates every registered filter on each row **at insert time** (host work, as in the reference);
* ``query_mask`` turns a query's filter into bits: a registered filter is its bit, an ``or`` of registered filters
  is the union of their bits.  A filter that is neither must be registered first (and the rows re-masked): a
  single AND-and-test cannot express ``and`` / ``not`` of bits, so a composite gets a bit of its own.

Value comparison follows ``evaluateFilterOperation`` (``FilterEvaluator.swift:332-370``): the metadata value is
turned into text and compared as text, also for the ordering operations.
"""
from __future__ import annotations

import dataclasses
import enum
import json
import math
import re
from typing import Callable, Optional, Sequence, Tuple, Union

import numpy as np


class FilterOperation(enum.Enum):
    equals = "equals"
    notEquals = "notEquals"
    lessThan = "lessThan"
    lessThanOrEqual = "lessThanOrEqual"
    greaterThan = "greaterThan"
    greaterThanOrEqual = "greaterThanOrEqual"
    contains = "contains"
    notContains = "notContains"
    startsWith = "startsWith"
    endsWith = "endsWith"
    in_ = "in"
    notIn = "notIn"
    regex = "regex"


class LogicalOperation(enum.Enum):
    and_ = "and"
    or_ = "or"
    not_ = "not"


@dataclasses.dataclass(frozen=True)
class MetadataFilter:
    key: str
    operation: FilterOperation
    value: str


@dataclasses.dataclass(frozen=True)
class VectorFilter:
    """``constraint`` is ("magnitude", lo, hi) or ("sparsity", lo, hi); ``dimension``/``range`` optionally bound one
    component (``FilterEvaluator.swift:150-180``).  The reference's ``.custom`` closure has no portable form."""
    constraint: Tuple[str, float, float]
    dimension: Optional[int] = None
    range: Optional[Tuple[float, float]] = None


@dataclasses.dataclass(frozen=True)
class CompositeFilter:
    operation: LogicalOperation
    filters: Tuple["SearchFilter", ...]


SearchFilter = Union[MetadataFilter, VectorFilter, CompositeFilter]


def describe(value) -> str:
    """``String(describing:)`` of a JSON value as ``JSONSerialization`` delivers it (``FilterEvaluator.swift:129``):
    text as is, numbers in their shortest decimal form, booleans as the NSNumber they are (1 / 0)."""
    if isinstance(value, bool):
        return "1" if value else "0"
    if isinstance(value, int):
        return str(value)
    if isinstance(value, float):
        return str(int(value)) if value.is_integer() and abs(value) < 1e15 else repr(value)
    if isinstance(value, str):
        return value
    return json.dumps(value)   # arrays / objects: the reference prints Foundation's debug form; not pinned


def evaluate_operation(value: str, op: FilterOperation, filter_value: str) -> bool:
    if op is FilterOperation.equals:
        return value == filter_value
    if op is FilterOperation.notEquals:
        return value != filter_value
    if op is FilterOperation.lessThan:
        return value < filter_value
    if op is FilterOperation.lessThanOrEqual:
        return value <= filter_value
    if op is FilterOperation.greaterThan:
        return value > filter_value
    if op is FilterOperation.greaterThanOrEqual:
        return value >= filter_value
    if op is FilterOperation.contains:
        return filter_value in value
    if op is FilterOperation.notContains:
        return filter_value not in value
    if op is FilterOperation.startsWith:
        return value.startswith(filter_value)
    if op is FilterOperation.endsWith:
        return value.endswith(filter_value)
    if op in (FilterOperation.in_, FilterOperation.notIn):
        # split(separator: ",") drops empty pieces; each piece is trimmed of spaces
        values = [p.strip(" \t") for p in filter_value.split(",") if p != ""]
        return (value in values) == (op is FilterOperation.in_)
    if op is FilterOperation.regex:
        try:
            return re.search(filter_value, value) is not None
        except re.error:
            return False
    raise ValueError(op)


def evaluate(flt: SearchFilter, metadata, vector) -> bool:
    """One filter on one row; ``metadata`` is the decoded JSON object (or None), ``vector`` its fp32 row."""
    if isinstance(flt, MetadataFilter):
        if not isinstance(metadata, dict) or flt.key not in metadata:
            return False                                       # no dictionary or no such key (:123-126)
        return evaluate_operation(describe(metadata[flt.key]), flt.operation, flt.value)
    if isinstance(flt, VectorFilter):
        v = np.asarray(vector, np.float32)
        if flt.dimension is not None and flt.dimension < v.size and flt.range is not None:
            if not (flt.range[0] <= float(v[flt.dimension]) <= flt.range[1]):
                return False
        kind, lo, hi = flt.constraint
        if kind == "magnitude":
            s = np.float32(0)
            for x in v:                                         # reduce(0) { $0 + $1 * $1 } in order
                s = np.float32(s + np.float32(x * x))
            return lo <= float(np.sqrt(s)) <= hi
        if kind == "sparsity":
            return lo <= float(np.float32(np.count_nonzero(v)) / np.float32(v.size)) <= hi
        raise ValueError(kind)
    if isinstance(flt, CompositeFilter):
        if flt.operation is LogicalOperation.and_:
            return all(evaluate(f, metadata, vector) for f in flt.filters)
        if flt.operation is LogicalOperation.or_:
            return any(evaluate(f, metadata, vector) for f in flt.filters)
        return True if not flt.filters else not evaluate(flt.filters[0], metadata, vector)   # only the first (:236-241)
    raise TypeError(type(flt))


class FilterBitmaskCompiler:
    """At most 64 registered filters, one bit each."""

    def __init__(self):
        self._bits = {}          # filter -> bit index

    @property
    def registered(self) -> Sequence[SearchFilter]:
        return list(self._bits)

    def register(self, flt: SearchFilter) -> int:
        if flt in self._bits:
            return self._bits[flt]
        if len(self._bits) >= 64:
            raise ValueError("all 64 mask bits are in use")
        self._bits[flt] = len(self._bits)
        return self._bits[flt]

    def row_masks(self, metadata: Sequence, vectors) -> np.ndarray:
        """uint64 mask per row: bit b set iff registered filter b passes.  ``metadata`` holds one JSON text
        (``bytes`` / ``str``), decoded object or None per row."""
        vectors = np.asarray(vectors, np.float32)
        if len(metadata) != vectors.shape[0]:
            raise ValueError("one metadata entry per row")
        out = np.zeros(vectors.shape[0], np.uint64)
        for r, md in enumerate(metadata):
            if isinstance(md, (bytes, bytearray, str)):
                try:
                    md = json.loads(md)
                except ValueError:
                    md = None                                   # undecodable metadata: every metadata filter fails
            m = 0
            for flt, bit in self._bits.items():
                if evaluate(flt, md, vectors[r]):
                    m |= 1 << bit
            out[r] = m
        return out

    def query_mask(self, flt: Optional[SearchFilter]) -> int:
        """The query-side mask.  ``None`` (no filter) selects every row that has any bit set; use all-ones row
        masks or an unfiltered search when rows may pass no registered filter."""
        if flt is None:
            return (1 << 64) - 1
        if flt in self._bits:
            return 1 << self._bits[flt]
        if isinstance(flt, CompositeFilter) and flt.operation is LogicalOperation.or_:
            m = 0
            for f in flt.filters:
                m |= self.query_mask(f)
            return m
        raise KeyError("filter is not registered (register it and rebuild the row masks): %r" % (flt,))

    def query_masks(self, filters: Sequence[Optional[SearchFilter]]) -> np.ndarray:
        return np.array([self.query_mask(f) for f in filters], np.uint64)
