"""TEST INFRASTRUCTURE — an independent restatement of the reference's filter evaluation, used by tests to check
the bitmask compiler.  Follows Core/FilterEvaluator.swift: evaluateMetadataFilter (:116-137), evaluateVectorFilter
(:150-186), evaluateCompositeFilter (:212-244), evaluateFilterOperation (:332-370), and the pre-filter order of
Indexes/IVFIndex.swift:163-172 (filter, then distances, then sort).  Filters are plain tuples here:
    ("meta", key, op, value) | ("vec", kind, lo, hi, dimension, range) | ("and"|"or"|"not", [filters])

Parity unpinned for: String(describing:) of nested JSON values, Swift's Unicode string ordering beyond ASCII, and
NSRegularExpression (ICU) patterns beyond the syntax Python's ``re`` shares with it.  The reference tree has no
golden vectors for filters.
"""
import json
import re

import numpy as np


def _text(v):
    if v is True:
        return "1"
    if v is False:
        return "0"
    if isinstance(v, int):
        return "%d" % v
    if isinstance(v, float):
        return "%d" % v if v == int(v) and abs(v) < 1e15 else repr(v)
    if isinstance(v, str):
        return v
    return json.dumps(v)


_OPS = {
    "equals": lambda a, b: a == b, "notEquals": lambda a, b: a != b,
    "lessThan": lambda a, b: a < b, "lessThanOrEqual": lambda a, b: a <= b,
    "greaterThan": lambda a, b: a > b, "greaterThanOrEqual": lambda a, b: a >= b,
    "contains": lambda a, b: a.find(b) >= 0, "notContains": lambda a, b: a.find(b) < 0,
    "startsWith": lambda a, b: a[:len(b)] == b, "endsWith": lambda a, b: b == "" or a[-len(b):] == b,
    "in": lambda a, b: a in [x.strip(" \t") for x in b.split(",") if x],
    "notIn": lambda a, b: a not in [x.strip(" \t") for x in b.split(",") if x],
}


def passes(flt, metadata_text, vector) -> bool:
    kind = flt[0]
    if kind == "meta":
        _, key, op, value = flt
        try:
            md = json.loads(metadata_text) if metadata_text is not None else None
        except ValueError:
            md = None
        if not isinstance(md, dict) or key not in md:
            return False
        have = _text(md[key])
        if op == "regex":
            try:
                return re.search(value, have) is not None
            except re.error:
                return False
        return bool(_OPS[op](have, value))
    if kind == "vec":
        _, c, lo, hi, dim, rng = flt
        v = np.asarray(vector, np.float32)
        if dim is not None and dim < v.size and rng is not None and not (rng[0] <= v[dim] <= rng[1]):
            return False
        if c == "magnitude":
            s = np.float32(0)
            for x in v:
                s = np.float32(s + np.float32(x * x))
            return bool(lo <= np.sqrt(s) <= hi)
        return bool(lo <= np.float32(np.count_nonzero(v)) / np.float32(v.size) <= hi)
    subs = flt[1]
    if kind == "and":
        return all(passes(f, metadata_text, vector) for f in subs)
    if kind == "or":
        return any(passes(f, metadata_text, vector) for f in subs)
    if kind == "not":
        return True if not subs else not passes(subs[0], metadata_text, vector)
    raise ValueError(kind)


def eligible_rows(flt, metadata_texts, vectors):
    return np.array([passes(flt, m, v) for m, v in zip(metadata_texts, vectors)], bool)
