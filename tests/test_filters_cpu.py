"""The bitmask compiler against the restatement of the reference's filter evaluation (Core/FilterEvaluator.swift):
for every registered filter, the rows whose mask bit is set are exactly the rows the reference's evaluator passes;
hand-worked cases pin the text comparison rules of evaluateFilterOperation (:332-370)."""
import json

import numpy as np
import pytest

from oracle import filter_ref as fr
from vectorstorekit_b200.filters import (CompositeFilter, FilterBitmaskCompiler, FilterOperation as Op,
                                         LogicalOperation as L, MetadataFilter, VectorFilter, evaluate_operation)


def _to_ref(f):
    if isinstance(f, MetadataFilter):
        return ("meta", f.key, f.operation.value, f.value)
    if isinstance(f, VectorFilter):
        return ("vec", f.constraint[0], f.constraint[1], f.constraint[2], f.dimension, f.range)
    return (f.operation.value, [_to_ref(s) for s in f.filters])


def test_operation_rules_by_hand():
    # values are compared as text, also for ordering: "10" < "9"
    assert evaluate_operation("10", Op.lessThan, "9")
    assert not evaluate_operation("10", Op.greaterThan, "9")
    assert evaluate_operation("abc", Op.contains, "bc") and evaluate_operation("abc", Op.notContains, "x")
    assert evaluate_operation("abc", Op.startsWith, "ab") and evaluate_operation("abc", Op.endsWith, "bc")
    # `in` splits on commas, drops empty pieces and trims spaces
    assert evaluate_operation("b", Op.in_, "a, b ,,c") and not evaluate_operation("", Op.in_, "a,,c")
    assert evaluate_operation("d", Op.notIn, "a, b ,c")
    assert evaluate_operation("cat-42", Op.regex, r"^cat-\d+$") and not evaluate_operation("x", Op.regex, "(")
    for op in Op:
        ref = fr.passes(("meta", "k", op.value, "m"), json.dumps({"k": "mm"}), [0.0])
        assert evaluate_operation("mm", op, "m") == ref, op


def test_describe_matches_restatement():
    comp = FilterBitmaskCompiler()
    f = [MetadataFilter("v", Op.equals, t) for t in ("7", "2.5", "1", "0", "x", "3")]
    for x in f:
        comp.register(x)
    md = [json.dumps({"v": v}) for v in (7, 2.5, True, False, "x", 3.0)]
    masks = comp.row_masks(md, np.zeros((6, 2), np.float32))
    assert [int(m) for m in masks] == [1 << i for i in range(6)]


def _random_rows(rng, n, d):
    cats = ["news", "sports", "tech", "art"]
    md = []
    for r in range(n):
        m = {"category": cats[rng.integers(0, 4)], "year": int(rng.integers(1990, 2025)), "score": float(np.round(rng.random() * 10, 2)),
             "public": bool(rng.integers(0, 2)), "title": "doc-%d" % r}
        if rng.random() < 0.1:
            del m["category"]
        md.append(json.dumps(m) if rng.random() > 0.02 else "not json")
    x = rng.standard_normal((n, d)).astype(np.float32)
    x[rng.random((n, d)) < 0.3] = 0
    return md, x


FILTERS = [
    MetadataFilter("category", Op.equals, "tech"),
    MetadataFilter("category", Op.in_, "news, art"),
    MetadataFilter("year", Op.greaterThanOrEqual, "2010"),
    MetadataFilter("public", Op.equals, "1"),
    MetadataFilter("title", Op.regex, r"doc-\d*7$"),
    MetadataFilter("missing", Op.notEquals, "x"),
    VectorFilter(("magnitude", 0.0, 2.5)),
    VectorFilter(("sparsity", 0.5, 1.0), dimension=1, range=(-0.5, 0.5)),
    CompositeFilter(L.and_, (MetadataFilter("category", Op.equals, "tech"), MetadataFilter("year", Op.lessThan, "2005"))),
    CompositeFilter(L.not_, (MetadataFilter("public", Op.equals, "1"), MetadataFilter("category", Op.equals, "tech"))),
    CompositeFilter(L.or_, (MetadataFilter("category", Op.equals, "art"),
                            CompositeFilter(L.and_, (VectorFilter(("magnitude", 0.0, 2.0)), MetadataFilter("score", Op.greaterThan, "5"))))),
    CompositeFilter(L.not_, ()),
]


def test_compiler_equals_reference_evaluation():
    rng = np.random.default_rng(11)
    md, x = _random_rows(rng, 600, 6)
    comp = FilterBitmaskCompiler()
    bits = [comp.register(f) for f in FILTERS]
    assert bits == list(range(len(FILTERS))) and comp.register(FILTERS[3]) == 3
    masks = comp.row_masks(md, x)
    for f, b in zip(FILTERS, bits):
        got = (masks >> np.uint64(b)) & np.uint64(1)
        want = fr.eligible_rows(_to_ref(f), md, x)
        assert np.array_equal(got.astype(bool), want), f
        assert 0 < want.sum() < 600 or isinstance(f, CompositeFilter) or f.key == "missing"
    # a query's mask: a registered filter is its bit; an `or` of registered filters is their union
    assert comp.query_mask(FILTERS[2]) == 1 << 2
    union = CompositeFilter(L.or_, (FILTERS[0], FILTERS[6]))
    qm = comp.query_mask(union)
    assert qm == (1 << 0) | (1 << 6)
    assert np.array_equal((masks & np.uint64(qm)) != 0, fr.eligible_rows(_to_ref(union), md, x))
    with pytest.raises(KeyError):
        comp.query_mask(CompositeFilter(L.and_, (FILTERS[0], FILTERS[6])))     # needs a bit of its own
    with pytest.raises(KeyError):
        comp.query_mask(MetadataFilter("year", Op.equals, "2000"))


def test_capacity_is_64_filters():
    comp = FilterBitmaskCompiler()
    for i in range(64):
        comp.register(MetadataFilter("k", Op.equals, str(i)))
    with pytest.raises(ValueError):
        comp.register(MetadataFilter("k", Op.equals, "64"))
    masks = comp.row_masks([json.dumps({"k": 63})], np.zeros((1, 1), np.float32))
    assert int(masks[0]) == 1 << 63
