"""Comparison rule for k-NN results, as the acceptance criterion states it: identical top-k ids
except for ties within 1e-5 relative distance, and distances within 1e-4 relative."""
import numpy as np

ID_TIE_RTOL = 1e-5
DIST_RTOL = 1e-4


def assert_topk_parity(got_d, got_i, ref_d, ref_i, id_tie_rtol=ID_TIE_RTOL, dist_rtol=DIST_RTOL, atol=1e-6):
    got_d, got_i, ref_d, ref_i = (np.asarray(a) for a in (got_d, got_i, ref_d, ref_i))
    assert got_d.shape == ref_d.shape and got_i.shape == ref_i.shape
    # distances position by position (both lists are ascending, so near-ties cannot hurt this)
    fin = np.isfinite(ref_d)
    assert np.array_equal(np.isfinite(got_d), fin), "different number of hits"
    scale = np.maximum(np.abs(ref_d[fin]), atol / dist_rtol)
    err = np.abs(got_d[fin] - ref_d[fin]) / scale
    assert err.size == 0 or err.max() <= dist_rtol, f"distance mismatch: max rel err {err.max():.3e}"
    assert np.array_equal(got_i < 0, ref_i < 0)
    mism = got_i != ref_i
    if not mism.any():
        return 0
    # every disagreeing slot must sit in a run of near-equal reference distances that explains it:
    # the id found there must appear in the reference row at a position whose distance is within the
    # tie tolerance, or be displaced across the k-th boundary by a tie with the last kept distance.
    bad = 0
    for q, j in zip(*np.nonzero(mism)):
        d_here = ref_d[q, j]
        tol = id_tie_rtol * max(abs(d_here), atol / id_tie_rtol)
        where = np.nonzero(ref_i[q] == got_i[q, j])[0]
        if where.size:
            ok = abs(ref_d[q, where[0]] - d_here) <= tol
        else:  # came from beyond the reference's k-th: must tie with the boundary distance
            ok = abs(got_d[q, j] - ref_d[q, -1]) <= id_tie_rtol * max(abs(ref_d[q, -1]), atol / id_tie_rtol) * 2
        bad += 0 if ok else 1
    assert bad == 0, f"{bad} id mismatches not explained by ties"
    return int(mism.sum())
