"""Numerical comparison used by the kernel tests.

A Frobenius-norm ratio alone lets a single wrong element, a bad boundary column or a dropped k-block
of one tile pass, so every comparison is made twice: the norm ratio against ``tol`` and an elementwise
bound ``|got - ref| <= 6 tol (|ref| + rms(ref))`` - no element may be off by more than a few times the
tolerated relative error measured against its own magnitude plus the tensor's typical magnitude."""
import torch


def close(got, ref, tol, what=""):
    g, r = got.float(), ref.float()
    assert g.shape == r.shape, (what, tuple(g.shape), tuple(r.shape))
    assert torch.isfinite(g).all(), (what, "non-finite values")
    rel = ((g - r).norm() / (r.norm() + 1e-12)).item()
    assert rel < tol, (what, "norm ratio", rel, tol)
    rms = r.pow(2).mean().sqrt()
    bound = 6.0 * tol * (r.abs() + rms) + 1e-6
    bad = (g - r).abs() > bound
    if bad.any():
        idx = bad.nonzero()[0].tolist()
        raise AssertionError((what, "elementwise", int(bad.sum()), "first at", idx, float(g[tuple(idx)]), float(r[tuple(idx)]),
                              float(bound[tuple(idx)])))
    return rel
