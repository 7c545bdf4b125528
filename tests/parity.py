"""Comparators of the parity tests.

The stated tolerance of the path (rtol 2e-2 / atol 2e-2 on bf16 outputs) is an
absolute bound, and attention over n unit-variance values has a standard
deviation of about sqrt(e / n): 0.03 at 3 000 keys, 0.005 at 131 072.  At long
context every element is below the absolute tolerance and that comparison alone
accepts any output, an all-zero one included.  The checks here are scale-free:
the error bound follows the size of the reference row, so they keep their teeth
at every context length.  Both are applied in addition to the stated tolerance,
never instead of it."""
import torch

TOL = dict(atol=2e-2, rtol=2e-2)
LSE_TOL = dict(atol=2e-3, rtol=2e-3)


def row_rms(ref: torch.Tensor) -> torch.Tensor:
    """Root mean square of every row (last axis) of ``ref``, kept as a trailing axis of 1."""
    return ref.float().pow(2).mean(-1, keepdim=True).sqrt()


def scale_free_violations(out: torch.Tensor, ref: torch.Tensor, atol_rms: float = 2e-2,
                          rtol: float = 2.0 ** -7, rel_l2: float = 1e-2) -> dict:
    """Counts of what ``assert_scale_free`` would object to (empty dict = passes).

    Elementwise: |out - ref| <= atol_rms * rms(ref row) + rtol * |ref|; rtol is two bf16
    units in the last place, atol_rms the path's 2e-2 taken relative to the row's own size.
    Per row: ||out - ref|| <= rel_l2 * ||ref||."""
    o, r = out.float(), ref.float()
    if o.shape != r.shape:
        return {"shape": (tuple(o.shape), tuple(r.shape))}
    bad = {}
    if not torch.isfinite(o).all():
        bad["non_finite"] = int((~torch.isfinite(o)).sum())
    rms = row_rms(r)
    err = (o - r).abs()
    over = err > atol_rms * rms + rtol * r.abs()
    if over.any():
        bad["elements"] = int(over.sum())
        bad["worst_over_rms"] = float((err / rms.clamp_min(1e-30)).max())
    l2 = (o - r).pow(2).sum(-1).sqrt()
    ref_l2 = r.pow(2).sum(-1).sqrt()
    rows = l2 > rel_l2 * ref_l2
    if rows.any():
        bad["rows"] = int(rows.sum())
        bad["worst_rel_l2"] = float((l2 / ref_l2.clamp_min(1e-30)).max())
    return bad


def assert_scale_free(out: torch.Tensor, ref: torch.Tensor, what: str = "output", **kw) -> None:
    bad = scale_free_violations(out, ref, **kw)
    assert not bad, f"{what}: scale-free comparison failed: {bad}"


def assert_attention_close(out: torch.Tensor, ref: torch.Tensor, lse: torch.Tensor = None,
                           ref_lse: torch.Tensor = None, what: str = "output") -> None:
    """The stated tolerance, the scale-free check and, when given, the row log-sum-exp
    against the oracle's (which pins QK^T, the mask and the softmax sums on their own)."""
    torch.testing.assert_close(out.float(), ref.float(), **TOL)
    assert_scale_free(out, ref, what)
    if lse is not None:
        torch.testing.assert_close(lse.float(), ref_lse.float(), **LSE_TOL)
