"""Error measures shared by the GPU parity tests.

A 16-bit result is compared with an fp32 reference through two normalised figures, both taken
against the reference tensor's OWN magnitude (never against max(1, magnitude): gradients of the
benchmark distribution are of order 1e-3, so an absolute floor would accept an all-zero result):

* ``max_rel``  = max|x - ref| / max|ref|       bound: 2e-2 (bf16), 5e-3 (fp16)
* ``rms_rel``  = ||x - ref||_2 / ||ref||_2     bound: 2e-2 (bf16), 5e-3 (fp16)

The second one makes the many small late-row elements count, which a max-abs figure dominated by a
few large early rows does not.
"""
import torch

MAX_REL = {torch.bfloat16: 2e-2, torch.float16: 5e-3, torch.float32: 1e-4}
RMS_REL = {torch.bfloat16: 2e-2, torch.float16: 5e-3, torch.float32: 1e-4}


def errors(got: torch.Tensor, ref: torch.Tensor, zero_below: float = 0.0):
    """(max_rel, rms_rel, max|ref|) of ``got`` against ``ref`` (both moved to fp32 on the reference's device).

    ``zero_below``: a reference whose largest element is below this is the oracle's fp32 rounding noise around a
    gradient that is exactly zero (a query that attends a single pair); it is compared as zero."""
    ref = ref.detach().float()
    got = got.detach().float().to(ref.device)
    mag = float(ref.abs().max())
    if mag < zero_below:
        z = float(got.abs().max())
        ok = z <= zero_below
        return (0.0 if ok else float("inf")), (0.0 if ok else float("inf")), 0.0
    nrm = float(ref.norm())
    diff = got - ref
    if mag == 0.0:
        # nothing attends anywhere: the result has to be exactly zero as well
        z = float(diff.abs().max())
        return (0.0 if z == 0.0 else float("inf")), (0.0 if z == 0.0 else float("inf")), 0.0
    return float(diff.abs().max()) / mag, float(diff.norm()) / nrm, mag


def assert_close(name: str, got: torch.Tensor, ref: torch.Tensor, dtype, scale: float = 1.0, report=None,
                 zero_below: float = 0.0):
    """Asserts both normalised bounds for ``dtype`` (times ``scale`` where a test documents why)."""
    assert torch.isfinite(got.float()).all(), f"{name}: non-finite values"
    max_rel, rms_rel, mag = errors(got, ref, zero_below)
    if report is not None:
        report[name] = (max_rel, rms_rel, mag)
    assert max_rel <= MAX_REL[dtype] * scale, f"{name}: max|err|/max|ref| = {max_rel:.3e} (max|ref| = {mag:.3e})"
    assert rms_rel <= RMS_REL[dtype] * scale, f"{name}: rms err / rms ref = {rms_rel:.3e} (max|ref| = {mag:.3e})"
    return max_rel, rms_rel


def fmt(report: dict) -> str:
    return "  ".join(f"{k}: max {v[0]:.2e} rms {v[1]:.2e} (|ref| {v[2]:.1e})" for k, v in report.items())
