"""A bounded device-side wait that runs out, on purpose and without a fault.

Every tensor-core kernel waits on its mbarriers through one bounded wait (``mbar_wait_limit``): after the limit the
CTA records a status bit, releases its tensor memory and returns.  ``tritt_selftest_wait_expiry`` runs exactly that
path in a one-CTA kernel whose producer can be told to skip its arrival, with the limit passed in (a few hundred
thousand ticks, i.e. well under a millisecond).  Checked here: the call returns, the status word is set, the context
stays usable (the next ordinary call is correct), and the Python layer raises at the next entry point."""
import pytest
import torch

from flash_trittention import _native
from oracle import trittention_oracle as orc

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
TICKS = 300_000


def _expiry(skip):
    st = _native.status_word(DEV)
    rc = _native.lib().tritt_selftest_wait_expiry(int(skip), TICKS, st.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0, _native.lib().tritt_last_error()


def _small_forward_is_correct():
    B, N, T, D = 1, 2, 96, 64
    q, k1, k2, v1, v2, _ = orc.make_inputs(B, N, T, D, scale=0.5, seed=3, dtype=torch.bfloat16)
    t = [x.to(DEV) for x in (q, k1, k2, v1, v2)]
    o, lse = torch.empty_like(t[0]), torch.empty(B, N, T, device=DEV)
    _native.tdp_fwd(*t, o, lse, 1 / D, True, None, None, None, None)
    torch.cuda.synchronize()
    z_ref, _ = orc.tdp_forward(*[x.float() for x in (q, k1, k2, v1, v2)], 1 / D, True)
    assert float((o.float().cpu() - z_ref).abs().max()) <= 2e-2 * float(z_ref.abs().max())


def test_wait_that_is_satisfied_leaves_the_status_clear():
    assert _native.read_status(DEV) == 0
    _expiry(skip=False)
    assert _native.read_status(DEV) == 0


def test_wait_that_runs_out_sets_the_status_and_the_context_survives():
    assert _native.read_status(DEV) == 0
    _expiry(skip=True)
    assert _native.read_status(DEV) == 128  # synchronises, returns the word and clears it
    _small_forward_is_correct()
    assert _native.read_status(DEV) == 0


def test_python_entry_points_raise_after_a_time_out():
    assert _native.read_status(DEV) == 0
    _expiry(skip=True)
    torch.cuda.synchronize()
    with pytest.raises(_native.TrittError, match="gave up waiting"):
        _small_forward_is_correct()   # the cheap check at the entry of tdp_fwd sees the word
    _small_forward_is_correct()       # the word was cleared by the raise: the next call runs
    _expiry(skip=True)
    with pytest.raises(_native.TrittError, match="wait-expiry self-test"):
        _native.check_status(DEV)     # the synchronising form
    assert _native.read_status(DEV) == 0


def test_limit_is_validated_on_the_host():
    assert _native.lib().tritt_selftest_wait_expiry(1, 0, None, None) < 0
