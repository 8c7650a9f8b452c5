"""The give-up path of the kernels' bounded waits, made to run out on purpose.

Every spin in the kernels is bounded; a wait that gives up writes a code into the
device status word, raises a CTA-wide abort flag so that the CTA's other waits
return too, and the kernel returns normally.  Here a one-CTA self-test kernel
waits on a barrier that nothing arrives at, with a limit of two milliseconds.
Nothing faults, traps or spins without bound, and the context stays usable: a
normal forward right afterwards must pass.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_wait_runs_out_and_context_survives():
    import _evoattn
    from oracle import evo_ref
    from _util import assert_parity, oracle_on_rounded, run_layer

    _evoattn.device_status()                       # clean before
    released = torch.zeros(1, dtype=torch.int32, device="cuda")
    _evoattn.selftest_wait_timeout(2_000_000, released, torch.cuda.current_stream().cuda_stream)
    with pytest.raises(_evoattn.EvoAttnError) as ei:
        _evoattn.device_status()
    assert ei.value.code == -8
    assert f"0x{(1 << 16) | 0xee:08x}" in str(ei.value)       # (ST_WAIT_TIMEOUT, site 0xee)
    # the CTA's other warp was released by the abort flag, not by its own (2 s) limit
    assert released.item() == 1
    # reading the status cleared it
    _evoattn.device_status()

    # the context is intact: a forward + backward right after passes parity
    q, k, v, mask, bias, d_o = evo_ref.make_inputs(1, 3, 136, 2, 32, 1.0, 1.0, "tail0to32", seed=9)
    got = run_layer(q, k, v, mask, bias, d_o)
    assert_parity(oracle_on_rounded(q, k, v, mask, bias, d_o), got, tag="after time-out")


def test_wait_limit_argument_is_checked():
    import _evoattn
    released = torch.zeros(1, dtype=torch.int32, device="cuda")
    for bad in (0, 10 ** 9):
        with pytest.raises(_evoattn.EvoAttnError) as ei:
            _evoattn.selftest_wait_timeout(bad, released, torch.cuda.current_stream().cuda_stream)
        assert ei.value.code == -1
