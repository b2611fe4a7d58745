"""The give-up path of a bounded device-side wait, on a flag that nothing sets (no fault, no hang: the wait is
limited to 0.2 s, the kernel returns normally and the context stays usable)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_wait_on_an_unset_flag_runs_out_and_reports():
    from oslo_b200 import ops
    from oslo_b200.utils.watchdog import OsloCommTimeout, raise_if_device_error
    ext = ops.load_ext(required=True)
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    ext.error_word(flag).zero_()
    waited = ext.wait_probe(flag, 1, 200.0)            # nobody ever writes 1
    torch.cuda.synchronize()
    assert 0.15e9 < int(waited.item()) < 0.9e9
    with pytest.raises(OsloCommTimeout):
        raise_if_device_error(flag)
    assert int(ext.error_word(flag).item()) == 0       # reported once, then cleared
    # a flag that is already set returns at once and leaves no error; the context is still usable
    flag.fill_(3)
    waited = ext.wait_probe(flag, 2, 200.0)
    torch.cuda.synchronize()
    assert int(waited.item()) < 0.05e9 and int(ext.error_word(flag).item()) == 0
    assert float((torch.ones(8, device="cuda") * 2).sum()) == 16.0
