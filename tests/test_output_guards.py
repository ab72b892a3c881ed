"""The guard mode of the GPU suite (K3G_TEST_GUARD=1, tests/conftest.py) checked on itself: a call that stores past
the tensor it was given must be reported.  The stray store is made on purpose but lands inside the guard band the
mode puts behind every output (memory the wrapper allocated), never in anyone else's memory."""
import pytest

from conftest import make_guarded_raw

pytestmark = pytest.mark.gpu


def test_guard_mode_reports_a_store_past_the_output_and_passes_a_store_inside_it(k3g, dev):
    import torch
    guarded = make_guarded_raw(k3g)
    s = k3g.current_stream()
    buf = torch.full((4, 256), 0x11, dtype=torch.uint8, device=dev)
    assert guarded("k3g_zero_rows", buf, 256, 1, 3, s) == 0                      # rows 1 and 2 of 4: inside
    torch.cuda.synchronize()
    assert buf[0].eq(0x11).all() and buf[1:3].eq(0).all() and buf[3].eq(0x11).all()
    short = torch.full((2, 256), 0x11, dtype=torch.uint8, device=dev)            # 2 rows given, 3 rows zeroed
    with pytest.raises(AssertionError, match="k3g_zero_rows stored outside its output"):
        guarded("k3g_zero_rows", short, 256, 0, 3, s)
