import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "kern-k3_b200"))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
sys.path.insert(0, os.path.join(ROOT, "tests"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 box)")


@pytest.fixture(scope="session")
def k3o():
    import k3o as mod
    mod.lib()
    return mod


@pytest.fixture(scope="session")
def k3g():
    """The C-ABI binding; building the library first if this is a fresh checkout."""
    lib = os.path.join(ROOT, "kern-k3_b200", "lib", "libk3g.so")
    if not os.path.exists(lib):
        sys.path.insert(0, os.path.join(ROOT, "kern-k3_b200"))
        import build
        build.build()
    import k3g as mod
    if os.environ.get("K3G_TEST_GUARD") == "1":
        _install_output_guards(mod)
    return mod


def _install_output_guards(mod):
    guarded_raw = make_guarded_raw(mod)

    def guarded_call(name, *args):
        rc = guarded_raw(name, *args)
        if rc != 0:
            raise mod.K3gError(name, rc)

    mod.raw, mod.call = guarded_raw, guarded_call


def make_guarded_raw(mod, guard_bytes=4096, max_bytes=1 << 28):
    """Opt-in mode of the GPU suite (K3G_TEST_GUARD=1): every device tensor a test passes for a non-const pointer
    parameter is replaced, for the duration of the call, by a view into the middle of a larger buffer whose first and
    last `guard_bytes` hold a pattern; the tensor's content is copied in before the call (in/out arguments keep their
    meaning) and back afterwards, and the call fails if either guard changed: a store outside the output it was
    given.  Left alone: entries that address memory through peer tables (the tables name the original buffers), calls
    made while the stream is being captured into a graph (the check synchronises), and calls whose output tensors
    overlap one another (two halves of one buffer)."""
    import torch
    plain_raw = mod.raw

    def guarded_raw(name, *args):
        spec = mod.PROTOTYPES[name]
        if len(args) != len(spec) or any("peer" in n for _, n in spec) or name.startswith(("k3g_peer_", "k3g_wait_status", "k3g_device_sms")):
            return plain_raw(name, *args)
        if torch.cuda.is_available() and torch.cuda.is_current_stream_capturing():
            return plain_raw(name, *args)
        outs = [a for (ty, _), a in zip(spec, args) if "*" in ty and "const" not in ty and isinstance(a, torch.Tensor) and a.is_cuda]
        spans = sorted((a.data_ptr(), a.data_ptr() + a.numel() * a.element_size()) for a in outs)
        if any(spans[i][1] > spans[i + 1][0] for i in range(len(spans) - 1)):
            return plain_raw(name, *args)
        swapped, new_args = [], list(args)
        for i, ((ty, pname), a) in enumerate(zip(spec, args)):
            if "*" not in ty or "const" in ty or not isinstance(a, torch.Tensor) or not a.is_cuda or not a.is_contiguous():
                continue
            nbytes = a.numel() * a.element_size()
            if nbytes == 0 or nbytes > max_bytes:
                continue
            buf = torch.empty(nbytes + 2 * guard_bytes, dtype=torch.uint8, device=a.device)
            buf[:guard_bytes] = 0xA5
            buf[guard_bytes + nbytes:] = 0xA5
            view = buf[guard_bytes:guard_bytes + nbytes]
            view.copy_(a.view(torch.uint8).reshape(-1))
            new_args[i] = view
            swapped.append((a, buf, view, nbytes, pname))
        rc = plain_raw(name, *new_args)
        for a, buf, view, nbytes, pname in swapped:
            a.view(torch.uint8).reshape(-1).copy_(view)
            ok = bool((buf[:guard_bytes] == 0xA5).all()) and bool((buf[guard_bytes + nbytes:] == 0xA5).all())
            assert ok, "%s stored outside its output `%s` (%d bytes)" % (name, pname, nbytes)
        return rc

    return guarded_raw


@pytest.fixture(scope="session")
def dev():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")
