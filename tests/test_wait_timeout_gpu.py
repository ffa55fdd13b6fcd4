"""The failure-detection path of the kernels: a device wait that runs out.

Every wait in the library's kernels is bounded (fluke_b200/csrc/sm100_ptx.cuh: mbar_wait on an
mbarrier, wait_counter on a counter another CTA increments). When the budget is spent the wait
records TIMEOUT | site << 8 in the device status word, raises the CTA's abort flag (and, for
counters, the launch's global abort word so that the other CTAs leave their loops too) and
returns false; the kernel then drains and exits, the context stays usable and the host reads
the word. The other GPU tests only ever see the word clear; here test-only kernels
(tests/csrc/wait_probe.cu, built into lib/libfluke_waitprobe.so) call the SAME wait routines on
a barrier nobody arrives at and a counter nobody increments, with a budget of about a
millisecond. Nothing faults, traps or hangs.
"""
import ctypes
import os

import pytest
import torch

from conftest import ROOT

pytestmark = pytest.mark.gpu
DEV = "cuda"
TIMEOUT = 1  # FLUKE_SM100_STATUS_TIMEOUT
LIMIT = 2_000_000  # cycles: about a millisecond at B200 clocks


@pytest.fixture(scope="module")
def probe():
    path = os.path.join(ROOT, "lib", "libfluke_waitprobe.so")
    if not os.path.isfile(path):
        from fluke_b200 import lib
        lib.build()
    p = ctypes.CDLL(path)
    P, I, U, LL = ctypes.c_void_p, ctypes.c_int, ctypes.c_uint, ctypes.c_longlong
    p.fluke_probe_wait_mbar.restype, p.fluke_probe_wait_mbar.argtypes = I, [I, LL, U, P, P]
    p.fluke_probe_wait_counter.restype, p.fluke_probe_wait_counter.argtypes = I, [P, U, LL, U, P, P]
    p.fluke_probe_read_status.restype, p.fluke_probe_read_status.argtypes = I, [ctypes.POINTER(U), I]
    return p


def _status(probe, reset=True):
    v = ctypes.c_uint(0)
    assert probe.fluke_probe_read_status(ctypes.byref(v), 1 if reset else 0) == 0
    return v.value


def test_mbarrier_wait_that_nobody_completes_gives_up_and_reports_its_site(probe):
    out = torch.zeros(3, dtype=torch.int64, device=DEV)
    assert _status(probe) == 0
    # a barrier that has been arrived at: the wait returns at once, nothing is recorded
    assert probe.fluke_probe_wait_mbar(1, LIMIT, 0x41, out.data_ptr(), None) == 0
    torch.cuda.synchronize()
    assert out.tolist()[:2] == [1, 0] and _status(probe) == 0
    # nobody arrives: the wait spends its budget, raises the abort flag and returns false
    assert probe.fluke_probe_wait_mbar(0, LIMIT, 0x41, out.data_ptr(), None) == 0
    torch.cuda.synchronize()
    ok, abort, cycles = out.tolist()
    assert ok == 0 and abort == 1
    assert LIMIT < cycles < 50 * LIMIT            # it waited for its budget, not for ever
    assert _status(probe, reset=False) == TIMEOUT | (0x41 << 8)
    # the word keeps the FIRST failure until it is read with reset
    assert probe.fluke_probe_wait_mbar(0, LIMIT, 0x42, out.data_ptr(), None) == 0
    torch.cuda.synchronize()
    assert _status(probe) == TIMEOUT | (0x41 << 8)
    assert _status(probe) == 0
    # the context is still usable
    assert float(torch.ones(4, device=DEV).sum()) == 4.0


def test_counter_wait_gives_up_raises_the_global_abort_word_and_obeys_it(probe):
    out = torch.zeros(3, dtype=torch.int64, device=DEV)
    words = torch.zeros(2, dtype=torch.int32, device=DEV)      # [counter, global abort word]
    assert _status(probe) == 0
    words[0] = 5
    assert probe.fluke_probe_wait_counter(words.data_ptr(), 5, LIMIT, 0x51, out.data_ptr(), None) == 0
    torch.cuda.synchronize()
    assert out.tolist()[:2] == [1, 0] and words.tolist() == [5, 0] and _status(probe) == 0
    # the counter never reaches the target
    assert probe.fluke_probe_wait_counter(words.data_ptr(), 6, LIMIT, 0x51, out.data_ptr(), None) == 0
    torch.cuda.synchronize()
    ok, abort, cycles = out.tolist()
    assert ok == 0 and abort == 1 and LIMIT < cycles < 50 * LIMIT
    assert words.tolist() == [5, 1]                               # the other CTAs of a launch would see this
    assert _status(probe) == TIMEOUT | (0x51 << 8)
    # a CTA that finds the global abort word raised leaves at once and records nothing of its own
    assert probe.fluke_probe_wait_counter(words.data_ptr(), 6, 400 * LIMIT, 0x52, out.data_ptr(), None) == 0
    torch.cuda.synchronize()
    ok, abort, cycles = out.tolist()
    assert ok == 0 and abort == 1 and cycles < LIMIT
    assert _status(probe) == 0
