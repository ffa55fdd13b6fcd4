"""Host-side state of the C boundary, exercised without a GPU: the launch stream and the LSTM
form selection are per host thread, and the table of re-ordered fp8 weights (reference-ABI fp8
entry points, include/fluke/fluke.h) survives more weights than it has slots, a failing
re-ordering and concurrent callers. The table's device calls are replaced by counting fakes
through fluke_fp8_cache_test_hooks."""
import ctypes
import threading

import pytest

P, I, Z = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t
MALLOC = ctypes.CFUNCTYPE(I, ctypes.POINTER(P), Z)
FREE = ctypes.CFUNCTYPE(I, P)
UNSHUFFLE = ctypes.CFUNCTYPE(I, P, P, I, I, P)
DEVICE = ctypes.CFUNCTYPE(I)


def test_launch_stream_is_per_host_thread(flib):
    """Two threads set different streams and each reads back its own; a new thread starts on the
    legacy default stream (NULL) whatever the others set."""
    seen = {}
    barrier = threading.Barrier(2)

    def worker(name, value):
        assert flib.fluke_get_stream() is None
        flib.fluke_set_stream(value)
        barrier.wait()          # both have set theirs
        seen[name] = flib.fluke_get_stream()
        barrier.wait()

    flib.fluke_set_stream(0x1000)
    ts = [threading.Thread(target=worker, args=("a", 0x2000)), threading.Thread(target=worker, args=("b", 0x3000))]
    [t.start() for t in ts]
    [t.join() for t in ts]
    assert seen == {"a": 0x2000, "b": 0x3000}
    assert flib.fluke_get_stream() == 0x1000
    flib.fluke_set_stream(None)


def test_lstm_form_selection_is_per_host_thread(flib):
    got = {}

    def worker():
        got["fresh"] = flib.fluke_sm100_lstm_last_form()   # nothing run on this thread yet
        flib.fluke_set_lstm_persistent(0)

    flib.fluke_set_lstm_persistent(2)
    t = threading.Thread(target=worker)
    t.start(); t.join()
    assert got["fresh"] == -1
    flib.fluke_set_lstm_persistent(1)


class FakeDevice:
    """Counting stand-ins for cudaMalloc / cudaFree / the re-ordering launch."""

    def __init__(self):
        self.next, self.live, self.freed, self.unshuffles, self.fail_unshuffle, self.device = 0x10000, set(), [], 0, False, 0
        self.lock = threading.Lock()
        self.c_malloc, self.c_free = MALLOC(self._malloc), FREE(self._free)
        self.c_unshuffle, self.c_device = UNSHUFFLE(self._unshuffle), DEVICE(lambda: self.device)

    def _malloc(self, out, nbytes):
        with self.lock:
            self.next += 0x1000
            self.live.add(self.next)
            out[0] = self.next
        return 0

    def _free(self, ptr):
        with self.lock:
            self.live.discard(ptr)
            self.freed.append(ptr)
        return 0

    def _unshuffle(self, dst, src, n, k, stream):
        with self.lock:
            self.unshuffles += 1
        return 700 if self.fail_unshuffle else 0


@pytest.fixture
def fake(flib):
    hooks = flib.fluke_fp8_cache_test_hooks
    hooks.restype, hooks.argtypes = None, [MALLOC, FREE, UNSHUFFLE, DEVICE]
    fd = FakeDevice()
    flib.fluke_fp8_release_weight(None)
    hooks(fd.c_malloc, fd.c_free, fd.c_unshuffle, fd.c_device)
    yield fd
    flib.fluke_fp8_release_weight(None)
    hooks(MALLOC(0), FREE(0), UNSHUFFLE(0), DEVICE(0))   # NULL pointers: back to the real calls


def test_fp8_weight_table_takes_more_weights_than_slots(flib, fake):
    """65 weights into 64 slots: every one is prepared, the oldest copy is freed to make room, a
    weight seen before is found again without another allocation, and release drops what is left."""
    for i in range(65):
        assert flib.fluke_fp8_prepare_weight(0x900000 + 16 * i, 2048, 512) == 0
    assert fake.unshuffles == 65 and len(fake.live) == 64 and len(fake.freed) == 1
    assert flib.fluke_fp8_prepare_weight(0x900000 + 16 * 64, 2048, 512) == 0      # the newest: cached
    assert fake.unshuffles == 65
    assert flib.fluke_fp8_prepare_weight(0x900000, 2048, 512) == 0                # the evicted one: made again
    assert fake.unshuffles == 66 and len(fake.live) == 64
    assert flib.fluke_fp8_release_weight(0x900000) == 1 and len(fake.live) == 63
    assert flib.fluke_fp8_release_weight(None) == 63 and not fake.live


def test_fp8_weight_table_keys_on_device_and_shape_and_frees_on_failure(flib, fake):
    assert flib.fluke_fp8_prepare_weight(0xA000, 1536, 512) == 0
    assert flib.fluke_fp8_prepare_weight(0xA000, 2048, 512) == 0     # same address, other shape: its own copy
    fake.device = 1
    assert flib.fluke_fp8_prepare_weight(0xA000, 1536, 512) == 0     # same address on another device
    assert fake.unshuffles == 3 and len(fake.live) == 3
    fake.fail_unshuffle = True
    assert flib.fluke_fp8_prepare_weight(0xB000, 1536, 512) != 0     # the launch fails: nothing kept, nothing leaked
    assert len(fake.live) == 3
    fake.fail_unshuffle = False
    assert flib.fluke_fp8_prepare_weight(0xB000, 1536, 512) == 0
    assert flib.fluke_fp8_prepare_weight(0xB000, 1530, 512) != 0     # N not a multiple of 16
    assert flib.fluke_fp8_prepare_weight(None, 1536, 512) != 0


def test_fp8_weight_table_with_concurrent_callers(flib, fake):
    """Eight threads prepare the same 16 weights at once: one copy per weight."""
    def worker():
        for i in range(16):
            assert flib.fluke_fp8_prepare_weight(0xC00000 + 64 * i, 2048, 512) == 0

    ts = [threading.Thread(target=worker) for _ in range(8)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    assert fake.unshuffles == 16 and len(fake.live) == 16
