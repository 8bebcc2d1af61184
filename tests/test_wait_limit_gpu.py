"""A bounded device-side wait that actually runs out — without a fault, a trap or a hang.  A loopback exchange handle
stands in for rank 0 of a group of two; the packets of rank 1's column block are never sent (det_debug_xchg_drop) and the
wait limit is set to about 2 ms of SM clock.  The gather kernel must return, the error word must say "wait expired", the
missing values must come back as zeros, and after det_clear_error the same handle must work again."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ERR_WAIT_EXPIRED = 1


def test_exchange_wait_runs_out_and_the_library_recovers(libs):
    d = libs.cuda()
    assert d.det_init() == 0
    m, slice_ = 2, 256
    h = d.det_xchg_create(16 * m * 2 * slice_ + 4096, 0, 2)
    d.det_xchg_open_loopback(h)
    local = (np.arange(m * slice_, dtype=np.float32) + 1.0)
    dl, df = d.det_malloc(local.nbytes), d.det_malloc(2 * local.nbytes)
    try:
        d.det_memcpy(dl, local.ctypes.data, local.nbytes, None)
        full = np.zeros((m, 2 * slice_), np.float32)

        def gather():
            d.det_memset(df, 0xFF, full.nbytes, None)
            d.det_xchg_all_gather(h, dl, df, m, slice_, None)
            d.det_memcpy(full.ctypes.data, df, full.nbytes, None)
            d.det_sync()
            return full.copy()

        want = np.concatenate([local.reshape(m, slice_)] * 2, axis=1)     # loopback: both column blocks carry the local slice
        assert np.array_equal(gather(), want)
        assert d.det_last_error() == 0

        d.det_debug_set_wait_limit(4_000_000)     # ~2 ms
        d.det_debug_xchg_drop(h, 1)
        got = gather()                            # returns: the wait for block 1 gives up
        assert d.det_last_error() == ERR_WAIT_EXPIRED
        assert np.array_equal(got[:, :slice_], want[:, :slice_])
        assert (got[:, slice_:] == 0).all()

        # the error is sticky until cleared: a later exchange does not poll, it returns zeros for what has not arrived
        d.det_debug_xchg_drop(h, -1)
        d.det_clear_error()
        d.det_debug_set_wait_limit(0)
        assert d.det_last_error() == 0
        for _ in range(3):                         # both staging slots are used again
            assert np.array_equal(gather(), want)
        assert d.det_last_error() == 0
    finally:
        d.det_debug_set_wait_limit(0)
        d.det_clear_error()
        d.det_free(dl)
        d.det_free(df)
        d.det_xchg_destroy(h)
