"""The exchange wait is bounded: when a peer never publishes (here: a flag word nothing sets), the wait
kernel gives up after its time limit, reports status 7, marks the flag words, and later waits on the same
words return at once.  No fault, trap or endless loop is involved: the kernel polls a word and returns."""

import time

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_exchange_wait_expires_and_then_gives_up_at_once(lib_built):
    from t81lib_b200 import _capi
    assert _capi.device_available(), _capi.last_error()
    dev = torch.device("cuda", 0)
    _capi.kernel_status(reset=True)
    words = torch.zeros(_capi.SYNC_WORDS, dtype=torch.int32, device=dev)
    words[1] = 1  # this rank has completed one exchange; the only "peer" has published none
    stream = torch.cuda.current_stream(dev).cuda_stream
    torch.cuda.synchronize(dev)
    t0 = time.time()
    _capi.check(_capi.lib.t81b200_exchange_wait(words.data_ptr(), 1, stream))
    torch.cuda.synchronize(dev)
    first = time.time() - t0
    assert 0.2 < first < 60.0          # it waited, and it stopped by itself
    assert int(words[2].item()) == 1   # marked
    assert _capi.kernel_status(reset=True) == 7
    t0 = time.time()
    _capi.check(_capi.lib.t81b200_exchange_wait(words.data_ptr(), 1, stream))
    torch.cuda.synchronize(dev)
    assert time.time() - t0 < 0.2      # no second time limit
    assert _capi.kernel_status(reset=True) == 7
    # a wait whose flag is there passes and leaves the status clean
    words.zero_()
    words[1] = 3
    words[16] = 3
    _capi.check(_capi.lib.t81b200_exchange_wait(words.data_ptr(), 1, stream))
    torch.cuda.synchronize(dev)
    assert _capi.kernel_status(reset=True) == 0
