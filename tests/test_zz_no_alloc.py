"""The allocation-free boundary entry point (gtok_x_boundaries_noalloc) against the regular
path (stage + replay + gtok_x_read_boundaries).  It exists for hosts that cannot call
cudaMalloc at the moment they need pre-token boundaries (a framework-owned memory pool,
a fixed set of plug-in buffers); here torch plays that host and owns the text and the
output buffer.  Bits are integers: the two results must be identical, and identical to
the pre-token starts of the CPU oracle, on two calls in a row (the second reuses the
library's built-in working memory with the first call's leftovers in it)."""
import ctypes

import numpy as np
import pytest

from conftest import tiny_vocab

pytestmark = pytest.mark.gpu


def _regular(g, data):
    g.stage(data)
    g.replay()
    return g.boundaries(len(data))


def _noalloc(g, data):
    import torch
    n = len(data)
    padded = np.zeros((n + 15) // 16 * 16, dtype=np.uint8)
    padded[:n] = np.frombuffer(data, dtype=np.uint8)
    text = torch.from_numpy(padded).cuda()
    words = (n + 4095) // 4096 * 128
    out = torch.full((words,), 0x5A5A5A5A, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    r = g.lib.gtok_x_boundaries_noalloc(g.handle, ctypes.c_void_p(text.data_ptr()), n, ctypes.c_void_p(out.data_ptr()), None)
    assert r == 0, g.lib.gtok_x_last_error()
    bits = np.unpackbits(out.cpu().numpy().view(np.uint8), bitorder="little")[:n]
    return np.nonzero(bits)[0].astype(np.uint32)


def test_noalloc_boundaries_match_regular_path_twice(built):
    from graphtok_b200 import GTok, synth
    g = GTok(tiny_vocab("llama3"), max_bytes=1 << 20)
    try:
        first = synth.text(4, 21, 700000)[:650000].decode("utf-8", "ignore").encode()    # long digit runs: exercises the look-back states
        second = synth.text(1, 22, 300000)[:123457].decode("utf-8", "ignore").encode()   # shorter: leftovers from the first call remain
        import oracle_lib
        import torch
        oracle = oracle_lib.Oracle(tiny_vocab("llama3"))
        for data in (first, second):
            dev_before = torch.cuda.current_device()
            got = _noalloc(g, data)
            assert torch.cuda.current_device() == dev_before
            assert np.array_equal(got, _regular(g, data))
            _, starts = oracle.encode_normalized(data, want_starts=True)
            # (a boundary bit on a stray continuation byte at the very start carries no pre-token; these texts have none)
            assert np.array_equal(got, starts)
        # beyond the fixed working memory: refused, with a message, and nothing run
        r = g.lib.gtok_x_boundaries_noalloc(g.handle, ctypes.c_void_p(256), (4 << 20) + 1, ctypes.c_void_p(256), None)
        assert r == -3 and b"exceeds" in g.lib.gtok_x_last_error()
    finally:
        g.close()
