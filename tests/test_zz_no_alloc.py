"""fortis_checksum_noalloc: the checksum entry for callers that cannot allocate device memory (fixed-budget hosts,
code between latency-critical launches).  It must agree with fortis_checksum, call
after call, although both of its calls reuse the same fixed scratch array.  Collected last on purpose."""
import ctypes

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

import fortis_b200


def test_no_alloc_checksum_matches_allocating_entry_twice_in_a_row():
    L = fortis_b200.load()
    rng = np.random.default_rng(17)
    out = torch.zeros(1, dtype=torch.float64, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    # two different arrays, back to back: the second call must not see the first call's partials
    for i, (n, dt) in enumerate(((3_000_001, torch.float32), (70_000, torch.float64))):
        a = torch.from_numpy(rng.normal(size=n)).to(dt).cuda()
        want = ctypes.c_double()
        assert L.fortis_checksum(a.data_ptr(), n, 0 if dt == torch.float32 else 1, ctypes.byref(want)) == 0
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        assert L.fortis_checksum_noalloc(a.data_ptr(), n, 0 if dt == torch.float32 else 1, out.data_ptr(), stream) == 0
        torch.cuda.synchronize()
        if i == 1:
            # the property in the entry's name: once the first call has resolved the array's address, a call leaves
            # the device's free memory exactly as it found it
            assert torch.cuda.mem_get_info()[0] == free_before
        got = float(out.item())
        # same tolerance as the other checksum tests: the two entries partition the sum differently
        assert abs(got - want.value) <= 1e-9 * max(1.0, float(a.abs().double().sum()))
    # empty input and the size limit
    assert L.fortis_checksum_noalloc(a.data_ptr(), 0, 0, out.data_ptr(), stream) == 0
    torch.cuda.synchronize()
    assert float(out.item()) == 0.0
    assert L.fortis_checksum_noalloc(a.data_ptr(), (1 << 28) + 1, 0, out.data_ptr(), stream) == -2
