"""xpkSortNoAlloc — the sort for callers that may not allocate (a frozen memory pool, a plugin that only
owns the buffers it was given, a section where cudaMalloc's device-wide synchronisation is unwelcome).

Called through the C ABI of libxpk.so twice in a row on the same device, so that the second call meets
the static scratch array as the first one left it, and compared bit for bit with the existing task-based
entry point on the same keys.  Collected last on purpose: a run that stops at the first failure has then
already been through every other test.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def _task_sort(pk, k):
    keys = torch.from_numpy(k.copy()).cuda()
    tmp = torch.empty_like(keys)
    scratch = torch.empty(pk.sort_scratch_bytes(keys.numel()), dtype=torch.uint8, device="cuda")
    t = pk.Task.sort(keys, tmp, scratch)
    t.launch(torch.cuda.current_stream().cuda_stream)
    assert t.wait().status == pk.STATUS_COMPLETED
    out = keys.cpu().numpy()
    t.destroy()
    return out


def test_no_alloc_sort_matches_task_sort_twice_in_a_row():
    from xsched_b200 import pk
    s = torch.cuda.current_stream().cuda_stream
    rng = np.random.default_rng(77)
    # second call: different size and value range, so stale histogram / look-back words would show
    cases = [rng.integers(-2**31, 2**31, size=(1 << 21) + 12345, dtype=np.int64).astype(np.int32),
             rng.integers(0, 1000, size=300_001, dtype=np.int64).astype(np.int32)]
    for k in cases:
        want = _task_sort(pk, k)
        keys = torch.from_numpy(k.copy()).cuda()
        tmp = torch.empty_like(keys)
        torch.cuda.synchronize()
        pk.sort_no_alloc(keys, tmp, s)
        torch.cuda.synchronize()
        got = keys.cpu().numpy()
        assert np.array_equal(got, want)          # integer sort: bit-exact
        assert np.array_equal(got, np.sort(k))


def test_no_alloc_sort_rejects_oversize_and_bad_pointers():
    from xsched_b200 import pk
    s = torch.cuda.current_stream().cuda_stream
    big = torch.zeros(pk.SORT_NOALLOC_MAX_KEYS + 1, dtype=torch.int32, device="cuda")
    with pytest.raises(pk.XpkError) as e:
        pk.sort_no_alloc(big, torch.empty_like(big), s)
    assert e.value.code == 7                       # XPK_ERR_TOO_LARGE
    small = torch.zeros(1024, dtype=torch.int32, device="cuda")
    with pytest.raises(pk.XpkError) as e:
        pk.sort_no_alloc(small[1:], small[1:].clone(), s)
    assert e.value.code == 2                       # XPK_ERR_ALIGNMENT
    # exactly the maximum is accepted
    exact = torch.randint(0, 2**31 - 1, (pk.SORT_NOALLOC_MAX_KEYS,), dtype=torch.int32, device="cuda")
    ref = torch.sort(exact).values
    pk.sort_no_alloc(exact, torch.empty_like(exact), s)
    torch.cuda.synchronize()
    assert torch.equal(exact, ref)
