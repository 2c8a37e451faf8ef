"""Parity of the preemptible sm_100a kernels (through the C ABI of libxpk.so) against the CPU oracle.

Bit-exact for triad / vector add / sort; GEMM within a stated tolerance of an fp64 product and
bit-exact between preempted and unpreempted runs.  Preemption is forced deterministically: the
first launch is confined to a few SMs so that the flag, raised right after the launch call
returns, always lands while most of the task is still unclaimed.
"""
import math

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def pk():
    from xsched_b200 import pk as _pk
    return _pk


@pytest.fixture(scope="module")
def ok():
    from oracle import kernels as _ok
    return _ok


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _run_to_completion(task, pk, max_rounds=10000):
    """Launch until COMPLETED, clearing the flag between rounds.  Returns the number of launches."""
    rounds = 0
    while True:
        task.launch(_stream())
        info = task.wait()
        rounds += 1
        assert info.status in (pk.STATUS_COMPLETED, pk.STATUS_PREEMPTED), f"status {info.status} err {info.error:#x}"
        if info.status == pk.STATUS_COMPLETED:
            return rounds
        task.set_flag(0)
        torch.cuda.synchronize()
        assert rounds < max_rounds


def _preempt_once(task, pk, sm_limit):
    """Start on `sm_limit` SMs, raise the flag at once, wait for the kernel to stop."""
    task.launch(_stream(), sm_limit=sm_limit)
    task.set_flag(1)
    info = task.wait()
    torch.cuda.synchronize()
    task.set_flag(0)
    torch.cuda.synchronize()
    return info


# --------------------------------------------------------------------------- triad / vecadd
@pytest.mark.parametrize("n", [1, 3, 4, 4095, 4096, 4097, 16384 + 5, (1 << 20) + 3, 1 << 24])
def test_triad_matches_oracle(pk, ok, n):
    g = torch.Generator(device="cpu").manual_seed(3)
    b = (torch.rand(n, generator=g) * 2 - 1).float()
    c = (torch.rand(n, generator=g) * 2 - 1).float()
    s = 1.7
    want = ok.triad(b.numpy(), c.numpy(), s)
    bd, cd = b.cuda(), c.cuda()
    for flags in (pk.FLAG_NONE, pk.FLAG_NON_PREEMPTIBLE):
        a = torch.zeros(n, device="cuda")
        t = pk.Task.triad(a, bd, cd, s, flags=flags)
        assert _run_to_completion(t, pk) == 1
        got = a.cpu().numpy()
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
        t.destroy()


@pytest.mark.parametrize("n", [7, 8192, (1 << 22) + 1])
def test_vecadd_matches_oracle(pk, ok, n):
    g = torch.Generator(device="cpu").manual_seed(4)
    a = (torch.rand(n, generator=g) * 2 - 1).float()
    b = (torch.rand(n, generator=g) * 2 - 1).float()
    want = ok.vecadd(a.numpy(), b.numpy())
    c = torch.zeros(n, device="cuda")
    t = pk.Task.vecadd(c, a.cuda(), b.cuda())
    _run_to_completion(t, pk)
    assert np.array_equal(c.cpu().numpy().view(np.uint32), want.view(np.uint32))
    t.destroy()


def test_triad_preempt_resume_bit_exact(pk, ok):
    n = (1 << 26) + 1234
    g = torch.Generator(device="cpu").manual_seed(5)
    b = (torch.rand(n, generator=g) * 2 - 1).float()
    c = (torch.rand(n, generator=g) * 2 - 1).float()
    want = ok.triad(b.numpy(), c.numpy(), -0.3)
    a = torch.zeros(n, device="cuda")
    t = pk.Task.triad(a, b.cuda(), c.cuda(), -0.3, tile_elems=8192)
    cuts = 0
    for _ in range(6):
        info = _preempt_once(t, pk, sm_limit=2)
        if info.status == pk.STATUS_COMPLETED:
            break
        assert info.status == pk.STATUS_PREEMPTED
        assert 0 <= info.tiles_done < info.tiles_total
        cuts += 1
    assert cuts >= 1, "the task was never caught mid-flight"
    _run_to_completion(t, pk)
    info = t.query()
    assert info.tiles_done == info.tiles_total and info.preemptions >= cuts
    assert np.array_equal(a.cpu().numpy().view(np.uint32), want.view(np.uint32))
    # relaunching a completed task does nothing and stays completed
    t.launch(_stream())
    assert t.wait().status == pk.STATUS_COMPLETED
    # reset rewinds the cursor
    a.zero_()
    t.reset(_stream())
    assert t.query().status == pk.STATUS_IDLE
    _run_to_completion(t, pk)
    assert np.array_equal(a.cpu().numpy().view(np.uint32), want.view(np.uint32))
    t.destroy()


def _free_gb():
    free, _ = torch.cuda.mem_get_info()
    return free / 2**30


@pytest.mark.parametrize("n", [1 << 31, (1 << 31) - 5])
def test_triad_2p31_elements_against_the_cpu_loop(pk, ok, n):
    """The size of the memory-bound workload configuration: 3 arrays of 2^31 fp32 (8 GiB each, byte offsets past
    2^32, so the 64-bit index path).  One forced preemption, then the WHOLE output is compared bit for bit with
    the CPU loop, chunk by chunk (the inputs are copied back from the device, so both sides see the same bits);
    the windows named below are the ones most likely to show an index that wrapped."""
    import psutil
    if _free_gb() < 30 or psutil.virtual_memory().available < 8 * 2**30:
        pytest.skip("needs 30 GB of device memory and 8 GB of host memory")
    g = torch.Generator(device="cuda").manual_seed(31)
    b = torch.rand(n, device="cuda", generator=g).mul_(2).sub_(1)
    c = torch.rand(n, device="cuda", generator=g).mul_(2).sub_(1)
    a = torch.full((n,), float("nan"), device="cuda")
    s = 0.4375
    t = pk.Task.triad(a, b, c, s)
    info = _preempt_once(t, pk, sm_limit=2)
    assert info.status == pk.STATUS_PREEMPTED and 0 <= info.tiles_done < info.tiles_total
    assert bool(torch.isnan(a[-1]))                    # the cut really left work undone
    _run_to_completion(t, pk)
    assert t.query().tiles_done == t.query().tiles_total

    def same(lo, hi):
        want = ok.triad(b[lo:hi].cpu().numpy(), c[lo:hi].cpu().numpy(), s)
        return np.array_equal(a[lo:hi].cpu().numpy().view(np.uint32), want.view(np.uint32))
    M1 = 1 << 20
    assert same(0, M1)                                  # first 1 Mi elements
    assert same((1 << 30) - M1 // 2, (1 << 30) + M1 // 2)   # straddles element 2^30 = byte offset 2^32
    assert same(n - M1 - 3, n)                          # last 1 Mi and the ragged tail
    chunk = 1 << 27
    h_gpu = h_cpu = 0
    for lo in range(0, n, chunk):
        hi = min(n, lo + chunk)
        bh, ch = b[lo:hi].cpu().numpy(), c[lo:hi].cpu().numpy()
        want = ok.triad(bh, ch, s)
        got = a[lo:hi].cpu().numpy()
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), f"chunk at {lo}"
        h_gpu = (h_gpu + ok.checksum_u32(got)) & (2**64 - 1)
        h_cpu = (h_cpu + ok.checksum_u32(want)) & (2**64 - 1)
    assert h_gpu == h_cpu                               # checksum of checksums over the full array
    t.destroy()


def test_flag_raised_before_launch_makes_no_progress(pk):
    n = 1 << 20
    a = torch.zeros(n, device="cuda")
    b = torch.ones(n, device="cuda")
    c = torch.ones(n, device="cuda")
    flag = pk.Flag()
    t = pk.Task.triad(a, b, c, 2.0, flag=flag)
    flag.set(1)
    torch.cuda.synchronize()
    t.launch(_stream())
    info = t.wait()
    assert info.status == pk.STATUS_PREEMPTED and info.tiles_done == 0
    assert float(a.abs().max()) == 0.0
    flag.set(0)
    torch.cuda.synchronize()
    _run_to_completion(t, pk)
    assert float((a - 3.0).abs().max()) == 0.0
    t.destroy()
    flag.destroy()


def test_rejects_bad_arguments(pk):
    a = torch.zeros(64, device="cuda")
    with pytest.raises(pk.XpkError) as e:
        pk.Task.triad(a[1:], a[1:], a[1:], 1.0)
    assert e.value.code == 2          # XPK_ERR_ALIGNMENT
    with pytest.raises(pk.XpkError) as e:
        pk.Task.triad(a, a, a, 1.0, tile_elems=1000)
    assert e.value.code == 1          # XPK_ERR_INVALID_VALUE
    x = torch.zeros(100, 64, device="cuda", dtype=torch.bfloat16)
    y = torch.zeros(256, 64, device="cuda", dtype=torch.bfloat16)
    z = torch.zeros(100, 256, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(pk.XpkError) as e:
        pk.Task.gemm(z, x, y)
    assert e.value.code == 4          # XPK_ERR_NOT_SUPPORTED


# --------------------------------------------------------------------------- radix sort
def _sort_buffers(pk, keys_np):
    keys = torch.from_numpy(keys_np.copy()).cuda()
    tmp = torch.empty_like(keys)
    scratch = torch.empty(pk.sort_scratch_bytes(keys.numel()), dtype=torch.uint8, device="cuda")
    return keys, tmp, scratch


@pytest.mark.parametrize("n", [1, 2, 100, 8191, 8192, 8193, 3 * 8192 + 17, (1 << 20) + 7])
@pytest.mark.parametrize("dist", ["full", "nonneg", "few"])
def test_sort_matches_oracle(pk, ok, n, dist):
    rng = np.random.default_rng(1000 + n)
    if dist == "full":
        k = rng.integers(-2**31, 2**31, size=n, dtype=np.int64).astype(np.int32)
    elif dist == "nonneg":
        k = rng.integers(0, 2**31, size=n, dtype=np.int64).astype(np.int32)
    else:
        k = rng.integers(-3, 4, size=n, dtype=np.int64).astype(np.int32)     # heavy duplicates
    want = ok.radix_sort_i32(k)
    for flags in (pk.FLAG_NONE, pk.FLAG_NON_PREEMPTIBLE):
        keys, tmp, scratch = _sort_buffers(pk, k)
        t = pk.Task.sort(keys, tmp, scratch, flags=flags)
        _run_to_completion(t, pk)
        assert np.array_equal(keys.cpu().numpy(), want)
        t.destroy()


def test_sort_16m_preempt_resume_bit_exact(pk, ok):
    n = 1 << 24
    k = np.random.default_rng(5).integers(0, 2**31, size=n, dtype=np.int64).astype(np.int32)
    want = ok.radix_sort_i32(k)
    keys, tmp, scratch = _sort_buffers(pk, k)
    t = pk.Task.sort(keys, tmp, scratch)
    cuts = 0
    for _ in range(8):
        info = _preempt_once(t, pk, sm_limit=3)
        if info.status == pk.STATUS_COMPLETED:
            break
        assert info.status == pk.STATUS_PREEMPTED, f"err {info.error:#x}"
        cuts += 1
    assert cuts >= 1
    _run_to_completion(t, pk)
    got = keys.cpu().numpy()
    assert np.array_equal(got, want)
    # sortedness + same multiset, independent of the oracle
    assert bool((torch.from_numpy(got)[1:] >= torch.from_numpy(got)[:-1]).all())
    assert ok.checksum_u32(np.sort(k)) == ok.checksum_u32(got)
    # a reset task sorts again from scratch (idempotence on sorted input)
    t.reset(_stream())
    _run_to_completion(t, pk)
    assert np.array_equal(keys.cpu().numpy(), want)
    t.destroy()


# --------------------------------------------------------------------------- GEMM
# The GEMM exists in two forms (one CTA per 256x256 tile; a pair of CTAs per 512x256 tile) that must write the same bytes.
FORMS = ["one", "pair"]


def _form_flag(pk, form):
    return {"one": pk.FLAG_GEMM_ONE_CTA, "pair": pk.FLAG_GEMM_CTA_PAIR}[form]


def _gemm_inputs(M, N, K, seed, std=1.0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    a = (torch.randn(M, K, generator=g) * std).to(torch.bfloat16)
    b = (torch.randn(N, K, generator=g) * std).to(torch.bfloat16)
    return a, b


def _check_rows(ok, c_gpu, a, b, rows):
    K = a.shape[1]
    a_bits = a.view(torch.int16).numpy().view(np.uint16)
    b_bits = b.view(torch.int16).numpy().view(np.uint16)
    ref = ok.gemm_bf16_rows(a_bits, b_bits, np.asarray(rows, dtype=np.uint32))
    got = c_gpu[rows].float().cpu().numpy().astype(np.float64)
    # bf16 output rounding (2^-9 relative, doubled) + fp32 accumulation slack
    tol = np.abs(ref) * 2.0**-8 + 1e-3 * math.sqrt(K)
    bad = np.abs(got - ref) > tol
    assert not bad.any(), f"{bad.sum()} of {bad.size} elements outside tolerance; max err {np.abs(got-ref).max()}"


@pytest.mark.parametrize("shape", [(128, 256, 64), (128, 256, 512), (256, 512, 256), (1024, 1024, 1024),
                                   (384, 768, 320), (2048, 4096, 192), (640, 256, 128), (4608, 5120, 256)])
def test_gemm_matches_oracle(pk, ok, shape):
    M, N, K = shape
    a, b = _gemm_inputs(M, N, K, seed=M + N + K)
    ad, bd = a.cuda(), b.cuda()
    outs = []
    for form in FORMS:
        for flags in (pk.FLAG_NONE, pk.FLAG_ABORT_INFLIGHT, pk.FLAG_NON_PREEMPTIBLE):
            c = torch.full((M, N), float("nan"), device="cuda", dtype=torch.bfloat16)
            t = pk.Task.gemm(c, ad, bd, flags=flags | _form_flag(pk, form))
            _run_to_completion(t, pk)
            outs.append(c)
            t.destroy()
    rows = sorted(set([0, 1, 63, 64, 127, M // 2, M - 1] + list(range(128, min(M, 136)))))
    _check_rows(ok, outs[0], a, b, rows)
    assert all(torch.equal(outs[0], o) for o in outs[1:])
    # library cross-check (different accumulation order, so only approximately equal)
    ref = (ad.float() @ bd.float().T)
    err = (outs[0].float() - ref).abs().max().item()
    assert err <= ref.abs().max().item() * 2.0**-7 + 1e-2


@pytest.mark.parametrize("form", FORMS)
@pytest.mark.parametrize("flags_name", ["tile", "abort"])
def test_gemm_preempt_resume_bit_exact(pk, ok, flags_name, form):
    M = N = K = 4096
    a, b = _gemm_inputs(M, N, K, seed=1)
    ad, bd = a.cuda(), b.cuda()
    base = torch.zeros(M, N, device="cuda", dtype=torch.bfloat16)
    t0 = pk.Task.gemm(base, ad, bd, flags=pk.FLAG_GEMM_ONE_CTA)
    _run_to_completion(t0, pk)
    t0.destroy()
    _check_rows(ok, base, a, b, [0, 777, 4095])

    flags = (pk.FLAG_ABORT_INFLIGHT if flags_name == "abort" else pk.FLAG_NONE) | _form_flag(pk, form)
    c = torch.zeros(M, N, device="cuda", dtype=torch.bfloat16)
    t = pk.Task.gemm(c, ad, bd, flags=flags)
    cuts = 0
    for _ in range(5):
        info = _preempt_once(t, pk, sm_limit=8)
        if info.status == pk.STATUS_COMPLETED:
            break
        assert info.status == pk.STATUS_PREEMPTED, f"err {info.error:#x}"
        assert info.tiles_done < info.tiles_total
        cuts += 1
    assert cuts >= 1
    _run_to_completion(t, pk)
    assert t.query().tiles_done == t.query().tiles_total
    assert torch.equal(c, base)
    t.destroy()


def _check_rows_scaled(ok, c_gpu, a, b, rows, scale):
    """Sampled rows against the fp64 product.  Tolerance: bf16 output rounding (2^-9 relative, doubled) plus
    1e-3 * sqrt(K) * scale absolute, scale = product of the operands' standard deviations (fp32 accumulation
    error is orders of magnitude below that)."""
    K = a.shape[1]
    a_bits = a.view(torch.int16).numpy().view(np.uint16)
    b_bits = b.view(torch.int16).numpy().view(np.uint16)
    ref = ok.gemm_bf16_rows(a_bits, b_bits, np.asarray(rows, dtype=np.uint32))
    got = c_gpu[rows].float().cpu().numpy().astype(np.float64)
    tol = np.abs(ref) * 2.0**-8 + 1e-3 * math.sqrt(K) * scale
    bad = np.abs(got - ref) > tol
    assert not bad.any(), f"{bad.sum()} of {bad.size} elements outside tolerance; max err {np.abs(got-ref).max()}"
    assert np.abs(ref).max() > 10 * tol.min()           # the rows are not trivially within tolerance


@pytest.mark.parametrize("form", FORMS)
@pytest.mark.parametrize("shape,b_std", [((8192, 8192, 8192), 1.0), ((16384, 14336, 4096), 0.02)],
                         ids=["8192cubed", "16384x4096_by_4096x14336_weights_0.02"])
def test_gemm_baseline_shapes_against_fp64_rows(pk, ok, shape, b_std, form):
    """The two GEMM shapes of the workload configurations (8192^3 with N(0,1) operands; the inference-shaped
    (16384x4096)(4096x14336) with weights ~ N(0, 0.02)): eleven sampled rows — first and last row of the first and
    last row-block, rows either side of the 128-row accumulator boundary — against the fp64 product, for a straight
    run and for a run cut at least three times with in-flight abort; the two runs must also agree bit for bit."""
    M, N, K = shape
    g = torch.Generator(device="cpu").manual_seed(M + K)
    a = torch.randn(M, K, generator=g).to(torch.bfloat16)
    b = (torch.randn(N, K, generator=g) * b_std).to(torch.bfloat16)
    ad, bd = a.cuda(), b.cuda()
    rows = [0, 127, 128, 255, 256, 383, 511, M // 2 + 1, M - 256, M - 129, M - 1]
    base = torch.full((M, N), float("nan"), device="cuda", dtype=torch.bfloat16)
    t0 = pk.Task.gemm(base, ad, bd, flags=pk.FLAG_ABORT_INFLIGHT | _form_flag(pk, form))
    assert _run_to_completion(t0, pk) == 1
    t0.destroy()
    assert not bool(torch.isnan(base).any())
    _check_rows_scaled(ok, base, a, b, rows, b_std)

    c = torch.full((M, N), float("nan"), device="cuda", dtype=torch.bfloat16)
    t = pk.Task.gemm(c, ad, bd, flags=pk.FLAG_ABORT_INFLIGHT | _form_flag(pk, form))
    cuts = 0
    for sm_limit in (4, 16, 64, 148, 148):
        info = _preempt_once(t, pk, sm_limit=sm_limit)
        if info.status == pk.STATUS_COMPLETED:
            break
        assert info.status == pk.STATUS_PREEMPTED, f"err {info.error:#x}"
        cuts += 1
    assert cuts >= 3
    _run_to_completion(t, pk)
    assert t.query().tiles_done == t.query().tiles_total
    assert torch.equal(c, base)
    _check_rows_scaled(ok, c, a, b, rows, b_std)
    t.destroy()


def test_sort_64m_keys_against_numpy(pk):
    """One size well above the workload's 16 Mi keys (the look-back words hold 30-bit counts): 64 Mi keys over the
    full int32 range, cut twice, against numpy's sort."""
    n = 1 << 26
    k = np.random.default_rng(64).integers(-2**31, 2**31, size=n, dtype=np.int64).astype(np.int32)
    keys, tmp, scratch = _sort_buffers(pk, k)
    t = pk.Task.sort(keys, tmp, scratch)
    for _ in range(2):
        info = _preempt_once(t, pk, sm_limit=6)
        assert info.status in (pk.STATUS_PREEMPTED, pk.STATUS_COMPLETED), f"err {info.error:#x}"
    _run_to_completion(t, pk)
    assert np.array_equal(keys.cpu().numpy(), np.sort(k))
    t.destroy()


@pytest.mark.parametrize("form", FORMS)
def test_gemm_stops_on_the_relayed_host_word_alone(pk, ok, form):
    """The flag's early-warning word in mapped host memory: a plain host store to it, with the device flag itself
    never written, must stop a running GEMM (the relay thread of its first CTA raises the flag), and the resumed
    task must give the bytes of a straight run."""
    import time
    M = N = K = 8192
    a, b = _gemm_inputs(M, N, K, seed=11)
    ad, bd = a.cuda(), b.cuda()
    base = torch.zeros(M, N, device="cuda", dtype=torch.bfloat16)
    t0 = pk.Task.gemm(base, ad, bd, flags=pk.FLAG_ABORT_INFLIGHT)
    _run_to_completion(t0, pk)
    t0.destroy()
    flag = pk.Flag()
    word = flag.attach_relay()
    c = torch.zeros(M, N, device="cuda", dtype=torch.bfloat16)
    t = pk.Task.gemm(c, ad, bd, flags=pk.FLAG_ABORT_INFLIGHT | _form_flag(pk, form), flag=flag)
    stopped = 0
    for _ in range(4):
        # ten launches back to back (7 ms of work), the word raised 200 us into them
        for _ in range(10):
            t.launch(_stream())
        time.sleep(0.0002)
        word.value = 1
        info = t.wait()
        torch.cuda.synchronize()
        if info.status == pk.STATUS_PREEMPTED:
            stopped += 1
            assert info.tiles_done < info.tiles_total
        word.value = 0
        flag.set(0)
        torch.cuda.synchronize()
        if info.status == pk.STATUS_COMPLETED:
            t.reset(_stream())
    assert stopped >= 1, "the relay never stopped the kernel"
    _run_to_completion(t, pk)
    assert torch.equal(c, base)
    t.destroy()
    flag.destroy()


def test_triad_stops_on_the_relayed_host_word_alone(pk, ok):
    """The stream kernels relay the early-warning word too (one thread in each of the grid's first CTAs): a plain
    host store, with the device flag never written, stops a running triad, and the resumed task gives the bytes of a
    straight run."""
    import time
    n = 1 << 30                                   # 12.9 GB of traffic: about 2 ms per pass
    g = torch.Generator(device="cuda").manual_seed(5)
    b = torch.rand(n, device="cuda", generator=g) * 2 - 1
    c = torch.rand(n, device="cuda", generator=g) * 2 - 1
    want = torch.empty(n, device="cuda")
    t0 = pk.Task.triad(want, b, c, 1.25, flags=pk.FLAG_NON_PREEMPTIBLE)
    _run_to_completion(t0, pk)
    t0.destroy()
    flag = pk.Flag()
    word = flag.attach_relay()
    a = torch.zeros(n, device="cuda")
    t = pk.Task.triad(a, b, c, 1.25, flag=flag)
    stopped = 0
    for _ in range(4):
        t.launch(_stream())
        time.sleep(0.0003)
        word.value = 1
        info = t.wait()
        torch.cuda.synchronize()
        if info.status == pk.STATUS_PREEMPTED:
            stopped += 1
            assert info.tiles_done < info.tiles_total
        word.value = 0
        flag.set(0)
        torch.cuda.synchronize()
        if info.status == pk.STATUS_COMPLETED:
            t.reset(_stream())
    assert stopped >= 1, "the relay never stopped the kernel"
    _run_to_completion(t, pk)
    assert torch.equal(a.view(torch.int32), want.view(torch.int32))
    t.destroy()
    flag.destroy()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_task_calls_from_a_thread_on_another_device(pk):
    """Launch / reset / flag writes switch to the task's device for the call: a worker thread that never chose a
    device (it is on device 0) can drive a task that lives on device 1."""
    import threading
    with torch.cuda.device(1):
        n = 1 << 22
        b = torch.rand(n, device="cuda:1"); c = torch.rand(n, device="cuda:1"); a = torch.empty(n, device="cuda:1")
        stream = torch.cuda.Stream(device=1)
        t = pk.Task.triad(a, b, c, 1.5)
        torch.cuda.synchronize()
    errors = []

    def run():
        try:
            assert torch.cuda.current_device() == 0
            t.reset(stream.cuda_stream)
            t.set_flag(0)
            t.launch(stream.cuda_stream)
            info = t.wait()
            assert info.status == pk.STATUS_COMPLETED
            assert torch.cuda.current_device() == 0           # the caller's device is put back
        except Exception as e:                                # noqa: BLE001
            errors.append(e)
    th = threading.Thread(target=run)
    th.start(); th.join()
    assert not errors, errors
    torch.cuda.synchronize(1)
    ref = torch.empty_like(a)
    t2 = None
    with torch.cuda.device(1):
        t2 = pk.Task.triad(ref, b, c, 1.5, flags=pk.FLAG_NON_PREEMPTIBLE)
        t2.launch(stream.cuda_stream); t2.wait()
        torch.cuda.synchronize()
    assert torch.equal(a, ref)
    t.destroy(); t2.destroy()
