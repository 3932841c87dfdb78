"""Each CUDA kernel alone against its plain statement (tests/kernel_refs.py), at sizes other
than the engine's: widths, head sizes, vocabularies and page sizes that are no powers of two."""
import math

import pytest
import torch

from kernel_refs import ReferenceKernels

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


@pytest.fixture(scope="module")
def K():
    from infurnace_b200.kernels import load_cuda_kernels
    return load_cuda_kernels()


REF = ReferenceKernels(torch.float64)


def tol(dtype):
    return dict(rtol=2e-5, atol=2e-6) if dtype == torch.float32 else dict(rtol=1.6e-2, atol=1e-3)


def rnd(shape, dtype, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n,hidden,vocab", [(1, 72, 333), (37, 1000, 129)])
def test_embed(K, dtype, n, hidden, vocab):
    table = rnd((vocab, hidden), dtype, 0)
    ids = torch.randint(0, vocab, (n,), dtype=torch.int32)
    ids[-1] = vocab - 1
    out = torch.empty((n, hidden), dtype=torch.float32, device="cuda")
    K.embed(table.cuda(), ids.cuda(), out)
    assert torch.equal(out.cpu(), table[ids.long()].float())


@pytest.mark.parametrize("dtype", DTYPES)
def test_random_normal_gives_the_hosts_bits(K, dtype):
    """The device's counter-based values equal the host's bit for bit (integer sum, exact scaling, one rounded
    multiply, one rounded addition), for a matrix (mean 0) and a norm weight (mean 1), at a length that is no
    multiple of anything."""
    from infurnace_b200.weights.random_init import normal_values, tensor_seed
    for name, n, mean, std in (("a.weight", 100_003, 0.0, 0.02), ("b.weight", 4097, 1.0, 0.1)):
        seed = tensor_seed(7, name)
        out = torch.empty(n, dtype=dtype, device="cuda")
        K.random_normal(out, seed, mean, std)
        assert torch.equal(out.cpu(), normal_values(seed, n, mean, std).to(dtype))


def test_a_row_without_valid_logits_cannot_send_the_embedding_out_of_range(K):
    """A row of logits that is all NaN (any NaN in the residual stream) still samples an id inside the
    vocabulary, on the greedy and on the temperature path; and an id outside the vocabulary that does reach
    the embedding (ids fed on the device are never seen by the host) reads nothing: zeros are written and
    the error word says so."""
    vocab, hidden = 333, 72
    logits = rnd((4, vocab), torch.float32, 5).cuda()
    logits[1] = float("nan")
    logits[3, 10:] = float("nan")
    out = torch.full((4,), -7, dtype=torch.int32, device="cuda")
    K.sample(logits, None, None, out)
    assert all(0 <= t < vocab for t in out.tolist()) and out[1].item() == 0
    temp = torch.tensor([0.7, 0.7, 0.0, 1.3], device="cuda")
    uni = torch.tensor([0.3, 0.9, 0.5, 0.99], device="cuda")
    out.fill_(-7)
    K.sample(logits, temp, uni, out)
    assert all(0 <= t < vocab for t in out.tolist())
    table = rnd((vocab, hidden), torch.bfloat16, 6).cuda()
    ids = torch.tensor([5, vocab, -1, 0x7fffffff, vocab - 1], dtype=torch.int32, device="cuda")
    x = torch.full((5, hidden), 9.0, dtype=torch.float32, device="cuda")
    K.check_device_errors()
    K.embed(table, ids, x)
    assert torch.equal(x[0], table[5].float()) and torch.equal(x[4], table[vocab - 1].float())
    assert float(x[1:4].abs().max()) == 0.0
    from infurnace_b200.errors import KernelError
    with pytest.raises(KernelError, match="outside the vocabulary"):
        K.check_device_errors()
    K.check_device_errors()          # the word was cleared


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("wdtype", DTYPES)
@pytest.mark.parametrize("n,hidden,splits", [(1, 72, 0), (5, 1000, 1), (33, 3001, 3), (90, 1024, 1), (64, 128, 0), (70, 2048, 2),
                                             (65, 640, 3), (3, 4096, 1), (80, 4096, 1), (100, 5120, 2), (64, 8192, 0),
                                             (70, 1000, 1), (66, 2052, 3), (64, 8196, 1)])
def test_rmsnorm(K, dtype, wdtype, n, hidden, splits):
    x = rnd((n, hidden), torch.float32, 1)
    w = (1 + 0.1 * rnd((hidden,), torch.float32, 2)).to(wdtype)
    delta = None if splits == 0 else rnd((n, hidden) if splits == 1 else (splits, n, hidden), torch.float32, 3)
    # without rows: x is updated
    x_ref, out_ref = x.clone(), torch.empty((n, hidden), dtype=dtype)
    REF.rmsnorm(x_ref, w, 1e-5, out_ref, delta=delta)
    x_gpu, out_gpu = x.cuda(), torch.empty((n, hidden), dtype=dtype, device="cuda")
    K.rmsnorm(x_gpu, w.cuda(), 1e-5, out_gpu, delta=None if delta is None else delta.cuda())
    torch.testing.assert_close(x_gpu.cpu(), x_ref, rtol=1e-6, atol=1e-6)
    torch.testing.assert_close(out_gpu.cpu().float(), out_ref.float(), **tol(dtype))
    # with rows: x is left alone
    rows = torch.tensor([n - 1, 0, n // 2], dtype=torch.int32)
    out_ref = torch.empty((3, hidden), dtype=dtype)
    REF.rmsnorm(x.clone(), w, 1e-5, out_ref, delta=delta, rows=rows)
    x_gpu, out_gpu = x.cuda(), torch.empty((3, hidden), dtype=dtype, device="cuda")
    K.rmsnorm(x_gpu, w.cuda(), 1e-5, out_gpu, delta=None if delta is None else delta.cuda(), rows=rows.cuda())
    assert torch.equal(x_gpu.cpu(), x)
    torch.testing.assert_close(out_gpu.cpu().float(), out_ref.float(), **tol(dtype))


@pytest.mark.parametrize("xd,wd,od", [(torch.float32, torch.float32, torch.float32),
                                      (torch.bfloat16, torch.bfloat16, torch.bfloat16),
                                      (torch.bfloat16, torch.bfloat16, torch.float32),
                                      (torch.bfloat16, torch.float32, torch.bfloat16),
                                      (torch.float32, torch.bfloat16, torch.float32)])
@pytest.mark.parametrize("n,o,k", [(1, 72, 72), (7, 333, 136), (130, 200, 1000), (64, 64, 16)])
@pytest.mark.parametrize("epilogue", ["none", "silu_gate"])
def test_linear(K, xd, wd, od, n, o, k, epilogue):
    x = rnd((n, k), xd, 4)
    w = rnd((2 * o if epilogue == "silu_gate" else o, k), wd, 5, scale=k ** -0.5)
    ref = torch.empty((n, o), dtype=od)
    REF.linear(x, w, ref, epilogue)
    out = torch.empty((n, o), dtype=od, device="cuda")
    K.linear(x.cuda(), w.cuda(), out, epilogue)
    torch.testing.assert_close(out.cpu().float(), ref.float(), **tol(od))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,d,rdim,inter,ps", [(4, 2, 16, 16, False, 16), (6, 3, 48, 48, False, 8),
                                                    (5, 1, 80, 32, True, 5), (8, 8, 128, 128, False, 16),
                                                    (4, 2, 64, 64, False, 16), (2, 1, 256, 256, False, 32),
                                                    (2, 2, 128, 64, False, 16), (2, 2, 64, 64, True, 16)])
def test_qk_norm_rope_store(K, dtype, nq, nkv, d, rdim, inter, ps):
    n, pages = 23, 9
    qkv = rnd((n, (nq + 2 * nkv) * d), dtype, 6)
    qw = (1 + 0.1 * rnd((d,), torch.float32, 7)).to(dtype)
    kw = (1 + 0.1 * rnd((d,), torch.float32, 8)).to(dtype)
    inv_freq = 1.0 / (10000.0 ** (torch.arange(0, rdim, 2, dtype=torch.float32) / rdim))
    positions = torch.randint(0, 5000, (n,), dtype=torch.int32)
    slots = torch.randperm(pages * ps)[:n].to(torch.int32)
    slots[3] = -1
    kv_ref = torch.zeros((pages, 2, nkv, ps, d), dtype=dtype)
    qkv_ref = qkv.clone()
    ReferenceKernels(torch.float32).qk_norm_rope_store(qkv_ref, nq, nkv, d, qw, kw, 1e-6, inv_freq, rdim, inter,
                                                       positions, slots, kv_ref)
    kv_gpu, qkv_gpu = torch.zeros_like(kv_ref, device="cuda"), qkv.cuda()
    K.qk_norm_rope_store(qkv_gpu, nq, nkv, d, qw.cuda(), kw.cuda(), 1e-6, inv_freq.cuda(), rdim, inter,
                         positions.cuda(), slots.cuda(), kv_gpu)
    t = dict(rtol=1e-4, atol=2e-5) if dtype == torch.float32 else dict(rtol=1.6e-2, atol=2e-2)
    torch.testing.assert_close(qkv_gpu.cpu().float(), qkv_ref.float(), **t)
    torch.testing.assert_close(kv_gpu.cpu().float(), kv_ref.float(), **t)
    # what was not addressed stays zero
    assert kv_gpu.cpu()[kv_ref == 0].abs().max() == 0
    # no norm, no rotation: a pure store
    kv2 = torch.zeros_like(kv_gpu)
    before = qkv_gpu.clone()
    K.qk_norm_rope_store(qkv_gpu, nq, nkv, d, None, None, 0.0, None, 0, False, positions.cuda(), slots.cuda(), kv2)
    assert torch.equal(before, qkv_gpu) and torch.equal(kv2, kv_gpu)


@pytest.mark.parametrize("nq,nkv,ps,norm,rotate", [(16, 8, 16, True, True), (3, 3, 8, True, True), (5, 1, 32, False, True),
                                                   (4, 2, 16, True, False)])
def test_qk_norm_rope_store_for_many_tokens_of_head_size_128(K, nq, nkv, ps, norm, rotate):
    """Steps of 64 tokens and more with bfloat16 heads of 128 run the form in which half a warp takes a head with 16
    bytes per lane (any number of heads, also odd ones); against the plain statement, with the angles from the table."""
    n, d, pages = 150, 128, 12
    qkv = rnd((n, (nq + 2 * nkv) * d), torch.bfloat16, 6)
    qw = (1 + 0.1 * rnd((d,), torch.float32, 7)).to(torch.bfloat16) if norm else None
    kw = (1 + 0.1 * rnd((d,), torch.float32, 8)).to(torch.bfloat16) if norm else None
    inv_freq = 1.0 / (1e6 ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
    positions = torch.randint(0, 5000, (n,), dtype=torch.int32)
    slots = torch.randperm(pages * ps)[:n].to(torch.int32) if pages * ps >= n else torch.arange(n, dtype=torch.int32) % (pages * ps)
    if pages * ps < n:
        pages = -(-n // ps)
        slots = torch.randperm(pages * ps)[:n].to(torch.int32)
    slots[3] = -1
    kv_ref = torch.zeros((pages, 2, nkv, ps, d), dtype=torch.bfloat16)
    qkv_ref = qkv.clone()
    ReferenceKernels(torch.float32).qk_norm_rope_store(qkv_ref, nq, nkv, d, qw, kw, 1e-6, inv_freq if rotate else None,
                                                       d if rotate else 0, False, positions, slots, kv_ref)
    table = None
    if rotate:
        table = torch.empty((n, d), dtype=torch.float32, device="cuda")
        K.rope_table(positions.cuda(), inv_freq.cuda(), table)
    kv_gpu, qkv_gpu = torch.zeros_like(kv_ref, device="cuda"), qkv.cuda()
    K.qk_norm_rope_store(qkv_gpu, nq, nkv, d, qw.cuda() if norm else None, kw.cuda() if norm else None, 1e-6,
                         inv_freq.cuda() if rotate else None, d if rotate else 0, False, positions.cuda(), slots.cuda(), kv_gpu,
                         rope_table=table)
    t = dict(rtol=1.6e-2, atol=2e-2)
    torch.testing.assert_close(qkv_gpu.cpu().float(), qkv_ref.float(), **t)
    torch.testing.assert_close(kv_gpu.cpu().float(), kv_ref.float(), **t)
    assert kv_gpu.cpu()[kv_ref == 0].abs().max() == 0


@pytest.mark.parametrize("n", [1, 5, 8, 13, 16, 40, 100, 128])
@pytest.mark.parametrize("nq,nkv,d,k,ps", [(16, 8, 128, 1024, 16), (4, 2, 64, 2048, 8), (2, 1, 256, 4096, 32), (3, 3, 128, 136, 16),
                                           (5, 1, 128, 2056, 32)])
@pytest.mark.parametrize("norm,rotate,scaled", [(True, True, False), (True, True, True), (False, True, False), (True, False, False)])
def test_qkv_product_with_norm_rotation_and_store_in_its_epilogue(K, n, nq, nkv, d, k, ps, norm, rotate, scaled):
    """The one-launch form of a step's q | k | v projection against its three steps in float64: the
    product (with the row factors of a folded norm before it, when ``scaled``), the RMSNorm of the q and k
    heads, the rotation, and k and v in the pages at the tokens' slots (one token stores nothing).  Up to 16
    rows on the few-rows kernel (a cluster per head), more rows of heads of 128 on the tcgen05 kernel whose
    clusters share the k range of a head."""
    width = (nq + 2 * nkv) * d
    if n > 16:
        w_probe = torch.empty((width, k), dtype=torch.bfloat16, device="cuda")
        can = K.can_fuse_qkv(n, torch.bfloat16, w_probe, d, d if rotate else 0, False, None)
        assert can == (d == 128 and k >= 512), "heads of 128 with enough of k for two CTAs run fused on tcgen05"
        if not can:
            pytest.skip("more than 16 rows run fused only with heads of 128 on tcgen05")
    x = rnd((n, k), torch.bfloat16, 1)
    w = rnd((width, k), torch.bfloat16, 2, scale=k ** -0.5)
    qw = (1 + 0.1 * rnd((d,), torch.float32, 3)).to(torch.bfloat16) if norm else None
    kw = (1 + 0.1 * rnd((d,), torch.float32, 4)) if norm else None          # float32 beside bfloat16 is refused below
    positions = torch.randint(0, 5000, (n,), dtype=torch.int32)
    inv_freq = 1.0 / (1e6 ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
    pages = max(7, -(-n // ps) + 1)
    slots = torch.randperm(pages * ps)[:n].to(torch.int32)
    if n > 2:
        slots[2] = -1
    parts = 5
    partials = torch.rand((parts, n)) * 40 + 1 if scaled else None
    # the three steps, in float64 on what the kernel is given
    y = x.double() @ w.double().t()
    if scaled:
        y = y * torch.rsqrt(partials.double().sum(0) / 77.0 + 1e-5)[:, None]
    qkv_ref = y.clone()
    kv_ref = torch.zeros((pages, 2, nkv, ps, d), dtype=torch.float64)
    kw_used = kw.to(torch.bfloat16) if norm else None
    ReferenceKernels(torch.float64).qk_norm_rope_store(qkv_ref, nq, nkv, d, qw, kw_used, 1e-6, inv_freq if rotate else None,
                                                       d if rotate else 0, False, positions, slots, kv_ref)
    table = None
    if rotate:
        table = torch.empty((n, d), dtype=torch.float32, device="cuda")
        K.rope_table(positions.cuda(), inv_freq.cuda(), table)
    assert K.can_fuse_qkv(n, torch.bfloat16, w.cuda(), d, d if rotate else 0, False, None)
    qkv = torch.full((n, width), float("nan"), dtype=torch.bfloat16, device="cuda")
    kv = torch.zeros((pages, 2, nkv, ps, d), dtype=torch.bfloat16, device="cuda")
    if norm:
        with pytest.raises(Exception, match="differ in dtype"):
            K.linear_qkv_rope_store(x.cuda(), w.cuda(), qkv, nq, nkv, d, qw.cuda(), kw.cuda(), 1e-6, table, slots.cuda(), kv)
    K.linear_qkv_rope_store(x.cuda(), w.cuda(), qkv, nq, nkv, d, qw.cuda() if norm else None, kw_used.cuda() if norm else None,
                            1e-6, table, slots.cuda(), kv,
                            row_scale=(partials.cuda(), parts, 1e-5, 77) if scaled else None)
    t = dict(rtol=1.6e-2, atol=2e-2)
    torch.testing.assert_close(qkv.cpu().double(), qkv_ref, **t)
    torch.testing.assert_close(kv.cpu().double(), kv_ref, **t)
    assert kv.cpu()[kv_ref == 0].abs().max() == 0                # what was not addressed stays zero


def _attention_case(dtype, nq, nkv, d, ps, window, q_lens, seq_lens, seed, spike=False):
    g = torch.Generator().manual_seed(seed)
    R = len(q_lens)
    pages_per = [-(-L // ps) for L in seq_lens]
    total_pages = sum(pages_per) + 3
    perm = torch.randperm(total_pages, generator=g).tolist()
    P = max(pages_per) + 1
    bt = torch.full((R, P), -1, dtype=torch.int32)
    it = iter(perm)
    for r in range(R):
        for j in range(pages_per[r]):
            bt[r, j] = next(it)
    kv = (torch.randn((total_pages, 2, nkv, ps, d), generator=g)).to(dtype)
    n = sum(q_lens)
    qkv = torch.randn((n, (nq + 2 * nkv) * d), generator=g).to(dtype)
    if spike:
        # a far key (position 1 of more than a hundred) of the last request gets a score far above
        # all others for the last query's first head; its value row is all sevens
        r = R - 1
        page, off = int(bt[r, 1 // ps]), 1 % ps
        q0 = qkv[n - 1, :d].float()
        kv[page, 0, 0, off] = (q0 / q0.norm() * 6.0 * math.sqrt(d)).to(dtype)
        kv[page, 1, 0, off] = 7.0
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32)
    sl = torch.tensor(seq_lens, dtype=torch.int32)
    if window:
        # pages wholly below every query's window are stale: poison them
        for r in range(R):
            first = max(0, (seq_lens[r] - q_lens[r]) - window + 1) // ps
            for j in range(first):
                kv[int(bt[r, j])] = float("nan")
                bt[r, j] = -1
    return qkv, kv, bt, cu, sl


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,d,ps,window", [(4, 2, 16, 16, 0), (8, 2, 32, 8, 24), (6, 3, 48, 32, 40),
                                                (16, 8, 128, 16, 0), (3, 1, 80, 5, 7), (2, 2, 256, 16, 0)])
def test_paged_attention(K, dtype, nq, nkv, d, ps, window):
    q_lens, seq_lens = [5, 1, 33, 1, 2], [5, 77, 100, 1, 130]
    qkv, kv, bt, cu, sl = _attention_case(dtype, nq, nkv, d, ps, window, q_lens, seq_lens, 9, spike=(window == 0))
    n = qkv.shape[0]
    ref = torch.empty((n, nq * d), dtype=dtype)
    REF.paged_attention(qkv, nq, nkv, d, kv, bt, cu, sl, ref, d ** -0.5, window, max(q_lens), max(seq_lens))
    out = torch.empty((n, nq * d), dtype=dtype, device="cuda")
    K.paged_attention(qkv.cuda(), nq, nkv, d, kv.cuda(), bt.cuda(), cu.cuda(), sl.cuda(), out, d ** -0.5, window,
                      max(q_lens), max(seq_lens))
    t = dict(rtol=1e-4, atol=1e-5) if dtype == torch.float32 else dict(rtol=1.6e-2, atol=1.6e-2)
    torch.testing.assert_close(out.cpu().float(), ref.float(), **t)
    if window == 0:
        assert ref[n - 1, :d].float().mean() > 6.0     # the far key dominates where it was planted


@pytest.mark.parametrize("vocab,rows", [(333, 3), (151936, 4), (1, 1), (5000, 7)])
def test_sample(K, vocab, rows):
    g = torch.Generator().manual_seed(10)
    logits = torch.randn((rows, vocab), generator=g) * 3
    if vocab > 10:
        logits[0, 7] = logits[0, 3] = logits[0].max() + 1      # a tie: the lower index wins
    temps = torch.tensor([0.0, 0.8, 1.5, 0.3, 0.0, 1.0, 0.05][:rows])
    u = torch.rand((rows,), generator=g)
    ref = torch.empty(rows, dtype=torch.int32)
    REF.sample(logits, temps, u, ref)
    out = torch.empty(rows, dtype=torch.int32, device="cuda")
    K.sample(logits.cuda(), temps.cuda(), u.cuda(), out)
    out = out.cpu()
    for m in range(rows):
        if out[m] != ref[m]:
            # float32 and float64 running sums may part only where u sits on a boundary
            p = torch.softmax(logits[m].double() / float(temps[m]), -1).cumsum(0)
            assert abs(int(out[m]) - int(ref[m])) == 1 and min(abs(p[int(out[m])] - u[m]), abs(p[int(ref[m])] - u[m])) < 1e-5
    # greedy without temperature arrays
    out2 = torch.empty(rows, dtype=torch.int32, device="cuda")
    K.sample(logits.cuda(), None, None, out2)
    assert torch.equal(out2.cpu().long(), logits.argmax(-1))
    if vocab > 10:
        assert int(out2[0]) == 3


@pytest.mark.parametrize("vocab,rows", [(151936, 1), (151937, 8), (32003, 64), (16384, 300)])
def test_greedy_with_several_blocks_per_row(K, vocab, rows):
    """The argmax of a large vocabulary is split over blocks: ties between slices go to the lower index, a row of
    NaN gives an index inside the vocabulary, the per-row counters are left at zero (a second call works), and
    the answer is the one-block-per-row kernel's."""
    g = torch.Generator().manual_seed(vocab + rows)
    logits = torch.randn((rows, vocab), generator=g) * 3
    top = logits.max() + 1
    logits[0, vocab - 1] = logits[0, 5] = top                    # a tie across the first and the last slice
    logits[rows // 2, 9000] = logits[rows // 2, 14001] = top      # and across neighbouring ones
    if rows > 2:
        logits[1] = float("nan")
    want = logits.argmax(-1)
    dev = logits.cuda()
    for _ in range(2):
        out = torch.full((rows,), -1, dtype=torch.int32, device="cuda")
        K.sample(dev, None, None, out)
        got = out.cpu().long()
        ok = torch.ones(rows, dtype=torch.bool)
        if rows > 2:
            ok[1] = False
            assert 0 <= int(got[1]) < vocab
        assert torch.equal(got[ok], want[ok])
    assert int(got[0]) == 5 and (rows == 1 or int(got[rows // 2]) == 9000)
    zeros = torch.zeros(rows, device="cuda")
    out = torch.empty(rows, dtype=torch.int32, device="cuda")
    K.sample(dev, zeros, zeros, out)                              # the one-block kernel, temperature 0
    assert torch.equal(out.cpu().long()[ok], want[ok])


def test_refusals(K):
    from infurnace_b200.errors import KernelError
    with pytest.raises(KernelError):
        K.paged_attention(torch.zeros((1, 3 * 512), device="cuda"), 1, 1, 512,
                          torch.zeros((1, 2, 1, 16, 512), device="cuda"), torch.zeros((1, 1), dtype=torch.int32, device="cuda"),
                          torch.tensor([0, 1], dtype=torch.int32, device="cuda"), torch.tensor([1], dtype=torch.int32, device="cuda"),
                          torch.zeros((1, 512), device="cuda"), 1.0, 0, 1, 1)
    with pytest.raises(KernelError):
        K.linear(torch.zeros((2, 8), device="cuda"), torch.zeros((4, 9), device="cuda"), torch.zeros((2, 4), device="cuda"))
    with pytest.raises(KernelError):
        K.embed(torch.zeros((4, 8), device="cuda", dtype=torch.float16), torch.zeros(2, dtype=torch.int32, device="cuda"),
                torch.zeros((2, 8), device="cuda"))


@pytest.mark.parametrize("nq,nkv,d,ps,window,splits", [(16, 8, 128, 16, 0, 5), (8, 2, 32, 8, 0, 3), (6, 3, 48, 32, 100, 4),
                                                       (4, 4, 64, 16, 0, 32), (16, 1, 16, 64, 0, 2)])
def test_attention_split_over_the_context(K, nq, nkv, d, ps, window, splits):
    """Decoded tokens and two-token portions with the context split over several CTAs (more
    splits than some requests have tiles), merged by the second kernel; prompts beside them."""
    dtype = torch.bfloat16
    g = nq // nkv
    small = max(1, 16 // g)
    q_lens, seq_lens = [1, min(2, small), 1, 40, 1], [700, 1000, 3, 300, 65]
    qkv, kv, bt, cu, sl = _attention_case(dtype, nq, nkv, d, ps, window, q_lens, seq_lens, 12, spike=(window == 0))
    n = qkv.shape[0]
    ref = torch.empty((n, nq * d), dtype=dtype)
    REF.paged_attention(qkv, nq, nkv, d, kv, bt, cu, sl, ref, d ** -0.5, window, max(q_lens), max(seq_lens))
    out = torch.full((n, nq * d), float("nan"), dtype=dtype, device="cuda")
    K._paged_attention_mma(qkv.cuda(), nq, nkv, d, kv.cuda(), bt.cuda(), cu.cuda(), sl.cuda(), out, d ** -0.5, window,
                           max(q_lens), max(seq_lens), n, len(q_lens), num_splits=splits)
    torch.testing.assert_close(out.cpu().float(), ref.float(), rtol=1.6e-2, atol=1.6e-2)


@pytest.mark.parametrize("od", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("n,o,k,splits", [(1, 72, 72, 1), (8, 4096, 1024, 2), (3, 1000, 3072, 7), (16, 333, 136, 1),
                                          (17, 64, 1024, 4), (64, 1024, 2048, 5), (33, 200, 1000, 3), (100, 130, 520, 2),
                                          (1, 151936, 1024, 1)])
@pytest.mark.parametrize("epilogue", ["none", "silu_gate"])
def test_linear_skinny(K, od, n, o, k, splits, epilogue):
    """The few-rows tensor-core product, with k split over several CTAs and merged by the last one;
    twice in a row, so that the counters it leaves behind are shown to be clean."""
    if o > 100000 and epilogue != "none":
        pytest.skip("one large case is enough")
    x = rnd((n, k), torch.bfloat16, 4)
    w = rnd((2 * o if epilogue == "silu_gate" else o, k), torch.bfloat16, 5, scale=k ** -0.5)
    ref = torch.empty((n, o), dtype=od)
    REF.linear(x, w, ref, epilogue)
    xg, wg = x.cuda(), w.cuda()
    for _ in range(2):
        out = torch.full((n, o), float("nan"), dtype=od, device="cuda")
        K._linear_skinny(xg, wg, out, n, o, k, 1 if epilogue == "silu_gate" else 0, splits=splits)
        torch.testing.assert_close(out.cpu().float(), ref.float(), rtol=1.6e-2 if od == torch.bfloat16 else 2e-4,
                                   atol=2e-3 if od == torch.bfloat16 else 1e-4)


@pytest.mark.parametrize("od", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("n,o,k", [(128, 128, 64), (65, 72, 72), (300, 333, 136), (2048, 1024, 1024), (130, 200, 1000),
                                   (257, 4096, 3072), (1000, 151936 // 64, 520)])
@pytest.mark.parametrize("epilogue", ["none", "silu_gate"])
@pytest.mark.parametrize("shape", [0, 1, 2, 3, 4, 5])
def test_linear_tcgen05(K, od, n, o, k, epilogue, shape):
    """The many-rows product on tcgen05 (TMA in, tensor memory accumulator): tiles that hang over
    the ends of all three dimensions, both epilogues, and each tile shape (0: the library's choice,
    narrow, deep, wide)."""
    x = rnd((n, k), torch.bfloat16, 4)
    w = rnd((2 * o if epilogue == "silu_gate" else o, k), torch.bfloat16, 5, scale=k ** -0.5)
    ref = torch.empty((n, o), dtype=od)
    REF.linear(x, w, ref, epilogue)
    out = torch.full((n, o), float("nan"), dtype=od, device="cuda")
    K._linear_tcgen05(x.cuda(), w.cuda(), out, n, o, k, 1 if epilogue == "silu_gate" else 0, shape=shape)
    K.check_device_errors()
    torch.testing.assert_close(out.cpu().float(), ref.float(), rtol=1.6e-2 if od == torch.bfloat16 else 2e-4,
                               atol=2e-3 if od == torch.bfloat16 else 1e-4)


@pytest.mark.parametrize("n", [1, 8, 9, 33, 64, 100, 300])
@pytest.mark.parametrize("hidden,inner,width2", [(72, 136, 40), (1000, 2048, 333), (1024, 3072, 4096), (2304, 1024, 520)])
@pytest.mark.parametrize("epilogue", ["none", "silu_gate"])
@pytest.mark.parametrize("gdt", [torch.bfloat16, torch.float32])
def test_linear_with_a_folded_norm(K, n, hidden, inner, width2, epilogue, gdt, monkeypatch):
    monkeypatch.setattr(K, "fold_max_rows", 64)
    monkeypatch.setattr(K, "tc_fold_max_rows", 1 << 20)
    _folded_norm_case(K, n, hidden, inner, width2, epilogue, gdt)


def test_linear_with_a_folded_norm_on_wide_tiles(K, monkeypatch):
    """The same where the first product has enough rows and features for tiles of 256 x 256."""
    monkeypatch.setattr(K, "tc_fold_max_rows", 1 << 20)
    _folded_norm_case(K, 1300, 4096, 512, 256, "none", torch.bfloat16)
    _folded_norm_case(K, 1300, 4096, 512, 256, "silu_gate", torch.float32)


def _folded_norm_case(K, n, hidden, inner, width2, epilogue, gdt):
    """x += a w1^T, RMSNorm, then a second product, with the norm done by the two products: the
    first writes x * g and partial sums of squares, the second multiplies its rows by the factor.
    Against the three steps done one after the other in float64.  The row counts and sizes reach
    the few-rows kernel and the tcgen05 kernel in its forms (one tile per CTA narrow and wide, the
    k range shared by a cluster, the persistent one for the second product), on either side.  (The
    engine folds up to fold_max_rows rows on the few-rows kernel; it takes as many as that product does.)"""
    a = rnd((n, inner), torch.bfloat16, 1)
    w1 = rnd((hidden, inner), torch.bfloat16, 2, scale=inner ** -0.5)
    x = rnd((n, hidden), torch.float32, 3)
    g = (1 + rnd((hidden,), torch.float32, 4, scale=0.1)).to(gdt)
    w2 = rnd((2 * width2 if epilogue == "silu_gate" else width2, hidden), torch.bfloat16, 5, scale=hidden ** -0.5)
    eps = 1e-5
    x_ref = x.double() + a.double() @ w1.double().t()
    r = torch.rsqrt((x_ref ** 2).mean(dim=1, keepdim=True) + eps)
    xg = (x_ref * g.double()).to(torch.bfloat16)           # what the first product hands over
    w1d, w2d = w1.cuda(), w2.cuda()
    assert K.can_fold_norm(n, torch.bfloat16, w2d, epilogue) and K.can_fold_norm(n, torch.bfloat16, w1d)
    parts = K.fold_parts(hidden, n, w1d)
    if not K._on_tcgen05(n, w1d):
        assert parts in (-(-hidden // 16), -(-hidden // 8))     # a CTA of the few-rows kernel takes 16 features, or 8 of a narrow product
    xd = x.cuda()
    vals = torch.full((n, hidden), float("nan"), dtype=torch.bfloat16, device="cuda")
    partials = torch.full((parts, n), float("nan"), dtype=torch.float32, device="cuda")
    K.linear_residual_norm(a.cuda(), w1d, xd, g.cuda(), vals, partials)
    # the few-rows kernel adds k in float32 registers; the tcgen05 accumulator is held to what its plain product is
    tol = dict(rtol=2e-4, atol=1e-4) if K._on_tcgen05(n, w1d) else dict(rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(xd.cpu().double(), x_ref, **tol)
    torch.testing.assert_close(partials.sum(dim=0).cpu().double(), (x_ref ** 2).sum(dim=1), rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(vals.cpu().float(), xg.float(), rtol=1e-2, atol=1e-3)
    # the second product is held to the values that were handed over (they may differ from xg in a last bfloat16 bit)
    ref = torch.empty((n, width2), dtype=torch.float64)
    REF.linear(vals.cpu().double() * r, w2, ref, epilogue)
    for od in (torch.bfloat16, torch.float32):
        out = torch.full((n, width2), float("nan"), dtype=od, device="cuda")
        K.linear(vals, w2d, out, epilogue, row_scale=(partials, parts, eps, hidden))
        torch.testing.assert_close(out.cpu().float(), ref.float(), rtol=1.6e-2 if od == torch.bfloat16 else 4e-3,
                                   atol=4e-3 if od == torch.bfloat16 else 2e-3)
    K.check_device_errors()
    if n > 64 and hidden % 8:                               # many rows on the plain kernel: no folded norm
        assert not K.can_fold_norm(n, torch.float32, w2d.float(), epilogue)


@pytest.mark.parametrize("n,o,k,splits", [(1, 128, 1024, 2), (9, 1024, 2048, 8), (64, 1000, 1096, 3), (128, 384, 4096, 5),
                                          (100, 72, 136, 2), (5, 200, 136, 8), (37, 4096, 12288, 4)])
@pytest.mark.parametrize("od", [torch.bfloat16, torch.float32])
def test_linear_tcgen05_with_a_shared_k_range(K, n, o, k, splits, od):
    """The tcgen05 product whose tiles' k range is shared by a cluster of CTAs: every cluster size class, a k range
    that does not divide (a CTA with fewer k blocks, one with none), features and rows that leave the tiles ragged;
    twice, with the same bits (the parts are added in a fixed order)."""
    x = rnd((n, k), torch.bfloat16, 4)
    w = rnd((o, k), torch.bfloat16, 5, scale=k ** -0.5)
    ref = torch.empty((n, o), dtype=od)
    REF.linear(x, w, ref, "none")
    outs = []
    for _ in range(2):
        out = torch.full((n, o), float("nan"), dtype=od, device="cuda")
        K._linear_tcgen05_split(x.cuda(), w.cuda(), out, n, o, k, splits)
        outs.append(out.cpu())
    K.check_device_errors()
    assert torch.equal(outs[0], outs[1])
    torch.testing.assert_close(outs[0].float(), ref.float(), rtol=1.6e-2 if od == torch.bfloat16 else 2e-4,
                               atol=2e-3 if od == torch.bfloat16 else 1e-4)


@pytest.mark.parametrize("od", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("n,o,k", [(1, 72, 72), (8, 4096, 1024), (3, 1000, 3072), (16, 333, 136), (17, 64, 1024),
                                   (64, 1024, 2048), (33, 200, 1000), (1, 151936, 1024), (9, 17, 8)])
@pytest.mark.parametrize("epilogue", ["none", "silu_gate"])
def test_linear_gemv(K, od, n, o, k, epilogue):
    """The few-rows product whose warps split k inside the CTA (no partial sums in global memory)."""
    if o > 100000 and epilogue != "none":
        pytest.skip("one large case is enough")
    x = rnd((n, k), torch.bfloat16, 4)
    w = rnd((2 * o if epilogue == "silu_gate" else o, k), torch.bfloat16, 5, scale=k ** -0.5)
    ref = torch.empty((n, o), dtype=od)
    REF.linear(x, w, ref, epilogue)
    out = torch.full((n, o), float("nan"), dtype=od, device="cuda")
    K._linear_gemv(x.cuda(), w.cuda(), out, n, o, k, 1 if epilogue == "silu_gate" else 0)
    torch.testing.assert_close(out.cpu().float(), ref.float(), rtol=1.6e-2 if od == torch.bfloat16 else 2e-4,
                               atol=2e-3 if od == torch.bfloat16 else 1e-4)


@pytest.mark.parametrize("nq,nkv,ps,window", [(16, 8, 16, 0), (4, 4, 16, 0), (8, 2, 32, 0), (16, 2, 64, 0), (16, 1, 16, 0),
                                              (16, 8, 16, 100), (2, 1, 32, 37)])
def test_attention_on_tcgen05(K, nq, nkv, ps, window):
    """Prompts and long portions of head size 128 on tcgen05 (S and P in tensor memory), beside
    decoded tokens that the small-q kernel takes in the same call: every group size that divides
    128, every page size the TMA path takes, with and without a window, portions that start deep
    inside a context and tiles that hang over the ends."""
    dtype, d = torch.bfloat16, 128
    q_lens, seq_lens = [200, 1, 130, 33, 1], [260, 50, 130, 500, 129]
    qkv, kv, bt, cu, sl = _attention_case(dtype, nq, nkv, d, ps, window, q_lens, seq_lens, 21, spike=(window == 0))
    n = qkv.shape[0]
    ref = torch.empty((n, nq * d), dtype=dtype)
    REF.paged_attention(qkv, nq, nkv, d, kv, bt, cu, sl, ref, d ** -0.5, window, max(q_lens), max(seq_lens))
    out = torch.full((n, nq * d), float("nan"), dtype=dtype, device="cuda")
    before = K.tc_attention_calls
    K.paged_attention(qkv.cuda(), nq, nkv, d, kv.cuda(), bt.cuda(), cu.cuda(), sl.cuda(), out, d ** -0.5, window,
                      max(q_lens), max(seq_lens))
    K.check_device_errors()
    assert K.tc_attention_calls == before + 1              # the tcgen05 kernel did run
    torch.testing.assert_close(out.cpu().float(), ref.float(), rtol=1.6e-2, atol=1.6e-2)


@pytest.mark.parametrize("q_lens,seq_lens,window", [([1300], [1300], 0), ([2048], [2048], 0), ([700, 1216, 3], [900, 1216, 40], 0),
                                                    ([1500], [1700], 300), ([1153], [1153], 0)])
def test_attention_on_tcgen05_with_more_items_than_sms(K, q_lens, seq_lens, window):
    """The kernel's grid is a CTA per SM; with more (query tile, kv head) items than SMs a CTA walks several, its
    barriers' phases, score buffers and stages carrying on from one item to the next: items with an odd number of
    key halves (the second stream skips the last tile), with a single half (the second stream has nothing), several
    requests in one launch, portions deep inside a context, a window."""
    nq, nkv, d, ps = 16, 8, 128, 16
    qkv, kv, bt, cu, sl = _attention_case(torch.bfloat16, nq, nkv, d, ps, window, q_lens, seq_lens, 33, spike=(window == 0))
    n = qkv.shape[0]
    assert -(-max(q_lens) // 64) * nkv > K.sm_count
    ref = torch.empty((n, nq * d), dtype=torch.bfloat16)
    REF.paged_attention(qkv, nq, nkv, d, kv, bt, cu, sl, ref, d ** -0.5, window, max(q_lens), max(seq_lens))
    for rep in range(2):
        out = torch.full((n, nq * d), float("nan"), dtype=torch.bfloat16, device="cuda")
        K.paged_attention(qkv.cuda(), nq, nkv, d, kv.cuda(), bt.cuda(), cu.cuda(), sl.cuda(), out, d ** -0.5, window,
                          max(q_lens), max(seq_lens))
        K.check_device_errors()
        torch.testing.assert_close(out.cpu().float(), ref.float(), rtol=1.6e-2, atol=1.6e-2)


@pytest.mark.parametrize("q_len", [65, 100, 105, 127, 128, 200])
def test_attention_on_tcgen05_waits_for_its_products(K, q_len):
    """A stream that works through exactly two halves of keys reads its accumulator after a wait by parity on the
    barrier of its P V products; a step that skipped the wait for the first half's products left that wait one phase
    short, and it passed while the products were still in flight whenever the values arrived late (found when a
    CTA's second query tile had two halves; the lengths here give one and two halves per stream and tile).
    The kernel is run many times on fresh, differently placed inputs; every run must agree with the plain statement."""
    nq, nkv, d, ps = 16, 8, 128, 16
    for rep in range(12):
        qkv, kv, bt, cu, sl = _attention_case(torch.bfloat16, nq, nkv, d, ps, 0, [q_len], [q_len], 100 + rep)
        n = qkv.shape[0]
        ref = torch.empty((n, nq * d), dtype=torch.bfloat16)
        REF.paged_attention(qkv, nq, nkv, d, kv, bt, cu, sl, ref, d ** -0.5, 0, q_len, q_len)
        junk = torch.full(((rep + 1) << 20,), float("nan"), device="cuda")         # shifts where the inputs land
        out = torch.full((n, nq * d), float("nan"), dtype=torch.bfloat16, device="cuda")
        K.paged_attention(qkv.cuda(), nq, nkv, d, kv.cuda(), bt.cuda(), cu.cuda(), sl.cuda(), out, d ** -0.5, 0, q_len, q_len)
        del junk
        torch.testing.assert_close(out.cpu().float(), ref.float(), rtol=1.6e-2, atol=1.6e-2)
    K.check_device_errors()
