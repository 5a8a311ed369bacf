"""Memory-bound kernels against plain PyTorch fp32 references."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _C():
    from meshslice_b200 import _native
    return _native.load(), _native.stream_ptr()


@pytest.mark.parametrize("cols,rows", [(1024, 301), (768, 43), (64, 1000), (2048, 300), (4096, 300), (12288, 300)])
def test_layernorm_fwd_bwd_single_pass(cols, rows):
    """Widths up to 2048 run several rows per CTA in the backward kernel (row counts that leave the last CTA
    partly empty included); wider rows one row per CTA with one, two or four vectors per thread."""
    C, st = _C()
    x = torch.randn(rows, cols, device="cuda").bfloat16()
    res = torch.randn(rows, cols, device="cuda").bfloat16()
    gamma = (1 + 0.1 * torch.randn(cols, device="cuda")).bfloat16()
    beta = (0.1 * torch.randn(cols, device="cuda")).bfloat16()
    h = torch.empty_like(x)
    y = torch.empty_like(x)
    mr = torch.empty(rows, 2, device="cuda")
    C.ln_fwd(0, x.data_ptr(), res.data_ptr(), h.data_ptr(), y.data_ptr(), gamma.data_ptr(), beta.data_ptr(),
             0, mr.data_ptr(), rows, cols, cols, 1e-5, st)
    h_ref = (x.float() + res.float())
    assert (h.float() - h_ref).abs().max() < 0.05
    hh = h.float().requires_grad_(True)
    g32, b32 = gamma.float().requires_grad_(True), beta.float().requires_grad_(True)
    y_ref = torch.nn.functional.layer_norm(hh, (cols,), g32, b32, 1e-5)
    assert (y.float() - y_ref).abs().max() < 0.05
    dy = torch.randn(rows, cols, device="cuda").bfloat16()
    dres = torch.randn(rows, cols, device="cuda").bfloat16()
    y_ref.backward(dy.float())
    dx = torch.empty_like(x)
    dg = torch.zeros(cols, device="cuda")
    db = torch.zeros(cols, device="cuda")
    C.ln_bwd(0, dy.data_ptr(), h.data_ptr(), gamma.data_ptr(), mr.data_ptr(), dres.data_ptr(), dx.data_ptr(),
             0, dg.data_ptr(), db.data_ptr(), rows, cols, cols, st)
    torch.cuda.synchronize()
    assert (dx.float() - (hh.grad + dres.float())).abs().max() < 0.06
    assert (dg - g32.grad).abs().max() < 0.05 * rows ** 0.5
    assert (db - b32.grad).abs().max() < 0.05 * rows ** 0.5


def test_layernorm_two_pass_equals_single_pass():
    """The column-sharded path: partial statistics per shard, summed, then applied."""
    C, st = _C()
    rows, cols, parts = 64, 2048, 4
    x = torch.randn(rows, cols, device="cuda").bfloat16()
    gamma = torch.ones(cols, device="cuda").bfloat16()
    y_full = torch.empty_like(x)
    mr = torch.empty(rows, 2, device="cuda")
    C.ln_fwd(0, x.data_ptr(), 0, 0, y_full.data_ptr(), gamma.data_ptr(), 0, 0, mr.data_ptr(), rows, cols, cols, 1e-5, st)
    w = cols // parts
    shards = [x[:, i * w:(i + 1) * w].contiguous() for i in range(parts)]
    stats = [torch.empty(rows, 2, device="cuda") for _ in range(parts)]
    for s, t in zip(shards, stats):
        C.ln_fwd(1, s.data_ptr(), 0, 0, 0, 0, 0, t.data_ptr(), 0, rows, w, cols, 1e-5, st)
    total = sum(stats)
    outs = []
    for i, s in enumerate(shards):
        y = torch.empty_like(s)
        g = gamma[i * w:(i + 1) * w].contiguous()
        C.ln_fwd(2, s.data_ptr(), 0, 0, y.data_ptr(), g.data_ptr(), 0, total.data_ptr(), mr.data_ptr(), rows, w, cols, 1e-5, st)
        outs.append(y)
    torch.cuda.synchronize()
    assert (torch.cat(outs, 1).float() - y_full.float()).abs().max() < 0.02


@pytest.mark.parametrize("affine", [True, False])
def test_layernorm_backward_two_pass_equals_single_pass(affine):
    """Backward of the column-sharded path (partial dot products per shard, summed, then applied) against the
    single-pass kernel on the whole row and against autograd in fp32."""
    C, st = _C()
    rows, cols, parts = 97, 4096, 4
    hbuf = torch.randn(rows, cols, device="cuda").bfloat16()
    dy = torch.randn(rows, cols, device="cuda").bfloat16()
    dres = torch.randn(rows, cols, device="cuda").bfloat16()
    gamma = (1.0 + 0.1 * torch.randn(cols, device="cuda")).bfloat16() if affine else None
    gp = gamma.data_ptr() if affine else 0
    mean = hbuf.float().mean(1)
    rstd = (hbuf.float().var(1, unbiased=False) + 1e-5).rsqrt()
    mr = torch.stack([mean, rstd], 1).contiguous()
    dx_full = torch.empty_like(hbuf)
    dg_full = torch.zeros(cols, device="cuda")
    db_full = torch.zeros(cols, device="cuda")
    C.ln_bwd(0, dy.data_ptr(), hbuf.data_ptr(), gp, mr.data_ptr(), dres.data_ptr(), dx_full.data_ptr(), 0,
             dg_full.data_ptr() if affine else 0, db_full.data_ptr() if affine else 0, rows, cols, cols, st)
    w = cols // parts
    # the shards stay referenced until the kernels have run (only raw pointers are passed)
    cut = lambda t: [t[:, i * w:(i + 1) * w].contiguous() for i in range(parts)]
    dys, hs, drs = cut(dy), cut(hbuf), cut(dres)
    gs = [gamma[i * w:(i + 1) * w].contiguous() for i in range(parts)] if affine else [None] * parts
    stats, dgs, dbs = [], [], []
    for i in range(parts):
        t = torch.empty(rows, 2, device="cuda")
        dg = torch.zeros(w, device="cuda")
        db = torch.zeros(w, device="cuda")
        C.ln_bwd(1, dys[i].data_ptr(), hs[i].data_ptr(), gs[i].data_ptr() if affine else 0, mr.data_ptr(), 0, 0,
                 t.data_ptr(), dg.data_ptr() if affine else 0, db.data_ptr() if affine else 0, rows, w, cols, st)
        stats.append(t); dgs.append(dg); dbs.append(db)
    total = sum(stats)
    outs = []
    for i in range(parts):
        dx = torch.empty(rows, w, device="cuda", dtype=torch.bfloat16)
        C.ln_bwd(2, dys[i].data_ptr(), hs[i].data_ptr(), gs[i].data_ptr() if affine else 0, mr.data_ptr(),
                 drs[i].data_ptr(), dx.data_ptr(), total.data_ptr(), 0, 0, rows, w, cols, st)
        outs.append(dx)
    torch.cuda.synchronize()
    assert (torch.cat(outs, 1).float() - dx_full.float()).abs().max() < 0.04
    hh = hbuf.float().requires_grad_(True)
    g32 = gamma.float().requires_grad_(True) if affine else None
    torch.nn.functional.layer_norm(hh, (cols,), g32, None, 1e-5).backward(dy.float())
    assert (dx_full.float() - (hh.grad + dres.float())).abs().max() < 0.06
    if affine:
        assert (torch.cat(dgs) - dg_full).abs().max() < 1e-2
        assert (dg_full - g32.grad).abs().max() < 0.05 * rows ** 0.5
        assert (torch.cat(dbs) - dy.float().sum(0)).abs().max() < 1e-2


def test_gelu_fwd_bwd():
    C, st = _C()
    x = torch.randn(1 << 16, device="cuda").bfloat16()
    dy = torch.randn(1 << 16, device="cuda").bfloat16()
    y = torch.empty_like(x)
    dx = torch.empty_like(x)
    C.gelu_fwd(x.data_ptr(), y.data_ptr(), x.numel(), st)
    C.gelu_bwd(dy.data_ptr(), x.data_ptr(), dx.data_ptr(), x.numel(), st)
    x32 = x.float().requires_grad_(True)
    ref = torch.nn.functional.gelu(x32, approximate="tanh")
    ref.backward(dy.float())
    assert (y.float() - ref).abs().max() < 0.02
    assert (dx.float() - x32.grad).abs().max() < 0.03


def test_adamw_matches_torch():
    C, st = _C()
    n = 4096 * 3
    p32 = torch.randn(n, device="cuda")
    g = torch.randn(n, device="cuda").bfloat16()
    p = p32.bfloat16()
    master = p32.clone()
    m = torch.zeros(n, device="cuda")
    v = torch.zeros(n, device="cuda")
    ref = p32.clone().requires_grad_(True)
    opt = torch.optim.AdamW([ref], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    for step in range(1, 4):
        ref.grad = g.float()
        opt.step()
        C.adamw_step(p.data_ptr(), master.data_ptr(), m.data_ptr(), v.data_ptr(), g.data_ptr(), 0, n, 1e-2,
                     0.9, 0.95, 1e-8, 0.1, 1 - 0.9 ** step, 1 - 0.95 ** step, 0, st)
    torch.cuda.synchronize()
    assert (master - ref.detach()).abs().max() < 1e-4
    assert (p.float() - ref.detach()).abs().max() < 0.02


def test_cross_entropy_vocab_parallel():
    C, st = _C()
    rows, vocab, parts = 96, 1000, 4
    vpad = 1024
    w = vpad // parts
    logits = (3 * torch.randn(rows, vpad, device="cuda")).bfloat16()
    tgt = torch.randint(0, vocab, (rows,), device="cuda")
    ref_l = logits.float()[:, :vocab].clone().requires_grad_(True)
    loss_ref = torch.nn.functional.cross_entropy(ref_l, tgt, reduction="mean")
    loss_ref.backward()
    mx, se, tl = [], [], []
    shards = [logits[:, i * w:(i + 1) * w].contiguous() for i in range(parts)]
    for i, s in enumerate(shards):
        a, b, c = (torch.empty(rows, device="cuda") for _ in range(3))
        C.ce_partial(s.data_ptr(), w, tgt.data_ptr(), rows, w, i * w, vocab, a.data_ptr(), b.data_ptr(), c.data_ptr(), st)
        mx.append(a); se.append(b); tl.append(c)
    gmax = torch.stack(mx).max(0).values
    gsum = sum(s * torch.exp(m - gmax) for s, m in zip(se, mx))
    tlog = sum(tl)
    loss = (torch.log(gsum) + gmax - tlog).mean()
    assert abs(loss.item() - loss_ref.item()) < 2e-3
    for i, s in enumerate(shards):
        C.ce_grad(s.data_ptr(), w, tgt.data_ptr(), rows, w, i * w, vocab, gmax.data_ptr(), gsum.data_ptr(), 1.0 / rows, st)
    torch.cuda.synchronize()
    grad = torch.cat(shards, 1).float()
    assert (grad[:, :vocab] - ref_l.grad).abs().max() < 2e-4
    assert grad[:, vocab:].abs().max() == 0


def test_embedding_fwd_bwd():
    C, st = _C()
    vocab, seq, nb, cols = 500, 16, 4, 256
    tok = torch.randint(0, vocab, (nb * seq,), device="cuda")
    te = torch.randn(vocab, cols, device="cuda").bfloat16()
    pe = torch.randn(seq, cols, device="cuda").bfloat16()
    out = torch.empty(nb * seq, cols, device="cuda", dtype=torch.bfloat16)
    C.embedding_fwd(tok.data_ptr(), te.data_ptr(), pe.data_ptr(), out.data_ptr(), nb * seq, seq, cols, st)
    ref = te.float()[tok] + pe.float().repeat(nb, 1)
    assert (out.float() - ref).abs().max() < 0.05
    dout = torch.randn(nb * seq, cols, device="cuda").bfloat16()
    dt = torch.zeros(vocab, cols, device="cuda")
    dp = torch.zeros(seq, cols, device="cuda")
    C.embedding_bwd(tok.data_ptr(), dout.data_ptr(), dt.data_ptr(), dp.data_ptr(), nb * seq, seq, cols, st)
    torch.cuda.synchronize()
    dt_ref = torch.zeros(vocab, cols, device="cuda").index_add_(0, tok, dout.float())
    dp_ref = dout.float().view(nb, seq, cols).sum(0)
    assert (dt - dt_ref).abs().max() < 1e-3
    assert (dp - dp_ref).abs().max() < 1e-3


def test_sumsq():
    C, st = _C()
    x = torch.randn(1 << 18, device="cuda").bfloat16()
    out = torch.zeros(1, device="cuda")
    C.sumsq(x.data_ptr(), 0, x.numel(), out.data_ptr(), st)
    torch.cuda.synchronize()
    assert abs(out.item() - (x.float() ** 2).sum().item()) / out.item() < 1e-4


def _emulated_exchange(n, rows, grid):
    """Descriptors of one row exchange among n emulated ranks that all live on this GPU: rank q's slot area and
    arrival counter are plain tensors.  The caller runs every rank's producer before any consumer, so no kernel
    waits for one that has not run; the consumers' waits are then satisfied on entry."""
    from meshslice_b200 import _native
    width = 4
    stride = rows * width
    slots = [torch.zeros(n * stride, device="cuda") for _ in range(n)]
    counters = [torch.zeros(16, dtype=torch.int32, device="cuda") for _ in range(n)]
    descs = []
    for q in range(n):
        descs.append(dict(n=n, me=q, dst=[slots[p].data_ptr() + q * stride * 4 for p in range(n)],
                          slots=slots[q].data_ptr(), stride=stride,
                          counter=[counters[p].data_ptr() for p in range(n)], my_counter=counters[q].data_ptr(),
                          target=(n - 1) * grid, timeout_ns=50_000_000, status=_native.status().dev))
    return descs, (slots, counters)


@pytest.mark.parametrize("n,w,rows", [(4, 1024, 203), (2, 4096, 64), (2, 256, 1000)])
def test_layernorm_row_exchange_emulated_ranks(n, w, rows):
    """LayerNorm forward and backward over a feature dimension split among n ranks, the partial row sums travelling
    through the in-kernel exchange (slots + arrival counters), against the single-device kernels on the whole rows.
    Narrow shards take the several-rows-per-CTA form of the backward kernel."""
    from meshslice_b200 import _native
    from meshslice_b200.ops import functional as F
    C, st = _C()
    cols = n * w
    cut = lambda t: [t[:, q * w:(q + 1) * w].contiguous() for q in range(n)]
    x = torch.randn(rows, cols, device="cuda").bfloat16()
    res = torch.randn(rows, cols, device="cuda").bfloat16()
    gamma = (1 + 0.1 * torch.randn(cols, device="cuda")).bfloat16()
    beta = (0.1 * torch.randn(cols, device="cuda")).bfloat16()
    h_ref, y_ref, mr_ref = F.ln_full(x, res, gamma, beta, 1e-5)
    xs, rs = cut(x), cut(res)
    gs = [gamma[q * w:(q + 1) * w].contiguous() for q in range(n)]
    bs = [beta[q * w:(q + 1) * w].contiguous() for q in range(n)]
    descs, keep = _emulated_exchange(n, rows, C.ln_grid(0, rows, w))
    hs = [F.ln_stats(xs[q], rs[q], exch=descs[q])[0] for q in range(n)]
    outs = [F.ln_apply(hs[q], None, gs[q], bs[q], cols, 1e-5, exch=descs[q]) for q in range(n)]
    _native.check_status()
    assert torch.equal(torch.cat(hs, 1), h_ref)
    assert (torch.cat([o[0] for o in outs], 1).float() - y_ref.float()).abs().max() < 0.02
    for q in range(n):
        assert (outs[q][1] - mr_ref).abs().max() < 1e-3
    # backward
    dy = torch.randn(rows, cols, device="cuda").bfloat16()
    dres = torch.randn(rows, cols, device="cuda").bfloat16()
    dg_ref = torch.zeros(cols, device="cuda")
    db_ref = torch.zeros(cols, device="cuda")
    dx_ref = F.ln_bwd_full(dy, h_ref, gamma, mr_ref, dg_ref, db_ref, dres)
    dys, drs = cut(dy), cut(dres)
    dgs = [torch.zeros(w, device="cuda") for _ in range(n)]
    dbs = [torch.zeros(w, device="cuda") for _ in range(n)]
    descs, keep2 = _emulated_exchange(n, rows, C.ln_grid(1, rows, w))
    for q in range(n):
        F.ln_bwd_stats(dys[q], hs[q], gs[q], mr_ref, dgs[q], dbs[q], exch=descs[q])
    dxs = [F.ln_bwd_apply(dys[q], hs[q], gs[q], mr_ref, None, cols, drs[q], exch=descs[q]) for q in range(n)]
    _native.check_status()
    assert (torch.cat(dxs, 1).float() - dx_ref.float()).abs().max() < 0.04
    assert (torch.cat(dgs) - dg_ref).abs().max() < 1e-2 * rows ** 0.5
    assert (torch.cat(dbs) - db_ref).abs().max() < 1e-2 * rows ** 0.5
    # every rank's counter has seen exactly the other ranks' CTAs
    for q in range(n):
        assert int(keep2[1][q][0]) == (n - 1) * C.ln_grid(1, rows, w)
