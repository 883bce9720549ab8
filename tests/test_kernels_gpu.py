"""Each CUDA kernel alone against a plain PyTorch float32 statement of the same operation, at
sizes other than the engine's."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def k():
    from gemmars_b200 import kernels
    return kernels


def _paged(nseq, lengths, nkv, hd, dtype, page=64, extra_pages=3, seed=0, ring=None):
    """A paged cache filled with random keys and values for sequences of the given lengths, with a
    shuffled page assignment; returns tensors and per-sequence dense [len, nkv, hd] copies."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    width = max(-(-max(lengths) // page), 1) if ring is None else ring
    n_pages = sum(min(-(-n // page), width) for n in lengths) + extra_pages
    kc = torch.randn((n_pages + 1, nkv, page, hd), generator=g, device="cuda").to(dtype)
    vc = torch.randn((n_pages + 1, nkv, hd, page), generator=g, device="cuda").to(dtype)
    perm = (torch.randperm(n_pages, generator=torch.Generator().manual_seed(seed)) + 1).tolist()
    table = torch.zeros((nseq + 1, width), dtype=torch.int32)
    dense = []
    for s, n in enumerate(lengths):
        for lp in range(min(-(-n // page), width)):
            table[s, lp] = perm.pop()
        ks = torch.zeros((n, nkv, hd), device="cuda")
        vs = torch.zeros((n, nkv, hd), device="cuda")
        for p in range(n):
            pg = int(table[s, (p // page) % width])
            ks[p] = kc[pg, :, p % page, :].float()
            vs[p] = vc[pg, :, :, p % page].float()
        dense.append((ks, vs))
    return kc, vc, table.cuda(), dense


def _attn_ref(q, ks, vs, pos, nh, window=None):
    """q: [nh, hd] float32 at position pos; ks, vs: [len, nkv, hd]."""
    nkv = ks.shape[1]
    lo = 0 if not window else max(0, pos + 1 - window)
    out = torch.zeros_like(q)
    for h in range(nh):
        g = h // (nh // nkv)
        s = ks[lo:pos + 1, g] @ q[h]
        out[h] = torch.softmax(s, 0) @ vs[lo:pos + 1, g]
    return out


@pytest.mark.parametrize("m,n,kk,mode", [(1, 128, 64, "f32"), (5, 100, 96, "bf16"), (17, 300, 200, "acc"),
                                          (64, 520, 1032, "bf16"), (100, 1000, 128, "f32"), (300, 384, 1024, "acc"),
                                          (515, 260, 2048, "bf16")])
def test_gemm_tc(k, m, n, kk, mode):
    torch.manual_seed(m + n)
    x = (torch.randn(m, kk, device="cuda") * 0.5).bfloat16()
    w = (torch.randn(n, kk, device="cuda") * 0.05).bfloat16()
    b = torch.randn(n, device="cuda") if m % 2 else None
    ref = x.float() @ w.float().T + (b if b is not None else 0)
    if mode == "bf16":
        out, tol = torch.zeros(m, n, device="cuda", dtype=torch.bfloat16), 2 ** -8
    elif mode == "f32":
        out, tol = torch.zeros(m, n, device="cuda"), 1e-5
    else:
        out, tol, ref = torch.ones(m, n, device="cuda"), 1e-5, ref + 1
    k.gemm_tc(x, w, out, b, accumulate=(mode == "acc"))
    assert (out.float() - ref).abs().max().item() <= tol * ref.abs().max().item() + 1e-6
    # the plain kernel on the same operands
    out2 = torch.ones_like(out) if mode == "acc" else torch.zeros_like(out)
    k.gemm_ref(x, w, out2, b, accumulate=(mode == "acc"))
    assert (out2.float() - ref).abs().max().item() <= tol * ref.abs().max().item() + 1e-6
    assert k.gemm_tc_status() == 0


@pytest.mark.parametrize("splits", [2, 4, 8])
def test_gemm_tc_cluster_split(k, splits):
    torch.manual_seed(splits)
    for bn, m in ((16, 3), (32, 29), (64, 64)):
        x = (torch.randn(m, 1600, device="cuda") * 0.5).bfloat16()
        w = (torch.randn(333, 1600, device="cuda") * 0.05).bfloat16()
        ref = x.float() @ w.float().T
        out = torch.zeros(m, 333, device="cuda")
        k.gemm_tc(x, w, out, bn=bn, splits=splits)
        assert (out - ref).abs().max().item() <= 1e-5 * ref.abs().max().item()
        again = torch.zeros_like(out)
        k.gemm_tc(x, w, again, bn=bn, splits=splits)
        assert torch.equal(out, again)                      # added in rank order: the same bits every run
        # added into a residual: every token of a rank's share keeps what was there (shares of
        # more than eight tokens with two and four ranks)
        acc = torch.full((m, 333), 3.0, device="cuda")
        k.gemm_tc(x, w, acc, accumulate=True, bn=bn, splits=splits)
        assert (acc - (ref + 3.0)).abs().max().item() <= 1e-5 * (ref.abs().max().item() + 3.0)
    assert k.gemm_tc_status() == 0


def test_gemm_ref_float32_rows_do_not_depend_on_the_batch(k):
    torch.manual_seed(1)
    x = torch.randn(70, 4128 + 32, device="cuda")
    w = torch.randn(37, 4128 + 32, device="cuda")
    full = torch.empty(70, 37, device="cuda")
    k.gemm_ref(x, w, full)
    assert (full - x.double() @ w.double().T).abs().max().item() < 2e-3
    for rows in (1, 2, 7):                                   # cf. src/qwen_mtp.rs:748-776
        part = torch.empty(rows, 37, device="cuda")
        k.gemm_ref(x[13:13 + rows], w, part)
        assert torch.equal(part, full[13:13 + rows])


def test_gemm_refuses_what_it_cannot_take(k):
    x = torch.randn(4, 100, device="cuda").bfloat16()
    w = torch.randn(8, 100, device="cuda").bfloat16()
    assert not k.gemm_tc_usable(x, w)                        # rows of 200 bytes: not a multiple of 16
    with pytest.raises(k.KernelError):
        k.gemm_tc(x, w, torch.empty(4, 8, device="cuda"))
    out = torch.empty(4, 8, device="cuda", dtype=torch.bfloat16)
    k.gemm(x, w, out)                                        # the dispatcher falls to the plain kernel
    assert (out.float() - x.float() @ w.float().T).abs().max().item() < 0.2
    with pytest.raises(k.KernelError, match="CUDA tensors only"):
        k.gemm_ref(x.cpu(), w.cpu(), out.cpu())


@pytest.mark.parametrize("rows,n,eps", [(3, 80, 1e-5), (17, 4100, 1e-6), (515, 4096, 1e-6), (600, 2564, 1e-5),
                                        (513, 5120, 1e-6), (512, 72, 1e-6), (514, 8200, 1e-6)])
def test_rmsnorm_and_gather(k, rows, n, eps):
    torch.manual_seed(rows)
    x = torch.randn(rows + 4, n, device="cuda") * 3
    w = torch.randn(n, device="cuda")
    ref = x * torch.rsqrt((x.double() ** 2).mean(-1, keepdim=True) + eps).float() * w
    for dt, tol in ((torch.float32, 1e-5), (torch.bfloat16, 2 ** -8)):
        out = torch.empty(rows + 4, n, device="cuda", dtype=dt)
        k.rmsnorm(x, w, out, eps)
        assert (out.float() - ref).abs().max().item() <= tol * ref.abs().max().item()
    idx = torch.tensor([rows + 3, 0, 2], dtype=torch.int32, device="cuda")
    out = torch.empty(3, n, device="cuda")
    k.rmsnorm(x, w, out, eps, idx)
    assert torch.allclose(out, ref[idx.long()], rtol=1e-5, atol=1e-5)


def test_embedding_and_gated_activation(k):
    torch.manual_seed(2)
    table = torch.randn(301, 72, device="cuda").bfloat16()
    tok = torch.tensor([300, 0, 17, 17], dtype=torch.int32, device="cuda")
    out = torch.empty(4, 72, device="cuda")
    k.embed_gather(table, tok, out, 1.5)
    assert torch.equal(out, table[tok.long()].float() * 1.5)
    for hidden in (4096, 2568, 70):       # 16 bytes at a time, with an edge; rows that are not 16-byte aligned
        table = torch.randn(301, hidden, device="cuda").bfloat16()
        out = torch.empty(4, hidden, device="cuda")
        k.embed_gather(table, tok, out, 0.75)
        assert torch.equal(out, table[tok.long()].float() * 0.75)
    table = torch.randn(301, 72, device="cuda")
    out = torch.empty(4, 72, device="cuda")
    k.embed_gather(table, tok, out, 1.0)
    assert torch.equal(out, table[tok.long()])
    gu = torch.randn(5, 2 * 112, device="cuda")
    act = torch.empty(5, 112, device="cuda")
    k.silu_mul(gu, act)
    g, u = gu[:, :112].double(), gu[:, 112:].double()
    assert (act - (g / (1 + torch.exp(-g)) * u).float()).abs().max().item() < 1e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("step", ["few", "prompt"])
@pytest.mark.parametrize("hd,rot,nh,nkv", [(48, 24, 5, 1), (16, 16, 4, 2), (128, 128, 8, 2), (64, 64, 7, 1), (32, 32, 3, 3),
                                            (256, 256, 2, 1), (96, 96, 2, 2)])
def test_head_norm_rope_cache(k, dtype, step, hd, rot, nh, nkv):
    """A step of a few tokens (one warp per head) and one of prompt size (64 tokens and more: in
    bfloat16 the kernel with several heads to a warp, and the values through the tile kernel)."""
    torch.manual_seed(hd)
    if step == "few":
        lengths = [70, 5]
        # sequence 0 appends positions 66..69, sequence 1 positions 0..4
        seqs, poss = [0] * 4 + [1] * 5, [66, 67, 68, 69, 0, 1, 2, 3, 4]
    else:
        lengths = [150, 37]
        # sequence 0 appends positions 60..149 (across page borders), sequence 1 its whole prompt
        seqs, poss = [0] * 90 + [1] * 37, list(range(60, 150)) + list(range(37))
    kc, vc, table, _ = _paged(2, lengths, nkv, hd, dtype)
    kc.zero_(); vc.zero_()
    tok_seq = torch.tensor(seqs, dtype=torch.int32, device="cuda")
    tok_pos = torch.tensor(poss, dtype=torch.int32, device="cuda")
    seq_slot = torch.tensor([0, 1], dtype=torch.int32, device="cuda")
    t = len(seqs)
    qkv = torch.randn(t, (nh + 2 * nkv) * hd, device="cuda").to(dtype)
    qw, kw = torch.rand(hd, device="cuda") + 0.5, torch.rand(hd, device="cuda") + 0.5
    theta, eps, scale = 5e4, 1e-5, hd ** -0.5
    inv = (1.0 / torch.pow(torch.tensor(theta, dtype=torch.float64), torch.arange(rot // 2, dtype=torch.float64) * 2 / rot)).float().cuda()
    src = qkv.float().view(t, nh + 2 * nkv, hd).clone()
    work = qkv.clone()
    k.head_norm_rope_cache(work, nh, nkv, hd, rot, qw, kw, eps, inv, scale, tok_pos, tok_seq, seq_slot, table, 64, kc, vc,
                           k.FLAG_NORM | k.FLAG_ROPE | k.FLAG_CACHE | k.FLAG_INPLACE)

    def ref_head(v, w, pos, s):
        v = v * torch.rsqrt((v.double() ** 2).mean() + eps).float() * w
        ang = (torch.tensor(float(pos), device="cuda") * inv).double()
        a, b = v[:rot // 2].double(), v[rot // 2:rot].double()
        out = v.double().clone()
        out[:rot // 2] = a * torch.cos(ang) - b * torch.sin(ang)
        out[rot // 2:rot] = b * torch.cos(ang) + a * torch.sin(ang)
        return (out * s).float()

    tol = 1e-5 if dtype == torch.float32 else 2 ** -7
    got = work.float().view(t, nh + 2 * nkv, hd)
    for i in range(t):
        pos, slot = int(tok_pos[i]), int(tok_seq[i])
        page = int(table[slot, pos // 64])
        for h in range(nh):
            assert (got[i, h] - ref_head(src[i, h], qw, pos, scale)).abs().max().item() <= tol * 4
        for h in range(nkv):
            want = ref_head(src[i, nh + h], kw, pos, 1.0)
            assert (got[i, nh + h] - want).abs().max().item() <= tol * 4
            assert (kc[page, h, pos % 64].float() - want).abs().max().item() <= tol * 4
            assert torch.equal(vc[page, h, :, pos % 64].float(), src[i, nh + nkv + h])     # values are cached raw
    assert float(kc[0].abs().sum()) == 0.0                                                    # nothing strays into page 0


@pytest.mark.parametrize("hd,nh,nkv,window", [(16, 4, 2, None), (32, 6, 3, 40), (48, 5, 1, None), (128, 8, 2, 100),
                                               (64, 12, 1, None), (128, 32, 1, None), (96, 3, 1, 50), (256, 4, 2, None)])
def test_attention_kernels_against_plain(k, hd, nh, nkv, window):
    """The plain kernel in both precisions and the decode kernel (1 and several shares), with a
    planted far key: one key far back gets a score that stands out, so a kernel that drops or
    misplaces a block of keys fails."""
    torch.manual_seed(hd + nh)
    lengths = [257, 64, 1, 131]
    for dtype in (torch.float32, torch.bfloat16):
        kc, vc, table, dense = _paged(4, lengths, nkv, hd, dtype, seed=hd)
        tok_seq = torch.arange(4, dtype=torch.int32, device="cuda")
        tok_pos = torch.tensor([n - 1 for n in lengths], dtype=torch.int32, device="cuda")
        seq_slot = torch.arange(4, dtype=torch.int32, device="cuda")
        q = (torch.randn(4, nh * hd, device="cuda") * hd ** -0.5).to(dtype)
        # plant: query head 0 of sequence 0 points at key 3 (or at the window's first key)
        far = 3 if window is None else max(0, lengths[0] - window)
        q0 = dense[0][0][far, 0] * (6.0 / hd ** 0.5)
        q[0, :hd] = q0.to(dtype)
        ref = torch.stack([_attn_ref(q[i].float().view(nh, hd), *dense[i], lengths[i] - 1, nh, window).view(-1)
                           for i in range(4)])
        tol = 2e-5 if dtype == torch.float32 else 2 ** -7
        out = torch.zeros(4, nh * hd, device="cuda", dtype=dtype)
        k.attention_ref(q, out, nh, kc, vc, table, 64, tok_pos, tok_seq, seq_slot, window)
        assert (out.float() - ref).abs().max().item() <= tol * max(1.0, ref.abs().max().item())
        if dtype == torch.bfloat16:
            for shares in (1, 3, 8):
                out2 = torch.zeros_like(out)
                k.attention_decode(q, out2, nh, kc, vc, table, 64, tok_pos, tok_seq, seq_slot, window, shares)
                err = (out2.float() - ref).abs().max().item()
                assert err <= tol * max(1.0, ref.abs().max().item()), f"shares={shares}: {err}"


@pytest.mark.parametrize("hd,nh,nkv,window,ring", [(64, 4, 2, None, None), (128, 8, 2, 100, None), (64, 12, 1, None, None),
                                                    (128, 32, 8, None, None), (128, 6, 3, 128, 3), (64, 16, 1, 70, None)])
def test_attention_decode_stream_against_plain(k, hd, nh, nkv, window, ring):
    """The decode kernel that streams pages through shared memory, with sequences of very unequal
    lengths (so that CTAs' ranges cut some (token, kv head) pairs into parts and hold others
    whole), with few and many CTAs (more CTAs than pages: some get none), a window's edge, a ring
    of pages, a planted far key, and scratch memory that starts out as NaN."""
    torch.manual_seed(hd + nh)
    lengths = [700, 64, 1, 131, 65, 2, 300]
    n = len(lengths)
    kc, vc, table, dense = _paged(n, lengths, nkv, hd, torch.bfloat16, seed=hd + 1, ring=ring)
    tok_seq = torch.arange(n, dtype=torch.int32, device="cuda")
    tok_pos = torch.tensor([x - 1 for x in lengths], dtype=torch.int32, device="cuda")
    seq_slot = torch.arange(n, dtype=torch.int32, device="cuda")
    q = (torch.randn(n, nh * hd, device="cuda") * hd ** -0.5).bfloat16()
    far = 3 if window is None else max(0, lengths[0] - window)
    q[0, :hd] = (dense[0][0][far, 0] * (6.0 / hd ** 0.5)).bfloat16()
    ref = torch.stack([_attn_ref(q[i].float().view(nh, hd), *dense[i], lengths[i] - 1, nh, window).view(-1)
                       for i in range(n)])
    k.attention_decode_stream(q, torch.zeros_like(q), nh, kc, vc, table, 64, tok_pos, tok_seq, seq_slot, window)
    for ctas in (None, 1, 2, 7, 500):
        k._decode_stream_scratch[q.device.index].fill_(float("nan"))
        out = torch.zeros_like(q)
        k.attention_decode_stream(q, out, nh, kc, vc, table, 64, tok_pos, tok_seq, seq_slot, window, ctas=ctas)
        err = (out.float() - ref).abs().max().item()
        assert err <= 2 ** -7 * max(1.0, ref.abs().max().item()), f"ctas={ctas}: {err}"
    # rows that belong to no sequence (the slot that pads a captured step), first, in the middle and
    # last: nothing is read for them, their rows are zero, the others as before
    skip = 1000
    for padded in ([0], [2, 3], [5, 6], [0, 1, 2, 3, 4, 5]):
        slots = seq_slot.clone()
        slots[padded] = skip
        for ctas in (None, 3):
            k._decode_stream_scratch[q.device.index].fill_(float("nan"))
            out = torch.full_like(q, 7.0)
            k.attention_decode_stream(q, out, nh, kc, vc, table, 64, tok_pos, tok_seq, slots, window, ctas=ctas, skip_slot=skip)
            want = ref.clone()
            want[padded] = 0
            err = (out.float() - want).abs().max().item()
            assert err <= 2 ** -7 * max(1.0, ref.abs().max().item()), f"padded={padded} ctas={ctas}: {err}"
    assert k.attention_decode_stream_status() == 0
    with pytest.raises(k.KernelError):
        k.attention_decode_stream(q, out, nh, kc, vc, table, 64, tok_pos, tok_seq, seq_slot, window, ctas=5000)


@pytest.mark.parametrize("hd,nh,nkv,window", [(16, 4, 2, None), (32, 6, 3, 40), (48, 5, 1, None), (128, 8, 2, 100),
                                               (64, 12, 12, None), (96, 3, 1, 50), (256, 4, 2, None)])
def test_attention_prefill_against_plain(k, hd, nh, nkv, window):
    """Packed prompts of unequal lengths, some continuing a sequence that is already cached; every
    token against the plain statement.  Sequence 1's last query points at a far key."""
    torch.manual_seed(hd * 3 + nh)
    starts, news = [0, 130, 63, 5], [100, 77, 1, 64]           # cached before the step, brought by the step
    lengths = [s + n for s, n in zip(starts, news)]
    kc, vc, table, dense = _paged(4, lengths, nkv, hd, torch.bfloat16, seed=hd + 1)
    cu = [0]
    for n in news:
        cu.append(cu[-1] + n)
    t = cu[-1]
    q = (torch.randn(t, nh * hd, device="cuda") * hd ** -0.5).bfloat16()
    far = 7 if window is None else lengths[1] - window
    q[cu[2] - 1, :hd] = (dense[1][0][far, 0] * (6.0 / hd ** 0.5)).bfloat16()
    tok_seq = torch.tensor([b for b, n in enumerate(news) for _ in range(n)], dtype=torch.int32, device="cuda")
    tok_pos = torch.tensor([starts[b] + i for b, n in enumerate(news) for i in range(n)], dtype=torch.int32, device="cuda")
    seq_slot = torch.arange(4, dtype=torch.int32, device="cuda")
    out = torch.zeros(t, nh * hd, device="cuda", dtype=torch.bfloat16)
    k.attention_prefill(q, out, nh, kc, vc, table, 64, torch.tensor(cu, dtype=torch.int32, device="cuda"),
                        torch.tensor(starts, dtype=torch.int32, device="cuda"), seq_slot, window)
    ref_kernel = torch.zeros_like(out)
    k.attention_ref(q, ref_kernel, nh, kc, vc, table, 64, tok_pos, tok_seq, seq_slot, window)
    worst = 0.0
    for i in range(t):
        b, pos = int(tok_seq[i]), int(tok_pos[i])
        ref = _attn_ref(q[i].float().view(nh, hd), *dense[b], pos, nh, window).view(-1)
        worst = max(worst, (out[i].float() - ref).abs().max().item() / max(1.0, ref.abs().max().item()))
        assert (ref_kernel[i].float() - ref).abs().max().item() <= 2 ** -7 * max(1.0, ref.abs().max().item())
    assert worst <= 2 ** -7, worst


@pytest.mark.parametrize("m,inter,kk,bn,splits", [(1, 192, 64, None, None), (8, 160, 96, None, None), (40, 1000, 512, None, None),
                                                  (200, 384, 1024, 128, 1), (300, 520, 256, 256, 1), (64, 640, 4096, 64, 4),
                                                  (7, 12288 // 8, 4096, 16, 2), (65, 200, 320, None, None),
                                                  (128, 392, 1024, None, None), (129, 136, 128, None, None)])
def test_gemm_tc_gated(k, m, inter, kk, bn, splits):
    """silu(x gate^T) * (x up^T) in one kernel against the two-step statement."""
    torch.manual_seed(m + inter)
    x = (torch.randn(m, kk, device="cuda") * 0.5).bfloat16()
    w = (torch.randn(2 * inter, kk, device="cuda") * 0.08).bfloat16()
    g = x.float() @ w[:inter].float().T
    u = x.float() @ w[inter:].float().T
    ref = g / (1 + torch.exp(-g)) * u
    out = torch.zeros(m, inter, device="cuda", dtype=torch.bfloat16)
    k.gemm_tc(x, w, out, swiglu=True, bn=bn, splits=splits)
    assert (out.float() - ref).abs().max().item() <= 2 ** -8 * ref.abs().max().item() + 1e-6
    out2 = torch.zeros_like(out)
    k.gemm_swiglu(x, w, out2)          # 65 to 128 tokens: tiles of 128 tokens; more: the prompt kernel
    assert (out2.float() - ref).abs().max().item() <= 2 ** -8 * ref.abs().max().item() + 1e-6
    assert torch.equal(out, out2) or bn is not None or m > 64
    assert k.gemm_tc_status() == 0


@pytest.mark.parametrize("hd,nh,nkv,window", [(64, 4, 2, None), (128, 8, 2, 100), (64, 6, 6, 70), (128, 4, 1, None)])
def test_attention_prefill_tc_against_plain(k, hd, nh, nkv, window):
    """The tcgen05 prompt kernel: packed prompts of unequal lengths (one longer than two tiles,
    one continuing a cached sequence across pages, single tokens), every token against the plain
    statement; a query at the end of a long sequence points at a far key."""
    torch.manual_seed(hd + nh)
    starts, news = [0, 130, 63, 5, 0], [300, 77, 1, 128, 129]
    lengths = [s + n for s, n in zip(starts, news)]
    kc, vc, table, dense = _paged(5, lengths, nkv, hd, torch.bfloat16, seed=hd + 2)
    cu = [0]
    for n in news:
        cu.append(cu[-1] + n)
    t = cu[-1]
    q = (torch.randn(t, nh * hd, device="cuda") * hd ** -0.5).bfloat16()
    far = 7 if window is None else lengths[0] - window
    q[cu[1] - 1, :hd] = (dense[0][0][far, 0] * (6.0 / hd ** 0.5)).bfloat16()
    tok_seq = [b for b, n in enumerate(news) for _ in range(n)]
    tok_pos = [starts[b] + i for b, n in enumerate(news) for i in range(n)]
    seq_slot = torch.arange(5, dtype=torch.int32, device="cuda")
    out = torch.zeros(t, nh * hd, device="cuda", dtype=torch.bfloat16)
    k.attention_prefill_tc(q, out, nh, kc, vc, table, 64, torch.tensor(cu, dtype=torch.int32, device="cuda"),
                           torch.tensor(starts, dtype=torch.int32, device="cuda"), seq_slot, window)
    torch.cuda.synchronize()
    assert k.attention_prefill_tc_status(hd) == 0
    worst, where = 0.0, None
    for i in range(t):
        ref = _attn_ref(q[i].float().view(nh, hd), *dense[tok_seq[i]], tok_pos[i], nh, window).view(-1)
        err = (out[i].float() - ref).abs().max().item() / max(1.0, ref.abs().max().item())
        if err > worst:
            worst, where = err, (tok_seq[i], tok_pos[i])
    assert worst <= 2 ** -7, (worst, where)


def test_attention_decode_at_forty_thousand_keys(k):
    """Both decode kernels far beyond the lengths of the other tests: sequences of 40,000, 9,000 and
    70 positions over shuffled pages, the first query aimed at one key near the start of its
    sequence (a far key among tens of thousands: a page that is skipped, read twice or taken from a
    neighbour's table shows), a window of 5,000 on the same data."""
    torch.manual_seed(11)
    nh, nkv, hd, page = 8, 2, 128, 64
    lengths = [40000, 9000, 70]
    width = -(-max(lengths) // page)
    n_pages = sum(-(-x // page) for x in lengths) + 2
    g = torch.Generator(device="cuda").manual_seed(4)
    kc = torch.randn((n_pages + 1, nkv, page, hd), generator=g, device="cuda").bfloat16()
    vc = torch.randn((n_pages + 1, nkv, hd, page), generator=g, device="cuda").bfloat16()
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(5)) + 1
    table = torch.zeros((len(lengths), width), dtype=torch.int32)
    at = 0
    for s_, x in enumerate(lengths):
        np_ = -(-x // page)
        table[s_, :np_] = perm[at:at + np_]
        at += np_
    table = table.cuda()
    dense = []
    for s_, x in enumerate(lengths):
        pages = table[s_, :-(-x // page)].long()
        ks = kc[pages].permute(0, 2, 1, 3).reshape(-1, nkv, hd)[:x].float()           # [pos, kv, hd]
        vs = vc[pages].permute(0, 3, 1, 2).reshape(-1, nkv, hd)[:x].float()
        dense.append((ks, vs))
    tok_seq = torch.arange(3, dtype=torch.int32, device="cuda")
    tok_pos = torch.tensor([x - 1 for x in lengths], dtype=torch.int32, device="cuda")
    for window, far in ((None, 77), (5000, 40000 - 4990)):
        q = (torch.randn(3, nh * hd, device="cuda") * hd ** -0.5).bfloat16()
        q[0, :hd] = (dense[0][0][far, 0] * (8.0 / hd ** 0.5)).bfloat16()
        ref = torch.stack([_attn_ref(q[i].float().view(nh, hd), *dense[i], lengths[i] - 1, nh, window).view(-1)
                           for i in range(3)])
        # the planted key carries the first head of the first query: without it the result is another
        lo = 0 if window is None else lengths[0] - window
        probs = torch.softmax(dense[0][0][lo:, 0] @ q[0, :hd].float(), 0)
        assert probs[far - lo] > 0.5
        out = torch.zeros_like(q)
        k.attention_decode_stream(q, out, nh, kc, vc, table, page, tok_pos, tok_seq, tok_seq, window)
        assert (out.float() - ref).abs().max().item() <= 2 ** -7 * max(1.0, ref.abs().max().item())
        for shares in (1, 16, 64):
            out = torch.zeros_like(q)
            k.attention_decode(q, out, nh, kc, vc, table, page, tok_pos, tok_seq, tok_seq, window, shares)
            assert (out.float() - ref).abs().max().item() <= 2 ** -7 * max(1.0, ref.abs().max().item()), shares
    assert k.attention_decode_stream_status() == 0


@pytest.mark.parametrize("m,n,kk,mode", [(200, 384, 1024, "bf16"), (300, 520, 256, "acc"), (515, 260, 2048, "bf16"),
                                          (130, 128, 64, "acc"), (1000, 777, 1000, "f32")])
def test_gemm_tc_persistent(k, m, n, kk, mode):
    """The prompt kernel (tiles walked by one CTA per SM, two accumulator buffers), also with so few
    CTAs that each walks many tiles."""
    torch.manual_seed(m + 3 * n)
    x = (torch.randn(m, kk, device="cuda") * 0.5).bfloat16()
    w = (torch.randn(n, kk, device="cuda") * 0.05).bfloat16()
    b = torch.randn(n, device="cuda") if m % 2 else None
    ref = x.float() @ w.float().T + (b if b is not None else 0)
    for bn in (128, 256):
        for ctas in (148, 3):
            if mode == "bf16":
                out, tol, want = torch.zeros(m, n, device="cuda", dtype=torch.bfloat16), 2 ** -8, ref
            elif mode == "f32":
                out, tol, want = torch.zeros(m, n, device="cuda"), 1e-5, ref
            else:
                out, tol, want = torch.ones(m, n, device="cuda"), 1e-5, ref + 1
            k.gemm_tc_persistent(x, w, out, b, accumulate=(mode == "acc"), bn=bn, ctas=ctas)
            assert (out.float() - want).abs().max().item() <= tol * want.abs().max().item() + 1e-6, (bn, ctas)
    inter = n // 2 * 2
    wg = (torch.randn(2 * inter, kk, device="cuda") * 0.08).bfloat16()
    g, u = x.float() @ wg[:inter].float().T, x.float() @ wg[inter:].float().T
    want = g / (1 + torch.exp(-g)) * u
    # gated: a tile is 64 gate rows and 64 up rows; tiles of 256, 128 and 48 tokens (the last: pieces
    # of 16 tokens, which only the gate warps finish), results that TMA can and cannot address
    for bn, ctas in ((None, 5), (None, 148), (128, 148), (48, 7)):
        out = torch.zeros(m, inter, device="cuda", dtype=torch.bfloat16)
        k.gemm_tc_persistent(x, wg, out, swiglu=True, bn=bn, ctas=ctas)
        assert (out.float() - want).abs().max().item() <= 2 ** -8 * want.abs().max().item() + 1e-6, (bn, ctas)
    assert k.gemm_tc_status() == 0


@pytest.mark.parametrize("m,n,kk", [(300, 520, 256), (515, 260, 2048), (1024, 1024, 1536), (700, 130, 72)])
def test_gemm_tc_persistent_split_last_round(k, m, n, kk):
    """A product that adds into its result and whose last round of tiles is not full: that round's
    tiles are cut into parts along the inner dimension, and the CTAs that hold the parts of a tile
    add them in order.  Against float32, against whole tiles, the same bits twice, and the words
    that order the parts back at zero."""
    torch.manual_seed(m + n)
    x = (torch.randn(m, kk, device="cuda") * 0.5).bfloat16()
    w = (torch.randn(n, kk, device="cuda") * 0.05).bfloat16()
    b = torch.randn(n, device="cuda")
    base = torch.randn(m, n, device="cuda")
    want = base + x.float() @ w.float().T + b
    for bn in (128, 256):
        tiles = -(-m // bn) * -(-n // 128)
        for ctas in (2, 3, 5, 7, 11, 148):
            outs = []
            for _ in range(2):
                out = base.clone()
                k.gemm_tc_persistent(x, w, out, b, accumulate=True, bn=bn, ctas=ctas, split_last=True)
                outs.append(out)
            assert torch.equal(outs[0], outs[1]), (bn, ctas)
            assert (outs[0] - want).abs().max().item() <= 1e-5 * want.abs().max().item() + 1e-6, (bn, ctas)
            whole = base.clone()
            k.gemm_tc_persistent(x, w, whole, b, accumulate=True, bn=bn, ctas=ctas, split_last=False)
            assert (outs[0] - whole).abs().max().item() <= 1e-5 * want.abs().max().item() + 1e-6, (bn, ctas)
            if tiles % ctas == 0 or kk < 2 * 4 * 64:
                assert torch.equal(outs[0], whole)      # nothing to cut: the same walk
    assert int(k._part_flags[x.device.index].abs().sum()) == 0
    assert k.gemm_tc_status() == 0


def test_dependent_launch_chain(k):
    """The builds with programmatic dependent launch, which let a kernel start under the one before
    it: a chain in which every kernel reads what the kernel before wrote (norm -> product ->
    accumulating product -> norm), repeated on the same buffers, against the same chain computed
    in float32.  A kernel that read or overwrote too early would show as a difference."""
    from gemmars_b200.csrc import build
    torch.manual_seed(5)
    t, h, inter = 333, 512, 768
    x0 = (torch.randn(t, h, device="cuda") * 0.5)
    w_norm = (torch.rand(h, device="cuda") + 0.5).bfloat16().float()
    w1 = (torch.randn(2 * inter, h, device="cuda") * 0.05).bfloat16()
    w2 = (torch.randn(h, inter, device="cuda") * 0.05).bfloat16()

    def plain(x):
        for _ in range(3):
            n = (x * torch.rsqrt((x * x).mean(-1, keepdim=True) + 1e-6) * w_norm).bfloat16().float()
            g, u = n @ w1[:inter].float().T, n @ w1[inter:].float().T
            a = (g / (1 + torch.exp(-g)) * u).bfloat16().float()
            x = x + a @ w2.float().T
        return x

    want = plain(x0.clone())
    build.set_pdl(True)
    try:
        x = x0.clone()
        n = torch.empty(t, h, device="cuda", dtype=torch.bfloat16)
        a = torch.empty(t, inter, device="cuda", dtype=torch.bfloat16)
        for _ in range(3):
            k.rmsnorm(x, w_norm, n, 1e-6)
            k.gemm_swiglu(n, w1, a)
            k.gemm(a, w2, x, accumulate=True)
    finally:
        build.set_pdl(False)
    assert (x - want).abs().max().item() <= 2e-2 * want.abs().max().item()
    assert k.gemm_tc_status() == 0


@pytest.mark.parametrize("m,nh,nkv,kk,splits,bias,norm,rope", [(8, 4, 2, 512, None, False, True, True), (1, 2, 1, 256, 1, True, True, True),
                                                                (31, 3, 3, 1024, 4, True, False, True), (32, 8, 0, 512, 8, False, True, False)])
def test_gemm_qkv_against_product_then_head_kernel(k, m, nh, nkv, kk, splits, bias, norm, rope):
    """The q/k/v product with norm, rotation, scale and cache write in its epilogue, against the
    product in float32 followed by the same steps in PyTorch; the cache must get exactly the step's
    rows and nothing else."""
    torch.manual_seed(m + nh)
    hd, n = 128, (nh + 2 * nkv) * 128
    x = (torch.randn(m, kk, device="cuda") * 0.5).bfloat16()
    w = (torch.randn(n, kk, device="cuda") * 0.05).bfloat16()
    b = torch.randn(n, device="cuda") * 0.1 if bias else None
    qw, kw = (torch.rand(hd, device="cuda") + 0.5, torch.rand(hd, device="cuda") + 0.5) if norm else (None, None)
    inv = ((1.0 / torch.pow(torch.tensor(1e4, dtype=torch.float64), torch.arange(hd // 2, dtype=torch.float64) * 2 / hd))
           .float().cuda() if rope else None)
    eps, scale = 1e-5, hd ** -0.5
    lengths = [70 + i for i in range(m)]                  # token i is position 69 + i of sequence i
    kc, vc, table, _ = _paged(m, lengths, max(nkv, 1), hd, torch.bfloat16, seed=3)
    kc.zero_(); vc.zero_()
    tok_pos = torch.tensor([n_ - 1 for n_ in lengths], dtype=torch.int32, device="cuda")
    tok_seq = torch.arange(m, dtype=torch.int32, device="cuda")
    qkv = torch.zeros(m, n, device="cuda", dtype=torch.bfloat16)
    k.gemm_qkv(x, w, b, qkv, nh, nkv, hd, qw, kw, eps, inv, scale, tok_pos, tok_seq, tok_seq,
               table if nkv else None, 64, kc if nkv else None, vc if nkv else None, splits=splits)
    ref = (x.float() @ w.float().T + (b if bias else 0)).view(m, nh + 2 * nkv, hd)

    def head(v, wt, pos, s):
        if norm:
            v = v * torch.rsqrt((v * v).mean() + eps) * wt
        if rope:
            ang = (torch.tensor(float(pos), device="cuda") * inv).double()
            a, bb = v[:64].double(), v[64:].double()
            v = torch.cat([a * torch.cos(ang) - bb * torch.sin(ang), bb * torch.cos(ang) + a * torch.sin(ang)]).float()
        return v * s
    got = qkv.float().view(m, nh + 2 * nkv, hd)
    tol = 2 ** -7
    for i in range(m):
        pos = int(tok_pos[i])
        page = int(table[i, pos // 64])
        for h in range(nh):
            want = head(ref[i, h], qw, pos, scale)
            assert (got[i, h] - want).abs().max().item() <= tol * max(1.0, want.abs().max().item())
        for h in range(nkv):
            want = head(ref[i, nh + h], kw, pos, 1.0)
            assert (kc[page, h, pos % 64].float() - want).abs().max().item() <= tol * max(1.0, want.abs().max().item())
            wantv = ref[i, nh + nkv + h]
            assert (vc[page, h, :, pos % 64].float() - wantv).abs().max().item() <= tol * max(1.0, wantv.abs().max().item())
    if nkv:
        assert int((kc.abs().sum(dim=(1, 3)) > 0).sum()) == m    # one row per token and no other
        assert float(kc[0].abs().sum()) == 0.0
    assert k.gemm_tc_status() == 0


def test_a_bounded_wait_that_runs_out_is_reported_and_leaves_the_context_usable(k):
    """A test build of the product kernel (-DGB_TEST_WITHHOLD_LOAD) never asks for the last block
    of tokens, so the wait for that block, shortened to 2^14 polls (-DGB_TEST_WAIT_LIMIT), runs
    out.  The kernel must not hang, trap or fault: it records the wait that gave up in its status
    word, frees its tensor memory and returns; ``check_status`` then raises, and the next
    ordinary launch on the same context is right and leaves the word clear."""
    from ctypes import c_int, c_longlong, c_void_p
    from gemmars_b200.csrc import build
    lib = build.load("gemm_tc", (("GB_TEST_WAIT_LIMIT", 1 << 14), ("GB_TEST_WITHHOLD_LOAD", 1)))
    f = lib.gb_gemm_tc
    f.restype = c_int
    f.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_longlong, c_longlong, c_int,
                  c_int, c_int, c_void_p]
    torch.manual_seed(0)
    m, n, kk = 8, 256, 512
    x = (torch.randn(m, kk, device="cuda") * 0.5).bfloat16()
    w = (torch.randn(n, kk, device="cuda") * 0.05).bfloat16()
    out = torch.zeros(m, n, device="cuda", dtype=torch.bfloat16)
    assert k.gemm_tc_status() == 0
    rc = f(x.data_ptr(), w.data_ptr(), None, out.data_ptr(), 0, m, n, kk, x.stride(0), out.stride(0), 16, 1, 4,
           torch.cuda.current_stream().cuda_stream)
    assert rc == 0                              # the launch itself is fine
    torch.cuda.synchronize()                    # and the kernel comes back
    with pytest.raises(k.KernelError, match="bounded wait ran out.*code 1"):
        k.check_status()
    k.check_status()                            # reading the word cleared it
    good = torch.zeros_like(out)
    k.gemm_tc(x, w, good)
    ref = x.float() @ w.float().T
    assert (good.float() - ref).abs().max().item() <= 2 ** -8 * ref.abs().max().item()
    assert not torch.equal(good, out)           # the launch that gave up did not finish its product
    assert k.gemm_tc_status() == 0


@pytest.mark.parametrize("nh,nkv,kk,bias,norm,rope,lengths,starts", [
    (4, 2, 512, False, True, True, [300], [0]),                       # one prompt, aligned: the fast value stores
    (3, 1, 256, True, True, True, [70, 1, 33, 150], [0, 5, 64, 37]),     # packed, unaligned, continuing sequences
    (2, 2, 1024, True, False, True, [129], [1000]),                    # no norm; a continuation at an odd place
    (2, 1, 512, False, True, False, [65, 65], [0, 31]),                # no rotation
    (5, 0, 512, True, True, True, [200], [3]),                         # queries only (a layer that reads another's cache)
])
def test_gemm_qkv_prompt_against_product_then_head_kernel(k, nh, nkv, kk, bias, norm, rope, lengths, starts):
    """The q/k/v product of a prompt step with norm, rotation, scale and cache write in its epilogue,
    against the plain product followed by the per-head kernel: the queries and the whole cache
    (so that nothing strays), for packed sequences that start at odd places, cross pages, and end
    in the middle of a tile."""
    torch.manual_seed(nh + kk)
    hd, n = 128, (nh + 2 * nkv) * 128
    m = sum(lengths)
    x = (torch.randn(m, kk, device="cuda") * 0.5).bfloat16()
    w = (torch.randn(n, kk, device="cuda") * 0.05).bfloat16()
    b = (torch.randn(n, device="cuda") * 0.1) if bias else None
    qw = (torch.rand(hd, device="cuda") + 0.5) if norm else None
    kw = (torch.rand(hd, device="cuda") + 0.5) if norm else None
    inv = (1.0 / (1e4 ** (torch.arange(64, dtype=torch.float64) / 64.0))).float().cuda() if rope else None
    eps, scale = 1e-6, hd ** -0.5
    tok_pos = torch.tensor([s + i for s, l in zip(starts, lengths) for i in range(l)], dtype=torch.int32, device="cuda")
    tok_seq = torch.tensor([q for q, l in enumerate(lengths) for _ in range(l)], dtype=torch.int32, device="cuda")
    slots = torch.arange(len(lengths), dtype=torch.int32, device="cuda")
    width = max(-(-(s + l) // 64) for s, l in zip(starts, lengths))
    pages = len(lengths) * width
    table = (torch.randperm(pages, generator=torch.Generator().manual_seed(1)) + 1).to(torch.int32).view(len(lengths), width).cuda()
    caches = []
    for fused in (False, True):
        kc = torch.zeros((pages + 1, max(nkv, 1), 64, hd), device="cuda", dtype=torch.bfloat16)
        vc = torch.zeros((pages + 1, max(nkv, 1), hd, 64), device="cuda", dtype=torch.bfloat16)
        if fused:
            q = torch.full((m, nh * hd), 9.0, device="cuda", dtype=torch.bfloat16)
            place = k.token_place(tok_pos, tok_seq, slots, table, 64) if nkv else None
            k.gemm_qkv_prompt(x, w, b, q, nh, nkv, hd, qw, kw, eps, k.rope_table(tok_pos, inv) if rope else None, scale,
                              place, 64, kc if nkv else None, vc if nkv else None)
        else:
            qkv = torch.zeros(m, n, device="cuda", dtype=torch.bfloat16)
            k.gemm(x, w, qkv, b)
            flags = (k.FLAG_NORM if norm else 0) | (k.FLAG_ROPE if rope else 0) | (k.FLAG_CACHE if nkv else 0) | k.FLAG_INPLACE
            k.head_norm_rope_cache(qkv, nh, nkv, hd, hd if rope else 0, qw, kw, eps, inv, scale, tok_pos, tok_seq, slots,
                                   table if nkv else None, 64, kc if nkv else None, vc if nkv else None, flags)
            q = qkv[:, :nh * hd]
        caches.append((q.float().clone(), kc.float().clone(), vc.float().clone()))
    (q0, k0, v0), (q1, k1, v1) = caches
    # the unfused path rounds the product to bfloat16 before the per-head work, the fused one does not
    for a, c, what in ((q0, q1, "queries"), (k0, k1, "keys"), (v0, v1, "values")):
        tol = 2 ** -6 * max(1.0, a.abs().max().item())
        assert (a - c).abs().max().item() <= tol, what
    assert float(k1[0].abs().sum()) == 0.0 and float(v1[0].abs().sum()) == 0.0          # nothing strays into page 0
    assert torch.equal(k0 != 0, k1 != 0) or (k0 - k1).abs().max().item() <= 2 ** -6      # the same places are written
    assert k.gemm_tc_status() == 0


@pytest.mark.parametrize("m,h,inter,bias", [(1, 256, 384, False), (8, 512, 640, True), (16, 384, 512, False), (33, 256, 896, True),
                                            (64, 512, 256, False)])
def test_a_norm_taken_into_the_products_around_it(k, m, h, inter, bias):
    """The product that adds into the residual also leaves bfloat16(residual * norm weight) and the
    rows' sums of squares; the products after it (plain, gated, and q/k/v with the per-head work)
    scale their results by each row's rstd.  Against the residual, an RMSNorm and the products
    stated in PyTorch float32."""
    torch.manual_seed(m + h)
    eps = 1e-5
    a = (torch.randn(m, inter, device="cuda") * 0.5).bfloat16()
    w_down = (torch.randn(h, inter, device="cuda") * 0.05).bfloat16()
    b_down = (torch.randn(h, device="cuda") * 0.1) if bias else None
    g = torch.rand(h, device="cuda") + 0.5
    residual = torch.randn(m, h, device="cuda") * 2
    want_res = residual + a.float() @ w_down.float().T + (b_down if bias else 0)
    res = residual.clone()
    left = k.gemm_tc(a, w_down, res, b_down, accumulate=True, splits=4, link_out=(g, eps))
    assert (res - want_res).abs().max().item() <= 1e-4 * want_res.abs().max().item()
    normed = want_res * (want_res.pow(2).mean(-1, keepdim=True) + eps).rsqrt() * g
    got_normed = left.materialize().float()
    assert (got_normed - normed).abs().max().item() <= 2 ** -7 * normed.abs().max().item()
    assert left.partial.shape == (-(-h // 128), 64)
    # a plain product after the norm
    w2 = (torch.randn(200, h, device="cuda") * 0.05).bfloat16()
    b2 = torch.randn(200, device="cuda") * 0.1
    out = torch.zeros(m, 200, device="cuda", dtype=torch.bfloat16)
    k.gemm_tc(left.rows, w2, out, b2, link_in=left)
    ref = normed @ w2.float().T + b2
    assert (out.float() - ref).abs().max().item() <= 2 ** -6 * ref.abs().max().item()
    # with the inner dimension split as well
    out.zero_()
    k.gemm_tc(left.rows, w2, out, b2, link_in=left, splits=2)
    assert (out.float() - ref).abs().max().item() <= 2 ** -6 * ref.abs().max().item()
    # the gated product after the norm
    wgu = (torch.randn(2 * 320, h, device="cuda") * 0.05).bfloat16()
    act = torch.zeros(m, 320, device="cuda", dtype=torch.bfloat16)
    for splits in (1, 2):
        act.zero_()
        k.gemm_tc(left.rows, wgu, act, swiglu=True, link_in=left, splits=splits)
        gate, up = normed @ wgu[:320].float().T, normed @ wgu[320:].float().T
        ref_act = torch.nn.functional.silu(gate) * up
        assert (act.float() - ref_act).abs().max().item() <= 2 ** -6 * max(1.0, ref_act.abs().max().item()), splits
    # the q/k/v product with the per-head work in its epilogue (queries only: no cache here)
    nh, hd = 2, 128
    wq = (torch.randn(nh * hd, h, device="cuda") * 0.05).bfloat16()
    qw = torch.rand(hd, device="cuda") + 0.5
    tok_pos = torch.arange(m, dtype=torch.int32, device="cuda")
    tok_seq = torch.zeros(m, dtype=torch.int32, device="cuda")
    q = torch.zeros(m, nh * hd, device="cuda", dtype=torch.bfloat16)
    k.gemm_qkv(left.rows, wq, None, q, nh, 0, hd, qw, qw, 1e-6, None, 0.5, tok_pos, tok_seq, tok_seq, None, 64, None, None,
               link_in=left)
    z = (normed @ wq.float().T).view(m, nh, hd)
    ref_q = (z * (z.pow(2).mean(-1, keepdim=True) + 1e-6).rsqrt() * qw * 0.5).view(m, nh * hd)
    assert (q.float() - ref_q).abs().max().item() <= 2 ** -6 * ref_q.abs().max().item()
    assert k.gemm_tc_status() == 0
