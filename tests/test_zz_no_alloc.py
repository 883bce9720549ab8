"""The decode-attention entry point that allocates nothing (gb_attention_decode_static).

Some hosts of the library cannot allocate device memory: they run inside a process that gave
all of it to its own pool, or they are not allowed to call cudaMalloc at all.  For them the
library keeps the split-attention scratch in a fixed 4 MiB device array.  This test calls that
entry point through its exported C symbol, twice in a row with different batches (the array
keeps what the first call left, which must not matter), and compares each result with a plain
float32 statement of attention and, bit for bit, with the ordinary entry point, which takes its
scratch from the caller.  It also checks that no device memory is taken, that one share (no
scratch) works, and where exactly the size limit lies.  It is collected last on purpose.
"""
from ctypes import c_int, c_longlong, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu

STATIC_FLOATS = 1 << 20
ERR_SIZE = -3
ERR_STATIC_SCRATCH = -5


def _cache(lengths, nkv, hd, seed):
    """A paged cache (pages handed out from the top down) and, per sequence, its keys and
    values as dense float32 [len, nkv, hd]."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    width = max(-(-n // 64) for n in lengths)
    pages = sum(-(-n // 64) for n in lengths)
    kc = torch.randn((pages + 1, nkv, 64, hd), generator=g, device="cuda").bfloat16()
    vc = torch.randn((pages + 1, nkv, hd, 64), generator=g, device="cuda").bfloat16()
    table = torch.zeros((len(lengths) + 1, width), dtype=torch.int32)
    nxt, dense = pages, []
    for s, n in enumerate(lengths):
        mine = []
        for lp in range(-(-n // 64)):
            table[s, lp] = nxt
            mine.append(nxt)
            nxt -= 1
        ks = torch.cat([kc[p].float().permute(1, 0, 2) for p in mine])[:n]      # [len, nkv, hd]
        vs = torch.cat([vc[p].float().permute(2, 0, 1) for p in mine])[:n]
        dense.append((ks, vs))
    return kc, vc, table.cuda(), dense


def _plain_attention(q, ks, vs, nh, window):
    """softmax(q K^T) V of the last position over the keys it may see; q [nh, hd] float32."""
    n, nkv = ks.shape[0], ks.shape[1]
    lo = max(0, n - window) if window else 0
    out = torch.zeros_like(q)
    for h in range(nh):
        g = h // (nh // nkv)
        out[h] = torch.softmax(ks[lo:, g] @ q[h], 0) @ vs[lo:, g]
    return out


def _entry(hd):
    from gemmars_b200.csrc import build
    lib = build.load("attention_decode", (("GB_HEAD_DIM", hd),))
    fn = lib.gb_attention_decode_static                     # the exported C symbol
    fn.restype = c_int
    fn.argtypes = [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                   c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]
    return fn


def _call(fn, q, out, kc, vc, table, nkv, hd, tok_pos, tok_seq, nh, window, shares):
    return fn(q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0), kc.data_ptr(), vc.data_ptr(), table.data_ptr(),
              table.shape[1], 64, nkv, hd, tok_pos.data_ptr(), tok_seq.data_ptr(), tok_seq.data_ptr(), q.shape[0], nh,
              window or 0, shares, torch.cuda.current_stream().cuda_stream)


def test_static_entry_point_matches_the_ordinary_one():
    from gemmars_b200 import kernels
    hd, nh, nkv = 64, 8, 2
    fn = _entry(hd)
    for call, (lengths, shares, window) in enumerate([([700, 64, 333, 1], 5, None), ([129, 1000], 3, 200),
                                                      ([500, 77], 1, None)]):
        torch.manual_seed(call)
        kc, vc, table, dense = _cache(lengths, nkv, hd, seed=call)
        n = len(lengths)
        tok_seq = torch.arange(n, dtype=torch.int32, device="cuda")
        tok_pos = torch.tensor([x - 1 for x in lengths], dtype=torch.int32, device="cuda")
        q = (torch.randn(n, nh * hd, device="cuda") * hd ** -0.5).bfloat16()
        # one key far back stands out for head 0 of the first sequence: a share that is lost shows
        far = 3 if not window else lengths[0] - window
        q[0, :hd] = (dense[0][0][far, 0] * (6.0 / hd ** 0.5)).bfloat16()
        plain = torch.stack([_plain_attention(q[i].float().view(nh, hd), *dense[i], nh, window).view(-1)
                             for i in range(n)])
        ordinary = torch.zeros(n, nh * hd, device="cuda", dtype=torch.bfloat16)
        kernels.attention_decode(q, ordinary, nh, kc, vc, table, 64, tok_pos, tok_seq, tok_seq, window, shares)
        got = torch.zeros_like(ordinary)
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        rc = _call(fn, q, got, kc, vc, table, nkv, hd, tok_pos, tok_seq, nh, window, shares)
        assert rc == 0, f"call {call}: returned {rc}"
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before          # nothing was allocated on the device
        scale = max(1.0, plain.abs().max().item())
        assert (got.float() - plain).abs().max().item() <= 2 ** -7 * scale, f"call {call}"
        assert torch.equal(got, ordinary), f"call {call}: differs from the ordinary entry point"


def test_static_entry_point_limit():
    """The largest batch that fits is accepted and right; one share more is refused with the
    scratch code and nothing runs; sizes that are no sizes are refused as such."""
    hd, nh, nkv, n = 64, 8, 2, 64
    fn = _entry(hd)
    lengths = [2100 - 17 * i for i in range(n)]
    kc, vc, table, dense = _cache(lengths, nkv, hd, seed=7)
    tok_seq = torch.arange(n, dtype=torch.int32, device="cuda")
    tok_pos = torch.tensor([x - 1 for x in lengths], dtype=torch.int32, device="cuda")
    torch.manual_seed(7)
    q = (torch.randn(n, nh * hd, device="cuda") * hd ** -0.5).bfloat16()
    fits = STATIC_FLOATS // (n * nh * (hd + 2))                 # 31 shares: 1,047,552 of 1,048,576 floats
    assert n * nh * fits * (hd + 2) <= STATIC_FLOATS < n * nh * (fits + 1) * (hd + 2)
    got = torch.zeros(n, nh * hd, device="cuda", dtype=torch.bfloat16)
    assert _call(fn, q, got, kc, vc, table, nkv, hd, tok_pos, tok_seq, nh, None, fits) == 0
    torch.cuda.synchronize()
    plain = torch.stack([_plain_attention(q[i].float().view(nh, hd), *dense[i], nh, None).view(-1) for i in range(n)])
    assert (got.float() - plain).abs().max().item() <= 2 ** -7 * max(1.0, plain.abs().max().item())
    untouched = torch.full_like(got, 3.0)
    assert _call(fn, q, untouched, kc, vc, table, nkv, hd, tok_pos, tok_seq, nh, None, fits + 1) == ERR_STATIC_SCRATCH
    # numbers that would wrap a 64-bit product are refused one by one, not multiplied
    assert _call(fn, q, untouched, kc, vc, table, nkv, hd, tok_pos, tok_seq, nh, None, 1 << 30) == ERR_SIZE
    assert _call(fn, q, untouched, kc, vc, table, nkv, hd + 16, tok_pos, tok_seq, nh, None, 2) == ERR_SIZE
    torch.cuda.synchronize()
    assert float((untouched.float() - 3.0).abs().max()) == 0.0
