"""The decode-attention entry point that allocates nothing (gb_attention_decode_static).

Some hosts of the library cannot allocate device memory: they run inside a process that gave
all of it to its own pool, or they are not allowed to call cudaMalloc at all.  For them the
library keeps the split-attention scratch in a fixed 4 MiB device array.  This test calls that
entry point through its exported C symbol, twice in a row with different batches (the array
keeps what the first call left, which must not matter), and compares with the ordinary entry
point, which takes its scratch from the caller.  It is collected last on purpose.
"""
import ctypes
from ctypes import c_int, c_longlong, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu

STATIC_FLOATS = 1 << 20
ERR_STATIC_SCRATCH = -5


def _cache(lengths, nkv, hd, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    width = max(-(-n // 64) for n in lengths)
    pages = sum(-(-n // 64) for n in lengths)
    kc = torch.randn((pages + 1, nkv, 64, hd), generator=g, device="cuda").bfloat16()
    vc = torch.randn((pages + 1, nkv, hd, 64), generator=g, device="cuda").bfloat16()
    table = torch.zeros((len(lengths) + 1, width), dtype=torch.int32)
    nxt = pages
    for s, n in enumerate(lengths):
        for lp in range(-(-n // 64)):
            table[s, lp] = nxt
            nxt -= 1
    return kc, vc, table.cuda()


def test_static_entry_point_matches_the_ordinary_one():
    from gemmars_b200 import kernels
    from gemmars_b200.csrc import build
    hd, nh, nkv = 64, 8, 2
    lib = build.load("attention_decode", (("GB_HEAD_DIM", hd),))
    fn = lib.gb_attention_decode_static                     # the exported C symbol
    fn.restype = c_int
    fn.argtypes = [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                   c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]
    stream = torch.cuda.current_stream().cuda_stream
    for call, (lengths, shares, window) in enumerate([([700, 64, 333, 1], 5, None), ([129, 1000], 3, 200)]):
        torch.manual_seed(call)
        kc, vc, table = _cache(lengths, nkv, hd, seed=call)
        n = len(lengths)
        tok_seq = torch.arange(n, dtype=torch.int32, device="cuda")
        tok_pos = torch.tensor([x - 1 for x in lengths], dtype=torch.int32, device="cuda")
        q = (torch.randn(n, nh * hd, device="cuda") * hd ** -0.5).bfloat16()
        want = torch.zeros(n, nh * hd, device="cuda", dtype=torch.bfloat16)
        kernels.attention_decode(q, want, nh, kc, vc, table, 64, tok_pos, tok_seq, tok_seq, window, shares)
        got = torch.zeros_like(want)
        free_before = torch.cuda.mem_get_info()[0]
        rc = fn(q.data_ptr(), q.stride(0), got.data_ptr(), got.stride(0), kc.data_ptr(), vc.data_ptr(), table.data_ptr(),
                table.shape[1], 64, nkv, hd, tok_pos.data_ptr(), tok_seq.data_ptr(), tok_seq.data_ptr(), n, nh,
                window or 0, shares, stream)
        assert rc == 0, f"call {call}: returned {rc}"
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before          # nothing was allocated on the device
        scale = max(1.0, want.float().abs().max().item())
        assert (got.float() - want.float()).abs().max().item() <= 2 ** -7 * scale
    # one share needs no scratch at all; too large a batch is refused with its own code, nothing runs
    rc = fn(q.data_ptr(), q.stride(0), got.data_ptr(), got.stride(0), kc.data_ptr(), vc.data_ptr(), table.data_ptr(),
            table.shape[1], 64, nkv, hd, tok_pos.data_ptr(), tok_seq.data_ptr(), tok_seq.data_ptr(), n, nh, 0, 1, stream)
    assert rc == 0
    too_many = STATIC_FLOATS // (n * nh * (hd + 2)) + 1
    rc = fn(q.data_ptr(), q.stride(0), got.data_ptr(), got.stride(0), kc.data_ptr(), vc.data_ptr(), table.data_ptr(),
            table.shape[1], 64, nkv, hd, tok_pos.data_ptr(), tok_seq.data_ptr(), tok_seq.data_ptr(), n, nh, 0, too_many,
            stream)
    assert rc == ERR_STATIC_SCRATCH
    torch.cuda.synchronize()
