"""Python faces of the CUDA units: argument checks, then one call into the compiled library.

Every function here works on CUDA tensors only and launches on PyTorch's current stream.  There
is no CPU or library fallback: a tensor that is not on a CUDA device, or a unit that cannot be
built, raises.

Two kernels keep scratch memory per device between their launches (the decode attention's parts,
the words that order the parts of a split prompt tile): work for one device is therefore launched
on one stream at a time, as the engine does; two engines on one device take turns.
"""
from __future__ import annotations

from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from .csrc import build

F32, BF16 = 0, 1
OUT_STORE, OUT_ACCUMULATE = 0, 1
FLAG_NORM, FLAG_ROPE, FLAG_CACHE, FLAG_INPLACE, FLAG_SINGLE = 1, 2, 4, 8, 32
MAX_TOP_K = 1024

_ERRORS = {-2: "unsupported element type", -3: "unsupported size", -4: "missing argument"}


class KernelError(RuntimeError):
    pass


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    raise KernelError(f"element type {dt} is not supported by the CUDA kernels (float32 or bfloat16)")


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _stream():
    # the raw handle of the current stream of the current device (what
    # torch.cuda.current_stream().cuda_stream gives, without building a Stream object per launch)
    return torch._C._cuda_getCurrentRawStream(torch.cuda.current_device())


_launches = [0]


def launch_count() -> int:
    """Kernels of this package launched so far (launches replayed from CUDA graphs included)."""
    return _launches[0]


def count_launches(n: int) -> None:
    _launches[0] += n


# Timing for --profile: an event after every launch; the time between two events is put down to
# the later kernel (kernels of one stream run one after the other).  Every face also says which
# category its kernel belongs to and how many bytes the launch has to move (weights, inputs,
# results, cached keys and values where the host knows the lengths), so that the report can give
# time, calls, bytes and bandwidth per category as the reference's does (src/prof.rs:8-83).
CATEGORIES = ("matmul", "attention", "norm", "elementwise", "embed", "lm_head", "sampling")
_profile = {"on": False, "events": [], "category": None}


def profile_start() -> None:
    """Starts collecting one CUDA event per launch (use without CUDA graphs)."""
    _profile["on"], _profile["events"] = True, []
    ev = torch.cuda.Event(enable_timing=True)
    ev.record()
    _profile["events"].append(("start", None, 0, ev))


class profile_category:
    """Within the block, launches are put down to ``name`` whatever their own category (the
    output head's product is a matmul that the report lists on its own)."""

    def __init__(self, name: str):
        self.name, self.before = name, None

    def __enter__(self):
        self.before, _profile["category"] = _profile["category"], self.name

    def __exit__(self, *exc):
        _profile["category"] = self.before


def profile_totals() -> dict:
    """{"kernels": {name: [calls, ms]}, "categories": {name: [calls, ms, bytes]}} since
    profile_start; stops collecting.  Synchronizes."""
    _profile["on"] = False
    torch.cuda.synchronize()
    ev = _profile["events"]
    per_kernel, per_cat = {}, {}
    for (_, _, _, a), (name, cat, nbytes, b) in zip(ev, ev[1:]):
        ms = a.elapsed_time(b)
        t = per_kernel.setdefault(name, [0, 0.0])
        t[0] += 1
        t[1] += ms
        c = per_cat.setdefault(cat, [0, 0.0, 0])
        c[0] += 1
        c[1] += ms
        c[2] += nbytes
    _profile["events"] = []
    return {"kernels": per_kernel, "categories": per_cat}


def profile_report(tokens: int = 1, totals: Optional[dict] = None) -> str:
    """The time since profile_start per category and per kernel, in the manner of the
    reference's --profile (src/prof.rs:51-83): ms a token, calls a token, us a call, and for the
    categories the bytes a token and the bandwidth they come to.  ``tokens``: the forward tokens
    that ran meanwhile."""
    totals = totals or profile_totals()
    tokens = max(1, tokens)
    whole = sum(t[1] for t in totals["kernels"].values()) or 1.0
    lines = [f"[profile over {tokens} forward tokens, {whole / tokens:.3f} ms/token on the device]",
             f"{'category':14s} {'ms/tok':>9s} {'calls/tok':>10s} {'us/call':>9s} {'MB/tok':>10s} {'GB/s':>8s} {'share':>7s}"]
    for cat in CATEGORIES + tuple(c for c in totals["categories"] if c not in CATEGORIES):
        if cat not in totals["categories"]:
            continue
        calls, ms, nbytes = totals["categories"][cat]
        lines.append(f"{str(cat):14s} {ms / tokens:9.4f} {calls / tokens:10.2f} {ms * 1e3 / calls:9.1f} "
                     f"{nbytes / tokens / 1e6:10.4f} {nbytes / max(ms, 1e-9) / 1e6:8.1f} {100 * ms / whole:6.1f}%")
    lines.append(f"{'kernel':28s} {'ms/tok':>9s} {'calls/tok':>10s} {'us/call':>9s} {'share':>7s}")
    for name, (calls, ms) in sorted(totals["kernels"].items(), key=lambda kv: -kv[1][1]):
        lines.append(f"{name:28s} {ms / tokens:9.4f} {calls / tokens:10.2f} {ms * 1e3 / calls:9.1f} {100 * ms / whole:6.1f}%")
    lines.append(f"{'total':28s} {whole / tokens:9.4f}")
    return "\n".join(lines)


def _check(code: int, what: str, category: str = "elementwise", nbytes: int = 0):
    if code == 0:
        _launches[0] += 1
        if _profile["on"]:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            _profile["events"].append((what, _profile["category"] or category, nbytes, ev))
        return
    if code < 0:
        raise KernelError(f"{what}: {_ERRORS.get(code, 'refused')} (code {code})")
    raise KernelError(f"{what}: CUDA launch failed with error {code}")


def _nbytes(*tensors) -> int:
    """Bytes of the given tensors (None counts nothing): what a launch reads and writes."""
    return sum(t.numel() * t.element_size() for t in tensors if t is not None) if _profile["on"] else 0


def _cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("the kernels of gemmars_b200 run on CUDA tensors only (got a CPU tensor); "
                              "there is no CPU path")


_sigs = {}


def _fn(unit: str, name: str, argtypes, defines=()):
    if build.pdl():
        defines = tuple(defines) + (build.PDL_DEFINE,)
    key = (unit, name, tuple(defines))
    f = _sigs.get(key)
    if f is None:
        lib = build.load(unit, defines)
        f = getattr(lib, name)
        f.argtypes = argtypes
        f.restype = c_int
        _sigs[key] = f
    return f


# --------------------------------------------------------------------------- elementwise

def embed_gather(table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor, scale: float = 1.0):
    """out[t] = table[tokens[t]] * scale; out is the float32 residual stream [T, H]."""
    _cuda(table, tokens, out)
    assert tokens.dtype == torch.int32 and out.dtype == torch.float32 and out.is_contiguous() and table.is_contiguous()
    f = _fn("elementwise", "gb_embed_gather",
            [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p])
    _check(f(table.data_ptr(), dtype_code(table.dtype), tokens.data_ptr(), out.data_ptr(), tokens.numel(),
             table.shape[1], table.shape[0], scale, _stream()), "embed_gather", "embed",
           _nbytes(out) + tokens.numel() * table.shape[1] * table.element_size())


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, eps: float,
            rows_index: Optional[torch.Tensor] = None):
    """out[r] = rmsnorm(x[rows_index[r] or r]) * weight.  x float32 [*, n]; weight float32 [n]."""
    _cuda(x, weight, out, rows_index)
    assert x.dtype == torch.float32 and weight.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous()
    n = x.shape[-1]
    rows = out.numel() // n
    assert weight.numel() == n and out.shape[-1] == n
    if rows_index is not None:
        assert rows_index.dtype == torch.int32 and rows_index.numel() == rows
    f = _fn("elementwise", "gb_rmsnorm",
            [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_float, c_void_p])
    _check(f(x.data_ptr(), weight.data_ptr(), out.data_ptr(), dtype_code(out.dtype), _ptr(rows_index), rows, n,
             eps, _stream()), "rmsnorm", "norm", _nbytes(out, weight) + rows * n * 4)


def head_norm_rope_cache(qkv, nh, nkv, hd, rot, q_weight, k_weight, eps, inv_freq, q_scale, tok_pos, tok_seq,
                         seq_slot, page_table, page_size, kcache, vcache, flags):
    """Per-head RMSNorm, rotation and scale of q and k in place in ``qkv`` [T, (nh+2nkv)*hd], and
    the write of k and v into the paged cache; ``flags`` selects the steps."""
    _cuda(qkv, q_weight, k_weight, inv_freq, tok_pos, tok_seq, seq_slot, page_table, kcache, vcache)
    assert qkv.is_contiguous() and qkv.shape[-1] == (nh + 2 * nkv) * hd
    if flags & FLAG_CACHE:
        assert kcache.dtype == qkv.dtype and vcache.dtype == qkv.dtype and kcache.is_contiguous()
        assert kcache.shape[1:] == (nkv, page_size, hd)
    f = _fn("elementwise", "gb_head_norm_rope_cache",
            [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_float, c_void_p, c_float,
             c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p])
    _check(f(qkv.data_ptr(), dtype_code(qkv.dtype), qkv.shape[0], nh, nkv, hd, rot, _ptr(q_weight), _ptr(k_weight),
             eps, _ptr(inv_freq), q_scale, tok_pos.data_ptr(), tok_seq.data_ptr(), seq_slot.data_ptr(),
             _ptr(page_table), page_table.shape[1] if page_table is not None else 1, page_size, _ptr(kcache),
             _ptr(vcache), flags, _stream()), "head_norm_rope_cache", "elementwise",
           _nbytes(qkv) * (2 if flags & FLAG_INPLACE else 1)
           + (qkv.shape[0] * 2 * nkv * hd * qkv.element_size() if flags & FLAG_CACHE else 0))
    if (flags & FLAG_CACHE) and not (flags & FLAG_SINGLE) and nkv > 0 and qkv.shape[0] >= 64:
        count_launches(1)   # prompts: the values go through a second, transposing kernel


def silu_mul(gu: torch.Tensor, out: torch.Tensor):
    """out[t, i] = silu(gu[t, i]) * gu[t, I + i]."""
    _cuda(gu, out)
    inter = out.shape[-1]
    assert gu.shape[-1] == 2 * inter and gu.dtype == out.dtype and gu.is_contiguous() and out.is_contiguous()
    f = _fn("elementwise", "gb_silu_mul", [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(gu.data_ptr(), out.data_ptr(), dtype_code(out.dtype), out.numel() // inter, inter, _stream()), "silu_mul",
           "elementwise", _nbytes(gu, out))


# --------------------------------------------------------------------------- matrix products

def gemm_ref(x, w, out, bias=None, accumulate=False):
    """out = x @ w.T (+ bias), or out += ... (float32 out) with ``accumulate``; CUDA cores, float32
    accumulation in ascending order of the inner index."""
    _cuda(x, w, out, bias)
    assert x.dtype == w.dtype and x.stride(-1) == 1 and out.stride(-1) == 1 and w.is_contiguous()
    m, k = x.shape
    n = w.shape[0]
    assert w.shape[1] == k and out.shape == (m, n)
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.numel() == n
    f = _fn("gemm_ref", "gb_gemm_ref",
            [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_longlong,
             c_longlong, c_void_p])
    _check(f(x.data_ptr(), w.data_ptr(), dtype_code(x.dtype), _ptr(bias), out.data_ptr(), dtype_code(out.dtype),
             OUT_ACCUMULATE if accumulate else OUT_STORE, m, n, k, x.stride(0), out.stride(0), _stream()), "gemm_ref",
           "matmul", _nbytes(x, w, bias, out) * 1 + (_nbytes(out) if accumulate else 0))


_sm_counts = {}


def sm_count(device=None) -> int:
    """Streaming multiprocessors of ``device`` (the current CUDA device when None), read once per
    device: tile splits, persistent grids and the decode attention's share of the cache are sized
    by it, so a part with fewer SMs (or a slice of one) is neither oversubscribed nor left idle."""
    index = torch.cuda.current_device() if device is None else torch.device(device).index
    if index is None:
        index = torch.cuda.current_device()
    n = _sm_counts.get(index)
    if n is None:
        n = _sm_counts[index] = int(torch.cuda.get_device_properties(index).multi_processor_count)
    return n


_TC_MODES = {(torch.bfloat16, False): 0, (torch.float32, False): 1, (torch.float32, True): 2}


def gemm_tc_usable(x, w) -> bool:
    """Whether the tensor-core kernel takes these operands (TMA wants 16-byte aligned rows)."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[1] % 8 == 0
            and x.stride(0) % 8 == 0 and x.stride(1) == 1 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_tc_tiling(m: int, n: int, k: int, gated: bool = False, sms: Optional[int] = None):
    """(tokens per tile, K splits) for an [m, k] x [n, k]^T product (``gated``: n features from
    2n rows, two accumulators per tile) on a device of ``sms`` multiprocessors (None: the current
    device's)."""
    sms = sms or sm_count()
    tiles_n = -(-n // 128)
    if m <= 64:
        bn = 16 if m <= 16 else (32 if m <= 32 else 64)
        tiles, kb = tiles_n, -(-k // 64)
        splits = 1
        # too few tiles to keep every SM streaming: split the inner dimension over a cluster, whose
        # ranks each add a share of the tile's tokens.  The CTAs wanted in all: two per SM for tiles of
        # 16 tokens, one per SM for wider tiles (every split sends all the tile's tokens' partial sums
        # once more through the cluster, which costs more the more tokens there are), about one per
        # SM for the gated product with 16 tokens and no split above that.  Measured with cold
        # weights at the layer sizes of 4B / 8B / 32B models (us, 1/2/4/8 splits):
        #  8 tokens: 6144x4096 22.6/15.4/13.6/12.8, 4096x12288 59/33/23/21, 10240x5120 28/23/21/24,
        #            gated 12288x4096 40/36/40/40, gated 25600x5120 82/86/86/95;
        # 32 tokens: 6144x2560 16/14/12/16, 6144x4096 23/17/16/18, 10240x5120 29/25/30/32,
        #            5120x8192 42/30/21/25, 5120x25600 121/72/51/58, 2560x4096 23/18/12/11;
        # 64 tokens: 6144x4096 23/20/18/23, 4096x4096 23/23/16/15, 10240x5120 30/29/34/39,
        #            5120x25600 122/83/58/63, gated 12288x4096 42/60/61/88.
        if gated:
            enough = sms + 2 if bn == 16 else 0
        else:
            enough = 2 * sms if bn == 16 else sms
        while splits < 8 and tiles * splits < enough and kb // (splits * 2) >= 4:
            splits *= 2
        return bn, splits
    best, best_score = 128, -1.0
    # a tile of 256 tokens runs the tensor pipe best; measured at 2,048 x 12,288 x 4,096 gated:
    # 384 us with 256-token tiles, 450 us with 128-token tiles
    for bn, tile_eff in ((256, 1.0), (128, 0.85 if gated else 0.92)):
        tiles = tiles_n * -(-m // bn)
        waves = -(-tiles // sms)
        fill = m / (-(-m // bn) * bn)
        score = tile_eff * fill * tiles / (waves * sms)
        if score > best_score:
            best, best_score = bn, score
    return best, 1


class UnscaledRows:
    """The input of an RMSNorm that is taken into the products around it (decode steps): ``rows``
    [tokens, width] = bfloat16(residual * the norm's weight), and ``partial`` [tiles, 64], the
    sums of squares of the residual's rows in tiles of 128 features, both left by the product
    that added into the residual.  The norm's output is rows * rstd, rstd[t] = (sum of
    partial[:, t] / width + eps) ** -0.5; the product that takes these rows applies rstd to its
    results instead (float32), so the norm needs no kernel of its own."""

    def __init__(self, rows, partial, eps: float, width: int):
        self.rows, self.partial, self.eps, self.width = rows, partial, float(eps), int(width)

    @property
    def shape(self):
        return self.rows.shape

    def materialize(self) -> torch.Tensor:
        """The norm's output as a plain tensor, for a consumer that cannot take unscaled rows."""
        m = self.rows.shape[0]
        rstd = (self.partial[:, :m].sum(0) / self.width + self.eps).rsqrt()
        return (self.rows.float() * rstd[:, None]).to(self.rows.dtype)


LINK_MAX_TOKENS = 64


def norm_link_usable(x, w, m: int, accumulate_splits: Optional[int] = None) -> bool:
    """Whether gemm_tc can take an RMSNorm into itself for these operands: at most 64 tokens on
    the tensor-core path; the product that leaves the rows must have its inner dimension split."""
    ok = m <= LINK_MAX_TOKENS and gemm_tc_usable(x, w)
    return ok and (accumulate_splits is None or accumulate_splits >= 2)


def gemm_tc(x, w, out, bias=None, accumulate=False, bn=None, splits=None, stages=4, swiglu=False, link_in=None,
            link_out=None):
    """out = x @ w.T (+ bias) (bfloat16 or float32 out) or out += ... (float32 out), bfloat16
    operands, on the tcgen05 tensor cores.  With ``swiglu``, w stacks a gate matrix over an up
    matrix ([2N, K]) and out[M, N] = silu(x @ gate.T) * (x @ up.T) in bfloat16.
    ``link_in``: an UnscaledRows whose ``rows`` are x: every token's results are scaled by its
    rstd.  ``link_out`` = (norm weight float32 [N], eps): with ``accumulate``, also leaves
    bfloat16(out * weight) and the sums of squares of out's rows, returned as UnscaledRows."""
    if link_in is not None:
        assert x is link_in.rows
    _cuda(x, w, out, bias)
    m, k = x.shape
    n = w.shape[0] // 2 if swiglu else w.shape[0]
    assert w.shape[1] == k and w.is_contiguous() and out.shape == (m, n) and out.stride(1) == 1
    if not gemm_tc_usable(x, w):
        raise KernelError("gemm_tc: operands must be bfloat16 with 16-byte aligned rows (K and the row stride "
                          "multiples of 8)")
    if swiglu:
        if out.dtype != torch.bfloat16 or accumulate or bias is not None or w.shape[0] % 2:
            raise KernelError("gemm_tc: the gated product writes bfloat16, without bias, from an even number of rows")
        mode = 3
    else:
        mode = _TC_MODES.get((out.dtype, bool(accumulate)))
    if mode is None:
        raise KernelError(f"gemm_tc: cannot {'add into' if accumulate else 'store'} {out.dtype}")
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.numel() == n
    auto_bn, auto_splits = gemm_tc_tiling(m, n, k, gated=swiglu)
    if link_in is None and link_out is None:
        f = _fn("gemm_tc", "gb_gemm_tc",
                [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_longlong, c_longlong, c_int,
                 c_int, c_int, c_void_p])
        _check(f(x.data_ptr(), w.data_ptr(), _ptr(bias), out.data_ptr(), mode, m, n, k, x.stride(0), out.stride(0),
                 bn or auto_bn, splits or auto_splits, stages, _stream()), "gemm_tc", "matmul",
               _nbytes(x, w, bias, out) + (_nbytes(out) if accumulate else 0))
        return None
    if m > LINK_MAX_TOKENS:
        raise KernelError(f"gemm_tc: a norm can be taken into the product for at most {LINK_MAX_TOKENS} tokens")
    left = None
    if link_out is not None:
        weight, eps = link_out
        if not accumulate or (splits or auto_splits) < 2:
            raise KernelError("gemm_tc: rows for a norm are left by a product that adds into the residual with its "
                              "inner dimension split")
        assert weight.dtype == torch.float32 and weight.numel() == n
        left = UnscaledRows(torch.empty((m, n), dtype=torch.bfloat16, device=x.device),
                            torch.empty((-(-n // 128), 64), dtype=torch.float32, device=x.device), eps, n)
    f = _fn("gemm_tc", "gb_gemm_tc_linked",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_longlong, c_longlong, c_int,
             c_int, c_int, c_void_p, c_int, c_float, c_int, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p])
    _check(f(x.data_ptr(), w.data_ptr(), _ptr(bias), out.data_ptr(), mode, m, n, k, x.stride(0), out.stride(0),
             bn or auto_bn, splits or auto_splits, stages,
             link_in.partial.data_ptr() if link_in is not None else None,
             link_in.partial.shape[0] if link_in is not None else 0, link_in.eps if link_in is not None else 0.0,
             link_in.width if link_in is not None else 0,
             link_out[0].data_ptr() if left is not None else None, left.rows.data_ptr() if left is not None else None,
             left.rows.stride(0) if left is not None else 0, left.partial.data_ptr() if left is not None else None,
             _stream()), "gemm_tc", "matmul",
           _nbytes(x, w, bias, out) + (_nbytes(out) if accumulate else 0) + (_nbytes(left.rows) if left is not None else 0))
    return left


_part_flags = {}
PERSISTENT_SPLIT_LAST_ROUND = True


def gemm_tc_persistent(x, w, out, bias=None, accumulate=False, swiglu=False, bn=None, ctas=None, split_last=None):
    """The tensor-core product for prompts (more than 64 rows of x): one CTA per SM walks the output
    tiles, and the epilogue of a tile runs while the next tile's MMAs fill the other accumulator
    buffer.  Operands and modes as gemm_tc.  Where the last round of tiles would leave SMs idle, a
    product that adds into ``out`` cuts that round's tiles into parts along the inner dimension,
    which are added in a fixed order (``split_last=False``: never)."""
    if split_last is None:
        split_last = PERSISTENT_SPLIT_LAST_ROUND
    _cuda(x, w, out, bias)
    m, k = x.shape
    n = w.shape[0] // 2 if swiglu else w.shape[0]
    assert w.shape[1] == k and w.is_contiguous() and out.shape == (m, n) and out.stride(1) == 1
    if not gemm_tc_usable(x, w):
        raise KernelError("gemm_tc_persistent: operands must be bfloat16 with 16-byte aligned rows")
    if swiglu:
        if out.dtype != torch.bfloat16 or accumulate or bias is not None or w.shape[0] % 2:
            raise KernelError("gemm_tc_persistent: the gated product writes bfloat16, without bias")
        mode = 3
    else:
        mode = _TC_MODES.get((out.dtype, bool(accumulate)))
    if mode is None:
        raise KernelError(f"gemm_tc_persistent: cannot {'add into' if accumulate else 'store'} {out.dtype}")
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.numel() == n
    if bn is None:
        # 256 tokens a tile.  Narrower tiles that fill the last round of tiles better were measured and
        # are slower: 240 tokens for 2,048 x 4,096 (1.5 % faster alone, 4 % slower inside a prompt step),
        # and 128 tokens where 256 leave the last round nearly empty (2,048 x 2,560 is 160 tiles on 148
        # SMs; a 2,048-token prompt of a 4B-shaped model took 20.5 ms against 18.4, of a 32B-shaped one
        # 35.3 ms against 30.9 over 16 layers)
        bn = 128 if m <= 128 else 256
    ctas = ctas or sm_count(x.device)
    flags = None
    if accumulate and split_last:
        # a word per tile of the last round and epilogue warp; zero between launches
        flags = _part_flags.get(x.device.index)
        if flags is None or flags.numel() < 4 * ctas:
            if flags is not None:
                _outgrown.append(flags)       # a captured step may still point at it: never freed
            flags = _part_flags[x.device.index] = torch.zeros(max(4 * ctas, 1024), dtype=torch.int32, device=x.device)
    f = _fn("gemm_tc", "gb_gemm_tc_persistent",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_longlong, c_longlong, c_int,
             c_int, c_void_p, c_void_p])
    _check(f(x.data_ptr(), w.data_ptr(), _ptr(bias), out.data_ptr(), mode, m, n, k, x.stride(0), out.stride(0), bn,
             ctas, _ptr(flags), _stream()), "gemm_tc_persistent", "matmul",
           _nbytes(x, w, bias, out) + (_nbytes(out) if accumulate else 0))


# measured inside replayed steps: +1.5 % tokens/s at batch 1 and 8 (8B layer sizes), even at batch 16
# (4B), -1.5 % at batch 24 (8B), -2.5 % at batch 32 (32B), -1 % at batch 64 (8B): a rank finishes
# its share of the tokens one after the other, three barriers each
QKV_FUSED_MAX_TOKENS = 16


QKV_KERNEL_MAX_TOKENS = 64     # what the kernel takes; the dispatch stops earlier, where it stops paying


def gemm_qkv_usable(x, w, nh: int, nkv: int, hd: int, rot: int, limit: Optional[int] = None) -> bool:
    """Whether the q/k/v product of a step can do the per-head work in its epilogue: a decode step
    in bfloat16 of at most ``limit`` tokens (None: as many as it pays for) with heads of 128 (a
    head is a tile of the product), rotated over all dims or not at all."""
    limit = QKV_FUSED_MAX_TOKENS if limit is None else limit
    return (x.dtype == torch.bfloat16 and x.shape[0] <= limit and hd == 128 and rot in (0, hd)
            and w.shape[0] == (nh + 2 * nkv) * hd and gemm_tc_usable(x, w))


def gemm_qkv(x, w, bias, qkv, nh, nkv, hd, q_weight, k_weight, eps, inv_freq, q_scale, tok_pos, tok_seq, seq_slot,
             page_table, page_size, kcache, vcache, bn=None, splits=None, link_in=None):
    """qkv[:, :nh*hd] = the step's queries, normed per head, rotated and scaled; the keys (normed,
    rotated) and the values go into the paged cache (``page_table`` None: into qkv as well): the
    q/k/v product and head_norm_rope_cache in one kernel.  See gemm_qkv_usable."""
    _cuda(x, w, bias, qkv, q_weight, k_weight, inv_freq, tok_pos, tok_seq, seq_slot, page_table, kcache, vcache)
    m, k = x.shape
    n = w.shape[0]
    assert qkv.dtype == torch.bfloat16 and qkv.shape == (m, n) and qkv.stride(1) == 1 and w.is_contiguous()
    if not gemm_qkv_usable(x, w, nh, nkv, hd, hd if inv_freq is not None else 0, limit=QKV_KERNEL_MAX_TOKENS):
        raise KernelError(f"gemm_qkv: needs bfloat16, at most {QKV_KERNEL_MAX_TOKENS} tokens and heads of 128")
    if page_table is not None:
        assert kcache.dtype == torch.bfloat16 and kcache.is_contiguous() and kcache.shape[1:] == (nkv, page_size, hd)
        assert vcache.is_contiguous() and vcache.shape[1:] == (nkv, hd, page_size)
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.numel() == n
    auto_bn, auto_splits = gemm_tc_tiling(m, n, k)
    f = _fn("gemm_tc", "gb_gemm_tc_qkv",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_int, c_int,
             c_void_p, c_void_p, c_void_p, c_float, c_float, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
             c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_float, c_int, c_void_p])
    if link_in is not None:
        assert x is link_in.rows
    _check(f(x.data_ptr(), w.data_ptr(), _ptr(bias), qkv.data_ptr(), m, n, k, x.stride(0), qkv.stride(0),
             bn or auto_bn, splits or auto_splits, _ptr(q_weight), _ptr(k_weight), _ptr(inv_freq), eps, q_scale, nh, nkv,
             tok_pos.data_ptr(), _ptr(tok_seq), _ptr(seq_slot), _ptr(page_table),
             page_table.shape[1] if page_table is not None else 1, page_size, _ptr(kcache), _ptr(vcache),
             link_in.partial.data_ptr() if link_in is not None else None,
             link_in.partial.shape[0] if link_in is not None else 0, link_in.eps if link_in is not None else 0.0,
             link_in.width if link_in is not None else 0, _stream()),
           "gemm_qkv", "matmul", _nbytes(x, w, bias, qkv))


def rope_table(tok_pos, inv_freq):
    """[tokens, half] pairs (cos, sin) of float32(position) * inv_freq, float32 [tokens, half, 2]:
    the angles of a step's packed tokens, computed once for all layers."""
    _cuda(tok_pos, inv_freq)
    assert tok_pos.dtype == torch.int32 and inv_freq.dtype == torch.float32
    ntok, half = tok_pos.numel(), inv_freq.numel()
    table = torch.empty((ntok, half, 2), dtype=torch.float32, device=tok_pos.device)
    f = _fn("gemm_tc", "gb_rope_table", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p])
    _check(f(tok_pos.data_ptr(), inv_freq.data_ptr(), table.data_ptr(), ntok, half, _stream()), "rope_table",
           "elementwise", _nbytes(table))
    return table


def token_place(tok_pos, tok_seq, seq_slot, page_table, page_size):
    """int32 [tokens, 2]: (page, position in the page) of every packed token of a step in the cache
    that ``page_table`` describes; made once a step for all the layers that share the table."""
    _cuda(tok_pos, tok_seq, seq_slot, page_table)
    ntok = tok_pos.numel()
    place = torch.empty((ntok, 2), dtype=torch.int32, device=tok_pos.device)
    f = _fn("gemm_tc", "gb_token_place", [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p])
    _check(f(tok_pos.data_ptr(), tok_seq.data_ptr(), seq_slot.data_ptr(), page_table.data_ptr(), page_table.shape[1],
             page_size, place.data_ptr(), ntok, _stream()), "token_place", "elementwise", _nbytes(place))
    return place


def gemm_qkv_prompt_usable(x, w, nh: int, nkv: int, hd: int, rot: int, page_size: int) -> bool:
    """Whether the q/k/v product of a prompt step can do the per-head work in its epilogue:
    bfloat16, more than 64 tokens, heads of 128 rotated over all dims or not at all."""
    return (x.dtype == torch.bfloat16 and x.shape[0] > 64 and hd == 128 and rot in (0, hd) and page_size % 8 == 0
            and w.shape[0] == (nh + 2 * nkv) * hd and gemm_tc_usable(x, w))


def gemm_qkv_prompt(x, w, bias, q_out, nh, nkv, hd, q_weight, k_weight, eps, table, q_scale, place, page_size, kcache,
                    vcache, ctas=None):
    """q_out[:, :nh*hd] = a prompt step's queries, normed per head, rotated and scaled; the keys
    (normed, rotated) and the values go into the paged cache: the q/k/v product of more than 64
    tokens and head_norm_rope_cache in one kernel.  ``table``: rope_table of the step's tokens
    (None: no rotation); ``place``: token_place of the step's tokens in this cache (None with no
    kv heads).  See gemm_qkv_prompt_usable."""
    _cuda(x, w, bias, q_out, q_weight, k_weight, table, place, kcache, vcache)
    m, k = x.shape
    n = w.shape[0]
    assert q_out.dtype == torch.bfloat16 and q_out.shape == (m, nh * hd) and q_out.stride(1) == 1 and w.is_contiguous()
    if not gemm_qkv_prompt_usable(x, w, nh, nkv, hd, hd if table is not None else 0, page_size):
        raise KernelError("gemm_qkv_prompt: needs bfloat16, more than 64 tokens and heads of 128")
    if nkv:
        assert kcache.dtype == torch.bfloat16 and kcache.is_contiguous() and kcache.shape[1:] == (nkv, page_size, hd)
        assert vcache.is_contiguous() and vcache.shape[1:] == (nkv, hd, page_size)
        assert place.dtype == torch.int32 and place.shape == (m, 2) and place.is_contiguous()
    if table is not None:
        assert table.dtype == torch.float32 and table.shape == (m, hd // 2, 2) and table.is_contiguous()
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.numel() == n
    f = _fn("gemm_tc", "gb_gemm_tc_qkv_prompt",
            [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_int, c_void_p, c_void_p,
             c_void_p, c_float, c_float, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p])
    _check(f(x.data_ptr(), w.data_ptr(), _ptr(bias), q_out.data_ptr(), m, n, k, x.stride(0), q_out.stride(0),
             ctas or sm_count(x.device), _ptr(q_weight), _ptr(k_weight), _ptr(table), eps, q_scale, nh, nkv,
             _ptr(place) if nkv else None, page_size, _ptr(kcache), _ptr(vcache), _stream()),
           "gemm_qkv_prompt", "matmul", _nbytes(x, w, bias, q_out) + m * 2 * nkv * hd * 2)


# 65 to 128 tokens (decoding above batch 64): a CTA per tile of 128 features x 128 tokens with both
# accumulators, 96 CTAs at 8B layer sizes, takes 42 us with cold weights where the prompt kernel's
# 192 tiles of 64 features take 54 (30.8 us of bytes); above 128 tokens the prompt kernel is ahead.
GATED_TILE_128_MAX_TOKENS = 128


def gemm_swiglu(x, w_gate_up, out):
    """out[M, N] = silu(x @ gate.T) * (x @ up.T) for w_gate_up = [gate; up] of 2N rows: one
    tensor-core kernel in bfloat16; two kernels (product, then activation) otherwise.  ``x`` may
    be UnscaledRows (a norm taken into this product)."""
    link = x if isinstance(x, UnscaledRows) else None
    if link is not None:
        if norm_link_usable(link.rows, w_gate_up, link.rows.shape[0]):
            gemm_tc(link.rows, w_gate_up, out, swiglu=True, link_in=link)
            return
        x = link.materialize()
    if x.dtype == torch.bfloat16 and gemm_tc_usable(x, w_gate_up):
        if x.shape[0] > GATED_TILE_128_MAX_TOKENS:
            gemm_tc_persistent(x, w_gate_up, out, swiglu=True)
        elif x.shape[0] > 64:
            gemm_tc(x, w_gate_up, out, swiglu=True, bn=128, splits=1)
        else:
            gemm_tc(x, w_gate_up, out, swiglu=True)
        return
    gu = torch.empty((x.shape[0], w_gate_up.shape[0]), dtype=x.dtype, device=x.device)
    gemm(x, w_gate_up, gu)
    silu_mul(gu, out)


_STATUS_ENTRIES = ("gb_gemm_tc_status", "gb_attention_prefill_tc_status", "gb_attention_decode_stream_status")


def _status(entry: str, reset: bool) -> int:
    """First non-zero status word among the loaded libraries that export ``entry`` (every build of
    a unit keeps a word of its own)."""
    first = 0
    for lib in build.loaded().values():
        try:
            f = getattr(lib, entry)
        except AttributeError:
            continue
        f.argtypes, f.restype = [c_int], c_int
        v = f(1 if reset else 0)
        first = first or v
    return first


def gemm_tc_status(reset: bool = True) -> int:
    """0, or the code of the first bounded wait that ran out in a gemm_tc launch (synchronizes)."""
    return _status("gb_gemm_tc_status", reset)


def check_status() -> None:
    """Raises if a bounded wait ran out in any tensor-core kernel since the last check: such a
    kernel gives up and leaves its output unfinished, so what was computed since must not be used.
    Synchronizes; the engine calls it before results leave it."""
    for entry in _STATUS_ENTRIES:
        v = _status(entry, True)
        if v:
            for flags in _part_flags.values():   # a kernel that gave up may have left a part's word set
                flags.zero_()
            raise KernelError(f"{entry[3:-7]}: a bounded wait ran out on the device (code {v}); "
                              "the results computed since the last check are not valid")


# --------------------------------------------------------------------------- attention

def attention_ref(q, out, nh, kcache, vcache, page_table, page_size, tok_pos, tok_seq, seq_slot, window=None, cache_bytes: int = 0):
    """Causal grouped-query attention of q [T, nh*hd] (row stride free) over the paged cache."""
    _cuda(q, out, kcache, vcache, page_table, tok_pos, tok_seq, seq_slot)
    nkv, hd = kcache.shape[1], kcache.shape[3]
    assert q.stride(-1) == 1 and out.stride(-1) == 1 and q.dtype == out.dtype == kcache.dtype
    f = _fn("attention_ref", "gb_attention_ref",
            [c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
             c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(f(q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0), dtype_code(q.dtype), kcache.data_ptr(),
             vcache.data_ptr(), page_table.data_ptr(), page_table.shape[1], page_size, nkv, hd, tok_pos.data_ptr(),
             tok_seq.data_ptr(), seq_slot.data_ptr(), q.shape[0], nh, window or 0, _stream()), "attention_ref",
           "attention", _nbytes(q, out) + cache_bytes)


def decode_shares(ntok: int, nh: int, nkv: int, longest: int) -> int:
    """CTAs along the keys per (token, kv head) for the decode attention kernel: about one CTA per
    SM in all (a CTA's fixed work, loading q and merging its warps, is paid once per share; measured
    at 8,192 keys: 16 shares are best for one sequence, 2 for eight, 1 for sixty-four), and never
    so many that a warp is left without a 32-key block."""
    rep = nh // nkv
    chunks = -(-rep // 16)
    base = max(1, ntok * nkv * chunks)
    blocks = -(-max(longest, 1) // 32)
    want = (sm_count() + base // 2) // base
    return max(1, min(want, blocks // 8, 64))


def attention_decode(q, out, nh, kcache, vcache, page_table, page_size, tok_pos, tok_seq, seq_slot, window=None,
                     shares=1, scratch=None, cache_bytes: int = 0):
    """bfloat16 attention of single positions (one CTA per token, kv head and share of the keys)
    over the paged cache; the unit is compiled for the cache's head size."""
    _cuda(q, out, kcache, vcache, page_table, tok_pos, tok_seq, seq_slot, scratch)
    nkv, hd = kcache.shape[1], kcache.shape[3]
    ntok = q.shape[0]
    assert q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and kcache.dtype == torch.bfloat16
    assert q.stride(-1) == 1 and out.stride(-1) == 1 and vcache.shape[2:] == (hd, page_size)
    if shares > 1:
        need = ntok * nh * shares * (hd + 2)
        if scratch is None:
            scratch = torch.empty(need, dtype=torch.float32, device=q.device)
        assert scratch.dtype == torch.float32 and scratch.numel() >= need
    f = _fn("attention_decode", "gb_attention_decode",
            [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
             c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
            defines=(("GB_HEAD_DIM", hd),))
    _check(f(q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0), kcache.data_ptr(), vcache.data_ptr(),
             page_table.data_ptr(), page_table.shape[1], page_size, nkv, hd, tok_pos.data_ptr(), tok_seq.data_ptr(),
             seq_slot.data_ptr(), ntok, nh, window or 0, shares, _ptr(scratch), _stream()), "attention_decode",
           "attention", _nbytes(q, out) + cache_bytes)
    if shares > 1:
        count_launches(1)   # the merge kernel


STREAM_DECODE_HEAD_DIMS = (64, 128)
STREAM_DECODE_MAX_TOKENS = 4096
_decode_stream_scratch = {}
_outgrown = []


def attention_decode_stream_usable(ntok: int, nh: int, nkv: int, hd: int, page_size: int) -> bool:
    return (hd in STREAM_DECODE_HEAD_DIMS and page_size == 64 and nh % nkv == 0 and nh // nkv <= 16
            and ntok <= STREAM_DECODE_MAX_TOKENS)


def attention_decode_stream(q, out, nh, kcache, vcache, page_table, page_size, tok_pos, tok_seq, seq_slot,
                            window=None, ctas=None, skip_slot=None, cache_bytes: int = 0):
    """bfloat16 attention of single positions with the cache streamed through shared memory by
    TMA: the pages that the step reads are dealt evenly to the CTAs as one flat list, whatever the
    lengths of the sequences; parts of a (token, kv head) that fall to different CTAs are added
    in key order by a second kernel.  Tokens of ``skip_slot`` (rows that pad a captured step) read
    nothing and get zeros."""
    _cuda(q, out, kcache, vcache, page_table, tok_pos, tok_seq, seq_slot)
    nkv, hd = kcache.shape[1], kcache.shape[3]
    ntok = q.shape[0]
    assert q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and kcache.dtype == torch.bfloat16
    assert q.stride(-1) == 1 and out.stride(-1) == 1 and vcache.shape[2:] == (hd, page_size)
    assert kcache.is_contiguous() and vcache.is_contiguous()
    if not attention_decode_stream_usable(ntok, nh, nkv, hd, page_size):
        raise KernelError(f"attention_decode_stream: head size {hd} (64 or 128), page size {page_size} (64), "
                          f"{nh // max(nkv, 1)} query heads per kv head (at most 16) or {ntok} tokens "
                          f"(at most {STREAM_DECODE_MAX_TOKENS}) not supported")
    defines = (("GB_HEAD_DIM", hd),)
    sig = [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_int, c_int,
           c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p]
    f = _fn("attention_decode_stream", "gb_attention_decode_stream", sig, defines=defines)
    if ctas is None:
        ctas = sm_count(q.device)   # one per SM; measured at 8,192 keys, batch 1 / 8 / 64: 17 / 54 / 323 us; two per SM: 24 / 58 / 329
    need = ctas * 2 * (nh // nkv) * (hd + 2) + ntok + 1
    scratch = _decode_stream_scratch.get(q.device.index)
    if scratch is None or scratch.numel() < need:
        if scratch is not None:
            _outgrown.append(scratch)     # a captured step may still point at it: never freed
        scratch = _decode_stream_scratch[q.device.index] = torch.empty(max(need, 1 << 20), dtype=torch.float32,
                                                                       device=q.device)
    _check(f(q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0), kcache.data_ptr(), vcache.data_ptr(),
             kcache.shape[0], page_table.data_ptr(), page_table.shape[1], page_size, nkv, hd, tok_pos.data_ptr(),
             tok_seq.data_ptr(), seq_slot.data_ptr(), ntok, nh, window or 0, -1 if skip_slot is None else skip_slot,
             ctas, scratch.data_ptr(), _stream()),
           "attention_decode_stream", "attention", _nbytes(q, out) + cache_bytes)
    count_launches(1)   # the merge kernel


def attention_decode_stream_status(reset: bool = True) -> int:
    return _status("gb_attention_decode_stream_status", reset)


def attention_prefill(q, out, nh, kcache, vcache, page_table, page_size, cu_seqlens, seq_start, seq_slot, window=None, cache_bytes: int = 0):
    """bfloat16 causal attention of packed prompt tokens (sequence b owns tokens cu_seqlens[b] to
    cu_seqlens[b + 1], at positions from seq_start[b]) over the paged cache, which already holds
    the step's own keys and values."""
    _cuda(q, out, kcache, vcache, page_table, cu_seqlens, seq_start, seq_slot)
    nkv, hd = kcache.shape[1], kcache.shape[3]
    assert q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and kcache.dtype == torch.bfloat16
    assert q.stride(-1) == 1 and out.stride(-1) == 1 and vcache.shape[2:] == (hd, page_size)
    f = _fn("attention_prefill", "gb_attention_prefill",
            [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
             c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
            defines=(("GB_HEAD_DIM", hd),))
    _check(f(q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0), kcache.data_ptr(), vcache.data_ptr(),
             page_table.data_ptr(), page_table.shape[1], page_size, nkv, hd, cu_seqlens.data_ptr(),
             seq_start.data_ptr(), seq_slot.data_ptr(), seq_slot.numel(), q.shape[0], nh, window or 0, _stream()),
           "attention_prefill", "attention", _nbytes(q, out) + cache_bytes)


TC_PREFILL_HEAD_DIMS = (64, 128)


def attention_prefill_tc(q, out, nh, kcache, vcache, page_table, page_size, cu_seqlens, seq_start, seq_slot,
                         window=None, cache_bytes: int = 0):
    """As attention_prefill, on the tcgen05 tensor cores (TMA-fed, S and O in tensor memory); head
    sizes 64 and 128."""
    _cuda(q, out, kcache, vcache, page_table, cu_seqlens, seq_start, seq_slot)
    nkv, hd = kcache.shape[1], kcache.shape[3]
    if hd not in TC_PREFILL_HEAD_DIMS:
        raise KernelError(f"attention_prefill_tc: head size {hd} is not supported (64 or 128)")
    assert q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and kcache.dtype == torch.bfloat16
    assert q.stride(-1) == 1 and out.stride(-1) == 1 and vcache.shape[2:] == (hd, page_size)
    assert kcache.is_contiguous() and vcache.is_contiguous() and kcache.shape[0] == vcache.shape[0]
    f = _fn("attention_prefill_tc", "gb_attention_prefill_tc",
            [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_int, c_int,
             c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
            defines=(("GB_HEAD_DIM", hd),))
    _check(f(q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0), kcache.data_ptr(), vcache.data_ptr(),
             kcache.shape[0], page_table.data_ptr(), page_table.shape[1], page_size, nkv, hd, cu_seqlens.data_ptr(),
             seq_start.data_ptr(), seq_slot.data_ptr(), seq_slot.numel(), q.shape[0], nh, window or 0, _stream()),
           "attention_prefill_tc", "attention", _nbytes(q, out) + cache_bytes)


def attention_prefill_tc_status(head_dim: int = 0, reset: bool = True) -> int:
    """0, or the code of the first bounded wait that ran out in attention_prefill_tc (synchronizes)."""
    return _status("gb_attention_prefill_tc_status", reset)


# --------------------------------------------------------------------------- sampling

_sample_scratch = {}
_sample_cut_scratch = {}


def sample(logits, out, temperature=None, top_k=None, top_p=None, uniform=None, wide=False, cap: Optional[int] = None):
    """out[r] = token drawn from logits[r] (float32 [rows, vocab]).  Rows whose temperature is
    <= 0 (or all rows when ``temperature`` is None) take the first maximum.  ``cap``: the largest
    top_k among the rows that have one from 1 to MAX_TOP_K (None: MAX_TOP_K when any row is
    sampled, 1 when all are greedy); a smaller cap is less work.  Rows with top_k = 0 (all tokens)
    or more than MAX_TOP_K candidates need ``wide``: they are sorted in scratch memory of 20 bytes
    per logit."""
    _cuda(logits, out, temperature, top_k, top_p, uniform)
    assert logits.dtype == torch.float32 and logits.stride(-1) == 1 and out.dtype == torch.int32
    rows, vocab = logits.shape
    if cap is None:
        cap = 1 if temperature is None else MAX_TOP_K
    cap = max(1, min(int(cap), MAX_TOP_K))
    sms = sm_count(logits.device)
    size = _fn("sampling", "gb_sample_scratch_bytes", [c_int, c_int, c_int, c_int])
    size.restype = c_longlong
    need = size(rows, vocab, cap, sms)
    if need < 0:
        raise KernelError(f"sample: a vocabulary of {vocab} with up to {cap} candidates a row is not supported "
                          "(at most 64 slices of 16,384 tokens, whose candidates together number at most 16,384)")
    cut = _sample_cut_scratch.get(logits.device.index)
    if cut is None or cut.numel() < need:
        if cut is not None:
            _outgrown.append(cut)         # a captured step may still point at it: never freed
        cut = _sample_cut_scratch[logits.device.index] = torch.empty(max(need, 1 << 20), dtype=torch.uint8,
                                                                     device=logits.device)
    scratch = None
    if wide and temperature is not None:
        need = 5 * rows * vocab
        scratch = _sample_scratch.get(logits.device.index)
        if scratch is None or scratch.numel() < need:
            scratch = _sample_scratch[logits.device.index] = torch.empty(need, dtype=torch.float32, device=logits.device)
    f = _fn("sampling", "gb_sample",
            [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
             c_int, c_int, c_void_p])
    _check(f(logits.data_ptr(), logits.stride(0), rows, vocab, _ptr(temperature), _ptr(top_k),
             _ptr(top_p), _ptr(uniform), out.data_ptr(), _ptr(scratch), cut.data_ptr(), cap, sms, _stream()),
           "sample", "sampling", _nbytes(logits))
    count_launches(1 if scratch is None else 2)


# --------------------------------------------------------------------------- choices by precision and shape

def gemm_units(compute: str):
    """The units ``gemm`` may launch for a model computed in ``compute``."""
    return [("gemm_ref", ())] if compute == "float32" else [("gemm_tc", ()), ("gemm_ref", ())]


# Whether the blocks take the RMSNorms of a decode step into the products around them (see
# UnscaledRows).  Measured as an upper bound, by skipping the norm kernels: 2 % of a step at 8B layer
# sizes, 5.6 % at 4B sizes.
NORM_LINKS = True


def gemm(x, w, out, bias=None, accumulate=False, then_norm=None):
    """out = x @ w.T (+ bias) or, with ``accumulate``, out += ...; picks the kernel for the
    precision and the shape: float32 runs on the CUDA cores in a fixed order; bfloat16 runs on the
    tensor cores, except for operands whose rows TMA cannot address (an inner size that is not
    a multiple of 8), which the plain kernel takes.  ``x`` may be UnscaledRows (a norm taken into
    this product).  ``then_norm`` = (weight, eps) of an RMSNorm that follows an accumulating
    product: where the kernel can, it leaves that norm's input as UnscaledRows, which is returned
    (None: the norm has to run by itself)."""
    link = x if isinstance(x, UnscaledRows) else None
    if link is not None:
        if norm_link_usable(link.rows, w, link.rows.shape[0]):
            x = link.rows
        else:
            x, link = link.materialize(), None
    if x.dtype == torch.bfloat16 and gemm_tc_usable(x, w):
        m, n, k = x.shape[0], w.shape[0], x.shape[1]
        if m > 64:
            gemm_tc_persistent(x, w, out, bias, accumulate)
            return None
        if then_norm is not None and not (accumulate and gemm_tc_tiling(m, n, k)[1] >= 2):
            then_norm = None
        return gemm_tc(x, w, out, bias, accumulate, link_in=link, link_out=then_norm)
    gemm_ref(x, w, out, bias, accumulate)
    return None


def attention_units(compute: str, head_dim: int):
    if compute == "float32":
        return [("attention_ref", ())]
    hd = (("GB_HEAD_DIM", head_dim),)
    prefill = "attention_prefill_tc" if head_dim in (64, 128) else "attention_prefill"
    units = [("attention_ref", ()), ("attention_decode", hd), (prefill, hd)]
    if head_dim in STREAM_DECODE_HEAD_DIMS:
        units.append(("attention_decode_stream", hd))
    return units


def attention(ctx, q, out, nh, kcache, vcache, page_table, page_size, window=None):
    """Attention of the step's queries over the cache; picks the kernel for the precision and
    for prompts or single tokens.  float32 always takes the plain kernel, whose arithmetic for a
    position does not depend on the batch."""
    cached = 0
    if _profile["on"] and ctx.host is not None:
        # keys and values the step has to read: each sequence's positions (its window's worth) once
        per_pos = 2 * kcache.shape[1] * kcache.shape[3] * kcache.element_size()
        for start, n in zip(ctx.host["seq_start"], ctx.host["seq_len"]):
            cached += per_pos * (min(start + n, window + n - 1) if window else start + n)
    if q.dtype == torch.bfloat16 and ctx.max_new <= DECODE_KERNEL_MAX_NEW:
        nkv = kcache.shape[1]
        if attention_decode_stream_usable(ctx.n_tokens, nh, nkv, kcache.shape[3], page_size):
            attention_decode_stream(q, out, nh, kcache, vcache, page_table, page_size, ctx.tok_pos, ctx.tok_seq,
                                    ctx.seq_slot, window, skip_slot=ctx.pad_slot, cache_bytes=cached)
            return
        shares = decode_shares(ctx.n_tokens, nh, nkv, ctx.max_total if window is None else min(ctx.max_total, window))
        attention_decode(q, out, nh, kcache, vcache, page_table, page_size, ctx.tok_pos, ctx.tok_seq, ctx.seq_slot,
                         window, shares, cache_bytes=cached)
        return
    if q.dtype == torch.bfloat16:
        prefill = attention_prefill_tc if kcache.shape[3] in TC_PREFILL_HEAD_DIMS else attention_prefill
        prefill(q, out, nh, kcache, vcache, page_table, page_size, ctx.cu_seqlens, ctx.seq_start, ctx.seq_slot, window,
                cache_bytes=cached)
        return
    attention_ref(q, out, nh, kcache, vcache, page_table, page_size, ctx.tok_pos, ctx.tok_seq, ctx.seq_slot, window,
                  cache_bytes=cached)


# a step whose sequences bring at most this many tokens each runs the per-position decode kernel
DECODE_KERNEL_MAX_NEW = 1
