"""Trace replay on the GPU against the plain implementation: each request alone and whole, with
its last 32 tokens one by one, and in batches of unequal lengths that follow one another so
that slots and pages are used again; in float32 and in bfloat16."""
import numpy as np
import pytest

import plain_qwen3 as plain
from replay_util import Trace, run_trace
from tiny_configs import TINY_A, TINY_B, TOL_BF16

pytestmark = pytest.mark.gpu

# lengths straddle the page size (64), the reference kernel's chunk (128) and TINY_B's window (40)
REQUESTS = {
    "A": (TINY_A, [15, 21, 9, 70, 40, 129]),
    "B": (TINY_B, [17, 33, 47, 80, 150, 41]),
}
GROUPS = [[0, 1, 2], [3, 4, 5]]
# float32: rounding of a float32 engine against a float64 oracle, logits of size ~1
TOL_F32 = 2e-5


def _requests(cfg, lengths, seed):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, cfg["vocab_size"], n).tolist() for n in lengths]


@pytest.fixture(scope="module")
def oracle(model_folders):
    out = {}
    for name, (cfg, lengths) in REQUESTS.items():
        folder = model_folders(cfg)
        pcfg, w = plain.load_folder(folder)
        reqs = _requests(cfg, lengths, seed=len(name) + lengths[0])
        out[name] = (folder, reqs, [plain.forward(pcfg, w, r) for r in reqs])
    return out


@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_all_cuttings_match_the_plain_implementation(name, dtype, oracle, tmp_path):
    folder, reqs, ref = oracle[name]
    tr = Trace()
    tr.whole("w", reqs)
    tr.tail("t", reqs)
    prompt_lens = [max(1, len(r) - 8 - 3 * i) for i, r in enumerate(reqs)]
    prompt_lens[2] = len(reqs[2])            # one request of the first batch is all prompt
    prompt_lens[1] = 1                       # and one starts from a single token
    tr.batches("b", reqs, GROUPS, prompt_lens)
    got = run_trace(tr, folder, dtype, str(tmp_path / "out"))
    tol = TOL_F32 if dtype == "float32" else TOL_BF16[name]
    scale = max(float(np.abs(r).max()) for r in ref)
    worst = {}
    for tag in "wtb":
        for i, r in enumerate(ref):
            for p in range(len(r)):
                row = got[(f"{tag}{i}", p)]
                err = float(np.abs(row - r[p]).max())
                if err > worst.get(tag, (0,))[0]:
                    worst[tag] = (err, i, p)
    for tag, (err, i, p) in worst.items():
        assert err <= tol * scale, f"cutting {tag!r}: request {i} position {p} is off by {err:.3e} (scale {scale:.2f})"
    # the cuttings agree with one another: exactly in float32, to rounding in bfloat16
    for i, r in enumerate(ref):
        for p in range(len(r)):
            a, b, c = got[(f"w{i}", p)], got[(f"t{i}", p)], got[(f"b{i}", p)]
            if dtype == "float32":
                assert np.array_equal(a, b) and np.array_equal(a, c), f"request {i} position {p} depends on the cutting"
            else:
                assert max(np.abs(a - b).max(), np.abs(a - c).max()) <= tol * scale


def test_pages_are_reused_within_a_tight_cache(oracle, tmp_path):
    """The cache is sized to the trace's own peak, so later requests must live in pages and slots
    that earlier ones gave back; a cache one page smaller must be refused."""
    folder, reqs, ref = oracle["A"]
    tr = Trace()
    tr.batches("b", reqs, GROUPS, [len(r) // 2 + 1 for r in reqs])
    peak = tr.max_tokens()
    got = run_trace(tr, folder, "float32", str(tmp_path / "tight"), max_tokens=peak)
    for i, r in enumerate(ref):
        assert np.abs(got[(f"b{i}", len(r) - 1)] - r[-1]).max() <= TOL_F32 * 2
    with pytest.raises(AssertionError, match="does not fit in the cache|cache is full"):
        run_trace(tr, folder, "float32", str(tmp_path / "short"), max_tokens=peak - 64)
