"""Small Zepalorn models and the ways of running them that the CPU and the GPU tests share.

The configurations differ from each other in every size and option: layer orders, layers that run on another layer's weights,
query/key groups of 1, 2 and 3, keys and values of different sizes, heads turned in part and in full, with and without
stretched frequencies, windows shorter and longer than a page with and without kept first tokens, chunks that end on and off
page borders, convolutions of 2, 3 and 4 taps, state groups and norm groups of 1 and more, layers without feed-forward. The
engine runs them through ``TraceReplayer`` (the step function, the cache manager, the kernels object it is given); the oracle
is ``plain_zepalorn.forward`` on whole sequences.
"""
from __future__ import annotations

import json
from pathlib import Path

import torch

import plain_zepalorn as plain
from luvutar_cases import cuts_of, load_plain, prompt, row_error, run_alone, run_mixed  # noqa: F401  (generic helpers)


def _rot(dims, base, scaling=None):
    r = {"dims": dims, "base": base}
    if scaling:
        r["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return r


def _delta(heads, kv_heads, dim, vdim, conv):
    return {"type": "channel_delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}}


def _attention(heads, kv_heads, dim, vdim, scale, window=None, keep_first=None, rot=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window:
        m["mask"] = {"size": window}
        if keep_first is not None:
            m["mask"]["keep_first"] = keep_first
    if rot:
        m["rot"] = rot
    return {"type": "attention", "mixer": m}


def _parallel(left, right):
    heads, kv_heads, dim, vdim, scale, conv, chunk, softcap, rot = left
    lm = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "conv": conv, "mask": {"size": chunk}, "rot": rot}
    if softcap:
        lm["softcap"] = softcap
    rm = dict(zip(("heads", "vdim", "state", "groups", "norm_groups", "conv"), right))
    return {"type": "parallel", "mixer": {"left": lm, "right": rm}}


def _ff(layer, ff, limit=2.0):
    layer = json.loads(json.dumps(layer))
    layer["mlp"] = {"kind": "dense", "ff": ff, "limit": limit} if ff else None
    return layer


def _again(layers, j):
    layer = json.loads(json.dumps(layers[j]))
    layer["weights_of"] = j
    return layer


def _model(vocab, width, eps, scale, layers, again=()):
    layers = list(layers)
    for j in again:
        layers.append(_again(layers, j))
    return {"architecture": "Zepalorn", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": scale}, "layers": layers}


CASES = {
    # (config, page size). A: every mixer; partly turned heads with stretched frequencies; a window of 19 (more than two pages of 8) that
    # keeps 3 tokens; chunks of 21; a layer without feed-forward; three layers run again on earlier weights, in another order
    "A": (_model(83, 48, 1e-5, 3.0, [
        _ff(_delta(4, 2, 16, 24, 3), 64, 1.5),
        _ff(_attention(6, 2, 24, 16, 0.2, window=19, keep_first=3, rot=_rot(16, 1000.0, (2.0, 64, 8.0, 1.0))), 40, 2.5),
        _ff(_parallel((4, 1, 32, 32, 0.18, 2, 21, 5.0, _rot(32, 100.0, (4.0, 32, 4.0, 0.5))), (4, 12, 16, 1, 1, 4)), None),
    ], again=(1, 0, 2)), 8),
    # B: the side-by-side mixer first; chunks of a page exactly; kept tokens that fill more than a page; fully turned heads of 64 without
    # stretching; an attention layer with neither rotation nor mask; one query/key head per head in the delta rule; sizes that are no
    # multiples of 32
    "B": (_model(120, 64, 1e-6, 1.0, [
        _ff(_parallel((2, 2, 16, 8, 0.25, 4, 16, None, _rot(8, 50.0)), (6, 16, 8, 2, 3, 2)), 96, 1.0),
        _ff(_delta(3, 3, 8, 40, 4), None),
        _ff(_attention(2, 1, 64, 64, 0.125, window=40, keep_first=17, rot=_rot(64, 10000.0)), 32, 3.0),
        _ff(_attention(3, 3, 8, 8, 0.35), 24, 2.0),
    ], again=(0,)), 16),
    # C: wider heads for the recurrences (a key size that is no power of two, values that do not fill a warp, a state of 40), a window
    # shorter than a page without kept tokens, chunks longer than the prompts' portions, three delta heads per query/key head
    "C": (_model(64, 40, 1e-5, 0.5, [
        _ff(_attention(4, 4, 16, 24, 0.25, window=5, keep_first=0, rot=_rot(8, 30.0, (8.0, 16, 2.0, 0.25))), 48, 2.0),
        _ff(_delta(6, 2, 40, 33, 2), 56, 0.75),
        _ff(_parallel((6, 3, 16, 16, 0.2, 3, 50, 2.0, _rot(16, 500.0, (3.0, 40, 16.0, 2.0))), (2, 20, 40, 2, 2, 3)), 32, 2.0),
    ]), 16),
}


def make_folder(tmp: Path, name: str, store: str = "float32", std: float = 0.08, seed: int = 11, sharp: float = 1.0) -> Path:
    """A model folder for case ``name`` with random weights. ``sharp`` multiplies the query projections, so that the softmax
    picks few keys and a key that is lost, or seen when it should not be, moves the logits by far more than rounding does."""
    from llm_infrence_engine_b200.weights.random_init import random_tensors
    from llm_infrence_engine_b200.weights.safetensors_io import write_safetensors

    cfg, _ = CASES[name]
    t = random_tensors(cfg, seed, std)
    if sharp != 1.0:
        for key in t:
            if key.endswith("mix.q") or key.endswith("left.q"):
                t[key] = t[key] * sharp
    dtype = {"float32": torch.float32, "bfloat16": torch.bfloat16}[store]
    folder = Path(tmp) / f"zepalorn_{name}_{store}_{sharp}"
    folder.mkdir(parents=True, exist_ok=True)
    write_safetensors(folder / "model.safetensors", {k: v.to(dtype).contiguous() for k, v in t.items()})
    (folder / "config.json").write_text(json.dumps(cfg))
    return folder


def replayer(folder, name, dtype, max_tokens, kernels=None, device="cuda:0", **kw):
    from llm_infrence_engine_b200.engine import TraceReplayer

    return TraceReplayer(str(folder), dtype, max_tokens, device=device, kernels=kernels, block_size=CASES[name][1], **kw)


def plain_logits(cfg, tensors, tokens):
    return plain.forward(cfg, tensors, tokens, torch.float64)


# float32: only the order of summation differs. bfloat16: activations are rounded to 8 bits between the kernels and every sublayer
# ends in a norm that brings its result back to full size, so the rounding of a dozen sublayers adds up to a few per cent of the
# logits' spread (measured 0.03 to 0.05 at these sizes); a wrong key or a lost state moves them by 0.3 and more
LIMIT = {"float32": 3e-5, "bfloat16": 1e-1}

# D: convolutions of a single tap (no state rows at all), and a first layer that runs on the weights of a LATER one
_d_layers = [_ff(_delta(2, 1, 16, 8, 1), 24, 2.0), _ff(_parallel((2, 2, 8, 8, 0.3, 1, 7, 3.0, _rot(4, 20.0)), (2, 8, 8, 1, 2, 1)), 16, 1.5), _ff(_delta(2, 1, 16, 8, 1), 24, 2.0)]
_d_layers[0]["weights_of"] = 2
# E: sizes that take the kernels' slow paths: a width that is no multiple of 8, heads of 20 and 10 entries (no 16-byte pieces), values
# of 12, 6 and 4, more kept tokens than the window is long, chunks of 3, convolutions of 8, 5 and 6 taps, a state of 12, pages of 4
CASES["E"] = (_model(57, 44, 1e-6, 2.0, [
    _ff(_delta(3, 1, 10, 6, 8), 52, 0.5),
    _ff(_attention(2, 2, 20, 12, 0.22, window=7, keep_first=9, rot=_rot(6, 7.0, (1.5, 24, 3.0, 0.5))), None),
    _ff(_parallel((3, 1, 12, 20, 0.3, 5, 3, 1.0, _rot(12, 40.0)), (5, 4, 12, 5, 5, 6)), 36, 4.0),
], again=(0,)), 4)
CASES["D"] = ({"architecture": "Zepalorn", "vocab": 40, "width": 24, "norm": {"eps": 1e-5}, "layers": _d_layers}, 8)
LENS = {"a": 150, "b": 67, "c": 41, "d": 9, "e": 118, "f": 2}


def setup_case(tmp, name, dtype, **kw):
    folder = make_folder(tmp, name, dtype, **kw)
    cfg, tensors = load_plain(folder)
    prompts = {k: prompt(cfg["vocab"], n, 3 + i) for i, (k, n) in enumerate(LENS.items())}
    want = {k: plain_logits(cfg, tensors, p) for k, p in prompts.items()}
    return folder, cfg, tensors, prompts, want


# ---------------------------------------------------------------------------------------------------------------------
# The checks themselves: each takes the kernels object and the device, so the same statements run on the CPU (torch
# stand-in kernels: the host side of the engine) and on the GPU (the package's kernels).

def check_whole_and_cut(case, name, dtype, kernels, device, limit=None):
    """Whole prompts; the last tokens one by one; portions of several sizes down to two tokens and one."""
    folder, cfg, tensors, prompts, want = case
    limit = limit or LIMIT[dtype]
    rp = replayer(folder, name, dtype, 192, kernels, device)
    n = 0
    for k, p in prompts.items():
        T = len(p)
        ways = {"whole": [(0, T)], "tail one by one": cuts_of(T, [max(1, T - 40)] + [1] * 40),
                "portions": cuts_of(T, [7, 2, 33, 1, 16, 3, 2, 64, 5]), "pairs": cuts_of(T, [2])}
        for what, cuts in ways.items():
            if what == "pairs" and T > 70:
                continue
            got = run_alone(rp, f"{k}{n}", p, cuts, n)
            n += len(cuts)
            err = row_error(got, want[k])
            assert err <= limit, f"{name} {dtype} request {k} ({T} tokens) {what}: {err:.3g}"
            rp.cache.check_invariants()
    assert rp.cache.num_free_slots() == 4 and all(p.num_free == p.capacity for p in rp.cache.pools)


def check_mixed(case, name, dtype, kernels, device, seeds=(0, 1)):
    """Batches of unequal requests on a pool that holds only the live ones (pages and state slots are used again): every
    request as if it ran alone."""
    folder, cfg, tensors, prompts, want = case
    for seed in seeds:
        lens = sorted((len(p) for p in prompts.values()), reverse=True)
        rp = replayer(folder, name, dtype, sum(-(-n // 64) * 64 for n in lens[:4]), kernels, device)
        got = run_mixed(rp, prompts, seed)
        for k in prompts:
            err = row_error(got[k], want[k])
            assert err <= LIMIT[dtype], f"{name} {dtype} mixed (seed {seed}) request {k}: {err:.3g}"
        assert rp.cache.num_free_slots() == 4 and all(p.num_free == p.capacity for p in rp.cache.pools)


def check_long_decoding(case, name, dtype, kernels, device, total=300):
    """A short prompt, then hundreds of tokens one by one: windows and chunks pass over decoded tokens and give their pages back,
    the kept first tokens stay, the states run on."""
    folder, cfg, tensors, prompts, want = case
    p = prompt(cfg["vocab"], total, 99)
    ref = plain_logits(cfg, tensors, p)
    rp = replayer(folder, name, dtype, 320, kernels, device)
    got = run_alone(rp, "long", p, cuts_of(total, [3] + [1] * total))
    err = row_error(got, ref)
    assert err <= LIMIT[dtype], f"{name} {dtype} long decoding: {err:.3g}"
    first = row_error(got[:4], ref[:4])
    assert first <= LIMIT[dtype], f"{name} {dtype} first tokens: {first:.3g}"
