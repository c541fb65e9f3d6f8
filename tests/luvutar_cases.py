"""Small Luvutar models and the ways of running them that the CPU and the GPU tests share.

The configurations differ from each other in every size and option: streams (none, 1, 2, 3, 5), groups of 1, 2, 3, 4 and 5
query heads per key/value head, values longer and shorter than keys, a rotation over part of the rotated entries,
windows shorter and longer than a page, distance tables of 6, 8 and 16 rows, a layer without feed-forward, layers
that read another layer's keys and values. The engine runs them through ``TraceReplayer`` (the step function, the
cache manager, the kernels object it is given); the oracle is ``plain_luvutar.forward`` on whole sequences.
"""
from __future__ import annotations

import json
from pathlib import Path

import torch

import plain_luvutar as plain


def _latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, window=None, rot=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale}
    if window:
        m["mask"] = {"size": window}
    if rot:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
    return {"type": "latent_attention", "mixer": m}


def _biased(heads, kv_heads, dim, vdim, scale, bias_max, temp=None, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "bias_max": bias_max}
    if temp:
        m["q_temp"] = {"coef": temp[0], "every": temp[1]}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m}


def _ff(layer, ff):
    layer["mlp"] = {"kind": "dense", "ff": ff} if ff else None
    return layer


def _model(vocab, width, eps, streams, layers):
    d = {"architecture": "Luvutar", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if streams is not None:
        d["streams"] = streams
    return d


CASES = {
    # two streams; a window shorter than a page; a partly rotated part; a layer without feed-forward; shared keys and values
    "P": (_model(97, 48, 1e-5, 2, [
        _ff(_latent(2, 16, 8, 24, 24, 40, 0.2, window=9, rot=(100.0, 8)), 64),
        _ff(_biased(4, 2, 16, 8, 0.3, 20, temp=(0.5, 5)), None),
        _ff(_biased(4, 2, 16, 8, 0.25, 20, temp=(0.25, 3), kv_from=1), 32),
        _ff(_latent(3, 8, 16, 16, 16, 24, 0.15, window=21, rot=(5000.0, 8)), 40),
    ]), {"l1.mix.rel": 8, "l2.mix.rel": 6}, 8),
    # one plain residual stream; one query head per key/value head; five heads on one latent; a window longer than a page; no window
    "Q": (_model(61, 40, 1e-6, None, [
        _ff(_biased(3, 3, 24, 24, 0.2, 50, temp=(0.3, 7)), 56),
        _ff(_latent(5, 12, 4, 8, 32, 16, 0.3, window=33, rot=(10000.0, 4)), 48),
        _ff(_latent(2, 8, 8, 8, 8, 8, 0.35, rot=(300.0, 8)), None),
        _ff(_biased(3, 3, 24, 24, 0.2, 50, kv_from=0), 24),
    ]), {"l0.mix.rel": 16, "l3.mix.rel": 16}, 16),
    # five streams; a single stream under hyper-connections is case S
    "R": (_model(120, 64, 1e-6, 5, [
        _ff(_biased(6, 1, 32, 40, 0.18, 12, temp=(0.7, 2)), 96),
        _ff(_latent(4, 16, 16, 32, 48, 64, 0.12, window=16, rot=(50.0, 16)), 72),
    ]), {"l0.mix.rel": 8}, 16),
    # heads of 64 and of 128 (keys) / 64 (values): in bfloat16 their prompt portions take the tensor-core kernel of their own
    "T": (_model(75, 56, 1e-6, 3, [
        _ff(_biased(6, 2, 64, 64, 0.12, 40, temp=(0.3, 11)), 48),
        _ff(_latent(2, 16, 16, 32, 24, 48, 0.2, window=30, rot=(1000.0, 16)), None),
        _ff(_biased(4, 1, 128, 64, 0.09, 25, temp=(0.2, 6)), 40),
        _ff(_biased(6, 2, 64, 64, 0.12, 40, kv_from=0), 32),
    ]), {"l0.mix.rel": 10, "l2.mix.rel": 8, "l3.mix.rel": 10}, 16),
    "S": (_model(50, 32, 1e-5, 1, [
        _ff(_latent(1, 8, 8, 8, 16, 16, 0.3, window=5, rot=(20.0, 8)), 32),
        _ff(_biased(2, 1, 8, 16, 0.4, 9, temp=(1.0, 4)), 16),
    ]), {"l1.mix.rel": 6}, 4),
}


def make_folder(tmp: Path, name: str, store: str = "float32", std: float = 0.08, seed: int = 11) -> Path:
    """A model folder for case ``name`` with random weights; distance tables get the row counts the case names."""
    from llm_infrence_engine_b200.weights.random_init import random_tensors
    from llm_infrence_engine_b200.weights.safetensors_io import write_safetensors

    cfg, rel_rows, _ = CASES[name]
    t = random_tensors(cfg, seed, std)
    g = torch.Generator().manual_seed(seed + 1)
    for key, rows in rel_rows.items():
        t[key] = torch.randn(rows, t[key].shape[1], generator=g) * 0.5
    for key in t:
        if key.endswith(".sink"):
            t[key] = torch.randn(t[key].shape, generator=g)          # sinks that matter
    dtype = {"float32": torch.float32, "bfloat16": torch.bfloat16}[store]
    folder = Path(tmp) / f"luvutar_{name}_{store}"
    folder.mkdir(parents=True, exist_ok=True)
    write_safetensors(folder / "model.safetensors", {k: v.to(dtype).contiguous() for k, v in t.items()})
    (folder / "config.json").write_text(json.dumps(cfg))
    return folder


def load_plain(folder: Path):
    from llm_infrence_engine_b200.weights.safetensors_io import SafetensorsFile

    f = SafetensorsFile(folder / "model.safetensors")
    try:
        tensors = {n: f.tensor(n).clone() for n in f.names()}
    finally:
        f.close()
    return json.loads((folder / "config.json").read_text()), tensors


def prompt(vocab: int, n: int, seed: int) -> list:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def replayer(folder, name, dtype, max_tokens, kernels=None, device="cuda:0", **kw):
    from llm_infrence_engine_b200.engine import TraceReplayer

    return TraceReplayer(str(folder), dtype, max_tokens, device=device, kernels=kernels, block_size=CASES[name][2], **kw)


def row_error(got: torch.Tensor, want: torch.Tensor) -> float:
    """Largest difference of a row of logits (its mean taken off, root mean square over the vocabulary), in units of the
    logits' own spread."""
    d = got.double() - want.double()
    d = d - d.mean(-1, keepdim=True)
    return float((d.pow(2).mean(-1).sqrt().max() / want.double().std()).item())


LIMIT = {"float32": 2e-5, "bfloat16": 4e-2}


def run_alone(rp, rid, tokens, cuts, step0=0):
    """One request through the replayer in the given portions ``[(lo, hi), ...]``; returns all its logits ``[T, vocab]``."""
    out = []
    for i, (lo, hi) in enumerate(cuts):
        end = [rid] if hi == len(tokens) else []
        out.append(rp.step({"step": step0 + i, "entries": [{"id": rid, "tokens": tokens[lo:hi], "want": list(range(hi - lo))}], "end": end}))
    return torch.cat(out)


def cuts_of(n: int, sizes) -> list:
    out, i, k = [], 0, 0
    while i < n:
        s = min(sizes[k % len(sizes)], n - i)
        out.append((i, i + s))
        i += s
        k += 1
    return out


def mixed_schedule(lens: dict, seed: int, max_live: int = 4):
    """Steps of up to ``max_live`` live requests: each step, every live request brings a portion of 2 to 40 tokens or, once
    most of it is in, single tokens; some sit a step out. Yields ``[(id, lo, hi), ...]`` per step."""
    g = torch.Generator().manual_seed(seed)
    waiting = list(lens)
    at = {}
    live = []
    while waiting or live:
        while waiting and len(live) < max_live and (not live or torch.rand(1, generator=g).item() < 0.6):
            rid = waiting.pop(0)
            live.append(rid)
            at[rid] = 0
        step = []
        for rid in list(live):
            if len(live) > 1 and torch.rand(1, generator=g).item() < 0.2:
                continue
            left = lens[rid] - at[rid]
            n = 1 if (at[rid] > 0.7 * lens[rid]) else int(torch.randint(2, 41, (1,), generator=g).item())
            n = min(n, left)
            step.append((rid, at[rid], at[rid] + n))
            at[rid] += n
            if at[rid] == lens[rid]:
                live.remove(rid)
        if step:
            yield step


def run_mixed(rp, prompts: dict, seed: int):
    """Runs ``mixed_schedule`` and returns every request's logits ``[T, vocab]``; checks the cache's invariants on the way."""
    lens = {k: len(v) for k, v in prompts.items()}
    got = {k: [] for k in prompts}
    for n, step in enumerate(mixed_schedule(lens, seed)):
        entries = [{"id": rid, "tokens": prompts[rid][lo:hi], "want": list(range(hi - lo))} for rid, lo, hi in step]
        end = [rid for rid, lo, hi in step if hi == lens[rid]]
        out = rp.step({"step": n, "entries": entries, "end": end})
        rp.cache.check_invariants()
        o = 0
        for rid, lo, hi in step:
            got[rid].append(out[o:o + hi - lo])
            o += hi - lo
    return {k: torch.cat(v) for k, v in got.items()}


def plain_logits(cfg, tensors, tokens):
    return plain.forward(cfg, tensors, tokens, torch.float64)


# ---------------------------------------------------------------------------------------------------------------------
# The checks themselves: each takes the kernels object and the device, so the same statements run on the CPU (torch
# stand-in kernels: the host side of the engine) and on the GPU (the package's kernels).

LENS = {"a": 150, "b": 67, "c": 41, "d": 9, "e": 118, "f": 2}


def setup_case(tmp, name, dtype):
    folder = make_folder(tmp, name, dtype)
    cfg, tensors = load_plain(folder)
    prompts = {k: prompt(cfg["vocab"], n, 3 + i) for i, (k, n) in enumerate(LENS.items())}
    want = {k: plain_logits(cfg, tensors, p) for k, p in prompts.items()}
    return folder, cfg, tensors, prompts, want


def check_whole_and_cut(case, name, dtype, kernels, device):
    """Whole prompts; the last tokens one by one; portions of several sizes down to two tokens and one."""
    folder, cfg, tensors, prompts, want = case
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
            assert err <= LIMIT[dtype], f"{name} {dtype} request {k} ({T} tokens) {what}: {err:.3g}"
            rp.cache.check_invariants()


def check_mixed(case, name, dtype, kernels, device, seeds=(0, 1)):
    """Batches of unequal requests on a pool that holds only the live ones: every request as if it ran alone."""
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
    """A short prompt, then hundreds of tokens one by one: windows pass over decoded tokens and give their pages back."""
    folder, cfg, tensors, prompts, want = case
    p = prompt(cfg["vocab"], total, 99)
    ref = plain_logits(cfg, tensors, p)
    rp = replayer(folder, name, dtype, 320, kernels, device)
    got = run_alone(rp, "long", p, cuts_of(total, [3] + [1] * total))
    err = row_error(got, ref)
    assert err <= LIMIT[dtype], f"{name} {dtype} long decoding: {err:.3g}"
    first = row_error(got[:4], ref[:4])
    assert first <= LIMIT[dtype], f"{name} {dtype} first tokens: {first:.3g}"
