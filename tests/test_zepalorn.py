"""Zepalorn on the CPU: the plain implementation's mechanisms one by one, configuration, builder, weights, cache groups and
states, and the engine's host side (step building, pages, windows, chunks, kept first tokens, state slots, scheduler) with the
torch stand-in kernels, against the plain implementation."""
import json
import math

import pytest
import torch

import plain_zepalorn as plain
from torch_kernels import TorchKernels
from zepalorn_cases import CASES, check_long_decoding, check_mixed, check_whole_and_cut, plain_logits, setup_case


@pytest.fixture(scope="module")
def cases(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("zepalorn")
    return {name: setup_case(tmp, name, "float32") for name in CASES}


# ------------------------------------------------------------------------------------------------ the plain implementation itself
def test_plain_mask_window_keeps_the_first_tokens():
    ok = plain.visible(12, "window", {"size": 4, "keep_first": 2})
    assert ok[9].nonzero().flatten().tolist() == [0, 1, 6, 7, 8, 9]      # i - j < 4, or j < 2
    assert ok[3].nonzero().flatten().tolist() == [0, 1, 2, 3]
    assert ok[5].nonzero().flatten().tolist() == [0, 1, 2, 3, 4, 5]     # the window still touches the kept ones
    ok = plain.visible(12, "chunk", {"size": 5})
    assert ok[9].nonzero().flatten().tolist() == [5, 6, 7, 8, 9] and ok[10].nonzero().flatten().tolist() == [10] and ok[4].sum() == 5


def test_plain_stretched_frequencies():
    f, mult = plain.rotary_frequencies({"dims": 8, "base": 100.0}, torch.float64)
    assert torch.allclose(f, torch.tensor([1.0, 100 ** -0.25, 0.1, 100 ** -0.75], dtype=torch.float64)) and mult == 1.0
    rot = {"dims": 8, "base": 100.0, "scaling": {"factor": 4.0, "original": 50, "fast": 4.0, "slow": 1.0}}
    g, mult = plain.rotary_frequencies(rot, torch.float64)
    # d(t) = 8 ln(50 / (2 pi t)) / (2 ln 100): d(4) = 0.597 -> lo = 0, d(1) = 1.80 -> hi = 2; ramp = 0, 1/2, 1, 1
    assert torch.allclose(g, f * torch.tensor([1.0, 0.5 / 4 + 0.5, 0.25, 0.25], dtype=torch.float64))
    assert mult == pytest.approx(0.1 * math.log(4.0) + 1.0)


def test_plain_rotation_layouts():
    x = torch.arange(12, dtype=torch.float64).view(1, 1, 12) + 1
    pos = torch.tensor([3])
    rot = {"dims": 4, "base": 10.0}
    f, _ = plain.rotary_frequencies(rot, torch.float64)
    a = 3 * f
    half = plain.rotate(x, pos, rot, interleaved=False)[0, 0]
    assert torch.allclose(half[[0, 2]], torch.stack([1 * a[0].cos() - 3 * a[0].sin(), 3 * a[0].cos() + 1 * a[0].sin()]))
    inter = plain.rotate(x, pos, rot, interleaved=True)[0, 0]
    assert torch.allclose(inter[[2, 3]], torch.stack([3 * a[1].cos() - 4 * a[1].sin(), 4 * a[1].cos() + 3 * a[1].sin()]))
    assert torch.equal(half[4:], x[0, 0, 4:]) and torch.equal(inter[4:], x[0, 0, 4:])       # the rest passes


def test_plain_convolution_and_recurrences_by_hand():
    u = torch.tensor([[1.0], [2.0], [3.0]], dtype=torch.float64)
    y = plain.causal_conv(u, torch.tensor([[10.0, 1.0]], dtype=torch.float64))      # the last column is the current token's
    assert y.flatten().tolist() == [1.0, 12.0, 23.0]
    # the delta rule writes before it reads: with beta = 1, no decay and unit key, reading with the key returns the value
    m = {"heads": 1, "kv_heads": 1, "dim": 2, "vdim": 2, "conv": 2}
    W = {"p.q": torch.eye(2), "p.k": torch.eye(2), "p.v": torch.eye(2), "p.q.conv": torch.tensor([[0.0, 1.0]] * 2), "p.k.conv": torch.tensor([[0.0, 1.0]] * 2),
         "p.v.conv": torch.tensor([[0.0, 1.0]] * 2), "p.b": torch.full((1, 2), 50.0), "p.a1": torch.zeros(1, 2), "p.a2": torch.zeros(2, 1),
         "p.dt_bias": torch.full((2,), -60.0), "p.A_log": torch.zeros(1), "p.g1": torch.zeros(1, 2), "p.g2": torch.zeros(2, 1), "p.norm": torch.ones(2),
         "p.o": torch.eye(2)}
    W = {k: v.double() for k, v in W.items()}
    h = torch.tensor([[3.0, 0.0]], dtype=torch.float64)
    out = plain.channel_delta(m, W, "p", h, 1e-12)
    # q = k = silu(3) e_0 made unit; v = silu(h); o = v (k . q) = v / sqrt(2); then the unit norm over vdim, times sigmoid(0) = 1/2
    v = plain.silu(h)
    want = v / v.pow(2).mean().sqrt() * 0.5
    assert torch.allclose(out, want, atol=1e-6)


def test_plain_feed_forward_clamps():
    f = {"ff": 2, "limit": 1.0}
    W = {"p.gate": torch.tensor([[5.0], [-5.0]]).double(), "p.up": torch.tensor([[5.0], [-5.0]]).double(), "p.down": torch.eye(2).double()}
    y = plain.feed_forward(f, W, "p", torch.tensor([[1.0]], dtype=torch.float64))[0]
    assert y[0].item() == pytest.approx(1.0 * torch.sigmoid(torch.tensor(1.702)).item() * 2.0)      # gate cut at 1, up cut at 1, plus one
    assert y[1].item() == pytest.approx(-5.0 * torch.sigmoid(torch.tensor(-5.0 * 1.702)).item() * 0.0, abs=1e-12)   # gate not cut below; up at -1


# ------------------------------------------------------------------------------------------------ configuration, builder, cache
def test_config_reads_every_key():
    from llm_infrence_engine_b200.config import ConfigError
    from llm_infrence_engine_b200.config.model_config import ZepalornConfig

    cfg = ZepalornConfig.from_dict(CASES["A"][0])
    assert (cfg.vocab, cfg.width, cfg.eps, cfg.embedding_scale) == (83, 48, 1e-5, 3.0) and len(cfg.layers) == 6
    d, a, p = cfg.layers[0], cfg.layers[1], cfg.layers[2]
    assert d.kind == "channel_delta" and (d.mixer.heads, d.mixer.kv_heads, d.mixer.dim, d.mixer.vdim, d.mixer.conv, d.ff, d.ff_limit) == (4, 2, 16, 24, 3, 64, 1.5)
    assert (a.mixer.mask_size, a.mixer.keep_first, a.mixer.chunked, a.mixer.rot.dims, a.mixer.rot.factor, a.mixer.rot.original) == (19, 3, False, 16, 2.0, 64.0)
    assert (p.mixer.left.chunked, p.mixer.left.mask_size, p.mixer.left.softcap, p.mixer.left.conv, p.mixer.left.qk_norm, p.mixer.left.interleaved) == (True, 21, 5.0, 2, True, True)
    assert (p.mixer.right.state, p.mixer.right.groups, p.mixer.right.norm_groups, p.mixer.right.conv) == (16, 1, 1, 4) and p.ff is None
    assert [layer.weights_of for layer in cfg.layers] == [None, None, None, 1, 0, 2]
    assert ZepalornConfig.from_dict(CASES["B"][0]).layers[3].mixer.rot is None
    for change in (lambda c: c["layers"][3].update(weights_of=4), lambda c: c["layers"][3]["mixer"].update(heads=3),
                   lambda c: c["layers"][0].update(type="convolution"), lambda c: c["layers"][2]["mixer"]["right"].update(norm_groups=5),
                   lambda c: c["layers"][1]["mixer"]["rot"].update(dims=26)):
        bad = json.loads(json.dumps(CASES["A"][0]))
        change(bad)
        with pytest.raises(ConfigError):
            ZepalornConfig.from_dict(bad)


def test_builder_names_the_checkpoint_tensors_and_the_cache():
    from llm_infrence_engine_b200.cache.spec import FixedStateSpec, PagedKVSpec
    from llm_infrence_engine_b200.engine.step import group_layout, has_fixed_state
    from llm_infrence_engine_b200.models import build_model_spec
    from llm_infrence_engine_b200.weights.loader import expected_tensors

    spec = build_model_spec(CASES["A"][0])
    names = set(expected_tensors(spec))
    assert {"embed", "final.norm", "l0.norm1", "l0.norm1b", "l0.norm2", "l0.norm2b", "l0.mix.q", "l0.mix.q.conv", "l0.mix.b", "l0.mix.A_log", "l0.mix.a1",
            "l0.mix.a2", "l0.mix.dt_bias", "l0.mix.g1", "l0.mix.g2", "l0.mix.norm", "l0.mix.o", "l0.mlp.gate", "l0.mlp.up", "l0.mlp.down", "l1.mix.q",
            "l1.mix.k", "l1.mix.v", "l1.mix.o", "l2.mix.left.q.conv", "l2.mix.left.q.norm", "l2.mix.left.k.norm", "l2.mix.left.out", "l2.mix.right.out",
            "l2.mix.right.in", "l2.mix.right.conv", "l2.mix.right.conv.b", "l2.mix.right.D", "l2.mix.right.norm", "l2.mix.right.o"} <= names
    assert not any(n.startswith(("l3.", "l4.", "l5.", "l2.mlp", "l2.norm2", "head", "l1.mix.q.conv")) for n in names)
    # a layer that runs on another's weights is that layer's part once more, with a cache entry of its own
    assert [(c.layer, c.cache, c.write) for c in spec.schedule] == [(0, 0, True), (1, 1, True), (2, 2, True), (1, 3, True), (0, 4, True), (2, 5, True)]
    specs = spec.cache_specs()
    assert specs[1] == PagedKVSpec(2, 24, 19, 16, 3, None) == specs[3]
    assert specs[0] == (FixedStateSpec((4, 24, 16)), FixedStateSpec((2, 2 * 2 * 16 + 4 * 24)))
    assert specs[2] == ((PagedKVSpec(1, 32, None, 32, 0, 21), FixedStateSpec((1, 4 * 32 + 32 + 32))), (FixedStateSpec((4, 12, 16)), FixedStateSpec((3, 48 + 32))))
    groups, of_entry = group_layout(specs)
    assert len(groups) == 2 and of_entry == [(None, None), 0, ((1, None), (None, None)), 0, (None, None), ((1, None), (None, None))]
    assert has_fixed_state(specs)


def test_weights_load_and_the_low_ranks_come_from_the_checkpoint(tmp_path):
    from llm_infrence_engine_b200.models import build_model_spec
    from llm_infrence_engine_b200.weights import load_weights
    from llm_infrence_engine_b200.weights.random_init import random_tensors
    from llm_infrence_engine_b200.weights.safetensors_io import write_safetensors

    cfg = CASES["C"][0]
    t = random_tensors(cfg, 1)
    g = torch.Generator().manual_seed(2)
    t["l1.mix.a1"], t["l1.mix.a2"] = torch.randn(5, 40, generator=g), torch.randn(6 * 40, 5, generator=g)     # ranks of 5 and 11: no config key names them
    t["l1.mix.g1"], t["l1.mix.g2"] = torch.randn(11, 40, generator=g), torch.randn(6 * 33, 11, generator=g)
    (tmp_path / "m").mkdir()
    write_safetensors(tmp_path / "m" / "model.safetensors", {k: v.contiguous() for k, v in t.items()})
    spec = build_model_spec(cfg)
    load_weights(spec, tmp_path / "m", torch.float32, "cpu")
    mixer = spec.layers[1].mixer
    assert (mixer.rank_a, mixer.rank_g) == (5, 11) and mixer.w_in.shape[0] % 8 == 0
    assert torch.equal(mixer.w_in[mixer.a1_col:mixer.a1_col + 5], t["l1.mix.a1"]) and torch.equal(mixer.w_in[mixer.g1_col:mixer.g1_col + 11], t["l1.mix.g1"])
    assert torch.equal(mixer.w_in[mixer.b_col:mixer.b_col + 6], t["l1.mix.b"]) and mixer.b_col % 8 == 0 and mixer.a1_col % 8 == 0 and mixer.g1_col % 8 == 0
    assert spec.head.matrix() is spec.embedding.table and spec.embedding.scale == 0.5
    assert spec.layers[0].mixer.conv_taps == 0 and spec.layers[2].mixer.left.conv_w.shape == ((6 + 3) * 16 + 3 * 16, 3)


def test_pages_of_windows_chunks_and_kept_tokens():
    from llm_infrence_engine_b200.cache.manager import CacheManager
    from llm_infrence_engine_b200.cache.spec import NULL_PAGE, PagedKVSpec

    ps = 8
    cm = CacheManager([PagedKVSpec(1, 8, 19, 8, 3, None), PagedKVSpec(1, 8, None, 8, 0, 21), PagedKVSpec(1, 8, 12, 8, 17, None)], 40, ps, 2)
    cm.admit("r")
    n = 0
    for step in [5, 30, 1, 1, 1, 40, 2, 1, 1, 1, 1, 1, 1, 1, 60]:
        cm.reserve("r", n, n + step)
        n += step
        cm.release_passed("r", n)
        cm.check_invariants()
        for g, spec in enumerate(cm.groups):
            table = cm.block_table("r", g)
            for page in range(len(table)):
                lo, hi = page * ps, page * ps + ps - 1
                first = max(0, n - spec.window + 1) if spec.window else 0
                if spec.chunk:
                    first = n // spec.chunk * spec.chunk
                needed = hi >= first or lo < spec.keep_first
                assert (table[page] != NULL_PAGE) == needed, (g, n, page)
    cm.free("r")
    assert all(p.num_free == p.capacity for p in cm.pools)


# ------------------------------------------------------------------------------------------------ the engine's host side
@pytest.mark.parametrize("name", sorted(CASES))
def test_engine_whole_and_cut_on_cpu(cases, name):
    check_whole_and_cut(cases[name], name, "float32", TorchKernels(), "cpu")


def test_engine_mixed_batches_on_cpu(cases):
    check_mixed(cases["A"], "A", "float32", TorchKernels(), "cpu", seeds=(0,))


def test_engine_long_decoding_on_cpu(cases):
    check_long_decoding(cases["B"], "B", "float32", TorchKernels(), "cpu", total=120)


def test_greedy_generation_through_the_entry_point_on_cpu(cases):
    from llm_infrence_engine_b200.engine import Engine

    folder, cfg, tensors, prompts, want = cases["C"]
    eng = Engine(folder, kernels=TorchKernels(), dtype="float32", device="cpu", max_len=128, max_seqs=3, block_size=16, num_blocks=20,
                 max_num_batched_tokens=24)
    ps = [prompts["c"], prompts["d"], prompts["f"], prompts["b"][:30]]
    results = eng.generate(ps, max_new_tokens=8)
    for p, r in zip(ps, results):
        seq = list(p) + r.token_ids
        ref = plain_logits(cfg, tensors, seq)[len(p) - 1:-1]
        assert r.token_ids == ref.argmax(-1).tolist()
    eng.cache.check_invariants()
    assert all(pool.num_free == pool.capacity for pool in eng.cache.pools)
