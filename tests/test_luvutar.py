"""Luvutar on the CPU: configuration, builder, weights, cache groups, and the engine's host side (step building, pages,
windows, shared keys and values, scheduler) with the torch stand-in kernels, against the plain implementation."""
import json

import pytest
import torch

import plain_luvutar as plain
from luvutar_cases import (CASES, LIMIT, check_long_decoding, check_mixed, check_whole_and_cut, load_plain, make_folder, plain_logits,
                           prompt, row_error, setup_case)
from torch_kernels import TorchKernels


@pytest.fixture(scope="module")
def cases(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("luvutar")
    return {name: setup_case(tmp, name, "float32") for name in CASES}


def test_config_reads_every_key():
    from llm_infrence_engine_b200.config import ConfigError, LuvutarConfig

    cfg = LuvutarConfig.from_dict(CASES["P"][0])
    assert cfg.streams == 2 and cfg.vocab == 97 and cfg.width == 48 and cfg.eps == 1e-5
    lat, att, shared = cfg.layers[0], cfg.layers[1], cfg.layers[2]
    assert lat.kind == "latent_attention" and (lat.mixer.window, lat.mixer.rot_dims, lat.mixer.rot_base, lat.ff) == (9, 8, 100.0, 64)
    assert att.kind == "attention" and (att.mixer.temp_coef, att.mixer.temp_every, att.mixer.bias_max, att.ff) == (0.5, 5, 20.0, None)
    assert shared.mixer.kv_from == 1
    assert LuvutarConfig.from_dict(CASES["Q"][0]).streams is None
    bad = json.loads(json.dumps(CASES["P"][0]))
    bad["layers"][2]["mixer"]["kv_from"] = 3
    with pytest.raises(ConfigError):
        LuvutarConfig.from_dict(bad)
    bad = json.loads(json.dumps(CASES["P"][0]))
    bad["layers"][0]["type"] = "convolution"
    with pytest.raises(ConfigError):
        LuvutarConfig.from_dict(bad)


def test_builder_names_the_checkpoint_tensors_and_the_cache():
    from llm_infrence_engine_b200.cache.spec import PagedKVSpec
    from llm_infrence_engine_b200.engine.step import group_layout
    from llm_infrence_engine_b200.models import build_model_spec
    from llm_infrence_engine_b200.weights.loader import expected_tensors

    spec = build_model_spec(CASES["P"][0])
    names = set(expected_tensors(spec))
    assert {"embed", "head", "final.norm", "l0.mix.dq", "l0.mix.dq.norm", "l0.mix.dkv", "l0.mix.uk", "l0.mix.uv", "l0.mix.sink", "l0.mix.g",
            "l1.mix.q", "l1.mix.k", "l1.mix.v", "l1.mix.rel", "l1.mix.g", "l1.mix.o", "l2.mix.q", "l2.mix.rel", "l0.hc1.in", "l0.hc2.mix",
            "l1.hc1.out", "l0.mlp.up", "l2.mlp.down", "l0.norm2"} <= names
    assert not {"l2.mix.k", "l2.mix.v", "l1.mlp.up", "l1.norm2", "l1.hc2.in"} & names     # shared keys and values; no feed-forward
    # layer 2 reads layer 1's cache entry; latent layers keep one row per token and no value pool; windows make groups of their own
    assert [(c.layer, c.cache, c.write) for c in spec.schedule] == [(0, 0, True), (1, 1, True), (2, 1, False), (3, 2, True)]
    specs = spec.cache_specs()
    assert specs[0] == PagedKVSpec(1, 48, 9, 0) and specs[1] == PagedKVSpec(2, 16, None, 8) and specs[2] == PagedKVSpec(1, 40, 21, 0)
    groups, of_entry = group_layout(specs)
    assert len(groups) == 3 and of_entry == [0, 1, 2]
    plain_residual = build_model_spec(CASES["Q"][0])
    assert plain_residual.streams is None and not any(n.startswith("l0.hc") for n in expected_tensors(plain_residual))


def test_loader_takes_the_table_rows_from_the_checkpoint(tmp_path):
    from llm_infrence_engine_b200.models import build_model_spec
    from llm_infrence_engine_b200.weights import load_weights
    from llm_infrence_engine_b200.weights.loader import WeightsError

    folder = make_folder(tmp_path, "P")
    spec = build_model_spec(CASES["P"][0])
    load_weights(spec, folder, torch.float32, "cpu")
    att = spec.layers[1].mixer
    assert att.rel.shape == (8, 4) and spec.layers[2].mixer.rel.shape == (6, 4)
    assert att.rel_rows.tolist() == [plain.distance_bucket(n, 8, 20.0) for n in range(20)]
    assert att.w_in.shape[0] % 8 == 0 and att.w_in.shape[0] >= 4 * 16 + 2 * 16 + 2 * 8 + 4
    cfg, tensors = load_plain(folder)
    assert torch.equal(spec.layers[0].norm1.weight, 1.0 + tensors["l0.norm1"])       # stored around zero
    assert torch.equal(spec.layers[0].mixer.q_norm, tensors["l0.mix.dq.norm"])        # a plain weight
    other = json.loads(json.dumps(CASES["P"][0]))
    other["layers"][1]["mixer"]["heads"] = 8
    with pytest.raises(WeightsError):
        load_weights(build_model_spec(other), folder, torch.float32, "cpu")


def test_distance_rows():
    from llm_infrence_engine_b200.parts.attention_biased import distance_rows

    for rows, far in ((8, 20.0), (16, 100.0), (6, 9.0), (32, 512.0)):
        got = distance_rows(rows, far)
        assert got[: rows // 2] == list(range(rows // 2)) and got == sorted(got) and max(got) <= rows - 1
        assert got == [plain.distance_bucket(n, rows, far) for n in range(len(got))]
        assert plain.distance_bucket(int(far), rows, far) == rows - 1 and plain.distance_bucket(10 * int(far), rows, far) == rows - 1


def test_plain_mechanisms():
    """The plain statements against facts that hold by construction."""
    g = torch.Generator().manual_seed(0)
    x = torch.randn(6, 3, 16, generator=g, dtype=torch.float64)
    pos = torch.arange(6)
    y = plain.rotate_pairs(x, pos, 100.0, 8)
    assert torch.equal(y[..., 8:], x[..., 8:]) and torch.equal(y[0], x[0])                         # the rest passes; position 0 does not turn
    assert torch.allclose(y[..., :8].pow(2).sum(-1), x[..., :8].pow(2).sum(-1))                    # a rotation keeps lengths
    a, b = plain.rotate_pairs(x[:, 0], pos, 100.0, 8), plain.rotate_pairs(x[:, 1], pos, 100.0, 8)
    shifted = plain.rotate_pairs(x[:, 0], pos + 5, 100.0, 8), plain.rotate_pairs(x[:, 1], pos + 5, 100.0, 8)
    assert torch.allclose((a[3, :8] * b[1, :8]).sum(), (shifted[0][3, :8] * shifted[1][1, :8]).sum())   # scores see the distance only
    assert torch.allclose(plain.gelu_tanh(torch.tensor([0.0, 10.0, -10.0], dtype=torch.float64)), torch.tensor([0.0, 10.0, 0.0], dtype=torch.float64), atol=1e-9)
    assert plain.query_temperature(torch.tensor([0, 3, 4, 9]), 0.5, 5, torch.float64).tolist() == pytest.approx([1.0, 1.0, 1 + 0.5 * 0.6931471805599453, 1 + 0.5 * 1.0986122886681098])
    xs = torch.randn(3, 4, 8, generator=g, dtype=torch.float64)
    eye, one = torch.eye(3, dtype=torch.float64), torch.ones(3, dtype=torch.float64)
    out = plain.hyper_step(xs, one / 3, eye, one, lambda u: 2 * u)      # identity mix: every stream gains the same result
    assert torch.allclose(out, xs + 2 * xs.mean(0)[None])


def test_window_sink_and_shared_keys_change_what_they_should(cases):
    folder, cfg, tensors, prompts, want = cases["P"]
    p = prompts["b"]
    wide = json.loads(json.dumps(cfg))
    wide["layers"][0]["mixer"]["mask"]["size"] = 10
    wide["layers"][3]["mixer"]["mask"]["size"] = 22
    a, b = want["b"], plain_logits(wide, tensors, p)
    assert torch.allclose(a[:9], b[:9], atol=1e-12) and not torch.allclose(a[9:], b[9:], atol=1e-6)     # one key more, from position 9 on
    no_sink = {k: (v - 30.0 if k.endswith(".sink") else v) for k, v in tensors.items()}
    assert not torch.allclose(a, plain_logits(cfg, no_sink, p), atol=1e-6)
    own = {k: v for k, v in tensors.items()}
    own["l1.mix.k"] = tensors["l1.mix.k"] * 1.5                       # the layer that shares them must feel layer 1's keys
    assert not torch.allclose(a, plain_logits(cfg, own, p), atol=1e-6)


@pytest.mark.parametrize("name", list(CASES))
def test_host_side_whole_and_cut(cases, name):
    check_whole_and_cut(cases[name], name, "float32", TorchKernels(), "cpu")


@pytest.mark.parametrize("name", ["P", "Q"])
def test_host_side_mixed_batches_on_reused_pages(cases, name):
    check_mixed(cases[name], name, "float32", TorchKernels(), "cpu", seeds=(0,))


def test_host_side_long_decoding(cases):
    check_long_decoding(cases["P"], "P", "float32", TorchKernels(), "cpu", total=120)


def test_greedy_generation_through_the_engine(cases):
    """The entry point and the scheduler: several prompts at once, a small token budget (prompts are cut), few pages."""
    from llm_infrence_engine_b200.engine import Engine

    folder, cfg, tensors, prompts, want = cases["P"]
    eng = Engine(folder, dtype="float32", device="cpu", kernels=TorchKernels(), max_len=128, max_seqs=3, block_size=8, num_blocks=40,
                 max_num_batched_tokens=24)
    ps = [prompts["c"], prompts["d"], prompts["f"], prompts["b"][:30]]
    results = eng.generate(ps, max_new_tokens=10)
    for p, r in zip(ps, results):
        seq = list(p)
        for _ in range(10):
            seq.append(int(plain_logits(cfg, tensors, seq)[-1].argmax()))
        assert r.token_ids == seq[len(p):]
    eng.cache.check_invariants()
