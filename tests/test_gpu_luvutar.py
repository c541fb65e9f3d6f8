"""Luvutar on the GPU: every new kernel against its plain torch statement, and the engine (both dtypes) against the plain
implementation: whole prompts, decoding token by token, portions down to two tokens, mixed batches on reused pages, long
decoding, greedy generation through the entry point, decode steps from CUDA graphs, and inputs made so that a far key,
a window's edge or a sink shows in the result."""
import math
from types import SimpleNamespace

import pytest
import torch

from luvutar_cases import (CASES, LIMIT, check_long_decoding, check_mixed, check_whole_and_cut, cuts_of, make_folder, plain_logits, prompt,
                           replayer, row_error, run_alone, setup_case)
from torch_kernels import TorchKernels

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]
TD = {"float32": torch.float32, "bfloat16": torch.bfloat16}


@pytest.fixture(scope="module")
def K():
    from llm_infrence_engine_b200.csrc import get_kernels

    return get_kernels()


@pytest.fixture(scope="module")
def cases(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("luvutar")
    return {(name, dtype): setup_case(tmp, name, dtype) for name in CASES for dtype in DTYPES}


def close(got, want, dtype, what, scale=None):
    tol = (2e-6 if dtype == "float32" else 1.2e-2) * max(1.0, float(want.float().abs().max()) if scale is None else scale)
    err = float((got.float().cpu() - want.float().cpu()).abs().max())
    assert err <= tol, f"{what} ({dtype}): {err:.3g} > {tol:.3g}"


def rnd(*shape, seed=0, scale=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale


# ---------------------------------------------------------------------------------------------------------------------
# kernels

@pytest.mark.parametrize("S,H,N", [(1, 40, 3), (2, 48, 17), (4, 320, 9), (5, 72, 33), (9, 64, 5), (16, 24, 4)])
@pytest.mark.parametrize("dtype", DTYPES)
def test_streams_kernels(K, S, H, N, dtype):
    ref = TorchKernels()
    x = rnd(N, H, seed=1)
    xs = K.streams_expand(x.cuda(), S)
    assert torch.equal(xs.cpu(), ref.streams_expand(x, S))
    xs_ref = rnd(N, S, H, seed=2)
    xs = xs_ref.clone().cuda()
    mix, co, ci, w = torch.eye(S) + rnd(S, S, seed=3, scale=0.2), 1 + rnd(S, seed=4, scale=0.3), rnd(S, seed=5), 1 + rnd(H, seed=6, scale=0.1)
    for y_dtype in (torch.float32, TD[dtype]):
        y = rnd(N, H, seed=7).to(y_dtype)
        # update alone (carried out by flush), then the norm alone
        K.streams_update(xs, y.cuda(), mix.cuda(), co.cuda())
        K.flush()
        ref.streams_update(xs_ref, y, mix, co)
        close(xs, xs_ref, "float32", "streams_update")
        got = K.streams_norm(xs, ci.cuda(), w.cuda(), 1e-5, TD[dtype])
        close(got, ref.streams_norm(xs_ref, ci, w, 1e-5, TD[dtype]), dtype, "streams_norm")
        # update and norm in one kernel
        K.streams_update(xs, y.cuda(), mix.cuda(), co.cuda())
        got = K.streams_norm(xs, ci.cuda(), w.cuda(), 1e-5, TD[dtype])
        ref.streams_update(xs_ref, y, mix, co)
        close(xs, xs_ref, "float32", "streams_update inside the norm")
        close(got, ref.streams_norm(xs_ref, ci, w, 1e-5, TD[dtype]), dtype, "streams_norm after an update")
        # chosen rows: the update is computed for them and not stored
        rows = torch.tensor([N - 1, 0], dtype=torch.int32)
        before = xs.clone()
        K.streams_update(xs, y.cuda(), mix.cuda(), co.cuda())
        got = K.streams_norm(xs, ci.cuda(), w.cuda(), 1e-5, TD[dtype], rows.cuda())
        assert torch.equal(xs, before)
        upd = xs_ref.clone()
        ref.streams_update(upd, y, mix, co)
        close(got, ref.streams_norm(upd, ci, w, 1e-5, TD[dtype], rows), dtype, "streams_norm of rows")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("N,F,Kdim", [(5, 72, 40), (200, 136, 64)])
def test_linear_act(K, dtype, N, F, Kdim):
    x, w = rnd(N, Kdim, seed=1).to(TD[dtype]), rnd(F, Kdim, seed=2, scale=0.5).to(TD[dtype])
    got = K.linear_act(x.cuda(), w.cuda(), "gelu_tanh", TD[dtype])
    close(got, TorchKernels().linear_act(x, w, "gelu_tanh", TD[dtype]), dtype, "linear_act")
    if dtype == "bfloat16" and N <= 128:   # the small-batch product's sums were read and cleared
        assert float(K._acc.abs().max()) == 0.0


def paged(N_ctx, page, nkv, dk, dv, dtype, seed=0, shared_values=False):
    """A pool with one request of ``N_ctx`` tokens on shuffled pages; returns pools, block table and the keys/values in order."""
    pages = -(-N_ctx // page)
    perm = (torch.randperm(pages, generator=torch.Generator().manual_seed(seed)) + 1).to(torch.int32)
    k = rnd(N_ctx, nkv, dk, seed=seed + 1).to(TD[dtype])
    v = k[..., :dv] if shared_values else rnd(N_ctx, nkv, dv, seed=seed + 2).to(TD[dtype])
    k_pool = torch.zeros(pages + 2, nkv, page, dk, dtype=TD[dtype])
    v_pool = None if shared_values else torch.zeros(pages + 2, nkv, page, dv, dtype=TD[dtype])
    for t in range(N_ctx):
        k_pool[perm[t // page], :, t % page] = k[t]
        if v_pool is not None:
            v_pool[perm[t // page], :, t % page] = v[t]
    table = torch.zeros(3, pages + 1, dtype=torch.int32)
    table[1, :pages] = perm
    return k_pool, v_pool, table, k, v


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,dk,dv,shared", [(4, 2, 16, 8, False), (6, 1, 64, 64, False), (5, 1, 20, 12, True), (8, 1, 128, 96, True),
                                                 (3, 3, 24, 40, False), (2, 1, 288, 256, True), (16, 2, 32, 32, False), (14, 2, 64, 64, False),
                                                 (16, 1, 576, 512, True), (40, 1, 48, 32, True), (4, 4, 128, 128, False), (6, 2, 80, 192, False),
                                                 (7, 1, 64, 128, False), (16, 4, 128, 64, False), (70, 1, 64, 64, False)])
def test_attention_ext_every_extra(K, dtype, nq, nkv, dk, dv, shared):
    """Positions spread over a request of 1,300 tokens (two key slices), each extra alone and all together."""
    ctx_len, page = 1300, 16
    k_pool, v_pool, table, _, _ = paged(ctx_len, page, nkv, dk, dv, dtype, 3, shared)
    pos = torch.tensor([0, 1, 15, 16, 17, 100, 1023, 1024, 1025, 1299] + list(range(1180, 1299, 3)), dtype=torch.int32).sort().values
    N = pos.shape[0]
    q = rnd(N, nq * dk + 8, seed=5, scale=0.5).to(TD[dtype])
    seq = torch.ones(N, dtype=torch.int32)
    rel, sink = rnd(8, nq, seed=6), rnd(nq, seed=7)
    from llm_infrence_engine_b200.parts.attention_biased import distance_rows

    rows = torch.tensor(distance_rows(8, 40.0), dtype=torch.int32)
    gate = rnd(N, nq * dv + 3, seed=8).to(TD[dtype])
    variants = {
        "plain": {}, "window": {"window": 37}, "temperature": {"temp": (0.4, 16)}, "bias": {"rel": rel, "rel_rows": rows},
        "sink": {"sink": sink}, "gate per head": {"gate": gate, "gate_col": 3, "gate_per_head": True},
        "gate per element": {"gate": gate, "gate_col": 0}, "two equal runs": {"num_splits": 2},
        "all": {"window": 700, "temp": (0.4, 16), "rel": rel, "rel_rows": rows, "sink": sink, "gate": gate, "gate_col": 1, "gate_per_head": True},
    }
    dev = lambda t: t.cuda() if isinstance(t, torch.Tensor) else t
    # with a description of the step (here: one request that brings all ten tokens) bfloat16 sizes that fit take the tensor-core kernel
    step = SimpleNamespace(seq_lens=[N], seq_starts_dev=torch.tensor([0, N], dtype=torch.int32).cuda(), max_seq_len=N, _tables={})
    for what, kw in variants.items():
        window = kw.pop("window", 0)
        want = TorchKernels().attention_ext(q, 8, nq, nkv, dk, dv, k_pool, v_pool, table, seq, pos, page, 0.3, window, ctx_len, **kw)
        for batch in (None, step, "other tensor-core kernel"):
            if batch == "other tensor-core kernel":   # sizes that the row-block-per-warp kernel takes: the split-part kernel as well
                if not (dtype == "bfloat16" and not shared and dk in (64, 128) and dv in (64, 128)):
                    continue
                K.use_fa_attention_ext, batch = False, step
            got = K.attention_ext(q.cuda(), 8, nq, nkv, dk, dv, k_pool.cuda(), dev(v_pool), table.cuda(), seq.cuda(), pos.cuda(), page, 0.3, window,
                                  ctx_len, batch=batch, **{k: dev(v) for k, v in kw.items()})
            # (scores of ten and more, sums over up to 576 products: their exponentials carry a few 1e-7 of relative error each)
            K.use_fa_attention_ext = True
            close(got, want, dtype, f"attention_ext {what} ({'generic' if batch is None else 'with the step'})",
                  scale=8.0 * max(1.0, dk / 64) ** 0.5 if dtype == "float32" else None)


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_ext_one_key_stands_out(K, dtype):
    """One key among 1,500 is made to match the query: the result is that key's value, whether it lies far back, at a page's
    border or on the window's edge; one step outside the window it is gone. A large sink empties the result."""
    ctx_len, page, dk, dv = 1500, 16, 32, 16
    k_pool, v_pool, table, k, v = paged(ctx_len, page, 1, dk, dv, dtype, 9)
    unit = torch.zeros(dk)
    unit[5] = 1.0
    for p, j, window, seen in ((1499, 3, 0, True), (1499, 1023, 0, True), (1499, 1024, 0, True), (1400, 15, 0, True), (1400, 16, 0, True),
                               (1499, 1499 - 99, 100, True), (1499, 1499 - 100, 100, False), (1200, 1200 - 511, 512, True),
                               (1200, 1200 - 512, 512, False), (700, 700, 1, True), (700, 699, 1, False)):
        kp = k_pool.clone()
        kp[table[1, j // page], 0, j % page] = (unit * 40.0).to(TD[dtype])
        q = (unit * 4.0).to(TD[dtype])[None]
        args = (1, 1, dk, dv, kp.cuda(), v_pool.cuda(), table.cuda(), torch.ones(1, dtype=torch.int32).cuda(),
                torch.tensor([p], dtype=torch.int32).cuda(), page, 1.0, window, ctx_len)
        one = SimpleNamespace(seq_lens=[1], seq_starts_dev=torch.tensor([0, 1], dtype=torch.int32).cuda(), max_seq_len=1, _tables={})
        got = K.attention_ext(q.cuda(), 0, *args).float().cpu()[0]
        assert (K.attention_ext(q.cuda(), 0, *args, batch=one).float().cpu()[0] - got).abs().max() < 2e-2   # the tensor-core kernel in bfloat16
        if seen:
            assert (got - v[j, 0].float()).abs().max() < 2e-2, f"key {j} from position {p} (window {window}) should own the result"
        else:
            assert (got - v[j, 0].float()).abs().max() > 0.3, f"key {j} from position {p} lies outside a window of {window}"
        if seen:
            sunk = K.attention_ext(q.cuda(), 0, *args, sink=torch.tensor([400.0]).cuda()).float().cpu()[0]
            assert sunk.abs().max() < 1e-3


@pytest.mark.parametrize("dtype", DTYPES)
def test_kv_store_and_latent_kernels(K, dtype):
    ref, T = TorchKernels(), TD[dtype]
    N, page = 21, 8
    slots = (torch.randperm(40, generator=torch.Generator().manual_seed(1))[:N] + 8).to(torch.int32)
    # kv_store
    nkv, dk, dv = 2, 24, 12
    z = rnd(N, 100, seed=2).to(T)
    pools = [torch.zeros(7, nkv, page, d, dtype=T) for d in (dk, dv)]
    dev_pools = [p.clone().cuda() for p in pools]
    K.kv_store(z.cuda(), 16, 16 + nkv * dk, slots.cuda(), *dev_pools, nkv, dk, dv, page)
    ref.kv_store(z, 16, 16 + nkv * dk, slots, *pools, nkv, dk, dv, page)
    assert torch.equal(dev_pools[0].cpu(), pools[0]) and torch.equal(dev_pools[1].cpu(), pools[1])
    # latent_prepare: both norms, the turned part (partly turned, and not at all), the cache row
    for q_rank, kv_rank, rot_dim, rot_dims in ((24, 40, 8, 8), (16, 24, 16, 8), (8, 8, 4, 0)):
        z = rnd(N, q_rank + kv_rank + rot_dim + 5, seed=3).to(T)
        pos = torch.arange(N, dtype=torch.int32) * 7
        inv = 1.0 / (50.0 ** (torch.arange(0, max(rot_dims, 2), 2).float() / max(rot_dims, 2)))
        cos, sin = ref.rope_tables(pos, inv) if rot_dims else (None, None)
        wq, wkv = 1 + rnd(q_rank, seed=4, scale=0.1), 1 + rnd(kv_rank, seed=5, scale=0.1)
        pool = torch.zeros(7, 1, page, kv_rank + rot_dim, dtype=T)
        dpool = pool.clone().cuda()
        dc = lambda t: None if t is None else t.cuda()
        got = K.latent_prepare(z.cuda(), q_rank, kv_rank, rot_dim, rot_dims, wq.cuda(), wkv.cuda(), 1e-5, dc(cos), dc(sin), slots.cuda(), dpool, page)
        want = ref.latent_prepare(z, q_rank, kv_rank, rot_dim, rot_dims, wq, wkv, 1e-5, cos, sin, slots, pool, page)
        close(got, want, dtype, "latent_prepare query latent")
        close(dpool, pool, dtype, "latent_prepare cache rows")
        untouched = dpool.clone()
        K.latent_prepare(z.cuda(), q_rank, kv_rank, rot_dim, rot_dims, wq.cuda(), wkv.cuda(), 1e-5, dc(cos), dc(sin), slots.cuda(), dpool, page, write=False)
        assert torch.equal(dpool, untouched)
        # latent_absorb / latent_expand
        H, d, dvv = 3, 12, 20
        q = rnd(N, H * (d + rot_dim), seed=6).to(T)
        w_uk = rnd(H * d, kv_rank, seed=7, scale=0.3).to(T)
        close(K.latent_absorb(q.cuda(), w_uk.cuda(), dc(cos), dc(sin), H, d, rot_dim, rot_dims, kv_rank),
              ref.latent_absorb(q, w_uk, cos, sin, H, d, rot_dim, rot_dims, kv_rank), dtype, "latent_absorb")
        o_lat = rnd(N, H * kv_rank, seed=8).to(T)
        w_uv = rnd(H, kv_rank, dvv, seed=9, scale=0.3).to(T)
        gate = rnd(N, 9 + H * dvv, seed=10).to(T)
        close(K.latent_expand(o_lat.cuda(), w_uv.cuda(), gate.cuda(), 9, H, kv_rank, dvv),
              ref.latent_expand(o_lat, w_uv, gate, 9, H, kv_rank, dvv), dtype, "latent_expand")


# ---------------------------------------------------------------------------------------------------------------------
# the engine

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CASES))
def test_whole_and_cut(cases, name, dtype):
    check_whole_and_cut(cases[(name, dtype)], name, dtype, None, "cuda:0")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(CASES))
def test_mixed_batches_on_reused_pages(cases, name, dtype):
    check_mixed(cases[(name, dtype)], name, dtype, None, "cuda:0")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["P", "R"])
def test_long_decoding_and_first_tokens(cases, name, dtype):
    check_long_decoding(cases[(name, dtype)], name, dtype, None, "cuda:0")


@pytest.mark.parametrize("name", ["P", "Q"])
def test_float32_does_not_depend_on_the_cut(cases, name):
    """In float32 a token's logits have the same bits whole, in portions, and beside other requests."""
    folder, cfg, tensors, prompts, want = cases[(name, "float32")]
    rp = replayer(folder, name, "float32", 512)
    p = prompts["a"]
    whole = run_alone(rp, "w", p, [(0, len(p))])
    assert torch.equal(whole, run_alone(rp, "x", p, cuts_of(len(p), [5, 2, 31, 1, 1, 64]), 10))
    both = rp.step({"step": 99, "entries": [{"id": "y", "tokens": prompts["b"], "want": []}, {"id": "z", "tokens": p, "want": list(range(len(p)))}],
                    "end": ["y", "z"]})
    assert torch.equal(whole, both)


@pytest.mark.parametrize("dtype", DTYPES)
def test_sharp_scores_show_a_wrong_key(tmp_path, dtype):
    """Weights ten times larger make the softmax pick few keys: a key that is lost or read from a wrong page moves the logits
    by far more than rounding does. Prompt and decoding, portions that end on page borders and one off."""
    folder = make_folder(tmp_path, "P", dtype, std=0.3, seed=5)
    from luvutar_cases import load_plain

    cfg, tensors = load_plain(folder)
    p = prompt(cfg["vocab"], 140, 21)
    ref = plain_logits(cfg, tensors, p)
    rp = replayer(folder, "P", dtype, 192)
    for n, sizes in enumerate(([140], [8, 8, 1, 7, 9, 15, 16, 17], [100] + [1] * 40)):
        got = run_alone(rp, f"s{n}", p, cuts_of(140, sizes), 100 * n)
        err = row_error(got, ref)
        assert err <= (1e-4 if dtype == "float32" else 0.15), f"sharp {dtype} {sizes[:3]}: {err:.3g}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("graphs", [False, True])
def test_greedy_generation_through_the_entry_point(cases, dtype, graphs):
    from llm_infrence_engine_b200.engine import Engine

    folder, cfg, tensors, prompts, want = cases[("P", dtype)]
    eng = Engine(folder, dtype=dtype, max_len=256, max_seqs=4, block_size=8, num_blocks=70, max_num_batched_tokens=48, cuda_graphs=graphs)
    ps = [prompts["c"], prompts["d"], prompts["f"], prompts["b"], prompts["e"][:50]]
    results = eng.generate(ps, max_new_tokens=24)
    for p, r in zip(ps, results):
        seq = list(p) + r.token_ids
        ref = plain_logits(cfg, tensors, seq)[len(p) - 1:-1]
        if dtype == "float32":
            assert r.token_ids == ref.argmax(-1).tolist()
        else:   # in bfloat16 a near tie may fall the other way: the chosen token must be (nearly) the best one
            chosen = ref.gather(1, torch.tensor(r.token_ids)[:, None])[:, 0]
            assert float((ref.max(-1).values - chosen).max()) <= 0.05 * float(ref.std())
    eng.cache.check_invariants()
    assert all(pool.num_free == pool.capacity for pool in eng.cache.pools)


def test_random_weights_and_the_command_line(tmp_path):
    import json
    import subprocess
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parent.parent
    (tmp_path / "cfg.json").write_text(json.dumps(CASES["R"][0]))
    out = subprocess.run([sys.executable, "-m", "llm_infrence_engine_b200", "--model", str(tmp_path / "m"), "--random-weights", str(tmp_path / "cfg.json"),
                          "--dtype", "float32", "--prompt-ids", "1 2 3 4 5", "--max-new-tokens", "6", "--max-len", "64", "--max-seqs", "2"],
                         cwd=root, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    tokens = json.loads(out.stdout.strip().splitlines()[0])["token_ids"]
    from luvutar_cases import load_plain

    cfg, tensors = load_plain(tmp_path / "m")
    seq = [1, 2, 3, 4, 5]
    for _ in range(6):
        seq.append(int(plain_logits(cfg, tensors, seq)[-1].argmax()))
    assert tokens == seq[5:]
