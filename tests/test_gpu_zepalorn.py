"""Zepalorn on the GPU: every new kernel against its plain torch statement, and the engine (both dtypes) against the plain
implementation: whole prompts, decoding token by token, portions down to two tokens, mixed batches on reused pages and state
slots, long decoding, greedy generation through the entry point, decode steps from CUDA graphs, and inputs made so that a far
key, a kept first token, or the edge of a window or a chunk shows in the result."""
from types import SimpleNamespace

import pytest
import torch

from torch_kernels import TorchKernels
from zepalorn_cases import (CASES, check_long_decoding, check_mixed, check_whole_and_cut, cuts_of, load_plain, make_folder, plain_logits, prompt,
                            replayer, row_error, run_alone, setup_case)

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]
TD = {"float32": torch.float32, "bfloat16": torch.bfloat16}


@pytest.fixture(scope="module")
def K():
    from llm_infrence_engine_b200.csrc import get_kernels

    return get_kernels()


@pytest.fixture(scope="module")
def cases(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("zepalorn")
    return {(name, dtype): setup_case(tmp, name, dtype) for name in CASES for dtype in DTYPES}


def close(got, want, dtype, what, scale=None, f32=2e-6):
    tol = (f32 if dtype == "float32" else 1.2e-2) * max(1.0, float(want.float().abs().max()) if scale is None else scale)
    err = float((got.float().cpu() - want.float().cpu()).abs().max())
    assert err <= tol, f"{what} ({dtype}): {err:.3g} > {tol:.3g}"


def rnd(*shape, seed=0, scale=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale


def ragged(lens, slots):
    """The description of a step whose requests bring ``lens`` rows and own the state rows ``slots``."""
    starts = [0]
    for n in lens:
        starts.append(starts[-1] + n)
    host = SimpleNamespace(seq_starts_dev=torch.tensor(starts, dtype=torch.int32), seq_slots=torch.tensor(slots, dtype=torch.int32),
                           num_seqs=len(lens), max_seq_len=max(lens), seq_lens=list(lens), _tables={})
    dev = SimpleNamespace(**{**host.__dict__, "seq_starts_dev": host.seq_starts_dev.cuda(), "seq_slots": host.seq_slots.cuda(), "_tables": {}})
    return host, dev


# ---------------------------------------------------------------------------------------------------------------------
# kernels

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("N,H", [(1, 8), (5, 48), (33, 250), (200, 1024), (3, 4100)])
def test_layernorm_and_the_norm_of_a_result(K, dtype, N, H):
    ref, T = TorchKernels(), TD[dtype]
    x = rnd(N, H, seed=1) + 0.5
    w, wb = 1 + rnd(H, seed=2, scale=0.1), 1 + rnd(H, seed=3, scale=0.1)
    xd = x.clone().cuda()
    close(K.layernorm(xd, w.cuda(), 1e-5, T), ref.layernorm(x, w, 1e-5, T), dtype, "layernorm")
    rows = torch.tensor([N - 1, 0], dtype=torch.int32)
    close(K.layernorm(xd, w.cuda(), 1e-5, T, rows.cuda()), ref.layernorm(x, w, 1e-5, T, rows), dtype, "layernorm of rows")
    for y_dtype in (torch.float32, T):
        y = (rnd(N, H, seed=4, scale=3.0) + 1.0).to(y_dtype)
        # the addition alone (carried out by flush), then added and normed in one kernel
        K.post_norm_add(xd, y.clone().cuda(), wb.cuda(), 1e-5)
        K.flush()
        ref.post_norm_add(x, y, wb, 1e-5)
        close(xd, x, "float32", "post_norm_add", f32=4e-6)
        K.post_norm_add(xd, y.clone().cuda(), wb.cuda(), 1e-5)
        got = K.layernorm(xd, w.cuda(), 1e-5, T)
        ref.post_norm_add(x, y, wb, 1e-5)
        close(xd, x, "float32", "post_norm_add inside the next norm", f32=4e-6)
        close(got, ref.layernorm(x, w, 1e-5, T), dtype, "layernorm after an addition", f32=4e-6)
        # chosen rows: the addition is computed for them and not stored
        before = xd.clone()
        K.post_norm_add(xd, y.clone().cuda(), wb.cuda(), 1e-5)
        got = K.layernorm(xd, w.cuda(), 1e-5, T, rows.cuda())
        assert torch.equal(xd, before)
        added = x.clone()
        ref.post_norm_add(added, y, wb, 1e-5)
        close(got, ref.layernorm(added, w, 1e-5, T, rows), dtype, "layernorm of rows after an addition", f32=4e-6)
    # a zeroed buffer that a sublayer added into is cleared behind the read
    buf = K.zeros_like_rows(xd)
    buf += rnd(N, H, seed=5).cuda()
    K.post_norm_add(xd, buf, wb.cuda(), 1e-5)
    K.layernorm(xd, w.cuda(), 1e-5, T)
    assert float(buf.abs().max()) == 0.0


@pytest.mark.parametrize("dtype", DTYPES)
def test_group_norm_with_gate_mix_of_two_and_gated_unit(K, dtype):
    ref, T = TorchKernels(), TD[dtype]
    for N, C, gs, shared in ((7, 96, 32, False), (3, 120, 40, True), (40, 512, 512, False), (2, 66, 33, True), (5, 2048, 1024, False)):
        x = rnd(N, C, seed=1, scale=2.0)
        gate = rnd(N, C + 11, seed=2).to(T)
        w = 1 + rnd(gs if shared else C, seed=3, scale=0.2)
        for gate_first in (True, False):
            got = K.group_rmsnorm_gate(x.cuda(), gate.cuda(), 5, w.cuda(), gs, 1e-5, gate_first, T)
            close(got, ref.group_rmsnorm_gate(x, gate, 5, w, gs, 1e-5, gate_first, T), dtype, f"group_rmsnorm_gate {N}x{C}/{gs} gate first {gate_first}")
    for N, H in ((1, 16), (9, 100), (130, 768)):
        wa, wb = 1 + rnd(H, seed=4, scale=0.1), 1 + rnd(H, seed=5, scale=0.1)
        for ta in (torch.float32, T):
            for tb in (torch.float32, T):
                a, b = rnd(N, H, seed=6, scale=4.0).to(ta), rnd(N, H, seed=7, scale=0.3).to(tb)
                y, yd = rnd(N, H, seed=8), rnd(N, H, seed=8).cuda()
                K.dual_rmsnorm_mix(a.cuda(), b.cuda(), wa.cuda(), wb.cuda(), 1e-6, 0.5, yd)
                ref.dual_rmsnorm_mix(a, b, wa, wb, 1e-6, 0.5, y)
                close(yd, y, "float32", "dual_rmsnorm_mix", f32=4e-6)
    for N, I in ((1, 8), (6, 100), (150, 384)):
        gu = rnd(N, 2 * I, seed=9, scale=2.0).to(T)
        got = K.glu_clamped(gu.cuda(), 1.5, 1.702, 1.0, T)
        close(got, ref.glu_clamped(gu, 1.5, 1.702, 1.0, T), dtype, "glu_clamped")
    if dtype == "bfloat16":   # a small batch: the gated unit reads the product's float32 sums and clears them
        x, w = rnd(5, 64, seed=10).to(T), rnd(2 * 40, 64, seed=11, scale=0.3).to(T)
        got = K.glu_clamped(K.linear(x.cuda(), w.cuda(), transient=True), 1.0, 1.702, 1.0, T)
        close(got, ref.glu_clamped(x.float() @ w.float().T, 1.0, 1.702, 1.0, T), dtype, "glu_clamped on a product's sums")
        assert float(K._acc.abs().max()) == 0.0
        # prompt portions: the unit is the epilogue of the tcgen05 gate/up product (one block per tile, and pairs of blocks from 1,024 rows on)
        for M, I, Kd in ((130, 40, 64), (300, 264, 96), (1100, 520, 128), (2048, 96, 256)):
            x, w = rnd(M, Kd, seed=12).to(T), rnd(2 * I, Kd, seed=13, scale=0.3).to(T)
            got = K.gate_up_act(x.cuda(), w.cuda(), T, glu=(1.25, 1.702, 1.0))
            close(got, ref.gate_up_act(x, w, T, glu=(1.25, 1.702, 1.0)), dtype, f"clamped unit as the product's epilogue, {M} rows")
        K.check_device_errors()
        # the second half of a low-rank projection reads its input where it lies, as a run of columns of wider rows
        z, w2 = rnd(200, 64, seed=14).to(T), rnd(48, 24, seed=15).to(T)
        close(K.linear(z.cuda()[:, 16:40], w2.cuda(), out_dtype=T), z[:, 16:40].float() @ w2.float().T, dtype, "linear on a run of columns")
        close(K.linear(z.cuda()[:3, 16:40], w2.cuda(), out_dtype=T), z[:3, 16:40].float() @ w2.float().T, dtype, "linear on a run of columns, few rows")
    else:
        z, w2 = rnd(20, 64, seed=14), rnd(48, 24, seed=15)
        close(K.linear(z.cuda()[:, 16:40], w2.cuda()), z[:, 16:40] @ w2.T, dtype, "linear on a run of columns", f32=4e-6)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,dk,dv,dims,inter,norm", [(4, 2, 16, 8, 16, False, False), (6, 2, 24, 16, 16, False, False), (4, 1, 32, 32, 32, True, True),
                                                          (3, 3, 64, 40, 8, True, True), (2, 1, 96, 96, 96, False, True), (5, 5, 20, 12, 0, False, True),
                                                          (8, 2, 128, 64, 64, True, False)])
def test_heads_normed_turned_and_stored(K, dtype, nq, nkv, dk, dv, dims, inter, norm):
    ref, T = TorchKernels(), TD[dtype]
    N, page = 19, 8
    slots = (torch.randperm(40, generator=torch.Generator().manual_seed(1))[:N] + 8).to(torch.int32)
    z = rnd(N, (nq + nkv) * dk + nkv * dv + 5, seed=2).to(T)
    pos = torch.arange(N, dtype=torch.int32) * 37
    cos = sin = None
    if dims:
        inv = 1.0 / (50.0 ** (torch.arange(0, dims, 2).float() / dims))
        cos, sin = ref.rope_tables(pos, inv, 1.13)
        gc, gs_ = K.rope_tables(pos.cuda(), inv.cuda(), 1.13)
        close(gc, cos, "float32", "rope_tables with a magnitude")
    qw, kw = (1 + rnd(dk, seed=3, scale=0.2), 1 + rnd(dk, seed=4, scale=0.2)) if norm else (None, None)
    pools = [torch.zeros(7, nkv, page, d, dtype=T) for d in (dk, dv)]
    dpools = [p.clone().cuda() for p in pools]
    dc = lambda t: None if t is None else t.cuda()
    got = K.qk_norm_rope_store(z.cuda(), nq, nkv, dk, dv, dc(qw), dc(kw), 1e-5, dc(cos), dc(sin), dims, inter, slots.cuda(), *dpools, page)
    want = ref.qk_norm_rope_store(z, nq, nkv, dk, dv, qw, kw, 1e-5, cos, sin, dims, inter, slots, *pools, page)
    close(got, want, dtype, "queries", f32=4e-6)
    close(dpools[0], pools[0], dtype, "keys in their pages", f32=4e-6)
    assert torch.equal(dpools[1].cpu(), pools[1])
    untouched = [p.clone() for p in dpools]
    K.qk_norm_rope_store(z.cuda(), nq, nkv, dk, dv, dc(qw), dc(kw), 1e-5, dc(cos), dc(sin), dims, inter, slots.cuda(), *dpools, page, write_kv=False)
    assert torch.equal(dpools[0], untouched[0]) and torch.equal(dpools[1], untouched[1])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("C,taps,bias,act", [(10, 2, False, None), (200, 4, True, "silu"), (384, 3, True, "silu"), (33, 8, False, "silu")])
def test_short_convolution_over_ragged_steps(K, dtype, C, taps, bias, act):
    """Three requests in three steps: long portions, portions shorter than the taps, single tokens; the state row of a request
    carries its last inputs from step to step."""
    ref, T = TorchKernels(), TD[dtype]
    w, b = rnd(C, taps, seed=1, scale=0.5), (rnd(C, seed=2) if bias else None)
    state = rnd(5, taps - 1, C, seed=3)
    dstate = state.clone().cuda()
    for step, lens in enumerate(([70, 1, 2], [1, 1, 1], [3, 40, 1], [2, 2, 129])):
        host, dev = ragged(lens, [3, 0, 4])
        z = rnd(sum(lens), C + 9, seed=10 + step).to(T)
        got = K.causal_conv(z.cuda(), 4, C, w.cuda(), None if b is None else b.cuda(), dstate, dev, act)
        want = ref.causal_conv(z, 4, C, w, b, state, host, act)
        close(got, want, dtype, f"causal_conv step {step}", f32=4e-6)
        assert torch.equal(dstate.cpu(), state), "the convolution's state is a copy of inputs"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,D,DV", [(4, 2, 16, 24), (3, 3, 8, 40), (6, 2, 40, 33), (2, 1, 128, 128), (2, 2, 64, 32), (1, 1, 200, 16)])
def test_delta_rule_over_ragged_steps(K, dtype, H, G, D, DV):
    ref, T = TorchKernels(), TD[dtype]
    state = torch.zeros(4, H, DV, D)
    dstate = state.clone().cuda()
    A_log, dt_bias = torch.log(0.5 + rnd(H, seed=1).abs()), rnd(H * D, seed=2) - 2.0
    for step, lens in enumerate(([37, 1, 5], [1, 1, 1], [2, 19, 1])):
        host, dev = ragged(lens, [2, 0, 1])
        N = sum(lens)
        qkv = rnd(N, 2 * G * D + H * DV + 3, seed=20 + step).to(T)
        a, b = rnd(N, H * D, seed=30 + step).to(T), rnd(N, H + 6, seed=40 + step, scale=2.0).to(T)
        got = K.delta_rule(qkv.cuda(), H, G, D, DV, a.cuda(), b.cuda(), 5, A_log.cuda(), dt_bias.cuda(), dstate, dev)
        want = ref.delta_rule(qkv, H, G, D, DV, a, b, 5, A_log, dt_bias, state, host)
        close(got, want, "float32", f"delta_rule step {step}", f32=2e-5)
        close(dstate, state, "float32", f"delta_rule state after step {step}", f32=2e-5)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,NS,DV", [(4, 1, 16, 12), (6, 2, 8, 16), (2, 2, 40, 20), (8, 1, 128, 64), (3, 3, 64, 33)])
def test_state_space_scan_over_ragged_steps(K, dtype, H, G, NS, DV):
    ref, T = TorchKernels(), TD[dtype]
    state = torch.zeros(4, H, DV, NS)
    dstate = state.clone().cuda()
    A_log, dt_bias, skip = torch.log(0.5 + rnd(H, seed=1).abs()), rnd(H, seed=2) - 1.0, 1 + rnd(H, seed=3, scale=0.2)
    for step, lens in enumerate(([41, 1, 3], [1, 1, 1], [2, 23, 1])):
        host, dev = ragged(lens, [3, 1, 0])
        N = sum(lens)
        xbc = rnd(N, H * DV + 2 * G * NS, seed=20 + step).to(T)
        dt = rnd(N, H + 7, seed=30 + step).to(T)
        got = K.ssm_scan(xbc.cuda(), H, G, NS, DV, dt.cuda(), 7, A_log.cuda(), dt_bias.cuda(), skip.cuda(), dstate, dev)
        want = ref.ssm_scan(xbc, H, G, NS, DV, dt, 7, A_log, dt_bias, skip, state, host)
        close(got, want, "float32", f"ssm_scan step {step}", scale=max(1.0, float(want.abs().max())), f32=1e-5)
        close(dstate, state, "float32", f"ssm_scan state after step {step}", f32=1e-5)


def paged(N_ctx, page, nkv, dk, dv, dtype, seed=0):
    """A pool with one request of ``N_ctx`` tokens on shuffled pages; returns pools, block table and the keys/values in order."""
    pages = -(-N_ctx // page)
    perm = (torch.randperm(pages, generator=torch.Generator().manual_seed(seed)) + 1).to(torch.int32)
    k, v = rnd(N_ctx, nkv, dk, seed=seed + 1).to(TD[dtype]), rnd(N_ctx, nkv, dv, seed=seed + 2).to(TD[dtype])
    k_pool, v_pool = torch.zeros(pages + 2, nkv, page, dk, dtype=TD[dtype]), torch.zeros(pages + 2, nkv, page, dv, dtype=TD[dtype])
    for t in range(N_ctx):
        k_pool[perm[t // page], :, t % page] = k[t]
        v_pool[perm[t // page], :, t % page] = v[t]
    table = torch.zeros(3, pages + 1, dtype=torch.int32)
    table[1, :pages] = perm
    return k_pool, v_pool, table, k, v


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,dk,dv", [(4, 2, 16, 8), (6, 1, 64, 64), (4, 2, 96, 96), (3, 3, 24, 40), (4, 4, 128, 128), (16, 4, 128, 64), (2, 1, 48, 32)])
def test_attention_masks_and_soft_cap(K, dtype, nq, nkv, dk, dv):
    """Positions spread over a request of 1,300 tokens, as a prompt portion and as single tokens; every kernel that takes the sizes."""
    ctx_len, page = 1300, 16
    k_pool, v_pool, table, _, _ = paged(ctx_len, page, nkv, dk, dv, dtype, 3)
    pos = torch.tensor([0, 1, 5, 6, 15, 16, 17, 100, 199, 200, 201, 1023, 1024, 1025, 1299] + list(range(1180, 1299, 3)), dtype=torch.int32).sort().values
    N = pos.shape[0]
    q = rnd(N, nq * dk + 8, seed=5, scale=0.5).to(TD[dtype])
    seq = torch.ones(N, dtype=torch.int32)
    variants = {"window with kept tokens": dict(window=136, keep_first=6), "short window, many kept": dict(window=9, keep_first=70),
                "kept tokens inside the window": dict(window=700, keep_first=3), "chunks": dict(chunk=200), "chunks of a page": dict(chunk=16),
                "soft cap": dict(softcap=1.5), "chunks and cap": dict(chunk=333, softcap=0.7), "window, kept, cap": dict(window=64, keep_first=64, softcap=2.0)}
    portion = SimpleNamespace(seq_lens=[N], seq_starts_dev=torch.tensor([0, N], dtype=torch.int32).cuda(), max_seq_len=N, _tables={})
    for what, kw in variants.items():
        kw = dict(kw)
        window = kw.pop("window", 0)
        want = TorchKernels().attention_ext(q, 8, nq, nkv, dk, dv, k_pool, v_pool, table, seq, pos, page, 0.3, window, ctx_len, **kw)
        for how in ("generic", "portion", "portion, split-part kernel", "single tokens", "two equal runs"):
            batch, more = None, {}
            if how.startswith("portion"):
                batch = portion
            if how == "single tokens":
                batch = SimpleNamespace(seq_lens=[1] * N, seq_starts_dev=torch.arange(N + 1, dtype=torch.int32).cuda(), max_seq_len=1, _tables={})
            if how == "two equal runs":
                batch, more = portion, {"num_splits": 2}
            K.use_fa_attention_ext = how != "portion, split-part kernel"
            try:
                got = K.attention_ext(q.cuda(), 8, nq, nkv, dk, dv, k_pool.cuda(), v_pool.cuda(), table.cuda(), seq.cuda(), pos.cuda(), page, 0.3, window,
                                      ctx_len, batch=batch, **kw, **more)
            finally:
                K.use_fa_attention_ext = True
            close(got, want, dtype, f"attention_ext {what} ({how})", scale=8.0 * max(1.0, dk / 64) ** 0.5 if dtype == "float32" else None)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("dk,dv", [(32, 16), (64, 64), (96, 96)])
def test_one_key_stands_out_at_every_edge(K, dtype, dk, dv):
    """One key among 1,500 is made to match the query: the result is that key's value when the key is seen (far back among the
    kept first tokens, at a page's border, on the inner edge of a window or a chunk) and something else when it is one step
    outside; for a single token and inside a prompt portion, on every kernel that takes the sizes."""
    ctx_len, page = 1500, 16
    k_pool, v_pool, table, k, v = paged(ctx_len, page, 1, dk, dv, dtype, 9)
    unit = torch.zeros(dk)
    unit[5] = 1.0
    cases_ = [  # position, key, mask, seen
        (1499, 1499 - 135, dict(window=136, keep_first=6), True), (1499, 1499 - 136, dict(window=136, keep_first=6), False),
        (1499, 5, dict(window=136, keep_first=6), True), (1499, 6, dict(window=136, keep_first=6), False), (1499, 0, dict(window=136, keep_first=6), True),
        (141, 5, dict(window=136, keep_first=6), True), (141, 6, dict(window=136, keep_first=6), True), (142, 6, dict(window=136, keep_first=6), False),
        (900, 15, dict(window=20, keep_first=17), True), (900, 16, dict(window=20, keep_first=17), True), (900, 17, dict(window=20, keep_first=17), False),
        (1399, 1200, dict(chunk=200), True), (1399, 1199, dict(chunk=200), False), (1400, 1399, dict(chunk=200), False), (1400, 1400, dict(chunk=200), True),
        (1023, 1008, dict(chunk=16), True), (1023, 1007, dict(chunk=16), False), (1024, 1023, dict(chunk=16), False),
        (700, 3, dict(), True), (1499, 1024, dict(), True),
    ]
    for p, j, mask, seen in cases_:
        mask = dict(mask)
        window = mask.pop("window", 0)
        kp = k_pool.clone()
        kp[table[1, j // page], 0, j % page] = (unit * 40.0).to(TD[dtype])
        # a portion of 24 tokens that ends at p: the row of p is the one that is looked at; and p as a single token
        first = max(0, p - 23)
        rows = p - first + 1
        q = (unit * 4.0).to(TD[dtype])[None].repeat(rows, 1)
        pos = torch.arange(first, p + 1, dtype=torch.int32)
        common = (1, 1, dk, dv, kp.cuda(), v_pool.cuda(), table.cuda())
        for how in ("generic", "portion", "portion, split-part kernel", "single"):
            if how == "single":
                batch = SimpleNamespace(seq_lens=[1], seq_starts_dev=torch.tensor([0, 1], dtype=torch.int32).cuda(), max_seq_len=1, _tables={})
                qq, pp = q[-1:], pos[-1:]
            else:
                batch = None if how == "generic" else SimpleNamespace(seq_lens=[rows], seq_starts_dev=torch.tensor([0, rows], dtype=torch.int32).cuda(),
                                                                      max_seq_len=rows, _tables={})
                qq, pp = q, pos
            K.use_fa_attention_ext = how != "portion, split-part kernel"
            try:
                got = K.attention_ext(qq.cuda(), 0, *common, torch.ones(pp.shape[0], dtype=torch.int32).cuda(), pp.cuda(), page, 1.0, window, ctx_len,
                                      batch=batch, **mask).float().cpu()[-1]
            finally:
                K.use_fa_attention_ext = True
            d = float((got - v[j, 0].float()).abs().max())
            if seen:
                assert d < 2e-2, f"key {j} from position {p} ({window}, {mask}; {how}) should own the result: {d:.3g}"
            else:
                assert d > 0.3, f"key {j} from position {p} ({window}, {mask}; {how}) must not be seen"


# ---------------------------------------------------------------------------------------------------------------------
# the engine

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(CASES))
def test_engine_whole_and_cut(cases, name, dtype):
    check_whole_and_cut(cases[(name, dtype)], name, dtype, None, "cuda:0")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(CASES))
def test_engine_mixed_batches_on_reused_pages_and_slots(cases, name, dtype):
    check_mixed(cases[(name, dtype)], name, dtype, None, "cuda:0")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(CASES))
def test_engine_long_decoding(cases, name, dtype):
    check_long_decoding(cases[(name, dtype)], name, dtype, None, "cuda:0")


@pytest.mark.parametrize("name", sorted(CASES))
def test_float32_does_not_depend_on_how_the_work_is_cut(cases, name):
    """In float32 the recurrences walk their rows in one order, the products and norms treat a row by itself and the attention
    cuts its keys at fixed places: the same bits whole, in portions, and one by one."""
    folder, cfg, tensors, prompts, want = cases[(name, "float32")]
    rp = replayer(folder, name, "float32", 192)
    p = prompts["e"]
    T = len(p)
    whole = run_alone(rp, "w", p, [(0, T)])
    for n, sizes in enumerate(([7, 2, 33, 1, 16, 3, 2, 64, 5], [T - 30] + [1] * 30, [2])):
        got = run_alone(rp, f"c{n}", p, cuts_of(T, sizes), 1000 * (n + 1))
        assert torch.equal(got, whole), f"{name}: portions of {sizes[:3]} differ by {float((got - whole).abs().max()):.3g}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_sharp_scores_show_a_wrong_key(tmp_path, name, dtype):
    """Query projections eight times larger make the softmax pick few keys: a key that is lost, read from a wrong page, or seen
    across the edge of a window or chunk moves the logits by far more than rounding does. Prompt and decoding, portions that end
    on page borders and one off, single tokens across the edges."""
    folder = make_folder(tmp_path, name, dtype, sharp=8.0, seed=5)
    cfg, tensors = load_plain(folder)
    p = prompt(cfg["vocab"], 140, 21)
    ref = plain_logits(cfg, tensors, p)
    rp = replayer(folder, name, dtype, 192)
    for n, sizes in enumerate(([140], [8, 8, 1, 7, 9, 15, 16, 17], [100] + [1] * 40, [15] + [1] * 125)):
        got = run_alone(rp, f"s{n}", p, cuts_of(140, sizes), 1000 * n)
        err = row_error(got, ref)
        # (float32 is the sharp detector here; in bfloat16 the peaked softmax also magnifies the rounding of q and k, measured up to 0.2)
        assert err <= (1e-4 if dtype == "float32" else 0.3), f"sharp {name} {dtype} {sizes[:3]}: {err:.3g}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("graphs", [False, True])
def test_greedy_generation_through_the_entry_point(cases, dtype, graphs):
    from llm_infrence_engine_b200.engine import Engine

    folder, cfg, tensors, prompts, want = cases[("A", dtype)]
    eng = Engine(folder, dtype=dtype, max_len=256, max_seqs=4, block_size=8, num_blocks=70, max_num_batched_tokens=48, cuda_graphs=graphs)
    if graphs:
        assert eng.runner.graphs.usable, "every part of the model only launches kernels: its decode steps are captured"
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


def test_preemption_recomputes_the_state(cases):
    """A pool too small for all requests: the youngest is preempted and later recomputed from its first token, its state rows
    starting from zero again. Same tokens as with room for all."""
    from llm_infrence_engine_b200.engine import Engine

    folder, cfg, tensors, prompts, want = cases[("B", "float32")]
    ps = [prompts["b"], prompts["c"], prompts["a"][:60], prompts["e"][:70]]
    big = Engine(folder, dtype="float32", max_len=160, max_seqs=4, block_size=16, num_blocks=60, max_num_batched_tokens=64)
    want_tokens = [r.token_ids for r in big.generate(ps, max_new_tokens=40)]
    small = Engine(folder, dtype="float32", max_len=160, max_seqs=4, block_size=16, num_blocks=19, max_num_batched_tokens=64)
    got = [r.token_ids for r in small.generate(ps, max_new_tokens=40)]
    assert small.preemptions > 0 and got == want_tokens
    small.cache.check_invariants()


def test_random_weights_and_the_command_line(tmp_path):
    import json
    import subprocess
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parent.parent
    (tmp_path / "cfg.json").write_text(json.dumps(CASES["C"][0]))
    out = subprocess.run([sys.executable, "-m", "llm_infrence_engine_b200", "--model", str(tmp_path / "m"), "--random-weights", str(tmp_path / "cfg.json"),
                          "--dtype", "float32", "--prompt-ids", "1 2 3 4 5", "--max-new-tokens", "6", "--max-len", "64", "--max-seqs", "2"],
                         cwd=root, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    tokens = json.loads(out.stdout.strip().splitlines()[0])["token_ids"]
    cfg, tensors = load_plain(tmp_path / "m")
    seq = [1, 2, 3, 4, 5]
    for t in tokens:
        assert t == int(plain_logits(cfg, tensors, seq)[-1].argmax())
        seq.append(t)
