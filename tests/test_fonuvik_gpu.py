"""The Fonuvik decoder on the GPU against its plain float64 restatement: each mechanism alone, then whole models cut in
every way (whole prompts, a tail decoded token by token, portions down to two tokens, mixed batches over a pool so small
that pages and state slots are used again), in true fp32 and in bf16, and greedy generation through the scheduler."""
import math
from types import SimpleNamespace

import pytest
import torch

from tests.fonuvik_cases import CASES, case, write_folder
from tests.helpers import collect, random_tokens, steps_mixed, steps_portions, steps_prefill_then_decode, steps_whole
from tests.plain import fonuvik_plain as plain

pytestmark = pytest.mark.gpu

FP32_TOL = 3e-5          # of the largest |logit|
BF16_TOL = 0.05          # of the largest |logit|
DEV = "cuda:0"
LENGTHS = {"a": [1, 2, 37, 130], "b": [5, 64, 99], "c": [3, 50, 290], "d": [17, 80], "e": [9, 120], "f": [2, 200]}


def tol(dtype):
    return FP32_TOL if dtype == "float32" else BF16_TOL


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for key in CASES:
        raw, weights = case(key)
        out[key] = (write_folder(str(tmp_path_factory.mktemp("fonuvik_" + key)), raw, weights), raw, weights)
    return out


def engine_for(folder, dtype, max_tokens=1024, page_size=16, max_requests=4):
    from microllm_rocm_b200.engine.loading import load_engine
    return load_engine(folder, dtype=dtype, page_size=page_size, max_tokens=max_tokens, max_requests=max_requests)


_plain = {}


def plain_logits(raw, weights, tokens):
    k = (id(weights), tuple(tokens))
    if k not in _plain:
        _plain[k] = plain.forward(raw, weights, list(tokens)).float()
    return _plain[k]


def compare(got, key, raw, weights, requests, dtype, share=0.1):
    """fp32: every position within the tolerance.  bf16 rounds the router's input (and the weights): where two experts' logits
    are a rounding error apart the choice flips, that position lands far off, and the recurrences' states carry a little of it
    to every later position of the request (the plain implementation does the same between fp32 weights and their bf16
    roundings).  So bf16 is held, over all positions of a case, to a small median error and to at most `share` of them over
    the tolerance."""
    errs = []
    for rid, toks in requests.items():
        ref = plain_logits(raw, weights, toks)
        rows = torch.stack([got[(rid, p)] for p in range(len(toks))])
        assert torch.isfinite(rows).all(), f"case {key} request {rid}: logits that are not finite"
        err = (rows - ref).abs().amax(dim=1) / ref.abs().max()
        if dtype == "float32" and bool((err > tol(dtype)).any()):
            pos = int((err > tol(dtype)).nonzero()[0])
            raise AssertionError(f"case {key} request {rid}: position {pos} of {len(toks)} is over the tolerance {tol(dtype)} "
                                 f"(error {float(err[pos]):.3e} of the largest |logit|)")
        errs.append(err)
    err = torch.cat(errs)
    over = int((err > tol(dtype)).sum())
    if dtype != "float32":
        assert over <= max(2, int(share * err.numel())) and float(err.median()) <= 0.4 * tol(dtype), \
            f"case {key}: {over} of {err.numel()} positions over the tolerance {tol(dtype)}, median error {float(err.median()):.3e}"
    print(f"[fonuvik parity] case {key} {dtype}: median error {float(err.median()):.3e}, worst {float(err.max()):.3e} of the largest |logit|, {over} over")
    return float(err.median())


def requests_for(raw, lengths, seed=0):
    return {f"r{i}": random_tokens(n, raw["vocab"], seed + 100 * i + n) for i, n in enumerate(lengths)}


def step_of(lengths, pos0, slots):
    """The per-sequence arrays a kernel sees of a step whose sequences bring `lengths` tokens from positions `pos0`."""
    starts = [0]
    for n in lengths:
        starts.append(starts[-1] + n)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    return SimpleNamespace(
        seq_starts=i32(starts), seq_pos0=i32(pos0), num_seqs=len(lengths), error_flag=torch.zeros(1, dtype=torch.int32, device=DEV),
        token_seq=i32([a for a, n in enumerate(lengths) for _ in range(n)]),
        positions=i32([p + i for p, n in zip(pos0, lengths) for i in range(n)])), i32(slots)


def scatter(got, out, spans):
    at = 0
    for i, (a, b) in enumerate(spans):
        got[i][a:b] = out[at:at + b - a]
        at += b - a


# ------------------------------------------------------------------------------------------- mechanisms alone
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_a_sum_normed_before_it_is_added_and_the_next_norm(out_dtype):
    from microllm_rocm_b200.kernels import ops
    torch.manual_seed(1)
    for width in (40, 257, 1024, 5000):
        x = torch.randn(9, width, device=DEV) * 3 + 1
        wp, wn = 1 + 0.3 * torch.randn(width, device=DEV), 1 + 0.3 * torch.randn(width, device=DEV)
        d1, d2 = torch.randn(3, 9, width, device=DEV), torch.randn(9, width, device=DEV) * 5          # three partial sums; one plain term
        stream, copy = x.clone(), torch.empty(9, width, dtype=out_dtype, device=DEV)
        ops.normed_add_rmsnorm(stream, [(0.7, d1), (1.3, d2)], wp, 1e-5, next_weight=wn, out=copy)
        d = 0.7 * d1.double().sum(0) + 1.3 * d2.double()
        want = x.double() + plain.rms(d, 1e-5) * wp.double()
        assert torch.allclose(stream.double(), want, atol=2e-5)
        assert torch.allclose(copy.double(), plain.rms(want, 1e-5) * wn.double(), atol=1e-5 if out_dtype == torch.float32 else 0.05)
        one = x.clone()
        ops.normed_add_rmsnorm(one, [(1.0, d2)], wp, 1e-5)                      # one term, nothing behind it
        assert torch.allclose(one.double(), x.double() + plain.rms(d2.double(), 1e-5) * wp.double(), atol=2e-5)
        # the norm of the sum is not the sum's scale: a term ten times as large adds the same
        again = x.clone()
        ops.normed_add_rmsnorm(again, [(10.0, d2)], wp, 1e-5)
        assert torch.allclose(again, one, atol=1e-4)


@pytest.mark.parametrize("table_dtype", [torch.float32, torch.bfloat16])
def test_normed_embedding(table_dtype):
    from microllm_rocm_b200.parts.base import EMBEDDINGS, Runtime
    torch.manual_seed(2)
    part = EMBEDDINGS["token_embedding"](dict(name="embed", vocab_size=50, hidden_size=24, norm=("embed.norm", 1e-3)), Runtime(torch.device(DEV), table_dtype))
    assert set(part.weight_specs()) == {"embed", "embed.norm"}
    table, w = (torch.randn(50, 24, device=DEV) * 0.01).to(table_dtype), 1 + 0.2 * torch.randn(24, device=DEV)
    part.bind({"embed": table, "embed.norm": w})
    ids = torch.tensor([3, 49, 0, 7, 7], dtype=torch.int32, device=DEV)
    got = part.forward(ids)
    want = plain.rms(table.double()[ids.long()], 1e-3) * w.double()               # small rows: eps matters
    assert got.dtype == torch.float32 and torch.allclose(got.double(), want, atol=1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width", [20, 64, 200])
def test_token_shift_over_steps_with_slots_used_again(dtype, width):
    """Three sequences through three steps of unequal portions (also single tokens), the previous input in slots that held
    another sequence before; against the shift of each whole sequence."""
    from microllm_rocm_b200.kernels import linear_attention
    torch.manual_seed(width)
    mu = torch.rand(5, width, device=DEV)
    seqs = [torch.randn(n, width, device=DEV).to(dtype) for n in (19, 5, 11)]
    state = torch.full((4, width), 777.0, device=DEV)                            # what an earlier request left in the slots
    cuts = [[(0, 7), (7, 8), (8, 19)], [(0, 1), (1, 3), (3, 5)], [(0, 2), (2, 9), (9, 11)]]
    got = [torch.empty(5, len(s), width, dtype=dtype, device=DEV) for s in seqs]
    for step in range(3):
        spans = [c[step] for c in cuts]
        ctx, slots = step_of([b - a for a, b in spans], [a for a, _ in spans], [2, 0, 3])
        x = torch.cat([s[a:b] for s, (a, b) in zip(seqs, spans)]).contiguous()
        out = torch.empty(5, x.shape[0], width, dtype=dtype, device=DEV)
        linear_attention.token_shift(x, mu, state, slots, ctx, out)
        assert int(ctx.error_flag.item()) == 0
        at = 0
        for i, (a, b) in enumerate(spans):
            got[i][:, a:b] = out[:, at:at + b - a]
            at += b - a
    assert float(state[1].min()) == 777.0                                        # a slot no sequence holds stays as it was
    for s, g in zip(seqs, got):
        h = s.double().cpu()
        back = plain.shifted(h) - h
        for j in range(5):
            want = h + back * mu[j].double().cpu()
            assert torch.allclose(g[j].double().cpu(), want, atol=1e-5 if dtype == torch.float32 else 0.03), j


@pytest.mark.parametrize("form", ["sigmoid_root", "double_exp"])
def test_decays_from_a_two_step_projection(form):
    """q * scale, k, v taken out of partial sums, and the decay, with the second step made in the kernel (any inner width)
    or ready-made by a product; extreme pre-activations stay finite and inside [0, 1]."""
    from microllm_rocm_b200.kernels import linear_attention
    torch.manual_seed(3)
    T, HK, HV, rank, tau = 13, 24, 20, 5, 7.0
    src = torch.randn(2, T, 2 * HK + HV + rank, device=DEV)
    src[:, 0, 2 * HK + HV:] *= 40.0                                              # one token with a huge pre-activation
    w2, bias = torch.randn(HK, rank, device=DEV), torch.randn(HK, device=DEV)
    act = "tanh" if form == "double_exp" else None
    full = src.double().sum(0).cpu()
    a = full[:, 2 * HK + HV:]
    z = (torch.tanh(a) if act else a) @ w2.double().cpu().T + bias.double().cpu()
    want = torch.exp(torch.nn.functional.logsigmoid(z) / tau) if form == "sigmoid_root" else torch.exp(-torch.exp(z))
    for ready in (False, True):
        q, k, decay = (torch.empty(T, HK, device=DEV) for _ in range(3))
        v = torch.empty(T, HV, device=DEV)
        more = dict(pre=(z - bias.double().cpu()).float().to(DEV)) if ready else dict(narrow=src, a_col=2 * HK + HV, w2=w2, narrow_act=act)
        linear_attention.decay_prepare(src, 0, src, HK, src, 2 * HK, 0.25, bias=bias, form=form, tau=tau, q_out=q, k_out=k, v_out=v,
                                       decay=decay, **more)
        assert torch.allclose(q.double().cpu(), full[:, :HK] * 0.25, atol=1e-6) and torch.allclose(k.double().cpu(), full[:, HK:2 * HK], atol=1e-6)
        assert torch.allclose(v.double().cpu(), full[:, 2 * HK:2 * HK + HV], atol=1e-6)
        assert torch.isfinite(decay).all() and float(decay.min()) >= 0.0 and float(decay.max()) <= 1.0
        assert torch.allclose(decay.double().cpu(), want, atol=2e-6), float((decay.double().cpu() - want).abs().max())
    assert float(want.min()) < 0.01 < 0.9 < float(want.max())                     # both ends of the range are in the test


@pytest.mark.parametrize("rule", ["decayed_sum", "bonus_read"])
@pytest.mark.parametrize("heads, dk, dv", [(3, 8, 12), (2, 20, 10), (2, 64, 64), (1, 136, 40), (5, 16, 16), (2, 24, 200)])
def test_recurrences_over_steps(rule, heads, dk, dv):
    """The scan over three steps of unequal portions, two sequences, state slots that held something else before; against
    the plain recurrence over each whole sequence.  The two rules differ in when the read-out happens, so each is also
    held against the other's result."""
    from microllm_rocm_b200.kernels import recurrent
    torch.manual_seed(dk + dv)
    lengths = [29, 6]
    q = [torch.randn(n, heads * dk, device=DEV) for n in lengths]
    k = [torch.randn(n, heads * dk, device=DEV) for n in lengths]
    a = [torch.rand(n, heads * dk, device=DEV) for n in lengths]
    v = [torch.randn(n, heads * dv, device=DEV) for n in lengths]
    u = torch.randn(heads, dk, device=DEV)
    state = torch.full((3, heads, dk, dv), 55.0, device=DEV)
    cuts = [[(0, 11), (11, 12), (12, 29)], [(0, 2), (2, 4), (4, 6)]]
    got = [torch.empty(n, heads * dv, device=DEV) for n in lengths]
    for step in range(3):
        spans = [c[step] for c in cuts]
        ctx, slots = step_of([b - a_ for a_, b in spans], [a_ for a_, _ in spans], [2, 1])
        cat = lambda xs: torch.cat([x[s:e] for x, (s, e) in zip(xs, spans)]).contiguous()
        o = torch.empty(sum(e - s for s, e in spans), heads * dv, device=DEV)
        recurrent.linear_scan(rule, cat(q), cat(k), cat(a), cat(v), o, state, slots, ctx, heads, dk, dv, bonus=u if rule == "bonus_read" else None)
        assert int(ctx.error_flag.item()) == 0
        scatter(got, o, spans)
    assert float(state[0].min()) == 55.0
    for i, n in enumerate(lengths):
        view = lambda x, d: x[i].double().cpu().view(n, heads, d)
        if rule == "decayed_sum":
            want, S = plain.decayed_sum(view(q, dk), view(k, dk), view(v, dv), view(a, dk))
            other, _ = plain.bonus_sum(view(q, dk), view(k, dk), view(v, dv), view(a, dk), u.double().cpu())
        else:
            want, S = plain.bonus_sum(view(q, dk), view(k, dk), view(v, dv), view(a, dk), u.double().cpu())
            other, _ = plain.decayed_sum(view(q, dk), view(k, dk), view(v, dv), view(a, dk))
        err = float((got[i].double().cpu() - want.reshape(n, -1)).abs().max())
        assert err < 2e-4 * max(1.0, float(want.abs().max())), err
        assert float((want - other).abs().max()) > 0.1
        assert torch.allclose(state[[2, 1][i]].double().cpu(), S, atol=2e-4 * max(1.0, float(S.abs().max())))


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_head_norm_with_a_shared_or_a_whole_weight_and_a_gate(out_dtype):
    from microllm_rocm_b200.kernels import linear_attention
    torch.manual_seed(4)
    atol = 1e-5 if out_dtype == torch.float32 else 0.05
    for heads, dv in ((3, 12), (1, 40), (2, 200)):
        T = 7
        o = torch.randn(T, heads * dv, device=DEV) * 0.01                         # small rows: eps matters
        gate = torch.randn(2, T, 5 + heads * dv, device=DEV)
        g = gate.double().sum(0).cpu()[:, 5:]
        for weight in (1 + 0.3 * torch.randn(dv, device=DEV), 1 + 0.3 * torch.randn(heads * dv, device=DEV)):
            out = torch.empty(T, heads * dv, dtype=out_dtype, device=DEV)
            linear_attention.head_norm_gate(o, weight, gate, 5, "silu", out, heads, dv, 1e-4)
            normed = plain.rms(o.double().cpu().view(T, heads, dv), 1e-4)
            w = weight.double().cpu()
            normed = (normed * w).reshape(T, -1) if w.numel() == dv else normed.reshape(T, -1) * w
            assert torch.allclose(out.double().cpu(), normed * plain.silu(g), atol=atol)
            linear_attention.head_norm_gate(o, weight, None, 0, "silu", out, heads, dv, 1e-4)
            assert torch.allclose(out.double().cpu(), normed, atol=atol)


def blocked_attention(q, k, v, scale, block, window=None):
    """q [T, H, dk], k [T, G, dk], v [T, G, dv] float64 -> [T, H, dv]: causal softmax attention inside blocks of positions."""
    T, H, _ = q.shape
    rep = H // k.shape[1]
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    ok = j <= i
    if block:
        ok = ok & (i // block == j // block)
    if window:
        ok = ok & (j > i - window)
    s = torch.einsum("thd,jhd->thj", q, k.repeat_interleave(rep, 1)) * scale
    s = s.masked_fill(~ok[:, None, :], -math.inf)
    return torch.einsum("thj,jhd->thd", torch.softmax(s, -1), v.repeat_interleave(rep, 1))


@pytest.mark.parametrize("heads, kv_heads, dk, dv, rot, block", [(3, 3, 16, 24, 0, 7), (4, 2, 32, 32, 12, 16), (2, 1, 10, 6, 10, 3), (1, 1, 136, 40, 4, None)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rotation_then_quotient_then_attention_in_blocks(heads, kv_heads, dk, dv, rot, block, dtype):
    """qk_prepare with the norm BEHIND the rotation and without weights, and the attention kernel of two widths with blocks of
    positions, against the plain functions: two sequences in one step, the second continuing (inside a block) from pages an
    earlier step wrote; scattered pages.  Without weights the place of the norm does not matter (a turn keeps a pair's
    length); with weights it does, and both places are held against the plain order of operations."""
    from microllm_rocm_b200.kernels import attention_kv
    torch.manual_seed(heads * dk + dv)
    page, n_pages = 8, 12
    lengths, scale = [21, 13], 0.3 * 16 / dk
    qc, kc, vc = heads * dk, kv_heads * dk, kv_heads * dv
    seqs = [torch.randn(n, qc + kc + vc, device=DEV) * (1 + torch.arange(qc + kc + vc, device=DEV) % 3) for n in lengths]
    sc = {"factor": 3.0, "low": 1.0, "high": 4.0, "original": 16}
    freq = plain.rescaled_frequencies(rot, 100.0, sc) if rot else None
    freq_dev = freq.float().to(DEV) if rot else None
    table = torch.tensor([[7, 2, 9], [11, 0, 4]], dtype=torch.int32, device=DEV)

    qn, kn = 1 + 0.4 * torch.randn(dk, device=DEV), 1 + 0.4 * torch.randn(dk, device=DEV)

    def run(norm, weights=False):
        pages = torch.zeros(n_pages, kv_heads * page * (dk + dv), dtype=dtype, device=DEV)
        outs = [[], []]
        for spans in ([(0, 21), (0, 5)], [None, (5, 13)]):
            live = [i for i, s in enumerate(spans) if s]
            ctx, _ = step_of([spans[i][1] - spans[i][0] for i in live], [spans[i][0] for i in live], [0] * len(live))
            rows = torch.cat([seqs[i][spans[i][0]:spans[i][1]] for i in live])
            src = torch.stack([rows * 0.5, rows * 0.5])
            T = rows.shape[0]
            q = torch.empty(T, qc, dtype=dtype, device=DEV)
            attention_kv.qk_prepare(src, 0, qc, qc + kc, q_norm=qn if weights else None, k_norm=kn if weights else None, eps=1e-5,
                                    freq=freq_dev, rot_dims=rot, magnitude=1.0,
                                    q_temp=None, positions=ctx.positions, token_seq=ctx.token_seq, block_table=table[live].contiguous(),
                                    pages=pages, page_size=page, q_out=q, heads=heads, kv_heads=kv_heads, dk=dk, dv=dv,
                                    error_flag=ctx.error_flag, norm=norm)
            o = torch.empty(T, heads * dv, dtype=dtype, device=DEV)
            attention_kv.paged_attention_kv(q, pages, o, ctx.positions, ctx.token_seq, table[live].contiguous(), page, heads, kv_heads, dk, dv,
                                            scale, None, None, 0, ctx.error_flag, chunk=block)
            assert int(ctx.error_flag.item()) == 0
            at = 0
            for i in live:
                n = spans[i][1] - spans[i][0]
                outs[i].append(o[at:at + n])
                at += n
        return [torch.cat(o).double().cpu() for o in outs]

    got, other, weighted, weighted_first = run("after"), run("before"), run("after", True), run("before", True)
    atol = 2e-5 if dtype == torch.float32 else 0.06
    near = lambda a, b: torch.allclose(a, b, atol=atol, rtol=0.0 if dtype == torch.float32 else 0.02)
    for i, s in enumerate(seqs):
        x, T = s.double().cpu(), lengths[i]
        pos = torch.arange(T)
        q, k = x[:, :qc].view(T, heads, dk), x[:, qc:qc + kc].view(T, kv_heads, dk)
        if rot:
            q, k = plain.rotate_pairs(q, pos, rot, freq), plain.rotate_pairs(k, pos, rot, freq)
        q, k = plain.rms(q, 1e-5), plain.rms(k, 1e-5)
        v = x[:, qc + kc:].view(T, kv_heads, dv)
        want = blocked_attention(q, k, v, scale, block).reshape(T, heads * dv)
        assert near(got[i], want), float((got[i] - want).abs().max())
        assert torch.allclose(want, plain.block_attention(q, k, v, scale, block).reshape(T, -1))
        assert near(other[i], want)
        q0, k0 = x[:, :qc].view(T, heads, dk), x[:, qc:qc + kc].view(T, kv_heads, dk)
        turn = (lambda t: plain.rotate_pairs(t, pos, rot, freq)) if rot else (lambda t: t)
        behind = blocked_attention(plain.rms(turn(q0), 1e-5) * qn.double().cpu(), plain.rms(turn(k0), 1e-5) * kn.double().cpu(), v, scale, block)
        front = blocked_attention(turn(plain.rms(q0, 1e-5) * qn.double().cpu()), turn(plain.rms(k0, 1e-5) * kn.double().cpu()), v, scale, block)
        assert near(weighted[i], behind.reshape(T, -1)) and near(weighted_first[i], front.reshape(T, -1))
        if rot:
            assert float((behind - front).abs().max()) > 0.01                     # the two orders really differ


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_block_edges_and_far_keys_on_the_kernel_of_two_widths(dtype):
    """The last query and one key point the same way, so that a single score stands out: at the far end of the query's block
    (300 keys back), at a page's last and first place, on the block's first position (seen) and one position in front of
    it (not seen), with and without a window on top."""
    from microllm_rocm_b200.kernels import attention_kv
    torch.manual_seed(5)
    heads, dk, dv, page, T = 2, 64, 24, 16, 700
    for target, block, window, seen in ((0, None, None, True), (T - 300, 350, None, True), (T - 1 - 15, 350, None, True), (T - 1 - 16, 350, None, True),
                                        (350, 350, None, True), (349, 350, None, False), (600, 100, None, True), (599, 100, None, False),
                                        (400, 350, 300, True), (399, 350, 300, False), (350, 350, 400, True), (349, 350, 400, False)):
        k, v = torch.randn(T, heads * dk, device=DEV), torch.randn(T, heads * dv, device=DEV)
        qrow = torch.randn(1, heads * dk, device=DEV)
        k[target] = qrow[0]
        src = torch.cat([qrow.expand(T, -1), k, v], 1).contiguous()
        ctx, _ = step_of([T], [0], [0])
        n_pages = -(-T // page)
        pages = torch.zeros(n_pages, heads * page * (dk + dv), dtype=dtype, device=DEV)
        table = torch.arange(n_pages - 1, -1, -1, dtype=torch.int32, device=DEV).view(1, n_pages)
        q = torch.empty(T, heads * dk, dtype=dtype, device=DEV)
        attention_kv.qk_prepare(src, 0, heads * dk, 2 * heads * dk, q_norm=None, k_norm=None, eps=1e-5, freq=None, rot_dims=0, magnitude=1.0,
                                q_temp=None, positions=ctx.positions, token_seq=ctx.token_seq, block_table=table, pages=pages,
                                page_size=page, q_out=q, heads=heads, kv_heads=heads, dk=dk, dv=dv, error_flag=ctx.error_flag, norm="after")
        o = torch.empty(T, heads * dv, dtype=dtype, device=DEV)
        attention_kv.paged_attention_kv(q, pages, o, ctx.positions, ctx.token_seq, table, page, heads, heads, dk, dv, 1.0, window, None, 0,
                                        ctx.error_flag, chunk=block)
        close = torch.allclose(o[-1].float(), v[target], atol=0.05)
        assert close == seen, (target, block, window)
        # the same query alone, as a decoded token that reads the pages
        ctx1, _ = step_of([1], [T - 1], [0])
        o1 = torch.empty(1, heads * dv, dtype=dtype, device=DEV)
        attention_kv.paged_attention_kv(q[-1:].contiguous(), pages, o1, ctx1.positions, ctx1.token_seq, table, page, heads, heads, dk, dv, 1.0,
                                        window, None, 0, ctx1.error_flag, chunk=block)
        assert torch.allclose(o1[0].float(), o[-1].float(), atol=1e-5 if dtype == torch.float32 else 0.02)


def shared_kernel_step(pages, table, lens, q_list, news, nh, nkv, d, scale, window, block):
    """One step on the attention kernels of one width: sequence s brings news[s] queries at its last positions."""
    from microllm_rocm_b200.kernels import attention
    from microllm_rocm_b200.parts.base import StepContext
    pos0 = [l - n for l, n in zip(lens, news)]
    starts = [0]
    for n in news:
        starts.append(starts[-1] + n)
    q = torch.cat([x.reshape(x.shape[0], nh * d) for x in q_list]).contiguous()
    positions = torch.cat([torch.arange(p, p + n, dtype=torch.int32) for p, n in zip(pos0, news)]).to(DEV)
    token_seq = torch.cat([torch.full((n,), s, dtype=torch.int32) for s, n in enumerate(news)]).to(DEV)
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = torch.full(q.shape, float("nan"), dtype=torch.bfloat16, device=DEV)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    ctx = StepContext(num_tokens=q.shape[0], num_seqs=len(news), token_ids=positions, positions=positions, token_seq=token_seq,
                      seq_starts=i32(starts), seq_pos0=i32(pos0), seq_lens=i32(lens), block_tables={}, state_slots=None,
                      logit_rows=None, error_flag=flag, seq_starts_host=starts, seq_pos0_host=pos0,
                      max_new_tokens=max(news), max_seq_len=max(lens))
    attention.paged_attention(q, pages, out, ctx, table, nh, nkv, d, scale, window, chunk=block)
    torch.cuda.synchronize()
    assert int(flag.item()) == 0
    return out.float().reshape(-1, nh, d)


@pytest.mark.parametrize("d, page", [(64, 16), (128, 64), (32, 16), (256, 16)])
@pytest.mark.parametrize("block", [200, 64, 37])
def test_blocks_of_positions_on_the_kernels_of_one_width(d, page, block):
    """bf16, the tensor-core kernels (prompt portions and every decode form): whole prompts, a portion that starts inside a
    block, and single decoded tokens on the last position of a block, on the first of the next and on the one after it,
    against the formula over the same bf16 keys and values.  A query on a block's first position sees itself alone."""
    from microllm_rocm_b200.kernels import attention
    if not attention.mma_supported(d, page):
        pytest.skip("no tensor-core kernel for this head size and page size")
    nh, nkv, n = 4, 2, 3 * block + 5
    gen = torch.Generator(device=DEV).manual_seed(d + block)
    blocks = -(-n // page)
    pages = torch.randn((blocks + 2, 2, nkv, page, d), generator=gen, device=DEV).bfloat16()
    table = torch.randperm(blocks + 2, generator=gen, device=DEV).to(torch.int32)[:blocks].view(1, blocks).contiguous()
    got = pages[table[0].long()]
    k = got[:, 0].permute(0, 2, 1, 3).reshape(-1, nkv, d)[:n].double().cpu()
    v = got[:, 1].permute(0, 2, 1, 3).reshape(-1, nkv, d)[:n].double().cpu()
    q = (torch.randn((n, nh, d), generator=gen, device=DEV) * 2.0).bfloat16()
    scale = 1.0 / math.sqrt(d)
    want = blocked_attention(q.double().cpu(), k, v, scale, block)

    def check(out, first, what):
        ref = want[first:first + out.shape[0]]
        err = (out.double().cpu() - ref).abs().amax(-1) / ref.abs().amax(-1).clamp_min(1e-3)
        assert torch.isfinite(out).all() and float(err.max()) < 0.03, (what, float(err.max()), int(err.argmax()))

    check(shared_kernel_step(pages, table, [n], [q], [n], nh, nkv, d, scale, None, block), 0, "whole prompt")
    start = 2 * block - 3                                                         # a portion from inside a block across two edges
    check(shared_kernel_step(pages, table, [n], [q[start:]], [n - start], nh, nkv, d, scale, None, block), start, "portion")
    for pos in (block - 1, block, block + 1, 2 * block - 1, 2 * block, n - 1):
        one = shared_kernel_step(pages, table, [pos + 1], [q[pos:pos + 1]], [1], nh, nkv, d, scale, None, block)
        check(one, pos, f"decoded token at {pos}")
        if pos % block == 0:
            rep = nh // nkv
            assert torch.allclose(one[0].double().cpu(), v[pos].repeat_interleave(rep, 0), atol=0.02)
    # several decoded tokens of unequal contexts in one step, one of them with a window on top of the blocks
    lens = [block, block + 1, 2 * block + 2, n]
    outs = shared_kernel_step(pages, table.expand(4, -1).contiguous(), lens, [q[l - 1:l] for l in lens], [1] * 4, nh, nkv, d, scale, None, block)
    for i, l in enumerate(lens):
        check(outs[i:i + 1], l - 1, f"batched decode at {l - 1}")
    w = block // 2
    ref = blocked_attention(q.double().cpu(), k, v, scale, block, window=w)
    both = shared_kernel_step(pages, table, [n], [q], [n], nh, nkv, d, scale, w, block)
    err = (both.double().cpu() - ref).abs().amax(-1) / ref.abs().amax(-1).clamp_min(1e-3)
    assert float(err.max()) < 0.03


# ------------------------------------------------------------------------------------------- whole models
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", ["a", "b"])
def test_every_layer_against_the_plain_residual_stream(folders, key, dtype):
    from microllm_rocm_b200.engine.step import StepEntry
    folder, raw, weights = folders[key]
    tokens = random_tokens(41, raw["vocab"], 5)
    want = []
    plain.forward(raw, weights, tokens, want)
    engine = engine_for(folder, dtype)
    got = {}
    engine.cache.add("x")
    engine.step([StepEntry("x", tokens, [])], tensor_sink=lambda name, t: got.__setitem__(name, None if t is None else t.float().cpu().clone()))
    engine.check_device_errors()
    for i, ref in enumerate(want):
        name = [n for n in got if n.startswith(f"run{i}.") and n.endswith(".residual")][0]
        err = float((got[name].double() - ref).abs().max() / ref.abs().max())
        assert err < (2e-5 if dtype == "float32" else 0.05), f"layer {i}: {err:.3e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", sorted(CASES))
@pytest.mark.parametrize("cut", ["whole", "tail", "portions"])
def test_one_request_at_a_time(folders, key, dtype, cut):
    folder, raw, weights = folders[key]
    reqs = requests_for(raw, LENGTHS[key])
    steps = {"whole": steps_whole, "tail": steps_prefill_then_decode, "portions": steps_portions}[cut](reqs)
    got = collect(engine_for(folder, dtype), steps)
    compare(got, key, raw, weights, reqs, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", ["a", "c", "e", "f"])
def test_mixed_batches_over_a_tight_pool(folders, key, dtype):
    """Up to four live requests, portions beside single tokens, some left out of a step; the pool holds just the peak and
    there are four state slots for ten requests, so pages and slots go from one request to the next (a slot's old state
    and previous input must not leak into the request that takes it)."""
    folder, raw, weights = folders[key]
    reqs = requests_for(raw, [60, 33, 150, 90, 47, 128, 75, 20, 101, 64], seed=9)
    steps, peak = steps_mixed(reqs, max_live=4, seed=3)
    engine = engine_for(folder, dtype, max_tokens=peak, max_requests=4)
    got = collect(engine, steps)
    compare(got, key, raw, weights, reqs, dtype)
    if "full" in engine.cache.groups:                          # a model of recurrence layers alone has no pages
        pool = engine.cache.groups["full"].pool
        assert pool.total_allocations > pool.num_pages, "the pool was never tight enough to use a page again"
    else:
        assert key == "e"
    assert engine.cache.slots.total_allocations > 4, "no state slot was used again"


def test_fp32_does_not_depend_on_cuts_batches_or_pages(folders):
    for key in ("a", "c"):
        folder, raw, weights = folders[key]
        reqs = requests_for(raw, [70, 133, 20, 45], seed=4)
        whole = collect(engine_for(folder, "float32"), steps_whole(reqs))
        portions = collect(engine_for(folder, "float32", page_size=8), steps_portions(reqs, sizes=(2, 9, 2, 30, 1, 5)))
        steps, peak = steps_mixed(reqs, max_live=3, seed=1)
        mixed = collect(engine_for(folder, "float32", max_tokens=peak), steps)
        for k in whole:
            assert torch.equal(whole[k], portions[k]) and torch.equal(whole[k], mixed[k]), f"case {key}: {k} differs between schedules"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", ["a", "c", "f"])
def test_far_keys_page_borders_and_block_edges_decide_the_output(tmp_path_factory, dtype, key):
    """Peaky softmax (its scale multiplied): single keys, far back in a block and at page borders, carry a position's output,
    and a position right behind a block's edge sees one or two keys only, so one key too many or too few shows; in a prompt
    of several hundred tokens and in the tokens decoded after it, with two page sizes and portions that end on, one before
    and one behind an edge."""
    raw, weights = case(key, seed=11, sharp=3.0)
    folder = write_folder(str(tmp_path_factory.mktemp("fonuvik_sharp")), raw, weights)
    block = (raw["layers"][[l["type"] for l in raw["layers"]].index("parallel")]["mixer"]["left"].get("mask") or {}).get("size") or 96
    edge = 3 * block if 3 * block + 40 < 700 else block
    reqs = {"long": random_tokens(700 if block < 700 else 330, raw["vocab"], 21), "edge": random_tokens(min(edge, 500) + 3, raw["vocab"], 22)}
    n = len(reqs["edge"])
    cuts = (n - 4, 1, 2, 1)                                                        # the portions end one before, on, and behind the edge
    for page_size, steps in ((16, steps_prefill_then_decode(reqs, tail=40)), (32, steps_portions(reqs, sizes=cuts + (127, 2, 33, 1, 64, 300)))):
        got = collect(engine_for(folder, dtype, max_tokens=1200, page_size=page_size), steps)
        compare(got, key + "-sharp", raw, weights, reqs, dtype)
    # the softmax really is peaky: with the plain scale the logits are far from these
    a = plain.forward(raw, weights, reqs["edge"][:60])
    b = plain.forward(case(key, seed=11)[0], weights, reqs["edge"][:60])
    assert float((a - b).abs().max() / a.abs().max()) > 3 * BF16_TOL


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", ["d", "e"])
def test_long_decoding_from_the_first_token(folders, dtype, key):
    """One token per step from position 0 on, over many pages: every step reads and writes the state slots."""
    folder, raw, weights = folders[key]
    reqs = {"d": random_tokens(150, raw["vocab"], 8)}
    got = collect(engine_for(folder, dtype, page_size=8), steps_prefill_then_decode(reqs, tail=149))
    compare(got, key, raw, weights, reqs, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_scheduler(folders, dtype):
    from microllm_rocm_b200.engine.llm import LLM
    from microllm_rocm_b200.sampling import GenerationConfig
    folder, raw, weights = folders["a"]
    prompts = [random_tokens(n, raw["vocab"], 50 + n) for n in (9, 40, 3)]
    llm = LLM(folder, dtype=dtype, page_size=16, max_tokens=512)
    outs = llm.generate(prompts, GenerationConfig(max_new_tokens=12, temperature=0.0))
    for prompt, got in zip(prompts, outs):
        assert len(got) == 12
        seq = list(prompt)
        for i, token in enumerate(got):
            ref = plain.forward(raw, weights, seq)[-1]
            if dtype == "float32":
                assert token == int(ref.argmax()), f"token {i} differs from the plain greedy choice"
            else:       # bf16 may leave the fp32 choice at a near tie: every pick must be a near maximum of the plain logits
                assert float(ref.max() - ref[token]) <= 0.05 * float(ref.abs().max())
            seq.append(token)
