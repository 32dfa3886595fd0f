"""The Lozepel decoder on the GPU against its plain float64 restatement: each mechanism alone, then whole models cut in
every way (whole prompts, a tail decoded token by token, portions down to two tokens, mixed batches over a pool so small
that pages and state slots are used again), in true fp32 and in bf16, and greedy generation through the scheduler."""
import math
from types import SimpleNamespace

import pytest
import torch

from tests.helpers import collect, random_tokens, steps_mixed, steps_portions, steps_prefill_then_decode, steps_whole
from tests.lozepel_cases import CASES, case, write_folder
from tests.plain import lozepel_plain as plain

pytestmark = pytest.mark.gpu

FP32_TOL = 3e-5          # of the largest |logit|
BF16_TOL = 0.05          # of the largest |logit|
DEV = "cuda:0"
LENGTHS = {"a": [1, 2, 37, 130], "b": [5, 64, 99], "c": [3, 50, 290], "d": [17, 80]}
F64 = torch.float64


def tol(dtype):
    return FP32_TOL if dtype == "float32" else BF16_TOL


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for key in CASES:
        raw, weights = case(key)
        out[key] = (write_folder(str(tmp_path_factory.mktemp("lozepel_" + key)), raw, weights), raw, weights)
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


def compare(got, key, raw, weights, requests, dtype, share=0.15, fp32_tol=FP32_TOL, median=0.4):
    """fp32: every position within the tolerance.  bf16 rounds the router's input (and the weights): where two choice scores
    are a rounding error apart the choice flips, that position lands far off, and the linear attention's state carries a
    little of it to every later position of the request.  So bf16 is held, over all positions of a case, to a small median
    error and to at most `share` of them over the tolerance."""
    errs = []
    for rid, toks in requests.items():
        ref = plain_logits(raw, weights, toks)
        rows = torch.stack([got[(rid, p)] for p in range(len(toks))])
        assert torch.isfinite(rows).all(), f"case {key} request {rid}: logits that are not finite"
        err = (rows - ref).abs().amax(dim=1) / ref.abs().max()
        if dtype == "float32" and bool((err > fp32_tol).any()):
            pos = int((err > fp32_tol).nonzero()[0])
            raise AssertionError(f"case {key} request {rid}: position {pos} of {len(toks)} is over the tolerance {fp32_tol} "
                                 f"(error {float(err[pos]):.3e} of the largest |logit|)")
        errs.append(err)
    err = torch.cat(errs)
    over = int((err > tol(dtype)).sum())
    if dtype != "float32":
        assert over <= max(2, int(share * err.numel())) and float(err.median()) <= median * tol(dtype), \
            f"case {key}: {over} of {err.numel()} positions over the tolerance {tol(dtype)}, median error {float(err.median()):.3e}"
    print(f"[lozepel parity] case {key} {dtype}: median error {float(err.median()):.3e}, worst {float(err.max()):.3e} of the largest |logit|, {over} over")
    return float(err.median())


def requests_for(raw, lengths, seed=0):
    return {f"r{i}": random_tokens(n, raw["vocab"], seed + 100 * i + n) for i, n in enumerate(lengths)}


def i32(v):
    return torch.tensor(v, dtype=torch.int32, device=DEV)


def step_of(lengths, pos0, slots, tokens=None):
    """The per-sequence arrays a kernel sees of a step whose sequences bring `lengths` tokens from positions `pos0`."""
    starts = [0]
    for n in lengths:
        starts.append(starts[-1] + n)
    return SimpleNamespace(
        seq_starts=i32(starts), seq_pos0=i32(pos0), num_seqs=len(lengths), error_flag=torch.zeros(1, dtype=torch.int32, device=DEV),
        token_seq=i32([a for a, n in enumerate(lengths) for _ in range(n)]), token_ids=i32(tokens if tokens is not None else [0] * starts[-1]),
        positions=i32([p + i for p, n in zip(pos0, lengths) for i in range(n)])), i32(slots)


# ------------------------------------------------------------------------------------------- mechanisms alone
@pytest.mark.parametrize("table_dtype", [torch.float32, torch.bfloat16])
def test_pair_table_over_steps_with_slots_used_again(table_dtype):
    """Three steps of unequal portions (one of a single token); the token in front of a step's first token comes from the
    sequence's slot; a sequence that starts in a slot another one left takes the table's last row, not that slot's token."""
    from microllm_rocm_b200.kernels import ops
    torch.manual_seed(2)
    buckets, a, b, W = 53, 40009, 7919, 40
    table = torch.randn(buckets + 1, W, device=DEV).to(table_dtype)
    token_table = torch.randn(60000, W, device=DEV).to(table_dtype)
    state = torch.full((4, 1), 123456, dtype=torch.int32, device=DEV)            # slots hold a pattern: nothing of it may be read
    seqs = {0: random_tokens(9, 60000, 1), 1: random_tokens(7, 60000, 2), 2: random_tokens(4, 60000, 3)}
    want = {s: table.double()[torch.tensor(plain.bigram_rows(t, buckets, a, b))] for s, t in seqs.items()}
    # (sequence, slot, first token, count) per step; sequence 2 starts in step 3 in the slot sequence 1 held
    plan = [[(0, 2, 0, 4), (1, 0, 0, 1)], [(0, 2, 4, 1), (1, 0, 1, 6)], [(0, 2, 5, 4), (2, 0, 0, 4)]]
    for step in plan:
        toks = [t for s, _, p, n in step for t in seqs[s][p:p + n]]
        ctx, slots = step_of([n for *_, n in step], [p for _, _, p, _ in step], [sl for _, sl, _, _ in step], toks)
        both = torch.full((len(toks), W), float("nan"), device=DEV)                 # token row and pair row gathered and added in one pass
        ops.bigram_add(both, table, ctx, state, slots, buckets, a, b, update_state=False, token_table=token_table)
        x = torch.zeros(len(toks), W, device=DEV)
        ops.bigram_add(x, table, ctx, state, slots, buckets, a, b)
        assert int(ctx.error_flag.item()) == 0
        assert torch.allclose(both, x + token_table.float()[torch.tensor(toks, device=DEV)], atol=1e-6)
        at = 0
        for s, _, p, n in step:
            assert torch.allclose(x[at:at + n].double().cpu(), want[s][p:p + n].cpu(), atol=1e-6), (s, p)
            at += n
    assert state[2, 0].item() == seqs[0][8] and state[0, 0].item() == seqs[2][3]
    assert state[1, 0].item() == 123456 and state[3, 0].item() == 123456            # other slots are not touched


def test_norm_over_whole_rows_of_two_column_blocks():
    from microllm_rocm_b200.kernels import attention_kv
    torch.manual_seed(3)
    T, qn, kn, rest = 7, 36, 20, 13
    parts = torch.randn(3, T, qn + kn + rest, device=DEV) * 2                       # three partial results
    wq, wk = 1 + 0.3 * torch.randn(qn, device=DEV), 1 + 0.3 * torch.randn(kn, device=DEV)
    out = torch.empty(T, qn + kn + rest, device=DEV)
    attention_kv.row_norm_columns(parts, out, 0, qn, wq, qn, kn, wk, 1e-4)
    x = parts.double().sum(0)
    assert torch.allclose(out[:, :qn].double(), plain.rms_quotient(x[:, :qn], 1e-4) * wq.double(), atol=1e-5)
    assert torch.allclose(out[:, qn:qn + kn].double(), plain.rms_quotient(x[:, qn:qn + kn], 1e-4) * wk.double(), atol=1e-5)
    assert torch.allclose(out[:, qn + kn:].double(), x[:, qn + kn:], atol=1e-5)            # the rest passes (summed)
    # per head it would be another number: the norm is over the row
    per_head = plain.rms_quotient(x[:, :qn].view(T, 3, 12), 1e-4).reshape(T, qn) * wq.double()
    assert not torch.allclose(out[:, :qn].double(), per_head, atol=1e-3)


def _attend(dtype, H, G, dk, dv, rot, lengths, pos0_tokens, scale, sink, cap, gate_per_head, bias, values_keys, norm_after, page_size=8,
            q_boost=None, same_keys=False):
    """Projection columns -> qk_prepare -> paged_attention_kv over scattered pages, in two steps (the second goes on from the
    first), against the plain formula over whole sequences.  Returns (got, want) [tokens of both steps, H * dv] per sequence."""
    from microllm_rocm_b200.kernels import attention_kv
    from microllm_rocm_b200.parts.base import Runtime
    from microllm_rocm_b200.parts.rotary import RotaryEmbedding
    torch.manual_seed(11)
    dt = torch.float32 if dtype == "float32" else torch.bfloat16
    A = len(lengths)
    total = [a + b for a, b in zip(pos0_tokens, lengths)]
    q_cols, k_cols, v_cols = H * dk, G * dk, 0 if values_keys else G * dv
    g_cols = H if gate_per_head else 0
    cols = q_cols + k_cols + v_cols + g_cols
    proj = [torch.randn(n, cols, dtype=F64) for n in total]
    if same_keys:                                                                 # every key of a sequence is nearly the same vector
        for x in proj:
            x[:, q_cols:q_cols + k_cols] = torch.randn(1, k_cols, dtype=F64) + 0.05 * torch.randn(x.shape[0], k_cols, dtype=F64)
    if q_boost:
        for a, (qt, kt, factor) in q_boost.items():                              # query qt and key kt point the same way, strongly
            for h in range(H):
                g = h // (H // G)
                proj[a][qt, h * dk:(h + 1) * dk] = proj[a][kt, q_cols + g * dk:q_cols + (g + 1) * dk] * factor
    b = torch.randn(cols, dtype=F64) * 0.5 if bias else None
    if b is not None:
        b[q_cols + k_cols:] = 0
    freq = None
    if rot:
        table = RotaryEmbedding(dict(head_dim=dk, rotary_dim=rot[0], theta=rot[1], layout="interleaved"), Runtime(torch.device(DEV), dt)).rotary_table(dk)
        freq = table.inv_freq
    pages_per_seq = [-(-n // page_size) for n in total]
    num_pages = sum(pages_per_seq) + 3
    order = torch.randperm(num_pages).tolist()                                    # scattered pages
    table_rows, at = [], 0
    for n in pages_per_seq:
        table_rows.append(order[at:at + n] + [-1] * (max(pages_per_seq) - n))
        at += n
    block_table = i32(table_rows)
    pages = torch.full((num_pages, G * page_size * (dk + dv)), float("nan"), dtype=dt, device=DEV)
    sink_t = torch.tensor(sink, dtype=torch.float32, device=DEV) if sink is not None else None
    got = [torch.zeros(n, H * dv, dtype=F64) for n in total]
    for first, counts in ((pos0_tokens and [0] * A, pos0_tokens), (pos0_tokens, lengths)):
        if not any(counts):
            continue
        live = [a for a in range(A) if counts[a] > 0]
        rows = torch.cat([proj[a][first[a]:first[a] + counts[a]] for a in live]).to(torch.float32).to(DEV)
        ctx, _ = step_of([counts[a] for a in live], [first[a] for a in live], [0] * len(live))
        T = rows.shape[0]
        q = torch.empty(T, H * dk, dtype=dt, device=DEV)
        attention_kv.qk_prepare(rows, 0, q_cols, q_cols + k_cols if v_cols else q_cols, q_norm=None, k_norm=None, eps=1e-5, freq=freq,
                                rot_dims=rot[0] if rot else 0, magnitude=1.0, q_temp=None, positions=ctx.positions, token_seq=ctx.token_seq,
                                block_table=block_table[live].contiguous(), pages=pages, page_size=page_size, q_out=q, heads=H, kv_heads=G,
                                dk=dk, dv=dv, error_flag=ctx.error_flag, norm="after" if norm_after else None,
                                bias=b.to(torch.float32).to(DEV) if b is not None else None)
        o = torch.empty(T, H * dv, dtype=dt, device=DEV)
        attention_kv.paged_attention_kv(q, pages, o, ctx.positions, ctx.token_seq, block_table[live].contiguous(), page_size, H, G, dk, dv, scale,
                                        None, rows if g_cols else None, q_cols + k_cols + v_cols, ctx.error_flag, gate_per_head=bool(g_cols),
                                        sink=sink_t, softcap=cap or 0.0)
        assert int(ctx.error_flag.item()) == 0
        at = 0
        for a in live:
            got[a][first[a]:first[a] + counts[a]] = o[at:at + counts[a]].double().cpu()
            at += counts[a]
    want = []
    for a in range(A):
        x = proj[a] + (b if b is not None else 0)
        qq, kk = x[:, :q_cols].view(-1, H, dk), x[:, q_cols:q_cols + k_cols].view(-1, G, dk)
        vv = kk.clone() if values_keys else x[:, q_cols + k_cols:q_cols + k_cols + v_cols].view(-1, G, dv)
        if rot:
            qq, kk = plain.rotate_pairs(qq, rot[0], rot[1]), plain.rotate_pairs(kk, rot[0], rot[1])
        if norm_after:
            qq, kk = plain.rms_quotient(qq, 1e-5), plain.rms_quotient(kk, 1e-5)
        o = plain.sink_attention(qq, kk, vv, scale, torch.tensor(sink if sink is not None else [-1e30] * H, dtype=F64), cap)
        if g_cols:
            o = o * torch.sigmoid(x[:, q_cols + k_cols + v_cols:])[:, :, None]
        want.append(o.reshape(-1, H * dv))
    return got, want


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,dk,dv,rot,sink,cap,gate,bias,vkeys,after", [
    (4, 2, 16, 16, (12, 5000.0), [0.0] * 4, None, True, True, True, False),           # values are the biased, unturned keys; one added to the denominator
    (3, 1, 24, 40, (24, 300.0), [1.5, -0.5, 4.0], 2.5, False, False, False, True),    # turned, then divided; capped scores; learned sinks
    (2, 2, 40, 136, None, [3.0, 0.5], None, True, False, False, False),               # no rotation; wide values; a gate per head
    (1, 1, 72, 8, (8, 100.0), None, 1.0, False, False, False, True),                  # no sink at all: the plain softmax is still there
])
def test_sink_cap_bias_and_head_gate(dtype, H, G, dk, dv, rot, sink, cap, gate, bias, vkeys, after):
    got, want = _attend(dtype, H, G, dk, dv, rot, lengths=[5, 1, 19], pos0_tokens=[21, 40, 0], scale=0.7, sink=sink, cap=cap,
                        gate_per_head=gate, bias=bias, values_keys=vkeys, norm_after=after)
    for g, w in zip(got, want):
        assert torch.allclose(g, w, atol=2e-5 if dtype == "float32" else 0.06), float((g - w).abs().max())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_sink_swallows_small_scores_and_is_neither_scaled_nor_capped(dtype):
    """Queries point away from every key (all keys of a sequence are nearly one vector; scores far below 0): with a sink of
    0 the weights nearly vanish, without it they sum to one.  With a large scale and a tight cap a sink of 6 weighs e^6
    against keys capped at e^2: a sink that was scaled or capped with the scores would weigh differently by far."""
    kw = dict(lengths=[3, 1], pos0_tokens=[30, 17], gate_per_head=False, bias=False, values_keys=False, norm_after=False)
    away = {0: (32, 5, -3.0), 1: (17, 2, -3.0)}
    got, want = _attend(dtype, 2, 1, 16, 16, None, scale=1.0, sink=[0.0, 0.0], cap=None, q_boost=away, same_keys=True, **kw)
    none, _ = _attend(dtype, 2, 1, 16, 16, None, scale=1.0, sink=None, cap=None, q_boost=away, same_keys=True, **kw)
    for a, t in ((0, 32), (1, 17)):
        assert torch.allclose(got[a][t], want[a][t], atol=1e-5 if dtype == "float32" else 0.02)
        assert float(got[a][t].abs().max()) < 1e-3 and float(none[a][t].abs().max()) > 0.02
    got, want = _attend(dtype, 2, 1, 16, 16, None, scale=9.0, sink=[6.0, 6.0], cap=2.0, **kw)
    _, capped = _attend(dtype, 2, 1, 16, 16, None, scale=9.0, sink=[2.0 * math.tanh(3.0)] * 2, cap=2.0, **kw)
    for g, w, c in zip(got, want, capped):
        assert torch.allclose(g, w, atol=1e-5 if dtype == "float32" else 0.02)
        assert float((w - c).abs().max()) > 0.2                                  # a capped sink would land elsewhere


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("qt,kt", [(299, 0), (299, 7), (299, 8), (200, 15), (200, 16), (64, 63), (64, 64)])
def test_one_score_that_stands_out(dtype, qt, kt):
    """One query and one key point the same way: the far end of 300 keys, a page's last and first place, the key right in
    front of the query and the query's own, in a prompt and (the step's one token) decoded."""
    boost = {0: (qt, kt, 2.5)}
    for lengths, pos0 in (([300], [0]), ([1], [qt])):                             # in a prompt; as the one token of a decode step
        got, want = _attend(dtype, 2, 1, 32, 24, None, lengths=lengths, pos0_tokens=pos0, scale=1.0, sink=[0.5, 0.5], cap=None,
                            gate_per_head=False, bias=False, values_keys=False, norm_after=False, q_boost=boost)
        assert torch.allclose(got[0][qt], want[0][qt], atol=1e-4 if dtype == "float32" else 0.06)
        # that one key carries the output: without it the row would be another
        assert float(want[0][qt].abs().max()) > 0.1


@pytest.mark.parametrize("heads,dk,dv,decay", [(3, 8, 12, (0.5, 0.9, 1.0)), (1, 136, 40, (0.97,)), (2, 64, 64, (0.999, 0.2))])
def test_fixed_decay_recurrence_over_steps(heads, dk, dv, decay):
    """silu on q, k, v; S <- d S + k v^T; o = S^T q over three steps of unequal portions in slots that hold a pattern, one
    sequence starting late in a slot that was used; then the norm over all heads together and the sigmoid gate."""
    from microllm_rocm_b200.kernels import linear_attention, recurrent
    torch.manual_seed(5)
    HK, HV = heads * dk, heads * dv
    cols = 2 * HK + 2 * HV
    seqs = {s: torch.randn(n, cols, dtype=F64) for s, n in ((0, 23), (1, 9), (2, 6))}
    state = torch.full((3, heads, dk, dv), 7.0, device=DEV)
    hd = torch.tensor(decay, dtype=torch.float32, device=DEV)
    norm_w = 1 + 0.2 * torch.randn(HV, device=DEV)
    got = {s: torch.zeros(x.shape[0], HV, dtype=F64) for s, x in seqs.items()}
    plan = [[(0, 1, 0, 17), (1, 0, 0, 1)], [(0, 1, 17, 1), (1, 0, 1, 8)], [(0, 1, 18, 5), (2, 0, 0, 6)]]
    for step in plan:
        rows = torch.cat([seqs[s][p:p + n] for s, _, p, n in step]).to(torch.float32).to(DEV)
        ctx, slots = step_of([n for *_, n in step], [p for _, _, p, _ in step], [sl for _, sl, _, _ in step])
        T = rows.shape[0]
        parts = torch.stack([rows * 0.25, rows * 0.75])                            # two partial results
        q, k, d, v, o = (torch.empty(T, n, device=DEV) for n in (HK, HK, HK, HV, HV))
        linear_attention.lightning_prepare(parts, 0, HK, 2 * HK, hd, q, k, v, d, heads, dk, dv)
        recurrent.linear_scan("decayed_sum", q, k, d, v, o, state, slots, ctx, heads, dk, dv)
        out = torch.empty(T, HV, device=DEV)
        linear_attention.row_norm_gate(o, norm_w, parts, 2 * HK + HV, out, 1e-5)
        assert int(ctx.error_flag.item()) == 0
        at = 0
        for s, _, p, n in step:
            got[s][p:p + n] = out[at:at + n].double().cpu()
            at += n
    for s, x in seqs.items():
        n = x.shape[0]
        o = plain.decayed_state(plain.silu(x[:, :HK]).view(n, heads, dk), plain.silu(x[:, HK:2 * HK]).view(n, heads, dk),
                                plain.silu(x[:, 2 * HK:2 * HK + HV]).view(n, heads, dv), list(decay)).reshape(n, HV)
        want = plain.rms_quotient(o, 1e-5) * norm_w.double().cpu() * torch.sigmoid(x[:, 2 * HK + HV:])
        assert torch.allclose(got[s], want, atol=3e-4, rtol=1e-4), (s, float((got[s] - want).abs().max()))


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_clamped_gate_activation(out_dtype):
    from microllm_rocm_b200.kernels import ops
    torch.manual_seed(6)
    rows, width, limit = 11, 37, 1.25
    parts = torch.randn(2, rows, 2 * width, device=DEV) * 1.5                      # values on both sides of the clamp
    out = torch.empty(rows, width, dtype=out_dtype, device=DEV)
    ops.gated_act_mul(parts, out, "clamped_swish", limit)
    x = parts.double().sum(0)
    g, u = x[:, :width].clamp(max=limit), x[:, width:].clamp(-limit, limit)
    want = g * torch.sigmoid(1.702 * g) * (u + 1)
    assert bool((x[:, :width] > limit).any()) and bool((x[:, width:] < -limit).any())
    assert torch.allclose(out.double(), want, atol=1e-5 if out_dtype == torch.float32 else 0.02)


@pytest.mark.parametrize("tokens", [1, 8, 9, 40, 130, 300])
def test_clamped_feed_forward_on_every_product_kernel(tokens):
    """The dense feed-forward part alone in bf16 at token counts that take each of its routes (the few-token kernels with
    the activation as their epilogue or behind partial sums, the streaming kernel, the library product with the activation
    kernel, the CTA-pair kernel) against float64 on the same bf16 weights; a limit that never bites must land elsewhere."""
    from microllm_rocm_b200.engine.loading import prepare_kernels
    from microllm_rocm_b200.parts.base import FEED_FORWARDS, Runtime
    torch.manual_seed(tokens)
    hidden, inter, limit = 256, 768, 0.75
    rt = Runtime(torch.device(DEV), torch.bfloat16)
    w = {"gate": torch.randn(inter, hidden, device=DEV) * hidden ** -0.5, "up": torch.randn(inter, hidden, device=DEV) * hidden ** -0.5,
         "down": torch.randn(hidden, inter, device=DEV) * inter ** -0.5}
    w = {k: v.to(torch.bfloat16) for k, v in w.items()}
    x = (torch.randn(tokens, hidden, device=DEV) * 1.5).to(torch.bfloat16)
    outs = {}
    for lim in (limit, 1e4):
        part = FEED_FORWARDS["swiglu"](dict(hidden_size=hidden, intermediate_size=inter, names=("gate", "up", "down"),
                                            activation="clamped_swish", limit=lim), rt)
        prepare_kernels(SimpleNamespace(parts=lambda: [part]))
        part.bind(dict(w))
        y = part.forward(x, None)
        outs[lim] = (y.sum(0) if y.dim() == 3 else y).double().cpu()
    wd = {"m." + k: v.double().cpu() for k, v in w.items()}
    want = plain.dense_ff({"limit": limit}, wd, "m.", x.double().cpu())
    assert float((outs[limit] - want).abs().max() / want.abs().max()) < 0.02
    assert float((outs[1e4] - want).abs().max() / want.abs().max()) > 0.05


@pytest.mark.parametrize("outputs,experts,top", [(10, 7, 3), (4, 2, 4), (3, 3, 1), (40, 33, 8)])
def test_choice_by_corrected_scores_weights_without_and_outputs_without_an_expert(outputs, experts, top):
    from microllm_rocm_b200.kernels import moe
    torch.manual_seed(7)
    T, W = 29, 24
    parts = torch.randn(2, T, outputs + 3, device=DEV) * 1.5                        # three padding columns, two partial results
    corr = torch.randn(outputs, device=DEV) * 0.3
    ids = torch.empty(T, top, dtype=torch.int32, device=DEV)
    weights = torch.empty(T, top, device=DEV)
    moe.select(parts, outputs, corr, top, ids, weights, scoring="softmax_all")
    chosen, w = plain.route(parts.double().sum(0)[:, :outputs].cpu(), corr.double().cpu(), top)
    assert ids.cpu().tolist() == chosen.tolist()
    assert torch.allclose(weights.double().cpu(), w, atol=1e-6)
    flipped = plain.route(parts.double().sum(0)[:, :outputs].cpu(), torch.zeros(outputs, dtype=F64), top)[0]
    assert outputs == top or flipped.tolist() != chosen.tolist()                    # the correction did steer some choice
    # pairs of real experts are listed by expert; the others are left out and take the token's own input
    offsets = torch.empty(experts + 1, dtype=torch.int32, device=DEV)
    order = torch.full((T * top,), -1, dtype=torch.int32, device=DEV)
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    moe.align(ids, experts, offsets, order, flag, passthrough=outputs - experts)
    assert flag.item() == 0
    flat = ids.flatten().cpu()
    assert offsets[experts].item() == int((flat < experts).sum())
    for e in range(experts):
        listed = sorted(order[offsets[e].item():offsets[e + 1].item()].cpu().tolist())
        assert listed == (flat == e).nonzero().flatten().tolist()
    y = torch.full((T * top, W), float("nan"), device=DEV)                          # rows of choices without an expert are never written
    real = (ids.flatten() < experts)
    y[real] = torch.randn(int(real.sum()), W, device=DEV)
    for dt in (torch.float32, torch.bfloat16):
        x = torch.randn(T, W, device=DEV).to(dt)
        out = torch.empty(T, W, device=DEV)
        moe.combine(y, weights, out, ids=ids, experts=experts, x=x)
        rows = torch.where(real[:, None], y, x.float().repeat_interleave(top, 0)).double().view(T, top, W)
        assert torch.allclose(out.double(), (weights.double()[:, :, None] * rows).sum(1), atol=1e-5)


def test_cap_on_the_logits():
    from microllm_rocm_b200.kernels import ops
    x = torch.linspace(-90, 90, 1001, device=DEV).view(7, 143).contiguous()
    want = 12.5 * torch.tanh(x.double() / 12.5)
    ops.softcap_rows(x, 12.5)
    assert torch.allclose(x.double(), want, atol=1e-5)


def one_width_step(pages, table, lens, q_list, news, nh, nkv, d, scale, sink, cap):
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
    ctx = StepContext(num_tokens=q.shape[0], num_seqs=len(news), token_ids=positions, positions=positions, token_seq=token_seq,
                      seq_starts=i32(starts), seq_pos0=i32(pos0), seq_lens=i32(lens), block_tables={}, state_slots=None,
                      logit_rows=None, error_flag=flag, seq_starts_host=starts, seq_pos0_host=pos0,
                      max_new_tokens=max(news), max_seq_len=max(lens))
    attention.paged_attention(q, pages, out, ctx, table, nh, nkv, d, scale, None, sink=sink, softcap=cap or 0.0)
    torch.cuda.synchronize()
    assert int(flag.item()) == 0
    return out.float().reshape(-1, nh, d)


@pytest.mark.parametrize("d, page", [(64, 16), (128, 64), (32, 16), (256, 16)])
@pytest.mark.parametrize("sink, cap", [((2.0, -1.0, 0.0, 5.0), None), ((0.5, 0.5, 3.0, -2.0), 1.5), (None, 4.0), ((60.0, -60.0, 9.0, 0.0), None)])
def test_sink_and_cap_on_the_kernels_of_one_width(d, page, sink, cap):
    """bf16, the tensor-core kernels (prompt portions, every decode form, decoded tokens beside portions) against the formula
    over the same bf16 keys and values: sinks of both signs (one far above every score, one far below), a tight cap."""
    from microllm_rocm_b200.kernels import attention
    if not attention.mma_supported(d, page):
        pytest.skip("no tensor-core kernel for this head size and page size")
    nh, nkv, n = 4, 2, 700
    gen = torch.Generator(device=DEV).manual_seed(d + (7 if cap else 0))
    blocks = -(-n // page)
    pages = torch.randn((blocks + 2, 2, nkv, page, d), generator=gen, device=DEV).bfloat16()
    table = torch.randperm(blocks + 2, generator=gen, device=DEV).to(torch.int32)[:blocks].view(1, blocks).contiguous()
    got = pages[table[0].long()]
    k = got[:, 0].permute(0, 2, 1, 3).reshape(-1, nkv, d)[:n].double().cpu()
    v = got[:, 1].permute(0, 2, 1, 3).reshape(-1, nkv, d)[:n].double().cpu()
    q = (torch.randn((n, nh, d), generator=gen, device=DEV) * 2.0).bfloat16()
    scale = 2.0 / math.sqrt(d)
    sink_t = torch.tensor(sink, dtype=torch.float32, device=DEV) if sink else None
    want = plain.sink_attention(q.double().cpu(), k, v, scale, torch.tensor(sink if sink else [-1e30] * nh, dtype=F64), cap)

    def check(out, rows, what):
        ref = want[rows]
        err = (out.double().cpu() - ref).abs().amax(-1) / ref.abs().amax(-1).clamp_min(0.05)
        assert torch.isfinite(out).all() and float(err.max()) < 0.04, (what, float(err.max()), int(err.argmax()))

    check(one_width_step(pages, table, [n], [q], [n], nh, nkv, d, scale, sink_t, cap), slice(0, n), "whole prompt")
    check(one_width_step(pages, table, [n], [q[300:]], [n - 300], nh, nkv, d, scale, sink_t, cap), slice(300, n), "portion")
    for pos in (0, 1, 127, 128, n - 1):
        check(one_width_step(pages, table, [pos + 1], [q[pos:pos + 1]], [1], nh, nkv, d, scale, sink_t, cap), slice(pos, pos + 1), f"decoded token at {pos}")
    lens = [1, 130, 500, n]                                                      # several decoded tokens of unequal contexts in one step
    outs = one_width_step(pages, table.expand(4, -1).contiguous(), lens, [q[l - 1:l] for l in lens], [1] * 4, nh, nkv, d, scale, sink_t, cap)
    for i, l in enumerate(lens):
        check(outs[i:i + 1], slice(l - 1, l), f"batched decode at {l - 1}")
    # a portion of one sequence beside a decoded token of another (the same pages under two tables)
    both = one_width_step(pages, table.expand(2, -1).contiguous(), [400, n], [q[250:400], q[n - 1:n]], [150, 1], nh, nkv, d, scale, sink_t, cap)
    check(both[:150], slice(250, 400), "portion beside a decoded token")
    check(both[150:], slice(n - 1, n), "decoded token beside a portion")


# ------------------------------------------------------------------------------------------- whole models
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", sorted(CASES))
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
        err = (got[name].double() - ref).abs().amax(1) / ref.abs().max()              # per token
        if dtype == "float32":
            assert float(err.max()) < 2e-5, f"layer {i}: {float(err.max()):.3e}"
        else:
            # bf16 rounds the router's input: a token whose two best choice scores are a rounding error apart takes another
            # expert and lands far off, and later tokens that attend to it move a little
            assert float(err.median()) < 0.02 and int((err > 0.05).sum()) <= len(tokens) // 4, f"layer {i}: {err.tolist()}"


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
@pytest.mark.parametrize("key", ["a", "b", "c"])
def test_mixed_batches_over_a_tight_pool(folders, key, dtype):
    """Up to four live requests, portions beside single tokens, some left out of a step; the pool holds just the peak and
    there are four state slots for ten requests, so pages and slots go from one request to the next (a slot's old state
    and previous token must not leak into the request that takes it)."""
    folder, raw, weights = folders[key]
    reqs = requests_for(raw, [60, 33, 150, 90, 47, 128, 75, 20, 101, 64], seed=9)
    steps, peak = steps_mixed(reqs, max_live=4, seed=3)
    engine = engine_for(folder, dtype, max_tokens=peak, max_requests=4)
    got = collect(engine, steps)
    compare(got, key, raw, weights, reqs, dtype)
    pool = engine.cache.groups["full"].pool
    assert pool.total_allocations > pool.num_pages, "the pool was never tight enough to use a page again"
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
@pytest.mark.parametrize("key", ["a", "c", "d"])
def test_far_keys_and_page_borders_decide_the_output(tmp_path_factory, dtype, key):
    """Peaky softmax (its scale and cap multiplied) with small sinks: single keys, far back and at page borders, carry a
    position's output, in a prompt of several hundred tokens and in the tokens decoded after it, with two page sizes and
    portions of many sizes.  Scores three times as large carry three times the rounding error into the exponentials: fp32 is
    held to 1e-4 of the largest logit here, bf16 to a median of 0.6 of its tolerance with a fifth of the positions over it."""
    raw, weights = case(key, seed=11, sharp=3.0, sink=-1.0)
    folder = write_folder(str(tmp_path_factory.mktemp("lozepel_sharp")), raw, weights)
    reqs = {"long": random_tokens(600, raw["vocab"], 21), "short": random_tokens(67, raw["vocab"], 22)}
    for page_size, steps in ((16, steps_prefill_then_decode(reqs, tail=40)), (32, steps_portions(reqs, sizes=(63, 1, 2, 1, 127, 2, 33, 1, 64, 300)))):
        got = collect(engine_for(folder, dtype, max_tokens=1200, page_size=page_size), steps)
        compare(got, key + "-sharp", raw, weights, reqs, dtype, share=0.2, fp32_tol=1e-4, median=0.6)
    # the softmax really is peaky: with the plain scale the logits are far from these
    a = plain.forward(raw, weights, reqs["short"][:60])
    b = plain.forward(case(key, seed=11, sink=-1.0)[0], weights, reqs["short"][:60])
    assert float((a - b).abs().max() / a.abs().max()) > 3 * BF16_TOL


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_large_sinks_show_in_the_logits(tmp_path_factory, dtype):
    """Sinks around 4 take much of every softmax's weight: a sink left out, scaled or capped would move the logits far."""
    raw, weights = case("a", seed=13, sink=4.0)
    folder = write_folder(str(tmp_path_factory.mktemp("lozepel_sinks")), raw, weights)
    reqs = requests_for(raw, [50, 3], seed=2)
    got = collect(engine_for(folder, dtype), steps_portions(reqs, sizes=(2, 7, 1, 30)))
    compare(got, "a-sinks", raw, weights, reqs, dtype)
    without = {n: (t - 30.0 if n.endswith("sink") else t) for n, t in weights.items()}
    a, b = plain.forward(raw, weights, reqs["r0"]), plain.forward(raw, without, reqs["r0"])
    assert float((a - b).abs().max() / a.abs().max()) > 3 * BF16_TOL


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", ["b", "d"])
def test_long_decoding_from_the_first_token(folders, dtype, key):
    """One token per step from position 0 on, over many pages: every step reads and writes the state slots (the linear
    attention's matrices and the embedding's previous token)."""
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


def test_random_config_from_the_command_line_presets():
    """The tiny preset with seeded random weights through the same entry the command line uses, against the plain
    implementation over the tensors the engine drew."""
    from microllm_rocm_b200.config import find_preset
    from microllm_rocm_b200.engine.loading import random_engine
    from microllm_rocm_b200.engine.step import StepEntry
    arch, cfg = find_preset("lozepel-tiny")
    engine = random_engine(cfg, seed=3, dtype="float32", max_tokens=256, max_requests=2)
    tokens = random_tokens(33, cfg.vocab, 4)
    engine.cache.add("x")
    logits = engine.step([StepEntry("x", tokens, list(range(33)))]).cpu()
    engine.check_device_errors()
    assert torch.isfinite(logits).all() and float(logits.abs().max()) <= cfg.logit_softcap
