"""Host-side tests of the Lozepel design: configuration, the model description (declared tensors, run order, caches, state
of the embedding), and facts of the plain implementation that the GPU tests lean on."""
import copy
import math

import pytest
import torch

from tests.lozepel_cases import CASES, case, write_folder
from tests.plain import lozepel_plain as plain


def _model(raw, dtype=torch.float32):
    from microllm_rocm_b200.config import get_architecture
    from microllm_rocm_b200.config.lozepel import LozepelConfig
    from microllm_rocm_b200.parts.base import Runtime
    from microllm_rocm_b200.parts.build import build_model
    arch = get_architecture("Lozepel")
    return build_model(arch.build_spec(LozepelConfig.from_dict(raw)), Runtime(torch.device("cpu"), dtype))


@pytest.mark.parametrize("key", sorted(CASES))
def test_declared_tensors_are_the_checkpoints(key):
    raw, weights = case(key)
    expected = _model(raw).expected_tensors()
    assert set(expected) == set(weights)
    for name, spec in expected.items():
        assert tuple(spec.shape) == tuple(weights[name].shape), name
    # a layer that reads another layer's keys and values has no key and value projections
    for i, layer in enumerate(raw["layers"]):
        if layer["mixer"].get("kv_from") is not None:
            assert f"l{i}.mix.k" not in expected and f"l{i}.mix.v" not in expected and f"l{i}.mix.q" in expected


def test_configuration_round_trip_and_choice_by_name(tmp_path):
    from microllm_rocm_b200.config.lozepel import LozepelConfig
    from microllm_rocm_b200.config.registry import load_config
    for key in CASES:
        raw, weights = case(key)
        folder = write_folder(str(tmp_path / key), raw, weights)
        arch, cfg = load_config(folder)
        assert arch.name == "Lozepel"
        again = LozepelConfig.from_dict(cfg.to_dict())
        assert again == cfg and hash(again) == hash(cfg)
        assert (cfg.bigram is None) == ("embedding" not in raw)
        assert cfg.logit_softcap == raw["logit_softcap"]


def test_presets_build():
    from microllm_rocm_b200.config import find_preset
    for name in ("lozepel-tiny", "lozepel-small", "lozepel-3b-layers"):
        arch, cfg = find_preset(name)
        spec = arch.build_spec(cfg)
        assert arch.name == "Lozepel" and len(spec.layers) == len(cfg.layers)
        assert spec.order[3].read_cache_of == 2


def test_refusals():
    from microllm_rocm_b200.config.lozepel import LozepelConfig
    from microllm_rocm_b200.config.qwen2 import ConfigError
    raw = case("a")[0]

    def broken(change):
        bad = copy.deepcopy(raw)
        change(bad)
        with pytest.raises(ConfigError):
            LozepelConfig.from_dict(bad)
    broken(lambda r: r.pop("norm"))
    broken(lambda r: r["layers"][0].__setitem__("type", "mamba"))
    broken(lambda r: r["layers"][0]["mixer"].__setitem__("kv_heads", 3))                  # 4 heads, 3 kv heads
    broken(lambda r: r["layers"][0]["mixer"].__setitem__("vdim", 24))                     # the values are the keys
    broken(lambda r: r["layers"][0]["mixer"]["rot"].__setitem__("dims", 13))
    broken(lambda r: r["layers"][1]["mixer"]["right"].__setitem__("decay", [0.5, 0.9]))   # three heads
    broken(lambda r: r["layers"][3]["mixer"].__setitem__("kv_from", 3))                   # not an earlier layer
    broken(lambda r: r["layers"][3]["mixer"].__setitem__("kv_from", 1))                   # not a layer of that kind
    broken(lambda r: r["layers"][3]["mixer"].__setitem__("dim", 32))                      # other keys than the layer it reads
    broken(lambda r: r["layers"][1]["mlp"]["router"].__setitem__("top", 7))               # five experts and one pass-through
    broken(lambda r: r["layers"][0]["mlp"].__setitem__("kind", "gelu"))
    broken(lambda r: r["embedding"]["bigram"].__setitem__("buckets", 0))
    broken(lambda r: r.__setitem__("logit_softcap", -1.0))


def test_run_order_and_caches():
    from microllm_rocm_b200.parts.base import FixedStateNeed, PagedKVNeed
    model = _model(case("c")[0])
    order = model.spec.order
    assert [r.layer for r in order] == [0, 1, 2, 3, 4]
    assert [r.read_cache_of for r in order] == [None, None, 0, None, 0]
    entries = model.cache_entries
    # the embedding's previous token, pages per owning attention run, a matrix state for the linear attention; readers own nothing
    assert set(entries) == {"embedding", "run0", "run1", "run3.left", "run3.right.state"}
    assert isinstance(entries["embedding"].need, FixedStateNeed) and entries["embedding"].need.dtype == torch.int32
    assert isinstance(entries["run0"].need, PagedKVNeed) and isinstance(entries["run3.right.state"].need, FixedStateNeed)
    assert model.run_cache[2] == ("run0", False) and model.run_cache[4] == ("run0", False)
    assert "embedding" not in _model(case("d")[0]).cache_entries                           # no pair table, no state
    # keys of 40 beside values of 136 share a page
    need = _model(case("d")[0]).cache_entries["run1"].need
    assert (need.head_dim, need.value_dim) == (40, 136)


def test_books_for_pages_and_states():
    from microllm_rocm_b200.cache.manager import CacheManager
    model = _model(case("a")[0])
    cache = CacheManager(model.cache_entries, page_size=8, num_pages=6, max_requests=2)
    assert cache.add("x") and cache.add("y") and not cache.add("z")
    assert cache.reserve("x", 20) and cache.reserve("y", 17)
    assert not cache.reserve("x", 40)
    cache.commit("x", 20)
    slot = cache.slot("x")
    cache.release("x")
    assert cache.add("z") and cache.slot("z") == slot                                      # the freed slot is the next one used
    cache.check()


def test_pair_rows_of_the_plain_embedding():
    assert plain.bigram_rows([5, 9, 9, 0], 7, 3, 2) == [7, (5 * 3 + 9 * 2) % 7, (9 * 3 + 9 * 2) % 7, (9 * 3) % 7]
    assert plain.bigram_rows([4], 11, 100, 100) == [11]
    big = plain.bigram_rows([2 ** 30, 2 ** 30 + 1], 1000003, 2 ** 30, 2 ** 29)             # no 32-bit wrap-around
    assert big[1] == (2 ** 30 * 2 ** 30 + (2 ** 30 + 1) * 2 ** 29) % 1000003


def test_plain_routing_by_hand():
    z = torch.tensor([[0.0, math.log(2.0), math.log(3.0), math.log(4.0)]], dtype=torch.float64)        # s = 0.1, 0.2, 0.3, 0.4
    none = torch.zeros(4, dtype=torch.float64)
    chosen, w = plain.route(z, none, 2)
    assert chosen.tolist() == [[3, 2]] and torch.allclose(w, torch.tensor([[0.4, 0.3]], dtype=torch.float64))
    # a correction steers the choice and leaves the weights alone; they are not renormalised
    chosen, w = plain.route(z, torch.tensor([0.5, 0.0, 0.0, 0.0], dtype=torch.float64), 2)
    assert chosen.tolist() == [[0, 3]] and torch.allclose(w, torch.tensor([[0.1, 0.4]], dtype=torch.float64))
    # an output without an expert passes the token's input on, times its weight
    mlp = {"router": {"experts": 1, "top": 2, "identity": 1}, "expert": {"ff": 2}}
    weights = {"m.router": torch.zeros(2, 3), "m.correction": torch.zeros(2), "m.e0.gate": torch.zeros(2, 3), "m.e0.up": torch.ones(2, 3),
               "m.e0.down": torch.ones(3, 2)}
    h = torch.tensor([[1.0, -2.0, 4.0]], dtype=torch.float64)
    assert torch.allclose(plain.routed_ff(mlp, weights, "m.", h), 0.5 * h)                 # silu(0) = 0: the expert adds nothing


def test_plain_sink_and_cap():
    q = torch.tensor([[[1.0, 0.0]]], dtype=torch.float64)
    k = torch.tensor([[[2.0, 0.0]]], dtype=torch.float64)
    v = torch.tensor([[[3.0, 5.0]]], dtype=torch.float64)
    # one key with score 2: p = e^2 / (e^sink + e^2)
    for sink in (0.0, 2.0, -30.0):
        o = plain.sink_attention(q, k, v, 1.0, torch.tensor([sink], dtype=torch.float64))
        assert torch.allclose(o[0, 0], v[0, 0] * math.exp(2.0) / (math.exp(sink) + math.exp(2.0)))
    # the cap bends the score, not the sink
    o = plain.sink_attention(q, k, v, 1.0, torch.tensor([2.0], dtype=torch.float64), cap=1.0)
    s = math.tanh(2.0)
    assert torch.allclose(o[0, 0], v[0, 0] * math.exp(s) / (math.exp(2.0) + math.exp(s)))


def test_plain_state_is_carried_and_decays():
    torch.manual_seed(0)
    q, k, v = (torch.randn(9, 2, 3, dtype=torch.float64) for _ in range(3))
    whole = plain.decayed_state(q, k, v, [0.5, 1.0])
    # by hand for the last token: o = sum_j d^(t-j) (q_t . k_j) v_j
    for h, d in enumerate((0.5, 1.0)):
        want = sum(d ** (8 - j) * float(q[8, h] @ k[j, h]) * v[j, h] for j in range(9))
        assert torch.allclose(whole[8, h], want)


def test_plain_dense_clamp():
    w = {"m.gate": torch.tensor([[1.0], [1.0]]), "m.up": torch.tensor([[1.0], [-1.0]]), "m.down": torch.eye(2)}
    y = plain.dense_ff({"limit": 2.0}, w, "m.", torch.tensor([[5.0]], dtype=torch.float64))
    g = 2.0 * (1 / (1 + math.exp(-1.702 * 2.0)))
    assert torch.allclose(y, torch.tensor([[g * 3.0, g * -1.0]], dtype=torch.float64))       # gate 5 -> 2; up 5 -> 2 and -5 -> -2
    y = plain.dense_ff({"limit": 2.0}, w, "m.", torch.tensor([[-5.0]], dtype=torch.float64))   # the gate has no floor
    g = -5.0 * (1 / (1 + math.exp(1.702 * 5.0)))
    assert torch.allclose(y, torch.tensor([[g * -1.0, g * 3.0]], dtype=torch.float64))
