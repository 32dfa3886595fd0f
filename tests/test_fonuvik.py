"""Host-side tests of the Fonuvik design: configuration, the model description, the cache manager's books for mixers
with pages and fixed-size state at once, and identities of the plain implementation that the GPU tests lean on."""
import copy
import math

import pytest
import torch

from tests.fonuvik_cases import CASES, case, with_ranks, write_folder
from tests.plain import fonuvik_plain as plain


def _model(raw, dtype=torch.float32):
    from microllm_rocm_b200.config import get_architecture
    from microllm_rocm_b200.config.fonuvik import FonuvikConfig
    from microllm_rocm_b200.parts.base import Runtime
    from microllm_rocm_b200.parts.build import build_model
    arch = get_architecture("Fonuvik")
    return build_model(arch.build_spec(FonuvikConfig.from_dict(raw)), Runtime(torch.device("cpu"), dtype))


def _ranked(key):
    raw, weights = case(key)
    return with_ranks(raw, weights), weights


@pytest.mark.parametrize("key", sorted(CASES))
def test_declared_tensors_are_the_checkpoints(key):
    raw, weights = _ranked(key)
    expected = _model(raw).expected_tensors()
    assert set(expected) == set(weights)
    for name, spec in expected.items():
        assert tuple(spec.shape) == tuple(weights[name].shape), name
    assert "head" not in expected                                         # the head is the embedding table


def test_inner_widths_come_from_the_tensors_shapes(tmp_path):
    from microllm_rocm_b200.config.fonuvik import FonuvikConfig
    from microllm_rocm_b200.config.qwen2 import ConfigError
    from microllm_rocm_b200.config.registry import load_config
    raw, weights = case("a")
    with pytest.raises(ConfigError):
        FonuvikConfig.from_dict(raw)                     # config.json alone does not say them
    folder = write_folder(str(tmp_path / "m"), raw, weights)
    arch, cfg = load_config(folder)
    assert arch.name == "Fonuvik"
    assert cfg.layers[0]["mixer"]["right"]["a_rank"] == CASES["a"]["ranks"][0]
    assert cfg.layers[1]["mixer"]["w_rank"] == CASES["a"]["ranks"][1]
    again = FonuvikConfig.from_dict(cfg.to_dict())
    assert again == cfg and hash(again) == hash(cfg)


def test_presets_build():
    from microllm_rocm_b200.config import find_preset
    for name in ("fonuvik-tiny", "fonuvik-small", "fonuvik-3b-layers"):
        arch, cfg = find_preset(name)
        assert arch.name == "Fonuvik" and len(arch.build_spec(cfg).layers) == len(cfg.layers)


def test_refusals():
    from microllm_rocm_b200.config.fonuvik import FonuvikConfig
    from microllm_rocm_b200.config.qwen2 import ConfigError
    good, _ = _ranked("a")

    def broken(change):
        raw = copy.deepcopy(good)
        change(raw)
        with pytest.raises(ConfigError):
            FonuvikConfig.from_dict(raw)
    broken(lambda r: r.pop("norm"))
    broken(lambda r: r["layers"][0].__setitem__("type", "mamba"))
    broken(lambda r: r["layers"][0]["mixer"]["left"]["rot"].__setitem__("dims", 13))
    broken(lambda r: r["layers"][0]["mixer"]["left"]["rot"].__setitem__("dims", 18))          # more than a head has
    broken(lambda r: r["layers"][0]["mixer"]["left"].__setitem__("kv_heads", 3))              # 4 heads do not divide
    broken(lambda r: r["layers"][0]["mixer"]["left"]["mask"].__setitem__("size", 0))
    broken(lambda r: r["layers"][0]["mixer"]["left"]["rot"]["scaling"].__setitem__("high", 1.0))
    broken(lambda r: r["layers"][0]["mixer"]["right"].__setitem__("tau", 0.0))
    broken(lambda r: r["layers"][0]["mlp"].__setitem__("kind", "dense"))
    broken(lambda r: r["layers"][0]["mlp"]["router"].__setitem__("top", 6))                    # of five experts
    broken(lambda r: r["layers"][1]["mixer"].pop("dim"))


def test_every_mixer_gets_its_caches():
    from microllm_rocm_b200.cache.manager import CacheManager, page_shape
    from microllm_rocm_b200.parts.base import FixedStateNeed, PagedKVNeed
    raw, _ = _ranked("a")
    model = _model(raw)
    assert set(model.cache_entries) == {"run0.left", "run0.right.state", "run1.state", "run1.shift", "run2.left", "run2.right.state"}
    kv = model.cache_entries["run0.left"].need
    assert isinstance(kv, PagedKVNeed) and (kv.head_dim, kv.value_dim) == (16, 24)
    assert page_shape(kv, 8) == (2 * 8 * (16 + 24),)
    assert model.cache_entries["run0.right.state"].need == FixedStateNeed((3, 8, 12), torch.float32)
    assert model.cache_entries["run1.state"].need == FixedStateNeed((3, 24, 24), torch.float32)
    assert model.cache_entries["run1.shift"].need == FixedStateNeed((64,), torch.float32)     # the previous token's input
    manager = CacheManager(model.cache_entries, page_size=8, num_pages=6, max_requests=2)
    assert manager.add("x") and manager.add("y") and not manager.add("z")
    assert manager.reserve("x", 30) and not manager.reserve("y", 30)
    manager.commit("x", 30); manager.release("x"); manager.check()
    assert manager.add("z") and manager.slot("z") == 0                              # the freed slot is used again
    # recurrence layers only: no pages at all, and the engine still runs on slots
    only, _ = _ranked("e")
    assert set(_model(only).cache_entries) == {"run0.state", "run0.shift", "run1.state", "run1.shift"}


def test_rescaled_frequencies_equal_the_plain_ones():
    from microllm_rocm_b200.parts.rotary import rescaled_frequencies
    for dims, base, sc in ((12, 5000.0, {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 48}),
                           (32, 5e5, {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 128}),
                           (6, 50.0, {"factor": 2.5, "low": 2.0, "high": 3.0, "original": 60})):
        freq = rescaled_frequencies(base, dims, sc)
        want = plain.rescaled_frequencies(dims, base, sc)
        assert torch.allclose(torch.from_numpy(freq).double(), want, rtol=1e-6)
        untouched = plain.rescaled_frequencies(dims, base, None)
        assert want[0] == untouched[0]                                               # the fastest pair keeps its frequency
        assert torch.isclose(want[-1], untouched[-1] / sc["factor"])                 # the slowest turns `factor` times slower
        ratio = want / untouched
        assert ((ratio > 1 / sc["factor"] + 1e-9) & (ratio < 1 - 1e-9)).any()        # and some pair lies between the two


def test_plain_recurrences_carry_their_state():
    torch.manual_seed(0)
    T, H, dk, dv = 23, 2, 5, 7
    q, k = torch.randn(T, H, dk, dtype=plain.F), torch.randn(T, H, dk, dtype=plain.F)
    v, a = torch.randn(T, H, dv, dtype=plain.F), torch.rand(T, H, dk, dtype=plain.F)
    u = torch.randn(H, dk, dtype=plain.F)
    whole, S = plain.decayed_sum(q, k, v, a)
    first, Sa = plain.decayed_sum(q[:9], k[:9], v[:9], a[:9])
    rest, Sb = plain.decayed_sum(q[9:], k[9:], v[9:], a[9:], Sa)
    assert torch.allclose(torch.cat([first, rest]), whole) and torch.allclose(Sb, S)
    # the read-out of the decayed sum sees the present token's write, whatever its decay: o_0 = v_0 (k_0 . q_0)
    assert torch.allclose(whole[0], v[0] * (k[0] * q[0]).sum(-1, keepdim=True))
    whole, S2 = plain.bonus_sum(q, k, v, a, u)
    first, Sa = plain.bonus_sum(q[:9], k[:9], v[:9], a[:9], u)
    rest, Sb = plain.bonus_sum(q[9:], k[9:], v[9:], a[9:], u, Sa)
    assert torch.allclose(torch.cat([first, rest]), whole) and torch.allclose(Sb, S2)
    # the bonus read sees the present token through u only: o_0 = v_0 (u k_0 . q_0); the state is the same sum
    assert torch.allclose(whole[0], v[0] * (u * k[0] * q[0]).sum(-1, keepdim=True)) and torch.allclose(S2, S)
    # the decay acts on the rows of key channels: a channel with decay 0 forgets, its neighbour with decay 1 keeps
    a2 = torch.ones(2, 1, 2, dtype=plain.F); a2[1, 0, 0] = 0.0
    k2, v2 = torch.ones(2, 1, 2, dtype=plain.F), torch.tensor([[[1.0]], [[10.0]]], dtype=plain.F)
    _, S3 = plain.decayed_sum(k2, k2, v2, a2)
    assert S3[0, :, 0].tolist() == [10.0, 11.0]


def test_plain_blocks_of_positions_and_token_shift():
    seen = plain.visible(9, 4)
    assert seen[3, 0] and seen[3, 3] and not seen[4, 3] and seen[4, 4] and seen[7, 4] and not seen[8, 7] and not seen[2, 3]
    assert torch.equal(plain.visible(9, None), torch.tril(torch.ones(9, 9, dtype=torch.bool)))
    assert torch.equal(plain.visible(9, 100), plain.visible(9, None))
    h = torch.arange(6, dtype=plain.F).view(3, 2) + 1
    assert plain.shifted(h).tolist() == [[0.0, 0.0], [1.0, 2.0], [3.0, 4.0]]
    assert plain.shifted(h[1:], h[0]).tolist() == [[1.0, 2.0], [3.0, 4.0]]


def test_plain_routing_weights():
    torch.manual_seed(3)
    h = torch.randn(6, 10, dtype=plain.F)
    w = {"m.router": torch.randn(5, 10, dtype=plain.F), "m.router.b": torch.tensor([0.0, 0.0, 50.0, 0.0, 0.0], dtype=plain.F)}
    ids, weights = plain.route(h, w, "m.", 2)
    assert (ids[:, 0] == 2).all()                                                  # the bias takes part in the choice
    assert torch.allclose(weights.sum(-1), torch.ones(6, dtype=plain.F)) and (weights[:, 0] > 0.99).all()      # and in the weights
    ids, weights = plain.route(h, w, "m.", 1)
    assert torch.equal(weights, torch.ones(6, 1, dtype=plain.F))                   # one expert: weight 1 whatever its logit
    assert math.isclose(float(plain.silu(torch.tensor(0.0, dtype=plain.F))), 0.0)
