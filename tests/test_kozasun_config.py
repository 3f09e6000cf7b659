"""Host-side pieces of the Kozasun architecture: configuration, run order, manifest, and the plain implementation's
own consistency (no GPU)."""
import copy

import numpy as np
import pytest
import torch

import kozasun_models as M
import plain_kozasun as P
from rustingstrata_b200.config import ConfigError, resolve_architecture
from rustingstrata_b200.config.kozasun_config import DenseConfig, KozasunConfig, MoeConfig
from rustingstrata_b200.models import manifest_for


@pytest.mark.parametrize("name", sorted(M.CONFIGS))
def test_manifest_follows_the_configuration(name):
    """The engine asks for exactly the tensors the configuration implies, with their shapes (derived independently)."""
    cfg = M.CONFIGS[name]
    got = {n: tuple(v.shape) for n, v in manifest_for(cfg).items() if not v.optional}
    assert got == M.tensor_shapes(cfg)


def test_architecture_is_found_by_its_key_and_sizes_come_from_the_file():
    cfg = M.CONFIGS["P"]
    arch = resolve_architecture(cfg)
    c = arch.config_class.from_dict(cfg)
    assert isinstance(c, KozasunConfig) and (c.vocab, c.width, c.eps, c.streams, c.embedding_scale) == (211, 96, 1e-6, 3, 0.25)
    spec = arch.build_spec(c)
    assert spec.n_streams == 3 and spec.embedding.params["scale"] == 0.25 and spec.embedding.params["copies"] == 3
    a = spec.layers[0].parts["mixer"].params
    assert (a["n_heads"], a["n_kv_heads"], a["dim"], a["vdim"], a["scale"], a["eps"], a["chunk"], a["window"]) == \
        (6, 2, 24, 40, 0.3, 1e-6, 20, None)
    assert (a["norm"], a["talk"], a["gate"], a["sink"], a["bias"]) == ("row", False, False, True, True)
    assert spec.layers[0].parts["mixer_position"].params == {"n_rot": 8, "base": 5000.0, "base_bits": 64}
    rt = spec.layers[1].parts["mixer"].params
    assert (rt["n_heads"], rt["dim"], rt["vdim"], tuple(rt["decay"])) == (3, 24, 20, (0.9, 0.97, 0.995))
    assert spec.layers[1].parts["mixer_position"].params["n_rot"] == 24
    la = spec.layers[2].parts["mixer"].params
    assert (la["n_heads"], la["dim"], la["vdim"], la["kv_rank"], la["rot_dim"], la["window"], la["scale"], la["gate"]) == \
        (3, 16, 24, 40, 0, 33, 0.25, True) and la["weights_bits"] == 32
    assert "feed_forward" not in spec.layers[2].parts and "mixer_position" not in spec.layers[2].parts
    assert spec.layers[0].parts["feed_forward"].params == {"hidden": 96, "intermediate": 160, "activation": "gelu_tanh"}
    m = spec.layers[1].parts["feed_forward"].params
    assert (m["experts"], m["top"], m["expert_ff"], m["shared_ff"], m["groups"], m["keep"], m["route_scale"]) == (6, 2, 40, 56, 3, 2, 1.5)
    assert (m["score"], m["renormalize"], m["expert"], m["correction"]) == ("sigmoid", False, "gated_silu", True)
    m = spec.layers[3].parts["feed_forward"].params
    assert (m["experts"], m["top"], m["shared_ff"], m["groups"], m["route_scale"]) == (5, 1, None, 0, 1.0)
    assert "mixer_position" not in spec.layers[3].parts
    # absent keys: no streams, no scale, kv heads equal to heads, value size equal to the key size
    q = arch.config_class.from_dict(M.CONFIGS["Q"])
    assert q.streams is None and q.embedding_scale == 1.0
    qs = arch.build_spec(q)
    assert qs.n_streams == 1 and not qs.layers[0].block.tensors and qs.layers[0].parts["mixer"].params["chunk"] is None
    bare = copy.deepcopy(M.CONFIGS["Q"])
    del bare["layers"][0]["mixer"]["kv_heads"], bare["layers"][0]["mixer"]["vdim"]
    b = arch.config_class.from_dict(bare).layers[0].mixer
    assert (b.kv_heads, b.vdim) == (5, 32)
    assert isinstance(q.layers[1].mlp, DenseConfig) and isinstance(q.layers[0].mlp, MoeConfig) and q.layers[2].mlp is None


def test_a_layer_that_uses_another_layers_tensors_is_one_more_entry_of_the_run_order():
    cfg = M.CONFIGS["P"]
    arch = resolve_architecture(cfg)
    spec = arch.build_spec(arch.config_class.from_dict(cfg))
    assert len(spec.layers) == 4
    assert [c.layer for c in spec.order] == [0, 1, 2, 0, 3, 2] and all(c.cache is None for c in spec.order)
    names = set(manifest_for(cfg))
    assert not any(n.startswith(("l3.", "l5.")) for n in names) and any(n.startswith("l4.") for n in names)
    # a layer may name a later layer, or one that itself names another: the tensors are those at the end of the chain
    c = copy.deepcopy(cfg)
    c["layers"] = [dict(c["layers"][2], weights_of=5), c["layers"][0], dict(c["layers"][2], weights_of=3), c["layers"][2],
                   dict(c["layers"][0], weights_of=1), dict(c["layers"][2], weights_of=2)]
    spec = arch.build_spec(arch.config_class.from_dict(c))
    assert len(spec.layers) == 2 and [x.layer for x in spec.order] == [0, 1, 0, 0, 1, 0]
    assert {n.split(".")[0] for n in manifest_for(c) if n.startswith("l")} == {"l1", "l3"}
    # an entry that differs from the named layer's in a constant runs that layer's tensors with its own constant
    c = copy.deepcopy(cfg)
    c["layers"][5]["mixer"]["mask"]["size"] = 12
    spec = arch.build_spec(arch.config_class.from_dict(c))
    assert [x.layer for x in spec.order] == [0, 1, 2, 0, 3, 4] and spec.layers[4].parts["mixer"].params["window"] == 12
    assert spec.layers[4].parts["mixer"].tensors == spec.layers[2].parts["mixer"].tensors
    assert set(manifest_for(c)) == set(manifest_for(cfg))


@pytest.mark.parametrize("bad", [
    lambda c: c.pop("norm"), lambda c: c["layers"][0].update(type="conv"), lambda c: c.pop("vocab"),
    lambda c: c["layers"][0]["mixer"]["rot"].update(dims=9), lambda c: c["layers"][0]["mixer"].update(kv_heads=4),
    lambda c: c["layers"][1]["mixer"].update(decay=[0.5]), lambda c: c["layers"][0]["mlp"].update(kind="routed"),
    lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(count=4), lambda c: c["layers"][1]["mlp"]["router"].update(top=5),
    lambda c: c["layers"][3].update(weights_of=3), lambda c: c["layers"][3].update(weights_of=6),
    lambda c: (c["layers"][3].update(weights_of=5), c["layers"][5].update(weights_of=3)),
    lambda c: c["layers"][3]["mixer"].update(heads=3), lambda c: c["layers"][2]["mixer"].pop("kv_rank"),
    lambda c: c["layers"][2]["mixer"]["mask"].update(size=0)])
def test_broken_configurations_are_refused_with_a_sentence(bad):
    cfg = copy.deepcopy(M.CONFIGS["P"])
    bad(cfg)
    with pytest.raises(ConfigError):
        KozasunConfig.from_dict(cfg)


def test_plain_pieces_against_closed_forms():
    """The plain implementation's own pieces: the rotation turns pairs of halves and keeps lengths, the masks count what
    they should, the sink takes its share, retention is the decayed sum written out, and the router keeps to its groups."""
    x = torch.randn(5, 2, 12, dtype=torch.float64)
    y = P.rotate_half(x, 100.0, 8)
    assert torch.allclose(y[..., 8:], x[..., 8:]) and torch.allclose(y[0], x[0])
    assert torch.allclose((y[..., :8] ** 2).sum(-1), (x[..., :8] ** 2).sum(-1))
    a = 3 * 100.0 ** (-2.0 / 8)
    assert torch.allclose(y[3, 0, 1], x[3, 0, 1] * np.cos(a) - x[3, 0, 5] * np.sin(a))
    assert torch.allclose(y[3, 0, 5], x[3, 0, 5] * np.cos(a) + x[3, 0, 1] * np.sin(a))
    assert P.visible(10, "chunk", 4).sum(1).tolist() == [1, 2, 3, 4, 1, 2, 3, 4, 1, 2]
    assert P.visible(10, "window", 4).sum(1).tolist() == [1, 2, 3, 4, 4, 4, 4, 4, 4, 4]
    assert P.visible(4, None, 0).sum(1).tolist() == [1, 2, 3, 4]
    pw = P.softmax_with_sink(torch.zeros(1, 3, 3, dtype=torch.float64), P.visible(3, None, 0), torch.zeros(1, dtype=torch.float64))
    assert torch.allclose(pw[0].sum(-1), torch.tensor([1 / 2, 2 / 3, 3 / 4], dtype=torch.float64))
    # retention with identity projections: o_t = sum_s decay^(t-s) (q_t . k_s) v_s
    D = 4
    eye = torch.eye(D, dtype=torch.float64)
    w = {"q": eye, "k": eye, "v": eye, "g": eye, "o": eye}
    h = torch.randn(6, D, dtype=torch.float64)
    m = {"heads": 1, "dim": D, "vdim": D, "decay": [0.5]}
    o = torch.stack([sum(0.5 ** (t - s) * (h[t] @ h[s]) * D ** -0.5 * h[s] for s in range(t + 1)) for t in range(6)])
    want = P.unit_rms(o, 1e-6) * P.silu(h)
    assert torch.allclose(P.retention(h, w, "", m, 1e-6), want)
    # the router: with corrections that lift group 1, nothing of group 0 is chosen although its plain scores are larger
    wr = {"router": torch.tensor([[3.0], [2.0], [-1.0], [-2.0]], dtype=torch.float64), "correction": torch.tensor([0.0, 0.0, 5.0, 5.0], dtype=torch.float64)}
    idx, wt = P.route(torch.ones(1, 1, dtype=torch.float64), wr, "", {"experts": 4, "top": 1, "scale": 2.0, "groups": {"count": 2, "keep": 1}})
    assert idx.tolist() == [[2]] and torch.allclose(wt, 2.0 * torch.sigmoid(torch.tensor([[-1.0]], dtype=torch.float64)))
