"""Host-side pieces of the Kupelix architecture: configuration, run order, manifest, and the plain implementation's
own consistency (no GPU)."""
import copy

import numpy as np
import pytest
import torch

import kupelix_models as M
import plain_kupelix as P
from rustingstrata_b200.config import ConfigError, resolve_architecture
from rustingstrata_b200.config.kupelix_config import KupelixConfig
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
    assert isinstance(c, KupelixConfig) and (c.vocab, c.width, c.eps, c.logit_scale, c.loop) == (211, 96, 1e-6, 0.25, (1, 4, 3))
    spec = arch.build_spec(c)
    a = spec.layers[1].parts["mixer"].params
    assert (a["n_heads"], a["n_kv_heads"], a["dim"], a["vdim"], a["scale"], a["eps"]) == (6, 2, 24, 40, 24 ** -0.5, 1e-6)
    assert spec.layers[1].parts["mixer_position"].params == {
        "n_rot": 8, "base": 5000.0, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64.0}}
    assert spec.layers[3].parts["mixer_position"].params["scaling"] is None
    d = spec.layers[4].parts["mixer"].params
    assert (d["n_heads"], d["n_qk_heads"], d["dim"], d["vdim"], d["taps"], d["decay_rank"], d["gate_rank"]) == (2, 2, 40, 12, 2, 7, 9)
    h = spec.layers[0].parts["mixer"].params
    assert (h["n_heads"], h["dim"], h["vdim"]) == (3, 24, 20)
    assert "feed_forward" not in spec.layers[2].parts
    assert spec.layers[0].parts["feed_forward"].params == {"hidden": 96, "intermediate": 160, "activation": "xielu"}
    assert spec.head.params["scale"] == 0.25
    q = arch.build_spec(arch.config_class.from_dict(M.CONFIGS["Q"]))
    assert "mixer_position" not in q.layers[0].parts and q.head.params["scale"] == 1.0


def test_inner_widths_of_the_low_rank_maps_come_from_the_tensors():
    cfg = copy.deepcopy(M.CONFIGS["P"])
    for L in cfg["layers"]:
        L["mixer"].pop("decay_rank", None)
        L["mixer"].pop("gate_rank", None)
    c = KupelixConfig.from_dict(cfg)
    assert c.layers[4].mixer.decay_rank is None
    c = c.resolve_shapes({"l4.mix.a1": (7, 96), "l4.mix.g1": (9, 96), "l2.mix.a1": (5, 96), "l2.mix.g1": (3, 96)})
    assert (c.layers[4].mixer.decay_rank, c.layers[4].mixer.gate_rank) == (7, 9)
    assert (c.layers[2].mixer.decay_rank, c.layers[2].mixer.gate_rank) == (5, 3)


def test_run_order_of_a_loop():
    """Layers before the loop once, the looped layers ``times`` times, each pass behind a re-entry, then the rest;
    every entry of the order is a call of its own (own cache and state)."""
    cfg = M.CONFIGS["P"]
    arch = resolve_architecture(cfg)
    spec = arch.build_spec(arch.config_class.from_dict(cfg))
    kinds = [(spec.layers[c.layer].block.kind, c.layer) for c in spec.order]
    want = [("parallel", 0)]
    for _ in range(3):
        want += [("stream_reentry", 5), ("parallel", 1), ("parallel", 2), ("parallel", 3)]
    want += [("parallel", 4)]
    assert kinds == want and all(c.cache is None for c in spec.order)
    assert [li for li, _ in P.run_order(cfg)] == [k[1] for k in kinds if k[0] == "parallel"]
    # without a loop there is no re-entry and no tensor for it
    q = arch.build_spec(arch.config_class.from_dict(M.CONFIGS["Q"]))
    assert [spec_l.block.kind for spec_l in q.layers] == ["parallel"] * 3 and "loop.in" not in manifest_for(M.CONFIGS["Q"])


@pytest.mark.parametrize("bad", [
    lambda c: c.pop("norm"), lambda c: c["layers"][0].update(type="conv"), lambda c: c["loop"].update(stop=9),
    lambda c: c["layers"][1]["mixer"]["rot"].update(dims=9), lambda c: c["layers"][1]["mixer"].update(kv_heads=4),
    lambda c: c["layers"][2]["mixer"].pop("conv"), lambda c: c["layers"][0]["mlp"].update(kind="routed"),
    lambda c: c["layers"][1]["mixer"]["rot"]["scaling"].update(high=1.0), lambda c: c.pop("vocab")])
def test_bad_configurations_are_refused_with_a_sentence(bad):
    c = copy.deepcopy(M.CONFIGS["P"])
    bad(c)
    with pytest.raises(ConfigError):
        KupelixConfig.from_dict(c)


# ----------------------------------------------------------------------------- the plain implementation against itself
def test_plain_recurrences_agree_with_their_unrolled_sums():
    """HGRN2's state is a decayed sum of gated writes; after t steps row i of S holds sum_s (prod_{r>s} f_r[i]) (1 - f_s[i]) v_s."""
    cfg = M.config(50, 32, [(M.hgrn2(2, 8, 6), None)])
    w = M.draw_weights(cfg, 1)
    h = torch.from_numpy(np.random.default_rng(0).standard_normal((9, 32)))
    m = cfg["layers"][0]["mixer"]
    got = P.hgrn2(h, w, "l0.mix.", m, 1e-6)
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    q = P.silu(h @ w["l0.mix.q"].T).reshape(9, H, dk)
    v = (h @ w["l0.mix.v"].T).reshape(9, H, dv)
    lo = w["l0.mix.lower"]
    f = (lo + (1 - lo) * torch.sigmoid(h @ w["l0.mix.f"].T + w["l0.mix.f.b"])).reshape(9, H, dk)
    o = torch.zeros(9, H, dv, dtype=torch.float64)
    for t in range(9):
        for s in range(t + 1):
            keep = torch.prod(f[s + 1:t + 1], dim=0)                       # [H, dk]
            o[t] += torch.einsum("hi,hj->hj", q[t] * keep * (1 - f[s]), v[s])
    o = o / torch.sqrt((o ** 2).mean(-1, keepdim=True) + 1e-6) * w["l0.mix.norm"]
    want = o.reshape(9, H * dv) @ w["l0.mix.o"].T
    assert torch.allclose(got, want, atol=1e-10)


def test_plain_attention_weights_and_sink_sum_to_one():
    """With values of all ones and no gate the output of a head is 1 - (the sink's share), below one and the same in
    every channel; a very low sink gives one."""
    cfg = M.config(50, 32, [(M.attention(2, 1, 8, 4, rot_dims=4), None)])
    w = M.draw_weights(cfg, 2)
    m = cfg["layers"][0]["mixer"]
    w["l0.mix.v"] = torch.zeros_like(w["l0.mix.v"])
    w["l0.mix.v.b"] = torch.ones_like(w["l0.mix.v.b"])
    w["l0.mix.g"] = torch.zeros_like(w["l0.mix.g"])                        # every gate one half
    w["l0.mix.o"] = torch.eye(32, 8, dtype=torch.float64)                # the first eight outputs are the heads themselves
    h = torch.from_numpy(np.random.default_rng(0).standard_normal((7, 32)))
    out = P.attention(h, w, "l0.mix.", m, 1e-6)[:, :8] * 2
    assert torch.all(out < 1.0) and torch.all(out > 0.0)
    assert torch.allclose(out[:, :4], out[:, :1].expand(-1, 4)) and torch.allclose(out[:, 4:8], out[:, 4:5].expand(-1, 4))
    w["l0.mix.sink"] = torch.full_like(w["l0.mix.sink"], -80.0)
    out = P.attention(h, w, "l0.mix.", m, 1e-6)[:, :8] * 2
    assert torch.allclose(out, torch.ones_like(out))


def test_plain_rotation_scales_long_wavelengths_only():
    rot = {"base": 100.0, "dims": 8, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}}
    f = P.rotary_frequencies(rot).numpy()
    raw = 100.0 ** (-np.arange(4) * 2 / 8)
    wl = 2 * np.pi / raw
    for i in range(4):
        if wl[i] < 64 / 4.0:
            assert np.isclose(f[i], raw[i])
        elif wl[i] > 64 / 1.0:
            assert np.isclose(f[i], raw[i] / 4.0)
        else:
            assert raw[i] / 4.0 < f[i] < raw[i]
    assert np.allclose(P.rotary_frequencies({"base": 100.0, "dims": 8}).numpy(), raw)
