"""Kupelix: a decoder of parallel layers (one norm feeds the mixer and the feed-forward, whose outputs join the stream
together) that mixes three kinds of token mixers freely and may repeat a run of layers, as a description in parts.

* Every layer is a ``parallel`` block with a ``layernorm`` norm (weight and bias).
* Mixers: ``talking_attention`` (biased projections, normed and rotated queries and keys with a wavelength-scaled
  interleaved rotation, scores mixed across heads, a sink, a gate per head), ``hgrn2`` and ``gated_delta`` (the gated
  delta rule with a decay per key channel and short convolutions).  Feed-forward: ``activation_mlp`` with xIELU, or none.
* ``loop``: layers start .. stop - 1 run ``times`` times in a row with the same weights; each pass has caches and
  state of its own (every entry of the run order owns its storage) and begins with a ``stream_reentry`` block
  x <- W_in [x ; embedding].
* The final norm is a ``layernorm``; the logits are multiplied by ``logit_scale``.
* Tensor names: embed, head, final.norm(.b), loop.in, and per layer l<i>.{norm1, norm1.b, mix.*, mlp.{up, down, act}}.
"""
from __future__ import annotations

from ..config.kupelix_config import ATTENTION, CHANNEL_DELTA, HGRN2, KupelixConfig
from ..config.registry import register_architecture
from ..parts.spec import LayerCall, LayerSpec, ModelSpec, PartSpec

DELTA_UNIT_EPS = 1e-6        # inside the root that makes the delta rule's queries and keys unit vectors
DEFAULT_LOW_RANK = 16        # inner width of the delta rule's low-rank maps when neither configuration nor checkpoint says


def build_kupelix_spec(cfg: KupelixConfig) -> ModelSpec:
    D = cfg.width
    norm = lambda name: PartSpec("layernorm", {"width": D, "eps": cfg.eps}, {"weight": name, "bias": name + ".b"})     # noqa: E731
    layers = []
    for i, L in enumerate(cfg.layers):
        p = f"l{i}."
        m = L.mixer
        parts = {"norm": norm(p + "norm1")}
        if L.type == ATTENTION:
            parts["mixer"] = PartSpec("talking_attention", {
                "hidden": D, "n_heads": m.heads, "n_kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale,
                "eps": cfg.eps, "window": None, "bias": True, "qk_norm": True, "talk": True, "sink": True, "gate": True}, {
                "q_proj": p + "mix.q", "k_proj": p + "mix.k", "v_proj": p + "mix.v", "o_proj": p + "mix.o",
                "q_bias": p + "mix.q.b", "k_bias": p + "mix.k.b", "v_bias": p + "mix.v.b", "q_norm": p + "mix.q.norm",
                "k_norm": p + "mix.k.norm", "talk": p + "mix.talk", "sink": p + "mix.sink", "g_proj": p + "mix.g"})
            if m.rot is not None:
                sc = m.rot.scaling
                parts["mixer_position"] = PartSpec("rope_interleaved", {
                    "n_rot": m.rot.dims, "base": m.rot.base,
                    "scaling": None if sc is None else {"factor": sc[0], "low": sc[1], "high": sc[2], "original": sc[3]}})
        elif L.type == HGRN2:
            parts["mixer"] = PartSpec("hgrn2", {"hidden": D, "n_heads": m.heads, "dim": m.dim, "vdim": m.vdim, "eps": cfg.eps,
                                                "f_bias": True}, {
                "q_proj": p + "mix.q", "f_proj": p + "mix.f", "f_bias": p + "mix.f.b", "lower": p + "mix.lower",
                "v_proj": p + "mix.v", "norm": p + "mix.norm", "o_proj": p + "mix.o"})
        elif L.type == CHANNEL_DELTA:
            parts["mixer"] = PartSpec("gated_delta", {
                "hidden": D, "n_heads": m.heads, "n_qk_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "taps": m.conv,
                "decay_rank": m.decay_rank or DEFAULT_LOW_RANK, "gate_rank": m.gate_rank or DEFAULT_LOW_RANK, "eps": cfg.eps,
                "unit_eps": DELTA_UNIT_EPS}, {
                "q_proj": p + "mix.q", "k_proj": p + "mix.k", "v_proj": p + "mix.v", "q_conv": p + "mix.q.conv",
                "k_conv": p + "mix.k.conv", "v_conv": p + "mix.v.conv", "b_proj": p + "mix.b", "a_log": p + "mix.A_log",
                "a1_proj": p + "mix.a1", "a2_proj": p + "mix.a2", "dt_bias": p + "mix.dt_bias", "g1_proj": p + "mix.g1",
                "g2_proj": p + "mix.g2", "norm": p + "mix.norm", "o_proj": p + "mix.o"})
        else:
            raise ValueError(f"layer {i}: unknown type {L.type!r}")
        if L.ff is not None:
            parts["feed_forward"] = PartSpec("activation_mlp", {"hidden": D, "intermediate": L.ff, "activation": "xielu"},
                                             {"up_proj": p + "mlp.up", "down_proj": p + "mlp.down", "act": p + "mlp.act"})
        layers.append(LayerSpec(PartSpec("parallel", {"hidden": D}), parts))

    n = len(cfg.layers)
    if cfg.loop is None:
        order = [LayerCall(i) for i in range(n)]
    else:
        start, stop, times = cfg.loop
        order = [LayerCall(i) for i in range(start)]
        layers.append(LayerSpec(PartSpec("stream_reentry", {"hidden": D, "vocab": cfg.vocab, "n_passes": 1, "index": 0},
                                         {"in_proj": "loop.in", "embedding": "embed"})))
        for _ in range(times):
            order.append(LayerCall(len(layers) - 1))
            order += [LayerCall(i) for i in range(start, stop)]
        order += [LayerCall(i) for i in range(stop, n)]
    return ModelSpec(
        name="kupelix", vocab_size=cfg.vocab, hidden_size=D, max_positions=cfg.max_positions,
        embedding=PartSpec("token_table", {"vocab": cfg.vocab, "width": D}, {"weight": "embed"}),
        layers=tuple(layers), order=tuple(order), final_norm=norm("final.norm"),
        head=PartSpec("linear", {"vocab": cfg.vocab, "width": D, "scale": cfg.logit_scale}, {"weight": "head"}))


register_architecture("Kupelix", KupelixConfig, build_kupelix_spec, aliases=("kupelix",), replace=True)
