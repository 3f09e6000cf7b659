"""Kozasun: a decoder over several residual streams that mixes chunked attention, retention and windowed latent
attention in any order, with dense or routed feed-forwards, as a description in parts.

* Embedding ``table_sum`` with a scale on the token row, copied into every stream.
* Every layer is a ``hyper_connection`` block with ``layernorm`` norms (weight and bias).
* Mixers: ``talking_attention`` without the mix and the gate (biased projections, one RMS norm over the whole q row and
  one over the whole k row, a rotated prefix of every head with halves paired, keys of the query's own block only, a
  sink in the denominator); ``retention`` (a fixed decay per head over a float32 state matrix, read-out norm, SiLU
  gate); ``latent_attention`` without rotated parts (a sliding window, a sigmoid gate per head).
* Feed-forwards: ``gated_mlp`` with the tanh form of GELU; ``routed_moe`` with sigmoid scores, a correction that steers
  the choice only, groups of experts, scaled weights that are not renormalised, SiLU-gated experts and a shared one.
* ``weights_of: j``: the layer is one more entry of the run order that names layer j (every entry owns its cache or
  state).
* Tensor names: embed, head, final.norm(.b), and per layer l<i>.{norm1(.b), norm2(.b), hc1.{in,out,mix},
  hc2.{in,out,mix}, mix.*, mlp.*}.
"""
from __future__ import annotations

from ..config.kozasun_config import ATTENTION, LATENT_ATTENTION, RETENTION, DenseConfig, KozasunConfig
from ..config.registry import register_architecture
from ..parts.spec import LayerCall, LayerSpec, ModelSpec, PartSpec


def build_kozasun_spec(cfg: KozasunConfig) -> ModelSpec:
    D = cfg.width
    S = cfg.streams or 1
    norm = lambda name, streams=1: PartSpec("layernorm", {"width": D, "eps": cfg.eps, "streams": streams},       # noqa: E731
                                            {"weight": name, "bias": name + ".b"})
    rope = lambda rot: PartSpec("rope_neox", {"n_rot": rot.dims, "base": rot.base, "base_bits": 64})             # noqa: E731
    layers, index, order = [], {}, []
    for i, L in enumerate(cfg.layers):
        # tensors: the layer's own, or those of the layer it names.  An entry that equals the named layer's is one more
        # call of that layer; one that differs in a constant (a mask's size, say) is a layer of its own on the same tensors.
        owner = i if L.weights_of is None else L.weights_of
        same = next((k for k, (o, other) in enumerate(index.get(owner, [])) if (other.type, other.mixer, other.mlp) ==
                     (L.type, L.mixer, L.mlp)), None)
        if same is not None:
            order.append(LayerCall(index[owner][same][0]))
            continue
        p = f"l{owner}."
        m = L.mixer
        parts = {"mixer_norm": norm(p + "norm1")}
        if L.type == ATTENTION:
            parts["mixer"] = PartSpec("talking_attention", {
                "hidden": D, "n_heads": m.heads, "n_kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale,
                "eps": cfg.eps, "window": None, "chunk": m.chunk, "bias": True, "qk_norm": True, "norm": "row", "talk": False,
                "sink": True, "gate": False}, {
                "q_proj": p + "mix.q", "k_proj": p + "mix.k", "v_proj": p + "mix.v", "o_proj": p + "mix.o",
                "q_bias": p + "mix.q.b", "k_bias": p + "mix.k.b", "v_bias": p + "mix.v.b", "q_norm": p + "mix.q.norm",
                "k_norm": p + "mix.k.norm", "sink": p + "mix.sink"})
            if m.rot is not None:
                parts["mixer_position"] = rope(m.rot)
        elif L.type == RETENTION:
            parts["mixer"] = PartSpec("retention", {"hidden": D, "n_heads": m.heads, "dim": m.dim, "vdim": m.vdim,
                                                    "decay": m.decay, "eps": cfg.eps, "gate": True}, {
                "q_proj": p + "mix.q", "k_proj": p + "mix.k", "v_proj": p + "mix.v", "g_proj": p + "mix.g", "o_proj": p + "mix.o"})
            if m.rot is not None:
                parts["mixer_position"] = rope(m.rot)
        elif L.type == LATENT_ATTENTION:
            parts["mixer"] = PartSpec("latent_attention", {
                "hidden": D, "n_heads": m.heads, "dim": m.dim, "rot_dim": 0, "vdim": m.vdim, "kv_rank": m.kv_rank,
                "scale": m.scale, "eps": cfg.eps, "window": m.window, "gate": True, "weights_bits": 32}, {
                "q_proj": p + "mix.q", "dkv_proj": p + "mix.dkv", "latent_norm": p + "mix.dkv.norm", "uk_proj": p + "mix.uk",
                "uv_proj": p + "mix.uv", "g_proj": p + "mix.g", "o_proj": p + "mix.o"})
        else:
            raise ValueError(f"layer {i}: unknown type {L.type!r}")
        block_tensors = {}
        if cfg.streams is not None:
            block_tensors.update(mixer_in=p + "hc1.in", mixer_out=p + "hc1.out", mixer_mix=p + "hc1.mix")
        ff = L.mlp
        if ff is not None:
            parts["feed_forward_norm"] = norm(p + "norm2")
            if isinstance(ff, DenseConfig):
                parts["feed_forward"] = PartSpec("gated_mlp", {"hidden": D, "intermediate": ff.ff, "activation": "gelu_tanh"},
                                                 {"gate_proj": p + "mlp.gate", "up_proj": p + "mlp.up", "down_proj": p + "mlp.down"})
            else:
                t = {"router": p + "mlp.router", "correction": p + "mlp.correction", "expert_gate": p + "mlp.e{e}.gate",
                     "expert_up": p + "mlp.e{e}.up", "expert_down": p + "mlp.e{e}.down"}
                if ff.shared_ff:
                    t.update(shared_gate=p + "mlp.shared.gate", shared_up=p + "mlp.shared.up", shared_down=p + "mlp.shared.down")
                parts["feed_forward"] = PartSpec("routed_moe", {
                    "hidden": D, "experts": ff.experts, "top": ff.top, "expert_ff": ff.expert_ff, "shared_ff": ff.shared_ff,
                    "correction": True, "score": "sigmoid", "groups": ff.groups[0] if ff.groups else 0,
                    "keep": ff.groups[1] if ff.groups else 0, "route_scale": ff.route_scale, "renormalize": False,
                    "expert": "gated_silu"}, t)
            if cfg.streams is not None:
                block_tensors.update(ff_in=p + "hc2.in", ff_out=p + "hc2.out", ff_mix=p + "hc2.mix")
        index.setdefault(owner, []).append((len(layers), L))
        order.append(LayerCall(len(layers)))
        layers.append(LayerSpec(PartSpec("hyper_connection", {"hidden": D, "streams": S}, block_tensors), parts))
    return ModelSpec(
        name="kozasun", vocab_size=cfg.vocab, hidden_size=D, max_positions=cfg.max_positions,
        embedding=PartSpec("table_sum", {"vocab": cfg.vocab, "width": D, "copies": S, "scale": cfg.embedding_scale,
                                         "bigram": None, "positions": 0}, {"weight": "embed"}),
        layers=tuple(layers), order=tuple(order), final_norm=norm("final.norm", S),
        head=PartSpec("linear", {"vocab": cfg.vocab, "width": D}, {"weight": "head"}), n_streams=S)


register_architecture("Kozasun", KozasunConfig, build_kozasun_spec, aliases=("kozasun",), replace=True)
