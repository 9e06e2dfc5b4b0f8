"""The Fakilorn decoder as data: which part sits in which layer.

A scaled token embedding without positions; a list of pre-norm layers, each an attention with
unit-RMS queries and keys, grouped key/value heads whose values may be smaller than the keys, an
output gate and values blended with those of the first blending layer, followed by a dense
squared-ReLU feed-forward, a feed-forward of routed experts, or none; a final LayerNorm; an
output head tied to the embedding table with a scale of its own.  Tensor names: ``embed``,
``l<i>.norm1`` (+ ``.b``), ``l<i>.mix.*``, ``l<i>.norm2``, ``l<i>.mlp.*``, ``final.norm``.
"""

from __future__ import annotations

from ..config.fakilorn_config import FakilornConfig
from ..config.registry import register_model
from ..parts.spec import LayerCall, LayerSpec, ModelSpec, PartSpec


def _norm(cfg: FakilornConfig, name: str, optional: bool = False) -> PartSpec:
    return PartSpec("layernorm", {"width": cfg.width, "eps": cfg.norm_eps, "bias": True, "gain_name": name,
                                  "shift_name": name + ".b", "optional": optional}, "", "norm")


@register_model("Fakilorn", "fakilorn", config_class=FakilornConfig)
def describe_fakilorn(cfg: FakilornConfig) -> ModelSpec:
    layers = []
    source_seen = False
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer.mixer
        # the first layer that blends values publishes its own; the others blend them in
        blend = None if not m.v_mix else ("blend" if source_seen else "source")
        source_seen = source_seen or m.v_mix
        parts = {
            "norm1": _norm(cfg, p + "norm1"),
            "mixer": PartSpec("gated_unit_attention", {
                "width": cfg.width, "n_head": m.heads, "n_kv_head": m.kv_heads, "head_dim": m.dim,
                "v_head_dim": m.vdim, "scale": m.scale, "eps": cfg.norm_eps, "unit_norm": True,
                "gate": True, "value_blend": blend, "blend_tensor": True}, "mix"),
        }
        arrangement = "pre_norm_mixer_only"
        if layer.mlp is None:
            # (a checkpoint may still hold the second norm of a layer without a feed-forward)
            parts["norm2"] = _norm(cfg, p + "norm2", optional=True)
        else:
            arrangement = "pre_norm"
            parts["norm2"] = _norm(cfg, p + "norm2")
            if layer.mlp.kind == "dense":
                parts["feed_forward"] = PartSpec("dense_mlp", {
                    "width": cfg.width, "inner": layer.mlp.ff, "bias": False, "activation": "relu_sq",
                    "fc_name": "up", "proj_name": "down"}, "mlp")
            else:
                parts["feed_forward"] = PartSpec("routed_experts", {
                    "width": cfg.width, "n_experts": layer.mlp.experts, "top": layer.mlp.top,
                    "inner": layer.mlp.ff, "shared_inner": layer.mlp.shared_ff, "shared_gate": True}, "mlp")
        layers.append(LayerSpec(p, parts, arrangement))
    return ModelSpec(
        architecture=cfg.architecture,
        width=cfg.width,
        vocab_size=cfg.vocab,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "width": cfg.width,
                                               "scale": cfg.embedding_scale, "tensor_name": "embed"}, ""),
        position=PartSpec("none", {}, ""),
        layers=tuple(layers),
        layer_order=tuple(LayerCall(i, i) for i in range(len(layers))),
        final_norm=_norm(cfg, "final.norm"),
        head=PartSpec("tied_head", {"vocab_size": cfg.vocab, "width": cfg.width, "tied_to": "embed",
                                    "scale": cfg.logit_scale, "stored_again": False}, "head"))
