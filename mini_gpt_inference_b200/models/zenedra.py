"""The Zenedra decoder as data: which part sits in which layer, and in which order layers run.

Token embedding plus a hashed token-pair embedding plus learned positions; pre-norm layers
(RMS norms with gains stored around zero) whose mixer is gated linear attention, attention over
blocks of positions with a distance bias and values that are the keys, or an mLSTM matrix memory,
and whose feed-forward is a gated tanh-GELU unit, routed clamped experts with a shared one, or
none; a range of layers that runs several times with the same weights, every pass with a cache
or state of its own and a re-entry step in front of it; a final RMS norm and an untied head.
Tensor names: ``embed``, ``bigram``, ``pos``, ``loop.in``, ``loop.step``, ``l<i>.norm1``,
``l<i>.mix.*``, ``l<i>.norm2``, ``l<i>.mlp.*``, ``final.norm``, ``head``.
"""

from __future__ import annotations

from ..config.registry import register_model
from ..config.zenedra_config import ZenedraConfig
from ..parts.spec import LayerCall, LayerSpec, ModelSpec, PartSpec

SLOPE_RATE = 8.0        # head h of H takes slope 2^(-8 (h + 1) / H) off a score per position of distance


def _norm(cfg: ZenedraConfig, name: str, optional: bool = False) -> PartSpec:
    return PartSpec("rmsnorm", {"width": cfg.width, "eps": cfg.norm_eps, "offset": 1.0, "weight_name": name,
                                "optional": optional}, "", "norm")


def _mixer(cfg: ZenedraConfig, m) -> PartSpec:
    if m.kind == "gla":
        return PartSpec("gated_linear_attention", {"width": cfg.width, "n_head": m.heads, "head_dim": m.dim,
                                                   "v_head_dim": m.vdim, "tau": m.tau, "eps": cfg.norm_eps}, "mix")
    if m.kind == "mlstm":
        return PartSpec("mlstm", {"width": cfg.width, "n_head": m.heads, "head_dim": m.dim, "v_head_dim": m.vdim,
                                  "gate_cap": m.gate_cap, "eps": cfg.norm_eps}, "mix")
    return PartSpec("gated_unit_attention", {
        "width": cfg.width, "n_head": m.heads, "n_kv_head": m.kv_heads, "head_dim": m.dim, "v_head_dim": m.vdim,
        "scale": m.scale, "eps": cfg.norm_eps, "unit_norm": True, "norm_weights": True, "gate": False, "bias": True,
        "values": "keys", "slope_rate": SLOPE_RATE, "block_mask": m.mask_size, "init": "fan_in"}, "mix")


def _feed_forward(cfg: ZenedraConfig, f) -> PartSpec:
    if f.kind == "dense":
        return PartSpec("gated_mlp", {"width": cfg.width, "inner": f.ff, "activation": "gelu_tanh"}, "mlp")
    return PartSpec("routed_experts", {
        "width": cfg.width, "n_experts": f.experts, "top": f.top, "inner": f.ff, "shared_inner": f.shared_ff,
        "shared_gate": False, "scoring": "sigmoid", "route_scale": f.route_scale, "correction": True,
        "groups": None if f.group_count is None else (f.group_count, f.group_keep),
        "activation": "clamped_swish", "limit": f.limit, "shared_limit": f.shared_limit, "init": "fan_in"}, "mlp")


@register_model("Zenedra", "zenedra", config_class=ZenedraConfig)
def describe_zenedra(cfg: ZenedraConfig) -> ModelSpec:
    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        parts = {"norm1": _norm(cfg, p + "norm1"), "mixer": _mixer(cfg, layer.mixer)}
        arrangement = "pre_norm_mixer_only"
        if layer.mlp is None:
            # (a checkpoint may still hold the second norm of a layer without a feed-forward)
            parts["norm2"] = _norm(cfg, p + "norm2", optional=True)
        else:
            arrangement = "pre_norm"
            parts["norm2"] = _norm(cfg, p + "norm2")
            parts["feed_forward"] = _feed_forward(cfg, layer.mlp)
        layers.append(LayerSpec(p, parts, arrangement))
    # every run of a layer has a cache entry of its own; a pass of the loop begins with the re-entry step
    order = []
    for n, (i, loop_pass) in enumerate(cfg.run_order()):
        begins = loop_pass is not None and i == cfg.loop_start
        order.append(LayerCall(i, n, True, 0 if begins else None, loop_pass if begins else 0))
    entries = ()
    if cfg.loop_times:
        entries = (PartSpec("embedding_reentry", {"width": cfg.width, "passes": cfg.loop_times}, "loop"),)
    return ModelSpec(
        architecture=cfg.architecture,
        width=cfg.width,
        vocab_size=cfg.vocab,
        embedding=PartSpec("hashed_pair_embedding", {
            "vocab_size": cfg.vocab, "width": cfg.width, "buckets": cfg.bigram_buckets,
            "mul_prev": cfg.bigram_mul_prev, "mul_cur": cfg.bigram_mul_cur, "tensor_name": "embed",
            "pair_name": "bigram"}, ""),
        position=PartSpec("learned_absolute", {"n_positions": cfg.max_positions, "width": cfg.width,
                                               "tensor_name": "pos"}, ""),
        layers=tuple(layers),
        layer_order=tuple(order),
        final_norm=_norm(cfg, "final.norm"),
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "width": cfg.width, "tensor_name": "head"}, ""),
        n_caches=len(order),
        entries=entries)
