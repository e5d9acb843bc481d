"""Mufevik as data: which parts, with which constants, under which tensor names.

Tensor names: ``embed``, ``head``, ``final.norm`` (one number), and per layer ``l<i>.``: ``norm1``, ``norm2`` (one number
each), ``hc1.*`` / ``hc2.*`` (in, out, mix) when the model carries several residual streams, ``mix.*`` and ``mlp.*``.
Without ``streams`` in the configuration the layers are plain pre-norm residual layers over one stream.
"""
from __future__ import annotations

from dataclasses import replace

from ..config.mufevik import DeltaMixer, MufevikConfig, ParallelMixer
from ..parts.base import LayerSpec, ModelSpec, PartSpec, default_schedule

LAYER_NAMES = {"mixer_norm": "norm1", "feed_forward_norm": "norm2", "mixer": "mix.", "feed_forward": "mlp.",
               "hyper1": "hc1.", "hyper2": "hc2."}
DEFAULT_DECAY_RANK = 32          # when neither the configuration nor a checkpoint gives it (random weights)


def decay_rank(side) -> int:
    return side.rank or DEFAULT_DECAY_RANK


def fit_config_to_checkpoint(cfg: MufevikConfig, shapes) -> MufevikConfig:
    """The rank of the decay's first projection is a size only its tensor gives: ``l<i>.mix.right.a1`` is [rank, width]."""
    layers = []
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        shape = shapes.get(f"l{i}.mix.right.a1")
        if isinstance(m, ParallelMixer) and not m.right.rank and shape is not None and len(shape) == 2:
            layer = replace(layer, mixer=replace(m, right=replace(m.right, rank=int(shape[0]))))
        layers.append(layer)
    return replace(cfg, layers=tuple(layers))


def model_spec(cfg: MufevikConfig) -> ModelSpec:
    norm = PartSpec("scalar_rms_norm", {"hidden_size": cfg.width, "eps": cfg.norm_eps, "weight_name": ""})
    block = PartSpec("hyper_connections", {"n_streams": cfg.streams}) if cfg.streams else PartSpec("pre_norm_residual", {})
    layers = []
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        if isinstance(m, ParallelMixer):
            l, r = m.left, m.right
            position = PartSpec("rope", {"head_dim": l.dim, "theta": l.rot_base, "rot_dim": l.rot_dims}) if l.rot_dims \
                else PartSpec("none", {})
            left = PartSpec("talking_heads_attention", {
                "hidden_size": cfg.width, "n_heads": l.heads, "n_kv_heads": l.kv_heads, "head_dim": l.dim, "value_dim": l.vdim,
                "softmax_scale": l.scale, "position": position})
            right = PartSpec("gated_linear_attention", {
                "hidden_size": cfg.width, "n_heads": r.heads, "head_dim": r.dim, "value_dim": r.vdim, "decay_rank": decay_rank(r),
                "tau": r.tau, "eps": cfg.norm_eps})
            mixer = PartSpec("parallel_mixers", {"hidden_size": cfg.width, "left": left, "right": right, "eps": cfg.norm_eps})
        elif isinstance(m, DeltaMixer):
            mixer = PartSpec("gated_delta_rule", {
                "hidden_size": cfg.width, "n_heads": m.heads, "n_qk_heads": m.kv_heads, "head_dim": m.dim, "value_dim": m.vdim,
                "conv_taps": m.conv, "eps": cfg.norm_eps})
        else:
            raise ValueError(f"layer {i}: unknown mixer {type(m).__name__}")
        ffn = None
        if layer.mlp is not None:
            p = layer.mlp
            ffn = PartSpec("routed_experts", {"hidden_size": cfg.width, "n_experts": p.experts, "top": p.top,
                                              "expert_size": p.expert_ff, "n_groups": p.group_count, "keep_groups": p.group_keep,
                                              "shared_size": p.shared_ff})
        layers.append(LayerSpec(block=block, mixer=mixer, feed_forward=ffn, mixer_norm=norm,
                                feed_forward_norm=norm if ffn is not None else None, prefix=f"l{i}.", names=LAYER_NAMES))
    return ModelSpec(
        architecture=cfg.architecture, hidden_size=cfg.width, vocab_size=cfg.vocab,
        embedding=PartSpec("scaled_embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "scale": 1.0,
                                                "weight_name": "embed"}),
        layers=layers, schedule=default_schedule(len(layers)), final_norm=norm,
        head=PartSpec("scaled_lm_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "scale": cfg.logit_scale,
                                         "weight_name": "head"}),
        embedding_name="", final_norm_name="final.norm", head_name="", streams=cfg.streams, max_positions=0)
