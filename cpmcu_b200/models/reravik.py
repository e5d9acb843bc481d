"""Reravik as data: which parts, with which constants, under which tensor names.

Tensor names: ``embed``, ``head``, ``final.norm`` (+ ``.b``), ``loop.step``, and per layer ``l<i>.`` the four norms
``norm1``, ``norm1b``, ``norm2``, ``norm2b`` (each with a ``.b`` bias), ``shift``, ``mix.*`` and ``mlp.*``.  Every run of
a layer in the schedule, repeats included, has a cache lane of its own.
"""
from __future__ import annotations

from ..config.reravik import LatentAttentionMixer, MinGruMixer, ReravikConfig
from ..parts.base import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

LAYER_NAMES = {"mixer_norm": "norm1", "post_mixer_norm": "norm1b", "feed_forward_norm": "norm2",
               "post_feed_forward_norm": "norm2b", "mixer": "mix.", "feed_forward": "mlp.", "shift": "shift"}
MINGRU_NAMES = {"z": "z", "z_bias": "z.b", "x": "x", "x_bias": "x.b", "g": "g", "o": "o"}
LATENT_NAMES = {"dq": "dq", "dq_norm": "dq.norm", "uq": "uq", "dkv": "dkv", "dkv_norm": "dkv.norm", "uk": "uk", "uv": "uv", "o": "o"}
MLP_NAMES = {"gate": "gate", "up": "up", "down": "down"}


def model_spec(cfg: ReravikConfig) -> ModelSpec:
    norm = PartSpec("layer_norm", {"hidden_size": cfg.width, "eps": cfg.norm_eps, "weight_name": "", "bias_name": ".b"})
    block = PartSpec("sandwich_norm_shift", {"hidden_size": cfg.width, "post_norm": norm})
    layers = []
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        if isinstance(m, MinGruMixer):
            mixer = PartSpec("min_gru", {"hidden_size": cfg.width, "width": m.width, "names": MINGRU_NAMES})
        elif isinstance(m, LatentAttentionMixer):
            mixer = PartSpec("latent_attention", {
                "hidden_size": cfg.width, "n_heads": m.heads, "head_dim": m.dim, "value_dim": m.vdim, "q_rank": m.q_rank,
                "kv_rank": m.kv_rank, "softmax_scale": m.scale, "eps": cfg.norm_eps, "window": m.window, "names": LATENT_NAMES})
        else:
            raise ValueError(f"layer {i}: unknown mixer {type(m).__name__}")
        ffn = None
        if layer.mlp is not None:
            ffn = PartSpec("gated_ffn", {"hidden_size": cfg.width, "intermediate_size": layer.mlp.ff,
                                         "activation": "gelu_tanh", "names": MLP_NAMES})
        layers.append(LayerSpec(block=block, mixer=mixer, feed_forward=ffn, mixer_norm=norm,
                                feed_forward_norm=norm if ffn is not None else None, prefix=f"l{i}.", names=LAYER_NAMES))
    schedule = [ScheduleEntry(layer=i, lane=k, writes_cache=True, enters_pass=t) for k, (i, t) in enumerate(cfg.runs())]
    return ModelSpec(
        architecture=cfg.architecture, hidden_size=cfg.width, vocab_size=cfg.vocab,
        embedding=PartSpec("sinusoidal_scaled_embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.width,
                                                           "scale": cfg.embedding_scale, "base": 10000.0,
                                                           "weight_name": "embed"}),
        layers=layers, schedule=schedule, final_norm=norm,
        head=PartSpec("scaled_lm_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "scale": 1.0, "weight_name": "head"}),
        embedding_name="", final_norm_name="final.norm", head_name="",
        pass_entry=PartSpec("reinject_with_step", {"passes": cfg.loop_times, "hidden_size": cfg.width, "table_name": "step"})
        if cfg.loop_times else None,
        pass_entry_name="loop.", max_positions=0)
