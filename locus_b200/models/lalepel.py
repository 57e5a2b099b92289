"""The Lalepel design as a plan of parts.

A decoder whose sublayers read the residual stream itself and whose outputs are normed before they are added
(arrangement ``output_norm``).  Each layer names its mixer -- ``latent_attention`` (low-rank query and key/value
latents, one rotated key part for all heads, interleaved rotary pairs with a long-context frequency ramp, a
sliding window, a sink per head in the softmax) or ``retention`` (a linear recurrence with a fixed decay per
head) -- and its feed-forward: a dense SwiGLU layer, routed experts of the form down(max(up h, 0)^2) with a router
bias, softmax weights over the picked logits and a sigmoid-gated shared expert, or none.  Tensor names: ``embed``,
``l<i>.norm1|norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``, ``head``.
"""
from __future__ import annotations

from ..config.base import ArchEntry, register_arch
from ..config.lalepel import (DenseFfConfig, LalepelConfig, LatentAttentionConfig, MoeFfConfig, RetentionConfig)
from ..parts.base import LayerCall, LayerSpec, ModelPlan, PartSpec

# positions are int32 and angles are formed in float64: nothing in the design bounds a context
MAX_POSITIONS = 1 << 30


def _mixer(cfg: LalepelConfig, m) -> PartSpec:
    if isinstance(m, LatentAttentionConfig):
        position = PartSpec("none")
        if m.rot_dims > 0:
            sc = m.rot_scaling
            position = PartSpec("rotary", {
                "head_dim": m.rot_dim, "theta": m.rot_base, "rot_dim": m.rot_dims, "interleaved": True,
                "scaling": None if sc is None else {"factor": sc.factor, "original": sc.original, "fast": sc.fast,
                                                    "slow": sc.slow}})
        return PartSpec("latent_attention", {
            "hidden": cfg.width, "n_heads": m.heads, "nope_dim": m.dim, "rot_dim": m.rot_dim, "v_dim": m.vdim,
            "q_rank": m.q_rank, "kv_rank": m.kv_rank, "scale": m.scale, "eps": cfg.eps, "window": m.window,
            "sink": True, "position": position})
    if isinstance(m, RetentionConfig):
        return PartSpec("retention", {"hidden": cfg.width, "n_heads": m.heads, "dim": m.dim, "v_dim": m.vdim,
                                      "decay": m.decay, "eps": cfg.eps})
    raise TypeError(m)


def _feed_forward(cfg: LalepelConfig, f) -> PartSpec:
    if f is None:
        return PartSpec("none")
    if isinstance(f, DenseFfConfig):
        return PartSpec("dense_mlp", {"hidden": cfg.width, "intermediate": f.ff,
                                      "names": {"gate": "gate", "up": "up", "down": "down"}})
    if isinstance(f, MoeFfConfig):
        return PartSpec("sparse_moe", {
            "hidden": cfg.width, "n_experts": f.experts, "top_k": f.top, "norm_topk": True,
            "expert_intermediate": f.expert_ff, "shared_intermediate": f.shared_ff, "shared_gate": True,
            "activation": "relu2", "router_bias": True,
            "names": {"router": "router", "router_bias": "router.b", "expert_up": "e{e}.up", "expert_down": "e{e}.down",
                      "shared": "shared", "shared_gate": "shared.sg"},
            "shared_names": {"up": "up", "down": "down"}})
    raise TypeError(f)


def build_plan(cfg: LalepelConfig) -> ModelPlan:
    norm = PartSpec("rmsnorm", {"width": cfg.width, "eps": cfg.eps})
    layers = [LayerSpec(prefix=f"l{i}", arrangement=PartSpec("output_norm", {"hidden": cfg.width}), norm=norm,
                        mixer=_mixer(cfg, layer.mixer), feed_forward=_feed_forward(cfg, layer.mlp))
              for i, layer in enumerate(cfg.layers)]
    return ModelPlan(
        architecture=cfg.architecture, hidden_size=cfg.width, vocab_size=cfg.vocab, max_positions=MAX_POSITIONS,
        eos_token_id=-1,
        embedding=PartSpec("embedding", {"vocab": cfg.vocab, "hidden": cfg.width, "prefix": "embed", "tensor": "embed"}),
        layers=layers, order=[LayerCall(i) for i in range(len(layers))],
        final_norm=PartSpec("rmsnorm", {"width": cfg.width, "eps": cfg.eps, "prefix": "final.norm", "tensor": "final.norm"}),
        head=PartSpec("linear", {"vocab": cfg.vocab, "hidden": cfg.width, "prefix": "head", "tensor": "head"}),
        config=cfg,
    )


register_arch(ArchEntry(
    name="Lalepel",
    description="Lalepel: sublayers normed on their output; latent attention (low-rank latents, shared rotated key "
                "part, ramped rotary frequencies, sliding window, softmax sink) and retention (linear recurrence "
                "with a fixed decay per head) mixers; dense SwiGLU or routed squared-ReLU experts with a router "
                "bias and a gated shared expert",
    parse_config=LalepelConfig.from_dict,
    build_plan=build_plan,
))
