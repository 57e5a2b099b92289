"""The Pozozen design as a plan of parts.

A decoder with several copies of the residual stream that every sublayer reads as a weighted sum through a layer norm
(weight and bias) and writes back into while the copies are mixed (arrangement ``streamed_pre_norm``).  Each layer
names its mixer -- ``mlstm`` (a matrix memory with exponential gating) or ``parallel`` (windowed grouped-query softmax
attention without positions beside a selective state-space recurrence, added with fixed factors) -- and its
feed-forward: routed SwiGLU experts with softmax scores, a selection-only correction, groups judged by their best
expert, identity experts and a shared expert, or none.  A stretch of layers may run several times in a row with the
same weights; every pass has its own cache and state.  Tensor names: ``embed``, ``l<i>.norm1|norm2`` (bias: ``.b``),
``l<i>.hc1|hc2.in|out|mix``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``, ``head``.
"""
from __future__ import annotations

from ..config.base import ArchEntry, register_arch
from ..config.pozozen import MLstmConfig, ParallelConfig, PozozenConfig, RoutedFfConfig
from ..parts.base import LayerCall, LayerSpec, ModelPlan, PartSpec

# no position enters any score: nothing in the design bounds a context
MAX_POSITIONS = 1 << 30


def _mixer(cfg: PozozenConfig, m) -> PartSpec:
    if isinstance(m, MLstmConfig):
        return PartSpec("mlstm", {"hidden": cfg.width, "n_heads": m.heads, "dim": m.dim, "v_dim": m.vdim,
                                  "gate_cap": m.gate_cap, "eps": cfg.eps})
    if isinstance(m, ParallelConfig):
        l, r = m.left, m.right
        left = PartSpec("attention", {
            "hidden": cfg.width, "n_heads": l.heads, "n_kv_heads": l.kv_heads, "head_dim": l.dim, "v_dim": l.vdim,
            "qkv_bias": True, "window": l.window, "softmax_scale": l.scale, "position": PartSpec("none"),
            "names": {"q": "q", "k": "k", "v": "v", "o": "o", "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b"}})
        right = PartSpec("state_space", {"hidden": cfg.width, "n_heads": r.heads, "v_dim": r.vdim, "state": r.state,
                                         "groups": r.groups, "taps": r.conv, "norm_groups": r.norm_groups, "eps": cfg.eps})
        return PartSpec("parallel", {"branches": (("left", left, m.left_scale), ("right", right, m.right_scale))})
    raise TypeError(m)


def _feed_forward(cfg: PozozenConfig, f) -> PartSpec:
    if f is None:
        return PartSpec("none")
    if isinstance(f, RoutedFfConfig):
        return PartSpec("sparse_moe", {
            "hidden": cfg.width, "n_experts": f.experts, "n_identity": f.identity, "top_k": f.top, "norm_topk": True,
            "expert_intermediate": f.expert_ff, "shared_intermediate": f.shared_ff, "shared_gate": False,
            "selection_bias": True, "n_group": f.group_count, "n_group_used": f.group_keep, "group_score": "best",
            "names": {"router": "router", "selection_bias": "correction", "expert_gate": "e{e}.gate",
                      "expert_up": "e{e}.up", "expert_down": "e{e}.down", "shared": "shared"},
            "shared_names": {"gate": "gate", "up": "up", "down": "down"}})
    raise TypeError(f)


def build_plan(cfg: PozozenConfig) -> ModelPlan:
    S = max(cfg.streams, 1)
    norm = PartSpec("layernorm", {"width": cfg.width, "eps": cfg.eps})
    arrangement = PartSpec("streamed_pre_norm", {"hidden": cfg.width, "streams": cfg.streams, "mult": cfg.residual_mult})
    layers = [LayerSpec(prefix=f"l{i}", arrangement=arrangement, norm=norm, mixer=_mixer(cfg, layer.mixer),
                        feed_forward=_feed_forward(cfg, layer.mlp))
              for i, layer in enumerate(cfg.layers)]
    return ModelPlan(
        architecture=cfg.architecture, hidden_size=cfg.width, vocab_size=cfg.vocab, max_positions=MAX_POSITIONS,
        eos_token_id=-1,
        embedding=PartSpec("embedding", {"vocab": cfg.vocab, "hidden": cfg.width, "prefix": "embed", "tensor": "embed",
                                         "copies": S}),
        layers=layers, order=[LayerCall(i) for i in cfg.run_order()],
        # the final norm reads the plain sum of the streams
        final_norm=PartSpec("layernorm", {"width": cfg.width, "eps": cfg.eps, "streams": S, "prefix": "final.norm",
                                          "tensor": "final.norm", "bias_tensor": "final.norm.b"}),
        head=PartSpec("linear", {"vocab": cfg.vocab, "hidden": cfg.width, "prefix": "head", "tensor": "head"}),
        config=cfg, residual_streams=S,
    )


register_arch(ArchEntry(
    name="Pozozen",
    description="Pozozen: pre-norm sublayers (layer norm with bias) over several mixed copies of the residual stream; "
                "mLSTM matrix memory and windowed grouped-query attention beside a Mamba-2 state-space recurrence as "
                "mixers; routed SwiGLU experts with a selection correction, expert groups, identity experts and a shared "
                "expert; a stretch of layers may run several times",
    parse_config=PozozenConfig.from_dict,
    build_plan=build_plan,
))
