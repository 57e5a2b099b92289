"""Block arrangements and the parts at the two ends of the model.

``PreNorm``: x += mixer(norm1(x)); x += feed_forward(norm2(x)) -- the residual placement
of the reference's forward (src/locus/model/llama.cpp:485-509).  The residual stream x is
float32 in every mode; the normed activations have the model's element type.

``OutputNorm``: x += norm1(mixer(x)); x += norm2(feed_forward(x)): the sublayers read x itself and the
norms sit on what they give.

``Embedding``: x = table[token] (llama.cpp:450).  ``LmHead``: logits = W . h in float32,
W being the embedding table when the head is tied (llama.cpp:292-297, 512-513): the head then
names the embedding's tensor as the source of its weight.
"""
from __future__ import annotations

import torch

from .. import kernels as K
from .base import (Arrangement, Part, PartSpec, TensorSource, make_part, register_arrangement,
                   register_embedding, register_head)


class PreNorm(Arrangement):
    def __init__(self, prefix: str, *, hidden: int, norm: PartSpec, mixer: PartSpec,
                 feed_forward: PartSpec, mixer_prefix: str = "self_attn", ff_prefix: str = "mlp",
                 norm1_name: str = "input_layernorm", norm2_name: str = "post_attention_layernorm") -> None:
        super().__init__(prefix)
        self.hidden = hidden
        self.norm1 = make_part("norm", norm, f"{prefix}.{norm1_name}")
        self.mixer = make_part("mixer", mixer, f"{prefix}.{mixer_prefix}")
        self.norm2 = make_part("norm", norm, f"{prefix}.{norm2_name}")
        self.ff = make_part("feed_forward", feed_forward, f"{prefix}.{ff_prefix}")

    takes_pending_add = True

    def sub_parts(self):
        return [self.norm1, self.mixer, self.norm2, self.ff]

    def forward(self, x, batch, cache, rt) -> None:
        T = batch.T
        h = rt.rows("block.h", self.hidden, rt.dtype, T)
        self.norm1.forward(x, h, add=rt.take_pending())
        self.mixer.forward(h, batch, cache, x, rt)
        self.norm2.forward(x, h)
        self.ff.forward(h, batch, x, rt)


class OutputNorm(Arrangement):
    """Norm on a sublayer's OUTPUT only: x += norm1(mixer(x)); x += norm2(feed_forward(x)).  The sublayers read
    the residual stream itself (in a bfloat16 model: its rounding to bfloat16); what they give is collected in
    float32 rows, normed with float32 statistics and added.  ``feed_forward`` may be absent (kind "none"): the
    layer is then its mixer alone and has no second norm."""

    def __init__(self, prefix: str, *, hidden: int, norm: PartSpec, mixer: PartSpec, feed_forward: PartSpec,
                 mixer_prefix: str = "mix", ff_prefix: str = "mlp", norm1_name: str = "norm1",
                 norm2_name: str = "norm2") -> None:
        super().__init__(prefix)
        self.hidden = hidden

        def norm_part(name):
            # the norms' tensors carry the plain name of the norm (no ".weight" behind it)
            spec = PartSpec(norm.kind, {**norm.args, "tensor": f"{prefix}.{name}"})
            return make_part("norm", spec, f"{prefix}.{name}")

        self.norm1 = norm_part(norm1_name)
        self.mixer = make_part("mixer", mixer, f"{prefix}.{mixer_prefix}")
        self.ff = None if feed_forward.kind == "none" else make_part("feed_forward", feed_forward, f"{prefix}.{ff_prefix}")
        self.norm2 = norm_part(norm2_name) if self.ff is not None else None

    def sub_parts(self):
        return [self.norm1, self.mixer] + ([self.norm2, self.ff] if self.ff is not None else [])

    def _read(self, x, rt, T):
        if rt.dtype == torch.float32:
            return x
        h = rt.rows("block.h", self.hidden, rt.dtype, T)
        K.cast_rows(x, h)
        return h

    def forward(self, x, batch, cache, rt) -> None:
        T = batch.T
        rt.defer_add = False   # what a sublayer gives is normed here, at once: nothing may be left pending
        y = rt.rows("block.y", self.hidden, torch.float32, T)
        h = self._read(x, rt, T)
        if self.mixer.can_overwrite:
            self.mixer.forward(h, batch, cache, y, rt, accumulate=False)
        else:
            y.zero_()
            self.mixer.forward(h, batch, cache, y, rt)
        self.norm1.forward_add(y, x)
        if self.ff is None:
            return
        h = self._read(x, rt, T)
        if self.ff.can_overwrite:
            self.ff.forward(h, batch, y, rt, accumulate=False)
        else:
            y.zero_()
            self.ff.forward(h, batch, y, rt)
        self.norm2.forward_add(y, x)


class Embedding(Part):
    def __init__(self, prefix: str, *, vocab: int, hidden: int, tensor: str = "") -> None:
        """``tensor``: the checkpoint tensor's name where it is not ``<prefix>.weight``."""
        super().__init__(prefix)
        self.vocab, self.hidden = int(vocab), int(hidden)
        self.tensor = str(tensor or prefix + ".weight")

    def param_shapes(self):
        return {"table": (self.vocab, self.hidden)}

    def sources(self):
        return [TensorSource(self.tensor, (self.vocab, self.hidden), "table")]

    def kernel_modules(self, dtype):
        return ["elementwise"]

    def forward(self, tokens: torch.Tensor, out: torch.Tensor) -> None:
        K.embed_rows(tokens, self.params["table"], out)


class LmHead(Part):
    """``tied_to``: the checkpoint tensor that is the head's weight when the head has none of its own
    (the embedding table of a tied model); two parts that name the same tensor share one device copy."""

    def __init__(self, prefix: str, *, vocab: int, hidden: int, tied_to: str = "", tensor: str = "") -> None:
        super().__init__(prefix)
        self.vocab, self.hidden, self.tied_to = int(vocab), int(hidden), str(tied_to or "")
        self.tensor = str(tensor or prefix + ".weight")   # the head's own tensor, when it is not tied

    def param_shapes(self):
        return {"weight": (self.vocab, self.hidden)}

    def sources(self):
        return [TensorSource(self.tied_to or self.tensor, (self.vocab, self.hidden), "weight")]

    def kernel_modules(self, dtype):
        return ["gemm_simt", "gemv"] + (["gemm_skinny", "gemm_tc"] if dtype == torch.bfloat16 else [])

    def forward(self, h: torch.Tensor, logits: torch.Tensor) -> None:
        K.linear(h, self.params["weight"], logits)


register_arrangement("pre_norm", PreNorm)
register_arrangement("output_norm", OutputNorm)
register_embedding("embedding", Embedding)
register_head("linear", LmHead)
