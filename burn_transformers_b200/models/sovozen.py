"""Sovozen as a plan of parts: pre-LayerNorm layers whose mixer is either attention over a low-rank latent (with a
rotated shared key part, a sink in the softmax and an output gate; some layers read an earlier layer's latent) or
linear attention with a per-head decay, a gated feed-forward where a layer has one, a scaled embedding and a scaled,
untied readout.

Checkpoint names: `embed`, `l<i>.norm1`, `l<i>.norm2`, `l<i>.mix.*`, `l<i>.mlp.*`, `final.norm`, `head`; matrices are
stored [out, in].  The projections that read the same input are one product here: their rows are laid end to end when
the weights are loaded (weights.spec.Concat).
"""
from __future__ import annotations

import math

from ..config.registry import Architecture, register_architecture
from ..config.sovozen import SovozenConfig
from ..engine.model import UNBOUNDED_CONTEXT, LayerCall, ModelPlan
from ..parts import (GatedFeedForward, InterleavedRotary, LatentAttention, LayerNorm, LightningAttention, LinearReadout,
                     NoPositions, PreNormBlock, TokenEmbedding)
from ..weights.spec import Concat, Stored


def build_sovozen(config: SovozenConfig) -> ModelPlan:
    config.validate()
    width, eps = config.width, config.eps
    std = width ** -0.5
    embedding = TokenEmbedding(config.vocab, width, 1.0, scale=config.embedding_scale)
    final_norm = LayerNorm(width, eps, bias=False)
    readout = LinearReadout(config.vocab, width, config.logit_scale, init_std=std)
    names = {"embed": (embedding, "weight"), "final.norm": (final_norm, "weight"), "head": (readout, "weight")}
    sources = {}
    blocks, schedule = [], []
    for i, layer in enumerate(config.layers):
        p = f"l{i}."
        m = layer["mixer"]
        norm1 = LayerNorm(width, eps, bias=False)
        names[p + "norm1"] = (norm1, "weight")
        reads = None
        if layer["type"] == "latent_attention":
            reads = m.get("kv_from")
            rot = m.get("rot") or {"dims": 0, "base": 1.0}
            rotary = InterleavedRotary(rot["dims"], rot["base"])
            out_std = (m["heads"] * m["vdim"]) ** -0.5
            mixer = LatentAttention(width, m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["scale"], eps,
                                    rotary, owns_latent=reads is None, sink=True, init_std=std, out_init_std=out_std)
            stacked = [(p + "mix.q", mixer.q_width), (p + "mix.g", mixer.gate_width)]
            if reads is None:
                stacked.append((p + "mix.dkv", mixer.latent_width))
                names[p + "mix.dkv.norm"] = (mixer, "latent_norm.weight")
            names.update({p + "mix.uk": (mixer, "uk.weight"), p + "mix.uv": (mixer, "uv.weight"),
                          p + "mix.sink": (mixer, "sink"), p + "mix.o": (mixer, "out.weight")})
        else:
            out_std = (m["heads"] * m["vdim"]) ** -0.5
            mixer = LightningAttention(width, m["heads"], m["dim"], m["vdim"], m["decay"], eps, init_std=std,
                                       out_init_std=out_std)
            stacked = [(p + "mix.q", mixer.qk_width), (p + "mix.k", mixer.qk_width), (p + "mix.v", mixer.v_width),
                       (p + "mix.g", mixer.v_width)]
            names.update({p + "mix.norm": (mixer, "norm.weight"), p + "mix.o": (mixer, "out.weight")})
        names[p + "mix.in"] = (mixer, "in.weight")
        sources[p + "mix.in"] = Concat(tuple(Stored(name) for name, _ in stacked), 0, tuple(size for _, size in stacked))
        norm2 = feed_forward = None
        if layer.get("mlp") is not None:
            inner = layer["mlp"]["ff"]
            norm2 = LayerNorm(width, eps, bias=False)
            feed_forward = GatedFeedForward(width, inner, "gelu_new", init_std=std, down_init_std=inner ** -0.5)
            names[p + "norm2"] = (norm2, "weight")
            names[p + "mlp.gate_up"] = (feed_forward, "gate_up.weight")
            names[p + "mlp.down"] = (feed_forward, "down.weight")
            sources[p + "mlp.gate_up"] = Concat((Stored(p + "mlp.gate"), Stored(p + "mlp.up")), 0, (inner, inner))
        blocks.append(PreNormBlock(norm1, mixer, norm2, feed_forward))
        schedule.append(LayerCall(i, cache=reads))
    return ModelPlan(config=config, embedding=embedding, positions=NoPositions(), blocks=blocks, schedule=schedule,
                     final_norm=final_norm, readout=readout, names=names, vocab=config.vocab, width=width,
                     max_context=UNBOUNDED_CONTEXT, sources=sources)


SOVOZEN = register_architecture(Architecture("sovozen", SovozenConfig.MODEL_TYPES, SovozenConfig, build_sovozen),
                                replace=True)
