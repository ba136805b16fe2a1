"""Gokezen as a plan of parts: token embedding plus a learned position vector; layers in which one RMS norm feeds a
mixer and a feed-forward side by side; the mixer itself is two side by side, a windowed softmax attention with shared
key heads and a matrix memory with exponential gates, each with a scale; the feed-forward is a gated dense one or routed
experts with a shared one; a run of layers may repeat with the same weights, every pass with a cache of its own and
opened by a learned vector; RMS norm and a readout with the embedding table.

Checkpoint names: `embed`, `pos`, `loop.step`, `l<i>.norm1`, `l<i>.mix.left.{q,k,v,o}`,
`l<i>.mix.right.{q,k,v,g,i,i.b,f,f.b,norm,o}`, `l<i>.mlp.{gate,up,down}` or `l<i>.mlp.{router,e<j>.*,shared.*}`,
`final.norm`; matrices are stored [out, in].  Projections that read the same input are one product here: their rows
are laid end to end when the weights are loaded.  The attention's heads are padded with zero channels up to a head size
its kernels take (keys and values may have different sizes in the file; zeros change neither scores nor outputs).
"""
from __future__ import annotations

from ..config.gokezen import GokezenConfig
from ..config.registry import Architecture, register_architecture
from ..engine.model import LayerCall, ModelPlan
from ..parts import (CausalSelfAttention, GatedFeedForward, LearnedPositions, MatrixMemory, ParallelBlock, RmsNorm,
                     RoutedFeedForward, SideBySideMixers, StreamVectors, TiedReadout, TokenEmbedding)
from ..weights.spec import Concat, PadBlocks, Stored


def attention_head_size(dim: int, vdim: int) -> int:
    """The head size the attention runs with: at least both sizes, a multiple of 16 (whole 16-byte pieces, and the
    tensor-core decode kernel's step), and 64 or 128 (the sizes of the tensor-core prompt kernel) when that is at most a
    third more."""
    size = -(-max(dim, vdim) // 16) * 16
    for full in (64, 128):
        if size < full <= size + size // 3:
            return full
    return size


def _padded(source, axis: int, block: int, padded: int):
    return source if block == padded else PadBlocks(source, axis, block, padded)


def build_gokezen(config: GokezenConfig) -> ModelPlan:
    config.validate()
    width, eps = config.width, config.eps
    std = width ** -0.5
    embedding = TokenEmbedding(config.vocab, width, 1.0)
    positions = LearnedPositions(config.max_positions, width, 0.1)
    final_norm = RmsNorm(width, eps)
    names = {"embed": (embedding, "weight"), "pos": (positions, "weight"), "final.norm": (final_norm, "weight")}
    sources = {}
    vectors = None
    if config.loop:
        vectors = StreamVectors(config.loop["times"], width, 0.1)
        names["loop.step"] = (vectors, "weight")
    blocks = []
    for i, layer in enumerate(config.layers):
        p = f"l{i}."
        m = layer["mixer"]
        norm = RmsNorm(width, eps)
        names[p + "norm1"] = (norm, "weight")
        # left: windowed attention; queries, keys and values are one product, [in, out] as the attention part keeps it
        c = m["left"]
        heads, kv_heads, dim, vdim = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
        size = attention_head_size(dim, vdim)
        left = CausalSelfAttention(width, heads, kv_heads, size, c["scale"], window=c["mask"]["size"], bias=False,
                                   init_std=std, out_init_std=(heads * vdim) ** -0.5, out_scale=m["left_scale"])
        names[p + "mix.left.qkv"] = (left, "qkv.weight")
        names[p + "mix.left.out"] = (left, "out.weight")
        sources[p + "mix.left.qkv"] = Concat(
            (_padded(Stored(p + "mix.left.q", transposed=True), 1, dim, size),
             _padded(Stored(p + "mix.left.k", transposed=True), 1, dim, size),
             _padded(Stored(p + "mix.left.v", transposed=True), 1, vdim, size)), 1,
            (heads * size, kv_heads * size, kv_heads * size))
        sources[p + "mix.left.out"] = _padded(Stored(p + "mix.left.o", transposed=True), 0, vdim, size)
        # right: the matrix memory; q, k, v, output gate and the two gates' rows are one product
        c = m["right"]
        right = MatrixMemory(width, c["heads"], c["dim"], c["vdim"], c["gate_cap"], eps, out_scale=m["right_scale"],
                             init_std=std, out_init_std=(c["heads"] * c["vdim"]) ** -0.5)
        r = p + "mix.right."
        names.update({r + "in": (right, "in.weight"), r + "i.b": (right, "i.bias"), r + "f.b": (right, "f.bias"),
                      r + "norm": (right, "norm.weight"), r + "o": (right, "out.weight")})
        gates = Concat((Stored(r + "i"), Stored(r + "f")), 0, (c["heads"], c["heads"]))
        sources[r + "in"] = Concat(
            (Stored(r + "q"), Stored(r + "k"), Stored(r + "v"), Stored(r + "g"),
             _padded(gates, 0, 2 * c["heads"], right.gates_width)), 0,
            (right.qk_width, right.qk_width, right.v_width, right.v_width, right.gates_width))
        mixer = SideBySideMixers(left, right)
        feed_forward = None
        mlp = layer.get("mlp")
        if mlp is not None and mlp["kind"] == "dense":
            feed_forward = _gated(names, sources, p + "mlp.", width, mlp["ff"], "gelu_new", 0.0, std)
        elif mlp is not None:
            shared = None
            if mlp.get("shared") is not None:
                shared = _gated(names, sources, p + "mlp.shared.", width, mlp["shared"]["ff"], "swish_clamp",
                                mlp["shared"]["limit"], std)
            router, inner = mlp["router"], mlp["expert"]["ff"]
            groups = router.get("groups") or {"count": 1, "keep": 1}
            n_experts = router["experts"]
            feed_forward = RoutedFeedForward(width, n_experts, router["top"], inner, activation="swish_clamp",
                                             limit=mlp["expert"]["limit"], n_groups=groups["count"], keep=groups["keep"],
                                             scale=router["scale"], shared=shared, init_std=std)
            f = p + "mlp."
            names.update({f + "router": (feed_forward, "router.weight"), f + "experts.in": (feed_forward, "in.weight"),
                          f + "experts.out": (feed_forward, "out.weight")})
            sources[f + "experts.in"] = Concat(
                tuple(Concat((Stored(f"{f}e{j}.gate"), Stored(f"{f}e{j}.up")), 0, (inner, inner)) for j in range(n_experts)),
                0, (2 * inner,) * n_experts)
            sources[f + "experts.out"] = Concat(tuple(Stored(f"{f}e{j}.down") for j in range(n_experts)), 0,
                                                (width,) * n_experts)
        blocks.append(ParallelBlock(norm, mixer, feed_forward))
    schedule = [LayerCall(i, opens=opens) for i, opens in config.run_order()]
    return ModelPlan(config=config, embedding=embedding, positions=positions, blocks=blocks, schedule=schedule,
                     final_norm=final_norm, readout=TiedReadout(embedding), names=names, vocab=config.vocab, width=width,
                     max_context=config.max_positions, sources=sources, stream_vectors=vectors)


def _gated(names, sources, prefix, width, inner, rule, limit, std):
    part = GatedFeedForward(width, inner, rule, limit=limit, init_std=std, down_init_std=inner ** -0.5)
    names[prefix + "gate_up"] = (part, "gate_up.weight")
    names[prefix + "down"] = (part, "down.weight")
    sources[prefix + "gate_up"] = Concat((Stored(prefix + "gate"), Stored(prefix + "up")), 0, (inner, inner))
    return part


GOKEZEN = register_architecture(Architecture("gokezen", GokezenConfig.MODEL_TYPES, GokezenConfig, build_gokezen),
                                replace=True)
