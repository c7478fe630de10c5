"""The architectures this engine knows: for each, its configuration class and the function
that writes the model down as data (which parts every layer has, and the order of runs).
"""
from __future__ import annotations

from ..parts.registry import register_architecture
from ..parts.spec import BlockSpec, ModelSpec, PartSpec, RunStep
from .bivizen_config import BivizenConfig
from .model_config import Qwen2Config
from .pefivik_config import PefivikConfig
from .tabopel_config import TabopelConfig
from .tomodra_config import TomodraConfig


# what follows "model.layers.N." in the names of each part's tensors
QWEN2_NAMES = {"mixer_norm": "input_layernorm.", "mixer": "self_attn.",
               "feed_forward_norm": "post_attention_layernorm.", "feed_forward": "mlp."}


def qwen2_spec(config: Qwen2Config) -> ModelSpec:
    """Qwen2ForCausalLM as AIR defines it (src/model/qwen2_contract.cpp:33-139) and
    computes it (src/reference/reference_executor.cpp:325-428): every layer is a pre-norm
    block of grouped-query attention with q/k/v bias and half-split rotary encoding, and a
    SwiGLU feed-forward; a final RMSNorm; an output matrix that is either lm_head.weight or
    the embedding table."""
    e, d = config.hidden_size, config.head_dim
    position = PartSpec("rope_half", {"rotary_dim": d, "theta": config.rope_theta,
                                      "max_positions": config.max_position_embeddings})
    layers = []
    for i in range(config.num_hidden_layers):
        norm = PartSpec("rms", {"size": e, "eps": config.rms_norm_eps})
        layers.append(BlockSpec(
            kind="pre_norm", prefix=f"model.layers.{i}.",
            parts={"mixer_norm": norm,
                   "mixer": PartSpec("attention", {
                       "hidden": e, "heads": config.num_attention_heads, "kv_heads": config.num_key_value_heads,
                       "head_dim": d, "qkv_bias": config.attention_bias, "window": config.layer_window(i),
                       "position": position}),
                   "feed_forward_norm": norm,
                   "feed_forward": PartSpec("swiglu", {"hidden": e, "intermediate": config.intermediate_size})},
            names=QWEN2_NAMES))
    return ModelSpec(
        architecture=config.architecture, hidden_size=e, vocab_size=config.vocab_size,
        max_positions=config.max_position_embeddings, layers=tuple(layers),
        order=tuple(RunStep(i) for i in range(config.num_hidden_layers)),
        final_norm=PartSpec("rms", {"size": e, "eps": config.rms_norm_eps}),
        embedding_name="model.embed_tokens.weight", final_norm_prefix="model.norm.",
        output_name=None if config.tie_word_embeddings else "lm_head.weight",
        eos_token_id=config.eos_token_id)


register_architecture("Qwen2ForCausalLM", Qwen2Config, qwen2_spec)


def bivizen_spec(config: BivizenConfig) -> ModelSpec:
    """Bivizen: every layer is a parallel block (one RMSNorm whose rows the mixer and the feed-forward both read,
    their outputs added to the stream together, each times a learned scale per column) whose mixer is softmax
    attention with its options, the gated delta rule or gated linear attention, as config.json lists them, and whose
    feed-forward is a gated one with limits.  Tensors: embed, l<i>.norm1, l<i>.mix.*, l<i>.mlp.*, l<i>.ls1, l<i>.ls2,
    final.norm, head."""
    e = config.width
    norm = PartSpec("rms", {"size": e, "eps": config.eps, "tensor": ""})
    layers, first_v_mix = [], True
    for i, l in enumerate(config.layers):
        if l.type == "attention":
            position = (PartSpec("rope_half_live", {"rotary_dim": l.rot_dims, "theta": l.rot_base}) if l.rot_dims
                        else PartSpec("none"))
            v_mix = None
            if l.v_mix:
                v_mix, first_v_mix = ("first" if first_v_mix else "mix"), False
            mixer = PartSpec("capped_attention", {
                "hidden": e, "heads": l.heads, "kv_heads": l.kv_heads, "head_dim": l.dim, "v_dim": l.vdim,
                "scale": l.scale, "softcap": l.softcap, "window": None, "qkv_bias": True, "head_gate": True,
                "v_mix": v_mix, "position": position})
        elif l.type == "delta":
            mixer = PartSpec("gated_delta", {"hidden": e, "heads": l.heads, "kv_heads": l.kv_heads, "head_dim": l.dim,
                                             "v_dim": l.vdim, "conv": l.conv, "eps": config.eps})
        else:
            mixer = PartSpec("gla", {"hidden": e, "heads": l.heads, "head_dim": l.dim, "v_dim": l.vdim, "tau": l.tau,
                                     "rank": l.rank, "eps": config.eps})
        parts = {"norm": norm, "mixer": mixer}
        names = {"norm": "norm1", "mixer": "mix.", "mixer_scale": "ls1", "feed_forward_scale": "ls2"}
        if l.mlp is not None:
            parts["feed_forward"] = PartSpec("clamped_glu", {"hidden": e, "intermediate": l.mlp.ff,
                                                             "limit": l.mlp.limit, "alpha": 1.702})
            names.update(feed_forward="mlp.")
        layers.append(BlockSpec(kind="parallel", prefix=f"l{i}.", parts=parts, names=names))
    return ModelSpec(
        architecture=config.architecture, hidden_size=e, vocab_size=config.vocab, max_positions=config.max_positions,
        layers=tuple(layers), order=tuple(RunStep(i) for i in range(len(layers))), final_norm=norm,
        embedding_name="embed", final_norm_prefix="final.norm", output_name="head", eos_token_id=config.eos_token_id)


register_architecture("Bivizen", BivizenConfig, bivizen_spec)


def tomodra_spec(config: TomodraConfig) -> ModelSpec:
    """Tomodra: every layer normalises after the sum (x = rms(alpha x + mixer(x)) w1; x = rms(alpha x + ff(x)) w2); its
    mixer is attention over a compressed latent inside a sliding window (a layer may read the latent that an earlier
    layer keeps) or grouped-query attention with normalised queries and keys, a rotation of neighbouring pairs with
    stretched frequencies, chunks and a sink in the softmax; its feed-forward is a mixture of experts whose weights
    multiply the experts' input, beside a gated shared expert.  Tensors: embed, l<i>.norm1, l<i>.norm2, l<i>.mix.*,
    l<i>.mlp.*, final.norm, head."""
    e = config.width
    layers, order = [], []
    # a latent's pages are kept as long as the widest window among the layers that read them needs them
    keep = {}
    for i, l in enumerate(config.layers):
        if l.type == "latent_attention":
            owner = i if l.kv_from is None else l.kv_from
            keep[owner] = max(keep.get(owner, 0), l.mask_size)
    for i, l in enumerate(config.layers):
        if l.type == "latent_attention":
            position = PartSpec("rope_live", {"rotary_dim": l.rot_dim, "theta": l.rot_base, "pairing": "half"})
            mixer = PartSpec("latent_attention", {
                "hidden": e, "heads": l.heads, "head_dim": l.dim, "rot_dim": l.rot_dim, "v_dim": l.vdim,
                "kv_rank": l.kv_rank, "scale": l.scale, "window": l.mask_size, "eps": config.eps,
                "borrows": l.kv_from is not None, "keep": keep[i if l.kv_from is None else l.kv_from],
                "position": position})
        else:
            position = PartSpec("rope_live", {"rotary_dim": l.rot_dims, "theta": l.rot_base, "pairing": "neighbours",
                                              "scaling": l.scaling.to_dict() if l.scaling is not None else None})
            mixer = PartSpec("normed_attention", {
                "hidden": e, "heads": l.heads, "kv_heads": l.kv_heads, "head_dim": l.dim, "v_dim": l.vdim,
                "scale": l.scale, "chunk": l.mask_size, "qk_norm": True, "sink": True, "eps": config.eps,
                "position": position})
        norm = PartSpec("rms_after", {"size": e, "eps": config.eps, "alpha": config.alpha, "tensor": ""})
        parts = {"mixer": mixer, "mixer_norm": norm}
        names = {"mixer": "mix.", "mixer_norm": "norm1", "feed_forward": "mlp.", "feed_forward_norm": "norm2"}
        if l.mlp is not None:
            parts["feed_forward"] = PartSpec("routed_experts", {
                "hidden": e, "experts": l.mlp.experts, "top": l.mlp.top, "intermediate": l.mlp.ff,
                "shared_intermediate": l.mlp.shared_ff, "shared_gate": bool(l.mlp.shared_ff), "score": "sigmoid",
                "renormalize": False})
        if l.mlp is not None or l.second_norm:
            parts["feed_forward_norm"] = norm
        layers.append(BlockSpec(kind="post_norm", prefix=f"l{i}.", parts=parts, names=names))
        order.append(RunStep(i, cache_from=l.kv_from if l.type == "latent_attention" else None))
    return ModelSpec(
        architecture=config.architecture, hidden_size=e, vocab_size=config.vocab, max_positions=config.max_positions,
        layers=tuple(layers), order=tuple(order),
        final_norm=PartSpec("rms", {"size": e, "eps": config.eps, "tensor": ""}),
        embedding_name="embed", final_norm_prefix="final.norm", output_name="head", eos_token_id=config.eos_token_id)


register_architecture("Tomodra", TomodraConfig, tomodra_spec)


def pefivik_spec(config: PefivikConfig) -> ModelSpec:
    """Pefivik: the embedding is the token's row plus a row of a second table chosen by a hash of the token and the one
    before it.  Every layer is a pre-norm block whose sub-layers' outputs are multiplied by one constant before they
    join the stream, and whose norms have ONE learned number each: x += m mixer(n1(x)); x += m ff(n2(x)).  The mixer is
    attention over a compressed latent without positions, with a sink in the softmax and a sigmoid gate per head, or
    HGRN2 (a matrix state per head; the complement of the forget gate stands where a key would); the feed-forward is a dense one with
    biases and the PolyNorm activation, or a mixture of gated experts chosen among the best groups, beside a shared
    expert.  A stretch of layers may run several times over with the same weights, every pass with a cache of its own;
    ahead of every pass the stream receives a row of the table loop.step, and ahead of every pass but the first the
    embedding's output once more.  The logits are soft-capped.  Tensors: embed, bigram, loop.step, l<i>.norm1,
    l<i>.norm2, l<i>.mix.*, l<i>.mlp.*, final.norm, head."""
    e = config.width
    norm = PartSpec("rms_scalar", {"size": e, "eps": config.eps, "tensor": ""})
    layers = []
    for i, l in enumerate(config.layers):
        if l.type == "latent_attention":
            mixer = PartSpec("latent_attention", {
                "hidden": e, "heads": l.heads, "head_dim": l.dim, "rot_dim": 0, "v_dim": l.vdim, "kv_rank": l.kv_rank,
                "scale": l.scale, "window": None, "eps": config.eps, "sink": True, "head_gate": True})
        else:
            mixer = PartSpec("hgrn2", {"hidden": e, "heads": l.heads, "head_dim": l.dim, "v_dim": l.vdim,
                                       "eps": config.eps})
        parts = {"mixer_norm": norm, "mixer": mixer}
        names = {"mixer_norm": "norm1", "mixer": "mix.", "feed_forward_norm": "norm2", "feed_forward": "mlp."}
        f = l.mlp
        if f is not None and f.kind == "dense":
            parts["feed_forward"] = PartSpec("polynorm_mlp", {"hidden": e, "intermediate": f.ff, "eps": config.eps})
        elif f is not None:
            parts["feed_forward"] = PartSpec("routed_experts", {
                "hidden": e, "experts": f.experts, "top": f.top, "intermediate": f.ff, "shared_intermediate": f.shared_ff,
                "shared_gate": False, "score": "sigmoid", "renormalize": True, "norm_eps": 1e-20, "route_scale": f.scale,
                "groups": (f.groups, f.keep) if f.groups > 1 else None, "weight_on": "output"})
        if f is not None:
            parts["feed_forward_norm"] = norm
        params = {"residual_scale": config.residual_mult}
        if f is None and l.second_norm:
            params["idle"] = (("norm2", ()),)      # a tensor of the file that the layer does not use
        layers.append(BlockSpec(kind="pre_norm", prefix=f"l{i}.", parts=parts, names=names, params=params))
    order = [RunStep(i) for i in range(config.loop_start)]
    tables = (("loop.step", config.loop_times),) if config.has_loop else ()
    if config.loops:
        for t in range(config.loop_times):
            order += [RunStep(i, add_embedding=(t > 0 and i == config.loop_start),
                              add_row=("loop.step", t) if i == config.loop_start else None)
                      for i in range(config.loop_start, config.loop_stop)]
    order += [RunStep(i) for i in range(config.loop_stop if config.loops else config.loop_start, len(layers))]
    return ModelSpec(
        architecture=config.architecture, hidden_size=e, vocab_size=config.vocab, max_positions=config.max_positions,
        layers=tuple(layers), order=tuple(order), final_norm=norm, embedding_name="embed", final_norm_prefix="final.norm",
        output_name="head", eos_token_id=config.eos_token_id, logit_softcap=config.logit_softcap,
        embedding=PartSpec("bigram_hash", {"vocab": config.vocab, "hidden": e, "buckets": config.buckets,
                                           "mul_prev": config.mul_prev, "mul_cur": config.mul_cur, "pairs": "bigram"}),
        stream_tables=tables)


register_architecture("Pefivik", PefivikConfig, pefivik_spec)


def tabopel_spec(config: TabopelConfig) -> ModelSpec:
    """Tabopel: the embedding's rows are multiplied by a constant.  Every layer has a norm on both sides of each
    sub-layer: x += n1b(mixer(n1(x))); x += n2b(ff(n2(x))).  The mixer is grouped-query attention behind short causal
    convolutions of q, k and v, with a sink of score 0 in the softmax and a sigmoid gate on the heads' outputs
    ("attention"); grouped-query attention with biases, queries and keys normalised as whole vectors, a soft cap and a
    learned sink per head ("attention_2"); or retention, linear attention with one constant decay per head
    ("retention").  All three rotate the first part of a head, the first with frequencies that may be slowed down in
    bands.  The feed-forward is a hidden layer with the squared rectifier, or a mixture of such experts chosen by
    softmax score plus a learned correction, some of which may be identity experts.  A stretch of layers may run several
    times over with the same weights, every pass with a cache of its own; ahead of every pass the stream receives a
    row of the table loop.step.  Tensors: embed, loop.step, l<i>.norm1, norm1b, norm2, norm2b, l<i>.mix.*, l<i>.mlp.*,
    final.norm, head."""
    e = config.width
    norm = PartSpec("rms", {"size": e, "eps": config.eps, "tensor": ""})
    layers = []
    for i, l in enumerate(config.layers):
        position = None
        if l.rot is not None and l.rot.dims:
            position = PartSpec("rope_live", {"rotary_dim": l.rot.dims, "theta": l.rot.base, "pairing": "half",
                                              "rule": "banded", "scaling": l.rot.scaling()})
        if l.type == "retention":
            mixer = PartSpec("retention", {"hidden": e, "heads": l.heads, "head_dim": l.dim, "v_dim": l.vdim,
                                           "decay": l.decay, "eps": config.eps, "position": position})
        else:
            first = l.type == "attention"
            mixer = PartSpec("normed_attention", {
                "hidden": e, "heads": l.heads, "kv_heads": l.kv_heads, "head_dim": l.dim, "v_dim": l.vdim,
                "scale": l.scale, "eps": config.eps,
                "position": position or PartSpec("rope_live", {"rotary_dim": 0, "theta": 1.0}),
                "qk_norm": False if first else "whole", "sink": "zero" if first else "learned",
                "qkv_bias": not first, "conv": l.conv if first else 0, "softcap": 0.0 if first else l.softcap,
                "out_gate": first})
        parts = {"mixer_norm": norm, "mixer": mixer, "mixer_out_norm": norm}
        names = {"mixer_norm": "norm1", "mixer": "mix.", "mixer_out_norm": "norm1b", "feed_forward_norm": "norm2",
                 "feed_forward": "mlp.", "feed_forward_out_norm": "norm2b"}
        f = l.mlp
        if f is not None and f.kind == "dense":
            parts["feed_forward"] = PartSpec("relu2_mlp", {"hidden": e, "intermediate": f.ff})
        elif f is not None:
            parts["feed_forward"] = PartSpec("routed_experts", {
                "hidden": e, "experts": f.experts, "top": f.top, "intermediate": f.ff, "score": "softmax",
                "renormalize": False, "weight_on": "output", "gated": False, "activation": "relu2",
                "choice_bias": True, "identity": f.identity})
        if f is not None:
            parts["feed_forward_norm"] = parts["feed_forward_out_norm"] = norm
        params = {"idle": tuple((n, (e,)) for n in l.idle)} if f is None and l.idle else {}
        layers.append(BlockSpec(kind="sandwich", prefix=f"l{i}.", parts=parts, names=names, params=params))
    order = [RunStep(i) for i in range(config.loop_start)]
    tables = (("loop.step", config.loop_times),) if config.has_loop else ()
    if config.loops:
        for t in range(config.loop_times):
            order += [RunStep(i, add_row=("loop.step", t) if i == config.loop_start else None)
                      for i in range(config.loop_start, config.loop_stop)]
    order += [RunStep(i) for i in range(config.loop_stop if config.loops else config.loop_start, len(layers))]
    return ModelSpec(
        architecture=config.architecture, hidden_size=e, vocab_size=config.vocab, max_positions=config.max_positions,
        layers=tuple(layers), order=tuple(order), final_norm=norm, embedding_name="embed", final_norm_prefix="final.norm",
        output_name="head", eos_token_id=config.eos_token_id, embedding_multiplier=config.embedding_scale,
        stream_tables=tables)


register_architecture("Tabopel", TabopelConfig, tabopel_spec)
