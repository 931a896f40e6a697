"""The Buguzen decoder, put together from the parts.

Layers as config.json lists them, each a pre-norm block: x += mixer(norm1(x)); x += ff(norm2(x)) where the layer
has a feed-forward; then the layer's token input (`TokenSide`) where the model has one.  The norm multiplies by
its stored weight.  A layer's mixer is linear attention with a fixed decay per head (`lightning`), attention with
two score maps per head whose difference is taken (`attention`), or attention whose values are its keys as
projected, with query and key norm and a sink (`attention_2`); the latter two have a window, biases and a
rotation over part of each vector.  The feed-forward is the gated dense one with ReLU on the gate.  With a
`loop`, layers start .. stop-1 run `times` times in a row on the same weights, each pass with cache entries of
its own, and a learned vector per pass is added to the stream before the pass's first layer.

Tensor names (matrices [out, in], named by their prefix alone):
    embed, head, final.norm, loop.step, side.embed, l<i>.norm1, l<i>.norm2
    l<i>.mix.{q,k,v,g,o,norm}                                          lightning
    l<i>.mix.{q,q.b,k,k.b,v,v.b,lq1,lk1,lq2,lk2,o}                     attention
    l<i>.mix.{q,q.b,k,k.b,q.norm,k.norm,sink,o}                        attention_2
    l<i>.mlp.{gate,up,down}       l<i>.side.{gate,proj,norm}
"""
from __future__ import annotations

from ..config.buguzen import BuguzenConfig
from ..config.registry import register_architecture
from ..engine.model import DecoderSpec, Run
from ..parts import (BuildOptions, DecayLinearAttention, MapsAttention, PassOffset, PreNormBlock, RMSNorm,
                     RotaryEncoding, SwiGLU, TokenEmbedding, TokenSide, TokenTable, VocabHead)


def _norm(opts, width, eps, name):
    return RMSNorm(opts, width, eps, name, weight_suffix="")


def _scaling(sc: dict | None) -> dict | None:
    """The configuration's rotation scaling in the words of `RotaryEncoding`: a factor alone divides every
    frequency; with low, high and an original length, long wavelengths are divided and the middle is blended."""
    if not sc:
        return None
    if "original" not in sc:
        return {"rope_type": "linear", "factor": sc["factor"]}
    return {"rope_type": "llama3", "factor": sc["factor"], "low_freq_factor": sc["low"],
            "high_freq_factor": sc["high"], "original_max_position_embeddings": sc["original"]}


@register_architecture("Buguzen", BuguzenConfig)
def build_buguzen(cfg: BuguzenConfig, opts: BuildOptions) -> DecoderSpec:
    E, eps = cfg.width, cfg.eps
    rotations: dict = {}          # layers with the same rotation share one table

    def rotation(dim, rot, pairing):
        if rot["dims"] == 0:          # nothing is rotated
            return None
        sc = rot.get("scaling") or {}
        key = (dim, rot["dims"], float(rot["base"]), pairing, tuple(sorted(sc.items())))
        if key not in rotations:
            rotations[key] = RotaryEncoding(opts, dim, rot["dims"], float(rot["base"]), pairing, _scaling(sc))
        return rotations[key]

    stream_parts = []
    table = None
    side_dim = cfg.token_side["dim"] if cfg.token_side else 0
    if side_dim:
        table = TokenTable(opts, cfg.vocab, len(cfg.layers) * side_dim, "side.embed")
        stream_parts.append(table)
    layers = []
    for i, layer in enumerate(cfg.layers):
        p, mx = f"l{i}", layer["mixer"]
        if layer["type"] == "lightning":
            mixer = DecayLinearAttention(opts, E, mx["heads"], mx["dim"], mx["vdim"], mx["decay"], eps, f"{p}.mix")
        elif layer["type"] == "attention":
            mixer = MapsAttention(opts, E, mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"],
                                  rotation(mx["dim"], mx["rot"], "llama"), f"{p}.mix", mx["scale"], eps,
                                  window=mx["mask"]["size"], n_maps=2, bias=True, difference=mx["diff"])
        else:
            mixer = MapsAttention(opts, E, mx["heads"], mx["kv_heads"], mx["dim"], None,
                                  rotation(mx["dim"], mx["rot"], "neox"), f"{p}.mix", mx["scale"], eps,
                                  window=mx["mask"]["size"], bias=True, qk_norm=True, values_are_keys=True, sink=True)
        mlp = layer.get("mlp")
        ffn = norm2 = None
        if mlp is not None:
            norm2 = _norm(opts, E, eps, f"{p}.norm2")
            ffn = SwiGLU(opts, E, mlp["ff"], f"{p}.mlp", names=("gate", "up", "down"), weight_suffix="",
                         activation="relu")
        side = TokenSide(opts, E, side_dim, table, i * side_dim, eps, f"{p}.side") if side_dim else None
        layers.append(PreNormBlock(_norm(opts, E, eps, f"{p}.norm1"), mixer, norm2, ffn, after=side))
    schedule = []
    offset_at = None
    if cfg.loop:
        offset_at = len(stream_parts)
        stream_parts.append(PassOffset(opts, cfg.loop["times"], E, "loop.step"))
    for i, t in cfg.run_order():
        first_of_pass = t is not None and i == cfg.loop["start"]
        schedule.append(Run(i, enter=(offset_at, t) if first_of_pass else None))
    return DecoderSpec(
        embedding=TokenEmbedding(opts, cfg.vocab, E, "embed", weight_suffix=""), layers=layers,
        final_norm=_norm(opts, E, eps, "final.norm"),
        head=VocabHead(opts, cfg.vocab, E, "head", weight_suffix=""),
        schedule=schedule, stream_parts=stream_parts, stop_token_ids=cfg.stop_tokens, vocab_size=cfg.vocab)
