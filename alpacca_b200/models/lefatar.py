"""The Lefatar decoder, put together from the parts.

Layers as config.json lists them, each a parallel block: h = norm1(x); x += mixer(h) + ff(h), with a norm
that multiplies by 1 + w for its stored w.  A layer's mixer is the matrix memory (`mlstm`) or causal attention over
a cached latent with a sink (`latent_attention`); its feed-forward is the gated dense one (SiLU), routed
experts (exact GELU, grouped router) or none.  A final norm of the same kind, then the head.

Tensor names (matrices [out, in], named by their prefix alone):
    embed, head, final.norm, l<i>.norm1
    l<i>.mix.{q,k,v,g,o,norm,i,i.b,f,f.b}                                mlstm
    l<i>.mix.{dq,dq.norm,uq,dkv,dkv.norm,uk,uv,sink,o}                  latent_attention
    l<i>.mlp.{gate,up,down}   or   l<i>.mlp.router, l<i>.mlp.e<j>.{up,down}
"""
from __future__ import annotations

from ..config.lefatar import LefatarConfig
from ..config.registry import register_architecture
from ..engine.model import DecoderSpec
from ..parts import (BuildOptions, LatentAttention, MatrixMemory, ParallelBlock, RMSNorm, RotaryEncoding, RoutedExperts,
                     SwiGLU, TokenEmbedding, VocabHead)


def _norm(opts, width, eps, name):
    return RMSNorm(opts, width, eps, name, weight_suffix="", unit_offset=True)


@register_architecture("Lefatar", LefatarConfig)
def build_lefatar(cfg: LefatarConfig, opts: BuildOptions) -> DecoderSpec:
    E, eps = cfg.width, cfg.eps
    rotations: dict = {}          # layers with the same rotation share one table
    layers = []
    for i, layer in enumerate(cfg.layers):
        p, mx = f"l{i}", layer["mixer"]
        if layer["type"] == "mlstm":
            mixer = MatrixMemory(opts, E, mx["heads"], mx["dim"], mx["vdim"], mx["gate_cap"], eps, f"{p}.mix")
        else:
            key = (mx["rot_dim"], mx["rot"]["dims"], float(mx["rot"]["base"]))
            if key not in rotations:
                rotations[key] = RotaryEncoding(opts, key[0], key[1], key[2], "llama")
            mixer = LatentAttention(opts, E, mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["q_rank"],
                                    mx["kv_rank"], mx["scale"], eps, rotations[key], f"{p}.mix")
        mlp = layer.get("mlp")
        if mlp is None:
            ffn = None
        elif mlp["kind"] == "dense":
            ffn = SwiGLU(opts, E, mlp["ff"], f"{p}.mlp", names=("gate", "up", "down"), weight_suffix="")
        else:
            rt = mlp["router"]
            ffn = RoutedExperts(opts, E, mlp["expert"]["ff"], rt["experts"], rt["top"], rt["groups"]["count"],
                                rt["groups"]["keep"], rt["scale"], f"{p}.mlp", activation="gelu")
        layers.append(ParallelBlock(_norm(opts, E, eps, f"{p}.norm1"), mixer, ffn))
    return DecoderSpec(
        embedding=TokenEmbedding(opts, cfg.vocab, E, "embed", weight_suffix=""), layers=layers,
        final_norm=_norm(opts, E, eps, "final.norm"),
        head=VocabHead(opts, cfg.vocab, E, "head", weight_suffix=""),
        stop_token_ids=cfg.stop_tokens, vocab_size=cfg.vocab)
