"""Weight import and export: an RWKV-6 ``.pth`` state dict (the tensor names of the reference's plain-torch model,
rwkv_v6_demo.py:62-101,167-172,195-241) to and from this package's ``model.RWKV6``, following the mapping of the
reference's converter (keras_torch_transport.py: ``TorchToKerasConvertor``):

* ``time_maa_w1`` [D, 5R] is five ``dense_a`` kernels side by side in the order w, k, v, r, g and ``time_maa_w2``
  [5, R, D] the five ``dense_b`` kernels in the same order, with ``time_maa_{w,k,v,r,g}`` as the ``dense_b`` biases
  (keras_torch_transport.py:85-101); this package keeps them in the order r, k, v, w, g of ``TimeMixInputs.ORDER``;
* ``time_decay_w1`` / ``time_decay_w2`` / ``time_decay`` are ``dense_w``'s two kernels and its bias (:116-118);
* ``time_faaaa`` is u (:120-121); ``ln_x`` is the per-head GroupNorm, reshaped to [heads, head_size] (:77-82);
* ``blocks.0.ln0`` is the LayerNorm behind the embedding (:48-51); ``ln1`` / ``ln2`` the block norms (:139-140);
  ``ln_out`` and ``head`` the output layer (:142-145).

``torch.nn.Linear`` stores [out, in] like the ``.pth`` file, so dense weights are copied as they are; the reference's
Keras layers store [in, out] (``_assign_dense`` transposes, :57-59), which ``reference_layer_weights`` reproduces for a
maintainer who fills the reference's Keras model from this package's weights.
"""
from __future__ import annotations

import re
from collections import OrderedDict

import numpy as np
import torch

from .model import RWKV6
from .time_mix_inputs import TimeMixInputs

_PTH_MIX_ORDER = ("w", "k", "v", "r", "g")                              # rwkv_v6_demo.py:116
_PERM = [_PTH_MIX_ORDER.index(c) for c in TimeMixInputs.ORDER]          # position in the .pth order of r, k, v, w, g


def _t(x) -> torch.Tensor:
    return x.detach() if isinstance(x, torch.Tensor) else torch.from_numpy(np.asarray(x))


def config_from_pth(sd) -> dict:
    """Model shape read off the tensors, as the reference's converter does (keras_torch_transport.py:17-25,32-39)."""
    vocab, emb = sd["emb.weight"].shape
    layers = 0
    for key in sd:
        m = re.match(r"^blocks\.(\d+)\.", key)
        if m:
            layers = max(layers, int(m.group(1)) + 1)
    heads, head_size = sd["blocks.0.att.time_faaaa"].shape
    hidden = sd["blocks.0.att.time_decay"].shape[-1]
    if not (hidden == emb == heads * head_size):
        raise ValueError(f"inconsistent shapes: hidden {hidden}, embedding {emb}, heads {heads} x head size {head_size}")
    return dict(num_layers=layers, vocabulary_size=int(vocab), hidden_size=int(hidden), head_size=int(head_size),
                decomposer_size=int(sd["blocks.0.att.time_maa_w2"].shape[1]),
                expand_size=int(sd["blocks.0.ffn.key.weight"].shape[0]),
                decay_rank=int(sd["blocks.0.att.time_decay_w1"].shape[1]))


def _pairs(model: RWKV6, i: int):
    """(parameter of this package, .pth name, to_model, to_pth) for block i; the two callables convert layouts."""
    blk = model.blocks[i]
    tm, cm, mi = blk.time_mix, blk.channel_mix, blk.time_mix.mix_inputs
    D, R = mi.hidden_size, mi.decomposer_size
    a, f = f"blocks.{i}.att.", f"blocks.{i}.ffn."
    same = (lambda x: x, lambda x: x)
    vec = (lambda x: x.reshape(-1), lambda x: x.reshape(1, 1, -1))
    tr = (lambda x: x.t(), lambda x: x.t())
    inv = [_PERM.index(j) for j in range(5)]
    yield mi.time_mix_x, a + "time_maa_x", *vec
    yield (mi.dense_a, a + "time_maa_w1", lambda x: x.reshape(D, 5, R)[:, _PERM].reshape(D, 5 * R),
           lambda x: x.reshape(D, 5, R)[:, inv].reshape(D, 5 * R))
    yield mi.dense_b, a + "time_maa_w2", lambda x: x[_PERM], lambda x: x[inv]
    for name, lin in (("receptance", tm.dense_r), ("key", tm.dense_k), ("value", tm.dense_v), ("gate", tm.dense_g),
                      ("output", tm.dense_o)):
        yield lin.weight, a + name + ".weight", *same
    yield tm.w_a.weight, a + "time_decay_w1", *tr
    yield tm.w_b.weight, a + "time_decay_w2", *tr
    yield tm.w_b.bias, a + "time_decay", *vec
    yield tm.time_faaaa, a + "time_faaaa", *same
    H, N = tm.num_heads, tm.head_size
    yield tm.group_norm.scale, a + "ln_x.weight", lambda x: x.reshape(H, N), lambda x: x.reshape(-1)
    yield tm.group_norm.offset, a + "ln_x.bias", lambda x: x.reshape(H, N), lambda x: x.reshape(-1)
    yield cm.time_mix_k, f + "time_maa_k", *vec
    yield cm.time_mix_r, f + "time_maa_r", *vec
    yield cm.dense_key.weight, f + "key.weight", *same
    yield cm.dense_receptance.weight, f + "receptance.weight", *same
    yield cm.dense_value.weight, f + "value.weight", *same
    for ln, mod in (("ln1", blk.layer_norm_att), ("ln2", blk.layer_norm_ffn)):
        yield mod.weight, f"blocks.{i}.{ln}.weight", *same
        yield mod.bias, f"blocks.{i}.{ln}.bias", *same


def _top_pairs(model: RWKV6):
    same = (lambda x: x, lambda x: x)
    yield model.embedding.weight, "emb.weight", *same
    yield model.embedding_ln.weight, "blocks.0.ln0.weight", *same
    yield model.embedding_ln.bias, "blocks.0.ln0.bias", *same
    yield model.output_ln.weight, "ln_out.weight", *same
    yield model.output_ln.bias, "ln_out.bias", *same
    yield model.output_layer.weight, "head.weight", *same


def load_pth(model: RWKV6, sd, strict: bool = True) -> RWKV6:
    """Copies a ``.pth`` state dict (tensors or numpy arrays) into ``model``; each parameter keeps its dtype and device.
    ``strict``: every tensor of ``sd`` must be used and every parameter of the model filled."""
    used = set()
    with torch.no_grad():
        for i in range(len(model.blocks)):
            mix_bias = []
            for p, name, to_model, _ in _pairs(model, i):
                p.copy_(to_model(_t(sd[name])).to(p.dtype))
                used.add(name)
            for c in TimeMixInputs.ORDER:
                name = f"blocks.{i}.att.time_maa_{c}"
                mix_bias.append(_t(sd[name]).reshape(1, -1))
                used.add(name)
            mb = model.blocks[i].time_mix.mix_inputs.bias_b
            mb.copy_(torch.stack(mix_bias).to(mb.dtype))
        for p, name, to_model, _ in _top_pairs(model):
            p.copy_(to_model(_t(sd[name])).to(p.dtype))
            used.add(name)
    if strict:
        extra = sorted(set(sd) - used)
        if extra:
            raise KeyError(f"tensors of the state dict with no counterpart in the model: {extra[:8]}")
    return model


def from_pth(sd, device="cuda", dtype=torch.float32) -> RWKV6:
    """Builds the model a state dict describes and loads it.  ``dtype`` bfloat16 keeps the small kernel operands fp32
    (``RWKV6.to_bf16_``)."""
    cfg = config_from_pth(sd)
    model = RWKV6(**cfg)
    load_pth(model, sd)
    model = model.to(device)
    if dtype == torch.bfloat16:
        model.to_bf16_()
    elif dtype != torch.float32:
        raise ValueError("dtype must be float32 or bfloat16")
    return model


def to_pth(model: RWKV6) -> "OrderedDict[str, torch.Tensor]":
    """The model's weights under the ``.pth`` names and layouts (fp32, on CPU): the inverse of ``load_pth``."""
    out = OrderedDict()
    f32 = lambda x: x.detach().to("cpu", torch.float32).contiguous()
    for p, name, _, to_pth_ in _top_pairs(model):
        out[name] = f32(to_pth_(p))
    for i in range(len(model.blocks)):
        for p, name, _, to_pth_ in _pairs(model, i):
            out[name] = f32(to_pth_(p.detach()))
        bias = model.blocks[i].time_mix.mix_inputs.bias_b.detach()
        for j, c in enumerate(TimeMixInputs.ORDER):
            out[f"blocks.{i}.att.time_maa_{c}"] = f32(bias[j].reshape(1, 1, -1))
    return out


def reference_layer_weights(sd) -> "OrderedDict[str, np.ndarray]":
    """The values the reference's converter assigns to its Keras model, keyed by the attribute path of the variable
    (``rwkv_blocks.<i>.time_mix.dense_xr.dense_a.kernel`` ...), in Keras layouts: Dense kernels are [in, out]
    (keras_torch_transport.py:57-59), GroupNorm scale and offset [heads, head_size] (:77-82), mixing vectors flat."""
    cfg = config_from_pth(sd)
    H, N = cfg["hidden_size"] // cfg["head_size"], cfg["head_size"]
    g = lambda name: np.asarray(_t(sd[name]).to(torch.float32).cpu().numpy())
    out = OrderedDict()
    out["embedding_layer.embedding.embeddings"] = g("emb.weight")
    out["embedding_layer.layer_norm.gamma"] = g("blocks.0.ln0.weight")
    out["embedding_layer.layer_norm.beta"] = g("blocks.0.ln0.bias")
    for i in range(cfg["num_layers"]):
        a, f, k = f"blocks.{i}.att.", f"blocks.{i}.ffn.", f"rwkv_blocks.{i}."
        w1 = g(a + "time_maa_w1").reshape(cfg["hidden_size"], 5, -1)
        w2 = g(a + "time_maa_w2")
        for j, c in enumerate(_PTH_MIX_ORDER):
            out[k + f"time_mix.dense_x{c}.dense_a.kernel"] = w1[:, j]
            out[k + f"time_mix.dense_x{c}.dense_b.kernel"] = w2[j]
            out[k + f"time_mix.dense_x{c}.dense_b.bias"] = g(a + "time_maa_" + c).reshape(-1)
        out[k + "time_mix.time_mix_x"] = g(a + "time_maa_x").reshape(-1)
        for name, layer in (("receptance", "dense_r"), ("key", "dense_k"), ("value", "dense_v"), ("gate", "dense_g"),
                            ("output", "dense_o")):
            out[k + f"time_mix.{layer}.kernel"] = g(a + name + ".weight").T
        out[k + "time_mix.dense_w.dense_a.kernel"] = g(a + "time_decay_w1")
        out[k + "time_mix.dense_w.dense_b.kernel"] = g(a + "time_decay_w2")
        out[k + "time_mix.dense_w.dense_b.bias"] = g(a + "time_decay").reshape(-1)
        out[k + "time_mix.time_faaaa"] = g(a + "time_faaaa")
        out[k + "time_mix.group_norm.scale"] = g(a + "ln_x.weight").reshape(H, N)
        out[k + "time_mix.group_norm.offset"] = g(a + "ln_x.bias").reshape(H, N)
        out[k + "channel_mix.time_mix_k"] = g(f + "time_maa_k").reshape(-1)
        out[k + "channel_mix.time_mix_r"] = g(f + "time_maa_r").reshape(-1)
        out[k + "channel_mix.dense_key.kernel"] = g(f + "key.weight").T
        out[k + "channel_mix.dense_receptance.kernel"] = g(f + "receptance.weight").T
        out[k + "channel_mix.dense_value.kernel"] = g(f + "value.weight").T
        out[k + "layer_norm_att.gamma"] = g(f"blocks.{i}.ln1.weight")
        out[k + "layer_norm_att.beta"] = g(f"blocks.{i}.ln1.bias")
        out[k + "layer_norm_ffn.gamma"] = g(f"blocks.{i}.ln2.weight")
        out[k + "layer_norm_ffn.beta"] = g(f"blocks.{i}.ln2.bias")
    out["output_layer.layer_norm.gamma"] = g("ln_out.weight")
    out["output_layer.layer_norm.beta"] = g("ln_out.bias")
    out["output_layer.output_layer.kernel"] = g("head.weight").T
    return out
