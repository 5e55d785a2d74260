"""RWKV-6 (Finch) language model in PyTorch around the B200 kernels of this package, shaped after the reference's Keras
model (rwkv6_model.py): EmbeddingLayer (:219-239), RWKV_Block (:197-215: x + TimeMix(LN(x)); x + ChannelMix(LN(x))),
TimeMix (:116-196), ChannelMix (:48-83), OutputLayer (:240-259), RWKV6 (:260-276).

Hand-written kernels: the WKV recurrence (``ops.wkv6``), the token-shift interpolations in front of the projections
(``time_mix_inputs``) and the per-head GroupNorm + gate behind it (``group_norm``).  The dense projections, layer norms,
embedding and loss are library calls (cuBLAS / ATen).  Used by ``bench.py --workload train_step`` and
``tests/test_gpu_model.py``; weights are random (no checkpoint can be loaded here).
"""
from __future__ import annotations

import torch
from torch import nn

from .group_norm import GroupNormGate
from .ops import wkv6
from .time_mix_inputs import TimeMixInputs, shift_mix_vector


class TimeMix(nn.Module):
    def __init__(self, hidden_size: int, head_size: int = 64, decomposer_size: int = 32, decay_rank: int = 64):
        super().__init__()
        D = hidden_size
        self.head_size, self.num_heads = head_size, D // head_size
        self.mix_inputs = TimeMixInputs(D, decomposer_size)
        self.dense_r = nn.Linear(D, D, bias=False)
        self.dense_k = nn.Linear(D, D, bias=False)
        self.dense_v = nn.Linear(D, D, bias=False)
        self.dense_g = nn.Linear(D, D, bias=False)
        # dense_w is a DecomposerDense(hidden_size, rank, use_bias=True): tanh(x A) B + b
        self.w_a = nn.Linear(D, decay_rank, bias=False)
        self.w_b = nn.Linear(decay_rank, D, bias=True)
        self.time_faaaa = nn.Parameter(torch.randn(self.num_heads, head_size) * 0.1)   # u, kept in fp32
        self.group_norm = GroupNormGate(D, head_size)
        self.dense_o = nn.Linear(D, D, bias=False)
        with torch.no_grad():
            self.w_b.bias.uniform_(-6.0, -1.0)  # decays exp(-exp(w)) spread between slow and fast channels

    def forward(self, x):
        xr, xk, xv, xw, xg = self.mix_inputs(x)
        r, k, v = self.dense_r(xr), self.dense_k(xk), self.dense_v(xv)
        w = self.w_b(torch.tanh(self.w_a(xw)))
        g = torch.nn.functional.silu(self.dense_g(xg))
        y = wkv6(r, k, v, w, self.time_faaaa, self.head_size)
        return self.dense_o(self.group_norm(y, g))


class ChannelMix(nn.Module):
    def __init__(self, hidden_size: int, expand_size: int):
        super().__init__()
        self.time_mix_k = nn.Parameter(torch.rand(hidden_size))
        self.time_mix_r = nn.Parameter(torch.rand(hidden_size))
        self.dense_key = nn.Linear(hidden_size, expand_size, bias=False)
        self.dense_value = nn.Linear(expand_size, hidden_size, bias=False)
        self.dense_receptance = nn.Linear(hidden_size, hidden_size, bias=False)

    def forward(self, x):
        xk = shift_mix_vector(x, self.time_mix_k)
        xr = shift_mix_vector(x, self.time_mix_r)
        k = torch.relu(self.dense_key(xk)) ** 2
        return torch.sigmoid(self.dense_receptance(xr)) * self.dense_value(k)


class Block(nn.Module):
    def __init__(self, hidden_size, head_size, decomposer_size, expand_size, decay_rank):
        super().__init__()
        self.layer_norm_att = nn.LayerNorm(hidden_size, eps=1e-5)
        self.layer_norm_ffn = nn.LayerNorm(hidden_size, eps=1e-5)
        self.time_mix = TimeMix(hidden_size, head_size, decomposer_size, decay_rank)
        self.channel_mix = ChannelMix(hidden_size, expand_size)

    def forward(self, x):
        x = x + self.time_mix(self.layer_norm_att(x))
        return x + self.channel_mix(self.layer_norm_ffn(x))


class RWKV6(nn.Module):
    def __init__(self, num_layers: int, vocabulary_size: int, hidden_size: int, head_size: int = 64, decomposer_size: int = 32,
                 expand_size: int | None = None, decay_rank: int = 64):
        super().__init__()
        expand_size = expand_size or int(hidden_size * 3.5)
        self.embedding = nn.Embedding(vocabulary_size, hidden_size)
        self.embedding_ln = nn.LayerNorm(hidden_size, eps=1e-5)
        self.blocks = nn.ModuleList(Block(hidden_size, head_size, decomposer_size, expand_size, decay_rank) for _ in range(num_layers))
        self.output_ln = nn.LayerNorm(hidden_size, eps=1e-5)
        self.output_layer = nn.Linear(hidden_size, vocabulary_size, bias=False)
        with torch.no_grad():
            self.embedding.weight.normal_(0.0, 0.02)

    def forward(self, tokens, checkpoint_blocks: bool = False):
        """``checkpoint_blocks``: keep only each block's input for the backward and recompute the block there (a
        24-layer, 2048-wide model at 32 k tokens per step would otherwise hold about 6 GB of activations per block)."""
        x = self.embedding_ln(self.embedding(tokens))
        for blk in self.blocks:
            if checkpoint_blocks and torch.is_grad_enabled():
                from torch.utils.checkpoint import checkpoint
                x = checkpoint(blk, x, use_reentrant=False)
            else:
                x = blk(x)
        return self.output_layer(self.output_ln(x))

    def to_bf16_(self):
        """bf16 weights for the projections and norms; the small fp32 operands of the kernels (u, GroupNorm scale and
        offset, the mixing vectors) stay fp32."""
        keep = ("time_faaaa", "group_norm.scale", "group_norm.offset", "time_mix_x", "time_mix_k", "time_mix_r")
        for name, p in self.named_parameters():
            if not name.endswith(keep):
                p.data = p.data.to(torch.bfloat16)
        return self
