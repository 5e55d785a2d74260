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

from . import decode_stages as ds
from .channel_mix_ops import relu_sq, sigmoid_mul
from .group_norm import GroupNormGate
from .group_norm import groupnorm_gate_forward_raw
from .ops import wkv6, wkv6_decode, wkv6_with_state
from .time_mix_inputs import TimeMixInputs, shift_mix_vector


_SIDE_STREAMS = {}


def _side_streams(device, n):
    """Streams for the independent matrix products of a decode step.  Each product streams its weights once and alone
    does not fill the memory system (16 rows: 70-80 % of the copy bandwidth, and the small LoRA products are pure
    latency), so independent ones are issued side by side; under CUDA-graph capture they become parallel branches."""
    key = (device.type, device.index)
    pool = _SIDE_STREAMS.setdefault(key, [])
    while len(pool) < n:
        pool.append(torch.cuda.Stream(device))
    return pool[:n]


class _Fork:
    """``with _Fork(device, n) as f: f.run(i, fn)`` runs fn on side stream i after everything issued so far on the
    current stream; leaving the block makes the current stream wait for all of them."""

    def __init__(self, device, n):
        self.main = torch.cuda.current_stream(device)
        self.streams = _side_streams(device, n)

    def __enter__(self):
        for st in self.streams:
            st.wait_stream(self.main)
        return self

    def run(self, i, fn):
        with torch.cuda.stream(self.streams[i]):
            return fn()

    def __exit__(self, *exc):
        for st in self.streams:
            self.main.wait_stream(st)
        return False


class TimeMix(nn.Module):
    parallel_decode_products = True    # measured per 7B-shape block inside a CUDA graph: 161 us against 171 us serial

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
        y = wkv6(r, k, v, w, self.time_faaaa, self.head_size)
        return self.dense_o(self.group_norm(y, self.dense_g(xg), gate_is_raw=True))   # SiLU of the gate inside the kernel

    def _project(self, xr, xk, xv, xw, xg):
        r, k, v = self.dense_r(xr), self.dense_k(xk), self.dense_v(xv)
        w = self.w_b(torch.tanh(self.w_a(xw)))
        return r, k, v, w, torch.nn.functional.silu(self.dense_g(xg))

    @torch.no_grad()
    def prefill(self, x):
        """Forward over a whole prompt; returns the output and the layer state (last input token, WKV state)."""
        r, k, v, w, g = self._project(*self.mix_inputs(x))
        y, S = wkv6_with_state(r, k, v, w, self.time_faaaa, self.head_size)
        gn = self.group_norm
        return self.dense_o(groupnorm_gate_forward_raw(y, g.contiguous(), gn.scale, gn.offset, gn.epsilon)), (x[:, -1:].clone(), S)

    @torch.no_grad()
    def decode(self, x, state):
        """One token ([B,1,D]) with the carried state; the state tensors are updated in place."""
        x_prev, S = state
        mi = self.mix_inputs
        B = x.shape[0]
        xs = x_prev - x                                                       # TimeShift for a single step
        x_mix = x + xs * mi.time_mix_x.to(x.dtype)
        h = torch.tanh(x_mix.reshape(B, -1) @ mi.dense_a.to(x.dtype)).reshape(B, 5, mi.decomposer_size).transpose(0, 1)
        l = torch.baddbmm(mi.bias_b.to(x.dtype), h, mi.dense_b.to(x.dtype)).reshape(5, B, 1, -1)
        r, k, v, w, g = self._project(*(x + xs * l))
        y, _ = wkv6_decode(r, k, v, w, self.time_faaaa, self.head_size, state=S, out_state=S)
        gn = self.group_norm
        out = self.dense_o(groupnorm_gate_forward_raw(y, g.contiguous(), gn.scale, gn.offset, gn.epsilon))
        x_prev.copy_(x)
        return out


    def _stacked_rkvg(self):
        """The kernels of dense_r, dense_k, dense_v, dense_g as one [4, D, D] tensor for the batched decode product.  Built
        on first use; the four parameters are re-pointed at its slices, so nothing is stored twice and in-place updates
        of a parameter (``weights.load_pth``) reach it.  Rebuilt when a parameter was replaced (dtype or device change)."""
        lins = (self.dense_r, self.dense_k, self.dense_v, self.dense_g)
        st = getattr(self, "_rkvg_stack", None)
        if st is None or any(l.weight.data_ptr() != st[j].data_ptr() or l.weight.dtype != st.dtype for j, l in enumerate(lins)):
            st = torch.stack([l.weight.data for l in lins])
            for j, l in enumerate(lins):
                l.weight.data = st[j]
            self._rkvg_stack = st
        return st

    @torch.no_grad()
    def decode_fused(self, x, ln, state):
        """The block's time-mix half for one token with fused element-wise stages: x [B, D] is the block input (before
        its LayerNorm ``ln``); returns x + TimeMix(LN(x)).  9 launches: 5 matrix products, tanh and 3 kernels of this package."""
        x_prev, S = state
        mi, gn, lin = self.mix_inputs, self.group_norm, torch.nn.functional.linear
        B, D = x.shape
        x_mix, _, xa, xs = ds.ln_shift_mix(x, ln.weight, ln.bias, ln.eps, x_prev.view(B, D), mi.time_mix_x, want_xa_xs=True)
        m = ds.lora_mix(x_mix @ mi.dense_a, mi.dense_b, mi.bias_b, xa, xs)            # r, k, v, g, w
        # r, k, v, g in one batched product over the stacked kernels (the four separate 16-row products spend 9.7 us each,
        # half of it ramp-up and tail: 37 us; batched 24 us), on a side stream beside the latency-bound decay LoRA chain
        stack = self._stacked_rkvg()
        if self.parallel_decode_products:
            with _Fork(x.device, 1) as f:
                y4 = f.run(0, lambda: torch.bmm(m[:4], stack.transpose(1, 2)))
                w = torch.addmm(self.w_b.bias, torch.tanh(lin(m[4], self.w_a.weight)), self.w_b.weight.t())
        else:
            y4 = torch.bmm(m[:4], stack.transpose(1, 2))
            w = torch.addmm(self.w_b.bias, torch.tanh(lin(m[4], self.w_a.weight)), self.w_b.weight.t())
        r, k, v, g_raw = y4[0], y4[1], y4[2], y4[3]
        z = ds.wkv6_decode_gated(r, k, v, w, self.time_faaaa, g_raw, gn.scale, gn.offset, gn.epsilon, self.head_size, S)
        return torch.addmm(x, z, self.dense_o.weight.t())


class ChannelMix(nn.Module):
    parallel_decode_products = False   # measured: the receptance product beside the key -> value chain is 1 % slower

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
        k = relu_sq(self.dense_key(xk))                                   # one kernel per direction instead of relu, pow
        return sigmoid_mul(self.dense_receptance(xr), self.dense_value(k))   # ... and of sigmoid, mul

    @torch.no_grad()
    def prefill(self, x):
        return self.forward(x), x[:, -1:].clone()

    @torch.no_grad()
    def decode(self, x, x_prev):
        xs = x_prev - x
        k = torch.relu(self.dense_key(x + xs * self.time_mix_k.to(x.dtype))) ** 2
        out = torch.sigmoid(self.dense_receptance(x + xs * self.time_mix_r.to(x.dtype))) * self.dense_value(k)
        x_prev.copy_(x)
        return out


    @torch.no_grad()
    def decode_fused(self, x, ln, x_prev):
        """x [B, D] is the block's running activation (before ``ln``); returns x + ChannelMix(LN(x)).  6 launches."""
        lin = torch.nn.functional.linear
        xk, xr, _, _ = ds.ln_shift_mix(x, ln.weight, ln.bias, ln.eps, x_prev.view(x.shape), self.time_mix_k, self.time_mix_r)
        if self.parallel_decode_products:
            with _Fork(x.device, 1) as f:       # the receptance product beside the key -> value chain
                rr = f.run(0, lambda: lin(xr, self.dense_receptance.weight))
                kv = lin(ds.relu_sq(lin(xk, self.dense_key.weight)), self.dense_value.weight)
        else:
            rr = lin(xr, self.dense_receptance.weight)
            kv = lin(ds.relu_sq(lin(xk, self.dense_key.weight)), self.dense_value.weight)
        return ds.sigmoid_mul_add(x, rr, kv)


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

    @torch.no_grad()
    def prefill(self, x):
        o, st_att = self.time_mix.prefill(self.layer_norm_att(x))
        x = x + o
        o, st_ffn = self.channel_mix.prefill(self.layer_norm_ffn(x))
        return x + o, (st_att, st_ffn)

    @torch.no_grad()
    def decode(self, x, state, fused: bool = True):
        st_att, st_ffn = state
        if fused:
            B, _, D = x.shape
            x2 = self.time_mix.decode_fused(x.reshape(B, D), self.layer_norm_att, st_att)
            return self.channel_mix.decode_fused(x2, self.layer_norm_ffn, st_ffn).view(B, 1, D)
        x = x + self.time_mix.decode(self.layer_norm_att(x), st_att)
        return x + self.channel_mix.decode(self.layer_norm_ffn(x), st_ffn)


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

    @torch.no_grad()
    def prefill(self, tokens):
        """Prompt pass: logits of the last position [B,1,V] and the per-layer states for ``decode``."""
        x = self.embedding_ln(self.embedding(tokens))
        states = []
        for blk in self.blocks:
            x, st = blk.prefill(x)
            states.append(st)
        return self.output_layer(self.output_ln(x[:, -1:])), states

    @torch.no_grad()
    def decode(self, token, states, fused: bool = True):
        """One new token per sequence ([B,1] ids); ``states`` is updated in place (CUDA-graph friendly).  ``fused``:
        the element-wise stages of every block run as this package's decode-stage kernels (15 launches per block
        instead of about 40 framework operations); False keeps the plain framework operations."""
        x = self.embedding_ln(self.embedding(token))
        for blk, st in zip(self.blocks, states):
            x = blk.decode(x, st, fused)
        return self.output_layer(self.output_ln(x))

    def to_bf16_(self):
        """bf16 weights for the projections and norms; the small fp32 operands of the kernels (u, GroupNorm scale and
        offset, the mixing vectors) stay fp32."""
        keep = ("time_faaaa", "group_norm.scale", "group_norm.offset", "time_mix_x", "time_mix_k", "time_mix_r")
        for name, p in self.named_parameters():
            if not name.endswith(keep):
                p.data = p.data.to(torch.bfloat16)
        return self
