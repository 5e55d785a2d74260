"""PyTorch ``RWKVKernelOperator``: same constructor, call signature, validation and dtype
policy as the reference operator (rwkv_kernel/torch_rwkv_kernel.py:7-168), backed by the
B200 library.

Differences from the reference, all toward its documented intent
(rwkv_kernel/__init__.py:14-37):
* ``max_sequence_length`` is advisory: T is a run-time value, there is no compile-time cap.
* the state path works (the reference's calls a symbol its extension does not export) and
  accepts fp32 / bf16 states for any input dtype;
* returned and initial states use the layout ``S[b, h, key, value]`` of the reference's
  non-CUDA operator (rwkv_kernel/ops_rwkv_kernal.py:85-91);
* ``u`` may be fp32 while r, k, v, w are bf16 (fp32 bonus, bf16 activations);
* kernels run on torch's current stream of the tensors' device.
"""
from __future__ import annotations

import torch

from .. import _lib, ops


class RWKVKernelOperator:
    def __init__(self, head_size, max_sequence_length=None, variant="auto", segments=1):
        """``segments``: 1 = one kernel walks each (batch, head) sequence; an integer G > 1 or "auto" cuts every
        sequence into G pieces along T that run concurrently (worth it when B*H is small; bf16, head size 64)."""
        self.head_size = int(head_size)
        self.max_sequence_length = max_sequence_length
        self.variant = _lib.VARIANTS[variant] if isinstance(variant, str) else int(variant)
        self.segments = segments

    def __call__(self, r, k, v, w, u, return_state=False, init_state=None, state_map=None):
        B, T, C = r.shape
        assert C % self.head_size == 0
        H = C // self.head_size
        if not isinstance(u, torch.Tensor):
            u = u.value  # a Keras variable (rwkv6_model.py:155 passes time_faaaa)

        assert r.is_cuda and k.is_cuda and v.is_cuda and w.is_cuda and u.is_cuda
        assert r.device == k.device == v.device == w.device == u.device
        assert r.dtype == k.dtype == v.dtype == w.dtype
        assert r.dtype in (torch.float32, torch.bfloat16, torch.float16)
        assert u.dtype == r.dtype or u.dtype == torch.float32
        assert u.numel() == C, "u must hold num_heads*head_size values"
        u = u.reshape(H, self.head_size)
        if not u.is_contiguous():
            u = u.contiguous()

        if init_state is not None:
            assert len(init_state.shape) in (3, 4), \
                "init_state must be (state_kinds<=B, H, N, N) or (H, N, N)"
            if len(init_state.shape) == 3:
                init_state = init_state[None, :]
            assert init_state.shape[1:] == (H, self.head_size, self.head_size) and init_state.shape[0] <= B, \
                "init_state must be (state_kinds<=B, H, N, N) or (H, N, N)"
            assert init_state.dtype in (torch.float32, torch.bfloat16), "init_state must be fp32 or bf16"
            assert init_state.is_cuda and init_state.device == r.device
            init_state = init_state.contiguous()

        if state_map is not None:
            if isinstance(state_map, list):
                state_map = torch.tensor(state_map, dtype=torch.int64)
            assert isinstance(state_map, torch.Tensor) and state_map.dtype in (torch.int32, torch.int64), \
                "state_map must be an int64 array of length B"
            state_map = state_map.to(torch.int64)
            assert state_map.shape == (B,), "state_map must have shape (B,)"

        if return_state:
            if init_state is None:
                assert state_map is None, "state_map needs an init_state"
            else:
                n_state = init_state.shape[0]
                if state_map is None:
                    assert n_state == 1 or n_state == B, "state_map cannot be inferred; pass it explicitly"
                else:
                    assert bool((state_map >= 0).all()) and bool((state_map < n_state).all()), \
                        f"state_map values must lie in [0, {n_state})"
                    state_map = state_map.to(r.device).contiguous()
            if (T == 1 and self.head_size == 64 and r.is_contiguous()
                    and (init_state is None or init_state.dtype == torch.float32)):
                with torch.no_grad():  # decode step: dedicated state-streaming kernel
                    return ops.wkv6_decode(r, k, v, w, u, self.head_size, state=init_state, state_map=state_map)
            return ops.wkv6_with_state(r, k, v, w, u, self.head_size, init_state=init_state, state_map=state_map,
                                       variant=self.variant)
        assert init_state is None and state_map is None, "init_state / state_map need return_state=True"
        G = self.segments
        if G != 1 and r.dtype == torch.bfloat16 and self.head_size == 64 and self.variant != _lib.VARIANT_SEQ and r.is_contiguous():
            from .. import segments as seg
            if G == "auto":
                G = seg.auto_segments(B, T, H)
            if G > 1 and T % G == 0:
                return seg.wkv6_segmented(r, k, v, w, u, self.head_size, segments=G), None
        return ops.wkv6(r, k, v, w, u, self.head_size, variant=self.variant), None
