"""Generates tests/golden/model_pth_small.npz by running the reference's own plain-torch RWKV-6 model
(rwkv_v6_demo.py: class RWKV) on CPU in float64, with the weights of ``oracle.rwkv6_model_oracle.synthetic_pth``
loaded through ``load_state_dict`` (so the tensor names are the ``.pth`` names) and fixed token ids.  The fixture
holds the token ids, the logits and the arguments of ``synthetic_pth``; the weights are rebuilt from the seed.

    REFERENCE_ROOT=/path/to/STAR-RWKV6 python tests/golden/make_golden_model.py
"""
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.environ.get("REFERENCE_ROOT", "/root/reference"))

import rwkv_v6_demo as ref  # noqa: E402  (the reference's module)
from oracle import rwkv6_model_oracle as mo  # noqa: E402

cfg = dict(num_layers=2, hidden=128, head_size=64, vocab=97, mix_rank=32, decay_rank=64, seed=5)
sd = mo.synthetic_pth(**cfg)
args = types.SimpleNamespace(n_layer=cfg["num_layers"], n_embd=cfg["hidden"], vocab_size=cfg["vocab"],
                             head_size_a=cfg["head_size"], head_size_divisor=8)
model = ref.RWKV(args).double()
missing = model.load_state_dict({k: torch.from_numpy(v).double() for k, v in sd.items()}, strict=True)
tokens = np.random.default_rng(11).integers(0, cfg["vocab"], size=(2, 24))
with torch.no_grad():
    logits = model(torch.from_numpy(tokens)).numpy()
np.savez_compressed(os.path.join(HERE, "model_pth_small.npz"), tokens=tokens, logits=logits,
                    **{"cfg_" + k: np.int64(v) for k, v in cfg.items()})
mine = mo.forward(sd, tokens, cfg["head_size"])
print("reference vs restatement, max abs:", np.abs(mine - logits).max(), "of", np.abs(logits).max())
