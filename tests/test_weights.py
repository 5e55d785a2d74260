"""Weight import: a ``.pth`` state dict into this package's model.

CPU: the model oracle against logits of the reference's own plain-torch model (fixture made by
tests/golden/make_golden_model.py), the name mapping both ways, error behaviour.
GPU: the imported model on the kernels of this package against the oracle: whole-sequence logits (fp32: max relative
error 1e-4; with every weight, activation and the logits themselves in bf16 through two blocks: 5e-2 of the largest
logit at worst and 1e-2 in the root mean square, the per-kernel bf16 bound of 2e-2 being tested kernel by kernel
elsewhere) and prefill followed by token-by-token decode."""
import os

import numpy as np
import pytest
import torch

from oracle import rwkv6_model_oracle as mo

TOL_F32 = 1e-4
TOL_BF16_MODEL, TOL_BF16_MODEL_RMS = 5e-2, 1e-2


def fixture(golden_dir):
    z = np.load(os.path.join(golden_dir, "model_pth_small.npz"))
    cfg = {k[4:]: int(z[k]) for k in z.files if k.startswith("cfg_")}
    return cfg, mo.synthetic_pth(**cfg), z["tokens"], z["logits"]


def test_oracle_matches_reference_model(golden_dir):
    cfg, sd, tokens, logits = fixture(golden_dir)
    mine = mo.forward(sd, tokens, cfg["head_size"])
    assert np.abs(mine - logits).max() <= 1e-12 * np.abs(logits).max()


def test_config_from_pth(golden_dir):
    from star_rwkv6_b200.weights import config_from_pth
    cfg, sd, _, _ = fixture(golden_dir)
    got = config_from_pth(sd)
    assert got == dict(num_layers=cfg["num_layers"], vocabulary_size=cfg["vocab"], hidden_size=cfg["hidden"],
                       head_size=cfg["head_size"], decomposer_size=cfg["mix_rank"], expand_size=448,
                       decay_rank=cfg["decay_rank"])
    bad = dict(sd)
    bad["blocks.0.att.time_faaaa"] = np.zeros((3, 64), np.float32)
    with pytest.raises(ValueError):
        config_from_pth(bad)


def test_round_trip_and_errors(golden_dir):
    from star_rwkv6_b200.model import RWKV6
    from star_rwkv6_b200.weights import config_from_pth, load_pth, to_pth
    _, sd, _, _ = fixture(golden_dir)
    model = load_pth(RWKV6(**config_from_pth(sd)), sd)
    back = to_pth(model)
    assert set(back) == set(sd)
    for name, val in sd.items():
        assert tuple(back[name].shape) == val.shape, name
        assert np.array_equal(back[name].numpy(), val), name
    # every parameter of the model was filled: a second, different dict changes all of them
    other = mo.synthetic_pth(**{**fixture(golden_dir)[0], "seed": 6})
    before = {n: p.detach().clone() for n, p in model.named_parameters()}
    load_pth(model, other)
    for n, p in model.named_parameters():
        assert not torch.equal(before[n], p.detach()), n
    with pytest.raises(KeyError):
        load_pth(model, {**sd, "blocks.0.att.unknown": np.zeros(1, np.float32)})
    short = dict(sd)
    del short["blocks.1.ffn.value.weight"]
    with pytest.raises(KeyError):
        load_pth(model, short)


def test_reference_layer_layouts(golden_dir):
    from star_rwkv6_b200.weights import reference_layer_weights
    cfg, sd, _, _ = fixture(golden_dir)
    lw = reference_layer_weights(sd)
    D, R = cfg["hidden"], cfg["mix_rank"]
    assert lw["rwkv_blocks.1.time_mix.dense_r.kernel"].shape == (D, D)
    assert np.array_equal(lw["rwkv_blocks.1.time_mix.dense_r.kernel"], sd["blocks.1.att.receptance.weight"].T)
    assert np.array_equal(lw["rwkv_blocks.0.time_mix.dense_xr.dense_a.kernel"],
                          sd["blocks.0.att.time_maa_w1"][:, 3 * R:4 * R])       # order w, k, v, r, g
    assert np.array_equal(lw["rwkv_blocks.0.time_mix.dense_xw.dense_b.kernel"], sd["blocks.0.att.time_maa_w2"][0])
    assert np.array_equal(lw["rwkv_blocks.0.time_mix.dense_w.dense_b.bias"], sd["blocks.0.att.time_decay"].reshape(-1))
    assert lw["rwkv_blocks.0.time_mix.group_norm.scale"].shape == (D // cfg["head_size"], cfg["head_size"])
    assert lw["output_layer.output_layer.kernel"].shape == (D, cfg["vocab"])
    n_per_block = 15 + 1 + 5 + 3 + 1 + 2 + 2 + 3 + 4
    assert len(lw) == 3 + 3 + cfg["num_layers"] * n_per_block


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,tol", [(torch.float32, TOL_F32), (torch.bfloat16, TOL_BF16_MODEL)])
def test_imported_model_matches_oracle(golden_dir, dtype, tol):
    from star_rwkv6_b200.weights import from_pth
    _, sd, tokens, logits = fixture(golden_dir)
    model = from_pth(sd, "cuda", dtype)
    with torch.no_grad():
        got = model(torch.from_numpy(tokens).cuda()).float().cpu().numpy()
    assert np.abs(got - logits).max() <= tol * np.abs(logits).max()
    if dtype == torch.bfloat16:
        assert np.sqrt(((got - logits) ** 2).mean()) <= TOL_BF16_MODEL_RMS * np.abs(logits).max()


@pytest.mark.gpu
def test_imported_model_prefill_decode(golden_dir):
    from star_rwkv6_b200.weights import from_pth
    _, sd, tokens, logits = fixture(golden_dir)
    model = from_pth(sd, "cuda", torch.float32)
    tok = torch.from_numpy(tokens).cuda()
    P = 16
    out, states = model.prefill(tok[:, :P])
    scale = np.abs(logits).max()
    assert np.abs(out[:, 0].cpu().numpy() - logits[:, P - 1]).max() <= TOL_F32 * scale
    for t in range(P, tokens.shape[1]):
        out = model.decode(tok[:, t:t + 1], states)
        assert np.abs(out[:, 0].cpu().numpy() - logits[:, t]).max() <= TOL_F32 * scale, t


def test_stacked_projection_kernels_follow_parameters(golden_dir):
    """The [4, D, D] stack behind the batched decode product shares storage with dense_r/k/v/g: an in-place load reaches
    it, a replaced parameter (dtype change) rebuilds it."""
    from star_rwkv6_b200.model import RWKV6
    from star_rwkv6_b200.weights import config_from_pth, load_pth
    _, sd, _, _ = fixture(golden_dir)
    model = RWKV6(**config_from_pth(sd))
    tm = model.blocks[1].time_mix
    st = tm._stacked_rkvg()
    D = tm.dense_r.weight.shape[0]
    assert st.shape == (4, D, D) and tm.dense_k.weight.data_ptr() == st[1].data_ptr()
    load_pth(model, sd)
    assert tm._stacked_rkvg() is st
    assert np.array_equal(st[2].numpy(), sd["blocks.1.att.value.weight"])
    assert np.array_equal(st[3].numpy(), sd["blocks.1.att.gate.weight"])
    model.to_bf16_()
    st2 = tm._stacked_rkvg()
    assert st2 is not st and st2.dtype == torch.bfloat16 and tm.dense_g.weight.data_ptr() == st2[3].data_ptr()
    assert torch.equal(st2[0], tm.dense_r.weight.data)
