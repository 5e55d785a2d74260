"""Fused softmax cross-entropy (loss and logit gradient in one pass) against the float64 oracle and against torch's own
fp32 cross_entropy + autograd on the same bf16 logits.  Loss: 1e-5 relative; gradient (stored in bf16): 5e-3 of its
largest entry."""
import numpy as np
import pytest
import torch

from oracle import lm_loss_oracle as lo

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,V", [(37, 1000), (5, 65536), (300, 4096), (2, 8)])
def test_lm_loss_matches_oracle_and_torch(rows, V):
    from star_rwkv6_b200.loss import lm_loss
    g = torch.Generator().manual_seed(rows + V)
    logits = (torch.randn(rows, V, generator=g) * 3).to(torch.bfloat16).cuda()
    targets = torch.randint(0, V, (rows,), generator=g).cuda()
    want_loss, want_grad = lo.lm_loss(logits.float().cpu().numpy(), targets.cpu().numpy())
    ref_in = logits.float().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(ref_in, targets)
    ref.backward()
    z = logits.clone().requires_grad_(True)
    zz = z * 1                                # a non-leaf, as a model's logits are
    loss = lm_loss(zz, targets)
    loss.backward()
    assert abs(loss.item() - want_loss) <= 1e-5 * abs(want_loss)
    assert abs(loss.item() - ref.item()) <= 1e-5 * abs(ref.item())
    got = z.grad.float().cpu().numpy()
    scale = np.abs(want_grad).max()
    assert np.abs(got - want_grad).max() <= 5e-3 * scale
    assert np.abs(got - ref_in.grad.cpu().numpy()).max() <= 5e-3 * scale


def test_lm_loss_ignored_targets_and_scaling():
    from star_rwkv6_b200.loss import lm_loss
    g = torch.Generator().manual_seed(1)
    rows, V = 16, 512
    logits = torch.randn(rows, V, generator=g).to(torch.bfloat16).cuda()
    targets = torch.randint(0, V, (rows,), generator=g)
    targets[3], targets[9] = -100, V + 5
    want_loss, want_grad = lo.lm_loss(logits.float().cpu().numpy(), targets.numpy())
    z = logits.clone().requires_grad_(True)
    loss = lm_loss(z * 1, targets.cuda())
    (loss * 2.5).backward()
    assert abs(loss.item() - want_loss) <= 1e-5 * abs(want_loss)
    got = z.grad.float().cpu().numpy()
    assert not got[3].any() and not got[9].any()
    assert np.abs(got - 2.5 * want_grad).max() <= 5e-3 * np.abs(2.5 * want_grad).max()


def test_lm_loss_falls_back_for_other_shapes():
    from star_rwkv6_b200.loss import lm_loss
    logits = torch.randn(4, 13, device="cuda").to(torch.bfloat16)      # V not a multiple of 8: library path
    targets = torch.tensor([0, 5, 12, 3], device="cuda")
    want = torch.nn.functional.cross_entropy(logits.float(), targets)
    assert abs(lm_loss(logits, targets).item() - want.item()) <= 1e-6
    # masked targets: the same definition as the fused path (zero loss for the row, mean over all rows)
    masked = torch.tensor([0, -100, 12, 40], device="cuda")
    rows = torch.nn.functional.cross_entropy(logits.float(), masked.clamp(0, 12), reduction="none")
    want = (rows[0] + rows[2]) / 4
    assert abs(lm_loss(logits, masked).item() - want.item()) <= 1e-6
