"""TEST INFRASTRUCTURE ONLY.  float64 numpy softmax cross-entropy (mean over rows with a valid target) and its gradient
with respect to the logits, the loss the training-step benchmark puts behind the model
(``torch.nn.functional.cross_entropy`` semantics).  The reference has no trainer (normal_trainer.py and
jax_distribution_trainer.py are empty), so there is nothing of its own to pin this against: "parity unpinned" for this
stage; tests/test_lm_loss.py additionally checks the kernel against torch's own fp32 cross_entropy and autograd.
Only tests may import this module."""
import numpy as np


def lm_loss(logits, targets):
    """logits [rows, V], targets [rows] (out-of-range = ignored).  Returns (mean loss over all rows, d loss / d logits).
    The mean is over all rows, ignored ones counting as zero (the kernel's convention: scale = 1 / rows)."""
    z = np.asarray(logits, np.float64)
    t = np.asarray(targets)
    rows, V = z.shape
    m = z.max(-1, keepdims=True)
    lse = m[:, 0] + np.log(np.exp(z - m).sum(-1))
    valid = (t >= 0) & (t < V)
    tc = np.where(valid, t, 0)
    loss_rows = np.where(valid, lse - z[np.arange(rows), tc], 0.0)
    p = np.exp(z - lse[:, None])
    p[np.arange(rows), tc] -= 1.0
    p *= valid[:, None] / rows
    return loss_rows.mean(), p
