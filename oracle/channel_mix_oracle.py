"""CPU oracle (numpy float64) of the channel-mix activations: relu_square (rwkv6_model.py:47-48) and the sigmoid gate
``o = sigmoid(r) * kv`` (rwkv6_model.py:64, :83), with their gradients in closed form.  Test infrastructure only."""
import numpy as np


def relu_sq(x):
    v = np.maximum(np.asarray(x, np.float64), 0.0)
    return v * v


def relu_sq_grad(x, gout):
    return np.asarray(gout, np.float64) * 2.0 * np.maximum(np.asarray(x, np.float64), 0.0)


def _sigmoid(r):
    return 1.0 / (1.0 + np.exp(-np.asarray(r, np.float64)))


def sigmoid_mul(r, kv):
    return _sigmoid(r) * np.asarray(kv, np.float64)


def sigmoid_mul_grad(r, kv, gout):
    s, g = _sigmoid(r), np.asarray(gout, np.float64)
    return g * np.asarray(kv, np.float64) * s * (1.0 - s), g * s
