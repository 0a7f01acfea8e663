"""Oracle: LinearCompressed.forward on CPU torch.  Test infrastructure only.

Restates transformersurgeon/blocks/linear_compressed.py:81-105: flatten leading dims,
optional `h = x @ V^T` (V = linear_V.weight [r, in]), `y = h @ U^T + b`
(U = weight [out, r or in]), restore the leading shape.  The intermediate h is rounded
to the module dtype because each F.linear returns that dtype.
"""
import torch
import torch.nn.functional as F


def linear_compressed_forward(x, weight, bias=None, v_weight=None):
    restore = None
    if x.dim() > 2:
        restore = x.shape[:-1]
        x = x.reshape(-1, x.shape[-1])
    if v_weight is not None:
        x = F.linear(x, v_weight)
    y = F.linear(x, weight, bias)
    if restore is not None:
        y = y.reshape(*restore, y.shape[-1])
    return y


def linear_compressed_fp32(x, weight, bias=None, v_weight=None):
    """Accuracy reference: the same two products in fp32 from the (dequantized) factors."""
    f = lambda t: None if t is None else t.float()
    return linear_compressed_forward(x.float(), f(weight), f(bias), f(v_weight))
