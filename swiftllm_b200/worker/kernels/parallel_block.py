"""Kernels of parallel decoder blocks with an fp32 residual stream (csrc/parallel_block.cu): fused residual add + RMS norm,
row-strided RMS norm, squared ReLU, and the mixture-of-experts router with its weight-applying activation.  The storage
dtype of activations may be float16, bfloat16 or float32; sums, norms and the router are fp32 in every case."""
import torch

from swiftllm_b200 import _lib


def add_rmsnorm_f32(residual: torch.Tensor, a, b, weight: torch.Tensor, eps: float, out: torch.Tensor = None) -> torch.Tensor:
    """residual (fp32 [T, W], updated in place) += a + b (either may be None); returns rmsnorm(residual) * weight in
    weight's dtype."""
    assert residual.dtype == torch.float32 and residual.is_contiguous() and weight.is_contiguous()
    _lib.require_device(residual)
    T, W = residual.shape
    if out is None:
        out = torch.empty((T, W), dtype=weight.dtype, device=residual.device)
    for x in (a, b):
        assert x is None or (x.dtype == weight.dtype and x.is_contiguous() and x.shape == residual.shape)
    _lib.check(_lib.lib().sllm_add_rmsnorm_f32(residual.data_ptr(), _lib.ptr(a), _lib.ptr(b), weight.data_ptr(), out.data_ptr(),
                                               eps, T, W, _lib.dtype_tag_f32(weight.dtype), _lib.stream()), "add_rmsnorm_f32")
    return out


def rmsnorm_strided(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS norm of x [T, n] (a column slice of a wider matrix is fine) -> new contiguous [T, n]."""
    assert x.dim() == 2 and x.stride(1) == 1 and weight.is_contiguous() and weight.dtype == x.dtype
    _lib.require_device(x)
    T, n = x.shape
    out = torch.empty((T, n), dtype=x.dtype, device=x.device)
    _lib.check(_lib.lib().sllm_rmsnorm_strided(x.data_ptr(), x.stride(0) if T > 1 else max(x.stride(0), n), weight.data_ptr(),
                                               out.data_ptr(), n, eps, T, n, _lib.dtype_tag_f32(x.dtype), _lib.stream()),
               "rmsnorm_strided")
    return out


def relu2_inplace(x: torch.Tensor):
    assert x.is_contiguous()
    _lib.require_device(x)
    _lib.check(_lib.lib().sllm_relu2_inplace(x.data_ptr(), x.numel(), _lib.dtype_tag_f32(x.dtype), _lib.stream()), "relu2_inplace")


def moe_route(logits: torch.Tensor, top: int) -> torch.Tensor:
    """logits fp32 [T, E] -> routing weights fp32 [T, E]: softmax over each row's `top` largest logits, 0 elsewhere."""
    assert logits.dtype == torch.float32 and logits.is_contiguous()
    _lib.require_device(logits)
    w = torch.empty_like(logits)
    _lib.check(_lib.lib().sllm_moe_route(logits.data_ptr(), w.data_ptr(), logits.shape[0], logits.shape[1], top, _lib.stream()),
               "moe_route")
    return w


def moe_relu2_scale_inplace(u: torch.Tensor, weights: torch.Tensor, ff: int):
    """u [T, E * ff] = relu(u)^2 * weights[t, column // ff]."""
    assert u.is_contiguous() and weights.dtype == torch.float32 and weights.is_contiguous()
    _lib.require_device(u)
    T, E = weights.shape
    assert u.shape == (T, E * ff)
    _lib.check(_lib.lib().sllm_moe_relu2_scale_inplace(u.data_ptr(), weights.data_ptr(), T, E, ff, _lib.dtype_tag_f32(u.dtype),
                                                       _lib.stream()), "moe_relu2_scale_inplace")
