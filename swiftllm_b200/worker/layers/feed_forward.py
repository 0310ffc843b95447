"""Feed-forward sublayers with the squared-ReLU activation: a dense one and a mixture of experts.

Mixture of experts.  Router logits are an fp32 GEMM; `moe_route` turns them into a [T, experts] weight matrix (softmax over the
`top` largest logits at their experts, exact zeros elsewhere).  The experts' up projections are ONE GEMM over the row-wise
concatenation of their weights, the activation kernel multiplies every expert's slice by the token's weight for that expert,
and ONE down GEMM over the column-wise concatenation then sums the chosen experts' weighted outputs.  No token permutation,
no host sync, fixed shapes (CUDA-graph friendly); the price is experts / top times the FLOPs of a gathered formulation, which
only matters once the step is compute-bound (a decode step streams every expert's weights anyway as soon as
tokens * top >= experts)."""
import torch

from swiftllm_b200.worker.kernels.linear import linear
from swiftllm_b200.worker.kernels.parallel_block import moe_relu2_scale_inplace, moe_route, relu2_inplace


class Relu2FeedForward:
    def __init__(self, spec, weight):
        self.spec, self.weight = spec, weight

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        u = linear(h, self.weight.up)
        relu2_inplace(u)
        return linear(u, self.weight.down)


class Relu2MixtureOfExperts:
    def __init__(self, spec, weight):
        self.spec, self.weight = spec, weight

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        w = self.weight
        logits = linear(h.float(), w.router)                    # fp32 GEMM (TF32 stays off)
        weights = moe_route(logits, self.spec.top)
        u = linear(h, w.up)                                     # [T, experts * ff]
        moe_relu2_scale_inplace(u, weights, self.spec.ff)
        return linear(u, w.down)


def build_feed_forward(spec, weight):
    if spec is None:
        return None
    return (Relu2FeedForward if spec.kind == "dense" else Relu2MixtureOfExperts)(spec, weight)
