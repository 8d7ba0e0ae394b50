"""A minimal stand-in for the patched reference module ``M`` built from the golden fixture
(tests/golden/moe_tiny.npz): it offers exactly the ``self`` contract the drop-in forwards read
(nanov41/_ref_patched_model.py:809-921 Gate / Expert / MoE), restated for tests."""
import types

import torch
import torch.nn as nn
import torch.nn.functional as F

from conftest import bf16_from_bits


class Linear(nn.Module):
    def __init__(self, w):
        super().__init__()
        self.weight = nn.Parameter(w.clone())
        self.scale = None

    def forward(self, x):
        return F.linear(x, self.weight)


class Expert(nn.Module):
    """_ref_patched_model.py:847-868."""

    def __init__(self, w1, w2, w3, limit):
        super().__init__()
        self.w1, self.w2, self.w3 = Linear(w1), Linear(w2), Linear(w3)
        self.swiglu_limit = limit

    def forward(self, x, weights=None):
        dtype = x.dtype
        gate, up = self.w1(x).float(), self.w3(x).float()
        if self.swiglu_limit > 0:
            up = torch.clamp(up, min=-self.swiglu_limit, max=self.swiglu_limit)
            gate = torch.clamp(gate, max=self.swiglu_limit)
        h = F.silu(gate) * up
        if weights is not None:
            h = weights * h
        return self.w2(h.to(dtype))


class Gate(nn.Module):
    """_ref_patched_model.py:809-844 with score_func='sqrtsoftplus', norm_topk_prob=True."""

    def __init__(self, weight, bias, topk, route_scale):
        super().__init__()
        self.weight = nn.Parameter(weight.clone())
        self.bias = nn.Parameter(bias.clone())
        self.topk, self.route_scale = topk, route_scale

    def forward(self, x, image_mask=None):
        scores = F.softplus(F.linear(x.float(), self.weight.float())).sqrt()
        indices = (scores + self.bias).topk(self.topk, dim=-1)[1]
        weights = scores.gather(1, indices)
        weights = weights / (weights.sum(dim=-1, keepdim=True) + 1e-20)
        return weights * self.route_scale, indices


class MoE(nn.Module):
    """_ref_patched_model.py:871-921 (single rank)."""

    def __init__(self, g):
        super().__init__()
        w1, w2, w3 = (bf16_from_bits(g[n]) for n in ("w1", "w2", "w3"))
        E = w1.shape[0]
        limit = float(g["swiglu_limit"])
        self.dim = w1.shape[2]
        self.n_routed_experts = self.n_local_experts = E
        self.experts_start_idx, self.experts_end_idx = 0, E
        self.gate = Gate(bf16_from_bits(g["gate_weight"]), torch.from_numpy(g["gate_bias"]),
                         g["route_indices"].shape[1], float(g["route_scale"]))
        self.experts = nn.ModuleList([Expert(w1[i], w2[i], w3[i], limit) for i in range(E)])
        self.shared_experts = Expert(*(bf16_from_bits(g["shared_" + n]) for n in ("w1", "w2", "w3")),
                                     limit)

    def forward(self, x, image_mask=None):
        shape = x.size()
        x = x.view(-1, self.dim)
        weights, indices = self.gate(x)
        y = torch.zeros_like(x, dtype=torch.float32)
        for i in range(self.n_routed_experts):
            idx, top = torch.where(indices == i)
            if idx.numel():
                y[idx] += self.experts[i](x[idx], weights[idx, top, None])
        y += self.shared_experts(x)
        return y.type_as(x).view(shape)


def make_M():
    """A fresh namespace with a ``MoE`` class, like the module object install(M) patches."""
    return types.SimpleNamespace(MoE=type("MoE", (MoE,), {}))
