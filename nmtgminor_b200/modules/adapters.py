"""Bottleneck adapters stored as ROWS of shared tables, one row per language / task.

Reference: onmt/models/deltalm/modules/efficient_adapters.py:18-125 (``EfficientAdapter``: residual adapter of Bapna &
Firat 2019 whose down / up projections, biases and LayerNorm scales for ``num_modules`` adapters are rows of shared
matrices, so every rank touches the same parameter tensors whichever adapter a batch selects).
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

_ACTS = {"relu": F.relu, "gelu": F.gelu, "silu": F.silu, "swish": F.silu, "tanh": torch.tanh}


class EfficientAdapter(nn.Module):
    def __init__(self, num_modules: int, input_size: int, bottleneck_size: int, activation_fn: str = "relu",
                 static_layernorm: bool = False):
        super().__init__()
        self.num_modules, self.input_size, self.bottleneck_size = num_modules, input_size, bottleneck_size
        self.static_layernorm = static_layernorm
        self.activation = _ACTS[activation_fn]
        down = torch.empty(num_modules, bottleneck_size, input_size)
        for i in range(num_modules):
            nn.init.kaiming_uniform_(down[i], a=math.sqrt(5))
        self.down_weight = nn.Parameter(down.view(num_modules, -1))
        self.down_bias = nn.Parameter(torch.zeros(num_modules, bottleneck_size))
        self.up_weight = nn.Parameter(torch.zeros(num_modules, input_size * bottleneck_size))   # zero: starts as identity
        self.up_bias = nn.Parameter(torch.zeros(num_modules, input_size))
        if not static_layernorm:
            self.layer_norm_gammas = nn.Parameter(torch.ones(num_modules, input_size))
            self.layer_norm_betas = nn.Parameter(torch.zeros(num_modules, input_size))
        for n, p in self.named_parameters():
            p.adapter, p.label = True, n

    def forward(self, x: torch.Tensor, index: int) -> torch.Tensor:
        d, b = self.input_size, self.bottleneck_size
        g = None if self.static_layernorm else self.layer_norm_gammas[index]
        beta = None if self.static_layernorm else self.layer_norm_betas[index]
        h = F.layer_norm(x.float(), (d,), g, beta)
        h = self.activation(F.linear(h, self.down_weight[index].view(b, d), self.down_bias[index]))
        h = F.linear(h, self.up_weight[index].view(d, b), self.up_bias[index])
        return x + h.to(x.dtype)
