"""Multi-head diagonal state-space (S4) layers and a speech encoder built from them.

Each head owns N complex diagonal states shared by its channels (tied state-space model); every channel has its own
time step.  The convolution kernel is obtained from the generating function of the bilinear discretisation evaluated
at the roots of unity, ``K(w) = 2 / (1 + w) * sum_n C_n B_n / (g(w) / dt - A_n)`` with ``g(w) = 2 (1 - w) / (1 + w)``:
the inner sum is the Cauchy kernel computed by ``ops.sequence.compute_kernel_coefficient`` (a CUDA kernel on GPU
tensors), followed by an inverse FFT; the sequence is then convolved with the kernel by FFT.  ``bidirectional`` adds a
second kernel applied to the reversed sequence.

Reference: onmt/models/speech_recognizer/mssm/mhs4.py:31-66 (bilinear discretisation), :127-500 (``TiedStateSpaceModel``),
:502-640 (``MHS4``), :644 (``build_stacked_mh_s4``), fft_convolution.py.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops.sequence import compute_kernel_coefficient
from .layers import pack_padded
from .speech_encoders import split_audio_batch


class TiedStateSpaceModel(nn.Module):
    def __init__(self, dim: int, heads: int = 4, state: int = 32, channels: int = 1, dt_min: float = 1e-3, dt_max: float = 1e-1):
        super().__init__()
        assert dim % heads == 0
        self.Q, self.Hh, self.N, self.C = heads, dim // heads, state, channels
        self.log_neg_real = nn.Parameter(torch.log(0.5 * torch.ones(heads, state)))
        self.imag = nn.Parameter(math.pi * torch.arange(state, dtype=torch.float32)[None, :].repeat(heads, 1))
        self.log_dt = nn.Parameter(torch.rand(heads, self.Hh) * (math.log(dt_max) - math.log(dt_min)) + math.log(dt_min))
        self.B = nn.Parameter(torch.randn(heads, 1, self.Hh, state, 2) * (0.5 / state) ** 0.5)
        self.Cm = nn.Parameter(torch.randn(heads, channels, self.Hh, state, 2) * (0.5 / state) ** 0.5)
        self.D = nn.Parameter(torch.ones(channels, dim))

    def kernel(self, L: int) -> torch.Tensor:
        """Convolution kernels ``[channels, L, dim]`` (real)."""
        dev = self.log_dt.device
        n = L + (L % 2)                                              # even FFT length
        w = torch.exp(-2j * math.pi * torch.arange(n // 2 + 1, device=dev) / n)
        z = 2 * (1 - w) / (1 + w + 1e-7)
        d = torch.complex(-torch.exp(self.log_neg_real), self.imag)                      # [Q, N]
        t = torch.exp(self.log_dt)                                                       # [Q, Hh]
        coeff = compute_kernel_coefficient(torch.view_as_real(z.to(torch.complex64)).contiguous(), d, t,
                                           torch.view_as_complex(self.B.contiguous()), torch.view_as_complex(self.Cm.contiguous()))
        khat = coeff[:, 0] * (2 / (1 + w + 1e-7))[None, None, :, None]                   # [Q, C, Lf, Hh]
        k = torch.fft.irfft(khat, n=n, dim=2)[:, :, :L]                                  # [Q, C, L, Hh]
        return k.permute(1, 2, 0, 3).reshape(self.C, L, self.Q * self.Hh)

    def forward(self, u: torch.Tensor) -> torch.Tensor:
        """u ``[B, T, dim]`` -> ``[B, T, dim]`` (channels summed; channel 1, if present, runs right to left)."""
        B, T, H = u.shape
        k = self.kernel(T)
        uf = u.float()
        n = 2 * T
        y = 0
        for c in range(self.C):
            x = uf if c == 0 else uf.flip(1)
            conv = torch.fft.irfft(torch.fft.rfft(x, n=n, dim=1) * torch.fft.rfft(k[c], n=n, dim=0)[None], n=n, dim=1)[:, :T]
            conv = conv + x * self.D[c]
            y = y + (conv if c == 0 else conv.flip(1))
        return y.to(u.dtype)


class MHS4Layer(nn.Module):
    """Pre-norm residual block: LayerNorm -> state-space mixing -> GELU -> output projection (+ dropout)."""

    def __init__(self, dim: int, heads: int = 4, state: int = 32, bidirectional: bool = True, dropout: float = 0.1):
        super().__init__()
        self.norm = nn.LayerNorm(dim)
        self.ssm = TiedStateSpaceModel(dim, heads, state, channels=2 if bidirectional else 1)
        self.out = nn.Linear(dim, dim)
        self.ffn_norm = nn.LayerNorm(dim)
        self.ffn = nn.Sequential(nn.Linear(dim, 4 * dim), nn.GELU(), nn.Linear(4 * dim, dim))
        self.dropout = dropout

    def forward(self, x, valid):
        h = self.ssm(self.norm(x) * valid[..., None])
        x = x + F.dropout(self.out(F.gelu(h)), self.dropout, self.training)
        return x + F.dropout(self.ffn(self.ffn_norm(x)), self.dropout, self.training)


class S4Encoder(nn.Module):
    """Speech encoder: (stacked) feature frames -> linear projection -> stack of ``MHS4Layer`` -> LayerNorm; returns the
    packed states and their ``PackedSeqs`` like the other speech encoders."""

    def __init__(self, input_size: int, dim: int = 512, layers: int = 6, heads: int = 4, state: int = 32, dropout: float = 0.1):
        super().__init__()
        self.dim = dim
        self.proj = nn.Linear(input_size, dim)
        self.layers = nn.ModuleList([MHS4Layer(dim, heads, state, True, dropout) for _ in range(layers)])
        self.final_norm = nn.LayerNorm(dim)

    def forward(self, source):
        feats, lengths = split_audio_batch(source)
        x = self.proj(feats.float())
        valid = (torch.arange(x.shape[1], device=x.device)[None, :] < lengths[:, None]).to(x.dtype)
        for layer in self.layers:
            x = layer(x, valid)
        packed, seqs = pack_padded(self.final_norm(x), lengths.clamp(max=x.shape[1]))
        return packed, seqs


def build_stacked_mh_s4(input_size: int, dim: int, layers: int, heads: int = 4, state: int = 32, dropout: float = 0.1) -> S4Encoder:
    return S4Encoder(input_size, dim, layers, heads, state, dropout)
