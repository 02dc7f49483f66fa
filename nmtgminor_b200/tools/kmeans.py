"""K-means over frame-level speech features (learning a codebook, quantising features to unit ids) and dumping
encoder features / wav2vec2 quantiser codebooks from a trained model.

The mini-batch k-means runs on whatever device the features live on: assignment is one matrix product per chunk
(GEMM-shaped, so it takes the tensor cores on a GPU), the update is a scatter-add.

Reference: learn_kmeans.py, quantize_kmeans.py, quantize_pretrained_hubert_kmeans.py, extract_wav2vec2_codebook.py,
extract_wav2vec2_tdnn.py, neural_feature_reader.py, verify_wav2vec2_feat.py.
"""
from __future__ import annotations

from typing import Iterable, List, Optional

import torch


class KMeans:
    def __init__(self, n_clusters: int, dim: int, device="cpu", seed: int = 0):
        self.n_clusters, self.dim = n_clusters, dim
        self.centroids = torch.zeros(n_clusters, dim, device=device)
        self.counts = torch.zeros(n_clusters, device=device)
        self.initialised = False
        self.gen = torch.Generator(device="cpu").manual_seed(seed)

    def _init(self, x):
        idx = torch.randperm(x.shape[0], generator=self.gen)[:self.n_clusters]
        if idx.numel() < self.n_clusters:
            idx = torch.cat([idx, torch.randint(0, x.shape[0], (self.n_clusters - idx.numel(),), generator=self.gen)])
        self.centroids.copy_(x[idx.to(x.device)].to(self.centroids.dtype))
        self.initialised = True

    @torch.no_grad()
    def assign(self, x, chunk: int = 65536):
        out = []
        c = self.centroids
        c_sq = (c * c).sum(1)
        for i in range(0, x.shape[0], chunk):
            xi = x[i:i + chunk].to(c.dtype)
            d = c_sq[None, :] - 2.0 * xi @ c.t()          # + |x|^2 is constant per row
            out.append(d.argmin(1))
        return torch.cat(out) if out else torch.zeros(0, dtype=torch.long, device=x.device)

    @torch.no_grad()
    def partial_fit(self, x):
        """One mini-batch step: per-centroid learning rate 1 / count (Sculley's update)."""
        x = x.to(self.centroids.device)
        if not self.initialised:
            self._init(x)
        a = self.assign(x)
        sums = torch.zeros_like(self.centroids).index_add_(0, a, x.to(self.centroids.dtype))
        n = torch.zeros_like(self.counts).index_add_(0, a, torch.ones_like(a, dtype=self.counts.dtype))
        self.counts += n
        seen = n > 0
        lr = (n / self.counts.clamp_min(1))[:, None]
        mean = sums / n.clamp_min(1)[:, None]
        self.centroids = torch.where(seen[:, None], (1 - lr) * self.centroids + lr * mean, self.centroids)
        return self

    def fit(self, batches: Iterable[torch.Tensor], epochs: int = 1):
        batches = list(batches)
        for _ in range(epochs):
            for b in batches:
                self.partial_fit(b)
        return self

    @torch.no_grad()
    def inertia(self, x):
        a = self.assign(x)
        return float(((x.to(self.centroids.dtype) - self.centroids[a]) ** 2).sum(1).mean())

    def state_dict(self):
        return {"centroids": self.centroids.cpu(), "counts": self.counts.cpu()}

    @classmethod
    def load(cls, sd, device="cpu"):
        km = cls(sd["centroids"].shape[0], sd["centroids"].shape[1], device)
        km.centroids, km.counts, km.initialised = sd["centroids"].to(device), sd["counts"].to(device), True
        return km


def learn_kmeans(feature_batches: Iterable[torch.Tensor], n_clusters: int, epochs: int = 2, device="cpu", seed: int = 0) -> KMeans:
    batches = [b.reshape(-1, b.shape[-1]) for b in feature_batches]
    return KMeans(n_clusters, batches[0].shape[-1], device, seed).fit(batches, epochs)


def quantize(km: KMeans, features: torch.Tensor, deduplicate: bool = False) -> List[int]:
    units = km.assign(features.reshape(-1, features.shape[-1]).to(km.centroids.device)).tolist()
    if deduplicate:
        units = [u for i, u in enumerate(units) if i == 0 or u != units[i - 1]]
    return units


@torch.no_grad()
def extract_features(model, waves: List[torch.Tensor], layer: Optional[int] = None, device=None) -> List[torch.Tensor]:
    """Frame-level encoder states for every waveform (``layer``: stop after that many encoder layers)."""
    from ..data.synthetic import synthetic_audio_batch  # noqa: F401  (documents the batch layout used below)
    from ..data.dataset import collate
    enc = model.encoder
    outs = []
    for w in waves:
        batch = collate([w.reshape(-1, 1).float()], None, round_to=1)
        if device is not None:
            batch = batch.cuda(device) if torch.device(device).type == "cuda" else batch
        kept = None
        if layer is not None and hasattr(enc, "layers"):
            kept = enc.layers
            enc.layers = torch.nn.ModuleList(list(kept)[:layer])
        try:
            context, src = model.encode(batch)
        finally:
            if kept is not None:
                enc.layers = kept
        n = int(src.cu[1])
        outs.append(context[:n].float().cpu())
    return outs


def extract_codebook(model) -> Optional[torch.Tensor]:
    """Entries of the wav2vec2 product quantiser (``[groups, entries, dim]``) when the encoder carries one."""
    for m in model.modules():
        if hasattr(m, "codebook") and torch.is_tensor(getattr(m, "codebook")):
            return m.codebook.detach().cpu()
        if m.__class__.__name__.lower().startswith("gumbelvectorquantizer") and hasattr(m, "vars"):
            return m.vars.detach().cpu()
    return None
