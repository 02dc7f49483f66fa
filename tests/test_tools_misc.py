import torch

from nmtgminor_b200.tools.kmeans import KMeans, learn_kmeans, quantize
from nmtgminor_b200.tools.text import Autoencoder, extract_vocab, normalize_text, train_autoencoder


def test_kmeans_recovers_separated_clusters():
    torch.manual_seed(0)
    centres = torch.tensor([[0.0, 0.0], [10.0, 0.0], [0.0, 10.0]])
    x = torch.cat([c + 0.1 * torch.randn(200, 2) for c in centres])
    best = min((learn_kmeans([x[torch.randperm(600)]], 3, epochs=5, seed=s) for s in range(4)), key=lambda k: k.inertia(x))
    assert best.inertia(x) < 0.1
    units = quantize(best, x)
    assert len(set(units[:200])) == 1 and len(set(units)) == 3
    assert quantize(best, x[:200], deduplicate=True) == [units[0]]
    again = KMeans.load(best.state_dict())
    assert torch.equal(again.assign(x), best.assign(x))


def test_text_tools_and_autoencoder():
    assert extract_vocab(["b a a", "a c b"], min_count=2) == ["a", "b"]
    assert normalize_text("  “Hello” ,  world !  ", lower=True) == '"hello" , world !'
    assert normalize_text("a, b.", strip_punct=True) == "a b"
    torch.manual_seed(0)
    basis = torch.randn(4, 16)
    states = [torch.tanh(torch.randn(50, 4) @ basis) for _ in range(4)]
    first = Autoencoder(16, 8).loss(states[0]).item()
    ae = train_autoencoder(states, inner_size=8, epochs=40, lr=5e-3)
    assert ae.loss(states[0]).item() < first


def test_speech_benchmark_dry_run(capsys):
    """``bench_speech.py --tiny`` runs both speech configurations through the training engine on the CPU."""
    import importlib.util
    import json
    import os
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("bench_speech", os.path.join(root, "bench_speech.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    for cfg in ("whisper_large_v2", "wav2vec2_mbart50"):
        mod.main(["--config", cfg, "--tiny", "--steps", "1", "--warmup", "1"])
        line = [l for l in capsys.readouterr().out.splitlines() if l.startswith("{")][-1]
        out = json.loads(line)
        assert out["value"] > 0 and out["audio_seconds_per_second"] > 0 and out["loss_per_token_after_warmup"] > 0
