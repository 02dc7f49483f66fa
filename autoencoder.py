#!/usr/bin/env python
"""python autoencoder.py -data <prefix> -load_from model.pt -save_model ae [-representation EncoderHiddenState|DecoderHiddenState]
       [-auto_encoder_hidden_size 100] [-auto_encoder_drop_out 0] [-epochs 5] [-learning_rate 1e-3] + the training options
Train a bottleneck auto-encoder on the hidden states of a trained translation model (one state vector per source token,
or per target token), e.g. for domain / anomaly scoring with eval_autoencoder.py.  The translation model is frozen.
(reference: autoencoder.py, ae/*)"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def hidden_states(model, batch, representation: str):
    """[tokens, H] states of ``batch`` from the frozen model: encoder outputs or decoder outputs (before the generator)."""
    with torch.no_grad():
        context, src = model.encode(batch)
        if representation.startswith("Encoder"):
            n = int(src.cu[-1])
            return context[:n].float()
        out = model(batch, compute_loss=False)
        n = int(out["tgt"].cu[-1])
        return out["hidden_packed"][:n].float()


def main(argv=None):
    from nmtgminor_b200.models.factory import build_model
    from nmtgminor_b200.options import backward_compatible, make_parser
    from nmtgminor_b200.tools.text import Autoencoder
    from nmtgminor_b200.train.checkpoint import load_model_state
    from train_distributed import load_data
    import argparse
    parser = make_parser(argparse.ArgumentParser(description="autoencoder.py"))
    parser.add_argument("-representation", default="EncoderHiddenState")
    parser.add_argument("-auto_encoder_hidden_size", type=int, default=100)
    parser.add_argument("-auto_encoder_drop_out", type=float, default=0.0)
    parser.add_argument("-auto_encoder_type", default="Baseline")
    opt = parser.parse_args(argv)
    if not opt.load_from:
        sys.exit("autoencoder.py needs -load_from <trained model>")
    torch.manual_seed(opt.seed)
    dicts, train, valid = load_data(opt)
    ckpt = torch.load(opt.load_from, map_location="cpu", weights_only=False)
    model = build_model(backward_compatible(ckpt["opt"]), ckpt["dicts"], remove_pretrain=True)
    load_model_state(model, ckpt["model"])
    dev = torch.device("cuda:%d" % opt.gpus[0]) if (torch.cuda.is_available() and opt.gpus) else torch.device("cpu")
    model = model.to(dev).eval()
    for p in model.parameters():
        p.requires_grad_(False)
    on = (lambda b: b.cuda(dev)) if dev.type == "cuda" else (lambda b: b)
    probe = hidden_states(model, on(train.get_batch(0)), opt.representation)
    ae = Autoencoder(probe.shape[-1], opt.auto_encoder_hidden_size, dropout=opt.auto_encoder_drop_out).to(dev)
    optim = torch.optim.Adam(ae.parameters(), lr=opt.learning_rate if opt.learning_rate < 0.1 else 1e-3)
    for epoch in range(1, opt.epochs + 1):
        total, count = 0.0, 0
        ae.train()
        for i in torch.randperm(len(train)).tolist():
            x = hidden_states(model, on(train.get_batch(i)), opt.representation)
            optim.zero_grad()
            loss = ae.loss(x)
            loss.backward()
            optim.step()
            total += float(loss) * x.shape[0]
            count += x.shape[0]
        msg = "Epoch %d: train reconstruction error %.6f" % (epoch, total / max(count, 1))
        if valid is not None and len(valid):
            ae.eval()
            vt, vc = 0.0, 0
            with torch.no_grad():
                for i in range(len(valid)):
                    x = hidden_states(model, on(valid.get_batch(i)), opt.representation)
                    vt += float(ae.loss(x)) * x.shape[0]
                    vc += x.shape[0]
            msg += "; valid %.6f" % (vt / max(vc, 1))
        print(msg, flush=True)
        torch.save({"autoencoder": ae.state_dict(), "input_size": probe.shape[-1], "hidden_size": opt.auto_encoder_hidden_size,
                    "representation": opt.representation, "epoch": epoch}, "%s_e%d.pt" % (opt.save_model, epoch))


if __name__ == "__main__":
    main()
