"""Per-rank trainer: builds the model, runs epochs, validates, checkpoints, logs.

One process per GPU.  The step itself is ``TrainEngine.train_step`` (fused kernels, flat optimiser, optional
CUDA graph); this class adds what surrounds it: process-group set-up, data iterators sharded by rank,
gradient accumulation over ``update_frequency`` micro-batches, token-normalised gradients
(``-normalize_gradient``), periodic validation and checkpointing (``-save_every``, ``-keep_save_files``,
``-save_metrics``), rank-0 logging of perplexity / learning rate / tokens per second, heartbeat for the
failure watchdog, and resume from a checkpoint (model, optimiser moments, update count, iterator position).

Reference behaviour: onmt/train_utils/mp_trainer.py:152-414 (set-up), :512-560 (save), :562-671 (eval),
:673-1160 (train_epoch), :1519-1690 (run).
"""
from __future__ import annotations

import math
import os
import time
from typing import Optional

import torch
import torch.distributed as dist

from .. import ops
from ..data.iterator import DataIterator, MultiDataIterator
from ..models.factory import build_model
from ..utils.logging import Logger
from .checkpoint import checkpoint_name, load_model_state, prune_checkpoints, save_checkpoint
from .engine import TrainEngine


def _is_list(x):
    return isinstance(x, (list, tuple))


class Trainer:
    def __init__(self, device, dicts, opt, constants=None, setup_optimizer: bool = True, init_distributed: bool = True):
        self.opt = opt
        self.dicts = dicts
        self.constants = constants
        self.world_size = len(opt.gpus) if getattr(opt, "gpus", None) else int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", device if isinstance(device, int) else 0)) if self.world_size > 1 else 0
        self.cuda = torch.cuda.is_available() and (getattr(opt, "gpus", None) not in (None, [], [-1]))
        if self.cuda:
            local = int(os.environ.get("LOCAL_RANK", device if isinstance(device, int) else 0))
            torch.cuda.set_device(local)
            self.device = torch.device("cuda", local)
        else:
            self.device = torch.device("cpu")
        if self.world_size > 1 and init_distributed and not dist.is_initialized():
            os.environ.setdefault("MASTER_ADDR", getattr(opt, "master_addr", "127.0.0.1") or "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", str(getattr(opt, "master_port", "8888")))
            dist.init_process_group("nccl" if self.cuda else "gloo", rank=self.rank, world_size=self.world_size)
        self.log = Logger(self.rank == 0)
        torch.manual_seed(getattr(opt, "seed", 9999))
        ops.manual_seed(getattr(opt, "seed", 9999) + 7919 * self.rank)

        self.log("[INFO] Building model ...")
        self.model = build_model(opt, dicts, constants=constants)
        n_params = sum(p.numel() for p in self.model.parameters() if p.requires_grad)
        self.log("[INFO] Total number of trainable parameters: %d" % n_params)
        checkpoint = None
        if getattr(opt, "load_from", ""):
            from .checkpoint import load_checkpoint
            checkpoint = load_checkpoint(opt.load_from)
            load_model_state(self.model, checkpoint["model"], verbose=self.rank == 0)
        self._resume_checkpoint = checkpoint

        grad_scale = 1.0
        ddp = None
        if self.world_size > 1:
            ddp = "nccl" if (getattr(opt, "nccl_ddp", False) or not self.cuda) else "fused"
        if getattr(opt, "fsdp", False) and self.cuda:
            ddp = "fsdp"
        self.engine = TrainEngine(self.model, opt, self.device, reducer=None,
                                  cuda_graph=self._graph_wanted(opt),
                                  grad_scale=grad_scale, ddp=ddp)
        self.optim = self.engine.optim
        # A data set cut by a token budget produces many shape classes, most of them rare.  Capturing a class costs about
        # four kernel-by-kernel steps and a replay saves about 4 % of one, so a class is captured at its eighth batch and a
        # full cache is never evicted: the frequent classes of a long run end up replayed, everything else runs eagerly
        # (measured with bench_cli.py: capturing at the third batch with eviction halved the throughput of a 60 k-sentence
        # corpus from its third epoch on).
        self.engine.capture_after = 8
        self.engine.evict_graphs = False
        if checkpoint is not None and not getattr(opt, "reset_optim", False) and checkpoint.get("optim") is not None:
            try:
                self.optim.load_state_dict(checkpoint["optim"])
            except Exception as exc:  # noqa: BLE001
                if getattr(self.optim, "distributed", None) is not None:
                    raise       # a sharded run with some ranks restored and others not would diverge silently
                self.log("[WARN] optimiser state not restored: %r" % (exc,))
            from .checkpoint import restore_rng_state
            restore_rng_state(checkpoint.get("rng"))      # same dropout masks and shuffles as the uninterrupted run
            if getattr(self.engine, "scaler", None) is not None and isinstance(checkpoint.get("scaler"), dict):
                self.engine.scaler.load_state_dict(checkpoint["scaler"])
        self.start_time = time.time()
        # -ema: exponential moving average of the parameters (one vector op on the flat master buffer per update),
        # used for validation and for the saved checkpoints
        self.ema = None
        if getattr(opt, "ema", False) and getattr(self.optim, "distributed", None) is None:
            from .finetune import FlatEMA
            self.ema = FlatEMA(self.engine.store, decay=getattr(opt, "ema_decay", 0.999) or 0.999)
        lora_rank = int(getattr(opt, "lora_rank", 0) or 0)
        if lora_rank > 0:
            raise RuntimeError("apply LoRA before building the trainer: use nmtgminor_b200.train.finetune.apply_lora on the model "
                               "returned by build_model (see finetune_whisper.py)")
        if self.cuda and ops.extension_available():
            # bound of every device-side wait for a peer: minutes in production (a slow data loader or a long validation
            # pass on one rank must not abort the run), short in tests
            ops.ext().set_peer_timeout_ms(float(getattr(opt, "peer_timeout", 0) or os.environ.get("NMTG_PEER_TIMEOUT_MS", 120000)))
        self.watchdog = None
        if getattr(opt, "watchdog_timeout", 0) and self.world_size > 1:
            from ..utils.watchdog import Heartbeat
            self.watchdog = Heartbeat(self.rank, self.world_size, timeout=opt.watchdog_timeout)

    def _graph_wanted(self, opt) -> bool:
        """The step is replayed from CUDA graphs (one per shape class of batches) by default on a GPU.  Off with
        ``-no_cuda_graph``, with gradient accumulation, and for models that skip layers at random (a captured graph
        would freeze one pattern)."""
        from ..parallel.sharded import skips_layers
        if not self.cuda or getattr(opt, "no_cuda_graph", False):
            return False
        if int(getattr(opt, "update_frequency", 1) or 1) > 1 or int(getattr(opt, "batch_size_update", -1) or -1) > 0:
            return False
        return not skips_layers(opt)

    # ------------------------------------------------------------------------------------------
    def is_main(self):
        return self.rank == 0

    def _all_reduce_scalars(self, values):
        if self.world_size <= 1:
            return values
        t = torch.tensor(values, dtype=torch.float64, device=self.device)
        dist.all_reduce(t)
        return t.tolist()

    def _iterator(self, data, epoch, seed_offset=0, shuffle=True):
        kw = dict(seed=getattr(self.opt, "seed", 9999) + seed_offset, num_workers=getattr(self.opt, "num_workers", 0),
                  epoch=epoch, buffer_size=getattr(self.opt, "buffer_size", 0), num_shards=self.world_size,
                  shard_id=self.rank, split_even=True, pin_memory=self.cuda or bool(getattr(self.opt, "pin_memory", False)),
                  shuffle=shuffle)
        if _is_list(data):
            return MultiDataIterator(list(data), **kw)
        return DataIterator(data, **kw)

    # ------------------------------------------------------------------------------------------
    @torch.no_grad()
    def eval(self, data):
        """Validation loss per target token and token accuracy over all ranks."""
        if data is None:
            return float("nan"), 0.0
        if self.ema is not None:
            self.ema.swap_in()
        self.model.eval()
        tot_loss = tot_words = tot_correct = 0.0
        for ds in (data if _is_list(data) else [data]):
            it = DataIterator(ds, num_shards=self.world_size, shard_id=self.rank, split_even=False, shuffle=False,
                              pin_memory=self.cuda).next_epoch_itr()
            for batch in it:
                loss, correct = self.engine.eval_step(batch)
                tot_loss += float(loss)
                tot_correct += float(correct)
                tot_words += batch.tgt_size
        tot_loss, tot_words, tot_correct = self._all_reduce_scalars([tot_loss, tot_words, tot_correct])
        if self.ema is not None:
            self.ema.swap_out()
        self.model.train()
        return tot_loss / max(tot_words, 1.0), tot_correct / max(tot_words, 1.0)

    def save(self, epoch: float, valid_ppl: float, itr=None, accuracy: float = 0.0):
        dist_opt = getattr(self.optim, "distributed", None)
        if dist_opt is not None:
            dist_opt.gather_master()         # collective: every rank refreshes its full fp32 copy from the piece owners
            self.optim.prepare_state_dict()  # collective: Adam moments of all pieces -> flat layout on rank 0
        name = None
        try:
            if self.is_main():
                if self.ema is not None:
                    self.ema.swap_in()
                try:
                    name = self._save_checkpoint_file(epoch, valid_ppl, itr, accuracy)
                finally:
                    if self.ema is not None:
                        self.ema.swap_out()
        finally:
            if dist_opt is not None and hasattr(dist_opt, "release_master"):
                dist_opt.release_master()
            # the other ranks wait here while rank 0 writes the file: without this they would run ahead into the next
            # step's gradient exchange and sit in a device-side wait (which is bounded, and would abort the run)
            if self.world_size > 1 and dist.is_initialized():
                dist.barrier()
        return name

    def _save_checkpoint_file(self, epoch: float, valid_ppl: float, itr=None, accuracy: float = 0.0):
        opt = self.opt
        metric = getattr(opt, "save_metrics", "ppl")
        value = valid_ppl if metric in ("ppl", "perplexity") else (1.0 - accuracy if metric == "accuracy" else valid_ppl)
        name = checkpoint_name(opt.save_model, "ppl", value, epoch)
        os.makedirs(os.path.dirname(os.path.abspath(name)), exist_ok=True)
        scaler = getattr(self.engine, "scaler", None)
        save_checkpoint(name, self.model, self.dicts, opt, epoch, self.optim, itr.state_dict() if itr is not None else None,
                        scaler=scaler.state_dict() if scaler is not None else None)
        prune_checkpoints(opt.save_model, getattr(opt, "keep_save_files", 5), "ppl")
        self.log("[INFO] Saved checkpoint %s" % name)
        return name

    # ------------------------------------------------------------------------------------------
    def _guarded_step(self, batch, update: bool):
        """One engine step; a batch that runs the device out of memory is dropped (its partial gradients with it) and
        training goes on, as in the reference (onmt/train_utils/mp_trainer.py: "out of memory" handling of the step;
        whisper/trainers/trainer_shuffle_ctc.py:169-177).  With several ranks the other ranks are already waiting in
        the gradient exchange of this step, so there the error is raised."""
        try:
            return self.engine.train_step(batch, update=update)[0]
        except torch.cuda.OutOfMemoryError:
            if self.world_size > 1:
                raise
            self.oom_skipped = getattr(self, "oom_skipped", 0) + 1
            self.log("[WARNING] out of device memory on a batch of %d source / %d target tokens; batch skipped (%d so far)"
                     % (batch.src_size, batch.tgt_size, self.oom_skipped))
            self.optim.zero_grad()
            torch.cuda.empty_cache()
            return torch.zeros((), device=self.engine.device if self.cuda else "cpu")

    def train_epoch(self, train_data, valid_data, epoch: int, resume_itr_state=None):
        opt = self.opt
        iterator = self._iterator(train_data, epoch)
        if resume_itr_state is not None:
            iterator.load_state_dict(resume_itr_state)
        epoch_itr = iterator.next_epoch_itr()
        n_batches = len(iterator)
        update_frequency = max(1, getattr(opt, "update_frequency", 1))
        log_interval = max(1, getattr(opt, "log_interval", 100))
        report = {"loss": 0.0, "tgt": 0.0, "src": 0.0, "sents": 0.0}
        epoch_loss = epoch_words = 0.0
        pending = []          # device loss tensors of the current logging window (read once per window)
        acc_words = 0
        t_window = time.time()
        counter = 0
        self.model.train()
        for i, batch in enumerate(epoch_itr):
            counter += 1
            acc_words += batch.tgt_size
            update = counter >= update_frequency or i == n_batches - 1
            bsu = int(getattr(opt, "batch_size_update", -1) or -1)
            if bsu > 0:       # -batch_size_update: step once this many target tokens have been accumulated (on this rank)
                update = acc_words >= bsu or i == n_batches - 1
            if update and getattr(opt, "normalize_gradient", False):
                total_words = self._all_reduce_scalars([float(acc_words)])[0]
                self.engine.grad_scale = 1.0 / max(total_words, 1.0)
            loss = self._guarded_step(batch, update)
            pending.append(loss if self.engine.use_graph is False else loss.clone())
            report["tgt"] += batch.tgt_size
            report["src"] += batch.src_size
            report["sents"] += batch.size
            if update:
                counter, acc_words = 0, 0
                if self.world_size > 1 and self.engine.peek_status():
                    torch.cuda.synchronize()
                    raise RuntimeError("a device kernel gave up waiting for a peer (status %d); aborting the run"
                                       % (ops.check_status() or self.engine.peek_status()))
                if self.ema is not None:
                    self.ema.update(self.optim._step)
                if self.watchdog is not None:
                    self.watchdog.beat(self.optim._step)
                n_up = self.optim._step
                save_every = getattr(opt, "save_every", 0)
                if save_every and save_every > 0 and n_up % save_every == 0:
                    vloss, vacc = self.eval(valid_data)
                    vppl = math.exp(min(vloss, 100)) if vloss == vloss else float("nan")
                    self.log("Validation perplexity: %g  accuracy: %.4f" % (vppl, vacc))
                    self.save(epoch - 1 + (i + 1) / max(n_batches, 1), vppl, iterator, vacc)
                max_step = getattr(opt, "max_step", 0)
                if max_step and n_up >= max_step:
                    self.log("[INFO] Reached the maximum number of updates (%d)" % max_step)
                    break
            if (i + 1) % log_interval == 0 or i == n_batches - 1:
                window_loss = float(torch.stack([p.reshape(()) for p in pending]).sum()) if pending else 0.0
                pending = []
                vals = self._all_reduce_scalars([window_loss, report["tgt"], report["src"]])
                dt = max(time.time() - t_window, 1e-9)
                epoch_loss += vals[0]
                epoch_words += vals[1]
                status = ops.check_status() if self.cuda and ops.extension_available() else 0
                if status:
                    raise RuntimeError("a device kernel gave up waiting (status %d); aborting the run" % status)
                scaler = getattr(self.engine, "scaler", None)
                extra = "" if scaler is None else " ; loss scale: %g (%d skipped)" % (scaler.get_scale(), scaler.skipped_steps())
                self.log("Epoch %2d, %5d/%5d; ppl: %8.2f ; lr: %.7f ; num updates: %7d ; %5.0f src tok/s; %5.0f tgt tok/s; %s elapsed%s"
                         % (epoch, i + 1, n_batches, math.exp(min(vals[0] / max(vals[1], 1.0), 100)), self.optim.current_lr(),
                            self.optim._step, vals[2] / dt, vals[1] / dt, _fmt_time(time.time() - self.start_time), extra))
                report = {"loss": 0.0, "tgt": 0.0, "src": 0.0, "sents": 0.0}
                t_window = time.time()
        return epoch_loss / max(epoch_words, 1.0), iterator

    def run(self, checkpoint=None, train_data=None, valid_data=None):
        opt = self.opt
        checkpoint = checkpoint if checkpoint is not None else self._resume_checkpoint
        start_epoch, resume_itr = 1, None
        if checkpoint is not None and not getattr(opt, "reset_optim", False):
            start_epoch = int(math.floor(checkpoint.get("epoch", 0))) + 1
            resume_itr = checkpoint.get("itr")
            if resume_itr is not None and resume_itr.get("iterations_in_epoch", 0) > 0:
                start_epoch = int(resume_itr.get("epoch", start_epoch))
        if getattr(opt, "run_validation_before_training", False) or getattr(opt, "max_step", 1) is not None and getattr(opt, "max_step", 1) < 0:
            vloss, vacc = self.eval(valid_data)
            self.log("Validation perplexity: %g  accuracy: %.4f" % (math.exp(min(vloss, 100)), vacc))
        self.start_time = time.time()
        last = None
        for epoch in range(start_epoch, start_epoch + getattr(opt, "epochs", 1)):
            train_loss, iterator = self.train_epoch(train_data, valid_data, epoch, resume_itr)
            resume_itr = None
            self.log("Train perplexity: %g" % math.exp(min(train_loss, 100)))
            vloss, vacc = self.eval(valid_data)
            vppl = math.exp(min(vloss, 100)) if vloss == vloss else float("nan")
            self.log("Validation perplexity: %g  accuracy: %.4f" % (vppl, vacc))
            last = self.save(float(epoch), vppl if vppl == vppl else math.exp(min(train_loss, 100)), None, vacc)
            self.optim.update_epoch(epoch)
            max_step = getattr(opt, "max_step", 0)
            if max_step and self.optim._step >= max_step:
                break
        if self.watchdog is not None:
            self.watchdog.stop()
        return last


def _fmt_time(sec: float) -> str:
    sec = int(sec)
    return "%02d:%02d:%02d" % (sec // 3600, (sec // 60) % 60, sec % 60)
