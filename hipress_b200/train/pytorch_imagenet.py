"""PyTorch training script (synthetic data, or an ImageNet-style directory with
``--train-dir``), flags as in the reference's
``horovod-torch/imageNet/pytorch_imagenet.py`` (``--batch-size --epochs
--num-iterations --model --algorithm``, README.md:184-186 of mark14wu/hipress).

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m hipress_b200.train.pytorch_imagenet --model vgg19 --algorithm tbq --batch-size 32
"""
from __future__ import annotations

import argparse
import itertools
import sys
import time

import torch

import hipress_b200 as hp
from hipress_b200.config import add_hipress_args, config_from_args
from hipress_b200.train.harness import build_job
from hipress_b200.utils import MetricsWriter, engine_metrics, load_checkpoint, save_checkpoint, setup_logging


def main(argv=None):
    ap = argparse.ArgumentParser(description="hipress_b200 synthetic-data training")
    ap.add_argument("--model", default="vgg19")
    ap.add_argument("--batch-size", type=int, default=None, help="per-GPU batch")
    ap.add_argument("--epochs", type=int, default=1)
    ap.add_argument("--num-iterations", type=int, default=20, help="iterations per epoch")
    ap.add_argument("--train-dir", default=None,
                    help="image models: ImageNet-style directory instead of synthetic data")
    ap.add_argument("--val-dir", default=None, help="image models: directory scored after every epoch")
    ap.add_argument("--workers", type=int, default=4, help="--train-dir: loader processes per rank")
    ap.add_argument("--warmup-iters", type=int, default=0, help="linear learning-rate warm-up")
    ap.add_argument("--lr-decay-epochs", default="", help="e.g. 30,60,80: multiply the rate by 0.1 there")
    ap.add_argument("--image-size", type=int, default=224)
    ap.add_argument("--num-classes", type=int, default=None)
    ap.add_argument("--seq-len", type=int, default=128)
    ap.add_argument("--lr", type=float, default=0.01)
    ap.add_argument("--fp32", action="store_true", help="no bf16 autocast")
    ap.add_argument("--checkpoint-dir", default=None)
    ap.add_argument("--resume", action="store_true")
    ap.add_argument("--metrics", default=None, help="JSONL file for per-step metrics")
    ap.add_argument("--heartbeat-timeout", type=float, default=0.0,
                    help="seconds without a peer's heartbeat before the job stops (0: no monitor)")
    ap.add_argument("--elastic", action="store_true",
                    help="with --heartbeat-timeout: when peers leave or go silent, the survivors "
                         "re-form a smaller job and continue")
    ap.add_argument("--elastic-port", type=int, default=0,
                    help="first rendezvous port of re-formed jobs (default MASTER_PORT + 1)")
    ap.add_argument("--inject-leave", default=None, metavar="RANK:STEP",
                    help="fault injection on the host: this rank leaves the job before that step")
    add_hipress_args(ap)
    a = ap.parse_args(argv)
    hp.init()
    log = setup_logging()
    cfg = config_from_args(a)
    job = build_job(a.model, cfg, batch=a.batch_size, seq_len=a.seq_len, lr=a.lr,
                    dtype=torch.float32 if a.fp32 else torch.bfloat16,
                    model_kwargs={"num_classes": a.num_classes} if a.num_classes else None)
    if a.train_dir and job.kind != "image":
        raise SystemExit("--train-dir is for the image models")
    start_epoch = 0
    if a.resume and a.checkpoint_dir:
        info = load_checkpoint(a.checkpoint_dir, job.model, job.optimizer, map_location=job.device)
        start_epoch = info["epoch"]
        log.info("resumed from %s at epoch %d", a.checkpoint_dir, start_epoch)
    mw = MetricsWriter(a.metrics)
    log.info("model %s, %d GPUs, batch %d/GPU, %s", a.model, hp.size(), job.batch,
             engine_metrics(job.optimizer.engine))
    cuda = job.device.type == "cuda"
    hosts = [job.host_batch(100 * hp.rank() + i) for i in range(4)]
    from hipress_b200.utils.health import HealthMonitor, PeerFailure, default_store

    def new_monitor():
        if a.heartbeat_timeout > 0 and hp.size() > 1:
            return HealthMonitor(default_store(), hp.rank(), hp.size(), timeout_s=a.heartbeat_timeout,
                                 interval_s=min(0.2, a.heartbeat_timeout / 4))
        return None

    monitor = new_monitor()
    leave_rank, leave_step = (int(v) for v in a.inject_leave.split(":")) if a.inject_leave else (-1, -1)
    generation = 0
    step = 0
    base_lrs = [g["lr"] for g in job.optimizer.param_groups]
    decay_at = [int(e) for e in a.lr_decay_epochs.split(",") if e.strip()]

    def set_lr(epoch, step):
        scale = 0.1 ** sum(epoch >= e for e in decay_at)
        if a.warmup_iters and step < a.warmup_iters:
            scale *= (step + 1) / a.warmup_iters
        for g, base in zip(job.optimizer.param_groups, base_lrs):
            g["lr"] = base * scale

    for epoch in range(start_epoch, a.epochs):
        if cuda:
            torch.cuda.synchronize()
        t0 = time.time()
        if a.train_dir:   # real data: a.num_iterations > 0 caps the epoch
            loader = job.image_folder_loader(a.train_dir, epoch=epoch, workers=a.workers,
                                             image_size=a.image_size)
            batches = job.stream_from(itertools.islice(loader, a.num_iterations or None))
        else:
            batches = job.stream_batches(hosts, a.num_iterations)
        for it, (x, y) in enumerate(batches):
            set_lr(epoch, step)
            if hp.rank() == leave_rank and step == leave_step and generation == 0:
                log.warning("leaving the job before step %d (injected)", step)
                if cuda:
                    torch.cuda.synchronize()
                if monitor is not None:
                    monitor.leave()
                time.sleep(max(1.0, 2 * a.heartbeat_timeout))   # stay reachable while the others regroup
                return 0
            if monitor is not None:
                # between steps, nothing of this rank in flight: a peer that left or went
                # silent is noticed here instead of inside the next collective
                try:
                    if step == leave_step and generation == 0 and leave_rank >= 0:
                        time.sleep(min(1.0, a.heartbeat_timeout))   # let the injected exit be announced
                    monitor.check()
                except PeerFailure as e:
                    if not a.elastic:
                        raise SystemExit(f"rank {hp.rank()}: {e}; stopping (no --elastic)")
                    from hipress_b200.parallel.elastic import reform_process_group, survivors_rendezvous
                    import os
                    generation += 1
                    log.warning("%s: re-forming the job without them", e)
                    if cuda:
                        torch.cuda.synchronize()
                    store, old_rank, old_world = default_store(), hp.rank(), hp.size()
                    monitor.close()
                    new_rank, new_world = survivors_rendezvous(store, old_rank, old_world, e.ranks,
                                                               generation=generation)
                    port = (a.elastic_port or int(os.environ.get("MASTER_PORT", "29500")) + 1) + generation - 1
                    reform_process_group(new_rank, new_world, port=port)
                    job.rebuild_optimizer()
                    monitor = new_monitor()
                    base_lrs = [g["lr"] for g in job.optimizer.param_groups]
                    log.warning("continuing as rank %d of %d", new_rank, new_world)
            loss = job.step(x, y)
            step += 1
            if it % 10 == 9 or it == a.num_iterations - 1 or (a.train_dir and it == 0):
                lv = loss.item()
                dt = time.time() - t0
                ips = job.batch * hp.size() * (it + 1) / dt
                log.info("epoch %d iter %d loss %.4f  %.1f samples/s", epoch, it + 1, lv, ips)
                mw.step(step, epoch=epoch, loss=lv, samples_per_s=round(ips, 1), ranks=hp.size(),
                        **engine_metrics(job.optimizer.engine))
        if a.val_dir:
            score = job.evaluate(job.image_folder_loader(a.val_dir, workers=a.workers,
                                                         image_size=a.image_size, train=False))
            log.info("epoch %d validation: top-1 %.4f, loss %.4f over %d images", epoch,
                     score["top1"], score["loss"], score["images"])
            mw.step(step, epoch=epoch, val_top1=round(score["top1"], 5), val_loss=round(score["loss"], 5),
                    val_images=score["images"])
        if a.checkpoint_dir:
            save_checkpoint(a.checkpoint_dir, job.model, job.optimizer, epoch=epoch + 1, step=step)
    job.optimizer.engine.check() if cuda else None
    if monitor is not None:
        monitor.leave()
    mw.close()
    job.optimizer.close()
    hp.shutdown()
    return 0


if __name__ == "__main__":
    sys.exit(main())
