#!/usr/bin/env python
"""Headline benchmark: images (or samples) per second of a full training step
(forward, backward with compressed gradient synchronisation, optimizer update) on
N GPUs of one box, device-timed, max over ranks.

    python bench.py                         # 1 GPU, VGG19 + TBQ + CaSync-Ring, batch 32/GPU
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 20 --warmup 5
    python bench.py --model resnet50        # ResNet-50 + DGC + CaSync-PS, batch 128/GPU
    python bench.py --model bert_large      # BERT-large MLM + onebit + CaSync-Ring, batch 32/GPU
    python bench.py --sync-backend allreduce   # uncompressed NCCL baseline (BL0)
    python bench.py --sync-backend host        # unfused compressed baseline (BL1)
    python bench.py --impl reference        # the reference itself (not installable offline)

After the product arm the same process times two baselines with the same model,
batch, warm-up and steps: torch DistributedDataParallel over NCCL (the conventional
uncompressed path the reference measures itself against, README.md:153 of
mark14wu/hipress) and this repo's unfused compressed schedule.  Their numbers, a
replica checksum and a one-step conservation check travel in the same JSON line.

Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

REFERENCE_UNAVAILABLE = (
    "mark14wu/hipress cannot be installed offline: no setup.py/pyproject.toml, and its runtime "
    "(src/CaSync), MXNet fork, torch extension and TF ops are empty git submodules")


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="hipress_b200", choices=["hipress_b200", "reference"])
    ap.add_argument("--model", default="vgg19",
                    choices=["vgg19", "resnet50", "bert_large", "bert_base", "lstm", "transformer"])
    ap.add_argument("--batch", type=int, default=None, help="per-GPU batch (default: headline config)")
    ap.add_argument("--seq-len", type=int, default=128)
    ap.add_argument("--comp-alg", default=None)
    ap.add_argument("--topo", default=None)
    ap.add_argument("--comp-threshold", type=int, default=262144)
    ap.add_argument("--comprplan", default="auto:bucketed",
                    help="SeCoPa plan: a plan file, 'auto' / 'auto:bucketed' (planner run in process with "
                         "the measured B200 cost profile of this world size; the size threshold decides "
                         "when there is none), or 'threshold'")
    ap.add_argument("--sync-backend", default="auto", choices=["auto", "fused", "host", "allreduce"])
    ap.add_argument("--ctas", type=int, default=None)
    ap.add_argument("--bucket-mb", type=int, default=None)
    ap.add_argument("--partition-sms", type=int, default=None)
    ap.add_argument("--partition-ctas", type=int, default=None)
    ap.add_argument("--overlap-optimizer", type=int, default=None, choices=[0, 1],
                    help="update each bucket's parameters right behind its synchronisation")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-baselines", action="store_true",
                    help="skip the torch-DDP and unfused arms that follow the product arm")
    ap.add_argument("--no-check", action="store_true", help="skip the one-step conservation check")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.p = None
        try:
            self.p = subprocess.Popen(
                ["nvidia-smi", "-i", str(index), f"--query-gpu={self.Q}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            pass

    def stop(self) -> dict:
        if self.p is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.p.terminate()
        try:
            out, _ = self.p.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.p.kill()
            out, _ = self.p.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for nm, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "samples": len(sm),
                "reasons": sorted(reasons)}


def physical_index(local: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local])
        except (ValueError, IndexError):
            return local
    return local


def timed_steps(job, pool, steps, warmup, sync_all, N, dev):
    """`warmup` untimed steps, then `steps` steps between two CUDA events (barrier +
    synchronize on both sides).  Returns (ms total, max over ranks; last loss)."""
    import torch
    import torch.distributed as dist
    for i in range(warmup):
        job.step(*pool[i % len(pool)])
    sync_all()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        loss = job.step(*pool[i % len(pool)])
    e1.record()
    sync_all()
    t = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    if N > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item(), loss


def timed_e2e(job, hosts, steps, sync_all, N, dev):
    """End to end: every step copies its inputs from pinned host memory and its loss
    is read back on the host.  Returns (ms total, max over ranks; last loss value)."""
    import torch
    import torch.distributed as dist
    for i in range(2):
        job.step(*job.to_device(*hosts[i % len(hosts)])).item()
    sync_all()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    # every step: one pinned-host -> device copy of its inputs and one device ->
    # host copy of its loss; the loss of step i is read on the host while step
    # i+1 is already queued, so the host never stalls the launch stream
    loss_host = [torch.zeros((), dtype=torch.float32).pin_memory() for _ in range(2)]
    loss_ev = [torch.cuda.Event(), torch.cuda.Event()]
    losses = []
    for i, (x, y) in enumerate(job.stream_batches(hosts, steps)):
        out = job.step(x, y)
        loss_host[i & 1].copy_(out, non_blocking=True)
        loss_ev[i & 1].record()
        if i > 0:
            loss_ev[(i - 1) & 1].synchronize()
            losses.append(float(loss_host[(i - 1) & 1]))
    loss_ev[(steps - 1) & 1].synchronize()
    losses.append(float(loss_host[(steps - 1) & 1]))
    e1.record()
    sync_all()
    t = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    if N > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item(), losses[-1]


def main():
    a = parse()
    if a.impl == "reference":
        if int(os.environ.get("RANK", "0")) == 0:     # one line per job, also under torchrun
            print(json.dumps({"impl": "reference", "unavailable": REFERENCE_UNAVAILABLE}), flush=True)
        return 0
    import torch
    import torch.distributed as dist
    import hipress_b200 as hp
    from hipress_b200.train.harness import HEADLINE, build_ddp_job, build_job
    from hipress_b200.utils.verify import one_step_check, replicas_identical

    hp.init()
    N, rank = hp.size(), hp.rank()
    if N != a.gpus and rank == 0:
        print(f"warning: --gpus {a.gpus} but world size is {N}", file=sys.stderr)
    torch.backends.cudnn.benchmark = True
    torch.backends.cuda.matmul.allow_tf32 = True
    torch.backends.cudnn.allow_tf32 = True
    head = HEADLINE[a.model]
    plan = None if a.comprplan in (None, "", "none", "threshold") else a.comprplan
    over = dict(algorithm=a.comp_alg or head["algorithm"], topology=(a.topo or head["topology"]).lower(),
                comp_threshold=a.comp_threshold, plan=plan, backend=a.sync_backend)
    if a.ctas:
        over["ctas"] = a.ctas
    if a.bucket_mb:
        over["bucket_bytes"] = a.bucket_mb << 20
    if a.partition_sms is not None:
        over["partition_sms"] = a.partition_sms
    if a.partition_ctas:
        over["partition_ctas"] = a.partition_ctas
    if a.overlap_optimizer is not None:
        over["overlap_optimizer"] = bool(a.overlap_optimizer)
    cfg = hp.HipressConfig.from_env(**over)
    job = build_job(a.model, cfg, batch=a.batch, seq_len=a.seq_len)
    eng = job.optimizer.engine
    dev = job.device
    unit = "images/s" if job.kind == "image" else "samples/s"

    def sync_all():
        torch.cuda.synchronize()
        if N > 1:
            dist.barrier()
        torch.cuda.synchronize()

    global_batch = job.batch * N
    per_s = lambda ms, steps: global_batch * steps / (ms * 1e-3)   # noqa: E731

    # ---------------- device-timed region: inputs already on the device -------------
    pool = [job.to_device(*job.host_batch(100 * rank + i)) for i in range(4)]
    for i in range(a.warmup):
        job.step(*pool[i % 4])
    sync_all()
    sampler = ClockSampler(physical_index(torch.cuda.current_device())) if rank == 0 else None
    l0 = eng.launch_count
    ms, loss = timed_steps(job, pool, a.steps, 0, sync_all, N, dev)
    launches = eng.launch_count - l0
    clocks = sampler.stop() if sampler else None
    eng.check()
    value = per_s(ms, a.steps)

    # ---------------- end to end: pinned host batch -> device every step, loss read back ----
    e2e = None
    hosts = [job.host_batch(7000 + 100 * rank + i) for i in range(4)]
    if not a.no_e2e:
        t, lv = timed_e2e(job, hosts, a.steps, sync_all, N, dev)
        e2e = {"value": round(per_s(t, a.steps), 2), "unit": unit,
               "ms_per_step": round(t / a.steps, 4),
               "h2d_bytes_per_step": job.h2d_bytes(*hosts[0]), "d2h_bytes_per_step": 4,
               "last_loss": lv}

    # ---------------- correctness evidence from the same run -------------------------
    identical = replicas_identical(job.model)
    check = one_step_check(job, *pool[0]) if not a.no_check else {}
    eng.check()
    st = eng.stats()
    job.optimizer.close()
    del job, eng
    torch.cuda.empty_cache()

    # ---------------- baseline arms, same process, same model / batch / steps --------
    baselines = {}
    if not a.no_baselines:
        ddp = build_ddp_job(a.model, batch=a.batch, seq_len=a.seq_len)
        t, _ = timed_steps(ddp, pool, a.steps, a.warmup, sync_all, N, dev)
        baselines["ddp_images_s" if unit == "images/s" else "ddp_samples_s"] = round(per_s(t, a.steps), 2)
        baselines["ddp_ms_per_step"] = round(t / a.steps, 4)
        baselines["ratio_vs_ddp"] = round(value / per_s(t, a.steps), 4)
        if e2e is not None:
            t, _ = timed_e2e(ddp, hosts, a.steps, sync_all, N, dev)
            baselines["ddp_e2e"] = round(per_s(t, a.steps), 2)
            baselines["e2e_ratio_vs_ddp"] = round(e2e["value"] / per_s(t, a.steps), 4)
        del ddp
        torch.cuda.empty_cache()
        if N > 1 and cfg.algorithm not in ("none", None, ""):
            ucfg = hp.HipressConfig.from_env(**{**over, "backend": "host"})
            unf = build_job(a.model, ucfg, batch=a.batch, seq_len=a.seq_len)
            t, _ = timed_steps(unf, pool, a.steps, a.warmup, sync_all, N, dev)
            baselines["unfused_images_s" if unit == "images/s" else "unfused_samples_s"] = \
                round(per_s(t, a.steps), 2)
            baselines["unfused_ms_per_step"] = round(t / a.steps, 4)
            baselines["ratio_vs_unfused"] = round(value / per_s(t, a.steps), 4)
            unf.optimizer.close()
            del unf
        baselines["what"] = ("ddp = torch DistributedDataParallel(gradient_as_bucket_view=True), NCCL, same "
                             "model/batch/precision/optimizer (bare model at 1 GPU); unfused = this "
                             "repo's schedule from separate encode/decode kernels around NCCL calls")

    if rank == 0:
        line = {
            "metric": ("images/sec" if unit == "images/s" else "samples/sec") +
                      f" {a.model} training step, device-timed, max over ranks",
            "value": round(value, 2), "unit": unit,
            "n_gpus": N, "steps": a.steps, "warmup": a.warmup, "ms_per_step": round(ms / a.steps, 4),
            "higher_is_better": True, "scaling": "weak",
            # the reference publishes no throughput: the anchor is the torch-DDP arm of this run
            "vs_baseline": baselines.get("ratio_vs_ddp"), "dtype": "bf16",
            "data": "synthetic (N(0,1) images / uniform token ids, random-init weights)",
            "impl": "hipress_b200",
            "config": {"model": a.model, "global_batch": global_batch, "per_gpu_batch": global_batch // N,
                       "seq_len": a.seq_len if unit != "images/s" else None,
                       "parallelism": f"dp{N}", "algorithm": cfg.algorithm, "topology": cfg.topology,
                       "comp_threshold": cfg.comp_threshold, "plan": st["plan"],
                       "plan_compressed_gradients": st["compressed_gradients"], "sync_backend": st["backend"],
                       "gradients": "fp32", "compressed_fraction":
                           round(st["compressed_elems"] / st["total_elems"], 4),
                       "buckets": st["buckets"], "ctas": cfg.ctas, "partition_sms": cfg.partition_sms,
                       "partition_ctas": cfg.partition_ctas,
                       "overlap_optimizer": cfg.overlap_optimizer,
                       "l2": "inputs larger than L2: weights+gradients+activations of one step "
                             "exceed the 126 MB L2 many times; no explicit flush"},
            "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "loss": float(loss.item()),
            "baselines": baselines, "replicas_identical": identical,
            "one_step_rel_err": check.get("one_step_rel_err"), "one_step_check": check,
        }
        print(json.dumps(line))
    hp.shutdown()
    return 0


if __name__ == "__main__":
    sys.exit(main())
