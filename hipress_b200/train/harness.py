"""Training harness shared by the launchers and the benchmark: builds one of the
headline jobs (model, synthetic data of the named shape, optimizer wrapped in
:class:`hipress_b200.DistributedOptimizer`) and exposes a ``step`` callable.

Data is synthetic, as in the reference's benchmark runs ("synthetic data",
README.md:153 of mark14wu/hipress): N(0,1) images with uniform random labels, or
uniform random token ids with 15 % of positions masked."""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F

from .. import DistributedOptimizer, HipressConfig, broadcast_parameters
from ..models import get_model
from ..parallel import comm

# model -> (per-GPU batch, algorithm, topology) of the headline configurations
HEADLINE = {
    "vgg19": dict(batch=32, algorithm="tbq", topology="ring"),
    "resnet50": dict(batch=128, algorithm="dgc", topology="ps"),
    "bert_large": dict(batch=32, algorithm="onebit", topology="ring"),
    "bert_base": dict(batch=32, algorithm="onebit", topology="ring"),
    "lstm": dict(batch=80, algorithm="tbq", topology="ring"),
    "transformer": dict(batch=64, algorithm="dgc", topology="ps"),
}


@dataclass
class Job:
    model: torch.nn.Module
    optimizer: DistributedOptimizer
    kind: str           # "image" | "mlm" | "lm"
    batch: int
    seq_len: int
    device: torch.device
    dtype: torch.dtype

    def _net(self):
        """The model itself (a DistributedDataParallel wrapper holds it as .module)."""
        return getattr(self.model, "module", self.model)

    # ---------------------------------------------------------------- data
    def host_batch(self, seed: int):
        """One synthetic batch in pinned host memory."""
        g = torch.Generator().manual_seed(seed)
        if self.kind == "image":
            x = torch.randn(self.batch, 3, 224, 224, generator=g)
            y = torch.randint(0, 1000, (self.batch,), generator=g)
        elif self.kind == "lm":   # next-token targets over uniform random ids
            V = self._net().vocab_size
            t = torch.randint(0, V, (self.batch, self.seq_len + 1), generator=g)
            x, y = t[:, :-1].contiguous(), t[:, 1:].contiguous()
        else:
            V = self._net().c.vocab_size
            x = torch.randint(0, V, (self.batch, self.seq_len), generator=g)
            y = torch.full((self.batch, self.seq_len), -100, dtype=torch.long)
            mask = torch.rand(self.batch, self.seq_len, generator=g) < 0.15
            mask[:, 0] |= ~mask.any(dim=1)  # at least one masked position per sample
            y[mask] = x[mask]
            x = x.clone()
            x[mask] = 103  # [MASK]
        if self.device.type == "cuda":
            if self.kind == "image":   # same memory layout as the model's input: the copy is pure DMA
                x = x.contiguous(memory_format=torch.channels_last)
            x, y = x.pin_memory(), y.pin_memory()
        return x, y

    def to_device(self, x, y):
        x = x.to(self.device, non_blocking=True)
        y = y.to(self.device, non_blocking=True)
        if self.kind == "image" and self.device.type == "cuda":
            x = x.contiguous(memory_format=torch.channels_last)
        return x, y

    def stream_batches(self, hosts, count: int):
        """Yields `count` device batches, copying batch i+1 from pinned host memory on
        a side stream while step i computes (one host-to-device copy per step).
        Two preallocated device buffers are reused in turn, so the copies are plain
        DMA transfers with no allocation and no layout kernel."""
        if self.device.type != "cuda":
            for i in range(count):
                yield self.to_device(*hosts[i % len(hosts)])
            return
        side = torch.cuda.Stream()
        fmt = torch.channels_last if hosts[0][0].dim() == 4 else torch.contiguous_format
        bufs = [(torch.empty_like(hosts[0][0], device=self.device, memory_format=fmt),
                 torch.empty_like(hosts[0][1], device=self.device)) for _ in range(2)]
        used = [None, None]   # event: the step that read this buffer has been queued and finished

        def issue(i):
            bx, by = bufs[i & 1]
            hx, hy = hosts[i % len(hosts)]
            if used[i & 1] is not None:
                side.wait_event(used[i & 1])
            with torch.cuda.stream(side):
                bx.copy_(hx, non_blocking=True)
                by.copy_(hy, non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(side)
            return bx, by, ev

        nxt = issue(0)
        for i in range(count):
            x, y, ev = nxt
            if i + 1 < count:
                nxt = issue(i + 1)
            cur = torch.cuda.current_stream()
            cur.wait_event(ev)
            yield x, y
            done = torch.cuda.Event()
            done.record(cur)
            used[i & 1] = done

    # ------------------------------------------------------------ real data
    def image_folder_loader(self, root, *, epoch: int = 0, workers: int = 4, image_size: int = 224,
                            train: bool = True):
        """ImageNet-style directory (one sub-directory per class) as a sharded,
        shuffled loader of pinned host batches: the data path of the reference's
        ``pytorch_imagenet.py`` (``--train-dir``), with the standard training
        augmentation.  Every rank reads a disjoint shard of each epoch."""
        from torch.utils.data import DataLoader
        from torch.utils.data.distributed import DistributedSampler
        from torchvision import datasets, transforms
        norm = transforms.Normalize(mean=[0.485, 0.456, 0.406], std=[0.229, 0.224, 0.225])
        if train:
            tf = transforms.Compose([transforms.RandomResizedCrop(image_size),
                                     transforms.RandomHorizontalFlip(), transforms.ToTensor(), norm])
        else:   # validation: resize the short side, centre crop, no shuffling, no dropped images
            tf = transforms.Compose([transforms.Resize(image_size * 8 // 7), transforms.CenterCrop(image_size),
                                     transforms.ToTensor(), norm])
        ds = datasets.ImageFolder(root, tf)
        sampler = DistributedSampler(ds, num_replicas=comm.size(), rank=comm.rank(), shuffle=train,
                                     drop_last=train)
        sampler.set_epoch(epoch)
        return DataLoader(ds, batch_size=self.batch, sampler=sampler, num_workers=workers,
                          pin_memory=self.device.type == "cuda", drop_last=train)

    @torch.no_grad()
    def evaluate(self, loader):
        """Top-1 accuracy and mean loss of an image model over `loader`, summed over
        all ranks (each rank scores its own shard)."""
        was = self.model.training
        self.model.eval()
        tot = torch.zeros(3, dtype=torch.float64, device=self.device)   # correct, loss sum, count
        for hx, hy in loader:
            x, y = self.to_device(hx, hy)
            with torch.autocast(self.device.type, dtype=self.dtype, enabled=self.dtype != torch.float32):
                out = self.model(x).float()
            tot[0] += (out.argmax(1) == y).sum()
            tot[1] += F.cross_entropy(out, y, reduction="sum")
            tot[2] += y.numel()
        comm.allreduce_(tot, average=False)
        self.model.train(was)
        n = max(tot[2].item(), 1.0)
        return {"top1": tot[0].item() / n, "loss": tot[1].item() / n, "images": int(tot[2].item())}

    def stream_from(self, host_batches):
        """Device batches from any iterable of host batches (a DataLoader), with the
        copy of batch i+1 issued on a side stream while step i computes."""
        it = iter(host_batches)
        if self.device.type != "cuda":
            for hx, hy in it:
                yield self.to_device(hx, hy)
            return
        first = next(it, None)
        if first is None:
            return
        side = torch.cuda.Stream()
        bufs = [(torch.empty_like(first[0], device=self.device), torch.empty_like(first[1], device=self.device))
                for _ in range(2)]
        used = [None, None]

        def issue(i, host):
            bx, by = bufs[i & 1]
            if used[i & 1] is not None:
                side.wait_event(used[i & 1])
            with torch.cuda.stream(side):
                bx.copy_(host[0], non_blocking=True)
                by.copy_(host[1], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(side)
            return bx, by, ev, host   # the host batch stays referenced until its copy is waited for

        i, nxt = 0, issue(0, first)
        while nxt is not None:
            x, y, ev, _ = nxt
            host = next(it, None)
            nxt = issue(i + 1, host) if host is not None else None
            cur = torch.cuda.current_stream()
            cur.wait_event(ev)
            if self.kind == "image":
                x = x.contiguous(memory_format=torch.channels_last)
            yield x, y
            done = torch.cuda.Event()
            done.record(cur)
            used[i & 1] = done
            i += 1

    def rebuild_optimizer(self):
        """After the process group was re-formed with another membership: a new
        DistributedOptimizer (buckets, arenas, hooks) around the same model and inner
        optimizer.  Compressor state is rank-local error memory of the old
        membership and starts from zero; parameters and optimizer state are taken
        from the new rank 0 so the replicas agree again."""
        old = self.optimizer
        inner, cfg = old.optimizer, old.config
        old.close(collective=False)   # the group its symmetric memory was built on is gone
        named = list(self.model.gluon_named_parameters()) if hasattr(self.model, "gluon_named_parameters") \
            else list(self.model.named_parameters())
        self.optimizer = DistributedOptimizer(inner, named, cfg)
        broadcast_parameters(self.model.state_dict(), root_rank=0)
        comm.broadcast_optimizer_state(self.optimizer, root_rank=0)

    def h2d_bytes(self, x, y):
        return x.numel() * x.element_size() + y.numel() * y.element_size()

    # ---------------------------------------------------------------- step
    def step(self, x, y):
        """Forward, backward (compressed synchronisation overlaps it), update.
        Returns the loss as a device tensor."""
        self.optimizer.zero_grad(set_to_none=True)
        with torch.autocast(self.device.type, dtype=self.dtype,
                            enabled=self.dtype != torch.float32):
            if self.kind == "image":
                loss = F.cross_entropy(self.model(x).float(), y)
            else:
                loss = self.model(x, y)
        loss.backward()
        self.optimizer.step()
        return loss.detach()


def build_job(model_name: str = "vgg19", config: HipressConfig | None = None, *, batch=None,
              seq_len: int = 128, dtype=torch.bfloat16, lr: float = 0.01, device=None,
              model_kwargs=None, seed: int = 0) -> Job:
    if not comm.is_initialized():
        comm.init()
    name = model_name.lower().replace("-", "_")
    head = HEADLINE.get(name, HEADLINE["vgg19"])
    cfg = config or HipressConfig.from_env(algorithm=head["algorithm"], topology=head["topology"])
    device = device or comm.device()
    torch.manual_seed(seed)  # same initial weights on every rank
    model = get_model(name, **(model_kwargs or {})).to(device)
    kind = "mlm" if name.startswith("bert") else ("lm" if name in ("lstm", "transformer") else "image")
    if kind == "image" and device.type == "cuda":
        model = model.to(memory_format=torch.channels_last)
    model.train()
    named = list(model.gluon_named_parameters()) if hasattr(model, "gluon_named_parameters") \
        else list(model.named_parameters())
    inner = torch.optim.SGD(model.parameters(), lr=lr, momentum=0.9,
                            **({"fused": True} if device.type == "cuda" else {}))
    opt = DistributedOptimizer(inner, named, cfg)
    broadcast_parameters(model.state_dict(), root_rank=0)
    return Job(model, opt, kind, batch or head["batch"], seq_len, device, dtype)


class _PlainOptimizer:
    """The face :class:`Job` expects of its optimizer, around a bare ``torch.optim``
    optimizer (the baseline whose gradients DistributedDataParallel synchronises)."""
    engine = None

    def __init__(self, optimizer):
        self.optimizer = optimizer

    def zero_grad(self, set_to_none: bool = True):
        self.optimizer.zero_grad(set_to_none=set_to_none)

    def step(self):
        return self.optimizer.step()

    def close(self):
        pass


def build_ddp_job(model_name: str = "vgg19", *, batch=None, seq_len: int = 128, dtype=torch.bfloat16,
                  lr: float = 0.01, device=None, model_kwargs=None, seed: int = 0,
                  bucket_cap_mb: int = 25) -> Job:
    """The conventional uncompressed baseline: the same model, data shapes, precision
    and optimizer under ``torch.nn.parallel.DistributedDataParallel`` (bucketed NCCL
    all-reduce overlapped with backward, gradients as views of the buckets).  It stands
    in for the reference's own uncompressed path ("the conventional PS and
    Ring-allreduce ... PS-Lite and NCCL", README.md:153 of mark14wu/hipress), which
    cannot be built here.  A lone process has no process group and runs the bare
    model: with one rank DDP would add nothing but its bookkeeping."""
    import torch.distributed as dist
    if not comm.is_initialized():
        comm.init()
    name = model_name.lower().replace("-", "_")
    head = HEADLINE.get(name, HEADLINE["vgg19"])
    device = device or comm.device()
    torch.manual_seed(seed)
    model = get_model(name, **(model_kwargs or {})).to(device)
    kind = "mlm" if name.startswith("bert") else ("lm" if name in ("lstm", "transformer") else "image")
    if kind == "image" and device.type == "cuda":
        model = model.to(memory_format=torch.channels_last)
    model.train()
    inner = torch.optim.SGD(model.parameters(), lr=lr, momentum=0.9,
                            **({"fused": True} if device.type == "cuda" else {}))
    if dist.is_initialized() and dist.get_world_size() > 1:
        from torch.nn.parallel import DistributedDataParallel as DDP
        model = DDP(model, device_ids=[device.index] if device.type == "cuda" else None,
                    gradient_as_bucket_view=True, bucket_cap_mb=bucket_cap_mb)
    return Job(model, _PlainOptimizer(inner), kind, batch or head["batch"], seq_len, device, dtype)
